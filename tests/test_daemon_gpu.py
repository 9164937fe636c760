"""The JSON-lines daemon of this repository (blackwell_b200/daemon/inference_server_w4a8.cpp, on the batched
decode-step driver) beside the reference's own daemon (server/inference_server_int4_batched.cu, compiled unmodified
against the reference's kernels by ``make -C oracle consumers``) on the same synthetic weight tree and tokenizer,
same request.

What can be compared: the two daemons cannot agree token for token.  Even with ``--act-bits 4`` (the reference's
INT4 activation rule and fp32 weight scales) this driver keeps a binary16 KV cache and fuses the norms, which changes
values in their last bits; INT4 activation rounding turns such a difference into whole quantization steps somewhere
in 36 layers, and the nearly flat logits of a random-weight model turn that into another greedy token (observed:
different first ids).  Token-level agreement with the reference is therefore asserted where the arithmetic is the
same -- the drop-in symbols, test_consumer_dropin_gpu.py -- and value-level agreement of this driver with the
reference's arithmetic step by step in test_decode_driver_gpu.py.  Here both daemons answer the same request (one-token
prompts: the reference's daemon mis-places multi-token prompts, see test_consumer_dropin_gpu.py), the protocol fields
are compared and both answers are printed; the int8 path is checked for what it must guarantee on its own: the
protocol, determinism, and that a prompt's result does not depend on what else is in the batch.
"""
import json
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
OURS = os.path.join(HERE, "..", "blackwell_b200", "lib", "inference_server_w4a8")
SRV_REF = os.path.join(HERE, "..", "oracle", "_ref", "inference_server_int4_batched_ref")


def _ask(cmd, cwd, requests):
    p = subprocess.Popen(cmd, cwd=cwd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    lines = []
    try:
        for r in requests:
            p.stdin.write(r + "\n")
            p.stdin.flush()
            lines.append(p.stdout.readline())
    finally:
        p.kill()
        p.wait(timeout=60)
    assert all(l.strip() for l in lines), p.stderr.read()[-2000:]
    return [json.loads(l) for l in lines]


@pytest.fixture(scope="module")
def tree(cuda, tmp_path_factory):
    from blackwell_b200 import weight_files as wf
    from blackwell_b200.shapes import ModelShape

    root = tmp_path_factory.mktemp("daemon")
    shape = ModelShape("consumer-8b", layers=36, hidden=4096, inter=12288, n_q_heads=32, n_kv_heads=8, head_dim=128,
                       vocab=151936)
    wf.write_linked_tree(str(root / "weights_int4_qwen3_8b"), shape, seed=123)
    wf.write_synthetic_tokenizer(str(root / "tokenizer_data.bin"), shape.vocab)
    return str(root), shape


@pytest.mark.timeout(1200)
def test_daemon_int8_protocol_determinism_and_batch_independence(tree):
    assert os.path.exists(OURS), "the daemon is built by python -m blackwell_b200._build"
    cwd, shape = tree
    reqs = ['{"prompts": ["The capital of France is", "Hi"], "max_tokens": 6, "temperature": 0.0}',
            '{"prompts": ["Hi"], "max_tokens": 6}',
            '{"prompts": ["The capital of France is", "Hi", "Two plus two is"], "max_tokens": 6}',
            '{"prompts": ["x"], "max_tokens": 3, "temperature": 0.8}',
            '{"nothing": 1}']
    out = _ask([OURS, "--batch", "2", "--max-seq", "256", "--act-bits", "8"], cwd, reqs)
    a, b, c, d, e = out
    assert len(a["tokens"]) == 2 and len(a["text"]) == 2
    for t in a["tokens"]:
        assert len(t) == 7 and all(0 <= i < shape.vocab for i in t)      # max_tokens + the id of the last prompt step
    assert b["tokens"][0] == a["tokens"][1]          # same prompt, other batch neighbour (idle slot)
    assert c["tokens"][:2] == a["tokens"]            # a third prompt runs as a second group
    assert len(c["tokens"]) == 3
    assert "error" in d and "error" in e
    # ids >= 256 decode as "<id>" with the synthetic tokenizer
    assert all(("<%d>" % i) in a["text"][0] for i in a["tokens"][0] if i >= 256)


@pytest.mark.timeout(1200)
@pytest.mark.skipif(not os.path.exists(SRV_REF), reason="oracle/_ref daemon not built")
def test_daemon_int4_mode_beside_the_reference_daemon(tree):
    cwd, shape = tree
    req = '{"prompts": ["A", "B"], "max_tokens": 6, "temperature": 0.0}'
    ours, = _ask([OURS, "--batch", "2", "--max-seq", "256", "--act-bits", "4"], cwd, [req])
    ref, = _ask([SRV_REF], cwd, [req])
    print("this daemon (W4A4 arithmetic):", ours["tokens"])
    print("reference daemon:", ref["tokens"])
    assert len(ours["tokens"]) == 2 and len(ref["tokens"]) == 2
    assert sorted(ours.keys()) == sorted(ref.keys()) == ["text", "tokens"]
    for o, r in zip(ours["tokens"], ref["tokens"]):
        assert len(o) == len(r) == 7 and all(0 <= i < shape.vocab for i in o)
