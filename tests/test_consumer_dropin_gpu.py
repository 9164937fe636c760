"""End-to-end drop-in: the reference's own batched text generator (bench/text_generate_int4_batched.cu, compiled
unmodified by ``make -C oracle consumers``) runs against this repository's library and against the reference's
kernels on the same synthetic weight tree.  Greedy decoding of a random-weight model is chaotic: its 151,936 logits
are nearly flat, so the first near-tie that the two libraries' different summation orders resolve differently ends
the common prefix (with this seed after six tokens); the test demands the first four generated tokens to agree and all
four sequences of a run (same prompt) to agree with one another in full.

The tree has the sizes the program hard-codes (36 layers, H 4096, I 12288, V 151936); one layer is written and
hard-linked 36 times.  The synthetic tokenizer decodes id i >= 256 as the text "<i>", so the printed text carries the
generated ids.  Skipped when the two binaries were not built (they need the reference's sources at build time).
"""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
REFDIR = os.path.join(HERE, "..", "oracle", "_ref")
OURS = os.path.join(REFDIR, "text_generate_int4_batched_ours")
REF = os.path.join(REFDIR, "text_generate_int4_batched_ref")


def _run(exe, cwd, wdir, batch, new_tokens):
    r = subprocess.run([exe, "The capital of France is", str(batch), str(new_tokens), wdir], cwd=cwd,
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, (r.stdout[-1500:], r.stderr[-1500:])
    assert "FAIL" not in r.stdout, r.stdout[-1500:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("[Prompt ")]
    stats = [l for l in r.stdout.splitlines() if l.startswith("Stats:")]
    return lines, (stats[0] if stats else "")


@pytest.mark.skipif(not (os.path.exists(OURS) and os.path.exists(REF)), reason="oracle/_ref consumers not built")
def test_reference_text_generator_runs_on_both_libraries(cuda, tmp_path):
    from blackwell_b200 import weight_files as wf
    from blackwell_b200.shapes import ModelShape

    shape = ModelShape("consumer-8b", layers=36, hidden=4096, inter=12288, n_q_heads=32, n_kv_heads=8, head_dim=128,
                       vocab=151936)
    wdir = str(tmp_path / "weights_int4_qwen3_8b")
    wf.write_linked_tree(wdir, shape, seed=123)
    wf.write_synthetic_tokenizer(str(tmp_path / "tokenizer_data.bin"), shape.vocab)
    batch, new_tokens = 4, 12
    ours, ours_stats = _run(OURS, str(tmp_path), wdir, batch, new_tokens)
    ref, ref_stats = _run(REF, str(tmp_path), wdir, batch, new_tokens)
    print("ours:", ours_stats, "| reference kernels:", ref_stats)
    assert len(ours) == batch and len(ref) == batch
    ids = re.findall(r"<(\d+)>", ours[0])
    assert len(ids) >= new_tokens - 2, ours[0]          # real token ids came out (bytes below 256 print as text)
    ref_ids = re.findall(r"<(\d+)>", ref[0])
    prefix = 0
    while prefix < min(len(ids), len(ref_ids)) and ids[prefix] == ref_ids[prefix]:
        prefix += 1
    print("common prefix of generated ids:", prefix, "of", len(ids))
    assert prefix >= 4, (ours[0], ref[0])
    for lines in (ours, ref):                            # same prompt, same continuation within a run
        assert all(l.split("] ", 1)[1] == lines[0].split("] ", 1)[1] for l in lines)


SRV_OURS = os.path.join(REFDIR, "inference_server_int4_batched_ours")
SRV_REF = os.path.join(REFDIR, "inference_server_int4_batched_ref")


def _ask_daemon(exe, cwd, requests):
    """Starts the reference's stdin/stdout JSON daemon, sends the request lines one by one, reads one response line for
    each and stops the process (it has no shutdown command and spins on end-of-file, so it is never left to read a
    closed pipe)."""
    import json

    p = subprocess.Popen([exe], cwd=cwd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    lines = []
    try:
        for request in requests:
            p.stdin.write(request + "\n")
            p.stdin.flush()
            lines.append(p.stdout.readline())
    finally:
        p.kill()
        p.wait(timeout=60)
    assert all(l.strip() for l in lines), p.stderr.read()[-1500:]
    return [json.loads(l) for l in lines]


@pytest.mark.timeout(900)
@pytest.mark.skipif(not (os.path.exists(SRV_OURS) and os.path.exists(SRV_REF)), reason="oracle/_ref daemons not built")
def test_reference_json_daemon_runs_on_both_libraries(cuda, tmp_path):
    """server/inference_server_int4_batched.cu, unmodified: one request over its JSON-lines protocol
    (:340-384), two prompts, greedy."""
    from blackwell_b200 import weight_files as wf
    from blackwell_b200.shapes import ModelShape

    shape = ModelShape("consumer-8b", layers=36, hidden=4096, inter=12288, n_q_heads=32, n_kv_heads=8, head_dim=128,
                       vocab=151936)
    wf.write_linked_tree(str(tmp_path / "weights_int4_qwen3_8b"), shape, seed=123)
    wf.write_synthetic_tokenizer(str(tmp_path / "tokenizer_data.bin"), shape.vocab)
    req = '{"prompts": ["The capital of France is", "Two plus two is"], "max_tokens": 8, "temperature": 0.0}'
    # One byte = one token with the merge-free synthetic tokenizer.  With a one-token prompt the daemon samples --
    # and therefore synchronises with the GPU -- after every step (server/inference_server_int4_batched.cu:283-297).
    req1 = '{"prompts": ["A"], "max_tokens": 6, "temperature": 0.0}'
    ours, ours1 = _ask_daemon(SRV_OURS, str(tmp_path), [req, req1])
    ref, ref1 = _ask_daemon(SRV_REF, str(tmp_path), [req, req1])
    assert len(ours["tokens"]) == 2 and len(ref["tokens"]) == 2 and len(ours["text"]) == 2
    for a in ours["tokens"]:
        assert 8 <= len(a) <= 9 and all(0 <= t < shape.vocab for t in a)   # max_tokens, plus the token of the last prompt step
    # With this library the daemon starts the first prompt exactly like the text generator above does with either
    # library (ids 47388, 48015, 118878 for this seed).
    assert ours["tokens"][0][:3] == [47388, 48015, 118878], ours["tokens"][0]
    print("daemon, this library:", ours["tokens"], ours1["tokens"])
    print("daemon, reference kernels:", ref["tokens"], ref1["tokens"])
    # The reference's own kernels do not reproduce those ids on a multi-token prompt -- nor their own from one run to the
    # next (50289, 89520, 147823 in one run, 62212, 53809, 57376 in another) -- and the cause is in the reference:
    # update_kv_cache and attention_decode_batched_gqa store seq_pos in ONE pinned host int and enqueue an asynchronous
    # host-to-device copy of it (src/kernels/decode.cu:252-283, 479-482, 599-601), which reads the int when the copy
    # EXECUTES; the daemon does not synchronise while it walks the prompt (:248-281, first sync at :297 once
    # step >= gen_start - 1), so the host has overwritten the int with later positions before earlier copies run and
    # prompt tokens land at wrong cache rows.  This library takes the position by value.  Where the daemon synchronises
    # every step -- the one-token prompt -- both libraries start with the same ids; further on the greedy paths part at
    # a near-tie of the random-weight logits (int4 activation rounding amplifies last-bit differences of the two
    # libraries' summation orders), as in the generator test.
    assert ours1["tokens"][0][:2] == ref1["tokens"][0][:2], (ours1["tokens"], ref1["tokens"])
