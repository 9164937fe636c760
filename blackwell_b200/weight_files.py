"""Reader / writer of the INT4 servers' weight tree (host side of ``csrc/weight_files.cu``).

Tree layout, as the reference's loaders expect it (bench/text_generate_int4_batched.cu:441-508,
server/inference_server_int4_batched.cu:150-184): per layer ``{l}_self_attn.{q,k,v,o}_proj`` and
``{l}_mlp.{gate,up,down}_proj`` as ``.int4_t`` + ``.scale_t`` pairs, ``{l}_input_layernorm.f32``,
``{l}_post_attention_layernorm.f32``, one ``qk_norms.f32`` holding [layer][q|k][head_dim], ``embed_tokens`` and
``lm_head`` pairs, ``final_norm.f32``.  ``write_synthetic_tree`` fills such a tree with seeded random weights in the
reference quantizer's value range (no checkpoint is available offline).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import _lib, synth
from .shapes import ModelShape

_L = _lib.load()


class bw_dev_w4(C.Structure):
    _fields_ = [("K", C.c_int), ("N", C.c_int), ("packed", C.c_void_p), ("scale_f32", C.c_void_p),
                ("scale_f16", C.c_void_p)]


_L.bw_w4_file_write.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
_L.bw_w4_file_dims.argtypes = [C.c_char_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
_L.bw_w4_file_read.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
_L.bw_w4_file_upload.argtypes = [C.c_char_p, C.c_int, C.c_int, C.POINTER(bw_dev_w4)]
_L.bw_w4_free.argtypes = [C.POINTER(bw_dev_w4)]
_L.bw_f32_file_write.argtypes = [C.c_char_p, C.c_void_p, C.c_size_t]
_L.bw_f32_file_read.argtypes = [C.c_char_p, C.c_void_p, C.c_size_t]

ERRORS = {-1: "cannot open", -2: "file length does not match its header", -3: "inconsistent header",
          -4: "bad argument", -5: "write failed"}


class WeightFileError(RuntimeError):
    def __init__(self, what: str, code: int):
        super().__init__(f"{what}: {ERRORS.get(code, 'cudaError %d' % code)}")
        self.code = code


def _chk(what, code):
    if code != 0:
        raise WeightFileError(what, code)


def write_w4(prefix: str, packed: np.ndarray, scales: np.ndarray):
    N, K2 = packed.shape
    K = 2 * K2
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    assert scales.shape == (N, K // 16)
    _chk(prefix, _L.bw_w4_file_write(prefix.encode(), packed.ctypes.data, scales.ctypes.data, K, N))


def dims_w4(prefix: str):
    K, N = C.c_int(0), C.c_int(0)
    _chk(prefix, _L.bw_w4_file_dims(prefix.encode(), C.byref(K), C.byref(N)))
    return K.value, N.value


def read_w4(prefix: str):
    K, N = dims_w4(prefix)
    packed = np.empty((N, K // 2), dtype=np.uint8)
    scales = np.empty((N, K // 16), dtype=np.float32)
    _chk(prefix, _L.bw_w4_file_read(prefix.encode(), packed.ctypes.data, scales.ctypes.data, K, N))
    return packed, scales


def write_f32(path: str, data: np.ndarray):
    data = np.ascontiguousarray(data, dtype=np.float32)
    _chk(path, _L.bw_f32_file_write(path.encode(), data.ctypes.data, data.size))


def read_f32(path: str, n: int) -> np.ndarray:
    out = np.empty((n,), dtype=np.float32)
    _chk(path, _L.bw_f32_file_read(path.encode(), out.ctypes.data, n))
    return out


class DeviceW4:
    """One projection uploaded by the library (cudaMalloc'd there, freed on close)."""

    def __init__(self, prefix: str, f32_scales: bool = True, f16_scales: bool = True):
        self._w = bw_dev_w4()
        _chk(prefix, _L.bw_w4_file_upload(prefix.encode(), int(f32_scales), int(f16_scales), C.byref(self._w)))
        self.K, self.N = self._w.K, self._w.N
        self.packed, self.scale_f32, self.scale_f16 = self._w.packed, self._w.scale_f32, self._w.scale_f16

    def close(self):
        _L.bw_w4_free(C.byref(self._w))
        self.packed = self.scale_f32 = self.scale_f16 = None


PROJECTIONS = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
               "mlp.up_proj", "mlp.down_proj")


def projection_dims(shape: ModelShape):
    H, Q, KV, I = shape.hidden, shape.n_q_heads * shape.head_dim, shape.n_kv_heads * shape.head_dim, shape.inter
    return {"self_attn.q_proj": (Q, H), "self_attn.k_proj": (KV, H), "self_attn.v_proj": (KV, H),
            "self_attn.o_proj": (H, Q), "mlp.gate_proj": (I, H), "mlp.up_proj": (I, H), "mlp.down_proj": (H, I)}


def write_synthetic_tree(root: str, shape: ModelShape, seed: int = 0, vocab: int | None = None):
    """Writes a complete tree for ``shape`` with seeded synthetic weights; returns the number of bytes written."""
    os.makedirs(root, exist_ok=True)
    vocab = vocab or shape.vocab
    total = 0
    dims = projection_dims(shape)
    qk = np.empty((shape.layers, 2, shape.head_dim), dtype=np.float32)
    for l in range(shape.layers):
        for j, name in enumerate(PROJECTIONS):
            N, K = dims[name]
            packed, sc16, sc32 = synth.int4_weights(N, K, seed + 100 * l + j)
            write_w4(os.path.join(root, f"{l}_{name}"), packed, sc32)
            total += packed.nbytes + 4 * sc16.size + 40
        write_f32(os.path.join(root, f"{l}_input_layernorm.f32"), synth.norm_weight(shape.hidden, seed + 100 * l + 50))
        write_f32(os.path.join(root, f"{l}_post_attention_layernorm.f32"),
                  synth.norm_weight(shape.hidden, seed + 100 * l + 51))
        qk[l, 0] = synth.norm_weight(shape.head_dim, seed + 100 * l + 52)
        qk[l, 1] = synth.norm_weight(shape.head_dim, seed + 100 * l + 53)
        total += 8 * shape.hidden
    write_f32(os.path.join(root, "qk_norms.f32"), qk)
    for j, name in enumerate(("embed_tokens", "lm_head")):
        packed, sc16, sc32 = synth.int4_weights(vocab, shape.hidden, seed + 90001 + j)
        write_w4(os.path.join(root, name), packed, sc32)
        total += packed.nbytes + 4 * sc16.size + 40
    write_f32(os.path.join(root, "final_norm.f32"), synth.norm_weight(shape.hidden, seed + 90003))
    return total + qk.nbytes + 4 * shape.hidden


def _byte_encoder_codepoints():
    """The byte -> unicode codepoint table of byte-level BPE (printable bytes map to themselves, the rest to 256+)."""
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    cps, extra = [0] * 256, 0
    for b in range(256):
        if b in keep:
            cps[b] = b
        else:
            cps[b] = 256 + extra
            extra += 1
    return cps


def write_synthetic_tokenizer(path: str, vocab: int):
    """A minimal ``tokenizer_data.bin`` in the layout ``BpeTokenizer::load`` reads (include/blackwell/bpe_tokenizer.h:
    168-296): header (vocab, merges, added), 256 byte-encoder codepoints, vocab entries (id u32, length u16, UTF-8),
    no added tokens, no merges.  Ids 0..255 are the single bytes; every other id decodes to the text ``<id>``, so
    that generated text shows the generated ids."""
    import struct

    cps = _byte_encoder_codepoints()
    with open(path, "wb") as f:
        f.write(struct.pack("<3I", vocab, 0, 0))
        f.write(struct.pack("<256I", *cps))
        for i in range(vocab):
            s = chr(cps[i]).encode("utf-8") if i < 256 else b"<%d>" % i
            f.write(struct.pack("<IH", i, len(s)))
            f.write(s)


def write_linked_tree(root: str, shape: ModelShape, seed: int = 0):
    """A full-size tree at the disk cost of one layer: layer 0 and the embedding are written, every other layer and
    ``lm_head`` are hard links to them (synthetic weights carry no meaning, the loaders only need the files)."""
    one = ModelShape(shape.name, 1, shape.hidden, shape.inter, shape.n_q_heads, shape.n_kv_heads, shape.head_dim,
                     shape.vocab, shape.eps)
    write_synthetic_tree(root, one, seed)
    for l in range(1, shape.layers):
        for name in PROJECTIONS:
            for ext in (".int4_t", ".scale_t"):
                os.link(os.path.join(root, f"0_{name}{ext}"), os.path.join(root, f"{l}_{name}{ext}"))
        for name in ("input_layernorm", "post_attention_layernorm"):
            os.link(os.path.join(root, f"0_{name}.f32"), os.path.join(root, f"{l}_{name}.f32"))
    qk = read_f32(os.path.join(root, "qk_norms.f32"), 2 * shape.head_dim)
    write_f32(os.path.join(root, "qk_norms.f32"), np.tile(qk, shape.layers))
    for ext in (".int4_t", ".scale_t"):
        os.remove(os.path.join(root, "lm_head" + ext))
        os.link(os.path.join(root, "embed_tokens" + ext), os.path.join(root, "lm_head" + ext))
