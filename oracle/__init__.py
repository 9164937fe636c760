"""CPU oracle for the INT4 block-16 GEMV decode path -- TEST INFRASTRUCTURE ONLY.

numpy-facing wrappers over ``oracle/liboracle.so`` (built from ``oracle.c`` by
``make -C oracle``).  Nothing in the shipped package imports this module; it is
used by the tests, by the smoke check and by the CPU-baseline leg of the
benchmark.  Each wrapper documents the reference file:line its C routine
follows (see the comments in ``oracle.c``).

Parity status: the reference has no golden vectors for this path; the oracle is
pinned against the reference's own CUDA kernels rebuilt for sm_100a (see
``oracle/ref_cuda.py``) through the fixtures in ``tests/golden/``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` into ``liboracle.so`` (gcc, OpenMP)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.orc_gemv_w4a8_f32.restype = C.c_int
        _lib.orc_gemv_w4a4_f32.restype = C.c_int
        _lib.orc_argmax.restype = C.c_int
        _lib.orc_max_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "oracle wants contiguous arrays"
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


# ---------------------------------------------------------------- conversions
def half_bits_to_float(h: np.ndarray) -> np.ndarray:
    h = _c(h, np.uint16)
    out = np.empty(h.shape, np.float32)
    lib().orc_half_to_float(_p(h), _p(out), C.c_long(h.size))
    return out


# ---------------------------------------------------------------- quantizers
def quantize_int4(x: np.ndarray):
    """x f32 [M][K] (or [K]) -> (packed u8 [M][K/2], scale f32 [M][K/16]).
    gemv_int8.cu:1628-1666."""
    x2 = _c(np.atleast_2d(x), np.float32)
    M, K = x2.shape
    assert K % 16 == 0
    out = np.empty((M, K // 2), np.uint8)
    sc = np.empty((M, K // 16), np.float32)
    lib().orc_quantize_int4(_p(x2), C.c_int(K), C.c_int(M), _p(out), _p(sc))
    if x.ndim == 1:
        return out[0], sc[0]
    return out, sc


def quantize_int8(x: np.ndarray):
    """x f32 [...] with size % 16 == 0 -> (q i8 same shape, scale f32 [size/16]).
    gemv_int8.cu:718-748."""
    xf = _c(x, np.float32)
    assert xf.size % 16 == 0
    out = np.empty(xf.shape, np.int8)
    sc = np.empty(xf.size // 16, np.float32)
    lib().orc_quantize_int8(_p(xf), C.c_long(xf.size), _p(out), _p(sc))
    if xf.ndim == 2:
        sc = sc.reshape(xf.shape[0], -1)
    return out, sc


def quantize_int4_fusedrule(x: np.ndarray):
    """Scale rule of the fused prologue kernels, one row.  fused_int4_ops.cu:155-327."""
    xf = _c(x, np.float32)
    K = xf.size
    out = np.empty(K // 2, np.uint8)
    sc = np.empty(K // 16, np.float32)
    lib().orc_quantize_int4_fusedrule(_p(xf), C.c_int(K), _p(out), _p(sc))
    return out, sc


def quantize_weights_int4(w: np.ndarray):
    """w f32 [N][K] -> (packed u8 [N][K/2], scale f32 [N][K/16]).
    scripts/quantize_llama32_1b.py:57-75."""
    w = _c(w, np.float32)
    N, K = w.shape
    out = np.empty((N, K // 2), np.uint8)
    sc = np.empty((N, K // 16), np.float32)
    lib().orc_quantize_weights_int4(_p(w), C.c_int(K), C.c_int(N), _p(out), _p(sc))
    return out, sc


# ---------------------------------------------------------------- block dots
def block_dots_w4a4(W: np.ndarray, x: np.ndarray) -> np.ndarray:
    W = _c(W, np.uint8)
    x = _c(x, np.uint8)
    N, K2 = W.shape
    dots = np.empty((N, K2 // 8), np.int32)
    lib().orc_block_dots_w4a4(_p(W), _p(x), C.c_int(K2 * 2), C.c_int(N), _p(dots))
    return dots


def block_dots_w4a8(W: np.ndarray, xq: np.ndarray) -> np.ndarray:
    W = _c(W, np.uint8)
    xq = _c(xq, np.int8)
    N, K2 = W.shape
    dots = np.empty((N, K2 // 8), np.int32)
    lib().orc_block_dots_w4a8(_p(W), _p(xq), C.c_int(K2 * 2), C.c_int(N), _p(dots))
    return dots


# ---------------------------------------------------------------------- GEMV
def _w4a4_args(x, xsc, W, Wsc):
    W = _c(W, np.uint8)
    Wsc = _c(Wsc, np.float32)
    x = _c(np.atleast_2d(x), np.uint8)
    xsc = _c(np.atleast_2d(xsc), np.float32)
    N, K2 = W.shape
    return x, xsc, W, Wsc, K2 * 2, N, x.shape[0]


def gemv_w4a4_exact(x, xsc, W, Wsc) -> np.ndarray:
    """Bit-level restatement of gemv_int4_batched_kernel.  gemv_int8.cu:913-984."""
    x, xsc, W, Wsc, K, N, M = _w4a4_args(x, xsc, W, Wsc)
    y = np.empty((M, N), np.float32)
    lib().orc_gemv_w4a4_exact(_p(y), _p(x), _p(xsc), _p(W), _p(Wsc), C.c_int(K), C.c_int(N), C.c_int(M))
    return y


def gemv_w4a4_f64(x, xsc, W, Wsc) -> np.ndarray:
    x, xsc, W, Wsc, K, N, M = _w4a4_args(x, xsc, W, Wsc)
    y = np.empty((M, N), np.float64)
    lib().orc_gemv_w4a4_f64(_p(y), _p(x), _p(xsc), _p(W), _p(Wsc), C.c_int(K), C.c_int(N), C.c_int(M))
    return y


def gemv_w4a4_f32(x, xsc, W, Wsc, threads: int = 0):
    x, xsc, W, Wsc, K, N, M = _w4a4_args(x, xsc, W, Wsc)
    y = np.empty((M, N), np.float32)
    used = lib().orc_gemv_w4a4_f32(_p(y), _p(x), _p(xsc), _p(W), _p(Wsc), C.c_int(K), C.c_int(N), C.c_int(M),
                                   C.c_int(threads))
    return y, used


def _w4a8_args(xq, xsc, W, Wsc_h):
    W = _c(W, np.uint8)
    Wsc_h = _c(Wsc_h.view(np.uint16) if Wsc_h.dtype == np.float16 else Wsc_h, np.uint16)
    xq = _c(np.atleast_2d(xq), np.int8)
    xsc = _c(np.atleast_2d(xsc), np.float32)
    N, K2 = W.shape
    return xq, xsc, W, Wsc_h, K2 * 2, N, xq.shape[0]


def gemv_w4a8_f64(xq, xsc, W, Wsc_h) -> np.ndarray:
    """W4A8, binary16 weight scales, double accumulation (ground truth)."""
    xq, xsc, W, Wsc_h, K, N, M = _w4a8_args(xq, xsc, W, Wsc_h)
    y = np.empty((M, N), np.float64)
    lib().orc_gemv_w4a8_f64(_p(y), _p(xq), _p(xsc), _p(W), _p(Wsc_h), C.c_int(K), C.c_int(N), C.c_int(M))
    return y


def gemv_w4a8_f32(xq, xsc, W, Wsc_h, threads: int = 0):
    """Scalar fp32 dequant-dot; the routine timed as the CPU baseline."""
    xq, xsc, W, Wsc_h, K, N, M = _w4a8_args(xq, xsc, W, Wsc_h)
    y = np.empty((M, N), np.float32)
    used = lib().orc_gemv_w4a8_f32(_p(y), _p(xq), _p(xsc), _p(W), _p(Wsc_h), C.c_int(K), C.c_int(N), C.c_int(M),
                                   C.c_int(threads))
    return y, used


def max_threads() -> int:
    return int(lib().orc_max_threads())


def dequant_row(row: int, W, Wsc) -> np.ndarray:
    """server/inference_server_int4_batched.cu:72-83."""
    W = _c(W, np.uint8)
    Wsc = _c(Wsc, np.float32)
    K = W.shape[1] * 2
    out = np.empty(K, np.float32)
    lib().orc_dequant_row(_p(out), C.c_long(row), _p(W), _p(Wsc), C.c_int(K))
    return out


# ---------------------------------------------------------- norm/elementwise
def rmsnorm(x, w, eps: float = 1e-6, reforder: bool = False) -> np.ndarray:
    """norm.cu:44-89,114-155.  ``reforder`` reproduces the reference reduction order (H <= 4096)."""
    x2 = _c(np.atleast_2d(x), np.float32)
    w = _c(w, np.float32)
    M, H = x2.shape
    out = np.zeros((M, H), np.float32)
    fn = lib().orc_rmsnorm_reforder if reforder else lib().orc_rmsnorm
    fn(_p(out), _p(x2), _p(w), C.c_int(H), C.c_float(eps), C.c_int(M))
    return out[0] if np.ndim(x) == 1 else out


def swiglu(g, u) -> np.ndarray:
    g = _c(g, np.float32)
    u = _c(u, np.float32)
    out = np.empty_like(g)
    lib().orc_swiglu(_p(out), _p(g), _p(u), C.c_long(g.size))
    return out


def swiglu_fusedform(g, u) -> np.ndarray:
    """fused_int4_ops.cu:270-277."""
    g = _c(g, np.float32)
    u = _c(u, np.float32)
    out = np.empty_like(g)
    lib().orc_swiglu_fusedform(_p(out), _p(g), _p(u), C.c_long(g.size))
    return out


def vector_add(a, b) -> np.ndarray:
    a = _c(a, np.float32)
    b = _c(b, np.float32)
    out = np.empty_like(a)
    lib().orc_vector_add(_p(out), _p(a), _p(b), C.c_long(a.size))
    return out


def head_norm(data, w, nh: int, hd: int, eps: float = 1e-6) -> np.ndarray:
    d = _c(data, np.float32).copy()
    w = _c(w, np.float32)
    lib().orc_head_norm(_p(d), _p(w), C.c_int(nh), C.c_int(hd), C.c_float(eps))
    return d


def rope(data, nh: int, hd: int, pos: int) -> np.ndarray:
    d = _c(data, np.float32).copy()
    lib().orc_rope(_p(d), C.c_int(nh), C.c_int(hd), C.c_int(pos))
    return d


# ------------------------------------------------------------------ KV/attn
def update_kv(kc, vc, k_new, v_new, seq_pos: int, nh: int, hd: int, max_seq: int) -> None:
    """In place on kc/vc (f32 [nh][max_seq][hd]).  decode.cu:27-46."""
    assert kc.dtype == np.float32 and vc.dtype == np.float32
    lib().orc_update_kv(_p(kc), _p(vc), _p(_c(k_new, np.float32)), _p(_c(v_new, np.float32)), C.c_int(seq_pos),
                        C.c_int(nh), C.c_int(hd), C.c_int(max_seq))


def attention_decode_gqa(Q, Kc, Vc, seq_pos, nqh, nkv, hd, max_seq, M, kv_batch_elems, kv_layer_elems):
    """decode.cu:375-466 (mathematics only).  ``seq_pos`` int or int array [M]."""
    Q = _c(Q, np.float32)
    Kc = _c(Kc, np.float32)
    Vc = _c(Vc, np.float32)
    per = not np.isscalar(seq_pos)
    sp = _c(np.atleast_1d(seq_pos), np.int32)
    out = np.empty(M * nqh * hd, np.float32)
    lib().orc_attention_decode_gqa(_p(out), _p(Q), _p(Kc), _p(Vc), _p(sp), C.c_int(int(per)), C.c_int(nqh),
                                   C.c_int(nkv), C.c_int(hd), C.c_int(max_seq), C.c_int(M),
                                   C.c_size_t(kv_batch_elems), C.c_size_t(kv_layer_elems))
    return out.reshape(M, nqh * hd)


def attention_decode_f16kv(Q, Kc_h, Vc_h, seq_pos, nqh, nkv, hd, max_seq, M):
    Q = _c(Q, np.float32)
    Kc_h = _c(Kc_h.view(np.uint16), np.uint16)
    Vc_h = _c(Vc_h.view(np.uint16), np.uint16)
    sp = _c(seq_pos, np.int32)
    out = np.empty(M * nqh * hd, np.float32)
    lib().orc_attention_decode_f16kv(_p(out), _p(Q), _p(Kc_h), _p(Vc_h), _p(sp), C.c_int(nqh), C.c_int(nkv),
                                     C.c_int(hd), C.c_int(max_seq), C.c_int(M))
    return out.reshape(M, nqh * hd)


# ------------------------------------------------------------------ sampling
def argmax(logits) -> int:
    logits = _c(logits, np.float32)
    return int(lib().orc_argmax(_p(logits), C.c_int(logits.size)))


def repetition_penalty(logits, recent, penalty: float) -> np.ndarray:
    out = _c(logits, np.float32).copy()
    recent = _c(recent, np.int32)
    lib().orc_repetition_penalty(_p(out), _p(recent), C.c_int(recent.size), C.c_float(penalty), C.c_int(out.size))
    return out
