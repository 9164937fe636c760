"""Tensor-level mirror of the reference's kernel interface for the decode path.

Every function has the name and argument order of its counterpart in the
reference's ``include/blackwell/kernels.h`` (and of the C entry point
``bw_<name>`` it calls); tensors are torch CUDA tensors used purely as device
memory, ``stream`` is a ``torch.cuda.Stream`` or None for the current stream.
Errors come back as the reference's do -- a cudaError_t -- and are raised as
``KernelError`` here.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_L = _lib.load()


class KernelError(RuntimeError):
    def __init__(self, name: str, code: int):
        super().__init__(f"{name} returned cudaError {code}")
        self.code = code


CUDA_ERROR_INVALID_VALUE = 1


def _s(stream):
    if stream is None:
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream)


def _p(t):
    if t is None:
        return C.c_void_p(0)
    if isinstance(t, int):
        return C.c_void_p(t)
    assert t.is_cuda, "device tensors only"
    return C.c_void_p(t.data_ptr())


def _chk(name, code):
    if code != 0:
        raise KernelError(name, code)


# ----------------------------------------------------------------------- GEMV
def gemv_int4_batched(y_out, x_packed, x_scale, W_packed, W_scale, K, N, M, stream=None):
    _chk("gemv_int4_batched", _L.bw_gemv_int4_batched(_p(y_out), _p(x_packed), _p(x_scale), _p(W_packed),
                                                      _p(W_scale), K, N, M, _s(stream)))


def gemv_int4_warp(y_out, x_packed, x_scale, W_packed, W_scale, K, N, stream=None):
    _chk("gemv_int4_warp", _L.bw_gemv_int4_warp(_p(y_out), _p(x_packed), _p(x_scale), _p(W_packed), _p(W_scale),
                                                K, N, _s(stream)))


def gemv_w4a8(y_out, x_q, x_scale, W_packed, W_scale_f16, K, N, M, stream=None):
    _chk("gemv_w4a8", _L.bw_gemv_w4a8(_p(y_out), _p(x_q), _p(x_scale), _p(W_packed), _p(W_scale_f16), K, N, M,
                                      _s(stream)))


def gemv_w4a8_f16in(y_out, x_f16, W_packed, W_scale_f16, K, N, M, stream=None):
    _chk("gemv_w4a8_f16in", _L.bw_gemv_w4a8_f16in(_p(y_out), _p(x_f16), _p(W_packed), _p(W_scale_f16), K, N, M,
                                                  _s(stream)))


def gemv_w4a8_f32in(y_out, x_f32, norm_weight, eps, W_packed, W_scale_f16, K, N, M, stream=None):
    _chk("gemv_w4a8_f32in", _L.bw_gemv_w4a8_f32in(_p(y_out), _p(x_f32), _p(norm_weight), C.c_float(eps),
                                                  _p(W_packed), _p(W_scale_f16), K, N, M, _s(stream)))


def gemv_w4a8_swiglu(y_out, gate, up, W_packed, W_scale_f16, K, N, M, stream=None):
    _chk("gemv_w4a8_swiglu", _L.bw_gemv_w4a8_swiglu(_p(y_out), _p(gate), _p(up), _p(W_packed), _p(W_scale_f16),
                                                    K, N, M, _s(stream)))


def gemv_int4_fused(y_out, x_f32, up, norm_weight, eps, W_packed, W_scale, K, N, M, stream=None):
    _chk("gemv_int4_fused", _L.bw_gemv_int4_fused(_p(y_out), _p(x_f32), _p(up), _p(norm_weight), C.c_float(eps),
                                                  _p(W_packed), _p(W_scale), K, N, M, _s(stream)))


def gemv_block_dots(dots, x, a8, W_packed, K, N, stream=None):
    _chk("gemv_block_dots", _L.bw_gemv_block_dots(_p(dots), _p(x), int(a8), _p(W_packed), K, N, _s(stream)))


# ----------------------------------------------------------------- quantizers
def quantize_int4(x_out_packed, x_out_sc, in_fp32, K, stream=None):
    _chk("quantize_int4", _L.bw_quantize_int4(_p(x_out_packed), _p(x_out_sc), _p(in_fp32), K, _s(stream)))


def quantize_int4_batched(x_out_packed, x_out_sc, in_fp32, K, M, stream=None):
    _chk("quantize_int4_batched", _L.bw_quantize_int4_batched(_p(x_out_packed), _p(x_out_sc), _p(in_fp32), K, M,
                                                              _s(stream)))


def quantize_int8(out_int8, out_scale, in_fp32, num_elements, stream=None):
    _chk("quantize_int8", _L.bw_quantize_int8(_p(out_int8), _p(out_scale), _p(in_fp32), num_elements, _s(stream)))


def quantize_int8_f16(out_int8, out_scale, in_f16, num_elements, stream=None):
    _chk("quantize_int8_f16", _L.bw_quantize_int8_f16(_p(out_int8), _p(out_scale), _p(in_f16), num_elements,
                                                      _s(stream)))


def fused_rmsnorm_quant_int4(x_out_packed, x_out_scale, proj, weight, N, eps, stream=None):
    _chk("fused_rmsnorm_quant_int4", _L.bw_fused_rmsnorm_quant_int4(_p(x_out_packed), _p(x_out_scale), _p(proj),
                                                                    _p(weight), N, C.c_float(eps), _s(stream)))


def fused_swiglu_quant_int4(out_packed, out_scale, gate, up, N, stream=None):
    _chk("fused_swiglu_quant_int4", _L.bw_fused_swiglu_quant_int4(_p(out_packed), _p(out_scale), _p(gate), _p(up),
                                                                  N, _s(stream)))


# ------------------------------------------------------------ norm/elementwise
def fused_rmsnorm(out, inp, weight, num_elements, eps, stream=None):
    _chk("fused_rmsnorm", _L.bw_fused_rmsnorm(_p(out), _p(inp), _p(weight), num_elements, C.c_float(eps),
                                              _s(stream)))


def fused_rmsnorm_batched(out, inp, weight, H, eps, M, stream=None):
    _chk("fused_rmsnorm_batched", _L.bw_fused_rmsnorm_batched(_p(out), _p(inp), _p(weight), H, C.c_float(eps), M,
                                                              _s(stream)))


def apply_swiglu(out, gate, up, num_elements, stream=None):
    _chk("apply_swiglu", _L.bw_apply_swiglu(_p(out), _p(gate), _p(up), num_elements, _s(stream)))


def vector_add_fp32(out, a, b, num_elements, stream=None):
    _chk("vector_add_fp32", _L.bw_vector_add_fp32(_p(out), _p(a), _p(b), num_elements, _s(stream)))


def fused_rope_decode(out_inplace, cos_cache, sin_cache, seq_pos_ptr, heads, head_dim, max_seq_len, stream=None):
    _chk("fused_rope_decode", _L.bw_fused_rope_decode(_p(out_inplace), _p(cos_cache), _p(sin_cache),
                                                      _p(seq_pos_ptr), heads, head_dim, max_seq_len, _s(stream)))


# --------------------------------------------------------------- KV, attention
def update_kv_cache(k_cache, v_cache, k_new, v_new, batch_idx, seq_pos, num_heads, head_dim, max_seq_len,
                    stream=None):
    _chk("update_kv_cache", _L.bw_update_kv_cache(_p(k_cache), _p(v_cache), _p(k_new), _p(v_new), batch_idx,
                                                  seq_pos, num_heads, head_dim, max_seq_len, _s(stream)))


def update_kv_cache_device(k_cache, v_cache, k_new, v_new, batch_idx, d_seq_pos, num_heads, head_dim, max_seq_len,
                           stream=None):
    _chk("update_kv_cache_device", _L.bw_update_kv_cache_device(_p(k_cache), _p(v_cache), _p(k_new), _p(v_new),
                                                                batch_idx, _p(d_seq_pos), num_heads, head_dim,
                                                                max_seq_len, _s(stream)))


def attention_decode_batched_gqa(output, Q, K_cache, V_cache, seq_pos, num_q_heads, num_kv_heads, head_dim,
                                 max_seq_len, M, kv_batch_elems, kv_layer_elems, stream=None):
    _chk("attention_decode_batched_gqa", _L.bw_attention_decode_batched_gqa(
        _p(output), _p(Q), _p(K_cache), _p(V_cache), seq_pos, num_q_heads, num_kv_heads, head_dim, max_seq_len, M,
        C.c_size_t(kv_batch_elems), C.c_size_t(kv_layer_elems), _s(stream)))


def attention_decode_batched_gqa_device(output, Q, K_cache, V_cache, d_seq_pos, num_q_heads, num_kv_heads, head_dim,
                                        max_seq_len, M, kv_batch_elems, kv_layer_elems, stream=None):
    _chk("attention_decode_batched_gqa_device", _L.bw_attention_decode_batched_gqa_device(
        _p(output), _p(Q), _p(K_cache), _p(V_cache), _p(d_seq_pos), num_q_heads, num_kv_heads, head_dim,
        max_seq_len, M, C.c_size_t(kv_batch_elems), C.c_size_t(kv_layer_elems), _s(stream)))


def attention_decode_f16kv(output, Q, K_cache, V_cache, d_seq_pos, ctx_hint, num_q_heads, num_kv_heads, head_dim,
                           max_seq_len, M, kv_batch_elems, kv_layer_elems, stream=None):
    _chk("attention_decode_f16kv", _L.bw_attention_decode_f16kv(
        _p(output), _p(Q), _p(K_cache), _p(V_cache), _p(d_seq_pos), ctx_hint, num_q_heads, num_kv_heads, head_dim,
        max_seq_len, M, C.c_size_t(kv_batch_elems), C.c_size_t(kv_layer_elems), _s(stream)))


# ------------------------------------------------------------------- sampling
def sample_argmax_gpu(logits, vocab, out_id, stream=None):
    _chk("sample_argmax_gpu", _L.bw_sample_argmax_gpu(_p(logits), vocab, _p(out_id), _s(stream)))


def sample_gpu(logits, vocab, temperature, top_k, out_id, rng_seed, step, stream=None):
    _chk("sample_gpu", _L.bw_sample_gpu(_p(logits), vocab, C.c_float(temperature), top_k, _p(out_id),
                                        C.c_ulonglong(rng_seed), step, _s(stream)))


def apply_repetition_penalty(logits, recent, num_recent, penalty, vocab, stream=None):
    _chk("apply_repetition_penalty", _L.bw_apply_repetition_penalty(_p(logits), _p(recent), num_recent,
                                                                    C.c_float(penalty), vocab, _s(stream)))


# -------------------------------------------------------------------- service
def device_status() -> int:
    v = C.c_int(0)
    _chk("device_status", _L.bw_device_status(C.byref(v)))
    return v.value


def set_tuning(key: int, value: int) -> None:
    _chk("set_tuning", _L.bw_set_tuning(key, value))


def launch_count(reset: bool = False) -> int:
    return int(_L.bw_launch_count(1 if reset else 0))


def attention_decode_batched_gqa_noalloc(output, Q, K_cache, V_cache, d_seq_pos, num_q_heads, num_kv_heads,
                                         head_dim, max_seq_len, M, kv_batch_elems, kv_layer_elems, stream=None):
    """Attention for callers that must not allocate (no counterpart in the reference): same arguments and
    results as ``attention_decode_batched_gqa_device``, split partials in a fixed 2 MiB array of the library."""
    _chk("attention_decode_batched_gqa_noalloc", _L.bw_attention_decode_batched_gqa_noalloc(
        _p(output), _p(Q), _p(K_cache), _p(V_cache), _p(d_seq_pos), num_q_heads, num_kv_heads, head_dim,
        max_seq_len, M, C.c_size_t(kv_batch_elems), C.c_size_t(kv_layer_elems), _s(stream)))


# ------------------------------------------------------------ decode-step glue
def gemv_w4a8_decode(y_out, y_stride, residual, x_f32, up, x_stride, norm_weight, eps, W_packed, W_scale_f16, K, N,
                     M, stream=None):
    _chk("gemv_w4a8_decode", _L.bw_gemv_w4a8_decode(
        _p(y_out), C.c_long(y_stride), _p(residual), _p(x_f32), _p(up), C.c_long(x_stride), _p(norm_weight),
        C.c_float(eps), _p(W_packed), _p(W_scale_f16), K, N, M, _s(stream)))


class _PendingArgs(C.Structure):
    _fields_ = [("y", C.c_void_p), ("residual", C.c_void_p), ("x_q", C.c_void_p), ("x_scale", C.c_void_p),
                ("x_block_sumsq", C.c_void_p), ("eps", C.c_float), ("gate", C.c_void_p), ("up", C.c_void_p),
                ("W_packed", C.c_void_p), ("W_scale_f16", C.c_void_p), ("K", C.c_int), ("N", C.c_int),
                ("next_norm_w", C.c_void_p), ("next_q", C.c_void_p), ("next_scale", C.c_void_p),
                ("next_block_sumsq", C.c_void_p), ("M", C.c_int), ("x_stride", C.c_long)]


def gemv_w4a8_pending(y, residual, W_packed, W_scale_f16, K, N, x_q=None, x_scale=None, x_block_sumsq=None, eps=0.0,
                      gate=None, up=None, next_norm_w=None, next_q=None, next_scale=None, next_block_sumsq=None,
                      M=1, x_stride=0, stream=None):
    """GEMV with the norm-pending hand-over (bw_gemv_w4a8_pending), 1 or 5..16 sequences."""
    def vp(t):
        if t is None:
            return None
        return t if isinstance(t, int) else t.data_ptr()

    a = _PendingArgs(vp(y), vp(residual), vp(x_q), vp(x_scale), vp(x_block_sumsq), float(eps), vp(gate), vp(up),
                     vp(W_packed), vp(W_scale_f16), K, N, vp(next_norm_w), vp(next_q), vp(next_scale),
                     vp(next_block_sumsq), int(M), int(x_stride))
    _chk("gemv_w4a8_pending", _L.bw_gemv_w4a8_pending(C.byref(a), _s(stream)))


def gemv_w4a8_q8_decode(y_out, y_stride, residual, x_q, x_scale, W_packed, W_scale_f16, K, N, M, stream=None):
    _chk("gemv_w4a8_q8_decode", _L.bw_gemv_w4a8_q8_decode(
        _p(y_out), C.c_long(y_stride), _p(residual), _p(x_q), _p(x_scale), _p(W_packed), _p(W_scale_f16), K, N, M,
        _s(stream)))


def qk_norm_rope_kv_f16(q_out, k_cache, v_cache, qkv, q_norm_w, k_norm_w, d_seq_pos, num_q_heads, num_kv_heads,
                        head_dim, max_seq_len, M, kv_batch_elems, kv_layer_elems, eps, rope_base, stream=None):
    _chk("qk_norm_rope_kv_f16", _L.bw_qk_norm_rope_kv_f16(
        _p(q_out), _p(k_cache), _p(v_cache), _p(qkv), _p(q_norm_w), _p(k_norm_w), _p(d_seq_pos), num_q_heads,
        num_kv_heads, head_dim, max_seq_len, M, C.c_size_t(kv_batch_elems), C.c_size_t(kv_layer_elems),
        C.c_float(eps), C.c_float(rope_base), _s(stream)))


def embed_gather_f16(x_out, table_f16, d_tokens, H, vocab, M, stream=None):
    _chk("embed_gather_f16", _L.bw_embed_gather_f16(_p(x_out), _p(table_f16), _p(d_tokens), H, vocab, M, _s(stream)))


def sample_argmax_batched(logits, row_stride, vocab, M, out_ids, seq_pos_to_advance=None, pos_limit=0, stream=None):
    _chk("sample_argmax_batched", _L.bw_sample_argmax_batched(_p(logits), C.c_long(row_stride), vocab, M,
                                                              _p(out_ids), _p(seq_pos_to_advance), int(pos_limit),
                                                              _s(stream)))


def sample_argmax_candidates(logits, row_stride, vocab, M, index_offset, cand_out_pairs, stream=None):
    _chk("sample_argmax_candidates", _L.bw_sample_argmax_candidates(_p(logits), C.c_long(row_stride), vocab, M,
                                                                    int(index_offset), _p(cand_out_pairs), _s(stream)))


def sample_argmax_merge(cand_all_pairs, world, M, out_ids, seq_pos_to_advance=None, pos_limit=0, stream=None):
    _chk("sample_argmax_merge", _L.bw_sample_argmax_merge(_p(cand_all_pairs), world, M, _p(out_ids),
                                                          _p(seq_pos_to_advance), int(pos_limit), _s(stream)))


def attention_decode_f16kv_fused_q8(output, out_q8, out_scale, qkv, q_norm_w, k_norm_w, k_cache, v_cache, d_seq_pos,
                                    ctx_hint, num_q_heads, num_kv_heads, head_dim, max_seq_len, M, kv_batch_elems,
                                    kv_layer_elems, eps, rope_base, stream=None):
    _chk("attention_decode_f16kv_fused_q8", _L.bw_attention_decode_f16kv_fused_q8(
        _p(output), _p(out_q8), _p(out_scale), _p(qkv), _p(q_norm_w), _p(k_norm_w), _p(k_cache), _p(v_cache),
        _p(d_seq_pos), ctx_hint, num_q_heads, num_kv_heads, head_dim, max_seq_len, M, C.c_size_t(kv_batch_elems),
        C.c_size_t(kv_layer_elems), C.c_float(eps), C.c_float(rope_base), _s(stream)))


def attention_decode_f16kv_fused(output, qkv, q_norm_w, k_norm_w, k_cache, v_cache, d_seq_pos, ctx_hint, num_q_heads,
                                 num_kv_heads, head_dim, max_seq_len, M, kv_batch_elems, kv_layer_elems, eps, rope_base,
                                 stream=None):
    _chk("attention_decode_f16kv_fused", _L.bw_attention_decode_f16kv_fused(
        _p(output), _p(qkv), _p(q_norm_w), _p(k_norm_w), _p(k_cache), _p(v_cache), _p(d_seq_pos), ctx_hint,
        num_q_heads, num_kv_heads, head_dim, max_seq_len, M, C.c_size_t(kv_batch_elems), C.c_size_t(kv_layer_elems),
        C.c_float(eps), C.c_float(rope_base), _s(stream)))
