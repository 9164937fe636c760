"""ctypes binding of the C decode-step driver (``bw_decode_*``, csrc/decode_engine.cu): a batched greedy generation
whose every step is one replay of a CUDA graph captured inside the library.  Used by the tests; a C or C++ host calls
the same functions directly (see include/blackwell_b200.h)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .kernels import KernelError, _s
from .shapes import ModelShape


class _Config(C.Structure):
    _fields_ = [("layers", C.c_int), ("hidden", C.c_int), ("inter", C.c_int), ("n_q_heads", C.c_int),
                ("n_kv_heads", C.c_int), ("head_dim", C.c_int), ("vocab", C.c_int), ("eps", C.c_float),
                ("rope_base", C.c_float), ("batch", C.c_int), ("max_seq", C.c_int), ("max_prompt", C.c_int),
                ("max_new", C.c_int), ("act_bits", C.c_int), ("use_graph", C.c_int), ("weights_dir", C.c_char_p)]


_L = _lib.load()
_L.bw_decode_create.argtypes = [C.POINTER(_Config), C.POINTER(C.c_void_p)]
_L.bw_decode_begin.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
_L.bw_decode_step.argtypes = [C.c_void_p, C.c_void_p]
_L.bw_decode_result.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
_L.bw_decode_buffers.argtypes = [C.c_void_p] + [C.POINTER(C.c_void_p)] * 6
_L.bw_decode_destroy.argtypes = [C.c_void_p]


def _chk(name, code):
    if code != 0:
        raise KernelError(name, code)


class DecodeDriver:
    def __init__(self, shape: ModelShape, weights_dir: str, batch: int, max_seq: int, max_prompt: int, max_new: int,
                 act_bits: int = 8, use_graph: bool = True, rope_base: float = 1000000.0):
        self.shape, self.batch, self.max_seq, self.max_new = shape, batch, max_seq, max_new
        cfg = _Config(shape.layers, shape.hidden, shape.inter, shape.n_q_heads, shape.n_kv_heads, shape.head_dim,
                      shape.vocab, shape.eps, rope_base, batch, max_seq, max_prompt, max_new, act_bits,
                      1 if use_graph else 0, weights_dir.encode())
        h = C.c_void_p()
        _chk("bw_decode_create", _L.bw_decode_create(C.byref(cfg), C.byref(h)))
        self._h = h

    def begin(self, prompts, stream=None):
        """prompts: list of ``batch`` lists of token ids (each at least one id)."""
        assert len(prompts) == self.batch
        longest = max(len(p) for p in prompts)
        table = np.zeros((self.batch, longest), np.int32)
        lens = np.zeros(self.batch, np.int32)
        for m, p in enumerate(prompts):
            table[m, :len(p)] = p
            lens[m] = len(p)
        _chk("bw_decode_begin", _L.bw_decode_begin(self._h, table.ctypes.data, lens.ctypes.data, longest, _s(stream)))

    def step(self, stream=None):
        _chk("bw_decode_step", _L.bw_decode_step(self._h, _s(stream)))

    def result(self, stream=None) -> np.ndarray:
        out = np.empty((self.batch, self.max_new), np.int32)
        _chk("bw_decode_result", _L.bw_decode_result(self._h, out.ctypes.data, _s(stream)))
        return out

    def buffers(self):
        """Device buffers as torch tensors: logits, hidden, positions, sampled ids, K cache, V cache."""
        import torch

        ptrs = [C.c_void_p() for _ in range(6)]
        _chk("bw_decode_buffers", _L.bw_decode_buffers(self._h, *[C.byref(p) for p in ptrs]))
        s, M = self.shape, self.batch
        kv = M * s.layers * s.n_kv_heads * self.max_seq * 128

        def view(ptr, n, typestr, dtype):
            class _H:
                pass

            h = _H()
            h.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (int(ptr.value), False), "version": 2}
            return torch.as_tensor(h, device="cuda").view(dtype) if dtype is not None else torch.as_tensor(h, device="cuda")

        return {
            "logits": view(ptrs[0], M * s.vocab, "<f4", None).view(M, s.vocab),
            "hidden": view(ptrs[1], M * s.hidden, "<f4", None).view(M, s.hidden),
            "pos": view(ptrs[2], M, "<i4", None),
            "sampled": view(ptrs[3], M, "<i4", None),
            "kc": view(ptrs[4], kv, "<i2", torch.float16).view(M, s.layers, s.n_kv_heads, self.max_seq, 128),
            "vc": view(ptrs[5], kv, "<i2", torch.float16).view(M, s.layers, s.n_kv_heads, self.max_seq, 128),
        }

    def close(self):
        if self._h:
            _L.bw_decode_destroy(self._h)
            self._h = None
