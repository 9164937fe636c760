"""Synthetic INT4 decode step for a Qwen3-shaped model, driven through the C ABI.

The call sequence is the reference's per-layer loop
(server/inference_server_int4_batched.cu:253-298) with the fusions applied: per layer

    qkv  = W_qkv  . q8(rmsnorm(x, rn_in))                      bw_gemv_w4a8_decode (norm prologue)
    q, K[pos], V[pos] = head-norm + RoPE + cache write          bw_qk_norm_rope_kv_f16
    attn = GQA attention over the binary16 cache                bw_attention_decode_f16kv
    x    = x + W_o . q8(attn)                                   bw_gemv_w4a8_decode (residual epilogue)
    gu   = W_gu . q8(rmsnorm(x, rn_post))                       bw_gemv_w4a8_decode (norm prologue)
    x    = x + W_down . q8(silu(gate) * up)                     bw_gemv_w4a8_decode (SwiGLU prologue + residual)

then logits = W_lm . q8(rmsnorm(x, rn_final)), greedy argmax, positions + 1, and the embedding lookup of the
next step reads the sampled ids from device memory, so a whole step is one CUDA graph.  Weights are random-init
in the block-16 INT4 format (no checkpoint is available offline).  With ``world > 1`` the layer is tensor-parallel:
QKV / gate+up / LM head by rows (whole heads), O / down along K, an all-reduce after O and after down, and an
all-gather of the per-rank (value, index) argmax candidates.
"""
from __future__ import annotations

import numpy as np
import torch

from . import kernels as k
from . import synth
from .shapes import ModelShape

ROPE_BASE = 1000000.0


class DecodeEngine:
    def __init__(self, shape: ModelShape, batch: int, max_seq: int, device, seed: int = 0, world: int = 1,
                 rank: int = 0, host_weights=None, exchange: str = "nccl"):
        assert shape.head_dim == 128
        assert shape.n_q_heads % world == 0 and shape.n_kv_heads % world == 0, "heads must split evenly"
        self.s, self.M, self.max_seq, self.dev = shape, batch, max_seq, device
        self.world, self.rank = world, rank
        # "nccl": torch.distributed all-reduce; "peer": the library's all-reduce over NVLink peer loads, the partial
        # sums written by the GEMV straight into the exchanged buffer
        assert exchange in ("nccl", "peer")
        self.exchange = exchange if world > 1 else "nccl"
        self.nq = shape.n_q_heads // world
        self.nkv = shape.n_kv_heads // world
        H, I = shape.hidden, shape.inter
        # K shards of the down projection on 32-element boundaries
        units = I // 32
        base, rem = divmod(units, world)
        self.i_local = (base + (1 if rank < rem else 0)) * 32
        self.i0 = (rank * base + min(rank, rem)) * 32
        v_base, v_rem = divmod(shape.vocab, world)
        self.v_local = v_base + (1 if rank < v_rem else 0)
        self.v0 = rank * v_base + min(rank, v_rem)
        self.qkv_n = (self.nq + 2 * self.nkv) * 128
        f32, dev = torch.float32, device
        M = batch

        def W(N, K, sd):
            if host_weights is not None:
                return host_weights(N, K, sd)
            return synth.int4_weights_device(N, K, sd, device=dev)

        self.layers = []
        for l in range(shape.layers):
            sd = seed + 1000 * l + 17 * rank
            L = {
                "qkv": W(self.qkv_n, H, sd + 1), "o": W(H, self.nq * 128, sd + 2),
                "gu": W(2 * self.i_local, H, sd + 3), "down": W(H, self.i_local, sd + 4),
                "rn_in": self._normw(H, seed + 1000 * l + 5), "rn_post": self._normw(H, seed + 1000 * l + 6),
                "qn": self._normw(128, seed + 1000 * l + 7), "kn": self._normw(128, seed + 1000 * l + 8),
            }
            self.layers.append(L)
        self.lm = W(self.v_local, H, seed + 900001 + 17 * rank)
        self.rn_final = self._normw(H, seed + 900002)
        self.embed = synth.activations_f16_device(shape.vocab, H, seed + 900003, device=dev) if host_weights is None \
            else host_weights("embed", shape.vocab, H)

        self.kv_layer = self.nkv * max_seq * 128
        self.kv_batch = shape.layers * self.kv_layer
        self.kc = torch.zeros((M, self.kv_batch), dtype=torch.float16, device=dev)
        self.vc = torch.zeros((M, self.kv_batch), dtype=torch.float16, device=dev)
        self.x = torch.zeros((M, H), dtype=f32, device=dev)
        self.qkv = torch.zeros((M, self.qkv_n), dtype=f32, device=dev)
        self.q = torch.zeros((M, self.nq * 128), dtype=f32, device=dev)
        self.attn = torch.zeros((M, self.nq * 128), dtype=f32, device=dev)
        self.gu = torch.zeros((M, 2 * self.i_local), dtype=f32, device=dev)
        self.part = torch.zeros((M, H), dtype=f32, device=dev)
        self.logits = torch.zeros((M, self.v_local), dtype=f32, device=dev)
        self.tokens = torch.zeros((M,), dtype=torch.int32, device=dev)
        self.pos = torch.zeros((M,), dtype=torch.int32, device=dev)
        self.ctx_hint = max_seq
        self.peer = None
        if self.exchange == "peer":
            from .peer import PeerComm

            self.peer = PeerComm(world, rank, M * H, dev)
            self.peer.connect_processes()
            self.peer_slots = [self.peer.slot(0, M, H), self.peer.slot(1, M, H)]
        if world > 1:
            self.cand = torch.zeros((M, 2), dtype=f32, device=dev)
            self.cand_all = torch.zeros((world, M, 2), dtype=f32, device=dev)

    def _normw(self, n, sd):
        return torch.from_numpy(synth.norm_weight(n, sd)).to(self.dev)

    # ------------------------------------------------------------------
    def fill_cache(self, ctx: int, seed: int = 77):
        """Pre-fills the cache with N(0,1) up to position ctx-1 and sets every sequence's position to ctx-1... the
        step then writes position ``ctx - 1`` itself, so pos starts at ctx - 1."""
        g = torch.Generator(device=self.dev)
        g.manual_seed(synth.SEED_BASE + seed + self.rank)
        for c in (self.kc, self.vc):
            v = c.view(self.M, self.s.layers, self.nkv, self.max_seq, 128)
            for l in range(self.s.layers):  # layer by layer: the fp32 staging buffer stays small
                tmp = torch.empty((self.M, self.nkv, ctx, 128), dtype=torch.float32, device=self.dev)
                tmp.normal_(0.0, 1.0, generator=g)
                v[:, l, :, :ctx].copy_(tmp)
                del tmp
        self.pos.fill_(ctx - 1)
        self.ctx_hint = min(self.max_seq, ctx + 64)

    def set_tokens(self, ids):
        self.tokens.copy_(torch.as_tensor(ids, dtype=torch.int32))

    def _partial_target(self):
        """Where the K-split GEMV writes its partial sums: a local tensor (NCCL) or the next exchange slot."""
        if self.peer is None:
            return self.part
        self._slot = self.peer.next_slot()
        return self.peer_slots[self._slot]

    def _exchange(self, part):
        """Sums the partial results over the ranks; afterwards ``self.x`` holds the new hidden state on every rank.
        A step makes an even number of exchanges (two per layer), so the slot order 0, 1, 0, 1 ... also holds across
        replays of a captured step."""
        if self.peer is None:
            import torch.distributed as dist

            dist.all_reduce(part)
            self.x, self.part = self.part, self.x
        else:
            self.peer.allreduce(self._slot, self.x, self.M * self.s.hidden)

    def step(self):
        """Enqueues one decode step for the whole batch on the current stream."""
        s, M, H = self.s, self.M, self.s.hidden
        eps = s.eps
        k.embed_gather_f16(self.x, self.embed, self.tokens, H, s.vocab, M)
        for l, L in enumerate(self.layers):
            off = l * self.kv_layer
            k.gemv_w4a8_decode(self.qkv, 0, None, self.x, None, 0, L["rn_in"], eps, L["qkv"][0], L["qkv"][1], H,
                               self.qkv_n, M)
            k.qk_norm_rope_kv_f16(self.q, self.kc, self.vc, self.qkv, L["qn"], L["kn"], self.pos, self.nq, self.nkv,
                                  128, self.max_seq, M, self.kv_batch, off, eps, ROPE_BASE)
            k.attention_decode_f16kv(self.attn, self.q, self.kc, self.vc, self.pos, self.ctx_hint, self.nq, self.nkv,
                                     128, self.max_seq, M, self.kv_batch, off)
            if self.world == 1:
                k.gemv_w4a8_decode(self.x, 0, self.x, self.attn, None, 0, None, 0.0, L["o"][0], L["o"][1],
                                   self.nq * 128, H, M)
            else:
                res = self.x if self.rank == 0 else None  # the residual enters the sum once
                part = self._partial_target()
                k.gemv_w4a8_decode(part, 0, res, self.attn, None, 0, None, 0.0, L["o"][0], L["o"][1],
                                   self.nq * 128, H, M)
                self._exchange(part)
            k.gemv_w4a8_decode(self.gu, 0, None, self.x, None, 0, L["rn_post"], eps, L["gu"][0], L["gu"][1], H,
                               2 * self.i_local, M)
            gate, up = self.gu, self.gu[:, self.i_local:]
            if self.world == 1:
                k.gemv_w4a8_decode(self.x, 0, self.x, gate, up.data_ptr(), 2 * self.i_local, None, 0.0, L["down"][0],
                                   L["down"][1], self.i_local, H, M)
            else:
                res = self.x if self.rank == 0 else None
                part = self._partial_target()
                k.gemv_w4a8_decode(part, 0, res, gate, up.data_ptr(), 2 * self.i_local, None, 0.0, L["down"][0],
                                   L["down"][1], self.i_local, H, M)
                self._exchange(part)
        k.gemv_w4a8_decode(self.logits, 0, None, self.x, None, 0, self.rn_final, eps, self.lm[0], self.lm[1], H,
                           self.v_local, M)
        if self.world == 1:
            k.sample_argmax_batched(self.logits, self.v_local, self.v_local, M, self.tokens, self.pos, self.max_seq - 1)
        else:
            self._tp_argmax()

    def _tp_argmax(self):
        """Local argmax, then an all-gather of (value, global index) pairs instead of 600 KB of logits."""
        import torch.distributed as dist

        M = self.M
        loc = torch.empty((M,), dtype=torch.int32, device=self.dev) if not hasattr(self, "_loc") else self._loc
        self._loc = loc
        k.sample_argmax_batched(self.logits, self.v_local, self.v_local, M, loc, self.pos, self.max_seq - 1)
        idx = loc.long()
        self.cand[:, 0] = self.logits.gather(1, idx[:, None])[:, 0]
        self.cand[:, 1] = (idx + self.v0).float()
        dist.all_gather_into_tensor(self.cand_all.view(-1), self.cand.view(-1))
        best = self.cand_all[:, :, 0].argmax(dim=0)
        self.tokens.copy_(self.cand_all[best, torch.arange(M, device=self.dev), 1].int())

    # bytes one step must read from HBM on this rank: weights once + the cache rows in use
    def step_bytes(self, ctx: int) -> int:
        wbytes = 0
        for L in self.layers:
            for key in ("qkv", "o", "gu", "down"):
                wbytes += L[key][0].numel() + L[key][1].numel() * 2
        wbytes += self.lm[0].numel() + self.lm[1].numel() * 2
        kv = 2 * self.M * self.s.layers * self.nkv * ctx * 128 * 2
        return wbytes + kv
