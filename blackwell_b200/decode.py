"""Synthetic INT4 decode step for a Qwen3-shaped model, driven through the C ABI.

The call sequence is the reference's per-layer loop
(server/inference_server_int4_batched.cu:253-298) with the fusions applied: per layer

    qkv  = W_qkv  . q8(rmsnorm(x, rn_in))                      bw_gemv_w4a8_decode (norm prologue)
    q, K[pos], V[pos] = head-norm + RoPE + cache write          bw_qk_norm_rope_kv_f16        } one launch with 4 or 8 query
    attn = GQA attention over the binary16 cache                bw_attention_decode_f16kv     } heads per kv head (_fused)
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
                 rank: int = 0, host_weights=None, exchange: str = "nccl", consistent: bool = False):
        """``consistent``: every rank derives its shard from the FULL matrices of one seed (generated on the host, so
        only for small shapes), which makes a tensor-parallel step comparable with the single-GPU one; otherwise each
        rank draws its own shard directly in HBM (benchmark sizes)."""
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

        def W(N, K, sd, kind=None):
            if host_weights is not None:
                return host_weights(N, K, sd)
            if consistent:
                return self._shard_of_full(kind, sd - 17 * rank)
            return synth.int4_weights_device(N, K, sd, device=dev)

        self.layers = []
        for l in range(shape.layers):
            sd = seed + 1000 * l + 17 * rank
            L = {
                "qkv": W(self.qkv_n, H, sd + 1, "qkv"), "o": W(H, self.nq * 128, sd + 2, "o"),
                "gu": W(2 * self.i_local, H, sd + 3, "gu"), "down": W(H, self.i_local, sd + 4, "down"),
                "rn_in": self._normw(H, seed + 1000 * l + 5), "rn_post": self._normw(H, seed + 1000 * l + 6),
                "qn": self._normw(128, seed + 1000 * l + 7), "kn": self._normw(128, seed + 1000 * l + 8),
            }
            self.layers.append(L)
        self.lm = W(self.v_local, H, seed + 900001 + 17 * rank, "lm")
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
        self.attn_q = torch.zeros((M, self.nq * 128), dtype=torch.int8, device=dev)      # the same, block-16 int8
        self.attn_qs = torch.zeros((M, self.nq * 8), dtype=f32, device=dev)
        # norm-pending hand-over between the GEMVs of a step (one sequence, one GPU): two sets, x after O and after down
        self.pend = [(torch.zeros((M, self.s.hidden), dtype=torch.int8, device=dev),
                      torch.zeros((M, self.s.hidden // 16), dtype=f32, device=dev),
                      torch.zeros((M, self.s.hidden // 16), dtype=f32, device=dev)) for _ in range(2)]
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
            self.cand = torch.zeros((M, 2), dtype=torch.int32, device=dev)
            self.cand_all = torch.zeros((world, M, 2), dtype=torch.int32, device=dev)

    def _normw(self, n, sd):
        return torch.from_numpy(synth.norm_weight(n, sd)).to(self.dev)

    def _shard_of_full(self, kind, sd):
        """This rank's shard of the full matrix of seed ``sd``: rows by whole heads (qkv), by the same range of gate
        and up (gu), by vocabulary range (lm); columns on 32-element boundaries (o: this rank's heads; down: its
        slice of the intermediate size)."""
        s, r, w = self.s, self.rank, self.world
        H, I = s.hidden, s.inter
        nqf, nkvf = s.n_q_heads, s.n_kv_heads
        if kind == "qkv":
            Wf, scf, _ = synth.int4_weights((nqf + 2 * nkvf) * 128, H, sd)
            rows = np.concatenate([np.arange(r * self.nq * 128, (r + 1) * self.nq * 128),
                                   nqf * 128 + np.arange(r * self.nkv * 128, (r + 1) * self.nkv * 128),
                                   (nqf + nkvf) * 128 + np.arange(r * self.nkv * 128, (r + 1) * self.nkv * 128)])
            Wl, scl = Wf[rows], scf[rows]
        elif kind == "gu":
            Wf, scf, _ = synth.int4_weights(2 * I, H, sd)
            rows = np.concatenate([np.arange(self.i0, self.i0 + self.i_local), I + np.arange(self.i0, self.i0 + self.i_local)])
            Wl, scl = Wf[rows], scf[rows]
        elif kind == "lm":
            Wf, scf, _ = synth.int4_weights(s.vocab, H, sd)
            Wl, scl = Wf[self.v0:self.v0 + self.v_local], scf[self.v0:self.v0 + self.v_local]
        elif kind == "o":
            Wf, scf, _ = synth.int4_weights(H, nqf * 128, sd)
            k0, kl = r * self.nq * 128, self.nq * 128
            Wl, scl = Wf[:, k0 // 2:(k0 + kl) // 2], scf[:, k0 // 16:(k0 + kl) // 16]
        elif kind == "down":
            Wf, scf, _ = synth.int4_weights(H, I, sd)
            Wl, scl = Wf[:, self.i0 // 2:(self.i0 + self.i_local) // 2], scf[:, self.i0 // 16:(self.i0 + self.i_local) // 16]
        else:
            raise ValueError(kind)
        Wd = torch.from_numpy(np.ascontiguousarray(Wl)).to(self.dev)
        sd_ = torch.from_numpy(np.ascontiguousarray(scl).view(np.int16)).to(self.dev).view(torch.float16)
        return Wd, sd_

    def fill_cache_consistent(self, ctx: int, seed: int = 77):
        """Like fill_cache, but the cache of the FULL model is drawn on the host from one seed and this rank keeps its
        kv heads, so that every world size sees the same context (small shapes only)."""
        full = synth.kv_cache_f16((2, self.M, self.s.layers, self.s.n_kv_heads, ctx, 128), seed)
        h0 = self.rank * self.nkv
        for c, src in ((self.kc, full[0]), (self.vc, full[1])):
            v = c.view(self.M, self.s.layers, self.nkv, self.max_seq, 128)
            part = np.ascontiguousarray(src[:, :, h0:h0 + self.nkv]).view(np.int16)
            v[:, :, :, :ctx].copy_(torch.from_numpy(part).to(self.dev).view(torch.float16))
        self.pos.fill_(ctx - 1)
        self.ctx_hint = min(self.max_seq, ctx + 64)

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
        # One sequence on one GPU: the O and down projections hand their result to the next GEMV already quantized
        # (bw_gemv_w4a8_pending), so that no CTA of the QKV / gate+up / LM-head GEMVs quantizes the hidden state.  (The
        # entry point also serves 5..16 sequences; there the hand-over measured no faster than the prep launches.)
        pending = M == 1 and self.world == 1 and self.nq // self.nkv in (4, 8) and H % 16 == 0
        pa, pb = self.pend
        for l, L in enumerate(self.layers):
            off = l * self.kv_layer
            if pending and l > 0:
                k.gemv_w4a8_pending(self.qkv, None, L["qkv"][0], L["qkv"][1], H, self.qkv_n, x_q=pb[0], x_scale=pb[1],
                                    x_block_sumsq=pb[2], eps=eps, M=M)
            else:
                k.gemv_w4a8_decode(self.qkv, 0, None, self.x, None, 0, L["rn_in"], eps, L["qkv"][0], L["qkv"][1], H,
                                   self.qkv_n, M)
            fused = self.nq // self.nkv in (4, 8)
            if fused:   # head norm + RoPE + KV write inside the tensor-core attention kernel, which also quantizes its
                # result for the O projection (the float copy is kept for inspection)
                k.attention_decode_f16kv_fused_q8(self.attn, self.attn_q, self.attn_qs, self.qkv, L["qn"], L["kn"],
                                                  self.kc, self.vc, self.pos, self.ctx_hint, self.nq, self.nkv, 128,
                                                  self.max_seq, M, self.kv_batch, off, eps, ROPE_BASE)
            else:
                k.qk_norm_rope_kv_f16(self.q, self.kc, self.vc, self.qkv, L["qn"], L["kn"], self.pos, self.nq,
                                      self.nkv, 128, self.max_seq, M, self.kv_batch, off, eps, ROPE_BASE)
                k.attention_decode_f16kv(self.attn, self.q, self.kc, self.vc, self.pos, self.ctx_hint, self.nq,
                                         self.nkv, 128, self.max_seq, M, self.kv_batch, off)
            def o_proj(y, res):
                if fused:
                    k.gemv_w4a8_q8_decode(y, 0, res, self.attn_q, self.attn_qs, L["o"][0], L["o"][1], self.nq * 128, H, M)
                else:
                    k.gemv_w4a8_decode(y, 0, res, self.attn, None, 0, None, 0.0, L["o"][0], L["o"][1], self.nq * 128,
                                       H, M)

            if pending:
                k.gemv_w4a8_pending(self.x, self.x, L["o"][0], L["o"][1], self.nq * 128, H, x_q=self.attn_q,
                                    x_scale=self.attn_qs, next_norm_w=L["rn_post"], next_q=pa[0], next_scale=pa[1],
                                    next_block_sumsq=pa[2], M=M)
            elif self.world == 1:
                o_proj(self.x, self.x)
            else:
                part = self._partial_target()
                o_proj(part, self.x if self.rank == 0 else None)   # the residual enters the sum once
                self._exchange(part)
            if pending:
                k.gemv_w4a8_pending(self.gu, None, L["gu"][0], L["gu"][1], H, 2 * self.i_local, x_q=pa[0],
                                    x_scale=pa[1], x_block_sumsq=pa[2], eps=eps, M=M)
            else:
                k.gemv_w4a8_decode(self.gu, 0, None, self.x, None, 0, L["rn_post"], eps, L["gu"][0], L["gu"][1], H,
                                   2 * self.i_local, M)
            gate, up = self.gu, self.gu[:, self.i_local:]
            if pending:
                nxt = self.layers[l + 1]["rn_in"] if l + 1 < len(self.layers) else self.rn_final
                k.gemv_w4a8_pending(self.x, self.x, L["down"][0], L["down"][1], self.i_local, H, gate=gate,
                                    up=up.data_ptr(), next_norm_w=nxt, next_q=pb[0], next_scale=pb[1],
                                    next_block_sumsq=pb[2], M=M, x_stride=2 * self.i_local)
            elif self.world == 1:
                k.gemv_w4a8_decode(self.x, 0, self.x, gate, up.data_ptr(), 2 * self.i_local, None, 0.0, L["down"][0],
                                   L["down"][1], self.i_local, H, M)
            else:
                res = self.x if self.rank == 0 else None
                part = self._partial_target()
                k.gemv_w4a8_decode(part, 0, res, gate, up.data_ptr(), 2 * self.i_local, None, 0.0, L["down"][0],
                                   L["down"][1], self.i_local, H, M)
                self._exchange(part)
        if pending:
            k.gemv_w4a8_pending(self.logits, None, self.lm[0], self.lm[1], H, self.v_local, x_q=pb[0], x_scale=pb[1],
                                x_block_sumsq=pb[2], eps=eps, M=M)
        else:
            k.gemv_w4a8_decode(self.logits, 0, None, self.x, None, 0, self.rn_final, eps, self.lm[0], self.lm[1], H,
                               self.v_local, M)
        if self.world == 1:
            k.sample_argmax_batched(self.logits, self.v_local, self.v_local, M, self.tokens, self.pos, self.max_seq - 1)
        else:
            self._tp_argmax()

    def _tp_argmax(self):
        """Local argmax into one (value, global index) pair per sequence, an all-gather of the pairs instead of
        600 KB of logits, and one kernel that picks the winner and advances the positions."""
        import torch.distributed as dist

        M = self.M
        k.sample_argmax_candidates(self.logits, self.v_local, self.v_local, M, self.v0, self.cand)
        dist.all_gather_into_tensor(self.cand_all.view(-1), self.cand.view(-1))
        k.sample_argmax_merge(self.cand_all, self.world, M, self.tokens, self.pos, self.max_seq - 1)

    # bytes one step must read from HBM on this rank: weights once + the cache rows in use
    def step_bytes(self, ctx: int) -> int:
        wbytes = 0
        for L in self.layers:
            for key in ("qkv", "o", "gu", "down"):
                wbytes += L[key][0].numel() + L[key][1].numel() * 2
        wbytes += self.lm[0].numel() + self.lm[1].numel() * 2
        kv = 2 * self.M * self.s.layers * self.nkv * ctx * 128 * 2
        return wbytes + kv
