"""Sub-layer blocks that are not tied to one model family: latent attention (with and without a rotated key part) and
routed experts.

Each block owns its weights in the layout its kernels want and exposes ``in_rows()`` -- the projection rows
that read the block's input -- so that a layer can stack the rows of all its blocks into ONE input GEMM
(the same fusion the multi-head families use for [q | k | v | up]).  All sizes and constants are constructor
arguments.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..ops import ACT_RELU2
from ..utils.tracing import trace


class LatentAttention:
    """Multi-head attention over a low-rank latent, no positional rotation.

        q = W_q h                  [heads * dim]
        c = rmsnorm(W_dkv h) * g   [rank]           <- the only thing cached
        k_h = W_uk,h c , v_h = W_uv,h c ;  o_h = softmax(scale * q_h . k_h) v_h   (causal)
        out = W_o concat_h(gate_h * o_h)            gate = sigmoid(W_g h) per head, if ``gated``

    Executed in the absorbed form (csrc/latent_attn.cu): q~_h = W_uk,h^T q_h, attention with key = value = c,
    o_h = W_uv,h o~_h.  The output gate rides on the epilogue of the last per-head product."""

    def __init__(self, heads: int, dim: int, vdim: int, rank: int, scale: float, gated: bool, eps: float):
        self.heads, self.dim, self.vdim, self.rank, self.scale, self.gated, self.eps = heads, dim, vdim, rank, scale, gated, eps
        self.w_q = self.w_dkv = self.w_g = self.norm_w = self.w_uk = self.w_uv = self.w_o = None

    def in_rows(self):
        rows = [self.w_q, self.w_dkv] + ([self.w_g] if self.gated else [])
        return torch.cat(rows, dim=0)

    def bind(self, base: int):
        """Column offsets of this block's outputs inside the layer's fused projection; returns the next free column."""
        self.q_off = base
        self.c_off = base + self.heads * self.dim
        self.g_off = self.c_off + self.rank if self.gated else -1
        self.w_q = self.w_dkv = self.w_g = None      # live on inside the layer's fused operand
        # W_uk is stored [(head, dim), rank]; the absorb product contracts over dim, so keep it as [(head, rank), dim]:
        # contraction index contiguous, the layout the per-head kernel stages with whole 16-byte vectors
        H, d, R = self.heads, self.dim, self.rank
        self.w_uk = self.w_uk.view(H, d, R).transpose(1, 2).contiguous().view(H * R, d)
        return self.c_off + self.rank + (self.heads if self.gated else 0)

    def forward(self, y, batch, cache, dtype):
        """y: the layer's fused 32-bit projection [T, *]; returns the block's 32-bit output [T, width]."""
        H, R = self.heads, self.rank
        with trace("latent_prep"):
            q, gate = ops.latent_prep(y, self.q_off, self.c_off, self.g_off, H * self.dim, R, H, self.norm_w, self.eps,
                                      batch.slot_mapping, cache, dtype)
        with trace("latent_absorb"):
            q_abs = ops.heads_matmul(q, self.w_uk, H, self.dim, R, False, out_dtype=ops.latent_query_dtype(cache, H, R))
        with trace("latent_attention"):
            o_lat = ops.latent_attention(q_abs, cache, batch, H, R, self.scale, dtype)
        with trace("latent_unabsorb"):
            ctx = ops.heads_matmul(o_lat, self.w_uv, H, R, self.vdim, False, row_scale=gate, out_dtype=dtype)
        with trace("gemm_out"):
            return ops.linear(ctx, self.w_o, out_dtype=torch.float32)


class RotaryLatentAttention:
    """Multi-head attention over a low-rank latent with a query latent and a rotated key part shared by all heads.

        c_q = rmsnorm(W_dq h) * g_q ;  q_h = W_uq,h c_q = [q_h^n (dim) | q_h^r (rot)]
        [c' | k^r] = W_dkv h ;  c = rmsnorm(c') * g_c  (rank) ;  k^r, q_h^r rotated by position (interleaved pairs, table)
        score_h = scale * (q_h^n . W_uk,h c + q_h^r . k^r) ;  causal softmax ;  o_h = sum_j p_hj W_uv,h c_j
        out = W_o (concat_h(o_h) * sigmoid(W_g h))            the gate is per channel and reads the layer's input

    Cached per token: [c | k^r] (rank + rot numbers).  Executed in the absorbed form of ``LatentAttention``: with
    q~_h = [W_uk,h^T q_h^n | q_h^r] the score is scale * q~_h . [c | k^r], so the cache row is key AND value of one shared
    head -- the value product carries rot extra columns that the un-absorption never reads.  ``width`` is the cache
    row: rank + rot, or the next size the tcgen05 multi-query kernels take (64 / 128 / 256, zero padded) where that costs
    at most a quarter more (16-bit CUDA).  The rotation is given as a frequency table and a magnitude
    (ops.rotary_frequencies), so any frequency schedule fits."""

    def __init__(self, heads: int, dim: int, rot: int, vdim: int, rank: int, q_rank: int, scale: float, eps: float, freq, mag: float):
        self.heads, self.dim, self.rot, self.vdim, self.rank, self.q_rank = heads, dim, rot, vdim, rank, q_rank
        self.scale, self.eps, self.freq, self.mag = scale, eps, freq, mag
        self.width = rank + rot
        self.w_dq = self.qn_w = self.w_uq = self.w_dkv = self.cn_w = self.w_uk = self.w_uv = self.w_g = self.w_o = None
        self.q_off = self.c_off = self.g_off = 0

    def choose_width(self, device, dtype) -> int:
        need = self.rank + self.rot
        if torch.device(device).type == "cuda" and dtype != torch.float32:
            for w in (64, 128, 256):
                if need <= w and 4 * (w - need) <= w:
                    self.width = w
                    break
        return self.width

    def weights(self):
        return [self.w_dq, self.qn_w, self.w_uq, self.w_dkv, self.cn_w, self.w_uk, self.w_uv, self.w_g, self.w_o]

    def in_rows(self):
        return torch.cat([self.w_dq, self.w_dkv, self.w_g], dim=0)

    def bind(self, base: int):
        self.q_off = base
        self.c_off = base + self.q_rank
        self.g_off = self.c_off + self.rank + self.rot
        self.w_dq = self.w_dkv = self.w_g = None
        self.freq = self.freq.to(torch.float64).to(self.w_o.device).contiguous()     # the kernels read the table on the device
        H, d, R = self.heads, self.dim, self.rank
        # [(head, dim), rank] -> [(head, rank), dim]: the absorption contracts over dim (see LatentAttention.bind)
        self.w_uk = self.w_uk.view(H, d, R).transpose(1, 2).contiguous().view(H * R, d)
        return self.g_off + H * self.vdim

    def forward(self, y, batch, cache, dtype):
        """y: the layer's fused 32-bit projection [T, *]; cache: this layer's latent plane [blocks, block_size, width]."""
        H, d, r, R, Wd = self.heads, self.dim, self.rot, self.rank, self.width
        with trace("latent_prep"):
            cq, gate = ops.latent_rope_prep(y, self.q_off, self.q_rank, self.c_off, R, r, self.g_off, H * self.vdim, self.qn_w,
                                            self.cn_w, self.eps, self.freq, self.mag, batch.positions, batch.slot_mapping, cache, dtype)
        with trace("gemm_uq"):
            q = ops.linear(cq, self.w_uq, out_dtype=torch.float32)
        with trace("latent_query_rope"):
            q_nope, q_abs = ops.latent_query_rope(q, H, d, r, R, Wd, self.freq, self.mag, batch.positions, dtype,
                                                  ops.latent_query_dtype(cache, H, Wd))
        with trace("latent_absorb"):
            ops.heads_matmul(q_nope, self.w_uk, H, d, R, False, out=q_abs, out_head_stride=Wd)
        with trace("latent_attention"):
            o_lat = ops.latent_attention(q_abs, cache, batch, H, Wd, self.scale, dtype)
        with trace("latent_unabsorb"):
            ctx = ops.heads_matmul(o_lat, self.w_uv, H, R, self.vdim, False, elem_scale=gate, x_head_stride=Wd, out_dtype=dtype)
        with trace("gemm_out"):
            return ops.linear(ctx, self.w_o, out_dtype=torch.float32)


_GROUPED_ROWS = int(os.environ.get("LLMSS_MOE_GROUPED_MIN_ROWS", "64"))   # grouped form from this many rows per expert on average
_FORCE_GROUPED = os.environ.get("LLMSS_MOE_FORCE_GROUPED", "0") == "1"
_GEMM_TFLOPS, _CALL_US = 1200.0, 30.0     # sustained tensor-core rate of the expert GEMMs; host cost of issuing one GEMM
_DENSE_MIN = int(os.environ.get("LLMSS_MOE_DENSE_MIN_TOKENS", "0"))   # 0: dense as soon as token x top pairs >= experts


class RoutedExperts:
    """Mixture of small feed-forward experts with group-limited top-k routing (csrc/moe.cu).

    Router logits come from the layer's fused input projection (32-bit accumulation).  A batch with fewer (token,
    chosen expert) pairs than experts gathers the chosen experts' weight rows per token -- it reads only those bytes.
    From there on a batch touches about every expert anyway, and 16-bit CUDA batches run the dense form: every expert's
    up-projection in one tensor-core GEMM (activation fused) that streams each weight once, each expert's block
    scaled by its routing weight (0 if not chosen), one GEMM over the side-by-side down matrices.  The dense form
    spends experts / top times the needed FLOPs, which is nothing while the step is bound by the weight bytes (decode,
    short portions; it is also free of host synchronisation, so it can sit in a captured decode graph).  Prompts long
    enough to give every expert ``LLMSS_MOE_GROUPED_MIN_ROWS`` rows on average run the grouped form: pairs sorted by
    expert on the device, one pair of tensor-core GEMMs per expert over its contiguous rows, 32-bit weighted sum per
    token.  ``LLMSS_MOE_DENSE_MIN_TOKENS`` moves the gather / dense switch."""

    def __init__(self, experts: int, top: int, groups: int, keep: int, route_scale: float, ff: int, act: int = ACT_RELU2,
                 gated: bool = False, score: str = "softmax", group_top: int = 1, renorm: bool = True):
        if experts % groups or not 0 < keep <= groups or not 0 < top <= keep * (experts // groups):
            raise ValueError(f"routed experts: bad routing sizes experts={experts} groups={groups} keep={keep} top={top}")
        self.experts, self.top, self.groups, self.keep, self.route_scale, self.ff, self.act = experts, top, groups, keep, route_scale, ff, act
        # gated: the hidden activation is act(W_gate h) * (W_up h); w_up then holds [E, 2 F, W], rows interleaved (gate_f, up_f)
        self.gated = gated
        # router variants (ops.moe_route): softmax or sigmoid scores; a per-expert ``correction`` added for the choice only;
        # a group scores as the sum of its ``group_top`` best; weights renormalised over the chosen experts or not
        self.score, self.group_top, self.renorm, self.correction = score, group_top, renorm, None
        self.z_off = 0
        self.w_router = self.w_up = self.w_down = None     # [E, W] | [E, F or 2 F, W] | [W, E * F]

    def in_rows(self):
        return self.w_router

    def _grouped_pays(self, T: int, W: int) -> bool:
        """Dense runs experts / top times the FLOPs in two launches; grouped runs the needed FLOPs in 2 x experts launches that
        the host issues one by one.  Estimate both (tensor-core rate and per-call host cost measured on B200) and take the
        cheaper; LLMSS_MOE_GROUPED_MIN_ROWS=1 with LLMSS_MOE_FORCE_GROUPED=1 forces the grouped form."""
        if _FORCE_GROUPED:
            return True
        dense_us = 4.0 * T * self.experts * self.ff * W / (_GEMM_TFLOPS * 1e6)
        grouped_us = max(2 * self.experts * _CALL_US, dense_us * self.top / self.experts) + 150.0
        return grouped_us < dense_us

    def bind(self, base: int):
        self.z_off = base
        self.w_router = None
        return base + self.experts

    def _route_kw(self):
        return dict(score=self.score, correction=self.correction, group_top=self.group_top, renorm=self.renorm)

    def forward(self, h, y=None):
        """``y``: a fused projection that holds the router logits at ``z_off`` (32-bit); without it the router runs as
        a GEMM of its own (32-bit accumulation and output)."""
        E, F = self.experts, self.ff
        if y is None:
            with trace("experts_router"):
                y = ops.linear(h, self.w_router, out_dtype=torch.float32)
        z = y[:, self.z_off:self.z_off + E]
        T = h.shape[0]
        if (h.is_cuda and h.dtype != torch.float32 and T * self.top >= _GROUPED_ROWS * E and self._grouped_pays(T, h.shape[1])
                and not torch.cuda.is_current_stream_capturing()):
            from ..ops import cuda_impl as cu

            with trace("experts_route"):
                ids, wts = ops.moe_route(z, E, self.top, self.groups, self.keep, self.route_scale, **self._route_kw())
            with trace("experts_grouped"):
                return cu.moe_experts_grouped(h, ids, wts, self.w_up, self.w_down, self.act, self.gated)
        if h.is_cuda and h.dtype != torch.float32 and T >= (_DENSE_MIN or -(-E // self.top)):
            from ..ops import cuda_impl as cu

            with trace("experts_route"):
                _, _, dense = cu.moe_route(z, E, self.top, self.groups, self.keep, self.route_scale, dense=True, **self._route_kw())
            with trace("experts_dense_up"):
                a = ops.linear(h, self.w_up.view(self.w_up.shape[0] * self.w_up.shape[1], -1), act=self.act, gated=self.gated)
                cu.moe_scale(a, dense, E, F)
            with trace("experts_dense_down"):
                return ops.linear(a, self.w_down, out_dtype=torch.float32)
        with trace("experts_route"):
            ids, wts = ops.moe_route(z, E, self.top, self.groups, self.keep, self.route_scale, **self._route_kw())
        with trace("experts_gather"):
            return ops.moe_experts(h, ids, wts, self.w_up, self.w_down, self.act, self.gated)
