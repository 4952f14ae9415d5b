"""Token mixers and feed-forward blocks over a 32-bit residual stream that are not tied to one model family:

  * ``LinearRecurrence`` layers -- RWKV-style time mixing (``WkvMixer``), lightning attention (``LightningMixer``) and
    Mamba-2 / state-space duality (``SsdMixer``) -- all on the one gated linear-recurrence op (ops.linear_scan) with a
    32-bit state per sequence, head and layer;
  * ``BiasedAttention`` -- grouped-query softmax attention with separate key / value sizes, short causal convolutions on
    q / k / v, per-head query / key norm, a position-dependent query temperature, a learned distance bias and a per-head
    output gate, over the paged cache;
  * ``ParallelPair`` -- two mixers side by side whose normed outputs are averaged;
  * ``WindowAttention`` -- grouped-query softmax attention over a sliding window with a linear distance penalty per head,
    query / key norm over the whole projection, a value norm, a factor per query head and a per-head output gate; a
    layer may attend over the pages another layer writes;
  * ``SinkAttention`` -- grouped-query softmax attention whose values are the projected keys, with rotary positions from
    a frequency table, unit-RMS queries / keys and a learned sink logit per head in the softmax denominator;
  * ``Hgrn2Mixer`` -- a gated linear recurrence whose forget gate (bounded from below) also sets the write strength;
  * ``DeltaMixer`` -- the gated delta rule (ops.delta_scan) behind short convolutions, with a gated per-head norm;
  * ``HyperConnection`` -- the read / mix / write weights of one sub-layer over several residual streams;
  * ``DenseFFN``.

Every block says what it keeps per sequence (``state_shapes``), which cache pages it needs (``kv_shape``), and maps
(x: the 32-bit residual, h: x in the compute type) to a 32-bit [T, width] output.  All sizes and constants are
constructor arguments.  ``lc`` is the layer's view of the cache (engine.kv_cache.HybridCache): ``lc.state(name)``,
``lc.k``, ``lc.v``.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..ops import (ACT_GELU_ERF, ACT_NONE, ACT_SILU, DECAY_HEAD, DECAY_TOKEN_CHANNEL, DECAY_TOKEN_HEAD, GATE_NONE, GATE_SIGMOID,
                   GATE_SILU, UNARY_NEG_EXP, UNARY_TANH)
from ..utils.tracing import trace

F32 = torch.float32


class LayerCacheView:
    """What one layer sees of a HybridCache: its own states and pages, under ``prefix`` for nested blocks.  ``pages_key``:
    the layer whose key / value pages this one reads (a layer that shares another layer's keys and values)."""

    def __init__(self, cache, key, prefix: str = "", pages_key=None):
        self.cache, self.key, self.prefix = cache, key, prefix
        self.pages_key = key if pages_key is None else pages_key

    def state(self, name: str):
        return self.cache.state(self.key, self.prefix + name)

    def sub(self, prefix: str) -> "LayerCacheView":
        return LayerCacheView(self.cache, self.key, self.prefix + prefix)

    @property
    def latent(self):
        return self.cache.latent(self.pages_key)

    @property
    def k(self):
        return self.cache.k(self.pages_key)

    @property
    def v(self):
        return self.cache.v(self.pages_key)


class WkvMixer:
    """RWKV-style time mixing with a data-dependent per-channel decay.

        mix_s = x + (x_prev - x) * mu_s                   s in (r, k, v, g, w); x_prev = previous token's input
        r, k, v = W_r mix_r, W_k mix_k, W_v mix_v         heads x dim;  gate = silu(W_g mix_g)
        log w   = -exp(W_w2 tanh(W_w1 mix_w) + w0)        per head and key channel
        o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t ;  S_t = diag(w_t) S_(t-1) + k_t v_t^T
        out = W_o (rms_div_per_head(o) * norm * gate)
    State per sequence: the previous input row and S (32-bit)."""

    def __init__(self, width: int, heads: int, dim: int, eps: float):
        self.width, self.heads, self.dim, self.eps = width, heads, dim, eps
        self.mu = self.w_r = self.w_k = self.w_v = self.w_g = self.w_w1 = self.w_w2 = self.w0 = self.u = self.norm_w = self.w_o = None

    def state_shapes(self):
        return {"shift": ((self.width,), F32), "S": ((self.heads, self.dim, self.dim), F32)}

    def kv_shape(self):
        return None

    def weights(self):
        return [self.mu, self.w_r, self.w_k, self.w_v, self.w_g, self.w_w1, self.w_w2, self.w0, self.u, self.norm_w, self.w_o]

    def forward(self, x, h, batch, lc, dtype):
        H, D = self.heads, self.dim
        with trace("token_shift"):
            mix = ops.token_shift(x, self.mu, batch, lc.state("shift"), out_dtype=dtype)     # [5, T, W]: r k v g w
        with trace("gemm_in"):
            r = ops.linear(mix[0], self.w_r, out_dtype=F32)
            k = ops.linear(mix[1], self.w_k, out_dtype=F32)
            v = ops.linear(mix[2], self.w_v, out_dtype=F32)
            g = ops.linear(mix[3], self.w_g, out_dtype=F32)
            lo = ops.unary(ops.linear(mix[4], self.w_w1, out_dtype=F32), UNARY_TANH, out_dtype=dtype)
            logw = ops.unary(ops.linear(lo, self.w_w2, self.w0, out_dtype=F32), UNARY_NEG_EXP)
        with trace("linear_scan"):
            o = ops.linear_scan(r, k, v, logw, DECAY_TOKEN_CHANNEL, batch, lc.state("S"), H, H, D, D, bonus=self.u, read_before=True)
        with trace("gated_rmsnorm"):
            y = ops.gated_rmsnorm(o, g, GATE_SILU, self.norm_w, H, self.eps, False, out_dtype=dtype)
        with trace("gemm_out"):
            return ops.linear(y, self.w_o, out_dtype=F32)


class LightningMixer:
    """Lightning (linear) attention with a fixed decay per head.

        q, k, v = silu(W_q h), silu(W_k h), silu(W_v h) ;  S_t = decay_h S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t
        out = W_o (rms_div(concat_h o) * norm * sigmoid(W_g h))
    One input GEMM over the stacked rows [g | q | k | v] (activation from the q rows on)."""

    def __init__(self, width: int, heads: int, dim: int, vdim: int, decay, eps: float):
        self.width, self.heads, self.dim, self.vdim, self.eps = width, heads, dim, vdim, eps
        self.decay_values = [float(d) for d in decay]
        assert len(self.decay_values) == heads, "lightning attention: one decay per head"
        self.w_in = self.decay = self.norm_w = self.w_o = None

    def state_shapes(self):
        return {"S": ((self.heads, self.dim, self.vdim), F32)}

    def kv_shape(self):
        return None

    def weights(self):
        return [self.w_in, self.norm_w, self.w_o]

    def set_weights(self, w_q, w_k, w_v, w_g, norm_w, w_o):
        self.w_in = torch.cat([w_g, w_q, w_k, w_v], dim=0).contiguous()
        self.norm_w, self.w_o = norm_w, w_o.contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=F32, device=w_o.device)

    def forward(self, x, h, batch, lc, dtype):
        H, D, Dv = self.heads, self.dim, self.vdim
        n_g, n_qk = H * Dv, H * D
        with trace("gemm_in"):
            y = ops.linear(h, self.w_in, act=ACT_SILU, act_start=n_g, out_dtype=F32)
        q, k, v = y[:, n_g:n_g + n_qk], y[:, n_g + n_qk:n_g + 2 * n_qk], y[:, n_g + 2 * n_qk:]
        with trace("linear_scan"):
            o = ops.linear_scan(q, k, v, self.decay, DECAY_HEAD, batch, lc.state("S"), H, H, D, Dv)
        with trace("gated_rmsnorm"):
            z = ops.gated_rmsnorm(o, y[:, :n_g], GATE_SIGMOID, self.norm_w, 1, self.eps, False, out_dtype=dtype)
        with trace("gemm_out"):
            return ops.linear(z, self.w_o, out_dtype=F32)


class BiasedAttention:
    """Grouped-query softmax attention, no rotation; positions enter through a query temperature and a distance bias.

        q, k, v = W h + b  ->  short causal convolution per channel  ->  per-head RMS norm of q and k (shared weights)
        q *= 1 + coef * ln(floor((p + 1) / every) + 1)
        score_ij = scale * q_i . k_j + rel[bucket(i - j), head] ,  j <= i ;  softmax ;  o_h *= sigmoid(W_g h)_h ;  W_o
    Keys have ``dim`` channels, values ``vdim``.  Cached: normed keys and convolved values (pages), the last taps - 1
    projected q / k / v rows (state).  ``in_rows()`` / ``in_bias()`` let a layer stack the projection with others."""

    def __init__(self, width, heads, kv_heads, dim, vdim, taps, scale, temp_coef, temp_every, bias_max, eps):
        self.width, self.heads, self.kv_heads, self.dim, self.vdim, self.taps = width, heads, kv_heads, dim, vdim, taps
        self.scale, self.temp_coef, self.temp_every, self.bias_max, self.eps = scale, temp_coef, temp_every, bias_max, eps
        self.n_qkv = heads * dim + kv_heads * dim + kv_heads * vdim
        self.w_rows = self.b_rows = self.conv_w = self.q_norm = self.k_norm = self.dist_bias = self.dist_bias_scaled = self.w_o = None
        self.off = 0

    def state_shapes(self):
        return {"conv": ((self.taps - 1, self.n_qkv), F32)} if self.taps > 1 else {}

    def kv_shape(self):
        return (self.kv_heads, self.dim, self.vdim)

    def weights(self):
        return [self.w_rows, self.b_rows, self.conv_w, self.q_norm, self.k_norm, self.dist_bias, self.w_o]

    def set_weights(self, wq, bq, wk, bk, wv, bv, cq, ck, cv, q_norm, k_norm, rel, w_g, w_o):
        self.w_rows = torch.cat([wq, wk, wv, w_g], dim=0)
        self.b_rows = torch.cat([bq, bk, bv, torch.zeros(w_g.shape[0], dtype=bq.dtype, device=bq.device)])
        self.conv_w = torch.cat([cq, ck, cv], dim=0).contiguous()
        self.q_norm, self.k_norm, self.w_o = q_norm, k_norm, w_o.contiguous()
        self.dist_bias = ops.distance_bias_table(rel.float().cpu(), self.bias_max).to(w_o.device)   # [heads, bias_max + 1] 32-bit
        # the same table in raw-score units, for the tensor-core kernels that add it before their one multiply by the scale
        self.dist_bias_scaled = (self.dist_bias / self.scale).contiguous() if self.scale > 0 else None

    def in_rows(self):
        return self.w_rows

    def in_bias(self):
        return self.b_rows

    def bind(self, base: int) -> int:
        self.off = base
        n = self.w_rows.shape[0]
        self.w_rows = self.b_rows = None
        return base + n

    def forward_projected(self, y, batch, lc, dtype):
        """y: the layer's fused 32-bit projection (bias added); this block's columns start at ``off``."""
        H, G, D, Dv = self.heads, self.kv_heads, self.dim, self.vdim
        qkv = y[:, self.off:self.off + self.n_qkv]
        gate = y[:, self.off + self.n_qkv:self.off + self.n_qkv + H]
        with trace("causal_conv"):
            qkv = ops.causal_conv(qkv, self.conv_w, None, ACT_NONE, batch, lc.state("conv") if self.taps > 1 else None)
        with trace("qknorm_kv_write"):
            q = ops.qknorm_kv_write(qkv, H, G, D, Dv, self.q_norm, self.k_norm, self.eps, self.temp_coef, self.temp_every,
                                    batch.positions, batch.slot_mapping, lc.k, lc.v, out_dtype=dtype)
        with trace("attention_bias"):
            ctx = ops.attention_bias(q, lc.k, lc.v, batch, H, G, D, Dv, self.scale, self.dist_bias, gate=gate, out_dtype=dtype,
                                     bias_over_scale=self.dist_bias_scaled)
        with trace("gemm_out"):
            return ops.linear(ctx, self.w_o, out_dtype=F32)


class SsdMixer:
    """Mamba-2 (state-space duality) layer.

        [z | x | B | C | dt] = W_in h ;  (x, B, C) <- silu(causal_conv(x, B, C) + b)
        dt = softplus(dt + dt_bias) ;  S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T ;  y_t = S_t^T C_t + D_h x_t
        out = W_o (rms_div_in_groups(y * silu(z)) * norm)
    heads x vdim inner channels, state size N, B / C shared by the heads of a group.  State per sequence: S (32-bit)
    and the last taps - 1 conv inputs."""

    def __init__(self, width, heads, vdim, state, groups, norm_groups, taps, eps):
        self.width, self.heads, self.vdim, self.n, self.groups, self.norm_groups, self.taps, self.eps = (
            width, heads, vdim, state, groups, norm_groups, taps, eps)
        self.inner = heads * vdim
        self.n_conv = self.inner + 2 * groups * state
        self.w_rows = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d = self.norm_w = self.w_o = None
        self.off = 0

    def state_shapes(self):
        s = {"S": ((self.heads, self.n, self.vdim), F32)}
        if self.taps > 1:
            s["conv"] = ((self.taps - 1, self.n_conv), F32)
        return s

    def kv_shape(self):
        return None

    def weights(self):
        return [self.w_rows, self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.d, self.norm_w, self.w_o]

    def in_rows(self):
        return self.w_rows

    def in_bias(self):
        return torch.zeros(self.w_rows.shape[0], dtype=self.w_rows.dtype, device=self.w_rows.device)

    def bind(self, base: int) -> int:
        self.off = base
        n = self.w_rows.shape[0]
        self.w_rows = None
        return base + n

    def forward_projected(self, y, batch, lc, dtype):
        H, Dv, N, G, inner = self.heads, self.vdim, self.n, self.groups, self.inner
        o0 = self.off
        z = y[:, o0:o0 + inner]
        xbc = y[:, o0 + inner:o0 + inner + self.n_conv]
        dt_raw = y[:, o0 + inner + self.n_conv:o0 + inner + self.n_conv + H]
        with trace("causal_conv"):
            xbc = ops.causal_conv(xbc, self.conv_w, self.conv_b, ACT_SILU, batch, lc.state("conv") if self.taps > 1 else None)
        xs, Bm, Cm = xbc[:, :inner], xbc[:, inner:inner + G * N], xbc[:, inner + G * N:]
        with trace("ssm_dt"):
            dt, logdecay = ops.ssm_dt(dt_raw, self.dt_bias, self.a_log)
        with trace("linear_scan"):
            o = ops.linear_scan(Cm, Bm, xs, logdecay, DECAY_TOKEN_HEAD, batch, lc.state("S"), H, G, N, Dv, v_scale=dt)
        with trace("gated_rmsnorm"):
            g = ops.gated_rmsnorm(o, z, GATE_SILU, self.norm_w, self.norm_groups, self.eps, True, skip_x=xs, skip_d=self.d,
                                  out_dtype=dtype)
        with trace("gemm_out"):
            return ops.linear(g, self.w_o, out_dtype=F32)


class ParallelPair:
    """Two mixers side by side on the same input: out = (rms_div(left) * w_left + rms_div(right) * w_right) / 2.
    Their input projections are stacked into ONE GEMM; the averaging rides on the layer's post-norm kernel (the layer
    asks for ``pair_weights``)."""

    def __init__(self, left, right):
        self.left, self.right = left, right
        self.w_in = self.b_in = self.w_left = self.w_right = None

    def state_shapes(self):
        s = {f"left.{k}": v for k, v in self.left.state_shapes().items()}
        s.update({f"right.{k}": v for k, v in self.right.state_shapes().items()})
        return s

    def kv_shape(self):
        return self.left.kv_shape() or self.right.kv_shape()

    def weights(self):
        return [self.w_in, self.b_in, self.w_left, self.w_right] + self.left.weights() + self.right.weights()

    def finalize(self):
        self.w_in = torch.cat([self.left.in_rows(), self.right.in_rows()], dim=0).contiguous()
        self.b_in = torch.cat([self.left.in_bias(), self.right.in_bias()]).contiguous()
        self.right.bind(self.left.bind(0))

    def forward_pair(self, x, h, batch, lc, dtype):
        with trace("gemm_in"):
            y = ops.linear(h, self.w_in, self.b_in, out_dtype=F32)
        kv_left = self.left.kv_shape() is not None
        a = self.left.forward_projected(y, batch, _PairView(lc, "left.", kv_left), dtype)
        b = self.right.forward_projected(y, batch, _PairView(lc, "right.", not kv_left), dtype)
        return a, b


class _PairView(LayerCacheView):
    def __init__(self, lc, prefix, owns_pages):
        super().__init__(lc.cache, lc.key, lc.prefix + prefix)
        self.owns_pages = owns_pages


class WindowAttention:
    """Grouped-query softmax attention without rotation over a sliding window.

        q, k, v = W h  ->  short causal convolution per channel
        q, k    <- rms_div over the token's WHOLE projection (all heads at once) * weight ;  v_g <- rms_div(v_g) per head
        score_ij = scale * temp_h * q_i . k_j - slope_h (i - j),  0 <= i - j < window ;  slope_h = 2^(-slope_exp (h + 1) / H)
        softmax ;  o_h *= sigmoid(W_g h)_h ;  W_o
    Cached: normed keys and normed values (pages), the last taps - 1 projected rows (state).  ``kv_from`` = key of
    another layer: this layer has no key / value tensors and attends over that layer's pages with queries of its own (the
    value norm has no weight, so the lender's normed values are this layer's).  ``window`` None: every earlier token."""

    def __init__(self, width, heads, kv_heads, dim, vdim, taps, scale, window, eps, slope_exp=8.0, kv_from=None):
        self.width, self.heads, self.kv_heads, self.dim, self.vdim, self.taps = width, heads, kv_heads, dim, vdim, taps
        self.scale, self.window, self.eps, self.slope_exp, self.kv_from = scale, window, eps, slope_exp, kv_from
        assert heads % kv_heads == 0, "window attention: query heads must be a multiple of key/value heads"
        self.own_kv = kv_from is None
        self.n_conv = heads * dim + ((kv_heads * dim + kv_heads * vdim) if self.own_kv else 0)
        self.w_in = self.conv_w = self.q_norm = self.k_norm = self.temp = self.slopes = self.window_table = self.w_o = None

    def state_shapes(self):
        return {"conv": ((self.taps - 1, self.n_conv), F32)} if self.taps > 1 else {}

    def kv_shape(self):
        return (self.kv_heads, self.dim, self.vdim) if self.own_kv else None

    def weights(self):
        return [self.w_in, self.conv_w, self.q_norm, self.k_norm, self.temp, self.w_o]

    def set_weights(self, wq, wk, wv, cq, ck, cv, q_norm, k_norm, temp, w_g, w_o):
        """wk / wv / ck / cv / k_norm are None for a layer that borrows its keys and values."""
        own = self.own_kv
        self.w_in = torch.cat([wq, wk, wv, w_g] if own else [wq, w_g], dim=0).contiguous()
        self.conv_w = torch.cat([cq, ck, cv] if own else [cq], dim=0).contiguous()
        self.q_norm, self.k_norm, self.temp, self.w_o = q_norm, k_norm, temp, w_o.contiguous()
        H = self.heads
        self.slopes = torch.tensor([2.0 ** (-self.slope_exp * (h + 1) / H) for h in range(H)], dtype=F32, device=w_o.device)
        # the window and the slopes as a distance table in raw-score units, for the tensor-core kernels (16-bit pages, equal key
        # and value size 64 / 128 / 256); the generic kernel takes window and slopes themselves
        self.window_table = (ops.window_bias_table(self.slopes, self.window, self.scale)
                             if self.window and self.scale > 0 and w_o.is_cuda and w_o.dtype != F32 and self.dim == self.vdim
                             and self.dim in (64, 128, 256) else None)

    def forward(self, h, batch, lc, dtype):
        """``lc``: this layer's cache view; its pages (``lc.k`` / ``lc.v``) are the lender's when keys and values are borrowed."""
        H, G, D, Dv = self.heads, self.kv_heads, self.dim, self.vdim
        with trace("gemm_in"):
            y = ops.linear(h, self.w_in, out_dtype=F32)
        qkv, gate = y[:, :self.n_conv], y[:, self.n_conv:self.n_conv + H]
        with trace("causal_conv"):
            qkv = ops.causal_conv(qkv, self.conv_w, None, ACT_NONE, batch, lc.state("conv") if self.taps > 1 else None)
        own = self.own_kv
        with trace("qknorm_kv_write"):
            q = ops.qknorm_kv_write(qkv, H, G if own else 0, D, Dv, self.q_norm, self.k_norm, self.eps, 0.0, 1, batch.positions,
                                    batch.slot_mapping, lc.k if own else None, lc.v if own else None, out_dtype=dtype,
                                    norm_whole=True, v_norm=True, q_head_scale=self.temp)
        with trace("attention_bias"):
            ctx = ops.attention_bias(q, lc.k, lc.v, batch, H, G, D, Dv, self.scale, None, gate=gate, out_dtype=dtype,
                                     window=self.window or 0, slopes=self.slopes, bias_over_scale=self.window_table)
        with trace("gemm_out"):
            return ops.linear(ctx, self.w_o, out_dtype=F32)


class SinkAttention:
    """Grouped-query softmax attention in which the raw key projection doubles as the value (no W_v), with an
    attention sink.

        q, k = W h ;  v = k                                          (v: before rotation and norm)
        q, k <- rotate(q, k) on the first 2 len(freq) channels of every head, pairs (i, i + n) (or interleaved)
        q, k <- rms_div per head (no weight), if ``unit_norm``
        p_ij = exp(scale q_i . k_j) / (sum_(j' <= i) exp(scale q_i . k_j') + exp(sink_h)) ;  o_i = sum_j p_ij v_j ;  W_o

    The rotation is a frequency table and a magnitude (ops.rotary_frequencies): linear interpolation, YaRN or none are
    tables.  Cached: prepared keys (K pages) and projected keys (V pages).  One input GEMM over the stacked rows [q | k]."""

    def __init__(self, width, heads, kv_heads, dim, scale, eps, freq, mag=1.0, interleaved=False, unit_norm=True):
        self.width, self.heads, self.kv_heads, self.dim, self.scale, self.eps = width, heads, kv_heads, dim, scale, eps
        self.freq, self.mag, self.interleaved, self.unit_norm = freq, mag, interleaved, unit_norm
        assert heads % kv_heads == 0, "sink attention: query heads must be a multiple of key/value heads"
        assert 2 * freq.numel() <= dim, "sink attention: more rotated channels than the head has"
        self.w_in = self.sinks = self.w_o = None

    def state_shapes(self):
        return {}

    def kv_shape(self):
        return (self.kv_heads, self.dim, self.dim)

    def latent_width(self):
        return None

    def weights(self):
        return [self.w_in, self.sinks, self.w_o]

    def set_weights(self, wq, wk, sinks, w_o):
        self.w_in = torch.cat([wq, wk], dim=0).contiguous()
        self.sinks, self.w_o = sinks, w_o.contiguous()
        self.freq = self.freq.to(torch.float64).to(w_o.device).contiguous()     # the kernels read the table on the device

    def forward(self, h, batch, lc, dtype):
        H, G, D = self.heads, self.kv_heads, self.dim
        with trace("gemm_in"):
            y = ops.linear(h, self.w_in, out_dtype=F32)
        with trace("rope_norm_kv_write"):
            q = ops.rope_norm_kv_write(y, H, G, D, self.freq, self.mag, self.interleaved, self.unit_norm, self.eps, batch.positions,
                                       batch.slot_mapping, lc.k, lc.v, out_dtype=dtype)
        with trace("attention_sink"):
            ctx = ops.attention_bias(q, lc.k, lc.v, batch, H, G, D, D, self.scale, None, out_dtype=dtype, sinks=self.sinks)
        with trace("gemm_out"):
            return ops.linear(ctx, self.w_o, out_dtype=F32)


class Hgrn2Mixer:
    """Gated linear recurrence in which the forget gate also decides what is written (HGRN2).

        q = silu(W_q h) ;  v = W_v h ;  f = lower + (1 - lower) sigmoid(W_f h + b_f)          per head and key channel
        S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T ;  o_t = S_t^T q_t
        out = W_o concat_h(rms_div(o_h) * norm)                                              norm [vdim] shared by the heads

    It is ops.linear_scan with key = 1 - f and a per-channel decay f (given as ln f).  State per sequence: S (32-bit).
    One input GEMM over the stacked rows [q | f | v]."""

    def __init__(self, width, heads, dim, vdim, eps):
        self.width, self.heads, self.dim, self.vdim, self.eps = width, heads, dim, vdim, eps
        self.n_qk = heads * dim
        self.w_in = self.b_in = self.lower = self.norm_w = self.w_o = None

    def state_shapes(self):
        return {"S": ((self.heads, self.dim, self.vdim), F32)}

    def kv_shape(self):
        return None

    def latent_width(self):
        return None

    def weights(self):
        return [self.w_in, self.b_in, self.lower, self.norm_w, self.w_o]

    def set_weights(self, wq, wf, bf, wv, lower, norm_w, w_o):
        self.w_in = torch.cat([wq, wf, wv], dim=0).contiguous()
        zq, zv = torch.zeros(wq.shape[0], dtype=bf.dtype, device=bf.device), torch.zeros(wv.shape[0], dtype=bf.dtype, device=bf.device)
        self.b_in = torch.cat([zq, bf, zv]).contiguous()
        self.lower, self.w_o = lower, w_o.contiguous()
        self.norm_w = norm_w.repeat(self.heads).contiguous()

    def forward(self, h, batch, lc, dtype):
        H, D, Dv, n = self.heads, self.dim, self.vdim, self.n_qk
        with trace("gemm_in"):
            y = ops.linear(h, self.w_in, self.b_in, out_dtype=F32)
        with trace("hgrn_gates"):
            q, k, logf = ops.hgrn_gates(y, n, self.lower)
        with trace("linear_scan"):
            o = ops.linear_scan(q, k, y[:, 2 * n:], logf, DECAY_TOKEN_CHANNEL, batch, lc.state("S"), H, H, D, Dv)
        with trace("gated_rmsnorm"):
            z = ops.gated_rmsnorm(o, None, GATE_NONE, self.norm_w, H, self.eps, False, out_dtype=dtype)
        with trace("gemm_out"):
            return ops.linear(z, self.w_o, out_dtype=F32)


class DeltaMixer:
    """Gated delta rule with one decay and one write strength per head and token.

        q, k, v = silu(causal_conv(W h)) ;  q, k <- unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q *= dim^(-1/2)
        beta = sigmoid(W_b h) ;  decay = exp(-exp(A_log_h) softplus(W_a h + dt_bias))
        S <- decay S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q
        out = W_o (rms_div_per_head(o) * norm * silu(W_g h))
    q / k have ``kv_heads`` heads shared by groups of the ``heads`` value heads.  State per sequence: S (32-bit) and the
    last taps - 1 projected rows.  One input GEMM over the stacked rows [q | k | v | g | a | b]."""

    UNIT_EPS = 1e-6

    def __init__(self, width, heads, kv_heads, dim, vdim, taps, eps):
        self.width, self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.eps = width, heads, kv_heads, dim, vdim, taps, eps
        assert heads % kv_heads == 0, "delta rule: value heads must be a multiple of query/key heads"
        self.n_qk, self.n_v = kv_heads * dim, heads * vdim
        self.n_conv = 2 * self.n_qk + self.n_v
        self.w_in = self.conv_w = self.dt_bias = self.a_log = self.norm_w = self.w_o = None

    def state_shapes(self):
        s = {"S": ((self.heads, self.dim, self.vdim), F32)}
        if self.taps > 1:
            s["conv"] = ((self.taps - 1, self.n_conv), F32)
        return s

    def kv_shape(self):
        return None

    def weights(self):
        return [self.w_in, self.conv_w, self.dt_bias, self.a_log, self.norm_w, self.w_o]

    def set_weights(self, wq, wk, wv, cq, ck, cv, w_b, w_a, dt_bias, a_log, norm_w, w_g, w_o):
        self.w_in = torch.cat([wq, wk, wv, w_g, w_a, w_b], dim=0).contiguous()
        self.conv_w = torch.cat([cq, ck, cv], dim=0).contiguous()
        self.dt_bias, self.a_log, self.w_o = dt_bias, a_log, w_o.contiguous()
        self.norm_w = norm_w.repeat(self.heads).contiguous()        # one weight of size vdim shared by the heads

    def forward(self, h, batch, lc, dtype):
        H, G, D, Dv = self.heads, self.kv_heads, self.dim, self.vdim
        nc, nv = self.n_conv, self.n_v
        with trace("gemm_in"):
            y = ops.linear(h, self.w_in, out_dtype=F32)
        gate, a_raw, b_raw = y[:, nc:nc + nv], y[:, nc + nv:nc + nv + H], y[:, nc + nv + H:nc + nv + 2 * H]
        with trace("causal_conv"):
            qkv = ops.causal_conv(y[:, :nc], self.conv_w, None, ACT_SILU, batch, lc.state("conv") if self.taps > 1 else None)
        with trace("ssm_dt"):
            _, log_decay = ops.ssm_dt(a_raw, self.dt_bias, self.a_log)
        with trace("delta_scan"):
            o = ops.delta_scan(qkv[:, :self.n_qk], qkv[:, self.n_qk:2 * self.n_qk], qkv[:, 2 * self.n_qk:], log_decay, b_raw, batch,
                               lc.state("S"), H, G, D, Dv, unit_eps=self.UNIT_EPS, q_scale=D ** -0.5, beta_sigmoid=True)
        with trace("gated_rmsnorm"):
            z = ops.gated_rmsnorm(o, gate, GATE_SILU, self.norm_w, H, self.eps, False, out_dtype=dtype)
        with trace("gemm_out"):
            return ops.linear(z, self.w_o, out_dtype=F32)


class HyperConnection:
    """Weights of one sub-layer over S residual streams: it reads u = sum_s w_in[s] x_s and writes
    x_t <- sum_s mix[s, t] x_s + w_out[t] y (ops.hyper_residual).  ``identity(S = 1)`` is the plain residual sum."""

    def __init__(self, w_in, mix, w_out):
        self.w_in, self.mix, self.w_out = w_in, mix, w_out

    @classmethod
    def identity(cls, device):
        one = torch.ones(1, dtype=F32, device=device)
        return cls(one, one.view(1, 1).clone(), one.clone())

    def weights(self):
        return [self.w_in, self.mix, self.w_out]


class DenseFFN:
    """W_down act(W_up h), activation in the up GEMM's epilogue."""

    def __init__(self, act: int = ACT_GELU_ERF):
        self.act = act
        self.w_up = self.w_down = None

    def weights(self):
        return [self.w_up, self.w_down]

    def forward(self, h):
        with trace("ffn_up"):
            a = ops.linear(h, self.w_up, act=self.act)
        with trace("ffn_down"):
            return ops.linear(a, self.w_down, out_dtype=F32)
