"""Plain-PyTorch fp32 oracles for every op in ``llmss_b200.ops``.

These are (a) the CPU execution path (BASELINE config 1: generate.py on CPU, TP=1; gloo
multi-process tests) and (b) the numerical reference every CUDA kernel in ``csrc/`` is
tested against (tests/test_gpu_*.py).  They mirror the math of the reference's ATen call
sites listed in SURVEY.md section 2.6 (G1-G16), not its code.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF, ACT_RELU, ACT_SILU, ACT_RELU2 = 0, 1, 2, 3, 4, 5
ACT_IDS = {
    None: ACT_NONE, "none": ACT_NONE,
    "gelu_new": ACT_GELU_TANH, "gelu_pytorch_tanh": ACT_GELU_TANH, "gelu_fast": ACT_GELU_TANH,
    "gelu": ACT_GELU_ERF, "relu": ACT_RELU, "silu": ACT_SILU, "swish": ACT_SILU, "relu2": ACT_RELU2,
}
NORM_LAYER, NORM_RMS, NORM_DYT = 0, 1, 2
ROPE_NONE, ROPE_GPTJ, ROPE_NEOX = 0, 1, 2


def apply_act(x: torch.Tensor, act: int) -> torch.Tensor:
    if act == ACT_NONE:
        return x
    if act == ACT_GELU_TANH:  # gelu_new == gelu_pytorch_tanh (gptj_modeling.py:266, gpt_bigcode_modeling.py:321)
        return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x * x * x)))
    if act == ACT_GELU_ERF:
        return F.gelu(x)
    if act == ACT_RELU:
        return F.relu(x)
    if act == ACT_SILU:
        return F.silu(x)
    if act == ACT_RELU2:
        return F.relu(x).square()
    raise ValueError(act)


def norm_residual(x, residual, weight, bias, eps: float, kind: int, out_dtype=None):
    """(x [+ residual]) -> (norm(sum), sum).  G2 + G13 fused (and the G18 capability)."""
    s = x.float() if residual is None else x.float() + residual.float()
    if kind == NORM_LAYER:
        y = F.layer_norm(s, (s.shape[-1],), weight.float(), None if bias is None else bias.float(), eps)
    else:
        var = s.pow(2).mean(-1, keepdim=True)
        y = s * torch.rsqrt(var + eps) * weight.float()
    od = out_dtype or x.dtype
    return y.to(od), s.to(od)


def linear(x, w, bias=None, act: int = ACT_NONE, gated: bool = False, act_start: int = 0,
           residual=None, out_dtype=None):
    """y = act(x @ w.T + bias) (+ residual).  ``w`` is [N, K] (HF nn.Linear layout).

    ``gated``: rows of w are interleaved (gate_0, up_0, gate_1, up_1, ...) and the result is
    act(gate) * up with N/2 columns (Llama SwiGLU fused into the epilogue).
    ``act_start``: activation applies to output features >= act_start only (GPT-J fused
    QKV + fc_in GEMM).
    """
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if gated:
        y = apply_act(y[..., 0::2], act) * y[..., 1::2]
    elif act != ACT_NONE:
        if act_start > 0:
            y = torch.cat([y[..., :act_start], apply_act(y[..., act_start:], act)], dim=-1)
        else:
            y = apply_act(y, act)
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def rope_cos_sin(positions: torch.Tensor, rotary_dim: int, base: float):
    inv_freq = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=positions.device) / rotary_dim))
    ang = positions.float()[:, None] * inv_freq[None, :]
    return torch.cos(ang), torch.sin(ang)  # [T, rotary_dim/2]


def apply_rope(x: torch.Tensor, cos, sin, rotary_dim: int, style: int) -> torch.Tensor:
    """x: [T, heads, d] fp32.  GPT-J = interleaved pairs (gptj_modeling.py:37-47); NeoX/Llama = half split."""
    if style == ROPE_NONE or rotary_dim == 0:
        return x
    rot, rest = x[..., :rotary_dim], x[..., rotary_dim:]
    c, s = cos[:, None, :], sin[:, None, :]
    if style == ROPE_GPTJ:
        x1, x2 = rot[..., 0::2], rot[..., 1::2]
        o1, o2 = x1 * c - x2 * s, x2 * c + x1 * s
        rot = torch.stack((o1, o2), dim=-1).flatten(-2)
    else:
        h = rotary_dim // 2
        x1, x2 = rot[..., :h], rot[..., h:]
        rot = torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)
    return torch.cat((rot, rest), dim=-1)


def rope_kv_write(qkv, positions, slot_mapping, k_cache, v_cache, hq: int, hkv: int, d: int,
                  rotary_dim: int, style: int, base: float, q_off: int, k_off: int, v_off: int):
    """RoPE on q,k in place inside ``qkv`` rows; write k,v to the paged cache (G5 + G6).

    qkv: [T, W] (row may be wider than the qkv columns); caches: [num_blocks, hkv, bs, d].
    slot = block * bs + offset; slot < 0 skips the write (padding rows of a captured graph).
    """
    T = qkv.shape[0]
    q = qkv[:, q_off:q_off + hq * d].reshape(T, hq, d).float()
    k = qkv[:, k_off:k_off + hkv * d].reshape(T, hkv, d).float()
    v = qkv[:, v_off:v_off + hkv * d].reshape(T, hkv, d)
    if style != ROPE_NONE and rotary_dim > 0:
        cos, sin = rope_cos_sin(positions, rotary_dim, base)
        q = apply_rope(q, cos, sin, rotary_dim, style)
        k = apply_rope(k, cos, sin, rotary_dim, style)
        qkv[:, q_off:q_off + hq * d] = q.reshape(T, hq * d).to(qkv.dtype)
        qkv[:, k_off:k_off + hkv * d] = k.reshape(T, hkv * d).to(qkv.dtype)
    bs = k_cache.shape[2]
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    blk, off = slots // bs, slots % bs
    k_cache[blk, :, off, :] = k[valid].to(k_cache.dtype)
    v_cache[blk, :, off, :] = v[valid].to(v_cache.dtype)


def attention_paged(q, k_cache, v_cache, block_tables, seq_lens, cu_q, scale: float):
    """Causal attention of packed queries against the paged cache (G7/G8 without S^2 masks).

    q: [T, hq, d]; sequence i owns query rows cu_q[i]:cu_q[i+1], which are the *last*
    q_len_i positions of its seq_lens[i] cached tokens.  Returns [T, hq, d] in q.dtype.
    """
    T, hq, d = q.shape
    hkv, bs = k_cache.shape[1], k_cache.shape[2]
    g = hq // hkv
    out = torch.zeros(T, hq, d, dtype=torch.float32, device=q.device)
    cu = cu_q.tolist()
    lens = seq_lens.tolist()
    for i in range(len(lens)):
        q0, q1 = cu[i], cu[i + 1]
        L, ql = lens[i], q1 - q0
        if ql == 0 or L == 0:
            continue
        nb = (L + bs - 1) // bs
        blocks = block_tables[i, :nb].long()
        k = k_cache[blocks].permute(1, 0, 2, 3).reshape(hkv, nb * bs, d)[:, :L].float()
        v = v_cache[blocks].permute(1, 0, 2, 3).reshape(hkv, nb * bs, d)[:, :L].float()
        qi = q[q0:q1].float().permute(1, 0, 2)  # [hq, ql, d]
        k = k.repeat_interleave(g, dim=0)
        v = v.repeat_interleave(g, dim=0)
        s = torch.matmul(qi, k.transpose(1, 2)) * scale  # [hq, ql, L]
        qpos = torch.arange(L - ql, L, device=q.device)[:, None]
        kpos = torch.arange(L, device=q.device)[None, :]
        s = s.masked_fill(kpos > qpos, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[q0:q1] = torch.matmul(p, v).permute(1, 0, 2)
    return out.to(q.dtype)


def embed(tokens, wte, positions=None, wpe=None, pos_offset: int = 0, out_dtype=None, scale: float = 1.0):
    """Token (+ learned position) embedding (G1; replicated tables, no collective).  With a 32-bit ``out_dtype``
    the two rows are summed in 32-bit (models that keep their residual stream in 32-bit).  ``scale`` multiplies the
    token row (32-bit output only)."""
    od = out_dtype or wte.dtype
    up = torch.float32 if od == torch.float32 else wte.dtype
    h = F.embedding(tokens.long(), wte).to(up)
    if scale != 1.0:
        h = h * scale
    if wpe is not None:
        h = h + F.embedding(positions.long() + pos_offset, wpe).to(up)
    return h.to(od)


# ----------------------------------------------------------------------------- 32-bit residual + Dynamic Tanh
def dyt_residual(resid, alpha: float, weight, bias, a=None, scale_a=None, b=None, scale_b=None, out_dtype=None,
                 want_norm: bool = True):
    """r' = r + scale_a * a + scale_b * b (all 32-bit);  returns (tanh(alpha r') * weight + bias in out_dtype, r')."""
    r = resid.float()
    for br, sc in ((a, scale_a), (b, scale_b)):
        if br is not None:
            r = r + (br.float() if sc is None else sc.float() * br.float())
    if not want_norm:
        return None, r
    y = torch.tanh(alpha * r) * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype or weight.dtype), r


def cast_concat(a, b, dtype):
    return torch.cat([a, b], dim=-1).to(dtype)


# ----------------------------------------------------------------------------- latent attention
def latent_prep(y, q_off: int, c_off: int, g_off: int, n_q: int, rank: int, heads: int, norm_w, eps: float,
                slot_mapping, cache, dtype):
    """y: [T, *] 32-bit fused projection.  RMS-norms the latent columns and writes them to the paged cache
    ([num_blocks, block_size, rank]); returns (q in `dtype`, sigmoid(gate columns) [T, heads] or None)."""
    c = y[:, c_off:c_off + rank].float()
    c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
    valid = slot_mapping >= 0
    flat = cache.view(-1, rank)
    flat[slot_mapping[valid].long()] = c[valid].to(cache.dtype)
    q = y[:, q_off:q_off + n_q].to(dtype)
    gate = torch.sigmoid(y[:, g_off:g_off + heads].float()) if g_off >= 0 else None
    return q, gate


def heads_matmul(x, w, heads: int, k: int, n: int, w_is_kn: bool, row_scale=None, out_dtype=None, x_head_stride=None,
                 elem_scale=None, out=None, out_head_stride=None):
    """Per-head product.  x: [T, heads * k]; w: [heads * k, n] (``w_is_kn``: rows index (head, k)) or [heads * n, k]
    (rows index (head, n)).  Returns [T, heads * n], optionally scaled per (token, head) by row_scale [T, heads] or per
    element by elem_scale [T, heads * n].  ``x_head_stride`` > k: head h reads x[:, h * stride : h * stride + k];
    ``out`` / ``out_head_stride``: head h writes out[:, h * stride : h * stride + n] of a given tensor."""
    T = x.shape[0]
    xs = x_head_stride or k
    xh = x.float().reshape(T, heads, xs)[:, :, :k]
    wh = w.float().view(heads, k, n) if w_is_kn else w.float().view(heads, n, k).transpose(1, 2)
    o = torch.einsum("thk,hkn->thn", xh, wh)
    if row_scale is not None:
        o = o * row_scale.float()[:, :, None]
    if elem_scale is not None:
        o = o * elem_scale.float().reshape(T, heads, n)
    if out is not None:
        out.view(T, heads, out_head_stride or n)[:, :, :n] = o.to(out.dtype)
        return out
    return o.reshape(T, heads * n).to(out_dtype or x.dtype)


def latent_attention(q_abs, cache, block_tables, seq_lens, cu_q, heads: int, rank: int, scale: float, out_dtype=None):
    """Absorbed latent attention: the cached latent is key and value of every head (see csrc/latent_attn.cu).
    q_abs: [T, heads * rank]; cache: [num_blocks, block_size, rank].  Returns [T, heads * rank]."""
    T = q_abs.shape[0]
    bs = cache.shape[1]
    out = torch.zeros(T, heads, rank, dtype=torch.float32, device=q_abs.device)
    cu, lens = cu_q.tolist(), seq_lens.tolist()
    for i, L in enumerate(lens):
        q0, q1 = cu[i], cu[i + 1]
        ql = q1 - q0
        if ql == 0 or L == 0:
            continue
        nb = (L + bs - 1) // bs
        c = cache[block_tables[i, :nb].long()].reshape(nb * bs, rank)[:L].float()
        qi = q_abs[q0:q1].float().view(ql, heads, rank)
        s = torch.einsum("thr,jr->htj", qi, c) * scale
        qpos = torch.arange(L - ql, L, device=c.device)[:, None]
        kpos = torch.arange(L, device=c.device)[None, :]
        s = s.masked_fill(kpos > qpos, float("-inf"))
        out[q0:q1] = torch.einsum("htj,jr->thr", torch.softmax(s, dim=-1), c)
    return out.reshape(T, heads * rank).to(out_dtype or q_abs.dtype)


# ----------------------------------------------------------------------------- routed experts
def moe_route(z, experts: int, top: int, groups: int, keep: int, route_scale: float, score: str = "softmax", correction=None,
              group_top: int = 1, renorm: bool = True):
    """Group-limited top-k routing on 32-bit logits z [T, experts] -> (ids [T, top] int32, weights [T, top] fp32).
    Scores s = softmax(z) or sigmoid(z) (``score``); experts are *chosen* by s + correction (``correction`` [experts], or
    none) while the weights are the chosen experts' s.  A group of neighbouring experts scores as the sum of its
    ``group_top`` largest choice scores (1: its best expert); only experts of the best ``keep`` groups are eligible (the
    rest is masked with -inf, not 0, because a choice score may be below 0).  ``renorm``: weights / (their sum + 1e-20); both forms
    times ``route_scale``.  Ties go to the lower index (stable sort), like the CUDA kernel."""
    zf = z.float()
    s = torch.softmax(zf, dim=-1) if score == "softmax" else torch.sigmoid(zf)
    c = s if correction is None else s + correction.float()
    T = s.shape[0]
    per = experts // groups
    gs = torch.sort(c.view(T, groups, per), dim=-1, descending=True, stable=True).values[:, :, :min(group_top, per)].sum(-1)
    best = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :keep]
    allow = torch.zeros(T, groups, dtype=torch.bool, device=z.device).scatter_(1, best, True)
    allow = allow[:, :, None].expand(T, groups, per).reshape(T, experts)
    idx = torch.sort(c.masked_fill(~allow, float("-inf")), dim=-1, descending=True, stable=True).indices[:, :top]
    w = s.gather(1, idx)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx.to(torch.int32), w * route_scale


def moe_experts(h, ids, wts, w_up, w_down, act: int, gated: bool = False):
    """out[t] = sum_k wts[t, k] * W_down[ids[t, k]] act(W_up[ids[t, k]] h[t]);  w_up [E, F, W]; w_down [W, E * F] (the
    experts' down matrices side by side); fp32 result.  ``gated``: w_up is [E, 2 F, W] with rows interleaved (gate_0, up_0,
    gate_1, ...) and the hidden activation is act(gate) * up."""
    T, W = h.shape
    E, F, _ = w_up.shape
    up = w_up.float()[ids.long()]                       # [T, top, F, W]
    a = torch.einsum("tkfw,tw->tkf", up, h.float())
    if gated:
        F //= 2
        a = (apply_act(a[..., 0::2], act) * a[..., 1::2]).to(h.dtype).float()
    else:
        a = apply_act(a, act).to(h.dtype).float()
    down = w_down.float().view(W, E, F).permute(1, 0, 2)[ids.long()]   # [T, top, W, F]
    return torch.einsum("tkwf,tkf,tk->tw", down, a, wts.float())


def _fmix32(x):
    x = x ^ (x >> 16)
    x = (x * 0x85EBCA6B) & 0xFFFFFFFF
    x = x ^ (x >> 13)
    x = (x * 0xC2B2AE35) & 0xFFFFFFFF
    return x ^ (x >> 16)


def rng_uniform(seed: torch.Tensor, step: torch.Tensor) -> torch.Tensor:
    """Counter-based uniforms in [0,1), one per row, keyed on the request's (seed, step) only (not on the
    batch row: a request samples the same tokens in any slot); bit-identical to csrc/sample.cu."""
    s, t = seed.long() & 0xFFFFFFFF, step.long() & 0xFFFFFFFF
    x = (0x9E3779B1 + t * 0x85EBCA77 + s * 0xC2B2AE3D) & 0xFFFFFFFF
    x = _fmix32(_fmix32(x))
    return (x >> 8).float() * (1.0 / 16777216.0)


MAX_CANDIDATES = 1024


def sample(logits, greedy, temperature, top_k, top_p, rng_state, vocab: Optional[int] = None,
           u_shift: float = 0.0) -> torch.Tensor:
    """Next-token choice per row (G15/G16 with the *intended* semantics).

    Order = the reference's warper list order (generate.py:114-120): top-p on the raw
    distribution, then top-k, then temperature; then one inverse-CDF draw over the
    survivors in (probability desc, index asc) order.  top_k == 0 means "off": with
    top_p < 1 the nucleus is searched among the 1024 most probable tokens; with
    top_p >= 1 it is a plain multinomial in index order.  ``rng_state`` is int32/int64
    [B, 2] = (seed, step) per row and its step column is advanced.  All ranks hold
    identical logits and rng state, so they agree without a broadcast (vs. N6).
    """
    B, V = logits.shape
    x = logits.float().clone()
    if vocab is not None and vocab < V:
        x[:, vocab:] = float("-inf")
        V = vocab
        x = x[:, :V]
    greedy = greedy.bool()
    arg = x.argmax(-1)
    # u_shift nudges the uniform draw (tests use it to find the rows whose choice sits on a CDF boundary)
    u = (rng_uniform(rng_state[:, 0], rng_state[:, 1]).double()[:, None] + u_shift).clamp(0.0, 1.0 - 2.0 ** -24)
    rng_state[:, 1] += 1
    xmax = x.max(-1, keepdim=True).values
    temp = temperature.float()[:, None]

    # candidate path
    sl, si = torch.sort(x, dim=-1, descending=True, stable=True)
    sp = torch.exp(sl - xmax) / torch.exp(x - xmax).sum(-1, keepdim=True)
    prev = torch.cumsum(sp, dim=-1) - sp
    k_eff = torch.where((top_k > 0) & (top_k <= MAX_CANDIDATES), top_k, torch.full_like(top_k, MAX_CANDIDATES))
    k_eff = k_eff.clamp(max=V).long()
    thr_k = torch.gather(sl, 1, (k_eff - 1)[:, None])
    cand = sl >= thr_k
    n_p = (cand & (prev < top_p.float()[:, None])).sum(-1).clamp(min=1)
    thr_p = torch.gather(sl, 1, (n_p - 1)[:, None])
    keep = cand & (sl >= thr_p)
    w = torch.where(keep, torch.exp((sl - xmax) / temp), torch.zeros_like(sl)).double()
    c = torch.cumsum(w, dim=-1)
    pick = (c <= u * c[:, -1:]).sum(-1)
    pick = torch.minimum(pick, keep.sum(-1) - 1)
    tok_cand = torch.gather(si, 1, pick[:, None])[:, 0]

    # plain multinomial path (index order)
    wf = torch.exp((x - xmax) / temp).double()
    cf = torch.cumsum(wf, dim=-1)
    tok_full = (cf <= u * cf[:, -1:]).sum(-1).clamp(max=V - 1)

    plain = (top_k <= 0) & (top_p.float() >= 1.0)
    tok = torch.where(plain, tok_full, tok_cand)
    return torch.where(greedy, arg, tok)


# --------------------------------------------------------------------------- vocab-parallel sampling oracle
def shard_summary(local_logits, offset: int, vocab: int, k: int):
    """What one TP rank would contribute to a vocab-parallel sampler (K11, general case) for its
    shard ``local_logits`` [B, Vb] whose column 0 is global token ``offset``: the local maximum, and
    every local element >= the local k-th largest (value, global index) -- ties included, which is
    what makes the merge exact (an element >= the global k-th value is >= its rank's local k-th value).
    Columns at or beyond ``vocab`` are padding."""
    x = local_logits.float().clone()
    B, Vb = x.shape
    n_valid = max(0, min(Vb, vocab - offset))
    x[:, n_valid:] = float("-inf")
    out = []
    for b in range(B):
        row = x[b, :n_valid]
        if n_valid == 0:
            out.append(dict(max=float("-inf"), vals=row.new_zeros(0), idx=torch.zeros(0, dtype=torch.long), row=row,
                            offset=offset))
            continue
        kk = min(k, n_valid)
        thr = torch.topk(row, kk).values[-1]
        sel = (row >= thr).nonzero()[:, 0]
        out.append(dict(max=row.max().item(), vals=row[sel], idx=sel + offset, row=row, offset=offset))
    return out


def sample_vocab_parallel(shards, greedy, temperature, top_k, top_p, rng_state, vocab: int, k_summary: int = 64,
                          u_shift: float = 0.0):
    """`sample()` computed from per-rank shard summaries only (the algorithm a vocab-parallel CUDA sampler
    follows; replaces the [B, V] logits all-gather of layers.py:131-135 + generate.py:109-129).

    ``shards``: list over ranks of fp32 [B, Vb] local logits (rank r starts at token r * Vb).
    Exchanged per row and rank: local max, local sum-exp, the local top-``k_summary`` candidates
    (+ ties); for the plain multinomial path two scalars (weight sum, count below the target).
    Rows whose effective k exceeds ``k_summary`` (top_k = 0 with top_p < 1 searches 1024 candidates)
    are outside this path -- the caller gathers the logits for them."""
    t = len(shards)
    B, Vb = shards[0].shape
    summ = [shard_summary(s, r * Vb, vocab, k_summary) for r, s in enumerate(shards)]
    u = (rng_uniform(rng_state[:, 0], rng_state[:, 1]).double() + u_shift).clamp(0.0, 1.0 - 2.0 ** -24)
    rng_state[:, 1] += 1
    toks = torch.zeros(B, dtype=torch.long)
    for b in range(B):
        rows = [summ[r][b] for r in range(t)]
        M = max(r_["max"] for r_ in rows)
        vals = torch.cat([r_["vals"] for r_ in rows])
        idx = torch.cat([r_["idx"] for r_ in rows])
        # global order: probability descending, index ascending
        o = torch.argsort(idx, stable=True)
        vals, idx = vals[o], idx[o]
        o = torch.argsort(vals, descending=True, stable=True)
        sl, si = vals[o], idx[o]
        if bool(greedy[b]):
            toks[b] = si[0]
            continue
        T = float(temperature[b])
        k, p = int(top_k[b]), float(top_p[b])
        if k <= 0 and p >= 1.0:
            # plain multinomial in index order: per-rank weight sums, then per-rank counts below the target
            w = [torch.exp((r_["row"] - M) / T).double() for r_ in rows]
            sums = [x.sum() for x in w]
            total = sum(sums)
            target = u[b] * total
            count, prefix = 0, 0.0
            for r in range(t):
                if len(w[r]):
                    count += int(((torch.cumsum(w[r], 0) + prefix) <= target).sum())
                prefix = prefix + sums[r]
            toks[b] = min(count, vocab - 1)
            continue
        k_eff = min(k if 0 < k <= MAX_CANDIDATES else MAX_CANDIDATES, vocab)
        if k_eff > k_summary:
            raise ValueError(f"row {b}: effective top-k {k_eff} exceeds the summary size {k_summary}")
        # global sum-exp from the ranks' (local max, local sum-exp) pairs
        Z = sum(float(torch.exp(r_["row"] - r_["max"]).sum()) * math.exp(r_["max"] - M) for r_ in rows if len(r_["row"]))
        thr_k = sl[k_eff - 1]
        head = sl >= thr_k            # complete: everything >= the global k-th value is in the union
        sl, si = sl[head], si[head]
        sp = torch.exp(sl - M) / Z
        prev = torch.cumsum(sp, 0) - sp
        n_p = max(int((prev < p).sum()), 1)
        keep = sl >= sl[n_p - 1]
        wt = torch.where(keep, torch.exp((sl - M) / T), torch.zeros_like(sl)).double()
        c = torch.cumsum(wt, 0)
        pick = min(int((c <= u[b] * c[-1]).sum()), int(keep.sum()) - 1)
        toks[b] = si[pick]
    return toks


# ----------------------------------------------------------------------------- recurrent layers, post-norm residual
# Conventions shared by the ops below.  A packed batch holds B sequences; sequence i owns rows cu_q[i]:cu_q[i+1], has
# seq_lens[i] tokens including those rows, and keeps its recurrent state in row state_slots[i] of every state tensor.
# A sequence whose first row is its position 0 starts from a zero state whatever its slot holds, so slots need no
# clearing when they are handed to a new sequence.  A slot < 0 marks an inert row (padding of a captured batch).
GATE_NONE, GATE_SILU, GATE_SIGMOID = 0, 1, 2
UNARY_TANH, UNARY_NEG_EXP = 0, 1
DECAY_HEAD, DECAY_TOKEN_HEAD, DECAY_TOKEN_CHANNEL = 0, 1, 2


def _seq_ranges(batch):
    cu, lens, slots = batch.cu_q.tolist(), batch.seq_lens.tolist(), batch.state_slots.tolist()
    for i in range(batch.num_seqs):
        q0, q1 = cu[i], cu[i + 1]
        if q1 > q0 and slots[i] >= 0:
            yield q0, q1, lens[i] - (q1 - q0), slots[i]


def _rms_div(x, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def embed_bigram(tokens, wte, table, mul_prev: int, mul_cur: int, buckets: int, batch, prev_state):
    """x[t] = wte[tok_t] + table[(prev * mul_prev + tok_t * mul_cur) mod buckets] in 32-bit; a sequence's first token
    takes row ``buckets``.  ``prev_state`` [slots] int32 keeps every sequence's last token between steps."""
    tok = tokens.long()
    x = F.embedding(tok, wte).float()
    for q0, q1, ctx, slot in _seq_ranges(batch):
        prev = torch.empty(q1 - q0, dtype=torch.long, device=tok.device)
        prev[1:] = tok[q0:q1 - 1]
        prev[0] = int(prev_state[slot]) if ctx > 0 else 0
        rows = (prev * mul_prev + tok[q0:q1] * mul_cur) % buckets
        if ctx == 0:
            rows[0] = buckets
        x[q0:q1] += F.embedding(rows, table).float()
        prev_state[slot] = tok[q1 - 1].to(prev_state.dtype)
    return x


def postnorm_residual(y, weight, eps: float, resid=None, y2=None, w_a=None, w_b=None, one_plus: bool = True, out_dtype=None):
    """Norm on a sub-layer's output, then the 32-bit residual sum.  n = rms_div(y) * (1 + weight) (``one_plus``) or
    * weight; with ``y2`` the input is first 0.5 * (rms_div(y) * w_a + rms_div(y2) * w_b) (two branches side by side).
    Returns (cast(resid + n), resid + n), or (cast(n), None) without a residual."""
    v = y.float()
    if y2 is not None:
        v = 0.5 * (_rms_div(v, eps) * w_a.float() + _rms_div(y2.float(), eps) * w_b.float())
    w = weight.float()
    n = _rms_div(v, eps) * ((1.0 + w) if one_plus else w)
    if resid is None:
        return n.to(out_dtype or weight.dtype), None
    r = resid.float() + n
    return r.to(out_dtype or weight.dtype), r


def token_shift(x, mu, batch, prev_state, out_dtype=None):
    """mix[s, t] = x[t] + (x[t - 1] - x[t]) * mu[s] for every mixing vector mu[s] (x[-1] of a sequence = 0);
    ``prev_state`` [slots, width] 32-bit carries each sequence's last row to its next step.  Returns [S, T, width]."""
    xf = x.float()
    prev = torch.zeros_like(xf)
    for q0, q1, ctx, slot in _seq_ranges(batch):
        prev[q0 + 1:q1] = xf[q0:q1 - 1]
        if ctx > 0:
            prev[q0] = prev_state[slot]
        prev_state[slot] = xf[q1 - 1]
    out = xf[None] + (prev - xf)[None] * mu.float()[:, None, :]
    return out.to(out_dtype or x.dtype)


def causal_conv(u, w, bias, act: int, batch, state, out_dtype=None):
    """Short causal convolution over time per channel: y_t = sum_j w[:, j] u_(t - taps + 1 + j) (+ bias), then ``act``.
    u [T, C] (a column view is fine), w [C, taps]; ``state`` [slots, taps - 1, C] 32-bit holds each sequence's last
    taps - 1 inputs (zeros before its start).  32-bit arithmetic; the result is 32-bit unless ``out_dtype`` says otherwise."""
    T, C = u.shape
    taps = w.shape[1]
    wf, uf = w.float(), u.float()
    y = torch.zeros(T, C, dtype=torch.float32, device=u.device)
    for q0, q1, ctx, slot in _seq_ranges(batch):
        hist = state[slot].float() if ctx > 0 and taps > 1 else torch.zeros(taps - 1, C, dtype=torch.float32, device=u.device)
        full = torch.cat([hist, uf[q0:q1]])
        for j in range(taps):
            y[q0:q1] += wf[:, j] * full[j:j + q1 - q0]
        if taps > 1:
            state[slot] = full[full.shape[0] - (taps - 1):]
    if bias is not None:
        y = y + bias.float()
    return apply_act(y, act).to(out_dtype or torch.float32)


def qknorm_kv_write(qkv, hq: int, hkv: int, dk: int, dv: int, q_w, k_w, eps: float, temp_coef: float, temp_every: int,
                    positions, slot_mapping, k_cache, v_cache, out_dtype=None, norm_whole: bool = False, v_norm: bool = False,
                    q_head_scale=None):
    """RMS norm of queries and keys, the query temperature 1 + coef * ln(floor((p + 1) / every) + 1) at position p
    (coef = 0: none), an optional factor per query head (``q_head_scale`` [hq]), and the append of k / v to the paged
    cache (k_cache [blocks, hkv, bs, dk], v_cache [blocks, hkv, bs, dv]).  The norm runs per head with one plain weight
    of size dk shared by the heads, or (``norm_whole``) over all heads of a token at once with a weight of the whole
    projection's size.  ``v_norm``: every value head is divided by its root mean square (no weight) before it is cached.
    qkv [T, hq*dk + hkv*dk + hkv*dv] 32-bit; hkv = 0: queries only (a layer that attends over another layer's pages).
    Returns the queries [T, hq * dk]."""
    T = qkv.shape[0]
    qf = qkv[:, :hq * dk].float()
    if norm_whole:
        q = (_rms_div(qf, eps) * q_w.float()).view(T, hq, dk)
    else:
        q = _rms_div(qf.view(T, hq, dk), eps) * q_w.float()
    if temp_coef != 0.0:
        temp = 1.0 + temp_coef * torch.log(torch.div(positions.long() + 1, temp_every, rounding_mode="floor").float() + 1.0)
        q = q * temp[:, None, None]
    if q_head_scale is not None:
        q = q * q_head_scale.float()[None, :, None]
    if hkv > 0:
        kf = qkv[:, hq * dk:(hq + hkv) * dk].float()
        if norm_whole:
            k = (_rms_div(kf, eps) * k_w.float()).view(T, hkv, dk)
        else:
            k = _rms_div(kf.view(T, hkv, dk), eps) * k_w.float()
        v = qkv[:, (hq + hkv) * dk:].float().view(T, hkv, dv)
        if v_norm:
            v = _rms_div(v, eps)
        bs = k_cache.shape[2]
        valid = slot_mapping >= 0
        slots = slot_mapping[valid].long()
        k_cache[slots // bs, :, slots % bs, :] = k[valid].to(k_cache.dtype)
        v_cache[slots // bs, :, slots % bs, :] = v[valid].to(v_cache.dtype)
    return q.reshape(T, hq * dk).to(out_dtype or k_cache.dtype)


def distance_bias_table(rel, max_distance: int):
    """Learned distance bias as a dense table: out[h, n] = rel[bucket(n), h] for n = 0 .. max_distance (larger distances
    use the last column).  Buckets: n itself below half of the B rows, then logarithmic up to ``max_distance``."""
    B, H = rel.shape
    half = B // 2
    cols = []
    for n in range(max_distance + 1):
        if n < half:
            b = n
        elif half == 0 or max_distance <= half:       # no logarithmic range left: everything from half on shares the last row
            b = B - 1
        else:
            b = min(B - 1, half + int(math.floor(math.log(n / half) / math.log(max_distance / half) * (B - half))))
        cols.append(rel[b].float())
    return torch.stack(cols, dim=1).contiguous()


# A scaled score that hides a key: exp(MASKED_SCORE - any real score) is exactly 0 in 32-bit, while the value is small enough
# that the rounding of products with it stays far below 1 (a huge value would turn the rounding error of scale * score into a
# huge exponent when a whole tile is hidden and the running maximum is the hidden score itself).
MASKED_SCORE = -30000.0


def window_bias_table(slopes, window: int, scale: float):
    """A sliding window plus a linear distance penalty as a distance table in raw-score units (the form the tensor-core
    attention kernels take): column d < window holds -slopes[h] * d / scale, the last column -- which those kernels use for
    every distance from ``window`` on -- hides the key."""
    d = torch.arange(window + 1, dtype=torch.float32, device=slopes.device)
    tab = -(slopes.float()[:, None] * d[None, :]) / float(scale)
    tab[:, window] = MASKED_SCORE / float(scale)
    return tab.contiguous()


def attention_bias(q, k_cache, v_cache, block_tables, seq_lens, cu_q, hq: int, hkv: int, dk: int, dv: int, scale: float,
                   dist_bias, gate=None, out_dtype=None, window: int = 0, slopes=None, sinks=None):
    """Causal softmax attention over the paged cache with key size dk, value size dv, grouped heads, an additive bias
    dist_bias[h, min(i - j, last)] per head and distance (or none), a linear penalty slopes[h] * (i - j) taken off the
    scores (or none), a sliding window (``window`` > 0: query i sees keys j with 0 <= i - j < window), an optional
    per-head output gate sigmoid(gate[t, h]), and an optional attention sink: ``sinks`` [hq] is a bare logit per head whose
    exponential is one more term of every softmax denominator of that head (nothing is added to the numerator, and the
    score scale does not apply to it)."""
    T = q.shape[0]
    bs, g = k_cache.shape[2], hq // hkv
    out = torch.zeros(T, hq, dv, dtype=torch.float32, device=q.device)
    cu, lens = cu_q.tolist(), seq_lens.tolist()
    for i, L in enumerate(lens):
        q0, q1 = cu[i], cu[i + 1]
        ql = q1 - q0
        if ql == 0 or L == 0:
            continue
        nb = (L + bs - 1) // bs
        blocks = block_tables[i, :nb].long()
        k = k_cache[blocks].permute(1, 0, 2, 3).reshape(hkv, nb * bs, dk)[:, :L].float().repeat_interleave(g, dim=0)
        v = v_cache[blocks].permute(1, 0, 2, 3).reshape(hkv, nb * bs, dv)[:, :L].float().repeat_interleave(g, dim=0)
        qi = q[q0:q1].float().view(ql, hq, dk).permute(1, 0, 2)
        s = torch.matmul(qi, k.transpose(1, 2)) * scale
        qpos = torch.arange(L - ql, L, device=q.device)[:, None]
        kpos = torch.arange(L, device=q.device)[None, :]
        if dist_bias is not None:
            dist = (qpos - kpos).clamp(min=0, max=dist_bias.shape[1] - 1)
            s = s + dist_bias.float()[:, dist.reshape(-1)].view(hq, ql, L)
        if slopes is not None:
            s = s - slopes.float()[:, None, None] * (qpos - kpos).float()[None]
        hidden = kpos > qpos
        if window > 0:
            hidden = hidden | (qpos - kpos >= window)
        s = s.masked_fill(hidden, float("-inf"))
        if sinks is not None:
            p = torch.softmax(torch.cat([s, sinks.float().view(hq, 1, 1).expand(hq, ql, 1)], dim=-1), dim=-1)[..., :L]
        else:
            p = torch.softmax(s, dim=-1)
        out[q0:q1] = torch.matmul(p, v).permute(1, 0, 2)
    if gate is not None:
        out = out * torch.sigmoid(gate.float())[:, :, None]
    return out.reshape(T, hq * dv).to(out_dtype or q.dtype)


def unary(x, op: int, out_dtype=None):
    y = torch.tanh(x.float()) if op == UNARY_TANH else -torch.exp(x.float())
    return y.to(out_dtype or x.dtype)


def ssm_dt(dt_raw, dt_bias, a_log):
    """Step sizes of a selective state-space layer: dt = softplus(dt_raw + dt_bias) (no clamp) and the log of the
    per-step decay, -exp(a_log) * dt; both [T, heads] 32-bit."""
    dt = F.softplus(dt_raw.float() + dt_bias.float(), threshold=30.0)
    return dt, -torch.exp(a_log.float()) * dt


def linear_scan(q, k, v, decay, decay_kind: int, batch, state, heads: int, qk_heads: int, dk: int, dv: int, bonus=None,
                v_scale=None, read_before: bool = False):
    """Gated linear recurrence per head, state S [dk, dv] in 32-bit:
         S_t = diag(a_t) S_(t-1) + k_t (c_t v_t)^T
         o_t = S_t^T q_t                                   (read_before = False)
         o_t = (S_(t-1) + diag(bonus) k_t (c_t v_t)^T)^T q_t     (read_before = True)
    q, k [T, qk_heads * dk] (head h reads q/k head h // (heads / qk_heads)), v [T, heads * dv], c = v_scale [T, heads] or 1.
    a_t: DECAY_HEAD -> decay[h]; DECAY_TOKEN_HEAD -> exp(decay[t, h]); DECAY_TOKEN_CHANNEL -> exp(decay[t, h * dk + i]).
    ``state`` [slots, heads, dk, dv].  Returns o [T, heads * dv] 32-bit."""
    T = v.shape[0]
    rep = heads // qk_heads
    qf = q.float().view(T, qk_heads, dk).repeat_interleave(rep, dim=1)
    kf = k.float().view(T, qk_heads, dk).repeat_interleave(rep, dim=1)
    vf = v.float().view(T, heads, dv)
    if v_scale is not None:
        vf = vf * v_scale.float()[:, :, None]
    if decay_kind == DECAY_HEAD:
        a = decay.float().view(1, heads, 1).expand(T, heads, dk)
    elif decay_kind == DECAY_TOKEN_HEAD:
        a = torch.exp(decay.float()).view(T, heads, 1).expand(T, heads, dk)
    else:
        a = torch.exp(decay.float()).view(T, heads, dk)
    out = torch.zeros(T, heads, dv, dtype=torch.float32, device=v.device)
    for q0, q1, ctx, slot in _seq_ranges(batch):
        S = state[slot].float().clone() if ctx > 0 else torch.zeros(heads, dk, dv, dtype=torch.float32, device=v.device)
        for t in range(q0, q1):
            kv = kf[t][:, :, None] * vf[t][:, None, :]
            if read_before:
                R = S + (bonus.float()[:, :, None] * kv if bonus is not None else 0.0)
                S = a[t][:, :, None] * S + kv
            else:
                S = a[t][:, :, None] * S + kv
                R = S
            out[t] = torch.einsum("hkv,hk->hv", R, qf[t])
        state[slot] = S
    return out.reshape(T, heads * dv)


def gated_rmsnorm(o, gate, gate_act: int, weight, groups: int, eps: float, gate_first: bool, skip_x=None, skip_d=None,
                  out_dtype=None):
    """Output stage of the recurrent mixers.  y = o (+ skip_d[h] * skip_x, head h = equal slices of the row); the row
    is cut into ``groups`` equal parts, each divided by its own root mean square, times ``weight``; the gate
    act(gate) multiplies before (``gate_first``) or after the norm."""
    T, C = o.shape
    y = o.float()
    if skip_x is not None:
        H = skip_d.numel()
        y = y + (skip_x.float().view(T, H, C // H) * skip_d.float()[None, :, None]).reshape(T, C)
    g = None
    if gate is not None and gate_act != GATE_NONE:
        g = F.silu(gate.float()) if gate_act == GATE_SILU else torch.sigmoid(gate.float())
    elif gate is not None:
        g = gate.float()
    if g is not None and gate_first:
        y = y * g
    y = _rms_div(y.view(T, groups, C // groups), eps).reshape(T, C)
    if weight is not None:
        y = y * weight.float()
    if g is not None and not gate_first:
        y = y * g
    return y.to(out_dtype or o.dtype)


# ----------------------------------------------------------------------------- several residual streams, delta rule
def embed_sinusoid(tokens, wte, scale: float, positions, streams: int = 1, base: float = 10000.0):
    """x[t] = wte[tok_t] * scale + pe(p_t) in 32-bit, pe(p)[c] = sin(p * base^(-2 (c // 2) / W)) for even c and cos of the
    same angle for odd c (angles in 64-bit).  Returns ``streams`` equal copies, [streams, T, W]."""
    W = wte.shape[1]
    c = torch.arange(W, device=wte.device)
    inv = torch.pow(torch.tensor(base, dtype=torch.float64, device=wte.device), -(2.0 * (c // 2).double()) / W)
    ang = positions.double()[:, None] * inv[None]
    pe = torch.where(c % 2 == 0, torch.sin(ang), torch.cos(ang))
    x = (F.embedding(tokens.long(), wte).float() * scale + pe.float())
    return x[None].repeat(streams, 1, 1).contiguous()


def hyper_residual(xs, y=None, mix=None, w_out=None, w_in=None, norm_w=None, eps: float = 0.0, out_dtype=None):
    """Residual update and read-out over several streams (hyper-connections), xs [S, T, W] 32-bit, in place:
         write (``y`` given):   xs_t <- sum_s mix[s, t] xs_s + w_out[t] * y      (all streams from the old ones)
         read (``w_in`` given): u = sum_s w_in[s] xs_s ;  returns rms_div(u) * norm_w, or u itself without ``norm_w``
    One stream with mix = [[1]], w_out = w_in = [1] is the plain pre-norm residual sum."""
    if y is not None:
        new = torch.einsum("st,sTw->tTw", mix.float(), xs) + w_out.float()[:, None, None] * y.float()[None]
        xs.copy_(new)
    if w_in is None:
        return None
    u = torch.einsum("s,sTw->Tw", w_in.float(), xs)
    if norm_w is not None:
        u = _rms_div(u, eps) * norm_w.float()
    return u.to(out_dtype or torch.float32)


def delta_scan(q, k, v, log_decay, beta, batch, state, heads: int, qk_heads: int, dk: int, dv: int, unit_eps=None,
               q_scale: float = 1.0, beta_sigmoid: bool = False):
    """Gated delta rule per head, state S [dk, dv] in 32-bit, in this order per token:
         S <- exp(log_decay_t) S ;  u = beta_t (v_t - S^T k_t) ;  S <- S + k_t u^T ;  o_t = S^T q_t
    q, k [T, qk_heads * dk] (head h reads q / k head h // (heads / qk_heads)); ``unit_eps``: q and k are first scaled to
    x / sqrt(sum(x^2) + unit_eps) per head; q is then multiplied by ``q_scale``.  v [T, heads * dv]; log_decay, beta
    [T, heads] (``beta_sigmoid``: beta is given before its sigmoid).  ``state`` [slots, heads, dk, dv].  o [T, heads * dv]."""
    T = v.shape[0]
    rep = heads // qk_heads
    qf, kf = q.float().view(T, qk_heads, dk), k.float().view(T, qk_heads, dk)
    if unit_eps is not None:
        qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + unit_eps)
        kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + unit_eps)
    qf = (qf * q_scale).repeat_interleave(rep, dim=1)
    kf = kf.repeat_interleave(rep, dim=1)
    vf = v.float().view(T, heads, dv)
    a = torch.exp(log_decay.float())
    b = torch.sigmoid(beta.float()) if beta_sigmoid else beta.float()
    out = torch.zeros(T, heads, dv, dtype=torch.float32, device=v.device)
    for q0, q1, ctx, slot in _seq_ranges(batch):
        S = state[slot].float().clone() if ctx > 0 else torch.zeros(heads, dk, dv, dtype=torch.float32, device=v.device)
        for t in range(q0, q1):
            S = S * a[t][:, None, None]
            u = b[t][:, None] * (vf[t] - torch.einsum("hkv,hk->hv", S, kf[t]))
            S = S + kf[t][:, :, None] * u[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, qf[t])
        state[slot] = S
    return out.reshape(T, heads * dv)


# ----------------------------------------------------------------------------- rotation by a frequency table, sandwich norms
def rotary_frequencies(dims: int, base: float, scaling=None):
    """Frequencies of a rotary position embedding over ``dims`` channels as a table, plus the factor on cos and sin:
    (f [dims / 2] float64, magnitude).  f_i = base^(-2 i / dims); ``scaling`` = {"factor"} divides every frequency (linear
    position interpolation); {"factor", "original", "fast", "slow"} blends per frequency (YaRN): with
    dim(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), dims - 1)
    and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency is f_i / factor * ramp_i + f_i (1 - ramp_i) and
    the magnitude 0.1 ln(factor) + 1.  The kernels take the table, so any other schedule is a different table."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor = float(scaling["factor"])
    if "original" not in scaling:
        return f / factor, 1.0
    orig, fast, slow = float(scaling["original"]), float(scaling["fast"]), float(scaling["slow"])

    def at(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo, hi = max(math.floor(at(fast)), 0), min(math.ceil(at(slow)), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def _rotate_by_table(x, positions, freq, mag: float, interleaved: bool):
    """x [T, heads, d] 32-bit: the first 2 * len(freq) channels of every head are rotated (angles in 64-bit), the rest pass."""
    n = freq.numel()
    if n == 0:
        return x
    ang = positions.double()[:, None] * freq.double().to(x.device)[None, :]
    c, s = (torch.cos(ang) * mag).float()[:, None, :], (torch.sin(ang) * mag).float()[:, None, :]
    part, rest = x[..., :2 * n], x[..., 2 * n:]
    if interleaved:
        u, v = part[..., 0::2], part[..., 1::2]
        out = torch.stack((u * c - v * s, v * c + u * s), dim=-1).flatten(-2)
    else:
        u, v = part[..., :n], part[..., n:]
        out = torch.cat((u * c - v * s, v * c + u * s), dim=-1)
    return torch.cat((out, rest), dim=-1)


def rope_norm_kv_write(qk, hq: int, hkv: int, d: int, freq, mag: float, interleaved: bool, unit_norm: bool, eps: float,
                       positions, slot_mapping, k_cache, v_cache, out_dtype=None):
    """Queries and keys of grouped-query attention in which the raw key projection doubles as the value.  qk [T, hq*d + hkv*d] 32-bit.
    q and k are rotated by the frequency table (pairs (2i, 2i+1) if ``interleaved`` else (i, i + n)), then -- ``unit_norm``
    -- every head is divided by its root mean square (no weight).  The prepared keys go to the K pages, the projected
    keys themselves (before rotation and norm) to the V pages.  Returns the queries [T, hq * d]."""
    T = qk.shape[0]
    q = qk[:, :hq * d].float().view(T, hq, d)
    k = qk[:, hq * d:(hq + hkv) * d].float().view(T, hkv, d)
    qr, kr = _rotate_by_table(q, positions, freq, mag, interleaved), _rotate_by_table(k, positions, freq, mag, interleaved)
    if unit_norm:
        qr, kr = _rms_div(qr, eps), _rms_div(kr, eps)
    bs = k_cache.shape[2]
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    k_cache[slots // bs, :, slots % bs, :] = kr[valid].to(k_cache.dtype)
    v_cache[slots // bs, :, slots % bs, :] = k[valid].to(v_cache.dtype)
    return qr.reshape(T, hq * d).to(out_dtype or k_cache.dtype)


def latent_rope_prep(y, q_off: int, q_rank: int, c_off: int, rank: int, rot: int, g_off: int, n_gate: int, qn_w, cn_w, eps: float,
                     freq, mag: float, positions, slot_mapping, cache, dtype):
    """First stage of latent attention with a rotated key part, on the layer's fused 32-bit projection y [T, *]:
    the query latent y[:, q_off : q_off + q_rank] is RMS-normed (weight ``qn_w``) and returned in ``dtype`` (the operand of the
    query up-projection; q_rank = 0: there is none); the key / value latent y[:, c_off : c_off + rank] is RMS-normed
    (weight ``cn_w``), the ``rot`` columns behind it are rotated (interleaved pairs) and not normed, and both are written
    side by side into the token's cache row (cache [num_blocks, block_size, >= rank + rot]; columns beyond are zeroed);
    sigmoid of the n_gate gate columns is returned in 32-bit ([T, n_gate], or None)."""
    T = y.shape[0]
    cq = None
    if q_rank > 0:
        cq = (_rms_div(y[:, q_off:q_off + q_rank].float(), eps) * qn_w.float()).to(dtype)
    c = _rms_div(y[:, c_off:c_off + rank].float(), eps) * cn_w.float()
    kr = _rotate_by_table(y[:, c_off + rank:c_off + rank + rot].float().reshape(T, 1, rot), positions, freq, mag, True).reshape(T, rot)
    width = cache.shape[-1]
    row = torch.zeros(T, width, dtype=torch.float32, device=y.device)
    row[:, :rank], row[:, rank:rank + rot] = c, kr
    valid = slot_mapping >= 0
    cache.view(-1, width)[slot_mapping[valid].long()] = row[valid].to(cache.dtype)
    gate = torch.sigmoid(y[:, g_off:g_off + n_gate].float()) if n_gate > 0 else None
    return cq, gate


def latent_query_rope(q, heads: int, d: int, rot: int, rank: int, width: int, freq, mag: float, positions, dtype, abs_dtype):
    """Second stage: q [T, heads * (d + rot)] (every head [d unrotated | rot rotated]).  Returns (q_nope [T, heads * d] in
    ``dtype`` -- the operand of the per-head key absorption -- and the absorbed-query buffer [T, heads * width] in
    ``abs_dtype`` whose columns [rank, rank + rot) of every head hold the rotated part (interleaved pairs); columns below
    ``rank`` are left for the absorption product, columns beyond rank + rot are zero."""
    T = q.shape[0]
    qh = q.float().view(T, heads, d + rot)
    qa = torch.zeros(T, heads, width, dtype=abs_dtype, device=q.device)
    qa[:, :, rank:rank + rot] = _rotate_by_table(qh[..., d:], positions, freq, mag, True).to(abs_dtype)
    return qh[..., :d].reshape(T, heads * d).to(dtype), qa.view(T, heads * width)


def hgrn_gates(y, n_qk: int, lower):
    """Inputs of a gated linear recurrence whose forget gate also decides what is written, from y [T, 2 n_qk + *] 32-bit
    = [q | f | ...]: q <- silu(q); f = lower + (1 - lower) sigmoid(f); returns (q, k = 1 - f, ln f), each [T, n_qk] 32-bit.
    1 - f is formed as (1 - lower) sigmoid(-f_raw), without cancellation."""
    q = F.silu(y[:, :n_qk].float())
    z = y[:, n_qk:2 * n_qk].float()
    lo = lower.float()
    f = lo + (1.0 - lo) * torch.sigmoid(z)
    k = (1.0 - lo) * torch.sigmoid(-z)
    return q, k, torch.log(f)


def sandwich_residual(resid, y, w_post, eps: float, w_next=None, history=None, index: int = 0, depth_w=None, out_dtype=None):
    """Residual update of a sub-layer that is normed on both sides, fused with the norm in front of the next one:
         r = resid + rms_div(y) * w_post                                (y None: r = resid)
         history given:  history[index] = r ;  r = sum_(j <= index) depth_w[j] * history[j]     (depth-weighted average)
         h = rms_div(r) * w_next                                        (w_next None: no h)
    resid [T, W] 32-bit, y [T, W] 32-bit, history [n, T, W] 32-bit.  Returns (h in ``out_dtype`` or None, r 32-bit)."""
    r = resid.float()
    if y is not None:
        r = r + _rms_div(y.float(), eps) * w_post.float()
    if history is not None:
        history[index] = r
        if depth_w is not None:
            r = torch.einsum("j,jtw->tw", depth_w.float()[:index + 1], history[:index + 1])
    h = None
    if w_next is not None:
        h = (_rms_div(r, eps) * w_next.float()).to(out_dtype or torch.float32)
    return h, r


def softcap(z, cap: float):
    """cap * tanh(z / cap), in place on 32-bit logits."""
    return z.copy_(cap * torch.tanh(z.float() / cap))
