"""Zenorax: a decoder-only design whose sub-layers are normed on both sides, whose mixers read a short causal convolution
of their normed input, and whose layers pass on a learned weighted average of all layer outputs so far.

    X_0 = embed[token] * scale                                                  (32-bit from here on)
    layer i, input x:   h = rms_div(x) * norm1 ;  h <- h + conv(h)              causal over time per channel, taps from config
                        x <- x + rms_div(mixer(h)) * norm1b
                        x <- x + rms_div(ffn(rms_div(x) * norm2)) * norm2b      (layers with a feed-forward)
                        X_(i+1) = x ;  the next layer (or the output) reads  sum_(j <= i+1) dwa[j] X_j
    mixers:  "latent_attention" (query latent, rotated key part, YaRN frequencies, per-channel output gate) -> blocks.RotaryLatentAttention
             "attention" (values = keys, rotate-half positions with linear scaling, unit-RMS q / k, sink)   -> mixers.SinkAttention
             "hgrn2" (gated linear recurrence)                                                              -> mixers.Hgrn2Mixer
    ffn:     routed experts W_down relu(W_up h)^2, sigmoid scores, choice by score + correction, groups scored by their two
             best, weights not renormalised                                                                 -> blocks.RoutedExperts
    logits = softcap * tanh(embed (rms_div(x) * final.norm) / softcap)          the embedding table is the output matrix

config.json keys: architecture, vocab, width, norm.eps, embedding.scale, canon.taps, logit_softcap,
layers[i].{type, mixer{...}, mlp{kind, expert.ff, router{experts, top, groups{count, keep}}} | null}.
Tensor names: embed, final.norm, l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.canon1 [width, taps], l<i>.dwa [i + 2],
l<i>.mix.*, l<i>.mlp.{router, correction, e<j>.up, e<j>.down} (listed with each loader below).

The model is a graph over the framework's ops.  What a sequence carries between steps lives in the engine's HybridCache:
K / V pages (attention), latent pages (latent attention), and one state slot for the recurrent states and every layer's
last taps - 1 normed rows.  Runner, block and slot allocators, batching and sampler drive it like the other families.
It runs unsharded (TP = 1).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch
from torch import nn

from .. import ops
from ..engine.batch import BatchInput
from ..engine.kv_cache import HybridCache
from ..ops import ACT_NONE, ACT_RELU2
from ..parallel.comm import comm_for
from ..utils.tracing import trace
from .blocks import RotaryLatentAttention, RoutedExperts
from .mixers import Hgrn2Mixer, LayerCacheView, SinkAttention

MIXER_TYPES = ("latent_attention", "attention", "hgrn2")
FFN_KINDS = ("moe",)
F32 = torch.float32


@dataclass
class ZenoraxSpec:
    hidden: int
    vocab: int
    eps: float
    embed_scale: float
    taps: int                    # canon.taps (0: no input convolution)
    softcap: float               # 0: none
    layers: List[dict] = field(default_factory=list)      # the config's layer entries, checked
    model_type: str = "zenorax"
    max_pos: int = 1 << 30       # rotary positions: no limit of its own
    default_seq_len: int = 4096  # block-table width when the caller names neither a length nor a pool
    learned_pos: bool = False

    @property
    def n_layers(self) -> int:
        return len(self.layers)


def zenorax_spec(config) -> ZenoraxSpec:
    c = config.raw if hasattr(config, "raw") else dict(config)
    layers = list(c["layers"])
    for i, lc in enumerate(layers):
        if lc["type"] not in MIXER_TYPES:
            raise ValueError(f"zenorax: layer {i} has unknown mixer type {lc['type']!r}; have {MIXER_TYPES}")
        f = lc.get("mlp")
        if f is not None and f.get("kind", "moe") not in FFN_KINDS:
            raise ValueError(f"zenorax: layer {i} has unknown feed-forward kind {f.get('kind')!r}; have {FFN_KINDS}")
        m = lc["mixer"]
        if lc["type"] == "attention" and int(m.get("vdim", m["dim"])) != int(m["dim"]):
            raise ValueError(f"zenorax: layer {i}: the values are the keys, so vdim must equal dim")
    return ZenoraxSpec(int(c["width"]), int(c["vocab"]), float(c["norm"]["eps"]), float((c.get("embedding") or {}).get("scale", 1.0)),
                       int((c.get("canon") or {}).get("taps", 0)), float(c.get("logit_softcap") or 0.0), layers)


def _rotary(rot: Optional[dict], default_dims: int):
    """(frequency table, magnitude) of a mixer's ``rot`` entry {base, dims, scaling}; no entry: no rotation."""
    if not rot:
        return torch.zeros(0, dtype=torch.float64), 1.0
    return ops.rotary_frequencies(int(rot.get("dims", default_dims)), float(rot["base"]), rot.get("scaling"))


def _build_mixer(kind: str, m: dict, width: int, eps: float):
    if kind == "hgrn2":
        return Hgrn2Mixer(width, int(m["heads"]), int(m["dim"]), int(m["vdim"]), eps)
    if kind == "attention":
        d = int(m["dim"])
        freq, mag = _rotary(m.get("rot"), d)
        return SinkAttention(width, int(m["heads"]), int(m["kv_heads"]), d, float(m.get("scale", d ** -0.5)), eps, freq, mag)
    d, r = int(m["dim"]), int(m["rot_dim"])
    freq, mag = _rotary(m.get("rot"), r)
    if 2 * freq.numel() > r:
        raise ValueError("zenorax: latent attention rotates more channels than rot_dim has")
    return RotaryLatentAttention(int(m["heads"]), d, r, int(m["vdim"]), int(m["kv_rank"]), int(m["q_rank"]),
                                 float(m.get("scale", (d + r) ** -0.5)), eps, freq, mag)


class ZenoraxLayer:
    __slots__ = ("kind", "mixer", "ffn", "norm1", "norm1b", "norm2", "norm2b", "canon_w", "dwa", "w_in")


class ZenoraxLM(nn.Module):
    """The decoder core the engine drives (same surface as DecoderLM: forward / forward_hidden / logits / make_cache)."""

    needs_state = True     # the runner gives every sequence a state slot, and neither shares nor evicts its pages

    def __init__(self, spec: ZenoraxSpec, process_group, device, dtype):
        super().__init__()
        self.spec = spec
        self.comm = comm_for(process_group, device)
        self.tp, self.rank = self.comm.size, self.comm.rank
        if self.tp != 1:
            raise NotImplementedError("zenorax runs unsharded: start it with one rank")
        self.device, self.dtype = torch.device(device), dtype
        self.vocab_blk = spec.vocab
        self.layers: List[ZenoraxLayer] = []
        for lc in spec.layers:
            L = ZenoraxLayer()
            L.kind = lc["type"]
            L.mixer = _build_mixer(lc["type"], lc["mixer"], spec.hidden, spec.eps)
            f = lc.get("mlp")
            L.ffn = None
            if f is not None:
                r = f["router"]
                g = r.get("groups") or {"count": 1, "keep": 1}
                L.ffn = RoutedExperts(int(r["experts"]), int(r["top"]), int(g["count"]), int(g["keep"]), 1.0, int(f["expert"]["ff"]),
                                      act=ACT_RELU2, score="sigmoid", group_top=2, renorm=False)
            L.norm1 = L.norm1b = L.norm2 = L.norm2b = L.canon_w = L.dwa = L.w_in = None
            self.layers.append(L)
        self.wte = self.final_w = None

    # ------------------------------------------------------------------ cache
    def default_block_size(self) -> int:
        return 64 if self.device.type == "cuda" else 16

    def make_cache(self, num_blocks: int, block_size: int, max_seqs: Optional[int] = None) -> HybridCache:
        kv, latents, states = {}, {}, {}
        for i, L in enumerate(self.layers):
            if isinstance(L.mixer, RotaryLatentAttention):
                latents[i] = L.mixer.choose_width(self.device, self.dtype)
            elif L.mixer.kv_shape() is not None:
                kv[i] = L.mixer.kv_shape()
            if L.canon_w is not None and L.canon_w.shape[1] > 1:
                states[(i, "canon")] = ((L.canon_w.shape[1] - 1, self.spec.hidden), F32)
            if not isinstance(L.mixer, RotaryLatentAttention):
                for name, sd in L.mixer.state_shapes().items():
                    states[(i, name)] = sd
        return HybridCache(kv, states, num_blocks, block_size, max_seqs or 1, self.dtype, self.device, latents=latents)

    def num_parameters_local(self) -> int:
        ts = [self.wte, self.final_w]
        for L in self.layers:
            ts += [L.norm1, L.norm1b, L.norm2, L.norm2b, L.canon_w, L.dwa, L.w_in] + L.mixer.weights()
            if L.ffn is not None:
                ts += [L.ffn.w_router, L.ffn.correction, L.ffn.w_up, L.ffn.w_down]
        return sum(t.numel() for t in ts if t is not None)

    def finalize(self):
        """Latent layers: the rows of everything that reads the mixer's input stacked into one projection."""
        for L in self.layers:
            if isinstance(L.mixer, RotaryLatentAttention):
                L.w_in = L.mixer.in_rows().contiguous()
                assert L.mixer.bind(0) == L.w_in.shape[0]
        return self

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, batch: BatchInput, kv: HybridCache, taps: Optional[list] = None) -> torch.Tensor:
        """Final-normed hidden states [T, width] of every packed token.  ``taps``: a list that receives the 32-bit
        residual stream that leaves every layer (debugging / tests)."""
        s, dt = self.spec, self.dtype
        assert batch.state_slots is not None, "zenorax: the batch names no state slots"
        n, T = len(self.layers), batch.tokens.numel()
        averaged = any(L.dwa is not None for L in self.layers)
        hist = torch.empty(n + 1, T, s.hidden, dtype=F32, device=self.device) if averaged else None
        with trace("embed"):
            x = ops.embed(batch.tokens, self.wte, out_dtype=F32, scale=s.embed_scale, out=hist[0] if averaged else None)

        def pre_dtype(L):       # a layer with an input convolution takes its normed input in 32-bit (the convolution rounds)
            return F32 if L.canon_w is not None else dt

        with trace("sandwich_residual"):
            h, _ = ops.sandwich_residual(x, None, None, s.eps, w_next=self.layers[0].norm1, out_dtype=pre_dtype(self.layers[0]))
        for i, L in enumerate(self.layers):
            lc = LayerCacheView(kv, i)
            if L.canon_w is not None:
                with trace("causal_conv"):
                    h = ops.causal_conv(h, L.canon_w, None, ACT_NONE, batch, lc.state("canon") if L.canon_w.shape[1] > 1 else None,
                                        out_dtype=dt)
            if isinstance(L.mixer, RotaryLatentAttention):
                with trace("gemm_in"):
                    y = ops.linear(h, L.w_in, out_dtype=F32)
                y = L.mixer.forward(y, batch, lc.latent, dt)
            else:
                y = L.mixer.forward(h, batch, lc, dt)
            w_post = L.norm1b
            if L.ffn is not None:
                with trace("sandwich_residual"):
                    h, x = ops.sandwich_residual(x, y, L.norm1b, s.eps, w_next=L.norm2, out_dtype=dt)
                y, w_post = L.ffn.forward(h), L.norm2b
            last = i == n - 1
            with trace("sandwich_residual"):
                h, x = ops.sandwich_residual(x, y, w_post, s.eps, w_next=self.final_w if last else self.layers[i + 1].norm1,
                                             history=hist, index=i + 1, depth_w=L.dwa,
                                             out_dtype=dt if last else pre_dtype(self.layers[i + 1]))
            if taps is not None:
                taps.append(x.clone())
        return h

    def logits(self, hidden_rows: torch.Tensor) -> torch.Tensor:
        with trace("lm_head"):
            z = ops.linear(hidden_rows, self.wte, out_dtype=torch.float32)
            return ops.softcap(z, self.spec.softcap) if self.spec.softcap else z

    local_logits = logits

    def forward(self, batch: BatchInput, kv, last_only: bool = True, gather_logits: bool = True) -> torch.Tensor:
        h = self.forward_hidden(batch, kv)
        if last_only:
            h = h.index_select(0, batch.last_idx)
        return self.logits(h)


# ---------------------------------------------------------------------------------------------------- weights
def _f32(t):
    """Small per-channel parameters are kept in 32-bit whatever the compute type (the checkpoint's values are exact in it)."""
    return t.float().contiguous()


def _load_latent(mx: RotaryLatentAttention, get, p):
    """<p>.dq [q_rank, W] + .dq.norm [q_rank]; <p>.uq [heads*(dim+rot_dim), q_rank]; <p>.dkv [kv_rank+rot_dim, W] + .dkv.norm
    [kv_rank]; <p>.uk [heads*dim, kv_rank]; <p>.uv [heads*vdim, kv_rank]; <p>.g [heads*vdim, W]; <p>.o [W, heads*vdim]."""
    mx.w_dq, mx.qn_w, mx.w_uq = get(f"{p}.dq"), _f32(get(f"{p}.dq.norm")), get(f"{p}.uq").contiguous()
    mx.w_dkv, mx.cn_w = get(f"{p}.dkv"), _f32(get(f"{p}.dkv.norm"))
    mx.w_uk, mx.w_uv = get(f"{p}.uk").contiguous(), get(f"{p}.uv").contiguous()
    mx.w_g, mx.w_o = get(f"{p}.g"), get(f"{p}.o").contiguous()


def _load_attention(mx: SinkAttention, get, p):
    """<p>.q [heads*dim, W]; <p>.k [kv_heads*dim, W]; <p>.sink [heads]; <p>.o [W, heads*dim]."""
    mx.set_weights(get(f"{p}.q"), get(f"{p}.k"), _f32(get(f"{p}.sink")), get(f"{p}.o"))


def _load_hgrn2(mx: Hgrn2Mixer, get, p):
    """<p>.q / .f [heads*dim, W]; <p>.f.b / .lower [heads*dim]; <p>.v [heads*vdim, W]; <p>.norm [vdim]; <p>.o [W, heads*vdim]."""
    mx.set_weights(get(f"{p}.q"), get(f"{p}.f"), get(f"{p}.f.b"), get(f"{p}.v"), _f32(get(f"{p}.lower")), _f32(get(f"{p}.norm")),
                   get(f"{p}.o"))


_LOADERS = {"latent_attention": _load_latent, "attention": _load_attention, "hgrn2": _load_hgrn2}


def load_zenorax(m: ZenoraxLM, w):
    get = w.get_tensor
    m.wte, m.final_w = get("embed").contiguous(), _f32(get("final.norm"))
    for i, L in enumerate(m.layers):
        p = f"l{i}"
        L.norm1, L.norm1b = _f32(get(f"{p}.norm1")), _f32(get(f"{p}.norm1b"))
        if w.has(f"{p}.canon1"):
            # h + conv(h) is one convolution whose last tap (the current token's) is 1 larger
            cw = _f32(get(f"{p}.canon1")).clone()
            cw[:, -1] += 1.0
            L.canon_w = cw
        L.dwa = _f32(get(f"{p}.dwa")) if w.has(f"{p}.dwa") else None
        _LOADERS[L.kind](L.mixer, get, f"{p}.mix")
        if L.ffn is None:
            continue
        L.norm2, L.norm2b = _f32(get(f"{p}.norm2")), _f32(get(f"{p}.norm2b"))
        ff, E = L.ffn, L.ffn.experts
        ff.w_router = get(f"{p}.mlp.router").contiguous()
        ff.correction = _f32(get(f"{p}.mlp.correction")) if w.has(f"{p}.mlp.correction") else None
        ff.w_up = torch.stack([get(f"{p}.mlp.e{e}.up") for e in range(E)]).contiguous()           # [E, F, W]
        ff.w_down = torch.cat([get(f"{p}.mlp.e{e}.down") for e in range(E)], dim=1).contiguous()   # [W, E * F]
