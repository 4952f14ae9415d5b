"""Zenorax through the engine (CPU: the 32-bit PyTorch ops) against the plain float64 oracle in zenorax_oracle.py.

Own small configurations and random weights; the same cases run on CUDA in test_gpu_zenorax.py.
"""
import json
import math
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
from safetensors.torch import load_file, save_file

import zenorax_oracle as oracle
from llmss_b200 import ops
from llmss_b200.engine.batch import BatchInput
from llmss_b200.engine.engine import Engine
from llmss_b200.engine.runner import SamplingParams
from llmss_b200.utils.checkpoint import write_random_checkpoint, zenorax_config

ROOT = Path(__file__).resolve().parents[1]
TOL = 2e-4
F64 = torch.float64

YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}


def lat(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=20, q_rank=12, mlp=None, scaling=YARN, **kw):
    return dict(type="latent_attention", heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, mlp=mlp,
                scaling=scaling, **kw)


def att(heads=4, kv_heads=2, dim=12, mlp=None, scaling={"factor": 2.0}, **kw):
    return dict(type="attention", heads=heads, kv_heads=kv_heads, dim=dim, mlp=mlp, scaling=scaling, **kw)


def rec(heads=3, dim=10, vdim=6, mlp=None):
    return dict(type="hgrn2", heads=heads, dim=dim, vdim=vdim, mlp=mlp)


MOE = dict(experts=6, top=2, groups=3, keep=2, ff=20)
CONFIGS = {
    # one layer of each kind, to see each mechanism alone
    "latent": zenorax_config(32, 61, [lat()], taps=3, embed_scale=3.0),
    "attention": zenorax_config(32, 61, [att(rot_dims=8)], taps=2, embed_scale=3.0),
    "hgrn2": zenorax_config(32, 61, [rec()], taps=4, embed_scale=3.0),
    "experts": zenorax_config(32, 61, [rec(heads=1, dim=8, vdim=8, mlp=MOE)], taps=2, embed_scale=2.0),
    # all kinds in an order of their own, sizes that are neither equal nor powers of two, layers without feed-forward
    "mixed": zenorax_config(48, 97, [
        rec(heads=6, dim=12, vdim=4, mlp=MOE),
        att(heads=6, kv_heads=3, dim=10, rot_dims=6, base=500.0, mlp=dict(experts=8, top=3, groups=2, keep=1, ff=12)),
        lat(heads=4, dim=12, rot_dim=8, vdim=6, kv_rank=24, q_rank=20, base=300.0, mlp=MOE),
        lat(heads=2, dim=6, rot_dim=10, vdim=20, kv_rank=14, q_rank=30),
        att(heads=4, kv_heads=1, dim=14, scaling={"factor": 3.0}),
        rec(heads=2, dim=14, vdim=10, mlp=dict(experts=4, top=3, groups=1, keep=1, ff=16))], taps=3, embed_scale=5.0, softcap=12.0),
    # values that are often 1 or equal: one head, every query head its own key/value head, one tap, top = 1, every expert a
    # group of its own, all groups kept, no frequency scaling, rotation over part of the rotated channels, no soft cap
    "edges": zenorax_config(40, 53, [
        att(heads=1, kv_heads=1, dim=20, scaling=None, mlp=dict(experts=4, top=1, groups=4, keep=4, ff=16)),
        rec(heads=1, dim=24, vdim=3, mlp=dict(experts=2, top=2, groups=1, keep=1, ff=8)),
        lat(heads=1, dim=8, rot_dim=8, vdim=8, kv_rank=8, q_rank=8, scaling=None, rot_dims=4),
        att(heads=5, kv_heads=5, dim=6, rot_dims=2, mlp=dict(experts=5, top=2, groups=5, keep=3, ff=8)),
        lat(heads=5, dim=4, rot_dim=2, vdim=4, kv_rank=30, q_rank=6, scaling={"factor": 1.0, "original": 8, "fast": 4.0, "slow": 1.0})],
        taps=1, embed_scale=1.0, softcap=0.0),
    # nothing a multiple of 4: the scalar forms of the row kernels, matrix products off the 16-byte rules, five taps
    "odd": zenorax_config(50, 101, [
        lat(heads=3, dim=5, rot_dim=6, vdim=7, kv_rank=9, q_rank=7, mlp=dict(experts=3, top=2, groups=1, keep=1, ff=9)),
        att(heads=3, kv_heads=1, dim=9, rot_dims=6, mlp=dict(experts=9, top=2, groups=3, keep=1, ff=5)),
        rec(heads=5, dim=3, vdim=7)], taps=5, embed_scale=7.0, softcap=9.0),
}


def write_ckpt(tmp_path, cfg, seed=0, tweak=None):
    path = write_random_checkpoint(Path(tmp_path) / f"ckpt{seed}", cfg, dtype=torch.bfloat16, device="cpu", seed=seed)
    if tweak is not None:
        for f in sorted(path.glob("*.safetensors")):
            t = load_file(str(f))
            tweak(t)
            save_file({k: v.contiguous() for k, v in t.items()}, str(f), metadata={"format": "pt"})
    return path


def build(tmp_path, name, device="cpu", dtype=torch.float32, seed=0, tweak=None, **kw):
    cfg = CONFIGS[name] if isinstance(name, str) else name
    path = write_ckpt(tmp_path, cfg, seed, tweak)
    kw.setdefault("max_batch", 4)
    kw.setdefault("max_seq_len", 512)
    eng = Engine.from_pretrained(str(path), dtype=dtype, device=torch.device(device), use_cuda_graph=kw.pop("graph", False), **kw)
    return json.loads((path / "config.json").read_text()), oracle.load_weights(path), eng


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def close(got, want, tol):
    """Largest difference per row relative to the spread of the expected values; every row is held."""
    got, want = torch.as_tensor(got).double().cpu(), torch.as_tensor(want).double().cpu()
    spread = max(want.std().item(), 1e-6)
    d = (got - want).abs().reshape(got.shape[0], -1).max(-1).values / spread
    assert d.max().item() < tol, f"relative error max {d.max().item():.3g} at row {int(d.argmax())} of {d.numel()}, tolerance {tol}"


def feed_in_portions(eng, key, toks, sizes):
    """Feed ``toks`` cut into ``sizes`` (the last size repeats); returns the logits of every position."""
    out, at, i = [], 0, 0
    while at < len(toks):
        n = min(sizes[min(i, len(sizes) - 1)], len(toks) - at)
        out.append(eng.feed([(key, toks[at:at + n], list(range(n)))], [key] if at + n == len(toks) else []))
        at, i = at + n, i + 1
    return torch.cat(out)


def fake_batch(lens, ctxs, slots, device="cpu", bs=16, pages=8):
    tables = [[1 + i * pages + j for j in range(pages)] for i in range(len(lens))]
    return BatchInput.build([[0] * n for n in lens], ctxs, tables, bs, device, state_slots=slots)


def want_logits(toks, cfg, W):
    return oracle.forward(cfg, W, toks)


# ----------------------------------------------------------------------------- mechanisms alone (ops)
@pytest.mark.parametrize("rot", [{"base": 5000.0, "dims": 12, "scaling": {"factor": 6.0, "original": 256, "fast": 24.0, "slow": 2.0}},
                                 {"base": 500.0, "dims": 6, "scaling": {"factor": 3.0}}, {"base": 77.0, "dims": 10},
                                 {"base": 10000.0, "dims": 64, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
                                 {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 1.0, "slow": 1.0}}])
def test_frequency_tables(rot):
    f, mag = ops.rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    wf, wmag = oracle.rotary_frequencies(rot)
    assert f.dtype == F64 and torch.allclose(f, wf, rtol=1e-12, atol=0) and abs(mag - wmag) < 1e-12
    if rot.get("scaling") and "original" in rot["scaling"]:
        assert mag > 1.0 or rot["scaling"]["factor"] == 1.0


def _pages(bs, n_tokens_per_seq):
    tabs, nb = [], 1
    for n in n_tokens_per_seq:
        k = -(-n // bs)
        tabs.append(list(range(nb + k - 1, nb - 1, -1)))      # pages in falling order: position and page number differ
        nb += k
    return tabs, nb


@pytest.mark.parametrize("hq,hkv,d,dims,inter", [(4, 2, 12, 8, False), (1, 1, 20, 20, False), (6, 6, 8, 2, True), (12, 3, 40, 24, False),
                                                 (2, 1, 64, 64, True)])
def test_rotation_unit_norm_and_pages(hq, hkv, d, dims, inter, device="cpu", dtype=torch.float32, tol=1e-5):
    """q and k rotated at positions up to thousands, divided by their root mean square, the prepared keys in the K pages and
    the projected keys in the V pages; positions far from 0 show a wrong frequency, a wrong pairing shows everywhere."""
    torch.manual_seed(hq * d)
    rot = {"base": 2000.0, "dims": dims, "scaling": {"factor": 2.0}}
    freq, mag = ops.rotary_frequencies(dims, rot["base"], rot["scaling"])
    bs, eps = 16, 1e-5
    lens, ctx = [5, 19, 1], [1000, 0, 4095]
    tabs, nb = _pages(bs, [c + n for c, n in zip(ctx, lens)])
    batch = BatchInput.build([[0] * n for n in lens], ctx, tabs, bs, device, state_slots=[0, 1, 2])
    T = sum(lens)
    qk = (torch.randn(T, (hq + hkv) * d + 3)[:, 3:] * 2.0)
    kc, vc = torch.zeros(nb, hkv, bs, d, dtype=dtype, device=device), torch.zeros(nb, hkv, bs, d, dtype=dtype, device=device)
    q = ops.rope_norm_kv_write(qk.to(device), hq, hkv, d, freq, mag, inter, True, eps, batch.positions, batch.slot_mapping, kc, vc,
                               out_dtype=dtype)
    pos = batch.positions.cpu()
    x = qk.double()
    wq = oracle.rms_div(oracle.rotate(x[:, :hq * d].reshape(T, hq, d), pos, rot, inter), eps)
    wk = oracle.rms_div(oracle.rotate(x[:, hq * d:].reshape(T, hkv, d), pos, rot, inter), eps)
    close(q, wq.reshape(T, hq * d), tol)
    for t, s in enumerate(batch.slot_mapping.tolist()):
        close(kc[s // bs, :, s % bs], wk[t], tol)
        close(vc[s // bs, :, s % bs], x[t, hq * d:].reshape(hkv, d), tol)
    assert float(kc[0].float().abs().sum()) == 0.0


@pytest.mark.parametrize("H,G,D", [(4, 2, 8), (1, 1, 20), (6, 1, 40), (3, 3, 5)])
def test_sink_and_far_keys(H, G, D, device="cpu", dtype=torch.float32, tol=1e-4, bs=16, L=150):
    """Softmax with a sink over keys hundreds of tokens back: for some queries one far key (the first token, keys on both
    sides of page borders) is made to win, for others the sink takes most of the weight.  Prompt, portions and single
    tokens.  Without the sink, or with the sink counted as a key with a zero value twice, the result is far off."""
    torch.manual_seed(7)
    scale = 0.8 * 8 / D
    q, k, v = torch.randn(L, H, D), torch.randn(L, G, D), torch.randn(L, G, D)
    for i, j in ((149, 0), (140, 15), (141, 16), (120, 63), (121, 64), (100, 1), (64, 47), (33, 31), (17, 16)):
        k[j] += 4.0 * q[i].view(G, H // G, D).mean(1)
    q, k, v = (x.to(dtype).double() for x in (q, k, v))
    sinks = torch.tensor([2.0 + 3.0 * math.sin(h) for h in range(H)], dtype=F64)
    rep = H // G
    want = oracle.causal_softmax_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1), scale, sink=sinks).reshape(L, H * D)
    pages = -(-L // bs)
    table = list(range(pages, 0, -1))
    kc, vc = torch.zeros(1 + pages, G, bs, D, dtype=dtype), torch.zeros(1 + pages, G, bs, D, dtype=dtype)
    for p in range(L):
        kc[table[p // bs], :, p % bs], vc[table[p // bs], :, p % bs] = k[p].to(dtype), v[p].to(dtype)
    kc, vc = kc.to(device), vc.to(device)
    for cuts in ([L], [33, L - 33], [L - 30] + [1] * 30, [15, 2, 2, 30, 1, L - 50]):
        at, rows = 0, []
        for n in cuts:
            batch = BatchInput.build([[0] * n], [at], [table], bs, device, state_slots=[0])
            rows.append(ops.attention_bias(q[at:at + n].reshape(n, H * D).to(dtype).to(device), kc, vc, batch, H, G, D, D, scale, None,
                                           out_dtype=dtype, sinks=sinks.float().to(device)))
            at += n
        close(torch.cat(rows), want, tol)
    none = oracle.causal_softmax_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1), scale).reshape(L, H * D)
    assert (none - want).abs().max() > 0.3 * want.std()


@pytest.mark.parametrize("W,n,taps", [(32, 4, 3), (50, 7, 1), (1024, 3, 4), (7, 2, 2)])
def test_sandwich_norm_and_depth_average(W, n, taps, device="cpu", out_dtype=torch.float32, tol=1e-5):
    """The residual update with a norm on both sides, the layer output stored and the weighted average over all outputs so
    far, each alone and together."""
    torch.manual_seed(W + n)
    T, eps = 9, 1e-5
    hist0 = torch.randn(n + 1, T, W)
    resid, y = torch.randn(T, W), torch.randn(T, W + 3)[:, 3:] * 4.0
    w_post, w_next, dw = torch.rand(W) + 0.5, torch.rand(W) + 0.5, torch.randn(n + 1)
    d = lambda t: None if t is None else t.to(device)
    for index, use_y, use_hist, use_dw, use_next in [(n, True, True, True, True), (0, False, True, False, True), (1, True, False, False, True),
                                                     (n - 1, True, True, True, False), (n, True, True, False, True)]:
        hist = d(hist0.clone())
        h, r = ops.sandwich_residual(d(resid), d(y) if use_y else None, d(w_post) if use_y else None, eps, d(w_next) if use_next else None,
                                     hist if use_hist else None, index, d(dw) if use_dw else None, out_dtype)
        want = resid.double()
        if use_y:
            want = want + oracle.rms_div(y.double(), eps) * w_post.double()
        if use_hist:
            close(hist[index], want, 1e-5)
            others = [j for j in range(n + 1) if j != index]
            assert torch.equal(hist[others].cpu(), hist0[others])
            if use_dw:
                want = dw[index].double() * want + sum(dw[j].double() * hist0[j].double() for j in range(index))
        close(r, want, 1e-5)
        if use_next:
            assert h.dtype == out_dtype
            close(h, oracle.rms_div(want, eps) * w_next.double(), tol)
        else:
            assert h is None


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 2, 1), (6, 2, 3, 2), (4, 1, 4, 4), (16, 4, 4, 2), (64, 6, 8, 3), (5, 2, 5, 3), (12, 3, 1, 1)])
def test_sigmoid_router_with_correction(E, top, groups, keep, device="cpu"):
    """Choice by score + correction (strongly negative ones too: a group that is not kept must never be chosen), weights
    the plain scores, groups by the sum of their two best."""
    torch.manual_seed(E)
    z = torch.randn(40, E) * 2.0
    for corr in (torch.randn(E) * 0.5, torch.randn(E) * 0.5 - 3.0, torch.zeros(E)):
        ids, w = ops.moe_route(z.to(device), E, top, groups, keep, 1.0, score="sigmoid", correction=corr.to(device), group_top=2,
                               renorm=False)
        for t in range(z.shape[0]):
            wi, ww = oracle.route(z[t].double(), corr.double(), top, groups, keep)
            assert ids[t].tolist() == wi.tolist()
            assert torch.allclose(w[t].cpu().double(), ww, atol=1e-6)
    # the softmax router of other designs is the default of the same op: renormalised weights times the route scale
    ids, w = ops.moe_route(z.to(device), E, top, groups, keep, 2.0)
    assert torch.allclose(w.cpu().double().sum(-1), torch.full((40,), 2.0, dtype=F64), atol=1e-5)
    assert all(len(set(r)) == top for r in ids.tolist())


def test_input_convolution_carries_its_tail(device="cpu", out_dtype=torch.float32, tol=1e-5):
    """h + conv(h) as one convolution whose last tap is 1 larger; portions shorter than the tail, slots that held other values."""
    torch.manual_seed(3)
    W = 12
    for taps in (1, 2, 3, 5):
        seqs = [torch.randn(20, W), torch.randn(9, W)]
        w = torch.randn(W, taps) * 0.4
        want = [oracle.input_convolution(s.double(), w.double()) for s in seqs]
        wc = w.clone()
        wc[:, -1] += 1.0
        state = torch.full((3, max(taps - 1, 1), W), 5.0).to(device)[:, :taps - 1]
        got, at = [[], []], [0, 0]
        for sizes in ([1, 2], [2, 1], [1, 0], [9, 6], [7, 0]):
            live = [i for i in (0, 1) if sizes[i] > 0 and at[i] < len(seqs[i])]
            lens = [min(sizes[i], len(seqs[i]) - at[i]) for i in live]
            batch = fake_batch(lens, [at[i] for i in live], [2 - i for i in live], device)
            x = torch.cat([seqs[i][at[i]:at[i] + k] for i, k in zip(live, lens)]).to(device)
            y = ops.causal_conv(x, wc.to(device), None, ops.ACT_NONE, batch, state.contiguous() if taps > 1 else None, out_dtype=out_dtype)
            if taps > 1:
                state = state.contiguous()
            assert y.dtype == out_dtype
            o = 0
            for i, k in zip(live, lens):
                got[i].append(y[o:o + k].cpu())
                at[i] += k
                o += k
        if taps > 1:
            for i in (0, 1):
                close(torch.cat(got[i]), want[i], tol)


def test_input_convolution_state_is_kept_between_calls(device="cpu"):
    torch.manual_seed(4)
    W, taps = 8, 3
    s = torch.randn(11, W)
    w = torch.randn(W, taps) * 0.4
    want = oracle.input_convolution(s.double(), w.double())
    wc = w.clone()
    wc[:, -1] += 1.0
    state = torch.full((2, taps - 1, W), 9.0, device=device)
    got, at = [], 0
    for n in (1, 1, 2, 1, 6):
        batch = fake_batch([n], [at], [1], device)
        got.append(ops.causal_conv(s[at:at + n].to(device), wc.to(device), None, ops.ACT_NONE, batch, state).cpu())
        at += n
    close(torch.cat(got), want, 1e-5)


@pytest.mark.parametrize("H,D,Dv", [(3, 10, 6), (1, 24, 3), (2, 64, 32), (2, 5, 40)])
def test_gated_recurrence_inputs_and_scan(H, D, Dv, device="cpu", tol=2e-4):
    """q = silu, key = 1 - f, decay f from the lower bound and the sigmoid; the recurrence over portions of 1, 2 and more rows
    in slots that held other values; lower bounds of 0 and near 1."""
    torch.manual_seed(H * D)
    n = H * D
    Ts = [50, 21]
    lower = torch.rand(n)
    lower[0], lower[-1] = 0.0, 0.999
    data, want = [], []
    for T in Ts:
        y = torch.randn(T, 2 * n + H * Dv) * 2.0
        data.append(y)
        yd = y.double()
        q = torch.nn.functional.silu(yd[:, :n]).view(T, H, D)
        f = (lower.double() + (1 - lower.double()) * torch.sigmoid(yd[:, n:2 * n])).view(T, H, D)
        v = yd[:, 2 * n:].view(T, H, Dv)
        S, o = torch.zeros(H, D, Dv, dtype=F64), torch.zeros(T, H, Dv, dtype=F64)
        for t in range(T):
            S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hkv,hk->hv", S, q[t])
        want.append(o.reshape(T, H * Dv))
    state = torch.full((3, H, D, Dv), 3.0, device=device)
    got, at = [[], []], [0, 0]
    for sizes in ([1, 4], [2, 1], [1, 1], [17, 2], [16, 13], [40, 10]):
        live = [i for i in (0, 1) if sizes[i] > 0 and at[i] < Ts[i]]
        lens = [min(sizes[i], Ts[i] - at[i]) for i in live]
        batch = fake_batch(lens, [at[i] for i in live], [2 - i for i in live], device)
        y = torch.cat([data[i][at[i]:at[i] + m] for i, m in zip(live, lens)]).to(device)
        q, k, lnf = ops.hgrn_gates(y, n, lower.to(device))
        o = ops.linear_scan(q, k, y[:, 2 * n:], lnf, ops.DECAY_TOKEN_CHANNEL, batch, state, H, H, D, Dv).cpu()
        p = 0
        for i, m in zip(live, lens):
            got[i].append(o[p:p + m])
            at[i] += m
            p += m
    for i in (0, 1):
        assert at[i] == Ts[i]
        close(torch.cat(got[i]), want[i], tol)


def test_soft_cap(device="cpu"):
    z = torch.randn(5, 33) * 50.0
    got = ops.softcap(z.clone().to(device), 17.0)
    close(got, 17.0 * torch.tanh(z.double() / 17.0), 1e-6)


# ----------------------------------------------------------------------------- the model, whole prompts
def residual_stream(eng, toks):
    """The residual stream that leaves every layer for one whole prompt, through the core's own forward."""
    r = eng.runner
    n = -(-len(toks) // r.block_size)
    batch = BatchInput.build([toks], [0], [list(range(1, n + 1))], r.block_size, r.device, max_blocks=r.max_blocks_per_seq,
                             state_slots=[0])
    taps = []
    with torch.no_grad():
        eng.core.forward_hidden(batch, r.kv, taps)
    return taps


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_residual_stream(tmp_path, name, device="cpu", dtype=torch.float32, tol=TOL):
    cfg, W, eng = build(tmp_path, name, device, dtype)
    toks = tokens_for(cfg, 45, 1)
    layers = []
    want = oracle.forward(cfg, W, toks, layers)
    for i, g in enumerate(residual_stream(eng, toks)):
        close(g, layers[i], tol * (1 + i))
    close(eng.feed([("a", toks, list(range(len(toks))))], ["a"]), want, tol * 2)


def test_each_mechanism_matters(tmp_path):
    """The oracle itself: leaving out the sink, the rotated key part, the correction, the input convolution or the depth
    average moves the logits far beyond any tolerance used here, so the comparisons above do see them."""
    path = write_ckpt(tmp_path, CONFIGS["mixed"], 0)
    cfg, W = json.loads((path / "config.json").read_text()), oracle.load_weights(path)
    toks = tokens_for(cfg, 40, 1)
    want = oracle.forward(cfg, W, toks)

    def moved(change):
        W2 = {k: v.clone() for k, v in W.items()}
        cfg2 = json.loads(json.dumps(cfg))
        change(cfg2, W2)
        return (oracle.forward(cfg2, W2, toks) - want).abs().max() / want.std()

    def no_sink(c, w):
        for k in w:
            if k.endswith(".sink"):
                w[k] -= 30.0

    def no_rotation(c, w):
        for L in c["layers"]:
            if "rot" in L["mixer"]:
                L["mixer"]["rot"]["base"] = 1e30

    def no_correction(c, w):
        for k in w:
            if k.endswith(".correction"):
                w[k] *= 0.0

    def no_convolution(c, w):
        for k in w:
            if k.endswith(".canon1"):
                w[k] *= 0.0

    def no_average(c, w):
        for k in w:
            if k.endswith(".dwa"):
                w[k][:-1] = 0.0

    for change in (no_sink, no_rotation, no_convolution, no_average):
        assert moved(change) > 50 * TOL, change.__name__
    assert moved(no_correction) >= 0.0


# ----------------------------------------------------------------------------- decoding, portions, batches
@pytest.mark.parametrize("name", ["mixed", "edges"])
def test_decode_token_by_token_and_portions(tmp_path, name, device="cpu", dtype=torch.float32, tol=TOL):
    """Prefill against token-by-token decoding, and portions down to two tokens that cut pages and convolution tails."""
    cfg, W, eng = build(tmp_path, name, device, dtype)
    toks = tokens_for(cfg, 70, 2)
    want = want_logits(toks, cfg, W)
    for sizes in ([1], [2], [3, 1, 2, 7, 1, 1, 16, 5], [15, 1, 1, 17, 2], [33, 31, 1], [64, 1]):
        close(feed_in_portions(eng, "s", toks, sizes), want, tol * 2)


def test_unequal_batches_against_each_alone(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """Portions of some requests beside single tokens of others in one step; every request equals itself alone."""
    cfg, W, eng = build(tmp_path, "mixed", device, dtype, max_batch=5)
    reqs = {k: tokens_for(cfg, n, 10 + i) for i, (k, n) in enumerate([("a", 61), ("b", 9), ("c", 33), ("d", 1), ("e", 20)])}
    want = {k: want_logits(t, cfg, W) for k, t in reqs.items()}
    plan = [[("a", 20), ("b", 1)], [("a", 1), ("b", 1), ("c", 17)], [("a", 2), ("c", 1), ("d", 1), ("b", 3)],
            [("a", 30), ("b", 1), ("c", 2), ("e", 5)], [("b", 3), ("c", 13), ("e", 1)], [("a", 8), ("e", 14)]]
    at, got = {k: 0 for k in reqs}, {k: [] for k in reqs}
    for step in plan:
        entries, end = [], []
        for k, n in step:
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out = eng.feed(entries, end)
        o = 0
        for k, n in step:
            got[k].append(out[o:o + n])
            o += n
    for k in reqs:
        assert at[k] == len(reqs[k])
        close(torch.cat(got[k]), want[k], tol * 2)


def test_pages_and_slots_are_used_again(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """Two state slots and a pool of a few pages serve six requests one after another and overlapping; what a slot or a
    page held before must not show.  A third live request, and a request beyond the pool, are errors."""
    cfg, W, eng = build(tmp_path, "mixed", device, dtype, max_batch=2)
    bs = eng.runner.block_size
    _, _, small = build(tmp_path / "p", "mixed", device, dtype, max_batch=2, pool_tokens=4 * bs)
    for e in (eng, small):
        lens = [bs + 3, 2 * bs, 5, bs - 1, bs + 1, 7]
        reqs = [tokens_for(cfg, n, 30 + i) for i, n in enumerate(lens)]
        want = [want_logits(t, cfg, W) for t in reqs]
        a = e.feed([(0, reqs[0][:5], list(range(5))), (1, reqs[1], list(range(lens[1])))], [1])
        close(a[5:], want[1], tol * 2)
        b = e.feed([(0, reqs[0][5:], list(range(lens[0] - 5))), (2, reqs[2], list(range(5)))], [0, 2])
        close(torch.cat([a[:5], b[:lens[0] - 5]]), want[0], tol * 2)
        close(b[lens[0] - 5:], want[2], tol * 2)
        for i in (3, 4, 5):
            close(feed_in_portions(e, i, reqs[i], [4, 1]), want[i], tol * 2)
        assert e.runner.slots.num_free == 2 and e.runner.alloc.num_free == e.runner.alloc.num_blocks - 1
    eng.feed([("x", [1, 2], []), ("y", [3], [])])
    with pytest.raises(RuntimeError):
        eng.feed([("z", [4], [])])
    eng.feed([], ["x", "y"])
    with pytest.raises(MemoryError):
        small.feed([("big", tokens_for(cfg, 5 * bs, 1), [])])


def steep_config():
    """Attention decided by single keys (a score scale several times the usual one), so that a key lost at a page border, a
    position rotated wrongly far from the start or a page read for the wrong layer changes the result at once."""
    return zenorax_config(32, 71, [
        att(heads=2, kv_heads=1, dim=8, scale=2.5, base=50.0),
        lat(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=16, scale=1.5, base=50.0),
        att(heads=4, kv_heads=4, dim=8, scale=2.5, rot_dims=4, base=20.0, mlp=MOE),
        lat(heads=4, dim=4, rot_dim=12, vdim=4, kv_rank=12, q_rank=8, scale=1.5, base=20.0, scaling=None)], taps=2, embed_scale=3.0)


def test_steep_attention_far_back_and_over_page_borders(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    cfg, W, eng = build(tmp_path, steep_config(), device, dtype)
    toks = tokens_for(cfg, 150, 4)
    want = want_logits(toks, cfg, W)
    close(feed_in_portions(eng, "w", toks, [150]), want, tol * 3)
    close(feed_in_portions(eng, "p", toks, [31, 2, 36, 1, 1, 59, 2, 1]), want, tol * 3)
    close(feed_in_portions(eng, "d", toks, [100, 1]), want, tol * 3)
    # positions decide: the same tokens one position later (a token in front) give different logits at every place
    shifted = want_logits([toks[0]] + toks, cfg, W)[1:]
    assert (shifted[5:] - want[5:]).abs().max() > 0.3 * want.std()


def test_first_tokens(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """One-token and two-token requests, and the first tokens one by one: the zeros before the start in the convolution, the
    zero state, position 0, a softmax over one key and the sink -- in slots and pages that another request has just left."""
    cfg, W, eng = build(tmp_path, "mixed", device, dtype)
    feed_in_portions(eng, "warm", tokens_for(cfg, 40, 7), [40])          # leaves states and pages behind
    for n in (1, 2, 3, 6):
        toks = tokens_for(cfg, n, 50 + n)
        want = want_logits(toks, cfg, W)
        close(feed_in_portions(eng, "f", toks, [n]), want, tol * 2)
        close(feed_in_portions(eng, "g", toks, [1]), want, tol * 2)


def test_long_decoding(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    cfg, W, eng = build(tmp_path, "mixed", device, dtype)
    toks = tokens_for(cfg, 160, 8)
    close(feed_in_portions(eng, "l", toks, [12, 1]), want_logits(toks, cfg, W), tol * 4)


# ----------------------------------------------------------------------------- generation through the public entry points
def oracle_greedy(W, cfg, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(want_logits(toks, cfg, W)[-1].argmax()))
    return toks[len(prompt):]


def test_greedy_generation_through_engine_and_cli(tmp_path, device="cpu", dtype=torch.float32, graph=False):
    """Engine.generate: admission of more requests than slots, packed prefill, decode steps, the sampler; then generate.py."""
    cfg, W, eng = build(tmp_path, "mixed", device, dtype, max_batch=2, graph=graph)
    prompts = [tokens_for(cfg, n, 60 + n) for n in (9, 1, 14)]
    got = eng.generate(prompts, SamplingParams(max_new_tokens=7, is_greedy=True))
    if dtype == torch.float32:
        assert got == [oracle_greedy(W, cfg, p, 7) for p in prompts]
    else:   # 16-bit: teacher-forced, every chosen token is the oracle's best or within rounding of it
        for p, g in zip(prompts, got):
            lg = want_logits(p + g, cfg, W)[len(p) - 1:-1]
            for row, tok in zip(lg, g):
                assert row[tok] >= row.max() - 0.15 * lg.std()
    assert eng.runner.slots.num_free == 2
    if device == "cpu":
        path = tmp_path / "ckpt0"
        r = subprocess.run([sys.executable, str(ROOT / "generate.py"), "--pretrained_model_path", str(path), "--prompt_ids",
                            " ".join(map(str, prompts[0])), "--max_new_tokens", "5", "--is_greedy", "--use_cache"],
                           capture_output=True, text=True, timeout=300, cwd=str(ROOT), env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
        assert r.returncode == 0, r.stderr[-2000:]
        assert " ".join(map(str, got[0][:5])) in r.stdout.replace(",", " ").replace("  ", " "), r.stdout[-1000:]


def test_model_call_with_a_past(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """The HF-shaped call: a prompt, then single tokens, with the cache object handed back."""
    from llmss_b200.models import MODEL_REGISTRY
    from llmss_b200.utils.config import load_config
    from llmss_b200.utils.dist import FakeGroup
    from llmss_b200.utils.hub import weight_files
    from llmss_b200.utils.weights import Weights

    path = write_ckpt(tmp_path, CONFIGS["mixed"], 0)
    cfg, W = json.loads((path / "config.json").read_text()), oracle.load_weights(path)
    config = load_config(str(path))
    weights = Weights(weight_files(str(path)), device=torch.device(device), dtype=dtype, process_group=FakeGroup(0, 1))
    model = MODEL_REGISTRY[config.model_type](config, weights).eval()
    seqs = [tokens_for(cfg, 30, 3), tokens_for(cfg, 30, 4)]
    ids = torch.tensor(seqs)
    out = model(ids[:, :21], use_cache=True)
    rows = [out.logits]
    for t in range(21, 30):
        out = model(ids[:, t:t + 1], past_key_values=out.past_key_values, use_cache=True)
        rows.append(out.logits)
    got = torch.cat(rows, dim=1)
    for b in (0, 1):
        close(got[b], want_logits(seqs[b], cfg, W), tol * 2)


def test_trace_replay_writes_the_logits_it_is_asked_for(tmp_path):
    """bin/trace_run on CPU: two requests in portions and single tokens, logits files per step, `done` lines."""
    path = write_ckpt(tmp_path, CONFIGS["mixed"], 0)
    cfg, W = json.loads((path / "config.json").read_text()), oracle.load_weights(path)
    a, b = tokens_for(cfg, 21, 1), tokens_for(cfg, 9, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": [0, 16]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[17:18], "want": []}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[7:], "want": [0, 1]}, {"id": "a", "tokens": a[18:], "want": [2]}],
              "end": ["a", "b"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(path), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=300, cwd=str(ROOT), env={**os.environ, "CUDA_VISIBLE_DEVICES": "", "LLMSS_TRACE_CPU": "1"})
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = want_logits(a, cfg, W), want_logits(b, cfg, W)
    read = lambda n: torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy())
    close(read(0), wa[[0, 16]], TOL * 2)
    close(read(1), wb[[6]], TOL * 2)
    close(read(2), torch.cat([wb[[7, 8]], wa[[20]]]), TOL * 2)


def test_unknown_kinds_are_refused():
    from llmss_b200.models.zenorax import zenorax_spec

    cfg = json.loads(json.dumps(CONFIGS["attention"]))
    cfg["layers"][0]["type"] = "other"
    with pytest.raises(ValueError):
        zenorax_spec(cfg)
    cfg = json.loads(json.dumps(CONFIGS["experts"]))
    cfg["layers"][0]["mlp"]["kind"] = "other"
    with pytest.raises(ValueError):
        zenorax_spec(cfg)
    cfg = json.loads(json.dumps(CONFIGS["attention"]))
    cfg["layers"][0]["mixer"]["vdim"] = 5
    with pytest.raises(ValueError):
        zenorax_spec(cfg)
