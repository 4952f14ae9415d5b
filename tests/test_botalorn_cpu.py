"""Botalorn through the engine (CPU: the 32-bit PyTorch ops) against the plain float64 oracle in botalorn_oracle.py.

Own small configurations and random weights; the same cases run on CUDA in test_gpu_botalorn.py.
"""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
from safetensors.torch import load_file, save_file

import botalorn_oracle as oracle
from llmss_b200 import ops
from llmss_b200.engine.batch import BatchInput
from llmss_b200.engine.engine import Engine
from llmss_b200.engine.runner import SamplingParams
from llmss_b200.utils.checkpoint import botalorn_config, write_random_checkpoint

ROOT = Path(__file__).resolve().parents[1]
TOL = 2e-4


def att(heads=3, kv_heads=1, dim=10, vdim=6, conv=3, window=12, mlp=None, **kw):
    return dict(type="attention", heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, window=window, mlp=mlp, **kw)


def dlt(heads=4, kv_heads=2, dim=10, vdim=6, conv=4, mlp=None):
    return dict(type="delta", heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, mlp=mlp)


FF = {"ff": 40}
CONFIGS = {
    # one layer of each kind, to see each mechanism alone
    "attention": botalorn_config(32, 61, [att()], streams=2, embed_scale=3.0),
    "delta": botalorn_config(32, 61, [dlt()], streams=2, embed_scale=3.0),
    "dense": botalorn_config(32, 61, [dlt(heads=1, kv_heads=1, dim=8, vdim=8, mlp=FF)], streams=3, embed_scale=2.0),
    "shared": botalorn_config(32, 61, [att(heads=4, kv_heads=2, window=9), att(heads=4, kv_heads=2, window=30, conv=2, kv_from=0)],
                              streams=2, embed_scale=3.0),
    # all kinds in an order of their own, sizes that are neither equal nor powers of two; two lenders, a borrower behind a
    # delta layer, layers without feed-forward, windows shorter and longer than a page
    "mixed": botalorn_config(48, 97, [
        dlt(heads=6, kv_heads=3, dim=12, vdim=4, conv=3, mlp=FF),
        att(heads=4, kv_heads=2, dim=12, vdim=8, conv=3, window=21, mlp=FF),
        att(heads=6, kv_heads=1, dim=8, vdim=12, conv=4, window=7),
        dlt(heads=2, kv_heads=2, dim=14, vdim=10, conv=2, mlp=FF),
        att(heads=4, kv_heads=2, dim=12, vdim=8, conv=2, window=40, kv_from=1, mlp=FF),
        att(heads=6, kv_heads=1, dim=8, vdim=12, conv=1, window=3, kv_from=2)], streams=3, embed_scale=5.0),
    # values that are often 1 or equal: one stream, one head, every query head its own key/value head, one tap, a window of
    # one token, a window longer than any test prompt, no window at all, one value head per query/key head
    "edges": botalorn_config(40, 53, [
        att(heads=1, kv_heads=1, dim=20, vdim=4, conv=1, window=1, mlp=FF),
        dlt(heads=1, kv_heads=1, dim=24, vdim=3, conv=1, mlp={"ff": 16}),
        att(heads=5, kv_heads=5, dim=6, vdim=10, conv=4, window=1000),
        att(heads=5, kv_heads=5, dim=6, vdim=10, conv=5, window=None, kv_from=2, mlp=FF),
        dlt(heads=3, kv_heads=3, dim=5, vdim=9, conv=5)], streams=1, embed_scale=1.0),
    # no hyper-connection tensors at all: the plain pre-norm residual sum
    "plain": botalorn_config(32, 61, [att(mlp=FF), dlt(mlp=FF)], streams=None, embed_scale=4.0),
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
    return oracle.forward(toks, cfg, W)[0]


# ----------------------------------------------------------------------------- mechanisms alone (ops)
@pytest.mark.parametrize("W,streams,scale", [(32, 1, 1.0), (50, 3, 12.0), (7, 2, 0.5)])
def test_embedding_with_sinusoid(W, streams, scale, device="cpu", dtype=torch.float32, tol=1e-5):
    torch.manual_seed(W)
    table = torch.randn(29, W).to(dtype)
    toks = torch.randint(0, 29, (11,), dtype=torch.int32)
    pos = torch.tensor([0, 1, 2, 3, 900, 901, 12345, 0, 1, 63, 64], dtype=torch.int32)
    xs = ops.embed_sinusoid(toks.to(device), table.to(device), scale, pos.to(device), streams)
    assert xs.shape == (streams, 11, W) and xs.dtype == torch.float32
    want = table.double().numpy()[toks.numpy()] * scale
    for i, p in enumerate(pos.tolist()):
        want[i] += oracle.sinusoid(p + 1, W)[p]
    for s in range(streams):
        close(xs[s], want, tol)


@pytest.mark.parametrize("S,W", [(1, 24), (2, 32), (3, 50), (5, 7), (11, 20)])
def test_hyper_residual_op(S, W, device="cpu", out_dtype=torch.float32, tol=1e-5):
    """Write only, read only, both at once, the read-out without a norm; the write takes every stream from the OLD ones."""
    torch.manual_seed(S * 100 + W)
    T, eps = 9, 1e-5
    xs0, y = torch.randn(S, T, W), torch.randn(T, W + 3)[:, 3:]            # y: a column view of a wider tensor
    mix, w_out, w_in, nw = torch.randn(S, S), torch.randn(S), torch.randn(S), torch.randn(W)
    d = lambda t: t.to(device)
    f = lambda t: t.double().numpy()
    written = oracle.hyper_write(f(xs0), f(y), f(mix), f(w_out))
    xs = d(xs0.clone())
    assert ops.hyper_residual(xs, d(y), d(mix), d(w_out)) is None
    close(xs.reshape(S * T, W), written.reshape(S * T, W), 1e-5)
    xs = d(xs0.clone())
    h = ops.hyper_residual(xs, None, None, None, d(w_in), d(nw), eps, out_dtype=out_dtype)
    assert torch.equal(xs.cpu(), xs0) and h.dtype == out_dtype
    close(h, oracle.rms_div(oracle.hyper_read(f(xs0), f(w_in)), eps) * f(nw), tol)
    xs = d(xs0.clone())
    h = ops.hyper_residual(xs, d(y), d(mix), d(w_out), d(w_in), d(nw), eps, out_dtype=out_dtype)
    close(xs.reshape(S * T, W), written.reshape(S * T, W), 1e-5)
    close(h, oracle.rms_div(oracle.hyper_read(written, f(w_in)), eps) * f(nw), tol)
    u = ops.hyper_residual(xs, None, None, None, d(torch.ones(S)))
    close(u, written.sum(0), 1e-5)


def test_token_shift_carries_the_previous_row(device="cpu"):
    torch.manual_seed(3)
    W = 12
    seqs = [torch.randn(20, W), torch.randn(9, W)]
    mu = torch.rand(1, W)
    want = [oracle.token_shift(s.double().numpy(), mu[0].double().numpy()) for s in seqs]
    state = torch.full((3, W), 5.0).to(device)
    got, at = [[], []], [0, 0]
    for sizes in ([1, 2], [2, 1], [1, 0], [9, 6], [7, 0]):
        live = [i for i in (0, 1) if sizes[i] > 0 and at[i] < len(seqs[i])]
        lens = [min(sizes[i], len(seqs[i]) - at[i]) for i in live]
        batch = fake_batch(lens, [at[i] for i in live], [2 - i for i in live], device)
        x = torch.cat([seqs[i][at[i]:at[i] + k] for i, k in zip(live, lens)]).to(device)
        y = ops.token_shift(x, mu.to(device), batch, state)[0].cpu()
        o = 0
        for i, k in zip(live, lens):
            got[i].append(y[o:o + k])
            at[i] += k
            o += k
    for i in (0, 1):
        close(torch.cat(got[i]), want[i], 1e-5)


@pytest.mark.parametrize("hq,hkv,dk,dv", [(4, 2, 10, 6), (1, 1, 20, 4), (6, 6, 8, 8), (12, 1, 40, 72)])
def test_whole_projection_norm_and_value_norm(hq, hkv, dk, dv, device="cpu", dtype=torch.float32, tol=1e-5):
    """Queries and keys normed over all heads of a token at once with a weight per channel, a factor per query head, values
    divided by their per-head root mean square, pages written through the slot mapping; then queries only."""
    torch.manual_seed(hq * dk)
    T, bs, eps = 7, 16, 1e-5
    n = hq * dk + hkv * dk + hkv * dv
    qkv = torch.randn(T, n + 5)[:, 5:] * 2.0
    q_w, k_w, hs = torch.randn(hq * dk), torch.randn(hkv * dk), torch.rand(hq) + 0.5
    kc, vc = torch.zeros(4, hkv, bs, dk, dtype=dtype), torch.zeros(4, hkv, bs, dv, dtype=dtype)
    slots = torch.tensor([bs + 3, bs + 4, 2 * bs + 15, 3 * bs, -1, 3 * bs + 1, bs + 5], dtype=torch.int32)
    pos = torch.arange(T, dtype=torch.int32)
    d = lambda t: t.to(device)
    kc, vc = d(kc), d(vc)
    q = ops.qknorm_kv_write(d(qkv), hq, hkv, dk, dv, d(q_w), d(k_w), eps, 0.0, 1, d(pos), d(slots), kc, vc, out_dtype=dtype,
                            norm_whole=True, v_norm=True, q_head_scale=d(hs))
    x = qkv.double().numpy()
    wq = oracle.rms_div(x[:, :hq * dk], eps) * q_w.double().numpy()
    wq = (wq.reshape(T, hq, dk) * hs.double().numpy()[None, :, None]).reshape(T, hq * dk)
    wk = (oracle.rms_div(x[:, hq * dk:(hq + hkv) * dk], eps) * k_w.double().numpy()).reshape(T, hkv, dk)
    wv = oracle.rms_div(x[:, (hq + hkv) * dk:].reshape(T, hkv, dv), eps)
    close(q, wq, tol)
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            close(kc[s // bs, :, s % bs], wk[t], tol)
            close(vc[s // bs, :, s % bs], wv[t], tol)
    assert float(kc[0].abs().sum()) == 0.0 and float(vc[0].abs().sum()) == 0.0
    q2 = ops.qknorm_kv_write(d(qkv[:, :hq * dk]), hq, 0, dk, dv, d(q_w), None, eps, 0.0, 1, d(pos), d(slots), None, None,
                             out_dtype=dtype, norm_whole=True, v_norm=True, q_head_scale=d(hs))
    close(q2, wq, tol)


def _paged(seq, bs, pages, dtype, device):
    """[L, heads, d] of one sequence -> a cache plane [1 + pages, heads, bs, d] holding it in pages pages .. 1 (reversed)."""
    L, h, dd = seq.shape
    plane = torch.zeros(1 + pages, h, bs, dd, dtype=dtype)
    table = list(range(pages, 0, -1))
    for p in range(L):
        plane[table[p // bs], :, p % bs] = seq[p].to(dtype)
    return plane.to(device), table


@pytest.mark.parametrize("window", [1, 2, 16, 17, 33, 100, None])
def test_window_edge_decides(window, device="cpu", dtype=torch.float32, tol=1e-4, D=8, Dv=6, bs=16, L=70, H=4, G=2):
    """One key just inside and one just outside the window are made to win the softmax (scaled so that either would take
    nearly all the weight): the result is right only if exactly the keys with 0 <= i - j < window are seen.  Keys sit on
    both sides of page borders; queries are a prompt, a portion over prior context, and single decoded tokens."""
    torch.manual_seed(5)
    factor, pages = 0.9 * 8 / D, -(-L // bs)
    q, k, v = torch.randn(L, H, D), torch.randn(L, G, D), torch.randn(L, G, Dv)
    w = window or L
    for i in range(L):                       # key i - w + 1 (inside) and key i - w (outside) both match query i strongly
        for j in (i - w + 1, i - w):
            if 0 <= j < i:
                k[j] += 3.0 * q[i].view(G, H // G, D).mean(1)
    q, k, v = (x.to(dtype).float() for x in (q, k, v))      # what a 16-bit run is given, exactly
    slopes = torch.tensor(oracle.head_slopes(H), dtype=torch.float32)
    gate = torch.randn(L, H)
    want = oracle.window_softmax(q.double().numpy(), k.double().numpy(), v.double().numpy(), np.full(H, factor), slopes.double().numpy(),
                                 window)
    want = (want * oracle.sigmoid(gate.double().numpy())[:, :, None]).reshape(L, H * Dv)
    kc, table = _paged(k, bs, pages, dtype, device)
    vc, _ = _paged(v, bs, pages, dtype, device)
    for cuts in ([L], [33, L - 33], [L - 20] + [1] * 20, [15, 2, 2, 30, 1, L - 50]):
        at, rows = 0, []
        for n in cuts:
            batch = BatchInput.build([[0] * n], [at], [table], bs, device, state_slots=[0])
            rows.append(ops.attention_bias(q[at:at + n].reshape(n, H * D).to(dtype).to(device), kc, vc, batch, H, G, D, Dv, factor, None,
                                           gate=gate[at:at + n].to(device), out_dtype=dtype, window=window or 0, slopes=slopes.to(device)))
            at += n
        close(torch.cat(rows), want, tol)
    if window is not None and window < L:    # the test is sharp: one key more, or one less, is far outside any tolerance used
        for off in (-1, 1):
            if window + off >= 1:
                other = oracle.window_softmax(q.double().numpy(), k.double().numpy(), v.double().numpy(), np.full(H, factor),
                                              slopes.double().numpy(), window + off)
                other = (other * oracle.sigmoid(gate.double().numpy())[:, :, None]).reshape(L, H * Dv)
                assert np.abs(other - want).max() > 0.5 * want.std()


@pytest.mark.parametrize("dk,dv,heads,qk_heads", [(10, 6, 4, 2), (16, 16, 2, 2), (5, 9, 3, 3), (24, 3, 1, 1), (40, 33, 2, 1)])
def test_delta_scan_op(dk, dv, heads, qk_heads, device="cpu", tol=2e-4):
    """Portions of 1, 2 and more rows of two sequences, states carried in slots that held other values before; unit
    vectors, the query scale and the sigmoid of the write strength inside the op."""
    torch.manual_seed(dk + dv)
    n = [60, 31]
    data, want = [], []
    for T in n:
        q, k, v = torch.randn(T, qk_heads, dk), torch.randn(T, qk_heads, dk), torch.randn(T, heads, dv)
        logd, b = -torch.rand(T, heads) * 0.7, torch.randn(T, heads) * 2.0
        data.append((q, k, v, logd, b))
        f = lambda x: x.double().numpy()
        o, _ = oracle.delta_rule(oracle.unit(f(q)) * dk ** -0.5, oracle.unit(f(k)), f(v), np.exp(f(logd)), oracle.sigmoid(f(b)))
        want.append(o.reshape(T, heads * dv))
    state = torch.full((3, heads, dk, dv), 3.0, device=device)
    got, at = [[], []], [0, 0]
    for sizes in ([1, 4], [2, 1], [1, 1], [17, 2], [16, 23], [40, 10]):
        live = [i for i in (0, 1) if sizes[i] > 0 and at[i] < n[i]]
        lens = [min(sizes[i], n[i] - at[i]) for i in live]
        batch = fake_batch(lens, [at[i] for i in live], [2 - i for i in live], device)
        cat = lambda j: torch.cat([data[i][j][at[i]:at[i] + m].flatten(1) for i, m in zip(live, lens)]).to(device)
        o = ops.delta_scan(cat(0), cat(1), cat(2), cat(3), cat(4), batch, state, heads, qk_heads, dk, dv, unit_eps=1e-6,
                           q_scale=dk ** -0.5, beta_sigmoid=True).cpu()
        p = 0
        for i, m in zip(live, lens):
            got[i].append(o[p:p + m])
            at[i] += m
            p += m
    for i in (0, 1):
        assert at[i] == n[i]
        close(torch.cat(got[i]), want[i], tol)


def test_delta_rule_overwrites_what_it_stored(device="cpu"):
    """With decay 1 and write strength 1 a key that comes again replaces its value (the rule's point): reading with that key
    returns the newest value, not the sum a plain linear recurrence would give."""
    dk, dv = 8, 4
    keys = torch.eye(dk)[[0, 1, 0, 2, 0]]
    vals = torch.arange(5 * dv, dtype=torch.float32).view(5, dv)
    batch = fake_batch([5], [0], [0], device)
    state = torch.zeros(1, 1, dk, dv, device=device)
    big = torch.full((5, 1), 30.0)
    o = ops.delta_scan(keys.to(device), keys.to(device), vals.to(device), torch.zeros(5, 1).to(device), big.to(device), batch, state,
                       1, 1, dk, dv, beta_sigmoid=True).cpu()
    close(o, vals, 1e-5)


# ----------------------------------------------------------------------------- the model, whole prompts
def residual_stream(eng, toks):
    """The summed residual streams after every layer for one whole prompt, through the core's own forward."""
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
    want, layers = oracle.forward(toks, cfg, W)
    for i, g in enumerate(residual_stream(eng, toks)):
        close(g, layers[i], tol * (1 + i))
    close(eng.feed([("a", toks, list(range(len(toks))))], ["a"]), want, tol * 2)


# ----------------------------------------------------------------------------- decoding, portions, batches
@pytest.mark.parametrize("name", ["mixed", "edges", "plain"])
def test_decode_token_by_token_and_portions(tmp_path, name, device="cpu", dtype=torch.float32, tol=TOL):
    """Prefill against token-by-token decoding, and portions down to two tokens that cut pages, windows and convolution tails."""
    cfg, W, eng = build(tmp_path, name, device, dtype)
    toks = tokens_for(cfg, 70, 2)
    want = want_logits(toks, cfg, W)
    for sizes in ([1], [2], [3, 1, 2, 7, 1, 1, 16, 5], [15, 1, 1, 17, 2], [33, 31, 1], [64, 1]):
        close(feed_in_portions(eng, "s", toks, sizes), want, tol * 2)


def test_unequal_batches_against_each_alone(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """Portions of some requests beside single tokens of others in one step; every request equals itself alone."""
    cfg, W, eng = build(tmp_path, "mixed", device, dtype)
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
        # r0 and r1 live together; r1 ends, r2 takes its slot and pages while r0 goes on; and so on
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


def steep(t):
    """Attention decided by single keys: a large factor per head, so that a key lost at a window's edge, a page read wrongly
    or a borrowed page of the wrong layer changes the result at once."""
    for k in list(t):
        if k.endswith(".mix.temp"):
            t[k] = (t[k].float() * 6.0).to(t[k].dtype)


def test_steep_attention_over_windows_and_page_borders(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """Windows of 16, 17 and 47 tokens around 16-token pages (CPU) and inside 64-token pages (CUDA), a lender and its borrower
    with different windows; prompts, portions and decoded tokens ask across the edges."""
    cfg = botalorn_config(32, 71, [
        att(heads=2, kv_heads=1, dim=8, vdim=8, conv=2, window=16),
        att(heads=4, kv_heads=4, dim=8, vdim=4, conv=3, window=47),
        att(heads=2, kv_heads=1, dim=8, vdim=8, conv=1, window=17, kv_from=0),
        att(heads=4, kv_heads=4, dim=8, vdim=4, conv=2, window=130, kv_from=1)], streams=2, embed_scale=3.0)
    cfg, W, eng = build(tmp_path, cfg, device, dtype, tweak=steep)
    toks = tokens_for(cfg, 150, 4)
    want = want_logits(toks, cfg, W)
    close(feed_in_portions(eng, "w", toks, [150]), want, tol * 3)
    close(feed_in_portions(eng, "p", toks, [31, 2, 36, 1, 1, 59, 2, 1]), want, tol * 3)
    close(feed_in_portions(eng, "d", toks, [100, 1]), want, tol * 3)
    # the windows decide: one token more in every window moves the logits by a thousand times the 32-bit tolerance
    cfg2 = json.loads(json.dumps(cfg))
    for L in cfg2["layers"]:
        L["mixer"]["mask"]["size"] += 1
    assert np.abs(want_logits(toks, cfg2, W) - want).max() > 0.3 * want.std()


def test_first_tokens(tmp_path, device="cpu", dtype=torch.float32, tol=TOL):
    """One-token and two-token requests, and the first tokens one by one: the zeros before the start in the token shift and
    the convolutions, the zero states, position 0 -- in slots and pages that another request has just left."""
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
                           capture_output=True, text=True, timeout=300, cwd=str(ROOT),
                           env={**__import__("os").environ, "CUDA_VISIBLE_DEVICES": ""})
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
    import os

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
    close(read(2), np.concatenate([wb[[7, 8]], wa[[20]]]), TOL * 2)


def test_unknown_kinds_and_bad_lenders_are_refused():
    from llmss_b200.models.botalorn import botalorn_spec

    cfg = json.loads(json.dumps(CONFIGS["attention"]))
    cfg["layers"][0]["type"] = "other"
    with pytest.raises(ValueError):
        botalorn_spec(cfg)
    cfg = json.loads(json.dumps(CONFIGS["dense"]))
    cfg["layers"][0]["mlp"]["kind"] = "other"
    with pytest.raises(ValueError):
        botalorn_spec(cfg)
    cfg = json.loads(json.dumps(CONFIGS["shared"]))
    cfg["layers"][1]["mixer"]["kv_from"] = 1          # itself
    with pytest.raises(ValueError):
        botalorn_spec(cfg)
    cfg = json.loads(json.dumps(CONFIGS["mixed"]))
    cfg["layers"][4]["mixer"]["kv_from"] = 0          # a delta layer has no pages
    with pytest.raises(ValueError):
        botalorn_spec(cfg)
