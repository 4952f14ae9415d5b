"""Zenorax on CUDA: rotation by a frequency table, the sandwich norm with depth-weighted averaging, the sigmoid router, the
attention sink, the gated-recurrence inputs, and the model through the engine, against the plain float64 oracle.

float32 runs everything in true 32-bit (tight tolerance); bfloat16 is what serving uses (tolerance of 16-bit rounding).
"""
import pytest
import torch

import test_zenorax_cpu as cases
from llmss_b200.utils.checkpoint import zenorax_config

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
MODES = [pytest.param(F32, 3e-4, id="f32"), pytest.param(BF16, 8e-2, id="bf16")]

# sizes the kernels tile differently: a latent row of 48 + 16 = 64 numbers (the tensor-core multi-query kernels in 16-bit) and
# one of 104 (the generic kernel), key sizes over one and several register strips of the recurrence, many query heads per
# key/value head, a width that takes the vector forms and fits the tensor-core GEMM's 16-byte rules
cases.CONFIGS["wide"] = zenorax_config(128, 211, [
    cases.lat(heads=8, dim=24, rot_dim=16, vdim=24, kv_rank=48, q_rank=40, mlp=dict(experts=8, top=2, groups=4, keep=2, ff=64)),
    cases.att(heads=12, kv_heads=1, dim=40, rot_dims=24, mlp=dict(experts=16, top=4, groups=4, keep=2, ff=32)),
    cases.rec(heads=2, dim=136, vdim=24),
    cases.lat(heads=3, dim=16, rot_dim=8, vdim=40, kv_rank=96, q_rank=64),
    cases.att(heads=4, kv_heads=2, dim=128, mlp=dict(experts=4, top=2, groups=2, keep=1, ff=128)),
    cases.rec(heads=4, dim=64, vdim=32, mlp=dict(experts=8, top=8, groups=1, keep=1, ff=16))], taps=4, embed_scale=11.0)


def spread_router(t):
    """16-bit runs: choice scores far apart, so that rounding does not flip a choice (a flip moves a position by a whole
    expert's output and, through the recurrent states, every later one).  Sigmoid scores saturate, so larger router
    logits would bring them closer; instead the logits shrink and the corrections are spaced widely, in a shuffled order."""
    for k in list(t):
        if k.endswith(".mlp.router"):
            t[k] = (t[k].float() * 0.3).to(t[k].dtype)
        if k.endswith(".mlp.correction"):
            n = t[k].numel()
            order = torch.randperm(n, generator=torch.Generator().manual_seed(n))
            t[k] = (0.5 * order.float() - 0.25 * n).to(t[k].dtype)


def test_loaded_library_is_the_in_tree_one():
    from llmss_b200.ops import _lib

    _lib.load()
    assert _lib.LOADED_FROM.endswith("llmss_b200/_C/libllmss_b200.so")


@pytest.mark.parametrize("hq,hkv,d,dims,inter", [(4, 2, 12, 8, False), (1, 1, 20, 20, False), (6, 6, 8, 2, True), (12, 3, 40, 24, False),
                                                 (2, 1, 64, 64, True), (32, 8, 128, 128, False), (9, 9, 300, 100, False), (80, 16, 128, 64, True),
                                                 (5, 5, 33, 6, False)])
def test_rotation_and_pages(hq, hkv, d, dims, inter):
    cases.test_rotation_unit_norm_and_pages(hq, hkv, d, dims, inter, "cuda", F32, 1e-5)
    cases.test_rotation_unit_norm_and_pages(hq, hkv, d, dims, inter, "cuda", BF16, 2e-2)


@pytest.mark.parametrize("H,G,D", [(4, 2, 8), (1, 1, 20), (6, 1, 40), (3, 3, 5), (8, 2, 64), (16, 2, 128)])
def test_sink_and_far_keys(H, G, D):
    cases.test_sink_and_far_keys(H, G, D, "cuda", F32, 1e-4, bs=64)
    cases.test_sink_and_far_keys(H, G, D, "cuda", F32, 1e-4, bs=16)
    cases.test_sink_and_far_keys(H, G, D, "cuda", BF16, 5e-2, bs=64)


def test_row_kernels():
    for W, n, taps in [(32, 4, 3), (50, 7, 1), (1024, 3, 4), (7, 2, 2), (2048, 18, 4), (12288, 2, 2), (8196, 1, 2)]:
        cases.test_sandwich_norm_and_depth_average(W, n, taps, "cuda", F32, 1e-5)
        cases.test_sandwich_norm_and_depth_average(W, n, taps, "cuda", BF16, 2e-2)
    cases.test_input_convolution_carries_its_tail("cuda", F32, 1e-5)
    cases.test_input_convolution_carries_its_tail("cuda", BF16, 2e-2)
    cases.test_input_convolution_state_is_kept_between_calls("cuda")
    cases.test_soft_cap("cuda")


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 2, 1), (6, 2, 3, 2), (4, 1, 4, 4), (16, 4, 4, 2), (64, 6, 8, 3), (5, 2, 5, 3), (12, 3, 1, 1),
                                               (256, 8, 8, 4), (160, 6, 40, 7)])
def test_router(E, top, groups, keep):
    cases.test_sigmoid_router_with_correction(E, top, groups, keep, "cuda")


@pytest.mark.parametrize("H,D,Dv", [(3, 10, 6), (1, 24, 3), (2, 64, 32), (2, 5, 40), (4, 128, 128), (2, 136, 24)])
def test_gated_recurrence(H, D, Dv):
    cases.test_gated_recurrence_inputs_and_scan(H, D, Dv, "cuda", 2e-4)


@pytest.mark.parametrize("dtype,tol", MODES)
@pytest.mark.parametrize("name", ["latent", "attention", "hgrn2", "experts", "mixed", "edges", "odd", "wide"])
def test_whole_prompt_and_residual_stream(tmp_path, name, dtype, tol):
    if dtype == BF16:
        cfg, W, eng = cases.build(tmp_path, name, "cuda", dtype, tweak=spread_router)
        toks = cases.tokens_for(cfg, 45, 1)
        want = cases.want_logits(toks, cfg, W)
        got = eng.feed([("a", toks, list(range(len(toks))))], ["a"]).double().cpu()
        d = (got - want).abs().max(-1).values / want.std()
        assert (d < tol).float().mean() >= 0.97 and d.max() < 10 * tol, d
    else:
        cases.test_whole_prompt_and_residual_stream(tmp_path, name, "cuda", dtype, tol)


@pytest.mark.parametrize("name", ["mixed", "edges", "odd", "wide"])
def test_decode_and_portions(tmp_path, name):
    cases.test_decode_token_by_token_and_portions(tmp_path, name, "cuda", F32, 3e-4)


def test_schedules_in_32_bit(tmp_path):
    cases.test_unequal_batches_against_each_alone(tmp_path / "a", "cuda", F32, 3e-4)
    cases.test_pages_and_slots_are_used_again(tmp_path / "b", "cuda", F32, 3e-4)
    cases.test_steep_attention_far_back_and_over_page_borders(tmp_path / "c", "cuda", F32, 3e-4)
    cases.test_first_tokens(tmp_path / "d", "cuda", F32, 3e-4)
    cases.test_long_decoding(tmp_path / "e", "cuda", F32, 3e-4)
    cases.test_model_call_with_a_past(tmp_path / "f", "cuda", F32, 3e-4)


def test_schedules_in_16_bit_agree_with_each_other(tmp_path):
    """bfloat16: portions, single tokens and mixed batches of the same request give the same logits up to rounding (the
    tensor-core latent kernels for portions and decode, the generic ones, the dense and the gathered expert forms)."""
    cfg, W, eng = cases.build(tmp_path, "wide", "cuda", BF16, tweak=spread_router)
    toks = cases.tokens_for(cfg, 150, 3)
    whole = cases.feed_in_portions(eng, "w", toks, [150]).double().cpu()
    want = cases.want_logits(toks, cfg, W)
    d = (whole - want).abs().max(-1).values / want.std()
    assert (d < 8e-2).float().mean() >= 0.95, d
    for sizes in ([100, 1], [31, 2, 36, 1, 1, 59, 2, 1], [64, 64, 1]):
        got = cases.feed_in_portions(eng, "p", toks, sizes).double().cpu()
        d = (got - whole).abs().max(-1).values / want.std()
        assert (d < 8e-2).float().mean() >= 0.95, (sizes, d)


def test_decode_batch_of_unequal_requests_in_16_bit(tmp_path):
    """bfloat16: three requests of different lengths decode together (the tensor-core decode kernels with the sink and over the
    latent rows, several sequences per launch); every request equals itself fed whole."""
    cfg, W, eng = cases.build(tmp_path, "wide", "cuda", BF16, tweak=spread_router)
    reqs = {k: cases.tokens_for(cfg, n, 20 + i) for i, (k, n) in enumerate([("a", 90), ("b", 171), ("c", 40)])}
    whole = {k: cases.feed_in_portions(eng, "w" + k, t, [len(t)]).double().cpu() for k, t in reqs.items()}
    std = max(v.std().item() for v in whole.values())
    tail = 12
    out = eng.feed([(k, t[:-tail], [len(t) - tail - 1]) for k, t in reqs.items()])
    got = {k: [out[i:i + 1]] for i, k in enumerate(reqs)}
    for j in range(tail):
        last = j == tail - 1
        out = eng.feed([(k, [t[len(t) - tail + j]], [0]) for k, t in reqs.items()], list(reqs) if last else [])
        for i, k in enumerate(reqs):
            got[k].append(out[i:i + 1])
    for k, t in reqs.items():
        d = (torch.cat(got[k]).double().cpu() - whole[k][len(t) - tail - 1:]).abs().max(-1).values / std
        assert d.max() < 8e-2, (k, d)


def test_latent_row_of_256_with_sixteen_heads(tmp_path):
    """bfloat16: a latent row of 192 + 64 numbers and 16 heads -- the tensor-core paged kernel for portions, the tensor-core
    decode kernel in two groups of eight heads for single tokens -- against the oracle."""
    cfg = zenorax_config(128, 211, [cases.lat(heads=16, dim=32, rot_dim=64, vdim=16, kv_rank=192, q_rank=64, scale=0.25),
                                    cases.att(heads=8, kv_heads=2, dim=64, scale=0.3)], taps=2, embed_scale=11.0)
    cfg, W, eng = cases.build(tmp_path, cfg, "cuda", BF16)
    toks = cases.tokens_for(cfg, 200, 5)
    want = cases.want_logits(toks, cfg, W)
    for sizes in ([200], [150, 1], [70, 3, 64, 1]):
        got = cases.feed_in_portions(eng, "p", toks, sizes).double().cpu()
        d = (got - want).abs().max(-1).values / want.std()
        assert d.max() < 8e-2, (sizes, d)


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_generation(tmp_path, dtype, graph):
    cases.test_greedy_generation_through_engine_and_cli(tmp_path, "cuda", dtype, graph)


def test_long_prompt_in_portions_against_the_cpu_engine(tmp_path):
    """700 tokens: the two-pass recurrence over chunks, a dozen pages, rotary positions in the hundreds; CUDA in 32-bit against
    the engine on CPU."""
    cfg, _, gpu = cases.build(tmp_path / "g", "wide", "cuda", F32, max_seq_len=1024)
    _, _, cpu = cases.build(tmp_path / "c", "wide", "cpu", F32, max_seq_len=1024)
    toks = cases.tokens_for(cfg, 700, 9)
    want = cpu.feed([("a", toks, [0, 1, 63, 64, 300, 511, 512, 698, 699])], ["a"])
    cases.close(gpu.feed([("a", toks, [0, 1, 63, 64, 300, 511, 512, 698, 699])], ["a"]), want, 3e-4)
    a = gpu.feed([("b", toks[:400], [0, 1, 63, 64, 300])], [])
    b = gpu.feed([("b", toks[400:699], [511 - 400, 512 - 400, 698 - 400])], [])
    c = gpu.feed([("b", toks[699:], [0])], ["b"])
    cases.close(torch.cat([a, b, c]), want, 3e-4)
