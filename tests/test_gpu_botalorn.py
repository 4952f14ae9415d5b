"""Botalorn on CUDA: the stream kernels (scaled sinusoidal embedding, hyper-connection write + normed read), the delta-rule
scan, window / slope attention, the general q / k / v preparation, and the model through the engine, against the plain
float64 oracle.

float32 runs everything in true 32-bit (tight tolerance); bfloat16 is what serving uses (tolerance of 16-bit rounding).
"""
import pytest
import torch

import test_botalorn_cpu as cases
from llmss_b200.utils.checkpoint import botalorn_config

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
MODES = [pytest.param(F32, 3e-4, id="f32"), pytest.param(BF16, 8e-2, id="bf16")]

# sizes the kernels tile differently: key sizes over one, two and several register strips of the delta scan, value sizes
# over a warp and over a block, many query heads per key/value head, widths that fit the tensor-core GEMM's 16-byte
# rules and take the vector path of the stream kernel, windows over several 64-token pages
cases.CONFIGS["wide"] = botalorn_config(128, 211, [
    cases.att(heads=12, kv_heads=1, dim=40, vdim=72, conv=4, window=100, mlp={"ff": 256}),
    cases.dlt(heads=4, kv_heads=2, dim=64, vdim=32, conv=4, mlp={"ff": 128}),
    cases.dlt(heads=2, kv_heads=1, dim=136, vdim=24, conv=3),
    cases.att(heads=4, kv_heads=2, dim=128, vdim=64, conv=3, window=70),
    cases.dlt(heads=1, kv_heads=1, dim=48, vdim=136, conv=2),
    cases.att(heads=12, kv_heads=1, dim=40, vdim=72, conv=2, window=65, kv_from=0, mlp={"ff": 256}),
    cases.dlt(heads=8, kv_heads=8, dim=16, vdim=16, conv=4)], streams=4, embed_scale=11.0)


def test_loaded_library_is_the_in_tree_one():
    from llmss_b200.ops import _lib

    _lib.load()
    assert _lib.LOADED_FROM.endswith("llmss_b200/_C/libllmss_b200.so")


def test_stream_kernels():
    for W, S, scale in [(32, 1, 1.0), (50, 3, 12.0), (7, 2, 0.5), (1024, 2, 32.0)]:
        cases.test_embedding_with_sinusoid(W, S, scale, "cuda", F32, 1e-5)
        cases.test_embedding_with_sinusoid(W, S, scale, "cuda", BF16, 1e-5)      # the table is exact in 16 bits, the sum 32-bit
    for S, W in [(1, 24), (2, 32), (3, 50), (5, 7), (8, 36), (11, 20), (16, 64), (2, 2048)]:
        cases.test_hyper_residual_op(S, W, "cuda", F32, 1e-5)
        cases.test_hyper_residual_op(S, W, "cuda", BF16, 2e-2)
    cases.test_token_shift_carries_the_previous_row("cuda")


@pytest.mark.parametrize("hq,hkv,dk,dv", [(4, 2, 10, 6), (1, 1, 20, 4), (6, 6, 8, 8), (12, 1, 40, 72), (32, 8, 128, 128)])
def test_qkv_preparation(hq, hkv, dk, dv):
    cases.test_whole_projection_norm_and_value_norm(hq, hkv, dk, dv, "cuda", F32, 1e-5)
    cases.test_whole_projection_norm_and_value_norm(hq, hkv, dk, dv, "cuda", BF16, 2e-2)


@pytest.mark.parametrize("window", [1, 2, 16, 17, 33, 100, None])
def test_window_edge(window):
    cases.test_window_edge_decides(window, "cuda", F32, 1e-4)
    cases.test_window_edge_decides(window, "cuda", BF16, 5e-2)


@pytest.mark.parametrize("d", [64, 128, 256])
@pytest.mark.parametrize("window", [1, 2, 63, 64, 65, 128, 150, 1000])
def test_window_edge_on_the_tensor_core_kernels(window, d):
    """16-bit pages with key size = value size 64 / 128 / 256: the window and the slopes ride on the tensor-core kernels as a
    distance table whose last column hides the key; the generic kernel on the same pages agrees."""
    from llmss_b200.ops import cuda_impl as cu

    assert cu.attention_bias_uses_tc(BF16, d, d, 64, 1.0)
    n0 = cu._lib.LAUNCHES["count"]
    cases.test_window_edge_decides(window, "cuda", BF16, 8e-2, D=d, Dv=d, bs=64, L=330)
    cu._BIAS_TC = False
    try:
        cases.test_window_edge_decides(window, "cuda", BF16, 8e-2, D=d, Dv=d, bs=64, L=330)
    finally:
        cu._BIAS_TC = True
    assert cu._lib.LAUNCHES["count"] > n0


@pytest.mark.parametrize("H,G", [(2, 2), (8, 1), (6, 3)])
def test_window_edge_on_the_tensor_core_kernels_by_group_size(H, G):
    """One query head per key/value head, and eight: the decode kernel's row packing differs."""
    for window in (64, 150):
        cases.test_window_edge_decides(window, "cuda", BF16, 8e-2, D=128, Dv=128, bs=64, L=330, H=H, G=G)
        cases.test_window_edge_decides(window, "cuda", BF16, 8e-2, D=64, Dv=64, bs=64, L=200, H=H, G=G)


# key size = value size 64 / 128 in 16-bit: attention on the tensor-core kernels, lenders and borrowers with other windows
cases.CONFIGS["tc_sizes"] = botalorn_config(128, 173, [
    cases.att(heads=4, kv_heads=2, dim=64, vdim=64, conv=3, window=50, mlp={"ff": 128}),
    cases.att(heads=2, kv_heads=1, dim=128, vdim=128, conv=2, window=100),
    cases.dlt(heads=2, kv_heads=1, dim=64, vdim=64, conv=4),
    cases.att(heads=4, kv_heads=2, dim=64, vdim=64, conv=2, window=64, kv_from=0),
    cases.att(heads=2, kv_heads=1, dim=128, vdim=128, conv=4, window=7, kv_from=1, mlp={"ff": 128})], streams=2, embed_scale=11.0)


def test_model_on_the_tensor_core_attention(tmp_path):
    cases.test_whole_prompt_and_residual_stream(tmp_path / "a", "tc_sizes", "cuda", BF16, 8e-2)
    cases.test_decode_token_by_token_and_portions(tmp_path / "b", "tc_sizes", "cuda", BF16, 8e-2)
    cases.test_whole_prompt_and_residual_stream(tmp_path / "c", "tc_sizes", "cuda", F32, 3e-4)
    cfg, W, gpu = cases.build(tmp_path / "d", "tc_sizes", "cuda", BF16, max_seq_len=1024)
    toks = cases.tokens_for(cfg, 400, 5)
    cases.close(cases.feed_in_portions(gpu, "p", toks, [250, 1, 1, 140, 1]), cases.want_logits(toks, cfg, W), 0.1)


@pytest.mark.parametrize("dk,dv,heads,qk_heads", [(10, 6, 4, 2), (16, 16, 2, 2), (5, 9, 3, 3), (24, 3, 1, 1), (40, 33, 2, 1),
                                                  (64, 64, 2, 2), (128, 128, 4, 2), (136, 24, 2, 1), (48, 136, 1, 1), (300, 8, 2, 2)])
def test_delta_scan_kernel(dk, dv, heads, qk_heads):
    cases.test_delta_scan_op(dk, dv, heads, qk_heads, "cuda", 2e-4)
    cases.test_delta_rule_overwrites_what_it_stored("cuda")


@pytest.mark.parametrize("dtype,tol", MODES)
@pytest.mark.parametrize("name", ["attention", "delta", "dense", "shared", "mixed", "edges", "plain", "wide"])
def test_model_whole_prompt(tmp_path, dtype, tol, name):
    cases.test_whole_prompt_and_residual_stream(tmp_path, name, "cuda", dtype, tol)


@pytest.mark.parametrize("dtype,tol", MODES)
def test_model_schedules(tmp_path, dtype, tol):
    for name in ("mixed", "edges", "plain", "wide"):
        cases.test_decode_token_by_token_and_portions(tmp_path / name, name, "cuda", dtype, tol)
    cases.test_unequal_batches_against_each_alone(tmp_path / "b", "cuda", dtype, tol)
    cases.test_first_tokens(tmp_path / "c", "cuda", dtype, tol)
    cases.test_long_decoding(tmp_path / "d", "cuda", dtype, tol)


@pytest.mark.parametrize("dtype,tol", MODES)
def test_model_pages_slots_windows(tmp_path, dtype, tol):
    cases.test_pages_and_slots_are_used_again(tmp_path / "a", "cuda", dtype, tol)
    cases.test_steep_attention_over_windows_and_page_borders(tmp_path / "b", "cuda", dtype, tol if dtype == F32 else 0.15)
    cases.test_model_call_with_a_past(tmp_path / "c", "cuda", dtype, tol)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("graph", [False, True])
def test_generation(tmp_path, dtype, graph):
    """Engine.generate with and without CUDA-graph decode steps (padded batch rows are inert: slot -1)."""
    cases.test_greedy_generation_through_engine_and_cli(tmp_path, "cuda", dtype, graph)


def test_cuda_equals_cpu_engine_on_a_replayed_schedule(tmp_path):
    """The same mixed schedule through the CPU ops and through the kernels, true 32-bit."""
    cfg, W, cpu = cases.build(tmp_path / "a", "wide", "cpu", F32)
    _, _, gpu = cases.build(tmp_path / "b", "wide", "cuda", F32)
    reqs = {k: cases.tokens_for(cfg, n, 90 + n) for k, n in (("a", 130), ("b", 70), ("c", 3))}
    plan = [[("a", 65), ("c", 1)], [("a", 1), ("b", 64), ("c", 2)], [("a", 63), ("b", 1)], [("a", 1), ("b", 5)]]
    at = {k: 0 for k in reqs}
    for step in plan:
        entries = []
        for k, n in step:
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
        cases.close(gpu.feed(entries), cpu.feed(entries), 3e-4)


@pytest.mark.parametrize("dtype,tol", [pytest.param(F32, 5e-4, id="f32"), pytest.param(BF16, 0.12, id="bf16")])
def test_long_prompt_in_portions_equals_the_cpu_engine(tmp_path, dtype, tol):
    """700 tokens over a dozen pages, windows that end inside the context, long portions with a single token between them --
    against the same model on the CPU ops fed in one piece."""
    cfg, W, cpu = cases.build(tmp_path / "a", "wide", "cpu", F32, max_seq_len=1024)
    _, _, gpu = cases.build(tmp_path / "b", "wide", "cuda", dtype, max_seq_len=1024)
    toks = cases.tokens_for(cfg, 700, 21)
    want = cases.feed_in_portions(cpu, "w", toks, [700])
    cases.close(cases.feed_in_portions(gpu, "p", toks, [300, 1, 257, 142]), want, tol)
    cases.close(cases.feed_in_portions(gpu, "q", toks, [255, 445]), want, tol)
