"""CPU: the Naforax worker's host path (registry, config, weight fusions and the reordering of query rows, runs of a repeated layer
range with their own cache slots and state tensors, batch metadata and segments, block / row / state reuse, the scheduler loop)
with the CUDA kernels replaced by the stand-ins of tests/cpu_shim.py, against oracle/naforax.py."""
import json
import os

import pytest
import torch

import bupozen_cases as B
import naforax_cases as C
from cpu_shim import product_on_cpu
from oracle import naforax as O
from test_bupozen_cpu import _make


@pytest.fixture()
def cpu():
    with product_on_cpu():
        yield _make


def test_registry_picks_the_worker_from_the_config():
    import swiftllm_b200
    from swiftllm_b200 import registry
    mc = registry.model_config_from_dict(C.full_config())
    assert isinstance(mc, swiftllm_b200.NaforaxModelConfig) and registry.model_class_for(mc) is swiftllm_b200.NaforaxModel
    assert {"sandwich_ops.cu", "scan_ops.cu", "window_attn.cu"} <= set(swiftllm_b200.NaforaxModel.NATIVE_SOURCES)
    assert "float32" in swiftllm_b200.NaforaxModel.DTYPES


def test_config_geometry_and_constants():
    import swiftllm_b200
    from swiftllm_b200.model_config import MinGruSpec, SelectiveScanSpec, WindowAttentionSpec
    mc = swiftllm_b200.NaforaxModelConfig(C.full_config())
    # layers 1 .. 3 run three times: 1 + 3 * 3 + 3 runs; every attention RUN owns cache rows [both maps' keys | values]
    assert mc.runs == [(0, 0)] + [(i, t) for t in range(3) for i in (1, 2, 3)] + [(4, 0), (5, 0), (6, 0)]
    assert mc.cache_slots_per_width == {2 * (2 * 10 + 6): 1, 4 * (2 * 8 + 12): 3, 1 * (2 * 6 + 20): 1}
    assert mc.cache_slot[0] == (52, 0) and mc.cache_slot[1] is None and [mc.cache_slot[r] for r in (2, 5, 8)] == [(112, 0), (112, 1), (112, 2)]
    assert mc.get_kvslot_size(torch.bfloat16) == (52 + 3 * 112 + 32) * 2
    a = mc.mixers[0]
    assert isinstance(a, WindowAttentionSpec) and a.maps == 2 and a.chunk == 7 and a.window == 0 and not a.sink and a.gate
    assert a.qk_weight_norm and a.bias and a.diff == 0.35 and not a.pair_halves and mc.mixers[4].rot_dims == 0
    assert isinstance(mc.mixers[1], MinGruSpec) and isinstance(mc.mixers[3], SelectiveScanSpec) and mc.mixers[5].conv == 1
    assert mc.ffs[0].activation == "gelu_glu" and mc.ffs[1].routing == "softmax_top" and mc.ffs[1].shared_gated
    assert mc.ffs[3].shared_ff == 0 and not mc.ffs[3].shared_gated and mc.ffs[3].top == 1 and mc.ffs[2] is None and mc.ffs[6] is None
    assert mc.norm_groups == 3 and mc.residual_mult == 0.6 and mc.canon_taps == 3 and mc.logit_softcap == 6.0 and mc.loop == (1, 4, 3)
    # state per sequence: input-convolution tails (fp32, two per run with a feed-forward, else one), recurrences, scans
    tails = 4 * 2 * 48 * (2 + 3 * (2 + 1 + 2) + 2 + 2 + 1)
    rec = 3 * 4 * 20 + 4 * 33
    scan = 3 * (4 * 18 * 5 + 2 * 3 * 18) + 4 * 7 * 40
    assert mc.get_state_size(torch.bfloat16) == tails + rec + scan
    plain = swiftllm_b200.NaforaxModelConfig(C.SINGLE["mamba_dense"])
    assert plain.loop is None and plain.runs == [(0, 0)] and plain.cache_slots_per_width == {}
    with pytest.raises(AssertionError):
        swiftllm_b200.NaforaxModelConfig(C.config([(C.mingru(), None)], width=50, groups=3))
    with pytest.raises(AssertionError):
        swiftllm_b200.NaforaxModelConfig(C.config([(C.mingru(), None)], loop=(0, 2, 2)))


def test_query_rows_are_grouped_by_key_head_and_map(cpu):
    """in_proj's query part is [key/value head][map][head of the group]; the bias moves with the rows."""
    cfg = C.config([(C.attn(heads=6, kv_heads=2, dim=4, vdim=3, dims=2), None)])
    t = O.random_tensors(cfg, seed=3, dtype=torch.float32)
    m = B.make_worker(cpu, cfg, t)
    w = m.weight.layers[0]
    q = t["l0.mix.q"].view(2, 3, 2, 4, 48)                  # [g, hh, map, dk, W]
    assert torch.equal(w.in_proj[:48].view(2, 2, 3, 4, 48), q.permute(0, 2, 1, 3, 4))
    assert torch.equal(w.in_bias[:48].view(2, 2, 3, 4), t["l0.mix.q.b"].view(2, 3, 2, 4).permute(0, 2, 1, 3))
    assert w.lam == pytest.approx(O.differential_factor(O.sub(t, "l0.mix."), 0.35), rel=1e-6)


def test_checkpoint_folder_roundtrip(tmp_path, cpu):
    import swiftllm_b200
    from safetensors.torch import save_file
    cfg = C.SINGLE["loop_everything_twice"]
    t = O.random_tensors(cfg, seed=9)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in t.items()}, os.path.join(tmp_path, "model.safetensors"))
    ec = swiftllm_b200.EngineConfig(model_path=str(tmp_path), use_dummy=False, block_size=4, gpu_mem_utilization=0.9, num_cpu_blocks=0,
                                    max_seqs_in_block_table=2, max_blocks_per_seq=8, max_batch_size=2, max_tokens_in_batch=64,
                                    dtype="float32")
    m = swiftllm_b200.create_model(ec)
    m.load_weights()
    m.init_kvcache_and_swap(8)
    toks = B.tokens_for(cfg, 9, 9)
    assert B.rel_err(B.run_portions(m, toks, 1, [4, 5]), O.forward(cfg, t, toks)) < B.TOL


@pytest.mark.parametrize("name", sorted(C.SINGLE))
def test_single_mechanisms(cpu, name):
    B.case_whole_prompt(cpu, C.SINGLE[name], n=17)


def test_whole_prompt(cpu):
    B.case_whole_prompt(cpu, C.full_config())


def test_prefill_vs_decode(cpu):
    B.case_prefill_vs_decode(cpu, C.full_config())


def test_portions(cpu):
    B.case_portions(cpu, C.full_config())


def test_mixed_batch(cpu):
    B.case_mixed_batch(cpu, C.full_config())


def test_blocks_and_rows_reused(cpu):
    B.case_blocks_and_rows_reused(cpu, C.full_config())


def test_state_rows_used_again(cpu):
    C.case_state_rows_used_again(cpu)


def test_long_decode(cpu):
    B.case_long_decode(cpu, C.config([(C.attn(chunk=11), C.dense()), (C.mingru(), None), (C.mamba(), C.moe())], loop=(0, 2, 2)), n=45)


def test_greedy_generation(cpu):
    B.case_greedy_generation(cpu, C.config([(C.mingru(), C.moe()), (C.attn(), C.dense()), (C.mamba(), None)], loop=(0, 2, 2)))


def test_convolutions_across_short_portions(cpu):
    C.case_convolutions_across_short_portions(cpu)


def test_router_scores_are_not_renormalised(cpu):
    C.case_router_scores_are_not_renormalised(cpu)


def test_lambda_and_head_norm(cpu):
    C.case_lambda_and_head_norm(cpu)


def test_first_tokens_and_block_borders(cpu):
    C.case_first_tokens_and_block_borders(cpu)


def test_chunk_edges(cpu):
    C.case_chunk_edges(cpu)


def test_far_key(cpu):
    C.case_far_key(cpu)


def test_slow_recurrences_remember(cpu):
    C.case_slow_recurrences_remember(cpu)


def test_passes_keep_their_own_state(cpu):
    C.case_passes_keep_their_own_state(cpu)
