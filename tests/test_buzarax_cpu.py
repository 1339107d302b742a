"""CPU: the Buzarax worker's host path (registry, config, weight fusions, batch metadata and segments, block / row / state reuse,
the scheduler loop) with the CUDA kernels replaced by the stand-ins of tests/cpu_shim.py, against oracle/buzarax.py."""
import json
import os

import pytest
import torch

import bupozen_cases as B
import buzarax_cases as C
from cpu_shim import product_on_cpu
from oracle import buzarax as O
from test_bupozen_cpu import _make


@pytest.fixture()
def cpu():
    with product_on_cpu():
        yield _make


def test_registry_picks_the_worker_from_the_config():
    import swiftllm_b200
    from swiftllm_b200 import registry
    mc = registry.model_config_from_dict(C.full_config())
    assert isinstance(mc, swiftllm_b200.BuzaraxModelConfig) and registry.model_class_for(mc) is swiftllm_b200.BuzaraxModel
    assert {"recurrent.cu", "stream_ops.cu", "window_attn.cu"} <= set(swiftllm_b200.BuzaraxModel.NATIVE_SOURCES)
    assert "float32" in swiftllm_b200.BuzaraxModel.DTYPES


def test_config_geometry_and_constants():
    import swiftllm_b200
    from swiftllm_b200.model_config import GatedRecurrenceSpec, ParallelMixerSpec
    mc = swiftllm_b200.BuzaraxModelConfig(C.full_config())
    # only the attention layers own cache rows: widths 2 * (10 + 6), 4 * (8 + 12), 1 * (6 + 20), 3 * (12 + 4)
    assert mc.cache_slots_per_width == {32: 1, 80: 1, 26: 1, 48: 1}
    assert mc.cache_slot[0] is None and mc.cache_slot[1] == (32, 0) and mc.cache_slot[6] == (48, 0)
    assert mc.get_kvslot_size(torch.bfloat16) == (32 + 80 + 26 + 48) * 2
    assert isinstance(mc.mixers[0], GatedRecurrenceSpec) and isinstance(mc.mixers[1], ParallelMixerSpec)
    a = mc.mixers[1].left
    assert a.pair_halves and a.qk_unit_norm and a.value_rotation and not a.gate and a.sink and a.window == 0
    assert a.rot_scaling == (3.0, 40.0, 8.0, 1.0) and a.softcap == 5.0 and a.out_scale == 0.7 and mc.mixers[1].right.out_scale == 1.3
    assert mc.mixers[2].left.rot_scaling is None and mc.mixers[2].left.softcap == 0.0 and mc.mixers[4].left.rot_dims == 0
    assert mc.mixers[5].conv == 1 and mc.mixers[3].blocks == 1 and mc.ffs[2] is None and mc.ffs[4].top == 1
    assert mc.ffs[1].activation == "clamped_glu" and mc.ffs[1].limit == 0.75 and mc.ffs[0].routing == "sigmoid_bias"
    assert mc.pair_hash.buckets == 53 and mc.logit_softcap == 6.0
    # state per sequence: last token + recurrences (fp32 state + tails) + linear-attention states
    rec = 4 * (24 + 20 + 33) + 2 * (3 * 24 + 1 * 20 + 0)
    lin = 4 * (3 * 5 * 7 + 1 * 9 * 4 + 4 * 12 * 3 + 3 * 5 * 7)
    assert mc.get_state_size(torch.bfloat16) == 4 + rec + lin
    with pytest.raises(AssertionError):
        swiftllm_b200.BuzaraxModelConfig(C.config([(C.rglru(width=10, blocks=3), None)]))


def test_stretched_frequencies_match_the_oracle():
    from swiftllm_b200.worker.token_model import rotary_frequencies
    for dims, base, sc in ((6, 100.0, (3.0, 40, 8.0, 1.0)), (12, 10000.0, (8.0, 16, 4.0, 0.5)), (10, 50.0, None), (64, 5e5, (16.0, 512, 32.0, 1.0))):
        rot = {"base": base, "dims": dims}
        if sc:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), sc))
        f, amp = rotary_frequencies(base, dims, tuple(float(x) for x in sc) if sc else None)
        rf, ramp = O.stretched_frequencies(rot)
        assert f == pytest.approx(rf, rel=1e-12) and amp == pytest.approx(ramp)


def test_checkpoint_folder_roundtrip(tmp_path, cpu):
    import swiftllm_b200
    from safetensors.torch import save_file
    cfg = C.SINGLE["parallel_top1"]
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


def test_greedy_generation(cpu):
    B.case_greedy_generation(cpu, C.config([(C.rglru(), C.moe()), (C.parallel(), C.dense())]))


def test_convolution_across_short_portions(cpu):
    C.case_convolution_across_short_portions(cpu)


def test_correction_changes_the_choice_only(cpu):
    C.case_correction_changes_the_choice_only(cpu)


def test_sink(cpu):
    C.case_sink(cpu)


def test_score_cap_binds(cpu):
    C.case_score_cap_binds(cpu)


def test_first_tokens_and_block_borders(cpu):
    C.case_first_tokens_and_block_borders(cpu)


def test_far_key(cpu):
    C.case_far_key(cpu)


def test_slow_recurrence_remembers(cpu):
    C.case_slow_recurrence_remembers(cpu)
