"""CPU: the Rivudra worker's host path (registry, config, weight fusions, batch metadata, block and row reuse, the scheduler
loop) with the CUDA kernels replaced by the stand-ins of tests/cpu_shim.py, against oracle/rivudra.py."""
import json
import os

import pytest
import torch

import bupozen_cases as B
import rivudra_cases as C
from cpu_shim import product_on_cpu
from oracle import rivudra as O
from test_bupozen_cpu import _make


@pytest.fixture()
def cpu():
    with product_on_cpu():
        yield _make


def test_registry_picks_the_worker_from_the_config():
    import swiftllm_b200
    from swiftllm_b200 import registry
    mc = registry.model_config_from_dict(C.full_config())
    assert isinstance(mc, swiftllm_b200.RivudraModelConfig) and registry.model_class_for(mc) is swiftllm_b200.RivudraModel
    assert "window_attn.cu" in swiftllm_b200.RivudraModel.NATIVE_SOURCES and "float32" in swiftllm_b200.RivudraModel.DTYPES


def test_config_geometry_and_constants():
    import swiftllm_b200
    mc = swiftllm_b200.RivudraModelConfig(C.full_config())
    # row width = kv heads * (dim + vdim): layers 0 and 3 share 2 * 17, the others have their own
    assert mc.cache_slots_per_width == {34: 2, 80: 1, 46: 1, 51: 1}
    assert mc.cache_slot[0] == (34, 0) and mc.cache_slot[3] == (34, 1) and mc.cache_slot[2] == (46, 0)
    assert mc.get_kvslot_size(torch.bfloat16) == (2 * 34 + 80 + 46 + 51) * 2
    assert mc.embedding_scale == 0.7 and mc.norm_unit_offset and mc.ffs[2] is None
    f = mc.ffs[1]
    assert (f.experts, f.top, f.groups, f.keep, f.shared_ff, f.limit, f.route_scale) == (8, 3, 2, 1, 0, 0.75, 1.25)
    assert mc.ffs[0].shared_ff == 9 and mc.ffs[0].shared_limit == 1.5 and mc.mixers[3].rot_dims == 0 and mc.mixers[2].window == 13
    with pytest.raises(AssertionError):      # 3 experts cannot come from one kept group of 2
        swiftllm_b200.RivudraModelConfig(C.config([(C.mixer(), C.moe(experts=6, top=3, groups=3, keep=1))]))


def test_checkpoint_folder_roundtrip(tmp_path, cpu):
    import swiftllm_b200
    from safetensors.torch import save_file
    cfg = C.SINGLE["moe"]
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


def test_long_decode(cpu):
    B.case_long_decode(cpu, C.config([(C.mixer(window=9), C.moe()), (C.mixer(window=4, kv_heads=1), None)]))


def test_greedy_generation(cpu):
    B.case_greedy_generation(cpu, C.config([(C.mixer(), C.moe()), (C.mixer(window=5), C.moe(shared=None))]))


def test_window_edges(cpu):
    C.case_window_edges(cpu)


def test_far_key(cpu):
    C.case_far_key(cpu)


def test_sink(cpu):
    C.case_sink(cpu)


def test_group_limit_binds(cpu):
    C.case_group_limit_binds(cpu)
