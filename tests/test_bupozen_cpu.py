"""CPU: the Bupozen worker's host path (registry, config, weight fusions, batch metadata, block and row reuse, the scheduler
loop) with the CUDA kernels replaced by the stand-ins of tests/cpu_shim.py, against oracle/bupozen.py."""
import json
import os

import pytest
import torch

import bupozen_cases as C
from cpu_shim import product_on_cpu
from oracle import bupozen as O


def _make(cfg, tensors, eng):
    import swiftllm_b200
    from swiftllm_b200.worker.weight import dict_getter
    ec = swiftllm_b200.EngineConfig(model_path="", use_dummy=False, block_size=eng["block_size"], gpu_mem_utilization=0.9,
                                    num_cpu_blocks=0, max_seqs_in_block_table=eng["rows"], max_blocks_per_seq=eng["num_blocks"],
                                    max_batch_size=4, max_tokens_in_batch=256, dtype=eng["dtype"])
    m = swiftllm_b200.create_model(ec, swiftllm_b200.registry.model_config_from_dict(cfg))
    m.load_weights(dict_getter(tensors))
    m.init_kvcache_and_swap(eng["num_blocks"])
    return m


@pytest.fixture()
def cpu():
    with product_on_cpu():
        yield _make


def test_registry_picks_the_worker_from_the_config():
    import swiftllm_b200
    from swiftllm_b200 import registry
    cfg = C.full_config()
    mc = registry.model_config_from_dict(cfg)
    assert isinstance(mc, swiftllm_b200.BupozenModelConfig) and registry.model_class_for(mc) is swiftllm_b200.BupozenModel
    llama = dict(model_type="llama", num_hidden_layers=1, num_attention_heads=2, hidden_size=16, vocab_size=8,
                 max_position_embeddings=16, intermediate_size=8, rms_norm_eps=1e-5, hidden_act="silu")
    assert registry.model_class_for(registry.model_config_from_dict(llama)) is swiftllm_b200.LlamaModel
    with pytest.raises(ValueError):
        registry.family_of({"model_type": "something else"})


def test_config_geometry():
    import swiftllm_b200
    mc = swiftllm_b200.BupozenModelConfig(C.full_config())
    # layers 0 and 4 share a row width (24 + 6), layer 2 has its own (72 + 4); borrowers point at their source's slot
    assert mc.cache_slots_per_width == {30: 2, 76: 1}
    assert mc.cache_slot[1] == mc.cache_slot[0] and mc.cache_slot[3] == mc.cache_slot[2] and mc.cache_slot[4] == (30, 1)
    assert mc.get_kvslot_size(torch.bfloat16) == (2 * 30 + 76) * 2
    assert mc.mixers[0].rot_dims == 4 and mc.mixers[0].window == 7 and mc.ffs[2] is None and mc.ffs[3].top == 1
    bad = C.config([(C.mixer(), C.DENSE), (C.mixer(kv_rank=32, kv_from=0), C.DENSE)])
    with pytest.raises(AssertionError):
        swiftllm_b200.BupozenModelConfig(bad)


def test_checkpoint_folder_roundtrip(tmp_path, cpu):
    """config.json + model.safetensors on disk -> create_model(engine_config) -> same logits as from the tensors in memory."""
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
    toks = C.tokens_for(cfg, 9, 9)
    assert C.rel_err(C.run_portions(m, toks, 1, [4, 5]), O.forward(cfg, t, toks)) < C.TOL


@pytest.mark.parametrize("name", sorted(C.SINGLE))
def test_single_mechanisms(cpu, name):
    C.case_whole_prompt(cpu, C.SINGLE[name], n=17)


def test_whole_prompt(cpu):
    C.case_whole_prompt(cpu, C.full_config())


def test_prefill_vs_decode(cpu):
    C.case_prefill_vs_decode(cpu, C.full_config())


def test_portions(cpu):
    C.case_portions(cpu, C.full_config())


def test_mixed_batch(cpu):
    C.case_mixed_batch(cpu, C.full_config())


def test_blocks_and_rows_reused(cpu):
    C.case_blocks_and_rows_reused(cpu, C.full_config())


def test_long_decode(cpu):
    C.case_long_decode(cpu, C.config([(C.mixer(window=9), C.DENSE), (C.mixer(window=4, kv_from=0), C.moe())]))


def test_greedy_generation(cpu):
    C.case_greedy_generation(cpu, C.config([(C.mixer(), C.DENSE), (C.mixer(window=5, kv_from=0), C.moe())]))


def test_partial_library_reports_missing_kernels_loudly():
    """A library built for one family (build(only=Worker.NATIVE_SOURCES)) binds a raising stand-in for every symbol it lacks."""
    import swiftllm_b200
    from swiftllm_b200 import _lib, build
    assert set(swiftllm_b200.BupozenModel.NATIVE_SOURCES) <= set(build.sources())
    assert swiftllm_b200.LlamaModel.NATIVE_SOURCES is None and "float32" in swiftllm_b200.BupozenModel.DTYPES \
        and "float32" not in swiftllm_b200.LlamaModel.DTYPES
    with pytest.raises(_lib.NativeLibraryError):
        _lib._missing_symbol("sllm_paged_attention")(1, 2, 3)
    with pytest.raises(AssertionError):
        build.build(only=["no_such_file.cu"])
