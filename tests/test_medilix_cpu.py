"""Medilix on the CPU: the engine's host logic (configuration, loading, cache layers of pages with kept
first tokens and of several states, state slots, batching, scheduling, the looped run order) and the
parts' wiring, with the torch statements of the kernels in place of the kernel table, against
tests/plain_medilix.py."""

import json

import pytest

import medilix_cases as mc
from emulated_ops import TorchOps

OPS, DEV = TorchOps(), "cpu"


def test_config_round_trip_run_order_and_sizes_from_tensor_shapes(tmp_path):
    import dataclasses

    from qwen3_runtime_b200.config import MedilixConfig, load_config, resolve_architecture
    from qwen3_runtime_b200.config.model_config import ConfigError
    from qwen3_runtime_b200.weights.loader import SafetensorsDir

    cfg = mc.CONFIGS["A"]["config"]
    raw = json.loads(json.dumps(cfg.to_hf_config()))
    assert resolve_architecture(raw).config_class is MedilixConfig
    folder = mc.make_dir(tmp_path, "A")
    _arch, read = load_config(folder)
    stored = json.loads((folder / "config.json").read_text())
    for layer in stored["layers"]:
        layer["mixer"].pop("decay_rank", None)  # a file as other tools write it does not say
    assert MedilixConfig.from_hf_config(stored) != cfg
    assert MedilixConfig.from_hf_config(stored).with_tensor_shapes(SafetensorsDir(folder).shape) == cfg
    assert read.with_tensor_shapes(SafetensorsDir(folder).shape) == cfg
    starts = [(i, s) for i, s in cfg.run_order()]
    assert starts == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert mc.CONFIGS["C"]["config"].run_order() == [(0, True), (1, False), (2, False)] * 2
    assert mc.CONFIGS["B"]["config"].run_order() == [(i, False) for i in range(4)]
    assert mc.CONFIGS["D"]["config"].run_order() == [(0, False), (1, True), (2, False)]
    assert dataclasses.replace(cfg, loop_times=0).run_order() == [(i, False) for i in range(4)]
    for key, value, match in ((("layers", 0, "type"), "something_else", "unknown layer type"),
                              (("loop", "stop"), 9, "loop"), (("layers", 0, "mlp", "kind"), "other", "feed-forward"),
                              (("norm", "groups"), 5, "norm.groups"),
                              (("layers", 1, "mlp", "router", "groups", "count"), 3, "equal groups"),
                              (("layers", 1, "mixer", "kv_heads"), 4, "multiple of kv_heads")):
        bad = json.loads(json.dumps(raw))
        at = bad
        for k in key[:-1]:
            at = at[k]
        at[key[-1]] = value
        with pytest.raises(ConfigError, match=match):
            MedilixConfig.from_hf_config(bad)


def test_cache_layers(tmp_path):
    """A pass of the loop has cache layers of its own; a window with kept first tokens is a paged group of its
    own kind; the memories, their running maxima, the previous rows and the previous token are state layers."""
    rt = mc.runtime(mc.make_dir(tmp_path, "A"), "A", "float32", OPS, DEV, pages=16)
    kinds = sorted((g.kind, g.window or 0) for g in rt.cache.groups)
    assert ("window", 20) in kinds and ("full", 0) in kinds
    memory, maximum = rt.storage.view(0)
    assert tuple(memory.state.shape[1:]) == (3, 20, 37) and tuple(maximum.state.shape[1:]) == (3,)
    pages = rt.storage.view(1)
    assert pages.k_pages.shape[-1] == 24 and pages.v_pages.shape[-1] == 40 and pages.window == 20
    assert rt.storage.view(3).k_pages.data_ptr() != pages.k_pages.data_ptr()  # the second pass's own pages
    memory, previous = rt.storage.view(2)
    assert tuple(memory.state.shape[1:]) == (3, 24, 24) and tuple(previous.state.shape[1:]) == (72,)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_schedules(tmp_path, name):
    mc.case_schedules(tmp_path, name, "float32", OPS, DEV)


def test_schedules_with_bfloat16_activations(tmp_path):
    mc.case_schedules(tmp_path, "C", "bfloat16", OPS, DEV, lengths=(40, 2, 21))


@pytest.mark.parametrize("name", ["A", "C"])
def test_residual_after_every_run(tmp_path, name):
    mc.case_residual_after_every_run(tmp_path, name, OPS, DEV)


def test_long_decode(tmp_path):
    mc.case_long_decode(tmp_path, "A", "float32", OPS, DEV, total=90)


@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens(tmp_path, name):
    mc.case_first_tokens(tmp_path, name, "float32", OPS, DEV)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_under_the_scheduler(tmp_path, name):
    mc.case_greedy_generation(tmp_path, name, "float32", OPS, DEV)


def test_mixers_alone():
    mc.case_mixer_alone("float32", OPS, DEV, "mlstm")
    mc.case_mixer_alone("float32", OPS, DEV, "mlstm", heads=1, dim=40, vdim=8, gate_cap=2.0)
    mc.case_mixer_alone("float32", OPS, DEV, "wkv")
    mc.case_mixer_alone("float32", OPS, DEV, "wkv", heads=1, dim=40, rank=3)
    mc.case_mixer_alone("float32", OPS, DEV, "attention")
    mc.case_mixer_alone("float32", OPS, DEV, "attention", page_size=4, heads=2, kv_heads=2, dim=16, vdim=8, mask=None)
    mc.case_mixer_alone("float32", OPS, DEV, "attention", heads=4, kv_heads=1, dim=8, vdim=24,
                        mask=dict(size=5, keep_first=11))


def test_memories():
    mc.case_stabilised_memory("float32", OPS, DEV)
    mc.case_bonus_memory("float32", OPS, DEV)
    mc.case_memories_remember_a_far_token("float32", OPS, DEV)


def test_attention_edges():
    mc.case_attention_edges("float32", OPS, DEV)
    mc.case_attention_edges("float32", OPS, DEV, window=8, keep=1, page_size=8, heads=1, kv_heads=1, D=20, Dv=8)


def test_token_state_and_norm():
    mc.case_token_state("float32", OPS, DEV)
    mc.case_token_state("float32", OPS, DEV, buckets=1, mul_prev=0, mul_cur=1)
    mc.case_grouped_norm("float32", OPS, DEV)


def test_routing_and_feed_forwards():
    mc.case_routing("float32", OPS, DEV)
    mc.case_feed_forwards_alone("float32", OPS, DEV)
    mc.case_feed_forwards_alone("float32", OPS, DEV, experts=3, identity=0, top=1, groups=None)
    mc.case_feed_forwards_alone("float32", OPS, DEV, experts=2, identity=4, top=6, groups=(3, 3))


def test_model_less_entry():
    """``LLM(model=None, architecture="Medilix")`` builds the design's tiny configuration."""
    from qwen3_runtime_b200 import LLM

    llm = LLM(None, architecture="Medilix", dtype="float32", device=DEV, ops=OPS, cuda_graph=False)
    out = llm.generate([[1, 2, 3], [4, 5]], max_tokens=5)
    assert [len(o) for o in out] == [5, 5]
