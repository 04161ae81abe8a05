"""Tabisun on the CPU: the engine's host logic (configuration, loading, layers that run another layer's
weights on a cache of their own, chunk groups of pages, batching, scheduling) and the parts' wiring, with the
torch statements of the kernels in place of the kernel table, against tests/plain_tabisun.py."""

import json

import pytest

import tabisun_cases as tc
from emulated_ops import TorchOps

OPS, DEV = TorchOps(), "cpu"


def test_config_round_trip_and_refusals(tmp_path):
    from qwen3_runtime_b200.config import TabisunConfig, load_config, resolve_architecture
    from qwen3_runtime_b200.config.model_config import ConfigError

    cfg = tc.CONFIGS["A"]["config"]
    raw = json.loads(json.dumps(cfg.to_hf_config()))
    assert resolve_architecture(raw).config_class is TabisunConfig
    assert TabisunConfig.from_hf_config(raw) == cfg
    _arch, read = load_config(tc.make_dir(tmp_path, "A"))
    assert read == cfg
    for name in ("B", "C", "D"):
        c = tc.CONFIGS[name]["config"]
        assert TabisunConfig.from_hf_config(json.loads(json.dumps(c.to_hf_config()))) == c
    for key, value, match in ((("layers", 0, "type"), "something_else", "unknown layer type"),
                              (("layers", 1, "mlp", "kind"), "other", "feed-forward"),
                              (("layers", 0, "mixer", "kv_heads"), 3, "multiple of kv_heads"),
                              (("layers", 1, "mixer", "vdim"), 8, "values are the keys"),
                              (("layers", 1, "mixer", "rot", "dims"), 26, "even and at most"),
                              (("layers", 3, "weights_of"), 3, "another layer"),
                              (("layers", 3, "weights_of"), 9, "another layer"),
                              (("layers", 3, "weights_of"), 1, "differs from layer"),
                              (("layers", 4, "weights_of"), 3, "differs from layer"),
                              (("norm", "eps"), 0.0, "norm.eps")):
        bad = json.loads(json.dumps(raw))
        at = bad
        for k in key[:-1]:
            at = at[k]
        at[key[-1]] = value
        with pytest.raises(ConfigError, match=match):
            TabisunConfig.from_hf_config(bad)


def test_tensor_names_and_cache_layers(tmp_path):
    """A layer that runs another layer's weights has no tensors and a cache layer of its own; chunked layers
    form a paged group that gives pages back; the latent layers hold one row per token."""
    from qwen3_runtime_b200.weights.random_init import expected_tensors_for

    names = set(expected_tensors_for(tc.CONFIGS["A"]["config"]))
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.lq1", "l1.mix.q.norm", "l2.mix.sink",
            "l2.mix.g", "l2.mix.dkv.norm", "l1.mlp.gate"} <= names
    assert not any(n.startswith(("l3.", "l4.")) for n in names) and "l1.mix.v" not in names and "l2.norm2" not in names
    assert {n for n in expected_tensors_for(tc.CONFIGS["C"]["config"]) if n.startswith("l3.")} >= {"l3.mix.q", "l3.norm2"}
    rt = tc.runtime(tc.make_dir(tmp_path, "A"), "A", "float32", OPS, DEV, pages=16)
    kinds = sorted((g.kind, g.chunk or 0) for g in rt.cache.groups)
    assert kinds == [("chunk", 20), ("full", 0), ("full", 0)]
    first, again = rt.storage.view(0), rt.storage.view(3)
    assert first.k_pages.shape[-1] == 24 and first.v_pages.shape[-1] == 20
    assert first.k_pages.data_ptr() != again.k_pages.data_ptr() and first.group == again.group
    assert rt.storage.view(2).latent_pages.shape[-1] == 56 and rt.storage.view(4).latent_pages is not None
    blocks = rt.runner.model.blocks
    assert len(blocks) == 3 and [r.block for r in rt.runner.model.spec.order] == [0, 1, 2, 0, 2]
    # a layer may name a layer that itself runs another's weights: both run the owner's
    import dataclasses

    cfg = tc.CONFIGS["A"]["config"]
    chained = dataclasses.replace(cfg, layers=(*cfg.layers, dataclasses.replace(cfg.layers[3], weights_of=3)))
    assert chained.owner_of(5) == 0 and chained.owner_of(3) == 0 and chained.owner_of(1) == 1


def test_chunk_pages():
    tc.case_chunk_pages()


def test_frequencies():
    tc.case_frequencies()


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_schedules(tmp_path, name):
    tc.case_schedules(tmp_path, name, "float32", OPS, DEV)


def test_schedules_with_bfloat16_activations(tmp_path):
    tc.case_schedules(tmp_path, "C", "bfloat16", OPS, DEV, lengths=(40, 2, 21))


@pytest.mark.parametrize("name", ["A", "B"])
def test_residual_after_every_run(tmp_path, name):
    tc.case_residual_after_every_run(tmp_path, name, OPS, DEV)


def test_long_decode(tmp_path):
    tc.case_long_decode(tmp_path, "A", "float32", OPS, DEV, total=90)


@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens(tmp_path, name):
    tc.case_first_tokens(tmp_path, name, "float32", OPS, DEV)


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_under_the_scheduler(tmp_path, name):
    tc.case_greedy_generation(tmp_path, name, "float32", OPS, DEV)


def test_mixers_alone():
    tc.case_mixer_alone("float32", OPS, DEV, "attention")
    tc.case_mixer_alone("float32", OPS, DEV, "attention", page_size=4, heads=2, kv_heads=2, dim=16, vdim=16, chunk=None)
    tc.case_mixer_alone("float32", OPS, DEV, "attention", heads=3, kv_heads=1, dim=8, vdim=40, chunk=7, diff=0.9)
    tc.case_mixer_alone("float32", OPS, DEV, "attention_2")
    tc.case_mixer_alone("float32", OPS, DEV, "attention_2", page_size=4, heads=2, kv_heads=2, dim=20, softcap=None,
                        rot=None)
    tc.case_mixer_alone("float32", OPS, DEV, "latent_attention")
    tc.case_mixer_alone("float32", OPS, DEV, "latent_attention", heads=1, dim=8, rot_dim=4, vdim=8, kv_rank=16,
                        rot=tc.RotaryConfig(dims=4, base=100.0))


def test_attention_edges():
    tc.case_differential_edges("float32", OPS, DEV)
    tc.case_differential_edges("float32", OPS, DEV, chunk=8, page_size=8, heads=1, kv_heads=1, D=20, Dv=8)
    tc.case_capped_far_key("float32", OPS, DEV, T=130)
    tc.case_capped_far_key("float32", OPS, DEV, T=130, chunk=48)
    tc.case_latent_far_key_and_sink("float32", OPS, DEV, T=130)


def test_norms_and_rotations():
    tc.case_layer_norms("float32", OPS, DEV)
    tc.case_rotations("float32", OPS, DEV)


def test_model_less_entry():
    """``LLM(model=None, architecture="Tabisun")`` builds the design's tiny configuration."""
    from qwen3_runtime_b200 import LLM

    llm = LLM(None, architecture="Tabisun", dtype="float32", device=DEV, ops=OPS, cuda_graph=False)
    out = llm.generate([[1, 2, 3], [4, 5]], max_tokens=5)
    assert [len(o) for o in out] == [5, 5]
