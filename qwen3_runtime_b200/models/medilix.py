"""Medilix expressed as data for the generic decoder.

The embedding is the token's row times a constant plus a row of a bigram table chosen by a hash of the
previous and the present token.  Every block reads the stream through two grouped RMS norms and adds
its mixer's and its feed-forward's outputs together (``parallel_norms``).  The mixer of a layer is a
gated matrix memory (``mlstm``), softmax attention with a window that keeps the first tokens, a sink and
an output gate, or token-shifted ``wkv``; the feed-forward is a clamped dense layer, routed experts
(softmax scores with a correction for the choice, groups, identity experts), or absent.  A run of layers
may be repeated with the same weights: every pass has cache layers of its own, and before a pass's first
layer the stream becomes ``loop.in`` times [stream; embedding output].
Tensor names: ``embed``, ``bigram``, ``loop.in``, ``l<i>.norm1 | norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.medilix_config import (BigramConfig, DenseConfig, GatedAttentionConfig, MedilixConfig,
                                     MedilixLayerConfig, MlstmConfig, MoeConfig, WkvConfig)
from ..config.registry import register_architecture
from ..config.spec import LayerRun, ModelSpec, PartSpec

LOOP_TABLE = "loop.in"


def _mixer_spec(cfg: MedilixConfig, layer: MedilixLayerConfig) -> PartSpec:
    m = layer.mixer
    if isinstance(m, MlstmConfig):
        return PartSpec("mlstm", dict(hidden_size=cfg.width, num_heads=m.heads, dim=m.dim, vdim=m.vdim,
                                      gate_cap=m.gate_cap, eps=cfg.norm_eps))
    if isinstance(m, GatedAttentionConfig):
        return PartSpec("sink_window_attention", dict(
            hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale,
            window=m.window, keep_first=m.keep_first, sink=0.0, gate="sigmoid", qk_norm_eps=cfg.norm_eps))
    if not m.decay_rank:
        raise ValueError("wkv: the decay's rank is not known yet; it is the row count of the stored w1 "
                         "(MedilixConfig.with_tensor_shapes)")
    return PartSpec("wkv", dict(hidden_size=cfg.width, num_heads=m.heads, dim=m.dim, decay_rank=m.decay_rank,
                                eps=cfg.norm_eps))


def _feed_forward_spec(cfg: MedilixConfig, f) -> PartSpec:
    if isinstance(f, DenseConfig):
        return PartSpec("clamped_mlp", dict(hidden_size=cfg.width, intermediate_size=f.ff, limit=f.limit,
                                            alpha=1.702, up_offset=1.0))
    return PartSpec("routed_experts", dict(
        hidden_size=cfg.width, num_experts=f.experts, num_identity=f.identity, top=f.top, expert_size=f.ff,
        activation="silu_glu", score="softmax_all", correction=True, renormalize=True, weight_on="output",
        groups=(f.groups, f.groups_keep) if f.groups > 1 else None))


def medilix_spec(cfg: MedilixConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(size=cfg.width, eps=cfg.norm_eps, weight_name="", groups=cfg.norm_groups))
    blocks = []
    for layer in cfg.layers:
        params = dict(mixer=_mixer_spec(cfg, layer), mixer_norm=norm, mixer_prefix="mix.", mixer_norm_prefix="norm1")
        if layer.mlp is not None:
            params.update(feed_forward=_feed_forward_spec(cfg, layer.mlp), feed_forward_norm=norm,
                          feed_forward_prefix="mlp.", feed_forward_norm_prefix="norm2")
        blocks.append(PartSpec("parallel_norms", params))
    order = tuple(LayerRun(block=layer, cache=run, mix_source=LOOP_TABLE if starts else None)
                  for run, (layer, starts) in enumerate(cfg.run_order()))
    big = cfg.bigram
    embedding = PartSpec("scaled_bigram", dict(
        vocab_size=cfg.vocab, hidden_size=cfg.width, scale=cfg.embed_scale, buckets=big.buckets if big else 0,
        mul_prev=big.mul_prev if big else 0, mul_cur=big.mul_cur if big else 0))
    tables = ((LOOP_TABLE, (cfg.width, 2 * cfg.width), "matrix"),) if cfg.loop_times else ()
    return ModelSpec(vocab_size=cfg.vocab, hidden_size=cfg.width, blocks=tuple(blocks), order=order,
                     final_norm=norm, tie_word_embeddings=False, embed_name="embed", head_name="head",
                     block_prefix="l{index}.", final_norm_prefix="final.norm", shared_tables=tables,
                     embedding=embedding)


def tiny_medilix_config() -> MedilixConfig:
    """A small model with every branch of the design: the three mixers, both feed-forwards, a layer
    without one, a loop in the middle."""
    moe = MoeConfig(experts=6, identity=2, top=3, ff=16, groups=4, groups_keep=3)
    layers = (
        MedilixLayerConfig("mlstm", MlstmConfig(heads=2, dim=16, vdim=24, gate_cap=10.0), DenseConfig(ff=48, limit=2.0)),
        MedilixLayerConfig("attention", GatedAttentionConfig(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.3, window=20,
                                                             keep_first=3), moe),
        MedilixLayerConfig("wkv", WkvConfig(heads=2, dim=16, decay_rank=8), None),
        MedilixLayerConfig("attention", GatedAttentionConfig(heads=2, kv_heads=1, dim=24, vdim=24, scale=0.2,
                                                             window=None, keep_first=0), DenseConfig(ff=40, limit=1.5)),
    )
    return MedilixConfig(vocab=64, width=40, norm_eps=1e-5, norm_groups=2, embed_scale=6.0,
                         bigram=BigramConfig(buckets=61, mul_prev=13, mul_cur=7), layers=layers,
                         loop_start=1, loop_stop=3, loop_times=2)


register_architecture(MedilixConfig.architecture, MedilixConfig, medilix_spec, tiny_config=tiny_medilix_config)
