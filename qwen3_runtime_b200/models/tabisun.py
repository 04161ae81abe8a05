"""Tabisun expressed as data for the generic decoder.

A block norms only its sublayers' outputs (``output_norm`` with layer norms that have a weight and no
bias): x += LN(mixer(x)); x += LN(ff(x)).  The mixer of a layer is differential attention under a chunked
mask (``attention``), grouped attention whose values are the projected keys, with scaled interleaved
rotary positions and capped scores (``attention_2``), or attention through a latent with a rotated key part
shared by the heads, ramp-scaled frequencies, a sink and an output gate (``latent_attention``); the
feed-forward is a dense SwiGLU layer or absent.  A layer may run another layer's weights on a cache of its
own.  The logits are capped.  Tensor names: ``embed``, ``l<i>.norm1 | norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.spec import LayerRun, ModelSpec, PartSpec
from ..config.tabisun_config import (DifferentialConfig, KeyValueConfig, LatentConfig, RotaryConfig, TabisunConfig,
                                     TabisunLayerConfig)


def _position(rot: RotaryConfig | None, pairing: str, kind: str) -> PartSpec | None:
    if rot is None:
        return None
    scaling = dict(rot.scaling, kind=kind) if rot.scaling else None
    return PartSpec("rotary_scaled", dict(rotary_dim=rot.dims, theta=rot.base, pairing=pairing, scaling=scaling))


def _mixer_spec(cfg: TabisunConfig, m) -> PartSpec:
    if isinstance(m, DifferentialConfig):
        return PartSpec("differential_attention", dict(
            hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale,
            diff=m.diff, eps=cfg.norm_eps, chunk=m.chunk))
    if isinstance(m, KeyValueConfig):
        return PartSpec("sink_window_attention", dict(
            hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.dim, scale=m.scale,
            window=None, sink=None, gate=None, qk_norm_eps=cfg.norm_eps, values="keys", softcap=m.softcap,
            position=_position(m.rot, "interleaved", "wavelength")))
    if isinstance(m, LatentConfig):
        return PartSpec("latent_attention", dict(
            hidden_size=cfg.width, num_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, q_rank=0,
            kv_rank=m.kv_rank, eps=cfg.norm_eps, scale=m.scale, window=None, sink=True, gate="sigmoid",
            position=_position(m.rot, "half", "ramp")))
    raise TypeError(f"no Tabisun mixer for {type(m).__name__}")


def tabisun_spec(cfg: TabisunConfig) -> ModelSpec:
    norm = PartSpec("layernorm", dict(size=cfg.width, eps=cfg.norm_eps, weight_name=""))
    blocks, names, block_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        params = dict(mixer=_mixer_spec(cfg, layer.mixer), mixer_out_norm=norm, mixer_prefix="mix.",
                      mixer_out_norm_prefix="norm1", feed_forward=None)
        if layer.ff:
            params.update(feed_forward=PartSpec("gated_mlp", dict(
                hidden_size=cfg.width, intermediate_size=layer.ff, activation="silu",
                names=dict(gate="gate", up="up", down="down"))),
                feed_forward_out_norm=norm, feed_forward_prefix="mlp.", feed_forward_out_norm_prefix="norm2")
        block_of[i] = len(blocks)
        blocks.append(PartSpec("output_norm", params))
        names.append(f"l{i}.")
    # a layer that runs another layer's weights is a second run of that block on a cache layer of its own
    order = tuple(LayerRun(block=block_of[cfg.owner_of(i)], cache=i) for i in range(len(cfg.layers)))
    return ModelSpec(vocab_size=cfg.vocab, hidden_size=cfg.width, blocks=tuple(blocks), order=order,
                     final_norm=norm, tie_word_embeddings=False, embed_name="embed", head_name="head",
                     block_prefix="l{index}.", block_names=tuple(names), final_norm_prefix="final.norm",
                     logit_softcap=cfg.logit_softcap)


def tiny_tabisun_config() -> TabisunConfig:
    """A small model with every branch of the design: the three mixers, a layer without a feed-forward, a
    layer that runs another one's weights."""
    diff = DifferentialConfig(heads=4, kv_heads=2, dim=8, vdim=24, scale=0.3, diff=0.4, chunk=12)
    kv = KeyValueConfig(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.25, softcap=20.0,
                        rot=RotaryConfig(dims=8, base=10000.0,
                                         scaling=(("factor", 4.0), ("low", 1.0), ("high", 4.0), ("original", 64.0))))
    latent = LatentConfig(heads=2, dim=16, rot_dim=8, vdim=24, kv_rank=32, scale=0.2,
                          rot=RotaryConfig(dims=8, base=10000.0,
                                           scaling=(("factor", 4.0), ("original", 32.0), ("fast", 16.0), ("slow", 1.0))))
    layers = (TabisunLayerConfig("attention", diff, 48), TabisunLayerConfig("attention_2", kv, None),
              TabisunLayerConfig("latent_attention", latent, 40), TabisunLayerConfig("attention", diff, 48, weights_of=0))
    return TabisunConfig(vocab=64, width=40, norm_eps=1e-5, layers=layers, logit_softcap=12.0)


register_architecture(TabisunConfig.architecture, TabisunConfig, tabisun_spec, tiny_config=tiny_tabisun_config)
