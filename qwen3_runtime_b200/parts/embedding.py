"""Embedding parts: what turns a step's token ids into the stream's first value.

``scaled_bigram``: ``x = embed[token] * scale + bigram[row]`` with ``row = (previous token * mul_prev +
token * mul_cur) mod buckets``, and row ``buckets`` (the table's last) for a sequence's first token.  The
previous token of a request is kept in a state slot (one int32 per request), so a portion that starts
in the middle of a sequence, or a decoded token whose predecessor the host has not read yet, finds it
on the device.  Without ``buckets`` the part is a scaled lookup only and keeps no state.
"""

from __future__ import annotations

import torch

from ..cache.layout import StateLayerSpec
from .base import BuildContext, ParamSpec, Part, ResidualStream, StepContext, register_part


class ScaledBigramEmbedding(Part):
    category = "embedding"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.vocab_size = int(spec["vocab_size"])
        self.hidden_size = int(spec["hidden_size"])
        self.scale = float(spec.get("scale", 1.0))
        self.buckets = int(spec.get("buckets") or 0)
        self.mul_prev = int(spec.get("mul_prev") or 0)
        self.mul_cur = int(spec.get("mul_cur") or 0)
        self.embed_name = str(spec.get("embed_name", "embed"))
        self.bigram_name = str(spec.get("bigram_name", "bigram"))
        self.table: torch.Tensor | None = None
        self.bigram: torch.Tensor | None = None

    def param_specs(self):
        specs = {self.embed_name: ParamSpec((self.vocab_size, self.hidden_size))}
        if self.buckets:
            specs[self.bigram_name] = ParamSpec((self.buckets + 1, self.hidden_size))
        return specs

    def load(self, tensors):
        self.table = tensors[self.embed_name].contiguous()
        self.bigram = tensors[self.bigram_name].contiguous() if self.buckets else None

    def kernel_groups(self):
        return ["token_state"]

    def cache_spec(self):
        return StateLayerSpec((1,), "int32") if self.buckets else None

    def start(self, step: StepContext, cache, keep_source: bool) -> ResidualStream:
        """The stream of a step: float32 rows of the embedding output; with ``keep_source`` also a buffer
        ``[tokens, 2 * hidden]`` in the compute dtype whose right half holds those rows."""
        T, W = step.num_tokens, self.hidden_size
        resid = torch.empty((T, W), dtype=torch.float32, device=self.ctx.device)
        pair = torch.empty((T, 2 * W), dtype=self.ctx.dtype, device=self.ctx.device) if keep_source else None
        self.ops.bigram_embed(step.token_ids, embed=self.table, scale=self.scale, bigram=self.bigram,
                              buckets=self.buckets, mul_prev=self.mul_prev, mul_cur=self.mul_cur,
                              prev_state=cache.state if cache is not None else None, positions=step.positions,
                              token_seq=step.token_seq, cu_seqlens=step.cu_seqlens, state_slots=step.state_slots,
                              num_seqs=step.num_seqs, out=resid, copy=pair[:, W:] if pair is not None else None)
        return ResidualStream.started(resid, pair)


register_part("embedding", "scaled_bigram", ScaledBigramEmbedding)
