"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, all in float32, one rounding at the end
(qwen3_runtime/layers/ops.py:17-20; residual form :28-37).  ``weight_offset``: the stored weight
is the deviation from this value, which is added to it when it is loaded (y = ... * (offset + w)).
``groups`` > 1: a row is cut into that many equal consecutive parts and each is divided by its own root
mean square (the weight still spans the whole row).
``layernorm``: y = (x - mean(x)) * rsqrt(mean((x - mean(x))^2) + eps) * w, a weight and no bias; the same part
with the mean taken off first (the same kernels with their ``center`` flags)."""

from __future__ import annotations

import torch

from .base import BuildContext, ParamSpec, Part, ResidualStream, register_part


class RMSNorm(Part):
    category = "norm"
    adds_partial_sums = True
    center = False  # True: a layer norm (the mean is taken off before the mean square)

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        # the stored tensor's name after the part's prefix ("" when the prefix is the whole name)
        self.weight_name = str(spec.get("weight_name", "weight"))
        self.weight_offset = float(spec.get("weight_offset", 0.0))
        self.groups = int(spec.get("groups") or 1)
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"rmsnorm: {self.size} elements do not split into {self.groups} equal groups")
        if self.center and self.groups > 1:
            raise ValueError("layernorm: no groups")
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {self.weight_name: ParamSpec((self.size,), "vector")}

    def load(self, tensors):
        self.weight = tensors[self.weight_name]
        if self.weight_offset:
            self.weight = (self.weight.float() + self.weight_offset).contiguous()

    def pending_scale(self) -> tuple:
        """This norm as something the next norm applies to what is pending (``ResidualStream.pending_norm``):
        ``(weight, eps)``, or ``(weight, eps, True)`` for a layer norm."""
        return (self.weight, self.eps, True) if self.center else (self.weight, self.eps)

    def kernel_groups(self):
        return ["norm"]

    def add_norm(self, stream: ResidualStream, rows: torch.Tensor | None = None,
                 num_rows: int | None = None, normalise: bool = True, second: "RMSNorm | None" = None):
        """Fold what is pending into the residual sum and return its normalised rows.

        With ``rows`` only those rows are normalised and the residual sum is left as
        it is (the final norm before the output head).  ``normalise=False``: the rows of the sum
        itself, rounded to the activation type (the stream as the input of a product).
        ``second``: another norm of the same size, groups and eps; the answer is then the pair
        ``(this norm's rows, the second norm's rows)`` of the same sum, made by one kernel."""
        n = stream.num_tokens if rows is None else (num_rows if num_rows is not None else rows.numel())
        if self.groups > 1 or second is not None or stream.pending_more is not None:
            if self.center:
                raise NotImplementedError("layernorm: one norm of one pending output at a time")
            return self._grouped(stream, rows, n, normalise, second)
        out = torch.empty((n, self.size), dtype=self.ctx.dtype, device=self.ctx.device)
        keep = rows is None
        extra = {}
        if stream.pending is not None and stream.pending_norm is not None:
            extra.update(post_weight=stream.pending_norm[0], post_eps=stream.pending_norm[1])
            if len(stream.pending_norm) > 2 and stream.pending_norm[2]:
                extra.update(post_center=True)
        if self.center and normalise:
            extra.update(center=True)
        if stream.add_source:
            if stream.embed is not None:
                raise ValueError("the embedding cannot be added again before it was read once")
            extra.update(add_ids=stream.source[0], add_table=stream.source[1])
        if stream.add_vector is not None:
            extra.update(add_vector=stream.add_vector)
        weight = self.weight if normalise else None
        if stream.embed is not None:
            ids, table = stream.embed
            if keep:
                stream.resid = torch.empty((stream.num_tokens, self.size), dtype=torch.float32,
                                           device=self.ctx.device)
            self.ops.fused_norm(out, weight, self.eps, resid=stream.resid if keep else None,
                                pending=stream.pending, ids=ids, table=table, rows=rows, write_resid=keep,
                                num_rows=n, **extra)
            if keep:
                stream.embed = None
        else:
            self.ops.fused_norm(out, weight, self.eps, resid=stream.resid, pending=stream.pending,
                                rows=rows, write_resid=keep, num_rows=n, **extra)
        if keep:
            stream.pending = None
            stream.pending_norm = None
            stream.add_source = False
            stream.add_vector = None
        return out


    def _grouped(self, stream: ResidualStream, rows, n: int, normalise: bool, second):
        """The general kernel: groups, two pending outputs, two weights."""
        if stream.embed is not None or stream.pending_norm is not None or stream.add_source or stream.add_vector is not None:
            raise NotImplementedError("rmsnorm: the grouped norm kernel folds pending outputs only (no embedding lookup, "
                                      "no normalised pending output, no added rows or vectors)")
        if second is not None and (second.size != self.size or second.groups != self.groups or second.eps != self.eps):
            raise ValueError("rmsnorm: two norms of one sum share size, groups and eps")
        keep = rows is None
        out = torch.empty((n, self.size), dtype=self.ctx.dtype, device=self.ctx.device)
        out2 = torch.empty_like(out) if second is not None else None
        self.ops.grouped_norm(out, self.weight if normalise else None, self.eps, self.groups, resid=stream.resid,
                              pending=stream.pending, pending_more=stream.pending_more, rows=rows, write_resid=keep,
                              num_rows=n, out2=out2, weight2=second.weight if second is not None else None)
        if keep:
            stream.pending = stream.pending_more = None
        return out if second is None else (out, out2)


def fold_stream(ops, stream: ResidualStream, out: torch.Tensor) -> torch.Tensor:
    """Add what is pending to the residual sum and write the sum, rounded to ``out``'s type, into ``out``
    (``[tokens, hidden]``, possibly a view of wider rows)."""
    if stream.embed is not None or stream.pending_norm is not None or stream.add_source or stream.add_vector is not None:
        raise NotImplementedError("fold_stream: the stream holds more than pending outputs")
    ops.grouped_norm(out, None, 0.0, 1, resid=stream.resid, pending=stream.pending, pending_more=stream.pending_more,
                     rows=None, write_resid=True, num_rows=stream.num_tokens)
    stream.pending = stream.pending_more = None
    return out


class LayerNorm(RMSNorm):
    center = True


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
