"""Routed feed-forward: many small gated layers, each token through a few of them.

    z = W_router h (float32)      s = score(z)      chosen = the ``top`` largest s
    out = sum over chosen e of expert_e(w_e * h)  (+ shared(h))      w_e = s_e

The score is a sigmoid and the weights are the chosen scores as they are (``renormalize``
divides them by their sum).  ``weight_on`` says what the weight multiplies: the expert's
``"input"`` or its ``"output"``; the two differ because an expert is not linear.  An expert is
the clamped gated layer

    g = min(W_gate x, limit)   u = clamp(W_up x, -limit, limit)   y = g * sigmoid(alpha g) * (u + up_offset)
    expert(x) = W_down y

``activation="relu2"``: an expert has no gate, expert(x) = W_down relu(W_up x)^2.
``score="softmax_chosen"``: the weights are the softmax over the chosen logits only.
``shared_gate="sigmoid"``: the shared expert's result is multiplied by sigmoid(w_sg . h), one number
per token (the stored ``shared.sg`` ``[1, width]`` rides along as one more row of the shared expert's
first product).

``activation="silu_glu"``: the plain gated unit silu(W_gate x) * (W_up x), no clamps.
``score="softmax_all"``: s is the softmax over all router outputs; the choice is made on s plus a stored
``correction`` per output (when ``correction`` is set), the weights are the chosen s themselves
(``renormalize`` divides them by their sum + 1e-20).  ``groups = (count, keep)``: the router outputs form
``count`` equal groups of neighbours, a group's score is the largest choice score in it, and only outputs
of the ``keep`` best groups can be chosen.  ``num_identity``: that many further router outputs (after the
stored experts') stand for experts that return their input; they have no tensors.

Tokens are grouped by expert on the device (no host round trip, so a step with experts can be
captured), each expert's products run over its own tokens only, and the results are summed per
token in float32.
"""

from __future__ import annotations

import torch

from .base import BuildContext, ParamSpec, Part, StepContext, register_part


class RoutedExperts(Part):
    category = "feed_forward"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.num_experts = int(spec["num_experts"])
        self.top = int(spec["top"])
        self.expert_size = int(spec["expert_size"])
        self.activation = spec.get("activation", "clamped_glu")
        self.gated = self.activation in ("clamped_glu", "silu_glu")
        self.limit = float(spec.get("limit") or 0.0)
        self.num_identity = int(spec.get("num_identity") or 0)
        self.correction = bool(spec.get("correction", False))
        self.groups = tuple(int(x) for x in spec["groups"]) if spec.get("groups") else None
        self.shared_gate = spec.get("shared_gate")
        self.alpha = float(spec.get("alpha", 1.702))
        self.up_offset = float(spec.get("up_offset", 1.0))
        if self.activation == "silu_glu":  # the clamped unit without clamps, with a plain sigmoid and no offset
            self.limit, self.alpha, self.up_offset = float("inf"), 1.0, 0.0
        self.score = spec.get("score", "sigmoid")
        self.renormalize = bool(spec.get("renormalize", False))
        self.weight_on = spec.get("weight_on", "input")
        self.shared_size = int(spec["shared_size"]) if spec.get("shared_size") else 0
        self.shared_limit = float(spec.get("shared_limit") or self.limit)
        if self.score not in ("sigmoid", "softmax_chosen", "softmax_all"):
            raise ValueError(f"routed_experts scores with 'sigmoid', 'softmax_chosen' or 'softmax_all', not {self.score!r}")
        if (self.correction or self.groups) and self.score != "softmax_all":
            raise ValueError("routed_experts: a correction and groups go with score='softmax_all'")
        if self.num_identity and self.weight_on != "output":
            raise ValueError("routed_experts: identity experts take their weight on the output")
        if self.activation not in ("clamped_glu", "silu_glu", "relu2"):
            raise ValueError(f"routed_experts: unknown activation {self.activation!r}")
        if self.gated and not self.limit > 0:
            raise ValueError("routed_experts: the clamped gated unit needs a positive limit")
        if not self.gated and self.weight_on != "output":
            raise ValueError("routed_experts: experts without a gate take their weight on the output")
        if self.shared_gate not in (None, "sigmoid") or (self.shared_gate and (self.gated or not self.shared_size)):
            raise ValueError("routed_experts: shared_gate is 'sigmoid' on an ungated shared expert, or absent")
        if self.weight_on not in ("input", "output"):
            raise ValueError("weight_on is 'input' or 'output'")
        if not 1 <= self.top <= self.num_experts + self.num_identity:
            raise ValueError("top must lie in 1..num_experts (+ identity experts)")
        self.router = self.gate_up = self.down = self.shared_gate_up = self.shared_down = None

    def param_specs(self):
        E, F, W = self.num_experts, self.expert_size, self.hidden_size
        specs = {}
        for e in range(E):
            if self.gated:
                specs[f"e{e}.gate"] = ParamSpec((F, W))
            specs[f"e{e}.up"] = ParamSpec((F, W))
            specs[f"e{e}.down"] = ParamSpec((W, F))
        specs["router"] = ParamSpec((E + self.num_identity, W), "matrix_f32")
        if self.correction:
            specs["correction"] = ParamSpec((E + self.num_identity,), "vector")
        if self.shared_size:
            if self.gated:
                specs["shared.gate"] = ParamSpec((self.shared_size, W))
            specs["shared.up"] = ParamSpec((self.shared_size, W))
            specs["shared.down"] = ParamSpec((W, self.shared_size))
            if self.shared_gate:
                specs["shared.sg"] = ParamSpec((1, W))
        return specs

    def load(self, tensors):
        E = self.num_experts
        if self.gated:  # per expert: gate rows, then up rows
            self.gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0)
                                        for e in range(E)]).contiguous()
        else:
            self.gate_up = torch.stack([tensors[f"e{e}.up"] for e in range(E)]).contiguous()
        self.down = torch.stack([tensors[f"e{e}.down"] for e in range(E)]).contiguous()
        self.router = tensors["router"].contiguous()
        self.correction_vec = tensors["correction"].contiguous() if self.correction else None
        if self.shared_size and self.gated:
            self.shared_gate_up = torch.cat([tensors["shared.gate"], tensors["shared.up"]], dim=0).contiguous()
            self.shared_down = tensors["shared.down"].contiguous()
        elif self.shared_size:
            # the up rows, then (with a gate) the gate's row, then zero rows up to a multiple of 8
            rows = [tensors["shared.up"]] + ([tensors["shared.sg"]] if self.shared_gate else [])
            pad = -sum(r.shape[0] for r in rows) % 8
            if pad:
                rows.append(rows[0].new_zeros((pad, rows[0].shape[1])))
            self.shared_gate_up = torch.cat(rows, dim=0).contiguous()
            self.shared_down = tensors["shared.down"].contiguous()

    def kernel_groups(self):
        groups = ["experts", "norm"]
        if self.ctx.dtype == torch.float32:
            groups.append("gemm_f32")
        else:
            groups += ["gemm_small_m", "gemm_stream"]
        return groups

    def forward(self, h: torch.Tensor, step: StepContext) -> torch.Tensor:
        ops = self.ops
        if self.score == "softmax_all":
            chosen, weights = ops.route_top(h, self.router, self.top, renormalize=self.renormalize, score=self.score,
                                            correction=self.correction_vec, groups=self.groups)
        else:
            chosen, weights = ops.route_top(h, self.router, self.top, renormalize=self.renormalize, score=self.score)
        shared = None
        if self.shared_size and not self.gated:
            up = ops.linear(h, self.shared_gate_up)
            mid = torch.empty((h.shape[0], self.shared_size), dtype=h.dtype, device=h.device)
            ops.relu_squared(up, mid)
            shared = ops.linear(mid, self.shared_down)
            return ops.routed_experts(h, chosen, weights, self.gate_up, self.down, weight_on="output", shared=shared,
                                      activation="relu2",
                                      shared_gate=up[:, self.shared_size] if self.shared_gate else None)
        if not self.gated:
            return ops.routed_experts(h, chosen, weights, self.gate_up, self.down, weight_on="output",
                                      activation="relu2")
        if self.shared_size:
            mid = torch.empty((h.shape[0], self.shared_size), dtype=h.dtype, device=h.device)
            ops.clamped_glu(ops.linear(h, self.shared_gate_up), mid, limit=self.shared_limit, alpha=self.alpha,
                            up_offset=self.up_offset)
            shared = ops.linear(mid, self.shared_down)
        extra = dict(num_identity=self.num_identity) if self.num_identity else {}
        return ops.routed_experts(h, chosen, weights, self.gate_up, self.down, limit=self.limit, alpha=self.alpha,
                                  up_offset=self.up_offset, weight_on=self.weight_on, shared=shared, **extra)


register_part("feed_forward", "routed_experts", RoutedExperts)
