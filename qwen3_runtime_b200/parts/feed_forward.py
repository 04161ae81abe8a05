"""Dense gated feed-forward (SwiGLU): down(silu(gate x) * up x), no biases
(qwen3_runtime/models/qwen3.py:130-138; layers/ops.py:23-25)."""

from __future__ import annotations

import torch

from .base import BuildContext, ParamSpec, Part, StepContext, register_part


class GatedMLP(Part):
    category = "feed_forward"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.intermediate_size = int(spec["intermediate_size"])
        activation = spec.get("activation", "silu")
        if activation != "silu":
            raise ValueError(f"gated_mlp has a silu kernel only, not {activation!r}")
        self.down_bias = bool(spec.get("down_bias", False))
        # the stored tensors' names (after the part's prefix), for checkpoints that call them otherwise
        names = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight",
                     down_bias="down_proj.bias")
        names.update(spec.get("names") or {})
        self.names = names
        self.gate_up_weight = self.down_weight = self.down_bias_vec = None

    def param_specs(self):
        n = self.names
        specs = {
            n["gate"]: ParamSpec((self.intermediate_size, self.hidden_size)),
            n["up"]: ParamSpec((self.intermediate_size, self.hidden_size)),
            n["down"]: ParamSpec((self.hidden_size, self.intermediate_size)),
        }
        if self.down_bias:
            specs[n["down_bias"]] = ParamSpec((self.hidden_size,), "vector")
        return specs

    def load(self, tensors):
        # one product for gate and up: gate rows first (utils/loader.py:51-53)
        n = self.names
        self.gate_up_weight = torch.cat([tensors[n["gate"]], tensors[n["up"]]], dim=0).contiguous()
        self.down_weight = tensors[n["down"]].contiguous()
        self.down_bias_vec = tensors.get(n["down_bias"])

    def kernel_groups(self):
        if self.ctx.dtype == torch.float32:
            return ["norm", "gemm_f32"]
        return ["norm", "gemm_small_m", "gemm_stream", "gemm_tcgen05"]

    def forward(self, h: torch.Tensor, step: StepContext) -> torch.Tensor:
        mid = torch.empty((h.shape[0], self.intermediate_size), dtype=h.dtype, device=h.device)
        self.ops.gated_linear(h, self.gate_up_weight, mid)
        if self.down_bias_vec is not None:
            return self.ops.linear(mid, self.down_weight, bias=self.down_bias_vec)
        return self.ops.linear(mid, self.down_weight, partial_sums=self.partial_sums_ok)


class ClampedMLP(Part):
    """A dense gated layer with clamped products: g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit),
    y = g * sigmoid(alpha g) * (u + up_offset), out = W_down y.  Stored tensors ``gate``, ``up``, ``down``."""

    category = "feed_forward"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.intermediate_size = int(spec["intermediate_size"])
        self.limit = float(spec["limit"])
        self.alpha = float(spec.get("alpha", 1.702))
        self.up_offset = float(spec.get("up_offset", 1.0))
        if not self.limit > 0:
            raise ValueError("clamped_mlp: the limit must be positive")
        self.gate_up_weight = self.down_weight = None

    def param_specs(self):
        F, W = self.intermediate_size, self.hidden_size
        return {"gate": ParamSpec((F, W)), "up": ParamSpec((F, W)), "down": ParamSpec((W, F))}

    def load(self, tensors):
        self.gate_up_weight = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.down_weight = tensors["down"].contiguous()

    def kernel_groups(self):
        return ["norm", "gemm_f32"] if self.ctx.dtype == torch.float32 else ["norm", "gemm_small_m", "gemm_stream"]

    def forward(self, h: torch.Tensor, step: StepContext) -> torch.Tensor:
        mid = torch.empty((h.shape[0], self.intermediate_size), dtype=h.dtype, device=h.device)
        self.ops.clamped_glu(self.ops.linear(h, self.gate_up_weight), mid, limit=self.limit, alpha=self.alpha,
                             up_offset=self.up_offset)
        return self.ops.linear(mid, self.down_weight, partial_sums=self.partial_sums_ok)


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "clamped_mlp", ClampedMLP)
