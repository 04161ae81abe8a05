"""Mixers with a matrix memory per (request, head) whose update is gated per token.

``mlstm``: exponential input and forget gates with a running maximum m as stabiliser (m starts at 0):

    li = cap * tanh((w_i . h + b_i) / cap)         lf = logsigmoid(cap * tanh((w_f . h + b_f) / cap))
    m_t = max(lf + m_(t-1), li)       a = exp(lf + m_(t-1) - m_t)       b = exp(li - m_t)
    S_t = a S_(t-1) + b k_t v_t^T     n_t = a n_(t-1) + b k_t           q = W_q h * dim^(-1/2)
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

The normaliser n is kept as one more value column of S (a column whose value is always 1), so the
state kernel serves it unchanged; m is a second small state.  Each head's o is divided by its root mean
square, multiplied by a weight over all heads' values and by sigmoid(W_g h), and projected.

``wkv``: each of r, k, v, g and the decay reads its own blend of the token's input and the previous
token's (``h + (h' - h) * mu``; h' is kept in a state slot), the decay per key channel is
``exp(-exp(W_w2 tanh(W_w1 x_w) + w0))``, and the present token counts with a bonus u instead of a decay:

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t        S_t = diag(w_t) S_(t-1) + k_t v_t^T

followed by the same unit norm per head, weight, times silu(W_g x_g), projection.

Gates, decays, their logarithms, the states and the unit norms are float32 whatever the compute dtype.
"""

from __future__ import annotations

import torch

from ..cache.layout import StateLayerSpec
from .base import BuildContext, ParamSpec, Part, StepContext, register_part
from .linear_state import _pad_rows, heads_view


def _product_groups(ctx: BuildContext) -> list[str]:
    return ["gemm_f32"] if ctx.dtype == torch.float32 else ["gemm_small_m", "gemm_stream"]


class MatrixLstm(Part):
    category = "mixer"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.dim = int(spec["dim"])
        self.vdim = int(spec["vdim"])
        self.cap = float(spec["gate_cap"])
        self.eps = float(spec["eps"])
        if self.dim > 256:
            raise ValueError(f"dim={self.dim} is not supported: the state kernel keeps up to 256 key rows per head")
        self.in_weight = self.o_weight = self.norm_weight = self.i_bias = self.f_bias = None
        self.starts: list[int] = []

    def param_specs(self):
        H, D, Dv, W = self.num_heads, self.dim, self.vdim, self.hidden_size
        return {"q": ParamSpec((H * D, W)), "k": ParamSpec((H * D, W)), "v": ParamSpec((H * Dv, W)),
                "g": ParamSpec((H * Dv, W)), "o": ParamSpec((W, H * Dv)), "norm": ParamSpec((H * Dv,), "vector"),
                "i": ParamSpec((H, W)), "i.b": ParamSpec((H,), "vector"),
                "f": ParamSpec((H, W)), "f.b": ParamSpec((H,), "vector")}

    def load(self, tensors):
        self.in_weight, self.starts = _pad_rows([tensors[n] for n in ("q", "k", "v", "g", "i", "f")])
        self.o_weight = tensors["o"].contiguous()
        self.norm_weight = tensors["norm"].contiguous()
        self.i_bias = tensors["i.b"].contiguous()
        self.f_bias = tensors["f.b"].contiguous()

    def kernel_groups(self):
        return ["linear_state", *_product_groups(self.ctx)]

    def cache_spec(self):
        # the memory with the normaliser as its last value column, and the running maximum
        return (StateLayerSpec((self.num_heads, self.dim, self.vdim + 1)), StateLayerSpec((self.num_heads,)))

    def forward(self, h: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        ops = self.ops
        memory, maximum = cache
        H, D, Dv = self.num_heads, self.dim, self.vdim
        s = self.starts
        proj = ops.linear(h, self.in_weight)
        q, k = heads_view(proj, s[0], H, D), heads_view(proj, s[1], H, D)
        v, g = heads_view(proj, s[2], H, Dv), heads_view(proj, s[3], H, Dv)
        decay, k_scale, m_run = ops.stabilised_gates(
            proj[:, s[4]:s[4] + H], proj[:, s[5]:s[5] + H], i_bias=self.i_bias, f_bias=self.f_bias, cap=self.cap,
            m_state=maximum.state, cu_seqlens=step.cu_seqlens, state_slots=step.state_slots, num_seqs=step.num_seqs)
        o = ops.decayed_state_scan(q, k, v, state=memory.state, cu_seqlens=step.cu_seqlens,
                                   state_slots=step.state_slots, num_seqs=step.num_seqs, token_decay=decay,
                                   token_k_scale=k_scale, ones_column=True, q_scale=D ** -0.5)
        ctx = torch.empty((h.shape[0], H * Dv), dtype=h.dtype, device=h.device)
        ops.head_norm_gate(o, g, ctx.unflatten(1, (H, Dv)), weight=self.norm_weight, eps=self.eps, gate_act="sigmoid",
                           per_head_weight=True, denominator=m_run)
        return ops.linear(ctx, self.o_weight)


class ShiftedWkv(Part):
    category = "mixer"
    BLENDS = ("r", "k", "v", "g", "w")

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.dim = int(spec["dim"])
        self.decay_rank = int(spec["decay_rank"])
        self.eps = float(spec["eps"])
        if self.dim > 256:
            raise ValueError(f"dim={self.dim} is not supported: the state kernel keeps up to 256 key rows per head")
        if self.decay_rank < 1:
            raise ValueError("wkv: the rank of the decay's product is the row count of the stored w1")
        self.weights: dict[str, torch.Tensor] = {}
        self.mu = self.w0 = self.bonus = self.norm_weight = None

    def param_specs(self):
        H, D, W, R = self.num_heads, self.dim, self.hidden_size, self.decay_rank
        specs = {f"mu.{s}": ParamSpec((W,), "vector") for s in self.BLENDS}
        specs.update({"r": ParamSpec((H * D, W)), "k": ParamSpec((H * D, W)), "v": ParamSpec((H * D, W)),
                      "g": ParamSpec((H * D, W)), "w1": ParamSpec((R, W)), "w2": ParamSpec((H * D, R)),
                      "w0": ParamSpec((H * D,), "vector"), "u": ParamSpec((H, D), "vector"),
                      "norm": ParamSpec((H * D,), "vector"), "o": ParamSpec((W, H * D))})
        return specs

    def load(self, tensors):
        self.weights = {n: tensors[n].contiguous() for n in ("r", "k", "v", "g", "w1", "w2", "o")}
        self.mu = torch.stack([tensors[f"mu.{s}"] for s in self.BLENDS]).contiguous()
        self.w0 = tensors["w0"].contiguous()
        self.bonus = tensors["u"].reshape(-1).contiguous()
        self.norm_weight = tensors["norm"].contiguous()

    def kernel_groups(self):
        return ["linear_state", "token_state", "norm", *_product_groups(self.ctx)]

    def cache_spec(self):
        # the memory, and the previous token's input row
        return (StateLayerSpec((self.num_heads, self.dim, self.dim)), StateLayerSpec((self.hidden_size,)))

    def forward(self, h: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        ops = self.ops
        memory, previous = cache
        H, D = self.num_heads, self.dim
        w = self.weights
        x = ops.token_shift_mix(h, self.mu, state=previous.state, positions=step.positions, token_seq=step.token_seq,
                                cu_seqlens=step.cu_seqlens, state_slots=step.state_slots, num_seqs=step.num_seqs)
        r = ops.linear(x[0], w["r"]).unflatten(1, (H, D))
        k = ops.linear(x[1], w["k"]).unflatten(1, (H, D))
        v = ops.linear(x[2], w["v"]).unflatten(1, (H, D))
        g = ops.linear(x[3], w["g"]).unflatten(1, (H, D))
        z = ops.linear(ops.tanh_rows(ops.linear(x[4], w["w1"])), w["w2"]).unflatten(1, (H, D))
        o = ops.decayed_state_scan(r, k, v, state=memory.state, cu_seqlens=step.cu_seqlens,
                                   state_slots=step.state_slots, num_seqs=step.num_seqs, decay_logits=z,
                                   decay_bias=self.w0, decay_mode="exp_neg_exp", bonus=self.bonus)
        ctx = torch.empty((h.shape[0], H * D), dtype=h.dtype, device=h.device)
        ops.head_norm_gate(o, g, ctx.unflatten(1, (H, D)), weight=self.norm_weight, eps=self.eps, gate_act="silu",
                           per_head_weight=True)
        return ops.linear(ctx, w["o"])


register_part("mixer", "mlstm", MatrixLstm)
register_part("mixer", "wkv", ShiftedWkv)
