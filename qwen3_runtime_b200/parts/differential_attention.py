"""Differential attention: two softmax maps per head over the same values, one subtracted from the other.

    q = W_q h  [heads, 2, dim]     k = W_k h  [kv_heads, 2, dim]     v = W_v h  [kv_heads, vdim]
    q, k: every map divided by its root mean square, times a weight of ``dim`` shared by heads and maps
    a_m(i) = sum_j softmax_j(scale * q_m(i) . k_m(j)) v(j)               m = 1, 2, over the keys i sees
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff                       one number for the layer
    o(i)   = a_1(i) - lambda * a_2(i);   o / sqrt(mean(o^2) + eps) * (1 - diff)   per head, no weight
    out    = W_o [o of all heads]

Positions do not enter the scores.  What a token sees: every j <= i, or with ``window`` the last ``window``
of them, or with ``chunk`` those of its own chunk (chunks of that many tokens counted from the sequence's
first token).  The cache is one paged layer: a key row holds both maps of a key head side by side, so that
one kernel scores both maps from one row and reads every value once for both sums; the subtraction and the
heads' norm are that kernel's epilogue.  In bfloat16 prompt portions run on the tensor cores and steps of one
token per sequence on a kernel that cuts the keys into slices (csrc/attention_diff.cu); float32, and sizes
those kernels refuse, run the general kernel (csrc/attention_generic.cu).
"""

from __future__ import annotations

import torch

from ..cache.layout import KVLayerSpec
from .base import BuildContext, ParamSpec, Part, StepContext, register_part
from .linear_state import _pad_rows


class DifferentialAttention(Part):
    category = "mixer"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.dim = int(spec["dim"])  # one map's query/key size
        self.vdim = int(spec["vdim"])
        self.scale = float(spec["scale"])
        self.diff = float(spec["diff"])
        self.eps = float(spec["eps"])
        self.window = spec.get("window") or None
        self.chunk = spec.get("chunk") or None
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.dim > 256 or self.vdim > 256:
            raise ValueError(f"dim={self.dim}, vdim={self.vdim}: the attention kernels take sizes up to 256")
        if self.window and self.chunk:
            raise ValueError("differential_attention: a window or chunks, not both")
        self.in_weight = self.o_weight = self.q_norm = self.k_norm = None
        self.starts: list[int] = []
        self.lam = 0.0

    def param_specs(self):
        H, G, D, Dv, W = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.hidden_size
        specs = {"q": ParamSpec((H * 2 * D, W)), "k": ParamSpec((G * 2 * D, W)), "v": ParamSpec((G * Dv, W)),
                 "q.norm": ParamSpec((D,), "vector"), "k.norm": ParamSpec((D,), "vector"),
                 "o": ParamSpec((W, H * Dv))}
        for name in ("lq1", "lk1", "lq2", "lk2"):
            specs[name] = ParamSpec((D,), "vector")
        return specs

    def load(self, tensors):
        self.in_weight, self.starts = _pad_rows([tensors["q"], tensors["k"], tensors["v"]])
        self.o_weight = tensors["o"].contiguous()
        self.q_norm, self.k_norm = tensors["q.norm"], tensors["k.norm"]
        # the layer's one number, in float32, worked out once
        first = (tensors["lq1"].float() * tensors["lk1"].float()).sum()
        second = (tensors["lq2"].float() * tensors["lk2"].float()).sum()
        self.lam = float(torch.exp(first) - torch.exp(second) + self.diff)

    def kernel_groups(self):
        groups = ["rope_kv", "attention_generic"]
        groups += ["gemm_f32"] if self.ctx.dtype == torch.float32 else ["gemm_small_m", "gemm_stream", "attention_diff"]
        return groups

    def cache_spec(self):
        return KVLayerSpec(self.num_kv_heads, 2 * self.dim, self.window, value_dim=self.vdim, chunk=self.chunk)

    def forward(self, h: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        ops = self.ops
        H, G, D, Dv = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        s = self.starts
        proj = ops.linear(h, self.in_weight)
        block_table = step.block_tables[cache.paged_index]
        ops.qk_norm_store(proj, num_heads=H, num_kv_heads=G, head_dim=2 * D, value_dim=Dv, k_start=s[1], v_start=s[2],
                          q_weight=self.q_norm, k_weight=self.k_norm, eps=self.eps, positions=step.positions,
                          token_seq=step.token_seq, block_table=block_table, k_pages=cache.k_pages,
                          v_pages=cache.v_pages, page_size=cache.page_size, write_kv=cache.writes, maps=2)
        ctx = torch.empty((h.shape[0], H * Dv), dtype=h.dtype, device=h.device)
        ops.differential_attention(proj, proj.stride(0), num_heads=H, num_kv_heads=G, map_dim=D, value_dim=Dv,
                                   k_pages=cache.k_pages, v_pages=cache.v_pages, block_table=block_table,
                                   token_seq=step.token_seq, positions=step.positions, out=ctx,
                                   page_size=cache.page_size, scale=self.scale, lam=self.lam, eps=self.eps,
                                   out_scale=1.0 - self.diff, window=self.window, chunk=self.chunk, step=step)
        return ops.linear(ctx, self.o_weight)


register_part("mixer", "differential_attention", DifferentialAttention)
