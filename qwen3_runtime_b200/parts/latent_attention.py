"""Attention through a low-rank latent, over a paged cache that holds the latent only.

    c_q = RMSNorm(W_dq h)                 q_h = W_uq,h c_q = [q_h^plain (dim) | q_h^rot (rot_dim)]
    [c_raw | k_raw^rot] = W_dkv h         c = RMSNorm(c_raw)        k^rot = rotate(k_raw^rot)
    k_h^plain = W_uk,h c                  v_h = W_uv,h c
    score_h(i, j) = scale * (q_h^plain(i) . k_h^plain(j) + rotate(q_h^rot(i)) . k^rot(j))

Per token the cache keeps one row ``[c | k^rot]`` for all heads.  Keys and values are never
expanded: since ``q^plain . (W_uk c) = (W_uk^T q^plain) . c`` the query is moved into the latent
space (one small product per head), attention runs over the cached rows with all heads sharing
them -- the value of a row is its first ``kv_rank`` elements -- and ``W_uv`` is applied to the
attended latent.  Optional: a window (the query at position p reads rows max(0, p - window + 1) .. p)
and a learned sink per head: a logit that enters the softmax denominator as exp(sink_h), unscaled,
with nothing to attend to behind it.  ``q_rank`` 0: the queries are one product of the input, ``q = W_q h``
(no query latent).  ``gate="sigmoid"``: the heads' outputs are multiplied by sigmoid(W_g h) before the output
product.  The position part says how pairs are formed (interleaved or halves) and may scale cos and sin by
a constant (its ``magnitude``).
"""

from __future__ import annotations

import torch

from ..cache.layout import LatentLayerSpec
from ..config.spec import PartSpec
from .base import BuildContext, ParamSpec, Part, StepContext, build_part, register_part
from .linear_state import _pad_rows


class LatentAttention(Part):
    category = "mixer"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.dim = int(spec["dim"])
        self.rot_dim = int(spec["rot_dim"])
        self.vdim = int(spec["vdim"])
        self.q_rank = int(spec.get("q_rank") or 0)
        self.gate = spec.get("gate")
        if self.gate not in (None, "sigmoid"):
            raise ValueError(f"latent_attention: gate is 'sigmoid' or absent, not {self.gate!r}")
        self.kv_rank = int(spec["kv_rank"])
        self.eps = float(spec["eps"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window") or None
        self.has_sink = bool(spec.get("sink", True))
        self.position = build_part("position", spec.get("position") or PartSpec("none"), ctx)
        if self.position.style == "rotary":
            if getattr(self.position, "pairing", None) not in ("interleaved", "half") \
                    or not hasattr(self.position, "inverse_frequencies"):
                raise ValueError("latent_attention rotates pairs by angles worked out from inverse frequencies; "
                                 "the position part offers none")
            if self.position.rotary_dim > self.rot_dim:
                raise ValueError("the position part rotates more dimensions than the rotated key part has")
        elif self.position.style != "none":
            raise ValueError(f"latent_attention has no {self.position.style!r} position encoding")
        self.row_width = self.kv_rank + self.rot_dim  # one cached row: latent, then the rotated key part
        self.pairing = getattr(self.position, "pairing", "interleaved")
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        self.starts: list[int] = []
        self.down_weight = self.uq_weight = self.uk_t = self.uv = self.o_weight = None
        self.q_norm_weight = self.kv_norm_weight = self.sink = None

    def param_specs(self):
        H = self.num_heads
        specs = {
            "dq": ParamSpec((self.q_rank, self.hidden_size)),
            "dq.norm": ParamSpec((self.q_rank,), "vector"),
            "uq": ParamSpec((H * (self.dim + self.rot_dim), self.q_rank)),
            "dkv": ParamSpec((self.row_width, self.hidden_size)),
            "dkv.norm": ParamSpec((self.kv_rank,), "vector"),
            "uk": ParamSpec((H * self.dim, self.kv_rank)),
            "uv": ParamSpec((H * self.vdim, self.kv_rank)),
            "o": ParamSpec((self.hidden_size, H * self.vdim)),
        }
        if not self.q_rank:  # q = W_q h
            del specs["dq"], specs["dq.norm"], specs["uq"]
            specs = {"q": ParamSpec((H * (self.dim + self.rot_dim), self.hidden_size)), **specs}
        if self.has_sink:
            specs["sink"] = ParamSpec((H,), "vector")
        if self.gate:
            specs["g"] = ParamSpec((H * self.vdim, self.hidden_size))
        return specs

    def load(self, tensors):
        H = self.num_heads
        # one product for everything that reads the input: rows of dq (or q), then dkv, then the gate,
        # each block starting at a 16-byte column of the product
        first = tensors["dq"] if self.q_rank else tensors["q"]
        if self.q_rank and not self.gate:
            self.down_weight, self.starts = torch.cat([first, tensors["dkv"]], dim=0).contiguous(), [0, self.q_rank]
        else:
            self.down_weight, self.starts = _pad_rows([first, tensors["dkv"]] + ([tensors["g"]] if self.gate else []))
        self.uq_weight = tensors["uq"].contiguous() if self.q_rank else None
        # per head [kv_rank, dim]: the product that moves a query into the latent space contracts
        # over dim, which is the stored matrix's row index
        self.uk_t = tensors["uk"].reshape(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = tensors["uv"].reshape(H, self.vdim, self.kv_rank).contiguous()
        self.o_weight = tensors["o"].contiguous()
        self.q_norm_weight = tensors.get("dq.norm")
        self.kv_norm_weight = tensors["dkv.norm"]
        self.sink = tensors.get("sink")

    def kernel_groups(self):
        groups = ["latent_attention", "head_gemm", *self.position.kernel_groups()]
        if self.ctx.dtype == torch.float32:
            groups.append("gemm_f32")
        else:
            groups += ["gemm_small_m", "gemm_stream"]
            if self.row_width % 16 == 0 and self.kv_rank % 16 == 0 and self.kv_rank <= 512:
                groups.append("latent_attention_tc")
        return groups

    def cache_spec(self):
        return LatentLayerSpec(self.row_width, self.window)

    def position_limit(self):
        return self.position.position_limit()

    def forward(self, h: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        ops = self.ops
        T, H = h.shape[0], self.num_heads
        inv_freq = self.position.inverse_frequencies() if self.position.style == "rotary" else None
        block_table = step.block_tables[cache.paged_index]
        turn = {} if self.pairing == "interleaved" and self.magnitude == 1.0 else dict(pairing=self.pairing,
                                                                                       magnitude=self.magnitude)
        down = ops.linear(h, self.down_weight)  # [T, q_rank (or the queries) | kv_rank | rot_dim | gate]
        if self.q_rank:
            c_q = torch.empty((T, self.q_rank), dtype=h.dtype, device=h.device)
            # query latent normalised; key latent normalised, key part rotated, both written to their page
            ops.latent_norm_rope_store(
                down[:, : self.q_rank + self.row_width], q_rank=self.q_rank, kv_rank=self.kv_rank,
                rot_dim=self.rot_dim, q_weight=self.q_norm_weight,
                kv_weight=self.kv_norm_weight, eps=self.eps, inv_freq=inv_freq, positions=step.positions,
                token_seq=step.token_seq, block_table=block_table, pages=cache.latent_pages, page_size=cache.page_size,
                write=cache.writes, q_out=c_q, **turn)
            q = ops.linear(c_q, self.uq_weight).view(T, H, self.dim + self.rot_dim)
        else:
            s = self.starts
            ops.latent_norm_rope_store(
                down[:, s[1]: s[1] + self.row_width], q_rank=0, kv_rank=self.kv_rank, rot_dim=self.rot_dim,
                q_weight=None, kv_weight=self.kv_norm_weight, eps=self.eps, inv_freq=inv_freq,
                positions=step.positions, token_seq=step.token_seq, block_table=block_table,
                pages=cache.latent_pages, page_size=cache.page_size, write=cache.writes, q_out=None, **turn)
            q = down[:, : H * (self.dim + self.rot_dim)].view(T, H, self.dim + self.rot_dim)
        q_lat = torch.empty((T, H, self.row_width), dtype=h.dtype, device=h.device)
        ops.head_linear(q[:, :, : self.dim], self.uk_t, q_lat[:, :, : self.kv_rank])
        ops.rotate_heads(q[:, :, self.dim:], q_lat[:, :, self.kv_rank:], positions=step.positions, inv_freq=inv_freq,
                         **turn)
        attended = torch.empty((T, H, self.kv_rank), dtype=h.dtype, device=h.device)
        ops.latent_attention(
            q_lat, pages=cache.latent_pages, value_dim=self.kv_rank, block_table=block_table,
            token_seq=step.token_seq, positions=step.positions, sink=self.sink, out=attended,
            page_size=cache.page_size, scale=self.scale, window=self.window, step=step)
        ctx_out = torch.empty((T, H, self.vdim), dtype=h.dtype, device=h.device)
        ops.head_linear(attended, self.uv, ctx_out)
        if self.gate:
            g0 = self.starts[2]
            ops.sigmoid_mul(ctx_out.view(T, H * self.vdim), down[:, g0: g0 + H * self.vdim])
        return ops.linear(ctx_out.view(T, H * self.vdim), self.o_weight)


register_part("mixer", "latent_attention", LatentAttention)
