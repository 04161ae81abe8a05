"""Softmax attention with grouped key/value heads, a window that keeps the sequence's first tokens, a
sink in the softmax and a gate on the heads' outputs.

    q, k, v, g = W_q h, W_k h, W_v h, W_g h              (one product)
    q, k: every head divided by its root mean square, times a weight shared by the heads (optional)
    score(i, j) = (q_i . k_j) * scale;  i sees j <= i with i - j < window or j < keep_first
    p_j = exp(s_j) / (exp(sink) + sum_j' exp(s_j'))      (``sink`` None: a plain softmax)
    out = W_o (heads' outputs * sigmoid(g))              (``gate`` None: no gate)

Keys and values may have unlike sizes per head.  The cache is a paged key/value layer whose group gives
back the pages that lie wholly between the kept first tokens and the window.  Further options:
``position`` (a rotary position part with inverse frequencies: q and k are turned after their norm, inside
the same kernel; without it positions do not enter the scores); ``softcap`` (scores become softcap *
tanh(score / softcap) after the scale); ``values="keys"`` (there is no W_v: the values are the keys as
projected, before norm and rotation); ``chunk`` (position i sees j <= i of its own chunk only, chunks of
that many tokens counted from the sequence's first token).
"""

from __future__ import annotations

import torch

from ..cache.layout import KVLayerSpec
from ..config.spec import PartSpec
from .base import BuildContext, ParamSpec, Part, StepContext, build_part, register_part
from .linear_state import _pad_rows


class SinkWindowAttention(Part):
    category = "mixer"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.dim = int(spec["dim"])
        self.vdim = int(spec["vdim"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window") or None
        self.keep_first = int(spec.get("keep_first") or 0) if self.window else 0
        self.sink = spec.get("sink")  # the sink's score (a number), or None
        self.gate = spec.get("gate")  # "sigmoid" or None
        self.qk_norm_eps = spec.get("qk_norm_eps")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.dim > 256 or self.vdim > 256:
            raise ValueError(f"dim={self.dim}, vdim={self.vdim}: the attention kernels take sizes up to 256")
        if self.gate not in (None, "sigmoid"):
            raise ValueError(f"sink_window_attention: gate is 'sigmoid' or absent, not {self.gate!r}")
        self.softcap = float(spec.get("softcap") or 0.0) or None
        self.chunk = int(spec.get("chunk") or 0) or None
        self.values_are_keys = spec.get("values", "own") == "keys"
        if spec.get("values", "own") not in ("own", "keys"):
            raise ValueError(f"sink_window_attention: values are 'own' or 'keys', not {spec.get('values')!r}")
        if self.values_are_keys and self.vdim != self.dim:
            raise ValueError("sink_window_attention: values that are the keys have the keys' size")
        if self.chunk and self.window:
            raise ValueError("sink_window_attention: a window or chunks, not both")
        self.position = build_part("position", spec.get("position") or PartSpec("none"), ctx)
        if self.position.style == "rotary":
            if not hasattr(self.position, "inverse_frequencies") or self.position.rotary_dim > self.dim:
                raise ValueError("sink_window_attention turns q and k by angles worked out from inverse "
                                 "frequencies over at most the head's size; the position part offers otherwise")
        elif self.position.style != "none":
            raise ValueError(f"sink_window_attention has no {self.position.style!r} position encoding")
        self.in_weight = self.o_weight = self.q_norm = self.k_norm = None
        self._tables = None
        self.starts: list[int] = []

    def param_specs(self):
        H, G, D, Dv, W = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.hidden_size
        specs = {"q": ParamSpec((H * D, W)), "k": ParamSpec((G * D, W)), "v": ParamSpec((G * Dv, W)),
                 "o": ParamSpec((W, H * Dv))}
        if self.values_are_keys:
            del specs["v"]
        if self.gate:
            specs["g"] = ParamSpec((H * Dv, W))
        if self.qk_norm_eps is not None:
            specs["q.norm"] = ParamSpec((D,), "vector")
            specs["k.norm"] = ParamSpec((D,), "vector")
        return specs

    def load(self, tensors):
        if self.values_are_keys:  # no W_v: the value heads are read where the key heads are
            self.in_weight, starts = _pad_rows([tensors["q"], tensors["k"]] + ([tensors["g"]] if self.gate else []))
            self.starts = [starts[0], starts[1], starts[1], *starts[2:]]
        else:
            blocks = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.gate else [])
            self.in_weight, self.starts = _pad_rows(blocks)
        self.o_weight = tensors["o"].contiguous()
        self.q_norm = tensors.get("q.norm")
        self.k_norm = tensors.get("k.norm")

    def kernel_groups(self):
        groups = ["rope_kv", "attention_generic"]
        groups += ["gemm_f32"] if self.ctx.dtype == torch.float32 else ["gemm_small_m", "gemm_stream"]
        if self._specialised():
            groups += ["attention_decode"] + (["attention_prefill"] if self.dim in (64, 128) else [])
        return groups

    def _specialised(self) -> bool:
        """Keys and values of one size that the split-KV decode kernel (64, 128, 256) and the tensor-core prompt
        kernel (64, 128) take (ops.paged_attention sends a dense output there), with the window's kept first tokens, the
        sink, the gate and capped scores."""
        return (self.ctx.dtype == torch.bfloat16 and self.dim == self.vdim and self.dim in (64, 128, 256)
                and self.num_heads // self.num_kv_heads <= 16 and not self.chunk)

    # positions for which the decode kernel that also makes the newest token's q and k keeps rotation tables;
    # steps that reach beyond run the q/k kernel (which needs none) and the plain decode kernel
    FUSED_POSITIONS = 32768

    def _fused_tables(self):
        """cos and sin ``[FUSED_POSITIONS, dim / 2]`` for the decode kernel that norms, turns and stores the newest
        token itself: the part's frequencies followed by zeros (pairs that do not turn), times the magnitude.
        None when this rotation cannot be put that way (halves pairing over a part of the head)."""
        if self._tables is None:
            pos = self.position
            inv = pos.inverse_frequencies()
            if pos.pairing == "half" and 2 * inv.numel() != self.dim:
                self._tables = False
            else:
                padded = torch.zeros(self.dim // 2, dtype=torch.float32, device=inv.device)
                padded[: inv.numel()] = inv
                cos, sin = self.ops.rope_table(padded, self.FUSED_POSITIONS)
                magnitude = float(getattr(pos, "magnitude", 1.0))
                if magnitude != 1.0:
                    cos, sin = cos * magnitude, sin * magnitude
                self._tables = (cos, sin)
        return self._tables or None

    def _slices_key(self):
        reach = self.window + self.keep_first if self.window else None  # the most keys a token sees
        return ("decode_slices", self.num_kv_heads, self.dim, reach)

    def step_choosers(self):
        """Into how many slices the split-KV decode kernel cuts the longest sequence's keys."""
        model = getattr(self.ops, "decode_slices_for", None)
        if model is None or not self._specialised():
            return {}
        key = self._slices_key()
        return {key: lambda kv_lens: model(kv_lens, key[1], key[2], key[3])}

    def cache_spec(self):
        return KVLayerSpec(self.num_kv_heads, self.dim, self.window, value_dim=self.vdim, keep_first=self.keep_first,
                           chunk=self.chunk)

    def position_limit(self):
        return self.position.position_limit()

    def forward(self, h: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        ops = self.ops
        H, G, D, Dv = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        s = self.starts
        proj = ops.linear(h, self.in_weight)
        block_table = step.block_tables[cache.paged_index]
        ctx = torch.empty((h.shape[0], H * Dv), dtype=h.dtype, device=h.device)
        gate = proj[:, s[3]:s[3] + H * Dv] if self.gate else None
        fusable = getattr(ops, "decode_new_token_ok", None)
        rotary = self.position.style == "rotary"
        tables = None
        if (fusable is not None and step.decode_only and cache.writes and self._specialised() and rotary
                and (step.captured_width * cache.page_size or step.max_kv_len) <= self.FUSED_POSITIONS):
            tables = self._fused_tables()
        cos, sin = tables if tables is not None else (None, None)
        if (fusable is not None and step.decode_only and cache.writes and self._specialised()
                and (not rotary or tables is not None)
                # q, k and v heads side by side, as that kernel reads them (v where k is, if the values are the keys)
                and s[1] == H * D and s[2] == (H * D if self.values_are_keys else (H + G) * D)
                and fusable(proj, num_heads=H, num_kv_heads=G, head_dim=D, cos=cos, q_weight=self.q_norm,
                            k_weight=self.k_norm)):
            # one kernel: norm (and rotation) of the newest q and k, cache write, split-KV attention with sink, gate
            # and capped scores
            width = step.captured_width
            ops.paged_attention_decode(
                proj, proj.stride(0), num_heads=H, num_kv_heads=G, head_dim=D, k_pages=cache.k_pages,
                v_pages=cache.v_pages, block_table=block_table, kv_lens=step.kv_lens, cu_seqlens=step.cu_seqlens,
                out=ctx, page_size=cache.page_size, scale=self.scale, window=self.window, num_seqs=step.num_seqs,
                max_kv_len=width * cache.page_size or step.max_kv_len,
                new_token=dict(q_weight=self.q_norm, k_weight=self.k_norm,
                               eps=self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, cos=cos, sin=sin,
                               pairing=getattr(self.position, "pairing", "half"),
                               values_are_keys=self.values_are_keys),
                num_splits=step.choices.get(self._slices_key()), longest=step.kv_longest, step=step,
                keep_first=self.keep_first, sink=self.sink, gate=gate, softcap=self.softcap)
            return ops.linear(ctx, self.o_weight)
        ops.qk_norm_store(proj, num_heads=H, num_kv_heads=G, head_dim=D, value_dim=Dv, k_start=s[1], v_start=s[2],
                          q_weight=self.q_norm, k_weight=self.k_norm,
                          eps=self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, positions=step.positions,
                          token_seq=step.token_seq, block_table=block_table, k_pages=cache.k_pages,
                          v_pages=cache.v_pages, page_size=cache.page_size, write_kv=cache.writes,
                          **(dict(inv_freq=self.position.inverse_frequencies(), pairing=self.position.pairing,
                                  magnitude=getattr(self.position, "magnitude", 1.0)) if rotary else {}))
        ops.paged_attention(proj, proj.stride(0), num_heads=H, num_kv_heads=G, head_dim=D, k_pages=cache.k_pages,
                            v_pages=cache.v_pages, block_table=block_table, token_seq=step.token_seq,
                            positions=step.positions, out=ctx, page_size=cache.page_size, scale=self.scale,
                            window=self.window, step=step, value_dim=Dv, keep_first=self.keep_first, sink=self.sink,
                            gate=gate, decode_slices=step.choices.get(self._slices_key()),
                            **(dict(chunk=self.chunk, softcap=self.softcap) if self.chunk or self.softcap else {}))
        return ops.linear(ctx, self.o_weight)


register_part("mixer", "sink_window_attention", SinkWindowAttention)
