"""Position encodings.  ``rope_neox``: rotate-half rotary embedding with fp32 tables
(qwen3_runtime/layers/rope.py:7-27).  ``none``: no position encoding.

A position part does not run a kernel of its own: the mixer applies it inside its
fused q/k kernel and asks the part for what that kernel needs.  The interface is

* ``style``: ``"none"`` or ``"rotary"``;
* for ``"rotary"``: :meth:`rotation_tables` -> ``(cos, sin)``, float32 ``[positions, pairs]``
  with the angle of rotation pair ``i`` at position ``p`` in ``[p, i]``; and ``pairing``, which
  two elements of a head pair ``i`` is: ``"half"`` -- ``(i, i + pairs)`` -- or
  ``"interleaved"`` -- ``(2i, 2i + 1)``.  ``2 * pairs`` may be less than the head size
  (partial rotary: the rest of the head is left as it is).

Any encoding that rotates pairs of elements by angles that depend on the absolute position
only (other frequency schedules, scaled or slowed positions, partial rotation, either
pairing) is such a part and needs no kernel change.
"""

from __future__ import annotations

import math

import torch

from .base import BuildContext, Part, register_part


class NoPosition(Part):
    category = "position"
    style = "none"

    def rotation_tables(self):
        return None


class RotaryNeox(Part):
    category = "position"
    style = "rotary"
    pairing = "half"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        # None: no tables (and no limit); the mixer's kernel works the angles out from the position
        # and device_inverse_frequencies()
        self.max_positions = int(spec["max_positions"]) if spec.get("max_positions") else None
        if self.rotary_dim < 2 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be a positive even number")

    def kernel_groups(self):
        return ["rope_kv"] if self.max_positions else []

    def position_limit(self):
        return self.max_positions

    def device_inverse_frequencies(self) -> torch.Tensor:
        """float32 ``[rotary_dim / 2]`` on the device, shared by the parts of one model."""
        key = ("rope_neox_inv", self.rotary_dim, self.theta)
        if key not in self.ctx.shared:
            self.ctx.shared[key] = self.inverse_frequencies().to(self.ctx.device)
        return self.ctx.shared[key]

    def inverse_frequencies(self) -> torch.Tensor:
        """inv_j = 1 / theta^(2j / rotary_dim), computed on the host in float32 exactly as
        the reference does (layers/rope.py:18), so both sides rotate by the same angles."""
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float) / self.rotary_dim
        return 1.0 / (self.theta ** exponents)

    def rotation_tables(self):
        if not self.max_positions:
            raise ValueError("rope_neox without max_positions keeps no tables")
        key = ("rope_neox", self.rotary_dim, self.theta, self.max_positions)
        if key not in self.ctx.shared:
            inv = self.inverse_frequencies().to(self.ctx.device)
            self.ctx.shared[key] = self.ops.rope_table(inv, self.max_positions)
        return self.ctx.shared[key]


class RotaryInterleaved(Part):
    """Pairs (2i, 2i + 1) of the first ``rotary_dim`` elements turn by ``p * theta^(-2i / rotary_dim)``.
    It keeps no table: the kernels that apply it work the angle out in float32 from the position and
    :meth:`inverse_frequencies`, so no position is out of reach.  (With ``max_positions`` it also
    offers tables, for mixers whose q/k kernel reads them.)"""

    category = "position"
    style = "rotary"
    pairing = "interleaved"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.max_positions = spec.get("max_positions")
        if self.rotary_dim < 2 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be a positive even number")

    def kernel_groups(self):
        return ["rope_kv"] if self.max_positions else []

    def position_limit(self):
        return int(self.max_positions) if self.max_positions else None

    def inverse_frequencies(self) -> torch.Tensor:
        """float32 ``[rotary_dim / 2]`` on the device, shared by the parts of one model."""
        key = ("rope_interleaved_inv", self.rotary_dim, self.theta)
        if key not in self.ctx.shared:
            exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float) / self.rotary_dim
            self.ctx.shared[key] = (1.0 / (self.theta ** exponents)).to(self.ctx.device)
        return self.ctx.shared[key]

    def rotation_tables(self):
        if not self.max_positions:
            raise ValueError("rope_interleaved without max_positions keeps no tables")
        key = ("rope_interleaved", self.rotary_dim, self.theta, int(self.max_positions))
        if key not in self.ctx.shared:
            self.ctx.shared[key] = self.ops.rope_table(self.inverse_frequencies(), int(self.max_positions))
        return self.ctx.shared[key]


class RotaryScaled(Part):
    """Rotation of the first ``rotary_dim`` elements by ``p * f_i``, f_i = theta^(-2i / rotary_dim) rescaled by a
    schedule, with either pairing and no table (the kernels work the angles out in float32 from the position
    and :meth:`inverse_frequencies`, so no position is out of reach).  ``scaling`` is None or a dictionary:

    ``kind="wavelength"`` (``factor, low, high, original``): with l = 2 pi / f, f stays where l < original / high,
    becomes f / factor where l > original / low, and in between, with s = (original / l - low) / (high - low),
    (1 - s) f / factor + s f (the schedule of Llama 3.1);
    ``kind="ramp"`` (``factor, original, fast, slow``): with index(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta),
    lo = max(floor(index(fast)), 0), hi = min(ceil(index(slow)), rotary_dim - 1) and r_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1), f_i becomes f_i / factor * r_i + f_i * (1 - r_i), and cos and sin are multiplied
    by :attr:`magnitude` = 0.1 ln(factor) + 1 (YaRN)."""

    category = "position"
    style = "rotary"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.pairing = str(spec.get("pairing", "half"))
        self.scaling = dict(spec.get("scaling") or {}) or None
        if self.rotary_dim < 2 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be a positive even number")
        if self.pairing not in ("half", "interleaved"):
            raise ValueError(f"rotation pairs are 'half' or 'interleaved', not {self.pairing!r}")
        if self.scaling is not None and self.scaling.get("kind") not in ("wavelength", "ramp"):
            raise ValueError(f"rotary_scaled: scaling kind is 'wavelength' or 'ramp', not {self.scaling.get('kind')!r}")
        self.magnitude = 1.0
        if self.scaling is not None and self.scaling["kind"] == "ramp":
            self.magnitude = 0.1 * math.log(float(self.scaling["factor"])) + 1.0

    def host_frequencies(self) -> list[float]:
        """The rescaled f_i, in double precision on the host."""
        n, base = self.rotary_dim, self.theta
        f = [base ** (-2.0 * i / n) for i in range(n // 2)]
        sc = self.scaling
        if sc is None:
            return f
        factor, original = float(sc["factor"]), float(sc["original"])
        if sc["kind"] == "wavelength":
            low, high = float(sc["low"]), float(sc["high"])
            out = []
            for fi in f:
                wave = 2.0 * math.pi / fi
                if wave < original / high:
                    out.append(fi)
                elif wave > original / low:
                    out.append(fi / factor)
                else:
                    s = (original / wave - low) / (high - low)
                    out.append((1.0 - s) * fi / factor + s * fi)
            return out

        def index_of(turns: float) -> float:
            return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(index_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(index_of(float(sc["slow"]))), n - 1)
        out = []
        for i, fi in enumerate(f):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(fi / factor * ramp + fi * (1.0 - ramp))
        return out

    def inverse_frequencies(self) -> torch.Tensor:
        """float32 ``[rotary_dim / 2]`` on the device, shared by the parts of one model."""
        key = ("rotary_scaled_inv", self.rotary_dim, self.theta, tuple(sorted((self.scaling or {}).items())))
        if key not in self.ctx.shared:
            self.ctx.shared[key] = torch.tensor(self.host_frequencies(), dtype=torch.float64).to(
                torch.float32).to(self.ctx.device)
        return self.ctx.shared[key]

    def rotation_tables(self):
        raise ValueError("rotary_scaled keeps no tables")


register_part("position", "none", NoPosition)
register_part("position", "rotary_scaled", RotaryScaled)
register_part("position", "rope_interleaved", RotaryInterleaved)
register_part("position", "rope_neox", RotaryNeox)
