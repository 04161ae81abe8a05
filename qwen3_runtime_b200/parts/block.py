"""Arrangement of parts in a block.  ``pre_norm``: x += mixer(norm(x)); x += ff(norm(x))
(qwen3_runtime/models/qwen3.py:159-187, where each add is fused with the next norm); the
feed-forward may be absent, and a ``side_input`` part may add something of its own to the stream
after the sublayers.
``sandwich_norm``: a norm before and after each sublayer, x += norm_b(mixer(norm(x))) and
x += norm_b(ff(norm(x))), the feed-forward being optional.
``parallel_norms``: mixer and feed-forward read the same stream through a norm each and are added
together, x += mixer(norm_a(x)) + ff(norm_b(x)); the feed-forward is optional.
``output_norm``: the sublayers read the stream itself and only their outputs are normed,
x += norm_a(mixer(x)); x += norm_b(ff(x)); the feed-forward is optional."""

from __future__ import annotations

from .base import BuildContext, Part, ResidualStream, StepContext, build_part, register_part


class PreNormBlock(Part):
    category = "block"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.mixer = build_part("mixer", spec["mixer"], ctx)
        self.mixer_norm = build_part("norm", spec["mixer_norm"], ctx)
        self.feed_forward = self.feed_forward_norm = self.side = None
        if spec.get("feed_forward") is not None:
            self.feed_forward = build_part("feed_forward", spec["feed_forward"], ctx)
            self.feed_forward_norm = build_part("norm", spec["feed_forward_norm"], ctx)
        if spec.get("side_input") is not None:
            self.side = build_part("side_input", spec["side_input"], ctx)
        # in this order the block's tensors are listed (and a seeded random model draws them)
        named = [(spec.get("mixer_prefix", "mixer."), self.mixer),
                 (spec.get("feed_forward_prefix", "feed_forward."), self.feed_forward),
                 (spec.get("mixer_norm_prefix", "mixer_norm."), self.mixer_norm),
                 (spec.get("feed_forward_norm_prefix", "feed_forward_norm."), self.feed_forward_norm),
                 (spec.get("side_input_prefix", "side_input."), self.side)]
        self.children = {prefix: part for prefix, part in named if part is not None}
        # full name -> (part, the part's own name for it); prefixes may be prefixes of one another
        self._owners = {prefix + name: (part, name) for prefix, part in self.children.items()
                        for name in part.param_specs()}
        # the mixer's output meets this block's second norm (or, without a feed-forward, whatever
        # takes the block's output); where the last sublayer's output goes only the model knows
        # (exit_to).  A side input folds the stream with the entry norm's kernel.
        self.entry_norm = self.mixer_norm
        if self.feed_forward is not None:
            self.mixer.partial_sums_ok = self.feed_forward_norm.adds_partial_sums
        elif self.side is not None:
            self.mixer.partial_sums_ok = self.mixer_norm.adds_partial_sums
        if self.feed_forward is not None and self.side is not None:
            self.feed_forward.partial_sums_ok = self.mixer_norm.adds_partial_sums

    def exit_to(self, norms) -> None:
        """``norms``: every norm that may fold this block's output into the residual sum."""
        if self.side is not None:
            return  # what leaves the block is the side input's output, a finished product
        last = self.feed_forward if self.feed_forward is not None else self.mixer
        last.partial_sums_ok = all(n.adds_partial_sums for n in norms)

    def param_specs(self):
        return {full: part.param_specs()[name] for full, (part, name) in self._owners.items()}

    def load(self, tensors):
        per_part: dict[int, dict] = {}
        for full, (part, name) in self._owners.items():
            per_part.setdefault(id(part), {})[name] = tensors[full]
        for part in self.children.values():
            part.load(per_part.get(id(part), {}))

    def kernel_groups(self):
        return [g for part in self.children.values() for g in part.kernel_groups()]

    def step_choosers(self):
        return {name: fn for part in self.children.values() for name, fn in part.step_choosers().items()}

    def cache_spec(self):
        return self.mixer.cache_spec()

    def position_limit(self):
        limits = [n for n in (part.position_limit() for part in self.children.values()) if n is not None]
        return min(limits) if limits else None

    def forward(self, stream: ResidualStream, step: StepContext, cache) -> None:
        h = self.mixer_norm.add_norm(stream)
        stream.pending = self.mixer.forward(h, step, cache)
        if self.feed_forward is not None:
            h = self.feed_forward_norm.add_norm(stream)
            stream.pending = self.feed_forward.forward(h, step)
        if self.side is not None:
            self.side.forward(stream, step, lambda s: self.mixer_norm.add_norm(s, normalise=False))


class SandwichNormBlock(Part):
    """A norm on the input and on the output of each sublayer.  The output norms run no kernel of
    their own: the block leaves the sublayer's output on the stream together with the output
    norm's weight, and whichever norm reads the stream next (this block's second input norm, the
    next block's first, the model's final norm) normalises it, adds it and normalises the sum in
    one kernel.  ``feed_forward`` may be None: the block is its mixer alone."""

    category = "block"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.mixer = build_part("mixer", spec["mixer"], ctx)
        self.mixer_norm = build_part("norm", spec["mixer_norm"], ctx)
        self.mixer_out_norm = build_part("norm", spec["mixer_out_norm"], ctx)
        self.children = {
            spec.get("mixer_prefix", "mixer."): self.mixer,
            spec.get("mixer_norm_prefix", "mixer_norm."): self.mixer_norm,
            spec.get("mixer_out_norm_prefix", "mixer_out_norm."): self.mixer_out_norm,
        }
        self.feed_forward = self.feed_forward_norm = self.feed_forward_out_norm = None
        if spec.get("feed_forward") is not None:
            self.feed_forward = build_part("feed_forward", spec["feed_forward"], ctx)
            self.feed_forward_norm = build_part("norm", spec["feed_forward_norm"], ctx)
            self.feed_forward_out_norm = build_part("norm", spec["feed_forward_out_norm"], ctx)
            self.children.update({
                spec.get("feed_forward_prefix", "feed_forward."): self.feed_forward,
                spec.get("feed_forward_norm_prefix", "feed_forward_norm."): self.feed_forward_norm,
                spec.get("feed_forward_out_norm_prefix", "feed_forward_out_norm."): self.feed_forward_out_norm,
            })
        self.entry_norm = self.mixer_norm
        # full name -> (part, the part's own name for it); prefixes may be prefixes of one another
        self._owners = {prefix + name: (part, name) for prefix, part in self.children.items()
                        for name in part.param_specs()}

    def exit_to(self, norms) -> None:
        """A sublayer's output is normalised before it is added, so it is never taken as partial sums."""

    def param_specs(self):
        return {full: part.param_specs()[name] for full, (part, name) in self._owners.items()}

    def load(self, tensors):
        per_part: dict[int, dict] = {}
        for full, (part, name) in self._owners.items():
            per_part.setdefault(id(part), {})[name] = tensors[full]
        for part in self.children.values():
            part.load(per_part.get(id(part), {}))

    def kernel_groups(self):
        return ["norm", *[g for part in self.children.values() for g in part.kernel_groups()]]

    def step_choosers(self):
        return {name: fn for part in self.children.values() for name, fn in part.step_choosers().items()}

    def cache_spec(self):
        return self.mixer.cache_spec()

    def position_limit(self):
        limits = [n for n in (part.position_limit() for part in self.children.values()) if n is not None]
        return min(limits) if limits else None

    def forward(self, stream: ResidualStream, step: StepContext, cache) -> None:
        h = self.mixer_norm.add_norm(stream)
        stream.pending = self.mixer.forward(h, step, cache)
        stream.pending_norm = self.mixer_out_norm.pending_scale()
        if self.feed_forward is not None:
            h = self.feed_forward_norm.add_norm(stream)
            stream.pending = self.feed_forward.forward(h, step)
            stream.pending_norm = self.feed_forward_out_norm.pending_scale()


class ParallelNormsBlock(Part):
    """x += mixer(norm_a(x)) + ff(norm_b(x)).  Both norms see the same sum, so one kernel folds what is
    pending, takes the mean squares once and writes both normalised rows; the two sublayers' outputs
    are left on the stream side by side and whichever norm reads the stream next adds both."""

    category = "block"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.mixer = build_part("mixer", spec["mixer"], ctx)
        self.mixer_norm = build_part("norm", spec["mixer_norm"], ctx)
        self.children = {spec.get("mixer_prefix", "mixer."): self.mixer,
                         spec.get("mixer_norm_prefix", "mixer_norm."): self.mixer_norm}
        self.feed_forward = self.feed_forward_norm = None
        if spec.get("feed_forward") is not None:
            self.feed_forward = build_part("feed_forward", spec["feed_forward"], ctx)
            self.feed_forward_norm = build_part("norm", spec["feed_forward_norm"], ctx)
            self.children.update({spec.get("feed_forward_prefix", "feed_forward."): self.feed_forward,
                                  spec.get("feed_forward_norm_prefix", "feed_forward_norm."): self.feed_forward_norm})
        self.entry_norm = self.mixer_norm
        self._owners = {prefix + name: (part, name) for prefix, part in self.children.items()
                        for name in part.param_specs()}

    def exit_to(self, norms) -> None:
        """Two outputs leave the block side by side, both finished products."""

    def param_specs(self):
        return {full: part.param_specs()[name] for full, (part, name) in self._owners.items()}

    def load(self, tensors):
        per_part: dict[int, dict] = {}
        for full, (part, name) in self._owners.items():
            per_part.setdefault(id(part), {})[name] = tensors[full]
        for part in self.children.values():
            part.load(per_part.get(id(part), {}))

    def kernel_groups(self):
        return ["norm", *[g for part in self.children.values() for g in part.kernel_groups()]]

    def step_choosers(self):
        return {name: fn for part in self.children.values() for name, fn in part.step_choosers().items()}

    def cache_spec(self):
        return self.mixer.cache_spec()

    def position_limit(self):
        limits = [n for n in (part.position_limit() for part in self.children.values()) if n is not None]
        return min(limits) if limits else None

    def forward(self, stream: ResidualStream, step: StepContext, cache) -> None:
        if self.feed_forward is None:
            h = self.mixer_norm.add_norm(stream)
            stream.pending = self.mixer.forward(h, step, cache)
            return
        h_mixer, h_ff = self.mixer_norm.add_norm(stream, second=self.feed_forward_norm)
        stream.pending = self.mixer.forward(h_mixer, step, cache)
        stream.pending_more = self.feed_forward.forward(h_ff, step)


class OutputNormBlock(Part):
    """x += norm_a(mixer(x)); x += norm_b(ff(x)): no norm on a sublayer's input.  The output norms run no
    kernel of their own: a sublayer's output is left on the stream with its norm, and whichever kernel reads
    the stream next (this block's fold before the feed-forward, the next block's before its mixer, the model's
    final norm) normalises it, adds it to the float32 sum and hands on the sum, rounded to the activation type
    (or its norm), in one pass.  ``feed_forward`` may be None."""

    category = "block"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.mixer = build_part("mixer", spec["mixer"], ctx)
        self.mixer_out_norm = build_part("norm", spec["mixer_out_norm"], ctx)
        self.children = {spec.get("mixer_prefix", "mixer."): self.mixer,
                         spec.get("mixer_out_norm_prefix", "mixer_out_norm."): self.mixer_out_norm}
        self.feed_forward = self.feed_forward_out_norm = None
        if spec.get("feed_forward") is not None:
            self.feed_forward = build_part("feed_forward", spec["feed_forward"], ctx)
            self.feed_forward_out_norm = build_part("norm", spec["feed_forward_out_norm"], ctx)
            self.children.update({
                spec.get("feed_forward_prefix", "feed_forward."): self.feed_forward,
                spec.get("feed_forward_out_norm_prefix", "feed_forward_out_norm."): self.feed_forward_out_norm})
        self.entry_norm = self.mixer_out_norm  # the part whose kernel reads the stream first
        self._owners = {prefix + name: (part, name) for prefix, part in self.children.items()
                        for name in part.param_specs()}

    def exit_to(self, norms) -> None:
        """A sublayer's output is normalised before it is added, so it is never taken as partial sums."""

    def param_specs(self):
        return {full: part.param_specs()[name] for full, (part, name) in self._owners.items()}

    def load(self, tensors):
        per_part: dict[int, dict] = {}
        for full, (part, name) in self._owners.items():
            per_part.setdefault(id(part), {})[name] = tensors[full]
        for part in self.children.values():
            part.load(per_part.get(id(part), {}))

    def kernel_groups(self):
        return ["norm", *[g for part in self.children.values() for g in part.kernel_groups()]]

    def step_choosers(self):
        return {name: fn for part in self.children.values() for name, fn in part.step_choosers().items()}

    def cache_spec(self):
        return self.mixer.cache_spec()

    def position_limit(self):
        limits = [n for n in (part.position_limit() for part in self.children.values()) if n is not None]
        return min(limits) if limits else None

    def forward(self, stream: ResidualStream, step: StepContext, cache) -> None:
        h = self.mixer_out_norm.add_norm(stream, normalise=False)  # the stream itself
        stream.pending = self.mixer.forward(h, step, cache)
        stream.pending_norm = self.mixer_out_norm.pending_scale()
        if self.feed_forward is not None:
            h = self.feed_forward_out_norm.add_norm(stream, normalise=False)
            stream.pending = self.feed_forward.forward(h, step)
            stream.pending_norm = self.feed_forward_out_norm.pending_scale()


register_part("block", "output_norm", OutputNormBlock)
register_part("block", "pre_norm", PreNormBlock)
register_part("block", "parallel_norms", ParallelNormsBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
