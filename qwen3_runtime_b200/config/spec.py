"""Architecture-neutral description of a model as data.

A model is a list of blocks, each made of parts (mixer, feed-forward, norms,
position encoding), and a *run order*: which block runs when and which cache it
reads and writes.  Parts are named by ``kind`` and carry their own sizes and
constants, so one model may use different mixers or feed-forwards in different
layers, and no part knows which model it is in.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered ``kind`` and the parameters that part understands."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerRun:
    """One entry of the run order.

    ``block`` indexes ``ModelSpec.blocks`` (a block may be named twice: its
    weights are shared).  ``cache`` is the id of the cache layer the mixer uses;
    two entries with the same ``cache`` share keys and values.  ``writes`` says
    whether this entry stores its own keys/values (or state) there or only reads
    what an earlier entry stored.  ``add_embedding``: the embedding output (the
    residual stream as it was before the first entry) is added to the stream right
    before this entry runs (a looped stack that is fed its input again).  ``add_row``
    ``(table, row)``: row ``row`` of the model's shared table ``table`` (``ModelSpec.shared_tables``),
    one vector of the model's width, is added to every token of the stream right before this
    entry runs (a learned vector per pass of a loop).  ``mix_source``: the name of a shared table
    ``[width, 2 * width]``; right before this entry runs the stream becomes that matrix times
    ``[stream; embedding output]`` (a looped stack whose every pass is fed the model's input again
    through a learned projection).
    """

    block: int
    cache: int
    writes: bool = True
    add_embedding: bool = False
    add_row: tuple[str, int] | None = None
    mix_source: str | None = None


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    blocks: tuple[PartSpec, ...]
    order: tuple[LayerRun, ...]
    final_norm: PartSpec
    tie_word_embeddings: bool
    embed_name: str = "model.embed_tokens.weight"
    head_name: str = "lm_head.weight"
    block_prefix: str = "model.layers.{index}."
    # each block's own prefix, for models whose stored blocks are not numbered 0, 1, 2, ... (None: block_prefix)
    block_names: tuple[str, ...] | None = None
    final_norm_prefix: str = "model.norm."
    # the head's epilogue: logits * logit_scale, then (if set) softcap * tanh(logits / softcap)
    logit_scale: float = 1.0
    logit_softcap: float | None = None
    # stored tensors that belong to no block: checkpoint name -> (shape, kind as in ParamSpec).  The
    # model loads them into ``BuildContext.shared`` under their names, where parts (a second embedding
    # that every block reads a slice of) and run entries (``LayerRun.add_row``) find them.
    shared_tables: tuple[tuple[str, tuple[int, ...], str], ...] = ()
    # An ``embedding`` part that makes the stream's first value from the step's tokens (and may keep
    # state per request, e.g. the previous token).  None: a plain lookup in ``embed_name``, done by the
    # first norm.  The part's tensors are stored under their own names (no prefix).
    embedding: PartSpec | None = None

    def __post_init__(self) -> None:
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ValueError("logit_softcap must be positive (or None)")
        if self.block_names is not None and len(self.block_names) != len(self.blocks):
            raise ValueError("block_names: one prefix per block")
        writers: set[int] = set()
        for run in self.order:
            if not 0 <= run.block < len(self.blocks):
                raise ValueError(f"run order names block {run.block}; the model has {len(self.blocks)}")
            if run.writes:
                if run.cache in writers:
                    raise ValueError(f"cache layer {run.cache} is written by two run entries")
                writers.add(run.cache)
            elif run.cache not in writers:
                raise ValueError(f"run entry reads cache layer {run.cache} before any entry writes it")
            if run.add_row is not None and run.add_row[0] not in {name for name, _s, _k in self.shared_tables}:
                raise ValueError(f"run entry adds a row of {run.add_row[0]!r}, which is no shared table of the model")
            if run.mix_source is not None and run.mix_source not in {name for name, _s, _k in self.shared_tables}:
                raise ValueError(f"run entry mixes through {run.mix_source!r}, which is no shared table of the model")

    def prefix_of(self, index: int) -> str:
        """The prefix of block ``index``'s stored tensors."""
        return self.block_names[index] if self.block_names is not None else self.block_prefix.format(index=index)

    @staticmethod
    def sequential_order(num_blocks: int) -> tuple[LayerRun, ...]:
        return tuple(LayerRun(block=i, cache=i) for i in range(num_blocks))
