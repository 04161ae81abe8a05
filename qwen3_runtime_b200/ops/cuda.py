"""The kernel table of the engine: thin Python wrappers over the ``extern "C"``
launchers in ``csrc/``.

There is one implementation per operation and no fallback: constructing
:class:`CudaOps` without a CUDA device, or without a working nvcc to build the
kernels, raises.  Wrappers check sizes and refuse, with a clear message, what a
kernel does not support; they never substitute another code path silently.
"""

from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_long, c_void_p

import torch

from . import build

_CODES = {1: "unsupported size or option", 2: "CUDA launch failed", 3: "bad argument"}


class KernelError(RuntimeError):
    pass


class KernelsUnavailable(RuntimeError):
    pass


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels exist for float32 and bfloat16, not {dtype}")


def _check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what}: {_CODES.get(code, code)}")


_SIGNATURES = {
    "norm": {
        "q3_fused_norm": [c_int, c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "q3_silu_mul": [c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "q3_add_bias": [c_int, c_void_p, c_long, c_void_p, c_int, c_int, c_void_p],
        "q3_logit_scale_cap": [c_void_p, c_long, c_float, c_float, c_void_p],
        "q3_fused_post_norm": [c_int, c_void_p, c_int, c_long, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p],
        "q3_sigmoid_mul": [c_int, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p],
        "q3_gelu_gate_rows": [c_int, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p, c_int, c_int,
                              c_void_p],
        "q3_relu_squared": [c_int, c_void_p, c_long, c_void_p, c_int, c_int, c_void_p],
        "q3_clamped_glu": [c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float, c_void_p],
        "q3_grouped_norm": [c_int, c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_long, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "q3_tanh_rows": [c_int, c_void_p, c_long, c_void_p],
    },
    "token_state": {
        "q3_bigram_embed": [c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_long, c_long, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_int,
                            c_void_p],
        "q3_token_shift_mix": [c_int, c_void_p, c_long, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    },
    "latent_attention": {
        "q3_latent_norm_rope_store": [c_int, c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                                      c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                      c_int, c_void_p, c_int, c_float, c_void_p],
        "q3_rotate_heads": [c_int, c_void_p, c_long, c_long, c_void_p, c_long, c_long, c_void_p, c_void_p, c_int,
                            c_int, c_int, c_int, c_int, c_float, c_void_p],
        "q3_latent_attention": [c_int, c_void_p, c_long, c_long, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_long, c_long, c_int, c_int, c_int, c_float, c_int,
                                c_void_p],
    },
    "latent_attention_tc": {
        "q3_latent_attention_tc": [c_void_p, c_long, c_long, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_long, c_long, c_int, c_int, c_int, c_int, c_float,
                                   c_int, c_int, c_void_p, c_void_p],
    },
    "head_gemm": {
        "q3_head_linear": [c_int, c_void_p, c_long, c_long, c_void_p, c_void_p, c_long, c_long, c_int, c_int, c_int,
                           c_int, c_void_p],
    },
    "experts": {
        "q3_route_top": [c_int, c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                         c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "q3_group_slots": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
        "q3_expert_gate_up_tc": [c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_float, c_void_p],
        "q3_expert_down_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                              c_void_p, c_void_p],
        "q3_expert_gate_up": [c_int, c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_int, c_float, c_float, c_float, c_void_p],
        "q3_expert_down": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                           c_void_p, c_void_p],
        "q3_expert_combine": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_int, c_int, c_int,
                              c_void_p, c_int, c_void_p, c_long, c_void_p],
        "q3_expert_up": [c_int, c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                         c_void_p, c_void_p, c_int, c_void_p],
        "q3_expert_up_tc": [c_void_p, c_long, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                            c_void_p, c_void_p, c_int, c_void_p],
    },
    "rope_kv": {
        "q3_qk_norm_rope_store": [c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                                  c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "q3_rope_table": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "q3_qk_norm_store": [c_int, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                             c_void_p, c_float, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p,
                             c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    },
    "attention_generic": {
        "q3_paged_attention_generic": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                       c_void_p, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                       c_int, c_int, c_int, c_float, c_void_p, c_long, c_int, c_float, c_void_p],
        "q3_paged_attention_diff": [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                    c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                    c_float, c_float, c_float, c_void_p],
    },
    "attention_diff": {
        "q3_diff_attention_prefill": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                      c_void_p, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                      c_int, c_int, c_float, c_float, c_float, c_void_p],
        "q3_diff_attention_decode": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                     c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                     c_int, c_int, c_int, c_float, c_float, c_float, c_void_p],
    },
    "linear_state": {
        "q3_decayed_state_scan": [c_int, c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_void_p, c_long,
                                  c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_float, c_float, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                  c_int, c_void_p, c_void_p],
        "q3_head_norm_gate": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_long, c_void_p, c_long,
                              c_float, c_int, c_int, c_int, c_int, c_void_p],
        "q3_stabilised_gates": [c_int, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    },
    "short_conv": {
        "q3_conv_rope_store": [c_int, c_void_p, c_long, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "q3_conv_state_update": [c_int, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    },
    "attention_decode": {
        "q3_paged_attention_decode": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                      c_float, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "q3_paged_attention_decode_sink": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p,
                                           c_int, c_float, c_void_p],
        "q3_paged_attention_decode_fused": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                            c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_float,
                                            c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
        "q3_paged_attention_decode_fused_sink": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                 c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_float,
                                                 c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_int, c_float, c_void_p, c_int, c_float, c_int, c_void_p],
    },
    "attention_prefill": {
        "q3_paged_attention_prefill": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                       c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                       c_void_p],
        "q3_paged_attention_prefill_sink": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                            c_int, c_int, c_float, c_void_p, c_int, c_float, c_void_p],
    },
    "attention_prefill_tc": {
        "q3_paged_attention_prefill_tc": [c_void_p, c_int, c_int, c_void_p, c_void_p, ctypes.c_long, c_void_p, c_int,
                                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_float, c_int, c_void_p, c_void_p],
    },
    "gemm_f32": {
        "q3_gemm_f32": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "gemm_small_m": {
        "q3_gemm_small_m": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "gemm_stream": {
        "q3_gemm_stream": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                           c_void_p, c_void_p],
        "q3_gemm_stream_parts": [c_int, c_int, c_int],
        "q3_gemm_stream_partial": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                   c_void_p, c_void_p],
    },
    "gemm_tcgen05": {
        "q3_gemm_tcgen05": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                            c_void_p],
        "q3_gemm_tcgen05_pair": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                 c_void_p, c_void_p],
    },
    "sampling": {
        "q3_argmax": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "q3_sample": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                      c_void_p],
        "q3_bias_penalty": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_float, c_float,
                            c_float, c_void_p],
        "q3_bias_penalty_rows": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p],
        "q3_filter": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    },
}


class _Span:
    """CUDA events around one launch, appended to the kernel table's timing records."""

    def __init__(self, ops, what: str):
        self.ops, self.what = ops, what

    def __enter__(self):
        self.start, self.stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.start.record()
        return self

    def __exit__(self, *exc):
        self.stop.record()
        nbytes, flops, tag = self.ops._cost
        self.ops._cost = (0, 0, "")
        self.ops.timing.append((self.what + tag, self.start, self.stop, nbytes, flops))
        return False


class CudaOps:
    """Kernels on the current CUDA device.  ``groups`` are compiled up front (in
    parallel); any other group is compiled when first used."""

    name = "cuda-sm100a"

    def __init__(self, groups: list[str] | None = None, large_gemm: str = "auto"):
        """``large_gemm`` picks the bfloat16 product for more than 16 tokens: ``"tcgen05"`` -- this
        engine's tcgen05/TMEM kernel for every such product; ``"library"`` -- the library's;
        ``"auto"`` (default) -- the tcgen05 kernel where it is at least as fast as the library
        on a B200 (the fused SwiGLU product of prompt-sized batches), the library elsewhere."""
        if large_gemm not in ("auto", "tcgen05", "library"):
            raise ValueError("large_gemm must be auto, tcgen05 or library")
        self.large_gemm = large_gemm
        self.prefill_attention = "tcgen05"  # "mma" keeps every prompt portion on the mma.sync kernel
        self.tcgen05_pairs = True           # False: the tcgen05 product never pairs SMs (cta_group::1 only)
        self.fuse_decode_new_token = True   # False: always the separate q/k norm + rotation + store kernel
        self.latent_attention_tc = True     # False: attention over latent rows always on the general kernel
        self.experts_tc = True              # False: the experts' products always on the FMA kernels
        self.differential_tc = True         # False: differential attention always on the general kernel
        self._tickets: torch.Tensor | None = None
        self._argmax_tickets: torch.Tensor | None = None
        # products of at most 16 tokens: "auto" -- the shared-memory stream (csrc/gemm_stream.cu) for the
        # large ones, the register stream (csrc/gemm_small_m.cu) for the rest; "stream" -- the first
        # for everything it supports; "registers" -- always the second
        self.small_gemm = "auto"
        # True: a product whose result a norm folds into the residual sum may come as fp32 partial
        # sums over ranges of K (linear(partial_sums=True)); False: always a finished product
        self.partial_sums = True
        self._parts_cache: dict[tuple, int] = {}
        self._slices_cache: dict[tuple, int] = {}
        if not torch.cuda.is_available():
            raise KernelsUnavailable(
                "qwen3_runtime_b200 runs on a CUDA device only (built for NVIDIA B200, sm_100a); "
                "no CUDA device is visible and there is no CPU path"
            )
        major, _minor = torch.cuda.get_device_capability()
        if major != 10:
            raise KernelsUnavailable(
                f"the kernels are compiled for sm_100a; this device reports sm_{major}{_minor}"
            )
        self._device_index = torch.cuda.current_device()
        self.SM_COUNT = torch.cuda.get_device_properties(self._device_index).multi_processor_count
        self._fn: dict[str, ctypes._CFuncPtr] = {}
        self.launches = 0  # kernels of this engine launched (or captured) through this table
        # Per-kernel timing, off by default: a list makes every launch through this table record
        # (kernel, start event, stop event, algorithmic bytes, flops) into it; see timed_kernels().
        self.timing: list | None = None
        self._cost = (0, 0, "")
        if groups:
            build.compile_groups([g for g in groups])

    def prepare(self, groups: list[str]) -> None:
        """Compile (in parallel) the kernel groups a model is going to use."""
        build.compile_groups([g for g in groups if g in _SIGNATURES])

    # ---- plumbing -------------------------------------------------------------------
    def _get(self, group: str, name: str):
        fn = self._fn.get(name)
        if fn is None:
            lib = build.load_group(group)
            fn = getattr(lib, name)
            fn.argtypes = _SIGNATURES[group][name]
            fn.restype = c_int
            self._fn[name] = fn
        return fn

    def _stream(self) -> int:
        """The current stream's handle.  Asked for at every launch (a captured step runs on another
        stream than an eager one), so through the raw query: ``torch.cuda.current_stream()`` builds
        a Stream object and looks the device up again each time, several microseconds a call."""
        if _raw_stream is not None:
            return _raw_stream(self._device_index)
        return torch.cuda.current_stream().cuda_stream

    def _call(self, group: str, name: str, what: str, *args) -> None:
        self.launches += 1
        if self.timing is not None:
            with self._timed(what):
                _check(self._get(group, name)(*args, self._stream()), what)
            return
        _check(self._get(group, name)(*args, self._stream()), what)

    # ---- per-kernel timing (a debugging and reporting aid; never on in a timed run) ------------
    def _costs(self, nbytes: float, flops: float = 0.0, tag: str = "") -> None:
        """What the next launch has to move and compute (and a tag that tells launches of one
        kernel apart, e.g. the sizes of a product), for the timing records."""
        self._cost = (float(nbytes), float(flops), tag)

    def _timed(self, what: str):
        return _Span(self, what)

    def timed_kernels(self) -> list[dict]:
        """Sum the records of :attr:`timing` per kernel: launches, microseconds (CUDA events around
        each launch, so kernels do not overlap their neighbours as they do in a captured step),
        algorithmic bytes and flops.  Waits for the device."""
        torch.cuda.synchronize()
        table: dict[str, dict] = {}
        for what, start, stop, nbytes, flops in self.timing or []:
            row = table.setdefault(what, dict(name=what, launches=0, us=0.0, bytes=0.0, flops=0.0))
            row["launches"] += 1
            row["us"] += start.elapsed_time(stop) * 1e3
            row["bytes"] += nbytes
            row["flops"] += flops
        return sorted(table.values(), key=lambda r: -r["us"])

    # ---- norms ----------------------------------------------------------------------
    def fused_norm(self, out, weight, eps, *, resid=None, pending=None, ids=None, table=None, rows=None,
                   write_resid=True, num_rows=None, post_weight=None, post_eps=0.0, add_ids=None, add_table=None,
                   add_vector=None, center=False, post_center=False):
        """RMSNorm of ``resid (+ pending)`` or of ``table[ids] (+ pending)``; see csrc/norm.cu.
        ``center`` / ``post_center``: the sum's norm / the pending output's norm is a layer norm with a
        weight and no bias (the mean is taken off and the variance is the mean squared deviation).
        ``pending`` is ``[rows, H]`` of the output's type, or fp32 ``[parts, rows, H]``: the
        partial sums of a product (:meth:`linear` with ``partial_sums``), added in order.
        ``post_weight`` / ``post_eps``: what is pending is RMS-normalised with this weight before it
        is added; ``add_ids`` / ``add_table``: embedding rows added to the sum as well;
        ``add_vector`` (float32 ``[H]``): added to every row's sum.  ``weight=None``: nothing is
        normalised, ``out`` gets the sum itself, rounded to its type."""
        H = out.shape[-1]
        n = out.shape[0] if num_rows is None else num_rows
        vocab = table.shape[0] if table is not None else 0
        if add_vector is not None and (add_vector.dtype != torch.float32 or add_vector.numel() != H
                                       or not add_vector.is_contiguous()):
            raise KernelError("fused_norm: add_vector is a dense float32 vector of the rows' width")
        if (post_weight is not None or add_ids is not None or add_vector is not None or weight is None
                or center or post_center):
            pparts = pstride = 0
            if pending is not None and pending.dim() == 3:
                if pending.dtype != torch.float32 or pending.stride(2) != 1 or pending.stride(1) != H:
                    raise KernelError("fused_norm: partial sums are fp32 [parts, rows, H] with dense rows")
                pparts, pstride = pending.shape[0], pending.stride(0)
            elif pending is not None and (pending.dtype != out.dtype or not pending.is_contiguous()):
                raise KernelError("fused_norm: a pending output that is normalised first is dense [rows, H] "
                                  "of the output's type")
            if add_table is not None:
                vocab = add_table.shape[0]
            if self.timing is not None:
                e = out.element_size()
                self._costs(n * H * (2 * e + (4 if resid is not None else 0) + (4 if write_resid else 0)
                                     + (e if add_ids is not None or table is not None else 0)))
            self._call("norm", "q3_fused_post_norm", "fused_post_norm", _dtype_code(out.dtype), _ptr(pending),
                       pparts, pstride, _ptr(post_weight), float(post_eps), _ptr(resid), _ptr(ids), _ptr(table), _ptr(add_ids),
                       _ptr(add_table), _ptr(add_vector), _ptr(rows), _ptr(weight), _ptr(out), n, H, float(eps),
                       int(bool(write_resid)), vocab, int(bool(post_center)) | (int(bool(center)) << 1))
            return out
        parts = stride = 0
        if pending is not None and pending.dim() == 3:
            if pending.dtype != torch.float32 or pending.stride(2) != 1 or pending.stride(1) != H:
                raise KernelError("fused_norm: partial sums are fp32 [parts, rows, H] with dense rows")
            parts, stride = pending.shape[0], pending.stride(0)
        elif pending is not None and pending.dtype != out.dtype:
            raise KernelError(f"fused_norm: pending is {pending.dtype}, the output {out.dtype}")
        if self.timing is not None:
            e = out.element_size()
            self._costs(n * H * (e + (4 if resid is not None else 0) + (4 if write_resid else 0)
                                 + (4 * parts if parts else (e if pending is not None else 0))
                                 + (table.element_size() if table is not None else 0)))
        self._call("norm", "q3_fused_norm", "fused_norm",
                   _dtype_code(out.dtype), _ptr(pending), parts, stride, _ptr(resid), _ptr(ids), _ptr(table), _ptr(rows),
                  _ptr(weight), _ptr(out), n, H, float(eps), int(bool(write_resid)), vocab)
        return out

    def grouped_norm(self, out, weight, eps, groups, *, resid, pending=None, pending_more=None, rows=None,
                     write_resid=True, num_rows=None, out2=None, weight2=None):
        """RMSNorm in ``groups`` equal consecutive parts of ``resid + pending + pending_more`` (each part divided
        by its own root mean square, the weight spanning the row), float32 throughout; see csrc/norm.cu.
        ``pending``: ``[rows, H]`` of the output's type or fp32 partial sums ``[parts, rows, H]``;
        ``pending_more``: ``[rows, H]`` of the output's type.  ``out2`` / ``weight2``: a second normalised copy
        of the same rows with another weight.  ``weight=None``: ``out`` (rows may be views of wider rows) gets
        the sum itself, rounded."""
        H = resid.shape[-1]
        n = out.shape[0] if num_rows is None else num_rows
        if resid.dtype != torch.float32 or not resid.is_contiguous() or out.shape[-1] != H or out.stride(-1) != 1:
            raise KernelError("grouped_norm: a dense float32 residual sum and output rows of its width")
        parts = stride = 0
        if pending is not None and pending.dim() == 3:
            if pending.dtype != torch.float32 or pending.stride(2) != 1 or pending.stride(1) != H:
                raise KernelError("grouped_norm: partial sums are fp32 [parts, rows, H] with dense rows")
            parts, stride = pending.shape[0], pending.stride(0)
        elif pending is not None and (pending.dtype != out.dtype or not pending.is_contiguous()):
            raise KernelError("grouped_norm: a pending output is dense [rows, H] of the output's type")
        if pending_more is not None and (pending_more.dtype != out.dtype or not pending_more.is_contiguous()):
            raise KernelError("grouped_norm: a second pending output is dense [rows, H] of the output's type")
        if out2 is not None and (weight2 is None or weight is None or not out2.is_contiguous()
                                 or out2.dtype != out.dtype):
            raise KernelError("grouped_norm: a second output is dense, of the first one's type, with a weight of its own")
        for w in (weight, weight2):
            if w is not None and (w.dtype != torch.float32 or w.numel() != H or not w.is_contiguous()):
                raise KernelError("grouped_norm: weights are dense float32 vectors of the rows' width")
        if self.timing is not None:
            e = out.element_size()
            self._costs(n * H * (4 + (4 if write_resid else 0) + e * (1 + (out2 is not None))
                                 + (4 * parts if parts else (e if pending is not None else 0))
                                 + (e if pending_more is not None else 0)))
        self._call("norm", "q3_grouped_norm", "grouped_norm", _dtype_code(out.dtype), _ptr(pending), parts, stride,
                   _ptr(pending_more), _ptr(resid), _ptr(rows), _ptr(weight), _ptr(weight2), _ptr(out), out.stride(0),
                   _ptr(out2), n, H, int(groups), float(eps), int(bool(write_resid)))
        return out

    def tanh_rows(self, x):
        """``x = tanh(x)`` in place (float32 math, one rounding)."""
        if not x.is_contiguous():
            raise KernelError("tanh_rows: a dense tensor")
        self._call("norm", "q3_tanh_rows", "tanh_rows", _dtype_code(x.dtype), _ptr(x), x.numel())
        return x

    # ---- what a layer keeps of a sequence's previous token (csrc/token_state.cu) -----------------
    def bigram_embed(self, ids, *, embed, scale, bigram, buckets, mul_prev, mul_cur, prev_state, positions,
                     token_seq, cu_seqlens, state_slots, num_seqs, out, copy=None):
        """``out[t] = embed[id_t] * scale + bigram[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets]`` (float32
        rows; row ``buckets`` for a sequence's first token); the token before a step's first comes from
        ``prev_state`` (int32 ``[slots, 1]``), which then takes the step's last token.  ``copy``: the same rows
        in the tables' type (may be a view of wider rows).  ``bigram=None``: the scaled lookup alone."""
        T, W = out.shape
        if out.dtype != torch.float32 or not out.is_contiguous() or not embed.is_contiguous() or embed.shape[1] != W:
            raise KernelError("bigram_embed: dense float32 output rows of the table's width")
        if bigram is not None and (bigram.dtype != embed.dtype or bigram.shape != (buckets + 1, W)
                                   or not bigram.is_contiguous() or prev_state is None
                                   or prev_state.dtype != torch.int32 or not prev_state.is_contiguous()):
            raise KernelError("bigram_embed: a dense bigram table [buckets + 1, width] of the embedding's type and "
                              "an int32 slot per request")
        if copy is not None and (copy.dtype != embed.dtype or copy.stride(1) != 1 or copy.shape != (T, W)):
            raise KernelError("bigram_embed: the copy has the tables' type and unit-stride rows")
        if self.timing is not None:
            e = embed.element_size()
            self._costs(T * W * (4 + e * (1 + (bigram is not None) + (copy is not None))))
        self.launches += int(bigram is not None)  # the slot's update is a kernel of its own
        self._call("token_state", "q3_bigram_embed", "bigram_embed", _dtype_code(embed.dtype), _ptr(ids), _ptr(embed),
                   float(scale), _ptr(bigram), int(buckets), int(mul_prev), int(mul_cur), _ptr(prev_state),
                   _ptr(positions), _ptr(token_seq), _ptr(cu_seqlens), _ptr(state_slots), _ptr(out), _ptr(copy),
                   copy.stride(0) if copy is not None else 0, T, int(num_seqs), W, embed.shape[0])
        return out

    def token_shift_mix(self, h, mu, *, state, positions, token_seq, cu_seqlens, state_slots, num_seqs):
        """``y[s, t] = h[t] + (h[t-1] - h[t]) * mu[s]`` for each row s of ``mu`` (float32 ``[n, W]``), h[-1] = 0
        for a sequence's first token; the row before a step's first comes from ``state`` (float32
        ``[slots, W]``), which then takes the step's last row.  Returns ``[n, T, W]`` of h's type."""
        T, W = h.shape
        n = mu.shape[0]
        if h.stride(1) != 1 or mu.dtype != torch.float32 or not mu.is_contiguous() or mu.shape[1] != W:
            raise KernelError("token_shift_mix: unit-stride rows and dense float32 blends [n, width]")
        if state.dtype != torch.float32 or not state.is_contiguous() or state.shape[1:] != (W,):
            raise KernelError("token_shift_mix: the state is dense float32 [slots, width]")
        out = torch.empty((n, T, W), dtype=h.dtype, device=h.device)
        if self.timing is not None:
            self._costs(T * W * h.element_size() * (n + 1))
        self.launches += 1  # the slot's update is a kernel of its own
        self._call("token_state", "q3_token_shift_mix", "token_shift_mix", _dtype_code(h.dtype), _ptr(h), h.stride(0),
                   _ptr(mu), n, _ptr(state), _ptr(positions), _ptr(token_seq), _ptr(cu_seqlens), _ptr(state_slots),
                   _ptr(out), T, int(num_seqs), W)
        return out

    def add_bias(self, out, bias):
        """``out[r] += bias`` in place (``bias`` float32): the bias of a projection."""
        N = out.shape[-1]
        if bias.dtype != torch.float32 or bias.numel() != N or out.stride(-1) != 1:
            raise KernelError("add_bias: a float32 bias of the output's width, rows dense")
        self._call("norm", "q3_add_bias", "add_bias", _dtype_code(out.dtype), _ptr(out), out.stride(0), _ptr(bias),
                   out.shape[0], N)
        return out

    def logit_scale_cap(self, logits, scale=1.0, cap=0.0):
        """``logits *= scale`` and, with ``cap > 0``, ``cap * tanh(logits / cap)``, in place (float32)."""
        if logits.dtype != torch.float32 or not logits.is_contiguous():
            raise KernelError("logit_scale_cap: contiguous float32 logits")
        self._call("norm", "q3_logit_scale_cap", "logit_scale_cap", _ptr(logits), logits.numel(), float(scale),
                   float(cap))
        return logits

    def silu_mul(self, gate_up, out):
        I = out.shape[-1]
        if self.timing is not None:
            self._costs(3 * out.shape[0] * I * out.element_size())
        self._call("norm", "q3_silu_mul", "silu_mul",
                   _dtype_code(out.dtype), _ptr(gate_up), _ptr(out), out.shape[0], I)
        return out

    def sigmoid_mul(self, x, gate):
        """``x *= sigmoid(gate)`` in place: ``x`` dense ``[rows, n]``, ``gate`` ``[rows, n]`` (a slice of wider
        rows will do); float32 math, one rounding."""
        rows, n = x.shape
        if not x.is_contiguous() or gate.shape != x.shape or gate.stride(1) != 1 or gate.dtype != x.dtype:
            raise KernelError("sigmoid_mul: dense rows and a gate of their shape and type with unit stride")
        if self.timing is not None:
            self._costs(3 * rows * n * x.element_size())
        self._call("norm", "q3_sigmoid_mul", "sigmoid_mul", _dtype_code(x.dtype), _ptr(x), _ptr(gate), gate.stride(0),
                   rows, n)
        return x

    def clamped_glu(self, gate_up, out, *, limit, alpha, up_offset):
        """``out = g * sigmoid(alpha g) * (u + up_offset)`` with ``g = min(gate, limit)`` and
        ``u = clamp(up, -limit, limit)``; rows of ``gate_up`` are ``[gate | up]`` (csrc/norm.cu)."""
        F = out.shape[-1]
        if gate_up.shape[-1] != 2 * F or not gate_up.is_contiguous() or not out.is_contiguous():
            raise KernelError("clamped_glu: dense [rows, 2F] in, dense [rows, F] out")
        if self.timing is not None:
            self._costs(3 * out.shape[0] * F * out.element_size())
        self._call("norm", "q3_clamped_glu", "clamped_glu", _dtype_code(out.dtype), _ptr(gate_up), _ptr(out),
                   out.shape[0], F, float(limit), float(alpha), float(up_offset))
        return out

    def relu_squared(self, x, out):
        """``out[t, i] = max(x[t, i], 0)^2`` for the leading ``out.shape[1]`` columns of ``x`` (rows of ``x``
        may be wider)."""
        n = out.shape[-1]
        if x.stride(1) != 1 or x.shape[1] < n or not out.is_contiguous() or x.dtype != out.dtype:
            raise KernelError("relu_squared: rows of at least the output's width, dense output of the same type")
        if self.timing is not None:
            self._costs(2 * out.shape[0] * n * out.element_size())
        self._call("norm", "q3_relu_squared", "relu_squared", _dtype_code(out.dtype), _ptr(x), x.stride(0), _ptr(out),
                   out.shape[0], n)
        return out

    def gelu_gate_rows(self, gate, ids, table, offset, out):
        """``out[t, i] = gelu_tanh(gate[t, i]) * table[ids[t], offset + i]`` (csrc/norm.cu)."""
        T, n = gate.shape
        if (not gate.is_contiguous() or not out.is_contiguous() or out.shape != gate.shape or table.stride(1) != 1
                or table.dtype != gate.dtype or offset + n > table.shape[1]):
            raise KernelError("gelu_gate_rows: dense [rows, n] gate and output, a table of the same type")
        self._call("norm", "q3_gelu_gate_rows", "gelu_gate_rows", _dtype_code(gate.dtype), _ptr(gate), _ptr(ids),
                   _ptr(table), table.stride(0), int(offset), table.shape[0], _ptr(out), T, n)
        return out

    # ---- decayed matrix state (csrc/linear_state.cu) and short convolution (csrc/short_conv.cu) ----
    def decayed_state_scan(self, q, k, v, *, state, cu_seqlens, state_slots, num_seqs, decay_logits=None,
                           decay_bias=None, tau=1.0, head_decay=None, inv_freq=None, positions=None, q_scale=1.0,
                           k_scale=1.0, decay_mode="sigmoid_pow", token_decay=None, token_k_scale=None, bonus=None,
                           ones_column=False):
        """``S_t = diag(a_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per (sequence, head) on the float32
        state ``[slots, H, D, Dv]`` of the sequences' slots; returns float32 ``o`` ``[T, H, Dv]``.
        ``q, k`` ``[T, H, D]``, ``v`` ``[T, H, Dv]`` (views of wider rows allowed).  The decay is
        ``sigmoid(decay_logits + decay_bias)^(1 / tau)`` per key channel, or ``head_decay`` (float32
        ``[H]``) per head.  ``inv_freq`` (float32 ``[pairs]``): q and k are rotated first (pair i =
        elements i and i + pairs); then multiplied by ``q_scale`` / ``k_scale``.
        ``decay_mode="exp_neg_exp"``: the decay is ``exp(-exp(decay_logits + decay_bias))``.  ``token_decay`` /
        ``token_k_scale`` (float32 ``[T, H]``): a decay per (token, head) in place of ``head_decay``, and a
        factor on k.  ``ones_column``: the values get one more column whose value is 1 (state and ``o`` then
        have ``Dv + 1`` columns; the last one of ``o`` is q times the decayed sum of the keys).  ``bonus``
        (float32 ``[H * D]``): ``o_t = (S_(t-1) + diag(bonus) k_t v_t^T)^T q_t``, the state read before its
        update."""
        T, H, D = q.shape
        Dv = v.shape[2] + int(bool(ones_column))
        modes = {"sigmoid_pow": 0, "exp_neg_exp": 1}
        if decay_mode not in modes:
            raise KernelError(f"decayed_state_scan: unknown decay mode {decay_mode!r}")
        for x, what in ((token_decay, "token_decay"), (token_k_scale, "token_k_scale")):
            if x is not None and (x.dtype != torch.float32 or x.shape != (T, H) or not x.is_contiguous()):
                raise KernelError(f"decayed_state_scan: {what} is dense float32 [tokens, heads]")
        if bonus is not None and (bonus.dtype != torch.float32 or bonus.numel() != H * D or not bonus.is_contiguous()):
            raise KernelError("decayed_state_scan: the bonus is dense float32 [heads * dim]")
        for x, what in ((q, "q"), (k, "k"), (v, "v")):
            if x.stride(2) != 1 or x.stride(1) != x.shape[2]:
                raise KernelError(f"decayed_state_scan: the heads of {what} lie side by side in a row")
        z = decay_logits
        if z is not None and (z.shape != q.shape or z.stride(2) != 1 or z.stride(1) != D):
            raise KernelError("decayed_state_scan: decay logits are laid out like q")
        if state.dtype != torch.float32 or state.shape[1:] != (H, D, Dv) or not state.is_contiguous():
            raise KernelError("decayed_state_scan: the state is dense float32 [slots, H, D, Dv]")
        out = torch.empty((T, H, Dv), dtype=torch.float32, device=q.device)
        pairs = inv_freq.numel() if inv_freq is not None else 0
        if self.timing is not None:
            e = q.element_size()
            self._costs(2 * num_seqs * H * D * Dv * 4 + T * H * ((3 if z is not None else 2) * D + Dv) * e
                        + T * H * Dv * 4, 6.0 * T * H * D * Dv)
        self._call("linear_state", "q3_decayed_state_scan", "decayed_state_scan", _dtype_code(q.dtype), _ptr(q),
                   q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(z), z.stride(0) if z is not None else 0,
                   _ptr(decay_bias), 1.0 / float(tau), _ptr(head_decay), _ptr(inv_freq), pairs, _ptr(positions),
                   float(q_scale), float(k_scale), _ptr(state), _ptr(cu_seqlens), _ptr(state_slots), _ptr(out),
                   int(num_seqs), H, D, Dv, modes[decay_mode], _ptr(token_decay), _ptr(token_k_scale),
                   int(bool(ones_column)), _ptr(bonus))
        return out

    def stabilised_gates(self, zi, zf, *, i_bias, f_bias, cap, m_state, cu_seqlens, state_slots, num_seqs):
        """The gates of a matrix memory with exponential gates and a running maximum m per (sequence, head)
        (float32 ``[slots, H]``, updated): ``li = cap tanh((zi + bi) / cap)``, ``lf = logsigmoid(cap tanh((zf +
        bf) / cap))``, ``m_t = max(lf + m_(t-1), li)``; returns float32 ``[T, H]`` ``decay = exp(lf + m_(t-1) -
        m_t)``, ``k_scale = exp(li - m_t)`` and ``m_t``.  ``zi``, ``zf``: ``[T, H]`` views of rows of one width."""
        T, H = zi.shape
        if zi.stride(1) != 1 or zf.stride(1) != 1 or zi.stride(0) != zf.stride(0) or zf.shape != zi.shape:
            raise KernelError("stabilised_gates: the two gates are [tokens, heads] views of rows of one width")
        if m_state.dtype != torch.float32 or not m_state.is_contiguous() or m_state.shape[1:] != (H,):
            raise KernelError("stabilised_gates: the running maximum is dense float32 [slots, heads]")
        for b in (i_bias, f_bias):
            if b is not None and (b.dtype != torch.float32 or b.numel() != H or not b.is_contiguous()):
                raise KernelError("stabilised_gates: biases are dense float32 [heads]")
        decay = torch.empty((3, T, H), dtype=torch.float32, device=zi.device)
        self._call("linear_state", "q3_stabilised_gates", "stabilised_gates", _dtype_code(zi.dtype), _ptr(zi), _ptr(zf),
                   zi.stride(0), _ptr(i_bias), _ptr(f_bias), float(cap), _ptr(m_state), _ptr(cu_seqlens),
                   _ptr(state_slots), _ptr(decay[0]), _ptr(decay[1]), _ptr(decay[2]), int(num_seqs), H)
        return decay[0], decay[1], decay[2]

    def head_norm_gate(self, o, gate, out, *, weight, eps, out_scale=1.0, gate_act="silu", per_head_weight=False,
                       denominator=None):
        """``out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * act(gate[t, h]) * out_scale``:
        ``o`` float32 ``[T, H, Dv]``, ``gate`` and ``out`` ``[T, H, Dv]`` views of rows, ``weight``
        float32 ``[Dv]`` (``per_head_weight``: ``[H * Dv]``) or None, ``gate_act`` ``"silu"`` or ``"sigmoid"``.
        ``denominator`` (float32 ``[T, H]``, a running maximum m): ``o`` has one more column c, and its values are
        first divided by ``max(|c|, exp(-m)) + 1e-6``."""
        T, H, Dv = out.shape
        acts = {"silu": 0, "sigmoid": 1}
        if gate_act not in acts:
            raise KernelError(f"head_norm_gate: unknown gate activation {gate_act!r}")
        for x in (gate, out):
            if x.shape != (T, H, Dv) or x.stride(2) != 1 or x.stride(1) != Dv:
                raise KernelError("head_norm_gate: gate and output are [T, H, Dv] with the heads side by side")
        if o.dtype != torch.float32 or not o.is_contiguous() or o.shape != (T, H, Dv + (denominator is not None)):
            raise KernelError("head_norm_gate: o is dense float32 [T, H, Dv] (one more column with a denominator)")
        if denominator is not None and (denominator.dtype != torch.float32 or denominator.shape != (T, H)
                                        or not denominator.is_contiguous()):
            raise KernelError("head_norm_gate: the denominator's maximum is dense float32 [T, H]")
        if weight is not None and weight.numel() != (H * Dv if per_head_weight else Dv):
            raise KernelError("head_norm_gate: the weight spans one head's values, or all heads' (per_head_weight)")
        if self.timing is not None:
            self._costs(T * H * Dv * (4 + 2 * out.element_size()))
        self._call("linear_state", "q3_head_norm_gate", "head_norm_gate", _dtype_code(out.dtype), _ptr(o),
                   _ptr(denominator), _ptr(weight), int(bool(per_head_weight)), float(eps), _ptr(gate), gate.stride(0),
                   _ptr(out), out.stride(0), float(out_scale), acts[gate_act], T, H, Dv)
        return out

    def conv_rope_store(self, x, *, num_heads, num_kv_heads, head_dim, value_dim, conv_weight, conv_state, inv_freq,
                        positions, token_seq, cu_seqlens, state_slots, num_seqs, block_table, k_pages, v_pages,
                        page_size, q_out, value_scale=1.0, write_kv=True):
        """Short causal convolution on every channel of ``x`` ``[T, q heads | k heads | v heads]``
        (``conv_weight`` float32 ``[taps, C]``, tap-major, or None; the rows before a step's first token come from
        ``conv_state`` float32 ``[slots, taps - 1, C]``, which is brought up to date afterwards), rotation
        of q and k (pair i = elements i and i + pairs, angle ``position * inv_freq[i]``), q into
        ``q_out``, k and ``value_scale * v`` into the token's page row (csrc/short_conv.cu)."""
        T = x.shape[0]
        C = (num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim
        taps = conv_weight.shape[0] if conv_weight is not None else 0
        if x.stride(1) != 1 or x.shape[1] != C or not q_out.is_contiguous():
            raise KernelError("conv_rope_store: rows of q, k and v heads; a dense q output")
        if taps and (conv_weight.dtype != torch.float32 or not conv_weight.is_contiguous()
                     or conv_weight.shape[1] != C):
            raise KernelError("conv_rope_store: a dense float32 weight [taps, channels]")
        if taps > 1 and (conv_state.dtype != torch.float32 or not conv_state.is_contiguous()
                         or conv_state.shape[1:] != (taps - 1, C)):
            raise KernelError("conv_rope_store: the state is dense float32 [slots, taps - 1, channels]")
        pairs = inv_freq.numel() if inv_freq is not None else 0
        if self.timing is not None:
            self._costs(2 * T * C * x.element_size())
        self._call("short_conv", "q3_conv_rope_store", "conv_rope_store", _dtype_code(x.dtype), _ptr(x), x.stride(0),
                   _ptr(conv_weight), taps, _ptr(conv_state) if taps > 1 else None, _ptr(positions), _ptr(token_seq),
                   _ptr(cu_seqlens), _ptr(state_slots), _ptr(inv_freq), pairs, _ptr(q_out), _ptr(k_pages),
                   _ptr(v_pages), _ptr(block_table), block_table.shape[1] if block_table is not None else 0, page_size,
                   T, num_heads, num_kv_heads, head_dim, value_dim, float(value_scale), int(bool(write_kv)))
        if taps > 1:
            self._call("short_conv", "q3_conv_state_update", "conv_state_update", _dtype_code(x.dtype), _ptr(x),
                       x.stride(0), _ptr(conv_state), _ptr(cu_seqlens), _ptr(state_slots), taps, C, int(num_seqs))

    # ---- attention through a latent (csrc/latent_attention.cu, csrc/head_gemm.cu) ---------------
    def latent_norm_rope_store(self, down, *, q_rank, kv_rank, rot_dim, q_weight, kv_weight, eps, inv_freq, positions,
                               token_seq, block_table, pages, page_size, write, q_out, pairing="interleaved",
                               magnitude=1.0):
        """Rows of ``down`` are ``[query latent | key latent | shared key part]``: the query latent is
        RMS-normalised into ``q_out``; the key latent is RMS-normalised, the key part rotated
        (angle ``position * inv_freq[i]``, pairs as ``pairing`` says, cos and sin times ``magnitude``),
        and both are written into the token's row of ``pages`` ``[pages, page_size, kv_rank + rot_dim]``.
        ``q_rank`` 0: no query latent (``q_weight`` and ``q_out`` None); ``down`` may be a slice of wider rows."""
        T = down.shape[0]
        if (down.stride(1) != 1 or down.shape[1] != q_rank + kv_rank + rot_dim
                or (q_out is not None and not q_out.is_contiguous()) or (q_rank > 0) != (q_out is not None)):
            raise KernelError("latent_norm_rope_store: rows of q_rank + kv_rank + rot_dim elements")
        if pages is not None and (pages.shape[-1] != kv_rank + rot_dim or not pages.is_contiguous()):
            raise KernelError("latent_norm_rope_store: pages are dense [pages, page_size, kv_rank + rot_dim]")
        pairs = inv_freq.numel() if inv_freq is not None else 0
        if self.timing is not None:
            self._costs(2 * T * (q_rank + kv_rank + rot_dim) * down.element_size())
        self._call("latent_attention", "q3_latent_norm_rope_store", "latent_norm_rope_store",
                   _dtype_code(down.dtype), _ptr(down), down.stride(0), q_rank, kv_rank, rot_dim, _ptr(q_weight),
                   _ptr(kv_weight), float(eps), _ptr(inv_freq), pairs, _ptr(positions), _ptr(token_seq),
                   _ptr(block_table), block_table.shape[1] if block_table is not None else 0, _ptr(pages),
                   page_size, T, int(bool(write)), _ptr(q_out), self.PAIRINGS[pairing], float(magnitude))

    @staticmethod
    def _head_strides(x, what):
        if x.dim() != 3 or x.stride(2) != 1:
            raise KernelError(f"{what}: [tokens, heads, n] with unit stride along n")
        return x.stride(0), x.stride(1)

    def rotate_heads(self, x, out, *, positions, inv_freq, pairing="interleaved", magnitude=1.0):
        """``out[t, h] = rotate(x[t, h])`` by the token's position (pairs as ``pairing`` says, cos and sin
        times ``magnitude``; elements beyond ``2 * len(inv_freq)`` are copied).  ``x`` and ``out`` may be
        slices of wider rows (with the halves pairing not the same ones)."""
        T, H, n = x.shape
        xs, os_ = self._head_strides(x, "rotate_heads"), self._head_strides(out, "rotate_heads")
        pairs = inv_freq.numel() if inv_freq is not None else 0
        self._call("latent_attention", "q3_rotate_heads", "rotate_heads", _dtype_code(x.dtype), _ptr(x), xs[0], xs[1],
                   _ptr(out), os_[0], os_[1], _ptr(positions), _ptr(inv_freq), pairs, n, H, T,
                   self.PAIRINGS[pairing], float(magnitude))
        return out

    def head_linear(self, x, weight, out):
        """``out[t, h] = weight[h] @ x[t, h]``: ``x`` ``[T, H, K]``, ``weight`` ``[H, N, K]`` dense, ``out``
        ``[T, H, N]``; ``x`` and ``out`` may be slices of wider rows (csrc/head_gemm.cu)."""
        T, H, K = x.shape
        N = weight.shape[1]
        if weight.shape != (H, N, K) or not weight.is_contiguous() or out.shape != (T, H, N) \
                or weight.dtype != x.dtype or out.dtype != x.dtype:
            raise KernelError(f"head_linear: x {list(x.shape)}, weight {list(weight.shape)}, out {list(out.shape)}")
        xs, os_ = self._head_strides(x, "head_linear"), self._head_strides(out, "head_linear")
        if self.timing is not None:
            e = x.element_size()
            self._costs((H * N * K + T * H * (K + N)) * e, 2.0 * T * H * N * K, f" {T}x{H}x{K}->{N}")
        if x.dtype == torch.bfloat16 and T > self.SMALL_M:
            # more than 16 tokens in bfloat16: the library's batched product, as for plain products
            if self.timing is not None:
                with self._timed("library_bmm"):
                    torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))
            else:
                torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))
            return out
        self._call("head_gemm", "q3_head_linear", "head_linear", _dtype_code(x.dtype), _ptr(x), xs[0], xs[1],
                   _ptr(weight), _ptr(out), os_[0], os_[1], T, H, N, K)
        return out

    def latent_attention(self, q, *, pages, value_dim, block_table, token_seq, positions, sink, out, page_size, scale,
                         window, step=None):
        """Causal attention of every token over its sequence's cached rows, all heads sharing them:
        ``q`` ``[T, H, width]`` already in the rows' space, ``pages`` ``[pages, page_size, width]``, the
        value of a row its first ``value_dim`` elements, ``out`` ``[T, H, value_dim]``.  ``sink``
        (float32 ``[H]`` or None) joins the softmax denominator; ``window``: the query at position p
        reads rows ``max(0, p - window + 1) .. p``."""
        T, H, width = q.shape
        if pages.shape[-1] != width or not pages.is_contiguous() or out.shape != (T, H, value_dim):
            raise KernelError("latent_attention: pages are dense [pages, page_size, width of q]")
        qs, os_ = self._head_strides(q, "latent_attention"), self._head_strides(out, "latent_attention")
        if self.timing is not None and step is not None:
            e = out.element_size()
            keys = pairs = 0
            cu = step.host_cu_seqlens
            for b, kv in enumerate(step.host_kv_lens):
                n = cu[b + 1] - cu[b] if len(cu) > b + 1 else 1
                seen = min(kv, (window or kv) + n - 1)
                keys += seen
                pairs += sum(min(kv - n + i + 1, window or kv) for i in range(n)) if n < 64 else \
                    n * min(kv, window or kv)
            self._costs(keys * width * e + T * H * (width + value_dim) * e, 2.0 * H * (width + value_dim) * pairs)
        if (self.latent_attention_tc and step is not None and out.dtype == torch.bfloat16 and width % 16 == 0
                and value_dim % 16 == 0 and value_dim <= 512 and qs[0] % 8 == 0 and qs[1] % 8 == 0
                and os_[0] % 2 == 0 and os_[1] % 2 == 0 and q.data_ptr() % 16 == 0 and pages.data_ptr() % 16 == 0
                and out.data_ptr() % 4 == 0 and (32 + 64) * (width + 8) * 2 + 14000 <= 220 * 1024):
            # bfloat16 on the tensor cores: 32 (token, head) rows per block, keys in tiles of 64
            splits, part = 1, None
            if step.max_query_len == 1:
                # few rows, many keys: cut every sequence's keys into slices so that about two blocks
                # per SM work.  The count comes from an upper bound of the lengths (in a captured step:
                # the block-table width it was captured for), never from the lengths of the moment.
                bound = step.captured_width * page_size or step.max_kv_len
                if window:
                    bound = min(bound, int(window) + 63)
                groups = -(-H // min(32, 1 << max(0, (H - 1).bit_length())))
                splits = max(1, min(-(-bound // 64), 2 * self.SM_COUNT // max(1, step.num_seqs * groups), 64))
                if splits > 1:
                    part = torch.empty(step.num_seqs * H * splits * (value_dim + 2), dtype=torch.float32,
                                       device=out.device)
                    self.launches += 1  # the merge of the slices
            self._call("latent_attention_tc", "q3_latent_attention_tc", "latent_attention_tc", _ptr(q), qs[0], qs[1],
                       _ptr(pages), width, value_dim, _ptr(block_table), block_table.shape[1], _ptr(step.cu_seqlens),
                       _ptr(step.kv_lens), _ptr(sink), _ptr(out), os_[0], os_[1], step.num_seqs,
                       step.max_query_len, H, page_size, float(scale), int(window or 0), splits, _ptr(part))
            return out
        self._call("latent_attention", "q3_latent_attention", "latent_attention", _dtype_code(out.dtype), _ptr(q),
                   qs[0], qs[1], _ptr(pages), width, value_dim, _ptr(block_table), block_table.shape[1],
                   _ptr(token_seq), _ptr(positions), _ptr(sink), _ptr(out), os_[0], os_[1], T, H, page_size,
                   float(scale), int(window or 0))
        return out

    # ---- routed experts (csrc/experts.cu) --------------------------------------------------------
    def route_top(self, h, router, top, renormalize=False, score="sigmoid", correction=None, groups=None):
        """``(chosen int32 [T, top], weights float32 [T, top])``: the float32 router product, the
        ``top`` largest per token in descending order (chosen on the logits, which order the experts as
        their sigmoids do without the ties of a saturated sigmoid; lowest index on an exact tie).
        ``score="sigmoid"``: the weights are the chosen logits' sigmoids (``renormalize``: divided by
        their sum); ``"softmax_chosen"``: the softmax over the chosen logits only; ``"softmax_all"``: s is
        the softmax over all outputs, the choice is made on ``s + correction`` (float32 ``[E]`` or None) among
        the outputs of the ``groups[1]`` best of ``groups[0]`` equal groups of neighbours (a group's score: its
        largest choice score), and the weights are the chosen s (``renormalize``: over their sum + 1e-20)."""
        if score not in ("sigmoid", "softmax_chosen", "softmax_all"):
            raise KernelError(f"route_top: unknown score {score!r}")
        mode = 3 if score == "softmax_all" else (2 if score == "softmax_chosen" else int(bool(renormalize)))
        T, W = h.shape
        E = router.shape[0]
        count, keep = (int(groups[0]), int(groups[1])) if groups else (0, 0)
        if mode != 3 and (correction is not None or groups):
            raise KernelError("route_top: a correction and groups go with score='softmax_all'")
        if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E
                                       or not correction.is_contiguous()):
            raise KernelError("route_top: the correction is a dense float32 vector, one number per router output")
        if count > 1 and (E % count or not 1 <= keep <= count or top > keep * (E // count)):
            raise KernelError(f"route_top: {E} outputs in {count} groups of which {keep} stay cannot give {top} choices")
        if router.dtype != torch.float32 or not router.is_contiguous() or router.shape[1] != W or h.stride(1) != 1:
            raise KernelError("route_top: a dense float32 router [experts, width]")
        chosen = torch.empty((T, top), dtype=torch.int32, device=h.device)
        weights = torch.empty((T, top), dtype=torch.float32, device=h.device)
        logits = torch.empty((T, E), dtype=torch.float32, device=h.device)
        if self.timing is not None:
            self._costs(E * W * 4 + T * W * h.element_size(), 2.0 * T * E * W)
        self.launches += 1  # two kernels: the logits, then the choice
        self._call("experts", "q3_route_top", "route_top", _dtype_code(h.dtype), _ptr(h), h.stride(0), _ptr(router),
                   T, E, W, top, mode, _ptr(logits), _ptr(chosen), _ptr(weights), _ptr(correction), count, keep,
                   int(bool(renormalize)))
        return chosen, weights

    def routed_experts(self, h, chosen, weights, gate_up, down, *, limit=0.0, alpha=1.0, up_offset=0.0,
                       weight_on="input", shared=None, activation="clamped_glu", shared_gate=None, num_identity=0):
        """Every token through its chosen experts: ``gate_up`` ``[E, 2F, W]`` (gate rows, then up
        rows), ``down`` ``[E, W, F]``; the slots are grouped by expert on the device, each expert's two
        products run over its slots only, and a token's results (and ``shared`` ``[T, W]``) are summed
        in float32.  ``activation="relu2"``: the experts have no gate, ``gate_up`` is the up weight
        ``[E, F, W]`` and the unit is the squared ReLU (the weight then multiplies the output).
        ``shared_gate`` ``[T]`` (a view of one column will do): ``shared`` is multiplied by its sigmoid.
        ``num_identity``: choices ``E .. E + num_identity - 1`` stand for experts that return their input; their
        slots run through no product and the token's own row is summed with the slot's weight."""
        T, W = h.shape
        num_identity = int(num_identity)
        if num_identity and weight_on != "output":
            raise KernelError("routed_experts: identity experts take their weight on the output")
        gated = activation == "clamped_glu"
        if activation not in ("clamped_glu", "relu2"):
            raise KernelError(f"routed_experts: unknown activation {activation!r}")
        E, F2, _ = gate_up.shape
        F, top = (F2 // 2 if gated else F2), chosen.shape[1]
        S = T * top
        dev = h.device
        if not (gate_up.is_contiguous() and down.is_contiguous() and down.shape == (E, W, F) and h.stride(1) == 1):
            raise KernelError("routed_experts: dense gate_up [E, 2F, W] (or up [E, F, W]) and down [E, W, F]")
        if shared is not None and (shared.shape != (T, W) or not shared.is_contiguous() or shared.dtype != h.dtype):
            raise KernelError("routed_experts: the shared expert's result is dense [tokens, width]")
        if not gated and weight_on != "output":
            raise KernelError("routed_experts: experts without a gate take their weight on the output")
        if shared_gate is not None and (shared is None or shared_gate.shape != (T,) or shared_gate.dtype != h.dtype):
            raise KernelError("routed_experts: one gate logit per token, of the activations' type")
        # identity experts are grouped like the stored ones (behind them); the products then stop at the stored
        # experts' last tile
        EA = E + num_identity
        plan = torch.empty(2 * (EA + 1) + S, dtype=torch.int32, device=dev)
        offsets, tile_offsets, order = plan[: EA + 1], plan[EA + 1: 2 * (EA + 1)], plan[2 * (EA + 1):]
        # bfloat16 with 16-byte rows: the products run on the tensor cores, in row tiles of 64 slots when
        # an expert gets about that many, else of 32
        tensor_cores = (self.experts_tc and h.dtype == torch.bfloat16 and W % 8 == 0 and F % 8 == 0
                        and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0)
        bm = 64 if tensor_cores and S >= 48 * E else 32
        self._call("experts", "q3_group_slots", "group_slots", _ptr(chosen), S, EA, bm, _ptr(offsets),
                   _ptr(tile_offsets), _ptr(order))
        mid = torch.empty((S, F), dtype=h.dtype, device=dev)
        y = torch.empty((S, W), dtype=h.dtype, device=dev)
        out = torch.empty((T, W), dtype=h.dtype, device=dev)
        code, e = _dtype_code(h.dtype), h.element_size()
        on_input = weight_on == "input"
        if self.timing is not None:  # every chosen expert's weights once, or once per slot when slots are few
            n_up = 2 if gated else 1
            self._costs(min(S, E) * n_up * F * W * e + T * W * e + S * F * e, 2.0 * n_up * S * F * W,
                        f" {S}x{W}->{n_up}x{F}")
        if not gated and tensor_cores:
            self._call("experts", "q3_expert_up_tc", "expert_up_tc", _ptr(h), h.stride(0), _ptr(gate_up), _ptr(mid), S,
                       E, F, W, top, bm, _ptr(offsets), _ptr(tile_offsets), _ptr(order), 1)
        elif not gated:
            self._call("experts", "q3_expert_up", "expert_up", code, _ptr(h), h.stride(0), _ptr(gate_up), _ptr(mid), S,
                       E, F, W, top, _ptr(offsets), _ptr(tile_offsets), _ptr(order), 1)
        elif tensor_cores:
            self._call("experts", "q3_expert_gate_up_tc", "expert_gate_up_tc", _ptr(h), h.stride(0), _ptr(gate_up),
                       _ptr(mid), S, E, F, W, top, bm, _ptr(offsets), _ptr(tile_offsets), _ptr(order), _ptr(weights),
                       int(on_input), float(limit), float(alpha), float(up_offset))
        else:
            self._call("experts", "q3_expert_gate_up", "expert_gate_up", code, _ptr(h), h.stride(0), _ptr(gate_up),
                       _ptr(mid), S, E, F, W, top, _ptr(offsets), _ptr(tile_offsets), _ptr(order), _ptr(weights),
                       int(on_input), float(limit), float(alpha), float(up_offset))
        if self.timing is not None:
            self._costs(min(S, E) * F * W * e + S * (F + W) * e, 2.0 * S * F * W, f" {S}x{F}->{W}")
        if tensor_cores:
            self._call("experts", "q3_expert_down_tc", "expert_down_tc", _ptr(mid), _ptr(down), _ptr(y), S, E, F, W,
                       bm, _ptr(offsets), _ptr(tile_offsets), _ptr(order))
        else:
            self._call("experts", "q3_expert_down", "expert_down", code, _ptr(mid), _ptr(down), _ptr(y), S, E, F, W,
                       _ptr(offsets), _ptr(tile_offsets), _ptr(order))
        if self.timing is not None:
            self._costs((S + T + (T if shared is not None else 0)) * W * e)
        self._call("experts", "q3_expert_combine", "expert_combine", code, _ptr(y),
                   None if on_input else _ptr(weights), _ptr(shared), _ptr(shared_gate),
                   shared_gate.stride(0) if shared_gate is not None else 0, _ptr(out), T, W, top,
                   _ptr(chosen) if num_identity else None, E, _ptr(h) if num_identity else None, h.stride(0))
        return out

    # ---- position encoding + cache write -----------------------------------------------
    def rope_table(self, inv_freq: torch.Tensor, max_positions: int):
        half = inv_freq.numel()
        cos = torch.empty((max_positions, half), dtype=torch.float32, device=inv_freq.device)
        sin = torch.empty_like(cos)
        self._call("rope_kv", "q3_rope_table", "rope_table",
                   _ptr(inv_freq), _ptr(cos), _ptr(sin), max_positions, half)
        return cos, sin

    PAIRINGS = {"half": 0, "interleaved": 1}

    def qk_norm_rope_store(self, qkv, *, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, cos, sin,
                           positions, token_seq, block_table, k_pages, v_pages, page_size, write_kv,
                           pairing="half"):
        """Per-head q/k norm, rotation by ``cos/sin[position]`` and the write of k and v into their
        pages (csrc/rope_kv.cu).  ``pairing`` says which two elements of a head rotation pair i
        is made of: ``"half"`` (i, i + rotary_dim/2) or ``"interleaved"`` (2i, 2i + 1)."""
        T = qkv.shape[0]
        rot_half = cos.shape[1] if cos is not None else 0
        max_pos = cos.shape[0] if cos is not None else 0
        max_pages = block_table.shape[1] if block_table is not None else 0
        if cos is not None and (max_pos < 1 or sin is None or sin.shape != cos.shape):
            raise KernelError("qk_norm_rope_store: bad argument: rotation tables need at least one position "
                              "and cos and sin of one shape")
        if head_dim * 16 > 48 * 1024:
            raise KernelError(f"qk_norm_rope_store: head_dim={head_dim} is too large (limit 3072)")
        if self.timing is not None:
            self._costs(2 * T * (num_heads + 2 * num_kv_heads) * head_dim * qkv.element_size())
        self._call("rope_kv", "q3_qk_norm_rope_store", "qk_norm_rope_store",
                   _dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), num_heads, num_kv_heads, head_dim,
                  _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), rot_half, max_pos,
                  _ptr(positions), _ptr(token_seq), _ptr(block_table), max_pages, _ptr(k_pages), _ptr(v_pages),
                  page_size, T, int(bool(write_kv)), self.PAIRINGS[pairing], _ptr(self._error_word(qkv.device)))

    def qk_norm_store(self, proj, *, num_heads, num_kv_heads, head_dim, value_dim, k_start, v_start, q_weight,
                      k_weight, eps, positions, token_seq, block_table, k_pages, v_pages, page_size, write_kv,
                      maps=1, num_value_heads=None, inv_freq=None, pairing="half", magnitude=1.0):
        """Per-head q/k RMSNorm (weights float32 shared by the heads, or None: as they are), an optional
        rotation, and the write of k and v into their pages (csrc/rope_kv.cu).  A row of ``proj`` holds the
        query heads from column 0, the key heads from ``k_start`` and the value heads (``value_dim`` each) from
        ``v_start`` (which may be ``k_start``: the values are the keys as projected); q is changed in place.
        ``maps``: a head is that many consecutive parts of ``head_dim / maps`` elements, each normalised by
        itself with the one weight of that size.  ``num_value_heads``: the values' head count when it is not the
        keys'.  ``inv_freq`` (float32 ``[pairs]``): the first ``2 * pairs`` elements of every part turn by
        ``position * inv_freq[i]``, pairs as ``pairing`` says, cos and sin times ``magnitude``; no table."""
        T = proj.shape[0]
        if proj.stride(1) != 1:
            raise KernelError("qk_norm_store: unit-stride rows")
        maps = int(maps)
        if maps < 1 or head_dim % maps:
            raise KernelError(f"qk_norm_store: a head of {head_dim} does not split into {maps} maps")
        for w in (q_weight, k_weight):
            if w is not None and (w.dtype != torch.float32 or w.numel() != head_dim // maps):
                raise KernelError("qk_norm_store: weights are float32 vectors of one map's size")
        nv = int(num_value_heads or num_kv_heads)
        pairs = inv_freq.numel() if inv_freq is not None else 0
        if inv_freq is not None and (inv_freq.dtype != torch.float32 or 2 * pairs > head_dim // maps):
            raise KernelError("qk_norm_store: float32 inverse frequencies, at most half a map's size of them")
        max_pages = block_table.shape[1] if block_table is not None else 0
        if self.timing is not None:
            self._costs(2 * T * ((num_heads + num_kv_heads) * head_dim + num_kv_heads * value_dim) * proj.element_size())
        self._call("rope_kv", "q3_qk_norm_store", "qk_norm_store", _dtype_code(proj.dtype), _ptr(proj), proj.stride(0),
                   num_heads, num_kv_heads, nv, head_dim, value_dim, int(k_start), int(v_start), _ptr(q_weight),
                   _ptr(k_weight), float(eps), maps, _ptr(inv_freq), pairs, self.PAIRINGS[pairing], float(magnitude),
                   _ptr(positions), _ptr(token_seq), _ptr(block_table), max_pages,
                   _ptr(k_pages), _ptr(v_pages), page_size, T, int(bool(write_kv)))

    # ---- attention --------------------------------------------------------------------
    def paged_attention(self, q, q_stride, *, num_heads, num_kv_heads, head_dim, k_pages, v_pages, block_table,
                        token_seq, positions, out, page_size, scale, window, step=None, decode_slices=None,
                        value_dim=None, keep_first=0, sink=None, gate=None, chunk=None, softcap=None):
        """Causal attention of every token of the step over its sequence's pages.  ``chunk``: position p sees
        keys from ``floor(p / chunk) * chunk`` on only.  ``softcap``: scores become ``softcap * tanh(score /
        softcap)`` after the scale.  ``value_dim``:
        values have a size of their own (``v_pages`` ``[pages, kv heads, page, value_dim]``); ``out`` may
        then be a view of wider rows, head h at column ``h * value_dim``.  ``keep_first``: with a window, the
        sequence's first tokens stay visible as well.  ``sink``: a score without a value that is added to the
        softmax's denominator.  ``gate`` ``[T, heads * value_dim]`` (a view of wider rows will do): the result
        is multiplied by its sigmoid."""
        T = out.shape[0]
        if head_dim > 256:
            raise KernelError(f"paged_attention: head_dim={head_dim} is not supported (sizes up to 256 are)")
        Dv = int(value_dim or head_dim)
        keep_first = int(keep_first or 0) if window else 0
        plain = not keep_first and sink is None and gate is None  # what the tcgen05 kernel takes
        dense = out.stride(0) == num_heads * Dv and Dv == head_dim
        extras = dict(keep_first=keep_first, sink=sink, gate=gate)
        chunk, softcap = int(chunk or 0), float(softcap or 0.0)
        if chunk:
            dense = False  # the specialised kernels know no chunks: the general kernel
        if softcap:
            plain = False  # the tcgen05 kernel knows no capped scores; the other specialised kernels do
            extras["softcap"] = softcap
        if gate is not None and (gate.stride(1) != 1 or gate.shape != (T, num_heads * Dv) or gate.dtype != out.dtype):
            raise KernelError("paged_attention: the gate is [tokens, heads * value_dim] of the output's type")
        if Dv > 256 or out.stride(1) != 1:
            raise KernelError(f"paged_attention: value_dim={Dv} is not supported (up to 256, unit stride)")
        if (dense and step is not None and step.decode_only and out.dtype == torch.bfloat16 and head_dim in (64, 128, 256)
                and num_heads // num_kv_heads <= 16 and q_stride % 8 == 0):
            return self.paged_attention_decode(
                q, q_stride, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, k_pages=k_pages,
                v_pages=v_pages, block_table=block_table, kv_lens=step.kv_lens, cu_seqlens=step.cu_seqlens,
                out=out, page_size=page_size, scale=scale, window=window, num_seqs=step.num_seqs,
                max_kv_len=step.captured_width * page_size or step.max_kv_len, step=step,
                num_splits=decode_slices, longest=getattr(step, "kv_longest", None), **extras)
        if (dense and step is not None and out.dtype == torch.bfloat16 and head_dim in (64, 128)
                and num_heads // num_kv_heads <= 16 and q_stride % 8 == 0):
            # portions of prompts on the tensor-core kernel, one-token sequences on the split-KV kernel
            group = num_heads // num_kv_heads
            cu = step.host_cu_seqlens
            qlens = [cu[b + 1] - cu[b] for b in range(step.num_seqs)]
            work = sum(-(-n * group // 128) for n in qlens if n > 1)
            done = False
            if (work and head_dim == 128 and not window and plain and 128 % group == 0 and page_size in (8, 16, 32, 64)
                    and self.prefill_attention == "tcgen05"):
                # tcgen05/TMEM kernel; it answers "unsupported" for what it does not take
                self.launches += 1
                pairs = sum(-(-(-(-n * group // 128)) // 2) for n in qlens if n > 1)  # two row blocks per work item
                launch = lambda: self._get("attention_prefill_tc", "q3_paged_attention_prefill_tc")(  # noqa: E731
                    _ptr(q), q_stride, q.shape[0], _ptr(k_pages), _ptr(v_pages),
                    k_pages.shape[0] * num_kv_heads * page_size, _ptr(block_table), block_table.shape[1],
                    _ptr(step.kv_lens), _ptr(step.cu_seqlens), _ptr(out), step.num_seqs, pairs, num_heads,
                    num_kv_heads, head_dim, page_size, float(scale), 1, _ptr(self._error_word(out.device)),
                    self._stream())
                if self.timing is not None:
                    self._costs(*self._attention_cost(step, num_heads, num_kv_heads, head_dim, out, prompts=True))
                    with self._timed("paged_attention_prefill_tc"):
                        code = launch()
                else:
                    code = launch()
                if code == 0:
                    done = True
                elif code != 1:
                    _check(code, "paged_attention_prefill_tc")
            if work and not done:
                if self.timing is not None:
                    self._costs(*self._attention_cost(step, num_heads, num_kv_heads, head_dim, out, prompts=True))
                self._call("attention_prefill", "q3_paged_attention_prefill_sink", "paged_attention_prefill",
                           _ptr(q), q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                           block_table.shape[1], _ptr(step.kv_lens), _ptr(step.cu_seqlens), _ptr(out),
                           step.num_seqs, work, num_heads, num_kv_heads, head_dim, page_size, float(scale),
                           int(window or 0), 1, keep_first, int(sink is not None), float(sink or 0.0), _ptr(gate),
                           gate.stride(0) if gate is not None else 0, softcap)
            if step.num_single:
                singles = [kv for kv, n in zip(step.host_kv_lens, qlens) if n == 1]
                longest = max(singles)
                self.paged_attention_decode(
                    q, q_stride, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                    k_pages=k_pages, v_pages=v_pages, block_table=block_table, kv_lens=step.kv_lens,
                    cu_seqlens=step.cu_seqlens, out=out, page_size=page_size, scale=scale, window=window,
                    num_seqs=step.num_single, max_kv_len=longest, seq_list=step.single_seqs, step=step,
                    num_splits=self.decode_slices_for(singles, num_kv_heads, head_dim,
                                                      window + keep_first if window else window), **extras)
            return out
        if self.timing is not None and step is not None:
            self._costs(*self._attention_cost(step, num_heads, num_kv_heads, head_dim, out))
        self._call("attention_generic", "q3_paged_attention_generic", "paged_attention",
                   _dtype_code(out.dtype), _ptr(q), q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                  block_table.shape[1], _ptr(token_seq), _ptr(positions), _ptr(out), out.stride(0), T, num_heads,
                  num_kv_heads, head_dim, Dv, page_size, float(scale), int(window or 0), int(keep_first or 0),
                  int(sink is not None), float(sink or 0.0), _ptr(gate), gate.stride(0) if gate is not None else 0,
                  chunk, softcap)
        return out

    def differential_attention(self, q, q_stride, *, num_heads, num_kv_heads, map_dim, value_dim, k_pages, v_pages,
                               block_table, token_seq, positions, out, page_size, scale, lam, eps, out_scale,
                               window=None, chunk=None, step=None):
        """Two softmax maps per head over the same values (csrc/attention_generic.cu): a query head is
        ``[q1 | q2]`` of ``map_dim`` each at column ``h * 2 * map_dim``, ``k_pages`` ``[pages, kv heads, page,
        2 * map_dim]`` hold ``[k1 | k2]``, ``v_pages`` ``[pages, kv heads, page, value_dim]``.  ``out[t, h] =
        (a1 - lam * a2)`` divided by its root mean square (``eps`` inside the root), times ``out_scale``."""
        T = out.shape[0]
        if map_dim > 256 or value_dim > 256 or out.stride(1) != 1:
            raise KernelError("differential_attention: map and value sizes up to 256, unit stride")
        if k_pages.shape[-1] != 2 * map_dim or v_pages.shape[-1] != value_dim:
            raise KernelError("differential_attention: key pages hold both maps, value pages the values")
        if self.timing is not None and step is not None:
            # a key row of two maps and a value row per key; two score products and two weighted sums per pair
            nbytes, _ = self._attention_cost(step, num_heads, num_kv_heads, map_dim + value_dim // 2, out)
            _, flops = self._attention_cost(step, num_heads, num_kv_heads, map_dim + value_dim, out)
            self._costs(nbytes, flops)
        group = num_heads // num_kv_heads
        if (self.differential_tc and step is not None and out.dtype == torch.bfloat16 and q_stride % 8 == 0
                and q.data_ptr() % 16 == 0 and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0):
            if step.decode_only and group in (1, 2, 4, 8) and map_dim % 8 == 0 and value_dim in (32, 64, 128):
                # one token per sequence: the keys cut into slices so that about two blocks per SM work.  The
                # count comes from an upper bound of the lengths (in a captured step: the block-table width it
                # was captured for), never from the lengths of the moment.
                bound = step.captured_width * page_size or step.max_kv_len
                for limit in (window, chunk):
                    if limit:
                        bound = min(bound, int(limit))
                blocks = max(1, step.num_seqs * num_kv_heads)
                # a block's 8 warps work on 8 / (group / heads per warp) tiles of 32 keys at a time; two blocks an SM
                round_keys = 32 * 8 // max(1, group // 2)
                splits = max(1, min(-(-bound // round_keys), (2 * self.SM_COUNT) // blocks, 64))
                mid = torch.empty(step.num_seqs * num_heads * splits * 2 * (value_dim + 2), dtype=torch.float32,
                                  device=out.device)
                self.launches += 1  # the merge of the slices
                self._call("attention_diff", "q3_diff_attention_decode", "differential_attention_decode", _ptr(q),
                           q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                           _ptr(step.kv_lens), _ptr(step.cu_seqlens), _ptr(out), out.stride(0), _ptr(mid),
                           step.num_seqs, num_heads, num_kv_heads, map_dim, value_dim, page_size, float(scale),
                           int(window or 0), int(chunk or 0), splits, float(lam), float(eps), float(out_scale))
                return out
            if map_dim in (32, 64, 128) and value_dim in (64, 128):
                cu = step.host_cu_seqlens
                work = sum(-(-(cu[b + 1] - cu[b]) * group // 128) for b in range(step.num_seqs) if cu[b + 1] > cu[b])
                self._call("attention_diff", "q3_diff_attention_prefill", "differential_attention_tc", _ptr(q),
                           q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                           _ptr(step.kv_lens), _ptr(step.cu_seqlens), _ptr(out), out.stride(0), step.num_seqs, work,
                           num_heads, num_kv_heads, map_dim, value_dim, page_size, float(scale), int(window or 0),
                           int(chunk or 0), float(lam), float(eps), float(out_scale))
                return out
        self._call("attention_generic", "q3_paged_attention_diff", "differential_attention", _dtype_code(out.dtype),
                   _ptr(q), q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                   _ptr(token_seq), _ptr(positions), _ptr(out), out.stride(0), T, num_heads, num_kv_heads, map_dim,
                   value_dim, page_size, float(scale), int(window or 0), int(chunk or 0), float(lam), float(eps),
                   float(out_scale))
        return out

    @staticmethod
    def _attention_cost(step, num_heads, num_kv_heads, head_dim, out, prompts=None):
        """(bytes, flops) of a step's attention: every key and value of each sequence read once, q
        read and the result written; 4 * heads * head_dim flops per (query, key) pair.
        ``prompts``: True counts only sequences that bring more than one token, False only those
        that bring one, None all."""
        e = out.element_size()
        keys = pairs = rows = 0
        cu = step.host_cu_seqlens
        for b, kv in enumerate(step.host_kv_lens):
            n = cu[b + 1] - cu[b] if len(cu) > b + 1 else 1
            if prompts is not None and (n > 1) != prompts:
                continue
            keys += kv
            rows += n
            pairs += n * kv - n * (n - 1) // 2
        return (2 * keys * num_kv_heads * head_dim * e + 2 * rows * num_heads * head_dim * e,
                4 * num_heads * head_dim * pairs)

    SM_COUNT = 148  # of a B200; replaced by the device's own count when the table is built
    TICKETS = 1 << 16  # ticket words for the merge by the last block: sequences x kv heads of one launch
    # blocks of the split-KV kernel that an SM holds, by head size (registers allow 4 / 3 / 2,
    # shared memory 6 / 3 / 1)
    DECODE_BLOCKS_PER_SM = {64: 4, 128: 3, 256: 1}

    def decode_splits(self, num_seqs: int, num_kv_heads: int, max_kv_len: int, head_dim: int = 128) -> int:
        """How many slices each sequence's keys are cut into when all that is known is their number
        and an upper bound of their length (a captured step without :meth:`decode_slices_for`)."""
        return self._decode_slices([-(-max(1, max_kv_len) // 64)] * max(1, num_seqs), num_kv_heads, head_dim)

    def decode_slices_for(self, kv_lens: list[int], num_kv_heads: int, head_dim: int, window: int | None) -> int:
        """Into how many slices the split-KV kernel cuts the longest of these sequences (asked once
        per decode step by the attention parts' chooser; answers are kept by the sequences' lengths
        in tiles of 64 keys)."""
        cap = (int(window) + 63) if window else None
        tiles = tuple(-(-(n if cap is None or n < cap else cap) // 64) for n in kv_lens)
        key = (num_kv_heads, head_dim, tiles)
        slices = self._slices_cache.get(key)
        if slices is None:
            if len(self._slices_cache) > 8192:
                self._slices_cache.clear()
            slices = self._slices_cache[key] = self._decode_slices(tiles, num_kv_heads, head_dim)
        return slices

    def _decode_slices(self, tiles, num_kv_heads: int, head_dim: int) -> int:
        """The slice count for sequences of ``tiles`` x 64 keys.  With ``s`` slices the longest
        sequence is cut into slices of ``ceil(longest / s)`` tiles and every other sequence into as
        many slices of that length as it needs (the kernel's rule), which gives the number of
        blocks.  The cost of a choice, in units of the time one key takes to stream when every block
        slot (3 per SM at head size 128) is busy: while all blocks fit the slots, keys per slice + 12 per slice (the
        last block of a pair merges them); beyond that, waves x (keys per slice + 384), the 384 being
        what a block pays besides its keys (lengths, block table and first tile at the start, the
        warps' merge and the ticket at the end), which a full machine no longer hides; waves are
        whole up to six and blocks / slots + 1/2 beyond (blocks of equal length start and end
        together at first and drift apart later).  Slices are at least 192 keys long, 64 with at most
        32 (sequence, kv head) pairs.  The constants are fitted to a sweep of 1..128 sequences x
        256..16384 keys x 1..64 slices on a B200 (8 kv heads of 128,
        ``python -m qwen3_runtime_b200.ops.tune decode_splits``): the choice is within 0.6 % of the
        best one on average and 13 % at worst for sequences of one length, and within a few percent
        for the mixed batches tried.  The reference's rule for an RTX 4090 looks at the number of
        sequences and the longest one (qwen3_runtime/kernels/triton_decode.py:122-133)."""
        import numpy as np

        t = np.asarray(tiles, dtype=np.int64)
        t = t[t > 0]
        if t.size == 0:
            return 1
        longest = int(t.max())
        slots = self.DECODE_BLOCKS_PER_SM.get(head_dim, 3) * self.SM_COUNT
        # a key of a smaller head streams faster, what a block pays besides its keys stays; merging a
        # slice costs in proportion to the head size, like a key
        fixed, per_slice = 384.0 * 128.0 / head_dim, 12.0
        floor = 1 if t.size * num_kv_heads <= 32 else 3  # tiles
        counts = np.arange(1, min(64, longest) + 1)
        slice_tiles = -(-longest // counts)
        counts = counts[(slice_tiles >= floor) | (counts == 1)]
        slice_tiles = -(-longest // counts)
        blocks = num_kv_heads * (-(-t[None, :] // slice_tiles[:, None])).sum(axis=1)
        per = 64.0 * slice_tiles
        waves = blocks / slots
        waves = np.where(waves <= 6, np.ceil(waves), waves + 0.5)
        cost = np.where(blocks <= slots, per, waves * (per + fixed)) + per_slice * counts
        return int(counts[int(np.argmin(cost))])

    def decode_new_token_ok(self, qkv, *, num_heads, num_kv_heads, head_dim, cos, q_weight, k_weight) -> bool:
        """Whether the split-KV kernel can make q, k and v of the newest token itself (per-head
        norm, rotation, cache write) for a step in which every sequence brings one token."""
        return (self.fuse_decode_new_token and qkv.dtype == torch.bfloat16 and head_dim in (64, 128, 256)
                and num_heads // num_kv_heads <= 16 and qkv.stride(0) % 8 == 0
                and (cos is None or 2 * cos.shape[1] == head_dim)
                and (q_weight is None) == (k_weight is None))

    def paged_attention_decode(self, q, q_stride, *, num_heads, num_kv_heads, head_dim, k_pages, v_pages,
                               block_table, kv_lens, cu_seqlens, out, page_size, scale, window, num_seqs,
                               max_kv_len, seq_list=None, num_splits=None, new_token=None, step=None,
                               merge_kernel=False, longest=None, keep_first=0, sink=None, gate=None, softcap=None):
        """Split-KV attention for sequences that bring one token each (csrc/attention_decode.cu).
        ``new_token`` (q_weight, k_weight, eps, cos, sin, optionally pairing and values_are_keys): ``q`` is
        the raw q/k/v projection (q/k only with values_are_keys: a key head as projected is its value) and the
        kernel also does the work of :meth:`qk_norm_rope_store` for the newest position of each sequence,
        ``kv_lens - 1``.  The slices of a sequence and kv head are merged
        by whichever of their blocks finishes last (a ticket word per pair); ``merge_kernel=True``
        asks for the second kernel that callers without ticket words get (the bits are the same).
        ``num_splits`` is the slice count of the longest sequence (a shorter one gets fewer slices of
        about the same length); ``longest``: a device int32 holding the longest of the sequences'
        lengths, when the caller has it (else every block works it out from ``kv_lens``).
        ``keep_first``, ``sink``, ``gate``, ``softcap``: as in :meth:`paged_attention`."""
        if out.dtype != torch.bfloat16 or head_dim not in (64, 128, 256) or num_heads // num_kv_heads > 16:
            raise KernelError("paged_attention_decode: bfloat16, head_dim 64/128/256 and groups of at most 16 only")
        keep_first = int(keep_first or 0) if window else 0
        if window:
            max_kv_len = min(max_kv_len, int(window) + keep_first + 63)
        splits = num_splits or self.decode_splits(num_seqs, num_kv_heads, max_kv_len, head_dim)
        mid_o = mid_lse = None
        tickets = None
        if splits > 1:
            mid_o = torch.empty((num_seqs, num_heads, splits, head_dim), dtype=torch.float32, device=out.device)
            mid_lse = torch.empty((num_seqs, num_heads, splits), dtype=torch.float32, device=out.device)
            if not merge_kernel and num_seqs * num_kv_heads <= self.TICKETS:
                if self._tickets is None:  # zero between launches: the kernel leaves them so
                    self._tickets = torch.zeros(self.TICKETS, dtype=torch.int32, device=out.device)
                tickets = self._tickets
            else:
                self.launches += 1  # the merge kernel
        err = _ptr(self._error_word(out.device))
        if self.timing is not None and step is not None:
            self._costs(*self._attention_cost(step, num_heads, num_kv_heads, head_dim, out, prompts=False))
        if new_token is not None:
            cos, sin = new_token["cos"], new_token["sin"]
            self._call("attention_decode", "q3_paged_attention_decode_fused_sink", "paged_attention_decode_fused",
                       _ptr(q), q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                       _ptr(kv_lens), _ptr(cu_seqlens), _ptr(seq_list), _ptr(out), _ptr(mid_o), _ptr(mid_lse),
                       num_seqs, num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0),
                       splits, _ptr(new_token["q_weight"]), _ptr(new_token["k_weight"]), float(new_token["eps"]),
                       _ptr(cos), _ptr(sin), cos.shape[0] if cos is not None else 0,
                       self.PAIRINGS[new_token.get("pairing", "half")], err, _ptr(tickets), _ptr(longest),
                       keep_first, int(sink is not None), float(sink or 0.0), _ptr(gate),
                       gate.stride(0) if gate is not None else 0, float(softcap or 0.0),
                       int(bool(new_token.get("values_are_keys"))))
            return out
        self._call("attention_decode", "q3_paged_attention_decode_sink", "paged_attention_decode",
                   _ptr(q), q_stride, _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                   _ptr(kv_lens), _ptr(cu_seqlens), _ptr(seq_list), _ptr(out), _ptr(mid_o), _ptr(mid_lse),
                   num_seqs, num_heads, num_kv_heads, head_dim, page_size, float(scale), int(window or 0), splits,
                   _ptr(tickets), _ptr(longest), keep_first, int(sink is not None), float(sink or 0.0), _ptr(gate),
                   gate.stride(0) if gate is not None else 0, float(softcap or 0.0))
        return out

    # ---- matrix products ----------------------------------------------------------------
    def linear(self, x, weight, out=None, out_dtype=None, partial_sums=False, bias=None):
        """See :meth:`_product`; ``bias`` (float32 ``[N]``) is added to the finished product, which
        then never comes as partial sums."""
        if bias is None:
            return self._product(x, weight, out, out_dtype, partial_sums)
        return self.add_bias(self._product(x, weight, out, out_dtype, False), bias)

    def _product(self, x, weight, out=None, out_dtype=None, partial_sums=False):
        """``x[M, K] @ weight[N, K]^T``.  float32: this engine's FMA kernel (no TF32).
        bfloat16, at most 16 tokens: one of this engine's two weight-streaming kernels
        (:meth:`_small_product`).  bfloat16, more tokens: the library product with fp32
        accumulation, as the reference's ``nn.Linear`` (qwen3_runtime/models/qwen3.py:76-77,
        134-135), or this engine's tcgen05 kernel with ``large_gemm="tcgen05"``.

        ``partial_sums``: the caller also takes float32 ``[parts, M, N]`` whose sum over the
        first axis is the product (what :meth:`fused_norm` accepts as ``pending``).  It gets
        that when the streaming kernel would cut K into ranges: the blocks then need not
        wait for one another to add their parts up."""
        M, K = x.shape
        N = weight.shape[0]
        if weight.shape[1] != K:
            raise KernelError(f"linear: x is [{M},{K}] but weight is {list(weight.shape)}")
        if self.timing is not None:
            e = x.element_size()
            oe = 4 if out_dtype == torch.float32 else e
            self._costs(N * K * e + M * K * e + M * N * oe, 2.0 * M * N * K, f" {M}x{K}->{N}")
        if (partial_sums and self.partial_sums and out is None and out_dtype is None and M > 0
                and self.small_gemm != "registers" and self._small_m_ok(x, weight)):
            parts = self._stream_parts(M, N, K)
            if parts > 1:
                planes = torch.empty((parts, M, N), dtype=torch.float32, device=x.device)
                self._call("gemm_stream", "q3_gemm_stream_partial", "gemm_stream_partial", _ptr(x), x.stride(0),
                           _ptr(weight), weight.stride(0), _ptr(planes), parts, M, N, K,
                           _ptr(self._error_word(x.device)))
                return planes
        if x.dtype == torch.float32:
            if out is None:
                out = torch.empty((M, N), dtype=torch.float32, device=x.device)
            self._call("gemm_f32", "q3_gemm_f32", "gemm_f32", _ptr(x), x.stride(0), _ptr(weight),
                       weight.stride(0), _ptr(out), out.stride(0), M, N, K)
            return out
        if self._small_m_ok(x, weight):
            odt = out_dtype or x.dtype
            if out is None:
                out = torch.empty((M, N), dtype=odt, device=x.device)
            self._small_product(1 if odt == torch.float32 else 0, x, weight, out, M, N, K)
            return out
        if self.large_gemm == "tcgen05" and self._tcgen05_ok(x, weight):
            return self.linear_tcgen05(x, weight, out=out, out_dtype=out_dtype)
        if self.timing is not None:
            with self._timed("library_mm"):
                return self._library_mm(x, weight, out, out_dtype)
        return self._library_mm(x, weight, out, out_dtype)

    @staticmethod
    def _library_mm(x, weight, out, out_dtype):
        if out_dtype is not None and out_dtype != x.dtype:
            if out is not None:
                return torch.mm(x, weight.t(), out_dtype=out_dtype, out=out)
            return torch.mm(x, weight.t(), out_dtype=out_dtype)
        if out is None:
            return torch.mm(x, weight.t())
        return torch.mm(x, weight.t(), out=out)

    def _tcgen05_ok(self, x, weight) -> bool:
        return (x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
                and weight.stride(0) % 8 == 0 and x.stride(1) == 1 and weight.stride(1) == 1
                and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)

    ERR_POSITION = 16  # csrc/rope_kv.cu, csrc/attention_decode.cu: a position outside the rotation tables

    def _error_word(self, device) -> torch.Tensor:
        if getattr(self, "_err", None) is None:
            self._err = torch.zeros(1, dtype=torch.int32, device=device)
        return self._err

    def raise_if_kernel_error(self) -> None:
        """A bounded wait inside a kernel expired (it gave up and returned).  Reads one int from
        the device, so call it where the host waits for the device anyway."""
        err = getattr(self, "_err", None)
        code = int(err.item()) if err is not None else 0
        if code == self.ERR_POSITION:
            err.zero_()
            raise KernelError("a token's position lies outside the rotation tables of the position encoding: "
                              "its query and key were left unrotated and the step's output is invalid")
        if code != 0:
            err.zero_()
            if self._tickets is not None:  # a kernel that gave up may have left tickets drawn
                self._tickets.zero_()
            if self._argmax_tickets is not None:
                self._argmax_tickets.zero_()
            raise KernelError("a bounded wait inside a kernel expired (tcgen05 product or attention, or the "
                              "streaming product): the kernel gave up and its output is invalid")

    def watch_kernel_errors(self) -> None:
        """Enqueue a copy of the error word to pinned host memory, without waiting for it.
        :meth:`raise_if_watched_error` looks at the copy once the host has waited for the
        device for a reason of its own (the sampled tokens), so a step pays no extra wait."""
        err = getattr(self, "_err", None)
        if err is None:
            return
        if getattr(self, "_err_host", None) is None:
            self._err_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self._err_host.copy_(err, non_blocking=True)

    def raise_if_watched_error(self) -> None:
        host = getattr(self, "_err_host", None)
        if host is not None and int(host[0]) != 0:
            host.zero_()
            self.raise_if_kernel_error()

    def linear_tcgen05(self, x, weight, out=None, out_dtype=None, mode=None, pair=None):
        """``x @ weight^T`` on tcgen05 tensor cores (csrc/gemm_tcgen05.cu).  ``mode=2``: SwiGLU with
        ``weight = [W_gate; W_up]``, ``out`` is ``[M, I]``.  ``pair``: the kernel that runs each
        256-token tile on two SMs (cta_group::2); default: when there are more than 128 tokens."""
        M, K = x.shape
        if not self._tcgen05_ok(x, weight):
            raise KernelError("gemm_tcgen05: bfloat16 operands with 16-byte aligned rows (K multiple of 8) only")
        if mode == 2:
            N = weight.shape[0] // 2
            odt = x.dtype
        else:
            N = weight.shape[0]
            odt = out_dtype or x.dtype
            mode = 1 if odt == torch.float32 else 0
        if out is None:
            out = torch.empty((M, N), dtype=odt, device=x.device)
        if pair is None:
            pair = self.tcgen05_pairs and M > 128 and self._tcgen05_plan(M, N)[0]
        self._call("gemm_tcgen05", "q3_gemm_tcgen05_pair" if pair else "q3_gemm_tcgen05", "gemm_tcgen05", mode,
                   _ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K,
                   _ptr(self._error_word(x.device)))
        return out

    def _tcgen05_plan(self, M: int, N: int) -> tuple[bool, float, float]:
        """(whether pairs of SMs should run the tiles, share of the token rows of the tiles that holds
        real tokens, share of the tile slots of all rounds that holds real work).  Both kernels work
        through their tiles in rounds over all SMs: 128 tokens x 128 features (of each of gate and up
        for SwiGLU) per SM, or 256 x 128 per pair.  A token count just above a multiple of the tile
        leaves most of the last token tile empty, a tile count just above a multiple of the SMs most of
        the last round."""
        cols = -(-N // 128)
        pairs = self.SM_COUNT // 2
        fill_1, fill_2 = M / (-(-M // 128) * 128), M / (-(-M // 256) * 256)
        single = (M / 128) * cols / (-(-(-(-M // 128) * cols) // self.SM_COUNT) * self.SM_COUNT)
        paired = (M / 256) * cols / (-(-(-(-M // 256) * cols) // pairs) * pairs)
        return (True, fill_2, paired) if paired >= single else (False, fill_1, single)

    SMALL_M = 16
    # The fused gate_up + SwiGLU product goes to the tcgen05 kernel when its token tiles are at least
    # this full and its rounds at least that full; else to the library product and a SwiGLU pass.
    # Measured at 129..4096 tokens x three model sizes: the library, with finer token tiles, wins
    # clearly (20-50 %) when the last token tile is mostly empty or the work fills less than a round
    # and a half; where only the last round is thin the two are within a few percent and the fused
    # kernel saves a launch and a pass over [tokens, 2 x intermediate].
    TCGEN05_MIN_TOKEN_FILL = 0.9
    TCGEN05_MIN_SHARE = 0.65

    def _stream_parts(self, M: int, N: int, K: int) -> int:
        """Ranges of K in the streaming kernel's partial-sum mode (0: it does not take the product)."""
        key = (M > 8, N, K)
        parts = self._parts_cache.get(key)
        if parts is None:
            parts = self._parts_cache[key] = int(self._get("gemm_stream", "q3_gemm_stream_parts")(M, N, K))
        return parts

    def _small_product(self, mode: int, x, weight, out, M, N, K) -> None:
        """A product of at most 16 tokens: the streaming kernel (csrc/gemm_stream.cu), or the
        register-streaming one (csrc/gemm_small_m.cu) for what the first refuses."""
        if self.small_gemm != "registers":
            self.launches += 1
            cost, span = self._cost, None
            if self.timing is not None:
                span = self._timed("gemm_stream").__enter__()
            code = self._get("gemm_stream", "q3_gemm_stream")(
                mode, _ptr(x), x.stride(0), _ptr(weight), weight.stride(0), _ptr(out), out.stride(0), M, N, K,
                int(self.small_gemm == "auto"), _ptr(self._error_word(x.device)), self._stream())
            if code == 0:
                if span is not None:
                    span.__exit__()
                return
            self._cost = cost  # refused before any launch: the register kernel takes the product
            self.launches -= 1
            if code != 1:
                _check(code, "gemm_stream")
        self._call("gemm_small_m", "q3_gemm_small_m", "gemm_small_m", mode, _ptr(x), x.stride(0), _ptr(weight),
                   weight.stride(0), _ptr(out), out.stride(0), M, N, K)

    def _small_m_ok(self, x, weight) -> bool:
        return (x.dtype == torch.bfloat16 and x.shape[0] <= self.SMALL_M and x.shape[1] % 8 == 0
                and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.stride(1) == 1
                and weight.stride(1) == 1 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)

    def gated_linear(self, x, gate_up_weight, out):
        """``out = silu(x @ W_gate^T) * (x @ W_up^T)`` with ``gate_up_weight = [W_gate; W_up]``:
        one kernel for a handful of tokens, else the product followed by the SwiGLU kernel."""
        M, K = x.shape
        I = out.shape[1]
        if self.timing is not None:
            e = x.element_size()
            self._costs((2 * I * K + M * K + M * I) * e, 4.0 * M * I * K, f" {M}x{K}->2x{I} swiglu")
        if self._small_m_ok(x, gate_up_weight):
            self._small_product(2, x, gate_up_weight, out, M, I, K)
            return out
        if self.large_gemm != "library" and self._tcgen05_ok(x, gate_up_weight):
            _pair, token_fill, share = self._tcgen05_plan(M, I)
            if self.large_gemm == "tcgen05" or (token_fill >= self.TCGEN05_MIN_TOKEN_FILL
                                                and share >= self.TCGEN05_MIN_SHARE):
                return self.linear_tcgen05(x, gate_up_weight, out=out, mode=2)
        return self.silu_mul(self.linear(x, gate_up_weight), out)

    # ---- sampling ---------------------------------------------------------------------
    def argmax(self, logits, want_logprob=False):
        R, V = logits.shape
        if self.timing is not None:
            self._costs(R * V * 4)
        token = torch.empty(R, dtype=torch.int32, device=logits.device)
        logprob = torch.empty(R, dtype=torch.float32, device=logits.device) if want_logprob else None
        slices, scratch, tickets = self._row_slices(logits)
        self._call("sampling", "q3_argmax", "argmax",
                   _ptr(logits), R, V, _ptr(token), _ptr(logprob), _ptr(scratch), _ptr(tickets), slices)
        return token, logprob

    def _row_slices(self, logits):
        """Few long rows: cut each into slices so that about two blocks per SM share the work; the
        slices' results meet in a scratch, and a ticket word per row tells the last block."""
        R, V = logits.shape
        slices = max(0, min(1024, 2 * self.SM_COUNT // max(R, 1), V // 2048))
        if slices <= 1 or R > self.TICKETS:
            return 0, None, None
        if self._argmax_tickets is None:  # zero between launches: the kernels leave them so
            self._argmax_tickets = torch.zeros(self.TICKETS, dtype=torch.int32, device=logits.device)
        scratch = torch.empty((R, slices, 4), dtype=torch.float32, device=logits.device)
        return slices, scratch, self._argmax_tickets

    def sample(self, logits, temperature, uniform, want_logprob=False):
        R, V = logits.shape
        token = torch.empty(R, dtype=torch.int32, device=logits.device)
        logprob = torch.empty(R, dtype=torch.float32, device=logits.device) if want_logprob else None
        slices, scratch, tickets = self._row_slices(logits)
        if self.timing is not None:
            self._costs(R * V * 4)
        self._call("sampling", "q3_sample", "sample", _ptr(logits), R, V, _ptr(temperature), _ptr(uniform),
                   _ptr(token), _ptr(logprob), _ptr(scratch), _ptr(tickets), slices)
        return token, logprob


    def bias_penalty_row(self, row, *, logit_bias, seen_ids, repetition_penalty, presence_penalty,
                         frequency_penalty):
        """Logit bias and repetition / presence / frequency penalties, in place on one fp32 row
        (qwen3_runtime/sampling.py:36-72)."""
        V = row.numel()
        dev = row.device
        bias_ids = bias_vals = seen = counts = None
        n_bias = n_seen = 0
        if logit_bias:
            n_bias = len(logit_bias)
            bias_ids = torch.tensor([int(k) for k in logit_bias], dtype=torch.int32, device=dev)
            bias_vals = torch.tensor([float(v) for v in logit_bias.values()], dtype=torch.float32, device=dev)
        if seen_ids and not (repetition_penalty == 1.0 and presence_penalty == 0.0 and frequency_penalty == 0.0):
            n_seen = len(seen_ids)
            seen = torch.tensor(seen_ids, dtype=torch.int32, device=dev)
            counts = torch.empty(V, dtype=torch.int32, device=dev)
        self._call("sampling", "q3_bias_penalty", "bias_penalty", _ptr(row), V, _ptr(bias_ids), _ptr(bias_vals),
                   n_bias, _ptr(seen), n_seen, _ptr(counts), float(repetition_penalty), float(presence_penalty),
                   float(frequency_penalty))
        return row

    def bias_penalty_rows(self, logits, rows, *, logit_bias, seen_ids, repetition_penalty, presence_penalty,
                          frequency_penalty):
        """:meth:`bias_penalty_row` for several rows of ``logits`` at once (lists with one entry per
        row of ``rows``): everything the rows need goes to the device as one integer and one float
        buffer, and one launch with a block per row works on them."""
        n, V, dev = len(rows), logits.shape[1], logits.device
        biases = [b or {} for b in logit_bias]
        ints, bias_off, seen_off = list(int(r) for r in rows), [0], [0]
        for b in biases:
            bias_off.append(bias_off[-1] + len(b))
        for s, rp, pp, fp in zip(seen_ids, repetition_penalty, presence_penalty, frequency_penalty):
            live = bool(s) and not (rp == 1.0 and pp == 0.0 and fp == 0.0)
            seen_off.append(seen_off[-1] + (len(s) if live else 0))
        packed = ints + bias_off + seen_off
        packed += [int(k) for b in biases for k in b]
        packed += [int(t) for s, a, z in zip(seen_ids, seen_off, seen_off[1:]) if z > a for t in s]
        floats = [float(v) for triple in zip(repetition_penalty, presence_penalty, frequency_penalty) for v in triple]
        floats += [float(v) for b in biases for v in b.values()]
        host_i = torch.tensor(packed, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        host_f = torch.tensor(floats, dtype=torch.float32).pin_memory().to(dev, non_blocking=True)
        counts = torch.empty((n, V), dtype=torch.int32, device=dev)
        o_bias, o_seen = n, 2 * n + 1
        o_bias_ids = 3 * n + 2
        o_seen_ids = o_bias_ids + bias_off[-1]
        self._call("sampling", "q3_bias_penalty_rows", "bias_penalty_rows", _ptr(logits), V, n, _ptr(host_i),
                   _ptr(host_i[o_bias:]), _ptr(host_i[o_bias_ids:]) if bias_off[-1] else None,
                   _ptr(host_f[3 * n:]) if bias_off[-1] else None, _ptr(host_i[o_seen:]),
                   _ptr(host_i[o_seen_ids:]) if seen_off[-1] else None, _ptr(counts), _ptr(host_f))
        return logits

    def filter_rows(self, logits, temperature, min_p, top_k, top_p):
        """Divide by the temperature, then min_p, top_k and top_p masks, in place on fp32 rows
        (qwen3_runtime/sampling.py:75-109, 130-135).  The four arguments are per-row device tensors."""
        R, V = logits.shape
        self._call("sampling", "q3_filter", "filter", _ptr(logits), R, V, _ptr(temperature), _ptr(min_p),
                   _ptr(top_k), _ptr(top_p))
        return logits


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
