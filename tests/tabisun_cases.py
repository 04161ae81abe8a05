"""Tabisun: engine and parts against the plain statement (tests/plain_tabisun.py), written once and run
on the CPU with the torch statements of the kernels and on the GPU with the kernels."""

from __future__ import annotations

import json
import math

import torch

import plain_tabisun as pl
from helpers import (first_mismatch, max_abs_diff, peak_tokens, random_ids, run_trace, trace_mixed, trace_portions,
                     trace_tail_decode, trace_whole)
from puladra_cases import _random_tensors, _step, _tolerance, _views_for
from qwen3_runtime_b200.config import PartSpec, TabisunConfig
from qwen3_runtime_b200.config.tabisun_config import (DifferentialConfig, KeyValueConfig, LatentConfig, RotaryConfig,
                                                      TabisunLayerConfig)
from qwen3_runtime_b200.engine.factory import build_engine, build_runtime, load_model
from qwen3_runtime_b200.parts import BuildContext, ResidualStream, build_part
from qwen3_runtime_b200.weights import write_random_model

TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
L = TabisunLayerConfig


def _wave(factor, low, high, original):
    return (("factor", factor), ("low", low), ("high", high), ("original", original))


def _ramp(factor, original, fast, slow):
    return (("factor", factor), ("original", original), ("fast", fast), ("slow", slow))


def _diff(**kw):
    base = dict(heads=4, kv_heads=2, dim=12, vdim=20, scale=0.3, diff=0.35, chunk=20)
    base.update(kw)
    return DifferentialConfig(**base)


def _kv(**kw):
    base = dict(heads=6, kv_heads=3, dim=24, vdim=24, scale=0.25, softcap=8.0,
                rot=RotaryConfig(dims=24, base=1e4, scaling=_wave(4.0, 1.0, 4.0, 64.0)))
    base.update(kw)
    if base["vdim"] != base["dim"]:
        base["vdim"] = base["dim"]
    return KeyValueConfig(**base)


def _latent(**kw):
    base = dict(heads=3, dim=20, rot_dim=12, vdim=28, kv_rank=44, scale=0.2,
                rot=RotaryConfig(dims=12, base=5e4, scaling=_ramp(6.0, 40.0, 8.0, 1.0)))
    base.update(kw)
    return LatentConfig(**base)


# Sizes no two of which are equal where the design lets them differ: key and value sizes, head counts with
# and without groups, a key size that is no multiple of 8, chunks that are no multiple of the page, of one
# token, larger than any request and absent; rotation over the whole head and over a part of it, with and
# without rescaling, wavelengths in all three bands; layers that run another layer's weights (also twice the
# same one), layers without a feed-forward, every order of the three mixers; capped and uncapped logits.
_D_DIFF = _diff(heads=4, kv_heads=1, dim=64, vdim=128, scale=0.125, diff=0.5, chunk=48)
_D_KV = _kv(heads=8, kv_heads=2, dim=64, scale=0.125, softcap=30.0,
            rot=RotaryConfig(dims=32, base=5e5, scaling=_wave(8.0, 1.0, 4.0, 256.0)))
_D_LATENT = _latent(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, scale=0.15,
                    rot=RotaryConfig(dims=16, base=1e4, scaling=_ramp(4.0, 128.0, 32.0, 1.0)))
_B_KV = _kv(heads=4, kv_heads=4, dim=16, scale=0.3, softcap=None, rot=RotaryConfig(dims=8, base=300.0))
CONFIGS = {
    "A": dict(page_size=8, seed=51, config=TabisunConfig(
        vocab=150, width=72, norm_eps=1e-5, logit_softcap=9.0,
        layers=(L("attention", _diff(), 56), L("attention_2", _kv(), 40), L("latent_attention", _latent(), None),
                L("attention", _diff(), 56, weights_of=0), L("latent_attention", _latent(), None, weights_of=2)))),
    "B": dict(page_size=4, seed=52, config=TabisunConfig(
        vocab=131, width=64, norm_eps=1e-6, logit_softcap=None,
        layers=(L("attention_2", _B_KV, None),
                L("attention", _diff(heads=2, kv_heads=1, dim=16, vdim=16, diff=0.3, chunk=1, scale=0.2), 48),
                L("latent_attention", _latent(heads=1, dim=8, rot_dim=4, vdim=8, kv_rank=16,
                                              rot=RotaryConfig(dims=4, base=100.0)), 24),
                L("attention_2", _B_KV, None, weights_of=0), L("attention_2", _B_KV, None, weights_of=0)))),
    "C": dict(page_size=16, seed=53, config=TabisunConfig(
        vocab=90, width=48, norm_eps=1e-5, logit_softcap=30.0,
        layers=(L("latent_attention", _latent(heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=32,
                                              rot=RotaryConfig(dims=16, base=1e4, scaling=_ramp(2.0, 16.0, 4.0, 2.0))), 32),
                L("attention", _diff(heads=2, kv_heads=2, dim=16, vdim=24, chunk=33, diff=0.1), 24),
                L("attention", _diff(heads=3, kv_heads=1, dim=8, vdim=40, chunk=None, diff=0.6), None),
                L("attention_2", _kv(heads=2, kv_heads=1, dim=40, softcap=3.0,
                                     rot=RotaryConfig(dims=40, base=50.0, scaling=_wave(16.0, 1.0, 2.0, 24.0))), 40)))),
    # sizes the bfloat16 tensor-core paths take (multiples of 16 everywhere, heads of 64)
    "D": dict(page_size=16, seed=54, config=TabisunConfig(
        vocab=210, width=128, norm_eps=1e-5, logit_softcap=20.0,
        layers=(L("attention_2", _D_KV, 96), L("latent_attention", _D_LATENT, 64), L("attention", _D_DIFF, 96),
                L("attention_2", _D_KV, 96, weights_of=0)))),
}

STD = 0.15  # spread of the random matrices: attention and the feed-forward have to matter


def make_dir(tmp_path, name):
    spec = CONFIGS[name]
    folder = tmp_path / f"tabisun_{name}"
    if not (folder / "model.safetensors").exists():
        from safetensors.torch import load_file, save_file

        write_random_model(spec["config"], folder, spec["seed"], std=STD, vector_std=0.1)
        t = load_file(str(folder / "model.safetensors"))
        for k in t:
            x = t[k].float()
            if k.split(".")[-1] in ("lq1", "lk1", "lq2", "lk2"):  # around zero: lambda stays of order one
                x = (x - 1.0) * 2.5
            elif k.endswith(".sink"):  # sinks that take a visible share of the weight, some negative
                x = (x - 1.0) * 20.0 + 1.0
            elif k == "embed":
                x = x * 6.0
            elif k.endswith((".q", ".k")):  # sharper scores
                x = x * 2.0
            t[k] = x.to(t[k].dtype)
        save_file(t, str(folder / "model.safetensors"))
    return folder


def read_dir(folder):
    from safetensors.torch import load_file

    return json.loads((folder / "config.json").read_text()), load_file(str(folder / "model.safetensors"))


def expected(folder, requests, dtype):
    """Plain logits per request and the tolerance: float32 a few 1e-5 of the logits' size; bfloat16 three
    times the distance between the plain statement with bfloat16 activations and the exact one."""
    raw, t = read_dir(folder)
    exact = {rid: pl.forward(raw, t, toks).float() for rid, toks in requests.items()}
    scale = max(float(v.abs().max()) for v in exact.values())
    if dtype == "float32":
        return exact, 5e-5 * max(1.0, scale)
    rounded = {rid: pl.forward(raw, t, toks, activations=torch.bfloat16).float() for rid, toks in requests.items()}
    noise = max(float((rounded[r] - exact[r]).abs().max()) for r in exact)
    return exact, 3.0 * noise


def runtime(folder, name, dtype, ops, device, pages, max_live=4, cuda_graph=False):
    model, _cfg, _ = load_model(folder, dtype=dtype, device=device, ops=ops)
    return build_runtime(model, block_size=CONFIGS[name]["page_size"], num_kv_blocks=pages, max_num_seqs=max_live,
                         cuda_graph=cuda_graph)


def requests_for(name, lengths, seed=0):
    vocab = CONFIGS[name]["config"].vocab
    return {f"r{i}": random_ids(vocab, n, 1000 * seed + i) for i, n in enumerate(lengths)}


def check(got, want, tol, what):
    bad = first_mismatch(got, want, tol)
    assert bad is None, f"{what}: request {bad[0]} position {bad[1]} differs by {bad[2]:.3g} (tolerance {tol:.3g})"
    print(f"{what}: worst difference {max_abs_diff(got, want):.3g} (tolerance {tol:.3g})")


def case_schedules(tmp_path, name, dtype, ops, device, lengths=(75, 9, 41, 2, 58, 1, 30), cuda_graph=False):
    """Whole prompts; the tail decoded token by token; portions down to two tokens; unequal requests side by
    side with pages and slots freed and used again (pages poisoned in between)."""
    folder = make_dir(tmp_path, name)
    requests = requests_for(name, lengths)
    want, tol = expected(folder, requests, dtype)
    ps = CONFIGS[name]["page_size"]
    results = {}
    for kind, steps in (("whole", trace_whole(requests)), ("tail", trace_tail_decode(requests, tail=30)),
                        ("portions", trace_portions(requests, seed=3)), ("mixed", trace_mixed(requests, seed=5))):
        rt = runtime(folder, name, dtype, ops, device, pages=-(-peak_tokens(steps, 64) // ps), cuda_graph=cuda_graph)
        results[kind] = run_trace(rt, steps, poison=True)
        check(results[kind], want, tol, f"{name} {dtype} {kind}")
        assert rt.cache.num_free_pages == rt.cache.num_pages
        assert rt.cache.slots.num_free == rt.cache.slots.num_slots
        assert sum(len(v) for v in results[kind].values()) == sum(lengths)
    whole = {rid: torch.stack([rows[p] for p in sorted(rows)]) for rid, rows in results["whole"].items()}
    cut_tol = tol if dtype == "bfloat16" else 2e-5 * max(1.0, max(float(v.abs().max()) for v in whole.values()))
    for kind in ("tail", "portions", "mixed"):
        check(results[kind], whole, cut_tol, f"{name} {dtype} {kind} against whole")


def case_residual_after_every_run(tmp_path, name, ops, device):
    """The stream after every layer run (a layer that runs another's weights counts by itself) against the
    plain model's."""
    folder = make_dir(tmp_path, name)
    raw, t = read_dir(folder)
    toks = requests_for(name, (23,), seed=4)["r0"]
    _logits, want = pl.forward(raw, t, toks, with_streams=True)
    rt = runtime(folder, name, "float32", ops, device, pages=-(-64 // CONFIGS[name]["page_size"]))
    got: list = []

    def watched(block, forward):
        def run(stream, step, cache):
            forward(stream, step, cache)
            # what the block left for the next kernel to norm and add
            weight, eps = stream.pending_norm[0], stream.pending_norm[1]
            y = stream.pending.float().cpu().double()
            y = pl.layer_norm(y, weight.cpu().double(), eps)
            got.append(stream.resid.cpu().double() + y)
        return run

    for block in rt.runner.model.blocks:
        block.forward = watched(block, block.forward)
    run_trace(rt, trace_whole({"r0": toks}))
    assert len(got) == len(want) == len(CONFIGS[name]["config"].layers)
    for run, (g, w) in enumerate(zip(got, want)):
        diff = float((g - w).abs().max())
        assert diff <= 3e-5 * max(1.0, float(w.abs().max())), f"{name}: stream after run {run} off by {diff:.3g}"


def case_long_decode(tmp_path, name, dtype, ops, device, total=150, cuda_graph=False):
    """A short prompt and then one token at a time, over many chunks and pages."""
    folder = make_dir(tmp_path, name)
    requests = requests_for(name, (total,), seed=7)
    want, tol = expected(folder, requests, dtype)
    toks = requests["r0"]
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": toks[:3], "want": [0, 1, 2]}], "end": []}]
    steps += [{"step": i - 2, "entries": [{"id": "r0", "tokens": [toks[i]], "want": [0]}],
               "end": ["r0"] if i == total - 1 else []} for i in range(3, total)]
    rt = runtime(folder, name, dtype, ops, device, pages=-(-(total + 63) // CONFIGS[name]["page_size"]),
                 cuda_graph=cuda_graph)
    check(run_trace(rt, steps), want, tol, f"{name} {dtype} long decode")
    assert rt.cache.num_free_pages == rt.cache.num_pages


def case_first_tokens(tmp_path, name, dtype, ops, device):
    """One-, two- and three-token sequences side by side, then sequences fed one token at a time from their
    first in the slots and pages the others left: a sink beside a single key, chunks not yet full."""
    folder = make_dir(tmp_path, name)
    requests = requests_for(name, (1, 2, 3, 1), seed=9)
    want, tol = expected(folder, requests, dtype)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in requests.items()],
              "end": list(requests)}]
    rt = runtime(folder, name, dtype, ops, device, pages=32)
    check(run_trace(rt, steps, poison=True), want, tol, f"{name} {dtype} first tokens")
    again = requests_for(name, (6, 5), seed=10)
    want, tol = expected(folder, again, dtype)
    steps = [{"step": i, "entries": [{"id": r, "tokens": [t[i]], "want": [0]} for r, t in again.items() if i < len(t)],
              "end": [r for r, t in again.items() if i == len(t) - 1]} for i in range(6)]
    check(run_trace(rt, steps), want, tol, f"{name} {dtype} first tokens one by one in used pages")


def case_greedy_generation(tmp_path, name, dtype, ops, device, cuda_graph=False, steps=12):
    """Greedy generation through the engine's own entry point, scheduler and sampler: unequal prompts side by
    side in a small pool, every token checked at its own place against the plain model given the tokens
    before it."""
    folder = make_dir(tmp_path, name)
    raw, t = read_dir(folder)
    prompts = list(requests_for(name, (17, 3, 29, 8), seed=13).values())
    engine = build_engine(folder, dtype=dtype, device=device, ops=ops, block_size=CONFIGS[name]["page_size"],
                          num_kv_blocks=-(-4 * 64 // CONFIGS[name]["page_size"]), max_num_seqs=3,
                          max_num_batched_tokens=24, cuda_graph=cuda_graph)
    outs = engine.generate_batch(prompts, max_tokens=steps)
    for prompt, out in zip(prompts, outs):
        assert len(out) == steps
        seq = list(prompt) + list(out[:-1])
        exact = pl.forward(raw, t, seq).float()[len(prompt) - 1:]
        if dtype == "float32":
            tol = 1e-4 * max(1.0, float(exact.abs().max()))
        else:
            rows = pl.forward(raw, t, seq, activations=torch.bfloat16).float()[len(prompt) - 1:]
            tol = 2 * 3.0 * float((rows - exact).abs().max())
        for i, tok in enumerate(out):
            gap = float(exact[i].max() - exact[i][tok])
            assert gap <= tol, f"token {i} ({tok}) is {gap:.3g} below the plain argmax (allowed {tol:.3g})"
    engine.runtime.cache.check_invariants()
    assert engine.runtime.cache.num_free_pages == engine.runtime.cache.num_pages


# ---- parts and kernels alone ---------------------------------------------------------------------

def _mixer_part(kind, width, eps, sizes, ctx):
    """The part of one mixer kind as the model builds it, with its plain statement ``plain(h, tensors)``."""
    from qwen3_runtime_b200.models.tabisun import _mixer_spec

    cfg = TabisunConfig(vocab=8, width=width, norm_eps=eps,
                        layers=(L(kind, {"attention": _diff, "attention_2": _kv, "latent_attention": _latent}[kind](**sizes),
                                  None),))
    m = cfg.layers[0].mixer
    plain = {"attention": pl.differential_attention, "attention_2": pl.key_value_attention,
             "latent_attention": pl.latent_attention}[kind]
    raw = m.to_raw()
    return build_part("mixer", _mixer_spec(cfg, m), ctx), lambda h, t: plain(h, t, "mix.", raw, eps)


def case_mixer_alone(dtype, ops, device, kind, *, T=45, page_size=8, cuts=(24, 1, 2, 18), **sizes):
    """A mixer on one sequence in portions (one of a single token, one of two) through a paged cache whose
    pages are out of order and hold NaN where nothing was written, against the plain statement on the whole
    sequence."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(5)
    width, eps = 64, 1e-5
    part, plain = _mixer_part(kind, width, eps, sizes, BuildContext(dt, torch.device(device), ops))
    tensors = _random_tensors(part, gen, dt, device)
    for name in ("lq1", "lk1", "lq2", "lk2"):
        if name in tensors:
            tensors[name] = (tensors[name] - 1.0) * 0.8
    if "sink" in tensors:  # large enough to take most of the weight from some heads
        tensors["sink"] = (tensors["sink"] - 1.0) * 10.0 + 2.0
    part.load(tensors)
    h = torch.randn((T, width), generator=gen).to(torch.bfloat16).float()
    want = plain(h.double(), {"mix." + k: v.double().cpu() for k, v in tensors.items()}).float()
    pages_needed = -(-T // page_size)
    table = list(reversed(range(1, pages_needed + 1)))  # not in order, page 0 unused
    spec = part.cache_spec()
    if hasattr(spec, "width"):  # a latent layer: one row per token
        pages = torch.full((pages_needed + 2, page_size, spec.width), float("nan"), dtype=dt, device=device)
        from qwen3_runtime_b200.cache.storage import CacheLayerView

        cache = CacheLayerView(0, 0, page_size, None, None, None, None, True, latent_pages=pages)
    else:
        cache = _views_for(spec, device, dt, page_size, pages_needed + 2, slots=3)
    got, lo = [], 0
    assert sum(cuts) == T
    for n in cuts:
        step = _step(list(range(lo, lo + n)), [0] * n, [table], device, slots=[2])
        got.append(part.forward(h[lo:lo + n].to(device=device, dtype=dt), step, cache).float().cpu())
        lo += n
    got = torch.cat(got)
    tol = _tolerance(dtype, want)
    diff = float((got - want).abs().max())
    assert diff <= tol, f"{kind} mixer ({dtype}, {sizes}): off by {diff:.3g} (allowed {tol:.3g})"
    if "sink" in tensors:  # the sink shows: the plain statement with sinks that weigh nothing gives another output
        without = {"mix." + k: v.double().cpu() for k, v in tensors.items()}
        without["mix.sink"] = torch.full_like(without["mix.sink"], -1e4)
        assert float((plain(h.double(), without).float() - want).abs().max()) > 0.02 * float(want.abs().max())


def _paged(x, table, page_size, pages, dt, device):
    """``x`` ``[T, heads, n]`` into NaN-filled pages ``[pages, heads, page_size, n]`` through ``table``."""
    out = torch.full((pages, x.shape[1], page_size, x.shape[2]), float("nan"), dtype=dt, device=device)
    for j in range(x.shape[0]):
        out[table[j // page_size], :, j % page_size] = x[j].to(dt)
    return out


def case_differential_edges(dtype, ops, device, *, chunk=12, page_size=8, heads=4, kv_heads=2, D=12, Dv=20, T=50,
                            lam=0.7):
    """The differential kernel alone with one key that takes nearly all the weight of *one* map when it is seen:
    in the query's chunk it decides that map's sum (so the output moves by the marked value), one position
    before the chunk's start it does not; for queries at a chunk's first, second and last position, at page
    borders, in a whole prompt, a portion of two and a single decoded token.  Pages are out of order and
    unused rows hold NaN."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(17)
    pages_needed = -(-T // page_size)
    table = list(reversed(range(1, pages_needed + 1)))
    cases = []
    for qi in (2 * chunk, 2 * chunk + 1, 3 * chunk - 1, T - 1):
        start = qi // chunk * chunk
        cases += [(chunk, qi, start, which) for which in (0, 1)] + [(chunk, qi, start - 1, 0)]
    cases += [(None, T - 1, 0, 1), (1, T - 1, T - 2, 0), (1, 7, 7, 1), (T + 5, T - 1, 1, 0)]
    for ch, qi, kj, which in cases:
        q = 0.3 * torch.randn((T, heads, 2, D), generator=gen)
        k = 0.3 * torch.randn((T, kv_heads, 2, D), generator=gen)
        v = torch.randn((T, kv_heads, Dv), generator=gen)
        k[kj, :, which, D - 3] += 8.0
        q[qi, :, which, D - 3] += 8.0
        q, k, v = (x.to(torch.bfloat16).float() for x in (q, k, v))
        want = pl.differential_core(q.double(), k.double(), v.double(), 1.0, lam, ch, 1e-5, 0.75).float()
        seen = kj <= qi and (ch is None or kj // ch == qi // ch)
        blind = k.clone()
        blind[kj, :, which, D - 3] -= 8.0
        moved = float((pl.differential_core(q.double(), blind.double(), v.double(), 1.0, lam, ch, 1e-5, 0.75).float()[qi]
                       - want[qi]).abs().max())
        lo_seen = qi // ch * ch if ch else 0
        if qi > lo_seen + 1:  # with a single visible key every softmax is 1 whatever the scores; with two the
            # other key may by chance have nearly the same value after the head's norm
            assert (moved > 0.05) == seen, "the marked key does not stand out as intended"
        k_pages = _paged(k.reshape(T, kv_heads, 2 * D), table, page_size, pages_needed + 2, dt, device)
        v_pages = _paged(v, table, page_size, pages_needed + 2, dt, device)
        for lo, hi in ((0, T), (qi - 1, qi + 1), (qi, qi + 1)):  # a whole prompt; a portion of two; one decoded token
            if lo < 0:
                continue
            step = _step(list(range(lo, hi)), [0] * (hi - lo), [table], device)
            wide = torch.zeros((hi - lo, heads * Dv + 16), dtype=dt, device=device)
            qd = q[lo:hi].reshape(hi - lo, heads * 2 * D).to(device=device, dtype=dt).contiguous()
            ops.differential_attention(qd, qd.stride(0), num_heads=heads, num_kv_heads=kv_heads, map_dim=D, value_dim=Dv,
                                       k_pages=k_pages, v_pages=v_pages, block_table=step.block_tables[0],
                                       token_seq=step.token_seq, positions=step.positions, out=wide[:, 8:8 + heads * Dv],
                                       page_size=page_size, scale=1.0, lam=lam, eps=1e-5, out_scale=0.75, chunk=ch,
                                       step=step)
            out = wide[:, 8:8 + heads * Dv].float().cpu().reshape(hi - lo, heads, Dv)
            diff = float((out - want[lo:hi]).abs().max())
            tol = 3e-5 if dtype == "float32" else 4e-2
            assert diff <= tol, f"chunk {ch}, query {qi}, key {kj} of map {which}, tokens {lo}..{hi}: off by {diff:.3g}"
            assert float(wide[:, :8].abs().max()) == 0 and float(wide[:, 8 + heads * Dv:].abs().max()) == 0


def case_capped_far_key(dtype, ops, device, *, page_size=16, heads=4, kv_heads=2, D=24, T=330, softcap=6.0, chunk=None):
    """Causal attention with capped scores over hundreds of keys, one of which, far back, would take all the
    weight without the cap and takes a bounded share with it; the values have the keys' size.  A whole prompt,
    a portion of two and a single decoded token; with ``chunk`` the same under a chunked mask in the general
    kernel (the far key is then out of sight)."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(19)
    pages_needed = -(-T // page_size)
    table = list(reversed(range(1, pages_needed + 1)))
    for qi, kj in ((T - 1, 5), (T - 1, T - 1 - page_size), (2 * T // 3, 0), (T - 2, T - 3)):
        q = 0.3 * torch.randn((T, heads, D), generator=gen)
        k = 0.3 * torch.randn((T, kv_heads, D), generator=gen)
        v = torch.randn((T, kv_heads, D), generator=gen)
        k[kj, :, 1] += 9.0
        q[qi, :, 1] += 9.0
        q, k, v = (x.to(torch.bfloat16).float() for x in (q, k, v))
        want = pl.capped_core(q.double(), k.double(), v.double(), 0.5, softcap).float()
        uncapped = pl.capped_core(q.double(), k.double(), v.double(), 0.5, None).float()
        assert float((uncapped[qi, 0] - v[kj, 0]).abs().max()) < 0.05  # without the cap the marked key is everything
        assert float((want[qi, 0] - v[kj, 0]).abs().max()) > 0.05  # with it the others keep a share
        assert float((want[qi] - uncapped[qi]).abs().max()) > 0.05
        if chunk:
            vis = pl.chunked(T, chunk)
            s = torch.einsum("ihd,jhd->hij", q.double(), k.double().repeat_interleave(heads // kv_heads, 1)) * 0.5
            s = softcap * torch.tanh(s / softcap)
            want = torch.einsum("hij,jhd->ihd", pl.softmax_rows(s, vis),
                                v.double().repeat_interleave(heads // kv_heads, 1)).float()
        k_pages = _paged(k, table, page_size, pages_needed + 2, dt, device)
        v_pages = _paged(v, table, page_size, pages_needed + 2, dt, device)
        for lo, hi in ((0, T), (qi - 1, qi + 1), (qi, qi + 1)):
            step = _step(list(range(lo, hi)), [0] * (hi - lo), [table], device)
            out = torch.zeros((hi - lo, heads * D), dtype=dt, device=device)
            qd = q[lo:hi].reshape(hi - lo, heads * D).to(device=device, dtype=dt).contiguous()
            ops.paged_attention(qd, qd.stride(0), num_heads=heads, num_kv_heads=kv_heads, head_dim=D, k_pages=k_pages,
                                v_pages=v_pages, block_table=step.block_tables[0], token_seq=step.token_seq,
                                positions=step.positions, out=out, page_size=page_size, scale=0.5, window=None,
                                step=step, value_dim=D, softcap=softcap, chunk=chunk)
            diff = float((out.float().cpu().reshape(hi - lo, heads, D) - want[lo:hi]).abs().max())
            tol = 3e-5 if dtype == "float32" else 4e-2
            assert diff <= tol, f"capped scores, query {qi}, key {kj}, tokens {lo}..{hi}: off by {diff:.3g}"


def case_latent_far_key_and_sink(dtype, ops, device, *, page_size=16, heads=4, rank=64, rot=16, T=330):
    """Attention over latent rows without a window: one row hundreds of tokens back takes nearly all the weight
    of the last query (and of one in the middle), unless the head's sink is larger still; a sink of a head that
    sees one row only halves (or nearly removes) that row's weight.  A whole prompt, a portion of two and a
    single decoded token over shuffled pages with NaN in unused rows."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(31)
    width = rank + rot
    pages_needed = -(-T // page_size)
    table = list(reversed(range(1, pages_needed + 1)))
    for qi, kj, sink_of_head0 in ((T - 1, 3, -30.0), (T - 1, T - 1 - 2 * page_size, 0.0), (T // 2, 0, 40.0)):
        rows = 0.3 * torch.randn((T, width), generator=gen)
        q = 0.3 * torch.randn((T, heads, width), generator=gen)
        rows[kj, rank - 2] += 7.0
        q[qi, :, rank - 2] += 7.0
        rows, q = rows.to(torch.bfloat16).float(), q.to(torch.bfloat16).float()
        sink = torch.tensor([sink_of_head0] + [0.5 * h for h in range(1, heads)])
        scores = torch.einsum("ihd,jd->hij", q.double(), rows.double()) * 0.5
        w = pl.softmax_rows(scores, pl.causal(T), sink=sink.double())
        want = torch.einsum("hij,jd->ihd", w, rows[:, :rank].double()).float()
        on_key = float((want[qi, 1] - rows[kj, :rank]).abs().max())
        assert on_key < 0.05, "the marked row does not stand out as intended"
        if sink_of_head0 > 30:  # a sink larger than the marked score leaves that head next to nothing
            assert float(want[qi, 0].abs().max()) < 0.05
        assert abs(float(w[1, 0, 0]) - 1 / (1 + math.exp(0.5 - float(scores[1, 0, 0])))) < 1e-9  # token 0: itself and the sink
        pages = torch.full((pages_needed + 2, page_size, width), float("nan"), dtype=dt, device=device)
        for j in range(T):
            pages[table[j // page_size], j % page_size] = rows[j].to(dt)
        for lo, hi in ((0, T), (qi - 1, qi + 1), (qi, qi + 1), (0, 1)):
            step = _step(list(range(lo, hi)), [0] * (hi - lo), [table], device)
            out = torch.zeros((hi - lo, heads, rank), dtype=dt, device=device)
            ops.latent_attention(q[lo:hi].to(device=device, dtype=dt).contiguous(), pages=pages, value_dim=rank,
                                 block_table=step.block_tables[0], token_seq=step.token_seq, positions=step.positions,
                                 sink=sink.to(device), out=out, page_size=page_size, scale=0.5, window=None, step=step)
            diff = float((out.float().cpu() - want[lo:hi]).abs().max())
            tol = 3e-5 if dtype == "float32" else 4e-2
            assert diff <= tol, f"latent rows, query {qi}, row {kj}, tokens {lo}..{hi}: off by {diff:.3g}"


def case_layer_norms(dtype, ops, device):
    """The norm kernel with its centering flags: a pending output layer-normed before it is added (dense rows
    and float32 partial-sum planes), the sum handed on as it is or layer-normed, on a subset of rows; widths
    with and without 16-byte rows."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(23)
    for W in (60, 64, 200):
        T = 9
        resid = torch.randn((T, W), generator=gen) * 3 + 1.5
        y = (torch.randn((T, W), generator=gen) * 2 - 0.7).to(dt).float()
        planes = torch.randn((3, T, W), generator=gen)
        w1, w2 = 1 + 0.2 * torch.randn(W, generator=gen), 1 + 0.2 * torch.randn(W, generator=gen)
        eps = 1e-5
        tol = 3e-5 if dtype == "float32" else 0.06
        for pending, y_sum in ((y.to(dt), y), (planes, planes.sum(0))):
            total = resid.double() + pl.layer_norm(y_sum.double(), w1.double(), eps)
            # the stream itself, rounded: what the next sublayer reads
            r = resid.clone().to(device)
            out = torch.empty((T, W), dtype=dt, device=device)
            ops.fused_norm(out, None, eps, resid=r, pending=pending.to(device), post_weight=w1.to(device), post_eps=eps,
                           post_center=True)
            assert float((r.cpu().double() - total).abs().max()) <= 3e-5
            assert float((out.float().cpu().double() - total).abs().max()) <= tol
            # the final norm on a few rows: the sum is left as it was
            r = resid.clone().to(device)
            rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=device)
            out = torch.empty((3, W), dtype=dt, device=device)
            ops.fused_norm(out, w2.to(device), eps, resid=r, pending=pending.to(device), rows=rows, write_resid=False,
                           num_rows=3, post_weight=w1.to(device), post_eps=eps, post_center=True, center=True)
            want = pl.layer_norm(total[[7, 0, 3]], w2.double(), eps)
            assert float((out.float().cpu().double() - want).abs().max()) <= tol
            assert torch.equal(r.cpu(), resid)
    # a row whose mean is far from zero and whose spread is small: the variance has to be that of the deviations
    x = (100.0 + 0.01 * torch.randn((2, 64), generator=gen))
    out = torch.empty((2, 64), dtype=torch.float32 if dtype == "float32" else dt, device=device)
    ops.fused_norm(out, torch.ones(64, device=device), 1e-5, resid=x.clone().to(device), center=True, write_resid=False)
    want = pl.layer_norm(x.double(), torch.ones(64, dtype=torch.float64), 1e-5)
    assert float((out.float().cpu().double() - want).abs().max()) <= (0.01 if dtype == "float32" else 0.1)


def case_rotations(dtype, ops, device):
    """The q/k kernel with heads made of two maps, with a rotation of a part of the head in either pairing and
    a magnitude, with values that are the keys as projected and with a value head count of its own; the latent
    row kernel and the heads' rotation with the halves pairing and a magnitude; positions in the hundreds."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(29)
    tol = 3e-5 if dtype == "float32" else 4e-2
    T, page_size = 11, 4
    positions = [0, 1, 2, 3, 250, 251, 252, 253, 254, 255, 256]
    table = list(reversed(range(1, 70)))
    step = _step(positions, [0] * T, [table], device)
    eps = 1e-5
    for H, G, D, rot, pairing, magnitude, maps, values_are_keys in (
            (4, 2, 24, 8, "interleaved", 1.0, 1, True), (4, 2, 24, 24, "half", 1.3, 1, False),
            (2, 1, 40, 0, "half", 1.0, 2, False), (3, 3, 16, 6, "half", 0.8, 1, True)):
        Dv = D if values_are_keys else 20
        cols = H * D + G * D + (0 if values_are_keys else G * Dv)
        proj = torch.randn((T, cols), generator=gen).to(dt)
        qw, kw = 1 + 0.2 * torch.randn(D // maps, generator=gen), 1 + 0.2 * torch.randn(D // maps, generator=gen)
        freqs = torch.tensor([0.7 ** i for i in range(rot // 2)], dtype=torch.float32) if rot else None
        x = proj.float()
        pos = torch.tensor(positions)
        q = pl.rms_norm(x[:, :H * D].reshape(T, H, maps, D // maps).double(), qw.double(), eps).reshape(T, H, D)
        k_raw = x[:, H * D:(H + G) * D].reshape(T, G, D)
        k = pl.rms_norm(k_raw.reshape(T, G, maps, D // maps).double(), kw.double(), eps).reshape(T, G, D)
        if rot:
            q = pl.rotate(q, pos, freqs.double(), pairing, magnitude)
            k = pl.rotate(k, pos, freqs.double(), pairing, magnitude)
        v = k_raw if values_are_keys else x[:, (H + G) * D:].reshape(T, G, Dv)
        k_pages = torch.full((70, G, page_size, D), float("nan"), dtype=dt, device=device)
        v_pages = torch.full((70, G, page_size, Dv), float("nan"), dtype=dt, device=device)
        pd = proj.clone().to(device)
        ops.qk_norm_store(pd, num_heads=H, num_kv_heads=G, head_dim=D, value_dim=Dv, k_start=H * D,
                          v_start=H * D if values_are_keys else (H + G) * D, q_weight=qw.to(device), k_weight=kw.to(device),
                          eps=eps, positions=step.positions, token_seq=step.token_seq, block_table=step.block_tables[0],
                          k_pages=k_pages, v_pages=v_pages, page_size=page_size, write_kv=True, maps=maps,
                          **(dict(inv_freq=freqs.to(device), pairing=pairing, magnitude=magnitude) if rot else {}))
        assert float((pd[:, :H * D].float().cpu().reshape(T, H, D) - q.float()).abs().max()) <= tol
        assert torch.equal(pd[:, H * D:].cpu(), proj[:, H * D:])  # keys and values as projected stay as they were
        for t, p in enumerate(positions):
            page = table[p // page_size]
            assert float((k_pages[page, :, p % page_size].float().cpu() - k[t].float()).abs().max()) <= tol
            assert torch.equal(v_pages[page, :, p % page_size].float().cpu(), v[t].to(dt).float())
    # the latent row: no query latent, halves pairing, a magnitude; a slice of wider rows
    C, R, H = 20, 12, 3
    freqs = torch.tensor([0.6 ** i for i in range(R // 2)], dtype=torch.float32)
    wide = torch.randn((T, 8 + C + R + 8), generator=gen).to(dt)
    cw = 1 + 0.2 * torch.randn(C, generator=gen)
    pages = torch.full((70, page_size, C + R), float("nan"), dtype=dt, device=device)
    wd = wide.to(device)
    ops.latent_norm_rope_store(wd[:, 8:8 + C + R], q_rank=0, kv_rank=C, rot_dim=R, q_weight=None, kv_weight=cw.to(device),
                               eps=eps, inv_freq=freqs.to(device), positions=step.positions, token_seq=step.token_seq,
                               block_table=step.block_tables[0], pages=pages, page_size=page_size, write=True, q_out=None,
                               pairing="half", magnitude=1.2)
    x = wide.float()[:, 8:8 + C + R].double()
    c = pl.rms_norm(x[:, :C], cw.double(), eps)
    kr = pl.rotate(x[:, None, C:], torch.tensor(positions), freqs.double(), "half", 1.2)[:, 0]
    for t, p in enumerate(positions):
        row = pages[table[p // page_size], p % page_size].float().cpu()
        assert float((row - torch.cat([c[t], kr[t]]).float()).abs().max()) <= tol
    xq = torch.randn((T, H, 8 + R), generator=gen).to(dt)
    out = torch.zeros((T, H, R + 4), dtype=dt, device=device)
    ops.rotate_heads(xq.to(device)[:, :, 8:], out[:, :, 4:], positions=step.positions, inv_freq=freqs[:4].to(device),
                     pairing="half", magnitude=1.2)
    want = pl.rotate(xq.float()[:, :, 8:].double(), torch.tensor(positions), freqs[:4].double(), "half", 1.2)
    assert float((out[:, :, 4:].float().cpu() - want.float()).abs().max()) <= tol
    assert float(out[:, :, :4].abs().max()) == 0


def case_frequencies():
    """The position part's frequencies against the plain statement's, in every band of both schedules."""
    ctx = BuildContext(torch.float32, torch.device("cpu"), None)
    for dims, base, scaling in ((24, 1e4, _wave(4.0, 1.0, 4.0, 64.0)), (64, 5e5, _wave(8.0, 1.0, 4.0, 8192.0)),
                                (8, 50.0, _wave(16.0, 1.0, 2.0, 24.0)), (16, 1e4, None)):
        spec = PartSpec("rotary_scaled", dict(rotary_dim=dims, theta=base, pairing="interleaved",
                                              scaling=dict(scaling, kind="wavelength") if scaling else None))
        part = build_part("position", spec, ctx)
        want = pl.scaled_frequencies_by_wavelength(dims, base, dict(scaling) if scaling else None, torch.float64)
        plainf = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
        assert torch.allclose(torch.tensor(part.host_frequencies(), dtype=torch.float64), want, rtol=1e-12)
        if scaling and dims > 8:
            ratio = want / plainf
            factor = dict(scaling)["factor"]
            assert float(ratio.max()) == 1.0 and abs(float(ratio.min()) - 1 / factor) < 1e-12  # both outer bands
            assert bool(((ratio > 1 / factor + 1e-9) & (ratio < 1 - 1e-9)).any())  # and the blend between them
        assert part.magnitude == 1.0
    for dims, base, scaling in ((12, 5e4, _ramp(6.0, 40.0, 8.0, 1.0)), (64, 1e4, _ramp(40.0, 4096.0, 32.0, 1.0)),
                                (16, 1e4, _ramp(2.0, 16.0, 4.0, 2.0)), (4, 100.0, _ramp(3.0, 8.0, 1.0, 1.0)),
                                (8, 1e4, None)):
        spec = PartSpec("rotary_scaled", dict(rotary_dim=dims, theta=base, pairing="half",
                                              scaling=dict(scaling, kind="ramp") if scaling else None))
        part = build_part("position", spec, ctx)
        want, magnitude = pl.ramped_frequencies(dims, base, dict(scaling) if scaling else None, torch.float64)
        assert torch.allclose(torch.tensor(part.host_frequencies(), dtype=torch.float64), want, rtol=1e-12)
        assert abs(part.magnitude - magnitude) < 1e-12 and (scaling is None or part.magnitude > 1.0)


def case_chunk_pages():
    """A chunk group gives back the pages that lie wholly before the chunk the next token falls in, and no
    page that a token of the current chunk may still read; pages come back when the request ends."""
    from qwen3_runtime_b200.cache.layout import CacheLayout, KVLayerSpec
    from qwen3_runtime_b200.cache.manager import FREED, CacheManager

    layout = CacheLayout({0: KVLayerSpec(2, 16, chunk=20), 1: KVLayerSpec(2, 16, chunk=20), 2: KVLayerSpec(2, 16),
                          3: KVLayerSpec(2, 16, chunk=7)})
    assert sorted((g.kind, g.chunk or 0) for g in layout.group_specs) == [("chunk", 7), ("chunk", 20), ("full", 0)]
    cm = CacheManager(layout.group_specs, 8, 16, 2)
    rc = cm.open("a")
    held = []
    for n in (19, 1, 1, 30, 9, 1):
        cm.reserve(rc, n)
        cm.commit(rc, n)
        cm.check_invariants()
        end = rc.num_computed
        for gi, table in zip(cm.paged_groups, rc.tables):
            g = cm.groups[gi]
            first = end // g.chunk * g.chunk if g.kind == "chunk" else 0
            for idx, page in enumerate(table):
                assert (page == FREED) == ((idx + 1) * 8 <= first), (g, end, idx)
        held.append(list(cm.num_free_pages))
    assert rc.num_computed == 61
    cm.close(rc)
    assert cm.num_free_pages == cm.num_pages
