"""Medilix: engine and parts against the plain statement (tests/plain_medilix.py), written once
and run on the CPU with the torch statements of the kernels and on the GPU with the kernels."""

from __future__ import annotations

import dataclasses
import json

import torch

import plain_medilix as pl
from helpers import (first_mismatch, max_abs_diff, peak_tokens, random_ids, run_trace, trace_mixed, trace_portions,
                     trace_tail_decode, trace_whole)
from puladra_cases import _random_tensors, _step, _tolerance, _views_for
from qwen3_runtime_b200.config import MedilixConfig, PartSpec
from qwen3_runtime_b200.config.medilix_config import (BigramConfig, DenseConfig, GatedAttentionConfig,
                                                      MedilixLayerConfig, MlstmConfig, MoeConfig, WkvConfig)
from qwen3_runtime_b200.engine.factory import build_engine, build_runtime, load_model
from qwen3_runtime_b200.parts import BuildContext, ResidualStream, build_part
from qwen3_runtime_b200.weights import write_random_model

TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _mlstm(**kw):
    base = dict(heads=3, dim=20, vdim=36, gate_cap=8.0)
    base.update(kw)
    return MlstmConfig(**base)


def _att(**kw):
    base = dict(heads=6, kv_heads=3, dim=24, vdim=40, scale=0.2, window=20, keep_first=3)
    base.update(kw)
    return GatedAttentionConfig(**base)


def _wkv(**kw):
    base = dict(heads=3, dim=24, decay_rank=6)
    base.update(kw)
    return WkvConfig(**base)


def _moe(**kw):
    base = dict(experts=6, identity=2, top=3, ff=24, groups=4, groups_keep=3)
    base.update(kw)
    return MoeConfig(**base)


L = MedilixLayerConfig

# Sizes no two of which are equal where the design lets them differ: key and value sizes, head counts, a
# head size that is no multiple of 8, norms in 3, 1, 2 and 4 groups, windows that are no multiple of the
# page, of one token, shorter than a page; none, 3, a page's worth and more than a page of kept first
# tokens; attention without a window; routing with and without groups, identity experts and none, top 1 and
# top everything, more identity experts than stored ones; a layer without a feed-forward; a loop of three
# passes in the middle, one from layer 0 over everything, one of a single pass over the last layer, none.
CONFIGS = {
    "A": dict(page_size=8, seed=41, config=MedilixConfig(
        vocab=150, width=72, norm_eps=1e-5, norm_groups=3, embed_scale=5.0, bigram=BigramConfig(97, 29, 13),
        loop_start=1, loop_stop=3, loop_times=3,
        layers=(L("mlstm", _mlstm(), DenseConfig(40, 1.5)),
                L("attention", _att(), _moe()),
                L("wkv", _wkv(), None),
                L("attention", _att(heads=2, kv_heads=1, dim=12, vdim=20, window=None, keep_first=0, scale=0.3),
                  _moe(experts=5, identity=0, top=1, ff=16, groups=1, groups_keep=1))))),
    "B": dict(page_size=4, seed=42, config=MedilixConfig(
        vocab=131, width=64, norm_eps=1e-6, norm_groups=1, embed_scale=1.0, bigram=BigramConfig(53, 1000003, 7919),
        layers=(L("wkv", _wkv(heads=2, dim=32, decay_rank=16), _moe(experts=4, identity=4, top=8, ff=24, groups=2,
                                                                    groups_keep=2)),
                L("attention", _att(heads=4, kv_heads=4, dim=16, vdim=8, window=1, keep_first=0), DenseConfig(56, 0.75)),
                L("mlstm", _mlstm(heads=1, dim=40, vdim=8, gate_cap=3.0), None),
                L("attention", _att(heads=4, kv_heads=1, dim=32, vdim=16, window=7, keep_first=9, scale=0.12), None)))),
    "C": dict(page_size=16, seed=43, config=MedilixConfig(
        vocab=90, width=48, norm_eps=1e-5, norm_groups=2, embed_scale=9.0, bigram=BigramConfig(31, 3, 5),
        loop_start=0, loop_stop=3, loop_times=2,
        layers=(L("attention", _att(heads=2, kv_heads=2, dim=16, vdim=24, window=33, keep_first=19), DenseConfig(32, 2.0)),
                L("wkv", _wkv(heads=2, dim=16, decay_rank=8), DenseConfig(24, 1.0)),
                L("mlstm", _mlstm(heads=2, dim=16, vdim=24, gate_cap=15.0), _moe(experts=2, identity=4, top=2, ff=16,
                                                                                 groups=6, groups_keep=2))))),
    # sizes the bfloat16 tensor-core paths take (multiples of 8 and 16 everywhere), keys and values of one size
    "D": dict(page_size=16, seed=44, config=MedilixConfig(
        vocab=210, width=128, norm_eps=1e-5, norm_groups=4, embed_scale=3.0, bigram=BigramConfig(509, 29, 19),
        loop_start=1, loop_stop=2, loop_times=1,
        layers=(L("mlstm", _mlstm(heads=2, dim=64, vdim=128, gate_cap=12.0), _moe(experts=8, identity=0, top=2, ff=64,
                                                                                  groups=4, groups_keep=2)),
                L("attention", _att(heads=8, kv_heads=2, dim=64, vdim=64, window=40, keep_first=16, scale=0.125),
                  DenseConfig(96, 1.0)),
                L("wkv", _wkv(heads=2, dim=64, decay_rank=16), _moe(experts=6, identity=2, top=3, ff=32, groups=2,
                                                                    groups_keep=1))))),
}

STD = 0.15  # spread of the random matrices: attention, states and experts have to matter
ROUTER_GAIN = 3.0  # routers are made decisive: a choice should not hang on a logit's last bit


def _every_expert(cfg: MedilixConfig) -> MedilixConfig:
    """The same model with every router output chosen for every token (no groups): whole models in bfloat16
    are tested in this form, since with many tokens some pair of choice scores always lies within bfloat16
    rounding and either choice is right.  The choice itself is tested in float32 on whole models and in
    bfloat16 on the feed-forward alone."""
    layers = tuple(dataclasses.replace(l, mlp=dataclasses.replace(l.mlp, top=l.mlp.experts + l.mlp.identity, groups=1,
                                                                  groups_keep=1))
                   if isinstance(l.mlp, MoeConfig) else l for l in cfg.layers)
    return dataclasses.replace(cfg, layers=layers)


for _name in ("A", "B", "C", "D"):
    CONFIGS[_name + "all"] = dict(CONFIGS[_name], config=_every_expert(CONFIGS[_name]["config"]))


def model_for(name, dtype):
    return name + "all" if dtype == "bfloat16" and not name.endswith("all") else name


def make_dir(tmp_path, name):
    spec = CONFIGS[name]
    folder = tmp_path / f"medilix_{name}"
    if not (folder / "model.safetensors").exists():
        from safetensors.torch import load_file, save_file

        write_random_model(spec["config"], folder, spec["seed"], std=STD, vector_std=0.1)
        t = load_file(str(folder / "model.safetensors"))
        for k in t:
            x = t[k].float()
            if k.endswith(".router"):
                x = x * ROUTER_GAIN
            elif k.endswith(".correction"):  # around zero, of the scores' own size, some of them negative
                x = (x - 1.0) * 1.5
            elif k.endswith(".mix.w0"):  # decays between about 0.5 and 0.99
                x = (x - 1.0) * 8.0 - 2.5
            elif k.endswith(".mix.f.b"):  # forget gates near one, so that the memory reaches far back
                x = x + 2.0
            elif ".mix.mu." in k:
                x = (x - 1.0) * 2.0 + 0.5
            elif k in ("embed", "bigram"):
                x = x * 4.0
            elif k == "loop.in":
                x = x * 3.0
            t[k] = x.to(t[k].dtype)
        save_file(t, str(folder / "model.safetensors"))
    return folder


def read_dir(folder):
    from safetensors.torch import load_file

    return json.loads((folder / "config.json").read_text()), load_file(str(folder / "model.safetensors"))


def expected(folder, requests, dtype):
    """Plain logits per request and the tolerance: float32 a few 1e-5 of the logits' size;
    bfloat16 three times the distance between the plain bfloat16 and the plain float32 logits."""
    raw, t = read_dir(folder)
    exact = {rid: pl.forward(raw, t, toks) for rid, toks in requests.items()}
    scale = max(float(v.abs().max()) for v in exact.values())
    if dtype == "float32":
        return exact, 5e-5 * max(1.0, scale)
    rounded = {rid: pl.forward(raw, t, toks, dtype=torch.bfloat16) for rid, toks in requests.items()}
    noise = max(float((rounded[r] - exact[r]).abs().max()) for r in exact)
    return rounded, 3.0 * noise


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
    """Whole prompts; the tail decoded token by token; portions down to two tokens; unequal requests
    side by side with pages and slots freed and used again (pages poisoned in between)."""
    name = model_for(name, dtype)
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
    """The stream after every layer run (a repeated layer counts each time) against the plain model's."""
    folder = make_dir(tmp_path, name)
    raw, t = read_dir(folder)
    toks = requests_for(name, (23,), seed=4)["r0"]
    want: list = []
    pl.forward(raw, t, toks, layers_out=want)
    rt = runtime(folder, name, "float32", ops, device, pages=-(-64 // CONFIGS[name]["page_size"]))
    got: list = []

    def watched(forward):
        def run(stream, step, cache):
            forward(stream, step, cache)
            v = stream.resid.clone()
            for extra in (stream.pending, stream.pending_more):  # what a block left for the next norm to add
                if extra is not None:
                    v = v + (extra.float() if extra.dim() == 2 else extra.sum(0))
            got.append(v.cpu())
        return run

    for block in rt.runner.model.blocks:
        block.forward = watched(block.forward)
    run_trace(rt, trace_whole({"r0": toks}))
    assert len(got) == len(want) == len(CONFIGS[name]["config"].run_order())
    for run, (g, w) in enumerate(zip(got, want)):
        diff = float((g - w).abs().max())
        assert diff <= 3e-5 * max(1.0, float(w.abs().max())), f"{name}: stream after run {run} off by {diff:.3g}"


def case_long_decode(tmp_path, name, dtype, ops, device, total=150, cuda_graph=False):
    """A short prompt and then one token at a time, far beyond every window and over many pages."""
    name = model_for(name, dtype)
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
    """One-, two- and three-token sequences side by side, then sequences fed one token at a time from
    their first in the slots the others left: the bigram's last row, the shifted input's zeros, states
    and running maxima from zero, windows not yet full."""
    name = model_for(name, dtype)
    folder = make_dir(tmp_path, name)
    requests = requests_for(name, (1, 2, 3, 1), seed=9)
    want, tol = expected(folder, requests, dtype)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in requests.items()],
              "end": list(requests)}]
    rt = runtime(folder, name, dtype, ops, device, pages=32)
    check(run_trace(rt, steps), want, tol, f"{name} {dtype} first tokens")
    again = requests_for(name, (6, 5), seed=10)
    want, tol = expected(folder, again, dtype)
    steps = [{"step": i, "entries": [{"id": r, "tokens": [t[i]], "want": [0]} for r, t in again.items() if i < len(t)],
              "end": [r for r, t in again.items() if i == len(t) - 1]} for i in range(6)]
    check(run_trace(rt, steps), want, tol, f"{name} {dtype} first tokens one by one in used slots")


def case_greedy_generation(tmp_path, name, dtype, ops, device, cuda_graph=False, steps=12):
    """Greedy generation through the engine's own entry point, scheduler and sampler: unequal prompts side
    by side in a small pool, every token checked at its own place against the plain model given the
    tokens before it."""
    name = model_for(name, dtype)
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
        exact = pl.forward(raw, t, seq)[len(prompt) - 1:]
        if dtype == "float32":
            rows, tol = exact, 1e-4 * max(1.0, float(exact.abs().max()))
        else:
            rows = pl.forward(raw, t, seq, dtype=torch.bfloat16)[len(prompt) - 1:]
            tol = 2 * 3.0 * float((rows - exact).abs().max())
        for i, tok in enumerate(out):
            gap = float(rows[i].max() - rows[i][tok])
            assert gap <= tol, f"token {i} ({tok}) is {gap:.3g} below the plain argmax (allowed {tol:.3g})"
    engine.runtime.cache.check_invariants()
    assert engine.runtime.cache.num_free_pages == engine.runtime.cache.num_pages


# ---- parts and kernels alone ---------------------------------------------------------------------

def _mixer_part(kind, width, eps, sizes, ctx):
    """The part of one mixer kind with its plain statement ``plain(h, tensors)``."""
    dt = ctx.dtype
    if kind == "mlstm":
        m = dict(heads=3, dim=20, vdim=36, gate_cap=8.0)
        m.update(sizes)
        spec = PartSpec("mlstm", dict(hidden_size=width, num_heads=m["heads"], dim=m["dim"], vdim=m["vdim"],
                                      gate_cap=m["gate_cap"], eps=eps))
        return build_part("mixer", spec, ctx), lambda h, t: pl.mlstm_mixer(h, m, t, "mix.", eps, dt)
    if kind == "wkv":
        m = dict(heads=3, dim=24, rank=6)
        m.update(sizes)
        spec = PartSpec("wkv", dict(hidden_size=width, num_heads=m["heads"], dim=m["dim"], decay_rank=m["rank"], eps=eps))
        return build_part("mixer", spec, ctx), lambda h, t: pl.wkv_mixer(h, m, t, "mix.", eps, dt)
    m = dict(heads=6, kv_heads=3, dim=24, vdim=40, scale=0.2, mask=dict(size=20, keep_first=3))
    m.update(sizes)
    mask = m.get("mask") or {}
    spec = PartSpec("sink_window_attention", dict(
        hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"],
        scale=m["scale"], window=mask.get("size"), keep_first=mask.get("keep_first", 0), sink=0.0, gate="sigmoid",
        qk_norm_eps=eps))
    return build_part("mixer", spec, ctx), lambda h, t: pl.attention_mixer(h, m, t, "mix.", eps, dt)


def case_mixer_alone(dtype, ops, device, kind, *, T=45, page_size=8, cuts=(24, 1, 2, 18), **sizes):
    """A mixer on one sequence in portions (one of a single token, one of two) through a paged cache whose
    pages are out of order and state slots that are not the first, against the plain statement on the
    whole sequence."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(5)
    width, eps = 64, 1e-5
    part, plain = _mixer_part(kind, width, eps, sizes, BuildContext(dt, torch.device(device), ops))
    tensors = _random_tensors(part, gen, dt, device)
    if kind == "wkv":  # decays of 0.4 to 0.99 and blends between the two tokens
        tensors["w0"] = (tensors["w0"] - 1.0) * 6.0 - 2.0
        for s in part.BLENDS:
            tensors[f"mu.{s}"] = (tensors[f"mu.{s}"] - 1.0) + 0.5
    part.load(tensors)
    h = torch.randn((T, width), generator=gen).to(torch.bfloat16).float()
    want = plain(h, {"mix." + k: v.float().cpu() for k, v in tensors.items()}).float()
    pages_needed = -(-T // page_size)
    table = list(reversed(range(1, pages_needed + 1)))  # not in order, page 0 unused
    cache = _views_for(part.cache_spec(), device, dt, page_size, pages_needed + 2, slots=3)
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


def case_attention_edges(dtype, ops, device, *, window=12, keep=3, page_size=8, heads=4, kv_heads=2, D=24, Dv=40, T=50,
                         dense_out=False, decode_slices=None):
    """The attention kernel alone with one key that takes nearly all the weight when it is seen: at distance
    window - 1 it decides the output, at distance window it does not, unless it is one of the kept first
    tokens (the last kept one is seen from everywhere, the one after it is not); for queries inside a prompt
    portion and as a single decoded token; keys at a page's last row, first row and inside one.  Where the
    few keys are seen (the sequence's first tokens, a window of one) the sink takes a large share: the plain
    output is far from a plain softmax's.  With a gate.  Pages are out of order and unused rows hold NaN.
    ``dense_out``: the output rows are not a slice of wider ones (what the kernels for keys and values of one
    size want); ``decode_slices``: the single token's keys are cut into that many slices."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(17)
    pages_needed = -(-T // page_size)
    table = list(reversed(range(1, pages_needed + 1)))
    cases = [(window, keep, qi, qi - dist) for qi in (window + 19, window + 20, window + 24, T - 1)
             for dist in (window - 1, window)]
    cases += [(window, keep, T - 1, keep - 1), (window, keep, T - 1, keep), (window, keep, window + keep + 2, 0),
              (window, 0, T - 1, 0), (window, page_size + 2, T - 1, page_size + 1), (window, page_size + 2, T - 1, page_size + 2),
              (None, 0, T - 1, 1), (None, 0, 20, 0), (1, 0, T - 1, T - 2), (1, 2, T - 1, 1)]
    for win, kp, qi, kj in cases:
        k = 0.3 * torch.randn((T, kv_heads, D), generator=gen)
        v = torch.randn((T, kv_heads, Dv), generator=gen)
        q = 0.3 * torch.randn((T, heads, D), generator=gen)
        g = torch.randn((T, heads * Dv), generator=gen)
        k[kj, :, D - 3] += 8.0
        q[qi, :, D - 3] += 8.0
        q, k, v, g = (x.to(torch.bfloat16).float() for x in (q, k, v, g))
        want = pl.sink_window_attention(q, k, v, 1.0, win, kp)
        seen = win is None or qi - kj < win or kj < kp
        on_key = float((want[qi, 0] - v[kj, 0]).abs().max())
        assert (on_key < 0.05) == seen, "the marked key does not stand out as intended"
        # the sink shows most where few keys are seen: token 0 sees itself only, and without the sink its weight would be 1
        plain_softmax = pl.sink_window_attention(q, k, v, 1.0, win, kp, sink=False)
        assert float((plain_softmax[0] - want[0]).abs().max()) > 0.05
        want = want * torch.sigmoid(g).reshape(T, heads, Dv)
        k_pages = torch.full((pages_needed + 2, kv_heads, page_size, D), float("nan"), dtype=dt, device=device)
        v_pages = torch.full((pages_needed + 2, kv_heads, page_size, Dv), float("nan"), dtype=dt, device=device)
        for j in range(T):
            k_pages[table[j // page_size], :, j % page_size] = k[j].to(dt)
            v_pages[table[j // page_size], :, j % page_size] = v[j].to(dt)
        for lo, hi in ((0, T), (qi - 1, qi + 1), (qi, qi + 1)):  # a whole prompt; a portion of two; one decoded token
            step = _step(list(range(lo, hi)), [0] * (hi - lo), [table], device)
            pad = 0 if dense_out else 8
            wide = torch.zeros((hi - lo, heads * Dv + 2 * pad), dtype=dt, device=device)
            qd = q[lo:hi].reshape(hi - lo, heads * D).to(device=device, dtype=dt).contiguous()
            ops.paged_attention(qd, qd.stride(0), num_heads=heads, num_kv_heads=kv_heads, head_dim=D, k_pages=k_pages,
                                v_pages=v_pages, block_table=step.block_tables[0], token_seq=step.token_seq,
                                positions=step.positions, out=wide[:, pad:pad + heads * Dv], page_size=page_size, scale=1.0,
                                window=win, step=step, value_dim=Dv, keep_first=kp, sink=0.0,
                                gate=g[lo:hi].to(device=device, dtype=dt),
                                **({"decode_slices": decode_slices} if decode_slices and hi - lo == 1 else {}))
            out = wide[:, pad:pad + heads * Dv].float().cpu().reshape(hi - lo, heads, Dv)
            diff = float((out - want[lo:hi]).abs().max())
            tol = 2e-5 if dtype == "float32" else 3e-2
            assert diff <= tol, f"window {win} keep {kp}, query {qi}, key {kj}, tokens {lo}..{hi}: off by {diff:.3g}"
            assert dense_out or (float(wide[:, :8].abs().max()) == 0 and float(wide[:, 8 + heads * Dv:].abs().max()) == 0)


def _portion_steps(portion_sets, device, slots):
    """Steps of several sequences side by side, ``portion_sets`` = per step the token count of each:
    yields ``(step, rows)`` with ``rows`` the (sequence, position) of every token of the step."""
    at = [0] * len(slots)
    for portions in portion_sets:
        rows, seqs, positions = [], [], []
        for b, n in enumerate(portions):
            rows += [(b, at[b] + i) for i in range(n)]
            seqs += [b] * n
            positions += list(range(at[b], at[b] + n))
        live = [b for b, n in enumerate(portions) if n]
        renum = {b: i for i, b in enumerate(live)}
        yield _step(positions, [renum[s] for s in seqs], [[0]] * len(live), device, slots=[slots[b] for b in live]), rows
        for b, n in enumerate(portions):
            at[b] += n


PORTION_SETS = ((9, 1), (1, 30), (2, 7), (0, 2), (58, 30))  # unequal portions side by side, one sequence left out once


def case_stabilised_memory(dtype, ops, device, *, H=3, D=20, Dv=36, cap=6.0):
    """The gates' kernel, the state kernel (per-token decays and key scales, a column of ones) and the division
    by the normaliser in the heads' norm, on two sequences in portions with their states in slots that others
    used before, against the plain recurrence.  Gate logits are large: input gates reach the cap on both
    sides, so that the running maximum moves, exp(-m) takes the denominator at the start (m starts at 0)
    and |n . q| later."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(11)
    B, T = 2, sum(p[0] for p in PORTION_SETS)
    rnd = lambda *shape: (0.5 * torch.randn(shape, generator=gen)).to(torch.bfloat16).float()  # noqa: E731
    q, k, v, g = rnd(B, T, H, D), rnd(B, T, H, D), rnd(B, T, H, Dv), rnd(B, T, H, Dv)
    zi, zf = 8.0 * rnd(B, T, H), 4.0 * rnd(B, T, H)
    bi, bf = rnd(H), rnd(H) + 2.0
    weight = 1.0 + rnd(H * Dv)
    eps = 1e-5
    want = []
    used_m, used_nq = 0, 0
    for b in range(B):
        li = cap * torch.tanh((zi[b] + bi) / cap)
        lf = torch.nn.functional.logsigmoid(cap * torch.tanh((zf[b] + bf) / cap))
        o = pl.stabilised_memory(q[b] * D ** -0.5, k[b], v[b], li, lf)
        trace = pl.stabilised_memory(q[b] * D ** -0.5, k[b], torch.ones(T, H, 1), li, lf)  # n . q / den
        used_nq += int((trace.abs() > 0.99).sum())
        used_m += int((trace.abs() < 0.9).sum())
        want.append(pl.head_unit_norm(o, eps) * weight.reshape(H, Dv) * torch.sigmoid(g[b]))
    assert used_m > 10 and used_nq > 10, "one of the denominator's two branches is hardly taken"
    slots = [3, 1]
    memory = torch.full((4, H, D, Dv + 1), float("nan"), dtype=torch.float32, device=device)
    m_state = torch.full((4, H), float("nan"), dtype=torch.float32, device=device)
    memory[slots] = 0.0
    m_state[slots] = 0.0
    got = [dict(), dict()]
    for step, rows in _portion_steps(PORTION_SETS, device, slots):
        pick = lambda x, t=dt: torch.stack([x[b, p] for b, p in rows]).to(device=device, dtype=t)  # noqa: E731
        kw = dict(cu_seqlens=step.cu_seqlens, state_slots=step.state_slots, num_seqs=step.num_seqs)
        decay, k_scale, m_run = ops.stabilised_gates(pick(zi), pick(zf), i_bias=bi.to(device), f_bias=bf.to(device),
                                                     cap=cap, m_state=m_state, **kw)
        o = ops.decayed_state_scan(pick(q), pick(k), pick(v), state=memory, token_decay=decay, token_k_scale=k_scale,
                                   ones_column=True, q_scale=D ** -0.5, **kw)
        out = torch.empty((len(rows), H, Dv), dtype=dt, device=device)
        ops.head_norm_gate(o, pick(g), out, weight=weight.to(device), eps=eps, gate_act="sigmoid", per_head_weight=True,
                           denominator=m_run)
        for i, (b, p) in enumerate(rows):
            got[b][p] = out[i].float().cpu()
    for b in range(B):
        n = len(got[b])
        diff = float((torch.stack([got[b][p] for p in range(n)]) - want[b][:n]).abs().max())
        tol = (5e-5 if dtype == "float32" else 3e-2) * max(1.0, float(want[b].abs().max()))
        assert diff <= tol, f"stabilised memory ({dtype}) sequence {b}: off by {diff:.3g}"
    assert torch.isnan(memory[0]).all() and torch.isnan(m_state[2]).all(), "a slot of another request was touched"


def case_bonus_memory(dtype, ops, device, *, H=3, D=20, Dv=36):
    """The state kernel with a decay exp(-exp(z + bias)) per token and key channel and a bonus for the present
    token, read before the update; two sequences in portions, slots used before."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(12)
    B, T = 2, sum(p[0] for p in PORTION_SETS)
    rnd = lambda *shape: (0.5 * torch.randn(shape, generator=gen)).to(torch.bfloat16).float()  # noqa: E731
    r, k, v = rnd(B, T, H, D), rnd(B, T, H, D), rnd(B, T, H, Dv)
    z = (2.0 * rnd(B, T, H, D) - 2.0).to(torch.bfloat16).float()
    bias, u = rnd(H * D), 1.0 + rnd(H, D)
    want = [pl.bonus_memory(r[b], k[b], v[b], torch.exp(-torch.exp(z[b] + bias.reshape(H, D))), u) for b in range(B)]
    assert float((want[0] - pl.bonus_memory(r[0], k[0], v[0], torch.exp(-torch.exp(z[0] + bias.reshape(H, D))),
                                            torch.ones(H, D))).abs().max()) > 0.1, "the bonus does not show"
    slots = [2, 0]
    state = torch.full((4, H, D, Dv), float("nan"), dtype=torch.float32, device=device)
    state[slots] = 0.0
    got = [dict(), dict()]
    for step, rows in _portion_steps(PORTION_SETS, device, slots):
        pick = lambda x: torch.stack([x[b, p] for b, p in rows]).to(device=device, dtype=dt)  # noqa: E731
        o = ops.decayed_state_scan(pick(r), pick(k), pick(v), state=state, cu_seqlens=step.cu_seqlens,
                                   state_slots=step.state_slots, num_seqs=step.num_seqs, decay_logits=pick(z),
                                   decay_bias=bias.to(device), decay_mode="exp_neg_exp", bonus=u.reshape(-1).to(device))
        for i, (b, p) in enumerate(rows):
            got[b][p] = o[i].float().cpu()
    for b in range(B):
        n = len(got[b])
        diff = float((torch.stack([got[b][p] for p in range(n)]) - want[b][:n]).abs().max())
        assert diff <= 3e-5 * max(1.0, float(want[b].abs().max())), f"bonus memory ({dtype}) sequence {b}: off by {diff:.3g}"
    assert torch.isnan(state[1]).all() and torch.isnan(state[3]).all(), "a slot of another request was touched"


def case_memories_remember_a_far_token(dtype, ops, device, *, T=400, H=2, D=16, Dv=8):
    """One key far back, in an earlier portion, that the last query asks for.  With forget gates (decays) near
    one its value comes through the state: a state that was lost, reset or mixed up between portions shows."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(2)
    q, k = 0.05 * torch.randn((T, H, D), generator=gen), 0.05 * torch.randn((T, H, D), generator=gen)
    v = 0.05 * torch.randn((T, H, Dv), generator=gen)
    far = 7
    k[far, :, 3] += 4.0
    q[T - 1, :, 3] += 4.0
    v[far] = torch.arange(1, Dv + 1).float()[None, :].expand(H, Dv)
    q, k, v = (x.to(torch.bfloat16).float() for x in (q, k, v))
    cuts = (100, 1, 150, 2, T - 253 - 1, 1)
    # the bonus form: decays 0.999 per token
    z = torch.full((T, H, D), -6.9).to(torch.bfloat16).float()
    want = pl.bonus_memory(q, k, v, torch.exp(-torch.exp(z)), torch.ones(H, D))
    assert float(want[T - 1, 0].abs().max()) > 50 * float(want[T - 2, 0].abs().max()), "the far token does not stand out"
    state = torch.zeros((2, H, D, Dv), dtype=torch.float32, device=device)
    outs, lo = [], 0
    for n in cuts:
        step = _step(list(range(lo, lo + n)), [0] * n, [[0]], device, slots=[1])
        cut = lambda x: x[lo:lo + n].to(device=device, dtype=dt)  # noqa: E731
        outs.append(ops.decayed_state_scan(cut(q), cut(k), cut(v), state=state, cu_seqlens=step.cu_seqlens,
                                           state_slots=step.state_slots, num_seqs=1, decay_logits=cut(z),
                                           decay_mode="exp_neg_exp", bonus=torch.ones(H * D, device=device)).cpu())
        lo += n
    diff = float((torch.cat(outs) - want).abs().max())
    assert diff <= 3e-5 * float(want.abs().max()), f"far token through the bonus state ({dtype}): off by {diff:.3g}"
    # the stabilised form: forget gates near one, the far token's input gate at the cap, the others' far below
    cap = 10.0
    zi = torch.full((T, H), -4.0)
    zi[far] = 30.0
    zf = torch.full((T, H), 7.0)
    li, lf = cap * torch.tanh(zi / cap), torch.nn.functional.logsigmoid(cap * torch.tanh(zf / cap))
    want = pl.stabilised_memory(q, k, v, li, lf)
    # the normaliser is the far key's too: the last token reads the far value itself, whatever decayed since
    assert float((want[T - 1, 0] - v[far, 0]).abs().max()) < 0.1, "the far token does not stand out"
    memory = torch.zeros((2, H, D, Dv + 1), dtype=torch.float32, device=device)
    m_state = torch.zeros((2, H), dtype=torch.float32, device=device)
    outs, lo = [], 0
    zero = torch.zeros(H, device=device)
    for n in cuts:
        step = _step(list(range(lo, lo + n)), [0] * n, [[0]], device, slots=[1])
        cut = lambda x, t=dt: x[lo:lo + n].to(device=device, dtype=t)  # noqa: E731
        kw = dict(cu_seqlens=step.cu_seqlens, state_slots=step.state_slots, num_seqs=1)
        decay, k_scale, m_run = ops.stabilised_gates(cut(zi), cut(zf), i_bias=zero, f_bias=zero, cap=cap,
                                                     m_state=m_state, **kw)
        o = ops.decayed_state_scan(cut(q), cut(k), cut(v), state=memory, token_decay=decay, token_k_scale=k_scale,
                                   ones_column=True, **kw).float().cpu()
        den = torch.maximum(o[:, :, Dv].abs(), torch.exp(-m_run.float().cpu())) + 1e-6
        outs.append(o[:, :, :Dv] / den[:, :, None])
        lo += n
    diff = float((torch.cat(outs) - want).abs().max())
    assert diff <= 5e-5 * float(want.abs().max()), f"far token through the stabilised state ({dtype}): off by {diff:.3g}"


def case_token_state(dtype, ops, device, *, W=40, vocab=50, buckets=23, mul_prev=1000003, mul_cur=7919):
    """The bigram embedding and the token shift alone: two sequences in portions (of one and of two tokens,
    one sequence left out of a step), previous token and previous row in slots that held other requests'
    before; a sequence's first token takes the table's last row and a zero previous row.  The products of
    the hash exceed 32 bits."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(21)
    B, T = 2, sum(p[0] for p in PORTION_SETS)
    toks = torch.randint(0, vocab, (B, T), generator=gen)
    embed = torch.randn((vocab, W), generator=gen).to(torch.bfloat16)
    bigram = torch.randn((buckets + 1, W), generator=gen).to(torch.bfloat16)
    cfg = dict(embedding=dict(scale=3.0, bigram=dict(buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur)))
    want_x = [pl.embedding(cfg, dict(embed=embed, bigram=bigram), toks[b].tolist()) for b in range(B)]
    h = torch.randn((B, T, W), generator=gen).to(torch.bfloat16).float()
    mu = torch.rand((5, W), generator=gen)
    want_mix = []
    for b in range(B):
        prev = torch.cat([torch.zeros(1, W), h[b, :-1]])
        want_mix.append(h[b][None] + (prev - h[b])[None] * mu[:, None, :])
    slots = [3, 1]
    prev_tok = torch.full((4, 1), 12345, dtype=torch.int32, device=device)
    prev_row = torch.full((4, W), float("nan"), dtype=torch.float32, device=device)
    prev_row[slots] = 7.0  # what an earlier request left: a first token must not read it
    for step, rows in _portion_steps(PORTION_SETS, device, slots):
        n = len(rows)
        ids = torch.tensor([int(toks[b, p]) for b, p in rows], dtype=torch.int32, device=device)
        out = torch.empty((n, W), dtype=torch.float32, device=device)
        copy = torch.zeros((n, 2 * W), dtype=dt, device=device)
        kw = dict(positions=step.positions, token_seq=step.token_seq, cu_seqlens=step.cu_seqlens,
                  state_slots=step.state_slots, num_seqs=step.num_seqs)
        ops.bigram_embed(ids, embed=embed.to(device=device, dtype=dt), scale=3.0, bigram=bigram.to(device=device, dtype=dt),
                         buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur, prev_state=prev_tok, out=out,
                         copy=copy[:, W:], **kw)
        x = ops.token_shift_mix(torch.stack([h[b, p] for b, p in rows]).to(device=device, dtype=dt), mu.to(device),
                                state=prev_row, **kw)
        for i, (b, p) in enumerate(rows):
            assert float((out[i].cpu() - want_x[b][p]).abs().max()) <= 1e-5, f"embedding of sequence {b} token {p}"
            assert float((copy[i, W:].float().cpu() - want_x[b][p]).abs().max()) <= (1e-5 if dtype == "float32" else 0.1)
            diff = float((x[:, i].float().cpu() - want_mix[b][:, p]).abs().max())
            assert diff <= (1e-5 if dtype == "float32" else 0.05), f"shifted input of sequence {b} token {p}: {diff:.3g}"
        assert float(copy[:, :W].abs().max()) == 0
    assert int(prev_tok[0, 0]) == 12345 and torch.isnan(prev_row[2]).all(), "a slot of another request was touched"


def case_grouped_norm(dtype, ops, device, W=60):
    """Norms in 1, 2, 3 and 5 groups, one and two weights on the same rows, with a pending sum added first."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(6)
    T, eps = 9, 1e-5
    for groups in (1, 2, 3, 5):
        resid = torch.randn((T, W), generator=gen) * torch.linspace(0.1, 9.0, W)  # parts of unlike size
        pending = torch.randn((2, T, W), generator=gen)
        w1, w2 = torch.randn(W, generator=gen), torch.randn(W, generator=gen)
        x = resid + pending.sum(0)
        r = resid.clone().to(device)
        out, out2 = (torch.empty((T, W), dtype=dt, device=device) for _ in range(2))
        ops.grouped_norm(out, w1.to(device), eps, groups, resid=r, pending=pending.to(device), out2=out2, weight2=w2.to(device))
        tol = 1e-5 if dtype == "float32" else 3e-2
        assert float((r.cpu() - x).abs().max()) <= 1e-5 * float(x.abs().max())
        for got, w in ((out, w1), (out2, w2)):
            want = pl.grouped_rms_norm(x, w, groups, eps)
            assert float((got.float().cpu() - want).abs().max()) <= tol * float(want.abs().max()), f"{groups} groups"
        if groups > 1:
            assert float((pl.grouped_rms_norm(x, w1, groups, eps) - pl.grouped_rms_norm(x, w1, 1, eps)).abs().max()) > 0.1


def case_routing(dtype, ops, device):
    """The choice alone on made-up scores.  A correction lifts an expert with a small score into the choice
    while its weight stays the small score; a group that is not kept loses an expert whose choice score would
    have been among the best; corrections make every choice score negative and the best groups are still
    those nearest to zero (a dropped group counts as minus infinity, not 0); groups of one; no groups."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(4)
    T, W = 33, 40
    h = torch.randn((T, W), generator=gen).to(dt).float()
    for E, ident, top, groups, shift in ((8, 0, 2, (4, 2), 0.0), (6, 2, 3, (4, 3), -5.0), (9, 0, 4, None, 0.0),
                                         (4, 4, 8, (2, 2), 0.0), (6, 6, 3, (12, 4), -1.0), (5, 0, 1, (1, 1), 0.5)):
        n_all = E + ident
        router = (0.4 * torch.randn((n_all, W), generator=gen))
        correction = 0.3 * torch.randn(n_all, generator=gen) + shift
        p = dict(router=dict(experts=E, identity=ident, top=top,
                             groups=dict(count=groups[0], keep=groups[1]) if groups else None))
        want_c, want_w = pl.route(h, p, {"router": router, "correction": correction}, "")
        chosen, weights = ops.route_top(h.to(device=device, dtype=dt), router.to(device), top, renormalize=True,
                                        score="softmax_all", correction=correction.to(device), groups=groups)
        order = chosen.long().cpu().argsort(-1)
        want_order = want_c.argsort(-1)
        assert torch.equal(chosen.long().cpu().gather(1, order), want_c.gather(1, want_order)), f"choice {E}+{ident} {groups}"
        assert float((weights.cpu().gather(1, order) - want_w.gather(1, want_order)).abs().max()) < 1e-5
        assert float((weights.sum(-1).cpu() - 1).abs().max()) < 1e-5
    # one token by hand: 8 router outputs in 4 groups of which 2 are kept, top 2
    eye = torch.zeros((8, W))
    z = torch.tensor([2.0, 0.0, 0.1, 1.9, 1.0, 1.1, -1.0, 0.5])
    one = torch.zeros((1, W))
    one[0, :8] = 1.0
    for e in range(8):
        eye[e, e] = z[e]
    corr = torch.tensor([0.0, 0.0, 0.0, -0.5, 0.0, 0.0, 0.9, 0.0])
    s = torch.softmax(z, -1)
    # choice scores: group 0 (s0, s1), group 1 (s2, s3 - .5), group 2 (s4, s5), group 3 (s6 + .9, s7): groups 3 and 0 are kept
    chosen, weights = ops.route_top(one.to(device=device, dtype=dt), eye.to(device), 2, renormalize=True, score="softmax_all",
                                    correction=corr.to(device), groups=(4, 2))
    assert sorted(chosen[0].tolist()) == [0, 6]
    got = dict(zip(chosen[0].tolist(), weights[0].tolist()))
    assert abs(got[6] - float(s[6] / (s[0] + s[6]))) < 1e-5, "the weight is the score without the correction"


def case_feed_forwards_alone(dtype, ops, device, *, experts=6, identity=2, top=3, groups=(4, 3), T=37):
    """The routed experts part (stored and identity experts) and the clamped dense layer against their plain
    statements.  The dense layer's inputs are large enough for all three clamps to bind."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(8)
    width, ff = 48, 40
    ctx = BuildContext(dt, torch.device(device), ops)
    spec = PartSpec("routed_experts", dict(
        hidden_size=width, num_experts=experts, num_identity=identity, top=top, expert_size=ff, activation="silu_glu",
        score="softmax_all", correction=True, renormalize=True, weight_on="output", groups=groups))
    part = build_part("feed_forward", spec, ctx)
    tensors = _random_tensors(part, gen, dt, device, std=0.4)
    tensors["correction"] = (tensors["correction"] - 1.0) * 0.5
    part.load(tensors)
    h = torch.randn((T, width), generator=gen).to(torch.bfloat16).float()
    p = dict(router=dict(experts=experts, identity=identity, top=top,
                         groups=dict(count=groups[0], keep=groups[1]) if groups else None), expert=dict(ff=ff))
    cpu = {"mlp." + k: v.float().cpu() for k, v in tensors.items()}
    want = pl.expert_feed_forward(h, p, cpu, "mlp.", dt).float()
    if identity:
        chosen, _ = pl.route(h, p, cpu, "mlp.")
        assert int((chosen >= experts).sum()) > T // 4, "identity experts are hardly chosen"
    got = part.forward(h.to(device=device, dtype=dt), None).float().cpu()
    tol = _tolerance(dtype, want)
    diff = float((got - want).abs().max())
    assert diff <= tol, f"routed experts ({dtype}, {top} of {experts}+{identity}): off by {diff:.3g} (allowed {tol:.3g})"
    limit = 0.75
    dense = build_part("feed_forward", PartSpec("clamped_mlp", dict(hidden_size=width, intermediate_size=ff, limit=limit,
                                                                    alpha=1.702, up_offset=1.0)), ctx)
    tensors = _random_tensors(dense, gen, dt, device, std=0.3)
    dense.load(tensors)
    cpu = {"mlp." + k: v.float().cpu() for k, v in tensors.items()}
    gate, up = pl.lin(h, cpu["mlp.gate"], dt), pl.lin(h, cpu["mlp.up"], dt)
    assert (gate > limit).any() and (gate < -limit).any() and (up > limit).any() and (up < -limit).any()
    want = pl.dense_feed_forward(h, dict(limit=limit), cpu, "mlp.", dt).float()
    got = dense.forward(h.to(device=device, dtype=dt), None).float().cpu()
    diff = float((got - want).abs().max())
    assert diff <= _tolerance(dtype, want), f"clamped dense layer ({dtype}): off by {diff:.3g}"
