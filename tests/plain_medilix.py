"""Medilix stated plainly: whole sequences, no cache, recurrences as loops over tokens, one function
per mechanism.  Shares no code with the package; the tests compare the engine with it.

``cfg`` is the design's config.json as a dict, ``w`` maps tensor names to tensors.  ``dtype`` is the
type of the matrix products' operands and results (float32: everything exact; bfloat16: products and
their activations rounded, everything the design wants in 32-bit kept there).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def lin(x: torch.Tensor, weight: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """y = W x for every row of x, operands and result in ``dtype``, accumulated in float32; returned as float32."""
    y = x.to(dtype).float() @ weight.to(dtype).float().t()
    return y.to(dtype).float()


def grouped_rms_norm(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """Every one of ``groups`` equal consecutive parts of a row divided by its own root mean square."""
    T, W = x.shape
    parts = x.float().reshape(T, groups, W // groups)
    parts = parts * torch.rsqrt(parts.pow(2).mean(-1, keepdim=True) + eps)
    return parts.reshape(T, W) * weight.float()


def head_unit_norm(o: torch.Tensor, eps: float) -> torch.Tensor:
    """``o`` [T, H, n]: every head divided by its root mean square."""
    return o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)


def embedding(cfg: dict, w: dict, tokens: list[int]) -> torch.Tensor:
    """Scaled token rows plus a row chosen by the hash of (previous token, token); the last row for a first token."""
    e = cfg["embedding"]
    ids = torch.tensor(tokens, dtype=torch.long)
    x = w["embed"].float()[ids] * float(e["scale"])
    big = e.get("bigram")
    if big:
        rows = []
        for t, tok in enumerate(tokens):
            if t == 0:
                rows.append(int(big["buckets"]))
            else:
                rows.append((tokens[t - 1] * int(big["mul_prev"]) + tok * int(big["mul_cur"])) % int(big["buckets"]))
        x = x + w["bigram"].float()[torch.tensor(rows, dtype=torch.long)]
    return x


def stabilised_memory(q, k, v, li, lf):
    """``q, k`` [T, H, D], ``v`` [T, H, Dv], log gates ``li, lf`` [T, H]: the matrix memory S, the sum of keys n
    and the running maximum m (all from zero), read after the update and divided by max(|n . q|, exp(-m)) + 1e-6."""
    T, H, D = q.shape
    Dv = v.shape[2]
    S = torch.zeros(H, D, Dv)
    n = torch.zeros(H, D)
    m = torch.zeros(H)
    out = torch.zeros(T, H, Dv)
    for t in range(T):
        m_new = torch.maximum(lf[t] + m, li[t])
        a = torch.exp(lf[t] + m - m_new)
        b = torch.exp(li[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    return out


def sink_window_attention(q, k, v, scale, window, keep, sink=True):
    """``q`` [T, H, D], ``k`` [T, G, D], ``v`` [T, G, Dv]: token i sees j <= i with i - j < window or j < keep
    (``window`` None: every j <= i); the softmax's denominator has one added (``sink`` False: a plain softmax)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2])
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & ((i - j < int(window)) | (j < int(keep)))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].t()) * scale
        s = s.masked_fill(~seen, float("-inf"))
        top = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - top)
        prob = e / ((torch.exp(-top) if sink else 0.0) + e.sum(-1, keepdim=True))
        out[:, hd] = prob @ v[:, g]
    return out


def bonus_memory(r, k, v, decay, u):
    """``r, k, decay`` [T, H, D], ``v`` [T, H, Dv], ``u`` [H, D]: the state is read before its update, the present
    token counting with the bonus u; then every key channel decays and the token is added."""
    T, H, D = r.shape
    S = torch.zeros(H, D, v.shape[2])
    out = torch.zeros(T, H, v.shape[2])
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    return out


def mlstm_mixer(h, p, w, prefix, eps, dtype):
    """Matrix memory with exponential gates and a running maximum as stabiliser (starting at 0)."""
    T = h.shape[0]
    H, D, Dv, cap = int(p["heads"]), int(p["dim"]), int(p["vdim"]), float(p["gate_cap"])
    q = lin(h, w[prefix + "q"], dtype).reshape(T, H, D) * D ** -0.5
    k = lin(h, w[prefix + "k"], dtype).reshape(T, H, D)
    v = lin(h, w[prefix + "v"], dtype).reshape(T, H, Dv)
    zi = lin(h, w[prefix + "i"], dtype) + w[prefix + "i.b"].float()
    zf = lin(h, w[prefix + "f"], dtype) + w[prefix + "f.b"].float()
    li = cap * torch.tanh(zi / cap)
    lf = F.logsigmoid(cap * torch.tanh(zf / cap))
    out = stabilised_memory(q, k, v, li, lf)
    o = head_unit_norm(out, eps).reshape(T, H * Dv) * w[prefix + "norm"].float()
    gate = torch.sigmoid(lin(h, w[prefix + "g"], dtype))
    return lin(o * gate, w[prefix + "o"], dtype)


def attention_mixer(h, p, w, prefix, eps, dtype):
    """Grouped heads, q/k unit norm with a shared weight, no positions in the scores, a window that also
    keeps the sequence's first tokens, a softmax whose denominator has one added, a sigmoid output gate."""
    T = h.shape[0]
    H, G, D, Dv = int(p["heads"]), int(p["kv_heads"]), int(p["dim"]), int(p["vdim"])
    mask = p.get("mask") or {}
    window, keep = mask.get("size"), int(mask.get("keep_first") or 0)
    q = lin(h, w[prefix + "q"], dtype).reshape(T, H, D)
    k = lin(h, w[prefix + "k"], dtype).reshape(T, G, D)
    v = lin(h, w[prefix + "v"], dtype).reshape(T, G, Dv)
    q = (head_unit_norm(q, eps) * w[prefix + "q.norm"].float()).to(dtype).float()
    k = (head_unit_norm(k, eps) * w[prefix + "k.norm"].float()).to(dtype).float()
    out = sink_window_attention(q, k, v, float(p["scale"]), window, keep)
    out = out.to(dtype).float().reshape(T, H * Dv)
    gate = torch.sigmoid(lin(h, w[prefix + "g"], dtype))
    return lin(out * gate, w[prefix + "o"], dtype)


def wkv_mixer(h, p, w, prefix, eps, dtype):
    """Token-shifted inputs, a decay per key channel and token, a bonus for the present token only."""
    T, W = h.shape
    H, D = int(p["heads"]), int(p["dim"])
    prev = torch.cat([torch.zeros(1, W), h[:-1]], dim=0)

    def mixed(s):
        return h + (prev - h) * w[prefix + "mu." + s].float()

    r = lin(mixed("r"), w[prefix + "r"], dtype).reshape(T, H, D)
    k = lin(mixed("k"), w[prefix + "k"], dtype).reshape(T, H, D)
    v = lin(mixed("v"), w[prefix + "v"], dtype).reshape(T, H, D)
    gate = F.silu(lin(mixed("g"), w[prefix + "g"], dtype))
    low = torch.tanh(lin(mixed("w"), w[prefix + "w1"], dtype)).to(dtype).float()
    z = lin(low, w[prefix + "w2"], dtype) + w[prefix + "w0"].float()
    decay = torch.exp(-torch.exp(z)).reshape(T, H, D)
    u = w[prefix + "u"].float().reshape(H, D)
    out = bonus_memory(r, k, v, decay, u)
    o = head_unit_norm(out, eps).reshape(T, H * D) * w[prefix + "norm"].float()
    return lin(o * gate, w[prefix + "o"], dtype)


def dense_feed_forward(h, p, w, prefix, dtype):
    limit = float(p["limit"])
    g = torch.clamp(lin(h, w[prefix + "gate"], dtype), max=limit)
    u = torch.clamp(lin(h, w[prefix + "up"], dtype), min=-limit, max=limit)
    y = (g * torch.sigmoid(1.702 * g) * (u + 1.0)).to(dtype).float()
    return lin(y, w[prefix + "down"], dtype)


def route(h, p, w, prefix):
    """``(chosen [T, top], weights [T, top])``: softmax over all router outputs, a correction added for the
    choice only, the choice limited to the best groups, weights renormalised over the chosen."""
    r = p["router"]
    n_all, top = int(r["experts"]) + int(r.get("identity") or 0), int(r["top"])
    z = h.float() @ w[prefix + "router"].float().t()
    s = torch.softmax(z, dim=-1)
    choice = s + w[prefix + "correction"].float()
    groups = r.get("groups")
    if groups and int(groups["count"]) > 1:
        count, keep = int(groups["count"]), int(groups["keep"])
        best = choice.reshape(-1, count, n_all // count).max(-1).values
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        choice = choice.masked_fill(~kept.repeat_interleave(n_all // count, dim=1), float("-inf"))
    chosen = choice.topk(top, dim=-1).indices
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20)


def expert_feed_forward(h, p, w, prefix, dtype, route_from=None):
    """Each token through its chosen experts; the last ``identity`` router outputs stand for experts that
    return their input."""
    n_real = int(p["router"]["experts"])
    chosen, weights = route(h.to(dtype).float() if route_from is None else route_from, p, w, prefix)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        x = h[t:t + 1]
        for e, wt in zip(chosen[t].tolist(), weights[t].tolist()):
            if e >= n_real:
                y = x.to(dtype).float()
            else:
                mid = (F.silu(lin(x, w[f"{prefix}e{e}.gate"], dtype)) * lin(x, w[f"{prefix}e{e}.up"], dtype))
                y = lin(mid.to(dtype).float(), w[f"{prefix}e{e}.down"], dtype)
            out[t] += wt * y[0]
    return out


def run_order(cfg: dict) -> list[tuple[int, bool]]:
    """(layer, whether a pass of the loop starts here), in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward(cfg: dict, w: dict, tokens: list[int], dtype: torch.dtype = torch.float32, layers_out: list | None = None):
    """Float32 logits ``[T, vocab]`` of one sequence.  ``layers_out``: a list that receives the residual sum
    after every layer run."""
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups") or 1)
    x0 = embedding(cfg, w, tokens)
    x = x0.clone()
    for layer, pass_starts in run_order(cfg):
        if pass_starts:
            x = lin(torch.cat([x, x0], dim=-1), w["loop.in"], dtype)
        L = cfg["layers"][layer]
        pre = f"l{layer}."
        h1 = grouped_rms_norm(x, w[pre + "norm1"], groups, eps).to(dtype).float()
        mix = {"mlstm": mlstm_mixer, "attention": attention_mixer, "wkv": wkv_mixer}[L["type"]]
        y = mix(h1, L["mixer"], w, pre + "mix.", eps, dtype)
        if L.get("mlp"):
            h2 = grouped_rms_norm(x, w[pre + "norm2"], groups, eps).to(dtype).float()
            if L["mlp"]["kind"] == "dense":
                y = y + dense_feed_forward(h2, L["mlp"], w, pre + "mlp.", dtype)
            else:
                y = y + expert_feed_forward(h2, L["mlp"], w, pre + "mlp.", dtype)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    h = grouped_rms_norm(x, w["final.norm"], groups, eps).to(dtype).float()
    return h @ w["head"].to(dtype).float().t()
