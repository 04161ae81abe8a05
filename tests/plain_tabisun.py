"""Tabisun stated plainly: whole sequences, no cache, one function per mechanism, float64 or float32.

Nothing here is shared with the package.  A model is ``(config, tensors)``: ``config`` the dictionary of a
config.json, ``tensors`` name -> tensor.  Notation: ``x`` is the stream ``[T, W]``; a layer computes
``x += LN_1(mixer(x))`` and ``x += LN_2(ff(x))`` with the sublayers reading ``x`` itself.
"""

from __future__ import annotations

import math

import torch

ACTIVATIONS = None  # a dtype: products' results and sublayer inputs are rounded to it (a model of 16-bit activations)


def _r(x):
    return x if ACTIVATIONS is None else x.to(ACTIVATIONS).to(x.dtype)


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def scaled_frequencies_by_wavelength(dims, base, scaling, dtype):
    """f_i = base^(-2i/dims); long waves slowed by ``factor``, short ones kept, a linear blend between."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=dtype)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for fi in f.tolist():
        wave = 2 * math.pi / fi
        if wave < original / high:
            out.append(fi)
        elif wave > original / low:
            out.append(fi / factor)
        else:
            s = (original / wave - low) / (high - low)
            out.append((1 - s) * fi / factor + s * fi)
    return torch.tensor(out, dtype=dtype)


def ramped_frequencies(dims, base, scaling, dtype):
    """(frequencies, magnitude): a ramp over the pair index between the fast and the slow turn counts
    blends f_i / factor with f_i; cos and sin are multiplied by 0.1 ln(factor) + 1."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return torch.tensor(f, dtype=dtype), 1.0
    factor, original, fast, slow = (float(scaling[k]) for k in ("factor", "original", "fast", "slow"))

    def index_of(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1 - ramp))
    return torch.tensor(out, dtype=dtype), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, pairing, magnitude=1.0):
    """x ``[T, heads, D]``: the first ``2 * len(freqs)`` elements of each head turn by position * f_i."""
    n = freqs.numel()
    ang = positions.to(freqs.dtype)[:, None] * freqs[None, :]
    cos, sin = (torch.cos(ang) * magnitude)[:, None, :], (torch.sin(ang) * magnitude)[:, None, :]
    out = x.clone()
    if pairing == "interleaved":
        u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2] = u * cos - v * sin
        out[..., 1:2 * n:2] = v * cos + u * sin
    else:
        u, v = x[..., :n], x[..., n:2 * n]
        out[..., :n] = u * cos - v * sin
        out[..., n:2 * n] = v * cos + u * sin
    return out


def softmax_rows(scores, visible, sink=None):
    """scores ``[H, T, T]``, visible ``[T, T]`` bool; ``sink`` ``[H]``: one more term exp(sink_h) in the
    denominator, with no value behind it."""
    s = scores.masked_fill(~visible[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


def causal(T):
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


def chunked(T, size):
    i = torch.arange(T)
    return (i[None, :] <= i[:, None]) & ((i[None, :] // size) == (i[:, None] // size))


def differential_core(q, k, v, scale, lam, chunk, eps, out_scale):
    """q ``[T, H, 2, D]``, k ``[T, G, 2, D]`` (normed), v ``[T, G, Dv]`` -> ``[T, H, Dv]``: per head
    a1 - lam * a2 over the same values, divided by its root mean square, times ``out_scale``."""
    T, H = q.shape[0], q.shape[1]
    rep = H // k.shape[1]
    visible = chunked(T, chunk) if chunk else causal(T)
    outs = []
    for hq in range(H):
        g = hq // rep
        a = [softmax_rows(((q[:, hq, which] @ k[:, g, which].T) * scale)[None], visible)[0] @ v[:, g]
             for which in range(2)]
        outs.append(rms_norm(a[0] - lam * a[1], None, eps) * out_scale)
    return torch.stack(outs, 1)


def differential_attention(h, t, p, m, eps):
    """Two score maps per head over shared values; o = a1 - lambda a2, unit RMS per head, times (1 - diff)."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = _r(rms_norm(_r(h @ t[p + "q"].T).view(T, H, 2, D), t[p + "q.norm"], eps))
    k = _r(rms_norm(_r(h @ t[p + "k"].T).view(T, G, 2, D), t[p + "k.norm"], eps))
    v = _r(h @ t[p + "v"].T).view(T, G, Dv)
    lam = (torch.exp((t[p + "lq1"] * t[p + "lk1"]).sum()) - torch.exp((t[p + "lq2"] * t[p + "lk2"]).sum())
           + m["diff"])
    chunk = (m.get("mask") or {}).get("size")
    o = _r(differential_core(q, k, v, m["scale"], lam, chunk, eps, 1 - m["diff"]))
    return o.reshape(T, H * Dv) @ t[p + "o"].T


def capped_core(q, k, v, scale, softcap):
    """q ``[T, H, D]``, k ``[T, G, D]``, v ``[T, G, Dv]`` -> ``[T, H, Dv]``: causal softmax of capped scores."""
    T, H = q.shape[0], q.shape[1]
    rep = H // k.shape[1]
    outs = []
    for hq in range(H):
        g = hq // rep
        s = (q[:, hq] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        outs.append(softmax_rows(s[None], causal(T))[0] @ v[:, g])
    return torch.stack(outs, 1)


def key_value_attention(h, t, p, m, eps):
    """Grouped heads whose values are the projected keys (before norm and rotation); capped scores."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = _r(h @ t[p + "q"].T).view(T, H, D)
    k_raw = _r(h @ t[p + "k"].T).view(T, G, D)
    q, k = rms_norm(q, t[p + "q.norm"], eps), rms_norm(k_raw, t[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot:
        pos = torch.arange(T)
        freqs = scaled_frequencies_by_wavelength(rot["dims"], rot["base"], rot.get("scaling"), h.dtype)
        q, k = rotate(q, pos, freqs, "interleaved"), rotate(k, pos, freqs, "interleaved")
    o = _r(capped_core(_r(q), _r(k), k_raw, m["scale"], m.get("softcap")))
    return o.reshape(T, H * D) @ t[p + "o"].T


def latent_attention(h, t, p, m, eps):
    """Keys and values expanded per head from a normed latent; one rotated key part for all heads; a sink in
    the softmax; a sigmoid gate on the heads' outputs."""
    T = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = _r(h @ t[p + "q"].T).view(T, H, D + R)
    down = _r(h @ t[p + "dkv"].T)
    c = _r(rms_norm(down[:, :C], t[p + "dkv.norm"], eps))
    rot = m["rot"]
    freqs, magnitude = ramped_frequencies(rot["dims"], rot["base"], rot.get("scaling"), h.dtype)
    pos = torch.arange(T)
    k_rot = rotate(down[:, None, C:], pos, freqs, "half", magnitude)[:, 0]
    q_rot = rotate(q[..., D:], pos, freqs, "half", magnitude)
    k_plain = (c @ t[p + "uk"].T).view(T, H, D)
    v = (c @ t[p + "uv"].T).view(T, H, Dv)
    scores = torch.einsum("ihd,jhd->hij", q[..., :D], k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    w = softmax_rows(scores * m["scale"], causal(T), sink=t[p + "sink"].to(h.dtype))
    o = _r(torch.einsum("hij,jhd->ihd", w, v).reshape(T, H * Dv))
    o = _r(o * torch.sigmoid(_r(h @ t[p + "g"].T)))
    return o @ t[p + "o"].T


MIXERS = {"attention": differential_attention, "attention_2": key_value_attention,
          "latent_attention": latent_attention}


def dense_feed_forward(h, t, p):
    z = h @ t[p + "gate"].T
    return _r((z * torch.sigmoid(z)) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def forward(config, tensors, tokens, dtype=torch.float64, with_streams=False, activations=None):
    """Logits ``[T, vocab]`` of one sequence (and the stream after every layer run).  ``activations``: a
    narrower type that sublayer inputs, products' results and sublayer outputs are rounded to, the stream,
    norms, scores and softmax staying in ``dtype``."""
    global ACTIVATIONS
    ACTIVATIONS = activations
    try:
        return _forward(config, tensors, tokens, dtype, with_streams)
    finally:
        ACTIVATIONS = None


def _forward(config, tensors, tokens, dtype, with_streams):
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    streams = []
    for i, layer in enumerate(config["layers"]):
        src = layer.get("weights_of", i)
        if src is None:
            src = i
        p = f"l{src}."
        x = x + layer_norm(_r(MIXERS[layer["type"]](_r(x), t, p + "mix.", layer["mixer"], eps)), t[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + layer_norm(_r(dense_feed_forward(_r(x), t, p + "mlp.")), t[p + "norm2"], eps)
        streams.append(x)
    logits = _r(layer_norm(x, t["final.norm"], eps)) @ t["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(streams)) if with_streams else logits
