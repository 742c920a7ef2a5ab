"""Plain, slow implementation of the Sapanex decoder, the oracle of its tests.

Whole sequences, no cache, no batching, one function per mechanism, elementary
torch operations in float64 unless told otherwise.  It shares no code with the
package under test: it takes a configuration dictionary and a dictionary of
tensors by their checkpoint names.

Notation.  ``x`` is the residual stream ``[T, width]`` of one sequence whose
positions are 0..T-1.  A layer is ``x <- N1(alpha x + Mix(x))`` followed, when it
has a feed-forward, by ``x <- N2(alpha x + FF(x))``, with
``N(y) = y / sqrt(mean(y^2) + eps) * gain``.
"""

from __future__ import annotations

import math

import torch


def rms_norm(y, gain, eps):
    """``y / sqrt(mean(y^2) + eps) * gain`` over the last axis."""
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * gain


def unit_rms(y, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def rotary_frequencies(dims, base, scaling):
    """(frequencies ``[dims/2]``, amplitude) of a rotation over ``dims`` dimensions.

    Plain: ``f_i = base^(-2i/dims)``, amplitude 1.  With YaRN scaling
    (factor s, original length L, fast and slow turn counts): the dimension at which a
    wave makes t turns over L is ``d(t) = dims ln(L / (2 pi t)) / (2 ln base)``;
    ``lo = max(floor d(fast), 0)``, ``hi = min(ceil d(slow), dims-1)``,
    ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``,
    ``f_i <- f_i / s * ramp_i + f_i (1 - ramp_i)``, amplitude ``0.1 ln s + 1``.
    """
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    amp = 1.0
    if scaling:
        s, orig = float(scaling["factor"]), float(scaling["original"])

        def d(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(d(float(scaling["fast"]))), 0)
        hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / s * ramp + f[i] * (1.0 - ramp)
        amp = 0.1 * math.log(s) + 1.0
    return torch.tensor(f, dtype=torch.float64), amp


def rotate_halves(t, positions, freqs, amp=1.0, sign=1.0):
    """Turn pairs (i, i + n/2) of the last axis (size n = 2 len(freqs)) of ``t``
    ``[T, heads, n]`` by ``sign * position * freqs[i]``; cos and sin times ``amp``."""
    half = freqs.numel()
    ang = sign * positions.to(torch.float64)[:, None] * freqs[None, :]
    c = (torch.cos(ang) * amp).to(t.dtype)[:, None, :]
    s = (torch.sin(ang) * amp).to(t.dtype)[:, None, :]
    u, v = t[..., :half], t[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s], dim=-1)


def visible_tokens(i, window):
    """Positions a query at ``i`` sees as single tokens."""
    return list(range(max(0, i - window + 1), i + 1)) if window else list(range(i + 1))


def visible_blocks(i, window, pool):
    """Pooled blocks a query at ``i`` sees: block b (positions bP..bP+P-1) when its last
    position is at most ``i - window``."""
    if not window or not pool:
        return []
    return [b for b in range((i + 1) // pool + 1) if b * pool + pool - 1 <= i - window]


def attention_mixer(h, w, prefix, m, eps):
    """Grouped-query attention with a sliding window and pooled blocks before it.

    ``m`` is the layer's ``mixer`` dictionary.  Queries and keys: projection, RMS norm
    with a gain over the whole projection (all heads at once), rotation of the first
    ``rot.dims`` dimensions of each head.  Values of position j are turned by j over all of
    ``vdim`` (plain frequencies of the same base), and each head's output at position i is
    turned back by -i.  Block b's key and value are the means of its tokens' keys and values
    as stored (after norm and rotation).  Tokens in the window and visible blocks share one
    softmax of ``scale * q.k``.
    """
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = h @ w[prefix + "q"].T
    k = h @ w[prefix + "k"].T
    v = h @ w[prefix + "v"].T
    q = rms_norm(q, w[prefix + "q.norm"], eps).view(T, H, D)
    k = rms_norm(k, w[prefix + "k.norm"], eps).view(T, G, D)
    v = v.view(T, G, V)
    rot = m.get("rot")
    if rot:
        rd = rot["dims"]
        f, amp = rotary_frequencies(rd, rot["base"], rot.get("scaling"))
        q = torch.cat([rotate_halves(q[..., :rd], pos, f, amp), q[..., rd:]], dim=-1)
        k = torch.cat([rotate_halves(k[..., :rd], pos, f, amp), k[..., rd:]], dim=-1)
        fv, _ = rotary_frequencies(V, rot["base"], None)
        v = rotate_halves(v, pos, fv)
    mask = m.get("mask") or {}
    window, pool = mask.get("size"), mask.get("pool")
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for i in range(T):
        toks = visible_tokens(i, window)
        blocks = visible_blocks(i, window, pool)
        keys = [k[b * pool:(b + 1) * pool].mean(0) for b in blocks] + [k[j] for j in toks]
        vals = [v[b * pool:(b + 1) * pool].mean(0) for b in blocks] + [v[j] for j in toks]
        K = torch.stack(keys)   # [n, G, D]
        Vv = torch.stack(vals)  # [n, G, V]
        for hh in range(H):
            g = hh // (H // G)
            p = torch.softmax((K[:, g] @ q[i, hh]) * m["scale"], dim=0)
            out[i, hh] = p @ Vv[:, g]
    if rot:
        out = rotate_halves(out, pos, fv, sign=-1.0)
    return out.reshape(T, H * V) @ w[prefix + "o"].T


def general_delta_mixer(h, w, prefix, m, eps, state=None):
    """Generalised delta rule with a matrix state per head.

    Per token and head, with key channel c and value channel d:
    ``decay_c = exp(-exp(-1/2) sigmoid(W2 tanh(W1 h) + w0)_c)``,
    ``rate_c = sigmoid(Wa h + ba)_c``, ``u = k / sqrt(sum k^2 + 1e-6)``,
    ``S <- diag(decay) S - (rate * u)(u^T S) + k v^T`` (both terms read the old S),
    ``o = S^T r``.  Each head's o is divided by its root mean square, all heads together
    times a gain, times ``sigmoid(Wg h)``, then the output projection.
    Returns (output, last state).
    """
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ w[prefix + "r"].T).view(T, H, D)
    k = (h @ w[prefix + "k"].T).view(T, H, D)
    v = (h @ w[prefix + "v"].T).view(T, H, D)
    gate = torch.sigmoid(h @ w[prefix + "g"].T)
    low = torch.tanh(h @ w[prefix + "w1"].T)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(low @ w[prefix + "w2"].T + w[prefix + "w0"]))
    decay = decay.view(T, H, D)
    rate = torch.sigmoid(h @ w[prefix + "a"].T + w[prefix + "a.b"]).view(T, H, D)
    S = torch.zeros(H, D, D, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, D, dtype=h.dtype)
    for t in range(T):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum(-1, keepdim=True) + 1e-6)
        uS = torch.einsum("hc,hcd->hd", u, S)
        S = decay[t][:, :, None] * S - (rate[t] * u)[:, :, None] * uS[:, None, :] \
            + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hcd,hc->hd", S, r[t])
    o = unit_rms(o, eps).reshape(T, H * D) * w[prefix + "norm"] * gate
    return o @ w[prefix + "o"].T, S


def feed_forward(h, w, prefix):
    """``W_down relu(W_up h)^2``."""
    return torch.relu(h @ w[prefix + "up"].T) ** 2 @ w[prefix + "down"].T


def run_layer(x, w, index, layer, cfg):
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    p = f"l{index}."
    if layer["type"] == "attention":
        mixed = attention_mixer(x, w, p + "mix.", layer["mixer"], eps)
    elif layer["type"] == "general_delta":
        mixed, _ = general_delta_mixer(x, w, p + "mix.", layer["mixer"], eps)
    else:
        raise ValueError(layer["type"])
    x = rms_norm(alpha * x + mixed, w[p + "norm1"], eps)
    if layer.get("mlp"):
        x = rms_norm(alpha * x + feed_forward(x, w, p + "mlp."), w[p + "norm2"], eps)
    return x


def forward(cfg, w, tokens, dtype=torch.float64, layers_out=None):
    """Logits ``[T, vocab]`` of one sequence; ``layers_out`` (a list) receives the residual
    stream after every layer."""
    w = {k: v.to(dtype) if v.is_floating_point() else v for k, v in w.items()}
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        x = run_layer(x, w, i, layer, cfg)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_norm(x, w["final.norm"], cfg["norm"]["eps"])
    return x @ w["embed"].T
