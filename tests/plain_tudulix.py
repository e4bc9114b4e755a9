"""A plain, slow restatement of the Tudulix design in NumPy float64: one function per mechanism,
whole sequences at once, no cache and no batching.  It shares no code with the package; the tests
compare the engine's logits (prefill, decoding through the cache, portions, mixed batches) with it.

Notation: ``x`` is ``[tokens, width]``; linear weights are ``[out, in]`` and applied as ``x @ W.T``.
Tensor names are the checkpoint's: ``l<i>.mix.q``, ``l<i>.mlp.e3.gate`` and so on.
"""

from __future__ import annotations

import numpy as np

__all__ = [
    "expert", "forward", "grouped_attention", "latent_attention", "layer", "layer_runs", "moe", "offset_norm", "rms_norm",
    "rotate_half", "rotate_pairs", "route", "softmax_rows", "window_mask",
]

SIGMOID_SLOPE = 1.702  # the design fixes the slope inside the experts' gate activation


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms_norm(x, weight, eps):
    """``x / sqrt(mean(x^2) + eps) * weight`` over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight


def offset_norm(x, weight, eps):
    """The layers' norm: its weight is an offset from one, ``1 + weight``."""
    return rms_norm(x, 1.0 + weight, eps)


def _angles(positions, dims, base):
    freq = base ** (-2.0 * np.arange(dims // 2) / dims)
    angle = positions[:, None].astype(np.float64) * freq[None, :]
    return np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]


def rotate_pairs(x, positions, dims, base):
    """Rotation of the first ``dims`` channels of ``x [tokens, heads, dim]``, channel ``2i`` paired with ``2i + 1``."""
    out = x.copy()
    if dims == 0:
        return out
    cos, sin = _angles(positions, dims, base)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def rotate_half(x, positions, dims, base):
    """Rotation of the first ``dims`` channels of ``x [tokens, heads, dim]``, channel ``i`` paired with ``i + dims/2``."""
    out = x.copy()
    half = dims // 2
    if half == 0:
        return out
    cos, sin = _angles(positions, dims, base)
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def window_mask(n, size):
    """``mask[i, j]``: position i sees j iff ``0 <= i - j < size``."""
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    return (j <= i) & (i - j < size)


def softmax_rows(scores, mask):
    scores = np.where(mask, scores, -np.inf)
    scores = scores - scores.max(axis=-1, keepdims=True)
    weights = np.exp(scores)
    return weights / weights.sum(axis=-1, keepdims=True)


def grouped_attention(h, w, prefix, c):
    """Softmax attention with grouped key/value heads, pairwise rotation of part of each head, a sliding window."""
    n = h.shape[0]
    heads, groups, dim, vdim = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (h @ w[prefix + "q"].T).reshape(n, heads, dim)
    k = (h @ w[prefix + "k"].T).reshape(n, groups, dim)
    v = (h @ w[prefix + "v"].T).reshape(n, groups, vdim)
    positions = np.arange(n)
    q = rotate_pairs(q, positions, c["rot"]["dims"], c["rot"]["base"])
    k = rotate_pairs(k, positions, c["rot"]["dims"], c["rot"]["base"])
    mask = window_mask(n, c["mask"]["size"])
    out = np.zeros((n, heads, vdim))
    per = heads // groups
    for head in range(heads):
        g = head // per
        out[:, head] = softmax_rows((q[:, head] @ k[:, g].T) * c["scale"], mask) @ v[:, g]
    return out.reshape(n, heads * vdim) @ w[prefix + "o"].T


def latent_attention(h, w, prefix, c, eps):
    """Attention whose keys and values are made from one small latent vector per token, with one rotated key part
    shared by all heads, and a sigmoid gate on the heads' outputs."""
    n = h.shape[0]
    heads, dim, rot, vdim, rank = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    q = (h @ w[prefix + "q"].T).reshape(n, heads, dim + rot)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    down = h @ w[prefix + "dkv"].T
    latent = rms_norm(down[:, :rank], w[prefix + "dkv.norm"], eps)
    k_rot = down[:, rank:].reshape(n, 1, rot)
    positions = np.arange(n)
    q_rot = rotate_half(q_rot, positions, rot, c["rot"]["base"])
    k_rot = rotate_half(k_rot, positions, rot, c["rot"]["base"])
    k_plain = (latent @ w[prefix + "uk"].T).reshape(n, heads, dim)
    v = (latent @ w[prefix + "uv"].T).reshape(n, heads, vdim)
    mask = window_mask(n, c["mask"]["size"])
    out = np.zeros((n, heads, vdim))
    for head in range(heads):
        scores = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot[:, 0].T) * c["scale"]
        out[:, head] = softmax_rows(scores, mask) @ v[:, head]
    gate = sigmoid(h @ w[prefix + "g"].T)
    return (out.reshape(n, heads * vdim) * gate) @ w[prefix + "o"].T


def expert(h, w, prefix, limit):
    """``down(g * sigmoid(1.702 g) * (u + 1))`` with ``g = min(gate h, limit)`` and ``u = clamp(up h, -limit, limit)``."""
    g = np.minimum(h @ w[prefix + "gate"].T, limit)
    u = np.clip(h @ w[prefix + "up"].T, -limit, limit)
    return (g * sigmoid(SIGMOID_SLOPE * g) * (u + 1.0)) @ w[prefix + "down"].T


def route(h, w, prefix, top):
    """The ``top`` experts with the largest biased logits and the softmax over just their logits:
    ``(chosen [tokens, top], weights [tokens, top])``."""
    logits = h @ w[prefix + "router"].T + w[prefix + "router.b"]
    chosen = np.argsort(-logits, axis=-1, kind="stable")[:, :top]
    picked = np.take_along_axis(logits, chosen, axis=-1)
    picked = np.exp(picked - picked.max(axis=-1, keepdims=True))
    return chosen, picked / picked.sum(axis=-1, keepdims=True)


def moe(h, w, prefix, c):
    chosen, weights = route(h, w, prefix, c["router"]["top"])
    out = np.zeros((h.shape[0], w[prefix + "e0.down"].shape[0]))
    for e in range(c["router"]["experts"]):
        for k in range(chosen.shape[1]):
            rows = np.nonzero(chosen[:, k] == e)[0]
            if rows.size:
                out[rows] += weights[rows, k, None] * expert(h[rows], w, f"{prefix}e{e}.", c["expert"]["limit"])
    if c.get("shared") is not None:
        out = out + expert(h, w, prefix + "shared.", c["shared"]["limit"])
    return out


def layer(x, w, index, entry, eps):
    """``x + norm1b(mixer(norm1(x)))`` and then, where the layer has a feed-forward, ``x + norm2b(ff(norm2(x)))``."""
    root = f"l{index}."
    h = offset_norm(x, w[root + "norm1"], eps)
    if entry["type"] == "attention":
        mixed = grouped_attention(h, w, root + "mix.", entry["mixer"])
    elif entry["type"] == "latent_attention":
        mixed = latent_attention(h, w, root + "mix.", entry["mixer"], eps)
    else:
        raise ValueError(entry["type"])
    x = x + offset_norm(mixed, w[root + "norm1b"], eps)
    if entry.get("mlp") is not None:
        h = offset_norm(x, w[root + "norm2"], eps)
        x = x + offset_norm(moe(h, w, root + "mlp.", entry["mlp"]), w[root + "norm2b"], eps)
    return x


def layer_runs(config):
    """The order in which layers run: ``(layer, starts a repeated pass after the first)``."""
    count = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(i, False) for i in range(count)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(start)]
    for turn in range(times):
        runs += [(i, turn > 0 and i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, count)]


def forward(tokens, w, config, collect=None):
    """Logits ``[tokens, vocab]`` of one sequence.  ``collect``: a list that receives the stream after every layer run."""
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * config["embedding"]["scale"]
    start = x.copy()
    for index, again in layer_runs(config):
        if again:
            x = x + start
        x = layer(x, w, index, config["layers"][index], eps)
        if collect is not None:
            collect.append(x.copy())
    x = offset_norm(x, w["final.norm"], eps)
    return (x @ w["head"].T) * config["logit_scale"]
