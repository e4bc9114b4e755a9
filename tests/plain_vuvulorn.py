"""A plain, slow restatement of the Vuvulorn design in NumPy float64: one function per mechanism,
whole sequences at once, no cache and no batching.  It shares no code with the package; the tests
compare the engine's logits (prefill, decoding through the cache, portions, mixed batches) with it.

Notation: ``x`` is ``[tokens, width]``; linear weights are ``[out, in]`` and applied as ``x @ W.T``.
Tensor names are the checkpoint's: ``l<i>.mix.left.q``, ``l<i>.mlp.e3.gate`` and so on.
"""

from __future__ import annotations

import numpy as np

__all__ = [
    "delta_rule", "dense_mlp", "forward", "gated_delta_mixer", "kept_window_mask", "layer", "moe_mlp", "parallel_mixer",
    "rms_norm", "rotate", "route", "short_convolution", "windowed_attention",
]


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_norm(x, weight, eps):
    """``x / sqrt(mean(x^2) + eps) * weight`` over the last axis (``weight=None``: no scale)."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if weight is None else y * weight


def rotate(x, positions, dims, base):
    """Rotary positions on the first ``dims`` channels of ``x [tokens, heads, dim]``: channel ``i`` pairs with
    ``i + dims/2``; the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * base^(-2i/dims)."""
    half = dims // 2
    out = x.copy()
    if half == 0:
        return out
    freq = base ** (-2.0 * np.arange(half) / dims)
    angle = positions[:, None].astype(np.float64) * freq[None, :]
    cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def kept_window_mask(n, size, keep_first):
    """``mask[i, j]``: position i sees j iff ``j <= i`` and (``i - j < size`` or ``j < keep_first``)."""
    i = np.arange(n)[:, None]
    j = np.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def windowed_attention(h, w, prefix, c, eps):
    """The softmax branch: biased q/k/v, per-head RMS norm of q and k (one weight for all heads), rotation,
    scaled scores under the window-with-kept-first-tokens mask, softmax, biased out-projection."""
    n = h.shape[0]
    heads, groups, dim, vdim = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (h @ w[prefix + "q"].T + w[prefix + "q.b"]).reshape(n, heads, dim)
    k = (h @ w[prefix + "k"].T + w[prefix + "k.b"]).reshape(n, groups, dim)
    v = (h @ w[prefix + "v"].T + w[prefix + "v.b"]).reshape(n, groups, vdim)
    q = rms_norm(q, w[prefix + "q.norm"], eps)
    k = rms_norm(k, w[prefix + "k.norm"], eps)
    positions = np.arange(n)
    q = rotate(q, positions, c["rot"]["dims"], c["rot"]["base"])
    k = rotate(k, positions, c["rot"]["dims"], c["rot"]["base"])
    mask = kept_window_mask(n, c["mask"]["size"], c["mask"]["keep_first"])
    out = np.zeros((n, heads, vdim))
    per = heads // groups
    for head in range(heads):
        g = head // per
        scores = (q[:, head] @ k[:, g].T) * c["scale"]
        scores = np.where(mask, scores, -np.inf)
        scores = scores - scores.max(axis=-1, keepdims=True)
        p = np.exp(scores)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, head] = p @ v[:, g]
    return out.reshape(n, heads * vdim) @ w[prefix + "o"].T + w[prefix + "o.b"]


def short_convolution(x, taps_weight):
    """Causal depthwise convolution over time: ``y[t, c] = sum_j weight[c, taps-1-j] * x[t-j, c]``
    (the last column multiplies the current token), zeros before the start."""
    n, channels = x.shape
    taps = taps_weight.shape[1]
    y = np.zeros_like(x)
    for j in range(taps):
        shifted = np.zeros_like(x)
        shifted[j:] = x[: n - j] if j else x
        y += shifted * taps_weight[None, :, taps - 1 - j]
    return y


def delta_rule(q, k, v, beta, g):
    """Per head, token by token: ``S <- g_t * S`` (one decay per key channel, acting on S's rows),
    ``u = beta_t (v_t - S^T k_t)``, ``S <- S + k_t u^T``, ``o_t = S^T q_t``.  Shapes: q, k, g ``[n, heads, dim]``,
    v ``[n, heads, vdim]``, beta ``[n, heads]``.  The state starts at zero."""
    n, heads, dim = q.shape
    vdim = v.shape[-1]
    out = np.zeros((n, heads, vdim))
    for head in range(heads):
        S = np.zeros((dim, vdim))
        for t in range(n):
            S = g[t, head][:, None] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, head])
            S = S + np.outer(k[t, head], u)
            out[t, head] = S.T @ q[t, head]
    return out


def gated_delta_mixer(h, w, prefix, c, eps):
    """The recurrent branch: projections, short convolutions with silu, unit q and k, beta, per-channel decay,
    the delta rule, per-head RMS norm of the read-out times a low-rank sigmoid gate, out-projection."""
    n = h.shape[0]
    heads, groups, dim, vdim = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    per = heads // groups
    q = silu(short_convolution(h @ w[prefix + "q"].T, w[prefix + "q.conv"])).reshape(n, groups, dim)
    k = silu(short_convolution(h @ w[prefix + "k"].T, w[prefix + "k.conv"])).reshape(n, groups, dim)
    v = silu(short_convolution(h @ w[prefix + "v"].T, w[prefix + "v.conv"])).reshape(n, heads, vdim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    q = np.repeat(q, per, axis=1)
    k = np.repeat(k, per, axis=1)
    beta = sigmoid(h @ w[prefix + "b"].T)
    step = softplus((h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "dt_bias"]).reshape(n, heads, dim)
    g = np.exp(-np.exp(w[prefix + "A_log"])[None, :, None] * step)
    o = delta_rule(q, k, v, beta, g)
    o = rms_norm(o, w[prefix + "norm"], eps)
    gate = sigmoid((h @ w[prefix + "g1"].T) @ w[prefix + "g2"].T).reshape(n, heads, vdim)
    return (o * gate).reshape(n, heads * vdim) @ w[prefix + "o"].T


def parallel_mixer(h, w, prefix, c, eps):
    left = windowed_attention(h, w, prefix + "left.", c["left"], eps)
    right = gated_delta_mixer(h, w, prefix + "right.", c["right"], eps)
    return c["left_scale"] * left + c["right_scale"] * right


def dense_mlp(h, w, prefix):
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h, router_weight, c):
    """Sigmoid scores; experts in ``groups.count`` equal groups of neighbours, a group scored by the sum of its two
    largest scores, only the best ``groups.keep`` groups eligible; the ``top`` largest eligible scores are chosen and
    are the weights as they are.  Returns ``(indices [n, top], weights [n, top])``."""
    scores = sigmoid(h @ router_weight.T)
    n, experts = scores.shape
    count, keep, top = c["groups"]["count"], c["groups"]["keep"], c["top"]
    grouped = scores.reshape(n, count, experts // count)
    group_score = np.sort(grouped, axis=-1)[..., -2:].sum(-1) if experts // count >= 2 else grouped.sum(-1)
    best = np.argsort(-group_score, axis=-1, kind="stable")[:, :keep]
    allowed = np.zeros((n, count), dtype=bool)
    np.put_along_axis(allowed, best, True, axis=-1)
    allowed = np.repeat(allowed, experts // count, axis=-1)
    masked = np.where(allowed, scores, -np.inf)
    chosen = np.argsort(-masked, axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(scores, chosen, axis=-1)


def moe_mlp(h, w, prefix, c):
    chosen, weights = route(h, w[prefix + "router"], c["router"])
    out = np.zeros((h.shape[0], w[prefix + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t], weights[t]):
            out[t] += s * dense_mlp(h[t : t + 1], w, f"{prefix}e{e}.")[0]
    return out


def layer(x, w, index, c, eps):
    """``x <- x + norm1(mixer(x))``, then ``x <- x + norm2(ff(x))``: the sublayers read the stream itself."""
    prefix = f"l{index}."
    if c["type"] != "parallel":
        raise ValueError(f"unknown layer type {c['type']!r}")
    x = x + rms_norm(parallel_mixer(x, w, prefix + "mix.", c["mixer"], eps), w[prefix + "norm1"], eps)
    mlp = c.get("mlp")
    if mlp is not None:
        y = dense_mlp(x, w, prefix + "mlp.") if mlp["kind"] == "dense" else moe_mlp(x, w, prefix + "mlp.", mlp)
        x = x + rms_norm(y, w[prefix + "norm2"], eps)
    return x


def forward(config, weights, tokens, return_layers=False):
    """Logits ``[tokens, vocab]`` of one whole sequence (float64)."""
    w = {name: np.asarray(value, dtype=np.float64) for name, value in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    streams = []
    for index, c in enumerate(config["layers"]):
        x = layer(x, w, index, c, eps)
        streams.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(streams)) if return_layers else logits
