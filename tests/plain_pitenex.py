"""Plain, slow Pitenex model in numpy float64: the yardstick for the Pitenex tests.

Whole sequences, no cache, no batching, one function per mechanism, nothing shared with the
package under test.  Notation: a sequence of n tokens is a matrix [n, width]; position p of a
sequence is row p; W x for a stored matrix W [out, in] is written ``x @ W.T``.

Mechanisms
----------
``bigram_rows``           which row of the hashed pair table every token adds to its embedding
``layer_norm``            (x - mean) / sqrt(var + eps) * w + b, var the mean squared deviation
``rotate_pairs``          elements (2i, 2i+1) of the first ``dims`` of a head turned by p * base^(-2i/dims)
``chunked_attention``     grouped-query attention whose keys and values have sizes of their own, a mask of
                          chunks counted from position 0, a sink term per head in the softmax's denominator
``short_conv``            causal convolution over time per channel (zeros before the start), then silu
``delta_rule``            the gated delta rule as a token-by-token recurrence with a decay per key channel
``delta_mixer``           projections, convolutions, unit vectors, the recurrence, the heads' norm and gate
``dense_ff``              down(gelu_tanh(gate x) * up x)
``expert_ff``             down(g sigmoid(1.702 g) (u + 1)) with g and u clamped
``route``                 softmax router with a correction on the choice only, the chosen scores renormed
``moe_ff``                the chosen experts (the last ones identities) plus the shared expert
``forward``               the whole model: logits at every position and the residual after every layer
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    rows = [buckets]
    for p in range(1, len(tokens)):
        rows.append((int(tokens[p - 1]) * mul_prev + int(tokens[p]) * mul_cur) % buckets)
    return np.asarray(rows[:len(tokens)], dtype=np.int64)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rotate_pairs(x, dims, base):
    """x [n, heads, size]: row p is at position p; only the first ``dims`` elements of a head turn."""
    n = x.shape[0]
    i = np.arange(dims // 2, dtype=F64)
    ang = np.arange(n, dtype=F64)[:, None] * (base ** (-2.0 * i / dims))[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def chunked_attention(h, w, m):
    """h [n, width]; w: the tensors q, k, v, sink, o; m: heads, kv_heads, dim, vdim, rot, scale, mask.size (absent: none)."""
    n = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(n, H, dim)
    k = (h @ w["k"].T).reshape(n, G, dim)
    v = (h @ w["v"].T).reshape(n, G, vdim)
    rot = m.get("rot")
    if rot and rot["dims"]:
        q, k = rotate_pairs(q, rot["dims"], float(rot["base"])), rotate_pairs(k, rot["dims"], float(rot["base"]))
    size = (m.get("mask") or {}).get("size") or n + 1          # no mask: every earlier key
    out = np.zeros((n, H, vdim), dtype=F64)
    for p in range(n):
        lo = (p // size) * size
        for hd in range(H):
            g = hd // (H // G)
            s = (k[lo:p + 1, g] @ q[p, hd]) * m["scale"]
            top = max(s.max(), w["sink"][hd])
            e = np.exp(s - top)
            out[p, hd] = (e @ v[lo:p + 1, g]) / (e.sum() + math.exp(w["sink"][hd] - top))
    return out.reshape(n, H * vdim) @ w["o"].T


def short_conv(x, taps_w):
    """x [n, channels], taps_w [channels, taps], the last column is the current token's."""
    n, taps = x.shape[0], taps_w.shape[1]
    y = np.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < n:
            y[back:] += x[:n - back] * taps_w[:, j]
    return silu(y)


def delta_rule(q, k, v, beta, g):
    """One head.  q, k [n, dim], v [n, vdim], beta [n], g [n, dim] (decay of the state's rows).  Returns o [n, vdim]."""
    n, dim = q.shape
    S = np.zeros((dim, v.shape[1]), dtype=F64)
    o = np.zeros_like(v)
    for t in range(n):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def delta_mixer(h, w, m, eps):
    n = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(h @ w["q"].T, w["q.conv"]).reshape(n, G, dim)
    k = short_conv(h @ w["k"].T, w["k.conv"]).reshape(n, G, dim)
    v = short_conv(h @ w["v"].T, w["v.conv"]).reshape(n, H, vdim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w["b"].T)                                                       # [n, H]
    dt = softplus((h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]).reshape(n, H, dim)
    g = np.exp(-np.exp(w["A_log"])[None, :, None] * dt)
    gate = sigmoid((h @ w["g1"].T) @ w["g2"].T).reshape(n, H, vdim)
    out = np.zeros((n, H, vdim), dtype=F64)
    for hd in range(H):
        kv = hd // (H // G)
        o = delta_rule(q[:, kv], k[:, kv], v[:, hd], beta[:, hd], g[:, hd])
        out[:, hd] = o / np.sqrt((o * o).mean(-1, keepdims=True) + eps) * w["norm"] * gate[:, hd]
    return out.reshape(n, H * vdim) @ w["o"].T


def parallel_mixer(h, w, m, eps):
    left = chunked_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, m["left"])
    right = delta_mixer(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def dense_ff(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def expert_ff(h, gate, up, down, limit):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, router, correction, top):
    """(chosen experts [n, top], their weights [n, top])."""
    z = h @ router.T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    chosen = np.argsort(-(s + correction), axis=-1, kind="stable")[:, :top]
    picked = np.take_along_axis(s, chosen, axis=-1)
    return chosen, picked / (picked.sum(-1, keepdims=True) + 1e-20)


def moe_ff(h, w, m):
    r = m["router"]
    E, top = r["experts"], r["top"]
    chosen, weight = route(h, w["router"], w["correction"], top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t], weight[t]):
            if e >= E:
                out[t] += a * h[t]                       # an identity expert
            else:
                out[t] += a * expert_ff(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], m["expert"]["limit"])[0]
    if m.get("shared"):
        out += expert_ff(h, w["shared.gate"], w["shared.up"], w["shared.down"], m["shared"]["limit"])
    return out


def forward(cfg, tensors, tokens):
    """(logits [n, vocab], residual after every layer [layers, n, width]) for one sequence."""
    W = {k: np.asarray(v, dtype=F64) for k, v in tensors.items()}
    big = cfg["embedding"]["bigram"]
    tokens = np.asarray(tokens, dtype=np.int64)
    x = W["embed"][tokens] + W["bigram"][bigram_rows(tokens, big["buckets"], big["mul_prev"], big["mul_cur"])]
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = layer_norm(x, W[pre + "norm1"], W[pre + "norm1.b"], eps)
        y = parallel_mixer(h, {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mix.")}, layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            wm = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mlp.")}
            y = y + (dense_ff(h, wm) if mlp["kind"] == "dense" else moe_ff(h, wm, mlp))
        x = x + mult * y
        after.append(x.copy())
    h = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return (h @ W["embed"].T) * cfg["logit_scale"], np.stack(after)
