"""Plain, slow Ranudra model in numpy float64: the yardstick for the Ranudra tests.

Whole sequences, no cache, no batching, one function per mechanism, nothing shared with the
package under test.  Notation: a sequence of n tokens is a matrix [n, width]; position p of a
sequence is row p; W x for a stored matrix W [out, in] is written ``x @ W.T``.

Mechanisms
----------
``layer_norm``            (x - mean) / sqrt(var + eps) * w, var the mean squared deviation
``rms_norm``              x / sqrt(mean(x^2) + eps) * w
``rotary_frequencies``    f_i = base^(-2i/dims), optionally blended YaRN-wise, and the factor on cos/sin
``rotate_pairs``          neighbouring elements (2i, 2i+1) turned by angle p * f_i
``latent_attention``      keys and values expanded from a normed latent and one shared rotated key part;
                          window, optional sink in the softmax denominator, gate per head or per element
``gla``                   gated linear attention as a token-by-token recurrence with a decay per key channel
``dense_ff``              down(relu(up x)^2)
``hyper_step``            one sublayer under hyper-connections (several residual streams)
``forward``               the whole model: logits at every position and the summed streams after every layer run
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rotary_frequencies(dims, base, scaling=None):
    """(f [dims/2], factor on cos and sin)."""
    i = np.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, freqs, mult):
    """x [n, ..., dims] with dims = 2 len(freqs): elements 2i and 2i+1 turned by positions * freqs[i]."""
    ang = np.asarray(positions, dtype=F64)[:, None] * freqs[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (freqs.shape[0],)
    c, s = (np.cos(ang) * mult).reshape(shape), (np.sin(ang) * mult).reshape(shape)
    u, v = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


def latent_attention(h, w, m, eps, sink=False, gate="head"):
    """h [n, width]; w: the mixer's tensors by local name; m: the mixer's record of config.json."""
    n = h.shape[0]
    H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(n)
    rcfg = m.get("rot") or {}
    if rot:
        freqs, mult = rotary_frequencies(rot, float(rcfg["base"]), rcfg.get("scaling"))
    else:
        freqs, mult = np.zeros(0, dtype=F64), 1.0             # no rotated part at all
    q = (h @ w["q"].T).reshape(n, H, dim + rot)
    q_plain, q_turn = q[..., :dim], rotate_pairs(q[..., dim:], pos, freqs, mult)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    k_turn = rotate_pairs(down[:, rank:], pos, freqs, mult)             # one for all heads
    k_plain = (c @ w["uk"].T).reshape(n, H, dim)
    v = (c @ w["uv"].T).reshape(n, H, vdim)
    scores = (np.einsum("ihd,jhd->hij", q_plain, k_plain) + np.einsum("ihd,jd->hij", q_turn, k_turn)) * m["scale"]
    size = (m.get("mask") or {}).get("size", 0)
    d = pos[:, None] - pos[None, :]
    visible = (d >= 0) & ((d < size) if size else True)
    scores = np.where(visible[None], scores, -np.inf)
    top = scores.max(-1, keepdims=True)
    if sink:
        top = np.maximum(top, w["sink"].reshape(H, 1, 1))
    e = np.exp(scores - top)
    den = e.sum(-1, keepdims=True)
    if sink:
        den = den + np.exp(w["sink"].reshape(H, 1, 1) - top)
    o = np.einsum("hij,jhd->ihd", e / den, v)
    g = sigmoid(h @ w["g"].T)
    if gate == "head":
        o = o * g[:, :, None]
        return o.reshape(n, H * vdim) @ w["o"].T
    return (o.reshape(n, H * vdim) * g) @ w["o"].T


def gla(h, w, m, eps):
    n = h.shape[0]
    H, dim, vdim, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w["q"].T).reshape(n, H, dim) * dim ** -0.5
    k = (h @ w["k"].T).reshape(n, H, dim)
    v = (h @ w["v"].T).reshape(n, H, vdim)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(n, H, dim)
    S = np.zeros((H, dim, vdim), dtype=F64)
    o = np.empty((n, H, vdim), dtype=F64)
    for t in range(n):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, w["norm"], eps)
    gz = h @ w["g"].T
    return (o.reshape(n, H * vdim) * (gz * sigmoid(gz))) @ w["o"].T


def dense_ff(h, w):
    return np.maximum(h @ w["up"].T, 0.0) ** 2 @ w["down"].T


MIXERS = {
    "latent_attention": lambda h, w, m, eps: latent_attention(h, w, m, eps, sink=False, gate="head"),
    "latent_attention_2": lambda h, w, m, eps: latent_attention(h, w, m, eps, sink=True, gate="element"),
    "gla": gla,
}


def hyper_step(xs, hc, norm_w, eps, sublayer):
    """xs [streams, n, width] -> the streams after one sublayer."""
    u = np.einsum("s,snd->nd", hc["in"], xs)
    y = sublayer(layer_norm(u, norm_w, eps))
    return np.einsum("st,snd->tnd", hc["mix"], xs) + hc["out"][:, None, None] * y[None]


def _sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens):
    """(logits [n, vocab], summed streams after every layer run [runs, n, width]); ``weights``: name -> float64."""
    eps = float(config["norm"]["eps"])
    x = weights["embed"][np.asarray(tokens)] * float(config["embedding"]["scale"])
    streams = config.get("streams")
    xs = np.repeat(x[None], streams, axis=0) if streams else None
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] \
        + list(range(loop["stop"], len(config["layers"])))
    after = []
    for i in order:
        layer, p = config["layers"][i], f"l{i}."
        mix_w = _sub(weights, p + "mix.")
        mixer = lambda h: MIXERS[layer["type"]](h, mix_w, layer["mixer"], eps)          # noqa: E731
        subs = [(1, mixer)]
        if layer.get("mlp"):
            assert layer["mlp"]["kind"] == "dense"
            ff_w = _sub(weights, p + "mlp.")
            subs.append((2, lambda h: dense_ff(h, ff_w)))
        for qn, fn in subs:
            if streams:
                xs = hyper_step(xs, _sub(weights, f"{p}hc{qn}."), weights[f"{p}norm{qn}"], eps, fn)
            else:
                x = x + fn(layer_norm(x, weights[f"{p}norm{qn}"], eps))
        after.append(xs.sum(0) if streams else x.copy())
    x = xs.sum(0) if streams else x
    return layer_norm(x, weights["final.norm"], eps) @ weights["embed"].T, np.stack(after)
