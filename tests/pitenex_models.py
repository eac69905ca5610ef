"""Small Pitenex configurations and weights for the tests, and the comparison with the plain model.

The configurations differ from each other in every size and option.  A: attention with values larger than keys,
smaller than keys and equal to them; chunks of 7, 33 (across a page border) and 64 positions; rotation of a part of a
head, of a whole head, of nothing; convolutions of 4, 2 and 3 taps; fewer query/key heads than value heads on the
right; a routed feed-forward with an identity expert and a shared one, a dense one, a layer without feed-forward.
B: a width that is no multiple of 8; heads of 64 on the left (the decode kernel for that size); a delta rule with 136
key channels and a convolution of one tap; one expert per token, no identity expert, no shared one; a layer whose
attention has no mask at all; low-rank projections of 5 and 3.  C: wider, for bfloat16.  D: a width that is no multiple
of 4; head sizes that the kernels pad to 112 and 48; chunks of one position (a query sees itself and the sink); five taps;
forty experts without a shared one; 130 value columns on 72 key channels.

Weights are made here, with activations of order one (so that attention is far from uniform and a chunk's edge, a
sink or a lost state shows), rounded to bfloat16 and stored as bfloat16.
"""
from __future__ import annotations

import os

import numpy as np

import plain_pitenex
from ranudra_models import _bf16, row_error, write_model


def _left(heads, kv, dim, vdim, size=None, rot=None, base=1000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    if size:
        m["mask"] = {"size": size}
    return m


def _right(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(experts, identity, top, ff, limit, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def _layer(left, right, ls, rs, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


CFG_A = {
    "architecture": "Pitenex", "vocab": 97, "width": 48, "embedding": {"bigram": {"buckets": 53, "mul_prev": 31, "mul_cur": 5}},
    "norm": {"eps": 1e-5}, "residual_mult": 0.6, "logit_scale": 1.5,
    "layers": [
        _layer(_left(4, 2, 16, 24, size=7, rot=8, base=100.0, scale=0.3), _right(4, 2, 12, 20, 4), 0.9, 1.2,
               _moe(5, 1, 2, 24, 0.8, shared=(40, 1.2))),
        _layer(_left(2, 2, 24, 16, size=33, rot=24, base=3000.0), _right(2, 1, 40, 8, 2), 1.3, 0.5, {"kind": "dense", "ff": 72}),
        _layer(_left(3, 1, 32, 32, size=64), _right(1, 1, 8, 40, 3), 0.4, 1.0, None),
    ],
}
CFG_B = {
    "architecture": "Pitenex", "vocab": 131, "width": 52, "embedding": {"bigram": {"buckets": 17, "mul_prev": 3, "mul_cur": 11}},
    "norm": {"eps": 2e-6}, "residual_mult": 1.0, "logit_scale": 0.5,
    "layers": [
        _layer(_left(1, 1, 64, 64, size=40, rot=32, base=5000.0), _right(2, 2, 136, 16, 1), 1.0, 1.0, _moe(3, 0, 1, 20, 2.0)),
        _layer(_left(6, 3, 8, 12, rot=8, base=50.0), _right(4, 1, 16, 16, 3), 0.7, 0.9, _moe(9, 3, 4, 12, 0.6, shared=(28, 3.0))),
    ],
}
CFG_C = {
    "architecture": "Pitenex", "vocab": 300, "width": 128, "embedding": {"bigram": {"buckets": 211, "mul_prev": 13, "mul_cur": 1}},
    "norm": {"eps": 1e-6}, "residual_mult": 0.5, "logit_scale": 3.0,
    "layers": [
        _layer(_left(4, 2, 32, 48, size=48, rot=16, base=20000.0), _right(4, 2, 64, 32, 3), 0.75, 1.25, {"kind": "dense", "ff": 160}),
        _layer(_left(8, 1, 128, 128, size=100, rot=128, base=500.0), _right(2, 2, 24, 96, 4), 1.0, 0.6,
               _moe(6, 2, 3, 64, 1.0, shared=(96, 1.5))),
    ],
}
CFG_D = {
    "architecture": "Pitenex", "vocab": 61, "width": 50, "embedding": {"bigram": {"buckets": 7, "mul_prev": 1, "mul_cur": 1}},
    "norm": {"eps": 1e-4}, "residual_mult": 0.9, "logit_scale": 1.0,
    "layers": [
        _layer(_left(2, 1, 96, 112, size=20, rot=10, base=7.0), _right(3, 3, 20, 12, 5), 1.0, 0.8, _moe(40, 0, 3, 8, 1.1)),
        _layer(_left(6, 2, 40, 24, size=1), _right(2, 1, 72, 130, 2), 0.5, 1.5, {"kind": "dense", "ff": 30}),
    ],
}
ALL = {"A": (CFG_A, (6, 10)), "B": (CFG_B, (5, 3)), "C": (CFG_C, (16, 8)), "D": (CFG_D, (2, 4))}


def make_weights(config, seed, ranks=(6, 10)):
    """name -> float32 array (every value a bfloat16 number).  ``ranks``: the inner sizes of the delta rule's two
    low-rank projections (decay, gate), which only the tensors' shapes give."""
    rng = np.random.default_rng(seed)
    D = config["width"]
    W = {}

    def mat(name, n_out, n_in, gain=1.0):
        W[name] = _bf16(rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in))

    def vec(name, n, lo, hi):
        W[name] = _bf16(rng.uniform(lo, hi, size=n))

    W["embed"] = _bf16(rng.standard_normal((config["vocab"], D)) * 0.5)
    W["bigram"] = _bf16(rng.standard_normal((config["embedding"]["bigram"]["buckets"] + 1, D)) * 0.5)
    vec("final.norm", D, 0.7, 1.3)
    vec("final.norm.b", D, -0.2, 0.2)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        vec(p + "norm1", D, 0.7, 1.3)
        vec(p + "norm1.b", D, -0.3, 0.3)
        left, right = layer["mixer"]["left"], layer["mixer"]["right"]
        mat(p + "mix.left.q", left["heads"] * left["dim"], D, 3.0)
        mat(p + "mix.left.k", left["kv_heads"] * left["dim"], D, 3.0)
        mat(p + "mix.left.v", left["kv_heads"] * left["vdim"], D)
        vec(p + "mix.left.sink", left["heads"], -1.0, 3.0)
        mat(p + "mix.left.o", D, left["heads"] * left["vdim"])
        H, G, dim, vdim, taps = right["heads"], right["kv_heads"], right["dim"], right["vdim"], right["conv"]
        for n, rows in (("q", G * dim), ("k", G * dim), ("v", H * vdim)):
            mat(p + f"mix.right.{n}", rows, D, 2.0)
            W[p + f"mix.right.{n}.conv"] = _bf16(rng.uniform(-0.8, 0.8, size=(rows, taps)))
        mat(p + "mix.right.b", H, D, 2.0)
        vec(p + "mix.right.A_log", H, -2.0, 0.5)
        vec(p + "mix.right.norm", vdim, 0.7, 1.3)
        mat(p + "mix.right.a1", ranks[0], D)
        mat(p + "mix.right.a2", H * dim, ranks[0], 2.0)
        vec(p + "mix.right.dt_bias", H * dim, -3.0, 1.0)
        mat(p + "mix.right.g1", ranks[1], D)
        mat(p + "mix.right.g2", H * vdim, ranks[1], 2.0)
        mat(p + "mix.right.o", D, H * vdim)
        mlp = layer["mlp"]
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            mat(p + "mlp.gate", mlp["ff"], D, 2.0)
            mat(p + "mlp.up", mlp["ff"], D)
            mat(p + "mlp.down", D, mlp["ff"])
            continue
        r = mlp["router"]
        mat(p + "mlp.router", r["experts"] + r["identity"], D, 3.0)
        vec(p + "mlp.correction", r["experts"] + r["identity"], -0.15, 0.15)
        groups = [(f"e{e}.", mlp["expert"]["ff"]) for e in range(r["experts"])]
        if mlp.get("shared"):
            groups.append(("shared.", mlp["shared"]["ff"]))
        for pre, ff in groups:
            mat(p + "mlp." + pre + "gate", ff, D, 2.0)
            mat(p + "mlp." + pre + "up", ff, D, 2.0)
            mat(p + "mlp." + pre + "down", D, ff)
    return W


def make_model_dir(base, name, seed=1):
    config, ranks = ALL[name]
    weights = make_weights(config, seed, ranks)
    return write_model(os.path.join(str(base), f"pitenex_{name}"), config, weights), config, weights


def plain_logits(config, weights, requests):
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    return {rid: plain_pitenex.forward(config, W, toks)[0] for rid, toks in requests.items()}


# float32: rounding alone.  bfloat16: activations are rounded to 8 bits between the parts of every sublayer; single rows
# are a few tenths off where a rounding tips a sharp softmax or a router's choice, the mean over all rows is held much
# tighter (a wrong mechanism moves every row by about one).
BOUND = {"float32": (3e-5, 1e-5), "bfloat16": (6e-1, 5e-2)}


def assert_rows_close(rows, want_by_request, dtype, what=""):
    worst, total = 0.0, 0.0
    for (rid, p), got in sorted(rows.items()):
        err = row_error(got, want_by_request[rid][p])
        worst, total = max(worst, err), total + err
        assert err <= BOUND[dtype][0], f"{what}: request {rid} position {p}: error {err:.3e} exceeds {BOUND[dtype][0]:.1e}"
    mean = total / max(len(rows), 1)
    assert mean <= BOUND[dtype][1], f"{what}: mean error {mean:.3e} exceeds {BOUND[dtype][1]:.1e}"
    return round(worst, 7), round(mean, 7)
