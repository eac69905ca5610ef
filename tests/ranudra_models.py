"""Small Ranudra configurations and weights for the tests, and the comparison with the plain model.

The configurations differ from each other in every size and option.  A: three residual streams, a run of layers
repeated three times in the middle, all three mixers, YaRN on one of them, short windows.  B: no streams (the
ordinary residual), no repeated run, a layer without feed-forward, a layer without window, a width that is no
multiple of 8, a cache row whose size is no multiple of 16, one head, no rotated part in one layer.  C: one stream
with connection weights, the whole model repeated twice, cache rows of 64 and 128 elements, twenty heads on one
cache row, a sink on the larger one.

Weights are made here, with activations of order one (so that attention is far from uniform and a window's edge, a
sink or a lost state shows), rounded to bfloat16 and stored as bfloat16.
"""
from __future__ import annotations

import json
import os

import numpy as np

import plain_qwen3
import plain_ranudra


def _latent(heads, dim, rot, vdim, rank, window=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank,
         "scale": scale if scale is not None else (dim + rot) ** -0.5}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
        if scaling:
            m["rot"]["scaling"] = scaling
    if window:
        m["mask"] = {"size": window}
    return m


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CFG_A = {
    "architecture": "Ranudra", "vocab": 97, "width": 48, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5}, "streams": 3,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _layer("latent_attention_2", _latent(3, 16, 8, 24, 24, window=7, base=300.0), 80),
        _layer("gla", {"heads": 2, "dim": 12, "vdim": 20, "tau": 4.0}, 64),
        _layer("latent_attention", _latent(5, 8, 16, 16, 32, window=40, base=5000.0,
                                           scaling={"factor": 4.0, "original": 32, "fast": 8.0, "slow": 2.0}), 72),
        _layer("gla", {"heads": 3, "dim": 8, "vdim": 8, "tau": 9.0}, 56),
    ],
}
CFG_B = {
    "architecture": "Ranudra", "vocab": 131, "width": 52, "embedding": {"scale": 0.7}, "norm": {"eps": 2e-6},
    "layers": [
        _layer("gla", {"heads": 1, "dim": 20, "vdim": 70, "tau": 2.5}, None),
        _layer("latent_attention", _latent(1, 12, 6, 10, 20, window=33, base=50.0), 100),
        _layer("latent_attention_2", _latent(4, 10, 0, 6, 18), 44),
    ],
}
CFG_C = {
    "architecture": "Ranudra", "vocab": 300, "width": 128, "embedding": {"scale": 11.0}, "norm": {"eps": 1e-6}, "streams": 1,
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        _layer("latent_attention", _latent(20, 8, 16, 8, 48, window=96, base=100000.0,
                                           scaling={"factor": 16.0, "original": 64, "fast": 16.0, "slow": 1.0}), 96),
        _layer("latent_attention_2", _latent(2, 32, 32, 40, 96, window=130, base=1000.0), 160),
    ],
}
ALL = {"A": (CFG_A, 3), "B": (CFG_B, 5), "C": (CFG_C, 2)}          # configuration, inner size of the decay projection


def _bf16(a):
    return plain_qwen3.bf16_round(np.asarray(a, dtype=np.float32)).astype(np.float32)


def make_weights(config, seed, decay_rank=4):
    """name -> float32 array (every value a bfloat16 number)."""
    rng = np.random.default_rng(seed)
    D, S = config["width"], config.get("streams")
    W = {}

    def mat(name, n_out, n_in, gain=1.0):
        W[name] = _bf16(rng.standard_normal((n_out, n_in)) * gain / np.sqrt(n_in))

    def vec(name, n, lo, hi):
        W[name] = _bf16(rng.uniform(lo, hi, size=n))

    W["embed"] = _bf16(rng.standard_normal((config["vocab"], D)) * 0.5)
    vec("final.norm", D, 0.7, 1.3)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        subs = [1] + ([2] if layer["mlp"] else [])
        for q in subs:
            vec(f"{p}norm{q}", D, 0.7, 1.3)
            if S:
                vec(f"{p}hc{q}.in", S, 0.2, 0.8)
                vec(f"{p}hc{q}.out", S, 0.3, 1.2)
                W[f"{p}hc{q}.mix"] = _bf16(0.8 * np.eye(S) + rng.uniform(-0.2, 0.2, size=(S, S)))
        H = m["heads"]
        if layer["type"] == "gla":
            mat(p + "mix.q", H * m["dim"], D, 2.0)
            mat(p + "mix.k", H * m["dim"], D)
            mat(p + "mix.v", H * m["vdim"], D)
            mat(p + "mix.g", H * m["vdim"], D)
            mat(p + "mix.o", D, H * m["vdim"])
            vec(p + "mix.norm", m["vdim"], 0.7, 1.3)
            mat(p + "mix.a1", decay_rank, D)
            mat(p + "mix.a2", H * m["dim"], decay_rank, 2.0)
            vec(p + "mix.a2.b", H * m["dim"], 0.0, 4.0)
        else:
            mat(p + "mix.q", H * (m["dim"] + m["rot_dim"]), D, 3.0)
            mat(p + "mix.dkv", m["kv_rank"] + m["rot_dim"], D, 2.0)
            vec(p + "mix.dkv.norm", m["kv_rank"], 0.7, 1.3)
            mat(p + "mix.uk", H * m["dim"], m["kv_rank"], 2.0)
            mat(p + "mix.uv", H * m["vdim"], m["kv_rank"])
            mat(p + "mix.o", D, H * m["vdim"])
            if layer["type"] == "latent_attention_2":
                vec(p + "mix.sink", H, -1.0, 3.0)
                mat(p + "mix.g", H * m["vdim"], D)
            else:
                mat(p + "mix.g", H, D)
        if layer["mlp"]:
            mat(p + "mlp.up", layer["mlp"]["ff"], D)
            mat(p + "mlp.down", D, layer["mlp"]["ff"])
    return W


def write_model(folder, config, weights):
    """config.json and model.safetensors (bfloat16) in ``folder``."""
    import torch
    from rust_inference_b200.weights.safetensors_io import save_safetensors
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    save_safetensors(os.path.join(folder, "model.safetensors"),
                     {k: torch.from_numpy(np.ascontiguousarray(v)).to(torch.bfloat16) for k, v in weights.items()})
    return folder


def make_model_dir(base, name, seed=1):
    config, rank = ALL[name]
    weights = make_weights(config, seed, rank)
    return write_model(os.path.join(str(base), f"ranudra_{name}"), config, weights), config, weights


def plain_logits(config, weights, requests):
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    return {rid: plain_ranudra.forward(config, W, toks)[0] for rid, toks in requests.items()}


def row_error(got, want):
    """The difference of two rows of logits with the mean taken off, relative to the spread of the wanted row."""
    d = got.astype(np.float64) - want
    d = d - d.mean()
    w = want - want.mean()
    return float(np.sqrt((d * d).mean()) / max(np.sqrt((w * w).mean()), 1e-30))


# float32: rounding alone (sums of a few hundred float32 terms over a dozen sublayers).  bfloat16: activations are
# rounded to 8 bits between the parts of every sublayer, and these weights make attention sharp and the layers deep
# (a run of layers three times over), so single rows are a few tenths off where a rounding tips a sharp softmax; the
# mean over all rows is held much tighter (a wrong mechanism moves every row by about one).  The same code runs both
# dtypes apart from the kernels, and what the bfloat16 kernels compute is held to 1.2 % by the kernel tests.
BOUND = {"float32": (2e-5, 1e-5), "bfloat16": (6e-1, 5e-2)}


def assert_rows_close(rows, want_by_request, dtype, what=""):
    worst, total = 0.0, 0.0
    for (rid, p), got in sorted(rows.items()):
        err = row_error(got, want_by_request[rid][p])
        worst, total = max(worst, err), total + err
        assert err <= BOUND[dtype][0], f"{what}: request {rid} position {p}: error {err:.3e} exceeds {BOUND[dtype][0]:.1e}"
    mean = total / max(len(rows), 1)
    assert mean <= BOUND[dtype][1], f"{what}: mean error {mean:.3e} exceeds {BOUND[dtype][1]:.1e}"
    return round(worst, 7), round(mean, 7)
