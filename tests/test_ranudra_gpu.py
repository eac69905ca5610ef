"""Ranudra on the GPU: each kernel against the plain formulas, then whole models through trace replay in three
cuttings (whole prompts; prompts then single tokens; batches of unequal requests that follow each other on the same
slots and pages), in float32 and bfloat16, against the plain model of tests/plain_ranudra.py."""
import numpy as np
import pytest
import torch

import helpers as H
import plain_ranudra as P
import ranudra_models as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _t(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV, dtype)


def _close(got, want, dtype, what):
    got, want = got.double().cpu().numpy(), np.asarray(want, dtype=np.float64)
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert err <= tol, f"{what}: error {err:.3e} of the largest value exceeds {tol:.1e}"


# ---- the norm over residual streams ------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S, dim, n", [(1, 52, 5), (3, 48, 70), (4, 3001, 9), (16, 8, 3)])
def test_stream_norm(S, dim, n, dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(S * dim)
    xs = rng.standard_normal((n, S, dim)) * 3 + 1.5
    y = _t(rng.standard_normal((n, dim)), dtype)
    mix, out, read = rng.uniform(-1, 1, (S, S)), rng.uniform(0.3, 1.2, S), rng.uniform(0.2, 0.8, S)
    gain, eps = rng.uniform(0.7, 1.3, dim), 1e-5
    yd = y.double().cpu().numpy()
    new = np.einsum("st,nsd->ntd", mix, xs.astype(np.float32).astype(np.float64)) + out[None, :, None] * yd[:, None, :]
    # with a pending output: the streams are updated in place and the weighted sum is normed
    resid = _t(xs)
    got = ops.stream_norm(resid, _t(gain), eps, dtype, "layernorm", delta=y, mix=_t(mix), out_w=_t(out), read=_t(read))
    _close(resid, new, torch.float32, "updated streams")
    _close(got, P.layer_norm(np.einsum("s,nsd->nd", read, new), gain, eps), dtype, "layer norm of the weighted sum")
    # without one, and RMS norm; absent weights mean identity, ones and the plain sum
    resid = _t(xs)
    got = ops.stream_norm(resid, _t(gain), eps, dtype, "rmsnorm")
    _close(got, P.rms_norm(xs.astype(np.float32).astype(np.float64).sum(1), gain, eps), dtype, "rms norm of the sum")
    assert torch.equal(resid, _t(xs))
    # a few rows only: nothing is written back
    rows = torch.tensor([n - 1, 0, n // 2], dtype=torch.int32, device=DEV)
    got = ops.stream_norm(resid, _t(gain), eps, dtype, "layernorm", delta=y, mix=_t(mix), out_w=_t(out), rows=rows)
    _close(got, P.layer_norm(new.sum(1), gain, eps)[rows.cpu().numpy()], dtype, "rows")
    assert torch.equal(resid, _t(xs))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_activation_and_gates(dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(1)
    table = _t(rng.standard_normal((37, 20)), dtype)
    ids = torch.tensor([3, 36, 0, 3], dtype=torch.int32, device=DEV)
    e = ops.embed(ids, table, scale=2.5, copies=3)
    assert e.shape == (4, 3, 20) and torch.equal(e[:, 0], e[:, 2])
    _close(e[:, 1], table.double().cpu().numpy()[[3, 36, 0, 3]] * 2.5, torch.float32, "scaled embedding")
    for n in (7, 1024):
        x = _t(rng.standard_normal((3, n)) * 2, dtype)
        xd = x.double().cpu().numpy()
        _close(ops.activation(x, "relu2"), np.maximum(xd, 0) ** 2, dtype, "relu2")
        _close(ops.activation(x, "gelu_tanh"), 0.5 * xd * (1 + np.tanh(np.sqrt(2 / np.pi) * (xd + 0.044715 * xd ** 3))), dtype, "gelu")
    # the activation in the product's epilogue (a handful of bfloat16 tokens) and as a kernel of its own (more)
    w = _t(rng.standard_normal((40, 64)) * 0.3, dtype)
    for m in (3, 12, 70):
        x = _t(rng.standard_normal((m, 64)), dtype)
        z = x.double().cpu().numpy() @ w.double().cpu().numpy().T
        _close(ops.linear_act(x, w, "relu2"), np.maximum(z, 0) ** 2, dtype, f"relu2 after a product of {m} tokens")
        _close(ops.linear_act(x, w, "gelu_tanh"), 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3))), dtype,
               f"gelu after a product of {m} tokens")
    wide = _t(rng.standard_normal((6, 50)) * 2, dtype)                 # gates are columns of a wider matrix
    wd = wide.double().cpu().numpy()
    for cols, per_head in ((slice(5, 9), True), (slice(10, 34), False)):
        x = _t(rng.standard_normal((6, 4, 6)), dtype)
        xd = x.double().cpu().numpy()
        g = P.sigmoid(wd[:, cols])
        want = xd * (g[:, :, None] if per_head else g.reshape(6, 4, 6))
        _close(ops.gate_heads(x, wide[:, cols], "sigmoid"), want, dtype, "gates")


def test_linear_heads_float32_is_exact_in_order():
    from rust_inference_b200 import ops
    rng = np.random.default_rng(2)
    wide = _t(rng.standard_normal((70, 5 * 23 + 4)))
    x = wide[:, 4:].view(70, 5, 23)[:, :, :17]                         # a slice of a projection: strided rows
    w = _t(rng.standard_normal((5, 9, 17)))
    got = ops.linear_heads(x, w)
    _close(got, np.einsum("thk,hnk->thn", x.double().cpu().numpy(), w.double().cpu().numpy()), torch.float32, "linear_heads")
    assert torch.equal(got[3:4], ops.linear_heads(x[3:4], w))           # a token's result does not depend on the batch
    xb, wb = x.to(torch.bfloat16), w.to(torch.bfloat16)
    _close(ops.linear_heads(xb, wb), np.einsum("thk,hnk->thn", xb.double().cpu().numpy(), wb.double().cpu().numpy()),
           torch.bfloat16, "linear_heads bf16")


# ---- gated linear attention -----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, dim, vdim", [(2, 12, 20), (1, 33, 70), (3, 64, 130), (2, 128, 33), (1, 136, 40)])
def test_gla_recurrence_and_state(H, dim, vdim, dtype):
    """Two sequences of unequal length in one call; then the same tokens in two calls (the state carries over, bit
    for bit in float32); slots used again start from zero."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(H * dim)
    lens, tau, eps = [37, 5], 3.0, 1e-5
    T = sum(lens)
    ncol = 2 * H * dim + 2 * H * vdim + 3
    proj = _t(rng.standard_normal((T, ncol)), dtype)
    z = _t(rng.standard_normal((T, H * dim)) * 2, dtype)
    bias, gain = rng.uniform(0, 3, H * dim), rng.uniform(0.7, 1.3, vdim)
    q_col, k_col, v_col, g_col = 3, 3 + H * dim, 3 + 2 * H * dim, 3 + 2 * H * dim + H * vdim
    pd, zd = proj.double().cpu().numpy(), z.double().cpu().numpy()
    want_o = np.zeros((T, H, vdim))
    t0 = 0
    for n in lens:
        a = (P.sigmoid(zd[t0:t0 + n] + bias) ** (1 / tau)).reshape(n, H, dim)
        q = pd[t0:t0 + n, q_col:q_col + H * dim].reshape(n, H, dim) * dim ** -0.5
        k = pd[t0:t0 + n, k_col:k_col + H * dim].reshape(n, H, dim)
        v = pd[t0:t0 + n, v_col:v_col + H * vdim].reshape(n, H, vdim)
        S = np.zeros((H, dim, vdim))
        for t in range(n):
            S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
            want_o[t0 + t] = np.einsum("hdv,hd->hv", S, q[t])
        t0 += n
    slots = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
    start = torch.tensor([0, lens[0], T], dtype=torch.int32, device=DEV)
    state = torch.zeros((3, H, dim, vdim), device=DEV)
    o = ops.gla_recurrent(proj, q_col, k_col, v_col, z, _t(bias), tau, dim ** -0.5, state, slots, start, H, dim, vdim)
    _close(o, want_o, torch.float32 if dtype == torch.float32 else dtype, "recurrence")
    assert float(state[1].abs().max()) == 0.0 and float(state[2].abs().max()) > 0.0
    # the same in pieces: 30 + 7 tokens of the first sequence, 2 + 3 of the second
    state2 = torch.zeros_like(state)
    cut = [30, 2]
    first = torch.cat([proj[:30], proj[37:39]]).contiguous(), torch.cat([z[:30], z[37:39]]).contiguous()
    rest = torch.cat([proj[30:37], proj[39:]]).contiguous(), torch.cat([z[30:37], z[39:]]).contiguous()
    o1 = ops.gla_recurrent(first[0], q_col, k_col, v_col, first[1], _t(bias), tau, dim ** -0.5, state2, slots,
                           torch.tensor([0, 30, 32], dtype=torch.int32, device=DEV), H, dim, vdim)
    o2 = ops.gla_recurrent(rest[0], q_col, k_col, v_col, rest[1], _t(bias), tau, dim ** -0.5, state2, slots,
                           torch.tensor([0, 7, 10], dtype=torch.int32, device=DEV), H, dim, vdim)
    assert torch.equal(torch.cat([o1[:30], o2[:7], o1[30:], o2[7:]]), o) and torch.equal(state2, state)
    # ... and token by token with the kernel's variant for steps of single tokens
    state3 = torch.zeros_like(state)
    one = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    outs = [ops.gla_recurrent(proj[t:t + 1].contiguous(), q_col, k_col, v_col, z[t:t + 1].contiguous(), _t(bias), tau,
                              dim ** -0.5, state3, slots[:1], one, H, dim, vdim, single=True) for t in range(lens[0])]
    assert torch.equal(torch.cat(outs), o[:lens[0]]) and torch.equal(state3[2], state[2])
    # norm over the value size, one gain for all heads, silu gate from columns of the projection
    y = ops.head_norm_gate(o, _t(gain), eps, proj[:, g_col:g_col + H * vdim], dtype, "silu")
    od = o.double().cpu().numpy()
    gz = pd[:, g_col:g_col + H * vdim]
    want = (P.rms_norm(od, gain, eps).reshape(T, H * vdim)) * gz * P.sigmoid(gz)
    _close(y, want, dtype, "norm and gate")


# ---- latent attention: the cache row, windows' edges, far keys, the sink ---------------------------------------------
def _latent_case(rng, n, H, rank, rot, window, hot_distance, dtype):
    """A sequence of n cached rows and queries at every position whose score against the row ``hot_distance`` back
    stands out (when that row is visible, it takes nearly all the weight)."""
    Dk = rank + rot
    rows = rng.standard_normal((n, Dk)) * 0.3
    q = rng.standard_normal((n, H, Dk)) * 0.3
    for i in range(hot_distance, n):
        q[i] += 4.0 * rows[i - hot_distance] / np.linalg.norm(rows[i - hot_distance]) ** 2 * 6.0
    return _t(rows, dtype), _t(q, dtype)


def _plain_attention(rows, q, window, scale, rank, sink):
    rows, q = rows.double().cpu().numpy(), q.double().cpu().numpy()
    n, H, _ = q.shape
    out = np.zeros((n, H, rank))
    for i in range(n):
        lo = max(0, i - window + 1) if window else 0
        s = np.einsum("hd,jd->hj", q[i], rows[lo:i + 1]) * scale
        top = s.max(-1, keepdims=True)
        if sink is not None:
            top = np.maximum(top, sink[:, None])
        e = np.exp(s - top)
        den = e.sum(-1, keepdims=True) + (np.exp(sink[:, None] - top) if sink is not None else 0.0)
        out[i] = (e / den) @ rows[lo:i + 1, :rank]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank, rot, H", [(24, 8, 3), (96, 32, 20), (20, 6, 2)])
@pytest.mark.parametrize("window, hot", [(40, 39), (40, 40), (0, 300), (33, 32), (7, 7), (64, 1)])
def test_attention_over_a_latent_pool(tmp_path, rank, rot, H, window, hot, dtype):
    """The attention kernels with one pool as keys and values, a window whose last visible key (or the first
    invisible one) carries the weight, a far key among hundreds, with and without a sink: a whole prompt, and the
    same queries one at a time over the growing cache."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(window * 1000 + hot + rank)
    n, P_ = 333, 32
    Dk, scale = rank + rot, 0.3
    rows, q = _latent_case(rng, n, H, rank, rot, window, hot, dtype)
    pages = -(-n // P_)
    order = rng.permutation(pages + 3)[:pages]                       # pages in no particular order
    pool = torch.zeros((pages + 3, 1, P_, Dk), dtype=dtype, device=DEV)
    for p in range(pages):
        chunk = rows[p * P_:(p + 1) * P_]
        pool[order[p], 0, :chunk.shape[0]] = chunk
    table = torch.full((2, pages), -1, dtype=torch.int32, device=DEV)
    table[1] = torch.from_numpy(order.astype(np.int32)).to(DEV)
    slot = torch.tensor([1], dtype=torch.int32, device=DEV)
    for sink in (None, rng.uniform(-1, 3, H)):
        want = _plain_attention(rows, q, window, scale, rank, sink)
        sk = None if sink is None else _t(sink)
        start = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        length = torch.tensor([n], dtype=torch.int32, device=DEV)
        fast = ops.fast_attention_supported(dtype, Dk, P_)
        if fast:
            got = ops.attention_prefill(q, pool, pool, table, slot, start, length, n, scale, window, sink=sk)
        else:
            got = ops.attention(q, pool, pool, table, slot, start, length, n, scale, window, sink=sk)
        _close(got[:, :, :rank], want, dtype, f"prompt, sink {sink is not None}")
        for i in list(range(0, n, 37)) + [hot, min(n - 1, hot + 1), n - 1]:
            length = torch.tensor([i + 1], dtype=torch.int32, device=DEV)
            qi = q[i:i + 1].contiguous()
            if fast:
                got = ops.attention_decode(qi, pool, pool, table, slot, length, scale, window, 1024, sink=sk)
            else:
                got = ops.attention(qi, pool, pool, table, slot, torch.tensor([0, 1], dtype=torch.int32, device=DEV), length,
                                    1, scale, window, sink=sk)
            _close(got[0, :, :rank], want[i], dtype, f"single token at {i}, sink {sink is not None}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prep_writes_rows_and_queries(dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(9)
    H, dim, rot, rank, eps = 3, 10, 6, 14, 1e-5
    T, P_ = 5, 32
    ncol = H * (dim + rot) + rank + rot + 2
    proj = _t(rng.standard_normal((T, ncol)), dtype)
    qa = _t(rng.standard_normal((T, H, rank)), dtype)
    gain = rng.uniform(0.7, 1.3, rank)
    pos = np.array([31, 32, 33, 0, 1])                                  # two sequences, one across a page's border
    f, mult = P.rotary_frequencies(rot, 77.0, {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0})
    ang = np.arange(64)[:, None] * f[None, :]
    table = _t(np.stack([np.cos(ang) * mult, np.sin(ang) * mult], -1))
    pool = torch.zeros((4, 1, P_, rank + rot), dtype=dtype, device=DEV)
    pages = torch.tensor([[2, 0], [3, -1]], dtype=torch.int32, device=DEV)
    tok_seq = torch.tensor([0, 0, 0, 1, 1], dtype=torch.int32, device=DEV)
    qf = ops.latent_prep(proj, 0, H * (dim + rot), qa, H, dim, rot, rank, _t(gain), eps, table, pool, pages, tok_seq,
                         _t(pos, torch.int32), torch.tensor([0, 1], dtype=torch.int32, device=DEV))
    pd = proj.double().cpu().numpy()
    down = pd[:, H * (dim + rot):H * (dim + rot) + rank + rot]
    want_rows = np.concatenate([P.rms_norm(down[:, :rank], gain, eps), P.rotate_pairs(down[:, rank:], pos, f, mult)], -1)
    got_rows = torch.stack([pool[2, 0, 31], pool[0, 0, 0], pool[0, 0, 1], pool[3, 0, 0], pool[3, 0, 1]])
    _close(got_rows, want_rows, dtype, "cache rows")
    q = pd[:, :H * (dim + rot)].reshape(T, H, dim + rot)
    want_q = np.concatenate([qa.double().cpu().numpy(), P.rotate_pairs(q[..., dim:], pos, f, mult)], -1)
    _close(qf, want_q, dtype, "query rows")


# ---- whole models ------------------------------------------------------------------------------------------------
LENGTHS = {"A": [5, 1, 31, 32, 33, 64, 65, 150, 2, 97], "B": [70, 1, 33, 140, 65, 8], "C": [200, 3, 129, 260, 64]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("ranudra")
    return {name: R.make_model_dir(base, name, seed=11 + i) for i, name in enumerate(R.ALL)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_three_ways(tmp_path, models, name, dtype):
    d, config, weights = models[name]
    reqs = H.random_requests(np.random.default_rng(7), config["vocab"], LENGTHS[name])
    want = R.plain_logits(config, weights, reqs)
    worst, by_cutting = {}, {}
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=60)),
                         ("batches", H.trace_batches(reqs, 4, [8, 3, 12, 0, 33]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, dtype, steps, out, device=DEV)
        rows = H.collect(steps, out, config["vocab"])
        assert len(rows) == sum(len(t) for t in reqs.values())
        worst[label] = R.assert_rows_close(rows, want, dtype, f"{name} {dtype} {label}")
        by_cutting[label] = rows
    if dtype == "float32":
        H.assert_rows_identical(by_cutting, f"{name} float32")
    print(f"{name} {dtype}: worst error = {worst}")


@pytest.mark.parametrize("kind", ["latent_attention", "latent_attention_2", "gla"])
def test_each_mixer_alone(tmp_path, kind):
    """A model of one layer of one mixer and no feed-forward: prompts against single tokens (long decoding over
    several pages and windows), float32."""
    layer = next(l for l in R.CFG_A["layers"] if l["type"] == kind)
    config = dict(R.CFG_A, layers=[dict(layer, mlp=None)], streams=2)
    config.pop("loop")
    weights = R.make_weights(config, 31, decay_rank=6)
    d = R.write_model(str(tmp_path / "m"), config, weights)
    reqs = H.random_requests(np.random.default_rng(3), config["vocab"], [180, 41])
    want = R.plain_logits(config, weights, reqs)
    rows = {}
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=170))):
        out = str(tmp_path / label)
        H.replay_inprocess(d, "float32", steps, out, device=DEV)
        rows[label] = H.collect(steps, out, config["vocab"])
        R.assert_rows_close(rows[label], want, "float32", f"{kind} {label}")
    H.assert_rows_identical(rows, kind)


def test_greedy_generation(models):
    """Greedy tokens through ``LLM.generate`` (its scheduler, CUDA graphs for the single-token steps, more requests
    than slots so that slots, pages and states are used again) against the plain model."""
    import rust_inference_b200 as ri
    d, config, weights = models["A"]
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    rng = np.random.default_rng(5)
    prompts = [[int(t) for t in rng.integers(0, config["vocab"], n)] for n in (9, 40, 1, 33, 17)]
    llm = ri.LLM(d, dtype="float32", max_pages=16, pages_per_seq=4, max_seqs=2)
    got = llm.generate(prompts, max_new_tokens=12)
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(12):
            logits = P.forward(config, W, seq)[0][-1]
            top = np.sort(logits)[-2:]
            if top[1] - top[0] < 1e-3 * np.abs(logits).max():
                break                                                  # a near tie: rounding may pick either
            seq.append(int(np.argmax(logits)))
        n = len(seq) - len(p)
        assert g[:n] == seq[len(p):]
    assert llm.engine.graph_replays > 0
