"""Pitenex on the GPU: each kernel against the plain formulas of tests/plain_pitenex.py, then whole models through trace
replay in several cuttings (whole prompts; prompts then single tokens; prompts in portions down to two tokens; batches of
unequal requests that follow each other on the same slots and pages), in float32 and bfloat16, against the plain model."""
import numpy as np
import pytest
import torch

import helpers as H
import pitenex_models as R
import plain_pitenex as P

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _t(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV, dtype)


def _i(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


def _np(t):
    return t.double().cpu().numpy()


def _close(got, want, dtype, what, tol32=2e-5, tol16=1.2e-2):
    got, want = _np(got), np.asarray(want, dtype=np.float64)
    tol = tol32 if dtype == torch.float32 else tol16
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    assert err <= tol, f"{what}: error {err:.3e} of the largest value exceeds {tol:.1e}"


def _tables(lengths):
    """tok_seq, seq_start for sequences that bring ``lengths`` tokens."""
    tok_seq = [b for b, n in enumerate(lengths) for _ in range(n)]
    return _i(tok_seq), _i(np.concatenate([[0], np.cumsum(lengths)]))


# ---- embedding with the hashed pair table ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding_in_portions_and_on_used_slots(dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(0)
    vocab, dim, buckets, mp, mc = 41, 20, 13, 31, 5
    table, pairs = _t(rng.standard_normal((vocab, dim)), dtype), _t(rng.standard_normal((buckets + 1, dim)), dtype)
    seqs = [[int(t) for t in rng.integers(0, vocab, n)] for n in (9, 1, 4)]
    want = [_np(table)[s] + _np(pairs)[P.bigram_rows(s, buckets, mp, mc)] for s in seqs]
    last = torch.full((5,), 7, dtype=torch.int32, device=DEV)            # slots hold an earlier sequence's token
    slots = [3, 0, 4]
    done = [0, 0, 0]
    got = [[], [], []]
    for cut in ([2, 1, 1], [1, 0, 1], [5, 0, 2], [1, 0, 0]):              # portions of 2, 1, 5 and 1 tokens; a sequence may pause
        live = [b for b in range(3) if cut[b]]
        ids = [t for b in live for t in seqs[b][done[b]:done[b] + cut[b]]]
        pos = [p for b in live for p in range(done[b], done[b] + cut[b])]
        tok_seq, seq_start = _tables([cut[b] for b in live])
        out = ops.embed_pair_hash(_i(ids), table, pairs, last, tok_seq, _i(pos), _i([slots[b] for b in live]), seq_start, mp, mc,
                                  single=all(cut[b] == 1 for b in live))
        at = 0
        for b in live:
            got[b].append(out[at:at + cut[b]])
            at += cut[b]
            done[b] += cut[b]
    for b in range(3):
        _close(torch.cat(got[b]), want[b], torch.float32, f"sequence {b}", tol32=1e-6)
    assert last[3].item() == seqs[0][-1] and last[0].item() == seqs[1][-1] and last[1].item() == 7


# ---- layer norm with a bias and several pending outputs ---------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, n", [(52, 5), (48, 70), (3001, 9)])
def test_layer_norm_with_bias_and_three_pending_outputs(dim, n, dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((n, 1, dim)) * 3 + 1.5
    ys = [_t(rng.standard_normal((n, dim)), dtype) for _ in range(3)]
    ws = [0.9 * 0.6, 1.2 * 0.6, 0.6]
    gain, bias, eps = rng.uniform(0.7, 1.3, dim), rng.uniform(-0.5, 0.5, dim), 1e-5
    new = x[:, 0].astype(np.float32).astype(np.float64) + sum(w * _np(y) for w, y in zip(ws, ys))
    resid = _t(x)
    wt = [torch.full((1,), w, dtype=torch.float32, device=DEV) for w in ws]
    got = ops.stream_norm(resid, _t(gain), eps, dtype, "layernorm", delta=ys[0], out_w=wt[0], bias=_t(bias),
                          more=((ys[1], wt[1]), (ys[2], wt[2])))
    _close(resid[:, 0], new, torch.float32, "residual after three outputs")
    _close(got, P.layer_norm(new, gain, bias, eps), dtype, "layer norm with bias")
    rows = _i([n - 1, 0])
    resid = _t(x)
    got = ops.stream_norm(resid, _t(gain), eps, dtype, "layernorm", delta=ys[0], out_w=wt[0], bias=_t(bias), more=((ys[1], wt[1]),),
                          rows=rows)
    two = x[:, 0].astype(np.float32).astype(np.float64) + ws[0] * _np(ys[0]) + ws[1] * _np(ys[1])
    _close(got, P.layer_norm(two, gain, bias, eps)[[n - 1, 0]], dtype, "rows")
    assert torch.equal(resid, _t(x))


# ---- the short convolution ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 4])
def test_short_conv_whole_in_portions_and_token_by_token(taps, dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(taps)
    C, n, col0 = (72, 23, 8) if taps == 4 else (70, 23, 8)         # 72 channels in a matrix of 88 columns: eight per thread
    x = _t(rng.standard_normal((n, col0 + C + (8 if taps == 4 else 5))), dtype)
    w = _t(rng.uniform(-0.8, 0.8, (C, taps)))
    wt = w.t().contiguous()
    want = P.short_conv(_np(x)[:, col0:col0 + C], _np(w))
    results = {}
    for label, cuts in (("whole", [n]), ("portions", [2, 1, 7, 2, 11]), ("single", [1] * n)):
        state = torch.full((3, taps - 1, C), 5.0, device=DEV)
        state[1].zero_()                                                  # the cache zeroes a slot that is given out
        outs, at = [], 0
        for c in cuts:
            tok_seq, seq_start = _tables([c])
            outs.append(ops.short_conv(x[at:at + c].contiguous(), col0, w, state, tok_seq, _i([1]), seq_start, single=(c == 1),
                                       weight_t=wt if label != "portions" else None))
            at += c
        results[label] = torch.cat(outs)
        _close(results[label], want, torch.float32, f"{label}, {taps} taps", tol32=1e-5)
        assert torch.all(state[0] == 5.0) and torch.all(state[2] == 5.0)
        if taps > 1:
            assert torch.equal(state[1], x[n - (taps - 1):, col0:col0 + C].float())
    assert torch.equal(results["whole"], results["portions"]) and torch.equal(results["whole"], results["single"])


# ---- the recurrence ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, dim, vdim", [(4, 2, 12, 20), (2, 2, 136, 16), (1, 1, 64, 70), (3, 1, 200, 8), (1, 1, 300, 9)])
def test_delta_rule_against_the_plain_recurrence(H, G, dim, vdim, dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(H * dim)
    lengths, slots = [37, 1, 6], [2, 0, 3]
    T = sum(lengths)
    C = 2 * G * dim + H * vdim
    qkv = _t(rng.standard_normal((T, C)))
    proj = _t(rng.standard_normal((T, 3 + H)) * 2, dtype)                 # beta's logits from column 3
    z = _t(rng.standard_normal((T, H * dim)) * 2, dtype)
    dt_bias, a_log = _t(rng.uniform(-3, 1, H * dim)), _t(rng.uniform(-2, 0.5, H))
    tok_seq, seq_start = _tables(lengths)
    state = torch.zeros((4, H, dim, vdim), device=DEV)
    o = ops.delta_rule_recurrent(qkv.clone(), 0, G * dim, 2 * G * dim, proj, 3, z, dt_bias, a_log, dim ** -0.5, state, _i(slots),
                                 seq_start, H, G, dim, vdim)                   # (the call makes q and k unit vectors in place)
    q = _np(qkv)[:, :G * dim].reshape(T, G, dim)
    k = _np(qkv)[:, G * dim:2 * G * dim].reshape(T, G, dim)
    v = _np(qkv)[:, 2 * G * dim:].reshape(T, H, vdim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = P.sigmoid(_np(proj)[:, 3:])
    g = np.exp(-np.exp(_np(a_log))[None, :, None] * P.softplus(_np(z) + _np(dt_bias)).reshape(T, H, dim))
    at = 0
    for n in lengths:
        for h in range(H):
            want = P.delta_rule(q[at:at + n, h // (H // G)], k[at:at + n, h // (H // G)], v[at:at + n, h], beta[at:at + n, h],
                                g[at:at + n, h])
            _close(o[at:at + n, h], want, torch.float32, f"head {h} of a sequence of {n}", tol32=3e-5)
        at += n
    assert torch.all(state[1] == 0)
    # the first sequence again in pieces and token by token, on another slot: the same bits, the same state
    n = lengths[0]
    for cuts in ([2, 9, 1, 25], [1] * n):
        st2 = torch.zeros_like(state)
        outs, at = [], 0
        for c in cuts:
            _, ss = _tables([c])
            outs.append(ops.delta_rule_recurrent(qkv[at:at + c].clone(), 0, G * dim, 2 * G * dim, proj[at:at + c].contiguous(), 3,
                                                 z[at:at + c].contiguous(), dt_bias, a_log, dim ** -0.5, st2, _i([1]), ss, H, G, dim,
                                                 vdim, single=(c == 1)))
            at += c
        assert torch.equal(torch.cat(outs), o[:n]) and torch.equal(st2[1], state[2])


# ---- rotation of neighbouring pairs, chunked mask, sink -----------------------------------------------------------------
def _paged(rng, k, v, page_size=32, spare=3):
    """Keys and values [n, KV, D] of one sequence in pools whose pages are in no order; slot 1 of 2."""
    n, KV, D = k.shape
    pages = -(-n // page_size)
    order = rng.permutation(pages + spare)[:pages]
    kp = torch.zeros((pages + spare, KV, page_size, D), dtype=k.dtype, device=DEV)
    vp = torch.zeros_like(kp)
    for p in range(n):
        kp[order[p // page_size], :, p % page_size] = k[p]
        vp[order[p // page_size], :, p % page_size] = v[p]
    table = torch.full((2, pages + 2), -1, dtype=torch.int32, device=DEV)
    table[1, :pages] = _i(order)
    return kp, vp, table


def _plain_chunked(q, k, v, sink, scale, size, positions):
    """q [rows, H, D] at ``positions``; k, v [n, KV, D]: softmax over the query's own chunk up to itself, with the sink."""
    H, KV = q.shape[1], k.shape[1]
    out = np.zeros(q.shape)
    for r, p in enumerate(positions):
        lo = (p // size) * size if size else 0
        for h in range(H):
            s = (k[lo:p + 1, h // (H // KV)] @ q[r, h]) * scale
            top = max(s.max(), sink[h])
            e = np.exp(s - top)
            out[r, h] = (e @ v[lo:p + 1, h // (H // KV)]) / (e.sum() + np.exp(sink[h] - top))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D, size", [(32, 7), (80, 33), (64, 90), (128, 40)])
def test_chunked_attention_with_a_loud_key_at_the_edges(D, size, dtype):
    """One key is made loud (its score stands out among hundreds).  Queries just inside its chunk must follow its value,
    queries just outside must not see it; in a prompt, in a portion of a prompt, and token by token."""
    from rust_inference_b200 import ops
    rng = np.random.default_rng(D + size)
    n, H, KV, scale = 300, 4, 2, 0.25
    k = rng.standard_normal((n, KV, D)) * 0.3
    v = rng.standard_normal((n, KV, D))
    q = rng.standard_normal((n, H, D)) * 0.3
    chunk0 = (n // size - 1) * size                       # the start of the last whole chunk
    loud = [chunk0 - 1, chunk0, 5]                        # the last key of a chunk, the first of the next, a far one
    direction = rng.standard_normal(D)
    direction /= np.linalg.norm(direction)
    for j in loud:
        k[j] += 6.0 * direction
    q += 4.0 * direction                                 # every query looks for the loud keys
    sink = rng.uniform(-1, 3, H)
    kt, vt, qt = _t(k, dtype), _t(v, dtype), _t(q, dtype)
    kp, vp, table = _paged(rng, kt, vt)
    want = _plain_chunked(_np(qt), _np(kt), _np(vt), sink, scale, size, range(n))
    slot, sink_t = _i([1]), _t(sink)
    tol = dict(tol32=3e-5, tol16=2e-2)
    # a whole prompt, and its last 100 tokens as a portion (the chunk does not start where the portion does)
    for first in (0, n - 100):
        new = n - first
        start, length = _i([0, new]), _i([n])
        got = ops.attention(qt[first:].contiguous(), kp, vp, table, slot, start, length, new, scale, sink=sink_t, chunk=size)
        _close(got, want[first:], dtype, f"rows kernel from {first}", **tol)
        if dtype == torch.bfloat16:
            got = ops.attention_prefill(qt[first:].contiguous(), kp, vp, table, slot, start, length, new, scale, 0, sink=sink_t,
                                        chunk=size)
            _close(got, want[first:], dtype, f"prefill kernel from {first}", **tol)
    # single tokens around the edges: the query at chunk0 - 1 sees the loud key there, the one at chunk0 only the next
    for p in (chunk0 - 1, chunk0, chunk0 + 1, chunk0 + size - 1, n - 1):
        length = _i([p + 1])
        got = ops.attention(qt[p:p + 1].contiguous(), kp, vp, table, slot, _i([0, 1]), length, 1, scale, sink=sink_t, chunk=size)
        _close(got, want[p:p + 1], dtype, f"rows kernel, token {p}", **tol)
        if dtype == torch.bfloat16:
            got = ops.attention_decode(qt[p:p + 1].contiguous(), kp, vp, table, slot, length, scale, 0, 1024, sink=sink_t, chunk=size)
            _close(got, want[p:p + 1], dtype, f"decode kernel, token {p}", **tol)
    # the loud key decides what its chunk's queries return, so a mask that is one token off cannot hide in the tolerance:
    # with the chunk's edge moved by one, the plain result itself changes by far more than the tolerance
    moved = _plain_chunked(_np(qt)[chunk0:chunk0 + 1], _np(kt), _np(vt), sink, scale, 0, [chunk0])
    assert np.abs(moved - want[chunk0]).max() > 0.2 * np.abs(want[chunk0]).max()


def test_pair_rotation_in_the_append_kernel():
    from rust_inference_b200 import ops
    from rust_inference_b200.config.specs import RopePairsSpec
    from rust_inference_b200.parts import BuildEnv, build_part
    rng = np.random.default_rng(5)
    T, H, KV, Dh, rot = 9, 3, 1, 48, 20
    part = build_part("position", RopePairsSpec(rotary_dim=rot, theta=300.0), BuildEnv(torch.float32, torch.device(DEV)))
    part.prepare(64)
    qkv = _t(rng.standard_normal((T, (H + 2 * KV) * Dh)))
    pos = [40 + t for t in range(T)]
    kp = torch.zeros((4, KV, 32, Dh), device=DEV)
    vp = torch.zeros_like(kp)
    table = _i([2, 0, 1, 3]).view(1, 4)
    tok_seq, _ = _tables([T])
    q = ops.qk_norm_rope_append(qkv, H, KV, Dh, None, None, 0.0, part.fused_table(), rot, kp, vp, table, tok_seq, _i(pos), _i([0]),
                                pairs=True)
    x = _np(qkv).reshape(T, H + 2 * KV, Dh)
    full = np.zeros((64, H + 1, Dh))
    full[pos] = x[:, :H + 1]
    turned = P.rotate_pairs(full, rot, 300.0)[pos]
    _close(q, turned[:, :H], torch.float32, "queries", tol32=1e-5)
    for t, p in enumerate(pos):
        page = [2, 0, 1, 3][p // 32]
        _close(kp[page, 0, p % 32], turned[t, H], torch.float32, "keys", tol32=1e-5)
        assert torch.equal(vp[page, 0, p % 32], qkv[t, (H + KV) * Dh:])


# ---- feed-forwards -------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gates(dtype):
    from rust_inference_b200 import ops
    rng = np.random.default_rng(2)
    for rows, inter, block in ((3, 24, 8), (70, 20, 20), (5, 7, 7)):
        gu = _t(rng.standard_normal((rows, 2 * inter)) * 2, dtype)
        x = _np(gu).reshape(rows, inter // block, 2, block)
        g, u = x[:, :, 0].reshape(rows, inter), x[:, :, 1].reshape(rows, inter)
        _close(ops.gated_act(gu, "silu", block), P.silu(g) * u, dtype, "silu")
        _close(ops.gated_act(gu, "gelu_tanh", block), P.gelu_tanh(g) * u, dtype, "gelu")
        gc, uc = np.minimum(g, 0.9), np.clip(u, -0.9, 0.9)
        _close(ops.gated_act(gu, "clamped_swish", block, 0.9, 1.702), gc * P.sigmoid(1.702 * gc) * (uc + 1), dtype, "clamped swish")
    # the gelu gate behind a product: in the weight-streaming product's epilogue for a handful of bfloat16 tokens, else after it
    inter, K = 40, 64
    wg, wu = _t(rng.standard_normal((inter, K)) * 0.3, dtype), _t(rng.standard_normal((inter, K)) * 0.3, dtype)
    stacked = torch.stack([wg.view(inter // 8, 8, K), wu.view(inter // 8, 8, K)], dim=1).reshape(2 * inter, K).contiguous()
    for m in (3, 12, 70):
        xin = _t(rng.standard_normal((m, K)), dtype)
        want = P.gelu_tanh(_np(xin) @ _np(wg).T) * (_np(xin) @ _np(wu).T)
        _close(ops.linear_gated(xin, stacked, 8, "gelu_tanh"), want, dtype, f"gelu-gated product of {m} tokens")


def test_router_choice_weights_and_ties():
    from rust_inference_b200 import ops
    rng = np.random.default_rng(3)
    T, D, N, top = 50, 36, 11, 4
    x = _t(rng.standard_normal((T, D)))
    router, corr = _t(rng.standard_normal((N, D)) * 0.5), _t(rng.uniform(-0.2, 0.2, N))
    idx, w = ops.moe_route(x, router, corr, top)
    chosen, weight = P.route(_np(x), _np(router), _np(corr), top)
    assert np.array_equal(idx.cpu().numpy(), chosen)
    _close(w, weight, torch.float32, "weights", tol32=1e-5)
    # a router too large for the kernel that takes a block per token, and rows that are no whole 16-byte pieces
    for T2, D2, N2 in ((5, 4096, 300), (9, 50, 13)):
        x2, r2, c2 = _t(rng.standard_normal((T2, D2))), _t(rng.standard_normal((N2, D2)) * 0.1), _t(rng.uniform(-0.05, 0.05, N2))
        idx, w = ops.moe_route(x2, r2, c2, 5)
        chosen, weight = P.route(_np(x2), _np(r2), _np(c2), 5)
        assert np.array_equal(idx.cpu().numpy(), chosen)
        _close(w, weight, torch.float32, "weights", tol32=1e-4)
    # equal choice scores: the lower index first; the correction changes the choice but not the weights
    router0 = torch.zeros((6, D), device=DEV)
    idx, w = ops.moe_route(x[:3].contiguous(), router0, torch.zeros(6, device=DEV), 3)
    assert idx.cpu().tolist() == [[0, 1, 2]] * 3 and torch.allclose(w, torch.full_like(w, 1 / 3))
    idx, w = ops.moe_route(x[:3].contiguous(), router0, _t([0.0, 0.5, 0.0, 0.0, 0.7, 0.0]), 2)
    assert idx.cpu().tolist() == [[4, 1]] * 3 and torch.allclose(w, torch.full_like(w, 0.5))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T, D, ff, E, ident, top", [(1, 48, 24, 5, 1, 2), (70, 52, 20, 3, 0, 1), (300, 64, 40, 9, 3, 4)])
def test_routed_feed_forward_against_the_plain_one(T, D, ff, E, ident, top, dtype):
    """The whole part (router, plan, grouped products, combination, shared expert) against the plain formulas."""
    from rust_inference_b200.config.specs import GatedFFSpec, MoESpec
    from rust_inference_b200.parts import BuildEnv, build_part
    rng = np.random.default_rng(T + D)
    expert = GatedFFSpec(D, ff, gate="clamped_swish", limit=0.8, alpha=1.702)
    spec = MoESpec(D, E, top, expert, identity=ident, shared=GatedFFSpec(D, 2 * ff, gate="clamped_swish", limit=1.5, alpha=1.702))
    part = build_part("ffn", spec, BuildEnv(dtype, torch.device(DEV)))
    W = {"router": rng.standard_normal((E + ident, D)) * 3 / np.sqrt(D), "correction": rng.uniform(-0.1, 0.1, E + ident)}
    for pre, f in [(f"e{e}.", ff) for e in range(E)] + [("shared.", 2 * ff)]:
        W[pre + "gate"], W[pre + "up"] = rng.standard_normal((f, D)) * 2 / np.sqrt(D), rng.standard_normal((f, D)) * 2 / np.sqrt(D)
        W[pre + "down"] = rng.standard_normal((D, f)) / np.sqrt(f)
    tensors = {k: _t(v, torch.float32 if k in ("router", "correction") else dtype) for k, v in W.items()}
    part.load(tensors)
    x = _t(rng.standard_normal((T, D)), dtype)
    got = part(x, None)
    Wd = {k: _np(v) for k, v in tensors.items()}
    m = {"router": {"experts": E, "identity": ident, "top": top}, "expert": {"limit": 0.8}, "shared": {"limit": 1.5}}
    want = P.moe_ff(_np(x), Wd, m)
    if dtype == torch.float32:
        _close(got, want, dtype, "routed feed-forward", tol32=3e-5)
    else:
        # bfloat16: the same choices (the router reads the same rounded input), products rounded to 8 bits
        err = np.abs(_np(got) - want).max(-1) / np.abs(want).max()
        assert np.median(err) < 1.5e-2 and err.max() < 6e-2


# ---- whole models ----------------------------------------------------------------------------------------------------------
def _portions(reqs, sizes):
    """Each request alone, its prompt brought in portions of ``sizes`` tokens (repeated), every position wanted."""
    steps, n = [], 0
    for rid, toks in reqs.items():
        at, j = 0, 0
        while at < len(toks):
            c = min(sizes[j % len(sizes)], len(toks) - at)
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[at:at + c], "want": list(range(c))}],
                          "end": [rid] if at + c == len(toks) else []})
            at, j, n = at + c, j + 1, n + 1
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_in_five_cuttings_matches_plain(tmp_path, name, dtype):
    d, config, weights = R.make_model_dir(tmp_path, name, seed=3)
    rng = np.random.default_rng(4)
    reqs = H.random_requests(rng, config["vocab"], [5, 1, 23, 150, 2, 70, 37])
    want = R.plain_logits(config, weights, reqs)
    by_cutting = {}
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=40)),
                         ("portions", _portions(reqs, [2, 7, 1, 33, 2])), ("pairs", _portions(reqs, [2])),
                         ("batches", H.trace_batches(reqs, 3, [6, 0, 9, 3, 70, 1, 36]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, dtype, steps, out, device="cuda:0")
        rows = H.collect(steps, out, config["vocab"])
        assert len(rows) == sum(len(t) for t in reqs.values())
        R.assert_rows_close(rows, want, dtype, f"{name} {label} {dtype}")
        by_cutting[label] = rows
    if dtype == "float32":
        H.assert_rows_identical(by_cutting, f"{name} float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_chunk_and_page_edges(tmp_path, dtype):
    """A short prompt, then 260 tokens one by one (graph replays), against the plain model: chunks of 7, 33 and 64 positions
    begin and end, pages behind a chunk go back to the free list and are used again."""
    d, config, weights = R.make_model_dir(tmp_path, "A", seed=6)
    rng = np.random.default_rng(7)
    reqs = H.random_requests(rng, config["vocab"], [270, 200])
    want = R.plain_logits(config, weights, reqs)
    steps = H.trace_batches(reqs, 2, [260, 195])
    out = str(tmp_path / "out")
    H.replay_inprocess(d, dtype, steps, out, device="cuda:0", max_tokens=640)
    R.assert_rows_close(H.collect(steps, out, config["vocab"]), want, dtype, f"long decoding {dtype}")


def test_greedy_generation_with_more_requests_than_slots(tmp_path):
    import rust_inference_b200 as ri
    d, config, weights = R.make_model_dir(tmp_path, "A", seed=8)
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    rng = np.random.default_rng(9)
    prompts = [[int(t) for t in rng.integers(0, config["vocab"], n)] for n in (3, 1, 9, 40, 2)]
    llm = ri.LLM(d, dtype="float32", max_pages=16, pages_per_seq=4, max_seqs=2)
    got = llm.generate(prompts, max_new_tokens=12)
    assert llm.engine.graph_replays > 0
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(12):
            seq.append(int(np.argmax(P.forward(config, W, seq)[0][-1])))
        assert g == seq[len(p):]
