"""Pitenex without a GPU: the configuration class, the tensor list, and the engine's host logic (a cache entry with pages,
two kinds of state and a chunked mask; the embedding's own state; slots used again) with the kernels replaced by the
stand-ins of tests/emu_ops.py, against the plain model of tests/plain_pitenex.py."""
import copy

import numpy as np
import pytest

import helpers as H
import pitenex_models as R


def test_spec_lists_parts_and_tensors():
    from rust_inference_b200.config import config_from_dict
    from rust_inference_b200.engine.model import expected_tensors
    cfg = config_from_dict(copy.deepcopy(R.CFG_A))
    assert type(cfg).__name__ == "PitenexConfig" and cfg.to_dict()["layers"] == R.CFG_A["layers"]
    spec = cfg.to_spec()
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2)]
    assert spec.tie_embeddings and spec.head.scale == 1.5 and spec.embedding.buckets == 53
    first = spec.layers[0]
    assert first.arrangement == "parallel" and first.link.scale == 0.6 and first.norm.bias_name == ".b"
    left, right = first.mixer.left, first.mixer.right
    assert (left.chunk, left.window, left.sink, left.head_dim, left.v_head_dim, left.position.rotary_dim) == (7, 0, True, 16, 24, 8)
    assert (right.num_heads, right.num_qk_heads, right.conv) == (4, 2, 4)
    assert first.ffn.kind == "moe" and (first.ffn.experts, first.ffn.identity, first.ffn.top) == (5, 1, 2)
    assert first.ffn.expert.gate == "clamped_swish" and first.ffn.shared.limit == 1.2
    assert spec.layers[1].ffn.gate == "gelu_tanh" and spec.layers[2].ffn is None
    assert spec.layers[2].mixer.left.position.kind == "none"
    # the low-rank projections' inner sizes come from the checkpoint (0 until then): names only
    assert set(expected_tensors(spec)) == set(R.make_weights(R.CFG_A, 0))


def test_ranks_come_from_the_checkpoint(tmp_path):
    from rust_inference_b200.config import load_config
    from rust_inference_b200.engine.model import expected_tensors
    d, config, weights = R.make_model_dir(tmp_path, "B", seed=1)
    cfg = load_config(d).with_checkpoint(d)
    shapes = {n: tuple(i.shape) for n, i in expected_tensors(cfg.to_spec()).items()}
    assert shapes == {n: w.shape for n, w in weights.items()}
    assert shapes["l0.mix.right.a1"] == (5, 52) and shapes["l1.mix.right.g2"] == (64, 3)


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="serial"), "not built"),
    (lambda c: c["layers"][1]["mlp"].update(kind="experts"), "not built"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c.pop("logit_scale"), "logit_scale"),
    (lambda c: c["embedding"]["bigram"].pop("buckets"), "buckets"),
])
def test_bad_configurations_are_refused(change, text):
    from rust_inference_b200.config import ConfigError, config_from_dict
    c = copy.deepcopy(R.CFG_A)
    change(c)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(c)


def test_cache_request_of_two_mixers_side_by_side():
    """Keys and values of the left mixer (one head size for both, the chunk as the mask) and the right one's two states."""
    import torch
    from rust_inference_b200.config import config_from_dict
    from rust_inference_b200.parts import BuildEnv, build_part
    spec = config_from_dict(copy.deepcopy(R.CFG_A)).to_spec()
    env = BuildEnv(torch.float32, torch.device("cpu"))
    r = build_part("mixer", spec.layers[0].mixer, env).cache_request()
    assert (r.kv_heads, r.head_dim, r.chunk, r.window, r.mask) == (2, 32, 7, 0, -7)
    assert r.state_shape == (4, 12, 20) and r.more_state == (((3, 2 * 2 * 12 + 4 * 20), torch.float32),)
    r = build_part("mixer", spec.layers[2].mixer, env).cache_request()
    assert (r.head_dim, r.chunk) == (32, 64)


def test_chunked_groups_give_pages_back():
    """A chunked group keeps the pages of the current chunk only."""
    from rust_inference_b200.cache.allocator import PageTable
    pt = PageTable(num_slots=2, num_pages=16, max_pages_per_seq=16, page_size=4, window=-10)
    assert pt.extend(0, 9) == 0 and pt.release_behind_window(0) == 0         # next query at 9: chunk starts at 0
    pt.extend(0, 1)
    assert pt.release_behind_window(0) == 2                                   # next query at 10: keys 0..7 are gone
    pt.extend(0, 13)
    assert pt.release_behind_window(0) == 3                                   # next query at 23: chunk starts at 20


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_replay_three_ways_matches_plain(tmp_path, emulated_ops, name):
    d, config, weights = R.make_model_dir(tmp_path, name, seed=3)
    rng = np.random.default_rng(4)
    reqs = H.random_requests(rng, config["vocab"], [5, 1, 23, 70, 2, 37])
    want = R.plain_logits(config, weights, reqs)
    for label, steps in (("whole", H.trace_whole(reqs)), ("tail", H.trace_tail(reqs, tail=12)),
                         ("batches", H.trace_batches(reqs, 3, [6, 0, 9, 3]))):
        out = str(tmp_path / f"out_{label}")
        H.replay_inprocess(d, "float32", steps, out)
        rows = H.collect(steps, out, config["vocab"])
        assert len(rows) == sum(len(t) for t in reqs.values())
        R.assert_rows_close(rows, want, "float32", f"{name} {label}")


def test_greedy_generation_matches_plain(tmp_path, emulated_ops):
    """Greedy tokens through the generation loop (two batches on the same slots) against the plain model."""
    import plain_pitenex as P
    import rust_inference_b200 as ri
    d, config, weights = R.make_model_dir(tmp_path, "A", seed=8)
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    prompts = [[5, 9, 2], [7], [90, 3, 3, 8, 1, 60, 4, 4, 12]]
    llm = ri.LLM(d, dtype="float32", device="cpu", max_pages=8, pages_per_seq=2, max_seqs=2, use_graphs=False)
    got = llm.generate(prompts, max_new_tokens=5)
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(5):
            seq.append(int(np.argmax(P.forward(config, W, seq)[0][-1])))
        assert g == seq[len(p):]
