"""Ranudra without a GPU: the configuration class, the tensor list, and the engine's host logic (schedule with a
repeated run, cache groups whose values are the keys, per-sequence state, slots used again) with the kernels
replaced by the stand-ins of tests/emu_ops.py, against the plain model of tests/plain_ranudra.py."""
import copy

import numpy as np
import pytest

import helpers as H
import ranudra_models as R


def test_spec_lists_parts_and_schedule():
    from rust_inference_b200.config import config_from_dict
    from rust_inference_b200.engine.model import expected_tensors
    cfg = config_from_dict(copy.deepcopy(R.CFG_A))
    assert type(cfg).__name__ == "RanudraConfig" and cfg.to_dict()["layers"] == R.CFG_A["layers"]
    spec = cfg.to_spec()
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2), (1, 3), (2, 4), (1, 5), (2, 6), (3, 7)]
    assert spec.tie_embeddings and spec.embedding.scale == 3.0 and spec.embedding.copies == 3
    first = spec.layers[0].mixer
    assert (first.sink, first.gate, first.window, first.position.yarn) == (True, "element", 7, None)
    third = spec.layers[2].mixer
    assert (third.sink, third.gate, third.window) == (False, "head", 40) and third.position.yarn == (4.0, 32.0, 8.0, 2.0)
    # the tensors follow from the parts; the decay projection's inner size comes from the checkpoint (0 until then)
    names = set(expected_tensors(spec))
    assert names == set(R.make_weights(R.CFG_A, 0))
    plain = config_from_dict(copy.deepcopy(R.CFG_B)).to_spec()
    assert plain.embedding.copies == 1 and plain.layers[0].ffn is None
    assert not any(".hc" in n or n == "l0.norm2" for n in expected_tensors(plain))
    assert plain.layers[2].mixer.position.kind == "none" and plain.layers[2].mixer.window == 0


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="conv"), "not built"),
    (lambda c: c["layers"][1]["mlp"].update(kind="experts"), "not built"),
    (lambda c: c.update(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
    (lambda c: c["layers"][0]["mixer"].update(rot_dim=7), "rot_dim"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=8), "dims"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.update(streams=40), "streams"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "tau"),
])
def test_bad_configurations_are_refused(change, text):
    from rust_inference_b200.config import ConfigError, config_from_dict
    c = copy.deepcopy(R.CFG_A)
    change(c)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(c)


def test_rotary_table_matches_the_plain_frequencies():
    """The angles of the pairwise rotation, with and without YaRN, against the plain functions."""
    import torch
    import plain_ranudra as P
    from rust_inference_b200.config.specs import RopePairsSpec
    from rust_inference_b200.parts import BuildEnv, build_part
    env = BuildEnv(torch.float32, torch.device("cpu"))
    for dims, base, yarn in ((16, 5000.0, (4.0, 32.0, 8.0, 2.0)), (6, 50.0, None), (32, 1e6, (40.0, 4096.0, 32.0, 1.0))):
        part = build_part("position", RopePairsSpec(rotary_dim=dims, theta=base, yarn=yarn), env)
        part.prepare(300)
        scaling = None if yarn is None else dict(zip(("factor", "original", "fast", "slow"), yarn))
        f, mult = P.rotary_frequencies(dims, base, scaling)
        ang = np.arange(300)[:, None] * f[None, :]
        want = np.stack([np.cos(ang) * mult, np.sin(ang) * mult], axis=-1)
        assert np.abs(part.fused_table().numpy() - want).max() < 3e-5


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_three_ways_matches_plain(tmp_path, emulated_ops, name):
    d, config, weights = R.make_model_dir(tmp_path, name, seed=3)
    rng = np.random.default_rng(4)
    reqs = H.random_requests(rng, config["vocab"], [5, 1, 23, 44, 2, 37])
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
    import plain_ranudra as P
    import rust_inference_b200 as ri
    d, config, weights = R.make_model_dir(tmp_path, "B", seed=8)
    W = {k: v.astype(np.float64) for k, v in weights.items()}
    prompts = [[5, 9, 2], [7], [100, 3, 3, 8, 1, 60]]
    llm = ri.LLM(d, dtype="float32", device="cpu", max_pages=8, pages_per_seq=2, max_seqs=2, use_graphs=False)
    got = llm.generate(prompts, max_new_tokens=5)
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(5):
            seq.append(int(np.argmax(P.forward(config, W, seq)[0][-1])))
        assert g == seq[len(p):]
