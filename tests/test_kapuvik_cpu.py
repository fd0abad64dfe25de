"""Kapuvik without a GPU: the configuration reader and its faults, the plan's tensor names, running order, stream
inputs and cache needs, random-model folders, and the plain mechanisms on cases worked out by hand."""
import copy
import json

import numpy as np
import pytest

import plain_kapuvik as K
from kapuvik_helpers import CONFIGS, lively_weights, tensor_shapes


def plan_of(raw):
    from velox_b200.config import resolve_architecture
    arch = resolve_architecture(raw)
    cfg = arch.config_class.from_dict(raw)
    return cfg, arch.plan(cfg)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plan_asks_for_the_tensors_of_the_design(name):
    from velox_b200.models.decoder import DecoderModel
    raw = CONFIGS[name]
    cfg, plan = plan_of(raw)
    assert type(cfg).__name__ == "KapuvikConfig" and cfg.to_dict()["layers"] == raw["layers"]
    model = DecoderModel(plan)
    assert {s.name: tuple(s.shape) for s in model.tensor_specs()} == tensor_shapes(raw)


def test_a_decay_projection_without_a_stated_middle_width_leaves_it_open():
    from velox_b200.models.decoder import DecoderModel
    raw = copy.deepcopy(CONFIGS["plain"])
    del raw["layers"][1]["mixer"]["rank"]
    shapes = {s.name: tuple(s.shape) for s in DecoderModel(plan_of(raw)[1]).tensor_specs()}
    assert shapes["l1.mix.a1"] == (-1, 64) and shapes["l1.mix.a2"] == (32, -1)


def test_running_order_stream_inputs_and_cache_needs():
    from velox_b200.models.decoder import DecoderModel
    from velox_b200.parts import CacheParts, FixedState, PagedKV, PagedLatent
    _, plan = plan_of(CONFIGS["odd"])
    assert plan.running_order() == [0, 1, 2, 1, 2, 1, 2, 3] == [i for i, _, _ in K.running_order(CONFIGS["odd"])]
    assert [(x.place, x.embedding, x.tensor, x.row, x.rows) for x in plan.stream_inputs] == \
        [(1, False, "loop.step", 0, 3), (3, True, "loop.step", 1, 3), (5, True, "loop.step", 2, 3)]
    specs = DecoderModel(plan).cache_specs()
    assert specs[0] == FixedState((3, 20, 24), "float32") and specs[1] == specs[3] == specs[5] == PagedLatent(26)
    assert specs[2] == CacheParts((PagedKV(2, 20, 0, 12, 0), FixedState((2, 10, 14), "float32")))
    _, plain = plan_of(CONFIGS["plain"])
    assert plain.running_order() == [0, 1, 2] and plain.stream_inputs == []


def test_every_place_of_a_looped_layer_has_a_cache_of_its_own():
    from velox_b200.cache.manager import CacheManager
    from velox_b200.models.decoder import DecoderModel
    model = DecoderModel(plan_of(CONFIGS["even"])[1])
    cache = CacheManager(model.cache_specs(), model.cache_sources(), page_size=16, num_pages=8, max_requests=2, max_blocks=8)
    widths = sorted(getattr(g.spec, "width", 0) or g.spec.head_dim for g in cache.groups)
    assert widths == [64, 128, 128]            # left keys of 64 (run twice: one group, two places), a latent row, left keys of 128
    assert sorted(len(g.layers) for g in cache.groups) == [1, 2, 2]


@pytest.mark.parametrize("damage,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][2]["mixer"]["left"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][2]["mixer"]["right"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(dims=40), "within"),
    (lambda c: c["layers"][1]["mixer"].update(rot_dim=5), "rot_dim"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"].update(tau=0), "tau"),
    (lambda c: c["layers"][0]["mlp"].update(limit=-1.0), "limit"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "dense"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
])
def test_faults_of_a_configuration_are_named(damage, word):
    from velox_b200.config import ConfigError
    raw = copy.deepcopy(CONFIGS["odd"])
    damage(raw)
    with pytest.raises(ConfigError) as e:
        plan_of(raw)
    assert word in str(e.value)


def test_a_random_model_folder_is_written_and_read_back(tmp_path):
    from velox_b200.config import load_config
    from velox_b200.weights.random_init import write_random_model
    from velox_b200.weights.safetensors_io import SafetensorsFile
    cfg, _ = plan_of(CONFIGS["odd"])
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=4)
    arch, back = load_config(folder)
    assert arch.name == "Kapuvik" and back == cfg
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    assert {n: tuple(f.info(n)[1]) for n in f.keys()} == tensor_shapes(CONFIGS["odd"])
    raw = copy.deepcopy(CONFIGS["plain"])
    del raw["layers"][1]["mixer"]["rank"]
    with pytest.raises(ValueError):
        write_random_model(str(tmp_path / "n"), plan_of(raw)[0], seed=4)


# -- the plain mechanisms on cases worked out by hand ---------------------------------------------------------------
def test_rotation_pairs_neighbours_or_halves():
    x = np.zeros((1, 1, 6))
    x[0, 0] = [1, 0, 2, 0, 9, 9]
    quarter = [np.pi / 2]        # position * base^0 for the first pair
    got = K.rotate(x, quarter, 1e30, 4, True)[0, 0]      # (0,1) turned a quarter, (2,3) by position / base: nothing
    assert np.allclose(got, [0, 1, 2, 0, 9, 9])
    got = K.rotate(x, quarter, 1e30, 4, False)[0, 0]     # pairs (0,2) and (1,3)
    assert np.allclose(got, [-2, 0, 1, 0, 9, 9])


def test_a_capped_score_cannot_dominate():
    q = np.array([[[0.0]], [[100.0]]])
    k = np.array([[[100.0]], [[0.0]]])
    v = np.array([[[1.0]], [[0.0]]])
    free = K.causal_softmax_attention(q, k, v, 1.0)[1, 0, 0]
    capped = K.causal_softmax_attention(q, k, v, 1.0, softcap=2.0)[1, 0, 0]
    assert free > 0.9999 and abs(capped - np.exp(2.0) / (np.exp(2.0) + 1.0)) < 1e-12


def test_the_state_walk_against_its_closed_form():
    rng = np.random.default_rng(0)
    T, H, D, Dv = 7, 2, 3, 4
    q, k, v = rng.normal(size=(T, H, D)), rng.normal(size=(T, H, D)), rng.normal(size=(T, H, Dv))
    decay = np.array([0.5, 1.0])
    got = K.decayed_state_walk(q, k, v, decay)
    for t in range(T):
        for h in range(H):
            want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert np.allclose(got[t, h], want)
    a = rng.uniform(0.2, 1.0, size=(T, H, D))            # a decay per channel and position: products over the way
    got = K.decayed_state_walk(q, k, v, a)
    t, h = T - 1, 1
    want = sum(np.sum(q[t, h] * k[j, h] * np.prod(a[j + 1:t + 1, h], axis=0)) * v[j, h] for j in range(t + 1))
    assert np.allclose(got[t, h], want)


def test_the_bounded_feed_forward_by_hand():
    P = {"gate": np.array([[1.0], [1.0]]), "gate.b": np.array([0.0, 5.0]), "up": np.array([[1.0], [-10.0]]),
         "up.b": np.array([0.5, 0.0]), "down": np.array([[1.0, 1.0]]), "down.b": np.array([0.25])}
    y = K.capped_feed_forward(np.array([[1.0]]), P, {"limit": 2.0})[0, 0]
    g0, g1 = 1.0, 2.0                                    # the second gate is cut at the limit
    want = g0 * K.sigmoid(1.702 * g0) * (1.5 + 1.0) + g1 * K.sigmoid(1.702 * g1) * (-2.0 + 1.0) + 0.25
    assert abs(y - want) < 1e-12


def test_every_pass_takes_its_vector_and_later_ones_the_embedding_again():
    cfg = CONFIGS["odd"]
    w = lively_weights(cfg, 1)
    toks = [3, 50, 7, 7, 99]
    base = K.forward(cfg, w, toks)
    for row in range(3):
        w2 = dict(w)
        w2["loop.step"] = w["loop.step"].copy()
        w2["loop.step"][row] += 1.0
        assert np.abs(K.forward(cfg, w2, toks) - base).max() > 1e-3
    # the same model with one pass takes no embedding again: scaling it shows in the loop only through layer 0's output
    one = copy.deepcopy(cfg)
    one["loop"]["times"] = 1
    w1 = dict(w)
    w1["loop.step"] = w["loop.step"][:1]
    assert K.running_order(one) == [(0, None, False), (1, 0, True), (2, 0, False), (3, None, False)]
    assert np.isfinite(K.forward(one, w1, toks)).all()
