"""Fovenex without a GPU: the configuration reader and its faults, the plan's tensor names, what every layer keeps in the
cache and whose rows it reads, random-model folders, and the plain mechanisms on cases worked out by hand."""
import copy
import json
import math

import numpy as np
import pytest

import plain_fovenex as F
from fovenex_helpers import CONFIGS, drawn_config, lively_weights, tensor_shapes


def plan_of(raw):
    from velox_b200.config import resolve_architecture
    arch = resolve_architecture(raw)
    cfg = arch.config_class.from_dict(raw)
    return cfg, arch.plan(cfg)


@pytest.mark.parametrize("name", sorted(CONFIGS) + ["drawn 0", "drawn 3", "drawn 6"])
def test_the_plan_asks_for_the_tensors_of_the_design(name):
    from velox_b200.models.decoder import DecoderModel
    raw = CONFIGS[name] if name in CONFIGS else drawn_config(int(name.split()[1]))
    cfg, plan = plan_of(raw)
    assert type(cfg).__name__ == "FovenexConfig" and cfg.to_dict()["layers"] == raw["layers"]
    assert plan_of(cfg.to_dict())[0] == cfg
    model = DecoderModel(plan)
    assert {s.name: tuple(s.shape) for s in model.tensor_specs()} == tensor_shapes(raw)


def test_what_the_layers_keep_and_whose_rows_they_read():
    from velox_b200.models.decoder import DecoderModel
    from velox_b200.parts import PagedKV, PagedLatent
    model = DecoderModel(plan_of(CONFIGS["even"])[1])
    specs = model.cache_specs()
    # key heads [kv head, map] of 64 channels with ONE value head per kv head; rows kept for the borrower's longer window
    assert specs[0] == PagedKV(4, 64, 0, 0, 0, 2) and specs[2] == PagedKV(2, 128, 50, 64, 0, 1)
    assert specs[1] == PagedLatent(128, 70) and specs[3] is None and specs[4] == PagedLatent(72, 16)
    assert model.cache_sources() == [None, None, None, 1, None]
    odd = DecoderModel(plan_of(CONFIGS["odd"])[1])
    assert odd.cache_specs()[0] == PagedLatent(26, 19) and odd.cache_specs()[4] == PagedLatent(32, 0)
    assert odd.cache_sources() == [None, None, 0, None, None]
    # an owner whose borrower has no window keeps every row
    raw = copy.deepcopy(CONFIGS["odd"])
    del raw["layers"][2]["mixer"]["mask"]
    assert DecoderModel(plan_of(raw)[1]).cache_specs()[0] == PagedLatent(26, 0)


def test_pages_of_shared_values_and_of_windowed_rows_in_the_books():
    from velox_b200.cache.manager import CacheManager
    from velox_b200.models.decoder import DecoderModel
    model = DecoderModel(plan_of(CONFIGS["even"])[1])
    cache = CacheManager(model.cache_specs(), model.cache_sources(), page_size=16, num_pages=12, max_requests=2, max_blocks=12)
    assert sorted(g.window for g in cache.groups) == [0, 16, 50, 70]
    by_window = {g.window: g for g in cache.groups}
    assert by_window[16].kind.page_bytes(by_window[16].spec, 16, 2) == 72 * 16 * 2
    # a page of keys and values: 4 key heads of 64 and 2 value heads of 64; 2 key heads of 128 and 1 value head of 64
    assert by_window[0].kind.page_bytes(by_window[0].spec, 16, 2) == (4 * 64 + 2 * 64) * 16 * 2
    assert by_window[50].kind.page_bytes(by_window[50].spec, 16, 2) == (2 * 128 + 64) * 16 * 2
    assert by_window[70].kind.page_bytes(by_window[70].spec, 16, 2) == 128 * 16 * 2


@pytest.mark.parametrize("change,fault", [
    (lambda c: c.pop("vocab"), "missing key 'vocab'"),
    (lambda c: c["norm"].pop("eps"), "missing key 'norm.eps'"),
    (lambda c: c.update(streams=17), "streams must lie in 0 .. 16"),
    (lambda c: c["layers"][0].update(type="conv"), "layers[0].type 'conv'"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "heads (4) is not a multiple of kv_heads (3)"),
    (lambda c: c["layers"][1]["mixer"].update(diff=1.0), "diff must lie in [0, 1)"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims (7) must be even"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "rot.scaling.fast must be a number"),
    (lambda c: c["layers"][0]["mixer"].update(rot_dim=5), "rot_dim (5) must be even"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size must be a positive integer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "kv_from 3 must name an earlier latent layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from 1 must name an earlier latent layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=24), "kv_rank, rot_dim and rotation must equal that layer's"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), "mlp.kind 'gated' is not 'dense'"),
    (lambda c: c["layers"][0]["mixer"].update(q_rank=0), "q_rank must be a positive integer"),
])
def test_faults_of_a_configuration_are_named(change, fault):
    from velox_b200.config import ConfigError
    raw = copy.deepcopy(CONFIGS["odd"])
    change(raw)
    with pytest.raises(ConfigError) as e:
        plan_of(raw)
    assert fault in str(e.value)


def test_absent_keys_mean_not_there():
    raw = copy.deepcopy(CONFIGS["plain"])
    cfg, plan = plan_of(raw)
    assert cfg.streams == 0 and cfg.residual_mult == 1.0
    assert all(l.block == "hyper_connections" and l.block_params["streams"] == 0 for l in plan.layers)
    assert plan.final_norm.params["streams"] == 1
    assert plan.layers[0].feed_forward is None and set(plan.layers[0].norms) == {"mixer"}
    assert plan.layers[1].mixer.params["window"] == 0 and plan.layers[1].mixer.params["position"].params["scaling"] is None


def test_a_random_model_folder_can_be_written_and_read_back(tmp_path):
    from velox_b200.config import load_config
    from velox_b200.weights.random_init import write_random_model
    from velox_b200.weights.safetensors_io import SafetensorsFile
    cfg, _ = plan_of(CONFIGS["five"])
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=4)
    arch, back = load_config(folder)
    assert arch.name == "Fovenex" and back == cfg
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    assert set(f.keys()) == set(tensor_shapes(CONFIGS["five"]))
    mix = f.tensor("l0.hc1.mix").float().numpy()
    assert mix.shape == (5, 5) and np.abs(mix - np.eye(5)).max() < 0.3      # (the copies start nearly unmixed)
    f.close()


# -- the plain mechanisms on cases worked out by hand ----------------------------------------------------------------------

def test_layer_norm_takes_the_mean_off_and_the_variance_from_the_deviations():
    x = np.array([[1.0, 3.0, 5.0, 7.0]])
    got = F.layer_norm(x, np.array([1.0, 2.0, 1.0, 0.5]), 0.0)
    assert np.allclose(got, np.array([[-3.0, -2.0, 1.0, 1.5]]) / math.sqrt(5.0))
    assert np.allclose(F.layer_norm(x + 100.0, np.ones(4), 0.0), F.layer_norm(x, np.ones(4), 0.0))


def test_the_window_counts_the_query_itself():
    p = F.masked_softmax(np.zeros((5, 5)), 2)
    assert np.allclose(p[3], [0, 0, 0.5, 0.5, 0]) and np.allclose(p[0], [1, 0, 0, 0, 0])
    assert np.allclose(F.masked_softmax(np.zeros((3, 3)), 1), np.eye(3))
    assert np.allclose(F.masked_softmax(np.zeros((3, 3)))[2], [1 / 3] * 3)


def test_stretched_frequencies_keep_the_fast_pairs_and_divide_the_slow_ones():
    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}}
    f, mag = F.rotary_frequencies(rot)
    plain, one = F.rotary_frequencies({"base": 10000.0, "dims": 16})
    # pair i turns 1024 f_i / (2 pi) times in 1024 positions: 163 (i = 0), 51.5, 16.3, 5.2, 1.6, 0.5, ...
    # lo = floor(16 ln(1024 / (64 pi)) / (2 ln 1e4)) = 1, hi = ceil(16 ln(1024 / (2 pi)) / (2 ln 1e4)) = 5
    assert one == 1.0 and abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    assert np.allclose(f[:2], plain[:2]) and np.allclose(f[5:], plain[5:] / 4.0)
    assert np.allclose(f[3], plain[3] / 4.0 * 0.5 + plain[3] * 0.5)
    x = np.zeros((1, 1, 16))
    x[0, 0, 0] = 1.0
    turned = F.rotate_half(x, [3], rot)
    assert np.allclose(turned[0, 0, [0, 8]], [mag * math.cos(3.0), mag * math.sin(3.0)]) and np.allclose(np.delete(turned[0, 0], [0, 8]), 0.0)


def test_lambda_comes_from_the_four_vectors_and_equal_maps_with_lambda_one_leave_nothing():
    rng = np.random.default_rng(0)
    T, E, H, D, Dv = 6, 8, 2, 4, 4
    m = {"heads": H, "kv_heads": 1, "dim": D, "vdim": Dv, "scale": 0.5, "diff": 0.2}
    P = {"q": rng.normal(size=(H * 2 * D, E)), "k": rng.normal(size=(2 * D, E)), "v": rng.normal(size=(Dv, E)), "o": np.eye(E)[:, :H * Dv],
         "q.norm": np.ones(D), "k.norm": np.ones(D), "g": np.zeros((H, E)),
         "lq1": np.full(D, 0.5), "lk1": np.full(D, 0.5), "lq2": np.full(D, 0.5), "lk2": np.full(D, 0.5)}
    h = rng.normal(size=(T, E))
    # lambda = e^1 - e^1 + 0.2; the first position sees one key: both maps are its value, o = 0.8 v, normed to unit size
    out = F.differential_attention(h, P, m, np.arange(T), 1e-12).reshape(T, H, Dv)
    v0 = h[0] @ P["v"].T
    assert np.allclose(out[0, 0], F.unit_rms(v0, 1e-12) * 0.8 * 0.5) and np.allclose(out[0, 0], out[0, 1])
    # equal maps (map 2's projections copied from map 1's) and lambda = e^(ln 2) - e^0 + 0 = 1: the difference vanishes
    P["q"] = P["q"].reshape(H, 2, D, E)[:, [0, 0]].reshape(H * 2 * D, E)
    P["k"] = P["k"].reshape(1, 2, D, E)[:, [0, 0]].reshape(2 * D, E)
    P["lq1"] = P["lk1"] = np.full(D, math.sqrt(math.log(2.0) / D))
    P["lq2"] = np.zeros(D)
    out = F.differential_attention(h, P, dict(m, diff=0.0), np.arange(T), 1e-6)
    assert np.abs(out).max() < 1e-9


def test_one_copy_with_unit_mixing_is_the_plain_residual_layer():
    cfg = copy.deepcopy(CONFIGS["plain"])
    w = lively_weights(cfg, 5)
    toks = [3, 9, 4, 4, 60, 1, 17]
    want = F.forward(cfg, w, toks)
    one = dict(cfg, streams=1)
    w1 = dict(w)
    for i, lay in enumerate(cfg["layers"]):
        for q in ["1"] + (["2"] if lay.get("mlp") is not None else []):
            w1["l%d.hc%s.in" % (i, q)], w1["l%d.hc%s.out" % (i, q)], w1["l%d.hc%s.mix" % (i, q)] = np.ones(1), np.ones(1), np.ones((1, 1))
    assert np.allclose(F.forward(one, w1, toks), want)
    # two copies that never mix and are read half and half: the same again
    two = dict(cfg, streams=2)
    w2 = dict(w)
    for i, lay in enumerate(cfg["layers"]):
        for q in ["1"] + (["2"] if lay.get("mlp") is not None else []):
            w2["l%d.hc%s.in" % (i, q)], w2["l%d.hc%s.out" % (i, q)], w2["l%d.hc%s.mix" % (i, q)] = np.full(2, 0.5), np.ones(2), np.eye(2)
    layers = []
    assert np.allclose(F.forward(two, w2, toks, layers_out=layers), want) and len(layers) == 3


def test_borrowed_rows_are_the_owners_and_the_window_is_the_borrowers():
    cfg = copy.deepcopy(CONFIGS["plain"])
    w = lively_weights(cfg, 6)
    toks = list(range(30))
    base = F.forward(cfg, w, toks)
    # the owner's projection changes the borrower's keys ...
    w2 = dict(w)
    w2["l0.mix.dkv"] = w["l0.mix.dkv"][::-1].copy()
    assert np.abs(F.forward(cfg, w2, toks) - base).max() > 1e-3
    # ... and a window on the borrower alone changes late rows and not the first ones
    cfg2 = copy.deepcopy(cfg)
    cfg2["layers"][2]["mixer"]["mask"] = {"size": 4}
    got = F.forward(cfg2, w, toks)
    assert np.allclose(got[:4], base[:4]) and np.abs(got[10:] - base[10:]).max() > 1e-4


def test_greedy_generation_appends_the_most_likely_token():
    cfg = CONFIGS["ones"]
    w = lively_weights(cfg, 2)
    out = F.greedy_generate(cfg, w, [5, 6, 7], 3)
    assert out[0] == int(np.argmax(F.forward(cfg, w, [5, 6, 7])[-1])) and len(out) == 3
    assert out[1] == int(np.argmax(F.forward(cfg, w, [5, 6, 7, out[0]])[-1]))
