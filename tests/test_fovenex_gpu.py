"""Fovenex in the engine against the plain implementation (`plain_fovenex.py`): the stream after every layer, whole
prompts, prompts against token-by-token decoding, portions down to two tokens, unequal requests in one batch against each
alone, pages that the windows give back and that are used again, long decoding that carries every window over decoded
tokens, other sizes, and greedy generation through the engine's own entry point and scheduler; in 32-bit (every value
within 1e-4) and in bfloat16 (by what rounding costs).  The cache pool is filled with NaN first."""
import numpy as np
import pytest

import plain_fovenex as F
from fovenex_helpers import CONFIGS, Oracle, compare, drawn_config, lively_weights, write_model
from helpers import RoundingJudge, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("fovenex")
    out = {}
    for name, cfg in CONFIGS.items():
        w = lively_weights(cfg, seed=17 + len(name))
        out[name] = (cfg, w, write_model(str(root / name), cfg, w))
    return out


def tokens_of(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


def engine_for(folder, dtype, pool_tokens, slots=4, page_size=16, graphs=True):
    from velox_b200 import Engine, EngineConfig
    return Engine(folder, EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=pool_tokens,
                                       max_running_requests=slots, max_model_len=pool_tokens, cuda_graphs=graphs),
                  poison_cache=True)


def run(engine, steps):
    """steps: [[(request, tokens, want)], ...] with ("end", request) entries to give a request's cache back.
    Returns the logits of every step that wanted some."""
    from velox_b200.engine import StepEntry
    out = []
    for step in steps:
        entries = []
        for e in step:
            if e[0] == "end":
                continue
            if not engine.cache.has_request(e[0]):
                assert engine.cache.add_request(e[0]) is not None
            entries.append(StepEntry(e[0], e[1], e[2]))
        logits = engine.run_step(entries) if entries else None
        out.append(None if logits is None else logits.cpu().numpy())
        for e in step:
            if e[0] == "end":
                engine.cache.release(e[1])
    engine.cache.check()
    return out


def portions(tokens, sizes, name):
    steps, at, k = [], 0, 0
    while at < len(tokens):
        s = min(sizes[k % len(sizes)], len(tokens) - at)
        steps.append([(name, tokens[at:at + s], list(range(s)))])
        at += s
        k += 1
    return steps


@pytest.mark.parametrize("name", ["odd", "even", "plain", "five"])
def test_the_sum_of_the_streams_after_every_layer(models, name):
    """In 32 bits, through the model's own blocks in an ordinary step: what the plain implementation has after every layer
    (the sum of the copies of the stream), whether the prompt comes whole or in two portions."""
    cfg, w, folder = models[name]
    toks = tokens_of(cfg, 29, 2)
    want = []
    F.forward(cfg, w, toks, layers_out=want)
    engine = engine_for(folder, "float32", 64, graphs=False)
    E = cfg["width"]
    seen = []
    engine.runner.model.probe = lambda place, x: seen.append((place, x.view(x.shape[0], -1, E).sum(1).cpu().numpy().astype(np.float64)))
    run(engine, [[("a", toks, [])], [("end", "a")], [("b", toks[:11], [])], [("b", toks[11:], [])]])
    runs = len(cfg["layers"])
    assert len(seen) == 3 * runs == 3 * len(want)
    for k, (place, got) in enumerate(seen[:runs]):
        assert place == k and np.abs(got - want[k]).max() <= 1e-4 * max(1.0, np.abs(want[k]).max()), "after layer %d" % k
    for k in range(runs):
        got = np.concatenate([seen[runs + k][1], seen[2 * runs + k][1]])
        assert np.abs(got - want[k]).max() <= 1e-4 * max(1.0, np.abs(want[k]).max()), "in two portions, after layer %d" % k


@pytest.mark.parametrize("name,dtype,length", [("odd", "float32", 150), ("even", "float32", 150), ("plain", "float32", 100),
                                               ("odd", "bfloat16", 150), ("even", "bfloat16", 150), ("plain", "bfloat16", 100),
                                               ("ones", "float32", 60), ("ones", "bfloat16", 60), ("five", "float32", 120),
                                               ("five", "bfloat16", 120)])
def test_whole_prompts_portions_and_decoding_agree_with_the_plain_implementation(models, name, dtype, length):
    cfg, w, folder = models[name]
    toks = tokens_of(cfg, length, 1)
    oracle = Oracle(cfg, w, toks)
    judge = RoundingJudge.of([oracle], "fovenex %s %s" % (name, dtype))
    engine = engine_for(folder, dtype, 160 + 64)
    ways = {
        "whole": [[("a", toks, list(range(len(toks))))]],
        "prompt then one by one": [[("a", toks[:length * 2 // 5], list(range(length * 2 // 5)))]]
                                  + [[("a", [t], [0])] for t in toks[length * 2 // 5:]],
        "token by token from the start": [[("a", [t], [0])] for t in toks[:50]],
        "portions 2 3 64 5 1 16 2": portions(toks, [2, 3, 64, 5, 1, 16, 2], "a"),
        "portions 17 31": portions(toks, [17, 31], "a"),
        "portions 2": portions(toks[:48], [2], "a"),
    }
    for what, steps in ways.items():
        got = np.concatenate([g for g in run(engine, steps + [[("end", "a")]]) if g is not None])
        compare(got, [(oracle, 0, len(got))], dtype, "%s, %s" % (name, what), judge)
    if dtype != "float32":
        judge.finish()


@pytest.mark.parametrize("seed", range(8))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    """Other sizes, layer orders, windows, numbers of copies of the stream and borrowings than the fixed configurations
    have: a request of 230 tokens whole, in portions of 2 to 130 tokens, as a prompt followed by single tokens, and three
    unequal requests that join and leave a batch."""
    cfg = drawn_config(seed)
    w = lively_weights(cfg, seed=seed)
    folder = write_model(str(tmp_path / "drawn"), cfg, w)
    a, b, c = [tokens_of(cfg, n, seed * 7 + i) for i, n in enumerate((230, 90, 33))]
    oa, ob, oc = Oracle(cfg, w, a), Oracle(cfg, w, b), Oracle(cfg, w, c)
    judge = RoundingJudge.of([oa, ob, oc], "fovenex drawn %d %s" % (seed, dtype))
    engine = engine_for(folder, dtype, 416)
    ways = {"whole": [[("a", a, list(range(len(a))))]],
            "portions": portions(a, [2, 64, 5, 1, 16, 130], "a"),
            "prompt then single tokens": [[("a", a[:150], list(range(150)))]] + [[("a", [t], [0])] for t in a[150:]]}
    for what, steps in ways.items():
        got = np.concatenate([g for g in run(engine, steps + [[("end", "a")]]) if g is not None])
        compare(got, [(oa, 0, len(got))], dtype, "drawn %d, %s" % (seed, what), judge)
    steps = [[("a", a[:40], list(range(40))), ("b", b[:60], list(range(60)))],
             [("a", a[40:41], [0]), ("b", b[60:90], list(range(30))), ("c", c[:20], list(range(20)))],
             [("a", a[41:100], list(range(59))), ("c", c[20:21], [0])],
             [("end", "b"), ("c", c[21:33], list(range(12))), ("a", a[100:101], [0])]]
    rows = [[(oa, 0, 40), (ob, 0, 60)], [(oa, 40, 41), (ob, 60, 90), (oc, 0, 20)], [(oa, 41, 100), (oc, 20, 21)],
            [(oc, 21, 33), (oa, 100, 101)]]
    got = [g for g in run(engine, steps + [[("end", "a"), ("end", "c")]]) if g is not None]
    for g, r in zip(got, rows):
        compare(g, r, dtype, "drawn %d, a batch that requests join and leave" % seed, judge)
    if dtype != "float32":
        judge.finish()


@pytest.mark.parametrize("name,dtype", [("even", "float32"), ("even", "bfloat16"), ("odd", "float32"), ("five", "bfloat16")])
def test_unequal_requests_in_one_batch_and_reused_pages(models, name, dtype):
    """Four live requests at most in a pool of 20 pages: requests of 1 to 130 tokens come, go on beside one another in
    portions and single tokens, are left out of steps, end, and their pages go to the next."""
    cfg, w, folder = models[name]
    lens = {"a": 130, "b": 37, "c": 1, "d": 64, "e": 90, "f": 2, "g": 70}
    toks = {k: tokens_of(cfg, n, 100 + i) for i, (k, n) in enumerate(lens.items())}
    oracle = {k: Oracle(cfg, w, t) for k, t in toks.items()}
    judge = RoundingJudge.of(oracle.values(), "fovenex mixed %s %s" % (name, dtype))
    engine = engine_for(folder, dtype, 20 * 16, slots=4)
    at = {k: 0 for k in toks}

    def take(k, n):
        lo = at[k]
        hi = min(lo + n, len(toks[k]))
        at[k] = hi
        return (k, toks[k][lo:hi], list(range(hi - lo)), lo)

    plan = [
        [("a", 33), ("b", 7), ("c", 1)], [("end", "c")],
        [("a", 1), ("b", 30), ("d", 2)], [("end", "b")],
        [("a", 64), ("d", 1), ("f", 2)], [("end", "f")],
        [("d", 61), ("e", 17)], [("end", "d")],
        [("a", 2), ("e", 1), ("g", 48)],
        [("e", 72)], [("end", "e")],
        [("a", 30), ("g", 1)], [("end", "a")],
        [("g", 21)], [("end", "g")],
    ]
    for step in plan:
        if step[0][0] == "end":
            run(engine, [[step[0]]])
            continue
        entries = [take(k, n) for k, n in step]
        got = run(engine, [[(k, t, want) for k, t, want, _ in entries]])[0]
        compare(got, [(oracle[k], lo, lo + len(t)) for k, t, _, lo in entries], dtype, "step %s" % (step,), judge)
    assert all(at[k] == len(toks[k]) for k in toks)
    assert all(g.allocator.num_free == g.allocator.num_pages for g in engine.cache.groups)
    if dtype != "float32":
        judge.finish()


def test_the_windows_give_pages_back_and_the_rows_a_borrower_needs_stay(models):
    """`even`: the rows of layer 1 (window 40) are read by layer 3 with a window of 70, so they are kept for 70 positions; layer
    4 keeps 16; the attention under a window keeps 50; the other attention keeps everything.  After 300 positions a
    request holds no more pages of a group than its longest window needs, and the logits are still right."""
    cfg, w, folder = models["even"]
    toks = tokens_of(cfg, 300, 5)
    oracle = Oracle(cfg, w, toks)
    engine = engine_for(folder, "float32", 320)
    steps = portions(toks[:280], [37, 64, 3], "a") + [[("a", [t], [0])] for t in toks[280:]]
    got = np.concatenate([g for g in run(engine, steps) if g is not None])
    assert_close(got, oracle.exact, "float32", "pages given back as the windows pass")
    held = {}
    for g, table in zip(engine.cache.groups, engine.cache.requests["a"].tables):
        held[g.window] = sum(1 for p in table if p >= 0)
    assert sorted(held) == [0, 16, 50, 70]
    assert held[0] == 19 and held[70] <= 6 and held[50] <= 5 and held[16] <= 2
    run(engine, [[("end", "a")]])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_request_beside_short_ones_in_a_pool_made_for_what_is_live(models, dtype):
    """700 tokens in portions that end inside pages, beside a request that decodes token by token, ends, and whose pages a
    third one takes."""
    cfg, w, folder = models["even"]
    toks = {"a": tokens_of(cfg, 700, 71), "b": tokens_of(cfg, 40, 72), "c": tokens_of(cfg, 60, 73)}
    oracle = {k: Oracle(cfg, w, t) for k, t in toks.items()}
    judge = RoundingJudge.of(oracle.values(), "fovenex long request %s" % dtype)
    engine = engine_for(folder, dtype, 704 + 64 + 64, slots=2)
    at = {k: 0 for k in toks}

    def take(k, n):
        lo = at[k]
        hi = min(lo + n, len(toks[k]))
        at[k] = hi
        return (k, toks[k][lo:hi], list(range(hi - lo)), lo)

    plan = [[("a", 128), ("b", 21)], [("a", 29), ("b", 1)], [("a", 2), ("b", 1)], [("a", 300), ("b", 1)]]
    plan += [[("a", 1), ("b", 1)] for _ in range(16)] + [[("end", "b")], [("a", 1), ("c", 33)], [("a", 224), ("c", 1)]]
    plan += [[("c", 2)], [("c", 24)], [("end", "a")], [("end", "c")]]
    for step in plan:
        if step[0][0] == "end":
            run(engine, [[step[0]]])
            continue
        entries = [take(k, n) for k, n in step]
        got = run(engine, [[(k, t, want) for k, t, want, _ in entries]])[0]
        compare(got, [(oracle[k], lo, lo + len(t)) for k, t, _, lo in entries], dtype, "step %s" % (step,), judge)
    assert all(at[k] == len(toks[k]) for k in toks)
    assert all(g.allocator.num_free == g.allocator.num_pages for g in engine.cache.groups)
    if dtype != "float32":
        judge.finish()


@pytest.mark.parametrize("name,dtype", [("even", "float32"), ("even", "bfloat16"), ("odd", "bfloat16")])
def test_long_decoding(models, name, dtype):
    """360 tokens one by one after a short prompt: every window passes over decoded tokens; the captured step is replayed."""
    cfg, w, folder = models[name]
    toks = tokens_of(cfg, 380, 9 + len(name))
    oracle = Oracle(cfg, w, toks)
    judge = RoundingJudge.of([oracle], "fovenex long decoding %s %s" % (name, dtype))
    engine = engine_for(folder, dtype, 384)
    steps = [[("a", toks[:20], list(range(20)))]] + [[("a", [t], [0])] for t in toks[20:]]
    got = np.concatenate(run(engine, steps))
    compare(got, [(oracle, 0, len(toks))], dtype, "long decoding", judge)
    if dtype != "float32":
        judge.finish()


def test_two_requests_decode_side_by_side_in_captured_steps(models):
    cfg, w, folder = models["odd"]
    ta, tb = tokens_of(cfg, 60, 21), tokens_of(cfg, 45, 22)
    oa, ob = Oracle(cfg, w, ta), Oracle(cfg, w, tb)
    engine = engine_for(folder, "float32", 128)
    run(engine, [[("a", ta[:30], []), ("b", tb[:15], [])]])
    for i in range(30):
        got = run(engine, [[("a", [ta[30 + i]], [0]), ("b", [tb[15 + i]], [0])]])[0]
        assert_close(got, np.stack([oa[30 + i], ob[15 + i]]), "float32", "decode step %d" % i)


def test_greedy_generation_through_the_engine(models):
    from velox_b200 import SamplingParams
    cfg, w, folder = models["odd"]
    engine = engine_for(folder, "float32", 256)
    prompts = [tokens_of(cfg, 19, 31), tokens_of(cfg, 3, 32), tokens_of(cfg, 40, 33)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0))
    for p, o in zip(prompts, outs):
        assert o == F.greedy_generate(cfg, w, p, 12)
    # a second round on the same engine: the pages of the first are used again
    outs2 = engine.generate(prompts[::-1], SamplingParams(max_tokens=5, temperature=0.0))
    assert outs2 == [o[:5] for o in outs[::-1]]


def test_generation_with_chunked_prompts_and_a_small_batch_budget(models):
    from velox_b200 import Engine, EngineConfig, SamplingParams
    cfg, w, folder = models["even"]
    engine = Engine(folder, EngineConfig(dtype="float32", page_size=16, max_cache_tokens=512, max_running_requests=3,
                                         max_model_len=256, max_batch_tokens=24, chunk_size=16))
    prompts = [tokens_of(cfg, n, 40 + n) for n in (50, 7, 33, 21)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))
    for p, o in zip(prompts, outs):
        assert o == F.greedy_generate(cfg, w, p, 6)


def test_the_command_line_writes_and_runs_a_random_model(tmp_path):
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    (tmp_path / "c.json").write_text(json.dumps(CONFIGS["odd"]))
    out = subprocess.run([sys.executable, "-m", "velox_b200", "random-model", "--config", str(tmp_path / "c.json"),
                          "--model-dir", str(tmp_path / "m"), "--seed", "3"], cwd=root, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert json.loads(out.stdout.strip().splitlines()[-1])["architecture"] == "Fovenex"
    gen = subprocess.run([sys.executable, "-m", "velox_b200", "generate", "--model-dir", str(tmp_path / "m"),
                          "--prompt-tokens", "5,6,7,8", "--max-tokens", "4", "--dtype", "float32"],
                         cwd=root, capture_output=True, text=True)
    assert gen.returncode == 0, gen.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_trace_runner_replays_requests_through_a_small_pool(models, tmp_path, dtype):
    """bin/trace_run as a user starts it (its own process, a pool of 24 pages): five requests, at most four of them live,
    portions beside single tokens, a request left out of steps, pages used again."""
    from helpers import run_trace
    cfg, w, folder = models["even"]
    toks = {k: tokens_of(cfg, n, 60 + i) for i, (k, n) in enumerate({"p": 100, "q": 37, "r": 64, "s": 2, "t": 90}.items())}
    oracle = {k: Oracle(cfg, w, t) for k, t in toks.items()}
    at = {k: 0 for k in toks}
    steps, expect = [], []

    def step(parts, end=()):
        entries, rows = [], []
        for k, n in parts:
            lo, hi = at[k], min(at[k] + n, len(toks[k]))
            at[k] = hi
            entries.append({"id": k, "tokens": toks[k][lo:hi], "want": list(range(hi - lo))})
            rows.append((oracle[k], lo, hi))
        steps.append({"step": len(steps), "entries": entries, "end": list(end)})
        expect.append(rows)
    step([("p", 40), ("q", 36), ("r", 1)])
    step([("p", 1), ("q", 1), ("r", 63), ("s", 2)], end=["q", "r", "s"])
    step([("t", 33)])                          # ("p" is left out of this step)
    step([("p", 59), ("t", 1)], end=["p"])
    step([("t", 56)], end=["t"])
    got = run_trace(folder, dtype, steps, 24 * 16, str(tmp_path / "out"), vocab=cfg["vocab"])
    judge = RoundingJudge.of(oracle.values(), "fovenex trace runner %s" % dtype)
    for n, rows in enumerate(expect):
        compare(got[n], rows, dtype, "step %d" % n, judge)
    if dtype != "float32":
        judge.finish()
