"""Small Fovenex configurations and lively random weights for the tests.

The weights are not the package's random-model weights (N(0, 0.02) everywhere would leave every softmax flat and every
gate at one half): matrices are N(0, gain / sqrt(inputs)), the mixing of the stream's copies is the identity plus noise,
so that a wrong key, a window that is one token off, borrowed rows that were not borrowed or a copy of the stream that was
mixed the wrong way round moves the logits by far more than rounding does.  Everything is rounded to bfloat16 before it
is written, so that the engine in either precision and the plain implementation read the same numbers.
"""
import json
import os

import numpy as np
import torch

import plain_fovenex as F


def dense(ff):
    return {"kind": "dense", "ff": ff}


def attention(heads, kv_heads, dim, vdim, scale, diff, rot=None, scaling=None, window=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, q_rank=None, window=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if q_rank:
        m["q_rank"] = q_rank
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def config(vocab, width, layers, eps=1e-5, streams=None, residual_mult=None):
    cfg = {"architecture": "Fovenex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    if residual_mult is not None:
        cfg["residual_mult"] = residual_mult
    return cfg


# sizes no fast kernel takes: a width that is no multiple of 16, three copies of the stream, heads of 10, 12 and 20 channels,
# rotations of a part of a head with stretched frequencies, values of another size than keys, a latent row of 26 elements, a
# window shorter than a page, a layer that borrows rows and looks further back than their owner, a layer without a
# feed-forward, a latent layer without a query latent and without a window
ODD = config(97, 72, [
    latent(3, 12, 6, 10, 20, 0.3, 1000.0, q_rank=14, window=7, mlp=dense(40)),
    attention(4, 2, 10, 12, 0.5, 0.25, rot=(300.0, 6), scaling=(4.0, 16, 4.0, 1.0)),
    latent(2, 8, 6, 14, 20, 0.35, 1000.0, q_rank=9, window=19, kv_from=0, mlp=dense(24)),
    attention(3, 3, 20, 20, 0.35, 0.4, rot=(50.0, 20), mlp=dense(32)),
    latent(2, 16, 8, 16, 24, 0.25, 100.0, mlp=dense(24)),
], streams=3, residual_mult=0.6)

# sizes the tensor-core kernels take (pages of 16): differential attention with keys of 64 and 128, one of them under a
# window; latent layers whose raised keys and values have 96 + 32, 128 + 64 and 64 + 64 channels, windows that end inside
# pages and blocks of raised rows, a window of exactly one page, a borrower with a longer window than the rows' owner
EVEN = config(160, 128, [
    attention(4, 2, 64, 64, 0.25, 0.2, rot=(10000.0, 32), scaling=(2.0, 64, 16.0, 1.0), mlp=dense(96)),
    latent(4, 32, 64, 32, 64, 0.18, 20000.0, q_rank=48, window=40, mlp=dense(64)),
    attention(2, 1, 128, 64, 0.18, 0.35, rot=(500.0, 128), window=50),
    latent(2, 64, 64, 64, 64, 0.15, 20000.0, q_rank=32, window=70, kv_from=1, mlp=dense(64)),
    latent(3, 32, 32, 64, 40, 0.2, 700.0, q_rank=24, window=16, mlp=dense(48)),
], streams=2, residual_mult=0.8)

# one stream without mixing tensors and without a multiplier; no stretched frequencies, no windows
PLAIN = config(90, 64, [
    latent(2, 16, 8, 16, 24, 0.25, 100.0, q_rank=12),
    attention(2, 2, 16, 16, 0.4, 0.3, rot=(100.0, 16), mlp=dense(48)),
    latent(2, 16, 8, 24, 24, 0.25, 100.0, q_rank=12, kv_from=0, mlp=dense(32)),
])

# what other configurations make larger: one copy of the stream WITH mixing tensors, one head, one key/value head, a window
# of one position, a difference weight of zero, a multiplier above one, a query latent wider than the width
ONES = config(50, 48, [
    attention(1, 1, 16, 8, 0.5, 0.0, rot=(20.0, 16), window=1, mlp=dense(16)),
    latent(1, 8, 4, 8, 12, 0.5, 30.0, q_rank=56, window=1, mlp=dense(16)),
    latent(1, 8, 4, 8, 12, 0.5, 30.0, q_rank=5, window=2, kv_from=1),
], streams=1, residual_mult=1.3)

# five copies of the stream (no kernel is specialised for that many), attention first, no feed-forward anywhere but the end
FIVE = config(64, 40, [
    attention(2, 1, 12, 20, 0.4, 0.5, rot=(1000.0, 4), scaling=(8.0, 8, 2.0, 0.5)),
    latent(5, 8, 8, 8, 16, 0.3, 500.0, q_rank=16, window=33),
    attention(6, 2, 8, 8, 0.6, 0.1, mlp=dense(20)),
], streams=5, residual_mult=0.5)

CONFIGS = {"odd": ODD, "even": EVEN, "plain": PLAIN, "ones": ONES, "five": FIVE}


def drawn_config(seed):
    """A configuration drawn from `seed`: two to six layers of either kind in any order, sizes from lists that hold what
    every kernel takes and what none does, windows of 1 to 200 positions or none, rows borrowed from any earlier owner,
    1 to 6 copies of the stream or a plain one."""
    rng = np.random.default_rng(5000 + seed)
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    width = pick([64, 96, 136, 200, 256])

    def ff():
        return None if rng.random() < 0.2 else dense(pick([32, 72, 128]))

    def att():
        D, G = pick([16, 32, 64, 128, 40, 24]), pick([1, 2, 3])
        H = G * pick([1, 2, 4])
        Dv = pick([D, 32, 64, 128]) if D in (64, 128) else pick([D, 20])
        dims = pick([D, D // 2 // 2 * 2])
        rot = None if rng.random() < 0.15 else (pick([1e4, 5e5, 100.0]), dims)
        scaling = None if rot is None or rng.random() < 0.4 else (pick([2.0, 4.0, 1.5]), pick([32, 256, 2048]), pick([32.0, 8.0]), pick([1.0, 2.0]))
        return attention(H, G, D, Dv, pick([1.0, 1.5]) / np.sqrt(D) * 2.0, pick([0.0, 0.1, 0.3, 0.6]), rot, scaling,
                         pick([None, None, 1, 30, 64, 100]), ff())

    owners = []

    def lat(i):
        window = pick([None, 1, 15, 16, 48, 96, 200])
        if owners and rng.random() < 0.45:
            j, (D, R, C, base) = owners[int(rng.integers(0, len(owners)))]
            D = pick([D, 32, 64])
            return latent(pick([1, 2, 5]), D, R, pick([32, 64, 20]), C, pick([0.1, 0.2]), base, pick([None, 24, 80]), window, j, ff())
        D, R = pick([(32, 32), (64, 64), (128, 64), (16, 16), (24, 8), (96, 32), (32, 64)])
        C, base = pick([24, 40, 96, 136, 264]), pick([100.0, 1e4, 5e5])
        owners.append((i, (D, R, C, base)))
        return latent(pick([1, 2, 5, 8]), D, R, pick([32, 64, 128, 20, D]), C, pick([0.1, 0.2]), base, pick([None, 24, 80, 136]), window, None, ff())

    n = int(rng.integers(2, 7))
    layers = [att() if rng.random() < 0.5 else lat(i) for i in range(n)]
    return config(pick([64, 300]), width, layers, streams=pick([None, 1, 2, 3, 4, 6]), residual_mult=pick([None, 0.5, 0.7, 1.0]))


def tensor_shapes(cfg):
    E, n, out = cfg["width"], int(cfg.get("streams") or 0), {}
    out["embed"] = (cfg["vocab"], E)
    for i, lay in enumerate(cfg["layers"]):
        p, m = "l%d." % i, lay["mixer"]
        subs = ["1"] + (["2"] if lay.get("mlp") is not None else [])
        for q in subs:
            out[p + "norm" + q] = (E,)
            out[p + "ls" + q] = (E,)
            if n:
                out.update({p + "hc%s.in" % q: (n,), p + "hc%s.out" % q: (n,), p + "hc%s.mix" % q: (n, n)})
        H = m["heads"]
        if lay["type"] == "attention":
            G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * 2 * D, E), p + "mix.k": (G * 2 * D, E), p + "mix.v": (G * Dv, E), p + "mix.o": (E, H * Dv),
                        p + "mix.q.norm": (D,), p + "mix.k.norm": (D,), p + "mix.g": (H, E)})
            out.update({p + "mix." + x: (D,) for x in ("lq1", "lk1", "lq2", "lk2")})
        else:
            D, R, Dv, C = m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            if m.get("q_rank"):
                out.update({p + "mix.dq": (m["q_rank"], E), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (H * (D + R), m["q_rank"])})
            else:
                out[p + "mix.q"] = (H * (D + R), E)
            if m.get("kv_from") is None:
                out.update({p + "mix.dkv": (C + R, E), p + "mix.dkv.norm": (C,)})
            out.update({p + "mix.uk": (H * D, C), p + "mix.uv": (H * Dv, C), p + "mix.g": (H * Dv, E), p + "mix.o": (E, H * Dv)})
        f = lay.get("mlp")
        if f is not None:
            out.update({p + "mlp.up": (f["ff"], E), p + "mlp.down": (E, f["ff"])})
    out["final.norm"] = (E,)
    out["head"] = (cfg["vocab"], E)
    return out


def lively_weights(cfg, seed):
    """{name: float64 array of bfloat16-representable values}."""
    rng = np.random.default_rng(seed)
    n = int(cfg.get("streams") or 0)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last == "mix" and len(shape) == 2 and ".hc" in name:
            x = np.eye(n) * 0.8 + 0.25 * rng.normal(size=shape)
        elif last == "in" and ".hc" in name:
            x = (1.0 + 0.4 * rng.normal(size=shape)) / np.sqrt(n)
        elif last == "out" and ".hc" in name:
            x = 1.0 + 0.4 * rng.normal(size=shape)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            x = rng.normal(size=shape) / np.sqrt(8.0 * shape[0])   # (lambda stays within some tenths of `diff`)
        elif len(shape) == 1:
            x = 1.0 + 0.2 * rng.normal(size=shape)        # norm weights and layer scales
        elif name == "embed":
            x = rng.normal(0.0, 1.0, shape)
        else:
            gain = 2.0 if last in ("q", "k", "g", "dq") else 1.0
            x = rng.normal(0.0, gain / np.sqrt(shape[1]), shape)
        w[name] = F.store_bfloat16(x)
    return w


def write_model(folder, cfg, w):
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: torch.from_numpy(np.ascontiguousarray(v)).to(torch.bfloat16) for k, v in w.items()},
              os.path.join(folder, "model.safetensors"))
    return folder


def shifted_store(f):
    """Another realisation of the same rounding: the values are rounded a little beside themselves (x f rounded, then
    taken back, f near one), so every value falls elsewhere between its two neighbours; the error has the same size."""
    return lambda x: F.store_bfloat16(np.asarray(x) * f) / f


STORES = (F.store_bfloat16, shifted_store(1.0 + 2.0 ** -9), shifted_store(1.0 - 3.0 * 2.0 ** -10), shifted_store(1.0 + 5.0 * 2.0 ** -11))


class Oracle:
    """Exact logits [T, V] of one whole sequence and, per row, what rounding every stored activation to bfloat16 costs
    (root-mean-square distance from the exact row; the largest of four realisations of the rounding, since a softmax near a
    tie scatters a single one)."""

    def __init__(self, cfg, w, tokens):
        self.exact = F.forward(cfg, w, tokens)
        costs = []
        for store in STORES:
            rounded = F.forward(cfg, w, tokens, store=store)
            costs.append(np.sqrt(np.mean(np.square(rounded - self.exact), axis=1)))
        self.cost = np.max(np.stack(costs), axis=0)

    def __getitem__(self, row):
        return self.exact[row]


def compare(got, oracles_rows, dtype, what, judge):
    """`oracles_rows`: [(oracle, first row, one past the last)] in the order of `got`'s rows."""
    from helpers import assert_close
    want = np.concatenate([o.exact[a:b] for o, a, b in oracles_rows])
    cost = np.concatenate([o.cost[a:b] for o, a, b in oracles_rows])
    assert got.shape == want.shape and np.isfinite(got).all(), what
    assert_close(got, want, dtype, what, cost=cost, judge=judge)
