"""Small Kapuvik configurations and lively random weights for the tests.

The weights are not the package's random-model weights (N(0, 0.02) everywhere would leave every softmax flat and
every gate at one half): matrices are N(0, gain / sqrt(inputs)), decay biases spread the decays between a fast and a
slow forgetting, so that a wrong key, a rotation of the wrong pairs, a lost state or a pass that skips its input moves the
logits by far more than rounding does.  Everything is rounded to bfloat16 before it is written, so that the engine in
either precision and the plain implementation read the same numbers.
"""
import json
import os

import numpy as np
import torch

import plain_kapuvik as K


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def side_by_side(left, right, left_scale=None, right_scale=None, mlp=None):
    m = {"left": left, "right": right}
    if left_scale is not None:
        m["left_scale"] = left_scale
    if right_scale is not None:
        m["right_scale"] = right_scale
    return {"type": "parallel", "mixer": m, "mlp": mlp}


def softmax_member(heads, kv_heads, dim, vdim, scale, softcap=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def retention_member(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim}}}


def gated(heads, dim, vdim, tau, rank, mlp=None):
    return {"type": "gla", "mlp": mlp, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}}


def config(vocab, width, layers, eps=1e-5, embedding_scale=None, logit_softcap=None, loop=None):
    cfg = {"architecture": "Kapuvik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if embedding_scale is not None:
        cfg["embedding"] = {"scale": embedding_scale}
    if logit_softcap is not None:
        cfg["logit_softcap"] = logit_softcap
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# sizes no fast kernel takes: a width that is no multiple of 16, heads of 20, 12, 10 and 18 channels; rotations of a part of
# a head only; two key/value heads for four query heads; values of another size than keys everywhere; a latent row of 26
# elements; a layer without a feed-forward; the middle layers gone through three times, starting after the first layer
ODD = config(101, 72, [
    gated(3, 20, 24, 7.0, 5, dense(40, 1.25)),
    latent(3, 12, 6, 10, 20, 0.3, 1000.0, dense(24, 2.0)),
    side_by_side(softmax_member(4, 2, 20, 12, 0.22, softcap=5.0, rot=(300.0, 8)),
                 retention_member(2, 10, 14, [0.9, 0.97], rot=(50.0, 6)), 0.7, 1.3, None),
    gated(2, 18, 10, 3.0, 4, dense(32, 0.75)),
], embedding_scale=1.5, logit_softcap=8.0, loop=(1, 3, 3))

# sizes the tensor-core kernels take (heads of 64 with values of 64, a latent row of 128 elements, pages of 16); the first two
# layers gone through twice; an attention without a bound on its scores and members without coefficients; a member without rotation
EVEN = config(160, 128, [
    side_by_side(softmax_member(4, 2, 64, 64, 0.12, softcap=20.0, rot=(10000.0, 64)),
                 retention_member(2, 64, 64, [0.98, 0.995], rot=(10000.0, 32)), 0.6, 0.9, dense(96, 1.5)),
    latent(4, 32, 64, 32, 64, 0.1, 20000.0, dense(64, 1.0)),
    gated(2, 64, 64, 12.0, 8, None),
    side_by_side(softmax_member(2, 1, 128, 64, 0.09, rot=(500.0, 32)), retention_member(4, 32, 32, [0.9, 0.95, 0.99, 1.0]),
                 mlp=dense(64, 3.0)),
], logit_softcap=12.0, loop=(0, 2, 2))

# no loop, no multiplier at the input, no bound on the logits, one layer of each kind, a single pass named as a loop elsewhere
PLAIN = config(90, 64, [
    latent(2, 16, 8, 16, 24, 0.25, 100.0, None),
    gated(2, 16, 16, 5.0, 3, dense(48, 1.0)),
    side_by_side(softmax_member(2, 2, 16, 16, 0.25, rot=(100.0, 16)), retention_member(2, 16, 16, [0.95, 0.9], rot=(100.0, 16)),
                 mlp=dense(32, 1.5)),
])

# sizes at the borders of the fast paths: a latent layer whose keys and values the tensor-core kernel takes but whose fused
# projection has rows of 180 elements (no multiple of 8: it goes the folded way), one that goes the raised way with values of
# another size than the first, linear attentions with heads of 72 and 136 channels (rows padded in shared memory), the whole
# model gone through twice
BORDERS = config(120, 96, [
    latent(2, 32, 32, 32, 20, 0.2, 3000.0, dense(40, 1.0)),
    gated(2, 72, 40, 9.0, 6, None),
    latent(3, 32, 32, 64, 40, 0.15, 700.0, dense(56, 2.5)),
    side_by_side(softmax_member(3, 1, 32, 32, 0.2, softcap=10.0, rot=(900.0, 16)),
                 retention_member(1, 136, 24, [0.97], rot=(200.0, 40)), 1.1, 0.4, dense(32, 1.0)),
], embedding_scale=0.75, logit_softcap=20.0, loop=(0, 4, 2))

CONFIGS = {"odd": ODD, "even": EVEN, "plain": PLAIN, "borders": BORDERS}


def drawn_config(seed):
    """A configuration drawn from `seed`: two to five layers of any kind in any order, sizes from lists that hold what every
    kernel takes and what none does (latent rows of 32 to 584 elements, 1 to 17 heads, keys of 16 to 200 channels, values of
    16 to 128), feed-forwards present or not, a loop over any run of layers one to three times, or none."""
    rng = np.random.default_rng(1000 + seed)
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    width = pick([64, 96, 136, 200, 256])

    def ff():
        return None if rng.random() < 0.15 else dense(pick([32, 72, 128]), pick([0.75, 1.5, 4.0]))

    def lat():
        D, R = pick([(32, 32), (64, 64), (128, 64), (16, 16), (24, 8), (96, 32), (32, 64), (192, 64)])
        Dv = pick([32, 64, 128, 20, D])
        return latent(pick([1, 2, 5, 8, 17]), D, R, Dv, pick([24, 40, 96, 136, 264, 520]), pick([0.1, 0.2]), pick([100.0, 1e4, 5e5]), ff())

    def gl():
        return gated(pick([1, 2, 6]), pick([16, 48, 64, 100, 144, 200]), pick([16, 32, 40, 64, 72]), pick([1.0, 4.0, 16.0]), pick([2, 8]), ff())

    def par():
        D, G = pick([16, 32, 64, 128, 40]), pick([1, 2])
        H = G * pick([1, 2, 3, 4])
        Dv = pick([D, 32, 64]) if D in (64, 128) else D
        left = softmax_member(H, G, D, Dv, pick([0.1, 0.2]), softcap=pick([None, 5.0, 30.0]), rot=(pick([1e4, 2e4]), pick([D, D // 2])))
        Dr, Hr = pick([16, 32, 64, 136]), pick([1, 3, 6])
        right = retention_member(Hr, Dr, pick([16, 32, 24]), [1.0 - 2.0 ** -float(rng.integers(3, 10)) for _ in range(Hr)],
                                 rot=None if rng.random() < 0.2 else (pick([1e4, 1e6]), pick([Dr, Dr // 2]) // 2 * 2))
        return side_by_side(left, right, pick([None, 0.8]), pick([None, 0.9]), ff())

    n = int(rng.integers(2, 6))
    layers = [pick([lat, gl, par])() for _ in range(n)]
    loop = None
    if rng.random() < 0.6:
        a = int(rng.integers(0, n))
        loop = (a, int(rng.integers(a + 1, n + 1)), int(rng.integers(1, 4)))
    return config(pick([64, 300]), width, layers, embedding_scale=pick([None, 0.5]), logit_softcap=pick([None, 15.0]), loop=loop)


def tensor_shapes(cfg):
    E, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], E)
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], E)
    for i, lay in enumerate(cfg["layers"]):
        p, m = "l%d." % i, lay["mixer"]
        out[p + "norm1"] = (E,)
        if lay["type"] == "parallel":
            a, b = m["left"], m["right"]
            out.update({p + "mix.left.q": (a["heads"] * a["dim"], E), p + "mix.left.k": (a["kv_heads"] * a["dim"], E),
                        p + "mix.left.v": (a["kv_heads"] * a["vdim"], E), p + "mix.left.o": (E, a["heads"] * a["vdim"]),
                        p + "mix.right.q": (b["heads"] * b["dim"], E), p + "mix.right.k": (b["heads"] * b["dim"], E),
                        p + "mix.right.v": (b["heads"] * b["vdim"], E), p + "mix.right.g": (b["heads"] * b["vdim"], E),
                        p + "mix.right.o": (E, b["heads"] * b["vdim"])})
        elif lay["type"] == "latent_attention":
            H = m["heads"]
            out.update({p + "mix.q": (H * (m["dim"] + m["rot_dim"]), E), p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], E),
                        p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * m["dim"], m["kv_rank"]),
                        p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.o": (E, H * m["vdim"])})
        else:
            H = m["heads"]
            out.update({p + "mix.q": (H * m["dim"], E), p + "mix.k": (H * m["dim"], E), p + "mix.v": (H * m["vdim"], E),
                        p + "mix.g": (H * m["vdim"], E), p + "mix.o": (E, H * m["vdim"]), p + "mix.norm": (m["vdim"],),
                        p + "mix.a1": (m["rank"], E), p + "mix.a2": (H * m["dim"], m["rank"]), p + "mix.a2.b": (H * m["dim"],)})
        f = lay.get("mlp")
        if f is not None:
            out.update({p + "mlp.gate": (f["ff"], E), p + "mlp.gate.b": (f["ff"],), p + "mlp.up": (f["ff"], E),
                        p + "mlp.up.b": (f["ff"],), p + "mlp.down": (E, f["ff"]), p + "mlp.down.b": (E,)})
    out["final.norm"] = (E,)
    out["head"] = (cfg["vocab"], E)
    return out


def lively_weights(cfg, seed):
    """{name: float64 array of bfloat16-representable values}."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name.endswith("a2.b"):
            x = rng.normal(1.5, 1.5, shape)               # decays from fast to slow
        elif name.endswith("dkv.norm") or name.endswith("mix.norm"):
            x = 1.0 + 0.2 * rng.normal(size=shape)        # plain weights
        elif name == "loop.step":
            x = 0.5 * rng.normal(size=shape)
        elif last == "b":
            x = 0.3 * rng.normal(size=shape)
        elif len(shape) == 1:
            x = 0.1 * rng.normal(size=shape)              # an offset: the multiplier is 1 + x
        elif name == "embed":
            x = rng.normal(0.0, 1.0, shape)
        else:
            gain = 2.0 if last in ("q", "k", "g", "a1", "a2") else 1.0
            x = rng.normal(0.0, gain / np.sqrt(shape[1]), shape)
        w[name] = K.store_bfloat16(x)
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
    return lambda x: K.store_bfloat16(np.asarray(x) * f) / f


STORES = (K.store_bfloat16, shifted_store(1.0 + 2.0 ** -9), shifted_store(1.0 - 3.0 * 2.0 ** -10), shifted_store(1.0 + 5.0 * 2.0 ** -11))


class Oracle:
    """Exact logits [T, V] of one whole sequence and, per row, what rounding every stored activation to
    bfloat16 costs (root-mean-square distance from the exact row).  A row's cost is one draw of a scattered quantity (the
    state of a linear attention carries a rounding over hundreds of positions, and a softmax near a tie amplifies it), so
    four realisations of the rounding are run and the largest distance is the row's cost."""

    def __init__(self, cfg, w, tokens):
        self.exact = K.forward(cfg, w, tokens)
        costs = []
        for store in STORES:
            rounded = K.forward(cfg, w, tokens, store=store)
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
