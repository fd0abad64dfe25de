"""Fovenex, plainly: numpy, float64, whole sequences, one function per mechanism.  It shares no code with the package
and knows no cache: every function takes all positions of one sequence at once.  `forward` takes the raw config.json
dictionary and a dictionary of arrays by tensor name.

Notation: streams X [n, T, E] (n copies of the stream); u the weighted sum a sublayer reads; matrices are stored
[out, in] and applied as h W^T.  `store` (the identity by default) is applied to whatever an engine with 16-bit
activations would keep in them: the normed input, the outputs of matrix products, what feeds the next product.  With
`store_bfloat16` a run shows what such rounding costs; norms, angles, scores, softmax weights and the streams stay
exact in either run.
"""
from __future__ import annotations

import math

import numpy as np


def store_bfloat16(x):
    """x rounded to bfloat16 (nearest even) and widened again."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64).reshape(a.shape)


def same(x):
    return x


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w, the variance being the mean squared deviation; no bias."""
    d = x - x.mean(axis=-1, keepdims=True)
    return d / np.sqrt(np.mean(d * d, axis=-1, keepdims=True) + eps) * w


def rotary_frequencies(rot):
    """The dims / 2 angular steps per position and the multiplier of cosines and sines.  With a `scaling` entry the
    low frequencies are divided by `factor`, the high ones kept, with a linear ramp between the two channel indices
    at which `original` positions make `fast` and `slow` turns; the multiplier is 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_index(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_index(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_index(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, rot):
    """x [T, heads, D]: channel i < dims/2 of every head is paired with channel i + dims/2 and the pair turned by
    position * frequency_i; channels from `dims` on pass."""
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    out = np.array(x, dtype=np.float64)
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def masked_softmax(scores, window=0):
    """Rows are queries, columns keys, both at positions 0..T-1: key j counts for query i iff 0 <= i - j (< window,
    if there is one)."""
    T = scores.shape[0]
    d = np.arange(T)[:, None] - np.arange(T)[None, :]
    mask = (d >= 0) & ((d < window) if window else True)
    s = np.where(mask, scores, -np.inf)
    p = np.exp(s - s.max(axis=1, keepdims=True))
    return p / p.sum(axis=1, keepdims=True)


def differential_attention(h, P, m, positions, eps, store=same):
    """Two softmax maps per head over the same values, o = a1 - lambda a2, each head's o divided by its root mean
    square, times (1 - diff), times a sigmoid gate per head, then the output projection."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = store(h @ P["q"].T).reshape(T, H * 2, D)
    k = store(h @ P["k"].T).reshape(T, G * 2, D)
    v = store(h @ P["v"].T).reshape(T, G, Dv)
    q = unit_rms(q, eps) * P["q.norm"]
    k = unit_rms(k, eps) * P["k.norm"]
    if m.get("rot"):
        q, k = rotate_half(q, positions, m["rot"]), rotate_half(k, positions, m["rot"])
    q, k = store(q), store(k)
    lam = math.exp(float(np.sum(P["lq1"] * P["lk1"]))) - math.exp(float(np.sum(P["lq2"] * P["lk2"]))) + m["diff"]
    gate = sigmoid(store(h @ P["g"].T))                      # [T, H]
    out = np.zeros((T, H, Dv))
    for hd in range(H):
        g = hd // (H // G)
        window = int((m.get("mask") or {}).get("size") or 0)
        maps = [masked_softmax((q[:, 2 * hd + i] @ k[:, 2 * g + i].T) * m["scale"], window) @ v[:, g] for i in (0, 1)]
        o = maps[0] - lam * maps[1]
        out[:, hd] = unit_rms(o, eps) * (1.0 - m["diff"]) * gate[:, hd:hd + 1]
    return store(store(out.reshape(T, H * Dv)) @ P["o"].T)


def latent_rows(h, P, m, positions, eps, store=same):
    """What a latent layer keeps per position: the normed latent vector [T, kv_rank] and the rotated shared key part
    [T, rot_dim]."""
    C, R = m["kv_rank"], m["rot_dim"]
    d = store(h @ P["dkv"].T)
    c = store(unit_rms(d[:, :C], eps) * P["dkv.norm"])
    r = store(rotate_half(d[:, None, C:], positions, dict(m["rot"], dims=R))[:, 0])
    return c, r


def latent_attention(h, P, m, positions, eps, rows, store=same):
    """Queries through a normed latent vector; keys and values raised per head from the rows (c, r) of this layer or of
    the layer it borrows them from; sliding window; a sigmoid gate element by element; output projection."""
    T = h.shape[0]
    H, D, R, Dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, r = rows
    if "dq" in P:
        cq = store(unit_rms(store(h @ P["dq"].T), eps) * P["dq.norm"])
        q = store(cq @ P["uq"].T).reshape(T, H, D + R)
    else:   # (queries straight from the layer's input)
        q = store(h @ P["q"].T).reshape(T, H, D + R)
    q = np.concatenate([q[..., :D], store(rotate_half(q[..., D:], positions, dict(m["rot"], dims=R)))], axis=-1)
    k = store(c @ P["uk"].T).reshape(T, H, D)
    v = store(c @ P["uv"].T).reshape(T, H, Dv)
    window = int((m.get("mask") or {}).get("size") or 0)
    out = np.zeros((T, H, Dv))
    for hd in range(H):
        s = (q[:, hd, :D] @ k[:, hd].T + q[:, hd, D:] @ r.T) * m["scale"]
        out[:, hd] = masked_softmax(s, window) @ v[:, hd]
    o = store(out.reshape(T, H * Dv)) * sigmoid(store(h @ P["g"].T))
    return store(store(o) @ P["o"].T)


def dense_feed_forward(h, P, store=same):
    return store(store(gelu_tanh(h @ P["up"].T)) @ P["down"].T)


def sub(tensors, prefix):
    return {k[len(prefix):]: np.asarray(v, dtype=np.float64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, store=same, layers_out=None):
    """Logits [T, vocab] of one sequence.  `layers_out`, a list, receives the sum of the streams after every layer."""
    eps, mult = float(config["norm"]["eps"]), float(config.get("residual_mult", 1.0))
    n = int(config.get("streams") or 0)
    T = len(tokens)
    positions = np.arange(T)
    x = np.asarray(tensors["embed"], dtype=np.float64)[np.asarray(tokens)]
    X = np.stack([x] * max(n, 1))
    kept = {}

    def sublayer(X, L, q, fn):
        if n:
            hc = sub(L, "hc%d." % q)
            u = np.einsum("s,ste->te", hc["in"], X)
        else:
            u = X[0]
        y = fn(store(layer_norm(u, L["norm%d" % q], eps))) * L["ls%d" % q]
        if n:
            return np.einsum("st,sne->tne", hc["mix"], X) + mult * hc["out"][:, None, None] * y[None]
        return X + mult * y[None]

    for i, layer in enumerate(config["layers"]):
        L = sub(tensors, "l%d." % i)
        P, m = sub(L, "mix."), layer["mixer"]
        if layer["type"] == "attention":
            mixer = lambda h: differential_attention(h, P, m, positions, eps, store)
        else:
            def mixer(h):
                if m.get("kv_from") is None:
                    kept[i] = latent_rows(h, P, m, positions, eps, store)
                return latent_attention(h, P, m, positions, eps, kept[i if m.get("kv_from") is None else m["kv_from"]], store)
        X = sublayer(X, L, 1, mixer)
        if layer.get("mlp") is not None:
            X = sublayer(X, L, 2, lambda h: dense_feed_forward(h, sub(L, "mlp."), store))
        if layers_out is not None:
            layers_out.append(X.sum(axis=0))
    x = store(layer_norm(X.sum(axis=0), np.asarray(tensors["final.norm"], dtype=np.float64), eps))
    return x @ np.asarray(tensors["head"], dtype=np.float64).T


def greedy_generate(config, tensors, prompt, n):
    """The n tokens that follow `prompt` when the most likely one is taken every time (the lowest index among equals)."""
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(np.argmax(forward(config, tensors, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
