"""Kapuvik, plainly: numpy, float64, whole sequences, one function per mechanism.  It shares no code with the
package and knows no cache: every function takes all positions of one sequence at once (the recurrences walk the
positions one by one).  `forward` takes the raw config.json dictionary and a dictionary of arrays by tensor name.

Notation: x [T, E] the stream; h the normed input of a layer; matrices are stored [out, in] and applied as h W^T.
`store` (the identity by default) is applied to whatever an engine with 16-bit activations would keep in them: the
normed input, the outputs of matrix products, what feeds the next product.  With `store_bfloat16` a run shows what
such rounding costs; norms, scores, softmax weights, decays, states and the stream stay exact in either run.
"""
from __future__ import annotations

import numpy as np


def store_bfloat16(x):
    """x rounded to bfloat16 (nearest even) and widened again."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64).reshape(a.shape)


def same(x):
    return x


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose multiplier is one plus the stored tensor."""
    return rms(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rotate(x, positions, base, dims, interleaved):
    """x [T, heads, D]: the first `dims` channels of every head turned by position * base^(-2i/dims); channel pairs
    are (2i, 2i+1) when `interleaved`, else (i, i + dims/2).  The other channels pass."""
    out = np.array(x, dtype=np.float64)
    half = dims // 2
    i = np.arange(half)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]   # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    if interleaved:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


def causal_softmax_attention(q, k, v, scale, softcap=0.0):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; query head h reads key/value head h // (H / G); position i sees j <= i.
    With `softcap` c > 0 a score s becomes c tanh(s / c) before the softmax."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    mask = np.tril(np.ones((T, T), dtype=bool))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * np.tanh(s / softcap)
        s = np.where(mask, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        out[:, h] = p @ v[:, g]
    return out


def softmax_member(h, P, m, positions, store=same):
    """Grouped softmax attention with rotated q and k (pairs of neighbours), a score multiplier and a cap."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = store(h @ P["q"].T).reshape(T, H, D)
    k = store(h @ P["k"].T).reshape(T, G, D)
    v = store(h @ P["v"].T).reshape(T, G, Dv)
    rot = m.get("rot")
    if rot:
        q = store(rotate(q, positions, rot["base"], rot["dims"], True))
        k = store(rotate(k, positions, rot["base"], rot["dims"], True))
    o = store(causal_softmax_attention(q, k, v, m["scale"], m.get("softcap") or 0.0))
    return store(o.reshape(T, H * Dv) @ P["o"].T)


def decayed_state_walk(q, k, v, decay):
    """q, k [T, H, D], v [T, H, Dv]; decay [H] or [T, H, D] (a number per key channel and position).
    S_t = decay (.) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t."""
    T, H, D = q.shape
    Dv = v.shape[2]
    S = np.zeros((H, D, Dv))
    out = np.zeros((T, H, Dv))
    for t in range(T):
        d = decay[:, None, None] if np.ndim(decay) == 1 else decay[t][:, :, None]
        S = d * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hdv,hd->hv", S, q[t])
    return out


def retention_member(h, P, m, positions, eps, store=same):
    """Linear attention with a fixed decay per head: rotated q and k (halves paired), k / sqrt(D), every head's output
    divided by its own root mean square, times silu of a gate projection."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = store(h @ P["q"].T).reshape(T, H, D)
    k = store(h @ P["k"].T).reshape(T, H, D)
    v = store(h @ P["v"].T).reshape(T, H, Dv)
    rot = m.get("rot")
    if rot:
        q = rotate(q, positions, rot["base"], rot["dims"], False)
        k = rotate(k, positions, rot["base"], rot["dims"], False)
    k = k * D ** -0.5
    o = rms(decayed_state_walk(q, k, v, np.asarray(m["decay"], dtype=np.float64)), eps)
    return store(store(o.reshape(T, H * Dv) * silu(store(h @ P["g"].T))) @ P["o"].T)


def side_by_side_mixer(h, P, m, positions, eps, store=same):
    left = softmax_member(h, {n[5:]: t for n, t in P.items() if n.startswith("left.")}, m["left"], positions, store)
    right = retention_member(h, {n[6:]: t for n, t in P.items() if n.startswith("right.")}, m["right"], positions, eps, store)
    return m.get("left_scale", 1.0) * left + m.get("right_scale", 1.0) * right


def latent_mixer(h, P, m, positions, eps, store=same):
    """Attention whose keys and values are raised from one normed latent vector per position; a rotated key part of its
    own is shared by all heads."""
    T = h.shape[0]
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = store(h @ P["q"].T).reshape(T, H, D + R)
    down = store(h @ P["dkv"].T)
    c = store(rms(down[:, :C], eps) * P["dkv.norm"])
    k_rot = store(rotate(down[:, None, C:], positions, m["rot"]["base"], R, True))           # [T, 1, R]
    q_rot = store(rotate(q[:, :, D:], positions, m["rot"]["base"], R, True))
    k_plain = store(c @ P["uk"].T).reshape(T, H, D)
    v = store(c @ P["uv"].T).reshape(T, H, Dv)
    qq = np.concatenate([q[:, :, :D], q_rot], axis=2)
    kk = np.concatenate([k_plain, np.broadcast_to(k_rot, (T, H, R))], axis=2)
    o = store(causal_softmax_attention(qq, kk, v, m["scale"]))
    return store(o.reshape(T, H * Dv) @ P["o"].T)


def gated_decay_mixer(h, P, m, eps, store=same):
    """Linear attention whose decay is a number per key channel and position, from a two-step projection."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = store(h @ P["q"].T).reshape(T, H, D) * D ** -0.5
    k = store(h @ P["k"].T).reshape(T, H, D)
    v = store(h @ P["v"].T).reshape(T, H, Dv)
    z = store(h @ P["a1"].T) @ P["a2"].T + P["a2.b"]
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, D)
    o = rms(decayed_state_walk(q, k, v, alpha), eps) * P["norm"]
    return store(store(o.reshape(T, H * Dv) * silu(store(h @ P["g"].T))) @ P["o"].T)


def capped_feed_forward(h, P, m, store=same):
    """g = min(gate, L); u = clamp(up, -L, L); down(g sigmoid(1.702 g) (u + 1)); every projection has a bias."""
    L = m["limit"]
    g = np.minimum(h @ P["gate"].T + P["gate.b"], L)
    u = np.clip(h @ P["up"].T + P["up.b"], -L, L)
    return store(store(g * sigmoid(1.702 * g) * (u + 1.0)) @ P["down"].T + P["down.b"])


def running_order(cfg):
    """[(layer, pass number or None, first of its pass)] in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop.get("times", 1) < 1:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    out = [(i, None, False) for i in range(a)]
    for t in range(times):
        out += [(i, t, i == a) for i in range(a, b)]
    return out + [(i, None, False) for i in range(b, n)]


def forward(cfg, W, tokens, return_layers=False, store=same):
    """float64 logits [T, vocab] of one sequence (and the stream after every layer run)."""
    W = {n: np.asarray(t, dtype=np.float64) for n, t in W.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = np.arange(T)
    x0 = W["embed"][np.asarray(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    x = x0.copy()
    seen = []
    for i, t, first in running_order(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t]
        layer = cfg["layers"][i]
        p = "l%d." % i
        h = store(offset_norm(x, W[p + "norm1"], eps))
        M = {n[len(p) + 4:]: a for n, a in W.items() if n.startswith(p + "mix.")}
        kind = layer["type"]
        if kind == "parallel":
            y = side_by_side_mixer(h, M, layer["mixer"], positions, eps, store)
        elif kind == "latent_attention":
            y = latent_mixer(h, M, layer["mixer"], positions, eps, store)
        elif kind == "gla":
            y = gated_decay_mixer(h, M, layer["mixer"], eps, store)
        else:
            raise ValueError(kind)
        if layer.get("mlp") is not None:
            F = {n[len(p) + 4:]: a for n, a in W.items() if n.startswith(p + "mlp.")}
            y = y + capped_feed_forward(h, F, layer["mlp"], store)
        x = x + y
        seen.append(x.copy())
    logits = store(offset_norm(x, W["final.norm"], eps)) @ W["head"].T
    cap = cfg.get("logit_softcap") or 0.0
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(seen)) if return_layers else logits


def greedy_generate(cfg, W, prompt, new_tokens):
    """The `new_tokens` most likely tokens one after the other (the lowest id among equals)."""
    toks = list(prompt)
    for _ in range(new_tokens):
        toks.append(int(np.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]
