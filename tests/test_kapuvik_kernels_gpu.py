"""The kernels behind Kapuvik's mechanisms, each alone against its plain function (`plain_kapuvik.py`): rotation of
neighbours or halves into pages, attention with bounded scores (far keys, page borders, the first tokens, a key that
would dominate without the bound), the latent row's preparation and attention over rows whose value lies inside the key,
the products per head, the state walk with a decay per head or per channel and position (carried over steps, with
rotation and multipliers), the per-head norm with a gate, the bounded feed-forward's activation, the sum of terms into
the stream with the next norm, and the bounded logits."""
import numpy as np
import pytest
import torch

import plain_kapuvik as K

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 8e-3}   # (a bfloat16 result is rounded once: 2^-8 of its size)


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(dtype)


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device=DEV)


def bf(x):
    return K.store_bfloat16(x)


def close(got, want, tol):
    got = got.float().cpu().numpy().astype(np.float64)
    scale = max(1.0, float(np.abs(want).max()))
    assert got.shape == want.shape and np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol * scale, "largest error %g of scale %g" % (np.abs(got - want).max(), scale)


def inv_freq(base, dims):
    return dev(np.asarray([np.float32(1.0) / np.float32(base ** (i / dims)) for i in range(0, dims, 2)], dtype=np.float32))


def paged(k, v, page_size, n_pages, seed):
    T, G, Dk = k.shape
    blocks = -(-T // page_size)
    table = np.random.default_rng(seed).permutation(n_pages)[:blocks]
    kp = np.full((n_pages, G, page_size, Dk), np.nan)
    vp = np.full((n_pages, G, page_size, v.shape[2]), np.nan)
    for j in range(T):
        kp[table[j // page_size], :, j % page_size] = k[j]
        vp[table[j // page_size], :, j % page_size] = v[j]
    return kp, vp, table


def block_table(table, blocks=96):
    bt = torch.full((1, blocks), -1, dtype=torch.int32, device=DEV)
    bt[0, :len(table)] = ints(table)
    return bt


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Dv,rot,interleaved", [(4, 2, 20, 12, 8, True), (2, 1, 64, 64, 64, True), (3, 3, 16, 16, 6, False),
                                                     (2, 2, 128, 128, 128, True)])
def test_rotation_of_neighbours_or_halves_into_pages(dtype, H, G, D, Dv, rot, interleaved):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(0)
    T, S = 9, 4
    x = bf(rng.normal(size=(T, (H + G) * D + G * Dv + 8)))
    pos = [0, 1, 2, 3, 40, 41, 90, 7, 8]     # (angles are float32: at position p they carry an error of p * 6e-8)
    slots = [5, 6, 7, 0, 1, 2, -1, 12, 13]
    qkv = dev(x, dtype)
    kp = torch.full((4, G, S, D), float("nan"), dtype=dtype, device=DEV)
    vp = torch.full((4, G, S, Dv), float("nan"), dtype=dtype, device=DEV)
    ops.qk_norm_rope_kv(qkv, None, None, 1e-6, inv_freq(300.0, rot), rot, ints(pos), ints(slots), kp, vp, H, G, D, Dv,
                        interleaved=interleaved)
    q = K.rotate(x[:, :H * D].reshape(T, H, D), pos, 300.0, rot, interleaved)
    k = K.rotate(x[:, H * D:(H + G) * D].reshape(T, G, D), pos, 300.0, rot, interleaved)
    close(qkv[:, :H * D], q.reshape(T, H * D), TOL[dtype])
    close(qkv[:, (H + G) * D + G * Dv:], x[:, (H + G) * D + G * Dv:], 0.0)      # columns past the values stay
    for t, s in enumerate(slots):
        if s >= 0:
            close(kp[s // S, :, s % S], k[t], TOL[dtype])
            close(vp[s // S, :, s % S], x[t, (H + G) * D:(H + G) * D + G * Dv].reshape(G, Dv), 0.0)
    assert torch.isnan(kp[3, :, 2:]).all()     # (slots 14, 15 were not written)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,Dk,Dv,cap", [(4, 2, 20, 12, 5.0), (4, 2, 64, 64, 20.0), (2, 1, 128, 64, 0.0), (6, 1, 64, 64, 30.0)])
def test_attention_with_bounded_scores_against_the_plain_function(dtype, H, G, Dk, Dv, cap):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(1)
    T = 150
    q, k, v = bf(3.0 * rng.normal(size=(T, H, Dk))), bf(rng.normal(size=(T, G, Dk))), bf(rng.normal(size=(T, G, Dv)))
    want = K.causal_softmax_attention(q, k, v, 0.3, cap).reshape(T, H * Dv)
    kp, vp, table = paged(k, v, 16, 12, 3)
    rows = [0, 1, 2, 15, 16, 17, 31, 32, 100, 149]
    got = ops.paged_attention_generic(dev(q[rows].reshape(len(rows), H * Dk), dtype), H * Dk, dev(kp, dtype), dev(vp, dtype),
                                      block_table(table), ints([0] * len(rows)), ints(rows), 0.3, 0, H, G, Dk, len(rows),
                                      v_head_dim=Dv, softcap=cap)
    close(got, want[rows], TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_key_that_would_dominate_is_held_by_the_bound_wherever_it_lies(dtype):
    """One key whose score is 400 before the bound, among 299 keys of score 0, at the first position, at page borders
    and far away: with a bound of 3 its weight is e^3 / (e^3 + visible - 1) exactly; without the bound it would be 1."""
    from velox_b200.csrc import ops
    T, D = 300, 32
    for spot in (0, 15, 16, 63, 64, 290):
        q = np.zeros((T, 1, D))
        q[:, 0, 0] = 20.0
        k = np.zeros((T, 1, D))
        k[spot, 0, 0] = 20.0
        v = np.zeros((T, 1, D))
        v[spot, 0, 5] = 1.0
        kp, vp, table = paged(k, v, 16, 24, spot)
        rows = [r for r in (spot - 1, spot, spot + 1, 299) if 0 <= r < T]
        got = ops.paged_attention_generic(dev(q[rows].reshape(len(rows), D), dtype), D, dev(kp, dtype), dev(vp, dtype),
                                          block_table(table), ints([0] * len(rows)), ints(rows), 1.0, 0, 1, 1, D, len(rows),
                                          softcap=3.0).float().cpu().numpy()
        for i, r in enumerate(rows):
            want = np.exp(3.0) / (np.exp(3.0) + r) if r >= spot else 0.0
            assert abs(got[i, 5] - want) <= TOL[dtype], (spot, r)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,R,Dv,C,interleaved", [(3, 12, 6, 10, 20, True), (4, 32, 64, 32, 64, True), (2, 16, 8, 16, 24, False),
                                                    (19, 8, 4, 8, 33, True), (2, 16, 32, 16, 300, True), (1, 8, 2, 8, 520, False),
                                                    (5, 16, 8, 16, 136, True)])
def test_latent_rows_are_prepared_cached_and_attended_as_the_plain_mixer_does(dtype, H, D, R, Dv, C, interleaved):
    """The mixer's middle (everything between its input projection and its output projection) on projected rows: the latent
    norm and the rotations into the page, the queries folded through W_uk, attention over rows whose value is the start of
    the key, the attended latent vector raised through W_uv; in two steps, the second reading what the first cached (its
    keys in one run, and cut into runs that a second kernel joins).  More heads than a block takes, an odd latent size,
    and rows beyond 256 and 512 elements are among the cases."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(2)
    T, S, base, scale = 70, 16, 500.0, 0.2
    q = bf(rng.normal(size=(T, H, D + R)))
    down = bf(rng.normal(size=(T, C + R)))
    wn, uk, uv = bf(1.0 + 0.2 * rng.normal(size=C)), bf(rng.normal(size=(H * D, C)) / np.sqrt(C)), bf(rng.normal(size=(H * Dv, C)) / np.sqrt(C))
    pos = np.arange(T)
    c = K.rms(down[:, :C], 1e-5) * wn
    k_rot = K.rotate(down[:, None, C:], pos, base, R, interleaved)
    q_rot = K.rotate(q[:, :, D:], pos, base, R, interleaved)
    kk = np.concatenate([(c @ uk.T).reshape(T, H, D), np.broadcast_to(k_rot, (T, H, R))], axis=2)
    want = K.causal_softmax_attention(np.concatenate([q[:, :, :D], q_rot], axis=2), kk, (c @ uv.T).reshape(T, H, Dv), scale)
    table = np.random.default_rng(5).permutation(8)[:5]
    pool = torch.full((8, 1, S, C + R), float("nan"), dtype=dtype, device=DEV)
    uk_t = dev(uk.reshape(H, D, C).transpose(0, 2, 1), dtype).contiguous()
    uv_d = dev(uv.reshape(H, Dv, C), dtype).contiguous()
    fr = inv_freq(base, R)
    outs = []
    for lo, hi in ((0, 37), (37, T)):
        n = hi - lo
        x = dev(np.concatenate([q[lo:hi].reshape(n, -1), down[lo:hi]], axis=1), dtype)
        qd, dd = x[:, :H * (D + R)], x[:, H * (D + R):]
        slots = [int(table[j // S]) * S + j % S for j in range(lo, hi)]
        qa = torch.empty((n, H, C + R), dtype=dtype, device=DEV)
        ops.latent_prep(dd, qd, qa, dev(wn), 1e-5, fr, interleaved, ints(range(lo, hi)), ints(slots), pool, H, D, R, C)
        ops.gemm_heads(qd.view(n, H, D + R)[:, :, :D], uk_t, qa[:, :, :C])
        lat = ops.latent_attention(qa, pool, block_table(table), ints([0] * n), ints(range(lo, hi)), scale, H, C, R)
        o = torch.empty((n, H, Dv), dtype=dtype, device=DEV)
        ops.gemm_heads(lat, uv_d, o)
        outs.append(o)
        if lo:
            # the same rows one at a time, their keys in runs (the bound on the keys is what asks for runs)
            cut = torch.cat([ops.latent_attention(qa[i:i + 1].contiguous(), pool, block_table(table), ints([0]), ints([lo + i]),
                                                  scale, H, C, R, max_kv=1000) for i in range(n - 3, n)])
            close(cut, lat[n - 3:].float().cpu().numpy().astype(np.float64), TOL[dtype])
    close(torch.cat(outs), want, 3 * TOL[dtype])
    for j in (0, 36, 37, T - 1):
        row = pool[int(table[j // S]), 0, j % S]
        close(row[:C], c[j], TOL[dtype])
        close(row[C:], k_rot[j, 0], TOL[dtype])


@pytest.mark.parametrize("H,D,R,Dv,C", [(3, 32, 64, 32, 40), (2, 64, 32, 64, 72), (5, 128, 64, 128, 96), (2, 32, 32, 64, 24)])
def test_raised_keys_and_values_under_the_tensor_core_prompt_kernel(H, D, R, Dv, C):
    """Two requests of unequal length in two steps each (the second step reads rows that the first cached, and is cut in the
    middle of a page and of a block of raised rows): the cached rows gathered out of scattered pages, one product that leaves
    every head's key and value side by side, the prompt kernel on those rows with the queries turned where they lie.
    Request b's first key is made to stand out for its last query, far behind it."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(12)
    S, base, scale, dtype = 16, 300.0, 0.15, torch.bfloat16
    lens, cuts = [150, 83], [70, 37]
    n_pages = 20
    pages = np.random.default_rng(13).permutation(n_pages)
    tables = [pages[:10], pages[10:16]]
    wn, uk, uv = bf(1.0 + 0.2 * rng.normal(size=C)), bf(rng.normal(size=(H * D, C)) / np.sqrt(C)), bf(rng.normal(size=(H * Dv, C)) / np.sqrt(C))
    w_raise = np.zeros((H, D + R + Dv, C + R))
    w_raise[:, :D, :C] = uk.reshape(H, D, C)
    w_raise[:, D:D + R, C:] = np.eye(R)
    w_raise[:, D + R:, :C] = uv.reshape(H, Dv, C)
    w_raise = dev(w_raise.reshape(-1, C + R), dtype)
    q = [bf(rng.normal(size=(n, H, D + R))) for n in lens]
    down = [bf(rng.normal(size=(n, C + R))) for n in lens]
    down[1][0, C:] *= 6.0           # the shared rotated part of request b's first key, and the last query's rotated part
    q[1][-1, :, D:] = bf(K.rotate(down[1][:1, None, C:], np.array([-(lens[1] - 1)]), base, R, True)[0])   # (turned back: it meets key 0)
    want = []
    for n, qq, dd in zip(lens, q, down):
        pos = np.arange(n)
        c = K.rms(dd[:, :C], 1e-5) * wn
        k_rot = K.rotate(dd[:, None, C:], pos, base, R, True)
        q_rot = K.rotate(qq[:, :, D:], pos, base, R, True)
        kk = np.concatenate([(c @ uk.T).reshape(n, H, D), np.broadcast_to(k_rot, (n, H, R))], axis=2)
        want.append(K.causal_softmax_attention(np.concatenate([qq[:, :, :D], q_rot], axis=2), kk, (c @ uv.T).reshape(n, H, Dv), scale))
    pool = torch.full((n_pages, 1, S, C + R), float("nan"), dtype=dtype, device=DEV)
    bt = torch.full((2, 12), -1, dtype=torch.int32, device=DEV)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = ints(t)
    fr = inv_freq(base, R)
    got = [[], []]
    for step in range(2):
        spans = [(0, c) if step == 0 else (c, n) for c, n in zip(cuts, lens)]
        x = dev(np.concatenate([np.concatenate([q[i][lo:hi].reshape(hi - lo, -1), down[i][lo:hi]], axis=1) for i, (lo, hi) in enumerate(spans)]), dtype)
        pos = [j for lo, hi in spans for j in range(lo, hi)]
        slots = [int(tables[i][j // S]) * S + j % S for i, (lo, hi) in enumerate(spans) for j in range(lo, hi)]
        news = [hi - lo for lo, hi in spans]
        cu, off = ints([0, news[0], news[0] + news[1]]), ints([lo for lo, _ in spans])
        ops.latent_prep(x[:, H * (D + R):], x[:, :H * (D + R)], None, dev(wn), 1e-5, fr, True, ints(pos), ints(slots), pool, H, D, R, C)
        plan = ops.RaisedPlan([hi for _, hi in spans], DEV)
        rows = ops.latent_gather(pool, bt, cu, off, plan)
        assert rows.shape[0] == sum(-(-hi // 64) * 64 for _, hi in spans) and torch.isfinite(rows.float()).all()
        kv = ops.gemm_bf16(rows, w_raise)
        o = ops.raised_attention(x, x.shape[1], kv, cu, off, plan, scale, H, D + R, Dv, max(news))
        got[0].append(o[:news[0]])
        got[1].append(o[news[0]:])
    for i in range(2):
        close(torch.cat(got[i]).view(lens[i], H, Dv), want[i], 3 * TOL[dtype])


def walk_case(rng, T, H, D, Dv, extra=0):
    x = bf(rng.normal(size=(T, 2 * H * D + H * Dv + extra)))
    return x, x[:, :H * D].reshape(T, H, D), x[:, H * D:2 * H * D].reshape(T, H, D), x[:, 2 * H * D:2 * H * D + H * Dv].reshape(T, H, Dv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Dv,rot,interleaved", [(2, 10, 14, 6, False), (2, 64, 64, 32, False), (3, 16, 40, 16, True), (1, 130, 8, 0, False)])
def test_the_state_walk_with_a_decay_per_head_rotation_and_multipliers_carries_its_state(dtype, H, D, Dv, rot, interleaved):
    """Two requests in three steps of unequal portions (down to single tokens) through states in slots 2 and 0; slot 1 keeps
    its poison.  A decay of exactly 1 is among the heads'."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(3)
    decay = np.array([0.9, 1.0, 0.97][:H])
    lens = {"a": 41, "b": 23}
    data = {n: walk_case(rng, t, H, D, Dv, extra=8) for n, t in lens.items()}
    want = {}
    for n, (x, q, k, v) in data.items():
        pos = np.arange(lens[n])
        if rot:
            q, k = K.rotate(q, pos, 50.0, rot, interleaved), K.rotate(k, pos, 50.0, rot, interleaved)
        want[n] = K.decayed_state_walk(q * 0.5, k * D ** -0.5, v, decay).reshape(lens[n], H * Dv)
    state = torch.full((3, H, D, Dv), float("nan"), device=DEV)
    state[0].zero_()
    state[2].zero_()
    at = {"a": 0, "b": 0}
    got = {"a": [], "b": []}
    for step in ([("a", 17), ("b", 1)], [("b", 21), ("a", 1)], [("a", 23), ("b", 1)]):
        rows = [data[n][0][at[n]:at[n] + m] for n, m in step]
        pos = [p for n, m in step for p in range(at[n], at[n] + m)]
        cu = np.cumsum([0] + [m for _, m in step])
        o = ops.linear_attention_walk(dev(np.concatenate(rows), dtype), 0, H * D, 2 * H * D, state, ints(cu),
                                      ints([2 if n == "a" else 0 for n, _ in step]), len(step), H, D, Dv, decay=dev(decay),
                                      inv_freq=inv_freq(50.0, rot) if rot else None, rot_dim=rot, interleaved=interleaved,
                                      positions=ints(pos), q_mul=0.5, k_mul=D ** -0.5)
        for i, (n, m) in enumerate(step):
            got[n].append(o[cu[i]:cu[i + 1]])
            at[n] += m
    for n in lens:
        close(torch.cat(got[n]), want[n], 1e-4)          # (the state and every sum are float32 in either engine)
    assert torch.isnan(state[1]).all() and torch.isfinite(state[0]).all() and torch.isfinite(state[2]).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Dv,tau", [(3, 20, 24, 7.0), (2, 64, 64, 12.0), (2, 18, 10, 1.0)])
def test_the_state_walk_with_a_decay_per_channel_and_position(dtype, H, D, Dv, tau):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(4)
    T = 50
    x, q, k, v = walk_case(rng, T, H, D, Dv)
    z = rng.normal(1.0, 3.0, size=(T, H * D)).astype(np.float32).astype(np.float64)
    z[7] = 40.0     # a decay of exactly one in 32 bits
    z[9] = -60.0    # and one that forgets everything
    alpha = (K.sigmoid(z) ** (1.0 / tau)).reshape(T, H, D)
    want = K.decayed_state_walk(q * D ** -0.5, k, v, alpha).reshape(T, H * Dv)
    state = torch.zeros((1, H, D, Dv), device=DEV)
    outs = []
    for lo, hi in ((0, 1), (1, 30), (30, 32), (32, T)):
        outs.append(ops.linear_attention_walk(dev(x[lo:hi], dtype), 0, H * D, 2 * H * D, state, ints([0, hi - lo]), ints([0]), 1,
                                              H, D, Dv, gate=dev(z[lo:hi]), gate_mul=1.0 / tau, q_mul=D ** -0.5))
    close(torch.cat(outs), want, 1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("per_channel", [False, True])
def test_stretches_walked_side_by_side_give_what_the_walk_in_order_gives(dtype, per_channel):
    """Three requests of 300, 1 and 77 rows whose states are not zero, cut into stretches of 64 and of 16 rows: the outputs
    and the states left in the slots are the plain walk's (with a rotation and multipliers for the decay per head)."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(8)
    H, D, Dv, lens = 2, 12, 20, [300, 1, 77]
    T = sum(lens)
    x, q, k, v = walk_case(rng, T, H, D, Dv)
    x = 0.5 * x
    q, k, v = 0.5 * q, 0.5 * k, 0.5 * v
    x = bf(x)
    q, k, v = (x[:, :H * D].reshape(T, H, D), x[:, H * D:2 * H * D].reshape(T, H, D), x[:, 2 * H * D:].reshape(T, H, Dv))
    start = rng.normal(size=(4, H, D, Dv))
    slots, offs = [2, 0, 3], [40, 7, 0]
    pos = np.concatenate([np.arange(o, o + n) for o, n in zip(offs, lens)])
    z = rng.normal(1.0, 1.5, size=(T, H * D))
    decay = np.array([0.9, 0.99])
    want_o, want_s = [], {}
    row = 0
    for n, slot in zip(lens, slots):
        sl = slice(row, row + n)
        if per_channel:
            qq, kk = q[sl] * D ** -0.5, k[sl]
            a = (K.sigmoid(z[sl]) ** (1.0 / 5.0)).reshape(n, H, D)
        else:
            qq = K.rotate(q[sl], pos[sl], 100.0, 8, False)
            kk = K.rotate(k[sl], pos[sl], 100.0, 8, False) * 0.3
            a = np.broadcast_to(decay[None, :, None], (n, H, D))
        S = start[slot].copy()
        out = np.zeros((n, H, Dv))
        for t in range(n):
            S = a[t][:, :, None] * S + kk[t][:, :, None] * v[sl][t][:, None, :]
            out[t] = np.einsum("hdv,hd->hv", S, qq[t])
        want_o.append(out.reshape(n, H * Dv))
        want_s[slot] = S
        row += n
    want_o = np.concatenate(want_o)
    cu = ints(np.concatenate([[0], np.cumsum(lens)]))
    for length in (64, 16):
        state = dev(start)
        plan = ops.StretchPlan(lens, DEV, length)
        assert plan.count == sum(-(-n // length) for n in lens)
        more = (dict(gate=dev(z), gate_mul=1.0 / 5.0, q_mul=D ** -0.5) if per_channel else
                dict(decay=dev(decay), inv_freq=inv_freq(100.0, 8), rot_dim=8, positions=ints(pos), k_mul=0.3))
        got = ops.linear_attention_walk(dev(x, dtype), 0, H * D, 2 * H * D, state, cu, ints(slots), 3, H, D, Dv, stretches=plan, **more)
        close(got, want_o, 1e-4)
        for slot, S in want_s.items():
            close(state[slot], S, 1e-4)
        assert torch.equal(state[1], dev(start)[1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Dv,weight,act", [(3, 24, True, "silu"), (2, 14, False, "silu"), (2, 64, True, "sigmoid")])
def test_every_head_is_normed_by_itself_and_gated(dtype, H, Dv, weight, act):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(5)
    T = 11
    o = rng.normal(size=(T, H, Dv)).astype(np.float32).astype(np.float64) * np.array([1e-3, 1.0, 50.0])[:H, None]
    g = bf(rng.normal(size=(T, H * Dv + 8)))
    w = bf(1.0 + 0.2 * rng.normal(size=Dv)) if weight else None
    want = K.rms(o, 1e-5) * (w if weight else 1.0)
    gate = g[:, :H * Dv]
    want = want.reshape(T, H * Dv) * (K.silu(gate) if act == "silu" else K.sigmoid(gate))
    got = ops.head_norm_gate(dev(o.reshape(T, H * Dv)), dev(g, dtype)[:, :H * Dv], dev(w) if weight else None, H, 1e-5, act)
    close(got, want, TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_bounded_activation_on_sums_with_biases(dtype):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(6)
    T, F = 13, 40
    sums = (3.0 * rng.normal(size=(T, 2 * F))).astype(np.float32).astype(np.float64)
    bias = bf(rng.normal(size=2 * F))
    g = np.minimum(sums[:, :F] + bias[:F], 1.25)
    u = np.clip(sums[:, F:] + bias[F:], -1.25, 1.25)
    want = g * K.sigmoid(1.702 * g) * (u + 1.0)
    assert (sums[:, :F] + bias[:F] > 1.25).any() and (sums[:, F:] + bias[F:] < -1.25).any()
    close(ops.capped_gated_act(dev(sums), dev(bias), 1.25, 1.702, dtype), want, TOL[dtype])
    close(ops.capped_gated_act(dev(sums), None, 1.25, 1.702, dtype),
          np.minimum(sums[:, :F], 1.25) * K.sigmoid(1.702 * np.minimum(sums[:, :F], 1.25)) * (np.clip(sums[:, F:], -1.25, 1.25) + 1.0), TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [72, 128, 1000])
def test_terms_rows_and_a_vector_go_into_the_stream_with_the_next_norm(dtype, width):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(7)
    T = 9
    res = rng.normal(size=(T, width)).astype(np.float32).astype(np.float64)
    ys = [bf(rng.normal(size=(T, width))) for _ in range(3)]
    rows, vec = rng.normal(size=(T, width)).astype(np.float32).astype(np.float64), rng.normal(size=width).astype(np.float32).astype(np.float64)
    w = bf(1.0 + 0.1 * rng.normal(size=width))
    total = res + 0.7 * ys[0] + 1.3 * ys[1] + ys[2] + rows + vec
    r = dev(res)
    normed = ops.sum_add_rmsnorm(r, [(dev(ys[0], dtype), 0.7), (dev(ys[1], dtype), 1.3), (dev(ys[2], dtype), 1.0)], dev(rows), dev(vec),
                                 dev(w), 1e-5, dtype)
    close(r, total, 2e-6)
    close(normed, K.rms(total, 1e-5) * w, TOL[dtype])
    r2 = dev(res)
    assert ops.sum_add_rmsnorm(r2, [(dev(ys[0], dtype), 1.0)]) is None       # one term, no norm
    close(r2, res + ys[0], 2e-6)
    r3 = dev(res)
    close(ops.sum_add_rmsnorm(r3, [], vec=dev(vec), weight=dev(w), eps=1e-5, out_dtype=dtype), K.rms(res + vec, 1e-5) * w, TOL[dtype])


def test_bounded_logits_and_products_per_head():
    from velox_b200.csrc import ops
    rng = np.random.default_rng(8)
    x = (20.0 * rng.normal(size=(5, 101))).astype(np.float32).astype(np.float64)
    close(ops.softcap_rows(dev(x), 8.0), 8.0 * np.tanh(x / 8.0), 2e-6)
    for dtype in (torch.float32, torch.bfloat16):
        a, w = bf(rng.normal(size=(70, 3, 12 + 5))), bf(rng.normal(size=(3, 20, 12)))
        out = torch.full((70, 3, 20 + 4), float("nan"), dtype=dtype, device=DEV)
        ops.gemm_heads(dev(a, dtype)[:, :, :12], dev(w, dtype), out[:, :, :20])
        close(out[:, :, :20], np.einsum("mhk,hnk->mhn", a[:, :, :12], w), 2 * TOL[dtype])
        assert torch.isnan(out[:, :, 20:]).all()
