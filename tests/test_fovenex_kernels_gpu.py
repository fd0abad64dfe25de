"""The kernels behind Fovenex's mechanisms, each alone against its plain function (`plain_fovenex.py`): the stream in
several copies (weighted sum and norm, update with mixing, the next norm in the same pass), the layer norm, stretched
rotation frequencies with their multiplier and value heads shared by pairs of key heads on the way into the pages, the two
softmax maps over shared values in the general and in the tensor-core kernels, their difference with norm and gate, the
gate element by element, and latent attention under a window, folded and raised, with a key that stands out just inside
and just outside the window, in prompts and for single tokens, where the pages before the window are gone."""
import numpy as np
import pytest
import torch

import plain_fovenex as F

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 8e-3}   # (a bfloat16 result is rounded once: 2^-8 of its size)


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(dtype)


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device=DEV)


def bf(x):
    return F.store_bfloat16(x)


def close(got, want, tol):
    got = got.float().cpu().numpy().astype(np.float64)
    scale = max(1.0, float(np.abs(want).max()))
    assert got.shape == want.shape and np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol * scale, "largest error %g of scale %g" % (np.abs(got - want).max(), scale)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,E,rms", [(1, 72, False), (2, 128, False), (3, 72, True), (4, 1000, False), (5, 40, False), (16, 24, False)])
def test_the_copies_of_the_stream_are_read_updated_and_read_again_in_one_pass(dtype, n, E, rms):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(n)
    T = 37
    X = rng.normal(size=(T, n, E))
    y = bf(rng.normal(size=(T, E)))
    cin, cout, mix = rng.normal(size=n), rng.normal(size=n), np.eye(n) + 0.3 * rng.normal(size=(n, n))
    ls, w, cin2 = 1.0 + 0.2 * rng.normal(size=E), 1.0 + 0.2 * rng.normal(size=E), rng.normal(size=n)
    norm = (lambda u, ww: F.unit_rms(u, 1e-5) * ww) if rms else (lambda u, ww: F.layer_norm(u, ww, 1e-5))
    x = dev(X.reshape(T, n * E))
    X32 = x.cpu().numpy().astype(np.float64).reshape(T, n, E)
    # the weighted sum and its norm, of all rows and of some
    h = ops.stream_norm(x, n, cin.tolist(), dev(w), 1e-5, dtype, rms=rms)
    close(h, norm(np.einsum("s,tse->te", cin, X32), w), TOL[dtype])
    rows = [5, 0, 36]
    h = ops.stream_norm(x, n, None, dev(w), 1e-5, dtype, rows=ints(rows), rms=rms)
    close(h, norm(X32.sum(1)[rows], w), TOL[dtype])
    # the update: all copies from the old ones, then the next reader's input from the new ones
    want = np.einsum("st,tse->tte", mix, X32) if False else np.stack([sum(mix[s, t] * X32[:, s] for s in range(n)) for t in range(n)], 1)
    want = want + 0.7 * cout[None, :, None] * (ls * y)[:, None, :]
    h = ops.stream_update(x, n, mix.tolist(), cout.tolist(), 0.7, dev(ls), dev(y, dtype), cin2.tolist(), dev(w), 1e-5, rms)
    close(x, want.reshape(T, n * E), 2e-6)
    close(h, norm(np.einsum("s,tse->te", cin2, want), w), TOL[dtype])
    # without a next reader, without a layer scale, identity mixing: the plain residual update on every copy
    before = x.cpu().numpy().astype(np.float64).reshape(T, n, E)
    assert ops.stream_update(x, n, None, None, 1.0, None, dev(y, dtype)) is None
    close(x, (before + y[:, None, :]).reshape(T, n * E), 2e-6)
    # the first layer's entry: one row stands for n equal copies, which are written out
    single = dev(X[:, 0])
    copies = torch.full((T, n * E), float("nan"), device=DEV)
    h = ops.stream_norm(None, n, cin.tolist(), dev(w), 1e-5, dtype, single=single, copies=copies, rms=rms)
    s32 = single.cpu().numpy().astype(np.float64)
    close(copies, np.tile(s32, (1, n)), 0.0)
    close(h, norm(cin.sum() * s32, w), TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,per,Dv,gated", [(4, 2, 12, True), (6, 3, 64, True), (2, 2, 20, False), (1, 1, 128, True)])
def test_the_difference_of_the_two_maps_is_normed_and_gated(dtype, H, per, Dv, gated):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(H)
    T, lam, diff = 19, 0.37, 0.3
    a = rng.normal(size=(T, H, 2, Dv))          # [head, map]
    gates = bf(rng.normal(size=(T, H + 3)))
    want = F.unit_rms(a[:, :, 0] - lam * a[:, :, 1], 1e-5) * (1.0 - diff)
    if gated:
        want = want * F.sigmoid(gates[:, 3:])[:, :, None]
    # the kernel's order: per key/value group its heads' first maps, then their second
    G = H // per
    maps = a.reshape(T, G, per, 2, Dv).transpose(0, 1, 3, 2, 4).reshape(T, 2 * H * Dv)
    got = ops.diff_combine(dev(maps), dev(gates, dtype), 3 if gated else -1, lam, 1.0 - diff, 1e-5, H, per, Dv, dtype)
    close(got, want.reshape(T, H * Dv), TOL[dtype])
    o, g = bf(rng.normal(size=(T, 40))), bf(rng.normal(size=(T, 56)))
    got = ops.sigmoid_gate(dev(o, dtype), dev(g, dtype)[:, 8:48])
    close(got, o * F.sigmoid(g[:, 8:48]), TOL[dtype])


def paged(k, v, page_size, n_pages, seed):
    """Keys [T, Gk, D] and values [T, Gv, Dv] into NaN-filled pools through a scattered table."""
    T = k.shape[0]
    table = np.random.default_rng(seed).permutation(n_pages)[:-(-T // page_size)]
    kp = np.full((n_pages, k.shape[1], page_size, k.shape[2]), np.nan)
    vp = np.full((n_pages, v.shape[1], page_size, v.shape[2]), np.nan)
    for j in range(T):
        kp[table[j // page_size], :, j % page_size] = k[j]
        vp[table[j // page_size], :, j % page_size] = v[j]
    return kp, vp, table


def block_table(table, blocks=96, first=0):
    bt = torch.full((1, blocks), -1, dtype=torch.int32, device=DEV)
    bt[0, first:len(table)] = ints(table[first:])
    return bt


def two_maps(q, k, v, scale, window=0):
    """q [T, H, 2, D], k [T, G, 2, D], v [T, G, Dv] -> the maps [T, H, 2, Dv]."""
    T, H = q.shape[:2]
    G = k.shape[1]
    out = np.zeros((T, H, 2, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for m in range(2):
            out[:, h, m] = F.masked_softmax((q[:, h, m] @ k[:, g, m].T) * scale, window) @ v[:, g]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Dv,rot,scaling", [(4, 2, 10, 12, 6, (4.0, 16, 4.0, 1.0)), (2, 1, 64, 64, 32, (2.0, 64, 16.0, 1.0)),
                                                  (3, 3, 16, 20, 16, None), (2, 2, 128, 64, 0, None), (5, 1, 72, 33, 26, (3.0, 32, 8.0, 2.0)),
                                                  (1, 1, 200, 64, 200, None), (3, 2, 48, 128, 24, (2.0, 32, 8.0, 1.0)), (2, 2, 32, 32, 32, None),
                                                  (5, 2, 64, 30, 0, None)])
@pytest.mark.parametrize("T", [45, 130])
def test_norm_stretched_rotation_and_the_write_of_shared_values(dtype, H, G, D, Dv, rot, scaling, T):
    """Both maps' queries and keys normed with one weight each and turned with halves paired by stretched frequencies and
    their multiplier; the keys of 2 G heads and the values of G heads written into pools of those sizes.  Few tokens take the
    kernel with a warp per head, many the kernels with a block per token (heads in registers for bfloat16)."""
    from velox_b200.csrc import ops
    from velox_b200.parts.position import RotaryPosition
    rng = np.random.default_rng(D)
    S = 16
    q, k, v = bf(rng.normal(size=(T, 2 * H, D))), bf(rng.normal(size=(T, 2 * G, D))), bf(rng.normal(size=(T, G, Dv)))
    qw, kw = bf(1.0 + 0.2 * rng.normal(size=D)), bf(1.0 + 0.2 * rng.normal(size=D))
    pos = np.arange(T) + 100
    spec = {"base": 300.0, "dims": rot}
    if scaling:
        spec["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    want_q, want_k = F.unit_rms(q, 1e-5) * qw, F.unit_rms(k, 1e-5) * kw
    inv_freq, magnitude = None, 1.0
    if rot:
        want_q, want_k = F.rotate_half(want_q, pos, spec), F.rotate_half(want_k, pos, spec)
        part = RotaryPosition("", head_dim=D, theta=300.0, rotary_dim=rot, scaling=spec.get("scaling"))
        inv_freq, magnitude = part.rotary_table(DEV)[0], part.magnitude
        f, mag = F.rotary_frequencies(spec)
        assert np.abs(inv_freq.cpu().numpy() - f).max() <= 1e-7 and abs(mag - magnitude) < 1e-12
    pad = (-(2 * (H + G) * D + G * Dv + 5)) % 8
    x = dev(np.concatenate([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), np.full((T, 5 + pad), 7.0)], 1), dtype)
    table = np.random.default_rng(3).permutation(12)[:-(-T // S)]
    k_pool = torch.full((12, 2 * G, S, D), float("nan"), dtype=dtype, device=DEV)
    v_pool = torch.full((12, G, S, Dv), float("nan"), dtype=dtype, device=DEV)
    slots = [int(table[j // S]) * S + j % S for j in range(T)]
    ops.qk_norm_rope_kv(x, dev(qw), dev(kw), 1e-5, inv_freq, rot, ints(pos), ints(slots), k_pool, v_pool, 2 * H, 2 * G, D, Dv,
                        num_v_heads=G, magnitude=magnitude)
    close(x[:, :2 * H * D], want_q.reshape(T, -1), TOL[dtype])
    assert (x[:, 2 * (H + G) * D + G * Dv:] == 7.0).all()
    for j in (0, 15, 16, T - 1):
        close(k_pool[int(table[j // S]), :, j % S], want_k[j], TOL[dtype])
        close(v_pool[int(table[j // S]), :, j % S], v[j], 0.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Dv,window", [(4, 2, 10, 12, 0), (4, 2, 64, 64, 0), (2, 1, 128, 64, 50), (6, 2, 64, 128, 0), (3, 3, 32, 32, 21),
                                             (2, 2, 64, 32, 16)])
def test_two_softmax_maps_over_shared_values_in_every_kernel(dtype, H, G, D, Dv, window):
    """Prompt portions and single tokens, the general kernel and (bfloat16, sizes they take) the tensor-core kernels with
    a token's keys in one run and cut into runs: 2 H query heads over 2 G key heads whose values G heads hold.  The first key is
    made to stand out for the last query's second map of head 0 only: seen from far away without a window, hidden under one."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(H * D)
    T, S, scale = 600, 16, 1.0 / np.sqrt(D)
    per = H // G
    q, k, v = bf(rng.normal(size=(T, H, 2, D))), bf(rng.normal(size=(T, G, 2, D))), bf(rng.normal(size=(T, G, Dv)))
    k[0, 0, 1] = bf(6.0 * k[0, 0, 1])
    q[-1, 0, 1] = bf(3.0 * k[0, 0, 1] / np.sqrt(np.mean(k[0, 0, 1] ** 2)))
    want = two_maps(q, k, v, scale, window)
    if not window:
        assert np.abs(want[-1, 0, 1] - v[0, 0]).max() < 1e-3      # (the far key is all that the map sees)
    # the kernels' order of heads: per key/value group its heads' first maps, then their second
    order = lambda a: a.reshape(T, G, per, 2, -1).transpose(0, 1, 3, 2, 4).reshape(T, 2 * H, -1)
    kp, vp, table = paged(k.reshape(T, 2 * G, D), v, S, 40, 1)
    k_pool, v_pool = dev(kp, dtype), dev(vp, dtype)
    pad = (-(2 * H * D)) % 8
    x = dev(np.concatenate([order(q).reshape(T, -1), np.zeros((T, pad))], 1), dtype)
    rows = list(range(T - 70, T)) if window else list(range(T))
    lo = rows[0]
    # under a window the pages before the window of the step's first query are gone
    bt = block_table(table, first=max(0, lo + 1 - window) // S if window else 0)
    xs = x[lo:].contiguous()
    args = dict(v_head_dim=Dv, v_share=2, out_float32=True)
    got = ops.paged_attention_generic(xs, xs.shape[1], k_pool, v_pool, bt, ints([0] * len(rows)), ints(rows), scale, window, 2 * H, 2 * G,
                                      D, len(rows), **args)
    close(got, order(want)[lo:].reshape(len(rows), -1), TOL[dtype])
    if not ops.biased_attention_supported(dtype, D, Dv, S):
        return
    got = ops.biased_prefill_attention(xs, xs.shape[1], k_pool, v_pool, bt, ints([0, len(rows)]), ints([lo]), scale, window, 0, 0.0,
                                       2 * H, 2 * G, D, Dv, 1, len(rows), len(rows), v_share=2, out_float32=True)
    assert got.dtype == torch.float32
    close(got, order(want)[lo:].reshape(len(rows), -1), TOL[dtype])
    last = x[T - 3:].contiguous()
    bt = block_table(table, first=max(0, T - 3 + 1 - window) // S if window else 0)
    for max_kv in (0, T):   # (the bound on the keys is what asks for runs)
        got = ops.biased_decode_attention(last, last.shape[1], k_pool, v_pool, bt, ints([0] * 3), ints(range(T - 3, T)), scale, window,
                                          0, 0.0, 2 * H, 2 * G, D, Dv, 3, max_kv=max_kv, v_share=2, out_float32=True)
        close(got, order(want)[T - 3:].reshape(3, -1), TOL[dtype])


def latent_case(rng, T, H, D, R, Dv, C, base, spike_at, query_at):
    """Projected rows of one request, with key row `spike_at` made to stand out for every head of the query at `query_at`."""
    q = bf(rng.normal(size=(T, H, D + R)))
    down = bf(rng.normal(size=(T, C + R)))
    down[spike_at, C:] = bf(5.0 * down[spike_at, C:])
    rot = {"base": base, "dims": R}
    # the query's rotated part is the key's, turned back by the distance: after the rotation the two are parallel
    back = F.rotate_half(down[spike_at:spike_at + 1, None, C:], np.array([spike_at - query_at]), rot)[0, 0]
    q[query_at, :, D:] = bf(4.0 * back / np.sqrt(np.mean(back ** 2)))
    return q, down


def latent_plain(q, down, wn, uk, uv, H, D, R, Dv, C, base, scale, window):
    T = q.shape[0]
    pos = np.arange(T)
    rot = {"base": base, "dims": R}
    c = F.unit_rms(down[:, :C], 1e-5) * wn
    r = F.rotate_half(down[:, None, C:], pos, rot)[:, 0]
    qr = F.rotate_half(q[:, :, D:], pos, rot)
    k, v = (c @ uk.T).reshape(T, H, D), (c @ uv.T).reshape(T, H, Dv)
    out = np.zeros((T, H, Dv))
    for h in range(H):
        out[:, h] = F.masked_softmax((q[:, h, :D] @ k[:, h].T + qr[:, h] @ r.T) * scale, window) @ v[:, h]
    return out, c, r


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,R,Dv,C,window", [(3, 12, 6, 10, 20, 7), (4, 32, 64, 32, 64, 40), (2, 64, 64, 64, 64, 96), (5, 16, 8, 16, 136, 33),
                                               (2, 32, 32, 64, 40, 16), (1, 8, 4, 8, 12, 1), (2, 16, 16, 16, 24, 0)])
@pytest.mark.parametrize("inside", [True, False])
def test_latent_attention_under_a_window_folded_and_raised(dtype, H, D, R, Dv, C, window, inside):
    """A request of 300 positions in two steps (a prompt portion cut inside a page, then a second portion), then its last
    rows once more as single tokens with their keys in runs.  One key stands out for the last query: it lies on the window's
    last position (`inside`) or one before it.  The pages that the window has passed are taken out of the block table before
    the second step, as the cache manager does."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(C + window)
    T, S, base, scale = 300, 16, 400.0, 0.2
    w = window or T
    spike = T - w + (0 if inside else -1)
    if spike < 0:
        pytest.skip("without a window nothing lies outside")
    q, down = latent_case(rng, T, H, D, R, Dv, C, base, spike, T - 1)
    wn, uk, uv = bf(1.0 + 0.2 * rng.normal(size=C)), bf(rng.normal(size=(H * D, C)) / np.sqrt(C)), bf(rng.normal(size=(H * Dv, C)) / np.sqrt(C))
    want, c, r = latent_plain(q, down, wn, uk, uv, H, D, R, Dv, C, base, scale, window)
    v_spike = (c[spike] @ uv.T).reshape(H, Dv)
    if inside:
        assert np.abs(want[-1] - v_spike).max() < 0.05 * np.abs(v_spike).max()      # (the key is nearly all the query sees)
    else:
        assert np.abs(want[-1] - v_spike).max() > 0.3 * np.abs(v_spike).max()
    n_pages = 30
    table = np.random.default_rng(5).permutation(n_pages)[:-(-T // S)]
    pool = torch.full((n_pages, 1, S, C + R), float("nan"), dtype=dtype, device=DEV)
    uk_t = dev(uk.reshape(H, D, C).transpose(0, 2, 1), dtype).contiguous()
    uv_d = dev(uv.reshape(H, Dv, C), dtype).contiguous()
    fr = dev(np.asarray(F.rotary_frequencies({"base": base, "dims": R})[0], dtype=np.float32))
    raised = dtype == torch.bfloat16 and ops.raised_attention_supported(dtype, D + R, Dv)
    if raised:
        w_raise = np.zeros((H, D + R + Dv, C + R))
        w_raise[:, :D, :C] = uk.reshape(H, D, C)
        w_raise[:, D:D + R, C:] = np.eye(R)
        w_raise[:, D + R:, :C] = uv.reshape(H, Dv, C)
        w_raise = dev(w_raise.reshape(-1, C + R), dtype)
    cut = 137
    outs, outs_raised = [], []
    for lo, hi in ((0, cut), (cut, T)):
        n = hi - lo
        gone = max(0, lo + 1 - w) // S if window else 0     # pages wholly before the window of the step's first query
        bt = block_table(table, first=gone)
        x = dev(np.concatenate([q[lo:hi].reshape(n, -1), down[lo:hi]], axis=1), dtype)
        qd, dd = x[:, :H * (D + R)], x[:, H * (D + R):]
        slots = [int(table[j // S]) * S + j % S for j in range(lo, hi)]
        qa = torch.empty((n, H, C + R), dtype=dtype, device=DEV)
        ops.latent_prep(dd, qd, qa, dev(wn), 1e-5, fr, False, ints(range(lo, hi)), ints(slots), pool, H, D, R, C)
        ops.gemm_heads(qd.view(n, H, D + R)[:, :, :D], uk_t, qa[:, :, :C])
        lat = ops.latent_attention(qa, pool, bt, ints([0] * n), ints(range(lo, hi)), scale, H, C, R, window=window)
        o = torch.empty((n, H, Dv), dtype=dtype, device=DEV)
        ops.gemm_heads(lat, uv_d, o)
        outs.append(o)
        if raised and (D + R) * H % 8 == 0 and x.shape[1] % 8 == 0:
            ops.latent_prep(None, qd, None, None, 1e-5, fr, False, ints(range(lo, hi)), None, None, H, D, R, C)   # (queries turned where they lie)
            plan = ops.RaisedPlan([hi], DEV, [lo], window)
            rows = ops.latent_gather(pool, bt, ints([0, n]), ints([lo]), plan)
            assert torch.isfinite(rows.float()).all() and rows.shape[0] == plan.rows <= -(-(n + w + 63) // 64) * 64 + 64
            kv = ops.gemm_bf16(rows, w_raise)
            outs_raised.append(ops.raised_attention(x, x.shape[1], kv, ints([0, n]), ints([lo]), plan, scale, H, D + R, Dv, n).view(n, H, Dv))
        if lo:
            # the last rows one at a time, their keys in runs (the bound on the keys is what asks for runs)
            gone = max(0, T - 3 + 1 - w) // S if window else 0
            bt1 = block_table(table, first=gone)
            single = torch.cat([ops.latent_attention(qa[i:i + 1].contiguous(), pool, bt1, ints([0]), ints([lo + i]), scale, H, C, R,
                                                     max_kv=1000, window=window) for i in range(n - 3, n)])
            close(single, lat[n - 3:].float().cpu().numpy().astype(np.float64), TOL[dtype])
    close(torch.cat(outs), want, 3 * TOL[dtype])
    if outs_raised:
        close(torch.cat(outs_raised), want, 3 * TOL[dtype])
