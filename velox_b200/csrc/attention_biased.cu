// Paged causal attention with positions in the SCORES instead of a rotation, bfloat16, on
// the tensor cores: for prompt portions and for single decoded tokens.
//
//   score(i, j) = q_i . k_j * scale - slope_h * (i - j),   slope_h = 2^(-bias_exp * (h + 1) / H)
//   query i sees key j  iff  j <= i and (window == 0 or i - j < window or j < keep_first)
//   keys of size DK (64, 128), values of size DV (32, 64, 128), which need not be equal; also equal sizes of
//   32, 48, 80, 96 and 112 (a row of a size that is no power of two lies in shared memory padded to the next one)
//   optionally a sink per query head: the softmax's denominator also holds exp(sinks[h]) (no key, no value,
//   not scaled), and an output gate: head h's output times sigmoid(g), g the element at column
//   gate_col + h of the token's row of `q`
//
// Portions: grid (query tile, head, segment); 4 warps.  A segment is a request's portion of this step
// (rows cu_seqlens[s] .. of positions kv_offsets[s] ..).  A step of single tokens has a kernel of its
// own further down, which deals one query's keys to the warps of a block.  A block takes 64 query rows: 64 / G consecutive tokens
// times the G query heads of one kv head when G is a power of two up to 16 (they share every
// key/value tile), else 64 tokens of one head; 16 rows per warp, held in registers as A
// operands.  It walks the tiles of 64 keys that hold kept first positions before the window,
// then the window's tiles up to the diagonal; K and V tiles are gathered page by page with
// cp.async into double-buffered, swizzled shared memory.  S = Q K^T by mma.sync.m16n8k16; scale,
// bias by distance and mask are applied to the float32 sums; running maximum and sum per row in
// float32 (online softmax, base 2).  The probabilities stay 32-bit in effect: P is cut into
// bfloat16 halves P = P_hi + P_lo (16 bits of mantissa together) and O += P_hi V + P_lo V.
//
// A key slot that the mask hides is never read from a page that may have been given back: its
// address is clamped to the nearest visible key.  The order of every sum depends only on the
// query's own position and the request's keys, so a token's result does not depend on what else is in
// the step (a token decoded alone and the same token inside a portion differ by rounding: other kernels).
#include "common.cuh"
#include "mma_helpers.cuh"

#define AB_WARPS 4
#define AB_BM 64
#define AB_BN 64
#define AB_LOG2E 1.4426950408889634f

// The least power of two that is not below n (n >= 4 here: heads of at least 32 elements).
__host__ __device__ constexpr int ab_pow2(int n) { return n <= 4 ? 4 : (n <= 8 ? 8 : 16); }

// A row's chunks of 16 bytes in shared memory: rows of whole groups of 8 chunks lie as they are (the XOR below stays inside
// a group), the others are padded to a power of two.
__host__ __device__ constexpr int ab_chunks(int n) { return n % 8 == 0 ? n : ab_pow2(n); }

// Where keys and values lie, in elements: key j of kv head hk of a request is at
//   k + page * k_page + hk * k_head + (j % S) * k_row,   page = table[j / S]
// (a page pool [pages, kv heads, S, size] has k_page = Hk S size, k_head = S size, k_row = size; rows [n, heads, sizes]
// that a matrix product left have k_row = the row's length and k_head = one head's share of it).  With `table_by_segment`
// the block table's row is the segment's number, not the request's.  With `v_share` > 1 that many consecutive key heads
// read one value head (v_page and v_head then count value heads); with `out_f32` the output is written as float32.
struct AbLayout {
    long long k_page, k_head, k_row, v_page, v_head, v_row;
    int table_by_segment;
    int v_share;
    int out_f32;
};

template <int CH> __device__ __forceinline__ int ab_swz(int r, int cc) {
    // 16-byte chunk cc of row r; rows of 8 or 16 chunks XOR the row's low bits, rows of 4 chunks
    // (two rows to a 128-byte line) every second row's
    return CH >= 8 ? (cc ^ (r & 7)) : (cc ^ ((r >> 1) & 3));
}

// The sink's share of a row's softmax: the denominator l (relative to the maximum m, base 2) gains
// 2^(sink - m); where the sink exceeds m the reference moves to the sink and `f` scales what was summed.
__device__ __forceinline__ void ab_add_sink(float sink_log2, float m, float& l, float& f) {
    f = 1.f;
    if (sink_log2 > m) {
        f = exp2f(m - sink_log2);
        l = l * f + 1.f;
    } else {
        l += exp2f(sink_log2 - m);
    }
}
__device__ __forceinline__ float ab_gate(const bf16* q, int q_row_stride, int row, int gate_col, int head) {
    return 1.f / (1.f + __expf(-__bfloat162float(q[(size_t)row * q_row_stride + gate_col + head])));
}

// A raw dot product as a score in units of log2: times scale, or, with a bound c on the scores (cap_log2 = c log2(e),
// cap_arg = scale / c), c tanh(dot * scale / c).
__device__ __forceinline__ float ab_score(float dot, float scale_log2, float cap_log2, float cap_arg) {
    return cap_arg > 0.f ? cap_log2 * tanhf(dot * cap_arg) : dot * scale_log2;
}

struct AbSegments {
    const int* cu_seqlens;    // portions: rows of segment s are [cu_seqlens[s], cu_seqlens[s + 1])
    const int* kv_offsets;    //           at positions kv_offsets[s] ..
    const int* seq_of_token;  // single tokens: segment s is token row s of request seq_of_token[s]
    const int* positions;     //           at position positions[s]
    const int* seq_list;      // portions: segment s is request seq_list[s] (null: request s)
};

template <int DK, int DV>
__global__ void __launch_bounds__(AB_WARPS * 32)
biased_attention_kernel(const bf16* __restrict__ q, int q_row_stride, const bf16* __restrict__ k_pool,
                        const bf16* __restrict__ v_pool, const int* __restrict__ block_table, int max_blocks,
                        AbSegments seg, bf16* __restrict__ out, int out_row_stride, float scale_log2, float bias_exp,
                        int window, int keep_first, int H, int Hk, int S, int share_log2,
                        const float* __restrict__ sinks, int gate_col, float cap_log2, float cap_arg, AbLayout lay) {
    extern __shared__ __align__(128) unsigned char ab_smem[];
    constexpr int KCH = DK / 8, VCH = DV / 8;
    constexpr int KCHP = ab_chunks(KCH), VCHP = ab_chunks(VCH);   // a row's place in shared memory
    constexpr int KROW = KCHP * 16, VROW = VCHP * 16;
    constexpr int K_BYTES = AB_BN * KROW, V_BYTES = AB_BN * VROW;
    constexpr int DVT = (DV + 31) / 32 * 4;   // output tiles of 8 columns, in fours (those past DV / 8 are computed on whatever
                                              // the row's padding holds and never stored)
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = gridDim.x - 1 - blockIdx.x, s = blockIdx.z;   // (the longest tiles first)
    const int share = 1 << share_log2;
    const int toks_per_tile = AB_BM >> share_log2;
    int row_base, n_new, off, seq;
    if (seg.cu_seqlens) {
        seq = seg.seq_list ? seg.seq_list[s] : s;
        row_base = seg.cu_seqlens[seq];
        n_new = seg.cu_seqlens[seq + 1] - row_base;
        off = seg.kv_offsets[seq];
    } else {
        row_base = s;
        n_new = 1;
        off = seg.positions[s];
        seq = seg.seq_of_token[s];
    }
    const int t0 = qt * toks_per_tile;
    if (t0 >= n_new) return;
    const int hk = share > 1 ? blockIdx.y : blockIdx.y / (H / Hk);
    const int head0 = share > 1 ? hk * share : blockIdx.y;
    const int* bt = block_table + (size_t)(lay.table_by_segment ? s : seq) * max_blocks;
    const int hv = lay.v_share > 1 ? hk / lay.v_share : hk;
    const int toks_live = min(toks_per_tile, n_new - t0);
    const int kv_hi = off + t0 + toks_live;                              // one past the tile's last visible key
    const int kv_lo = window > 0 ? max(0, off + t0 + 1 - window) : 0;    // first key of the first row's window
    const int tile_lo = kv_lo / AB_BN, tile_hi = (kv_hi + AB_BN - 1) / AB_BN;
    const int kept = window > 0 ? keep_first : 0;
    const int n_kept_tiles = min((kept + AB_BN - 1) / AB_BN, tile_lo);   // tiles with kept positions, before the window's
    const int n_tiles = n_kept_tiles + tile_hi - tile_lo;

    unsigned char* q_s = ab_smem;                    // [64][DK, padded]
    unsigned char* kv_s = ab_smem + AB_BM * KROW;  // 2 stages x (K tile, V tile)

    for (int c = threadIdx.x; c < AB_BM * KCH; c += AB_WARPS * 32) {
        const int r = c / KCH, cc = c % KCH;
        const int tr = min(t0 + (r >> share_log2), n_new - 1);   // rows past the end repeat the last token
        const int hd = head0 + (r & (share - 1));
        cp_async16(q_s + r * KROW + (ab_swz<KCHP>(r, cc) << 4),
                   q + (size_t)(row_base + tr) * q_row_stride + (size_t)hd * DK + cc * 8);
    }
    cp_async_commit();

    auto tile_of = [&](int i) { return i < n_kept_tiles ? i : tile_lo + i - n_kept_tiles; };
    auto issue = [&](int i, int stage) {
        const int tile = tile_of(i);
        unsigned char* ks = kv_s + (size_t)stage * (K_BYTES + V_BYTES);
        unsigned char* vs = ks + K_BYTES;
        for (int c = threadIdx.x; c < AB_BN * KCH; c += AB_WARPS * 32) {
            const int r = c / KCH, cc = c % KCH;
            int key = tile * AB_BN + r;
            // a hidden slot repeats the nearest key that is not hidden: the kept ones stay where they are,
            // the others move into [kv_lo, kv_hi) (in a tile before the window: onto the last kept key)
            if (key >= kept) key = i < n_kept_tiles ? kept - 1 : max(min(key, kv_hi - 1), kv_lo);
            key = min(key, kv_hi - 1);
            const int page = bt[key / S];
            cp_async16(ks + r * KROW + (ab_swz<KCHP>(r, cc) << 4),
                       k_pool + (size_t)page * lay.k_page + (size_t)hk * lay.k_head + (size_t)(key % S) * lay.k_row + cc * 8);
        }
        for (int c = threadIdx.x; c < AB_BN * VCH; c += AB_WARPS * 32) {
            const int r = c / VCH, cc = c % VCH;
            int key = tile * AB_BN + r;
            if (key >= kept) key = i < n_kept_tiles ? kept - 1 : max(min(key, kv_hi - 1), kv_lo);
            key = min(key, kv_hi - 1);
            const int page = bt[key / S];
            cp_async16(vs + r * VROW + (ab_swz<VCHP>(r, cc) << 4),
                       v_pool + (size_t)page * lay.v_page + (size_t)hv * lay.v_head + (size_t)(key % S) * lay.v_row + cc * 8);
        }
    };
    issue(0, 0);
    cp_async_commit();

    cp_async_wait<1>();   // the queries have landed
    __syncthreads();
    unsigned qf[DK / 16][4];
    {
        const int mi = lane >> 3;
        const int r = warp * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
            const int cc = 2 * kk + (mi >> 1);
            ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], q_s + r * KROW + (ab_swz<KCHP>(r, cc) << 4));
        }
    }

    float o[DVT][4];
#pragma unroll
    for (int i = 0; i < DVT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int r0 = warp * 16 + (lane >> 2);
    const int pos0 = off + t0 + (r0 >> share_log2), pos1 = off + t0 + ((r0 + 8) >> share_log2);
    const int lo0 = window > 0 ? pos0 + 1 - window : 0, lo1 = window > 0 ? pos1 + 1 - window : 0;
    const int hd0 = head0 + (r0 & (share - 1)), hd1 = head0 + ((r0 + 8) & (share - 1));
    const float sl0 = bias_exp > 0.f ? exp2f(-bias_exp * (float)(hd0 + 1) / (float)H) * AB_LOG2E : 0.f;
    const float sl1 = bias_exp > 0.f ? exp2f(-bias_exp * (float)(hd1 + 1) / (float)H) * AB_LOG2E : 0.f;
    const int warp_hi = off + t0 + ((warp * 16 + 15) >> share_log2) + 1;
    const int warp_lo = window > 0 ? off + t0 + ((warp * 16) >> share_log2) + 1 - window : 0;

    for (int i = 0; i < n_tiles; ++i) {
        const int stage = i & 1;
        if (i + 1 < n_tiles) issue(i + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const unsigned char* ks = kv_s + (size_t)stage * (K_BYTES + V_BYTES);
        const unsigned char* vs = ks + K_BYTES;
        const int key_base = tile_of(i) * AB_BN;
        if (key_base < warp_hi && (key_base + AB_BN > warp_lo || key_base < kept)) {   // warp-uniform
            float sc[AB_BN / 16][2][4];
            bool vis[AB_BN / 16];
            const int mi = lane >> 3;
            const int rr = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
            for (int kg = 0; kg < AB_BN / 16; ++kg) {
                const int key0 = key_base + kg * 16;
                vis[kg] = key0 < warp_hi && (key0 + 16 > warp_lo || key0 < kept);
#pragma unroll
                for (int c = 0; c < 4; ++c) sc[kg][0][c] = sc[kg][1][c] = 0.f;
            }
            if (vis[0] && vis[1] && vis[2] && vis[3]) {
                // the common tile, wholly visible to the warp: k steps outermost, so that the eight accumulators
                // of a step are independent and their multiply-accumulates overlap
#pragma unroll
                for (int kk = 0; kk < DK / 16; ++kk) {
                    const int cc = 2 * kk + (mi & 1);
#pragma unroll
                    for (int kg = 0; kg < AB_BN / 16; ++kg) {
                        const int r = kg * 16 + rr;
                        unsigned b00, b01, b10, b11;
                        ldmatrix_x4(b00, b01, b10, b11, ks + r * KROW + (ab_swz<KCHP>(r, cc) << 4));
                        mma_bf16(sc[kg][0], qf[kk], b00, b01);
                        mma_bf16(sc[kg][1], qf[kk], b10, b11);
                    }
                }
            } else {
#pragma unroll
                for (int kg = 0; kg < AB_BN / 16; ++kg) {
                    if (!vis[kg]) continue;
                    const int r = kg * 16 + rr;
#pragma unroll
                    for (int kk = 0; kk < DK / 16; ++kk) {
                        const int cc = 2 * kk + (mi & 1);
                        unsigned b00, b01, b10, b11;
                        ldmatrix_x4(b00, b01, b10, b11, ks + r * KROW + (ab_swz<KCHP>(r, cc) << 4));
                        mma_bf16(sc[kg][0], qf[kk], b00, b01);
                        mma_bf16(sc[kg][1], qf[kk], b10, b11);
                    }
                }
            }
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int pos = hrow ? pos1 : pos0, lo = hrow ? lo1 : lo0;
                const float sl = hrow ? sl1 : sl0;
                float mx = -INFINITY;
#pragma unroll
                for (int kg = 0; kg < AB_BN / 16; ++kg)
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const int key = key_base + kg * 16 + nt * 8 + ((lane & 3) << 1) + c;
                            const bool ok = vis[kg] && key <= pos && (key >= lo || key < kept);
                            float& v = sc[kg][nt][2 * hrow + c];
                            v = ok ? ab_score(v, scale_log2, cap_log2, cap_arg) - sl * (float)(pos - key) : -INFINITY;
                            mx = fmaxf(mx, v);
                        }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m[hrow], mx);
                const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m[hrow] - m_new);
                float ps = 0.f;
#pragma unroll
                for (int kg = 0; kg < AB_BN / 16; ++kg)
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            float& v = sc[kg][nt][2 * hrow + c];
                            v = (m_new == -INFINITY) ? 0.f : exp2f(v - m_new);
                            ps += v;
                        }
                l[hrow] = l[hrow] * alpha + ps;
                m[hrow] = m_new;
#pragma unroll
                for (int i2 = 0; i2 < DVT; ++i2) {
                    o[i2][2 * hrow] *= alpha;
                    o[i2][2 * hrow + 1] *= alpha;
                }
            }
            // O += P V with P = P_hi + P_lo
#pragma unroll
            for (int kg = 0; kg < AB_BN / 16; ++kg) {
                if (!vis[kg]) continue;
                unsigned hi[4], lw[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float a = sc[kg][x >> 1][2 * (x & 1)], b = sc[kg][x >> 1][2 * (x & 1) + 1];
                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b);
                    const float2 back = __bfloat1622float2(h2);
                    hi[x] = *reinterpret_cast<const unsigned*>(&h2);
                    lw[x] = pack_bf16(a - back.x, b - back.y);
                }
                const int r = kg * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
                for (int nt = 0; nt < DVT; nt += 4) {   // (two loads, then four independent pairs of products)
                    unsigned v[2][4];
#pragma unroll
                    for (int u = 0; u < 2; ++u)
                        ldmatrix_x4_trans(v[u][0], v[u][1], v[u][2], v[u][3],
                                          vs + r * VROW + (ab_swz<VCHP>(r, nt + 2 * u + (mi >> 1)) << 4));
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        mma_bf16(o[nt + 2 * u], hi, v[u][0], v[u][1]);
                        mma_bf16(o[nt + 2 * u + 1], hi, v[u][2], v[u][3]);
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        mma_bf16(o[nt + 2 * u], lw, v[u][0], v[u][1]);
                        mma_bf16(o[nt + 2 * u + 1], lw, v[u][2], v[u][3]);
                    }
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
        l[hrow] += __shfl_xor_sync(0xffffffffu, l[hrow], 1);
        l[hrow] += __shfl_xor_sync(0xffffffffu, l[hrow], 2);
        const int r = r0 + 8 * hrow;
        const int tok = r >> share_log2;
        if (tok >= toks_live) continue;
        const int hd = head0 + (r & (share - 1));
        float f = 1.f;
        if (sinks) ab_add_sink(sinks[hd] * AB_LOG2E, m[hrow], l[hrow], f);
        if (gate_col >= 0) f *= ab_gate(q, q_row_stride, row_base + t0 + tok, gate_col, hd);
        const float inv = f / l[hrow];
        const size_t at = (size_t)(row_base + t0 + tok) * out_row_stride + (size_t)hd * DV + ((lane & 3) << 1);
        if (lay.out_f32) {
            float* dst = reinterpret_cast<float*>(out) + at;
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt)
                *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][2 * hrow] * inv, o[nt][2 * hrow + 1] * inv);
            continue;
        }
        bf16* dst = out + at;
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt)
            *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) =
                __floats2bfloat162_rn(o[nt][2 * hrow] * inv, o[nt][2 * hrow + 1] * inv);
    }
}

// ---- single tokens: the keys of one query dealt to the warps of a block ----
// grid (kv head, or head when the group is no power of two up to 16; token row); 8 warps.  The visible keys of
// a token (the kept first ones, then the window's) are numbered 0 .. n-1 and taken 16 at a time; group g goes to
// warp g mod 8, which gathers its keys and values itself (cp.async, two stages of its own, no block barrier),
// forms the scores of the group's query heads (rows of one m16 tile) and keeps a running maximum, sum and
// output of its own.  At the end the warps' parts are added in warp order.
#define AD_WARPS 8

template <int DK, int DV>
__global__ void __launch_bounds__(AD_WARPS * 32)
biased_decode_kernel(const bf16* __restrict__ q, int q_row_stride, const bf16* __restrict__ k_pool,
                     const bf16* __restrict__ v_pool, const int* __restrict__ block_table, int max_blocks,
                     const int* __restrict__ seq_of_token, const int* __restrict__ positions, bf16* __restrict__ out,
                     int out_row_stride, float scale_log2, float bias_exp, int window, int keep_first, int H, int Hk,
                     int S, int share_log2, float* __restrict__ scratch, const float* __restrict__ sinks, int gate_col,
                     float cap_log2, float cap_arg, int v_share, int out_f32) {
    extern __shared__ __align__(128) unsigned char ad_smem[];
    constexpr int KCH = DK / 8, VCH = DV / 8;
    constexpr int KCHP = ab_pow2(KCH), VCHP = ab_pow2(VCH);
    constexpr int KROW = KCHP * 16, VROW = VCHP * 16;
    constexpr int K_BYTES = 16 * KROW, V_BYTES = 16 * VROW;
    constexpr int WARP_BYTES = 2 * (K_BYTES + V_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y;
    const int share = 1 << share_log2;
    const int hk = share > 1 ? blockIdx.x : blockIdx.x / (H / Hk);
    const int head0 = share > 1 ? hk * share : blockIdx.x;
    unsigned char* q_s = ad_smem;                                  // [16][DK]
    unsigned char* mine = ad_smem + 16 * KROW + warp * WARP_BYTES;
    float* part = reinterpret_cast<float*>(ad_smem + 16 * KROW); // after the walk: [warp][16 rows][DV + 2]
    pdl_wait();
    pdl_trigger();
    const int pos = positions[t];
    const int* bt = block_table + (size_t)seq_of_token[t] * max_blocks;
    const int kv_len = pos + 1;
    const int start = (window > 0 && kv_len > window) ? kv_len - window : 0;
    const int nkept = window > 0 ? min(keep_first, start) : 0;
    const int nkeys = nkept + kv_len - start;
    // with gridDim.z > 1 the groups of 16 keys are cut into as many runs, one a block; the runs' parts go to the
    // scratch and a second kernel adds them in order
    const int all_groups = (nkeys + 15) >> 4;
    const int per_run = (all_groups + (int)gridDim.z - 1) / (int)gridDim.z;
    const int g_lo = (int)blockIdx.z * per_run;
    const int ngroups = min(all_groups, g_lo + per_run);   // (one past this block's last group)

    for (int c = threadIdx.x; c < 16 * KCH; c += AD_WARPS * 32) {
        const int r = c / KCH, cc = c % KCH;
        const int hd = head0 + min(r, share - 1);   // rows past the group repeat its last head
        *reinterpret_cast<uint4*>(q_s + r * KROW + (ab_swz<KCHP>(r, cc) << 4)) =
            *reinterpret_cast<const uint4*>(q + (size_t)t * q_row_stride + (size_t)hd * DK + cc * 8);
    }
    auto issue = [&](int g, int stage) {
        unsigned char* ks = mine + stage * (K_BYTES + V_BYTES);
        unsigned char* vs = ks + K_BYTES;
        for (int c = lane; c < 16 * KCH; c += 32) {
            const int r = c / KCH, cc = c % KCH;
            const int n = min(g * 16 + r, nkeys - 1);
            const int key = n < nkept ? n : start + n - nkept;
            const int page = bt[key / S];
            cp_async16(ks + r * KROW + (ab_swz<KCHP>(r, cc) << 4),
                       k_pool + (((size_t)page * Hk + hk) * S + (key % S)) * DK + cc * 8);
        }
        for (int c = lane; c < 16 * VCH; c += 32) {
            const int r = c / VCH, cc = c % VCH;
            const int n = min(g * 16 + r, nkeys - 1);
            const int key = n < nkept ? n : start + n - nkept;
            const int page = bt[key / S];
            cp_async16(vs + r * VROW + (ab_swz<VCHP>(r, cc) << 4),
                       v_pool + (((size_t)page * (Hk / v_share) + hk / v_share) * S + (key % S)) * DV + cc * 8);
        }
    };
    if (g_lo + warp < ngroups) issue(g_lo + warp, 0);
    cp_async_commit();
    __syncthreads();   // the queries are in shared memory
    const int mi = lane >> 3;
    unsigned qf[DK / 16][4];
    {
        const int r = ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk)
            ldmatrix_x4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], q_s + r * KROW + (ab_swz<KCHP>(r, 2 * kk + (mi >> 1)) << 4));
    }
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int r0 = lane >> 2;
    const int hd0 = head0 + min(r0, share - 1), hd1 = head0 + min(r0 + 8, share - 1);
    const float sl[2] = {bias_exp > 0.f ? exp2f(-bias_exp * (float)(hd0 + 1) / (float)H) * AB_LOG2E : 0.f,
                         bias_exp > 0.f ? exp2f(-bias_exp * (float)(hd1 + 1) / (float)H) * AB_LOG2E : 0.f};
    int it = 0;
    for (int g = g_lo + warp; g < ngroups; g += AD_WARPS, ++it) {
        const int stage = it & 1;
        if (g + AD_WARPS < ngroups) issue(g + AD_WARPS, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        const unsigned char* ks = mine + stage * (K_BYTES + V_BYTES);
        const unsigned char* vs = ks + K_BYTES;
        float sc[2][4];
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[0][c] = sc[1][c] = 0.f;
        {
            const int r = ((mi >> 1) << 3) + (lane & 7);
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk) {
                unsigned b00, b01, b10, b11;
                ldmatrix_x4(b00, b01, b10, b11, ks + r * KROW + (ab_swz<KCHP>(r, 2 * kk + (mi & 1)) << 4));
                mma_bf16(sc[0], qf[kk], b00, b01);
                mma_bf16(sc[1], qf[kk], b10, b11);
            }
        }
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int n = g * 16 + nt * 8 + ((lane & 3) << 1) + c;
                    const int key = n < nkept ? n : start + n - nkept;
                    float& v = sc[nt][2 * hrow + c];
                    v = n < nkeys ? ab_score(v, scale_log2, cap_log2, cap_arg) - sl[hrow] * (float)(pos - key) : -INFINITY;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m[hrow], mx);   // (a group has at least one visible key: never -inf)
            const float alpha = exp2f(m[hrow] - m_new);
            float ps = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    float& v = sc[nt][2 * hrow + c];
                    v = exp2f(v - m_new);
                    ps += v;
                }
            l[hrow] = l[hrow] * alpha + ps;
            m[hrow] = m_new;
#pragma unroll
            for (int i2 = 0; i2 < DV / 8; ++i2) {
                o[i2][2 * hrow] *= alpha;
                o[i2][2 * hrow + 1] *= alpha;
            }
        }
        unsigned hi[4], lw[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const float a = sc[x >> 1][2 * (x & 1)], b = sc[x >> 1][2 * (x & 1) + 1];
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b);
            const float2 back = __bfloat1622float2(h2);
            hi[x] = *reinterpret_cast<const unsigned*>(&h2);
            lw[x] = pack_bf16(a - back.x, b - back.y);
        }
        const int rv = ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int nt = 0; nt < DV / 8; nt += 2) {
            unsigned v00, v01, v10, v11;
            ldmatrix_x4_trans(v00, v01, v10, v11, vs + rv * VROW + (ab_swz<VCHP>(rv, nt + (mi >> 1)) << 4));
            mma_bf16(o[nt], hi, v00, v01);
            mma_bf16(o[nt + 1], hi, v10, v11);
            mma_bf16(o[nt], lw, v00, v01);
            mma_bf16(o[nt + 1], lw, v10, v11);
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    __syncthreads();   // every warp is done with its stages: the same memory now takes the warps' parts
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
        l[hrow] += __shfl_xor_sync(0xffffffffu, l[hrow], 1);
        l[hrow] += __shfl_xor_sync(0xffffffffu, l[hrow], 2);
        float* p = part + ((size_t)warp * 16 + r0 + 8 * hrow) * (DV + 2);
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            p[nt * 8 + ((lane & 3) << 1)] = o[nt][2 * hrow];
            p[nt * 8 + ((lane & 3) << 1) + 1] = o[nt][2 * hrow + 1];
        }
        if ((lane & 3) == 0) { p[DV] = m[hrow]; p[DV + 1] = l[hrow]; }
    }
    __syncthreads();
    const int live = share;   // rows that are query heads
    for (int e = threadIdx.x; e < live * DV; e += AD_WARPS * 32) {
        const int r = e / DV, d = e - r * DV;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, part[((size_t)w * 16 + r) * (DV + 2) + DV]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) {
            const float* p = part + ((size_t)w * 16 + r) * (DV + 2);
            const float f = p[DV] == -INFINITY ? 0.f : exp2f(p[DV] - M);
            L += p[DV + 1] * f;
            acc += p[d] * f;
        }
        if (gridDim.z == 1) {
            float f = 1.f;
            if (sinks) ab_add_sink(sinks[head0 + r] * AB_LOG2E, M, L, f);
            if (gate_col >= 0) f *= ab_gate(q, q_row_stride, t, gate_col, head0 + r);
            const size_t at = (size_t)t * out_row_stride + (size_t)(head0 + r) * DV + d;
            if (out_f32) reinterpret_cast<float*>(out)[at] = acc * f / L;
            else out[at] = __float2bfloat16_rn(acc * f / L);
        } else {
            float* dst = scratch + (((size_t)t * H + head0 + r) * gridDim.z + blockIdx.z) * (DV + 2);
            dst[d] = acc;
            if (d == 0) { dst[DV] = M; dst[DV + 1] = L; }
        }
    }
}

// The runs' parts of one (token, head), added in order: out = sum_z acc_z 2^(M_z - M) / sum_z L_z 2^(M_z - M).
__global__ void biased_decode_join_kernel(const float* __restrict__ scratch, bf16* __restrict__ out, int out_row_stride,
                                          int H, int DV, int runs, const float* __restrict__ sinks,
                                          const bf16* __restrict__ qrows, int q_row_stride, int gate_col, int out_f32) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* p = scratch + ((size_t)t * H + h) * runs * (DV + 2);
    float M = -INFINITY;
    for (int z = 0; z < runs; ++z) M = fmaxf(M, p[(size_t)z * (DV + 2) + DV]);
    for (int d = threadIdx.x; d < DV; d += blockDim.x) {
        float L = 0.f, acc = 0.f;
        for (int z = 0; z < runs; ++z) {
            const float* q = p + (size_t)z * (DV + 2);
            const float f = q[DV] == -INFINITY ? 0.f : exp2f(q[DV] - M);
            L += q[DV + 1] * f;
            acc += q[d] * f;
        }
        float f = 1.f;
        if (sinks) ab_add_sink(sinks[h] * AB_LOG2E, M, L, f);
        if (gate_col >= 0) f *= ab_gate(qrows, q_row_stride, t, gate_col, h);
        const size_t at = (size_t)t * out_row_stride + (size_t)h * DV + d;
        if (out_f32) reinterpret_cast<float*>(out)[at] = acc * f / L;
        else out[at] = __float2bfloat16_rn(acc * f / L);
    }
}

template <int DK, int DV>
static int launch_biased_decode(const bf16* q, int q_row_stride, const bf16* k_pool, const bf16* v_pool,
                                const int* block_table, int max_blocks, const int* seq_of_token, const int* positions,
                                bf16* out, int out_row_stride, float scale, float bias_exp, int window, int keep_first,
                                int tokens, int H, int Hk, int S, float* scratch, int runs, const float* sinks, int gate_col,
                                float softcap, int v_share, int out_f32, cudaStream_t stream) {
    constexpr int KROW = ab_pow2(DK / 8) * 16, VROW = ab_pow2(DV / 8) * 16;
    const size_t walk = (size_t)AD_WARPS * 2 * (16 * KROW + 16 * VROW), parts = (size_t)AD_WARPS * 16 * (DV + 2) * 4;
    const size_t smem = 16 * KROW + (walk > parts ? walk : parts);
    static bool configured[VX_MAX_DEVICES];
    if (int rc = vx_configure_smem(biased_decode_kernel<DK, DV>, smem, configured)) return rc;
    const int G = H / Hk;
    int share_log2 = 0;
    if (G > 1 && G <= 16 && (G & (G - 1)) == 0)
        while ((1 << share_log2) < G) ++share_log2;
    if (runs < 1 || !scratch) runs = 1;
    dim3 grid(share_log2 ? Hk : H, tokens, runs);
    VX_LAUNCH_K(VX_K_ATTENTION, (biased_decode_kernel<DK, DV>), grid, AD_WARPS * 32, smem, stream, q, q_row_stride, k_pool,
                v_pool, block_table, max_blocks, seq_of_token, positions, out, out_row_stride, scale * AB_LOG2E, bias_exp,
                window, keep_first, H, Hk, S, share_log2, scratch, sinks, gate_col, softcap * AB_LOG2E,
                softcap > 0.f ? scale / softcap : 0.f, v_share, out_f32);
    if (runs > 1)
        VX_LAUNCH_K(VX_K_JOIN, biased_decode_join_kernel, dim3(tokens, H), DV >= 128 ? 128 : 64, 0, stream, (const float*)scratch,
                    out, out_row_stride, H, DV, runs, sinks, q, q_row_stride, gate_col, out_f32);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

template <int DK, int DV>
static int launch_biased(const bf16* q, int q_row_stride, const bf16* k_pool, const bf16* v_pool, const int* block_table,
                         int max_blocks, AbSegments seg, bf16* out, int out_row_stride, float scale, float bias_exp,
                         int window, int keep_first, int segments, int max_new, int H, int Hk, int S, const float* sinks,
                         int gate_col, float softcap, const AbLayout* layout, int v_share, int out_f32, cudaStream_t stream) {
    constexpr int KROW = ab_chunks(DK / 8) * 16, VROW = ab_chunks(DV / 8) * 16;
    const size_t smem = (size_t)AB_BM * KROW + 2 * ((size_t)AB_BN * KROW + (size_t)AB_BN * VROW);
    static bool configured[VX_MAX_DEVICES];
    if (int rc = vx_configure_smem(biased_attention_kernel<DK, DV>, smem, configured)) return rc;
    const int G = H / Hk;
    int share_log2 = 0;
    if (G > 1 && G <= 16 && (G & (G - 1)) == 0)
        while ((1 << share_log2) < G) ++share_log2;
    const int toks_per_tile = AB_BM >> share_log2;
    AbLayout lay = {(long long)Hk * S * DK, (long long)S * DK, DK, (long long)(Hk / v_share) * S * DV, (long long)S * DV, DV, 0,
                    v_share, out_f32};
    if (layout) lay = *layout;
    dim3 grid((max_new + toks_per_tile - 1) / toks_per_tile, share_log2 ? Hk : H, segments);
    VX_LAUNCH_K(VX_K_ATTENTION, (biased_attention_kernel<DK, DV>), grid, AB_WARPS * 32, smem, stream, q, q_row_stride, k_pool,
                v_pool, block_table, max_blocks, seg, out, out_row_stride, scale * AB_LOG2E, bias_exp, window, keep_first, H,
                Hk, S, share_log2, sinks, gate_col, softcap * AB_LOG2E, softcap > 0.f ? scale / softcap : 0.f, lay);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// Portions: cu_seqlens and kv_offsets given, `segments` requests of up to `max_new` tokens.  Single tokens:
// cu_seqlens null, seq_of_token and positions given, `segments` token rows (max_new = 1); with `runs` > 1 and a
// float32 scratch of segments * H * runs * (DV + 2) elements a token's keys are cut into runs, a block each.
// With softcap c > 0 a scaled score s becomes c tanh(s / c) before the bias by distance and the softmax.
static int biased_attention_any(const void* q, int q_row_stride, const void* k_pool, const void* v_pool,
                                       const int* block_table, int max_blocks, const int* cu_seqlens, const int* kv_offsets,
                                       const int* seq_of_token, const int* positions, void* out, int out_row_stride,
                                       float scale, float bias_exp, int window, int keep_first, int segments, int max_new,
                                       int H, int Hk, int DK, int DV, int S, float* scratch, int runs, const float* sinks,
                                       int gate_col, float softcap, const int* seq_list, const AbLayout* layout,
                                       int v_share, int out_f32, cudaStream_t stream) {
    if (segments <= 0 || max_new <= 0) return VX_OK;
    if (v_share <= 0) v_share = 1;
    if (softcap < 0.f || Hk % v_share || (layout && v_share > 1)) return VX_ERR_SHAPE;
    if (H <= 0 || Hk <= 0 || H % Hk || S <= 0 || S % 16 || window < 0 || keep_first < 0 || bias_exp < 0.f) return VX_ERR_SHAPE;
    if (cu_seqlens ? !kv_offsets : (!seq_of_token || !positions || max_new != 1)) return VX_ERR_SHAPE;
    if (H > 65535 || segments > 65535) return VX_ERR_LIMIT;
    if ((q_row_stride & 7) || (((uintptr_t)q) & 15) || (out_row_stride & 1) || (((uintptr_t)out) & (out_f32 ? 7 : 3)))
        return VX_ERR_ALIGN;
    if (layout && (!cu_seqlens || ((layout->k_page | layout->k_head | layout->k_row | layout->v_page | layout->v_head | layout->v_row) & 7) ||
                   (((uintptr_t)k_pool | (uintptr_t)v_pool) & 15)))
        return VX_ERR_ALIGN;
    if (!cu_seqlens) {
        if (segments > 65535 || seq_list) return VX_ERR_LIMIT;
#define AD_GO(K_, V_)                                                                                                       \
    if (DK == K_ && DV == V_)                                                                                               \
        return launch_biased_decode<K_, V_>((const bf16*)q, q_row_stride, (const bf16*)k_pool, (const bf16*)v_pool,       \
                                            block_table, max_blocks, seq_of_token, positions, (bf16*)out, out_row_stride, \
                                            scale, bias_exp, window, keep_first, segments, H, Hk, S, scratch, runs, sinks,  \
                                            gate_col, softcap, v_share, out_f32, stream)
        AD_GO(64, 32); AD_GO(64, 64); AD_GO(64, 128); AD_GO(128, 32); AD_GO(128, 64); AD_GO(128, 128);
        AD_GO(32, 32); AD_GO(48, 48); AD_GO(80, 80); AD_GO(96, 96); AD_GO(112, 112);
#undef AD_GO
        return VX_ERR_SHAPE;
    }
    AbSegments seg = {cu_seqlens, kv_offsets, seq_of_token, positions, seq_list};
#define AB_GO(K_, V_)                                                                                                     \
    if (DK == K_ && DV == V_)                                                                                             \
        return launch_biased<K_, V_>((const bf16*)q, q_row_stride, (const bf16*)k_pool, (const bf16*)v_pool, block_table, \
                                     max_blocks, seg, (bf16*)out, out_row_stride, scale, bias_exp, window, keep_first,    \
                                     segments, max_new, H, Hk, S, sinks, gate_col, softcap, layout, v_share, out_f32, stream)
    AB_GO(64, 32); AB_GO(64, 64); AB_GO(64, 128); AB_GO(128, 32); AB_GO(128, 64); AB_GO(128, 128);
    AB_GO(32, 32); AB_GO(48, 48); AB_GO(80, 80); AB_GO(96, 96); AB_GO(112, 112);
    AB_GO(192, 128); AB_GO(192, 64); AB_GO(96, 64); AB_GO(96, 32); AB_GO(256, 128);   // (portions only: no kernel for single tokens)
#undef AB_GO
    return VX_ERR_SHAPE;
}

// `v_share` > 1: that many consecutive key heads read one value head (the value pool is [page, Hk / v_share, S, DV]);
// `out_f32`: out is float32 [tokens, out_row_stride] whatever the inputs' type.
extern "C" int vx_biased_attention_shared(const void* q, int q_row_stride, const void* k_pool, const void* v_pool,
                                          const int* block_table, int max_blocks, const int* cu_seqlens, const int* kv_offsets,
                                          const int* seq_of_token, const int* positions, void* out, int out_row_stride,
                                          float scale, float bias_exp, int window, int keep_first, int segments, int max_new,
                                          int H, int Hk, int DK, int DV, int S, float* scratch, int runs, const float* sinks,
                                          int gate_col, float softcap, int v_share, int out_f32, cudaStream_t stream) {
    return biased_attention_any(q, q_row_stride, k_pool, v_pool, block_table, max_blocks, cu_seqlens, kv_offsets, seq_of_token,
                                positions, out, out_row_stride, scale, bias_exp, window, keep_first, segments, max_new, H, Hk,
                                DK, DV, S, scratch, runs, sinks, gate_col, softcap, nullptr, nullptr, v_share, out_f32, stream);
}

extern "C" int vx_biased_attention_cap(const void* q, int q_row_stride, const void* k_pool, const void* v_pool,
                                       const int* block_table, int max_blocks, const int* cu_seqlens, const int* kv_offsets,
                                       const int* seq_of_token, const int* positions, void* out, int out_row_stride,
                                       float scale, float bias_exp, int window, int keep_first, int segments, int max_new,
                                       int H, int Hk, int DK, int DV, int S, float* scratch, int runs, const float* sinks,
                                       int gate_col, float softcap, cudaStream_t stream) {
    return vx_biased_attention_shared(q, q_row_stride, k_pool, v_pool, block_table, max_blocks, cu_seqlens, kv_offsets,
                                      seq_of_token, positions, out, out_row_stride, scale, bias_exp, window, keep_first, segments,
                                      max_new, H, Hk, DK, DV, S, scratch, runs, sinks, gate_col, softcap, 1, 0, stream);
}

// Portions whose keys and values lie as rows that a matrix product left: key j of head hk of segment s at
// k + (table[s][j / S] * S + j % S) * k_row + hk * k_head (values alike); segment s is request seq_list[s] (null: s) in
// cu_seqlens and kv_offsets.  Causal, with a window > 0 only the last `window` positions up to a query's own (the table
// then needs true entries only from the block of the first key that the segment's first query sees); no bias by
// distance, no sink or gate.
extern "C" int vx_biased_attention_rows_window(const void* q, int q_row_stride, const void* k, long long k_row, long long k_head,
                                               const void* v, long long v_row, long long v_head, const int* block_table,
                                               int max_blocks, const int* cu_seqlens, const int* kv_offsets, const int* seq_list,
                                               void* out, int out_row_stride, float scale, int segments, int max_new, int H,
                                               int Hk, int DK, int DV, int S, float softcap, int window, cudaStream_t stream) {
    AbLayout lay = {k_row * S, k_head, k_row, v_row * S, v_head, v_row, 1, 1, 0};
    if (k_row < DK || v_row < DV || window < 0) return VX_ERR_SHAPE;
    return biased_attention_any(q, q_row_stride, k, v, block_table, max_blocks, cu_seqlens, kv_offsets, nullptr, nullptr, out,
                                out_row_stride, scale, 0.f, window, 0, segments, max_new, H, Hk, DK, DV, S, nullptr, 1, nullptr, -1,
                                softcap, seq_list, &lay, 1, 0, stream);
}

extern "C" int vx_biased_attention_rows(const void* q, int q_row_stride, const void* k, long long k_row, long long k_head,
                                        const void* v, long long v_row, long long v_head, const int* block_table,
                                        int max_blocks, const int* cu_seqlens, const int* kv_offsets, const int* seq_list,
                                        void* out, int out_row_stride, float scale, int segments, int max_new, int H, int Hk,
                                        int DK, int DV, int S, float softcap, cudaStream_t stream) {
    return vx_biased_attention_rows_window(q, q_row_stride, k, k_row, k_head, v, v_row, v_head, block_table, max_blocks,
                                           cu_seqlens, kv_offsets, seq_list, out, out_row_stride, scale, segments, max_new, H, Hk,
                                           DK, DV, S, softcap, 0, stream);
}

extern "C" int vx_biased_attention(const void* q, int q_row_stride, const void* k_pool, const void* v_pool,
                                   const int* block_table, int max_blocks, const int* cu_seqlens, const int* kv_offsets,
                                   const int* seq_of_token, const int* positions, void* out, int out_row_stride,
                                   float scale, float bias_exp, int window, int keep_first, int segments, int max_new,
                                   int H, int Hk, int DK, int DV, int S, float* scratch, int runs, const float* sinks,
                                   int gate_col, cudaStream_t stream) {
    return vx_biased_attention_cap(q, q_row_stride, k_pool, v_pool, block_table, max_blocks, cu_seqlens, kv_offsets,
                                   seq_of_token, positions, out, out_row_stride, scale, bias_exp, window, keep_first, segments,
                                   max_new, H, Hk, DK, DV, S, scratch, runs, sinks, gate_col, 0.f, stream);
}
