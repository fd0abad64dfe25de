// Kernels around mixers with a recurrent state or a latent cache, and around blocks whose
// sublayers run side by side:
//   linear_attention_walk   S_p = a_p (.) S_(p-1) + k_p v_p^T, o_p = S_p^T q_p with the decay a number per
//                           head or a number per key channel and position; q and k optionally rotated by
//                           position and multiplied by numbers on the way in
//   stretch_log_decay, stretch_scan   a long portion cut into stretches that are walked side by side
//   head_norm_gate          every head's output divided by its root mean square (optionally times a
//                           weight shared by the heads), times silu or sigmoid of a gate projection
//   latent_prep             the down-projected row of a latent attention: norm of the latent part, rotation
//                           of the shared key part, both into the page; rotation of the queries' rotated part
//   capped_gated_act        min(g, L) sigmoid(s min(g, L)) (clamp(u, -L, L) + 1) on float32 sums plus biases
//   sum_add_rmsnorm         residual += c0 y0 + c1 y1 + c2 y2 + rows + vector; optionally the norm of the sum
//   softcap_rows            c tanh(x / c)
// All statistics, sums, angles, decays and states are float32; T is the element type of
// the activations that feed matrix products.
#include "common.cuh"

#define LW_COLS 32      // state columns of a block
#define LW_CC 4         // ... of a thread
#define LW_GROUPS 16    // row groups: 4 in a warp (lane bits 3, 4) times 4 warps
#define LW_CHUNK 16     // tokens staged at a time
#define LW_THREADS 128
// q, k and, with a gate, the decays of a chunk (rows padded to 16 R, R <= 16), v, the warps' partial outputs
#define LW_SMEM(DP, GATED) (sizeof(float) * LW_CHUNK * (((GATED) ? 3 : 2) * (DP) + LW_COLS + 4 * LW_COLS))
#define LW_MAX_SMEM LW_SMEM(256, 1)

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// A block owns LW_COLS columns of one head's state of one request; a thread owns a tile of R consecutive rows by 4
// consecutive columns (rows [g R, g R + R) for its row group g = 4 warp + (lane >> 3), columns 4 (lane & 7) ..), so a
// token costs it 2 (3 with a gate) R / 4 + 1 reads of 16 bytes from shared memory for 3 R 4 multiply-adds.  Tokens are
// staged LW_CHUNK at a time in shared memory, in float32, rows padded to 16 R with q = k = 0: q and k as the projection left
// them, turned by position * inv_freq[i] on the first rot_dim channels (pairs (i, i + rot_dim/2), or (2i, 2i + 1) when
// `interleaved`), then times q_mul / k_mul.  The decay of channel d at token t is decay[h] (`gate` null), or
// exp(gate_mul * log_sigmoid(gate[t, h D + d])): sigmoid(z)^(gate_mul), formed through the logarithm.  A token's output
// column is summed over a thread's rows in order, then over the 4 row groups of a warp by two exchanges, then over the warps
// in warp order (through shared memory, once a chunk): an order fixed by D alone.
__device__ __forceinline__ void lw_load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void lw_load8(const bf16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h2[e]);
        v[2 * e] = f.x;
        v[2 * e + 1] = f.y;
    }
}

template <typename T, int R, bool GATED>
__global__ void __launch_bounds__(LW_THREADS, 4)
linear_attention_walk_kernel(const T* __restrict__ x, int ldx, int q_col, int k_col, int v_col,
                             const float* __restrict__ decay, const float* __restrict__ gate, int ldg, float gate_mul,
                             const float* __restrict__ inv_freq, int rot_dim, int interleaved,
                             const int* __restrict__ positions, float q_mul, float k_mul, float* __restrict__ state,
                             const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                             float* __restrict__ out, int H, int D, int Dv, int fresh) {
    extern __shared__ __align__(16) float smem[];
    constexpr int DP = LW_GROUPS * R;
    float* q_s = smem;                            // [LW_CHUNK][DP]
    float* k_s = q_s + LW_CHUNK * DP;             // [LW_CHUNK][DP]
    float* v_s = k_s + LW_CHUNK * DP;             // [LW_CHUNK][LW_COLS]
    float* o_s = v_s + LW_CHUNK * LW_COLS;        // [4 warps][LW_CHUNK][LW_COLS]
    float* a_s = o_s + 4 * LW_CHUNK * LW_COLS;    // [LW_CHUNK][DP] (with a gate only)
    const int col0 = blockIdx.x * LW_COLS, h = blockIdx.y, seq = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cg = lane & 7, row0 = (warp * 4 + (lane >> 3)) * R, c0 = col0 + cg * LW_CC;
    const float dec = GATED ? 1.f : decay[h];
    const int half = rot_dim >> 1;
    const bool by_eights = (D & 7) == 0 && ((size_t)ldx * sizeof(T) & 15) == 0 && (((uintptr_t)(x + q_col)) & 15) == 0 &&
                           (((uintptr_t)(x + k_col)) & 15) == 0 && (!GATED || ((ldg & 3) == 0 && (((uintptr_t)gate) & 15) == 0));
    pdl_wait();
    pdl_trigger();
    const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
    float* st = state + (((size_t)state_slots[seq] * H + h) * D) * Dv;
    float S[R][LW_CC];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < LW_CC; ++c)
            S[r][c] = (!fresh && row0 + r < D && c0 + c < Dv) ? st[(size_t)(row0 + r) * Dv + c0 + c] : 0.f;
    for (int tb = t0; tb < t1; tb += LW_CHUNK) {
        const int n = min(LW_CHUNK, t1 - tb);
        __syncthreads();
        // q and k of channels that are not turned take their multipliers here, the turned ones after the turn
        auto stage = [&](int i) {
            const int tt = i / DP, d = i - tt * DP;
            float qv = 0.f, kv = 0.f, av = 1.f;
            if (d < D) {
                const T* row = x + (size_t)(tb + tt) * ldx + (size_t)h * D + d;
                const bool turned = inv_freq && d < rot_dim;
                qv = to_f32(row[q_col]) * (turned ? 1.f : q_mul);
                kv = to_f32(row[k_col]) * (turned ? 1.f : k_mul);
                if (GATED) av = expf(gate_mul * log_sigmoid(gate[(size_t)(tb + tt) * ldg + (size_t)h * D + d]));
            }
            q_s[i] = qv;
            k_s[i] = kv;
            if (GATED) a_s[i] = av;
        };
        auto stage_v = [&](int i) {
            const int tt = i / LW_COLS, cc = i - tt * LW_COLS;
            v_s[i] = (col0 + cc < Dv) ? to_f32(x[(size_t)(tb + tt) * ldx + v_col + (size_t)h * Dv + col0 + cc]) : 0.f;
        };
        // eight channels at a time where rows, columns and sizes lie on 16-byte borders
        auto stage8 = [&](int g) {
            const int tt = g / (DP / 8), d = (g - tt * (DP / 8)) * 8;
            float qv[8], kv[8], av[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) { qv[e] = 0.f; kv[e] = 0.f; av[e] = 1.f; }
            if (d < D) {
                const T* row = x + (size_t)(tb + tt) * ldx + (size_t)h * D + d;
                lw_load8(row + q_col, qv);
                lw_load8(row + k_col, kv);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const bool turned = inv_freq && d + e < rot_dim;
                    qv[e] *= turned ? 1.f : q_mul;
                    kv[e] *= turned ? 1.f : k_mul;
                }
                if (GATED) {
                    lw_load8(gate + (size_t)(tb + tt) * ldg + (size_t)h * D + d, av);
#pragma unroll
                    for (int e = 0; e < 8; ++e) av[e] = expf(gate_mul * log_sigmoid(av[e]));
                }
            }
            const int i = tt * DP + d;
            *reinterpret_cast<float4*>(q_s + i) = make_float4(qv[0], qv[1], qv[2], qv[3]);
            *reinterpret_cast<float4*>(q_s + i + 4) = make_float4(qv[4], qv[5], qv[6], qv[7]);
            *reinterpret_cast<float4*>(k_s + i) = make_float4(kv[0], kv[1], kv[2], kv[3]);
            *reinterpret_cast<float4*>(k_s + i + 4) = make_float4(kv[4], kv[5], kv[6], kv[7]);
            if (GATED) {
                *reinterpret_cast<float4*>(a_s + i) = make_float4(av[0], av[1], av[2], av[3]);
                *reinterpret_cast<float4*>(a_s + i + 4) = make_float4(av[4], av[5], av[6], av[7]);
            }
        };
        if (n == LW_CHUNK && by_eights) {
#pragma unroll
            for (int it = 0; it < LW_CHUNK * DP / 8 / LW_THREADS; ++it) stage8(threadIdx.x + it * LW_THREADS);
#pragma unroll
            for (int it = 0; it < LW_CHUNK * LW_COLS / LW_THREADS; ++it) stage_v(threadIdx.x + it * LW_THREADS);
        } else if (n == LW_CHUNK) {   // a whole chunk: a fixed number of rounds, so that a thread's loads are all in flight together
#pragma unroll
            for (int it = 0; it < LW_CHUNK * DP / LW_THREADS; ++it) stage(threadIdx.x + it * LW_THREADS);
#pragma unroll
            for (int it = 0; it < LW_CHUNK * LW_COLS / LW_THREADS; ++it) stage_v(threadIdx.x + it * LW_THREADS);
        } else {
            for (int i = threadIdx.x; i < n * DP; i += LW_THREADS) stage(i);
            for (int i = threadIdx.x; i < n * LW_COLS; i += LW_THREADS) stage_v(i);
        }
        __syncthreads();
        if (inv_freq && half > 0) {
            for (int i = threadIdx.x; i < n * half; i += LW_THREADS) {
                const int tt = i / half, p = i - tt * half;
                float sn, cs;
                sincosf((float)positions[tb + tt] * inv_freq[p], &sn, &cs);
                const int ia = tt * DP + (interleaved ? 2 * p : p), ib = tt * DP + (interleaved ? 2 * p + 1 : p + half);
                const float qa = q_s[ia], qb = q_s[ib], ka = k_s[ia], kb = k_s[ib];
                q_s[ia] = (qa * cs - qb * sn) * q_mul;
                q_s[ib] = (qb * cs + qa * sn) * q_mul;
                k_s[ia] = (ka * cs - kb * sn) * k_mul;
                k_s[ib] = (kb * cs + ka * sn) * k_mul;
            }
            __syncthreads();
        }
        for (int tt = 0; tt < n; ++tt) {
            const float4 v4 = *reinterpret_cast<const float4*>(v_s + tt * LW_COLS + cg * LW_CC);
            const float v[LW_CC] = {v4.x, v4.y, v4.z, v4.w};
            float o[LW_CC] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r4 = 0; r4 < R; r4 += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(k_s + tt * DP + row0 + r4);
                const float4 q4 = *reinterpret_cast<const float4*>(q_s + tt * DP + row0 + r4);
                float4 a4 = make_float4(dec, dec, dec, dec);
                if (GATED) a4 = *reinterpret_cast<const float4*>(a_s + tt * DP + row0 + r4);
                const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w}, aa[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int c = 0; c < LW_CC; ++c) {
                        S[r4 + r][c] = fmaf(aa[r], S[r4 + r][c], kk[r] * v[c]);
                        o[c] = fmaf(S[r4 + r][c], qq[r], o[c]);
                    }
            }
            if (out) {
                // over the warp's 4 row groups: the upper pair keeps columns 2, 3 and the lower pair 0, 1, then odd groups keep
                // the second of their two; lane (g, cg) ends with column 4 cg + 2 (g >> 1) + (g & 1)
                const bool hi = lane & 16, mid = lane & 8;
                const float r0 = __shfl_xor_sync(0xffffffffu, hi ? o[0] : o[2], 16);
                const float r1 = __shfl_xor_sync(0xffffffffu, hi ? o[1] : o[3], 16);
                const float a0 = (hi ? o[2] : o[0]) + r0, a1 = (hi ? o[3] : o[1]) + r1;
                const float r2 = __shfl_xor_sync(0xffffffffu, mid ? a0 : a1, 8);
                o_s[(warp * LW_CHUNK + tt) * LW_COLS + cg * LW_CC + (hi ? 2 : 0) + (mid ? 1 : 0)] = (mid ? a1 : a0) + r2;
            }
        }
        if (out) {
            __syncthreads();
            for (int i = threadIdx.x; i < n * LW_COLS; i += LW_THREADS) {
                const int tt = i / LW_COLS, cc = i - tt * LW_COLS;
                if (col0 + cc < Dv)
                    out[(size_t)(tb + tt) * H * Dv + (size_t)h * Dv + col0 + cc] =
                        ((o_s[i] + o_s[LW_CHUNK * LW_COLS + i]) + o_s[2 * LW_CHUNK * LW_COLS + i]) + o_s[3 * LW_CHUNK * LW_COLS + i];
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < LW_CC; ++c)
            if (row0 + r < D && c0 + c < Dv) st[(size_t)(row0 + r) * Dv + c0 + c] = S[r][c];
}

template <typename T>
static int launch_linear_attention_walk(const T* x, int ldx, int q_col, int k_col, int v_col, const float* decay,
                                        const float* gate, int ldg, float gate_mul, const float* inv_freq, int rot_dim,
                                        int interleaved, const int* positions, float q_mul, float k_mul, float* state,
                                        const int* cu_seqlens, const int* state_slots, float* out, int seqs, int H, int D,
                                        int Dv, int fresh, cudaStream_t stream) {
    dim3 grid((Dv + LW_COLS - 1) / LW_COLS, H, seqs);
    static bool configured[8][VX_MAX_DEVICES];
#define LW_GO(R_, G_, SLOT)                                                                                                \
    do {                                                                                                                   \
        if (int rc = vx_configure_smem(linear_attention_walk_kernel<T, R_, G_>, LW_MAX_SMEM, configured[SLOT])) return rc; \
        VX_LAUNCH_K(VX_K_ATTENTION, (linear_attention_walk_kernel<T, R_, G_>), grid, LW_THREADS, LW_SMEM(LW_GROUPS * R_, G_), \
                    stream, x, ldx, q_col, k_col, v_col, decay, gate, ldg, gate_mul, inv_freq, rot_dim, interleaved,       \
                    positions, q_mul, k_mul, state, cu_seqlens, state_slots, out, H, D, Dv, fresh);                        \
    } while (0)
#define LW_GO_R(R_, SLOT)                                                                                                  \
    do {                                                                                                                   \
        if (gate) LW_GO(R_, true, 2 * SLOT); else LW_GO(R_, false, 2 * SLOT + 1);                                          \
    } while (0)
    if (D <= 64) LW_GO_R(4, 0);
    else if (D <= 128) LW_GO_R(8, 1);
    else if (D <= 192) LW_GO_R(12, 2);
    else LW_GO_R(16, 3);
#undef LW_GO_R
#undef LW_GO
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// x: rows with q, k [H, D] and v [H, Dv] at the given columns.  decay [H] or gate [tokens, ldg] (float32; one
// of the two).  state float32 [slot, H, D, Dv], read (from zero instead with `fresh`) and written back.  out float32
// [tokens, H * Dv], or null where only the states are wanted.
extern "C" int vx_linear_attention_walk_parts(const void* x, int ldx, int q_col, int k_col, int v_col, const float* decay,
                                              const float* gate, int ldg, float gate_mul, const float* inv_freq, int rot_dim,
                                              int interleaved, const int* positions, float q_mul, float k_mul, float* state,
                                              const int* cu_seqlens, const int* state_slots, float* out, int seqs, int H,
                                              int D, int Dv, int fresh, int dtype, cudaStream_t stream) {
    if (seqs <= 0) return VX_OK;
    if (H <= 0 || D <= 0 || Dv <= 0 || D > 256 || q_col < 0 || k_col < 0 || v_col < 0) return VX_ERR_SHAPE;
    if ((decay == nullptr) == (gate == nullptr)) return VX_ERR_SHAPE;
    if (gate && ldg < H * D) return VX_ERR_SHAPE;
    if (rot_dim < 0 || rot_dim > D || (rot_dim & 1) || (inv_freq && rot_dim > 0 && !positions)) return VX_ERR_SHAPE;
    if (seqs > 65535 || H > 65535) return VX_ERR_LIMIT;
    if (dtype == VX_F32)
        return launch_linear_attention_walk<float>((const float*)x, ldx, q_col, k_col, v_col, decay, gate, ldg, gate_mul,
                                                   inv_freq, rot_dim, interleaved, positions, q_mul, k_mul, state,
                                                   cu_seqlens, state_slots, out, seqs, H, D, Dv, fresh, stream);
    if (dtype == VX_BF16)
        return launch_linear_attention_walk<bf16>((const bf16*)x, ldx, q_col, k_col, v_col, decay, gate, ldg, gate_mul,
                                                  inv_freq, rot_dim, interleaved, positions, q_mul, k_mul, state,
                                                  cu_seqlens, state_slots, out, seqs, H, D, Dv, fresh, stream);
    return VX_ERR_DTYPE;
}

extern "C" int vx_linear_attention_walk(const void* x, int ldx, int q_col, int k_col, int v_col, const float* decay,
                                        const float* gate, int ldg, float gate_mul, const float* inv_freq, int rot_dim,
                                        int interleaved, const int* positions, float q_mul, float k_mul, float* state,
                                        const int* cu_seqlens, const int* state_slots, float* out, int seqs, int H,
                                        int D, int Dv, int dtype, cudaStream_t stream) {
    if (!out) return VX_ERR_SHAPE;
    return vx_linear_attention_walk_parts(x, ldx, q_col, k_col, v_col, decay, gate, ldg, gate_mul, inv_freq, rot_dim,
                                          interleaved, positions, q_mul, k_mul, state, cu_seqlens, state_slots, out, seqs, H,
                                          D, Dv, 0, dtype, stream);
}

// A long portion walked in stretches side by side.  With every stretch's own contribution S_loc[c] (the walk from a zero
// state, `fresh`) and the decay over the whole stretch A_c (per head, or per key channel), the state at a stretch's start
// follows from the one before it: S_start[c + 1] = diag(A_c) S_start[c] + S_loc[c]; a second walk of every stretch from its
// start state gives the outputs.  Two kernels around the walks:
//   stretch_log_decay  log A_c [stretch, H D] = sum over the stretch's tokens of gate_mul * log_sigmoid(gate)
//   stretch_scan       per request, in the order of its stretches: parts[c] (holding S_loc[c]) takes S_start[c]; the state
//                      slot takes the state after the last stretch.  One thread per state element.
__global__ void stretch_log_decay_kernel(const float* __restrict__ gate, int ldg, float gate_mul,
                                         const int* __restrict__ cu_stretch, float* __restrict__ log_a, int HD) {
    pdl_wait();
    pdl_trigger();
    const int c = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= HD) return;
    float sum = 0.f;
    for (int t = cu_stretch[c]; t < cu_stretch[c + 1]; ++t) sum += gate_mul * log_sigmoid(gate[(size_t)t * ldg + i]);
    log_a[(size_t)c * HD + i] = sum;
}

__global__ void stretch_scan_kernel(float* __restrict__ parts, float* __restrict__ state, const float* __restrict__ log_a,
                                    const float* __restrict__ decay, const int* __restrict__ cu_stretch,
                                    const int* __restrict__ first_stretch, const int* __restrict__ state_slots, int H, int D,
                                    int Dv) {
    pdl_wait();
    pdl_trigger();
    const int seq = blockIdx.y;
    const size_t per = (size_t)H * D * Dv;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per) return;
    const int hd = (int)(e / Dv), h = hd / D;
    float* st = state + (size_t)state_slots[seq] * per + e;
    float S = *st;
    const float l2 = decay ? log2f(decay[h]) : 0.f;
    const int last = first_stretch[seq + 1];
    for (int c = first_stretch[seq]; c < last; c += 4) {   // (four stretches' reads in flight before the first write)
        float loc[4], a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (c + u >= last) continue;
            loc[u] = parts[(size_t)(c + u) * per + e];
            a[u] = log_a ? expf(log_a[(size_t)(c + u) * H * D + hd])
                         : exp2f((float)(cu_stretch[c + u + 1] - cu_stretch[c + u]) * l2);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (c + u >= last) continue;
            parts[(size_t)(c + u) * per + e] = S;
            S = fmaf(a[u], S, loc[u]);
        }
    }
    *st = S;
}

extern "C" int vx_stretch_log_decay(const float* gate, int ldg, float gate_mul, const int* cu_stretch, float* log_a,
                                    int stretches, int HD, cudaStream_t stream) {
    if (stretches <= 0) return VX_OK;
    if (HD <= 0 || ldg < HD) return VX_ERR_SHAPE;
    if (stretches > 65535) return VX_ERR_LIMIT;
    VX_LAUNCH_K(VX_K_ELEMENTWISE, stretch_log_decay_kernel, dim3((HD + 127) / 128, stretches), 128, 0, stream, gate, ldg,
                gate_mul, cu_stretch, log_a, HD);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// parts float32 [stretch, H, D, Dv]; log_a [stretch, H D] or null with decay [H]; the stretches of request i are
// first_stretch[i] .. first_stretch[i + 1] - 1, stretch c holds token rows cu_stretch[c] .. cu_stretch[c + 1] - 1.
extern "C" int vx_stretch_scan(float* parts, float* state, const float* log_a, const float* decay, const int* cu_stretch,
                               const int* first_stretch, const int* state_slots, int seqs, int H, int D, int Dv,
                               cudaStream_t stream) {
    if (seqs <= 0) return VX_OK;
    if (H <= 0 || D <= 0 || Dv <= 0 || ((log_a == nullptr) == (decay == nullptr))) return VX_ERR_SHAPE;
    const size_t per = (size_t)H * D * Dv;
    if (seqs > 65535 || (per + 255) / 256 > 0x7fffffffULL) return VX_ERR_LIMIT;
    VX_LAUNCH_K(VX_K_ELEMENTWISE, stretch_scan_kernel, dim3((unsigned)((per + 255) / 256), seqs), 256, 0, stream, parts, state,
                log_a, decay, cu_stretch, first_stretch, state_slots, H, D, Dv);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// One warp per (token, head): out = o / sqrt(mean(o^2) + eps) (* w[d]) * act(g), act = sigmoid (0) or silu (1).
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ g, int ldg,
                                      const float* __restrict__ w, T* __restrict__ out, int rows, int H, int Dv, float eps,
                                      int gate_act) {
    pdl_wait();
    pdl_trigger();
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= rows * H) return;
    const int t = unit / H, h = unit - t * H;
    const float* src = o + ((size_t)t * H + h) * Dv;
    float ss = 0.f;
    for (int d = lane; d < Dv; d += 32) { const float v = src[d]; ss += v * v; }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)Dv + eps);
    const T* gr = g + (size_t)t * ldg + (size_t)h * Dv;
    T* dst = out + ((size_t)t * H + h) * Dv;
    for (int d = lane; d < Dv; d += 32) {
        const float z = to_f32(gr[d]);
        const float sg = 1.f / (1.f + expf(-z));
        float v = src[d] * rstd;
        if (w) v *= w[d];
        dst[d] = from_f32<T>(v * (gate_act ? z * sg : sg));
    }
}

extern "C" int vx_head_norm_gate(const float* o, const void* g, int ldg, const float* w, void* out, int rows, int H,
                                 int Dv, float eps, int gate_act, int dtype, cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (H <= 0 || Dv <= 0 || ldg < H * Dv) return VX_ERR_SHAPE;
    const int warps = 4;
    const long long blocks = ((long long)rows * H + warps - 1) / warps;
    if (blocks > 0x7fffffffLL) return VX_ERR_LIMIT;
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (head_norm_gate_kernel<float>), (unsigned)blocks, warps * 32, 0, stream, o, (const float*)g, ldg, w, (float*)out, rows, H, Dv, eps, gate_act);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (head_norm_gate_kernel<bf16>), (unsigned)blocks, warps * 32, 0, stream, o, (const bf16*)g, ldg, w, (bf16*)out, rows, H, Dv, eps, gate_act);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// One block per token.  down [tokens, ldd]: C latent channels, then R channels of the key part that all heads
// share.  The latent part is RMS-normed with a plain weight and written, followed by the rotated key part
// (pairs (2i, 2i + 1) when `interleaved`, else (i, i + R/2), angle position * inv_freq[i]), to
// pool[slot] (rows of C + R elements; a negative slot writes nothing).  The queries q [tokens, ldq] hold, per
// head, D channels that stay and then R that are rotated the same way and written to the last R channels of the
// head's row of qa [tokens, H, C + R] (whose first C channels another kernel fills).
template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ down, int ldd, T* q, int ldq, T* qa,
                                   const float* __restrict__ w, float eps, const float* __restrict__ inv_freq,
                                   int interleaved, const int* __restrict__ positions,
                                   const int* __restrict__ slot_mapping, T* __restrict__ pool, int H, int D, int R, int C) {
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    const int half = R >> 1;
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    const T* dr = down ? down + (size_t)t * ldd : nullptr;   // (no row of its own: a layer that reads another's cache)
    float ss = 0.f;
    if (dr && slot >= 0)
        for (int i = threadIdx.x; i < C; i += blockDim.x) { const float v = to_f32(dr[i]); ss += v * v; }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)C + eps);
    if (dr && slot >= 0) {
        T* dst = pool + (size_t)slot * (C + R);
        for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = from_f32<T>(to_f32(dr[i]) * rstd * w[i]);
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
            const float a = to_f32(dr[C + ia]), b = to_f32(dr[C + ib]);
            dst[C + ia] = from_f32<T>(a * cs - b * sn);
            dst[C + ib] = from_f32<T>(b * cs + a * sn);
        }
    }
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, p = i - h * half;
        float sn, cs;
        sincosf(pos * inv_freq[p], &sn, &cs);
        T* qr = q + (size_t)t * ldq + (size_t)h * (D + R) + D;
        T* qo = qa ? qa + ((size_t)t * H + h) * (C + R) + C : qr;   // (without folded queries: turned where they are)
        const int ia = interleaved ? 2 * p : p, ib = interleaved ? 2 * p + 1 : p + half;
        const float a = to_f32(qr[ia]), b = to_f32(qr[ib]);
        qo[ia] = from_f32<T>(a * cs - b * sn);
        qo[ib] = from_f32<T>(b * cs + a * sn);
    }
}

extern "C" int vx_latent_prep(const void* down, int ldd, void* q, int ldq, void* qa, const float* w, float eps,
                              const float* inv_freq, int interleaved, const int* positions, const int* slot_mapping,
                              void* pool, int tokens, int H, int D, int R, int C, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (H <= 0 || D < 0 || R < 0 || (R & 1) || C <= 0 || (down && ldd < C + R) || ldq < H * (D + R)) return VX_ERR_SHAPE;
    if (R > 0 && !inv_freq) return VX_ERR_SHAPE;
    if (slot_mapping && (!pool || !down)) return VX_ERR_SHAPE;
    const int threads = C >= 512 ? 256 : 128;
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ROPE, (latent_prep_kernel<float>), tokens, threads, 0, stream, (const float*)down, ldd, (float*)q, ldq, (float*)qa, w, eps, inv_freq, interleaved, positions, slot_mapping, (float*)pool, H, D, R, C);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ROPE, (latent_prep_kernel<bf16>), tokens, threads, 0, stream, (const bf16*)down, ldd, (bf16*)q, ldq, (bf16*)qa, w, eps, inv_freq, interleaved, positions, slot_mapping, (bf16*)pool, H, D, R, C);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// sums [rows, 2 inner] float32: all gates, then all ups (without their biases); bias [2 inner] float32 or null.
// g = min(gate, L), u = clamp(up, -L, L); out = g sigmoid(slope g) (u + 1) in T.
template <typename T>
__global__ void capped_gated_act_kernel(const float* __restrict__ sums, const float* __restrict__ bias, T* __restrict__ out,
                                        long long total, int inner, float limit, float slope) {
    pdl_wait();
    pdl_trigger();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / inner;
        const int c = (int)(i - r * inner);
        float g = sums[r * 2 * inner + c], u = sums[r * 2 * inner + inner + c];
        if (bias) { g += bias[c]; u += bias[inner + c]; }
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        out[i] = from_f32<T>(g / (1.f + expf(-slope * g)) * (u + 1.f));
    }
}

extern "C" int vx_capped_gated_act(const float* sums, const float* bias, void* out, int rows, int inner, float limit,
                                   float slope, int dtype, cudaStream_t stream) {
    if (rows <= 0 || inner <= 0) return VX_OK;
    const long long total = (long long)rows * inner;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (capped_gated_act_kernel<float>), blocks, 256, 0, stream, sums, bias, (float*)out, total, inner, limit, slope);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (capped_gated_act_kernel<bf16>), blocks, 256, 0, stream, sums, bias, (bf16*)out, total, inner, limit, slope);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// One block per row.  residual (float32, in place) += c0 y0 + c1 y1 + c2 y2 + rows_add + vec, every term
// optional; then, with a weight, normed = residual / sqrt(mean(residual^2) + eps) * w in T.
template <typename T>
__global__ void sum_add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ y0, float c0,
                                       const T* __restrict__ y1, float c1, const T* __restrict__ y2, float c2,
                                       const float* __restrict__ rows_add, const float* __restrict__ vec,
                                       const float* __restrict__ w, T* __restrict__ normed, int width, float eps) {
    extern __shared__ float row_s[];
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = residual[base + i];
        float add = 0.f;
        if (y0) add = c0 * to_f32(y0[base + i]);
        if (y1) add += c1 * to_f32(y1[base + i]);
        if (y2) add += c2 * to_f32(y2[base + i]);
        v += add;
        if (rows_add) v += rows_add[base + i];
        if (vec) v += vec[i];
        residual[base + i] = v;
        row_s[i] = v;
        ss += v * v;
    }
    if (!w) return;
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) normed[base + i] = from_f32<T>(row_s[i] * rstd * w[i]);
}

extern "C" int vx_sum_add_rmsnorm(float* residual, const void* y0, float c0, const void* y1, float c1, const void* y2,
                                  float c2, const float* rows_add, const float* vec, const float* w, void* normed,
                                  int rows, int width, float eps, int dtype, cudaStream_t stream) {
    if (rows <= 0) return VX_OK;
    if (width <= 0 || (w && !normed)) return VX_ERR_SHAPE;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    const size_t smem = sizeof(float) * width;
    if (smem > 48 * 1024) return VX_ERR_LIMIT;
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (sum_add_rmsnorm_kernel<float>), rows, threads, smem, stream, residual, (const float*)y0, c0, (const float*)y1, c1, (const float*)y2, c2, rows_add, vec, w, (float*)normed, width, eps);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (sum_add_rmsnorm_kernel<bf16>), rows, threads, smem, stream, residual, (const bf16*)y0, c0, (const bf16*)y1, c1, (const bf16*)y2, c2, rows_add, vec, w, (bf16*)normed, width, eps);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

__global__ void softcap_rows_kernel(const float* __restrict__ x, float* __restrict__ out, long long total, float cap) {
    pdl_wait();
    pdl_trigger();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        out[i] = cap * tanhf(x[i] / cap);
}

extern "C" int vx_softcap_rows(const float* x, float* out, long long total, float cap, cudaStream_t stream) {
    if (total <= 0) return VX_OK;
    if (!(cap > 0.f)) return VX_ERR_SHAPE;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    VX_LAUNCH_K(VX_K_ELEMENTWISE, softcap_rows_kernel, blocks, 256, 0, stream, x, out, total, cap);
    VX_LAUNCH_CHECK();
    return VX_OK;
}
