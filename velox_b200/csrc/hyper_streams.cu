// A residual stream kept in several copies ("streams"), and the layer norm that reads them.
//
// The stream of a token is n rows of E float32 values, X[t] = [x_0 | x_1 | ... | x_(n-1)].  A sublayer reads ONE row,
// a weighted sum of the copies, normed; its output y is written back to all copies at once together with a mixing of
// the copies among themselves:
//   u      = sum_s in[s] x_s                         stream_norm      (then the norm of u, in the element type T)
//   x_t'   = sum_s mix[s, t] x_s + c out[t] ls (.) y   stream_update    (ls: a vector that scales y channel by channel;
//                                                                      mix is indexed [from, to]; all t from the OLD x_s)
// and stream_update may go on, in the same pass, with the NEXT sublayer's u and its norm, so that a sublayer costs one
// elementwise kernel.  With n = 1, mix = out = in = 1 this is the plain residual update with a layer scale.
// The norm is a layer norm without bias, (u - mean) / sqrt(mean((u - mean)^2) + eps) * w (the variance from the
// deviations, in a second pass over the row held in shared memory), or, with `rms`, u / sqrt(mean(u^2) + eps) * w.
// Everything is float32 but y and the normed output.
//
// One block per token.  stream_norm takes an optional list of rows (only those tokens are normed: the last norm before
// the output head), and an optional single-copy source: the token's row x [E] stands for n equal copies, which the
// kernel writes out (the first layer's entry).
#include "common.cuh"

#define HS_MAX_STREAMS 16
#define HS_THREADS 256
#define HS_MAX_THREADS 1024

// VEC consecutive channels of a row at a time: float4 of the stream, 8 or 16 bytes of T.
template <int VEC> __device__ __forceinline__ void hs_load(const float* p, float (&v)[VEC]) {
    if constexpr (VEC == 4) { const float4 t = *reinterpret_cast<const float4*>(p); v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w; }
    else v[0] = p[0];
}
template <int VEC> __device__ __forceinline__ void hs_load(const bf16* p, float (&v)[VEC]) {
    if constexpr (VEC == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    } else v[0] = __bfloat162float(p[0]);
}
template <int VEC> __device__ __forceinline__ void hs_store(float* p, const float (&v)[VEC]) {
    if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else p[0] = v[0];
}

struct HsCoef {
    float in[HS_MAX_STREAMS];
};

// The norm of the row u_s[0 .. E) (shared memory, complete and visible to the block) into out.
template <typename T>
__device__ __forceinline__ void hs_norm_row(const float* u_s, const float* __restrict__ w, float eps, T* __restrict__ out, int E,
                                            int rms, float* scratch) {
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
        for (int i = threadIdx.x; i < E; i += blockDim.x) s += u_s[i];
        mean = block_sum(s, scratch) / (float)E;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) { const float d = u_s[i] - mean; ss += d * d; }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)E + eps);
    for (int i = threadIdx.x; i < E; i += blockDim.x) out[i] = from_f32<T>((u_s[i] - mean) * rstd * w[i]);
}

template <typename T>
__global__ void __launch_bounds__(HS_MAX_THREADS)
stream_norm_kernel(const float* __restrict__ x, int n, HsCoef c, const float* __restrict__ single, float* __restrict__ copies,
                   const float* __restrict__ w, float eps, const int* __restrict__ rows, T* __restrict__ out, int E, int rms) {
    extern __shared__ float hs_u[];
    __shared__ float scratch[32];
    pdl_wait();
    pdl_trigger();
    const int r = blockIdx.x, t = rows ? rows[r] : r;
    if (single) {
        float total = 0.f;
        for (int s = 0; s < n; ++s) total += c.in[s];
        const float* src = single + (size_t)t * E;
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            const float v = src[i];
            if (copies)
                for (int s = 0; s < n; ++s) copies[((size_t)t * n + s) * E + i] = v;
            hs_u[i] = total * v;
        }
    } else {
        const float* src = x + (size_t)t * n * E;
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            float u = 0.f;
            for (int s = 0; s < n; ++s) u = fmaf(c.in[s], src[(size_t)s * E + i], u);
            hs_u[i] = u;
        }
    }
    __syncthreads();
    hs_norm_row<T>(hs_u, w, eps, out + (size_t)r * E, E, rms, scratch);
}

struct HsMix {
    float mix[HS_MAX_STREAMS * HS_MAX_STREAMS];   // [from * n + to]
    float out[HS_MAX_STREAMS];                     // already times the multiplier of the branch
    float in_next[HS_MAX_STREAMS];
};

template <typename T, int N, int VEC>
__global__ void __launch_bounds__(HS_MAX_THREADS)
stream_update_kernel(float* __restrict__ x, int n_dyn, const __grid_constant__ HsMix m, const float* __restrict__ ls,
                     const T* __restrict__ y, int ldy, const float* __restrict__ w_next, float eps, T* __restrict__ h_out,
                     int E, int rms) {
    extern __shared__ __align__(16) float hs_u[];
    __shared__ float scratch[32];
    constexpr int NMAX = N > 0 ? N : HS_MAX_STREAMS;
    const int n = N > 0 ? N : n_dyn;
    const int t = blockIdx.x;
    float* xr = x + (size_t)t * n * E;
    pdl_wait();
    pdl_trigger();
    const T* yr = y + (size_t)t * ldy;
    for (int i = threadIdx.x * VEC; i < E; i += blockDim.x * VEC) {
        float old[NMAX][VEC], b[VEC], scale[VEC], u[VEC];
#pragma unroll
        for (int s = 0; s < NMAX; ++s)
            if (s < n) hs_load<VEC>(xr + (size_t)s * E + i, old[s]);
        hs_load<VEC>(yr + i, b);
        if (ls) {
            hs_load<VEC>(ls + i, scale);
#pragma unroll
            for (int e = 0; e < VEC; ++e) b[e] *= scale[e];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) u[e] = 0.f;
#pragma unroll
        for (int to = 0; to < NMAX; ++to) {
            if (to >= n) break;
            float v[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                v[e] = m.out[to] * b[e];
#pragma unroll
                for (int s = 0; s < NMAX; ++s)
                    if (s < n) v[e] = fmaf(m.mix[s * n + to], old[s][e], v[e]);
                u[e] = fmaf(m.in_next[to], v[e], u[e]);
            }
            hs_store<VEC>(xr + (size_t)to * E + i, v);
        }
        if (w_next) hs_store<VEC>(hs_u + i, u);
    }
    if (!w_next) return;
    __syncthreads();
    hs_norm_row<T>(hs_u, w_next, eps, h_out + (size_t)t * E, E, rms, scratch);
}

// Threads of a block for rows of E channels taken VEC at a time: one pass over the row where 1,024 threads reach.
static int hs_threads(int E, int vec) {
    const int want = ((E + vec - 1) / vec + 31) / 32 * 32;
    return want < 64 ? 64 : (want > HS_MAX_THREADS ? HS_MAX_THREADS : want);
}

static int hs_fill(float* dst, const float* src, int n) {
    for (int i = 0; i < n; ++i) dst[i] = src ? src[i] : 1.f;
    return 0;
}

// x float32 [tokens, n, E] (or, with `single` float32 [tokens, E], n equal copies of it, written to `copies` if given);
// in_coef: n HOST floats (null: ones); out [rows or tokens, E] in `dtype`; rows: int32 token rows on the device, or null.
extern "C" int vx_stream_norm(const float* x, int n, const float* in_coef, const float* single, float* copies,
                              const float* w, float eps, const int* rows, int n_rows, void* out, int tokens, int E, int rms,
                              int dtype, cudaStream_t stream) {
    const int count = rows ? n_rows : tokens;
    if (count <= 0) return VX_OK;
    if (n <= 0 || n > HS_MAX_STREAMS || E <= 0 || (!x && !single) || !w) return VX_ERR_SHAPE;
    if ((size_t)E * sizeof(float) > 200 * 1024) return VX_ERR_LIMIT;
    HsCoef c;
    hs_fill(c.in, in_coef, n);
    const size_t smem = (size_t)E * sizeof(float);
    static bool configured[2][VX_MAX_DEVICES];
    if (dtype == VX_F32) {
        if (int rc = vx_configure_smem(stream_norm_kernel<float>, 200 * 1024, configured[0])) return rc;
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (stream_norm_kernel<float>), count, hs_threads(E, 1), smem, stream, x, n, c, single, copies, w, eps,
                    rows, (float*)out, E, rms);
    } else if (dtype == VX_BF16) {
        if (int rc = vx_configure_smem(stream_norm_kernel<bf16>, 200 * 1024, configured[1])) return rc;
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (stream_norm_kernel<bf16>), count, hs_threads(E, 1), smem, stream, x, n, c, single, copies, w, eps,
                    rows, (bf16*)out, E, rms);
    } else {
        return VX_ERR_DTYPE;
    }
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// x float32 [tokens, n, E], updated in place; mix: n * n HOST floats [from, to] (null: the identity), out_coef: n HOST
// floats (null: ones), `mult` multiplies the branch; ls: float32 [E] on the device or null; y [tokens, ldy >= E] in `dtype`.
// With w_next (float32 [E] on the device): in_next (n HOST floats, null: ones) and h_out [tokens, E] in `dtype` take the norm
// of the next sublayer's input.
extern "C" int vx_stream_update(float* x, int n, const float* mix, const float* out_coef, float mult, const float* ls,
                                const void* y, int ldy, const float* in_next, const float* w_next, float eps, void* h_out,
                                int tokens, int E, int rms, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (n <= 0 || n > HS_MAX_STREAMS || E <= 0 || ldy < E || !x || !y || (w_next && !h_out)) return VX_ERR_SHAPE;
    if ((size_t)E * sizeof(float) > 200 * 1024) return VX_ERR_LIMIT;
    HsMix m;
    for (int s = 0; s < n; ++s)
        for (int t = 0; t < n; ++t) m.mix[s * n + t] = mix ? mix[s * n + t] : (s == t ? 1.f : 0.f);
    for (int s = 0; s < n; ++s) {
        m.out[s] = (out_coef ? out_coef[s] : 1.f) * mult;
        m.in_next[s] = in_next ? in_next[s] : 1.f;
    }
    const size_t smem = w_next ? (size_t)E * sizeof(float) : 0;
    static bool configured[8][VX_MAX_DEVICES];
#define HS_GO(T, N, VEC, SLOT)                                                                                             \
    do {                                                                                                                   \
        if (int rc = vx_configure_smem(stream_update_kernel<T, N, VEC>, 200 * 1024, configured[SLOT])) return rc;          \
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (stream_update_kernel<T, N, VEC>), tokens, hs_threads(E, VEC), smem, stream, x, n, m, ls, \
                    (const T*)y, ldy, w_next, eps, (T*)h_out, E, rms);                                                      \
    } while (0)
    // four channels a thread where every row starts on a 16-byte border (the general instantiation keeps one: its copies
    // would not fit the registers of 1,024 threads)
    const bool vec = !(E & 3) && !(ldy & 3) && !(((uintptr_t)x | (uintptr_t)ls | (uintptr_t)y) & 15);
    if (dtype == VX_F32) {
        if (n == 1 && vec) HS_GO(float, 1, 4, 0);
        else if (n == 2 && vec) HS_GO(float, 2, 4, 1);
        else if (n == 4 && vec) HS_GO(float, 4, 4, 2);
        else HS_GO(float, 0, 1, 3);
    } else if (dtype == VX_BF16) {
        if (n == 1 && vec) HS_GO(bf16, 1, 4, 4);
        else if (n == 2 && vec) HS_GO(bf16, 2, 4, 5);
        else if (n == 4 && vec) HS_GO(bf16, 4, 4, 6);
        else HS_GO(bf16, 0, 1, 7);
    } else {
        return VX_ERR_DTYPE;
    }
#undef HS_GO
    VX_LAUNCH_CHECK();
    return VX_OK;
}
