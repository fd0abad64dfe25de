// What follows the softmax maps of a differential attention, and a gate that multiplies a row element by element.
//
// diff_combine: a head's two maps a1, a2 (attention outputs over the same values, float32) become
//   o = a1 - lambda a2,   o <- o / sqrt(mean(o^2) + eps) * post,   o <- o * sigmoid(g_h)
// with one lambda for the layer and one gate logit g_h per head, read from column gate_col + h of the token's row of
// `gates` (no gate: gate_col < 0).  The maps lie as 2 H heads of Dv values a token, ordered by key/value group: the group's
// `per` heads of map 1, then its `per` heads of map 2 (the order in which grouped attention kernels want the query heads
// of a key head side by side).  The output is [tokens, H * Dv] in the element type T, heads in their own order.
// A warp per (token, head); all sums float32.
//
// sigmoid_gate: out[r, i] = o[r, i] * sigmoid(g[r, i]), the sigmoid and the product in float32.
#include "common.cuh"

#define DC_WARPS 4

template <typename T, typename TA>
__global__ void diff_combine_kernel(const TA* __restrict__ maps, const T* __restrict__ gates, int ldg, int gate_col,
                                    T* __restrict__ out, float lambda, float post, float eps, int tokens, int H, int per, int Dv) {
    pdl_wait();
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * DC_WARPS + warp;
    if (item >= (long long)tokens * H) return;
    const int t = (int)(item / H), h = (int)(item - (long long)t * H);
    const int g = h / per, i = h - g * per;
    const TA* a1 = maps + ((size_t)t * 2 * H + (size_t)g * 2 * per + i) * Dv;
    const TA* a2 = a1 + (size_t)per * Dv;
    float ss = 0.f;
    for (int d = lane; d < Dv; d += 32) {
        const float o = to_f32(a1[d]) - lambda * to_f32(a2[d]);
        ss += o * o;
    }
    ss = warp_sum(ss);
    float f = rsqrtf(ss / (float)Dv + eps) * post;
    if (gate_col >= 0) f *= 1.f / (1.f + expf(-to_f32(gates[(size_t)t * ldg + gate_col + h])));
    T* dst = out + ((size_t)t * H + h) * Dv;
    for (int d = lane; d < Dv; d += 32) dst[d] = from_f32<T>((to_f32(a1[d]) - lambda * to_f32(a2[d])) * f);
}

// maps [tokens, 2 H, Dv] float32 (`maps_f32`) or in `dtype`; gates [tokens, ldg] in `dtype`; out [tokens, H, Dv] in `dtype`.
extern "C" int vx_diff_combine(const void* maps, int maps_f32, const void* gates, int ldg, int gate_col, void* out, float lambda,
                               float post, float eps, int tokens, int H, int per, int Dv, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (H <= 0 || per <= 0 || H % per || Dv <= 0 || (gate_col >= 0 && (!gates || gate_col + H > ldg))) return VX_ERR_SHAPE;
    const long long items = (long long)tokens * H;
    const unsigned blocks = (unsigned)((items + DC_WARPS - 1) / DC_WARPS);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (diff_combine_kernel<float, float>), blocks, DC_WARPS * 32, 0, stream, (const float*)maps,
                    (const float*)gates, ldg, gate_col, (float*)out, lambda, post, eps, tokens, H, per, Dv);
    else if (dtype == VX_BF16 && maps_f32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (diff_combine_kernel<bf16, float>), blocks, DC_WARPS * 32, 0, stream, (const float*)maps,
                    (const bf16*)gates, ldg, gate_col, (bf16*)out, lambda, post, eps, tokens, H, per, Dv);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (diff_combine_kernel<bf16, bf16>), blocks, DC_WARPS * 32, 0, stream, (const bf16*)maps,
                    (const bf16*)gates, ldg, gate_col, (bf16*)out, lambda, post, eps, tokens, H, per, Dv);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ o, int ldo, const T* __restrict__ g, int ldg, T* __restrict__ out,
                                    int ldout, long long total, int cols) {
    pdl_wait();
    pdl_trigger();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / cols;
        const int c = (int)(idx - r * cols);
        const float z = to_f32(g[r * ldg + c]);
        out[r * ldout + c] = from_f32<T>(to_f32(o[r * ldo + c]) / (1.f + expf(-z)));
    }
}

// bfloat16 rows whose pointers and strides lie on 16-byte borders: eight elements a thread.
__global__ void sigmoid_gate8_kernel(const bf16* __restrict__ o, int ldo, const bf16* __restrict__ g, int ldg, bf16* __restrict__ out,
                                     int ldout, long long total8, int cols8) {
    pdl_wait();
    pdl_trigger();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / cols8;
        const int c = (int)(idx - r * cols8) * 8;
        const uint4 a = *reinterpret_cast<const uint4*>(o + r * ldo + c), b = *reinterpret_cast<const uint4*>(g + r * ldg + c);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
        uint4 res;
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 x = __bfloat1622float2(a2[e]), z = __bfloat1622float2(b2[e]);
            r2[e] = __floats2bfloat162_rn(x.x / (1.f + expf(-z.x)), x.y / (1.f + expf(-z.y)));
        }
        *reinterpret_cast<uint4*>(out + r * ldout + c) = res;
    }
}

extern "C" int vx_sigmoid_gate(const void* o, int ldo, const void* g, int ldg, void* out, int ldout, int rows, int cols,
                               int dtype, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return VX_OK;
    if (ldo < cols || ldg < cols || ldout < cols) return VX_ERR_SHAPE;
    const long long total = (long long)rows * cols;
    const unsigned blocks = (unsigned)((total + 255) / 256 > 148LL * 16 ? 148LL * 16 : (total + 255) / 256);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (sigmoid_gate_kernel<float>), blocks, 256, 0, stream, (const float*)o, ldo, (const float*)g, ldg,
                    (float*)out, ldout, total, cols);
    else if (dtype == VX_BF16 && !((cols | ldo | ldg | ldout) & 7) && !(((uintptr_t)o | (uintptr_t)g | (uintptr_t)out) & 15)) {
        const long long total8 = total / 8;
        const unsigned blocks8 = (unsigned)((total8 + 255) / 256 > 148LL * 16 ? 148LL * 16 : (total8 + 255) / 256);
        VX_LAUNCH_K(VX_K_ELEMENTWISE, sigmoid_gate8_kernel, blocks8, 256, 0, stream, (const bf16*)o, ldo, (const bf16*)g, ldg,
                    (bf16*)out, ldout, total8, cols / 8);
    } else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (sigmoid_gate_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)o, ldo, (const bf16*)g, ldg,
                    (bf16*)out, ldout, total, cols);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}
