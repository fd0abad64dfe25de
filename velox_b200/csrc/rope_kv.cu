// Per-head RMSNorm of queries and keys, rotary position encoding, and the write
// of the new keys and values into the paged cache, in one pass over the packed
// projection output.
//
// qkv is [tokens, row_stride] with, in each row, H query heads, then Hk key
// heads, each of D elements, then Hk value heads of Dv elements (Dv = D unless the
// caller says otherwise; a row may go on with columns that are not touched here).
// One warp handles one head of one token:
//   q, k:  x = x * rsqrt(mean(x^2) + eps) * w[d]          (if a weight is given)
//          pairs (i, i + rot/2), i < rot/2, rotated by angle = pos * inv_freq[i]
//          (half-split convention; with `interleaved` the pairs are (2i, 2i + 1) instead;
//          angle, sine and cosine in float32, computed here rather than read from a
//          table rounded to the element type)
//   q is written back in place; k goes to k_pool, v (untouched) to v_pool at
//   slot_mapping[token] = page * S + offset, pools laid out [page, Hk, S, D] and [page, Hk, S, Dv].
// A token whose slot is negative writes nothing.  Without a slot mapping (a layer
// that reads another layer's cache, or a caller that encodes positions itself)
// nothing is written to the pools and the keys are normed and rotated in place.
#include "common.cuh"

#define ROPE_WARPS 4
#define ROPE_MAX_D 512

template <typename T>
__global__ void qk_norm_rope_kv_kernel(T* __restrict__ qkv, int row_stride,
                                       const float* __restrict__ q_weight,
                                       const float* __restrict__ k_weight, float eps,
                                       const float* __restrict__ inv_freq, int rot_dim,
                                       const int* __restrict__ positions,
                                       const int* __restrict__ slot_mapping, T* __restrict__ k_pool,
                                       T* __restrict__ v_pool, int H, int Hk, int D, int S, int Dv, int interleaved,
                                       int Hv, float magnitude) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * ROPE_WARPS + warp;
    if (head >= H + Hk + Hv) return;
    float* buf = smem + warp * D;
    T* src = qkv + (size_t)t * row_stride + (size_t)head * D;
    const int slot = slot_mapping ? slot_mapping[t] : -1;

    if (head >= H + Hk) {  // value head: copy into the cache
        if (slot < 0) return;
        const int hk = head - H - Hk;
        const T* vsrc = qkv + (size_t)t * row_stride + (size_t)(H + Hk) * D + (size_t)hk * Dv;
        T* dst = v_pool + (((size_t)(slot / S) * Hv + hk) * S + (slot % S)) * Dv;
        for (int d = lane; d < Dv; d += 32) dst[d] = vsrc[d];
        return;
    }
    const bool is_q = head < H;
    if (!is_q && slot_mapping && slot < 0) return;
    const float* w = is_q ? q_weight : k_weight;

    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
        const float x = to_f32(src[d]);
        buf[d] = x;
        ss += x * x;
    }
    if (w) {
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / (float)D + eps);
        for (int d = lane; d < D; d += 32) buf[d] = buf[d] * rstd * w[d];
    }
    __syncwarp();
    if (inv_freq && rot_dim > 0) {
        const int half = rot_dim >> 1;
        const float pos = (float)positions[t];
        for (int i = lane; i < half; i += 32) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            sn *= magnitude;
            cs *= magnitude;
            const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
            const float a = buf[ia], b = buf[ib];
            buf[ia] = a * cs - b * sn;
            buf[ib] = a * sn + b * cs;
        }
        __syncwarp();
    }
    if (is_q || !slot_mapping) {  // without a slot mapping keys are treated in place too
        for (int d = lane; d < D; d += 32) src[d] = from_f32<T>(buf[d]);
    } else {
        const int hk = head - H;
        T* dst = k_pool + (((size_t)(slot / S) * Hk + hk) * S + (slot % S)) * D;
        for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(buf[d]);
    }
}

// The same for many tokens (a prompt portion) at any head size: one block per token works through all heads of its row,
// eight warps taking the heads in turn, with the token's cosines and sines (times `magnitude`) computed once into shared
// memory instead of once per head.  The arithmetic of a head is the kernel's above.
#define ROPE_ROW_WARPS 8
#define ROPE_ROW_MIN_TOKENS 64   // tokens from which this variant is used
template <typename T>
__global__ void __launch_bounds__(ROPE_ROW_WARPS * 32)
qk_norm_rope_kv_row_kernel(T* __restrict__ qkv, int row_stride, const float* __restrict__ q_weight,
                           const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq, int rot_dim,
                           const int* __restrict__ positions, const int* __restrict__ slot_mapping, T* __restrict__ k_pool,
                           T* __restrict__ v_pool, int H, int Hk, int D, int S, int Dv, int interleaved, int Hv, float magnitude) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float smem[];
    const int half = (inv_freq && rot_dim > 0) ? rot_dim >> 1 : 0;
    float* cs_s = smem;                 // [half] cosines, then [half] sines
    float* bufs = smem + 2 * half;      // [warps][D]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        cs_s[i] = cs * magnitude;
        cs_s[half + i] = sn * magnitude;
    }
    __syncthreads();
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    float* buf = bufs + warp * D;
    for (int head = warp; head < H + Hk + Hv; head += ROPE_ROW_WARPS) {
        if (head >= H + Hk) {  // value head: copy into the cache
            if (slot < 0) continue;
            const int hk = head - H - Hk;
            const T* vsrc = qkv + (size_t)t * row_stride + (size_t)(H + Hk) * D + (size_t)hk * Dv;
            T* dst = v_pool + (((size_t)(slot / S) * Hv + hk) * S + (slot % S)) * Dv;
            for (int d = lane; d < Dv; d += 32) dst[d] = vsrc[d];
            continue;
        }
        const bool is_q = head < H;
        if (!is_q && slot_mapping && slot < 0) continue;
        const float* w = is_q ? q_weight : k_weight;
        T* src = qkv + (size_t)t * row_stride + (size_t)head * D;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float x = to_f32(src[d]);
            buf[d] = x;
            ss += x * x;
        }
        if (w) {
            ss = warp_sum(ss);
            const float rstd = rsqrtf(ss / (float)D + eps);
            for (int d = lane; d < D; d += 32) buf[d] = buf[d] * rstd * w[d];
        }
        __syncwarp();
        for (int i = lane; i < half; i += 32) {
            const float cs = cs_s[i], sn = cs_s[half + i];
            const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
            const float a = buf[ia], b = buf[ib];
            buf[ia] = a * cs - b * sn;
            buf[ib] = a * sn + b * cs;
        }
        __syncwarp();
        T* dst = src;
        if (!is_q && slot_mapping) dst = k_pool + (((size_t)(slot / S) * Hk + (head - H)) * S + (slot % S)) * D;
        for (int d = lane; d < D; d += 32) dst[d] = from_f32<T>(buf[d]);
        __syncwarp();
    }
}

// The same again for bfloat16 heads of an even size up to 64 PAIRS elements: the head stays in registers, a lane holding the
// element pairs (2 l, 2 l + 1) + 64 j; only the normed channels that are turned pass through shared memory, once, so that a
// lane can read its channels' partners (i +- rot/2, or its own pair when neighbours are paired).
template <int PAIRS>
__global__ void __launch_bounds__(ROPE_ROW_WARPS * 32)
qk_norm_rope_kv_row_pairs_kernel(bf16* __restrict__ qkv, int row_stride, const float* __restrict__ q_weight,
                                 const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq, int rot_dim,
                                 const int* __restrict__ positions, const int* __restrict__ slot_mapping, bf16* __restrict__ k_pool,
                                 bf16* __restrict__ v_pool, int H, int Hk, int D, int S, int Dv, int interleaved, int Hv, float magnitude) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float smem[];
    const int half = (inv_freq && rot_dim > 0) ? rot_dim >> 1 : 0;
    const int rot = 2 * half;
    float* cs_s = smem;                 // [half] cosines, then [half] sines
    float* bufs = smem + 2 * half;      // [warps][rot]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        cs_s[i] = cs * magnitude;
        cs_s[half + i] = sn * magnitude;
    }
    __syncthreads();
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    float* buf = bufs + warp * rot;
    for (int head = warp; head < H + Hk + Hv; head += ROPE_ROW_WARPS) {
        if (head >= H + Hk) {  // value head: copy into the cache
            if (slot < 0) continue;
            const int hk = head - H - Hk;
            const bf16* vsrc = qkv + (size_t)t * row_stride + (size_t)(H + Hk) * D + (size_t)hk * Dv;
            bf16* dst = v_pool + (((size_t)(slot / S) * Hv + hk) * S + (slot % S)) * Dv;
            if (!(Dv & 1) && !((((uintptr_t)vsrc) | ((uintptr_t)dst)) & 3)) {
                for (int d = 2 * lane; d < Dv; d += 64)
                    *reinterpret_cast<unsigned*>(dst + d) = *reinterpret_cast<const unsigned*>(vsrc + d);
            } else {
                for (int d = lane; d < Dv; d += 32) dst[d] = vsrc[d];
            }
            continue;
        }
        const bool is_q = head < H;
        if (!is_q && slot_mapping && slot < 0) continue;
        const float* w = is_q ? q_weight : k_weight;
        bf16* src = qkv + (size_t)t * row_stride + (size_t)head * D;
        float2 x[PAIRS];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) {
            const int d = 2 * lane + 64 * j;
            x[j] = d < D ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + d)) : make_float2(0.f, 0.f);
            ss += x[j].x * x[j].x + x[j].y * x[j].y;
        }
        if (w) {
            ss = warp_sum(ss);
            const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const int d = 2 * lane + 64 * j;
                if (d < D) { x[j].x = x[j].x * rstd * w[d]; x[j].y = x[j].y * rstd * w[d + 1]; }
            }
        }
        if (half) {
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const int d = 2 * lane + 64 * j;
                if (d < rot) *reinterpret_cast<float2*>(buf + d) = x[j];
            }
            __syncwarp();
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const int d = 2 * lane + 64 * j;
                if (d >= rot) continue;
                if (interleaved) {   // the pair (d, d + 1) is pair d / 2 of the rotation
                    const float cs = cs_s[d >> 1], sn = cs_s[half + (d >> 1)];
                    const float a = x[j].x, b = x[j].y;
                    x[j] = make_float2(a * cs - b * sn, a * sn + b * cs);
                } else if (d < half) {   // (half is even or odd: the two channels are looked at one by one)
                    const float a0 = x[j].x, b0 = buf[d + half];
                    x[j].x = a0 * cs_s[d] - b0 * cs_s[half + d];
                    if (d + 1 < half) x[j].y = x[j].y * cs_s[d + 1] - buf[d + 1 + half] * cs_s[half + d + 1];
                    else x[j].y = buf[d + 1 - half] * cs_s[half + d + 1 - half] + x[j].y * cs_s[d + 1 - half];
                } else {
                    x[j].x = buf[d - half] * cs_s[half + d - half] + x[j].x * cs_s[d - half];
                    x[j].y = buf[d + 1 - half] * cs_s[half + d + 1 - half] + x[j].y * cs_s[d + 1 - half];
                }
            }
            __syncwarp();   // (the warp's next head writes the same buffer)
        }
        bf16* dst = src;
        if (!is_q && slot_mapping) dst = k_pool + (((size_t)(slot / S) * Hk + (head - H)) * S + (slot % S)) * D;
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) {
            const int d = 2 * lane + 64 * j;
            if (d < D) *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(x[j].x, x[j].y);
        }
    }
}

// And for bfloat16 heads of up to 64 channels (a multiple of 4): TWO heads a warp, sixteen lanes each, a lane holding four
// consecutive channels (one 8-byte load and store).  A head of 64 channels is one 128-byte line, and a warp that works on
// one such head at a time spends most of its time on what a head costs whatever its size (the norm's sum over the lanes,
// the exchange of the turned channels, the slot's address).  Value heads are copied by whole warps afterwards.
__global__ void __launch_bounds__(ROPE_ROW_WARPS * 32)
qk_norm_rope_kv_row_half_kernel(bf16* __restrict__ qkv, int row_stride, const float* __restrict__ q_weight,
                                const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq, int rot_dim,
                                const int* __restrict__ positions, const int* __restrict__ slot_mapping, bf16* __restrict__ k_pool,
                                bf16* __restrict__ v_pool, int H, int Hk, int D, int S, int Dv, int interleaved, int Hv, float magnitude) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ float smem[];
    const int half = (inv_freq && rot_dim > 0) ? rot_dim >> 1 : 0;
    const int rot = 2 * half;
    float* cs_s = smem;                 // [half] cosines, then [half] sines
    float* bufs = smem + 2 * half;      // [warps][2 heads][rot]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int l16 = lane & 15, sub = lane >> 4;
    const int t = blockIdx.x;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        cs_s[i] = cs * magnitude;
        cs_s[half + i] = sn * magnitude;
    }
    __syncthreads();
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    float* buf = bufs + (warp * 2 + sub) * rot;
    const int d = 4 * l16;
    for (int base = warp * 2; base < H + Hk; base += 2 * ROPE_ROW_WARPS) {
        const int head = base + sub;
        const bool is_q = head < H;
        const bool live = head < H + Hk && d < D && (is_q || !slot_mapping || slot >= 0);
        const float* w = is_q ? q_weight : k_weight;
        bf16* src = qkv + (size_t)t * row_stride + (size_t)head * D;
        float x[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
            const uint2 raw = *reinterpret_cast<const uint2*>(src + d);
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
        }
        if (q_weight || k_weight) {   // (the same for both halves of the warp: all lanes take part in the exchanges)
            float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // (stays within the head's sixteen lanes)
            const float rstd = rsqrtf(ss / (float)D + eps);
            if (live && w) {
                const float4 w4 = *reinterpret_cast<const float4*>(w + d);
                x[0] = x[0] * rstd * w4.x; x[1] = x[1] * rstd * w4.y; x[2] = x[2] * rstd * w4.z; x[3] = x[3] * rstd * w4.w;
            }
        }
        if (half) {
            if (live && d < rot) *reinterpret_cast<float4*>(buf + d) = make_float4(x[0], x[1], x[2], x[3]);   // (rot is a multiple of 4)
            __syncwarp();
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = d + e;
                if (!live || i >= rot) continue;
                if (interleaved) {
                    const float cs = cs_s[i >> 1], sn = cs_s[half + (i >> 1)], other = buf[i ^ 1];
                    x[e] = (i & 1) ? other * sn + x[e] * cs : x[e] * cs - other * sn;
                } else if (i < half) {
                    x[e] = x[e] * cs_s[i] - buf[i + half] * cs_s[half + i];
                } else {
                    x[e] = buf[i - half] * cs_s[half + i - half] + x[e] * cs_s[i - half];
                }
            }
            __syncwarp();   // (the warp's next heads write the same buffers)
        }
        if (live) {
            bf16* dst = src;
            if (!is_q && slot_mapping) dst = k_pool + (((size_t)(slot / S) * Hk + (head - H)) * S + (slot % S)) * D;
            uint2 out;
            *reinterpret_cast<__nv_bfloat162*>(&out.x) = __floats2bfloat162_rn(x[0], x[1]);
            *reinterpret_cast<__nv_bfloat162*>(&out.y) = __floats2bfloat162_rn(x[2], x[3]);
            *reinterpret_cast<uint2*>(dst + d) = out;
        }
    }
    if (slot < 0) return;
    for (int hk = warp; hk < Hv; hk += ROPE_ROW_WARPS) {
        const bf16* vsrc = qkv + (size_t)t * row_stride + (size_t)(H + Hk) * D + (size_t)hk * Dv;
        bf16* dst = v_pool + (((size_t)(slot / S) * Hv + hk) * S + (slot % S)) * Dv;
        if (!(Dv & 3) && !((((uintptr_t)vsrc) | ((uintptr_t)dst)) & 7)) {
            for (int c = 4 * lane; c < Dv; c += 128) *reinterpret_cast<uint2*>(dst + c) = *reinterpret_cast<const uint2*>(vsrc + c);
        } else {
            for (int c = lane; c < Dv; c += 32) dst[c] = vsrc[c];
        }
    }
}

// The arithmetic of a head of 128 written out with explicit roundings, so that the
// two kernels below give the same bits whatever the compiler would like to fuse.
__device__ __forceinline__ float head128_squares(float2 lo, float2 hi) {
    return __fmaf_rn(hi.y, hi.y, __fmaf_rn(hi.x, hi.x, __fmaf_rn(lo.y, lo.y, __fmul_rn(lo.x, lo.x))));
}
__device__ __forceinline__ void rotate_pair(float a, float b, float cs, float sn, float& ra, float& rb) {
    ra = __fmaf_rn(a, cs, -__fmul_rn(b, sn));
    rb = __fmaf_rn(a, sn, __fmul_rn(b, cs));
}

// The same for bfloat16 heads of 128 with full rotation, the whole head in
// registers: lane l holds elements 2l, 2l+1 (first half) and 64+2l, 64+2l+1 (their
// partners), loaded and stored as pairs.  Eight warps, one head each.
#define ROPE128_WARPS 8
__global__ void __launch_bounds__(ROPE128_WARPS * 32)
qk_norm_rope_kv_128_kernel(bf16* __restrict__ qkv, int row_stride, const float* __restrict__ q_weight,
                           const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
                           const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                           bf16* __restrict__ k_pool, bf16* __restrict__ v_pool, int H, int Hk, int S) {
    constexpr int D = 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int head = blockIdx.y * ROPE128_WARPS + warp;
    // What depends on no earlier kernel is fetched before the wait: the norm's weights, the
    // frequencies, and the step's description (copied to the device before the step's first kernel).
    const bool in_range = head < H + 2 * Hk;
    const bool is_q = head < H;
    const float* w = is_q ? q_weight : k_weight;
    float2 wl = make_float2(1.f, 1.f), wh = wl, f = make_float2(0.f, 0.f);
    float pos = 0.f;
    int slot = -1;
    if (in_range) {
        slot = slot_mapping ? slot_mapping[t] : -1;
        if (head < H + Hk) {
            if (w) { wl = reinterpret_cast<const float2*>(w)[lane]; wh = reinterpret_cast<const float2*>(w + 64)[lane]; }
            if (inv_freq) { f = reinterpret_cast<const float2*>(inv_freq)[lane]; pos = (float)positions[t]; }
        }
    }
    pdl_wait();
    pdl_trigger();
    if (!in_range) return;
    bf16* src = qkv + (size_t)t * row_stride + (size_t)head * D;
    if (head >= H + Hk) {  // value head: copy into the cache (8 bytes per lane)
        if (slot < 0) return;
        const int hk = head - H - Hk;
        bf16* dst = v_pool + (((size_t)(slot / S) * Hk + hk) * S + (slot % S)) * D;
        reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(src)[lane];
        return;
    }
    if (!is_q && slot_mapping && slot < 0) return;
    float2 lo = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src)[lane]);
    float2 hi = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src + 64)[lane]);
    if (w) {
        const float ss = warp_sum(head128_squares(lo, hi));
        const float rstd = rsqrtf(ss / (float)D + eps);
        lo.x = __fmul_rn(__fmul_rn(lo.x, rstd), wl.x); lo.y = __fmul_rn(__fmul_rn(lo.y, rstd), wl.y);
        hi.x = __fmul_rn(__fmul_rn(hi.x, rstd), wh.x); hi.y = __fmul_rn(__fmul_rn(hi.y, rstd), wh.y);
    }
    if (inv_freq) {
        float sn, cs, a0, b0, a1, b1;
        sincosf(__fmul_rn(pos, f.x), &sn, &cs);
        rotate_pair(lo.x, hi.x, cs, sn, a0, b0);
        sincosf(__fmul_rn(pos, f.y), &sn, &cs);
        rotate_pair(lo.y, hi.y, cs, sn, a1, b1);
        lo = make_float2(a0, a1);
        hi = make_float2(b0, b1);
    }
    bf16* dst = src;
    if (!is_q && slot_mapping)
        dst = k_pool + (((size_t)(slot / S) * Hk + (head - H)) * S + (slot % S)) * D;
    reinterpret_cast<__nv_bfloat162*>(dst)[lane] = __floats2bfloat162_rn(lo.x, lo.y);
    reinterpret_cast<__nv_bfloat162*>(dst + 64)[lane] = __floats2bfloat162_rn(hi.x, hi.y);
}

// The same for many tokens (a prompt portion): one block per token works through
// all heads of its row, eight warps taking the heads in turn, with the token's 64
// cosines and sines computed once into shared memory instead of once per head
// (40 or more heads share them; the sincosf calls were most of the kernel's time).
#define ROPE128_TOKEN_MIN 64   // tokens from which this variant is used
__global__ void __launch_bounds__(ROPE128_WARPS * 32)
qk_norm_rope_kv_128_row_kernel(bf16* __restrict__ qkv, int row_stride, const float* __restrict__ q_weight,
                               const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
                               const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                               bf16* __restrict__ k_pool, bf16* __restrict__ v_pool, int H, int Hk, int S) {
    pdl_wait();
    pdl_trigger();
    constexpr int D = 128;
    __shared__ float2 cs_sn[D / 2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    if (inv_freq && threadIdx.x < D / 2) {
        float sn, cs;
        sincosf(__fmul_rn((float)positions[t], inv_freq[threadIdx.x]), &sn, &cs);
        cs_sn[threadIdx.x] = make_float2(cs, sn);
    }
    __syncthreads();
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    for (int head = warp; head < H + 2 * Hk; head += ROPE128_WARPS) {
        bf16* src = qkv + (size_t)t * row_stride + (size_t)head * D;
        if (head >= H + Hk) {  // value head: copy into the cache (8 bytes per lane)
            if (slot < 0) continue;
            const int hk = head - H - Hk;
            bf16* dst = v_pool + (((size_t)(slot / S) * Hk + hk) * S + (slot % S)) * D;
            reinterpret_cast<uint2*>(dst)[lane] = reinterpret_cast<const uint2*>(src)[lane];
            continue;
        }
        const bool is_q = head < H;
        if (!is_q && slot_mapping && slot < 0) continue;
        const float* w = is_q ? q_weight : k_weight;
        float2 lo = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src)[lane]);
        float2 hi = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(src + 64)[lane]);
        if (w) {
            const float ss = warp_sum(head128_squares(lo, hi));
            const float rstd = rsqrtf(ss / (float)D + eps);
            const float2 wl = reinterpret_cast<const float2*>(w)[lane], wh = reinterpret_cast<const float2*>(w + 64)[lane];
            lo.x = __fmul_rn(__fmul_rn(lo.x, rstd), wl.x); lo.y = __fmul_rn(__fmul_rn(lo.y, rstd), wl.y);
            hi.x = __fmul_rn(__fmul_rn(hi.x, rstd), wh.x); hi.y = __fmul_rn(__fmul_rn(hi.y, rstd), wh.y);
        }
        if (inv_freq) {
            const float2 c0 = cs_sn[2 * lane], c1 = cs_sn[2 * lane + 1];
            float a0, b0, a1, b1;
            rotate_pair(lo.x, hi.x, c0.x, c0.y, a0, b0);
            rotate_pair(lo.y, hi.y, c1.x, c1.y, a1, b1);
            lo = make_float2(a0, a1);
            hi = make_float2(b0, b1);
        }
        bf16* dst = src;
        if (!is_q && slot_mapping)
            dst = k_pool + (((size_t)(slot / S) * Hk + (head - H)) * S + (slot % S)) * D;
        reinterpret_cast<__nv_bfloat162*>(dst)[lane] = __floats2bfloat162_rn(lo.x, lo.y);
        reinterpret_cast<__nv_bfloat162*>(dst + 64)[lane] = __floats2bfloat162_rn(hi.x, hi.y);
    }
}

// `Hv` value heads follow the key heads in a row (0: as many as key heads; fewer where several key heads share a
// value head: the value pool is then [page, Hv, S, Dv]); cosines and sines are multiplied by `magnitude` (a rotation
// whose frequencies were stretched may lengthen the rotated channels by a fixed factor).
extern "C" int vx_qk_norm_rope_kv_shared(void* qkv, int row_stride, const float* q_weight,
                                         const float* k_weight, float eps, const float* inv_freq,
                                         int rot_dim, const int* positions, const int* slot_mapping,
                                         void* k_pool, void* v_pool, int tokens, int H, int Hk, int D, int S,
                                         int dtype, int Dv, int interleaved, int Hv, float magnitude, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (Dv <= 0) Dv = D;
    if (Hv <= 0) Hv = Hk;
    if (H <= 0 || Hk <= 0 || D <= 0 || S <= 0 || D > ROPE_MAX_D || Dv > ROPE_MAX_D) return VX_ERR_SHAPE;
    if (rot_dim < 0 || rot_dim > D || (rot_dim & 1)) return VX_ERR_SHAPE;
    if (row_stride < (H + Hk) * D + Hv * Dv) return VX_ERR_SHAPE;
    if (slot_mapping && (!k_pool || !v_pool)) return VX_ERR_SHAPE;
    if (!inv_freq || rot_dim == 0) interleaved = 0;
    if (Hv == Hk && magnitude == 1.f && !interleaved && dtype == VX_BF16 && D == 128 && Dv == D && (rot_dim == D || !inv_freq) && !(row_stride & 3) &&
        !((((uintptr_t)qkv) | ((uintptr_t)k_pool) | ((uintptr_t)v_pool)) & 7)) {
        if (tokens >= ROPE128_TOKEN_MIN) {
            VX_LAUNCH_K(VX_K_ROPE, qk_norm_rope_kv_128_row_kernel, tokens, ROPE128_WARPS * 32, 0, stream, (bf16*)qkv,
                        row_stride, q_weight, k_weight, eps, (rot_dim == D) ? inv_freq : (const float*)nullptr,
                        positions, slot_mapping, (bf16*)k_pool, (bf16*)v_pool, H, Hk, S);
            VX_LAUNCH_CHECK();
            return VX_OK;
        }
        dim3 grid128(tokens, (H + 2 * Hk + ROPE128_WARPS - 1) / ROPE128_WARPS);
        VX_LAUNCH_K(VX_K_ROPE, qk_norm_rope_kv_128_kernel, grid128, ROPE128_WARPS * 32, 0, stream, (bf16*)qkv,
                    row_stride, q_weight, k_weight, eps, (rot_dim == D) ? inv_freq : (const float*)nullptr, positions,
                    slot_mapping, (bf16*)k_pool, (bf16*)v_pool, H, Hk, S);
        VX_LAUNCH_CHECK();
        return VX_OK;
    }
    if (tokens >= ROPE_ROW_MIN_TOKENS && dtype == VX_BF16 && !(D & 3) && D <= 64 && !(row_stride & 3) && !(rot_dim & 3) &&
        !((((uintptr_t)qkv) | ((uintptr_t)k_pool)) & 7) && !((((uintptr_t)q_weight) | ((uintptr_t)k_weight)) & 15)) {
        // (the buffers' rows lie on 16-byte borders: rot_dim is a multiple of 4)
        const size_t half_smem = ((size_t)rot_dim + (size_t)ROPE_ROW_WARPS * 2 * rot_dim) * sizeof(float);
        VX_LAUNCH_K(VX_K_ROPE, qk_norm_rope_kv_row_half_kernel, tokens, ROPE_ROW_WARPS * 32, half_smem, stream, (bf16*)qkv, row_stride,
                    q_weight, k_weight, eps, inv_freq, rot_dim, positions, slot_mapping, (bf16*)k_pool, (bf16*)v_pool, H, Hk, D, S, Dv,
                    interleaved, Hv, magnitude);
        VX_LAUNCH_CHECK();
        return VX_OK;
    }
    if (tokens >= ROPE_ROW_MIN_TOKENS && dtype == VX_BF16 && !(D & 1) && D <= 256 && !(row_stride & 1) &&
        !((((uintptr_t)qkv) | ((uintptr_t)k_pool)) & 3)) {
        const size_t pairs_smem = ((size_t)rot_dim + (size_t)ROPE_ROW_WARPS * rot_dim) * sizeof(float);
#define ROPE_PAIRS_GO(P_)                                                                                                   \
    VX_LAUNCH_K(VX_K_ROPE, (qk_norm_rope_kv_row_pairs_kernel<P_>), tokens, ROPE_ROW_WARPS * 32, pairs_smem, stream, (bf16*)qkv, \
                row_stride, q_weight, k_weight, eps, inv_freq, rot_dim, positions, slot_mapping, (bf16*)k_pool, (bf16*)v_pool, H, \
                Hk, D, S, Dv, interleaved, Hv, magnitude)
        if (D <= 64) ROPE_PAIRS_GO(1);
        else if (D <= 128) ROPE_PAIRS_GO(2);
        else ROPE_PAIRS_GO(4);
#undef ROPE_PAIRS_GO
        VX_LAUNCH_CHECK();
        return VX_OK;
    }
    if (tokens >= ROPE_ROW_MIN_TOKENS) {
        const size_t row_smem = ((size_t)rot_dim + (size_t)ROPE_ROW_WARPS * D) * sizeof(float);   // (at most 18 KB)
        if (dtype == VX_F32)
            VX_LAUNCH_K(VX_K_ROPE, (qk_norm_rope_kv_row_kernel<float>), tokens, ROPE_ROW_WARPS * 32, row_smem, stream, (float*)qkv, row_stride, q_weight, k_weight, eps, inv_freq, rot_dim, positions, slot_mapping,
                (float*)k_pool, (float*)v_pool, H, Hk, D, S, Dv, interleaved, Hv, magnitude);
        else if (dtype == VX_BF16)
            VX_LAUNCH_K(VX_K_ROPE, (qk_norm_rope_kv_row_kernel<bf16>), tokens, ROPE_ROW_WARPS * 32, row_smem, stream, (bf16*)qkv, row_stride, q_weight, k_weight, eps, inv_freq, rot_dim, positions, slot_mapping,
                (bf16*)k_pool, (bf16*)v_pool, H, Hk, D, S, Dv, interleaved, Hv, magnitude);
        else
            return VX_ERR_DTYPE;
        VX_LAUNCH_CHECK();
        return VX_OK;
    }
    dim3 grid(tokens, (H + Hk + Hv + ROPE_WARPS - 1) / ROPE_WARPS);
    const size_t smem = (size_t)ROPE_WARPS * D * sizeof(float);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ROPE, (qk_norm_rope_kv_kernel<float>), grid, ROPE_WARPS * 32, smem, stream, (float*)qkv, row_stride, q_weight, k_weight, eps, inv_freq, rot_dim, positions, slot_mapping,
            (float*)k_pool, (float*)v_pool, H, Hk, D, S, Dv, interleaved, Hv, magnitude);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ROPE, (qk_norm_rope_kv_kernel<bf16>), grid, ROPE_WARPS * 32, smem, stream, (bf16*)qkv, row_stride, q_weight, k_weight, eps, inv_freq, rot_dim, positions, slot_mapping,
            (bf16*)k_pool, (bf16*)v_pool, H, Hk, D, S, Dv, interleaved, Hv, magnitude);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

extern "C" int vx_qk_norm_rope_kv_pairs(void* qkv, int row_stride, const float* q_weight,
                                        const float* k_weight, float eps, const float* inv_freq,
                                        int rot_dim, const int* positions, const int* slot_mapping,
                                        void* k_pool, void* v_pool, int tokens, int H, int Hk, int D, int S,
                                        int dtype, int Dv, int interleaved, cudaStream_t stream) {
    return vx_qk_norm_rope_kv_shared(qkv, row_stride, q_weight, k_weight, eps, inv_freq, rot_dim, positions, slot_mapping,
                                     k_pool, v_pool, tokens, H, Hk, D, S, dtype, Dv, interleaved, 0, 1.f, stream);
}

// The half-split rotation under its first name.
extern "C" int vx_qk_norm_rope_kv(void* qkv, int row_stride, const float* q_weight,
                                  const float* k_weight, float eps, const float* inv_freq,
                                  int rot_dim, const int* positions, const int* slot_mapping,
                                  void* k_pool, void* v_pool, int tokens, int H, int Hk, int D, int S,
                                  int dtype, int Dv, cudaStream_t stream) {
    return vx_qk_norm_rope_kv_pairs(qkv, row_stride, q_weight, k_weight, eps, inv_freq, rot_dim, positions, slot_mapping,
                                    k_pool, v_pool, tokens, H, Hk, D, S, dtype, Dv, 0, stream);
}
