// Attention over cached latent rows: every position keeps ONE row of W = C + R elements (C latent channels, then R
// rotated channels that all heads share), and a query head brings a folded query of the same width, so that
//   score(i, j) = qa_i . row_j * scale,   causal softmax,   out_i = sum_j w_ij row_j[0 .. C)
// (the value is the first C elements of the key's row).  All heads of a token read the same rows, so a block stages
// a tile of rows once for up to sixteen heads.
//
// One block per (token row, group of 16 heads, run of keys); a warp per 4 heads.  A tile of 32 rows is copied into shared
// memory as float32, each row on a stride of 4 (mod 32) elements, so that lane j reads row j sixteen bytes at a time without
// bank conflicts; the folded queries lie beside the tile and are read as broadcasts.  A lane forms the products of row j with
// its warp's 4 queries (every element of the row read once for the four), the warp keeps a running maximum, sum and
// accumulator per head (lane l owns value channels 4 (l + 32 i) .. + 3) and adds the 32 rows in key order, every element of a
// row again read once for the four heads.  With `runs` > 1 a token's tiles are dealt to the runs in contiguous stretches,
// every run writes (maximum, sum, accumulator) to a scratch buffer, and a join kernel adds them in run order.  Scores,
// weights and sums are float32; the order of every sum depends on the token's own position and on `runs` alone.
#include "common.cuh"

#define AL_WARPS 4
#define AL_HW 4                       // heads of a warp
#define AL_HEADS (AL_WARPS * AL_HW)   // heads of a block
#define AL_TILE 32

__host__ __device__ inline int al_row_stride(int W) {   // the least number >= W that is 4 mod 32
    const int w4 = (W + 3) & ~3;
    return w4 + ((4 - w4) & 31);
}

template <typename T>
__device__ __forceinline__ void al_stage_row(float* dst, const T* src, int W, int Wp, int lane) {
    for (int d = lane; d < Wp; d += 32) dst[d] = d < W ? to_f32(src[d]) : 0.f;
}
template <>
__device__ __forceinline__ void al_stage_row<bf16>(float* dst, const bf16* src, int W, int Wp, int lane) {
    if ((W & 7) == 0 && (((uintptr_t)src) & 15) == 0) {   // eight elements a load
        for (int d = lane * 8; d < W; d += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(src + d);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
            const float2 c = __bfloat1622float2(h2[2]), e = __bfloat1622float2(h2[3]);
            *reinterpret_cast<float4*>(dst + d) = make_float4(a.x, a.y, b.x, b.y);
            *reinterpret_cast<float4*>(dst + d + 4) = make_float4(c.x, c.y, e.x, e.y);
        }
        return;
    }
    for (int d = lane; d < Wp; d += 32) dst[d] = d < W ? __bfloat162float(src[d]) : 0.f;
}

// ROWS rows (row i: `src[i]`, null: zeros) into shared memory rows `dst0 + i * dst_stride`.  bfloat16 rows of a multiple of 8
// elements on 16-byte addresses: every load of the batch is issued before the first conversion, so the batch costs one
// trip to memory.
template <int ROWS>
__device__ __forceinline__ void al_stage_rows(float* dst0, int dst_stride, const float* const (&src)[ROWS], int W, int Wp, int lane) {
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        float* dst = dst0 + i * dst_stride;
        if (src[i]) al_stage_row<float>(dst, src[i], W, Wp, lane);
        else for (int d = lane; d < Wp; d += 32) dst[d] = 0.f;
    }
}
template <int ROWS>
__device__ __forceinline__ void al_stage_rows(float* dst0, int dst_stride, const bf16* const (&src)[ROWS], int W, int Wp, int lane) {
    bool fast = (W & 7) == 0;
#pragma unroll
    for (int i = 0; i < ROWS; ++i) fast = fast && (((uintptr_t)src[i]) & 15) == 0;
    if (!fast) {
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            float* dst = dst0 + i * dst_stride;
            if (src[i]) al_stage_row<bf16>(dst, src[i], W, Wp, lane);
            else for (int d = lane; d < Wp; d += 32) dst[d] = 0.f;
        }
        return;
    }
    uint4 raw[ROWS][4];   // (rows of up to 1,024 elements: 4 pieces of 256)
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int d = lane * 8 + c * 256;
            raw[i][c] = (src[i] && d < W) ? *reinterpret_cast<const uint4*>(src[i] + d) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int d = lane * 8 + c * 256;
            if (d >= W) continue;
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[i][c]);
            const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
            const float2 e = __bfloat1622float2(h2[2]), f = __bfloat1622float2(h2[3]);
            float* dst = dst0 + i * dst_stride + d;
            *reinterpret_cast<float4*>(dst) = make_float4(a.x, a.y, b.x, b.y);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(e.x, e.y, f.x, f.y);
        }
}

template <typename T, int NR4>
__global__ void __launch_bounds__(AL_WARPS * 32)
latent_attention_kernel(const T* __restrict__ qa, const T* __restrict__ pool, const int* __restrict__ block_table,
                        int max_blocks, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                        T* __restrict__ out, float* __restrict__ scratch, float scale, int H, int C, int R, int S, int runs,
                        int window) {
    extern __shared__ __align__(16) float al_smem[];
    const int W = C + R, Wp = (W + 3) & ~3, ld = al_row_stride(W);
    float* k_s = al_smem;                    // [AL_TILE][ld]
    float* q_s = k_s + AL_TILE * ld;         // [AL_HEADS][Wp]
    float* p_s = q_s + AL_HEADS * Wp;        // [AL_WARPS][AL_TILE][AL_HW]
    const int t = blockIdx.x, h0 = blockIdx.y * AL_HEADS, run = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hw0 = h0 + warp * AL_HW;       // the warp's first head
    pdl_wait();
    pdl_trigger();
    const int kv_len = positions[t] + 1;
    const int* bt = block_table + (size_t)seq_of_token[t] * max_blocks;
    // with a window only the last `window` positions count: the tiles before the first of them are never touched (their
    // pages may be gone), and in its tile the rows before it are staged as zeros and left out of the softmax
    const int start = (window > 0 && kv_len > window) ? kv_len - window : 0;
    const int first_tile = start / AL_TILE;
    const int tiles = (kv_len + AL_TILE - 1) / AL_TILE;
    const int per_run = (tiles - first_tile + runs - 1) / runs;
    const int tile0 = first_tile + run * per_run, tile1 = min(tiles, tile0 + per_run);

    {
        const T* src[AL_HEADS / AL_WARPS];
#pragma unroll
        for (int i = 0; i < AL_HEADS / AL_WARPS; ++i) {
            const int hh = warp + i * AL_WARPS;
            src[i] = h0 + hh < H ? qa + ((size_t)t * H + h0 + hh) * W : nullptr;
        }
        al_stage_rows<AL_HEADS / AL_WARPS>(q_s + warp * Wp, AL_WARPS * Wp, src, W, Wp, lane);
    }

    float acc[AL_HW][NR4][4];
#pragma unroll
    for (int hh = 0; hh < AL_HW; ++hh)
#pragma unroll
        for (int i = 0; i < NR4; ++i) acc[hh][i][0] = acc[hh][i][1] = acc[hh][i][2] = acc[hh][i][3] = 0.f;
    float m[AL_HW], l[AL_HW];
#pragma unroll
    for (int hh = 0; hh < AL_HW; ++hh) { m[hh] = -INFINITY; l[hh] = 0.f; }
    const float* qw = q_s + warp * AL_HW * Wp;
    float* pw = p_s + warp * AL_TILE * AL_HW;

    for (int tile = tile0; tile < tile1; ++tile) {
        const int j0 = tile * AL_TILE, n = min(AL_TILE, kv_len - j0);
        __syncthreads();   // the tile before this one has been used (and, the first time, the queries are written)
        const int lo = max(0, start - j0);   // rows of the tile before the window
        const int my_page = (lane < n && lane >= lo) ? bt[(j0 + lane) / S] : 0;   // (one trip to the table for the tile's 32 rows)
#pragma unroll
        for (int b = 0; b < AL_TILE / AL_WARPS; b += 4) {   // four rows of the warp's eight at a time
            const T* src[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = warp + (b + i) * AL_WARPS;
                const int page = __shfl_sync(0xffffffffu, my_page, r);
                src[i] = (r < n && r >= lo) ? pool + ((size_t)page * S + ((j0 + r) % S)) * W : nullptr;
            }
            al_stage_rows<4>(k_s + (warp + b * AL_WARPS) * ld, AL_WARPS * ld, src, W, Wp, lane);
        }
        __syncthreads();
        if (hw0 >= H) continue;
        float dot[AL_HW] = {0.f, 0.f, 0.f, 0.f};
        const float* kr = k_s + lane * ld;
#pragma unroll 4
        for (int d = 0; d < Wp; d += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
            for (int hh = 0; hh < AL_HW; ++hh) {
                const float4 q4 = *reinterpret_cast<const float4*>(qw + hh * Wp + d);
                dot[hh] = fmaf(q4.x, k4.x, dot[hh]);
                dot[hh] = fmaf(q4.y, k4.y, dot[hh]);
                dot[hh] = fmaf(q4.z, k4.z, dot[hh]);
                dot[hh] = fmaf(q4.w, k4.w, dot[hh]);
            }
        }
        float p[AL_HW];
#pragma unroll
        for (int hh = 0; hh < AL_HW; ++hh) {
            const bool seen = lane < n && lane >= lo;
            const float s = seen ? dot[hh] * scale : -INFINITY;
            const float m_new = fmaxf(m[hh], warp_max(s));
            p[hh] = seen ? expf(s - m_new) : 0.f;
            const float alpha = expf(m[hh] - m_new);   // m = -inf before the first tile: 0
            l[hh] = l[hh] * alpha + warp_sum(p[hh]);
#pragma unroll
            for (int i = 0; i < NR4; ++i) {
                acc[hh][i][0] *= alpha; acc[hh][i][1] *= alpha; acc[hh][i][2] *= alpha; acc[hh][i][3] *= alpha;
            }
            m[hh] = m_new;
        }
        __syncwarp();
        *reinterpret_cast<float4*>(pw + lane * AL_HW) = make_float4(p[0], p[1], p[2], p[3]);
        __syncwarp();
#pragma unroll 2
        for (int jj = lo; jj < n; ++jj) {
            const float4 p4 = *reinterpret_cast<const float4*>(pw + jj * AL_HW);
            const float pj[AL_HW] = {p4.x, p4.y, p4.z, p4.w};
            const float* vr = k_s + jj * ld;
#pragma unroll
            for (int i = 0; i < NR4; ++i) {
                const int d = 4 * (lane + 32 * i);
                if (d < C) {
                    const float4 v4 = *reinterpret_cast<const float4*>(vr + d);
#pragma unroll
                    for (int hh = 0; hh < AL_HW; ++hh) {
                        acc[hh][i][0] = fmaf(pj[hh], v4.x, acc[hh][i][0]);
                        acc[hh][i][1] = fmaf(pj[hh], v4.y, acc[hh][i][1]);
                        acc[hh][i][2] = fmaf(pj[hh], v4.z, acc[hh][i][2]);
                        acc[hh][i][3] = fmaf(pj[hh], v4.w, acc[hh][i][3]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int hh = 0; hh < AL_HW; ++hh) {
        const int h = hw0 + hh;
        if (h >= H) continue;
        if (runs == 1) {
            const float inv = 1.f / l[hh];   // (a token always sees itself: l > 0)
            T* dst = out + ((size_t)t * H + h) * C;
#pragma unroll
            for (int i = 0; i < NR4; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int d = 4 * (lane + 32 * i) + c;
                    if (d < C) dst[d] = from_f32<T>(acc[hh][i][c] * inv);
                }
            continue;
        }
        float* dst = scratch + (((size_t)t * H + h) * runs + run) * (C + 2);
        if (lane == 0) { dst[0] = m[hh]; dst[1] = l[hh]; }
#pragma unroll
        for (int i = 0; i < NR4; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int d = 4 * (lane + 32 * i) + c;
                if (d < C) dst[2 + d] = acc[hh][i][c];
            }
    }
}

// One block per (token, head): the runs' parts added in run order.  Every run's weight exp(m_r - M) / L is formed once, in
// shared memory (runs <= AL_MAX_RUNS); a channel's sum then has all its reads in flight together.
#define AL_MAX_RUNS 1024
template <typename T>
__global__ void latent_attention_join_kernel(const float* __restrict__ scratch, T* __restrict__ out, int H, int C, int runs) {
    __shared__ float w_s[AL_MAX_RUNS];
    __shared__ float l_s[AL_MAX_RUNS];
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* src = scratch + ((size_t)t * H + h) * runs * (C + 2);
    for (int r = threadIdx.x; r < runs; r += blockDim.x) {
        w_s[r] = src[(size_t)r * (C + 2)];
        l_s[r] = src[(size_t)r * (C + 2) + 1];
    }
    __syncthreads();
    float M = -INFINITY;
    for (int r = 0; r < runs; ++r) M = fmaxf(M, w_s[r]);
    float L = 0.f;
    for (int r = 0; r < runs; ++r)
        if (w_s[r] != -INFINITY) L += l_s[r] * expf(w_s[r] - M);
    __syncthreads();
    for (int r = threadIdx.x; r < runs; r += blockDim.x) w_s[r] = w_s[r] != -INFINITY ? expf(w_s[r] - M) / L : 0.f;
    __syncthreads();
    for (int d = threadIdx.x; d < C; d += blockDim.x) {
        float o = 0.f;
#pragma unroll 16
        for (int r = 0; r < runs; ++r) o = fmaf(w_s[r], src[(size_t)r * (C + 2) + 2 + d], o);
        out[((size_t)t * H + h) * C + d] = from_f32<T>(o);
    }
}

template <typename T>
static int launch_latent_attention(const T* qa, const T* pool, const int* block_table, int max_blocks, const int* seq_of_token,
                                   const int* positions, T* out, float* scratch, float scale, int tokens, int H, int C, int R,
                                   int S, int runs, int window, cudaStream_t stream) {
    const int W = C + R, Wp = (W + 3) & ~3;
    const size_t smem = sizeof(float) * ((size_t)AL_TILE * al_row_stride(W) + (size_t)AL_HEADS * Wp + AL_WARPS * AL_TILE * AL_HW);
    const size_t smem_max = sizeof(float) * ((size_t)AL_TILE * al_row_stride(1024) + (size_t)AL_HEADS * 1024 + AL_WARPS * AL_TILE * AL_HW);
    dim3 grid(tokens, (H + AL_HEADS - 1) / AL_HEADS, runs);
    static bool configured[4][VX_MAX_DEVICES];
#define AL_GO(NR4, SLOT)                                                                                              \
    do {                                                                                                              \
        if (int rc = vx_configure_smem(latent_attention_kernel<T, NR4>, smem_max, configured[SLOT])) return rc;        \
        VX_LAUNCH_K(VX_K_ATTENTION, (latent_attention_kernel<T, NR4>), grid, AL_WARPS * 32, smem, stream, qa, pool,    \
                    block_table, max_blocks, seq_of_token, positions, out, scratch, scale, H, C, R, S, runs, window);  \
    } while (0)
    if (C <= 128) AL_GO(1, 0);
    else if (C <= 256) AL_GO(2, 1);
    else if (C <= 512) AL_GO(4, 2);
    else AL_GO(8, 3);
#undef AL_GO
    if (runs > 1)
        VX_LAUNCH_K(VX_K_JOIN, (latent_attention_join_kernel<T>), dim3(tokens, H), min(1024, (C + 31) / 32 * 32), 0, stream,
                    (const float*)scratch, out, H, C, runs);   // (a thread per channel: its reads over the runs in flight together)
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// qa [tokens, H, C + R] folded queries; pool [pages, 1, S, C + R]; token row t is request seq_of_token[t] at position
// positions[t] and sees positions 0 .. positions[t], with a window > 0 only the last `window` of them.  out [tokens, H, C].
// scratch: float32, tokens * H * runs * (C + 2) elements, needed for runs > 1.
extern "C" int vx_latent_attention_window(const void* qa, const void* pool, const int* block_table, int max_blocks,
                                          const int* seq_of_token, const int* positions, void* out, float* scratch, float scale,
                                          int tokens, int H, int C, int R, int S, int runs, int window, int dtype,
                                          cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (window < 0) return VX_ERR_SHAPE;
    if (H <= 0 || C <= 0 || R < 0 || S <= 0 || max_blocks <= 0 || C + R > 1024 || runs < 1 || runs > AL_MAX_RUNS) return VX_ERR_SHAPE;
    if (runs > 1 && !scratch) return VX_ERR_SHAPE;
    if ((H + AL_HEADS - 1) / AL_HEADS > 65535 || runs > 65535) return VX_ERR_LIMIT;
    if (dtype == VX_F32)
        return launch_latent_attention<float>((const float*)qa, (const float*)pool, block_table, max_blocks, seq_of_token,
                                              positions, (float*)out, scratch, scale, tokens, H, C, R, S, runs, window, stream);
    if (dtype == VX_BF16)
        return launch_latent_attention<bf16>((const bf16*)qa, (const bf16*)pool, block_table, max_blocks, seq_of_token,
                                             positions, (bf16*)out, scratch, scale, tokens, H, C, R, S, runs, window, stream);
    return VX_ERR_DTYPE;
}

extern "C" int vx_latent_attention(const void* qa, const void* pool, const int* block_table, int max_blocks,
                                   const int* seq_of_token, const int* positions, void* out, float* scratch, float scale,
                                   int tokens, int H, int C, int R, int S, int runs, int dtype, cudaStream_t stream) {
    return vx_latent_attention_window(qa, pool, block_table, max_blocks, seq_of_token, positions, out, scratch, scale, tokens,
                                      H, C, R, S, runs, 0, dtype, stream);
}

// The cached rows of the segments of a step, gathered page by page into one matrix: segment s (request seq_list[s], or
// s) holds positions 0 .. kv_offsets + new tokens - 1; its rows start at row table[s][0] * S_out of `rows` and are filled
// with zeros up to the next multiple of S_out.  With a window > 0 only the positions from
// first = floor(max(0, kv_offsets + 1 - window), S_out) on are copied (what the segment's first query sees, from a block's
// start), position j to row table[s][0] * S_out + j - first.  grid (run of 32 rows, segment); 8 warps, a warp per row.
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ pool, const int* __restrict__ block_table, int max_blocks,
                                     const int* __restrict__ cu_seqlens, const int* __restrict__ kv_offsets,
                                     const int* __restrict__ seq_list, const int* __restrict__ out_table, int out_blocks,
                                     T* __restrict__ rows, int W, int S, int S_out, int window) {
    pdl_wait();
    pdl_trigger();
    const int s = blockIdx.y, seq = seq_list ? seq_list[s] : s;
    const int kv_len = kv_offsets[seq] + cu_seqlens[seq + 1] - cu_seqlens[seq];
    const int seen_from = window > 0 ? max(0, kv_offsets[seq] + 1 - window) : 0;
    const int first = seen_from / S_out * S_out;
    const int padded = (kv_len + S_out - 1) / S_out * S_out;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* bt = block_table + (size_t)seq * max_blocks;
    const size_t base = (size_t)out_table[(size_t)s * out_blocks] * S_out;
    for (int j = first + blockIdx.x * 32 + warp; j < min(padded, first + blockIdx.x * 32 + 32); j += 8) {
        T* dst = rows + (base + j - first) * W;
        if (j < kv_len && j >= seen_from) {   // (a position before the window may lie in a page that was given back)
            const T* src = pool + ((size_t)bt[j / S] * S + (j % S)) * W;
            for (int d = lane; d < W; d += 32) dst[d] = src[d];
        } else {
            for (int d = lane; d < W; d += 32) dst[d] = from_f32<T>(0.f);
        }
    }
}

// pool [pages, 1, S, W]; out_table int32 [segments, out_blocks]: the blocks of S_out rows that segment s takes in `rows`
// (consecutive, the first one listed first); max_kv bounds the rows that any segment takes (its positions after the step,
// less the ones before its window's first block).
extern "C" int vx_latent_gather_window(const void* pool, const int* block_table, int max_blocks, const int* cu_seqlens,
                                       const int* kv_offsets, const int* seq_list, const int* out_table, int out_blocks, void* rows,
                                       int segments, int max_kv, int W, int S, int S_out, int window, int dtype,
                                       cudaStream_t stream) {
    if (segments <= 0 || max_kv <= 0) return VX_OK;
    if (W <= 0 || S <= 0 || S_out <= 0 || max_blocks <= 0 || out_blocks <= 0 || window < 0) return VX_ERR_SHAPE;
    if (segments > 65535) return VX_ERR_LIMIT;
    const int padded = (max_kv + S_out - 1) / S_out * S_out;
    dim3 grid((padded + 31) / 32, segments);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (latent_gather_kernel<float>), grid, 256, 0, stream, (const float*)pool, block_table,
                    max_blocks, cu_seqlens, kv_offsets, seq_list, out_table, out_blocks, (float*)rows, W, S, S_out, window);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (latent_gather_kernel<bf16>), grid, 256, 0, stream, (const bf16*)pool, block_table,
                    max_blocks, cu_seqlens, kv_offsets, seq_list, out_table, out_blocks, (bf16*)rows, W, S, S_out, window);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

extern "C" int vx_latent_gather(const void* pool, const int* block_table, int max_blocks, const int* cu_seqlens,
                                const int* kv_offsets, const int* seq_list, const int* out_table, int out_blocks, void* rows,
                                int segments, int max_kv, int W, int S, int S_out, int dtype, cudaStream_t stream) {
    return vx_latent_gather_window(pool, block_table, max_blocks, cu_seqlens, kv_offsets, seq_list, out_table, out_blocks, rows,
                                   segments, max_kv, W, S, S_out, 0, dtype, stream);
}
