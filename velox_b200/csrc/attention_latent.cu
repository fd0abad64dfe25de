// Attention over cached latent rows: every position keeps ONE row of W = C + R elements (C latent channels, then R
// rotated channels that all heads share), and a query head brings a folded query of the same width, so that
//   score(i, j) = qa_i . row_j * scale,   causal softmax,   out_i = sum_j w_ij row_j[0 .. C)
// (the value is the first C elements of the key's row).  All heads of a token read the same rows, so a block stages
// a tile of rows once for up to eight heads.
//
// One block per (token row, group of 8 heads, run of keys); a warp per head.  A tile of 32 rows is copied into shared
// memory as float32, each row on an odd stride, so that lane j forms the whole product qa . row_j without bank
// conflicts (the folded queries lie beside the tile, read as broadcasts); the warp keeps a running maximum, sum and
// accumulator (lane l owns value channels l, l + 32, ...) and adds the 32 rows in key order.  With `runs` > 1 a token's
// tiles are dealt to the runs in contiguous stretches, every run writes (maximum, sum, accumulator) to a scratch
// buffer, and a join kernel adds them in run order.  Scores, weights and sums are float32; the order of every sum
// depends on the token's own position and on `runs` alone.
#include "common.cuh"

#define AL_WARPS 8
#define AL_TILE 32

template <typename T, int NR>
__global__ void __launch_bounds__(AL_WARPS * 32)
latent_attention_kernel(const T* __restrict__ qa, const T* __restrict__ pool, const int* __restrict__ block_table,
                        int max_blocks, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                        T* __restrict__ out, float* __restrict__ scratch, float scale, int H, int C, int R, int S, int runs) {
    extern __shared__ float al_smem[];
    const int W = C + R, ld = W | 1;
    float* k_s = al_smem;                    // [AL_TILE][ld]
    float* q_s = k_s + AL_TILE * ld;         // [AL_WARPS][W]
    const int t = blockIdx.x, h0 = blockIdx.y * AL_WARPS, run = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = h0 + warp;
    const bool live = h < H;
    pdl_wait();
    pdl_trigger();
    const int kv_len = positions[t] + 1;
    const int* bt = block_table + (size_t)seq_of_token[t] * max_blocks;
    const int tiles = (kv_len + AL_TILE - 1) / AL_TILE;
    const int per_run = (tiles + runs - 1) / runs;
    const int tile0 = run * per_run, tile1 = min(tiles, tile0 + per_run);

    const int heads_here = min(AL_WARPS, H - h0);
    for (int i = threadIdx.x; i < heads_here * W; i += blockDim.x)
        q_s[i] = to_f32(qa[((size_t)t * H + h0) * W + i]);

    float acc[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const float* qh = q_s + warp * W;

    for (int tile = tile0; tile < tile1; ++tile) {
        const int j0 = tile * AL_TILE, n = min(AL_TILE, kv_len - j0);
        __syncthreads();   // the tile before this one has been used (and, the first time, the queries are written)
        for (int r = warp; r < n; r += AL_WARPS) {
            const int j = j0 + r;
            const T* src = pool + ((size_t)bt[j / S] * S + (j % S)) * W;
            float* dst = k_s + r * ld;
            for (int d = lane; d < W; d += 32) dst[d] = to_f32(src[d]);
        }
        __syncthreads();
        if (!live) continue;
        float s = -INFINITY;
        if (lane < n) {
            const float* kr = k_s + lane * ld;
            float dot = 0.f;
            for (int d = 0; d < W; ++d) dot = fmaf(qh[d], kr[d], dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = lane < n ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);   // m = -inf before the first tile: 0
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < NR; ++i) acc[i] *= alpha;
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const float* vr = k_s + jj * ld;
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                const int d = lane + 32 * i;
                if (d < C) acc[i] = fmaf(pj, vr[d], acc[i]);
            }
        }
        m = m_new;
    }
    if (!live) return;
    if (runs == 1) {
        const float inv = 1.f / l;   // (a token always sees itself: l > 0)
        T* dst = out + ((size_t)t * H + h) * C;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int d = lane + 32 * i;
            if (d < C) dst[d] = from_f32<T>(acc[i] * inv);
        }
        return;
    }
    float* dst = scratch + (((size_t)t * H + h) * runs + run) * (C + 2);
    if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int d = lane + 32 * i;
        if (d < C) dst[2 + d] = acc[i];
    }
}

// One block per (token, head): the runs' parts added in run order.
template <typename T>
__global__ void latent_attention_join_kernel(const float* __restrict__ scratch, T* __restrict__ out, int H, int C, int runs) {
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* src = scratch + ((size_t)t * H + h) * runs * (C + 2);
    float M = -INFINITY;
    for (int r = 0; r < runs; ++r) M = fmaxf(M, src[(size_t)r * (C + 2)]);
    float L = 0.f;
    for (int r = 0; r < runs; ++r) {
        const float mr = src[(size_t)r * (C + 2)];
        if (mr != -INFINITY) L += src[(size_t)r * (C + 2) + 1] * expf(mr - M);
    }
    for (int d = threadIdx.x; d < C; d += blockDim.x) {
        float o = 0.f;
        for (int r = 0; r < runs; ++r) {
            const float mr = src[(size_t)r * (C + 2)];
            if (mr != -INFINITY) o += src[(size_t)r * (C + 2) + 2 + d] * expf(mr - M);
        }
        out[((size_t)t * H + h) * C + d] = from_f32<T>(o / L);
    }
}

template <typename T>
static int launch_latent_attention(const T* qa, const T* pool, const int* block_table, int max_blocks, const int* seq_of_token,
                                   const int* positions, T* out, float* scratch, float scale, int tokens, int H, int C, int R,
                                   int S, int runs, cudaStream_t stream) {
    const int W = C + R;
    const size_t smem = sizeof(float) * ((size_t)AL_TILE * (W | 1) + (size_t)AL_WARPS * W);
    const size_t smem_max = sizeof(float) * ((size_t)AL_TILE * 1025 + (size_t)AL_WARPS * 1024);
    dim3 grid(tokens, (H + AL_WARPS - 1) / AL_WARPS, runs);
    static bool configured[3][VX_MAX_DEVICES];
#define AL_GO(NR, SLOT)                                                                                               \
    do {                                                                                                              \
        if (int rc = vx_configure_smem(latent_attention_kernel<T, NR>, smem_max, configured[SLOT])) return rc;         \
        VX_LAUNCH_K(VX_K_ATTENTION, (latent_attention_kernel<T, NR>), grid, AL_WARPS * 32, smem, stream, qa, pool,     \
                    block_table, max_blocks, seq_of_token, positions, out, scratch, scale, H, C, R, S, runs);          \
    } while (0)
    if (C <= 256) AL_GO(8, 0);
    else if (C <= 512) AL_GO(16, 1);
    else AL_GO(32, 2);
#undef AL_GO
    if (runs > 1)
        VX_LAUNCH_K(VX_K_JOIN, (latent_attention_join_kernel<T>), dim3(tokens, H), C >= 256 ? 128 : 64, 0, stream,
                    (const float*)scratch, out, H, C, runs);
    VX_LAUNCH_CHECK();
    return VX_OK;
}

// qa [tokens, H, C + R] folded queries; pool [pages, 1, S, C + R]; token row t is request seq_of_token[t] at position
// positions[t] and sees positions 0 .. positions[t].  out [tokens, H, C].  scratch: float32, tokens * H * runs * (C + 2)
// elements, needed for runs > 1.
extern "C" int vx_latent_attention(const void* qa, const void* pool, const int* block_table, int max_blocks,
                                   const int* seq_of_token, const int* positions, void* out, float* scratch, float scale,
                                   int tokens, int H, int C, int R, int S, int runs, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return VX_OK;
    if (H <= 0 || C <= 0 || R < 0 || S <= 0 || max_blocks <= 0 || C + R > 1024 || runs < 1) return VX_ERR_SHAPE;
    if (runs > 1 && !scratch) return VX_ERR_SHAPE;
    if ((H + AL_WARPS - 1) / AL_WARPS > 65535 || runs > 65535) return VX_ERR_LIMIT;
    if (dtype == VX_F32)
        return launch_latent_attention<float>((const float*)qa, (const float*)pool, block_table, max_blocks, seq_of_token,
                                              positions, (float*)out, scratch, scale, tokens, H, C, R, S, runs, stream);
    if (dtype == VX_BF16)
        return launch_latent_attention<bf16>((const bf16*)qa, (const bf16*)pool, block_table, max_blocks, seq_of_token,
                                             positions, (bf16*)out, scratch, scale, tokens, H, C, R, S, runs, stream);
    return VX_ERR_DTYPE;
}

// The cached rows of the segments of a step, gathered page by page into one matrix: segment s (request seq_list[s], or
// s) holds positions 0 .. kv_offsets + new tokens - 1; its rows start at row table[s][0] * S_out of `rows` and are filled
// with zeros up to the next multiple of S_out.  grid (run of 32 rows, segment); 8 warps, a warp per row.
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ pool, const int* __restrict__ block_table, int max_blocks,
                                     const int* __restrict__ cu_seqlens, const int* __restrict__ kv_offsets,
                                     const int* __restrict__ seq_list, const int* __restrict__ out_table, int out_blocks,
                                     T* __restrict__ rows, int W, int S, int S_out) {
    pdl_wait();
    pdl_trigger();
    const int s = blockIdx.y, seq = seq_list ? seq_list[s] : s;
    const int kv_len = kv_offsets[seq] + cu_seqlens[seq + 1] - cu_seqlens[seq];
    const int padded = (kv_len + S_out - 1) / S_out * S_out;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* bt = block_table + (size_t)seq * max_blocks;
    const size_t base = (size_t)out_table[(size_t)s * out_blocks] * S_out;
    for (int j = blockIdx.x * 32 + warp; j < min(padded, blockIdx.x * 32 + 32); j += 8) {
        T* dst = rows + (base + j) * W;
        if (j < kv_len) {
            const T* src = pool + ((size_t)bt[j / S] * S + (j % S)) * W;
            for (int d = lane; d < W; d += 32) dst[d] = src[d];
        } else {
            for (int d = lane; d < W; d += 32) dst[d] = from_f32<T>(0.f);
        }
    }
}

// pool [pages, 1, S, W]; out_table int32 [segments, out_blocks]: the blocks of S_out rows that segment s takes in `rows`
// (consecutive, the first one listed first); max_kv bounds any segment's positions after the step.
extern "C" int vx_latent_gather(const void* pool, const int* block_table, int max_blocks, const int* cu_seqlens,
                                const int* kv_offsets, const int* seq_list, const int* out_table, int out_blocks, void* rows,
                                int segments, int max_kv, int W, int S, int S_out, int dtype, cudaStream_t stream) {
    if (segments <= 0 || max_kv <= 0) return VX_OK;
    if (W <= 0 || S <= 0 || S_out <= 0 || max_blocks <= 0 || out_blocks <= 0) return VX_ERR_SHAPE;
    if (segments > 65535) return VX_ERR_LIMIT;
    const int padded = (max_kv + S_out - 1) / S_out * S_out;
    dim3 grid((padded + 31) / 32, segments);
    if (dtype == VX_F32)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (latent_gather_kernel<float>), grid, 256, 0, stream, (const float*)pool, block_table,
                    max_blocks, cu_seqlens, kv_offsets, seq_list, out_table, out_blocks, (float*)rows, W, S, S_out);
    else if (dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_ELEMENTWISE, (latent_gather_kernel<bf16>), grid, 256, 0, stream, (const bf16*)pool, block_table,
                    max_blocks, cu_seqlens, kv_offsets, seq_list, out_table, out_blocks, (bf16*)rows, W, S, S_out);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}
