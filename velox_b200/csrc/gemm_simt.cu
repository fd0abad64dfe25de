// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]): the plain matrix product.
//
// Multiply-adds on the CUDA cores in float32, no tensor cores, no reduced
// precision mode: this is the matrix product of the 32-bit path, and the
// reference against which the tensor-core products are checked.  Every output
// element is the sum over k in ascending order, so a row's result does not
// depend on how many rows the call has.  Any M, N, K.
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16

template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
gemm_nt_simt_kernel(const TA* __restrict__ A, const TA* __restrict__ W, const float* __restrict__ bias,
                    TC* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc, long long sa, long long sw,
                    long long sc) {
    pdl_wait();
    pdl_trigger();
    A += (size_t)blockIdx.z * sa;   // (a batch of products: member z has its own A, W and C, no bias)
    W += (size_t)blockIdx.z * sw;
    C += (size_t)blockIdx.z * sc;
    __shared__ float As[GS_BK][GS_BM + 1];
    __shared__ float Ws[GS_BK][GS_BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    const int lk = tid & 15, lr = tid >> 4;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GS_BK) {
        const int k = k0 + lk;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = lr + 16 * i;
            const int m = m0 + r, n = n0 + r;
            As[lk][r] = (m < M && k < K) ? to_f32(A[(size_t)m * lda + k]) : 0.f;
            Ws[lk][r] = (n < N && k < K) ? to_f32(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GS_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty + 16 * i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            C[(size_t)m * ldc + n] = from_f32<TC>(v);
        }
    }
}

// in_dtype: element type of A and W; out_dtype: element type of C.
// A batch of `batch` products: member z reads A + z sa, W + z sw and writes C + z sc (strides in elements).
extern "C" int vx_gemm_nt_simt_batched(const void* A, const void* W, const float* bias, void* C, int M, int N,
                                       int K, int lda, int ldw, int ldc, int batch, long long sa, long long sw,
                                       long long sc, int in_dtype, int out_dtype, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return VX_OK;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return VX_ERR_SHAPE;
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM, batch);
    if (grid.y > 65535 || batch > 65535) return VX_ERR_LIMIT;
    if (in_dtype == VX_F32 && out_dtype == VX_F32)
        VX_LAUNCH_K(VX_K_GEMM, (gemm_nt_simt_kernel<float, float>), grid, 256, 0, stream, (const float*)A, (const float*)W, bias, (float*)C, M, N, K, lda, ldw, ldc, sa, sw, sc);
    else if (in_dtype == VX_BF16 && out_dtype == VX_BF16)
        VX_LAUNCH_K(VX_K_GEMM, (gemm_nt_simt_kernel<bf16, bf16>), grid, 256, 0, stream, (const bf16*)A, (const bf16*)W, bias, (bf16*)C, M, N, K, lda, ldw, ldc, sa, sw, sc);
    else if (in_dtype == VX_BF16 && out_dtype == VX_F32)
        VX_LAUNCH_K(VX_K_GEMM, (gemm_nt_simt_kernel<bf16, float>), grid, 256, 0, stream, (const bf16*)A, (const bf16*)W, bias, (float*)C, M, N, K, lda, ldw, ldc, sa, sw, sc);
    else
        return VX_ERR_DTYPE;
    VX_LAUNCH_CHECK();
    return VX_OK;
}

extern "C" int vx_gemm_nt_simt(const void* A, const void* W, const float* bias, void* C, int M, int N,
                               int K, int lda, int ldw, int ldc, int in_dtype, int out_dtype,
                               cudaStream_t stream) {
    return vx_gemm_nt_simt_batched(A, W, bias, C, M, N, K, lda, ldw, ldc, 1, 0, 0, 0, in_dtype, out_dtype, stream);
}

// A batch of products of FEW rows (M <= 8, a decode step's tokens): member z's C[m, n] = sum_k A[m, k] W[n, k] with
// bfloat16 A and W and K a multiple of 8.  One warp per output column n of a member: the M rows of A lie in shared
// memory as float32, a lane reads 8 consecutive k of W's row at a time (16 bytes) and keeps M partial sums, which
// the warp adds at the end.  W is read once, by as many blocks as the batch has members times N / 8, where the tiled
// kernel above would give each member N / 64 blocks that walk K in steps of 16.  The order of a sum is fixed by K alone.
#define GF_WARPS 8
#define GF_MAX_M 8
template <typename TC>
__global__ void __launch_bounds__(GF_WARPS * 32)
gemm_few_rows_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, TC* __restrict__ C, int M, int N, int K, int lda,
                     int ldw, int ldc, long long sa, long long sw, long long sc) {
    extern __shared__ float gf_a[];   // [M][K]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * GF_WARPS + warp;
    W += (size_t)blockIdx.y * sw;
    // the weights depend on no earlier kernel: the lane's first piece is asked for before the wait
    uint4 first = make_uint4(0u, 0u, 0u, 0u);
    if (n < N && lane * 8 < K) first = *reinterpret_cast<const uint4*>(W + (size_t)n * ldw + lane * 8);
    pdl_wait();
    pdl_trigger();
    A += (size_t)blockIdx.y * sa;
    C += (size_t)blockIdx.y * sc;
    for (int i = threadIdx.x; i < M * K; i += blockDim.x) {
        const int m = i / K, k = i - m * K;
        gf_a[i] = __bfloat162float(A[(size_t)m * lda + k]);
    }
    __syncthreads();
    if (n >= N) return;
    float acc[GF_MAX_M];
#pragma unroll
    for (int m = 0; m < GF_MAX_M; ++m) acc[m] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 raw = k == lane * 8 ? first : *reinterpret_cast<const uint4*>(W + (size_t)n * ldw + k);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float w[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            w[2 * e] = f.x;
            w[2 * e + 1] = f.y;
        }
#pragma unroll
        for (int m = 0; m < GF_MAX_M; ++m) {
            if (m >= M) break;
            const float4 a0 = *reinterpret_cast<const float4*>(gf_a + m * K + k), a1 = *reinterpret_cast<const float4*>(gf_a + m * K + k + 4);
            acc[m] = fmaf(a0.x, w[0], acc[m]); acc[m] = fmaf(a0.y, w[1], acc[m]);
            acc[m] = fmaf(a0.z, w[2], acc[m]); acc[m] = fmaf(a0.w, w[3], acc[m]);
            acc[m] = fmaf(a1.x, w[4], acc[m]); acc[m] = fmaf(a1.y, w[5], acc[m]);
            acc[m] = fmaf(a1.z, w[6], acc[m]); acc[m] = fmaf(a1.w, w[7], acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < GF_MAX_M; ++m) {
        if (m >= M) break;
        const float v = warp_sum(acc[m]);
        if (lane == 0) C[(size_t)m * ldc + n] = from_f32<TC>(v);
    }
}

// A, W bfloat16; C bfloat16 or float32 (`out_dtype`).  M <= 8, K a multiple of 8 up to 4,096, W's rows on 16-byte
// addresses (ldw and sw multiples of 8, the pointer aligned).
extern "C" int vx_gemm_few_rows_batched(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                                        int batch, long long sa, long long sw, long long sc, int out_dtype, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return VX_OK;
    if (M > GF_MAX_M || K <= 0 || (K & 7) || K > 4096 || lda < K || ldw < K || ldc < N) return VX_ERR_SHAPE;
    if ((ldw & 7) || (sw & 7) || (((uintptr_t)W) & 15)) return VX_ERR_ALIGN;
    dim3 grid((N + GF_WARPS - 1) / GF_WARPS, batch);
    if (batch > 65535) return VX_ERR_LIMIT;
    const size_t smem = (size_t)M * K * sizeof(float);
    static bool configured[2][VX_MAX_DEVICES];
    if (out_dtype == VX_BF16) {
        if (int rc = vx_configure_smem(gemm_few_rows_kernel<bf16>, (size_t)GF_MAX_M * 4096 * sizeof(float), configured[0])) return rc;
        VX_LAUNCH_K(VX_K_GEMM, (gemm_few_rows_kernel<bf16>), grid, GF_WARPS * 32, smem, stream, (const bf16*)A, (const bf16*)W, (bf16*)C,
                    M, N, K, lda, ldw, ldc, sa, sw, sc);
    } else if (out_dtype == VX_F32) {
        if (int rc = vx_configure_smem(gemm_few_rows_kernel<float>, (size_t)GF_MAX_M * 4096 * sizeof(float), configured[1])) return rc;
        VX_LAUNCH_K(VX_K_GEMM, (gemm_few_rows_kernel<float>), grid, GF_WARPS * 32, smem, stream, (const bf16*)A, (const bf16*)W, (float*)C,
                    M, N, K, lda, ldw, ldc, sa, sw, sc);
    } else {
        return VX_ERR_DTYPE;
    }
    VX_LAUNCH_CHECK();
    return VX_OK;
}
