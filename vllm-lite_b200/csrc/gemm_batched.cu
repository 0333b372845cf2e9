// Many small matrix products in one launch:  C_b[M, N] = A_b[M, K] * W_b[N, K]^T.
//
// Two uses.  (1) One product per head on column slices of wide activations (the latent attention's
// query absorption and value expansion): batch b reads A + b * a_bs with row stride lda, W + b * w_bs,
// and writes C + b * c_bs with row stride ldc.  (2) One product per expert on rows that were sorted by
// expert (routed feed-forwards): `tile_group[y]` names the weight matrix (W + g * w_gs) of the tile of
// BM rows number y, or is negative for a tile beyond the sorted rows, which does nothing.
//
// Plain FFMA with float32 accumulation in both dtypes: every output element is the sum over
// k = 0..K-1 in that order, whatever else is in the launch, so a row's result does not depend on its
// place or on its neighbours.  In float32 this is the true 32-bit product; in bfloat16 it is the
// fallback for the sizes that the tensor-core version does not take.
// Tiles of BM x 64 x 16 (BM = 64 or 16), 256 threads; any M, N, K.
#include "common.cuh"

#define GB_BN 64
#define GB_BK 16

template <typename T, int BM>
__global__ void __launch_bounds__(256)
gemm_batched_nt_kernel(const T* __restrict__ A, const T* __restrict__ W, T* __restrict__ C, int M, int N, int K,
                       int lda, int ldw, int ldc, long long a_bs, long long w_bs, long long c_bs,
                       const int* __restrict__ tile_group, long long w_gs) {
    constexpr int TM = BM / 16;
    __shared__ float As[GB_BK][BM + 4];
    __shared__ float Ws[GB_BK][GB_BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * GB_BN;
    const T* Ab = A + (size_t)blockIdx.z * a_bs;
    const T* Wb = W + (size_t)blockIdx.z * w_bs;
    T* Cb = C + (size_t)blockIdx.z * c_bs;
    if (tile_group) {
        const int g = tile_group[blockIdx.y];
        if (g < 0) return;
        Wb += (size_t)g * w_gs;
    }
    float acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GB_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            const int n = n0 + r;
            Ws[kk][r] = (n < N && k < K) ? to_f32(Wb[(size_t)n * ldw + k]) : 0.f;
            if (r < BM) {
                const int m = m0 + r;
                As[kk][r] = (m < M && k < K) ? to_f32(Ab[(size_t)m * lda + k]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GB_BK; ++kk) {
            float a[TM], b[4];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) Cb[(size_t)m * ldc + n] = from_f32<T>(acc[i][j]);
        }
    }
}

template <typename T>
static int launch_batched(const T* A, const T* W, T* C, int M, int N, int K, int lda, int ldw, int ldc,
                          long long a_bs, long long w_bs, long long c_bs, int batch, const int* tile_group,
                          long long w_gs, int bm, cudaStream_t s) {
    dim3 grid((N + GB_BN - 1) / GB_BN, (M + bm - 1) / bm, batch);
    if (grid.y > 65535 || grid.z > 65535) return VL_ERR_UNSUPPORTED;
    if (bm == 64)
        return vl_launch(gemm_batched_nt_kernel<T, 64>, grid, dim3(256), 0, s, A, W, C, M, N, K, lda, ldw, ldc,
                         a_bs, w_bs, c_bs, tile_group, w_gs);
    return vl_launch(gemm_batched_nt_kernel<T, 16>, grid, dim3(256), 0, s, A, W, C, M, N, K, lda, ldw, ldc,
                     a_bs, w_bs, c_bs, tile_group, w_gs);
}

// bm: rows per tile, 64 or 16.  With tile_group, M is the padded number of sorted rows (a multiple of bm).
extern "C" int vl_gemm_batched_nt(const void* A, const void* W, void* C, int dtype, int M, int N, int K,
                                  int lda, int ldw, int ldc, long long a_bs, long long w_bs, long long c_bs,
                                  int batch, const int* tile_group, long long w_gs, int bm, void* stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return VL_OK;
    if (K <= 0 || lda < K || ldw < K || ldc < N || (bm != 64 && bm != 16)) return VL_ERR_ARGUMENT;
    if (tile_group && M % bm) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return launch_batched<float>((const float*)A, (const float*)W, (float*)C, M, N, K, lda, ldw, ldc,
                                     a_bs, w_bs, c_bs, batch, tile_group, w_gs, bm, s);
    if (dtype == VL_BF16)
        return launch_batched<bf16>((const bf16*)A, (const bf16*)W, (bf16*)C, M, N, K, lda, ldw, ldc,
                                    a_bs, w_bs, c_bs, batch, tile_group, w_gs, bm, s);
    return VL_ERR_UNSUPPORTED;
}
