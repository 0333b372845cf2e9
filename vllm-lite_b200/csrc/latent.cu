// Latent attention: the step between the down-projections and the attention over the latent cache.
//
// A token's row of the stacked down-projection holds [a_q (q_rank values) | a_kv (kv_rank values)].
// Both halves are RMS-normed with a weight of their own (float32 arithmetic):
//     c_q = a_q  / sqrt(mean(a_q^2)  + eps) * w_q      -> cq_out [T, q_rank]   (input of the query up-projection)
//     c   = a_kv / sqrt(mean(a_kv^2) + eps) * w_kv     -> cache row `slots[t]` (the only thing kept per token)
// The cache row is `row_width` wide (kv_rank rounded up to what the attention kernels take); the tail is
// written as zeros, so that keys of any rank are plain rows of a one-head cache [pages, 1, page_size, row_width].
// One block of 128 threads per token; the order of every sum depends on the sizes alone.
// A negative slot (a padded token of a graph step) writes no cache row; a slot outside the pool sets
// VL_DEV_BAD_SLOT and is skipped.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(128)
latent_norm_write_kernel(const T* __restrict__ proj, int ld, int q_rank, int kv_rank,
                         const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                         T* __restrict__ cq_out, const int* __restrict__ slots, T* __restrict__ cache,
                         int row_width, long long num_slots, unsigned* err) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * ld;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += 128) { const float v = to_f32(row[i]); sq += v * v; }
    for (int i = threadIdx.x; i < kv_rank; i += 128) { const float v = to_f32(row[q_rank + i]); sk += v * v; }
    sq = block_sum<128>(sq, scratch);
    sk = block_sum<128>(sk, scratch);
    const float iq = 1.0f / sqrtf(sq / (float)q_rank + eps);
    const float ik = 1.0f / sqrtf(sk / (float)kv_rank + eps);
    T* cq = cq_out + (size_t)t * q_rank;
    for (int i = threadIdx.x; i < q_rank; i += 128) cq[i] = from_f32<T>(to_f32(row[i]) * iq * wq[i]);
    if (!slots) return;
    const long long slot = slots[t];
    if (slot < 0) return;
    if (slot >= num_slots) {
        if (threadIdx.x == 0) atomicOr(err, VL_DEV_BAD_SLOT);
        return;
    }
    T* dst = cache + (size_t)slot * row_width;
    for (int i = threadIdx.x; i < row_width; i += 128)
        dst[i] = i < kv_rank ? from_f32<T>(to_f32(row[q_rank + i]) * ik * wkv[i]) : from_f32<T>(0.f);
}

extern "C" int vl_latent_norm_write(const void* proj, int dtype, int ld, int T, int q_rank, int kv_rank,
                                    const float* wq, const float* wkv, float eps, void* cq_out,
                                    const int* slots, void* cache, int row_width, long long num_slots,
                                    unsigned* err, void* stream) {
    if (T <= 0) return VL_OK;
    if (q_rank <= 0 || kv_rank <= 0 || ld < q_rank + kv_rank || row_width < kv_rank) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(latent_norm_write_kernel<float>, dim3(T), dim3(128), 0, s, (const float*)proj, ld, q_rank, kv_rank,
                         wq, wkv, eps, (float*)cq_out, slots, (float*)cache, row_width, num_slots, err);
    if (dtype == VL_BF16)
        return vl_launch(latent_norm_write_kernel<bf16>, dim3(T), dim3(128), 0, s, (const bf16*)proj, ld, q_rank, kv_rank,
                         wq, wkv, eps, (bf16*)cq_out, slots, (bf16*)cache, row_width, num_slots, err);
    return VL_ERR_UNSUPPORTED;
}
