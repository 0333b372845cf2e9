// Several residual streams per token (hyper-connections) and the element-wise tanh norm.
//
// A model with S streams keeps x_1 .. x_S per token, float32 [T, S, H].  Around a sub-layer f with the
// learned numbers in[S], out[S] and mix[S, S] (indexed [from, to]):
//     u = sum_s in[s] x_s          h = norm(u)          y = f(h)
//     x_t <- sum_s mix[s, t] x_s + out[t] y             (all t at once, from the old streams)
// vl_hc_step does, for every (token, column), any of these in ONE pass over the streams, in this order:
//   spread   the streams start as S copies of a single stream x (the embedding's output)
//   update   the write-back of the sub-layer that just ran (y given)
//   read     u for the NEXT sub-layer and its norm (in given): h = tanh(alpha u) w + b, or u itself
//   total    sum_s x_s (what a model's last norm reads)
// so a layer costs one pass per sub-layer.  Sums run over s in ascending order, in float32.
//
// vl_dyt_rows is the same norm on rows of a single stream:  out[r] = tanh(alpha x[row r]) w + b
// (no mean, no variance; alpha a learned scalar), with an optional pending delta added into x first.
#include "common.cuh"

#define HC_MAX_STREAMS 16

// SMAX: the most streams this instance holds in registers; VEC: neighbouring columns per thread (4: 16-byte accesses
// of the float32 streams).  The learned numbers sit in shared memory, read by all threads alike.
template <typename TY, int SMAX, int VEC>
__global__ void __launch_bounds__(256)
hc_step_kernel(float* __restrict__ streams, const float* __restrict__ single, const TY* __restrict__ y,
               const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ inw,
               const float* __restrict__ alpha, const float* __restrict__ w, const float* __restrict__ b,
               TY* __restrict__ h, float* __restrict__ total, int S, int H, size_t n) {
    __shared__ float s_mix[SMAX * SMAX], s_out[SMAX], s_in[SMAX];
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) s_mix[i] = mix ? mix[i] : 0.f;
    if (threadIdx.x < S) {
        s_out[threadIdx.x] = outw ? outw[threadIdx.x] : 0.f;
        s_in[threadIdx.x] = inw ? inw[threadIdx.x] : 0.f;
    }
    const float al = alpha ? alpha[0] : 0.f;
    pdl_launch_dependents();
    pdl_wait();
    __syncthreads();
    const size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;       // H is a multiple of VEC
    if (idx >= n) return;
    const size_t t = idx / H;
    const int c = (int)(idx - t * H);
    float* xs = streams + t * (size_t)S * H + c;
    float old[SMAX][VEC], now[SMAX][VEC];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
        if (s < S) {
            const float* src = single ? single + idx : xs + (size_t)s * H;
            if (VEC == 4) {
                const float4 v = *reinterpret_cast<const float4*>(src);
                old[s][0] = v.x; old[s][1 % VEC] = v.y; old[s][2 % VEC] = v.z; old[s][3 % VEC] = v.w;
            } else {
                old[s][0] = src[0];
            }
        }
    }
    if (y) {
        float yv[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) yv[e] = to_f32(y[idx + e]);
#pragma unroll
        for (int d = 0; d < SMAX; ++d) {
            if (d < S) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    float acc = 0.f;
#pragma unroll
                    for (int s = 0; s < SMAX; ++s)
                        if (s < S) acc += s_mix[s * S + d] * old[s][e];
                    now[d][e] = acc + s_out[d] * yv[e];
                }
            }
        }
    } else {
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                if (s < S) now[s][e] = old[s][e];
    }
    if (y || single) {
#pragma unroll
        for (int s = 0; s < SMAX; ++s) {
            if (s < S) {
                if (VEC == 4)
                    *reinterpret_cast<float4*>(xs + (size_t)s * H) = make_float4(now[s][0], now[s][1 % VEC], now[s][2 % VEC], now[s][3 % VEC]);
                else
                    xs[(size_t)s * H] = now[s][0];
            }
        }
    }
    if (inw) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < SMAX; ++s)
                if (s < S) u += s_in[s] * now[s][e];
            if (w) u = tanhf(al * u) * w[c + e] + b[c + e];
            h[idx + e] = from_f32<TY>(u);
        }
    }
    if (total) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < SMAX; ++s)
                if (s < S) u += now[s][e];
            total[idx + e] = u;
        }
    }
}

template <typename TY>
static int hc_launch(float* streams, const float* single, const TY* y, const float* mix, const float* outw, const float* inw,
                     const float* alpha, const float* w, const float* b, TY* h, float* total, int T, int S, int H,
                     cudaStream_t s) {
    const size_t n = (size_t)T * H;
    const bool vec = H % 4 == 0 && S <= 8 && (((uintptr_t)streams | (uintptr_t)single) & 15) == 0;
    const size_t threads = vec ? n / 4 : n;
    const dim3 grid((unsigned)((threads + 255) / 256)), block(256);
#define HC_GO(SMAX, VEC) return vl_launch(hc_step_kernel<TY, SMAX, VEC>, grid, block, 0, s, streams, single, y, mix, outw, inw, \
                                          alpha, w, b, h, total, S, H, n)
    if (vec && S <= 4) HC_GO(4, 4);
    if (vec) HC_GO(8, 4);
    if (S <= 4) HC_GO(4, 1);
    if (S <= 8) HC_GO(8, 1);
    HC_GO(HC_MAX_STREAMS, 1);
#undef HC_GO
}

extern "C" int vl_hc_step(float* streams, const float* single, const void* y, int dtype, const float* mix,
                          const float* outw, const float* inw, const float* alpha, const float* w, const float* b,
                          void* h, float* total, int T, int S, int H, void* stream) {
    if (T <= 0 || H <= 0) return VL_OK;
    if (S <= 0 || S > HC_MAX_STREAMS) return VL_ERR_UNSUPPORTED;
    if ((y && (!mix || !outw)) || (inw && !h) || (w && (!alpha || !b))) return VL_ERR_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return hc_launch<float>(streams, single, (const float*)y, mix, outw, inw, alpha, w, b, (float*)h, total, T, S, H, s);
    if (dtype == VL_BF16)
        return hc_launch<bf16>(streams, single, (const bf16*)y, mix, outw, inw, alpha, w, b, (bf16*)h, total, T, S, H, s);
    return VL_ERR_UNSUPPORTED;
}

template <typename TO>
__global__ void __launch_bounds__(256)
dyt_rows_kernel(float* __restrict__ x, const TO* __restrict__ delta, const int* __restrict__ rows,
                const float* __restrict__ alpha, const float* __restrict__ w, const float* __restrict__ b,
                TO* __restrict__ out, int H, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const size_t r = idx / H;
    const int c = (int)(idx - r * H);
    const size_t src = (rows ? (size_t)rows[r] : r) * H + c;
    float v = x[src];
    if (delta) {
        v += to_f32(delta[src]);
        if (!rows) x[src] = v;
    }
    out[idx] = from_f32<TO>(tanhf(alpha[0] * v) * w[c] + b[c]);
}

extern "C" int vl_dyt_rows(float* x, const void* delta, const int* rows, const float* alpha, const float* w,
                           const float* b, void* out, int dtype, int R, int H, void* stream) {
    if (R <= 0 || H <= 0) return VL_OK;
    const size_t n = (size_t)R * H;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(dyt_rows_kernel<float>, dim3(blocks), dim3(256), 0, s, x, (const float*)delta, rows, alpha, w, b,
                         (float*)out, H, n);
    if (dtype == VL_BF16)
        return vl_launch(dyt_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, s, x, (const bf16*)delta, rows, alpha, w, b,
                         (bf16*)out, H, n);
    return VL_ERR_UNSUPPORTED;
}
