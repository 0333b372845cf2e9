// Mixers that carry a state of fixed size from token to token: a short causal convolution and three
// linear recurrences, each over the tokens that a step brings for every request, from the state the
// steps before left in the request's slot.  A decoded token is a portion of one token: the same kernels.
//
// A step's tokens lie flat, request b owns rows cu[b] .. cu[b+1]-1 and the state row slots[b]; a request
// without tokens (padding of a replayed step) is skipped.  Everything that enters a recurrence is float32:
// decays and their logarithms, softplus and exponentials, step sizes, gates, unit norms and the state.
//
//   vl_short_conv   out[t, c] = act(bias[c] + sum_j w[c, j] in[t - (taps-1) + j, c]), zeros before a request's
//                   first token; the last taps-1 inputs of every channel are part of the state
//   vl_ssd_scan     S <- exp(-exp(A_log) dt) S + dt B x^T,  y = S^T C + D x          (S: N x P per head, dt =
//                   softplus(raw + bias); heads share B and C in groups)
//   vl_mlstm_scan   m' = max(f + m, i);  S <- e^(f+m-m') S + e^(i-m') k v^T;  n likewise with k alone;
//                   o = S^T q / (max(|n.q|, e^(-m')) + den_eps);  i = cap tanh(a/cap), f = logsigmoid(cap tanh(b/cap))
//   vl_delta_scan   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   (g one decay per key
//                   channel, q and k unit vectors per head, q scaled)
//   vl_gate_norm    RMS norm over equal parts of a row with a weight and a gate (silu or sigmoid), the gate
//                   before or after the norm
//
// Layout of the scans: a block owns (head, request, tile of value columns); a column of the state is held in
// registers by L lanes of a warp (row r of the state by lane r mod L), so a token costs each lane N/L
// multiply-adds and one or two butterfly sums over the L lanes.  The per-token vectors of a chunk of tokens
// are staged in shared memory by the whole block.  The order of every sum depends on the sizes alone.
#include "common.cuh"

#define RC_THREADS 128
#define RC_ROWS 16            // state rows per lane, at most
#define RC_CHUNK 8            // tokens staged at a time

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float group_sum(float v, int L) {
    for (int o = L >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
static inline int lanes_for(int N) {
    int L = 1;
    while (L * RC_ROWS < N) L <<= 1;
    return L;
}

// ------------------------------------------------------------------------------------------ convolution
template <typename TP>
__global__ void __launch_bounds__(256)
short_conv_kernel(const TP* __restrict__ in, int ld, int col0, int C, const float* __restrict__ w,
                  const float* __restrict__ bias, int taps, float* __restrict__ state, long long state_stride,
                  const int* __restrict__ cu, const int* __restrict__ slots, float* __restrict__ out, int act) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    const int s0 = cu[b], n = cu[b + 1] - s0;
    if (n <= 0) return;
    const int c = blockIdx.x * 32 + threadIdx.x;
    const bool live = c < C;
    float* st = state + (long long)slots[b] * state_stride;          // [(taps-1), C]
    const int back = taps - 1;
    if (live) {
        for (int t = threadIdx.y; t < n; t += blockDim.y) {
            float acc = bias ? bias[c] : 0.f;
            for (int j = 0; j < taps; ++j) {
                const int at = t - back + j;
                const float v = at >= 0 ? to_f32(in[(size_t)(s0 + at) * ld + col0 + c]) : st[(size_t)(at + back) * C + c];
                acc += w[(size_t)c * taps + j] * v;
            }
            out[(size_t)(s0 + t) * C + c] = act ? silu_f(acc) : acc;
        }
    }
    __syncthreads();
    if (live && threadIdx.y == 0) {
        for (int j = 0; j < back; ++j) {                              // reads run ahead of the writes
            const int at = n - back + j;
            st[(size_t)j * C + c] = at >= 0 ? to_f32(in[(size_t)(s0 + at) * ld + col0 + c]) : st[(size_t)(at + back) * C + c];
        }
    }
}

extern "C" int vl_short_conv(const void* in, int dtype, int ld, int col0, int C, const float* w, const float* bias,
                             int taps, float* state, long long state_stride, const int* cu, const int* slots,
                             int B, float* out, int act, void* stream) {
    if (B <= 0 || C <= 0) return VL_OK;
    if (taps <= 0 || col0 < 0 || col0 + C > ld) return VL_ERR_ARGUMENT;
    dim3 grid((C + 31) / 32, B), block(32, 8);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(short_conv_kernel<float>, grid, block, 0, s, (const float*)in, ld, col0, C, w, bias, taps, state,
                         state_stride, cu, slots, out, act);
    if (dtype == VL_BF16)
        return vl_launch(short_conv_kernel<bf16>, grid, block, 0, s, (const bf16*)in, ld, col0, C, w, bias, taps, state,
                         state_stride, cu, slots, out, act);
    return VL_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------ state space
// xbc float32 [T, C]: x (H*P) | B (G*N) | C (G*N), the convolution's output.  raw_dt: column dt_col + h of `proj`.
// state [slots][H][N][P].  y float32 [T, H*P].
template <typename TP>
__global__ void __launch_bounds__(RC_THREADS)
ssd_scan_kernel(const float* __restrict__ xbc, int C, const TP* __restrict__ proj, int ld, int dt_col,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dw,
                float* __restrict__ state, long long state_stride, const int* __restrict__ cu,
                const int* __restrict__ slots, float* __restrict__ y, int H, int G, int N, int P, int L) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int s0 = cu[b], n = cu[b + 1] - s0;
    if (n <= 0) return;
    const int CT = RC_THREADS / L, tid = threadIdx.x;
    const int col = tid / L, l = tid % L;
    const int p0 = blockIdx.z * CT, p = p0 + col;
    const bool live = p < P;
    const int g = h / (H / G), inner = H * P;
    float* sB = sm;                               // [chunk][N]
    float* sC = sB + RC_CHUNK * N;                // [chunk][N]
    float* sX = sC + RC_CHUNK * N;                // [chunk][CT]
    float* sDt = sX + RC_CHUNK * CT;              // [chunk]
    float* sA = sDt + RC_CHUNK;                   // [chunk]
    float* S = state + (long long)slots[b] * state_stride + (size_t)h * N * P;
    float s[RC_ROWS];
#pragma unroll
    for (int i = 0; i < RC_ROWS; ++i) {
        const int r = l + L * i;
        s[i] = (live && r < N) ? S[(size_t)r * P + p] : 0.f;
    }
    const float rate = expf(A_log[h]), skip = Dw[h], bias = dt_bias[h];
    for (int t0 = 0; t0 < n; t0 += RC_CHUNK) {
        const int m = min(RC_CHUNK, n - t0);
        __syncthreads();
        for (int i = tid; i < m * N; i += RC_THREADS) {
            const int k = i / N, r = i - k * N;
            const float* row = xbc + (size_t)(s0 + t0 + k) * C + inner + (size_t)g * N + r;
            sB[k * N + r] = row[0];
            sC[k * N + r] = row[(size_t)G * N];
        }
        for (int i = tid; i < m * CT; i += RC_THREADS) {
            const int k = i / CT, c = i - k * CT;
            sX[i] = p0 + c < P ? xbc[(size_t)(s0 + t0 + k) * C + (size_t)h * P + p0 + c] : 0.f;
        }
        if (tid < m) {
            const float dt = softplus_f(to_f32(proj[(size_t)(s0 + t0 + tid) * ld + dt_col + h]) + bias);
            sDt[tid] = dt;
            sA[tid] = expf(-rate * dt);
        }
        __syncthreads();
        for (int k = 0; k < m; ++k) {
            const float a = sA[k], xv = sX[k * CT + col], dx = sDt[k] * xv;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < RC_ROWS; ++i) {
                const int r = l + L * i;
                if (r < N) {
                    s[i] = a * s[i] + sB[k * N + r] * dx;
                    acc += s[i] * sC[k * N + r];
                }
            }
            acc = group_sum(acc, L);
            if (live && l == 0) y[(size_t)(s0 + t0 + k) * inner + (size_t)h * P + p] = acc + skip * xv;
        }
    }
#pragma unroll
    for (int i = 0; i < RC_ROWS; ++i) {
        const int r = l + L * i;
        if (live && r < N) S[(size_t)r * P + p] = s[i];
    }
}

extern "C" int vl_ssd_scan(const float* xbc, int C, const void* proj, int dtype, int ld, int dt_col, const float* dt_bias,
                           const float* A_log, const float* Dw, float* state, long long state_stride, const int* cu,
                           const int* slots, int B, float* y, int H, int G, int N, int P, void* stream) {
    if (B <= 0) return VL_OK;
    if (H <= 0 || G <= 0 || H % G || N <= 0 || P <= 0 || C != H * P + 2 * G * N) return VL_ERR_ARGUMENT;
    const int L = lanes_for(N);
    if (L > 32) return VL_ERR_UNSUPPORTED;
    const int CT = RC_THREADS / L;
    dim3 grid(H, B, (P + CT - 1) / CT);
    const size_t smem = sizeof(float) * (size_t)(RC_CHUNK * (2 * N + CT + 2));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(ssd_scan_kernel<float>, grid, dim3(RC_THREADS), smem, s, xbc, C, (const float*)proj, ld, dt_col,
                         dt_bias, A_log, Dw, state, state_stride, cu, slots, y, H, G, N, P, L);
    if (dtype == VL_BF16)
        return vl_launch(ssd_scan_kernel<bf16>, grid, dim3(RC_THREADS), smem, s, xbc, C, (const bf16*)proj, ld, dt_col,
                         dt_bias, A_log, Dw, state, state_stride, cu, slots, y, H, G, N, P, L);
    return VL_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------ matrix memory
// proj [T, ld]: q at q_col (H*D), k at k_col (H*D), v at v_col (H*P), raw gates at i_col, f_col (H each).
// state per slot: S [H][D][P], then n [H][Z][D], then m [H][Z], Z = the number of column tiles of a head
// (vl_mlstm_state_floats): blocks of one head run at different times, so each keeps its own n and m.  o float32 [T, H*P].
template <typename TP>
__global__ void __launch_bounds__(RC_THREADS)
mlstm_scan_kernel(const TP* __restrict__ proj, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                  const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale, float den_eps,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ cu,
                  const int* __restrict__ slots, float* __restrict__ o, int H, int D, int P, int L) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int s0 = cu[b], n = cu[b + 1] - s0;
    if (n <= 0) return;
    const int CT = RC_THREADS / L, tid = threadIdx.x;
    const int col = tid / L, l = tid % L;
    const int p0 = blockIdx.z * CT, p = p0 + col;
    const bool live = p < P;
    float* sQ = sm;                               // [chunk][D]
    float* sK = sQ + RC_CHUNK * D;                // [chunk][D]
    float* sV = sK + RC_CHUNK * D;                // [chunk][CT]
    float* sKeep = sV + RC_CHUNK * CT;            // [chunk]
    float* sPut = sKeep + RC_CHUNK;               // [chunk]
    float* sFloor = sPut + RC_CHUNK;              // [chunk]
    float* sM = sFloor + RC_CHUNK;                // [1]
    float* base = state + (long long)slots[b] * state_stride;
    float* S = base + (size_t)h * D * P;
    const int Z = gridDim.z, z = blockIdx.z;          // every tile of columns keeps n and m for itself
    float* nv = base + (size_t)H * D * P + ((size_t)h * Z + z) * D;
    float* mv = base + (size_t)H * D * P + (size_t)H * Z * D + (size_t)h * Z + z;
    float s[RC_ROWS], nr[RC_ROWS];
#pragma unroll
    for (int i = 0; i < RC_ROWS; ++i) {
        const int r = l + L * i;
        s[i] = (live && r < D) ? S[(size_t)r * P + p] : 0.f;
        nr[i] = r < D ? nv[r] : 0.f;
    }
    if (tid == 0) sM[0] = mv[0];
    for (int t0 = 0; t0 < n; t0 += RC_CHUNK) {
        const int m = min(RC_CHUNK, n - t0);
        __syncthreads();
        for (int i = tid; i < m * D; i += RC_THREADS) {
            const int k = i / D, r = i - k * D;
            const TP* row = proj + (size_t)(s0 + t0 + k) * ld + (size_t)h * D + r;
            sQ[i] = to_f32(row[q_col]) * q_scale;
            sK[i] = to_f32(row[k_col]);
        }
        for (int i = tid; i < m * CT; i += RC_THREADS) {
            const int k = i / CT, c = i - k * CT;
            sV[i] = p0 + c < P ? to_f32(proj[(size_t)(s0 + t0 + k) * ld + v_col + (size_t)h * P + p0 + c]) : 0.f;
        }
        if (tid == 0) {
            float mx = sM[0];
            for (int k = 0; k < m; ++k) {
                const TP* row = proj + (size_t)(s0 + t0 + k) * ld + h;
                const float ig = cap * tanhf((to_f32(row[i_col]) + i_bias[h]) / cap);
                const float fa = cap * tanhf((to_f32(row[f_col]) + f_bias[h]) / cap);
                const float fg = fminf(fa, 0.f) - log1pf(expf(-fabsf(fa)));          // log sigmoid
                const float nm = fmaxf(fg + mx, ig);
                sKeep[k] = expf(fg + mx - nm);
                sPut[k] = expf(ig - nm);
                sFloor[k] = expf(-nm);
                mx = nm;
            }
            sM[0] = mx;
        }
        __syncthreads();
        for (int k = 0; k < m; ++k) {
            const float keep = sKeep[k], pv = sPut[k] * sV[k * CT + col], put = sPut[k];
            float acc = 0.f, den = 0.f;
#pragma unroll
            for (int i = 0; i < RC_ROWS; ++i) {
                const int r = l + L * i;
                if (r < D) {
                    const float kv = sK[k * D + r], qv = sQ[k * D + r];
                    s[i] = keep * s[i] + kv * pv;
                    nr[i] = keep * nr[i] + put * kv;
                    acc += s[i] * qv;
                    den += nr[i] * qv;
                }
            }
            acc = group_sum(acc, L);
            den = group_sum(den, L);
            if (live && l == 0)
                o[(size_t)(s0 + t0 + k) * H * P + (size_t)h * P + p] = acc / (fmaxf(fabsf(den), sFloor[k]) + den_eps);
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RC_ROWS; ++i) {
        const int r = l + L * i;
        if (live && r < D) S[(size_t)r * P + p] = s[i];
        if (col == 0 && r < D) nv[r] = nr[i];
    }
    if (tid == 0) mv[0] = sM[0];
}

extern "C" long long vl_mlstm_state_floats(int H, int D, int P) {
    const int L = lanes_for(D);
    if (L > 32 || H <= 0 || D <= 0 || P <= 0) return -1;
    const int CT = RC_THREADS / L, Z = (P + CT - 1) / CT;
    return (long long)H * D * P + (long long)H * Z * D + (long long)H * Z;
}

extern "C" int vl_mlstm_scan(const void* proj, int dtype, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                             const float* i_bias, const float* f_bias, float cap, float q_scale, float den_eps, float* state,
                             long long state_stride, const int* cu, const int* slots, int B, float* o, int H, int D, int P,
                             void* stream) {
    if (B <= 0) return VL_OK;
    if (H <= 0 || D <= 0 || P <= 0 || !(cap > 0.f)) return VL_ERR_ARGUMENT;
    const int L = lanes_for(D);
    if (L > 32) return VL_ERR_UNSUPPORTED;
    const int CT = RC_THREADS / L;
    dim3 grid(H, B, (P + CT - 1) / CT);
    const size_t smem = sizeof(float) * (size_t)(RC_CHUNK * (2 * D + CT + 3) + 1);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(mlstm_scan_kernel<float>, grid, dim3(RC_THREADS), smem, s, (const float*)proj, ld, q_col, k_col, v_col,
                         i_col, f_col, i_bias, f_bias, cap, q_scale, den_eps, state, state_stride, cu, slots, o, H, D, P, L);
    if (dtype == VL_BF16)
        return vl_launch(mlstm_scan_kernel<bf16>, grid, dim3(RC_THREADS), smem, s, (const bf16*)proj, ld, q_col, k_col, v_col,
                         i_col, f_col, i_bias, f_bias, cap, q_scale, den_eps, state, state_stride, cu, slots, o, H, D, P, L);
    return VL_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------ delta rule
// qkv float32 [T, C]: q (G*D) | k (G*D) | v (H*P), the convolutions' output.  raw decay: columns dcol .. of `decay` (rows dld wide),
// raw beta: column beta_col + h of `proj`.  state [slots][H][D][P].  o float32 [T, H*P].
template <typename TP>
__global__ void __launch_bounds__(RC_THREADS)
delta_scan_kernel(const float* __restrict__ qkv, int C, const TP* __restrict__ decay, int dld, int dcol,
                  const float* __restrict__ dt_bias,
                  const float* __restrict__ A_log, const TP* __restrict__ proj, int ld, int beta_col, float q_scale,
                  float unit_eps, float* __restrict__ state, long long state_stride, const int* __restrict__ cu,
                  const int* __restrict__ slots, float* __restrict__ o, int H, int G, int D, int P, int L) {
    extern __shared__ float sm[];
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int s0 = cu[b], n = cu[b + 1] - s0;
    if (n <= 0) return;
    const int CT = RC_THREADS / L, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col = tid / L, l = tid % L;
    const int p0 = blockIdx.z * CT, p = p0 + col;
    const bool live = p < P;
    const int g = h / (H / G);
    float* sQ = sm;                               // [chunk][D]
    float* sK = sQ + RC_CHUNK * D;                // [chunk][D]
    float* sG = sK + RC_CHUNK * D;                // [chunk][D]
    float* sV = sG + RC_CHUNK * D;                // [chunk][CT]
    float* sBeta = sV + RC_CHUNK * CT;            // [chunk]
    float* S = state + (long long)slots[b] * state_stride + (size_t)h * D * P;
    float s[RC_ROWS];
#pragma unroll
    for (int i = 0; i < RC_ROWS; ++i) {
        const int r = l + L * i;
        s[i] = (live && r < D) ? S[(size_t)r * P + p] : 0.f;
    }
    const float rate = expf(A_log[h]);
    for (int t0 = 0; t0 < n; t0 += RC_CHUNK) {
        const int m = min(RC_CHUNK, n - t0);
        __syncthreads();
        for (int k = warp; k < m; k += RC_THREADS / 32) {             // a warp per token: unit vectors and decays
            const size_t t = (size_t)(s0 + t0 + k);
            const float* qrow = qkv + t * C + (size_t)g * D;
            const float* krow = qrow + (size_t)G * D;
            float qq = 0.f, kk = 0.f;
            for (int r = lane; r < D; r += 32) { qq += qrow[r] * qrow[r]; kk += krow[r] * krow[r]; }
            qq = warp_sum(qq);
            kk = warp_sum(kk);
            const float qn = q_scale / sqrtf(qq + unit_eps), kn = 1.f / sqrtf(kk + unit_eps);
            for (int r = lane; r < D; r += 32) {
                sQ[k * D + r] = qrow[r] * qn;
                sK[k * D + r] = krow[r] * kn;
                const float step = softplus_f(to_f32(decay[t * (size_t)dld + dcol + (size_t)h * D + r]) + dt_bias[(size_t)h * D + r]);
                sG[k * D + r] = expf(-rate * step);
            }
            if (lane == 0) sBeta[k] = sigmoid_f(to_f32(proj[t * ld + beta_col + h]));
        }
        for (int i = tid; i < m * CT; i += RC_THREADS) {
            const int k = i / CT, c = i - k * CT;
            sV[i] = p0 + c < P ? qkv[(size_t)(s0 + t0 + k) * C + (size_t)2 * G * D + (size_t)h * P + p0 + c] : 0.f;
        }
        __syncthreads();
        for (int k = 0; k < m; ++k) {
            float back = 0.f;
#pragma unroll
            for (int i = 0; i < RC_ROWS; ++i) {
                const int r = l + L * i;
                if (r < D) {
                    s[i] *= sG[k * D + r];
                    back += s[i] * sK[k * D + r];
                }
            }
            back = group_sum(back, L);
            const float u = sBeta[k] * (sV[k * CT + col] - back);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < RC_ROWS; ++i) {
                const int r = l + L * i;
                if (r < D) {
                    s[i] += sK[k * D + r] * u;
                    acc += s[i] * sQ[k * D + r];
                }
            }
            acc = group_sum(acc, L);
            if (live && l == 0) o[(size_t)(s0 + t0 + k) * H * P + (size_t)h * P + p] = acc;
        }
    }
#pragma unroll
    for (int i = 0; i < RC_ROWS; ++i) {
        const int r = l + L * i;
        if (live && r < D) S[(size_t)r * P + p] = s[i];
    }
}

extern "C" int vl_delta_scan(const float* qkv, int C, const void* decay, int dld, int dcol, const float* dt_bias, const float* A_log,
                             const void* proj, int dtype, int ld, int beta_col, float q_scale, float unit_eps, float* state,
                             long long state_stride, const int* cu, const int* slots, int B, float* o, int H, int G, int D,
                             int P, void* stream) {
    if (B <= 0) return VL_OK;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || P <= 0 || C != 2 * G * D + H * P) return VL_ERR_ARGUMENT;
    const int L = lanes_for(D);
    if (L > 32) return VL_ERR_UNSUPPORTED;
    const int CT = RC_THREADS / L;
    dim3 grid(H, B, (P + CT - 1) / CT);
    const size_t smem = sizeof(float) * (size_t)(RC_CHUNK * (3 * D + CT + 1));
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(delta_scan_kernel<float>, grid, dim3(RC_THREADS), smem, s, qkv, C, (const float*)decay, dld, dcol, dt_bias, A_log,
                         (const float*)proj, ld, beta_col, q_scale, unit_eps, state, state_stride, cu, slots, o, H, G, D, P, L);
    if (dtype == VL_BF16)
        return vl_launch(delta_scan_kernel<bf16>, grid, dim3(RC_THREADS), smem, s, qkv, C, (const bf16*)decay, dld, dcol, dt_bias, A_log,
                         (const bf16*)proj, ld, beta_col, q_scale, unit_eps, state, state_stride, cu, slots, o, H, G, D, P, L);
    return VL_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------------------------------ gate and norm
// y float32 [T, W] in parts of `part` columns; a warp per (token, part).  gate (TP, column gate_col of rows `ld` wide):
// kind 1 silu, 2 sigmoid, 0 none.  gate_first: out = rms(y * gate) * w, else out = rms(y) * w * gate.
// w float32 [wlen], indexed by column modulo wlen (wlen = W: one weight per column; wlen = part: shared by the parts).
#define RC_GATE_SILU 1
#define RC_GATE_SIGMOID 2
template <typename TP>
__global__ void __launch_bounds__(128)
gate_norm_kernel(const float* __restrict__ y, const TP* __restrict__ gate, int ld, int gate_col, int gate_kind, int gate_first,
                 const float* __restrict__ w, int wlen, float eps, TP* __restrict__ out, int W, int part, size_t groups) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t gi = (size_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (gi >= groups) return;
    const int lane = threadIdx.x & 31;
    const int per_row = W / part;
    const size_t t = gi / per_row;
    const int c0 = (int)(gi - t * per_row) * part;
    const float* row = y + t * W + c0;
    const TP* grow = gate ? gate + t * ld + gate_col + c0 : nullptr;
    float ss = 0.f;
    for (int c = lane; c < part; c += 32) {
        float v = row[c];
        if (gate_first && grow) {
            const float gv = to_f32(grow[c]);
            v *= gate_kind == RC_GATE_SILU ? silu_f(gv) : sigmoid_f(gv);
        }
        ss += v * v;
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / part + eps);
    for (int c = lane; c < part; c += 32) {
        float v = row[c];
        float gv = 1.f;
        if (grow) {
            gv = to_f32(grow[c]);
            gv = gate_kind == RC_GATE_SILU ? silu_f(gv) : sigmoid_f(gv);
        }
        if (gate_first) v = v * gv * inv * w[(c0 + c) % wlen];
        else v = v * inv * w[(c0 + c) % wlen] * gv;
        out[t * W + c0 + c] = from_f32<TP>(v);
    }
}

extern "C" int vl_gate_norm(const float* y, const void* gate, int dtype, int ld, int gate_col, int gate_kind, int gate_first,
                            const float* w, int wlen, float eps, void* out, int T, int W, int part, void* stream) {
    if (T <= 0 || W <= 0) return VL_OK;
    if (part <= 0 || W % part || wlen <= 0 || (gate && (gate_kind < 1 || gate_kind > 2))) return VL_ERR_ARGUMENT;
    const size_t groups = (size_t)T * (W / part);
    const unsigned blocks = (unsigned)((groups + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == VL_F32)
        return vl_launch(gate_norm_kernel<float>, dim3(blocks), dim3(128), 0, s, y, (const float*)gate, ld, gate_col, gate_kind,
                         gate_first, w, wlen, eps, (float*)out, W, part, groups);
    if (dtype == VL_BF16)
        return vl_launch(gate_norm_kernel<bf16>, dim3(blocks), dim3(128), 0, s, y, (const bf16*)gate, ld, gate_col, gate_kind,
                         gate_first, w, wlen, eps, (bf16*)out, W, part, groups);
    return VL_ERR_UNSUPPORTED;
}
