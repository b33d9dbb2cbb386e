// The residual stream with a multiplier on what is added, and norms over pieces of rows.
//
//   qnn_add_scaled_rmsnorm   resid += scale * y;  optionally out = rmsnorm(resid) * (w + offset)
//                            (a sublayer's output scaled by a constant, the add and the next
//                            pre-norm in one kernel; float32 sums, float32 stream)
//   qnn_rmsnorm_strided      RMS norm of N columns of rows that lie `ldx` apart, written to one or
//                            two places with a row pitch of their own (a piece of a stacked
//                            product's output normed into a packed buffer)
//   qnn_scale_heads          x[t, h, :] *= sigmoid(gate[t, h]): a gate per head, float32 math
//   qnn_gate_heads           the same with the gate's logits x . w_h formed in the kernel
//   qnn_small_linear_f32     x w^T with float32 sums and float32 results, for the few outputs that feed
//                            float32 math (gates, decay logits)
#include "common.cuh"

using namespace qnn;

namespace {

__global__ void add_scaled_rmsnorm_kernel(float* __restrict__ resid, const void* __restrict__ y, int y_dt, float scale,
                                          const void* __restrict__ w, int w_dt, float eps, float offset,
                                          void* __restrict__ out, int out_dt, int H) {
    __shared__ float red[32];
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = resid[base + i] + scale * load_as_f(y, y_dt, base + i);
        resid[base + i] = v;
        ss += v * v;
    }
    if (out == nullptr) return;
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)          // each thread re-reads what it wrote itself
        store_from_f(out, out_dt, base + i, resid[base + i] * inv * (load_as_f(w, w_dt, i) + offset));
}

__global__ void rmsnorm_strided_kernel(const void* __restrict__ x, int x_dt, long long ldx, const void* __restrict__ w,
                                       int w_dt, float eps, void* __restrict__ out, int out_dt, long long ldo,
                                       void* __restrict__ out2, long long ldo2, int N) {
    __shared__ float red[32];
    pdl_wait();
    const size_t xb = (size_t)blockIdx.x * ldx;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float v = load_as_f(x, x_dt, xb + i);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float v = load_as_f(x, x_dt, xb + i) * inv * load_as_f(w, w_dt, i);
        store_from_f(out, out_dt, (size_t)blockIdx.x * ldo + i, v);
        if (out2) store_from_f(out2, out_dt, (size_t)blockIdx.x * ldo2 + i, v);
    }
}

__global__ void copy_rows_kernel(const void* __restrict__ src, int dt, long long lds, void* __restrict__ dst,
                                 long long ldd, int N) {
    pdl_wait();
    for (int i = threadIdx.x; i < N; i += blockDim.x)
        store_from_f(dst, dt, (size_t)blockIdx.x * ldd + i, load_as_f(src, dt, (size_t)blockIdx.x * lds + i));
}

__global__ void scale_heads_kernel(void* __restrict__ x, int dt, const float* __restrict__ gate, int H, int D, size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = gate[i / D];                       // rows are [H][D], gates [H] per row: the same quotient
    store_from_f(x, dt, i, load_as_f(x, dt, i) * (1.f / (1.f + expf(-g))));
}

// What becomes of a sum: itself; or, with a bias and 1/tau, the decay sigmoid(sum + bias[n])^(1/tau), formed as
// exp(log_sigmoid(.) / tau) with the accurate exponential and logarithm.
__device__ __forceinline__ float finish(float d, const void* bias, int bias_dt, float inv_tau, int n) {
    if (bias == nullptr) return d;
    const float z = d + load_as_f(bias, bias_dt, n);
    return expf(inv_tau * (fminf(z, 0.f) - log1pf(expf(-fabsf(z)))));
}

// out[t, n] = x[t, :] . w[n, :], float32 sums and float32 out, for the few outputs that feed float32 math
// (gates, decay logits).  Long rows: a warp per output, lanes stride the inner size.
template <typename TX, typename TW>
__global__ void small_linear_warp_kernel(const TX* __restrict__ x, const TW* __restrict__ w, float* __restrict__ out,
                                         int N, int K, size_t total, const void* __restrict__ bias, int bias_dt,
                                         float inv_tau) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (i >= total) return;
    const size_t t = i / N;
    const TX* xr = x + t * K;
    const TW* wr = w + (i - t * N) * K;
    float d = 0.f;
    for (int k = lane; k < K; k += 32) d += to_f(xr[k]) * to_f(wr[k]);
    d = warp_sum(d);
    if (lane == 0) out[i] = finish(d, bias, bias_dt, inv_tau, (int)(i - t * N));
}
// Short rows: a thread per output; a block owns 8 rows x 32 outputs and reads their inner elements through shared
// memory (the weight rows of neighbouring outputs lie K elements apart: read directly, every load of a warp
// would touch 32 lines).
constexpr int SL_ROWS = 8, SL_OUTS = 32, SL_MAXK = 128;
template <typename TX, typename TW>
__global__ void __launch_bounds__(SL_ROWS * SL_OUTS)
small_linear_thread_kernel(const TX* __restrict__ x, const TW* __restrict__ w, float* __restrict__ out, int T, int N, int K,
                           const void* __restrict__ bias, int bias_dt, float inv_tau) {
    __shared__ float xs[SL_ROWS][SL_MAXK], ws[SL_OUTS][SL_MAXK + 1];
    pdl_wait();
    const int t0 = blockIdx.y * SL_ROWS, n0 = blockIdx.x * SL_OUTS;
    for (int idx = threadIdx.x; idx < SL_ROWS * K; idx += blockDim.x) {
        const int r = idx / K, kk = idx - r * K;
        xs[r][kk] = t0 + r < T ? to_f(x[(size_t)(t0 + r) * K + kk]) : 0.f;
    }
    for (int idx = threadIdx.x; idx < SL_OUTS * K; idx += blockDim.x) {
        const int c = idx / K, kk = idx - c * K;
        ws[c][kk] = n0 + c < N ? to_f(w[(size_t)(n0 + c) * K + kk]) : 0.f;
    }
    __syncthreads();
    const int r = threadIdx.x / SL_OUTS, c = threadIdx.x % SL_OUTS;
    if (t0 + r >= T || n0 + c >= N) return;
    float d = 0.f;
    for (int kk = 0; kk < K; ++kk) d += xs[r][kk] * ws[c][kk];
    out[(size_t)(t0 + r) * N + n0 + c] = finish(d, bias, bias_dt, inv_tau, n0 + c);
}

// o[t, h, :] *= sigmoid(x[t, :] . w[h, :]): the gate per head formed (float32) and applied in one kernel; a block per
// row, the warps share the heads.  A lane's terms and the order of their sum depend on the width only.
template <typename TX, typename TW>
__global__ void gate_heads_kernel(const TX* __restrict__ x, const TW* __restrict__ w, int W, void* __restrict__ o, int o_dt,
                                  int H, int D) {
    extern __shared__ float gate[];                       // [H]
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const TX* xr = x + (size_t)blockIdx.x * W;
    constexpr int VX = Vec16<TX>::N, VW = Vec16<TW>::N, V = VX > VW ? VX : VW;
    const bool vec = (W % V) == 0 && ((((uintptr_t)x | (uintptr_t)w) & 15) == 0);
    for (int h = warp; h < H; h += nwarp) {
        const TW* wr = w + (size_t)h * W;
        float d = 0.f;
        if (vec) {                                          // 16-byte loads where the rows allow
            for (int i = lane * V; i < W; i += 32 * V) {
                float xf[V], wf[V];
#pragma unroll
                for (int j = 0; j < V; j += VX) { Vec16<TX> v; v.load(xr + i + j); v.unpack(xf + j); }
#pragma unroll
                for (int j = 0; j < V; j += VW) { Vec16<TW> v; v.load(wr + i + j); v.unpack(wf + j); }
#pragma unroll
                for (int j = 0; j < V; ++j) d += xf[j] * wf[j];
            }
        } else {
            for (int i = lane; i < W; i += 32) d += to_f(xr[i]) * to_f(wr[i]);
        }
        d = warp_sum(d);
        if (lane == 0) gate[h] = 1.f / (1.f + expf(-d));
    }
    __syncthreads();
    const size_t base = (size_t)blockIdx.x * H * D;
    for (int i = threadIdx.x; i < H * D; i += blockDim.x)
        store_from_f(o, o_dt, base + i, load_as_f(o, o_dt, base + i) * gate[i / D]);
}

inline int row_threads(int n) { return n >= 2048 ? 512 : (n >= 512 ? 256 : 128); }

}  // namespace

QNN_API int qnn_add_scaled_rmsnorm(float* resid, const void* y, int y_dt, float scale, const void* w, int w_dt, float eps,
                                   int unit_offset, void* out, int out_dt, int T, int H, cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0 || (out != nullptr && w == nullptr)) return QNN_ERR_ARGUMENT;
    launch_pdl(add_scaled_rmsnorm_kernel, dim3(T), dim3(row_threads(H)), 0, st, resid, y, y_dt, scale, w, w_dt, eps,
               unit_offset ? 1.f : 0.f, out, out_dt, H);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_rmsnorm_strided(const void* x, int x_dt, long long ldx, const void* w, int w_dt, float eps, void* out,
                                int out_dt, long long ldo, void* out2, long long ldo2, int T, int N, cudaStream_t st) {
    if (T <= 0) return 0;
    if (N <= 0 || ldx < N || ldo < N || (out2 && ldo2 < N)) return QNN_ERR_ARGUMENT;
    launch_pdl(rmsnorm_strided_kernel, dim3(T), dim3(row_threads(N)), 0, st, x, x_dt, ldx, w, w_dt, eps, out, out_dt, ldo,
               out2, ldo2, N);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_copy_rows(const void* src, int dt, long long lds, void* dst, long long ldd, int T, int N, cudaStream_t st) {
    if (T <= 0) return 0;
    if (N <= 0 || lds < N || ldd < N) return QNN_ERR_ARGUMENT;
    launch_pdl(copy_rows_kernel, dim3(T), dim3(row_threads(N)), 0, st, src, dt, lds, dst, ldd, N);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_scale_heads(void* x, int dt, const float* gate, int T, int H, int D, cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0 || D <= 0) return QNN_ERR_ARGUMENT;
    const size_t n = (size_t)T * H * D;
    launch_pdl(scale_heads_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, dt, gate, H, D, n);
    QNN_LAUNCH_CHECK();
}

// bias (may be null) and tau: out = sigmoid(x w^T + bias)^(1/tau) instead of x w^T.
QNN_API int qnn_small_linear_f32(const void* x, int x_dt, const void* w, int w_dt, float* out, int T, int N, int K,
                                 const void* bias, int bias_dt, float tau, cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    if (K <= 0 || (bias != nullptr && !(tau > 0.f))) return QNN_ERR_ARGUMENT;
    const float inv_tau = bias != nullptr ? 1.f / tau : 0.f;
    const size_t total = (size_t)T * N;
#define QNN_SL(TX, TW)                                                                                               \
    if (K > SL_MAXK)                                                                                                 \
        launch_pdl(small_linear_warp_kernel<TX, TW>, dim3((unsigned)((total + 7) / 8)), dim3(256), 0, st,            \
                   (const TX*)x, (const TW*)w, out, N, K, total, bias, bias_dt, inv_tau);                            \
    else                                                                                                             \
        launch_pdl(small_linear_thread_kernel<TX, TW>, dim3((N + SL_OUTS - 1) / SL_OUTS, (T + SL_ROWS - 1) / SL_ROWS), \
                   dim3(SL_ROWS * SL_OUTS), 0, st, (const TX*)x, (const TW*)w, out, T, N, K, bias, bias_dt, inv_tau);
    if (x_dt == QNN_DT_BF16 && w_dt == QNN_DT_BF16) { QNN_SL(bf16, bf16) }
    else if (x_dt == QNN_DT_BF16) { QNN_SL(bf16, float) }
    else if (w_dt == QNN_DT_BF16) { QNN_SL(float, bf16) }
    else { QNN_SL(float, float) }
#undef QNN_SL
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_gate_heads(const void* x, int x_dt, const void* w, int w_dt, int W, void* o, int o_dt, int T, int H, int D,
                           cudaStream_t st) {
    if (T <= 0) return 0;
    if (W <= 0 || H <= 0 || D <= 0 || (size_t)H * sizeof(float) > 48 * 1024) return QNN_ERR_ARGUMENT;
    const dim3 grid(T), block(row_threads(H * D));
    const size_t smem = (size_t)H * sizeof(float);
#define QNN_GH(TX, TW) launch_pdl(gate_heads_kernel<TX, TW>, grid, block, smem, st, (const TX*)x, (const TW*)w, W, o, o_dt, H, D)
    if (x_dt == QNN_DT_BF16 && w_dt == QNN_DT_BF16) QNN_GH(bf16, bf16);
    else if (x_dt == QNN_DT_BF16) QNN_GH(bf16, float);
    else if (w_dt == QNN_DT_BF16) QNN_GH(float, bf16);
    else QNN_GH(float, float);
#undef QNN_GH
    QNN_LAUNCH_CHECK();
}
