// Layer norm and what sits around a residual stream whose sublayers are normed on their way OUT:
//
//   qnn_layernorm          out = (x - mean) / sqrt(var + eps) * w      var = mean of the squared deviations
//   qnn_add_layernorm      resid += layernorm(y + bias) * w;  optionally copy = resid in another element type
//                          (the next sublayer reads the stream itself, so the copy is its input)
//   qnn_mean_rmsnorm       out = (1/n) sum_b  y_b / sqrt(mean(y_b^2) + eps) * w_b      (branches side by side)
//   qnn_add_mean_layernorm the two above in one kernel: resid += layernorm(mean of the normed branches) * w
//   qnn_add_bias           y[t, :] += bias
//   qnn_activation         out = act(x) elementwise (gelu_tanh, silu, squared relu)
//
// All sums are float32; a block per row; the order of a row's sums depends on the width only.
#include "common.cuh"

using namespace qnn;

namespace {

constexpr int MAX_BRANCHES = 4;
struct Branches {
    const void* y[MAX_BRANCHES];
    const void* w[MAX_BRANCHES];
    int n;
};

__global__ void layernorm_kernel(const void* __restrict__ x, int x_dt, const void* __restrict__ w, int w_dt, float eps,
                                 void* __restrict__ out, int out_dt, int H) {
    __shared__ float red[32];
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) s += load_as_f(x, x_dt, base + i);
    const float mean = block_sum(s, red) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = load_as_f(x, x_dt, base + i) - mean;
        ss += d * d;
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        store_from_f(out, out_dt, base + i, (load_as_f(x, x_dt, base + i) - mean) * inv * load_as_f(w, w_dt, i));
}

// The row that is normed is held in shared memory as float32 (row[H]) once it has been formed.
__device__ __forceinline__ void add_layernorm_of_row(float* __restrict__ row, float* red, float* __restrict__ resid,
                                                     const void* __restrict__ w, int w_dt, float eps,
                                                     void* __restrict__ copy, int copy_dt, int H) {
    const size_t base = (size_t)blockIdx.x * H;
    float s = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) s += row[i];
    const float mean = block_sum(s, red) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = row[i] - mean;
        ss += d * d;
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = resid[base + i] + (row[i] - mean) * inv * load_as_f(w, w_dt, i);
        resid[base + i] = v;
        if (copy != nullptr) store_from_f(copy, copy_dt, base + i, v);
    }
}

__global__ void add_layernorm_kernel(float* __restrict__ resid, const void* __restrict__ y, int y_dt,
                                     const void* __restrict__ bias, int b_dt, const void* __restrict__ w, int w_dt,
                                     float eps, void* __restrict__ copy, int copy_dt, int H) {
    extern __shared__ float row[];
    __shared__ float red[32];
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        row[i] = load_as_f(y, y_dt, base + i) + (bias != nullptr ? load_as_f(bias, b_dt, i) : 0.f);
    __syncthreads();
    add_layernorm_of_row(row, red, resid, w, w_dt, eps, copy, copy_dt, H);
}

// row[i] = (1/n) sum_b y_b[i] * inv_b * w_b[i]
__device__ __forceinline__ void mean_of_normed(float* __restrict__ row, float* red, const Branches& br, int y_dt, int w_dt,
                                               float eps, int H) {
    const size_t base = (size_t)blockIdx.x * H;
    float inv[MAX_BRANCHES];
#pragma unroll
    for (int b = 0; b < MAX_BRANCHES; ++b) {
        inv[b] = 0.f;
        if (b < br.n) {
            float ss = 0.f;
            for (int i = threadIdx.x; i < H; i += blockDim.x) {
                const float v = load_as_f(br.y[b], y_dt, base + i);
                ss += v * v;
            }
            inv[b] = rsqrtf(block_sum(ss, red) / (float)H + eps);
        }
    }
    const float share = 1.f / (float)br.n;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.f;
#pragma unroll
        for (int b = 0; b < MAX_BRANCHES; ++b)
            if (b < br.n) acc += load_as_f(br.y[b], y_dt, base + i) * inv[b] * load_as_f(br.w[b], w_dt, i);
        row[i] = acc * share;
    }
}

__global__ void mean_rmsnorm_kernel(Branches br, int y_dt, int w_dt, float eps, void* __restrict__ out, int out_dt, int H) {
    extern __shared__ float row[];
    __shared__ float red[32];
    pdl_wait();
    mean_of_normed(row, red, br, y_dt, w_dt, eps, H);
    const size_t base = (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) store_from_f(out, out_dt, base + i, row[i]);   // a thread's own elements
}

__global__ void add_mean_layernorm_kernel(float* __restrict__ resid, Branches br, int y_dt, int bw_dt, float eps_branch,
                                          const void* __restrict__ w, int w_dt, float eps, void* __restrict__ copy,
                                          int copy_dt, int H) {
    extern __shared__ float row[];
    __shared__ float red[32];
    pdl_wait();
    mean_of_normed(row, red, br, y_dt, bw_dt, eps_branch, H);
    __syncthreads();
    add_layernorm_of_row(row, red, resid, w, w_dt, eps, copy, copy_dt, H);
}

__global__ void add_bias_kernel(void* __restrict__ y, int dt, const void* __restrict__ bias, int b_dt, int N, size_t total) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    store_from_f(y, dt, i, load_as_f(y, dt, i) + load_as_f(bias, b_dt, i % N));
}

__global__ void activation_kernel(const void* __restrict__ x, int dt, void* __restrict__ out, int act, size_t total) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    store_from_f(out, dt, i, activate(load_as_f(x, dt, i), act));
}

inline int row_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

inline int fill(Branches& br, const void* const* ys, const void* const* ws, int n) {
    if (n < 1 || n > MAX_BRANCHES) return QNN_ERR_UNSUPPORTED;
    br.n = n;
    for (int b = 0; b < MAX_BRANCHES; ++b) {
        br.y[b] = b < n ? ys[b] : nullptr;
        br.w[b] = b < n ? ws[b] : nullptr;
    }
    return 0;
}

}  // namespace

QNN_API int qnn_layernorm(const void* x, int x_dt, const void* w, int w_dt, float eps, void* out, int out_dt, int T, int H,
                          cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0) return QNN_ERR_ARGUMENT;
    launch_pdl(layernorm_kernel, dim3(T), dim3(row_threads(H)), 0, st, x, x_dt, w, w_dt, eps, out, out_dt, H);
    QNN_LAUNCH_CHECK();
}

// resid: [T, H] float32, in place.  bias may be null.  copy may be null; else it gets the new stream in `copy_dt`.
QNN_API int qnn_add_layernorm(float* resid, const void* y, int y_dt, const void* bias, int b_dt, const void* w, int w_dt,
                              float eps, void* copy, int copy_dt, int T, int H, cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0) return QNN_ERR_ARGUMENT;
    if ((size_t)H * sizeof(float) > 160 * 1024) return QNN_ERR_UNSUPPORTED;
    const size_t smem = (size_t)H * sizeof(float);
    static bool set = false;
    if (smem > 40 * 1024 && !set) {      // beside the static shared memory
        cudaFuncSetAttribute(add_layernorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        set = true;
    }
    launch_pdl(add_layernorm_kernel, dim3(T), dim3(row_threads(H)), smem, st, resid, y, y_dt, bias, b_dt, w, w_dt, eps, copy,
               copy_dt, H);
    QNN_LAUNCH_CHECK();
}

// ys, ws: n pointers each (host arrays): the branches' rows [T, H] of `y_dt` and their weights [H] of `w_dt`.
QNN_API int qnn_mean_rmsnorm(const void* const* ys, const void* const* ws, int n, int y_dt, int w_dt, float eps, void* out,
                             int out_dt, int T, int H, cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0) return QNN_ERR_ARGUMENT;
    if ((size_t)H * sizeof(float) > 160 * 1024) return QNN_ERR_UNSUPPORTED;
    Branches br;
    if (int rc = fill(br, ys, ws, n)) return rc;
    const size_t smem = (size_t)H * sizeof(float);
    static bool set = false;
    if (smem > 40 * 1024 && !set) {      // beside the static shared memory
        cudaFuncSetAttribute(mean_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        set = true;
    }
    launch_pdl(mean_rmsnorm_kernel, dim3(T), dim3(row_threads(H)), smem, st, br, y_dt, w_dt, eps, out, out_dt, H);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_add_mean_layernorm(float* resid, const void* const* ys, const void* const* ws, int n, int y_dt, int bw_dt,
                                   float eps_branch, const void* w, int w_dt, float eps, void* copy, int copy_dt, int T,
                                   int H, cudaStream_t st) {
    if (T <= 0) return 0;
    if (H <= 0) return QNN_ERR_ARGUMENT;
    if ((size_t)H * sizeof(float) > 160 * 1024) return QNN_ERR_UNSUPPORTED;
    Branches br;
    if (int rc = fill(br, ys, ws, n)) return rc;
    const size_t smem = (size_t)H * sizeof(float);
    static bool set = false;
    if (smem > 40 * 1024 && !set) {      // beside the static shared memory
        cudaFuncSetAttribute(add_mean_layernorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        set = true;
    }
    launch_pdl(add_mean_layernorm_kernel, dim3(T), dim3(row_threads(H)), smem, st, resid, br, y_dt, bw_dt, eps_branch, w,
               w_dt, eps, copy, copy_dt, H);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_add_bias(void* y, int dt, const void* bias, int b_dt, int T, int N, cudaStream_t st) {
    if (T <= 0) return 0;
    if (N <= 0) return QNN_ERR_ARGUMENT;
    const size_t total = (size_t)T * N;
    launch_pdl(add_bias_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, y, dt, bias, b_dt, N, total);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_activation(const void* x, int dt, void* out, int act, long long total, cudaStream_t st) {
    if (total <= 0) return 0;
    launch_pdl(activation_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, x, dt, out, act, (size_t)total);
    QNN_LAUNCH_CHECK();
}
