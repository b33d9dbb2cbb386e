// Gated linear attention: a matrix state per (sequence, head) that decays per key channel.
//
//   S_t = diag(a_t) S_{t-1} + k_t v_t^T          S: [dim, vdim], float32, kept per cache slot
//   o_t = S_t^T (q_t * q_scale)
//   a_t = sigmoid(z_t + bias)^(1/tau) = exp(log_sigmoid(z_t + bias) / tau)       (float32)
//
//   qnn_gla_scan        walks the rows of every sequence of a step in order, from the slot's state and back
//                       into it: whole prompts, portions and single tokens are the same launch
//   qnn_gla_norm_gate   per head: RMS norm of o over vdim with a weight shared by the heads, times silu(g)
//
// The scan: a block owns 32 value columns of one (sequence, head).  Four lanes share a column, each with every
// fourth key channel of the state in registers; q, k, the decay and v of 16 rows at a time are staged in
// shared memory (the decay's exponential is formed once there, not once per column).  The order of the sums
// depends on dim only, so a row gives the same numbers in any batch and any cutting of its sequence.
#include "common.cuh"

using namespace qnn;

namespace {

constexpr int GLA_COLS = 32;      // value columns of a block
constexpr int GLA_SHARE = 4;      // lanes that share a column
constexpr int GLA_ROWS = 16;      // rows staged at a time
constexpr int GLA_THREADS = GLA_COLS * GLA_SHARE;

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T, int RPT>
__global__ void __launch_bounds__(GLA_THREADS)
gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                const float* __restrict__ z, long long ldz, const void* __restrict__ bias, int bias_dt, float inv_tau,
                float q_scale, const int* __restrict__ seq_row0, const int* __restrict__ seq_len,
                const int* __restrict__ slots, float* __restrict__ state, float* __restrict__ out, long long ldo,
                int H, int dim, int vdim) {
    constexpr int DIMP = RPT * GLA_SHARE;                    // key channels with padding
    extern __shared__ float sm[];
    float* sq = sm;                                          // [GLA_ROWS][DIMP]
    float* sk = sq + GLA_ROWS * DIMP;
    float* sa = sk + GLA_ROWS * DIMP;
    float* sv = sa + GLA_ROWS * DIMP;                        // [GLA_ROWS][GLA_COLS]
    const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * GLA_COLS;
    pdl_wait();
    const int slot = slots[b];
    const int row0 = seq_row0 ? seq_row0[b] : b;
    const int n = seq_len ? seq_len[b] : 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int part = lane & (GLA_SHARE - 1), cl = warp * (32 / GLA_SHARE) + (lane >> 2);
    const int col = c0 + cl;
    const bool live = slot >= 0 && col < vdim;
    float S[RPT];
    float* my_state = state + (((size_t)(slot < 0 ? 0 : slot) * H + h) * dim) * vdim + col;
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
        const int i = r * GLA_SHARE + part;
        S[r] = (live && i < dim) ? my_state[(size_t)i * vdim] : 0.f;
    }
    for (int t0 = 0; t0 < n; t0 += GLA_ROWS) {
        const int nt = min(GLA_ROWS, n - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * DIMP; idx += GLA_THREADS) {
            const int tt = idx / DIMP, i = idx - tt * DIMP;
            float qv = 0.f, kv = 0.f, av = 1.f;
            if (i < dim) {
                const size_t row = (size_t)(row0 + t0 + tt);
                qv = to_f(q[row * ld + h * dim + i]) * q_scale;
                kv = to_f(k[row * ld + h * dim + i]);
                av = expf(inv_tau * log_sigmoid(z[row * ldz + h * dim + i] + load_as_f(bias, bias_dt, h * dim + i)));
            }
            sq[idx] = qv;
            sk[idx] = kv;
            sa[idx] = av;
        }
        for (int idx = threadIdx.x; idx < nt * GLA_COLS; idx += GLA_THREADS) {
            const int tt = idx / GLA_COLS, c = idx - tt * GLA_COLS;
            sv[idx] = (c0 + c < vdim) ? to_f(v[(size_t)(row0 + t0 + tt) * ld + h * vdim + c0 + c]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = sv[tt * GLA_COLS + cl];
            const float* aq = sq + tt * DIMP + part;
            const float* ak = sk + tt * DIMP + part;
            const float* aa = sa + tt * DIMP + part;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < RPT; ++r) {
                S[r] = aa[r * GLA_SHARE] * S[r] + ak[r * GLA_SHARE] * vj;
                acc += S[r] * aq[r * GLA_SHARE];
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (part == 0 && col < vdim) out[(size_t)(row0 + t0 + tt) * ldo + h * vdim + col] = slot >= 0 ? acc : 0.f;
        }
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
            const int i = r * GLA_SHARE + part;
            if (i < dim) my_state[(size_t)i * vdim] = S[r];
        }
    }
}

// a warp per (row, head)
template <typename T>
__global__ void gla_norm_gate_kernel(const float* __restrict__ o, long long ldo, const void* __restrict__ w, int w_dt,
                                     float eps, const T* __restrict__ g, long long ldg, T* __restrict__ out,
                                     long long ld_out, int rows, int H, int vdim) {
    pdl_wait();
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= rows * H) return;
    const int t = unit / H, h = unit - t * H;
    const float* orow = o + (size_t)t * ldo + h * vdim;
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) ss += orow[j] * orow[j];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)vdim + eps);
    for (int j = lane; j < vdim; j += 32) {
        const float gv = to_f(g[(size_t)t * ldg + h * vdim + j]);
        out[(size_t)t * ld_out + h * vdim + j] = from_f<T>(orow[j] * inv * load_as_f(w, w_dt, j) * silu(gv));
    }
}

template <typename T>
int scan_launch(const void* q, const void* k, const void* v, long long ld, const float* z, long long ldz, const void* bias,
                int bias_dt, float inv_tau, float q_scale, const int* seq_row0, const int* seq_len, const int* slots,
                float* state, float* out, long long ldo, int B, int H, int dim, int vdim, cudaStream_t st) {
    const dim3 grid((vdim + GLA_COLS - 1) / GLA_COLS, H, B);
    const int rpt = (dim + GLA_SHARE - 1) / GLA_SHARE;
#define QNN_GLA(RPTV)                                                                                                \
    {                                                                                                                \
        const size_t smem = (size_t)(3 * GLA_ROWS * RPTV * GLA_SHARE + GLA_ROWS * GLA_COLS) * sizeof(float);         \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(gla_scan_kernel<T, RPTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        launch_pdl(gla_scan_kernel<T, RPTV>, grid, dim3(GLA_THREADS), smem, st, (const T*)q, (const T*)k,           \
                   (const T*)v, ld, z, ldz, bias, bias_dt, inv_tau, q_scale, seq_row0, seq_len, slots, state, out,   \
                   ldo, H, dim, vdim);                                                                               \
    }
    if (rpt <= 4) QNN_GLA(4)
    else if (rpt <= 8) QNN_GLA(8)
    else if (rpt <= 16) QNN_GLA(16)
    else if (rpt <= 32) QNN_GLA(32)
    else if (rpt <= 64) QNN_GLA(64)
    else return QNN_ERR_UNSUPPORTED;
#undef QNN_GLA
    QNN_LAUNCH_CHECK();
}

}  // namespace

// q, k: [rows, H*dim] and v: [rows, H*vdim] of `dtype`, one row pitch `ld` (pieces of one stacked product);
// z: decay logits [rows, H*dim] float32; bias: [H*dim]; seq_row0 / seq_len: first row and row count of each
// of the B sequences (both null: sequence b is row b alone); slots: the state slot of each sequence, negative
// for a row of no sequence (its output is zero, no state is touched); state: [slots, H, dim, vdim] float32;
// out: [rows, H*vdim] float32.  dim up to 256.
QNN_API int qnn_gla_scan(const void* q, const void* k, const void* v, long long ld, int dtype, const float* z,
                         long long ldz, const void* bias, int bias_dt, float tau, float q_scale, const int* seq_row0,
                         const int* seq_len, const int* slots, float* state, float* out, long long ldo, int B, int H,
                         int dim, int vdim, cudaStream_t st) {
    if (B <= 0) return 0;
    if (H <= 0 || dim <= 0 || vdim <= 0 || !(tau > 0.f) || H > 65535 || B > 65535) return QNN_ERR_ARGUMENT;
    if ((seq_row0 == nullptr) != (seq_len == nullptr)) return QNN_ERR_ARGUMENT;
    if (dtype == QNN_DT_BF16)
        return scan_launch<bf16>(q, k, v, ld, z, ldz, bias, bias_dt, 1.f / tau, q_scale, seq_row0, seq_len, slots, state,
                                 out, ldo, B, H, dim, vdim, st);
    return scan_launch<float>(q, k, v, ld, z, ldz, bias, bias_dt, 1.f / tau, q_scale, seq_row0, seq_len, slots, state, out,
                              ldo, B, H, dim, vdim, st);
}

QNN_API int qnn_gla_norm_gate(const float* o, long long ldo, const void* w, int w_dt, float eps, const void* g,
                              long long ldg, void* out, long long ld_out, int dtype, int rows, int H, int vdim,
                              cudaStream_t st) {
    if (rows <= 0) return 0;
    if (H <= 0 || vdim <= 0) return QNN_ERR_ARGUMENT;
    const int warps = 4;
    const dim3 grid(((size_t)rows * H + warps - 1) / warps);
    if (dtype == QNN_DT_BF16)
        launch_pdl(gla_norm_gate_kernel<bf16>, grid, dim3(warps * 32), 0, st, o, ldo, w, w_dt, eps, (const bf16*)g, ldg,
                   (bf16*)out, ld_out, rows, H, vdim);
    else
        launch_pdl(gla_norm_gate_kernel<float>, grid, dim3(warps * 32), 0, st, o, ldo, w, w_dt, eps, (const float*)g, ldg,
                   (float*)out, ld_out, rows, H, vdim);
    QNN_LAUNCH_CHECK();
}
