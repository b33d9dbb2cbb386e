// Gated linear attention: a matrix state per (sequence, head) that decays per key channel.
//
//   S_t = diag(a_t) S_{t-1} + k_t v_t^T          S: [dim, vdim], float32, kept per cache slot
//   o_t = S_t^T (q_t * q_scale)
//   a_t = sigmoid(z_t + bias)^(1/tau) = exp(log_sigmoid(z_t + bias) / tau)       (float32; formed by the kernel
//                                                  that forms z, see qnn_small_linear_f32)
//
//   qnn_gla_scan        walks the rows of every sequence of a step in order, from the slot's state and back
//                       into it: whole prompts, portions and single tokens are the same launch
//   qnn_gla_norm_gate   per head: RMS norm of o over vdim with a weight shared by the heads, times silu(g)
//
// The scan: a block owns 32 value columns of one (sequence, head).  Four lanes share a column, each with a quarter of
// the key channels of the state in registers; q, k, the decay and v of 16 rows at a time are staged in shared memory,
// the next 16 rows' loads in flight while these are walked; a lane reads its channels as 16-byte pieces.  The
// order of the sums depends on dim only, so a row gives the same numbers in any batch and any cutting of its sequence.
#include "common.cuh"

using namespace qnn;

namespace {

constexpr int GLA_COLS = 32;      // value columns of a block
constexpr int GLA_SHARE = 4;      // lanes that share a column
constexpr int GLA_ROWS = 16;      // rows staged at a time
constexpr int GLA_THREADS = GLA_COLS * GLA_SHARE;

// One chunk of GLA_ROWS rows in shared memory: q, k, decay as [row][part][channel of the part] with a pad of 4 floats
// between the parts (the four lanes of a column read 16 bytes each from four different banks), then v [row][column].
template <int RPT>
struct GlaChunk {
    static constexpr int PART = RPT + 4, ROW = GLA_SHARE * PART, ARRAY = GLA_ROWS * ROW;
    static constexpr int FLOATS = 3 * ARRAY + GLA_ROWS * GLA_COLS;
    static constexpr int PER_THREAD = GLA_ROWS * RPT * GLA_SHARE / GLA_THREADS;      // staged elements of one array per thread
    static constexpr int V_PER_THREAD = GLA_ROWS * GLA_COLS / GLA_THREADS;
};

template <typename T, int RPT>
__global__ void __launch_bounds__(GLA_THREADS)
gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, long long ld,
                const float* __restrict__ decay, long long ldd, float q_scale, const int* __restrict__ seq_row0,
                const int* __restrict__ seq_len, const int* __restrict__ slots, float* __restrict__ state,
                float* __restrict__ out, long long ldo, int H, int dim, int vdim) {
    using C = GlaChunk<RPT>;
    constexpr int DIMP = RPT * GLA_SHARE;                    // key channels with padding
    constexpr bool AHEAD = RPT <= 32;                        // the next chunk's loads in registers while this one is walked
    extern __shared__ __align__(16) float sm[];
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
        const int i = part * RPT + r;
        S[r] = (live && i < dim) ? my_state[(size_t)i * vdim] : 0.f;
    }
    float rq[C::PER_THREAD], rk[C::PER_THREAD], ra[C::PER_THREAD], rv[C::V_PER_THREAD];
    auto fetch = [&](int t0) {                               // global memory -> registers (rows beyond the sequence: nothing)
        const int nt = min(GLA_ROWS, n - t0);
#pragma unroll
        for (int e = 0; e < C::PER_THREAD; ++e) {
            const int idx = threadIdx.x + e * GLA_THREADS, tt = idx / DIMP, i = idx - tt * DIMP;
            rq[e] = 0.f; rk[e] = 0.f; ra[e] = 1.f;
            if (tt < nt && i < dim) {
                const size_t row = (size_t)(row0 + t0 + tt);
                rq[e] = to_f(q[row * ld + h * dim + i]) * q_scale;
                rk[e] = to_f(k[row * ld + h * dim + i]);
                ra[e] = decay[row * ldd + h * dim + i];
            }
        }
#pragma unroll
        for (int e = 0; e < C::V_PER_THREAD; ++e) {
            const int idx = threadIdx.x + e * GLA_THREADS, tt = idx / GLA_COLS, c = idx - tt * GLA_COLS;
            rv[e] = (tt < nt && c0 + c < vdim) ? to_f(v[(size_t)(row0 + t0 + tt) * ld + h * vdim + c0 + c]) : 0.f;
        }
    };
    auto put = [&](float* buf) {                             // registers -> shared memory
#pragma unroll
        for (int e = 0; e < C::PER_THREAD; ++e) {
            const int idx = threadIdx.x + e * GLA_THREADS, tt = idx / DIMP, i = idx - tt * DIMP;
            const int at = tt * C::ROW + (i / RPT) * C::PART + (i % RPT);
            buf[at] = rq[e];
            buf[C::ARRAY + at] = rk[e];
            buf[2 * C::ARRAY + at] = ra[e];
        }
#pragma unroll
        for (int e = 0; e < C::V_PER_THREAD; ++e) buf[3 * C::ARRAY + threadIdx.x + e * GLA_THREADS] = rv[e];
    };
    fetch(0);
    put(sm);
    __syncthreads();
    int cur = 0;
    for (int t0 = 0; t0 < n; t0 += GLA_ROWS) {
        const int nt = min(GLA_ROWS, n - t0);
        const bool more = t0 + GLA_ROWS < n;
        float* buf = sm + (AHEAD ? cur * C::FLOATS : 0);
        if (AHEAD && more) fetch(t0 + GLA_ROWS);
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = buf[3 * C::ARRAY + tt * GLA_COLS + cl];
            const float4* aq = reinterpret_cast<const float4*>(buf + tt * C::ROW + part * C::PART);
            const float4* ak = reinterpret_cast<const float4*>(buf + C::ARRAY + tt * C::ROW + part * C::PART);
            const float4* aa = reinterpret_cast<const float4*>(buf + 2 * C::ARRAY + tt * C::ROW + part * C::PART);
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < RPT / 4; ++j) {
                const float4 a4 = aa[j], k4 = ak[j], q4 = aq[j];
                S[4 * j] = a4.x * S[4 * j] + k4.x * vj;
                acc += S[4 * j] * q4.x;
                S[4 * j + 1] = a4.y * S[4 * j + 1] + k4.y * vj;
                acc += S[4 * j + 1] * q4.y;
                S[4 * j + 2] = a4.z * S[4 * j + 2] + k4.z * vj;
                acc += S[4 * j + 2] * q4.z;
                S[4 * j + 3] = a4.w * S[4 * j + 3] + k4.w * vj;
                acc += S[4 * j + 3] * q4.w;
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (part == 0 && col < vdim) out[(size_t)(row0 + t0 + tt) * ldo + h * vdim + col] = slot >= 0 ? acc : 0.f;
        }
        if (more) {
            if (AHEAD) {
                put(sm + (cur ^ 1) * C::FLOATS);             // nobody reads that buffer: its chunk was walked a round ago
                cur ^= 1;
            } else {
                __syncthreads();
                fetch(t0 + GLA_ROWS);
                put(sm);
            }
            __syncthreads();
        }
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < RPT; ++r) {
            const int i = part * RPT + r;
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
int scan_launch(const void* q, const void* k, const void* v, long long ld, const float* decay, long long ldd, float q_scale,
                const int* seq_row0, const int* seq_len, const int* slots, float* state, float* out, long long ldo, int B,
                int H, int dim, int vdim, cudaStream_t st) {
    const dim3 grid((vdim + GLA_COLS - 1) / GLA_COLS, H, B);
    const int rpt = (dim + GLA_SHARE - 1) / GLA_SHARE;
#define QNN_GLA(RPTV)                                                                                                \
    {                                                                                                                \
        const size_t smem = (size_t)GlaChunk<RPTV>::FLOATS * sizeof(float) * (RPTV <= 32 ? 2 : 1);                   \
        static bool set = false;                                                                                     \
        if (smem > 48 * 1024 && !set) {                                                                              \
            cudaFuncSetAttribute(gla_scan_kernel<T, RPTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
            set = true;                                                                                              \
        }                                                                                                            \
        launch_pdl(gla_scan_kernel<T, RPTV>, grid, dim3(GLA_THREADS), smem, st, (const T*)q, (const T*)k,           \
                   (const T*)v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, H, dim, vdim);   \
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
// decay: the decays a [rows, H*dim] float32 (qnn_small_linear_f32 forms them in its epilogue); seq_row0 / seq_len:
// first row and row count of each of the B sequences (both null: sequence b is row b alone); slots: the state slot
// of each sequence, negative for a row of no sequence (its output is zero, no state is touched); state:
// [slots, H, dim, vdim] float32; out: [rows, H*vdim] float32.  dim up to 256.
QNN_API int qnn_gla_scan(const void* q, const void* k, const void* v, long long ld, int dtype, const float* decay,
                         long long ldd, float q_scale, const int* seq_row0, const int* seq_len, const int* slots,
                         float* state, float* out, long long ldo, int B, int H, int dim, int vdim, cudaStream_t st) {
    if (B <= 0) return 0;
    if (H <= 0 || dim <= 0 || vdim <= 0 || H > 65535 || B > 65535) return QNN_ERR_ARGUMENT;
    if ((seq_row0 == nullptr) != (seq_len == nullptr)) return QNN_ERR_ARGUMENT;
    if (dtype == QNN_DT_BF16)
        return scan_launch<bf16>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, B, H, dim,
                                 vdim, st);
    return scan_launch<float>(q, k, v, ld, decay, ldd, q_scale, seq_row0, seq_len, slots, state, out, ldo, B, H, dim, vdim,
                              st);
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
