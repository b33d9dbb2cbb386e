// Routed experts, on the device from the router to the sum, so that a decode step stays one CUDA graph.
//
//   qnn_moe_route      router logits (float32 sums), a score function, the `top` best experts of every row
//                      (ties to the lower index) and their scores
//   qnn_moe_plan       rows grouped by expert: offsets, a permutation, and a list of (expert, first row) tiles of
//                      up to 16 rows; one block
//   qnn_moe_gate_up    per tile: gathered rows (times their score, when the score goes on the input) against the
//                      expert's stacked gate|up matrix, then the gated activation
//   qnn_moe_down       per tile: the expert's down matrix; rows go back to where they came from (float32),
//                      times their score when the score goes on the output
//   qnn_moe_combine    out[t] = sum over a row's experts (+ a shared expert's output), float32
//   qnn_gated_act_clamped   the clamped activation for a dense product: g = min(gate, limit),
//                      u = clamp(up, -limit, limit), g * sigmoid(alpha g) * (u + 1)
//
// The two tile kernels are plain FMA kernels for both element types: 16 rows x 128 output columns per block,
// 32 inner elements at a time through shared memory.  Sums run over the inner size in a fixed order, so a row's
// result does not depend on which other rows share its tile.
#include "common.cuh"

using namespace qnn;

#define QNN_MOE_SCORE_SIGMOID 0
#define QNN_MOE_SCORE_SOFTMAX 1
#define QNN_GATED_SWIGLU_CLAMPED 2          // after QNN_ACT_GELU_TANH 0 and QNN_ACT_SILU 1

namespace {

constexpr int TILE_ROWS = 16;
constexpr int TILE_COLS = 128;
constexpr int TILE_K = 32;
constexpr int MAX_TOP = 16;

// ---- router ----------------------------------------------------------------------------------------

template <typename TX, typename TW>
__global__ void moe_route_kernel(const TX* __restrict__ x, const TW* __restrict__ wr, int T, int W, int E, int top,
                                 int score_fn, int renorm, int* __restrict__ sel_e, float* __restrict__ sel_w) {
    extern __shared__ float sc[];                       // [warps][E]
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* s = sc + (size_t)warp * E;
    const TX* xr = x + (size_t)t * W;
    for (int e = 0; e < E; ++e) {
        const TW* wrow = wr + (size_t)e * W;
        float d = 0.f;
        for (int i = lane; i < W; i += 32) d += to_f(xr[i]) * to_f(wrow[i]);
        d = warp_sum(d);
        if (lane == 0) s[e] = d;
    }
    __syncwarp();
    // Both score functions rise with the logit, so the experts are chosen by their logits (a sigmoid that has
    // run into 1.0 would tie where the logits still differ) and only the chosen ones' scores are formed.
    float m = -INFINITY, sum = 1.f;
    if (score_fn == QNN_MOE_SCORE_SOFTMAX) {
        for (int e = lane; e < E; e += 32) m = fmaxf(m, s[e]);
        m = warp_max(m);
        sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += expf(s[e] - m);
        sum = warp_sum(sum);
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = s[e];
            if (v > best) { best = v; arg = e; }          // ascending e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = 0;                    // logits that are all NaN: any expert, the model's logits will show it
        best = score_fn == QNN_MOE_SCORE_SOFTMAX ? expf(best - m) / sum : 1.f / (1.f + expf(-best));
        total += best;
        if (lane == 0) {
            sel_e[(size_t)t * top + k] = arg;
            sel_w[(size_t)t * top + k] = best;
            s[arg] = -INFINITY;
        }
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int k = 0; k < top; ++k) sel_w[(size_t)t * top + k] /= total;
}

// ---- grouping ----------------------------------------------------------------------------------------

// offsets: [E + 1]; perm: [n] sorted place -> entry (row * top + k); tiles: [max_tiles][2] (expert, first sorted
// place); n_tiles: [1].  Which of an expert's rows comes first varies from run to run; no result depends on it.
__global__ void moe_plan_kernel(const int* __restrict__ sel_e, int n, int E, int* __restrict__ offsets,
                                int* __restrict__ perm, int* __restrict__ tiles, int* __restrict__ n_tiles) {
    extern __shared__ int cnt[];                        // [E] counts, then [E] running places
    int* at = cnt + E;
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[sel_e[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = o;
            at[e] = o;
            for (int r = 0; r < cnt[e]; r += TILE_ROWS) {
                tiles[2 * nt] = e;
                tiles[2 * nt + 1] = o + r;
                ++nt;
            }
            o += cnt[e];
        }
        offsets[E] = o;
        *n_tiles = nt;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) perm[atomicAdd(&at[sel_e[i]], 1)] = i;
}

// ---- tiles ---------------------------------------------------------------------------------------------

__device__ __forceinline__ float gated(float g, float u, int act, float limit, float alpha) {
    if (act == QNN_GATED_SWIGLU_CLAMPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g * (1.f / (1.f + expf(-alpha * g))) * (u + 1.f);
    }
    return activate(g, act) * u;
}

// acc[m][r] += sum_k xs[k][r] * w_m[col][k] over K, for NM matrices whose rows `col` lie `K` apart.
// xs is filled by `fill(k0, kn)` for each block of inner elements.
template <typename TW, int NM, typename Fill>
__device__ __forceinline__ void tile_product(const TW* const (&w)[NM], int col0, int n_cols, int K, float (*xs)[TILE_ROWS],
                                             float (*ws)[TILE_K][TILE_COLS + 1], float (&acc)[NM][TILE_ROWS], Fill fill) {
    for (int k0 = 0; k0 < K; k0 += TILE_K) {
        const int kn = min(TILE_K, K - k0);
        __syncthreads();
        fill(k0, kn);
#pragma unroll
        for (int m = 0; m < NM; ++m)
            for (int idx = threadIdx.x; idx < TILE_COLS * TILE_K; idx += TILE_COLS) {
                const int c = idx / TILE_K, kk = idx - c * TILE_K;
                ws[m][kk][c] = (c < n_cols && kk < kn) ? to_f(w[m][(size_t)(col0 + c) * K + k0 + kk]) : 0.f;
            }
        __syncthreads();
#pragma unroll 4
        for (int kk = 0; kk < TILE_K; ++kk) {
            float xv[TILE_ROWS];
#pragma unroll
            for (int r = 0; r < TILE_ROWS; r += 4) {
                const float4 f = *reinterpret_cast<const float4*>(&xs[kk][r]);
                xv[r] = f.x; xv[r + 1] = f.y; xv[r + 2] = f.z; xv[r + 3] = f.w;
            }
#pragma unroll
            for (int m = 0; m < NM; ++m) {
                const float wv = ws[m][kk][threadIdx.x];
#pragma unroll
                for (int r = 0; r < TILE_ROWS; ++r) acc[m][r] += xv[r] * wv;
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(TILE_COLS)
moe_gate_up_kernel(const T* __restrict__ x, int W, const T* __restrict__ w_gu, int ff, const int* __restrict__ offsets,
                   const int* __restrict__ perm, const float* __restrict__ sel_w, const int* __restrict__ tiles,
                   const int* __restrict__ n_tiles, int top, int scale_input, int act, float limit, float alpha,
                   T* __restrict__ hidden) {
    __shared__ __align__(16) float xs[TILE_K][TILE_ROWS];
    __shared__ float ws[2][TILE_K][TILE_COLS + 1];
    __shared__ int src_row[TILE_ROWS];
    __shared__ float src_w[TILE_ROWS];
    pdl_wait();
    if ((int)blockIdx.x >= *n_tiles) return;
    const int e = tiles[2 * blockIdx.x], p0 = tiles[2 * blockIdx.x + 1];
    const int rows = min(TILE_ROWS, offsets[e + 1] - p0);
    const int col0 = blockIdx.y * TILE_COLS, n_cols = min(TILE_COLS, ff - col0);
    if (threadIdx.x < TILE_ROWS) {
        const int entry = threadIdx.x < rows ? perm[p0 + threadIdx.x] : -1;
        src_row[threadIdx.x] = entry < 0 ? -1 : entry / top;
        src_w[threadIdx.x] = (entry < 0 || !scale_input) ? 1.f : sel_w[entry];
    }
    const T* wg = w_gu + (size_t)e * 2 * ff * W;
    const T* const w2[2] = {wg, wg + (size_t)ff * W};
    float acc[2][TILE_ROWS];
#pragma unroll
    for (int r = 0; r < TILE_ROWS; ++r) acc[0][r] = acc[1][r] = 0.f;
    tile_product<T, 2>(w2, col0, n_cols, W, xs, ws, acc, [&](int k0, int kn) {
        for (int idx = threadIdx.x; idx < TILE_ROWS * TILE_K; idx += TILE_COLS) {
            const int r = idx / TILE_K, kk = idx - r * TILE_K;
            const int row = src_row[r];
            xs[kk][r] = (row >= 0 && kk < kn) ? to_f(x[(size_t)row * W + k0 + kk]) * src_w[r] : 0.f;
        }
    });
    if ((int)threadIdx.x < n_cols)
        for (int r = 0; r < rows; ++r)
            hidden[(size_t)(p0 + r) * ff + col0 + threadIdx.x] = from_f<T>(gated(acc[0][r], acc[1][r], act, limit, alpha));
}

template <typename T>
__global__ void __launch_bounds__(TILE_COLS)
moe_down_kernel(const T* __restrict__ hidden, int ff, const T* __restrict__ w_down, int W, const int* __restrict__ offsets,
                const int* __restrict__ perm, const float* __restrict__ sel_w, const int* __restrict__ tiles,
                const int* __restrict__ n_tiles, int scale_output, float* __restrict__ ys) {
    __shared__ __align__(16) float xs[TILE_K][TILE_ROWS];
    __shared__ float ws[1][TILE_K][TILE_COLS + 1];
    pdl_wait();
    if ((int)blockIdx.x >= *n_tiles) return;
    const int e = tiles[2 * blockIdx.x], p0 = tiles[2 * blockIdx.x + 1];
    const int rows = min(TILE_ROWS, offsets[e + 1] - p0);
    const int col0 = blockIdx.y * TILE_COLS, n_cols = min(TILE_COLS, W - col0);
    const T* const w1[1] = {w_down + (size_t)e * W * ff};
    float acc[1][TILE_ROWS];
#pragma unroll
    for (int r = 0; r < TILE_ROWS; ++r) acc[0][r] = 0.f;
    tile_product<T, 1>(w1, col0, n_cols, ff, xs, ws, acc, [&](int k0, int kn) {
        for (int idx = threadIdx.x; idx < TILE_ROWS * TILE_K; idx += TILE_COLS) {
            const int r = idx / TILE_K, kk = idx - r * TILE_K;
            xs[kk][r] = (r < rows && kk < kn) ? to_f(hidden[(size_t)(p0 + r) * ff + k0 + kk]) : 0.f;
        }
    });
    if ((int)threadIdx.x < n_cols)
        for (int r = 0; r < rows; ++r) {
            const int entry = perm[p0 + r];
            ys[(size_t)entry * W + col0 + threadIdx.x] = acc[0][r] * (scale_output ? sel_w[entry] : 1.f);
        }
}

__global__ void moe_combine_kernel(const float* __restrict__ ys, int top, const void* __restrict__ shared, int shared_dt,
                                   float* __restrict__ out, int W, size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / W, c = i - t * W;
    float s = shared ? load_as_f(shared, shared_dt, i) : 0.f;
    for (int k = 0; k < top; ++k) s += ys[(t * top + k) * W + c];
    out[i] = s;
}

template <typename T>
__global__ void gated_act_clamped_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, float limit, float alpha,
                                         size_t n) {
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / I, c = i - t * I;
    out[i] = from_f<T>(gated(to_f(gu[t * 2 * I + c]), to_f(gu[t * 2 * I + I + c]), QNN_GATED_SWIGLU_CLAMPED, limit, alpha));
}

}  // namespace

QNN_API int qnn_moe_route(const void* x, int x_dt, const void* w_router, int w_dt, int T, int W, int E, int top,
                          int score_fn, int renorm, int* sel_e, float* sel_w, cudaStream_t st) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || top > MAX_TOP || W <= 0) return QNN_ERR_ARGUMENT;
    const int warps = 4;
    const size_t smem = (size_t)warps * E * sizeof(float);
    if (smem > 48 * 1024) return QNN_ERR_UNSUPPORTED;
    const dim3 grid((T + warps - 1) / warps), block(warps * 32);
#define QNN_ROUTE(TX, TW)                                                                                         \
    launch_pdl(moe_route_kernel<TX, TW>, grid, block, smem, st, (const TX*)x, (const TW*)w_router, T, W, E, top,  \
               score_fn, renorm, sel_e, sel_w)
    if (x_dt == QNN_DT_BF16 && w_dt == QNN_DT_BF16) QNN_ROUTE(bf16, bf16);
    else if (x_dt == QNN_DT_BF16) QNN_ROUTE(bf16, float);
    else if (w_dt == QNN_DT_BF16) QNN_ROUTE(float, bf16);
    else QNN_ROUTE(float, float);
#undef QNN_ROUTE
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_moe_max_tiles(int n_entries, int E) { return (n_entries + TILE_ROWS - 1) / TILE_ROWS + E; }

QNN_API int qnn_moe_plan(const int* sel_e, int n, int E, int* offsets, int* perm, int* tiles, int* n_tiles,
                         cudaStream_t st) {
    if (n <= 0) return 0;
    if (E <= 0 || (size_t)2 * E * sizeof(int) > 48 * 1024) return QNN_ERR_ARGUMENT;
    launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), st, sel_e, n, E, offsets, perm, tiles,
               n_tiles);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_moe_gate_up(const void* x, int dtype, int W, const void* w_gu, int ff, const int* offsets, const int* perm,
                            const float* sel_w, const int* tiles, const int* n_tiles, int max_tiles, int top,
                            int scale_input, int act, float limit, float alpha, void* hidden, cudaStream_t st) {
    if (max_tiles <= 0) return 0;
    if (W <= 0 || ff <= 0 || top <= 0) return QNN_ERR_ARGUMENT;
    const dim3 grid(max_tiles, (ff + TILE_COLS - 1) / TILE_COLS);
    if (grid.y > 65535) return QNN_ERR_UNSUPPORTED;
    if (dtype == QNN_DT_BF16)
        launch_pdl(moe_gate_up_kernel<bf16>, grid, dim3(TILE_COLS), 0, st, (const bf16*)x, W, (const bf16*)w_gu, ff, offsets,
                   perm, sel_w, tiles, n_tiles, top, scale_input, act, limit, alpha, (bf16*)hidden);
    else
        launch_pdl(moe_gate_up_kernel<float>, grid, dim3(TILE_COLS), 0, st, (const float*)x, W, (const float*)w_gu, ff,
                   offsets, perm, sel_w, tiles, n_tiles, top, scale_input, act, limit, alpha, (float*)hidden);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_moe_down(const void* hidden, int dtype, int ff, const void* w_down, int W, const int* offsets,
                         const int* perm, const float* sel_w, const int* tiles, const int* n_tiles, int max_tiles,
                         int scale_output, float* ys, cudaStream_t st) {
    if (max_tiles <= 0) return 0;
    if (W <= 0 || ff <= 0) return QNN_ERR_ARGUMENT;
    const dim3 grid(max_tiles, (W + TILE_COLS - 1) / TILE_COLS);
    if (grid.y > 65535) return QNN_ERR_UNSUPPORTED;
    if (dtype == QNN_DT_BF16)
        launch_pdl(moe_down_kernel<bf16>, grid, dim3(TILE_COLS), 0, st, (const bf16*)hidden, ff, (const bf16*)w_down, W,
                   offsets, perm, sel_w, tiles, n_tiles, scale_output, ys);
    else
        launch_pdl(moe_down_kernel<float>, grid, dim3(TILE_COLS), 0, st, (const float*)hidden, ff, (const float*)w_down, W,
                   offsets, perm, sel_w, tiles, n_tiles, scale_output, ys);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_moe_combine(const float* ys, int top, const void* shared, int shared_dt, float* out, int T, int W,
                            cudaStream_t st) {
    if (T <= 0) return 0;
    const size_t n = (size_t)T * W;
    launch_pdl(moe_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, ys, top, shared, shared_dt, out, W,
               n);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_gated_act_clamped(const void* gu, void* out, int dtype, int T, int I, float limit, float alpha,
                                  cudaStream_t st) {
    if (T <= 0) return 0;
    const size_t n = (size_t)T * I;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == QNN_DT_BF16)
        launch_pdl(gated_act_clamped_kernel<bf16>, grid, dim3(256), 0, st, (const bf16*)gu, (bf16*)out, I, limit, alpha, n);
    else
        launch_pdl(gated_act_clamped_kernel<float>, grid, dim3(256), 0, st, (const float*)gu, (float*)out, I, limit, alpha,
                   n);
    QNN_LAUNCH_CHECK();
}
