// State-space duality mixer (Mamba-2), the parts that are not matrix products:
//
//   scan:  dt = softplus(dt_raw + dt_bias[h]);  a = exp(-exp(A_log[h]) * dt)
//          S_t = a S_(t-1) + dt * B_t x_t^T      (S: N x V per head, from zero, 32-bit, carried per request)
//          y_t = S_t^T C_t + D[h] x_t
//   norm:  v = y * silu(z);  out = v / sqrt(mean_group(v^2) + eps) * w    (groups of equal consecutive parts)
//
// x, B and C are columns of one row per token (what the convolution wrote): x [H, V] first, then B
// [G, N], then C [G, N]; head h reads group h / (H / G). Everything here is 32-bit arithmetic; the
// storage type T is only what x, B, C and z are read as and what the norm's result is rounded to.
//
// The scan walks a sequence's tokens in order. A block owns (32 columns of V, a head, a sequence); a
// thread owns one column and R consecutive rows of S in registers, the block's `slices` warps cover
// N = slices * R rows. Tokens are staged 16 at a time in shared memory (x, B, C, and dt and the decay
// formed once per token); every thread then walks the 16 tokens with multiply-adds only, leaves its
// partial sums of S^T C in shared memory, and the block adds the slices' partial sums in a fixed
// order. The state's arithmetic does not depend on how a request's tokens were cut into steps: a
// step continues from the stored S exactly where the step before left it.
#include <math.h>

#include "common.cuh"

namespace {
enum : int { TK_K_SSD = 11 };
constexpr int SSD_COLS = 32;     // columns of V a block owns (one per lane)
constexpr int SSD_TOK = 16;      // tokens staged at a time
constexpr int SSD_MAX_SLICES = 8;
}  // namespace

template <typename T, int R>
__global__ void __launch_bounds__(SSD_COLS* SSD_MAX_SLICES)
ssd_scan_kernel(const T* xbc, int64_t xbc_stride, const float* dt_raw, int64_t dt_stride,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                const float* __restrict__ D_skip, float* state, const int* cu_seqlens, const int* seq_ctx,
                const int* seq_slot, float* y, int H, int V, int N, int G) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float smem[];
    const int slices = blockDim.y, NP = slices * R;          // rows of S the block covers (>= N)
    float* xs = smem;                                        // [TOK][COLS]
    float* Bs = xs + SSD_TOK * SSD_COLS;                     // [TOK][NP]
    float* Cs = Bs + SSD_TOK * NP;                           // [TOK][NP]
    float* part = Cs + SSD_TOK * NP;                         // [slices][TOK][COLS]
    __shared__ float dts[SSD_TOK], decay[SSD_TOK];

    const int s = blockIdx.z, h = blockIdx.y, p0 = blockIdx.x * SSD_COLS;
    const int first = cu_seqlens[s], len = cu_seqlens[s + 1] - first;
    if (len <= 0) return;
    const int lane = threadIdx.x, slice = threadIdx.y;
    const int tid = slice * SSD_COLS + lane, threads = slices * SSD_COLS;
    const int p = p0 + lane, n0 = slice * R;
    const int g = h / (H / G);
    const int inner = H * V;
    const float A = expf(A_log[h]), Dh = D_skip[h], bias = dt_bias[h];
    float* st = state + ((size_t)TK_SLOT(TK_K_SSD, seq_slot[s]) * H + h) * N * V;

    float S[R];
#pragma unroll
    for (int r = 0; r < R; ++r) S[r] = 0.f;
    if (seq_ctx[s] > 0 && p < V) {
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (n0 + r < N) S[r] = st[(size_t)(n0 + r) * V + p];
    }

    for (int t0 = 0; t0 < len; t0 += SSD_TOK) {
        const int nt = min(SSD_TOK, len - t0);
        for (int i = tid; i < nt * SSD_COLS; i += threads) {
            const int t = i / SSD_COLS, c = i % SSD_COLS;
            xs[i] = p0 + c < V ? to_f<T>(xbc[(size_t)(first + t0 + t) * xbc_stride + h * V + p0 + c]) : 0.f;
        }
        for (int i = tid; i < nt * NP; i += threads) {
            const int t = i / NP, n = i % NP;
            const T* row = xbc + (size_t)(first + t0 + t) * xbc_stride + inner + g * N;
            Bs[i] = n < N ? to_f<T>(row[n]) : 0.f;
            Cs[i] = n < N ? to_f<T>(row[(size_t)G * N + n]) : 0.f;
        }
        if (tid < nt) {
            const float v = dt_raw[(size_t)(first + t0 + tid) * dt_stride + h] + bias;
            const float dt = v > 20.f ? v : log1pf(expf(v));
            dts[tid] = dt;
            decay[tid] = expf(-A * dt);
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float a = decay[t], bx = dts[t] * xs[t * SSD_COLS + lane];
            const float* Bt = Bs + t * NP + n0;
            const float* Ct = Cs + t * NP + n0;
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; r += 4) {
                const float4 b = *reinterpret_cast<const float4*>(Bt + r);
                const float4 c = *reinterpret_cast<const float4*>(Ct + r);
                S[r] = fmaf(bx, b.x, a * S[r]);
                S[r + 1] = fmaf(bx, b.y, a * S[r + 1]);
                S[r + 2] = fmaf(bx, b.z, a * S[r + 2]);
                S[r + 3] = fmaf(bx, b.w, a * S[r + 3]);
                acc = fmaf(S[r], c.x, acc);
                acc = fmaf(S[r + 1], c.y, acc);
                acc = fmaf(S[r + 2], c.z, acc);
                acc = fmaf(S[r + 3], c.w, acc);
            }
            part[(slice * SSD_TOK + t) * SSD_COLS + lane] = acc;
        }
        __syncthreads();
        for (int i = tid; i < nt * SSD_COLS; i += threads) {
            const int t = i / SSD_COLS, c = i % SSD_COLS;
            if (p0 + c >= V) continue;
            float sum = 0.f;
            for (int k = 0; k < slices; ++k) sum += part[(k * SSD_TOK + t) * SSD_COLS + c];
            y[(size_t)(first + t0 + t) * inner + h * V + p0 + c] = fmaf(Dh, xs[i], sum);
        }
        __syncthreads();
    }
    if (p < V) {
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (n0 + r < N) st[(size_t)(n0 + r) * V + p] = S[r];
    }
}

template <typename T, int R>
static int launch_ssd(const void* xbc, int64_t xbc_stride, const float* dt_raw, int64_t dt_stride, const float* dt_bias,
                      const float* A_log, const float* D_skip, float* state, const int* cu_seqlens, const int* seq_ctx,
                      const int* seq_slot, int n_seqs, float* y, int H, int V, int N, int G, cudaStream_t stream) {
    const int slices = (N + R - 1) / R;
    const size_t smem = ((size_t)SSD_TOK * SSD_COLS + 2 * (size_t)SSD_TOK * slices * R +
                         (size_t)slices * SSD_TOK * SSD_COLS) * sizeof(float);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        cudaFuncSetAttribute(ssd_scan_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        raised = true;
    }
    tk_launch(ssd_scan_kernel<T, R>, dim3((V + SSD_COLS - 1) / SSD_COLS, H, n_seqs), dim3(SSD_COLS, slices), smem,
              stream, (const T*)xbc, xbc_stride, dt_raw, dt_stride, dt_bias, A_log, D_skip, state, cu_seqlens, seq_ctx,
              seq_slot, y, H, V, N, G);
    return 0;
}

TK_API int tk_ssd_max_state() { return 32 * SSD_MAX_SLICES; }

// xbc: [T, >= H V + 2 G N] rows `xbc_stride` apart (type dtype); dt_raw: float32 [T, >= H] rows `dt_stride`
// apart; dt_bias, A_log, D_skip: float32 [H]; state: float32 [slots, H, N, V]; y: float32 [T, H V].
TK_API int tk_ssd_scan(const void* xbc, int64_t xbc_stride, const float* dt_raw, int64_t dt_stride,
                       const float* dt_bias, const float* A_log, const float* D_skip, float* state,
                       const int* cu_seqlens, const int* seq_ctx, const int* seq_slot, int n_seqs, float* y, int H,
                       int V, int N, int G, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(H > 0 && V > 0 && N > 0 && G > 0 && H % G == 0, "state-space scan: %d heads in %d groups", H, G);
    TK_CHECK_ARG(N <= tk_ssd_max_state(), "state-space scan: a state of %d rows; up to %d are built", N,
                 tk_ssd_max_state());
    TK_CHECK_ARG(n_seqs >= 0, "state-space scan: bad sizes");
    if (n_seqs == 0) return 0;
#define TK_SSD(TT)                                                                                                  \
    do {                                                                                                            \
        if (N <= 8 * SSD_MAX_SLICES)                                                                                \
            launch_ssd<TT, 8>(xbc, xbc_stride, dt_raw, dt_stride, dt_bias, A_log, D_skip, state, cu_seqlens,        \
                              seq_ctx, seq_slot, n_seqs, y, H, V, N, G, stream);                                    \
        else if (N <= 16 * SSD_MAX_SLICES)                                                                          \
            launch_ssd<TT, 16>(xbc, xbc_stride, dt_raw, dt_stride, dt_bias, A_log, D_skip, state, cu_seqlens,       \
                               seq_ctx, seq_slot, n_seqs, y, H, V, N, G, stream);                                   \
        else                                                                                                        \
            launch_ssd<TT, 32>(xbc, xbc_stride, dt_raw, dt_stride, dt_bias, A_log, D_skip, state, cu_seqlens,       \
                               seq_ctx, seq_slot, n_seqs, y, H, V, N, G, stream);                                   \
    } while (0)
    if (dtype == TK_F32) TK_SSD(float);
    else if (dtype == TK_BF16) TK_SSD(__nv_bfloat16);
    else TK_CHECK_ARG(false, "state-space scan: unknown dtype %d", dtype);
#undef TK_SSD
    TK_CHECK_LAUNCH("ssd_scan");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// out = group_norm(y * silu(z)) * w: one warp per (row, group). A lane keeps its elements in
// registers when the group is short enough (ITEMS per lane), else it forms them a second time.
// ---------------------------------------------------------------------------------------------
template <typename T, int ITEMS>
__global__ void __launch_bounds__(128)
gated_group_norm_kernel(const float* y, const T* z, int64_t z_stride, const float* __restrict__ w, float eps, T* out,
                        int rows, int width, int groups) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (warp >= rows * groups) return;
    const int r = warp / groups, gw = width / groups, c0 = (warp % groups) * gw;
    auto at = [&](int i) {
        const float zv = to_f<T>(z[(size_t)r * z_stride + c0 + i]);
        return y[(size_t)r * width + c0 + i] * (zv / (1.0f + expf(-zv)));
    };
    float ss = 0.f;
    if constexpr (ITEMS > 0) {
        float keep[ITEMS];
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int i = lane + 32 * k;
            keep[k] = i < gw ? at(i) : 0.f;
            ss += keep[k] * keep[k];
        }
        const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)gw + eps);
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int i = lane + 32 * k;
            if (i < gw) out[(size_t)r * width + c0 + i] = from_f<T>(keep[k] * rstd * w[c0 + i]);
        }
    } else {
        for (int i = lane; i < gw; i += 32) {
            const float v = at(i);
            ss += v * v;
        }
        const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)gw + eps);
        for (int i = lane; i < gw; i += 32) out[(size_t)r * width + c0 + i] = from_f<T>(at(i) * rstd * w[c0 + i]);
    }
}

// y: float32 [rows, width]; z: [rows, width] (type dtype) rows `z_stride` apart; w: float32 [width];
// out: [rows, width] (type dtype).
TK_API int tk_gated_group_norm(const float* y, const void* z, int64_t z_stride, const float* w, float eps, void* out,
                               int rows, int width, int groups, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && width > 0 && groups > 0 && width % groups == 0,
                 "gated group norm: a row of %d in %d groups", width, groups);
    if (rows == 0) return 0;
    const int gw = width / groups;
    const int warps = rows * groups;
    dim3 grid((warps + 3) / 4), block(128);
#define TK_GGN(TT)                                                                                               \
    do {                                                                                                         \
        if (gw <= 32 * 4)                                                                                        \
            tk_launch(gated_group_norm_kernel<TT, 4>, grid, block, 0, stream, y, (const TT*)z, z_stride, w, eps,  \
                      (TT*)out, rows, width, groups);                                                            \
        else if (gw <= 32 * 16)                                                                                  \
            tk_launch(gated_group_norm_kernel<TT, 16>, grid, block, 0, stream, y, (const TT*)z, z_stride, w, eps, \
                      (TT*)out, rows, width, groups);                                                            \
        else                                                                                                     \
            tk_launch(gated_group_norm_kernel<TT, 0>, grid, block, 0, stream, y, (const TT*)z, z_stride, w, eps,  \
                      (TT*)out, rows, width, groups);                                                            \
    } while (0)
    if (dtype == TK_F32) TK_GGN(float);
    else if (dtype == TK_BF16) TK_GGN(__nv_bfloat16);
    else TK_CHECK_ARG(false, "gated group norm: unknown dtype %d", dtype);
#undef TK_GGN
    TK_CHECK_LAUNCH("gated_group_norm");
    return 0;
}
