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
// The scan walks a sequence's tokens in order. A block owns (32 columns of V, a head, a sequence), and,
// when a step has too few of those to fill the GPU, a half or a quarter of the state's rows; a
// thread owns one column and R consecutive rows of S in registers, the block's `slices` warps cover
// N = slices * R rows. Tokens are staged 16 at a time in shared memory (x, B, C, and dt and the decay
// formed once per token; the next 16 are asked for before the walk and wait in registers meanwhile);
// every thread then walks the 16 tokens with multiply-adds only, leaves its
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

// Two 32-bit multiply-adds in one instruction (sm_100's packed form): d = a * b + c on both halves, each
// rounded as the scalar instruction rounds.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)),
          "l"(reinterpret_cast<unsigned long long&>(c)));
    return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
    return d;
}

// XC: values of x a thread keeps for the stage ahead (TOK * COLS over the block's threads: 2 with eight
// slices, 4 with four or more, else 16); 0: nothing is kept ahead, a stage's rows go from memory to
// shared memory directly, which costs fewer registers and is what a step of single tokens wants.
template <typename T, int R, int XC>
__global__ void __launch_bounds__(SSD_COLS* SSD_MAX_SLICES, XC > 0 ? 2 : 4)
ssd_scan_kernel(const T* xbc, int64_t xbc_stride, const float* dt_raw, int64_t dt_stride,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                const float* __restrict__ D_skip, float* state, const int* cu_seqlens, const int* seq_ctx,
                const int* seq_slot, float* y, int64_t y_part, int H, int V, int N, int G, int split) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float smem[];
    const int slices = blockDim.y, NP = slices * R;          // rows of S the block covers
    float* __restrict__ xs = smem;                           // [TOK][COLS]
    float* __restrict__ Bs = xs + SSD_TOK * SSD_COLS;        // [TOK][NP]
    float* __restrict__ Cs = Bs + SSD_TOK * NP;              // [TOK][NP]
    float* __restrict__ part = Cs + SSD_TOK * NP;            // [slices][TOK][COLS]
    __shared__ float dts[SSD_TOK], decay[SSD_TOK];

    // blockIdx.x = (chunk of 32 columns, part of the rows): `split` blocks share a head's rows, each
    // with its own sum of S^T C over its rows, which the reader of y adds up
    const int s = blockIdx.z, h = blockIdx.y, p0 = (blockIdx.x / split) * SSD_COLS;
    const int row0 = (blockIdx.x % split) * NP;              // the block's first row of S
    const int first = cu_seqlens[s], len = cu_seqlens[s + 1] - first;
    if (len <= 0) return;
    const int lane = threadIdx.x, slice = threadIdx.y;
    const int tid = slice * SSD_COLS + lane, threads = slices * SSD_COLS;
    const int p = p0 + lane, n0 = slice * R;             // (n0: within the block's rows)
    const int g = h / (H / G);
    const int inner = H * V;
    const float A = expf(A_log[h]), Dh = D_skip[h], bias = dt_bias[h];
    float* st = state + ((size_t)TK_SLOT(TK_K_SSD, seq_slot[s]) * H + h) * N * V;

    float2 S[R / 2];                                  // rows n0 + 2 k and n0 + 2 k + 1 side by side
#pragma unroll
    for (int r = 0; r < R / 2; ++r) S[r] = make_float2(0.f, 0.f);
    if (seq_ctx[s] > 0 && p < V) {
#pragma unroll
        for (int r = 0; r < R / 2; ++r) {
            if (row0 + n0 + 2 * r < N) S[r].x = st[(size_t)(row0 + n0 + 2 * r) * V + p];
            if (row0 + n0 + 2 * r + 1 < N) S[r].y = st[(size_t)(row0 + n0 + 2 * r + 1) * V + p];
        }
    }

    // A stage's rows are asked for one stage ahead and wait in registers while the stage before is
    // walked, so that the walk never waits for memory: per thread TOK * R / 32 values of B and of C
    // (TOK * NP of each over 32 * slices threads), up to XC of x, one of dt.
    constexpr int BC = XC > 0 ? SSD_TOK * R / 32 : 1;
    T rb[BC], rc[BC], rx[XC > 0 ? XC : 1];
    float rdt = 0.f;
    auto fetch = [&](int t0) {
        const int nt = min(SSD_TOK, len - t0);
#pragma unroll
        for (int k = 0; k < BC; ++k) {
            const int i = tid + k * threads, t = i / NP, n = row0 + i % NP;
            const bool ok = t < nt && n < N;
            const T* row = xbc + (size_t)(first + t0 + (ok ? t : 0)) * xbc_stride + inner + g * N;
            rb[k] = ok ? row[n] : from_f<T>(0.f);
            rc[k] = ok ? row[(size_t)G * N + n] : from_f<T>(0.f);
        }
#pragma unroll
        for (int k = 0; k < XC; ++k) {
            const int i = tid + k * threads, t = i / SSD_COLS, c = i % SSD_COLS;
            const bool ok = t < nt && p0 + c < V;
            rx[k] = ok ? xbc[(size_t)(first + t0 + t) * xbc_stride + h * V + p0 + c] : from_f<T>(0.f);
        }
        if (tid < nt) rdt = dt_raw[(size_t)(first + t0 + tid) * dt_stride + h];
    };
    if constexpr (XC > 0) fetch(0);

    for (int t0 = 0; t0 < len; t0 += SSD_TOK) {
        const int nt = min(SSD_TOK, len - t0);
        if constexpr (XC > 0) {
#pragma unroll
            for (int k = 0; k < BC; ++k) {
                const int i = tid + k * threads;
                Bs[i] = to_f<T>(rb[k]);
                Cs[i] = to_f<T>(rc[k]);
            }
#pragma unroll
            for (int k = 0; k < XC; ++k) {
                const int i = tid + k * threads;
                if (i < SSD_TOK * SSD_COLS) xs[i] = to_f<T>(rx[k]);
            }
        } else {
            for (int i = tid; i < nt * SSD_COLS; i += threads) {
                const int t = i / SSD_COLS, c = i % SSD_COLS;
                xs[i] = p0 + c < V ? to_f<T>(xbc[(size_t)(first + t0 + t) * xbc_stride + h * V + p0 + c]) : 0.f;
            }
            for (int i = tid; i < nt * NP; i += threads) {
                const int t = i / NP, n = row0 + i % NP;
                const T* row = xbc + (size_t)(first + t0 + t) * xbc_stride + inner + g * N;
                Bs[i] = n < N ? to_f<T>(row[n]) : 0.f;
                Cs[i] = n < N ? to_f<T>(row[(size_t)G * N + n]) : 0.f;
            }
            if (tid < nt) rdt = dt_raw[(size_t)(first + t0 + tid) * dt_stride + h];
        }
        if (tid < SSD_TOK) {
            // (a stage's unused tokens leave the state as it is: a step of 0 and a decay of 1)
            const float v = rdt + bias;
            const float dt = tid < nt ? (v > 20.f ? v : log1pf(expf(v))) : 0.f;
            dts[tid] = dt;
            decay[tid] = expf(-A * dt);
        }
        __syncthreads();
        if constexpr (XC > 0) {
            if (t0 + SSD_TOK < len) fetch(t0 + SSD_TOK);
        }
        const int walk = XC > 0 ? SSD_TOK : nt;          // (a fixed count lets the next token's loads start early)
#pragma unroll(XC > 0 ? 4 : 1)
        for (int t = 0; t < walk; ++t) {
            const float a = decay[t], bx = dts[t] * xs[t * SSD_COLS + lane];
            const float* Bt = Bs + t * NP + n0;
            const float* Ct = Cs + t * NP + n0;
            if constexpr (XC > 0) {
                const float2 a2 = make_float2(a, a), bx2 = make_float2(bx, bx);
                float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
                for (int r = 0; r < R; r += 4) {
                    const float4 b = *reinterpret_cast<const float4*>(Bt + r);
                    const float4 c = *reinterpret_cast<const float4*>(Ct + r);
                    S[r / 2] = fma2(bx2, make_float2(b.x, b.y), mul2(a2, S[r / 2]));
                    S[r / 2 + 1] = fma2(bx2, make_float2(b.z, b.w), mul2(a2, S[r / 2 + 1]));
                    acc0 = fma2(S[r / 2], make_float2(c.x, c.y), acc0);
                    acc1 = fma2(S[r / 2 + 1], make_float2(c.z, c.w), acc1);
                }
                part[(slice * SSD_TOK + t) * SSD_COLS + lane] = (acc0.x + acc0.y) + (acc1.x + acc1.y);
            } else {
                // a step of single tokens streams the state through: few registers, many resident warps
                // (the same products and sums in the same order as the packed form)
                float ax = 0.f, ay = 0.f, az = 0.f, aw = 0.f;
#pragma unroll
                for (int r = 0; r < R; r += 4) {
                    const float4 b = *reinterpret_cast<const float4*>(Bt + r);
                    const float4 c = *reinterpret_cast<const float4*>(Ct + r);
                    S[r / 2].x = fmaf(bx, b.x, a * S[r / 2].x);
                    S[r / 2].y = fmaf(bx, b.y, a * S[r / 2].y);
                    S[r / 2 + 1].x = fmaf(bx, b.z, a * S[r / 2 + 1].x);
                    S[r / 2 + 1].y = fmaf(bx, b.w, a * S[r / 2 + 1].y);
                    ax = fmaf(S[r / 2].x, c.x, ax);
                    ay = fmaf(S[r / 2].y, c.y, ay);
                    az = fmaf(S[r / 2 + 1].x, c.z, az);
                    aw = fmaf(S[r / 2 + 1].y, c.w, aw);
                }
                part[(slice * SSD_TOK + t) * SSD_COLS + lane] = (ax + ay) + (az + aw);
            }
        }
        __syncthreads();
        for (int i = tid; i < nt * SSD_COLS; i += threads) {
            const int t = i / SSD_COLS, c = i % SSD_COLS;
            if (p0 + c >= V) continue;
            float sum = 0.f;
            for (int k = 0; k < slices; ++k) sum += part[(k * SSD_TOK + t) * SSD_COLS + c];
            y[(size_t)(blockIdx.x % split) * y_part + (size_t)(first + t0 + t) * inner + h * V + p0 + c] =
                row0 == 0 ? fmaf(Dh, xs[i], sum) : sum;
        }
        __syncthreads();
    }
    if (p < V) {
#pragma unroll
        for (int r = 0; r < R / 2; ++r) {
            if (row0 + n0 + 2 * r < N) st[(size_t)(row0 + n0 + 2 * r) * V + p] = S[r].x;
            if (row0 + n0 + 2 * r + 1 < N) st[(size_t)(row0 + n0 + 2 * r + 1) * V + p] = S[r].y;
        }
    }
}

template <typename T, int R, int XC>
static void launch_ssd_as(const void* xbc, int64_t xbc_stride, const float* dt_raw, int64_t dt_stride,
                          const float* dt_bias, const float* A_log, const float* D_skip, float* state,
                          const int* cu_seqlens, const int* seq_ctx, const int* seq_slot, int n_seqs, float* y,
                          int64_t y_part, int H, int V, int N, int G, int split, cudaStream_t stream) {
    const int slices = (N + R - 1) / R / split;
    const size_t smem = ((size_t)SSD_TOK * SSD_COLS + 2 * (size_t)SSD_TOK * slices * R +
                         (size_t)slices * SSD_TOK * SSD_COLS) * sizeof(float);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        cudaFuncSetAttribute(ssd_scan_kernel<T, R, XC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        raised = true;
    }
    tk_launch(ssd_scan_kernel<T, R, XC>, dim3((V + SSD_COLS - 1) / SSD_COLS * split, H, n_seqs), dim3(SSD_COLS, slices),
              smem, stream, (const T*)xbc, xbc_stride, dt_raw, dt_stride, dt_bias, A_log, D_skip, state, cu_seqlens,
              seq_ctx, seq_slot, y, y_part, H, V, N, G, split);
}

// `ahead`: whether stages are asked for a stage ahead (steps with prompt portions)
template <typename T, int R>
static int launch_ssd(const void* xbc, int64_t xbc_stride, const float* dt_raw, int64_t dt_stride, const float* dt_bias,
                      const float* A_log, const float* D_skip, float* state, const int* cu_seqlens, const int* seq_ctx,
                      const int* seq_slot, int n_seqs, float* y, int64_t y_part, int H, int V, int N, int G, bool ahead,
                      int split, cudaStream_t stream) {
    const int slices = (N + R - 1) / R / split;
#define TK_SSD_AS(XC)                                                                                                \
    launch_ssd_as<T, R, XC>(xbc, xbc_stride, dt_raw, dt_stride, dt_bias, A_log, D_skip, state, cu_seqlens, seq_ctx, \
                            seq_slot, n_seqs, y, y_part, H, V, N, G, split, stream)
    if (!ahead) TK_SSD_AS(0);
    else if (slices >= 8) TK_SSD_AS(2);
    else if (slices >= 4) TK_SSD_AS(4);
    else if (slices >= 2) TK_SSD_AS(8);
    else TK_SSD_AS(16);
#undef TK_SSD_AS
    return 0;
}

TK_API int tk_ssd_max_state() { return 32 * SSD_MAX_SLICES; }

// Into how many blocks a head's rows are split for a step of `tokens` tokens in `n_seqs` sequences: 1
// while the unsplit blocks fill the GPU or every sequence brings one token; else 2 or 4 (each block
// keeps four slices, i.e. four warps, at least), so that one long portion is walked by all of the GPU. y then has that
// many parts.
TK_API int tk_ssd_split(int tokens, int n_seqs, int H, int V, int N, int sm_count) {
    if (tokens <= n_seqs || N <= 0) return 1;
    const int R = N <= 8 * SSD_MAX_SLICES ? 8 : (N <= 16 * SSD_MAX_SLICES ? 16 : 32);
    const int slices = (N + R - 1) / R;
    const int blocks = (V + SSD_COLS - 1) / SSD_COLS * H * n_seqs;
    for (int split = 4; split > 1; split /= 2)
        if (slices % split == 0 && slices / split >= 4 && blocks * split <= 2 * sm_count) return split;
    return 1;
}

// xbc: [T, >= H V + 2 G N] rows `xbc_stride` apart (type dtype); dt_raw: float32 [T, >= H] rows `dt_stride`
// apart; dt_bias, A_log, D_skip: float32 [H]; state: float32 [slots, H, N, V]; y: float32 [T, H V];
// tokens: T, the rows of the step; split (tk_ssd_split): y is [split, T, H V], parts to be added up.
TK_API int tk_ssd_scan(const void* xbc, int64_t xbc_stride, const float* dt_raw, int64_t dt_stride,
                       const float* dt_bias, const float* A_log, const float* D_skip, float* state,
                       const int* cu_seqlens, const int* seq_ctx, const int* seq_slot, int n_seqs, int tokens,
                       float* y, int split, int H, int V, int N, int G, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(H > 0 && V > 0 && N > 0 && G > 0 && H % G == 0, "state-space scan: %d heads in %d groups", H, G);
    TK_CHECK_ARG(N <= tk_ssd_max_state(), "state-space scan: a state of %d rows; up to %d are built", N,
                 tk_ssd_max_state());
    TK_CHECK_ARG(n_seqs >= 0, "state-space scan: bad sizes");
    if (n_seqs == 0) return 0;
    const bool ahead = tokens > n_seqs;              // some sequence brings more than one token
    const int64_t y_part = (int64_t)tokens * H * V;
    {
        const int R = N <= 8 * SSD_MAX_SLICES ? 8 : (N <= 16 * SSD_MAX_SLICES ? 16 : 32);
        TK_CHECK_ARG(split >= 1 && ((N + R - 1) / R) % split == 0, "state-space scan: %d rows in %d parts", N, split);
    }
#define TK_SSD(TT)                                                                                                  \
    do {                                                                                                            \
        if (N <= 8 * SSD_MAX_SLICES)                                                                                \
            launch_ssd<TT, 8>(xbc, xbc_stride, dt_raw, dt_stride, dt_bias, A_log, D_skip, state, cu_seqlens,        \
                              seq_ctx, seq_slot, n_seqs, y, y_part, H, V, N, G, ahead, split, stream);              \
        else if (N <= 16 * SSD_MAX_SLICES)                                                                          \
            launch_ssd<TT, 16>(xbc, xbc_stride, dt_raw, dt_stride, dt_bias, A_log, D_skip, state, cu_seqlens,       \
                               seq_ctx, seq_slot, n_seqs, y, y_part, H, V, N, G, ahead, split, stream);             \
        else                                                                                                        \
            launch_ssd<TT, 32>(xbc, xbc_stride, dt_raw, dt_stride, dt_bias, A_log, D_skip, state, cu_seqlens,       \
                               seq_ctx, seq_slot, n_seqs, y, y_part, H, V, N, G, ahead, split, stream);             \
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
gated_group_norm_kernel(const float* y, int parts, const T* z, int64_t z_stride, const float* __restrict__ w, float eps,
                        T* out, int rows, int width, int groups) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (warp >= rows * groups) return;
    const int r = warp / groups, gw = width / groups, c0 = (warp % groups) * gw;
    auto at = [&](int i) {
        const float zv = to_f<T>(z[(size_t)r * z_stride + c0 + i]);
        float v = y[(size_t)r * width + c0 + i];
        for (int k = 1; k < parts; ++k) v += y[((size_t)k * rows + r) * width + c0 + i];
        return v * (zv / (1.0f + expf(-zv)));
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

// y: float32 [parts, rows, width], the parts to be added up; z: [rows, width] (type dtype) rows `z_stride` apart; w: float32 [width];
// out: [rows, width] (type dtype).
TK_API int tk_gated_group_norm(const float* y, int parts, const void* z, int64_t z_stride, const float* w, float eps, void* out,
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
            tk_launch(gated_group_norm_kernel<TT, 4>, grid, block, 0, stream, y, parts, (const TT*)z, z_stride, w, eps,  \
                      (TT*)out, rows, width, groups);                                                            \
        else if (gw <= 32 * 16)                                                                                  \
            tk_launch(gated_group_norm_kernel<TT, 16>, grid, block, 0, stream, y, parts, (const TT*)z, z_stride, w, eps, \
                      (TT*)out, rows, width, groups);                                                            \
        else                                                                                                     \
            tk_launch(gated_group_norm_kernel<TT, 0>, grid, block, 0, stream, y, parts, (const TT*)z, z_stride, w, eps,  \
                      (TT*)out, rows, width, groups);                                                            \
    } while (0)
    if (dtype == TK_F32) TK_GGN(float);
    else if (dtype == TK_BF16) TK_GGN(__nv_bfloat16);
    else TK_CHECK_ARG(false, "gated group norm: unknown dtype %d", dtype);
#undef TK_GGN
    TK_CHECK_LAUNCH("gated_group_norm");
    return 0;
}
