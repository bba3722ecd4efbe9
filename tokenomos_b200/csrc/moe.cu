// Mixture of experts: routing, the sort of (token, expert) pairs into per-expert row blocks, a
// grouped / batched matrix product on the CUDA cores, and the weighted combination.
//
//   route:   s = softmax(z[0:E]) (32-bit); the `top` largest (ties: the lowest index);
//            w_k = s_k / (sum of the chosen s + 1e-20) * scale;  gate = sigmoid(z[E]) if the row has one
//   sort:    pairs (token, k) grouped by expert, every expert's block padded to whole tiles of
//            `tile` rows, so that a tile of the product belongs to one expert
//   product: C[m, :] = act(A[row(m), :] . W[g]^T), g the group of m's tile (or the batch index)
//   combine: out[t] = sum_k w[t, k] * Y[row of (t, k)] + gate[t] * shared[t]
#include <math.h>

#include "common.cuh"

namespace {
constexpr int ROUTE_WARPS = 4;
constexpr int MAX_TOP = 32;
constexpr int TM = 64, TN = 64, TKK = 16, GEMM_THREADS = 256;
}  // namespace

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float* logits, int64_t ld, int tokens, int E, int top, float scale, int has_gate,
                 int* idx_out, float* w_out, float* gate_out) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= tokens) return;
    float* z = smem + (size_t)warp * E;
    const float* row = logits + (size_t)t * ld;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) {
        const float v = row[e];
        z[e] = v;
        mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    if (!(mx > -INFINITY)) mx = 0.f;                // a row without a finite value (padding of a recorded step)
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float p = expf(z[e] - mx);
        z[e] = p;
        sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    float chosen_sum = 0.f;
    float my_w = 0.f;                               // lane k keeps the k-th chosen score
    int my_e = 0;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best) { best = v; at = e; }     // ascending e: the lowest index of equal values stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at == 0x7fffffff) { at = k < E ? k : 0; best = 0.f; }    // nothing comparable: stay inside the table
        if (lane == 0) z[at] = -INFINITY;
        __syncwarp();
        const float s = best / sum;
        chosen_sum += s;
        if (lane == (k & 31)) { my_w = s; my_e = at; }
    }
    if (lane < top) {
        idx_out[(size_t)t * top + lane] = my_e;
        w_out[(size_t)t * top + lane] = my_w / (chosen_sum + 1e-20f) * scale;
    }
    if (has_gate && lane == 0) gate_out[t] = 1.0f / (1.0f + expf(-row[E]));
}

TK_API int tk_moe_route(const float* logits, int64_t ld, int tokens, int E, int top, float scale, int has_gate,
                        int* idx_out, float* w_out, float* gate_out, cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && E > 0 && top > 0 && top <= E && top <= MAX_TOP, "moe_route: %d of %d experts (at most %d)",
                 top, E, MAX_TOP);
    TK_CHECK_ARG((size_t)E * ROUTE_WARPS * 4 <= 48 * 1024, "moe_route: %d experts do not fit shared memory", E);
    TK_CHECK_ARG(ld >= E + (has_gate ? 1 : 0), "moe_route: rows of %lld for %d experts", (long long)ld, E);
    if (tokens == 0) return 0;
    tk_launch(moe_route_kernel, dim3((tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32),
              (size_t)E * ROUTE_WARPS * sizeof(float), stream, logits, ld, tokens, E, top, scale, has_gate, idx_out,
              w_out, gate_out);
    TK_CHECK_LAUNCH("moe_route");
    return 0;
}

// One block. row_token[cap_rows]: the token whose input a row of the sorted layout reads (-1:
// padding); pair_row[pairs]: where pair (token * top + k) sits; tile_expert[cap_rows / tile]: the
// expert of each tile (-1: unused); expert_end[E] (optional): the row after each expert's block.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* idx, int pairs, int top, int E, int tile, int cap_rows, int* row_token, int* pair_row,
                int* tile_expert, int* expert_end) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int ism[];
    int* count = ism;
    int* start = ism + E;
    int* cursor = ism + 2 * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0, cursor[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&count[idx[p]], 1);
    for (int r = threadIdx.x; r < cap_rows; r += blockDim.x) row_token[r] = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at;
            const int tiles = (count[e] + tile - 1) / tile;
            for (int k = 0; k < tiles; ++k) tile_expert[at / tile + k] = e;
            at += tiles * tile;
            if (expert_end != nullptr) expert_end[e] = at;      // where the expert's padded block ends
        }
        for (int k = at / tile; k < cap_rows / tile; ++k) tile_expert[k] = -1;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = idx[p];
        const int r = start[e] + atomicAdd(&cursor[e], 1);
        row_token[r] = p / top;
        pair_row[p] = r;
    }
}

TK_API int tk_moe_sort(const int* idx, int pairs, int top, int E, int tile, int cap_rows, int* row_token,
                       int* pair_row, int* tile_expert, int* expert_end, cudaStream_t stream) {
    TK_CHECK_ARG(pairs >= 0 && top > 0 && E > 0 && tile > 0, "moe_sort: bad sizes");
    TK_CHECK_ARG(cap_rows % tile == 0 && cap_rows >= pairs + (E < pairs ? E : pairs) * (tile - 1),
                 "moe_sort: %d rows cannot hold %d pairs of %d experts in tiles of %d", cap_rows, pairs, E, tile);
    TK_CHECK_ARG((size_t)E * 12 <= 48 * 1024, "moe_sort: %d experts do not fit shared memory", E);
    if (pairs == 0) return 0;
    tk_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int), stream, idx, pairs, top, E, tile,
              cap_rows, row_token, pair_row, tile_expert, expert_end);
    TK_CHECK_LAUNCH("moe_sort");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// C[m, n] = act(sum_k A[row(m), k] * W[g][n, k]) on the CUDA cores, 32-bit FMA accumulation.
// Grouped (tile_group given): m runs over the sorted layout, the group of a 64-row tile is
// tile_group[tile] (-1: nothing to do), row(m) = row_index[m] if given (-1: a row of zeros).
// Batched (no tile_group): blockIdx.z is the group; A, W and C advance by their group strides.
// act 1: relu(v)^2.
// ---------------------------------------------------------------------------------------------
template <typename TA, typename TO>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_grouped_simt_kernel(const TA* A, int64_t lda, int64_t a_gs, const int* row_index,
                         const TA* __restrict__ W, int64_t ldw, int64_t w_gs, const int* tile_group, TO* C,
                         int64_t ldc, int64_t c_gs, int M, int N, int K, int act) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float As[TKK][TM + 4];
    __shared__ float Ws[TKK][TN + 4];
    __shared__ int rows_s[TM];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    if (tile_group != nullptr) {
        const int g = tile_group[blockIdx.y];
        if (g < 0) return;
        W += (size_t)g * w_gs;
    } else {
        A += (size_t)blockIdx.z * a_gs;
        W += (size_t)blockIdx.z * w_gs;
        C += (size_t)blockIdx.z * c_gs;
    }
    if (tid < TM) {
        const int m = m0 + tid;
        rows_s[tid] = m < M ? (row_index != nullptr ? row_index[m] : m) : -1;
    }
    __syncthreads();
    const int tx = tid & 15, ty = tid >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const int arow = rows_s[lr];
    for (int k0 = 0; k0 < K; k0 += TKK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int n = n0 + lr;
            As[lk + e][lr] = (arow >= 0 && k < K) ? to_f<TA>(A[(size_t)arow * lda + k]) : 0.f;
            Ws[lk + e][lr] = (n < N && k < K) ? to_f<TA>(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TKK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (act == 1) { v = fmaxf(v, 0.f); v *= v; }
            C[(size_t)m * ldc + n] = from_f<TO>(v);
        }
    }
}

TK_API int tk_gemm_grouped_tile() { return TM; }

TK_API int tk_gemm_grouped_simt(const void* A, int64_t lda, int64_t a_gs, const int* row_index, const void* W,
                                int64_t ldw, int64_t w_gs, const int* tile_group, void* C, int64_t ldc,
                                int64_t c_gs, int M, int N, int K, int groups, int act, int dtype,
                                cudaStream_t stream) {
    TK_CHECK_ARG(M >= 0 && N > 0 && K > 0 && groups >= 1, "gemm_grouped: bad sizes M=%d N=%d K=%d", M, N, K);
    TK_CHECK_ARG(ldw >= K && ldc >= N, "gemm_grouped: leading dimensions too small");
    TK_CHECK_ARG(act == 0 || act == 1, "gemm_grouped: activation %d", act);
    if (M == 0) return 0;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, tile_group != nullptr ? 1 : groups);
    if (dtype == TK_F32)
        tk_launch(gemm_grouped_simt_kernel<float, float>, grid, dim3(GEMM_THREADS), 0, stream, (const float*)A, lda,
                  a_gs, row_index, (const float*)W, ldw, w_gs, tile_group, (float*)C, ldc, c_gs, M, N, K, act);
    else if (dtype == TK_BF16)
        tk_launch(gemm_grouped_simt_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(GEMM_THREADS), 0, stream,
                  (const __nv_bfloat16*)A, lda, a_gs, row_index, (const __nv_bfloat16*)W, ldw, w_gs, tile_group,
                  (__nv_bfloat16*)C, ldc, c_gs, M, N, K, act);
    else
        TK_CHECK_ARG(false, "gemm_grouped: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("gemm_grouped_simt");
    return 0;
}

// out[t] = sum_k w[t, k] * Y[pair_row[t * top + k]] + gate[t] * shared[t]   (32-bit sum, one rounding)
template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const T* Y, const int* pair_row, const float* w, const T* shared, const float* gate, T* out,
                   int top, int width) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ int rows[MAX_TOP];
    __shared__ float ws[MAX_TOP];
    const size_t t = blockIdx.x;
    if (threadIdx.x < top) {
        rows[threadIdx.x] = pair_row[t * top + threadIdx.x];
        ws[threadIdx.x] = w[t * top + threadIdx.x];
    }
    __syncthreads();
    const float g = shared != nullptr ? (gate != nullptr ? gate[t] : 1.f) : 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < top; ++k) v = fmaf(ws[k], to_f<T>(Y[(size_t)rows[k] * width + i]), v);
        if (shared != nullptr) v = fmaf(g, to_f<T>(shared[t * width + i]), v);
        out[t * width + i] = from_f<T>(v);
    }
}

TK_API int tk_moe_combine(const void* Y, const int* pair_row, const float* w, const void* shared,
                          const float* gate, void* out, int tokens, int top, int width, int dtype,
                          cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && top > 0 && top <= MAX_TOP && width > 0, "moe_combine: bad sizes");
    if (tokens == 0) return 0;
    if (dtype == TK_F32)
        tk_launch(moe_combine_kernel<float>, dim3(tokens), dim3(256), 0, stream, (const float*)Y, pair_row, w,
                  (const float*)shared, gate, (float*)out, top, width);
    else if (dtype == TK_BF16)
        tk_launch(moe_combine_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), 0, stream, (const __nv_bfloat16*)Y,
                  pair_row, w, (const __nv_bfloat16*)shared, gate, (__nv_bfloat16*)out, top, width);
    else
        TK_CHECK_ARG(false, "moe_combine: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("moe_combine");
    return 0;
}

// x = relu(x)^2 in place
template <typename T>
__global__ void relu2_kernel(T* x, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f<T>(x[i]), 0.f);
        x[i] = from_f<T>(v * v);
    }
}

TK_API int tk_relu2(void* x, int64_t n, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(n >= 0, "relu2: bad size");
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (dtype == TK_F32) tk_launch(relu2_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, (size_t)n);
    else if (dtype == TK_BF16)
        tk_launch(relu2_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, (size_t)n);
    else TK_CHECK_ARG(false, "relu2: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("relu2");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// The same product on the tensor cores for bfloat16: mma.sync m16n8k16, 32-bit accumulation, a
// 64 x 128 tile per CTA (8 warps of 32 x 32), K in steps of 32 through a three-stage cp.async
// pipeline, operands read with ldmatrix from rows padded to 80 bytes. Gathered rows (a row index
// of -1, rows beyond M, columns beyond N or K) are zero-filled by the copy itself. Needs K and N
// in whole 16-byte chunks and 16-byte aligned rows.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int GK = 32, GLD = 40, G_THREADS = 256;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
}  // namespace

// GM: rows of a tile (64: 8 warps of 32 x 32; 128: 8 warps of 64 x 32); GSTAGES: copies in flight.
// gate (batched form only): C[g][m][:] *= sigmoid(gate[m * gate_stride + g]).
// act 1: relu(v)^2. act 2: the weight's rows are gates and ups alternating in runs of 8; C has N / 2
// columns, silu(gate) * up.
// GN: columns of a tile (128, or 64 for steps of a few rows: twice the CTAs to stream the weights).
template <int GM, int GSTAGES, int GN>
__global__ void __launch_bounds__(G_THREADS)
gemm_grouped_mma_kernel(const __nv_bfloat16* A, int64_t lda, int64_t a_gs, const int* row_index,
                        const __nv_bfloat16* __restrict__ W, int64_t ldw, int64_t w_gs, const int* tile_group,
                        __nv_bfloat16* C, int64_t ldc, int64_t c_gs, int M, int N, int K, int act,
                        const __nv_bfloat16* gate, int64_t gate_stride) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char gsm[];
    __nv_bfloat16 (*As)[GM * GLD] = reinterpret_cast<__nv_bfloat16 (*)[GM * GLD]>(gsm);
    __nv_bfloat16 (*Ws)[GN * GLD] = reinterpret_cast<__nv_bfloat16 (*)[GN * GLD]>(gsm + (size_t)GSTAGES * GM * GLD * 2);
    __shared__ int rows_s[GM];
    constexpr int MI = GM / 32;              // m16 blocks of a warp's tile
    constexpr int NJ = GN / 32;              // n8 blocks of a warp's tile (its columns: GN / 4)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
    if (tile_group != nullptr) {
        const int g = tile_group[blockIdx.y];
        if (g < 0) return;
        W += (size_t)g * w_gs;
    } else {
        A += (size_t)blockIdx.z * a_gs;
        W += (size_t)blockIdx.z * w_gs;
        C += (size_t)blockIdx.z * c_gs;
    }
    if (tid < GM) {
        const int m = m0 + tid;
        rows_s[tid] = m < M ? (row_index != nullptr ? row_index[m] : m) : -1;
    }
    __syncthreads();
    const int a_chunk = (tid & 3) * 8;          // 16-byte chunks: 4 a row, rows 64 apart per thread
    int a_src[GM / 64];
#pragma unroll
    for (int i = 0; i < GM / 64; ++i) a_src[i] = rows_s[(tid >> 2) + i * 64];
    const int gz = tile_group != nullptr ? 0 : blockIdx.z;
    const int ktiles = (K + GK - 1) / GK;
    auto load = [&](int kt, int stage) {
        const int k = kt * GK + a_chunk;
#pragma unroll
        for (int i = 0; i < GM / 64; ++i) {
            const bool av = a_src[i] >= 0 && k < K;
            cp_async16(&As[stage][((tid >> 2) + i * 64) * GLD + a_chunk],
                       av ? (const void*)(A + (size_t)a_src[i] * lda + k) : (const void*)A, av);
        }
#pragma unroll
        for (int i = 0; i < GN / 64; ++i) {
            const int r = (tid >> 2) + i * 64;
            const int n = n0 + r;
            const bool wv = n < N && k < K;
            cp_async16(&Ws[stage][r * GLD + a_chunk], wv ? (const void*)(W + (size_t)n * ldw + k) : (const void*)W, wv);
        }
    };
    for (int s = 0; s < GSTAGES - 1; ++s) {
        if (s < ktiles) load(s, s);
        cp_async_commit();
    }
    const int wm = (warp >> 2) * (GM / 2), wn = (warp & 3) * (GN / 4);
    float acc[MI][NJ][4];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NJ; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
    for (int kt = 0; kt < ktiles; ++kt) {
        cp_async_wait<GSTAGES - 2>();
        __syncthreads();
        if (kt + GSTAGES - 1 < ktiles) load(kt + GSTAGES - 1, (kt + GSTAGES - 1) % GSTAGES);
        cp_async_commit();
        const __nv_bfloat16* as = As[kt % GSTAGES];
        const __nv_bfloat16* ws = Ws[kt % GSTAGES];
#pragma unroll
        for (int kk = 0; kk < GK; kk += 16) {
            unsigned a[MI][4], b[NJ / 2][4];
#pragma unroll
            for (int i = 0; i < MI; ++i)
                ldmatrix_x4(a[i], as + (wm + i * 16 + (lane & 15)) * GLD + kk + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < NJ / 2; ++j)
                ldmatrix_x4(b[j], ws + (wn + j * 16 + (lane & 7) + (lane >> 4) * 8) * GLD + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int i = 0; i < MI; ++i)
#pragma unroll
                for (int j = 0; j < NJ; ++j) mma_bf16(acc[i][j], a[i], b[j >> 1][(j & 1) * 2], b[j >> 1][(j & 1) * 2 + 1]);
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < MI; ++i) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = m0 + wm + i * 16 + (lane >> 2) + half * 8;
            if (m >= M) continue;
            const float gv = gate != nullptr ? 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)m * gate_stride + gz]))) : 1.0f;
            if (act == 2) {
                // gate and up rows of the weight alternate in runs of 8: a warp's n8 blocks 2 jj and
                // 2 jj + 1 are the gates and the ups of the same eight units, in the same lanes.
                // Both are rounded to the storage type first, as a product that is stored would be.
#pragma unroll
                for (int jj = 0; jj < NJ / 2; ++jj) {
                    const int n = n0 + wn + jj * 16 + (lane & 3) * 2;
                    if (n >= N) continue;
                    float y[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float g = __bfloat162float(__float2bfloat16_rn(acc[i][2 * jj][half * 2 + e]));
                        const float u = __bfloat162float(__float2bfloat16_rn(acc[i][2 * jj + 1][half * 2 + e]));
                        y[e] = g / (1.f + expf(-g)) * u * gv;
                    }
                    *reinterpret_cast<__nv_bfloat162*>(C + (size_t)m * ldc + (n >> 4) * 8 + (lane & 3) * 2) =
                        __floats2bfloat162_rn(y[0], y[1]);
                }
                continue;
            }
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int n = n0 + wn + j * 8 + (lane & 3) * 2;
                if (n >= N) continue;
                float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
                if (act == 1) {
                    v0 = fmaxf(v0, 0.f); v0 *= v0;
                    v1 = fmaxf(v1, 0.f); v1 *= v1;
                }
                *reinterpret_cast<__nv_bfloat162*>(C + (size_t)m * ldc + n) = __floats2bfloat162_rn(v0 * gv, v1 * gv);
            }
        }
    }
}

TK_API int tk_gemm_grouped_mma(const void* A, int64_t lda, int64_t a_gs, const int* row_index, const void* W,
                               int64_t ldw, int64_t w_gs, const int* tile_group, void* C, int64_t ldc,
                               int64_t c_gs, int M, int N, int K, int groups, int act, int tile_rows,
                               const void* gate, int64_t gate_stride, cudaStream_t stream) {
    TK_CHECK_ARG(M >= 0 && N > 0 && K > 0 && groups >= 1, "gemm_grouped_mma: bad sizes M=%d N=%d K=%d", M, N, K);
    TK_CHECK_ARG(tile_rows == 64 || tile_rows == 128, "gemm_grouped_mma: tiles of %d rows; 64 or 128", tile_rows);
    TK_CHECK_ARG(gate == nullptr || tile_group == nullptr, "gemm_grouped_mma: the row gate belongs to the batched form");
    TK_CHECK_ARG(K % 8 == 0 && N % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && ldc % 2 == 0 && a_gs % 8 == 0 &&
                     w_gs % 8 == 0 && c_gs % 2 == 0,
                 "gemm_grouped_mma: K, N and the strides must be whole 16-byte chunks");
    TK_CHECK_ARG(((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0 && ((uintptr_t)C % 4) == 0,
                 "gemm_grouped_mma: operands must be 16-byte aligned");
    TK_CHECK_ARG(act == 0 || act == 1 || (act == 2 && N % 16 == 0), "gemm_grouped_mma: activation %d with %d columns", act, N);
    if (M == 0) return 0;
    // few row tiles (a step of a few tokens streams the weights): columns in tiles of 64, so that
    // twice as many CTAs share the stream and an SM holds four of them
    const int m_tiles = (M + tile_rows - 1) / tile_rows;
    const int groups_z = tile_group != nullptr ? 1 : groups;
    const bool narrow = tile_rows == 64 && (long long)m_tiles * groups_z * ((N + 127) / 128) <= 2 * 148;
    const int gn = narrow ? 64 : 128;
    dim3 grid((N + gn - 1) / gn, m_tiles, groups_z);
#define TK_GG(GMV, ST, GNV)                                                                                         \
    do {                                                                                                            \
        const size_t smem = (size_t)ST * (GMV + GNV) * GLD * 2;                                                     \
        cudaFuncSetAttribute(gemm_grouped_mma_kernel<GMV, ST, GNV>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                             (int)smem);                                                                            \
        tk_launch(gemm_grouped_mma_kernel<GMV, ST, GNV>, grid, dim3(G_THREADS), smem, stream,                       \
                  (const __nv_bfloat16*)A, lda, a_gs, row_index, (const __nv_bfloat16*)W, ldw, w_gs, tile_group,    \
                  (__nv_bfloat16*)C, ldc, c_gs, M, N, K, act, (const __nv_bfloat16*)gate, gate_stride);             \
    } while (0)
    if (narrow) TK_GG(64, 6, 64);
    else if (tile_rows == 64) TK_GG(64, 5, 128);
    else TK_GG(128, 4, 128);
#undef TK_GG
    TK_CHECK_LAUNCH("gemm_grouped_mma");
    return 0;
}

// out[r] = index[r] >= 0 ? table[index[r]] : 0  (bfloat16 or float rows): the experts' input rows in
// the sorted layout, for a product that cannot gather by itself
template <typename T>
__global__ void gather_rows_or_zero_kernel(const T* table, const int* index, T* out, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = index[r];
    T* dst = out + (size_t)r * width;
    constexpr int VEC = 16 / sizeof(T);
    if (width % VEC == 0) {
        const uint4* s4 = src >= 0 ? reinterpret_cast<const uint4*>(table + (size_t)src * width) : nullptr;
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < width / VEC; i += blockDim.x) d4[i] = s4 != nullptr ? s4[i] : make_uint4(0, 0, 0, 0);
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src >= 0 ? table[(size_t)src * width + i] : from_f<T>(0.f);
    }
}

TK_API int tk_gather_rows_or_zero(const void* table, const int* index, void* out, int rows, int width, int dtype,
                                  cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && width > 0, "gather_rows_or_zero: bad sizes");
    if (rows == 0) return 0;
    if (dtype == TK_F32)
        tk_launch(gather_rows_or_zero_kernel<float>, dim3(rows), dim3(128), 0, stream, (const float*)table, index,
                  (float*)out, width);
    else if (dtype == TK_BF16)
        tk_launch(gather_rows_or_zero_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, stream,
                  (const __nv_bfloat16*)table, index, (__nv_bfloat16*)out, width);
    else
        TK_CHECK_ARG(false, "gather_rows_or_zero: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("gather_rows_or_zero");
    return 0;
}
