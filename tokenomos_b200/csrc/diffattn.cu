// Attention whose heads carry several score maps over the same values (differential attention):
//
//   write:    from the fused projection's rows [q | k | v] (q: H heads of `maps` parts of D columns; k: G heads
//             laid out likewise; v: G heads of V) the queries as the attention kernels take them and the
//             new keys and values into the paged cache, positions entering nowhere (no rotation).
//             A head's map m is an attention of its own whose score reads part m of the query and of the
//             key only. It is handed to the kernels as one query head of the key's full width with
//             zeros outside its part: q_out[t, h * maps + m] = [0 .. q[t, h, m] .. 0], so that
//             q_out . k = q[m] . k[m], against G key heads [k[0] | k[1] | ..] that are stored once.
//             maps == 1 is the plain copy: an encoding that does nothing to q and k.
//   combine:  o = a_1 - lambda a_2 per head (a_m: map m's output), o <- o / sqrt(mean(o^2) + eps) * coef.
//
// Storage float or bfloat16 (T); the combination and its statistics are 32-bit.
#include <math.h>

#include "common.cuh"

namespace {
enum : int { TK_K_QKV_MAPS = 12 };
}

template <typename T>
__global__ void __launch_bounds__(128)
qkv_maps_write_kernel(const T* qkv, int64_t stride, const int* positions, const int* tok_seq, const int* block_table,
                      int bt_stride, T* q_out, T* pool, int H, int G, int D, int V, int maps, int P, int Dp) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = qkv + (size_t)t * stride;
    const int DK = maps * D;                          // a key head's width, and an expanded query head's
    // queries: [H, maps, D] -> [H * maps, maps * D]
    T* qo = q_out + (size_t)t * H * maps * DK;
    for (int i = threadIdx.x; i < H * maps * DK; i += blockDim.x) {
        const int c = i % DK, hm = i / DK;
        const int m = hm % maps, h = hm / maps;
        const int part = c / D;
        qo[i] = part == m ? row[(size_t)(h * maps + m) * D + (c - m * D)] : from_f<T>(0.f);
    }
    if (pool == nullptr) return;
    const int pos = positions[t];
    const int page = TK_PAGE(TK_K_QKV_MAPS, block_table[(size_t)tok_seq[t] * bt_stride + pos / P]);
    // [page][K | V][head][slot in page][Dp]
    T* kd = pool + (((size_t)page * 2 + 0) * G * P + pos % P) * Dp;
    T* vd = pool + (((size_t)page * 2 + 1) * G * P + pos % P) * Dp;
    const T* k = row + (size_t)H * DK;
    const T* v = k + (size_t)G * DK;
    for (int i = threadIdx.x; i < G * DK; i += blockDim.x) kd[(size_t)(i / DK) * P * Dp + i % DK] = k[i];
    for (int i = threadIdx.x; i < G * V; i += blockDim.x) vd[(size_t)(i / V) * P * Dp + i % V] = v[i];
}

// The same, 16 bytes at a time: bfloat16 with D, V, the rows' distance and the cache row whole 16-byte
// chunks, so that a chunk of the expanded query lies wholly inside or outside its map's part.
__global__ void __launch_bounds__(128)
qkv_maps_write_vec_kernel(const __nv_bfloat16* qkv, int64_t stride, const int* positions, const int* tok_seq,
                          const int* block_table, int bt_stride, __nv_bfloat16* q_out, __nv_bfloat16* pool, int H, int G,
                          int D, int V, int maps, int P, int Dp) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const uint4* row = reinterpret_cast<const uint4*>(qkv + (size_t)t * stride);
    const int DK = maps * D, dk8 = DK / 8, d8 = D / 8, v8 = V / 8;
    uint4* qo = reinterpret_cast<uint4*>(q_out + (size_t)t * H * maps * DK);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x; i < H * maps * dk8; i += blockDim.x) {
        const int c = i % dk8, hm = i / dk8;
        const int m = hm % maps;
        qo[i] = c / d8 == m ? row[hm * d8 + (c - m * d8)] : zero;
    }
    if (pool == nullptr) return;
    const int pos = positions[t];
    const int page = TK_PAGE(TK_K_QKV_MAPS, block_table[(size_t)tok_seq[t] * bt_stride + pos / P]);
    uint4* kd = reinterpret_cast<uint4*>(pool + (((size_t)page * 2 + 0) * G * P + pos % P) * Dp);
    uint4* vd = reinterpret_cast<uint4*>(pool + (((size_t)page * 2 + 1) * G * P + pos % P) * Dp);
    const uint4* k = row + (size_t)H * dk8;
    const uint4* v = k + (size_t)G * dk8;
    const size_t head = (size_t)P * Dp / 8;
    for (int i = threadIdx.x; i < G * dk8; i += blockDim.x) kd[(size_t)(i / dk8) * head + i % dk8] = k[i];
    for (int i = threadIdx.x; i < G * v8; i += blockDim.x) vd[(size_t)(i / v8) * head + i % v8] = v[i];
}

// qkv: [T, >= (H + G) maps D + G V] rows `stride` apart; q_out: [T, H maps, maps D]; pool (null: the layer
// has no keys of its own): [pages, 2, G, P, Dp] with Dp >= max(maps D, V).
TK_API int tk_qkv_maps_write(const void* qkv, int64_t stride, const int* positions, const int* tok_seq,
                             const int* block_table, int bt_stride, void* q_out, void* pool, int tokens, int H, int G,
                             int D, int V, int maps, int P, int Dp, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && H > 0 && G >= 0 && D > 0 && V > 0 && maps >= 1, "qkv_maps_write: bad sizes");
    TK_CHECK_ARG(pool == nullptr || (block_table != nullptr && P > 0 && G > 0 && Dp >= maps * D && Dp >= V),
                 "qkv_maps_write: cache rows of %d for keys of %d and values of %d", Dp, maps * D, V);
    if (tokens == 0) return 0;
    if (dtype == TK_BF16 && D % 8 == 0 && V % 8 == 0 && stride % 8 == 0 && (pool == nullptr || Dp % 8 == 0) &&
        ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)pool & 15) == 0) {
        tk_launch(qkv_maps_write_vec_kernel, dim3(tokens), dim3(128), 0, stream, (const __nv_bfloat16*)qkv, stride, positions,
                  tok_seq, block_table, bt_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, H, G, D, V, maps, P, Dp);
        TK_CHECK_LAUNCH("qkv_maps_write_vec");
        return 0;
    }
    if (dtype == TK_F32)
        tk_launch(qkv_maps_write_kernel<float>, dim3(tokens), dim3(128), 0, stream, (const float*)qkv, stride, positions,
                  tok_seq, block_table, bt_stride, (float*)q_out, (float*)pool, H, G, D, V, maps, P, Dp);
    else if (dtype == TK_BF16)
        tk_launch(qkv_maps_write_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, (const __nv_bfloat16*)qkv,
                  stride, positions, tok_seq, block_table, bt_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pool, H, G,
                  D, V, maps, P, Dp);
    else
        TK_CHECK_ARG(false, "qkv_maps_write: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("qkv_maps_write");
    return 0;
}

// One warp per (token, head); a lane keeps its V / 32 values of o in registers.
template <typename T, int ITEMS>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const T* a, T* out, int rows, int V, float lambda, float coef, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const T* a1 = a + (size_t)warp * 2 * V;
    const T* a2 = a1 + V;
    float keep[ITEMS], ss = 0.f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
        const int i = lane + 32 * k;
        keep[k] = i < V ? fmaf(-lambda, to_f<T>(a2[i]), to_f<T>(a1[i])) : 0.f;
        ss += keep[k] * keep[k];
    }
    const float rstd = coef / sqrtf(warp_sum(ss) / (float)V + eps);
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
        const int i = lane + 32 * k;
        if (i < V) out[(size_t)warp * V + i] = from_f<T>(keep[k] * rstd);
    }
}

// a: [rows, 2, V] (a row is a (token, head); its two maps' outputs side by side); out: [rows, V].
TK_API int tk_diff_combine(const void* a, void* out, int rows, int V, float lambda, float coef, float eps, int dtype,
                           cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && V > 0 && V <= 256, "diff_combine: values of %d; up to 256 are built", V);
    if (rows == 0) return 0;
    dim3 grid((rows + 3) / 4), block(128);
#define TK_DC(TT, N)                                                                                              \
    tk_launch(diff_combine_kernel<TT, N>, grid, block, 0, stream, (const TT*)a, (TT*)out, rows, V, lambda, coef, eps)
    if (dtype == TK_F32) {
        if (V <= 128) TK_DC(float, 4);
        else TK_DC(float, 8);
    } else if (dtype == TK_BF16) {
        if (V <= 128) TK_DC(__nv_bfloat16, 4);
        else TK_DC(__nv_bfloat16, 8);
    } else {
        TK_CHECK_ARG(false, "diff_combine: unknown dtype %d", dtype);
    }
#undef TK_DC
    TK_CHECK_LAUNCH("diff_combine");
    return 0;
}
