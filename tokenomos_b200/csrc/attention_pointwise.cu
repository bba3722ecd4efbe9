// Paged attention whose weights are not a softmax: every visible key gets a weight of its own,
//
//     s_ij = (q_i . k_j) * scale * temp(i)            temp(i) = 1 + coef * ln(floor((i + 1) / every) + 1)
//     s_ij <- cap * tanh(s_ij / cap)                  (cap > 0)
//     s_ij <- s_ij - r1[h] * ln(1 + r2[h] * (i - j))  (a bias by distance, per head)
//     w_ij = sigmoid(s_ij + b[h])                     (not normalised over the keys)
//     o_i  = sum_{j <= i, visible} w_ij v_j
//
// Every option is a parameter (coef 0 or every 0: no temperature; cap 0: none; r1 null: no distance
// bias; b null: 0). Scores, weights and sums are 32-bit whatever the storage type. The tile
// scheme is the generic softmax kernel's: one block takes a tile of rows that share a KV head, the
// rows being (token, query head in the group) pairs; every key is read from the cache, the step's
// own included. This form runs on the CUDA cores and takes any head sizes; the tensor-core form
// for bfloat16 is below it.
#include <math.h>

#include "common.cuh"

namespace {
enum : int { TK_K_ATTN_POINT = 9 };
constexpr int BM = 16;       // rows per block
constexpr int BN = 32;       // keys per iteration
constexpr int THREADS = 128; // 8 threads per row
constexpr int MAX_D = 256;

struct PointOptions {
    float scale, cap, temp_coef;
    int temp_every;
    const float* r1;     // [H] or null
    const float* r2;
    const float* head_bias;
    int window;
};

__device__ __forceinline__ float temperature(const PointOptions& o, int pos) {
    if (o.temp_every <= 0 || o.temp_coef == 0.f) return 1.f;
    return 1.f + o.temp_coef * logf((float)((pos + 1) / o.temp_every) + 1.f);
}

// the weight of key j for a query at position i of head parameters (a1, a2, hb), from the raw dot
__device__ __forceinline__ float point_weight(float dot, float row_scale, float cap, float inv_cap, bool has_r,
                                              float a1, float a2, float hb, int dist) {
    float s = dot * row_scale;
    if (cap > 0.f) s = cap * tanhf(s * inv_cap);
    if (has_r) s -= a1 * log1pf(a2 * (float)dist);
    s += hb;
    return 1.f / (1.f + expf(-s));
}
}  // namespace

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_pointwise_kernel(const T* q, const T* kv_pool, T* out, const int* positions, const int* tok_seq,
                      const int* block_table, int bt_stride, const int* tile_tok0, const int* tile_ntok, int H,
                      int Hkv, int D, int Dv, int Dp, int P, PointOptions opt, int heads_per_chunk) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int DP = D + 1;
    float* Qs = smem;                 // [BM][D+1]
    float* Ks = Qs + BM * DP;         // [BN][D+1]
    float* Vs = Ks + BN * DP;         // [BN][Dv]
    float* Ss = Vs + BN * Dv;         // [BM][BN+1]
    __shared__ int row_pos[BM];

    const int G = H / Hkv;
    const int chunks = (G + heads_per_chunk - 1) / heads_per_chunk;
    const int kvh = blockIdx.y / chunks;
    const int chunk = blockIdx.y % chunks;
    const int g0 = chunk * heads_per_chunk;
    const int gh = min(heads_per_chunk, G - g0);
    const int tok0 = tile_tok0[blockIdx.x];
    const int ntok = tile_ntok[blockIdx.x];
    if (ntok <= 0) return;
    const int rows = ntok * gh;
    const int seq = tok_seq[tok0];
    const int tid = threadIdx.x;

    for (int i = tid; i < BM * D; i += THREADS) {
        const int r = i / D, c = i % D;
        float v = 0.f;
        if (r < rows) {
            const int t = tok0 + r / gh, h = kvh * G + g0 + r % gh;
            v = to_f<T>(q[((size_t)t * H + h) * D + c]);
        }
        Qs[r * DP + c] = v;
    }
    if (tid < BM) row_pos[tid] = tid < rows ? positions[tok0 + tid / gh] : -1;
    __syncthreads();

    const int pos_first = row_pos[0];
    const int pos_last = row_pos[rows - 1];
    const int lo = opt.window > 0 ? max(0, pos_first - opt.window + 1) : 0;
    const int r = tid >> 3, sub = tid & 7;
    const int my_pos = row_pos[r];
    const int my_head = kvh * G + g0 + (r < rows ? r % gh : 0);
    const bool has_r = opt.r1 != nullptr;
    const float a1 = has_r ? opt.r1[my_head] : 0.f, a2 = has_r ? opt.r2[my_head] : 0.f;
    const float hb = opt.head_bias != nullptr ? opt.head_bias[my_head] : 0.f;
    const float row_scale = opt.scale * temperature(opt, max(my_pos, 0));
    const float inv_cap = opt.cap > 0.f ? 1.f / opt.cap : 0.f;
    float acc[MAX_D / 8];
#pragma unroll
    for (int k = 0; k < MAX_D / 8; ++k) acc[k] = 0.f;

    const int n_it = (pos_last - lo) / BN + 1;
    for (int it = 0; it < n_it; ++it) {
        const int j0 = lo + it * BN;
        {
            const int kk = tid >> 2, part = tid & 3;
            const int j = j0 + kk;
            if (j <= pos_last) {
                const int page = TK_PAGE(TK_K_ATTN_POINT, block_table[(size_t)seq * bt_stride + j / P]);
                const size_t base = ((size_t)page * 2 * Hkv * P + (size_t)kvh * P + (j % P)) * Dp;
                const size_t vbase = base + (size_t)Hkv * P * Dp;
                for (int c = part; c < D; c += 4) Ks[kk * DP + c] = to_f<T>(kv_pool[base + c]);
                for (int c = part; c < Dv; c += 4) Vs[kk * Dv + c] = to_f<T>(kv_pool[vbase + c]);
            } else {
                for (int c = part; c < D; c += 4) Ks[kk * DP + c] = 0.f;
                for (int c = part; c < Dv; c += 4) Vs[kk * Dv + c] = 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int kk = sub + 8 * jj;
            const int j = j0 + kk;
            float d = 0.f;
            const float* qr = Qs + r * DP;
            const float* kr = Ks + kk * DP;
            for (int c = 0; c < D; ++c) d += qr[c] * kr[c];
            const bool visible = my_pos >= 0 && j <= my_pos && (opt.window <= 0 || my_pos - j < opt.window);
            Ss[r * (BN + 1) + kk] = visible ? point_weight(d, row_scale, opt.cap, inv_cap, has_r, a1, a2, hb, my_pos - j)
                                            : 0.f;
        }
        __syncthreads();
        const float* pr = Ss + r * (BN + 1);
#pragma unroll
        for (int k = 0; k < MAX_D / 8; ++k) {
            const int c = sub + 8 * k;
            if (c < Dv) {
                float a = acc[k];
                for (int kk = 0; kk < BN; ++kk) a = fmaf(pr[kk], Vs[kk * Dv + c], a);
                acc[k] = a;
            }
        }
        __syncthreads();
    }
    if (r < rows) {
        const int t = tok0 + r / gh;
#pragma unroll
        for (int k = 0; k < MAX_D / 8; ++k) {
            const int c = sub + 8 * k;
            if (c < Dv) out[((size_t)t * H + my_head) * Dv + c] = from_f<T>(acc[k]);
        }
    }
}

TK_API int tk_attn_pointwise_rows() { return BM; }

// q: [T, H, D]; out: [T, H, Dv]; kv_pool: [pages, 2, Hkv, P, Dp]; tiles: first token and token count
// of each tile (tokens of one sequence, consecutive positions); window <= 0: none.
TK_API int tk_attn_pointwise(const void* q, const void* kv_pool, void* out, const int* positions,
                             const int* tok_seq, const int* block_table, int bt_stride, const int* tile_tok0,
                             const int* tile_ntok, int n_tiles, int tokens_per_tile, int H, int Hkv, int D, int Dv,
                             int Dp, int P, int window, float scale, float cap, float temp_coef, int temp_every,
                             const float* r1, const float* r2, const float* head_bias, int dtype,
                             cudaStream_t stream) {
    TK_CHECK_ARG(H > 0 && Hkv > 0 && H % Hkv == 0, "attention: %d query heads over %d KV heads", H, Hkv);
    TK_CHECK_ARG(D > 0 && D <= MAX_D && Dv > 0 && Dv <= MAX_D, "attention: head sizes %d / %d outside 1..%d", D, Dv, MAX_D);
    TK_CHECK_ARG(Dp >= D && Dp >= Dv, "attention: cache rows of %d for heads of %d and %d", Dp, D, Dv);
    TK_CHECK_ARG((r1 == nullptr) == (r2 == nullptr), "attention: the distance bias has two numbers per head");
    TK_CHECK_ARG(P > 0 && n_tiles >= 0 && cap >= 0.f, "attention: bad page size, tile count or cap");
    if (n_tiles == 0) return 0;
    const int G = H / Hkv;
    TK_CHECK_ARG(tokens_per_tile >= 1 && tokens_per_tile <= BM, "attention: %d tokens per tile", tokens_per_tile);
    const int heads_per_chunk = min(G, BM / tokens_per_tile);
    const int chunks = (G + heads_per_chunk - 1) / heads_per_chunk;
    const size_t smem = ((size_t)BM * (D + 1) + (size_t)BN * (D + 1) + (size_t)BN * Dv + (size_t)BM * (BN + 1)) * sizeof(float);
    PointOptions opt{scale, cap, temp_coef, temp_every, r1, r2, head_bias, window};
    dim3 grid(n_tiles, Hkv * chunks);
    if (dtype == TK_F32) {
        cudaFuncSetAttribute(attn_pointwise_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(attn_pointwise_kernel<float>, grid, dim3(THREADS), smem, stream, (const float*)q,
                  (const float*)kv_pool, (float*)out, positions, tok_seq, block_table, bt_stride, tile_tok0,
                  tile_ntok, H, Hkv, D, Dv, Dp, P, opt, heads_per_chunk);
    } else if (dtype == TK_BF16) {
        cudaFuncSetAttribute(attn_pointwise_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tk_launch(attn_pointwise_kernel<__nv_bfloat16>, grid, dim3(THREADS), smem, stream, (const __nv_bfloat16*)q,
                  (const __nv_bfloat16*)kv_pool, (__nv_bfloat16*)out, positions, tok_seq, block_table, bt_stride,
                  tile_tok0, tile_ntok, H, Hkv, D, Dv, Dp, P, opt, heads_per_chunk);
    } else {
        TK_CHECK_ARG(false, "attention: unknown dtype %d", dtype);
    }
    TK_CHECK_LAUNCH("attn_pointwise");
    return 0;
}
