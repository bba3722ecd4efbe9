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
// own included. This form runs on the CUDA cores and takes any head sizes and both storage types;
// the tensor-core form for bfloat16 (heads of 64 and 128) is below it.
#include <math.h>

#include "paged_tiles.cuh"

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

// ---------------------------------------------------------------------------------------------
// The tensor-core form (bfloat16, key size = value size = 64 or 128, warp-level mma.sync
// m16n8k16). No running maximum and no rescaling: every weight is final when it is formed, so a
// block of scores goes S = Q K^T -> w(S) in 32-bit -> O += round16(w) V and shares of the keys
// add up.
//   prompt portions: a CTA takes up to 64 rows (64 / G tokens of one sequence, G heads each), four
//     warps of 16 rows, and walks the keys in tiles of 64 through a double-buffered cp.async
//     pipeline.
//   single tokens: a token's G heads are the (padded) 16 rows of all four warps; warp w takes keys
//     16 w .. 16 w + 15 of every tile and the four sums meet in shared memory; `nsplit` CTAs share
//     a token's keys, each writes its sum in 32-bit and a second kernel adds the shares.
// The weight function uses the special-function unit's exponential and logarithm (2 ulp in
// 32-bit, far below the 16-bit rounding of the weights where they meet the values).
// ---------------------------------------------------------------------------------------------
namespace {

// A row's constants, with the weight carried in base-2 logarithms so that every special function is
// one instruction: with E = 2^(c1 dot), the negated score times log2(e) is
//     s2 = k2 / (1 + E) + k0 + a1 log2(1 + a2 dist),   k2 = 2 cap log2(e), k0 = -(cap + hb) log2(e)
// (cap tanh(z) = cap - 2 cap / (1 + e^(2z)), c1 = 2 scale log2(e) / cap), and the weight 1 / (1 + 2^s2).
// Without a cap s2 = c1 dot + k0 + ..., c1 = -scale log2(e), k0 = -hb log2(e).
struct RowConst { float c1, k2, k0, a1, a2; };

__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_fast(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_fast(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// an overflowing power of two is +inf and its reciprocal 0: the limits come out without clamps
__device__ __forceinline__ float point_weight_fast(float dot, const RowConst& rc, bool capped, bool has_r, float dist) {
    float s2 = capped ? fmaf(rc.k2, rcp_fast(1.f + ex2_fast(dot * rc.c1)), rc.k0) : fmaf(dot, rc.c1, rc.k0);
    if (has_r) s2 = fmaf(rc.a1, lg2_fast(fmaf(rc.a2, dist, 1.f)), s2);
    return rcp_fast(1.f + ex2_fast(s2));
}

// keys k0 .. k0 + NK - 1 of a staged 64-key tile whose first key is position j0
template <int D, int NK>
__device__ __forceinline__ void point_block(const uint32_t (&qf)[D / 16][4], uint32_t ktile, uint32_t vtile, int k0,
                                            int j0, int pos_lo, int pos_hi, const RowConst& rlo, const RowConst& rhi,
                                            bool capped, bool has_r, int window, float (&o)[D / 8][4]) {
    const int lane = threadIdx.x & 31;
    const int t = lane & 3;
    const int mi = lane >> 3, r = lane & 7;
    float s[NK / 8][4];
#pragma unroll
    for (int n = 0; n < NK / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
    for (int np = 0; np < NK / 16; ++np) {
        const int key = k0 + np * 16 + r + 8 * (mi >> 1);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t b[4];
            ldmatrix_x4(b, ktile + tile_off<D>(key, ks * 2 + (mi & 1)));
            mma16816(s[2 * np], qf[ks], b[0], b[1]);
            mma16816(s[2 * np + 1], qf[ks], b[2], b[3]);
        }
    }
    uint32_t pf[NK / 16][4];
    const float pos_lo_f = (float)pos_lo, pos_hi_f = (float)pos_hi, key_f = (float)(j0 + k0 + 2 * t);
    const float window_f = window > 0 ? (float)window : INFINITY;
#pragma unroll
    for (int n = 0; n < NK / 8; ++n) {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            // distances as differences of floats (exact below 2^24): no conversion per score
            const float dist = ((e < 2) ? pos_lo_f : pos_hi_f) - (key_f + (float)(n * 8 + (e & 1)));
            const bool visible = dist >= 0.f && dist < window_f;         // a padding row's position is -1
            p[e] = visible ? point_weight_fast(s[n][e], (e < 2) ? rlo : rhi, capped, has_r, dist) : 0.f;
        }
        // the C layout of two neighbouring 8-key tiles is the A layout of one 16-key step
        pf[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
        pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
    }
#pragma unroll
    for (int ks = 0; ks < NK / 16; ++ks) {
        const int key = k0 + ks * 16 + r + 8 * (mi & 1);
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, vtile + tile_off<D>(key, dp * 2 + (mi >> 1)));
            mma16816(o[2 * dp], pf[ks], b[0], b[1]);
            mma16816(o[2 * dp + 1], pf[ks], b[2], b[3]);
        }
    }
}

// Query fragments of 16 rows from global memory: row r is (token tok0 + r / G, head h0 + r % G);
// rows at or past `rows` read as zero.
template <int D>
__device__ __forceinline__ void point_load_q(uint32_t (&qf)[D / 16][4], const __nv_bfloat16* q, int row0, int rows,
                                             int tok0, int G, int H, int h0) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = row0 + g + 8 * half;
        const bool ok = r < rows;
        const __nv_bfloat16* src = ok ? q + ((size_t)(tok0 + r / G) * H + h0 + r % G) * D : q;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t lo = 0u, hi = 0u;
            if (ok) {
                lo = *reinterpret_cast<const uint32_t*>(src + ks * 16 + 2 * t);
                hi = *reinterpret_cast<const uint32_t*>(src + ks * 16 + 8 + 2 * t);
            }
            qf[ks][half] = lo;
            qf[ks][half + 2] = hi;
        }
    }
}

template <int D, bool SINGLE>
__global__ void __launch_bounds__(128, (D == 64 ? 4 : 2))
attn_pointwise_mma_kernel(const __nv_bfloat16* q, const __nv_bfloat16* pool, __nv_bfloat16* out, float* partial,
                          const int* positions, const int* tok_seq, const int* block_table, int bt_stride,
                          const int* tile_tok0, const int* tile_ntok, const int* singles, int n_units, int H, int Hkv,
                          int P, int p_shift, PointOptions opt, int nsplit) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    constexpr int TILE_BYTES = 64 * D * 2;
    const uint32_t smem = (uint32_t)__cvta_generic_to_shared(smem_raw);      // [stage][K | V][64][D]
    const int G = H / Hkv;
    const int kvh = blockIdx.x % Hkv;
    // prompt tiles in reverse: a tile late in its sequence reads the most keys and starts first
    const int unit = SINGLE ? blockIdx.x / Hkv : n_units - 1 - blockIdx.x / Hkv;
    int tok0, ntok;
    if (SINGLE) {
        tok0 = singles != nullptr ? singles[unit] : unit;
        ntok = 1;
        if (tok0 < 0) return;        // an unused entry of a fixed-length list (captured steps)
    } else {
        tok0 = tile_tok0[unit];
        ntok = tile_ntok[unit];
        if (ntok <= 0) return;       // an unused entry of a fixed-length tile list (captured steps)
    }
    const int rows = ntok * G;
    const int seq = tok_seq[tok0];
    const int* bt_row = block_table + (size_t)seq * bt_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2;
    const int pos_first = positions[tok0];
    const int pos_last = pos_first + ntok - 1;       // consecutive positions within a tile
    const int lo = opt.window > 0 ? max(0, pos_first - opt.window + 1) : 0;
    const int j_begin = (lo / 64) * 64;
    const int row0 = SINGLE ? 0 : warp * 16;

    uint32_t qf[D / 16][4];
    point_load_q<D>(qf, q, row0, rows, tok0, G, H, kvh * G);
    const int r_lo = row0 + g, r_hi = r_lo + 8;
    const int pos_lo = r_lo < rows ? pos_first + r_lo / G : -1;
    const int pos_hi = r_hi < rows ? pos_first + r_hi / G : -1;
    const bool has_r = opt.r1 != nullptr;
    const bool capped = opt.cap > 0.f;
    auto row_const = [&](int r, int pos) {
        RowConst c{0.f, 0.f, 0.f, 0.f, 0.f};
        if (pos >= 0) {
            constexpr float LOG2E = 1.4426950408889634f;
            const int head = kvh * G + r % G;
            const float scale = opt.scale * temperature(opt, pos);
            const float hb = opt.head_bias != nullptr ? opt.head_bias[head] : 0.f;
            if (has_r) c.a1 = opt.r1[head], c.a2 = opt.r2[head];
            if (capped) {
                c.c1 = 2.f * LOG2E * scale / opt.cap;
                c.k2 = 2.f * LOG2E * opt.cap;
                c.k0 = -LOG2E * (opt.cap + hb);
            } else {
                c.c1 = -LOG2E * scale;
                c.k0 = -LOG2E * hb;
            }
        }
        return c;
    };
    const RowConst rlo = row_const(r_lo, pos_lo), rhi = row_const(r_hi, pos_hi);
    // the warp's own key range: nothing above its last row's position, nothing a window hides
    const int w_last_row = min(rows, row0 + 16) - 1;
    const int w_pos_max = w_last_row >= row0 ? pos_first + w_last_row / G : -1;
    const int w_pos_min = pos_first + row0 / G;

    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;

    // this CTA's share of the key tiles
    const int n_all = (pos_last - j_begin) / 64 + 1;
    const int per = (n_all + nsplit - 1) / nsplit;
    const int it0 = blockIdx.y * per, it1 = min(n_all, it0 + per);

    PagedLoader<D, 64, 128> loader;
    loader.init(tid, kvh, Hkv, P, p_shift);
    auto issue = [&](int it) {
        const uint32_t base = smem + (uint32_t)((it - it0) & 1) * 2 * TILE_BYTES;
        const int j0 = j_begin + it * 64;
        if (p_shift >= 0) {
            loader.issue_looked_up(base, base + TILE_BYTES, pool, j0, lo, pos_last);
            if (it + 1 < it1) loader.lookup(bt_row, j0 + 64, lo, pos_last);
        } else {
            load_tile<D>(base, pool, bt_row, j0, 64, lo, pos_last, kvh, Hkv, P, 0, tid, 128);
            load_tile<D>(base + TILE_BYTES, pool, bt_row, j0, 64, lo, pos_last, kvh, Hkv, P, 1, tid, 128);
        }
        cp_async_commit();
    };
    if (it0 < it1) {
        if (p_shift >= 0) loader.lookup(bt_row, j_begin + it0 * 64, lo, pos_last);
        issue(it0);
    }
    for (int it = it0; it < it1; ++it) {
        cp_async_wait<0>();
        __syncthreads();
        if (it + 1 < it1) issue(it + 1);
        const int j0 = j_begin + it * 64;
        const uint32_t base = smem + (uint32_t)((it - it0) & 1) * 2 * TILE_BYTES;
        if (SINGLE) {
            const int k0 = warp * 16;
            if (w_pos_max >= j0 + k0 && (opt.window <= 0 || j0 + k0 + 15 > w_pos_min - opt.window))
                point_block<D, 16>(qf, base, base + TILE_BYTES, k0, j0, pos_lo, pos_hi, rlo, rhi, capped,
                                   has_r, opt.window, o);
        } else if (w_pos_max >= j0 && (opt.window <= 0 || j0 + 63 > w_pos_min - opt.window)) {
            point_block<D, 64>(qf, base, base + TILE_BYTES, 0, j0, pos_lo, pos_hi, rlo, rhi, capped, has_r,
                               opt.window, o);
        }
    }
    const int t = lane & 3;
    if (!SINGLE) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = row0 + g + 8 * half;
            if (r >= rows) continue;
            __nv_bfloat16* dst = out + ((size_t)(tok0 + r / G) * H + kvh * G + r % G) * D;
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
                *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = pack_bf16(o[n][half * 2], o[n][half * 2 + 1]);
        }
        return;
    }
    // single tokens: the four warps' sums over their keys meet in shared memory
    __syncthreads();                                  // every warp is done with the staged tiles
    float* sums = reinterpret_cast<float*>(smem_raw); // [4][16][D]
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        float* dst = sums + ((size_t)warp * 16 + g + 8 * half) * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
            *reinterpret_cast<float2*>(dst + n * 8 + 2 * t) = make_float2(o[n][half * 2], o[n][half * 2 + 1]);
    }
    __syncthreads();
    for (int i = tid; i < rows * D; i += 128) {
        const int r = i / D, c = i % D;
        const float v = sums[(size_t)r * D + c] + sums[(size_t)(16 + r) * D + c] + sums[(size_t)(32 + r) * D + c] +
                        sums[(size_t)(48 + r) * D + c];
        const int head = kvh * G + r;
        if (nsplit == 1) out[((size_t)tok0 * H + head) * D + c] = __float2bfloat16(v);
        else partial[(((size_t)blockIdx.y * n_units + unit) * H + head) * D + c] = v;
    }
}

// out rows of the listed tokens = the sum of their `nsplit` shares
__global__ void __launch_bounds__(256)
attn_pointwise_sum_kernel(const float* partial, __nv_bfloat16* out, const int* singles, int n_units, int HD, int nsplit) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_units * HD) return;
    const int unit = (int)(i / HD), c = (int)(i % HD);
    const int tok = singles != nullptr ? singles[unit] : unit;
    if (tok < 0) return;             // an unused entry of a fixed-length list (captured steps)
    float v = 0.f;
    for (int s = 0; s < nsplit; ++s) v += partial[((size_t)s * n_units + unit) * HD + c];
    out[(size_t)tok * HD + c] = __float2bfloat16(v);
}

int shift_of(int P) {
    int s = 0;
    while ((1 << s) < P) ++s;
    return (1 << s) == P ? s : -1;
}
}  // namespace

// Whether the tensor-core form takes the shape: bfloat16, key size = value size = cache row of
// 64 or 128, at most 16 query heads per key/value head.
TK_API int tk_attn_pointwise_mma_supported(int H, int Hkv, int D, int Dv, int Dp) {
    return H > 0 && Hkv > 0 && H % Hkv == 0 && H / Hkv <= 16 && D == Dv && D == Dp && (D == 64 || D == 128);
}

TK_API int tk_attn_pointwise_mma_tokens(int H, int Hkv) { return 64 / (H / Hkv); }

// Prompt portions: tiles of tk_attn_pointwise_mma_tokens tokens (first token and count per tile).
// Single tokens (`n_single` > 0): the rows `singles` lists (null: rows 0 .. n_single - 1), each
// shared `nsplit` ways over its keys; partial float32 [nsplit, n_single, H, D] when nsplit > 1.
TK_API int tk_attn_pointwise_mma(const void* q, const void* kv_pool, void* out, const int* positions,
                                 const int* tok_seq, const int* block_table, int bt_stride, const int* tile_tok0,
                                 const int* tile_ntok, int n_tiles, const int* singles, int n_single, int nsplit,
                                 float* partial, int H, int Hkv, int D, int P, int window, float scale, float cap,
                                 float temp_coef, int temp_every, const float* r1, const float* r2,
                                 const float* head_bias, cudaStream_t stream) {
    TK_CHECK_ARG(tk_attn_pointwise_mma_supported(H, Hkv, D, D, D), "attention: %d / %d heads of %d are not the tensor-core form's",
                 H, Hkv, D);
    TK_CHECK_ARG((r1 == nullptr) == (r2 == nullptr), "attention: the distance bias has two numbers per head");
    TK_CHECK_ARG(P > 0 && n_tiles >= 0 && n_single >= 0 && cap >= 0.f && nsplit >= 1, "attention: bad sizes");
    TK_CHECK_ARG(nsplit == 1 || partial != nullptr, "attention: shares need scratch memory");
    PointOptions opt{scale, cap, temp_coef, temp_every, r1, r2, head_bias, window};
    const int smem = 4 * 64 * D * 2;
    const int shift = shift_of(P);
    auto q16 = (const __nv_bfloat16*)q;
    auto pool = (const __nv_bfloat16*)kv_pool;
    auto o16 = (__nv_bfloat16*)out;
#define TK_PW(DD, SINGLE, grid, units, ns)                                                                          \
    do {                                                                                                            \
        cudaFuncSetAttribute(attn_pointwise_mma_kernel<DD, SINGLE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
        tk_launch(attn_pointwise_mma_kernel<DD, SINGLE>, grid, dim3(128), smem, stream, q16, pool, o16, partial,    \
                  positions, tok_seq, block_table, bt_stride, tile_tok0, tile_ntok, singles, units, H, Hkv, P, shift, \
                  opt, ns);                                                                                         \
    } while (0)
    if (n_tiles > 0) {
        dim3 grid(n_tiles * Hkv, 1);
        if (D == 64) TK_PW(64, false, grid, n_tiles, 1);
        else TK_PW(128, false, grid, n_tiles, 1);
        TK_CHECK_LAUNCH("attn_pointwise_mma");
    }
    if (n_single > 0) {
        dim3 grid(n_single * Hkv, nsplit);
        if (D == 64) TK_PW(64, true, grid, n_single, nsplit);
        else TK_PW(128, true, grid, n_single, nsplit);
        TK_CHECK_LAUNCH("attn_pointwise_mma");
        if (nsplit > 1) {
            const size_t n = (size_t)n_single * H * D;
            tk_launch(attn_pointwise_sum_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream,
                      (const float*)partial, o16, singles, n_single, H * D, nsplit);
            TK_CHECK_LAUNCH("attn_pointwise_sum");
        }
    }
#undef TK_PW
    return 0;
}
