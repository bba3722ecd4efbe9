// Attention over a cache of latents: every position keeps one row [c (R) | k_rot (Dr)], the
// normed key/value latent and one rotated key part that all heads share. With the keys'
// up-projection taken into the queries (q_lat[h] = W_uk[h]^T q[h]) a head's score is
// (q_lat . c + q_rot . k_rot) * scale and its output, before the values' up-projection, is
// sum_j p_j c_j: attention with one key/value head whose key is the whole row and whose value
// is the row's first R columns.
//
//   prepare: c_q = rmsnorm(row[0:Rq]) * wq;  c = rmsnorm(row[Rq:Rq+R]) * wkv -> cache;
//            k_rot = rotate(row[Rq+R : Rq+R+Dr]) -> cache      (interleaved pairs, 32-bit angles)
//   rotate_q: the last Dr columns of every query head, in place
//   attention: 32-bit scores, softmax and sums; storage float or bfloat16
#include <math.h>

#include "common.cuh"

namespace {
enum : int { TK_K_LATENT = 8 };
constexpr int BM = 16;       // rows (token x head) per block
constexpr int BN = 32;       // keys per iteration
constexpr int THREADS = 128; // 8 threads per row
}  // namespace

// (u, v) at columns (2i, 2i + 1), i < rot / 2, turned by pos * freq[i]; other columns unchanged
template <typename T>
__device__ __forceinline__ float rotated(const T* src, int c, int rot, const float* cs, const float* sn) {
    const float x = to_f<T>(src[c]);
    if (c >= rot) return x;
    const int i = c >> 1;
    const float y = to_f<T>(src[c ^ 1]);
    return (c & 1) ? x * cs[i] + y * sn[i] : x * cs[i] - y * sn[i];
}

// grid (tokens, 2): block (t, 0) norms the query latent, block (t, 1) norms the key/value latent,
// rotates the shared key part and writes both into the cache
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* proj, int64_t proj_stride, const float* __restrict__ wq,
                      const float* __restrict__ wkv, float eps, const float* __restrict__ freq,
                      const int* positions, const int* tok_seq, const int* block_table, int bt_stride,
                      T* cq_out, T* cache, int Rq, int R, int Dr, int rot, int P) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    __shared__ float red[33];
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * proj_stride;
    if (blockIdx.y == 0) {
        if (Rq == 0) return;
        float ss = 0.f;
        for (int i = threadIdx.x; i < Rq; i += blockDim.x) {
            const float v = to_f<T>(row[i]);
            ss += v * v;
        }
        const float rq = 1.0f / sqrtf(block_sum(ss, red) / (float)Rq + eps);
        for (int i = threadIdx.x; i < Rq; i += blockDim.x)
            cq_out[(size_t)t * Rq + i] = from_f<T>(to_f<T>(row[i]) * rq * wq[i]);
        return;
    }
    if (cache == nullptr) return;        // the layer reads another layer's latents: queries only
    float* cs = smem;
    float* sn = smem + rot / 2;
    const int pos = positions[t];
    const int page = TK_PAGE(TK_K_LATENT, block_table[(size_t)tok_seq[t] * bt_stride + pos / P]);
    for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) sincosf((float)pos * freq[i], &sn[i], &cs[i]);
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = to_f<T>(row[Rq + i]);
        ss += v * v;
    }
    const float rk = 1.0f / sqrtf(block_sum(ss, red) / (float)R + eps);   // (its barriers also publish cs / sn)
    T* dst = cache + ((size_t)page * P + pos % P) * (R + Dr);
    for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_f<T>(to_f<T>(row[Rq + i]) * rk * wkv[i]);
    for (int i = threadIdx.x; i < Dr; i += blockDim.x) dst[R + i] = from_f<T>(rotated<T>(row + Rq + R, i, rot, cs, sn));
}

TK_API int tk_latent_prepare(const void* proj, int64_t proj_stride, const float* wq, const float* wkv,
                             float eps, const float* freq, const int* positions, const int* tok_seq,
                             const int* block_table, int bt_stride, void* cq_out, void* cache, int tokens,
                             int Rq, int R, int Dr, int rot, int P, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && Rq >= 0 && R > 0 && Dr >= 0 && P > 0, "latent_prepare: bad sizes");
    TK_CHECK_ARG(rot % 2 == 0 && rot >= 0 && rot <= Dr, "latent_prepare: %d rotated columns of %d", rot, Dr);
    if (tokens == 0) return 0;
    const size_t smem = (size_t)(rot + 2) * sizeof(float);
    if (dtype == TK_F32)
        tk_launch(latent_prepare_kernel<float>, dim3(tokens, 2), dim3(128), smem, stream, (const float*)proj,
                  proj_stride, wq, wkv, eps, freq, positions, tok_seq, block_table, bt_stride, (float*)cq_out,
                  (float*)cache, Rq, R, Dr, rot, P);
    else if (dtype == TK_BF16)
        tk_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(tokens, 2), dim3(128), smem, stream,
                  (const __nv_bfloat16*)proj, proj_stride, wq, wkv, eps, freq, positions, tok_seq, block_table,
                  bt_stride, (__nv_bfloat16*)cq_out, (__nv_bfloat16*)cache, Rq, R, Dr, rot, P);
    else
        TK_CHECK_ARG(false, "latent_prepare: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("latent_prepare");
    return 0;
}

// q [tokens, H, D + Dr]: the last Dr columns of every head rotated in place. One block per token.
template <typename T>
__global__ void __launch_bounds__(128)
latent_rotate_q_kernel(T* q, const float* __restrict__ freq, const int* positions, int H, int D, int Dr, int rot) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    float* cs = smem;
    float* sn = smem + rot / 2;
    const int t = blockIdx.x;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) sincosf((float)pos * freq[i], &sn[i], &cs[i]);
    __syncthreads();
    // a thread takes a pair of columns, so that both are read before either is written
    const int pairs = rot / 2;
    for (int k = threadIdx.x; k < H * pairs; k += blockDim.x) {
        const int h = k / pairs, i = k % pairs;
        T* p = q + ((size_t)t * H + h) * (D + Dr) + D + 2 * i;
        const float u = to_f<T>(p[0]), v = to_f<T>(p[1]);
        p[0] = from_f<T>(u * cs[i] - v * sn[i]);
        p[1] = from_f<T>(v * cs[i] + u * sn[i]);
    }
}

TK_API int tk_latent_rotate_q(void* q, const float* freq, const int* positions, int tokens, int H, int D,
                              int Dr, int rot, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && H > 0 && D >= 0 && Dr >= 0, "latent_rotate_q: bad sizes");
    TK_CHECK_ARG(rot % 2 == 0 && rot >= 0 && rot <= Dr, "latent_rotate_q: %d rotated columns of %d", rot, Dr);
    if (tokens == 0 || rot == 0) return 0;
    const size_t smem = (size_t)(rot + 2) * sizeof(float);
    if (dtype == TK_F32)
        tk_launch(latent_rotate_q_kernel<float>, dim3(tokens), dim3(128), smem, stream, (float*)q, freq, positions,
                  H, D, Dr, rot);
    else if (dtype == TK_BF16)
        tk_launch(latent_rotate_q_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), smem, stream, (__nv_bfloat16*)q,
                  freq, positions, H, D, Dr, rot);
    else
        TK_CHECK_ARG(false, "latent_rotate_q: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("latent_rotate_q");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Attention over the latent cache, general form: any sizes, either storage type, 32-bit
// arithmetic throughout. A block takes a tile of rows (token, head): consecutive tokens of one
// sequence times a chunk of heads. Key j is visible to a query at position i iff
// 0 <= i - j < window (window <= 0: every earlier key).
//   q_lat [H, tokens, R] (row stride R),  q_rot: column D.. of q [tokens, H, D + Dr]
//   out   [H, tokens, R]
// ---------------------------------------------------------------------------------------------
template <typename T, int ACC>
__global__ void __launch_bounds__(THREADS)
attn_latent_kernel(const T* q_lat, const T* q, const T* cache, T* out, const int* positions,
                   const int* tok_seq, const int* block_table, int bt_stride, const int* tile_tok0,
                   const int* tile_ntok, int tokens, int H, int D, int R, int Dr, int P, int window,
                   float scale, int heads_per_chunk) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int DK = R + Dr, DP = DK + 1;
    float* Qs = smem;                 // [BM][DK + 1]
    float* Ks = Qs + BM * DP;         // [BN][DK + 1]
    float* Ss = Ks + BN * DP;         // [BM][BN + 1]
    __shared__ int row_pos[BM];

    const int chunk = blockIdx.y;
    const int g0 = chunk * heads_per_chunk;
    const int gh = min(heads_per_chunk, H - g0);
    const int tok0 = tile_tok0[blockIdx.x];
    const int ntok = tile_ntok[blockIdx.x];
    if (ntok <= 0) return;
    const int rows = ntok * gh;
    const int seq = tok_seq[tok0];
    const int tid = threadIdx.x;

    for (int i = tid; i < BM * DK; i += THREADS) {
        const int r = i / DK, c = i % DK;
        float v = 0.f;
        if (r < rows) {
            const int t = tok0 + r / gh, h = g0 + r % gh;
            v = c < R ? to_f<T>(q_lat[((size_t)h * tokens + t) * R + c])
                      : to_f<T>(q[((size_t)t * H + h) * (D + Dr) + D + (c - R)]);
        }
        Qs[r * DP + c] = v;
    }
    if (tid < BM) row_pos[tid] = tid < rows ? positions[tok0 + tid / gh] : -1;
    __syncthreads();

    const int pos_first = row_pos[0];
    const int pos_last = row_pos[rows - 1];
    const int lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int r = tid >> 3, sub = tid & 7;
    const int my_pos = row_pos[r];
    float m_i = -INFINITY, l_i = 0.f;
    float acc[ACC];
#pragma unroll
    for (int k = 0; k < ACC; ++k) acc[k] = 0.f;

    const int n_it = (pos_last - lo) / BN + 1;
    for (int it = 0; it < n_it; ++it) {
        const int j0 = lo + it * BN;
        {
            const int kk = tid >> 2, part = tid & 3;
            const int j = j0 + kk;
            if (j <= pos_last) {
                const int page = TK_PAGE(TK_K_LATENT, block_table[(size_t)seq * bt_stride + j / P]);
                const T* src = cache + ((size_t)page * P + (j % P)) * DK;
                for (int c = part; c < DK; c += 4) Ks[kk * DP + c] = to_f<T>(src[c]);
            } else {
                for (int c = part; c < DK; c += 4) Ks[kk * DP + c] = 0.f;
            }
        }
        __syncthreads();
        float s[4];
        float mx = -INFINITY;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int kk = sub + 8 * jj;
            const int j = j0 + kk;
            float d = 0.f;
            const float* qr = Qs + r * DP;
            const float* kr = Ks + kk * DP;
            for (int c = 0; c < DK; ++c) d = fmaf(qr[c], kr[c], d);
            d *= scale;
            const bool visible = my_pos >= 0 && j <= pos_last && j <= my_pos && (window <= 0 || my_pos - j < window);
            s[jj] = visible ? d : -INFINITY;
            mx = fmaxf(mx, s[jj]);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        const float m_new = fmaxf(m_i, mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = expf(m_i - m_safe);
        float psum = 0.f;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const float p = expf(s[jj] - m_safe);
            psum += p;
            Ss[r * (BN + 1) + sub + 8 * jj] = p;
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        psum += __shfl_xor_sync(0xffffffffu, psum, 4);
        l_i = l_i * alpha + psum;
        m_i = m_new;
        __syncthreads();
        const float* pr = Ss + r * (BN + 1);
#pragma unroll
        for (int k = 0; k < ACC; ++k) {
            const int c = sub + 8 * k;
            if (c < R) {
                float a = acc[k] * alpha;
                for (int kk = 0; kk < BN; ++kk) a = fmaf(pr[kk], Ks[kk * DP + c], a);
                acc[k] = a;
            }
        }
        __syncthreads();
    }
    if (r < rows) {
        const int t = tok0 + r / gh, h = g0 + r % gh;
        const float inv = l_i > 0.f ? 1.0f / l_i : 0.f;
#pragma unroll
        for (int k = 0; k < ACC; ++k) {
            const int c = sub + 8 * k;
            if (c < R) out[((size_t)h * tokens + t) * R + c] = from_f<T>(acc[k] * inv);
        }
    }
}

TK_API int tk_attn_latent_rows() { return BM; }
TK_API int tk_attn_latent_max_rank() { return 512; }

template <typename T, int ACC>
static int launch_attn_latent(const void* q_lat, const void* q, const void* cache, void* out, const int* positions,
                              const int* tok_seq, const int* block_table, int bt_stride, const int* tile_tok0,
                              const int* tile_ntok, int n_tiles, int tokens, int H, int D, int R, int Dr, int P,
                              int window, float scale, int heads_per_chunk, cudaStream_t stream) {
    const int DK = R + Dr;
    const size_t smem = ((size_t)(BM + BN) * (DK + 1) + (size_t)BM * (BN + 1)) * sizeof(float);
    TK_CHECK_ARG(smem <= 220 * 1024, "latent attention: rows of %d columns do not fit shared memory", DK);
    cudaFuncSetAttribute(attn_latent_kernel<T, ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid(n_tiles, (H + heads_per_chunk - 1) / heads_per_chunk);
    tk_launch(attn_latent_kernel<T, ACC>, grid, dim3(THREADS), smem, stream, (const T*)q_lat, (const T*)q,
              (const T*)cache, (T*)out, positions, tok_seq, block_table, bt_stride, tile_tok0, tile_ntok, tokens, H,
              D, R, Dr, P, window, scale, heads_per_chunk);
    return 0;
}

TK_API int tk_attn_latent(const void* q_lat, const void* q, const void* cache, void* out, const int* positions,
                          const int* tok_seq, const int* block_table, int bt_stride, const int* tile_tok0,
                          const int* tile_ntok, int n_tiles, int tokens_per_tile, int tokens, int H, int D, int R,
                          int Dr, int P, int window, float scale, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(H > 0 && R > 0 && R <= 512 && Dr >= 0 && D >= 0, "latent attention: bad sizes H=%d R=%d Dr=%d", H, R, Dr);
    TK_CHECK_ARG(P > 0 && n_tiles >= 0 && tokens >= 0, "latent attention: bad page size or counts");
    TK_CHECK_ARG(tokens_per_tile >= 1 && tokens_per_tile <= BM, "latent attention: %d tokens per tile", tokens_per_tile);
    if (n_tiles == 0) return 0;
    const int hpc = min(H, BM / tokens_per_tile);
    int rc;
#define TK_AL(TT)                                                                                                  \
    (R <= 64 ? launch_attn_latent<TT, 8>(q_lat, q, cache, out, positions, tok_seq, block_table, bt_stride, tile_tok0, \
                                        tile_ntok, n_tiles, tokens, H, D, R, Dr, P, window, scale, hpc, stream)      \
     : R <= 128 ? launch_attn_latent<TT, 16>(q_lat, q, cache, out, positions, tok_seq, block_table, bt_stride,        \
                                            tile_tok0, tile_ntok, n_tiles, tokens, H, D, R, Dr, P, window, scale,    \
                                            hpc, stream)                                                            \
     : R <= 256 ? launch_attn_latent<TT, 32>(q_lat, q, cache, out, positions, tok_seq, block_table, bt_stride,        \
                                            tile_tok0, tile_ntok, n_tiles, tokens, H, D, R, Dr, P, window, scale,    \
                                            hpc, stream)                                                            \
                : launch_attn_latent<TT, 64>(q_lat, q, cache, out, positions, tok_seq, block_table, bt_stride,        \
                                            tile_tok0, tile_ntok, n_tiles, tokens, H, D, R, Dr, P, window, scale,    \
                                            hpc, stream))
    if (dtype == TK_F32) rc = TK_AL(float);
    else if (dtype == TK_BF16) rc = TK_AL(__nv_bfloat16);
    else TK_CHECK_ARG(false, "latent attention: unknown dtype %d", dtype);
#undef TK_AL
    if (rc) return rc;
    TK_CHECK_LAUNCH("attn_latent");
    return 0;
}

// out[t, h, :] = x[h, t, :] * sigmoid(g[t, h])   (x [H, tokens, Dv] -> out [tokens, H, Dv]); g may be
// a column block of a wider row (g_stride). g null: the transposition alone.
template <typename T>
__global__ void head_gate_transpose_kernel(const T* x, const T* g, int64_t g_stride, T* out, int tokens, int H, int Dv) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)tokens * H * Dv;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % Dv);
        const size_t th = i / Dv;
        const int h = (int)(th % H);
        const size_t t = th / H;
        float v = to_f<T>(x[((size_t)h * tokens + t) * Dv + c]);
        if (g != nullptr) v *= 1.0f / (1.0f + expf(-to_f<T>(g[t * g_stride + h])));
        out[i] = from_f<T>(v);
    }
}

TK_API int tk_head_gate_transpose(const void* x, const void* g, int64_t g_stride, void* out, int tokens, int H,
                                  int Dv, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(tokens >= 0 && H > 0 && Dv > 0, "head_gate_transpose: bad sizes");
    if (tokens == 0) return 0;
    const size_t n = (size_t)tokens * H * Dv;
    const int blocks = (int)((n + 255) / 256 < (size_t)(148 * 16) ? (n + 255) / 256 : (size_t)(148 * 16));
    if (dtype == TK_F32)
        tk_launch(head_gate_transpose_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x,
                  (const float*)g, g_stride, (float*)out, tokens, H, Dv);
    else if (dtype == TK_BF16)
        tk_launch(head_gate_transpose_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                  (const __nv_bfloat16*)x, (const __nv_bfloat16*)g, g_stride, (__nv_bfloat16*)out, tokens, H, Dv);
    else
        TK_CHECK_ARG(false, "head_gate_transpose: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("head_gate_transpose");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// The same attention on the tensor cores for bfloat16 (mma.sync m16n8k16, 32-bit scores, softmax
// and sums). A CTA of 8 warps takes 32 rows (tokens x heads of one tile) and walks the keys 64 at
// a time through a two-stage cp.async pipeline; a key row [c | k_rot] is staged once and serves
// as the key (all of it) and as the value (its first R columns, read transposed by ldmatrix).
// Scores: warp (row group, key quarter) forms S[16 x 16] over the whole row; the row maxima meet
// in shared memory; P goes to shared memory in 16 bits. Output: warp (row group, column quarter)
// accumulates O[16 x R/4]. Needs R % 32 == 0, R <= 512, Dr % 16 == 0, D % 8 == 0.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int AM = 32, AN = 64, A_THREADS = 256, PLD = AN + 8;

__device__ __forceinline__ void a_cp_async16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void a_ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void a_ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void a_mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
}  // namespace

// MAXNB: n8 blocks of the output a warp may hold. RG: row groups of 16 rows a CTA takes: 2 (32 rows,
// four warps a group: 16 keys each in the score phase, R / 4 columns each in the output phase) or 1
// (16 rows, all eight warps on them: 8 keys and R / 8 columns each; for steps of single tokens,
// whose tiles are one token's heads).
template <int MAXNB, int RG>
__global__ void __launch_bounds__(A_THREADS, 1)
attn_latent_mma_kernel(const __nv_bfloat16* q_lat, const __nv_bfloat16* q, const __nv_bfloat16* cache,
                       __nv_bfloat16* out, const int* positions, const int* tok_seq, const int* block_table,
                       int bt_stride, const int* tile_tok0, const int* tile_ntok, int tokens, int H, int D, int R,
                       int Dr, int P, int window, float scale, int heads_per_chunk, int nsplit, float* part_o,
                       float* part_ml) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int NQ = 8 / RG;               // warps of a row group
    constexpr int AMR = 16 * RG;             // rows of the CTA
    constexpr int KW = AN / NQ;              // keys a warp scores
    constexpr int NJS = KW / 8;              // n8 blocks of those
    const int DK = R + Dr, KLD = DK + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [AMR][KLD]
    __nv_bfloat16* Ks = Qs + AMR * KLD;                                      // [2][AN][KLD]
    __nv_bfloat16* Ps = Ks + 2 * AN * KLD;                                   // [AMR][PLD]
    float* red_max = reinterpret_cast<float*>(Ps + AMR * PLD);               // [8 warps][16]
    float* red_sum = red_max + 128;                                          // [8 warps][16]
    __shared__ int row_pos[AM];

    const int g0 = blockIdx.y * heads_per_chunk;
    const int gh = min(heads_per_chunk, H - g0);
    const int tok0 = tile_tok0[blockIdx.x];
    const int ntok = tile_ntok[blockIdx.x];
    if (ntok <= 0) return;
    const int rows = ntok * gh;
    const int seq = tok_seq[tok0];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rg = warp / NQ, wq = warp % NQ;
    const int chunks = DK / 8;

    if (tid < AMR) row_pos[tid] = tid < rows ? positions[tok0 + tid / gh] : -1;
    // the queries: [q in the latent's space | rotated part], rows beyond the tile's are zero
    for (int c = tid; c < AMR * chunks; c += A_THREADS) {
        const int r = c / chunks, ch = c % chunks;
        const bool valid = r < rows;
        const void* src = q_lat;
        if (valid) {
            const int t = tok0 + r / gh, h = g0 + r % gh;
            src = ch * 8 < R ? (const void*)(q_lat + ((size_t)h * tokens + t) * R + ch * 8)
                             : (const void*)(q + ((size_t)t * H + h) * (D + Dr) + D + (ch * 8 - R));
        }
        a_cp_async16(Qs + r * KLD + ch * 8, src, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    __syncthreads();
    const int pos_first = row_pos[0];
    const int pos_last = row_pos[rows - 1];
    const int lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int n_all = (pos_last - lo) / AN + 1;
    // this CTA's share of the key tiles (blockIdx.z of nsplit; an empty share leaves zeros)
    const int per_split = (n_all + nsplit - 1) / nsplit;
    const int it_begin = blockIdx.z * per_split;
    const int n_it = min(n_all, it_begin + per_split);

    auto load_keys = [&](int it, int stage) {
        const int key = tid >> 2;
        const int j = lo + it * AN + key;
        const bool valid = j <= pos_last;
        const __nv_bfloat16* src = cache;
        if (valid) {
            const int page = TK_PAGE(TK_K_LATENT, block_table[(size_t)seq * bt_stride + j / P]);
            src = cache + ((size_t)page * P + (j % P)) * DK;
        }
        __nv_bfloat16* dst = Ks + ((size_t)stage * AN + key) * KLD;
        for (int ch = tid & 3; ch < chunks; ch += 4) a_cp_async16(dst + ch * 8, src + ch * 8, valid);
    };
    if (it_begin < n_it) load_keys(it_begin, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");

    const int r0 = rg * 16 + (lane >> 2), r1 = r0 + 8;
    const int pos0 = row_pos[r0], pos1 = row_pos[r1];
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float acc[MAXNB][4];
#pragma unroll
    for (int j = 0; j < MAXNB; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    const int nb = R / (8 * NQ);            // n8 blocks of my share of the columns
    const int col0 = wq * (R / NQ);

    for (int it = it_begin; it < n_it; ++it) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (it + 1 < n_it) load_keys(it + 1, (it + 1 - it_begin) & 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const __nv_bfloat16* ks = Ks + (size_t)((it - it_begin) & 1) * AN * KLD;
        // ---- scores of my 16 rows against my 16 keys ----
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            const __nv_bfloat16* qa = Qs + (rg * 16 + (lane & 15)) * KLD + (lane >> 4) * 8;
            if constexpr (NJS == 2) {
                const __nv_bfloat16* kb = ks + (wq * 16 + (lane & 7) + (lane >> 4) * 8) * KLD + ((lane >> 3) & 1) * 8;
                for (int k = 0; k < DK; k += 16) {
                    unsigned a[4], b[4];
                    a_ldmatrix_x4(a, qa + k);
                    a_ldmatrix_x4(b, kb + k);
                    a_mma_bf16(s[0], a, b[0], b[1]);
                    a_mma_bf16(s[1], a, b[2], b[3]);
                }
            } else {
                // 8 keys a warp: their K steps two at a time (one ldmatrix brings k .. k + 31 of the 8 keys)
                const __nv_bfloat16* kb = ks + (wq * 8 + (lane & 7)) * KLD + (lane >> 3) * 8;
                int k = 0;
                for (; k + 32 <= DK; k += 32) {
                    unsigned a0[4], a1[4], b[4];
                    a_ldmatrix_x4(a0, qa + k);
                    a_ldmatrix_x4(a1, qa + k + 16);
                    a_ldmatrix_x4(b, kb + k);
                    a_mma_bf16(s[0], a0, b[0], b[1]);
                    a_mma_bf16(s[1], a1, b[2], b[3]);
                }
                if (k < DK) {       // a last step of 16 (the row's pad keeps the ldmatrix inside the tile)
                    unsigned a0[4], b[4];
                    a_ldmatrix_x4(a0, qa + k);
                    a_ldmatrix_x4(b, kb + k - 16);
                    a_mma_bf16(s[0], a0, b[2], b[3]);
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) s[0][e] += s[1][e];
            }
        }
        const int jbase = lo + it * AN + wq * KW + (lane & 3) * 2;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int jn = 0; jn < NJS; ++jn)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = jbase + jn * 8 + e;
                const bool v0 = j <= pos0 && (window <= 0 || pos0 - j < window);
                const bool v1 = j <= pos1 && (window <= 0 || pos1 - j < window);
                s[jn][e] = v0 ? s[jn][e] * scale : -INFINITY;
                s[jn][2 + e] = v1 ? s[jn][2 + e] * scale : -INFINITY;
                mx0 = fmaxf(mx0, s[jn][e]);
                mx1 = fmaxf(mx1, s[jn][2 + e]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if ((lane & 3) == 0) {
            red_max[(rg * NQ + wq) * 16 + (lane >> 2)] = mx0;
            red_max[(rg * NQ + wq) * 16 + (lane >> 2) + 8] = mx1;
        }
        __syncthreads();
        float n0 = m0, n1 = m1;
#pragma unroll
        for (int w = 0; w < NQ; ++w) {
            n0 = fmaxf(n0, red_max[(rg * NQ + w) * 16 + (lane >> 2)]);
            n1 = fmaxf(n1, red_max[(rg * NQ + w) * 16 + (lane >> 2) + 8]);
        }
        const float s0 = n0 == -INFINITY ? 0.f : n0, s1 = n1 == -INFINITY ? 0.f : n1;
        const float alpha0 = expf(m0 - s0), alpha1 = expf(m1 - s1);
        m0 = n0;
        m1 = n1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int jn = 0; jn < NJS; ++jn) {
            const float p00 = expf(s[jn][0] - s0), p01 = expf(s[jn][1] - s0);
            const float p10 = expf(s[jn][2] - s1), p11 = expf(s[jn][3] - s1);
            ps0 += p00 + p01;
            ps1 += p10 + p11;
            const int col = wq * KW + jn * 8 + (lane & 3) * 2;
            *reinterpret_cast<__nv_bfloat162*>(Ps + r0 * PLD + col) = __floats2bfloat162_rn(p00, p01);
            *reinterpret_cast<__nv_bfloat162*>(Ps + r1 * PLD + col) = __floats2bfloat162_rn(p10, p11);
        }
        l0 = l0 * alpha0 + ps0;             // (my keys' share of the row sums; the quad is summed at the end)
        l1 = l1 * alpha1 + ps1;
#pragma unroll
        for (int j = 0; j < MAXNB; ++j) {
            acc[j][0] *= alpha0; acc[j][1] *= alpha0;
            acc[j][2] *= alpha1; acc[j][3] *= alpha1;
        }
        __syncthreads();
        // ---- my 16 rows x my quarter of the latent's columns += P . V ----
#pragma unroll
        for (int kk = 0; kk < AN; kk += 16) {
            unsigned a[4];
            a_ldmatrix_x4(a, Ps + (rg * 16 + (lane & 15)) * PLD + kk + (lane >> 4) * 8);
            const __nv_bfloat16* vb = ks + (kk + (lane & 7) + ((lane >> 3) & 1) * 8) * KLD + col0 + (lane >> 4) * 8;
#pragma unroll
            for (int jp = 0; jp < (MAXNB + 1) / 2; ++jp) {
                if (jp * 2 < nb) {
                    unsigned b[4];
                    a_ldmatrix_x4_trans(b, vb + jp * 16);
                    a_mma_bf16(acc[jp * 2], a, b[0], b[1]);
                    if (jp * 2 + 1 < MAXNB && jp * 2 + 1 < nb) a_mma_bf16(acc[jp * 2 + 1 < MAXNB ? jp * 2 + 1 : 0], a, b[2], b[3]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // the row sums: over the quad, then over the four key quarters
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();
    if ((lane & 3) == 0) {
        red_sum[(rg * NQ + wq) * 16 + (lane >> 2)] = l0;
        red_sum[(rg * NQ + wq) * 16 + (lane >> 2) + 8] = l1;
    }
    __syncthreads();
    float t0 = 0.f, t1 = 0.f;
#pragma unroll
    for (int w = 0; w < NQ; ++w) {
        t0 += red_sum[(rg * NQ + w) * 16 + (lane >> 2)];
        t1 += red_sum[(rg * NQ + w) * 16 + (lane >> 2) + 8];
    }
    if (nsplit > 1) {
        // my share, not normalised, with its maximum and sum: the merge kernel finishes the rows
        const size_t base = (size_t)blockIdx.z * H * tokens;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? r1 : r0;
            if (r >= rows) continue;
            const int t = tok0 + r / gh, h = g0 + r % gh;
            const size_t row = base + (size_t)h * tokens + t;
            if (wq == 0 && (lane & 3) == 0) {
                part_ml[row * 2] = half ? m1 : m0;
                part_ml[row * 2 + 1] = half ? t1 : t0;
            }
#pragma unroll
            for (int j = 0; j < MAXNB; ++j) {
                if (j >= nb) break;
                const int col = col0 + j * 8 + (lane & 3) * 2;
                *reinterpret_cast<float2*>(part_o + row * R + col) = make_float2(acc[j][half * 2], acc[j][half * 2 + 1]);
            }
        }
        return;
    }
    const float inv0 = t0 > 0.f ? 1.0f / t0 : 0.f, inv1 = t1 > 0.f ? 1.0f / t1 : 0.f;
#pragma unroll
    for (int j = 0; j < MAXNB; ++j) {
        if (j >= nb) break;
        const int col = col0 + j * 8 + (lane & 3) * 2;
        if (r0 < rows) {
            const int t = tok0 + r0 / gh, h = g0 + r0 % gh;
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)h * tokens + t) * R + col) =
                __floats2bfloat162_rn(acc[j][0] * inv0, acc[j][1] * inv0);
        }
        if (r1 < rows) {
            const int t = tok0 + r1 / gh, h = g0 + r1 % gh;
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)h * tokens + t) * R + col) =
                __floats2bfloat162_rn(acc[j][2] * inv1, acc[j][3] * inv1);
        }
    }
}

TK_API int tk_attn_latent_mma_rows() { return AM; }

// 1 when the tensor-core form takes these sizes
TK_API int tk_attn_latent_mma_supported(int D, int R, int Dr) {
    return (R % 32 == 0 && R >= 32 && R <= 512 && Dr % 16 == 0 && Dr >= 16 && D % 8 == 0) ? 1 : 0;
}

TK_API int tk_attn_latent_mma(const void* q_lat, const void* q, const void* cache, void* out, const int* positions,
                              const int* tok_seq, const int* block_table, int bt_stride, const int* tile_tok0,
                              const int* tile_ntok, int n_tiles, int tokens_per_tile, int tokens, int H, int D, int R,
                              int Dr, int P, int window, float scale, int nsplit, float* part_o, float* part_ml,
                              int rows16, cudaStream_t stream) {
    TK_CHECK_ARG(nsplit >= 1 && nsplit <= 64 && (nsplit == 1 || (part_o != nullptr && part_ml != nullptr)),
                 "latent attention (mma): %d shares of the keys need scratch memory", nsplit);
    TK_CHECK_ARG(tk_attn_latent_mma_supported(D, R, Dr), "latent attention (mma): sizes D=%d R=%d Dr=%d", D, R, Dr);
    TK_CHECK_ARG(H > 0 && P > 0 && n_tiles >= 0 && tokens >= 0, "latent attention (mma): bad counts");
    TK_CHECK_ARG(tokens_per_tile >= 1 && tokens_per_tile <= AM, "latent attention (mma): %d tokens per tile", tokens_per_tile);
    if (n_tiles == 0) return 0;
    // one row group of 16 rows for tiles of one token (steps of single tokens), where the latent
    // divides over eight warps
    const bool one = rows16 != 0 && tokens_per_tile == 1 && R % 64 == 0;
    const int am = one ? 16 : AM;
    const int hpc = min(H, am / tokens_per_tile);
    const int KLD = R + Dr + 8;
    const size_t smem = (size_t)(am + 2 * AN) * KLD * 2 + (size_t)am * PLD * 2 + 256 * sizeof(float);
    dim3 grid(n_tiles, (H + hpc - 1) / hpc, nsplit);
#define TK_ALM2(NB, RGV)                                                                                           \
    do {                                                                                                           \
        cudaFuncSetAttribute(attn_latent_mma_kernel<NB, RGV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        tk_launch(attn_latent_mma_kernel<NB, RGV>, grid, dim3(A_THREADS), smem, stream, (const __nv_bfloat16*)q_lat, \
                  (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, positions, tok_seq,   \
                  block_table, bt_stride, tile_tok0, tile_ntok, tokens, H, D, R, Dr, P, window, scale, hpc, nsplit, \
                  part_o, part_ml);                                                                                \
    } while (0)
#define TK_ALM(NB) do { if (one) TK_ALM2(NB, 1); else TK_ALM2(NB, 2); } while (0)
    const int nb = one ? R / 64 : R / 32;
    if (nb <= 2) TK_ALM(2);
    else if (nb <= 4) TK_ALM(4);
    else if (nb <= 8) TK_ALM(8);
    else TK_ALM(16);
#undef TK_ALM
#undef TK_ALM2
    TK_CHECK_LAUNCH("attn_latent_mma");
    return 0;
}

// out[h, t, :] = sum_s w_s O_s / sum_s w_s l_s with w_s = exp(m_s - max m): the shares of a row's keys
// that several CTAs took, merged. One block per row (h, t).
__global__ void __launch_bounds__(128)
attn_latent_merge_kernel(const float* part_o, const float* part_ml, __nv_bfloat16* out, int rows, int R, int nsplit) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float w_s[64];
    __shared__ float inv_s;
    const size_t row = blockIdx.x;
    if (threadIdx.x < 32) {
        // the shares' maxima and sums in one trip: lane s takes shares s and s + 32
        float m[2], l[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int s = threadIdx.x + 32 * k;
            m[k] = s < nsplit ? part_ml[((size_t)s * rows + row) * 2] : -INFINITY;
            l[k] = s < nsplit ? part_ml[((size_t)s * rows + row) * 2 + 1] : 0.f;
        }
        const float mx = warp_max(fmaxf(m[0], m[1]));
        float total = 0.f;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float w = (m[k] == -INFINITY) ? 0.f : expf(m[k] - mx);
            w_s[threadIdx.x + 32 * k] = w;
            total += w * l[k];
        }
        total = warp_sum(total);
        if (threadIdx.x == 0) inv_s = total > 0.f ? 1.0f / total : 0.f;
    }
    __syncthreads();
    const float inv = inv_s;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float w = w_s[s];
            if (w != 0.f) v = fmaf(w, part_o[((size_t)s * rows + row) * R + c], v);
        }
        out[row * R + c] = __float2bfloat16_rn(v * inv);
    }
}

TK_API int tk_attn_latent_merge(const float* part_o, const float* part_ml, void* out, int rows, int R, int nsplit,
                                cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && R > 0 && nsplit >= 1, "latent attention merge: bad sizes");
    if (rows == 0) return 0;
    tk_launch(attn_latent_merge_kernel, dim3(rows), dim3(128), 0, stream, part_o, part_ml, (__nv_bfloat16*)out, rows, R,
              nsplit);
    TK_CHECK_LAUNCH("attn_latent_merge");
    return 0;
}
