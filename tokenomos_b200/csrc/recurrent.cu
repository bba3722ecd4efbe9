// Recurrent mixers' state updates: kernels that walk a sequence's tokens in order with the state
// in registers. The state is 32-bit whatever the storage type, and so is everything that enters
// a recurrence after the projections: gates, decays and their logarithms, exponentials, maxima.
// A sequence at position 0 starts from zeros whatever its state row holds; a portion's kernel
// reads the row once, walks the portion's tokens and writes the row once.
//
// 1. Real-gated linear recurrent unit (per channel c of block b = c / w):
//        r = sigmoid(zr + br),  i = sigmoid(zi + bi),  log a = decay[c] * r  (decay = -8 softplus(lam))
//        S_t = a S_(t-1) + sqrt(1 - a^2) * i * u_t ;   out_t = S_t * gelu_tanh(y_t)
//    zr, zi: the block-diagonal gate products of u, 32-bit, laid out [blocks, T, 2 w].
//
// 2. Matrix memory (per head; S [dim, vd], n [dim], running maximum m, all from zero):
//        i = cap tanh(zi / cap),  f = logsigmoid(cap tanh(zf / cap))
//        m_t = max(f + m_(t-1), i);  S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T;  n_t likewise with k
//        o_t = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6)
//    n is kept as one more column of S (a value that is always 1), so the scan yields the
//    numerators and n . q alike; a second kernel divides, norms each head's output to unit root
//    mean square, applies the norm's weight and the sigmoid gate, and commits m.
#include <math.h>

#include "common.cuh"

namespace {
enum : int { TK_K_RECURRENT = 10 };

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float log_sigmoid(float z) {
    return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z));
}
}  // namespace

// ---------------------------------------------------------------------------------------------
// 1. gated linear recurrence: one thread per (sequence, channel)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
rglru_scan_kernel(const float* z, int Tz, const float* __restrict__ rb, const float* __restrict__ ib,
                  const float* __restrict__ decay, const T* u, int64_t u_stride, const T* y, int64_t y_stride,
                  float* state, const int* cu_seqlens, const int* seq_ctx, const int* seq_slot, T* out, int W, int w) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y;
    const int first = cu_seqlens[s], len = cu_seqlens[s + 1] - first;
    if (len <= 0) return;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int blk = c / w, o = c % w;
    const float* zr = z + ((size_t)blk * Tz) * 2 * w + o;      // + t * 2 w ; the input gate w further
    const float br = rb[c], bi = ib[c], dc = decay[c];
    float* st = state + (size_t)TK_SLOT(TK_K_RECURRENT, seq_slot[s]) * W + c;
    float S = seq_ctx[s] > 0 ? *st : 0.f;
    constexpr int U = 4;
    for (int t0 = 0; t0 < len; t0 += U) {
        float vr[U], vi[U], vu[U], vy[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const int t = first + min(t0 + k, len - 1);
            vr[k] = zr[(size_t)t * 2 * w];
            vi[k] = zr[(size_t)t * 2 * w + w];
            vu[k] = to_f<T>(u[(size_t)t * u_stride + c]);
            vy[k] = to_f<T>(y[(size_t)t * y_stride + c]);
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            if (t0 + k >= len) break;
            const float r = sigmoid_f(vr[k] + br), i = sigmoid_f(vi[k] + bi);
            const float log_a = dc * r;
            const float a = expf(log_a);
            const float mult = sqrtf(fmaxf(-expm1f(2.f * log_a), 0.f));      // sqrt(1 - a^2)
            S = fmaf(a, S, mult * i * vu[k]);
            out[(size_t)(first + t0 + k) * W + c] = from_f<T>(S * gelu_tanh(vy[k]));
        }
    }
    *st = S;
}

// Long portions of few sequences: a sequence's portion is cut into RS_SL slices of equal length and a
// block walks all of them at once, RS_CH channels wide (few channels a block: a portion of 2,048
// tokens of 1,024 channels is 128 blocks). The recurrence is linear in S, so a slice is
// the map S -> A S + B with A the product of its a_t and B what it leaves from zero: the first pass
// forms (A, B) per slice, every thread then chains the slices before its own from the stored state,
// and the second pass walks the slice again from there and writes the outputs.
namespace {
constexpr int RS_CH = 8;     // channels per block
constexpr int RS_SL = 128;   // slices per portion
constexpr int RS_KEEP = 16;  // a slice of up to this many tokens keeps its (a_t, b_t) in registers between the passes
}

template <typename T>
__global__ void __launch_bounds__(RS_CH * RS_SL)
rglru_scan_sliced_kernel(const float* __restrict__ z, int Tz, const float* __restrict__ rb,
                         const float* __restrict__ ib, const float* __restrict__ decay, const T* __restrict__ u,
                         int64_t u_stride, const T* __restrict__ y, int64_t y_stride, float* state,
                         const int* cu_seqlens, const int* seq_ctx, const int* seq_slot, T* __restrict__ out, int W,
                         int w) {
    __shared__ float A_s[RS_SL][RS_CH], B_s[RS_SL][RS_CH];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y;
    const int first = cu_seqlens[s], len = cu_seqlens[s + 1] - first;
    if (len <= 0) return;
    const int cl = threadIdx.x % RS_CH, sl = threadIdx.x / RS_CH;
    const int c = min(blockIdx.x * RS_CH + cl, W - 1);
    const bool live = blockIdx.x * RS_CH + cl < W;
    const int per = (len + RS_SL - 1) / RS_SL;
    const int t_begin = first + min(sl * per, len), t_end = first + min(sl * per + per, len);
    const int blk = c / w, o = c % w;
    const float* zr = z + ((size_t)blk * Tz) * 2 * w + o;
    const float br = rb[c], bi = ib[c], dc = decay[c];
    auto coef = [&](int t, float& a, float& x) {
        const float r = sigmoid_f(zr[(size_t)t * 2 * w] + br), i = sigmoid_f(zr[(size_t)t * 2 * w + w] + bi);
        const float log_a = dc * r;
        a = expf(log_a);
        x = sqrtf(fmaxf(-expm1f(2.f * log_a), 0.f)) * i * to_f<T>(u[(size_t)t * u_stride + c]);
    };
    float* st = state + (size_t)TK_SLOT(TK_K_RECURRENT, seq_slot[s]) * W + c;
    float S = seq_ctx[s] > 0 ? *st : 0.f;
    float A = 1.f, B = 0.f;
    if (per <= RS_KEEP) {
        float ka[RS_KEEP], kx[RS_KEEP];
        const int cnt = t_end - t_begin;
#pragma unroll
        for (int k = 0; k < RS_KEEP; ++k) {
            ka[k] = 1.f;
            kx[k] = 0.f;
            if (k < cnt) coef(t_begin + k, ka[k], kx[k]);
        }
#pragma unroll
        for (int k = 0; k < RS_KEEP; ++k) {
            B = fmaf(ka[k], B, kx[k]);
            A *= ka[k];
        }
        A_s[sl][cl] = A;
        B_s[sl][cl] = B;
        __syncthreads();
        for (int j = 0; j < sl; ++j) S = fmaf(A_s[j][cl], S, B_s[j][cl]);
#pragma unroll
        for (int k = 0; k < RS_KEEP; ++k) {
            if (k >= cnt) break;
            const int t = t_begin + k;
            S = fmaf(ka[k], S, kx[k]);
            if (live) out[(size_t)t * W + c] = from_f<T>(S * gelu_tanh(to_f<T>(y[(size_t)t * y_stride + c])));
        }
    } else {
#pragma unroll 4
        for (int t = t_begin; t < t_end; ++t) {
            float a, x;
            coef(t, a, x);
            B = fmaf(a, B, x);
            A *= a;
        }
        A_s[sl][cl] = A;
        B_s[sl][cl] = B;
        __syncthreads();
        for (int j = 0; j < sl; ++j) S = fmaf(A_s[j][cl], S, B_s[j][cl]);
#pragma unroll 4
        for (int t = t_begin; t < t_end; ++t) {
            float a, x;
            coef(t, a, x);
            S = fmaf(a, S, x);
            if (live) out[(size_t)t * W + c] = from_f<T>(S * gelu_tanh(to_f<T>(y[(size_t)t * y_stride + c])));
        }
    }
    if (live && sl == RS_SL - 1) *st = S;      // the slices after the portion's end are empty: this is the last state
}

// z float32 [blocks, Tz, 2 w] (r gate then i gate per block); rb, ib, decay float32 [W]; u, y [T, >= W]
// with row strides; state float32 [slots, W]; out [T, W] contiguous.
TK_API int tk_rglru_scan(const float* z, int Tz, const float* rb, const float* ib, const float* decay, const void* u,
                         int64_t u_stride, const void* y, int64_t y_stride, float* state, const int* cu_seqlens,
                         const int* seq_ctx, const int* seq_slot, int n_seqs, void* out, int W, int blocks, int dtype,
                         cudaStream_t stream) {
    TK_CHECK_ARG(W > 0 && blocks > 0 && W % blocks == 0, "gated recurrence: %d channels in %d blocks", W, blocks);
    TK_CHECK_ARG(n_seqs >= 0 && Tz >= 0, "gated recurrence: bad sizes");
    if (n_seqs == 0) return 0;
    if (Tz >= 2 * RS_SL * n_seqs) {      // long portions: slices of the time axis side by side
        dim3 sgrid((W + RS_CH - 1) / RS_CH, n_seqs);
        if (dtype == TK_F32)
            tk_launch(rglru_scan_sliced_kernel<float>, sgrid, dim3(RS_CH * RS_SL), 0, stream, z, Tz, rb, ib, decay,
                      (const float*)u, u_stride, (const float*)y, y_stride, state, cu_seqlens, seq_ctx, seq_slot,
                      (float*)out, W, W / blocks);
        else if (dtype == TK_BF16)
            tk_launch(rglru_scan_sliced_kernel<__nv_bfloat16>, sgrid, dim3(RS_CH * RS_SL), 0, stream, z, Tz, rb, ib,
                      decay, (const __nv_bfloat16*)u, u_stride, (const __nv_bfloat16*)y, y_stride, state, cu_seqlens,
                      seq_ctx, seq_slot, (__nv_bfloat16*)out, W, W / blocks);
        else
            TK_CHECK_ARG(false, "gated recurrence: unknown dtype %d", dtype);
        TK_CHECK_LAUNCH("rglru_scan_sliced");
        return 0;
    }
    dim3 grid((W + 127) / 128, n_seqs);
    if (dtype == TK_F32)
        tk_launch(rglru_scan_kernel<float>, grid, dim3(128), 0, stream, z, Tz, rb, ib, decay, (const float*)u, u_stride,
                  (const float*)y, y_stride, state, cu_seqlens, seq_ctx, seq_slot, (float*)out, W, W / blocks);
    else if (dtype == TK_BF16)
        tk_launch(rglru_scan_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, z, Tz, rb, ib, decay,
                  (const __nv_bfloat16*)u, u_stride, (const __nv_bfloat16*)y, y_stride, state, cu_seqlens, seq_ctx,
                  seq_slot, (__nv_bfloat16*)out, W, W / blocks);
    else
        TK_CHECK_ARG(false, "gated recurrence: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("rglru_scan");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// 2. matrix memory: one warp per (sequence, head, group of CW columns of [S | n]); a lane holds
// the rows d = lane + 32 j of its columns. The state is kept [head, column, d] so that a warp's
// reads and writes of it are contiguous. A block's warps share a head: they stage 32 (16) tokens of
// q, k and their columns of v in shared memory together (the next round's loads are in flight
// while this round is walked). Each warp forms the round's gates with a lane per token: the
// running maximum m -> max(f + m, i) is a scan over maps of that form, which compose as
// (f2, i2) o (f1, i1) = (f1 + f2, max(f2 + i1, i2)). The walk itself is then multiply-adds only,
// and the per-token partial sums of MSB tokens x CW columns are reduced over the lanes together,
// each lane ending with one of the 32 totals.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int CW = 4;        // columns per warp
constexpr int MWARPS = 4;    // warps per block
constexpr int MSB = 8;       // tokens reduced together: MSB * CW = 32 partial sums a lane
static_assert(MSB * CW == 32, "one total per lane");
}

template <typename T, int DPL>
__global__ void __launch_bounds__(32 * MWARPS)
mlstm_scan_kernel(const T* qkv, int64_t stride, int q_off, int k_off, int v_off, const float* gates, int64_t g_stride,
                  float cap, float q_scale, float* S_state, const float* m_state, const int* cu_seqlens,
                  const int* seq_ctx, const int* seq_slot, float* num, float* m_out, int H, int dim, int vd) {
    constexpr int DP = 32 * DPL;                          // the key size, padded
    constexpr int MTC = DPL <= 4 ? 32 : 16;               // tokens staged per round (what shared memory holds)
    static_assert(MTC % MSB == 0 && MTC <= 32, "a lane per token of a round");
    constexpr int NE = MTC * DP / (32 * MWARPS);          // elements of q (and of k) a thread stages per round
    constexpr int NV = MTC * MWARPS * CW / (32 * MWARPS); // and of v
    __shared__ float q_s[MTC][DP], k_s[MTC][DP];
    __shared__ __align__(16) float v_s[MTC][MWARPS * CW];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.z, h = blockIdx.y;
    const int first = cu_seqlens[s], len = cu_seqlens[s + 1] - first;
    if (len <= 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cols = vd + 1;
    const int cb = blockIdx.x * MWARPS * CW;              // the block's first column
    const int c0 = cb + warp * CW;                        // the warp's; past the end, the warp only stages
    const int slot = TK_SLOT(TK_K_RECURRENT, seq_slot[s]);
    const bool fresh = seq_ctx[s] <= 0;
    float* Sg = S_state + (((size_t)slot * H + h) * cols + c0) * dim;
    float Sr[CW][DPL];
#pragma unroll
    for (int c = 0; c < CW; ++c)
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
            const int d = lane + 32 * j;
            Sr[c][j] = (!fresh && c0 + c < cols && d < dim) ? Sg[(size_t)c * dim + d] : 0.f;
        }
    float m = fresh ? 0.f : m_state[(size_t)slot * H + h];
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;

    T qr[NE], kr[NE];
    float vr[NV], gi = 0.f, gf = 0.f;
    auto fetch = [&](int t0) {      // tokens t0 .. t0 + MTC - 1 of the portion; zeros past its end
#pragma unroll
        for (int e = 0; e < NE; ++e) {
            const int idx = tid + e * 32 * MWARPS, tok = idx / DP, d = idx % DP;
            const bool ok = t0 + tok < len && d < dim;
            const T* row = qkv + (size_t)(first + min(t0 + tok, len - 1)) * stride + h * dim + min(d, dim - 1);
            qr[e] = ok ? row[q_off] : from_f<T>(0.f);
            kr[e] = ok ? row[k_off] : from_f<T>(0.f);
        }
#pragma unroll
        for (int e = 0; e < NV; ++e) {
            const int idx = tid + e * 32 * MWARPS, tok = idx / (MWARPS * CW), col = cb + idx % (MWARPS * CW);
            const bool ok = t0 + tok < len;
            const T* row = qkv + (size_t)(first + min(t0 + tok, len - 1)) * stride + v_off + h * vd;
            vr[e] = !ok ? 0.f : col < vd ? to_f<T>(row[col]) : col == vd ? 1.f : 0.f;
        }
        if (lane < MTC && t0 + lane < len) {
            gi = gates[(size_t)(first + t0 + lane) * g_stride + h];
            gf = gates[(size_t)(first + t0 + lane) * g_stride + H + h];
        }
    };
    fetch(0);
    for (int t0 = 0; t0 < len; t0 += MTC) {
#pragma unroll
        for (int e = 0; e < NE; ++e) {
            const int idx = tid + e * 32 * MWARPS;
            q_s[idx / DP][idx % DP] = to_f<T>(qr[e]) * q_scale;
            k_s[idx / DP][idx % DP] = to_f<T>(kr[e]);
        }
#pragma unroll
        for (int e = 0; e < NV; ++e) {
            const int idx = tid + e * 32 * MWARPS;
            v_s[idx / (MWARPS * CW)][idx % (MWARPS * CW)] = vr[e];
        }
        const float zi = gi, zf = gf;
        __syncthreads();
        if (t0 + MTC < len) fetch(t0 + MTC);

        // the round's gates, a lane per token; lanes past the round's tokens hold the identity map
        const int n = min(MTC, len - t0);
        float ig = -INFINITY, fg = 0.f;
        if (lane < n) {
            ig = cap > 0.f ? cap * tanhf(zi * inv_cap) : zi;
            fg = log_sigmoid(cap > 0.f ? cap * tanhf(zf * inv_cap) : zf);
        }
        float fa = fg, ia = ig;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float fp = __shfl_up_sync(0xffffffffu, fa, o), ip = __shfl_up_sync(0xffffffffu, ia, o);
            if (lane >= o) {
                ia = fmaxf(fa + ip, ia);
                fa += fp;
            }
        }
        const float m_t = fmaxf(fa + m, ia);
        float m_prev = __shfl_up_sync(0xffffffffu, m_t, 1);
        if (lane == 0) m_prev = m;
        const float df_l = expf(fg + m_prev - m_t), di_l = lane < n ? expf(ig - m_t) : 0.f;
        m = __shfl_sync(0xffffffffu, m_t, 31);
        if (cb == 0 && warp == 0 && lane < n) m_out[(size_t)(first + t0 + lane) * H + h] = m_t;

        if (c0 < cols) {
            for (int sb = 0; sb < n; sb += MSB) {
                float part[MSB * CW];
#pragma unroll
                for (int tt = 0; tt < MSB; ++tt) {
                    const int tk = sb + tt;      // past the round's tokens: a decay of 1 and nothing added
                    const float df = __shfl_sync(0xffffffffu, df_l, tk), di = __shfl_sync(0xffffffffu, di_l, tk);
                    const float4 v4 = *reinterpret_cast<const float4*>(&v_s[tk][warp * CW]);
                    const float dv[CW] = {di * v4.x, di * v4.y, di * v4.z, di * v4.w};
                    float kk[DPL], qq[DPL];
#pragma unroll
                    for (int j = 0; j < DPL; ++j) {
                        kk[j] = k_s[tk][lane + 32 * j];
                        qq[j] = q_s[tk][lane + 32 * j];
                    }
#pragma unroll
                    for (int c = 0; c < CW; ++c) {
                        float p = 0.f;
#pragma unroll
                        for (int j = 0; j < DPL; ++j) {
                            Sr[c][j] = fmaf(df, Sr[c][j], dv[c] * kk[j]);
                            p = fmaf(Sr[c][j], qq[j], p);
                        }
                        part[tt * CW + c] = p;
                    }
                }
                // 32 sums over the lanes at once: each exchange halves what a lane still holds
#pragma unroll
                for (int r = 0; r < 5; ++r) {
                    const int sh = 16 >> r, half = 16 >> r;
                    const bool up = (lane & sh) != 0;
#pragma unroll
                    for (int i = 0; i < half; ++i) {
                        const float keep = up ? part[i + half] : part[i];
                        const float send = up ? part[i] : part[i + half];
                        part[i] = keep + __shfl_xor_sync(0xffffffffu, send, sh);
                    }
                }
                const int tt = lane / CW, c = lane % CW;
                if (sb + tt < n && c0 + c < cols)
                    num[((size_t)(first + t0 + sb + tt) * H + h) * cols + c0 + c] = part[0];
            }
        }
        __syncthreads();      // the round's tiles may be overwritten
    }
    if (c0 < cols) {
#pragma unroll
        for (int c = 0; c < CW; ++c)
#pragma unroll
            for (int j = 0; j < DPL; ++j) {
                const int d = lane + 32 * j;
                if (c0 + c < cols && d < dim) Sg[(size_t)c * dim + d] = Sr[c][j];
            }
    }
}

// Steps of single tokens (a few tokens a sequence at most): no staging and few registers, so that
// many warps are resident while the state, which is nearly all of the traffic, streams through.
// No warp waits for another: each forms the gates and the running maximum itself.
template <typename T, int DPL>
__global__ void __launch_bounds__(32 * MWARPS)
mlstm_token_kernel(const T* qkv, int64_t stride, int q_off, int k_off, int v_off, const float* gates, int64_t g_stride,
                  float cap, float q_scale, float* S_state, const float* m_state, const int* cu_seqlens,
                  const int* seq_ctx, const int* seq_slot, float* num, float* m_out, int H, int dim, int vd) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.z, h = blockIdx.y;
    const int first = cu_seqlens[s], len = cu_seqlens[s + 1] - first;
    if (len <= 0) return;
    const int lane = threadIdx.x & 31;
    const int group = blockIdx.x * MWARPS + (threadIdx.x >> 5);
    const int cols = vd + 1;
    const int c0 = group * CW;
    if (c0 >= cols) return;
    const int slot = TK_SLOT(TK_K_RECURRENT, seq_slot[s]);
    const bool fresh = seq_ctx[s] <= 0;
    float* Sg = S_state + (((size_t)slot * H + h) * cols + c0) * dim;
    float Sr[CW][DPL];
#pragma unroll
    for (int c = 0; c < CW; ++c)
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
            const int d = lane + 32 * j;
            Sr[c][j] = (!fresh && c0 + c < cols && d < dim) ? Sg[(size_t)c * dim + d] : 0.f;
        }
    float m = fresh ? 0.f : m_state[(size_t)slot * H + h];
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;

    // the next token's inputs are fetched while this one's are used
    float qn[DPL], kn[DPL], vn[CW], zin, zfn;
    auto fetch = [&](int t) {
        const T* row = qkv + (size_t)t * stride;
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
            const int d = lane + 32 * j;
            qn[j] = d < dim ? to_f<T>(row[q_off + h * dim + d]) : 0.f;
            kn[j] = d < dim ? to_f<T>(row[k_off + h * dim + d]) : 0.f;
        }
#pragma unroll
        for (int c = 0; c < CW; ++c) {
            const int col = c0 + c;
            vn[c] = col < vd ? to_f<T>(row[v_off + h * vd + col]) : (col == vd ? 1.f : 0.f);
        }
        zin = gates[(size_t)t * g_stride + h];
        zfn = gates[(size_t)t * g_stride + H + h];
    };
    fetch(first);
    for (int i = 0; i < len; ++i) {
        float q[DPL], k[DPL], v[CW];
#pragma unroll
        for (int j = 0; j < DPL; ++j) { q[j] = qn[j] * q_scale; k[j] = kn[j]; }
#pragma unroll
        for (int c = 0; c < CW; ++c) v[c] = vn[c];
        const float zi = zin, zf = zfn;
        if (i + 1 < len) fetch(first + i + 1);
        const float ig = cap > 0.f ? cap * tanhf(zi * inv_cap) : zi;
        const float fg = log_sigmoid(cap > 0.f ? cap * tanhf(zf * inv_cap) : zf);
        const float m_new = fmaxf(fg + m, ig);
        const float df = expf(fg + m - m_new), di = expf(ig - m_new);
        m = m_new;
        float part[CW];
#pragma unroll
        for (int c = 0; c < CW; ++c) {
            float p = 0.f;
            const float dv = di * v[c];
#pragma unroll
            for (int j = 0; j < DPL; ++j) {
                Sr[c][j] = fmaf(df, Sr[c][j], dv * k[j]);
                p = fmaf(Sr[c][j], q[j], p);
            }
            part[c] = p;
        }
#pragma unroll
        for (int c = 0; c < CW; ++c) part[c] = warp_sum(part[c]);
        if (lane == 0) {
            float* o = num + ((size_t)(first + i) * H + h) * cols + c0;
#pragma unroll
            for (int c = 0; c < CW; ++c)
                if (c0 + c < cols) o[c] = part[c];
            if (group == 0) m_out[(size_t)(first + i) * H + h] = m;
        }
    }
#pragma unroll
    for (int c = 0; c < CW; ++c)
#pragma unroll
        for (int j = 0; j < DPL; ++j) {
            const int d = lane + 32 * j;
            if (c0 + c < cols && d < dim) Sg[(size_t)c * dim + d] = Sr[c][j];
        }
}

// qkv: [T, stride] rows holding q (H x dim) at column q_off, k at k_off, v (H x vd) at v_off; gates
// float32 [T, g_stride]: H input-gate then H forget-gate pre-activations (biases added); S_state
// float32 [slots, H, vd + 1, dim]; m_state float32 [slots, H] (read only here); num float32
// [T, H, vd + 1]: S^T q per column, the last being n . q; m_out float32 [T, H].
TK_API int tk_mlstm_scan(const void* qkv, int64_t stride, int q_off, int k_off, int v_off, const float* gates,
                         int64_t g_stride, float cap, float q_scale, float* S_state, const float* m_state,
                         const int* cu_seqlens, const int* seq_ctx, const int* seq_slot, int n_seqs, int n_tokens,
                         float* num, float* m_out, int H, int dim, int vd, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(H > 0 && dim > 0 && vd > 0, "matrix memory: bad sizes");
    TK_CHECK_ARG(dim <= 256, "matrix memory: a key size of %d is above the 256 the scan keeps in registers", dim);
    if (n_seqs <= 0) return 0;
    const int groups = (vd + 1 + CW - 1) / CW;
    dim3 grid((groups + MWARPS - 1) / MWARPS, H, n_seqs);
    const int dpl = (dim + 31) / 32;
    const bool tokens = n_tokens < 4 * n_seqs;      // single tokens, not portions
#define TK_MS(TT, N)                                                                                              \
    tk_launch(tokens ? mlstm_token_kernel<TT, N> : mlstm_scan_kernel<TT, N>, grid, dim3(32 * MWARPS), 0, stream, \
              (const TT*)qkv, stride, q_off, k_off, v_off, gates, g_stride, cap, q_scale, S_state, m_state,       \
              cu_seqlens, seq_ctx, seq_slot, num, m_out, H, dim, vd)
#define TK_MS_T(TT)                                    \
    do {                                               \
        if (dpl <= 1) TK_MS(TT, 1);                    \
        else if (dpl <= 2) TK_MS(TT, 2);               \
        else if (dpl <= 4) TK_MS(TT, 4);               \
        else TK_MS(TT, 8);                             \
    } while (0)
    if (dtype == TK_F32) TK_MS_T(float);
    else if (dtype == TK_BF16) TK_MS_T(__nv_bfloat16);
    else TK_CHECK_ARG(false, "matrix memory: unknown dtype %d", dtype);
#undef TK_MS_T
#undef TK_MS
    TK_CHECK_LAUNCH("mlstm_scan");
    return 0;
}

// One warp per (token, head): o = num / (max(|n . q|, e^(-m)) + 1e-6), divided by its root mean
// square, times the norm's weight, times sigmoid(gate). The last token of a sequence commits m.
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_norm_gate_kernel(const float* num, const float* m_out, float* m_state, const float* __restrict__ weight,
                       const T* gate, int64_t gate_stride, const int* tok_seq, const int* cu_seqlens,
                       const int* seq_slot, T* out, int T_, int H, int vd, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= T_ * H) return;
    const int t = wid / H, h = wid % H, lane = threadIdx.x & 31;
    const float* row = num + (size_t)wid * (vd + 1);
    constexpr int NR = 8;      // a lane's first NR columns stay in registers; all their loads are in flight together
    float rv[NR], gv[NR], wv[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int c = lane + 32 * j;
        const bool in = c < vd;
        rv[j] = in ? row[c] : 0.f;
        wv[j] = in ? weight[h * vd + c] : 0.f;
        gv[j] = (in && gate != nullptr) ? to_f<T>(gate[(size_t)t * gate_stride + h * vd + c]) : 0.f;
    }
    const float m = m_out[wid];
    const float den = fmaxf(fabsf(row[vd]), expf(-m)) + 1e-6f;
    const float inv = 1.f / den;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        rv[j] *= inv;
        ss = fmaf(rv[j], rv[j], ss);
    }
    for (int c = lane + 32 * NR; c < vd; c += 32) {
        const float o = row[c] * inv;
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / (float)vd + eps);
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int c = lane + 32 * j;
        if (c >= vd) break;
        float o = rv[j] * rstd * wv[j];
        if (gate != nullptr) o *= sigmoid_f(gv[j]);
        out[(size_t)t * H * vd + h * vd + c] = from_f<T>(o);
    }
    for (int c = lane + 32 * NR; c < vd; c += 32) {
        float o = row[c] * inv * rstd * weight[h * vd + c];
        if (gate != nullptr) o *= sigmoid_f(to_f<T>(gate[(size_t)t * gate_stride + h * vd + c]));
        out[(size_t)t * H * vd + h * vd + c] = from_f<T>(o);
    }
    if (lane == 0) {
        const int s = tok_seq[t];
        if (cu_seqlens[s + 1] - 1 == t) m_state[(size_t)TK_SLOT(TK_K_RECURRENT, seq_slot[s]) * H + h] = m;
    }
}

// num float32 [T, H, vd + 1], m_out float32 [T, H] (what tk_mlstm_scan left); weight float32 [H vd];
// gate [T, >= H vd] with a row stride, or null; out [T, H vd] contiguous; m_state float32 [slots, H].
TK_API int tk_mlstm_norm_gate(const float* num, const float* m_out, float* m_state, const float* weight,
                              const void* gate, int64_t gate_stride, const int* tok_seq, const int* cu_seqlens,
                              const int* seq_slot, void* out, int T_, int H, int vd, float eps, int dtype,
                              cudaStream_t stream) {
    TK_CHECK_ARG(T_ >= 0 && H > 0 && vd > 0, "matrix memory: bad sizes");
    if (T_ == 0) return 0;
    dim3 grid((T_ * H + 3) / 4);
    if (dtype == TK_F32)
        tk_launch(mlstm_norm_gate_kernel<float>, grid, dim3(128), 0, stream, num, m_out, m_state, weight,
                  (const float*)gate, gate_stride, tok_seq, cu_seqlens, seq_slot, (float*)out, T_, H, vd, eps);
    else if (dtype == TK_BF16)
        tk_launch(mlstm_norm_gate_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, num, m_out, m_state, weight,
                  (const __nv_bfloat16*)gate, gate_stride, tok_seq, cu_seqlens, seq_slot, (__nv_bfloat16*)out, T_, H,
                  vd, eps);
    else
        TK_CHECK_ARG(false, "matrix memory: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("mlstm_norm_gate");
    return 0;
}
