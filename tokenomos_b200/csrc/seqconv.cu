// Causal convolution over time on each channel, with its state:
//
//     y_t[c] = (residual ? u_t[c] : 0) + bias[c] + sum_j taps[c, j] * u_(t - K + 1 + j)[c]
//
// (`act` 1: y <- silu(y), formed in 32-bit before the one rounding)
// within each sequence, zeros before its start; the last K - 1 inputs u of every sequence are the
// request's state (float32 [slots, K - 1, C]; a 16-bit input widens exactly). The input rows may
// be a column block of a wider tensor (a fused projection). The channels from `c_paged` on do not
// go to `out` but into a paged key/value pool [pages, 2, Hkv, P, Dp]: Hkv key heads of Dk
// channels, then Hkv value heads of Dv, each token's row at its position through the block table.
// `plain`: the input itself in the output's type, written beside the result (what another reader
// of the same rows takes).
//
// One block per (tile of consecutive tokens of one sequence, 256 channels); a thread walks its
// tile's tokens with the last K - 1 inputs in registers. Only the tile at offset 0 of a portion
// reads the state, and it alone writes it, after reading: tiles are at least K - 1 tokens long,
// so no later tile needs the state.
#include "common.cuh"

namespace {
enum : int { TK_K_SEQ_CONV = 8 };
constexpr int MAX_TAPS = 8;

struct PagedDest {
    void* pool;              // nullptr: no paged channels
    const int* block_table;  // [S, bt_stride]
    int bt_stride, P, Hkv, Dk, Dv, Dp;
};
}  // namespace

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
seq_conv_kernel(const TI* in, int64_t in_stride, const float* __restrict__ taps, const float* __restrict__ bias,
                float* state, const int* cu_seqlens, const int* seq_ctx, const int* seq_slot,
                const int* tile_seq, const int* tile_tok0, const int* tile_off, const int* tile_n, TO* out,
                int64_t out_stride, TO* plain, int64_t plain_stride, int K, int C, int residual, int act,
                int c_paged, PagedDest dest) {
    pdl_launch_dependents();
    pdl_wait();
    // The walk is bound by the latency of dependent loads, so they are asked for as early as their
    // addresses are known: the tile's four numbers together, then the tile's first inputs and the
    // inputs before it beside the sequence's numbers (only the choice between those inputs and the
    // state needs the sequence's context).
    constexpr int AHEAD = 8;                          // inputs in flight
    const int n = tile_n[blockIdx.x], s = tile_seq[blockIdx.x], tok0 = tile_tok0[blockIdx.x], off = tile_off[blockIdx.x];
    if (n <= 0) return;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float ahead[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) ahead[k] = to_f<TI>(in[(size_t)(tok0 + min(k, n - 1)) * in_stride + c]);
    float before[MAX_TAPS];                           // before[d - 1]: the input d tokens back within the portion
#pragma unroll
    for (int d = 1; d < MAX_TAPS; ++d)
        before[d - 1] = (d < K && off - d >= 0) ? to_f<TI>(in[(size_t)(tok0 - d) * in_stride + c]) : 0.f;
    const int ctx = seq_ctx[s];
    const int pos0 = ctx + off;                       // position of the tile's first token
    float w[MAX_TAPS], past[MAX_TAPS];                // past[d - 1]: the input d positions back
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) w[j] = j < K ? taps[(size_t)c * K + j] : 0.f;
    const float b = bias != nullptr ? bias[c] : 0.f;
    float* st = (state != nullptr && K > 1)
                    ? state + (size_t)TK_SLOT(TK_K_SEQ_CONV, seq_slot[s]) * (K - 1) * C + c : nullptr;
    float old[MAX_TAPS];                              // the state as it was (offset-0 tiles)
#pragma unroll
    for (int r = 0; r < MAX_TAPS; ++r) old[r] = 0.f;
    if (off == 0 && ctx > 0 && st != nullptr) {
#pragma unroll
        for (int r = 0; r < MAX_TAPS - 1; ++r)
            if (r < K - 1) old[r] = st[(size_t)r * C];           // row r: position ctx - (K - 1) + r
    }
#pragma unroll
    for (int d = 1; d < MAX_TAPS; ++d) {
        float v = 0.f;
        if (d < K && pos0 - d >= 0) {
            if (off - d >= 0) v = before[d - 1];
            else v = old[K - 1 - d];                  // off == 0 (tiles are >= K - 1 long) and ctx > 0
        }
        past[d - 1] = v;
    }
    // where this channel's results go
    const bool paged = dest.pool != nullptr && c >= c_paged;
    size_t page_part = 0;                             // offset within a page
    if (paged) {
        const int cc = c - c_paged;
        const int keys = dest.Hkv * dest.Dk;
        const int which = cc >= keys;
        const int e = which ? cc - keys : cc;
        const int D = which ? dest.Dv : dest.Dk;
        page_part = ((size_t)which * dest.Hkv + e / D) * dest.P * dest.Dp + e % D;
    }
    const size_t page_size = (size_t)2 * dest.Hkv * dest.P * dest.Dp;
    for (int i0 = 0; i0 < n; i0 += AHEAD) {
        if (i0 > 0) {
#pragma unroll
            for (int k = 0; k < AHEAD; ++k)
                ahead[k] = to_f<TI>(in[(size_t)(tok0 + min(i0 + k, n - 1)) * in_stride + c]);
        }
#pragma unroll
        for (int k = 0; k < AHEAD; ++k) {
            const int i = i0 + k;
            if (i >= n) break;
            const float cur = ahead[k];
            float acc = (residual ? cur : 0.f) + b;
            acc = fmaf(w[K - 1], cur, acc);
#pragma unroll
            for (int d = 1; d < MAX_TAPS; ++d)
                if (d < K) acc = fmaf(w[K - 1 - d], past[d - 1], acc);
            if (act) acc = acc / (1.0f + expf(-acc));
            if (paged) {
                const int pos = pos0 + i;
                const int page = TK_PAGE(TK_K_SEQ_CONV, dest.block_table[(size_t)s * dest.bt_stride + pos / dest.P]);
                reinterpret_cast<TO*>(dest.pool)[(size_t)page * page_size + page_part + (size_t)(pos % dest.P) * dest.Dp] =
                    from_f<TO>(acc);
            } else {
                out[(size_t)(tok0 + i) * out_stride + c] = from_f<TO>(acc);
                if (plain != nullptr) plain[(size_t)(tok0 + i) * plain_stride + c] = from_f<TO>(cur);
            }
#pragma unroll
            for (int d = MAX_TAPS - 1; d >= 2; --d) past[d - 1] = past[d - 2];
            past[0] = cur;
        }
    }
    if (off == 0 && st != nullptr) {
        const int first = cu_seqlens[s], len = cu_seqlens[s + 1] - first;
        // row r of the new state: position ctx + len - (K - 1) + r
#pragma unroll
        for (int r = 0; r < MAX_TAPS - 1; ++r) {
            if (r >= K - 1) break;
            const int p = len - (K - 1) + r;          // relative to the portion's first token
            float v = 0.f;
            if (p >= 0) v = to_f<TI>(in[(size_t)(first + p) * in_stride + c]);
            else if (ctx + p >= 0) v = old[r + len];  // old row of position ctx + p
            st[(size_t)r * C] = v;
        }
    }
}

// in: [T, >= C] with row stride in_stride (type in_dtype); taps float32 [C, K]; bias float32 [C] or
// null; state float32 [slots, K - 1, C] (null with K == 1); tiles: runs of one sequence's
// consecutive tokens, each at least K - 1 long but for a portion's last; out: [T, >= c_paged or C]
// (type out_dtype), plain likewise or null; pool (type out_dtype) null: every channel goes to out.
TK_API int tk_seq_conv(const void* in, int64_t in_stride, int in_dtype, const float* taps, const float* bias,
                       float* state, const int* cu_seqlens, const int* seq_ctx, const int* seq_slot,
                       const int* tile_seq, const int* tile_tok0, const int* tile_off, const int* tile_n,
                       int n_tiles, void* out, int64_t out_stride, void* plain, int64_t plain_stride, int out_dtype,
                       int K, int C, int residual, int act, int c_paged, void* pool, const int* block_table,
                       int bt_stride, int P, int Hkv, int Dk, int Dv, int Dp, cudaStream_t stream) {
    TK_CHECK_ARG(K >= 1 && K <= MAX_TAPS, "sequence conv: %d taps; 1..%d are built", K, MAX_TAPS);
    TK_CHECK_ARG(K == 1 || state != nullptr, "sequence conv: %d taps need a state", K);
    TK_CHECK_ARG(C > 0 && n_tiles >= 0, "sequence conv: bad sizes");
    TK_CHECK_ARG(!(in_dtype == TK_BF16 && out_dtype == TK_F32), "sequence conv: a 16-bit input with a 32-bit output is not built");
    if (pool != nullptr) {
        TK_CHECK_ARG(block_table != nullptr && P > 0 && Hkv > 0 && Dk > 0 && Dv > 0 && Dp >= Dk && Dp >= Dv &&
                         c_paged >= 0 && c_paged + Hkv * (Dk + Dv) == C,
                     "sequence conv: %d channels do not end in %d key/value heads of %d and %d", C, Hkv, Dk, Dv);
    } else {
        c_paged = C;
    }
    TK_CHECK_ARG(out != nullptr || c_paged == 0, "sequence conv: no output");
    if (n_tiles == 0) return 0;
    PagedDest dest{pool, block_table, bt_stride, P, Hkv, Dk, Dv, Dp};
    dim3 grid(n_tiles, (C + 255) / 256);
#define TK_SC(TI, TO)                                                                                       \
    tk_launch(seq_conv_kernel<TI, TO>, grid, dim3(256), 0, stream, (const TI*)in, in_stride, taps, bias,    \
              state, cu_seqlens, seq_ctx, seq_slot, tile_seq, tile_tok0, tile_off, tile_n, (TO*)out,        \
              out_stride, (TO*)plain, plain_stride, K, C, residual, act, c_paged, dest)
    if (in_dtype == TK_F32 && out_dtype == TK_F32) TK_SC(float, float);
    else if (in_dtype == TK_F32 && out_dtype == TK_BF16) TK_SC(float, __nv_bfloat16);
    else if (in_dtype == TK_BF16 && out_dtype == TK_BF16) TK_SC(__nv_bfloat16, __nv_bfloat16);
    else TK_CHECK_ARG(false, "sequence conv: unknown dtypes %d -> %d", in_dtype, out_dtype);
#undef TK_SC
    TK_CHECK_LAUNCH("seq_conv");
    return 0;
}
