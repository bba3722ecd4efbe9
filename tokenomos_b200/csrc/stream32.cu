// Row-wise kernels for models whose residual stream is kept in 32-bit whatever the storage type
// of the activations: the stream's adds with the RMSNorm that follows them, a clamped gated
// activation, and an element-wise sigmoid gate. Inputs and outputs of the projections around
// them are float or bfloat16 (T); every sum, statistic and product here is formed in 32-bit and
// a T output is rounded exactly once.
#include <math.h>

#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// stream' = stream + x + rows + vec  (each addend optional, added in this order, 32-bit);
// y = T(stream' * rsqrt(mean(stream'^2) + eps) * w)   (w optional: without it only the adds)
// One block per row. A thread keeps its elements of the row in registers when the row is short
// enough (ITEMS per thread), else it reads its own writes back from stream_out.
// ---------------------------------------------------------------------------------------------
template <typename T, int ITEMS>
__global__ void __launch_bounds__(256)
stream32_add_norm_kernel(const float* stream_in, const T* x, int64_t x_stride, const T* rows_add,
                         const float* __restrict__ vec_add, const float* __restrict__ w, float eps,
                         float* stream_out, T* y, float* y32, int width) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    auto sum_at = [&](int i) {
        float v = stream_in != nullptr ? stream_in[r * width + i] : 0.f;
        if (x != nullptr) v += to_f<T>(x[r * x_stride + i]);
        if (rows_add != nullptr) v += to_f<T>(rows_add[r * width + i]);
        if (vec_add != nullptr) v += vec_add[i];
        if (stream_out != nullptr) stream_out[r * width + i] = v;
        return v;
    };
    float ss = 0.f;
    if constexpr (ITEMS > 0) {
        float keep[ITEMS];
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            keep[k] = i < width ? sum_at(i) : 0.f;
            ss += keep[k] * keep[k];
        }
        if (w == nullptr) return;
        const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < width) {
                const float o = keep[k] * rstd * w[i];
                if (y != nullptr) y[r * width + i] = from_f<T>(o);
                if (y32 != nullptr) y32[r * width + i] = o;
            }
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float v = sum_at(i);
            ss += v * v;
        }
        if (w == nullptr) return;
        const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float o = stream_out[r * width + i] * rstd * w[i];
            if (y != nullptr) y[r * width + i] = from_f<T>(o);
            if (y32 != nullptr) y32[r * width + i] = o;
        }
    }
}

// The same with 16 bytes of the stream (four elements) per thread and step, the row in registers:
// one trip to memory. Needs width % 4 == 0, rows of x a multiple of four elements apart, every
// base 16-byte aligned (8-byte for 16-bit inputs), and width <= 4 * ITEMS * blockDim.
template <typename T>
struct Quad {
    static __device__ __forceinline__ float4 load(const T* p);
    static __device__ __forceinline__ void store(T* p, float4 v);
};
template <>
struct Quad<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <>
struct Quad<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<const uint32_t*>(&a);
        raw.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename T, int ITEMS>
__global__ void __launch_bounds__(256)
stream32_add_norm_vec_kernel(const float* stream_in, const T* x, int64_t x_stride, const T* rows_add,
                             const float* __restrict__ vec_add, const float* __restrict__ w, float eps,
                             float* stream_out, T* y, float* y32, int width) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    float4 keep[ITEMS];
    float ss = 0.f;
    // every load of the row is asked for before the first sum
    float4 a[ITEMS], b[ITEMS], c[ITEMS];
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        a[k] = b[k] = c[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < width) {
            if (stream_in != nullptr) a[k] = *reinterpret_cast<const float4*>(stream_in + r * width + i);
            if (x != nullptr) b[k] = Quad<T>::load(x + r * x_stride + i);
            if (rows_add != nullptr) c[k] = Quad<T>::load(rows_add + r * width + i);
        }
    }
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < width) {
            // (the same order of sums as the scalar kernel: stream, x, rows, vector)
            v = a[k];
            if (x != nullptr) v = make_float4(v.x + b[k].x, v.y + b[k].y, v.z + b[k].z, v.w + b[k].w);
            if (rows_add != nullptr) v = make_float4(v.x + c[k].x, v.y + c[k].y, v.z + c[k].z, v.w + c[k].w);
            if (vec_add != nullptr) {
                const float4 d = *reinterpret_cast<const float4*>(vec_add + i);
                v = make_float4(v.x + d.x, v.y + d.y, v.z + d.z, v.w + d.w);
            }
            if (stream_out != nullptr) *reinterpret_cast<float4*>(stream_out + r * width + i) = v;
        }
        keep[k] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (w == nullptr) return;
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        if (i < width) {
            const float4 g = *reinterpret_cast<const float4*>(w + i);
            const float4 o = make_float4(keep[k].x * rstd * g.x, keep[k].y * rstd * g.y, keep[k].z * rstd * g.z,
                                         keep[k].w * rstd * g.w);
            if (y != nullptr) Quad<T>::store(y + r * width + i, o);
            if (y32 != nullptr) *reinterpret_cast<float4*>(y32 + r * width + i) = o;
        }
    }
}

template <typename T>
static int launch_stream32(const float* stream_in, const void* x, int64_t x_stride, const void* rows_add,
                           const float* vec_add, const float* w, float eps, float* stream_out, void* y,
                           float* y32, int rows, int width, cudaStream_t stream) {
    const int threads = width >= 1024 ? 256 : 128;
    const int per_thread = (width + threads - 1) / threads;
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    const bool vec = width % 4 == 0 && x_stride % 4 == 0 && aligned(stream_in) && aligned(stream_out) &&
                     aligned(vec_add) && aligned(w) && aligned(y32) && ((uintptr_t)x & 7) == 0 && ((uintptr_t)rows_add & 7) == 0 &&
                     ((uintptr_t)y & 7) == 0 && (sizeof(T) == 2 || (aligned(x) && aligned(rows_add) && aligned(y)));
    if (vec && width <= 4 * 2 * threads) {
        tk_launch(stream32_add_norm_vec_kernel<T, 2>, dim3(rows), dim3(threads), 0, stream, stream_in, (const T*)x,
                  x_stride, (const T*)rows_add, vec_add, w, eps, stream_out, (T*)y, y32, width);
        return 0;
    }
    if (vec && width <= 4 * 6 * threads) {
        tk_launch(stream32_add_norm_vec_kernel<T, 6>, dim3(rows), dim3(threads), 0, stream, stream_in, (const T*)x,
                  x_stride, (const T*)rows_add, vec_add, w, eps, stream_out, (T*)y, y32, width);
        return 0;
    }
    if (per_thread <= 8)
        tk_launch(stream32_add_norm_kernel<T, 8>, dim3(rows), dim3(threads), 0, stream, stream_in, (const T*)x,
                  x_stride, (const T*)rows_add, vec_add, w, eps, stream_out, (T*)y, y32, width);
    else
        tk_launch(stream32_add_norm_kernel<T, 0>, dim3(rows), dim3(threads), 0, stream, stream_in, (const T*)x,
                  x_stride, (const T*)rows_add, vec_add, w, eps, stream_out, (T*)y, y32, width);
    return 0;
}

// stream_in / stream_out: float [rows, width] (may be the same buffer; stream_out may be null only
// when the row fits the register path, i.e. width <= 2048, and the new stream is not wanted);
// x: T rows `x_stride` elements apart; rows_add: T [rows, width]; vec_add, w: float [width].
TK_API int tk_stream32_add_norm(const float* stream_in, const void* x, int64_t x_stride, const void* rows_add,
                                const float* vec_add, const float* w, float eps, float* stream_out, void* y,
                                float* y32, int rows, int width, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && width > 0, "stream32_add_norm: bad sizes rows=%d width=%d", rows, width);
    TK_CHECK_ARG(stream_in != nullptr || x != nullptr || rows_add != nullptr, "stream32_add_norm: nothing to add up");
    TK_CHECK_ARG(stream_out != nullptr || (w != nullptr && width <= 2048),
                 "stream32_add_norm: a row of %d without a stream to write", width);
    TK_CHECK_ARG(w == nullptr || y != nullptr || y32 != nullptr, "stream32_add_norm: a norm weight without an output");
    if (rows == 0) return 0;
    if (dtype == TK_F32)
        launch_stream32<float>(stream_in, x, x_stride, rows_add, vec_add, w, eps, stream_out, y, y32, rows, width, stream);
    else if (dtype == TK_BF16)
        launch_stream32<__nv_bfloat16>(stream_in, x, x_stride, rows_add, vec_add, w, eps, stream_out, y, y32, rows,
                                       width, stream);
    else
        TK_CHECK_ARG(false, "stream32_add_norm: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("stream32_add_norm");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// clamped gated activation: g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + shift); gu = [gate (inter) | up (inter)] per row, or
// (block > 0) gate and up alternating in runs of `block` channels, the layout a decode product
// with the activation in its epilogue wants of the weight rows. limit <= 0: no clamp.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void glu_clamped_kernel(const T* gu, T* out, int inter, int block, float limit, float alpha, float shift) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const T* row = gu + t * 2 * inter;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < inter; c += gridDim.y * blockDim.x) {
        const int gi = block > 0 ? (c / block) * 2 * block + c % block : c;
        float g = to_f<T>(row[gi]);
        float u = to_f<T>(row[block > 0 ? gi + block : inter + c]);
        if (limit > 0.f) {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
        }
        out[t * inter + c] = from_f<T>(g / (1.0f + expf(-alpha * g)) * (u + shift));
    }
}

// 16 bytes of gate and of up per thread (bfloat16, inter % 8 == 0): the sigmoid through the
// special-function unit's exponential and reciprocal, whose error (a few ulp of a float) is far
// below the one 16-bit rounding that follows.
__global__ void __launch_bounds__(256)
glu_clamped_vec_kernel(const __nv_bfloat16* gu, __nv_bfloat16* out, int inter, int block, float limit, float alpha,
                       float shift) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const __nv_bfloat16* row = gu + t * 2 * inter;
    const float k = -alpha * 1.4426950408889634f;
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8; c < inter; c += gridDim.y * blockDim.x * 8) {
        const int gi = block > 0 ? (c / block) * 2 * block + c % block : c;
        const uint4 graw = *reinterpret_cast<const uint4*>(row + gi);
        const uint4 uraw = *reinterpret_cast<const uint4*>(row + (block > 0 ? gi + block : inter + c));
        const uint32_t* g2 = reinterpret_cast<const uint32_t*>(&graw);
        const uint32_t* u2 = reinterpret_cast<const uint32_t*>(&uraw);
        uint4 packed;
        uint32_t* o2 = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float2 g = make_float2(__uint_as_float(g2[e] << 16), __uint_as_float(g2[e] & 0xffff0000u));
            float2 u = make_float2(__uint_as_float(u2[e] << 16), __uint_as_float(u2[e] & 0xffff0000u));
            if (limit > 0.f) {
                g.x = fminf(g.x, limit), g.y = fminf(g.y, limit);
                u.x = fminf(fmaxf(u.x, -limit), limit), u.y = fminf(fmaxf(u.y, -limit), limit);
            }
            const float a = g.x * rcp_approx(1.0f + ex2_approx(g.x * k)) * (u.x + shift);
            const float b = g.y * rcp_approx(1.0f + ex2_approx(g.y * k)) * (u.y + shift);
            const __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
            o2[e] = *reinterpret_cast<const uint32_t*>(&r);
        }
        *reinterpret_cast<uint4*>(out + t * inter + c) = packed;
    }
}

TK_API int tk_glu_clamped(const void* gu, void* out, int rows, int inter, int block, float limit, float alpha,
                          float shift, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && inter > 0, "glu_clamped: bad sizes rows=%d inter=%d", rows, inter);
    TK_CHECK_ARG(block >= 0 && (block == 0 || inter % block == 0), "glu_clamped: runs of %d channels do not divide %d",
                 block, inter);
    if (rows == 0) return 0;
    const int threads = 256;
    const dim3 grid(rows, min(ceil_div(inter, threads), 64));
    if (dtype == TK_BF16 && inter % 8 == 0 && (block == 0 || block % 8 == 0) && (uintptr_t)gu % 16 == 0 &&
        (uintptr_t)out % 16 == 0) {
        tk_launch(glu_clamped_vec_kernel, dim3(rows, min(ceil_div(inter, threads * 8), 64)), dim3(threads), 0, stream,
                  (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inter, block, limit, alpha, shift);
        TK_CHECK_LAUNCH("glu_clamped_vec");
        return 0;
    }
    if (dtype == TK_F32)
        tk_launch(glu_clamped_kernel<float>, grid, dim3(threads), 0, stream, (const float*)gu, (float*)out, inter, block,
                  limit, alpha, shift);
    else if (dtype == TK_BF16)
        tk_launch(glu_clamped_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)gu,
                  (__nv_bfloat16*)out, inter, block, limit, alpha, shift);
    else
        TK_CHECK_ARG(false, "glu_clamped: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("glu_clamped");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// element-wise sigmoid gate, in place: x[t, c] = T(x[t, c] * sigmoid(g[t, c])); g's rows may be
// `ldg` elements apart (a column block of a wider projection's output)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void sigmoid_gate_kernel(T* x, const T* g, int64_t ldg, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
        const float gate = to_f<T>(g[t * ldg + c]);
        x[t * width + c] = from_f<T>(to_f<T>(x[t * width + c]) / (1.0f + expf(-gate)));
    }
}

TK_API int tk_sigmoid_gate(void* x, const void* g, int64_t ldg, int rows, int width, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && width > 0, "sigmoid_gate: bad sizes rows=%d width=%d", rows, width);
    if (rows == 0) return 0;
    const int threads = 256;
    const dim3 grid(rows, min(ceil_div(width, threads), 64));
    if (dtype == TK_F32)
        tk_launch(sigmoid_gate_kernel<float>, grid, dim3(threads), 0, stream, (float*)x, (const float*)g, ldg, width);
    else if (dtype == TK_BF16)
        tk_launch(sigmoid_gate_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (__nv_bfloat16*)x,
                  (const __nv_bfloat16*)g, ldg, width);
    else
        TK_CHECK_ARG(false, "sigmoid_gate: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("sigmoid_gate");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// The stream's add with a norm in groups, and a gate on what is added:
//   stream' = stream + x * sigmoid(gate)      (x optional; gate optional: the plain add)
//   y = T(stream' / sqrt(mean_group(stream'^2) + eps) * w)
// The row is split into `groups` equal consecutive parts, each divided by its own root mean square.
// One warp per (row, group); a lane keeps its elements in registers when the group is short enough
// (ITEMS per lane: 4 elements at a time where VEC, which wants the group a multiple of 4 and every
// row 16-byte aligned), else it reads its own writes back from stream_out.
// ---------------------------------------------------------------------------------------------
// sigmoid(g): 16-bit storage takes the special-function unit's exponential and reciprocal (a few ulp of a
// float, far below the rounding of the gate itself), 32-bit storage the accurate functions
template <typename T>
__device__ __forceinline__ float gate_of(float g) {
    if constexpr (sizeof(T) == 2) return rcp_approx(1.0f + ex2_approx(g * TK_NEG_LOG2E));
    return 1.0f / (1.0f + expf(-g));
}

template <typename T, int ITEMS, bool VEC>
__global__ void __launch_bounds__(128)
stream32_group_norm_kernel(const float* stream_in, const T* x, int64_t x_stride, const T* gate, int64_t gate_stride,
                           const float* __restrict__ w, float eps, float* stream_out, T* y, int rows, int width,
                           int groups) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (warp >= rows * groups) return;
    const int gw = width / groups, c0 = (warp % groups) * gw;
    const size_t r = warp / groups;
    if constexpr (VEC) {
        float4 keep[ITEMS];
        float4 a[ITEMS], b[ITEMS], g[ITEMS];
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int i = (lane + 32 * k) * 4;
            a[k] = b[k] = g[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < gw) {
                if (stream_in != nullptr) a[k] = *reinterpret_cast<const float4*>(stream_in + r * width + c0 + i);
                if (x != nullptr) b[k] = Quad<T>::load(x + r * x_stride + c0 + i);
                if (gate != nullptr) g[k] = Quad<T>::load(gate + r * gate_stride + c0 + i);
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int i = (lane + 32 * k) * 4;
            float4 v = a[k];
            if (x != nullptr) {
                if (gate != nullptr) {
                    b[k].x *= gate_of<T>(g[k].x), b[k].y *= gate_of<T>(g[k].y);
                    b[k].z *= gate_of<T>(g[k].z), b[k].w *= gate_of<T>(g[k].w);
                }
                v = make_float4(v.x + b[k].x, v.y + b[k].y, v.z + b[k].z, v.w + b[k].w);
            }
            if (i < gw && stream_out != nullptr) *reinterpret_cast<float4*>(stream_out + r * width + c0 + i) = v;
            keep[k] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        if (w == nullptr) return;
        const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)gw + eps);
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int i = (lane + 32 * k) * 4;
            if (i < gw) {
                const float4 q = *reinterpret_cast<const float4*>(w + c0 + i);
                Quad<T>::store(y + r * width + c0 + i, make_float4(keep[k].x * rstd * q.x, keep[k].y * rstd * q.y,
                                                                   keep[k].z * rstd * q.z, keep[k].w * rstd * q.w));
            }
        }
    } else {
        auto sum_at = [&](int i) {
            float v = stream_in != nullptr ? stream_in[r * width + c0 + i] : 0.f;
            if (x != nullptr) {
                float add = to_f<T>(x[r * x_stride + c0 + i]);
                if (gate != nullptr) add *= gate_of<T>(to_f<T>(gate[r * gate_stride + c0 + i]));
                v += add;
            }
            if (stream_out != nullptr) stream_out[r * width + c0 + i] = v;
            return v;
        };
        float ss = 0.f;
        if constexpr (ITEMS > 0) {
            float keep[ITEMS];
#pragma unroll
            for (int k = 0; k < ITEMS; ++k) {
                const int i = lane + 32 * k;
                keep[k] = i < gw ? sum_at(i) : 0.f;
                ss += keep[k] * keep[k];
            }
            if (w == nullptr) return;
            const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)gw + eps);
#pragma unroll
            for (int k = 0; k < ITEMS; ++k) {
                const int i = lane + 32 * k;
                if (i < gw) y[r * width + c0 + i] = from_f<T>(keep[k] * rstd * w[c0 + i]);
            }
        } else {
            for (int i = lane; i < gw; i += 32) {
                const float v = sum_at(i);
                ss += v * v;
            }
            if (w == nullptr) return;
            const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)gw + eps);
            for (int i = lane; i < gw; i += 32)
                y[r * width + c0 + i] = from_f<T>(stream_out[r * width + c0 + i] * rstd * w[c0 + i]);
        }
    }
}

template <typename T>
static void launch_group_norm(const float* stream_in, const void* x, int64_t x_stride, const void* gate,
                              int64_t gate_stride, const float* w, float eps, float* stream_out, void* y, int rows,
                              int width, int groups, cudaStream_t stream) {
    const int gw = width / groups;
    const int warps = rows * groups;
    dim3 grid((warps + 3) / 4), block(128);
    auto aligned = [](const void* p, int to) { return ((uintptr_t)p & (to - 1)) == 0; };
    const int tb = sizeof(T) == 2 ? 8 : 16;
    const bool vec = gw % 4 == 0 && x_stride % 4 == 0 && gate_stride % 4 == 0 && aligned(stream_in, 16) &&
                     aligned(stream_out, 16) && aligned(w, 16) && aligned(x, tb) && aligned(gate, tb) && aligned(y, tb);
#define TK_GN(ITEMS, VEC)                                                                                          \
    tk_launch(stream32_group_norm_kernel<T, ITEMS, VEC>, grid, block, 0, stream, stream_in, (const T*)x, x_stride,  \
              (const T*)gate, gate_stride, w, eps, stream_out, (T*)y, rows, width, groups)
    if (vec && gw <= 128 * 1) TK_GN(1, true);
    else if (vec && gw <= 128 * 2) TK_GN(2, true);
    else if (vec && gw <= 128 * 4) TK_GN(4, true);
    else if (vec && gw <= 128 * 8) TK_GN(8, true);
    else if (gw <= 32 * 8) TK_GN(8, false);
    else TK_GN(0, false);
#undef TK_GN
}

// stream_in / stream_out: float [rows, width] (may be the same buffer; stream_out may be null only when
// a group fits the register path, gw <= 256 or, 16-byte aligned, 1024); x, gate: T rows `x_stride` /
// `gate_stride` elements apart; w: float [width] or null (the add alone).
TK_API int tk_stream32_group_norm(const float* stream_in, const void* x, int64_t x_stride, const void* gate,
                                  int64_t gate_stride, const float* w, float eps, float* stream_out, void* y, int rows,
                                  int width, int groups, int dtype, cudaStream_t stream) {
    TK_CHECK_ARG(rows >= 0 && width > 0 && groups > 0 && width % groups == 0,
                 "stream32_group_norm: a row of %d in %d groups", width, groups);
    TK_CHECK_ARG(stream_in != nullptr || x != nullptr, "stream32_group_norm: nothing to add up");
    TK_CHECK_ARG(gate == nullptr || x != nullptr, "stream32_group_norm: a gate without rows to gate");
    TK_CHECK_ARG(stream_out != nullptr, "stream32_group_norm: no stream to write");
    TK_CHECK_ARG(w == nullptr || y != nullptr, "stream32_group_norm: a norm weight without an output");
    if (rows == 0) return 0;
    if (dtype == TK_F32)
        launch_group_norm<float>(stream_in, x, x_stride, gate, gate_stride, w, eps, stream_out, y, rows, width, groups,
                                 stream);
    else if (dtype == TK_BF16)
        launch_group_norm<__nv_bfloat16>(stream_in, x, x_stride, gate, gate_stride, w, eps, stream_out, y, rows, width,
                                         groups, stream);
    else
        TK_CHECK_ARG(false, "stream32_group_norm: unknown dtype %d", dtype);
    TK_CHECK_LAUNCH("stream32_group_norm");
    return 0;
}
