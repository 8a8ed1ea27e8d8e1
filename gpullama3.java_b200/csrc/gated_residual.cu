// Kernels of a block whose sublayers read the 32-bit residual stream as it is and whose results are gated, normed and
// then added:
//
//   gated_norm_step    z = (y (+ yb)) * sigmoid(r + rb)                  the sublayer's result y times its gate, whose
//                      x <- x + (z - mean(z)) / sqrt(var(z) + eps) * w + b    logits r come from a product over the
//                      y <- 0 ;  xc = x in the run's type (optional)      sublayer's own input; a layer norm; the sum
//                      the same without a gate and without the mean: x <- x + w * y / sqrt(mean(y^2) + eps)
//                      and, for the last such step of a layer whose results are mixed, depth_average in the same pass
//   depth_average      level[n] = x ;  x <- sum_(j <= n) c[j] level[j] ;  xc = x (optional): every layer's result is
//                      kept for the pass, and what the next layer reads is a learned mix of all of them
//   cast_rows          xc = x in the run's type (what a product over the stream itself reads)
//   bias_act_rows      u <- act(u + bias) in place on a product's result; act: the square of max(., 0)
//   token_gate_rows    g[t, j] = gelu_tanh(a[t, j]) * table[token[t], j]: a few numbers per token id that the stream gates
//
// Every kernel here is launched with programmatic dependent launch and waits for its predecessor before it touches memory.
// A CTA per token row for the three steps: a thread keeps its share of the row (the elements tid, tid + 256, ...) in
// registers between the one fetch and the one store when the row has at most 256 * 32 numbers; longer rows are
// evaluated again in each pass.  Mean and variance are two sums over the same kept values (the variance is the mean of
// the squared deviations), every sum in a fixed order.  All arithmetic is 32-bit.
#include "common.cuh"

namespace b200 {

constexpr int kStepThreads = 256;

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

struct GatedNormArgs {
    float* y;               // [T][dim] the sublayer's result, cleared on the way out
    const float* y_bias;    // [dim] or null
    const void* r;          // [T][ld_r] gate logits (32-bit or the run's type), or null (no gate)
    int ld_r;
    const float* r_bias;    // [dim] or null
    const float* w;         // [dim]
    const float* b;         // [dim] or null (rms form: no mean taken off, no bias)
    float* x;               // [T][dim]
    void* xc;               // [T][dim] in the run's type, or null
    int dim;
    float eps;
    int center;             // 1: layer norm; 0: divide by the root mean square only
    float* levels;          // [> n][level_stride] or null; not null: the new x is filed as level n and what is left as
    size_t level_stride;    // the stream (and in xc) is sum_(j <= n) c[j] level[j], as depth_average does it
    int n;
    const float* c;         // [n + 1]
    // not null: a step in which every sequence brings one token also reads for the next block's mixer, a convolution
    // over time on the stream as it is left: read = h + sum_j conv_w[:, j] h_(t - taps + 1 + j), the older inputs from
    // conv_state[slots[t]] ([taps - 1][dim], oldest first), which moves on by this token when conv_update
    const float* conv_w;    // [dim][taps]
    float* conv_state;
    size_t slot_stride;
    const int* slots;       // [T]
    int taps, conv_update;
    void* read;             // [T][dim] in xc's type
};

// The next reader's convolution for one number of token t (sums run from the oldest tap to the newest, then the input
// itself, as the convolution kernels do).
template <typename TC>
__device__ __forceinline__ void read_ahead(const GatedNormArgs& a, int t, int i, float v) {
    float* st = a.conv_state + (size_t)a.slots[t] * a.slot_stride + i;
    const float* w = a.conv_w + (size_t)i * a.taps;
    float acc = 0.f;
    for (int m = 0; m + 1 < a.taps; ++m) {
        const float older = st[(size_t)m * a.dim];
        acc += w[m] * older;
        if (a.conv_update && m > 0) st[(size_t)(m - 1) * a.dim] = older;
    }
    if (a.conv_update && a.taps > 1) st[(size_t)(a.taps - 2) * a.dim] = v;
    acc += w[a.taps - 1] * v;
    ((TC*)a.read)[(size_t)t * a.dim + i] = from_f32<TC>(acc + v);
}

// The mix over the levels for one number: files `value` as level n, returns sum_j c[j] level[j] (j in order).
__device__ __forceinline__ float mix_levels(const GatedNormArgs& a, size_t at, float value) {
    a.levels[(size_t)a.n * a.level_stride + at] = value;
    float acc = 0.f;
    for (int j = 0; j < a.n; ++j) acc += a.c[j] * a.levels[(size_t)j * a.level_stride + at];
    return acc + a.c[a.n] * value;
}

// NV > 0: the row's values stay in registers (dim <= NV * kStepThreads); NV == 0: any size, evaluated per pass.
template <typename TR, typename TC, int NV>
__global__ void __launch_bounds__(kStepThreads)
gated_norm_step_kernel(GatedNormArgs a) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x, dim = a.dim;
    float* yr = a.y + (size_t)t * dim;
    float* xr = a.x + (size_t)t * dim;
    const TR* rr = a.r ? (const TR*)a.r + (size_t)t * a.ld_r : nullptr;
    auto value = [&](int i) {
        float z = yr[i] + (a.y_bias ? a.y_bias[i] : 0.f);
        if (rr) z *= sigmoid_f(to_f32<TR>(rr[i]) + (a.r_bias ? a.r_bias[i] : 0.f));
        return z;
    };
    constexpr int N = NV > 0 ? NV : 1;
    float keep[N];
    float sum = 0.f;
    if (NV > 0) {
#pragma unroll
        for (int j = 0; j < N; ++j) {
            const int i = tid + j * kStepThreads;
            keep[j] = i < dim ? value(i) : 0.f;
            sum += keep[j];
        }
    } else {
        for (int i = tid; i < dim; i += kStepThreads) sum += value(i);
    }
    float mean = 0.f;
    if (a.center) mean = block_sum(sum, scratch) / (float)dim;
    float ss = 0.f;
    if (NV > 0) {
#pragma unroll
        for (int j = 0; j < N; ++j) {
            const int i = tid + j * kStepThreads;
            const float d = i < dim ? keep[j] - mean : 0.f;
            ss += d * d;
        }
    } else {
        for (int i = tid; i < dim; i += kStepThreads) {
            const float d = value(i) - mean;
            ss += d * d;
        }
    }
    const float scale = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + a.eps);
    TC* xc = a.xc ? (TC*)a.xc + (size_t)t * dim : nullptr;
    auto finish = [&](int i, float z) {
        float v = xr[i] + ((z - mean) * scale * a.w[i] + (a.b ? a.b[i] : 0.f));
        if (a.levels) v = mix_levels(a, (size_t)t * dim + i, v);
        xr[i] = v;
        yr[i] = 0.f;
        if (xc) xc[i] = from_f32<TC>(v);
        if (a.conv_w) read_ahead<TC>(a, t, i, v);
    };
    if (NV > 0) {
#pragma unroll
        for (int j = 0; j < N; ++j) {
            const int i = tid + j * kStepThreads;
            if (i < dim) finish(i, keep[j]);
        }
    } else {
        for (int i = tid; i < dim; i += kStepThreads) finish(i, value(i));
    }
}

// Four numbers of type T as floats, and back (16-byte or 8-byte accesses; the caller checks the alignment).
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xffff0000u));
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 w;
    w.x = *reinterpret_cast<const uint32_t*>(&lo);
    w.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = w;
}

// The same step for rows of whole groups of four numbers (dim <= 4 NV kStepThreads): a thread keeps NV groups of four in
// registers and moves them with 16-byte accesses, all of a row's fetches in flight together.
template <typename TR, typename TC, int NV>
__global__ void __launch_bounds__(kStepThreads)
gated_norm_step_vec_kernel(GatedNormArgs a) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x, dim = a.dim;
    float* yr = a.y + (size_t)t * dim;
    float* xr = a.x + (size_t)t * dim;
    const TR* rr = a.r ? (const TR*)a.r + (size_t)t * a.ld_r : nullptr;
    float4 z[NV], xv[NV];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = (tid + j * kStepThreads) * 4;
        z[j] = xv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < dim) {
            z[j] = load4<float>(yr + i);
            xv[j] = load4<float>(xr + i);
            if (a.y_bias) {
                const float4 b = load4<float>(a.y_bias + i);
                z[j].x += b.x; z[j].y += b.y; z[j].z += b.z; z[j].w += b.w;
            }
            if (rr) {
                float4 r = load4<TR>(rr + i);
                if (a.r_bias) {
                    const float4 b = load4<float>(a.r_bias + i);
                    r.x += b.x; r.y += b.y; r.z += b.z; r.w += b.w;
                }
                z[j].x *= sigmoid_f(r.x); z[j].y *= sigmoid_f(r.y); z[j].z *= sigmoid_f(r.z); z[j].w *= sigmoid_f(r.w);
            }
            sum += (z[j].x + z[j].y) + (z[j].z + z[j].w);
        }
    }
    float mean = 0.f;
    if (a.center) mean = block_sum(sum, scratch) / (float)dim;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = (tid + j * kStepThreads) * 4;
        if (i < dim) {
            const float d0 = z[j].x - mean, d1 = z[j].y - mean, d2 = z[j].z - mean, d3 = z[j].w - mean;
            ss += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
        }
    }
    const float scale = 1.0f / sqrtf(block_sum(ss, scratch) / (float)dim + a.eps);
    TC* xc = a.xc ? (TC*)a.xc + (size_t)t * dim : nullptr;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = (tid + j * kStepThreads) * 4;
        if (i >= dim) continue;
        const float4 w = load4<float>(a.w + i);
        const float4 b = a.b ? load4<float>(a.b + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 v;
        v.x = xv[j].x + ((z[j].x - mean) * scale * w.x + b.x);
        v.y = xv[j].y + ((z[j].y - mean) * scale * w.y + b.y);
        v.z = xv[j].z + ((z[j].z - mean) * scale * w.z + b.z);
        v.w = xv[j].w + ((z[j].w - mean) * scale * w.w + b.w);
        if (a.levels) {
            const size_t at = (size_t)t * dim + i;
            store4<float>(a.levels + (size_t)a.n * a.level_stride + at, v);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < a.n; ++k) {
                const float4 l = load4<float>(a.levels + (size_t)k * a.level_stride + at);
                const float ck = a.c[k];
                acc.x += ck * l.x; acc.y += ck * l.y; acc.z += ck * l.z; acc.w += ck * l.w;
            }
            const float cn = a.c[a.n];
            v = make_float4(acc.x + cn * v.x, acc.y + cn * v.y, acc.z + cn * v.z, acc.w + cn * v.w);
        }
        store4<float>(xr + i, v);
        store4<float>(yr + i, make_float4(0.f, 0.f, 0.f, 0.f));
        if (xc) store4<TC>(xc + i, v);
        if (a.conv_w) {
            read_ahead<TC>(a, t, i, v.x);
            read_ahead<TC>(a, t, i + 1, v.y);
            read_ahead<TC>(a, t, i + 2, v.z);
            read_ahead<TC>(a, t, i + 3, v.w);
        }
    }
}

// level[n] = x ; x <- sum_j c[j] level[j] (j = 0 .. n, in that order) ; xc = x.  Elementwise: a thread per four numbers
// where the rows allow 16-byte accesses (depth_average_vec_kernel), else per number.
template <typename TR>
__global__ void __launch_bounds__(256)
depth_average_vec_kernel(float* __restrict__ levels, size_t level_stride, int n, const float* __restrict__ c,
                         float* __restrict__ x, TR* __restrict__ xc, size_t total4) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t q = (size_t)blockIdx.x * blockDim.x + threadIdx.x; q < total4; q += (size_t)gridDim.x * blockDim.x) {
        const size_t i = q * 4;
        const float4 newest = load4<float>(x + i);
        store4<float>(levels + (size_t)n * level_stride + i, newest);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < n; ++j) {
            const float4 v = load4<float>(levels + (size_t)j * level_stride + i);
            const float cj = c[j];
            acc.x += cj * v.x; acc.y += cj * v.y; acc.z += cj * v.z; acc.w += cj * v.w;
        }
        const float cn = c[n];
        acc.x += cn * newest.x; acc.y += cn * newest.y; acc.z += cn * newest.z; acc.w += cn * newest.w;
        store4<float>(x + i, acc);
        if (xc) store4<TR>(xc + i, acc);
    }
}

template <typename TR>
__global__ void __launch_bounds__(256)
depth_average_kernel(float* __restrict__ levels, size_t level_stride, int n, const float* __restrict__ c,
                     float* __restrict__ x, TR* __restrict__ xc, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float newest = x[i];
        levels[(size_t)n * level_stride + i] = newest;
        float acc = 0.f;
        for (int j = 0; j < n; ++j) acc += c[j] * levels[(size_t)j * level_stride + i];
        acc += c[n] * newest;
        x[i] = acc;
        if (xc) xc[i] = from_f32<TR>(acc);
    }
}

template <typename TR>
__global__ void __launch_bounds__(256)
cast_rows_kernel(const float* __restrict__ x, TR* __restrict__ xc, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        xc[i] = from_f32<TR>(x[i]);
}

template <typename TR>
__global__ void __launch_bounds__(256)
bias_act_rows_kernel(TR* __restrict__ u, int ld, const float* __restrict__ bias, int n) {
    pdl_launch_dependents();
    pdl_wait();
    TR* ur = u + (size_t)blockIdx.x * ld;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < n; e += gridDim.y * blockDim.x) {
        const float z = fmaxf(to_f32<TR>(ur[e]) + (bias ? bias[e] : 0.f), 0.f);
        ur[e] = from_f32<TR>(z * z);
    }
}

// g[t, j] = gelu_tanh(a[t, j]) * table[token[t]][j] for j < n, zero for n <= j < width (columns a product's K is padded to)
template <typename TR, typename TT>
__global__ void __launch_bounds__(128)
token_gate_rows_kernel(const TR* __restrict__ a, int ld_a, const int* __restrict__ tokens, const TT* __restrict__ table,
                       int ld_table, int n_rows_table, TR* __restrict__ g, int ld_g, int n, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : (tok >= n_rows_table ? n_rows_table - 1 : tok);
    const TT* e = table + (size_t)tok * ld_table;
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        g[(size_t)t * ld_g + j] = from_f32<TR>(j < n ? gelu_tanh_f(to_f32<TR>(a[(size_t)t * ld_a + j])) * to_f32<TT>(e[j]) : 0.f);
}

template <typename TR, typename TC>
static int launch_gated_norm(const GatedNormArgs& a, int n_tokens, cudaStream_t stream) {
    // rows of whole groups of four whose every pointer lies on a 16-byte boundary (8 bytes for 16-bit rows) go four at a time
    const uintptr_t all = (uintptr_t)a.y | (uintptr_t)a.x | (uintptr_t)a.w | (uintptr_t)a.b | (uintptr_t)a.y_bias |
                          (uintptr_t)a.r_bias | (uintptr_t)a.r | (uintptr_t)a.xc | (uintptr_t)a.levels;
    if (a.dim % 4 == 0 && a.ld_r % 4 == 0 && (all & 15) == 0 && a.level_stride % 4 == 0 && a.dim <= 32 * kStepThreads) {
        const int per4 = (a.dim / 4 + kStepThreads - 1) / kStepThreads;
#define B200_GATED_NORM_VEC(NV) \
    return launch_pdl(gated_norm_step_vec_kernel<TR, TC, NV>, dim3(n_tokens), dim3(kStepThreads), 0, stream, a)
        if (per4 <= 1) B200_GATED_NORM_VEC(1);
        else if (per4 <= 2) B200_GATED_NORM_VEC(2);
        else if (per4 <= 4) B200_GATED_NORM_VEC(4);
        else B200_GATED_NORM_VEC(8);
#undef B200_GATED_NORM_VEC
    }
    const int per = (a.dim + kStepThreads - 1) / kStepThreads;
#define B200_GATED_NORM_CASE(NV) \
    return launch_pdl(gated_norm_step_kernel<TR, TC, NV>, dim3(n_tokens), dim3(kStepThreads), 0, stream, a)
    if (per <= 1) B200_GATED_NORM_CASE(1);
    else if (per <= 2) B200_GATED_NORM_CASE(2);
    else if (per <= 4) B200_GATED_NORM_CASE(4);
    else if (per <= 8) B200_GATED_NORM_CASE(8);
    else if (per <= 16) B200_GATED_NORM_CASE(16);
    else if (per <= 32) B200_GATED_NORM_CASE(32);
    else B200_GATED_NORM_CASE(0);
#undef B200_GATED_NORM_CASE
}

}  // namespace b200

// `center` 1: x += layer norm of the gated result (w, b); 0: x += w * z / rms(z) (b ignored).  `r` null: no gate.
// `r_dtype`: the gate logits' type; `dtype`: that of xc.  `levels` not null: the new x is filed as level `n` of
// levels [> n][level_stride] and the stream becomes sum_(j <= n) c[j] level[j] (c on the device), as b200_depth_average does it.
// `conv_w` not null (a step of one token per sequence): `read` receives what the next block's mixer reads (GatedNormArgs).
extern "C" int b200_gated_norm_step(float* y, const float* y_bias, const void* r, int ld_r, int r_dtype, const float* r_bias,
                                    const float* w, const float* b, float* x, void* xc, int dtype, int n_tokens, int dim,
                                    float eps, int center, float* levels, long long level_stride, int n, const float* c,
                                    const float* conv_w, float* conv_state, long long slot_stride, const int* slots, int taps,
                                    int conv_update, void* read, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dim < 1 || !y || !w || !x || (r && ld_r < dim)) return b200::kErrBadArgument;
    if (levels && (n < 0 || !c || level_stride < (long long)n_tokens * dim)) return b200::kErrBadArgument;
    if (conv_w && (!read || !slots || taps < 1 || (taps > 1 && (!conv_state || slot_stride < (long long)(taps - 1) * dim))))
        return b200::kErrBadArgument;
    const b200::GatedNormArgs a = {y, y_bias, r, ld_r, r_bias, w, center ? b : nullptr, x, xc, dim, eps, center ? 1 : 0,
                                   levels, (size_t)(levels ? level_stride : 0), n, c,
                                   conv_w, conv_state, (size_t)slot_stride, slots, taps, conv_update, read};
    B200_DISPATCH_DTYPE(r_dtype, TR, B200_DISPATCH_DTYPE2(dtype, TC, return b200::launch_gated_norm<TR, TC>(a, n_tokens, stream)));
    return 0;
}

// levels [>= n + 1][level_stride] 32-bit; c [n + 1] on the device; x [total] becomes the mix, its old value level n.
extern "C" int b200_depth_average(float* levels, long long level_stride, int n, const float* c, float* x, void* xc, int dtype,
                                  long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (n < 0 || !levels || !c || !x || level_stride < total) return b200::kErrBadArgument;
    if (total % 4 == 0 && level_stride % 4 == 0 && (((uintptr_t)levels | (uintptr_t)x | (uintptr_t)xc) & 15) == 0) {
        const long long blocks4 = (total / 4 + 255) / 256;
        const int grid4 = (int)(blocks4 < 148 * 16 ? blocks4 : 148 * 16);
        B200_DISPATCH_DTYPE(dtype, T,
            return b200::launch_pdl(b200::depth_average_vec_kernel<T>, dim3(grid4), dim3(256), 0, stream, levels,
                                    (size_t)level_stride, n, c, x, (T*)xc, (size_t)(total / 4)));
    }
    const long long blocks = (total + 255) / 256;
    const int grid = (int)(blocks < 148 * 16 ? blocks : 148 * 16);
    B200_DISPATCH_DTYPE(dtype, T,
        return b200::launch_pdl(b200::depth_average_kernel<T>, dim3(grid), dim3(256), 0, stream, levels, (size_t)level_stride, n, c,
                                x, (T*)xc, (size_t)total));
    return 0;
}

extern "C" int b200_cast_rows(const float* x, void* xc, int dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const long long blocks = (total + 255) / 256;
    const int grid = (int)(blocks < 148 * 16 ? blocks : 148 * 16);
    B200_DISPATCH_DTYPE(dtype, T, return b200::launch_pdl(b200::cast_rows_kernel<T>, dim3(grid), dim3(256), 0, stream, x, (T*)xc,
                                                          (size_t)total));
    return 0;
}

// act 0: max(u + bias, 0)^2
extern "C" int b200_bias_act_rows(void* u, int ld, int dtype, const float* bias, int n_tokens, int n, int act,
                                  cudaStream_t stream) {
    if (act != 0) return b200::kErrBadArgument;
    if (n_tokens <= 0 || n <= 0) return 0;
    const int ny = (n + 1023) / 1024;
    B200_DISPATCH_DTYPE(dtype, T,
        return b200::launch_pdl(b200::bias_act_rows_kernel<T>, dim3(n_tokens, ny > 64 ? 64 : ny), dim3(256), 0, stream, (T*)u, ld,
                                bias, n));
    return 0;
}

extern "C" int b200_token_gate_rows(const void* a, int ld_a, int dtype, const int* tokens, const void* table, int table_dtype,
                                    int ld_table, int n_rows_table, void* g, int ld_g, int n_tokens, int n, int width,
                                    cudaStream_t stream) {
    if (n_tokens <= 0 || width <= 0) return 0;
    if (n < 0 || n > width || ld_g < width || n_rows_table < 1) return b200::kErrBadArgument;
    B200_DISPATCH_DTYPE(dtype, T,
        B200_DISPATCH_DTYPE2(table_dtype, TT,
            return b200::launch_pdl(b200::token_gate_rows_kernel<T, TT>, dim3(n_tokens), dim3(128), 0, stream, (const T*)a, ld_a,
                                    tokens, (const TT*)table, ld_table, n_rows_table, (T*)g, ld_g, n, width)));
    return 0;
}

