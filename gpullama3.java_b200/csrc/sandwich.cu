// Kernels of a block that norms both what a sublayer reads and what it returns, over rows of the 32-bit residual stream.
//
//   group_rmsnorm    out[r] = w * x[rows[r]] / rms, the row cut into `groups` equal consecutive parts that are each
//                    divided by their own root mean square sqrt(mean(part^2) + eps)
//   sandwich_step    what happens between two sublayers, in one pass over a token's row:
//                        x <- x + mult * (wb * y / rms_groups(y)) (+ offset)      the sublayer's result y, normed, joins the stream
//                        y <- 0                                                 (the next sublayer's last product adds into it)
//                        out = wn * x / rms_groups(x)                           the next sublayer's input, if one follows
//   add_row          x[t] += row for every token (a vector that joins the stream between two runs of layers)
//
// A CTA per token.  Rows of whole 128-number pieces per part (up to 8192 numbers) stay in registers between their one
// fetch and their one store (sandwich_step_rows_kernel, which in decode steps also applies the next reader's convolution
// over time); the kernels below take every other size.  A part is cut into slices, one warp each, so that the CTA's warps are all busy whatever the number of
// groups; a part's sum of squares is the sum of its slices' sums in slice order (no atomics).  All arithmetic is 32-bit.
#include "common.cuh"

namespace b200 {

constexpr int kSandwichWarps = 8;

struct SlicePlan {
    int groups, per_group, slices, per_slice;   // per_group = dim / groups; a group in `slices` slices of per_slice (the last shorter)
};

__device__ __forceinline__ SlicePlan plan_slices(int dim, int groups) {
    SlicePlan p;
    p.groups = groups;
    p.per_group = dim / groups;
    int s = kSandwichWarps / groups;
    if (s < 1) s = 1;
    while (s > 1 && p.per_group / s < 128) --s;          // a slice shorter than 128 numbers is not worth a warp
    p.per_slice = ((p.per_group + s - 1) / s + 3) / 4 * 4;
    p.slices = (p.per_group + p.per_slice - 1) / p.per_slice;
    return p;
}

// 1 / rms of every group of `v`-values that `value(i)` yields for element i of the row; partial[] and scale[] are shared.
template <typename F>
__device__ __forceinline__ void group_scales(const SlicePlan& p, float eps, float* partial, float* scale, F value) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int units = p.groups * p.slices;
    for (int u = warp; u < units; u += kSandwichWarps) {
        const int g = u / p.slices, s = u % p.slices;
        const int lo = g * p.per_group + s * p.per_slice, hi = min(lo + p.per_slice, (g + 1) * p.per_group);
        float ss = 0.f;
        for (int i = lo + lane; i < hi; i += 32) {
            const float v = value(i);
            ss += v * v;
        }
        ss = warp_sum(ss);
        if (lane == 0) partial[u] = ss;
    }
    __syncthreads();
    for (int g = threadIdx.x; g < p.groups; g += blockDim.x) {
        float ss = 0.f;
        for (int s = 0; s < p.slices; ++s) ss += partial[g * p.slices + s];
        scale[g] = 1.0f / sqrtf(ss / (float)p.per_group + eps);
    }
    __syncthreads();
}

template <typename TO>
__global__ void __launch_bounds__(kSandwichWarps * 32)
group_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                     const int* __restrict__ rows, int dim, int groups, float eps) {
    extern __shared__ float shared[];
    const SlicePlan p = plan_slices(dim, groups);
    float* partial = shared;
    float* scale = shared + p.groups * p.slices;
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
    group_scales(p, eps, partial, scale, [&](int i) { return xr[i]; });
    TO* o = out + (size_t)r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = from_f32<TO>(w[i] * (scale[i / p.per_group] * xr[i]));
}

template <typename TO>
__global__ void __launch_bounds__(kSandwichWarps * 32)
sandwich_step_kernel(float* __restrict__ y, const float* __restrict__ wb, float mult, float* __restrict__ x,
                     const float* __restrict__ offset, const float* __restrict__ wn, TO* __restrict__ out, int dim,
                     int groups, float eps) {
    extern __shared__ float shared[];
    const SlicePlan p = plan_slices(dim, groups);
    float* partial = shared;
    float* scale = shared + p.groups * p.slices;
    const int t = blockIdx.x;
    float* yr = y + (size_t)t * dim;
    float* xr = x + (size_t)t * dim;
    group_scales(p, eps, partial, scale, [&](int i) { return yr[i]; });
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = xr[i] + mult * (wb[i] * (scale[i / p.per_group] * yr[i]));
        if (offset) v += offset[i];
        xr[i] = v;
        yr[i] = 0.f;
    }
    if (wn == nullptr) return;
    __syncthreads();   // every thread re-reads what others wrote; scale[] and partial[] are free again
    group_scales(p, eps, partial, scale, [&](int i) { return xr[i]; });
    TO* o = out + (size_t)t * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = from_f32<TO>(wn[i] * (scale[i / p.per_group] * xr[i]));
}

// The same step when the row is a whole number of 128-number pieces and so is every group (dim <= 1024 NV): a thread
// keeps NV pieces of four numbers of y and of x in registers, so each is fetched once and all fetches are in flight
// together; a warp's 128 numbers lie in one group, their sum of squares is one partial, and a group's sum is that of its
// partials in order.  With `conv_w` the normed rows are the input of a convolution over time whose older inputs all
// come from the slot's state (every sequence of the step brings one token): out = h + sum_j w[:, j] h_(t - taps + 1 + j),
// and the state moves on by this token (`conv_update`).
template <typename TO, int NV>
__global__ void __launch_bounds__(kSandwichWarps * 32)
sandwich_step_rows_kernel(float* __restrict__ y, const float* __restrict__ wb, float mult, float* __restrict__ x,
                          const float* __restrict__ offset, const float* __restrict__ wn, TO* __restrict__ out, int dim,
                          int groups, float eps, const float* __restrict__ conv_w, float* __restrict__ conv_state,
                          size_t slot_stride, const int* __restrict__ slots, int taps, int conv_update) {
    __shared__ float partial[NV * kSandwichWarps];
    __shared__ float scale[NV * kSandwichWarps];
    constexpr int threads = kSandwichWarps * 32;
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int per_group = dim / groups, pieces = per_group / 128, n_pieces = dim / 128;
    float4* yr = reinterpret_cast<float4*>(y + (size_t)t * dim);
    float4* xr = reinterpret_cast<float4*>(x + (size_t)t * dim);
    float4 yv[NV], xv[NV], wv[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = tid + j * threads;
        if (v * 4 < dim) {
            yv[j] = yr[v];
            xv[j] = xr[v];
            wv[j] = reinterpret_cast<const float4*>(wb)[v];
        } else {
            yv[j] = xv[j] = wv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    auto group_scales = [&](const float4 (&a)[NV]) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const float ss = warp_sum((a[j].x * a[j].x + a[j].y * a[j].y) + (a[j].z * a[j].z + a[j].w * a[j].w));
            if (lane == 0) partial[j * kSandwichWarps + warp] = ss;    // piece j * warps + warp of the row
        }
        __syncthreads();
        if (tid < groups) {
            float ss = 0.f;
            for (int p = 0; p < pieces; ++p) ss += partial[tid * pieces + p];
            scale[tid] = 1.0f / sqrtf(ss / (float)per_group + eps);
        }
        __syncthreads();
    };
    group_scales(yv);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = tid + j * threads;
        if (v * 4 >= dim) continue;
        const float s = scale[(j * kSandwichWarps + warp) / pieces];
        xv[j].x += mult * (wv[j].x * (s * yv[j].x));
        xv[j].y += mult * (wv[j].y * (s * yv[j].y));
        xv[j].z += mult * (wv[j].z * (s * yv[j].z));
        xv[j].w += mult * (wv[j].w * (s * yv[j].w));
        if (offset) {
            const float4 o = reinterpret_cast<const float4*>(offset)[v];
            xv[j].x += o.x; xv[j].y += o.y; xv[j].z += o.z; xv[j].w += o.w;
        }
        xr[v] = xv[j];
        yr[v] = zero;
    }
    if (wn == nullptr) return;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = tid + j * threads;
        if (v * 4 < dim) wv[j] = reinterpret_cast<const float4*>(wn)[v];
    }
    group_scales(xv);    // (the barrier inside also orders the reads of scale[] above before its rewriting)
    float* st = conv_w ? conv_state + (size_t)slots[t] * slot_stride : nullptr;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = tid + j * threads;
        if (v * 4 >= dim) continue;
        const float s = scale[(j * kSandwichWarps + warp) / pieces];
        float h[4] = {wv[j].x * (s * xv[j].x), wv[j].y * (s * xv[j].y), wv[j].z * (s * xv[j].z), wv[j].w * (s * xv[j].w)};
        if (conv_w) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int m = 0; m + 1 < taps; ++m) {
                const float4 old = *reinterpret_cast<const float4*>(st + (size_t)m * dim + 4 * v);
                const float o4[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] += conv_w[(size_t)(4 * v + e) * taps + m] * o4[e];
                if (conv_update && m > 0) *reinterpret_cast<float4*>(st + (size_t)(m - 1) * dim + 4 * v) = old;
            }
            if (conv_update && taps > 1) *reinterpret_cast<float4*>(st + (size_t)(taps - 2) * dim + 4 * v) = make_float4(h[0], h[1], h[2], h[3]);
#pragma unroll
            for (int e = 0; e < 4; ++e) h[e] = (acc[e] + conv_w[(size_t)(4 * v + e) * taps + taps - 1] * h[e]) + h[e];
        }
        TO* o = out + (size_t)t * dim + 4 * v;
        if constexpr (sizeof(TO) == 4) {
            *reinterpret_cast<float4*>(o) = make_float4(h[0], h[1], h[2], h[3]);
        } else {
            const __nv_bfloat162 a = __floats2bfloat162_rn(h[0], h[1]), b = __floats2bfloat162_rn(h[2], h[3]);
            *reinterpret_cast<uint2*>(o) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
        }
    }
}

__global__ void add_row_kernel(float* __restrict__ x, const float* __restrict__ row, int dim) {
    float* xr = x + (size_t)blockIdx.x * dim;
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i < dim) xr[i] += row[i];
}

static bool groups_fit(int dim, int groups) {
    if (groups < 1 || dim < groups || dim % groups) return false;
    int s = kSandwichWarps / groups;
    if (s < 1) s = 1;
    return (long long)groups * (s + 1) <= 12 * 1024;   // what the CTA keeps of them in shared memory
}

static size_t scratch_bytes(int groups) {
    int s = kSandwichWarps / groups;
    if (s < 1) s = 1;
    return sizeof(float) * ((size_t)groups * s + groups);
}

}  // namespace b200

extern "C" int b200_group_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int* rows, int n_rows,
                                  int dim, int groups, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!b200::groups_fit(dim, groups)) return b200::kErrUnsupportedSize;
    const size_t smem = b200::scratch_bytes(groups);
    if (smem > 48 * 1024) return b200::kErrUnsupportedSize;
    B200_DISPATCH_DTYPE(out_dtype, TO,
        b200::group_rmsnorm_kernel<TO><<<n_rows, b200::kSandwichWarps * 32, smem, stream>>>(x, w, (TO*)out, rows, dim, groups, eps));
    return b200::launch_status();
}

namespace b200 {

// Whether the kernel that keeps a token's row in registers takes these sizes: whole 128-number pieces per group, at most
// 8 pieces of four numbers per thread, every row and vector 16-byte aligned.
static bool rows_fit(int dim, int groups, const void* a, const void* b, const void* c, const void* d, const void* e, const void* f) {
    if (groups < 1 || dim % groups || (dim / groups) % 128 || dim > 8 * 1024) return false;
    return (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d | (uintptr_t)e | (uintptr_t)f) & 15) == 0;
}

template <typename TO>
static void launch_rows(float* y, const float* wb, float mult, float* x, const float* offset, const float* next_w, TO* out,
                        int n_tokens, int dim, int groups, float eps, const float* conv_w, float* conv_state,
                        size_t slot_stride, const int* slots, int taps, int conv_update, cudaStream_t stream) {
    const int nv = (dim + 1023) / 1024;
#define B200_ROWS(NV)                                                                                                      \
    sandwich_step_rows_kernel<TO, NV><<<n_tokens, kSandwichWarps * 32, 0, stream>>>(y, wb, mult, x, offset, next_w, out, dim,   \
                                                                                 groups, eps, conv_w, conv_state, slot_stride, \
                                                                                 slots, taps, conv_update)
    if (nv <= 1) B200_ROWS(1);
    else if (nv == 2) B200_ROWS(2);
    else if (nv <= 4) B200_ROWS(4);
    else B200_ROWS(8);
#undef B200_ROWS
}

}  // namespace b200

// `offset` (a row added to the stream behind the normed result) and `next_w` with `out` (the norm of the updated stream)
// are optional.
extern "C" int b200_sandwich_step(float* y, const float* wb, float mult, float* x, const float* offset, const float* next_w,
                                  void* out, int out_dtype, int n_tokens, int dim, int groups, float eps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!b200::groups_fit(dim, groups)) return b200::kErrUnsupportedSize;
    if ((next_w == nullptr) != (out == nullptr)) return b200::kErrBadArgument;
    if (b200::rows_fit(dim, groups, y, wb, x, offset, next_w, out)) {
        B200_DISPATCH_DTYPE(out_dtype, TO,
            b200::launch_rows<TO>(y, wb, mult, x, offset, next_w, (TO*)out, n_tokens, dim, groups, eps, nullptr, nullptr, 0, nullptr,
                                  0, 0, stream));
        return b200::launch_status();
    }
    const size_t smem = b200::scratch_bytes(groups);
    if (smem > 48 * 1024) return b200::kErrUnsupportedSize;
    B200_DISPATCH_DTYPE(out_dtype, TO,
        b200::sandwich_step_kernel<TO><<<n_tokens, b200::kSandwichWarps * 32, smem, stream>>>(y, wb, mult, x, offset, next_w,
                                                                                             (TO*)out, dim, groups, eps));
    return b200::launch_status();
}

// Whether b200_sandwich_step_conv takes these sizes (the pointers' alignment is checked by the call itself).
extern "C" int b200_sandwich_step_conv_fits(int dim, int groups) {
    return b200::rows_fit(dim, groups, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr) ? 1 : 0;
}

// The step with the convolution that the next reader puts in front of its first product, for steps in which every
// sequence brings one token: out = h + conv(h) of the normed updated stream h, the older inputs from conv_state
// [slot][taps - 1][dim] (oldest first), which moves on by this token when `conv_update` is set.  slots[t]: token t's slot.
extern "C" int b200_sandwich_step_conv(float* y, const float* wb, float mult, float* x, const float* offset, const float* next_w,
                                       void* out, int out_dtype, int n_tokens, int dim, int groups, float eps,
                                       const float* conv_w, float* conv_state, long long slot_stride, const int* slots, int taps,
                                       int conv_update, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!next_w || !out || !conv_w || !slots || taps < 1 || (taps > 1 && !conv_state)) return b200::kErrBadArgument;
    if (!b200::rows_fit(dim, groups, y, wb, x, offset, next_w, out) || slot_stride % 4 || ((uintptr_t)conv_state & 15))
        return b200::kErrUnsupportedSize;
    B200_DISPATCH_DTYPE(out_dtype, TO,
        b200::launch_rows<TO>(y, wb, mult, x, offset, next_w, (TO*)out, n_tokens, dim, groups, eps, conv_w, conv_state,
                              (size_t)slot_stride, slots, taps, conv_update, stream));
    return b200::launch_status();
}

extern "C" int b200_add_row(float* x, const float* row, int n_tokens, int dim, cudaStream_t stream) {
    if (n_tokens <= 0 || dim <= 0) return 0;
    if ((dim + 255) / 256 > 65535) return b200::kErrUnsupportedSize;
    b200::add_row_kernel<<<dim3(n_tokens, (dim + 255) / 256), 256, 0, stream>>>(x, row, dim);
    return b200::launch_status();
}
