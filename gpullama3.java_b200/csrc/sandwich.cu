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
// A CTA per token.  A part is cut into slices, one warp each, so that the CTA's warps are all busy whatever the number of
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

// `offset` (a row added to the stream behind the normed result) and `next_w` with `out` (the norm of the updated stream)
// are optional.
extern "C" int b200_sandwich_step(float* y, const float* wb, float mult, float* x, const float* offset, const float* next_w,
                                  void* out, int out_dtype, int n_tokens, int dim, int groups, float eps, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (!b200::groups_fit(dim, groups)) return b200::kErrUnsupportedSize;
    if ((next_w == nullptr) != (out == nullptr)) return b200::kErrBadArgument;
    const size_t smem = b200::scratch_bytes(groups);
    if (smem > 48 * 1024) return b200::kErrUnsupportedSize;
    B200_DISPATCH_DTYPE(out_dtype, TO,
        b200::sandwich_step_kernel<TO><<<n_tokens, b200::kSandwichWarps * 32, smem, stream>>>(y, wb, mult, x, offset, next_w,
                                                                                             (TO*)out, dim, groups, eps));
    return b200::launch_status();
}

extern "C" int b200_add_row(float* x, const float* row, int n_tokens, int dim, cudaStream_t stream) {
    if (n_tokens <= 0 || dim <= 0) return 0;
    if ((dim + 255) / 256 > 65535) return b200::kErrUnsupportedSize;
    b200::add_row_kernel<<<dim3(n_tokens, (dim + 255) / 256), 256, 0, stream>>>(x, row, dim);
    return b200::launch_status();
}
