// Small per-element and per-row kernels that several parts share.
//   softcap_rows       x <- cap * tanh(x / cap), in place on 32-bit logits
//   gated_rmsnorm      out[t, h, :] = x[t, h, :] / sqrt(mean(x^2) + eps) * w * act(gate[t, h, :]), act sigmoid or SiLU
//                      per (token, head) row of 32-bit numbers: the output norm of a recurrent mixer; with `gate_first`
//                      the row is multiplied by act(gate) first and the norm runs over the gated row; with
//                      `weight_per_row` every row has weights of its own (w holds n_heads * d numbers), so that the rows
//                      may be any equal parts of the mixer's output, not its heads; a warp per row, or a CTA per row
//                      of 512 numbers and more
//   gate_rows          x[t, :n] <- x[t, :n] * sigmoid(gate[t, :n]) (or SiLU), in place: a gate on a mixer's output
//   scale_rows         x <- x * s, in place on 32-bit logits
//   differential_heads out[t, h, :] = post * o / sqrt(mean(o^2) + eps) * sigmoid(gate[t, h, :]) with o = a1 - lambda a2, where
//                      a1 and a2 are the results of two attention maps over the same values that lie as neighbouring
//                      heads (2h, 2h + 1) of `d_pad` numbers of which the first `d` count; a warp per (token, head)
#include "common.cuh"

namespace b200 {

__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

// a warp per (token, head) row
template <typename T>
__global__ void __launch_bounds__(128)
gated_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, const T* __restrict__ gate, int ld_gate,
                     T* __restrict__ out, int n_heads, int d, int n_rows, float eps, int gate_act, int gate_first,
                     int weight_per_row) {
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const int t = row / n_heads, h = row % n_heads;
    const float* xr = x + (size_t)row * d;
    const T* g = gate + (size_t)t * ld_gate + (size_t)h * d;
    const float* wr = w + (weight_per_row ? (size_t)h * d : 0);
    auto act = [&](int e) {
        const float z = to_f32<T>(g[e]);
        const float sig = 1.0f / (1.0f + expf(-z));
        return gate_act == 1 ? z * sig : sig;
    };
    float ss = 0.f;
    for (int e = lane; e < d; e += 32) {
        const float v = gate_first ? xr[e] * act(e) : xr[e];
        ss += v * v;
    }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    T* o = out + (size_t)row * d;
    for (int e = lane; e < d; e += 32)
        o[e] = from_f32<T>(gate_first ? (xr[e] * act(e)) * scale * wr[e] : xr[e] * scale * wr[e] * act(e));
}

// a CTA per row, for rows too long for one warp (a norm over a large part of the mixer's output); the gated values stay
// in registers between the two passes when the row has at most kWideKeep numbers per thread
constexpr int kWideThreads = 256, kWideKeep = 8;
template <typename T>
__global__ void __launch_bounds__(kWideThreads)
gated_rmsnorm_wide_kernel(const float* __restrict__ x, const float* __restrict__ w, const T* __restrict__ gate, int ld_gate,
                          T* __restrict__ out, int n_heads, int d, float eps, int gate_act, int gate_first, int weight_per_row) {
    __shared__ float scratch[33];
    const int row = blockIdx.x;
    const int t = row / n_heads, h = row % n_heads;
    const float* xr = x + (size_t)row * d;
    const T* g = gate + (size_t)t * ld_gate + (size_t)h * d;
    const float* wr = w + (weight_per_row ? (size_t)h * d : 0);
    auto act = [&](int e) {
        const float z = to_f32<T>(g[e]);
        const float sig = 1.0f / (1.0f + expf(-z));
        return gate_act == 1 ? z * sig : sig;
    };
    float keep[kWideKeep], ss = 0.f;
#pragma unroll
    for (int i = 0; i < kWideKeep; ++i) {
        const int e = threadIdx.x + i * kWideThreads;
        keep[i] = e < d ? (gate_first ? xr[e] * act(e) : xr[e]) : 0.f;
        ss += keep[i] * keep[i];
    }
    for (int e = threadIdx.x + kWideKeep * kWideThreads; e < d; e += kWideThreads) {
        const float v = gate_first ? xr[e] * act(e) : xr[e];
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    T* o = out + (size_t)row * d;
#pragma unroll
    for (int i = 0; i < kWideKeep; ++i) {
        const int e = threadIdx.x + i * kWideThreads;
        if (e < d) o[e] = from_f32<T>(gate_first ? keep[i] * scale * wr[e] : keep[i] * scale * wr[e] * act(e));
    }
    for (int e = threadIdx.x + kWideKeep * kWideThreads; e < d; e += kWideThreads)
        o[e] = from_f32<T>(gate_first ? (xr[e] * act(e)) * scale * wr[e] : xr[e] * scale * wr[e] * act(e));
}

template <typename T>
__global__ void gate_rows_kernel(T* __restrict__ x, int ld_x, const T* __restrict__ gate, int ld_gate, int n, int gate_act) {
    T* xr = x + (size_t)blockIdx.x * ld_x;
    const T* g = gate + (size_t)blockIdx.x * ld_gate;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < n; e += gridDim.y * blockDim.x) {
        const float z = to_f32<T>(g[e]);
        const float sig = 1.0f / (1.0f + expf(-z));
        xr[e] = from_f32<T>(to_f32<T>(xr[e]) * (gate_act == 1 ? z * sig : sig));
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
differential_heads_kernel(const T* __restrict__ maps, const T* __restrict__ gate, int ld_gate, T* __restrict__ out,
                          int n_heads, int d, int d_pad, int n_rows, float lambda, float post, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const int t = row / n_heads, h = row % n_heads;
    const T* a1 = maps + ((size_t)row * 2) * d_pad;
    const T* a2 = a1 + d_pad;
    float ss = 0.f;
    for (int e = lane; e < d; e += 32) {
        const float o = to_f32<T>(a1[e]) - lambda * to_f32<T>(a2[e]);
        ss += o * o;
    }
    ss = warp_sum(ss);
    const float scale = post / sqrtf(ss / (float)d + eps);
    const T* g = gate ? gate + (size_t)t * ld_gate + (size_t)h * d : nullptr;
    T* o_row = out + (size_t)row * d;
    for (int e = lane; e < d; e += 32) {
        float o = (to_f32<T>(a1[e]) - lambda * to_f32<T>(a2[e])) * scale;
        if (g) o *= 1.0f / (1.0f + expf(-to_f32<T>(g[e])));
        o_row[e] = from_f32<T>(o);
    }
}

__global__ void scale_kernel(float* __restrict__ x, size_t n, float s) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] *= s;
}

}  // namespace b200

extern "C" int b200_softcap_rows(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (!(cap > 0.f)) return b200::kErrBadArgument;
    const long long blocks = (n + 255) / 256;
    b200::softcap_kernel<<<(int)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, stream>>>(x, (size_t)n, cap);
    return b200::launch_status();
}

extern "C" int b200_gated_rmsnorm(const float* x, const float* w, const void* gate, int ld_gate, void* out, int dtype,
                                  int n_tokens, int n_heads, int d, float eps, int gate_act, int gate_first,
                                  int weight_per_row, cudaStream_t stream) {
    if (gate_act != 0 && gate_act != 1) return b200::kErrBadArgument;   // 0 sigmoid, 1 SiLU
    if (n_tokens <= 0 || n_heads <= 0) return 0;
    if (d < 1) return b200::kErrBadArgument;
    const long long rows = (long long)n_tokens * n_heads;
    if (rows > 0x7fffffffLL) return b200::kErrUnsupportedSize;
    B200_DISPATCH_DTYPE(dtype, T,
        if (d >= 512)      // (a warp would walk such a row in 16 or more rounds, twice)
            b200::gated_rmsnorm_wide_kernel<T><<<(int)rows, b200::kWideThreads, 0, stream>>>(x, w, (const T*)gate, ld_gate, (T*)out,
                                                                                           n_heads, d, eps, gate_act, gate_first,
                                                                                           weight_per_row);
        else
            b200::gated_rmsnorm_kernel<T><<<(int)((rows + 3) / 4), 128, 0, stream>>>(x, w, (const T*)gate, ld_gate, (T*)out,
                                                                                     n_heads, d, (int)rows, eps, gate_act, gate_first,
                                                                                     weight_per_row));
    return b200::launch_status();
}

extern "C" int b200_gate_rows(void* x, int ld_x, const void* gate, int ld_gate, int dtype, int n_tokens, int n, int gate_act,
                              cudaStream_t stream) {
    if (gate_act != 0 && gate_act != 1) return b200::kErrBadArgument;
    if (n_tokens <= 0 || n <= 0) return 0;
    const int ny = (n + 1023) / 1024;
    B200_DISPATCH_DTYPE(dtype, T,
        b200::gate_rows_kernel<T><<<dim3(n_tokens, ny > 64 ? 64 : ny), 256, 0, stream>>>((T*)x, ld_x, (const T*)gate, ld_gate, n,
                                                                                        gate_act));
    return b200::launch_status();
}

extern "C" int b200_scale_rows(float* x, long long n, float s, cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long blocks = (n + 255) / 256;
    b200::scale_kernel<<<(int)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, stream>>>(x, (size_t)n, s);
    return b200::launch_status();
}

// maps [T][2 n_heads][d_pad], gate [T][ld_gate] (or null), out [T][n_heads d], all of the run's type
extern "C" int b200_differential_heads(const void* maps, const void* gate, int ld_gate, void* out, int dtype, int n_tokens,
                                       int n_heads, int d, int d_pad, float lambda, float post, float eps,
                                       cudaStream_t stream) {
    if (n_tokens <= 0 || n_heads <= 0) return 0;
    if (d < 1 || d_pad < d || (gate && ld_gate < n_heads * d)) return b200::kErrBadArgument;
    const long long rows = (long long)n_tokens * n_heads;
    if (rows > 0x7fffffffLL) return b200::kErrUnsupportedSize;
    B200_DISPATCH_DTYPE(dtype, T,
        return b200::launch_pdl(b200::differential_heads_kernel<T>, dim3((int)((rows + 3) / 4)), dim3(128), 0, stream,
                                (const T*)maps, (const T*)gate, ld_gate, (T*)out, n_heads, d, d_pad, (int)rows, lambda, post, eps));
    return 0;
}
