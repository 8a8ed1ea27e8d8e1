// The gated delta rule with one decay per key channel (or one per head, which is the same rule with all channels of a
// head decaying alike), and the short causal convolution in front of it.
//
// Per sequence and head the mixer keeps a matrix S [d_k, d_v] of 32-bit numbers.  A token with unit-length
// query q and key k [d_k], value v [d_v], write strength beta and per-channel decay g [d_k] in (0, 1) does
//     S <- diag(g) S ;  u = beta (v - S^T k) ;  S <- S + k u^T ;  o = S^T q
// in this order (the read-out sees the token's own write).  Column j of S only ever meets column j of v, u and o, so
// the columns are independent chains:
// a thread holds RPT rows of one column in registers (four neighbouring rows per piece of 4 R rows: a lane reads them as
// one 16-byte word, and the R neighbouring lanes that share a column read neighbouring words of shared memory),
// d_k <= R * RPT, rows beyond d_k are zero and stay zero, and the two
// sums over the rows that a token needs are finished by log2(R) exchanges.
// What the chains read is made first, for all tokens at once, by delta_rule_prepare (unit norms of q and k from the
// convolution's output, the query scale, beta = sigmoid(.), g = exp(-exp(A_log) softplus(a + dt_bias)), all 32-bit);
// the scan takes tokens in chunks of kChunk through shared memory, the next chunk on its way (cp.async) while one
// is walked.  The same kernels serve a prompt, a portion of one and a single decoded token: a
// sequence's tokens are rows cu_seqlens[i] .. cu_seqlens[i + 1] of the step, its state sits in its cache slot.
//
// The convolution: channel c of token t gets sum_j w[c, j] x[t - (taps - 1) + j, c] followed by SiLU, where inputs
// before the step's first token come from the slot's state (the last taps - 1 inputs of the sequence, zero at its
// start); conv_state_update then stores the step's last taps - 1 inputs there (a step in which every sequence brings
// one token does both in one kernel, causal_conv_single).
//
// The same scan also runs the recurrences without the delta correction (linear_scan): S <- diag(g) S + k (beta v)^T,
// o = S^T q + skip v, which is gated linear attention (a decay per key channel, g = sigmoid(.)^(1/tau), beta = 1) and the
// state-space recurrence with a scalar decay per head (q = C, k = B, g = exp(-exp(A_log) dt), beta = dt = softplus(.),
// skip = D); linear_scan_prepare makes their rows.  causal_conv is the convolution in its general form: input and output
// types of their own, an optional bias, SiLU or no activation, and optionally the input added to the result.
#include "common.cuh"

namespace b200 {

constexpr int kScanThreads = 128;
constexpr int kChunk = 16;
constexpr int kMaxTaps = 16;

template <typename T, int VEC> struct ConvVec;
template <typename T> struct ConvVec<T, 1> {
    __device__ static void load(const T* p, float (&f)[1]) { f[0] = to_f32<T>(p[0]); }
    __device__ static void store(T* p, const float (&f)[1]) { p[0] = from_f32<T>(f[0]); }
};
template <> struct ConvVec<float, 4> {
    __device__ static void load(const float* p, float (&f)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    __device__ static void store(float* p, const float (&f)[4]) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct ConvVec<__nv_bfloat16, 8> {
    __device__ static void load(const __nv_bfloat16* p, float (&f)[8]) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ static void store(__nv_bfloat16* p, const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// A thread takes VEC neighbouring channels of one token (16 bytes per access when the sizes and pointers allow).
template <typename T, int VEC>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, int ld_x, const float* __restrict__ w,
                                        const float* __restrict__ state, size_t slot_stride, const int* __restrict__ slots,
                                        const int* __restrict__ seq_ids, const int* __restrict__ cu_seqlens,
                                        T* __restrict__ out, int ld_out, int channels, int taps) {
    const int t = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (c >= channels) return;
    const int seq = seq_ids[t];
    const int local = t - cu_seqlens[seq];
    const float* st = state + (size_t)slots[seq] * slot_stride;   // [taps - 1][channels], oldest first
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;          // how many tokens before t
        float v[VEC];
        if (local - back >= 0) {
            ConvVec<T, VEC>::load(x + (size_t)(t - back) * ld_x + c, v);
        } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = st[(size_t)(taps - 1 + local - back) * channels + c + e];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] += w[(size_t)(c + e) * taps + j] * v[e];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = acc[e] / (1.0f + expf(-acc[e]));
    ConvVec<T, VEC>::store(out + (size_t)t * ld_out + c, acc);
}

template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ x, int ld_x, float* __restrict__ state, size_t slot_stride,
                                         const int* __restrict__ slots, const int* __restrict__ cu_seqlens, int channels,
                                         int taps) {
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int first = cu_seqlens[seq], n = cu_seqlens[seq + 1] - first;
    float* st = state + (size_t)slots[seq] * slot_stride;
    float fresh[kMaxTaps];
#pragma unroll
    for (int m = 0; m < kMaxTaps; ++m) {
        if (m >= taps - 1) break;
        const int idx = n - (taps - 1) + m;     // among the step's tokens; negative: still an older input
        fresh[m] = idx >= 0 ? to_f32<T>(x[(size_t)(first + idx) * ld_x + c]) : st[(size_t)(m + n) * channels + c];
    }
#pragma unroll
    for (int m = 0; m < kMaxTaps; ++m) {
        if (m >= taps - 1) break;
        st[(size_t)m * channels + c] = fresh[m];
    }
}

// The convolution in its general form, VEC neighbouring channels of one token per thread.
template <typename TI, typename TO, int VEC>
__global__ void causal_conv_kernel(const TI* __restrict__ x, int ld_x, const float* __restrict__ w, const float* __restrict__ bias,
                                   const float* __restrict__ state, size_t slot_stride, const int* __restrict__ slots,
                                   const int* __restrict__ seq_ids, const int* __restrict__ cu_seqlens, TO* __restrict__ out,
                                   int ld_out, int channels, int taps, int activation, int add_input) {
    const int t = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (c >= channels) return;
    const int seq = seq_ids[t];
    const int local = t - cu_seqlens[seq];
    const float* st = state + (size_t)slots[seq] * slot_stride;   // [taps - 1][channels], oldest first
    float acc[VEC], own[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = bias ? bias[c + e] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;          // how many tokens before t
        float v[VEC];
        if (local - back >= 0) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = to_f32<TI>(x[(size_t)(t - back) * ld_x + c + e]);
        } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = st[(size_t)(taps - 1 + local - back) * channels + c + e];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            acc[e] += w[(size_t)(c + e) * taps + j] * v[e];
            if (back == 0) own[e] = v[e];
        }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        if (activation == 1) acc[e] = acc[e] / (1.0f + expf(-acc[e]));
        if (add_input) acc[e] += own[e];
        out[(size_t)t * ld_out + c + e] = from_f32<TO>(acc[e]);
    }
}

// The same convolution for steps of many tokens: a thread takes 4 neighbouring channels of kConvRun consecutive tokens of
// the step.  It asks for all the rows it needs at once (the run's own and the MAXT - 1 before it: 16 or 8 bytes per
// row), so every input row is fetched from memory once per run instead of once per tap, and then walks the run; a token
// among the first taps - 1 of its sequence takes its older inputs from the slot's state.  Sums run from the oldest tap
// to the newest, as in the kernel above.
constexpr int kConvRun = 8;

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&f)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&f)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

template <typename TI, typename TO, int MAXT>
__global__ void __launch_bounds__(128)
causal_conv_run_kernel(const TI* __restrict__ x, int ld_x, const float* __restrict__ w, const float* __restrict__ bias,
                       const float* __restrict__ state, size_t slot_stride, const int* __restrict__ slots,
                       const int* __restrict__ seq_ids, const int* __restrict__ cu_seqlens, TO* __restrict__ out, int ld_out,
                       int channels, int taps, int activation, int add_input, int n_tokens) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= channels) return;
    const int t0 = blockIdx.y * kConvRun;
    // rows t0 - (MAXT - 1) .. t0 + kConvRun - 1 of the step (those of them that exist and that some tap reads)
    float rows[kConvRun + MAXT - 1][4];
    int seq[kConvRun], first[kConvRun];
#pragma unroll
    for (int k = 0; k < kConvRun + MAXT - 1; ++k) {
        const int t = t0 - (MAXT - 1) + k;
        if (t >= 0 && t < n_tokens && (MAXT - 1 - k) <= taps - 1) {
            load4<TI>(x + (size_t)t * ld_x + c, rows[k]);
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) rows[k][e] = 0.f;
        }
    }
#pragma unroll
    for (int i = 0; i < kConvRun; ++i) seq[i] = t0 + i < n_tokens ? seq_ids[t0 + i] : 0;
#pragma unroll
    for (int i = 0; i < kConvRun; ++i) first[i] = cu_seqlens[seq[i]];
    // tap j of the layer stands at wt[MAXT - taps + j]: the newest tap last, zeros in front of the oldest
    float wt[MAXT][4], b[4];
#pragma unroll
    for (int m = 0; m < MAXT; ++m) {
        const int j = m - (MAXT - taps);
#pragma unroll
        for (int e = 0; e < 4; ++e) wt[m][e] = j >= 0 ? w[(size_t)(c + e) * taps + j] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) b[e] = bias ? bias[c + e] : 0.f;
#pragma unroll
    for (int i = 0; i < kConvRun; ++i) {
        const int t = t0 + i;
        if (t >= n_tokens) break;
        const int local = t - first[i];
        float acc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = b[e];
#pragma unroll
        for (int m = 0; m < MAXT; ++m) {
            const int back = MAXT - 1 - m;
            if (back > taps - 1) continue;
            if (local - back >= 0) {
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] += wt[m][e] * rows[i + m][e];
            } else {
                const float* st = state + (size_t)slots[seq[i]] * slot_stride + (size_t)(taps - 1 + local - back) * channels + c;
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[e] += wt[m][e] * st[e];
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (activation == 1) acc[e] = acc[e] / (1.0f + expf(-acc[e]));
            if (add_input) acc[e] += rows[i + MAXT - 1][e];
        }
        store4<TO>(out + (size_t)t * ld_out + c, acc);
    }
}

// The same convolution for steps in which every sequence brings exactly one token (decoding): the token's older inputs
// all come from its slot's state, and the thread that read them also moves the state on by one token, so the step needs
// no second kernel.  VEC neighbouring channels per thread; sums run from the oldest tap to the newest as above.
template <typename TI, typename TO, int VEC>
__global__ void __launch_bounds__(128)
causal_conv_single_kernel(const TI* __restrict__ x, int ld_x, const float* __restrict__ w, const float* __restrict__ bias,
                          float* __restrict__ state, size_t slot_stride, const int* __restrict__ slots,
                          const int* __restrict__ seq_ids, TO* __restrict__ out, int ld_out, int channels, int taps,
                          int activation, int add_input, int update_state) {
    const int t = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (c >= channels) return;
    float* st = state + (size_t)slots[seq_ids[t]] * slot_stride + c;   // [taps - 1][channels], oldest first
    float own[VEC], acc[VEC], newer[VEC];
    if constexpr (VEC == 4) {
        load4<TI>(x + (size_t)t * ld_x + c, own);
    } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) own[e] = to_f32<TI>(x[(size_t)t * ld_x + c + e]);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = bias ? bias[c + e] : 0.f;
    for (int m = 0; m + 1 < taps; ++m) {
        if constexpr (VEC == 4) {
            load4<float>(st + (size_t)m * channels, newer);
        } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) newer[e] = st[(size_t)m * channels + e];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] += w[(size_t)(c + e) * taps + m] * newer[e];
        if (update_state && m > 0) {
            if constexpr (VEC == 4) {
                store4<float>(st + (size_t)(m - 1) * channels, newer);
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) st[(size_t)(m - 1) * channels + e] = newer[e];
            }
        }
    }
    if (update_state && taps > 1) {
        if constexpr (VEC == 4) {
            store4<float>(st + (size_t)(taps - 2) * channels, own);
        } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) st[(size_t)(taps - 2) * channels + e] = own[e];
        }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        acc[e] += w[(size_t)(c + e) * taps + taps - 1] * own[e];
        if (activation == 1) acc[e] = acc[e] / (1.0f + expf(-acc[e]));
        if (add_input) acc[e] += own[e];
    }
    if constexpr (VEC == 4) {
        store4<TO>(out + (size_t)t * ld_out + c, acc);
    } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) out[(size_t)t * ld_out + c + e] = from_f32<TO>(acc[e]);
    }
}

// What the scan needs of every token, made by a kernel of its own over all tokens at once (a warp per token and head):
// one row of 32-bit numbers per (head, token), [q | k | g (each d_pad wide, zeros behind the d_k) | v (d_v) | beta | k . q | skip (unused here) | fill
// to a multiple of 4], q and k of unit length (q also scaled), g = exp(-exp(A_log) softplus(a + dt_bias)),
// beta = sigmoid(.).  Rows of one head lie token after token, so a chunk of a sequence's tokens is one contiguous piece
// that the scan brings into shared memory as it is.
struct PrepareArgs {
    const void* qkv;        // [T, ld_qkv]: convolved q [kv_heads d_k], k [kv_heads d_k], v [heads d_v]
    int ld_qkv;
    const void* beta;       // [T, ld_beta], column h: before the sigmoid
    int ld_beta;
    const void* decay;      // [T, ld_decay], column h d_k + i: before dt_bias and softplus
    int ld_decay;
    const float* dt_bias;   // [heads d_k]
    const float* a_log;     // [heads]
    float* rows;            // [heads, T, row]
    int n_tokens, heads, kv_heads, d_k, d_v, d_pad, row;
    float q_scale, unit_eps;
    int decay_per_head;     // 1: one decay per head (decay column h, dt_bias[h]) in place of one per key channel
};

__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void __launch_bounds__(128)
delta_rule_prepare_kernel(PrepareArgs a) {
    const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (unit >= (long long)a.n_tokens * a.heads) return;
    const size_t t = (size_t)(unit / a.heads);
    const int h = (int)(unit % a.heads), kvh = h / (a.heads / a.kv_heads);
    const T* qr = (const T*)a.qkv + t * a.ld_qkv + (size_t)kvh * a.d_k;
    const T* kr = qr + (size_t)a.kv_heads * a.d_k;
    const T* vr = (const T*)a.qkv + t * a.ld_qkv + 2 * (size_t)a.kv_heads * a.d_k + (size_t)h * a.d_v;
    const T* dr = (const T*)a.decay + t * a.ld_decay + (a.decay_per_head ? (size_t)h : (size_t)h * a.d_k);
    float* out = a.rows + ((size_t)h * a.n_tokens + t) * a.row;
    float sq = 0.f, sk = 0.f, qk = 0.f;
    for (int i = lane; i < a.d_k; i += 32) {
        const float qv = to_f32<T>(qr[i]), kv = to_f32<T>(kr[i]);
        sq += qv * qv;
        sk += kv * kv;
        qk += qv * kv;
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    qk = warp_sum(qk);
    const float fq = a.q_scale / sqrtf(sq + a.unit_eps), fk = 1.0f / sqrtf(sk + a.unit_eps);
    const float neg_rate = -expf(a.a_log[h]);
    const float g_head = a.decay_per_head ? expf(neg_rate * softplus(to_f32<T>(dr[0]) + a.dt_bias[h])) : 0.f;
    for (int i = lane; i < a.d_pad; i += 32) {
        const bool in = i < a.d_k;
        out[i] = in ? to_f32<T>(qr[i]) * fq : 0.f;
        out[a.d_pad + i] = in ? to_f32<T>(kr[i]) * fk : 0.f;
        out[2 * a.d_pad + i] = !in ? 0.f : a.decay_per_head ? g_head
                                         : expf(neg_rate * softplus(to_f32<T>(dr[i]) + a.dt_bias[(size_t)h * a.d_k + i]));
    }
    for (int j = lane; j < a.d_v; j += 32) out[3 * a.d_pad + j] = to_f32<T>(vr[j]);
    if (lane == 0) {
        out[3 * a.d_pad + a.d_v] = 1.0f / (1.0f + expf(-to_f32<T>(((const T*)a.beta)[t * a.ld_beta + h])));
        out[3 * a.d_pad + a.d_v + 1] = qk * fq * fk;   // k . q of the unit vectors (q scaled)
    }
}

// The rows of the recurrences without the delta correction, in the layout the scan reads: [q | k | g | v | beta | k . q |
// skip].  q rows are scaled by q_scale; the decay is exp(-exp(A_log[h]) softplus(z + bias)) (kind 0) or
// sigmoid(z + bias)^power (kind 1: exp(-softplus(-(z + bias)) power)), per key channel or per head; beta is 1, or the step
// size softplus(z + bias) of a per-head decay of kind 0 (`step_scales_value`); skip is skip[h] or 0.
struct LinearPrepareArgs {
    const void* q;          // [T, ld_q], head kvh of kv_heads at column kvh d_k
    int ld_q;
    const void* k;          // [T, ld_k], likewise
    int ld_k;
    const void* v;          // [T, ld_v], head h at column h d_v
    int ld_v;
    const void* decay;      // [T, ld_decay]: column h d_k + i, or h when there is one decay per head
    int ld_decay;
    const float* decay_bias;   // laid out like a row of `decay`, or null
    const float* a_log;     // [heads], kind 0
    const float* skip;      // [heads] or null
    float* rows;            // [heads, T, row]
    int n_tokens, heads, kv_heads, d_k, d_v, d_pad, row;
    float q_scale, power;
    int decay_kind, decay_per_head, step_scales_value;
};

template <typename T>
__global__ void __launch_bounds__(128)
linear_scan_prepare_kernel(LinearPrepareArgs a) {
    const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (unit >= (long long)a.n_tokens * a.heads) return;
    const size_t t = (size_t)(unit / a.heads);
    const int h = (int)(unit % a.heads), kvh = h / (a.heads / a.kv_heads);
    const T* qr = (const T*)a.q + t * a.ld_q + (size_t)kvh * a.d_k;
    const T* kr = (const T*)a.k + t * a.ld_k + (size_t)kvh * a.d_k;
    const T* vr = (const T*)a.v + t * a.ld_v + (size_t)h * a.d_v;
    const size_t d_at = a.decay_per_head ? (size_t)h : (size_t)h * a.d_k;
    const T* dr = (const T*)a.decay + t * a.ld_decay + d_at;
    const float* br = a.decay_bias ? a.decay_bias + d_at : nullptr;
    float* out = a.rows + ((size_t)h * a.n_tokens + t) * a.row;
    const float neg_rate = a.decay_kind == 0 ? -expf(a.a_log[h]) : 0.f;
    auto decay_of = [&](float z, float& step) {
        if (a.decay_kind == 0) {
            step = softplus(z);
            return expf(neg_rate * step);
        }
        step = 1.f;
        return expf(-softplus(-z) * a.power);
    };
    float step_head = 1.f;
    const float g_head = a.decay_per_head ? decay_of(to_f32<T>(dr[0]) + (br ? br[0] : 0.f), step_head) : 0.f;
    float qk = 0.f;
    for (int i = lane; i < a.d_pad; i += 32) {
        const bool in = i < a.d_k;
        const float qv = in ? to_f32<T>(qr[i]) * a.q_scale : 0.f, kv = in ? to_f32<T>(kr[i]) : 0.f;
        qk += qv * kv;
        out[i] = qv;
        out[a.d_pad + i] = kv;
        float unused;
        out[2 * a.d_pad + i] = !in ? 0.f : a.decay_per_head ? g_head : decay_of(to_f32<T>(dr[i]) + (br ? br[i] : 0.f), unused);
    }
    qk = warp_sum(qk);
    for (int j = lane; j < a.d_v; j += 32) out[3 * a.d_pad + j] = to_f32<T>(vr[j]);
    if (lane == 0) {
        out[3 * a.d_pad + a.d_v] = (a.step_scales_value && a.decay_per_head) ? step_head : 1.f;
        out[3 * a.d_pad + a.d_v + 1] = qk;
        out[3 * a.d_pad + a.d_v + 2] = a.skip ? a.skip[h] : 0.f;
    }
}

struct ScanArgs {
    const float* rows;      // [heads, T, row] as delta_rule_prepare leaves them
    float* state;           // per slot: [heads][d_k][d_v]
    size_t slot_stride;
    const int* slots;
    const int* cu_seqlens;
    float* out;             // [T, heads d_v] 32-bit
    int n_tokens, heads, d_k, d_v, row;
};

__device__ __forceinline__ void copy_async_16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Shared memory holds two chunks of kChunk prepared rows.  While one chunk is walked the next one is on its way.
// R lanes share a column and hold RPT rows each; a CTA of 128 threads owns 128 / R columns.
// LINEAR: without the delta correction, u = beta v and the read-out gains skip v.
template <int RPT, int R, bool LINEAR>
__global__ void __launch_bounds__(kScanThreads)
delta_rule_scan_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float smem[];
    constexpr int dpad = R * RPT, cols = kScanThreads / R;
    const int per_chunk = kChunk * a.row;

    const int h = blockIdx.y, seq = blockIdx.z, col0 = blockIdx.x * cols;
    const int tid = threadIdx.x;
    const int col = col0 + tid / R, r = tid % R;
    const bool live = col < a.d_v;
    const int v_at = 3 * dpad + min(col, a.d_v - 1), b_at = 3 * dpad + a.d_v;
    const int first = a.cu_seqlens[seq], n = a.cu_seqlens[seq + 1] - first;
    float* S_g = a.state + (size_t)a.slots[seq] * a.slot_stride + (size_t)h * a.d_k * a.d_v;
    const float* rows = a.rows + ((size_t)h * a.n_tokens + first) * a.row;

    auto fetch = [&](int base, float* buf) {
        const int floats = min(kChunk, n - base) * a.row;       // a multiple of 4; both ends 16-byte aligned
        const float* src = rows + (size_t)base * a.row;
        for (int i = tid * 4; i < floats; i += kScanThreads * 4) copy_async_16(buf + i, src + i);
        copy_async_commit();
    };

    // register i of lane r holds row (i / 4) * 4 R + 4 r + i % 4: four neighbouring rows per lane and piece, so a lane
    // reads them as one 16-byte word and the R lanes of a column read neighbouring words
    float S[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int rw = (i >> 2) * (4 * R) + 4 * r + (i & 3);
        S[i] = (live && rw < a.d_k) ? S_g[(size_t)rw * a.d_v + col] : 0.f;
    }

    fetch(0, smem);
    int which = 0;
    for (int base = 0; base < n; base += kChunk) {
        const int m = min(kChunk, n - base);
        const float* buf = smem + which * per_chunk;
        if (base + kChunk < n) {
            fetch(base + kChunk, smem + (which ^ 1) * per_chunk);
            copy_async_wait<1>();
        } else {
            copy_async_wait<0>();
        }
        __syncthreads();
        float* out = a.out + ((size_t)first + base) * a.heads * a.d_v + (size_t)h * a.d_v + col;
        // (without the correction a token's write does not wait for a sum over the rows: eight tokens' loads go out together)
#pragma unroll(LINEAR ? 8 : 2)
        for (int tt = 0; tt < m; ++tt) {
            const float4* qp = reinterpret_cast<const float4*>(buf + tt * a.row) + r;
            const float4* kp = qp + dpad / 4;
            const float4* gp = kp + dpad / 4;
            const float v = buf[tt * a.row + v_at], beta = buf[tt * a.row + b_at], kq = buf[tt * a.row + b_at + 1];
            // with S' = diag(g) S:  o = (S' + k u^T)^T q = S'^T q + u (k . q), so both sums over the rows are taken from
            // S' in one pass and one round of exchanges, and k . q comes prepared with the token
            float d[4] = {0.f, 0.f, 0.f, 0.f}, e[4] = {0.f, 0.f, 0.f, 0.f}, kk[RPT];
#pragma unroll
            for (int c = 0; c < RPT / 4; ++c) {
                const float4 g4 = gp[c * R], k4 = kp[c * R], q4 = qp[c * R];
                const float gv[4] = {g4.x, g4.y, g4.z, g4.w}, kv[4] = {k4.x, k4.y, k4.z, k4.w}, qv[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    S[4 * c + j] *= gv[j];
                    if constexpr (!LINEAR) d[j] += S[4 * c + j] * kv[j];
                    e[j] += S[4 * c + j] * qv[j];
                    kk[4 * c + j] = kv[j];
                }
            }
            float dot = (d[0] + d[1]) + (d[2] + d[3]), read = (e[0] + e[1]) + (e[2] + e[3]);
#pragma unroll
            for (int o = R >> 1; o > 0; o >>= 1) {
                if constexpr (!LINEAR) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                read += __shfl_xor_sync(0xffffffffu, read, o);
            }
            const float u = LINEAR ? beta * v : beta * (v - dot);
            if (live && r == 0)
                out[(size_t)tt * a.heads * a.d_v] = LINEAR ? read + u * kq + buf[tt * a.row + b_at + 2] * v : read + u * kq;
#pragma unroll
            for (int i = 0; i < RPT; ++i) S[i] += kk[i] * u;
        }
        __syncthreads();   // the chunk has been walked: its buffer may be filled again
        which ^= 1;
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int rw = (i >> 2) * (4 * R) + 4 * r + (i & 3);
        if (live && rw < a.d_k) S_g[(size_t)rw * a.d_v + col] = S[i];
    }
}

template <int RPT, int R, bool LINEAR>
static int launch_scan(const ScanArgs& a, int n_seqs, cudaStream_t stream) {
    constexpr int cols = kScanThreads / R;
    const size_t smem = sizeof(float) * 2 * (size_t)kChunk * a.row;
    auto kernel = delta_rule_scan_kernel<RPT, R, LINEAR>;
    if (smem > 48 * 1024) {
        const int e = (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != 0) return e;
    }
    dim3 grid((a.d_v + cols - 1) / cols, a.heads, n_seqs);
    kernel<<<grid, kScanThreads, smem, stream>>>(a);
    return launch_status();
}

template <int RPT, bool LINEAR>
static int launch_scan_lanes(const ScanArgs& a, int lanes, int n_seqs, cudaStream_t stream) {
    switch (lanes) {
        case 1: return launch_scan<RPT, 1, LINEAR>(a, n_seqs, stream);
        case 2: return launch_scan<RPT, 2, LINEAR>(a, n_seqs, stream);
        case 4: return launch_scan<RPT, 4, LINEAR>(a, n_seqs, stream);
        case 8: return launch_scan<RPT, 8, LINEAR>(a, n_seqs, stream);
        case 16: return launch_scan<RPT, 16, LINEAR>(a, n_seqs, stream);
    }
    return kErrUnsupportedSize;
}

template <bool LINEAR>
static int launch_scan_rows(const ScanArgs& a, int rpt, int lanes, int n_seqs, cudaStream_t stream) {
    switch (rpt) {
        case 8: return launch_scan_lanes<8, LINEAR>(a, lanes, n_seqs, stream);
        case 12: return launch_scan_lanes<12, LINEAR>(a, lanes, n_seqs, stream);
        case 16: return launch_scan_lanes<16, LINEAR>(a, lanes, n_seqs, stream);
        case 24: return launch_scan_lanes<24, LINEAR>(a, lanes, n_seqs, stream);
        case 32: return launch_scan_lanes<32, LINEAR>(a, lanes, n_seqs, stream);
    }
    return kErrUnsupportedSize;
}

}  // namespace b200

extern "C" int b200_causal_conv_silu(const void* x, int ld_x, const float* w, float* state, long long slot_stride,
                                     const int* slots, const int* seq_ids, const int* cu_seqlens, void* out, int ld_out,
                                     int dtype, int n_tokens, int n_seqs, int channels, int taps, int update_state,
                                     cudaStream_t stream) {
    if (n_tokens <= 0 || channels <= 0) return 0;
    if (taps < 1 || taps > b200::kMaxTaps) return b200::kErrUnsupportedSize;
    if (n_tokens > 65535 || n_seqs > 65535) return b200::kErrUnsupportedSize;
    dim3 grid((channels + 127) / 128, n_tokens), grid_u((channels + 127) / 128, n_seqs);
    const int vec = dtype == b200::kF32 ? 4 : 8;
    const bool wide = channels % vec == 0 && ld_x % vec == 0 && ld_out % vec == 0 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0;
    const dim3 grid_v((channels / vec + 127) / 128, n_tokens);
    // steps of many tokens: runs of tokens per thread (the general kernel with SiLU, no bias, nothing added)
    const bool runs = wide && n_tokens >= 8 * b200::kConvRun && taps <= 8;
    const dim3 grid_r((channels / 4 + 127) / 128, (n_tokens + b200::kConvRun - 1) / b200::kConvRun);
    // every sequence brings one token: one kernel reads the slot's state and moves it on
    if (n_tokens == n_seqs) {
        const size_t size = dtype == b200::kF32 ? 4 : 2;
        const bool wide4 = channels % 4 == 0 && ld_x % 4 == 0 && ld_out % 4 == 0 && slot_stride % 4 == 0 &&
                           (uintptr_t)x % (4 * size) == 0 && (uintptr_t)out % (4 * size) == 0 && (uintptr_t)state % 16 == 0;
        const dim3 grid_s(((wide4 ? channels / 4 : channels) + 127) / 128, n_tokens);
        B200_DISPATCH_DTYPE(dtype, T,
            if (wide4)
                b200::causal_conv_single_kernel<T, T, 4><<<grid_s, 128, 0, stream>>>((const T*)x, ld_x, w, nullptr, state, (size_t)slot_stride,
                                                                                   slots, seq_ids, (T*)out, ld_out, channels, taps, 1, 0,
                                                                                   update_state);
            else
                b200::causal_conv_single_kernel<T, T, 1><<<grid_s, 128, 0, stream>>>((const T*)x, ld_x, w, nullptr, state, (size_t)slot_stride,
                                                                                   slots, seq_ids, (T*)out, ld_out, channels, taps, 1, 0,
                                                                                   update_state));
        return b200::launch_status();
    }
    if (runs) {
        B200_DISPATCH_DTYPE(dtype, T,
            if (taps <= 4)
                b200::causal_conv_run_kernel<T, T, 4><<<grid_r, 128, 0, stream>>>((const T*)x, ld_x, w, nullptr, state, (size_t)slot_stride,
                                                                                slots, seq_ids, cu_seqlens, (T*)out, ld_out, channels,
                                                                                taps, 1, 0, n_tokens);
            else
                b200::causal_conv_run_kernel<T, T, 8><<<grid_r, 128, 0, stream>>>((const T*)x, ld_x, w, nullptr, state, (size_t)slot_stride,
                                                                                slots, seq_ids, cu_seqlens, (T*)out, ld_out, channels,
                                                                                taps, 1, 0, n_tokens));
    } else if (dtype == b200::kF32 && wide)
        b200::causal_conv_silu_kernel<float, 4><<<grid_v, 128, 0, stream>>>((const float*)x, ld_x, w, state, (size_t)slot_stride, slots,
                                                                            seq_ids, cu_seqlens, (float*)out, ld_out, channels, taps);
    else if (dtype == b200::kBF16 && wide)
        b200::causal_conv_silu_kernel<__nv_bfloat16, 8><<<grid_v, 128, 0, stream>>>((const __nv_bfloat16*)x, ld_x, w, state, (size_t)slot_stride, slots,
                                                                                    seq_ids, cu_seqlens, (__nv_bfloat16*)out, ld_out, channels, taps);
    B200_DISPATCH_DTYPE(dtype, T,
        if (!wide && !runs)
            b200::causal_conv_silu_kernel<T, 1><<<grid, 128, 0, stream>>>((const T*)x, ld_x, w, state, (size_t)slot_stride, slots,
                                                                          seq_ids, cu_seqlens, (T*)out, ld_out, channels, taps);
        if (update_state && taps > 1)
            b200::conv_state_update_kernel<T><<<grid_u, 128, 0, stream>>>((const T*)x, ld_x, state, (size_t)slot_stride, slots,
                                                                          cu_seqlens, channels, taps));
    return b200::launch_status();
}

// The general convolution: x [T, >= channels] of `in_dtype`, out of `out_dtype`; `bias` [channels] or null; `activation`
// 0 none, 1 SiLU; `add_input`: out = x + conv(x) (after the activation).  State as for b200_causal_conv_silu.
extern "C" int b200_causal_conv(const void* x, int ld_x, int in_dtype, const float* w, const float* bias, float* state,
                                long long slot_stride, const int* slots, const int* seq_ids, const int* cu_seqlens, void* out,
                                int ld_out, int out_dtype, int n_tokens, int n_seqs, int channels, int taps, int activation,
                                int add_input, int update_state, cudaStream_t stream) {
    if (n_tokens <= 0 || channels <= 0) return 0;
    if (taps < 1 || taps > b200::kMaxTaps || (activation != 0 && activation != 1)) return b200::kErrUnsupportedSize;
    if (n_tokens > 65535 || n_seqs > 65535) return b200::kErrUnsupportedSize;
    const bool wide = channels % 4 == 0;
    const dim3 grid(((wide ? channels / 4 : channels) + 127) / 128, n_tokens), grid_u((channels + 127) / 128, n_seqs);
    // steps of many tokens, when every access of four channels is aligned: runs of tokens per thread
    const size_t in_size = in_dtype == b200::kF32 ? 4 : 2, out_size = out_dtype == b200::kF32 ? 4 : 2;
    const bool runs = wide && n_tokens >= 8 * b200::kConvRun && taps <= 8 && ld_x % 4 == 0 && ld_out % 4 == 0 &&
                      (uintptr_t)x % (4 * in_size) == 0 && (uintptr_t)out % (4 * out_size) == 0;
    const dim3 grid_r((channels / 4 + 127) / 128, (n_tokens + b200::kConvRun - 1) / b200::kConvRun);
    // every sequence brings one token: one kernel reads the slot's state and moves it on
    if (n_tokens == n_seqs) {
        const bool wide4 = wide && ld_x % 4 == 0 && ld_out % 4 == 0 && slot_stride % 4 == 0 && (uintptr_t)x % (4 * in_size) == 0 &&
                           (uintptr_t)out % (4 * out_size) == 0 && (uintptr_t)state % 16 == 0;
        const dim3 grid_s(((wide4 ? channels / 4 : channels) + 127) / 128, n_tokens);
        B200_DISPATCH_DTYPE(in_dtype, TI,
            B200_DISPATCH_DTYPE2(out_dtype, TO,
                if (wide4)
                    b200::causal_conv_single_kernel<TI, TO, 4><<<grid_s, 128, 0, stream>>>((const TI*)x, ld_x, w, bias, state, (size_t)slot_stride,
                                                                                         slots, seq_ids, (TO*)out, ld_out, channels, taps,
                                                                                         activation, add_input, update_state);
                else
                    b200::causal_conv_single_kernel<TI, TO, 1><<<grid_s, 128, 0, stream>>>((const TI*)x, ld_x, w, bias, state, (size_t)slot_stride,
                                                                                         slots, seq_ids, (TO*)out, ld_out, channels, taps,
                                                                                         activation, add_input, update_state)));
        return b200::launch_status();
    }
    B200_DISPATCH_DTYPE(in_dtype, TI,
        B200_DISPATCH_DTYPE2(out_dtype, TO,
            if (runs && taps <= 4)
                b200::causal_conv_run_kernel<TI, TO, 4><<<grid_r, 128, 0, stream>>>((const TI*)x, ld_x, w, bias, state, (size_t)slot_stride,
                                                                                  slots, seq_ids, cu_seqlens, (TO*)out, ld_out, channels,
                                                                                  taps, activation, add_input, n_tokens);
            else if (runs)
                b200::causal_conv_run_kernel<TI, TO, 8><<<grid_r, 128, 0, stream>>>((const TI*)x, ld_x, w, bias, state, (size_t)slot_stride,
                                                                                  slots, seq_ids, cu_seqlens, (TO*)out, ld_out, channels,
                                                                                  taps, activation, add_input, n_tokens);
            else if (wide)
                b200::causal_conv_kernel<TI, TO, 4><<<grid, 128, 0, stream>>>((const TI*)x, ld_x, w, bias, state, (size_t)slot_stride,
                                                                            slots, seq_ids, cu_seqlens, (TO*)out, ld_out, channels,
                                                                            taps, activation, add_input);
            else
                b200::causal_conv_kernel<TI, TO, 1><<<grid, 128, 0, stream>>>((const TI*)x, ld_x, w, bias, state, (size_t)slot_stride,
                                                                            slots, seq_ids, cu_seqlens, (TO*)out, ld_out, channels,
                                                                            taps, activation, add_input));
        if (update_state && taps > 1)
            b200::conv_state_update_kernel<TI><<<grid_u, 128, 0, stream>>>((const TI*)x, ld_x, state, (size_t)slot_stride, slots,
                                                                          cu_seqlens, channels, taps));
    return b200::launch_status();
}

// The rows a thread holds (rows_per_thread: 8, 12, 16, 24 or 32) times the lanes that share a column (a power of two up
// to 16) must cover d_k; b200_delta_rule_plan picks the pair for a d_k (0 when none fits): the fewest rows beyond d_k,
// then the fewest rows per thread (shared memory is read once per row and token by every warp).
extern "C" int b200_delta_rule_plan(int d_k, int* rows_per_thread, int* lanes) {
    const int options[5] = {8, 12, 16, 24, 32};
    int best = 0, best_pad = 1 << 30;
    for (int oi = 0; oi < 5; ++oi)
        for (int R = 1; R <= 16; R *= 2) {
            const int pad = options[oi] * R;
            if (pad >= d_k && pad < best_pad) {
                best_pad = pad;
                best = options[oi];
                *rows_per_thread = options[oi];
                *lanes = R;
            }
        }
    return best;
}

// Floats of one (token, head) row of the scratch that b200_delta_rule_scan needs: n_tokens * heads * this many
// (0 for a d_k no kernel holds).
extern "C" int b200_delta_rule_row(int d_k, int d_v) {
    int rpt = 0, lanes = 0;
    if (!b200_delta_rule_plan(d_k, &rpt, &lanes)) return 0;
    return (3 * rpt * lanes + d_v + 3 + 3) / 4 * 4;
}

extern "C" int b200_delta_rule_scan(const void* qkv, int ld_qkv, const void* beta, int ld_beta, const void* decay,
                                    int ld_decay, const float* dt_bias, const float* a_log, float* state,
                                    long long slot_stride, const int* slots, const int* cu_seqlens, float* out,
                                    float* scratch, int dtype, int n_tokens, int n_seqs, int heads, int kv_heads, int d_k,
                                    int d_v, float q_scale, float unit_eps, int decay_per_head, cudaStream_t stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (heads < 1 || kv_heads < 1 || heads % kv_heads || d_k < 1 || d_v < 1 || n_seqs > 65535 || heads > 65535 || !scratch)
        return b200::kErrBadArgument;
    int rpt = 0, lanes = 0;
    if (!b200_delta_rule_plan(d_k, &rpt, &lanes)) return b200::kErrUnsupportedSize;
    const int row = b200_delta_rule_row(d_k, d_v);
    if ((uintptr_t)scratch % 16) return b200::kErrBadArgument;
    b200::PrepareArgs p = {qkv, ld_qkv, beta, ld_beta, decay, ld_decay, dt_bias, a_log, scratch, n_tokens, heads, kv_heads,
                           d_k, d_v, rpt * lanes, row, q_scale, unit_eps, decay_per_head ? 1 : 0};
    const long long units = (long long)n_tokens * heads;
    B200_DISPATCH_DTYPE(dtype, T,
        b200::delta_rule_prepare_kernel<T><<<(unsigned)((units + 3) / 4), 128, 0, stream>>>(p));
    b200::ScanArgs a = {scratch, state, (size_t)slot_stride, slots, cu_seqlens, out, n_tokens, heads, d_k, d_v, row};
    return b200::launch_scan_rows<false>(a, rpt, lanes, n_seqs, stream);
}

// The recurrence without the delta correction over a packed step; see LinearPrepareArgs for the operands.  q, k, v and
// decay share one storage type; state and out as for b200_delta_rule_scan.
extern "C" int b200_linear_scan(const void* q, int ld_q, const void* k, int ld_k, const void* v, int ld_v, const void* decay,
                                int ld_decay, const float* decay_bias, const float* a_log, const float* skip, float* state,
                                long long slot_stride, const int* slots, const int* cu_seqlens, float* out, float* scratch,
                                int dtype, int n_tokens, int n_seqs, int heads, int kv_heads, int d_k, int d_v, float q_scale,
                                float power, int decay_kind, int decay_per_head, int step_scales_value, cudaStream_t stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (heads < 1 || kv_heads < 1 || heads % kv_heads || d_k < 1 || d_v < 1 || n_seqs > 65535 || heads > 65535 || !scratch)
        return b200::kErrBadArgument;
    if ((decay_kind != 0 && decay_kind != 1) || (decay_kind == 0 && !a_log)) return b200::kErrBadArgument;
    int rpt = 0, lanes = 0;
    if (!b200_delta_rule_plan(d_k, &rpt, &lanes)) return b200::kErrUnsupportedSize;
    const int row = b200_delta_rule_row(d_k, d_v);
    if ((uintptr_t)scratch % 16) return b200::kErrBadArgument;
    b200::LinearPrepareArgs p = {q, ld_q, k, ld_k, v, ld_v, decay, ld_decay, decay_bias, a_log, skip, scratch, n_tokens, heads,
                                 kv_heads, d_k, d_v, rpt * lanes, row, q_scale, power, decay_kind, decay_per_head ? 1 : 0,
                                 step_scales_value ? 1 : 0};
    const long long units = (long long)n_tokens * heads;
    B200_DISPATCH_DTYPE(dtype, T,
        b200::linear_scan_prepare_kernel<T><<<(unsigned)((units + 3) / 4), 128, 0, stream>>>(p));
    b200::ScanArgs a = {scratch, state, (size_t)slot_stride, slots, cu_seqlens, out, n_tokens, heads, d_k, d_v, row};
    return b200::launch_scan_rows<true>(a, rpt, lanes, n_seqs, stream);
}
