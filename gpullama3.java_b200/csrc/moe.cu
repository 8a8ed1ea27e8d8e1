// A routed feed-forward (mixture of experts): the router, and the experts for steps of few tokens.
//
//   moe_route     per token: logits z = W_r h (+ bias) (32-bit sums, W_r kept in 32 bits), scores s = softmax(z) over all experts.
//                 The experts form `n_groups` equal groups of neighbours; a group's score is its best expert's score, and
//                 only experts of the `keep_groups` best groups may be chosen.  The `top` allowed experts with the
//                 largest scores are chosen (ties: the lower index); their weights are their scores over the sum of
//                 the chosen scores (+ norm_eps).  A CTA per token.
//   moe_group     the (token, choice) pairs ordered by expert (counting sort; the order inside an expert's run does not
//                 change any result, a row of a product depends on its own input row only).
//   moe_rows      steps of few tokens: every expert's rows as a weight-streaming product whose row counts are read on
//                 the device, so a decode step's launches do not depend on the routing; an expert's weights are read once
//                 for all tokens that chose it (in groups of eight), an expert nobody chose is not read.  Used twice:
//                 gate and up rows with the gated epilogue (the same codes as the products' gated epilogues), then down.
//                 bfloat16 runs on the tensor cores (mma.sync, the eight rows as a tile's columns), float32 on the FMA pipe.
//   moe_gather    prompts: the inputs copied into the order of their experts, so that each expert's rows are one dense
//                 product for the tensor-core kernels.
//   moe_combine   the experts' results carried back, weighted and summed in the order of choice, into the 32-bit
//                 residual stream.
#include "common.cuh"

namespace b200 {

constexpr int kMaxExperts = 1024;

template <typename T> struct Piece;  // 16 bytes of storage type T as floats
template <> struct Piece<float> {
    static constexpr int kElems = 4;
    __device__ static void load(const float* p, float* f) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
};
template <> struct Piece<__nv_bfloat16> {
    static constexpr int kElems = 8;
    __device__ static void load(const __nv_bfloat16* p, float* f) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// sum_k w[k] x[k] over a warp: lanes take 16-byte pieces of the weight row when VEC, single elements otherwise;
// x is in shared memory as floats
template <typename T, bool VEC>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const float* __restrict__ x, int K, int lane) {
    float acc = 0.f;
    if (VEC) {
        constexpr int E = Piece<T>::kElems;
        for (int k = lane * E; k < K; k += 32 * E) {
            float f[E];
            Piece<T>::load(w + k, f);
#pragma unroll
            for (int e = 0; e < E; ++e) acc += f[e] * x[k + e];
        }
    } else {
        for (int k = lane; k < K; k += 32) acc += to_f32<T>(w[k]) * x[k];
    }
    return warp_sum(acc);
}

// ------------------------------------------------------------------------------------------------ router
struct RouteArgs {
    const void* h;          // [T][ld_h], the run's storage type
    int ld_h;
    const float* router;    // [n_experts][width]
    int* chosen;            // [T][top]
    float* weights;         // [T][top]
    float* scores;          // [T][n_experts] or null: the softmax scores, for inspection
    int n_tokens, width, n_experts, n_groups, keep_groups, top;
    float norm_eps;
    const float* bias;      // [n_experts] added to the logits, or null
};

constexpr int kRouteThreads = 128;

// A CTA per token: its warps share out the experts' logits (16 bytes of a router row per lane and step when the rows
// allow), then the first warp does the softmax and the choice.
template <typename T>
__global__ void __launch_bounds__(kRouteThreads)
moe_route_kernel(RouteArgs a) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* x = smem;                       // the token's input
    float* s = x + a.width;                // logits, then scores; chosen or barred ones turn negative
    float* gs = s + a.n_experts;           // group scores
    const int t = blockIdx.x;
    const T* hr = (const T*)a.h + (size_t)t * a.ld_h;
    for (int k = threadIdx.x; k < a.width; k += kRouteThreads) x[k] = to_f32<T>(hr[k]);
    __syncthreads();
    const bool vec = a.width % 4 == 0 && ((uintptr_t)a.router & 15) == 0;
    for (int e = warp; e < a.n_experts; e += kRouteThreads / 32) {
        const float* w = a.router + (size_t)e * a.width;
        const float z = vec ? warp_dot<float, true>(w, x, a.width, lane) : warp_dot<float, false>(w, x, a.width, lane);
        if (lane == 0) s[e] = z + (a.bias ? a.bias[e] : 0.f);
    }
    __syncthreads();
    if (warp != 0) return;
    float m = -INFINITY;
    for (int e = lane; e < a.n_experts; e += 32) m = fmaxf(m, s[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < a.n_experts; e += 32) sum += expf(s[e] - m);
    sum = warp_sum(sum);
    for (int e = lane; e < a.n_experts; e += 32) {
        s[e] = expf(s[e] - m) / sum;
        if (a.scores) a.scores[(size_t)t * a.n_experts + e] = s[e];
    }
    __syncwarp();
    // groups: keep the best `keep_groups`, bar the experts of the others
    const int per = a.n_experts / a.n_groups;
    if (a.keep_groups < a.n_groups) {
        for (int g = lane; g < a.n_groups; g += 32) {
            float best = -1.f;
            for (int i = 0; i < per; ++i) best = fmaxf(best, s[g * per + i]);
            gs[g] = best;
        }
        __syncwarp();
        for (int r = 0; r < a.keep_groups; ++r) {
            float bv = -2.f;
            int bi = 0x7fffffff;
            for (int g = lane; g < a.n_groups; g += 32)
                if (gs[g] > bv) { bv = gs[g]; bi = g; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) gs[bi] = -3.f;    // taken
            __syncwarp();
        }
        for (int e = lane; e < a.n_experts; e += 32)
            if (gs[e / per] != -3.f) s[e] = -1.f - s[e];   // barred: negative
        __syncwarp();
    }
    // the `top` best allowed experts, one after the other
    float chosen_sum = 0.f;
    float my_w = 0.f;
    int my_e = 0;
    for (int r = 0; r < a.top; ++r) {
        float bv = -1.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < a.n_experts; e += 32)
            if (s[e] > bv) { bv = s[e]; bi = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        chosen_sum += bv;
        if (lane == r) { my_w = bv; my_e = bi; }
        if (lane == 0) s[bi] = -1.f;
        __syncwarp();
    }
    if (lane < a.top) {
        a.chosen[(size_t)t * a.top + lane] = my_e;
        a.weights[(size_t)t * a.top + lane] = my_w / (chosen_sum + a.norm_eps);
    }
}

// ------------------------------------------------------------------------------------------------ experts, few rows each
__device__ __forceinline__ float gated_value(float gate, float up, int act, float limit, float slope) {
    if (act == 2) {
        const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);
        return g / (1.0f + expf(-slope * g)) * (u + 1.0f);
    }
    if (act == 1) return 0.5f * gate * (1.0f + tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate))) * up;
    return gate / (1.0f + expf(-gate)) * up;
}

constexpr int kRowsWarps = 8;
constexpr int kRowsTokens = 8;    // rows of A that meet a weight row while it is in registers

struct RowsArgs {
    const void* a;          // rows of A, [.][ld_a]: row order[p] / top when `order` is given, row p otherwise
    int ld_a;
    const int* order;
    int top;
    const void* w;          // [n_experts][n_out (2 n_out when gated: gate and up rows interleaved)][K]
    const int* offsets;     // [n_experts + 1]: expert e owns places offsets[e] .. offsets[e + 1] - 1
    void* out;              // gated: [.][ld_out] of the run's type; plain: 32-bit
    int ld_out;
    int K, n_out, units_per_cta;
    int act;
    float limit, slope;
};

__device__ __forceinline__ uint4 load_streamed(const void* p) {    // weights pass once: they need not stay in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
template <typename T> __device__ __forceinline__ void unpack16(const uint4& v, float* f);
template <> __device__ __forceinline__ void unpack16<float>(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// out[p] = A[row(p)] W_e^T (gated: act of the gate and up sums) for the places p of expert e = blockIdx.y: a weight-
// streaming product.  The CTA stages up to kRowsTokens rows of A in shared memory; a warp carries two weight rows at a
// time through its registers (a gate row and its up row, or two neighbouring rows of a plain product), four 16-byte
// pieces of each in flight, once per staged group, and keeps a sum per staged row and weight row.  An expert nobody
// chose costs its CTAs one read of two integers.  Sums run over k in a fixed order: a row's result does not depend on
// its place.
template <typename T, bool GATED, bool VEC>
__global__ void __launch_bounds__(kRowsWarps * 32)
moe_rows_kernel(RowsArgs r) {
    extern __shared__ __align__(16) unsigned char raw[];
    T* xs = reinterpret_cast<T*>(raw);                 // [kRowsTokens][K]
    constexpr int E = Piece<T>::kElems;
    const int e = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lo = r.offsets[e], hi = r.offsets[e + 1];
    if (hi <= lo) return;
    const int n_rows = GATED ? 2 * r.n_out : r.n_out;  // weight rows of the expert
    const T* w = (const T*)r.w + (size_t)e * n_rows * r.K;
    for (int g0 = lo; g0 < hi; g0 += kRowsTokens) {
        const int cnt = min(kRowsTokens, hi - g0);
        __syncthreads();                               // (the group before has been read)
        for (int m = 0; m < cnt; ++m) {
            const int p = g0 + m;
            const T* src = (const T*)r.a + (size_t)(r.order ? r.order[p] / r.top : p) * r.ld_a;
            if (VEC) {
                for (int k = threadIdx.x * E; k < r.K; k += kRowsWarps * 32 * E)
                    *reinterpret_cast<uint4*>(xs + (size_t)m * r.K + k) = *reinterpret_cast<const uint4*>(src + k);
            } else {
                for (int k = threadIdx.x; k < r.K; k += kRowsWarps * 32) xs[(size_t)m * r.K + k] = src[k];
            }
        }
        __syncthreads();
        for (int unit = warp; unit < r.units_per_cta; unit += kRowsWarps) {
            const int row0 = 2 * (blockIdx.x * r.units_per_cta + unit);      // this warp's two weight rows: row0, row0 + 1
            if (row0 >= n_rows) break;
            const bool second = row0 + 1 < n_rows;
            const T* w0 = w + (size_t)row0 * r.K;
            const T* w1 = second ? w0 + r.K : w0;
            float acc0[kRowsTokens], acc1[kRowsTokens];
#pragma unroll
            for (int m = 0; m < kRowsTokens; ++m) acc0[m] = acc1[m] = 0.f;
            if (VEC) {
                constexpr int U = 4;                   // pieces of each row in flight
                for (int k0 = lane * E; k0 < r.K; k0 += U * 32 * E) {
                    uint4 p0[U], p1[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int k = k0 + u * 32 * E;
                        if (k < r.K) {
                            p0[u] = load_streamed(w0 + k);
                            p1[u] = load_streamed(w1 + k);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int k = k0 + u * 32 * E;
                        if (k < r.K) {
                            float f0[E], f1[E];
                            unpack16<T>(p0[u], f0);
                            unpack16<T>(p1[u], f1);
#pragma unroll
                            for (int m = 0; m < kRowsTokens; ++m) {
                                if (m < cnt) {
                                    float xv[E];
                                    Piece<T>::load(xs + (size_t)m * r.K + k, xv);
#pragma unroll
                                    for (int i = 0; i < E; ++i) {
                                        acc0[m] += f0[i] * xv[i];
                                        acc1[m] += f1[i] * xv[i];
                                    }
                                }
                            }
                        }
                    }
                }
            } else {
                for (int k = lane; k < r.K; k += 32) {
                    const float a0 = to_f32<T>(w0[k]), a1 = to_f32<T>(w1[k]);
#pragma unroll
                    for (int m = 0; m < kRowsTokens; ++m) {
                        if (m < cnt) {
                            const float xv = to_f32<T>(xs[(size_t)m * r.K + k]);
                            acc0[m] += a0 * xv;
                            acc1[m] += a1 * xv;
                        }
                    }
                }
            }
#pragma unroll
            for (int m = 0; m < kRowsTokens; ++m) {
                if (m < cnt) {
                    const float s0 = warp_sum(acc0[m]), s1 = warp_sum(acc1[m]);
                    if (lane == 0) {
                        const size_t at = (size_t)(g0 + m) * r.ld_out;
                        if (GATED) {
                            ((T*)r.out)[at + row0 / 2] = from_f32<T>(gated_value(s0, s1, r.act, r.limit, r.slope));
                        } else {
                            ((float*)r.out)[at + row0] = s0;
                            if (second) ((float*)r.out)[at + row0 + 1] = s1;
                        }
                    }
                }
            }
        }
    }
}

// The same product for bfloat16 on the tensor cores (mma.sync m16n8k16): the eight staged rows of A are the eight
// columns of the tiles, sixteen weight rows their rows.  A lane loads 16 bytes of weight rows g and g + 8 (the 8 t-th
// elements of a block of 32 along K) and 16 bytes of staged row g at the same place; the four pairs of those elements
// feed two MMAs, which amounts to a fixed permutation of K inside the block, the same for both operands.  A CTA of
// eight warps owns 8 / KS tiles of weight rows and cuts K into KS parts, one warp per (tile, part), up to eight blocks of
// each weight row in flight per lane; the parts' sums meet in shared memory and are added in part order.  Rows of the
// group that do not exist are zeros.
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool GATED>
__global__ void __launch_bounds__(kRowsWarps * 32)
moe_rows_mma_kernel(RowsArgs r, int k_parts) {
    extern __shared__ __align__(16) unsigned char raw[];
    const int ldx = r.K + 8;                                    // (16 bytes of padding: the eight rows start in different banks)
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(raw);  // [kRowsTokens][ldx]
    float* part = reinterpret_cast<float*>(xs + (size_t)kRowsTokens * ldx);   // [kRowsWarps][32][4]
    const int e = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int lo = r.offsets[e], hi = r.offsets[e + 1];
    if (hi <= lo) return;
    const int n_rows = GATED ? 2 * r.n_out : r.n_out;
    const __nv_bfloat16* w = (const __nv_bfloat16*)r.w + (size_t)e * n_rows * r.K;
    const int tiles_per_cta = kRowsWarps / k_parts, tile = warp / k_parts, kp = warp % k_parts;
    const int row0 = (blockIdx.x * tiles_per_cta + tile) * 16;
    const int n_kb = r.K / 32, per_part = (n_kb + k_parts - 1) / k_parts;
    const int kb_lo = kp * per_part, kb_hi = min(n_kb, kb_lo + per_part);
    const bool live = row0 < n_rows;
    const __nv_bfloat16* wa = w + (size_t)min(row0 + g, n_rows - 1) * r.K + 8 * t;       // (rows beyond the last: read, never stored)
    const __nv_bfloat16* wb = w + (size_t)min(row0 + g + 8, n_rows - 1) * r.K + 8 * t;
    for (int g0 = lo; g0 < hi; g0 += kRowsTokens) {
        const int cnt = min(kRowsTokens, hi - g0);
        __syncthreads();                               // (the group before has been read, its partial sums too)
        for (int m = 0; m < kRowsTokens; ++m) {
            uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)m * ldx);
            if (m < cnt) {
                const int p = g0 + m;
                const uint4* src = reinterpret_cast<const uint4*>((const __nv_bfloat16*)r.a + (size_t)(r.order ? r.order[p] / r.top : p) * r.ld_a);
                for (int i = threadIdx.x; i < r.K / 8; i += kRowsWarps * 32) dst[i] = src[i];
            } else {
                for (int i = threadIdx.x; i < r.K / 8; i += kRowsWarps * 32) dst[i] = make_uint4(0, 0, 0, 0);
            }
        }
        __syncthreads();
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
            constexpr int U = 8;
            const __nv_bfloat16* xr = xs + (size_t)g * ldx + 8 * t;
            for (int kb = kb_lo; kb < kb_hi; kb += U) {
                uint4 A[U], B[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (kb + u < kb_hi) {
                        A[u] = load_streamed(wa + (size_t)(kb + u) * 32);
                        B[u] = load_streamed(wb + (size_t)(kb + u) * 32);
                    }
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (kb + u < kb_hi) {
                        const uint4 X = *reinterpret_cast<const uint4*>(xr + (size_t)(kb + u) * 32);
                        mma_bf16(d, A[u].x, B[u].x, A[u].y, B[u].y, X.x, X.y);
                        mma_bf16(d, A[u].z, B[u].z, A[u].w, B[u].w, X.z, X.w);
                    }
            }
        }
        if (k_parts > 1) {
            float4* mine = reinterpret_cast<float4*>(part) + warp * 32 + lane;
            *mine = make_float4(d[0], d[1], d[2], d[3]);
            __syncthreads();
            if (kp == 0) {
                for (int q = 1; q < k_parts; ++q) {
                    const float4 o = reinterpret_cast<const float4*>(part)[(warp + q) * 32 + lane];
                    d[0] += o.x; d[1] += o.y; d[2] += o.z; d[3] += o.w;
                }
            }
        }
        if (live && kp == 0) {
            // d[0], d[1]: weight row row0 + g, staged rows 2 t and 2 t + 1;  d[2], d[3]: weight row row0 + g + 8
            if (GATED) {
                float up[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) up[i] = __shfl_xor_sync(0xffffffffu, d[i], 4);   // the odd row next to this even one
                if ((g & 1) == 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int m = 2 * t + (i & 1), row = row0 + g + (i >> 1) * 8;
                        if (m < cnt && row + 1 < n_rows)
                            ((__nv_bfloat16*)r.out)[(size_t)(g0 + m) * r.ld_out + row / 2] =
                                __float2bfloat16_rn(gated_value(d[i], up[i], r.act, r.limit, r.slope));
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int m = 2 * t + (i & 1), row = row0 + g + (i >> 1) * 8;
                    if (m < cnt && row < n_rows) ((float*)r.out)[(size_t)(g0 + m) * r.ld_out + row] = d[i];
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ prompts: order by expert
// One CTA.  offsets[e] .. offsets[e + 1]: the run of expert e among the ordered pairs; order[p]: which pair stands at
// place p; place[pair]: where a pair stands.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, int* __restrict__ offsets,
                 int* __restrict__ order, int* __restrict__ place) {
    __shared__ int count[kMaxExperts + 1];
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&count[chosen[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_experts; ++e) {
            const int n = count[e];
            offsets[e] = run;
            count[e] = run;      // from here on: the next free place of the expert's run
            run += n;
        }
        offsets[n_experts] = run;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int at = atomicAdd(&count[chosen[p]], 1);
        order[at] = p;
        place[p] = at;
    }
}

// x_sorted[p] = h[order[p] / top]; 16 bytes per thread and step when the rows allow
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, int ld_h, const int* __restrict__ order, T* __restrict__ out,
                                  int width, int top, int vec) {
    const int p = blockIdx.x;
    const T* src = h + (size_t)(order[p] / top) * ld_h;
    T* dst = out + (size_t)p * width;
    if (vec) {
        const int n = width * (int)sizeof(T) / 16;
        for (int i = threadIdx.x; i < n; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int k = threadIdx.x; k < width; k += blockDim.x) dst[k] = src[k];
    }
}

// residual[t] += sum_k weights[t][k] o[place[t top + k]], in the order of choice
__global__ void moe_combine_kernel(const float* __restrict__ o, const int* __restrict__ place, const float* __restrict__ weights,
                                   float* __restrict__ residual, int width, int top) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float total = 0.f;
        for (int k = 0; k < top; ++k)
            total += weights[(size_t)t * top + k] * o[(size_t)place[(size_t)t * top + k] * width + c];
        residual[(size_t)t * width + c] += total;
    }
}

}  // namespace b200

namespace b200 {
// Routing without a router: row tokens[t] of a table names the token's experts, all weighted alike.
__global__ void moe_table_route_kernel(const int* __restrict__ tokens, const int* __restrict__ table, int* __restrict__ chosen,
                                       float* __restrict__ weights, int n, int top, int n_experts) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = table[(size_t)tokens[i / top] * top + i % top];
    chosen[i] = min(max(e, 0), n_experts - 1);   // (a table entry outside the experts cannot index past them)
    weights[i] = 1.0f / (float)top;
}
}  // namespace b200

extern "C" int b200_moe_table_route(const int* tokens, const int* table, int* chosen, float* weights, int n_tokens, int top,
                                    int n_experts, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (top < 1 || n_experts < 1) return b200::kErrBadArgument;
    const int n = n_tokens * top;
    b200::moe_table_route_kernel<<<(n + 255) / 256, 256, 0, stream>>>(tokens, table, chosen, weights, n, top, n_experts);
    return b200::launch_status();
}

extern "C" int b200_moe_route(const void* h, int ld_h, int dtype, const float* router, int* chosen, float* weights,
                              float* scores, int n_tokens, int width, int n_experts, int n_groups, int keep_groups, int top,
                              float norm_eps, const float* bias, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_experts < 1 || n_experts > b200::kMaxExperts || top < 1 || top > 32 || top > n_experts || n_groups < 1 ||
        n_experts % n_groups || keep_groups < 1 || keep_groups > n_groups || top > keep_groups * (n_experts / n_groups))
        return b200::kErrBadArgument;
    const size_t smem = sizeof(float) * ((size_t)width + n_experts + n_groups);
    if (smem > 200 * 1024) return b200::kErrUnsupportedSize;
    const b200::RouteArgs a = {h, ld_h, router, chosen, weights, scores, n_tokens, width, n_experts, n_groups, keep_groups, top, norm_eps, bias};
    B200_DISPATCH_DTYPE(dtype, T,
        auto kernel = b200::moe_route_kernel<T>;
        if (smem > 48 * 1024) {
            const int e = (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != 0) return e;
        }
        kernel<<<n_tokens, b200::kRouteThreads, smem, stream>>>(a));
    return b200::launch_status();
}

// One product per expert over the places offsets[e] .. offsets[e + 1] - 1 (see moe_rows_kernel).  gated: w holds gate
// and up rows interleaved and `out` is of the run's type; else `out` is 32-bit.  act: 0 SiLU, 1 GELU (tanh form), 2 clamped.
extern "C" int b200_moe_rows(const void* a, int ld_a, int dtype, const int* order, int top, const void* w, const int* offsets,
                             void* out, int ld_out, int n_experts, int K, int n_out, int gated, int act, float limit,
                             float slope, cudaStream_t stream) {
    if (n_experts <= 0 || n_out <= 0) return 0;
    if (K < 1 || act < 0 || act > 2 || (order && top < 1) || n_experts > 65535) return b200::kErrBadArgument;
    const size_t el = dtype == b200::kF32 ? 4 : 2;
    const size_t smem = (size_t)b200::kRowsTokens * K * el;
    if (smem > 200 * 1024) return b200::kErrUnsupportedSize;
    const int per16 = 16 / (int)el;
    const bool vec = K % per16 == 0 && ld_a % per16 == 0 && ((((uintptr_t)a) | ((uintptr_t)w)) & 15) == 0;
    const int units = gated ? n_out : (n_out + 1) / 2;     // pairs of weight rows
    b200::RowsArgs r = {a, ld_a, order, top, w, offsets, out, ld_out, K, n_out, units >= 1024 ? 16 : 8, act, limit, slope};
    const dim3 grid((units + r.units_per_cta - 1) / r.units_per_cta, n_experts);
    if (dtype == b200::kBF16 && vec && K % 32 == 0) {
        // tensor cores: tiles of 16 weight rows; K is cut among a CTA's warps until the grid has about eight CTAs per SM (the
        // experts nobody chose leave theirs at once, and short CTAs even out what the SMs get)
        const long long tiles = (long long)((gated ? 2 * n_out : n_out) + 15) / 16 * n_experts;
        int k_parts = 1;
        while (k_parts < b200::kRowsWarps && tiles * k_parts / b200::kRowsWarps < 8LL * b200::device_sm_count() && K / 32 >= 2 * k_parts)
            k_parts *= 2;
        const int per_cta = b200::kRowsWarps / k_parts;
        const dim3 mma_grid(((gated ? 2 * n_out : n_out) + 16 * per_cta - 1) / (16 * per_cta), n_experts);
        const size_t mma_smem = (size_t)b200::kRowsTokens * (K + 8) * 2 + sizeof(float) * b200::kRowsWarps * 32 * 4;
        if (mma_smem <= 200 * 1024) {
            if (gated) {
                auto kernel = b200::moe_rows_mma_kernel<true>;
                if (mma_smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mma_smem) != cudaSuccess)
                    return (int)cudaGetLastError();
                kernel<<<mma_grid, b200::kRowsWarps * 32, mma_smem, stream>>>(r, k_parts);
            } else {
                auto kernel = b200::moe_rows_mma_kernel<false>;
                if (mma_smem > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mma_smem) != cudaSuccess)
                    return (int)cudaGetLastError();
                kernel<<<mma_grid, b200::kRowsWarps * 32, mma_smem, stream>>>(r, k_parts);
            }
            return b200::launch_status();
        }
    }
#define B200_ROWS_GO(T, G, V)                                                                                         \
    do {                                                                                                              \
        auto kernel = b200::moe_rows_kernel<T, G, V>;                                                                 \
        if (smem > 48 * 1024) {                                                                                       \
            const int e = (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
            if (e != 0) return e;                                                                                     \
        }                                                                                                             \
        kernel<<<grid, b200::kRowsWarps * 32, smem, stream>>>(r);                                                     \
    } while (0)
    B200_DISPATCH_DTYPE(dtype, T,
        if (gated) { if (vec) B200_ROWS_GO(T, true, true); else B200_ROWS_GO(T, true, false); }
        else { if (vec) B200_ROWS_GO(T, false, true); else B200_ROWS_GO(T, false, false); });
#undef B200_ROWS_GO
    return b200::launch_status();
}

extern "C" int b200_moe_group(const int* chosen, int n_pairs, int n_experts, int* offsets, int* order, int* place,
                              cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (n_experts < 1 || n_experts > b200::kMaxExperts) return b200::kErrBadArgument;
    b200::moe_group_kernel<<<1, 1024, 0, stream>>>(chosen, n_pairs, n_experts, offsets, order, place);
    return b200::launch_status();
}

extern "C" int b200_moe_gather(const void* h, int ld_h, int dtype, const int* order, void* out, int n_pairs, int width,
                               int top, cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    const int el = dtype == b200::kF32 ? 4 : 2;
    const int vec = (width * el) % 16 == 0 && (ld_h * el) % 16 == 0 && ((((uintptr_t)h) | ((uintptr_t)out)) & 15) == 0;
    B200_DISPATCH_DTYPE(dtype, T,
        b200::moe_gather_kernel<T><<<n_pairs, 128, 0, stream>>>((const T*)h, ld_h, order, (T*)out, width, top, vec));
    return b200::launch_status();
}

extern "C" int b200_moe_combine(const float* o, const int* place, const float* weights, float* residual, int n_tokens,
                                int width, int top, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    b200::moe_combine_kernel<<<n_tokens, 256, 0, stream>>>(o, place, weights, residual, width, top);
    return b200::launch_status();
}
