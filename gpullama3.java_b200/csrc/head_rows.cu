// What happens to the rows of a projection between the product and the attention kernels, for mixers whose
// queries, keys, values or latents are not used as the product leaves them:
//     z = x[src + r d .. + d] (+ bias)              one row of d numbers per (token, head)
//     z <- z / sqrt(mean(z^2) + eps)                (optional: an RMS norm per row, or one over all rows of the
//                                                   segment at once, before they are split into heads; 32-bit)
//     z <- z * weight[0 .. d)                       (optional: the norm's weight, shared by the rows or one per element
//                                                   of the segment)
//     z <- z * mul                                  (a score scale folded into the queries, or 1)
//     z <- (1 - lambda) z + lambda other[...]       (optional: mixed with the same element of another layer's rows of the
//                                                   same token, lambda a number in device memory; 32-bit)
//     dst[dst_off + r d_pad .. + d_pad] = z, 0, ..., 0   (rows may be widened with zeros to the size a kernel takes; `lead` of
//                                                   the zeros may stand in front of z, so that two rows that share a
//                                                   wider key row each meet their own part of it)
//     (z[2i], z[2i+1]) <- turned by position * inv_freq[i]   (optional: rotary position encoding over the row's interleaved
//                                                   pairs, the angle, its cosine and sine in 32 bits; `mul` then also carries
//                                                   a factor on cosine and sine)
// A segment's rows need not lie back to back (`src_stride`: a part of every head of a wider projection; 0 as a stride:
// every row reads the same numbers, one row shared by all heads) nor be written back to back (`dst_stride`), and a row may
// fill only some columns of a cache row (`dst_off` columns in, `cache_dim` the cache's row size), so that two segments can
// make up one key row.
// A segment's rows go to a dense buffer (queries), or straight into the paged cache at the token's position: as key
// rows ([page][kv_head][position][d_pad]) or as value rows (transposed, [page][kv_head][d_pad][position]), so that
// a mixer without rotation needs no other kernel between its projection and attention.
// Up to six such segments of a token's row are handled by one launch (queries, keys and values of an attention
// layer; a latent that is stored once as keys and once as values).  A warp per (token, row), or a CTA per token when a
// segment's norm runs over all its rows.
#include "common.cuh"

namespace b200 {

constexpr int kRowSegments = 6;
constexpr int kSegmentWords = 20;   // 32-bit words of one segment record at the C interface (17 used)
constexpr int kRowThreads = 128;

struct RowSegment {
    int src_off, n_rows, d, dst_off, d_pad;
    int bias_off;     // into `bias`, -1: none
    int norm;         // 1: divide by the row's root mean square; 2: by that of all the segment's rows together
    int weight_off;   // into `weight`, -1: none
    float mul;
    int target;       // 0: dst; 1: key rows of the cache; 2: value rows of the cache
    int weight_per_row;  // 1: the weight has n_rows * d entries (one per element of the segment), 0: d (shared by the rows)
    int mix_off;      // column of `other` where this segment's counterpart starts, -1: no mixing
    int rotate;       // 1: the row's pairs (2i, 2i + 1) are turned by position * inv_freq[i] (d even, no mixing)
    int src_stride;   // numbers between two rows of the source (-1: d)
    int dst_stride;   // numbers between two rows written to dst (-1: d_pad)
    int cache_dim;    // row size of the cache the segment goes into (-1: d_pad); the segment starts dst_off columns in
    int lead;         // zeros written in front of the row: of the d_pad numbers the first `lead` are zero, then the d, then zeros
};
struct MixSource {
    const void* other;      // [T][ld_other], the run's storage type
    int ld_other;
    const float* lambda;    // one number
};
struct CacheTarget {
    const int* positions;
    const int* seq_ids;
    const int* page_table;
    int table_stride;
    void* k_pool;
    void* v_pool;
    const float* inv_freq;   // for segments that rotate
};
struct RowSegments {
    RowSegment seg[kRowSegments];
    int n;
    int total_rows;
};

// One (token, row): `whole` is the segment's 1 / rms when its norm runs over all its rows (made once per token by the
// caller), unused otherwise.
template <typename T>
__device__ __forceinline__ void head_row(const T* __restrict__ src, int ld_src, T* __restrict__ dst, int ld_dst,
                                         const float* __restrict__ bias, const float* __restrict__ weight, const RowSegment& g,
                                         int t, int row, int lane, float eps, float whole, const CacheTarget& cache,
                                         const MixSource& mix) {
    const T* x = src + (size_t)t * ld_src + g.src_off + (size_t)row * (g.src_stride >= 0 ? g.src_stride : g.d);
    const float* b = g.bias_off >= 0 ? bias + g.bias_off + (size_t)row * g.d : nullptr;
    float factor = g.mul;
    if (g.norm == 2) {
        factor *= whole;
    } else if (g.norm) {
        float ss = 0.f;
        for (int e = lane; e < g.d; e += 32) {
            const float z = to_f32<T>(x[e]) + (b ? b[e] : 0.f);
            ss += z * z;
        }
        ss = warp_sum(ss);
        factor *= 1.0f / sqrtf(ss / (float)g.d + eps);
    }
    const float* w = g.weight_off >= 0 ? weight + g.weight_off + (g.weight_per_row ? (size_t)row * g.d : 0) : nullptr;
    const T* other = g.mix_off >= 0 ? (const T*)mix.other + (size_t)t * mix.ld_other + g.mix_off + (size_t)row * g.d : nullptr;
    const float lambda = other ? mix.lambda[0] : 0.f;
    T* o = dst + (size_t)t * ld_dst + g.dst_off + (size_t)row * (g.dst_stride >= 0 ? g.dst_stride : g.d_pad);
    size_t step = 1;
    if (g.target != 0) {   // the row's place in the page of this token's position (n_rows = the cache's kv heads)
        const int pos = cache.positions[t];
        const int dim = g.cache_dim >= 0 ? g.cache_dim : g.d_pad;
        const size_t page = cache.page_table[(size_t)cache.seq_ids[t] * cache.table_stride + pos / kPageTokens];
        const size_t head = (page * g.n_rows + row) * kPageTokens * dim;
        if (g.target == 1) {
            o = (T*)cache.k_pool + head + (size_t)(pos % kPageTokens) * dim + (g.cache_dim >= 0 ? g.dst_off : 0);
        } else {
            o = (T*)cache.v_pool + head + (size_t)(g.cache_dim >= 0 ? g.dst_off : 0) * kPageTokens + (pos % kPageTokens);
            step = kPageTokens;
        }
    }
    int d_pad = g.d_pad;
    if (g.lead > 0) {
        for (int e = lane; e < g.lead; e += 32) o[(size_t)e * step] = from_f32<T>(0.f);
        o += (size_t)g.lead * step;
        d_pad -= g.lead;
    }
    if (g.rotate) {
        const float pos = (float)cache.positions[t];
        for (int i = lane; 2 * i < d_pad; i += 32) {
            float z0 = 0.f, z1 = 0.f;
            if (2 * i + 1 < g.d) {
                const float u = (to_f32<T>(x[2 * i]) + (b ? b[2 * i] : 0.f)) * factor * (w ? w[2 * i] : 1.f);
                const float v = (to_f32<T>(x[2 * i + 1]) + (b ? b[2 * i + 1] : 0.f)) * factor * (w ? w[2 * i + 1] : 1.f);
                float sn, cs;
                sincosf(pos * cache.inv_freq[i], &sn, &cs);
                z0 = u * cs - v * sn;
                z1 = v * cs + u * sn;
            }
            o[(size_t)(2 * i) * step] = from_f32<T>(z0);
            if (2 * i + 1 < d_pad) o[(size_t)(2 * i + 1) * step] = from_f32<T>(z1);
        }
        return;
    }
    for (int e = lane; e < d_pad; e += 32) {
        float z = 0.f;
        if (e < g.d) {
            z = (to_f32<T>(x[e]) + (b ? b[e] : 0.f)) * factor;
            if (w) z *= w[e];
            if (other) z = (1.0f - lambda) * z + lambda * to_f32<T>(other[e]);
        }
        o[(size_t)e * step] = from_f32<T>(z);
    }
}

// A warp per (token, row); grid (tokens, rows / warps).
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
head_rows_kernel(const T* __restrict__ src, int ld_src, T* __restrict__ dst, int ld_dst, const float* __restrict__ bias,
                 const float* __restrict__ weight, RowSegments segs, float eps, CacheTarget cache, MixSource mix) {
    const int t = blockIdx.x, lane = threadIdx.x & 31;
    int row = blockIdx.y * (kRowThreads / 32) + (threadIdx.x >> 5);
    if (row >= segs.total_rows) return;
    int s = 0;
    while (s + 1 < segs.n && row >= segs.seg[s].n_rows) {
        row -= segs.seg[s].n_rows;
        ++s;
    }
    head_row<T>(src, ld_src, dst, ld_dst, bias, weight, segs.seg[s], t, row, lane, eps, 0.f, cache, mix);
}

// For launches in which some segment's norm runs over all its rows: a CTA sums such a segment once (its threads in a
// fixed order), then its warps take the token's rows in turn.
constexpr int kTokenThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kTokenThreads)
head_rows_token_kernel(const T* __restrict__ src, int ld_src, T* __restrict__ dst, int ld_dst, const float* __restrict__ bias,
                       const float* __restrict__ weight, RowSegments segs, float eps, CacheTarget cache, MixSource mix) {
    __shared__ float scratch[33];
    __shared__ float whole[kRowSegments];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int s = 0; s < segs.n; ++s) {
        const RowSegment& g = segs.seg[s];
        if (g.norm != 2) continue;
        const T* xs = src + (size_t)t * ld_src + g.src_off;
        const float* bs = g.bias_off >= 0 ? bias + g.bias_off : nullptr;
        const int n = g.n_rows * g.d;
        float ss = 0.f;
        for (int e = threadIdx.x; e < n; e += kTokenThreads) {
            const float z = to_f32<T>(xs[e]) + (bs ? bs[e] : 0.f);
            ss += z * z;
        }
        ss = block_sum(ss, scratch);
        if (threadIdx.x == 0) whole[s] = 1.0f / sqrtf(ss / (float)n + eps);
    }
    __syncthreads();
    // the token's rows, numbered through the segments, are shared out among the warps of the token's CTAs (gridDim.y of
    // them: a step of few tokens has several per token, each of which has summed for itself)
    const int n_warps = (int)gridDim.y * (kTokenThreads / 32);
    for (int flat = (int)blockIdx.y * (kTokenThreads / 32) + warp; flat < segs.total_rows; flat += n_warps) {
        int s = 0, row = flat;
        while (s + 1 < segs.n && row >= segs.seg[s].n_rows) {
            row -= segs.seg[s].n_rows;
            ++s;
        }
        head_row<T>(src, ld_src, dst, ld_dst, bias, weight, segs.seg[s], t, row, lane, eps, whole[s], cache, mix);
    }
}

}  // namespace b200

// `segments`: n_segments records of twenty 32-bit words each (src_off, n_rows, d, dst_off, d_pad, bias_off, norm,
// weight_off, mul as float bits, target, weight_per_row, mix_off, rotate, src_stride, dst_stride, cache_dim, lead; the rest
// unused), read on the host.  Segments with a cache target need positions, seq_ids,
// page_table and the pools; their n_rows is the number of kv heads of the cache entry and d_pad its head size.
extern "C" int b200_head_rows(const void* src, int ld_src, void* dst, int ld_dst, int dtype, const float* bias,
                              const float* weight, const int* segments, int n_segments, int n_tokens, float eps,
                              const int* positions, const int* seq_ids, const int* page_table, int table_stride,
                              void* k_pool, void* v_pool, const void* other, int ld_other, const float* lambda,
                              const float* inv_freq, cudaStream_t stream) {
    if (n_tokens <= 0 || n_segments <= 0) return 0;
    if (n_segments > b200::kRowSegments) return b200::kErrBadArgument;
    b200::RowSegments segs = {};
    segs.n = n_segments;
    for (int i = 0; i < n_segments; ++i) {
        const int* p = segments + b200::kSegmentWords * i;
        b200::RowSegment& g = segs.seg[i];
        g.src_off = p[0]; g.n_rows = p[1]; g.d = p[2]; g.dst_off = p[3]; g.d_pad = p[4];
        g.bias_off = p[5]; g.norm = p[6]; g.weight_off = p[7];
        union { int i; float f; } u;
        u.i = p[8];
        g.mul = u.f;
        g.target = p[9];
        g.weight_per_row = p[10];
        g.mix_off = p[11];
        g.rotate = p[12]; g.src_stride = p[13]; g.dst_stride = p[14]; g.cache_dim = p[15]; g.lead = p[16];
        if (g.lead < 0 || g.lead + g.d > g.d_pad) return b200::kErrBadArgument;
        if (g.rotate && (!inv_freq || !positions || g.d % 2 || g.mix_off >= 0)) return b200::kErrBadArgument;
        if (g.cache_dim >= 0 && (g.target == 0 || g.dst_off < 0 || g.dst_off + g.d_pad > g.cache_dim)) return b200::kErrBadArgument;
        if (g.norm < 0 || g.norm > 2) return b200::kErrBadArgument;
        if (g.mix_off >= 0 && (other == nullptr || lambda == nullptr)) return b200::kErrBadArgument;
        if (g.target < 0 || g.target > 2) return b200::kErrBadArgument;
        if (g.target != 0 && (!positions || !seq_ids || !page_table || (g.target == 1 ? !k_pool : !v_pool))) return b200::kErrBadArgument;
        if (g.target == 0 && dst == nullptr) return b200::kErrBadArgument;
        if (g.n_rows < 0 || g.d < 1 || g.d_pad < g.d) return b200::kErrBadArgument;
        if ((g.bias_off >= 0 && bias == nullptr) || (g.weight_off >= 0 && weight == nullptr)) return b200::kErrBadArgument;
        segs.total_rows += g.n_rows;
    }
    if (segs.total_rows == 0) return 0;
    const int per_cta = b200::kRowThreads / 32;
    dim3 grid(n_tokens, (segs.total_rows + per_cta - 1) / per_cta);
    if (grid.y > 65535) return b200::kErrUnsupportedSize;
    const b200::CacheTarget cache = {positions, seq_ids, page_table, table_stride, k_pool, v_pool, inv_freq};
    const b200::MixSource mix = {other, ld_other, lambda};
    bool per_token = false;
    for (int i = 0; i < n_segments; ++i) per_token = per_token || segs.seg[i].norm == 2;
    if (per_token) {
        const int per_cta_rows = b200::kTokenThreads / 32;
        const int ny = n_tokens >= 512 ? 1 : (segs.total_rows + per_cta_rows - 1) / per_cta_rows;
        const dim3 token_grid(n_tokens, ny > 16 ? 16 : ny);
        B200_DISPATCH_DTYPE(dtype, T,
            b200::head_rows_token_kernel<T><<<token_grid, b200::kTokenThreads, 0, stream>>>((const T*)src, ld_src, (T*)dst, ld_dst,
                                                                                          bias, weight, segs, eps, cache, mix));
        return b200::launch_status();
    }
    B200_DISPATCH_DTYPE(dtype, T,
        b200::head_rows_kernel<T><<<grid, b200::kRowThreads, 0, stream>>>((const T*)src, ld_src, (T*)dst, ld_dst, bias,
                                                                          weight, segs, eps, cache, mix));
    return b200::launch_status();
}
