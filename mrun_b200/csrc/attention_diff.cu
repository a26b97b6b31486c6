// Differential attention over the paged cache: every query head runs two softmax attentions
// ("maps") with keys of their own over the same values and combines them,
//
//     o = a1 - lambda * a2,   o <- o / sqrt(mean(o^2) + eps) * out_scale      (per head)
//
// Layouts.  A token's projected row is [q | k | v] with q = [map][head][D], k = [map][kv head][D]
// and v = [kv head][V].  The key pages are [map][pages][kv heads][page_size][D], so each map is a
// page tensor of the ordinary grouped-query shape; the value pages are [chunk][pages][kv heads]
// [page_size][Dv] with chunks * Dv = V (one chunk of V features, or V cut into chunks of D so
// that a map and a chunk can go through the kernels for equal key and value sizes).
//
// Kernels:
//   diff_rope_cache   rotates the first rot_dims features of every q and k vector (half-split
//                     pairing, table of (cos, sin) per token and pair), q in place, k and v into
//                     the pages
//   diff_attention    both maps, the combination and the head norm in one pass on CUDA cores in
//                     32-bit arithmetic, for any sizes: one block a (token, head), keys in tiles
//                     of 128 in position order
//   diff_combine      the combination and the head norm for map outputs that other attention
//                     kernels made
#include "common.cuh"

using namespace mrun;

namespace {

constexpr int THREADS = 128;

template <typename TA>
__global__ void __launch_bounds__(THREADS)
diff_rope_cache_kernel(TA* __restrict__ qkv, long ld, const float2* __restrict__ rot, int rot_dims,
                       const int* __restrict__ slots, TA* __restrict__ k_cache, TA* __restrict__ v_cache,
                       long pages, int H, int G, int D, int V, int Dv, int page_size) {
    const int t = blockIdx.x, tid = threadIdx.x;
    TA* row = qkv + (size_t)t * ld;
    const int half = rot_dims / 2;
    const int slot = slots ? slots[t] : -1;
    const int vectors = 2 * H + 2 * G;
    const float2* table = rot + (size_t)t * half;
    // the rotating pairs of every q and k vector
    for (int e = tid; e < vectors * half; e += THREADS) {
        const int vec = e / half, i = e - vec * half;
        TA* x = row + (size_t)vec * D;
        const float2 cs = table[i];
        const float u = to_float(x[i]), w = to_float(x[i + half]);
        x[i] = from_float<TA>(u * cs.x - w * cs.y);
        x[i + half] = from_float<TA>(w * cs.x + u * cs.y);
    }
    if (slot < 0) return;
    __syncthreads();
    const int page = slot / page_size, off = slot % page_size;
    const TA* k = row + (size_t)2 * H * D;
    for (int e = tid; e < 2 * G * D; e += THREADS) {
        const int vec = e / D, d = e - vec * D;
        const int m = vec / G, g = vec - m * G;
        k_cache[((((size_t)m * pages + page) * G + g) * page_size + off) * D + d] = k[e];
    }
    const TA* v = k + (size_t)2 * G * D;
    for (int e = tid; e < G * V; e += THREADS) {
        const int g = e / V, d = e - g * V;
        const int c = d / Dv, dd = d - c * Dv;
        v_cache[((((size_t)c * pages + page) * G + g) * page_size + off) * Dv + dd] = v[e];
    }
}

template <typename TA>
__global__ void __launch_bounds__(THREADS)
diff_attention_kernel(const TA* __restrict__ q, long q_stride, TA* __restrict__ out, const TA* __restrict__ k_cache,
                      const TA* __restrict__ v_cache, const int* __restrict__ block_tables, int max_blocks,
                      const int* __restrict__ token_slot, const int* __restrict__ positions, long pages, int H,
                      int G, int D, int V, int Dv, int page_size, float scale, float lambda, float eps,
                      float out_scale, int window) {
    extern __shared__ float smem[];
    float* q1 = smem;                      // D
    float* q2 = q1 + D;                    // D
    float* p1 = q2 + D;                    // THREADS
    float* p2 = p1 + THREADS;              // THREADS
    int* rows = (int*)(p2 + THREADS);      // THREADS: (page * G + kv head) * page_size + offset of each key
    __shared__ float scratch[33];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t];
    TA* dst = out + ((size_t)t * H + h) * V;
    if (pos < 0) {  // padding token
        for (int d = tid; d < V; d += THREADS) dst[d] = from_float<TA>(0.f);
        return;
    }
    const int g = h / (H / G);
    const int* table = block_tables + (size_t)token_slot[t] * max_blocks;
    const TA* qrow = q + (size_t)t * q_stride;
    for (int d = tid; d < D; d += THREADS) {
        q1[d] = to_float(qrow[(size_t)h * D + d]);
        q2[d] = to_float(qrow[((size_t)H + h) * D + d]);
    }
    __syncthreads();
    const size_t map_stride = (size_t)pages * G * page_size * D;
    const size_t chunk_stride = (size_t)pages * G * page_size * Dv;

    const int lo = first_visible(pos, window);
    float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
    float acc1[8], acc2[8];  // V <= 8 * THREADS
#pragma unroll
    for (int i = 0; i < 8; ++i) acc1[i] = acc2[i] = 0.f;

    for (int tile0 = lo; tile0 <= pos; tile0 += THREADS) {
        const int key = tile0 + tid;
        const bool valid = key <= pos;
        float s1 = -INFINITY, s2 = -INFINITY;
        if (valid) {
            const int page = table[key / page_size];
            const long row = ((long)page * G + g) * page_size + key % page_size;
            rows[tid] = (int)row;
            const TA* k1 = k_cache + row * D;
            const TA* k2 = k1 + map_stride;
            float d1 = 0.f, d2 = 0.f;
            for (int d = 0; d < D; ++d) {
                d1 = fmaf(q1[d], to_float(k1[d]), d1);
                d2 = fmaf(q2[d], to_float(k2[d]), d2);
            }
            s1 = d1 * scale;
            s2 = d2 * scale;
        }
        const float n1 = fmaxf(m1, block_max(s1, scratch));
        const float n2 = fmaxf(m2, block_max(s2, scratch));
        const float e1 = valid ? expf(s1 - n1) : 0.f, e2 = valid ? expf(s2 - n2) : 0.f;
        p1[tid] = e1;
        p2[tid] = e2;
        const float sum1 = block_sum(e1, scratch);      // has a __syncthreads after the stores above
        const float sum2 = block_sum(e2, scratch);
        const float c1 = (m1 == -INFINITY) ? 0.f : expf(m1 - n1);
        const float c2 = (m2 == -INFINITY) ? 0.f : expf(m2 - n2);
        l1 = l1 * c1 + sum1; m1 = n1;
        l2 = l2 * c2 + sum2; m2 = n2;
        const int n = min(THREADS, pos - tile0 + 1);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = tid + i * THREADS;
            if (d < V) {
                const int c = d / Dv;
                const TA* vcol = v_cache + (size_t)c * chunk_stride + (d - c * Dv);
                float a1 = acc1[i] * c1, a2 = acc2[i] * c2;
                for (int j = 0; j < n; ++j) {
                    const float vv = to_float(vcol[(long)rows[j] * Dv]);
                    a1 = fmaf(p1[j], vv, a1);
                    a2 = fmaf(p2[j], vv, a2);
                }
                acc1[i] = a1; acc2[i] = a2;
            }
        }
        __syncthreads();
    }
    const float i1 = 1.f / l1, i2 = 1.f / l2;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = tid + i * THREADS;
        if (d < V) {
            acc1[i] = acc1[i] * i1 - lambda * (acc2[i] * i2);
            ss = fmaf(acc1[i], acc1[i], ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = out_scale / sqrtf(ss / (float)V + eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = tid + i * THREADS;
        if (d < V) dst[d] = from_float<TA>(acc1[i] * inv);
    }
}

// maps: [map][chunk][tokens][H * Dv] as the other kernels wrote them; a warp a (token, head).
template <typename TA>
__global__ void __launch_bounds__(THREADS)
diff_combine_kernel(const TA* __restrict__ maps, TA* __restrict__ out, long pairs, long tokens, int H, int V, int Dv,
                    float lambda, float eps, float out_scale) {
    const long pair = (long)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (pair >= pairs) return;
    const long t = pair / H;
    const int h = (int)(pair - t * H);
    const int chunks = V / Dv;
    const size_t chunk_stride = (size_t)tokens * H * Dv, map_stride = chunk_stride * chunks;
    float ss = 0.f;
    for (int d = lane; d < V; d += 32) {
        const int c = d / Dv;
        const size_t at = (size_t)c * chunk_stride + ((size_t)t * H + h) * Dv + (d - c * Dv);
        const float o = to_float(maps[at]) - lambda * to_float(maps[map_stride + at]);
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)V + eps);
    for (int d = lane; d < V; d += 32) {
        const int c = d / Dv;
        const size_t at = (size_t)c * chunk_stride + ((size_t)t * H + h) * Dv + (d - c * Dv);
        const float o = to_float(maps[at]) - lambda * to_float(maps[map_stride + at]);
        out[((size_t)t * H + h) * V + d] = from_float<TA>(o * inv);
    }
}

}  // namespace

// qkv: row t at qkv + t * ld = [2 * H * D | 2 * G * D | G * V].  rot: float32 [tokens, rot_dims / 2, 2].
// slots: page * page_size + offset of each token's place in the pages, negative = none.
MRUN_API int mrun_diff_rope_cache(void* qkv, long ld, int act_dtype, const float* rot, int rot_dims, const int* slots,
                                  void* k_cache, void* v_cache, long pages, int tokens, int H, int G, int D, int V,
                                  int Dv, int page_size, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && H > 0 && G > 0 && D > 0 && V > 0 && Dv > 0 && V % Dv == 0 && page_size > 0,
                 "diff_rope_cache: bad sizes");
    MRUN_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= D, "diff_rope_cache: %d rotating features of %d",
                 rot_dims, D);
    MRUN_REQUIRE(rot_dims == 0 || rot != nullptr, "diff_rope_cache: no rotation table");
    MRUN_REQUIRE(ld >= (long)2 * H * D + 2 * G * D + G * V, "diff_rope_cache: row stride %ld below the row", ld);
    if (tokens == 0) return 0;
    if (act_dtype == MRUN_F32)
        diff_rope_cache_kernel<float><<<tokens, THREADS, 0, stream>>>((float*)qkv, ld, (const float2*)rot, rot_dims,
                                                                       slots, (float*)k_cache, (float*)v_cache, pages,
                                                                       H, G, D, V, Dv, page_size);
    else if (act_dtype == MRUN_BF16)
        diff_rope_cache_kernel<__nv_bfloat16><<<tokens, THREADS, 0, stream>>>(
            (__nv_bfloat16*)qkv, ld, (const float2*)rot, rot_dims, slots, (__nv_bfloat16*)k_cache,
            (__nv_bfloat16*)v_cache, pages, H, G, D, V, Dv, page_size);
    else
        return mrun_set_error("diff_rope_cache: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("diff_rope_cache");
    return 0;
}

MRUN_API int mrun_diff_attention(const void* q, long q_stride, void* out, const void* k_cache, const void* v_cache,
                                 int act_dtype, const int* block_tables, int max_blocks, const int* token_slot,
                                 const int* positions, long pages, int tokens, int H, int G, int D, int V, int Dv,
                                 int page_size, float scale, float lambda, float eps, float out_scale, int window,
                                 cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && H > 0 && G > 0 && D > 0 && V > 0 && Dv > 0 && V % Dv == 0 && page_size > 0 &&
                 max_blocks > 0, "diff_attention: bad sizes");
    MRUN_REQUIRE(H % G == 0, "diff_attention: heads=%d is not a multiple of kv_heads=%d", H, G);
    MRUN_REQUIRE(V <= 8 * THREADS, "diff_attention: value size %d exceeds the supported %d", V, 8 * THREADS);
    MRUN_REQUIRE(D <= 4096, "diff_attention: key size %d exceeds the supported 4096", D);
    MRUN_REQUIRE(H <= 65535, "diff_attention: heads=%d exceeds 65535", H);
    MRUN_REQUIRE(pages * G * page_size < (1L << 31), "diff_attention: the cache has too many rows");
    MRUN_REQUIRE(window >= 0, "diff_attention: window=%d is negative (this attention has no chunked form)", window);
    if (tokens == 0) return 0;
    const dim3 grid(tokens, H);
    const size_t smem = (size_t)(2 * D + 3 * THREADS) * sizeof(float);
    if (act_dtype == MRUN_F32)
        diff_attention_kernel<float><<<grid, THREADS, smem, stream>>>(
            (const float*)q, q_stride, (float*)out, (const float*)k_cache, (const float*)v_cache, block_tables,
            max_blocks, token_slot, positions, pages, H, G, D, V, Dv, page_size, scale, lambda, eps, out_scale, window);
    else if (act_dtype == MRUN_BF16)
        diff_attention_kernel<__nv_bfloat16><<<grid, THREADS, smem, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
            (const __nv_bfloat16*)v_cache, block_tables, max_blocks, token_slot, positions, pages, H, G, D, V, Dv,
            page_size, scale, lambda, eps, out_scale, window);
    else
        return mrun_set_error("diff_attention: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("diff_attention");
    return 0;
}

MRUN_API int mrun_diff_combine(const void* maps, void* out, int act_dtype, int tokens, int H, int V, int Dv,
                               float lambda, float eps, float out_scale, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && H > 0 && V > 0 && Dv > 0 && V % Dv == 0, "diff_combine: bad sizes");
    if (tokens == 0) return 0;
    const long pairs = (long)tokens * H;
    const unsigned blocks = (unsigned)((pairs + THREADS / 32 - 1) / (THREADS / 32));
    if (act_dtype == MRUN_F32)
        diff_combine_kernel<float><<<blocks, THREADS, 0, stream>>>((const float*)maps, (float*)out, pairs, tokens, H, V,
                                                                    Dv, lambda, eps, out_scale);
    else if (act_dtype == MRUN_BF16)
        diff_combine_kernel<__nv_bfloat16><<<blocks, THREADS, 0, stream>>>(
            (const __nv_bfloat16*)maps, (__nv_bfloat16*)out, pairs, tokens, H, V, Dv, lambda, eps, out_scale);
    else
        return mrun_set_error("diff_combine: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("diff_combine");
    return 0;
}
