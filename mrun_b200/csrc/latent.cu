// Kernels of the parts that a latent-attention decoder with sandwich norms and routed
// feed-forwards adds to the step: all of them memory-bound, 32-bit arithmetic, one rounding into
// the activation dtype.
//
//   latent_prepare    the down-projections' rows -> normed query latent, and the token's cache row
//                     [normed key/value latent | rotated shared key part | zeros]
//   latent_query      the rotated part of every query head into the attention's query rows
//   post_norm_add     stream += scale * rmsnorm(branch) * w_post, then rmsnorm(stream) * w_next
//   route_top_k       router logits -> a dense row of expert weights (zero where not chosen)
//   relu2_scaled      relu(u)^2 times the expert weight of the column's expert
//   soft_cap          cap * tanh(x / cap) in place
//   scale             x * factor in place
#include "common.cuh"

using namespace mrun;

namespace {

// Rotation of pair i of a vector whose first `dims` features rotate: interleaved pairing takes
// features (2i, 2i + 1), half-split pairing (i, i + dims / 2).
__device__ __forceinline__ void pair_features(int i, int dims, int interleaved, int& a, int& b) {
    if (interleaved) { a = 2 * i; b = 2 * i + 1; }
    else { a = i; b = i + dims / 2; }
}

// ------------------------------------------------------------------------------------------
// One block a token.  down[t] = [query latent (q_rank) | key/value latent (kv_rank) | shared key
// part (rot_dim)], the stacked down-projections' output.  The two latents are RMS-normed with
// their weights (eps inside the root); the shared key part is not normed, its first `rot_dims`
// features rotate by the token's table row.  The cache row of width `width` >= kv_rank + rot_dim
// is filled to its end with zeros, so that an attention kernel may take it as a key of that size.
// ------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const TA* __restrict__ down, long ld, const float* __restrict__ q_weight,
                      const float* __restrict__ kv_weight, float eps, const float2* __restrict__ rot,
                      int rot_dims, int interleaved, const int* __restrict__ slots, TA* __restrict__ cq,
                      TA* __restrict__ cache, int q_rank, int kv_rank, int rot_dim, int width) {
    __shared__ float scratch[33];
    const int t = blockIdx.x, tid = threadIdx.x;
    const TA* row = down + (size_t)t * ld;
    const TA* kv = row + q_rank;
    const int slot = slots ? slots[t] : -1;      // negative: a padding row, or a run that only reads another's cache
    // both totals of squares from one sweep over the row (measured on B200: a warp a token, and
    // prefetches of the norm weights during the sweep, were both slower than this)
    float ss_q = 0.f, ss_kv = 0.f;
    for (int i = tid; i < q_rank; i += blockDim.x) { const float v = to_float(row[i]); ss_q += v * v; }
    if (slot >= 0)
        for (int i = tid; i < kv_rank; i += blockDim.x) { const float v = to_float(kv[i]); ss_kv += v * v; }
    if (q_rank > 0) {
        ss_q = block_sum(ss_q, scratch);
        const float inv = rsqrtf(ss_q / (float)q_rank + eps);
        for (int i = tid; i < q_rank; i += blockDim.x)
            cq[(size_t)t * q_rank + i] = from_float<TA>(to_float(row[i]) * inv * q_weight[i]);
    }
    if (slot < 0) return;
    ss_kv = block_sum(ss_kv, scratch);
    const float inv = rsqrtf(ss_kv / (float)kv_rank + eps);
    TA* dst = cache + (size_t)slot * width;
    for (int i = tid; i < kv_rank; i += blockDim.x)
        dst[i] = from_float<TA>(to_float(kv[i]) * inv * kv_weight[i]);
    const TA* kr = kv + kv_rank;
    const int pairs = rot_dims / 2;
    for (int i = tid; i < pairs; i += blockDim.x) {
        int a, b;
        pair_features(i, rot_dims, interleaved, a, b);
        const float2 cs = rot[(size_t)t * pairs + i];
        const float u = to_float(kr[a]), v = to_float(kr[b]);
        dst[kv_rank + a] = from_float<TA>(u * cs.x - v * cs.y);
        dst[kv_rank + b] = from_float<TA>(v * cs.x + u * cs.y);
    }
    for (int i = rot_dims + tid; i < rot_dim; i += blockDim.x) dst[kv_rank + i] = kr[i];
    for (int i = kv_rank + rot_dim + tid; i < width; i += blockDim.x) dst[i] = from_float<TA>(0.f);
}

// ------------------------------------------------------------------------------------------
// q[t, h] = [plain part (dim) | rotated part (rot_dim)].  The attention's query row of head h is
// [plain part taken through the key up-projection (kv_rank, written by the product before) |
// rotated part | zeros]; this kernel fills everything after the first kv_rank features.
// ------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(256)
latent_query_kernel(const TA* __restrict__ q, long ldq, const float2* __restrict__ rot, int rot_dims, int interleaved,
                    TA* __restrict__ q_att, int heads, int dim, int rot_dim, int kv_rank, int width) {
    const int t = blockIdx.x;
    const int pairs = rot_dims / 2, tail = width - kv_rank;
    for (int item = threadIdx.x; item < heads * tail; item += blockDim.x) {
        const int h = item / tail, j = item - h * tail;
        const TA* src = q + (size_t)t * ldq + (size_t)h * (dim + rot_dim) + dim;
        TA* dst = q_att + ((size_t)t * heads + h) * width + kv_rank;
        if (j >= rot_dim) { dst[j] = from_float<TA>(0.f); continue; }
        if (j >= rot_dims) { dst[j] = src[j]; continue; }
        int i, other;
        float sign;
        if (interleaved) { i = j >> 1; other = j ^ 1; sign = (j & 1) ? 1.f : -1.f; }
        else if (j < pairs) { i = j; other = j + pairs; sign = -1.f; }
        else { i = j - pairs; other = j - pairs; sign = 1.f; }
        const float2 cs = rot[(size_t)t * pairs + i];
        dst[j] = from_float<TA>(to_float(src[j]) * cs.x + sign * to_float(src[other]) * cs.y);
    }
}

// ------------------------------------------------------------------------------------------
// The residual sum of a layer whose branch output is normed before it is added:
//   v = stream[src] + scale * branch[src] * rsqrt(mean(branch^2) + eps) * w_post
//   rows == null: stream[src] = v
//   out[r] = v * rsqrt(mean(v^2) + eps) * w_next          (left out when w_next is null)
// With `rows` the kernel reads row rows[r] and leaves the stream as it is.  The branch comes in
// 32-bit (the product before it writes 32-bit sums).  One block of 256 threads a row.
// ------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(256)
post_norm_add_kernel(float* __restrict__ stream, const float* __restrict__ branch,
                     const float* __restrict__ w_post, float scale, float eps_post,
                     const float* __restrict__ w_next, float eps_next, TA* __restrict__ out,
                     const int* __restrict__ rows, int hidden) {
    extern __shared__ float row_buf[];
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float ss = 0.f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float b = branch[src + h];
        row_buf[h] = b;
        ss += b * b;
    }
    ss = block_sum(ss, scratch);
    const float inv_b = rsqrtf(ss / (float)hidden + eps_post) * scale;
    float sv = 0.f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float v = stream[src + h] + row_buf[h] * inv_b * w_post[h];
        row_buf[h] = v;
        if (!rows) stream[src + h] = v;
        sv += v * v;
    }
    if (!w_next) return;
    sv = block_sum(sv, scratch);
    const float inv_v = rsqrtf(sv / (float)hidden + eps_next);
    TA* dst = out + (size_t)r * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x)
        dst[h] = from_float<TA>(row_buf[h] * inv_v * w_next[h]);
}

// The same for widths that are a multiple of 8 and at most 8192: a thread keeps up to four
// 8-value chunks of the stream and of the branch in registers, so a row is read once, with all its
// loads in flight together.  One block of 256 threads a row: the order of additions depends on
// the width only.
template <typename TA>
__global__ void __launch_bounds__(256)
post_norm_add_vec_kernel(float* __restrict__ stream, const float* __restrict__ branch,
                         const float* __restrict__ w_post, float scale, float eps_post,
                         const float* __restrict__ w_next, float eps_next, TA* __restrict__ out,
                         const int* __restrict__ rows, int hidden) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    const int chunks = hidden >> 3;
    float v[4][8], b[4][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            Vec8<float>::load(branch + src + c * 8, b[i]);
            Vec8<float>::load(stream + src + c * 8, v[i]);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += b[i][e] * b[i][e];
        }
    }
    ss = block_sum(ss, scratch);
    const float inv_b = rsqrtf(ss / (float)hidden + eps_post) * scale;
    float sv = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            float w[8];
            Vec8<float>::load(w_post + c * 8, w);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[i][e] += b[i][e] * inv_b * w[e];
                sv += v[i][e] * v[i][e];
            }
            if (!rows) Vec8<float>::store(stream + src + c * 8, v[i]);
        }
    }
    if (!w_next) return;
    sv = block_sum(sv, scratch);
    const float inv_v = rsqrtf(sv / (float)hidden + eps_next);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            float w[8], y[8];
            Vec8<float>::load(w_next + c * 8, w);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = v[i][e] * inv_v * w[e];
            Vec8<TA>::store(out + (size_t)r * hidden + c * 8, y);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Router: one warp a token.  score = softmax over all experts (kind 0), a sigmoid of each
// logit (kind 1) or the logit itself (kind 2); the `top` largest scores are chosen (the smaller
// index wins a tie); the output row holds the chosen experts' scores, divided by their sum if
// `renormalize`, and zero elsewhere; with kind 2 it holds the softmax over the chosen logits
// only.  `bias` (nullable, one entry an expert) is added to the logits first; a row of logits
// starts `ldz` entries after the one before.  `chosen` (nullable) gets the expert ids in the
// order they were picked.
// ------------------------------------------------------------------------------------------
constexpr int ROUTE_MAX_PER_LANE = 16;      // experts <= 512

// PER_LANE: experts a lane holds (experts <= 32 * PER_LANE)
template <int PER_LANE>
__global__ void __launch_bounds__(128)
route_top_k_kernel(const float* __restrict__ logits, long ldz, const float* __restrict__ bias,
                   float* __restrict__ weights, int* __restrict__ chosen, int tokens, int experts, int top, int kind,
                   int renormalize) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const float* z = logits + (size_t)t * ldz;
    float s[PER_LANE];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int e = lane + 32 * i;
        s[i] = e < experts ? z[e] + (bias ? bias[e] : 0.f) : -INFINITY;
        m = fmaxf(m, s[i]);
    }
    if (kind == 2) {
        // the logits themselves are the scores
    } else if (kind == 0) {
        m = warp_max(m);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int e = lane + 32 * i;
            s[i] = e < experts ? expf(s[i] - m) : 0.f;
            sum += s[i];
        }
        sum = warp_sum(sum);
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) s[i] = s[i] / sum;
    } else {
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int e = lane + 32 * i;
            s[i] = e < experts ? 1.f / (1.f + expf(-s[i])) : 0.f;
        }
    }
    float w[PER_LANE];
    unsigned taken = 0;
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) w[i] = 0.f;
    float first = 0.f;          // kind 2: the largest chosen logit, which the exponentials are taken against
    for (int k = 0; k < top; ++k) {
        float best = kind == 2 ? -INFINITY : -1.f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < experts && !(taken >> i & 1u) && (s[i] > best || (best_e == 0x7fffffff && s[i] == best))) {
                best = s[i]; best_e = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (kind == 2) {
            if (k == 0) first = best;
            best = expf(best - first);
        }
        if ((best_e & 31) == lane) {
            const int i = best_e >> 5;
#pragma unroll
            for (int j = 0; j < PER_LANE; ++j)
                if (j == i) { w[j] = best; taken |= 1u << j; }
        }
        total += best;
        if (chosen && lane == 0) chosen[(size_t)t * top + k] = best_e;
    }
    const float norm = (renormalize || kind == 2) ? 1.f / total : 1.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int e = lane + 32 * i;
        if (e < experts) weights[(size_t)t * experts + e] = w[i] * norm;
    }
}

// ------------------------------------------------------------------------------------------
// act[t, c] = relu(u[t, c])^2 * weight, where column c < experts * ff belongs to expert c / ff
// and takes weights[t, c / ff]; the columns after them (a shared expert) take 1.
// ------------------------------------------------------------------------------------------
template <typename TA>
__global__ void relu2_scaled_kernel(const TA* __restrict__ u, TA* __restrict__ act,
                                    const float* __restrict__ weights, long total, int columns, int experts,
                                    int ff) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long t = i / columns;
    const int c = (int)(i - t * columns);
    const float v = fmaxf(to_float(u[i]), 0.f);
    const int e = c / ff;
    const float w = (weights && e < experts) ? weights[t * experts + e] : 1.f;
    act[i] = from_float<TA>(v * v * w);
}

// Eight columns a thread, for column counts and expert sizes that are multiples of 8 (a chunk then
// lies inside one expert): grid.x walks the tokens, grid.y the chunks of a row.
template <typename TA>
__global__ void __launch_bounds__(256)
relu2_scaled_vec_kernel(const TA* __restrict__ u, TA* __restrict__ act, const float* __restrict__ weights,
                        int columns, int experts, int ff) {
    const long t = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= columns) return;
    const int e = c / ff;
    const float w = (weights && e < experts) ? weights[t * experts + e] : 1.f;
    float v[8];
    Vec8<TA>::load(u + t * columns + c, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float x = fmaxf(v[i], 0.f);
        v[i] = x * x * w;
    }
    Vec8<TA>::store(act + t * columns + c, v);
}

__global__ void soft_cap_kernel(float* __restrict__ x, long total, float cap) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] = cap * tanhf(x[i] / cap);
}

__global__ void scale_kernel(float* __restrict__ x, long total, float factor) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) x[i] *= factor;
}

}  // namespace

MRUN_API int mrun_latent_prepare(const void* down, int act_dtype, long ld, const float* q_weight,
                                 const float* kv_weight, float eps, const float* rot, int rot_dims,
                                 int interleaved, const int* slots, void* cq, void* cache, int tokens,
                                 int q_rank, int kv_rank, int rot_dim, int width, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && q_rank >= 0 && kv_rank > 0 && rot_dim >= 0 && width >= kv_rank + rot_dim,
                 "latent_prepare: bad sizes q_rank=%d kv_rank=%d rot_dim=%d width=%d", q_rank, kv_rank, rot_dim, width);
    MRUN_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot_dim,
                 "latent_prepare: %d rotating features of %d", rot_dims, rot_dim);
    MRUN_REQUIRE(ld >= q_rank + kv_rank + rot_dim, "latent_prepare: row stride %ld below the row's width", ld);
    MRUN_REQUIRE(rot_dims == 0 || rot != nullptr, "latent_prepare: no rotation table");
    if (tokens == 0) return 0;
    if (act_dtype == MRUN_F32)
        latent_prepare_kernel<float><<<tokens, 256, 0, stream>>>(
            (const float*)down, ld, q_weight, kv_weight, eps, (const float2*)rot, rot_dims, interleaved, slots,
            (float*)cq, (float*)cache, q_rank, kv_rank, rot_dim, width);
    else if (act_dtype == MRUN_BF16)
        latent_prepare_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(
            (const __nv_bfloat16*)down, ld, q_weight, kv_weight, eps, (const float2*)rot, rot_dims, interleaved,
            slots, (__nv_bfloat16*)cq, (__nv_bfloat16*)cache, q_rank, kv_rank, rot_dim, width);
    else
        return mrun_set_error("latent_prepare: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("latent_prepare");
    return 0;
}

MRUN_API int mrun_latent_query(const void* q, long ldq, int act_dtype, const float* rot, int rot_dims, int interleaved,
                               void* q_att, int tokens, int heads, int dim, int rot_dim, int kv_rank, int width,
                               cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && heads > 0 && dim >= 0 && rot_dim >= 0 && kv_rank > 0 && width >= kv_rank + rot_dim,
                 "latent_query: bad sizes heads=%d dim=%d rot_dim=%d kv_rank=%d width=%d", heads, dim, rot_dim,
                 kv_rank, width);
    MRUN_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot_dim,
                 "latent_query: %d rotating features of %d", rot_dims, rot_dim);
    MRUN_REQUIRE(rot_dims == 0 || rot != nullptr, "latent_query: no rotation table");
    MRUN_REQUIRE(ldq >= (long)heads * (dim + rot_dim), "latent_query: rows of %ld entries do not hold the heads", ldq);
    if (tokens == 0 || width == kv_rank) return 0;
    if (act_dtype == MRUN_F32)
        latent_query_kernel<float><<<tokens, 256, 0, stream>>>((const float*)q, ldq, (const float2*)rot, rot_dims,
                                                               interleaved, (float*)q_att, heads, dim, rot_dim,
                                                               kv_rank, width);
    else if (act_dtype == MRUN_BF16)
        latent_query_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(
            (const __nv_bfloat16*)q, ldq, (const float2*)rot, rot_dims, interleaved, (__nv_bfloat16*)q_att, heads, dim,
            rot_dim, kv_rank, width);
    else
        return mrun_set_error("latent_query: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("latent_query");
    return 0;
}

MRUN_API int mrun_post_norm_add(float* stream_rows, const float* branch, const float* w_post, float scale,
                                float eps_post, const float* w_next, float eps_next, void* out, int act_dtype,
                                const int* rows, int n_rows, int hidden, cudaStream_t stream) {
    MRUN_REQUIRE(n_rows >= 0 && hidden > 0, "post_norm_add: bad sizes rows=%d hidden=%d", n_rows, hidden);
    MRUN_REQUIRE(hidden <= 12 * 1024, "post_norm_add: hidden=%d exceeds the supported 12288", hidden);
    MRUN_REQUIRE(w_next == nullptr || out != nullptr, "post_norm_add: a next norm needs an output");
    if (n_rows == 0) return 0;
    const bool aligned = (((uintptr_t)stream_rows | (uintptr_t)branch | (uintptr_t)w_post | (uintptr_t)w_next |
                           (uintptr_t)out) & 15) == 0;
    if (hidden % 8 == 0 && hidden <= 8192 && aligned && (act_dtype == MRUN_F32 || act_dtype == MRUN_BF16)) {
        if (act_dtype == MRUN_F32)
            post_norm_add_vec_kernel<float><<<n_rows, 256, 0, stream>>>(stream_rows, branch, w_post, scale, eps_post,
                                                                        w_next, eps_next, (float*)out, rows, hidden);
        else
            post_norm_add_vec_kernel<__nv_bfloat16><<<n_rows, 256, 0, stream>>>(
                stream_rows, branch, w_post, scale, eps_post, w_next, eps_next, (__nv_bfloat16*)out, rows, hidden);
        MRUN_CHECK_LAUNCH("post_norm_add");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (act_dtype == MRUN_F32)
        post_norm_add_kernel<float><<<n_rows, 256, smem, stream>>>(stream_rows, branch, w_post, scale, eps_post,
                                                                   w_next, eps_next, (float*)out, rows, hidden);
    else if (act_dtype == MRUN_BF16)
        post_norm_add_kernel<__nv_bfloat16><<<n_rows, 256, smem, stream>>>(
            stream_rows, branch, w_post, scale, eps_post, w_next, eps_next, (__nv_bfloat16*)out, rows, hidden);
    else
        return mrun_set_error("post_norm_add: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("post_norm_add");
    return 0;
}

MRUN_API int mrun_route_top_k(const float* logits, long ldz, const float* bias, float* weights, int* chosen, int tokens,
                              int experts, int top, int kind, int renormalize, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && top <= experts,
                 "route_top_k: bad sizes tokens=%d experts=%d top=%d", tokens, experts, top);
    MRUN_REQUIRE(experts <= 32 * ROUTE_MAX_PER_LANE, "route_top_k: %d experts exceed the supported %d", experts,
                 32 * ROUTE_MAX_PER_LANE);
    MRUN_REQUIRE(kind >= 0 && kind <= 2, "route_top_k: unknown score function %d", kind);
    MRUN_REQUIRE(ldz >= experts, "route_top_k: rows of %ld entries do not hold %d experts", ldz, experts);
    if (tokens == 0) return 0;
    const dim3 grid((tokens + 3) / 4);
    if (experts <= 32)
        route_top_k_kernel<1><<<grid, 128, 0, stream>>>(logits, ldz, bias, weights, chosen, tokens, experts, top, kind, renormalize);
    else if (experts <= 128)
        route_top_k_kernel<4><<<grid, 128, 0, stream>>>(logits, ldz, bias, weights, chosen, tokens, experts, top, kind, renormalize);
    else
        route_top_k_kernel<ROUTE_MAX_PER_LANE><<<grid, 128, 0, stream>>>(logits, ldz, bias, weights, chosen, tokens,
                                                                        experts, top, kind, renormalize);
    MRUN_CHECK_LAUNCH("route_top_k");
    return 0;
}

MRUN_API int mrun_relu2_scaled(const void* u, void* act, int act_dtype, const float* weights, int tokens,
                               int columns, int experts, int ff, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && columns > 0 && experts >= 0 && ff > 0 && (long)experts * ff <= columns,
                 "relu2_scaled: bad sizes columns=%d experts=%d ff=%d", columns, experts, ff);
    const long total = (long)tokens * columns;
    if (total == 0) return 0;
    const bool aligned = (((uintptr_t)u | (uintptr_t)act) & 15) == 0;
    const int chunk_blocks = (columns / 8 + 255) / 256;
    if (columns % 8 == 0 && ff % 8 == 0 && aligned && chunk_blocks <= 65535 &&
        (act_dtype == MRUN_F32 || act_dtype == MRUN_BF16)) {
        const dim3 grid(tokens, chunk_blocks);
        if (act_dtype == MRUN_F32)
            relu2_scaled_vec_kernel<float><<<grid, 256, 0, stream>>>((const float*)u, (float*)act, weights, columns,
                                                                     experts, ff);
        else
            relu2_scaled_vec_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
                (const __nv_bfloat16*)u, (__nv_bfloat16*)act, weights, columns, experts, ff);
        MRUN_CHECK_LAUNCH("relu2_scaled");
        return 0;
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (act_dtype == MRUN_F32)
        relu2_scaled_kernel<float><<<blocks, 256, 0, stream>>>((const float*)u, (float*)act, weights, total, columns,
                                                              experts, ff);
    else if (act_dtype == MRUN_BF16)
        relu2_scaled_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
            (const __nv_bfloat16*)u, (__nv_bfloat16*)act, weights, total, columns, experts, ff);
    else
        return mrun_set_error("relu2_scaled: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("relu2_scaled");
    return 0;
}

MRUN_API int mrun_scale_f32(float* x, long total, float factor, cudaStream_t stream) {
    MRUN_REQUIRE(total >= 0, "scale: bad size %ld", total);
    if (total == 0) return 0;
    scale_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(x, total, factor);
    MRUN_CHECK_LAUNCH("scale");
    return 0;
}

MRUN_API int mrun_soft_cap(float* x, long total, float cap, cudaStream_t stream) {
    MRUN_REQUIRE(total >= 0 && cap > 0.f, "soft_cap: bad sizes or a cap that is not positive");
    if (total == 0) return 0;
    soft_cap_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(x, total, cap);
    MRUN_CHECK_LAUNCH("soft_cap");
    return 0;
}
