// A routed feed-forward's prompt steps: the (token, chosen expert) pairs sorted by expert, so that
// every expert's rows lie together and a grouped product runs each expert on its own rows only.
//
//   moe_count     how many pairs each expert has
//   moe_place     the experts' row ranges (running totals), and for every pair its row: the row's
//                 source token and weight, and where each token finds its pairs' rows again
//   gather_rows   x_sorted[row] = x[source token of row]
//   relu2_rows    relu(u)^2 times the row's weight
//   combine_rows  out[t] = base[t] + the rows of token t's pairs, added in the order they were chosen
//
// And two kernels for experts that are chosen by a table instead of a router and have a gate:
//
//   table_route   a token's experts are row token_id of an integer table [vocab, top]; each
//                 weighs 1 / top (the dense weight row and the chosen list, as route_top_k gives them)
//   clamped_glu   a block of columns [gate (ff) | up (ff)] per expert: g = min(gate, limit),
//                 u = clamp(up, -limit, limit), y = g * sigmoid(alpha * g) * (u + 1), times the
//                 token's weight of the block's expert or the row's weight
//
// And the choice of a router with sigmoid scores and groups of experts:
//
//   route_grouped the experts form equal groups of neighbours; a group's score is the sum of its
//                 group_top largest scores; only experts of the keep best groups can be chosen;
//                 the top allowed experts with the largest scores weigh score / (sum + 1e-20) *
//                 scale; one more logit column, if there is one, becomes the sigmoid weight of a
//                 shared expert
//
// Inside an expert's range the rows stand in the order in which the pairs arrived (an atomic
// counter); a row's result does not depend on where in the range it stands, and the combine adds
// a token's rows in a fixed order, so the output has the same bits every run.
#include "common.cuh"

using namespace mrun;

namespace {

__global__ void moe_count_kernel(const int* __restrict__ chosen, int pairs, int experts, int* __restrict__ counts) {
    extern __shared__ int local[];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) local[e] = 0;
    __syncthreads();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += gridDim.x * blockDim.x) {
        const int e = chosen[i];
        if (e >= 0 && e < experts) atomicAdd(local + e, 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        if (local[e]) atomicAdd(counts + e, local[e]);
}

// One block.  ends[e] = pairs of experts 0..e; cursor[e] = where expert e's range starts.
__global__ void moe_scan_kernel(const int* __restrict__ counts, int experts, int* __restrict__ ends,
                                int* __restrict__ cursor) {
    if (threadIdx.x == 0) {
        int total = 0;
        for (int e = 0; e < experts; ++e) {
            cursor[e] = total;
            total += counts[e];
            ends[e] = total;
        }
    }
}

__global__ void moe_place_kernel(const int* __restrict__ chosen, const float* __restrict__ weights, int pairs,
                                 int experts, int top, int* __restrict__ cursor, int* __restrict__ source,
                                 float* __restrict__ row_weight, int* __restrict__ dest) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pairs) return;
    const int e = chosen[i], t = i / top;
    const int row = atomicAdd(cursor + e, 1);
    source[row] = t;
    row_weight[row] = weights[(size_t)t * experts + e];
    dest[i] = row;
}

template <typename TA>
__global__ void gather_rows_kernel(const TA* __restrict__ x, const int* __restrict__ source, TA* __restrict__ out,
                                   int width) {
    const size_t row = blockIdx.x;
    const TA* src = x + (size_t)source[row] * width;
    TA* dst = out + row * width;
    if ((width & 7) == 0 && ((((uintptr_t)x) | ((uintptr_t)out)) & 15) == 0 && sizeof(TA) == 2) {
        for (int c = threadIdx.x; c < width / 8; c += blockDim.x)
            reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
    }
}

// VEC: eight values a thread and step (the width a multiple of 8, the pointers on 16 bytes).
template <typename TA, bool VEC>
__global__ void relu2_rows_kernel(const TA* __restrict__ u, TA* __restrict__ act, const float* __restrict__ row_weight,
                                  int width) {
    const size_t row = blockIdx.x;
    const float w = row_weight[row];
    if constexpr (VEC) {
        for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
            float v[8];
            Vec8<TA>::load(u + row * width + c, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float x = fmaxf(v[i], 0.f);
                v[i] = x * x * w;
            }
            Vec8<TA>::store(act + row * width + c, v);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            const float v = fmaxf(to_float(u[row * width + c]), 0.f);
            act[row * width + c] = from_float<TA>(v * v * w);
        }
    }
}

template <typename TA, typename TB, bool VEC>
__global__ void combine_rows_kernel(const TB* __restrict__ base, const TA* __restrict__ rows,
                                    const int* __restrict__ dest, float* __restrict__ out, int top, int width) {
    const size_t t = blockIdx.x;
    if constexpr (VEC) {
        for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
            float s[8];
            if (base) Vec8<TB>::load(base + t * width + c, s);
            else
#pragma unroll
                for (int i = 0; i < 8; ++i) s[i] = 0.f;
            for (int k = 0; k < top; ++k) {
                float r[8];
                Vec8<TA>::load(rows + (size_t)dest[t * top + k] * width + c, r);
#pragma unroll
                for (int i = 0; i < 8; ++i) s[i] += r[i];
            }
            Vec8<float>::store(out + t * width + c, s);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            float s = base ? to_float(base[t * width + c]) : 0.f;
            for (int k = 0; k < top; ++k) s += to_float(rows[(size_t)dest[t * top + k] * width + c]);
            out[t * width + c] = s;
        }
    }
}

// A warp a token.
__global__ void table_route_kernel(const int* __restrict__ ids, const int* __restrict__ table, float* __restrict__ weights,
                                   int* __restrict__ chosen, int tokens, int vocab, int experts, int top) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    for (int e = lane; e < experts; e += 32) weights[(size_t)t * experts + e] = 0.f;
    __syncwarp();
    const float share = 1.f / (float)top;
    for (int j = lane; j < top; j += 32) {
        const int e = ok ? table[(size_t)id * top + j] : -1;
        if (chosen) chosen[(size_t)t * top + j] = (e >= 0 && e < experts) ? e : 0;
        if (e >= 0 && e < experts) weights[(size_t)t * experts + e] = share;
    }
}

// A warp a token.  logits: row t at logits + t * ldz, experts columns and then `extra` (0 or 1)
// more.  weights: dense [tokens, experts]; shared_w: [tokens] or null; chosen: [tokens, top] or
// null.  Ties go to the lower index.  Shared memory: experts + groups floats a warp.
__global__ void __launch_bounds__(128)
route_grouped_kernel(const float* __restrict__ logits, long ldz, float* __restrict__ weights,
                     float* __restrict__ shared_w, int* __restrict__ chosen, int tokens, int experts, int top,
                     int groups, int keep, int group_top, float scale) {
    extern __shared__ float route_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= tokens) return;
    float* s = route_smem + (size_t)warp * (experts + groups);
    float* gs = s + experts;
    const float* z = logits + (size_t)t * ldz;
    for (int e = lane; e < experts; e += 32) {
        s[e] = 1.f / (1.f + expf(-z[e]));
        weights[(size_t)t * experts + e] = 0.f;
    }
    if (shared_w && lane == 0) shared_w[t] = 1.f / (1.f + expf(-z[experts]));
    __syncwarp();
    const int size = experts / groups;
    if (groups > 1) {
        // a group's score: its group_top largest scores, found one after the other in the order
        // (larger score, then lower index)
        for (int g = lane; g < groups; g += 32) {
            float sum = 0.f, last = INFINITY;
            int last_i = -1;
            for (int k = 0; k < group_top && k < size; ++k) {
                float best = -1.f;
                int best_i = size;
                for (int i = 0; i < size; ++i) {
                    const float v = s[g * size + i];
                    const bool after = v < last || (v == last && i > last_i);
                    if (after && (v > best || (v == best && i < best_i))) { best = v; best_i = i; }
                }
                sum += best; last = best; last_i = best_i;
            }
            gs[g] = sum;
        }
        __syncwarp();
        // the keep best groups stay; the scores of the others leave the choice
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int best_g = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (gs[g] > best || (gs[g] == best && g < best_g)) { best = gs[g]; best_g = g; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
                if (ob > best || (ob == best && og < best_g)) { best = ob; best_g = og; }
            }
            __syncwarp();
            if (lane == 0) gs[best_g] = -INFINITY;      // marks a group that stays
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32)
            if (gs[e / size] != -INFINITY) s[e] = -1.f;
        __syncwarp();
    }
    float total = 0.f, mine = 0.f;       // lane k keeps the score of the k-th choice
    int mine_e = -1;
    for (int k = 0; k < top; ++k) {
        float best = -1.f;
        int best_e = 0x7fffffff;
        for (int e = lane; e < experts; e += 32)
            if (s[e] > best || (s[e] == best && e < best_e)) { best = s[e]; best_e = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        __syncwarp();
        if (lane == 0) s[best_e] = -2.f;
        __syncwarp();
        total += best;
        if (chosen && lane == 0) chosen[(size_t)t * top + k] = best_e;
        if (k == lane) { mine = best; mine_e = best_e; }
    }
    // the weights need the total of all choices: lane k kept the k-th choice (chosen experts
    // stand as -2 in s)
    const float norm = scale / (total + 1e-20f);
    if (top <= 32) {
        if (lane < top) weights[(size_t)t * experts + mine_e] = mine * norm;
    } else {
        // more than 32 choices: recompute every chosen expert's score from its logit
        for (int e = lane; e < experts; e += 32)
            if (s[e] == -2.f) weights[(size_t)t * experts + e] = (1.f / (1.f + expf(-z[e]))) * norm;
    }
}

// u: row r at u + r * ldu, blocks * 2 * ff columns; act: row r at act + r * lda, blocks * ff
// columns.  weights: per (row, block) when per_block (row r at weights + r * ldw), else one per row
// (at weights + r * ldw), or null.
template <typename TA, bool EXACT>
__global__ void clamped_glu_kernel(const TA* __restrict__ u, long ldu, TA* __restrict__ act, long lda,
                                   const float* __restrict__ weights, long ldw, int per_block, long total, int blocks,
                                   int ff, float limit, float alpha, float up_offset, const float* __restrict__ bias) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long row = i / ((long)blocks * ff);
    const int c = (int)(i - row * blocks * ff);
    const int e = c / ff, j = c - e * ff;
    const TA* base = u + row * ldu + (size_t)e * 2 * ff;
    const float* b = bias ? bias + (size_t)e * 2 * ff : nullptr;
    const float g = fminf(to_float(base[j]) + (b ? b[j] : 0.f), limit);
    const float up = fminf(fmaxf(to_float(base[ff + j]) + (b ? b[ff + j] : 0.f), -limit), limit);
    const float w = weights ? (per_block ? weights[row * ldw + e] : weights[row * ldw]) : 1.f;
    float s;
    if constexpr (EXACT) s = 1.f / (1.f + expf(-alpha * g));
    else s = __fdividef(1.f, 1.f + __expf(-alpha * g));
    act[row * lda + c] = from_float<TA>(g * s * (up + up_offset) * w);
}

// Eight outputs a thread (ff a multiple of 8, 16-byte aligned rows): grid.x walks the rows, grid.y the chunks.
template <typename TA, bool EXACT>
__global__ void __launch_bounds__(256)
clamped_glu_vec_kernel(const TA* __restrict__ u, long ldu, TA* __restrict__ act, long lda,
                       const float* __restrict__ weights, long ldw, int per_block, int blocks, int ff, float limit,
                       float alpha, float up_offset, const float* __restrict__ bias) {
    const long row = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= blocks * ff) return;
    const int e = c / ff, j = c - e * ff;
    const TA* base = u + row * ldu + (size_t)e * 2 * ff;
    float g[8], up[8];
    Vec8<TA>::load(base + j, g);
    Vec8<TA>::load(base + ff + j, up);
    if (bias) {         // the biases of the two projections, laid out like a row of u
        float bg[8], bu[8];
        Vec8<float>::load(bias + (size_t)e * 2 * ff + j, bg);
        Vec8<float>::load(bias + (size_t)e * 2 * ff + ff + j, bu);
#pragma unroll
        for (int i = 0; i < 8; ++i) { g[i] += bg[i]; up[i] += bu[i]; }
    }
    const float w = weights ? (per_block ? weights[row * ldw + e] : weights[row * ldw]) : 1.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float gv = fminf(g[i], limit);
        const float uv = fminf(fmaxf(up[i], -limit), limit);
        float s;
        if constexpr (EXACT) s = 1.f / (1.f + expf(-alpha * gv));
        else s = __fdividef(1.f, 1.f + __expf(-alpha * gv));
        g[i] = gv * s * (uv + up_offset) * w;
    }
    Vec8<TA>::store(act + row * lda + c, g);
}

}  // namespace

MRUN_API int mrun_table_route(const int* ids, const int* table, float* weights, int* chosen, int tokens, int vocab,
                              int experts, int top, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && vocab > 0 && experts > 0 && top > 0 && top <= experts,
                 "table_route: bad sizes tokens=%d vocab=%d experts=%d top=%d", tokens, vocab, experts, top);
    if (tokens == 0) return 0;
    table_route_kernel<<<(tokens + 3) / 4, 128, 0, stream>>>(ids, table, weights, chosen, tokens, vocab, experts, top);
    MRUN_CHECK_LAUNCH("table_route");
    return 0;
}

MRUN_API int mrun_route_grouped(const float* logits, long ldz, float* weights, float* shared_w, int* chosen, int tokens,
                                int experts, int top, int groups, int keep, int group_top, float scale,
                                cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && experts > 0 && top > 0 && groups > 0 && keep > 0 && group_top > 0,
                 "route_grouped: bad sizes tokens=%d experts=%d top=%d groups=%d", tokens, experts, top, groups);
    MRUN_REQUIRE(experts % groups == 0 && keep <= groups && top <= keep * (experts / groups),
                 "route_grouped: %d experts in %d groups of which %d stay cannot give %d choices", experts, groups, keep, top);
    MRUN_REQUIRE(experts + groups <= 2048, "route_grouped: %d experts exceed the supported 2048", experts + groups);
    MRUN_REQUIRE(ldz >= experts + (shared_w ? 1 : 0), "route_grouped: the logits' row stride is below the row");
    if (tokens == 0) return 0;
    const size_t smem = 4 * (size_t)(experts + groups) * sizeof(float);
    route_grouped_kernel<<<(tokens + 3) / 4, 128, smem, stream>>>(logits, ldz, weights, shared_w, chosen, tokens, experts,
                                                                top, groups, keep, group_top, scale);
    MRUN_CHECK_LAUNCH("route_grouped");
    return 0;
}

// limit: the clamp of gate and up (infinity: none); up_offset: what is added to up before the product;
// bias (nullable): float32 [blocks * 2 * ff], added to gate and up before the clamp.
MRUN_API int mrun_clamped_glu(const void* u, long ldu, void* act, long lda, int act_dtype, const float* weights, long ldw,
                              int per_block, int rows, int blocks, int ff, float limit, float alpha, float up_offset,
                              const float* bias, cudaStream_t stream) {
    MRUN_REQUIRE(rows >= 0 && blocks > 0 && ff > 0, "clamped_glu: bad sizes rows=%d blocks=%d ff=%d", rows, blocks, ff);
    MRUN_REQUIRE(ldu >= (long)blocks * 2 * ff && lda >= (long)blocks * ff, "clamped_glu: a row stride below the row");
    if (rows == 0) return 0;
    const long total = (long)rows * blocks * ff;
    const unsigned grid = (unsigned)((total + 255) / 256);
    const size_t unit = act_dtype == MRUN_F32 ? 4 : 2;
    if (ff % 8 == 0 && ((((uintptr_t)u) | ((uintptr_t)act) | ((uintptr_t)bias)) & 15) == 0 && (ldu * unit) % 16 == 0 && (lda * unit) % 16 == 0 &&
        rows <= 0x7fffffff) {
        const dim3 vec_grid(rows, (blocks * ff / 8 + 255) / 256);
        if (act_dtype == MRUN_F32)
            clamped_glu_vec_kernel<float, true><<<vec_grid, 256, 0, stream>>>((const float*)u, ldu, (float*)act, lda, weights,
                                                                               ldw, per_block, blocks, ff, limit, alpha,
                                                                               up_offset, bias);
        else if (act_dtype == MRUN_BF16)
            clamped_glu_vec_kernel<__nv_bfloat16, false><<<vec_grid, 256, 0, stream>>>(
                (const __nv_bfloat16*)u, ldu, (__nv_bfloat16*)act, lda, weights, ldw, per_block, blocks, ff, limit, alpha,
                up_offset, bias);
        else
            return mrun_set_error("clamped_glu: unknown dtype code %d", act_dtype);
        MRUN_CHECK_LAUNCH("clamped_glu");
        return 0;
    }
    if (act_dtype == MRUN_F32)
        clamped_glu_kernel<float, true><<<grid, 256, 0, stream>>>((const float*)u, ldu, (float*)act, lda, weights, ldw,
                                                                   per_block, total, blocks, ff, limit, alpha, up_offset, bias);
    else if (act_dtype == MRUN_BF16)
        clamped_glu_kernel<__nv_bfloat16, false><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)u, ldu, (__nv_bfloat16*)act,
                                                                            lda, weights, ldw, per_block, total, blocks, ff,
                                                                            limit, alpha, up_offset, bias);
    else
        return mrun_set_error("clamped_glu: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("clamped_glu");
    return 0;
}

// counts, ends, cursor: int32 [experts] (counts zeroed by the caller); source, row_weight: [pairs];
// dest: [pairs] (= [tokens, top]).
MRUN_API int mrun_moe_sort(const int* chosen, const float* weights, int tokens, int experts, int top, int* counts,
                           int* ends, int* cursor, int* source, float* row_weight, int* dest, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && experts > 0 && experts <= 4096 && top > 0 && top <= experts,
                 "moe_sort: bad sizes tokens=%d experts=%d top=%d", tokens, experts, top);
    const long pairs = (long)tokens * top;
    MRUN_REQUIRE(pairs < (1L << 31), "moe_sort: %ld pairs exceed the supported 2^31", pairs);
    if (pairs == 0) return 0;
    const int blocks = (int)((pairs + 255) / 256);
    moe_count_kernel<<<blocks < 512 ? blocks : 512, 256, experts * sizeof(int), stream>>>(chosen, (int)pairs, experts, counts);
    MRUN_CHECK_LAUNCH("moe_sort (count)");
    moe_scan_kernel<<<1, 32, 0, stream>>>(counts, experts, ends, cursor);
    MRUN_CHECK_LAUNCH("moe_sort (scan)");
    moe_place_kernel<<<blocks, 256, 0, stream>>>(chosen, weights, (int)pairs, experts, top, cursor, source, row_weight, dest);
    MRUN_CHECK_LAUNCH("moe_sort (place)");
    return 0;
}

MRUN_API int mrun_gather_rows(const void* x, int act_dtype, const int* source, void* out, int rows, int width,
                              cudaStream_t stream) {
    MRUN_REQUIRE(rows >= 0 && width > 0, "gather_rows: bad sizes rows=%d width=%d", rows, width);
    if (rows == 0) return 0;
    if (act_dtype == MRUN_BF16)
        gather_rows_kernel<__nv_bfloat16><<<rows, 128, 0, stream>>>((const __nv_bfloat16*)x, source, (__nv_bfloat16*)out, width);
    else if (act_dtype == MRUN_F32)
        gather_rows_kernel<float><<<rows, 128, 0, stream>>>((const float*)x, source, (float*)out, width);
    else
        return mrun_set_error("gather_rows: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("gather_rows");
    return 0;
}

MRUN_API int mrun_relu2_rows(const void* u, void* act, int act_dtype, const float* row_weight, int rows, int width,
                             cudaStream_t stream) {
    MRUN_REQUIRE(rows >= 0 && width > 0, "relu2_rows: bad sizes rows=%d width=%d", rows, width);
    if (rows == 0) return 0;
    const bool vec = width % 8 == 0 && ((((uintptr_t)u) | ((uintptr_t)act)) & 15) == 0;
    if (act_dtype == MRUN_BF16 && vec)
        relu2_rows_kernel<__nv_bfloat16, true><<<rows, 128, 0, stream>>>((const __nv_bfloat16*)u, (__nv_bfloat16*)act, row_weight, width);
    else if (act_dtype == MRUN_BF16)
        relu2_rows_kernel<__nv_bfloat16, false><<<rows, 256, 0, stream>>>((const __nv_bfloat16*)u, (__nv_bfloat16*)act, row_weight, width);
    else if (act_dtype == MRUN_F32)
        relu2_rows_kernel<float, false><<<rows, 256, 0, stream>>>((const float*)u, (float*)act, row_weight, width);
    else
        return mrun_set_error("relu2_rows: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("relu2_rows");
    return 0;
}

// base: [tokens, width] in the activation dtype (base_f32 = 0) or float32 (1), or null.
MRUN_API int mrun_combine_rows(const void* base, int base_f32, const void* rows, int act_dtype, const int* dest,
                               float* out, int tokens, int top, int width, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && top > 0 && width > 0, "combine_rows: bad sizes tokens=%d top=%d width=%d", tokens, top, width);
    MRUN_REQUIRE(act_dtype == MRUN_BF16, "combine_rows: the sorted path runs in bfloat16");
    if (tokens == 0) return 0;
    const bool vec = width % 8 == 0 && ((((uintptr_t)base) | ((uintptr_t)rows) | ((uintptr_t)out)) & 15) == 0;
    using bf16 = __nv_bfloat16;
    if (base_f32 && vec)
        combine_rows_kernel<bf16, float, true><<<tokens, 128, 0, stream>>>((const float*)base, (const bf16*)rows, dest, out, top, width);
    else if (base_f32)
        combine_rows_kernel<bf16, float, false><<<tokens, 256, 0, stream>>>((const float*)base, (const bf16*)rows, dest, out, top, width);
    else if (vec)
        combine_rows_kernel<bf16, bf16, true><<<tokens, 128, 0, stream>>>((const bf16*)base, (const bf16*)rows, dest, out, top, width);
    else
        combine_rows_kernel<bf16, bf16, false><<<tokens, 256, 0, stream>>>((const bf16*)base, (const bf16*)rows, dest, out, top, width);
    MRUN_CHECK_LAUNCH("combine_rows");
    return 0;
}
