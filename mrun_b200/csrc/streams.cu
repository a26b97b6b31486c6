// Several residual streams a token (hyper-connections).
//
// A model with S streams keeps [tokens, S, width] 32-bit rows instead of one residual row.  A
// sublayer reads a weighted sum of the streams and writes back into all of them:
//
//     u      = sum_s in[s] * x_s                       (what the sublayer's norm sees)
//     x_t'   = sum_s mix[s, t] * x_s + out[t] * y      (all streams at once from the old ones)
//
// The write of one sublayer and the read of the next are one kernel here: the block of a token
// loads its S rows once, applies the pending write (if any), stores the new rows, forms the next
// sublayer's u and norms it.  With S = 1, mix = out = in = 1 this is the plain residual sum
// followed by an RMS norm.  All sums are 32-bit and run over s in rising order, so a row's bits
// depend on the row only.
//
// Kernels:
//   embed_streams   the embedding row of a token copied into each of its S streams
//   embed_bigram    the same with the row times a scale plus a row of a second table, chosen by a
//                   hash of the token and the one before it (the request's state across steps)
//   streams_step    pending write + read + RMS norm (eps inside the root), see above
#include "common.cuh"

using namespace mrun;

namespace {

constexpr int MAX_STREAMS = 8;

template <typename TW>
__global__ void embed_streams_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                     float* __restrict__ out, int hidden, int vocab, int copies) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const TW* row = table + (size_t)(ok ? id : 0) * hidden;
    float* dst = out + (size_t)t * copies * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float v = ok ? to_float(row[h]) : 0.f;
        for (int s = 0; s < copies; ++s) dst[(size_t)s * hidden + h] = v;
    }
}

// The row of the pair table for every token: a hash of the token and the one before it in its
// request, the table's last row for a request's first token, -1 for a padding row.  The token
// before a step's first token of a request is the request's state.  A token is the first of its
// segment when the row before it belongs to another request or is not the position before.
__global__ void bigram_rows_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                   const int* __restrict__ token_slot, const int* __restrict__ state,
                                   int* __restrict__ rows, int tokens, int vocab, int buckets, long long mul_prev,
                                   long long mul_cur) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens) return;
    const int pos = positions[t], id = ids[t];
    if (pos < 0 || id < 0 || id >= vocab) { rows[t] = -1; return; }
    if (pos == 0) { rows[t] = buckets; return; }
    const bool first = t == 0 || token_slot[t - 1] != token_slot[t] || positions[t - 1] != pos - 1;
    const int before = first ? state[token_slot[t]] : ids[t - 1];
    rows[t] = (int)(((long long)before * mul_prev + (long long)id * mul_cur) % (long long)buckets);
}

// out[t, s] = table[ids[t]] * scale + pairs[rows[t]] for each of the S streams; the block of a
// request's last token of the step leaves that token as the request's state.
template <typename TW>
__global__ void embed_bigram_kernel(const TW* __restrict__ table, const TW* __restrict__ pairs,
                                    const int* __restrict__ ids, const int* __restrict__ positions,
                                    const int* __restrict__ token_slot, const int* __restrict__ rows,
                                    int* __restrict__ state, float* __restrict__ out, int tokens, int hidden, int vocab,
                                    int copies, float scale) {
    const int t = blockIdx.x;
    const int id = ids[t], pos = positions[t];
    const bool ok = pos >= 0 && id >= 0 && id < vocab;
    const TW* row = table + (size_t)(ok ? id : 0) * hidden;
    const int pair = (pairs && ok) ? rows[t] : -1;
    const TW* add = pair >= 0 ? pairs + (size_t)pair * hidden : nullptr;
    float* dst = out + (size_t)t * copies * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        float v = ok ? to_float(row[h]) * scale : 0.f;
        if (add) v += to_float(add[h]);
        for (int s = 0; s < copies; ++s) dst[(size_t)s * hidden + h] = v;
    }
    if (state && ok && threadIdx.x == 0) {
        const bool last = t == tokens - 1 || token_slot[t + 1] != token_slot[t] || positions[t + 1] != pos + 1;
        if (last) state[token_slot[t]] = id;
    }
}

// One block a row.  `rows` (optional) names the tokens to read: the streams are then left as they
// are and row r of the outputs belongs to token rows[r].  `y` is the pending sublayer output
// (32-bit, one row a token) or null; `norm_w` null leaves u un-normed (32-bit output `u_out`).
template <typename TO>
__global__ void __launch_bounds__(256)
streams_step_kernel(float* __restrict__ streams, const float* __restrict__ y, const float* __restrict__ mix,
                    const float* __restrict__ out_c, const float* __restrict__ in_c,
                    const float* __restrict__ norm_w, float eps, TO* __restrict__ h_out,
                    float* __restrict__ u_out, const int* __restrict__ rows, int S, int width) {
    extern __shared__ float u_row[];          // width
    __shared__ float scratch[33];
    __shared__ float c_mix[MAX_STREAMS * MAX_STREAMS], c_out[MAX_STREAMS], c_in[MAX_STREAMS];
    const int r = blockIdx.x, tid = threadIdx.x;
    const long t = rows ? rows[r] : r;
    if (tid < S * S) c_mix[tid] = (y && mix) ? mix[tid] : ((tid / S == tid % S) ? 1.f : 0.f);
    if (tid < S) { c_out[tid] = (y && out_c) ? out_c[tid] : (y ? 1.f : 0.f); c_in[tid] = in_c ? in_c[tid] : 1.f; }
    __syncthreads();
    float* x = streams + t * S * width;
    float ss = 0.f;
    for (int c = tid; c < width; c += blockDim.x) {
        float old[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s) old[s] = s < S ? x[(size_t)s * width + c] : 0.f;
        float u = 0.f;
        if (y) {
            const float yv = y[t * width + c];
#pragma unroll
            for (int to = 0; to < MAX_STREAMS; ++to) {
                if (to < S) {
                    float v = 0.f;
#pragma unroll
                    for (int s = 0; s < MAX_STREAMS; ++s)
                        if (s < S) v = fmaf(c_mix[s * S + to], old[s], v);
                    v = fmaf(c_out[to], yv, v);
                    if (!rows) x[(size_t)to * width + c] = v;
                    u = fmaf(c_in[to], v, u);
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < S) u = fmaf(c_in[s], old[s], u);
        }
        u_row[c] = u;
        ss += u * u;
    }
    if (u_out)
        for (int c = tid; c < width; c += blockDim.x) u_out[(size_t)r * width + c] = u_row[c];
    if (!norm_w) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)width + eps);
    for (int c = tid; c < width; c += blockDim.x)
        h_out[(size_t)r * width + c] = from_float<TO>(u_row[c] * inv * norm_w[c]);
}

// The same with four columns a thread (width a multiple of 4): 16-byte loads and stores, the row's
// u kept in registers between the sweep and the norm (width <= 4 * 256 * VEC_SWEEPS).
constexpr int VEC_SWEEPS = 8;

template <typename TO>
__global__ void __launch_bounds__(256)
streams_step_vec_kernel(float* __restrict__ streams, const float* __restrict__ y, const float* __restrict__ mix,
                        const float* __restrict__ out_c, const float* __restrict__ in_c,
                        const float* __restrict__ norm_w, float eps, TO* __restrict__ h_out,
                        float* __restrict__ u_out, const int* __restrict__ rows, int S, int width) {
    __shared__ float scratch[33];
    __shared__ float c_mix[MAX_STREAMS * MAX_STREAMS], c_out[MAX_STREAMS], c_in[MAX_STREAMS];
    const int r = blockIdx.x, tid = threadIdx.x;
    const long t = rows ? rows[r] : r;
    if (tid < S * S) c_mix[tid] = (y && mix) ? mix[tid] : ((tid / S == tid % S) ? 1.f : 0.f);
    if (tid < S) { c_out[tid] = (y && out_c) ? out_c[tid] : (y ? 1.f : 0.f); c_in[tid] = in_c ? in_c[tid] : 1.f; }
    __syncthreads();
    float* x = streams + t * S * width;
    float4 u_keep[VEC_SWEEPS];
    float ss = 0.f;
#pragma unroll
    for (int sweep = 0; sweep < VEC_SWEEPS; ++sweep) {
        const int c = (sweep * 256 + tid) * 4;
        u_keep[sweep] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c >= width) continue;
        float4 old[MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < MAX_STREAMS; ++s)
            if (s < S) old[s] = *reinterpret_cast<const float4*>(x + (size_t)s * width + c);
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
        if (y) {
            const float4 yv = *reinterpret_cast<const float4*>(y + t * width + c);
#pragma unroll
            for (int to = 0; to < MAX_STREAMS; ++to) {
                if (to < S) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int s = 0; s < MAX_STREAMS; ++s)
                        if (s < S) {
                            const float m = c_mix[s * S + to];
                            v.x = fmaf(m, old[s].x, v.x); v.y = fmaf(m, old[s].y, v.y);
                            v.z = fmaf(m, old[s].z, v.z); v.w = fmaf(m, old[s].w, v.w);
                        }
                    const float o = c_out[to], w_in = c_in[to];
                    v.x = fmaf(o, yv.x, v.x); v.y = fmaf(o, yv.y, v.y); v.z = fmaf(o, yv.z, v.z); v.w = fmaf(o, yv.w, v.w);
                    if (!rows) *reinterpret_cast<float4*>(x + (size_t)to * width + c) = v;
                    u.x = fmaf(w_in, v.x, u.x); u.y = fmaf(w_in, v.y, u.y); u.z = fmaf(w_in, v.z, u.z); u.w = fmaf(w_in, v.w, u.w);
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
                if (s < S) {
                    const float w_in = c_in[s];
                    u.x = fmaf(w_in, old[s].x, u.x); u.y = fmaf(w_in, old[s].y, u.y);
                    u.z = fmaf(w_in, old[s].z, u.z); u.w = fmaf(w_in, old[s].w, u.w);
                }
        }
        u_keep[sweep] = u;
        ss += u.x * u.x; ss += u.y * u.y; ss += u.z * u.z; ss += u.w * u.w;
        if (u_out) *reinterpret_cast<float4*>(u_out + (size_t)r * width + c) = u;
    }
    if (!norm_w) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int sweep = 0; sweep < VEC_SWEEPS; ++sweep) {
        const int c = (sweep * 256 + tid) * 4;
        if (c >= width) continue;
        const float4 w = *reinterpret_cast<const float4*>(norm_w + c);
        const float4 u = u_keep[sweep];
        TO* dst = h_out + (size_t)r * width + c;
        dst[0] = from_float<TO>(u.x * inv * w.x); dst[1] = from_float<TO>(u.y * inv * w.y);
        dst[2] = from_float<TO>(u.z * inv * w.z); dst[3] = from_float<TO>(u.w * inv * w.w);
    }
}

}  // namespace

MRUN_API int mrun_embed_streams(const void* table, int table_dtype, const int* ids, float* out, int tokens,
                                int hidden, int vocab, int copies, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0 && copies >= 1,
                 "embed_streams: bad sizes tokens=%d hidden=%d vocab=%d copies=%d", tokens, hidden, vocab, copies);
    if (tokens == 0) return 0;
    if (table_dtype == MRUN_F32)
        embed_streams_kernel<float><<<tokens, 256, 0, stream>>>((const float*)table, ids, out, hidden, vocab, copies);
    else if (table_dtype == MRUN_BF16)
        embed_streams_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>((const __nv_bfloat16*)table, ids, out,
                                                                         hidden, vocab, copies);
    else
        return mrun_set_error("embed_streams: unknown dtype code %d", table_dtype);
    MRUN_CHECK_LAUNCH("embed_streams");
    return 0;
}

// table: [vocab, hidden]; pairs: [buckets + 1, hidden] in the same dtype, or null (no second
// table); state: int32 [slots], the last token each request brought; rows: int32 [tokens] scratch.
MRUN_API int mrun_embed_bigram(const void* table, const void* pairs, int table_dtype, const int* ids,
                               const int* positions, const int* token_slot, int* state, int* rows, float* out,
                               int tokens, int hidden, int vocab, int copies, float scale, int buckets, long mul_prev,
                               long mul_cur, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0 && copies >= 1,
                 "embed_bigram: bad sizes tokens=%d hidden=%d vocab=%d copies=%d", tokens, hidden, vocab, copies);
    MRUN_REQUIRE(pairs == nullptr || (buckets > 0 && state != nullptr && rows != nullptr && mul_prev >= 0 && mul_cur >= 0),
                 "embed_bigram: a pair table needs buckets, multipliers, a state and scratch rows");
    if (tokens == 0) return 0;
    if (pairs) {
        bigram_rows_kernel<<<(tokens + 127) / 128, 128, 0, stream>>>(ids, positions, token_slot, state, rows, tokens,
                                                                     vocab, buckets, mul_prev, mul_cur);
        MRUN_CHECK_LAUNCH("embed_bigram (rows)");
    }
    if (table_dtype == MRUN_F32)
        embed_bigram_kernel<float><<<tokens, 256, 0, stream>>>((const float*)table, (const float*)pairs, ids, positions,
                                                                token_slot, rows, pairs ? state : nullptr, out, tokens,
                                                                hidden, vocab, copies, scale);
    else if (table_dtype == MRUN_BF16)
        embed_bigram_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(
            (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, ids, positions, token_slot, rows,
            pairs ? state : nullptr, out, tokens, hidden, vocab, copies, scale);
    else
        return mrun_set_error("embed_bigram: unknown dtype code %d", table_dtype);
    MRUN_CHECK_LAUNCH("embed_bigram");
    return 0;
}

// streams: float32 [tokens, S, width].  y: float32 [tokens, width] or null.  mix: [S, S] indexed
// [from, to]; out_c, in_c: [S] (null: ones).  norm_w: float32 [width] or null.  h_out: [n_rows,
// width] in out_dtype (needed with norm_w); u_out: float32 [n_rows, width] or null.
MRUN_API int mrun_streams_step(float* streams, const float* y, const float* mix, const float* out_c,
                               const float* in_c, const float* norm_w, float eps, void* h_out, int out_dtype,
                               float* u_out, const int* rows, int n_rows, int S, int width, cudaStream_t stream) {
    MRUN_REQUIRE(n_rows >= 0 && width > 0, "streams_step: bad sizes rows=%d width=%d", n_rows, width);
    MRUN_REQUIRE(S >= 1 && S <= MAX_STREAMS, "streams_step: %d streams, the kernel takes 1 to %d", S, MAX_STREAMS);
    MRUN_REQUIRE(width <= 12000, "streams_step: width=%d exceeds the supported 12000", width);
    MRUN_REQUIRE(norm_w == nullptr || h_out != nullptr, "streams_step: a norm needs an output");
    MRUN_REQUIRE(norm_w != nullptr || u_out != nullptr, "streams_step: nothing to write");
    if (n_rows == 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    const bool aligned = ((((uintptr_t)streams) | ((uintptr_t)y) | ((uintptr_t)norm_w) | ((uintptr_t)u_out)) & 15) == 0;
    if (width % 4 == 0 && width <= 4 * 256 * VEC_SWEEPS && aligned) {
        if (out_dtype == MRUN_F32)
            streams_step_vec_kernel<float><<<n_rows, 256, 0, stream>>>(streams, y, mix, out_c, in_c, norm_w, eps,
                                                                        (float*)h_out, u_out, rows, S, width);
        else if (out_dtype == MRUN_BF16)
            streams_step_vec_kernel<__nv_bfloat16><<<n_rows, 256, 0, stream>>>(
                streams, y, mix, out_c, in_c, norm_w, eps, (__nv_bfloat16*)h_out, u_out, rows, S, width);
        else
            return mrun_set_error("streams_step: unknown dtype code %d", out_dtype);
        MRUN_CHECK_LAUNCH("streams_step");
        return 0;
    }
    if (out_dtype == MRUN_F32)
        streams_step_kernel<float><<<n_rows, 256, smem, stream>>>(streams, y, mix, out_c, in_c, norm_w, eps,
                                                                   (float*)h_out, u_out, rows, S, width);
    else if (out_dtype == MRUN_BF16)
        streams_step_kernel<__nv_bfloat16><<<n_rows, 256, smem, stream>>>(
            streams, y, mix, out_c, in_c, norm_w, eps, (__nv_bfloat16*)h_out, u_out, rows, S, width);
    else
        return mrun_set_error("streams_step: unknown dtype code %d", out_dtype);
    MRUN_CHECK_LAUNCH("streams_step");
    return 0;
}
