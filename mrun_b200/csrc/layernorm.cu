// Layer norm without a bias fused with the residual sum, the mean of two RMS-normed branches, and
// the two as one kernel.
//
// All arithmetic is 32-bit; a row is one block of 256 threads whatever the batch, so the order of
// additions depends on the width only.
#include "common.cuh"

using namespace mrun;

namespace {

// ------------------------------------------------------------------------------------------
// Residual add + layer norm.
//   v = resid[src] + delta[src]   (delta may be null; it is 32-bit or of the activation type)
//   if rows == null: resid[src] = v            (the stream advances)
//   mu = mean(v); var = mean((v - mu)^2); out[r] = (v - mu) * rsqrt(var + eps) * weight
// The variance is taken from the deviations in a second pass over the staged row, not from
// mean(v^2) - mu^2.  With `rows` the kernel reads row rows[r] and leaves the stream untouched.
// ------------------------------------------------------------------------------------------
template <typename TA, typename TD>
__global__ void add_layernorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                     const float* __restrict__ weight, float eps, TA* __restrict__ out,
                                     const int* __restrict__ rows, int hidden) {
    extern __shared__ float row_buf[];
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float s = 0.f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        float v = resid[src + h];
        if (delta) v += to_float(delta[src + h]);
        row_buf[h] = v;
        s += v;
    }
    const float mu = block_sum(s, scratch) / (float)hidden;
    float ss = 0.f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float d = row_buf[h] - mu;
        ss += d * d;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    TA* dst = out + (size_t)r * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float v = row_buf[h];
        if (!rows && delta) resid[src + h] = v;
        dst[h] = from_float<TA>((v - mu) * inv * weight[h]);
    }
}

// The same for widths that are a multiple of 8 and at most 8192: every thread keeps up to four
// 8-element chunks in registers and moves them with 16-byte loads and stores.
template <typename TA, typename TD>
__global__ void __launch_bounds__(256)
add_layernorm_vec_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const float* __restrict__ weight,
                         float eps, TA* __restrict__ out, const int* __restrict__ rows, int hidden) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    const int chunks = hidden >> 3;
    float v[4][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            Vec8<float>::load(resid + src + c * 8, v[i]);
            if (delta) {
                float d[8];
                Vec8<TD>::load(delta + src + c * 8, d);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[i][e] += d[e];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) s += v[i][e];
        }
    }
    const float mu = block_sum(s, scratch) / (float)hidden;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float d = v[i][e] - mu;
                ss += d * d;
            }
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            if (!rows && delta) Vec8<float>::store(resid + src + c * 8, v[i]);
            float w[8], y[8];
            Vec8<float>::load(weight + c * 8, w);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = (v[i][e] - mu) * inv * w[e];
            Vec8<TA>::store(out + (size_t)r * hidden + c * 8, y);
        }
    }
}

template <typename TA, typename TD>
int launch_add_layernorm(float* resid, const void* delta, const float* weight, float eps, void* out, const int* rows,
                         int n_rows, int hidden, cudaStream_t stream) {
    const bool aligned = (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
    if (hidden % 8 == 0 && hidden <= 8192 && aligned) {
        MRUN_CHECK_CUDA(launch_kernel(add_layernorm_vec_kernel<TA, TD>, dim3(n_rows), dim3(256), 0, stream, resid,
                                      (const TD*)delta, weight, eps, (TA*)out, rows, hidden), "add_layernorm");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 48 * 1024)
        MRUN_CHECK_CUDA(cudaFuncSetAttribute(add_layernorm_kernel<TA, TD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem), "add_layernorm");
    add_layernorm_kernel<TA, TD><<<n_rows, 256, smem, stream>>>(resid, (const TD*)delta, weight, eps, (TA*)out, rows,
                                                                hidden);
    return 0;
}

// ------------------------------------------------------------------------------------------
// out = share * (rmsnorm(a) * wa + rmsnorm(b) * wb), row by row: two branches that read the same
// input, each divided by its root mean square over the row (eps inside the root) and multiplied
// by its own weight.  a and b are 32-bit (the branches' last products write 32-bit sums); out is
// 32-bit, the not-yet-added branch output that the next norm folds into the stream.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
pair_norm_mean_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ wa,
                      const float* __restrict__ wb, float eps, float share, float* __restrict__ out, int hidden) {
    __shared__ float scratch[33];
    const size_t row = (size_t)blockIdx.x * hidden;
    float sa = 0.f, sb = 0.f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float x = a[row + h], y = b[row + h];
        sa += x * x;
        sb += y * y;
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ia = rsqrtf(sa / (float)hidden + eps), ib = rsqrtf(sb / (float)hidden + eps);
    for (int h = threadIdx.x; h < hidden; h += blockDim.x)
        out[row + h] = share * (a[row + h] * ia * wa[h] + b[row + h] * ib * wb[h]);
}

// ------------------------------------------------------------------------------------------
// The two steps above as one: v = resid + share * (rmsnorm(a) * wa + rmsnorm(b) * wb), then the
// layer norm of v with `weight`.  rows == null: resid = v (the stream advances); with `rows` the
// kernel reads row rows[r] of resid, a and b and leaves the stream as it is.  The row is staged
// in shared memory.
// ------------------------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(256)
pair_norm_add_layernorm_kernel(float* __restrict__ resid, const float* __restrict__ a, const float* __restrict__ b,
                               const float* __restrict__ wa, const float* __restrict__ wb, float eps_pair, float share,
                               const float* __restrict__ weight, float eps, TA* __restrict__ out,
                               const int* __restrict__ rows, int hidden) {
    extern __shared__ float row_buf[];
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float sa = 0.f, sb = 0.f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float x = a[src + h], y = b[src + h];
        sa += x * x;
        sb += y * y;
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ia = rsqrtf(sa / (float)hidden + eps_pair), ib = rsqrtf(sb / (float)hidden + eps_pair);
    float s = 0.f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float v = resid[src + h] + share * (a[src + h] * ia * wa[h] + b[src + h] * ib * wb[h]);
        row_buf[h] = v;
        s += v;
    }
    const float mu = block_sum(s, scratch) / (float)hidden;
    float ss = 0.f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float d = row_buf[h] - mu;
        ss += d * d;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    TA* dst = out + (size_t)r * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float v = row_buf[h];
        if (!rows) resid[src + h] = v;
        dst[h] = from_float<TA>((v - mu) * inv * weight[h]);
    }
}

// The same for widths that are a multiple of 8 and at most 8192: both branches and the stream are
// read once, in 16-byte pieces, and kept in registers through the four sums.
template <typename TA>
__global__ void __launch_bounds__(256)
pair_norm_add_layernorm_vec_kernel(float* __restrict__ resid, const float* __restrict__ a, const float* __restrict__ b,
                                   const float* __restrict__ wa, const float* __restrict__ wb, float eps_pair, float share,
                                   const float* __restrict__ weight, float eps, TA* __restrict__ out,
                                   const int* __restrict__ rows, int hidden) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    const int chunks = hidden >> 3;
    float va[4][8], vb[4][8], v[4][8];
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            Vec8<float>::load(a + src + c * 8, va[i]);
            Vec8<float>::load(b + src + c * 8, vb[i]);
            Vec8<float>::load(resid + src + c * 8, v[i]);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                sa += va[i][e] * va[i][e];
                sb += vb[i][e] * vb[i][e];
            }
        }
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ia = rsqrtf(sa / (float)hidden + eps_pair), ib = rsqrtf(sb / (float)hidden + eps_pair);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            float x[8], y[8];
            Vec8<float>::load(wa + c * 8, x);
            Vec8<float>::load(wb + c * 8, y);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[i][e] += share * (va[i][e] * ia * x[e] + vb[i][e] * ib * y[e]);
                s += v[i][e];
            }
        }
    }
    const float mu = block_sum(s, scratch) / (float)hidden;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float d = v[i][e] - mu;
                ss += d * d;
            }
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            if (!rows) Vec8<float>::store(resid + src + c * 8, v[i]);
            float w[8], y[8];
            Vec8<float>::load(weight + c * 8, w);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = (v[i][e] - mu) * inv * w[e];
            Vec8<TA>::store(out + (size_t)r * hidden + c * 8, y);
        }
    }
}

}  // namespace

// delta_dtype: the type of `delta` (MRUN_F32, or the activation type `act_dtype`).
MRUN_API int mrun_add_layernorm(float* resid, const void* delta, int delta_dtype, const float* weight, float eps,
                                void* out, int act_dtype, const int* rows, int n_rows, int hidden,
                                cudaStream_t stream) {
    MRUN_REQUIRE(n_rows >= 0 && hidden > 0, "add_layernorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    MRUN_REQUIRE((size_t)hidden * sizeof(float) <= 200 * 1024, "add_layernorm: hidden=%d exceeds the supported 51200",
                 hidden);
    MRUN_REQUIRE(act_dtype == MRUN_F32 || act_dtype == MRUN_BF16, "add_layernorm: unknown dtype code %d", act_dtype);
    MRUN_REQUIRE(delta == nullptr || delta_dtype == MRUN_F32 || delta_dtype == act_dtype,
                 "add_layernorm: delta has dtype code %d, expected 32-bit or the activation type %d", delta_dtype, act_dtype);
    if (n_rows == 0) return 0;
    int rc;
    if (act_dtype == MRUN_F32)
        rc = launch_add_layernorm<float, float>(resid, delta, weight, eps, out, rows, n_rows, hidden, stream);
    else if (delta == nullptr || delta_dtype == MRUN_BF16)
        rc = launch_add_layernorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, weight, eps, out, rows, n_rows, hidden, stream);
    else
        rc = launch_add_layernorm<__nv_bfloat16, float>(resid, delta, weight, eps, out, rows, n_rows, hidden, stream);
    if (rc) return rc;
    MRUN_CHECK_LAUNCH("add_layernorm");
    return 0;
}

MRUN_API int mrun_pair_norm_mean(const float* a, const float* b, const float* wa, const float* wb, float eps,
                                 float share, float* out, int rows, int hidden, cudaStream_t stream) {
    MRUN_REQUIRE(rows >= 0 && hidden > 0, "pair_norm_mean: bad sizes rows=%d hidden=%d", rows, hidden);
    if (rows == 0) return 0;
    pair_norm_mean_kernel<<<rows, 256, 0, stream>>>(a, b, wa, wb, eps, share, out, hidden);
    MRUN_CHECK_LAUNCH("pair_norm_mean");
    return 0;
}

MRUN_API int mrun_pair_norm_add_layernorm(float* resid, const float* a, const float* b, const float* wa, const float* wb,
                                          float eps_pair, float share, const float* weight, float eps, void* out,
                                          int act_dtype, const int* rows, int n_rows, int hidden, cudaStream_t stream) {
    MRUN_REQUIRE(n_rows >= 0 && hidden > 0, "pair_norm_add_layernorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    MRUN_REQUIRE((size_t)hidden * sizeof(float) <= 200 * 1024, "pair_norm_add_layernorm: hidden=%d exceeds the supported 51200",
                 hidden);
    if (n_rows == 0) return 0;
    const bool aligned = (((uintptr_t)resid | (uintptr_t)a | (uintptr_t)b | (uintptr_t)wa | (uintptr_t)wb | (uintptr_t)weight |
                           (uintptr_t)out) & 15) == 0;
    if (hidden % 8 == 0 && hidden <= 8192 && aligned && (act_dtype == MRUN_F32 || act_dtype == MRUN_BF16)) {
        if (act_dtype == MRUN_F32)
            pair_norm_add_layernorm_vec_kernel<float><<<n_rows, 256, 0, stream>>>(resid, a, b, wa, wb, eps_pair, share, weight,
                                                                                  eps, (float*)out, rows, hidden);
        else
            pair_norm_add_layernorm_vec_kernel<__nv_bfloat16><<<n_rows, 256, 0, stream>>>(
                resid, a, b, wa, wb, eps_pair, share, weight, eps, (__nv_bfloat16*)out, rows, hidden);
        MRUN_CHECK_LAUNCH("pair_norm_add_layernorm");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (act_dtype == MRUN_F32) {
        if (smem > 48 * 1024)
            MRUN_CHECK_CUDA(cudaFuncSetAttribute(pair_norm_add_layernorm_kernel<float>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "pair_norm_add_layernorm");
        pair_norm_add_layernorm_kernel<float><<<n_rows, 256, smem, stream>>>(resid, a, b, wa, wb, eps_pair, share, weight, eps,
                                                                             (float*)out, rows, hidden);
    } else if (act_dtype == MRUN_BF16) {
        if (smem > 48 * 1024)
            MRUN_CHECK_CUDA(cudaFuncSetAttribute(pair_norm_add_layernorm_kernel<__nv_bfloat16>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "pair_norm_add_layernorm");
        pair_norm_add_layernorm_kernel<__nv_bfloat16><<<n_rows, 256, smem, stream>>>(resid, a, b, wa, wb, eps_pair, share, weight,
                                                                                     eps, (__nv_bfloat16*)out, rows, hidden);
    } else {
        return mrun_set_error("pair_norm_add_layernorm: unknown dtype code %d", act_dtype);
    }
    MRUN_CHECK_LAUNCH("pair_norm_add_layernorm");
    return 0;
}
