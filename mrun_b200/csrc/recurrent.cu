// Mixers that carry a state of fixed size from token to token, and the short causal convolutions
// in front of them.
//
// A step's tokens come as segments (one per request: rows seg_q_start[s] .. seg_q_start[s+1] of
// the flat batch, state slot seg_slot[s]); a segment of zero rows is padding.  Every kernel reads
// the state its request left, walks the segment's tokens in order and leaves the state for the
// next step, so a token's result does not depend on how the request was cut into steps or on the
// requests beside it.  States and all arithmetic of the recurrences are 32-bit.
//
// Kernels:
//   causal_conv     y_t = sum_j w[:, j] x_(t - taps + 1 + j) per channel (the last tap meets the
//                   token itself; zeros before the sequence's start), either added to x_t or
//                   passed through SiLU; the last taps - 1 inputs of a request are its state
//   decay_scan      per head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t (linear attention
//                   with one decay a head; q, k, v optionally through SiLU on the way in)
//   delta_scan      per head, with a decay per key channel g = exp(-exp(A_h) softplus(a + bias)),
//                   a write strength beta = sigmoid(b) and unit-length q (times dim^-1/2) and k:
//                   S <- g * S (rows); u = beta (v - S^T k); S <- S + k u^T; o = S^T q
//   gated_scan      per head, with a decay per key channel g = sigmoid(a + bias)^(1/tau) and q
//                   times dim^-1/2: S <- g * S (rows) + k v^T; o = S^T q (gated linear attention)
//   gated_norm      per group of n outputs: o / sqrt(mean(o^2) + eps) * w * f(gate), f the sigmoid
//                   or SiLU
#include "common.cuh"

using namespace mrun;

namespace {

constexpr int MAX_TAPS = 8;
constexpr int CONV_TILE = 16;       // tokens a block walks; at least MAX_TAPS - 1 (measured: 8 is slower, every block loads its weights)

template <bool EXACT> __device__ __forceinline__ float silu_f(float z) {
    if constexpr (EXACT) return z / (1.f + expf(-z));
    else return __fdividef(z, 1.f + __expf(-z));
}

// grid (channel chunks, token tiles, segments); a thread a channel.  Only a segment's first tile
// reads the state (its tokens have fewer than taps - 1 tokens of the step before them), and that
// block also leaves the new state once it has read the old one.
template <typename TA>
__global__ void __launch_bounds__(128)
causal_conv_kernel(const TA* __restrict__ x, long ldx, const float* __restrict__ w, TA* __restrict__ state,
                   TA* __restrict__ out, long ldo, const int* __restrict__ seg_q_start,
                   const int* __restrict__ seg_slot, int C, int taps, int residual, int silu) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seg = blockIdx.z;
    const int q0 = seg_q_start[seg], n = seg_q_start[seg + 1] - q0;
    const int l0 = blockIdx.y * CONV_TILE;
    if (c >= C || l0 >= n) return;
    TA* st = state + (size_t)seg_slot[seg] * (taps - 1) * C + c;
    float wv[MAX_TAPS], hist[MAX_TAPS - 1];      // hist[j - 1]: the input j tokens back
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) wv[j] = j < taps ? w[(size_t)c * taps + (taps - 1 - j)] : 0.f;   // wv[j]: of the input j back
#pragma unroll
    for (int j = 1; j < MAX_TAPS; ++j) {
        hist[j - 1] = 0.f;
        if (j < taps) {
            const int l = l0 - j;
            hist[j - 1] = l >= 0 ? to_float(x[(size_t)(q0 + l) * ldx + c]) : to_float(st[(size_t)(l + taps - 1) * C]);
        }
    }
    const int end = min(n, l0 + CONV_TILE);
    for (int l = l0; l < end; ++l) {
        const float cur = to_float(x[(size_t)(q0 + l) * ldx + c]);
        float acc = 0.f;
#pragma unroll
        for (int j = MAX_TAPS - 1; j >= 1; --j)          // oldest input first
            if (j < taps) acc = fmaf(wv[j], hist[j - 1], acc);
        acc = fmaf(wv[0], cur, acc);
        float y = residual ? cur + acc : acc;
        if (silu) y = silu_f<true>(y);
        out[(size_t)(q0 + l) * ldo + c] = from_float<TA>(y);
#pragma unroll
        for (int j = MAX_TAPS - 1; j >= 2; --j) hist[j - 1] = hist[j - 2];
        hist[0] = cur;
    }
    if (blockIdx.y == 0) {
        float fresh[MAX_TAPS - 1];
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i) {
            fresh[i] = 0.f;
            if (i < taps - 1) {
                const int l = n - (taps - 1) + i;
                fresh[i] = l >= 0 ? to_float(x[(size_t)(q0 + l) * ldx + c]) : to_float(st[(size_t)(l + taps - 1) * C]);
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i)
            if (i < taps - 1) st[(size_t)i * C] = from_float<TA>(fresh[i]);
    }
}

// The same with eight channels a thread (channels a multiple of 8, rows on 16-byte boundaries):
// 16-byte loads and stores, four tokens' loads in flight.
template <typename TA>
__global__ void __launch_bounds__(128)
causal_conv_vec_kernel(const TA* __restrict__ x, long ldx, const float* __restrict__ w, TA* __restrict__ state,
                       TA* __restrict__ out, long ldo, const int* __restrict__ seg_q_start,
                       const int* __restrict__ seg_slot, int C, int taps, int residual, int silu) {
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    const int seg = blockIdx.z;
    const int q0 = seg_q_start[seg], n = seg_q_start[seg + 1] - q0;
    const int l0 = blockIdx.y * CONV_TILE;
    if (c >= C || l0 >= n) return;
    TA* st = state + (size_t)seg_slot[seg] * (taps - 1) * C + c;
    float wv[8][MAX_TAPS], hist[MAX_TAPS - 1][8];      // hist[j - 1]: the inputs j tokens back
#pragma unroll
    for (int ch = 0; ch < 8; ++ch)
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j) wv[ch][j] = j < taps ? w[(size_t)(c + ch) * taps + (taps - 1 - j)] : 0.f;
#pragma unroll
    for (int j = 1; j < MAX_TAPS; ++j) {
        if (j < taps) {
            const int l = l0 - j;
            if (l >= 0) Vec8<TA>::load(x + (size_t)(q0 + l) * ldx + c, hist[j - 1]);
            else Vec8<TA>::load(st + (size_t)(l + taps - 1) * C, hist[j - 1]);
        } else {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) hist[j - 1][ch] = 0.f;
        }
    }
    const int end = min(n, l0 + CONV_TILE);
    for (int lb = l0; lb < end; lb += 4) {
        float cur[4][8];
#pragma unroll
        for (int k = 0; k < 4; ++k)
            if (lb + k < end) Vec8<TA>::load(x + (size_t)(q0 + lb + k) * ldx + c, cur[k]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (lb + k >= end) break;
            float y[8];
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                float acc = 0.f;
#pragma unroll
                for (int j = MAX_TAPS - 1; j >= 1; --j)          // oldest input first
                    if (j < taps) acc = fmaf(wv[ch][j], hist[j - 1][ch], acc);
                acc = fmaf(wv[ch][0], cur[k][ch], acc);
                float v = residual ? cur[k][ch] + acc : acc;
                if (silu) v = silu_f<true>(v);
                y[ch] = v;
            }
            Vec8<TA>::store(out + (size_t)(q0 + lb + k) * ldo + c, y);
#pragma unroll
            for (int j = MAX_TAPS - 1; j >= 2; --j)
#pragma unroll
                for (int ch = 0; ch < 8; ++ch) hist[j - 1][ch] = hist[j - 2][ch];
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) hist[0][ch] = cur[k][ch];
        }
    }
    if (blockIdx.y == 0) {
        float fresh[MAX_TAPS - 1][8];
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i) {
            if (i < taps - 1) {
                const int l = n - (taps - 1) + i;
                if (l >= 0) Vec8<TA>::load(x + (size_t)(q0 + l) * ldx + c, fresh[i]);
                else Vec8<TA>::load(st + (size_t)(l + taps - 1) * C, fresh[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < MAX_TAPS - 1; ++i)
            if (i < taps - 1) Vec8<TA>::store(st + (size_t)i * C, fresh[i]);
    }
}

// ------------------------------------------------------------------------------------------
// The scans, in two kernels.
//
// scan_prepare (a block a token, nothing sequential): everything a token brings to the recurrence
// as 32-bit rows: q and k per q/k head (through SiLU, or made unit vectors with q times D^-1/2),
// v (through SiLU or as it is), and for the delta rule the decays g per head and key channel and
// the write strengths beta.
//
// scan (grid: value-column groups x heads x segments, SCAN_WARPS warps a block): a warp's lanes
// are R row slices x C = 32 / R columns; lane (r, c) owns up to 16 key rows of column c of the
// head's state in registers; sums over the key rows meet by shuffles across the slices (a fixed
// butterfly), and nothing in the walk waits for another warp.  The prepared rows of the segment's
// tokens are copied `stage` at a time into one of two shared-memory buffers (asynchronous copies
// of the next tokens run under the walk over the present ones); a slice's rows start on a
// 16-byte boundary, one bank group after the slice before, and are read four at a time.
// ------------------------------------------------------------------------------------------
constexpr int SCAN_HEAD_DECAY = 0, SCAN_DELTA = 1, SCAN_GATED = 2;      // which recurrence a scan runs
constexpr int SCAN_WARPS = 4;
constexpr int SCAN_ROWS = 16;       // key rows a lane holds at most

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename TA>
__global__ void __launch_bounds__(256)
scan_prepare_kernel(const TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v, long ld,
                    const float* __restrict__ a, const TA* __restrict__ b, long ldb, const float* __restrict__ a_log,
                    const float* __restrict__ dt_bias, float* __restrict__ qf, float* __restrict__ kf,
                    float* __restrict__ gf, float* __restrict__ vf, float* __restrict__ bf, int G, int H, int D, int V,
                    int mode, int silu_inputs, float tau) {
    const bool delta = mode == SCAN_DELTA;
    const size_t t = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int head = warp; head < G; head += 8) {
        const TA* qr = q + t * ld + (size_t)head * D;
        const TA* kr = k + t * ld + (size_t)head * D;
        float sq = 0.f, sk = 0.f;
        for (int i = lane; i < D; i += 32) {
            float qv = to_float(qr[i]), kv = to_float(kr[i]);
            if (silu_inputs) { qv = silu_f<true>(qv); kv = silu_f<true>(kv); }
            sq = fmaf(qv, qv, sq);
            sk = fmaf(kv, kv, sk);
        }
        float fq = 1.f, fk = 1.f;
        if (delta) {                // unit length per head (1e-6 inside the root), q times D^-1/2
            sq = warp_sum(sq); sk = warp_sum(sk);
            fq = (1.f / sqrtf((float)D)) / sqrtf(sq + 1e-6f);
            fk = 1.f / sqrtf(sk + 1e-6f);
        } else if (mode == SCAN_GATED) {
            fq = 1.f / sqrtf((float)D);
        }
        for (int i = lane; i < D; i += 32) {
            float qv = to_float(qr[i]), kv = to_float(kr[i]);
            if (silu_inputs) { qv = silu_f<true>(qv); kv = silu_f<true>(kv); }
            qf[(t * G + head) * D + i] = qv * fq;
            kf[(t * G + head) * D + i] = kv * fk;
        }
    }
    for (int e = tid; e < H * V; e += 256) {
        float vv = to_float(v[t * ld + e]);
        if (silu_inputs) vv = silu_f<true>(vv);
        vf[t * H * V + e] = vv;
    }
    if (delta) {
        for (int e = tid; e < H * D; e += 256) {
            const float step = softplus_f(a[t * H * D + e] + dt_bias[e]);
            gf[t * H * D + e] = expf(-expf(a_log[e / D]) * step);
        }
        for (int e = tid; e < H; e += 256) bf[t * H + e] = 1.f / (1.f + expf(-to_float(b[t * ldb + e])));
    } else if (mode == SCAN_GATED) {    // sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau)
        for (int e = tid; e < H * D; e += 256)
            gf[t * H * D + e] = expf(-softplus_f(-(a[t * H * D + e] + dt_bias[e])) / tau);
    }
}

template <int R> __device__ __forceinline__ float slices_sum(float v) {
#pragma unroll
    for (int o = 16; o >= 32 / R; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void copy_async_4(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

__device__ __forceinline__ void copy_async_16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

template <int R, int MODE, bool FULL>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
scan_kernel(const float* __restrict__ qf, const float* __restrict__ kf, const float* __restrict__ gf,
            const float* __restrict__ vf, const float* __restrict__ bf, const float* __restrict__ decay,
            float* __restrict__ state, float* __restrict__ out, const int* __restrict__ seg_q_start,
            const int* __restrict__ seg_slot, int group, int G, int H, int D, int V, int stage) {
    extern __shared__ __align__(16) float smem[];
    constexpr bool DELTA = MODE == SCAN_DELTA, DECAYS = MODE != SCAN_HEAD_DECAY;     // DECAYS: a decay per key row
    constexpr int C = 32 / R, COLS = SCAN_WARPS * C, THREADS = SCAN_WARPS * 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.y, seg = blockIdx.z;
    const int q0 = seg_q_start[seg], n = seg_q_start[seg + 1] - q0;
    if (n <= 0) return;
    const int r = lane / C, c = lane % C;
    const int col0 = blockIdx.x * COLS, col = col0 + warp * C + c;
    const bool live = col < V;
    const int per = (((D + R - 1) / R) + 3) & ~3;     // rows a slice, a multiple of 4, at most SCAN_ROWS
    const int row0 = r * per;
    const int mine = max(0, min(per, D - row0));
    const int ps = per + 4, Dp = R * ps;              // row i of a staged vector sits at (i / per) * ps + i % per
    const int kh = h / group;                         // the q/k head this head reads
    const int vectors = DECAYS ? 3 : 2;
    const int buffer = stage * (vectors * Dp + COLS) + stage;         // floats of one buffer

    float S[SCAN_ROWS];
    float* st = state + (((size_t)seg_slot[seg] * H + h) * D) * V + col;
#pragma unroll
    for (int i = 0; i < SCAN_ROWS; ++i) S[i] = (live && i < mine) ? st[(size_t)(row0 + i) * V] : 0.f;
    const float head_decay = DECAYS ? 0.f : decay[h];

    auto fetch = [&](int which, int t0) {             // tokens t0 .. of the segment into buffer `which`
        const int m = min(stage, n - t0);
        float* qs = smem + which * buffer;
        float* ks = qs + stage * Dp;
        float* gs = ks + stage * Dp;
        float* vs = qs + vectors * stage * Dp;
        float* bs = vs + stage * COLS;
        if ((D & 3) == 0) {                           // 16 bytes a copy: a slice's rows are a multiple of four
            const int D4 = D >> 2;
            for (int e = tid; e < m * D4; e += THREADS) {
                const int tt = e / D4, i = (e - tt * D4) * 4;
                const size_t row = (size_t)(q0 + t0 + tt);
                const int at = tt * Dp + (i / per) * ps + i % per;
                copy_async_16(qs + at, qf + (row * G + kh) * D + i);
                copy_async_16(ks + at, kf + (row * G + kh) * D + i);
                if constexpr (DECAYS) copy_async_16(gs + at, gf + (row * H + h) * D + i);
            }
        } else {
            for (int e = tid; e < m * D; e += THREADS) {
                const int tt = e / D, i = e - tt * D;
                const size_t row = (size_t)(q0 + t0 + tt);
                const int at = tt * Dp + (i / per) * ps + i % per;
                copy_async_4(qs + at, qf + (row * G + kh) * D + i);
                copy_async_4(ks + at, kf + (row * G + kh) * D + i);
                if constexpr (DECAYS) copy_async_4(gs + at, gf + (row * H + h) * D + i);
            }
        }
        for (int e = tid; e < m * COLS; e += THREADS) {
            const int tt = e / COLS, j = e - tt * COLS;
            if (col0 + j < V) copy_async_4(vs + e, vf + ((size_t)(q0 + t0 + tt) * H + h) * V + col0 + j);
        }
        if constexpr (DELTA)
            if (tid < m) copy_async_4(bs + tid, bf + (size_t)(q0 + t0 + tid) * H + h);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    fetch(0, 0);
    int which = 0;
    for (int t0 = 0; t0 < n; t0 += stage, which ^= 1) {
        const int m = min(stage, n - t0);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                              // these tokens are here; the other buffer has been walked
        if (t0 + stage < n) fetch(which ^ 1, t0 + stage);
        const float* qs = smem + which * buffer + r * ps;
        const float* ks = qs + stage * Dp;
        const float* gs = ks + stage * Dp;
        const float* vs = smem + which * buffer + vectors * stage * Dp + warp * C + c;
        const float* bs = smem + which * buffer + vectors * stage * Dp + stage * COLS;
#pragma unroll 2
        for (int tt = 0; tt < m; ++tt) {
            const float4* q4 = reinterpret_cast<const float4*>(qs + tt * Dp);
            const float4* k4 = reinterpret_cast<const float4*>(ks + tt * Dp);
            const float4* g4 = reinterpret_cast<const float4*>(gs + tt * Dp);
            const float vv = live ? vs[tt * COLS] : 0.f;
            // the slice's rows of k, q (and g) of this token: FULL slices (every lane holds
            // SCAN_ROWS rows) need no bound checks
            float kr[SCAN_ROWS], qr[SCAN_ROWS], gr[SCAN_ROWS];
#pragma unroll
            for (int j = 0; j < SCAN_ROWS / 4; ++j) {
                if (FULL || 4 * j < mine) {
                    const float4 kv = k4[j], qv = q4[j];
                    kr[4 * j] = kv.x; kr[4 * j + 1] = kv.y; kr[4 * j + 2] = kv.z; kr[4 * j + 3] = kv.w;
                    qr[4 * j] = qv.x; qr[4 * j + 1] = qv.y; qr[4 * j + 2] = qv.z; qr[4 * j + 3] = qv.w;
                    if constexpr (DECAYS) {
                        const float4 gv = g4[j];
                        gr[4 * j] = gv.x; gr[4 * j + 1] = gv.y; gr[4 * j + 2] = gv.z; gr[4 * j + 3] = gv.w;
                    }
                }
            }
            float o[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (DELTA) {
                float kd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int i = 0; i < SCAN_ROWS; ++i)
                    if (FULL || i < mine) { S[i] *= gr[i]; kd[i & 3] = fmaf(S[i], kr[i], kd[i & 3]); }
                const float u = bs[tt] * (vv - slices_sum<R>((kd[0] + kd[1]) + (kd[2] + kd[3])));
#pragma unroll
                for (int i = 0; i < SCAN_ROWS; ++i)
                    if (FULL || i < mine) { S[i] = fmaf(kr[i], u, S[i]); o[i & 3] = fmaf(S[i], qr[i], o[i & 3]); }
            } else if constexpr (MODE == SCAN_GATED) {
#pragma unroll
                for (int i = 0; i < SCAN_ROWS; ++i)
                    if (FULL || i < mine) { S[i] = fmaf(gr[i], S[i], kr[i] * vv); o[i & 3] = fmaf(S[i], qr[i], o[i & 3]); }
            } else {
#pragma unroll
                for (int i = 0; i < SCAN_ROWS; ++i)
                    if (FULL || i < mine) { S[i] = fmaf(head_decay, S[i], kr[i] * vv); o[i & 3] = fmaf(S[i], qr[i], o[i & 3]); }
            }
            const float total = slices_sum<R>((o[0] + o[1]) + (o[2] + o[3]));
            if (live && r == 0) out[(size_t)(q0 + t0 + tt) * ((size_t)H * V) + (size_t)h * V + col] = total;
        }
    }
#pragma unroll
    for (int i = 0; i < SCAN_ROWS; ++i)
        if (live && i < mine) st[(size_t)(row0 + i) * V] = S[i];
}

// A warp a (token, group).
template <typename TA>
__global__ void __launch_bounds__(128)
gated_norm_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_len, const TA* __restrict__ gate,
                  long ldg, float eps, TA* __restrict__ out, long pairs, int groups, int n, int gate_silu) {
    const long pair = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (pair >= pairs) return;
    const long t = pair / groups;
    const int g = (int)(pair - t * groups);
    const float* row = o + (t * groups + g) * n;
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)n + eps);
    for (int i = lane; i < n; i += 32) {
        const int c = g * n + i;
        const float gv = to_float(gate[t * ldg + c]);
        out[(t * groups + g) * n + i] = from_float<TA>(row[i] * inv * w[c % w_len] * ((gate_silu ? gv : 1.f) / (1.f + expf(-gv))));
    }
}

// scratch: float32, scan_scratch_floats() of them.
// A block a (token, group), for groups of many features.  The sums differ from the warp kernel's in
// their order; which of the two runs depends on the group's size only.
template <typename TA>
__global__ void __launch_bounds__(256)
gated_norm_block_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_len, const TA* __restrict__ gate,
                        long ldg, float eps, TA* __restrict__ out, int groups, int n, int gate_silu) {
    __shared__ float scratch[33];
    const long pair = blockIdx.x;
    const long t = pair / groups;
    const int g = (int)(pair - t * groups);
    const float* row = o + (t * groups + g) * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) ss = fmaf(row[i], row[i], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += 256) {
        const int c = g * n + i;
        const float gv = to_float(gate[t * ldg + c]);
        out[(t * groups + g) * n + i] = from_float<TA>(row[i] * inv * w[c % w_len] * ((gate_silu ? gv : 1.f) / (1.f + expf(-gv))));
    }
}

template <typename TA, int MODE>
int launch_scan(const void* q, const void* k, const void* v, long ld, int group, const float* a, const void* b,
                long ldb, const float* a_log, const float* dt_bias, const float* decay, float* state, float* out,
                float* scratch, const int* seg_q_start, const int* seg_slot, int segments, int tokens, int H, int D,
                int V, int silu_inputs, float tau, cudaStream_t stream) {
    constexpr bool DECAYS = MODE != SCAN_HEAD_DECAY;
    const int G = H / group;
    float* qf = scratch;
    float* kf = qf + (size_t)tokens * G * D;
    float* gf = kf + (size_t)tokens * G * D;          // the three that are copied 16 bytes at a time first
    float* vf = gf + (DECAYS ? (size_t)tokens * H * D : 0);
    float* bf = vf + (size_t)tokens * H * V;
    scan_prepare_kernel<TA><<<tokens, 256, 0, stream>>>((const TA*)q, (const TA*)k, (const TA*)v, ld, a, (const TA*)b, ldb,
                                                       a_log, dt_bias, qf, kf, gf, vf, bf, G, H, D, V, MODE,
                                                       silu_inputs, tau);
    const int R = D <= 16 ? 1 : D <= 32 ? 2 : D <= 64 ? 4 : D <= 128 ? 8 : 16;   // row slices: at most 16 rows a lane
    const int cols = SCAN_WARPS * (32 / R);
    const int per = (((D + R - 1) / R) + 3) & ~3;
    const int stage = D <= 128 ? 16 : 8;
    const dim3 grid((V + cols - 1) / cols, H, segments);
    const size_t smem = sizeof(float) * 2 * ((size_t)stage * ((DECAYS ? 3 : 2) * R * (per + 4) + cols) + stage);
#define MRUN_SCAN_AS(SLICES, WHOLE)                                                                                 \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(scan_kernel<SLICES, MODE, WHOLE>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                 (int)smem);                                                                       \
        scan_kernel<SLICES, MODE, WHOLE><<<grid, SCAN_WARPS * 32, smem, stream>>>(                                 \
            qf, kf, gf, vf, bf, decay, state, out, seg_q_start, seg_slot, group, G, H, D, V, stage);               \
    } while (0)
#define MRUN_SCAN(SLICES)                                                                                          \
    do {                                                                                                           \
        if (D == SLICES * SCAN_ROWS) MRUN_SCAN_AS(SLICES, true);          /* every lane holds SCAN_ROWS rows */   \
        else MRUN_SCAN_AS(SLICES, false);                                                                          \
    } while (0)
    if (R == 1) MRUN_SCAN(1);
    else if (R == 2) MRUN_SCAN(2);
    else if (R == 4) MRUN_SCAN(4);
    else if (R == 8) MRUN_SCAN(8);
    else MRUN_SCAN(16);
#undef MRUN_SCAN_AS
#undef MRUN_SCAN
    return 0;
}

}  // namespace

// x: row t at x + t * ldx, C channels; w: float32 [C, taps]; state: [slots, taps - 1, C] in the
// activation dtype; out: row t at out + t * ldo.  seg_q_start: int32 [segments + 1].
MRUN_API int mrun_causal_conv(const void* x, long ldx, const float* w, void* state, void* out, long ldo, int act_dtype,
                              const int* seg_q_start, const int* seg_slot, int segments, int max_q_len, int C,
                              int taps, int residual, int silu, cudaStream_t stream) {
    MRUN_REQUIRE(C > 0 && segments >= 0 && max_q_len >= 0, "causal_conv: bad sizes");
    MRUN_REQUIRE(taps >= 1 && taps <= MAX_TAPS, "causal_conv: %d taps, the kernel takes 1 to %d", taps, MAX_TAPS);
    MRUN_REQUIRE(ldx >= C && ldo >= C, "causal_conv: a row stride below the %d channels", C);
    MRUN_REQUIRE(segments <= 65535, "causal_conv: %d segments exceed 65535", segments);
    if (segments == 0 || max_q_len == 0) return 0;
    const int tiles = (max_q_len + CONV_TILE - 1) / CONV_TILE;
    MRUN_REQUIRE(tiles <= 65535, "causal_conv: a segment of %d tokens is too long", max_q_len);
    const size_t unit = act_dtype == MRUN_F32 ? 4 : 2;
    const bool vec = C % 8 == 0 && (ldx * unit) % 16 == 0 && (ldo * unit) % 16 == 0 &&
                     ((((uintptr_t)x) | ((uintptr_t)out) | ((uintptr_t)state)) & 15) == 0 && (C * unit) % 16 == 0;
    if (vec) {
        const dim3 vec_grid((C / 8 + 127) / 128, tiles, segments);
        if (act_dtype == MRUN_F32)
            causal_conv_vec_kernel<float><<<vec_grid, 128, 0, stream>>>((const float*)x, ldx, w, (float*)state, (float*)out,
                                                                         ldo, seg_q_start, seg_slot, C, taps, residual, silu);
        else if (act_dtype == MRUN_BF16)
            causal_conv_vec_kernel<__nv_bfloat16><<<vec_grid, 128, 0, stream>>>(
                (const __nv_bfloat16*)x, ldx, w, (__nv_bfloat16*)state, (__nv_bfloat16*)out, ldo, seg_q_start, seg_slot, C,
                taps, residual, silu);
        else
            return mrun_set_error("causal_conv: unknown dtype code %d", act_dtype);
        MRUN_CHECK_LAUNCH("causal_conv");
        return 0;
    }
    const dim3 grid((C + 127) / 128, tiles, segments);
    if (act_dtype == MRUN_F32)
        causal_conv_kernel<float><<<grid, 128, 0, stream>>>((const float*)x, ldx, w, (float*)state, (float*)out, ldo,
                                                             seg_q_start, seg_slot, C, taps, residual, silu);
    else if (act_dtype == MRUN_BF16)
        causal_conv_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
            (const __nv_bfloat16*)x, ldx, w, (__nv_bfloat16*)state, (__nv_bfloat16*)out, ldo, seg_q_start, seg_slot, C,
            taps, residual, silu);
    else
        return mrun_set_error("causal_conv: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("causal_conv");
    return 0;
}

// q, k: row t at + t * ld, [H / group heads, D]; v: [H, V] likewise.  state: float32 [slots, H, D, V];
// out: float32 [tokens, H * V].  decay: float32 [H].  scratch: float32, mrun_scan_scratch_floats() of them
// (the prepared rows; a token's row of the batch is its row there, padding rows included).
MRUN_API long mrun_scan_scratch_floats(int tokens, int H, int G, int D, int V, int delta) {
    return (long)tokens * (2L * G * D + (long)H * V + (delta ? (long)H * D + H : 0));
}

MRUN_API int mrun_decay_scan(const void* q, const void* k, const void* v, long ld, int act_dtype, const float* decay,
                             float* state, float* out, float* scratch, const int* seg_q_start, const int* seg_slot,
                             int segments, int tokens, int H, int D, int V, int silu_inputs, cudaStream_t stream) {
    MRUN_REQUIRE(H > 0 && D > 0 && V > 0 && segments >= 0, "decay_scan: bad sizes");
    MRUN_REQUIRE(D <= 256, "decay_scan: key size %d exceeds the supported 256", D);
    MRUN_REQUIRE(H <= 65535 && segments <= 65535, "decay_scan: %d heads or %d segments exceed 65535", H, segments);
    if (segments == 0 || tokens == 0) return 0;
    if (act_dtype == MRUN_F32)
        launch_scan<float, SCAN_HEAD_DECAY>(q, k, v, ld, 1, nullptr, nullptr, 0, nullptr, nullptr, decay, state, out, scratch,
                                            seg_q_start, seg_slot, segments, tokens, H, D, V, silu_inputs, 1.f, stream);
    else if (act_dtype == MRUN_BF16)
        launch_scan<__nv_bfloat16, SCAN_HEAD_DECAY>(q, k, v, ld, 1, nullptr, nullptr, 0, nullptr, nullptr, decay, state, out,
                                                    scratch, seg_q_start, seg_slot, segments, tokens, H, D, V, silu_inputs,
                                                    1.f, stream);
    else
        return mrun_set_error("decay_scan: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("decay_scan");
    return 0;
}

// q, k: [H / group heads, D] a row (stride ld); v: [H, V] (stride ld); a: float32 [tokens, H * D];
// b: row t at b + t * ldb, [H]; a_log: float32 [H]; dt_bias: float32 [H * D].
MRUN_API int mrun_delta_scan(const void* q, const void* k, const void* v, long ld, int act_dtype, int group,
                             const float* a, const void* b, long ldb, const float* a_log, const float* dt_bias,
                             float* state, float* out, float* scratch, const int* seg_q_start, const int* seg_slot,
                             int segments, int tokens, int H, int D, int V, cudaStream_t stream) {
    MRUN_REQUIRE(H > 0 && D > 0 && V > 0 && segments >= 0 && group > 0 && H % group == 0, "delta_scan: bad sizes");
    MRUN_REQUIRE(D <= 256, "delta_scan: key size %d exceeds the supported 256", D);
    MRUN_REQUIRE(H <= 65535 && segments <= 65535, "delta_scan: %d heads or %d segments exceed 65535", H, segments);
    if (segments == 0 || tokens == 0) return 0;
    if (act_dtype == MRUN_F32)
        launch_scan<float, SCAN_DELTA>(q, k, v, ld, group, a, b, ldb, a_log, dt_bias, nullptr, state, out, scratch,
                                       seg_q_start, seg_slot, segments, tokens, H, D, V, 0, 1.f, stream);
    else if (act_dtype == MRUN_BF16)
        launch_scan<__nv_bfloat16, SCAN_DELTA>(q, k, v, ld, group, a, b, ldb, a_log, dt_bias, nullptr, state, out, scratch,
                                               seg_q_start, seg_slot, segments, tokens, H, D, V, 0, 1.f, stream);
    else
        return mrun_set_error("delta_scan: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("delta_scan");
    return 0;
}

// q, k: [H, D] a row (stride ld); v: [H, V] (stride ld); a: float32 [tokens, H * D], the decay
// projection's output; bias: float32 [H * D]; the decay is sigmoid(a + bias)^(1 / tau).
MRUN_API int mrun_gated_scan(const void* q, const void* k, const void* v, long ld, int act_dtype, const float* a,
                             const float* bias, float tau, float* state, float* out, float* scratch,
                             const int* seg_q_start, const int* seg_slot, int segments, int tokens, int H, int D, int V,
                             cudaStream_t stream) {
    MRUN_REQUIRE(H > 0 && D > 0 && V > 0 && segments >= 0 && tau > 0.f, "gated_scan: bad sizes");
    MRUN_REQUIRE(D <= 256, "gated_scan: key size %d exceeds the supported 256", D);
    MRUN_REQUIRE(H <= 65535 && segments <= 65535, "gated_scan: %d heads or %d segments exceed 65535", H, segments);
    if (segments == 0 || tokens == 0) return 0;
    if (act_dtype == MRUN_F32)
        launch_scan<float, SCAN_GATED>(q, k, v, ld, 1, a, nullptr, 0, nullptr, bias, nullptr, state, out, scratch,
                                       seg_q_start, seg_slot, segments, tokens, H, D, V, 0, tau, stream);
    else if (act_dtype == MRUN_BF16)
        launch_scan<__nv_bfloat16, SCAN_GATED>(q, k, v, ld, 1, a, nullptr, 0, nullptr, bias, nullptr, state, out, scratch,
                                               seg_q_start, seg_slot, segments, tokens, H, D, V, 0, tau, stream);
    else
        return mrun_set_error("gated_scan: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("gated_scan");
    return 0;
}

// o: float32 [tokens, groups * n]; w: float32 [w_len], element c of a row takes w[c % w_len];
// gate: row t at gate + t * ldg; out: dense [tokens, groups * n].  gate_silu: the gate passes SiLU
// instead of the sigmoid.
MRUN_API int mrun_gated_norm(const float* o, const float* w, int w_len, const void* gate, long ldg, int act_dtype,
                             float eps, void* out, int tokens, int groups, int n, int gate_silu, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && groups > 0 && n > 0 && w_len > 0, "gated_norm: bad sizes");
    MRUN_REQUIRE(ldg >= (long)groups * n, "gated_norm: the gate's row stride %ld is below the row", ldg);
    if (tokens == 0) return 0;
    const long pairs = (long)tokens * groups;
    const unsigned blocks = (unsigned)((pairs + 3) / 4);
    if (n >= 1024) {            // a block a pair
        if (act_dtype == MRUN_F32)
            gated_norm_block_kernel<float><<<(unsigned)pairs, 256, 0, stream>>>(o, w, w_len, (const float*)gate, ldg, eps,
                                                                                 (float*)out, groups, n, gate_silu);
        else if (act_dtype == MRUN_BF16)
            gated_norm_block_kernel<__nv_bfloat16><<<(unsigned)pairs, 256, 0, stream>>>(
                o, w, w_len, (const __nv_bfloat16*)gate, ldg, eps, (__nv_bfloat16*)out, groups, n, gate_silu);
        else
            return mrun_set_error("gated_norm: unknown dtype code %d", act_dtype);
        MRUN_CHECK_LAUNCH("gated_norm");
        return 0;
    }
    if (act_dtype == MRUN_F32)
        gated_norm_kernel<float><<<blocks, 128, 0, stream>>>(o, w, w_len, (const float*)gate, ldg, eps, (float*)out,
                                                              pairs, groups, n, gate_silu);
    else if (act_dtype == MRUN_BF16)
        gated_norm_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(o, w, w_len, (const __nv_bfloat16*)gate, ldg, eps,
                                                                      (__nv_bfloat16*)out, pairs, groups, n, gate_silu);
    else
        return mrun_set_error("gated_norm: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("gated_norm");
    return 0;
}
