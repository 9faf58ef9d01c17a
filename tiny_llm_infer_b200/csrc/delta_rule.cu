// The delta rule with a decay per head and key channel, as a recurrence over a state S [dk, dv] per
// (request, head) that lives in float32 and is carried from step to step:
//
//   S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t.
//
// Three kernels serve a step, prompt portions and single tokens alike:
//
//   delta_prepare  one block per token: the short causal convolution of the q, k and v channels (taps
//                  reaching before the portion come from the request's state), SiLU, unit length of q
//                  and k per head (q times a scale), g = exp(-rate_h softplus(a + bias)) and
//                  beta = sigmoid(b); all results in float32.
//   delta_scan     one block per (portion, head, group of value columns): a column of S is independent of
//                  the others, so a thread keeps a slice of one column in registers (the dk rows are dealt
//                  to R neighbouring lanes, which add their partial dot products with shuffles) and walks
//                  the portion's tokens, which come through two stages of shared memory sixteen at a time
//                  (cp.async: the next sixteen are on their way while these are walked).
//   delta_finish   one block per token: o divided by its root mean square per head, times a weight, times
//                  sigmoid(gate); the block of a portion's last token also moves the convolution's
//                  window of the request's state on.
//
// State of a request: [heads][per][dv][R] floats of S (row i = r * per + il; rows past dk stay zero), then
// [taps - 1][channels] inputs of the convolution, the newest last.  R and per follow from dk alone
// (`tllm_delta_rule_lanes`), so every step of a request finds the layout the last one left.
#include "common.cuh"

namespace tllm {

constexpr int kScanMaxPer = 16;     // rows of a column that one thread keeps
constexpr int kScanChunk = 16;      // tokens staged at a time

static inline int delta_lanes(int dk) {
    int r = 4;
    while (r < 32 && (dk + r - 1) / r > kScanMaxPer) r *= 2;
    return r;
}

__device__ __forceinline__ float softplus_f32(float x) {
    return x > 20.0f ? x : log1pf(expf(x));
}

// ---------------------------------------------------------------- prepare
template <typename T>
__global__ void delta_prepare_kernel(const T* proj, int ld, const T* __restrict__ conv_w, int taps,
                                     const float* a, int lda, const float* __restrict__ dt_bias,
                                     const float* __restrict__ rate, const int* __restrict__ token_slot,
                                     const float* state, long long state_stride, long long tail_off,
                                     int heads, int kv_heads, int dk, int dv, float q_scale, float unit_eps,
                                     float* qn, float* kn, float* vv, float* decay, float* beta, int n_rows,
                                     int decay_per_head, int beta_col) {
    extern __shared__ float y[];                 // [channels] after convolution and SiLU
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int qk = kv_heads * dk, channels = 2 * qk + heads * dv;
    int back = 0;                                // rows before this one that belong to the same portion
    for (int j = 1; j < taps; ++j) {
        if (t - j >= 0 && token_slot[t - j] == slot) back = j;
        else break;
    }
    const float* tail = state + (long long)slot * state_stride + tail_off;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const float w = to_f32<T>(conv_w[(size_t)c * taps + (taps - 1 - j)]);
            float x;
            if (j <= back) x = to_f32<T>(proj[(size_t)(t - j) * ld + c]);
            else x = tail[(size_t)(taps - 1 - (j - back)) * channels + c];
            acc += w * x;
        }
        y[c] = acc / (1.0f + expf(-acc));
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int u = warp; u < 2 * kv_heads; u += warps) {          // q heads, then k heads
        const float* src = y + (size_t)u * dk;
        float sum = 0.0f;
        for (int e = lane; e < dk; e += 32) sum += src[e] * src[e];
        sum = warp_sum(sum);
        const bool is_q = u < kv_heads;
        const float sc = (is_q ? q_scale : 1.0f) / sqrtf(sum + unit_eps);
        float* dst = is_q ? qn + (size_t)t * qk + (size_t)u * dk : kn + (size_t)t * qk + (size_t)(u - kv_heads) * dk;
        for (int e = lane; e < dk; e += 32) dst[e] = src[e] * sc;
    }
    for (int e = threadIdx.x; e < heads * dv; e += blockDim.x) vv[(size_t)t * heads * dv + e] = y[2 * qk + e];
    for (int e = threadIdx.x; e < heads * dk; e += blockDim.x) {
        const int ai = decay_per_head ? e / dk : e;          // one decay per head serves all its key channels
        const float x = a[(size_t)t * lda + ai] + dt_bias[ai];
        decay[(size_t)t * heads * dk + e] = expf(-rate[e / dk] * softplus_f32(x));
    }
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        const float b = to_f32<T>(proj[(size_t)t * ld + beta_col + h]);
        beta[(size_t)t * heads + h] = 1.0f / (1.0f + expf(-b));
    }
}

// 8-element accesses of either storage type (the convolution's inputs and taps), and of float32
template <typename T> struct Ld8;
template <> struct Ld8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Ld8<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};

// The same with eight channels per thread and access (rows of proj, the taps as [taps][channels], dk and dv
// multiples of eight, everything on 16-byte boundaries).
// TAPS: the number of taps if it is 2, 3 or 4 (their loads are then all issued before the first product), 0 for
// any other number.
template <typename T, int TAPS>
__global__ void delta_prepare_vec_kernel(const T* proj, int ld, const T* __restrict__ conv_t, int taps,
                                         const float* a, int lda, const float* __restrict__ dt_bias,
                                         const float* __restrict__ rate, const int* __restrict__ token_slot,
                                         const float* state, long long state_stride, long long tail_off,
                                         int heads, int kv_heads, int dk, int dv, float q_scale, float unit_eps,
                                         float* qn, float* kn, float* vv, float* decay, float* beta, int n_rows,
                                         int decay_per_head, int beta_col) {
    extern __shared__ __align__(16) float y[];   // [2 * kv_heads * dk] q and k after convolution and SiLU
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int qk = kv_heads * dk, channels = 2 * qk + heads * dv;
    int back = 0;
    for (int j = 1; j < taps; ++j) {
        if (t - j >= 0 && token_slot[t - j] == slot) back = j;
        else break;
    }
    const float* tail = state + (long long)slot * state_stride + tail_off;
    // With few rows a token's work is dealt to gridDim.y blocks: whole q and k heads (their norms need the
    // head together), an even share of the v channels, of the decays, and the betas to the first.
    const int Y = gridDim.y, yb = blockIdx.y;
    const int u0 = (2 * kv_heads * yb) / Y, u1 = (2 * kv_heads * (yb + 1)) / Y;         // q heads, then k heads
    const int vc = heads * dv / 8, v0 = 2 * qk + (vc * yb / Y) * 8, v1 = 2 * qk + (vc * (yb + 1) / Y) * 8;
    auto conv8 = [&](int c, float (&acc)[8]) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
        if (TAPS > 0) {
            float w[TAPS > 0 ? TAPS : 1][8], x[TAPS > 0 ? TAPS : 1][8];
#pragma unroll
            for (int j = 0; j < TAPS; ++j) {
                Ld8<T>::load(conv_t + (size_t)(TAPS - 1 - j) * channels + c, w[j]);
                if (j <= back) Ld8<T>::load(proj + (size_t)(t - j) * ld + c, x[j]);
                else Ld8<float>::load(tail + (size_t)(TAPS - 1 - (j - back)) * channels + c, x[j]);
            }
#pragma unroll
            for (int j = 0; j < TAPS; ++j)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] += w[j][e] * x[j][e];
        } else {
            for (int j = 0; j < taps; ++j) {
                float w[8], x[8];
                Ld8<T>::load(conv_t + (size_t)(taps - 1 - j) * channels + c, w);
                if (j <= back) Ld8<T>::load(proj + (size_t)(t - j) * ld + c, x);
                else Ld8<float>::load(tail + (size_t)(taps - 1 - (j - back)) * channels + c, x);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] += w[e] * x[e];
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = acc[e] / (1.0f + expf(-acc[e]));
    };
    for (int c = u0 * dk + threadIdx.x * 8; c < u1 * dk; c += blockDim.x * 8) {
        float acc[8];
        conv8(c, acc);
        Ld8<float>::store(y + (c - u0 * dk), acc);
    }
    for (int c = v0 + threadIdx.x * 8; c < v1; c += blockDim.x * 8) {
        float acc[8];
        conv8(c, acc);
        Ld8<float>::store(vv + (size_t)t * heads * dv + (c - 2 * qk), acc);
    }
    const int dq = heads * dk / 4, e0 = (dq * yb / Y) * 4, e1 = (dq * (yb + 1) / Y) * 4;
    for (int e = e0 + threadIdx.x * 4; e < e1; e += blockDim.x * 4) {
        float4 x, b;
        if (decay_per_head) {                        // dk is a multiple of eight: the four share a head
            const float xa = a[(size_t)t * lda + e / dk], xb = dt_bias[e / dk];
            x = make_float4(xa, xa, xa, xa);
            b = make_float4(xb, xb, xb, xb);
        } else {
            x = *reinterpret_cast<const float4*>(a + (size_t)t * lda + e);
            b = *reinterpret_cast<const float4*>(dt_bias + e);
        }
        const float rt = rate[e / dk];
        float4 g;
        g.x = expf(-rt * softplus_f32(x.x + b.x)); g.y = expf(-rt * softplus_f32(x.y + b.y));
        g.z = expf(-rt * softplus_f32(x.z + b.z)); g.w = expf(-rt * softplus_f32(x.w + b.w));
        *reinterpret_cast<float4*>(decay + (size_t)t * heads * dk + e) = g;
    }
    if (yb == 0)
        for (int h = threadIdx.x; h < heads; h += blockDim.x) {
            const float b = to_f32<T>(proj[(size_t)t * ld + beta_col + h]);
            beta[(size_t)t * heads + h] = 1.0f / (1.0f + expf(-b));
        }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int u = u0 + warp; u < u1; u += warps) {
        const float* src = y + (size_t)(u - u0) * dk;
        float sum = 0.0f;
        for (int e = lane * 4; e < dk; e += 128) {
            const float4 v = *reinterpret_cast<const float4*>(src + e);
            sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        sum = warp_sum(sum);
        const bool is_q = u < kv_heads;
        const float sc = (is_q ? q_scale : 1.0f) / sqrtf(sum + unit_eps);
        float* dst = is_q ? qn + (size_t)t * qk + (size_t)u * dk : kn + (size_t)t * qk + (size_t)(u - kv_heads) * dk;
        for (int e = lane * 4; e < dk; e += 128) {
            float4 v = *reinterpret_cast<const float4*>(src + e);
            v.x *= sc; v.y *= sc; v.z *= sc; v.w *= sc;
            *reinterpret_cast<float4*>(dst + e) = v;
        }
    }
}

// ---------------------------------------------------------------- scan
template <int R>
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = R / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void cp_async_f32(float* dst, const float* src, bool valid) {
    const int bytes = valid ? 4 : 0;                 // zero fill where there is nothing to read
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_f32x4(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

// A lane r of a column keeps the rows i = r * per + il, il < per, as PER registers; in shared memory a token's
// k (and q, g) row is laid out [R][PER + 4]: a lane's rows are neighbours, so it reads them four at a time, and
// the four floats between the lanes' runs keep those reads off each other's banks.
template <int R, int PER>
struct ScanLayout {
    static constexpr int kRow = R * (PER + 4);                               // floats of one token's k (or q, g) row
    __host__ __device__ static constexpr int stage_floats(int cols) {       // k, q, g, the value columns, the betas, the keeps
        return (kScanChunk * (3 * kRow + cols + 2) + 3) / 4 * 4;
    }
};

// R lanes share a column, each keeps PER rows of it at most.  The chunks of tokens come through two stages
// filled by cp.async, so that the next chunk is on its way while this one is walked.  A token's step, per
// thread: S <- g S, dot = sum S k, u = beta (v - dot), S <- S + k u, o = sum S q.  Only S is carried from token
// to token; the read-out's sum is off that path.
//
// MODE picks the recurrence.  kScanDelta: the delta rule above.  kScanPlain: no correction, S <- g S + k (b v)^T with
// the write strength b (one where `beta` is null).  kScanMemory: a matrix memory whose two gates come as logarithms
// (`beta` the write's, `fgate` the keep's) and are held under a running maximum m kept per column in the request's
// state at `aux_off`: m' = max(f + m, i), S <- exp(f + m - m') S + exp(i - m') k v^T; its last value column is the
// normaliser (the prepare kernel feeds it ones), whose read-out leaves as max(|n . q|, exp(-m')) + floor_eps in
// `den` while the other columns go to o_raw [., heads, dv - 1].  kScanHeadDecay: kScanPlain with one decay per
// (token, head) for all rows of S and a write strength likewise, S <- a S + k (w v)^T; the decays come in `beta`
// [., heads], the strengths in `fgate` [., heads], and `decay` is not read.
enum ScanMode : int { kScanDelta = 0, kScanPlain = 1, kScanMemory = 2, kScanHeadDecay = 3 };

template <int R, int PER, int MODE>
__global__ void __launch_bounds__(256, 2)
delta_scan_kernel(const int* __restrict__ seg_info, const int* __restrict__ token_slot,
                  const float* qn, const float* kn, const float* vv, const float* decay,
                  const float* beta, float* state, long long state_stride, int heads,
                  int kv_heads, int dk, int dv, int cols, int vec, float* o_raw,
                  const float* fgate, long long aux_off, float floor_eps, float* den) {
    extern __shared__ __align__(16) float sm[];
    using L = ScanLayout<R, PER>;
    constexpr int kLane = PER + 4;
    TLLM_PDL_ENTER();
    const int seg = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * cols;
    int slot, start, len;
    if (seg_info != nullptr) {
        slot = seg_info[4 * seg]; start = seg_info[4 * seg + 1]; len = seg_info[4 * seg + 2];
    } else {
        slot = token_slot[seg]; start = seg; len = 1;
    }
    if (slot < 0 || len <= 0) return;
    const int per = (dk + R - 1) / R;
    const int r = threadIdx.x % R, jl = threadIdx.x / R;       // lane of the column, column of the block
    const int j = col0 + jl;
    const bool live = j < dv;
    const int kvh = head / (heads / kv_heads);
    const int stage_floats = L::stage_floats(cols);
    float* o_s = sm + 2 * stage_floats;               // [chunk][cols]
    // rows that no copy writes (past per in a lane, past dk in the last lanes) are zeros: they add nothing
    if (per < PER || dk < R * per) {
        for (int i = threadIdx.x; i < 2 * stage_floats; i += blockDim.x) sm[i] = 0.0f;
        __syncthreads();
    }

    auto issue = [&](int c0, int st) {
        const int n = min(kScanChunk, len - c0);
        float* k_s = sm + st * stage_floats;
        float* q_s = k_s + kScanChunk * L::kRow;
        float* g_s = q_s + kScanChunk * L::kRow;
        float* v_s = g_s + kScanChunk * L::kRow;
        float* b_s = v_s + kScanChunk * cols;
        float* f_s = b_s + kScanChunk;
        if (vec) {                                    // dk and per multiples of four: four rows of one lane at a time
            const int quads = dk >> 2;
            for (int i = threadIdx.x; i < n * quads; i += blockDim.x) {
                const int tt = i / quads, e = (i - tt * quads) * 4;
                const int at = tt * L::kRow + (e / per) * kLane + e % per;
                const size_t row = (size_t)(start + c0 + tt);
                cp_async_f32x4(k_s + at, kn + (row * kv_heads + kvh) * dk + e);
                cp_async_f32x4(q_s + at, qn + (row * kv_heads + kvh) * dk + e);
                if (MODE == kScanDelta || MODE == kScanPlain) cp_async_f32x4(g_s + at, decay + (row * heads + head) * dk + e);
            }
        } else {
            for (int i = threadIdx.x; i < n * dk; i += blockDim.x) {
                const int tt = i / dk, e = i - tt * dk;
                const int at = tt * L::kRow + (e / per) * kLane + e % per;
                const size_t row = (size_t)(start + c0 + tt);
                cp_async_f32(k_s + at, kn + (row * kv_heads + kvh) * dk + e, true);
                cp_async_f32(q_s + at, qn + (row * kv_heads + kvh) * dk + e, true);
                if (MODE == kScanDelta || MODE == kScanPlain) cp_async_f32(g_s + at, decay + (row * heads + head) * dk + e, true);
            }
        }
        for (int i = threadIdx.x; i < n * cols; i += blockDim.x) {
            const int tt = i / cols, e = i - tt * cols;
            const bool in = col0 + e < dv;
            cp_async_f32(v_s + i, vv + ((size_t)(start + c0 + tt) * heads + head) * dv + (in ? col0 + e : 0), in);
        }
        if (beta != nullptr)
            for (int i = threadIdx.x; i < n; i += blockDim.x)
                cp_async_f32(b_s + i, beta + (size_t)(start + c0 + i) * heads + head, true);
        if (MODE == kScanMemory || MODE == kScanHeadDecay)
            for (int i = threadIdx.x; i < n; i += blockDim.x)
                cp_async_f32(f_s + i, fgate + (size_t)(start + c0 + i) * heads + head, true);
        asm volatile("cp.async.commit_group;\n" ::);
    };

    issue(0, 0);
    // in the request's state the element (row r * per + il, column j) lies at [il][j][r]: a warp reads whole lines
    float* st_ptr = state + (long long)slot * state_stride + (size_t)head * per * dv * R;
    float2 S2[PER / 2];                               // rows il = 2 p and 2 p + 1 of this lane
#pragma unroll
    for (int il = 0; il < PER; il += 2) {
        S2[il >> 1].x = (live && il < per) ? st_ptr[((size_t)il * dv + j) * R + r] : 0.0f;
        S2[il >> 1].y = (live && il + 1 < per) ? st_ptr[((size_t)(il + 1) * dv + j) * R + r] : 0.0f;
    }

    float* top_ptr = state + (long long)slot * state_stride + aux_off + (size_t)head * dv + j;
    float top = (MODE == kScanMemory && live) ? *top_ptr : 0.0f;      // running maximum of the gates' logarithms
    const bool has_beta = beta != nullptr;
    int stage = 0;
    for (int c0 = 0; c0 < len; c0 += kScanChunk, stage ^= 1) {
        const int n = min(kScanChunk, len - c0);
        if (c0 + kScanChunk < len) {
            issue(c0 + kScanChunk, stage ^ 1);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        const float* k_s = sm + stage * stage_floats;
        const float* q_s = k_s + kScanChunk * L::kRow;
        const float* g_s = q_s + kScanChunk * L::kRow;
        const float* v_s = g_s + kScanChunk * L::kRow;
        const float* b_s = v_s + kScanChunk * cols;
        const float* f_s = b_s + kScanChunk;
        // every thread walks the tokens (the shuffles want whole warps); one without a column carries zeros
        // two rows at a time with the packed float32 instructions of sm_100 (each half rounds as the scalar
        // instruction would): Sg = S g, dot += Sg k, S = Sg + k u, o += S q: four instructions for two rows
        auto step = [&](int tt) -> float {
            const float4* kr = reinterpret_cast<const float4*>(k_s + tt * L::kRow + r * kLane);
            const float4* qr = reinterpret_cast<const float4*>(q_s + tt * L::kRow + r * kLane);
            const float4* gr = reinterpret_cast<const float4*>(g_s + tt * L::kRow + r * kLane);
            float2 kk[PER / 2];
            float2 dot_a = make_float2(0.0f, 0.0f), dot_b = dot_a;
            float write = 1.0f;
            float2 keep2 = make_float2(1.0f, 1.0f);
            if (MODE == kScanMemory) {
                const float fi = f_s[tt], ii = b_s[tt];
                const float top_new = fmaxf(fi + top, ii);
                const float keep = expf(fi + top - top_new);
                write = expf(ii - top_new);
                top = top_new;
                keep2 = make_float2(keep, keep);
            } else if (MODE == kScanPlain) {
                write = has_beta ? b_s[tt] : 1.0f;
            } else if (MODE == kScanHeadDecay) {
                keep2 = make_float2(b_s[tt], b_s[tt]);
                write = f_s[tt];
            }
#pragma unroll
            for (int il = 0; il < PER; il += 4) {
                const float4 k4 = kr[il >> 2];
                kk[il >> 1] = make_float2(k4.x, k4.y);
                kk[(il >> 1) + 1] = make_float2(k4.z, k4.w);
                if (MODE == kScanMemory || MODE == kScanHeadDecay) {
                    S2[il >> 1] = __fmul2_rn(S2[il >> 1], keep2);
                    S2[(il >> 1) + 1] = __fmul2_rn(S2[(il >> 1) + 1], keep2);
                } else {
                    const float4 g4 = gr[il >> 2];
                    S2[il >> 1] = __fmul2_rn(S2[il >> 1], make_float2(g4.x, g4.y));
                    S2[(il >> 1) + 1] = __fmul2_rn(S2[(il >> 1) + 1], make_float2(g4.z, g4.w));
                }
                if (MODE == kScanDelta) {
                    dot_a = __ffma2_rn(S2[il >> 1], kk[il >> 1], dot_a);
                    dot_b = __ffma2_rn(S2[(il >> 1) + 1], kk[(il >> 1) + 1], dot_b);
                }
            }
            float u;
            if (MODE == kScanDelta) {
                const float2 dsum = __fadd2_rn(dot_a, dot_b);
                const float dot = lanes_sum<R>(dsum.x + dsum.y);
                u = b_s[tt] * (v_s[tt * cols + jl] - dot);
            } else {
                u = write * v_s[tt * cols + jl];
            }
            const float2 u2 = make_float2(u, u);
            float2 o_a = make_float2(0.0f, 0.0f), o_b = o_a;
#pragma unroll
            for (int il = 0; il < PER; il += 4) {
                const float4 q4 = qr[il >> 2];
                S2[il >> 1] = __ffma2_rn(kk[il >> 1], u2, S2[il >> 1]);
                S2[(il >> 1) + 1] = __ffma2_rn(kk[(il >> 1) + 1], u2, S2[(il >> 1) + 1]);
                o_a = __ffma2_rn(S2[il >> 1], make_float2(q4.x, q4.y), o_a);
                o_b = __ffma2_rn(S2[(il >> 1) + 1], make_float2(q4.z, q4.w), o_b);
            }
            const float2 osum = __fadd2_rn(o_a, o_b);
            const float o = lanes_sum<R>(osum.x + osum.y);
            if (MODE == kScanMemory && j == dv - 1) return fmaxf(fabsf(o), expf(-top)) + floor_eps;
            return o;
        };
        if (n == kScanChunk) {
            // a whole chunk: unrolled, the read-outs kept in registers until the end, so that no store to shared
            // memory stands between a token's loads and the next one's and they can be issued ahead
            float o_reg[kScanChunk];
#pragma unroll
            for (int tt = 0; tt < kScanChunk; ++tt) o_reg[tt] = step(tt);
            if (r == 0) {
#pragma unroll
                for (int tt = 0; tt < kScanChunk; ++tt) o_s[tt * cols + jl] = o_reg[tt];
            }
        } else {
            for (int tt = 0; tt < n; ++tt) {
                const float oq = step(tt);
                if (r == 0) o_s[tt * cols + jl] = oq;
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < n * cols; i += blockDim.x) {
            const int tt = i / cols, e = i - tt * cols;
            const size_t at = (size_t)(start + c0 + tt) * heads + head;
            if (MODE == kScanMemory) {
                if (col0 + e < dv - 1) o_raw[at * (dv - 1) + col0 + e] = o_s[i];
                else if (col0 + e == dv - 1) den[at] = o_s[i];
            } else if (col0 + e < dv) {
                o_raw[at * dv + col0 + e] = o_s[i];
            }
        }
    }
    if (MODE == kScanMemory && live && r == 0) *top_ptr = top;
    if (live) {
#pragma unroll
        for (int il = 0; il < PER; il += 2) {
            if (il < per) st_ptr[((size_t)il * dv + j) * R + r] = S2[il >> 1].x;
            if (il + 1 < per) st_ptr[((size_t)(il + 1) * dv + j) * R + r] = S2[il >> 1].y;
        }
    }
}

// ---------------------------------------------------------------- finish
// gate_act: 0 sigmoid(gate), 1 SiLU(gate).  weight_stride: 0 where the heads share one weight of dv numbers, dv
// where every head has its own.  den: a divisor per (token, head) applied before the root mean square, or null.
__device__ __forceinline__ float finish_gate(float g, int act) {
    const float sg = 1.0f / (1.0f + expf(-g));
    return act == 1 ? g * sg : sg;
}

template <typename T, typename TG>
__global__ void delta_finish_kernel(const float* o_raw, const TG* gate, int ldg, const float* __restrict__ weight,
                                    float eps, const int* __restrict__ token_slot, int n_rows, int heads, int dv,
                                    T* out, const T* proj, int ld, int channels, int taps, float* state,
                                    long long state_stride, long long tail_off, const float* den, int gate_act,
                                    int weight_stride) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    if (slot < 0) {
        for (int e = threadIdx.x; e < heads * dv; e += blockDim.x) out[(size_t)t * heads * dv + e] = from_f32<T>(0.0f);
        return;
    }
    for (int h = warp; h < heads; h += warps) {
        const float* src = o_raw + ((size_t)t * heads + h) * dv;
        const float dn = den != nullptr ? den[(size_t)t * heads + h] : 1.0f;
        float sum = 0.0f;
        for (int e = lane; e < dv; e += 32) { const float x = src[e] / dn; sum += x * x; }
        sum = warp_sum(sum);
        const float sc = 1.0f / sqrtf(sum / (float)dv + eps);
        for (int e = lane; e < dv; e += 32) {
            const float g = to_f32<TG>(gate[(size_t)t * ldg + (size_t)h * dv + e]);
            out[((size_t)t * heads + h) * dv + e] =
                from_f32<T>(src[e] / dn * sc * weight[(size_t)h * weight_stride + e] * finish_gate(g, gate_act));
        }
    }
    // the portion's last row moves the convolution's window on: its taps - 1 newest inputs
    if (taps > 1 && (t + 1 >= n_rows || token_slot[t + 1] != slot)) {
        int len = 1;                                 // rows of the portion, as far as the window reaches
        while (len < taps - 1 && t - len >= 0 && token_slot[t - len] == slot) ++len;
        float* tail = state + (long long)slot * state_stride + tail_off;
        const int keep = taps - 1;
        for (int c = threadIdx.x; c < channels; c += blockDim.x) {
            for (int i = 0; i < keep; ++i) {         // ascending: an old entry is read before its place is written
                const int from_end = keep - i;       // this entry is the from_end-th newest input
                float x;
                if (from_end <= len) x = to_f32<T>(proj[(size_t)(t + 1 - from_end) * ld + c]);
                else x = tail[(size_t)(i + len) * channels + c];
                tail[(size_t)i * channels + c] = x;
            }
        }
    }
}

// The same with four elements per lane and access, and the window of the convolution moved eight channels at a
// time (dv a multiple of four, channels and the rows of proj multiples of eight, 16-byte boundaries).
template <typename TG> __device__ __forceinline__ float4 load_gate4(const TG* p);
template <> __device__ __forceinline__ float4 load_gate4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load_gate4<bf16>(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <typename T, typename TG>
__global__ void delta_finish_vec_kernel(const float* o_raw, const TG* gate, int ldg, const float* __restrict__ weight,
                                        float eps, const int* __restrict__ token_slot, int n_rows, int heads, int dv,
                                        T* out, const T* proj, int ld, int channels, int taps, float* state,
                                        long long state_stride, long long tail_off, const float* den, int gate_act,
                                        int weight_stride) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    if (slot < 0) {
        for (int e = threadIdx.x; e < heads * dv; e += blockDim.x) out[(size_t)t * heads * dv + e] = from_f32<T>(0.0f);
        return;
    }
    const int Y = gridDim.y, yb = blockIdx.y;          // with few rows a token's heads and channels are dealt to gridDim.y blocks
    for (int h = heads * yb / Y + warp; h < heads * (yb + 1) / Y; h += warps) {
        const float* src = o_raw + ((size_t)t * heads + h) * dv;
        const float dn = den != nullptr ? den[(size_t)t * heads + h] : 1.0f;
        float sum = 0.0f;
        for (int e = lane * 4; e < dv; e += 128) {
            float4 v = *reinterpret_cast<const float4*>(src + e);
            v.x /= dn; v.y /= dn; v.z /= dn; v.w /= dn;
            sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        sum = warp_sum(sum);
        const float sc = 1.0f / sqrtf(sum / (float)dv + eps);
        for (int e = lane * 4; e < dv; e += 128) {
            const float4 v = *reinterpret_cast<const float4*>(src + e);
            const float4 g = load_gate4<TG>(gate + (size_t)t * ldg + (size_t)h * dv + e);
            const float4 w = *reinterpret_cast<const float4*>(weight + (size_t)h * weight_stride + e);
            T* dst = out + ((size_t)t * heads + h) * dv + e;
            dst[0] = from_f32<T>(v.x / dn * sc * w.x * finish_gate(g.x, gate_act));
            dst[1] = from_f32<T>(v.y / dn * sc * w.y * finish_gate(g.y, gate_act));
            dst[2] = from_f32<T>(v.z / dn * sc * w.z * finish_gate(g.z, gate_act));
            dst[3] = from_f32<T>(v.w / dn * sc * w.w * finish_gate(g.w, gate_act));
        }
    }
    if (taps > 1 && (t + 1 >= n_rows || token_slot[t + 1] != slot)) {
        int len = 1;
        while (len < taps - 1 && t - len >= 0 && token_slot[t - len] == slot) ++len;
        float* tail = state + (long long)slot * state_stride + tail_off;
        const int keep = taps - 1;
        const int cc = channels / 8;
        for (int c = (cc * yb / Y) * 8 + threadIdx.x * 8; c < (cc * (yb + 1) / Y) * 8; c += blockDim.x * 8) {
            for (int i = 0; i < keep; ++i) {         // ascending: an old entry is read before its place is written
                const int from_end = keep - i;
                float x[8];
                if (from_end <= len) Ld8<T>::load(proj + (size_t)(t + 1 - from_end) * ld + c, x);
                else Ld8<float>::load(tail + (size_t)(i + len) * channels + c, x);
                Ld8<float>::store(tail + (size_t)i * channels + c, x);
            }
        }
    }
}

// ---------------------------------------------------------------- inputs of the recurrences without a correction
// One block per token.  proj[t] = q (heads x dk) | k (heads x dk) | v (heads x dv) | anything, in the storage type;
// q times a scale, k and v as they are, all widened to float32 for the scan.  `kind` says what the gates are made of:
//   kLinearChannelDecay  z [T, heads * dk] float32 + bias: a decay per key channel, sigmoid(z)^(inv_tau), made as
//                        exp(inv_tau * logsigmoid(z));
//   kLinearLogGates      z [T, 2 heads] float32 + bias = write logits | keep logits, each capped as cap tanh(. / cap);
//                        the write's logarithm is the capped logit, the keep's is logsigmoid of its capped logit; the
//                        values get one more column of ones (the normaliser of a matrix memory), vv is [T, heads, dv + 1].
enum LinearKind : int { kLinearChannelDecay = 0, kLinearLogGates = 1 };

__device__ __forceinline__ float log_sigmoid_f32(float z) {
    return fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
}

template <typename T>
__global__ void linear_prepare_kernel(const T* proj, int ld, const float* z, int ldz, const float* __restrict__ z_bias,
                                      int kind, float p0, const int* __restrict__ token_slot, int heads, int dk, int dv,
                                      float q_scale, float* qn, float* kn, float* vv, float* decay, float* wgate,
                                      float* fgate) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    if (token_slot[t] < 0) return;
    const T* row = proj + (size_t)t * ld;
    const int qk = heads * dk;
    for (int e = threadIdx.x; e < qk; e += blockDim.x) {
        qn[(size_t)t * qk + e] = to_f32<T>(row[e]) * q_scale;
        kn[(size_t)t * qk + e] = to_f32<T>(row[qk + e]);
    }
    if (kind == kLinearChannelDecay) {
        for (int e = threadIdx.x; e < heads * dv; e += blockDim.x) vv[(size_t)t * heads * dv + e] = to_f32<T>(row[2 * qk + e]);
        for (int e = threadIdx.x; e < qk; e += blockDim.x)
            decay[(size_t)t * qk + e] = expf(p0 * log_sigmoid_f32(z[(size_t)t * ldz + e] + z_bias[e]));
    } else {
        const int cols = dv + 1;
        for (int e = threadIdx.x; e < heads * cols; e += blockDim.x) {
            const int h = e / cols, c = e - h * cols;
            vv[(size_t)t * heads * cols + e] = c < dv ? to_f32<T>(row[2 * qk + h * dv + c]) : 1.0f;
        }
        for (int h = threadIdx.x; h < heads; h += blockDim.x) {
            const float zi = z[(size_t)t * ldz + h] + z_bias[h];
            const float zf = z[(size_t)t * ldz + heads + h] + z_bias[heads + h];
            wgate[(size_t)t * heads + h] = p0 * tanhf(zi / p0);
            fgate[(size_t)t * heads + h] = log_sigmoid_f32(p0 * tanhf(zf / p0));
        }
    }
}

}  // namespace tllm

using namespace tllm;

extern "C" {

// Inputs of a recurrence without a correction from the fused projections; see linear_prepare_kernel.  p0: 1 / tau
// of the channel decays, or the cap of the gates' logits.
int tllm_linear_prepare(const void* proj, int ld, int dtype, const float* z, int ldz, const float* z_bias, int kind,
                        float p0, const int* token_slot, int heads, int dk, int dv, float q_scale, float* qn, float* kn,
                        float* vv, float* decay, float* wgate, float* fgate, int n_rows, cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && heads > 0 && dk > 0 && dv > 0 && p0 > 0.0f, "linear_prepare: bad sizes");
    TLLM_REQUIRE(kind == kLinearChannelDecay || kind == kLinearLogGates, "linear_prepare: unknown kind %d", kind);
    TLLM_REQUIRE(ld >= 2 * heads * dk + heads * dv && ldz >= (kind == kLinearChannelDecay ? heads * dk : 2 * heads),
                 "linear_prepare: rows too short");
    TLLM_REQUIRE(kind == kLinearChannelDecay ? decay != nullptr : (wgate != nullptr && fgate != nullptr),
                 "linear_prepare: no place for the gates");
    if (n_rows == 0) return 0;
    if (dtype == kBF16)
        launch_pdl(kPdlOther, linear_prepare_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)proj, ld, z, ldz,
                   z_bias, kind, p0, token_slot, heads, dk, dv, q_scale, qn, kn, vv, decay, wgate, fgate);
    else if (dtype == kF32)
        launch_pdl(kPdlOther, linear_prepare_kernel<float>, dim3(n_rows), dim3(256), 0, stream, (const float*)proj, ld, z, ldz,
                   z_bias, kind, p0, token_slot, heads, dk, dv, q_scale, qn, kn, vv, decay, wgate, fgate);
    else TLLM_REQUIRE(false, "linear_prepare: unknown dtype %d", dtype);
    return finish_launch("linear_prepare");
}

// Lanes that share a column of the state for keys of width dk (the state's layout depends on it).
int tllm_delta_rule_lanes(int dk) { return delta_lanes(dk); }

// Floats of one request's state: S of every head in the scan's layout, then the convolution's window.
long long tllm_delta_rule_state_floats(int heads, int kv_heads, int dk, int dv, int taps) {
    const int r = delta_lanes(dk), per = (dk + r - 1) / r;
    return (long long)heads * per * r * dv + (long long)(taps - 1) * (2 * kv_heads * dk + heads * dv);
}

// conv_w [channels, taps], and conv_t, the same taps as [taps, channels] (null: the scalar kernel serves).
int tllm_delta_prepare(const void* proj, int ld, int dtype, const void* conv_w, const void* conv_t, int taps, const float* a,
                       int lda, const float* dt_bias, const float* rate, const int* token_slot, const float* state,
                       long long state_stride, int heads, int kv_heads, int dk, int dv, float q_scale,
                       float unit_eps, float* qn, float* kn, float* vv, float* decay, float* beta, int n_rows,
                       int decay_per_head, int beta_col, cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0 && taps > 0,
                 "delta_prepare: bad sizes");
    const int channels = 2 * kv_heads * dk + heads * dv;
    if (beta_col < 0) beta_col = channels;
    TLLM_REQUIRE(ld >= beta_col + heads && beta_col >= channels && lda >= (decay_per_head ? heads : heads * dk),
                 "delta_prepare: rows too short");
    if (n_rows == 0) return 0;
    const int r = delta_lanes(dk), per = (dk + r - 1) / r;
    TLLM_REQUIRE(per <= kScanMaxPer, "delta_prepare: keys of width %d are too wide", dk);
    const long long tail_off = (long long)heads * per * r * dv;
    const auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec = conv_t != nullptr && dk % 8 == 0 && dv % 8 == 0 && ld % 8 == 0 && tail_off % 4 == 0 &&
                     (decay_per_head || (lda % 4 == 0 && al(a) && al(dt_bias))) &&
                     state_stride % 4 == 0 && al(proj) && al(conv_t) && al(state) && al(qn) && al(kn) &&
                     al(vv) && al(decay);
    // blocks per token: one where the rows fill the GPU, else up to a q or k head each
    const int sms_p = sm_count_cached() > 0 ? sm_count_cached() : 148;
    int split = 1;
    if (vec) while (split * 2 <= 2 * kv_heads && (long long)n_rows * split < 2LL * sms_p) split *= 2;
    const size_t smem = (size_t)(vec ? (2 * kv_heads + split - 1) / split * dk + dk : channels) * sizeof(float);
    TLLM_REQUIRE(smem <= 200 * 1024, "delta_prepare: %d channels do not fit in shared memory", channels);
#define PREP_VEC(T, N)                                                                                           \
    do {                                                                                                         \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(delta_prepare_vec_kernel<T, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) { set_error("delta_prepare: %s", cudaGetErrorString(e)); return (int)e; }      \
        }                                                                                                        \
        launch_pdl(kPdlOther, delta_prepare_vec_kernel<T, N>, dim3(n_rows, split), dim3(split > 1 ? 128 : 256), smem, stream, \
                   (const T*)proj, ld, (const T*)conv_t, taps, a, lda, dt_bias, rate, token_slot, state, state_stride,   \
                   tail_off, heads, kv_heads, dk, dv, q_scale, unit_eps, qn, kn, vv, decay, beta, n_rows,      \
                   decay_per_head, beta_col);                                                                    \
    } while (0)
#define PREP(T)                                                                                                  \
    do {                                                                                                         \
        if (vec) {                                                                                               \
            if (taps == 2) PREP_VEC(T, 2);                                                                       \
            else if (taps == 3) PREP_VEC(T, 3);                                                                  \
            else if (taps == 4) PREP_VEC(T, 4);                                                                  \
            else PREP_VEC(T, 0);                                                                                 \
            break;                                                                                               \
        }                                                                                                        \
        if (smem > 48 * 1024) {                                                                                  \
            cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) { set_error("delta_prepare: %s", cudaGetErrorString(e)); return (int)e; }      \
        }                                                                                                        \
        launch_pdl(kPdlOther, delta_prepare_kernel<T>, dim3(n_rows), dim3(256), smem, stream, (const T*)proj, ld, \
                   (const T*)conv_w, taps, a, lda, dt_bias, rate, token_slot, state, state_stride, tail_off,     \
                   heads, kv_heads, dk, dv, q_scale, unit_eps, qn, kn, vv, decay, beta, n_rows,                  \
                   decay_per_head, beta_col);                                                                    \
    } while (0)
    if (dtype == kBF16) PREP(bf16);
    else if (dtype == kF32) PREP(float);
    else TLLM_REQUIRE(false, "delta_prepare: unknown dtype %d", dtype);
#undef PREP
#undef PREP_VEC
    return finish_launch("delta_prepare");
}

// seg_info: int[segments][4] = slot, first row, length, first position; null: every row is a portion of one token.
int tllm_delta_scan(const int* seg_info, int segments, const int* token_slot, const float* qn, const float* kn,
                    const float* vv, const float* decay, const float* beta, float* state, long long state_stride,
                    int heads, int kv_heads, int dk, int dv, float* o_raw, int mode, const float* fgate,
                    long long aux_off, float floor_eps, float* den, cudaStream_t stream) {
    TLLM_REQUIRE(segments >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dk > 0 && dv > 0,
                 "delta_scan: bad sizes");
    TLLM_REQUIRE(mode == kScanDelta || mode == kScanPlain || mode == kScanMemory || mode == kScanHeadDecay,
                 "delta_scan: unknown recurrence %d", mode);
    TLLM_REQUIRE(mode == kScanMemory ? (beta != nullptr && fgate != nullptr && den != nullptr && dv >= 2 && aux_off > 0)
                 : mode == kScanHeadDecay ? (beta != nullptr && fgate != nullptr) : decay != nullptr, "delta_scan: the recurrence lacks an operand");
    TLLM_REQUIRE(mode != kScanDelta || beta != nullptr, "delta_scan: the delta rule needs its betas");
    TLLM_REQUIRE(heads <= 65535, "delta_scan: %d heads", heads);
    if (segments == 0) return 0;
    const int r = delta_lanes(dk), per = (dk + r - 1) / r;
    TLLM_REQUIRE(per <= kScanMaxPer, "delta_scan: keys of width %d are too wide", dk);
    // columns per block: whole warps, at most 256 threads, not wider than the values, and at least a block per
    // multiprocessor in all where the value width allows it (a column does not depend on the others, so the
    // result is the same however they are dealt)
    int cols = 256 / r;
    const int min_cols = 32 / r > 1 ? 32 / r : 1;
    const int sms = sm_count_cached() > 0 ? sm_count_cached() : 148;
    while (cols > min_cols && cols / 2 >= dv) cols /= 2;
    while (cols > min_cols && (long long)segments * heads * ((dv + cols - 1) / cols) < sms) cols /= 2;
    const int col_blocks = (dv + cols - 1) / cols;
    const int threads = cols * r;
    TLLM_REQUIRE(col_blocks <= 65535, "delta_scan: sizes %d x %d do not fit", dk, dv);
    const auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const int vec = dk % 4 == 0 && per % 4 == 0 && aligned(qn) && aligned(kn) && (decay == nullptr || aligned(decay));
#define SCAN(RR, PP)                                                                                             \
    do {                                                                                                         \
        if (mode == kScanDelta) SCAN_MODE(RR, PP, kScanDelta);                                                   \
        else if (mode == kScanPlain) SCAN_MODE(RR, PP, kScanPlain);                                              \
        else if (mode == kScanHeadDecay) SCAN_MODE(RR, PP, kScanHeadDecay);                                      \
        else SCAN_MODE(RR, PP, kScanMemory);                                                                     \
    } while (0)
#define SCAN_MODE(RR, PP, MM)                                                                                           \
    do {                                                                                                         \
        const size_t smem = ((size_t)2 * ScanLayout<RR, PP>::stage_floats(cols) + (size_t)kScanChunk * cols) * sizeof(float); \
        TLLM_REQUIRE(smem <= 200 * 1024, "delta_scan: sizes %d x %d do not fit", dk, dv);                         \
        static OncePerDevice configured;                                                                         \
        if (configured.first()) {                                                                                \
            cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<RR, PP, MM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            if (e != cudaSuccess) { set_error("delta_scan: %s", cudaGetErrorString(e)); return (int)e; }         \
            configured.done();                                                                                   \
        }                                                                                                        \
        launch_pdl(kPdlOther, delta_scan_kernel<RR, PP, MM>, dim3(segments, heads, col_blocks), dim3(threads), smem, stream, \
                   seg_info, token_slot, qn, kn, vv, decay, beta, state, state_stride, heads, kv_heads, dk, dv,  \
                   cols, vec, o_raw, fgate, aux_off, floor_eps, den);                                            \
    } while (0)
    if (r == 4 && per <= 4) SCAN(4, 4);
    else if (r == 4 && per <= 8) SCAN(4, 8);
    else if (r == 4) SCAN(4, 16);
    else if (r == 8) SCAN(8, 16);
    else if (r == 16) SCAN(16, 16);
    else SCAN(32, 16);
#undef SCAN
#undef SCAN_MODE
    return finish_launch("delta_scan");
}

// gate: float32 (gate_f32) or the storage type; state_dv: value columns of S in the state's layout (dv, or more where
// the recurrence keeps columns of its own); with taps 1 neither proj nor the state are touched.
int tllm_delta_finish(const float* o_raw, const void* gate, int gate_f32, int ldg, const float* weight, float eps,
                      const int* token_slot, int n_rows, int heads, int kv_heads, int dk, int dv, void* out,
                      int dtype, const void* proj, int ld, int taps, float* state, long long state_stride,
                      const float* den, int gate_act, int weight_stride, cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && heads > 0 && dv > 0 && eps > 0.0f && ldg >= heads * dv, "delta_finish: bad sizes");
    TLLM_REQUIRE((gate_act == 0 || gate_act == 1) && (weight_stride == 0 || weight_stride == dv), "delta_finish: bad options");
    if (n_rows == 0) return 0;
    const int channels = 2 * kv_heads * dk + heads * dv;
    const int r = delta_lanes(dk), per = (dk + r - 1) / r;
    const long long tail_off = (long long)heads * per * r * dv;
    const auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec = dv % 4 == 0 && ldg % 4 == 0 && al(o_raw) && (reinterpret_cast<uintptr_t>(gate) & 7u) == 0 && al(weight) &&
                     (gate_f32 || dtype == kF32 ? al(gate) : true) &&
                     (taps <= 1 || (channels % 8 == 0 && ld % 8 == 0 && tail_off % 4 == 0 && state_stride % 4 == 0 && al(proj) && al(state)));
    const int sms_f = sm_count_cached() > 0 ? sm_count_cached() : 148;
    int split = 1;
    while (vec && split * 2 <= heads && (long long)n_rows * split < 2LL * sms_f) split *= 2;
#define FIN(T, TG)                                                                                                         \
    do {                                                                                                                   \
        if (vec)                                                                                                           \
            launch_pdl(kPdlOther, delta_finish_vec_kernel<T, TG>, dim3(n_rows, split), dim3(split > 1 ? 128 : 256), 0, stream, o_raw, (const TG*)gate, ldg, weight, eps, \
                       token_slot, n_rows, heads, dv, (T*)out, (const T*)proj, ld, channels, taps, state, state_stride, tail_off, den, gate_act, weight_stride); \
        else                                                                                                               \
            launch_pdl(kPdlOther, delta_finish_kernel<T, TG>, dim3(n_rows), dim3(256), 0, stream, o_raw, (const TG*)gate, ldg, weight, eps, \
                       token_slot, n_rows, heads, dv, (T*)out, (const T*)proj, ld, channels, taps, state, state_stride, tail_off, den, gate_act, weight_stride); \
    } while (0)
    if (dtype == kBF16) { if (gate_f32) FIN(bf16, float); else FIN(bf16, bf16); }
    else if (dtype == kF32) FIN(float, float);
    else TLLM_REQUIRE(false, "delta_finish: unknown dtype %d", dtype);
#undef FIN
    return finish_launch("delta_finish");
}

}  // extern "C"
