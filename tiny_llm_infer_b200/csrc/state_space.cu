// A selective state space with one decay per head, as the recurrence the scan kernel of delta_rule.cu walks
// (its form without a correction): per head a state S [N, P] in float32, carried from step to step,
//
//   S <- exp(-rate_h dt) S + B (dt x)^T;   y = S^T C + D_h x
//
// with N the state width, P the head's width, B and C shared by the heads of a group (they are the scan's keys
// and queries, dt x its values, and the decay is one number per head for all N rows).  Two kernels stand around
// the scan, for prompt portions and single tokens alike:
//
//   ssd_prepare  per token: the short causal convolution (with a bias) over the channels x | B | C of the
//                fused projection (taps that reach before the portion come from the request's state) and SiLU;
//                dt = softplus(dt + dt_bias) without a clamp; then C, B, x, and per head dt and the decay, in
//                float32 (the scan multiplies x by dt as its write strength, the finish kernel by D).
//   ssd_finish   per token: (y + D x) silu(z), an RMS norm over each of `norm_groups` equal parts of
//                the row, a weight; the block of a portion's last token moves the convolution's window of the
//                request's state on.
//
// A row of the projection is z (heads P) | x (heads P) | B (groups N) | C (groups N) | dt (heads).  State of a
// request: S of every head in the scan's layout, then [taps - 1][channels] float32 inputs of the convolution,
// the newest last.  Everything behind the projection is float32 in both storage types.
#include "common.cuh"

namespace tllm {

__device__ __forceinline__ float ssd_softplus(float x) {
    return x > 20.0f ? x : log1pf(expf(x));
}

// Eight elements at a time in either storage type.
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

// A token's channels are dealt to gridDim.y blocks (few rows would leave the GPU idle otherwise); the first
// makes the token's step sizes.  VEC: eight channels per thread and access (the taps as [taps][channels],
// head width, the widths of x and of B and rows of proj multiples of eight, 16-byte boundaries); else one.
// keep [n_rows, heads] receives the decay exp(-rate_h dt) of every head, which the scan applies to all rows of S,
// and step [n_rows, heads] dt itself.  TAPS: the number of taps if it is 2, 3 or 4 (their loads are then all
// issued before the first product), 0 for any other number.
template <typename T, bool VEC, int TAPS>
__global__ void ssd_prepare_kernel(const T* proj, int ld, const T* __restrict__ conv_w, const float* __restrict__ conv_b,
                                   int taps, const float* __restrict__ dt_bias, const float* __restrict__ rate,
                                   const int* __restrict__ token_slot,
                                   const float* state, long long state_stride, long long tail_off, int heads,
                                   int groups, int N, int P, float* qn, float* kn, float* vv, float* keep,
                                   float* step) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int inner = heads * P, gn = groups * N, channels = inner + 2 * gn;
    int back = 0;                                // rows before this one that belong to the same portion
    for (int j = 1; j < taps; ++j) {
        if (t - j >= 0 && token_slot[t - j] == slot) back = j;
        else break;
    }
    const float* tail = state + (long long)slot * state_stride + tail_off;
    const T* row = proj + (size_t)t * ld;
    if (blockIdx.y == 0)
        for (int h = threadIdx.x; h < heads; h += blockDim.x) {
            const float d = ssd_softplus(to_f32<T>(row[2 * inner + 2 * gn + h]) + dt_bias[h]);
            keep[(size_t)t * heads + h] = expf(-rate[h] * d);
            step[(size_t)t * heads + h] = d;
        }
    constexpr int kStep = VEC ? 8 : 1;
    const int units = channels / kStep;
    const int u0 = (int)((long long)units * blockIdx.y / gridDim.y), u1 = (int)((long long)units * (blockIdx.y + 1) / gridDim.y);
    for (int u = u0 + threadIdx.x; u < u1; u += blockDim.x) {
        const int c = u * kStep;
        float acc[kStep];
        if constexpr (VEC) {
            if (conv_b != nullptr) Ld8<float>::load(conv_b + c, reinterpret_cast<float (&)[8]>(acc));
            else for (int e = 0; e < kStep; ++e) acc[e] = 0.0f;
            if constexpr (TAPS > 0) {
                float w[TAPS > 0 ? TAPS : 1][8], x[TAPS > 0 ? TAPS : 1][8];
#pragma unroll
                for (int j = 0; j < TAPS; ++j) {
                    Ld8<T>::load(conv_w + (size_t)(TAPS - 1 - j) * channels + c, w[j]);     // the taps as [taps][channels]
                    if (j <= back) Ld8<T>::load(proj + (size_t)(t - j) * ld + inner + c, x[j]);
                    else Ld8<float>::load(tail + (size_t)(TAPS - 1 - (j - back)) * channels + c, x[j]);
                }
#pragma unroll
                for (int j = 0; j < TAPS; ++j)
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] += w[j][e] * x[j][e];
            } else {
                for (int j = 0; j < taps; ++j) {
                    float w[8], x[8];
                    Ld8<T>::load(conv_w + (size_t)(taps - 1 - j) * channels + c, w);
                    if (j <= back) Ld8<T>::load(proj + (size_t)(t - j) * ld + inner + c, x);
                    else Ld8<float>::load(tail + (size_t)(taps - 1 - (j - back)) * channels + c, x);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] += w[e] * x[e];
                }
            }
        } else {
            acc[0] = conv_b != nullptr ? conv_b[c] : 0.0f;
            for (int j = 0; j < taps; ++j) {
                const float w = to_f32<T>(conv_w[(size_t)c * taps + (taps - 1 - j)]);
                const float x = j <= back ? to_f32<T>(proj[(size_t)(t - j) * ld + inner + c])
                                          : tail[(size_t)(taps - 1 - (j - back)) * channels + c];
                acc[0] += w * x;
            }
        }
#pragma unroll
        for (int e = 0; e < kStep; ++e) acc[e] = acc[e] / (1.0f + expf(-acc[e]));
        if (c < inner) {                         // x: the scan's values (it multiplies them by dt) and the read-out's D x
            if constexpr (VEC) Ld8<float>::store(vv + (size_t)t * inner + c, reinterpret_cast<float (&)[8]>(acc));
            else vv[(size_t)t * inner + c] = acc[0];
        } else {
            float* dst = c < inner + gn ? kn + (size_t)t * gn + (c - inner) : qn + (size_t)t * gn + (c - inner - gn);
            if constexpr (VEC) Ld8<float>::store(dst, reinterpret_cast<float (&)[8]>(acc));
            else dst[0] = acc[0];
        }
    }
}

// A token's norm parts are dealt to gridDim.y blocks (at most one block per part), and so are the channels of
// the convolution's window when the token is the last of its portion.
// xs [n_rows, inner]: x after convolution and SiLU; skip_d [heads]: y gets skip_d[h] * x added.  A block whose parts
// are at least as many as its warps gives each warp parts of its own (no barrier on the way); else all threads
// share a part.
template <typename T, bool VEC>
__global__ void ssd_finish_kernel(const float* o_raw, const float* xs, const float* __restrict__ skip_d, int P, const T* proj, int ld,
                                  const float* __restrict__ weight, float eps, int norm_groups,
                                  const int* __restrict__ token_slot, int n_rows, int inner, int channels, int taps,
                                  float* state, long long state_stride, long long tail_off, T* out) {
    extern __shared__ __align__(16) float g[];   // the gated read-out of one norm part, per warp or for the block
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    const int part = inner / norm_groups;
    const int p0 = norm_groups * blockIdx.y / gridDim.y, p1 = norm_groups * (blockIdx.y + 1) / gridDim.y;
    if (slot < 0) {
        for (int e = p0 * part + threadIdx.x; e < p1 * part; e += blockDim.x) out[(size_t)t * inner + e] = from_f32<T>(0.0f);
        return;
    }
    const T* row = proj + (size_t)t * ld;
    constexpr int kStep = VEC ? 8 : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const bool by_warp = p1 - p0 >= warps;       // the same for all threads of the block
    // a group (a warp, or the whole block) walks one part: gated read-out into shared memory, sum, scaling
    const int first = by_warp ? p0 + warp : p0, stride_p = by_warp ? warps : 1;
    const int tid = by_warp ? lane : threadIdx.x, nthr = by_warp ? 32 : blockDim.x;
    for (int p = first; p < p1; p += stride_p) {
        const size_t base = (size_t)t * inner + (size_t)p * part;
        float* gp = g + (by_warp ? (size_t)warp * part : 0);
        float sum = 0.0f;
        for (int e = tid * kStep; e < part; e += nthr * kStep) {
            float o[kStep], x[kStep], z[kStep];
            if constexpr (VEC) {
                Ld8<float>::load(o_raw + base + e, reinterpret_cast<float (&)[8]>(o));
                Ld8<float>::load(xs + base + e, reinterpret_cast<float (&)[8]>(x));
                Ld8<T>::load(row + (size_t)p * part + e, reinterpret_cast<float (&)[8]>(z));
            } else {
                o[0] = o_raw[base + e]; x[0] = xs[base + e]; z[0] = to_f32<T>(row[(size_t)p * part + e]);
            }
            const float d = skip_d[((size_t)p * part + e) / P];       // (eight neighbours share a head in the vector form)
#pragma unroll
            for (int i = 0; i < kStep; ++i) {
                const float v = (o[i] + d * x[i]) * (z[i] / (1.0f + expf(-z[i])));
                gp[e + i] = v;
                sum += v * v;
            }
        }
        if (by_warp) { sum = warp_sum(sum); __syncwarp(); }
        else sum = block_sum(sum, scratch);      // (its barriers also order the writes of g before the reads below)
        const float sc = 1.0f / sqrtf(sum / (float)part + eps);
        for (int e = tid * kStep; e < part; e += nthr * kStep) {
            if constexpr (VEC) {
                float w[8], v[8];
                Ld8<float>::load(weight + (size_t)p * part + e, w);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = gp[e + i] * sc * w[i];
                Ld8<T>::store(out + base + e, v);
            } else {
                out[base + e] = from_f32<T>(gp[e] * sc * weight[(size_t)p * part + e]);
            }
        }
        if (by_warp) __syncwarp();
        else __syncthreads();                    // g is written again for the next part
    }
    // the portion's last row moves the convolution's window on: its taps - 1 newest inputs
    if (taps > 1 && (t + 1 >= n_rows || token_slot[t + 1] != slot)) {
        int len = 1;                                 // rows of the portion, as far as the window reaches
        while (len < taps - 1 && t - len >= 0 && token_slot[t - len] == slot) ++len;
        float* tail = state + (long long)slot * state_stride + tail_off;
        const int keep = taps - 1;
        const int c0 = (int)((long long)channels * blockIdx.y / gridDim.y), c1 = (int)((long long)channels * (blockIdx.y + 1) / gridDim.y);
        for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
            for (int i = 0; i < keep; ++i) {         // ascending: an old entry is read before its place is written
                const int from_end = keep - i;       // this entry is the from_end-th newest input
                float x;
                if (from_end <= len) x = to_f32<T>(proj[(size_t)(t + 1 - from_end) * ld + inner + c]);
                else x = tail[(size_t)(i + len) * channels + c];
                tail[(size_t)i * channels + c] = x;
            }
        }
    }
}

// Blocks that share a token when the tokens alone would leave the GPU idle.
static int token_split(int rows, int most) {
    const int sms = sm_count_cached() > 0 ? sm_count_cached() : 148;
    int split = 1;
    while (split * 2 <= most && (long long)rows * split < 2LL * sms) split *= 2;
    return split;
}

}  // namespace tllm

using namespace tllm;

extern "C" {

// conv_w [channels, taps] in the storage type and conv_t, the same taps as [taps, channels] (null: one channel
// per thread), conv_b [channels] float32 or null; dt_bias and rate (the positive decay rate per head) [heads]
// float32.  tail_off: floats of S before the convolution's window in a request's state.  Outputs
// float32: qn (C) and kn (B) [n_rows, groups N], vv (x) [n_rows, heads P], decay and step (dt) [n_rows, heads].
int tllm_ssd_prepare(const void* proj, int ld, int dtype, const void* conv_w, const void* conv_t, const float* conv_b, int taps,
                     const float* dt_bias, const float* rate, const int* token_slot,
                     const float* state, long long state_stride, long long tail_off, int heads, int groups, int N,
                     int P, float* qn, float* kn, float* vv, float* decay, float* step, int n_rows,
                     cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && heads > 0 && groups > 0 && heads % groups == 0 && N > 0 && P > 0 && taps > 0,
                 "ssd_prepare: bad sizes");
    const int inner = heads * P, channels = inner + 2 * groups * N;
    TLLM_REQUIRE(ld >= inner + channels + heads, "ssd_prepare: rows of %d are too short", ld);
    TLLM_REQUIRE(taps == 1 || state != nullptr, "ssd_prepare: no state for the convolution's window");
    if (n_rows == 0) return 0;
    const auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec = conv_t != nullptr && P % 8 == 0 && (groups * N) % 8 == 0 && ld % 8 == 0 && tail_off % 4 == 0 &&
                     state_stride % 4 == 0 && al(proj) && al(conv_t) && al(conv_b) && al(state) && al(qn) && al(kn) &&
                     al(vv);
    const int split = token_split(n_rows, channels / 256 > 0 ? channels / 256 : 1);
#define PREP_T(T, V, N)                                                                                             \
    launch_pdl(kPdlOther, ssd_prepare_kernel<T, V, N>, dim3(n_rows, split), dim3(split > 1 ? 128 : 256), 0, stream, \
               (const T*)proj, ld, (const T*)(V ? conv_t : conv_w), conv_b, taps, dt_bias, rate, token_slot, \
               state, state_stride, tail_off, heads, groups, N_state, P, qn, kn, vv, decay, step)
#define PREP(T)                                                                                                     \
    do {                                                                                                            \
        if (!vec) PREP_T(T, false, 0);                                                                              \
        else if (taps == 2) PREP_T(T, true, 2);                                                                     \
        else if (taps == 3) PREP_T(T, true, 3);                                                                     \
        else if (taps == 4) PREP_T(T, true, 4);                                                                     \
        else PREP_T(T, true, 0);                                                                                    \
    } while (0)
    const int N_state = N;
    if (dtype == kBF16) PREP(bf16);
    else if (dtype == kF32) PREP(float);
    else TLLM_REQUIRE(false, "ssd_prepare: unknown dtype %d", dtype);
#undef PREP_T
#undef PREP
    return finish_launch("ssd_prepare");
}

// o_raw (the scan's read-out) and xs (x after convolution and SiLU) [n_rows, inner] float32; skip_d [inner / P]
// float32; proj as in ssd_prepare (z in its first `inner` columns, the convolution's inputs behind them); weight
// [inner] float32; out [n_rows, inner] in the storage type.
int tllm_ssd_finish(const float* o_raw, const float* xs, const float* skip_d, int P, const void* proj, int ld, int dtype, const float* weight,
                    float eps, int norm_groups, const int* token_slot, int n_rows, int inner, int channels, int taps,
                    float* state, long long state_stride, long long tail_off, void* out, cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && inner > 0 && norm_groups > 0 && inner % norm_groups == 0 && eps > 0.0f && taps > 0,
                 "ssd_finish: bad sizes");
    TLLM_REQUIRE(ld >= inner + channels, "ssd_finish: rows of %d are too short", ld);
    if (n_rows == 0) return 0;
    TLLM_REQUIRE(P > 0 && inner % P == 0, "ssd_finish: heads of %d in rows of %d", P, inner);
    const int part = inner / norm_groups;
    const int split = token_split(n_rows, norm_groups);
    const int per_block = (norm_groups + split - 1) / split;
    const size_t smem = (size_t)part * (per_block >= 8 ? 8 : 1) * sizeof(float);        // a part per warp, or one for the block
    TLLM_REQUIRE(smem <= 200 * 1024, "ssd_finish: parts of %d do not fit in shared memory", part);
    const auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec = part % 8 == 0 && P % 8 == 0 && ld % 8 == 0 && al(o_raw) && al(xs) && al(proj) && al(weight) && al(out);
#define FIN(T, V)                                                                                                   \
    do {                                                                                                            \
        if (smem > 48 * 1024) {                                                                                     \
            cudaError_t e = cudaFuncSetAttribute(ssd_finish_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) { set_error("ssd_finish: %s", cudaGetErrorString(e)); return (int)e; }            \
        }                                                                                                           \
        launch_pdl(kPdlOther, ssd_finish_kernel<T, V>, dim3(n_rows, split), dim3(256), smem, stream, o_raw, xs,     \
                   skip_d, P, (const T*)proj, ld, weight, eps, norm_groups, token_slot, n_rows, inner, channels, taps, state,  \
                   state_stride, tail_off, (T*)out);                                                                \
    } while (0)
    if (dtype == kBF16) { if (vec) FIN(bf16, true); else FIN(bf16, false); }
    else if (dtype == kF32) { if (vec) FIN(float, true); else FIN(float, false); }
    else TLLM_REQUIRE(false, "ssd_finish: unknown dtype %d", dtype);
#undef FIN
    return finish_launch("ssd_finish");
}

}  // extern "C"
