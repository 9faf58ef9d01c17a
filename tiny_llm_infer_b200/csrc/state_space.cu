// A selective state space with one decay per head, as the recurrence the scan kernel of delta_rule.cu walks
// (its form without a correction): per head a state S [N, P] in float32, carried from step to step,
//
//   S <- exp(-rate_h dt) S + B (dt x)^T;   y = S^T C + D_h x
//
// with N the state width, P the head's width, B and C shared by the heads of a group (they are the scan's keys
// and queries, dt x its values, and the decay is one number per head for all N rows).  Two kernels stand around
// the scan, for prompt portions and single tokens alike:
//
//   ssd_prepare  one block per token: the short causal convolution (with a bias) over the channels x | B | C of the
//                fused projection (taps that reach before the portion come from the request's state) and SiLU;
//                dt = softplus(dt + dt_bias) without a clamp; then C, B, dt x, the decays and D x in float32.
//   ssd_finish   one block per token: (y + D x) silu(z), an RMS norm over each of `norm_groups` equal parts of
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

template <typename T>
__global__ void ssd_prepare_kernel(const T* proj, int ld, const T* __restrict__ conv_w, const float* __restrict__ conv_b,
                                   int taps, const float* __restrict__ dt_bias, const float* __restrict__ rate,
                                   const float* __restrict__ skip_d, const int* __restrict__ token_slot,
                                   const float* state, long long state_stride, long long tail_off, int heads,
                                   int groups, int N, int P, float* qn, float* kn, float* vv, float* decay,
                                   float* skip) {
    extern __shared__ float y[];                 // [channels] after convolution and SiLU, then dt [heads]
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int inner = heads * P, gn = groups * N, channels = inner + 2 * gn;
    float* dt = y + channels;
    int back = 0;                                // rows before this one that belong to the same portion
    for (int j = 1; j < taps; ++j) {
        if (t - j >= 0 && token_slot[t - j] == slot) back = j;
        else break;
    }
    const float* tail = state + (long long)slot * state_stride + tail_off;
    const T* row = proj + (size_t)t * ld;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float acc = conv_b != nullptr ? conv_b[c] : 0.0f;
        for (int j = 0; j < taps; ++j) {
            const float w = to_f32<T>(conv_w[(size_t)c * taps + (taps - 1 - j)]);
            float x;
            if (j <= back) x = to_f32<T>(proj[(size_t)(t - j) * ld + inner + c]);
            else x = tail[(size_t)(taps - 1 - (j - back)) * channels + c];
            acc += w * x;
        }
        y[c] = acc / (1.0f + expf(-acc));
    }
    for (int h = threadIdx.x; h < heads; h += blockDim.x)
        dt[h] = ssd_softplus(to_f32<T>(row[2 * inner + 2 * gn + h]) + dt_bias[h]);
    __syncthreads();
    for (int e = threadIdx.x; e < inner; e += blockDim.x) {
        const int h = e / P;
        vv[(size_t)t * inner + e] = dt[h] * y[e];
        skip[(size_t)t * inner + e] = skip_d[h] * y[e];
    }
    for (int e = threadIdx.x; e < gn; e += blockDim.x) {
        kn[(size_t)t * gn + e] = y[inner + e];
        qn[(size_t)t * gn + e] = y[inner + gn + e];
    }
    for (int e = threadIdx.x; e < heads * N; e += blockDim.x) {
        const int h = e / N;
        decay[(size_t)t * heads * N + e] = expf(-rate[h] * dt[h]);
    }
}

template <typename T>
__global__ void ssd_finish_kernel(const float* o_raw, const float* skip, const T* proj, int ld,
                                  const float* __restrict__ weight, float eps, int norm_groups,
                                  const int* __restrict__ token_slot, int n_rows, int inner, int channels, int taps,
                                  float* state, long long state_stride, long long tail_off, T* out) {
    extern __shared__ float g[];                 // [inner] the gated read-out
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) {
        for (int e = threadIdx.x; e < inner; e += blockDim.x) out[(size_t)t * inner + e] = from_f32<T>(0.0f);
        return;
    }
    const T* row = proj + (size_t)t * ld;
    for (int e = threadIdx.x; e < inner; e += blockDim.x) {
        const float z = to_f32<T>(row[e]);
        g[e] = (o_raw[(size_t)t * inner + e] + skip[(size_t)t * inner + e]) * (z / (1.0f + expf(-z)));
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int part = inner / norm_groups;
    for (int p = warp; p < norm_groups; p += warps) {
        const float* src = g + (size_t)p * part;
        float sum = 0.0f;
        for (int e = lane; e < part; e += 32) sum += src[e] * src[e];
        sum = warp_sum(sum);
        const float sc = 1.0f / sqrtf(sum / (float)part + eps);
        for (int e = lane; e < part; e += 32)
            out[(size_t)t * inner + (size_t)p * part + e] = from_f32<T>(src[e] * sc * weight[(size_t)p * part + e]);
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
                if (from_end <= len) x = to_f32<T>(proj[(size_t)(t + 1 - from_end) * ld + inner + c]);
                else x = tail[(size_t)(i + len) * channels + c];
                tail[(size_t)i * channels + c] = x;
            }
        }
    }
}

}  // namespace tllm

using namespace tllm;

extern "C" {

// conv_w [channels, taps] in the storage type, conv_b [channels] float32 or null; dt_bias, rate (the positive
// decay rate per head) and skip_d [heads] float32.  tail_off: floats of S before the convolution's window in
// a request's state.  Outputs float32: qn (C) and kn (B) [n_rows, groups N], vv (dt x) and skip (D x) [n_rows,
// heads P], decay [n_rows, heads N].
int tllm_ssd_prepare(const void* proj, int ld, int dtype, const void* conv_w, const float* conv_b, int taps,
                     const float* dt_bias, const float* rate, const float* skip_d, const int* token_slot,
                     const float* state, long long state_stride, long long tail_off, int heads, int groups, int N,
                     int P, float* qn, float* kn, float* vv, float* decay, float* skip, int n_rows,
                     cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && heads > 0 && groups > 0 && heads % groups == 0 && N > 0 && P > 0 && taps > 0,
                 "ssd_prepare: bad sizes");
    const int inner = heads * P, channels = inner + 2 * groups * N;
    TLLM_REQUIRE(ld >= inner + channels + heads, "ssd_prepare: rows of %d are too short", ld);
    TLLM_REQUIRE(taps == 1 || state != nullptr, "ssd_prepare: no state for the convolution's window");
    if (n_rows == 0) return 0;
    const size_t smem = (size_t)(channels + heads) * sizeof(float);
    TLLM_REQUIRE(smem <= 200 * 1024, "ssd_prepare: %d channels do not fit in shared memory", channels);
#define PREP(T)                                                                                                     \
    do {                                                                                                            \
        if (smem > 48 * 1024) {                                                                                     \
            cudaError_t e = cudaFuncSetAttribute(ssd_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) { set_error("ssd_prepare: %s", cudaGetErrorString(e)); return (int)e; }           \
        }                                                                                                           \
        launch_pdl(kPdlOther, ssd_prepare_kernel<T>, dim3(n_rows), dim3(256), smem, stream, (const T*)proj, ld,     \
                   (const T*)conv_w, conv_b, taps, dt_bias, rate, skip_d, token_slot, state, state_stride, tail_off, \
                   heads, groups, N, P, qn, kn, vv, decay, skip);                                                   \
    } while (0)
    if (dtype == kBF16) PREP(bf16);
    else if (dtype == kF32) PREP(float);
    else TLLM_REQUIRE(false, "ssd_prepare: unknown dtype %d", dtype);
#undef PREP
    return finish_launch("ssd_prepare");
}

// o_raw (the scan's read-out) and skip [n_rows, inner] float32; proj as in ssd_prepare (z in its first `inner`
// columns, the convolution's inputs behind them); weight [inner] float32; out [n_rows, inner] in the storage type.
int tllm_ssd_finish(const float* o_raw, const float* skip, const void* proj, int ld, int dtype, const float* weight,
                    float eps, int norm_groups, const int* token_slot, int n_rows, int inner, int channels, int taps,
                    float* state, long long state_stride, long long tail_off, void* out, cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && inner > 0 && norm_groups > 0 && inner % norm_groups == 0 && eps > 0.0f && taps > 0,
                 "ssd_finish: bad sizes");
    TLLM_REQUIRE(ld >= inner + channels, "ssd_finish: rows of %d are too short", ld);
    if (n_rows == 0) return 0;
    const size_t smem = (size_t)inner * sizeof(float);
    TLLM_REQUIRE(smem <= 200 * 1024, "ssd_finish: rows of %d do not fit in shared memory", inner);
#define FIN(T)                                                                                                      \
    do {                                                                                                            \
        if (smem > 48 * 1024) {                                                                                     \
            cudaError_t e = cudaFuncSetAttribute(ssd_finish_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) { set_error("ssd_finish: %s", cudaGetErrorString(e)); return (int)e; }            \
        }                                                                                                           \
        launch_pdl(kPdlOther, ssd_finish_kernel<T>, dim3(n_rows), dim3(256), smem, stream, o_raw, skip,             \
                   (const T*)proj, ld, weight, eps, norm_groups, token_slot, n_rows, inner, channels, taps, state,  \
                   state_stride, tail_off, (T*)out);                                                                \
    } while (0)
    if (dtype == kBF16) FIN(bf16);
    else if (dtype == kF32) FIN(float);
    else TLLM_REQUIRE(false, "ssd_finish: unknown dtype %d", dtype);
#undef FIN
    return finish_launch("ssd_finish");
}

}  // extern "C"
