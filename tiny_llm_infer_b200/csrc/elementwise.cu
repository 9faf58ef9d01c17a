// Embedding gather, residual-add + RMSNorm, SwiGLU and storage-type conversion.
//
// What the reference does with separate launches (embed_kernel_cuda.cu:6-28,
// add_kernel_cuda.cu:7-14 followed by rmsnorm_kernel_cuda.cu:8-39,
// swiglu_kernel_cuda.cu:7-27) is fused here around one rule: the residual stream is
// a float32 tensor that only this file's kernels write, so the residual sum and the
// norm's mean are 32-bit in both storage modes.
//
// Pointers to what an earlier kernel of the step has written carry no __restrict__: with
// programmatic dependent launch this kernel may start before that kernel ends, and the
// read-only load path the compiler would otherwise choose may then return stale data.
//
// Every kernel has a vector form (16-byte loads and stores, eight elements per thread per
// access, every load of a row issued before the first dependent instruction) for widths that
// are multiples of eight, and a scalar form that takes any width.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace tllm {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int finish_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}

// ---------------------------------------------------------------- 8-element accesses
template <typename T> struct Vec8;
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Vec8<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};

// ---------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :] * scale, widened to float32 before the product (scale 1 for a plain look-up).  Rows with ids[t] < 0 (padding of a
// fixed-size batch) become zero.  Ids are range-checked on the host; the clamp below
// only keeps a faulty caller from reading outside the table.
template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab, float scale) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    if (id < 0) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.0f;
        return;
    }
    if (id >= vocab) id = vocab - 1;
    const TW* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32<TW>(src[i]) * scale;
}

template <typename TW>
__global__ void embedding_vec_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                     float* __restrict__ out, int hidden, int vocab, float scale) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    const bool pad = id < 0;
    if (id >= vocab) id = vocab - 1;
    const TW* src = table + (size_t)(pad ? 0 : id) * hidden;
    for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) {
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (!pad) Vec8<TW>::load(src + c * 8, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] *= scale;
        Vec8<float>::store(dst + c * 8, v);
    }
}

// ---------------------------------------------------------------- add + RMSNorm
// v = h[r, :] (+ delta[r, :]);  out[o, :] = gain * v / sqrt(mean(v^2) + eps).
// Without `rows`: r = o = blockIdx.x and v is written back to h (the residual sum).
// With `rows`: r = rows[o], h is left as it is (used for the last norm, on the rows
// whose logits are wanted).  gain is read as float32 or bfloat16.
template <typename TD, typename TG, typename TO>
__global__ void add_rmsnorm_kernel(float* h, const TD* delta,
                                   const TG* __restrict__ gain, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows,
                                   int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    TO* dst = out + (size_t)o * width;
    if (r < 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_f32<TO>(0.0f);
        return;
    }
    float* hr = h + (size_t)r * width;
    const TD* dr = delta ? delta + (size_t)r * width : nullptr;
    const bool write_back = (rows == nullptr) && (dr != nullptr);
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = hr[i];
        if (dr) v += to_f32<TD>(dr[i]);
        if (write_back) hr[i] = v;
        sum += v * v;
    }
    sum = block_sum(sum, scratch);
    const float scale = 1.0f / sqrtf(sum / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = hr[i];                       // already holds the sum when written back
        if (dr && !write_back) v += to_f32<TD>(dr[i]);
        dst[i] = from_f32<TO>(to_f32<TG>(gain[i]) * v * scale);
    }
}

// Vector form: the row lives in registers between the sum and the scaling, CHUNKS groups of
// eight elements per thread (width <= blockDim * 8 * CHUNKS, width a multiple of 8).
template <typename TD, typename TG, typename TO, int CHUNKS>
__global__ void add_rmsnorm_vec_kernel(float* h, const TD* delta,
                                       const TG* __restrict__ gain, float eps, TO* __restrict__ out,
                                       const int* __restrict__ rows, int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    TO* dst = out + (size_t)o * width;
    const int n_chunks = width >> 3;
    if (r < 0) {
        const float zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) Vec8<TO>::store(dst + c * 8, zero);
        return;
    }
    float* hr = h + (size_t)r * width;
    const TD* dr = delta ? delta + (size_t)r * width : nullptr;
    const bool write_back = (rows == nullptr) && (dr != nullptr);
    float v[CHUNKS][8], d[CHUNKS][8];
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            Vec8<float>::load(hr + c * 8, v[j]);
            if (dr) Vec8<TD>::load(dr + c * 8, d[j]);
        }
    }
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (dr) v[j][e] += d[j][e];
                sum += v[j][e] * v[j][e];
            }
            if (write_back) Vec8<float>::store(hr + c * 8, v[j]);
        }
    }
    sum = block_sum(sum, scratch);
    const float scale = 1.0f / sqrtf(sum / (float)width + eps);
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            float g[8];
            Vec8<TG>::load(gain + c * 8, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] = g[e] * v[j][e] * scale;
            Vec8<TO>::store(dst + c * 8, g);
        }
    }
}

// ---------------------------------------------------------------- norm of a weighted sum, written back as the stream
// For layers that norm after the sum:  v = alpha * h[r, :] + sum_i c_i * d_i[r, :] (+ bias[:]);
// h[r, :] = gain * v / sqrt(mean(v^2) + eps)  (float32, the new stream), out[r, :] = the same in the storage
// type, which the next sub-layer reads.  Up to kMaxSumTerms outputs d_i in the storage type, each with one
// float32 number c_i; gain and bias are float32 vectors.  With no outputs and alpha = 1 it is the plain norm
// of the stream.
constexpr int kMaxSumTerms = 4;
struct SumTerms {
    const void* d[kMaxSumTerms];
    float c[kMaxSumTerms];
    int n;
};

template <typename TD>
__global__ void sum_rmsnorm_kernel(float* h, SumTerms ts, float alpha, const float* __restrict__ bias,
                                   const float* __restrict__ gain, float eps, TD* __restrict__ out, int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int r = blockIdx.x;
    float* hr = h + (size_t)r * width;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = alpha * hr[i];
        for (int k = 0; k < ts.n; ++k) v += ts.c[k] * to_f32<TD>(((const TD*)ts.d[k])[(size_t)r * width + i]);
        if (bias != nullptr) v += bias[i];
        hr[i] = v;
        sum += v * v;
    }
    sum = block_sum(sum, scratch);
    const float scale = 1.0f / sqrtf(sum / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = gain[i] * hr[i] * scale;
        hr[i] = v;
        out[(size_t)r * width + i] = from_f32<TD>(v);
    }
}

template <typename TD, int CHUNKS, int N>
__global__ void sum_rmsnorm_vec_kernel(float* h, SumTerms ts, float alpha, const float* __restrict__ bias,
                                       const float* __restrict__ gain, float eps, TD* __restrict__ out, int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int r = blockIdx.x;
    const int n_chunks = width >> 3;
    float* hr = h + (size_t)r * width;
    float v[CHUNKS][8], d[CHUNKS][N > 0 ? N : 1][8];
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            Vec8<float>::load(hr + c * 8, v[j]);
#pragma unroll
            for (int k = 0; k < N; ++k) Vec8<TD>::load((const TD*)ts.d[k] + (size_t)r * width + c * 8, d[j][k]);
        }
    }
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (bias != nullptr) Vec8<float>::load(bias + c * 8, b);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float x = alpha * v[j][e];
#pragma unroll
                for (int k = 0; k < N; ++k) x += ts.c[k] * d[j][k][e];
                x += b[e];
                v[j][e] = x;
                sum += x * x;
            }
        }
    }
    sum = block_sum(sum, scratch);
    const float scale = 1.0f / sqrtf(sum / (float)width + eps);
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            float g[8];
            Vec8<float>::load(gain + c * 8, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] = g[e] * v[j][e] * scale;
            Vec8<float>::store(hr + c * 8, g);
            Vec8<TD>::store(out + (size_t)r * width + c * 8, g);
        }
    }
}

// ---------------------------------------------------------------- scaled sum of several outputs + layer norm
// For blocks whose sub-layers all read one norm's output and whose outputs are added together, each times a
// vector of its own (a layer scale, a mixing weight, a residual multiplier, all folded into one float32 vector
// per output):  v = h[r, :] + sum_i s_i[:] * d_i[r, :]  (float32, written back without `rows`),
// out[o, :] = gain * (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps).  Rows as in add_rmsnorm.
constexpr int kMaxScaledDeltas = 4;
struct ScaledDeltas {
    const void* d[kMaxScaledDeltas];
    const float* s[kMaxScaledDeltas];
    int n;
};

template <typename TD, typename TG, typename TO>
__global__ void scaled_add_layernorm_kernel(float* h, ScaledDeltas ds, const TG* __restrict__ gain, float eps,
                                            TO* __restrict__ out, const int* __restrict__ rows, int width) {
    extern __shared__ float ln_row[];            // [width]
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    TO* dst = out + (size_t)o * width;
    if (r < 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_f32<TO>(0.0f);
        return;
    }
    float* hr = h + (size_t)r * width;
    const bool write_back = rows == nullptr && ds.n > 0;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = hr[i];
        for (int k = 0; k < ds.n; ++k) v += ds.s[k][i] * to_f32<TD>(((const TD*)ds.d[k])[(size_t)r * width + i]);
        if (write_back) hr[i] = v;
        ln_row[i] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)width;
    float sq = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float d = ln_row[i] - mean;
        sq += d * d;
    }
    const float scale = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        dst[i] = from_f32<TO>(to_f32<TG>(gain[i]) * (ln_row[i] - mean) * scale);
}

// Vector form: the row stays in registers, CHUNKS groups of eight elements per thread.  The number of outputs N
// is a compile-time constant, so that a chunk's loads (the stream, N outputs, N scale vectors) are all in flight
// before the first sum.
template <typename TD, typename TG, typename TO, int CHUNKS, int N>
__global__ void scaled_add_layernorm_vec_kernel(float* h, ScaledDeltas ds, const TG* __restrict__ gain, float eps,
                                                TO* __restrict__ out, const int* __restrict__ rows, int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    TO* dst = out + (size_t)o * width;
    const int n_chunks = width >> 3;
    if (r < 0) {
        const float zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) Vec8<TO>::store(dst + c * 8, zero);
        return;
    }
    float* hr = h + (size_t)r * width;
    const bool write_back = rows == nullptr && N > 0;
    float v[CHUNKS][8];
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            Vec8<float>::load(hr + c * 8, v[j]);
            float d[N > 0 ? N : 1][8], s[N > 0 ? N : 1][8];
#pragma unroll
            for (int k = 0; k < N; ++k) {
                Vec8<TD>::load((const TD*)ds.d[k] + (size_t)r * width + c * 8, d[k]);
                Vec8<float>::load(ds.s[k] + c * 8, s[k]);
            }
#pragma unroll
            for (int k = 0; k < N; ++k) {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[j][e] += s[k][e] * d[k][e];
            }
            if (write_back) Vec8<float>::store(hr + c * 8, v[j]);
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += v[j][e];
        }
    }
    const float mean = block_sum(sum, scratch) / (float)width;
    float sq = 0.0f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[j][e] -= mean;
                sq += v[j][e] * v[j][e];
            }
        }
    }
    const float scale = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            float g[8];
            Vec8<TG>::load(gain + c * 8, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] = g[e] * v[j][e] * scale;
            Vec8<TO>::store(dst + c * 8, g);
        }
    }
}

// ---------------------------------------------------------------- norm of a sub-layer's output + add + RMSNorm
// For blocks that norm a sub-layer's output before the residual sum ("sandwich" norms):
// d' = post_gain * d / sqrt(mean(d^2) + post_eps);  v = h[r, :] + d';  out[o, :] = gain * v / sqrt(mean(v^2) + eps).
// Rows and write-back as in add_rmsnorm; d' never leaves the registers, so the residual sum takes the
// normed output in float32 whatever the storage type.
template <typename TD, typename TG, typename TO>
__global__ void postnorm_add_rmsnorm_kernel(float* h, const TD* delta, const TG* __restrict__ post_gain,
                                            float post_eps, const TG* __restrict__ gain, float eps,
                                            TO* __restrict__ out, const int* __restrict__ rows, int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    TO* dst = out + (size_t)o * width;
    if (r < 0) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_f32<TO>(0.0f);
        return;
    }
    float* hr = h + (size_t)r * width;
    const TD* dr = delta + (size_t)r * width;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float d = to_f32<TD>(dr[i]);
        sum += d * d;
    }
    sum = block_sum(sum, scratch);
    const float post_scale = 1.0f / sqrtf(sum / (float)width + post_eps);
    float sum2 = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = hr[i] + to_f32<TD>(dr[i]) * post_scale * to_f32<TG>(post_gain[i]);
        sum2 += v * v;
    }
    sum2 = block_sum(sum2, scratch);
    const float scale = 1.0f / sqrtf(sum2 / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = hr[i] + to_f32<TD>(dr[i]) * post_scale * to_f32<TG>(post_gain[i]);
        if (rows == nullptr) hr[i] = v;
        dst[i] = from_f32<TO>(v * scale * to_f32<TG>(gain[i]));
    }
}

template <typename TD, typename TG, typename TO, int CHUNKS>
__global__ void postnorm_add_rmsnorm_vec_kernel(float* h, const TD* delta, const TG* __restrict__ post_gain,
                                                float post_eps, const TG* __restrict__ gain, float eps,
                                                TO* __restrict__ out, const int* __restrict__ rows, int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    TO* dst = out + (size_t)o * width;
    const int n_chunks = width >> 3;
    if (r < 0) {
        const float zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) Vec8<TO>::store(dst + c * 8, zero);
        return;
    }
    float* hr = h + (size_t)r * width;
    const TD* dr = delta + (size_t)r * width;
    float v[CHUNKS][8], d[CHUNKS][8];
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            Vec8<float>::load(hr + c * 8, v[j]);
            Vec8<TD>::load(dr + c * 8, d[j]);
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += d[j][e] * d[j][e];
        }
    }
    sum = block_sum(sum, scratch);
    const float post_scale = 1.0f / sqrtf(sum / (float)width + post_eps);
    float sum2 = 0.0f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            float g[8];
            Vec8<TG>::load(post_gain + c * 8, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[j][e] += d[j][e] * post_scale * g[e];
                sum2 += v[j][e] * v[j][e];
            }
            if (rows == nullptr) Vec8<float>::store(hr + c * 8, v[j]);
        }
    }
    sum2 = block_sum(sum2, scratch);
    const float scale = 1.0f / sqrtf(sum2 / (float)width + eps);
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            float g[8];
            Vec8<TG>::load(gain + c * 8, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] = v[j][e] * scale * g[e];
            Vec8<TO>::store(dst + c * 8, g);
        }
    }
}

// ---------------------------------------------------------------- SwiGLU
// out[t, i] = act(gate) * up in float32; act is silu(x) = x / (1 + exp(-x)) or the tanh form of
// GELU (`gate_act` in common.cuh).  Stacked columns: gate at
// gu[t, i], up at gu[t, inter + i].  Interleaved by eight: columns come in groups of sixteen,
// eight gates followed by their eight ups, so gate at gu[t, 16 (i / 8) + i % 8] and up 8 further.
template <typename T>
__global__ void swiglu_kernel(const T* gu, T* out, int inter, int interleaved, int act,
                              size_t total) {
    TLLM_PDL_ENTER();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const size_t t = idx / inter, i = idx - t * inter;
        const size_t gi = interleaved ? 16 * (i >> 3) + (i & 7) : i, ui = interleaved ? gi + 8 : inter + i;
        const float g = to_f32<T>(gu[t * 2 * inter + gi]);
        const float u = to_f32<T>(gu[t * 2 * inter + ui]);
        out[idx] = from_f32<T>(gate_act(g, act) * u);
    }
}

template <typename T>
__global__ void swiglu_vec_kernel(const T* gu, T* out, int inter, int interleaved, int act,
                                  size_t total_chunks) {
    TLLM_PDL_ENTER();
    const int per_row = inter >> 3;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total_chunks; idx += stride) {
        const size_t t = idx / per_row, c = idx - t * per_row;
        float g[8], u[8];
        Vec8<T>::load(gu + t * 2 * inter + (interleaved ? c * 16 : c * 8), g);
        Vec8<T>::load(gu + t * 2 * inter + (interleaved ? c * 16 + 8 : inter + c * 8), u);
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] = gate_act(g[e], act) * u[e];
        Vec8<T>::store(out + t * inter + c * 8, g);
    }
}

// ---------------------------------------------------------------- embedding + learned position + norm
// v = table[ids[t], :] * scale + pos_table[positions[t], :] (the position part only if a table is given);
// out[t, :] = gain * v / sqrt(mean(v^2) + eps) if a gain is given, else v.  All in float32; `gain` is
// float32 and holds the factor itself.  Rows with ids[t] < 0 become zero.
template <typename TW>
__global__ void embedding_norm_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                      const TW* __restrict__ table, const TW* __restrict__ pos_table,
                                      const float* __restrict__ gain, float eps, float scale, float* __restrict__ out,
                                      int hidden, int vocab, int max_positions) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    if (id < 0) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.0f;
        return;
    }
    if (id >= vocab) id = vocab - 1;
    const TW* src = table + (size_t)id * hidden;
    const TW* prow = nullptr;
    if (pos_table != nullptr) {
        int p = positions[t];
        p = p < 0 ? 0 : (p >= max_positions ? max_positions - 1 : p);     // the host refuses positions past the table
        prow = pos_table + (size_t)p * hidden;
    }
    float sum = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = to_f32<TW>(src[i]) * scale;
        if (prow != nullptr) v += to_f32<TW>(prow[i]);
        dst[i] = v;
        sum += v * v;
    }
    if (gain == nullptr) return;
    sum = block_sum(sum, scratch);
    const float sc = 1.0f / sqrtf(sum / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = dst[i] * sc * gain[i];
}

// Vector form: the row stays in registers between the sum and the scaling (hidden a multiple of 8, at most
// blockDim * 8 * CHUNKS).
template <typename TW, int CHUNKS>
__global__ void embedding_norm_vec_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                          const TW* __restrict__ table, const TW* __restrict__ pos_table,
                                          const float* __restrict__ gain, float eps, float scale, float* __restrict__ out,
                                          int hidden, int vocab, int max_positions) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    int id = ids[t];
    float* dst = out + (size_t)t * hidden;
    const int n_chunks = hidden >> 3;
    if (id < 0) {
        const float zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) Vec8<float>::store(dst + c * 8, zero);
        return;
    }
    if (id >= vocab) id = vocab - 1;
    const TW* src = table + (size_t)id * hidden;
    const TW* prow = nullptr;
    if (pos_table != nullptr) {
        int p = positions[t];
        p = p < 0 ? 0 : (p >= max_positions ? max_positions - 1 : p);
        prow = pos_table + (size_t)p * hidden;
    }
    float v[CHUNKS][8];
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            Vec8<TW>::load(src + c * 8, v[j]);
            float p[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (prow != nullptr) Vec8<TW>::load(prow + c * 8, p);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                v[j][e] = v[j][e] * scale + p[e];
                sum += v[j][e] * v[j][e];
            }
        }
    }
    float sc = 1.0f;
    if (gain != nullptr) {
        sum = block_sum(sum, scratch);
        sc = 1.0f / sqrtf(sum / (float)hidden + eps);
    }
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            if (gain != nullptr) {
                float g[8];
                Vec8<float>::load(gain + c * 8, g);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[j][e] = v[j][e] * sc * g[e];
            }
            Vec8<float>::store(dst + c * 8, v[j]);
        }
    }
}

// ---------------------------------------------------------------- residual sum without a norm behind it
// For blocks whose sub-layers read the stream itself: h[r, :] += d' and out[r, :] = h[r, :] in the storage
// type, with d' = delta, or, with `post_gain`, post_gain * delta / sqrt(mean(delta^2) + post_eps) in float32.
template <typename TD, typename TG, typename TO>
__global__ void stream_add_kernel(float* h, const TD* delta, const TG* __restrict__ post_gain, float post_eps,
                                  TO* __restrict__ out, int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int r = blockIdx.x;
    float* hr = h + (size_t)r * width;
    TO* dst = out + (size_t)r * width;
    if (delta == nullptr) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_f32<TO>(hr[i]);
        return;
    }
    const TD* dr = delta + (size_t)r * width;
    float post_scale = 1.0f;
    if (post_gain != nullptr) {
        float sum = 0.0f;
        for (int i = threadIdx.x; i < width; i += blockDim.x) { const float d = to_f32<TD>(dr[i]); sum += d * d; }
        sum = block_sum(sum, scratch);
        post_scale = 1.0f / sqrtf(sum / (float)width + post_eps);
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float d = to_f32<TD>(dr[i]);
        if (post_gain != nullptr) d = d * post_scale * to_f32<TG>(post_gain[i]);
        const float v = hr[i] + d;
        hr[i] = v;
        dst[i] = from_f32<TO>(v);
    }
}

// Vector form of stream_add: the row lives in registers between the delta's sum of squares and the writes
// (width a multiple of 8, at most blockDim * 8 * CHUNKS).
template <typename TD, typename TG, typename TO, int CHUNKS>
__global__ void stream_add_vec_kernel(float* h, const TD* delta, const TG* __restrict__ post_gain, float post_eps,
                                      TO* __restrict__ out, int width) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int r = blockIdx.x;
    float* hr = h + (size_t)r * width;
    TO* dst = out + (size_t)r * width;
    const TD* dr = delta != nullptr ? delta + (size_t)r * width : nullptr;
    const int n_chunks = width >> 3;
    float v[CHUNKS][8], d[CHUNKS][8];
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            Vec8<float>::load(hr + c * 8, v[j]);
            if (dr != nullptr) {
                Vec8<TD>::load(dr + c * 8, d[j]);
#pragma unroll
                for (int e = 0; e < 8; ++e) sum += d[j][e] * d[j][e];
            }
        }
    }
    float post_scale = 1.0f;
    if (post_gain != nullptr) {
        sum = block_sum(sum, scratch);
        post_scale = 1.0f / sqrtf(sum / (float)width + post_eps);
    }
#pragma unroll
    for (int j = 0; j < CHUNKS; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < n_chunks) {
            if (dr != nullptr) {
                if (post_gain != nullptr) {
                    float g[8];
                    Vec8<TG>::load(post_gain + c * 8, g);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[j][e] += d[j][e] * post_scale * g[e];
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[j][e] += d[j][e];
                }
                Vec8<float>::store(hr + c * 8, v[j]);
            }
            Vec8<TO>::store(dst + c * 8, v[j]);
        }
    }
}

// ---------------------------------------------------------------- activations
// out = act(x) (codes of `gate_act`), or, with a table, out[t, j] = act(x[t, j]) * table[ids[t], col0 + j]:
// a gate on a per-token vector looked up by the token's id.
template <typename T>
__global__ void activation_kernel(const T* x, T* out, int act, int width, size_t total, const int* __restrict__ ids,
                                  const T* __restrict__ table, int ldt, int col0, int vocab) {
    TLLM_PDL_ENTER();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        float v = gate_act(to_f32<T>(x[idx]), act);
        if (table != nullptr) {
            const size_t t = idx / width, j = idx - t * width;
            int id = ids[t];
            if (id < 0) { out[idx] = from_f32<T>(0.0f); continue; }
            if (id >= vocab) id = vocab - 1;
            v *= to_f32<T>(table[(size_t)id * ldt + col0 + j]);
        }
        out[idx] = from_f32<T>(v);
    }
}

// Vector form without a table: eight elements per access.
template <typename T>
__global__ void activation_vec_kernel(const T* x, T* out, int act, size_t chunks) {
    TLLM_PDL_ENTER();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < chunks; idx += stride) {
        float v[8];
        Vec8<T>::load(x + idx * 8, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = gate_act(v[e], act);
        Vec8<T>::store(out + idx * 8, v);
    }
}

// x <- cap * tanh(x / cap), in place (a bound on logits).
__global__ void softcap_kernel(float* x, float cap, float inv_cap, size_t n) {
    TLLM_PDL_ENTER();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < n; idx += stride) x[idx] = cap * tanhf(x[idx] * inv_cap);
}

__global__ void feed_tokens_kernel(int* ids, const int* places, const int* rows, const int* sampled, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ids[places[i]] = sampled[rows[i]];
}

template <typename TS, typename TD>
__global__ void cast_kernel(const TS* __restrict__ src, TD* __restrict__ dst, size_t n) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < n; idx += stride) dst[idx] = from_f32<TD>(to_f32<TS>(src[idx]));
}

static int grid_for(size_t total, int block) {
    size_t g = (total + block - 1) / block;
    const size_t cap = 148 * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename TD, typename TG, typename TO>
static int launch_add_rmsnorm_typed(float* h, const void* delta, const void* gain, float eps, void* out,
                                    const int* rows, int n_out, int width, cudaStream_t stream) {
    const bool vec = width % 8 == 0 && aligned16(h) && aligned16(delta) && aligned16(gain) && aligned16(out);
    const int chunks = width / 8;
    if (vec && chunks <= 1024 * 4) {
        int block = 64;
        while (block < 1024 && block < chunks) block *= 2;
        const int per_thread = (chunks + block - 1) / block;
#define VEC_LAUNCH(C)                                                                 \
    launch_pdl(kPdlNorm, add_rmsnorm_vec_kernel<TD, TG, TO, C>, dim3(n_out), dim3(block), 0, stream, \
               h, (const TD*)delta, (const TG*)gain, eps, (TO*)out, rows, width)
        if (per_thread <= 1) VEC_LAUNCH(1);
        else if (per_thread <= 2) VEC_LAUNCH(2);
        else VEC_LAUNCH(4);
#undef VEC_LAUNCH
    } else {
        const int block = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
        launch_pdl(kPdlNorm, add_rmsnorm_kernel<TD, TG, TO>, dim3(n_out), dim3(block), 0, stream,
                   h, (const TD*)delta, (const TG*)gain, eps, (TO*)out, rows, width);
    }
    return finish_launch("add_rmsnorm");
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* h, const void* delta, const void* gain, int gain_dtype,
                              float eps, void* out, const int* rows, int n_out, int width,
                              cudaStream_t stream) {
    if (gain_dtype == kBF16)
        return launch_add_rmsnorm_typed<TD, bf16, TO>(h, delta, gain, eps, out, rows, n_out, width, stream);
    return launch_add_rmsnorm_typed<TD, float, TO>(h, delta, gain, eps, out, rows, n_out, width, stream);
}

template <typename TD, typename TG, typename TO>
static int launch_postnorm_typed(float* h, const void* delta, const void* post_gain, float post_eps,
                                 const void* gain, float eps, void* out, const int* rows, int n_out,
                                 int width, cudaStream_t stream) {
    const bool vec = width % 8 == 0 && aligned16(h) && aligned16(delta) && aligned16(gain) &&
                     aligned16(post_gain) && aligned16(out);
    const int chunks = width / 8;
    if (vec && chunks <= 1024 * 4) {
        int block = 64;
        while (block < 1024 && block < chunks) block *= 2;
        const int per_thread = (chunks + block - 1) / block;
#define VEC_LAUNCH(C)                                                                                        \
    launch_pdl(kPdlNorm, postnorm_add_rmsnorm_vec_kernel<TD, TG, TO, C>, dim3(n_out), dim3(block), 0, stream, \
               h, (const TD*)delta, (const TG*)post_gain, post_eps, (const TG*)gain, eps, (TO*)out, rows, width)
        if (per_thread <= 1) VEC_LAUNCH(1);
        else if (per_thread <= 2) VEC_LAUNCH(2);
        else VEC_LAUNCH(4);
#undef VEC_LAUNCH
    } else {
        const int block = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
        launch_pdl(kPdlNorm, postnorm_add_rmsnorm_kernel<TD, TG, TO>, dim3(n_out), dim3(block), 0, stream,
                   h, (const TD*)delta, (const TG*)post_gain, post_eps, (const TG*)gain, eps, (TO*)out, rows, width);
    }
    return finish_launch("postnorm_add_rmsnorm");
}

template <typename TD, typename TG, typename TO>
static int launch_scaled_layernorm_typed(float* h, const ScaledDeltas& ds, const void* gain, float eps, void* out,
                                         const int* rows, int n_out, int width, cudaStream_t stream) {
    bool vec = width % 8 == 0 && aligned16(h) && aligned16(gain) && aligned16(out);
    for (int k = 0; k < ds.n; ++k) vec = vec && aligned16(ds.d[k]) && aligned16(ds.s[k]);
    const int chunks = width / 8;
    if (vec && chunks <= 1024 * 4) {
        int block = 64;
        while (block < 1024 && block < chunks) block *= 2;
        const int per_thread = (chunks + block - 1) / block;
#define VEC_LAUNCH_N(C, N)                                                                                       \
    launch_pdl(kPdlNorm, scaled_add_layernorm_vec_kernel<TD, TG, TO, C, N>, dim3(n_out), dim3(block), 0, stream, \
               h, ds, (const TG*)gain, eps, (TO*)out, rows, width)
#define VEC_LAUNCH(C)                                            \
    switch (ds.n) {                                              \
        case 0: VEC_LAUNCH_N(C, 0); break;                       \
        case 1: VEC_LAUNCH_N(C, 1); break;                       \
        case 2: VEC_LAUNCH_N(C, 2); break;                       \
        case 3: VEC_LAUNCH_N(C, 3); break;                       \
        default: VEC_LAUNCH_N(C, 4); break;                      \
    }
        if (per_thread <= 1) { VEC_LAUNCH(1) }
        else if (per_thread <= 2) { VEC_LAUNCH(2) }
        else { VEC_LAUNCH(4) }
#undef VEC_LAUNCH
#undef VEC_LAUNCH_N
    } else {
        const size_t smem = (size_t)width * sizeof(float);
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(scaled_add_layernorm_kernel<TD, TG, TO>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) { set_error("scaled_add_layernorm: %s", cudaGetErrorString(e)); return (int)e; }
        }
        const int block = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
        launch_pdl(kPdlNorm, scaled_add_layernorm_kernel<TD, TG, TO>, dim3(n_out), dim3(block), smem, stream,
                   h, ds, (const TG*)gain, eps, (TO*)out, rows, width);
    }
    return finish_launch("scaled_add_layernorm");
}

template <typename TD>
static int launch_sum_rmsnorm_typed(float* h, const SumTerms& ts, float alpha, const float* bias, const float* gain,
                                    float eps, void* out, int n_rows, int width, cudaStream_t stream) {
    bool vec = width % 8 == 0 && aligned16(h) && aligned16(gain) && aligned16(out) && aligned16(bias);
    for (int k = 0; k < ts.n; ++k) vec = vec && aligned16(ts.d[k]);
    const int chunks = width / 8;
    if (vec && chunks <= 1024 * 4) {
        int block = 64;
        while (block < 1024 && block < chunks) block *= 2;
        const int per_thread = (chunks + block - 1) / block;
#define VEC_LAUNCH_N(C, N)                                                                                 \
    launch_pdl(kPdlNorm, sum_rmsnorm_vec_kernel<TD, C, N>, dim3(n_rows), dim3(block), 0, stream, h, ts,    \
               alpha, bias, gain, eps, (TD*)out, width)
#define VEC_LAUNCH(C)                                            \
    switch (ts.n) {                                              \
        case 0: VEC_LAUNCH_N(C, 0); break;                       \
        case 1: VEC_LAUNCH_N(C, 1); break;                       \
        case 2: VEC_LAUNCH_N(C, 2); break;                       \
        case 3: VEC_LAUNCH_N(C, 3); break;                       \
        default: VEC_LAUNCH_N(C, 4); break;                      \
    }
        if (per_thread <= 1) { VEC_LAUNCH(1) }
        else if (per_thread <= 2) { VEC_LAUNCH(2) }
        else { VEC_LAUNCH(4) }
#undef VEC_LAUNCH
#undef VEC_LAUNCH_N
    } else {
        const int block = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
        launch_pdl(kPdlNorm, sum_rmsnorm_kernel<TD>, dim3(n_rows), dim3(block), 0, stream, h, ts, alpha, bias, gain,
                   eps, (TD*)out, width);
    }
    return finish_launch("sum_rmsnorm");
}

}  // namespace tllm

using namespace tllm;

extern "C" {

// h <- gain * v / sqrt(mean(v^2) + eps) with v = alpha * h + sum_i coefs[i] * deltas[i] (+ bias), every row; out gets
// the new h in the storage type `act_dtype` (that of the deltas).  gain and bias float32; bias may be null.
int tllm_sum_rmsnorm(float* h, const void* const* deltas, const float* coefs, int n, float alpha, const float* bias,
                     const float* gain, float eps, void* out, int act_dtype, int n_rows, int width, cudaStream_t stream) {
    TLLM_REQUIRE(n_rows >= 0 && width > 0 && n >= 0 && n <= kMaxSumTerms, "sum_rmsnorm: bad sizes");
    TLLM_REQUIRE(eps > 0.0f && gain != nullptr && out != nullptr, "sum_rmsnorm: missing operand");
    if (n_rows == 0) return 0;
    SumTerms ts;
    ts.n = n;
    for (int k = 0; k < kMaxSumTerms; ++k) { ts.d[k] = k < n ? deltas[k] : nullptr; ts.c[k] = k < n ? coefs[k] : 0.0f; }
    if (act_dtype == kBF16) return launch_sum_rmsnorm_typed<bf16>(h, ts, alpha, bias, gain, eps, out, n_rows, width, stream);
    if (act_dtype == kF32) return launch_sum_rmsnorm_typed<float>(h, ts, alpha, bias, gain, eps, out, n_rows, width, stream);
    TLLM_REQUIRE(false, "sum_rmsnorm: unknown dtype %d", act_dtype);
}

// h += sum over `n` outputs of scales[i] * deltas[i] (float32 vectors of the row's width; outputs in the
// storage type), then the layer norm of the sum (mean taken off, gain, no bias).  `n` may be 0.
int tllm_scaled_add_layernorm(float* h, const void* const* deltas, const float* const* scales, int n, const void* gain,
                              int gain_dtype, float eps, void* out, int act_dtype, const int* rows, int n_out,
                              int width, cudaStream_t stream) {
    TLLM_REQUIRE(n_out >= 0 && width > 0 && n >= 0 && n <= kMaxScaledDeltas, "scaled_add_layernorm: bad sizes");
    TLLM_REQUIRE(width <= 50 * 1024, "scaled_add_layernorm: rows of %d elements are too wide", width);
    TLLM_REQUIRE(gain_dtype == kBF16 || gain_dtype == kF32, "scaled_add_layernorm: unknown gain dtype");
    TLLM_REQUIRE(eps > 0.0f && gain != nullptr, "scaled_add_layernorm: eps must be positive and the gain given");
    if (n_out == 0) return 0;
    ScaledDeltas ds = {};
    ds.n = n;
    for (int k = 0; k < n; ++k) {
        TLLM_REQUIRE(deltas[k] != nullptr && scales[k] != nullptr, "scaled_add_layernorm: missing operand");
        ds.d[k] = deltas[k];
        ds.s[k] = scales[k];
    }
#define LNORM(TD, TG, TO) launch_scaled_layernorm_typed<TD, TG, TO>(h, ds, gain, eps, out, rows, n_out, width, stream)
    if (act_dtype == kBF16) return gain_dtype == kBF16 ? LNORM(bf16, bf16, bf16) : LNORM(bf16, float, bf16);
    if (act_dtype == kF32) return gain_dtype == kBF16 ? LNORM(float, bf16, float) : LNORM(float, float, float);
#undef LNORM
    TLLM_REQUIRE(false, "scaled_add_layernorm: unknown dtype %d", act_dtype);
}

const char* tllm_last_error() { return g_error; }

int tllm_embedding(const int* ids, const void* table, int table_dtype, float* out, int tokens,
                   int hidden, int vocab, float scale, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes");
    TLLM_REQUIRE(table_dtype == kBF16 || table_dtype == kF32, "embedding: unknown dtype %d", table_dtype);
    if (tokens == 0) return 0;
    const bool vec = hidden % 8 == 0 && aligned16(table) && aligned16(out);
    const int block = vec ? (hidden >= 2048 ? 256 : 128) : (hidden >= 1024 ? 256 : 128);
    if (table_dtype == kBF16) {
        if (vec) launch_pdl(kPdlOther, embedding_vec_kernel<bf16>, dim3(tokens), dim3(block), 0, stream, ids, (const bf16*)table, out, hidden, vocab, scale);
        else launch_pdl(kPdlOther, embedding_kernel<bf16>, dim3(tokens), dim3(block), 0, stream, ids, (const bf16*)table, out, hidden, vocab, scale);
    } else {
        if (vec) launch_pdl(kPdlOther, embedding_vec_kernel<float>, dim3(tokens), dim3(block), 0, stream, ids, (const float*)table, out, hidden, vocab, scale);
        else launch_pdl(kPdlOther, embedding_kernel<float>, dim3(tokens), dim3(block), 0, stream, ids, (const float*)table, out, hidden, vocab, scale);
    }
    return finish_launch("embedding");
}

// Embedding with an optional learned position table and an optional norm (gain in float32, the factor itself).
int tllm_embedding_norm(const int* ids, const int* positions, const void* table, const void* pos_table, int table_dtype,
                        const float* gain, float eps, float scale, float* out, int tokens, int hidden, int vocab,
                        int max_positions, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding_norm: bad sizes");
    TLLM_REQUIRE(pos_table == nullptr || (positions != nullptr && max_positions > 0), "embedding_norm: a position table without positions");
    TLLM_REQUIRE(gain == nullptr || eps > 0.0f, "embedding_norm: eps must be positive");
    if (tokens == 0) return 0;
    const int block = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (hidden % 8 == 0 && hidden / 8 <= 1024 * 4 && aligned16(table) && aligned16(pos_table) && aligned16(gain) && aligned16(out)
        && (table_dtype == kBF16 || table_dtype == kF32)) {
        int vblock = 64;
        while (vblock < 1024 && vblock < hidden / 8) vblock *= 2;
        const int per_thread = (hidden / 8 + vblock - 1) / vblock;
#define EVEC(TW, C) launch_pdl(kPdlOther, embedding_norm_vec_kernel<TW, C>, dim3(tokens), dim3(vblock), 0, stream, ids, positions, \
                               (const TW*)table, (const TW*)pos_table, gain, eps, scale, out, hidden, vocab, max_positions)
        if (table_dtype == kBF16) { if (per_thread <= 1) EVEC(bf16, 1); else if (per_thread <= 2) EVEC(bf16, 2); else EVEC(bf16, 4); }
        else { if (per_thread <= 1) EVEC(float, 1); else if (per_thread <= 2) EVEC(float, 2); else EVEC(float, 4); }
#undef EVEC
        return finish_launch("embedding_norm");
    }
    if (table_dtype == kBF16)
        launch_pdl(kPdlOther, embedding_norm_kernel<bf16>, dim3(tokens), dim3(block), 0, stream, ids, positions, (const bf16*)table,
                   (const bf16*)pos_table, gain, eps, scale, out, hidden, vocab, max_positions);
    else if (table_dtype == kF32)
        launch_pdl(kPdlOther, embedding_norm_kernel<float>, dim3(tokens), dim3(block), 0, stream, ids, positions, (const float*)table,
                   (const float*)pos_table, gain, eps, scale, out, hidden, vocab, max_positions);
    else TLLM_REQUIRE(false, "embedding_norm: unknown dtype %d", table_dtype);
    return finish_launch("embedding_norm");
}

// h += delta (normed first if `post_gain` is given) and out = h in the storage type `act_dtype` (also delta's).
int tllm_stream_add(float* h, const void* delta, const void* post_gain, int gain_dtype, float post_eps, void* out,
                    int act_dtype, int rows, int width, cudaStream_t stream) {
    TLLM_REQUIRE(rows >= 0 && width > 0, "stream_add: bad sizes");
    TLLM_REQUIRE(post_gain == nullptr || (delta != nullptr && post_eps > 0.0f), "stream_add: a gain without a delta or eps");
    TLLM_REQUIRE(gain_dtype == kBF16 || gain_dtype == kF32, "stream_add: unknown gain dtype");
    if (rows == 0) return 0;
    const int block = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    const bool vec = width % 8 == 0 && aligned16(h) && aligned16(delta) && aligned16(post_gain) && aligned16(out) && width / 8 <= 1024 * 4;
    int vblock = 64;
    while (vblock < 1024 && vblock < width / 8) vblock *= 2;
    const int per_thread = vec ? (width / 8 + vblock - 1) / vblock : 0;
#define SADD(TD, TG, TO)                                                                                                   \
    do {                                                                                                                   \
        if (vec && per_thread <= 1)                                                                                        \
            launch_pdl(kPdlNorm, stream_add_vec_kernel<TD, TG, TO, 1>, dim3(rows), dim3(vblock), 0, stream, h, (const TD*)delta, \
                       (const TG*)post_gain, post_eps, (TO*)out, width);                                                   \
        else if (vec && per_thread <= 2)                                                                                   \
            launch_pdl(kPdlNorm, stream_add_vec_kernel<TD, TG, TO, 2>, dim3(rows), dim3(vblock), 0, stream, h, (const TD*)delta, \
                       (const TG*)post_gain, post_eps, (TO*)out, width);                                                   \
        else if (vec)                                                                                                      \
            launch_pdl(kPdlNorm, stream_add_vec_kernel<TD, TG, TO, 4>, dim3(rows), dim3(vblock), 0, stream, h, (const TD*)delta, \
                       (const TG*)post_gain, post_eps, (TO*)out, width);                                                   \
        else                                                                                                               \
            launch_pdl(kPdlNorm, stream_add_kernel<TD, TG, TO>, dim3(rows), dim3(block), 0, stream, h, (const TD*)delta,   \
                       (const TG*)post_gain, post_eps, (TO*)out, width);                                                   \
    } while (0)
    if (act_dtype == kBF16) { if (gain_dtype == kBF16) SADD(bf16, bf16, bf16); else SADD(bf16, float, bf16); }
    else if (act_dtype == kF32) { if (gain_dtype == kBF16) SADD(float, bf16, float); else SADD(float, float, float); }
    else TLLM_REQUIRE(false, "stream_add: unknown dtype %d", act_dtype);
#undef SADD
    return finish_launch("stream_add");
}

int tllm_softcap(float* x, float cap, long long n, cudaStream_t stream) {
    TLLM_REQUIRE(n >= 0 && cap > 0.0f, "softcap: bad arguments");
    if (n == 0) return 0;
    launch_pdl(kPdlOther, softcap_kernel, dim3(grid_for((size_t)n, 256)), dim3(256), 0, stream, x, cap, 1.0f / cap, (size_t)n);
    return finish_launch("softcap");
}

// out = act(x), times table[ids[t], col0 + j] where a table is given (x and out [tokens, width]).
int tllm_activation(const void* x, void* out, int dtype, int act, int tokens, int width, const int* ids,
                    const void* table, int ldt, int col0, int vocab, cudaStream_t stream) {
    TLLM_REQUIRE(act == kActSilu || act == kActGeluTanh || act == kActGeluErf || act == kActRelu2, "activation: unknown activation %d", act);
    TLLM_REQUIRE(tokens >= 0 && width > 0, "activation: bad sizes");
    TLLM_REQUIRE(table == nullptr || (ids != nullptr && col0 >= 0 && col0 + width <= ldt && vocab > 0), "activation: bad table");
    const size_t total = (size_t)tokens * width;
    if (total == 0) return 0;
    const int block = 256, grid = grid_for(total, block);
    if (table == nullptr && total % 8 == 0 && aligned16(x) && aligned16(out) && (dtype == kBF16 || dtype == kF32)) {
        const size_t chunks = total / 8;
        const int vgrid = grid_for(chunks, block);
        if (dtype == kBF16)
            launch_pdl(kPdlSwiglu, activation_vec_kernel<bf16>, dim3(vgrid), dim3(block), 0, stream, (const bf16*)x, (bf16*)out, act, chunks);
        else
            launch_pdl(kPdlSwiglu, activation_vec_kernel<float>, dim3(vgrid), dim3(block), 0, stream, (const float*)x, (float*)out, act, chunks);
        return finish_launch("activation");
    }
    if (dtype == kBF16)
        launch_pdl(kPdlSwiglu, activation_kernel<bf16>, dim3(grid), dim3(block), 0, stream, (const bf16*)x, (bf16*)out, act, width, total,
                   ids, (const bf16*)table, ldt, col0, vocab);
    else if (dtype == kF32)
        launch_pdl(kPdlSwiglu, activation_kernel<float>, dim3(grid), dim3(block), 0, stream, (const float*)x, (float*)out, act, width, total,
                   ids, (const float*)table, ldt, col0, vocab);
    else TLLM_REQUIRE(false, "activation: unknown dtype %d", dtype);
    return finish_launch("activation");
}

// act_dtype is the storage type of both `delta` and `out`.
int tllm_add_rmsnorm(float* h, const void* delta, const void* gain, int gain_dtype, float eps,
                     void* out, int act_dtype, const int* rows, int n_out, int width,
                     cudaStream_t stream) {
    TLLM_REQUIRE(n_out >= 0 && width > 0, "add_rmsnorm: bad sizes");
    TLLM_REQUIRE(gain_dtype == kBF16 || gain_dtype == kF32, "add_rmsnorm: unknown gain dtype");
    TLLM_REQUIRE(eps > 0.0f, "add_rmsnorm: eps must be positive");
    if (n_out == 0) return 0;
    if (act_dtype == kBF16)
        return launch_add_rmsnorm<bf16, bf16>(h, delta, gain, gain_dtype, eps, out, rows, n_out, width, stream);
    if (act_dtype == kF32)
        return launch_add_rmsnorm<float, float>(h, delta, gain, gain_dtype, eps, out, rows, n_out, width, stream);
    TLLM_REQUIRE(false, "add_rmsnorm: unknown dtype %d", act_dtype);
}

// As tllm_add_rmsnorm with `delta` normed (gain `post_gain`, `post_eps`) before it is added.  Both
// gains have the storage type `gain_dtype`.
int tllm_postnorm_add_rmsnorm(float* h, const void* delta, const void* post_gain, float post_eps,
                              const void* gain, int gain_dtype, float eps, void* out, int act_dtype,
                              const int* rows, int n_out, int width, cudaStream_t stream) {
    TLLM_REQUIRE(n_out >= 0 && width > 0, "postnorm_add_rmsnorm: bad sizes");
    TLLM_REQUIRE(delta != nullptr && post_gain != nullptr && gain != nullptr, "postnorm_add_rmsnorm: missing operand");
    TLLM_REQUIRE(gain_dtype == kBF16 || gain_dtype == kF32, "postnorm_add_rmsnorm: unknown gain dtype");
    TLLM_REQUIRE(eps > 0.0f && post_eps > 0.0f, "postnorm_add_rmsnorm: eps must be positive");
    if (n_out == 0) return 0;
#define POSTNORM(TD, TG, TO) launch_postnorm_typed<TD, TG, TO>(h, delta, post_gain, post_eps, gain, eps, out, rows, n_out, width, stream)
    if (act_dtype == kBF16) return gain_dtype == kBF16 ? POSTNORM(bf16, bf16, bf16) : POSTNORM(bf16, float, bf16);
    if (act_dtype == kF32) return gain_dtype == kBF16 ? POSTNORM(float, bf16, float) : POSTNORM(float, float, float);
#undef POSTNORM
    TLLM_REQUIRE(false, "postnorm_add_rmsnorm: unknown dtype %d", act_dtype);
}

int tllm_swiglu(const void* gate_up, void* out, int dtype, int tokens, int inter, int interleaved,
                int act, cudaStream_t stream) {
    TLLM_REQUIRE(act == kActSilu || act == kActGeluTanh, "swiglu: unknown activation %d", act);
    TLLM_REQUIRE(tokens >= 0 && inter > 0, "swiglu: bad sizes");
    TLLM_REQUIRE(!interleaved || inter % 8 == 0, "swiglu: interleaved columns need a multiple of 8, not %d", inter);
    TLLM_REQUIRE(dtype == kBF16 || dtype == kF32, "swiglu: unknown dtype %d", dtype);
    const size_t total = (size_t)tokens * inter;
    if (total == 0) return 0;
    const int block = 256;
    if (inter % 8 == 0 && aligned16(gate_up) && aligned16(out)) {
        const size_t chunks = total / 8;
        const int grid = grid_for(chunks, block);
        if (dtype == kBF16)
            launch_pdl(kPdlSwiglu, swiglu_vec_kernel<bf16>, dim3(grid), dim3(block), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, interleaved, act, chunks);
        else
            launch_pdl(kPdlSwiglu, swiglu_vec_kernel<float>, dim3(grid), dim3(block), 0, stream, (const float*)gate_up, (float*)out, inter, interleaved, act, chunks);
    } else {
        const int grid = grid_for(total, block);
        if (dtype == kBF16)
            launch_pdl(kPdlSwiglu, swiglu_kernel<bf16>, dim3(grid), dim3(block), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, interleaved, act, total);
        else
            launch_pdl(kPdlSwiglu, swiglu_kernel<float>, dim3(grid), dim3(block), 0, stream, (const float*)gate_up, (float*)out, inter, interleaved, act, total);
    }
    return finish_launch("swiglu");
}

// ids[places[i]] = sampled[rows[i]] for i < n: tokens that a step still being sampled from gives
// the next step, without the host in between.  All four are device arrays of int32.
int tllm_feed_tokens(int* ids, const int* places, const int* rows, const int* sampled, int n, cudaStream_t stream) {
    TLLM_REQUIRE(n >= 0 && ids && places && rows && sampled, "feed_tokens: bad arguments");
    if (n == 0) return 0;
    feed_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(ids, places, rows, sampled, n);
    return finish_launch("feed_tokens");
}

int tllm_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n,
              cudaStream_t stream) {
    TLLM_REQUIRE(n >= 0, "cast: bad size");
    if (n == 0) return 0;
    const int block = 256, grid = grid_for((size_t)n, block);
    if (src_dtype == kBF16 && dst_dtype == kF32)
        cast_kernel<bf16, float><<<grid, block, 0, stream>>>((const bf16*)src, (float*)dst, (size_t)n);
    else if (src_dtype == kF32 && dst_dtype == kBF16)
        cast_kernel<float, bf16><<<grid, block, 0, stream>>>((const float*)src, (bf16*)dst, (size_t)n);
    else
        TLLM_REQUIRE(false, "cast: unsupported pair %d -> %d", src_dtype, dst_dtype);
    return finish_launch("cast");
}

}  // extern "C"
