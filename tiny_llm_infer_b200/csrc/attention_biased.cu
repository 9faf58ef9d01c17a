// Attention over the paged cache with a modified score: keys and values in planes of their own
// (their widths may differ), and between the dot product and the softmax any of
//   a cap          s <- cap * tanh(s / cap),
//   a distance bias s <- s - slope[head] * (pos_query - pos_key),
//   a chunk mask   keys only from the query's own chunk of `chunk` positions (counted from 0),
//   a window       keys pos - window + 1 .. pos,
//   a sink         one more term in the softmax's denominator that carries no value: exp(0), or exp(z_h) with a
//                  learned number z_h per query head (`sink_logit`; it is not scaled, capped or biased),
// and after the softmax an output gate: out *= sigmoid(gate).  Values may also be the first dv elements of
// wider rows (`v_row` elements from one value to the next; the attention over compressed vectors that serve
// as keys and, in part, as values passes the key plane twice).  Every constant is an argument; a
// zero (or a null pointer) switches its step off, and with all of them off this is plain causal
// attention.
//
// Four kernels.  `qkv_unit_store`: per-head RMS norm of queries and keys (with or without gains)
// and the write of keys and values into their pages.  `attention_biased_general`: one block per
// (token, query head), any widths up to 512, float32 or bfloat16; the float32 path and the fallback.
// `attention_biased_prefill`: bfloat16 prompt portions on mma.sync tiles, 64 query rows of one head
// per block, widths up to 128 (padded with zeros to 64 or 128 in shared memory).
// `attention_biased_decode`: one-token rows on the same tiles, one block per (row, key/value head, run of
// keys): the query heads of the group are the rows of the tile, so keys and values are read once for all.
//
// Scores, the cap, the bias, the softmax and the gate are float32 in both storage types.  The order of
// the additions for a (request, position, head) depends on the position and the constants only.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace tllm {

struct ScoreMod {
    float scale, softcap;
    int chunk, window, sink;
    const float* dist_bias;      // [query heads][dist_len] float32 added to the score by distance, or null
    int dist_len;                // distances from dist_len - 1 on share the last entry
    int gate_per_head;           // the output gate holds one number per query head instead of one per element
};

// Place of the gate of element e of a head within the token's gate row.
__device__ __forceinline__ size_t gate_at(int per_head, int head, int dv, int e) {
    return per_head ? (size_t)head : (size_t)head * dv + e;
}

// The learned bias of a head for a key `dist` tokens back (0 without a table).
__device__ __forceinline__ float dist_bias_of(const ScoreMod& m, int head, int dist) {
    if (m.dist_bias == nullptr) return 0.0f;
    return m.dist_bias[(size_t)head * m.dist_len + min(max(dist, 0), m.dist_len - 1)];
}

static inline int page_shift_of(int page_size) {
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    return (1 << shift) == page_size ? shift : -1;
}

__device__ __forceinline__ int first_key(int pos, const ScoreMod& m) {
    int lo = 0;
    if (m.chunk > 0) lo = (pos / m.chunk) * m.chunk;
    if (m.window > 0 && pos - m.window + 1 > lo) lo = pos - m.window + 1;
    return lo;
}

__device__ __forceinline__ float mod_score(float dot, float slope, int dist, const ScoreMod& m) {
    float s = dot * m.scale;
    if (m.softcap > 0.0f) s = m.softcap * tanhf(s / m.softcap);
    return s - slope * (float)dist;
}

// ---------------------------------------------------------------- norm of q and k, write of k and v
// proj[t] = q heads | k heads | v heads | (anything else).  One warp per head of a token.
template <typename T>
__global__ void qkv_unit_store_kernel(const T* proj, int row_stride, const T* __restrict__ q_gain,
                                      const T* __restrict__ k_gain, float eps, int do_norm,
                                      const int* __restrict__ positions, const int* __restrict__ token_slot,
                                      const int* __restrict__ block_table, int max_pages, int page_size,
                                      T* k_plane, T* v_plane, long long page_stride, T* q_out,
                                      int q_heads, int kv_heads, int dk, int dv, int store,
                                      const float* __restrict__ inv_freq, int rot_dims, float temp_coef,
                                      int temp_every, int v_from_k, const float* __restrict__ bias) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int pos = positions[t];
    const T* row = proj + (size_t)t * row_stride;
    // element c of the row as the kernel sees it: the projection plus its bias, if it has one, in float32
    auto at = [&](size_t c) -> float { return to_f32<T>(row[c]) + (bias != nullptr ? bias[c] : 0.0f); };
    long long page_base = -1;
    int in_page = 0;
    if (store) {
        const int page = block_table[(size_t)slot * max_pages + pos / page_size];
        page_base = (long long)page * page_stride;
        in_page = pos % page_size;
        if (page < 0) store = 0;          // no page held: nothing to write (the host reserves before a step)
    }
    const int total = q_heads + 2 * kv_heads;
    for (int head = warp; head < total; head += warps) {
        if (head < q_heads + kv_heads) {
            const bool is_q = head < q_heads;
            const size_t src = (size_t)head * dk;
            const T* gain = is_q ? q_gain : k_gain;
            float sum = 0.0f;
            for (int e = lane; e < dk; e += 32) {
                const float x = at(src + e);
                sum += x * x;
            }
            sum = warp_sum(sum);
            const float sc = do_norm ? 1.0f / sqrtf(sum / (float)dk + eps) : 1.0f;
            T* dst;
            if (is_q) dst = q_out + ((size_t)t * q_heads + head) * dk;
            else if (store) dst = k_plane + page_base + ((size_t)(head - q_heads) * page_size + in_page) * dk;
            else continue;
            // a query's temperature grows with the logarithm of its position counted in runs of temp_every
            const float temp = (is_q && temp_every > 0) ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f) : 1.0f;
            const int half = rot_dims >> 1;
            for (int e = lane; e < dk; e += 32) {
                float x = at(src + e) * sc;
                if (gain != nullptr && do_norm) x *= to_f32<T>(gain[e]);
                if (e < rot_dims) {               // element e turns with its partner half a rotated width away
                    const int partner = e < half ? e + half : e - half;
                    float y = at(src + partner) * sc;
                    if (gain != nullptr && do_norm) y *= to_f32<T>(gain[partner]);
                    const float ang = (float)pos * inv_freq[e < half ? e : e - half];
                    const float c = cosf(ang), sn = sinf(ang);
                    x = e < half ? x * c - y * sn : x * c + y * sn;
                }
                dst[e] = from_f32<T>(x * temp);
            }
        } else if (store) {
            const int g = head - q_heads - kv_heads;
            // values of their own, or the keys as they were projected (before their norm)
            const size_t src = v_from_k ? (size_t)(q_heads + g) * dk
                                        : (size_t)(q_heads + kv_heads) * dk + (size_t)g * dv;
            T* dst = v_plane + page_base + ((size_t)g * page_size + in_page) * dv;
            if (bias != nullptr) for (int e = lane; e < dv; e += 32) dst[e] = from_f32<T>(at(src + e));
            else for (int e = lane; e < dv; e += 32) dst[e] = row[src + e];
        }
    }
}

// The same for bfloat16 rows whose widths are multiples of eight: a group of GS lanes (a power of two; dk / 8 of
// them at work) holds a head, eight elements to a lane, so a warp takes 32 / GS heads at once with 16-byte
// loads and stores.  The token's cosines and sines are made once, in shared memory, for all its heads; the
// partner of a rotated element sits half / 8 lanes away (half a multiple of eight).  The arithmetic per
// element is that of the kernel above.
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}

template <int GS>
__global__ void __launch_bounds__(256)
qkv_unit_store_vec_kernel(const bf16* proj, int row_stride, const bf16* __restrict__ q_gain,
                          const bf16* __restrict__ k_gain, float eps, int do_norm,
                          const int* __restrict__ positions, const int* __restrict__ token_slot,
                          const int* __restrict__ block_table, int max_pages, int page_size, bf16* k_plane,
                          bf16* v_plane, long long page_stride, bf16* q_out, int q_heads, int kv_heads, int dk,
                          int dv, int store, const float* __restrict__ inv_freq, int rot_dims, float temp_coef,
                          int temp_every, int v_from_k, const float* __restrict__ bias) {
    extern __shared__ float cos_sin[];                      // cos of the token's `half` angles, then their sines
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) return;                                    // the whole block
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int pos = positions[t];
    const int half = rot_dims >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float ang = (float)pos * inv_freq[i];
        cos_sin[i] = cosf(ang);
        cos_sin[half + i] = sinf(ang);
    }
    if (half > 0) __syncthreads();
    const bf16* row = proj + (size_t)t * row_stride;
    long long page_base = -1;
    int in_page = 0;
    if (store) {
        const int page = block_table[(size_t)slot * max_pages + pos / page_size];
        page_base = (long long)page * page_stride;
        in_page = pos % page_size;
        if (page < 0) store = 0;
    }
    constexpr int kPerWarp = 32 / GS;
    const int grp = lane / GS, gl = lane % GS, e0 = gl * 8;
    const int normed = q_heads + kv_heads;
    const float q_temp = temp_every > 0 ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f) : 1.0f;
    for (int base = warp * kPerWarp; base < normed; base += warps * kPerWarp) {
        const int head = base + grp;
        const bool is_q = head < q_heads;
        const bool active = head < normed && e0 < dk;
        float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        if (active) {
            load8(row + (size_t)head * dk + e0, v);
            if (bias != nullptr) {                           // the projection's bias, added in float32
                const float4 b0 = *reinterpret_cast<const float4*>(bias + (size_t)head * dk + e0);
                const float4 b1 = *reinterpret_cast<const float4*>(bias + (size_t)head * dk + e0 + 4);
                v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
            }
        }
        float sum = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) sum += v[e] * v[e];
#pragma unroll
        for (int o = GS / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float sc = do_norm ? 1.0f / sqrtf(sum / (float)dk + eps) : 1.0f;
        const bf16* gain = is_q ? q_gain : k_gain;
        if (active && gain != nullptr && do_norm) {
            float gn[8];
            load8(gain + e0, gn);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = v[e] * sc * gn[e];
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] *= sc;
        }
        if (half > 0) {                                      // every lane takes part in the exchange
            const bool turns = e0 < rot_dims, low = e0 < half;
            const int from = turns ? (low ? lane + half / 8 : lane - half / 8) : lane;
            const int i0 = low ? e0 : e0 - half;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float y = __shfl_sync(0xffffffffu, v[e], from);
                if (turns) {
                    const float c = cos_sin[i0 + e], sn = cos_sin[half + i0 + e];
                    v[e] = low ? v[e] * c - y * sn : v[e] * c + y * sn;
                }
            }
        }
        if (!active) continue;
        bf16* dst;
        if (is_q) dst = q_out + ((size_t)t * q_heads + head) * dk;
        else if (store) dst = k_plane + page_base + ((size_t)(head - q_heads) * page_size + in_page) * dk;
        else continue;
        const float temp = is_q ? q_temp : 1.0f;
        uint4 raw;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(v[2 * e] * temp, v[2 * e + 1] * temp);
        *reinterpret_cast<uint4*>(dst + e0) = raw;
    }
    if (store) {
        // values of their own, or the keys as they were projected (before their norm): 16 bytes a thread
        const int per_head = dv / 8;
        const bf16* src0 = v_from_k ? row + (size_t)q_heads * dk : row + (size_t)normed * dk;
        for (int c = threadIdx.x; c < kv_heads * per_head; c += blockDim.x) {
            const int g = c / per_head, j = c - g * per_head;
            bf16* dst = v_plane + page_base + ((size_t)g * page_size + in_page) * dv + j * 8;
            if (bias == nullptr) {
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src0 + (size_t)g * dv + j * 8);
                continue;
            }
            float v[8];
            load8(src0 + (size_t)g * dv + j * 8, v);
            const float* b = bias + (src0 - row) + (size_t)g * dv + j * 8;
            uint4 raw;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(v[2 * e] + b[2 * e], v[2 * e + 1] + b[2 * e + 1]);
            *reinterpret_cast<uint4*>(dst) = raw;
        }
    }
}

// ---------------------------------------------------------------- general kernel
constexpr int kGenWarps = 4;

template <typename T, int CK, int CV>
__global__ void attention_biased_general_kernel(
    const T* q, const T* k_plane, const T* v_plane, long long page_stride,
    const int* __restrict__ positions, const int* __restrict__ token_slot,
    const int* __restrict__ block_table, int max_pages, int page_size, int q_heads, int kv_heads,
    int dk, int dv, ScoreMod mod, const float* __restrict__ slopes, const float* __restrict__ sink_logit, int v_row,
    const T* gate, int gate_stride, T* __restrict__ out) {
    extern __shared__ float smem[];
    TLLM_PDL_ENTER();
    float* qs = smem;                             // [dk]
    float* acc_s = smem + dk;                     // [warps][dv]
    float* m_s = acc_s + kGenWarps * dv;          // [warps]
    float* l_s = m_s + kGenWarps;                 // [warps]

    const int head = blockIdx.x, t = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    T* dst = out + ((size_t)t * q_heads + head) * dv;
    const int slot = token_slot[t];
    if (slot < 0) {
        for (int e = threadIdx.x; e < dv; e += blockDim.x) dst[e] = from_f32<T>(0.0f);
        return;
    }
    const int pos = positions[t];
    const int lo = first_key(pos, mod);
    const int g = head / (q_heads / kv_heads);
    const float slope = slopes != nullptr ? slopes[head] : 0.0f;
    const T* qsrc = q + ((size_t)t * q_heads + head) * dk;
    for (int e = threadIdx.x; e < dk; e += blockDim.x) qs[e] = to_f32<T>(qsrc[e]);
    __syncthreads();

    const int* table = block_table + (size_t)slot * max_pages;
    // the sink is a key of score 0 (or of the head's learned score) without a value; warp 0 starts from it
    float m = (mod.sink && warp == 0) ? (sink_logit != nullptr ? sink_logit[head] : 0.0f) : -INFINITY;
    float l = (mod.sink && warp == 0) ? 1.0f : 0.0f;
    float acc[CV];
#pragma unroll
    for (int c = 0; c < CV; ++c) acc[c] = 0.0f;

    for (int j = lo + warp; j <= pos; j += kGenWarps) {
        const int page = table[j / page_size];
        if (page < 0) continue;
        const size_t in_page = (size_t)g * page_size + (j % page_size);
        const T* kp = k_plane + (long long)page * page_stride + in_page * dk;
        const T* vp = v_plane + (long long)page * page_stride + in_page * v_row;
        float dot = 0.0f;
#pragma unroll
        for (int c = 0; c < CK; ++c) {
            const int e = lane + 32 * c;
            if (e < dk) dot += qs[e] * to_f32<T>(kp[e]);
        }
        dot = warp_sum(dot);
        const float s = mod_score(dot, slope, pos - j, mod) + dist_bias_of(mod, head, pos - j);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int c = 0; c < CV; ++c) {
            const int e = lane + 32 * c;
            if (e < dv) acc[c] = acc[c] * corr + p * to_f32<T>(vp[e]);
        }
        m = m_new;
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int c = 0; c < CV; ++c) {
        const int e = lane + 32 * c;
        if (e < dv) acc_s[warp * dv + e] = acc[c];
    }
    __syncthreads();
    float mm = m_s[0];
#pragma unroll
    for (int w = 1; w < kGenWarps; ++w) mm = fmaxf(mm, m_s[w]);
    float w_scale[kGenWarps], total = 0.0f;
#pragma unroll
    for (int w = 0; w < kGenWarps; ++w) {
        w_scale[w] = (m_s[w] == -INFINITY) ? 0.0f : expf(m_s[w] - mm);
        total += l_s[w] * w_scale[w];
    }
    const float inv = total > 0.0f ? 1.0f / total : 0.0f;
    const T* grow = gate != nullptr ? gate + (size_t)t * gate_stride + gate_at(mod.gate_per_head, head, dv, 0) : nullptr;
    for (int e = threadIdx.x; e < dv; e += blockDim.x) {
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < kGenWarps; ++w) v += acc_s[w * dv + e] * w_scale[w];
        v *= inv;
        if (grow != nullptr) v *= 1.0f / (1.0f + expf(-to_f32<T>(grow[mod.gate_per_head ? 0 : e])));
        dst[e] = from_f32<T>(v);
    }
}

template <typename T>
static int launch_general(const void* q, const void* kp, const void* vp, long long page_stride,
                          const int* positions, const int* token_slot, const int* block_table,
                          int max_pages, int page_size, int tokens, int q_heads, int kv_heads, int dk,
                          int dv, ScoreMod mod, const float* slopes, const float* sink_logit, int v_row,
                          const void* gate, int gate_stride, void* out, cudaStream_t stream) {
    const dim3 grid(q_heads, tokens), block(kGenWarps * 32);
    const size_t smem = ((size_t)dk + (size_t)kGenWarps * dv + 2 * kGenWarps) * sizeof(float);
    const int ck = (dk + 31) / 32, cv = (dv + 31) / 32;
    const int c = ck > cv ? ck : cv;
#define LAUNCH(C)                                                                                           \
    launch_pdl(kPdlAttention, attention_biased_general_kernel<T, C, C>, grid, block, smem, stream,          \
               (const T*)q, (const T*)kp, (const T*)vp, page_stride, positions, token_slot, block_table,    \
               max_pages, page_size, q_heads, kv_heads, dk, dv, mod, slopes, sink_logit, v_row, (const T*)gate, gate_stride, (T*)out)
    if (c <= 1) LAUNCH(1);
    else if (c <= 2) LAUNCH(2);
    else if (c <= 4) LAUNCH(4);
    else if (c <= 8) LAUNCH(8);
    else LAUNCH(16);
#undef LAUNCH
    return finish_launch("attention_biased_general");
}

constexpr float kLog2e = 1.4426950408889634f;

// tanh(x) = 1 - 2 / (e^2x + 1): absolute error of a few 1e-7 with the fast exponential and division,
// which the cap multiplies; |x| is clamped where tanh is 1 to the last bit anyway.
__device__ __forceinline__ float fast_tanh(float x) {
    x = fminf(fmaxf(x, -15.0f), 15.0f);
    return 1.0f - __fdividef(2.0f, __expf(2.0f * x) + 1.0f);
}

// 2^x by the hardware approximation alone (exp2f adds a range reduction for denormal results; here a
// weight that small is zero anyway).  2^-inf = 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Page and place in the page of a key: a shift and a mask where the page size is a power of two
// (`shift` >= 0), else a division.
__device__ __forceinline__ void page_of(int key, int page_size, int shift, int& page_index, int& in_page) {
    if (shift >= 0) { page_index = key >> shift; in_page = key & (page_size - 1); }
    else { page_index = key / page_size; in_page = key - page_index * page_size; }
}

// The modified score times log2(e), for exp2f.  `dist` comes as a float and 1 / cap as a factor: a
// conversion or a division per score would go through the same slow unit as the exponentials.  No
// branch: the capped and the plain score are both made and one is kept, so that the scores of a tile
// are independent chains the scheduler can interleave (with the mask as a condition around the
// arithmetic every score was a branch of its own, and the chains ran one after the other).
__device__ __forceinline__ float mod_score_fast(float dot, float slope_log2e, float dist, const ScoreMod& m, float inv_cap) {
    const float plain = dot * m.scale;
    const float capped = m.softcap * fast_tanh(plain * inv_cap);
    const float s = m.softcap > 0.0f ? capped : plain;
    return s * kLog2e - slope_log2e * dist;
}

// ---------------------------------------------------------------- prompt portions, bfloat16, mma.sync
// A block owns 64 consecutive query rows of one portion and one query head and walks the keys its rows
// can see in tiles of 64 (flash-attention style: S and the softmax in float32 registers, P V accumulated
// in float32).  Keys and values are staged by cp.async in two buffers; a row of a tile is padded by 16
// bytes so that ldmatrix meets no bank conflict, and widths below DKP / DVP are filled with zeros.
constexpr int kPfWarps = 4, kPfM = 64, kPfN = 64, kPfPad = 8;

template <int DKP, int DVP>
__global__ void __launch_bounds__(kPfWarps * 32, 3)
attention_biased_prefill_kernel(const bf16* q, const bf16* k_plane, const bf16* v_plane, long long page_stride,
                                const int* __restrict__ seg_info, const int* __restrict__ tiles,
                                const int* __restrict__ block_table, int max_pages, int page_size,
                                int page_shift, int q_heads, int kv_heads, int dk, int dv, ScoreMod mod,
                                const float* __restrict__ slopes, const float* __restrict__ sink_logit, int v_row,
                                const bf16* gate, int gate_stride, bf16* __restrict__ out) {
    extern __shared__ __align__(128) unsigned char pf_smem[];
    TLLM_PDL_ENTER();
    constexpr int kKRow = DKP + kPfPad, kVRow = DVP + kPfPad;           // elements per padded row
    constexpr int kKBytes = kPfN * kKRow * 2, kVBytes = kPfN * kVRow * 2;
    const int seg = tiles[2 * blockIdx.x], q_off = tiles[2 * blockIdx.x + 1];
    const int head = blockIdx.y;
    const int slot = seg_info[4 * seg], start = seg_info[4 * seg + 1];
    const int len = seg_info[4 * seg + 2], pos0 = seg_info[4 * seg + 3];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = head / (q_heads / kv_heads);
    const int* table = block_table + (size_t)slot * max_pages;
    const float slope2 = (slopes != nullptr ? slopes[head] : 0.0f) * kLog2e;
    const float inv_cap = mod.softcap > 0.0f ? 1.0f / mod.softcap : 0.0f;

    const int rows_here = min(kPfM, len - q_off);
    const int first_pos = pos0 + q_off, last_pos = first_pos + rows_here - 1;
    const int lo_all = first_key(first_pos, mod);
    const int kt_first = lo_all / kPfN, kt_last = last_pos / kPfN;

    const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
    const bool v_lo = r_lo < rows_here, v_hi = r_hi < rows_here;
    const int p_lo = first_pos + r_lo, p_hi = first_pos + r_hi;
    const int f_lo = first_key(p_lo, mod), f_hi = first_key(p_hi, mod);
    const bf16* q_lo = q + ((size_t)(start + q_off + r_lo) * q_heads + head) * dk;
    const bf16* q_hi = q + ((size_t)(start + q_off + r_hi) * q_heads + head) * dk;
    uint32_t qa[DKP / 16][4];
#pragma unroll
    for (int ks = 0; ks < DKP / 16; ++ks) {
        const int c0 = ks * 16 + (lane & 3) * 2;
        qa[ks][0] = (v_lo && c0 < dk) ? *reinterpret_cast<const uint32_t*>(q_lo + c0) : 0u;
        qa[ks][1] = (v_hi && c0 < dk) ? *reinterpret_cast<const uint32_t*>(q_hi + c0) : 0u;
        qa[ks][2] = (v_lo && c0 + 8 < dk) ? *reinterpret_cast<const uint32_t*>(q_lo + c0 + 8) : 0u;
        qa[ks][3] = (v_hi && c0 + 8 < dk) ? *reinterpret_cast<const uint32_t*>(q_hi + c0 + 8) : 0u;
    }
    const int w_first = first_pos + warp * 16;
    const int w_last = min(w_first + 15, last_pos);
    const int w_lo = first_key(w_first, mod);
    const int w_hi_lo = first_key(w_first + 15, mod);                  // the latest first key among the warp's rows

    float o[DVP / 8][4];
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    // the sink: a key of score 0 (or the head's learned score) without a value, counted once per row (by the
    // first lane of its four)
    float m_lo = mod.sink ? (sink_logit != nullptr ? sink_logit[head] * kLog2e : 0.0f) : -INFINITY, m_hi = m_lo;
    float l_lo = (mod.sink && (lane & 3) == 0) ? 1.0f : 0.0f, l_hi = l_lo;

    auto issue = [&](int kt, int stage) {
        const uint32_t ks = smem_u32(pf_smem + (size_t)stage * (kKBytes + kVBytes));
        const uint32_t vs = ks + kKBytes;
        constexpr int kKC = DKP / 8, kVC = DVP / 8;
        // a thread keeps its 16-byte column and walks the rows: one look-up of the page per row
        for (int row = threadIdx.x / kKC, chunk = threadIdx.x % kKC; row < kPfN; row += kPfWarps * 32 / kKC) {
            const int key = kt * kPfN + row;
            int page_index, place;
            page_of(key, page_size, page_shift, page_index, place);
            const int page = (key <= last_pos && key >= lo_all) ? table[page_index] : -1;
            const bool ok = page >= 0;
            const long long page_at = ok ? (long long)page * page_stride : 0;
            const long long in_page = (long long)g * page_size + place;
            const bool k_ok = ok && chunk * 8 < dk;
            cp_async_16(ks + (row * kKRow + chunk * 8) * 2, k_plane + (k_ok ? page_at + in_page * dk + chunk * 8 : 0), k_ok);
            if (kKC == kVC) {
                const bool v_ok = ok && chunk * 8 < dv;
                cp_async_16(vs + (row * kVRow + chunk * 8) * 2, v_plane + (v_ok ? page_at + in_page * v_row + chunk * 8 : 0), v_ok);
            }
        }
        if (kKC != kVC) {
            for (int row = threadIdx.x / kVC, chunk = threadIdx.x % kVC; row < kPfN; row += kPfWarps * 32 / kVC) {
                const int key = kt * kPfN + row;
                int page_index, place;
                page_of(key, page_size, page_shift, page_index, place);
                const int page = (key <= last_pos && key >= lo_all) ? table[page_index] : -1;
                const bool v_ok = page >= 0 && chunk * 8 < dv;
                cp_async_16(vs + (row * kVRow + chunk * 8) * 2, v_plane + (v_ok ? (long long)page * page_stride + ((long long)g * page_size + place) * v_row + chunk * 8 : 0), v_ok);
            }
        }
        cp_async_commit();
    };

    issue(kt_first, 0);
    for (int kt = kt_first; kt <= kt_last; ++kt) {
        const int stage = (kt - kt_first) & 1;
        if (kt + 1 <= kt_last) {
            issue(kt + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int key0 = kt * kPfN;
        const bool active = warp * 16 < rows_here && key0 <= w_last && key0 + kPfN - 1 >= w_lo;
        if (active) {
            const uint32_t ks_base = smem_u32(pf_smem + (size_t)stage * (kKBytes + kVBytes));
            const uint32_t vs_base = ks_base + kKBytes;
            const int mid = lane >> 3, mrow = lane & 7;
            float s[kPfN / 8][4];
#pragma unroll
            for (int i = 0; i < kPfN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < DKP / 16; ++ks) {               // columns past dk are zeros on both sides
#pragma unroll
                for (int nt2 = 0; nt2 < kPfN / 16; ++nt2) {
                    uint32_t kb[4];
                    ldmatrix_x4(kb, ks_base + ((nt2 * 16 + (mid >> 1) * 8 + mrow) * kKRow + ks * 16 + (mid & 1) * 8) * 2);
                    const uint32_t b0[2] = {kb[0], kb[1]}, b1[2] = {kb[2], kb[3]};
                    mma_bf16_16816(s[2 * nt2], qa[ks], b0);
                    mma_bf16_16816(s[2 * nt2 + 1], qa[ks], b1);
                }
            }
            const int key_base = key0 + (lane & 3) * 2;
            const float d_lo = (float)(p_lo - key_base), d_hi = (float)(p_hi - key_base);
            // a tile that every row of the warp sees whole needs no masks (most tiles of a long prompt)
            const bool inner = key0 + kPfN - 1 <= w_first && key0 >= w_hi_lo;
            float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < kPfN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float back = (float)(nt * 8 + e);          // a constant once the loops are unrolled
                    s[nt][e] = mod_score_fast(s[nt][e], slope2, d_lo - back, mod, inv_cap);
                    s[nt][2 + e] = mod_score_fast(s[nt][2 + e], slope2, d_hi - back, mod, inv_cap);
                }
            if (mod.dist_bias != nullptr) {
                // a tile that lies beyond the table for every row of the warp gets the table's last entry;
                // only the few tiles near the diagonal look distances up one by one
                const float* tb = mod.dist_bias + (size_t)head * mod.dist_len;
                const int lastd = mod.dist_len - 1;
                if (first_pos + warp * 16 - (key0 + kPfN - 1) >= lastd) {
                    const float far = tb[lastd] * kLog2e;
#pragma unroll
                    for (int nt = 0; nt < kPfN / 8; ++nt) { s[nt][0] += far; s[nt][1] += far; s[nt][2] += far; s[nt][3] += far; }
                } else {
                    const int n_lo = p_lo - key_base, n_hi = p_hi - key_base;
#pragma unroll
                    for (int nt = 0; nt < kPfN / 8; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            s[nt][e] += tb[min(max(n_lo - (nt * 8 + e), 0), lastd)] * kLog2e;
                            s[nt][2 + e] += tb[min(max(n_hi - (nt * 8 + e), 0), lastd)] * kLog2e;
                        }
                }
            }
            if (!inner) {
#pragma unroll
                for (int nt = 0; nt < kPfN / 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int j = key_base + nt * 8 + e;
                        s[nt][e] = (j <= p_lo && j >= f_lo) ? s[nt][e] : -INFINITY;
                        s[nt][2 + e] = (j <= p_hi && j >= f_hi) ? s[nt][2 + e] : -INFINITY;
                    }
            }
#pragma unroll
            for (int nt = 0; nt < kPfN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    tmax_lo = fmaxf(tmax_lo, s[nt][e]);
                    tmax_hi = fmaxf(tmax_hi, s[nt][2 + e]);
                }
            tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
            tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
            tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
            tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
            const float mn_lo = fmaxf(m_lo, tmax_lo), mn_hi = fmaxf(m_hi, tmax_hi);
            const float ms_lo = mn_lo == -INFINITY ? 0.0f : mn_lo, ms_hi = mn_hi == -INFINITY ? 0.0f : mn_hi;
            const float c_lo = fast_exp2(m_lo - ms_lo), c_hi = fast_exp2(m_hi - ms_hi);
            m_lo = mn_lo;
            m_hi = mn_hi;
            float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
            for (int nt = 0; nt < kPfN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    s[nt][e] = fast_exp2(s[nt][e] - ms_lo);
                    s[nt][2 + e] = fast_exp2(s[nt][2 + e] - ms_hi);
                    sum_lo += s[nt][e];
                    sum_hi += s[nt][2 + e];
                }
            l_lo = l_lo * c_lo + sum_lo;
            l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i) {
                o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi;
            }
#pragma unroll
            for (int kk = 0; kk < kPfN / 16; ++kk) {
                const uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                                        pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                                        pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
                for (int c = 0; c < DVP / 8; c += 2) {             // value columns past dv are zeros
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, vs_base + ((kk * 16 + (mid & 1) * 8 + mrow) * kVRow + (c + (mid >> 1)) * 8) * 2);
                    const uint32_t b0[2] = {vb[0], vb[1]}, b1[2] = {vb[2], vb[3]};
                    mma_bf16_16816(o[c], pa, b0);
                    mma_bf16_16816(o[c + 1], pa, b1);
                }
            }
        }
        __syncthreads();
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = l_lo > 0.0f ? 1.0f / l_lo : 0.0f, inv_hi = l_hi > 0.0f ? 1.0f / l_hi : 0.0f;
    const size_t row_lo = start + q_off + r_lo, row_hi = start + q_off + r_hi;
    bf16* o_lo = out + (row_lo * q_heads + head) * dv;
    bf16* o_hi = out + (row_hi * q_heads + head) * dv;
    const bf16* g_lo = gate != nullptr ? gate + row_lo * gate_stride + gate_at(mod.gate_per_head, head, dv, 0) : nullptr;
    const bf16* g_hi = gate != nullptr ? gate + row_hi * gate_stride + gate_at(mod.gate_per_head, head, dv, 0) : nullptr;
    const int g_step = mod.gate_per_head ? 0 : 1;
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i) {
        const int col = i * 8 + (lane & 3) * 2;
        if (col >= dv) continue;
        if (v_lo) {
            float a = o[i][0] * inv_lo, b = o[i][1] * inv_lo;
            if (g_lo != nullptr) {
                a *= 1.0f / (1.0f + expf(-__bfloat162float(g_lo[col * g_step])));
                b *= 1.0f / (1.0f + expf(-__bfloat162float(g_lo[(col + 1) * g_step])));
            }
            *reinterpret_cast<uint32_t*>(o_lo + col) = pack_bf16(a, b);
        }
        if (v_hi) {
            float a = o[i][2] * inv_hi, b = o[i][3] * inv_hi;
            if (g_hi != nullptr) {
                a *= 1.0f / (1.0f + expf(-__bfloat162float(g_hi[col * g_step])));
                b *= 1.0f / (1.0f + expf(-__bfloat162float(g_hi[(col + 1) * g_step])));
            }
            *reinterpret_cast<uint32_t*>(o_hi + col) = pack_bf16(a, b);
        }
    }
}

template <int DKP, int DVP>
static int launch_biased_prefill(const void* q, const void* kp, const void* vp, long long page_stride,
                                 const int* seg_info, const int* tiles, int n_tiles, const int* block_table,
                                 int max_pages, int page_size, int q_heads, int kv_heads, int dk, int dv,
                                 ScoreMod mod, const float* slopes, const float* sink_logit, int v_row, const void* gate,
                                 int gate_stride, void* out, cudaStream_t stream) {
    const size_t smem = (size_t)2 * kPfN * ((DKP + kPfPad) + (DVP + kPfPad)) * 2;
    static OncePerDevice configured;
    if (configured.first()) {
        cudaError_t e = cudaFuncSetAttribute(attention_biased_prefill_kernel<DKP, DVP>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { set_error("attention_biased_prefill: %s", cudaGetErrorString(e)); return (int)e; }
        configured.done();
    }
    launch_pdl(kPdlAttention, attention_biased_prefill_kernel<DKP, DVP>, dim3(n_tiles, q_heads), dim3(kPfWarps * 32),
               smem, stream, (const bf16*)q, (const bf16*)kp, (const bf16*)vp, page_stride, seg_info, tiles,
               block_table, max_pages, page_size, page_shift_of(page_size), q_heads, kv_heads, dk, dv, mod, slopes, sink_logit, v_row,
               (const bf16*)gate, gate_stride, (bf16*)out);
    return finish_launch("attention_biased_prefill");
}

// ---------------------------------------------------------------- one-token rows, bfloat16, mma.sync
// One block per (row, key/value head, run of keys) (per sixteen query heads of it, if it serves more).  The query heads of the group are the 16 rows of the
// tensor-core tile (the first `group` of them real), so keys and values are read once for all of them.
// The block stages tiles of 64 keys like the prompt kernel; each of its four warps takes 16 keys of a
// tile and keeps its own running maximum, sum and value sums (base 2), which meet in shared memory in
// the order of the warps.  With one run per row the block writes the result; with more (a grid that
// would not fill the GPU, long reaches) it leaves unnormalised sums, maximum and weight per run, and a
// second kernel adds the runs in their order.  The sink belongs to the first warp of the first run.
template <int DKP, int DVP>
__global__ void __launch_bounds__(kPfWarps * 32, 2)
attention_biased_decode_kernel(const bf16* q, const bf16* k_plane, const bf16* v_plane, long long page_stride,
                               const int* __restrict__ positions, const int* __restrict__ token_slot,
                               const int* __restrict__ rows, const int* __restrict__ block_table, int max_pages,
                               int page_size, int page_shift, int q_heads, int kv_heads, int dk, int dv, ScoreMod mod,
                               const float* __restrict__ slopes, const float* __restrict__ sink_logit, int v_row,
                               const bf16* gate, int gate_stride, int splits, int sub_groups, float* part,
                               bf16* __restrict__ out) {
    extern __shared__ __align__(128) unsigned char pf_smem[];
    TLLM_PDL_ENTER();
    constexpr int kKRow = DKP + kPfPad, kVRow = DVP + kPfPad;
    constexpr int kKBytes = kPfN * kKRow * 2, kVBytes = kPfN * kVRow * 2;
    const int t = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
    // a key/value head's query heads fill the tile's 16 rows; more of them (multi-query attention over many
    // heads) are dealt to `sub_groups` blocks that read the same keys
    const int g = blockIdx.y / sub_groups, split = blockIdx.z;
    const int group = q_heads / kv_heads / sub_groups;
    const int head0 = g * (q_heads / kv_heads) + (blockIdx.y % sub_groups) * group;
    const int slot = token_slot[t];
    const int rec = dv + 2;
    if (slot < 0) {
        if (splits == 1)
            for (int i = threadIdx.x; i < group * dv; i += blockDim.x)
                out[((size_t)t * q_heads + head0) * dv + i] = __float2bfloat16_rn(0.0f);
        return;                       // the combining kernel writes the zeros of a row without a request
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int lo = first_key(pos, mod);
    const int* table = block_table + (size_t)slot * max_pages;
    int kt_first = lo / kPfN, kt_last = pos / kPfN;
    if (splits > 1) {
        const int per = (kt_last - kt_first + splits) / splits;
        kt_first += split * per;
        kt_last = min(kt_last, kt_first + per - 1);
    }

    const int r_lo = lane >> 2, r_hi = r_lo + 8;                       // rows of the tile: heads of the group
    const bool v_lo = r_lo < group, v_hi = r_hi < group;
    const float slope_lo = (slopes != nullptr && v_lo) ? slopes[head0 + r_lo] * kLog2e : 0.0f;
    const float slope_hi = (slopes != nullptr && v_hi) ? slopes[head0 + r_hi] * kLog2e : 0.0f;
    const float inv_cap = mod.softcap > 0.0f ? 1.0f / mod.softcap : 0.0f;
    const bf16* q_lo = q + ((size_t)t * q_heads + head0 + r_lo) * dk;
    const bf16* q_hi = q + ((size_t)t * q_heads + head0 + r_hi) * dk;
    uint32_t qa[DKP / 16][4];
#pragma unroll
    for (int ks = 0; ks < DKP / 16; ++ks) {
        const int c0 = ks * 16 + (lane & 3) * 2;
        qa[ks][0] = (v_lo && c0 < dk) ? *reinterpret_cast<const uint32_t*>(q_lo + c0) : 0u;
        qa[ks][1] = (v_hi && c0 < dk) ? *reinterpret_cast<const uint32_t*>(q_hi + c0) : 0u;
        qa[ks][2] = (v_lo && c0 + 8 < dk) ? *reinterpret_cast<const uint32_t*>(q_lo + c0 + 8) : 0u;
        qa[ks][3] = (v_hi && c0 + 8 < dk) ? *reinterpret_cast<const uint32_t*>(q_hi + c0 + 8) : 0u;
    }
    float o[DVP / 8][4];
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    const bool first = mod.sink && warp == 0 && split == 0;
    float m_lo = first ? 0.0f : -INFINITY, m_hi = m_lo;
    if (first && sink_logit != nullptr) {            // the heads' learned sink scores, in base 2 like the scores
        m_lo = v_lo ? sink_logit[head0 + r_lo] * kLog2e : 0.0f;
        m_hi = v_hi ? sink_logit[head0 + r_hi] * kLog2e : 0.0f;
    }
    float l_lo = (first && (lane & 3) == 0) ? 1.0f : 0.0f, l_hi = l_lo;

    auto issue = [&](int kt, int stage) {
        const uint32_t ks = smem_u32(pf_smem + (size_t)stage * (kKBytes + kVBytes));
        const uint32_t vs = ks + kKBytes;
        constexpr int kKC = DKP / 8, kVC = DVP / 8;
        for (int row = threadIdx.x / kKC, chunk = threadIdx.x % kKC; row < kPfN; row += kPfWarps * 32 / kKC) {
            const int key = kt * kPfN + row;
            int page_index, place;
            page_of(key, page_size, page_shift, page_index, place);
            const int page = (key <= pos && key >= lo) ? table[page_index] : -1;
            const bool ok = page >= 0;
            const long long page_at = ok ? (long long)page * page_stride : 0;
            const long long in_page = (long long)g * page_size + place;
            const bool k_ok = ok && chunk * 8 < dk;
            cp_async_16(ks + (row * kKRow + chunk * 8) * 2, k_plane + (k_ok ? page_at + in_page * dk + chunk * 8 : 0), k_ok);
            if (kKC == kVC) {
                const bool v_ok = ok && chunk * 8 < dv;
                cp_async_16(vs + (row * kVRow + chunk * 8) * 2, v_plane + (v_ok ? page_at + in_page * v_row + chunk * 8 : 0), v_ok);
            }
        }
        if (kKC != kVC) {
            for (int row = threadIdx.x / kVC, chunk = threadIdx.x % kVC; row < kPfN; row += kPfWarps * 32 / kVC) {
                const int key = kt * kPfN + row;
                int page_index, place;
                page_of(key, page_size, page_shift, page_index, place);
                const int page = (key <= pos && key >= lo) ? table[page_index] : -1;
                const bool v_ok = page >= 0 && chunk * 8 < dv;
                cp_async_16(vs + (row * kVRow + chunk * 8) * 2, v_plane + (v_ok ? (long long)page * page_stride + ((long long)g * page_size + place) * v_row + chunk * 8 : 0), v_ok);
            }
        }
        cp_async_commit();
    };

    if (kt_first <= kt_last) issue(kt_first, 0);
    for (int kt = kt_first; kt <= kt_last; ++kt) {
        const int stage = (kt - kt_first) & 1;
        if (kt + 1 <= kt_last) {
            issue(kt + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int key0 = kt * kPfN + warp * 16;                          // this warp's 16 keys of the tile
        if (key0 <= pos && key0 + 15 >= lo) {
            const uint32_t ks_base = smem_u32(pf_smem + (size_t)stage * (kKBytes + kVBytes));
            const uint32_t vs_base = ks_base + kKBytes;
            const int mid = lane >> 3, mrow = lane & 7;
            float s[2][4];
            s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < DKP / 16; ++ks) {
                uint32_t kb[4];
                ldmatrix_x4(kb, ks_base + ((warp * 16 + (mid >> 1) * 8 + mrow) * kKRow + ks * 16 + (mid & 1) * 8) * 2);
                const uint32_t b0[2] = {kb[0], kb[1]}, b1[2] = {kb[2], kb[3]};
                mma_bf16_16816(s[0], qa[ks], b0);
                mma_bf16_16816(s[1], qa[ks], b1);
            }
            const int key_base = key0 + (lane & 3) * 2;
            const float d0 = (float)(pos - key_base);
            float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = key_base + nt * 8 + e;
                    const bool seen = j <= pos && j >= lo;
                    const float dist = d0 - (float)(nt * 8 + e);
                    float a = mod_score_fast(s[nt][e], slope_lo, dist, mod, inv_cap);
                    float b = mod_score_fast(s[nt][2 + e], slope_hi, dist, mod, inv_cap);
                    if (mod.dist_bias != nullptr) {
                        a += dist_bias_of(mod, head0 + (v_lo ? r_lo : 0), pos - j) * kLog2e;
                        b += dist_bias_of(mod, head0 + (v_hi ? r_hi : 0), pos - j) * kLog2e;
                    }
                    s[nt][e] = (seen && v_lo) ? a : -INFINITY;
                    s[nt][2 + e] = (seen && v_hi) ? b : -INFINITY;
                    tmax_lo = fmaxf(tmax_lo, s[nt][e]);
                    tmax_hi = fmaxf(tmax_hi, s[nt][2 + e]);
                }
            tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
            tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
            tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
            tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
            const float mn_lo = fmaxf(m_lo, tmax_lo), mn_hi = fmaxf(m_hi, tmax_hi);
            const float ms_lo = mn_lo == -INFINITY ? 0.0f : mn_lo, ms_hi = mn_hi == -INFINITY ? 0.0f : mn_hi;
            const float c_lo = fast_exp2(m_lo - ms_lo), c_hi = fast_exp2(m_hi - ms_hi);
            m_lo = mn_lo;
            m_hi = mn_hi;
            float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    s[nt][e] = fast_exp2(s[nt][e] - ms_lo);
                    s[nt][2 + e] = fast_exp2(s[nt][2 + e] - ms_hi);
                    sum_lo += s[nt][e];
                    sum_hi += s[nt][2 + e];
                }
            l_lo = l_lo * c_lo + sum_lo;
            l_hi = l_hi * c_hi + sum_hi;
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i) {
                o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi;
            }
            const uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                                    pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
#pragma unroll
            for (int c = 0; c < DVP / 8; c += 2) {
                uint32_t vb[4];
                ldmatrix_x4_trans(vb, vs_base + ((warp * 16 + (mid & 1) * 8 + mrow) * kVRow + (c + (mid >> 1)) * 8) * 2);
                const uint32_t b0[2] = {vb[0], vb[1]}, b1[2] = {vb[2], vb[3]};
                mma_bf16_16816(o[c], pa, b0);
                mma_bf16_16816(o[c + 1], pa, b1);
            }
        }
        __syncthreads();
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    // the warps meet: [warp][head of the group][dv + 2] floats, over the staging buffers (all reads of which are done)
    float* meet = reinterpret_cast<float*>(pf_smem);
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i) {
        const int col = i * 8 + (lane & 3) * 2;
        if (col >= dv) continue;
        if (v_lo) { float* d = meet + ((size_t)warp * group + r_lo) * rec; d[col] = o[i][0]; d[col + 1] = o[i][1]; }
        if (v_hi) { float* d = meet + ((size_t)warp * group + r_hi) * rec; d[col] = o[i][2]; d[col + 1] = o[i][3]; }
    }
    if ((lane & 3) == 0) {
        if (v_lo) { float* d = meet + ((size_t)warp * group + r_lo) * rec; d[dv] = m_lo; d[dv + 1] = l_lo; }
        if (v_hi) { float* d = meet + ((size_t)warp * group + r_hi) * rec; d[dv] = m_hi; d[dv + 1] = l_hi; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < group * dv; i += blockDim.x) {
        const int h = i / dv, e = i % dv;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kPfWarps; ++w) mm = fmaxf(mm, meet[((size_t)w * group + h) * rec + dv]);
        float total = 0.0f, v = 0.0f;
#pragma unroll
        for (int w = 0; w < kPfWarps; ++w) {
            const float* src = meet + ((size_t)w * group + h) * rec;
            const float wt = src[dv] == -INFINITY ? 0.0f : fast_exp2(src[dv] - mm);
            total += src[dv + 1] * wt;
            v += src[e] * wt;
        }
        if (splits > 1) {
            // [row of the grid][head][split][dv + 2]: sums, then maximum (base 2) and weight
            float* dst = part + (((size_t)blockIdx.x * q_heads + head0 + h) * splits + split) * rec;
            dst[e] = v;
            if (e == 0) { dst[dv] = mm; dst[dv + 1] = total; }
            continue;
        }
        v = total > 0.0f ? v / total : 0.0f;
        if (gate != nullptr)
            v *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)t * gate_stride + gate_at(mod.gate_per_head, head0 + h, dv, e)])));
        out[((size_t)t * q_heads + head0 + h) * dv + e] = __float2bfloat16_rn(v);
    }
}

// The runs of a (row, head) added in their order, the gate applied, the result written.
__global__ void attention_biased_combine_kernel(const float* part, const int* __restrict__ token_slot,
                                                const int* __restrict__ rows, int q_heads, int dv, int splits,
                                                const bf16* gate, int gate_stride, int gate_per_head,
                                                bf16* __restrict__ out) {
    TLLM_PDL_ENTER();
    const int t = rows != nullptr ? rows[blockIdx.x] : blockIdx.x;
    const int head = blockIdx.y, rec = dv + 2;
    bf16* dst = out + ((size_t)t * q_heads + head) * dv;
    if (token_slot[t] < 0) {
        for (int e = threadIdx.x; e < dv; e += blockDim.x) dst[e] = __float2bfloat16_rn(0.0f);
        return;
    }
    const float* src = part + ((size_t)blockIdx.x * q_heads + head) * splits * rec;
    float mm = -INFINITY;
    for (int s2 = 0; s2 < splits; ++s2) mm = fmaxf(mm, src[s2 * rec + dv]);
    for (int e = threadIdx.x; e < dv; e += blockDim.x) {
        float total = 0.0f, v = 0.0f;
        for (int s2 = 0; s2 < splits; ++s2) {
            const float ms = src[s2 * rec + dv];
            const float w = ms == -INFINITY ? 0.0f : fast_exp2(ms - mm);
            total += src[s2 * rec + dv + 1] * w;
            v += src[s2 * rec + e] * w;
        }
        v = total > 0.0f ? v / total : 0.0f;
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)t * gate_stride + gate_at(gate_per_head, head, dv, e)])));
        dst[e] = __float2bfloat16_rn(v);
    }
}

// Blocks that share a key/value head's query heads in the one-token kernel: the fewest that leave each at
// most the tile's 16 rows and divide the heads evenly; 0 if there is no such number.
static int biased_sub_groups(int group) {
    for (int s = 1; s <= group; ++s)
        if (group % s == 0 && group / s <= 16) return s;
    return 0;
}

template <int DKP, int DVP>
static int launch_biased_decode(const void* q, const void* kp, const void* vp, long long page_stride,
                                const int* positions, const int* token_slot, const int* rows, int n_rows,
                                const int* block_table, int max_pages, int page_size, int q_heads, int kv_heads,
                                int dk, int dv, ScoreMod mod, const float* slopes, const float* sink_logit, int v_row,
                                const void* gate, int gate_stride, int splits, float* part, void* out, cudaStream_t stream) {
    const size_t smem = (size_t)2 * kPfN * ((DKP + kPfPad) + (DVP + kPfPad)) * 2;      // also holds the warps' meeting
    static OncePerDevice configured;
    if (configured.first()) {
        cudaError_t e = cudaFuncSetAttribute(attention_biased_decode_kernel<DKP, DVP>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { set_error("attention_biased_decode: %s", cudaGetErrorString(e)); return (int)e; }
        configured.done();
    }
    const int sub_groups = biased_sub_groups(q_heads / kv_heads);
    launch_pdl(kPdlAttention, attention_biased_decode_kernel<DKP, DVP>, dim3(n_rows, kv_heads * sub_groups, splits), dim3(kPfWarps * 32),
               smem, stream, (const bf16*)q, (const bf16*)kp, (const bf16*)vp, page_stride, positions, token_slot,
               rows, block_table, max_pages, page_size, page_shift_of(page_size), q_heads, kv_heads, dk, dv, mod, slopes, sink_logit, v_row,
               (const bf16*)gate, gate_stride, splits, sub_groups, part, (bf16*)out);
    if (splits > 1)
        launch_pdl(kPdlCombine, attention_biased_combine_kernel, dim3(n_rows, q_heads), dim3(dv >= 128 ? 128 : 64), 0, stream,
                   (const float*)part, token_slot, rows, q_heads, dv, splits, (const bf16*)gate, gate_stride, mod.gate_per_head, (bf16*)out);
    return finish_launch("attention_biased_decode");
}

}  // namespace tllm

using namespace tllm;

extern "C" {

int tllm_qkv_unit_store(const void* proj, int row_stride, const void* q_gain, const void* k_gain, float eps,
                        int do_norm, const int* positions, const int* token_slot, const int* block_table,
                        int max_pages, int page_size, void* k_plane, void* v_plane, long long page_stride,
                        void* q_out, int dtype, int tokens, int q_heads, int kv_heads, int dk, int dv,
                        int store, const float* inv_freq, int rot_dims, float temp_coef, int temp_every, int v_from_k,
                        const float* bias, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && dk > 0 && dv > 0, "qkv_unit_store: bad sizes");
    TLLM_REQUIRE(row_stride >= (q_heads + kv_heads) * dk + (v_from_k ? 0 : kv_heads * dv), "qkv_unit_store: rows of %d are too short", row_stride);
    TLLM_REQUIRE(rot_dims >= 0 && rot_dims <= dk && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq != nullptr),
                 "qkv_unit_store: a rotation of %d of %d elements", rot_dims, dk);
    TLLM_REQUIRE(!v_from_k || dv == dk, "qkv_unit_store: keys of width %d cannot serve as values of width %d", dk, dv);
    TLLM_REQUIRE(temp_every >= 0, "qkv_unit_store: negative constant");
    TLLM_REQUIRE(!do_norm || eps > 0.0f, "qkv_unit_store: eps must be positive");
    TLLM_REQUIRE(!store || (k_plane && v_plane && block_table && page_size > 0 && max_pages > 0),
                 "qkv_unit_store: no cache to write to");
    TLLM_REQUIRE(q_out != nullptr, "qkv_unit_store: no place for the queries");
    if (tokens == 0) return 0;
    const int heads = q_heads + 2 * kv_heads;
    const int warps = heads >= 8 ? 8 : (heads >= 4 ? 4 : 2);
#define STORE(T)                                                                                              \
    launch_pdl(kPdlQk, qkv_unit_store_kernel<T>, dim3(tokens), dim3(warps * 32), 0, stream, (const T*)proj,   \
               row_stride, (const T*)q_gain, (const T*)k_gain, eps, do_norm, positions, token_slot,           \
               block_table, max_pages, page_size, (T*)k_plane, (T*)v_plane, page_stride, (T*)q_out, q_heads,  \
               kv_heads, dk, dv, store, inv_freq, rot_dims, temp_coef, temp_every, v_from_k, bias)
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    const bool vec = dtype == kBF16 && dk % 8 == 0 && dv % 8 == 0 && dk <= 256 && rot_dims % 16 == 0 &&
                     row_stride % 8 == 0 && page_stride % 8 == 0 && aligned16(proj) && aligned16(q_out) &&
                     aligned16(k_plane) && aligned16(v_plane) && aligned16(q_gain) && aligned16(k_gain) && aligned16(bias);
#define STORE_VEC(GS)                                                                                             \
    launch_pdl(kPdlQk, qkv_unit_store_vec_kernel<GS>, dim3(tokens), dim3(256), (size_t)rot_dims * sizeof(float),  \
               stream, (const bf16*)proj, row_stride, (const bf16*)q_gain, (const bf16*)k_gain, eps, do_norm,     \
               positions, token_slot, block_table, max_pages, page_size, (bf16*)k_plane, (bf16*)v_plane,          \
               page_stride, (bf16*)q_out, q_heads, kv_heads, dk, dv, store, inv_freq, rot_dims, temp_coef,        \
               temp_every, v_from_k, bias)
    if (vec) {
        if (dk <= 8) STORE_VEC(1);
        else if (dk <= 16) STORE_VEC(2);
        else if (dk <= 32) STORE_VEC(4);
        else if (dk <= 64) STORE_VEC(8);
        else if (dk <= 128) STORE_VEC(16);
        else STORE_VEC(32);
    } else if (dtype == kBF16) STORE(bf16);
    else if (dtype == kF32) STORE(float);
    else TLLM_REQUIRE(false, "qkv_unit_store: unknown dtype %d", dtype);
#undef STORE
#undef STORE_VEC
    return finish_launch("qkv_unit_store");
}

int tllm_attention_biased_general(
    const void* q, const void* k_plane, const void* v_plane, long long page_stride, const int* positions,
    const int* token_slot, const int* block_table, int max_pages, int page_size, int dtype, int tokens,
    int q_heads, int kv_heads, int dk, int dv, float scale, float softcap, int chunk, int window, int sink,
    const float* slopes, const float* sink_logit, const float* dist_bias, int dist_len, int v_row, const void* gate, int gate_stride, int gate_per_head, void* out, cudaStream_t stream) {
    if (v_row <= 0) v_row = dv;
    TLLM_REQUIRE(dist_bias == nullptr || dist_len > 0, "attention_biased: an empty table of biases");
    TLLM_REQUIRE(v_row >= dv, "attention_biased: values of width %d in rows of %d", dv, v_row);
    TLLM_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
                 "attention_biased: %d query heads over %d key/value heads", q_heads, kv_heads);
    TLLM_REQUIRE(dk > 0 && dk <= 512 && dv > 0 && dv <= 512, "attention_biased: widths %d, %d outside 1..512", dk, dv);
    TLLM_REQUIRE(page_size > 0 && max_pages > 0, "attention_biased: bad page geometry");
    TLLM_REQUIRE(tokens <= 65535, "attention_biased: %d tokens in one step exceed 65535", tokens);
    TLLM_REQUIRE(chunk >= 0 && window >= 0 && softcap >= 0.0f, "attention_biased: negative constant");
    if (tokens == 0) return 0;
    const ScoreMod mod{scale, softcap, chunk, window, sink ? 1 : 0, dist_bias, dist_len, gate_per_head ? 1 : 0};
    if (dtype == kBF16)
        return launch_general<bf16>(q, k_plane, v_plane, page_stride, positions, token_slot, block_table, max_pages,
                                    page_size, tokens, q_heads, kv_heads, dk, dv, mod, slopes, sink_logit, v_row, gate, gate_stride, out, stream);
    if (dtype == kF32)
        return launch_general<float>(q, k_plane, v_plane, page_stride, positions, token_slot, block_table, max_pages,
                                     page_size, tokens, q_heads, kv_heads, dk, dv, mod, slopes, sink_logit, v_row, gate, gate_stride, out, stream);
    TLLM_REQUIRE(false, "attention_biased: unknown dtype %d", dtype);
}

// Whether the two bfloat16 kernels below take these sizes (else the general kernel serves).
int tllm_attention_biased_fast_ok(int q_heads, int kv_heads, int dk, int dv) {
    return q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && biased_sub_groups(q_heads / kv_heads) > 0 &&
           kv_heads * biased_sub_groups(q_heads / kv_heads) <= 65535 &&
           dk % 8 == 0 && dv % 8 == 0 && dk > 0 && dv > 0 && dk <= 128 && dv <= 128;
}

// seg_info: int[segments][4] = slot, first row, length, position of the first row.
// tiles: int[n_tiles][2] = segment, offset of the block's first query row in the segment.
int tllm_attention_biased_prefill(
    const void* q, const void* k_plane, const void* v_plane, long long page_stride, const int* seg_info,
    const int* tiles, int n_tiles, const int* block_table, int max_pages, int page_size, int q_heads,
    int kv_heads, int dk, int dv, float scale, float softcap, int chunk, int window, int sink,
    const float* slopes, const float* sink_logit, const float* dist_bias, int dist_len, int v_row, const void* gate, int gate_stride, int gate_per_head, void* out, cudaStream_t stream) {
    if (v_row <= 0) v_row = dv;
    TLLM_REQUIRE(dist_bias == nullptr || dist_len > 0, "attention_biased_prefill: an empty table of biases");
    TLLM_REQUIRE(v_row >= dv && v_row % 8 == 0, "attention_biased_prefill: values of width %d in rows of %d", dv, v_row);
    TLLM_REQUIRE(tllm_attention_biased_fast_ok(q_heads, kv_heads, dk, dv), "attention_biased_prefill: sizes %d/%d heads, widths %d/%d", q_heads, kv_heads, dk, dv);
    TLLM_REQUIRE(page_size > 0 && max_pages > 0 && n_tiles >= 0 && q_heads <= 65535, "attention_biased_prefill: bad geometry");
    TLLM_REQUIRE(chunk >= 0 && window >= 0 && softcap >= 0.0f, "attention_biased_prefill: negative constant");
    TLLM_REQUIRE(gate == nullptr || gate_per_head || gate_stride % 2 == 0, "attention_biased_prefill: odd gate stride");
    if (n_tiles == 0) return 0;
    const ScoreMod mod{scale, softcap, chunk, window, sink ? 1 : 0, dist_bias, dist_len, gate_per_head ? 1 : 0};
#define PF(A, B) launch_biased_prefill<A, B>(q, k_plane, v_plane, page_stride, seg_info, tiles, n_tiles, block_table, max_pages, \
                                             page_size, q_heads, kv_heads, dk, dv, mod, slopes, sink_logit, v_row, gate, gate_stride, out, stream)
    if (dk <= 64) return dv <= 64 ? PF(64, 64) : PF(64, 128);
    return dv <= 64 ? PF(128, 64) : PF(128, 128);
#undef PF
}

// rows: indices of the one-token rows (null: rows 0 .. n_rows - 1).  splits: runs of keys per (row,
// key/value head), each a block; with more than one, `part` holds n_rows * q_heads * splits * (dv + 2) floats.
int tllm_attention_biased_decode(
    const void* q, const void* k_plane, const void* v_plane, long long page_stride, const int* positions,
    const int* token_slot, const int* rows, int n_rows, const int* block_table, int max_pages, int page_size,
    int q_heads, int kv_heads, int dk, int dv, float scale, float softcap, int chunk, int window, int sink,
    const float* slopes, const float* sink_logit, const float* dist_bias, int dist_len, int v_row, const void* gate,
    int gate_stride, int gate_per_head, int splits, float* part, void* out, cudaStream_t stream) {
    if (v_row <= 0) v_row = dv;
    TLLM_REQUIRE(dist_bias == nullptr || dist_len > 0, "attention_biased_decode: an empty table of biases");
    TLLM_REQUIRE(v_row >= dv && v_row % 8 == 0, "attention_biased_decode: values of width %d in rows of %d", dv, v_row);
    TLLM_REQUIRE(tllm_attention_biased_fast_ok(q_heads, kv_heads, dk, dv), "attention_biased_decode: sizes %d/%d heads, widths %d/%d", q_heads, kv_heads, dk, dv);
    TLLM_REQUIRE(page_size > 0 && max_pages > 0 && n_rows >= 0 && kv_heads <= 65535, "attention_biased_decode: bad geometry");
    TLLM_REQUIRE(chunk >= 0 && window >= 0 && softcap >= 0.0f, "attention_biased_decode: negative constant");
    TLLM_REQUIRE(splits >= 1 && splits <= 64 && (splits == 1 || part != nullptr), "attention_biased_decode: %d runs of keys", splits);
    if (n_rows == 0) return 0;
    const ScoreMod mod{scale, softcap, chunk, window, sink ? 1 : 0, dist_bias, dist_len, gate_per_head ? 1 : 0};
#define DEC(A, B) launch_biased_decode<A, B>(q, k_plane, v_plane, page_stride, positions, token_slot, rows, n_rows, block_table, \
                                             max_pages, page_size, q_heads, kv_heads, dk, dv, mod, slopes, sink_logit, v_row, gate, gate_stride, \
                                             splits, part, out, stream)
    if (dk <= 64) return dv <= 64 ? DEC(64, 64) : DEC(64, 128);
    return dv <= 64 ? DEC(128, 64) : DEC(128, 128);
#undef DEC
}

}  // extern "C"
