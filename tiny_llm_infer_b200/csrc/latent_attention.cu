// Attention whose keys and values are made from one small vector per token (a latent c of width
// `rank`) and one rotated key part of width `rot` that all heads share.  The cache holds [c | rotated
// part] per token, one plane of one "head", and nothing per head.  The per-head matrices that would make
// keys (Wk_h c) and values (Wv_h c) are moved to the query's side instead:
//
//   q_h . (Wk_h c) = (Wk_h^T q_h) . c            so the score is [Wk_h^T q_h | rotated q_h] . [c | rotated k]
//   sum_j p_j (Wv_h c_j) = Wv_h (sum_j p_j c_j)  so the attention returns a mix of latents per head
//
// which makes the attention itself multi-query attention over the cached vectors (the paged kernels with
// the modified score serve it: keys of width rank + rot, values the first `rank` elements of the same
// rows).  This file has what goes around it:
//
//   latent_norm_store  per token: RMS norm of the query's latent (for the product that makes the queries),
//                      RMS norm of c, rotation of the shared key part, write of [c | rotated] into its page.
//   latent_query       per token and head: [Wk_h^T q_h (made by a batched product) | rotated part of q_h].
//   heads_gate         per token: out[t, h, :] = x[h, t, :] * sigmoid(gate[t, h, :]), the batched product's
//                      [heads, tokens, width] order turned back into rows.
//
// The rotation pairs neighbours (2i, 2i + 1) of the first `rot_dims` elements, or, `half_pairs`, elements i and
// i + rot_dims / 2: (u, v) -> (u cos a - v sin a, v cos a + u sin a) * mag, a = position * freq_i as a float32
// product, cos and sin from the precise functions.
#include "common.cuh"

namespace tllm {

template <typename T>
__global__ void latent_norm_store_kernel(const T* proj, int ld, int q_rank, int rank, int rot, int rot_dims,
                                         const float* __restrict__ q_gain, const float* __restrict__ c_gain,
                                         float eps, const float* __restrict__ freq, float mag,
                                         const int* __restrict__ positions, const int* __restrict__ token_slot,
                                         const int* __restrict__ block_table, int max_pages, int page_size,
                                         T* plane, long long page_stride, T* cq, int store, int half_pairs) {
    __shared__ float scratch[32];
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int slot = token_slot[t];
    if (slot < 0) {                           // a row without a request: a defined, harmless latent
        for (int e = threadIdx.x; e < q_rank; e += blockDim.x) cq[(size_t)t * q_rank + e] = from_f32<T>(0.0f);
        return;
    }
    const T* row = proj + (size_t)t * ld;
    if (q_rank > 0) {
        float sum = 0.0f;
        for (int e = threadIdx.x; e < q_rank; e += blockDim.x) { const float x = to_f32<T>(row[e]); sum += x * x; }
        sum = block_sum(sum, scratch);
        const float sc = 1.0f / sqrtf(sum / (float)q_rank + eps);
        for (int e = threadIdx.x; e < q_rank; e += blockDim.x)
            cq[(size_t)t * q_rank + e] = from_f32<T>(to_f32<T>(row[e]) * sc * q_gain[e]);
    }
    if (!store) return;
    const int pos = positions[t];
    const int page = block_table[(size_t)slot * max_pages + pos / page_size];
    if (page < 0) return;                     // no page held: nothing to write (the host reserves before a step)
    T* dst = plane + (long long)page * page_stride + (size_t)(pos % page_size) * (rank + rot);
    const T* c = row + q_rank;
    float sum = 0.0f;
    for (int e = threadIdx.x; e < rank; e += blockDim.x) { const float x = to_f32<T>(c[e]); sum += x * x; }
    sum = block_sum(sum, scratch);
    const float sc = 1.0f / sqrtf(sum / (float)rank + eps);
    for (int e = threadIdx.x; e < rank; e += blockDim.x) dst[e] = from_f32<T>(to_f32<T>(c[e]) * sc * c_gain[e]);
    const T* kr = c + rank;
    for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
        const float a = (float)pos * freq[i];
        const float cs = cosf(a) * mag, sn = sinf(a) * mag;
        const int iu = half_pairs ? i : 2 * i, iv = half_pairs ? i + rot_dims / 2 : 2 * i + 1;
        const float u = to_f32<T>(kr[iu]), v = to_f32<T>(kr[iv]);
        dst[rank + iu] = from_f32<T>(u * cs - v * sn);
        dst[rank + iv] = from_f32<T>(v * cs + u * sn);
    }
    for (int e = rot_dims + threadIdx.x; e < rot; e += blockDim.x) dst[rank + e] = kr[e];
}

// q [T, heads, plain + rot] in rows of ldq elements; lat [heads, T, rank]; out [T, heads, rank + rot]
template <typename T>
__global__ void latent_query_kernel(const T* q, int ldq, const T* lat, int heads, int plain, int rot, int rot_dims, int rank,
                                    const float* __restrict__ freq, float mag, const int* __restrict__ positions,
                                    const int* __restrict__ token_slot, int tokens, T* out, int half_pairs) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const int width = rank + rot;
    if (token_slot[t] < 0) {
        for (int i = threadIdx.x; i < heads * width; i += blockDim.x) out[(size_t)t * heads * width + i] = from_f32<T>(0.0f);
        return;
    }
    const int pos = positions[t];
    const int total = heads * width, per_block = (total + gridDim.y - 1) / gridDim.y;     // few rows: a row over several blocks
    const int i_end = min(total, (int)(blockIdx.y + 1) * per_block);
    for (int i = blockIdx.y * per_block + threadIdx.x; i < i_end; i += blockDim.x) {
        const int h = i / width, e = i - h * width;
        T* dst = out + ((size_t)t * heads + h) * width;
        if (e < rank) {
            dst[e] = lat[((size_t)h * tokens + t) * rank + e];
            continue;
        }
        const int d = e - rank;
        const T* src = q + (size_t)t * ldq + (size_t)h * (plain + rot) + plain;
        if (d >= rot_dims) { dst[e] = src[d]; continue; }
        const int hw = rot_dims >> 1;
        const int pair = half_pairs ? (d < hw ? d : d - hw) : d >> 1;
        const bool second = half_pairs ? d >= hw : (d & 1);
        const float a = (float)pos * freq[pair];
        const float cs = cosf(a) * mag, sn = sinf(a) * mag;
        const float u = to_f32<T>(src[half_pairs ? pair : 2 * pair]), v = to_f32<T>(src[half_pairs ? pair + hw : 2 * pair + 1]);
        dst[e] = from_f32<T>(second ? v * cs + u * sn : u * cs - v * sn);
    }
}

// x [heads, T, width]; gate rows of stride ldg, one number per element or, `per_head`, one per head; out [T, heads * width]
template <typename T>
__global__ void heads_gate_kernel(const T* x, const T* gate, int ldg, int heads, int width, int tokens,
                                  const int* __restrict__ token_slot, T* out, int per_head) {
    TLLM_PDL_ENTER();
    const int t = blockIdx.x;
    const bool pad = token_slot != nullptr && token_slot[t] < 0;
    const int total = heads * width, per_block = (total + gridDim.y - 1) / gridDim.y;
    const int i_end = min(total, (int)(blockIdx.y + 1) * per_block);
    for (int i = blockIdx.y * per_block + threadIdx.x; i < i_end; i += blockDim.x) {
        const int h = i / width, e = i - h * width;
        float v = 0.0f;
        if (!pad) {
            v = to_f32<T>(x[((size_t)h * tokens + t) * width + e]);
            if (gate != nullptr) v *= 1.0f / (1.0f + expf(-to_f32<T>(gate[(size_t)t * ldg + (per_head ? h : i)])));
        }
        out[(size_t)t * heads * width + i] = from_f32<T>(v);
    }
}

// Blocks that share a row of `elements` when the rows alone would leave the GPU idle: at least 256 elements each.
static int row_split(int rows, int elements) {
    const int sms = sm_count_cached() > 0 ? sm_count_cached() : 148;
    int split = 1;
    while (split < 64 && (long long)rows * split < 2LL * sms && elements / (split * 2) >= 256) split *= 2;
    return split;
}

}  // namespace tllm

using namespace tllm;

extern "C" {

int tllm_latent_norm_store(const void* proj, int ld, int dtype, int q_rank, int rank, int rot, int rot_dims,
                           const float* q_gain, const float* c_gain, float eps, const float* freq, float mag,
                           const int* positions, const int* token_slot, const int* block_table, int max_pages,
                           int page_size, void* plane, long long page_stride, void* cq, int store, int tokens,
                           int half_pairs, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && q_rank >= 0 && rank > 0 && rot >= 0 && rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0,
                 "latent_norm_store: bad sizes");
    TLLM_REQUIRE(ld >= q_rank + rank + rot && eps > 0.0f, "latent_norm_store: rows too short");
    TLLM_REQUIRE(!store || (plane && block_table && page_size > 0 && max_pages > 0), "latent_norm_store: no cache to write to");
    TLLM_REQUIRE(q_rank == 0 || (cq != nullptr && q_gain != nullptr), "latent_norm_store: no place for the query's latent");
    if (tokens == 0) return 0;
#define STORE(T)                                                                                                   \
    launch_pdl(kPdlQk, latent_norm_store_kernel<T>, dim3(tokens), dim3(128), 0, stream, (const T*)proj, ld, q_rank, \
               rank, rot, rot_dims, q_gain, c_gain, eps, freq, mag, positions, token_slot, block_table, max_pages,  \
               page_size, (T*)plane, page_stride, (T*)cq, store, half_pairs)
    if (dtype == kBF16) STORE(bf16);
    else if (dtype == kF32) STORE(float);
    else TLLM_REQUIRE(false, "latent_norm_store: unknown dtype %d", dtype);
#undef STORE
    return finish_launch("latent_norm_store");
}

int tllm_latent_query(const void* q, int ldq, const void* lat, int dtype, int heads, int plain, int rot, int rot_dims, int rank,
                      const float* freq, float mag, const int* positions, const int* token_slot, int tokens, void* out,
                      int half_pairs, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && heads > 0 && plain >= 0 && rot >= 0 && rank > 0 && rot_dims <= rot && rot_dims % 2 == 0,
                 "latent_query: bad sizes");
    TLLM_REQUIRE(ldq >= heads * (plain + rot), "latent_query: rows of %d are too short", ldq);
    if (tokens == 0) return 0;
    const int split = row_split(tokens, heads * (rank + rot));
    if (dtype == kBF16)
        launch_pdl(kPdlQk, latent_query_kernel<bf16>, dim3(tokens, split), dim3(256), 0, stream, (const bf16*)q, ldq, (const bf16*)lat, heads,
                   plain, rot, rot_dims, rank, freq, mag, positions, token_slot, tokens, (bf16*)out, half_pairs);
    else if (dtype == kF32)
        launch_pdl(kPdlQk, latent_query_kernel<float>, dim3(tokens, split), dim3(256), 0, stream, (const float*)q, ldq, (const float*)lat, heads,
                   plain, rot, rot_dims, rank, freq, mag, positions, token_slot, tokens, (float*)out, half_pairs);
    else TLLM_REQUIRE(false, "latent_query: unknown dtype %d", dtype);
    return finish_launch("latent_query");
}

int tllm_heads_gate(const void* x, const void* gate, int ldg, int dtype, int heads, int width, int tokens,
                    const int* token_slot, void* out, int per_head, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && heads > 0 && width > 0 && (gate == nullptr || ldg >= (per_head ? heads : heads * width)), "heads_gate: bad sizes");
    if (tokens == 0) return 0;
    const int split = row_split(tokens, heads * width);
    if (dtype == kBF16)
        launch_pdl(kPdlOther, heads_gate_kernel<bf16>, dim3(tokens, split), dim3(256), 0, stream, (const bf16*)x, (const bf16*)gate, ldg,
                   heads, width, tokens, token_slot, (bf16*)out, per_head);
    else if (dtype == kF32)
        launch_pdl(kPdlOther, heads_gate_kernel<float>, dim3(tokens, split), dim3(256), 0, stream, (const float*)x, (const float*)gate, ldg,
                   heads, width, tokens, token_slot, (float*)out, per_head);
    else TLLM_REQUIRE(false, "heads_gate: unknown dtype %d", dtype);
    return finish_launch("heads_gate");
}

}  // extern "C"
