// Mixture of experts: routing, the plan of a step's rows per expert, the experts' products over
// those rows, and the sum of what they return.  Everything the plan needs stays on the device, so a
// step with a router can be captured as a CUDA graph like any other.
//
//   route    z [T, E] float32 router logits -> the `top` experts with the largest z per token
//            (lowest index first on ties) and their weights, sigmoid(z) or softmax over the chosen;
//            `route_grouped`: scores over all experts (softmax or sigmoid), a learned correction added for
//            the choice only, experts in equal groups of neighbours of which only the best few may be
//            chosen from, the weights the chosen experts' scores as they are;
//   plan     counting sort of the T * top assignments by expert: offsets per expert, the row every
//            assignment gets, and the list of (expert, first row) tiles of the rows (64 for the mma.sync
//            products of this file, 128 for the grouped tcgen05 product);
//   products C[row] = A[row] . W_e^T for the expert e that owns the row.  The first product can
//            gather its rows from the tokens (scaled by the assignment's weight, for routers whose
//            weight multiplies the expert's input) and apply act(gate) * up in its epilogue; bfloat16
//            runs on mma.sync tiles (64 rows x 64 weight rows x 32 deep, operands prefetched through
//            registers), float32 and odd sizes run one thread per output with the sum over k in order;
//            steps with many rows take the grouped form of the tcgen05 product instead (gemm_tcgen05.cu),
//            which reads its rows by TMA: `gather` lays the token rows out in the plan's order first;
//   combine  out[t] = shared[t] + sum over the token's assignments of (weight *) y[row], in float32; an
//            assignment to an expert past the last real one (an identity expert) adds the token's input instead.
//
// A row's result does not depend on which other rows share its tile or its expert.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace tllm {

constexpr int kTileRows = 64;

// ---------------------------------------------------------------- route
// One warp per token.  E <= 1024: lane l looks at experts l, l + 32, ...; a bit per expert marks
// the ones already taken.
__global__ void moe_route_kernel(const float* z, int tokens, int experts, int top, int softmax_weights,
                                 int* __restrict__ ids, float* __restrict__ weights) {
    TLLM_PDL_ENTER();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= tokens) return;
    const float* row = z + (size_t)warp * experts;
    uint32_t taken = 0;
    float denom = 0.0f, first = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int c = 0, e = lane; e < experts; ++c, e += 32) {
            if (taken & (1u << c)) continue;
            const float v = row[e];
            if (v > best || (v == best && e < best_e) || best_e == 0x7fffffff) { best = v; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (oe != 0x7fffffff && (best_e == 0x7fffffff || ov > best || (ov == best && oe < best_e))) { best = ov; best_e = oe; }
        }
        if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
        if (k == 0) first = best;
        float w;
        if (softmax_weights) { w = expf(best - first); denom += w; }
        else w = 1.0f / (1.0f + expf(-best));
        if (lane == 0) { ids[(size_t)warp * top + k] = best_e; weights[(size_t)warp * top + k] = w; }
    }
    if (softmax_weights && lane == 0)
        for (int k = 0; k < top; ++k) weights[(size_t)warp * top + k] /= denom;
}

// Routing over scores of all experts.  One warp per token, E <= 1024; shared memory per warp: E choice scores,
// then one number per group.  score s = softmax(z) over all E (score_mode 1) or sigmoid(z) (0); choice = s +
// correction (if given); a group's score is its largest choice; only experts of the `keep` best groups can be
// chosen (lowest index first on ties, for groups and experts alike); weights are the scores s themselves.
__global__ void moe_route_grouped_kernel(const float* z, int tokens, int experts, int top, int score_mode,
                                         const float* __restrict__ correction, int groups, int keep,
                                         int* __restrict__ ids, float* __restrict__ weights) {
    extern __shared__ float route_smem[];
    TLLM_PDL_ENTER();
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warp = blockIdx.x * (blockDim.x >> 5) + wib;
    if (warp >= tokens) return;
    float* choice = route_smem + (size_t)wib * (experts + groups);
    float* gscore = choice + experts;
    const float* row = z + (size_t)warp * experts;
    float top_z = -INFINITY;
    for (int e = lane; e < experts; e += 32) top_z = fmaxf(top_z, row[e]);
    top_z = warp_max(top_z);
    float denom = 0.0f;
    if (score_mode == 1) {
        for (int e = lane; e < experts; e += 32) denom += expf(row[e] - top_z);
        denom = warp_sum(denom);
    }
    auto score_of = [&](int e) -> float {
        return score_mode == 1 ? expf(row[e] - top_z) / denom : 1.0f / (1.0f + expf(-row[e]));
    };
    for (int e = lane; e < experts; e += 32) choice[e] = score_of(e) + (correction != nullptr ? correction[e] : 0.0f);
    __syncwarp();
    const int size = experts / groups;
    if (groups > 1) {
        for (int g = lane; g < groups; g += 32) {
            float m = -INFINITY;
            for (int i = 0; i < size; ++i) m = fmaxf(m, choice[g * size + i]);
            gscore[g] = m;
        }
        __syncwarp();
        // the best `keep` groups stay; a group that is taken is marked by a NaN-free sentinel: +inf
        for (int k = 0; k < keep; ++k) {
            float best = -INFINITY;
            int best_g = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float v = gscore[g];
                if (v == INFINITY) continue;                   // already kept
                if (best_g == 0x7fffffff || v > best) { best = v; best_g = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
                if (og != 0x7fffffff && (best_g == 0x7fffffff || ov > best || (ov == best && og < best_g))) { best = ov; best_g = og; }
            }
            if (lane == 0 && best_g != 0x7fffffff) gscore[best_g] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32)
            if (gscore[e / size] != INFINITY) choice[e] = -INFINITY;
        __syncwarp();
    }
    uint32_t taken = 0;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int c = 0, e = lane; e < experts; ++c, e += 32) {
            if (taken & (1u << c)) continue;
            const float v = choice[e];
            if (best_e == 0x7fffffff || v > best) { best = v; best_e = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (oe != 0x7fffffff && (best_e == 0x7fffffff || ov > best || (ov == best && oe < best_e))) { best = ov; best_e = oe; }
        }
        if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
        if (lane == 0) { ids[(size_t)warp * top + k] = best_e; weights[(size_t)warp * top + k] = score_of(best_e); }
    }
}

// ---------------------------------------------------------------- plan
// One block.  ints: offsets [E + 1] | n_tiles [1] | row_of [n] | src_of [n] | expert_of_row [n] |
// tile_expert [max tiles] | tile_row0 [max tiles].
// Experts from `real` on have no matrices (their assignments get rows, and no tiles).
__global__ void moe_plan_kernel(const int* ids, int n, int experts, int real, int tile_rows, int* offsets, int* n_tiles,
                                int* row_of, int* src_of, int* expert_of_row, int* tile_expert, int* tile_row0) {
    extern __shared__ int plan_smem[];
    TLLM_PDL_ENTER();
    int* count = plan_smem;                 // [E]
    int* cursor = plan_smem + experts;      // [E]
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&count[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < experts; ++e) {
            offsets[e] = cursor[e] = at;
            if (e < real)
                for (int r = at; r < at + count[e]; r += tile_rows) { tile_expert[tiles] = e; tile_row0[tiles] = r; ++tiles; }
            at += count[e];
        }
        offsets[experts] = at;
        *n_tiles = tiles;
    }
    __syncthreads();
    // rows of an expert in the order of the assignments: thread 0 of each expert's turn would be exact but
    // slow; the order within an expert changes no row's value, so the rows are handed out atomically
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = ids[i];
        const int r = atomicAdd(&cursor[e], 1);
        row_of[i] = r;
        src_of[r] = i;
        expert_of_row[r] = e;
    }
}

// ---------------------------------------------------------------- products, bfloat16 on mma.sync
constexpr int kGM = kTileRows, kGN = 64, kGK = 32, kGPad = 8, kGThreads = 128;

__device__ __forceinline__ uint4 scale8(uint4 raw, float w) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        h[i] = __floats2bfloat162_rn(f.x * w, f.y * w);
    }
    return raw;
}

// Row of an expert's gate|up matrix that holds output column `col`'s gate (or up) weights: stacked
// ([gate; up]) or interleaved by eight (eight gate rows, their eight up rows, and so on).
__device__ __forceinline__ int gate_up_row(int col, bool up, int n, int interleaved) {
    if (interleaved) return 16 * (col >> 3) + (col & 7) + (up ? 8 : 0);
    return up ? n + col : col;
}

// MODE 1 (gated): a block's 64 weight rows are, per warp column of 32, sixteen gate rows and the sixteen up rows
// that belong to them; the block writes 32 columns of act(gate) * up in bfloat16.  Otherwise 64 columns
// of the plain product, in float32 (MODE 0) or, with the activation on every output, in bfloat16 (MODE 2).
template <int MODE, bool GATHER>
__global__ void __launch_bounds__(kGThreads)
moe_grouped_mma_kernel(const bf16* A, int lda, const int* src_of, const float* weight_of, int top,
                       const bf16* W, long long w_stride, const int* tile_expert, const int* tile_row0,
                       const int* n_tiles, const int* offsets, int N, int K, int act, int interleaved, void* C) {
    __shared__ __align__(16) bf16 As[2][kGM][kGK + kGPad];
    __shared__ __align__(16) bf16 Bs[2][kGN][kGK + kGPad];
    constexpr bool GATED = MODE == 1;
    TLLM_PDL_ENTER();
    if ((int)blockIdx.y >= *n_tiles) return;
    const int e = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y];
    const int rows_here = min(kGM, offsets[e + 1] - row0);
    constexpr int kCols = GATED ? kGN / 2 : kGN;
    const int n0 = blockIdx.x * kCols;
    const bf16* We = W + (long long)e * w_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 1, wn = warp & 1;

    // the two 16-byte pieces of each operand tile this thread moves
    const bf16* a_src[2];
    const bf16* b_src[2];
    float a_w[2];
    int piece_row[2], piece_col[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int c = tid + kGThreads * i, r = c >> 2, kc = (c & 3) * 8;
        piece_row[i] = r;
        piece_col[i] = kc;
        a_src[i] = nullptr;
        a_w[i] = 1.0f;
        if (r < rows_here) {
            if (GATHER) {
                const int a = src_of[row0 + r];
                a_src[i] = A + (size_t)(a / top) * lda + kc;
                if (weight_of != nullptr) a_w[i] = weight_of[a];
            } else {
                a_src[i] = A + (size_t)(row0 + r) * lda + kc;
            }
        }
        int wrow;      // row of the expert's weight that lands in row r of the tile
        if (GATED) {
            const int half = r >> 5, j = r & 31;
            const int col = n0 + half * 16 + (j & 15);
            wrow = col < N ? gate_up_row(col, j >= 16, N, interleaved) : -1;
        } else {
            wrow = n0 + r < N ? n0 + r : -1;
        }
        b_src[i] = wrow >= 0 ? We + (size_t)wrow * K + kc : nullptr;
    }
    uint4 a_reg[2], b_reg[2];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const bool in_k = k0 + piece_col[i] < K;
            a_reg[i] = (a_src[i] != nullptr && in_k) ? *reinterpret_cast<const uint4*>(a_src[i] + k0) : make_uint4(0, 0, 0, 0);
            b_reg[i] = (b_src[i] != nullptr && in_k) ? __ldg(reinterpret_cast<const uint4*>(b_src[i] + k0)) : make_uint4(0, 0, 0, 0);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint4 a = a_reg[i];
            if (GATHER && a_w[i] != 1.0f) a = scale8(a, a_w[i]);
            *reinterpret_cast<uint4*>(&As[buf][piece_row[i]][piece_col[i]]) = a;
            *reinterpret_cast<uint4*>(&Bs[buf][piece_row[i]][piece_col[i]]) = b_reg[i];
        }
    };

    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;

    const int k_tiles = (K + kGK - 1) / kGK;
    fetch(0);
    stash(0);
    __syncthreads();
    for (int kt = 0; kt < k_tiles; ++kt) {
        const int cur = kt & 1;
        if (kt + 1 < k_tiles) fetch((kt + 1) * kGK);
#pragma unroll
        for (int ks = 0; ks < kGK; ks += 16) {
            uint32_t af[2][4], bfrag[2][4];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) {
                const int r = wm * 32 + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(af[mi], smem_u32(&As[cur][r][ks + (lane >> 4) * 8]));
            }
#pragma unroll
            for (int nj = 0; nj < 2; ++nj) {
                const int r = wn * 32 + nj * 16 + (lane & 7) + (lane >> 4) * 8;
                ldmatrix_x4(bfrag[nj], smem_u32(&Bs[cur][r][ks + ((lane >> 3) & 1) * 8]));
            }
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) {
                    const uint32_t b[2] = {bfrag[ni >> 1][(ni & 1) * 2], bfrag[ni >> 1][(ni & 1) * 2 + 1]};
                    mma_bf16_16816(acc[mi][ni], af[mi], b);
                }
        }
        if (kt + 1 < k_tiles) stash(cur ^ 1);
        __syncthreads();
    }

#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int r = wm * 32 + mi * 16 + (lane >> 2) + hrow * 8;
            if (r >= rows_here) continue;
            if (GATED) {
                bf16* out = (bf16*)C + (size_t)(row0 + r) * N;
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    const int col = n0 + wn * 16 + ni * 8 + (lane & 3) * 2;
                    const float g0 = acc[mi][ni][hrow * 2], g1 = acc[mi][ni][hrow * 2 + 1];
                    const float u0 = acc[mi][ni + 2][hrow * 2], u1 = acc[mi][ni + 2][hrow * 2 + 1];
                    if (col < N) out[col] = __float2bfloat16_rn(gate_act(g0, act) * u0);
                    if (col + 1 < N) out[col + 1] = __float2bfloat16_rn(gate_act(g1, act) * u1);
                }
            } else if (MODE == 2) {
                bf16* out = (bf16*)C + (size_t)(row0 + r) * N;
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) {
                    const int col = n0 + wn * 32 + ni * 8 + (lane & 3) * 2;
                    if (col < N) out[col] = __float2bfloat16_rn(gate_act(acc[mi][ni][hrow * 2], act));
                    if (col + 1 < N) out[col + 1] = __float2bfloat16_rn(gate_act(acc[mi][ni][hrow * 2 + 1], act));
                }
            } else {
                float* out = (float*)C + (size_t)(row0 + r) * N;
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) {
                    const int col = n0 + wn * 32 + ni * 8 + (lane & 3) * 2;
                    if (col < N) out[col] = acc[mi][ni][hrow * 2];
                    if (col + 1 < N) out[col + 1] = acc[mi][ni][hrow * 2 + 1];
                }
            }
        }
}

// ---------------------------------------------------------------- products, plain
// One thread per output: float32 sum over k in order.  TA: storage type of A and of a gated (MODE 1) or
// activated (MODE 2) result; MODE 0 leaves float32.
template <typename TA, int MODE, bool GATHER>
__global__ void moe_grouped_plain_kernel(const TA* A, int lda, const int* src_of, const float* weight_of, int top,
                                         const TA* W, long long w_stride, const int* expert_of_row, int rows,
                                         int N, int K, int act, int interleaved, int real, void* C) {
    constexpr bool GATED = MODE == 1;
    TLLM_PDL_ENTER();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * N) return;
    if (expert_of_row[idx / N] >= real) return;      // a row of an expert without matrices
    const int r = (int)(idx / N), n = (int)(idx % N);
    const TA* a;
    float w = 1.0f;
    if (GATHER) {
        const int s = src_of[r];
        a = A + (size_t)(s / top) * lda;
        if (weight_of != nullptr) w = weight_of[s];
    } else {
        a = A + (size_t)r * lda;
    }
    const TA* We = W + (long long)expert_of_row[r] * w_stride;
    const TA* wg = We + (size_t)(GATED ? gate_up_row(n, false, N, interleaved) : n) * K;
    float g = 0.0f, u = 0.0f;
    if (GATED) {
        const TA* wu = We + (size_t)gate_up_row(n, true, N, interleaved) * K;
        for (int k = 0; k < K; ++k) {
            const float x = to_f32<TA>(from_f32<TA>(to_f32<TA>(a[k]) * w));     // the rounding of the scaled row
            g += x * to_f32<TA>(wg[k]);
            u += x * to_f32<TA>(wu[k]);
        }
        ((TA*)C)[idx] = from_f32<TA>(gate_act(g, act) * u);
    } else {
        for (int k = 0; k < K; ++k) g += to_f32<TA>(from_f32<TA>(to_f32<TA>(a[k]) * w)) * to_f32<TA>(wg[k]);
        if (MODE == 2) ((TA*)C)[idx] = from_f32<TA>(gate_act(g, act));
        else ((float*)C)[idx] = g;
    }
}

// ---------------------------------------------------------------- gather
// xs[row] = x[token of the row] (* the assignment's weight): the experts' rows one after the other, for a
// product that reads its rows by TMA.  16 bytes per thread.
__global__ void moe_gather_kernel(const bf16* x, const int* src_of, const float* weight_of, int top, bf16* xs,
                                  int width, size_t total_chunks) {
    TLLM_PDL_ENTER();
    const int per_row = width >> 3;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total_chunks; idx += stride) {
        const size_t r = idx / per_row, c = idx - r * per_row;
        const int a = src_of[r];
        uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(a / top) * width + c * 8);
        if (weight_of != nullptr) raw = scale8(raw, weight_of[a]);
        *reinterpret_cast<uint4*>(xs + r * width + c * 8) = raw;
    }
}

// ---------------------------------------------------------------- combine
// x, expert_of_row, real: where given, an assignment whose expert is `real` or later adds the token's own row
// of x (times the weight) instead of a row of y.
template <typename T, typename TY>
__global__ void moe_combine_kernel(const TY* y, const int* row_of, const float* weight_of, int top,
                                   const T* shared, T* out, int width, size_t total, const T* x,
                                   const int* expert_of_row, int real) {
    TLLM_PDL_ENTER();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const size_t t = idx / width, i = idx - t * width;
        float v = shared != nullptr ? to_f32<T>(shared[idx]) : 0.0f;
        for (int k = 0; k < top; ++k) {
            const int row = row_of[t * top + k];
            const float yv = (x != nullptr && expert_of_row[row] >= real) ? to_f32<T>(x[idx])
                                                                         : to_f32<TY>(y[(size_t)row * width + i]);
            v += weight_of != nullptr ? weight_of[t * top + k] * yv : yv;
        }
        out[idx] = from_f32<T>(v);
    }
}

}  // namespace tllm

using namespace tllm;

extern "C" {

int tllm_moe_tile_rows() { return kTileRows; }

int tllm_moe_route(const float* z, int tokens, int experts, int top, int softmax_weights, int* ids,
                   float* weights, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && experts > 0 && experts <= 1024 && top > 0 && top <= experts,
                 "moe_route: %d experts, top %d", experts, top);
    if (tokens == 0) return 0;
    const int warps = 4;
    launch_pdl(kPdlOther, moe_route_kernel, dim3((tokens + warps - 1) / warps), dim3(warps * 32), 0, stream,
               z, tokens, experts, top, softmax_weights, ids, weights);
    return finish_launch("moe_route");
}

// score_mode: 0 sigmoid(z), 1 softmax(z) over all experts.  correction [experts] float32 or null.  groups equal
// groups of neighbouring experts, of which the `keep` with the best member may be chosen from.
int tllm_moe_route_grouped(const float* z, int tokens, int experts, int top, int score_mode, const float* correction,
                           int groups, int keep, int* ids, float* weights, cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && experts > 0 && experts <= 1024 && top > 0 && top <= experts,
                 "moe_route_grouped: %d experts, top %d", experts, top);
    TLLM_REQUIRE(score_mode == 0 || score_mode == 1, "moe_route_grouped: unknown scores %d", score_mode);
    TLLM_REQUIRE(groups > 0 && experts % groups == 0 && keep > 0 && keep <= groups && keep * (experts / groups) >= top,
                 "moe_route_grouped: %d groups of %d experts, %d kept, top %d", groups, experts, keep, top);
    if (tokens == 0) return 0;
    const int warps = 4;
    launch_pdl(kPdlOther, moe_route_grouped_kernel, dim3((tokens + warps - 1) / warps), dim3(warps * 32),
               (size_t)warps * (experts + groups) * sizeof(float), stream, z, tokens, experts, top, score_mode,
               correction, groups, keep, ids, weights);
    return finish_launch("moe_route_grouped");
}

int tllm_moe_plan(const int* ids, int n, int experts, int real, int tile_rows, int* offsets, int* n_tiles, int* row_of,
                  int* src_of, int* expert_of_row, int* tile_expert, int* tile_row0, cudaStream_t stream) {
    TLLM_REQUIRE(n > 0 && experts > 0 && experts <= 4096 && tile_rows > 0 && real >= 0 && real <= experts, "moe_plan: bad sizes");
    launch_pdl(kPdlOther, moe_plan_kernel, dim3(1), dim3(1024), (size_t)2 * experts * sizeof(int), stream,
               ids, n, experts, real, tile_rows, offsets, n_tiles, row_of, src_of, expert_of_row, tile_expert, tile_row0);
    return finish_launch("moe_plan");
}

// rows: all rows of the plan (tokens * top); max_tiles: bound on the plan's tiles.  mode 1 (gated): W is
// [experts][2 N][K] (gate rows, then up rows) and C [rows, N] in the storage type; else W is
// [experts][N][K] and C [rows, N] float32 (mode 0) or act(.) in the storage type (mode 2).  gather: A is
// [tokens, K] and row r reads token src_of[r] / top, scaled by weight_of[src_of[r]] if that is given.
// real: experts that have matrices (rows of later ones are left alone).
int tllm_moe_grouped(const void* A, int lda, const int* src_of, const float* weight_of, int top, const void* W,
                     long long w_stride, const int* tile_expert, const int* tile_row0, const int* n_tiles,
                     const int* offsets, const int* expert_of_row, int rows, int max_tiles, int N, int K,
                     int dtype, int mode, int gather, int act, int interleaved, int real, void* C, cudaStream_t stream) {
    const bool gated = mode == 1;
    TLLM_REQUIRE(mode >= 0 && mode <= 2, "moe_grouped: unknown mode %d", mode);
    TLLM_REQUIRE(!interleaved || (gated && N % 8 == 0), "moe_grouped: interleaved gate and up rows need N %% 8 == 0");
    TLLM_REQUIRE(rows >= 0 && N > 0 && K > 0 && max_tiles > 0, "moe_grouped: bad sizes");
    TLLM_REQUIRE(dtype == kBF16 || dtype == kF32, "moe_grouped: unknown dtype %d", dtype);
    TLLM_REQUIRE(max_tiles <= 65535, "moe_grouped: %d row tiles exceed 65535", max_tiles);
    if (rows == 0) return 0;
    const bool aligned = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15u) == 0;
    if (dtype == kBF16 && K % 8 == 0 && lda % 8 == 0 && aligned) {
        const int cols = gated ? kGN / 2 : kGN;
        const dim3 grid((N + cols - 1) / cols, max_tiles), block(kGThreads);
#define MMA(G, H)                                                                                              \
    launch_pdl(kPdlOther, moe_grouped_mma_kernel<G, H>, grid, block, 0, stream, (const bf16*)A, lda, src_of,    \
               weight_of, top, (const bf16*)W, w_stride, tile_expert, tile_row0, n_tiles, offsets, N, K, act, interleaved, C)
        if (gated && gather) MMA(1, true);
        else if (gated) MMA(1, false);
        else if (mode == 2 && gather) MMA(2, true);
        else if (mode == 2) MMA(2, false);
        else if (gather) MMA(0, true);
        else MMA(0, false);
#undef MMA
        return finish_launch("moe_grouped");
    }
    const size_t total = (size_t)rows * N;
    const dim3 grid((unsigned)((total + 255) / 256)), block(256);
#define PLAIN(T, G, H)                                                                                          \
    launch_pdl(kPdlOther, moe_grouped_plain_kernel<T, G, H>, grid, block, 0, stream, (const T*)A, lda, src_of,  \
               weight_of, top, (const T*)W, w_stride, expert_of_row, rows, N, K, act, interleaved, real, C)
#define PLAIN_T(T)                                         \
    do {                                                   \
        if (gated && gather) PLAIN(T, 1, true);            \
        else if (gated) PLAIN(T, 1, false);                \
        else if (mode == 2 && gather) PLAIN(T, 2, true);   \
        else if (mode == 2) PLAIN(T, 2, false);            \
        else if (gather) PLAIN(T, 0, true);                \
        else PLAIN(T, 0, false);                           \
    } while (0)
    if (dtype == kBF16) PLAIN_T(bf16);
    else PLAIN_T(float);
#undef PLAIN_T
#undef PLAIN
    return finish_launch("moe_grouped");
}

// y_dtype: float32 rows, or rows in the storage type (the grouped tcgen05 product writes bfloat16).
int tllm_moe_gather(const void* x, const int* src_of, const float* weight_of, int top, void* xs, int rows, int width,
                    cudaStream_t stream) {
    TLLM_REQUIRE(rows >= 0 && width > 0 && width % 8 == 0 && top > 0, "moe_gather: bad sizes");
    const size_t chunks = (size_t)rows * (width / 8);
    if (chunks == 0) return 0;
    size_t g = (chunks + 255) / 256;
    launch_pdl(kPdlOther, moe_gather_kernel, dim3((unsigned)(g > 148 * 16 ? 148 * 16 : g)), dim3(256), 0, stream,
               (const bf16*)x, src_of, weight_of, top, (bf16*)xs, width, chunks);
    return finish_launch("moe_gather");
}

// x, expert_of_row, real: all or none; assignments to experts from `real` on add the token's row of x.
int tllm_moe_combine(const void* y, int y_dtype, const int* row_of, const float* weight_of, int top, const void* shared,
                     void* out, int dtype, int tokens, int width, const void* x, const int* expert_of_row, int real,
                     cudaStream_t stream) {
    TLLM_REQUIRE(tokens >= 0 && width > 0 && top > 0, "moe_combine: bad sizes");
    TLLM_REQUIRE(x == nullptr || expert_of_row != nullptr, "moe_combine: identity experts need the rows' experts");
    const size_t total = (size_t)tokens * width;
    if (total == 0) return 0;
    const int block = 256;
    size_t g = (total + block - 1) / block;
    const int grid = (int)(g > 148 * 16 ? 148 * 16 : g);
    if (dtype == kBF16 && y_dtype == kBF16)
        launch_pdl(kPdlOther, moe_combine_kernel<bf16, bf16>, dim3(grid), dim3(block), 0, stream, (const bf16*)y, row_of, weight_of, top,
                   (const bf16*)shared, (bf16*)out, width, total, (const bf16*)x, expert_of_row, real);
    else if (dtype == kBF16 && y_dtype == kF32)
        launch_pdl(kPdlOther, moe_combine_kernel<bf16, float>, dim3(grid), dim3(block), 0, stream, (const float*)y, row_of, weight_of, top,
                   (const bf16*)shared, (bf16*)out, width, total, (const bf16*)x, expert_of_row, real);
    else if (dtype == kF32 && y_dtype == kF32)
        launch_pdl(kPdlOther, moe_combine_kernel<float, float>, dim3(grid), dim3(block), 0, stream, (const float*)y, row_of, weight_of, top,
                   (const float*)shared, (float*)out, width, total, (const float*)x, expert_of_row, real);
    else
        TLLM_REQUIRE(false, "moe_combine: unknown dtypes %d, %d", dtype, y_dtype);
    return finish_launch("moe_combine");
}

}  // extern "C"
