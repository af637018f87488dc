// A routed feed-forward (mixture of experts) without a trip to the host:
//   route_top    softmax over the experts' logits in float, the ``top`` largest scores and their experts per token
//   plan         a counting sort of the (token, choice) pairs by expert, and the list of row tiles of every expert
//   gate/up      act[row] = silu(h[token(row)] Wg[e]^T) * (h[token(row)] Wu[e]^T) over the sorted rows
//   down         y[row] = act[row] Wd[e]^T, float
//   combine      out[token] = sum over its choices of weight * y[row of the pair] (+ a shared expert's output)
// The grids of the two products are sized for the worst case (every expert adds at most one partial tile); blocks
// beyond the tiles that the plan counted return at once.  The order of the rows inside an expert's range depends on
// the order in which threads take their places; a row's result does not, and a token's sum is taken in the order of
// its choices.
#define FE_PDL_CLASS 128
#include <math_constants.h>
#include <mma.h>

#include "common.cuh"

using namespace fe;

constexpr int ROUTE_MAX_EXPERTS = 1024;

// What an expert does with its gate and up products.  limit 0: silu(g) * u.  limit > 0 (the clamped form):
// g <- min(g, limit), u <- clamp(u, -limit, limit), then g * sigmoid(1.702 g) * (u + 1).
__device__ __forceinline__ float expert_activation(float g, float u, float limit) {
    if (limit > 0.f) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
    }
    return g / (1.f + expf(-g)) * u;
}

// What an expert without a gate does with its one product.
__device__ __forceinline__ float squared_relu(float z) { return z > 0.f ? z * z : 0.f; }

// One warp per token.  ties go to the lower expert index.  ``over_chosen`` 0: the weights are the chosen experts' shares of
// the softmax over all logits; 1: the ``top`` largest logits are chosen and the weights are the softmax over those alone.
// ``correction`` (one number per expert, may be null; over_chosen 0 only): added to the shares for the choice, not for the
// weights.  ``groups`` > 1: the experts form that many equal groups of neighbours; a group's score is its largest (corrected)
// share, and only experts of the ``keep`` best groups can be chosen (ties to the lower group).
__global__ void route_top_kernel(const float* __restrict__ logits, int* __restrict__ chosen, float* __restrict__ weights,
                                 int T, int experts, int top, float scale, int over_chosen, const float* __restrict__ correction,
                                 int groups, int keep) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float rows[];               // a warp: what it ranks by [experts], the shares [experts], groups [2 groups]
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + w;
    if (t >= T) return;
    float* s = rows + (size_t)w * (2 * experts + 2 * groups);
    float* share_of = s + experts;
    float* group_score = share_of + experts;      // [groups], then 1 for a kept group [groups]
    float* group_kept = group_score + groups;
    const bool corrected = !over_chosen && (correction != nullptr || groups > 1);
    const float* z = logits + (size_t)t * experts;
    float m = -CUDART_INF_F;
    for (int e = lane; e < experts; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) {
        const float p = expf(z[e] - m);
        s[e] = over_chosen ? z[e] : p;            // what the experts are ranked by
        sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    if (corrected) {
        // ranked by share + correction; the share itself is kept for the weight
        for (int e = lane; e < experts; e += 32) {
            const float share = s[e] / sum;
            share_of[e] = share;
            s[e] = share + (correction ? correction[e] : 0.f);
        }
        __syncwarp();
        if (groups > 1) {
            const int size = experts / groups;
            for (int g = lane; g < groups; g += 32) {
                float best = -CUDART_INF_F;
                for (int e = g * size; e < (g + 1) * size; ++e) best = fmaxf(best, s[e]);
                group_score[g] = best;
                group_kept[g] = 0.f;
            }
            __syncwarp();
            for (int pick = 0; pick < keep; ++pick) {
                float best = -CUDART_INF_F;
                int at = groups;
                for (int g = lane; g < groups; g += 32)
                    if (group_kept[g] == 0.f && (at == groups || group_score[g] > best)) { best = group_score[g]; at = g; }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                    if (oa < groups && (at >= groups || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
                }
                if (at < groups && lane == 0) group_kept[at] = 1.f;
                __syncwarp();
            }
            for (int e = lane; e < experts; e += 32)
                if (group_kept[e / size] == 0.f) s[e] = -CUDART_INF_F;
            __syncwarp();
        }
    }
    float chosen_sum = 0.f;
    for (int c = 0; c < top; ++c) {
        float best = -CUDART_INF_F;
        int at = experts;
        for (int e = lane; e < experts; e += 32)
            if (s[e] > best) { best = s[e]; at = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= experts) at = 0;                // nothing left to rank (logits that are not numbers): a weight of zero
        if (lane == 0) {
            const float share = over_chosen ? expf(best - m) : best;      // m is the largest logit, the first one chosen
            chosen[(size_t)t * top + c] = at;
            if (corrected) weights[(size_t)t * top + c] = share_of[at] * scale;
            else weights[(size_t)t * top + c] = over_chosen ? share : share / sum * scale;
            chosen_sum += share;
            s[at] = -CUDART_INF_F;
        }
        __syncwarp();
    }
    if (over_chosen && lane == 0) {
        const float inv = scale / chosen_sum;
        for (int c = 0; c < top; ++c) weights[(size_t)t * top + c] *= inv;
    }
}

extern "C" int fe_route_top(const float* logits, int* chosen, float* weights, int T, int experts, int top, float scale,
                            int over_chosen, const float* correction, int groups, int keep, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && experts >= 1 && experts <= ROUTE_MAX_EXPERTS && top >= 1 && top <= experts,
               "route_top: bad sizes (experts %d, top %d; at most %d experts)", experts, top, ROUTE_MAX_EXPERTS);
    FE_REQUIRE(groups >= 1 && experts % groups == 0 && keep >= 1 && keep <= groups && top <= keep * (experts / groups),
               "route_top: %d groups of which %d are kept do not fit %d experts with %d chosen", groups, keep, experts, top);
    FE_REQUIRE(!over_chosen || (correction == nullptr && groups == 1), "route_top: a correction and groups rank shares of the softmax over all experts");
    if (T == 0) return 0;
    const int warps = 4;
    fe::launch(route_top_kernel, (T + warps - 1) / warps, warps * 32, (size_t)warps * (2 * experts + 2 * groups) * sizeof(float), stream,
               logits, chosen, weights, T, experts, top, scale, over_chosen, correction, groups, keep);
    return fe_check_launch("route_top");
}

// One block.  pairs = T * top.  Outputs: offsets[experts + 1] (rows of expert e are offsets[e] .. offsets[e+1]),
// row_of_pair[pairs], pair_of_row[pairs], and the tiles of ``tile_rows`` rows: tile_expert[], tile_row0[], with
// tiles[0] = how many there are.  A choice in [experts, experts + identity) stands for an expert that returns its input: it
// gets no row (row_of_pair = -2) and the combination adds the token's own row for it.
__global__ void route_plan_kernel(const int* __restrict__ chosen, int pairs, int experts, int identity, int tile_rows, int* __restrict__ offsets,
                                  int* __restrict__ row_of_pair, int* __restrict__ pair_of_row, int* __restrict__ tiles,
                                  int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    __shared__ int count[ROUTE_MAX_EXPERTS];
    __shared__ int cursor[ROUTE_MAX_EXPERTS];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
        else if ((e < 0 || e >= experts + identity) && status) atomicOr(status, FE_STATUS_BAD_SLOT);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, n = 0;
        for (int e = 0; e < experts; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            for (int r0 = 0; r0 < count[e]; r0 += tile_rows) {
                tile_expert[n] = e;
                tile_row0[n] = at + r0;
                ++n;
            }
            at += count[e];
        }
        offsets[experts] = at;
        tiles[0] = n;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e < 0 || e >= experts) { row_of_pair[p] = (e >= experts && e < experts + identity) ? -2 : -1; continue; }
        const int row = atomicAdd(&cursor[e], 1);
        row_of_pair[p] = row;
        pair_of_row[row] = p;
    }
}

// The two grouped products.  Tile 64 rows x 64 columns, 16 of K a stage, 256 threads with 4 x 4 outputs each; float
// accumulation in ascending k.  MODE 1 (GATED): columns n and n + F of the expert's matrix are taken together and
// silu(gate) * up is written (compute type); MODE 2: an expert without a gate, relu(product)^2 is written (compute type);
// MODE 0: the plain product is written in float.
namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T, int MODE>
__global__ void __launch_bounds__(256)
routed_product_kernel(const T* __restrict__ A, const int* __restrict__ pair_of_row, int top, const T* __restrict__ W,
                      void* __restrict__ out, const int* __restrict__ offsets, const int* __restrict__ tiles,
                      const int* __restrict__ tile_expert, const int* __restrict__ tile_row0, int N, int K, float limit) {
    griddep_wait();
    griddep_launch_dependents();
    constexpr bool GATED = MODE == 1;
    if ((int)blockIdx.y >= tiles[0]) return;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float Us[GATED ? BK : 1][BN + 4];
    __shared__ int source[BM];
    const int e = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y];
    const int rows = min(BM, offsets[e + 1] - row0);
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int n0 = blockIdx.x * BN;
    // which row of A a sorted row reads: the token of its pair (first product), or the sorted row itself (second)
    if (tid < BM) source[tid] = tid < rows ? (pair_of_row ? pair_of_row[row0 + tid] / top : row0 + tid) : -1;
    __syncthreads();
    const T* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
    float acc[TM][TN], acu[GATED ? TM : 1][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = 0.f;
            if (GATED) acu[i][j] = 0.f;
        }
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < (BM * BK) / 256; ++i) {
            const int idx = tid + i * 256;
            const int r = idx / BK, c = idx % BK;
            const int gk = k0 + c, gn = n0 + r;
            const int src = source[r];
            As[c][r] = (src >= 0 && gk < K) ? to_float(A[(size_t)src * K + gk]) : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? to_float(We[(size_t)gn * K + gk]) : 0.f;
            if (GATED) Us[c][r] = (gn < N && gk < K) ? to_float(We[(size_t)(N + gn) * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN], u[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) {
                w[j] = Ws[k][tx * TN + j];
                if (GATED) u[j] = Us[k][tx * TN + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                    if (GATED) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = ty * TM + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            const size_t at = (size_t)(row0 + r) * N + gn;
            if (GATED) {
                const float g = acc[i][j];
                reinterpret_cast<T*>(out)[at] = from_float<T>(expert_activation(g, acu[i][j], limit));
            } else if (MODE == 2) {
                reinterpret_cast<T*>(out)[at] = from_float<T>(squared_relu(acc[i][j]));
            } else {
                reinterpret_cast<float*>(out)[at] = acc[i][j];
            }
        }
    }
}

// The same products for a handful of rows (a decode step): bound by reading the experts' matrices once.  A tile is up
// to 8 sorted rows of one expert (4 where the experts have four rows or fewer on average: half the accumulators, so two
// blocks share a multiprocessor and twice the loads are in flight); a block stages them in shared memory and its 8 warps take 4 output columns each,
// one after the other: the lanes walk K in 16-byte pieces of the expert's row (and of the paired "up" row when
// GATED), multiply with all rows, and add up over the warp.
constexpr int FEW_ROWS = 8, FEW_ROWS_SMALL = 4, FEW_WARPS = 8, FEW_COLS = 4;

template <typename T, int MODE, int ROWS>
__global__ void __launch_bounds__(FEW_WARPS * 32)
routed_product_few_kernel(const T* __restrict__ A, const int* __restrict__ pair_of_row, int top, const T* __restrict__ W,
                          void* __restrict__ out, const int* __restrict__ offsets, const int* __restrict__ tiles,
                          const int* __restrict__ tile_expert, const int* __restrict__ tile_row0, int N, int K, float limit) {
    griddep_wait();
    griddep_launch_dependents();
    constexpr bool GATED = MODE == 1;
    if ((int)blockIdx.y >= tiles[0]) return;
    extern __shared__ __align__(16) unsigned char few_smem[];
    T* rows_s = reinterpret_cast<T*>(few_smem);                 // [ROWS][K]
    const int e = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y];
    const int rows = min(ROWS, offsets[e + 1] - row0);
    for (int idx = threadIdx.x; idx < ROWS * K; idx += blockDim.x) {
        const int r = idx / K, k = idx % K;
        T v = from_float<T>(0.f);
        if (r < rows) {
            const int src = pair_of_row ? pair_of_row[row0 + r] / top : row0 + r;
            v = A[(size_t)src * K + k];
        }
        rows_s[idx] = v;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
    constexpr int PIECE = 16 / sizeof(T);                       // elements of a 16-byte piece
    const int nbase = (blockIdx.x * FEW_WARPS + warp) * FEW_COLS;
    if (nbase >= N) return;
    if (K % PIECE == 0) {
        // the warp's columns side by side: every step has one 16-byte load per column (and paired "up" column) in flight
        float acc[FEW_COLS][ROWS], acu[GATED ? FEW_COLS : 1][ROWS];
#pragma unroll
        for (int c = 0; c < FEW_COLS; ++c)
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                acc[c][r] = 0.f;
                if (GATED) acu[c][r] = 0.f;
            }
        for (int k = lane * PIECE; k < K; k += 32 * PIECE) {
            float w[FEW_COLS][8], u[GATED ? FEW_COLS : 1][8];
#pragma unroll
            for (int c = 0; c < FEW_COLS; ++c) {
                const int n = min(nbase + c, N - 1);            // a column beyond the edge repeats the last one and is not written
                const T* wg = We + (size_t)n * K + k;
                const T* wu = We + (size_t)(N + n) * K + k;
                if (sizeof(T) == 2) {
                    load8<T>(wg, w[c]);
                    if (GATED) load8<T>(wu, u[c]);
                } else {
                    const float4 w4 = *reinterpret_cast<const float4*>(wg);
                    w[c][0] = w4.x; w[c][1] = w4.y; w[c][2] = w4.z; w[c][3] = w4.w;
                    if (GATED) {
                        const float4 u4 = *reinterpret_cast<const float4*>(wu);
                        u[c][0] = u4.x; u[c][1] = u4.y; u[c][2] = u4.z; u[c][3] = u4.w;
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (r < rows) {                                  // the same for the whole block
                    float a[8];
                    if (sizeof(T) == 2) {
                        load8<T>(rows_s + r * K + k, a);
                    } else {
                        const float4 a4 = *reinterpret_cast<const float4*>(rows_s + r * K + k);
                        a[0] = a4.x; a[1] = a4.y; a[2] = a4.z; a[3] = a4.w;
                    }
#pragma unroll
                    for (int c = 0; c < FEW_COLS; ++c)
#pragma unroll
                        for (int x = 0; x < PIECE; ++x) {
                            acc[c][r] = fmaf(a[x], w[c][x], acc[c][r]);
                            if (GATED) acu[c][r] = fmaf(a[x], u[c][x], acu[c][r]);
                        }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < FEW_COLS; ++c)
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                if (r >= rows) continue;
                const float g = warp_sum(acc[c][r]);
                const float u = GATED ? warp_sum(acu[c][r]) : 0.f;
                if (lane == 0 && nbase + c < N) {
                    const size_t at = (size_t)(row0 + r) * N + nbase + c;
                    if (GATED) reinterpret_cast<T*>(out)[at] = from_float<T>(expert_activation(g, u, limit));
                    else if (MODE == 2) reinterpret_cast<T*>(out)[at] = from_float<T>(squared_relu(g));
                    else reinterpret_cast<float*>(out)[at] = g;
                }
            }
        return;
    }
    for (int c = 0; c < FEW_COLS; ++c) {
        const int n = nbase + c;
        if (n >= N) break;
        const T* wg = We + (size_t)n * K;
        const T* wu = We + (size_t)(N + n) * K;
        float acc[ROWS], acu[GATED ? ROWS : 1];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            acc[r] = 0.f;
            if (GATED) acu[r] = 0.f;
        }
        for (int k = lane; k < K; k += 32) {
            const float w = to_float(wg[k]);
            const float u = GATED ? to_float(wu[k]) : 0.f;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const float a = to_float(rows_s[r * K + k]);
                acc[r] = fmaf(a, w, acc[r]);
                if (GATED) acu[r] = fmaf(a, u, acu[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float g = warp_sum(acc[r]);
            const float u = GATED ? warp_sum(acu[r]) : 0.f;
            if (lane == 0 && r < rows) {
                const size_t at = (size_t)(row0 + r) * N + n;
                if (GATED) reinterpret_cast<T*>(out)[at] = from_float<T>(expert_activation(g, u, limit));
                else if (MODE == 2) reinterpret_cast<T*>(out)[at] = from_float<T>(squared_relu(g));
                else reinterpret_cast<float*>(out)[at] = g;
            }
        }
    }
}

// The two products on tensor cores (bfloat16, float accumulation; mma.sync through the wmma interface).  Tile 64 rows x
// 64 columns (and the 64 paired "up" columns when GATED), 32 of K a stage, 4 warps with 32 x 32 outputs each.
constexpr int TBM = 64, TBN = 64, TBK = 32, TLD = TBK + 8;

template <int MODE, bool GATED = (MODE == 1)>
__global__ void __launch_bounds__(128)
routed_product_mma_kernel(const bf16* __restrict__ A, const int* __restrict__ pair_of_row, int top, const bf16* __restrict__ W,
                          void* __restrict__ out, const int* __restrict__ offsets, const int* __restrict__ tiles,
                          const int* __restrict__ tile_expert, const int* __restrict__ tile_row0, int N, int K, float limit) {
    using namespace nvcuda;
    griddep_wait();
    griddep_launch_dependents();
    if ((int)blockIdx.y >= tiles[0]) return;
    __shared__ __align__(32) bf16 As[TBM][TLD];
    __shared__ __align__(32) bf16 Ws[TBN][TLD];
    __shared__ __align__(32) bf16 Us[GATED ? TBN : 1][TLD];
    __shared__ __align__(32) float stage[4][GATED ? 2 : 1][16][20];
    __shared__ int source[TBM];
    const int e = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y];
    const int rows = min(TBM, offsets[e + 1] - row0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 1, wn = warp & 1;
    const int n0 = blockIdx.x * TBN;
    if (tid < TBM) source[tid] = tid < rows ? (pair_of_row ? pair_of_row[row0 + tid] / top : row0 + tid) : -1;
    __syncthreads();
    const bf16* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2][2], acu[GATED ? 2 : 1][2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            wmma::fill_fragment(acc[i][j], 0.f);
            if (GATED) wmma::fill_fragment(acu[i][j], 0.f);
        }
    const bool pieces = K % 8 == 0;
    const bf16 zero = __float2bfloat16_rn(0.f);
    for (int k0 = 0; k0 < K; k0 += TBK) {
        // 64 rows x 32 columns = 256 pieces of 8 elements per operand, two a thread
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int piece = tid + i * 128;
            const int r = piece >> 2, c = (piece & 3) * 8;
            const int src = source[r], gn = n0 + r, gk = k0 + c;
            uint4 a = make_uint4(0, 0, 0, 0), w = a, u = a;
            if (pieces && gk < K) {
                if (src >= 0) a = *reinterpret_cast<const uint4*>(A + (size_t)src * K + gk);
                if (gn < N) {
                    w = *reinterpret_cast<const uint4*>(We + (size_t)gn * K + gk);
                    if (GATED) u = *reinterpret_cast<const uint4*>(We + (size_t)(N + gn) * K + gk);
                }
                *reinterpret_cast<uint4*>(&As[r][c]) = a;
                *reinterpret_cast<uint4*>(&Ws[r][c]) = w;
                if (GATED) *reinterpret_cast<uint4*>(&Us[r][c]) = u;
            } else {
                for (int x = 0; x < 8; ++x) {
                    const bool in = gk + x < K;
                    As[r][c + x] = (in && src >= 0) ? A[(size_t)src * K + gk + x] : zero;
                    Ws[r][c + x] = (in && gn < N) ? We[(size_t)gn * K + gk + x] : zero;
                    if (GATED) Us[r][c + x] = (in && gn < N) ? We[(size_t)(N + gn) * K + gk + x] : zero;
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TBK; kk += 16) {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> fa[2];
            wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> fb[2], fu[GATED ? 2 : 1];
#pragma unroll
            for (int i = 0; i < 2; ++i) wmma::load_matrix_sync(fa[i], &As[wm * 32 + i * 16][kk], TLD);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                wmma::load_matrix_sync(fb[j], &Ws[wn * 32 + j * 16][kk], TLD);
                if (GATED) wmma::load_matrix_sync(fu[j], &Us[wn * 32 + j * 16][kk], TLD);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    wmma::mma_sync(acc[i][j], fa[i], fb[j], acc[i][j]);
                    if (GATED) wmma::mma_sync(acu[i][j], fa[i], fu[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            wmma::store_matrix_sync(&stage[warp][0][0][0], acc[i][j], 20, wmma::mem_row_major);
            if (GATED) wmma::store_matrix_sync(&stage[warp][GATED ? 1 : 0][0][0], acu[i][j], 20, wmma::mem_row_major);
            __syncwarp();
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const int el = lane + 32 * s;
                const int rr = el >> 4, cc = el & 15;
                const int r = wm * 32 + i * 16 + rr, gn = n0 + wn * 32 + j * 16 + cc;
                if (r < rows && gn < N) {
                    const size_t at = (size_t)(row0 + r) * N + gn;
                    const float g = stage[warp][0][rr][cc];
                    if (GATED) reinterpret_cast<bf16*>(out)[at] = __float2bfloat16_rn(expert_activation(g, stage[warp][GATED ? 1 : 0][rr][cc], limit));
                    else if (MODE == 2) reinterpret_cast<bf16*>(out)[at] = __float2bfloat16_rn(squared_relu(g));
                    else reinterpret_cast<float*>(out)[at] = g;
                }
            }
            __syncwarp();
        }
}

// The tensor-core products once more for K a multiple of 8 (rows start on 16-byte boundaries): tiles of 128 rows x 64
// columns (and the 64 paired "up" columns), 8 warps of 32 x 32 outputs, and the operands of the next 32 of K on their way
// into the other half of shared memory (cp.async, 16 bytes a copy, zero fill for rows and columns beyond the edge)
// while the tensor cores work on this one.
constexpr int PBM = 128, PBN = 64, PBK = 32, PLD = PBK + 8, PSTAGES = 2;
constexpr int PIPE_STAGE_ELEMS = (PBM + 2 * PBN) * PLD;        // A, W and U of one stage
constexpr int PIPE_SMEM_BYTES = PSTAGES * PIPE_STAGE_ELEMS * 2;

__device__ __forceinline__ void copy16(void* dst, const void* src, bool real) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = real ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

template <int MODE, bool GATED = (MODE == 1)>
__global__ void __launch_bounds__(256)
routed_product_pipe_kernel(const bf16* __restrict__ A, const int* __restrict__ pair_of_row, int top, const bf16* __restrict__ W,
                           void* __restrict__ out, const int* __restrict__ offsets, const int* __restrict__ tiles,
                           const int* __restrict__ tile_expert, const int* __restrict__ tile_row0, int N, int K, float limit) {
    using namespace nvcuda;
    griddep_wait();
    griddep_launch_dependents();
    if ((int)blockIdx.y >= tiles[0]) return;
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    bf16* stages = reinterpret_cast<bf16*>(pipe_smem);
    __shared__ int source[PBM];
    const int e = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y];
    const int rows = min(PBM, offsets[e + 1] - row0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 1, wn = warp & 1;
    const int n0 = blockIdx.x * PBN;
    if (tid < PBM) source[tid] = tid < rows ? (pair_of_row ? pair_of_row[row0 + tid] / top : row0 + tid) : -1;
    __syncthreads();
    const bf16* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2][2], acu[GATED ? 2 : 1][2];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            wmma::fill_fragment(acc[i][j], 0.f);
            if (GATED) wmma::fill_fragment(acu[i][j], 0.f);
        }
    auto load_stage = [&](int stage, int k0) {
        bf16* As = stages + stage * PIPE_STAGE_ELEMS;
        bf16* Ws = As + PBM * PLD;
        bf16* Us = Ws + PBN * PLD;
        // A: 128 rows x 4 pieces = 512 copies, two a thread; W and U: 64 rows x 4 pieces = 256 copies each, one a thread
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int piece = tid + i * 256;
            const int r = piece >> 2, c = (piece & 3) * 8;
            const int src = source[r];
            const bool real = src >= 0 && k0 + c < K;
            copy16(As + r * PLD + c, real ? A + (size_t)src * K + k0 + c : A, real);
        }
        {
            const int r = tid >> 2, c = (tid & 3) * 8;
            const bool real = n0 + r < N && k0 + c < K;
            copy16(Ws + r * PLD + c, real ? We + (size_t)(n0 + r) * K + k0 + c : We, real);
            if (GATED) copy16(Us + r * PLD + c, real ? We + (size_t)(N + n0 + r) * K + k0 + c : We, real);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int steps = (K + PBK - 1) / PBK;
    load_stage(0, 0);
    for (int step = 0; step < steps; ++step) {
        if (step + 1 < steps) {
            load_stage((step + 1) & 1, (step + 1) * PBK);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const bf16* As = stages + (step & 1) * PIPE_STAGE_ELEMS;
        const bf16* Ws = As + PBM * PLD;
        const bf16* Us = Ws + PBN * PLD;
#pragma unroll
        for (int kk = 0; kk < PBK; kk += 16) {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> fa[2];
            wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> fb[2], fu[GATED ? 2 : 1];
#pragma unroll
            for (int i = 0; i < 2; ++i) wmma::load_matrix_sync(fa[i], As + (wm * 32 + i * 16) * PLD + kk, PLD);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                wmma::load_matrix_sync(fb[j], Ws + (wn * 32 + j * 16) * PLD + kk, PLD);
                if (GATED) wmma::load_matrix_sync(fu[j], Us + (wn * 32 + j * 16) * PLD + kk, PLD);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    wmma::mma_sync(acc[i][j], fa[i], fb[j], acc[i][j]);
                    if (GATED) wmma::mma_sync(acu[i][j], fa[i], fu[j], acu[i][j]);
                }
        }
        __syncthreads();                          // this stage is free for the copies of the step after next
    }
    // the accumulators pass through shared memory (the pipeline's, which is idle now), a 16 x 16 piece a warp at a time
    float* mine = reinterpret_cast<float*>(pipe_smem) + warp * 2 * 16 * 20;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            wmma::store_matrix_sync(mine, acc[i][j], 20, wmma::mem_row_major);
            if (GATED) wmma::store_matrix_sync(mine + 16 * 20, acu[i][j], 20, wmma::mem_row_major);
            __syncwarp();
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const int el = lane + 32 * s;
                const int rr = el >> 4, cc = el & 15;
                const int r = wm * 32 + i * 16 + rr, gn = n0 + wn * 32 + j * 16 + cc;
                if (r < rows && gn < N) {
                    const size_t at = (size_t)(row0 + r) * N + gn;
                    const float g = mine[rr * 20 + cc];
                    if (GATED) reinterpret_cast<bf16*>(out)[at] = __float2bfloat16_rn(expert_activation(g, mine[16 * 20 + rr * 20 + cc], limit));
                    else if (MODE == 2) reinterpret_cast<bf16*>(out)[at] = __float2bfloat16_rn(squared_relu(g));
                    else reinterpret_cast<float*>(out)[at] = g;
                }
            }
            __syncwarp();
        }
}

// out[t] = sum_c weights[t][c] * y[row_of_pair[t top + c]] (+ shared[t]); a choice of an expert that returns its input
// (row -2) adds weights[t][c] * h[t]
template <typename T>
__global__ void routed_combine_kernel(const float* __restrict__ y, const int* __restrict__ row_of_pair,
                                      const float* __restrict__ weights, const T* __restrict__ shared, T* __restrict__ out,
                                      int top, int D, const T* __restrict__ h) {
    griddep_wait();
    griddep_launch_dependents();
    const int t = blockIdx.x;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < D; j += gridDim.y * blockDim.x) {
        float total = 0.f;
        for (int c = 0; c < top; ++c) {
            const int row = row_of_pair[(size_t)t * top + c];
            if (row >= 0) total = fmaf(weights[(size_t)t * top + c], y[(size_t)row * D + j], total);
            else if (row == -2 && h) total = fmaf(weights[(size_t)t * top + c], to_float(h[(size_t)t * D + j]), total);
        }
        if (shared) total += to_float(shared[(size_t)t * D + j]);
        out[(size_t)t * D + j] = from_float<T>(total);
    }
}
}  // namespace

extern "C" long long fe_routed_experts_workspace(int T, int top, int experts, int D, int F, int dtype) {
    const long long pairs = (long long)T * top;
    const long long tiles = (pairs + FEW_ROWS_SMALL - 1) / FEW_ROWS_SMALL + experts;      // the most tiles any form of the products makes
    const long long ints = (experts + 1) + 2 * pairs + 1 + 2 * tiles;
    const long long width = dtype == FE_F32 ? 4 : 2;
    return ((ints * 4 + 255) / 256 + (pairs * F * width + 255) / 256 + (pairs * D * 4 + 255) / 256) * 256;
}

// h [T, D]; chosen, weights [T, top]; gate_up [experts, 2F, D]; down [experts, D, F]; shared [T, D] or null; out [T, D].
// limit: 0 for silu(gate) * up, else the clamped activation (see expert_activation).  single 1: the experts have no gate,
// gate_up is [experts, F, D] and an expert is down(relu(up h)^2).  identity: choices in [experts, experts + identity) stand
// for experts that return their input.
extern "C" int fe_routed_experts(const void* h, const int* chosen, const float* weights, const void* gate_up, const void* down,
                                 const void* shared, void* out, void* workspace, long long workspace_bytes, int T, int top,
                                 int experts, int D, int F, int dtype, float limit, int* status, int single, int identity,
                                 cudaStream_t stream) {
    FE_REQUIRE(limit >= 0.f, "routed_experts: the activation's limit is 0 (plain silu) or positive");
    FE_REQUIRE(T >= 0 && top >= 1 && experts >= 1 && experts <= ROUTE_MAX_EXPERTS && D > 0 && F > 0, "routed_experts: bad sizes");
    FE_REQUIRE(dtype == FE_F32 || dtype == FE_BF16, "routed_experts: unknown dtype %d", dtype);
    if (T == 0) return 0;
    FE_REQUIRE(workspace_bytes >= fe_routed_experts_workspace(T, top, experts, D, F, dtype), "routed_experts: workspace too small");
    const long long pairs = (long long)T * top;
    const int max_tiles = (int)((pairs + BM - 1) / BM + experts);
    const long long most_tiles = (pairs + FEW_ROWS_SMALL - 1) / FEW_ROWS_SMALL + experts;
    FE_REQUIRE(max_tiles <= 65535, "routed_experts: too many rows in one step (%lld pairs)", pairs);
    int* offsets = (int*)workspace;
    int* row_of_pair = offsets + experts + 1;
    int* pair_of_row = row_of_pair + pairs;
    int* tiles = pair_of_row + pairs;
    int* tile_expert = tiles + 1;
    int* tile_row0 = tile_expert + most_tiles;
    const long long ints = (experts + 1) + 2 * pairs + 1 + 2 * most_tiles;
    char* act = (char*)workspace + (ints * 4 + 255) / 256 * 256;
    const long long width = dtype == FE_F32 ? 4 : 2;
    float* y = (float*)(act + (pairs * F * width + 255) / 256 * 256);
    const int threads = D >= 1024 ? 256 : 128;
    const long long width_bytes = dtype == FE_F32 ? 4 : 2;
    const int few_rows = pairs <= (long long)FEW_ROWS_SMALL * experts ? FEW_ROWS_SMALL : FEW_ROWS;
    const size_t few_smem1 = (size_t)few_rows * D * width_bytes, few_smem2 = (size_t)few_rows * F * width_bytes;
    const bool few = pairs <= 64 && few_smem1 <= 160 * 1024 && few_smem2 <= 160 * 1024;
    // tensor cores with 128-row tiles and pipelined copies when rows start on 16-byte boundaries in both products
    const bool piped = !few && dtype == FE_BF16 && D % 8 == 0 && F % 8 == 0;
    FE_REQUIRE(identity >= 0 && (single == 0 || single == 1), "routed_experts: bad options");
    fe::launch(route_plan_kernel, 1, 256, 0, stream, chosen, (int)pairs, experts, identity, few ? few_rows : (piped ? PBM : BM), offsets,
               row_of_pair, pair_of_row, tiles, tile_expert, tile_row0, status);
    const int* c_pairs = pair_of_row;
    const int* c_none = nullptr;
    const int *c_offsets = offsets, *c_tiles = tiles, *c_expert = tile_expert, *c_row0 = tile_row0;
#define FE_ROUTED_PRODUCTS(KERNEL1, KERNEL2, TYPE, GRID1, GRID2, THREADS, SMEM1, SMEM2)                                                   \
    fe::launch(KERNEL1, GRID1, THREADS, SMEM1, stream, (const TYPE*)h, c_pairs, top, (const TYPE*)gate_up, (void*)act, c_offsets, c_tiles, \
               c_expert, c_row0, F, D, limit);                                                                                            \
    fe::launch(KERNEL2, GRID2, THREADS, SMEM2, stream, (const TYPE*)act, c_none, top, (const TYPE*)down, (void*)y, c_offsets, c_tiles,    \
               c_expert, c_row0, D, F, 0.f)
    if (few) {
        const int few_tiles = (int)((pairs + few_rows - 1) / few_rows + experts);
        const int per_block = FEW_WARPS * FEW_COLS;
        const dim3 g1((F + per_block - 1) / per_block, few_tiles), g2((D + per_block - 1) / per_block, few_tiles);
#define FE_ROUTED_FEW(TYPE, ROWS)                                                                                                       \
    do {                                                                                                                                \
        cudaError_t err = cudaSuccess;                                                                                                  \
        if (few_smem1 > 48 * 1024)                                                                                                      \
            err = cudaFuncSetAttribute(routed_product_few_kernel<TYPE, 1, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)few_smem1); \
        if (err == cudaSuccess && few_smem2 > 48 * 1024)                                                                                \
            err = cudaFuncSetAttribute(routed_product_few_kernel<TYPE, 0, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)few_smem2); \
        if (err == cudaSuccess && few_smem1 > 48 * 1024)                                                                                \
            err = cudaFuncSetAttribute(routed_product_few_kernel<TYPE, 2, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)few_smem1); \
        FE_REQUIRE(err == cudaSuccess, "routed_experts: %s", cudaGetErrorString(err));                                                  \
        if (single) {                                                                                                                   \
            FE_ROUTED_PRODUCTS((routed_product_few_kernel<TYPE, 2, ROWS>), (routed_product_few_kernel<TYPE, 0, ROWS>), TYPE, g1, g2,    \
                               FEW_WARPS * 32, few_smem1, few_smem2);                                                                   \
        } else {                                                                                                                        \
            FE_ROUTED_PRODUCTS((routed_product_few_kernel<TYPE, 1, ROWS>), (routed_product_few_kernel<TYPE, 0, ROWS>), TYPE, g1, g2,    \
                               FEW_WARPS * 32, few_smem1, few_smem2);                                                                   \
        }                                                                                                                               \
    } while (0)
        if (dtype == FE_F32) {
            if (few_rows == FEW_ROWS_SMALL) FE_ROUTED_FEW(float, FEW_ROWS_SMALL);
            else FE_ROUTED_FEW(float, FEW_ROWS);
        } else {
            if (few_rows == FEW_ROWS_SMALL) FE_ROUTED_FEW(bf16, FEW_ROWS_SMALL);
            else FE_ROUTED_FEW(bf16, FEW_ROWS);
        }
#undef FE_ROUTED_FEW
    } else {
        const dim3 grid1((F + BN - 1) / BN, max_tiles), grid2((D + BN - 1) / BN, max_tiles);
        if (dtype == FE_F32) {
            if (single) { FE_ROUTED_PRODUCTS((routed_product_kernel<float, 2>), (routed_product_kernel<float, 0>), float, grid1, grid2, 256, 0, 0); }
            else { FE_ROUTED_PRODUCTS((routed_product_kernel<float, 1>), (routed_product_kernel<float, 0>), float, grid1, grid2, 256, 0, 0); }
        } else if (piped) {
            cudaError_t err = cudaFuncSetAttribute(routed_product_pipe_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PIPE_SMEM_BYTES);
            if (err == cudaSuccess) err = cudaFuncSetAttribute(routed_product_pipe_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, PIPE_SMEM_BYTES);
            if (err == cudaSuccess) err = cudaFuncSetAttribute(routed_product_pipe_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PIPE_SMEM_BYTES);
            FE_REQUIRE(err == cudaSuccess, "routed_experts: %s", cudaGetErrorString(err));
            const dim3 p1((F + PBN - 1) / PBN, max_tiles), p2((D + PBN - 1) / PBN, max_tiles);
            if (single) { FE_ROUTED_PRODUCTS((routed_product_pipe_kernel<2>), (routed_product_pipe_kernel<0>), bf16, p1, p2, 256, PIPE_SMEM_BYTES, PIPE_SMEM_BYTES); }
            else { FE_ROUTED_PRODUCTS((routed_product_pipe_kernel<1>), (routed_product_pipe_kernel<0>), bf16, p1, p2, 256, PIPE_SMEM_BYTES, PIPE_SMEM_BYTES); }
        } else {
            if (single) { FE_ROUTED_PRODUCTS((routed_product_mma_kernel<2>), (routed_product_mma_kernel<0>), bf16, grid1, grid2, 128, 0, 0); }
            else { FE_ROUTED_PRODUCTS((routed_product_mma_kernel<1>), (routed_product_mma_kernel<0>), bf16, grid1, grid2, 128, 0, 0); }
        }
    }
#undef FE_ROUTED_PRODUCTS
    const int stretches = T >= 512 ? 1 : (D + threads - 1) / threads;          // few tokens: one column a thread
    const dim3 combine(T, stretches < 65535 ? stretches : 65535);
    if (dtype == FE_F32)
        fe::launch(routed_combine_kernel<float>, combine, threads, 0, stream, (const float*)y, (const int*)row_of_pair, weights,
                   (const float*)shared, (float*)out, top, D, identity ? (const float*)h : (const float*)nullptr);
    else
        fe::launch(routed_combine_kernel<bf16>, combine, threads, 0, stream, (const float*)y, (const int*)row_of_pair, weights,
                   (const bf16*)shared, (bf16*)out, top, D, identity ? (const bf16*)h : (const bf16*)nullptr);
    return fe_check_launch("routed_experts");
}

// ---------------------------------------------------------------------------------------------
// The pieces on their own, for a caller that takes the two products elsewhere (the grouped tcgen05 GEMM of the
// bfloat16 library): the plan, the rows of h gathered into sorted order, and the combination.
extern "C" int fe_routed_plan(const int* chosen, int pairs, int experts, int tile_rows, int* offsets, int* row_of_pair,
                              int* pair_of_row, int* tiles, int* tile_expert, int* tile_row0, int* status, int identity, cudaStream_t stream) {
    FE_REQUIRE(pairs >= 1 && experts >= 1 && experts <= ROUTE_MAX_EXPERTS && tile_rows >= 1 && identity >= 0, "routed_plan: bad sizes");
    fe::launch(route_plan_kernel, 1, 256, 0, stream, chosen, pairs, experts, identity, tile_rows, offsets, row_of_pair, pair_of_row, tiles,
               tile_expert, tile_row0, status);
    return fe_check_launch("routed_plan");
}

namespace {
// sorted[row] = h[pair_of_row[row] / top]: 16 bytes a thread and step (bytes_per_row is a multiple of 16)
__global__ void routed_gather_kernel(const uint4* __restrict__ h, const int* __restrict__ pair_of_row, int top,
                                     uint4* __restrict__ sorted, int pieces, const int* __restrict__ sorted_rows) {
    griddep_wait();
    griddep_launch_dependents();
    const int row = blockIdx.x;
    if (sorted_rows && row >= *sorted_rows) return;          // pairs that have no row (experts that return their input)
    const int src = pair_of_row[row] / top;
    for (int p = threadIdx.x; p < pieces; p += blockDim.x) sorted[(size_t)row * pieces + p] = h[(size_t)src * pieces + p];
}
}  // namespace

// sorted_rows (may be null): where the number of sorted rows lies on the device, when it can be fewer than ``pairs``
extern "C" int fe_routed_gather(const void* h, const int* pair_of_row, int top, void* sorted, int pairs, long long bytes_per_row,
                                const int* sorted_rows,
                                cudaStream_t stream) {
    FE_REQUIRE(pairs >= 1 && top >= 1 && bytes_per_row > 0 && bytes_per_row % 16 == 0 && ((((size_t)h) | ((size_t)sorted)) & 15) == 0,
               "routed_gather: rows must be multiples of 16 bytes on 16-byte boundaries");
    fe::launch(routed_gather_kernel, pairs, 128, 0, stream, (const uint4*)h, pair_of_row, top, (uint4*)sorted, (int)(bytes_per_row / 16), sorted_rows);
    return fe_check_launch("routed_gather");
}

extern "C" int fe_routed_combine(const float* y, const int* row_of_pair, const float* weights, const void* shared, void* out, int T,
                                 int top, int D, int dtype, const void* identity_rows, cudaStream_t stream) {
    FE_REQUIRE(T >= 1 && top >= 1 && D >= 1, "routed_combine: bad sizes");
    const int threads = D >= 1024 ? 256 : 128;
    const int stretches = T >= 512 ? 1 : (D + threads - 1) / threads;
    const dim3 grid(T, stretches < 65535 ? stretches : 65535);
    if (dtype == FE_F32)
        fe::launch(routed_combine_kernel<float>, grid, threads, 0, stream, y, row_of_pair, weights, (const float*)shared, (float*)out, top, D,
                   (const float*)identity_rows);
    else if (dtype == FE_BF16)
        fe::launch(routed_combine_kernel<bf16>, grid, threads, 0, stream, y, row_of_pair, weights, (const bf16*)shared, (bf16*)out, top, D,
                   (const bf16*)identity_rows);
    else
        FE_REQUIRE(false, "routed_combine: unknown dtype %d", dtype);
    return fe_check_launch("routed_combine");
}
