// Attention over a cached latent: what a step does around the paged attention kernel.
//
// Per token the cache keeps one row [latent (rank) | rotated key part (rot_dim) | zeros up to ``row``]; the queries go
// to the attention kernel as rows of the same layout per head: [query in latent space | rotated query part | zeros].
// The kernel below assembles both: it norms the latent (float RMS norm with a weight), rotates the key part and the
// heads' query parts (interleaved pairs (2i, 2i+1) of the first rot_dims entries by position * inv_freq[i], float
// sine and cosine), writes the token's row into its cache slot and the query rows into one tensor.
//
// Also here: the batched float product that maps the heads' queries into the latent space and the attention's output
// out of it, one small matrix per head, with arbitrary row and batch strides on both sides.
#define FE_PDL_CLASS 4      // FE_PDL_ELEMENTWISE
#include "common.cuh"

using namespace fe;

// grid: one block per token.
//   q        [T, heads, dim + rot_dim]   the query projection (compute type)
//   q_latent [heads, T, rank]            the plain query parts times W_uk per head (compute type)
//   down     [T, rank + rot_dim]         the latent's projection, float
//   cache    [pages, 1, page_size, row]  slot = page * page_size + offset; a negative slot writes nothing
//   queries  [T, heads, row]
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ q, const T* __restrict__ q_latent, const float* __restrict__ down,
                                      const float* __restrict__ norm_weight, float eps, const int* __restrict__ positions,
                                      const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ slot_mapping,
                                      T* __restrict__ cache, long long num_slots, T* __restrict__ queries, int T_tokens,
                                      int heads, int dim, int rot_dim, int rank, int row, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float trig[];             // cos [rot_dims / 2], sin [rot_dims / 2]
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int half = rot_dims / 2;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        trig[i] = c;
        trig[half + i] = s;
    }
    // ``down`` null: a layer that reads the rows another layer cached; only the queries are made
    const float* dr = down ? down + (size_t)t * (rank + rot_dim) : nullptr;
    float ss = 0.f;
    if (dr)
        for (int j = threadIdx.x; j < rank; j += blockDim.x) ss += dr[j] * dr[j];
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)rank + eps);      // also orders the writes of trig

    T* dst = nullptr;
    if (slot_mapping && dr) {
        const long long slot = slot_mapping[t];
        if (slot >= num_slots) {
            if (threadIdx.x == 0 && status) atomicOr(status, FE_STATUS_BAD_SLOT);
        } else if (slot >= 0) {
            dst = cache + (size_t)slot * row;
        }
    }
    if (dst) {
        for (int j = threadIdx.x; j < row; j += blockDim.x) {
            float v = 0.f;
            if (j < rank) {
                v = dr[j] * inv * norm_weight[j];
            } else if (j < rank + rot_dim) {
                const int e = j - rank;
                v = dr[j];
                if (e < rot_dims) {
                    const int i = e >> 1;
                    const float other = dr[rank + (e ^ 1)];
                    v = (e & 1) ? fmaf(v, trig[i], other * trig[half + i]) : fmaf(v, trig[i], -other * trig[half + i]);
                }
            }
            dst[j] = from_float<T>(v);
        }
    }
    const int qw = dim + rot_dim;
    for (int e = threadIdx.x; e < heads * row; e += blockDim.x) {
        const int h = e / row, j = e % row;
        float v = 0.f;
        if (j < rank) {
            v = to_float(q_latent[((size_t)h * T_tokens + t) * rank + j]);
        } else if (j < rank + rot_dim) {
            const int c = j - rank;
            const T* qr = q + ((size_t)t * heads + h) * qw + dim;
            v = to_float(qr[c]);
            if (c < rot_dims) {
                const int i = c >> 1;
                const float other = to_float(qr[c ^ 1]);
                v = (c & 1) ? fmaf(v, trig[i], other * trig[half + i]) : fmaf(v, trig[i], -other * trig[half + i]);
            }
        }
        queries[((size_t)t * heads + h) * row + j] = from_float<T>(v);
    }
}

extern "C" int fe_latent_prepare(const void* q, const void* q_latent, const float* down, const float* norm_weight, float eps,
                                 const int* positions, const float* inv_freq, int rot_dims, const int* slot_mapping, void* cache,
                                 long long num_slots, void* queries, int T, int heads, int dim, int rot_dim, int rank, int row,
                                 int dtype, int* status, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && heads > 0 && dim > 0 && rot_dim >= 0 && rank > 0 && row >= rank + rot_dim && rot_dims >= 0 &&
                   rot_dims <= rot_dim && rot_dims % 2 == 0,
               "latent_prepare: bad sizes");
    if (T == 0) return 0;
    const size_t smem = (size_t)(rot_dims > 0 ? rot_dims : 2) * sizeof(float);
    if (dtype == FE_F32)
        fe::launch(latent_prepare_kernel<float>, T, 256, smem, stream, (const float*)q, (const float*)q_latent, down, norm_weight, eps,
                   positions, inv_freq, rot_dims, slot_mapping, (float*)cache, num_slots, (float*)queries, T, heads, dim, rot_dim,
                   rank, row, status);
    else if (dtype == FE_BF16)
        fe::launch(latent_prepare_kernel<bf16>, T, 256, smem, stream, (const bf16*)q, (const bf16*)q_latent, down, norm_weight, eps,
                   positions, inv_freq, rot_dims, slot_mapping, (bf16*)cache, num_slots, (bf16*)queries, T, heads, dim, rot_dim,
                   rank, row, status);
    else
        FE_REQUIRE(false, "latent_prepare: unknown dtype %d", dtype);
    return fe_check_launch("latent_prepare");
}

// ---------------------------------------------------------------------------------------------
// C[b][M, N] = A[b][M, K] . W[b][N, K]^T in true float on CUDA cores, b = 0 .. batch - 1.  Row strides lda, ldw, ldc and
// batch strides sa, sw, sc in elements.  Every output is one chain of fused multiply-adds over ascending k, so a row's
// result does not depend on which other rows are in the step.
namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
gemm_fp32_batched_kernel(const float* __restrict__ A, long long lda, long long sa, const float* __restrict__ W, long long ldw,
                         long long sw, float* __restrict__ C, long long ldc, long long sc, int M, int N, int K) {
    griddep_wait();
    griddep_launch_dependents();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    A += (size_t)blockIdx.z * sa;
    W += (size_t)blockIdx.z * sw;
    C += (size_t)blockIdx.z * sc;
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < (BM * BK) / 256; ++i) {
            const int idx = tid + i * 256;
            const int r = idx / BK, c = idx % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
            Ws[c][r] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
        }
    }
}
}  // namespace

extern "C" int fe_gemm_fp32_batched(const float* A, long long lda, long long sa, const float* W, long long ldw, long long sw,
                                    float* C, long long ldc, long long sc, int M, int N, int K, int batch, cudaStream_t stream) {
    FE_REQUIRE(M >= 0 && N > 0 && K > 0 && batch >= 0 && batch <= 65535, "gemm_fp32_batched: bad sizes M=%d N=%d K=%d batch=%d", M, N, K, batch);
    if (M == 0 || batch == 0) return 0;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
    FE_REQUIRE(grid.y <= 65535, "gemm_fp32_batched: too many rows (%d)", M);
    fe::launch(gemm_fp32_batched_kernel, grid, 256, 0, stream, A, lda, sa, W, ldw, sw, C, ldc, sc, M, N, K);
    return fe_check_launch("gemm_fp32_batched");
}
