// Operations on the residual stream that layers of several designs share:
//   a token embedding with a second, hashed table of (previous token, token) pairs added,
//   RMSNorm in groups fused with the residual add,
//   a learned average over the streams of all layers so far ("depth average"),
//   elementwise activations (tanh, xIELU).
// All arithmetic is float; the stream itself is float.
#define FE_PDL_CLASS 4      // FE_PDL_ELEMENTWISE
#include "common.cuh"

using namespace fe;

// ---------------------------------------------------------------------------------------------
// out[t] = table[id_t] + pairs[row_t], row_t = (previous token * mul_prev + id_t * mul_cur) mod buckets, and row
// ``buckets`` for a sequence's first token (position 0).  The token before a portion's first token is the seat's
// entry of ``previous`` (what the step before left there); the block of a request's first row reads it and then
// writes the request's last token of this step in its place, so no other block touches that entry.
// One block per token.
template <typename T>
__global__ void embedding_hashed_pairs_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                              const T* __restrict__ pairs, int* previous, const int* __restrict__ seats,
                                              const int* __restrict__ cu_q, const int* __restrict__ q_start,
                                              const int* __restrict__ token_req, float* __restrict__ out, int D, int V,
                                              int buckets, long long mul_prev, long long mul_cur, int n_seats,
                                              int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    const int t = blockIdx.x;
    const int r = token_req[t];
    const int first = cu_q[r];
    const int pos = q_start[r] + (t - first);
    const int seat = seats[r];
    const bool seated = seat >= 0 && seat < n_seats;
    const int id = ids[t];
    int before = 0;
    if (t > first) before = ids[t - 1];
    else if (pos > 0 && seated) before = previous[seat];
    float* o = out + (size_t)t * D;
    if (id < 0 || id >= V || before < 0 || before >= V) {
        if (threadIdx.x == 0 && status) atomicOr(status, FE_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < D; j += blockDim.x) o[j] = 0.f;
    } else {
        const long long row = pos == 0 ? (long long)buckets : ((long long)before * mul_prev + (long long)id * mul_cur) % buckets;
        const T* a = table + (size_t)id * D;
        const T* b = pairs + (size_t)row * D;
        for (int j = threadIdx.x; j < D; j += blockDim.x) o[j] = to_float(a[j]) + to_float(b[j]);
    }
    if (t == first && seated) {
        __syncthreads();                                   // every thread has read the entry
        if (threadIdx.x == 0) previous[seat] = ids[cu_q[r + 1] - 1];
    }
}

extern "C" int fe_embedding_hashed_pairs(const int* ids, const void* table, const void* pairs, int* previous, const int* seats,
                                         const int* cu_q, const int* q_start, const int* token_req, float* out, int T, int D,
                                         int V, int buckets, long long mul_prev, long long mul_cur, int n_seats, int dtype,
                                         int* status, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && D > 0 && V > 0 && buckets > 0 && n_seats >= 0, "embedding_hashed_pairs: bad sizes");
    if (T == 0) return 0;
    const int threads = D >= 1024 ? 256 : 128;
    if (dtype == FE_F32)
        fe::launch(embedding_hashed_pairs_kernel<float>, T, threads, 0, stream, ids, (const float*)table, (const float*)pairs,
                   previous, seats, cu_q, q_start, token_req, out, D, V, buckets, mul_prev, mul_cur, n_seats, status);
    else if (dtype == FE_BF16)
        fe::launch(embedding_hashed_pairs_kernel<bf16>, T, threads, 0, stream, ids, (const bf16*)table, (const bf16*)pairs,
                   previous, seats, cu_q, q_start, token_req, out, D, V, buckets, mul_prev, mul_cur, n_seats, status);
    else
        FE_REQUIRE(false, "embedding_hashed_pairs: unknown dtype %d", dtype);
    return fe_check_launch("embedding_hashed_pairs");
}

// ---------------------------------------------------------------------------------------------
// Residual add + RMSNorm in ``groups`` equal consecutive parts of the row, each with its own 1/sqrt(mean(part^2) + eps);
// the whole row is then multiplied by the weight.  rows == nullptr: residual += delta in place, every row normalised;
// rows given: only those rows are read and nothing is written back.  One block per output row; the row is staged in
// shared memory.
constexpr int MAX_NORM_GROUPS = 64;

template <typename T>
__global__ void add_group_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                         const float* __restrict__ weight, float eps, T* __restrict__ out,
                                         const int* __restrict__ rows, int H, int groups, int n_rows_total) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float row[];
    __shared__ float scratch[33];
    __shared__ float inverse[MAX_NORM_GROUPS];
    const int i = blockIdx.x;
    int r = rows ? rows[i] : i;
    if (r < 0 || r >= n_rows_total) r = 0;          // guarded: rows are checked on the host
    float* res = residual + (size_t)r * H;
    const T* del = delta ? delta + (size_t)r * H : nullptr;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = res[j];
        if (del) {
            v += to_float(del[j]);
            if (!rows) res[j] = v;
        }
        row[j] = v;
    }
    __syncthreads();
    const int part = H / groups;
    for (int g = 0; g < groups; ++g) {
        float ss = 0.f;
        for (int j = threadIdx.x; j < part; j += blockDim.x) {
            const float v = row[g * part + j];
            ss += v * v;
        }
        const float total = block_sum(ss, scratch);
        if (threadIdx.x == 0) inverse[g] = rsqrtf(total / (float)part + eps);
    }
    __syncthreads();
    T* o = out + (size_t)i * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = from_float<T>(row[j] * inverse[j / part] * weight[j]);
}

extern "C" int fe_add_group_rmsnorm(float* residual, const void* delta, const float* weight, float eps, void* out,
                                    const int* rows, int n_out, int H, int groups, int n_rows_total, int dtype,
                                    cudaStream_t stream) {
    FE_REQUIRE(n_out >= 0 && H > 0 && groups >= 1 && groups <= MAX_NORM_GROUPS && H % groups == 0,
               "add_group_rmsnorm: bad sizes n=%d H=%d groups=%d (at most %d groups, which divide H)", n_out, H, groups, MAX_NORM_GROUPS);
    if (n_out == 0) return 0;
    const size_t smem = (size_t)H * sizeof(float);
    FE_REQUIRE(smem <= 200 * 1024, "add_group_rmsnorm: hidden size %d needs %zu bytes of shared memory (limit 204800)", H, smem);
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    cudaError_t err = cudaSuccess;
    if (dtype == FE_F32) {
        if (smem > 48 * 1024) err = cudaFuncSetAttribute(add_group_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        FE_REQUIRE(err == cudaSuccess, "add_group_rmsnorm: %s", cudaGetErrorString(err));
        fe::launch(add_group_rmsnorm_kernel<float>, n_out, threads, smem, stream, residual, (const float*)delta, weight, eps,
                   (float*)out, rows, H, groups, n_rows_total);
    } else if (dtype == FE_BF16) {
        if (smem > 48 * 1024) err = cudaFuncSetAttribute(add_group_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        FE_REQUIRE(err == cudaSuccess, "add_group_rmsnorm: %s", cudaGetErrorString(err));
        fe::launch(add_group_rmsnorm_kernel<bf16>, n_out, threads, smem, stream, residual, (const bf16*)delta, weight, eps,
                   (bf16*)out, rows, H, groups, n_rows_total);
    } else {
        FE_REQUIRE(false, "add_group_rmsnorm: unknown dtype %d", dtype);
    }
    return fe_check_launch("add_group_rmsnorm");
}

// ---------------------------------------------------------------------------------------------
// The end of a layer whose branches run side by side, with an average over depth:
//   X_new = x + (a + b)              (a, b: the branches' outputs; b may be absent)
//   history[depth + 1] = X_new       (history[0] = x first when depth == 0: the embedding's output)
//   x <- sum_{j = 0 .. depth + 1} alpha[j] * history[j]
// history is [layers + 1][n] float, n = tokens * width.
template <typename T>
__global__ void depth_average_kernel(float* __restrict__ history, float* __restrict__ x, const T* __restrict__ a,
                                     const T* __restrict__ b, const float* __restrict__ alpha, int depth, long long n) {
    griddep_wait();
    griddep_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float xv = x[i];
    float delta = to_float(a[i]);
    if (b) delta += to_float(b[i]);
    const float fresh = xv + delta;
    float total;
    if (depth == 0) {
        history[i] = xv;
        total = alpha[0] * xv;
    } else {
        total = alpha[0] * history[i];
        for (int j = 1; j <= depth; ++j) total += alpha[j] * history[(long long)j * n + i];
    }
    history[(long long)(depth + 1) * n + i] = fresh;
    x[i] = total + alpha[depth + 1] * fresh;
}

extern "C" int fe_depth_average(float* history, float* x, const void* a, const void* b, const float* alpha, int depth,
                                long long n, int dtype, cudaStream_t stream) {
    FE_REQUIRE(depth >= 0 && n >= 0 && a != nullptr, "depth_average: bad arguments");
    if (n == 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (dtype == FE_F32)
        fe::launch(depth_average_kernel<float>, blocks, threads, 0, stream, history, x, (const float*)a, (const float*)b, alpha, depth, n);
    else if (dtype == FE_BF16)
        fe::launch(depth_average_kernel<bf16>, blocks, threads, 0, stream, history, x, (const bf16*)a, (const bf16*)b, alpha, depth, n);
    else
        FE_REQUIRE(false, "depth_average: unknown dtype %d", dtype);
    return fe_check_launch("depth_average");
}

// ---------------------------------------------------------------------------------------------
// Elementwise activations.  kind 0: tanh.  kind 1: xIELU with the two numbers params = (p, q) on the device:
//   z > 0: softplus(p) z^2 + z/2;    z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2.
// kind 2: the square of relu(z).
__device__ __forceinline__ float softplusf(float v) { return log1pf(expf(v)); }

template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, int kind,
                                  const float* __restrict__ params) {
    griddep_wait();
    griddep_launch_dependents();
    float up = 0.f, down = 0.f;
    if (kind == 1) {
        up = softplusf(params[0]);
        down = 0.5f + softplusf(params[1]);
    }
    const long long stride = (long long)gridDim.x * blockDim.x, first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (n % 8 == 0 && ((((size_t)x) | ((size_t)out)) & 31) == 0) {           // eight elements a thread and step
        for (long long i = first * 8; i < n; i += stride * 8) {
            float z[8];
            load8<T>(x + i, z);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (kind == 0) z[e] = tanhf(z[e]);
                else if (kind == 2) z[e] = z[e] > 0.f ? z[e] * z[e] : 0.f;
                else z[e] = z[e] > 0.f ? fmaf(up * z[e], z[e], 0.5f * z[e]) : fmaf(down, expm1f(z[e]) - z[e], 0.5f * z[e]);
            }
            store8<T>(out + i, z);
        }
        return;
    }
    for (long long i = first; i < n; i += stride) {
        const float z = to_float(x[i]);
        float y;
        if (kind == 0) y = tanhf(z);
        else if (kind == 2) y = z > 0.f ? z * z : 0.f;
        else y = z > 0.f ? fmaf(up * z, z, 0.5f * z) : fmaf(down, expm1f(z) - z, 0.5f * z);
        out[i] = from_float<T>(y);
    }
}

extern "C" int fe_activation(const void* x, void* out, long long n, int kind, const float* params, int dtype,
                             cudaStream_t stream) {
    FE_REQUIRE(n >= 0 && (kind == 0 || kind == 2 || (kind == 1 && params != nullptr)), "activation: bad arguments (kind %d)", kind);
    if (n == 0) return 0;
    const int threads = 256;
    const long long want = (n / 8 + threads) / threads;
    const long long most = (long long)fe_sm_count() * 16;
    const unsigned blocks = (unsigned)(want < most ? (want > 0 ? want : 1) : most);
    if (dtype == FE_F32)
        fe::launch(activation_kernel<float>, blocks, threads, 0, stream, (const float*)x, (float*)out, n, kind, params);
    else if (dtype == FE_BF16)
        fe::launch(activation_kernel<bf16>, blocks, threads, 0, stream, (const bf16*)x, (bf16*)out, n, kind, params);
    else
        FE_REQUIRE(false, "activation: unknown dtype %d", dtype);
    return fe_check_launch("activation");
}
