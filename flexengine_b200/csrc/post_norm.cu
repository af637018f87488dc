// Kernels of a layer whose sublayers have a norm on both sides, x <- x + N_b(sublayer(N_a(x))):
//   post norm + residual add + next norm   y' = w_b (y + bias) / rms(y + bias);  x += y';  out = w x / rms(x)   (one pass)
//   the same without a next norm           out = [x | extra] in the compute type: the rows a product reads that re-enters
//                                          the stream from the stream and the embedding's output
//   logits                                 z <- cap tanh(z scale / cap)
//   gated activation with biases           act(gate + b_g) * (up + b_u) from a float product
// All arithmetic is float.  The residual stream is float; a branch output comes in float or in the compute type.
#define FE_PDL_CLASS 4
#include "common.cuh"

using namespace fe;

namespace {

template <typename T> __device__ __forceinline__ void load4(const T* p, float* v);
template <> __device__ __forceinline__ void load4<float>(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}
template <> __device__ __forceinline__ void load4<bf16>(const bf16* p, float* v) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
    v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float* v);
template <> __device__ __forceinline__ void store4<float>(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, const float* v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&a);
    raw.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

}  // namespace

// One block per output row; the row is staged in shared memory (H floats).  V = 4: H is a multiple of 4 and every row
// starts on a 16-byte boundary (8 for the compute type's rows), four columns a thread and load; V = 1: any H.
//   delta  (may be null)  the branch output [T, H], TD float or the compute type; bias (may be null) is added to it
//   post_w (may be null)  the branch's own norm: delta <- post_w delta / sqrt(mean(delta^2) + post_eps)
//   rows   (may be null)  only these rows are read and nothing is written back to the stream
//   w      (may be null)  the next norm's weight; null: out receives the stream's rows as they are
//   extra  (may be null)  float [T, extra_cols], copied behind the H columns of out (ldo >= H + extra_cols)
template <typename T, typename TD, int V>
__global__ void post_norm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, const float* __restrict__ bias,
                                 const float* __restrict__ post_w, float post_eps, const float* __restrict__ w, float eps,
                                 T* __restrict__ out, long long ldo, const int* __restrict__ rows, int H,
                                 const float* __restrict__ extra, int extra_cols, int T_tokens) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[33];
    const int b = blockIdx.x;
    const int r = rows ? rows[b] : b;
    if (r < 0 || r >= T_tokens) return;
    float* x = residual + (size_t)r * H;
    const float inv_h = 1.f / (float)H;
    float ss = 0.f;
    if (delta) {
        const TD* y = delta + (size_t)r * H;
        for (int j = threadIdx.x * V; j < H; j += blockDim.x * V) {
            float v[V];
            if (V == 4) load4<TD>(y + j, v);
            else v[0] = to_float(y[j]);
#pragma unroll
            for (int e = 0; e < V; ++e) {
                if (bias) v[e] += bias[j + e];
                ss = fmaf(v[e], v[e], ss);
                row[j + e] = v[e];
            }
        }
        float inv = 1.f;
        if (post_w) inv = rsqrtf(block_sum(ss, scratch) * inv_h + post_eps);
        ss = 0.f;
        for (int j = threadIdx.x * V; j < H; j += blockDim.x * V) {
            float v[V];
            if (V == 4) load4<float>(x + j, v);
            else v[0] = x[j];
#pragma unroll
            for (int e = 0; e < V; ++e) {
                v[e] = post_w ? fmaf(row[j + e] * inv, post_w[j + e], v[e]) : v[e] + row[j + e];
                ss = fmaf(v[e], v[e], ss);
                row[j + e] = v[e];
            }
            if (!rows) {
                if (V == 4) store4<float>(x + j, v);
                else x[j] = v[0];
            }
        }
    } else {
        for (int j = threadIdx.x * V; j < H; j += blockDim.x * V) {
            float v[V];
            if (V == 4) load4<float>(x + j, v);
            else v[0] = x[j];
#pragma unroll
            for (int e = 0; e < V; ++e) {
                ss = fmaf(v[e], v[e], ss);
                row[j + e] = v[e];
            }
        }
    }
    float inv = 1.f;
    if (w) inv = rsqrtf(block_sum(ss, scratch) * inv_h + eps);
    T* o = out + (size_t)b * ldo;
    for (int j = threadIdx.x * V; j < H; j += blockDim.x * V) {
        float v[V];
#pragma unroll
        for (int e = 0; e < V; ++e) v[e] = w ? row[j + e] * inv * w[j + e] : row[j + e];
        if (V == 4) store4<T>(o + j, v);
        else o[j] = from_float<T>(v[0]);
    }
    if (extra) {
        const float* src = extra + (size_t)r * extra_cols;
        for (int j = threadIdx.x; j < extra_cols; j += blockDim.x) o[H + j] = from_float<T>(src[j]);
    }
}

template <typename T, typename TD>
static int launch_post_norm(float* residual, const void* delta, const float* bias, const float* post_w, float post_eps, const float* w,
                            float eps, void* out, long long ldo, const int* rows, int n_out, int H, const float* extra, int extra_cols,
                            int T_tokens, cudaStream_t stream) {
    const size_t smem = (size_t)H * sizeof(float);
    const bool vec = H % 4 == 0 && ldo % 4 == 0 && (((size_t)residual | (size_t)delta | (size_t)out | (size_t)bias | (size_t)post_w | (size_t)w) & 15) == 0;
    int threads = vec ? (H / 4 + 31) / 32 * 32 : (H + 31) / 32 * 32;
    threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(post_norm_kernel<T, TD, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(post_norm_kernel<T, TD, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (vec)
        fe::launch(post_norm_kernel<T, TD, 4>, n_out, threads, smem, stream, residual, (const TD*)delta, bias, post_w, post_eps, w, eps,
                   (T*)out, ldo, rows, H, extra, extra_cols, T_tokens);
    else
        fe::launch(post_norm_kernel<T, TD, 1>, n_out, threads, smem, stream, residual, (const TD*)delta, bias, post_w, post_eps, w, eps,
                   (T*)out, ldo, rows, H, extra, extra_cols, T_tokens);
    return fe_check_launch("post_norm");
}

// delta_dtype / dtype: FE_F32 or FE_BF16 (the branch output and the rows written).  See the kernel for the rest.
extern "C" int fe_post_norm(float* residual, const void* delta, int delta_dtype, const float* bias, const float* post_w, float post_eps,
                            const float* w, float eps, void* out, long long ldo, const int* rows, int n_out, int H, const float* extra,
                            int extra_cols, int T, int dtype, cudaStream_t stream) {
    FE_REQUIRE(n_out >= 0 && H > 0 && T >= 0 && extra_cols >= 0 && ldo >= (long long)H + (extra ? extra_cols : 0) && H <= 56 * 1024,
               "post_norm: bad sizes (H %d, row stride %lld)", H, ldo);
    FE_REQUIRE((dtype == FE_F32 || dtype == FE_BF16) && (delta_dtype == FE_F32 || delta_dtype == FE_BF16), "post_norm: unknown dtype");
    FE_REQUIRE(!(dtype == FE_F32 && delta_dtype == FE_BF16), "post_norm: a bfloat16 branch beside float rows");
    if (n_out == 0) return 0;
    if (dtype == FE_F32)
        return launch_post_norm<float, float>(residual, delta, bias, post_w, post_eps, w, eps, out, ldo, rows, n_out, H, extra, extra_cols, T, stream);
    if (delta_dtype == FE_F32)
        return launch_post_norm<bf16, float>(residual, delta, bias, post_w, post_eps, w, eps, out, ldo, rows, n_out, H, extra, extra_cols, T, stream);
    return launch_post_norm<bf16, bf16>(residual, delta, bias, post_w, post_eps, w, eps, out, ldo, rows, n_out, H, extra, extra_cols, T, stream);
}

// ---------------------------------------------------------------------------------------------
// z <- cap * tanh(z * scale / cap) in place (cap 0: z <- z * scale), float logits.
__global__ void scale_softcap_kernel(float* __restrict__ z, long long n, float scale, float cap) {
    griddep_wait();
    griddep_launch_dependents();
    const float inv = cap > 0.f ? 1.f / cap : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = z[i] * scale;
        z[i] = cap > 0.f ? cap * tanhf(v * inv) : v;
    }
}

extern "C" int fe_scale_softcap(float* z, long long n, float scale, float cap, cudaStream_t stream) {
    FE_REQUIRE(n >= 0 && cap >= 0.f, "scale_softcap: bad sizes");
    if (n == 0) return 0;
    const long long want = (n + 255) / 256;
    fe::launch(scale_softcap_kernel, (unsigned)(want < 4096 ? want : 4096), 256, 0, stream, z, n, scale, cap);
    return fe_check_launch("scale_softcap");
}

// ---------------------------------------------------------------------------------------------
// out[t, j] = act(gu[t, j] + bias[j]) * (gu[t, I + j] + bias[I + j]); gu float or the compute type, out the compute type.
// act 0: silu; 1: the tanh form of GELU.
template <typename TI, typename T>
__global__ void gated_activation_bias_kernel(const TI* __restrict__ gu, const float* __restrict__ bias, T* __restrict__ out, long long total,
                                             int I, int act) {
    griddep_wait();
    griddep_launch_dependents();
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long t = e / I;
        const int j = (int)(e - t * I);
        float g = to_float(gu[t * 2 * I + j]), u = to_float(gu[t * 2 * I + I + j]);
        if (bias) {
            g += bias[j];
            u += bias[I + j];
        }
        const float a = act == 0 ? g / (1.f + expf(-g)) : 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
        out[e] = from_float<T>(a * u);
    }
}

extern "C" int fe_gated_activation_bias(const void* gu, int in_dtype, const float* bias, void* out, int T, int I, int act, int dtype,
                                        cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && I > 0 && (act == 0 || act == 1), "gated_activation_bias: bad sizes or activation");
    const long long total = (long long)T * I;
    if (total == 0) return 0;
    const long long want = (total + 255) / 256;
    const unsigned blocks = (unsigned)(want < 65535LL * 8 ? want : 65535LL * 8);
    if (in_dtype == FE_F32 && dtype == FE_F32)
        fe::launch(gated_activation_bias_kernel<float, float>, blocks, 256, 0, stream, (const float*)gu, bias, (float*)out, total, I, act);
    else if (in_dtype == FE_F32 && dtype == FE_BF16)
        fe::launch(gated_activation_bias_kernel<float, bf16>, blocks, 256, 0, stream, (const float*)gu, bias, (bf16*)out, total, I, act);
    else if (in_dtype == FE_BF16 && dtype == FE_BF16)
        fe::launch(gated_activation_bias_kernel<bf16, bf16>, blocks, 256, 0, stream, (const bf16*)gu, bias, (bf16*)out, total, I, act);
    else
        FE_REQUIRE(false, "gated_activation_bias: unknown dtypes %d -> %d", in_dtype, dtype);
    return fe_check_launch("gated_activation_bias");
}
