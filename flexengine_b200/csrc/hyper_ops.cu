// Kernels of decoders that keep several residual streams and of the mixers such designs bring along:
//   embedding into S copies of the stream, scaled;
//   the norm that reads a learned sum of the streams, with the sublayer before written into them in the same pass;
//   token shift (a row blended with the row of the token before, kept per request between steps);
//   what attention does between its projection and its scores: a short causal convolution over time with a kept history,
//     rotation of part of every head, unit norm of queries and keys, the cache write, all padded to one head size;
//   per-head output gates; the minGRU recurrence; a gated activation with a choice of gate function.
// All arithmetic is float; exp, tanh, sine, cosine and rsqrt are the accurate library forms.
#define FE_PDL_CLASS 4      // FE_PDL_ELEMENTWISE
#include "common.cuh"

using namespace fe;

namespace {

// 1 / (1 + exp(-x)): the accurate exponential, then the hardware's reciprocal (2 ulp; a full division is half of what a
// gate costs where a kernel does little else, as the recurrence does)
__device__ __forceinline__ float sigmoidf(float x) { return __fdividef(1.f, 1.f + expf(-x)); }

constexpr int MAX_STREAMS = 16;

}  // namespace

// ---------------------------------------------------------------------------------------------
// out[s, t, :] = table[ids[t], :] * scale for every stream s.
template <typename T>
__global__ void embedding_streams_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                         int T_tokens, int H, int V, float scale, int streams, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool bad = id < 0 || id >= V;
    if (bad && threadIdx.x == 0 && status) atomicOr(status, FE_STATUS_BAD_TOKEN);
    const T* row = table + (size_t)(bad ? 0 : id) * H;
    const size_t plane = (size_t)T_tokens * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float v = bad ? 0.f : to_float(row[j]) * scale;
        for (int s = 0; s < streams; ++s) out[s * plane + (size_t)t * H + j] = v;
    }
}

extern "C" int fe_embedding_streams(const int* ids, const void* table, float* out, int T, int H, int V, float scale, int streams,
                                    int dtype, int* status, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && H > 0 && V > 0 && streams >= 1, "embedding_streams: bad sizes T=%d H=%d V=%d streams=%d", T, H, V, streams);
    if (T == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == FE_F32)
        fe::launch(embedding_streams_kernel<float>, T, threads, 0, stream, ids, (const float*)table, out, T, H, V, scale, streams, status);
    else if (dtype == FE_BF16)
        fe::launch(embedding_streams_kernel<bf16>, T, threads, 0, stream, ids, (const bf16*)table, out, T, H, V, scale, streams, status);
    else
        FE_REQUIRE(false, "embedding_streams: unknown dtype %d", dtype);
    return fe_check_launch("embedding_streams");
}

// ---------------------------------------------------------------------------------------------
// One block per output row.  x [S, T, H] float.  If y is given, the sublayer before is put into the streams first:
//   x_t <- sum_s mix[s, t] x_s + write[t] * y * sigmoid(gate + gate_bias)         (every stream from the old ones)
// then u = sum_s read[s] x_s (read null: the plain sum), out = u * rsqrt(mean(u^2) + eps) * weight.
// rows == nullptr: row i, and the new streams are written back; rows != nullptr: output row i reads row rows[i] and the
// streams are left as they are.  u is staged in shared memory (H floats).
template <typename T, int SMAX>
__global__ void stream_rmsnorm_kernel(float* __restrict__ x, int S, int T_tokens, int H, const float* __restrict__ read,
                                      const float* __restrict__ weight, float eps, const T* __restrict__ y,
                                      const T* __restrict__ gate, const float* __restrict__ gate_bias,
                                      const float* __restrict__ mix, const float* __restrict__ write,
                                      const int* __restrict__ rows, T* __restrict__ out, const float* __restrict__ shift_mu,
                                      float* kept, long long kept_stride, const int* __restrict__ seats, int n_seats,
                                      T* __restrict__ shifted) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float u_row[];
    __shared__ float scratch[33];
    __shared__ float s_mix[SMAX * SMAX], s_write[SMAX], s_read[SMAX];
    for (int e = threadIdx.x; e < S * S; e += blockDim.x) s_mix[e] = mix ? mix[e] : 0.f;
    for (int e = threadIdx.x; e < S; e += blockDim.x) {
        s_write[e] = write ? write[e] : 0.f;
        s_read[e] = read ? read[e] : 1.f;
    }
    __syncthreads();
    const int i = blockIdx.x;
    int r = rows ? rows[i] : i;
    if (r < 0 || r >= T_tokens) r = 0;              // guarded: rows are checked on the host
    const size_t plane = (size_t)T_tokens * H;
    float* base = x + (size_t)r * H;
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) v[s] = s < S ? base[s * plane + j] : 0.f;
        float u = 0.f;
        if (y) {
            const float g = to_float(y[(size_t)r * H + j]) * sigmoidf(to_float(gate[(size_t)r * H + j]) + gate_bias[j]);
#pragma unroll
            for (int t = 0; t < SMAX; ++t) {
                if (t < S) {
                    float n = 0.f;
#pragma unroll
                    for (int s = 0; s < SMAX; ++s)
                        if (s < S) n = fmaf(s_mix[s * S + t], v[s], n);
                    n = fmaf(s_write[t], g, n);
                    if (!rows) base[t * plane + j] = n;
                    u = fmaf(s_read[t], n, u);
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < SMAX; ++s)
                if (s < S) u = fmaf(s_read[s], v[s], u);
        }
        u_row[j] = u;
        ss += u * u;
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)H + eps);
    T* o = out + (size_t)i * H;
    // ``shifted``: row i is request i's one token of the step; the token shift of the normed row is done here as well
    float* mine = nullptr;
    if (shifted) {
        const int seat = seats[i];
        if (seat >= 0 && seat < n_seats) mine = kept + (size_t)seat * kept_stride;
    }
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const T v = from_float<T>(u_row[j] * inv * weight[j]);
        o[j] = v;
        if (shifted) {
            const float x = to_float(v), before = mine ? mine[j] : 0.f;
            shifted[(size_t)i * H + j] = from_float<T>(fmaf(before - x, shift_mu[j], x));
            if (mine) mine[j] = x;
        }
    }
}

// The same, four columns a thread at a time (H % 4 == 0): 16-byte loads and stores of the float streams.
template <typename T> struct Quad;
template <> struct Quad<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Quad<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                           __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<const unsigned*>(&a);
        raw.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

// ITERS > 0: the row takes at most ITERS rounds of the block, and a thread asks for everything it reads of the row before it
// works on any of it (the kernel waits for memory, not for arithmetic); ITERS == 0: any width, round by round.
template <typename T, int SMAX, int ITERS>
__global__ void stream_rmsnorm_vec_kernel(float* __restrict__ x, int S, int T_tokens, int H, const float* __restrict__ read,
                                          const float* __restrict__ weight, float eps, const T* __restrict__ y,
                                          const T* __restrict__ gate, const float* __restrict__ gate_bias,
                                          const float* __restrict__ mix, const float* __restrict__ write,
                                          const int* __restrict__ rows, T* __restrict__ out, const float* __restrict__ shift_mu,
                                          float* kept, long long kept_stride, const int* __restrict__ seats, int n_seats,
                                          T* __restrict__ shifted) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float u_row[];
    __shared__ float scratch[33];
    __shared__ float s_mix[SMAX * SMAX], s_write[SMAX], s_read[SMAX];
    for (int e = threadIdx.x; e < S * S; e += blockDim.x) s_mix[e] = mix ? mix[e] : 0.f;
    for (int e = threadIdx.x; e < S; e += blockDim.x) {
        s_write[e] = write ? write[e] : 0.f;
        s_read[e] = read ? read[e] : 1.f;
    }
    const int i = blockIdx.x;
    int r = rows ? rows[i] : i;
    if (r < 0 || r >= T_tokens) r = 0;              // guarded: rows are checked on the host
    const size_t plane = (size_t)T_tokens * H;
    float* base = x + (size_t)r * H;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    float ss = 0.f;
    // columns j .. j + 3 of the row: the streams' values v, and of what goes into them y, gate and the gate's bias
    auto columns = [&](int j, const float4* v, float4 yy, float4 gg, float4 bb) {
        float4 u = zero;
        if (y) {
            const float4 g = make_float4(yy.x * sigmoidf(gg.x + bb.x), yy.y * sigmoidf(gg.y + bb.y), yy.z * sigmoidf(gg.z + bb.z),
                                         yy.w * sigmoidf(gg.w + bb.w));
#pragma unroll
            for (int t = 0; t < SMAX; ++t) {
                if (t < S) {
                    float4 n = zero;
#pragma unroll
                    for (int s = 0; s < SMAX; ++s) {
                        if (s < S) {
                            const float m = s_mix[s * S + t];
                            n.x = fmaf(m, v[s].x, n.x); n.y = fmaf(m, v[s].y, n.y); n.z = fmaf(m, v[s].z, n.z); n.w = fmaf(m, v[s].w, n.w);
                        }
                    }
                    const float w = s_write[t], rd = s_read[t];
                    n.x = fmaf(w, g.x, n.x); n.y = fmaf(w, g.y, n.y); n.z = fmaf(w, g.z, n.z); n.w = fmaf(w, g.w, n.w);
                    if (!rows) Quad<float>::store(base + t * plane + j, n);
                    u.x = fmaf(rd, n.x, u.x); u.y = fmaf(rd, n.y, u.y); u.z = fmaf(rd, n.z, u.z); u.w = fmaf(rd, n.w, u.w);
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < SMAX; ++s) {
                if (s < S) {
                    const float rd = s_read[s];
                    u.x = fmaf(rd, v[s].x, u.x); u.y = fmaf(rd, v[s].y, u.y); u.z = fmaf(rd, v[s].z, u.z); u.w = fmaf(rd, v[s].w, u.w);
                }
            }
        }
        *reinterpret_cast<float4*>(u_row + j) = u;
        ss += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
    };
    if (ITERS > 0) {
        constexpr int N = ITERS > 0 ? ITERS : 1;
        float4 v[N][SMAX], yy[N], gg[N], bb[N];
#pragma unroll
        for (int it = 0; it < N; ++it) {
            const int j = (it * blockDim.x + threadIdx.x) * 4;
            const bool in = j < H;
#pragma unroll
            for (int s = 0; s < SMAX; ++s) v[it][s] = (in && s < S) ? Quad<float>::load(base + s * plane + j) : zero;
            yy[it] = (in && y) ? Quad<T>::load(y + (size_t)r * H + j) : zero;
            gg[it] = (in && y) ? Quad<T>::load(gate + (size_t)r * H + j) : zero;
            bb[it] = (in && y) ? Quad<float>::load(gate_bias + j) : zero;
        }
        __syncthreads();                             // the mixing weights are in shared memory
#pragma unroll
        for (int it = 0; it < N; ++it) {
            const int j = (it * blockDim.x + threadIdx.x) * 4;
            if (j < H) columns(j, v[it], yy[it], gg[it], bb[it]);
        }
    } else {
        __syncthreads();
        for (int j = threadIdx.x * 4; j < H; j += blockDim.x * 4) {
            float4 v[SMAX];
#pragma unroll
            for (int s = 0; s < SMAX; ++s) v[s] = s < S ? Quad<float>::load(base + s * plane + j) : zero;
            const float4 yy = y ? Quad<T>::load(y + (size_t)r * H + j) : zero, gg = y ? Quad<T>::load(gate + (size_t)r * H + j) : zero;
            columns(j, v, yy, gg, y ? Quad<float>::load(gate_bias + j) : zero);
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)H + eps);
    T* o = out + (size_t)i * H;
    // ``shifted``: row i is request i's one token of the step; the token shift of the normed row is done here as well (on the
    // row as it was rounded, so that the kept row is what a later step reads of it)
    float* mine = nullptr;
    if (shifted) {
        const int seat = seats[i];
        if (seat >= 0 && seat < n_seats) mine = kept + (size_t)seat * kept_stride;
    }
    for (int j = threadIdx.x * 4; j < H; j += blockDim.x * 4) {
        const float4 u = *reinterpret_cast<const float4*>(u_row + j), w = Quad<float>::load(weight + j);
        Quad<T>::store(o + j, make_float4(u.x * inv * w.x, u.y * inv * w.y, u.z * inv * w.z, u.w * inv * w.w));
        if (shifted) {
            const float4 x = Quad<T>::load(o + j), m = Quad<float>::load(shift_mu + j);
            const float4 before = mine ? Quad<float>::load(mine + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            Quad<T>::store(shifted + (size_t)i * H + j, make_float4(fmaf(before.x - x.x, m.x, x.x), fmaf(before.y - x.y, m.y, x.y),
                                                                      fmaf(before.z - x.z, m.z, x.z), fmaf(before.w - x.w, m.w, x.w)));
            if (mine) Quad<float>::store(mine + j, x);
        }
    }
}

template <typename T>
static int launch_stream_rmsnorm(float* x, int S, int T_tokens, int H, const float* read, const float* weight, float eps, const void* y,
                                 const void* gate, const float* gate_bias, const float* mix, const float* write, const int* rows,
                                 int n_out, void* out, const float* shift_mu, float* kept, long long kept_stride, const int* seats,
                                 int n_seats, void* shifted, cudaStream_t stream) {
    const size_t smem = (size_t)H * sizeof(float);
    // four columns a thread when every row, of the streams and of what goes into them, starts on a 16-byte boundary; with up
    // to four streams and rows of up to 8,192 columns a thread takes its columns in at most two rounds, loaded together
    const bool vec = H % 4 == 0 && S <= 8 && (((size_t)x | (size_t)weight | (size_t)gate_bias) & 15) == 0 &&
                     (((size_t)y | (size_t)gate | (size_t)out | (size_t)shifted | (size_t)shift_mu | (size_t)kept) & 15) == 0 &&
                     kept_stride % 4 == 0;
    const bool staged = vec && S <= 4 && H <= 8192;
    int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (vec) threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    if (staged) {
        threads = ((H + 7) / 8 + 31) / 32 * 32;      // two rounds of four columns
        if (threads < 64) threads = 64;
    }
#define FE_LAUNCH_STREAM_NORM_PLAIN(SMAX)                                                                                 \
    fe::launch(stream_rmsnorm_kernel<T, SMAX>, n_out, threads, smem, stream, x, S, T_tokens, H, read, weight, eps,       \
               (const T*)y, (const T*)gate, gate_bias, mix, write, rows, (T*)out, shift_mu, kept, kept_stride, seats, n_seats, \
               (T*)shifted)
#define FE_LAUNCH_STREAM_NORM_VEC(SMAX, ITERS)                                                                            \
    fe::launch(stream_rmsnorm_vec_kernel<T, SMAX, ITERS>, n_out, threads, smem, stream, x, S, T_tokens, H, read, weight, \
               eps, (const T*)y, (const T*)gate, gate_bias, mix, write, rows, (T*)out, shift_mu, kept, kept_stride, seats,       \
               n_seats, (T*)shifted)
    if (staged) {
        if (S <= 1) FE_LAUNCH_STREAM_NORM_VEC(1, 2);
        else if (S <= 2) FE_LAUNCH_STREAM_NORM_VEC(2, 2);
        else FE_LAUNCH_STREAM_NORM_VEC(4, 2);
    } else if (vec) {
        if (S <= 4) FE_LAUNCH_STREAM_NORM_VEC(4, 0);
        else FE_LAUNCH_STREAM_NORM_VEC(8, 0);
    } else if (S <= 1) FE_LAUNCH_STREAM_NORM_PLAIN(1);
    else if (S <= 2) FE_LAUNCH_STREAM_NORM_PLAIN(2);
    else if (S <= 4) FE_LAUNCH_STREAM_NORM_PLAIN(4);
    else if (S <= 8) FE_LAUNCH_STREAM_NORM_PLAIN(8);
    else FE_LAUNCH_STREAM_NORM_PLAIN(16);
#undef FE_LAUNCH_STREAM_NORM_PLAIN
#undef FE_LAUNCH_STREAM_NORM_VEC
    return fe_check_launch("stream_rmsnorm");
}

// ``shifted`` (may be null): a step in which row i is request i's one token; the token shift of the normed rows is then done
// here too: shifted = h + (kept[seat] - h) * shift_mu, and the seat keeps h (``kept`` [seats, stride] float; a seat below 0 reads
// zeros and keeps nothing).  Only with rows == nullptr.
extern "C" int fe_stream_rmsnorm(float* x, int S, int T, int H, const float* read, const float* weight, float eps, const void* y,
                                 const void* gate, const float* gate_bias, const float* mix, const float* write, const int* rows,
                                 int n_out, void* out, const float* shift_mu, float* kept, long long kept_stride, const int* seats,
                                 int n_seats, void* shifted, int dtype, cudaStream_t stream) {
    FE_REQUIRE(S >= 1 && S <= MAX_STREAMS && T >= 0 && H > 0 && n_out >= 0, "stream_rmsnorm: bad sizes S=%d T=%d H=%d", S, T, H);
    FE_REQUIRE((size_t)H * sizeof(float) <= 48 * 1024, "stream_rmsnorm: rows of %d floats do not fit shared memory", H);
    FE_REQUIRE(y == nullptr || (gate && gate_bias && mix && write), "stream_rmsnorm: an update needs its gate, bias, mix and write");
    FE_REQUIRE(shifted == nullptr || (rows == nullptr && shift_mu && kept && seats && kept_stride >= H && n_out == T),
               "stream_rmsnorm: the token shift needs all rows, its weights, the kept rows and the seats");
    if (n_out == 0 || T == 0) return 0;
    if (dtype == FE_F32)
        return launch_stream_rmsnorm<float>(x, S, T, H, read, weight, eps, y, gate, gate_bias, mix, write, rows, n_out, out, shift_mu, kept,
                                            kept_stride, seats, n_seats, shifted, stream);
    if (dtype == FE_BF16)
        return launch_stream_rmsnorm<bf16>(x, S, T, H, read, weight, eps, y, gate, gate_bias, mix, write, rows, n_out, out, shift_mu, kept,
                                           kept_stride, seats, n_seats, shifted, stream);
    FE_REQUIRE(false, "stream_rmsnorm: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------------
// out = h + (h' - h) * mu, h' the row of the token before.  A request's first token of the step takes the row its seat
// kept (``kept`` [seats, stride] float; zeros for a seat below 0), and the thread that read it writes the request's last
// row of this step in its place, element by element, so nobody else touches it.
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ h, const float* __restrict__ mu, float* kept, long long kept_stride,
                                   const int* __restrict__ seats, const int* __restrict__ cu_q, const int* __restrict__ token_req,
                                   T* __restrict__ out, int D, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    const int t = blockIdx.x;
    const int r = token_req[t];
    const int first = cu_q[r];
    const int seat = seats[r];
    float* mine = (seat >= 0 && seat < n_seats) ? kept + (size_t)seat * kept_stride : nullptr;
    const T* row = h + (size_t)t * D;
    const T* prev = t > first ? h + (size_t)(t - 1) * D : nullptr;
    const T* last = h + (size_t)(cu_q[r + 1] - 1) * D;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < D; j += gridDim.y * blockDim.x) {
        const float x = to_float(row[j]);
        float before = 0.f;
        if (prev) before = to_float(prev[j]);
        else if (mine) {
            before = mine[j];
            mine[j] = to_float(last[j]);
        }
        out[(size_t)t * D + j] = from_float<T>(fmaf(before - x, mu[j], x));
    }
}

// The same, eight columns a thread (D and the kept rows' stride multiples of 8): 16- and 32-byte loads and stores.
template <typename T>
__global__ void token_shift_vec_kernel(const T* __restrict__ h, const float* __restrict__ mu, float* kept, long long kept_stride,
                                       const int* __restrict__ seats, const int* __restrict__ cu_q, const int* __restrict__ token_req,
                                       T* __restrict__ out, int T_tokens, int D, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    const int per_row = D >> 3;
    const long long total = (long long)T_tokens * per_row;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(e / per_row), j = (int)(e - (long long)t * per_row) << 3;
        const int r = token_req[t];
        const int first = cu_q[r];
        float x[8], before[8], m[8];
        load8<T>(h + (size_t)t * D + j, x);
        load8<float>(mu + j, m);
        if (t > first) {
            load8<T>(h + (size_t)(t - 1) * D + j, before);
        } else {
            const int seat = seats[r];
            if (seat >= 0 && seat < n_seats) {
                float* mine = kept + (size_t)seat * kept_stride + j;
                float last[8];
                load8<float>(mine, before);
                load8<T>(h + (size_t)(cu_q[r + 1] - 1) * D + j, last);
                store8<float>(mine, last);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) before[i] = 0.f;
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = fmaf(before[i] - x[i], m[i], x[i]);
        store8<T>(out + (size_t)t * D + j, x);
    }
}

extern "C" int fe_token_shift(const void* h, const float* mu, float* kept, long long kept_stride, const int* seats, const int* cu_q,
                              const int* token_req, void* out, int T, int D, int n_seats, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && D > 0 && n_seats >= 0 && kept_stride >= D, "token_shift: bad sizes");
    if (T == 0) return 0;
    if (D % 8 == 0 && kept_stride % 8 == 0 && (((size_t)h | (size_t)out | (size_t)mu | (size_t)kept) & 31) == 0 &&
        (dtype == FE_F32 || dtype == FE_BF16)) {
        const long long total = (long long)T * (D >> 3), want = (total + 255) / 256;
        const int blocks = (int)(want < 65535LL * 4 ? want : 65535LL * 4);
        if (dtype == FE_F32)
            fe::launch(token_shift_vec_kernel<float>, blocks, 256, 0, stream, (const float*)h, mu, kept, kept_stride, seats, cu_q, token_req,
                       (float*)out, T, D, n_seats);
        else
            fe::launch(token_shift_vec_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)h, mu, kept, kept_stride, seats, cu_q, token_req,
                       (bf16*)out, T, D, n_seats);
        return fe_check_launch("token_shift");
    }
    const int threads = D >= 1024 ? 256 : 128;
    const int stretches = T >= 512 ? 1 : (D + threads - 1) / threads;
    const dim3 grid(T, stretches < 65535 ? stretches : 65535);
    if (dtype == FE_F32)
        fe::launch(token_shift_kernel<float>, grid, threads, 0, stream, (const float*)h, mu, kept, kept_stride, seats, cu_q, token_req,
                   (float*)out, D, n_seats);
    else if (dtype == FE_BF16)
        fe::launch(token_shift_kernel<bf16>, grid, threads, 0, stream, (const bf16*)h, mu, kept, kept_stride, seats, cu_q, token_req,
                   (bf16*)out, D, n_seats);
    else
        FE_REQUIRE(false, "token_shift: unknown dtype %d", dtype);
    return fe_check_launch("token_shift");
}

// ---------------------------------------------------------------------------------------------
// Between the projection and the scores.  ``proj`` [T, ld] holds q | k | v of every token: ``heads`` query heads and
// ``kv_heads`` key heads of ``dim`` entries, ``kv_heads`` value heads of ``vdim``.  One block per token; its warps share out
// the token's heads of q, k and v:
//   convolution (taps > 0): y_t[c] = sum_j conv[j, c] * u_(t - taps + 1 + j)[c] over the request's own rows, those before
//     this step from ``history`` [seats, (taps - 1) * C] (oldest first; zeros for a seat below 0); the table is held tap by
//     tap, [taps, C], so that the lanes of a warp read neighbouring numbers;
//   rotation (q, k): entries i and i + rot/2 of the head's first ``rot`` turn by position * inv_freq[i]; the token's sines
//     and cosines are worked out once, by the whole block, for all of its heads;
//   unit norm (q, k; qk_norm): the head divided by sqrt(mean of its squares + eps);
//   q into ``q_out`` [T, heads * head], k and v into their cache slots [pages, kv_heads, ps, head], zeros beyond dim / vdim.
// The history of a channel is read only by the first taps - 1 tokens of the request's portion.  The block of the portion's
// first token therefore runs all of them, one after the other, and then brings the history up to date (the blocks of the
// other early tokens do nothing), so that no block reads what another one writes.
// PER > 0: a head's size is 32 * PER and a lane owns PER consecutive entries, moved with one load and one store each (rows
// start on 16-byte boundaries); PER == 0: any size, entry c = lane + 32 k.
namespace {

template <typename T, int PER> struct Lanes;          // PER consecutive elements of T as floats
template <int PER> struct Lanes<float, PER> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
#pragma unroll
        for (int i = 0; i < PER; ++i) v[i] = p[i];
    }
    static __device__ __forceinline__ void store(float* p, const float* v) {
#pragma unroll
        for (int i = 0; i < PER; ++i) p[i] = v[i];
    }
};
template <> struct Lanes<float, 4> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Lanes<float, 8> {
    static __device__ __forceinline__ void load(const float* p, float* v) { load8<float>(p, v); }
    static __device__ __forceinline__ void store(float* p, const float* v) { store8<float>(p, v); }
};
template <int PER> struct Lanes<bf16, PER> {
    static __device__ __forceinline__ void load(const bf16* p, float* v) {
#pragma unroll
        for (int i = 0; i < PER; ++i) v[i] = __bfloat162float(p[i]);
    }
    static __device__ __forceinline__ void store(bf16* p, const float* v) {
#pragma unroll
        for (int i = 0; i < PER; ++i) p[i] = __float2bfloat16_rn(v[i]);
    }
};
template <> struct Lanes<bf16, 2> {
    static __device__ __forceinline__ void load(const bf16* p, float* v) {
        const unsigned raw = *reinterpret_cast<const unsigned*>(p);
        v[0] = __uint_as_float(raw << 16); v[1] = __uint_as_float(raw & 0xffff0000u);
    }
    static __device__ __forceinline__ void store(bf16* p, const float* v) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]); }
};
template <> struct Lanes<bf16, 4> {
    static __device__ __forceinline__ void load(const bf16* p, float* v) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
        v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
    }
    static __device__ __forceinline__ void store(bf16* p, const float* v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<const unsigned*>(&a);
        raw.y = *reinterpret_cast<const unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};
template <> struct Lanes<bf16, 8> {
    static __device__ __forceinline__ void load(const bf16* p, float* v) { load8<bf16>(p, v); }
    static __device__ __forceinline__ void store(bf16* p, const float* v) { store8<bf16>(p, v); }
};

}  // namespace

template <typename T, int PER>
__global__ void qkv_conv_rope_norm_cache_kernel(const T* __restrict__ proj, long long ld, const float* __restrict__ conv, float* history,
                                                long long history_stride, int taps, const int* __restrict__ seats,
                                                const int* __restrict__ cu_q, const int* __restrict__ token_req,
                                                const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot,
                                                int qk_norm, float eps, const int* __restrict__ slot_mapping, T* __restrict__ kc,
                                                T* __restrict__ vc, T* __restrict__ q_out, int T_tokens, int heads, int kv_heads, int dim,
                                                int vdim, int head, int ps, long long num_slots, int n_seats, int* __restrict__ status,
                                                const float* __restrict__ q_weight, const float* __restrict__ k_weight, float temp_coef,
                                                int temp_every) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float staged[];
    constexpr int LIMIT = PER > 0 ? PER : 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int half = rot >> 1;
    float* cosines = staged;                               // [half], then the sines [half], then a head per warp
    float* sines = staged + half;
    float* buf = staged + rot + (size_t)warp * head;
    const int per_token = heads + 2 * kv_heads;
    const int tok = blockIdx.x;
    const int C = (heads + kv_heads) * dim + kv_heads * vdim;
    const int r = token_req[tok];
    const int first = cu_q[r], n = cu_q[r + 1] - first, li = tok - first;
    const int seat = seats[r];
    const int back = taps > 1 ? taps - 1 : 0;
    float* hist = (back && history && seat >= 0 && seat < n_seats) ? history + (size_t)seat * history_stride : nullptr;
    int reps = 1;
    if (back) {
        if (li == 0) reps = min(n, back);
        else if (li < back) return;
    }
    for (int rep = 0; rep < reps; ++rep) {
        const int t = tok + rep, lt = li + rep;
        if (inv_freq && rot > 0) {
            const float pos = (float)positions[t];
            for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &sines[i], &cosines[i]);
        }
        __syncthreads();
        for (int hs = warp; hs < per_token; hs += warps) {
            // which head this is: 0 query, 1 key, 2 value; its first channel and its size
            const int what = hs < heads ? 0 : (hs < heads + kv_heads ? 1 : 2);
            const int index = what == 0 ? hs : (what == 1 ? hs - heads : hs - heads - kv_heads);
            const int hd = what == 2 ? vdim : dim;
            const int ch0 = what == 0 ? index * dim : (what == 1 ? (heads + index) * dim : (heads + kv_heads) * dim + index * vdim);
            // this lane's entries: PER consecutive ones from lane * PER, or lane, lane + 32, ...
            const int rounds = PER > 0 ? 1 : (hd + 31) / 32;
            for (int k = 0; k < rounds; ++k) {
                const int c = PER > 0 ? lane * PER : lane + 32 * k;
                if (c >= hd) continue;
                const int ch = ch0 + c;
                float acc[LIMIT];
                if (conv) {
#pragma unroll
                    for (int e = 0; e < LIMIT; ++e) acc[e] = 0.f;
                    // four taps at a time: their loads are all on their way before the first is used
#pragma unroll 4
                    for (int j = 0; j < taps; ++j) {
                        const int from = lt - (taps - 1 - j);
                        float u[LIMIT], w[LIMIT];
                        Lanes<float, LIMIT>::load(conv + (size_t)j * C + ch, w);
                        if (from >= 0) Lanes<T, LIMIT>::load(proj + (size_t)(first + from) * ld + ch, u);
                        else if (hist) Lanes<float, LIMIT>::load(hist + (size_t)(back + from) * C + ch, u);
                        else {
#pragma unroll
                            for (int e = 0; e < LIMIT; ++e) u[e] = 0.f;
                        }
#pragma unroll
                        for (int e = 0; e < LIMIT; ++e) acc[e] = fmaf(w[e], u[e], acc[e]);
                    }
                } else {
                    Lanes<T, LIMIT>::load(proj + (size_t)t * ld + ch, acc);
                }
#pragma unroll
                for (int e = 0; e < LIMIT; ++e) buf[c + e] = acc[e];
            }
            __syncwarp();
            float inv = 1.f;
            if (what != 2) {
                if (inv_freq && rot > 0) {
                    for (int i = lane; i < half; i += 32) {
                        const float s = sines[i], c = cosines[i];
                        const float a = buf[i], b = buf[i + half];
                        buf[i] = a * c - b * s;
                        buf[i + half] = b * c + a * s;
                    }
                    __syncwarp();
                }
                if (qk_norm) {
                    float ss = 0.f;
                    for (int c = lane; c < hd; c += 32) ss = fmaf(buf[c], buf[c], ss);
                    ss = warp_sum(ss);
                    inv = rsqrtf(ss / (float)hd + eps);
                }
            }
            // after the norm: its weight (one table for the query heads, one for the key heads) and, for a query, the
            // temperature of its position, 1 + coef ln(floor((p + 1) / every) + 1)
            const float* wt = what == 0 ? q_weight : (what == 1 ? k_weight : nullptr);
            if (what == 0 && temp_coef != 0.f) inv *= 1.f + temp_coef * logf((float)((positions[t] + 1) / temp_every) + 1.f);
            T* dst = nullptr;
            if (what == 0) {
                dst = q_out + (size_t)t * heads * head + (size_t)index * head;
            } else if (slot_mapping) {
                const int slot = slot_mapping[t];
                if (slot >= 0) {
                    if (slot >= num_slots) {
                        if (lane == 0 && status) atomicOr(status, FE_STATUS_BAD_SLOT);
                    } else {
                        const long long page = slot / ps, off = slot % ps;
                        dst = (what == 1 ? kc : vc) + ((page * kv_heads + index) * ps + off) * head;
                    }
                }
            }
            if (dst) {
                if (PER > 0) {
                    float v[LIMIT];
#pragma unroll
                    for (int e = 0; e < LIMIT; ++e) v[e] = buf[lane * LIMIT + e] * inv * (wt ? wt[lane * LIMIT + e] : 1.f);
                    Lanes<T, LIMIT>::store(dst + lane * LIMIT, v);
                    for (int c = hd + lane; c < head; c += 32) dst[c] = from_float<T>(0.f);
                } else {
                    for (int c = lane; c < head; c += 32) dst[c] = from_float<T>(c < hd ? buf[c] * inv * (wt ? wt[c] : 1.f) : 0.f);
                }
            }
            __syncwarp();
        }
        __syncthreads();                 // before the next token's sines and cosines go where these are
    }
    if (hist && li == 0) {
        // the last ``back`` projected rows of the request, oldest first: what was kept moves up, this step's rows follow
        for (int ch = threadIdx.x; ch < C; ch += blockDim.x) {
            for (int m = 0; m < back; ++m) {
                const int from = m + n;
                hist[(size_t)m * C + ch] = from < back ? hist[(size_t)from * C + ch] : to_float(proj[(size_t)(first + from - back) * ld + ch]);
            }
        }
    }
}

template <typename T>
static int launch_qkv_prepare(const void* proj, long long ld, const float* conv, float* history, long long history_stride, int taps,
                              const int* seats, const int* cu_q, const int* token_req, const int* positions, const float* inv_freq, int rot,
                              int qk_norm, float eps, const int* slot_mapping, void* kc, void* vc, void* q_out, int T_tokens, int heads,
                              int kv_heads, int dim, int vdim, int head, int ps, long long num_slots, int n_seats, int* status,
                              const float* q_weight, const float* k_weight, float temp_coef, int temp_every, cudaStream_t stream) {
    const int per_token = heads + 2 * kv_heads;
    // up to 16 warps share out the token's heads evenly: 24 heads are two rounds of 12 warps
    const int rounds = (per_token + 15) / 16;
    int warps = (per_token + rounds - 1) / rounds;
    const int fit = (int)((48 * 1024 - (size_t)rot * sizeof(float)) / ((size_t)head * sizeof(float)));      // a head per warp in shared memory
    if (warps > fit) warps = fit;
    const size_t smem = ((size_t)rot + (size_t)warps * head) * sizeof(float);
    // a lane owns consecutive entries when both head sizes are the same multiple of 32 and every row it touches starts on a
    // 16-byte boundary
    const long long C = (long long)(heads + kv_heads) * dim + (long long)kv_heads * vdim;
    const bool aligned = dim == vdim && dim % 32 == 0 && dim <= 256 && ld % 8 == 0 && head % 8 == 0 && C % 4 == 0 && history_stride % 4 == 0 &&
                         (((size_t)proj | (size_t)kc | (size_t)vc | (size_t)q_out | (size_t)history | (size_t)conv) & 15) == 0;
    const int per = aligned ? dim / 32 : 0;
#define FE_LAUNCH_QKV_PREPARE(PER)                                                                                                   \
    fe::launch(qkv_conv_rope_norm_cache_kernel<T, PER>, T_tokens, warps * 32, smem, stream, (const T*)proj, ld, conv, history,     \
               history_stride, taps, seats, cu_q, token_req, positions, inv_freq, rot, qk_norm, eps, slot_mapping, (T*)kc, (T*)vc,  \
               (T*)q_out, T_tokens, heads, kv_heads, dim, vdim, head, ps, num_slots, n_seats, status, q_weight, k_weight, temp_coef,     \
               temp_every)
    if (per == 1) FE_LAUNCH_QKV_PREPARE(1);
    else if (per == 2) FE_LAUNCH_QKV_PREPARE(2);
    else if (per == 4) FE_LAUNCH_QKV_PREPARE(4);
    else if (per == 8) FE_LAUNCH_QKV_PREPARE(8);
    else FE_LAUNCH_QKV_PREPARE(0);
#undef FE_LAUNCH_QKV_PREPARE
    return fe_check_launch("qkv_conv_rope_norm_cache");
}

extern "C" int fe_qkv_conv_rope_norm_cache(const void* proj, long long ld, const float* conv, float* history, long long history_stride,
                                           int taps, const int* seats, const int* cu_q, const int* token_req, const int* positions,
                                           const float* inv_freq, int rot, int qk_norm, float eps, const int* slot_mapping, void* kc,
                                           void* vc, void* q_out, int T, int heads, int kv_heads, int dim, int vdim, int head, int ps,
                                           long long num_slots, int n_seats, int dtype, int* status, const float* q_weight,
                                           const float* k_weight, float temp_coef, int temp_every, cudaStream_t stream) {
    FE_REQUIRE((q_weight == nullptr) == (k_weight == nullptr) && (temp_coef == 0.f || temp_every > 0),
               "qkv_conv_rope_norm_cache: norm weights come in pairs, and a temperature needs a positive period");
    FE_REQUIRE(T >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && head >= dim && head >= vdim && head <= 1024,
               "qkv_conv_rope_norm_cache: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d head=%d", heads, kv_heads, dim, vdim, head);
    FE_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dim && ps > 0 && taps >= 0, "qkv_conv_rope_norm_cache: bad rotation, page size or taps");
    FE_REQUIRE(conv != nullptr || taps == 0, "qkv_conv_rope_norm_cache: taps without a table");
    FE_REQUIRE(taps <= 1 || history != nullptr, "qkv_conv_rope_norm_cache: a convolution of several taps needs its history");
    const long long C = (long long)(heads + kv_heads) * dim + (long long)kv_heads * vdim;
    FE_REQUIRE(ld >= C && (taps <= 1 || history_stride >= (taps - 1) * C), "qkv_conv_rope_norm_cache: rows too short");
    if (T == 0) return 0;
    if (dtype == FE_F32)
        return launch_qkv_prepare<float>(proj, ld, conv, history, history_stride, taps, seats, cu_q, token_req, positions, inv_freq, rot,
                                         qk_norm, eps, slot_mapping, kc, vc, q_out, T, heads, kv_heads, dim, vdim, head, ps, num_slots,
                                         n_seats, status, q_weight, k_weight, temp_coef, temp_every, stream);
    if (dtype == FE_BF16)
        return launch_qkv_prepare<bf16>(proj, ld, conv, history, history_stride, taps, seats, cu_q, token_req, positions, inv_freq, rot,
                                        qk_norm, eps, slot_mapping, kc, vc, q_out, T, heads, kv_heads, dim, vdim, head, ps, num_slots,
                                        n_seats, status, q_weight, k_weight, temp_coef, temp_every, stream);
    FE_REQUIRE(false, "qkv_conv_rope_norm_cache: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------------
// Between the projection and the scores, second form: norms over whole projections, and values that turn.  ``proj`` [T, ld]
// holds q | k | v as above.  One block per token:
//   norm (q_weight, k_weight given): the token's whole query projection (all heads at once) is divided by its root mean
//     square and multiplied by a weight of heads * dim numbers; the whole key projection likewise (kv_heads * dim);
//   rotation (q, k), after the norm: the first ``rot`` entries of every head turn by position * inv_freq[i]; pairs are
//     (2i, 2i + 1) when ``interleaved``, else (i, i + rot/2);
//   values (v_inv_freq given): all ``vdim`` entries of every value head turn by position * v_inv_freq[m], pairs laid out
//     the same way;
//   q into ``q_out`` [T, heads * head], k and v into their cache slots [pages, kv_heads, ps, head], zeros beyond dim / vdim.
// The token's row is staged in shared memory as floats; sines and cosines are worked out once a token, in float.
namespace {

// entry c of a head whose first ``dims`` entries turn: the entry after the turn.  ``at`` points at the head's first entry.
__device__ __forceinline__ float turned_entry(const float* at, int c, int dims, int interleaved, const float* cosines,
                                              const float* sines, float sign) {
    const float v = at[c];
    if (c >= dims) return v;
    const int half = dims >> 1;
    int i, partner;
    bool second;
    if (interleaved) { i = c >> 1; partner = c ^ 1; second = c & 1; }
    else { second = c >= half; i = second ? c - half : c; partner = second ? c - half : c + half; }
    const float other = at[partner], co = cosines[i], si = sign * sines[i];
    return second ? fmaf(v, co, other * si) : fmaf(v, co, -other * si);
}

template <typename T>
__global__ void qkv_norm_rope_cache_kernel(const T* __restrict__ proj, long long ld, const float* __restrict__ q_weight,
                                           const float* __restrict__ k_weight, float eps, const int* __restrict__ positions,
                                           const float* __restrict__ inv_freq, int rot, int interleaved,
                                           const float* __restrict__ v_inv_freq, const int* __restrict__ slot_mapping,
                                           T* __restrict__ kc, T* __restrict__ vc, T* __restrict__ q_out, int heads, int kv_heads,
                                           int dim, int vdim, int head, int ps, long long num_slots, int* __restrict__ status) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float staged[];
    __shared__ float scratch[33];
    const int tok = blockIdx.x;
    const int qw = heads * dim, kw = kv_heads * dim, vw = kv_heads * vdim;
    const int C = qw + kw + vw;
    const int half = rot >> 1, vhalf = v_inv_freq ? vdim >> 1 : 0;
    float* row = staged;                              // [C]
    float* cosines = staged + C;                      // [half], then the sines [half]
    float* sines = cosines + half;
    float* vcos = sines + half;                       // [vhalf], then [vhalf]
    float* vsin = vcos + vhalf;
    const float pos = (float)positions[tok];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &sines[i], &cosines[i]);
    for (int i = threadIdx.x; i < vhalf; i += blockDim.x) sincosf(pos * v_inv_freq[i], &vsin[i], &vcos[i]);
    const T* src = proj + (size_t)tok * ld;
    float ssq = 0.f, ssk = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float v = to_float(src[c]);
        row[c] = v;
        if (c < qw) ssq = fmaf(v, v, ssq);
        else if (c < qw + kw) ssk = fmaf(v, v, ssk);
    }
    if (q_weight) {
        const float inv_q = rsqrtf(block_sum(ssq, scratch) / (float)qw + eps);
        const float inv_k = rsqrtf(block_sum(ssk, scratch) / (float)kw + eps);
        for (int c = threadIdx.x; c < qw + kw; c += blockDim.x)
            row[c] *= c < qw ? inv_q * q_weight[c] : inv_k * k_weight[c - qw];
    }
    __syncthreads();
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (slot_mapping) {
        const int slot = slot_mapping[tok];
        if (slot >= 0) {
            if (slot >= num_slots) {
                if (threadIdx.x == 0 && status) atomicOr(status, FE_STATUS_BAD_SLOT);
            } else {
                const long long page = slot / ps, off = slot % ps;
                kdst = kc + ((page * kv_heads) * ps + off) * head;          // head 0; the next head is ps * head further
                vdst = vc + ((page * kv_heads) * ps + off) * head;
            }
        }
    }
    T* qdst = q_out + (size_t)tok * heads * head;
    const int per_token = heads + 2 * kv_heads;
    for (int e = threadIdx.x; e < per_token * head; e += blockDim.x) {
        const int hs = e / head, c = e - hs * head;
        float v = 0.f;
        if (hs < heads + kv_heads) {
            if (c < dim) v = turned_entry(row + (size_t)hs * dim, c, rot, interleaved, cosines, sines, 1.f);
            if (hs < heads) qdst[(size_t)hs * head + c] = from_float<T>(v);
            else if (kdst) kdst[(size_t)(hs - heads) * ps * head + c] = from_float<T>(v);
        } else if (vdst) {
            const int index = hs - heads - kv_heads;
            if (c < vdim) v = turned_entry(row + qw + kw + (size_t)index * vdim, c, vhalf * 2, interleaved, vcos, vsin, 1.f);
            vdst[(size_t)index * ps * head + c] = from_float<T>(v);
        }
    }
}

// out[t, h, :vdim] = the first vdim entries of head h of mixed[t] turned BACK by the token's position (pair m by
// -position * inv_freq[m]), times ``scale``; the padding of the attention kernels' head size is dropped on the way.
template <typename T>
__global__ void unrotate_heads_kernel(const T* __restrict__ mixed, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                      T* __restrict__ out, long long ldo, int heads, int head, int vdim, int interleaved, float scale) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ float trig[];                  // cos [vdim / 2], sin [vdim / 2]
    const int tok = blockIdx.x, half = vdim >> 1;
    const float pos = (float)positions[tok];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &trig[half + i], &trig[i]);
    __syncthreads();
    const T* src = mixed + (size_t)tok * heads * head;
    T* dst = out + (size_t)tok * ldo;
    for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        const float u = to_float(src[(size_t)h * head + a]), v = to_float(src[(size_t)h * head + b]);
        const float co = trig[i], si = trig[half + i];
        dst[(size_t)h * vdim + a] = from_float<T>((u * co + v * si) * scale);
        dst[(size_t)h * vdim + b] = from_float<T>((v * co - u * si) * scale);
    }
}

}  // namespace

extern "C" int fe_qkv_norm_rope_cache(const void* proj, long long ld, const float* q_weight, const float* k_weight, float eps,
                                      const int* positions, const float* inv_freq, int rot, int interleaved, const float* v_inv_freq,
                                      const int* slot_mapping, void* kc, void* vc, void* q_out, int T, int heads, int kv_heads, int dim,
                                      int vdim, int head, int ps, long long num_slots, int dtype, int* status, cudaStream_t stream) {
    FE_REQUIRE((q_weight == nullptr) == (k_weight == nullptr), "qkv_norm_rope_cache: the norm weights come in pairs");
    FE_REQUIRE(T >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && head >= dim && head >= vdim && head <= 1024,
               "qkv_norm_rope_cache: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d head=%d", heads, kv_heads, dim, vdim, head);
    FE_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dim && ps > 0 && (inv_freq != nullptr || rot == 0) && (v_inv_freq == nullptr || vdim % 2 == 0),
               "qkv_norm_rope_cache: bad rotation or page size");
    const long long C = (long long)(heads + kv_heads) * dim + (long long)kv_heads * vdim;
    FE_REQUIRE(ld >= C, "qkv_norm_rope_cache: rows too short");
    if (T == 0) return 0;
    const size_t smem = ((size_t)C + rot + (v_inv_freq ? vdim : 0)) * sizeof(float);
    FE_REQUIRE(smem <= 200 * 1024, "qkv_norm_rope_cache: a token's projections need %zu bytes of shared memory (limit 204800)", smem);
    FE_REQUIRE(dtype == FE_F32 || dtype == FE_BF16, "qkv_norm_rope_cache: unknown dtype %d", dtype);
    const int threads = C >= 2048 ? 512 : 256;
#define FE_LAUNCH_QKV_NORM(TYPE)                                                                                                        \
    do {                                                                                                                                \
        if (smem > 48 * 1024) {                                                                                                         \
            cudaError_t err = cudaFuncSetAttribute(qkv_norm_rope_cache_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            FE_REQUIRE(err == cudaSuccess, "qkv_norm_rope_cache: %s", cudaGetErrorString(err));                                          \
        }                                                                                                                               \
        fe::launch(qkv_norm_rope_cache_kernel<TYPE>, T, threads, smem, stream, (const TYPE*)proj, ld, q_weight, k_weight, eps, positions, \
                   inv_freq, rot, interleaved, v_inv_freq, slot_mapping, (TYPE*)kc, (TYPE*)vc, (TYPE*)q_out, heads, kv_heads, dim, vdim,    \
                   head, ps, num_slots, status);                                                                                        \
    } while (0)
    if (dtype == FE_F32) FE_LAUNCH_QKV_NORM(float);
    else FE_LAUNCH_QKV_NORM(bf16);
#undef FE_LAUNCH_QKV_NORM
    return fe_check_launch("qkv_norm_rope_cache");
}

extern "C" int fe_unrotate_heads(const void* mixed, const int* positions, const float* inv_freq, void* out, long long ldo, int T,
                                 int heads, int head, int vdim, int interleaved, float scale, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && heads > 0 && vdim > 0 && vdim % 2 == 0 && head >= vdim && ldo >= (long long)heads * vdim && inv_freq != nullptr,
               "unrotate_heads: bad sizes");
    FE_REQUIRE(dtype == FE_F32 || dtype == FE_BF16, "unrotate_heads: unknown dtype %d", dtype);
    if (T == 0) return 0;
    const size_t smem = (size_t)vdim * sizeof(float);
    const int threads = heads * vdim >= 2048 ? 512 : 256;
    if (dtype == FE_F32)
        fe::launch(unrotate_heads_kernel<float>, T, threads, smem, stream, (const float*)mixed, positions, inv_freq, (float*)out, ldo, heads,
                   head, vdim, interleaved, scale);
    else
        fe::launch(unrotate_heads_kernel<bf16>, T, threads, smem, stream, (const bf16*)mixed, positions, inv_freq, (bf16*)out, ldo, heads,
                   head, vdim, interleaved, scale);
    return fe_check_launch("unrotate_heads");
}

// ---------------------------------------------------------------------------------------------
// out[t, h, :vdim] = mixed[t, h, :vdim] * sigmoid(gate) * scale: every head's output times its gate, the padding of the
// attention kernels' head size dropped on the way.  The gate of entry c of head h is gates[t * ld + h] (one a head), or
// gates[t * ld + h * vdim + c] with ``per_element``.  A row of out is ldo entries long (a view of a wider buffer).
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ mixed, const T* __restrict__ gates, long long ld, T* __restrict__ out,
                                 long long ldo, long long total, int heads, int head, int vdim, int per_element, float scale) {
    griddep_wait();
    griddep_launch_dependents();
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(e % vdim);
        const long long th = e / vdim;
        const int h = (int)(th % heads);
        const long long t = th / heads;
        const float g = to_float(gates[t * ld + (per_element ? h * vdim + c : h)]);
        out[t * ldo + h * vdim + c] = from_float<T>(to_float(mixed[(t * heads + h) * head + c]) * sigmoidf(g) * scale);
    }
}

// The same, eight columns of one head a thread (vdim, head and the row lengths multiples of 8): 16- or 32-byte loads and stores.
template <typename T>
__global__ void head_gate_vec_kernel(const T* __restrict__ mixed, const T* __restrict__ gates, long long ld, T* __restrict__ out,
                                     long long ldo, long long groups, int heads, int head, int vdim, int per_element, float scale) {
    griddep_wait();
    griddep_launch_dependents();
    const int per_head = vdim >> 3;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < groups; e += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(e % per_head) << 3;
        const long long th = e / per_head;
        const int h = (int)(th % heads);
        const long long t = th / heads;
        float v[8], g[8];
        load8<T>(mixed + (t * heads + h) * head + c, v);
        if (per_element) {
            load8<T>(gates + t * ld + h * vdim + c, g);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= sigmoidf(g[i]) * scale;
        } else {
            const float one = sigmoidf(to_float(gates[t * ld + h])) * scale;
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= one;
        }
        store8<T>(out + t * ldo + h * vdim + c, v);
    }
}

extern "C" int fe_head_gate(const void* mixed, const void* gates, long long ld, void* out, long long ldo, int T, int heads, int head,
                            int vdim, int per_element, float scale, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && heads > 0 && head >= vdim && vdim > 0 && ldo >= (long long)heads * vdim, "head_gate: bad sizes");
    FE_REQUIRE(dtype == FE_F32 || dtype == FE_BF16, "head_gate: unknown dtype %d", dtype);
    const long long total = (long long)T * heads * vdim;
    if (total == 0) return 0;
    const bool gates_fit = !per_element || (ld % 8 == 0 && ((size_t)gates & 31) == 0);
    if (vdim % 8 == 0 && head % 8 == 0 && ldo % 8 == 0 && gates_fit && (((size_t)mixed | (size_t)out) & 31) == 0) {
        const long long groups = total / 8, want = (groups + 255) / 256;
        const int blocks = (int)(want < 65535LL * 4 ? want : 65535LL * 4);
        if (dtype == FE_F32)
            fe::launch(head_gate_vec_kernel<float>, blocks, 256, 0, stream, (const float*)mixed, (const float*)gates, ld, (float*)out, ldo,
                       groups, heads, head, vdim, per_element, scale);
        else
            fe::launch(head_gate_vec_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)mixed, (const bf16*)gates, ld, (bf16*)out, ldo,
                       groups, heads, head, vdim, per_element, scale);
        return fe_check_launch("head_gate");
    }
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 65535LL * 4 ? want : 65535LL * 4);
    if (dtype == FE_F32)
        fe::launch(head_gate_kernel<float>, blocks, 256, 0, stream, (const float*)mixed, (const float*)gates, ld, (float*)out, ldo, total,
                   heads, head, vdim, per_element, scale);
    else
        fe::launch(head_gate_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)mixed, (const bf16*)gates, ld, (bf16*)out, ldo, total,
                   heads, head, vdim, per_element, scale);
    return fe_check_launch("head_gate");
}

// ---------------------------------------------------------------------------------------------
// The minGRU recurrence.  zxg [T, 3 W] float holds, per token, the projections of the gate, the candidate and the output
// gate before their biases and activations:
//   z = sigmoid(zxg[:, c] + bias[c]);  u = zxg[:, W + c] + bias[W + c];  cand = u >= 0 ? u + 1/2 : sigmoid(u);
//   S <- (1 - z) S + z cand;   out = S * silu(zxg[:, 2 W + c]).
// S of a request lives in state[seat, :W] (zeros and nothing kept for a seat below 0).
namespace {

struct GruStep { float a, b; };      // S <- a S + b

__device__ __forceinline__ GruStep gru_step(float zl, float xl, float bz, float bx) {
    const float z = sigmoidf(zl + bz);
    const float u = xl + bx;
    const float cand = u >= 0.f ? u + 0.5f : sigmoidf(u);
    return GruStep{1.f - z, z * cand};
}
__device__ __forceinline__ float silu(float g) { return g * sigmoidf(g); }

constexpr int GRU_AHEAD = 8;         // tokens whose values are asked for together: the chain of S waits for memory once per 8

}  // namespace

// One thread per (request, channel) walks the request's tokens in order.
template <typename T>
__global__ void mingru_walk_kernel(const float* __restrict__ zxg, const float* __restrict__ bias, float* state, long long state_stride,
                                   const int* __restrict__ seats, const int* __restrict__ cu_q, T* __restrict__ out, int W, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int r = blockIdx.y;
    const int seat = seats[r];
    float* mine = (seat >= 0 && seat < n_seats) ? state + (size_t)seat * state_stride : nullptr;
    float S = mine ? mine[c] : 0.f;
    const float bz = bias[c], bx = bias[W + c];
    const int begin = cu_q[r], end = cu_q[r + 1];
    const size_t ld = (size_t)3 * W;
    for (int t0 = begin; t0 < end; t0 += GRU_AHEAD) {
        float zl[GRU_AHEAD], xl[GRU_AHEAD], gl[GRU_AHEAD];
#pragma unroll
        for (int i = 0; i < GRU_AHEAD; ++i) {
            const int t = min(t0 + i, end - 1);
            zl[i] = zxg[t * ld + c]; xl[i] = zxg[t * ld + W + c]; gl[i] = zxg[t * ld + 2 * W + c];
        }
#pragma unroll
        for (int i = 0; i < GRU_AHEAD; ++i) {
            if (t0 + i < end) {
                const GruStep s = gru_step(zl[i], xl[i], bz, bx);
                S = fmaf(s.a, S, s.b);
                out[(size_t)(t0 + i) * W + c] = from_float<T>(S * silu(gl[i]));
            }
        }
    }
    if (mine) mine[c] = S;
}

// Long portions: the recurrence is linear in S, so a request's tokens are cut into blocks of ``span``.  The first kernel
// folds every block into (A, B) with S_end = A S_begin + B and copies the kept state aside; the second starts every block
// from the S that the blocks before it give (folded in order from that copy), walks it and writes the outputs; the last
// block keeps S.  Scratch per request: [max_blocks][A | B][W], then the copy of the kept state [W].
__global__ void mingru_fold_kernel(const float* __restrict__ zxg, const float* __restrict__ bias, const float* __restrict__ state,
                                   long long state_stride, const int* __restrict__ seats, const int* __restrict__ cu_q,
                                   float* __restrict__ folds, int W, int span, int max_blocks, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int r = blockIdx.z, blk = blockIdx.y;
    const int begin = cu_q[r] + blk * span, end = min(cu_q[r + 1], begin + span);
    if (blk == 0) {
        const int seat = seats[r];
        folds[((size_t)r * (2 * max_blocks + 1) + 2 * max_blocks) * W + c] =
            (seat >= 0 && seat < n_seats) ? state[(size_t)seat * state_stride + c] : 0.f;
    }
    if (begin >= end) return;
    const float bz = bias[c], bx = bias[W + c];
    const size_t ld = (size_t)3 * W;
    float A = 1.f, B = 0.f;
    for (int t0 = begin; t0 < end; t0 += GRU_AHEAD) {
        float zl[GRU_AHEAD], xl[GRU_AHEAD];
#pragma unroll
        for (int i = 0; i < GRU_AHEAD; ++i) {
            const int t = min(t0 + i, end - 1);
            zl[i] = zxg[t * ld + c]; xl[i] = zxg[t * ld + W + c];
        }
#pragma unroll
        for (int i = 0; i < GRU_AHEAD; ++i) {
            if (t0 + i < end) {
                const GruStep s = gru_step(zl[i], xl[i], bz, bx);
                A *= s.a;
                B = fmaf(s.a, B, s.b);
            }
        }
    }
    float* f = folds + ((size_t)r * (2 * max_blocks + 1) + 2 * blk) * W;
    f[c] = A;
    f[W + c] = B;
}

template <typename T>
__global__ void mingru_blocks_kernel(const float* __restrict__ zxg, const float* __restrict__ bias, float* state, long long state_stride,
                                     const int* __restrict__ seats, const int* __restrict__ cu_q, const float* __restrict__ folds,
                                     T* __restrict__ out, int W, int span, int max_blocks, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int r = blockIdx.z, blk = blockIdx.y;
    const int begin = cu_q[r] + blk * span, last = cu_q[r + 1], end = min(last, begin + span);
    if (begin >= end) return;
    const int seat = seats[r];
    float* mine = (seat >= 0 && seat < n_seats) ? state + (size_t)seat * state_stride : nullptr;
    // the kept state is read from the copy the kernel before made: the request's last block overwrites the original, and it
    // may be done before another block of the request has begun
    const float* f = folds + (size_t)r * (2 * max_blocks + 1) * W;
    float S = f[(size_t)2 * max_blocks * W + c];
    for (int b = 0; b < blk; ++b) S = fmaf(f[(size_t)b * 2 * W + c], S, f[(size_t)b * 2 * W + W + c]);
    const float bz = bias[c], bx = bias[W + c];
    const size_t ld = (size_t)3 * W;
    for (int t0 = begin; t0 < end; t0 += GRU_AHEAD) {
        float zl[GRU_AHEAD], xl[GRU_AHEAD], gl[GRU_AHEAD];
#pragma unroll
        for (int i = 0; i < GRU_AHEAD; ++i) {
            const int t = min(t0 + i, end - 1);
            zl[i] = zxg[t * ld + c]; xl[i] = zxg[t * ld + W + c]; gl[i] = zxg[t * ld + 2 * W + c];
        }
#pragma unroll
        for (int i = 0; i < GRU_AHEAD; ++i) {
            if (t0 + i < end) {
                const GruStep s = gru_step(zl[i], xl[i], bz, bx);
                S = fmaf(s.a, S, s.b);
                out[(size_t)(t0 + i) * W + c] = from_float<T>(S * silu(gl[i]));
            }
        }
    }
    if (mine && end == last) mine[c] = S;
}

// Floats of scratch the blocked form needs: (A, B) per request, block and channel, and a copy of every request's state.
extern "C" long long fe_mingru_scan_scratch_floats(int requests, int W, int max_q_len, int span) {
    if (span <= 0 || max_q_len <= span) return 0;
    return (long long)requests * (2 * ((max_q_len + span - 1) / span) + 1) * W;
}

// ``span`` > 0 and ``max_q_len`` > span: the blocked form over blocks of ``span`` tokens (``folds``: scratch); else one walk.
extern "C" int fe_mingru_scan(const float* zxg, const float* bias, float* state, long long state_stride, const int* seats,
                              const int* cu_q, void* out, int requests, int W, int n_seats, int max_q_len, int span, float* folds,
                              int dtype, cudaStream_t stream) {
    FE_REQUIRE(requests >= 0 && W > 0 && n_seats >= 0 && state_stride >= W, "mingru_scan: bad sizes");
    FE_REQUIRE(dtype == FE_F32 || dtype == FE_BF16, "mingru_scan: unknown dtype %d", dtype);
    if (requests == 0) return 0;
    const int threads = 128;
    const int columns = (W + threads - 1) / threads;
    FE_REQUIRE(requests <= 65535, "mingru_scan: too many requests");
    if (span > 0 && max_q_len > span) {
        FE_REQUIRE(folds != nullptr, "mingru_scan: the blocked form needs scratch memory");
        const int max_blocks = (max_q_len + span - 1) / span;
        FE_REQUIRE(max_blocks <= 65535, "mingru_scan: too many blocks of tokens");
        const dim3 grid(columns, max_blocks, requests);
        fe::launch(mingru_fold_kernel, grid, threads, 0, stream, zxg, bias, (const float*)state, state_stride, seats, cu_q, folds, W, span,
                   max_blocks, n_seats);
        if (fe_check_launch("mingru_scan fold")) return 1;
        if (dtype == FE_F32)
            fe::launch(mingru_blocks_kernel<float>, grid, threads, 0, stream, zxg, bias, state, state_stride, seats, cu_q,
                       (const float*)folds, (float*)out, W, span, max_blocks, n_seats);
        else
            fe::launch(mingru_blocks_kernel<bf16>, grid, threads, 0, stream, zxg, bias, state, state_stride, seats, cu_q,
                       (const float*)folds, (bf16*)out, W, span, max_blocks, n_seats);
        return fe_check_launch("mingru_scan blocks");
    }
    const dim3 grid(columns, requests);
    if (dtype == FE_F32)
        fe::launch(mingru_walk_kernel<float>, grid, threads, 0, stream, zxg, bias, state, state_stride, seats, cu_q, (float*)out, W, n_seats);
    else
        fe::launch(mingru_walk_kernel<bf16>, grid, threads, 0, stream, zxg, bias, state, state_stride, seats, cu_q, (bf16*)out, W, n_seats);
    return fe_check_launch("mingru_scan");
}

// ---------------------------------------------------------------------------------------------
// out = act(gate) * up with gate_up = [gate | up] per row; act 0: silu, 1: the tanh form of GELU,
//   gelu(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long total, int I, int act) {
    griddep_wait();
    griddep_launch_dependents();
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long t = e / I;
        const int j = (int)(e - t * I);
        const float g = to_float(gate_up[t * 2 * I + j]), u = to_float(gate_up[t * 2 * I + I + j]);
        const float a = act == 0 ? silu(g) : 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
        out[e] = from_float<T>(a * u);
    }
}

extern "C" int fe_gated_activation(const void* gate_up, void* out, int T, int I, int act, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && I > 0 && (act == 0 || act == 1), "gated_activation: bad sizes or activation %d", act);
    const long long total = (long long)T * I;
    if (total == 0) return 0;
    const long long want = (total + 255) / 256;
    const int blocks = (int)(want < 65535LL * 8 ? want : 65535LL * 8);
    if (dtype == FE_F32)
        fe::launch(gated_activation_kernel<float>, blocks, 256, 0, stream, (const float*)gate_up, (float*)out, total, I, act);
    else if (dtype == FE_BF16)
        fe::launch(gated_activation_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)gate_up, (bf16*)out, total, I, act);
    else
        FE_REQUIRE(false, "gated_activation: unknown dtype %d", dtype);
    return fe_check_launch("gated_activation");
}
