// A linear-recurrent mixer with a matrix state per head (key channel x value channel) and a decay per key channel
// that depends on the token:
//   blends   x_s = h + (h' - h) * mu_s, h' the row of the token before (s = r, k, v, g, w)
//   decay    w_t = exp(-exp(logit_t + w0))                              (float)
//   output   o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j])
//   state    S[i][j] <- w_t[i] S[i][j] + k_t[i] v_t[j]                  (float, carried from step to step per request)
//   finish   y = o / rms(o per head) * weight * silu(g)
// The projections r, k, v, g come in the compute type; everything else here is float.
#define FE_PDL_CLASS 128
#include "common.cuh"

using namespace fe;

// ---------------------------------------------------------------------------------------------
// Blocks (token, stretch of columns): one column a thread in a step of few tokens, so that a handful of rows is still
// a few dozen blocks.  ``state`` rows are seats; the kept row of a seat (the last normalised input of the step before)
// starts at ``offset`` floats into its row.  The block of a request's first token reads the kept row and writes the
// request's last row of this step in its place, element by element in the same thread, so nobody else touches it.
template <typename T>
__global__ void token_shift_blend_kernel(const T* __restrict__ h, const float* __restrict__ mu, float* state,
                                         long long state_stride, long long offset, const int* __restrict__ seats,
                                         const int* __restrict__ cu_q, const int* __restrict__ token_req,
                                         T* __restrict__ blends, float* __restrict__ blend_w, int T_tokens, int D, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    const int t = blockIdx.x;
    const int r = token_req[t];
    const int first = cu_q[r];
    const int seat = seats[r];
    const bool seated = seat >= 0 && seat < n_seats;
    float* kept = seated ? state + (size_t)seat * state_stride + offset : nullptr;
    const T* row = h + (size_t)t * D;
    const T* prev = t > first ? h + (size_t)(t - 1) * D : nullptr;
    const T* last = h + (size_t)(cu_q[r + 1] - 1) * D;
    const size_t plane = (size_t)T_tokens * D;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < D; j += gridDim.y * blockDim.x) {
        const float x = to_float(row[j]);
        float before;
        if (prev) before = to_float(prev[j]);
        else if (kept) {
            before = kept[j];
            kept[j] = to_float(last[j]);
        } else before = 0.f;
        const float diff = before - x;
        const size_t at = (size_t)t * D + j;
#pragma unroll
        for (int s = 0; s < 4; ++s) blends[s * plane + at] = from_float<T>(fmaf(diff, mu[(size_t)s * D + j], x));
        blend_w[at] = fmaf(diff, mu[(size_t)4 * D + j], x);
    }
}

extern "C" int fe_token_shift_blend(const void* h, const float* mu, float* state, long long state_stride, long long offset,
                                    const int* seats, const int* cu_q, const int* token_req, void* blends, float* blend_w,
                                    int T, int D, int n_seats, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && D > 0 && n_seats >= 0 && offset >= 0 && offset + D <= state_stride, "token_shift_blend: bad sizes");
    if (T == 0) return 0;
    const int threads = D >= 1024 ? 256 : 128;
    const int stretches = T >= 512 ? 1 : (D + threads - 1) / threads;
    const dim3 grid(T, stretches < 65535 ? stretches : 65535);
    if (dtype == FE_F32)
        fe::launch(token_shift_blend_kernel<float>, grid, threads, 0, stream, (const float*)h, mu, state, state_stride, offset, seats,
                   cu_q, token_req, (float*)blends, blend_w, T, D, n_seats);
    else if (dtype == FE_BF16)
        fe::launch(token_shift_blend_kernel<bf16>, grid, threads, 0, stream, (const bf16*)h, mu, state, state_stride, offset, seats,
                   cu_q, token_req, (bf16*)blends, blend_w, T, D, n_seats);
    else
        FE_REQUIRE(false, "token_shift_blend: unknown dtype %d", dtype);
    return fe_check_launch("token_shift_blend");
}

// ---------------------------------------------------------------------------------------------
// The recurrence.  The value channels of a head do not depend on one another, so a block owns a slice of them: one
// block per (request, head, slice), a warp per 8 value channels of the slice.  The lanes of a warp are 8 groups of key
// channels x 4 pairs of value channels; a thread keeps IPT key channels x 2 value channels of the state in registers
// (head size <= 8 IPT; channels beyond the head size are zeros that change nothing).  Tokens are walked in tiles of
// WKV_TILE: r, k and the decay of all key channels and v of the slice lie in shared memory, the next tile's values are
// already on their way from global memory into registers while this one is walked, and the eight partial sums of an
// output meet through three shuffles.  How many slices a head is cut into is chosen so that the blocks about fill the
// device (a prompt of one request) or is one (a decode step of many requests).  A seat below 0 (a padding request)
// starts from zero and keeps nothing.
constexpr int WKV_TILE = 8;

template <typename T, int IPT, int PER, bool TWO, int G>
__global__ void __launch_bounds__(512) wkv_recurrence_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                                      const float* __restrict__ logits, const float* __restrict__ w0,
                                      const float* __restrict__ u, float* state, long long state_stride,
                                      const int* __restrict__ seats, const int* __restrict__ cu_q, float* __restrict__ out,
                                      int heads, int d, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    constexpr int GP = IPT + 4;                   // a group's stretch in shared memory, padded against bank conflicts
    constexpr int ROW = G * GP;                   // G groups of key channels a warp (8 or 16)
    constexpr int LANES_J = 32 / G;               // lanes of a group: value channels side by side
    extern __shared__ __align__(16) float smem[];
    float* rs = smem;                             // [TILE][ROW]
    float* ks = rs + WKV_TILE * ROW;
    float* ws = ks + WKV_TILE * ROW;
    float* vs = ws + WKV_TILE * ROW;              // [TILE][columns of this block]
    const int req = blockIdx.x, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int WARP_COLUMNS = LANES_J * (TWO ? 2 : 1);     // TWO: a thread owns two value channels, else one (half the chain a token)
    const int columns = (blockDim.x >> 5) * WARP_COLUMNS;    // value channels of this block
    const int j0 = blockIdx.z * columns;
    const int group = lane / LANES_J;
    const int local = warp * WARP_COLUMNS + (lane % LANES_J) * (TWO ? 2 : 1);  // this thread's value channels within the block's slice
    const int j = j0 + local;
    const bool own0 = j < d, own1 = TWO && j + 1 < d;
    const int seat = seats[req];
    const bool seated = seat >= 0 && seat < n_seats;
    float* mine = seated ? state + (size_t)seat * state_stride + (size_t)head * d * d : nullptr;
    const int inner = heads * d;
    float S0[IPT], S1[IPT], bonus[IPT];
#pragma unroll
    for (int x = 0; x < IPT; ++x) {
        const int i = group * IPT + x;
        S0[x] = (own0 && i < d && mine) ? mine[(size_t)i * d + j] : 0.f;
        S1[x] = (own1 && i < d && mine) ? mine[(size_t)i * d + j + 1] : 0.f;
        bonus[x] = i < d ? u[head * d + i] : 0.f;
    }
    for (int e = threadIdx.x; e < 3 * WKV_TILE * ROW + WKV_TILE * columns; e += blockDim.x) smem[e] = 0.f;
    const int begin = cu_q[req], end = cu_q[req + 1];
    // what a thread stages of a tile: elements e = threadIdx.x + n blockDim.x of [TILE][d] (r, k, decay) and of
    // [TILE][columns] (v).  Where they lie does not depend on the tile, so it is worked out once; the loads of a tile are
    // unconditional (an element beyond the tile's end reads the tile's first token again) and nothing is done with
    // what they bring until the tile is staged, so that all of them are in flight together while the tile before is walked.
    constexpr int PV = (PER + 3) / 4 + 1;
    int from[PER], to[PER], token[PER], vfrom[PV], vtoken[PV];
    float base[PER];
    T raw_r[PER], raw_k[PER], raw_v[PV];
    float raw_w[PER];
#pragma unroll
    for (int n = 0; n < PER; ++n) {
        const int e = threadIdx.x + n * blockDim.x;
        const int tt = e / d, i = e - tt * d;
        token[n] = tt < WKV_TILE ? tt : WKV_TILE;                  // WKV_TILE: never staged
        from[n] = tt < WKV_TILE ? tt * inner + i : 0;
        to[n] = tt * ROW + (i / IPT) * GP + i % IPT;
        base[n] = w0[head * d + i];
    }
#pragma unroll
    for (int n = 0; n < PV; ++n) {
        const int e = threadIdx.x + n * blockDim.x;
        const int tt = e / columns, c = e - tt * columns;
        const bool real = tt < WKV_TILE && j0 + c < d;
        vtoken[n] = real ? tt : WKV_TILE;
        vfrom[n] = real ? tt * inner + j0 + c : 0;
    }
    auto fetch = [&](int t0) {
        const int count = min(WKV_TILE, end - t0);
        const size_t origin = (size_t)t0 * inner + (size_t)head * d;
#pragma unroll
        for (int n = 0; n < PER; ++n) {
            const size_t at = origin + (token[n] < count ? from[n] : 0);
            raw_r[n] = r[at];
            raw_k[n] = k[at];
            raw_w[n] = logits[at];
        }
#pragma unroll
        for (int n = 0; n < PV; ++n) raw_v[n] = v[origin + (vtoken[n] < count ? vfrom[n] : 0)];
    };
    auto stage = [&](int t0) {
        const int count = min(WKV_TILE, end - t0);
#pragma unroll
        for (int n = 0; n < PER; ++n) {
            if (token[n] < count) {
                rs[to[n]] = to_float(raw_r[n]);
                ks[to[n]] = to_float(raw_k[n]);
                ws[to[n]] = expf(-expf(raw_w[n] + base[n]));
            }
        }
#pragma unroll
        for (int n = 0; n < PV; ++n) {
            const int e = threadIdx.x + n * blockDim.x;
            if (vtoken[n] < count) vs[e] = to_float(raw_v[n]);
        }
    };
    if (begin < end) fetch(begin);
    __syncthreads();                              // the zeros are written
    for (int t0 = begin; t0 < end; t0 += WKV_TILE) {
        const int count = min(WKV_TILE, end - t0);
        stage(t0);
        __syncthreads();
        if (t0 + WKV_TILE < end) fetch(t0 + WKV_TILE);
        auto walk = [&](int tt) {
            float2 vj;
            if (TWO) vj = *reinterpret_cast<const float2*>(vs + tt * columns + local);
            else vj = make_float2(vs[tt * columns + local], 0.f);
            const float* rt = rs + tt * ROW + group * GP;
            const float* kt = ks + tt * ROW + group * GP;
            const float* wt = ws + tt * ROW + group * GP;
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int x = 0; x < IPT; x += 4) {
                const float4 r4 = *reinterpret_cast<const float4*>(rt + x);
                const float4 k4 = *reinterpret_cast<const float4*>(kt + x);
                const float4 w4 = *reinterpret_cast<const float4*>(wt + x);
                const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    const float kv0 = kk[y] * vj.x, kv1 = kk[y] * vj.y;
                    acc0 = fmaf(rr[y], fmaf(bonus[x + y], kv0, S0[x + y]), acc0);
                    S0[x + y] = fmaf(ww[y], S0[x + y], kv0);
                    if (TWO) {
                        acc1 = fmaf(rr[y], fmaf(bonus[x + y], kv1, S1[x + y]), acc1);
                        S1[x + y] = fmaf(ww[y], S1[x + y], kv1);
                    }
                }
            }
#pragma unroll
            for (int o = LANES_J; o < 32; o <<= 1) {
                acc0 += __shfl_xor_sync(0xffffffffu, acc0, o);
                if (TWO) acc1 += __shfl_xor_sync(0xffffffffu, acc1, o);
            }
            if (group == 0) {
                float* o = out + (size_t)(t0 + tt) * inner + (size_t)head * d + j;
                if (own0) o[0] = acc0;
                if (own1) o[1] = acc1;
            }
        };
        if (count == WKV_TILE) {
#pragma unroll
            for (int tt = 0; tt < WKV_TILE; ++tt) walk(tt);       // unrolled: a token's shuffles overlap the next token's products
        } else {
            for (int tt = 0; tt < count; ++tt) walk(tt);
        }
        __syncthreads();                          // everyone is done with this tile before the next one is staged
    }
    if (mine) {
#pragma unroll
        for (int x = 0; x < IPT; ++x) {
            const int i = group * IPT + x;
            if (i < d && own0) mine[(size_t)i * d + j] = S0[x];
            if (i < d && own1) mine[(size_t)i * d + j + 1] = S1[x];
        }
    }
}

template <typename T, int IPT, int G>
static int launch_wkv(const void* r, const void* k, const void* v, const float* logits, const float* w0, const float* u,
                      float* state, long long state_stride, const int* seats, const int* cu_q, float* out, int requests,
                      int heads, int d, int n_seats, cudaStream_t stream) {
    // A warp per 8 value channels (two a thread) when the step has blocks to fill the device several times over, else per 4
    // (one a thread): a block walks its tokens one after the other, so with few blocks what counts is how long one warp
    // needs for a token, and half the channels are half the chain (one prompt of 2,048 tokens, 32 heads of 64: 0.42 ms with
    // two a thread).  A head is cut into slices until the blocks about fill the device twice, but a block keeps four warps
    // at least: every block stages r, k and the decay of all key channels for itself (one value channel a thread: four
    // slices of four warps 0.34 ms, two of eight 0.53).
    const long long units = (long long)requests * heads;
    const bool two = G == 8 && units >= 4LL * fe_sm_count();
    const int warp_columns = (32 / G) * (two ? 2 : 1);
    const int head_warps = (d + warp_columns - 1) / warp_columns;
    const int most = head_warps / 4 > 1 ? head_warps / 4 : 1;      // a block keeps four warps at least (two: 0.55 ms)
    int slices = (int)((2LL * fe_sm_count() + units - 1) / units);
    slices = slices < 1 ? 1 : (slices > most ? most : slices);
    int warps = (head_warps + slices - 1) / slices;
    if (warps > 16) warps = 16;                                    // 512 threads a block
    slices = (head_warps + warps - 1) / warps;
    // a thread stages at most PER elements of r, k and the decay of a tile: TILE x d over 32 x warps threads
    const int need = (WKV_TILE * d + warps * 32 - 1) / (warps * 32);
    const size_t smem = ((size_t)3 * WKV_TILE * G * (IPT + 4) + (size_t)WKV_TILE * warps * warp_columns) * sizeof(float);
#define FE_WKV_LAUNCH2(PER, TWO)                                                                                                       \
    fe::launch(wkv_recurrence_kernel<T, IPT, PER, TWO, G>, dim3(requests, heads, slices), warps * 32, smem, stream, (const T*)r, (const T*)k, \
               (const T*)v, logits, w0, u, state, state_stride, seats, cu_q, out, heads, d, n_seats)
#define FE_WKV_LAUNCH(PER)             \
    do {                               \
        if (G == 8 && two) FE_WKV_LAUNCH2(PER, (G == 8)); \
        else FE_WKV_LAUNCH2(PER, false);    \
    } while (0)
    if (need <= 2) FE_WKV_LAUNCH(2);
    else if (need <= 4) FE_WKV_LAUNCH(4);
    else if (need <= 8) FE_WKV_LAUNCH(8);
    else if (need <= 16) FE_WKV_LAUNCH(16);
    else FE_WKV_LAUNCH(32);
#undef FE_WKV_LAUNCH
#undef FE_WKV_LAUNCH2
    return fe_check_launch("wkv_recurrence");
}

template <typename T>
static int dispatch_wkv(const void* r, const void* k, const void* v, const float* logits, const float* w0, const float* u,
                        float* state, long long state_stride, const int* seats, const int* cu_q, float* out, int requests,
                        int heads, int d, int n_seats, cudaStream_t stream) {
#define FE_WKV(IPT, G) return launch_wkv<T, IPT, G>(r, k, v, logits, w0, u, state, state_stride, seats, cu_q, out, requests, heads, d, n_seats, stream)
    // (sixteen groups of key channels a warp, two value channels across, were measured too: 0.61 against 0.34 ms)
    if (d <= 32) FE_WKV(4, 8);
    if (d <= 64) FE_WKV(8, 8);
    FE_WKV(16, 8);
#undef FE_WKV
}

extern "C" int fe_wkv_recurrence(const void* r, const void* k, const void* v, const float* logits, const float* w0,
                                 const float* u, float* state, long long state_stride, const int* seats, const int* cu_q,
                                 float* out, int requests, int heads, int d, int n_seats, int dtype, cudaStream_t stream) {
    FE_REQUIRE(requests >= 0 && heads > 0 && d > 0 && d <= 128 && n_seats >= 0 && (long long)heads * d * d <= state_stride,
               "wkv_recurrence: bad sizes (heads %d, head size %d; head sizes up to 128)", heads, d);
    FE_REQUIRE(heads <= 65535 && requests <= 2147483647, "wkv_recurrence: too many heads (%d)", heads);
    if (requests == 0) return 0;
    if (dtype == FE_F32)
        return dispatch_wkv<float>(r, k, v, logits, w0, u, state, state_stride, seats, cu_q, out, requests, heads, d, n_seats, stream);
    if (dtype == FE_BF16)
        return dispatch_wkv<bf16>(r, k, v, logits, w0, u, state, state_stride, seats, cu_q, out, requests, heads, d, n_seats, stream);
    FE_REQUIRE(false, "wkv_recurrence: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------------
// y[t, head] = o[t, head] / sqrt(mean(o[t, head]^2) + eps) * weight * silu(g) * scale: one warp per (token, head).
// ``weight`` may be null (a unit norm).  A row of g is ldg entries long and a row of out ldo (views of wider buffers).
template <typename T>
__global__ void head_rmsnorm_gate_kernel(const float* __restrict__ o, const float* __restrict__ weight, const T* __restrict__ g,
                                         long long ldg, T* __restrict__ out, long long ldo, float eps, float scale, long long pairs,
                                         int heads, int d) {
    griddep_wait();
    griddep_launch_dependents();
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (warp >= pairs) return;
    const int lane = threadIdx.x & 31;
    const int head = (int)(warp % heads);
    const long long t = warp / heads;
    const float* x = o + warp * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)d + eps) * scale;
    for (int i = lane; i < d; i += 32) {
        const float gate = to_float(g[t * ldg + head * d + i]);
        const float w = weight ? weight[head * d + i] : 1.f;
        out[t * ldo + head * d + i] = from_float<T>(x[i] * inv * w * (gate / (1.f + expf(-gate))));
    }
}

extern "C" int fe_head_rmsnorm_gate(const float* o, const float* weight, const void* g, long long ldg, void* out, long long ldo, float eps,
                                    float scale, int T, int heads, int d, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && heads > 0 && d > 0 && ldg >= (long long)heads * d && ldo >= (long long)heads * d, "head_rmsnorm_gate: bad sizes");
    if (T == 0) return 0;
    const long long pairs = (long long)T * heads;
    const unsigned blocks = (unsigned)((pairs + 3) / 4);
    if (dtype == FE_F32)
        fe::launch(head_rmsnorm_gate_kernel<float>, blocks, 128, 0, stream, o, weight, (const float*)g, ldg, (float*)out, ldo, eps, scale,
                   pairs, heads, d);
    else if (dtype == FE_BF16)
        fe::launch(head_rmsnorm_gate_kernel<bf16>, blocks, 128, 0, stream, o, weight, (const bf16*)g, ldg, (bf16*)out, ldo, eps, scale,
                   pairs, heads, d);
    else
        FE_REQUIRE(false, "head_rmsnorm_gate: unknown dtype %d", dtype);
    return fe_check_launch("head_rmsnorm_gate");
}
