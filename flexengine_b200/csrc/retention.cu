// Retention: linear attention with one fixed decay per head, no softmax and no denominator.
//   S_t = a_h S_(t-1) + k_t v_t^T ;   o_t = S_t^T q_t          S [d, dv] float per request and head
// Kernels (all arithmetic float):
//   rotate_heads      float rows of heads from a projection: the first ``rot`` entries of a head turned by
//                     position * inv_freq (pairs i, i + rot/2), runs of heads times a factor each
//   retention_scan    the recurrence token by token over the step's portions, the state in registers
//   retention_chunks  the same for long portions in blocks of tokens: inside a block of C tokens
//                       o_a = a^(a+1) S_0^T q_a + sum_(b <= a) a^(a-b) (q_a . k_b) v_b
//                       S_C = a^C S_0 + sum_b a^(C-1-b) k_b v_b^T
//                     so that the blocks of a portion are summed independently and then chained
//   retention_decode  a step of one token a request: rotation, recurrence, the head's unit norm and the gate in one kernel
#define FE_PDL_CLASS 128
#include "common.cuh"

using namespace fe;

namespace {

// ---------------------------------------------------------------------------------------------
// One thread per (token, head, pair of turned entries or entry that passes).
template <typename T>
__global__ void rotate_heads_kernel(const T* __restrict__ proj, long long ld, const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int rot, float* __restrict__ out, long long total, int heads,
                                    int dim, int first_heads, float first_scale, float rest_scale) {
    griddep_wait();
    griddep_launch_dependents();
    const int half = rot >> 1;
    const int per_head = dim - half;                       // pairs, then the entries behind the turned ones
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(e % per_head);
        const long long th = e / per_head;
        const int h = (int)(th % heads);
        const long long t = th / heads;
        const float f = h < first_heads ? first_scale : rest_scale;
        const T* src = proj + t * ld + (long long)h * dim;
        float* dst = out + (t * heads + h) * dim;
        if (c < half) {
            float s, co;
            sincosf((float)positions[t] * inv_freq[c], &s, &co);
            const float a = to_float(src[c]), b = to_float(src[c + half]);
            dst[c] = (a * co - b * s) * f;
            dst[c + half] = (b * co + a * s) * f;
        } else {
            dst[c + half] = to_float(src[c + half]) * f;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The recurrence token by token.  A block owns a slice of the value channels of one (request, head); the lanes of a warp
// are 8 groups of key channels x 4 value channels; a thread keeps IPT key channels of one value channel of the state in
// registers (d <= 8 IPT; channels beyond d are zeros).  Tokens are walked in tiles of SCAN_TILE staged in shared memory.
constexpr int SCAN_TILE = 8;

template <typename TV, int IPT>
__global__ void __launch_bounds__(512)
retention_scan_kernel(const float* __restrict__ qk, const TV* __restrict__ values, long long ldv, const float* __restrict__ decay,
                      float* state, long long state_stride, const int* __restrict__ seats, const int* __restrict__ cu_q,
                      float* __restrict__ out, int heads, int d, int dv, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    constexpr int GP = IPT + 4;
    constexpr int ROW = 8 * GP;
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;                             // [TILE][ROW]
    float* ks = qs + SCAN_TILE * ROW;
    float* vs = ks + SCAN_TILE * ROW;             // [TILE][columns]
    const int req = blockIdx.x, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int columns = (blockDim.x >> 5) * 4;
    const int j0 = blockIdx.z * columns;
    const int group = lane >> 2;
    const int local = warp * 4 + (lane & 3);
    const int j = j0 + local;
    const bool own = j < dv;
    const int seat = seats[req];
    float* mine = (seat >= 0 && seat < n_seats) ? state + (size_t)seat * state_stride + (size_t)head * d * dv : nullptr;
    const float a = decay[head];
    float S[IPT];
#pragma unroll
    for (int x = 0; x < IPT; ++x) {
        const int i = group * IPT + x;
        S[x] = (own && i < d && mine) ? mine[(size_t)i * dv + j] : 0.f;
    }
    for (int e = threadIdx.x; e < 2 * SCAN_TILE * ROW + SCAN_TILE * columns; e += blockDim.x) smem[e] = 0.f;
    const int begin = cu_q[req], end = cu_q[req + 1];
    const long long row = 2LL * heads * d;
    __syncthreads();
    for (int t0 = begin; t0 < end; t0 += SCAN_TILE) {
        const int count = min(SCAN_TILE, end - t0);
        for (int e = threadIdx.x; e < count * d; e += blockDim.x) {
            const int tt = e / d, i = e - tt * d;
            const float* src = qk + (size_t)(t0 + tt) * row + (size_t)head * d + i;
            const int to = tt * ROW + (i / IPT) * GP + i % IPT;
            qs[to] = src[0];
            ks[to] = src[(size_t)heads * d];
        }
        for (int e = threadIdx.x; e < count * columns; e += blockDim.x) {
            const int tt = e / columns, c = e - tt * columns;
            if (j0 + c < dv) vs[e] = to_float(values[(size_t)(t0 + tt) * ldv + (size_t)head * dv + j0 + c]);
        }
        __syncthreads();
        for (int tt = 0; tt < count; ++tt) {
            const float vj = vs[tt * columns + local];
            const float* qt = qs + tt * ROW + group * GP;
            const float* kt = ks + tt * ROW + group * GP;
            float acc = 0.f;
#pragma unroll
            for (int x = 0; x < IPT; x += 4) {
                const float4 q4 = *reinterpret_cast<const float4*>(qt + x);
                const float4 k4 = *reinterpret_cast<const float4*>(kt + x);
                const float qq[4] = {q4.x, q4.y, q4.z, q4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    S[x + y] = fmaf(a, S[x + y], kk[y] * vj);
                    acc = fmaf(qq[y], S[x + y], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            if (group == 0 && own) out[(size_t)(t0 + tt) * heads * dv + (size_t)head * dv + j] = acc;
        }
        __syncthreads();
    }
    if (mine && own) {
#pragma unroll
        for (int x = 0; x < IPT; ++x) {
            const int i = group * IPT + x;
            if (i < d) mine[(size_t)i * dv + j] = S[x];
        }
    }
}

template <typename TV, int IPT>
int launch_scan(const float* qk, const void* values, long long ldv, const float* decay, float* state, long long state_stride,
                const int* seats, const int* cu_q, float* out, int requests, int heads, int d, int dv, int n_seats, cudaStream_t stream) {
    // a head's value channels are cut into slices until the blocks about fill the device twice; a block keeps two warps at least
    const long long units = (long long)requests * heads;
    const int head_warps = (dv + 3) / 4;
    const int most = head_warps / 2 > 1 ? head_warps / 2 : 1;
    int slices = (int)((2LL * fe_sm_count() + units - 1) / units);
    slices = slices < 1 ? 1 : (slices > most ? most : slices);
    int warps = (head_warps + slices - 1) / slices;
    if (warps > 16) warps = 16;
    slices = (head_warps + warps - 1) / warps;
    const size_t smem = ((size_t)2 * SCAN_TILE * 8 * (IPT + 4) + (size_t)SCAN_TILE * warps * 4) * sizeof(float);
    fe::launch(retention_scan_kernel<TV, IPT>, dim3(requests, heads, slices), warps * 32, smem, stream, qk, (const TV*)values, ldv, decay,
               state, state_stride, seats, cu_q, out, heads, d, dv, n_seats);
    return fe_check_launch("retention_scan");
}

template <typename TV>
int dispatch_scan(const float* qk, const void* values, long long ldv, const float* decay, float* state, long long state_stride,
                  const int* seats, const int* cu_q, float* out, int requests, int heads, int d, int dv, int n_seats, cudaStream_t stream) {
#define FE_SCAN(IPT) return launch_scan<TV, IPT>(qk, values, ldv, decay, state, state_stride, seats, cu_q, out, requests, heads, d, dv, n_seats, stream)
    if (d <= 32) FE_SCAN(4);
    if (d <= 64) FE_SCAN(8);
    if (d <= 128) FE_SCAN(16);
    FE_SCAN(32);
#undef FE_SCAN
}

}  // namespace

// out float [T, heads dim]; proj [T, >= heads dim] with rows ld entries long; the first ``first_heads`` heads are multiplied by
// first_scale, the others by rest_scale.
extern "C" int fe_rotate_heads(const void* proj, long long ld, const int* positions, const float* inv_freq, int rot, float* out, int T,
                               int heads, int dim, int first_heads, float first_scale, float rest_scale, int dtype, cudaStream_t stream) {
    FE_REQUIRE(T >= 0 && heads > 0 && dim > 0 && rot >= 0 && rot % 2 == 0 && rot <= dim && ld >= (long long)heads * dim,
               "rotate_heads: bad sizes (heads %d of %d, %d turned)", heads, dim, rot);
    FE_REQUIRE(rot == 0 || inv_freq != nullptr, "rotate_heads: a rotation needs its frequencies");
    FE_REQUIRE(dtype == FE_F32 || dtype == FE_BF16, "rotate_heads: unknown dtype %d", dtype);
    const long long total = (long long)T * heads * (dim - rot / 2);
    if (total == 0) return 0;
    const long long want = (total + 255) / 256;
    const unsigned blocks = (unsigned)(want < 65535LL * 8 ? want : 65535LL * 8);
    if (dtype == FE_F32)
        fe::launch(rotate_heads_kernel<float>, blocks, 256, 0, stream, (const float*)proj, ld, positions, inv_freq, rot, out, total, heads,
                   dim, first_heads, first_scale, rest_scale);
    else
        fe::launch(rotate_heads_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)proj, ld, positions, inv_freq, rot, out, total, heads,
                   dim, first_heads, first_scale, rest_scale);
    return fe_check_launch("rotate_heads");
}

// qk float [T, 2 heads d] (queries, then keys); values [T, >= heads dv] in ``dtype`` with rows ldv entries long; decay float
// [heads]; state float [n_seats, >= heads d dv]; out float [T, heads dv].
extern "C" int fe_retention_scan(const float* qk, const void* values, long long ldv, const float* decay, float* state,
                                 long long state_stride, const int* seats, const int* cu_q, float* out, int requests, int heads, int d,
                                 int dv, int n_seats, int dtype, cudaStream_t stream) {
    FE_REQUIRE(requests >= 0 && heads > 0 && heads <= 65535 && d > 0 && d <= 256 && dv > 0 && n_seats >= 0 &&
                   (long long)heads * d * dv <= state_stride && ldv >= (long long)heads * dv,
               "retention_scan: bad sizes (heads %d, key size %d up to 256, value size %d)", heads, d, dv);
    FE_REQUIRE(dtype == FE_F32 || dtype == FE_BF16, "retention_scan: unknown dtype %d", dtype);
    if (requests == 0) return 0;
    if (dtype == FE_F32)
        return dispatch_scan<float>(qk, values, ldv, decay, state, state_stride, seats, cu_q, out, requests, heads, d, dv, n_seats, stream);
    return dispatch_scan<bf16>(qk, values, ldv, decay, state, state_stride, seats, cu_q, out, requests, heads, d, dv, n_seats, stream);
}
