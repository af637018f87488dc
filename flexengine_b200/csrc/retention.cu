// Retention: linear attention with one fixed decay per head, no softmax and no denominator.
//   S_t = a_h S_(t-1) + k_t v_t^T ;   o_t = S_t^T q_t          S [d, dv] float per request and head
// Kernels (all arithmetic float):
//   rotate_heads      float rows of heads from a projection: the first ``rot`` entries of a head turned by
//                     position * inv_freq (pairs i, i + rot/2), runs of heads times a factor each
//   retention_scan    the recurrence token by token over the step's portions, the state in registers
//   retention_chunks  the same for long portions in blocks of C = 64 tokens.  Inside a block that starts from S_0
//                       o_n = a^(n+1) S_0^T q_n + sum_(b <= n) a^(n-b) (q_n . k_b) v_b
//                       S_C = a^C S_0 + sum_b a^(C-1-b) k_b v_b^T
//                     so three launches do a step: every block's own sum of k v^T (independent of the others), the chain
//                     S_0 -> S_C -> ... over a portion's blocks (elementwise), and every block's outputs from the state
//                     before it (independent again).  The products are tiled 64 x 64 over shared memory, 4 x 4 a thread.
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
    float* dots = vs + SCAN_TILE * columns;       // [TILE] q_t . k_t
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
        // o_t = a S_(t-1)^T q_t + (q_t . k_t) v_t: the token's own share as ONE factor for all value channels, as the blocks of
        // tokens have it, so that a head whose q . k nearly cancels keeps its direction through the unit norm that follows
        for (int tt = warp; tt < count; tt += blockDim.x >> 5) {
            float dot = 0.f;
            for (int i = lane; i < d; i += 32) {
                const int at = tt * ROW + (i / IPT) * GP + i % IPT;
                dot = fmaf(qs[at], ks[at], dot);
            }
            dot = warp_sum(dot);
            if (lane == 0) dots[tt] = dot;
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
                    acc = fmaf(qq[y], S[x + y], acc);
                    S[x + y] = fmaf(a, S[x + y], kk[y] * vj);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            if (group == 0 && own) out[(size_t)(t0 + tt) * heads * dv + (size_t)head * dv + j] = fmaf(a, acc, dots[tt] * vj);
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
    const size_t smem = ((size_t)2 * SCAN_TILE * 8 * (IPT + 4) + (size_t)SCAN_TILE * warps * 4 + SCAN_TILE) * sizeof(float);
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


// ---------------------------------------------------------------------------------------------
// Long portions in blocks of CHUNK tokens.  Block c of request r has row cu_q[r] / CHUNK + r + c of ``sums``
// ([rows, heads d dv] float): the rows of different requests never meet, and T / CHUNK + requests rows hold a step.
constexpr int CHUNK = 64;                // tokens a block
constexpr int TILE = 64;                 // key channels or value channels a tile
constexpr int PITCH = CHUNK + 4;         // a transposed tile's row: float4 reads stay aligned, stores spread over banks
static_assert(CHUNK == TILE, "a block of tokens and a tile of channels are loaded by the same loops");

__device__ __forceinline__ size_t chunk_row(const int* __restrict__ cu_q, int r) { return (size_t)(cu_q[r] / CHUNK + r); }

// sums[row][head] <- sum_b a^(len-1-b) k_b v_b^T over the block's len tokens.  Grid (block of tokens, request,
// head x tile of key channels x tile of value channels), 256 threads as 16 x 16, a thread 4 key x 4 value channels.
template <typename TV>
__global__ void __launch_bounds__(256)
retention_chunk_sums_kernel(const float* __restrict__ qk, const TV* __restrict__ values, long long ldv, const float* __restrict__ decay,
                            const int* __restrict__ cu_q, float* __restrict__ sums, int heads, int d, int dv, int nd, int nv) {
    griddep_wait();
    griddep_launch_dependents();
    __shared__ __align__(16) float ks[CHUNK * TILE];
    __shared__ __align__(16) float vs[CHUNK * TILE];
    __shared__ float pw[CHUNK];
    const int c = blockIdx.x, r = blockIdx.y;
    int z = blockIdx.z;
    const int vt = z % nv;
    z /= nv;
    const int dt = z % nd, head = z / nd;
    const int begin = cu_q[r] + c * CHUNK, end = cu_q[r + 1];
    if (begin >= end) return;
    const int len = min(CHUNK, end - begin);
    const int tid = threadIdx.x;
    if (tid < CHUNK) pw[tid] = tid < len ? (float)pow((double)decay[head], (double)(len - 1 - tid)) : 0.f;
    __syncthreads();
    const size_t row = 2 * (size_t)heads * d;
    for (int e = tid; e < CHUNK * TILE; e += 256) {
        const int b = e / TILE, i = e - b * TILE;
        const int gi = dt * TILE + i, gj = vt * TILE + i;
        const bool in = b < len;
        ks[e] = (in && gi < d) ? pw[b] * qk[(size_t)(begin + b) * row + (size_t)heads * d + (size_t)head * d + gi] : 0.f;
        vs[e] = (in && gj < dv) ? to_float(values[(size_t)(begin + b) * ldv + (size_t)head * dv + gj]) : 0.f;
    }
    __syncthreads();
    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4] = {};
    for (int b = 0; b < len; ++b) {
        const float4 k4 = *reinterpret_cast<const float4*>(ks + b * TILE + ty * 4);
        const float4 v4 = *reinterpret_cast<const float4*>(vs + b * TILE + tx * 4);
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) acc[x][y] = fmaf(kk[x], vv[y], acc[x][y]);
    }
    float* to = sums + ((chunk_row(cu_q, r) + c) * heads + head) * (size_t)d * dv;
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        const int gi = dt * TILE + ty * 4 + x;
        if (gi >= d) continue;
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            const int gj = vt * TILE + tx * 4 + y;
            if (gj < dv) to[(size_t)gi * dv + gj] = acc[x][y];
        }
    }
}

// One thread an entry of the state: S walks the portion's blocks, leaving in each block's row what S was BEFORE that
// block in place of the block's sum, and ends in the seat.
__global__ void __launch_bounds__(256)
retention_chunk_chain_kernel(const float* __restrict__ decay, float* state, long long state_stride, const int* __restrict__ seats,
                             const int* __restrict__ cu_q, float* sums, int heads, int d, int dv, int n_seats) {
    griddep_wait();
    griddep_launch_dependents();
    const int r = blockIdx.x;
    const size_t per = (size_t)heads * d * dv;
    const size_t e = (size_t)blockIdx.y * blockDim.x + threadIdx.x;
    const int n = cu_q[r + 1] - cu_q[r];
    if (e >= per || n <= 0) return;
    const int head = (int)(e / ((size_t)d * dv));
    const int blocks = (n + CHUNK - 1) / CHUNK;
    const double a = (double)decay[head];
    const float whole = (float)pow(a, (double)CHUNK), last = (float)pow(a, (double)(n - (blocks - 1) * CHUNK));
    const int seat = seats[r];
    float* mine = (seat >= 0 && seat < n_seats) ? state + (size_t)seat * state_stride + e : nullptr;
    float S = mine ? *mine : 0.f;
    float* p = sums + chunk_row(cu_q, r) * per + e;
    constexpr int AHEAD = 8;                      // the sums of so many blocks are asked for at once: the chain waits on memory
    for (int c0 = 0; c0 < blocks; c0 += AHEAD, p += AHEAD * per) {
        float u[AHEAD];
#pragma unroll
        for (int x = 0; x < AHEAD; ++x) u[x] = c0 + x < blocks ? __ldcs(p + x * per) : 0.f;
#pragma unroll
        for (int x = 0; x < AHEAD; ++x) {
            if (c0 + x >= blocks) break;
            p[x * per] = S;
            S = fmaf(c0 + x == blocks - 1 ? last : whole, S, u[x]);
        }
    }
    if (mine) *mine = S;
}

// A block's outputs for a tile of value channels: W = (Q K^T) with entry (n, b) times a^(n-b) where b <= n, else 0;
// out = diag(a^(n+1)) Q S_0 + W V.  Q, K and S_0 pass through shared memory in tiles of key channels; W takes the keys' place.
// Grid (block of tokens, request, head x tile of value channels), 256 threads as 16 x 16, a thread 4 tokens x 4 columns.
constexpr size_t CHUNK_OUT_SMEM = ((size_t)2 * TILE * PITCH + (size_t)TILE * TILE + (size_t)CHUNK * TILE + CHUNK + 4) * sizeof(float);

template <typename TV>
__global__ void __launch_bounds__(256)
retention_chunk_out_kernel(const float* __restrict__ qk, const TV* __restrict__ values, long long ldv, const float* __restrict__ decay,
                           const int* __restrict__ cu_q, const float* __restrict__ sums, float* __restrict__ out, int heads, int d, int dv,
                           int nd, int nv) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ __align__(16) float smem[];
    float* qT = smem;                            // [TILE][PITCH]: key channel i of token n at i * PITCH + n
    float* kT = qT + TILE * PITCH;               // the same of the keys; later W as [b][n]
    float* sS = kT + TILE * PITCH;               // [TILE][TILE] the state before the block, key channel x value channel
    float* vS = sS + TILE * TILE;                // [CHUNK][TILE]
    float* pw = vS + CHUNK * TILE;               // [CHUNK + 1] powers of the decay
    const int c = blockIdx.x, r = blockIdx.y;
    const int vt = blockIdx.z % nv, head = blockIdx.z / nv;
    const int begin = cu_q[r] + c * CHUNK, end = cu_q[r + 1];
    if (begin >= end) return;
    const int len = min(CHUNK, end - begin);
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    if (tid <= CHUNK) pw[tid] = (float)pow((double)decay[head], (double)tid);
    for (int e = tid; e < CHUNK * TILE; e += 256) {
        const int b = e / TILE, j = e - b * TILE, gj = vt * TILE + j;
        vS[e] = (b < len && gj < dv) ? to_float(values[(size_t)(begin + b) * ldv + (size_t)head * dv + gj]) : 0.f;
    }
    const size_t row = 2 * (size_t)heads * d;
    const float* before = sums + ((chunk_row(cu_q, r) + c) * heads + head) * (size_t)d * dv;
    float W[4][4] = {}, O[4][4] = {};
    for (int dt = 0; dt < nd; ++dt) {
        __syncthreads();
        for (int e = tid; e < CHUNK * TILE; e += 256) {
            const int n = e / TILE, i = e - n * TILE, gi = dt * TILE + i;
            const bool in = n < len && gi < d;
            const float* src = qk + (size_t)(begin + n) * row + (size_t)head * d + gi;
            qT[i * PITCH + n] = in ? src[0] : 0.f;
            kT[i * PITCH + n] = in ? src[(size_t)heads * d] : 0.f;
            const int gj = vt * TILE + i;                                       // here n walks key channels, i value channels
            sS[e] = (dt * TILE + n < d && gj < dv) ? before[(size_t)(dt * TILE + n) * dv + gj] : 0.f;
        }
        __syncthreads();
#pragma unroll 4
        for (int i = 0; i < TILE; ++i) {
            const float4 q4 = *reinterpret_cast<const float4*>(qT + i * PITCH + ty * 4);
            const float4 k4 = *reinterpret_cast<const float4*>(kT + i * PITCH + tx * 4);
            const float4 s4 = *reinterpret_cast<const float4*>(sS + i * TILE + tx * 4);
            const float qq[4] = {q4.x, q4.y, q4.z, q4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    W[x][y] = fmaf(qq[x], kk[y], W[x][y]);
                    O[x][y] = fmaf(qq[x], ss[y], O[x][y]);
                }
        }
    }
    __syncthreads();
#pragma unroll
    for (int y = 0; y < 4; ++y) {
        const int b = tx * 4 + y;
        float w[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int n = ty * 4 + x;
            w[x] = b <= n ? W[x][y] * pw[n - b] : 0.f;
        }
        *reinterpret_cast<float4*>(kT + b * PITCH + ty * 4) = make_float4(w[0], w[1], w[2], w[3]);
    }
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) O[x][y] *= pw[ty * 4 + x + 1];
    __syncthreads();
    const int seen = min(len, ty * 4 + 4);                                       // tokens after a thread's last one weigh nothing
    for (int b = 0; b < seen; ++b) {
        const float4 w4 = *reinterpret_cast<const float4*>(kT + b * PITCH + ty * 4);
        const float4 v4 = *reinterpret_cast<const float4*>(vS + b * TILE + tx * 4);
        const float ww[4] = {w4.x, w4.y, w4.z, w4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) O[x][y] = fmaf(ww[x], vv[y], O[x][y]);
    }
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        const int n = ty * 4 + x;
        if (n >= len) continue;
#pragma unroll
        for (int y = 0; y < 4; ++y) {
            const int gj = vt * TILE + tx * 4 + y;
            if (gj < dv) out[(size_t)(begin + n) * heads * dv + (size_t)head * dv + gj] = O[x][y];
        }
    }
}

template <typename TV>
int launch_chunks(const float* qk, const void* values, long long ldv, const float* decay, float* state, long long state_stride,
                  const int* seats, const int* cu_q, float* out, float* sums, int requests, int most_blocks, int heads, int d, int dv,
                  int n_seats, cudaStream_t stream) {
    static bool opted = false;
    if (!opted) {
        const cudaError_t err = cudaFuncSetAttribute(retention_chunk_out_kernel<TV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     (int)CHUNK_OUT_SMEM);
        FE_REQUIRE(err == cudaSuccess, "retention_chunks: %s", cudaGetErrorString(err));
        opted = true;
    }
    const int nd = (d + TILE - 1) / TILE, nv = (dv + TILE - 1) / TILE;
    const size_t per = (size_t)heads * d * dv;
    fe::launch(retention_chunk_sums_kernel<TV>, dim3(most_blocks, requests, heads * nd * nv), 256, 0, stream, qk, (const TV*)values, ldv,
               decay, cu_q, sums, heads, d, dv, nd, nv);
    fe::launch(retention_chunk_chain_kernel, dim3(requests, (unsigned)((per + 255) / 256)), 256, 0, stream, decay, state, state_stride,
               seats, cu_q, sums, heads, d, dv, n_seats);
    fe::launch(retention_chunk_out_kernel<TV>, dim3(most_blocks, requests, heads * nv), 256, CHUNK_OUT_SMEM, stream, qk, (const TV*)values,
               ldv, decay, cu_q, (const float*)sums, out, heads, d, dv, nd, nv);
    return fe_check_launch("retention_chunks");
}


// ---------------------------------------------------------------------------------------------
// A step of ONE token a request: rotation, recurrence, the head's unit norm and the gate in one kernel.  Block per
// (request, head); its threads are ``groups`` runs of key channels x ``columns`` value channels, so that the state's rows
// are read and written side by side and many of them are in flight; the runs' shares of S^T q meet in shared memory.
template <typename T>
__global__ void __launch_bounds__(1024)
retention_decode_kernel(const T* __restrict__ proj, long long ld, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                        int rot, float key_scale, const float* __restrict__ decay, float* state, long long state_stride,
                        const int* __restrict__ seats, T* __restrict__ out, long long ldo, float eps, float scale, int heads, int d,
                        int dv, int n_seats, int groups) {
    griddep_wait();
    griddep_launch_dependents();
    extern __shared__ __align__(16) float smem[];
    const int columns = blockDim.x / groups;
    float* qs = smem;                               // [d] rotated query
    float* ks = qs + d;                             // [d] rotated key, scaled
    float* os = ks + d;                             // [dv] the head's output before its norm
    float* part = os + dv;                          // [groups][columns]
    float* red = part + groups * columns;           // [33]
    const int r = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const T* row = proj + (size_t)r * ld;
    const T* qrow = row + (size_t)head * d;
    const T* krow = row + (size_t)heads * d + (size_t)head * d;
    const int half = rot >> 1;
    for (int i = tid; i < d; i += blockDim.x) {
        float q = to_float(qrow[i]), k = to_float(krow[i]);
        if (i < rot) {
            const bool low = i < half;
            const int other = low ? i + half : i - half;
            float sn, cs;
            sincosf((float)positions[r] * inv_freq[low ? i : i - half], &sn, &cs);
            const float qo = to_float(qrow[other]), ko = to_float(krow[other]);
            q = low ? q * cs - qo * sn : q * cs + qo * sn;
            k = low ? k * cs - ko * sn : k * cs + ko * sn;
        }
        qs[i] = q;
        ks[i] = k * key_scale;
    }
    __syncthreads();
    float dot = 0.f;
    for (int i = 0; i < d; ++i) dot = fmaf(qs[i], ks[i], dot);
    const int seat = seats[r];
    float* mine = (seat >= 0 && seat < n_seats) ? state + (size_t)seat * state_stride + (size_t)head * d * dv : nullptr;
    const float a = decay[head];
    const int g = tid / columns, jj = tid - g * columns;
    const int per = (d + groups - 1) / groups;
    const int i0 = g * per, i1 = min(d, i0 + per);
    const T* vrow = row + 2 * (size_t)heads * d + (size_t)head * dv;
    float ss = 0.f;
    for (int j0 = 0; j0 < dv; j0 += columns) {
        const int j = j0 + jj;
        const bool own = g < groups && j < dv;
        const float vj = own ? to_float(vrow[j]) : 0.f;
        float acc = 0.f;
        if (own && mine) {
            float* col = mine + j;
            for (int i = i0; i < i1; i += 8) {          // eight rows asked for before any is written
                float sv[8];
#pragma unroll
                for (int x = 0; x < 8; ++x) sv[x] = i + x < i1 ? col[(size_t)(i + x) * dv] : 0.f;
#pragma unroll
                for (int x = 0; x < 8; ++x) {
                    if (i + x >= i1) break;
                    acc = fmaf(qs[i + x], sv[x], acc);
                    col[(size_t)(i + x) * dv] = fmaf(a, sv[x], ks[i + x] * vj);
                }
            }
        }
        if (g < groups) part[g * columns + jj] = acc;
        __syncthreads();
        if (g == 0 && j < dv) {
            float sum = 0.f;
            for (int x = 0; x < groups; ++x) sum += part[x * columns + jj];
            const float o = fmaf(a, sum, dot * vj);
            os[j] = o;
            ss = fmaf(o, o, ss);
        }
        __syncthreads();
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)dv + eps) * scale;
    const T* grow = vrow + (size_t)heads * dv;
    for (int j = tid; j < dv; j += blockDim.x) {
        const float gate = to_float(grow[j]);
        out[(size_t)r * ldo + (size_t)head * dv + j] = from_float<T>(os[j] * inv * (gate / (1.f + expf(-gate))));
    }
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

// The same as fe_retention_scan for steps with long portions, in blocks of 64 tokens (three launches).  ``sums`` is scratch:
// float [tokens / 64 + requests, heads d dv] (fe_retention_chunk_rows says how many rows); ``most_tokens`` is the longest
// portion of the step or more.
extern "C" int fe_retention_chunk_tokens() { return CHUNK; }

extern "C" int fe_retention_chunks(const float* qk, const void* values, long long ldv, const float* decay, float* state,
                                   long long state_stride, const int* seats, const int* cu_q, float* out, float* sums, int requests,
                                   int most_tokens, int heads, int d, int dv, int n_seats, int dtype, cudaStream_t stream) {
    FE_REQUIRE(requests >= 0 && requests <= 65535 && heads > 0 && d > 0 && dv > 0 && n_seats >= 0 && most_tokens >= 0 &&
                   (long long)heads * d * dv <= state_stride && ldv >= (long long)heads * dv &&
                   (long long)heads * ((d + TILE - 1) / TILE) * ((dv + TILE - 1) / TILE) <= 65535,
               "retention_chunks: bad sizes (heads %d, key size %d, value size %d, %d requests)", heads, d, dv, requests);
    FE_REQUIRE(dtype == FE_F32 || dtype == FE_BF16, "retention_chunks: unknown dtype %d", dtype);
    if (requests == 0 || most_tokens == 0) return 0;
    const int most_blocks = (most_tokens + CHUNK - 1) / CHUNK;
    if (dtype == FE_F32)
        return launch_chunks<float>(qk, values, ldv, decay, state, state_stride, seats, cu_q, out, sums, requests, most_blocks, heads, d, dv,
                                    n_seats, stream);
    return launch_chunks<bf16>(qk, values, ldv, decay, state, state_stride, seats, cu_q, out, sums, requests, most_blocks, heads, d, dv,
                               n_seats, stream);
}

// A step of one token a request in one kernel.  proj [R, >= 2 heads d + 2 heads dv] = q | k | v | g in ``dtype`` with rows ld
// entries long; the keys are multiplied by key_scale after the rotation; out [R, >= heads dv] in ``dtype`` with rows ldo long gets
// every head divided by its root mean square, times silu(g), times scale.
extern "C" int fe_retention_decode(const void* proj, long long ld, const int* positions, const float* inv_freq, int rot, float key_scale,
                                   const float* decay, float* state, long long state_stride, const int* seats, void* out, long long ldo,
                                   float eps, float scale, int requests, int heads, int d, int dv, int n_seats, int dtype,
                                   cudaStream_t stream) {
    FE_REQUIRE(requests >= 0 && heads > 0 && heads <= 65535 && d > 0 && dv > 0 && n_seats >= 0 && rot >= 0 && rot % 2 == 0 && rot <= d &&
                   (long long)heads * d * dv <= state_stride && ld >= 2LL * heads * d + 2LL * heads * dv && ldo >= (long long)heads * dv,
               "retention_decode: bad sizes (heads %d, key size %d, value size %d, %d turned)", heads, d, dv, rot);
    FE_REQUIRE(rot == 0 || inv_freq != nullptr, "retention_decode: a rotation needs its frequencies");
    FE_REQUIRE(dtype == FE_F32 || dtype == FE_BF16, "retention_decode: unknown dtype %d", dtype);
    if (requests == 0) return 0;
    int columns = ((dv < 256 ? dv : 256) + 31) / 32 * 32;
    int groups = 512 / columns;
    groups = groups < 1 ? 1 : (groups > d ? d : groups);
    const size_t smem = ((size_t)2 * d + dv + (size_t)groups * columns + 33) * sizeof(float);
    FE_REQUIRE(smem <= 48 * 1024, "retention_decode: key size %d and value size %d need more shared memory than a block has", d, dv);
    if (dtype == FE_F32)
        fe::launch(retention_decode_kernel<float>, dim3(requests, heads), groups * columns, smem, stream, (const float*)proj, ld, positions,
                   inv_freq, rot, key_scale, decay, state, state_stride, seats, (float*)out, ldo, eps, scale, heads, d, dv, n_seats, groups);
    else
        fe::launch(retention_decode_kernel<bf16>, dim3(requests, heads), groups * columns, smem, stream, (const bf16*)proj, ld, positions,
                   inv_freq, rot, key_scale, decay, state, state_stride, seats, (bf16*)out, ldo, eps, scale, heads, d, dv, n_seats, groups);
    return fe_check_launch("retention_decode");
}
