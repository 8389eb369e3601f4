// A request's longer runs of tokens through the matrix-state recurrences, a chunk of tokens at a time.
//
// Both recurrences have the form S_t = keep_t S_{t-1} + take_t k_t v_t^T with the read-out S_t^T q_t, so over a chunk
// of tokens that starts from the carried S_0
//
//     S_t^T q_t = A_t S_0^T q_t + sum_{s <= t} W_ts (q_t . k_s) v_s,        S_last = A_last S_0 + sum_s W_(last)s k_s v_s^T,
//
// where, with G_t the sum of the logarithms of keep_1..keep_t inside the chunk:
//
//   * state space:    W_ts = exp(G_t - G_s) dt_s, A_t = exp(G_t); q = C, k = B, v = x, and D x_t is added;
//   * matrix memory:  with b_s = i_s - G_s and X_t = max(m_0, max_{s <= t} b_s), the running maximum is m_t = G_t + X_t,
//                     W_ts = exp(b_s - X_t), A_t = exp(m_0 - X_t); the normaliser is the same sum with k alone, the
//                     read-out is divided by max(|n_t . q_t|, exp(-m_t)) + 1e-6.
//
// (The state-space form is the same with b_s = -G_s, X_t = -G_t and m_0 = 0, times dt_s.)  No exponent is positive.
// A block owns (request, head, a run of value columns) and goes through the request's chunks in order with its part
// of the state in shared memory; inside a chunk the scores, the read-out and the state's update are small 32-bit
// matrix products over shared tiles, a thread holding a 4 x 4 tile of each.  Gates, decays, scores, sums and the
// state are 32-bit.  The matrix memory's new normaliser and maximum go to a side buffer and from there to the slot in
// a second kernel, since every block of a head reads the old ones.
#include "common.cuh"
#include "state_math.cuh"

namespace {

constexpr int CHUNK = 64;         // tokens a chunk
constexpr int PITCH = CHUNK + 4;  // floats a row of the tiles that keep a chunk's tokens along a row
constexpr int THREADS = 256;      // 16 x 16 threads, 4 x 4 entries each

struct ChunkScan {
    const float* q;  // [*, groups d] (row stride q_stride): what reads the state
    const float* k;  // [*, groups d]: what is written along the state's rows
    const float* v;  // [*, heads dv]: what is written along the state's columns
    long q_stride, k_stride, v_stride;
    const float* gate_a;  // [*, heads]: state space: step size before softplus; matrix memory: input gate before its cap
    const float* gate_b;  // [*, heads]: matrix memory: forget gate before its cap
    long gate_a_stride, gate_b_stride;
    const float* bias_a;  // [heads] or null
    const float* bias_b;  // [heads] or null
    const float* rate;    // [heads]: state space: logarithm of the decay rate
    const float* skip;    // [heads]: state space: weight of v in the read-out
    float cap, q_scale;
    float* state;  // [slots, state_len]
    long state_len, s_off, n_off, m_off;
    float* tail;  // [requests, heads, d + 1]: matrix memory: the new normaliser and maximum
    const int* query_start;
    const int* slots;
    float* out;  // [*, heads dv]
    int heads, groups, d, dv, cols, num_slots, memory;
};

__host__ __device__ inline int cols_pitch(int cols) { return (cols + 15) / 16 * 16; }

// A 4-byte copy from global to shared memory that the thread does not wait for (any address, any stride).
__device__ __forceinline__ void copy_async(float* to, const float* from) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(to)), "l"(from) : "memory");
}
__device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// `len` rows of `d` columns from `from` (row stride `stride`) into a tile that keeps tokens along a row, [d][PITCH];
// the columns of tokens that the chunk does not have are zero.
__device__ __forceinline__ void fetch_across(float* tile, const float* from, long stride, int len, int d) {
    for (int i = threadIdx.x; i < CHUNK * d; i += THREADS) {
        const int t = i / d, kd = i - t * d;
        if (t < len) copy_async(tile + kd * PITCH + t, from + t * stride + kd);
        else tile[kd * PITCH + t] = 0.0f;
    }
}

// `len` rows of `cols` columns into a tile [CHUNK][cp]; zero elsewhere.
__device__ __forceinline__ void fetch_along(float* tile, const float* from, long stride, int len, int cols, int cp) {
    for (int i = threadIdx.x; i < CHUNK * cp; i += THREADS) {
        const int t = i / cp, c = i - t * cp;
        if (t < len && c < cols) copy_async(tile + i, from + t * stride + c);
        else tile[i] = 0.0f;
    }
}

__host__ __device__ inline long chunk_scan_floats(int d, int cols) {
    const int cp = cols_pitch(cols);
    return 2L * d * PITCH + (long)CHUNK * PITCH + (long)CHUNK * cp + (long)d * cp + d + 5 * CHUNK + 8;
}

// Warp 0: the chunk's gates.  Lane l has tokens 2l and 2l + 1, so that the sums and maxima along the chunk are one
// scan over the lanes.  b[s], X[t], c[s] (dt or 1), last[s] = W_(last)s, floor[t] = exp(-m_t); scal[1] = A_last,
// scal[2] = the maximum after the chunk.
__device__ __forceinline__ void chunk_gates(const ChunkScan& a, int head, long row0, int len, float m0, float* sB, float* sX,
                                            float* sC, float* sLast, float* sFloor, float* scal) {
    const int lane = threadIdx.x;
    float g[2], u[2], c[2];
    const float ba = a.bias_a ? a.bias_a[head] : 0.0f, bb = a.bias_b ? a.bias_b[head] : 0.0f;
    const float rate = a.memory ? 0.0f : -expf(a.rate[head]);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int t = 2 * lane + e;
        g[e] = 0.0f, u[e] = -INFINITY, c[e] = 0.0f;
        if (t < len) {
            const float ra = a.gate_a[(row0 + t) * a.gate_a_stride + head] + ba;
            if (a.memory) {
                const float rb = a.gate_b[(row0 + t) * a.gate_b_stride + head] + bb;
                u[e] = a.cap * tanhf(ra / a.cap);
                g[e] = sf_log_sigmoid(a.cap * tanhf(rb / a.cap));
                c[e] = 1.0f;
            } else {
                const float dt = sf_softplus(ra);
                g[e] = rate * dt, u[e] = 0.0f, c[e] = dt;
            }
        }
    }
    float sum = g[0] + g[1];
    for (int off = 1; off < 32; off <<= 1) {
        const float other = __shfl_up_sync(0xffffffffu, sum, off);
        if (lane >= off) sum += other;
    }
    const float G1 = sum, G0 = sum - g[1];
    float G[2] = {G0, G1}, b[2], X[2];
    if (a.memory) {
        b[0] = u[0] - G[0], b[1] = u[1] - G[1];
        float peak = fmaxf(b[0], b[1]);
        for (int off = 1; off < 32; off <<= 1) {
            const float other = __shfl_up_sync(0xffffffffu, peak, off);
            if (lane >= off) peak = fmaxf(peak, other);
        }
        float before = __shfl_up_sync(0xffffffffu, peak, 1);
        before = lane == 0 ? m0 : fmaxf(before, m0);
        X[0] = fmaxf(before, b[0]);
        X[1] = fmaxf(X[0], b[1]);
    } else {
        b[0] = X[0] = -G[0];
        b[1] = X[1] = -G[1];
    }
    const int last = len - 1;
    const float X_last = __shfl_sync(0xffffffffu, (last & 1) ? X[1] : X[0], last >> 1);
    const float G_last = __shfl_sync(0xffffffffu, (last & 1) ? G[1] : G[0], last >> 1);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int t = 2 * lane + e;
        const bool live = t < len;
        sB[t] = live ? b[e] : 0.0f;
        sX[t] = live ? X[e] : 0.0f;
        sC[t] = c[e];
        sLast[t] = live ? expf(b[e] - X_last) * c[e] : 0.0f;
        sFloor[t] = (live && a.memory) ? expf(-(G[e] + X[e])) : 0.0f;
    }
    if (lane == 0) {
        scal[1] = expf(m0 - X_last);
        scal[2] = a.memory ? G_last + X_last : 0.0f;
    }
}

__global__ void __launch_bounds__(THREADS) chunk_scan_kernel(const ChunkScan a) {
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int request = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * a.cols;
    const int cols = min(a.cols, a.dv - col0), cp = cols_pitch(a.cols), J = cols_pitch(cols) / 16;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4, d = a.d;
    float* sQ = smem;                  // [d][PITCH]: q of the chunk; tokens along a row
    float* sK = sQ + (long)d * PITCH;  // [d][PITCH]
    float* sP = sK + (long)d * PITCH;  // [CHUNK][PITCH]: weighted scores, [s][t]
    float* sV = sP + CHUNK * PITCH;    // [CHUNK][cp]
    float* sS = sV + CHUNK * cp;       // [d][cp]: this block's columns of the state
    float* sN = sS + (long)d * cp;     // [d]: the normaliser
    float* sB = sN + d;
    float* sX = sB + CHUNK;
    float* sC = sX + CHUNK;
    float* sLast = sC + CHUNK;
    float* sFloor = sLast + CHUNK;
    float* scal = sFloor + CHUNK;  // [0] the maximum before the chunk, [1] A_last, [2] the maximum after it
    const long first = a.query_start[request];
    const int count = (int)(a.query_start[request + 1] - first);
    const int slot = a.slots[request];
    const int group = head / (a.heads / a.groups);
    pdl_wait();
    if (slot < 0 || slot >= a.num_slots || count <= 0) return;
    float* base = a.state + slot * a.state_len;
    float* Sg = base + a.s_off + (long)head * d * a.dv + col0;
    for (int i = tid; i < d * cp; i += THREADS) {
        const int kd = i / cp, c = i - kd * cp;
        sS[i] = c < cols ? Sg[(long)kd * a.dv + c] : 0.0f;
    }
    for (int kd = tid; kd < d; kd += THREADS) sN[kd] = a.memory ? base[a.n_off + (long)head * d + kd] : 0.0f;
    if (tid == 0) scal[0] = a.memory ? base[a.m_off + head] : 0.0f;
    __syncthreads();

    // A chunk's q, k and v come by copies that nobody waits for until the chunk begins: q's tile is free after the
    // read-out and is filled for the next chunk while the state is brought up to date; k and v follow after that,
    // beside the next chunk's gates.
    const float* q_from = a.q + (long)group * d;
    const float* k_from = a.k + (long)group * d;
    const float* v_from = a.v + (long)head * a.dv + col0;
    {
        const int len = min(CHUNK, count);
        fetch_across(sQ, q_from + first * a.q_stride, a.q_stride, len, d);
        fetch_across(sK, k_from + first * a.k_stride, a.k_stride, len, d);
        fetch_along(sV, v_from + first * a.v_stride, a.v_stride, len, cols, cp);
    }
    const float q_scale = a.q_scale;

    for (int c0 = 0; c0 < count; c0 += CHUNK) {
        const int len = min(CHUNK, count - c0);
        const int next_len = min(CHUNK, count - c0 - CHUNK);  // <= 0: this chunk is the last
        const long row0 = first + c0;
        if (tid < 32) chunk_gates(a, head, row0, len, scal[0], sB, sX, sC, sLast, sFloor, scal);
        copies_wait();
        __syncthreads();

        // weighted scores of tokens t = 4 ty + i against s = 4 tx + j, stored [s][t]
        {
            float acc[4][4] = {};
            if (4 * tx <= 4 * ty + 3 && 4 * tx < len) {
                for (int kd = 0; kd < d; ++kd) {
                    const float4 qv = *reinterpret_cast<const float4*>(sQ + kd * PITCH + 4 * ty);
                    const float4 kv = *reinterpret_cast<const float4*>(sK + kd * PITCH + 4 * tx);
                    const float qs[4] = {qv.x, qv.y, qv.z, qv.w}, ks[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qs[i], ks[j], acc[i][j]);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int s = 4 * tx + j;
                float p[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int t = 4 * ty + i;
                    p[i] = (s <= t && t < len) ? acc[i][j] * q_scale * expf(sB[s] - sX[t]) * sC[s] : 0.0f;
                }
                *reinterpret_cast<float4*>(sP + s * PITCH + 4 * ty) = make_float4(p[0], p[1], p[2], p[3]);
            }
        }
        __syncthreads();

        // the read-out of tokens t = 4 ty + i at columns tx + 16 j
        {
            float o[4][4] = {}, den[4] = {};
            for (int kd = 0; kd < d; ++kd) {
                const float4 qv = *reinterpret_cast<const float4*>(sQ + kd * PITCH + 4 * ty);
                const float qs[4] = {qv.x, qv.y, qv.z, qv.w};
                const float nv = sN[kd];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (j < J) {
                        const float sv = sS[kd * cp + tx + 16 * j];
#pragma unroll
                        for (int i = 0; i < 4; ++i) o[i][j] = fmaf(qs[i], sv, o[i][j]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) den[i] = fmaf(qs[i], nv, den[i]);
            }
            const float m0 = scal[0];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float carried = expf(m0 - sX[4 * ty + i]) * q_scale;
                den[i] *= carried;
#pragma unroll
                for (int j = 0; j < 4; ++j) o[i][j] *= carried;
            }
            const int s_end = min(4 * ty + 4, len);
            for (int s = 0; s < s_end; ++s) {
                const float4 pv = *reinterpret_cast<const float4*>(sP + s * PITCH + 4 * ty);
                const float ps[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (j < J) {
                        const float vv = sV[s * cp + tx + 16 * j];
#pragma unroll
                        for (int i = 0; i < 4; ++i) o[i][j] = fmaf(ps[i], vv, o[i][j]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) den[i] += ps[i];
            }
            const float skip = a.memory ? 0.0f : a.skip[head];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int t = 4 * ty + i;
                if (t >= len) continue;
                const float under = a.memory ? 1.0f / (fmaxf(fabsf(den[i]), sFloor[t]) + 1e-6f) : 1.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = tx + 16 * j;
                    if (j < J && c < cols) {
                        const float value = a.memory ? o[i][j] * under : fmaf(skip, sV[t * cp + c], o[i][j]);
                        a.out[(row0 + t) * ((long)a.heads * a.dv) + (long)head * a.dv + col0 + c] = value;
                    }
                }
            }
        }
        __syncthreads();  // everyone has read the state and the normaliser of the chunk's start, and q
        if (next_len > 0) fetch_across(sQ, q_from + (row0 + CHUNK) * a.q_stride, a.q_stride, next_len, d);

        // the state after the chunk: rows r0 + 4 ty + i, columns tx + 16 j
        const float kept = scal[1];
        for (int r0 = 0; r0 < d; r0 += 64) {
            float acc[4][4] = {};
            const int kd0 = r0 + 4 * ty;
            for (int s = 0; s < len; ++s) {
                const float w = sLast[s];
                float ks[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) ks[i] = kd0 + i < d ? sK[(kd0 + i) * PITCH + s] * w : 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (j < J) {
                        const float vv = sV[s * cp + tx + 16 * j];
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[i][j] = fmaf(ks[i], vv, acc[i][j]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (j < J && kd0 + i < d) {
                        float* at = sS + (kd0 + i) * cp + tx + 16 * j;
                        *at = fmaf(kept, *at, acc[i][j]);
                    }
        }
        if (a.memory) {
            for (int kd = tid; kd < d; kd += THREADS) {
                float acc = 0.0f;
                for (int s = 0; s < len; ++s) acc = fmaf(sLast[s], sK[kd * PITCH + s], acc);
                sN[kd] = fmaf(kept, sN[kd], acc);
            }
        }
        if (tid == 0) scal[0] = scal[2];  // (the read-out, which needs the old one, lies behind the barrier above)
        __syncthreads();  // the tiles and the gates are free for the next chunk
        if (next_len > 0) {
            fetch_across(sK, k_from + (row0 + CHUNK) * a.k_stride, a.k_stride, next_len, d);
            fetch_along(sV, v_from + (row0 + CHUNK) * a.v_stride, a.v_stride, next_len, cols, cp);
        }
    }
    for (int i = tid; i < d * cp; i += THREADS) {
        const int kd = i / cp, c = i - kd * cp;
        if (c < cols) Sg[(long)kd * a.dv + c] = sS[i];
    }
    if (a.memory && blockIdx.z == 0) {
        float* mine = a.tail + ((long)request * a.heads + head) * (d + 1);
        for (int kd = tid; kd < d; kd += THREADS) mine[kd] = sN[kd];
        if (tid == 0) mine[d] = scal[0];
    }
}

// A thread per (request, head, entry): the new normaliser and maximum go to the request's slot.
__global__ void chunk_tail_kernel(const float* __restrict__ tail, float* __restrict__ state, long state_len, long n_off, long m_off,
                                  const int* __restrict__ query_start, const int* __restrict__ slots, int requests, int heads, int d,
                                  int num_slots) {
    pdl_launch_dependents();
    pdl_wait();
    const long at = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (at >= (long)requests * heads * (d + 1)) return;
    const int entry = (int)(at % (d + 1));
    const long unit = at / (d + 1);
    const int head = (int)(unit % heads), request = (int)(unit / heads);
    const int slot = slots[request];
    if (slot < 0 || slot >= num_slots || query_start[request + 1] <= query_start[request]) return;
    float* base = state + slot * state_len;
    if (entry < d) base[n_off + (long)head * d + entry] = tail[at];
    else base[m_off + head] = tail[at];
}

// How many value columns a block takes: as many as fit shared memory, fewer (16 at least) while the grid would leave
// most of the device idle.  0 when even 16 do not fit.
int choose_cols(int requests, int heads, int d, int dv, long* bytes) {
    int device = 0, limit = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        return 0;
    int cols = dv < 64 ? dv : 64;
    while (cols > 16 && (chunk_scan_floats(d, cols) * 4 > limit || (long)requests * heads * ((dv + cols - 1) / cols) < sms))
        cols = cols > 32 ? cols - 16 : 16;
    *bytes = chunk_scan_floats(d, cols) * 4;
    return *bytes <= limit ? cols : 0;
}

int chunk_scan_launch(ChunkScan a, int requests, cudaStream_t stream) {
    long bytes = 0;
    a.cols = choose_cols(requests, a.heads, a.d, a.dv, &bytes);
    if (a.cols <= 0) return KIRAI_ERR_UNSUPPORTED;
    static long granted = 0;  // (one device a process)
    if (bytes > granted) {
        if (cudaFuncSetAttribute(chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
            return launch_status();
        granted = bytes;
    }
    const int pieces = (a.dv + a.cols - 1) / a.cols;
    int status = launch_pdl(chunk_scan_kernel, dim3(requests, a.heads, pieces), dim3(THREADS), (size_t)bytes, stream, 1u, a);
    if (status != 0 || !a.memory) return status;
    const long units = (long)requests * a.heads * (a.d + 1);
    return launch_pdl(chunk_tail_kernel, dim3((unsigned)((units + 255) / 256)), dim3(256), 0, stream, 1u, (const float*)a.tail,
                      a.state, a.state_len, a.n_off, a.m_off, a.query_start, a.slots, requests, a.heads, a.d, a.num_slots);
}

}  // namespace

// 1 when a head of d state rows fits the chunked kernels' shared memory, else 0 (the walk takes such a head).
KIRAI_EXPORT int kirai_state_chunks_fit(int d) {
    int device = 0, limit = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess)
        return 0;
    return d > 0 && chunk_scan_floats(d, 16) * 4 <= limit ? 1 : 0;
}

KIRAI_EXPORT int kirai_state_chunk_tokens() { return CHUNK; }

// The state-space recurrence in chunks; the arguments of kirai_ssm_walk.
KIRAI_EXPORT int kirai_ssm_chunks(const float* xbc, const float* dt_raw, long dt_stride, const float* dt_bias, const float* a_log,
                                  const float* d_skip, float* state, long state_len, long ssm_off, const int* query_start,
                                  const int* slots, float* y, int requests, int heads, int groups, int N, int P, int num_slots,
                                  cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || P <= 0 || ssm_off < 0 || ssm_off + (long)heads * N * P > state_len)
        return KIRAI_ERR_BAD_SIZE;
    const long inner = (long)heads * P, channels = inner + 2L * groups * N;
    ChunkScan a = {};
    a.q = xbc + inner + (long)groups * N, a.k = xbc + inner, a.v = xbc;
    a.q_stride = a.k_stride = a.v_stride = channels;
    a.gate_a = dt_raw, a.gate_a_stride = dt_stride, a.bias_a = dt_bias, a.rate = a_log, a.skip = d_skip;
    a.cap = 1.0f, a.q_scale = 1.0f;
    a.state = state, a.state_len = state_len, a.s_off = ssm_off;
    a.query_start = query_start, a.slots = slots, a.out = y;
    a.heads = heads, a.groups = groups, a.d = N, a.dv = P, a.num_slots = num_slots, a.memory = 0;
    return chunk_scan_launch(a, requests, stream);
}

// The matrix memory in chunks; the arguments of kirai_matrix_memory_walk and `tail` [requests, heads, d + 1] (float32).
KIRAI_EXPORT int kirai_matrix_memory_chunks(const float* rows, long row_stride, const float* in_bias, const float* keep_bias,
                                            float cap, float q_scale, float* state, long state_len, const int* query_start,
                                            const int* slots, float* o, float* tail, int requests, int heads, int d, int dv,
                                            int num_slots, cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (heads <= 0 || d <= 0 || dv <= 0 || !(cap > 0.0f) || !tail || (long)heads * d * dv + (long)heads * d + heads > state_len)
        return KIRAI_ERR_BAD_SIZE;
    ChunkScan a = {};
    a.q = rows, a.k = rows + (long)heads * d, a.v = rows + 2L * heads * d;
    a.q_stride = a.k_stride = a.v_stride = row_stride;
    a.gate_a = a.v + (long)heads * dv, a.gate_b = a.gate_a + heads;
    a.gate_a_stride = a.gate_b_stride = row_stride;
    a.bias_a = in_bias, a.bias_b = keep_bias;
    a.cap = cap, a.q_scale = q_scale;
    a.state = state, a.state_len = state_len, a.s_off = 0, a.n_off = (long)heads * d * dv, a.m_off = a.n_off + (long)heads * d;
    a.tail = tail;
    a.query_start = query_start, a.slots = slots, a.out = o;
    a.heads = heads, a.groups = heads, a.d = d, a.dv = dv, a.num_slots = num_slots, a.memory = 1;
    return chunk_scan_launch(a, requests, stream);
}
