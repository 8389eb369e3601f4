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
    const int lane = threadIdx.x & 31;
    for (int t = threadIdx.x >> 5; t < CHUNK; t += THREADS / 32) {  // a warp takes a token's row
        const float* row = from + t * stride;
        if (t < len)
            for (int kd = lane; kd < d; kd += 32) copy_async(tile + kd * PITCH + t, row + kd);
        else
            for (int kd = lane; kd < d; kd += 32) tile[kd * PITCH + t] = 0.0f;
    }
}

// `len` rows of `cols` columns into a tile [CHUNK][cp]; zero elsewhere.
__device__ __forceinline__ void fetch_along(float* tile, const float* from, long stride, int len, int cols, int cp) {
    const int c = threadIdx.x & 15;
    for (int t = threadIdx.x >> 4; t < CHUNK; t += THREADS / 16) {
        const float* row = from + t * stride;
        for (int at = c; at < cp; at += 16) {
            if (t < len && at < cols) copy_async(tile + t * cp + at, row + at);
            else tile[t * cp + at] = 0.0f;
        }
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
        scal[3] = X_last, scal[4] = G_last;
    }
}

// The tiles of a block, in this order in shared memory.
struct Tiles {
    float *Q, *K, *P, *V, *S, *N, *B, *X, *C, *Last, *Floor, *scal;
    __device__ Tiles(float* smem, int d, int cp) {
        Q = smem;                   // [d][PITCH]: q of the chunk; tokens along a row
        K = Q + (long)d * PITCH;    // [d][PITCH]
        P = K + (long)d * PITCH;    // [CHUNK][PITCH]: weighted scores, [s][t]
        V = P + CHUNK * PITCH;      // [CHUNK][cp]
        S = V + CHUNK * cp;         // [d][cp]: this block's columns of the state
        N = S + (long)d * cp;       // [d]: the normaliser
        B = N + d, X = B + CHUNK, C = X + CHUNK, Last = C + CHUNK, Floor = Last + CHUNK;
        scal = Floor + CHUNK;  // [0] the maximum before the chunk, [1] A_last, [2] the maximum after it, [3] X_last, [4] G_last
    }
};

// Weighted scores of tokens t = 4 ty + i against s = 4 tx + j, stored [s][t].
__device__ __forceinline__ void chunk_scores(const Tiles& w, int d, int len, float q_scale) {
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    if (4 * tx <= 4 * ty + 3 && 4 * tx < len) {
#pragma unroll 4
        for (int kd = 0; kd < d; ++kd) {
            const float4 qv = *reinterpret_cast<const float4*>(w.Q + kd * PITCH + 4 * ty);
            const float4 kv = *reinterpret_cast<const float4*>(w.K + kd * PITCH + 4 * tx);
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
            p[i] = (s <= t && t < len) ? acc[i][j] * q_scale * expf(w.B[s] - w.X[t]) * w.C[s] : 0.0f;
        }
        *reinterpret_cast<float4*>(w.P + s * PITCH + 4 * ty) = make_float4(p[0], p[1], p[2], p[3]);
    }
}

// The read-out of tokens t = 4 ty + i at columns tx + 16 j, from the state of the chunk's start and the chunk's scores.
template <int J>
__device__ __forceinline__ void chunk_read_out(const ChunkScan& a, const Tiles& w, int head, int col0, int cols, long row0, int len) {
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4, d = a.d;
    constexpr int cp = 16 * J;
    float o[4][J] = {}, den[4] = {};
#pragma unroll 4
    for (int kd = 0; kd < d; ++kd) {
        const float4 qv = *reinterpret_cast<const float4*>(w.Q + kd * PITCH + 4 * ty);
        const float qs[4] = {qv.x, qv.y, qv.z, qv.w};
        const float nv = w.N[kd];
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const float sv = w.S[kd * cp + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i][j] = fmaf(qs[i], sv, o[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) den[i] = fmaf(qs[i], nv, den[i]);
    }
    const float m0 = w.scal[0];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float carried = expf(m0 - w.X[4 * ty + i]) * a.q_scale;
        den[i] *= carried;
#pragma unroll
        for (int j = 0; j < J; ++j) o[i][j] *= carried;
    }
    const int s_end = min(4 * ty + 4, len);
#pragma unroll 4
    for (int s = 0; s < s_end; ++s) {
        const float4 pv = *reinterpret_cast<const float4*>(w.P + s * PITCH + 4 * ty);
        const float ps[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const float vv = w.V[s * cp + tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i][j] = fmaf(ps[i], vv, o[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) den[i] += ps[i];
    }
    const float skip = a.memory ? 0.0f : a.skip[head];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = 4 * ty + i;
        if (t >= len) continue;
        const float under = a.memory ? 1.0f / (fmaxf(fabsf(den[i]), w.Floor[t]) + 1e-6f) : 1.0f;
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const int c = tx + 16 * j;
            if (c < cols) {
                const float value = a.memory ? o[i][j] * under : fmaf(skip, w.V[t * cp + c], o[i][j]);
                a.out[(row0 + t) * ((long)a.heads * a.dv) + (long)head * a.dv + col0 + c] = value;
            }
        }
    }
}

// The state and the normaliser after the chunk: S <- kept S + sum_s Last[s] k_s v_s^T, rows r0 + 4 ty + i, columns tx + 16 j.
template <int J>
__device__ __forceinline__ void chunk_update(const Tiles& w, int d, int len, float kept, bool memory) {
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    constexpr int cp = 16 * J;
    for (int r0 = 0; r0 < d; r0 += 64) {
        float acc[4][J] = {};
        const int kd0 = r0 + 4 * ty;
#pragma unroll 4
        for (int s = 0; s < len; ++s) {
            const float weight = w.Last[s];
            float ks[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) ks[i] = kd0 + i < d ? w.K[(kd0 + i) * PITCH + s] * weight : 0.0f;
#pragma unroll
            for (int j = 0; j < J; ++j) {
                const float vv = w.V[s * cp + tx + 16 * j];
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[i][j] = fmaf(ks[i], vv, acc[i][j]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < J; ++j)
                if (kd0 + i < d) {
                    float* at = w.S + (kd0 + i) * cp + tx + 16 * j;
                    *at = fmaf(kept, *at, acc[i][j]);
                }
    }
    if (memory) {
        for (int kd = tid; kd < d; kd += THREADS) {
            float acc = 0.0f;
            for (int s = 0; s < len; ++s) acc = fmaf(w.Last[s], w.K[kd * PITCH + s], acc);
            w.N[kd] = fmaf(kept, w.N[kd], acc);
        }
    }
}

// J: runs of 16 value columns that a block has (the columns beyond the last piece's own are zero and are not written).
// A block goes through its request's chunks in order.
template <int J>
__global__ void __launch_bounds__(THREADS) chunk_scan_kernel(const ChunkScan a) {
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int request = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * a.cols;
    const int cols = min(a.cols, a.dv - col0), cp = 16 * J;
    const int tid = threadIdx.x, d = a.d;
    const Tiles w(smem, d, cp);
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
        w.S[i] = c < cols ? Sg[(long)kd * a.dv + c] : 0.0f;
    }
    for (int kd = tid; kd < d; kd += THREADS) w.N[kd] = a.memory ? base[a.n_off + (long)head * d + kd] : 0.0f;
    if (tid == 0) w.scal[0] = a.memory ? base[a.m_off + head] : 0.0f;
    __syncthreads();

    // A chunk's q, k and v come by copies that nobody waits for until the chunk begins: q's tile is free after the
    // read-out and is filled for the next chunk while the state is brought up to date; k and v follow after that,
    // beside the next chunk's gates.
    const float* q_from = a.q + (long)group * d;
    const float* k_from = a.k + (long)group * d;
    const float* v_from = a.v + (long)head * a.dv + col0;
    {
        const int len = min(CHUNK, count);
        fetch_across(w.Q, q_from + first * a.q_stride, a.q_stride, len, d);
        fetch_across(w.K, k_from + first * a.k_stride, a.k_stride, len, d);
        fetch_along(w.V, v_from + first * a.v_stride, a.v_stride, len, cols, cp);
    }
    for (int c0 = 0; c0 < count; c0 += CHUNK) {
        const int len = min(CHUNK, count - c0);
        const int next_len = min(CHUNK, count - c0 - CHUNK);  // <= 0: this chunk is the last
        const long row0 = first + c0;
        if (tid < 32) chunk_gates(a, head, row0, len, w.scal[0], w.B, w.X, w.C, w.Last, w.Floor, w.scal);
        copies_wait();
        __syncthreads();
        chunk_scores(w, d, len, a.q_scale);
        __syncthreads();
        chunk_read_out<J>(a, w, head, col0, cols, row0, len);
        __syncthreads();  // everyone has read the state and the normaliser of the chunk's start, and q
        if (next_len > 0) fetch_across(w.Q, q_from + (row0 + CHUNK) * a.q_stride, a.q_stride, next_len, d);
        chunk_update<J>(w, d, len, w.scal[1], a.memory != 0);
        if (tid == 0) w.scal[0] = w.scal[2];  // (the read-out, which needs the old one, lies behind the barrier above)
        __syncthreads();  // the tiles and the gates are free for the next chunk
        if (next_len > 0) {
            fetch_across(w.K, k_from + (row0 + CHUNK) * a.k_stride, a.k_stride, next_len, d);
            fetch_along(w.V, v_from + (row0 + CHUNK) * a.v_stride, a.v_stride, next_len, cols, cp);
        }
    }
    for (int i = tid; i < d * cp; i += THREADS) {
        const int kd = i / cp, c = i - kd * cp;
        if (c < cols) Sg[(long)kd * a.dv + c] = w.S[i];
    }
    if (a.memory && blockIdx.z == 0) {
        float* mine = a.tail + ((long)request * a.heads + head) * (d + 1);
        for (int kd = tid; kd < d; kd += THREADS) mine[kd] = w.N[kd];
        if (tid == 0) mine[d] = w.scal[0];
    }
}

// ---- long runs: the chunks side by side ------------------------------------------------------------------------------
// A run of many chunks leaves a block of the kernel above alone with a long chain.  Three launches take the chain out of
// the heavy work:
//   1. chunk_local: block (chunk of the step, head, run of columns) finds the chunk's own share of the state as if the
//      chunk began from nothing: U = sum_s exp(b_s - X'_last) take_s k_s v_s^T (and u with k alone), with X'_t the maximum
//      of b over the chunk's tokens so far, and notes X'_last and G_last;
//   2. chunk_carry: a thread per entry of a head's state walks the request's chunks: it leaves the state at each
//      chunk's START where U was and moves on by S <- exp(M - Xf) S + exp(X'_last - Xf) U, Xf = max(M, X'_last),
//      M <- G_last + Xf (the state space has M = 0 throughout and X'_last = -G_last, so S <- exp(G_last) S + U);
//   3. chunk_out: block (chunk, head, run of columns) reads the chunk's tokens out of the state at its start.
// The step's chunks are numbered request by request; a block finds its request by a walk over the row boundaries.
struct ChunkPlace {
    int request, chunk, chunks, len;
    long row0;
};

__device__ __forceinline__ bool find_chunk(const int* __restrict__ query_start, int requests, int at, ChunkPlace& place) {
    for (int r = 0; r < requests; ++r) {
        const int first = query_start[r], count = query_start[r + 1] - first;
        const int chunks = (count + CHUNK - 1) / CHUNK;
        if (at < chunks) {
            place.request = r, place.chunk = at, place.chunks = chunks;
            place.len = min(CHUNK, count - at * CHUNK);
            place.row0 = (long)first + (long)at * CHUNK;
            return true;
        }
        at -= chunks;
    }
    return false;
}

struct ChunkSide {
    float* U;      // [chunks of the step, heads, d, dv]: a chunk's own share, then the state at its start
    float* u;      // [chunks, heads, d]: likewise for the normaliser (matrix memory)
    float* marks;  // [chunks, heads, 3]: X'_last, G_last, then the maximum at the chunk's start
};

template <int J>
__global__ void __launch_bounds__(THREADS) chunk_local_kernel(const ChunkScan a, const ChunkSide side, int requests) {
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int head = blockIdx.y, col0 = blockIdx.z * a.cols;
    const int cols = min(a.cols, a.dv - col0), cp = 16 * J;
    const int tid = threadIdx.x, d = a.d;
    const Tiles w(smem, d, cp);
    ChunkPlace at;
    const bool found = find_chunk(a.query_start, requests, blockIdx.x, at);
    pdl_wait();
    if (!found) return;
    const int group = head / (a.heads / a.groups);
    fetch_across(w.K, a.k + (long)group * d + at.row0 * a.k_stride, a.k_stride, at.len, d);
    fetch_along(w.V, a.v + (long)head * a.dv + col0 + at.row0 * a.v_stride, a.v_stride, at.len, cols, cp);
    for (int i = tid; i < d * cp; i += THREADS) w.S[i] = 0.0f;
    for (int kd = tid; kd < d; kd += THREADS) w.N[kd] = 0.0f;
    if (tid < 32) chunk_gates(a, head, at.row0, at.len, a.memory ? -INFINITY : 0.0f, w.B, w.X, w.C, w.Last, w.Floor, w.scal);
    copies_wait();
    __syncthreads();
    chunk_update<J>(w, d, at.len, 0.0f, a.memory != 0);
    __syncthreads();
    const long unit = (long)blockIdx.x * a.heads + head;
    float* U = side.U + unit * d * a.dv + col0;
    for (int i = tid; i < d * cp; i += THREADS) {
        const int kd = i / cp, c = i - kd * cp;
        if (c < cols) U[(long)kd * a.dv + c] = w.S[i];
    }
    if (blockIdx.z == 0) {
        if (a.memory)
            for (int kd = tid; kd < d; kd += THREADS) side.u[unit * d + kd] = w.N[kd];
        if (tid == 0) side.marks[unit * 3] = w.scal[3], side.marks[unit * 3 + 1] = w.scal[4];
    }
}

// Block (request, head, run of 256 entries): entries 0 .. d dv - 1 are the state's, the next d the normaliser's.
__global__ void __launch_bounds__(256) chunk_carry_kernel(const ChunkScan a, const ChunkSide side, int requests) {
    pdl_launch_dependents();
    const int request = blockIdx.x, head = blockIdx.y;
    const long entry = blockIdx.z * 256L + threadIdx.x;
    const long cells = (long)a.d * a.dv;
    int before = 0;
    for (int r = 0; r < request; ++r) before += (a.query_start[r + 1] - a.query_start[r] + CHUNK - 1) / CHUNK;
    const int chunks = (a.query_start[request + 1] - a.query_start[request] + CHUNK - 1) / CHUNK;
    const int slot = a.slots[request];
    pdl_wait();
    if (slot < 0 || slot >= a.num_slots || chunks <= 0 || entry >= cells + (a.memory ? a.d : 0)) return;
    float* base = a.state + slot * a.state_len;
    const bool of_state = entry < cells;
    float* mine = of_state ? base + a.s_off + (long)head * cells + entry : base + a.n_off + (long)head * a.d + (entry - cells);
    float value = *mine;
    float M = a.memory ? base[a.m_off + head] : 0.0f;
    const long stride = of_state ? (long)a.heads * cells : (long)a.heads * a.d;
    float* share = of_state ? side.U + ((long)before * a.heads + head) * cells + entry
                            : side.u + ((long)before * a.heads + head) * a.d + (entry - cells);
    float ahead = *share;
    for (int c = 0; c < chunks; ++c, share += stride) {
        const long unit = (long)(before + c) * a.heads + head;
        const float x_last = side.marks[unit * 3], g_last = side.marks[unit * 3 + 1];
        const float xf = fmaxf(M, x_last);
        const float own = ahead;
        if (c + 1 < chunks) ahead = share[stride];  // (another chunk's entry: the store below does not touch it)
        *share = value;
        if (entry == 0) side.marks[unit * 3 + 2] = M;
        value = fmaf(expf(M - xf), value, expf(x_last - xf) * own);
        M = a.memory ? g_last + xf : 0.0f;
    }
    *mine = value;  // (the maximum goes to the slot from the last chunk's block of the next launch: every block here reads the old one)
}

template <int J>
__global__ void __launch_bounds__(THREADS) chunk_out_kernel(const ChunkScan a, const ChunkSide side, int requests) {
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    const int head = blockIdx.y, col0 = blockIdx.z * a.cols;
    const int cols = min(a.cols, a.dv - col0), cp = 16 * J;
    const int tid = threadIdx.x, d = a.d;
    const Tiles w(smem, d, cp);
    ChunkPlace at;
    const bool found = find_chunk(a.query_start, requests, blockIdx.x, at);
    const int slot = found ? a.slots[at.request] : -1;
    pdl_wait();
    if (!found || slot < 0 || slot >= a.num_slots) return;
    const int group = head / (a.heads / a.groups);
    fetch_across(w.Q, a.q + (long)group * d + at.row0 * a.q_stride, a.q_stride, at.len, d);
    fetch_across(w.K, a.k + (long)group * d + at.row0 * a.k_stride, a.k_stride, at.len, d);
    fetch_along(w.V, a.v + (long)head * a.dv + col0 + at.row0 * a.v_stride, a.v_stride, at.len, cols, cp);
    const long unit = (long)blockIdx.x * a.heads + head;
    const float* U = side.U + unit * d * a.dv + col0;
    for (int i = tid; i < d * cp; i += THREADS) {
        const int kd = i / cp, c = i - kd * cp;
        if (c < cols) copy_async(w.S + i, U + (long)kd * a.dv + c);
        else w.S[i] = 0.0f;
    }
    for (int kd = tid; kd < d; kd += THREADS) {
        if (a.memory) copy_async(w.N + kd, side.u + unit * d + kd);
        else w.N[kd] = 0.0f;
    }
    const float m0 = a.memory ? side.marks[unit * 3 + 2] : 0.0f;
    if (tid == 0) w.scal[0] = m0;
    if (tid < 32) chunk_gates(a, head, at.row0, at.len, m0, w.B, w.X, w.C, w.Last, w.Floor, w.scal);
    copies_wait();
    __syncthreads();
    chunk_scores(w, d, at.len, a.q_scale);
    __syncthreads();
    chunk_read_out<J>(a, w, head, col0, cols, at.row0, at.len);
    if (a.memory && tid == 0 && blockIdx.z == 0 && at.chunk == at.chunks - 1)
        a.state[slot * a.state_len + a.m_off + head] = w.scal[2];
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
int choose_cols(int requests, int heads, int d, int dv, bool side_by_side, long* bytes) {
    int device = 0, limit = 0, sms = 0, all = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&all, cudaDevAttrMaxSharedMemoryPerMultiprocessor, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        return 0;
    int cols = dv < 64 ? dv : 64;
    // blocks that do not wait for one another hide each other's copies and gates: two a processor, while 32 columns stay
    while (side_by_side && cols > 32 && 2 * (chunk_scan_floats(d, cols) * 4 + 1024) > all) cols -= 16;
    while (cols > 16 && (chunk_scan_floats(d, cols) * 4 > limit || (long)requests * heads * ((dv + cols - 1) / cols) < sms))
        cols = cols > 32 ? cols - 16 : 16;
    *bytes = chunk_scan_floats(d, cols) * 4;
    return *bytes <= limit ? cols : 0;
}

template <typename Kernel>
int grant_shared(Kernel kernel, long bytes, long* granted) {
    if (bytes <= *granted) return 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) return launch_status();
    *granted = bytes;
    return 0;
}

#define KIRAI_BY_RUNS(runs, name) ((runs) == 1 ? name<1> : (runs) == 2 ? name<2> : (runs) == 3 ? name<3> : name<4>)

// `units` > 0: the chunks side by side, with `side`'s buffers for `units` chunks (at least tokens / 64 + requests).
int chunk_scan_launch(ChunkScan a, int requests, int units, ChunkSide side, cudaStream_t stream) {
    long bytes = 0;
    a.cols = choose_cols(units > 0 ? units : requests, a.heads, a.d, a.dv, units > 0, &bytes);
    if (a.cols <= 0) return KIRAI_ERR_UNSUPPORTED;
    const int runs = cols_pitch(a.cols) / 16;
    const int pieces = (a.dv + a.cols - 1) / a.cols;
    static long granted[3][5] = {};  // (one device a process)
    if (units > 0) {
        auto local = KIRAI_BY_RUNS(runs, chunk_local_kernel);
        auto out = KIRAI_BY_RUNS(runs, chunk_out_kernel);
        int status = grant_shared(local, bytes, &granted[1][runs]);
        if (status == 0) status = grant_shared(out, bytes, &granted[2][runs]);
        if (status == 0)
            status = launch_pdl(local, dim3(units, a.heads, pieces), dim3(THREADS), (size_t)bytes, stream, 1u, a, side, requests);
        const long entries = (long)a.d * a.dv + (a.memory ? a.d : 0);
        if (status == 0)
            status = launch_pdl(chunk_carry_kernel, dim3(requests, a.heads, (unsigned)((entries + 255) / 256)), dim3(256), 0, stream, 1u,
                                a, side, requests);
        if (status == 0)
            status = launch_pdl(out, dim3(units, a.heads, pieces), dim3(THREADS), (size_t)bytes, stream, 1u, a, side, requests);
        return status;
    }
    auto kernel = KIRAI_BY_RUNS(runs, chunk_scan_kernel);
    int status = grant_shared(kernel, bytes, &granted[0][runs]);
    if (status != 0) return status;
    status = launch_pdl(kernel, dim3(requests, a.heads, pieces), dim3(THREADS), (size_t)bytes, stream, 1u, a);
    if (status != 0 || !a.memory) return status;
    const long tail_units = (long)requests * a.heads * (a.d + 1);
    return launch_pdl(chunk_tail_kernel, dim3((unsigned)((tail_units + 255) / 256)), dim3(256), 0, stream, 1u, (const float*)a.tail,
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

// The state-space recurrence in chunks; the arguments of kirai_ssm_walk, and for the chunks side by side (units > 0)
// side_state [units, heads, N, P] and side_marks [units, heads, 3] (float32).
KIRAI_EXPORT int kirai_ssm_chunks(const float* xbc, const float* dt_raw, long dt_stride, const float* dt_bias, const float* a_log,
                                  const float* d_skip, float* state, long state_len, long ssm_off, const int* query_start,
                                  const int* slots, float* y, int requests, int heads, int groups, int N, int P, int num_slots,
                                  int units, float* side_state, float* side_marks, cudaStream_t stream) {
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
    if (units > 0 && (!side_state || !side_marks)) return KIRAI_ERR_BAD_SIZE;
    return chunk_scan_launch(a, requests, units, ChunkSide{side_state, nullptr, side_marks}, stream);
}

// The matrix memory in chunks; the arguments of kirai_matrix_memory_walk and `tail` [requests, heads, d + 1] (float32), or
// for the chunks side by side (units > 0) side_state [units, heads, d, dv], side_norm [units, heads, d], side_marks
// [units, heads, 3].
KIRAI_EXPORT int kirai_matrix_memory_chunks(const float* rows, long row_stride, const float* in_bias, const float* keep_bias,
                                            float cap, float q_scale, float* state, long state_len, const int* query_start,
                                            const int* slots, float* o, float* tail, int requests, int heads, int d, int dv,
                                            int num_slots, int units, float* side_state, float* side_norm, float* side_marks,
                                            cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (heads <= 0 || d <= 0 || dv <= 0 || !(cap > 0.0f) || (!tail && units <= 0) || (long)heads * d * dv + (long)heads * d + heads > state_len)
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
    if (units > 0 && (!side_state || !side_norm || !side_marks)) return KIRAI_ERR_BAD_SIZE;
    return chunk_scan_launch(a, requests, units, ChunkSide{side_state, side_norm, side_marks}, stream);
}
