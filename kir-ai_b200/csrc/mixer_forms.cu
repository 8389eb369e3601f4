// Row-wise kernels of mixers and norms beside those of elementwise.cu and layer_forms.cu:
//
//   * layer norm with a weight and no bias, with the residual add (and a bias of the sub-layer before) fused in:
//     (x - mean) / sqrt(var + eps) * w, var the mean of the squared deviations, statistics in 32-bit;
//   * token shift: a row h_t becomes h_t + (h_{t-1} - h_t) * mu, h_{t-1} the previous token's row as it was before
//     the replacement (a request's state slot keeps its last row between steps, zeros at its start);
//   * the minGRU recurrence S_t = (1 - z_t) S_{t-1} + z_t c_t, element by element, state in 32-bit in the slot,
//     as a walk over a request's tokens (steps of few tokens) and as a scan over pieces of SCAN_PIECE tokens
//     (prompt portions): the pieces' (product of 1 - z, end state from zero) first, then every piece's incoming
//     state, then the rows;
//   * the preparation of attention with biases, a rotation of a part of each head and a factor per head: queries
//     out (heads padded to the cache's row width), keys and values to their pages;
//   * the preparation of latent attention: RMS norms of the query latent and of the key/value latent, rotation of
//     the shared key part, the latent row to the pages (as key row [latent, rotated part] and as value row [latent]);
//   * small element-wise steps: a sigmoid gate on padded heads, a gated activation, a bias on rows.
//
// What enters a norm, a rotation or a recurrence is read in 32-bit (the products before these kernels leave 32-bit
// rows); only what a product reads next is rounded to the runtime dtype.
#include "common.cuh"

// ------------------------------------------------------------ add + layer norm
// One block per produced row.  resid[row] += delta[row] + delta_bias (when the stream is updated: no row_index);
// out[row] = LN(resid[row]) * weight.  With row_index only those rows are produced, the stream stays as it is.
// With a token shift (mu, state, slots given; a step in which every request brings ONE token, row r being request
// r's): the normed row h is mixed with the request's slot, out = h + (state[slot] - h) * mu, and the slot gets h.
struct ShiftArgs {
    const float* mu;
    float* state;
    const int* slots;
    int num_slots;
};

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
}
template <>
__device__ __forceinline__ void load4<bf16>(const bf16* p, float (&v)[4]) {
    const uint2 q = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&q.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&q.y);
    v[0] = __low2float(lo), v[1] = __high2float(lo), v[2] = __low2float(hi), v[3] = __high2float(hi);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* p, const float (&v)[4]) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 q;
    q.x = *reinterpret_cast<const uint32_t*>(&lo), q.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = q;
}

template <typename T, typename O>
__global__ void add_layernorm_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ delta_bias,
                                     const float* __restrict__ weight, O* __restrict__ out, const int* __restrict__ row_index,
                                     int hidden, float eps, ShiftArgs shift) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float row_s[];  // [hidden]
    __shared__ float scratch[32];
    const int produced = blockIdx.x;
    const size_t row = row_index ? (size_t)row_index[produced] : (size_t)produced;
    float* x = resid + row * hidden;
    const T* d = delta ? delta + row * hidden : nullptr;
    float acc = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = x[i];
        if (d) v += to_f32<T>(d[i]);
        if (delta_bias) v += delta_bias[i];
        row_s[i] = v;
        if (!row_index && (d || delta_bias)) x[i] = v;
        acc += v;
    }
    const float mean = block_sum(acc, scratch) / (float)hidden;
    float dev = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float c = row_s[i] - mean;
        dev = fmaf(c, c, dev);
    }
    const float variance = block_sum(dev, scratch) / (float)hidden + eps;
    const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
    O* dst = out + (size_t)produced * hidden;
    float* kept = nullptr;
    if (shift.mu) {
        const int slot = shift.slots[produced];
        if (slot < 0 || slot >= shift.num_slots) return;
        kept = shift.state + (size_t)slot * hidden;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float h = (row_s[i] - mean) * scale * weight[i];
        if (kept) {
            const float before = kept[i];
            kept[i] = h;
            h += (before - h) * shift.mu[i];
        }
        dst[i] = from_f32<O>(h);
    }
}

// The same with 16-byte loads and the row kept in registers (width a multiple of 4, at most 4 * VEC * blockDim values,
// every pointer on a 16-byte boundary).
template <typename T, typename O, int VEC>
__global__ void add_layernorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ delta_bias,
                                         const float* __restrict__ weight, O* __restrict__ out, const int* __restrict__ row_index,
                                         int hidden, float eps, ShiftArgs shift) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int produced = blockIdx.x;
    const size_t row = row_index ? (size_t)row_index[produced] : (size_t)produced;
    float* x = resid + row * hidden;
    const T* d = delta ? delta + row * hidden : nullptr;
    const int quads = hidden >> 2;
    float kept[VEC][4];
    float acc = 0.0f;
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = (threadIdx.x + n * blockDim.x) * 4;
        if (i < hidden) {
            load4<float>(x + i, kept[n]);
            if (d) {
                float add[4];
                load4<T>(d + i, add);
#pragma unroll
                for (int j = 0; j < 4; ++j) kept[n][j] += add[j];
            }
            if (delta_bias) {
                float add[4];
                load4<float>(delta_bias + i, add);
#pragma unroll
                for (int j = 0; j < 4; ++j) kept[n][j] += add[j];
            }
            if (!row_index && (d || delta_bias)) store4<float>(x + i, kept[n]);
            acc += (kept[n][0] + kept[n][1]) + (kept[n][2] + kept[n][3]);
        }
    }
    (void)quads;
    const float mean = block_sum(acc, scratch) / (float)hidden;
    float dev = 0.0f;
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = (threadIdx.x + n * blockDim.x) * 4;
        if (i < hidden) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                kept[n][j] -= mean;
                dev = fmaf(kept[n][j], kept[n][j], dev);
            }
        }
    }
    const float variance = block_sum(dev, scratch) / (float)hidden + eps;
    const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
    O* dst = out + (size_t)produced * hidden;
    float* slot_row = nullptr;
    if (shift.mu) {
        const int slot = shift.slots[produced];
        if (slot < 0 || slot >= shift.num_slots) return;
        slot_row = shift.state + (size_t)slot * hidden;
    }
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = (threadIdx.x + n * blockDim.x) * 4;
        if (i < hidden) {
            float w[4], h[4];
            load4<float>(weight + i, w);
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = kept[n][j] * scale * w[j];
            if (slot_row) {
                float before[4], mu[4];
                load4<float>(slot_row + i, before);
                load4<float>(shift.mu + i, mu);
                store4<float>(slot_row + i, h);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] += (before[j] - h[j]) * mu[j];
            }
            store4<O>(dst + i, h);
        }
    }
}

template <typename T, typename O>
static int add_layernorm_launch(float* resid, const void* delta, const float* delta_bias, const float* weight, void* out,
                                const int* row_index, int rows, int hidden, float eps, ShiftArgs shift, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || (size_t)hidden * sizeof(float) > 200 * 1024) return KIRAI_ERR_BAD_SIZE;
    if (shift.mu && (!shift.state || !shift.slots || row_index)) return KIRAI_ERR_BAD_SIZE;
    const bool aligned = hidden % 4 == 0 && (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)delta_bias | (uintptr_t)weight |
                                              (uintptr_t)out | (uintptr_t)shift.mu | (uintptr_t)shift.state) & 15) == 0;
    if (aligned && hidden <= 4 * 4 * 512) {
        const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
        const int vec = (hidden / 4 + threads - 1) / threads;
#define KIRAI_LN(V)                                                                                                       \
    if (vec <= V)                                                                                                         \
        return launch_pdl(add_layernorm_vec_kernel<T, O, V>, dim3(rows), dim3(threads), 0, stream, 1u, resid, (const T*)delta, \
                          delta_bias, weight, (O*)out, row_index, hidden, eps, shift)
        KIRAI_LN(1);
        KIRAI_LN(2);
        KIRAI_LN(4);
#undef KIRAI_LN
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    auto kernel = add_layernorm_kernel<T, O>;
    if (smem > 48 * 1024) {
        const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    return launch_pdl(kernel, dim3(rows), dim3(threads), smem, stream, 1u, resid, (const T*)delta, delta_bias, weight, (O*)out,
                      row_index, hidden, eps, shift);
}

// delta in the runtime dtype (f32 / bf16); the normed rows in that dtype, or (``wide``) in 32-bit for a token shift
// that runs as a kernel of its own.  shift_mu, shift_state [num_slots, hidden], slots: the fused token shift of a
// step of single tokens (all null: none).
KIRAI_EXPORT int kirai_add_layernorm_f32(float* resid, const void* delta, const float* delta_bias, const float* weight,
                                         void* out, const int* row_index, int rows, int hidden, float eps, int wide,
                                         const float* shift_mu, float* shift_state, const int* slots, int num_slots,
                                         cudaStream_t stream) {
    return add_layernorm_launch<float, float>(resid, delta, delta_bias, weight, out, row_index, rows, hidden, eps,
                                              ShiftArgs{shift_mu, shift_state, slots, num_slots}, stream);
}
KIRAI_EXPORT int kirai_add_layernorm_bf16(float* resid, const void* delta, const float* delta_bias, const float* weight,
                                          void* out, const int* row_index, int rows, int hidden, float eps, int wide,
                                          const float* shift_mu, float* shift_state, const int* slots, int num_slots,
                                          cudaStream_t stream) {
    const ShiftArgs shift{shift_mu, shift_state, slots, num_slots};
    if (wide) return add_layernorm_launch<bf16, float>(resid, delta, delta_bias, weight, out, row_index, rows, hidden, eps, shift, stream);
    return add_layernorm_launch<bf16, bf16>(resid, delta, delta_bias, weight, out, row_index, rows, hidden, eps, shift, stream);
}

// ------------------------------------------------------------------ token shift
// One block per token row.  The row before a request's first row of this step is its slot of `state`; the block of
// that first row reads the slot and then puts the request's last row of this step there, so no slot is read and
// written by different blocks.
template <typename O, bool VEC>
__global__ void token_shift_kernel(const float* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state,
                                   const int* __restrict__ request_of_token, const int* __restrict__ query_start,
                                   const int* __restrict__ slots, O* __restrict__ out, int hidden, int num_slots) {
    pdl_launch_dependents();
    const int row = blockIdx.x;
    const int request = request_of_token[row];
    const int first = query_start[request], last = query_start[request + 1] - 1;
    const int slot = slots[request];
    pdl_wait();
    const float* cur = h + (size_t)row * hidden;
    O* dst = out + (size_t)row * hidden;
    const bool is_first = row == first;
    if (is_first && (slot < 0 || slot >= num_slots)) return;
    float* kept = is_first ? state + (size_t)slot * hidden : nullptr;
    const float* prev = is_first ? kept : cur - hidden;
    const float* end = h + (size_t)last * hidden;
    if (VEC) {
        // four columns at a time (the width and every pointer allow 16-byte accesses; see the launch)
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float c[4], p[4], m[4];
            load4<float>(cur + i, c);
            load4<float>(prev + i, p);
            load4<float>(mu + i, m);
            if (is_first) {
                float e[4];
                load4<float>(end + i, e);
                store4<float>(kept + i, e);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) c[j] += (p[j] - c[j]) * m[j];
            store4<O>(dst + i, c);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            const float c = cur[i];
            const float p = prev[i];
            if (is_first) kept[i] = end[i];
            dst[i] = from_f32<O>(c + (p - c) * mu[i]);
        }
    }
}

template <typename O>
static int token_shift_launch(const float* h, const float* mu, float* state, const int* request_of_token,
                              const int* query_start, const int* slots, void* out, int rows, int hidden, int num_slots,
                              cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0) return KIRAI_ERR_BAD_SIZE;
    const int threads = hidden >= 4096 ? 256 : 128;
    const bool vec = hidden % 4 == 0 && (((uintptr_t)h | (uintptr_t)mu | (uintptr_t)state | (uintptr_t)out) & 15) == 0;
    return launch_pdl(vec ? token_shift_kernel<O, true> : token_shift_kernel<O, false>, dim3(rows), dim3(threads), 0, stream, 1u, h,
                      mu, state, request_of_token, query_start, slots, (O*)out, hidden, num_slots);
}

KIRAI_EXPORT int kirai_token_shift_f32(const float* h, const float* mu, float* state, const int* request_of_token,
                                       const int* query_start, const int* slots, void* out, int rows, int hidden,
                                       int num_slots, cudaStream_t stream) {
    return token_shift_launch<float>(h, mu, state, request_of_token, query_start, slots, out, rows, hidden, num_slots, stream);
}
KIRAI_EXPORT int kirai_token_shift_bf16(const float* h, const float* mu, float* state, const int* request_of_token,
                                        const int* query_start, const int* slots, void* out, int rows, int hidden,
                                        int num_slots, cudaStream_t stream) {
    return token_shift_launch<bf16>(h, mu, state, request_of_token, query_start, slots, out, rows, hidden, num_slots, stream);
}

// ----------------------------------------------------------------------- minGRU
// zxg [T, 3 W] (float32): the stacked product, columns [0, W) the gate's, [W, 2W) the candidate's, [2W, 3W) the
// output gate's pre-activations.  z = sigmoid(. + zb); u = . + xb; c = u + 1/2 where u >= 0, sigmoid(u) below;
// S <- (1 - z) S + z c; out = S * silu(g).
__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }
// The same from the fast exponential and division (relative error about 1e-6): for the serving path, whose gates'
// pre-activations come out of bfloat16 products; the 32-bit path keeps the exact forms.
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
template <bool FAST>
__device__ __forceinline__ float sigmoid_as(float x) { return FAST ? sigmoid_fast(x) : sigmoid_f32(x); }
template <typename O>
struct serves_rounded { static constexpr bool value = false; };
template <>
struct serves_rounded<bf16> { static constexpr bool value = true; };

template <bool FAST>
__device__ __forceinline__ void mingru_terms(const float* __restrict__ row, int width, int ch, float zb, float xb, float& z, float& c) {
    z = sigmoid_as<FAST>(row[ch] + zb);
    const float u = row[width + ch] + xb;
    c = u >= 0.0f ? u + 0.5f : sigmoid_as<FAST>(u);
}

// A thread per (request, channel) walks the request's tokens of this step in order.
template <typename O>
__global__ void mingru_walk_kernel(const float* __restrict__ zxg, long row_stride, const float* __restrict__ z_bias,
                                   const float* __restrict__ x_bias, float* __restrict__ state,
                                   const int* __restrict__ query_start, const int* __restrict__ slots, O* __restrict__ out,
                                   int width, int num_slots) {
    pdl_launch_dependents();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int request = blockIdx.y;
    const int first = query_start[request], end = query_start[request + 1];
    const int slot = slots[request];
    if (ch >= width || slot < 0 || slot >= num_slots) return;
    const float zb = z_bias ? z_bias[ch] : 0.0f, xb = x_bias ? x_bias[ch] : 0.0f;
    pdl_wait();
    float s = state[(size_t)slot * width + ch];
#pragma unroll 8
    for (int t = first; t < end; ++t) {
        const float* row = zxg + (size_t)t * row_stride;
        float z, c;
        mingru_terms<serves_rounded<O>::value>(row, width, ch, zb, xb, z, c);
        s = fmaf(z, c - s, s);  // (1 - z) s + z c
        const float g = row[2 * width + ch];
        out[(size_t)t * width + ch] = from_f32<O>(s * g * sigmoid_as<serves_rounded<O>::value>(g));
    }
    state[(size_t)slot * width + ch] = s;
}

#define SCAN_PIECE 32

// Pieces of SCAN_PIECE tokens, counted from the request's first row of this step.  Pass 1: a thread per (piece,
// channel) leaves the piece's decay (product of 1 - z) and its end state from a zero start.
template <bool FAST>
__global__ void mingru_piece_kernel(const float* __restrict__ zxg, long row_stride, const float* __restrict__ z_bias,
                                    const float* __restrict__ x_bias, const int* __restrict__ query_start,
                                    float* __restrict__ decay, float* __restrict__ ends, int width, int max_pieces) {
    pdl_launch_dependents();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int piece = blockIdx.y, request = blockIdx.z;
    const int first = query_start[request] + piece * SCAN_PIECE;
    const int end = min(query_start[request + 1], first + SCAN_PIECE);
    if (ch >= width || first >= end) return;
    const float zb = z_bias ? z_bias[ch] : 0.0f, xb = x_bias ? x_bias[ch] : 0.0f;
    pdl_wait();
    float a = 1.0f, s = 0.0f;
#pragma unroll 8
    for (int t = first; t < end; ++t) {
        float z, c;
        mingru_terms<FAST>(zxg + (size_t)t * row_stride, width, ch, zb, xb, z, c);
        a *= 1.0f - z;
        s = fmaf(z, c - s, s);
    }
    const size_t at = ((size_t)request * max_pieces + piece) * width + ch;
    decay[at] = a;
    ends[at] = s;
}

// Pass 2: a thread per (request, channel) turns the pieces' end states into the state each piece starts from
// (in place in `ends`) and leaves the request's new state in its slot.
__global__ void mingru_carry_kernel(const float* __restrict__ decay, float* __restrict__ ends, float* __restrict__ state,
                                    const int* __restrict__ query_start, const int* __restrict__ slots, int width,
                                    int max_pieces, int num_slots) {
    pdl_launch_dependents();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int request = blockIdx.y;
    const int tokens = query_start[request + 1] - query_start[request];
    const int pieces = (tokens + SCAN_PIECE - 1) / SCAN_PIECE;
    const int slot = slots[request];
    if (ch >= width || slot < 0 || slot >= num_slots) return;
    pdl_wait();
    float s = state[(size_t)slot * width + ch];
    // eight pieces' terms are asked for at once, so that the chain of multiply-adds does not wait on each load
    for (int p0 = 0; p0 < pieces; p0 += 8) {
        float a[8], b[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const size_t at = ((size_t)request * max_pieces + min(p0 + k, pieces - 1)) * width + ch;
            a[k] = decay[at];
            b[k] = ends[at];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (p0 + k < pieces) {
                ends[((size_t)request * max_pieces + p0 + k) * width + ch] = s;
                s = fmaf(a[k], s, b[k]);
            }
        }
    }
    state[(size_t)slot * width + ch] = s;
}

// Pass 3: a thread per (piece, channel) walks its piece again from the incoming state and writes the rows.
template <typename O>
__global__ void mingru_rows_kernel(const float* __restrict__ zxg, long row_stride, const float* __restrict__ z_bias,
                                   const float* __restrict__ x_bias, const int* __restrict__ query_start,
                                   const float* __restrict__ incoming, O* __restrict__ out, int width, int max_pieces) {
    pdl_launch_dependents();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int piece = blockIdx.y, request = blockIdx.z;
    const int first = query_start[request] + piece * SCAN_PIECE;
    const int end = min(query_start[request + 1], first + SCAN_PIECE);
    if (ch >= width || first >= end) return;
    const float zb = z_bias ? z_bias[ch] : 0.0f, xb = x_bias ? x_bias[ch] : 0.0f;
    pdl_wait();
    float s = incoming[((size_t)request * max_pieces + piece) * width + ch];
#pragma unroll 8
    for (int t = first; t < end; ++t) {
        const float* row = zxg + (size_t)t * row_stride;
        float z, c;
        mingru_terms<serves_rounded<O>::value>(row, width, ch, zb, xb, z, c);
        s = fmaf(z, c - s, s);
        const float g = row[2 * width + ch];
        out[(size_t)t * width + ch] = from_f32<O>(s * g * sigmoid_as<serves_rounded<O>::value>(g));
    }
}

// scratch: 2 * requests * ceil(max_query_len / SCAN_PIECE) * width floats when max_query_len > walk_limit, else unused.
template <typename O>
static int mingru_launch(const float* zxg, long row_stride, const float* z_bias, const float* x_bias, float* state,
                         const int* query_start, const int* slots, void* out, float* scratch, int requests,
                         int max_query_len, int width, int num_slots, int walk_limit, cudaStream_t stream) {
    if (requests <= 0 || max_query_len <= 0) return 0;
    if (width <= 0 || requests > 65535) return KIRAI_ERR_BAD_SIZE;
    const int threads = 128;
    const unsigned blocks = (unsigned)((width + threads - 1) / threads);
    if (max_query_len <= walk_limit || !scratch) {
        return launch_pdl(mingru_walk_kernel<O>, dim3(blocks, requests), dim3(threads), 0, stream, 1u, zxg, row_stride, z_bias,
                          x_bias, state, query_start, slots, (O*)out, width, num_slots);
    }
    const int max_pieces = (max_query_len + SCAN_PIECE - 1) / SCAN_PIECE;
    if (max_pieces > 65535) return KIRAI_ERR_BAD_SIZE;
    float* decay = scratch;
    float* ends = scratch + (size_t)requests * max_pieces * width;
    int status = launch_pdl(mingru_piece_kernel<serves_rounded<O>::value>, dim3(blocks, max_pieces, requests), dim3(threads), 0, stream, 1u, zxg, row_stride,
                            z_bias, x_bias, query_start, decay, ends, width, max_pieces);
    if (status) return status;
    status = launch_pdl(mingru_carry_kernel, dim3(blocks, requests), dim3(threads), 0, stream, 1u, (const float*)decay, ends, state,
                        query_start, slots, width, max_pieces, num_slots);
    if (status) return status;
    return launch_pdl(mingru_rows_kernel<O>, dim3(blocks, max_pieces, requests), dim3(threads), 0, stream, 1u, zxg, row_stride,
                      z_bias, x_bias, query_start, (const float*)ends, (O*)out, width, max_pieces);
}

KIRAI_EXPORT int kirai_mingru_piece_tokens() { return SCAN_PIECE; }

KIRAI_EXPORT int kirai_mingru_f32(const float* zxg, long row_stride, const float* z_bias, const float* x_bias, float* state,
                                  const int* query_start, const int* slots, void* out, float* scratch, int requests,
                                  int max_query_len, int width, int num_slots, int walk_limit, cudaStream_t stream) {
    return mingru_launch<float>(zxg, row_stride, z_bias, x_bias, state, query_start, slots, out, scratch, requests,
                                max_query_len, width, num_slots, walk_limit, stream);
}
KIRAI_EXPORT int kirai_mingru_bf16(const float* zxg, long row_stride, const float* z_bias, const float* x_bias, float* state,
                                   const int* query_start, const int* slots, void* out, float* scratch, int requests,
                                   int max_query_len, int width, int num_slots, int walk_limit, cudaStream_t stream) {
    return mingru_launch<bf16>(zxg, row_stride, z_bias, x_bias, state, query_start, slots, out, scratch, requests,
                               max_query_len, width, num_slots, walk_limit, stream);
}

// ------------------------------------- attention preparation: bias, rotation, factor
// One block per token.  qkv row (float32): nq heads of dk, then nkv heads of dk, then nkv heads of dv (further
// columns, as an output gate's, are not touched).  Columns [rot_off, rot_off + rot_dims) of every query and key head
// are rotated, column i of the first half with column i + rot_dims / 2, by position * inv_freq[i]; query head h is
// multiplied by q_factor[h]; cosine and sine are multiplied by rot_amp (1: a plain rotation).  Queries leave as [nq, dpad] rows with zeros beyond dk; keys and values go to the
// token's row of its page, cache [pages, 2, nkv, page, dpad].
template <typename T>
__device__ __forceinline__ void rotate_head_to(const float* __restrict__ src, const float* __restrict__ bias, T* __restrict__ dst,
                                               int width, int rot_off, int rot_dims, const float* __restrict__ inv_freq,
                                               float pos, float factor, int lane, int lanes, float rot_amp = 1.0f) {
    const int half = rot_dims >> 1;
    for (int c = lane; c < width; c += lanes) {
        const int r = c - rot_off;
        if (r >= 0 && r < rot_dims) {
            if (r >= half) continue;  // written with its partner
            const float u = src[c] + (bias ? bias[c] : 0.0f);
            const float v = src[c + half] + (bias ? bias[c + half] : 0.0f);
            float sn, cs;
            sincosf(pos * inv_freq[r], &sn, &cs);
            sn *= rot_amp;
            cs *= rot_amp;
            dst[c] = from_f32<T>((u * cs - v * sn) * factor);
            dst[c + half] = from_f32<T>((v * cs + u * sn) * factor);
        } else {
            dst[c] = from_f32<T>((src[c] + (bias ? bias[c] : 0.0f)) * factor);
        }
    }
}

template <typename T>
__global__ void qkv_rope_write_kernel(const float* __restrict__ qkv, long qkv_stride, const float* __restrict__ q_bias,
                                      const float* __restrict__ k_bias, const float* __restrict__ v_bias,
                                      const float* __restrict__ q_factor, const float* __restrict__ inv_freq, int rot_off,
                                      int rot_dims, float rot_amp, T* __restrict__ q_out, T* __restrict__ cache,
                                      const int* __restrict__ block_table, const int* __restrict__ request_of_token,
                                      const int* __restrict__ positions, int q_heads, int kv_heads, int dk, int dv, int dpad,
                                      int page_size, int table_width, int num_pages, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    const int token = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int position = positions[token];
    long page_base = -1;
    if (kv_heads > 0) {
        const int logical = position / page_size;
        const int page = logical < table_width ? block_table[(long)request_of_token[token] * table_width + logical] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(error_flag, KIRAI_FLAG_NO_PAGE_WRITE);
        } else {
            page_base = (((long)page * 2) * kv_heads * page_size + (position % page_size)) * (long)dpad;
        }
    }
    pdl_wait();
    const float pos = (float)position;
    const float* src = qkv + (size_t)token * qkv_stride;
    const long head_rows = (long)page_size * dpad;
    // a warp per head: query heads, then key heads, then value heads
    for (int unit = warp; unit < q_heads + 2 * kv_heads; unit += warps) {
        if (unit < q_heads) {
            T* dst = q_out + ((size_t)token * q_heads + unit) * dpad;
            rotate_head_to<T>(src + (size_t)unit * dk, q_bias ? q_bias + (size_t)unit * dk : nullptr, dst, dk, rot_off, rot_dims,
                              inv_freq, pos, q_factor ? q_factor[unit] : 1.0f, lane, 32, rot_amp);
            for (int c = dk + lane; c < dpad; c += 32) dst[c] = from_f32<T>(0.0f);
        } else if (page_base >= 0 && unit < q_heads + kv_heads) {
            const int head = unit - q_heads;
            rotate_head_to<T>(src + (size_t)q_heads * dk + (size_t)head * dk, k_bias ? k_bias + (size_t)head * dk : nullptr,
                              cache + page_base + head * head_rows, dk, rot_off, rot_dims, inv_freq, pos, 1.0f, lane, 32, rot_amp);
        } else if (page_base >= 0) {
            const int head = unit - q_heads - kv_heads;
            const float* v = src + (size_t)(q_heads + kv_heads) * dk + (size_t)head * dv;
            T* dst = cache + page_base + (long)kv_heads * head_rows + head * head_rows;
            for (int c = lane; c < dv; c += 32) dst[c] = from_f32<T>(v[c] + (v_bias ? v_bias[(size_t)head * dv + c] : 0.0f));
        }
    }
}

template <typename T>
static int qkv_rope_write_launch(const float* qkv, long qkv_stride, const float* q_bias, const float* k_bias, const float* v_bias,
                                 const float* q_factor, const float* inv_freq, int rot_off, int rot_dims, float rot_amp, void* q_out, void* cache,
                                 const int* block_table, const int* request_of_token, const int* positions, int tokens,
                                 int q_heads, int kv_heads, int dk, int dv, int dpad, int page_size, int table_width,
                                 int num_pages, int* error_flag, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (q_heads <= 0 || kv_heads < 0 || dk <= 0 || dv <= 0 || dpad < dk || dpad < dv || page_size <= 0) return KIRAI_ERR_BAD_SIZE;
    if (rot_dims < 0 || rot_dims % 2 || rot_off < 0 || rot_off + rot_dims > dk || (rot_dims > 0 && !inv_freq)) return KIRAI_ERR_BAD_SIZE;
    if (kv_heads > 0 && !cache) return KIRAI_ERR_BAD_SIZE;
    const int units = q_heads + 2 * kv_heads;
    const int threads = units >= 8 ? 256 : 32 * units;
    return launch_pdl(qkv_rope_write_kernel<T>, dim3(tokens), dim3(threads), 0, stream, 1u, qkv, qkv_stride, q_bias, k_bias, v_bias,
                      q_factor, inv_freq, rot_off, rot_dims, rot_amp, (T*)q_out, (T*)cache, block_table, request_of_token, positions,
                      q_heads, kv_heads, dk, dv, dpad, page_size, table_width, num_pages, error_flag);
}

KIRAI_EXPORT int kirai_qkv_rope_write_f32(const float* qkv, long qkv_stride, const float* q_bias, const float* k_bias,
                                          const float* v_bias, const float* q_factor, const float* inv_freq, int rot_off,
                                          int rot_dims, float rot_amp, void* q_out, void* cache, const int* block_table,
                                          const int* request_of_token, const int* positions, int tokens, int q_heads,
                                          int kv_heads, int dk, int dv, int dpad, int page_size, int table_width,
                                          int num_pages, int* error_flag, cudaStream_t stream) {
    return qkv_rope_write_launch<float>(qkv, qkv_stride, q_bias, k_bias, v_bias, q_factor, inv_freq, rot_off, rot_dims, rot_amp, q_out,
                                        cache, block_table, request_of_token, positions, tokens, q_heads, kv_heads, dk, dv, dpad,
                                        page_size, table_width, num_pages, error_flag, stream);
}
KIRAI_EXPORT int kirai_qkv_rope_write_bf16(const float* qkv, long qkv_stride, const float* q_bias, const float* k_bias,
                                           const float* v_bias, const float* q_factor, const float* inv_freq, int rot_off,
                                           int rot_dims, float rot_amp, void* q_out, void* cache, const int* block_table,
                                           const int* request_of_token, const int* positions, int tokens, int q_heads,
                                           int kv_heads, int dk, int dv, int dpad, int page_size, int table_width,
                                           int num_pages, int* error_flag, cudaStream_t stream) {
    return qkv_rope_write_launch<bf16>(qkv, qkv_stride, q_bias, k_bias, v_bias, q_factor, inv_freq, rot_off, rot_dims, rot_amp, q_out,
                                       cache, block_table, request_of_token, positions, tokens, q_heads, kv_heads, dk, dv, dpad,
                                       page_size, table_width, num_pages, error_flag, stream);
}

// --------------------------------------------------- latent attention preparation
// One block per token.  down row (float32): q_rank columns of the query latent, kv_rank of the key/value latent,
// rot_dims of the key part that all heads share.  Both latents are divided by their root mean square (eps inside
// the root) and multiplied by a weight per column; the shared key part is rotated whole (column i with column
// i + rot_dims / 2, cosine and sine times rot_amp).  The query latent leaves as [q_rank] in the runtime dtype; the page row of the token gets
// [latent, rotated part] as its key row and [latent] as its value row (cache [pages, 2, 1, page, dpad], the rest of
// a row stays zero).
template <typename T>
__global__ void latent_prepare_kernel(const float* __restrict__ down, long down_stride, const float* __restrict__ q_weight,
                                      const float* __restrict__ kv_weight, const float* __restrict__ inv_freq, float rot_amp,
                                      float eps, T* __restrict__ q_latent, T* __restrict__ cache, const int* __restrict__ block_table,
                                      const int* __restrict__ request_of_token, const int* __restrict__ positions, int q_rank,
                                      int kv_rank, int rot_dims, int dpad, int page_size, int table_width, int num_pages,
                                      int* __restrict__ error_flag) {
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const int token = blockIdx.x;
    const int position = positions[token];
    long page_base = -1;
    {
        const int logical = position / page_size;
        const int page = logical < table_width ? block_table[(long)request_of_token[token] * table_width + logical] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(error_flag, KIRAI_FLAG_NO_PAGE_WRITE);
        } else {
            page_base = (((long)page * 2) * page_size + (position % page_size)) * (long)dpad;
        }
    }
    pdl_wait();
    const float* src = down + (size_t)token * down_stride;
    float q_acc = 0.0f, kv_acc = 0.0f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) q_acc = fmaf(src[i], src[i], q_acc);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) kv_acc = fmaf(src[q_rank + i], src[q_rank + i], kv_acc);
    const float q_var = q_rank > 0 ? block_sum(q_acc, scratch) / (float)q_rank + eps : 1.0f;
    const float kv_var = block_sum(kv_acc, scratch) / (float)kv_rank + eps;
    const float q_scale = q_var == 0.0f ? 0.0f : 1.0f / sqrtf(q_var);
    const float kv_scale = kv_var == 0.0f ? 0.0f : 1.0f / sqrtf(kv_var);
    T* q_dst = q_latent + (size_t)token * q_rank;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) q_dst[i] = from_f32<T>(src[i] * q_scale * q_weight[i]);
    if (page_base < 0) return;
    T* key = cache + page_base;
    T* value = cache + page_base + (long)page_size * dpad;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
        const T c = from_f32<T>(src[q_rank + i] * kv_scale * kv_weight[i]);
        key[i] = c;
        value[i] = c;
    }
    const int half = rot_dims >> 1;
    const float pos = (float)position;
    const float* shared_part = src + q_rank + kv_rank;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float u = shared_part[i], v = shared_part[i + half];
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        sn *= rot_amp;
        cs *= rot_amp;
        key[kv_rank + i] = from_f32<T>(u * cs - v * sn);
        key[kv_rank + i + half] = from_f32<T>(v * cs + u * sn);
    }
}

template <typename T>
static int latent_prepare_launch(const float* down, long down_stride, const float* q_weight, const float* kv_weight,
                                 const float* inv_freq, float rot_amp, float eps, void* q_latent, void* cache, const int* block_table,
                                 const int* request_of_token, const int* positions, int tokens, int q_rank, int kv_rank,
                                 int rot_dims, int dpad, int page_size, int table_width, int num_pages, int* error_flag,
                                 cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (q_rank < 0 || kv_rank <= 0 || rot_dims < 0 || rot_dims % 2 || dpad < kv_rank + rot_dims || page_size <= 0 || !cache)
        return KIRAI_ERR_BAD_SIZE;
    const int threads = (q_rank + kv_rank) >= 1024 ? 256 : 128;
    return launch_pdl(latent_prepare_kernel<T>, dim3(tokens), dim3(threads), 0, stream, 1u, down, down_stride, q_weight, kv_weight,
                      inv_freq, rot_amp, eps, (T*)q_latent, (T*)cache, block_table, request_of_token, positions, q_rank, kv_rank, rot_dims,
                      dpad, page_size, table_width, num_pages, error_flag);
}

KIRAI_EXPORT int kirai_latent_prepare_f32(const float* down, long down_stride, const float* q_weight, const float* kv_weight,
                                          const float* inv_freq, float rot_amp, float eps, void* q_latent, void* cache, const int* block_table,
                                          const int* request_of_token, const int* positions, int tokens, int q_rank,
                                          int kv_rank, int rot_dims, int dpad, int page_size, int table_width, int num_pages,
                                          int* error_flag, cudaStream_t stream) {
    return latent_prepare_launch<float>(down, down_stride, q_weight, kv_weight, inv_freq, rot_amp, eps, q_latent, cache, block_table,
                                        request_of_token, positions, tokens, q_rank, kv_rank, rot_dims, dpad, page_size,
                                        table_width, num_pages, error_flag, stream);
}
KIRAI_EXPORT int kirai_latent_prepare_bf16(const float* down, long down_stride, const float* q_weight, const float* kv_weight,
                                           const float* inv_freq, float rot_amp, float eps, void* q_latent, void* cache, const int* block_table,
                                           const int* request_of_token, const int* positions, int tokens, int q_rank,
                                           int kv_rank, int rot_dims, int dpad, int page_size, int table_width, int num_pages,
                                           int* error_flag, cudaStream_t stream) {
    return latent_prepare_launch<bf16>(down, down_stride, q_weight, kv_weight, inv_freq, rot_amp, eps, q_latent, cache, block_table,
                                       request_of_token, positions, tokens, q_rank, kv_rank, rot_dims, dpad, page_size,
                                       table_width, num_pages, error_flag, stream);
}

// ------------------------------------------------- a product per head, then a gate
// x [T, heads, pad] holds K used columns a head; w [heads, N, K] one matrix a head; out [T, heads * N]:
//   out[t, h * N + v] = (sum_k w[h, v, k] x[t, h, k]) * sigmoid(gate[t, h * N + v])        (no gate: the product alone)
// in 32-bit accumulation.  This is what latent attention needs between its attention over the shared latent and its
// output projection when the heads' values pass a gate: the heads' sums of latents go through each head's value
// matrix.  A block takes HEAD_TOKENS tokens of one head and a run of output columns; the tokens' rows lie in shared
// memory in 32-bit, a warp takes one output column at a time, its lanes stride over k (the matrix row is read
// coalesced, once per block) and keep one partial sum a token.
#define HEAD_TOKENS 16
#define HEAD_K_PIECE 512
template <typename T>
__global__ void __launch_bounds__(256)
head_linear_gate_kernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ gate, long gate_stride,
                        T* __restrict__ out, int tokens, int heads, int pad, int K, int N, int columns_a_block) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float rows_s[HEAD_TOKENS][HEAD_K_PIECE];
    const int head = blockIdx.y;
    const int first = blockIdx.x * HEAD_TOKENS;
    const int count = min(HEAD_TOKENS, tokens - first);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int col_lo = blockIdx.z * columns_a_block, col_hi = min(N, col_lo + columns_a_block);
    for (int v0 = col_lo; v0 < col_hi; v0 += warps) {
        // every warp walks the same k pieces, so the block meets at the barriers whatever its column
        const int v = v0 + warp;
        float acc[HEAD_TOKENS];
#pragma unroll
        for (int t = 0; t < HEAD_TOKENS; ++t) acc[t] = 0.0f;
        for (int k0 = 0; k0 < K; k0 += HEAD_K_PIECE) {
            const int piece = min(HEAD_K_PIECE, K - k0);
            if (K > HEAD_K_PIECE || v0 == col_lo) {
                __syncthreads();
                for (int i = threadIdx.x; i < HEAD_TOKENS * piece; i += blockDim.x) {
                    const int t = i / piece, k = i - t * piece;
                    rows_s[t][k] = t < count ? to_f32<T>(x[((size_t)(first + t) * heads + head) * pad + k0 + k]) : 0.0f;
                }
                __syncthreads();
            }
            if (v < col_hi) {
                const T* row = w + ((size_t)head * N + v) * K + k0;
                for (int k = lane; k < piece; k += 32) {
                    const float weight = to_f32<T>(row[k]);
#pragma unroll
                    for (int t = 0; t < HEAD_TOKENS; ++t) acc[t] = fmaf(weight, rows_s[t][k], acc[t]);
                }
            }
        }
        if (v < col_hi) {
#pragma unroll
            for (int t = 0; t < HEAD_TOKENS; ++t) {
                const float total = warp_sum(acc[t]);
                if (lane == (t & 31) && t < count) {
                    const size_t at = (size_t)head * N + v;
                    float value = total;
                    if (gate) value *= 1.0f / (1.0f + expf(-gate[(size_t)(first + t) * gate_stride + at]));
                    out[(size_t)(first + t) * heads * N + at] = from_f32<T>(value);
                }
            }
        }
    }
}

template <typename T>
static int head_linear_gate_launch(const void* x, const void* w, const float* gate, long gate_stride, void* out, int tokens,
                                   int heads, int pad, int K, int N, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || heads > 65535 || K <= 0 || N <= 0 || pad < K) return KIRAI_ERR_BAD_SIZE;
    const int tiles = (tokens + HEAD_TOKENS - 1) / HEAD_TOKENS;
    // few tokens: a head's columns are cut over several blocks, so that the matrices are read by enough of them
    int cuts = 1;
    while ((long)tiles * heads * cuts < 296 && N / (cuts * 2) >= 8 && cuts < 64) cuts *= 2;
    const int columns = (N + cuts - 1) / cuts;
    return launch_pdl(head_linear_gate_kernel<T>, dim3(tiles, heads, (N + columns - 1) / columns), dim3(256), 0, stream, 1u,
                      (const T*)x, (const T*)w, gate, gate_stride, (T*)out, tokens, heads, pad, K, N, columns);
}

KIRAI_EXPORT int kirai_head_linear_gate_f32(const void* x, const void* w, const float* gate, long gate_stride, void* out, int tokens,
                                            int heads, int pad, int K, int N, cudaStream_t stream) {
    return head_linear_gate_launch<float>(x, w, gate, gate_stride, out, tokens, heads, pad, K, N, stream);
}
KIRAI_EXPORT int kirai_head_linear_gate_bf16(const void* x, const void* w, const float* gate, long gate_stride, void* out, int tokens,
                                             int heads, int pad, int K, int N, cudaStream_t stream) {
    return head_linear_gate_launch<bf16>(x, w, gate, gate_stride, out, tokens, heads, pad, K, N, stream);
}

// For many tokens the same product runs on the tensor cores as a grouped product whose groups are the heads: the
// attention's rows [T, heads, pad] are laid out head by head ([heads, Tpad, pad], Tpad a multiple of 128, zero rows
// behind a head's last token), every 128-row tile is multiplied with its head's matrix, and the gate kernel brings
// the 32-bit result [heads, Tpad, N] back token by token, times sigmoid(gate), in bfloat16.
__global__ void head_major_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, int tokens, int padded_tokens, int heads,
                                  int pad) {
    pdl_launch_dependents();
    pdl_wait();
    const int chunks = pad >> 3;  // 16-byte pieces of a row
    const long total = (long)heads * padded_tokens * chunks;
    for (long at = (long)blockIdx.x * blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x) {
        const int c = (int)(at % chunks);
        const long row = at / chunks;
        const int t = (int)(row % padded_tokens), h = (int)(row / padded_tokens);
        uint4 value = make_uint4(0u, 0u, 0u, 0u);
        if (t < tokens) value = reinterpret_cast<const uint4*>(x + ((size_t)t * heads + h) * pad)[c];
        reinterpret_cast<uint4*>(out + (size_t)row * pad)[c] = value;
    }
}

KIRAI_EXPORT int kirai_head_major_bf16(const void* x, void* out, int tokens, int padded_tokens, int heads, int pad,
                                       cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || pad <= 0 || padded_tokens < tokens) return KIRAI_ERR_BAD_SIZE;
    if (pad % 8 != 0 || (((uintptr_t)x | (uintptr_t)out) & 15) != 0) return KIRAI_ERR_BAD_ALIGN;
    const long total = (long)heads * padded_tokens * (pad / 8);
    const unsigned blocks = (unsigned)min((total + 255) / 256, (long)148 * 32);
    return launch_pdl(head_major_kernel, dim3(blocks), dim3(256), 0, stream, 1u, (const bf16*)x, (bf16*)out, tokens, padded_tokens,
                      heads, pad);
}

__global__ void head_gate_rows_kernel(const float* __restrict__ y, const float* __restrict__ gate, long gate_stride,
                                      bf16* __restrict__ out, int tokens, int padded_tokens, int heads, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const long total = (long)tokens * heads * n;
    for (long at = (long)blockIdx.x * blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x) {
        const int v = (int)(at % n);
        const long rest = at / n;
        const int h = (int)(rest % heads), t = (int)(rest / heads);
        float value = y[((size_t)h * padded_tokens + t) * n + v];
        if (gate) value *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + (size_t)h * n + v]));
        out[at] = __float2bfloat16_rn(value);
    }
}

// The same, four columns a thread (n and the gate's row stride multiples of 4, 16-byte aligned buffers).
__global__ void head_gate_rows_vec_kernel(const float* __restrict__ y, const float* __restrict__ gate, long gate_stride,
                                          bf16* __restrict__ out, int tokens, int padded_tokens, int heads, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int quads = n >> 2;
    const long total = (long)tokens * heads * quads;
    for (long at = (long)blockIdx.x * blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x) {
        const int q = (int)(at % quads);
        const long rest = at / quads;
        const int h = (int)(rest % heads), t = (int)(rest / heads);
        float4 value = reinterpret_cast<const float4*>(y + ((size_t)h * padded_tokens + t) * n)[q];
        if (gate) {
            const float4 g = reinterpret_cast<const float4*>(gate + (size_t)t * gate_stride + (size_t)h * n)[q];
            value.x *= 1.0f / (1.0f + expf(-g.x)), value.y *= 1.0f / (1.0f + expf(-g.y));
            value.z *= 1.0f / (1.0f + expf(-g.z)), value.w *= 1.0f / (1.0f + expf(-g.w));
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(value.x, value.y), hi = __floats2bfloat162_rn(value.z, value.w);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        reinterpret_cast<uint2*>(out)[at] = packed;
    }
}

KIRAI_EXPORT int kirai_head_gate_rows_bf16(const float* y, const float* gate, long gate_stride, void* out, int tokens,
                                           int padded_tokens, int heads, int n, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || n <= 0 || padded_tokens < tokens) return KIRAI_ERR_BAD_SIZE;
    if (n % 4 == 0 && gate_stride % 4 == 0 && (((uintptr_t)y | (uintptr_t)gate | (uintptr_t)out) & 15) == 0) {
        const long pieces = (long)tokens * heads * (n / 4);
        const unsigned vec_blocks = (unsigned)min((pieces + 255) / 256, (long)148 * 32);
        return launch_pdl(head_gate_rows_vec_kernel, dim3(vec_blocks), dim3(256), 0, stream, 1u, y, gate, gate_stride, (bf16*)out,
                          tokens, padded_tokens, heads, n);
    }
    const long total = (long)tokens * heads * n;
    const unsigned blocks = (unsigned)min((total + 255) / 256, (long)148 * 32);
    return launch_pdl(head_gate_rows_kernel, dim3(blocks), dim3(256), 0, stream, 1u, y, gate, gate_stride, (bf16*)out, tokens,
                      padded_tokens, heads, n);
}

// ------------------------------------------------------------- element-wise steps
// x [T, heads, dpad] (in place) *= sigmoid(gate[T, heads * used]) on the first `used` columns of every head; gate is
// a run of columns of a 32-bit product (row stride gate_stride).
template <typename T, bool VEC>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, const float* __restrict__ gate, long gate_stride, long rows, int heads,
                                    int used, int dpad) {
    pdl_launch_dependents();
    pdl_wait();
    const long per_row = (long)heads * used;
    if (VEC) {
        // four columns of one head at a time (used, dpad, the gate's stride and the pointers allow 16-byte accesses)
        const long quads = rows * per_row / 4;
        for (long at = blockIdx.x * (long)blockDim.x + threadIdx.x; at < quads; at += (long)gridDim.x * blockDim.x) {
            const long row = (at * 4) / per_row;
            const int col = (int)(at * 4 - row * per_row);
            const int head = col / used, c = col - head * used;
            T* p = x + (row * heads + head) * dpad + c;
            float v[4], g[4];
            load4<T>(p, v);
            load4<float>(gate + row * gate_stride + col, g);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] *= sigmoid_as<serves_rounded<T>::value>(g[j]);
            store4<T>(p, v);
        }
    } else {
        const long total = rows * per_row;
        for (long at = blockIdx.x * (long)blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x) {
            const long row = at / per_row;
            const int col = (int)(at - row * per_row);
            const int head = col / used, c = col - head * used;
            T* p = x + (row * heads + head) * dpad + c;
            *p = from_f32<T>(to_f32<T>(*p) * sigmoid_f32(gate[row * gate_stride + col]));
        }
    }
}

template <typename T>
static int sigmoid_gate_launch(void* x, const float* gate, long gate_stride, int rows, int heads, int used, int dpad,
                               cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || used <= 0 || dpad < used) return KIRAI_ERR_BAD_SIZE;
    const bool vec = used % 4 == 0 && dpad % 4 == 0 && gate_stride % 4 == 0 && (((uintptr_t)x | (uintptr_t)gate) & 15) == 0;
    const long total = (long)rows * heads * used / (vec ? 4 : 1);
    const int threads = 256;
    const unsigned blocks = (unsigned)min((total + threads - 1) / threads, (long)148 * 16);
    return launch_pdl(vec ? sigmoid_gate_kernel<T, true> : sigmoid_gate_kernel<T, false>, dim3(blocks), dim3(threads), 0, stream, 1u,
                      (T*)x, gate, gate_stride, (long)rows, heads, used, dpad);
}

KIRAI_EXPORT int kirai_sigmoid_gate_f32(void* x, const float* gate, long gate_stride, int rows, int heads, int used, int dpad,
                                        cudaStream_t stream) {
    return sigmoid_gate_launch<float>(x, gate, gate_stride, rows, heads, used, dpad, stream);
}
KIRAI_EXPORT int kirai_sigmoid_gate_bf16(void* x, const float* gate, long gate_stride, int rows, int heads, int used, int dpad,
                                         cudaStream_t stream) {
    return sigmoid_gate_launch<bf16>(x, gate, gate_stride, rows, heads, used, dpad, stream);
}

// out [T, I] = act(gate) * up for gate_up [T, 2 I] (gate half first); act 0: silu, 1: the tanh form of gelu,
// 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))).
__device__ __forceinline__ float gelu_tanh_f32(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// act 2: g' = min(gate, limit), u' = clamp(up, -limit, limit), g' * sigmoid(slope * g') * (u' + 1).
template <typename T>
__global__ void gated_activation_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long rows, int inter, int act,
                                        float limit, float slope) {
    pdl_launch_dependents();
    pdl_wait();
    const long total = rows * inter;
    for (long at = blockIdx.x * (long)blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x) {
        const long row = at / inter;
        const int c = (int)(at - row * inter);
        const float g = to_f32<T>(gate_up[row * 2 * inter + c]);
        const float u = to_f32<T>(gate_up[row * 2 * inter + inter + c]);
        if (act == 2) {
            out[at] = from_f32<T>(clamped_gated_f32(g, u, limit, slope));
            continue;
        }
        const float a = act == 1 ? gelu_tanh_f32(g) : g * sigmoid_f32(g);
        out[at] = from_f32<T>(a * u);
    }
}

// The same for bfloat16 rows whose width is a multiple of 8: eight columns a thread, 16-byte loads and stores.
__global__ void gated_activation_vec_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, long rows, int inter, int act,
                                            float limit, float slope) {
    pdl_launch_dependents();
    pdl_wait();
    const int pieces = inter >> 3;
    const long total = rows * pieces;
    for (long at = blockIdx.x * (long)blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x) {
        const long row = at / pieces;
        const int c = (int)(at - row * pieces);
        const uint4 g4 = reinterpret_cast<const uint4*>(gate_up + row * 2 * inter)[c];
        const uint4 u4 = reinterpret_cast<const uint4*>(gate_up + row * 2 * inter + inter)[c];
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
        const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
        uint4 packed;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(gp[j]), u = __bfloat1622float2(up[j]);
            float a, b;
            if (act == 2) {
                a = clamped_gated_f32(g.x, u.x, limit, slope);
                b = clamped_gated_f32(g.y, u.y, limit, slope);
            } else {
                a = (act == 1 ? gelu_tanh_f32(g.x) : g.x * sigmoid_f32(g.x)) * u.x;
                b = (act == 1 ? gelu_tanh_f32(g.y) : g.y * sigmoid_f32(g.y)) * u.y;
            }
            op[j] = __floats2bfloat162_rn(a, b);
        }
        reinterpret_cast<uint4*>(out + row * inter)[c] = packed;
    }
}

template <typename T>
static int gated_activation_launch(const void* gate_up, void* out, int rows, int inter, int act, float limit, float slope,
                                   cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (inter <= 0 || act < 0 || act > 2 || (act == 2 && !(limit > 0.0f))) return KIRAI_ERR_BAD_SIZE;
    if (sizeof(T) == 2 && inter % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
        const long pieces = (long)rows * (inter / 8);
        const unsigned vec_blocks = (unsigned)min((pieces + 255) / 256, (long)148 * 16);
        return launch_pdl(gated_activation_vec_kernel, dim3(vec_blocks), dim3(256), 0, stream, 1u, (const bf16*)gate_up, (bf16*)out,
                          (long)rows, inter, act, limit, slope);
    }
    const long total = (long)rows * inter;
    const int threads = 256;
    const unsigned blocks = (unsigned)min((total + threads - 1) / threads, (long)148 * 16);
    return launch_pdl(gated_activation_kernel<T>, dim3(blocks), dim3(threads), 0, stream, 1u, (const T*)gate_up, (T*)out, (long)rows,
                      inter, act, limit, slope);
}

KIRAI_EXPORT int kirai_gated_activation_f32(const void* gate_up, void* out, int rows, int inter, int act, float limit, float slope,
                                            cudaStream_t stream) {
    return gated_activation_launch<float>(gate_up, out, rows, inter, act, limit, slope, stream);
}
KIRAI_EXPORT int kirai_gated_activation_bf16(const void* gate_up, void* out, int rows, int inter, int act, float limit, float slope,
                                             cudaStream_t stream) {
    return gated_activation_launch<bf16>(gate_up, out, rows, inter, act, limit, slope, stream);
}

// x [T, width] (in place) += bias [width] (float32).
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, long rows, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const long total = rows * width;
    for (long at = blockIdx.x * (long)blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x)
        x[at] = from_f32<T>(to_f32<T>(x[at]) + bias[at % width]);
}

template <typename T>
static int add_bias_launch(void* x, const float* bias, int rows, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return KIRAI_ERR_BAD_SIZE;
    const long total = (long)rows * width;
    const int threads = 256;
    const unsigned blocks = (unsigned)min((total + threads - 1) / threads, (long)148 * 16);
    return launch_pdl(add_bias_kernel<T>, dim3(blocks), dim3(threads), 0, stream, 1u, (T*)x, bias, (long)rows, width);
}

KIRAI_EXPORT int kirai_add_bias_f32(void* x, const float* bias, int rows, int width, cudaStream_t stream) {
    return add_bias_launch<float>(x, bias, rows, width, stream);
}
KIRAI_EXPORT int kirai_add_bias_bf16(void* x, const float* bias, int rows, int width, cudaStream_t stream) {
    return add_bias_launch<bf16>(x, bias, rows, width, stream);
}
