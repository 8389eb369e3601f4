// Row-wise kernels of layer forms beside the pre-norm / rotary ones of elementwise.cu:
//
//   * embedding rows times a constant, plus a sinusoidal position vector (column 2i the sine and column 2i + 1
//     the cosine of position * frequency[i], angles in 32-bit);
//   * the norm on a sub-layer's OUTPUT: stream += y / sqrt(mean(y^2) + eps) * w, with the runtime-dtype copy of the
//     new stream that the next sub-layer reads written in the same pass; the same followed by the norm that reads the
//     stream next (norm_add_norm), and with the stream's copy written into a run of columns of a wider buffer
//     (stream_copy: two streams side by side for one product);
//   * relu(z)^2 in place;
//   * the preparation of attention whose q, k, v projections carry biases and whose queries and keys are normed
//     over the WHOLE projection (all heads of a token at once, one weight per column), with keys and values of
//     their own widths: bias, norm, queries out (heads padded to the cache's head width), keys and values to their
//     pages.
//
// Statistics, biases and norm weights are 32-bit; the products that feed these kernels leave 32-bit rows.
#include "common.cuh"

// ------------------------------------------------- scaled embedding + sinusoid
template <typename T, typename C>
__global__ void embedding_sinusoid_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                          const int* __restrict__ positions, const float* __restrict__ freq,
                                          float* __restrict__ out, C* __restrict__ copy, int hidden, int vocab,
                                          float scale, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    pdl_wait();
    const int token = blockIdx.x;
    const int id = ids[token];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(error_flag, KIRAI_FLAG_BAD_TOKEN);
        return;
    }
    const float pos = freq ? (float)positions[token] : 0.0f;
    const T* row = table + (size_t)id * hidden;
    float* dst = out + (size_t)token * hidden;
    C* dst_copy = copy ? copy + (size_t)token * hidden : nullptr;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = to_f32<T>(row[i]) * scale;
        if (freq) {
            const float angle = pos * freq[i >> 1];
            v += (i & 1) ? cosf(angle) : sinf(angle);
        }
        dst[i] = v;
        if (dst_copy) dst_copy[i] = from_f32<C>(v);
    }
}

template <typename T>
static int embedding_sinusoid_launch(const void* table, const int* ids, const int* positions, const float* freq,
                                     float* out, void* copy, int tokens, int hidden, int vocab, float scale,
                                     int* error_flag, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    return launch_pdl(embedding_sinusoid_kernel<T, bf16>, dim3(tokens), dim3(256), 0, stream, 1u, (const T*)table, ids,
                      positions, freq, out, (bf16*)copy, hidden, vocab, scale, error_flag);
}

// out [T, H] (float32) = table[id] * scale (+ the sinusoid of the token's position when freq [ceil(H/2)] is given);
// copy (bf16, may be null) receives the same rows rounded.
KIRAI_EXPORT int kirai_embedding_sinusoid_f32(const void* table, const int* ids, const int* positions, const float* freq,
                                              float* out, void* copy, int tokens, int hidden, int vocab, float scale,
                                              int* error_flag, cudaStream_t stream) {
    return embedding_sinusoid_launch<float>(table, ids, positions, freq, out, copy, tokens, hidden, vocab, scale, error_flag, stream);
}
KIRAI_EXPORT int kirai_embedding_sinusoid_bf16(const void* table, const int* ids, const int* positions, const float* freq,
                                               float* out, void* copy, int tokens, int hidden, int vocab, float scale,
                                               int* error_flag, cudaStream_t stream) {
    return embedding_sinusoid_launch<bf16>(table, ids, positions, freq, out, copy, tokens, hidden, vocab, scale, error_flag, stream);
}

// ------------------------------------------------------- norm on the output
// One block per row: resid[row] += y[row] * rsqrt(mean(y[row]^2) + eps) * weight; copy[row] = bf16(resid[row]).
__global__ void norm_add_kernel(float* __restrict__ resid, const float* __restrict__ y, const float* __restrict__ weight,
                                bf16* __restrict__ copy, int hidden, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int row = blockIdx.x;
    const float* src = y + (size_t)row * hidden;
    float* dst = resid + (size_t)row * hidden;
    bf16* dst_copy = copy ? copy + (size_t)row * hidden : nullptr;
    float acc = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = src[i];
        acc = fmaf(v, v, acc);
    }
    const float variance = block_sum(acc, scratch) / (float)hidden + eps;
    const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = dst[i] + src[i] * scale * weight[i];
        dst[i] = v;
        if (dst_copy) dst_copy[i] = __float2bfloat16_rn(v);
    }
}

// The same with 16-byte loads, the row of y kept in registers between the statistics and the add (width a multiple
// of 4, at most 4 * VEC * blockDim values).
template <int VEC>
__global__ void norm_add_vec_kernel(float* __restrict__ resid, const float* __restrict__ y, const float* __restrict__ weight,
                                    bf16* __restrict__ copy, int hidden, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int row = blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(y + (size_t)row * hidden);
    float4* dst = reinterpret_cast<float4*>(resid + (size_t)row * hidden);
    const float4* w4 = reinterpret_cast<const float4*>(weight);
    const int quads = hidden >> 2;
    float4 kept[VEC];
    float acc = 0.0f;
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < quads) {
            kept[n] = src[i];
            acc = fmaf(kept[n].x, kept[n].x, acc);
            acc = fmaf(kept[n].y, kept[n].y, acc);
            acc = fmaf(kept[n].z, kept[n].z, acc);
            acc = fmaf(kept[n].w, kept[n].w, acc);
        }
    }
    const float variance = block_sum(acc, scratch) / (float)hidden + eps;
    const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < quads) {
            float4 r = dst[i];
            const float4 w = w4[i];
            r.x += kept[n].x * scale * w.x;
            r.y += kept[n].y * scale * w.y;
            r.z += kept[n].z * scale * w.z;
            r.w += kept[n].w * scale * w.w;
            dst[i] = r;
            if (copy) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo);
                packed.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(copy + (size_t)row * hidden + 4 * (size_t)i) = packed;
            }
        }
    }
}

KIRAI_EXPORT int kirai_norm_add(float* resid, const float* y, const float* weight, void* copy, int rows, int hidden,
                                float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0) return KIRAI_ERR_BAD_SIZE;
    const bool aligned = hidden % 4 == 0 && (((uintptr_t)resid | (uintptr_t)y | (uintptr_t)weight | (uintptr_t)copy) & 15) == 0;
    if (aligned && hidden <= 4 * 4 * 512) {
        const int threads = hidden <= 4 * 4 * 128 ? 128 : (hidden <= 4 * 4 * 256 ? 256 : 512);
        return launch_pdl(norm_add_vec_kernel<4>, dim3(rows), dim3(threads), 0, stream, 1u, resid, y, weight, (bf16*)copy, hidden, eps);
    }
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    return launch_pdl(norm_add_kernel, dim3(rows), dim3(threads), 0, stream, 1u, resid, y, weight, (bf16*)copy, hidden, eps);
}

// -------------------------------------- norm on the output, then the next norm
// One block per produced row.  With a sub-layer's 32-bit output y: the stream takes y / rms(y) * w_add, and the sum
// leaves under the next norm, sum / rms(sum) * w_next, in the runtime dtype: one pass over the row where the two
// kernels made three.  With row_index only those rows are produced and the stream is not written (the rows ahead of
// the logits).  The row is kept in shared memory (32-bit) between the two statistics.
template <typename T>
__global__ void norm_add_norm_kernel(float* __restrict__ resid, const float* __restrict__ y, const float* __restrict__ w_add,
                                     const float* __restrict__ w_next, T* __restrict__ out, const int* __restrict__ row_index,
                                     int hidden, float eps_add, float eps_next) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float row_s[];  // [hidden]
    __shared__ float scratch[32];
    const int row = row_index ? row_index[blockIdx.x] : (int)blockIdx.x;
    const float* src = y + (size_t)row * hidden;
    float* stream = resid + (size_t)row * hidden;
    T* dst = out + (size_t)blockIdx.x * hidden;
    float acc = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = src[i];
        row_s[i] = v;
        acc = fmaf(v, v, acc);
    }
    const float var_add = block_sum(acc, scratch) / (float)hidden + eps_add;
    const float scale_add = var_add == 0.0f ? 0.0f : 1.0f / sqrtf(var_add);
    acc = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = stream[i] + row_s[i] * scale_add * w_add[i];
        row_s[i] = v;
        if (!row_index) stream[i] = v;
        acc = fmaf(v, v, acc);
    }
    const float var_next = block_sum(acc, scratch) / (float)hidden + eps_next;
    const float scale_next = var_next == 0.0f ? 0.0f : 1.0f / sqrtf(var_next);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_f32<T>(row_s[i] * scale_next * w_next[i]);
}

// The same with 16-byte loads, the row kept in registers between the two statistics and the output (width a multiple
// of 4, at most 4 * VEC * blockDim values).
template <typename T, int VEC>
__global__ void norm_add_norm_vec_kernel(float* __restrict__ resid, const float* __restrict__ y, const float* __restrict__ w_add,
                                         const float* __restrict__ w_next, T* __restrict__ out, const int* __restrict__ row_index,
                                         int hidden, float eps_add, float eps_next) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int row = row_index ? row_index[blockIdx.x] : (int)blockIdx.x;
    const float4* src = reinterpret_cast<const float4*>(y + (size_t)row * hidden);
    float4* stream = reinterpret_cast<float4*>(resid + (size_t)row * hidden);
    const float4* wa = reinterpret_cast<const float4*>(w_add);
    const float4* wn = reinterpret_cast<const float4*>(w_next);
    const int quads = hidden >> 2;
    float4 kept[VEC], old[VEC];
    float acc = 0.0f;
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < quads) {
            kept[n] = src[i];
            old[n] = stream[i];
            acc += (kept[n].x * kept[n].x + kept[n].y * kept[n].y) + (kept[n].z * kept[n].z + kept[n].w * kept[n].w);
        }
    }
    const float var_add = block_sum(acc, scratch) / (float)hidden + eps_add;
    const float scale_add = var_add == 0.0f ? 0.0f : 1.0f / sqrtf(var_add);
    acc = 0.0f;
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < quads) {
            const float4 w = wa[i];
            float4 r = old[n];
            r.x += kept[n].x * scale_add * w.x, r.y += kept[n].y * scale_add * w.y;
            r.z += kept[n].z * scale_add * w.z, r.w += kept[n].w * scale_add * w.w;
            kept[n] = r;
            if (!row_index) stream[i] = r;
            acc += (r.x * r.x + r.y * r.y) + (r.z * r.z + r.w * r.w);
        }
    }
    const float var_next = block_sum(acc, scratch) / (float)hidden + eps_next;
    const float scale_next = var_next == 0.0f ? 0.0f : 1.0f / sqrtf(var_next);
    T* dst = out + (size_t)blockIdx.x * hidden;
#pragma unroll
    for (int n = 0; n < VEC; ++n) {
        const int i = threadIdx.x + n * blockDim.x;
        if (i < quads) {
            const float4 w = wn[i];
            const float4 r = kept[n];
            const float a = r.x * scale_next * w.x, b = r.y * scale_next * w.y, c = r.z * scale_next * w.z, d = r.w * scale_next * w.w;
            if (sizeof(T) == 4) {
                reinterpret_cast<float4*>(dst)[i] = make_float4(a, b, c, d);
            } else {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
                uint2 packed;
                packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                reinterpret_cast<uint2*>(dst)[i] = packed;
            }
        }
    }
}

template <typename T>
static int norm_add_norm_launch(float* resid, const float* y, const float* w_add, const float* w_next, void* out,
                                const int* row_index, int rows, int hidden, float eps_add, float eps_next, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || hidden > 12 * 1024) return KIRAI_ERR_BAD_SIZE;
    const bool aligned = hidden % 4 == 0 &&
                         (((uintptr_t)resid | (uintptr_t)y | (uintptr_t)w_add | (uintptr_t)w_next | (uintptr_t)out) & 15) == 0;
    if (aligned && hidden <= 4 * 4 * 512) {
        const int vec_threads = hidden <= 4 * 4 * 128 ? 128 : (hidden <= 4 * 4 * 256 ? 256 : 512);
        return launch_pdl(norm_add_norm_vec_kernel<T, 4>, dim3(rows), dim3(vec_threads), 0, stream, 1u, resid, y, w_add, w_next, (T*)out,
                          row_index, hidden, eps_add, eps_next);
    }
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    return launch_pdl(norm_add_norm_kernel<T>, dim3(rows), dim3(threads), (size_t)hidden * sizeof(float), stream, 1u, resid, y, w_add,
                      w_next, (T*)out, row_index, hidden, eps_add, eps_next);
}

KIRAI_EXPORT int kirai_norm_add_norm_f32(float* resid, const float* y, const float* w_add, const float* w_next, void* out,
                                         const int* row_index, int rows, int hidden, float eps_add, float eps_next,
                                         cudaStream_t stream) {
    return norm_add_norm_launch<float>(resid, y, w_add, w_next, out, row_index, rows, hidden, eps_add, eps_next, stream);
}
KIRAI_EXPORT int kirai_norm_add_norm_bf16(float* resid, const float* y, const float* w_add, const float* w_next, void* out,
                                          const int* row_index, int rows, int hidden, float eps_add, float eps_next,
                                          cudaStream_t stream) {
    return norm_add_norm_launch<bf16>(resid, y, w_add, w_next, out, row_index, rows, hidden, eps_add, eps_next, stream);
}

// ------------------------------------------------- the stream beside other rows
// One block per row: with y, the stream first takes y / rms(y) * weight (as norm_add); then the row leaves in the
// runtime dtype at out[row * out_stride ...], a run of columns of a wider buffer (two streams side by side, read by one
// product).  Without y it is a copy alone; `resid` is then only read.
template <typename T>
__global__ void stream_copy_kernel(float* __restrict__ resid, const float* __restrict__ y, const float* __restrict__ weight,
                                   T* __restrict__ out, long out_stride, int hidden, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int row = blockIdx.x;
    float* stream = resid + (size_t)row * hidden;
    T* dst = out + (size_t)row * out_stride;
    if (!y) {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_f32<T>(stream[i]);
        return;
    }
    const float* src = y + (size_t)row * hidden;
    float acc = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) acc = fmaf(src[i], src[i], acc);
    const float variance = block_sum(acc, scratch) / (float)hidden + eps;
    const float scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = stream[i] + src[i] * scale * weight[i];
        stream[i] = v;
        dst[i] = from_f32<T>(v);
    }
}

template <typename T>
static int stream_copy_launch(float* resid, const float* y, const float* weight, void* out, long out_stride, int rows, int hidden,
                              float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (hidden <= 0 || out_stride < hidden || (y && !weight)) return KIRAI_ERR_BAD_SIZE;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    return launch_pdl(stream_copy_kernel<T>, dim3(rows), dim3(threads), 0, stream, 1u, resid, y, weight, (T*)out, out_stride, hidden, eps);
}

KIRAI_EXPORT int kirai_stream_copy_f32(float* resid, const float* y, const float* weight, void* out, long out_stride, int rows,
                                       int hidden, float eps, cudaStream_t stream) {
    return stream_copy_launch<float>(resid, y, weight, out, out_stride, rows, hidden, eps, stream);
}
KIRAI_EXPORT int kirai_stream_copy_bf16(float* resid, const float* y, const float* weight, void* out, long out_stride, int rows,
                                        int hidden, float eps, cudaStream_t stream) {
    return stream_copy_launch<bf16>(resid, y, weight, out, out_stride, rows, hidden, eps, stream);
}

// ------------------------------------------------------------ relu(z)^2 in place
template <typename T>
__global__ void relu2_kernel(T* __restrict__ x, long count) {
    pdl_launch_dependents();
    pdl_wait();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long)gridDim.x * blockDim.x) {
        const float z = to_f32<T>(x[i]);
        x[i] = from_f32<T>(z > 0.0f ? z * z : 0.0f);
    }
}

KIRAI_EXPORT int kirai_relu2_f32(void* x, long count, cudaStream_t stream) {
    if (count <= 0) return 0;
    const unsigned blocks = (unsigned)min((count + 255) / 256, (long)148 * 16);
    return launch_pdl(relu2_kernel<float>, dim3(blocks), dim3(256), 0, stream, 1u, (float*)x, count);
}
KIRAI_EXPORT int kirai_relu2_bf16(void* x, long count, cudaStream_t stream) {
    if (count <= 0) return 0;
    const unsigned blocks = (unsigned)min((count + 255) / 256, (long)148 * 16);
    return launch_pdl(relu2_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, 1u, (bf16*)x, count);
}

// ------------------------------------------------------------ 32-bit -> bf16
__global__ void round_rows_kernel(const float* __restrict__ src, bf16* __restrict__ dst, long count) {
    pdl_launch_dependents();
    pdl_wait();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) dst[i] = __float2bfloat16_rn(src[i]);
}
KIRAI_EXPORT int kirai_round_rows_bf16(const float* src, void* dst, long count, cudaStream_t stream) {
    if (count <= 0) return 0;
    return launch_pdl(round_rows_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, stream, 1u, src, (bf16*)dst, count);
}

// ------------------------------------- bias + norm over the whole projection + cache write
// One block per token.  qkv [T, nq dk + nkv dk + nkv dv] (float32, as the stacked product left it; nkv = 0 for a layer
// that reads another layer's keys and values).  Queries: + bias, times rsqrt(mean over all nq dk columns + eps) and
// the column's weight, written to q_out [T, nq, dpad] (columns dk.. of a head zero).  Keys the same over their nkv dk
// columns, written to the token's page row (first dk columns of the cache's dpad); values + bias to theirs (first dv
// columns).  The cache is [pages, 2, nkv, page, dpad]; its columns beyond dk and dv are never written and stay zero
// from creation.  A null bias adds nothing, a null norm weight leaves the rows unnormed.
template <typename T>
__device__ __forceinline__ void store4(T* dst, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
template <>
__device__ __forceinline__ void store4<bf16>(bf16* dst, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&lo);
    packed.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
}

template <typename T, bool VEC>
__global__ void qkv_wide_norm_write_kernel(const float* __restrict__ qkv, long qkv_stride, const float* __restrict__ q_bias,
                                           const float* __restrict__ k_bias, const float* __restrict__ v_bias,
                                           const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                                           T* __restrict__ q_out, T* __restrict__ cache, const int* __restrict__ block_table,
                                           const int* __restrict__ request_of_token, const int* __restrict__ positions,
                                           int q_heads, int kv_heads, int dk, int dv, int dpad, int page_size,
                                           int table_width, int num_pages, int* __restrict__ error_flag) {
    pdl_launch_dependents();
    extern __shared__ float row_s[];  // [nq dk + nkv dk]
    __shared__ float scratch[32];
    const int token = blockIdx.x;
    const int q_cols = q_heads * dk, k_cols = kv_heads * dk, v_cols = kv_heads * dv;
    // where this token's keys and values go: known before the product that made qkv has ended
    long page_base = -1;
    if (kv_heads > 0) {
        const int pos = positions[token];
        const int logical = pos / page_size;
        const int page = logical < table_width ? block_table[(long)request_of_token[token] * table_width + logical] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(error_flag, KIRAI_FLAG_NO_PAGE_WRITE);
        } else {
            page_base = (((long)page * 2) * kv_heads * page_size + (pos % page_size)) * (long)dpad;
        }
    }
    pdl_wait();
    const float* src = qkv + (size_t)token * qkv_stride;
    float q_acc = 0.0f, k_acc = 0.0f;
    if (VEC) {
        // four columns at a time (every width and pointer allows 16-byte loads; see the launch)
        for (int i = threadIdx.x * 4; i < q_cols + k_cols; i += blockDim.x * 4) {
            const bool is_q = i < q_cols;
            const float* bias = is_q ? q_bias : k_bias;
            float4 v = *reinterpret_cast<const float4*>(src + i);
            if (bias) {
                const float4 b = *reinterpret_cast<const float4*>(bias + (is_q ? i : i - q_cols));
                v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
            }
            *reinterpret_cast<float4*>(row_s + i) = v;
            const float sq = (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            if (is_q) q_acc += sq;
            else k_acc += sq;
        }
    } else {
        for (int i = threadIdx.x; i < q_cols + k_cols; i += blockDim.x) {
            const bool is_q = i < q_cols;
            const float* bias = is_q ? q_bias : k_bias;
            const float v = src[i] + (bias ? bias[is_q ? i : i - q_cols] : 0.0f);
            row_s[i] = v;
            if (is_q) q_acc = fmaf(v, v, q_acc);
            else k_acc = fmaf(v, v, k_acc);
        }
    }
    const float q_total = block_sum(q_acc, scratch);
    const float k_total = kv_heads > 0 ? block_sum(k_acc, scratch) : 0.0f;
    __syncthreads();
    float q_scale = 1.0f, k_scale = 1.0f;
    if (q_weight) {
        const float variance = q_total / (float)q_cols + eps;
        q_scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
    }
    if (k_weight && kv_heads > 0) {
        const float variance = k_total / (float)k_cols + eps;
        k_scale = variance == 0.0f ? 0.0f : 1.0f / sqrtf(variance);
    }
    T* q_dst = q_out + (size_t)token * q_heads * dpad;
    const long head_rows = (long)page_size * dpad;  // from one kv head's rows of a page to the next head's
    const long value_base = page_base + (long)kv_heads * head_rows;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < q_heads * dpad; i += blockDim.x * 4) {
            const int head = i / dpad, c = i - head * dpad;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (c < dk) {
                const int col = head * dk + c;
                v = *reinterpret_cast<const float4*>(row_s + col);
                const float4 w = q_weight ? *reinterpret_cast<const float4*>(q_weight + col) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
                v.x *= q_scale * w.x, v.y *= q_scale * w.y, v.z *= q_scale * w.z, v.w *= q_scale * w.w;
            }
            store4<T>(q_dst + i, v);
        }
        if (page_base < 0) return;
        for (int i = threadIdx.x * 4; i < k_cols; i += blockDim.x * 4) {
            const int head = i / dk, c = i - head * dk;
            float4 v = *reinterpret_cast<const float4*>(row_s + q_cols + i);
            const float4 w = k_weight ? *reinterpret_cast<const float4*>(k_weight + i) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
            v.x *= k_scale * w.x, v.y *= k_scale * w.y, v.z *= k_scale * w.z, v.w *= k_scale * w.w;
            store4<T>(cache + page_base + head * head_rows + c, v);
        }
        for (int i = threadIdx.x * 4; i < v_cols; i += blockDim.x * 4) {
            const int head = i / dv, c = i - head * dv;
            float4 v = *reinterpret_cast<const float4*>(src + q_cols + k_cols + i);
            if (v_bias) {
                const float4 b = *reinterpret_cast<const float4*>(v_bias + i);
                v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
            }
            store4<T>(cache + value_base + head * head_rows + c, v);
        }
    } else {
    for (int i = threadIdx.x; i < q_heads * dpad; i += blockDim.x) {
        const int head = i / dpad, c = i - head * dpad;
        float v = 0.0f;
        if (c < dk) {
            const int col = head * dk + c;
            v = row_s[col] * q_scale * (q_weight ? q_weight[col] : 1.0f);
        }
        q_dst[i] = from_f32<T>(v);
    }
    if (page_base < 0) return;
    for (int i = threadIdx.x; i < k_cols; i += blockDim.x) {
        const int head = i / dk, c = i - head * dk;
        cache[page_base + head * head_rows + c] = from_f32<T>(row_s[q_cols + i] * k_scale * (k_weight ? k_weight[i] : 1.0f));
    }
    for (int i = threadIdx.x; i < v_cols; i += blockDim.x) {
        const int head = i / dv, c = i - head * dv;
        const float v = src[q_cols + k_cols + i] + (v_bias ? v_bias[i] : 0.0f);
        cache[value_base + head * head_rows + c] = from_f32<T>(v);
    }
    }
}

template <typename T>
static int qkv_wide_norm_write_launch(const float* qkv, long qkv_stride, const float* q_bias, const float* k_bias,
                                      const float* v_bias, const float* q_weight, const float* k_weight, float eps,
                                      void* q_out, void* cache, const int* block_table, const int* request_of_token,
                                      const int* positions, int tokens, int q_heads, int kv_heads, int dk, int dv, int dpad,
                                      int page_size, int table_width, int num_pages, int* error_flag, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (q_heads <= 0 || kv_heads < 0 || dk <= 0 || dv <= 0 || dpad < dk || dpad < dv || page_size <= 0) return KIRAI_ERR_BAD_SIZE;
    if (kv_heads > 0 && !cache) return KIRAI_ERR_BAD_SIZE;
    const size_t smem = (size_t)(q_heads + kv_heads) * dk * sizeof(float);
    if (smem > 200 * 1024) return KIRAI_ERR_BAD_SIZE;
    // four columns at a time where every width, stride and pointer is a multiple of four values
    const bool vec = dk % 4 == 0 && dv % 4 == 0 && dpad % 4 == 0 && qkv_stride % 4 == 0 &&
                     (((uintptr_t)qkv | (uintptr_t)q_bias | (uintptr_t)k_bias | (uintptr_t)v_bias | (uintptr_t)q_weight |
                       (uintptr_t)k_weight | (uintptr_t)q_out | (uintptr_t)cache) & 15) == 0;
    auto kernel = vec ? qkv_wide_norm_write_kernel<T, true> : qkv_wide_norm_write_kernel<T, false>;
    if (smem > 48 * 1024) {
        const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    const int cols = (q_heads + kv_heads) * dk;
    const int threads = cols >= 4096 ? 512 : (cols >= 1024 ? 256 : 128);
    return launch_pdl(kernel, dim3(tokens), dim3(threads), smem, stream, 1u, qkv, qkv_stride, q_bias, k_bias, v_bias, q_weight,
                      k_weight, eps, (T*)q_out, (T*)cache, block_table, request_of_token, positions, q_heads, kv_heads, dk, dv,
                      dpad, page_size, table_width, num_pages, error_flag);
}

KIRAI_EXPORT int kirai_qkv_wide_norm_write_f32(const float* qkv, long qkv_stride, const float* q_bias, const float* k_bias,
                                               const float* v_bias, const float* q_weight, const float* k_weight, float eps,
                                               void* q_out, void* cache, const int* block_table, const int* request_of_token,
                                               const int* positions, int tokens, int q_heads, int kv_heads, int dk, int dv,
                                               int dpad, int page_size, int table_width, int num_pages, int* error_flag,
                                               cudaStream_t stream) {
    return qkv_wide_norm_write_launch<float>(qkv, qkv_stride, q_bias, k_bias, v_bias, q_weight, k_weight, eps, q_out, cache,
                                             block_table, request_of_token, positions, tokens, q_heads, kv_heads, dk, dv, dpad,
                                             page_size, table_width, num_pages, error_flag, stream);
}
KIRAI_EXPORT int kirai_qkv_wide_norm_write_bf16(const float* qkv, long qkv_stride, const float* q_bias, const float* k_bias,
                                                const float* v_bias, const float* q_weight, const float* k_weight, float eps,
                                                void* q_out, void* cache, const int* block_table, const int* request_of_token,
                                                const int* positions, int tokens, int q_heads, int kv_heads, int dk, int dv,
                                                int dpad, int page_size, int table_width, int num_pages, int* error_flag,
                                                cudaStream_t stream) {
    return qkv_wide_norm_write_launch<bf16>(qkv, qkv_stride, q_bias, k_bias, v_bias, q_weight, k_weight, eps, q_out, cache,
                                            block_table, request_of_token, positions, tokens, q_heads, kv_heads, dk, dv, dpad,
                                            page_size, table_width, num_pages, error_flag, stream);
}
