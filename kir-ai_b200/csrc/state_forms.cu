// Kernels of mixers whose state is a matrix built from outer products, and the row-wise forms around them:
//
//   * Dynamic Tanh in the place of a norm, with the residual add fused in: the stream gets factor * (d1 + d2) added
//     and the row leaves as tanh(alpha * x) * w + b; no statistics of the row are taken;
//   * the mean of two sub-layers' outputs, each divided by its root mean square over the row and multiplied by a
//     weight of its own (two mixers that read the same rows side by side);
//   * a causal convolution over a few taps per channel with silu, whose last taps - 1 input rows are state of the
//     request, and the kernel that moves that state on;
//   * the state-space recurrence S <- exp(-exp(A) dt) S + dt B x^T, y = S^T C + D x, per head, as a walk over a
//     request's tokens of the step;
//   * the matrix memory with exponential gates: S <- keep S + take k v^T and a normaliser n <- keep n + take k under a
//     running maximum m of the gates' logarithms, o = S^T q / (max(|n . q|, exp(-m)) + 1e-6);
//   * a gate on rows followed or preceded by a unit-RMS norm over equal groups of columns;
//   * a sigmoid gate with one number per head, a soft cap on rows of logits, and the gated activation of stacked
//     experts times each token's routing weight.
//
// States, gates, decays, step sizes and norms are 32-bit.  A walk keeps a head's state in registers: thread (p, s)
// of a block holds rows s, s + SPLIT, ... of column p, and the SPLIT threads of a column sit side by side in a warp,
// so the sums over the state's rows are shuffles and a token costs no block-wide barrier.
#include "common.cuh"
#include "state_math.cuh"

// ------------------------------------------------------------------ add + Dynamic Tanh
// One block per produced row.  Without row_index: resid[row] += factor * (d1[row] + d2[row]) (either may be null) and
// out[row] = tanh(alpha * resid[row]) * w + b.  With row_index only those rows are produced and the stream stays.
template <typename O>
__global__ void add_dyt_kernel(float* __restrict__ resid, const float* __restrict__ d1, const float* __restrict__ d2, float factor,
                               const float* __restrict__ alpha, const float* __restrict__ w, const float* __restrict__ b,
                               O* __restrict__ out, const int* __restrict__ row_index, int width) {
    pdl_launch_dependents();
    pdl_wait();
    const long row = blockIdx.x;
    const long src = row_index ? row_index[row] : row;
    const float a = alpha[0];
    float* x = resid + src * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = x[c];
        if (d1 || d2) {
            const float add = (d1 ? d1[src * width + c] : 0.0f) + (d2 ? d2[src * width + c] : 0.0f);
            v = fmaf(factor, add, v);
            if (!row_index) x[c] = v;
        }
        out[row * width + c] = from_f32<O>(fmaf(tanhf(a * v), w[c], b[c]));
    }
}

template <typename O>
static int add_dyt_launch(float* resid, const float* d1, const float* d2, float factor, const float* alpha, const float* w,
                          const float* b, void* out, const int* row_index, int rows, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || !alpha || !w || !b) return KIRAI_ERR_BAD_SIZE;
    const int threads = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
    return launch_pdl(add_dyt_kernel<O>, dim3(rows), dim3(threads), 0, stream, 1u, resid, d1, d2, factor, alpha, w, b, (O*)out,
                      row_index, width);
}

KIRAI_EXPORT int kirai_add_dyt_f32(float* resid, const float* d1, const float* d2, float factor, const float* alpha,
                                   const float* w, const float* b, void* out, const int* row_index, int rows, int width,
                                   cudaStream_t stream) {
    return add_dyt_launch<float>(resid, d1, d2, factor, alpha, w, b, out, row_index, rows, width, stream);
}
KIRAI_EXPORT int kirai_add_dyt_bf16(float* resid, const float* d1, const float* d2, float factor, const float* alpha,
                                    const float* w, const float* b, void* out, const int* row_index, int rows, int width,
                                    cudaStream_t stream) {
    return add_dyt_launch<bf16>(resid, d1, d2, factor, alpha, w, b, out, row_index, rows, width, stream);
}

// resid += factor * (d1 + d2), nothing else (for a norm that does not take the sum itself).
__global__ void add_scaled_kernel(float* __restrict__ resid, const float* __restrict__ d1, const float* __restrict__ d2,
                                  float factor, long total) {
    pdl_launch_dependents();
    pdl_wait();
    for (long at = blockIdx.x * (long)blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x)
        resid[at] = fmaf(factor, d1[at] + (d2 ? d2[at] : 0.0f), resid[at]);
}

KIRAI_EXPORT int kirai_add_scaled(float* resid, const float* d1, const float* d2, float factor, long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (!d1) return KIRAI_ERR_BAD_SIZE;
    const unsigned blocks = (unsigned)min((total + 255) / 256, (long)148 * 16);
    return launch_pdl(add_scaled_kernel, dim3(blocks), dim3(256), 0, stream, 1u, resid, d1, d2, factor, total);
}

// ------------------------------------------------ mean of two unit-RMS rows, each with a weight
// out[row] = (a[row] / rms(a[row]) * wa + b[row] / rms(b[row]) * wb) / 2, rms with eps inside the root.
__global__ void rms_pair_mean_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ wa,
                                     const float* __restrict__ wb, float eps, float* __restrict__ out, int width) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const long row = blockIdx.x;
    const float* pa = a + row * width;
    const float* pb = b + row * width;
    float sa = 0.0f, sb = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        sa = fmaf(pa[c], pa[c], sa);
        sb = fmaf(pb[c], pb[c], sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ra = rsqrtf(sa / (float)width + eps), rb = rsqrtf(sb / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        out[row * width + c] = 0.5f * (pa[c] * ra * wa[c] + pb[c] * rb * wb[c]);
}

KIRAI_EXPORT int kirai_rms_pair_mean(const float* a, const float* b, const float* wa, const float* wb, float eps, float* out,
                                     int rows, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (width <= 0) return KIRAI_ERR_BAD_SIZE;
    const int threads = width >= 1024 ? 256 : 128;
    return launch_pdl(rms_pair_mean_kernel, dim3(rows), dim3(threads), 0, stream, 1u, a, b, wa, wb, eps, out, width);
}

// ------------------------------------------------------- gate and unit-RMS norm over groups
// A warp per (row, group), or a block where a group is wide.  y [T, width] (float32, row stride y_stride), gate
// (float32, row stride g_stride), weight [width].  mode 0: v = y * silu(gate), out = v / rms_group(v) * weight (the gate
// comes before the norm); mode 1: out = y / rms_group(y) * weight * sigmoid(gate) (the gate comes after it).
template <typename O, int WARPS>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, long y_stride, const float* __restrict__ gate, long g_stride,
                                        const float* __restrict__ weight, float eps, O* __restrict__ out, long rows, int groups,
                                        int group_width, int mode) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    // WARPS == 1: eight units a block, a warp each; else one unit a block
    const int lane = WARPS == 1 ? (threadIdx.x & 31) : threadIdx.x;
    const int step = WARPS * 32;
    const long unit = WARPS == 1 ? blockIdx.x * (long)(blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
    if (unit >= rows * groups) return;
    const long row = unit / groups;
    const int group = (int)(unit - row * groups);
    const int c0 = group * group_width;
    const float* py = y + row * y_stride + c0;
    const float* pg = gate + row * g_stride + c0;
    float sum = 0.0f;
    for (int c = lane; c < group_width; c += step) {
        const float v = mode == 0 ? py[c] * sf_silu(pg[c]) : py[c];
        sum = fmaf(v, v, sum);
    }
    sum = WARPS == 1 ? warp_sum(sum) : block_sum(sum, scratch);
    const float r = rsqrtf(sum / (float)group_width + eps);
    O* po = out + row * (long)groups * group_width + c0;
    for (int c = lane; c < group_width; c += step) {
        const float v = mode == 0 ? py[c] * sf_silu(pg[c]) : py[c] * sf_sigmoid(pg[c]);
        po[c] = from_f32<O>(v * r * weight[c0 + c]);
    }
}

template <typename O>
static int gated_group_norm_launch(const float* y, long y_stride, const float* gate, long g_stride, const float* weight, float eps,
                                   void* out, int rows, int groups, int group_width, int mode, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (groups <= 0 || group_width <= 0 || mode < 0 || mode > 1) return KIRAI_ERR_BAD_SIZE;
    const long units = (long)rows * groups;
    if (group_width >= 512)
        return launch_pdl(gated_group_norm_kernel<O, 8>, dim3((unsigned)units), dim3(256), 0, stream, 1u, y, y_stride, gate, g_stride,
                          weight, eps, (O*)out, (long)rows, groups, group_width, mode);
    return launch_pdl(gated_group_norm_kernel<O, 1>, dim3((unsigned)((units + 7) / 8)), dim3(256), 0, stream, 1u, y, y_stride, gate,
                      g_stride, weight, eps, (O*)out, (long)rows, groups, group_width, mode);
}

KIRAI_EXPORT int kirai_gated_group_norm_f32(const float* y, long y_stride, const float* gate, long g_stride, const float* weight,
                                            float eps, void* out, int rows, int groups, int group_width, int mode,
                                            cudaStream_t stream) {
    return gated_group_norm_launch<float>(y, y_stride, gate, g_stride, weight, eps, out, rows, groups, group_width, mode, stream);
}
KIRAI_EXPORT int kirai_gated_group_norm_bf16(const float* y, long y_stride, const float* gate, long g_stride, const float* weight,
                                             float eps, void* out, int rows, int groups, int group_width, int mode,
                                             cudaStream_t stream) {
    return gated_group_norm_launch<bf16>(y, y_stride, gate, g_stride, weight, eps, out, rows, groups, group_width, mode, stream);
}

// -------------------------------------------------------------- causal convolution + silu
// Blocks (token, run of channels).  in [T, channels] (float32, row stride in_stride): what the convolution reads; taps_w
// [channels, taps], whose last column weighs the token itself; the rows before a request's first row of this step are
// the request's `taps - 1` kept rows, state [slots, state_len] from column conv_off, [taps - 1, channels], the newest
// last (zeros at a sequence's start).  out [T, channels] (float32) = silu(bias + sum_j w[c, j] * in[t - (taps - 1) + j, c]).
__global__ void conv_silu_kernel(const float* __restrict__ in, long in_stride, const float* __restrict__ taps_w,
                                 const float* __restrict__ bias, const float* __restrict__ state, long state_len, long conv_off,
                                 const int* __restrict__ request_of_token, const int* __restrict__ query_start,
                                 const int* __restrict__ slots, float* __restrict__ out, int channels, int taps, int num_slots) {
    pdl_launch_dependents();
    const long token = blockIdx.x;
    const int request = request_of_token[token];
    const long first = query_start[request];
    const int slot = slots[request];
    pdl_wait();
    if (slot < 0 || slot >= num_slots) return;
    const int local = (int)(token - first);
    const float* kept = state + slot * state_len + conv_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        float acc = bias ? bias[c] : 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int at = local - (taps - 1) + j;
            const float v = at >= 0 ? in[(first + at) * in_stride + c] : kept[(long)(taps - 1 + at) * channels + c];
            acc = fmaf(taps_w[(long)c * taps + j], v, acc);
        }
        out[token * channels + c] = sf_silu(acc);
    }
}

// A thread per (request, channel): the kept rows become the last taps - 1 input rows of the request after this step.
__global__ void conv_state_kernel(const float* __restrict__ in, long in_stride, float* __restrict__ state, long state_len,
                                  long conv_off, const int* __restrict__ query_start, const int* __restrict__ slots, int requests,
                                  int channels, int taps, int num_slots) {
    pdl_launch_dependents();
    pdl_wait();
    const long at = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (at >= (long)requests * channels) return;
    const int request = (int)(at / channels), c = (int)(at - (long)request * channels);
    const int slot = slots[request];
    if (slot < 0 || slot >= num_slots) return;
    const long first = query_start[request];
    const int count = (int)(query_start[request + 1] - first);
    float* kept = state + slot * state_len + conv_off;
    // ascending: entry k takes input row count - (taps - 1) + k, or the kept row count + k (> k, not yet overwritten)
    for (int k = 0; k < taps - 1; ++k) {
        const int src = count - (taps - 1) + k;
        kept[(long)k * channels + c] = src >= 0 ? in[(first + src) * in_stride + c] : kept[(long)(count + k) * channels + c];
    }
}

KIRAI_EXPORT int kirai_conv_silu(const float* in, long in_stride, const float* taps_w, const float* bias, float* state,
                                 long state_len, long conv_off, const int* request_of_token, const int* query_start,
                                 const int* slots, float* out, int tokens, int requests, int channels, int taps, int num_slots,
                                 cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (channels <= 0 || taps <= 0 || requests <= 0 || conv_off < 0 || conv_off + (long)(taps - 1) * channels > state_len)
        return KIRAI_ERR_BAD_SIZE;
    const int threads = channels >= 1024 ? 256 : 128;
    // few tokens: a token's channels spread over several blocks, so that a step of single tokens fills more of the device
    int spread = 1;
    while (spread < 16 && tokens * spread < 256 && threads * spread * 2 <= channels) spread *= 2;
    int status = launch_pdl(conv_silu_kernel, dim3(tokens, spread), dim3(threads), 0, stream, 1u, in, in_stride, taps_w, bias,
                            (const float*)state, state_len, conv_off, request_of_token, query_start, slots, out, channels, taps,
                            num_slots);
    if (status != 0 || taps == 1) return status;
    const long units = (long)requests * channels;
    return launch_pdl(conv_state_kernel, dim3((unsigned)((units + 255) / 256)), dim3(256), 0, stream, 1u, in, in_stride, state,
                      state_len, conv_off, query_start, slots, requests, channels, taps, num_slots);
}

// ------------------------------------------------------------------ state-space walk
// Block (request, head); thread (p, s): column p of the head's state [N, P], rows s, s + SPLIT, ...
// xbc [T, inner + 2 G N] (float32): x, then B, then C, after convolution and silu; dt_raw (float32, row stride
// dt_stride): the step sizes before softplus; y [T, inner] (float32) = S^T C + D x.
template <int REGS>
__global__ void __launch_bounds__(256) ssm_walk_kernel(const float* __restrict__ xbc, const float* __restrict__ dt_raw, long dt_stride,
                                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                                float* __restrict__ state, long state_len, long ssm_off, const int* __restrict__ query_start,
                                const int* __restrict__ slots, float* __restrict__ y, int heads, int groups, int N, int P,
                                int split, int num_slots) {
    pdl_launch_dependents();
    const int request = blockIdx.x, head = blockIdx.y;
    const int p = blockIdx.z * (blockDim.x / split) + threadIdx.x / split, s = threadIdx.x % split;
    const long first = query_start[request];
    const int count = (int)(query_start[request + 1] - first);
    const int slot = slots[request];
    const int group = head / (heads / groups);
    const int inner = heads * P, channels = inner + 2 * groups * N;
    const float decay_rate = -expf(a_log[head]), skip = d_skip[head], bias = dt_bias[head];
    pdl_wait();
    if (slot < 0 || slot >= num_slots) return;
    const bool live = p < P;
    float* mine = state + slot * state_len + ssm_off + ((long)head * N) * P + p;
    float S[REGS];
#pragma unroll
    for (int i = 0; i < REGS; ++i) {
        const int n = s + i * split;
        S[i] = (live && n < N) ? mine[(long)n * P] : 0.0f;
    }
    for (int t = 0; t < count; ++t) {
        const long row = first + t;
        const float dt = sf_softplus(dt_raw[row * dt_stride + head] + bias);
        const float decay = expf(decay_rate * dt);
        const float* r = xbc + row * channels;
        const float x = live ? r[head * P + p] : 0.0f;
        const float* Bv = r + inner + group * N;
        const float* Cv = Bv + groups * N;
        const float take = dt * x;
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int n = s + i * split;
            if (n < N) {
                S[i] = fmaf(decay, S[i], take * Bv[n]);
                acc = fmaf(S[i], Cv[n], acc);
            }
        }
        for (int offset = split >> 1; offset > 0; offset >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, offset);
        if (live && s == 0) y[row * inner + head * P + p] = fmaf(skip, x, acc);
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int n = s + i * split;
            if (n < N) mine[(long)n * P] = S[i];
        }
    }
}

// How a walk spreads a head's state [rows, cols] over blocks of at most 256 threads: `split` threads a column (a power
// of two, at most 32; 16 rows a thread where that suffices), as many whole columns a block as fit, and `chunks` blocks
// a head.  Returns the registers' template size, 0 when a column is too long.
static int walk_shape(int rows, int cols, int* split, int* threads, int* chunks) {
    int sp = 1;
    while (sp < 32 && sp * 16 < rows) sp *= 2;
    const int per = (rows + sp - 1) / sp;
    int per_block = 256 / sp;
    if (per_block > cols) per_block = cols;
    // (a block's thread count is a multiple of 32 and of `split`, so that every column's threads share a warp)
    *threads = ((per_block * sp + 31) / 32) * 32;
    per_block = *threads / sp;
    *split = sp;
    *chunks = (cols + per_block - 1) / per_block;
    return per <= 4 ? 4 : per <= 16 ? 16 : per <= 64 ? 64 : 0;
}

KIRAI_EXPORT int kirai_ssm_walk(const float* xbc, const float* dt_raw, long dt_stride, const float* dt_bias, const float* a_log,
                                const float* d_skip, float* state, long state_len, long ssm_off, const int* query_start,
                                const int* slots, float* y, int requests, int heads, int groups, int N, int P, int num_slots,
                                cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || P <= 0 || ssm_off < 0 || ssm_off + (long)heads * N * P > state_len)
        return KIRAI_ERR_BAD_SIZE;
    int split, threads, chunks;
    const int regs = walk_shape(N, P, &split, &threads, &chunks);
    if (!regs) return KIRAI_ERR_BAD_SIZE;
#define KIRAI_SSM(R)                                                                                                         \
    return launch_pdl(ssm_walk_kernel<R>, dim3(requests, heads, chunks), dim3(threads), 0, stream, 1u, xbc, dt_raw, dt_stride, \
                      dt_bias, a_log, d_skip, state, state_len, ssm_off, query_start, slots, y, heads, groups, N, P, split,  \
                      num_slots)
    if (regs == 4) KIRAI_SSM(4);
    if (regs == 16) KIRAI_SSM(16);
    KIRAI_SSM(64);
#undef KIRAI_SSM
}

// ------------------------------------------------------------------ matrix-memory walk
// Block (request, head, chunk of columns); thread (p, s): column p of the head's memory S [d, dv], rows s, s + SPLIT,
// ..., and the same rows of the normaliser n [d] (every column walks its own copy, so nothing is exchanged for it).
// The walk only reads the normaliser and the maximum; a second kernel, a thread per (request, head, row), walks them
// once more and stores them, after every block of the walk has read the old ones.
// rows (float32, row stride): q [H d], k [H d], v [H dv], then the input gates' [H] and the forget gates' [H]
// pre-activations.  state [slots, state_len]: S [H, d, dv], then n [H, d], then m [H].  o [T, H dv] (float32).
template <int REGS>
__global__ void __launch_bounds__(256) matrix_memory_walk_kernel(const float* __restrict__ rows, long row_stride, const float* __restrict__ in_bias,
                                          const float* __restrict__ keep_bias, float cap, float q_scale, float* __restrict__ state,
                                          long state_len, const int* __restrict__ query_start, const int* __restrict__ slots,
                                          float* __restrict__ o, int heads, int d, int dv, int split, int num_slots) {
    pdl_launch_dependents();
    const int request = blockIdx.x, head = blockIdx.y;
    const int p = blockIdx.z * (blockDim.x / split) + threadIdx.x / split, s = threadIdx.x % split;
    const long first = query_start[request];
    const int count = (int)(query_start[request + 1] - first);
    const int slot = slots[request];
    const float ib = in_bias ? in_bias[head] : 0.0f, fb = keep_bias ? keep_bias[head] : 0.0f;
    pdl_wait();
    if (slot < 0 || slot >= num_slots) return;
    const bool live = p < dv;
    float* base = state + slot * state_len;
    float* mine = base + ((long)head * d) * dv + p;
    const float* norm = base + (long)heads * d * dv + (long)head * d;
    const float* peak_at = base + (long)heads * d * dv + (long)heads * d + head;
    float S[REGS], nn[REGS];
#pragma unroll
    for (int i = 0; i < REGS; ++i) {
        const int r = s + i * split;
        S[i] = (live && r < d) ? mine[(long)r * dv] : 0.0f;
        nn[i] = r < d ? norm[r] : 0.0f;
    }
    float peak = *peak_at;
    const long k_off = (long)heads * d, v_off = 2L * heads * d, i_off = v_off + (long)heads * dv, f_off = i_off + heads;
    for (int t = 0; t < count; ++t) {
        const float* r = rows + (first + t) * row_stride;
        const float log_in = cap * tanhf((r[i_off + head] + ib) / cap);
        const float log_keep = sf_log_sigmoid(cap * tanhf((r[f_off + head] + fb) / cap));
        const float new_peak = fmaxf(log_keep + peak, log_in);
        const float keep = expf(log_keep + peak - new_peak), take = expf(log_in - new_peak);
        peak = new_peak;
        const float* q = r + (long)head * d;
        const float* k = r + k_off + (long)head * d;
        const float v = live ? r[v_off + (long)head * dv + p] : 0.0f;
        const float take_v = take * v;
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int row = s + i * split;
            if (row < d) {
                const float kd = k[row], qd = q[row] * q_scale;
                S[i] = fmaf(keep, S[i], take_v * kd);
                nn[i] = fmaf(keep, nn[i], take * kd);
                num = fmaf(S[i], qd, num);
                den = fmaf(nn[i], qd, den);
            }
        }
        for (int offset = split >> 1; offset > 0; offset >>= 1) {
            num += __shfl_xor_sync(0xffffffffu, num, offset);
            den += __shfl_xor_sync(0xffffffffu, den, offset);
        }
        if (live && s == 0) o[(first + t) * (long)heads * dv + (long)head * dv + p] = num / (fmaxf(fabsf(den), expf(-peak)) + 1e-6f);
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < REGS; ++i) {
            const int r = s + i * split;
            if (r < d) mine[(long)r * dv] = S[i];
        }
    }
}

// A block per (request, head), a thread per row of the normaliser: the same gates once more, n and m stored.
__global__ void matrix_memory_norm_kernel(const float* __restrict__ rows, long row_stride, const float* __restrict__ in_bias,
                                          const float* __restrict__ keep_bias, float cap, float* __restrict__ state, long state_len,
                                          const int* __restrict__ query_start, const int* __restrict__ slots, int heads, int d, int dv,
                                          int num_slots) {
    pdl_launch_dependents();
    pdl_wait();
    const int request = blockIdx.x, head = blockIdx.y;
    const int slot = slots[request];
    if (slot < 0 || slot >= num_slots) return;
    const long first = query_start[request];
    const int count = (int)(query_start[request + 1] - first);
    float* base = state + slot * state_len;
    float* norm = base + (long)heads * d * dv + (long)head * d;
    float* peak_at = base + (long)heads * d * dv + (long)heads * d + head;
    const float ib = in_bias ? in_bias[head] : 0.0f, fb = keep_bias ? keep_bias[head] : 0.0f;
    const long k_off = (long)heads * d, i_off = 2L * heads * d + (long)heads * dv, f_off = i_off + heads;
    const float old_peak = *peak_at;
    float peak = old_peak;
    for (int row = threadIdx.x; row < d; row += blockDim.x) {
        float nn = norm[row];
        peak = old_peak;
        for (int t = 0; t < count; ++t) {
            const float* r = rows + (first + t) * row_stride;
            const float log_in = cap * tanhf((r[i_off + head] + ib) / cap);
            const float log_keep = sf_log_sigmoid(cap * tanhf((r[f_off + head] + fb) / cap));
            const float new_peak = fmaxf(log_keep + peak, log_in);
            nn = fmaf(expf(log_keep + peak - new_peak), nn, expf(log_in - new_peak) * r[k_off + (long)head * d + row]);
            peak = new_peak;
        }
        norm[row] = nn;
    }
    __syncthreads();  // every thread of the head has read the old maximum
    if (threadIdx.x == 0) *peak_at = peak;
}

KIRAI_EXPORT int kirai_matrix_memory_walk(const float* rows, long row_stride, const float* in_bias, const float* keep_bias, float cap,
                                          float q_scale, float* state, long state_len, const int* query_start, const int* slots,
                                          float* o, int requests, int heads, int d, int dv, int num_slots, cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (heads <= 0 || d <= 0 || dv <= 0 || !(cap > 0.0f) || (long)heads * d * dv + (long)heads * d + heads > state_len)
        return KIRAI_ERR_BAD_SIZE;
    int split, threads, chunks;
    const int regs = walk_shape(d, dv, &split, &threads, &chunks);
    if (!regs) return KIRAI_ERR_BAD_SIZE;
    int status;
#define KIRAI_MM(R)                                                                                                            \
    status = launch_pdl(matrix_memory_walk_kernel<R>, dim3(requests, heads, chunks), dim3(threads), 0, stream, 1u, rows,       \
                        row_stride, in_bias, keep_bias, cap, q_scale, state, state_len, query_start, slots, o, heads, d, dv,   \
                        split, num_slots)
    if (regs == 4) KIRAI_MM(4);
    else if (regs == 16) KIRAI_MM(16);
    else KIRAI_MM(64);
#undef KIRAI_MM
    if (status != 0) return status;
    const int norm_threads = d >= 256 ? 256 : ((d + 31) / 32) * 32;
    return launch_pdl(matrix_memory_norm_kernel, dim3(requests, heads), dim3(norm_threads), 0, stream, 1u, rows, row_stride, in_bias,
                      keep_bias, cap, state, state_len, query_start, slots, heads, d, dv, num_slots);
}

// ------------------------------------------------------------------ small element-wise steps
// x [T, heads * dpad] (in place): the first `used` columns of head h times sigmoid(gate[t, h]) (float32, row stride).
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const float* __restrict__ gate, long gate_stride, long rows, int heads,
                                 int used, int dpad) {
    pdl_launch_dependents();
    pdl_wait();
    const long per_row = (long)heads * used, total = rows * per_row;
    for (long at = blockIdx.x * (long)blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x) {
        const long row = at / per_row;
        const int col = (int)(at - row * per_row);
        const int head = col / used, c = col - head * used;
        T* p = x + (row * heads + head) * dpad + c;
        *p = from_f32<T>(to_f32<T>(*p) * sf_sigmoid(gate[row * gate_stride + head]));
    }
}

template <typename T>
static int head_gate_launch(void* x, const float* gate, long gate_stride, int rows, int heads, int used, int dpad,
                            cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || used <= 0 || dpad < used) return KIRAI_ERR_BAD_SIZE;
    const long total = (long)rows * heads * used;
    const unsigned blocks = (unsigned)min((total + 255) / 256, (long)148 * 16);
    return launch_pdl(head_gate_kernel<T>, dim3(blocks), dim3(256), 0, stream, 1u, (T*)x, gate, gate_stride, (long)rows, heads, used,
                      dpad);
}

KIRAI_EXPORT int kirai_head_gate_f32(void* x, const float* gate, long gate_stride, int rows, int heads, int used, int dpad,
                                     cudaStream_t stream) {
    return head_gate_launch<float>(x, gate, gate_stride, rows, heads, used, dpad, stream);
}
KIRAI_EXPORT int kirai_head_gate_bf16(void* x, const float* gate, long gate_stride, int rows, int heads, int used, int dpad,
                                      cudaStream_t stream) {
    return head_gate_launch<bf16>(x, gate, gate_stride, rows, heads, used, dpad, stream);
}

// logits (float32, in place) <- cap * tanh(logits / cap)
__global__ void softcap_kernel(float* __restrict__ x, float cap, long total) {
    pdl_launch_dependents();
    pdl_wait();
    for (long at = blockIdx.x * (long)blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x)
        x[at] = cap * tanhf(x[at] / cap);
}

KIRAI_EXPORT int kirai_softcap_rows(float* x, float cap, long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (!(cap > 0.0f)) return KIRAI_ERR_BAD_SIZE;
    const unsigned blocks = (unsigned)min((total + 255) / 256, (long)148 * 16);
    return launch_pdl(softcap_kernel, dim3(blocks), dim3(256), 0, stream, 1u, x, cap, total);
}

// Stacked gated experts: gate_up [T, experts * 2 ff], per expert ff gate columns and then ff up columns;
// out [T, experts * ff] = act(gate) * up * gates[t, expert] (gates float32 [T, experts], zero where not chosen).
// act 0: silu, 1: the tanh form of gelu, 2: the clamped form (clamped_gated_f32 with `limit` and `slope`).
// `interleaved`: an expert's columns come as 8 gate columns, their 8 up columns, 8 gate columns, ... (the order in which
// the tensor-core product's gated epilogue wants the matrices' rows; ff a multiple of 8).
template <typename T>
__global__ void gated_expert_gate_kernel(const T* __restrict__ gate_up, const float* __restrict__ gates, T* __restrict__ out,
                                         long rows, int experts, int ff, int act, float limit, float slope, int interleaved) {
    pdl_launch_dependents();
    pdl_wait();
    const long per_row = (long)experts * ff, total = rows * per_row;
    for (long at = blockIdx.x * (long)blockDim.x + threadIdx.x; at < total; at += (long)gridDim.x * blockDim.x) {
        const long row = at / per_row;
        const int col = (int)(at - row * per_row);
        const int e = col / ff, j = col - e * ff;
        const float weight = gates[row * experts + e];
        float value = 0.0f;
        if (weight != 0.0f) {
            const T* src = gate_up + row * 2 * per_row + (long)e * 2 * ff;
            const int at_gate = interleaved ? ((j >> 3) << 4) + (j & 7) : j;
            const float g = to_f32<T>(src[at_gate]), u = to_f32<T>(src[interleaved ? at_gate + 8 : ff + j]);
            value = act == 2 ? clamped_gated_f32(g, u, limit, slope) * weight : (act == 1 ? sf_gelu_tanh(g) : sf_silu(g)) * u * weight;
        }
        out[at] = from_f32<T>(value);
    }
}

template <typename T>
static int gated_expert_gate_launch(const void* gate_up, const float* gates, void* out, int rows, int experts, int ff, int act,
                                    float limit, float slope, int interleaved, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (experts <= 0 || ff <= 0 || act < 0 || act > 2 || (act == 2 && !(limit > 0.0f)) || (interleaved && ff % 8 != 0))
        return KIRAI_ERR_BAD_SIZE;
    const long total = (long)rows * experts * ff;
    const unsigned blocks = (unsigned)min((total + 255) / 256, (long)148 * 16);
    return launch_pdl(gated_expert_gate_kernel<T>, dim3(blocks), dim3(256), 0, stream, 1u, (const T*)gate_up, gates, (T*)out,
                      (long)rows, experts, ff, act, limit, slope, interleaved);
}

KIRAI_EXPORT int kirai_gated_expert_gate_f32(const void* gate_up, const float* gates, void* out, int rows, int experts, int ff,
                                             int act, float limit, float slope, int interleaved, cudaStream_t stream) {
    return gated_expert_gate_launch<float>(gate_up, gates, out, rows, experts, ff, act, limit, slope, interleaved, stream);
}
KIRAI_EXPORT int kirai_gated_expert_gate_bf16(const void* gate_up, const float* gates, void* out, int rows, int experts, int ff,
                                              int act, float limit, float slope, int interleaved, cudaStream_t stream) {
    return gated_expert_gate_launch<bf16>(gate_up, gates, out, rows, experts, ff, act, limit, slope, interleaved, stream);
}
