// Shared helpers of the hand-written sm_100a kernels: precision conversion,
// warp and block reductions, the export macro and the launch-status convention.
//
// Every exported entry point returns an int: 0 on success, otherwise the
// cudaError_t of the launch (or a negative code for a refused argument, see
// KIRAI_ERR_*).  Nothing here allocates; callers pass every buffer.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define KIRAI_EXPORT extern "C" __attribute__((visibility("default")))

// Refusals (negative so that they never collide with a cudaError_t).
#define KIRAI_ERR_BAD_SIZE (-2)
#define KIRAI_ERR_BAD_ALIGN (-3)
#define KIRAI_ERR_UNSUPPORTED (-4)

// Values of the device error word (set instead of faulting; read by the host after a step).
#define KIRAI_FLAG_BAD_TOKEN 1
#define KIRAI_FLAG_NO_PAGE_WRITE 2
#define KIRAI_FLAG_NO_PAGE_READ 3
#define KIRAI_FLAG_WAIT_RAN_OUT 4
#define KIRAI_FLAG_NO_MAXIMUM 5

typedef __nv_bfloat16 bf16;

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the total.  The
// order of the additions depends only on the block size, so a row's result
// does not depend on which other rows run beside it.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats of shared memory */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    float total = (lane < warps) ? scratch[lane] : 0.0f;
    total = warp_sum(total);
    return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    float total = (lane < warps) ? scratch[lane] : -INFINITY;
    total = warp_max(total);
    return total;
}

// A gated activation with clamped inputs: g' = min(gate, limit), u' = clamp(up, -limit, limit), and the result is
// g' * sigmoid(slope * g') * (u' + 1).
__device__ __forceinline__ float clamped_gated_f32(float gate, float up, float limit, float slope) {
    const float g = fminf(gate, limit);
    const float u = fminf(fmaxf(up, -limit), limit);
    return g / (1.0f + expf(-slope * g)) * (u + 1.0f);
}

// ---- which keys a query sees, and what becomes of a score -------------------
// `window` > 0: the last `window` keys up to the query's own position; `window` < 0: the keys of the query's own
// chunk of -window positions (chunks counted from position 0 of the sequence); 0: every key up to its own position.
// The first visible key never decreases with the position.
// A window may also keep a sequence's first `keep` keys visible to every later position, at their true positions:
// position i sees j <= i when i - j < window or j < keep.  Such a mask travels in the same integer as
// window + (keep << MASK_KEEP_SHIFT) (window below 2^20, keep below 2^11); mask_keep and mask_window take it apart, and
// kernels walk the key tiles [0, ceil(keep / tile)) and then those from the window's first tile on (the two runs
// joined when they meet), masking key j when first_visible_key(pos, window) > j >= keep.
#define MASK_KEEP_SHIFT 20
__host__ __device__ __forceinline__ int mask_keep(int code) { return code > 0 ? code >> MASK_KEEP_SHIFT : 0; }
__host__ __device__ __forceinline__ int mask_window(int code) { return code > 0 ? code & ((1 << MASK_KEEP_SHIFT) - 1) : code; }

// The key tiles a query range walks under such a mask: `kept` tiles from tile 0, then tiles from `first` on.
// Iteration `it` reads tile it < kept ? it : first + it - kept.
struct TileRuns {
    int kept, first;
    __host__ __device__ __forceinline__ int tile(int it) const { return it < kept ? it : first + it - kept; }
};
__host__ __device__ __forceinline__ TileRuns tile_runs(int key_lo, int keep, int tile_keys) {
    TileRuns runs;
    runs.first = key_lo / tile_keys;
    runs.kept = keep > 0 ? (keep + tile_keys - 1) / tile_keys : 0;
    if (runs.kept >= runs.first) {  // the runs meet: one run from tile 0
        runs.kept = 0;
        runs.first = keep > 0 ? 0 : runs.first;
    }
    return runs;
}

__host__ __device__ __forceinline__ int first_visible_key(int pos, int window) {
    if (window > 0) return pos - window + 1 > 0 ? pos - window + 1 : 0;
    if (window < 0) return pos - pos % (-window);
    return 0;
}

// A raw score (q . k) in the base-2 exponent's units: times scale * log2(e), or, with a soft cap c,
// c * tanh(score * scale / c) * log2(e).  tanh(x) = 1 - 2 / (e^(2x) + 1) costs one exponential and one reciprocal (the
// absolute error stays near 1e-7; large |x| needs no clamp: the exponential gives inf or 0 there, and the reciprocal of
// inf is 0), and the factors around it are folded on the host: cap_in = 2 log2(e) scale / c, cap_log2 = c log2(e)
// (0: no cap), cap_out = -2 cap_log2, so that a capped score is a multiply, ex2, an add, rcp and a multiply-add.
struct ScoreForm {
    float scale_log2, cap_in, cap_log2, cap_out;
};

static inline ScoreForm make_score_form(float scale, float softcap) {
    ScoreForm form;
    form.scale_log2 = scale * 1.4426950408889634f;
    form.cap_in = softcap > 0.0f ? 2.0f * 1.4426950408889634f * scale / softcap : 0.0f;
    form.cap_log2 = softcap > 0.0f ? softcap * 1.4426950408889634f : 0.0f;
    form.cap_out = -2.0f * form.cap_log2;
    return form;
}

__device__ __forceinline__ float capped_exponent(float raw, const ScoreForm& form) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(raw * form.cap_in));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
    return fmaf(form.cap_out, r, form.cap_log2);
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch -----------------------------------------
// Kernels of the forward pass are launched so that a kernel may begin (set up, prefetch what
// does not depend on its predecessor) while the kernel before it in the stream drains.  A kernel
// calls pdl_launch_dependents() as soon as its successor may start and pdl_wait() before it
// touches anything its predecessor wrote; without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <cstdlib>
static inline bool pdl_enabled() {
    static const bool enabled = [] {
        const char* value = std::getenv("KIRAI_PDL");
        return !(value && value[0] == '0');
    }();
    return enabled;
}

// Launches `kernel` with programmatic stream serialization (and, if cluster_z > 1, as clusters of
// (1, 1, cluster_z) CTAs).  Returns the launch status.
template <typename... Params, typename... Args>
static inline int launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             unsigned cluster_z, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attrs[2];
    unsigned count = 0;
    if (pdl_enabled()) {
        attrs[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    if (cluster_z > 1) {
        attrs[count].id = cudaLaunchAttributeClusterDimension;
        attrs[count].val.clusterDim.x = 1;
        attrs[count].val.clusterDim.y = 1;
        attrs[count].val.clusterDim.z = cluster_z;
        ++count;
    }
    config.attrs = attrs;
    config.numAttrs = count;
    const cudaError_t err = cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
    if (err != cudaSuccess) return (int)err;
    return (int)cudaGetLastError();
}

// The same with thread-block clusters of any shape.
template <typename... Params, typename... Args>
static inline int launch_pdl_clusters(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      dim3 cluster, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attrs[2];
    unsigned count = 0;
    if (pdl_enabled()) {
        attrs[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[count].val.programmaticStreamSerializationAllowed = 1;
        ++count;
    }
    attrs[count].id = cudaLaunchAttributeClusterDimension;
    attrs[count].val.clusterDim.x = cluster.x;
    attrs[count].val.clusterDim.y = cluster.y;
    attrs[count].val.clusterDim.z = cluster.z;
    ++count;
    config.attrs = attrs;
    config.numAttrs = count;
    const cudaError_t err = cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
    if (err != cudaSuccess) return (int)err;
    return (int)cudaGetLastError();
}
