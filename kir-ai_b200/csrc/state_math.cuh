// Scalar forms that the kernels of recurrent mixers share, all in 32-bit.
#pragma once
#include "common.cuh"

__device__ __forceinline__ float sf_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float sf_silu(float x) { return x * sf_sigmoid(x); }
__device__ __forceinline__ float sf_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sf_log_sigmoid(float x) { return -sf_softplus(-x); }
__device__ __forceinline__ float sf_gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
