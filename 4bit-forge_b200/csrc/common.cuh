// Shared helpers of the forge_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/forge_b200.h"

namespace forge {

void set_error(const char *fmt, ...);
void note_launch();
#define FORGE_NOTE_LAUNCH() ::forge::note_launch()

inline int check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return FORGE_ERR_LAUNCH;
    }
    return FORGE_OK;
}

#define FORGE_REQUIRE(cond, msg)                          \
    do {                                                  \
        if (!(cond)) {                                    \
            ::forge::set_error("%s: %s", __func__, msg);  \
            return FORGE_ERR_INVALID;                     \
        }                                                 \
    } while (0)

__host__ __device__ static inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ static inline int64_t imin64(int64_t a, int64_t b) { return a < b ? a : b; }

__device__ __forceinline__ float ld_as_f32(const void *p, int dtype, int64_t i) {
    if (dtype == FORGE_DTYPE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
    return reinterpret_cast<const float *>(p)[i];
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_down_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_down_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum_down(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace forge
