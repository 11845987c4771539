// Epilogue pieces shared by the matmul kernels: activation, bias lookup in a tiled [32, N] bf16
// tensor, and output addressing for tiled / row-major results.
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace ttb {

__device__ __forceinline__ float apply_activation(float v, int act) {
    switch (act) {
        case TTB_ACT_RELU: return fmaxf(v, 0.0f);
        case TTB_ACT_GELU: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
        case TTB_ACT_SILU: return v / (1.0f + __expf(-v));
        default: return v;
    }
}

// Same with the activation known at compile time. Epilogues branch on the activation once, outside their element
// loops: a runtime switch inside the loop makes the compiler evaluate erf, exp and the division for every element.
template <int ACT>
__device__ __forceinline__ float apply_activation_t(float v) {
    if (ACT == TTB_ACT_RELU) return fmaxf(v, 0.0f);
    if (ACT == TTB_ACT_GELU) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    if (ACT == TTB_ACT_SILU) return v / (1.0f + __expf(-v));
    return v;
}
#define TTB_DISPATCH_ACT(act, CALL)                         \
    switch (act) {                                          \
        case TTB_ACT_RELU: { constexpr int ACT = TTB_ACT_RELU; CALL; break; } \
        case TTB_ACT_GELU: { constexpr int ACT = TTB_ACT_GELU; CALL; break; } \
        case TTB_ACT_SILU: { constexpr int ACT = TTB_ACT_SILU; CALL; break; } \
        default: { constexpr int ACT = TTB_ACT_NONE; CALL; break; }           \
    }

// Element offset of (row r, column c) inside a tiled 2-D slab with Wt tiles per tile row.
__device__ __forceinline__ int64_t tiled_offset(int64_t r, int64_t c, int64_t Wt) {
    const int64_t tile = (r >> 5) * Wt + (c >> 5);
    const int rr = (int)(r & 31), cc = (int)(c & 31);
    return tile * 1024 + 256 * (2 * (rr >> 4) + (cc >> 4)) + 16 * (rr & 15) + (cc & 15);
}

// First row of a tiled [32, N] bf16 bias.
__device__ __forceinline__ float bias_at(const uint16_t *bias, int64_t n) {
    const int64_t off = (n >> 5) * 1024 + 256 * ((n & 31) >> 4) + (n & 15);
    return __uint_as_float(((uint32_t)__ldg(bias + off)) << 16);
}

__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }

}  // namespace ttb
