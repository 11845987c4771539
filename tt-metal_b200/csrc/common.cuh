// Shared helpers for the libttb translation units: error reporting behind the C ABI and the
// block-float code <-> fp32-bit conversions used by the conversion and matmul kernels.
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "ttb.h"

namespace ttb {

// Records a message for ttb_last_error() on the calling thread and returns `code`.
int32_t fail(int32_t code, const char *fmt, ...);

#define TTB_CUDA_TRY(expr)                                                                   \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess)                                                              \
            return ::ttb::fail(TTB_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                               __FILE__, __LINE__);                                          \
    } while (0)

// After a kernel launch: surfaces launch-configuration errors without synchronising.
#define TTB_LAUNCH_CHECK(name)                                                               \
    do {                                                                                     \
        cudaError_t e__ = cudaGetLastError();                                                \
        if (e__ != cudaSuccess)                                                              \
            return ::ttb::fail(TTB_E_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

constexpr int kTile = 32;
constexpr int kTileElems = 1024;
constexpr int kBfp8TileBytes = 1088;
constexpr int kBfp4TileBytes = 576;

__host__ __device__ constexpr int bfp_tile_bytes(int fmt) { return fmt == TTB_BFLOAT8_B ? kBfp8TileBytes : kBfp4TileBytes; }
inline int64_t round_up32(int64_t v) { return (v + 31) / 32 * 32; }

// fp32 bits -> sign + MB-bit mantissa code under shared exponent E (E >= exponent field of u).
// Integer-only: hidden one OR-ed in unconditionally, truncating alignment shift, add-half then
// shift, mantissa saturation, sign dropped on a zero mantissa.
template <int MB>
__device__ __forceinline__ uint32_t bfp_to_code(uint32_t u, uint32_t E) {
    if ((u & 0x7fffffffu) == 0) return 0;
    uint32_t man = (u & 0x007fffffu) | 0x00800000u;
    uint32_t d = E - ((u >> 23) & 0xffu);
    man = d >= 24 ? 0u : (man >> d);
    constexpr int S = 24 - MB;
    man = (man + (1u << (S - 1))) >> S;
    man = min(man, (1u << MB) - 1u);
    uint32_t sign = man ? (u >> 31) : 0u;
    return (sign << MB) | man;
}

// code -> fp32 bits: normalise the mantissa, drop the exponent by the shift count in wrapping
// 32-bit arithmetic (no clamp), zero mantissa gives a signed zero.
template <int MB>
__device__ __forceinline__ uint32_t bfp_from_code(uint32_t code, uint32_t E) {
    uint32_t sign = (code >> MB) & 1u;
    uint32_t man = code & ((1u << MB) - 1u);
    if (man == 0) return sign << 31;
    uint32_t cnt = (uint32_t)(__clz((int)man) - (32 - MB));
    man = (man << (cnt + 1)) & ((1u << MB) - 1u);
    uint32_t exp = E - cnt;
    return (sign << 31) | (exp << 23) | (man << (23 - MB));
}

__device__ __forceinline__ uint32_t exp_field(uint32_t u) { return (u >> 23) & 0xffu; }

}  // namespace ttb
