// Pieces shared by the two decode (small row count) matmul kernels: launch arguments, activation addressing and
// the epilogue's finish-and-store step.
#pragma once
#include "epilogue.cuh"
#include "sm100_ptx.cuh"

namespace ttb {

struct DecodeArgs {
    const uint8_t *w;
    const uint16_t *a;
    const uint16_t *bias;
    void *out;
    float *partial;   // ordered mode: one fp32 partial per split; accumulate mode: unused
    float *accum;     // accumulate mode: one fp32 tile per output tile, zero between launches
    int *counters;
    int64_t K, N;
    int Kt, Nt;
    int nkb, kb_per_split, splits;
    int act, out_dtype, a_row_major, out_row_major;
    int ordered;      // 1: add the split-K partials in split order (bit-reproducible); 0: red.add into `accum`
    int *status;  // device status word raised by bounded waits that run out
};

// Adds four floats to global memory with one vector reduction (no return value, any order).
__device__ __forceinline__ void red_add_f32x4(float *addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Global element offset of the 8-element activation chunk (row r, columns k..k+7).
__device__ __forceinline__ int64_t act_chunk_offset(const DecodeArgs &p, int64_t r, int64_t k) {
    if (p.a_row_major) return r * p.K + k;
    return ((r >> 5) * p.Kt + (k >> 5)) * 1024 + 256 * (2 * (int)((r & 31) >> 4) + (int)((k & 31) >> 4)) + 16 * (int)(r & 15) +
           (int)(k & 15);
}

// Bias, activation and store of 16 consecutive rows (row0 + col0 .. + 15, col0 a multiple of 16) of output column n.
// In the tiled layout those 16 elements sit 16 apart inside one face, in the row-major layout N apart.
// Element offset of the chunk (row r, K-block 0, 8-element chunk kc of the block's 32 columns) and the constant step from
// one K-block to the next: a K-block is one tile column in the tiled layout (1024 elements on), 32 elements in row-major.
__device__ __forceinline__ int64_t act_chunk_base(const DecodeArgs &p, int64_t r, int kc) {
    if (p.a_row_major) return r * p.K + kc * 8;
    return (r >> 5) * p.Kt * 1024 + 256 * (2 * (int)((r & 31) >> 4) + (kc >> 1)) + 16 * (int)(r & 15) + (kc & 1) * 8;
}
__device__ __forceinline__ int act_chunk_step(const DecodeArgs &p) { return p.a_row_major ? 32 : 1024; }

template <int ACT>
__device__ __forceinline__ void finish_and_store_t(const DecodeArgs &p, const float (&v)[16], int64_t row0, int col0, int64_t n) {
    const float bias = p.bias ? bias_at(p.bias, n) : 0.0f;
    const int64_t r0 = row0 + col0;
    const int64_t base = p.out_row_major ? r0 * p.N + n : tiled_offset(r0, n, p.Nt);
    const int64_t stride = p.out_row_major ? p.N : 16;
    if (p.out_dtype == TTB_FLOAT32) {
        float *o = reinterpret_cast<float *>(p.out) + base;
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j * stride] = apply_activation_t<ACT>(v[j] + bias);
    } else {
        uint16_t *o = reinterpret_cast<uint16_t *>(p.out) + base;
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j * stride] = f32_to_bf16_bits(apply_activation_t<ACT>(v[j] + bias));
    }
}

template <int NB>
__device__ __forceinline__ void finish_and_store(const DecodeArgs &p, const float (&v)[16], int64_t row0, int col0, int64_t n) {
    TTB_DISPATCH_ACT(p.act, finish_and_store_t<ACT>(p, v, row0, col0, n));
}

}  // namespace ttb
