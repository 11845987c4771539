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
    float *partial;
    int *counters;
    int64_t K, N;
    int Kt, Nt;
    int nkb, kb_per_split, splits;
    int act, out_dtype, a_row_major, out_row_major;
    int *status;  // device status word raised by bounded waits that run out
};

// Global element offset of the 8-element activation chunk (row r, columns k..k+7).
__device__ __forceinline__ int64_t act_chunk_offset(const DecodeArgs &p, int64_t r, int64_t k) {
    if (p.a_row_major) return r * p.K + k;
    return ((r >> 5) * p.Kt + (k >> 5)) * 1024 + 256 * (2 * (int)((r & 31) >> 4) + (int)((k & 31) >> 4)) + 16 * (int)(r & 15) +
           (int)(k & 15);
}

template <int NB>
__device__ __forceinline__ void finish_and_store(const DecodeArgs &p, const float (&v)[16], int64_t row0, int col0, int64_t n) {
    const float bias = p.bias ? bias_at(p.bias, n) : 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int64_t r = row0 + col0 + j;
        const float y = apply_activation(v[j] + bias, p.act);
        const int64_t off = p.out_row_major ? r * p.N + n : tiled_offset(r, n, p.Nt);
        if (p.out_dtype == TTB_FLOAT32)
            reinterpret_cast<float *>(p.out)[off] = y;
        else
            reinterpret_cast<uint16_t *>(p.out)[off] = f32_to_bf16_bits(y);
    }
}

}  // namespace ttb
