// Pad / unpad of row-major tensors of up to four dimensions on the device: the data movement of Tensor::pad / Tensor::unpad
// (tt_eager/tensor/tensor_impl.hpp:508-677). One thread per output element; the innermost dimension is contiguous in both
// tensors, so warps read and write whole runs. Also the elementwise product of two bfloat16 tensors (the unfused form of
// the gated MLP's multiply).
#include <cuda_bf16.h>

#include "common.cuh"

namespace ttb {
namespace {

struct Dims4 {
    int64_t v[4];
};

template <typename T>
__global__ void pad_kernel(const T *__restrict__ src, T *__restrict__ dst, Dims4 in, Dims4 out, Dims4 start, T pad_value) {
    const int64_t total = out.v[0] * out.v[1] * out.v[2] * out.v[3];
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i;
        const int64_t d3 = r % out.v[3]; r /= out.v[3];
        const int64_t d2 = r % out.v[2]; r /= out.v[2];
        const int64_t d1 = r % out.v[1]; r /= out.v[1];
        const int64_t d0 = r;
        const int64_t s0 = d0 - start.v[0], s1 = d1 - start.v[1], s2 = d2 - start.v[2], s3 = d3 - start.v[3];
        const bool inside = s0 >= 0 && s0 < in.v[0] && s1 >= 0 && s1 < in.v[1] && s2 >= 0 && s2 < in.v[2] && s3 >= 0 && s3 < in.v[3];
        dst[i] = inside ? src[((s0 * in.v[1] + s1) * in.v[2] + s2) * in.v[3] + s3] : pad_value;
    }
}

template <typename T>
__global__ void unpad_kernel(const T *__restrict__ src, T *__restrict__ dst, Dims4 in, Dims4 out, Dims4 start) {
    const int64_t total = out.v[0] * out.v[1] * out.v[2] * out.v[3];
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i;
        const int64_t d3 = r % out.v[3]; r /= out.v[3];
        const int64_t d2 = r % out.v[2]; r /= out.v[2];
        const int64_t d1 = r % out.v[1]; r /= out.v[1];
        const int64_t d0 = r;
        dst[i] = src[(((d0 + start.v[0]) * in.v[1] + d1 + start.v[1]) * in.v[2] + d2 + start.v[2]) * in.v[3] + d3 + start.v[3]];
    }
}

__global__ void mul_bf16_kernel(const uint4 *__restrict__ a, const uint4 *__restrict__ b, uint4 *__restrict__ out, int64_t nvec) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 x = __ldg(a + i), y = __ldg(b + i);
        const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
        uint32_t r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // fp32 product of the two bf16 values, rounded to nearest even once
            const float lo = __uint_as_float(xs[j] << 16) * __uint_as_float(ys[j] << 16);
            const float hi = __uint_as_float(xs[j] & 0xffff0000u) * __uint_as_float(ys[j] & 0xffff0000u);
            r[j] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo)) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi)) << 16);
        }
        out[i] = make_uint4(r[0], r[1], r[2], r[3]);
    }
}

int grid_for(int64_t total) {
    const int64_t blocks = (total + 255) / 256;
    return (int)(blocks < 148 * 16 ? (blocks > 0 ? blocks : 1) : 148 * 16);
}

}  // namespace
}  // namespace ttb

using namespace ttb;

extern "C" int32_t ttb_pad(const void *src, void *dst, int32_t elem_size, const int64_t *in_shape, const int64_t *out_shape,
                           const int64_t *start, uint32_t pad_bits, void *stream) {
    if (!src || !dst || !in_shape || !out_shape || !start) return fail(TTB_E_INVALID, "ttb_pad: null pointer");
    if (elem_size != 2 && elem_size != 4) return fail(TTB_E_INVALID, "ttb_pad: element size must be 2 or 4 bytes");
    Dims4 in, out, st;
    for (int i = 0; i < 4; ++i) {
        in.v[i] = in_shape[i]; out.v[i] = out_shape[i]; st.v[i] = start[i];
        if (in.v[i] <= 0 || out.v[i] <= 0 || st.v[i] < 0 || in.v[i] + st.v[i] > out.v[i])
            return fail(TTB_E_INVALID, "ttb_pad: the input (%lld at offset %lld) does not fit the output (%lld) in dimension %d", (long long)in.v[i],
                        (long long)st.v[i], (long long)out.v[i], i);
    }
    const int64_t total = out.v[0] * out.v[1] * out.v[2] * out.v[3];
    if (elem_size == 4)
        pad_kernel<uint32_t><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>((const uint32_t *)src, (uint32_t *)dst, in, out, st, pad_bits);
    else
        pad_kernel<uint16_t><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>((const uint16_t *)src, (uint16_t *)dst, in, out, st, (uint16_t)pad_bits);
    TTB_LAUNCH_CHECK("pad");
    return TTB_OK;
}

extern "C" int32_t ttb_unpad(const void *src, void *dst, int32_t elem_size, const int64_t *in_shape, const int64_t *start,
                             const int64_t *end, void *stream) {
    if (!src || !dst || !in_shape || !start || !end) return fail(TTB_E_INVALID, "ttb_unpad: null pointer");
    if (elem_size != 2 && elem_size != 4) return fail(TTB_E_INVALID, "ttb_unpad: element size must be 2 or 4 bytes");
    Dims4 in, out, st;
    for (int i = 0; i < 4; ++i) {
        in.v[i] = in_shape[i]; st.v[i] = start[i]; out.v[i] = end[i] - start[i] + 1;
        if (in.v[i] <= 0 || st.v[i] < 0 || end[i] < st.v[i] || end[i] >= in.v[i])
            return fail(TTB_E_INVALID, "ttb_unpad: the slice [%lld, %lld] leaves the tensor (%lld) in dimension %d", (long long)st.v[i],
                        (long long)end[i], (long long)in.v[i], i);
    }
    const int64_t total = out.v[0] * out.v[1] * out.v[2] * out.v[3];
    if (elem_size == 4)
        unpad_kernel<uint32_t><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>((const uint32_t *)src, (uint32_t *)dst, in, out, st);
    else
        unpad_kernel<uint16_t><<<grid_for(total), 256, 0, (cudaStream_t)stream>>>((const uint16_t *)src, (uint16_t *)dst, in, out, st);
    TTB_LAUNCH_CHECK("unpad");
    return TTB_OK;
}

extern "C" int32_t ttb_mul_bf16(const void *a, const void *b, void *out, int64_t count, void *stream) {
    if (!a || !b || !out) return fail(TTB_E_INVALID, "ttb_mul_bf16: null pointer");
    if (count <= 0 || count % 8) return fail(TTB_E_INVALID, "ttb_mul_bf16: the element count must be a positive multiple of 8");
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(TTB_E_INVALID, "ttb_mul_bf16: tensors must be 16-byte aligned");
    mul_bf16_kernel<<<grid_for(count / 8), 256, 0, (cudaStream_t)stream>>>((const uint4 *)a, (const uint4 *)b, (uint4 *)out, count / 8);
    TTB_LAUNCH_CHECK("mul_bf16");
    return TTB_OK;
}
