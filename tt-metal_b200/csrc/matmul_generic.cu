// Shape-generic matmul on the CUDA cores: any M, K, N that are multiples of 32, every supported
// weight dtype. One 256-thread block owns a 32x32 output tile and walks K one tile at a time,
// expanding block-float weight tiles to fp32 in shared memory. It is the correctness anchor for the
// tensor-core kernels (same operands, same fp32 accumulation) and serves shapes their tiling does
// not cover; it is not meant to be fast.
#include "epilogue.cuh"

namespace ttb {
namespace {

struct GenericArgs {
    const uint16_t *a;
    const uint8_t *w;
    const uint16_t *bias;
    void *out;
    int64_t M, K, N;  // M already includes the batch when the weight is shared: rows = batch * M
    int w_dtype, out_dtype, act, a_row_major, out_row_major;
    // batched second operand (blockIdx.z = batch entry): distances between consecutive entries, in elements of a / out
    // and in bytes of w; all zero for a shared weight
    int64_t a_bstride, w_bstride, out_bstride;
};

// (row, col) of face-order index k inside a tile.
__device__ __forceinline__ void face_rc(int k, int &r, int &c) {
    const int f = k >> 8;
    r = ((f >> 1) << 4) + ((k >> 4) & 15);
    c = ((f & 1) << 4) + (k & 15);
}

__global__ void __launch_bounds__(256) matmul_generic_kernel(GenericArgs p) {
    __shared__ float As[32][33];
    __shared__ float Ws[32][33];
    const int t = threadIdx.x;
    const int64_t nt = blockIdx.x, mt = blockIdx.y;
    const int64_t Kt = p.K / 32, Nt = p.N / 32;
    const int ty = t >> 4, tx = t & 15;
    const int64_t bz = blockIdx.z;
    const uint16_t *const a_base = p.a + bz * p.a_bstride;
    const uint8_t *const w_base = p.w + bz * p.w_bstride;
    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int64_t kt = 0; kt < Kt; ++kt) {
        // activations: four consecutive face-order elements per thread
        {
            int r, c;
            face_rc(4 * t, r, c);
            uint2 v;
            if (p.a_row_major)
                v = __ldg(reinterpret_cast<const uint2 *>(a_base + (mt * 32 + r) * p.K + kt * 32 + c));
            else
                v = __ldg(reinterpret_cast<const uint2 *>(a_base + (mt * Kt + kt) * 1024 + 4 * t));
            As[r][c + 0] = __uint_as_float(v.x << 16);
            As[r][c + 1] = __uint_as_float(v.x & 0xffff0000u);
            As[r][c + 2] = __uint_as_float(v.y << 16);
            As[r][c + 3] = __uint_as_float(v.y & 0xffff0000u);
        }
        {
            int r, c;
            face_rc(4 * t, r, c);
            const int64_t tile = kt * Nt + nt;
            uint32_t u[4];
            if (p.w_dtype == TTB_BFLOAT16) {
                uint2 v = __ldg(reinterpret_cast<const uint2 *>(w_base + (tile * 1024 + 4 * t) * 2));
                u[0] = v.x << 16; u[1] = v.x & 0xffff0000u; u[2] = v.y << 16; u[3] = v.y & 0xffff0000u;
            } else if (p.w_dtype == TTB_BFLOAT8_B) {
                const uint8_t *tb = w_base + tile * kBfp8TileBytes;
                const uint32_t E = __ldg(tb + (t >> 2));
                const uint32_t cw = __ldg(reinterpret_cast<const uint32_t *>(tb + 64 + 4 * t));
#pragma unroll
                for (int i = 0; i < 4; ++i) u[i] = bfp_from_code<7>((cw >> (8 * i)) & 0xff, E);
            } else {
                const uint8_t *tb = w_base + tile * kBfp4TileBytes;
                const uint32_t E = __ldg(tb + (t >> 2));
                const uint32_t cw = __ldg(reinterpret_cast<const uint16_t *>(tb + 64 + 2 * t));
#pragma unroll
                for (int i = 0; i < 4; ++i) u[i] = bfp_from_code<3>((cw >> (4 * i)) & 0xf, E);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) Ws[r][c + i] = __uint_as_float(u[i]);
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) {
            const float a0 = As[2 * ty][kk], a1 = As[2 * ty + 1][kk];
            const float w0 = Ws[kk][2 * tx], w1 = Ws[kk][2 * tx + 1];
            acc[0][0] = fmaf(a0, w0, acc[0][0]);
            acc[0][1] = fmaf(a0, w1, acc[0][1]);
            acc[1][0] = fmaf(a1, w0, acc[1][0]);
            acc[1][1] = fmaf(a1, w1, acc[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int64_t r = mt * 32 + 2 * ty + i, c = nt * 32 + 2 * tx + j;
            float v = acc[i][j];
            if (p.bias) v += bias_at(p.bias, c);
            v = apply_activation(v, p.act);
            const int64_t off = bz * p.out_bstride + (p.out_row_major ? r * p.N + c : tiled_offset(r, c, Nt));
            if (p.out_dtype == TTB_FLOAT32)
                reinterpret_cast<float *>(p.out)[off] = v;
            else
                reinterpret_cast<uint16_t *>(p.out)[off] = f32_to_bf16_bits(v);
        }
}

}  // namespace

int32_t launch_matmul_generic(const void *a, const void *w, int w_dtype, const void *bias, void *out, int out_dtype,
                              int64_t rows, int64_t K, int64_t N, int act, int flags, cudaStream_t stream) {
    GenericArgs p;
    p.a = (const uint16_t *)a; p.w = (const uint8_t *)w; p.bias = (const uint16_t *)bias; p.out = out;
    p.M = rows; p.K = K; p.N = N;
    p.w_dtype = w_dtype; p.out_dtype = out_dtype; p.act = act;
    p.a_row_major = (flags & TTB_MM_A_ROW_MAJOR) != 0;
    p.out_row_major = (flags & TTB_MM_OUT_ROW_MAJOR) != 0;
    p.a_bstride = p.w_bstride = p.out_bstride = 0;
    if (rows / 32 > 65535) return fail(TTB_E_UNSUPPORTED, "ttb_matmul (generic kernel): more than 65535 row tiles");
    dim3 grid((unsigned)(N / 32), (unsigned)(rows / 32));
    matmul_generic_kernel<<<grid, 256, 0, stream>>>(p);
    TTB_LAUNCH_CHECK("matmul_generic");
    return TTB_OK;
}

// out[b] = a[b] x w[b] for `batch` independent [M, K] x [K, N] products (tiled operands).
int32_t launch_bmm_generic(const void *a, const void *w, int w_dtype, void *out, int out_dtype, int64_t batch, int64_t M, int64_t K,
                           int64_t N, cudaStream_t stream) {
    GenericArgs p;
    p.a = (const uint16_t *)a; p.w = (const uint8_t *)w; p.bias = nullptr; p.out = out;
    p.M = M; p.K = K; p.N = N;
    p.w_dtype = w_dtype; p.out_dtype = out_dtype; p.act = TTB_ACT_NONE;
    p.a_row_major = 0;
    p.out_row_major = 0;
    p.a_bstride = M * K;
    p.out_bstride = M * N;
    p.w_bstride = w_dtype == TTB_BFLOAT16 ? K * N * 2 : K * N / 1024 * bfp_tile_bytes(w_dtype);
    if (M / 32 > 65535 || batch > 65535) return fail(TTB_E_UNSUPPORTED, "ttb_bmm: more than 65535 row tiles or batch entries");
    dim3 grid((unsigned)(N / 32), (unsigned)(M / 32), (unsigned)batch);
    matmul_generic_kernel<<<grid, 256, 0, stream>>>(p);
    TTB_LAUNCH_CHECK("bmm_generic");
    return TTB_OK;
}

}  // namespace ttb
