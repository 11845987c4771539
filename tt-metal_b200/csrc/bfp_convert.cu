// Layout conversion and block-float pack / unpack kernels for sm_100a, plus their C-ABI entry points.
//
// All four conversions are HBM-bound byte shuffles (4 + 1.0625 bytes per element for bfloat8_b).
// Work unit: a "strip" of up to four horizontally adjacent 32x32 tiles. One 256-thread block
// handles one strip; a warp reads or writes 128 consecutive row-major columns (512 B of fp32) per
// row so that the row-major side is fully coalesced, and the packed side is staged in shared memory
// so that whole tiles (1088 / 576 contiguous bytes each, four tiles adjacent) move as 16-byte vectors.
// Four lanes own one face row (16 values = one shared exponent) and agree on the exponent by shuffles.
#include "common.cuh"

namespace ttb {
namespace {

constexpr int kStripTiles = 4;
constexpr int kThreads = 256;

__device__ __forceinline__ int64_t imin(int64_t a, int64_t b) { return a < b ? a : b; }

template <typename T>
struct Src;  // loads four consecutive source values as fp32 bit patterns
template <>
struct Src<float> {
    static __device__ __forceinline__ void load4(const float *p, bool vec, int valid, uint32_t (&u)[4]) {
        if (vec) {
            uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
            u[0] = v.x; u[1] = v.y; u[2] = v.z; u[3] = v.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) u[i] = i < valid ? __float_as_uint(__ldg(p + i)) : 0u;
        }
    }
};
template <>
struct Src<uint16_t> {  // bf16: exact widening to fp32 bits
    static __device__ __forceinline__ void load4(const uint16_t *p, bool vec, int valid, uint32_t (&u)[4]) {
        if (vec) {
            uint2 v = __ldg(reinterpret_cast<const uint2 *>(p));
            u[0] = v.x << 16; u[1] = v.x & 0xffff0000u; u[2] = v.y << 16; u[3] = v.y & 0xffff0000u;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) u[i] = i < valid ? ((uint32_t)__ldg(p + i)) << 16 : 0u;
        }
    }
};

template <typename T>
struct Dst;  // stores four consecutive fp32 bit patterns
template <>
struct Dst<float> {
    static __device__ __forceinline__ void store4(float *p, bool vec, int valid, const uint32_t (&u)[4]) {
        if (vec) {
            *reinterpret_cast<uint4 *>(p) = make_uint4(u[0], u[1], u[2], u[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i < valid) p[i] = __uint_as_float(u[i]);
        }
    }
};
template <>
struct Dst<uint16_t> {  // bf16: the unpacked values have zero low halves, so this is exact
    static __device__ __forceinline__ void store4(uint16_t *p, bool vec, int valid, const uint32_t (&u)[4]) {
        if (vec) {
            *reinterpret_cast<uint2 *>(p) = make_uint2((u[0] >> 16) | (u[1] & 0xffff0000u), (u[2] >> 16) | (u[3] & 0xffff0000u));
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i < valid) p[i] = (uint16_t)(u[i] >> 16);
        }
    }
};

// Shared exponent of the face row owned by a group of four adjacent lanes.
__device__ __forceinline__ uint32_t row_exponent(const uint32_t (&u)[4]) {
    uint32_t e = max(max(exp_field(u[0]), exp_field(u[1])), max(exp_field(u[2]), exp_field(u[3])));
    e = max(e, __shfl_xor_sync(0xffffffffu, e, 1));
    e = max(e, __shfl_xor_sync(0xffffffffu, e, 2));
    return e;
}

// Codes of four values under the face-row exponent; with TWO the pack -> unpack -> pack sequence
// of the reference's host from_torch is applied to the group of 16.
template <int MB, bool TWO>
__device__ __forceinline__ void encode4(uint32_t (&u)[4], uint32_t &E, uint32_t (&c)[4]) {
    E = row_exponent(u);
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = bfp_to_code<MB>(u[i], E);
    if (TWO) {
#pragma unroll
        for (int i = 0; i < 4; ++i) u[i] = bfp_from_code<MB>(c[i], E);
        E = row_exponent(u);
#pragma unroll
        for (int i = 0; i < 4; ++i) c[i] = bfp_to_code<MB>(u[i], E);
    }
}

template <int MB, bool TWO>
__device__ __forceinline__ void decode4(const uint32_t (&c)[4], uint32_t E, uint32_t (&u)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) u[i] = bfp_from_code<MB>(c[i], E);
    if (TWO) {
        uint32_t c2[4], E2;
        encode4<MB, false>(u, E2, c2);
#pragma unroll
        for (int i = 0; i < 4; ++i) u[i] = bfp_from_code<MB>(c2[i], E2);
    }
}

struct StripGeom {
    int64_t H, W;        // logical rows / columns of one outer slice
    int64_t Ht, Wt;      // tiles per slice vertically / horizontally (padded)
    int64_t strips_x;    // strips per tile row
};

// ---------------------------------------------------------------------------------------------
// Row-major [outer, H, W] (fp32 or bf16) -> packed tiles, zero padding to 32 fused.
template <int MB, typename S, bool TWO>
__global__ void __launch_bounds__(kThreads) pack_rowmajor_kernel(const S *__restrict__ src, uint8_t *__restrict__ dst,
                                                                  StripGeom g, bool vec_ok) {
    constexpr int TB = MB == 7 ? kBfp8TileBytes : kBfp4TileBytes;
    __shared__ __align__(16) uint8_t stage[kStripTiles * TB];
    const int64_t strip = blockIdx.x;
    const int64_t tile_row = strip / g.strips_x;           // over outer * Ht
    const int64_t sx = strip % g.strips_x;
    const int64_t o = tile_row / g.Ht, hr = tile_row % g.Ht;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_in_strip = lane >> 3;
    const int64_t col = sx * 128 + lane * 4;
    const int ntiles = (int)imin(kStripTiles, g.Wt - sx * kStripTiles);

    uint32_t u[4][4];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int r = it * 8 + warp;
        const int64_t h = hr * 32 + r;
        const int64_t rem = g.W - col;
        const int valid = (h < g.H && rem > 0) ? (int)imin(4, rem) : 0;
        const S *p = src + ((o * g.H + h) * g.W + col);
        if (valid == 0) {
            u[it][0] = u[it][1] = u[it][2] = u[it][3] = 0u;
        } else {
            Src<S>::load4(p, vec_ok && valid == 4, valid, u[it]);
        }
    }
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int r = it * 8 + warp;
        uint32_t E, c[4];
        encode4<MB, TWO>(u[it], E, c);
        const int face = 2 * (r >> 4) + ((lane >> 2) & 1);
        const int fr = r & 15;
        uint8_t *t = stage + tile_in_strip * TB;
        if ((lane & 3) == 0) t[16 * face + fr] = (uint8_t)E;
        const int k = 256 * face + 16 * fr + 4 * (lane & 3);
        if (MB == 7)
            *reinterpret_cast<uint32_t *>(t + 64 + k) = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
        else
            *reinterpret_cast<uint16_t *>(t + 64 + (k >> 1)) = (uint16_t)(c[0] | (c[1] << 4) | (c[2] << 8) | (c[3] << 12));
    }
    __syncthreads();
    uint4 *out = reinterpret_cast<uint4 *>(dst + (tile_row * g.Wt + sx * kStripTiles) * TB);
    const uint4 *in = reinterpret_cast<const uint4 *>(stage);
    for (int i = threadIdx.x; i < ntiles * (TB / 16); i += kThreads) out[i] = in[i];
}

// Tiled source (already in face order) -> packed tiles; one thread per four consecutive values.
template <int MB, typename S, bool TWO>
__global__ void __launch_bounds__(kThreads) pack_tiled_kernel(const S *__restrict__ src, uint8_t *__restrict__ dst,
                                                               int64_t nquads) {
    constexpr int TB = MB == 7 ? kBfp8TileBytes : kBfp4TileBytes;
    int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool live = q < nquads;
    if (!live) q = nquads - 1;  // keep every lane in the shuffles
    uint32_t u[4], E, c[4];
    Src<S>::load4(src + q * 4, true, 4, u);
    encode4<MB, TWO>(u, E, c);
    if (!live) return;
    const int64_t tile = q >> 8;
    const int w = (int)(q & 255);
    uint8_t *t = dst + tile * TB;
    if ((w & 3) == 0) t[w >> 2] = (uint8_t)E;
    if (MB == 7)
        *reinterpret_cast<uint32_t *>(t + 64 + 4 * w) = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
    else
        *reinterpret_cast<uint16_t *>(t + 64 + 2 * w) = (uint16_t)(c[0] | (c[1] << 4) | (c[2] << 8) | (c[3] << 12));
}

// Packed tiles -> row-major [outer, H, W] (fp32 or bf16), padding dropped.
template <int MB, typename D, bool TWO>
__global__ void __launch_bounds__(kThreads) unpack_rowmajor_kernel(const uint8_t *__restrict__ src, D *__restrict__ dst,
                                                                    StripGeom g, bool vec_ok) {
    constexpr int TB = MB == 7 ? kBfp8TileBytes : kBfp4TileBytes;
    __shared__ __align__(16) uint8_t stage[kStripTiles * TB];
    const int64_t strip = blockIdx.x;
    const int64_t tile_row = strip / g.strips_x;
    const int64_t sx = strip % g.strips_x;
    const int64_t o = tile_row / g.Ht, hr = tile_row % g.Ht;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntiles = (int)imin(kStripTiles, g.Wt - sx * kStripTiles);
    {
        const uint4 *in = reinterpret_cast<const uint4 *>(src + (tile_row * g.Wt + sx * kStripTiles) * TB);
        uint4 *st = reinterpret_cast<uint4 *>(stage);
        for (int i = threadIdx.x; i < kStripTiles * (TB / 16); i += kThreads)
            st[i] = i < ntiles * (TB / 16) ? __ldg(in + i) : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    const int tile_in_strip = lane >> 3;
    const int64_t col = sx * 128 + lane * 4;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int r = it * 8 + warp;
        const int face = 2 * (r >> 4) + ((lane >> 2) & 1);
        const int fr = r & 15;
        const uint8_t *t = stage + tile_in_strip * TB;
        const uint32_t E = t[16 * face + fr];
        const int k = 256 * face + 16 * fr + 4 * (lane & 3);
        uint32_t c[4], u[4];
        if (MB == 7) {
            uint32_t w = *reinterpret_cast<const uint32_t *>(t + 64 + k);
            c[0] = w & 0xff; c[1] = (w >> 8) & 0xff; c[2] = (w >> 16) & 0xff; c[3] = w >> 24;
        } else {
            uint32_t w = *reinterpret_cast<const uint16_t *>(t + 64 + (k >> 1));
            c[0] = w & 0xf; c[1] = (w >> 4) & 0xf; c[2] = (w >> 8) & 0xf; c[3] = (w >> 12) & 0xf;
        }
        decode4<MB, TWO>(c, E, u);
        const int64_t h = hr * 32 + r;
        const int64_t rem = g.W - col;
        const int valid = (h < g.H && rem > 0) ? (int)imin(4, rem) : 0;
        if (valid) Dst<D>::store4(dst + ((o * g.H + h) * g.W + col), vec_ok && valid == 4, valid, u);
    }
}

// Packed tiles -> tiled values (face order); one thread per four consecutive values.
template <int MB, typename D, bool TWO>
__global__ void __launch_bounds__(kThreads) unpack_tiled_kernel(const uint8_t *__restrict__ src, D *__restrict__ dst,
                                                                 int64_t nquads) {
    constexpr int TB = MB == 7 ? kBfp8TileBytes : kBfp4TileBytes;
    int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool live = q < nquads;
    if (!live) q = nquads - 1;
    const int64_t tile = q >> 8;
    const int w = (int)(q & 255);
    const uint8_t *t = src + tile * TB;
    const uint32_t E = __ldg(t + (w >> 2));
    uint32_t c[4], u[4];
    if (MB == 7) {
        uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(t + 64 + 4 * w));
        c[0] = v & 0xff; c[1] = (v >> 8) & 0xff; c[2] = (v >> 16) & 0xff; c[3] = v >> 24;
    } else {
        uint32_t v = __ldg(reinterpret_cast<const uint16_t *>(t + 64 + 2 * w));
        c[0] = v & 0xf; c[1] = (v >> 4) & 0xf; c[2] = (v >> 8) & 0xf; c[3] = (v >> 12) & 0xf;
    }
    decode4<MB, TWO>(c, E, u);
    if (live) Dst<D>::store4(dst + q * 4, true, 4, u);
}

// Row-major <-> tiled for plain 2- and 4-byte elements. Four elements per thread; on the tiled side
// four lanes cover one 16-element face row, so stores/loads there are whole 32- or 64-byte runs.
template <typename E4 /* uint2 = 4 x 2 bytes, uint4 = 4 x 4 bytes */, typename E1, bool TILIZE>
__global__ void __launch_bounds__(kThreads) relayout_kernel(const E1 *__restrict__ src, E1 *__restrict__ dst, StripGeom g,
                                                            bool vec_ok) {
    const int64_t strip = blockIdx.x;
    const int64_t tile_row = strip / g.strips_x;
    const int64_t sx = strip % g.strips_x;
    const int64_t o = tile_row / g.Ht, hr = tile_row % g.Ht;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t tile = tile_row * g.Wt + sx * kStripTiles + (lane >> 3);
    const int64_t col = sx * 128 + lane * 4;
    if (sx * kStripTiles + (lane >> 3) >= g.Wt) return;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int r = it * 8 + warp;
        const int64_t h = hr * 32 + r;
        const int face = 2 * (r >> 4) + ((lane >> 2) & 1);
        const int64_t ti = tile * 1024 + 256 * face + 16 * (r & 15) + 4 * (lane & 3);
        const int64_t ri = (o * g.H + h) * g.W + col;
        const int64_t rem = g.W - col;
        const int valid = (h < g.H && rem > 0) ? (int)imin(4, rem) : 0;
        if (TILIZE) {
            E4 v;
            E1 *e = reinterpret_cast<E1 *>(&v);
            if (vec_ok && valid == 4) {
                v = __ldg(reinterpret_cast<const E4 *>(src + ri));
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) e[i] = i < valid ? __ldg(src + ri + i) : (E1)0;
            }
            *reinterpret_cast<E4 *>(dst + ti) = v;
        } else if (valid) {
            E4 v = __ldg(reinterpret_cast<const E4 *>(src + ti));
            if (vec_ok && valid == 4) {
                *reinterpret_cast<E4 *>(dst + ri) = v;
            } else {
                const E1 *e = reinterpret_cast<const E1 *>(&v);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (i < valid) dst[ri + i] = e[i];
            }
        }
    }
}

int32_t make_geom(const char *who, int64_t outer, int64_t H, int64_t W, StripGeom &g, int64_t &nstrips) {
    if (outer <= 0 || H <= 0 || W <= 0) return fail(TTB_E_INVALID, "%s: outer, H and W must be positive", who);
    g.H = H; g.W = W;
    g.Ht = (H + 31) / 32; g.Wt = (W + 31) / 32;
    g.strips_x = (g.Wt + kStripTiles - 1) / kStripTiles;
    nstrips = outer * g.Ht * g.strips_x;
    if (nstrips > 0x7fffffffLL) return fail(TTB_E_INVALID, "%s: tensor too large for one launch", who);
    return TTB_OK;
}

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

}  // namespace
}  // namespace ttb

using namespace ttb;

extern "C" {

int32_t ttb_tilize(const void *src, void *dst, int32_t elem, int64_t outer, int64_t H, int64_t W, void *stream) {
    if (!src || !dst) return fail(TTB_E_INVALID, "ttb_tilize: null pointer");
    if (elem != 2 && elem != 4) return fail(TTB_E_INVALID, "ttb_tilize: element size must be 2 or 4 bytes, got %d", elem);
    StripGeom g; int64_t n;
    if (int32_t rc = make_geom("ttb_tilize", outer, H, W, g, n)) return rc;
    if (!aligned(dst, 4 * elem)) return fail(TTB_E_INVALID, "ttb_tilize: destination must be %d-byte aligned", 4 * elem);
    const bool vec = (W % 4 == 0) && aligned(src, 4 * elem);
    auto s = (cudaStream_t)stream;
    if (elem == 2)
        relayout_kernel<uint2, uint16_t, true><<<(unsigned)n, kThreads, 0, s>>>((const uint16_t *)src, (uint16_t *)dst, g, vec);
    else
        relayout_kernel<uint4, uint32_t, true><<<(unsigned)n, kThreads, 0, s>>>((const uint32_t *)src, (uint32_t *)dst, g, vec);
    TTB_LAUNCH_CHECK("tilize");
    return TTB_OK;
}

int32_t ttb_untilize(const void *src, void *dst, int32_t elem, int64_t outer, int64_t H, int64_t W, void *stream) {
    if (!src || !dst) return fail(TTB_E_INVALID, "ttb_untilize: null pointer");
    if (elem != 2 && elem != 4) return fail(TTB_E_INVALID, "ttb_untilize: element size must be 2 or 4 bytes, got %d", elem);
    StripGeom g; int64_t n;
    if (int32_t rc = make_geom("ttb_untilize", outer, H, W, g, n)) return rc;
    if (!aligned(src, 4 * elem)) return fail(TTB_E_INVALID, "ttb_untilize: source must be %d-byte aligned", 4 * elem);
    const bool vec = (W % 4 == 0) && aligned(dst, 4 * elem);
    auto s = (cudaStream_t)stream;
    if (elem == 2)
        relayout_kernel<uint2, uint16_t, false><<<(unsigned)n, kThreads, 0, s>>>((const uint16_t *)src, (uint16_t *)dst, g, vec);
    else
        relayout_kernel<uint4, uint32_t, false><<<(unsigned)n, kThreads, 0, s>>>((const uint32_t *)src, (uint32_t *)dst, g, vec);
    TTB_LAUNCH_CHECK("untilize");
    return TTB_OK;
}

int32_t ttb_pack_bfp(const void *src, int32_t src_dtype, void *dst, int32_t fmt, int64_t outer, int64_t H, int64_t W,
                     int32_t src_row_major, int32_t two_pass, void *stream) {
    if (!src || !dst) return fail(TTB_E_INVALID, "ttb_pack_bfp: null pointer");
    if (fmt != TTB_BFLOAT8_B && fmt != TTB_BFLOAT4_B) return fail(TTB_E_INVALID, "ttb_pack_bfp: fmt must be bfloat8_b or bfloat4_b");
    if (src_dtype != TTB_FLOAT32 && src_dtype != TTB_BFLOAT16)
        return fail(TTB_E_INVALID, "ttb_pack_bfp: source dtype must be float32 or bfloat16");
    if (!aligned(dst, 16)) return fail(TTB_E_INVALID, "ttb_pack_bfp: destination must be 16-byte aligned");
    const int esz = src_dtype == TTB_FLOAT32 ? 4 : 2;
    auto s = (cudaStream_t)stream;
    if (src_row_major) {
        StripGeom g; int64_t n;
        if (int32_t rc = make_geom("ttb_pack_bfp", outer, H, W, g, n)) return rc;
        const bool vec = (W % 4 == 0) && aligned(src, 4 * esz);
#define TTB_PACK_RM(MB, S, TWO) \
    pack_rowmajor_kernel<MB, S, TWO><<<(unsigned)n, kThreads, 0, s>>>((const S *)src, (uint8_t *)dst, g, vec)
        if (fmt == TTB_BFLOAT8_B) {
            if (esz == 4) { if (two_pass) TTB_PACK_RM(7, float, true); else TTB_PACK_RM(7, float, false); }
            else          { if (two_pass) TTB_PACK_RM(7, uint16_t, true); else TTB_PACK_RM(7, uint16_t, false); }
        } else {
            if (esz == 4) { if (two_pass) TTB_PACK_RM(3, float, true); else TTB_PACK_RM(3, float, false); }
            else          { if (two_pass) TTB_PACK_RM(3, uint16_t, true); else TTB_PACK_RM(3, uint16_t, false); }
        }
#undef TTB_PACK_RM
    } else {
        if (outer <= 0 || H <= 0 || W <= 0 || H % 32 || W % 32)
            return fail(TTB_E_INVALID, "ttb_pack_bfp: a tiled source needs positive H, W that are multiples of 32");
        if (!aligned(src, 4 * esz)) return fail(TTB_E_INVALID, "ttb_pack_bfp: tiled source must be %d-byte aligned", 4 * esz);
        const int64_t nquads = outer * H * W / 4;
        const int64_t nb = (nquads + kThreads - 1) / kThreads;
        if (nb > 0x7fffffffLL) return fail(TTB_E_INVALID, "ttb_pack_bfp: tensor too large for one launch");
#define TTB_PACK_T(MB, S, TWO) pack_tiled_kernel<MB, S, TWO><<<(unsigned)nb, kThreads, 0, s>>>((const S *)src, (uint8_t *)dst, nquads)
        if (fmt == TTB_BFLOAT8_B) {
            if (esz == 4) { if (two_pass) TTB_PACK_T(7, float, true); else TTB_PACK_T(7, float, false); }
            else          { if (two_pass) TTB_PACK_T(7, uint16_t, true); else TTB_PACK_T(7, uint16_t, false); }
        } else {
            if (esz == 4) { if (two_pass) TTB_PACK_T(3, float, true); else TTB_PACK_T(3, float, false); }
            else          { if (two_pass) TTB_PACK_T(3, uint16_t, true); else TTB_PACK_T(3, uint16_t, false); }
        }
#undef TTB_PACK_T
    }
    TTB_LAUNCH_CHECK("pack_bfp");
    return TTB_OK;
}

int32_t ttb_unpack_bfp(const void *src, int32_t fmt, void *dst, int32_t dst_dtype, int64_t outer, int64_t H, int64_t W,
                       int32_t dst_row_major, int32_t two_pass, void *stream) {
    if (!src || !dst) return fail(TTB_E_INVALID, "ttb_unpack_bfp: null pointer");
    if (fmt != TTB_BFLOAT8_B && fmt != TTB_BFLOAT4_B) return fail(TTB_E_INVALID, "ttb_unpack_bfp: fmt must be bfloat8_b or bfloat4_b");
    if (dst_dtype != TTB_FLOAT32 && dst_dtype != TTB_BFLOAT16)
        return fail(TTB_E_INVALID, "ttb_unpack_bfp: destination dtype must be float32 or bfloat16");
    if (!aligned(src, 16)) return fail(TTB_E_INVALID, "ttb_unpack_bfp: source must be 16-byte aligned");
    const int esz = dst_dtype == TTB_FLOAT32 ? 4 : 2;
    auto s = (cudaStream_t)stream;
    if (dst_row_major) {
        StripGeom g; int64_t n;
        if (int32_t rc = make_geom("ttb_unpack_bfp", outer, H, W, g, n)) return rc;
        const bool vec = (W % 4 == 0) && aligned(dst, 4 * esz);
#define TTB_UNPACK_RM(MB, D, TWO) \
    unpack_rowmajor_kernel<MB, D, TWO><<<(unsigned)n, kThreads, 0, s>>>((const uint8_t *)src, (D *)dst, g, vec)
        if (fmt == TTB_BFLOAT8_B) {
            if (esz == 4) { if (two_pass) TTB_UNPACK_RM(7, float, true); else TTB_UNPACK_RM(7, float, false); }
            else          { if (two_pass) TTB_UNPACK_RM(7, uint16_t, true); else TTB_UNPACK_RM(7, uint16_t, false); }
        } else {
            if (esz == 4) { if (two_pass) TTB_UNPACK_RM(3, float, true); else TTB_UNPACK_RM(3, float, false); }
            else          { if (two_pass) TTB_UNPACK_RM(3, uint16_t, true); else TTB_UNPACK_RM(3, uint16_t, false); }
        }
#undef TTB_UNPACK_RM
    } else {
        if (outer <= 0 || H <= 0 || W <= 0 || H % 32 || W % 32)
            return fail(TTB_E_INVALID, "ttb_unpack_bfp: a tiled destination needs positive H, W that are multiples of 32");
        if (!aligned(dst, 4 * esz)) return fail(TTB_E_INVALID, "ttb_unpack_bfp: tiled destination must be %d-byte aligned", 4 * esz);
        const int64_t nquads = outer * H * W / 4;
        const int64_t nb = (nquads + kThreads - 1) / kThreads;
        if (nb > 0x7fffffffLL) return fail(TTB_E_INVALID, "ttb_unpack_bfp: tensor too large for one launch");
#define TTB_UNPACK_T(MB, D, TWO) unpack_tiled_kernel<MB, D, TWO><<<(unsigned)nb, kThreads, 0, s>>>((const uint8_t *)src, (D *)dst, nquads)
        if (fmt == TTB_BFLOAT8_B) {
            if (esz == 4) { if (two_pass) TTB_UNPACK_T(7, float, true); else TTB_UNPACK_T(7, float, false); }
            else          { if (two_pass) TTB_UNPACK_T(7, uint16_t, true); else TTB_UNPACK_T(7, uint16_t, false); }
        } else {
            if (esz == 4) { if (two_pass) TTB_UNPACK_T(3, float, true); else TTB_UNPACK_T(3, float, false); }
            else          { if (two_pass) TTB_UNPACK_T(3, uint16_t, true); else TTB_UNPACK_T(3, uint16_t, false); }
        }
#undef TTB_UNPACK_T
    }
    TTB_LAUNCH_CHECK("unpack_bfp");
    return TTB_OK;
}

}  // extern "C"
