// Layout conversion and block-float pack / unpack kernels for sm_100a, plus their C-ABI entry points.
//
// All four conversions are HBM-bound byte shuffles (4 + 1.0625 bytes per element for bfloat8_b).
// Work unit: a "strip" of up to four horizontally adjacent 32x32 tiles. One 256-thread block
// handles one strip; eight threads cover the 128 row-major columns of one row (64 contiguous bytes of fp32 each), and the
// packed side is staged in shared memory so that whole tiles (1088 / 576 contiguous bytes each, four tiles adjacent) move
// as 16-byte vectors.
// One thread owns one face row (16 values = one shared exponent): no shuffles, and its 16 codes leave as one 16-byte
// (bfloat8_b) or 8-byte (bfloat4_b) store.
//
// Arithmetic. The reference's integer recipe per value - align the 24-bit significand to the row exponent E with a
// truncating shift, add half, shift again, saturate - equals floor(|x| * 2^(133 - E) + 1/2) (bfloat8_b; 129 - E for
// bfloat4_b), because floor((floor(a) + c) / n) = floor((a + c) / n) for integers c, n. One fused multiply-add with
// round-toward-zero, |x| * 2^(133-E) + 32768.5, leaves exactly that integer in bits 8..15 of the result (the binade
// [2^15, 2^16) has a grid of 2^-8, rounding toward zero onto it cannot cross an integer), so a code costs one FMA and a
// byte select; signs, the saturation of 128 to 127 and the dropped sign of a zero mantissa are fixed up four codes at a
// time with byte-parallel integer operations. Rows where this shortcut would differ from the integer recipe - E < 24
// (denormal inputs keep their forced hidden bit, the scale would overflow) or E = 255 (Inf / NaN) - take the integer
// recipe itself. Unpacking is the mirror image: (sign << 31) | (mantissa << 16) is, read as a float, mantissa * 2^-133, and
// two multiplications by powers of two give mantissa * 2^(E - 133) exactly; rows with E < 7 or E = 255, where the
// reference's unclamped exponent arithmetic wraps, take the integer recipe.
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

// ---- one face row (16 values) at a time --------------------------------------------------------------------------
__device__ __forceinline__ float fma_rz(float a, float b, float c) {
    float d;
    asm("fma.rz.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Shared exponent of 16 values: the largest exponent field.
__device__ __forceinline__ uint32_t row_exponent16(const uint32_t (&u)[16]) {
    uint32_t m = u[0] & 0x7fffffffu;
#pragma unroll
    for (int i = 1; i < 16; ++i) m = max(m, u[i] & 0x7fffffffu);
    return m >> 23;
}

// Codes of 16 values under their shared exponent E, packed as the reference packs them: bfloat8_b one byte per value
// (four words), bfloat4_b one nibble per value, even value in the low nibble (two words).
template <int MB>
__device__ __forceinline__ void encode_row(const uint32_t (&u)[16], uint32_t E, uint32_t (&w)[4]) {
    constexpr uint32_t kMant = MB == 7 ? 0x7f7f7f7fu : 0x07070707u;        // mantissa bits of a code, per byte
    constexpr uint32_t kTop = MB == 7 ? 0x80808080u : 0x08080808u;         // the bit above them: sign, or a mantissa of 2^MB
    if (E >= 24u && E <= 254u) {
        const float scale = __uint_as_float(((MB == 7 ? 260u : 256u) - E) << 23);   // 2^(133 - E) / 2^(129 - E)
        uint32_t cw[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t t[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) t[i] = __float_as_uint(fma_rz(fabsf(__uint_as_float(u[4 * q + i])), scale, 32768.5f));
            // mantissas (0 .. 2^MB) in bytes; signs from the top bytes of the values
            uint32_t m = __byte_perm(__byte_perm(t[0], t[1], 0x0051u), __byte_perm(t[2], t[3], 0x0051u), 0x5410u);
            uint32_t sg = __byte_perm(__byte_perm(u[4 * q], u[4 * q + 1], 0x0073u), __byte_perm(u[4 * q + 2], u[4 * q + 3], 0x0073u), 0x5410u);
            if (MB == 3) sg >>= 4;
            m -= (m >> MB) & 0x01010101u;                                   // saturate 2^MB to 2^MB - 1
            const uint32_t nz = (m + kMant) & kTop;                         // top bit set where the mantissa is not zero
            cw[q] = m | (sg & nz);                                          // the sign survives only beside a mantissa
        }
        if (MB == 7) {
            w[0] = cw[0]; w[1] = cw[1]; w[2] = cw[2]; w[3] = cw[3];
        } else {
            w[0] = __byte_perm(cw[0], cw[1], 0x6420u) | (__byte_perm(cw[0], cw[1], 0x7531u) << 4);
            w[1] = __byte_perm(cw[2], cw[3], 0x6420u) | (__byte_perm(cw[2], cw[3], 0x7531u) << 4);
            w[2] = w[3] = 0u;
        }
    } else {
        // the integer recipe itself
        w[0] = w[1] = w[2] = w[3] = 0u;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t c = bfp_to_code<MB>(u[i], E);
            if (MB == 7) w[i >> 2] |= c << (8 * (i & 3));
            else w[i >> 3] |= c << (4 * (i & 7));
        }
    }
}

// The inverse: 16 codes (packed as above) under exponent E -> fp32 bit patterns.
template <int MB>
__device__ __forceinline__ void decode_row(const uint32_t (&w)[4], uint32_t E, uint32_t (&u)[16]) {
    if (E >= 7u && E <= 254u) {
        // value = +-m * 2^(E - 133) (bfloat8_b) or +-m * 2^(E - 129): the code's bits placed as a subnormal float times 2^E,
        // in two exact steps because 2^E alone need not be a float
        const uint32_t e1 = min(E, 127u), e2 = E - e1;
        const float s1 = __uint_as_float((e1 + 127u) << 23), s2 = __uint_as_float((e2 + 127u) << 23);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            uint32_t x;
            if (MB == 7) {
                x = __byte_perm(w[i >> 2], 0u, 0x0044u | ((uint32_t)(i & 3) << 12) | ((uint32_t)(i & 3) << 8)) & 0x807f0000u;   // [0, 0, c, c]
            } else {
                const uint32_t c = (w[i >> 3] >> (4 * (i & 7))) & 0xfu;
                x = ((c & 8u) << 28) | ((c & 7u) << 20);
            }
            u[i] = __float_as_uint(__uint_as_float(x) * s1 * s2);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t c = MB == 7 ? (w[i >> 2] >> (8 * (i & 3))) & 0xffu : (w[i >> 3] >> (4 * (i & 7))) & 0xfu;
            u[i] = bfp_from_code<MB>(c, E);
        }
    }
}

// Four codes of one face row (bfloat8_b: the four bytes of `cw`; bfloat4_b: its four low nibbles) -> fp32 bit patterns.
template <int MB>
__device__ __forceinline__ void decode4(uint32_t cw, uint32_t E, uint32_t (&u)[4]) {
    if (E >= 7u && E <= 254u) {
        const uint32_t e1 = min(E, 127u), e2 = E - e1;
        const float s1 = __uint_as_float((e1 + 127u) << 23), s2 = __uint_as_float((e2 + 127u) << 23);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t x;
            if (MB == 7) {
                x = __byte_perm(cw, 0u, 0x0044u | ((uint32_t)i << 12) | ((uint32_t)i << 8)) & 0x807f0000u;   // [0, 0, c, c]
            } else {
                const uint32_t c = (cw >> (4 * i)) & 0xfu;
                x = ((c & 8u) << 28) | ((c & 7u) << 20);
            }
            u[i] = __float_as_uint(__uint_as_float(x) * s1 * s2);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) u[i] = bfp_from_code<MB>(MB == 7 ? (cw >> (8 * i)) & 0xffu : (cw >> (4 * i)) & 0xfu, E);
    }
}

// Pack of one face row; with TWO the pack -> unpack -> pack sequence of the reference's host from_torch.
template <int MB, bool TWO>
__device__ __forceinline__ void pack_row(uint32_t (&u)[16], uint32_t &E, uint32_t (&w)[4]) {
    E = row_exponent16(u);
    encode_row<MB>(u, E, w);
    if (TWO) {
        decode_row<MB>(w, E, u);
        E = row_exponent16(u);
        encode_row<MB>(u, E, w);
    }
}
// Unpack of one face row; with TWO unpack -> pack -> unpack as the reference's to_torch does.
template <int MB, bool TWO>
__device__ __forceinline__ void unpack_row(const uint32_t (&w)[4], uint32_t E, uint32_t (&u)[16]) {
    decode_row<MB>(w, E, u);
    if (TWO) {
        uint32_t E2, w2[4];
        pack_row<MB, false>(u, E2, w2);
        decode_row<MB>(w2, E2, u);
    }
}

struct StripGeom {
    int64_t H, W;        // logical rows / columns of one outer slice
    int64_t Ht, Wt;      // tiles per slice vertically / horizontally (padded)
    int64_t strips_x;    // strips per tile row
};

// ---------------------------------------------------------------------------------------------
// Row-major [outer, H, W] (fp32 or bf16) -> packed tiles, zero padding to 32 fused.
// Thread t of a block: row t / 8 of the strip's tile row, 16-column group t % 8 of its 128 columns.
template <int MB, typename S, bool TWO>
__global__ void __launch_bounds__(kThreads) pack_rowmajor_kernel(const S *__restrict__ src, uint8_t *__restrict__ dst,
                                                                  StripGeom g, bool vec_ok) {
    constexpr int TB = MB == 7 ? kBfp8TileBytes : kBfp4TileBytes;
    __shared__ __align__(16) uint8_t stage[kStripTiles * TB];
    const int64_t strip = blockIdx.x;
    const int64_t tile_row = strip / g.strips_x;           // over outer * Ht
    const int64_t sx = strip % g.strips_x;
    const int64_t o = tile_row / g.Ht, hr = tile_row % g.Ht;
    const int r = threadIdx.x >> 3, grp = threadIdx.x & 7;
    const int64_t col = sx * 128 + grp * 16;
    const int64_t h = hr * 32 + r;
    const int ntiles = (int)imin(kStripTiles, g.Wt - sx * kStripTiles);

    uint32_t u[16];
    {
        const int64_t rem = h < g.H ? g.W - col : 0;
        const S *p = src + ((o * g.H + h) * g.W + col);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int valid = rem > 4 * q ? (int)imin(4, rem - 4 * q) : 0;
            uint32_t v[4] = {0u, 0u, 0u, 0u};
            if (valid) Src<S>::load4(p + 4 * q, vec_ok && valid == 4, valid, v);
            u[4 * q] = v[0]; u[4 * q + 1] = v[1]; u[4 * q + 2] = v[2]; u[4 * q + 3] = v[3];
        }
    }
    uint32_t E, w[4];
    pack_row<MB, TWO>(u, E, w);
    {
        const int face = 2 * (r >> 4) + (grp & 1), fr = r & 15;
        uint8_t *t = stage + (grp >> 1) * TB;
        t[16 * face + fr] = (uint8_t)E;
        if (MB == 7)
            *reinterpret_cast<uint4 *>(t + 64 + 256 * face + 16 * fr) = make_uint4(w[0], w[1], w[2], w[3]);
        else
            *reinterpret_cast<uint2 *>(t + 64 + 128 * face + 8 * fr) = make_uint2(w[0], w[1]);
    }
    __syncthreads();
    uint4 *out = reinterpret_cast<uint4 *>(dst + (tile_row * g.Wt + sx * kStripTiles) * TB);
    const uint4 *in = reinterpret_cast<const uint4 *>(stage);
    for (int i = threadIdx.x; i < ntiles * (TB / 16); i += kThreads) out[i] = in[i];
}

// Tiled source (already in face order) -> packed tiles; one thread per face row of 16 consecutive values.
template <int MB, typename S, bool TWO>
__global__ void __launch_bounds__(kThreads) pack_tiled_kernel(const S *__restrict__ src, uint8_t *__restrict__ dst,
                                                               int64_t nrows) {
    constexpr int TB = MB == 7 ? kBfp8TileBytes : kBfp4TileBytes;
    const int64_t q = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (q >= nrows) return;
    uint32_t u[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t v[4];
        Src<S>::load4(src + q * 16 + 4 * i, true, 4, v);
        u[4 * i] = v[0]; u[4 * i + 1] = v[1]; u[4 * i + 2] = v[2]; u[4 * i + 3] = v[3];
    }
    uint32_t E, w[4];
    pack_row<MB, TWO>(u, E, w);
    uint8_t *t = dst + (q >> 6) * TB;
    const int row = (int)(q & 63);
    t[row] = (uint8_t)E;
    if (MB == 7)
        *reinterpret_cast<uint4 *>(t + 64 + 16 * row) = make_uint4(w[0], w[1], w[2], w[3]);
    else
        *reinterpret_cast<uint2 *>(t + 64 + 8 * row) = make_uint2(w[0], w[1]);
}

// Packed tiles -> row-major [outer, H, W] (fp32 or bf16), padding dropped. Four values per thread: a warp writes 128
// consecutive columns (512 B of fp32) of one row with one store instruction. (One face row per thread, as in the packers,
// makes every store instruction write half sectors: measured 15 % slower.) The two-pass form needs whole face rows and keeps
// the row-per-thread mapping.
template <int MB, typename D, bool TWO>
__global__ void __launch_bounds__(kThreads) unpack_rowmajor_kernel(const uint8_t *__restrict__ src, D *__restrict__ dst,
                                                                    StripGeom g, bool vec_ok) {
    constexpr int TB = MB == 7 ? kBfp8TileBytes : kBfp4TileBytes;
    __shared__ __align__(16) uint8_t stage[kStripTiles * TB];
    const int64_t strip = blockIdx.x;
    const int64_t tile_row = strip / g.strips_x;
    const int64_t sx = strip % g.strips_x;
    const int64_t o = tile_row / g.Ht, hr = tile_row % g.Ht;
    const int ntiles = (int)imin(kStripTiles, g.Wt - sx * kStripTiles);
    {
        const uint4 *in = reinterpret_cast<const uint4 *>(src + (tile_row * g.Wt + sx * kStripTiles) * TB);
        uint4 *st = reinterpret_cast<uint4 *>(stage);
        for (int i = threadIdx.x; i < kStripTiles * (TB / 16); i += kThreads)
            st[i] = i < ntiles * (TB / 16) ? __ldg(in + i) : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    if (TWO) {
        const int r = threadIdx.x >> 3, grp = threadIdx.x & 7;
        const int64_t col = sx * 128 + grp * 16;
        const int64_t h = hr * 32 + r;
        const int64_t rem = h < g.H ? g.W - col : 0;
        if (rem <= 0) return;
        const int face = 2 * (r >> 4) + (grp & 1), fr = r & 15;
        const uint8_t *t = stage + (grp >> 1) * TB;
        const uint32_t E = t[16 * face + fr];
        uint32_t w[4] = {0u, 0u, 0u, 0u}, u[16];
        if (MB == 7) {
            const uint4 v = *reinterpret_cast<const uint4 *>(t + 64 + 256 * face + 16 * fr);
            w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
        } else {
            const uint2 v = *reinterpret_cast<const uint2 *>(t + 64 + 128 * face + 8 * fr);
            w[0] = v.x; w[1] = v.y;
        }
        unpack_row<MB, true>(w, E, u);
        D *p = dst + ((o * g.H + h) * g.W + col);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int valid = rem > 4 * q ? (int)imin(4, rem - 4 * q) : 0;
            const uint32_t v[4] = {u[4 * q], u[4 * q + 1], u[4 * q + 2], u[4 * q + 3]};
            if (valid) Dst<D>::store4(p + 4 * q, vec_ok && valid == 4, valid, v);
        }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
        const uint32_t cw = MB == 7 ? *reinterpret_cast<const uint32_t *>(t + 64 + k) : (uint32_t)*reinterpret_cast<const uint16_t *>(t + 64 + (k >> 1));
        uint32_t u[4];
        decode4<MB>(cw, E, u);
        const int64_t h = hr * 32 + r;
        const int64_t rem = g.W - col;
        const int valid = (h < g.H && rem > 0) ? (int)imin(4, rem) : 0;
        if (valid) Dst<D>::store4(dst + ((o * g.H + h) * g.W + col), vec_ok && valid == 4, valid, u);
    }
}

// Packed tiles -> tiled values (face order); four consecutive values per thread (a face row per thread in the two-pass form).
template <int MB, typename D, bool TWO>
__global__ void __launch_bounds__(kThreads) unpack_tiled_kernel(const uint8_t *__restrict__ src, D *__restrict__ dst,
                                                                 int64_t nrows) {
    constexpr int TB = MB == 7 ? kBfp8TileBytes : kBfp4TileBytes;
    const int64_t id = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (TWO) {
        const int64_t q = id;
        if (q >= nrows) return;
        const uint8_t *t = src + (q >> 6) * TB;
        const int row = (int)(q & 63);
        const uint32_t E = __ldg(t + row);
        uint32_t w[4] = {0u, 0u, 0u, 0u}, u[16];
        if (MB == 7) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(t + 64 + 16 * row));
            w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
        } else {
            const uint2 v = __ldg(reinterpret_cast<const uint2 *>(t + 64 + 8 * row));
            w[0] = v.x; w[1] = v.y;
        }
        unpack_row<MB, true>(w, E, u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t v[4] = {u[4 * i], u[4 * i + 1], u[4 * i + 2], u[4 * i + 3]};
            Dst<D>::store4(dst + q * 16 + 4 * i, true, 4, v);
        }
        return;
    }
    if (id >= nrows * 4) return;
    const int64_t tile = id >> 8;
    const int wq = (int)(id & 255);   // which group of four values of the tile
    const uint8_t *t = src + tile * TB;
    const uint32_t E = __ldg(t + (wq >> 2));
    const uint32_t cw = MB == 7 ? __ldg(reinterpret_cast<const uint32_t *>(t + 64 + 4 * wq)) : (uint32_t)__ldg(reinterpret_cast<const uint16_t *>(t + 64 + 2 * wq));
    uint32_t u[4];
    decode4<MB>(cw, E, u);
    Dst<D>::store4(dst + id * 4, true, 4, u);
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
        const int64_t nrows = outer * H * W / 16;
        const int64_t nb = (nrows + kThreads - 1) / kThreads;
        if (nb > 0x7fffffffLL) return fail(TTB_E_INVALID, "ttb_pack_bfp: tensor too large for one launch");
#define TTB_PACK_T(MB, S, TWO) pack_tiled_kernel<MB, S, TWO><<<(unsigned)nb, kThreads, 0, s>>>((const S *)src, (uint8_t *)dst, nrows)
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
        const int64_t nrows = outer * H * W / 16;
        const int64_t nb = ((two_pass ? nrows : nrows * 4) + kThreads - 1) / kThreads;
        if (nb > 0x7fffffffLL) return fail(TTB_E_INVALID, "ttb_unpack_bfp: tensor too large for one launch");
#define TTB_UNPACK_T(MB, D, TWO) unpack_tiled_kernel<MB, D, TWO><<<(unsigned)nb, kThreads, 0, s>>>((const uint8_t *)src, (D *)dst, nrows)
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
