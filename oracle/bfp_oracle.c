/*
 * CPU oracle for the block-float weight path: TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement (integer arithmetic on raw IEEE-754 bit patterns) of the
 * reference's host tilize / bfloat8_b / bfloat4_b pack / unpack routines. It exists so that
 * the CUDA kernels can be checked bit for bit; no product code path may call it.
 * Each function names the reference source it follows (paths inside the tt-metal tree).
 *
 * Parity status: PINNED. tests/test_oracle.py checks every function here against the
 * reference's own headers compiled out of tree (oracle/_ref/libttref.so, built by the
 * Makefile beside this file) and against golden vectors under tests/golden/.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>

#define ORC_BFP8_B 0
#define ORC_BFP4_B 1

/* Bytes of one packed 32x32 tile: 64 exponent bytes + 1024 codes of 8 or 4 bits.
 * tt_metal/common/tt_backend_api_types.hpp:109-132 (tile_size), constants.hpp. */
static inline size_t tile_bytes(int fmt) { return fmt == ORC_BFP8_B ? 1088 : 576; }

/* Position of element (r, c) of a 32x32 tile inside the 4-face tile: faces ordered
 * top-left, top-right, bottom-left, bottom-right, each 16x16 row-major.
 * tt_metal/common/test_tiles.hpp:24-65 (convert_to_tile_layout). */
static inline int face_index(int r, int c) { return 256 * (2 * (r >> 4) + (c >> 4)) + 16 * (r & 15) + (c & 15); }

/* Row-major [outer, H, W] -> tiles (row-major over (outer*H/32, W/32)) of four faces.
 * H and W must be multiples of 32. elem = bytes per element (2 or 4).
 * tt_metal/common/test_tiles.hpp:124-158 (tilize_nchw) then :24-65 (convert_to_tile_layout),
 * composed as in convert_layout :178-213. */
void orc_tilize(const void *src, void *dst, int elem, int64_t outer, int64_t H, int64_t W) {
    const uint8_t *s = (const uint8_t *)src;
    uint8_t *d = (uint8_t *)dst;
    int64_t wt = W / 32;
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t w = 0; w < W; ++w) {
                int64_t t = (o * (H / 32) + h / 32) * wt + w / 32;
                int64_t di = 1024 * t + face_index((int)(h & 31), (int)(w & 31));
                memcpy(d + di * elem, s + ((o * H + h) * W + w) * elem, (size_t)elem);
            }
}

/* Inverse of orc_tilize. test_tiles.hpp:67-88 (convert_to_flat_layout) then :91-119 (untilize_nchw). */
void orc_untilize(const void *src, void *dst, int elem, int64_t outer, int64_t H, int64_t W) {
    const uint8_t *s = (const uint8_t *)src;
    uint8_t *d = (uint8_t *)dst;
    int64_t wt = W / 32;
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t w = 0; w < W; ++w) {
                int64_t t = (o * (H / 32) + h / 32) * wt + w / 32;
                int64_t si = 1024 * t + face_index((int)(h & 31), (int)(w & 31));
                memcpy(d + ((o * H + h) * W + w) * elem, s + si * elem, (size_t)elem);
            }
}

/* Shared exponent of 16 fp32 values = the largest biased exponent field.
 * tt_metal/common/blockfloat_common.hpp:19-47 (get_max_exp, is_exp_a = false). */
static inline uint32_t max_exp16(const uint32_t *u) {
    uint32_t m = 0;
    for (int i = 0; i < 16; ++i) {
        uint32_t e = (u[i] & 0x7f800000u) >> 23;
        if (e > m) m = e;
    }
    return m;
}

/* One fp32 bit pattern -> sign + mantissa code under the shared exponent.
 * mbits = 7 (bfloat8_b) or 3 (bfloat4_b).
 * tt_metal/common/bfloat8.hpp:23-87 (convert_u32_to_bfp8) and
 * blockfloat_common.hpp:67-147 (convert_u32_to_bfp<Fmt>): hidden one OR-ed in even for a zero
 * exponent field, truncating alignment shift, then add-half and shift (round half up),
 * mantissa saturates, the sign is dropped when the mantissa rounds to zero. */
static inline uint32_t to_code(uint32_t u, uint32_t shared_exp, int mbits) {
    if ((u & 0x7fffffffu) == 0) return 0;
    uint32_t man = (u & 0x007fffffu) | (1u << 23);
    uint32_t exp = (u & 0x7f800000u) >> 23;
    uint32_t sign = u >> 31;
    if (shared_exp >= exp) {
        uint32_t diff = shared_exp - exp;
        while (diff > 31) { man >>= 31; diff -= 31; }
        man >>= diff;
    }
    int shift = 24 - mbits;
    uint32_t maxv = (1u << mbits) - 1;
    man += 1u << (shift - 1);
    man >>= shift;
    if (man > maxv) man = maxv;
    if (man == 0) sign = 0;
    return (sign << mbits) | man;
}

/* Pack ntiles*1024 fp32 values (given as raw bits) into ntiles packed tiles.
 * in_tile_row_major = 0: the input already is in 4-face order, consumed sequentially;
 * in_tile_row_major = 1: each tile's 1024 values are a row-major 32x32 block.
 * Output per tile: 64 exponent bytes (byte 16*face + row), then the codes face by face;
 * bfloat8_b one byte per code, bfloat4_b two codes per byte with the even element low.
 * bfloat8.hpp:102-173 (pack_fp32_vec_as_bfp8_tiles), bfloat4.hpp:23-25 and
 * blockfloat_common.hpp:174-258 (pack_fp32_vec_as_bfp_tiles), :149-172 (word packing),
 * :49-57 (exponent word packing). */
void orc_pack_bfp(const uint32_t *bits, uint8_t *out, int fmt, int64_t ntiles, int in_tile_row_major) {
    int mbits = fmt == ORC_BFP8_B ? 7 : 3;
    size_t tb = tile_bytes(fmt);
    for (int64_t t = 0; t < ntiles; ++t) {
        const uint32_t *tin = bits + t * 1024;
        uint8_t *tout = out + (size_t)t * tb;
        uint8_t *data = tout + 64;
        if (fmt == ORC_BFP4_B) memset(data, 0, 512);
        for (int f = 0; f < 4; ++f)
            for (int i = 0; i < 16; ++i) {
                uint32_t row[16];
                for (int j = 0; j < 16; ++j) {
                    int idx = in_tile_row_major ? ((f >> 1) * 16 + i) * 32 + (f & 1) * 16 + j : 256 * f + 16 * i + j;
                    row[j] = tin[idx];
                }
                uint32_t e = max_exp16(row);
                tout[16 * f + i] = (uint8_t)e;
                for (int j = 0; j < 16; ++j) {
                    uint32_t c = to_code(row[j], e, mbits);
                    int k = 256 * f + 16 * i + j;
                    if (fmt == ORC_BFP8_B) data[k] = (uint8_t)c;
                    else data[k >> 1] |= (uint8_t)((c & 0xf) << (4 * (k & 1)));
                }
            }
    }
}

/* One code -> fp32 bits. The leading one of the mantissa is shifted up to the top mantissa
 * bit, the exponent drops by the shift count in wrapping 32-bit arithmetic (no clamp), a zero
 * mantissa yields a signed zero.
 * bfloat8.hpp:206-258, bfloat4.hpp:76-158. */
static inline uint32_t from_code(uint32_t code, uint32_t shared_exp, int mbits) {
    uint32_t sign = code >> mbits;
    uint32_t man = code & ((1u << mbits) - 1);
    if (man == 0) return sign << 31;
    uint32_t top = 1u << (mbits - 1);
    uint32_t cnt = 0;
    while (man < top) { man <<= 1; ++cnt; }
    man = (man << 1) & ((1u << mbits) - 1);
    uint32_t exp = shared_exp - cnt; /* wraps like the reference's epi32 subtraction */
    return (sign << 31) | (exp << 23) | (man << (23 - mbits));
}

/* Unpack ntiles packed tiles to fp32 bits, 4-face order (in_tile_row_major = 0) or each
 * tile as a row-major 32x32 block (1).
 * bfloat8.hpp:175-265 (unpack_bfp8_tiles_into_float_vec), bfloat4.hpp:33-164. */
void orc_unpack_bfp(const uint8_t *in, uint32_t *bits, int fmt, int64_t ntiles, int in_tile_row_major) {
    int mbits = fmt == ORC_BFP8_B ? 7 : 3;
    size_t tb = tile_bytes(fmt);
    for (int64_t t = 0; t < ntiles; ++t) {
        const uint8_t *tin = in + (size_t)t * tb;
        const uint8_t *data = tin + 64;
        uint32_t *tout = bits + t * 1024;
        for (int f = 0; f < 4; ++f)
            for (int i = 0; i < 16; ++i) {
                uint32_t e = tin[16 * f + i];
                for (int j = 0; j < 16; ++j) {
                    int k = 256 * f + 16 * i + j;
                    uint32_t c = fmt == ORC_BFP8_B ? data[k] : (uint32_t)((data[k >> 1] >> (4 * (k & 1))) & 0xf);
                    int idx = in_tile_row_major ? ((f >> 1) * 16 + i) * 32 + (f & 1) * 16 + j : k;
                    tout[idx] = from_code(c, e, mbits);
                }
            }
    }
}

/* What ttnn.from_torch(dtype=bfloat8_b|bfloat4_b, layout=TILE_LAYOUT) leaves in the tensor's
 * buffer for a row-major fp32 [outer, H, W] input with H, W multiples of 32, following the
 * reference's steps literally: pack the row-major stream 16 values at a time, unpack, tilize
 * the fp32 values, pack again.
 * tt_eager/tt_lib/csrc/tt_lib_bindings_tensor_pytensor.cpp:145-160 (first pack),
 * tt_eager/tensor/tensor_impl.cpp:179-197, 232-250 (to_layout_bfloat8_b / 4_b).
 * scratch must hold 2 * outer*H*W uint32 plus the packed size in bytes. */
void orc_from_torch_bfp(const uint32_t *rm_bits, uint8_t *out, int fmt, int64_t outer, int64_t H, int64_t W,
                        uint8_t *scratch) {
    int64_t n = outer * H * W, ntiles = n / 1024;
    uint32_t *u1 = (uint32_t *)scratch;
    uint32_t *u2 = u1 + n;
    uint8_t *p1 = (uint8_t *)(u2 + n);
    orc_pack_bfp(rm_bits, p1, fmt, ntiles, 0);
    orc_unpack_bfp(p1, u1, fmt, ntiles, 0);
    orc_tilize(u1, u2, 4, outer, H, W);
    orc_pack_bfp(u2, out, fmt, ntiles, 0);
}

/* What ttnn.to_torch returns (fp32, row-major [outer, H, W]) for a tiled packed tensor:
 * unpack, untilize, pack as a row-major stream, unpack again.
 * tt_eager/tensor/tensor_impl.cpp:179-197 (to ROW_MAJOR), pytensor.cpp:382-393 (final unpack). */
void orc_to_torch_bfp(const uint8_t *in, uint32_t *rm_bits, int fmt, int64_t outer, int64_t H, int64_t W,
                      uint8_t *scratch) {
    int64_t n = outer * H * W, ntiles = n / 1024;
    uint32_t *u1 = (uint32_t *)scratch;
    uint32_t *u2 = u1 + n;
    uint8_t *p1 = (uint8_t *)(u2 + n);
    orc_unpack_bfp(in, u1, fmt, ntiles, 0);
    orc_untilize(u1, u2, 4, outer, H, W);
    orc_pack_bfp(u2, p1, fmt, ntiles, 0);
    orc_unpack_bfp(p1, rm_bits, fmt, ntiles, 0);
}
