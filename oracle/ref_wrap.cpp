// C entry points around the reference's own host headers, compiled from where they lie in the
// reference tree (nothing is copied). TEST INFRASTRUCTURE ONLY: it validates the C restatement
// in bfp_oracle.c and serves as the timed CPU baseline; no product code path may call it.
#include <cstdint>
#include <cstring>
#include <vector>
#include "common/bfloat8.hpp"
#include "common/bfloat4.hpp"
#include "common/test_tiles.hpp"

namespace {
std::vector<uint32_t> shape4(int64_t outer, int64_t H, int64_t W) {
    return {1u, static_cast<uint32_t>(outer), static_cast<uint32_t>(H), static_cast<uint32_t>(W)};
}
std::vector<uint32_t> pack(const std::vector<float>& v, int fmt, bool rm) {
    return fmt == 0 ? pack_fp32_vec_as_bfp8_tiles(v, rm, false) : pack_fp32_vec_as_bfp4_tiles(v, rm, false);
}
std::vector<float> unpack(const std::vector<uint32_t>& v, int fmt, bool rm) {
    return fmt == 0 ? unpack_bfp8_tiles_into_float_vec(v, rm, false) : unpack_bfp4_tiles_into_float_vec(v, rm, false);
}
size_t words_per_tile(int fmt) { return fmt == 0 ? 272 : 144; }
}  // namespace

extern "C" {

void ref_tilize_f32(const float* src, float* dst, int64_t outer, int64_t H, int64_t W) {
    std::vector<float> in(src, src + outer * H * W);
    auto out = convert_layout(in, shape4(outer, H, W), TensorLayout::LIN_ROW_MAJOR, TensorLayout::TILED32_4FACES);
    std::memcpy(dst, out.data(), out.size() * sizeof(float));
}

void ref_untilize_f32(const float* src, float* dst, int64_t outer, int64_t H, int64_t W) {
    std::vector<float> in(src, src + outer * H * W);
    auto out = convert_layout(in, shape4(outer, H, W), TensorLayout::TILED32_4FACES, TensorLayout::LIN_ROW_MAJOR);
    std::memcpy(dst, out.data(), out.size() * sizeof(float));
}

void ref_pack_bfp(const float* src, uint32_t* dst, int fmt, int64_t ntiles, int in_tile_row_major) {
    std::vector<float> in(src, src + ntiles * 1024);
    auto out = pack(in, fmt, in_tile_row_major != 0);
    std::memcpy(dst, out.data(), out.size() * sizeof(uint32_t));
}

void ref_unpack_bfp(const uint32_t* src, float* dst, int fmt, int64_t ntiles, int in_tile_row_major) {
    std::vector<uint32_t> in(src, src + ntiles * words_per_tile(fmt));
    auto out = unpack(in, fmt, in_tile_row_major != 0);
    std::memcpy(dst, out.data(), out.size() * sizeof(float));
}

// The steps ttnn.from_torch(dtype=bfloat8_b|bfloat4_b, layout=TILE_LAYOUT) performs on the host.
void ref_from_torch_bfp(const float* src, uint32_t* dst, int fmt, int64_t outer, int64_t H, int64_t W) {
    std::vector<float> in(src, src + outer * H * W);
    auto p1 = pack(in, fmt, false);
    auto u1 = unpack(p1, fmt, false);
    auto t1 = convert_layout(u1, shape4(outer, H, W), TensorLayout::LIN_ROW_MAJOR, TensorLayout::TILED32_4FACES);
    auto out = pack(t1, fmt, false);
    std::memcpy(dst, out.data(), out.size() * sizeof(uint32_t));
}

// The steps ttnn.to_torch performs on the host for a tiled block-float tensor.
void ref_to_torch_bfp(const uint32_t* src, float* dst, int fmt, int64_t outer, int64_t H, int64_t W) {
    int64_t ntiles = outer * H * W / 1024;
    std::vector<uint32_t> in(src, src + ntiles * words_per_tile(fmt));
    auto u1 = unpack(in, fmt, false);
    auto r1 = convert_layout(u1, shape4(outer, H, W), TensorLayout::TILED32_4FACES, TensorLayout::LIN_ROW_MAJOR);
    auto p1 = pack(r1, fmt, false);
    auto out = unpack(p1, fmt, false);
    std::memcpy(dst, out.data(), out.size() * sizeof(float));
}

}  // extern "C"
