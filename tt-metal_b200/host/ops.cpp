#include "ops.hpp"

#include <algorithm>
#include <cstring>

namespace ttnn_b200 {
namespace {

Device *current_or_default_device() {
    int32_t n = 0;
    check(ttb_device_count(&n), "ttnn: this conversion runs on the GPU and no CUDA device is usable");
    if (n <= 0) throw_error("ttnn: this conversion runs on the GPU (there is no CPU fallback) and no CUDA device is visible");
    int32_t cur = 0;
    check(ttb_get_device(&cur), "ttnn");
    return open_device(cur);
}

std::shared_ptr<DeviceBuffer> upload(Device *dev, const void *src, int64_t bytes) {
    auto b = allocate_device_buffer(dev, bytes);
    check(ttb_memcpy_h2d(b->ptr, src, (size_t)bytes, nullptr), "ttnn: host to device copy");
    return b;
}

void download(void *dst, const DeviceBuffer &b, int64_t bytes) {
    check(ttb_memcpy_d2h(dst, b.ptr, (size_t)bytes, nullptr), "ttnn: device to host copy");
    check(ttb_stream_synchronize(nullptr), "ttnn: device to host copy");
    // what is handed to the host has been computed without a wait running out
    if (b.device) b.device->check_device_status("ttnn: device to host copy");
}

Tensor to_host_storage(const Tensor &t) {
    auto h = std::make_shared<HostBuffer>();
    const int64_t bytes = t.buffer_bytes();
    h->bytes.resize((size_t)bytes);
    t.device()->make_current();
    download(h->bytes.data(), *t.device_buffer(), bytes);
    return Tensor(h, t.shape(), t.dtype(), t.layout());
}

Tensor to_device_storage(const Tensor &t, Device *dev) {
    auto b = upload(dev, t.host_buffer()->bytes.data(), t.buffer_bytes());
    return Tensor(b, t.shape(), t.dtype(), t.layout());
}

int ttb_dtype(DataType d) { return static_cast<int>(d); }

}  // namespace

Tensor from_host_buffer(const void *src, const std::vector<int64_t> &dims, DataType src_dtype, DataType dtype, Layout layout,
                        Device *device) {
    if (!src) throw_error("ttnn.from_torch: null data pointer");
    if (dims.empty()) throw_error("ttnn.from_torch: rank-0 tensors are not supported");
    Shape logical(dims);
    if (is_block_float(dtype)) {
        if (dims.size() < 2) throw_error("ttnn.from_torch: bfloat8_b/bfloat4_b requires at least 2 dimensions!");
        if (layout != Layout::TILE) throw_error("ttnn.from_torch: bfloat8_b/bfloat4_b requires TILE_LAYOUT!");
        if (src_dtype != DataType::FLOAT32 && src_dtype != DataType::BFLOAT16)
            throw_error("ttnn.from_torch: block-float tensors are packed from float32 or bfloat16 data");
    } else if (src_dtype != dtype) {
        throw_error("ttnn.from_torch: the host data must already have the requested element type");
    }
    if (!is_block_float(dtype) && layout == Layout::ROW_MAJOR && device == nullptr) {
        auto h = std::make_shared<HostBuffer>();
        h->bytes.assign((const uint8_t *)src, (const uint8_t *)src + logical.volume() * element_size(dtype));
        return Tensor(h, logical, dtype, layout);
    }
    Device *dev = device ? device : current_or_default_device();
    dev->make_current();
    const int64_t src_bytes = logical.volume() * element_size(src_dtype);
    auto staged = upload(dev, src, src_bytes);
    Tensor out;
    if (layout == Layout::ROW_MAJOR) {
        // the source (possibly a temporary of the caller, possibly pinned: then the copy is truly asynchronous) may be
        // released or overwritten as soon as this returns
        check(ttb_stream_synchronize(nullptr), "ttnn.from_torch");
        out = Tensor(staged, logical, dtype, layout);
    } else {
        Shape shape = logical.tile_padded();
        int64_t outer, H, W;
        logical.as_outer_hw(outer, H, W, false);
        auto dstb = allocate_device_buffer(dev, physical_bytes(shape, dtype, layout));
        if (is_block_float(dtype))
            check(ttb_pack_bfp(staged->ptr, ttb_dtype(src_dtype), dstb->ptr, ttb_dtype(dtype), outer, H, W, 1, /*two_pass=*/1, nullptr),
                  "ttnn.from_torch");
        else
            check(ttb_tilize(staged->ptr, dstb->ptr, element_size(dtype), outer, H, W, nullptr), "ttnn.from_torch");
        check(ttb_stream_synchronize(nullptr), "ttnn.from_torch");  // the staging buffer is released on return
        out = Tensor(dstb, shape, dtype, layout);
    }
    if (device == nullptr) return to_host_storage(out);
    return out;
}

DataType host_dtype_of(const Tensor &t) { return is_block_float(t.dtype()) ? DataType::FLOAT32 : t.dtype(); }

void to_host_buffer(const Tensor &t, void *dst) {
    if (!dst) throw_error("ttnn.to_torch: null destination");
    if (!t.is_allocated()) throw_error("ttnn.to_torch: the tensor has been deallocated");
    const Shape &shape = t.shape();
    if (t.storage_type() != StorageType::DEVICE && !is_block_float(t.dtype()) && t.layout() == Layout::ROW_MAJOR &&
        !shape.has_padding()) {
        std::memcpy(dst, t.host_buffer()->bytes.data(), (size_t)t.buffer_bytes());
        return;
    }
    Tensor d = t.storage_type() == StorageType::DEVICE ? t : to_device_storage(t, current_or_default_device());
    Device *dev = d.device();
    dev->make_current();
    int64_t outer, H, W;
    shape.as_outer_hw(outer, H, W, false);
    const DataType hd = host_dtype_of(d);
    const int64_t out_bytes = shape.volume() * element_size(hd);
    if (d.layout() == Layout::ROW_MAJOR && !is_block_float(d.dtype())) {
        if (shape.has_padding()) throw_error("ttnn.to_torch: padded row-major tensors are not supported");
        download(dst, *d.device_buffer(), out_bytes);
        return;
    }
    if (d.layout() != Layout::TILE) throw_error("ttnn.to_torch: block-float tensors must be in TILE_LAYOUT on this path");
    const size_t r = shape.rank();
    for (size_t i = 0; i + 2 < r; ++i)
        if (shape.padded()[i] != shape.dims()[i]) throw_error("ttnn.to_torch: padding is only supported on the last two dimensions");
    auto tmp = allocate_device_buffer(dev, out_bytes);
    if (is_block_float(d.dtype()))
        check(ttb_unpack_bfp(d.data(), ttb_dtype(d.dtype()), tmp->ptr, TTB_FLOAT32, outer, H, W, 1, /*two_pass=*/1, nullptr), "ttnn.to_torch");
    else
        check(ttb_untilize(d.data(), tmp->ptr, element_size(d.dtype()), outer, H, W, nullptr), "ttnn.to_torch");
    download(dst, *tmp, out_bytes);
}

Tensor to_layout(const Tensor &t, Layout layout) {
    if (layout != Layout::ROW_MAJOR && layout != Layout::TILE) throw_error("ttnn.to_layout: Unsupported layout!");
    if (t.layout() == layout) return t;
    const bool on_device = t.storage_type() == StorageType::DEVICE;
    Tensor d = on_device ? t : to_device_storage(t, current_or_default_device());
    Device *dev = d.device();
    dev->make_current();
    const Shape &shape = d.shape();
    int64_t outer, H, W;
    Tensor out;
    if (is_block_float(d.dtype())) {
        // The block-float "row-major" form is the packing of the row-major fp32 stream, 16 values per shared
        // exponent (to_layout_bfloat8_b / _4_b, tensor_impl.cpp:179-250); both directions go through fp32.
        shape.as_outer_hw(outer, H, W, true);
        auto f32 = allocate_device_buffer(dev, shape.padded_volume() * 4);
        auto dstb = allocate_device_buffer(dev, d.buffer_bytes());
        const int fmt = ttb_dtype(d.dtype());
        if (layout == Layout::ROW_MAJOR) {
            check(ttb_unpack_bfp(d.data(), fmt, f32->ptr, TTB_FLOAT32, outer, H, W, 1, 0, nullptr), "ttnn.to_layout");
            check(ttb_pack_bfp(f32->ptr, TTB_FLOAT32, dstb->ptr, fmt, 1, 32, shape.padded_volume() / 32, 0, 0, nullptr), "ttnn.to_layout");
        } else {
            check(ttb_unpack_bfp(d.data(), fmt, f32->ptr, TTB_FLOAT32, 1, 32, shape.padded_volume() / 32, 0, 0, nullptr), "ttnn.to_layout");
            check(ttb_pack_bfp(f32->ptr, TTB_FLOAT32, dstb->ptr, fmt, outer, H, W, 1, 0, nullptr), "ttnn.to_layout");
        }
        check(ttb_stream_synchronize(nullptr), "ttnn.to_layout");
        out = Tensor(dstb, Shape(shape.dims(), shape.padded()), d.dtype(), layout);
    } else if (layout == Layout::TILE) {
        if (shape.rank() < 2) throw_error("ttnn.to_layout: TILE_LAYOUT needs at least 2 dimensions");
        Shape padded = Shape(shape.dims()).tile_padded();
        if (shape.has_padding() && !(shape.padded() == padded.padded()))
            throw_error("ttnn.to_layout: unsupported padding on a row-major tensor");
        shape.as_outer_hw(outer, H, W, false);
        auto dstb = allocate_device_buffer(dev, physical_bytes(padded, d.dtype(), layout));
        if (shape.has_padding()) {
            shape.as_outer_hw(outer, H, W, true);  // already stored padded
        }
        check(ttb_tilize(d.data(), dstb->ptr, element_size(d.dtype()), outer, H, W, nullptr), "ttnn.to_layout");
        out = Tensor(dstb, padded, d.dtype(), layout);
    } else {
        // TILE -> ROW_MAJOR keeps the padded extents as the stored shape, like the reference's host untilize.
        shape.as_outer_hw(outer, H, W, true);
        auto dstb = allocate_device_buffer(dev, d.buffer_bytes());
        check(ttb_untilize(d.data(), dstb->ptr, element_size(d.dtype()), outer, H, W, nullptr), "ttnn.to_layout");
        out = Tensor(dstb, shape, d.dtype(), layout);
    }
    return on_device ? out : to_host_storage(out);
}

// to_layout(tensor, TILE_LAYOUT, dtype=...) on a device tensor: the reference's ttl.tensor.tilize(output_dtype=dtype)
// (ttnn/ttnn/operations/core.py:677-711). Row-major (or already tiled) bfloat16 / float32 data becomes a tiled tensor of
// `dtype`; for block-float targets the device packer applies exactly the host packer's arithmetic (one pass), with the zero
// padding to tile multiples fused. Block-float sources unpack to bfloat16 / float32 tiles.
Tensor to_tile_layout_as(const Tensor &t, DataType dtype) {
    if (t.storage_type() != StorageType::DEVICE) throw_error(std::string("Unsupported datatype conversion to ") + to_string(dtype));
    if (!t.is_allocated()) throw_error("ttnn.to_layout: the tensor has been deallocated");
    if (dtype == t.dtype()) return to_layout(t, Layout::TILE);
    Device *dev = t.device();
    dev->make_current();
    const Shape &shape = t.shape();
    if (shape.rank() < 2) throw_error("ttnn.to_layout: TILE_LAYOUT needs at least 2 dimensions");
    int64_t outer, H, W;
    if (is_block_float(dtype)) {
        if (t.dtype() != DataType::BFLOAT16 && t.dtype() != DataType::FLOAT32)
            throw_error(std::string("Unsupported datatype conversion to ") + to_string(dtype));
        const bool row_major = t.layout() == Layout::ROW_MAJOR;
        if (row_major && shape.has_padding()) throw_error("ttnn.to_layout: unsupported padding on a row-major tensor");
        Shape out_shape = row_major ? Shape(shape.dims()).tile_padded() : shape;
        shape.as_outer_hw(outer, H, W, /*padded=*/!row_major);
        auto dstb = allocate_device_buffer(dev, physical_bytes(out_shape, dtype, Layout::TILE));
        check(ttb_pack_bfp(t.data(), ttb_dtype(t.dtype()), dstb->ptr, ttb_dtype(dtype), outer, H, W, row_major ? 1 : 0, /*two_pass=*/0, nullptr),
              "ttnn.to_layout");
        check(ttb_stream_synchronize(nullptr), "ttnn.to_layout");   // block-float tensors are complete when they are returned
        return Tensor(dstb, out_shape, dtype, Layout::TILE);
    }
    if (is_block_float(t.dtype()) && (dtype == DataType::BFLOAT16 || dtype == DataType::FLOAT32)) {
        if (t.layout() != Layout::TILE) throw_error(std::string("Unsupported datatype conversion to ") + to_string(dtype));
        shape.as_outer_hw(outer, H, W, /*padded=*/true);
        auto dstb = allocate_device_buffer(dev, physical_bytes(shape, dtype, Layout::TILE));
        check(ttb_unpack_bfp(t.data(), ttb_dtype(t.dtype()), dstb->ptr, ttb_dtype(dtype), outer, H, W, /*dst_row_major=*/0, 0, nullptr), "ttnn.to_layout");
        return Tensor(dstb, shape, dtype, Layout::TILE);
    }
    throw_error(std::string("Unsupported datatype conversion to ") + to_string(dtype));
    return t;
}

Tensor to_device(const Tensor &t, Device *device) {
    if (!device) throw_error("ttnn.to_device: device must not be None");
    if (t.storage_type() == StorageType::DEVICE) {
        if (t.device() != device) throw_error("ttnn.to_device: the tensor already lives on another device");
        return t;
    }
    if (!t.is_allocated()) throw_error("ttnn.to_device: the tensor has been deallocated");
    return to_device_storage(t, device);
}

Tensor from_device(const Tensor &t) {
    if (t.storage_type() != StorageType::DEVICE) return t;
    if (!t.is_allocated()) throw_error("ttnn.from_device: the tensor has been deallocated");
    return to_host_storage(t);
}

Tensor wrap_device_memory(uint64_t ptr, const Shape &shape, DataType dtype, Layout layout, Device *device) {
    if (!device) throw_error("ttnn: wrap_device_memory needs a device");
    return Tensor(borrow_device_buffer(device, reinterpret_cast<void *>(ptr), physical_bytes(shape, dtype, layout)), shape, dtype, layout);
}

// ---- pad / unpad -----------------------------------------------------------------------------------------
namespace {

std::vector<int64_t> as4(const std::vector<int64_t> &v, int64_t fill, const char *what) {
    if (v.empty() || v.size() > 4) throw_error(std::string(what) + ": shapes have one to four dimensions");
    std::vector<int64_t> out(4 - v.size(), fill);
    out.insert(out.end(), v.begin(), v.end());
    return out;
}

uint32_t pad_bits(DataType d, float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    switch (d) {
        case DataType::FLOAT32: return u;
        case DataType::BFLOAT16: return u >> 16;                       // the reference's bfloat16(float) truncates (bfloat16.hpp:27-38)
        case DataType::UINT32: return (uint32_t)v;
        case DataType::UINT16: return (uint32_t)(uint16_t)v;
        default: return u;
    }
}

// Runs `body(src_dev, dst_dev)` on fp32 views of a block-float tensor in stored order and packs the result again.
template <typename F>
Tensor through_fp32(const Tensor &d, Device *dev, int64_t out_volume, const Shape &out_shape, F body, const char *op) {
    const int fmt = static_cast<int>(d.dtype());
    const int64_t in_volume = d.shape().padded_volume();
    if (in_volume % 1024 || out_volume % 1024) throw_error(std::string(op) + ": block-float tensors hold whole groups of 1024 values");
    auto in32 = allocate_device_buffer(dev, in_volume * 4);
    auto out32 = allocate_device_buffer(dev, out_volume * 4);
    auto dstb = allocate_device_buffer(dev, physical_bytes(out_shape, d.dtype(), d.layout()));
    check(ttb_unpack_bfp(d.data(), fmt, in32->ptr, TTB_FLOAT32, 1, 32, in_volume / 32, 0, 0, nullptr), op);
    body(in32->ptr, out32->ptr);
    check(ttb_pack_bfp(out32->ptr, TTB_FLOAT32, dstb->ptr, fmt, 1, 32, out_volume / 32, 0, 0, nullptr), op);
    check(ttb_stream_synchronize(nullptr), op);
    return Tensor(dstb, out_shape, d.dtype(), d.layout());
}

}  // namespace

Tensor pad(const Tensor &t, const std::vector<int64_t> &output_shape, const std::vector<int64_t> &input_start, float pad_value) {
    const char *op = "Tensor.pad";
    if (!t.is_allocated()) throw_error(std::string(op) + ": the tensor has been deallocated");
    if (t.layout() != Layout::ROW_MAJOR) throw_error(std::string(op) + ": Tensor layout must be ROW_MAJOR for padding");
    const std::vector<int64_t> in = as4(t.shape().padded(), 1, op), out = as4(output_shape, 1, op), st = as4(input_start, 0, op);
    for (int i = 0; i < 4; ++i)
        if (st[i] < 0 || in[i] + st[i] > out[i]) throw_error(std::string(op) + ": the input tensor does not fit the output shape at the given start");
    const bool on_device = t.storage_type() == StorageType::DEVICE;
    Tensor d = on_device ? t : to_device_storage(t, current_or_default_device());
    Device *dev = d.device();
    dev->make_current();
    const Shape out_shape(std::vector<int64_t>(out.end() - (std::ptrdiff_t)std::max(output_shape.size(), t.shape().rank()), out.end()));
    const int64_t out_volume = out[0] * out[1] * out[2] * out[3];
    Tensor result;
    if (is_block_float(d.dtype())) {
        uint32_t bits;
        std::memcpy(&bits, &pad_value, 4);
        result = through_fp32(d, dev, out_volume, out_shape, [&](void *src, void *dst) {
            check(ttb_pad(src, dst, 4, in.data(), out.data(), st.data(), bits, nullptr), op);
        }, op);
    } else {
        auto dstb = allocate_device_buffer(dev, out_volume * element_size(d.dtype()));
        check(ttb_pad(d.data(), dstb->ptr, element_size(d.dtype()), in.data(), out.data(), st.data(), pad_bits(d.dtype(), pad_value), nullptr), op);
        result = Tensor(dstb, out_shape, d.dtype(), Layout::ROW_MAJOR);
    }
    return on_device ? result : to_host_storage(result);
}

Tensor unpad(const Tensor &t, const std::vector<int64_t> &start, const std::vector<int64_t> &end) {
    const char *op = "Tensor.unpad";
    if (!t.is_allocated()) throw_error(std::string(op) + ": the tensor has been deallocated");
    if (t.layout() != Layout::ROW_MAJOR) throw_error(std::string(op) + ": Tensor layout must be ROW_MAJOR for unpadding");
    const std::vector<int64_t> in = as4(t.shape().padded(), 1, op), st = as4(start, 0, op), en = as4(end, 0, op);
    std::vector<int64_t> out(4);
    for (int i = 0; i < 4; ++i) {
        if (st[i] < 0 || en[i] < st[i] || en[i] >= in[i]) throw_error(std::string(op) + ": the slice must lie inside the tensor, start <= end");
        out[i] = en[i] - st[i] + 1;
    }
    const bool on_device = t.storage_type() == StorageType::DEVICE;
    Tensor d = on_device ? t : to_device_storage(t, current_or_default_device());
    Device *dev = d.device();
    dev->make_current();
    const Shape out_shape(std::vector<int64_t>(out.end() - (std::ptrdiff_t)std::max(start.size(), t.shape().rank()), out.end()));
    const int64_t out_volume = out[0] * out[1] * out[2] * out[3];
    Tensor result;
    if (is_block_float(d.dtype())) {
        result = through_fp32(d, dev, out_volume, out_shape, [&](void *src, void *dst) {
            check(ttb_unpad(src, dst, 4, in.data(), st.data(), en.data(), nullptr), op);
        }, op);
    } else {
        auto dstb = allocate_device_buffer(dev, out_volume * element_size(d.dtype()));
        check(ttb_unpad(d.data(), dstb->ptr, element_size(d.dtype()), in.data(), st.data(), en.data(), nullptr), op);
        result = Tensor(dstb, out_shape, d.dtype(), Layout::ROW_MAJOR);
    }
    return on_device ? result : to_host_storage(result);
}

Tensor pad_to_tile(const Tensor &t, float pad_value) {
    const Shape &s = t.shape();
    if (s.rank() < 2) throw_error("Tensor.pad_to_tile: at least two dimensions are needed");
    std::vector<int64_t> out = s.padded();
    out[out.size() - 2] = (out[out.size() - 2] + 31) / 32 * 32;
    out[out.size() - 1] = (out[out.size() - 1] + 31) / 32 * 32;
    Tensor p = pad(t, out, std::vector<int64_t>(out.size(), 0), pad_value);
    // the result remembers the extents it was padded from, like Shape(..., Padding) in the reference
    Tensor r = p;
    return r.reshape(Shape(s.padded(), out));
}

Tensor unpad_from_tile(const Tensor &t, const std::vector<int64_t> &output_shape) {
    const std::vector<int64_t> &in = t.shape().padded();
    if (output_shape.size() != in.size() || in.size() < 2) throw_error("Tensor.unpad_from_tile: the output shape must have the tensor's rank");
    const size_t r = in.size();
    for (size_t i = 0; i + 2 < r; ++i)
        if (in[i] != output_shape[i]) throw_error("Tensor.unpad_from_tile: Input shape must match output shape apart from last 2 dims");
    if (in[r - 2] % 32 || in[r - 1] % 32) throw_error("Tensor.unpad_from_tile: Last 2 dims of input shape must be multiples of 32");
    if (!(in[r - 2] - 32 < output_shape[r - 2] && output_shape[r - 2] <= in[r - 2] && in[r - 1] - 32 < output_shape[r - 1] && output_shape[r - 1] <= in[r - 1]))
        throw_error("Tensor.unpad_from_tile: Last 2 dims of output must be within range to have been padded to input");
    std::vector<int64_t> end(output_shape);
    for (auto &v : end) v -= 1;
    return unpad(t, std::vector<int64_t>(r, 0), end);
}

Tensor multiply(const Tensor &a, const Tensor &b) {
    const char *op = "ttnn.mul";
    if (a.storage_type() != StorageType::DEVICE || b.storage_type() != StorageType::DEVICE) throw_error(std::string(op) + ": both tensors must be on device");
    if (!a.is_allocated() || !b.is_allocated()) throw_error(std::string(op) + ": tensors must be allocated");
    if (a.device() != b.device()) throw_error(std::string(op) + ": operands must be on the same device");
    if (a.dtype() != DataType::BFLOAT16 || b.dtype() != DataType::BFLOAT16) throw_error(std::string(op) + ": both tensors must be bfloat16");
    if (!(a.shape() == b.shape()) || a.layout() != b.layout()) throw_error(std::string(op) + ": both tensors must have the same shape and layout");
    Device *dev = a.device();
    dev->make_current();
    auto outb = allocate_device_buffer(dev, a.buffer_bytes());
    check(ttb_mul_bf16(a.data(), b.data(), outb->ptr, a.shape().padded_volume(), nullptr), op);
    return Tensor(outb, a.shape(), a.dtype(), a.layout());
}

// ---- matmul / linear ----------------------------------------------------------------------------------
namespace {

void validate_operand(const char *op, const char *name, const Tensor &t, bool weight) {
    // validate_input_tensor with the matmul TensorSchema: rank 2..4, {bf16, bfp8, bfp4}, TILE layout, on device
    // (ttnn/cpp/ttnn/operations/matmul.hpp:39-42, ttnn/cpp/ttnn/validation.hpp:18-75).
    const std::string who = std::string(op) + ": Tensor " + name;
    if (t.shape().rank() < 2 || t.shape().rank() > 4)
        throw_error(who + " must be of rank 2, 3 or 4, but got " + std::to_string(t.shape().rank()));
    const DataType d = t.dtype();
    if (d != DataType::BFLOAT16 && d != DataType::BFLOAT8_B && d != DataType::BFLOAT4_B)
        throw_error(who + " must be of type bfloat16, bfloat8_b or bfloat4_b, but got " + to_string(d));
    if (t.layout() != Layout::TILE) throw_error(who + " must be of layout Layout.TILE, but got " + to_string(t.layout()));
    if (t.storage_type() != StorageType::DEVICE) throw_error(who + " must be on device!");
    if (!t.is_allocated()) throw_error(who + " must be allocated!");
    (void)weight;
}

int activation_code(const std::optional<std::string> &act) {
    if (!act) return TTB_ACT_NONE;
    if (*act == "relu") return TTB_ACT_RELU;
    if (*act == "gelu") return TTB_ACT_GELU;
    if (*act == "silu") return TTB_ACT_SILU;
    throw_error("ttnn.linear: Unsupported activation function " + *act);
}

Tensor run_matmul(const char *op, const Tensor &a_in, const Tensor &b, const std::optional<Tensor> &bias, std::optional<DataType> dtype,
                  const std::optional<std::string> &activation) {
    validate_operand(op, "input_tensor_a", a_in, false);
    validate_operand(op, "input_tensor_b", b, true);
    if (a_in.device() != b.device()) throw_error(std::string(op) + ": operands must be on the same device");
    const Shape &sa = a_in.shape(), &sb = b.shape();
    const int64_t width_a = sa[-1], height_b = sb[-2];
    if (width_a != height_b) throw_error(std::string(op) + ": The width of the first tensor must be equal to the height of the second tensor");
    const auto &pa = sa.padded(), &pb = sb.padded();
    const int64_t Mp = pa[pa.size() - 2], Kp = pa[pa.size() - 1], Np = pb[pb.size() - 1];
    if (pb[pb.size() - 2] != Kp) throw_error(std::string(op) + ": padded inner dimensions disagree");
    int64_t batch = 1, batch_b = 1;
    for (size_t i = 0; i + 2 < pa.size(); ++i) batch *= pa[i];
    for (size_t i = 0; i + 2 < pb.size(); ++i) batch_b *= pb[i];
    // The second operand is either one [K, N] matrix shared by every batch entry of the first, or carries the first
    // operand's batch (tt::tt_metal::bmm, tt_eager/tt_dnn/op_library/bmm/bmm_op.cpp:518-626).
    const bool batched_b = batch_b != 1;
    if (batched_b) {
        if (batch_b != batch) throw_error(std::string(op) + ": a batched second operand must have the batch dimensions of the first");
        if (bias) throw_error(std::string(op) + ": bias is not supported with a batched second operand");
        if (activation) throw_error(std::string(op) + ": a fused activation is not supported with a batched second operand");
    }
    // output dtype = dtype or the first operand's (bmm_op.cpp:1148-1161); block-float outputs are the host packer's
    // arithmetic applied to the fp32 result
    const DataType out_dtype = dtype.value_or(a_in.dtype());
    if (out_dtype != DataType::BFLOAT16 && out_dtype != DataType::FLOAT32 && !is_block_float(out_dtype))
        throw_error(std::string(op) + ": output dtype must be bfloat16, float32, bfloat8_b or bfloat4_b");
    Device *dev = a_in.device();
    dev->make_current();
    // block-float activations (bmm_op.cpp:839 admits them) are expanded to bfloat16 first: exact
    Tensor a = a_in;
    if (is_block_float(a_in.dtype())) {
        int64_t outer, H, W;
        sa.as_outer_hw(outer, H, W, /*padded=*/true);
        auto ab = allocate_device_buffer(dev, sa.padded_volume() * 2);
        check(ttb_unpack_bfp(a_in.data(), ttb_dtype(a_in.dtype()), ab->ptr, TTB_BFLOAT16, outer, H, W, /*dst_row_major=*/0, 0, nullptr), op);
        a = Tensor(ab, sa, DataType::BFLOAT16, Layout::TILE);
    }
    const void *bias_ptr = nullptr;
    if (bias) {
        // TILE layout, [.., N] padded to one tile row: [1,1,32,N] in the reference (bmm_op.cpp:859-863).
        const Tensor &bt = *bias;
        if (bt.layout() != Layout::TILE || bt.dtype() != DataType::BFLOAT16 || bt.storage_type() != StorageType::DEVICE)
            throw_error(std::string(op) + ": bias must be a bfloat16 TILE_LAYOUT tensor on device");
        const auto &pbias = bt.shape().padded();
        if (bt.shape()[-1] != sb[-1] || pbias[pbias.size() - 1] != Np || bt.shape().padded_volume() != 32 * Np)
            throw_error(std::string(op) + ": bias must have shape [1, N] padded to one tile row");
        bias_ptr = bt.data();
    }
    // output shape: a's dims with the last replaced by N; padding follows a except the last dim follows b
    std::vector<int64_t> od = sa.dims(), op_ = sa.padded();
    od.back() = sb[-1];
    op_.back() = Np;
    Shape out_shape(od, op_);
    const DataType kernel_out = is_block_float(out_dtype) ? DataType::FLOAT32 : out_dtype;
    auto outb = allocate_device_buffer(dev, physical_bytes(out_shape, kernel_out, Layout::TILE));
    if (batched_b) {
        check(ttb_bmm(a.data(), ttb_dtype(a.dtype()), b.data(), ttb_dtype(b.dtype()), outb->ptr, ttb_dtype(kernel_out), batch, Mp, Kp, Np, nullptr), op);
    } else {
        const int64_t ws_bytes = ttb_matmul_workspace_bytes(ttb_dtype(b.dtype()), batch, Mp, Kp, Np, 0);
        void *ws = ws_bytes > 0 ? dev->workspace(ws_bytes) : nullptr;
        // Every producer of a block-float tensor on this API (from_torch, to_layout, load_tensor, to_device) has finished on the
        // device before it returns, so a block-float weight is complete long before this launch is enqueued and the kernel may
        // stream it while the previous kernel drains.
        const int flags = TTB_MM_WORKSPACE_ZEROED | (is_block_float(b.dtype()) ? TTB_MM_WEIGHTS_RESIDENT : 0);
        check(ttb_matmul(a.data(), ttb_dtype(a.dtype()), b.data(), ttb_dtype(b.dtype()), bias_ptr, outb->ptr, ttb_dtype(kernel_out), batch, Mp,
                         Kp, Np, activation_code(activation), flags, ws, ws_bytes, nullptr),
              op);
    }
    if (!is_block_float(out_dtype)) return Tensor(outb, out_shape, out_dtype, Layout::TILE);
    // pack the fp32 tiles (already in tile order) with the device packer: bit-exact with packing the fp32 result on the host
    auto packed = allocate_device_buffer(dev, physical_bytes(out_shape, out_dtype, Layout::TILE));
    int64_t outer, H, W;
    out_shape.as_outer_hw(outer, H, W, /*padded=*/true);
    check(ttb_pack_bfp(outb->ptr, TTB_FLOAT32, packed->ptr, ttb_dtype(out_dtype), outer, H, W, /*src_row_major=*/0, /*two_pass=*/0, nullptr), op);
    check(ttb_stream_synchronize(nullptr), op);   // block-float tensors are complete when they are returned
    return Tensor(packed, out_shape, out_dtype, Layout::TILE);
}

}  // namespace

Tensor matmul(const Tensor &a, const Tensor &b, std::optional<DataType> dtype, const std::optional<MatmulProgramConfig> &program_config) {
    std::optional<std::string> act;
    if (program_config && program_config->fused_activation) act = program_config->fused_activation;
    return run_matmul("ttnn.matmul", a, b, std::nullopt, dtype, act);
}

Tensor linear(const Tensor &a, const Tensor &b, const std::optional<Tensor> &bias, std::optional<DataType> dtype,
              const std::optional<std::string> &activation, const std::optional<MatmulProgramConfig> &program_config) {
    std::optional<std::string> act = activation;
    if (!act && program_config && program_config->fused_activation) act = program_config->fused_activation;
    return run_matmul("ttnn.linear", a, b, bias, dtype, act);
}

}  // namespace ttnn_b200
