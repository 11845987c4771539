// Host-side data model of the ttnn surface: enums, Shape with tile padding, Device, Tensor with owned-host or
// device storage, and the per-op configuration structs the reference API accepts.
//
// Mirrors tt_eager/tensor/{tensor,types}.hpp (Tensor, Storage, Shape/Padding, DataType, Layout, StorageType),
// ttnn/cpp/ttnn/types.hpp (ttnn::Shape, CoreGrid) and the program / compute-kernel configuration structs of
// tt_eager/tt_dnn/op_library/bmm/bmm_op.hpp:176-281 and compute_kernel_config.hpp:10-44. Everything that
// touches the GPU goes through the C ABI in ttb.h; this layer has no CUDA or torch types.
#pragma once
#include <cstdint>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "ttb.h"

namespace ttnn_b200 {

// Numeric values follow tt::tt_metal::DataType / Layout (tt_eager/tensor/types.hpp:24-34).
enum class DataType : int { BFLOAT16 = 0, FLOAT32 = 1, UINT32 = 2, BFLOAT8_B = 3, BFLOAT4_B = 4, UINT16 = 6, INVALID = 7 };
enum class Layout : int { ROW_MAJOR = 0, TILE = 1, INVALID = 2 };
enum class StorageType : int { OWNED = 0, DEVICE = 1, BORROWED = 2, MULTI_DEVICE = 3, MULTI_DEVICE_HOST = 4 };
enum class BufferType : int { DRAM = 0, L1 = 1 };
enum class TensorMemoryLayout : int { INTERLEAVED = 0, SINGLE_BANK = 1, HEIGHT_SHARDED = 2, WIDTH_SHARDED = 3, BLOCK_SHARDED = 4 };
enum class MathFidelity : int { LoFi = 0, HiFi2 = 2, HiFi3 = 3, HiFi4 = 4 };

constexpr int TILE_SIZE = 32;

[[noreturn]] void throw_error(const std::string &msg);
// Turns a non-zero libttb status into a std::runtime_error carrying ttb_last_error().
void check(int32_t rc, const char *what);

inline bool is_block_float(DataType d) { return d == DataType::BFLOAT8_B || d == DataType::BFLOAT4_B; }
int element_size(DataType d);  // bytes per element for plain types; throws for block-float
const char *to_string(DataType d);
const char *to_string(Layout l);

// A ranked shape that remembers both the logical extents and the extents after padding the last two
// dimensions to tiles, like ttnn::Shape (ttnn/cpp/ttnn/types.hpp).
class Shape {
   public:
    Shape() = default;
    explicit Shape(std::vector<int64_t> dims) : dims_(dims), padded_(std::move(dims)) {}
    Shape(std::vector<int64_t> dims, std::vector<int64_t> padded);
    size_t rank() const { return dims_.size(); }
    const std::vector<int64_t> &dims() const { return dims_; }
    const std::vector<int64_t> &padded() const { return padded_; }
    int64_t operator[](int64_t i) const;
    int64_t volume() const;
    int64_t padded_volume() const;
    Shape with_tile_padding() const { return Shape(padded_, padded_); }
    // Same logical dims, last two padded dims rounded up to 32.
    Shape tile_padded() const;
    bool has_padding() const { return dims_ != padded_; }
    bool operator==(const Shape &o) const { return dims_ == o.dims_ && padded_ == o.padded_; }
    std::string repr() const;
    // [outer, H, W] views used by the kernels (rank >= 2 for tiled data; rank-1 counts as H = 1).
    void as_outer_hw(int64_t &outer, int64_t &H, int64_t &W, bool padded) const;

   private:
    std::vector<int64_t> dims_, padded_;
};

struct MemoryConfig {
    TensorMemoryLayout memory_layout = TensorMemoryLayout::INTERLEAVED;
    BufferType buffer_type = BufferType::DRAM;
    bool operator==(const MemoryConfig &o) const { return memory_layout == o.memory_layout && buffer_type == o.buffer_type; }
};

struct CoreGrid {
    int x = 1, y = 1;
    int num_cores() const { return x * y; }
};

// Accepted for source compatibility; the GPU kernels always accumulate in fp32 at full operand precision.
struct ComputeKernelConfig {
    MathFidelity math_fidelity = MathFidelity::HiFi4;
    bool math_approx_mode = true;
    bool fp32_dest_acc_en = true;
    bool packer_l1_acc = false;
};

// The reference's four matmul program configs carry Tensix tiling parameters. They are kept as hints: the
// only field that changes what is computed is the fused activation.
struct MatmulProgramConfig {
    std::string kind = "default";  // default | multi_core_reuse | mcast_1d | mcast_2d
    int compute_grid_x = 0, compute_grid_y = 0;
    int in0_block_w = 0, out_subblock_h = 0, out_subblock_w = 0, per_core_M = 0, per_core_N = 0;
    bool fuse_batch = true, mcast_in0 = true, transpose_mcast = false;
    std::optional<std::string> fused_activation;
};

// One CUDA device. Opened through open_device(); tensors keep their device alive through the pool.
class Device {
   public:
    explicit Device(int id) : id_(id) {}
    int id() const { return id_; }
    void make_current() const;
    void synchronize();
    // Reads (and clears) the device status word after the default stream has drained. A bounded device-side wait that ran
    // out (a peer that never stored its slice, a lost barrier arrival) left counters and partial sums behind in the
    // scratch: it is cleared here, so that later matmuls start from zeros, and the error is raised.
    void check_device_status(const char *what);
    // Grow-only scratch used by matmul's split-K reduction, zeroed when (re)allocated.
    void *workspace(int64_t bytes);
    ~Device();

   private:
    int id_;
    void *workspace_ = nullptr;
    int64_t workspace_bytes_ = 0;
};

Device *open_device(int device_id);
void close_device(Device *device);
int device_count();

struct HostBuffer {
    std::vector<uint8_t> bytes;
};
struct DeviceBuffer {
    void *ptr = nullptr;
    int64_t bytes = 0;
    Device *device = nullptr;
    bool owned = true;
    std::shared_ptr<DeviceBuffer> parent;   // set for a view into another buffer, which it keeps alive
    ~DeviceBuffer();
};

class Tensor {
   public:
    Tensor() = default;
    Tensor(std::shared_ptr<HostBuffer> h, Shape s, DataType d, Layout l) : host_(std::move(h)), shape_(std::move(s)), dtype_(d), layout_(l) {}
    Tensor(std::shared_ptr<DeviceBuffer> b, Shape s, DataType d, Layout l) : dev_(std::move(b)), shape_(std::move(s)), dtype_(d), layout_(l) {}

    const Shape &shape() const { return shape_; }
    DataType dtype() const { return dtype_; }
    Layout layout() const { return layout_; }
    StorageType storage_type() const { return dev_ ? StorageType::DEVICE : StorageType::OWNED; }
    bool is_allocated() const { return (dev_ && dev_->ptr) || (host_ && !host_->bytes.empty()); }
    Device *device() const { return dev_ ? dev_->device : nullptr; }
    MemoryConfig memory_config() const { return MemoryConfig{}; }
    int64_t buffer_bytes() const;             // size of the physical buffer for shape/dtype/layout
    const void *data() const;                 // host or device pointer
    void *data();
    uint64_t buffer_address() const { return reinterpret_cast<uint64_t>(data()); }
    void deallocate(bool force = false);
    Tensor reshape(const Shape &s) const;     // metadata only; volumes must agree
    std::string repr() const;

    const std::shared_ptr<HostBuffer> &host_buffer() const { return host_; }
    const std::shared_ptr<DeviceBuffer> &device_buffer() const { return dev_; }

   private:
    std::shared_ptr<HostBuffer> host_;
    std::shared_ptr<DeviceBuffer> dev_;
    Shape shape_;
    DataType dtype_ = DataType::INVALID;
    Layout layout_ = Layout::INVALID;
};

int64_t physical_bytes(const Shape &shape, DataType dtype, Layout layout);
std::shared_ptr<DeviceBuffer> allocate_device_buffer(Device *device, int64_t bytes);
// Returns every cached free block to the CUDA allocator.
void release_cached_blocks();
// Wraps device memory owned by someone else (e.g. a collective's output buffer); never freed here.
std::shared_ptr<DeviceBuffer> borrow_device_buffer(Device *device, void *ptr, int64_t bytes);
// A part of `parent` (several results of one launch share one allocation); keeps the parent alive.
std::shared_ptr<DeviceBuffer> view_device_buffer(const std::shared_ptr<DeviceBuffer> &parent, void *ptr, int64_t bytes);

}  // namespace ttnn_b200
