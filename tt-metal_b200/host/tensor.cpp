#include "tensor.hpp"

#include <map>
#include <mutex>
#include <sstream>

namespace ttnn_b200 {

void throw_error(const std::string &msg) { throw std::runtime_error(msg); }

void check(int32_t rc, const char *what) {
    if (rc != TTB_OK) throw_error(std::string(what) + ": " + ttb_last_error());
}

int element_size(DataType d) {
    switch (d) {
        case DataType::BFLOAT16:
        case DataType::UINT16: return 2;
        case DataType::FLOAT32:
        case DataType::UINT32: return 4;
        default: throw_error("element_size: block-float and invalid data types have no per-element size");
    }
}

const char *to_string(DataType d) {
    switch (d) {
        case DataType::BFLOAT16: return "DataType.BFLOAT16";
        case DataType::FLOAT32: return "DataType.FLOAT32";
        case DataType::UINT32: return "DataType.UINT32";
        case DataType::BFLOAT8_B: return "DataType.BFLOAT8_B";
        case DataType::BFLOAT4_B: return "DataType.BFLOAT4_B";
        case DataType::UINT16: return "DataType.UINT16";
        default: return "DataType.INVALID";
    }
}
const char *to_string(Layout l) { return l == Layout::TILE ? "Layout.TILE" : l == Layout::ROW_MAJOR ? "Layout.ROW_MAJOR" : "Layout.INVALID"; }

Shape::Shape(std::vector<int64_t> dims, std::vector<int64_t> padded) : dims_(std::move(dims)), padded_(std::move(padded)) {
    if (dims_.size() != padded_.size()) throw_error("ttnn.Shape: shape and padded shape must have the same rank");
    for (size_t i = 0; i < dims_.size(); ++i)
        if (padded_[i] < dims_[i]) throw_error("ttnn.Shape: padded shape must not be smaller than the shape");
}
int64_t Shape::operator[](int64_t i) const {
    const int64_t r = (int64_t)dims_.size();
    if (i < 0) i += r;
    if (i < 0 || i >= r) throw_error("ttnn.Shape: index out of range");
    return dims_[i];
}
int64_t Shape::volume() const {
    int64_t v = 1;
    for (auto d : dims_) v *= d;
    return v;
}
int64_t Shape::padded_volume() const {
    int64_t v = 1;
    for (auto d : padded_) v *= d;
    return v;
}
Shape Shape::tile_padded() const {
    std::vector<int64_t> p = dims_;
    const size_t r = p.size();
    if (r >= 1) p[r - 1] = (p[r - 1] + 31) / 32 * 32;
    if (r >= 2) p[r - 2] = (p[r - 2] + 31) / 32 * 32;
    return Shape(dims_, p);
}
std::string Shape::repr() const {
    std::ostringstream os;
    os << "ttnn.Shape([";
    for (size_t i = 0; i < dims_.size(); ++i) {
        if (i) os << ", ";
        os << dims_[i];
        if (padded_[i] != dims_[i]) os << "[" << padded_[i] << "]";
    }
    os << "])";
    return os.str();
}
void Shape::as_outer_hw(int64_t &outer, int64_t &H, int64_t &W, bool padded) const {
    const auto &d = padded ? padded_ : dims_;
    const size_t r = d.size();
    if (r == 0) throw_error("ttnn.Shape: rank-0 tensors are not supported");
    W = d[r - 1];
    H = r >= 2 ? d[r - 2] : 1;
    // the outer extent is never padded: tile padding only applies to the last two dimensions
    outer = 1;
    for (size_t i = 0; i + 2 < r; ++i) outer *= padded_[i];
}

// ---- devices ---------------------------------------------------------------------------------------
namespace {
std::mutex g_pool_mutex;
std::map<int, std::unique_ptr<Device>> g_pool;
}  // namespace

void Device::make_current() const { check(ttb_set_device(id_), "ttnn.open_device"); }
void Device::synchronize() {
    make_current();
    check(ttb_device_synchronize(), "ttnn.synchronize_device");
    check_device_status("ttnn.synchronize_device");
}
void Device::check_device_status(const char *what) {
    const int32_t rc = ttb_check_status(nullptr);
    if (rc == TTB_OK) return;
    const std::string message = ttb_last_error();
    if (rc == TTB_E_TIMEOUT && workspace_) {
        ttb_memset(workspace_, 0, (size_t)workspace_bytes_, nullptr);
        ttb_stream_synchronize(nullptr);
    }
    throw_error(std::string(what) + ": " + message +
                (rc == TTB_E_TIMEOUT ? " (the matmul scratch was cleared; results since the last check are invalid, and a mesh whose gather "
                                       "timed out must be reopened)"
                                     : ""));
}
void *Device::workspace(int64_t bytes) {
    if (bytes <= workspace_bytes_) return workspace_;
    make_current();
    if (workspace_) {
        check(ttb_device_synchronize(), "ttnn: workspace growth");
        check(ttb_free(workspace_), "ttnn: workspace growth");
        workspace_ = nullptr;
        workspace_bytes_ = 0;
    }
    const int64_t want = std::max<int64_t>(bytes, 8 << 20);
    check(ttb_malloc(&workspace_, (size_t)want), "ttnn: workspace allocation");
    check(ttb_memset(workspace_, 0, (size_t)want, nullptr), "ttnn: workspace allocation");
    workspace_bytes_ = want;
    return workspace_;
}
Device::~Device() {
    if (workspace_) ttb_free(workspace_);
}

int device_count() {
    int32_t n = 0;
    check(ttb_device_count(&n), "ttnn.get_num_devices");
    return n;
}

// One Device object per id, kept in a process-wide pool like ttnn/cpp/ttnn/device.cpp:18-26.
Device *open_device(int device_id) {
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    auto it = g_pool.find(device_id);
    if (it == g_pool.end()) {
        const int n = device_count();
        if (device_id < 0 || device_id >= n)
            throw_error("ttnn.open_device: device " + std::to_string(device_id) + " does not exist (" + std::to_string(n) + " CUDA devices visible)");
        it = g_pool.emplace(device_id, std::make_unique<Device>(device_id)).first;
    }
    it->second->make_current();
    return it->second.get();
}
void close_device(Device *device) {
    if (!device) return;
    device->synchronize();  // tensors may outlive the call; the pool entry stays valid until process exit
}

// ---- buffers and tensors ----------------------------------------------------------------------------
// Freed device blocks are kept in per-device size classes and handed out again without calling the CUDA
// allocator (whose free synchronises the device). All work runs in stream order on one stream, so a block may
// be reused as soon as its tensor is gone. Stands in for the reference's device allocator (tt_metal/impl/allocator).
namespace {
std::mutex g_block_mutex;
std::map<std::pair<int, int64_t>, std::vector<void *>> g_free_blocks;

int64_t size_class(int64_t bytes) {
    if (bytes <= 512) return 512;
    if (bytes < (1 << 20)) return (bytes + 4095) / 4096 * 4096;
    return (bytes + (2 << 20) - 1) / (2 << 20) * (2 << 20);
}
}  // namespace

DeviceBuffer::~DeviceBuffer() {
    if (ptr && owned) {
        std::lock_guard<std::mutex> lock(g_block_mutex);
        g_free_blocks[{device ? device->id() : 0, size_class(bytes)}].push_back(ptr);
    }
}

void release_cached_blocks() {
    std::lock_guard<std::mutex> lock(g_block_mutex);
    for (auto &kv : g_free_blocks) {
        ttb_set_device(kv.first.first);
        for (void *p : kv.second) ttb_free(p);
    }
    g_free_blocks.clear();
}

std::shared_ptr<DeviceBuffer> allocate_device_buffer(Device *device, int64_t bytes) {
    if (!device) throw_error("ttnn: a device is required to allocate device memory");
    auto b = std::make_shared<DeviceBuffer>();
    b->device = device;
    b->bytes = bytes;
    const int64_t cls = size_class(bytes);
    {
        std::lock_guard<std::mutex> lock(g_block_mutex);
        auto it = g_free_blocks.find({device->id(), cls});
        if (it != g_free_blocks.end() && !it->second.empty()) {
            b->ptr = it->second.back();
            it->second.pop_back();
            return b;
        }
    }
    device->make_current();
    int32_t rc = ttb_malloc(&b->ptr, (size_t)cls);
    if (rc != TTB_OK) {
        release_cached_blocks();  // give cached blocks back and try once more
        device->make_current();
        check(ttb_malloc(&b->ptr, (size_t)cls), "ttnn: device allocation");
    }
    return b;
}

std::shared_ptr<DeviceBuffer> borrow_device_buffer(Device *device, void *ptr, int64_t bytes) {
    auto b = std::make_shared<DeviceBuffer>();
    b->device = device;
    b->ptr = ptr;
    b->bytes = bytes;
    b->owned = false;
    return b;
}

std::shared_ptr<DeviceBuffer> view_device_buffer(const std::shared_ptr<DeviceBuffer> &parent, void *ptr, int64_t bytes) {
    auto b = std::make_shared<DeviceBuffer>();
    b->device = parent->device;
    b->ptr = ptr;
    b->bytes = bytes;
    b->owned = false;
    b->parent = parent;
    return b;
}

int64_t physical_bytes(const Shape &shape, DataType dtype, Layout layout) {
    if (is_block_float(dtype)) {
        if (shape.padded_volume() % 1024) throw_error("ttnn: block-float tensors must hold whole 32x32 tiles");
        return shape.padded_volume() / 1024 * (dtype == DataType::BFLOAT8_B ? 1088 : 576);
    }
    (void)layout;
    return shape.padded_volume() * element_size(dtype);
}

int64_t Tensor::buffer_bytes() const { return physical_bytes(shape_, dtype_, layout_); }
const void *Tensor::data() const {
    if (dev_) return dev_->ptr;
    if (host_) return host_->bytes.data();
    return nullptr;
}
void *Tensor::data() { return const_cast<void *>(static_cast<const Tensor *>(this)->data()); }

void Tensor::deallocate(bool force) {
    // Like the reference (tt_eager/tensor/tensor.cpp:65-117): release now if this is the last reference or force.
    if (dev_ && (force || dev_.use_count() == 1) && dev_->ptr && dev_->owned) {
        std::lock_guard<std::mutex> lock(g_block_mutex);
        g_free_blocks[{dev_->device ? dev_->device->id() : 0, size_class(dev_->bytes)}].push_back(dev_->ptr);
        dev_->ptr = nullptr;
    }
    if (host_ && (force || host_.use_count() == 1)) {
        host_->bytes.clear();
        host_->bytes.shrink_to_fit();
    }
}

Tensor Tensor::reshape(const Shape &s) const {
    if (s.volume() != shape_.volume() && s.padded_volume() != shape_.padded_volume())
        throw_error("ttnn.reshape: cannot reshape " + shape_.repr() + " into " + s.repr());
    if (s.padded_volume() != shape_.padded_volume())
        throw_error("ttnn.reshape: the padded volume must stay the same (" + shape_.repr() + " -> " + s.repr() + ")");
    if (layout_ == Layout::TILE) {
        const auto &a = shape_.padded(), &b = s.padded();
        const size_t ra = a.size(), rb = b.size();
        const bool same_tiles = ra >= 2 && rb >= 2 && a[ra - 1] == b[rb - 1] && a[ra - 2] == b[rb - 2];
        if (!same_tiles && !(ra >= 2 && rb >= 2 && b[rb - 1] % 32 == 0 && b[rb - 2] % 32 == 0 && a[ra - 1] == b[rb - 1]))
            throw_error("ttnn.reshape: a tiled tensor can only be reshaped without moving data across tile rows");
    }
    Tensor t = *this;
    t.shape_ = s;
    return t;
}

std::string Tensor::repr() const {
    std::ostringstream os;
    os << "ttnn.Tensor(shape=" << shape_.repr() << ", dtype=" << to_string(dtype_) << ", layout=" << to_string(layout_)
       << ", storage=" << (dev_ ? "DEVICE" : "OWNED") << ")";
    return os.str();
}

}  // namespace ttnn_b200
