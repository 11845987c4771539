#include "ccl.hpp"

#include <cstring>

#include "ops.hpp"

namespace ttnn_b200 {

// ---- communicator ------------------------------------------------------------------------------------------
std::string Comm::make_unique_id() {
    std::string id(TTB_COMM_ID_BYTES, '\0');
    ttnn_b200::check(ttb_comm_unique_id(id.data()), "ttnn: communicator id");
    return id;
}

Comm::Comm(int ranks, int rank, const std::string &unique_id, int64_t timeout_ms) : ranks_(ranks), rank_(rank) {
    if ((int)unique_id.size() != TTB_COMM_ID_BYTES) throw_error("ttnn: a communicator id has " + std::to_string(TTB_COMM_ID_BYTES) + " bytes");
    ttnn_b200::check(ttb_comm_init(&handle_, ranks, rank, unique_id.data(), timeout_ms), "ttnn.open_device_mesh");
}

Comm::~Comm() {
    if (handle_) ttb_comm_destroy(handle_);
}

void Comm::check(int64_t timeout_ms) const {
    if (!handle_) throw_error("ttnn: the communicator was aborted");
    ttnn_b200::check(ttb_comm_check(handle_, timeout_ms), "ttnn: communicator");
}

void Comm::abort() {
    if (handle_) ttb_comm_abort(handle_);
    handle_ = nullptr;
}

// ---- all_gather --------------------------------------------------------------------------------------------
GatherPlan plan_all_gather(const Shape &shape, DataType dtype, Layout layout, int dim, int ranks) {
    const int rank = (int)shape.rank();
    const int d = dim < 0 ? dim + rank : dim;
    if (d < 0 || d >= rank) throw_error("ttnn.all_gather: dim " + std::to_string(dim) + " is out of range for a rank-" + std::to_string(rank) + " tensor");
    const bool tiled = layout == Layout::TILE;
    if (tiled && rank < 2) throw_error("ttnn.all_gather: tiled tensors have at least two dimensions");
    const auto &dims = shape.dims(), &padded = shape.padded();
    int64_t outer_rows = 1;
    for (int i = 0; i < rank - (tiled ? 2 : 1); ++i) outer_rows *= padded[i];
    GatherPlan g;
    if (tiled) {
        g.rows = outer_rows * (padded[rank - 2] / 32);
        const int64_t tile_bytes = dtype == DataType::BFLOAT8_B ? 1088 : dtype == DataType::BFLOAT4_B ? 576 : 1024 * element_size(dtype);
        g.row_bytes = (padded[rank - 1] / 32) * tile_bytes;   // one tile row of this rank's shard
    } else {
        g.rows = outer_rows;
        g.row_bytes = padded[rank - 1] * element_size(dtype);
    }
    bool leading_ones = true;
    for (int i = 0; i < d; ++i) leading_ones = leading_ones && padded[i] == 1;
    if (d == rank - 1) {
        g.interleave = g.rows > 1;
    } else if (tiled && d == rank - 2 && outer_rows == 1) {
        if (dims[d] != padded[d]) throw_error("ttnn.all_gather: cannot concatenate padded tile rows");
        g.interleave = false;   // shards are whole contiguous blocks: the rank-major concatenation is the result
    } else if (leading_ones) {
        g.interleave = false;
    } else {
        throw_error("ttnn.all_gather: gathering along dim " + std::to_string(dim) + " of a rank-" + std::to_string(rank) + " tensor is not supported");
    }
    std::vector<int64_t> od = dims, op = padded;
    od[d] *= ranks;
    op[d] *= ranks;
    g.out_shape = Shape(od, op);
    return g;
}

Tensor all_gather(const Tensor &t, int dim, Comm &comm) {
    if (t.storage_type() != StorageType::DEVICE) throw_error("ttnn.all_gather: the tensor must be on device");
    if (!t.is_allocated()) throw_error("ttnn.all_gather: the tensor has been deallocated");
    const int n = comm.ranks();
    const GatherPlan g = plan_all_gather(t.shape(), t.dtype(), t.layout(), dim, n);
    Device *dev = t.device();
    dev->make_current();
    const int64_t bytes = t.buffer_bytes();
    auto staged = allocate_device_buffer(dev, bytes * n);
    check(ttb_all_gather(comm.handle(), t.data(), staged->ptr, bytes, nullptr), "ttnn.all_gather");
    if (!g.interleave) return Tensor(staged, g.out_shape, t.dtype(), t.layout());
    auto out = allocate_device_buffer(dev, bytes * n);
    check(ttb_gather_interleave(staged->ptr, out->ptr, 1, n, g.rows, g.row_bytes, nullptr), "ttnn.all_gather");
    return Tensor(out, g.out_shape, t.dtype(), t.layout());
}

// ---- ring of gather points -----------------------------------------------------------------------------------
GatherRing::GatherRing(int rank, std::vector<uint64_t> arena_bases, int slots, int64_t counter_bytes, int64_t slot_bytes)
    : rank_(rank), slots_(slots), counter_bytes_(counter_bytes), slot_bytes_(slot_bytes), bases_(std::move(arena_bases)) {
    const int world = (int)bases_.size();
    if (world < 2 || world > TTB_MAX_RANKS) throw_error("the gather epilogue serves 2.." + std::to_string(TTB_MAX_RANKS) + " ranks");
    if (rank < 0 || rank >= world) throw_error("ttnn: rank outside the mesh");
    if (slots < 2) throw_error("a gather ring needs at least two points: consecutive gathers must not share a buffer");
    if (counter_bytes < (int64_t)slots * 256) throw_error("ttnn: the counter area of a gather ring holds 256 bytes per point");
    gathers_.resize(slots);
    waits_.resize(slots);
    for (int s = 0; s < slots; ++s) {
        ttb_peer_gather &g = gathers_[s];
        std::memset(&g, 0, sizeof(g));
        g.ranks = world;
        g.rank = rank;
        for (int r = 0; r < world; ++r) {
            g.out[r] = reinterpret_cast<void *>(bases_[r] + counter_bytes + (uint64_t)s * slot_bytes);
            g.arrived[r] = reinterpret_cast<uint32_t *>(bases_[r] + (uint64_t)s * 256);
        }
        g.expected = reinterpret_cast<uint32_t *>(bases_[rank] + (uint64_t)s * 256 + 128);
        waits_[s].arrived = reinterpret_cast<const uint32_t *>(bases_[rank] + (uint64_t)s * 256);
        waits_[s].expected = reinterpret_cast<const uint32_t *>(bases_[rank] + (uint64_t)s * 256 + 128);
    }
}

int GatherRing::take(int64_t nbytes) {
    if (nbytes > slot_bytes_)
        throw_error("gathered tensor of " + std::to_string(nbytes) + " bytes exceeds the ring's " + std::to_string(slot_bytes_) + "-byte buffers");
    const int s = next_;
    next_ = (s + 1) % slots_;
    return s;
}

void *GatherRing::out_ptr(int slot) const { return reinterpret_cast<void *>(bases_[rank_] + counter_bytes_ + (uint64_t)slot * slot_bytes_); }

void GatherRing::stream_wait(int slot) const { check(ttb_peer_wait(&waits_.at(slot), nullptr), "ttnn: waiting for a gathered tensor"); }

// ---- several linears of one activation in one launch ---------------------------------------------------------
namespace {
int activation_code_of(const std::optional<std::string> &act) {
    if (!act) return TTB_ACT_NONE;
    if (*act == "relu") return TTB_ACT_RELU;
    if (*act == "gelu") return TTB_ACT_GELU;
    if (*act == "silu") return TTB_ACT_SILU;
    throw_error("ttnn.linear: Unsupported activation function " + *act);
}
}  // namespace

std::vector<Tensor> linear_multi(const Tensor &x, const std::vector<Tensor> &weights, const std::vector<std::optional<Tensor>> &biases,
                                 const std::optional<std::string> &activation, GatherRing *ring, bool gather_first, int wait_slot,
                                 int *gather_slot, bool gated) {
    const char *op = gated ? "ttnn.linear_gated" : "ttnn.linear_multi";
    if (gated && weights.size() != 2) throw_error(std::string(op) + ": takes the two weights of the gate and up projections");
    const int n = (int)weights.size();
    if (n < 1 || n > TTB_MAX_GROUP) throw_error(std::string(op) + ": between one and four weights per launch");
    if (!biases.empty() && (int)biases.size() != n) throw_error(std::string(op) + ": one bias (or None) per weight");
    if (x.dtype() != DataType::BFLOAT16 || x.layout() != Layout::TILE || x.storage_type() != StorageType::DEVICE || !x.is_allocated())
        throw_error(std::string(op) + ": the activation must be a bfloat16 TILE_LAYOUT tensor on device");
    const auto &xp = x.shape().padded();
    int64_t rows = 1;
    for (size_t i = 0; i + 1 < xp.size(); ++i) rows *= xp[i];
    const int64_t K = xp.back();
    const DataType fmt = weights[0].dtype();
    const void *w_ptr[TTB_MAX_GROUP] = {}, *b_ptr[TTB_MAX_GROUP] = {};
    void *o_ptr[TTB_MAX_GROUP] = {};
    int64_t N[TTB_MAX_GROUP] = {}, Nl[TTB_MAX_GROUP] = {};
    bool any_bias = false;
    for (int j = 0; j < n; ++j) {
        const Tensor &w = weights[j];
        if (!is_block_float(w.dtype()) || w.dtype() != fmt || w.layout() != Layout::TILE)
            throw_error(std::string(op) + ": weights must be TILE_LAYOUT tensors of one block-float dtype");
        if (w.storage_type() != StorageType::DEVICE || !w.is_allocated()) throw_error(std::string(op) + ": weights must be on device");
        if (w.device() != x.device()) throw_error(std::string(op) + ": operands must be on the same device");
        const auto &wp = w.shape().padded();
        if (wp.size() < 2 || wp[wp.size() - 2] != K) throw_error(std::string(op) + ": The width of the first tensor must be equal to the height of the second tensor");
        for (size_t i = 0; i + 2 < wp.size(); ++i)
            if (wp[i] != 1) throw_error(std::string(op) + ": The width of the first tensor must be equal to the height of the second tensor");
        w_ptr[j] = w.data();
        N[j] = wp.back();
        Nl[j] = w.shape()[-1];
        if (!biases.empty() && biases[j]) {
            const Tensor &bt = *biases[j];
            if (bt.layout() != Layout::TILE || bt.dtype() != DataType::BFLOAT16 || bt.storage_type() != StorageType::DEVICE || bt.shape().padded_volume() != 32 * N[j])
                throw_error(std::string(op) + ": bias must be a bfloat16 TILE_LAYOUT tensor [1, N] on device");
            b_ptr[j] = bt.data();
            any_bias = true;
        }
    }
    Device *dev = x.device();
    dev->make_current();
    if (gated && N[0] != N[1]) throw_error(std::string(op) + ": both weights must have the same shape");
    if (gated && rows % 64 == 0) {
        // the fused form serves 32-row blocks; otherwise two linears and their product (same values, three launches)
        if (gather_first || wait_slot >= 0) throw_error(std::string(op) + ": the gathered form needs a row count of 32, 96, 160 or 224");
        Tensor g = linear(x, weights[0], biases.empty() ? std::nullopt : biases[0], std::nullopt, activation, std::nullopt);
        Tensor u = linear(x, weights[1], biases.empty() ? std::nullopt : biases[1], std::nullopt, std::nullopt, std::nullopt);
        if (gather_slot) *gather_slot = -1;
        return {multiply(g, u)};
    }
    if ((gather_first || wait_slot >= 0) && !ring) throw_error(std::string(op) + ": gathering or waiting needs the mesh's ring of gather points");
    const int G = gather_first ? ring->ranks() : 1;
    int slot = -1;
    if (gather_first) slot = ring->take((int64_t)G * rows * N[0] * 2);
    // one allocation for all local outputs of the launch
    const int first_local = gather_first ? 1 : 0;
    const int n_out = gated ? 1 : n;
    int64_t total = 0;
    for (int j = first_local; j < n_out; ++j) total += rows * N[j];
    std::shared_ptr<DeviceBuffer> block = total ? allocate_device_buffer(dev, total * 2) : nullptr;
    int64_t off = 0;
    for (int j = first_local; j < n_out; ++j) {
        o_ptr[j] = static_cast<uint8_t *>(block->ptr) + off * 2;
        off += rows * N[j];
    }
    const int64_t need = gated ? ttb_matmul_gated_workspace_bytes(static_cast<int>(fmt), 1, rows, K, N[0])
                               : ttb_matmul_multi_workspace_bytes(static_cast<int>(fmt), 1, rows, K, n, N);
    void *ws = need > 0 ? dev->workspace(need) : nullptr;
    check(ttb_matmul_multi(x.data(), TTB_BFLOAT16, n, w_ptr, static_cast<int>(fmt), any_bias ? b_ptr : nullptr, o_ptr, TTB_BFLOAT16, 1, rows, K, N,
                           activation_code_of(activation), TTB_MM_WORKSPACE_ZEROED | TTB_MM_WEIGHTS_RESIDENT | (gated ? TTB_MM_GATED : 0), ws, need,
                           gather_first ? ring->gather(slot) : nullptr, wait_slot >= 0 ? ring->wait(wait_slot) : nullptr, nullptr),
          op);
    if (gather_slot) *gather_slot = slot;
    std::vector<int64_t> lead(x.shape().dims().begin(), x.shape().dims().end() - 1), lead_p(xp.begin(), xp.end() - 1);
    std::vector<Tensor> results;
    for (int j = 0; j < n_out; ++j) {
        std::vector<int64_t> d = lead, dp = lead_p;
        if (j < first_local) {
            d.push_back(G * Nl[j]);
            dp.push_back(G * N[j]);
            results.emplace_back(borrow_device_buffer(dev, ring->out_ptr(slot), (int64_t)G * rows * N[j] * 2), Shape(d, dp), DataType::BFLOAT16, Layout::TILE);
        } else {
            d.push_back(Nl[j]);
            dp.push_back(N[j]);
            results.emplace_back(view_device_buffer(block, o_ptr[j], rows * N[j] * 2), Shape(d, dp), DataType::BFLOAT16, Layout::TILE);
        }
    }
    return results;
}

}  // namespace ttnn_b200
