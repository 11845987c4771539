// Tensor-parallel pieces of the ttnn surface on one-process-per-GPU meshes: the communicator, ttnn.all_gather, and the
// linears whose epilogue is the all-gather (several weights of one activation in one launch).
//
// Mirrors ttnn.all_gather (ttnn/ttnn/operations/ccl.py:26-39) on top of the AllGather op
// (tt_eager/tt_dnn/op_library/all_gather/all_gather_op.cpp:18-104); the fused linears stand in for the sequences
// matmul -> all_gather -> matmul of the tensor-parallel decoders (models/demos/llama2_70b/tt/llama_mlp_optimized.py:165-228).
#pragma once
#include <optional>
#include <string>
#include <vector>

#include "tensor.hpp"

namespace ttnn_b200 {

// NCCL communicator of a mesh, behind the C ABI (ttb_comm_*). The unique id is made on one rank and handed to the others
// by the caller (any transport); construction waits at most `timeout_ms` for every rank to join.
class Comm {
   public:
    static std::string make_unique_id();
    Comm(int ranks, int rank, const std::string &unique_id, int64_t timeout_ms);
    ~Comm();
    Comm(const Comm &) = delete;
    Comm &operator=(const Comm &) = delete;
    int ranks() const { return ranks_; }
    int rank() const { return rank_; }
    void *handle() const { return handle_; }
    void check(int64_t timeout_ms) const;   // throws on an asynchronous error or when enqueued work does not start in time
    void abort();                           // tears down without waiting for the peers; the object is unusable afterwards

   private:
    void *handle_ = nullptr;
    int ranks_ = 0, rank_ = 0;
};

// How the rank-major concatenation an all-gather leaves relates to the gathered tensor (pure shape logic).
struct GatherPlan {
    bool interleave = false;      // rows x [ranks x row_bytes] has to be re-ordered from [ranks][rows][row_bytes]
    int64_t rows = 0, row_bytes = 0;
    Shape out_shape;
};
GatherPlan plan_all_gather(const Shape &shape, DataType dtype, Layout layout, int dim, int ranks);

// out = concat over ranks of `t` along `dim`, on every rank; dtype and layout preserved.
Tensor all_gather(const Tensor &t, int dim, Comm &comm);

// A ring of gather points in peer-mapped memory (see ttb_matmul_peer in ttb.h). Every rank holds an arena of the same
// layout - per point a 256-byte counter block (arrived at +0, expected at +128), then one buffer per point - and knows the
// address of every rank's arena as mapped into this process. The arenas are allocated, exported and mapped by the caller.
class GatherRing {
   public:
    GatherRing(int rank, std::vector<uint64_t> arena_bases, int slots, int64_t counter_bytes, int64_t slot_bytes);
    int ranks() const { return (int)bases_.size(); }
    int slots() const { return slots_; }
    int64_t slot_bytes() const { return slot_bytes_; }
    int take(int64_t nbytes);                 // next point of the ring (all ranks call this in the same order)
    const ttb_peer_gather *gather(int slot) const { return &gathers_.at(slot); }
    const ttb_peer_wait_t *wait(int slot) const { return &waits_.at(slot); }
    void *out_ptr(int slot) const;
    void stream_wait(int slot) const;         // holds the stream until the point is complete on this rank

   private:
    int rank_, slots_, next_ = 0;
    int64_t counter_bytes_, slot_bytes_;
    std::vector<uint64_t> bases_;
    std::vector<ttb_peer_gather> gathers_;
    std::vector<ttb_peer_wait_t> waits_;
};

// [linear(x, w, bias=b, activation=act) for (w, b) in zip(weights, biases)] as one launch (ttb_matmul_multi). With
// `gather_first` the first result is gathered over the ranks by the kernel's epilogue into the ring's next point, whose index
// is returned in *gather_slot; `wait_slot` >= 0 names the point of `ring` the activation came from (the kernel waits for it
// itself).
// `gated`: exactly two weights of one shape; the single result is activation(x w0 + b0) * (x w1 + b1), the gate multiply of
// the gated MLP formed inside the launch (row counts that are multiples of 64 run the two linears and the product as
// separate launches).
std::vector<Tensor> linear_multi(const Tensor &x, const std::vector<Tensor> &weights, const std::vector<std::optional<Tensor>> &biases,
                                 const std::optional<std::string> &activation, GatherRing *ring, bool gather_first, int wait_slot,
                                 int *gather_slot, bool gated = false);

}  // namespace ttnn_b200
