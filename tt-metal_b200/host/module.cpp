// pybind11 surface `_ttnn`: the classes and functions the Python `ttnn` package re-exports.
// Stands in for PYBIND11_MODULE(_ttnn) (ttnn/cpp/pybind11/__init__.cpp:19-38) and the Tensor class of tt_lib
// (tt_eager/tt_lib/csrc/tt_lib_bindings_tensor_pytensor.cpp:581-1399), restricted to the block-float weight path.
// torch tensors never cross this boundary: the Python side passes data pointers and shapes.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "ccl.hpp"
#include "ops.hpp"

namespace py = pybind11;
using namespace ttnn_b200;

PYBIND11_MODULE(_ttnn, m) {
    m.doc() = "B200-native host layer of the ttnn block-float weight path";

    py::enum_<DataType>(m, "DataType")
        .value("BFLOAT16", DataType::BFLOAT16).value("FLOAT32", DataType::FLOAT32).value("UINT32", DataType::UINT32)
        .value("BFLOAT8_B", DataType::BFLOAT8_B).value("BFLOAT4_B", DataType::BFLOAT4_B).value("UINT16", DataType::UINT16);
    py::enum_<Layout>(m, "Layout").value("ROW_MAJOR", Layout::ROW_MAJOR).value("TILE", Layout::TILE);
    py::enum_<StorageType>(m, "StorageType")
        .value("OWNED", StorageType::OWNED).value("DEVICE", StorageType::DEVICE).value("BORROWED", StorageType::BORROWED)
        .value("MULTI_DEVICE", StorageType::MULTI_DEVICE).value("MULTI_DEVICE_HOST", StorageType::MULTI_DEVICE_HOST);
    py::enum_<BufferType>(m, "BufferType").value("DRAM", BufferType::DRAM).value("L1", BufferType::L1);
    py::enum_<TensorMemoryLayout>(m, "TensorMemoryLayout")
        .value("INTERLEAVED", TensorMemoryLayout::INTERLEAVED).value("SINGLE_BANK", TensorMemoryLayout::SINGLE_BANK)
        .value("HEIGHT_SHARDED", TensorMemoryLayout::HEIGHT_SHARDED).value("WIDTH_SHARDED", TensorMemoryLayout::WIDTH_SHARDED)
        .value("BLOCK_SHARDED", TensorMemoryLayout::BLOCK_SHARDED);
    py::enum_<MathFidelity>(m, "MathFidelity")
        .value("LoFi", MathFidelity::LoFi).value("HiFi2", MathFidelity::HiFi2).value("HiFi3", MathFidelity::HiFi3).value("HiFi4", MathFidelity::HiFi4);

    py::class_<Shape>(m, "Shape")
        .def(py::init<std::vector<int64_t>>(), py::arg("shape"))
        .def(py::init<std::vector<int64_t>, std::vector<int64_t>>(), py::arg("shape"), py::arg("padded_shape"))
        .def("__len__", &Shape::rank)
        .def("__getitem__", [](const Shape &s, int64_t i) {
            const int64_t r = (int64_t)s.rank();
            if (i < -r || i >= r) throw py::index_error();
            return s[i];
        })
        .def("__iter__", [](const Shape &s) { return py::iter(py::cast(s.dims())); })
        .def("__eq__", [](const Shape &a, const Shape &b) { return a == b; })
        .def("__eq__", [](const Shape &a, const std::vector<int64_t> &b) { return a.dims() == b; })
        .def("__repr__", &Shape::repr)
        .def("with_tile_padding", &Shape::with_tile_padding)
        .def_property_readonly("rank", &Shape::rank)
        .def_property_readonly("value", [](const Shape &s) { return s.dims(); })
        .def_property_readonly("padded", [](const Shape &s) { return s.padded(); });

    py::class_<MemoryConfig>(m, "MemoryConfig")
        .def(py::init([](TensorMemoryLayout l, BufferType b) { return MemoryConfig{l, b}; }),
             py::arg("memory_layout") = TensorMemoryLayout::INTERLEAVED, py::arg("buffer_type") = BufferType::DRAM)
        .def_readwrite("memory_layout", &MemoryConfig::memory_layout)
        .def_readwrite("buffer_type", &MemoryConfig::buffer_type)
        .def("__eq__", [](const MemoryConfig &a, const MemoryConfig &b) { return a == b; })
        .def("__repr__", [](const MemoryConfig &c) {
            return std::string("MemoryConfig(buffer_type=") + (c.buffer_type == BufferType::DRAM ? "DRAM" : "L1") + ")";
        });

    py::class_<CoreGrid>(m, "CoreGrid")
        .def(py::init([](int x, int y) { return CoreGrid{x, y}; }), py::kw_only(), py::arg("x"), py::arg("y"))
        .def_readonly("x", &CoreGrid::x).def_readonly("y", &CoreGrid::y)
        .def_property_readonly("num_cores", &CoreGrid::num_cores)
        .def("__repr__", [](const CoreGrid &g) { return "ttnn.CoreGrid(x=" + std::to_string(g.x) + ", y=" + std::to_string(g.y) + ")"; });

    py::class_<ComputeKernelConfig>(m, "ComputeKernelConfig")
        .def(py::init([](MathFidelity f, bool approx, bool fp32, bool l1acc) { return ComputeKernelConfig{f, approx, fp32, l1acc}; }),
             py::kw_only(), py::arg("math_fidelity") = MathFidelity::HiFi4, py::arg("math_approx_mode") = true,
             py::arg("fp32_dest_acc_en") = true, py::arg("packer_l1_acc") = false)
        .def_readwrite("math_fidelity", &ComputeKernelConfig::math_fidelity)
        .def_readwrite("math_approx_mode", &ComputeKernelConfig::math_approx_mode)
        .def_readwrite("fp32_dest_acc_en", &ComputeKernelConfig::fp32_dest_acc_en)
        .def_readwrite("packer_l1_acc", &ComputeKernelConfig::packer_l1_acc);

    py::class_<MatmulProgramConfig>(m, "MatmulProgramConfig")
        .def(py::init<>())
        .def_readwrite("kind", &MatmulProgramConfig::kind)
        .def_readwrite("compute_grid_x", &MatmulProgramConfig::compute_grid_x)
        .def_readwrite("compute_grid_y", &MatmulProgramConfig::compute_grid_y)
        .def_readwrite("in0_block_w", &MatmulProgramConfig::in0_block_w)
        .def_readwrite("out_subblock_h", &MatmulProgramConfig::out_subblock_h)
        .def_readwrite("out_subblock_w", &MatmulProgramConfig::out_subblock_w)
        .def_readwrite("per_core_M", &MatmulProgramConfig::per_core_M)
        .def_readwrite("per_core_N", &MatmulProgramConfig::per_core_N)
        .def_readwrite("fuse_batch", &MatmulProgramConfig::fuse_batch)
        .def_readwrite("mcast_in0", &MatmulProgramConfig::mcast_in0)
        .def_readwrite("transpose_mcast", &MatmulProgramConfig::transpose_mcast)
        .def_readwrite("fused_activation", &MatmulProgramConfig::fused_activation);

    py::class_<Device>(m, "Device")
        .def("id", &Device::id)
        .def("synchronize", &Device::synchronize)
        .def("__repr__", [](const Device &d) { return "ttnn.Device(id=" + std::to_string(d.id()) + ", NVIDIA sm_100a)"; });

    m.def("open_device", &open_device, py::arg("device_id"), py::return_value_policy::reference);
    m.def("close_device", &close_device, py::arg("device"));
    m.def("get_num_devices", &device_count);
    m.def("release_cached_blocks", &release_cached_blocks);

    py::class_<Tensor>(m, "Tensor")
        .def_property_readonly("shape", &Tensor::shape)
        .def_property_readonly("dtype", &Tensor::dtype)
        .def_property_readonly("layout", &Tensor::layout)
        .def("get_dtype", &Tensor::dtype)
        .def("get_layout", &Tensor::layout)
        .def("get_legacy_shape", &Tensor::shape)
        .def("device", &Tensor::device, py::return_value_policy::reference)
        .def("storage_type", &Tensor::storage_type)
        .def("is_allocated", &Tensor::is_allocated)
        .def("memory_config", &Tensor::memory_config)
        .def("deallocate", &Tensor::deallocate, py::arg("force") = false)
        .def("buffer_address", &Tensor::buffer_address)
        .def("buffer_bytes", &Tensor::buffer_bytes)
        .def("reshape", [](const Tensor &t, const Shape &s) { return t.reshape(s); })
        .def("reshape", [](const Tensor &t, const std::vector<int64_t> &dims) { return t.reshape(Shape(dims)); })
        .def("to", [](const Tensor &t, Layout l) { return to_layout(t, l); })
        .def("to", [](const Tensor &t, Device *d) { return to_device(t, d); }, py::keep_alive<0, 2>())
        .def("to", [](const Tensor &t, Device *d, const MemoryConfig &) { return to_device(t, d); }, py::keep_alive<0, 2>())
        .def("cpu", [](const Tensor &t) { return from_device(t); })
        .def("pad", [](const Tensor &t, const std::vector<int64_t> &output_tensor_shape, const std::vector<int64_t> &input_tensor_start,
                       float pad_value) { return pad(t, output_tensor_shape, input_tensor_start, pad_value); },
             py::arg("output_tensor_shape"), py::arg("input_tensor_start"), py::arg("pad_value"))
        .def("unpad", [](const Tensor &t, const std::vector<int64_t> &output_tensor_start, const std::vector<int64_t> &output_tensor_end) {
                 return unpad(t, output_tensor_start, output_tensor_end);
             }, py::arg("output_tensor_start"), py::arg("output_tensor_end"))
        .def("pad_to_tile", [](const Tensor &t, float pad_value) { return pad_to_tile(t, pad_value); }, py::arg("pad_value"))
        .def("unpad_from_tile", [](const Tensor &t, const std::vector<int64_t> &output_tensor_shape) { return unpad_from_tile(t, output_tensor_shape); },
             py::arg("output_tensor_shape"))
        .def("host_dtype", [](const Tensor &t) { return host_dtype_of(t); })
        .def("copy_to_host_pointer", [](const Tensor &t, uint64_t ptr) {
            py::gil_scoped_release release;
            to_host_buffer(t, reinterpret_cast<void *>(ptr));
        })
        .def("buffer", [](const Tensor &t) {
            // raw bytes of the physical buffer (packed tiles for block-float), copied to the host
            Tensor h = from_device(t);
            const auto &b = h.host_buffer()->bytes;
            return py::bytes(reinterpret_cast<const char *>(b.data()), b.size());
        })
        .def("__repr__", &Tensor::repr);

    m.def("from_host_pointer",
          [](uint64_t ptr, const std::vector<int64_t> &dims, DataType src_dtype, DataType dtype, Layout layout, Device *device) {
              py::gil_scoped_release release;
              return from_host_buffer(reinterpret_cast<const void *>(ptr), dims, src_dtype, dtype, layout, device);
          },
          py::arg("ptr"), py::arg("shape"), py::arg("src_dtype"), py::arg("dtype"), py::arg("layout"), py::arg("device").none(true),
          py::keep_alive<0, 6>());
    m.def("tensor_from_buffer",
          [](py::bytes data, const Shape &shape, DataType dtype, Layout layout) {
              // host tensor over a copy of the physical buffer bytes (the inverse of Tensor.buffer())
              std::string raw = data;
              if ((int64_t)raw.size() != physical_bytes(shape, dtype, layout))
                  throw std::runtime_error("ttnn.load_tensor: buffer size does not match shape, dtype and layout");
              auto h = std::make_shared<HostBuffer>();
              h->bytes.assign(raw.begin(), raw.end());
              return Tensor(h, shape, dtype, layout);
          },
          py::arg("data"), py::arg("shape"), py::arg("dtype"), py::arg("layout"));
    m.def("wrap_device_memory", &wrap_device_memory, py::arg("ptr"), py::arg("shape"), py::arg("dtype"), py::arg("layout"), py::arg("device"),
          py::keep_alive<0, 5>());
    m.def("to_layout", &to_layout);
    m.def("to_tile_layout_as", &to_tile_layout_as);
    m.def("to_device", &to_device, py::keep_alive<0, 2>());
    m.def("from_device", &from_device);

    // ---- tensor parallel: communicator, all_gather, gather ring, fused linears -------------------------------------
    py::class_<Comm>(m, "Comm")
        .def(py::init([](int ranks, int rank, py::bytes unique_id, int64_t timeout_ms) {
                 std::string id = unique_id;
                 py::gil_scoped_release release;
                 return std::make_unique<Comm>(ranks, rank, id, timeout_ms);
             }),
             py::arg("ranks"), py::arg("rank"), py::arg("unique_id"), py::arg("timeout_ms") = 120000)
        .def_static("make_unique_id", []() { return py::bytes(Comm::make_unique_id()); })
        .def_property_readonly("ranks", &Comm::ranks)
        .def_property_readonly("rank", &Comm::rank)
        .def("check", &Comm::check, py::arg("timeout_ms") = 10000)
        .def("abort", &Comm::abort);
    m.def("plan_all_gather",
          [](const Shape &shape, DataType dtype, Layout layout, int dim, int ranks) {
              const GatherPlan g = plan_all_gather(shape, dtype, layout, dim, ranks);
              return py::make_tuple(g.interleave, g.rows, g.row_bytes, g.out_shape);
          },
          py::arg("shape"), py::arg("dtype"), py::arg("layout"), py::arg("dim"), py::arg("ranks"));
    m.def("all_gather", &all_gather, py::arg("tensor"), py::arg("dim"), py::arg("comm"));
    py::class_<GatherRing>(m, "GatherRing")
        .def(py::init<int, std::vector<uint64_t>, int, int64_t, int64_t>(), py::arg("rank"), py::arg("arena_bases"), py::arg("slots"),
             py::arg("counter_bytes"), py::arg("slot_bytes"))
        .def_property_readonly("slots", &GatherRing::slots)
        .def_property_readonly("slot_bytes", &GatherRing::slot_bytes)
        .def("take", &GatherRing::take)
        .def("stream_wait", &GatherRing::stream_wait)
        .def("out_ptr", [](const GatherRing &r, int slot) { return reinterpret_cast<uint64_t>(r.out_ptr(slot)); });
    m.def("linear_multi",
          [](const Tensor &x, const std::vector<Tensor> &weights, const std::vector<std::optional<Tensor>> &biases,
             const std::optional<std::string> &activation, GatherRing *ring, bool gather_first, int wait_slot, bool gated) {
              int slot = -1;
              std::vector<Tensor> out = linear_multi(x, weights, biases, activation, ring, gather_first, wait_slot, &slot, gated);
              return py::make_tuple(out, slot);
          },
          py::arg("input_tensor"), py::arg("weights"), py::arg("biases"), py::arg("activation").none(true), py::arg("ring").none(true),
          py::arg("gather_first") = false, py::arg("wait_slot") = -1, py::arg("gated") = false);
    m.def("nvtx_push", [](const std::string &name) { ttb_nvtx_push(name.c_str()); });
    m.def("nvtx_pop", []() { ttb_nvtx_pop(); });
    m.def("mul", &multiply, py::arg("input_tensor_a"), py::arg("input_tensor_b"));
    m.def("matmul", &matmul, py::arg("input_tensor_a"), py::arg("input_tensor_b"), py::kw_only(), py::arg("dtype") = std::nullopt,
          py::arg("program_config") = std::nullopt);
    m.def("linear", &linear, py::arg("input_tensor_a"), py::arg("input_tensor_b"), py::kw_only(), py::arg("bias") = std::nullopt,
          py::arg("dtype") = std::nullopt, py::arg("activation") = std::nullopt, py::arg("program_config") = std::nullopt);
}
