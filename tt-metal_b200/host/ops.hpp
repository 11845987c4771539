// Operations of the ttnn surface that sit on the block-float weight path: conversion at the torch boundary,
// layout / device moves, matmul and linear. Each mirrors the validation, shape rules and error behaviour of the
// reference routine named beside it and runs the work through the C ABI in ttb.h.
#pragma once
#include <optional>
#include <string>

#include "tensor.hpp"

namespace ttnn_b200 {

// torch -> Tensor. `src` is a contiguous host buffer of logical shape `dims` holding `src_dtype` elements
// (FLOAT32 or BFLOAT16 when the target is block-float; otherwise equal to `dtype`).
// convert_torch_tensor_to_tt_tensor (tt_eager/tt_lib/csrc/tt_lib_bindings_tensor_pytensor.cpp:26-167) followed by
// Tensor::to(Layout) (tt_eager/tensor/tensor_impl.cpp:179-250) and to(Device).
Tensor from_host_buffer(const void *src, const std::vector<int64_t> &dims, DataType src_dtype, DataType dtype, Layout layout,
                        Device *device);

// Tensor -> torch. Writes the logical (unpadded) tensor row-major into `dst`: fp32 for block-float tensors, the
// tensor's own element type otherwise. convert_tt_tensor_to_torch_tensor (pytensor.cpp:354-412).
void to_host_buffer(const Tensor &t, void *dst);
DataType host_dtype_of(const Tensor &t);

Tensor to_layout(const Tensor &t, Layout layout);   // Tensor::to(Layout), tensor_impl.hpp:158-171
Tensor to_tile_layout_as(const Tensor &t, DataType dtype);  // ttl.tensor.tilize(output_dtype=...), core.py:677-711
Tensor to_device(const Tensor &t, Device *device);  // Tensor::to(Device*), tensor_impl.hpp:246-269
Tensor from_device(const Tensor &t);                // Tensor::cpu(), tensor_impl.hpp:341-358
// Device tensor over memory owned by the caller (used for collective outputs).
Tensor wrap_device_memory(uint64_t ptr, const Shape &shape, DataType dtype, Layout layout, Device *device);

// Tensor::pad / unpad / pad_to_tile / unpad_from_tile (tt_eager/tensor/tensor.cpp:209-254, tensor_impl.hpp:508-677,
// tensor_impl.cpp:200-283): row-major tensors of up to four dimensions; block-float tensors go through fp32 as in the
// reference (unpack in stored order, pad, pack in stored order). `end` is inclusive.
Tensor pad(const Tensor &t, const std::vector<int64_t> &output_shape, const std::vector<int64_t> &input_start, float pad_value);
Tensor unpad(const Tensor &t, const std::vector<int64_t> &start, const std::vector<int64_t> &end);
Tensor pad_to_tile(const Tensor &t, float pad_value);
Tensor unpad_from_tile(const Tensor &t, const std::vector<int64_t> &output_shape);

// Elementwise product of two bfloat16 device tensors of one shape and layout (ttl.tensor.mul as the gated MLP uses it,
// models/demos/llama2_70b/tt/llama_mlp_optimized.py:191-197).
Tensor multiply(const Tensor &a, const Tensor &b);

// ttnn::operations::matmul::{matmul, linear} (ttnn/cpp/ttnn/operations/matmul.hpp:44-213) on top of
// tt::operations::primary::matmul (tt_eager/tt_dnn/op_library/bmm/bmm_op.cpp:828-1149).
Tensor matmul(const Tensor &a, const Tensor &b, std::optional<DataType> dtype, const std::optional<MatmulProgramConfig> &program_config);
Tensor linear(const Tensor &a, const Tensor &b, const std::optional<Tensor> &bias, std::optional<DataType> dtype,
              const std::optional<std::string> &activation, const std::optional<MatmulProgramConfig> &program_config);

}  // namespace ttnn_b200
