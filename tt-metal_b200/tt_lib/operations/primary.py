"""tt_lib.operations.primary: matmul / matmul_1d and their program configs
(tt_eager/tt_lib/csrc/operations/primary/module.hpp:53-403, tt_eager/tt_dnn/op_library/bmm/bmm_op.hpp:284-346)."""
import ttnn
from ttnn.operations.matmul import (MatmulDefaultProgramConfig, MatmulMultiCoreReuseProgramConfig,  # noqa: F401
                                    MatmulMultiCoreReuseMultiCastProgramConfig, MatmulMultiCoreReuseMultiCast1DProgramConfig)


def _activation_of(program_config):
    act = getattr(program_config, "fused_activation", None) if program_config is not None else None
    return act


def matmul(input_tensor_a, input_tensor_b, bias=None, program_config=None, output_mem_config=None, output_dtype=None,
           compute_kernel_config=None, untilize_out=False):
    """tt::operations::primary::matmul: a @ b (+ bias), the activation a program config carries fused, output dtype
    `output_dtype` (default: the first operand's)."""
    if untilize_out:
        out = ttnn.linear(input_tensor_a, input_tensor_b, bias=bias, dtype=output_dtype, program_config=program_config)
        return ttnn.to_layout(out, ttnn.ROW_MAJOR_LAYOUT)
    return ttnn.linear(input_tensor_a, input_tensor_b, bias=bias, dtype=output_dtype, program_config=program_config)


def matmul_1d(input_tensor_a, input_tensor_b, bias=None, program_config=None, output_mem_config=None, output_dtype=None,
              compute_kernel_config=None, untilize_out=False):
    """tt::operations::primary::matmul_1d: the 1-D multicast form the decode matmuls use; same result as matmul."""
    return matmul(input_tensor_a, input_tensor_b, bias, program_config, output_mem_config, output_dtype, compute_kernel_config, untilize_out)
