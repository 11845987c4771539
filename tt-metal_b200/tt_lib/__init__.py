"""`tt_lib` spellings of the block-float weight path, for call sites written against the older API.

The 70B decoder of the reference calls `tt_lib.operations.primary.matmul_1d`, `tt_lib.tensor.all_gather` and
`tt_lib.tensor.mul` (models/demos/llama2_70b/tt/llama_mlp_optimized.py:165-228); its weights are `tt_lib.tensor.Tensor`s made
by `torch2tt_tensor` (models/utility_functions.py). Everything here forwards to the `ttnn` package next to this one
(tt_eager/tt_lib/csrc/operations/primary/module.hpp:53-403, tt_eager/tt_lib/csrc/tt_lib_bindings_tensor_pytensor.cpp:581-1399);
memory-config and program-config arguments are accepted and have no effect on a GPU with one kind of device memory.
One process drives one GPU: the per-device lists the reference passes around have one entry here."""
from . import tensor, operations, device  # noqa: F401
