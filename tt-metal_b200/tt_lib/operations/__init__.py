"""tt_lib.operations: the `primary` namespace holds the program-config driven matmuls."""
from . import primary  # noqa: F401
