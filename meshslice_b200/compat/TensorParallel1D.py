"""Names of TensorParallel1D.py mapped to this package."""
from ..parallel.tensor_parallel_1d import (SPMDWang, createShardedMatrix, fsdp as FSDP,  # noqa: F401
                                           wang_1d_is as Wang_1DIS, wang_1d_os as Wang_1DOS,
                                           wang_dp_os as Wang_DPOS)
