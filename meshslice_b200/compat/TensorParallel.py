"""Names of TensorParallel.py mapped to this package."""
from ..parallel.mesh import DistMesh, EmuMesh, ShardedTensor  # noqa: F401
from ..parallel.tensor_parallel import (SPMD, allclose, createMultihostMatrix,  # noqa: F401
                                        cannon_ls as Cannon_LS, cannon_os as Cannon_OS, cannon_rs as Cannon_RS,
                                        collective_ls as Collective_LS, collective_os as Collective_OS,
                                        collective_rs as Collective_RS, meshslice_ls as MeshFlow_LS,
                                        meshslice_os as MeshFlow_OS, meshslice_rs as MeshFlow_RS,
                                        wang_ls as Wang_LS, wang_os as Wang_OS, wang_rs as Wang_RS)
