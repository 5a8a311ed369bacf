"""Names of Autotuner.py mapped to this package."""
from ..autotuner import (Autotuner, ComputeGraph, FFLayerModel, base_overheads, build_transformerBlock,  # noqa: F401
                         bws, latencies, possibleK)
