"""Names of ShardedLayers.py mapped to this package."""
from ..models.sharded_layers import (ShardedAttention, ShardedFFLayer, ShardedLayerNorm,  # noqa: F401
                                     TransformerBlock)
