from .fps_sharded import fps_sharded
from .layout import ShardLayout, compute_shard_layout

__all__ = ["fps_sharded", "compute_shard_layout", "ShardLayout"]
