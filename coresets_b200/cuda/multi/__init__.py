from .fps_sharded import fps_sharded
from .layout import ShardLayout, compute_shard_layout
from .sharded import accrete_sharded, accrete_voronoi_multi_sharded
from .replicated import accrete_voronoi_multi

__all__ = ["fps_sharded", "compute_shard_layout", "ShardLayout", "accrete_sharded",
           "accrete_voronoi_multi", "accrete_voronoi_multi_sharded"]
