"""The reference's plain-torch backend (src/coresets/pytorch/): runs wherever ``X`` lives, one dense
matrix-vector product per pick.  Not the accelerated path -- ``fps_cuda`` / ``fps_sharded`` never
come through here -- but part of the package's public names (``coresets.fps``)."""
from .accrete import accrete
from .accrete_distributed import accrete as accrete_distributed
from .fps import fps, fps_update, voronoi_fps

__all__ = ["accrete", "accrete_distributed", "fps", "fps_update", "voronoi_fps"]
