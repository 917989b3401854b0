"""coresets_b200 -- B200-native farthest point sampling behind the API of the ``coresets``
reference package (src/coresets/__init__.py:1-20): ``fps_cuda``, ``fps_sharded``,
``compute_shard_layout``, ``accrete`` / ``accrete_sharded``, ``save_result`` / ``load_result``,
``warmup_fast_fps``, the plain-torch ``fps`` and the ``io`` module.  ``import coresets_b200 as coresets`` is the intended switch.
"""
from . import io
from ._version import __version__
from .cuda import accrete, warmup_fast_fps
from .cuda.fps import fps as fps_cuda
from .cuda.multi import accrete_sharded, compute_shard_layout, fps_sharded
from .io import load_result, save_result
from .pytorch import fps

__all__ = [
    "accrete",
    "accrete_sharded",
    "fps",
    "fps_cuda",
    "fps_sharded",
    "compute_shard_layout",
    "warmup_fast_fps",
    "save_result",
    "load_result",
    "io",
    "__version__",
]
