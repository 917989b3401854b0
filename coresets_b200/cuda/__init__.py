from . import multi
from .accrete import accrete
from .fps import fps
from .._native import ensure_compiled


def warmup_fast_fps() -> None:
    """Load (and if necessary compile) the native library ahead of timing-sensitive code.
    Counterpart of the reference's ``warmup_fast_fps`` (src/coresets/cuda/extension.py:84-85)."""
    ensure_compiled()


__all__ = ["accrete", "fps", "warmup_fast_fps", "multi"]
