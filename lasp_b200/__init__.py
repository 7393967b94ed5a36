"""lasp_b200: LASP's linear-attention operators on hand-written sm_100a CUDA.

Same names and signatures as the reference's ``lasp`` package.
"""
from .lasp_cache import lasp_cache, lasp_cache_  # noqa: F401
from .lasp_fuse import lasp_fuse, lasp_fuse_  # noqa: F401
from .lasp_fuse_parallel import lasp_fuse_parallel, lasp_fuse_parallel_  # noqa: F401
from .lasp_naive import lasp_naive, lasp_naive_  # noqa: F401
from .lightning_attention import lightning_attn, lightning_attn_  # noqa: F401
from .utils import *  # noqa: F401,F403
from ._core import lightning_attn_fused  # noqa: F401
from ._core import sequence_parallel_fused as lasp_fuse_parallel_fused  # noqa: F401


def check_faults(clear: bool = True) -> None:
    """Synchronise the current CUDA stream and raise ``lasp_b200.engine.KernelFault`` if a kernel of the
    library has given up on one of its bounded waits (for instance a sequence-parallel peer that never
    delivered its state) since the last check.  The operators make this check themselves, one step late
    and without stalling the stream; call it where a synchronisation is acceptable (end of a step)."""
    from . import engine
    engine.check_faults(clear)

__version__ = "0.1.0"
