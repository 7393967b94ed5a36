"""Import alias: ``from lasp import lightning_attn, lasp_fuse, ...`` resolves to
lasp_b200, so callers written against the reference package need no edits."""
from lasp_b200 import *  # noqa: F401,F403
from lasp_b200 import (  # noqa: F401
    lasp_cache, lasp_cache_, lasp_fuse, lasp_fuse_, lasp_fuse_parallel, lasp_fuse_parallel_,
    lasp_naive, lasp_naive_, lightning_attn, lightning_attn_,
)
