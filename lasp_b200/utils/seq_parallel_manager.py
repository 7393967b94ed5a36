"""DP x SP process-group bookkeeping with the reference's function names.

Same mapping as lasp/utils/seq_parallel_manager.py:37-106 of the reference:
with ``world = dp * sp`` ranks, sequence-parallel groups are runs of ``sp``
consecutive global ranks (sp_rank = rank % sp) and data-parallel groups take
every ``sp``-th rank (dp_rank = rank // sp).  Example dp=2, sp=4 on 8 ranks:
SP groups (0,1,2,3)(4,5,6,7), DP groups (0,4)(1,5)(2,6)(3,7).

Differences from the reference, all on paths that raise there:
  * ``dp * sp`` must equal the world size (the reference only checks
    divisibility by sp, :46-51);
  * ``get_data_parallel_group(with_sequence_parallel=True)`` returns the group
    of all ranks (the reference leaves that global unassigned, :79-83);
  * ``get_data_parallel_src_rank()`` returns the first rank of the caller's
    data-parallel group (the reference never fills its rank list, :179-185).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist


class _Groups:
    """Everything initialize_lasp creates; one instance per process."""

    def __init__(self):
        self.clear()

    def clear(self):
        self.dp_group = None
        self.sp_group = None
        self.all_group = None
        self.dp_ranks = None
        self.sp_ranks = None
        self.sp_world_override = None
        self.sp_rank_override = None
        self.buffer = None


_G = _Groups()


def dp_sp_layout(world_size: int, data_parallel_size: int, sequence_parallel_size: int):
    """Pure function: (list of DP rank tuples, list of SP rank tuples)."""
    dp, sp = int(data_parallel_size), int(sequence_parallel_size)
    if dp < 1 or sp < 1:
        raise RuntimeError(f"data_parallel_size ({dp}) and sequence_parallel_size ({sp}) must be positive")
    if world_size % sp != 0:
        raise RuntimeError(f"world_size ({world_size}) is not divisible by sequence_parallel_size {sp})")
    if dp * sp != world_size:
        raise RuntimeError(f"data_parallel_size ({dp}) x sequence_parallel_size ({sp}) != world_size ({world_size})")
    dp_groups = [tuple(range(i, world_size, sp)) for i in range(sp)]
    sp_groups = [tuple(range(i * sp, (i + 1) * sp)) for i in range(dp)]
    return dp_groups, sp_groups


def initialize_lasp(data_parallel_size: int = 1, sequence_parallel_size: int = 1) -> None:
    """Create the DP, world and SP groups (collective: every rank must call it).

    Group creation order matches the reference (DP groups, the all-ranks group,
    SP groups) so that mixed deployments create communicators in step.
    """
    assert dist.is_initialized()
    assert _G.dp_group is None, "data parallel group is already initialized"
    assert _G.sp_group is None, "sequence parallel group is already initialized"
    world = dist.get_world_size()
    me = dist.get_rank()
    dp_groups, sp_groups = dp_sp_layout(world, data_parallel_size, sequence_parallel_size)
    for ranks in dp_groups:
        g = dist.new_group(list(ranks))
        if me in ranks:
            _G.dp_group, _G.dp_ranks = g, ranks
    _G.all_group = dist.new_group(list(range(world)))
    for ranks in sp_groups:
        g = dist.new_group(list(ranks))
        if me in ranks:
            _G.sp_group, _G.sp_ranks = g, ranks
    _set_global_memory_buffer()


def get_seq_parallel_send_rank() -> int:
    """Global rank of the previous chunk's owner: the rank that sends the KV
    state to this one in forward (lasp/utils/seq_parallel_manager.py:25-28)."""
    return (dist.get_rank() - 1) % dist.get_world_size()


def get_seq_parallel_receive_rank() -> int:
    """Global rank of the next chunk's owner: it receives this rank's KV state
    in forward (lasp/utils/seq_parallel_manager.py:31-34)."""
    return (dist.get_rank() + 1) % dist.get_world_size()


def is_unitialized() -> bool:
    return _G.dp_group is None


def sequence_parallel_is_initialized() -> bool:
    return _G.sp_group is not None and _G.dp_group is not None


def get_sequence_parallel_group():
    assert _G.sp_group is not None, "sequence parallel group is not initialized"
    return _G.sp_group


def get_data_parallel_group(with_sequence_parallel: bool = False):
    if with_sequence_parallel:
        assert _G.all_group is not None, "sequence data parallel group is not initialized"
        return _G.all_group
    assert _G.dp_group is not None, "data parallel group is not initialized"
    return _G.dp_group


def set_sequence_parallel_world_size(world_size) -> None:
    _G.sp_world_override = world_size


def get_sequence_parallel_world_size() -> int:
    if _G.sp_world_override is not None:
        return _G.sp_world_override
    return dist.get_world_size(group=get_sequence_parallel_group())


def set_sequence_parallel_rank(rank) -> None:
    _G.sp_rank_override = rank


def get_sequence_parallel_rank() -> int:
    if _G.sp_rank_override is not None:
        return _G.sp_rank_override
    return dist.get_rank(group=get_sequence_parallel_group())


def get_sequence_parallel_src_rank() -> int:
    """Global rank of the first member of the caller's SP group."""
    size = get_sequence_parallel_world_size()
    return (dist.get_rank() // size) * size


def get_data_parallel_src_rank() -> int:
    assert _G.dp_ranks is not None, "Data parallel group is not initialized"
    return _G.dp_ranks[0]


def get_data_parallel_world_size(with_sequence_parallel: bool = False) -> int:
    # like the reference (:188-192) the flag does not change the answer
    return dist.get_world_size(group=get_data_parallel_group(False))


def get_data_parallel_rank(with_sequence_parallel: bool = False) -> int:
    return dist.get_rank(group=get_data_parallel_group(False))


class GlobalMemoryBuffer:
    """Named, grow-only scratch tensors (lasp/utils/seq_parallel_manager.py:232-256).
    Buffers of one name must not be in use by two callers at once."""

    def __init__(self):
        self.buffer = {}

    def get_tensor(self, tensor_shape, dtype, name):
        need = math.prod(tensor_shape)
        held = self.buffer.get((name, dtype))
        if held is None or held.numel() < need:
            held = torch.empty(need, dtype=dtype, device=torch.cuda.current_device(), requires_grad=False)
            self.buffer[(name, dtype)] = held
        return held[:need].view(*tensor_shape)


def _set_global_memory_buffer() -> None:
    assert _G.buffer is None, "global memory buffer is already initialized"
    _G.buffer = GlobalMemoryBuffer()


def get_global_memory_buffer() -> GlobalMemoryBuffer:
    assert _G.buffer is not None, "global memory buffer is not initialized"
    return _G.buffer


def destroy_global_memory_buffer() -> None:
    _G.buffer = None


def destroy_parallel_groups() -> None:
    _G.clear()


def get_rank(group) -> int:
    return dist.get_rank(group=group)
