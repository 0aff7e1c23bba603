"""DistributedDataParallel communication hook: gradient buckets through gpubridge.

``model.register_comm_hook(None, gpubridge_b200.ddp_comm_hook)`` keeps DDP's bucketing and
its overlap with backward and hands every bucket to :func:`gpubridge_b200.all_reduce` with
``ReduceOp.AVG`` and ``async_op=True`` (reference: src/gpubridge/ddp.py:41-52).  On a GPU
group with a fabric that is one fused kernel per bucket on the communication stream: the
hierarchical reduction, the optional compressed bridge leg and the division by the world
size happen in the same launch, and the returned future is stream-ordered, so the host
thread driving backward never blocks.
"""
import torch
import torch.distributed as dist
from torch.distributed import ReduceOp

from gpubridge_b200.collectives import all_reduce


# The annotations are real objects, not strings: DDP checks them when the hook is registered.
def ddp_comm_hook(state: object, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Average one gradient bucket over every rank; ``state`` may be a Topology (a
    subgroup's) or None for the initialised world."""
    from gpubridge_b200.topology import Topology
    topology = state if isinstance(state, Topology) else None
    work = all_reduce(bucket.buffer(), op=ReduceOp.AVG, async_op=True, _topology=topology)
    assert work is not None
    return work.get_future()
