"""Group-wide collectives: validate the call, then hand it to the active policy.

Every check runs before any communication and depends only on the call's arguments and on
state that is identical on every rank (policy, bridge transport, group size), so a rejected
call is rejected on every rank alike (reference: src/gpubridge/collectives.py:35-352).
``async_op=True`` returns a :class:`~gpubridge_b200.work.Work`.  A policy that only
enqueues device work (the fused NVLink kernels) starts on the calling thread, ordered by
events, and a blocking call of it is stream-ordered like an NCCL call; every other policy
runs on the rank's worker thread, first in first out.
"""
from __future__ import annotations

import weakref
from collections.abc import Callable

import torch
from torch.distributed import ReduceOp

from gpubridge_b200 import observe
from gpubridge_b200 import work as _work
from gpubridge_b200.policies import CollectivePolicy, implements, policies_implementing
from gpubridge_b200.topology import Topology, get_topology
from gpubridge_b200.work import Work

#: Dtypes every path supports (Gloo, NCCL and the fused kernels).  bool is left out (its SUM
#: is a logical OR), and so are int16/uint16/uint32/float8, which Gloo rejects.
SUPPORTED_DTYPES = (torch.float16, torch.bfloat16, torch.float32, torch.float64,
                    torch.int8, torch.uint8, torch.int32, torch.int64)
_FLOATS = SUPPORTED_DTYPES[:4]
_OP_NAMES = ((ReduceOp.SUM, "sum"), (ReduceOp.AVG, "avg"), (ReduceOp.MAX, "max"),
             (ReduceOp.MIN, "min"))
REDUCE_OPS = dict(_OP_NAMES)


_OP_FAST: dict = {"sum": "sum", "avg": "avg", "max": "max", "min": "min"}
for _known, _name in _OP_NAMES:
    try:
        _OP_FAST[_known] = _name          # the enum members hash; a ReduceOp(...) instance may not
    except TypeError:
        pass


def _op_name(op, fn: str) -> str:
    try:
        fast = _OP_FAST.get(op)
    except TypeError:
        fast = None
    if fast is not None:
        return fast
    for known, name in _OP_NAMES:
        try:
            if op == known:
                return name
        except TypeError:
            break
    raise ValueError(f"gpubridge.{fn} supports ReduceOp.SUM, AVG, MAX and MIN, got {op}. "
                     "PRODUCT is not supported: NCCL and Gloo aren't shown to agree on every dtype.")


def _check_tensor(tensor, topology: Topology) -> None:
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"expected a torch.Tensor, got {type(tensor).__name__}")
    if tensor.dtype not in SUPPORTED_DTYPES:
        names = ", ".join(str(d).removeprefix("torch.") for d in SUPPORTED_DTYPES)
        raise ValueError(f"gpubridge doesn't support {tensor.dtype}: a dtype must work on both "
                         f"the island backend and Gloo. Supported: {names}.")
    if tensor.device != topology.device:
        hint = (" (tensors stay on CPU in simulation and CPU-only mode)"
                if topology.simulated else "")
        raise ValueError(f"tensor is on {tensor.device} but this rank communicates on "
                         f"{topology.device}{hint}")
    if not tensor.is_contiguous():
        raise ValueError("tensor must be contiguous")


def _check_avg(name: str, dtype: torch.dtype, fn: str) -> None:
    if name == "avg" and dtype not in _FLOATS:
        raise ValueError(f"gpubridge.{fn} with ReduceOp.AVG needs a floating-point tensor, got "
                         f"{dtype}: AVG divides the sum by the world size, and an integer "
                         "division would need a rounding rule. Use SUM and divide yourself.")


def _supported_ops(policy: CollectivePolicy, topology: Topology) -> frozenset[str]:
    cached = getattr(policy, "_gb_reduce_ops", None)
    if cached is not None and cached[0]() is topology:
        return cached[1]
    supported = policy.supported_reduce_ops(topology)
    try:
        policy._gb_reduce_ops = (weakref.ref(topology), supported)  # type: ignore[attr-defined]
    except (AttributeError, TypeError):
        pass
    return supported


def _check_reduce_op(policy, name: str, topology: Topology, fn: str) -> None:
    supported = _supported_ops(policy, topology)
    if name not in supported:
        raise NotImplementedError(
            f"gpubridge.{fn} with {name.upper()}: collective policy {policy.name!r} with bridge "
            f"transport {topology.peers[topology.rank].bridge!r} supports only "
            f"{', '.join(sorted(n.upper() for n in supported))}.")


def _check_implements(policy, fn: str, topology: Topology) -> None:
    if not implements(policy, fn):
        usable = ", ".join(policies_implementing(fn, topology.layout))
        raise NotImplementedError(f"collective policy {policy.name!r} doesn't implement {fn}. "
                                  f"Policies that do and fit this cluster: {usable or 'none'}.")


def _check_pair(output, input, topology, fn, *, big, small) -> None:  # noqa: A002
    _check_tensor(output, topology)
    _check_tensor(input, topology)
    if output.dtype != input.dtype:
        raise ValueError(f"gpubridge.{fn}: output is {output.dtype} but input is {input.dtype}")
    world = topology.world_size
    if big.numel() != world * small.numel():
        raise ValueError(
            f"gpubridge.{fn}: {'output' if big is output else 'input'} must have world_size "
            f"({world}) times as many elements as the {'input' if big is output else 'output'} "
            f"({small.numel()}), got {big.numel()}")


def _start(topology: Topology, op: str, policy: CollectivePolicy | None,
           run: Callable[[], None], tensors: list[torch.Tensor], result,
           async_op: bool) -> Work | None:
    observe.refuse_in_callback(op)
    fused = policy is not None and policy.stream_ordered(topology)
    if fused:
        fabric = topology.fabric
        if not async_op:
            _work.drain()
            fabric.check()
            run()                      # on the caller's stream, ordered like an NCCL call
            return None
        return _work.launch(topology.device, op, lambda: fabric.on_comm_stream(run, tensors),
                            result, check=fabric.check, stream=fabric.comm_stream)
    if async_op:
        return _work.submit(topology.device, op, run, tensors, result)
    _work.drain()
    run()
    return None


def all_reduce(tensor: torch.Tensor, op=ReduceOp.SUM, *, async_op: bool = False,
               _topology: Topology | None = None) -> Work | None:
    """Reduce ``tensor`` over every rank of the group, in place (SUM, AVG, MAX, MIN).

    Every rank must pass the same shape and dtype.  AVG needs a floating-point dtype; it is
    the SUM divided by the group size, identically on every rank (inside the kernel on the
    fused path).  Raises ``ValueError`` for an unsupported op or dtype, a tensor on the wrong
    device or not contiguous; ``NotImplementedError`` when policy or transport can't carry
    the op; ``RuntimeError`` when not initialised.
    """
    topology = _topology or get_topology()
    name = _op_name(op, "all_reduce")
    _check_tensor(tensor, topology)
    _check_avg(name, tensor.dtype, "all_reduce")
    policy = topology.policy.select_policy(tensor.nbytes)
    base = "sum" if name == "avg" else name
    _check_reduce_op(policy, base, topology, "all_reduce")
    world = topology.world_size

    def run() -> None:
        with observe.collective(topology, "all_reduce", tensor, policy=policy.name,
                                reduce_op=name):
            if name == "avg" and policy.fuses_average(topology):
                policy.all_reduce(tensor, topology, divide=world)
            elif base == "sum":
                policy.all_reduce(tensor, topology)
                if name == "avg":
                    tensor.div_(world)
            else:
                policy.all_reduce(tensor, topology, op=base)

    return _start(topology, "all_reduce", policy, run, [tensor], tensor, async_op)


def broadcast(tensor: torch.Tensor, src: int, *, async_op: bool = False,
              _topology: Topology | None = None) -> Work | None:
    """Copy ``tensor`` from global rank ``src`` to every rank of the group, in place."""
    topology = _topology or get_topology()
    if src not in topology.layout.members:
        if not topology.layout.ranks:
            raise ValueError(f"src must be a rank in [0, {topology.world_size}), got {src}")
        raise ValueError(f"src must be one of the group's ranks "
                         f"{list(topology.layout.members)}, got {src}")
    _check_tensor(tensor, topology)
    policy = topology.policy.select_policy(tensor.nbytes)

    def run() -> None:
        with observe.collective(topology, "broadcast", tensor, src=src, policy=policy.name):
            policy.broadcast(tensor, src, topology)

    return _start(topology, "broadcast", policy, run, [tensor], tensor, async_op)


def all_gather_into_tensor(output: torch.Tensor, input: torch.Tensor, *,  # noqa: A002
                           async_op: bool = False,
                           _topology: Topology | None = None) -> Work | None:
    """``output`` = every rank's ``input`` back to back, ordered by rank."""
    topology = _topology or get_topology()
    _check_pair(output, input, topology, "all_gather_into_tensor", big=output, small=input)
    policy = topology.policy.select_policy(output.nbytes)
    _check_implements(policy, "all_gather_into_tensor", topology)

    def run() -> None:
        with observe.collective(topology, "all_gather_into_tensor", input, policy=policy.name):
            policy.all_gather_into_tensor(output, input, topology)

    return _start(topology, "all_gather_into_tensor", policy, run, [output, input], output,
                  async_op)


def reduce_scatter_tensor(output: torch.Tensor, input: torch.Tensor, op=ReduceOp.SUM, *,  # noqa: A002
                          async_op: bool = False,
                          _topology: Topology | None = None) -> Work | None:
    """Reduce every rank's ``input`` (SUM or AVG) and leave slice ``r`` on rank ``r``;
    ``input`` is not modified."""
    topology = _topology or get_topology()
    name = _op_name(op, "reduce_scatter_tensor")
    if name not in ("sum", "avg"):
        raise ValueError(f"gpubridge.reduce_scatter_tensor supports SUM and AVG, got {op}")
    _check_pair(output, input, topology, "reduce_scatter_tensor", big=input, small=output)
    _check_avg(name, input.dtype, "reduce_scatter_tensor")
    policy = topology.policy.select_policy(input.nbytes)
    _check_implements(policy, "reduce_scatter_tensor", topology)
    world = topology.world_size

    def run() -> None:
        with observe.collective(topology, "reduce_scatter_tensor", input, policy=policy.name,
                                reduce_op=name):
            if name == "avg" and policy.fuses_average(topology):
                policy.reduce_scatter_tensor(output, input, topology, divide=world)
            else:
                policy.reduce_scatter_tensor(output, input, topology)
                if name == "avg":
                    output.div_(world)

    return _start(topology, "reduce_scatter_tensor", policy, run, [output, input], output,
                  async_op)


def barrier(*, async_op: bool = False, _topology: Topology | None = None) -> Work | None:
    """Block until every rank of the group reaches this call.  On GPUs the rank's queued
    device work finishes first, so earlier collectives are complete locally on return."""
    topology = _topology or get_topology()

    def run() -> None:
        with observe.collective(topology, "barrier"):
            if not topology.simulated:
                torch.cuda.synchronize(topology.device)
            if topology.fabric is not None:
                topology.fabric.barrier()
                torch.cuda.current_stream(topology.device).synchronize()
                topology.fabric.check()
            else:
                topology.world_group.barrier()

    return _start(topology, "barrier", None, run, [], None, async_op)
