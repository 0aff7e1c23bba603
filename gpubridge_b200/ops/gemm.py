"""All-gather fused into a tcgen05 GEMM (``csrc/gb_gemm.cu``): ``y = x @ gather(w_shards).T``.

The FSDP2 pattern "all-gather the sharded Linear weight, then run the Linear" as one
persistent kernel: communication blocks bring the peers' shards over NVLink into a local
gathered weight and raise a flag per shard; GEMM blocks (TMA -> shared memory ->
``tcgen05.mma`` -> tensor memory -> epilogue) start on the local shard at once and take each
remote shard as soon as its flag is up.  Replaces ``dist.all_gather_into_tensor`` +
``F.linear`` (reference: src/gpubridge/torch_backend.py:271-285).
"""
from __future__ import annotations

import ctypes

import torch

from gpubridge_b200.ops import _lib

launches = 0


class AllGatherLinear:
    """State of one fused all-gather + GEMM site: the gathered weight, the shard flags and the
    call counter.  ``fabric`` is the team's :class:`~gpubridge_b200.ops.fabric.Fabric` (one of a
    single rank works too: then this is a plain tcgen05 GEMM)."""

    def __init__(self, fabric, out_features: int, in_features: int, comm_blocks: int = 16,
                 pair: bool | None = None, gathered: torch.Tensor | None = None) -> None:
        if out_features % fabric.world:
            raise ValueError("out_features must divide evenly over the team")
        if in_features % 8:
            raise ValueError("in_features must be a multiple of 8 (16-byte rows for TMA)")
        self.fabric, self.N, self.K = fabric, out_features, in_features
        device = fabric.device
        # ``gathered``: a caller-owned [out, in] bf16 buffer (layers of one shape can share it)
        self.gathered = (torch.empty((out_features, in_features), dtype=torch.bfloat16, device=device)
                         if gathered is None else gathered)
        assert self.gathered.shape == (out_features, in_features) and self.gathered.is_contiguous()
        self.flags = torch.zeros(fabric.world, dtype=torch.int32, device=device)
        self.error = torch.zeros(1, dtype=torch.int32, device=device)
        self.epoch = 0
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        # pair: CTA pairs (tcgen05 cta_group::2) share the weight operand; GPUBRIDGE_GEMM_PAIR=0
        # selects the single-CTA kernel
        import os
        self.pair = (os.environ.get("GPUBRIDGE_GEMM_PAIR", "1") != "0") if pair is None else pair
        self.comm_blocks = comm_blocks + (comm_blocks & 1 if self.pair else 0)
        self.gemm_blocks = max(2, sms - self.comm_blocks)
        if self.pair:
            self.gemm_blocks -= self.gemm_blocks & 1
        shard_bytes = out_features // fabric.world * in_features * 2
        if fabric.world > 1 and shard_bytes > fabric.len_ag:
            raise ValueError(f"a weight shard of {shard_bytes} bytes exceeds the fabric's staging "
                             f"area ({fabric.len_ag}); raise GPUBRIDGE_FABRIC_BYTES")

    def __call__(self, x: torch.Tensor, shard: torch.Tensor) -> torch.Tensor:
        """``x``: [M, K] bf16; ``shard``: this rank's [N / world, K] rows.  Returns [M, N]."""
        global launches
        assert x.dtype == torch.bfloat16 and shard.dtype == torch.bfloat16
        assert x.is_contiguous() and shard.is_contiguous() and x.shape[1] == self.K
        assert shard.shape == (self.N // self.fabric.world, self.K)
        fabric = self.fabric
        y = torch.empty((x.shape[0], self.N), dtype=torch.bfloat16, device=x.device)
        self.epoch += 1
        current = fabric._begin()
        try:
            with torch.cuda.stream(fabric.comm_stream):
                entry = fabric.lib.gb_allgather_gemm_pair if self.pair else fabric.lib.gb_allgather_gemm
                code = entry(
                    ctypes.byref(fabric.team), y.data_ptr(), x.data_ptr(), shard.data_ptr(),
                    self.gathered.data_ptr(), self.flags.data_ptr(), self.error.data_ptr(),
                    self.epoch, x.shape[0], self.N, self.K, fabric.off_ag, 2 * fabric.len_ag,
                    self.gemm_blocks,
                    self.comm_blocks, torch.cuda.current_stream(x.device).cuda_stream)
                if code == -3:
                    raise RuntimeError("cuTensorMapEncodeTiled is unavailable or refused the shapes")
                _lib.check(code, "gb_allgather_gemm")
        finally:
            fabric._end(current)
        launches += 1
        return y

    def check(self) -> None:
        """Raise if a wait inside the kernel ran out (reads one word from the device)."""
        code = int(self.error.item())
        if code:
            raise RuntimeError(f"gb_allgather_gemm: a bounded wait ran out (code {code})")


class GemmReduceScatter:
    """``out = mean over ranks of (a @ b.T)[rows of this rank]`` in one kernel
    (``csrc/gb_gemm_rs.cu``): a tcgen05 GEMM whose epilogue stores every row of the product
    into its owner's workspace over NVLink (bf16 partials, the slot of the sending rank), then
    a team barrier and the fp32 sum of the slots of the own rows.  ``a``: [P, R], ``b``: [Q, R],
    both bf16 and contiguous; P divides over the team, Q and R are multiples of 8.  The weight
    gradient of a row-sharded Linear is ``GemmReduceScatter(fabric)(dy.T, x.T)``.

    Stages through the fabric's reduce-scatter region; :meth:`fits` says whether the shapes do.
    """

    def __init__(self, fabric) -> None:
        self.fabric = fabric
        self.error = torch.zeros(1, dtype=torch.int32, device=fabric.device)
        self.region = (fabric.off_rs, 4 * fabric.len_rs)

    def fits(self, P: int, Q: int, R: int) -> bool:
        world = self.fabric.world
        if P % world or Q % 8 or R % 8 or min(P, Q, R) <= 0:
            return False
        need = self.fabric.lib.gb_gemm_reduce_scatter_bytes(world, P, Q)
        return 0 < need // 2 <= self.region[1] // 2

    def __call__(self, a: torch.Tensor, b: torch.Tensor, divide: int | None = None,
                 out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        global launches
        assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
        assert a.is_contiguous() and b.is_contiguous() and a.shape[1] == b.shape[1]
        assert out_dtype in (torch.bfloat16, torch.float32)
        fabric = self.fabric
        P, R = a.shape
        Q = b.shape[0]
        if not self.fits(P, Q, R):
            raise ValueError(f"shapes [{P}, {R}] x [{Q}, {R}] do not fit the fused GEMM + reduce-scatter "
                             f"(rows over {fabric.world} ranks, multiples of 8, staging "
                             f"{self.region[1] // 2} bytes per collective)")
        out = torch.empty((P // fabric.world, Q), dtype=out_dtype, device=a.device)
        current = fabric._begin()
        try:
            with torch.cuda.stream(fabric.comm_stream):
                code = fabric.lib.gb_gemm_reduce_scatter(
                    ctypes.byref(fabric.team), out.data_ptr(), a.data_ptr(), b.data_ptr(),
                    self.error.data_ptr(), P, Q, R, self.region[0], self.region[1],
                    int(divide or 0), int(out_dtype == torch.float32), 0,
                    torch.cuda.current_stream(a.device).cuda_stream)
                if code == -3:
                    raise RuntimeError("cuTensorMapEncodeTiled is unavailable or refused the shapes")
                if code == -4:
                    raise RuntimeError("the fabric's reduce-scatter region is too small for these shapes")
                _lib.check(code, "gb_gemm_reduce_scatter")
                for t in (a, b, out):
                    t.record_stream(fabric.comm_stream)
        finally:
            fabric._end(current)
        launches += 1
        return out

    def check(self) -> None:
        """Raise if a wait inside the kernel ran out (reads one word from the device)."""
        code = int(self.error.item())
        if code:
            raise RuntimeError(f"the fused GEMM + reduce-scatter gave up on a wait (code {code})")
        self.fabric.check()
