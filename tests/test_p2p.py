"""The host-staged point-to-point engine between islands, on CPU ranks: ordering within a lane,
independence of lanes (tags), sizes from empty to chunked, payload mismatch as an exception,
a peer that never posts (deadline), a peer that has gone (failure seen by the survivor), and
a teardown that does not wait for anybody.  (Reference: tests/test_p2p.py.)"""
import pytest
import torch

from _harness import TWO_BY_TWO, run_ranks


def _pair(rank):
    """Ranks 0 and 2 are in different islands (2+2): they take the bridged route."""
    return {0: 2, 2: 0}.get(rank)


def _ordering_and_tags(rank, world):
    import torch.distributed as dist
    dist.barrier()
    peer = _pair(rank)
    if peer is not None:
        # ten messages on one lane arrive in the order sent
        if rank == 0:
            works = [dist.isend(torch.full((64,), float(i)), peer, tag=1) for i in range(10)]
            [w.wait() for w in works]
        else:
            bufs = [torch.empty(64) for _ in range(10)]
            works = [dist.irecv(b, peer, tag=1) for b in bufs]
            [w.wait() for w in works]
            assert [float(b[0]) for b in bufs] == [float(i) for i in range(10)]
        # two lanes (tags) do not block each other: receive in the opposite order
        if rank == 0:
            a, b = dist.isend(torch.full((31,), 11.0), peer, tag=101), dist.isend(torch.full((31,), 22.0), peer, tag=102)
            a.wait(), b.wait()
        else:
            y, x = torch.empty(31), torch.empty(31)
            dist.recv(y, peer, tag=102)
            dist.recv(x, peer, tag=101)
            assert float(x[0]) == 11.0 and float(y[0]) == 22.0
        # sizes: empty, one element, odd, large; several dtypes
        for dtype in (torch.float32, torch.int64, torch.bfloat16, torch.uint8):
            for n in (0, 1, 4099, 300_001):
                data = (torch.arange(n) % 13).to(dtype)
                if rank == 0:
                    dist.send(data, peer, tag=7)
                else:
                    got = torch.full((n,), 99, dtype=dtype)
                    dist.recv(got, peer, tag=7)
                    assert torch.equal(got, data), (dtype, n)
    dist.barrier()
    return True


def test_ordering_tags_and_sizes(tmp_path):
    run_ranks(TWO_BY_TWO, _ordering_and_tags, tmp_path, mode="backend", timeout=180)


def test_chunked_transfers(tmp_path):
    run_ranks(TWO_BY_TWO, _ordering_and_tags, tmp_path, mode="backend", timeout=180,
              env={"GPUBRIDGE_P2P_CHUNK_BYTES": "64K"})


def _mismatch(rank, world):
    import torch.distributed as dist
    dist.barrier()
    peer = _pair(rank)
    caught = None
    if peer is not None:
        try:
            if rank == 0:
                dist.send(torch.zeros(100), peer, tag=5)
            else:
                dist.recv(torch.zeros(50), peer, tag=5)        # half the size: must not abort
        except (ValueError, RuntimeError) as exc:
            caught = str(exc)
    return caught


def test_payload_mismatch_raises_on_both_sides(tmp_path):
    out = run_ranks(TWO_BY_TWO, _mismatch, tmp_path, mode="backend", timeout=120)
    assert out[0] and "mismatch" in out[0]
    assert out[2] and "mismatch" in out[2]
    assert out[1] is None and out[3] is None


def _missing_peer(rank, world):
    """Rank 2 never posts the receive: rank 0's send runs into the group's deadline."""
    import time
    from datetime import timedelta
    import torch.distributed as dist
    dist.barrier()
    took = None
    if rank == 0:
        t0 = time.monotonic()
        work = dist.isend(torch.zeros(10), 2, tag=9)
        try:
            work.wait(timedelta(seconds=3))
        except (TimeoutError, RuntimeError) as exc:
            took = (time.monotonic() - t0, type(exc).__name__)
    else:
        time.sleep(4)
    return took


def test_missing_peer_times_out(tmp_path):
    out = run_ranks(TWO_BY_TWO, _missing_peer, tmp_path, mode="backend", timeout=120)
    took, kind = out[0]
    assert took < 20 and kind in ("TimeoutError", "RuntimeError")


def _teardown(rank, world):
    """Destroying the group with an operation still pending returns promptly."""
    import time
    import torch.distributed as dist
    dist.barrier()
    if rank == 0:
        dist.isend(torch.zeros(10), 2, tag=11)          # never matched
    time.sleep(0.2)
    t0 = time.monotonic()
    return t0


def test_teardown_is_bounded(tmp_path):
    import time
    before = time.monotonic()
    run_ranks(TWO_BY_TWO, _teardown, tmp_path, mode="backend", timeout=120)
    assert time.monotonic() - before < 60
