"""The whole-tensor pinned staging of a leader's bridge step, with copies that run only when
somebody waits for them (the lanes of ``tests/_staging.py``): the bridge reads the buffer only
after the copy out, the next collective's copy out waits for the last copy back, buffers grow
only after that copy back and are reused otherwise, ``close`` waits too - and a staging layer
that drops the wait loses the first result (the negative control).
(Reference: tests/test_pinned_staging.py.)"""
import torch

from _staging import Lane
from gpubridge_b200 import staging


class Deferred(staging.WholeStaging):
    """Copies are queued on one lane (one stream) and run when waited for."""

    def __init__(self):
        super().__init__(torch.device("cpu"))
        self.journal: list = []
        self.lane = Lane(self.journal)
        self.allocations: list[int] = []
        self.count = 0

    def _allocate(self, nbytes):
        self.allocations.append(nbytes)
        return torch.full((nbytes,), 0xEE, dtype=torch.uint8)

    def _copy(self, dst, src, after):
        self.count += 1
        return self.lane.queue(f"copy{self.count}", lambda: dst.copy_(src), after)

    def _wait(self, event):
        event.settle()


class ForgetsTheCopyBack(Deferred):
    """Broken on purpose: a copy out does not wait for the previous copy back, and - as on a
    GPU whose copy engine is late - that copy back runs only when somebody asks for it."""

    def __init__(self):
        super().__init__()
        self.back = Lane(self.journal)

    def to_device(self, tensor, host):
        self.count += 1
        self.copied_back = self.back.queue(f"back{self.count}", lambda: tensor.copy_(host), None)

    def _copy(self, dst, src, after):
        return super()._copy(dst, src, None)


def bridge_step(stage, tensor):
    host = stage.to_host(tensor)
    seen = host.clone()                                            # what the bridge would send
    host.mul_(2)                                                   # what the bridge leaves: the "sum"
    stage.to_device(tensor, host)
    return seen


def test_the_bridge_reads_the_buffer_only_after_the_copy_out():
    stage = Deferred()
    t = torch.arange(100, dtype=torch.float32)
    seen = bridge_step(stage, t)
    assert torch.equal(seen, torch.arange(100, dtype=torch.float32))       # not the 0xEE the buffer was born with
    assert stage.journal == [("ran", "copy1")]                     # the copy back is still only queued
    assert torch.equal(t, torch.arange(100, dtype=torch.float32))
    stage.close()
    assert torch.equal(t, 2 * torch.arange(100, dtype=torch.float32))


def test_the_next_collective_waits_for_the_last_copy_back():
    stage = Deferred()
    a, b = torch.full((50,), 3.0), torch.full((50,), 10.0)
    bridge_step(stage, a)
    seen_b = bridge_step(stage, b)                                 # reuses the buffer a's result still sits in
    assert torch.equal(a, torch.full((50,), 6.0))                  # a got its result before the buffer was reused
    assert torch.equal(seen_b, torch.full((50,), 10.0))
    assert [label for _, label in stage.journal] == ["copy1", "copy2", "copy3"]
    stage.close()
    assert torch.equal(b, torch.full((50,), 20.0))


def test_without_that_wait_the_first_result_is_overwritten():
    stage = ForgetsTheCopyBack()
    a, b = torch.full((50,), 3.0), torch.full((50,), 10.0)
    bridge_step(stage, a)
    bridge_step(stage, b)
    stage.back.run_until(stage.copied_back)                        # everything queued has run by now
    assert not torch.equal(a, torch.full((50,), 6.0))              # a's copy back read b's data
    assert torch.equal(a, torch.full((50,), 20.0))


def test_a_larger_tensor_gets_a_new_buffer_after_the_last_copy_back():
    stage = Deferred()
    small, large = torch.full((10,), 1.0), torch.full((1000,), 5.0)
    bridge_step(stage, small)
    old = stage.buffer
    seen = bridge_step(stage, large)
    assert stage.allocations == [40, 4000] and stage.buffer is not old
    assert torch.equal(small, torch.full((10,), 2.0))              # copied back before its buffer was let go
    assert torch.equal(seen, torch.full((1000,), 5.0))
    stage.close()
    assert torch.equal(large, torch.full((1000,), 10.0))


def test_a_smaller_tensor_reuses_the_buffer_and_other_dtypes_and_shapes_fit():
    stage = Deferred()
    bridge_step(stage, torch.ones(1000))
    for t in (torch.ones(10), torch.ones(20, 30, dtype=torch.float16), torch.ones(7, dtype=torch.float64),
              torch.ones(1000)):
        want = 2 * t.clone()
        bridge_step(stage, t)
        stage._wait(stage.copied_back)
        assert torch.equal(t, want)
    assert stage.allocations == [4000]
    host = stage.to_host(torch.ones(3, 5, dtype=torch.int32))
    assert host.shape == (3, 5) and host.dtype == torch.int32


def test_close_waits_for_the_last_copy_back_and_lets_go_of_the_buffer():
    stage = Deferred()
    t = torch.full((8,), 4.0)
    bridge_step(stage, t)
    assert torch.equal(t, torch.full((8,), 4.0))
    stage.close()
    assert torch.equal(t, torch.full((8,), 8.0)) and stage.buffer is None and stage.copied_back is None
    stage.close()                                                  # twice is fine
    bridge_step(stage, t)                                          # and it can be used again afterwards
    stage.close()
    assert torch.equal(t, torch.full((8,), 16.0)) and stage.allocations == [32, 32]


def test_cpu_devices_need_no_staging():
    assert staging.make_bridge_staging(torch.device("cpu")) is None
    plain = staging.make_staging(torch.device("cpu"), 1 << 20, 2)
    assert type(plain) is staging.HostStaging
    chunk = torch.arange(6.0)
    assert plain.slot(0, chunk) is chunk                           # the bridge works on the tensor where it lies
    assert plain.to_host(chunk, chunk) is None and plain.to_device(chunk, chunk) is None
    plain.begin(chunk), plain.wait_host(None), plain.end(None), plain.close()
