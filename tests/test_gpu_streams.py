"""Stream ordering of the fused collectives and of pinned staging, on one GPU.

Each test writes its input only after a stretch of queued GPU work (until then the tensor
holds a poison value) or reads its output straight after the call, so a missing
stream-to-stream wait shows as wrong values.  ``MUTATIONS`` names, for every switch of
``gpubridge_b200._mutation``, the test that must fail when the switch is on;
``python -m gpubridge_b200.kit.stream_mutations`` runs them both ways (the reference audits
its own stream fixes the same way: scripts/gpu/stream_mutations.py).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

POISON = -1000.0
BUSY = 0.05          # seconds of queued GPU work ahead of the input's last write
N = 1 << 22

MUTATIONS = {
    "comm-ignores-caller": ("sync collective starts before the caller's queued work",
                            "test_sync_collective_waits_for_caller"),
    "caller-ignores-comm": ("caller's stream does not wait for a sync collective",
                            "test_caller_waits_for_sync_collective"),
    "async-ignores-caller": ("async collective starts before the caller's queued work",
                             "test_async_collective_waits_for_caller"),
    "wait-skips-stream": ("Work.wait() orders no stream",
                          "test_wait_orders_the_callers_stream"),
    "staging-ignores-caller": ("pinned staging copies start before the caller's queued work",
                               "test_staging_waits_for_caller"),
}


@pytest.fixture()
def team():
    from gpubridge_b200.ops import fabric as F
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    t = F.create_single(device)
    yield t
    torch.cuda.synchronize()
    t.check()
    t.close()


def _late_input(device, value):
    """A tensor that holds poison until BUSY seconds of queued work have run."""
    from gpubridge_b200.kit import queue_gpu_delay
    x = torch.full((N,), POISON, device=device)
    queue_gpu_delay(device, BUSY)
    x.fill_(value)
    return x


def _wrong(t, value):
    bad = int((t != value).sum())
    return f"{bad} elements wrong" if bad else ""


# Every scenario runs twice and only the second pass is judged: the first use of a kernel in a
# process loads its module, which synchronises the device and would hide a missing wait.

def test_sync_collective_waits_for_caller(team):
    for _ in range(2):
        out = torch.zeros(N, device=team.device)
        x = _late_input(team.device, 3.0)
        team.all_reduce(x, "sum", None, "striped", out=out)
        torch.cuda.synchronize()
        verdict = _wrong(out, 3.0)
    assert not verdict, verdict


def test_caller_waits_for_sync_collective(team):
    big = 1 << 26                                   # 256 MiB: the kernel runs for a while
    x = torch.full((big,), 5.0, device=team.device)
    for _ in range(2):
        out = torch.full((big,), POISON, device=team.device)
        torch.cuda.synchronize()
        team.all_reduce(x, "sum", None, "striped", out=out)
        seen = out[-4096:].clone()                  # queued on the caller's stream at once
        torch.cuda.synchronize()
        verdict = _wrong(seen, 5.0)
    assert not verdict, verdict


def _launch_async(team, x, out):
    from gpubridge_b200 import work as W
    return W.launch(team.device, "all_reduce",
                    lambda: team.on_comm_stream(
                        lambda: team.all_reduce(x, "sum", None, "striped", out=out), [x, out]),
                    out, check=team.check, stream=team.comm_stream)


def test_async_collective_waits_for_caller(team):
    for _ in range(2):
        out = torch.zeros(N, device=team.device)
        x = _late_input(team.device, 7.0)
        work = _launch_async(team, x, out)
        work.wait()
        torch.cuda.synchronize()
        verdict = _wrong(out, 7.0)
    assert not verdict, verdict


def test_wait_orders_the_callers_stream(team):
    big = 1 << 26
    x = torch.full((big,), 9.0, device=team.device)
    for _ in range(2):
        out = torch.full((big,), POISON, device=team.device)
        torch.cuda.synchronize()
        work = _launch_async(team, x, out)
        work.wait()                                 # orders this stream; the host does not block
        seen = out[-4096:].clone()
        torch.cuda.synchronize()
        verdict = _wrong(seen, 9.0)
    assert not verdict, verdict


def test_staging_waits_for_caller():
    from gpubridge_b200.staging import ChunkStaging
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    staging = ChunkStaging(device, N * 4, 2)
    for _ in range(2):
        x = _late_input(device, 11.0)
        staging.begin(x)
        slot = staging.slot(0, x)
        done = staging.to_host(slot, x)
        staging.wait_host(done)
        host = slot.clone()
        torch.cuda.synchronize()
        verdict = _wrong(host, 11.0)
    staging.close()
    assert not verdict, verdict
