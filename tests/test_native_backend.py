"""backend="gpubridge_native": the C++ c10d::Backend in front of the Python process group.

CPU ranks have no NVLink fabric, so every collective here crosses C++ into the Python group
and back - which is the part a CPU can test: registration, the hand-over of every call of the
surface, Work and future plumbing, subgroups, DDP, and that a second job in the same process
gets fresh objects.  The engine's planning is held to the Python planner in
test_engine_parity.py; the launches themselves need GPUs (tests marked gpu)."""
import os
import subprocess
import sys
import textwrap

import pytest

from gpubridge_b200.ops import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.skipif(not _lib.available(), reason="the native library is not built")

RANKS = textwrap.dedent('''
    import torch, torch.distributed as dist
    import gpubridge_b200.native_backend as nb

    def job(round_):
        dist.init_process_group(backend="gpubridge_native")
        r, w = dist.get_rank(), dist.get_world_size()
        assert dist.get_backend() == "gpubridge_native"
        t = torch.full((5,), float(r + 1)); dist.all_reduce(t)
        assert t[0].item() == w * (w + 1) / 2
        t = torch.full((5,), float(r + 1)); dist.all_reduce(t, op=dist.ReduceOp.AVG)
        assert t[0].item() == (w + 1) / 2
        t = torch.full((5,), r + 1, dtype=torch.int64); dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t[0].item() == w
        b = torch.arange(4.) if r == 1 else torch.zeros(4); dist.broadcast(b, 1)
        assert b.tolist() == [0, 1, 2, 3]
        out = torch.zeros(w * 3); dist.all_gather_into_tensor(out, torch.full((3,), float(r)))
        assert out.view(w, 3)[:, 0].tolist() == list(range(w))
        rs = torch.zeros(2); dist.reduce_scatter_tensor(rs, torch.arange(2. * w))
        assert rs.tolist() == [w * 2. * r, w * (2. * r + 1)]
        lists = [torch.zeros(2) for _ in range(w)]; dist.all_gather(lists, torch.full((2,), float(r)))
        assert [x[0].item() for x in lists] == list(range(w))
        objs = [None] * w; dist.all_gather_object(objs, {"rank": r})
        assert [o["rank"] for o in objs] == list(range(w))
        work = dist.all_reduce(torch.ones(3), async_op=True)
        assert work.wait() and work.is_completed()
        assert work.get_future().wait()[0].tolist() == [w] * 3
        dist.barrier()
        if r == 0:
            dist.send(torch.tensor([7.]), 1)
        elif r == 1:
            x = torch.zeros(1); dist.recv(x, 0); assert x.item() == 7
        peer = r ^ 1
        got = torch.zeros(3)
        ops = [dist.P2POp(dist.isend, torch.full((3,), float(r)), peer), dist.P2POp(dist.irecv, got, peer)]
        for w_ in dist.batch_isend_irecv(ops):        # torch's own helper: the backend coalesces
            w_.wait()
        assert got.tolist() == [float(peer)] * 3
        sub = dist.new_group([0, 1])
        if r < 2:
            s = torch.ones(2) * (r + 1); dist.all_reduce(s, group=sub); assert s[0] == 3
        backend = nb.backend_of()
        assert backend.native_calls == 0 and backend.fallback_calls >= 9       # CPU ranks: no fabric
        assert nb.python_group_of() is not None
        torch.manual_seed(0)
        model = torch.nn.Linear(4, 2)
        ddp = torch.nn.parallel.DistributedDataParallel(model)
        torch.manual_seed(10 + r)
        ddp(torch.randn(3, 4)).sum().backward()
        g = model.weight.grad.clone(); hi = g.clone(); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert torch.equal(g, hi)
        with_bad_op = torch.ones(2)
        try:
            dist.all_reduce(with_bad_op, op=dist.ReduceOp.BXOR)
        except (RuntimeError, ValueError, NotImplementedError) as exc:
            assert "gpubridge" in str(exc)
        else:
            raise AssertionError("BXOR went through")
        dist.destroy_process_group()
        assert nb.backend_of.__module__ and not nb._made, nb._made

    job(0)
    job(1)            # a second job in the same process gets fresh objects
    print("ok")
''')


def test_cpp_backend_hands_the_whole_surface_over(tmp_path):
    script = tmp_path / "ranks.py"
    script.write_text(RANKS)
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1", GPUBRIDGE_VENDOR="nvidia",
               GPUBRIDGE_SPLIT_TEST="half")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
           "--master-addr", "127.0.0.1", "--master-port", "29771", str(script)]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, (done.stdout + done.stderr)[-4000:]
    assert done.stdout.count("ok") == 4


def test_front_end_switch_for_programs_that_name_the_python_backend(tmp_path):
    script = tmp_path / "ranks.py"
    script.write_text(textwrap.dedent('''
        import torch, torch.distributed as dist
        import gpubridge_b200, gpubridge_b200.native_backend as nb
        dist.init_process_group(backend="gpubridge")
        t = torch.ones(4) * (dist.get_rank() + 1)
        dist.all_reduce(t)
        assert t[0].item() == 3
        assert nb.backend_of() is not None and nb.backend_of().fallback_calls >= 1
        dist.destroy_process_group()
        print("ok")
    '''))
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1", GPUBRIDGE_VENDOR="nvidia",
               GPUBRIDGE_SPLIT_TEST="half", GPUBRIDGE_FRONT_END="native")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29774", str(script)]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, (done.stdout + done.stderr)[-3000:]
    assert done.stdout.count("ok") == 2


@pytest.mark.parametrize("extra", [[], ["--hsdp", "2"]])
def test_fsdp2_and_hsdp_bit_for_bit_through_the_cpp_front_end(extra):
    """The FSDP2 / HSDP example's --verify (parameters equal a single-process replay, bit for
    bit) with the C++ backend under torch's own ProcessGroup: device-mesh subgroups included."""
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="1", GPUBRIDGE_VENDOR="nvidia",
               GPUBRIDGE_SPLIT_TEST="half")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
           "--master-addr", "127.0.0.1", "--master-port", "29773" if extra else "29772",
           os.path.join(ROOT, "examples", "fsdp2_torch_backend.py"), "--verify", "--backend",
           "gpubridge_native", *extra]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, (done.stdout + done.stderr)[-4000:]
    assert "bit for bit" in done.stdout


def test_the_backend_suite_passes_through_the_cpp_front_end():
    """Every test of the Python backend's suite (DDP, every collective, refusals with their
    reasons, FSDP2, HSDP, subgroups, re-init) once more with GPUBRIDGE_FRONT_END=native."""
    env = dict(os.environ, PYTHONPATH=ROOT, GPUBRIDGE_FRONT_END="native")
    done = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_backend.py"),
                           "-q", "-x", "-p", "no:cacheprovider"], env=env, cwd=ROOT, capture_output=True,
                          text=True, timeout=1200)
    assert done.returncode == 0, done.stdout[-4000:]
