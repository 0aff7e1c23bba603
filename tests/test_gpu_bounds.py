"""The fused collectives under the checked library (``GPUBRIDGE_BOUNDS=1``, built with
``-DGB_BOUNDS``): every 16-byte access and every bulk-copy source of the kernels is compared
with the ranges the host allowed for the call (workspaces of all ranks, switch memory, the
call's tensors).  The whole collectives scenario of the fabric suite - odd sizes, every
dtype, every collective, compressed and plain - must finish with no access outside them, for
one island and for two."""
import pytest
import torch

from _harness import gpu_ranks, run_ranks
from test_gpu_fabric import _collectives

pytestmark = pytest.mark.gpu
WORLD = min(torch.cuda.device_count(), 4) if torch.cuda.is_available() else 0


def _checked(rank, topology, policy):
    from gpubridge_b200.ops import _lib
    assert _lib.BOUNDS and _lib.path().endswith("_bounds.so")
    return _collectives(rank, topology, policy)


@pytest.mark.skipif(WORLD < 2, reason="needs two GPUs")
@pytest.mark.parametrize("split", [{}, {"GPUBRIDGE_SPLIT_TEST": "half"}], ids=["one-island", "half"])
def test_collectives_touch_only_allowed_memory(tmp_path, split):
    env = dict(split, GPUBRIDGE_BOUNDS="1")
    out = run_ranks(gpu_ranks(WORLD), _checked, tmp_path, "auto", env=env, timeout=300)
    assert all(launches > 0 for _, launches in out)
