"""The cross-entropy entry point that allocates nothing (``gb_xent_fwd_bwd_noalloc``).

Some users of the library cannot hand it scratch memory: they run inside another program's
memory pool, or on a path where calling cudaMalloc is not allowed or not safe.  For them the
library keeps the scratch in a fixed device array of its own.  This test calls that entry
point through its exported C symbol, exactly as such a caller would, twice in a row (the
array keeps the first call's contents, so the second call checks that nothing stale leaks
through), and compares loss and gradient with the ordinary entry point, which takes its
scratch from the caller.  It is collected last so that a failure here cannot hide one
elsewhere, and it passes on its own in a fresh process as well as after the other tests.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from gpubridge_b200.ops import _lib
    lib = _lib.lib()
    vp, sz, i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    lib.gb_xent_fwd_bwd_noalloc.argtypes = [vp, i, vp, sz, sz, sz, vp, vp]
    lib.gb_xent_fwd_bwd_noalloc.restype = i
    lib.gb_xent_noalloc_error.argtypes = [i]
    lib.gb_xent_noalloc_error.restype = ctypes.c_char_p
    return lib


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_point_matches_the_ordinary_one(dtype):
    lib = _library()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    stream = torch.cuda.current_stream(device).cuda_stream
    code = 1 if dtype is torch.bfloat16 else 0
    for call, (rows, vocab, ld) in enumerate([(300, 50257, 50304), (77, 1000, 1000)]):
        torch.manual_seed(call)
        base = (torch.randn(rows, ld, device=device) * 3).to(dtype)
        targets = torch.randint(vocab, (rows,), device=device)
        # the ordinary entry point, scratch from the caller
        want = base.clone()
        row_loss = torch.empty(rows, dtype=torch.float32, device=device)
        counter = torch.zeros(1, dtype=torch.int32, device=device)
        want_loss = torch.empty((), dtype=torch.float32, device=device)
        assert lib.gb_xent_fwd_bwd(want.data_ptr(), code, targets.data_ptr(), rows, vocab, ld,
                                   row_loss.data_ptr(), counter.data_ptr(), want_loss.data_ptr(),
                                   stream) == 0
        # the entry point under test: inputs and outputs only
        got = base.clone()
        got_loss = torch.empty((), dtype=torch.float32, device=device)
        status = lib.gb_xent_fwd_bwd_noalloc(got.data_ptr(), code, targets.data_ptr(), rows,
                                             vocab, ld, got_loss.data_ptr(), stream)
        assert status == 0, lib.gb_xent_noalloc_error(status).decode()
        torch.cuda.synchronize(device)
        assert torch.allclose(got_loss, want_loss, rtol=1e-4, atol=1e-4), (call, got_loss, want_loss)
        tol = 2e-2 if dtype is torch.bfloat16 else 1e-5
        assert torch.allclose(got.float(), want.float(), rtol=tol, atol=tol / rows), call
        # and both agree with plain PyTorch in fp32
        ref = torch.nn.functional.cross_entropy(base[:, :vocab].float(), targets)
        assert torch.allclose(got_loss, ref, rtol=1e-4, atol=1e-4)


def test_no_alloc_entry_point_refuses_too_many_rows():
    lib = _library()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    dummy = torch.zeros(8, device=device)
    status = lib.gb_xent_fwd_bwd_noalloc(dummy.data_ptr(), 0, dummy.data_ptr(), 65537, 4, 4,
                                         dummy.data_ptr(),
                                         torch.cuda.current_stream(device).cuda_stream)
    assert status == -2
    assert b"65536" in lib.gb_xent_noalloc_error(status)
