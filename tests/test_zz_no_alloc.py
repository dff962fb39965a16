"""The allocation-free single linear (glmflash_exl3_linear_static) against the caller-scratch entry point.

Collected last on purpose: a run that stops at the first failure has then already run every other test.  Some
hosts cannot let a library allocate device memory (they own the whole heap, or an allocator call would stall their
serving streams); for them the library carries its scratch as a built-in array.  The two entry points run the same
kernels, so their outputs must be identical bit for bit -- on the first call, and on a second call with other
inputs that finds the previous call's leftovers in the shared array."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(a, cuda):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a.view(np.int32) if a.dtype == np.uint32 else a)).to(cuda)


def test_static_linear_matches_scratch_linear_twice(pkg, synth, cuda):
    import torch
    K, N = 2048, 1536
    for call, (seed, rows) in enumerate([(11, 16), (12, 3)]):          # two calls in a row, different inputs and row counts
        g = synth.rng(seed)
        x = _dev(g.standard_normal((rows, K)).astype(np.float16), cuda)
        words = _dev(g.integers(0, 1 << 32, size=(K // 16, N // 16, 32), dtype=np.uint64).astype(np.uint32), cuda)
        suh, svh = _dev(synth.scales(g, 1, K)[0], cuda), _dev(synth.scales(g, 1, N)[0], cuda)
        got = pkg.exl3_linear_static(x, words, suh, svh, K, N)
        torch.cuda.synchronize()
        want = pkg.exl3_linear(x, words, suh, svh, K, N)
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}: outputs differ"


def test_static_linear_rejects_oversize(pkg, cuda):
    import torch
    L = pkg.lib()
    assert L.glmflash_exl3_linear_static_max_bytes() >= L.glmflash_exl3_linear_scratch_bytes(4096, 2048) > 0
    d = torch.zeros(64, dtype=torch.int32, device=cuda)
    p = C.c_void_p(d.data_ptr())
    rc = L.glmflash_exl3_linear_static(None, p, 1, p, p, p, 8192, 1536, p)
    assert rc == -1 and b"built-in scratch" in L.glmflash_error()
