"""The allocation-free GroupSum entry point (dl_groupsum_f32_static), through the C ABI.

Some users of the library cannot allocate device memory themselves -- a binding that only passes on
the buffers its framework gave it, a server whose memory pool is fixed -- so they cannot supply the
workspace that dl_groupsum_f32 needs.  For them the library keeps 256 KiB of scratch per GPU inside
itself.  This test checks that the variant gives the same numbers as the workspace version, twice in
a row (the built-in scratch is shared and keeps the previous call's contents), and that shapes beyond
the built-in scratch are refused.  It is collected last so that a failure here cannot hide another.
"""
import pytest
import torch

from difflogic_b200 import _native as N

pytestmark = pytest.mark.gpu


def _both(lib, x, k, tau):
    n, batch = x.shape
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.zeros(lib.dl_groupsum_workspace_bytes(n, batch, k), dtype=torch.uint8, device="cuda")
    ref = torch.empty(batch, k, device="cuda")
    got = torch.full((batch, k), float("nan"), device="cuda")
    N.check(lib.dl_groupsum_f32(x.data_ptr(), ref.data_ptr(), ws.data_ptr(), n, batch, k, tau, stream))
    N.check(lib.dl_groupsum_f32_static(x.data_ptr(), got.data_ptr(), n, batch, k, tau, stream))
    torch.cuda.synchronize()
    return ref, got


@pytest.mark.parametrize("shape", [(16000, 128, 10), (300, 37, 3), (6400, 512, 2)])
def test_static_scratch_groupsum_matches_workspace_version(shape):
    lib = N.lib()
    n, batch, k = shape
    g = torch.Generator().manual_seed(n + batch)
    for call in range(2):  # second call: the scratch still holds the first call's partial sums
        x = torch.rand(n, batch, generator=g).cuda()
        ref, got = _both(lib, x, k, 7.0)
        expect = x.double().reshape(k, n // k, batch).sum(1).T / 7.0
        assert torch.allclose(got.double(), expect, rtol=1e-5, atol=1e-6), call
        assert torch.equal(got, ref), call  # same kernel, same order of summation


def test_static_scratch_groupsum_refuses_what_does_not_fit():
    lib = N.lib()
    limit = lib.dl_groupsum_static_limit_bytes()
    assert limit == 256 << 10
    n, batch, k = 6400, 16384, 2  # two pieces per class: 2 * 2 * 16384 partial sums + counters > 256 KiB
    assert lib.dl_groupsum_workspace_bytes(n, batch, k) > limit
    x = torch.zeros(16, device="cuda")  # never read: the size check comes first
    status = lib.dl_groupsum_f32_static(x.data_ptr(), x.data_ptr(), n, batch, k, 1.0, None)
    assert status == N.DL_ERR_TOO_LARGE
    with pytest.raises(RuntimeError, match="scratch"):
        N.check(status)
