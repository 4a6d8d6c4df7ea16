"""The allocation-free GroupSum entry point (dl_groupsum_f32_static), through the C ABI.

Some users of the library cannot allocate device memory themselves -- a binding that only passes on
the buffers its framework gave it, a server whose memory pool is fixed -- so they cannot supply the
workspace that dl_groupsum_f32 needs.  For them the library keeps 256 KiB of scratch per GPU inside
itself.  These tests check that the variant gives the same numbers as the workspace version, twice in
a row and across changes of shape (the built-in scratch is shared and keeps the previous call's contents),
on shapes that really run the kernel that uses the scratch, and that shapes beyond the built-in scratch are
refused.  It is collected last so that a failure here cannot hide another.
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


# (n, batch, k).  dl_groupsum_f32 has two kernels: one that needs no scratch (several pieces per class and classes of
# 64 .. 4096 rows) and one that keeps partial sums and counters in the workspace.  Only the second one touches the
# built-in array, so most shapes here are picked to take it: classes shorter than 64 or longer than 4096 rows.
SCRATCH_SHAPES = [(64, 1024, 2), (36, 130, 1), (100000, 128, 10), (60, 37, 3)]
NO_SCRATCH_SHAPES = [(16000, 128, 10), (6400, 512, 2)]


@pytest.mark.parametrize("shape", SCRATCH_SHAPES + NO_SCRATCH_SHAPES)
def test_static_scratch_groupsum_matches_workspace_version(shape):
    lib = N.lib()
    n, batch, k = shape
    if shape in SCRATCH_SHAPES:
        # more than the 4096 bytes of counters: the shape stores partial sums, i.e. it really runs the scratch kernel
        assert 4096 < lib.dl_groupsum_workspace_bytes(n, batch, k) <= lib.dl_groupsum_static_limit_bytes()
    g = torch.Generator().manual_seed(n + batch)
    for call in range(2):  # second call: the scratch still holds the first call's partial sums
        x = torch.rand(n, batch, generator=g).cuda()
        ref, got = _both(lib, x, k, 7.0)
        expect = x.double().reshape(k, n // k, batch).sum(1).T / 7.0
        assert torch.allclose(got.double(), expect, rtol=1e-5, atol=1e-6), call
        assert torch.equal(got, ref), call  # same kernel, same order of summation


def test_static_scratch_survives_a_change_of_shape():
    """Two different shapes back to back share the array: what the first left behind must not leak into the second."""
    lib = N.lib()
    g = torch.Generator().manual_seed(5)
    for n, batch, k in [(100000, 128, 10), (64, 1024, 2), (36, 130, 1), (100000, 128, 10)]:
        x = torch.rand(n, batch, generator=g).cuda()
        ref, got = _both(lib, x, k, 3.0)
        assert torch.equal(got, ref), (n, batch, k)


def test_static_scratch_groupsum_with_the_scratch_kernel_forced():
    """The shape of a real network head (16000 rows, batch 128, 10 classes) through the scratch kernel: the switch that
    forces it is process-wide, so both entry points run the same kernel."""
    lib = N.lib()
    x = torch.rand(16000, 128, generator=torch.Generator().manual_seed(9)).cuda()
    with N.tuning(N.TUNE_GROUPSUM_KERNEL, 1):
        assert lib.dl_groupsum_workspace_bytes(16000, 128, 10) > 4096
        for _ in range(2):
            ref, got = _both(lib, x, 10, 30.0)
            assert torch.equal(got, ref)
    expect = x.double().reshape(10, 1600, 128).sum(1).T / 30.0
    assert torch.allclose(got.double(), expect, rtol=1e-5, atol=1e-6)


def test_static_scratch_groupsum_refuses_what_does_not_fit():
    lib = N.lib()
    limit = lib.dl_groupsum_static_limit_bytes()
    assert limit == 256 << 10
    n, batch, k = 100000, 3712, 10  # classes of 10000 rows in 2 pieces: 10 * 2 * 3712 partial sums + counters > 256 KiB
    assert lib.dl_groupsum_workspace_bytes(n, batch, k) > limit
    x = torch.zeros(16, device="cuda")  # never read: the size check comes first
    status = lib.dl_groupsum_f32_static(x.data_ptr(), x.data_ptr(), n, batch, k, 1.0, None)
    assert status == N.DL_ERR_TOO_LARGE
    with pytest.raises(RuntimeError, match="scratch"):
        N.check(status)


def test_static_scratch_groupsum_takes_any_size_that_needs_no_scratch():
    """(6400, 16384, 2): the workspace version would want 512 KiB, but this shape runs the kernel without scratch."""
    lib = N.lib()
    n, batch, k = 6400, 16384, 2
    assert lib.dl_groupsum_workspace_bytes(n, batch, k) > lib.dl_groupsum_static_limit_bytes()
    x = torch.rand(n, batch, generator=torch.Generator().manual_seed(3)).cuda()
    ref, got = _both(lib, x, k, 2.0)
    assert torch.equal(got, ref)
