"""The bounded waits of the peer-memory exchange kernels, made to run out on ONE GPU.

Rank 0 of a world of two is driven through the C ABI; its "peer" is a second set of buffers in the same process
(same GPU, ordinary memory) that no kernel ever drives, so the flags rank 0 waits for are never raised.  With a
short time limit the kernels must give up, report through the error word of the bucket's state, and leave
parameters, moments and step count exactly as they were.  Then the test plays the peer by hand (raises its flags)
and the next call must work.  Nothing here faults or waits without a limit.
"""
import ctypes

import pytest
import torch

from difflogic_b200 import _native as N

pytestmark = pytest.mark.gpu

MAX_RANKS = 16


def _flag(bucket, peer, which):
    return (bucket * MAX_RANKS + peer) * 2 + which


def _ptrs(*tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


@pytest.mark.parametrize("bucket,whole", [(0, 0), (3, 0), (1, 1)])
def test_exchange_wait_runs_out_and_leaves_everything_untouched(bucket, whole):
    lib = N.lib()
    n, lr, beta1, beta2, eps = 4096, 0.01, 0.9, 0.999, 1e-8
    g = torch.Generator().manual_seed(17 + bucket)
    own_p, peer_p = torch.randn(n, generator=g).cuda(), torch.randn(n, generator=g).cuda()
    own_g, peer_g = torch.randn(n, generator=g).cuda(), torch.randn(n, generator=g).cuda()
    words = lib.dl_exchange_flag_bytes() // 4
    own_f = torch.zeros(words, dtype=torch.int32, device="cuda")
    peer_f = torch.zeros(words, dtype=torch.int32, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    state = torch.zeros(16, dtype=torch.int32, device="cuda")
    params, grads, flags = _ptrs(own_p, peer_p), _ptrs(own_g, peer_g), _ptrs(own_f, peer_f)
    stream = torch.cuda.current_stream().cuda_stream
    before = own_p.clone()

    def one_step(limit_us):
        N.check(lib.dl_exchange_bucket_f32(params, grads, flags, 0, 2, m.data_ptr(), v.data_ptr(), 0, n, bucket, lr, beta1, beta2, eps,
                                           state.data_ptr(), 1, whole, limit_us, N.LAUNCH_PLAIN, stream))
        torch.cuda.synchronize()

    one_step(2000)   # 2 ms: nobody raises the peer's flags, the wait for its gradients runs out
    s = state.tolist()
    assert s[2] == 1, "the error word must be set"
    assert s[0] == 0 and s[1] == 0 and s[3] == 0, "step count untouched, tickets re-armed"
    assert torch.equal(own_p, before) and not m.any() and not v.any()
    # rank 0 did announce its gradients to itself and to the peer, and never announced a finished slice
    assert int(own_f[_flag(bucket, 0, 0)]) == 1 and int(peer_f[_flag(bucket, 0, 0)]) == 1
    assert int(own_f[_flag(bucket, 0, 1)]) == 0 and int(peer_f[_flag(bucket, 0, 1)]) == 0

    # the peer "arrives": its gradients and its slice (the second half of peer_p) are declared complete
    own_f[_flag(bucket, 1, 0)] = 1
    own_f[_flag(bucket, 1, 1)] = 1
    state[2] = 0
    one_step(0)      # default limit; every flag is there already
    s = state.tolist()
    assert s[2] == 0 and s[0] == 1 and s[1] == 0 and s[3] == 0
    half = n if whole else n // 2      # one pass: this rank updates the whole bucket itself
    ref = before[:half].cpu().clone().requires_grad_(True)
    ref.grad = ((own_g[:half] + peer_g[:half]) * 0.5).cpu()
    torch.optim.Adam([ref], lr=lr, betas=(beta1, beta2), eps=eps).step()
    assert torch.allclose(own_p[:half].cpu(), ref.detach(), rtol=1e-6, atol=1e-7)   # own slice: Adam on the mean gradient
    if not whole:
        assert torch.equal(own_p[half:], peer_p[half:])                             # other slice: fetched from the peer
        assert m[half:].abs().max().item() == 0.0                                   # moments of the peer's slice untouched


def test_backward_w_announces_the_bucket_when_its_last_kernel_is_through():
    """dl_backward_w_announce_f32 on one GPU, world of one: same gradient as the plain kernel; the flag word carries the
    bucket's next step number only after BOTH kernels that share the bucket have run; the counters are back at zero."""
    from difflogic_b200 import ops
    from tests.helpers import random_layer
    lib = N.lib()
    a, b, w = random_layer(40, 96, seed=4)
    a, b, w = a.cuda(), b.cuda(), w.cuda()
    x = torch.rand(40, 52, device="cuda")
    gy = torch.randn(96, 52, device="cuda")
    ref = ops.logic_backward_w(x, a, b, gy, w, ops.W_LOGITS)
    flags = torch.zeros(lib.dl_exchange_flag_bytes() // 4, dtype=torch.int32, device="cuda")
    state = torch.zeros(16, dtype=torch.int32, device="cuda")
    state[0] = 6                                   # six steps done: the seventh is announced
    tickets = torch.zeros(2, dtype=torch.int32, device="cuda")
    kernels = torch.zeros(1, dtype=torch.int32, device="cuda")
    bucket, word = 2, lib.dl_exchange_flag_word(2, 0, 0)
    assert word == _flag(2, 0, 0)
    out1, out2 = torch.empty_like(ref), torch.empty_like(ref)
    ops.logic_backward_w_announce(x, a, b, gy, w, out1, 1, _ptrs(flags), 0, 1, bucket, state, tickets[0:], kernels, 2)
    torch.cuda.synchronize()
    assert int(flags[word]) == 0 and int(kernels[0]) == 1 and int(tickets[0]) == 0
    ops.logic_backward_w_announce(x, a, b, gy, w, out2, 1, _ptrs(flags), 0, 1, bucket, state, tickets[1:], kernels, 2)
    torch.cuda.synchronize()
    assert int(flags[word]) == 7 and int(kernels[0]) == 0 and not tickets.any()
    assert torch.equal(out1, ref) and torch.equal(out2, ref)
    assert int(flags.ne(0).sum()) == 1


def test_exchange_entry_points_validate_their_arguments():
    lib = N.lib()
    t = torch.zeros(64, device="cuda")
    f = torch.zeros(lib.dl_exchange_flag_bytes() // 4, dtype=torch.int32, device="cuda")
    st = torch.zeros(16, dtype=torch.int32, device="cuda")
    one = _ptrs(t)
    flags = _ptrs(f)
    args = (t.data_ptr(), t.data_ptr())
    tail = (0.01, 0.9, 0.999, 1e-8, st.data_ptr(), 1, 0, 0, 0, None)
    assert lib.dl_exchange_bucket_f32(one, one, flags, 1, 1, *args, 0, 64, 0, *tail) == N.DL_ERR_INVALID_ARG    # rank outside the world
    assert lib.dl_exchange_bucket_f32(one, one, flags, 0, 1, *args, 0, 62, 0, *tail) == N.DL_ERR_INVALID_ARG    # count not a multiple of 4
    assert lib.dl_exchange_bucket_f32(one, one, flags, 0, 1, *args, 0, 64, 32, *tail) == N.DL_ERR_INVALID_ARG   # bucket
    assert lib.dl_exchange_bucket_f32(one, one, flags, 0, 17, *args, 0, 64, 0, *tail) == N.DL_ERR_INVALID_ARG   # world
    assert lib.dl_exchange_announce(flags, 0, 1, 40, st.data_ptr(), None) == N.DL_ERR_INVALID_ARG


@pytest.mark.parametrize("world,rank,whole", [(8, 3, 0), (8, 7, 1), (4, 0, 0), (4, 2, 1), (3, 1, 0), (2, 1, 0)])
def test_exchange_kernel_for_every_world_size_with_the_peers_played_by_hand(world, rank, whole):
    """One rank of a world of 2, 3, 4 or 8 on ONE GPU: the other ranks are buffers in the same process whose flags are
    raised beforehand, so no wait has anything to wait for.  Checks the arithmetic of every variant of the kernel: the
    mean over all ranks' gradients in this rank's slice (the whole bucket in the one-pass form), Adam on it, and the
    other ranks' slices fetched from their parameter buffers.  The bucket is not a multiple of the slice size."""
    lib = N.lib()
    n, off, lr, beta1, beta2, eps, bucket = 4 * 1237, 64, 0.01, 0.9, 0.999, 1e-8, 5
    total = off + n + 32
    g = torch.Generator().manual_seed(100 * world + rank)
    params = [torch.randn(total, generator=g).cuda() for _ in range(world)]
    grads = [torch.randn(total, generator=g).cuda() for _ in range(world)]
    words = lib.dl_exchange_flag_bytes() // 4
    flags = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(world)]
    for p in range(world):
        if p != rank:
            flags[rank][_flag(bucket, p, 0)] = 1
            flags[rank][_flag(bucket, p, 1)] = 1
    m, v = torch.zeros(total, device="cuda"), torch.zeros(total, device="cuda")
    state = torch.zeros(16, dtype=torch.int32, device="cuda")
    before = params[rank].clone()
    N.check(lib.dl_exchange_bucket_f32(_ptrs(*params), _ptrs(*grads), _ptrs(*flags), rank, world, m.data_ptr(), v.data_ptr(), off, n,
                                       bucket, lr, beta1, beta2, eps, state.data_ptr(), 1, whole, 0, N.LAUNCH_PLAIN,
                                       torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    s = state.tolist()
    assert s[0] == 1 and s[1] == 0 and s[2] == 0 and s[3] == 0
    per = -(-(n // 4) // world) * 4                       # floats per slice
    lo = off + min(rank * per, n)
    hi = min(lo + per, off + n)
    if whole:
        lo, hi = off, off + n
    mean = grads[0].clone()
    for p in range(1, world):
        mean += grads[p]                                  # rank order, as the kernel adds them
    mean *= 1.0 / world
    ref = before[lo:hi].cpu().clone().requires_grad_(True)
    ref.grad = mean[lo:hi].cpu()
    torch.optim.Adam([ref], lr=lr, betas=(beta1, beta2), eps=eps).step()
    got = params[rank]
    assert torch.allclose(got[lo:hi].cpu(), ref.detach(), rtol=1e-6, atol=1e-7)
    assert torch.equal(got[:off], before[:off]) and torch.equal(got[off + n:], before[off + n:])   # outside the bucket
    if not whole:
        for p in range(world):
            if p == rank:
                continue
            plo = off + min(p * per, n)
            phi = min(plo + per, off + n)
            assert torch.equal(got[plo:phi], params[p][plo:phi])
        assert not m[off:lo].any() and not m[hi:off + n].any()
    # every rank was told about this rank's gradients and its finished slice
    for p in range(world):
        assert int(flags[p][_flag(bucket, rank, 0)]) == 1 and int(flags[p][_flag(bucket, rank, 1)]) == 1


def test_rank_barrier_passes_when_the_peers_are_there_and_runs_out_when_not():
    lib = N.lib()
    words = lib.dl_exchange_flag_bytes() // 4
    own_f = torch.zeros(words, dtype=torch.int32, device="cuda")
    peer_f = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(2)]
    flags = _ptrs(peer_f[0], own_f, peer_f[1])          # this is rank 1 of three
    state = torch.zeros(16, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    slot = 31

    def barrier(limit_us):
        N.check(lib.dl_rank_barrier(flags, 1, 3, slot, state.data_ptr(), limit_us, stream))
        torch.cuda.synchronize()

    barrier(2000)                      # nobody else is there: the wait runs out after 2 ms
    assert state.tolist()[:3] == [0, 0, 1]
    # this rank did tell everybody that it had arrived
    assert all(int(f[_flag(slot, 1, 0)]) == 1 for f in (own_f, peer_f[0], peer_f[1]))
    state.zero_()
    own_f[_flag(slot, 0, 0)] = 1       # the peers arrive (played by hand)
    own_f[_flag(slot, 2, 0)] = 1
    barrier(2000)
    assert state.tolist()[:3] == [1, 0, 0]
    own_f[_flag(slot, 0, 0)] = 2
    barrier(2000)                      # second barrier: rank 2 has not arrived yet
    assert state.tolist()[:3] == [1, 0, 1]
    # a world of one has nobody to wait for
    alone = torch.zeros(16, dtype=torch.int32, device="cuda")
    N.check(lib.dl_rank_barrier(_ptrs(own_f), 0, 1, 30, alone.data_ptr(), 2000, stream))
    torch.cuda.synchronize()
    assert alone.tolist()[:3] == [1, 0, 0]
    assert lib.dl_rank_barrier(flags, 3, 3, slot, state.data_ptr(), 0, stream) == N.DL_ERR_INVALID_ARG
    assert lib.dl_rank_barrier(flags, 0, 3, 32, state.data_ptr(), 0, stream) == N.DL_ERR_INVALID_ARG


def test_bounded_mbarrier_wait_of_the_staged_kernels_runs_out_and_returns():
    """The wait helper of the bulk-copy kernels, on a barrier that nobody completes: it must give up after its poll limit
    (2^16 here; the kernels use 2^24), the kernel must return, and the library must work afterwards."""
    import time
    lib = N.lib()
    result = torch.zeros(2, dtype=torch.int32, device="cuda")
    errors_before = lib.dl_async_error()
    t0 = time.perf_counter()
    N.check(lib.dl_selftest_bounded_wait(result.data_ptr(), 1 << 16, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert result.tolist() == [1, 1]
    assert lib.dl_async_error() == errors_before
    assert lib.dl_selftest_bounded_wait(result.data_ptr(), 0, None) == N.DL_ERR_INVALID_ARG
    x = torch.arange(12, dtype=torch.float32, device="cuda").view(3, 4)
    from difflogic_b200 import ops
    assert torch.equal(ops.transpose(x), x.t().contiguous())
