"""The exchange with the flags inside the data (dl_exchange_packets_f32), one rank of a world of 2, 3, 4 or 8 on ONE GPU.

The other ranks are played by hand: their gradient packets and parameter packets are written into this rank's inboxes
before the launch (so no wait has anything to wait for), and what this rank pushed is read out of theirs afterwards.
The result must equal, bit for bit, what dl_exchange_bucket_f32 makes of the same numbers.  A launch with empty inboxes
must give up within its time limit and say so.  Nothing here faults or waits without a limit.
"""
import ctypes

import pytest
import torch

from difflogic_b200 import _native as N

pytestmark = pytest.mark.gpu

MAX_RANKS = 16


def _ptrs(*tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _flag(bucket, peer, which):
    return (bucket * MAX_RANKS + peer) * 2 + which


class Inbox:
    """world regions of `stride` float4 slots; a slot is 4 packets {value, epoch} of 8 bytes in two planes."""

    def __init__(self, world, stride):
        self.world, self.stride = world, stride
        self.t = torch.zeros(world * stride * 4, dtype=torch.int64, device="cuda")

    def _views(self, region, slot0, k):
        half = self.world * self.stride * 2
        base = (region * self.stride + slot0) * 2
        return self.t[base:base + 2 * k].view(k, 2), self.t[half + base:half + base + 2 * k].view(k, 2)

    def put(self, region, slot0, values, epoch):
        k = values.numel() // 4
        bits = values.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        packets = (bits | (epoch << 32)).view(k, 4)
        a, b = self._views(region, slot0, k)
        a.copy_(packets[:, :2])
        b.copy_(packets[:, 2:])

    def get(self, region, slot0, k):
        a, b = self._views(region, slot0, k)
        packets = torch.cat([a, b], dim=1).reshape(-1)
        return (packets & 0xFFFFFFFF).to(torch.int32).view(torch.float32), packets >> 32


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (3, 1), (4, 2), (8, 7), (8, 0)])
def test_packet_exchange_equals_the_flag_exchange(world, rank):
    lib = N.lib()
    n4, off, lr, beta1, beta2, eps = 1237, 64, 0.01, 0.9, 0.999, 1e-8
    n, total = 4 * n4, 64 + 4 * 1237 + 32
    per = -(-n4 // world)
    inbox_off, stride = 5, per + 9
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(1000 * world + rank)
    param = torch.randn(total, generator=g).cuda()
    ref_params = [param.clone() for _ in range(world)]          # the flag exchange runs on copies of everything
    m, v = torch.zeros(total, device="cuda"), torch.zeros(total, device="cuda")
    ref_m, ref_v = m.clone(), v.clone()
    state, ref_state = (torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(2))
    gin = [Inbox(world, stride) for _ in range(world)]
    pin = [Inbox(world, stride) for _ in range(world)]
    flags = [torch.zeros(lib.dl_exchange_flag_bytes() // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    slice_of = lambda p: (min(p * per, n4), min(min(p * per, n4) + per, n4))       # in float4 within the bucket
    my_lo, my_hi = slice_of(rank)

    for epoch in (1, 2):
        grads = [torch.randn(total, generator=g).cuda() for _ in range(world)]
        new_slices = {p: torch.randn(4 * (slice_of(p)[1] - slice_of(p)[0]), generator=g).cuda() for p in range(world) if p != rank}
        for p in range(world):
            if p == rank:
                continue
            # what rank p would have pushed: its gradients of MY slice, and (later) its new parameters of ITS slice
            gin[rank].put(p, inbox_off, grads[p][off + 4 * my_lo:off + 4 * my_hi], epoch)
            pin[rank].put(p, inbox_off, new_slices[p], epoch)
            lo, hi = slice_of(p)
            ref_params[p][off + 4 * lo:off + 4 * hi] = new_slices[p]
            flags[rank][_flag(0, p, 0)] = epoch
            flags[rank][_flag(0, p, 1)] = epoch
        outside = param.clone()
        N.check(lib.dl_exchange_packets_f32(param.data_ptr(), grads[rank].data_ptr(), _ptrs(*[b.t for b in gin]),
                                            _ptrs(*[b.t for b in pin]), rank, world, m.data_ptr(), v.data_ptr(), off, n, inbox_off,
                                            stride, lr, beta1, beta2, eps, state.data_ptr(), 0, 0, N.LAUNCH_PLAIN, stream))
        N.check(lib.dl_exchange_bucket_f32(_ptrs(*ref_params), _ptrs(*grads), _ptrs(*flags), rank, world, ref_m.data_ptr(),
                                           ref_v.data_ptr(), off, n, 0, lr, beta1, beta2, eps, ref_state.data_ptr(), 1, 0, 0,
                                           N.LAUNCH_PLAIN, stream))
        torch.cuda.synchronize()
        assert state.tolist()[:4] == [epoch, 0, 0, 0] and ref_state.tolist()[:4] == [epoch, 0, 0, 0]
        assert torch.equal(param, ref_params[rank]) and torch.equal(m, ref_m) and torch.equal(v, ref_v)
        assert torch.equal(param[:off], outside[:off]) and torch.equal(param[off + n:], outside[off + n:])
        for p in range(world):
            if p == rank:
                continue
            lo, hi = slice_of(p)
            # this rank's gradients of p's slice arrived in p's inbox, region `rank`, with this step's epoch ...
            values, epochs = gin[p].get(rank, inbox_off, hi - lo)
            assert torch.equal(values, grads[rank][off + 4 * lo:off + 4 * hi]) and bool((epochs == epoch).all())
            # ... and so did the new parameters of this rank's slice
            values, epochs = pin[p].get(rank, inbox_off, my_hi - my_lo)
            assert torch.equal(values, param[off + 4 * my_lo:off + 4 * my_hi]) and bool((epochs == epoch).all())
            # nothing was written outside the bucket's slots of that region
            assert not gin[p].t[(rank * stride) * 2:(rank * stride + inbox_off) * 2].any()


def test_packet_exchange_gives_up_when_no_packet_arrives():
    lib = N.lib()
    world, rank, n4, off = 2, 0, 600, 0
    per, stride = 300, 300
    param = torch.randn(4 * n4, device="cuda")
    grad = torch.randn(4 * n4, device="cuda")
    m, v = torch.zeros(4 * n4, device="cuda"), torch.zeros(4 * n4, device="cuda")
    state = torch.zeros(16, dtype=torch.int32, device="cuda")
    gin = [Inbox(world, stride) for _ in range(world)]
    pin = [Inbox(world, stride) for _ in range(world)]
    before = param.clone()
    N.check(lib.dl_exchange_packets_f32(param.data_ptr(), grad.data_ptr(), _ptrs(*[b.t for b in gin]), _ptrs(*[b.t for b in pin]),
                                        rank, world, m.data_ptr(), v.data_ptr(), off, 4 * n4, 0, stride, 0.01, 0.9, 0.999, 1e-8,
                                        state.data_ptr(), 0, 2000, N.LAUNCH_PLAIN, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    s = state.tolist()
    assert s[2] == 1 and s[0] == 0 and s[3] == 0          # error word set, step count untouched, ticket re-armed
    assert torch.equal(param, before) and not m.any()      # no gradient packet of the peer ever came: nothing was updated
    values, epochs = gin[1].get(0, 0, per)                 # the pushes of this rank went out all the same
    assert torch.equal(values, grad[4 * per:]) and bool((epochs == 1).all())
    # arguments are checked before anything is launched
    bad = lib.dl_exchange_packets_f32(param.data_ptr(), grad.data_ptr(), _ptrs(*[b.t for b in gin]), _ptrs(*[b.t for b in pin]),
                                      rank, world, m.data_ptr(), v.data_ptr(), off, 4 * n4, 1, stride, 0.01, 0.9, 0.999, 1e-8,
                                      state.data_ptr(), 0, 2000, N.LAUNCH_PLAIN, None)
    assert bad == N.DL_ERR_INVALID_ARG                      # the bucket's slots do not fit the region


@pytest.mark.parametrize("world,rank,n_out,bucket_offset", [(2, 1, 200, 0), (4, 0, 1000, 64), (3, 2, 77, 0), (8, 5, 512, 128)])
def test_backward_w_pushes_the_other_ranks_slices_as_packets(world, rank, n_out, bucket_offset):
    """dl_backward_w_push_f32: the same gradient as the plain kernel, and every element that belongs to another rank's
    slice of the bucket sits in that rank's inbox (this rank's region) as a packet with the bucket's next epoch."""
    from difflogic_b200 import ops
    from tests.helpers import random_layer
    n_in, batch = 96, 128
    a, b, w = random_layer(n_in, n_out, seed=world * 10 + rank)
    g = torch.Generator().manual_seed(5)
    x, gy = torch.rand(n_in, batch, generator=g).cuda(), torch.randn(n_out, batch, generator=g).cuda()
    a, b, w = a.cuda(), b.cuda(), w.cuda()
    plain = ops.logic_backward_w(x, a, b, gy, w, ops.W_LOGITS)
    bucket_count = bucket_offset + 16 * n_out + 32          # the layer is one of several parameters of the bucket
    n4 = bucket_count // 4
    per = -(-n4 // world)
    inbox_off, stride = 3, per + 7
    gin = [Inbox(world, stride) for _ in range(world)]
    state = torch.zeros(16, dtype=torch.int32, device="cuda")
    state[0] = 6                                            # six steps done: the packets carry 7
    out = torch.empty_like(plain)
    ops.logic_backward_w_push(x, a, b, gy, w, out, 1, _ptrs(*[bx.t for bx in gin]), rank, world, bucket_offset, bucket_count,
                              inbox_off, stride, state)
    torch.cuda.synchronize()
    assert torch.equal(out, plain)
    bucket = torch.zeros(bucket_count, device="cuda")
    bucket[bucket_offset:bucket_offset + 16 * n_out] = plain.reshape(-1)
    layer = torch.zeros(bucket_count, dtype=torch.bool, device="cuda")
    layer[bucket_offset:bucket_offset + 16 * n_out] = True
    for p in range(world):
        lo, hi = min(p * per, n4), min(min(p * per, n4) + per, n4)
        values, epochs = gin[p].get(rank, inbox_off, hi - lo)
        mine = layer[4 * lo:4 * hi]
        if p == rank:
            assert not gin[p].t.any()                       # nothing is sent to oneself
            continue
        assert torch.equal(values[mine], bucket[4 * lo:4 * hi][mine]) and bool((epochs[mine] == 7).all())
        assert bool((epochs[~mine] == 0).all())             # floats of the bucket outside this layer: not this kernel's
        for q in range(world):
            if q != rank:
                assert not gin[p].get(q, 0, stride)[1].any()    # other senders' regions untouched


def test_packet_exchange_after_a_push_does_not_push_again():
    lib = N.lib()
    world, rank, n4 = 2, 0, 512
    per, stride = 256, 256
    param, grad = torch.randn(4 * n4, device="cuda"), torch.randn(4 * n4, device="cuda")
    m, v = torch.zeros(4 * n4, device="cuda"), torch.zeros(4 * n4, device="cuda")
    state = torch.zeros(16, dtype=torch.int32, device="cuda")
    gin = [Inbox(world, stride) for _ in range(world)]
    pin = [Inbox(world, stride) for _ in range(world)]
    peer_grad, peer_new = torch.randn(4 * per, device="cuda"), torch.randn(4 * per, device="cuda")
    gin[0].put(1, 0, peer_grad, 1)
    pin[0].put(1, 0, peer_new, 1)
    N.check(lib.dl_exchange_packets_f32(param.data_ptr(), grad.data_ptr(), _ptrs(*[b.t for b in gin]), _ptrs(*[b.t for b in pin]),
                                        rank, world, m.data_ptr(), v.data_ptr(), 0, 4 * n4, 0, stride, 0.01, 0.9, 0.999, 1e-8,
                                        state.data_ptr(), 1, 2000, N.LAUNCH_PLAIN, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert state.tolist()[:4] == [1, 0, 0, 0]
    assert not gin[1].t.any()                               # pushed = 1: the gradients were not sent (again)
    assert torch.equal(param[4 * per:], peer_new)           # the peer's slice was collected
    assert bool((pin[1].get(0, 0, per)[1] == 1).all())      # and this rank's new slice went out
