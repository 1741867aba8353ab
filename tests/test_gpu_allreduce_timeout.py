"""The bounded wait of the peer-memory all-reduce, on one GPU and without any fault: a link
of two ranks is set up with both receive buffers in local memory and only rank 0 ever calls.
Rank 0 pushes its packets, polls its own buffer for rank 1's, finds none, and after the poll
limit (set low for the test) gives up: the call returns, the device error word reads 0x1ff
(b200q_device_error -> 0x101ff), the context stays usable and a later call with a present
peer works.  The reference's kernels wait without a bound
(csrc/custom_all_reduce.cuh:180-262), so it has no test of this kind."""
import ctypes

import pytest

pytestmark = pytest.mark.gpu


def test_all_reduce_gives_up_when_the_peer_never_sends():
    import torch

    from vllm_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    vp = ctypes.c_void_p
    world, max_bytes, n = 2, 1 << 16, 4096
    nbuf = lib.b200q_all_reduce_buffer_bytes(world, max_bytes)
    bufs = [torch.zeros(nbuf, dtype=torch.uint8, device=dev) for _ in range(world)]
    ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    state = torch.zeros(lib.b200q_all_reduce_state_bytes() // 4, dtype=torch.int32, device=dev)
    x = torch.ones(n, dtype=torch.bfloat16, device=dev)
    out = torch.full((n,), 7.0, dtype=torch.bfloat16, device=dev)
    stream = vp(torch.cuda.current_stream().cuda_stream)
    assert lib.b200q_device_error(1) == 0
    lib.b200q_all_reduce_set_poll_limit(2000)
    try:
        rc = lib.b200q_all_reduce(vp(ptrs.data_ptr()), vp(state.data_ptr()), 0, world, max_bytes,
                                  vp(x.data_ptr()), vp(out.data_ptr()), n, _lib.BF16, stream)
        _lib.check(rc, "b200q_all_reduce")
        torch.cuda.synchronize()                      # the kernel came back by itself
        assert lib.b200q_device_error(1) == 0x101FF   # and said why
        assert lib.b200q_device_error(0) == 0         # reading with reset cleared the word
        assert bool((out == 7.0).all())               # no output was written for the lost peer
    finally:
        lib.b200q_all_reduce_set_poll_limit(0)
    # the context is intact: with "rank 1" played by a second link state on the same buffers,
    # both calls complete and agree on the sum
    for b in bufs:
        b.zero_()
    state0 = torch.zeros_like(state)
    state1 = torch.zeros_like(state)
    y = torch.full((n,), 2.0, dtype=torch.bfloat16, device=dev)
    out0, out1 = torch.empty_like(x), torch.empty_like(x)
    # rank 1 first, with a short limit: its own packets land in rank 0's buffer before it
    # gives up waiting for rank 0 (the two "ranks" run one after the other on one GPU and so
    # must not wait for each other); rank 0 then finds rank 1's packets already there
    lib.b200q_all_reduce_set_poll_limit(2000)
    rc = lib.b200q_all_reduce(vp(ptrs.data_ptr()), vp(state1.data_ptr()), 1, world, max_bytes,
                              vp(y.data_ptr()), vp(out1.data_ptr()), n, _lib.BF16, stream)
    _lib.check(rc, "b200q_all_reduce")
    torch.cuda.synchronize()
    assert lib.b200q_device_error(1) == 0x101FF
    lib.b200q_all_reduce_set_poll_limit(0)
    rc = lib.b200q_all_reduce(vp(ptrs.data_ptr()), vp(state0.data_ptr()), 0, world, max_bytes,
                              vp(x.data_ptr()), vp(out0.data_ptr()), n, _lib.BF16, stream)
    _lib.check(rc, "b200q_all_reduce")
    torch.cuda.synchronize()
    assert lib.b200q_device_error(1) == 0
    assert bool((out0 == 3.0).all())
