"""A bounded wait that runs out, on one GPU (needs a B200).

``grb_peer_allreduce_bf16`` is called as rank 0 of a group of two whose second rank does not exist: its control block and
receive area are plain local buffers that nobody ever posts to.  The wait for the peer's flag has a limit of a few
milliseconds (a launch argument), so the kernel gives up by itself: the call returns, the status word carries
GRB_STATUS_TIMEOUT, the output is left alone and the context stays usable.  No kernel here waits for another kernel and
nothing faults, traps or spins without a limit.  The healthy call afterwards has the peer's flag and data put in place
by the host before the launch, so its wait is satisfied at the first poll.

The discipline mirrored here is the reference's per-lane status word, written on every exit path instead of a trap
(context-runtime/georefine_context_runtime/context_tiled_packet.cuh:32-33).
"""
import ctypes
import time

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

GRB_STATUS_TIMEOUT = 16
FLAG_STRIDE = 32          # u32 slots between two ranks' flags in a control block (csrc/peer_reduce.cuh)


@pytest.mark.parametrize("elems", [4096, 128 * 5120])   # one CTA; 128 CTAs that each wait for the flag
def test_peer_wait_gives_up_after_its_limit_and_the_next_call_works(elems):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from georefine_b200 import _native

    lib = _native.lib()
    dev = torch.device("cuda:0")
    block = 2 * elems
    control_words = int(lib.grb_peer_control_bytes()) // 4
    controls = [torch.zeros(control_words + 64, device=dev, dtype=torch.int32) for _ in range(2)]
    receives = [torch.zeros(2 * 2 * block, device=dev, dtype=torch.uint8) for _ in range(2)]
    aligned = lambda t, a: (t.data_ptr() + a - 1) // a * a
    cptr = (ctypes.c_void_p * 2)(*[aligned(c, 128) for c in controls])
    rptr = (ctypes.c_void_p * 2)(*[aligned(r, 16) for r in receives])
    partial = torch.randn(elems, device=dev).to(torch.bfloat16)
    out = torch.full((elems,), 7.0, device=dev, dtype=torch.bfloat16)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    stream = torch.cuda.current_stream(dev).cuda_stream

    t0 = time.perf_counter()
    rc = lib.grb_peer_allreduce_bf16(partial.data_ptr(), rptr, cptr, block, 0, 2, out.data_ptr(), elems, 5_000_000,
                                     status.data_ptr(), stream)
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert int(status.item()) & GRB_STATUS_TIMEOUT
    assert 0.004 <= waited < 1.0, f"the wait took {waited:.3f} s for a 5 ms limit"
    assert bool((out == 7.0).all()), "a timed-out reduction must not write its output"

    # what a caller does after a timeout: clear the status word and every rank's control block
    status.zero_()
    for c in controls:
        c.zero_()
    # the second rank's contribution to call 1 (parity 1), placed by the host: data in rank 0's receive block
    # [parity 1][source rank 1], then the flag ready[1] = 1 in rank 0's control block
    theirs = torch.randn(elems, device=dev).to(torch.bfloat16)
    offset0 = aligned(receives[0], 16) - receives[0].data_ptr()
    at = offset0 + (1 * 2 + 1) * block
    receives[0][at:at + 2 * elems].copy_(theirs.view(torch.uint8))
    flag0 = (aligned(controls[0], 128) - controls[0].data_ptr()) // 4
    controls[0][flag0 + 1 * FLAG_STRIDE] = 1
    torch.cuda.synchronize()
    rc = lib.grb_peer_allreduce_bf16(partial.data_ptr(), rptr, cptr, block, 0, 2, out.data_ptr(), elems, 5_000_000,
                                     status.data_ptr(), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = (partial.float() + theirs.float()).to(torch.bfloat16)
    assert torch.equal(out, want)
    # the push went where a peer would read it: rank 1's receive block [parity 1][source rank 0]
    offset1 = aligned(receives[1], 16) - receives[1].data_ptr()
    at = offset1 + (1 * 2 + 0) * block
    assert torch.equal(receives[1][at:at + 2 * elems].view(torch.bfloat16), partial)


def test_a_single_rank_group_never_waits():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from georefine_b200 import _native

    lib = _native.lib()
    dev = torch.device("cuda:0")
    elems = 1024
    control = torch.zeros(int(lib.grb_peer_control_bytes()) // 4 + 64, device=dev, dtype=torch.int32)
    receive = torch.zeros(2 * 4096 + 16, device=dev, dtype=torch.uint8)
    cptr = (ctypes.c_void_p * 1)((control.data_ptr() + 127) // 128 * 128)
    rptr = (ctypes.c_void_p * 1)((receive.data_ptr() + 15) // 16 * 16)
    partial = torch.randn(elems, device=dev).to(torch.bfloat16)
    out = torch.empty(elems, device=dev, dtype=torch.bfloat16)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    for _ in range(3):
        assert lib.grb_peer_allreduce_bf16(partial.data_ptr(), rptr, cptr, 4096, 0, 1, out.data_ptr(), elems, 1_000_000,
                                           status.data_ptr(), torch.cuda.current_stream(dev).cuda_stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.equal(out, partial)
