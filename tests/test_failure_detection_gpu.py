"""A bounded device-side wait that runs out, made to happen safely: a group of two whose second rank
never pushes.  One GPU, one process; the kernel of "rank 0" pushes its partial sums into both exchange
buffers, polls its own buffer for rank 1's, gives up after its limit (about a second), records 0x701
(wait on rank 1 ran out) in the buffer's status word and returns.  Nothing faults, nothing hangs: the
context stays usable and the next call on the handle gives the right answer."""
import numpy as np
import pytest

import nvfp4
import oracle_binding as ob
import util

pytestmark = pytest.mark.gpu

SLOTS_OFF = 4096          # layout of an exchange buffer: status word at 0, pairs from 4096 (include/nvfp4_b200.h)


@pytest.mark.parametrize("M", [1, 12])                   # the 8-token GEMV and the 9..16-token one
def test_peer_that_never_pushes_runs_the_wait_out(handle, M):
    import time
    import torch
    N, K = 512, 1024
    packed, scale = util.make_weight(N, K, seed=5)
    A = util.make_bf16((M, K), seed=6)
    slot_pairs = 16 * N
    nbytes = SLOTS_OFF + 2 * 2 * slot_pairs * 8
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    dC = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
    torch.cuda.synchronize()
    t0 = time.monotonic()
    st = handle.linear_reduce_peers(util.to_dev(A), M, util.to_dev(packed), util.to_dev(scale), 1.0, N, K, dC, bufs, 0, slot_pairs,
                                    check=False)
    assert st == 0                                        # the launch itself is fine
    torch.cuda.synchronize()                              # ... and the kernel returns by itself
    dt = time.monotonic() - t0
    status = int(bufs[0][:4].view(torch.int32).item())
    assert status in (0x701, 0x711), hex(status)          # rank 1's pairs never came (8-token / wide kernel)
    assert 0.3 < dt < 10.0
    assert int(bufs[1][:4].view(torch.int32).item()) == 0
    # rank 0's own pairs did arrive in rank 1's buffer: the push side worked
    pushed = bufs[1][SLOTS_OFF:SLOTS_OFF + 2 * 2 * slot_pairs * 8].view(torch.int32).view(-1, 2)
    assert int((pushed[:, 1] == 1).sum().item()) == M * N
    # the context is intact: an ordinary call on the same handle
    dC2 = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    handle.linear(util.to_dev(A), M, util.to_dev(packed), util.to_dev(scale), 1.0, N, K, dC2)
    torch.cuda.synchronize()
    assert ob.rel_frobenius(util.to_host_u16(dC2), ob.linear(A, packed, scale, 1.0, mode=ob.GEMV)) <= 1e-3
    assert handle.device_status() == 0


def test_group_of_two_on_one_gpu_completes_when_both_push(handle):
    """The same set-up with both ranks' kernels launched one after the other (each pushes first, polls
    afterwards: rank 0's kernel runs out its wait unless rank 1's pairs are there, so rank 1 goes first
    here, gives up, and rank 0 then finds everything and finishes) -- the positive counterpart, which
    also shows that the status word is per buffer."""
    import torch
    M, N, K = 2, 512, 1024
    packed, scale = util.make_weight(N, K, seed=7)
    A = [util.make_bf16((M, K), seed=8 + r) for r in range(2)]
    slot_pairs = 16 * N
    nbytes = SLOTS_OFF + 2 * 2 * slot_pairs * 8
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    outs = [torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda") for _ in range(2)]
    dp, ds = util.to_dev(packed), util.to_dev(scale)
    handle.linear_reduce_peers(util.to_dev(A[1]), M, dp, ds, 1.0, N, K, outs[1], bufs, 1, slot_pairs)     # gives up on rank 0
    handle.linear_reduce_peers(util.to_dev(A[0]), M, dp, ds, 1.0, N, K, outs[0], bufs, 0, slot_pairs)     # finds both
    torch.cuda.synchronize()
    assert int(bufs[1][:4].view(torch.int32).item()) == 0x700
    assert int(bufs[0][:4].view(torch.int32).item()) == 0
    want = ob.bf16_to_f32(ob.linear(A[0], packed, scale, 1.0, mode=ob.GEMV)) + ob.bf16_to_f32(ob.linear(A[1], packed, scale, 1.0, mode=ob.GEMV))
    got = ob.bf16_to_f32(util.to_host_u16(outs[0]))
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 5e-3      # the oracle's partials are rounded to BF16 here, the kernel's are not
