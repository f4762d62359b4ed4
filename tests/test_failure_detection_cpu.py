"""Failure detection on the host, among CPU ranks: the pre-flight of a tensor-parallel step
(nvfp4_tp.StepGuard) finds a rank that is about to enqueue another token count, a rank that failed
before the step, and a rank that never shows up -- each within its deadline and before anything would
be enqueued -- and the communicator's watchdog entry points check their arguments.  No GPU takes part."""
import os
import socket
import time

import pytest

import nvfp4
import nvfp4_tp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q):
    import datetime
    from torch.distributed import TCPStore
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    guard = nvfp4_tp.StepGuard(store, rank, world, deadline_s=1.5)
    out = []

    def attempt(fn):
        t0 = time.monotonic()
        try:
            fn()
            out.append(("ok", "", time.monotonic() - t0))
        except nvfp4_tp.TpStepError as e:
            out.append(("error", str(e), time.monotonic() - t0))

    attempt(lambda: guard.check(4))                                   # step 0: all agree
    attempt(lambda: guard.check(5 if rank == 1 else 4))               # step 1: rank 1 holds another token count
    if rank == 1:                                                     # step 2: rank 1 hits an exception before the step
        try:
            raise ValueError("weights not loaded")
        except ValueError as e:
            guard.fail(e)
            out.append(("failed", "", 0.0))
    else:
        attempt(lambda: guard.check(4))
    if rank == 1:                                                     # step 3: rank 1 is stuck elsewhere and never reports
        time.sleep(2.0)
        guard.step += 1
        out.append(("absent", "", 0.0))
    else:
        attempt(lambda: guard.check(4))
    attempt(lambda: guard.check(2))                                   # step 4: the group goes on
    q.put((rank, out))
    time.sleep(0.5)                                                   # the master's store outlives the others' last reads


def test_step_guard_among_three_cpu_ranks():
    import torch.multiprocessing as mp
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        assert res[r][0][0] == "ok"
        assert res[r][4][0] == "ok"
    for r in (0, 2):
        kind, msg, dt = res[r][1]
        assert kind == "error" and "rank 1 is about to enqueue 5 tokens" in msg and dt < 1.5
        kind, msg, dt = res[r][2]
        assert kind == "error" and "rank 1 failed before the step" in msg and "weights not loaded" in msg and dt < 1.5
        kind, msg, dt = res[r][3]
        assert kind == "error" and "did not report within 1.5 s" in msg and 1.4 < dt < 5.0
    kind, msg, _ = res[1][1]
    assert kind == "error" and "about to enqueue 4 tokens, this rank 5" in msg


def test_communicator_watchdog_entry_points_check_their_arguments():
    comm = nvfp4_tp.Comm(None, 0, 1)                     # a group of one: no library communicator behind it
    try:
        assert comm.state() == 0
        comm.set_deadline_ms(250)
        with pytest.raises(nvfp4.Nvfp4Error):
            comm.set_deadline_ms(0)
        comm.abort()
        assert comm.state() == -1
    finally:
        comm.close()
    lib = nvfp4_tp.load()
    assert lib.nvfp4_tp_comm_state(None, None) == -1
    assert lib.nvfp4_tp_comm_abort(None) == -1
    assert lib.nvfp4_tp_comm_set_deadline_ms(None, 5) == -1
    with pytest.raises(nvfp4.Nvfp4Error):                # rank outside the world
        nvfp4_tp.Comm(None, 2, 2)
