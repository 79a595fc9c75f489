"""Shared helpers for the multi-process CPU tests."""
import os
import socket
import sys
import traceback

import torch
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, ret, hard_exit=False):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    try:
        ret[rank] = fn(rank, world, *args)
        if hard_exit:
            # the rank may still own threads blocked in a collective that will never complete (that is what
            # the test provokes); leave without running their destructors
            sys.stdout.flush()
            os._exit(0)
    except BaseException:
        ret[rank] = ("__error__", traceback.format_exc())
        raise


def run_ranks(fn, world, *args, timeout=240, hard_exit=False):
    """Run ``fn(rank, world, *args)`` in ``world`` spawned processes (launcher-style env) and return
    the list of their return values."""
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, ret, hard_exit)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    out = [ret.get(r) for r in range(world)]
    for r, o in enumerate(out):
        if isinstance(o, tuple) and len(o) == 2 and o[0] == "__error__":
            raise AssertionError(f"rank {r} failed:\n{o[1]}")
    assert not alive, "ranks timed out"
    for p in procs:
        assert p.exitcode == 0, f"rank exit code {p.exitcode}"
    return out
