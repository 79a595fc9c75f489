"""Regenerates ``reference_schedule_tables.json`` from a checkout of the reference implementation.

    python tests/data/dump_reference_schedules.py --reference <path to kaist-ina/TSPipe>

Only the reference's scheduler module is imported (`tspipe/scheduler.py:553-596`, ``schedule_generator``); its
``BatchQueue`` dependency is replaced by a stub that never blocks, so no GPU, RPC or model is needed.  Each table is
a list of clocks, each clock a list with one entry per device: ``null`` (idle), ``["OPT", batch]``,
``["B", batch, view, nano-batch]`` or ``["T" | "O", batch, view, microbatch, model_update_ver]``.
Tables: ``tspipe_n{N}_s{S}`` (N stages, S synchronous warm-up batches) and ``gpipe_n{N}_u{U}`` (GPipe emulation
with U microbatches).
"""
import argparse
import json
import os
import sys
import types


def load_scheduler(reference: str):
    class BatchQueue:
        def wait_batch(self, b):
            pass

    bo = types.ModuleType("tspipe.batch_ops")
    bo.BatchQueue = BatchQueue
    pkg = types.ModuleType("tspipe")
    pkg.__path__ = [os.path.join(reference, "tspipe")]
    sys.modules["tspipe"], sys.modules["tspipe.batch_ops"] = pkg, bo
    from tspipe.scheduler import TSPipeScheduler
    return TSPipeScheduler, BatchQueue


def dump(sched_cls, queue_cls, n, clocks, skip=0, gpipe=None):
    cfg = {"gpipe_emulation": {"enabled": gpipe is not None, "num_ubatch": gpipe or 1},
           "optimizer": {"num_skip_initial_staleness": skip}}
    gen = sched_cls(cfg, queue_cls(), n).schedule_generator()
    rows = []
    for _ in range(clocks):
        row = []
        for x in next(gen):
            if x is None:
                row.append(None)
            elif x.optimize:
                row.append(["OPT", x.batch_idx])
            elif x.backprop:
                row.append(["B", x.batch_idx, x.view_idx, x.i])
            else:
                row.append(["T" if x.is_target else "O", x.batch_idx, x.view_idx, x.i, x.model_update_ver])
        rows.append(row)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                  "reference_schedule_tables.json"))
    a = ap.parse_args()
    sched_cls, queue_cls = load_scheduler(a.reference)
    out = {}
    for n, clocks in [(2, 60), (3, 110), (4, 160), (8, 330)]:
        for skip in (0, 1, 2):
            out[f"tspipe_n{n}_s{skip}"] = dump(sched_cls, queue_cls, n, clocks + skip * 40, skip)
    for n, u, clocks in [(1, 2, 30), (2, 3, 60), (4, 4, 90)]:
        out[f"gpipe_n{n}_u{u}"] = dump(sched_cls, queue_cls, n, clocks, 0, u)
    with open(a.out, "w") as f:
        json.dump(out, f, separators=(",", ":"))


if __name__ == "__main__":
    main()
