"""Schedule goldens and structural properties.

``tests/data/reference_schedule_tables.json`` holds clock-by-clock tables dumped from the reference generator
(`tspipe/scheduler.py:553-596`) by ``tests/data/dump_reference_schedules.py`` (it imports only the reference's
scheduler module, with a non-blocking stub for its batch queue).

One deliberate deviation: in the synchronous warm-up batches (``num_skip_initial_staleness``) the reference runs U
backward items per view (`tspipe/scheduler.py:51-121`), this generator 2U nano-batches as in every other batch;
the comparison below therefore leaves the backward items of those batches out."""
import json
import os

import pytest
from hypothesis import given, settings, strategies as st

from tspipe_b200.schedule import (OpKind, ScheduleSpec, check_programs, device_program, simulate,
                                  steady_state_period)

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "data", "reference_schedule_tables.json")))


def _ref_columns(table, n):
    cols = [[] for _ in range(n)]
    for row in table:
        for j, c in enumerate(row):
            if c is not None:
                cols[j].append(tuple(c[:4]) if c[0] != "OPT" else ("OPT", c[1]))
    return cols


def _mine(op):
    if op.kind == OpKind.OPT:
        return ("OPT", op.batch)
    return (op.kind.name, op.batch, op.view, op.ub)


@pytest.mark.parametrize("n", [2, 3, 4, 8])
@pytest.mark.parametrize("skip", [0, 1, 2])
def test_device_order_matches_reference(n, skip):
    cols = _ref_columns(GOLD[f"tspipe_n{n}_s{skip}"], n)
    spec = ScheduleSpec(n_stages=n, skip_staleness=skip)
    for j in range(n):
        # the reference's synchronous warm-up batches use U backward pieces instead of 2U: compare
        # everything but the backward items of those batches
        ref = [c for c in cols[j] if not (c[0] == "B" and c[1] <= skip)]
        gen = device_program(spec, j)
        mine = []
        while len(mine) < len(ref):
            op = next(gen)
            if op.kind == OpKind.LOSS or (op.kind == OpKind.B and op.batch <= skip):
                continue
            mine.append(_mine(op))
        # the dump is cut at an arbitrary clock: compare the common prefix minus the ragged tail
        k = len(ref) - 2 * n
        assert mine[:k] == ref[:k], f"stage {j}"


@pytest.mark.parametrize("n,u", [(1, 2), (2, 3), (4, 4)])
def test_gpipe_emulation_matches_reference(n, u):
    cols = _ref_columns(GOLD[f"gpipe_n{n}_u{u}"], n)
    spec = ScheduleSpec(n_stages=n, n_ubatch=u, gpipe=True)
    for j in range(n):
        gen = (op for op in device_program(spec, j) if op.kind != OpKind.LOSS)
        k = len(cols[j]) - 2 * n
        mine = [_mine(next(gen)) for _ in range(k)]
        assert mine == cols[j][:k]


@pytest.mark.parametrize("n", [2, 3, 4, 8])
def test_clock_table_matches_reference_steady_state(n):
    """The greedy unit-time simulation reproduces the reference table clock for clock."""
    ref = GOLD[f"tspipe_n{n}_s0"]
    spec = ScheduleSpec(n_stages=n)
    table = simulate(spec, 10)
    for c in range(min(len(ref), len(table)) - 4 * n):
        for j in range(n):
            r, m = ref[c][j], table[c][j]
            if r is None:
                assert m is None, (c, j)
            else:
                assert m is not None, (c, j, r)
                assert _mine(m) == (tuple(r[:4]) if r[0] != "OPT" else ("OPT", r[1])), (c, j)


@pytest.mark.parametrize("n", [2, 3, 4, 8])
def test_steady_state_is_bubble_free(n):
    period, busy = steady_state_period(ScheduleSpec(n_stages=n))
    assert period == 8 * (n - 1) + 1
    assert busy == 1.0


@settings(max_examples=60, deadline=None)
@given(n=st.integers(1, 6), u=st.integers(1, 6), split=st.integers(1, 3), kd=st.booleans(),
       skip=st.integers(0, 2), gpipe=st.booleans())
def test_program_properties(n, u, split, kd, skip, gpipe):
    spec = ScheduleSpec(n_stages=n, n_ubatch=u, bwd_split=split, kd=kd, skip_staleness=skip, gpipe=gpipe)
    check_programs(spec, 5)
    simulate(spec, 4)          # raises on deadlock


def test_kd_filter_matches_reference_rule():
    """KD keeps teacher view 1 / student view 0 of the SSL order (`tspipe/tspipe.py:310-320`)."""
    for n in (2, 3, 4):
        ssl = ScheduleSpec(n_stages=n)
        kd = ScheduleSpec(n_stages=n, kd=True)
        for j in range(n):
            a = [op for op in device_program(ssl, j, 1, 4)
                 if op.kind in (OpKind.OPT, OpKind.LOSS) or (op.view == 1) == (op.kind == OpKind.T)]
            b = list(device_program(kd, j, 1, 4))
            assert [(o.kind, o.batch, o.view, o.ub) for o in a] == [(o.kind, o.batch, o.view, o.ub) for o in b]
