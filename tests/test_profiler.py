import csv

from tspipe_b200.profiler import Operation, TSPipeProfiler, profile_semantic


def test_profiler_writes_reference_schema(tmp_path):
    path = tmp_path / "profile_out.csv"
    with TSPipeProfiler(filename=str(path), cuda_events=False) as prof:
        with Operation("compute", 3, 1, 2, True, None, 0):
            pass
        with prof.operation("backward", 3, 0, 5, False, 1):
            pass
        profile_semantic(4, 0, 0, False, None, None, "feed_batch")
    rows = list(csv.reader(open(path)))
    assert rows[0] == TSPipeProfiler.HEADER
    ops = [r[-1] for r in rows[1:]]
    assert ops == ["compute", "compute_finish", "backward", "backward_finish", "feed_batch"]
    assert rows[1][1:5] == ["3", "1", "2", "1"]
    assert float(rows[2][0]) >= float(rows[1][0])
