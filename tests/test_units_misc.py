"""Host-side units: run log and throughput meter, message layout of the peer links, wire forms of channels-last
tensors, key chunking of the fused contrastive loss, parameter routes of a momentum teacher in split placement."""
import pytest
import torch
from torch import nn


def test_throughput_meter_overall_and_recent():
    from tspipe_b200.run_log import ThroughputMeter
    m = ThroughputMeter(window=3)
    assert m.overall() == 0.0 and m.recent() == 0.0
    for i in range(6):
        m.add(100, now=10.0 + i)           # one batch of 100 samples per second
    assert m.samples == 600 and m.batches == 6
    assert m.overall(now=16.0) == pytest.approx(100.0)
    assert m.recent() == pytest.approx(100.0)
    m.add(400, now=16.0)                   # a burst shows in the window, less in the overall rate
    assert m.recent() > m.overall(now=16.0)


def test_run_log_writes_scalars_and_model(tmp_path):
    from tspipe_b200.run_log import RunLog, join_partitions

    class FakePipe:
        def state_dicts(self):
            return ({0: {"a.weight": torch.ones(2)}, 1: {"b.weight": torch.zeros(3)}}, {0: {"a.weight": torch.ones(2) * 2}})
    lin = nn.Linear(2, 2)
    opt = torch.optim.SGD(lin.parameters(), lr=0.1)
    log = RunLog(str(tmp_path), tensorboard=False)
    log.scalar("loss", 1.5, 1)
    log.scalar("loss", 1.25, 2)
    path = log.save_final(FakePipe(), opt)
    log.close()
    rows = (tmp_path / "scalars.csv").read_text().splitlines()
    assert rows[0] == "wall_time,step,tag,value" and rows[1].endswith(",1,loss,1.5") and len(rows) == 3
    sd = torch.load(path, weights_only=False)
    assert list(sd["online_network_state_dict"]) == ["a.weight", "b.weight"]
    assert torch.equal(sd["target_network_state_dict"]["a.weight"], torch.full((2,), 2.0))
    assert "param_groups" in sd["optimizer_state_dict"]
    with pytest.raises(KeyError):
        join_partitions({0: {"k": torch.ones(1)}, 1: {"k": torch.ones(1)}})
    off = RunLog(str(tmp_path / "none"), enabled=False)
    off.scalar("loss", 1.0, 1)
    assert off.save_final(FakePipe(), opt) is None and not (tmp_path / "none").exists()


def test_peer_link_message_layout_is_aligned_and_ordered():
    from tspipe_b200.comm.peer_link import _layout, _nbytes
    specs = [((3, 5), torch.bfloat16), ((), torch.float32), ((7,), torch.int64), ((0, 4), torch.float32)]
    offs, need = _layout(specs)
    assert all(o % 256 == 0 for o in offs) and need % 256 == 0
    for (shape, dtype), a, b in zip(specs, offs, offs[1:] + [need]):
        assert b - a >= _nbytes(shape, dtype)
    assert _layout([]) == ([], 256)


@pytest.mark.parametrize("channels_last", [False, True])
def test_wire_form_round_trip(channels_last):
    from tspipe_b200.comm.links import wire_empty, wire_form
    x = torch.randn(2, 6, 3, 5).contiguous(memory_format=torch.channels_last)
    w = wire_form(x, channels_last)
    assert w.is_contiguous()
    if channels_last:
        assert w.data_ptr() == x.data_ptr() and w.shape == (2, 3, 5, 6)          # a view, no transpose
    buf, t = wire_empty(tuple(x.shape), x.dtype, None, channels_last)
    buf.copy_(w)
    assert t.shape == x.shape and torch.equal(t, x)
    assert t.is_contiguous(memory_format=torch.channels_last) == channels_last or not channels_last
    v = torch.randn(4, 9)
    assert wire_form(v, channels_last) is v


def test_contrastive_loss_key_chunks():
    from tspipe_b200.ops import gemm
    assert gemm.nce_key_chunks(4096, 4096) == 4            # 32 query tiles x 4 chunks = 128 CTAs
    assert gemm.nce_key_chunks(128, 128) == 1              # one key tile pair cannot be split
    assert gemm.nce_key_chunks(4096, 4160) == 1            # keys do not divide into 128-row chunks
    for n, nk in [(512, 4096), (1024, 1024), (256, 256), (8192, 8192)]:
        c = gemm.nce_key_chunks(n, nk)
        assert c >= 1 and nk % c == 0 and (c == 1 or (nk // c) % 64 == 0 and nk // c >= 128)
    gemm.set_nce_key_split(False)
    try:
        assert gemm.nce_key_chunks(4096, 4096) == 1
    finally:
        gemm.set_nce_key_split(True)


@pytest.mark.parametrize("cut_on,cut_tg", [([2, 2, 1], [3, 1]), ([5], [2, 2]), ([1, 4], [4])])
def test_split_placement_routes_cover_every_teacher_parameter_once(cut_on, cut_tg):
    from tspipe_b200.runtime.ema_plan import build_ema_plans, layout_offsets, split_placement_routes
    torch.manual_seed(0)
    layers = [nn.Linear(8, 8) for _ in range(4)]
    student = layers + [nn.Linear(8, 3)]                    # the last student layer has no teacher counterpart
    teacher = [nn.Linear(8, 8) for _ in range(4)]

    def cut(mods, sizes):
        out, i = [], 0
        for s in sizes:
            out.append(nn.Sequential(*mods[i:i + s]))
            i += s
        return out
    parts_on, parts_tg = cut(student, cut_on), cut(teacher, cut_tg)
    sources, dests = split_placement_routes(build_ema_plans(parts_on, parts_tg), len(parts_tg), len(parts_on))
    flat_s = []
    for part in parts_on:                                   # flat student buffers as the runtime lays them out
        ps = list(part.parameters())
        offs = layout_offsets(ps)
        buf = torch.zeros((offs[-1] + ps[-1].numel() + 63) // 64 * 64 if ps else 64)
        for p, o in zip(ps, offs):
            buf[o:o + p.numel()] = p.detach().reshape(-1)
        flat_s.append(buf)
    want = [p for l in layers for p in l.parameters()]     # teacher parameter i <-> student parameter i
    i = 0
    for jt, part in enumerate(parts_tg):
        ps = list(part.parameters())
        offs = layout_offsets(ps)
        got = torch.full(((offs[-1] + ps[-1].numel() + 63) // 64 * 64,), float("nan"))
        for js, runs in sources[jt].items():
            packed = torch.cat([flat_s[js][o:o + n] for o, n in dests[js][jt]])      # what the student rank sends
            pos = 0
            for t_off, _, n in runs:
                got[t_off:t_off + n] = packed[pos:pos + n]
                pos += n
            assert pos == packed.numel()
        for p, o in zip(ps, offs):
            assert torch.equal(got[o:o + p.numel()], want[i].detach().reshape(-1))
            i += 1
    assert i == len(want)


def test_bench_cuts_and_grids_are_consistent():
    """The benchmark's ResNet-50 cuts cover the 30 student / 26 teacher children, cut both networks at the same
    children (so that the momentum update stays local to a stage), and its pipelined grids use every GPU."""
    import itertools
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    from tspipe_b200.models.resnet import byol_networks
    online, target, predictor = byol_networks("resnet50", 64, 32)
    n_on, n_tg = len(online) + len(predictor), len(target)
    for pp, (on, tg) in bench.BYOL_SPLITS.items():
        assert len(on) == len(tg) == pp and sum(on) == n_on and sum(tg) == n_tg and min(on + tg) >= 1
        assert list(itertools.accumulate(on))[:-1] == list(itertools.accumulate(tg))[:-1]
        assert on[0] >= 4                      # conv1, bn1, relu, maxpool stay together (they run as one fused stem)
    for world in (1, 2, 4, 8):
        for pp, dp, ub in bench.pipeline_grids(world, "byol"):
            assert pp * dp == world and pp in bench.BYOL_SPLITS and (128 * world // dp) % ub == 0
    assert bench.pipeline_grids(8, "moco") == []
