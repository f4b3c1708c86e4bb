"""Routing-trace replay: the text format of `recordRouteTrace` (RealForwardRunner.swift:1208-1237) read back as a
routing source.  Host logic on CPU; the replay through the routed kernels is a GPU test."""
import numpy as np
import pytest

from nvmai_b200 import route_trace as rt


TEXT = ("0 0 1 2 3 4 5 6 7 8\n"
        "0 1 9 10 11 12 13 14 15 16\n"
        "\n"
        "1 0 1 2 3 4 20 21 22 23\n"
        "1 1 16 15 14 13 12 11 10 9\n")


def test_parse_reads_the_recorded_line_format():
    tr = rt.parse(TEXT, num_experts=32)
    assert len(tr) == 4 and tr.top_k == 8 and tr.layer_ids() == [0, 1]
    pos, ids = tr.layer_rows(0)
    assert pos.tolist() == [0, 1]
    assert ids[1].tolist() == [1, 2, 3, 4, 20, 21, 22, 23]
    st = tr.stats(window=2)
    assert st["reuse"] == pytest.approx((0.5 + 1.0) / 2)        # layer 0 keeps 4 of 8, layer 1 all 8
    assert st["distinct_per_window"] == pytest.approx((12 + 8) / 2)
    assert rt.parse(tr.format(), num_experts=32).experts.tolist() == tr.experts.tolist()


def test_parse_from_file_and_cut_off_last_line(tmp_path):
    path = tmp_path / "trace.txt"
    path.write_text(TEXT + "2 0 1 2 3")          # the writer was stopped in the middle of a line
    tr = rt.parse(path, num_experts=32)
    assert len(tr) == 4


@pytest.mark.parametrize("bad,what", [("0 0 1 2 3 4 5 6 7\n", "fields"), ("0 0 1 2 3 4 5 6 7 x\n", "integer"),
                                      ("0 0 1 2 3 4 5 6 7 32\n", "expert id"), ("0 0 1 1 3 4 5 6 7 8\n", "twice"),
                                      ("0 4 1 2 3 4 5 6 7 8\n", "out of range"), ("-1 0 1 2 3 4 5 6 7 8\n", "out of range")])
def test_parse_rejects_malformed_lines_with_the_line_number(bad, what):
    with pytest.raises(rt.RouteTraceError) as ei:
        rt.parse(TEXT + bad, num_experts=32, num_layers=4)
    assert "line 6" in str(ei.value) and what in str(ei.value)


def test_a_position_recorded_twice_keeps_the_last_record_and_batches_wrap():
    tr = rt.parse(TEXT + "1 0 24 25 26 27 28 29 30 31\n", num_experts=32)
    pos, ids = tr.layer_rows(0)
    assert pos.tolist() == [0, 1] and ids[1].tolist() == list(range(24, 32))
    b = tr.batch(0, first_row=1, rows=3)
    assert b.shape == (3, 8) and b[0].tolist() == ids[1].tolist() and b[1].tolist() == ids[0].tolist()
    with pytest.raises(rt.RouteTraceError):
        tr.batch(7, 0, 1)


def test_synthesized_trace_has_the_requested_reuse():
    tr = rt.synthesize(400, 2, num_experts=256, reuse=0.38, seed=3)
    assert len(tr) == 800
    st = rt.parse(tr.format()).stats()
    assert 0.36 < st["reuse"] < 0.48          # kept experts plus chance repeats of popular ones
    assert all(len(set(r)) == 8 for r in tr.experts.tolist())
    assert rt.synthesize(50, 1, reuse=0.0, zipf=0.0, seed=4).stats()["reuse"] < 0.1


def test_route_log_of_a_step_round_trips_through_the_trace_format():
    """the [layers][rows][top_k] record a resident-kernel step leaves behind, written as `position layer e0..e7`
    lines and parsed back: row r of the step is position first + r"""
    rng = np.random.default_rng(3)
    layers, rows, k, e = 5, 3, 8, 64
    log = np.stack([[rng.choice(e, size=k, replace=False) for _ in range(rows)] for _ in range(layers)]).astype(np.uint32)
    tr = rt.from_route_log(log, 40, num_experts=e)
    text = tr.format()
    assert len(text.splitlines()) == layers * rows
    assert text.splitlines()[0].split()[:2] == ["40", "0"]
    back = rt.parse(text, num_experts=e, top_k=k)
    for l in range(layers):
        pos, ids = back.layer_rows(l)
        assert pos.tolist() == [40, 41, 42]
        np.testing.assert_array_equal(ids, log[l].astype(np.int32))
    one = rt.from_route_log(log[:, 0, :], 7, num_experts=e)          # a one-row step: [layers][top_k]
    assert len(one) == layers and int(one.positions[0]) == 7
