"""Host-side helpers of bench.py that need no GPU: the byte counts the roofline uses and the reduction of the resident
kernels' per-block timer marks."""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import bench  # noqa: E402
from nvmai_b200 import format as fmt  # noqa: E402


def test_algorithmic_bytes_match_the_blob_layout():
    off, stride = fmt.expert_offsets(bench.D, bench.F, 4)
    assert bench.expert_bytes(4) == stride == 1769472
    assert bench.expert_bytes(8) == fmt.expert_offsets(bench.D, bench.F, 8)[1] == 3342336
    # 8 routed + 1 shared expert, the fp16 router, the gate row, x (fp16) and y (fp32)
    want = 9 * 1769472 + bench.E * bench.D * 2 + bench.D * 2 + bench.D * 2 + bench.D * 4
    assert bench.layer_bytes(4) == want == 16990208


def test_block_trace_summary_reduces_marks_per_layer():
    layers, blocks = 6, 5
    tr = np.zeros((layers, blocks, 16), dtype=np.uint64)
    base = 1_000_000
    for l in range(layers):
        for b in range(blocks):
            t0 = base + l * 20_000 + b * 100             # a layer every 20 us, blocks 0.1 us apart
            tr[l, b, 0] = t0
            tr[l, b, 1] = t0 + 1_000
            tr[l, b, 9] = t0 + 15_000
    out = bench.block_trace_summary(tr, 1, "synthetic marks")
    marks = out["us_after_first_input_row_min_median_max"]
    assert marks["input row normalised"] == [0.0, 0.2, 0.4]
    assert marks["router logits stored"] == [1.0, 1.2, 1.4]
    assert marks["block output stored"] == [15.0, 15.2, 15.4]
    assert "top-k done" not in marks                      # a mark nobody wrote is left out
    assert out["layer_period_us_median"] == 20.0
    assert set(out["blocks_most_often_last"]["block output stored"][:3]) == {2, 3, 4}      # the three last of every layer
