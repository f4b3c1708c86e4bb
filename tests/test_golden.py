"""Golden vectors made with the reference's own C kernel (tests/golden/make_golden.py).

CPU tests: the oracle's own arithmetic reproduces them without the reference library (the
fixtures were produced where the reference checkout was present; they travel, it does not).
GPU tests: the CUDA decode and prefill paths reproduce them through the C ABI."""
import ctypes as C
import hashlib
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
for p_ in (ROOT, ROOT / "tests", ROOT / "tests" / "golden"):
    if str(p_) not in sys.path:
        sys.path.insert(0, str(p_))

from nvmai_b200 import synthetic                      # noqa: E402
from nvmai_b200 import format as fmt                  # noqa: E402
from oracle import oracle as orc                      # noqa: E402
import gpu_util as gu                                 # noqa: E402
import make_golden as mg                              # noqa: E402

GOLDEN = ROOT / "tests" / "golden"
LAYER_CASES = [c[0] for c in mg.CASES]


def _load_case(name):
    g = np.load(GOLDEN / f"{name}.npz")
    host, cfg, x = mg.case_inputs(int(g["bits"]), int(g["meta"]), int(g["d"]), int(g["f"]), int(g["experts"]), int(g["rows"]),
                                  int(g["layer_seed"]), int(g["x_seed"]))
    assert mg.digest(host, x) == str(g["sha256"]), "the seeded generator no longer reproduces the fixture's inputs"
    return g, host, cfg, x


def test_reference_kernel_fixture_matches_oracle_gemv():
    g = np.load(GOLDEN / "int4_affine_gemv_96x512.npz")
    rng = np.random.default_rng(int(g["seed"]))
    rows, n = int(g["rows"]), int(g["n"])
    packed, scales, biases = synthetic.affine_tensor(rng, rows, n, 4, fmt.META_BF16)
    x = rng.normal(0.0, 1.0, size=n).astype(np.float32)
    assert hashlib.sha256(packed.tobytes() + scales.tobytes() + biases.tobytes() + x.tobytes()).hexdigest() == str(g["sha256"])
    y = np.zeros(rows, dtype=np.float32)
    orc.lib().orc_affine_gemv_f32(4, fmt.META_BF16, orc.ptr(packed), orc.ptr(scales), orc.ptr(biases), orc.ptr(x), rows, n,
                                  orc.ptr(y))
    # same factoring, different association of the fp32 sums inside a group
    assert np.max(np.abs(y - g["y"])) <= 1e-4 * np.max(np.abs(g["y"]))


@pytest.mark.parametrize("name", LAYER_CASES)
def test_layer_fixture_matches_oracle(name):
    g, host, cfg, x = _load_case(name)
    L, keep = gu.oracle_layer(host, cfg)
    lib = orc.lib()
    for t in range(int(g["rows"])):
        xr = np.ascontiguousarray(x[t])
        idx = np.zeros(8, dtype=np.uint32)
        w16 = np.zeros(8, dtype=np.uint16)
        h2 = np.zeros(cfg.d, dtype=np.float32)
        m = np.zeros(1, dtype=np.float32)
        lib.orc_gpu_layer_decode(C.byref(L), orc.ptr(xr), None, orc.ptr(idx), orc.ptr(w16), orc.ptr(h2), orc.ptr(m))
        assert idx.tolist() == g["idx"][t].tolist()
        assert w16.tolist() == g["w16"][t].tolist()
        cpu = np.zeros(cfg.d, dtype=np.float32)
        lib.orc_cpu_layer_decode(C.byref(L), orc.ptr(xr), orc.ptr(idx), orc.ptr(w16), orc.ptr(cpu), orc.ref_gemv4_ptr())
        assert orc.rel_error(cpu, g["y_cpu"][t]) < 1e-5          # restated GEMV (or the reference's, when present) vs the fixture
        assert orc.rel_error(h2, g["y_cpu"][t]) < 1e-3           # shader-semantics flavour vs the reference CPU path


@pytest.mark.gpu
@pytest.mark.parametrize("name", LAYER_CASES)
def test_cuda_decode_and_prefill_match_layer_fixture(name):
    import torch
    from nvmai_b200 import MoE
    g, host, cfg, x = _load_case(name)
    rows = int(g["rows"])
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    xd = gu.to_dev(x)
    for path in ("decode", "prefill"):
        y = gu.dev_empty(rows * cfg.d, "f32")
        idx = gu.dev_empty(rows * 8, "u32")
        w = gu.dev_empty(rows * 8, "f16")
        if path == "decode":
            moe.layer_decode(0, xd, rows, h2_out=y, out_idx=idx, out_w=w)
        else:
            moe.layer_prefill(0, xd, rows, y_out=y, out_idx=idx, out_w=w)
        moe.synchronize()
        torch.cuda.synchronize()
        assert np.array_equal(gu.from_dev(idx, np.uint32).reshape(rows, 8), g["idx"]), path
        got_w = orc.f16_bits_to_f32(gu.from_dev(w, np.uint16).reshape(rows, 8))
        assert np.max(np.abs(got_w - orc.f16_bits_to_f32(g["w16"]))) < 1e-3, path
        got = y.cpu().numpy().reshape(rows, cfg.d)
        for t in range(rows):
            assert orc.rel_error(got[t], g["y_cpu"][t]) < 1e-3, f"{path} row {t}"
