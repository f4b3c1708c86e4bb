"""The C-ABI library loads without a GPU and exports exactly what the header declares."""
import ctypes as C
import re
from pathlib import Path

import pytest

from nvmai_b200 import _lib, build

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def declared_symbols():
    text = (ROOT / "include" / "nvmai_cuda_moe.h").read_text()
    return re.findall(r"NVMAI_API[^;(]*?\b(nvmai_cuda_moe_\w+)\s*\(", text)


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.PROTOTYPES, f"{name} has no ctypes prototype"
    assert set(_lib.PROTOTYPES) == set(names)


def test_struct_layouts_match_the_reference_abi():
    """MoEExpertOffsets is 9 x u32 = 36 bytes (MoE.swift:4-29 / moe.metal:141-151)."""
    assert C.sizeof(_lib.ExpertOffsets) == 36
    assert C.sizeof(_lib.Config) == 14 * 4
    assert C.sizeof(_lib.AffineTensor) == 24


def test_expert_offsets_without_gpu(lib):
    """CPUExpertFFNTests.swift:56-67 through the product's own offset function."""
    o = _lib.ExpertOffsets()
    assert lib.nvmai_cuda_moe_expert_offsets(2048, 512, 4, C.byref(o)) == 1_769_472
    assert (o.gate_w, o.gate_s, o.up_w, o.down_w) == (0, 524_288, 589_824, 1_179_648)
    assert lib.nvmai_cuda_moe_expert_offsets(2048, 512, 8, C.byref(o)) == 3_342_336


@pytest.mark.parametrize("field,value,code", [
    ("d", 100, _lib.EINVAL),            # D % 64 (MoE.swift:163)
    ("num_experts", 300, _lib.ERANGE),  # <= 256 (MoE.swift:164)
    ("routed_bits", 6, _lib.EINVAL),
    ("top_k", 0, _lib.ERANGE),
    ("max_tokens", 0, _lib.EINVAL),
    ("router_kind", 3, _lib.EINVAL),
])
def test_create_rejects_bad_config_before_touching_the_device(lib, field, value, code):
    cfg = _lib.Config(2048, 512, 512, 256, 8, 4, 4, 0, 0, 0, 0, 0, 1, 1)
    setattr(cfg, field, value)
    err = C.c_int(0)
    assert lib.nvmai_cuda_moe_create(C.byref(cfg), C.byref(err)) is None
    assert err.value == code


def test_error_strings(lib):
    assert lib.nvmai_cuda_moe_error_string(0) == b"ok"
    assert b"range" in lib.nvmai_cuda_moe_error_string(_lib.ERANGE)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.lib()
