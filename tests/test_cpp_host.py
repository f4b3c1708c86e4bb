"""The C++ host mirror (include/nvmai_cuda_moe.hpp): compiles on CPU, and on a GPU its check
program (tests/cpp/host_mirror_check.cpp) drives router, routed phases and the fused decode
entry through the mirror against the oracle."""
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

CUDA = Path("/usr/local/cuda")
BUILD = ROOT / "tests" / "cpp" / "_build"


def _compile() -> Path:
    from nvmai_b200 import build as nb
    nb.build()
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "liboracle.so"], check=True, capture_output=True)
    BUILD.mkdir(exist_ok=True)
    exe = BUILD / "host_mirror_check"
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", f"-I{ROOT / 'include'}", f"-I{CUDA / 'include'}",
           str(ROOT / "tests" / "cpp" / "host_mirror_check.cpp"), "-o", str(exe),
           f"-L{ROOT / 'nvmai_b200'}", "-lnvmai_cuda_moe", f"-L{ROOT / 'oracle'}", "-loracle",
           f"-L{CUDA / 'lib64'}", "-lcudart",
           f"-Wl,-rpath,{ROOT / 'nvmai_b200'}", f"-Wl,-rpath,{ROOT / 'oracle'}", f"-Wl,-rpath,{CUDA / 'lib64'}"]
    subprocess.run(cmd, check=True)
    return exe


@pytest.mark.skipif(shutil.which("g++") is None or not (CUDA / "include" / "cuda_runtime.h").exists(),
                    reason="needs g++ and the CUDA headers")
def test_host_mirror_compiles():
    assert _compile().exists()


@pytest.mark.gpu
def test_host_mirror_check_program():
    exe = _compile()
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASSED" in r.stdout
