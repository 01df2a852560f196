"""Builds and runs the torch-free C++ checks of the C ABI (tests/standalone/*.cu): plain host programs
linking libmgr_b200.so, in the manner of the reference's stand-alone test (rmsnorm_standalone.cu) -- one
for RMSNorm forward/backward, one for a whole SwiGLU MLP forward+backward. Needs nvcc and a GPU."""
import shutil
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("program", ["rmsnorm_abi_check", "swiglu_abi_check"])
def test_standalone_cpp_program_passes(built_lib, tmp_path, program):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("nvcc not available")
    exe = tmp_path / program
    lib_dir = ROOT / "mgrrmsnorm_b200" / "lib"
    cmd = [nvcc, "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", f"-I{ROOT / 'include'}",
           str(ROOT / "tests" / "standalone" / f"{program}.cu"), str(ROOT / "oracle" / "mgr_oracle.c"),
           f"-L{lib_dir}", "-lmgr_b200", "-Xlinker", f"-rpath={lib_dir}", "-o", str(exe)]
    build = subprocess.run(cmd, capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "Validation PASSED" in run.stdout
