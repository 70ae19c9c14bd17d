"""Sanitizer builds of the host-only C++ pieces (no CUDA needed): the worker pool behind the pageable-copy
staging ring under AddressSanitizer+UBSan and under ThreadSanitizer, and the stream layer's decision logic
(wait with a deadline against a query that never succeeds, timestamp accumulation, the in-flight write log)."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "cpp" / "copy_pool_test.cpp"
INC = ROOT / "librecuda_b200" / "csrc" / "driverapi"


@pytest.mark.parametrize("san", ["address,undefined", "thread"])
def test_copy_pool_under_sanitizers(tmp_path, san):
    exe = tmp_path / "copy_pool_test"
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={san}", "-fno-omit-frame-pointer", f"-I{INC}",
                            str(SRC), "-o", str(exe), "-pthread"], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    if san == "thread" and "FATAL: ThreadSanitizer: unexpected memory mapping" in run.stderr:
        pytest.skip("ThreadSanitizer cannot run under this kernel's address-space layout")
    assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]
    assert "copy pool ok" in run.stdout


def test_stream_layer_host_logic(tmp_path):
    src = ROOT / "tests" / "cpp" / "host_logic_test.cpp"
    exe = tmp_path / "host_logic_test"
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-Wall", "-Wextra", "-Werror", "-fsanitize=address,undefined",
                            "-fno-omit-frame-pointer", f"-I{INC}", str(src), "-o", str(exe), "-pthread"],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]
    assert "host logic ok" in run.stdout
