"""A C++ program that uses the additive libreCu* entry points exactly as a consumer of the library would
(#include <librecuda.h>, link `driverapi`): compiled and linked here without a GPU, run on the GPU."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests" / "cpp" / "additive_api_test.cpp"
LIBDIR = ROOT / "librecuda_b200" / "lib"


def _build(tmp_path) -> Path:
    assert (LIBDIR / "libdriverapi.so").exists(), "build the library first: python -m librecuda_b200.build"
    exe = tmp_path / "additive_api_test"
    build = subprocess.run(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-O1", f"-I{ROOT / 'include'}", str(SRC),
                            f"-L{LIBDIR}", "-ldriverapi", f"-Wl,-rpath,{LIBDIR}", "-o", str(exe)],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    return exe


def test_consumer_program_compiles_and_links_against_the_headers(tmp_path):
    assert _build(tmp_path).exists()


@pytest.mark.gpu
def test_consumer_program_runs(tmp_path):
    exe = _build(tmp_path)
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, (run.stdout + run.stderr)[-3000:]
    assert "additive API ok" in run.stdout
