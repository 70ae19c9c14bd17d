"""Runs the reference's own test programs -- built unmodified against this library by
oracle/build_compat.sh -- on the GPU and checks what they print against the reference's known answers
(tests/*/main.cpp in the reference).  Skipped when the binaries were not built (no reference checkout at
build time)."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
COMPAT = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "compat"

EXPECT = {
    "dma_chronological_consistency": ["Memory is equal!"],
    "memcopy": ["1, 2, 3, 4, 5, 6, 7, 8, 9, 10,"],
    "indexing": ["Num functions: 1", 'function "write_float"'],
    "write_float": ["419.314"],
    "dynamic_shared_mem": ["314.314"],
    "kernel_struct_param": ["64"],
    "compute_chronological_consistency": ["Dst compute value (post exec): 2", "Dst dma value (post exec): 1"],
    "stream_events": ["Elapsed: ", "Dst value (post exec): 2"],
    "async_kernels": [],
    "many_kernels_launch": [],
}
FORBID = ["[CUDA ERROR]", "Mismatch", "Not all values were filled"]


@pytest.mark.parametrize("name", sorted(EXPECT))
def test_reference_program(name):
    exe = COMPAT / name / name
    if not exe.exists():
        pytest.skip("compat programs not built (oracle/build_compat.sh needs a reference checkout)")
    res = subprocess.run([str(exe)], cwd=str(exe.parent), capture_output=True, text=True, timeout=600)
    text = res.stdout + res.stderr
    assert res.returncode == 0, text[-2000:]
    for bad in FORBID:
        assert bad not in text, text[-2000:]
    for want in EXPECT[name]:
        assert want in text, text[-2000:]
    if name == "async_kernels":
        # five async launches of the ~100 ms kernel must overlap; five ordered ones must not
        import re

        took = {k: int(v) for k, v in re.findall(r"(Single|5xAsync|5xSync) kernel took: (\d+)ms", text)}
        assert set(took) == {"Single", "5xAsync", "5xSync"}, text[-2000:]
        assert took["5xAsync"] < 0.6 * took["5xSync"], took
        assert took["5xSync"] > 3 * took["Single"] * 0.8, took
