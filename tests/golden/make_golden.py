"""Generates tests/golden/ref_d2d_golden.json from the reference itself.

Needs oracle/_ref/libref_memcopy.so (built by oracle/build_ref.sh from a reference checkout): the
reference's unmodified driverapi/src/memcopy.cpp dispatcher and driverapi/kernels/memcpy/memcpy.cu
kernels compiled for the host.  For every size in SIZES it records the launch plan the reference issues
(kernel, grid, byte offset, n, async flag) and, for sizes it can execute in bounds, the SHA-256 of the
destination buffer after copying the seeded source (seed 1) -- so the oracle and the CUDA path can be
pinned to the reference on machines that have no reference checkout.

    python tests/golden/make_golden.py
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402

MiB = 1 << 20
SIZES = sorted({
    1, 2, 3, 4, 5, 7, 8, 15, 16, 17, 40, 255, 256, 257, 1023, 1024, 1025, 4095, 4096, 4097, 65535, 65536,
    MiB - 1, MiB, MiB + 1, MiB + 3, MiB + 4, MiB + 131, MiB + 4096, MiB + 4099, 2 * MiB, 2 * MiB + 5,
    16 * MiB + 4100, 128 * MiB, 256 * MiB - 4096, 256 * MiB, 256 * MiB + 1, 1024 * MiB + 7, 8192 * MiB,
})
EXEC_LIMIT = 32 * MiB  # sizes the host emulation copies in well under a second


def main():
    if oracle.ref is None:
        raise SystemExit("oracle/_ref/libref_memcopy.so missing: run oracle/build_ref.sh with the reference mounted")
    cases = []
    for size in SIZES:
        execute = size <= EXEC_LIMIT
        src = oracle.random_bytes(size if execute else 1, seed=1)
        dst = np.zeros((size if execute else 1) + 16, np.uint8)
        sync_log = oracle.reference_d2d(dst, src, size, execute=execute, async_=False)
        case = {"size": size, "launches": [list(map(int, l)) for l in sync_log]}
        if execute:
            case["dst_sha256"] = hashlib.sha256(dst[:size].tobytes()).hexdigest()
            case["guard_clean"] = bool((dst[size:] == 0).all())
        async_log = oracle.reference_d2d(np.zeros(1, np.uint8), np.zeros(1, np.uint8), size, execute=False, async_=True)
        case["async_flags_when_async"] = [int(l[5]) for l in async_log]
        cases.append(case)
    out = Path(__file__).with_name("ref_d2d_golden.json")
    out.write_text(json.dumps({"seed": 1, "cases": cases}, indent=1) + "\n")
    print(f"wrote {out} ({len(cases)} cases)")


if __name__ == "__main__":
    main()
