"""Runs the small parity cases through the bounds-checking build of the library (libfkb200_check.so).

Started by tests/test_gpu_checked_build.py as a child process with FKB200_LIBRARY pointing at the checking build, so
that the ordinary library of the parent test process stays the one that is loaded there.  Every kernel access to a
source image, a destination or shared memory is compared with what the block's plane allows before it is made; an
access outside would be skipped and reported (FKB_ERR_DEVICE_BOUNDS), never made.  The run passes when every case is
bit-exact against the plain-C checker AND no access was refused; then, with the test-only option that makes the
checker treat the last rows of every destination as outside, the same plans must report the refusal, leave those rows
untouched, and fault nothing.  Prints one line per case and a summary; exit code 0 on success.
"""
import sys

import numpy as np
import torch

from fusedkernellibrary_b200 import abi
from oracle import port
from tests import cases as tc
from tests.test_gpu_parity import DeviceArrays


def main() -> int:
    lib = abi.load_library()
    lib.fkb_debug_bounds_checked.restype = int
    if lib.fkb_debug_bounds_checked() != 1:
        print("the loaded library is not the bounds-checking build")
        return 2
    port.build()
    oracle = port
    failures = 0
    cases = tc.small_cases()
    for case in cases:
        expected = {k: v.copy() for k, v in tc.run_on_host(case, oracle).items()}
        dev = DeviceArrays(case)
        plan = abi.DevicePlan(case.build(dev.ptr))
        plan.launch()
        try:
            status = plan.check()
        except abi.FkbError as e:
            print(f"FAIL {case.name}: {e}")
            failures += 1
            plan.destroy()
            continue
        bad = [k for k, v in case.outputs.items() if not np.array_equal(tc.bits(dev.download(k, v)), tc.bits(expected[k]))]
        if status != 0 or bad:
            print(f"FAIL {case.name}: status {status}, differing outputs {bad}")
            failures += 1
        plan.destroy()
    print(f"{len(cases) - failures} of {len(cases)} cases clean under the bounds-checking build")

    # the checker itself: hide the last 2 rows of every destination; stores into them are refused and reported
    refused = 0
    probe = [c for c in cases if c.name in ("c1_dense_aligned", "c3_small", "c2_readme", "c4_exact3", "g3_saturate_u8")]
    for case in probe:
        dev = DeviceArrays(case, fill=0xAB)
        plan = abi.DevicePlan(case.build(dev.ptr))
        plan.set_option(abi.PLAN_TEST_SHRINK_BOUNDS, 2)
        plan.launch()
        try:
            plan.check()
            print(f"FAIL {case.name}: hidden rows were written without a report")
            failures += 1
        except abi.FkbError as e:
            if e.status == abi.ERR_DEVICE_BOUNDS:
                refused += 1
            else:
                print(f"FAIL {case.name}: {e}")
                failures += 1
        plan.destroy()
    torch.cuda.synchronize()
    print(f"{refused} of {len(probe)} plans with hidden rows reported FKB_ERR_DEVICE_BOUNDS")
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
