"""The bounds-checking build (libfkb200_check.so) as the stand-in for a memory checker.

`python -m fusedkernellibrary_b200.build --check` compiles the same sources with -DFKB_CHECK_BOUNDS: every access of a
kernel to a source image, to a destination (row by row, so that the padding between rows counts as outside) and to
shared memory is compared with what the block's plane allows before it is made; an access outside is skipped and the
plan's status word reports it (FKB_ERR_DEVICE_BOUNDS).  Nothing in it traps or faults.  The small cases - 1x1, odd
widths, pitches, crops on the image edge, empty regions, column tiles, ragged segment ends, every staged body - run
through it in a child process (tests/checked_build_runner.py), must be bit-exact and must not trip the checker; with
the test-only option that hides the last rows of a destination from the checker the same plans must report it.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from fusedkernellibrary_b200 import abi

ROOT = Path(__file__).resolve().parent.parent


def test_the_checking_build_exports_the_same_entry_points():
    if not abi.CHECK_LIB_PATH.exists():
        pytest.skip("libfkb200_check.so not built (python -m fusedkernellibrary_b200.build --check)")
    import ctypes as C
    lib = C.CDLL(str(abi.CHECK_LIB_PATH))
    for name in abi.EXPORTS:
        assert hasattr(lib, name), name
    assert lib.fkb_debug_bounds_checked() == 1
    assert abi.load_library().fkb_debug_bounds_checked() == 0


@pytest.mark.gpu
def test_small_cases_are_clean_under_the_checking_build():
    if not abi.CHECK_LIB_PATH.exists():
        pytest.skip("libfkb200_check.so not built (python -m fusedkernellibrary_b200.build --check)")
    env = dict(os.environ, FKB200_LIBRARY=str(abi.CHECK_LIB_PATH), PYTHONPATH=str(ROOT))
    r = subprocess.run([sys.executable, "-m", "tests.checked_build_runner"], cwd=str(ROOT), env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    assert "cases clean under the bounds-checking build" in r.stdout
    assert "5 of 5 plans with hidden rows reported FKB_ERR_DEVICE_BOUNDS" in r.stdout, r.stdout[-2000:]
