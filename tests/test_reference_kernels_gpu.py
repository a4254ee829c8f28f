"""The reference's own kernels, compiled here and run again, against the committed numbers.

Needs an unmodified copy of the reference's ``cuda/`` folder under ``baseline/_ref`` (or
where ``BINFER_REFERENCE_DIR`` points); without one the test is skipped, and
``tests/test_plain_against_reference_kernels.py`` still holds the plain implementation to
the numbers that an earlier run of these kernels left in ``tests/golden/``.
"""
import importlib.util
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _script():
    path = os.path.join(HERE, "golden", "make_reference_kernel_golden.py")
    spec = importlib.util.spec_from_file_location("make_reference_kernel_golden", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_kernels_give_the_committed_numbers(cuda_device, tmp_path):
    ref_dir = os.environ.get("BINFER_REFERENCE_DIR", os.path.join(ROOT, "baseline", "_ref"))
    if not os.path.exists(os.path.join(ref_dir, "cuda", "kernels", "bf16_kernels.cu")):
        pytest.skip(f"no copy of the reference's kernels under {ref_dir}")
    m = _script()
    lib = m.build(ref_dir, str(tmp_path))
    now = m.run_cases(lib)
    golden = np.load(os.path.join(HERE, "golden", "reference_kernels.npz"))
    assert set(golden.files) == set(now)
    for name in golden.files:
        assert np.array_equal(golden[name], now[name]), f"{name} differs from the committed run"
