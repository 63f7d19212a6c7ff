"""The plain implementation against stored outputs of the reference's own kernels.

``tests/golden/reference_kernel_outputs.npz`` was written by
``tests/golden/make_reference_kernel_outputs.py`` on a B200 from the reference's CUDA sources
compiled unmodified for sm_100 (see baseline/reference_kernels.py).  Here the plain functions
compute the same cases on the CPU and must agree within each case's bound, so the plain
implementation stays pinned on the reference's code on machines without a GPU.
"""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import reference_cases as RC                               # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernel_outputs.npz")
CASES = RC.all_cases()


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_plain_matches_stored_reference_output(case):
    assert os.path.exists(GOLDEN), "tests/golden/reference_kernel_outputs.npz is part of the repository"
    stored = np.load(GOLDEN)
    got = {k.split("/", 1)[1]: stored[k] for k in stored.files if k.startswith(case.name + "/")}
    assert got, f"no stored output for {case.name}: run tests/golden/make_reference_kernel_outputs.py again"
    case.check(got, case.plain(case.make()))
