"""The plain implementation against the reference's own kernels, both run here on a GPU.

The reference's CUDA sources are compiled unmodified for sm_100 into
``baseline/_ref/libairun_ref_kernels.so`` (``python baseline/reference_kernels.py --build
<reference checkout>``); without that library the tests are skipped, and
``tests/test_reference_golden.py`` still compares the plain implementation with the outputs
these kernels gave when the library was there.
"""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import reference_cases as RC                               # noqa: E402

pytestmark = pytest.mark.gpu

CASES = RC.all_cases()


@pytest.fixture(scope="module")
def kernels():
    rk = RC._rk()
    if not rk.available():
        pytest.skip("the reference's kernels are not built here (baseline/_ref/libairun_ref_kernels.so)")
    return rk.load()


@pytest.mark.parametrize("case", CASES, ids=[c.name for c in CASES])
def test_plain_matches_reference_kernel(kernels, case):
    d = case.make()
    case.check(case.reference(d), case.plain(d))


def test_reference_decode_rows_agree_with_its_single_sequence_path(kernels):
    """Several conversations decoded in one step (the batched path bench.py's reference arm times) give
    what each gives alone."""
    import numpy as np
    import torch
    rk = RC._rk()
    cfg = RC.WHOLE["gqa64"]
    W = {k: v.to("cuda:0") for k, v in RC.whole_model_weights(cfg, 32).items()}
    g = np.random.default_rng(3)
    prompts = [g.integers(0, cfg["vocab_size"], size=n).tolist() for n in (5, 17, 30)]
    nxt = [int(t) for t in g.integers(0, cfg["vocab_size"], size=3)]
    alone = rk.ReferenceDecoder(cfg, W, ctx=64, slots=3, max_batch=32)
    want = []
    for s, p in enumerate(prompts):
        alone.forward(s, p)
        want.append(alone.forward(s, [nxt[s]]).clone())
    together = rk.ReferenceDecoder(cfg, W, ctx=64, slots=3, max_batch=32)
    for s, p in enumerate(prompts):
        together.forward(s, p)
    got = together.decode_rows([(s, nxt[s]) for s in range(3)])
    torch.cuda.synchronize()
    for s in range(3):
        assert float((got[s] - want[s]).abs().max()) <= 2e-4 * float(want[s].abs().max()) + 1e-5
