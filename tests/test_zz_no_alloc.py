"""The allocation-free cross-entropy entry point (tt_softmax_cross_entropy_static) must give
what the handle-based entry gives.  It serves hosts that cannot call cudaMalloc (their own
allocator owns the device heap, or they are only handed a stream and buffers), so it keeps
its per-row scratch in an array inside the library image.  Two calls in a row are checked
because that array is shared and keeps the previous call's contents.  This file sorts last
on purpose: a run that stops at the first failure has then already run everything else."""
import numpy as np
import pytest
import torch

import oracle
from tensotron_b200 import runtime

pytestmark = pytest.mark.gpu


def _case(seed, rows, classes):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy((rng.standard_normal((rows, classes)) * 3).astype(np.float32)).cuda()
    y = torch.from_numpy(rng.integers(0, classes, rows).astype(np.int32)).cuda()
    return x, y


def test_static_cross_entropy_matches_handle_entry_twice(rt):
    # second call has fewer rows than the first: stale slots of the shared array must not leak in
    for seed, rows, classes in ((1, 8192, 10), (2, 1000, 37)):
        x, y = _case(seed, rows, classes)
        d_ref, l_ref = torch.empty_like(x), torch.zeros(1, device="cuda")
        rt.LaunchSoftmaxCrossEntropy(x, y, d_ref, l_ref, rows, classes, 1.0 / rows)
        d_new, l_new = torch.full_like(x, float("nan")), torch.full((1,), float("nan"), device="cuda")
        runtime.softmax_cross_entropy_static(x, y, d_new, l_new, rows, classes, 1.0 / rows)
        torch.cuda.synchronize()
        # same kernels, same fixed summation order: the tolerance of the other cross-entropy
        # tests (1e-5 relative) is met with identical bits
        assert torch.equal(d_new, d_ref)
        assert torch.equal(l_new, l_ref)
        assert abs(l_new.item() - l_ref.item()) <= 1e-5 * max(1.0, abs(l_ref.item()))
        # and against the CPU oracle, like the handle-based entry's own parity test
        lo, do = oracle.cross_entropy(x.cpu().numpy(), y.cpu().numpy())
        assert abs(l_new.item() - lo) <= 1e-5 * max(1.0, abs(lo))
        np.testing.assert_allclose(d_new.cpu().numpy(), do, atol=1e-9, rtol=2e-5)


def test_static_cross_entropy_refuses_oversize_and_bad_arguments(rt):
    x, y = _case(3, 4, 3)
    with pytest.raises(runtime.TensotronGemmError) as e:
        runtime.softmax_cross_entropy_static(x, y, None, None, runtime.STATIC_CE_MAX_ROWS + 1, 3, 1.0)
    assert e.value.status == 6
    with pytest.raises(runtime.TensotronGemmError):
        runtime.softmax_cross_entropy_static(None, y, None, None, 4, 3, 1.0)
