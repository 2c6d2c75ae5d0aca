"""CPU suite: the C-ABI library loads, exports every declared symbol, and its host-only
logic behaves like the reference's (no compute call is made without a GPU)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from tensotron_b200 import runtime


def test_library_exports_every_declared_symbol(gemm_lib):
    header = open(os.path.join(ROOT, "include", "tensotron_gemm.h")).read()
    declared = re.findall(r"TT_API\s+(?:const\s+char\*|int|size_t)\s+(tt_\w+)\s*\(", header)
    assert len(declared) >= 18
    for name in declared:
        assert getattr(gemm_lib, name) is not None, name
    assert sorted(declared) == sorted(runtime.EXPORTS)
    assert b"sm_100a" in gemm_lib.tt_version()


def test_broadcast_batch_matches_reference_rules(gemm_lib):
    # BASELINE bmm config: A [32,1,384,256] x B [1,16,256,192]
    dims, aBs, bBs = runtime.broadcast_batch([32, 1], [98304, 98304], [1, 16], [786432, 49152])
    assert dims == [32, 16] and aBs == [98304, 0] and bBs == [0, 49152]
    # rank promotion: (4,2,3) @ (3,5) -> b has no batch axes
    assert runtime.broadcast_batch([4], [6], [], []) == ([4], [6], [0])
    assert runtime.broadcast_batch([2, 1], [6, 6], [2], [15]) == ([2, 2], [6, 0], [0, 15])
    with pytest.raises(runtime.TensotronGemmError):
        runtime.broadcast_batch([3], [6], [4], [15])


def test_shard_range_is_the_ceil_block_split(gemm_lib):
    for total, world in ((16384, 8), (32, 3), (5, 8), (0, 2), (1000, 7)):
        per = -(-total // world)
        covered = 0
        for rank in range(world):
            s, c = runtime.shard_range(total, world, rank)
            assert s == min(total, rank * per) and c == min(total, s + per) - s
            covered += c
        assert covered == total
    with pytest.raises(runtime.TensotronGemmError):
        runtime.shard_range(10, 2, 2)


def test_null_handle_and_bad_arguments_are_status_codes(gemm_lib):
    assert gemm_lib.tt_matmul(None, None, None, None, None, 1, 1, 1, 1, 1, 1, 1) == 1
    assert gemm_lib.tt_destroy(None) == 1
    assert gemm_lib.tt_set_math_mode(None, 0) == 1
    assert gemm_lib.tt_create(0, 0, None) == 1
    assert gemm_lib.tt_last_error(None) == b"null handle"


def test_create_without_device_fails_cleanly(gemm_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = ctypes.c_void_p()
    assert gemm_lib.tt_create(0, 0, ctypes.byref(h)) != 0
    assert not h.value
    with pytest.raises(runtime.TensotronGemmError):
        runtime.TensorRuntime(0)


def test_missing_library_is_loud(tmp_path):
    with pytest.raises(ImportError):
        runtime.load_library(str(tmp_path / "nope.so"))
