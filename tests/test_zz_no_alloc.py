"""The allocation-free dispatch sort (`imx_moe_sort_static`) against the regular
entry point (`imx_moe_sort`).

Some hosts of this library may not allocate device memory themselves, e.g. an
engine thread whose framework owns the device allocator and enforces a memory
cap, so that every byte has to come from that allocator.  For them the sort's
scratch lives in a fixed array inside the library.  The test drives both entry
points through the C ABI on the same ids, twice in a row (the array keeps the
previous call's contents), and requires bit-identical results; it also checks
that an input beyond the built-in capacity is refused with a message.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from ironmlx_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def _sort(fn_static: bool, ids_dev, e):
    a = ids_dev.numel()
    i32 = dict(dtype=torch.int32, device=ids_dev.device)
    counts, offsets = torch.empty(e, **i32), torch.empty(e + 1, **i32)
    perm, inv = torch.empty(a, **i32), torch.empty(a, **i32)
    lib = _lib.lib()
    if fn_static:
        _lib.check(lib.imx_moe_sort_static(ids_dev.data_ptr(), a, e, counts.data_ptr(), offsets.data_ptr(),
                                           perm.data_ptr(), inv.data_ptr(), ops.stream_ptr()))
    else:
        nb = C.c_size_t(0)
        _lib.check(lib.imx_moe_sort_scratch_bytes(a, e, C.byref(nb)))
        scratch = torch.zeros(max(nb.value, 256), dtype=torch.uint8, device=ids_dev.device)
        _lib.check(lib.imx_moe_sort(ids_dev.data_ptr(), a, e, counts.data_ptr(), offsets.data_ptr(), perm.data_ptr(),
                                    inv.data_ptr(), scratch.data_ptr(), scratch.numel(), ops.stream_ptr()))
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in (counts, offsets, perm, inv)]


def test_static_sort_matches_regular_sort_twice(cuda):
    rng = np.random.default_rng(77)
    # first call: large enough for the multi-block path (uses the scratch); second: different size and
    # expert count, so stale contents of the shared array would show
    for n_assign, e in [(8192 * 8, 256), (20000, 96), (512, 256)]:
        ids = torch.from_numpy(rng.integers(0, e, size=n_assign).astype(np.int32)).to(cuda)
        want = _sort(False, ids, e)
        got = _sort(True, ids, e)
        for w, g in zip(want, got):
            assert np.array_equal(w, g)


def test_static_sort_refuses_oversized_input(cuda):
    ids = torch.zeros(262144 + 1, dtype=torch.int32, device=cuda)
    out = torch.empty(262145, dtype=torch.int32, device=cuda)
    rc = _lib.lib().imx_moe_sort_static(ids.data_ptr(), ids.numel(), 8, out.data_ptr(), out.data_ptr(),
                                        out.data_ptr(), out.data_ptr(), ops.stream_ptr())
    assert rc == _lib.ERR_INVALID and b"exceed the built-in scratch" in _lib.lib().imx_last_error()
