"""GPU tests of the library's onesweep radix sort through the C ABI (inpc_sort_pairs): exact
agreement with a stable reference sort for ragged sizes, partial bit ranges and skewed keys."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _sort(keys, vals, end_bit):
    from inpc_b200 import _cabi
    n = keys.numel()
    k, v = keys.clone(), vals.clone()
    ka, va = torch.empty_like(k), torch.empty_like(v)
    ws = torch.empty(max(int(_cabi.lib().inpc_sort_workspace_bytes(n)), 256), dtype=torch.uint8, device=DEV)
    alt = C.c_int(0)
    _cabi.check(_cabi.lib().inpc_sort_pairs(k.data_ptr(), ka.data_ptr(), v.data_ptr(), va.data_ptr(), n, end_bit, ws.data_ptr(),
                                           C.byref(alt), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return (ka, va) if alt.value else (k, v)


def _check(keys64, end_bit):
    n = keys64.numel()
    vals = torch.arange(n, device=DEV, dtype=torch.int32)
    k, v = _sort(keys64.to(torch.int32), vals, end_bit)
    masked = keys64 & ((1 << end_bit) - 1)
    _, order = torch.sort(masked, stable=True)
    assert torch.equal(v.to(torch.int64), order)
    assert torch.equal(k.to(torch.int64) & 0xFFFFFFFF, keys64[order])


@pytest.mark.parametrize("n", [0, 1, 2, 31, 8191, 8192, 8193, 100_003, 1 << 20, 3_000_001])
def test_sort_full_keys(n):
    g = torch.Generator(device=DEV).manual_seed(n)
    _check(torch.randint(0, 1 << 32, (n,), generator=g, device=DEV, dtype=torch.int64), 32)


@pytest.mark.parametrize("end_bit", [1, 6, 8, 12, 14, 17, 24])
def test_sort_partial_bits_is_stable(end_bit):
    g = torch.Generator(device=DEV).manual_seed(end_bit)
    # high bits are set on purpose: they must be ignored and carried along unchanged
    _check(torch.randint(0, 1 << 32, (777_777,), generator=g, device=DEV, dtype=torch.int64), end_bit)


def test_sort_skewed_and_constant_keys():
    g = torch.Generator(device=DEV).manual_seed(5)
    n = 1_500_000
    hot = torch.full((n,), 0x40490FDB, device=DEV, dtype=torch.int64)             # one key repeated
    _check(hot, 32)
    few = torch.randint(0, 3, (n,), generator=g, device=DEV, dtype=torch.int64) * 0x01010101
    _check(few, 32)
    depth_like = (torch.rand((n,), generator=g, device=DEV) * 3 + 1.5).view(torch.int32).to(torch.int64)
    _check(depth_like, 32)


def test_sort_full_size_depth_keys():
    """The bench's size: 2^23 pairs with 27 significant bits (three passes), keys larger than L2."""
    g = torch.Generator(device=DEV).manual_seed(23)
    _check(torch.randint(0, 1 << 27, (1 << 23,), generator=g, device=DEV, dtype=torch.int64), 27)


def test_sort_rejects_bad_arguments():
    from inpc_b200 import _cabi
    rc = _cabi.lib().inpc_sort_pairs(None, None, None, None, 10, 40, None, None, None)
    assert rc == -1 and b"end_bit" in _cabi.lib().inpc_last_error()
    rc = _cabi.lib().inpc_sort_pairs(None, None, None, None, 10, 32, None, None, None)
    assert rc == -1
