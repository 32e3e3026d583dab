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


def test_lookback_wait_runs_out_and_is_reported():
    """The bounded look-back wait in its failing form: a test hook runs the sort with tile 0 of every pass leaving
    before it publishes and a wait limit of 2^10 polls.  The tiles behind it must give up (microseconds), report
    through the status words of that call, finish with every write inside the buffers, and leave the context
    usable; the next entry point of the same host thread returns INPC_E_DEVICE with the look-back message."""
    from inpc_b200 import _cabi
    L = _cabi.lib()
    n = 100_000                                   # 13 tiles of 8192 pairs
    g = torch.Generator(device=DEV).manual_seed(3)
    keys = torch.randint(0, 1 << 31, (n,), generator=g, device=DEV, dtype=torch.int64).to(torch.int32)
    vals = torch.arange(n, device=DEV, dtype=torch.int32)
    guard = 4096                                  # canaries around every buffer: nothing may be written outside [0, n)
    bufs = [torch.full((n + 2 * guard,), -7, dtype=torch.int32, device=DEV) for _ in range(4)]
    k, ka, v, va = [b[guard:guard + n] for b in bufs]
    k.copy_(keys); v.copy_(vals)
    ws = torch.empty(int(L.inpc_sort_workspace_bytes(n)), dtype=torch.uint8, device=DEV)
    ticket = C.c_longlong(0)
    stream = torch.cuda.current_stream().cuda_stream
    _cabi.check(L.inpc_debug_sort_lookback_timeout(k.data_ptr(), ka.data_ptr(), v.data_ptr(), va.data_ptr(), n, 16, ws.data_ptr(),
                                                   C.byref(ticket), stream))
    torch.cuda.synchronize()                      # returns: nothing hangs
    assert ticket.value > 0 and ticket.value == L.inpc_last_call_ticket()
    words = (C.c_uint * 4)()
    assert L.inpc_call_status(ticket.value, words) == -4          # INPC_E_DEVICE
    assert words[0] == 1 and b"predecessor tile" in L.inpc_last_error()
    for b in bufs:                                # no write left its buffer
        assert bool((b[:guard] == -7).all()) and bool((b[guard + n:] == -7).all())
    # the failure also surfaces at this thread's next call, once
    k2, v2 = keys.clone(), vals.clone()
    alt = C.c_int(0)
    rc = L.inpc_sort_pairs(k2.data_ptr(), torch.empty_like(k2).data_ptr(), v2.data_ptr(), torch.empty_like(v2).data_ptr(), n, 16,
                           ws.data_ptr(), C.byref(alt), stream)
    assert rc == -4 and b"inpc_debug_sort_lookback_timeout" in L.inpc_last_error()
    # ... and the library works again afterwards
    _check(keys.to(torch.int64) & 0xFFFFFFFF, 16)
    assert L.inpc_call_status(L.inpc_last_call_ticket(), None) == 0
