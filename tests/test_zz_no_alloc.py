"""GPU test of inpc_sort_pairs_static, the sort variant for callers that must not allocate device
memory (its scratch is a fixed array inside the library).  Called through the C ABI and compared bit
for bit with the ordinary entry point, on two calls in a row so that the second one meets the first
one's leftovers in the shared array.  Lives in a file pytest collects last."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(fn_name, keys, vals, end_bit, warmed_up=False):
    from inpc_b200 import _cabi
    L = _cabi.lib()
    n = keys.numel()
    k, v = keys.clone(), vals.clone()
    ka, va = torch.empty_like(k), torch.empty_like(v)
    alt = C.c_int(0)
    stream = torch.cuda.current_stream().cuda_stream
    if fn_name == "static":
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        _cabi.check(L.inpc_sort_pairs_static(k.data_ptr(), ka.data_ptr(), v.data_ptr(), va.data_ptr(), n, end_bit, C.byref(alt), stream))
        assert torch.cuda.memory_allocated() == before          # nothing went through torch's allocator either
        if warmed_up:
            # ... and the driver hands out no device memory either (the very first call on a device may load the
            # kernels' module, which is why the comparison starts with the second one)
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_before
        words = (C.c_uint * 4)()
        assert L.inpc_sort_pairs_static_status(stream, words) == 0 and list(words) == [0, 0, 0, 0]
    else:
        ws = torch.empty(max(int(L.inpc_sort_workspace_bytes(n)), 256), dtype=torch.uint8, device=DEV)
        _cabi.check(L.inpc_sort_pairs(k.data_ptr(), ka.data_ptr(), v.data_ptr(), va.data_ptr(), n, end_bit, ws.data_ptr(),
                                      C.byref(alt), stream))
    torch.cuda.synchronize()
    return (ka, va) if alt.value else (k, v)


def test_static_sort_matches_workspace_sort_on_consecutive_calls():
    g = torch.Generator(device=DEV).manual_seed(77)
    cases = [(1 << 20, 32), (300_001, 14), (8193, 32), (1 << 20, 12)]      # the last reuses the array after a full-size call
    for i, (n, end_bit) in enumerate(cases):
        keys = torch.randint(0, 1 << 32, (n,), generator=g, device=DEV, dtype=torch.int64).to(torch.int32)
        vals = torch.arange(n, device=DEV, dtype=torch.int32)
        sk, sv = _run("static", keys, vals, end_bit, warmed_up=i > 0)
        wk, wv = _run("workspace", keys, vals, end_bit)
        assert torch.equal(sk, wk) and torch.equal(sv, wv)                  # integer work: bit-exact
        order = torch.sort(keys.to(torch.int64) & ((1 << end_bit) - 1), stable=True).indices
        assert torch.equal(sv.to(torch.int64), order)


def test_static_sort_rejects_sizes_beyond_its_capacity():
    from inpc_b200 import _cabi
    L = _cabi.lib()
    rc = L.inpc_sort_pairs_static(None, None, None, None, (1 << 20) + 1, 32, None, None)
    assert rc == -5
    msg = L.inpc_last_error().decode()
    assert "capacity" in msg and "1048576" in msg
    assert L.inpc_sort_pairs_static(None, None, None, None, 0, 32, None, None) == 0
