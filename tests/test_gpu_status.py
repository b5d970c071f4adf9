"""A bounded wait that runs out, made on purpose and harmlessly: the self-test kernel waits on an
mbarrier nobody arrives on (nothing in flight) for two million cycles (about a millisecond), gives
up, records its code and exits. The host must see SPARSE_B200_ERR_TIMEOUT with that code, the
context must stay usable and the next real launch must be correct."""
import ctypes

import pytest
import torch

import oracle
from oracle import inputs as gen

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_reports_and_leaves_the_context_usable():
    import sparse_attention_b200_b200 as m
    from sparse_attention_b200_b200 import _lib as L
    lib = L.lib()
    m.device_status()                                       # healthy before
    observed = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    rc = lib.sparse_b200_selftest_bounded_wait(ctypes.c_int64(2_000_000), L.ptr(observed), L.current_stream())
    assert rc == 0
    torch.cuda.synchronize()                                # the kernel ended by itself
    assert observed.tolist() == [0, 1]                      # the wait gave up; the other warp saw the abort flag
    rc = lib.sparse_b200_check_status()
    assert rc == L.ERR_TIMEOUT and b"0x7e57" in lib.sparse_b200_last_error()
    assert lib.sparse_b200_check_status() == 0              # reading it cleared it
    # the Python mirror raises
    L.check(lib.sparse_b200_selftest_bounded_wait(ctypes.c_int64(500_000), None, L.current_stream()))
    with pytest.raises(m.SparseB200Error, match="0x7e57"):
        m.device_status()
    m.device_status()
    # limits are checked on the host
    assert lib.sparse_b200_selftest_bounded_wait(ctypes.c_int64(0), None, None) == L.ERR_INVALID
    assert lib.sparse_b200_selftest_bounded_wait(ctypes.c_int64(10**9), None, None) == L.ERR_INVALID
    # the next real launch on the same context is correct
    q, k, v = gen.make_qkv(1, 4, 2, 256, 1024, seed=5)
    ids = gen.make_ids(1, 2, 2, 8, 3, 6)
    out, lse = m.attention(q.cuda(), k.cuda(), v.cuda(), ids.cuda(), return_lse=True)
    torch.cuda.synchronize()
    m.device_status()
    ref_o, ref_l = oracle.gather_attention(q, k, v, ids)
    d = (out.float().cpu() - ref_o).abs()
    assert d.max() <= 2e-2 and d.mean() <= 2e-3
    assert torch.all((lse.cpu() - ref_l).abs() <= 1e-3 * ref_l.abs().clamp_min(1.0))
