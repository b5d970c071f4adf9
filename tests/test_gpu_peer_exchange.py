"""The peer-memory merge of the cross-GPU KV split (csrc/peer_exchange.cu), as far as one GPU shows it:
the merge kernel over R separate partial buffers against the single-buffer Combine kernel (bit-identical),
the flag signalling, a wait that runs out by construction (a flag nothing sets: the kernel records a status
code and returns, the context stays usable), and the whole `KVSplit.run_peer` step for a group of one rank.
The two-GPU run is in test_gpu_multi.py."""
import ctypes
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def sp():
    import sparse_attention_b200_b200 as m
    return m


def _partials(ranks, rows, seed):
    g = torch.Generator().manual_seed(seed)
    o = torch.randn((ranks, rows, 128), generator=g).to(torch.bfloat16)
    l = torch.randn((ranks, rows), generator=g) * 3
    l[0, 5] = float("-inf")                       # one rank without keys for a row
    l[:, 9] = float("-inf")                       # a row without keys anywhere
    o[:, 9] = float("nan")                        # ... whose partials are garbage
    o[0, 5] = float("nan")
    return o.cuda(), l.cuda()


@pytest.mark.parametrize("ranks", [1, 2, 4, 8])
def test_merge_over_separate_buffers_equals_the_combine_kernel(ranks):
    from sparse_attention_b200_b200 import _lib
    m = sp()
    rows = 1000                                    # not a multiple of the 16 rows of a CTA
    o, l = _partials(ranks, rows, 40 + ranks)
    from sparse_attention_b200_b200.sharding import _gpu_combine
    ref_o, ref_l = _gpu_combine(o, l)              # sparse_b200_combine on one rank-major buffer
    parts = [o[r].clone() for r in range(ranks)]   # R separate allocations, as R ranks would hold them
    lses = [l[r].clone() for r in range(ranks)]
    flags = torch.zeros(32, dtype=torch.int32, device="cuda")
    L = _lib.lib()
    arr = ctypes.c_void_p * ranks
    targets = arr(*[flags.data_ptr() + 4 * r for r in range(ranks)])
    _lib.check(L.sparse_b200_peer_signal(targets, ranks, 7, _lib.current_stream()))
    out = torch.full((rows, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    out_lse = torch.full((rows,), float("nan"), device="cuda")
    _lib.check(L.sparse_b200_combine_peer(
        arr(*[p.data_ptr() for p in parts]), arr(*[x.data_ptr() for x in lses]), _lib.ptr(flags), 7, 1000,
        _lib.ptr(out), _lib.ptr(out_lse), ctypes.c_int64(rows), ranks, _lib.current_stream()))
    torch.cuda.synchronize()
    m.device_status()
    assert flags[:ranks].tolist() == [7] * ranks
    assert torch.equal(out.view(torch.int16), ref_o.view(torch.int16))
    assert torch.equal(out_lse.view(torch.int32), ref_l.view(torch.int32))
    assert torch.isfinite(out.float()).all() and out_lse[9] == float("-inf") and (out[9] == 0).all()


def test_a_wait_that_nothing_satisfies_gives_up_with_a_status_code():
    from sparse_attention_b200_b200 import _lib
    m = sp()
    L = _lib.lib()
    flags = torch.zeros(32, dtype=torch.int32, device="cuda")
    _lib.check(L.sparse_b200_peer_wait(_lib.ptr(flags), 2, 1, 30, _lib.current_stream()))      # 30 ms
    torch.cuda.synchronize()
    with pytest.raises(m.SparseB200Error, match="0xb00"):
        m.device_status()
    # the merge kernel: flag 0 is there, flag 1 never comes: every CTA returns without writing
    o, l = _partials(2, 64, 3)
    flags[0] = 1
    out = torch.full((64, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    arr = ctypes.c_void_p * 2
    _lib.check(L.sparse_b200_combine_peer(
        arr(o[0].data_ptr(), o[1].data_ptr()), arr(l[0].data_ptr(), l[1].data_ptr()), _lib.ptr(flags), 1, 30,
        _lib.ptr(out), None, ctypes.c_int64(64), 2, _lib.current_stream()))
    torch.cuda.synchronize()
    with pytest.raises(m.SparseB200Error, match="0xb11"):
        m.device_status()
    assert torch.isnan(out.float()).all()
    # the context is intact: the same call with the flag set works
    flags[1] = 1
    _lib.check(L.sparse_b200_combine_peer(
        arr(o[0].data_ptr(), o[1].data_ptr()), arr(l[0].data_ptr(), l[1].data_ptr()), _lib.ptr(flags), 1, 30,
        _lib.ptr(out), None, ctypes.c_int64(64), 2, _lib.current_stream()))
    torch.cuda.synchronize()
    m.device_status()
    assert torch.isfinite(out.float()).all()


def test_rejected_arguments():
    from sparse_attention_b200_b200 import _lib
    L = _lib.lib()
    o, l = _partials(3, 32, 1)
    out = torch.empty((32, 128), dtype=torch.bfloat16, device="cuda")
    arr = ctypes.c_void_p * 3
    rc = L.sparse_b200_combine_peer(arr(*[o[r].data_ptr() for r in range(3)]), arr(*[l[r].data_ptr() for r in range(3)]),
                                    None, 0, 10, _lib.ptr(out), None, ctypes.c_int64(32), 3, _lib.current_stream())
    assert rc == _lib.ERR_INVALID                    # 3 ranks are not compiled in
    rc = L.sparse_b200_peer_signal((ctypes.c_void_p * 1)(None), 1, 1, _lib.current_stream())
    assert rc == _lib.ERR_INVALID


def test_run_peer_with_one_rank_is_the_attention_itself():
    """A group of one rank: exchange memory made by the library and wrapped as tensors, the attention kernel
    writes into it, three epochs of the flag hand-shake with itself; the result is the plain call's."""
    import torch.distributed as dist
    import oracle
    from oracle import inputs as gen
    from sparse_attention_b200_b200 import sharding
    m = sp()
    if dist.is_initialized():
        pytest.skip("a process group of another test is alive")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    try:
        q, k, v = gen.make_qkv(1, 8, 1, 384, 2048, seed=4, k_block_offset=0.5)
        ids = oracle.summary_select(q, k, 4, 4)[3].cuda()
        qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
        plain_o, plain_l = m.attention(qc, kc, vc, ids, return_lse=True)
        ex = sharding.PeerExchange(8 * 384, torch.device("cuda", 0))
        split = sharding.KVSplit()
        for _ in range(3):
            ex.o.fill_(float("nan"))
            o, l = split.run_peer(ex, qc, kc, vc, ids, 16)
            torch.cuda.synchronize()
            m.device_status()
            assert torch.equal(o.view(torch.int16), plain_o.reshape(-1, 128).view(torch.int16))
            assert torch.equal(l, plain_l.reshape(-1))
        assert ex.flags[0, 0].item() == 3 and ex.flags[1, 0].item() == 3
        o, l = split.run_scatter(ex, qc, kc, vc, ids, 16)          # one slice: the scatter form degenerates too
        torch.cuda.synchronize()
        m.device_status()
        assert torch.equal(o.view(torch.int16), plain_o.reshape(-1, 128).view(torch.int16))
        assert torch.equal(l, plain_l.reshape(-1))
        ex.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("owners,shape", [(2, (1, 8, 1, 512, 2048, 6)), (4, (2, 4, 2, 256, 1024, 5)),
                                          (3, (1, 3, 3, 384, 1024, 4)), (1, (1, 2, 1, 128, 512, 3))])
def test_scatter_launch_writes_each_slice_of_rows_to_its_destination(owners, shape):
    """sparse_b200_q_centric_scatter with the destinations in local memory: slice j of the flattened rows lands in
    buffer j, bit-identical to the plain call (pair mode, split mode, ragged counts with empty lists)."""
    from sparse_attention_b200_b200 import _lib
    m = sp()
    b, hq, hkv, sq, skv, topk = shape
    g = torch.Generator().manual_seed(sum(shape))
    q = torch.randn((b, hq, sq, 128), generator=g).to(torch.bfloat16).cuda()
    k = torch.randn((b, hkv, skv, 128), generator=g).to(torch.bfloat16).cuda()
    v = torch.randn((b, hkv, skv, 128), generator=g).to(torch.bfloat16).cuda()
    nb, qb = skv // 128, sq // 128
    ids = torch.stack([torch.randperm(nb, generator=g)[:topk] for _ in range(b * hkv * qb)]).to(torch.int32) \
        .reshape(b, hkv, qb, topk).cuda()
    counts = torch.randint(0, topk + 1, (b, hkv, qb), generator=g, dtype=torch.int32).cuda()
    ref = torch.empty_like(q)
    ref_l = torch.empty(q.shape[:3], device="cuda")
    m.attention_out(q, k, v, ids, ref, counts, ref_l, balance=False)
    rows = b * hq * sq
    per = rows // owners
    outs = [torch.full((per, 128), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(owners)]
    lses = [torch.full((per,), float("nan"), device="cuda") for _ in range(owners)]
    arr = ctypes.c_void_p * owners
    _lib.check(_lib.lib().sparse_b200_q_centric_scatter(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ids), _lib.ptr(counts), arr(*[t.data_ptr() for t in outs]),
        arr(*[t.data_ptr() for t in lses]), owners, b, hq, hkv, sq, skv, topk, _lib.current_stream()))
    torch.cuda.synchronize()
    m.device_status()
    assert torch.equal(torch.cat(outs).view(torch.int16), ref.reshape(-1, 128).view(torch.int16))
    assert torch.equal(torch.cat(lses).view(torch.int32), ref_l.reshape(-1).view(torch.int32))


def test_scatter_launch_rejects_slices_that_cut_a_tile():
    from sparse_attention_b200_b200 import _lib
    q = torch.zeros((1, 3, 128, 128), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((1, 3, 256, 128), dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros((1, 3, 1, 1), dtype=torch.int32, device="cuda")
    outs = [torch.empty((192, 128), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    lses = [torch.empty((192,), device="cuda") for _ in range(2)]
    arr = ctypes.c_void_p * 2
    rc = _lib.lib().sparse_b200_q_centric_scatter(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(k), _lib.ptr(ids), None, arr(*[t.data_ptr() for t in outs]),
        arr(*[t.data_ptr() for t in lses]), 2, 1, 3, 3, 128, 256, 1, _lib.current_stream())
    assert rc == _lib.ERR_INVALID                    # 384 rows / 2 = 192: not whole 128-row tiles
