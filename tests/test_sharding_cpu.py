"""Host-side sharding logic on CPU: group partition and the KV-split exchange +
merge with two gloo ranks (the attention / combine stages are the oracle here;
on GPUs they are the CUDA kernels, see tests/test_gpu_multi.py)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from oracle import inputs as gen
from sparse_attention_b200_b200 import sharding


def test_group_range_covers_everything_once():
    for n in (1, 7, 8, 16, 33):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                a, b = sharding.group_range(n, world, r)
                assert 0 <= a <= b <= n and (b - a) in (n // world, n // world + 1)
                seen += list(range(a, b))
            assert seen == list(range(n))
    assert [sharding.group_range(8, 8, r) for r in range(8)] == [(r, r + 1) for r in range(8)]
    assert sharding.kv_block_range(8192, 2, 1) == (4096, 8192)
    assert sharding.kv_block_range(10, 4, 3) == (9, 10)


def test_group_view_is_a_view_and_matches_whole():
    q, k, v = gen.make_qkv(2, 8, 4, 256, 512, seed=3)
    ids = gen.make_ids(2, 4, 2, 4, 2, 4)
    whole, _ = oracle.gather_attention(q, k, v, ids)
    parts = []
    for r in range(4):
        a, b = sharding.group_range(8, 4, r)
        qv, kv, vv, iv, _ = sharding.group_view(q, k, v, ids, a, b)
        assert qv.data_ptr() == q.view(8, 2, 256, 128)[a].data_ptr()
        o, _ = oracle.gather_attention(qv, kv, vv, iv)
        parts.append(o)
    assert torch.equal(torch.cat(parts).reshape(whole.shape), whole)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v = gen.make_qkv(1, 4, 2, 256, 2048, seed=11)
        ids = gen.make_ids(1, 2, 2, 16, 6, 12, "unsorted")
        ids[0, 0, 0] = torch.tensor([0, 1, 2, 3, 4, 5], dtype=torch.int32)      # all in rank 0's range
        kv_blocks = 16
        lo, hi = sharding.kv_block_range(kv_blocks, world, rank)
        k_local = k[:, :, lo * 128:hi * 128].contiguous()
        v_local = v[:, :, lo * 128:hi * 128].contiguous()

        def filter_fn(i, c, nb, ranks, r):
            a, b = sharding.kv_block_range(nb, ranks, r)
            fi, fc = oracle.filter_ids_to_range(i, a, b, c)
            return (fi - a).clamp_(min=0), fc

        def attention_fn(qq, kk, vv, ii, cc):
            o, l = oracle.gather_attention(qq, kk, vv, ii, cc)
            return o, l

        def combine_fn(po, pl):
            return oracle.combine_partials(po.permute(1, 0, 2), pl.permute(1, 0))

        split = sharding.KVSplit(None, filter_fn, attention_fn, combine_fn)
        o_slice, l_slice = split.run(q, k_local, v_local, ids, kv_blocks)
        whole_o, whole_l = oracle.gather_attention(q, k, v, ids)
        rows = whole_l.numel() // world
        ref_o = whole_o.reshape(-1, 128)[rank * rows:(rank + 1) * rows]
        ref_l = whole_l.reshape(-1)[rank * rows:(rank + 1) * rows]
        ok = torch.allclose(o_slice, ref_o, atol=2e-6) and torch.allclose(l_slice, ref_l, atol=2e-6)
        # pipelined form (chunks of head pairs, owner = chunk % ranks): every chunk merged exactly once
        qg, kg, vg, ig, _ = sharding.group_view(q, k_local, v_local, ids, 0, 2)
        merged = split.run_pipelined(qg, kg, vg, ig, kv_blocks, heads_per_chunk=1)
        plan = split.chunks(qg, 1)
        ok = ok and sorted(merged) == [c for c in range(len(plan)) if c % world == rank]
        for c, (oc, lc) in merged.items():
            grp, h0, nh = plan[c]
            ok = ok and torch.allclose(oc, whole_o[0, grp * 2 + h0:grp * 2 + h0 + nh].reshape(-1, 128), atol=2e-6)
            ok = ok and torch.allclose(lc, whole_l[0, grp * 2 + h0:grp * 2 + h0 + nh].reshape(-1), atol=2e-6)
        # a rank with an empty filtered list contributed (0, -inf) for that row block
        _, cnt = filter_fn(ids, None, kv_blocks, world, rank)
        if rank == 1:
            ok = ok and int(cnt[0, 0, 0]) == 0
        result[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_kv_split_two_gloo_ranks():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert dict(result) == {0: True, 1: True}
