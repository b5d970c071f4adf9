"""Two-GPU run of the KV-range split (NCCL send/recv exchange + Combine kernel, and the merge
over peer memory) and of the head-group sharding. Skipped on a box with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, result):
    import oracle
    from oracle import inputs as gen
    import sparse_attention_b200_b200 as sp
    from sparse_attention_b200_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        # KV split: group size 8, 64 KV blocks, top-8, R4 indexer picks the lists on every rank alike
        q, k, v = gen.make_qkv(1, 16, 2, 512, 8192, seed=21, k_block_offset=0.5)
        ids = sp.SummarySelector(q.cuda(), k.cuda(), 4, topk=8).run()
        ref_ids = oracle.summary_select(q, k, 4, 8)[3]
        ok = torch.equal(ids.cpu(), ref_ids)
        lo, hi = sharding.kv_block_range(64, world, rank)
        k_local = k[:, :, lo * 128:hi * 128].contiguous().cuda()
        v_local = v[:, :, lo * 128:hi * 128].contiguous().cuda()
        split = sharding.KVSplit()
        o_slice, l_slice = split.run(q.cuda(), k_local, v_local, ids, 64)
        torch.cuda.synchronize()
        sp.device_status()
        whole_o, whole_l = oracle.gather_attention(q, k, v, ref_ids)
        rows = whole_l.numel() // world
        ref_o = whole_o.reshape(-1, 128)[rank * rows:(rank + 1) * rows]
        ref_l = whole_l.reshape(-1)[rank * rows:(rank + 1) * rows]
        d = (o_slice.float().cpu() - ref_o).abs()
        ok = ok and d.max().item() <= 2e-2 and d.mean().item() <= 2e-3
        ok = ok and bool(torch.all((l_slice.cpu() - ref_l).abs() <= 1e-3 * ref_l.abs().clamp_min(1.0)))
        # the same merge over peer memory (IPC-mapped exchange memory, flags, merge kernel loading the peer's
        # rows): bit-identical to the send/recv form, over several steps of the ready / done hand-shake
        ex = sharding.PeerExchange(whole_l.numel(), torch.device("cuda", rank))
        for _ in range(4):
            o_peer, l_peer = split.run_peer(ex, q.cuda(), k_local, v_local, ids, 64)
            torch.cuda.synchronize()
            sp.device_status()
            ok = ok and torch.equal(o_peer.view(torch.int16), o_slice.view(torch.int16)) and torch.equal(l_peer, l_slice)
        ok = ok and ex.flags[:, :world].tolist() == [[4] * world, [4] * world]
        # ... and with the transfer inside the attention kernel (tiles stored straight into the merging rank's memory)
        for _ in range(3):
            o_sc, l_sc = split.run_scatter(ex, q.cuda(), k_local, v_local, ids, 64)
            torch.cuda.synchronize()
            sp.device_status()
            ok = ok and torch.equal(o_sc.view(torch.int16), o_slice.view(torch.int16)) and torch.equal(l_sc, l_slice)
        ex.close()
        # pipelined form: chunks of two heads, the exchange of one under the attention of the next
        qg, kg, vg, ig, _ = sharding.group_view(q.cuda(), k_local, v_local, ids, 0, 2)
        merged = split.run_pipelined(qg, kg, vg, ig, 64, heads_per_chunk=2)
        torch.cuda.synchronize()
        sp.device_status()
        plan = split.chunks(qg, 2)
        ok = ok and sorted(merged) == [c for c in range(len(plan)) if c % world == rank]
        for c, (oc, lc) in merged.items():
            grp, h0, nh = plan[c]
            ref_oc = whole_o[0, grp * 8 + h0:grp * 8 + h0 + nh].reshape(-1, 128)
            ref_lc = whole_l[0, grp * 8 + h0:grp * 8 + h0 + nh].reshape(-1)
            dc = (oc.float().cpu() - ref_oc).abs()
            ok = ok and dc.max().item() <= 2e-2 and dc.mean().item() <= 2e-3
            ok = ok and bool(torch.all((lc.cpu() - ref_lc).abs() <= 1e-3 * ref_lc.abs().clamp_min(1.0)))
        # head-group sharding: no collective, each rank its own groups
        a, b = sharding.group_range(2, world, rank)
        if b > a:                                  # with more ranks than groups some ranks hold none
            qv, kv, vv, iv, _ = sharding.group_view(q.cuda(), k.cuda(), v.cuda(), ids, a, b)
            og = sp.attention(qv, kv, vv, iv)
            dg = (og.float().cpu().reshape(-1, 512, 128) - whole_o[0, a * 8:b * 8]).abs()
            ok = ok and dg.max().item() <= 2e-2
        result[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_kv_split_and_group_sharding(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert dict(result) == {r: True for r in range(world)}
