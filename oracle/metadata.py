"""Scheduling metadata oracles (CPU, plain Python/torch). Test infrastructure only."""
import torch

BLOCK = 128


def split_kv_segments(ids, kv_blocks, nseg, counts=None):
    """KV-range segmentation used by the KV-centric operator.

    Segment s owns KV blocks [s*W, (s+1)*W) with W = ceil(kv_blocks / nseg).
    For every list the ids owned by a segment are kept in their original order
    and packed to the front. Returns seg_ids [nseg,B,Hkv,Qt,K] (tail entries
    repeat the segment's first block id, which is always in range) and
    seg_counts [nseg,B,Hkv,Qt]. This replaces the reference's per-block
    reverse index (attention/kv_centric/metadata.py:43-72) by a per-KV-range
    one: every (query block, KV range) pair becomes one task whose partial
    (O, LSE) is merged afterwards, instead of one partial per selected block.
    """
    from .attention import filter_ids_to_range
    width = (kv_blocks + nseg - 1) // nseg
    seg_ids, seg_counts = [], []
    for s in range(nseg):
        i, c = filter_ids_to_range(ids, s * width, min((s + 1) * width, kv_blocks), counts)
        seg_ids.append(i)
        seg_counts.append(c)
    return torch.stack(seg_ids), torch.stack(seg_counts)


def build_reverse_plan(selected, kv_blocks, group_size):
    """Per-token reverse index, any TopK.

    Restates attention/kv_centric/metadata.py:43-72 (`build_plan`): rows are
    (batch*Hkv + head)*kv_blocks + block; each row lists the (query, rank)
    edges that selected the block, in (query, rank) order; tasks cut a row
    into chunks of 128/group_size queries.
    selected: [B,Hkv,Sq,K] int32 (per TOKEN). Returns dict of int32 tensors
    row_ptr [rows+1], query_ids [E], ranks [E], tasks [T,4] =
    (group, block, edge start, edge count).
    """
    batch, hkv, sq, topk = selected.shape
    rows = [[] for _ in range(batch * hkv * kv_blocks)]
    for group_id, lists in enumerate(selected.reshape(-1, sq, topk).tolist()):
        for query, ids in enumerate(lists):
            for rank, block in enumerate(ids):
                rows[group_id * kv_blocks + block].append((query, rank))
    row_ptr, qids, ranks, tasks = [0], [], [], []
    chunk = BLOCK // group_size
    for row, edges in enumerate(rows):
        start = len(qids)
        qids.extend(q for q, _ in edges)
        ranks.extend(r for _, r in edges)
        for off in range(0, len(edges), chunk):
            tasks.append((row // kv_blocks, row % kv_blocks, start + off, min(chunk, len(edges) - off)))
        row_ptr.append(len(qids))
    return {"row_ptr": torch.tensor(row_ptr, dtype=torch.int32),
            "query_ids": torch.tensor(qids, dtype=torch.int32),
            "ranks": torch.tensor(ranks, dtype=torch.int32),
            "tasks": torch.tensor(tasks, dtype=torch.int32).reshape(-1, 4)}


def validate_reverse_plan(plan, selected, kv_blocks, group_size, ordered=True):
    """Exact edge coverage audit, after metadata.py:75-117. With ordered=False
    the order of edges inside a row is free (a GPU build fills rows with
    atomics), everything else must match exactly."""
    batch, hkv, sq, topk = selected.shape
    ptr = plan["row_ptr"].tolist()
    qids, ranks = plan["query_ids"].tolist(), plan["ranks"].tolist()
    edges = selected.numel()
    nrows = batch * hkv * kv_blocks
    assert len(ptr) == nrows + 1 and ptr[0] == 0 and ptr[-1] == edges
    assert all(a <= b for a, b in zip(ptr, ptr[1:]))
    flat = selected.reshape(-1, sq, topk).tolist()
    seen = set()
    for row in range(nrows):
        group, block = divmod(row, kv_blocks)
        prev = (-1, -1)
        for e in range(ptr[row], ptr[row + 1]):
            qi, r = qids[e], ranks[e]
            assert 0 <= qi < sq and 0 <= r < topk
            key = (group, qi, r)
            assert key not in seen and flat[group][qi][r] == block
            seen.add(key)
            if ordered:
                assert (qi, r) > prev
                prev = (qi, r)
    assert len(seen) == edges
    visits = [0] * edges
    for group, block, start, count in plan["tasks"].tolist():
        row = group * kv_blocks + block
        assert 0 < count <= BLOCK // group_size
        assert ptr[row] <= start and start + count <= ptr[row + 1]
        for e in range(start, start + count):
            visits[e] += 1
    assert all(c == 1 for c in visits)
    return True
