"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations. Test infrastructure only (the benchmark builds its
own device-side inputs; these CPU generators serve the parity tests).

Families follow benchmarks/ch4_selectors/reference.py:6-25 (gaussian) and
attention/q_centric/progression_validation.py:12-41 (make_inputs / make_ids).
"""
import random

import torch

BLOCK = 128


def make_qkv(b, hq, hkv, sq, skv, seed=17, scale=1.0, k_block_offset=0.0):
    """Q,K,V ~ N(0,scale) in fp32 then bf16; optionally a per-128-key-block
    offset ~ N(0, k_block_offset) is added to K before the cast."""
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn((b, hq, sq, 128), generator=gen) * scale
    k = torch.randn((b, hkv, skv, 128), generator=gen) * scale
    v = torch.randn((b, hkv, skv, 128), generator=gen)
    if k_block_offset:
        off = torch.randn((b, hkv, skv // BLOCK, 1, 128), generator=gen) * k_block_offset
        k = (k.reshape(b, hkv, skv // BLOCK, BLOCK, 128) + off).reshape(b, hkv, skv, 128)
    return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)


def make_ids(b, hkv, qtiles, kvtiles, topk, seed, pattern="independent"):
    """progression_validation.py:21-41: distinct block ids per list; sorted
    ascending unless 'unsorted' / 'reverse'; 'paired' repeats the previous
    list on odd query tiles."""
    assert 0 < topk <= kvtiles
    rng = random.Random(seed)
    out = []
    for _ in range(b):
        heads = []
        for _ in range(hkv):
            rows = []
            for qt in range(qtiles):
                if pattern == "paired" and qt % 2:
                    row = list(rows[-1])
                else:
                    row = rng.sample(range(kvtiles), topk)
                    if pattern != "unsorted":
                        row.sort(reverse=pattern == "reverse")
                rows.append(row)
            heads.append(rows)
        out.append(heads)
    return torch.tensor(out, dtype=torch.int32)
