"""Seeded inputs of the golden cases. Imported by the script that generated
the fixtures (make_golden.py, which runs the untouched reference functions on
them) and by the tests (which run the oracle and the CUDA path on them)."""
import hashlib

import torch

from oracle import inputs as gen


def digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        t = t.contiguous()
        h.update(t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bool else t.numpy().tobytes())
    return h.hexdigest()


def attention_masked_case():
    """Shape the reference masked oracle accepts: TopK 16 (its fixed constant),
    >= 16 KV blocks, per-token lists obtained by repeating the block lists."""
    q, k, v = gen.make_qkv(1, 4, 2, 256, 2560, seed=1701, k_block_offset=0.5)
    ids = gen.make_ids(1, 2, 2, 20, 16, seed=2301, pattern="unsorted")
    return q, k, v, ids


def attention_gather_cases():
    """(shape, topk, pattern, scale) in the style of the reference gate list
    (progression_validation.py:82-98), sized for the CPU."""
    specs = [((1, 2, 2, 256, 128), 1, "independent", 1.0),
             ((1, 4, 2, 256, 512), 3, "unsorted", 1.0),
             ((1, 8, 1, 128, 1024), 8, "reverse", 2.0)]
    out = []
    for i, (shape, topk, pattern, scale) in enumerate(specs):
        b, hq, hkv, sq, skv = shape
        q, k, v = gen.make_qkv(b, hq, hkv, sq, skv, seed=1800 + i, scale=scale)
        ids = gen.make_ids(b, hkv, sq // 128, skv // 128, topk, 2400 + i, pattern)
        out.append((q, k, v, ids))
    return out


def selector_inputs(family, seed=17, batch=1, sq=512, skv=4096):
    """The two input families of benchmarks/ch4_selectors/reference.py:6-25 with
    a CPU generator (the reference hard-codes device='cuda'); H16/Hkv1."""
    import math
    g = torch.Generator().manual_seed(seed)

    def rand(shape):
        return torch.randn(shape, generator=g)
    if family == "gaussian":
        q, k = rand((batch, 16, sq, 128)), rand((batch, 1, skv, 128))
    elif family == "cancellation_stress":
        qt, nt = sq // 128, skv // 128
        centers = rand((batch, nt, 128))
        centers = centers / centers.norm(dim=-1, keepdim=True) * math.sqrt(128)
        order = torch.rand((batch, qt, nt), generator=g).argsort(dim=-1)
        targets = order[..., :4][:, :, torch.arange(16) % 4].permute(0, 2, 1)
        qc = centers[torch.arange(batch)[:, None, None], targets]
        signs = torch.where(torch.arange(128) < 64, 1.0, -1.0)[None, None, None, :, None]
        q = (qc[..., None, :] * signs + .1 * rand((batch, 16, qt, 128, 128))).reshape(batch, 16, sq, 128)
        k = (centers[:, None, :, None, :] * signs + .1 * rand((batch, 1, nt, 128, 128))).reshape(batch, 1, skv, 128)
    elif family == "zeros":
        q, k = torch.zeros((batch, 16, sq, 128)), torch.zeros((batch, 1, skv, 128))
    else:
        raise ValueError(family)
    return q.to(torch.bfloat16), k.to(torch.bfloat16)


def fp4_case(batch=1, hidx=2, len_q=256, len_kv=2048, seed=313):
    """Random packed codes and 'varied' scales, as make_synthetic_fp4_inputs
    (indexers/fp4/fp4.py:88-119) draws them; one shared key head."""
    g = torch.Generator().manual_seed(seed)
    pages = batch * (len_kv // 128)
    qp = torch.randint(256, (batch * len_q, hidx, 64), dtype=torch.uint8, generator=g)
    kp = torch.randint(256, (pages, 1, 128, 64), dtype=torch.uint8, generator=g)
    choices = torch.tensor([0.25, 0.375, 0.5, 0.75, 1.0, 1.5, 2.0])

    def scales(shape):
        return choices[torch.randint(len(choices), shape, generator=g)].to(torch.float8_e4m3fn)
    return qp, scales((batch * len_q, hidx, 8)), kp, scales((pages, 1, 128, 8)), batch, len_q, len_kv


def reverse_plan_case():
    """Per-token lists, TopK 16 (the reference constant), 32 KV blocks."""
    g = torch.Generator().manual_seed(37)
    b, hkv, sq, nb = 2, 2, 19, 32
    sel = torch.empty((b, hkv, sq, 16), dtype=torch.int32)
    for bi in range(b):
        for h in range(hkv):
            for qi in range(sq):
                sel[bi, h, qi] = torch.randperm(nb, generator=g)[:16].to(torch.int32)
    return sel, nb


def combine_case():
    """benchmarks of validate_gpu.py:30-40: random partials, LSE * 20, one row
    with -1000 everywhere but a single +1000."""
    g = torch.Generator().manual_seed(951)
    partial = torch.randn((2, 2, 5, 16, 128), generator=g)
    lses = torch.randn((2, 2, 5, 16), generator=g) * 20
    lses[0, 0, 0].fill_(-1000)
    lses[0, 0, 0, 5] = 1000
    return partial, lses
