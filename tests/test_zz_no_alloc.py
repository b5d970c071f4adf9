"""The allocation-free summary indexer against the regular entry point.

Some callers of this library cannot allocate device memory at the point where
they need block ids (a framework pool that owns the device, a serving loop with
a fixed memory budget, a plugin that only receives inputs and outputs), so
sparse_b200_indexer_summary_noalloc keeps its pooled descriptors in an 8 MiB
array inside the library. The array is shared and keeps the last call's
contents, so the check runs two different problems back to back and requires
ids and scores identical to the regular entry point both times. Collected last
on purpose: a failure here must not hide the rest of the suite."""
import ctypes

import pytest
import torch

from oracle import inputs as gen


def _lib():
    from sparse_attention_b200_b200 import _lib as L
    return L


def _call_pair(q, k, r, topk):
    L = _lib()
    lib = L.lib()
    b, hq, sq, _ = q.shape
    hkv, skv = k.shape[1:3]
    qt, nt = sq // 128, skv // 128
    dev = q.device
    st = L.current_stream()
    # regular entry point: caller-supplied descriptor workspaces
    qd = torch.empty((b, hq, qt, r, 128), dtype=torch.bfloat16, device=dev)
    kd = torch.empty((b, hkv, nt, r, 128), dtype=torch.bfloat16, device=dev)
    s_ref = torch.empty((b, hkv, qt, nt), dtype=torch.float32, device=dev)
    i_ref = torch.empty((b, hkv, qt, topk), dtype=torch.int32, device=dev)
    L.check(lib.sparse_b200_indexer_summary(L.ptr(q), L.ptr(k), L.ptr(qd), L.ptr(kd), L.ptr(s_ref), L.ptr(i_ref),
                                            b, hq, hkv, sq, skv, r, topk, st))
    # allocation-free entry point: inputs and outputs only
    s_new = torch.full_like(s_ref, float("nan"))
    i_new = torch.full_like(i_ref, -1)
    L.check(lib.sparse_b200_indexer_summary_noalloc(L.ptr(q), L.ptr(k), L.ptr(s_new), L.ptr(i_new),
                                                    b, hq, hkv, sq, skv, r, topk, st))
    torch.cuda.synchronize()
    return (s_ref, i_ref), (s_new, i_new)


@pytest.mark.gpu
def test_noalloc_indexer_matches_regular_entry_twice_in_a_row():
    problems = [
        # B, Hq, Hkv, Sq, Skv, R, topk
        (1, 8, 8, 4096, 4096, 1, 8),      # configuration 1
        (2, 8, 2, 512, 2048, 4, 5),       # smaller, other R: stale descriptors must not leak
    ]
    for seed, (b, hq, hkv, sq, skv, r, topk) in enumerate(problems):
        q, k, _ = gen.make_qkv(b, hq, hkv, sq, skv, seed=900 + seed, k_block_offset=0.5)
        (s_ref, i_ref), (s_new, i_new) = _call_pair(q.cuda(), k.cuda(), r, topk)
        assert torch.equal(i_new, i_ref)          # ids are compared exactly everywhere in this suite
        assert torch.equal(s_new, s_ref)          # and so are the scores (same fixed arithmetic)
    # scores output is optional
    L = _lib()
    q, k, _ = gen.make_qkv(1, 4, 2, 256, 1024, seed=77)
    ids = torch.empty((1, 2, 2, 3), dtype=torch.int32, device="cuda")
    qc, kc = q.cuda(), k.cuda()          # keep the device copies alive across the call
    L.check(L.lib().sparse_b200_indexer_summary_noalloc(L.ptr(qc), L.ptr(kc), None, L.ptr(ids),
                                                        1, 4, 2, 256, 1024, 2, 3, L.current_stream()))
    torch.cuda.synchronize()
    import oracle
    assert torch.equal(ids.cpu(), oracle.summary_select(q, k, 2, 3)[3])


@pytest.mark.gpu
def test_noalloc_indexer_at_its_limits():
    """The ends of the built-in array and of the shared score buffer: exactly 32768 descriptors
    with 4096 KV blocks, group size x R = 16 (the widest padded row block), and R = 2."""
    g = torch.Generator(device="cuda").manual_seed(901)
    problems = [
        (1, 1, 1, 524288, 524288, 4, 64),     # (4096 + 4096) blocks x R4 = 32768 descriptors, nt = 4096
        (1, 16, 4, 1024, 2048, 4, 7),         # group 4 x R4 = 16
        (1, 8, 1, 512, 4096, 2, 9),           # group 8 x R2 = 16, R = 2
        (2, 4, 4, 256, 512, 2, 4),            # R = 2, group 1
    ]
    for (b, hq, hkv, sq, skv, r, topk) in problems:
        q = torch.randn((b, hq, sq, 128), device="cuda", generator=g).to(torch.bfloat16)
        k = (torch.randn((b, hkv, skv // 128, 128, 128), device="cuda", generator=g)
             + 0.5 * torch.randn((b, hkv, skv // 128, 1, 128), device="cuda", generator=g)) \
            .reshape(b, hkv, skv, 128).to(torch.bfloat16)
        (s_ref, i_ref), (s_new, i_new) = _call_pair(q, k, r, topk)
        assert torch.equal(i_new, i_ref)
        assert torch.equal(s_new, s_ref)
    from sparse_attention_b200_b200 import device_status
    device_status()


def test_noalloc_indexer_rejects_sizes_beyond_its_scratch():
    """Validation happens before any CUDA call, so this runs without a GPU too."""
    L = _lib()
    lib = L.lib()
    p = ctypes.c_void_p(4096)
    # (16 + 8) heads x 2048 blocks x R4 = 196608 descriptors > 32768
    rc = lib.sparse_b200_indexer_summary_noalloc(p, p, None, p, 1, 16, 8, 262144, 262144, 4, 64, None)
    assert rc == L.ERR_INVALID and b"8 MiB" in lib.sparse_b200_last_error()
    rc = lib.sparse_b200_indexer_summary_noalloc(p, p, None, p, 1, 16, 1, 256, 1024, 4, 4, None)
    assert rc == L.ERR_INVALID and b"must not exceed 16" in lib.sparse_b200_last_error()
    rc = lib.sparse_b200_indexer_summary_noalloc(p, p, None, p, 1, 1, 1, 128, 128 * 8192, 1, 4, None)
    assert rc == L.ERR_INVALID and b"4096" in lib.sparse_b200_last_error()
