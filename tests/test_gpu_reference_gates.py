"""The reference's OWN gate functions, run against this library.

The reference sources are not part of this repository: `python baseline/build_reference_kernels.py
--ref <checkout>` copies them, unmodified, into the git-ignored baseline/_ref/. Where they are
present, these tests import the reference's gate modules as they are and point them at this
library through the operator names / module interface the gates use:

* attention/q_centric/progression_validation.py:78-169 `check_stage_correctness` obtains its
  kernels from torch.ops.xomtention_progression (progression.py:29-58 only builds the reference
  extension when that operator is missing); sparse_attention_b200_b200.torch_ops registers the
  name over libsparse_b200.so first. Ten shape cases + three more for the GQA path, the `_out` form,
  CUDA-graph replays with changed inputs, seven rejected inputs.
* attention/kv_centric/validate_gpu.py:131-172 `run_suite` calls `api.attention(..., plan,
  return_debug)` and `api.load_extension().combine`; a stand-in `api` module routes both to the
  per-token KV-centric operator. Sixteen cases (sampled partials, analytic cases, reorder,
  non-default stream, repeat) + the Combine unit with +-1000 LSEs.

* attention/kv_centric/optimization_round11/api11.py `Prepared`, the reference's host class for its round-11
  KV-centric operator, used as it is over torch.ops.xomtention_kvopt11 from this library: all five variants
  (split8 and tma8 with fp32 partials, split8_bf16, tma8_bf16 and tma16_bf16; its planner's chunk sizes 8 and 16,
  token-major q and partials), its own audit of the task lists.

Skipped, with the reason, when baseline/_ref/ does not hold the reference files."""
import os
import sys
import types

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _need(*paths):
    missing = [p for p in paths if not os.path.exists(os.path.join(REF, p))]
    if missing:
        pytest.skip("reference sources not present under baseline/_ref/: " + ", ".join(missing))


@pytest.mark.parametrize("version", ["p02", "p03"])
def test_reference_q_centric_gate(version):
    _need("q_centric/progression_validation.py", "q_centric/progression.py", "q_centric/checkpoints.py")
    from sparse_attention_b200_b200 import torch_ops, device_status
    torch_ops.register(("xomtention_progression",))
    sys.path.insert(0, os.path.join(REF, "q_centric"))
    try:
        import progression_validation as gate
        result = gate.check_stage_correctness(version)
    finally:
        sys.path.remove(os.path.join(REF, "q_centric"))
    device_status()
    assert result["passed"] and len(result["rejected_inputs"]) == 7 and len(result["dynamic_graph_checks"]) == 3
    print(f"{version}: {len(result['cases'])} cases, persistent two-wave max abs {result['persistent_two_wave_max_abs']:.4g}")


def test_reference_kv_centric_gate():
    _need("kv_centric/validate_gpu.py", "kv_centric/metadata.py", "kv_centric/reference.py")
    import sparse_attention_b200_b200 as sp
    import pathlib
    kv_dir = os.path.join(REF, "kv_centric")

    # stand-in for attention/kv_centric/api.py: same names, same call forms, this library underneath
    api = types.ModuleType("api")
    api.ROOT = pathlib.Path(kv_dir)

    class _Ext:
        @staticmethod
        def combine(partial, lses):
            return sp.combine(partial, lses)

    def attention(q, k, v, selected, *, plan=None, return_debug=False):
        prep = sp.PreparedTokens(q, k, v, selected.to(q.device).contiguous())
        prep.poison()
        out, lse = prep.run()
        if return_debug:
            return out, lse, prep.partial, prep.lses
        return out
    api.attention = attention
    api.load_extension = lambda: _Ext
    saved = sys.modules.get("api")
    sys.modules["api"] = api
    sys.path.insert(0, kv_dir)
    try:
        import validate_gpu
        report = validate_gpu.run_suite(smoke=False)
    finally:
        sys.path.remove(kv_dir)
        if saved is None:
            sys.modules.pop("api", None)
        else:
            sys.modules["api"] = saved
    sp.device_status()
    assert report["passed"] and len(report["cases"]) == 16
    print(f"kv gate: max output abs {report['max_output_abs']:.4g}, max lse abs {report['max_lse_abs']:.4g}")


def test_reference_operator_names_head_major_chain():
    """xomtention_kvopt11::{metadata_out, main_out, combine_out, main_tm_out, combine_tm_out} and xomtention_tile_topk::* as torch
    operators: the chain equals the Python mirror bit for bit (no reference sources needed)."""
    import oracle
    from oracle import inputs as gen
    import sparse_attention_b200_b200 as sp
    from sparse_attention_b200_b200 import torch_ops
    ops = torch_ops.register(("xomtention_kvopt11", "xomtention_tile_topk"))
    kv = ops["xomtention_kvopt11"]
    b, hq, hkv, sq, skv, topk = 2, 16, 2, 200, 4096, 16
    g = hq // hkv
    q, k, v = gen.make_qkv(b, hq, hkv, sq, skv, seed=77)
    gen_ = torch.Generator().manual_seed(78)
    selected = torch.stack([torch.randperm(skv // 128, generator=gen_)[:topk] for _ in range(b * hkv * sq)]) \
        .to(torch.int32).reshape(b, hkv, sq, topk)
    qc, kc, vc, sel = q.cuda(), k.cuda(), v.cuda(), selected.cuda()
    rows, edges = b * hkv * (skv // 128), selected.numel()
    ints = lambda n: torch.empty(n, dtype=torch.int32, device="cuda")
    counts, row_ptr, chunks, task_ptr = ints(rows + 1), ints(rows + 1), ints(rows + 1), ints(rows + 1)
    cursors, qids, ranks, error = ints(rows), ints(edges), ints(edges), torch.zeros(1, dtype=torch.int32, device="cuda")
    bound = min(edges, -(-edges // (128 // g)) + rows)
    tasks = torch.zeros((bound, 4), dtype=torch.int32, device="cuda")
    temp = torch.empty(kv.metadata_temp_bytes(rows), dtype=torch.uint8, device="cuda")
    kv.metadata_out(sel, counts, row_ptr, cursors, qids, ranks, chunks, task_ptr, tasks, error, temp, skv // 128, g, 1)
    partial = torch.full((b, hq, sq, topk, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    lses = torch.full((b, hq, sq, topk), float("nan"), device="cuda")
    kv.main_out(qc, kc, vc, tasks, qids, ranks, partial, lses, -1)
    out = torch.empty_like(qc)
    out_lse = torch.empty((b, hq, sq), device="cuda")
    kv.combine_out(partial, lses, out, out_lse)
    torch.cuda.synchronize()
    sp.device_status()
    assert int(error.item()) == 0
    prep = sp.PreparedTokens(qc, kc, vc, sel)
    o2, l2 = prep.run()
    assert torch.equal(out, o2) and torch.equal(out_lse, l2)
    with pytest.raises(RuntimeError):
        kv.metadata_out(sel, counts, row_ptr, cursors, qids, ranks, chunks, task_ptr, tasks, error, temp, skv // 128, g, 3)
    with pytest.raises(RuntimeError):                                  # bf16 variant, fp32 buffer
        kv.main_out(qc, kc, vc, tasks, qids, ranks, partial.float(), lses, -1)
    with pytest.raises(RuntimeError):                                  # a token-major variant
        kv.main_out(qc, kc, vc, tasks, qids, ranks, partial, lses, 1)
    partial32 = torch.full(partial.shape, float("nan"), device="cuda")
    lses32 = torch.full_like(lses, float("nan"))
    kv.main_out(qc, kc, vc, tasks, qids, ranks, partial32, lses32, -2)  # the fp32 control (wrapper11.cpp:66-70)
    out32 = torch.full_like(out, float("nan"))
    out_lse32 = torch.full_like(out_lse, float("nan"))
    kv.combine_out(partial32, lses32, out32, out_lse32)
    torch.cuda.synchronize()
    sp.device_status()
    assert torch.equal(partial32.to(torch.bfloat16), partial) and torch.equal(lses32, lses)
    assert torch.equal(out_lse32, out_lse)
    torch.testing.assert_close(out32.float(), out.float(), atol=0.02, rtol=0.02)
    # the token-major pair (main_tm_out + combine_tm_out, wrapper11.cpp:94-133): q [B,Sq,Hq,128], partials
    # [B,Sq,TopK,Hq,128]; the merged output is the head-major chain's, bit for bit
    q_tm = qc.permute(0, 2, 1, 3).contiguous()
    partial_tm = torch.full((b, sq, topk, hq, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
    lses_tm = torch.full((b, hq, sq, topk), float("nan"), device="cuda")
    kv.main_tm_out(q_tm, kc, vc, tasks, qids, ranks, partial_tm, lses_tm, 1)
    out_tm = torch.full_like(qc, float("nan"))
    out_lse_tm = torch.full((b, hq, sq), float("nan"), device="cuda")
    kv.combine_tm_out(partial_tm, lses_tm, out_tm, out_lse_tm)
    torch.cuda.synchronize()
    sp.device_status()
    assert torch.equal(partial_tm.permute(0, 3, 1, 2, 4), partial) and torch.equal(lses_tm, lses)
    assert torch.equal(out_tm, out) and torch.equal(out_lse_tm, out_lse)
    with pytest.raises(RuntimeError):
        kv.main_tm_out(q_tm, kc, vc, tasks, qids, ranks, partial_tm, lses_tm, 0)     # fp32 partials are not served
    with pytest.raises(RuntimeError):
        kv.combine_tm_out(partial, lses, out_tm, out_lse_tm)                        # head-major partials
    # tile_topk operators against the Python mirror
    scores = torch.randn((2, 32, 2 * 256), device="cuda")
    tk = ops["xomtention_tile_topk"]
    ids = tk.tile_topk(scores, 2, 256)
    ids2 = torch.empty_like(ids)
    tk.tile_topk_out(scores, ids2, 2, 256)
    assert torch.equal(ids, ids2) and torch.equal(ids, sp.tile_topk(scores, batch_size=2, len_q=256, topk=16))
    assert torch.equal(ids.cpu(), oracle.fp4_select(scores.cpu(), 2, 256, 16))


def test_reference_round11_prepared_class_runs_on_this_library():
    """attention/kv_centric/optimization_round11/api11.py `Prepared` (the reference's own host class: GPUPlan with
    its chunk sizes, main_out / main_tm_out, combine_out / combine_tm_out, partial_view) used as it is, with
    torch.ops.xomtention_kvopt11 coming from this library instead of the reference's extension: outputs and
    partials equal this library's Python mirror bit for bit for all five variants (split8, split8_bf16, tma8,
    tma8_bf16, tma16_bf16), and the reference's own audit of the task lists (gpu_plan.py:47-73) passes."""
    _need("kv_centric/optimization_round11/api11.py", "kv_centric/optimization_round4/gpu_plan.py",
          "kv_centric/optimization_round4/planning.py", "kv_centric/metadata.py")
    import sparse_attention_b200_b200 as sp
    from sparse_attention_b200_b200 import torch_ops
    torch_ops.register(("xomtention_kvopt11",))
    r11 = os.path.join(REF, "kv_centric", "optimization_round11")
    sys.path.insert(0, r11)
    try:
        import api11
        api11._OPS = torch.ops.xomtention_kvopt11          # what load_extension() would set after building its own
        api11.old_plan.load_extension = lambda: api11._OPS
        gen_ = torch.Generator().manual_seed(5)
        for b, hkv, g, sq, skv in ((2, 1, 16, 300, 4096), (1, 2, 8, 520, 2048)):
            hq = hkv * g
            q_tm = torch.randn((b, sq, hq, 128), generator=gen_).to(torch.bfloat16).cuda()
            k = torch.randn((b, hkv, skv, 128), generator=gen_).to(torch.bfloat16).cuda()
            v = torch.randn((b, hkv, skv, 128), generator=gen_).to(torch.bfloat16).cuda()
            selected = torch.stack([torch.randperm(skv // 128, generator=gen_)[:16] for _ in range(b * hkv * sq)]) \
                .to(torch.int32).reshape(b, hkv, sq, 16)
            sel = selected.cuda()
            ours = sp.PreparedTokens(q_tm.permute(0, 2, 1, 3).contiguous(), k, v, sel)
            ours.run()
            for variant in (-1, 1, 2):
                prep = api11.Prepared(q_tm, k, v, sel, variant=variant)
                prep.poison()
                prep.run()
                torch.cuda.synchronize()
                sp.device_status()
                assert torch.equal(prep.out, ours.out) and torch.equal(prep.out_lse, ours.out_lse), variant
                assert torch.equal(prep.partial_view(), ours.partial) and torch.equal(prep.lses, ours.lses), variant
                report = prep.plan.audit(selected)
                assert report["exact_coverage"] and report["gpu_error"] == 0, variant
            # the fp32 controls (split8 = -2, the class's default, and tma8 = 0): same kernels with fp32 partials
            ours32 = sp.PreparedTokens(q_tm.permute(0, 2, 1, 3).contiguous(), k, v, sel, partial_f32=True)
            ours32.run()
            assert torch.equal(ours32.partial.to(torch.bfloat16), ours.partial) and torch.equal(ours32.lses, ours.lses)
            for prep in (api11.Prepared(q_tm, k, v, sel), api11.Prepared(q_tm, k, v, sel, variant=0)):
                assert prep.partial.dtype == torch.float32
                prep.poison()
                prep.run()
                torch.cuda.synchronize()
                sp.device_status()
                assert torch.equal(prep.partial_view(), ours32.partial) and torch.equal(prep.lses, ours32.lses)
                assert torch.equal(prep.out, ours32.out) and torch.equal(prep.out_lse, ours.out_lse)
                torch.testing.assert_close(prep.out.float(), ours.out.float(), atol=0.02, rtol=0.02)
    finally:
        sys.path.remove(r11)
