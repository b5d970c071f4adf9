"""Generate tests/golden/*.npz by running the UNTOUCHED reference functions
(imported from a checkout of the reference project) on the seeded inputs of
cases.py. Run once, on a machine that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

The fixtures hold the reference outputs plus a digest of the inputs, so a
drift of the input generators is detected instead of silently comparing
different data. Nothing here runs on the GPU box.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests.golden import cases  # noqa: E402


def load(ref_root, rel, name, extra_path=None):
    if extra_path:
        sys.path.insert(0, os.path.join(ref_root, extra_path))
    spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root):
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    kvref = load(ref_root, "attention/kv_centric/reference.py", "ref_kv_reference",
                 "attention/kv_centric")
    kvmeta = sys.modules["metadata"]
    sys.path.insert(0, os.path.join(ref_root, "attention/q_centric"))
    qval = load(ref_root, "attention/q_centric/progression_validation.py", "ref_q_validation")
    selref = load(ref_root, "benchmarks/ch4_selectors/reference.py", "ref_sel_reference")
    fp4ref = load(ref_root, "indexers/fp4/fp4_reference.py", "ref_fp4_reference")
    topkref = load(ref_root, "indexers/fp4/reference.py", "ref_fp4_topk")

    # 1. masked attention (attention/kv_centric/reference.py:7-31)
    q, k, v, ids = cases.attention_masked_case()
    per_token = ids.repeat_interleave(128, dim=2).contiguous()
    o, lse = kvref.attention_reference(q, k, v, per_token)
    np.savez_compressed(os.path.join(HERE, "attention_masked.npz"), o=o.numpy(), lse=lse.numpy(),
                        digest=cases.digest(q, k, v, ids))

    # 2. gather attention (attention/q_centric/progression_validation.py:44-62)
    outs = {}
    for i, (q, k, v, ids) in enumerate(cases.attention_gather_cases()):
        outs[f"o{i}"] = qval.reference(q, k, v, ids).numpy()
        outs[f"digest{i}"] = cases.digest(q, k, v, ids)
    np.savez_compressed(os.path.join(HERE, "attention_gather.npz"), **outs)

    # 3. R1 / R4 selectors (benchmarks/ch4_selectors/reference.py:28-38)
    outs = {}
    for family in ("gaussian", "cancellation_stress", "zeros"):
        q, k = cases.selector_inputs(family)
        for r in (1, 4):
            qd, kd, scores, sel = selref.summary_reference(q, k, r)
            tag = f"{family}_r{r}"
            outs[tag + "_qd"] = qd.view(torch.int16).numpy()
            outs[tag + "_kd"] = kd.view(torch.int16).numpy()
            outs[tag + "_scores"] = scores.numpy()
            outs[tag + "_ids"] = sel.numpy()
        outs[family + "_digest"] = cases.digest(q, k)
    np.savez_compressed(os.path.join(HERE, "selectors.npz"), **outs)

    # 4. NVFP4 scores + tile top-k (indexers/fp4/fp4_reference.py, reference.py)
    qp, qs, kp, ks, b, lq, lkv = cases.fp4_case()
    inputs = {"q": qp, "k": kp, "q_scale": qs, "k_scale": ks, "batch_size": b,
              "hkv": qp.shape[1], "len_q": lq, "len_kv": lkv}
    scores = fp4ref.fp4_scores_reference(inputs)
    sel = topkref.tile_topk_reference(scores, batch_size=b, len_q=lq)
    np.savez_compressed(os.path.join(HERE, "fp4.npz"), scores=scores.numpy(), ids=sel.numpy(),
                        digest=cases.digest(qp, qs.view(torch.uint8), kp, ks.view(torch.uint8)))

    # 5. per-token reverse plan (attention/kv_centric/metadata.py:43-72)
    sel, nb = cases.reverse_plan_case()
    outs = {}
    for g in (1, 4, 16):
        plan = kvmeta.build_plan(sel, nb, g)
        outs[f"g{g}_row_ptr"] = plan.row_ptr.numpy()
        outs[f"g{g}_query_ids"] = plan.query_ids.numpy()
        outs[f"g{g}_ranks"] = plan.ranks.numpy()
        outs[f"g{g}_tasks"] = plan.tasks.numpy()
    np.savez_compressed(os.path.join(HERE, "reverse_plan.npz"), digest=cases.digest(sel), **outs)

    # 6. combine (attention/kv_centric/reference.py:34-39)
    partial, lses = cases.combine_case()
    o, lse = kvref.combine_reference(partial, lses)
    np.savez_compressed(os.path.join(HERE, "combine.npz"), o=o.numpy(), lse=lse.numpy(),
                        digest=cases.digest(partial, lses))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/a/checkout/of/the/reference")
    main(sys.argv[1])
