"""CPU oracle for the block-sparse attention hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this module;
it is the checker used by the test-suite, by the smoke check and by the CPU
baseline leg of the benchmark. Every function restates, on the CPU and in
fp32 torch/numpy arithmetic, one function of the reference project and names
the reference file and lines it follows.

Parity status
-------------
* attention / combine / reverse-index / R1-R4 selectors / NVFP4 dequant-score /
  tile top-k: pinned against the untouched reference functions (imported from
  the reference checkout when the golden fixtures were generated; the fixtures
  and the generating script live in tests/golden/).
* bf16 -> NVFP4 quantisation: PARITY UNPINNED. The reference feeds random
  packed bytes to its scorer and contains no quantiser; the rule used here is
  stated in oracle/fp4.py.
"""
from .attention import (masked_attention, gather_attention, combine_partials,
                        expand_block_ids, filter_ids_to_range)
from .selectors import (pool_descriptors, summary_scores, summary_select,
                        stable_topk)
from .fp4 import (quantize_nvfp4, quantize_queries, quantize_keys, group_mean, dequantize_nvfp4, fp4_scores, fp4_scores_varlen, fp4_tile_scores,
                  fp4_select, E2M1_VALUES)
from .metadata import build_reverse_plan, validate_reverse_plan, split_kv_segments
from . import inputs
