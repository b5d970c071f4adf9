"""B200-native block-sparse attention hot path (host-side mirror of the reference interface)."""
from ._lib import SparseB200Error, device_status, lib  # noqa: F401
from .q_centric import attention, attention_out, attention_partial_out, stage_functions  # noqa: F401
from .kv_centric import Prepared, PreparedTokens, kv_centric_attention, combine  # noqa: F401
from .indexers import (SummarySelector, summary_indexed_attention_out, quantize_queries, quantize_keys, prepare_fp4_inputs,  # noqa: F401
                       fp4_block_scores, fp4_block_scores_varlen, tile_topk, tile_topk_out, fp4_indexer, fp4_indexer_fast,
                       indexed_attention, Fp4Pipeline)
from . import sharding  # noqa: F401
from .host_io import HostPipeline  # noqa: F401
