"""B200-native block-sparse attention hot path (host-side mirror of the reference interface)."""
from ._lib import SparseB200Error, device_status, lib  # noqa: F401
from .q_centric import attention, attention_out, attention_partial_out, stage_functions  # noqa: F401
