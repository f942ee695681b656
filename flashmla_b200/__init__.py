"""flashmla_b200: B200 (sm_100a) MLA decode / sparse-prefill kernels behind the FlashMLA Python API."""
from .flash_mla_interface import (
    FlashMLASchedMeta,
    get_mla_metadata,
    flash_mla_with_kvcache,
    flash_mla_sparse_fwd,
    set_impl,
    check_status,
)

__all__ = [
    "FlashMLASchedMeta",
    "get_mla_metadata",
    "flash_mla_with_kvcache",
    "flash_mla_sparse_fwd",
    "set_impl",
    "check_status",
]
