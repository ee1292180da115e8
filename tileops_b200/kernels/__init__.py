from .call_spec import AttentionCall, CallSpec
from .gqa_decode import (
    GQADecodePagedFp8Sm100Kernel,
    GQADecodePagedSm100Kernel,
    GQADecodeSm100Kernel,
    gqa_decode_paged_block_ns,
)
from .gqa_prefill import (
    GQAPrefillPagedFp8CacheSm100Kernel,
    GQAPrefillPagedRopeSm100Kernel,
    GQAPrefillPagedSm100Kernel,
    GQAPrefillSm100Kernel,
    GQAPrefillVarlenSm100Kernel,
    GQASlidingWindowSm100Kernel,
    GQASlidingWindowVarlenSm100Kernel,
)
from .kernel_base import Kernel
from .mha_decode import MHADecodePagedSm100Kernel, MHADecodeSm100Kernel

__all__ = [
    "AttentionCall", "CallSpec", "Kernel", "GQADecodeSm100Kernel", "GQADecodePagedSm100Kernel",
    "GQADecodePagedFp8Sm100Kernel", "GQAPrefillSm100Kernel", "GQAPrefillVarlenSm100Kernel",
    "GQAPrefillPagedSm100Kernel", "GQAPrefillPagedRopeSm100Kernel", "GQAPrefillPagedFp8CacheSm100Kernel", "GQASlidingWindowSm100Kernel", "GQASlidingWindowVarlenSm100Kernel", "gqa_decode_paged_block_ns", "MHADecodeSm100Kernel", "MHADecodePagedSm100Kernel",
]
