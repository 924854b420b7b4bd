"""flashloop_b200: B200-native kernels for FlashLoop's late-loop decode path.

Same module and symbol names as the reference's ``flashloop`` package for the parts
of the decode hot path it replaces (``packing``, ``kivi_backend``, ``selection``,
``cache``, ``prefill``, ``engine``, ``config``).  The kernels are hand-written CUDA for sm_100a behind a C ABI
(``include/flashloop_b200.h``); there is no Triton path, no backend dispatch and no
CPU fallback.
"""

from .cache import CrossLoopKVCache, CrossLoopKVLayer, CrossLoopKVLayerBuilder
from .config import FlashLoopConfig
from .engine import DecodeOutput, DecodeReceipt, EngineState, FlashLoopEngine, PrefillOutput
from .kivi_backend import KiviPacked4Bit, pack_kivi_k_per_channel, pack_kivi_v_per_token
from .packing import Packed4Bit, pack_k_per_channel, pack_v_per_token
from .selection import DecodeSelection, select_decode_keys, select_prefill_tokens

__all__ = [
    "CrossLoopKVCache",
    "CrossLoopKVLayer",
    "CrossLoopKVLayerBuilder",
    "DecodeOutput",
    "DecodeReceipt",
    "DecodeSelection",
    "EngineState",
    "FlashLoopConfig",
    "FlashLoopEngine",
    "KiviPacked4Bit",
    "Packed4Bit",
    "PrefillOutput",
    "pack_k_per_channel",
    "pack_kivi_k_per_channel",
    "pack_kivi_v_per_token",
    "pack_v_per_token",
    "select_decode_keys",
    "select_prefill_tokens",
]
