"""sps_b200: the SPS Transformer attention hot path as hand-written sm_100a CUDA.

The package is a thin host layer over ``libspsattn.so`` (C ABI in ``include/spsattn.h``):
prefill attention (``attention``), segmented decode attention and the decode KV-cache
update (``decode``), ``install()`` which rebinds the reference model classes to them, and
``generation`` (``SPSGenerator``): batched prefill + graph-replayed greedy decode of the
reference's decoder around those kernels.
"""

from . import _lib
from .attention import (check_device_status, full_attention, prefill_attention,
                        reverse_sps_sliding_attention, rope_cast, sps_sliding_attention)
from .decode import (KVSegment, PackedKVSegment, decode_attention, fill_decode_caches, fused_sps_kv_update,
                     masked_kv_attention, segmented_q1_attention, segmented_q2_attention,
                     triton_segmented_q2_attention)
from .generation import SPSDims, SPSGenerator, bind_generate, generator_for
from .install import install

__all__ = [
    "KVSegment", "PackedKVSegment", "SPSDims", "SPSGenerator", "bind_generate", "generator_for",
    "check_device_status", "decode_attention", "fill_decode_caches",
    "full_attention",
    "fused_sps_kv_update", "install", "masked_kv_attention", "prefill_attention",
    "reverse_sps_sliding_attention", "rope_cast", "segmented_q1_attention", "segmented_q2_attention",
    "sps_sliding_attention", "triton_segmented_q2_attention",
]
