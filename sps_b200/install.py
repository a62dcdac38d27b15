"""Drop the CUDA kernels into the reference model classes by rebinding module-level names.

The reference reaches its attention kernels through plain module attributes
(src/modeling/models/sps/core.py:68, reverse_sps/core.py:85, full_attention_model.py:110 and
:550, reverse_sps/inference.py:312, :354, :206); ``install()`` points each of them at the
function of the same signature in this package.  It needs the reference's ``modeling`` package
on ``sys.path`` and does nothing else to it.  The three prefill functions are autograd functions
(head_dim 64 and 128), so a model bound this way trains through them as it does through the
reference's (triton_sps_flash_attention.py:491-720); the decode functions are for generation
and refuse inputs that require grad.
"""

from __future__ import annotations

import importlib

from . import attention, decode

_BINDINGS = (
    ("modeling.models.sps.core", "triton_sps_sliding_attention", attention.sps_sliding_attention),
    ("modeling.models.reverse_sps.core", "triton_reverse_sps_sliding_attention",
     attention.reverse_sps_sliding_attention),
    ("modeling.models.delayed_state.core", "triton_reverse_sps_sliding_attention",
     attention.reverse_sps_sliding_attention),
    ("modeling.models.full_attention_model", "triton_full_attention", attention.full_attention),
    ("modeling.models.full_attention_model", "masked_kv_attention", decode.masked_kv_attention),
    ("modeling.models.reverse_sps.inference", "triton_segmented_q2_attention",
     decode.segmented_q2_attention),
    ("modeling.models.reverse_sps.inference", "masked_kv_attention", decode.masked_kv_attention),
    ("modeling.models.reverse_sps.inference", "fused_sps_kv_update", decode.fused_sps_kv_update),
)


def install(strict: bool = False) -> list:
    """Rebind every reference name that exists; returns the list of (module, name) rebound.
    With ``strict`` a missing module or attribute raises instead of being skipped."""
    done = []
    for mod_name, attr, fn in _BINDINGS:
        try:
            mod = importlib.import_module(mod_name)
        except Exception:
            if strict:
                raise
            continue
        if not hasattr(mod, attr):
            if strict:
                raise AttributeError(f"{mod_name} has no attribute {attr}")
            continue
        setattr(mod, attr, fn)
        done.append((mod_name, attr))
    return done
