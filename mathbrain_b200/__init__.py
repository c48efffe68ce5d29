"""mathbrain_b200: B200 (sm_100a) kernels for MathBrain's Per-Slot-EMA hot path behind the reference's
operator names.  See include/mbema.h for the C ABI underneath."""
import sys
import types

from . import _lib
from .ops import (HAS_TRITON, device_status, check_status, clear_status, status_word, FlashEMAFunction, FlashEMARowsFunction, shared_slot_rows, slot_grad_scatter, SlotLayerNormFunction, project_slot_rows, FusedGatingFunction, TileStates, _build_unique_index,
                  compute_query_ema_history, fused_apply_symmetric_query_gating, get_options, options,
                  precompute_boundaries, set_options)

__all__ = ["HAS_TRITON", "FlashEMAFunction", "FlashEMARowsFunction", "shared_slot_rows", "slot_grad_scatter", "SlotLayerNormFunction", "project_slot_rows", "FusedGatingFunction", "TileStates", "_build_unique_index",
           "compute_query_ema_history", "fused_apply_symmetric_query_gating", "precompute_boundaries",
           "set_options", "device_status", "check_status", "clear_status", "status_word", "get_options", "options", "install_as_mathbrain", "library_path"]


def library_path():
    """Path of the shared library the operators call into."""
    return _lib.LIB_PATH


def install_as_mathbrain():
    """Register modules named like the reference's operator modules (mathbrain.triton_ema_query,
    mathbrain.triton_fused_gating, mathbrain.triton_flash_ema) that resolve to this package's operators, so that
    the reference's `mathbrain/model.py` (its import lines 6-9) picks them up unchanged.  Call it before
    importing `mathbrain.model`; an already imported reference module of the same name is replaced."""
    from . import ops

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    mod("mathbrain.triton_ema_query", HAS_TRITON=True, compute_query_ema_history=ops.compute_query_ema_history)
    mod("mathbrain.triton_fused_gating", HAS_TRITON=True, FusedGatingFunction=ops.FusedGatingFunction,
        fused_apply_symmetric_query_gating=ops.fused_apply_symmetric_query_gating)
    mod("mathbrain.triton_flash_ema", HAS_TRITON=True, FlashEMAFunction=ops.FlashEMAFunction,
        precompute_boundaries=ops.precompute_boundaries, _build_unique_index=ops._build_unique_index)
