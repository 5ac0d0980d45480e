"""B200 (sm_100a) implementation of ThunderWorld's selective-FP4-repair hot path.

Public surface follows the reference package `thunderworld_fp4`
(packages/fp4-repair/src/thunderworld_fp4/__init__.py): importing configuration needs no CUDA; the
operators load lazily. Every operator calls hand-written CUDA through the C ABI in `include/twb200.h`;
nothing falls back to another backend.
"""
from .config import (PRESETS, RepairConfig, RepairPolicy, RepairRule, preset, LinearRepairConfig, InferenceConfig)
from .head_finding import config_from_head_scores, make_repair_mask, policy_from_head_atlas

__version__ = '0.1.0'
__all__ = ['PRESETS', 'RepairConfig', 'RepairPolicy', 'RepairRule', 'preset', 'fp4_attention', 'FP4Attention',
           'LinearRepairConfig', 'InferenceConfig', 'FP4Linear', 'Native', 'config_from_head_scores',
           'make_repair_mask', 'policy_from_head_atlas']


def fp4_attention(*args, **kwargs):
    from .runtime import fp4_attention as implementation
    return implementation(*args, **kwargs)


def __getattr__(name):
    if name == 'FP4Attention':
        from .runtime import FP4Attention
        return FP4Attention
    if name == 'FP4Linear':
        from .linear import FP4Linear
        return FP4Linear
    if name == 'Native':
        from .native import Native
        return Native
    raise AttributeError(name)
