"""B200 (sm_100a) implementation of ThunderWorld's selective-FP4-repair hot path.

Public surface follows the reference package `thunderworld_fp4`
(packages/fp4-repair/src/thunderworld_fp4/__init__.py). Every operator calls hand-written CUDA
through the C ABI in `include/twb200.h`; nothing falls back to another backend.
"""
__version__ = '0.1.0'
