"""ctypes binding of libtwb200.so. There is no fallback: a missing or stale library raises.

Same loading discipline as the reference's CUTLASS bridge
(packages/fp4-repair/src/thunderworld_fp4/cutlass/backend.py:24-28, cutlass/artifact.py:8-17):
dlopen a plain C-ABI shared object built offline and check its recorded hashes.
"""
import ctypes
import hashlib
import json
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / 'libtwb200.so'
META_PATH = HERE / 'libtwb200.build.json'

_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


class QuantizeArgs(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ('x', 'prescale', 'sensitivity', 'factor', 'wg', 'alpha', 'codes', 'scales',
                                   'scales_swz', 'mask', 'workspace')] + \
               [(n, _i) for n in ('m', 'k', 'mp', 'repair', 'na', 'factor_given')] + \
               [(n, _f) for n in ('base', 'res', 'gain', 'energy')] + [('swz_rows', _i)]


class RepairIO(ctypes.Structure):
    """Reference RepairIO (cutlass/backend.py:10-12) + bank_blocks + atom-layout residual scales."""
    _fields_ = [(n, _vp) for n in ('ac', 'ascale', 'wc', 'ws', 'wr', 'wrs', 'wi', 'off', 'wloc', 'mask')] + \
               [(n, _i) for n in ('m', 'mp', 'n', 'k', 'na', 'hasw', 'cross', 'shared', 'dense', 'bank_blocks')] + \
               [(n, _vp) for n in ('a1s_swz', 'wrs_swz', 'bias')] + [('mask_per_n', _i), ('kernel', _i), ('activation', _i),
                ('stats', _vp), ('stats_scratch', _vp)]


_ll = ctypes.c_longlong


class PackRowsArgs(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ('x', 'codes', 'scales', 'scales_swz', 'factors', 'energy')] + \
               [(n, _ll) for n in ('stride_row', 'stride_head')] + \
               [(n, _i) for n in ('rows', 'heads', 'rows_padded', 'repair', 'transpose_v', 'need_energy')]


class SelectArgs(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ('q', 'k', 'energy', 'flags', 'pvflags', 'counts', 'pvcounts')] + \
               [(n, _ll) for n in ('q_stride_row', 'q_stride_head', 'k_stride_row', 'k_stride_head')] + \
               [(n, _i) for n in ('m', 'n', 'hq', 'hk', 'terms', 'pv_terms')]


class AttentionArgs(ctypes.Structure):
    _fields_ = [(n, _vp) for n in ('qc', 'kc', 'vc', 'sfq', 'sfk', 'sfv', 'qf', 'kf', 'vf', 'flags', 'pvflags', 'out',
                                   'workspace')] + \
               [(n, _i) for n in ('m', 'n', 'hq', 'hk', 'mp', 'np', 'repair', 'full', 'terms', 'pv_repair', 'pv_full',
                                  'pv_terms')]


_lib = None


def _sha(path):
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()


def load():
    """Return the loaded library; raise RuntimeError if it has not been built or fails its hash check."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists() or not META_PATH.exists():
        raise RuntimeError(f'{LIB_PATH.name} is not built; run `python -m thunderworld_b200.build` '
                           '(nvcc, sm_100a). There is no CPU or Triton fallback.')
    meta = json.loads(META_PATH.read_text())
    if meta.get('library_sha256') != _sha(LIB_PATH):
        raise RuntimeError('libtwb200.so does not match its build record; rebuild it')
    from . import build as _build
    if meta.get('sources_sha256') != _build.source_hash():
        raise RuntimeError('libtwb200.so was built from other sources than the ones beside it; rebuild it '
                           '(`python -m thunderworld_b200.build`)')
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.tw_status.argtypes = [_i]; lib.tw_status.restype = ctypes.c_char_p
    lib.tw_abi_version.argtypes = []; lib.tw_abi_version.restype = _i
    lib.tw_quantize_workspace.argtypes = [_i, _i]; lib.tw_quantize_workspace.restype = ctypes.c_size_t
    lib.tw_quantize.argtypes = [ctypes.POINTER(QuantizeArgs), _vp]; lib.tw_quantize.restype = _i
    lib.tw_quantize_static.argtypes = [ctypes.POINTER(QuantizeArgs), _vp]; lib.tw_quantize_static.restype = _i
    lib.tw_quantize_static_max_tiles.argtypes = []; lib.tw_quantize_static_max_tiles.restype = _i
    lib.tw_swizzle_scales.argtypes = [_vp, _i, _i, _vp, _vp]; lib.tw_swizzle_scales.restype = _i
    lib.tw_activation_rank.argtypes = [_vp, _vp, _i, _i, _vp, _vp]; lib.tw_activation_rank.restype = _i
    lib.tw_selftest_bounded_wait.argtypes = [_vp, _ll, _vp]; lib.tw_selftest_bounded_wait.restype = _i
    lib.tw_workspace.argtypes = [_i] * 3; lib.tw_workspace.restype = ctypes.c_size_t
    lib.tw_fused.argtypes = [_i] * 3 + [_vp] * 8 + [ctypes.POINTER(RepairIO)]; lib.tw_fused.restype = _i
    lib.tw_fused_tile_n.argtypes = [_i]; lib.tw_fused_tile_n.restype = _i
    for name, args in (('tw_pack_rows', PackRowsArgs), ('tw_select_tiles', SelectArgs), ('tw_attention', AttentionArgs)):
        getattr(lib, name).argtypes = [ctypes.POINTER(args), _vp]
        getattr(lib, name).restype = _i
    lib.tw_attention_workspace.argtypes = [_i] * 4; lib.tw_attention_workspace.restype = ctypes.c_size_t
    lib.tw_activate.argtypes = [_vp] * 5 + [_ll, _i, _vp]; lib.tw_activate.restype = _i
    lib.tw_rms_norm.argtypes = [_vp] * 7 + [_i] * 3 + [ctypes.c_float, _vp]; lib.tw_rms_norm.restype = _i
    lib.tw_rms_norm_heads.argtypes = [_vp, _vp, _ll, _i, _ll, _ll, ctypes.c_float, _vp]; lib.tw_rms_norm_heads.restype = _i
    lib.tw_rope_heads.argtypes = [_vp, _vp, _ll, _i, _ll, _ll, _vp, _vp, _ll, _i, _i, ctypes.c_float, _vp]; lib.tw_rope_heads.restype = _i
    lib.tw_gate_residual.argtypes = [_vp] * 3 + [_i] * 3 + [_vp]; lib.tw_gate_residual.restype = _i
    _lib = lib
    return lib


calls = 0        # C-ABI calls that returned success (the benchmark reports them as its launch count)


def check(status):
    global calls
    calls += 1
    if status:
        raise RuntimeError(load().tw_status(status).decode())


EXPORTS = ('tw_status', 'tw_abi_version', 'tw_quantize_workspace', 'tw_quantize', 'tw_quantize_static',
           'tw_quantize_static_max_tiles', 'tw_swizzle_scales', 'tw_activation_rank', 'tw_selftest_bounded_wait',
           'tw_workspace', 'tw_fused', 'tw_fused_tile_n', 'tw_pack_rows', 'tw_select_tiles', 'tw_attention',
           'tw_attention_workspace', 'tw_activate', 'tw_rms_norm', 'tw_rms_norm_heads', 'tw_rope_heads', 'tw_gate_residual')
