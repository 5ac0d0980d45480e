"""Thin torch-facing wrappers: pass data_ptr()s and the current stream to the C ABI.

Host-side mirror of the reference's packers and launch wrappers:
  _pack                 thunderworld_fp4/linear.py:13-25
  pack (calibrated)     thunderworld_fp4/_calibrated.py:60-71
  pack_sparse           thunderworld_fp4/_sparse_pack.py:77-93
  pack_with_factor      thunderworld_fp4/_fusion.py:37-42
  pack_input / swizzle  thunderworld_fp4/cutlass/packing.py:85-109, cutlass/layout.py:16-25
  CutlassFused.run_packed  thunderworld_fp4/cutlass/backend.py:48-71
torch is used for device memory and streams only.
"""
import ctypes
from dataclasses import dataclass
import torch
from . import _lib


def cdiv(a, b):
    return (a + b - 1) // b


def require_sm100(device):
    if device.type != 'cuda':
        raise ValueError('a CUDA device is required')
    if torch.cuda.get_device_capability(device)[0] != 10:
        raise RuntimeError('thunderworld_b200 kernels are built for sm_100a (B200) only; no fallback exists')


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(device):
    return torch.cuda.current_stream(device).cuda_stream


@dataclass
class Packed:
    """Quantized activation: the reference's (codes, scales, factor, mp) tuple plus the atom-layout
    scales and alpha that the fused GEMM reads (reference: cutlass/packing.py CutlassPacked)."""
    codes: torch.Tensor          # uint8 [planes, mp, k/2]
    scales: torch.Tensor         # float8_e4m3fn [planes, mp, k/16]
    factor: torch.Tensor         # float32 scalar
    mp: int
    scales_swz: torch.Tensor     # uint8 [planes, ceil(m/128)*128, k/16] atom layout
    alpha: torch.Tensor          # float32 scalar = factor * wg (when wg was given)
    mask: torch.Tensor           # bool [ceil(m/128), k/128] or None

    @property
    def native(self):
        return self.codes, self.scales, self.factor, self.mp

    def __iter__(self):          # unpack like the reference tuple
        return iter(self.native)


# One scratch buffer per device and kernel family, shared by every call: like the reference engine,
# callers issue one request at a time on one stream (docs/INFERENCE.md:51 of the reference).
_workspaces = {}


def _workspace(device, nbytes, key):
    ws = _workspaces.get((device, key))
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 256), device=device, dtype=torch.uint8)
        _workspaces[(device, key)] = ws
    return ws


def quantize(x, prescale=None, *, repair=1, mask=None, na=0, sensitivity=None, factor=None, wg=None,
             base=1., res=1., gain=1., energy=1., workspace=None, out=None):
    """bf16 [m,k] -> Packed. repair: 0 base only, 1 full residual, 2 residual under `mask`,
    3 online selection of `na` K128 blocks per M128 row block (mask is written)."""
    if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError('expected contiguous BF16 [M,K]')
    require_sm100(x.device)
    m, k = x.shape
    if m == 0:
        raise ValueError('empty activation rows are unsupported')
    if k % 128:
        raise ValueError('K must be a multiple of 128')
    lib = _lib.load()
    # with preallocated outputs the planes may hold more rows than m (a shard of a larger gathered tensor)
    mp = cdiv(m, 16) * 16 if out is None else int(out.codes.shape[1])
    mb = cdiv(m, 128)
    if mp < cdiv(m, 16) * 16:
        raise ValueError('preallocated planes are too small')
    planes = 2 if repair else 1
    dev = x.device
    if out is None:
        codes = torch.empty((planes, mp, k // 2), device=dev, dtype=torch.uint8)
        scales = torch.empty((planes, mp, k // 16), device=dev, dtype=torch.float8_e4m3fn)
        swz = torch.empty((planes, mb * 128, k // 16), device=dev, dtype=torch.uint8)
        fac = torch.empty((), device=dev, dtype=torch.float32) if factor is None else factor
        alpha = torch.empty((), device=dev, dtype=torch.float32)
        if repair == 3 and mask is None:
            mask = torch.empty((mb, k // 128), device=dev, dtype=torch.bool)
    else:
        codes, scales, swz, fac, alpha = out.codes, out.scales, out.scales_swz, out.factor, out.alpha
        mask = out.mask if mask is None else mask
    if repair in (2, 3) and (mask is None or mask.dtype != torch.bool or tuple(mask.shape) != (mb, k // 128)
                             or not mask.is_contiguous()):
        raise ValueError(f'mask must be contiguous bool {(mb, k // 128)}')
    if workspace is None:
        workspace = _workspace(dev, lib.tw_quantize_workspace(m, k), 'q')
    args = _lib.QuantizeArgs(_ptr(x), _ptr(prescale), _ptr(sensitivity), _ptr(fac), _ptr(wg), _ptr(alpha),
                             _ptr(codes), _ptr(scales), _ptr(swz), _ptr(mask), _ptr(workspace),
                             m, k, mp, int(repair), int(na), int(factor is not None),
                             float(base), float(res), float(gain), float(energy), int(swz.shape[1]))
    with torch.cuda.device(dev):
        _lib.check(lib.tw_quantize(ctypes.byref(args), _stream(dev)))
    return Packed(codes, scales, fac, mp, swz, alpha, mask)


def swizzle(scales):
    """Row-major E4M3 [rows, cols] -> atom layout uint8 [ceil(rows/128)*128, cols]."""
    if scales.dtype not in (torch.float8_e4m3fn, torch.uint8) or not scales.is_contiguous() or scales.ndim != 2:
        raise ValueError('Contiguous E4M3 scales required')
    rows, cols = scales.shape
    if cols % 4:
        raise ValueError('Scale columns must be divisible by four')
    require_sm100(scales.device)
    out = torch.empty((cdiv(rows, 128) * 128, cols), device=scales.device, dtype=torch.uint8)
    with torch.cuda.device(scales.device):
        _lib.check(_lib.load().tw_swizzle_scales(scales.data_ptr(), rows, cols, out.data_ptr(), _stream(scales.device)))
    return out


def activation_rank(x, prescale=None):
    """int32 [ceil(m/128), k/128]: rank of every K128 block within its M128 row block by sampled energy
    (reference: activation_rank, thunderworld_fp4/_linear_kernels.py:23-34). One launch, no host sync."""
    if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.shape[1] % 128 or x.shape[0] == 0:
        raise ValueError('expected contiguous BF16 [M,K] with K a multiple of 128')
    require_sm100(x.device)
    m, k = x.shape
    rank = torch.empty((cdiv(m, 128), k // 128), device=x.device, dtype=torch.int32)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().tw_activation_rank(_ptr(x), _ptr(prescale), m, k, _ptr(rank), _stream(x.device)))
    return rank


def selftest_bounded_wait(device=None, limit_cycles=2_000_000):
    """Make a bounded device-side wait run out on purpose (a barrier nothing signals) and return the status word
    that `device_status` then reports; the word is left set so that the caller can see and reset it."""
    dev = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
    ws = _workspace(dev, 256, 'g')
    with torch.cuda.device(dev):
        _lib.check(_lib.load().tw_selftest_bounded_wait(_ptr(ws), int(limit_cycles), _stream(dev)))
    return device_status(dev)


def fused_gemm(m, n, k, packed, wc, ws_swz, alpha, *, na=0, mask=None, wr=None, wrs_swz=None, wi=None, off=None,
               wloc=None, cross=False, shared=False, dense=False, ws=None, wrs=None, out=None, workspace=None,
               mask_per_n=False, bias=None, kernel=0, activation=None, want_stats=False):
    """One launch of the repaired GEMM; returns bf16 [m,n]. activation='gelu_tanh' applies the activation to the
    bf16-rounded result in the epilogue (the bits activate_with_factor would give); with want_stats the call returns
    (out, stats) with stats = float32 [2] = (max|out| / 2688, max|out|)."""
    lib = _lib.load()
    dev = wc.device
    require_sm100(dev)
    if out is None:
        out = torch.empty((m, n), device=dev, dtype=torch.bfloat16)
    if workspace is None:
        workspace = _workspace(dev, lib.tw_workspace(m, n, k), 'g')
    hasw = wr is not None and wr.numel() > 0
    a0s = packed.scales_swz[0]
    a1s = packed.scales_swz[1] if packed.scales_swz.shape[0] > 1 else None
    io = _lib.RepairIO(_ptr(packed.codes), _ptr(packed.scales), _ptr(wc), _ptr(ws), _ptr(wr) if hasw else None,
                       _ptr(wrs) if hasw else None, _ptr(wi), _ptr(off), _ptr(wloc), _ptr(mask),
                       m, packed.mp, n, k, int(na), int(hasw), int(cross), int(shared), int(dense),
                       int(wr.shape[0]) if hasw else 0, _ptr(a1s) if na else None, _ptr(wrs_swz) if hasw else None,
                       _ptr(bias), int(mask_per_n), int(kernel), 0, None, None)
    stats = None
    if activation is not None:
        if activation != 'gelu_tanh':
            raise ValueError('the GEMM epilogue fuses gelu_tanh only')
        io.activation = ACT_MODES[activation]
        if want_stats:
            stats, scratch = _stats(dev, True)
            io.stats, io.stats_scratch = _ptr(stats), _ptr(scratch)
    elif want_stats:
        raise ValueError('stats come with a fused activation')
    with torch.cuda.device(dev):
        _lib.check(lib.tw_fused(m, n, k, packed.codes.data_ptr(), wc.data_ptr(), a0s.data_ptr(), ws_swz.data_ptr(),
                                out.data_ptr(), alpha.data_ptr(), workspace.data_ptr(), _stream(dev), ctypes.byref(io)))
    return (out, stats) if want_stats else out


STATUS_KEYS = {'g': 0, 'a': 0, 'q': 8}   # workspace -> byte offset of its device status word: fused GEMM, attention, quantizer


def device_status(device=None):
    """Worst status word any kernel of this device wrote on a bounded-wait timeout (0 = none); synchronises.
    Covers the fused GEMM, the attention kernel and the single-pass quantizer's grid barrier: each writes into its own workspace."""
    dev = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:
        dev = torch.device('cuda', torch.cuda.current_device())
    worst = 0
    for key, offset in STATUS_KEYS.items():
        ws = _workspaces.get((dev, key))
        if ws is not None:
            worst = max(worst, int(ws[offset:offset + 4].view(torch.int32).item()))
    return worst


def reset_device_status(device=None):
    """Clear the status words (after a reported timeout has been handled)."""
    dev = torch.device('cuda', torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:
        dev = torch.device('cuda', torch.cuda.current_device())
    for key, offset in STATUS_KEYS.items():
        ws = _workspaces.get((dev, key))
        if ws is not None:
            ws[offset:offset + 4].zero_()


# ---- pointwise producers with fused tensor factor -----------------------------------------------
# Host mirrors of activate_with_factor (thunderworld_fp4/_fusion.py:26-34) and nemotron_norm
# (thunderworld_fp4/cosmos/norm_fusion.py:29-43); same argument checks and error types.
ACT_MODES = {'relu2': 0, 'mul': 1, 'gelu_tanh': 2}


def _check_bf16(*tensors):
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError('expected contiguous CUDA BF16 tensors')


def _stats(device, want):
    """(stats[2] float32, scratch) or (None, None). The scratch word pair is zeroed once per device."""
    if not want:
        return None, None
    return torch.empty(2, device=device, dtype=torch.float32), _workspace(device, 8, 'pointwise')


def activate_with_factor(a, b=None, *, mode=None, want_factor=True, return_stats=False):
    """y = relu(a)^2 (b None), a * b, or gelu_tanh(a) (mode='gelu_tanh'); returns (y, factor) with
    factor = max|y| / 2688 as a 0-d float32 tensor (or None); return_stats: the pair (factor, max|y|) instead."""
    if torch.is_grad_enabled() and (a.requires_grad or (b is not None and b.requires_grad)):
        raise RuntimeError('fused activations are inference only')
    _check_bf16(a, b)
    if b is not None and b.shape != a.shape:
        raise ValueError('operands must have equal shapes')
    require_sm100(a.device)
    mode = ACT_MODES[mode or ('relu2' if b is None else 'mul')]
    y = torch.empty_like(a)
    stats, scratch = _stats(a.device, want_factor)
    _lib.check(_lib.load().tw_activate(_ptr(a), _ptr(b), _ptr(y), _ptr(stats), _ptr(scratch), a.numel(), mode, _stream(a.device)))
    return y, (None if stats is None else (stats if return_stats else stats[0]))


def rms_norm(x, weight=None, eps=1e-6, *, shift=None, scale=None, want_factor=False, return_stats=False):
    """RMSNorm over the last dimension, optional weight, optional AdaLN modulation with shift/scale of shape
    [batch, hidden] (x is [batch, tokens, hidden]). Returns y or (y, factor); return_stats: (y, (factor, max|y|))."""
    if torch.is_grad_enabled() and x.requires_grad:
        raise RuntimeError('Fused RMSNorm requires inference mode')
    _check_bf16(x, weight, shift, scale)
    hidden = x.shape[-1]
    if weight is not None and weight.numel() != hidden:
        raise ValueError('Fused RMSNorm supports BF16 inputs matching the weight')
    if (shift is None) != (scale is None):
        raise ValueError('shift and scale come together')
    rows = x.numel() // hidden
    per_batch = rows
    if shift is not None:
        if shift.shape != scale.shape or shift.shape[-1] != hidden or rows % (shift.numel() // hidden):
            raise ValueError('shift/scale must be [batch, hidden] with batch dividing the rows of x')
        per_batch = rows // (shift.numel() // hidden)
    require_sm100(x.device)
    y = torch.empty_like(x)
    stats, scratch = _stats(x.device, want_factor)
    _lib.check(_lib.load().tw_rms_norm(_ptr(x), _ptr(weight), _ptr(shift), _ptr(scale), _ptr(y), _ptr(stats), _ptr(scratch),
                                       rows, hidden, per_batch, float(eps), _stream(x.device)))
    if not want_factor:
        return y
    return (y, stats) if return_stats else (y, stats[0])


def rms_norm_heads(x, eps=1e-6):
    """RMSNorm over head_dim = 128 of a (possibly strided) view [..., tokens, heads, 128] whose leading
    dimensions fold into the token stride; returns a contiguous tensor of the same shape."""
    if x.dtype != torch.bfloat16 or not x.is_cuda or x.shape[-1] != 128 or x.stride(-1) != 1:
        raise ValueError('expected a CUDA BF16 view [..., heads, 128] with unit inner stride')
    require_sm100(x.device)
    heads = x.shape[-2]
    lead = x.reshape(-1, heads, 128) if x.dim() != 3 else x       # a view when the leading dims are foldable
    if lead.data_ptr() != x.data_ptr():
        raise ValueError('leading dimensions must fold into one token stride')
    y = torch.empty(x.shape, device=x.device, dtype=x.dtype)
    _lib.check(_lib.load().tw_rms_norm_heads(_ptr(lead), _ptr(y), lead.shape[0], heads, lead.stride(0), lead.stride(1),
                                             float(eps), _stream(x.device)))
    return y


def rope_heads(x, cos, sin, *, norm=False, eps=1e-6):
    """Rotary embedding of a (possibly strided) bf16 view [..., tokens, heads, 128] with the reference's rounding
    sequence (fused_rope, thunderworld_fp4/cosmos/pipeline_tuning.py:57-63); cos / sin [table_rows, 128], float32 or
    bf16, row token % table_rows. norm=True runs the head RMSNorm first in the same pass. Returns a contiguous tensor."""
    if x.dtype != torch.bfloat16 or not x.is_cuda or x.shape[-1] != 128 or x.stride(-1) != 1:
        raise ValueError('expected a CUDA BF16 view [..., heads, 128] with unit inner stride')
    if cos.shape != sin.shape or cos.ndim != 2 or cos.shape[1] != 128 or cos.dtype != sin.dtype or \
            cos.dtype not in (torch.float32, torch.bfloat16) or not cos.is_contiguous() or not sin.is_contiguous():
        raise ValueError('cos / sin must be contiguous [rows, 128] tables of one dtype (float32 or bfloat16)')
    require_sm100(x.device)
    heads = x.shape[-2]
    lead = x.reshape(-1, heads, 128) if x.dim() != 3 else x
    if lead.data_ptr() != x.data_ptr():
        raise ValueError('leading dimensions must fold into one token stride')
    y = torch.empty(x.shape, device=x.device, dtype=x.dtype)
    _lib.check(_lib.load().tw_rope_heads(_ptr(lead), _ptr(y), lead.shape[0], heads, lead.stride(0), lead.stride(1), _ptr(cos),
                                         _ptr(sin), cos.shape[0], int(cos.dtype == torch.bfloat16), int(norm), float(eps),
                                         _stream(x.device)))
    return y


def gate_residual_(x, gate, y):
    """x += gate[:, None, :] * y in place; x, y [batch, tokens, hidden], gate [batch, hidden]."""
    _check_bf16(x, gate, y)
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    if y.shape != x.shape or gate.shape[-1] != hidden or rows % (gate.numel() // hidden):
        raise ValueError('shapes do not match')
    require_sm100(x.device)
    _lib.check(_lib.load().tw_gate_residual(_ptr(x), _ptr(gate), _ptr(y), rows, hidden, rows // (gate.numel() // hidden),
                                            _stream(x.device)))
    return x
