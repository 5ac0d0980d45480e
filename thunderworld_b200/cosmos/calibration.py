"""Calibration-side tooling of the repaired linear: per-channel prescale proposals, the outlier proposal that
reserves W1 tiles, and the CPU weight encoder that honours it. Host-side, CPU-runnable, pure torch.

Mirrors packages/fp4-repair/src/thunderworld_fp4/cosmos/calibration.py:5-73 (prescale_candidates, panel_objective,
decode, quantize_weight, outlier_mask) so that assets prepared by either code base interchange: same candidate
names and clamps, same byte formats, same mandatory-tile rule. The GPU path never calls this module at run time;
`native.quantize_weight` is the device-side encoder for weights that carry no outlier removal.
"""
import torch

_LEVELS = (0., .5, 1., 1.5, 2., 3., 4., 6.)
_EDGES = (.25, .75, 1.25, 1.75, 2.5, 3.5, 5.)


def _balanced(s):
    """Scale a positive vector so that min * max == 1 (geometric centring)."""
    return s / (s.min() * s.max()).sqrt()


def prescale_candidates(rms, weight):
    """Yield (name, d): X is multiplied by d before its bf16 rounding, W is divided by d (X d) @ (W / d)^T.
    `rms`: per-input-channel activation RMS [K]; `weight` [N, K]. Every d lies in [1/16, 16]."""
    rms = rms.float().clamp_min(1e-6)
    wmax = weight.float().abs().amax(0).clamp_min(1e-6)
    yield 'identity', torch.ones_like(rms)
    for alpha in (0., .25, .5, .75, 1.):
        s = _balanced(rms.pow(alpha) / wmax.pow(1 - alpha))          # AWQ-style s: activations shrink by s
        yield f'awq_alpha_{alpha:g}', (1 / s).clamp(1 / 16, 16)
    legacy = (rms.sqrt() / wmax.sqrt()).clamp(1 / 16, 16)            # the earlier orientation, kept as a control
    yield 'legacy_orientation', _balanced(legacy).clamp(1 / 16, 16)


def panel_objective(errors):
    """Score of a candidate over calibration panels: mean error plus a quarter of the worst panel."""
    errors = list(errors)
    if not errors:
        raise ValueError('No calibration panels')
    return sum(errors) / len(errors) + .25 * max(errors)


def decode(codes, scales, factor):
    """codes u8 [..., K/2] (even k in the low nibble), scales [..., K/16], factor -> float32 [..., K]."""
    levels = torch.tensor(_LEVELS, device=codes.device)
    ids = torch.stack((codes & 15, codes >> 4), -1).flatten(-2).long()
    value = levels[ids & 7] * torch.where(ids >= 8, -1., 1.)
    return (value.unflatten(-1, (-1, 16)) * scales.float()[..., None]).flatten(-2) * factor


def _encode(z, multiplier):
    groups = z.unflatten(-1, (-1, 16))
    scales = (groups.abs().amax(-1) * multiplier / 6).clamp(2. ** -9, 448.).to(torch.float8_e4m3fn)
    v = (groups / scales.float()[..., None]).flatten(-2)
    mag = v.abs()
    ids = torch.zeros_like(mag, dtype=torch.uint8)
    for i, edge in enumerate(_EDGES):                # round to nearest code, exact midpoints to the even code
        ids += (mag >= edge) if i % 2 else (mag > edge)
    ids |= torch.signbit(v).to(torch.uint8) << 3
    return ids[..., 0::2] | (ids[..., 1::2] << 4), scales


def quantize_weight(weight, prescale, *, base=1., residual=1., remove=None):
    """Offline NVFP4 encoder of W / d: (codes u8 [2, N, K/2], scales e4m3 [2, N, K/16], factor). Elements under
    `remove` (outlier proposal) are zeroed in the base plane only, so the residual plane carries them whole."""
    w = (weight.float() / prescale).bfloat16().float()
    peak = w.abs().amax()
    factor = torch.where(peak > 0, peak / torch.full_like(peak, 2688.), torch.ones_like(peak))   # tensor divisor: IEEE division on any device
    z = w / factor
    c0, s0 = _encode(z if remove is None else z.masked_fill(remove, 0.), base)
    c1, s1 = _encode(z - decode(c0, s0, torch.ones_like(factor)), residual)
    return torch.stack((c0, c1)), torch.stack((s0, s1)), factor


def outlier_mask(weight, prescale, activation_rms, reserved_blocks, threshold):
    """At most one contribution outlier per group of 16 along K, only inside the reserved W1 tiles.
    Returns (bool mask [N, K], tuple of tile ids nb*KB + kb that thereby become mandatory)."""
    n, k = weight.shape
    if n % 128 or k % 128 or threshold not in (None, 2., 3.):
        raise ValueError('Invalid outlier proposal')
    mask = torch.zeros_like(weight, dtype=torch.bool)
    if threshold is None:
        return mask, ()
    groups = (weight.float().abs() * activation_rms[None, :]).unflatten(1, (k // 16, 16))
    peak, index = groups.max(-1)
    hit = peak > threshold * groups.square().mean(-1).sqrt()
    allowed = torch.zeros(n // 128 * (k // 128), device=weight.device, dtype=torch.bool)
    ids = torch.as_tensor(reserved_blocks, device=weight.device, dtype=torch.long)
    if ids.numel():
        allowed[ids] = True
    hit &= allowed.reshape(n // 128, k // 128).repeat_interleave(128, 0).repeat_interleave(8, 1)
    mask.unflatten(1, (k // 16, 16)).scatter_(2, index[..., None], hit[..., None])
    tiles = mask.reshape(n // 128, 128, k // 128, 128).any(3).any(1).flatten().nonzero().flatten().tolist()
    return mask, tuple(tiles)
