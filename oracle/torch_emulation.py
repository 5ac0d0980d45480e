"""Multi-threaded CPU emulation of the repaired NVFP4 linear in torch: TEST AND BASELINE INFRASTRUCTURE ONLY.

A torch restatement of the reference's own PyTorch FP4 emulation for this path, the "reference's PyTorch
emulation path timed on the host CPU cores" that the benchmark reports beside the GPU numbers:

  quantize            thunderworld_fp4/cosmos/calibration.py:30-54  (_encode, quantize_weight: tensor factor
                      max|bf16(x*d)| / 2688, per-16 E4M3 scale clamp(amax*mult/6, 2^-9, 448), E2M1 round to
                      nearest with ties to the even code, residual plane of z - deq(base))
  decode              calibration.py:24-28
  repair_linear       the decoded fp32 matmuls per term of thunderworld_fp4/_native.py:11-62
  select_blocks       the stable-argsort selector of thunderworld_fp4/_sparse_pack.py:46-61

It exists because the numpy oracle (oracle/nvfp4_oracle.py) runs its elementwise quantizer on one thread; this
file uses torch's threaded elementwise kernels and matmuls so that the CPU baseline uses every host core.
tests/test_oracle_torch.py pins it bit for bit to the numpy oracle and to the reference-run fixtures.
Only tests/ and bench.py's cpu_baseline / --impl reference legs may import it.
"""
import torch

EDGES = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)     # midpoints between the E2M1 magnitudes 0 .5 1 1.5 2 3 4 6
LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _e2m1_ids(v):
    """4-bit codes of round-to-nearest(v), ties to the even code, saturating at 6; bit 3 = sign (of zero too)."""
    mag = v.abs()
    ids = torch.zeros_like(mag, dtype=torch.uint8)
    for i, edge in enumerate(EDGES):
        # a value exactly on the midpoint between codes i and i+1 goes to the even one of the two
        ids += (mag >= edge) if i % 2 else (mag > edge)
    return ids | (torch.signbit(v).to(torch.uint8) << 3)


def _encode(z, multiplier):
    g = z.reshape(z.shape[0], -1, 16)
    scales = (g.abs().amax(-1) * multiplier / 6).clamp(2.0 ** -9, 448.0).to(torch.float8_e4m3fn)
    ids = _e2m1_ids((g / scales.float()[..., None]).reshape(z.shape))
    return ids[:, 0::2] | (ids[:, 1::2] << 4), scales


def decode(codes, scales, factor=1.0):
    """codes u8 [..., K/2], scales e4m3 [..., K/16] -> float32 [..., K]."""
    levels = torch.tensor(LEVELS)
    ids = torch.stack((codes & 15, codes >> 4), -1).reshape(*codes.shape[:-1], -1).long()
    val = levels[ids & 7] * torch.where(ids >= 8, -1.0, 1.0)
    return (val.reshape(*scales.shape, 16) * scales.float()[..., None]).reshape(val.shape) * factor


def quantize(x, prescale=None, *, base=1.0, residual=1.0, factor=None):
    """x float32 [R, K] (bf16 values) -> codes u8 [2, R, K/2], scales e4m3 [2, R, K/16], factor (0-d)."""
    y = (x if prescale is None else x * prescale).bfloat16().float()
    if factor is None:
        peak = y.abs().amax()
        factor = torch.where(peak > 0, peak / 2688.0, torch.ones_like(peak))
    z = y / factor
    c0, s0 = _encode(z, base)
    c1, s1 = _encode(z - decode(c0, s0), residual)
    return torch.stack((c0, c1)), torch.stack((s0, s1)), factor


def select_blocks(x, factor, codes0, scales0, sensitivity, count):
    """Top-`count` K128 blocks per M128 row block by sum(residual^2 * sensitivity), lower index wins ties."""
    m, k = x.shape
    r = x - decode(codes0, scales0, factor)
    w = r.double() ** 2 * sensitivity.double()
    mb = (m + 127) // 128
    pad = torch.zeros(mb * 128, k, dtype=torch.float64)
    pad[:m] = w
    score = pad.reshape(mb, 128, k // 128, 128).sum((1, 3))
    idx = torch.argsort(score, dim=1, descending=True, stable=True)[:, :count]
    return torch.zeros(mb, k // 128, dtype=torch.bool).scatter_(1, idx, True)


def repair_linear(ac, asc, af, wc, wsc, wf, m, *, a_mask=None, w_tiles=(), cross=False):
    """bf16( (A0 W0^T + A1|mask W0^T + A0 W1|tiles^T [+ A1|mask W1|tiles^T]) * af * wf ), float32 accumulation."""
    n, k = wc.shape[1], wc.shape[2] * 2
    a0 = decode(ac[0][:m], asc[0][:m])
    w0 = decode(wc[0], wsc[0])
    acc = a0 @ w0.T
    a1 = None
    if a_mask is not None and bool(a_mask.any()):
        a1 = decode(ac[1][:m], asc[1][:m]) * a_mask.repeat_interleave(128, 0)[:m].repeat_interleave(128, 1)
        acc += a1 @ w0.T
    w_tiles = list(w_tiles)
    if w_tiles:
        keep = torch.zeros(n // 128 * (k // 128), dtype=torch.bool)
        keep[w_tiles] = True
        w1 = decode(wc[1], wsc[1]) * keep.reshape(n // 128, k // 128).repeat_interleave(128, 0).repeat_interleave(128, 1)
        acc += a0 @ w1.T
        if cross and a1 is not None:
            acc += a1 @ w1.T
    return (acc * (af * wf)).bfloat16()
