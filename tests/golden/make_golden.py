"""Generate the golden fixtures in this folder from the reference's own CPU code.

Run once, where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/ThunderWorld

It imports `thunderworld_fp4.cosmos.calibration` (quantize_weight, decode) and
`packages/fp4-repair/tests/oracle.py` (quant_ref) from that checkout, feeds them
seeded inputs and stores inputs and outputs as small .npz files. The tests read
only the .npz files; the reference is not needed to run them.
"""
import argparse
import os
import sys
import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True)
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, 'packages/fp4-repair/src'))
    sys.path.insert(0, os.path.join(args.reference, 'packages/fp4-repair/tests'))
    import torch
    from thunderworld_fp4.cosmos import calibration
    import oracle as ref_oracle
    here = os.path.dirname(os.path.abspath(__file__))
    torch.manual_seed(0)

    def u8(t):
        return t.view(torch.uint8).numpy() if t.dtype == torch.float8_e4m3fn else t.numpy()

    # 1. tensor-wide-factor quantizer: plain, with outliers, with prescale, calibrated multipliers
    cases = {}
    for name, (m, k, base, res, outliers, prescaled) in {
        'plain': (48, 256, 1., 1., False, False),
        'outlier': (160, 512, 1., 1., True, False),
        'prescale': (32, 384, 1., 1., True, True),
        'calib_a': (64, 256, .875, 1.125, True, False),
        'calib_b': (64, 256, .75, .875, False, False),
        'ties': (16, 128, 1., 1., False, False),
        'zeros': (16, 128, 1., 1., False, False),
    }.items():
        x = torch.randn(m, k)
        if outliers:
            cols = torch.randperm(k)[:max(1, round(.005 * k))]
            x[:, cols] *= 20
        if name == 'ties':
            # exact multiples of the E2M1 midpoints after scaling: amax 6*2**j per group
            grid = torch.tensor([.25, .75, 1.25, 1.75, 2.5, 3.5, 5., 6., -.25, -.75, -2.5, -5., 0., -0., 3., 1.])
            x = grid.repeat(m, k // 16) * 4.
            x[0, 0] = 2688. / 8            # pins factor to a power of two
        if name == 'zeros':
            x = torch.zeros(m, k)
        x = x.bfloat16()
        d = (torch.rand(k) * 1.5 + .5) if prescaled else torch.ones(k)
        # The activation path rounds bf16(x*d) (_linear_kernels.py:42) and then runs the same
        # encoder as quantize_weight; feed the encoder that bf16 tensor with a unit divisor.
        y = (x.float() * d).bfloat16()
        codes, scales, factor = calibration.quantize_weight(y.float(), torch.ones(k), base=base, residual=res)
        dec = calibration.decode(codes, scales.float(), factor)
        cases[name] = dict(x=x.float().numpy(), d=d.numpy(), base=np.float32(base), res=np.float32(res),
                           codes=codes.numpy(), scales=u8(scales), factor=factor.numpy(), decoded=dec.numpy())
    np.savez_compressed(os.path.join(here, 'quantize_linear.npz'),
                        **{f'{n}/{k}': v for n, c in cases.items() for k, v in c.items()})

    # 2. per-row-factor quantizer of the attention path (dequantized base / residual)
    rows = {}
    for name, x in {
        'randn': torch.randn(40, 128) * torch.rand(40, 1) * 3,
        'prob': torch.softmax(torch.randn(24, 128) * 3, -1),
        'zero_row': torch.cat([torch.zeros(1, 128), torch.randn(7, 128)]),
    }.items():
        b, r = ref_oracle.quant_ref(x)
        rows[name] = dict(x=x.numpy(), base=b.numpy(), residual=r.numpy())
    np.savez_compressed(os.path.join(here, 'quantize_rows.npz'),
                        **{f'{n}/{k}': v for n, c in rows.items() for k, v in c.items()})

    # 3. every E4M3 rounding decision: a sweep of positive float32 values against torch's cast
    sweep = torch.cat([torch.linspace(0, 1, 4097)[1:] * 2 ** e for e in range(-10, 9)]).clamp(1 / 512, 448)
    sweep = torch.cat([sweep, torch.tensor([1 / 512, 448., 0.0029296875, 0.0048828125, 0.017578125])])
    np.savez_compressed(os.path.join(here, 'e4m3_sweep.npz'), x=sweep.numpy(),
                        byte=sweep.to(torch.float8_e4m3fn).view(torch.uint8).numpy())

    # 4. a small repaired linear with decoded fp32 emulation (term structure of the native gemm)
    m, n, k = 200, 256, 384
    a = torch.randn(m, k); a[:, torch.randperm(k)[:3]] *= 20; a = a.bfloat16()
    w = (torch.randn(n, k) * .02).bfloat16()
    mp = (m + 15) // 16 * 16
    ap_ = torch.cat([a.float(), torch.zeros(mp - m, k)])
    ac, asc, af = calibration.quantize_weight(ap_, torch.ones(k))
    wc, wsc, wf = calibration.quantize_weight(w.float(), torch.ones(k))
    one = torch.ones(())
    a0, a1 = calibration.decode(ac[0], asc[0].float(), one)[:m], calibration.decode(ac[1], asc[1].float(), one)[:m]
    w0, w1 = calibration.decode(wc[0], wsc[0].float(), one), calibration.decode(wc[1], wsc[1].float(), one)
    a_mask = torch.tensor([[True, False, True], [False, True, False]])
    w_tiles = [0, 4, 5]
    keep = torch.zeros(n // 128, k // 128, dtype=torch.bool); keep.flatten()[w_tiles] = True
    a1m = a1 * a_mask.repeat_interleave(128, 0)[:m].repeat_interleave(128, 1)
    w1m = w1 * keep.repeat_interleave(128, 0).repeat_interleave(128, 1)
    acc3 = a0.double() @ w0.double().T + a1m.double() @ w0.double().T + a0.double() @ w1m.double().T
    acc4 = acc3 + a1m.double() @ w1m.double().T
    scale = float(af * wf)
    np.savez_compressed(os.path.join(here, 'repair_linear.npz'), a=a.float().numpy(), w=w.float().numpy(),
                        ac=ac.numpy(), asc=u8(asc), af=af.numpy(), wc=wc.numpy(), wsc=u8(wsc), wf=wf.numpy(),
                        a_mask=a_mask.numpy(), w_tiles=np.array(w_tiles), y3=(acc3 * scale).float().numpy(),
                        y4=(acc4 * scale).float().numpy())
    print('golden fixtures written to', here)


if __name__ == '__main__':
    main()
