"""Generate the golden fixtures in this folder from the reference's own CPU code.

Run once, where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/ThunderWorld

It imports `thunderworld_fp4.cosmos.calibration` (quantize_weight, decode) and
`packages/fp4-repair/tests/oracle.py` (quant_ref, reference) from that checkout, feeds them
seeded inputs and stores inputs and outputs as small .npz files. The streaming-attention flow
(`reference`) normally decodes the GPU packer's bytes; here its `decoded_inputs` is replaced by the
same decode built from the reference's own CPU `quant_ref`, so the whole flow runs without a GPU. The
current-residual selector fixture restates the torch loop of the reference's own selector test
(tests/test_adaptive_repair.py:52-63) on the CPU encoder. The tests read
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

    # 5. streaming attention flow: tests/oracle.py:reference on CPU, fed with quant_ref-decoded operands
    def cpu_decoded_inputs(q, k, v, repair):
        m, n, h, hk = q.shape[1], k.shape[1], q.shape[2], k.shape[2]
        mp, npad = (m + 15) // 16 * 16, (n + 127) // 128 * 128
        nt = npad // 128

        def planes(rows2d):
            b, r = ref_oracle.quant_ref(rows2d)
            return torch.stack([b, r if repair else torch.zeros_like(r)])

        def pad(x, rows):
            return torch.cat([x, torch.zeros(rows - x.shape[0], 128)])
        qp = torch.stack([planes(pad(q[0, :, i].float(), mp)) for i in range(h)], 1)
        kp = torch.stack([planes(pad(k[0, :, i].float(), npad)) for i in range(hk)], 1)
        vs = []
        for i in range(hk):
            rows = pad(v[0, :, i].float(), npad).reshape(nt, 128, 128).transpose(1, 2).reshape(npad, 128)
            pl = planes(rows)                                   # rows = (tile, channel), columns = tokens
            vs.append(pl.reshape(2, nt, 128, 128).transpose(-1, -2).reshape(2, npad, 128))
        return qp, kp, torch.stack(vs, 1)
    ref_oracle.decoded_inputs = cpu_decoded_inputs
    att = {}
    for name, (m, n, h, hk, repair, terms, pvterms, splits) in {
        'base': (200, 300, 2, 1, False, 3, 3, 1),
        'repair3': (200, 300, 4, 2, True, 3, 3, 2),
        'repair4_pv2': (130, 520, 2, 2, True, 4, 2, 1),
    }.items():
        gq = torch.Generator().manual_seed(len(name))
        mk = lambda s_, h_: (torch.randn(1, s_, h_, 128, generator=gq) * (torch.rand(h_, generator=gq) * 1.5 + .5)[None, None, :, None]).bfloat16()
        q, k, v = mk(m, h), mk(n, hk), mk(n, hk)
        mb, nt = (m + 127) // 128, (n + 127) // 128
        flags = (torch.rand(h, mb, nt, generator=gq) < .5).int() * 2 + 1
        pvflags = (torch.rand(h, mb, nt, generator=gq) < .5).int() * 2 + 1
        out = ref_oracle.reference(q, k, v, flags, repair, terms=terms, splits=splits, pvflags=pvflags, pvterms=pvterms)
        bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)            # bf16 bit patterns
        att[name] = dict(q_bf16=bits(q[0]), k_bf16=bits(k[0]), v_bf16=bits(v[0]), flags=flags.numpy(),
                         pvflags=pvflags.numpy(), repair=np.int32(repair), terms=np.int32(terms), pvterms=np.int32(pvterms),
                         out=out[0].numpy())
    np.savez_compressed(os.path.join(here, 'attention_flow.npz'),
                        **{f'{n}/{k}': v for n, c in att.items() for k, v in c.items()})

    # 6. current-residual selector (sparse packer): residual energy x sensitivity per (M128, K128), stable
    #    descending rank, top `count`, optional energy-prefix stop
    sel = {}
    for name, (m, k, count) in {'m129': (129, 512, 2), 'm416': (416, 512, 2), 'wide': (300, 2048, 8)}.items():
        gs = torch.Generator().manual_seed(49 + m)
        x = torch.randn(m, k, generator=gs).bfloat16()
        x[:, :128] *= 8
        d = torch.linspace(.5, 2, k)
        sens = torch.linspace(.1, 4, k)
        y = (x.float() * d).bfloat16().float()
        codes, scales, factor = calibration.quantize_weight(y, torch.ones(k), base=.875, residual=1.125)
        residual = y - calibration.decode(codes[0], scales[0].float(), factor)
        mbn, kbn = (m + 127) // 128, k // 128
        masks, scores = {}, torch.zeros(mbn, kbn)
        for energy in (.5, .75, 1.):
            expected = torch.zeros(mbn, kbn, dtype=torch.bool)
            for mb in range(mbn):
                score = (residual[mb * 128:(mb + 1) * 128].square() * sens).reshape(-1, kbn, 128).sum((0, 2))
                scores[mb] = score
                order = score.argsort(descending=True, stable=True)
                running = 0.
                for index in order[:count]:
                    if energy == 1 or running < float(score.sum()) * energy:
                        expected[mb, index] = True
                    running += float(score[index])
            masks[energy] = expected.numpy()
        sel[name] = dict(x_bf16=x.view(torch.int16).numpy().view(np.uint16), d=d.numpy(), sens=sens.numpy(), count=np.int32(count), scores=scores.numpy(),
                         mask_050=masks[.5], mask_075=masks[.75], mask_100=masks[1.])
    np.savez_compressed(os.path.join(here, 'selector.npz'),
                        **{f'{n}/{k}': v for n, c in sel.items() for k, v in c.items()})
    print('golden fixtures written to', here)


if __name__ == '__main__':
    main()
