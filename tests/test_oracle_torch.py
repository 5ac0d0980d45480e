"""The threaded torch emulation (CPU baseline of the benchmark) against the numpy oracle and the fixtures
produced by the reference's own CPU encoder: packed bytes bit for bit, outputs to float32 rounding."""
import os
import numpy as np
import pytest
import torch
from oracle import nvfp4_oracle as o
from oracle import torch_emulation as te
from test_oracle_golden import load


def u8(t):
    return t.view(torch.uint8).numpy() if t.dtype == torch.float8_e4m3fn else t.numpy()


@pytest.mark.parametrize('case', ['plain', 'outlier', 'prescale', 'calib_a', 'calib_b', 'ties', 'zeros'])
def test_quantizer_matches_reference_fixtures(golden_dir, case):
    g = load(golden_dir, 'quantize_linear.npz')[case]
    codes, scales, factor = te.quantize(torch.from_numpy(g['x']), torch.from_numpy(g['d']), base=float(g['base']),
                                        residual=float(g['res']))
    assert np.float32(factor.item()) == g['factor']
    assert np.array_equal(codes.numpy(), g['codes']) and np.array_equal(u8(scales), g['scales'])
    assert np.array_equal(te.decode(codes, scales, factor).numpy(), g['decoded'])


def test_repaired_linear_and_selector_match_numpy_oracle():
    m, n, k = 300, 256, 512
    x, w = o.synthetic_activation(m, k, 5), o.synthetic_weight(n, k, 5)
    ac, asb, af = o.quantize_linear_input(x, rows_padded=304)
    wc, wsb, wf = o.quantize_weight(w)
    xt = torch.cat([torch.from_numpy(x), torch.zeros(4, k)])
    tc, ts, tf = te.quantize(xt)
    assert np.array_equal(tc.numpy(), ac) and np.array_equal(u8(ts), asb) and np.float32(tf.item()) == af
    twc, tws, twf = te.quantize(torch.from_numpy(w))
    assert np.array_equal(twc.numpy(), wc) and np.array_equal(u8(tws), wsb)
    sens = (w.astype(np.float64) ** 2).sum(0).astype(np.float32)
    scores, _ = o.residual_scores(x, None, sens)
    want_mask = o.choose_blocks(scores, 2)
    mask = te.select_blocks(torch.from_numpy(x), tf, tc[0][:m], ts[0][:m], torch.from_numpy(sens), 2)
    assert np.array_equal(mask.numpy(), want_mask)
    tiles = o.seeded_tiles(n // 128, k // 128, 0.5, 1)
    want = o.repair_linear(ac, asb, af, wc, wsb, wf, m, a_mask=want_mask, w_tiles=tiles, cross=True)
    got = te.repair_linear(tc, ts, tf, twc, tws, twf, m, a_mask=mask, w_tiles=tiles, cross=True).float().numpy()
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel < 2e-3                      # bf16 outputs: a different float32 summation order flips last bits
