"""The numpy oracle against fixtures produced by the reference's own CPU encoder."""
import os
import numpy as np
import pytest
from oracle import nvfp4_oracle as o


def load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    out = {}
    for key in z.files:
        case, field = key.split('/') if '/' in key else (None, key)
        if case is None:
            out[field] = z[key]
        else:
            out.setdefault(case, {})[field] = z[key]
    return out


def test_e4m3_rounding_matches_torch_cast(golden_dir):
    g = load(golden_dir, 'e4m3_sweep.npz')
    value, byte = o.e4m3_round(g['x'])
    assert np.array_equal(byte, g['byte'])
    assert np.array_equal(o.e4m3_decode(byte), value)


def test_e4m3_all_bytes_roundtrip():
    bytes_ = np.arange(0, 127, dtype=np.uint8)        # 0x7f is NaN
    v = o.e4m3_decode(bytes_)
    assert v[-1] == 448 and v[1] == 2.0 ** -9
    _, again = o.e4m3_round(v)
    assert np.array_equal(again, bytes_)


@pytest.mark.parametrize('case', ['plain', 'outlier', 'prescale', 'calib_a', 'calib_b', 'ties', 'zeros'])
def test_linear_quantizer_bit_exact(golden_dir, case):
    g = load(golden_dir, 'quantize_linear.npz')[case]
    codes, scales, factor = o.quantize_linear_input(g['x'], g['d'], base=float(g['base']), residual=float(g['res']))
    assert np.float32(factor) == g['factor']
    assert np.array_equal(codes, g['codes'])
    assert np.array_equal(scales, g['scales'])
    assert np.array_equal(o.decode(codes, scales, factor), g['decoded'])


@pytest.mark.parametrize('case', ['randn', 'prob', 'zero_row'])
def test_row_quantizer_matches_reference_oracle(golden_dir, case):
    g = load(golden_dir, 'quantize_rows.npz')[case]
    base, residual = o.quant_ref(g['x'])
    assert np.array_equal(base, g['base'])
    assert np.array_equal(residual, g['residual'])


def test_repair_linear_terms(golden_dir):
    g = load(golden_dir, 'repair_linear.npz')
    m = g['a'].shape[0]
    mp = (m + 15) // 16 * 16
    ac, asc, af = o.quantize_linear_input(g['a'], rows_padded=mp)
    wc, wsc, wf = o.quantize_weight(g['w'])
    for mine, ref in ((ac, g['ac']), (asc, g['asc']), (wc, g['wc']), (wsc, g['wsc'])):
        assert np.array_equal(mine, ref)
    assert af == g['af'] and wf == g['wf']
    tiles = [int(t) for t in g['w_tiles']]
    y3 = o.repair_linear(ac, asc, af, wc, wsc, wf, m, a_mask=g['a_mask'], w_tiles=tiles,
                         accumulate=np.float64, round_bf16=False)
    y4 = o.repair_linear(ac, asc, af, wc, wsc, wf, m, a_mask=g['a_mask'], w_tiles=tiles, cross=True,
                         accumulate=np.float64, round_bf16=False)
    assert np.allclose(y3, g['y3'], rtol=1e-6, atol=1e-7)
    assert np.allclose(y4, g['y4'], rtol=1e-6, atol=1e-7)
    # fp32 accumulation stays within the documented tolerance of the fp64 emulation
    y3f = o.repair_linear(ac, asc, af, wc, wsc, wf, m, a_mask=g['a_mask'], w_tiles=tiles, round_bf16=False)
    rel = np.linalg.norm(y3f - g['y3']) / np.linalg.norm(g['y3'])
    assert rel < 1e-5


def test_scale_swizzle_is_a_permutation_with_documented_offsets():
    rng = np.random.default_rng(0)
    s = rng.integers(1, 120, size=(200, 16), dtype=np.uint8)
    z = o.swizzle_scales(s)
    assert z.shape == (256, 16)
    flat = z.reshape(-1)
    # cutlass/packing.py:24-25 byte map, spelled out independently
    for row, col in ((0, 0), (1, 0), (31, 3), (32, 0), (127, 15), (128, 0), (199, 7)):
        off = (row // 128) * 128 * 16 + (col // 4) * 512 + (row % 32) * 16 + ((row % 128) // 32) * 4 + col % 4
        assert flat[off] == s[row, col]
    assert np.sort(flat[flat > 0]).tolist() == np.sort(s.reshape(-1)).tolist()


def test_choose_blocks_ties_and_energy():
    scores = np.array([[3., 1., 3., 0.], [0., 0., 0., 0.]])
    mask = o.choose_blocks(scores, 2)
    assert mask.tolist() == [[True, False, True, False], [True, True, False, False]]
    mask = o.choose_blocks(np.array([[10., 1., 1., 1.]]), 3, energy=0.7)
    assert mask.tolist() == [[True, False, False, False]]
    # all-zero residual needs no repair under an energy stop (before < 0 is never true)
    assert not o.choose_blocks(np.zeros((1, 4)), 2, energy=0.5).any()


def test_issued_flops_matches_ledger_formula():
    m, n, k = 3840, 2048, 2048
    tiles = o.seeded_tiles(16, 16, 0.25)
    assert len(tiles) == 64
    f = o.issued_flops(m, n, k, a_full=True, w_tiles=tiles)
    assert f == 2 * m * n * k * 2 + 2 * m * 128 * 128 * 64
    assert abs(f / 1e9 - 72.5) < 0.1


def _bf16(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize('case', ['base', 'repair3', 'repair4_pv2'])
def test_attention_flow_matches_reference_run(golden_dir, case):
    """oracle.attention_reference against outputs of the reference's tests/oracle.py:reference, run on CPU with
    its own quant_ref decode (splits 1 and 2, 2/3/4 terms, separate PV flags, GQA, ragged M and N).
    Both are float32 flows over identical quantized operands; they differ in the summation order of the
    float32 matmuls and of the split merge, and a P value on a rounding boundary can take the other code."""
    g = load(golden_dir, 'attention_flow.npz')[case]
    got = o.attention_reference(_bf16(g['q_bf16']), _bf16(g['k_bf16']), _bf16(g['v_bf16']), g['flags'],
                                repair=bool(g['repair']), terms=int(g['terms']), pvflags=g['pvflags'],
                                pvterms=int(g['pvterms']))
    want = g['out']
    assert got.shape == want.shape
    rel = np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want)
    assert rel < 2e-4, rel


@pytest.mark.parametrize('case', ['m129', 'm416', 'wide'])
def test_selector_matches_reference_loop(golden_dir, case):
    """oracle.residual_scores + choose_blocks against the stable-argsort selector loop of the reference's own
    test (tests/test_adaptive_repair.py:52-63) evaluated on the reference's CPU encoder, with and without the
    energy-prefix stop."""
    g = load(golden_dir, 'selector.npz')[case]
    x = _bf16(g['x_bf16'])
    scores, _ = o.residual_scores(x, g['d'], g['sens'], base=0.875)
    assert np.allclose(scores, g['scores'], rtol=2e-5, atol=0)
    for energy, key in ((0.5, 'mask_050'), (0.75, 'mask_075'), (1.0, 'mask_100')):
        assert np.array_equal(o.choose_blocks(scores, int(g['count']), energy), g[key]), energy
