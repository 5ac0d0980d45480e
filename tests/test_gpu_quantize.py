"""GPU parity of the activation quantizer: packed bytes bit-exact against the CPU oracle and
against the committed fixtures of the reference encoder. Calls go through the C ABI (ctypes)."""
import os
import numpy as np
import pytest
import torch
from oracle import nvfp4_oracle as o

pytestmark = pytest.mark.gpu


def gpu_quantize(x, d=None, **kw):
    from thunderworld_b200 import ops
    xt = torch.from_numpy(x).cuda().bfloat16()
    dt = None if d is None else torch.from_numpy(d).cuda().float()
    p = ops.quantize(xt, dt, **kw)
    torch.cuda.synchronize()
    return p


def as_np(t):
    return (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).cpu().numpy()


@pytest.mark.parametrize('case', ['plain', 'outlier', 'prescale', 'calib_a', 'calib_b', 'ties', 'zeros'])
def test_matches_reference_fixture(golden_dir, case):
    z = np.load(os.path.join(golden_dir, 'quantize_linear.npz'))
    g = {k.split('/')[1]: z[k] for k in z.files if k.startswith(case + '/')}
    p = gpu_quantize(g['x'], g['d'] if case == 'prescale' else None, repair=1, base=float(g['base']), res=float(g['res']))
    m = g['x'].shape[0]
    assert np.float32(p.factor.item()) == g['factor']
    assert np.array_equal(as_np(p.codes)[:, :m], g['codes'])
    assert np.array_equal(as_np(p.scales)[:, :m], g['scales'])


@pytest.mark.parametrize('m,k,seed', [(129, 256, 1), (416, 1024, 2), (3840, 2048, 0), (16, 128, 3), (1, 128, 4)])
def test_matches_oracle_full_residual(m, k, seed):
    x = o.synthetic_activation(m, k, seed)
    mp = (m + 15) // 16 * 16
    codes, scales, factor = o.quantize_linear_input(x, rows_padded=mp)
    p = gpu_quantize(x, repair=1)
    assert np.float32(p.factor.item()) == factor
    assert np.array_equal(as_np(p.codes), codes)
    assert np.array_equal(as_np(p.scales), scales)
    # atom-layout copies hold the same bytes, padding rows zero
    for plane in range(2):
        assert np.array_equal(as_np(p.scales_swz[plane]), o.swizzle_scales(scales[plane]))


def test_base_only_and_given_factor():
    x = o.synthetic_activation(200, 384, 5)
    codes, scales, factor = o.quantize_linear_input(x, rows_padded=208)
    p = gpu_quantize(x, repair=0)
    assert p.codes.shape[0] == 1
    assert np.array_equal(as_np(p.codes)[0], codes[0]) and np.array_equal(as_np(p.scales)[0], scales[0])
    f2 = np.float32(factor * 1.25)
    c2, s2, _ = o.quantize_linear_input(x, factor=f2, rows_padded=208)
    p2 = gpu_quantize(x, repair=1, factor=torch.tensor(float(f2), device='cuda'))
    assert np.array_equal(as_np(p2.codes), c2) and np.array_equal(as_np(p2.scales), s2)


def test_union_mask_zero_fills_unselected_residual():
    m, k = 300, 512
    x = o.synthetic_activation(m, k, 6)
    rng = np.random.default_rng(0)
    mask = rng.random((3, 4)) < 0.5
    codes, scales, _ = o.quantize_linear_input(x, rows_padded=304)
    codes, scales = o.zero_unselected_residual(codes, scales, mask)
    p = gpu_quantize(x, repair=2, mask=torch.from_numpy(mask).cuda())
    assert np.array_equal(as_np(p.codes), codes)
    assert np.array_equal(as_np(p.scales), scales)


def test_calibrated_gain_and_prescale():
    m, k = 64, 256
    x = o.synthetic_activation(m, k, 7)
    d = (np.random.default_rng(1).random(k) * 1.5 + 0.5).astype(np.float32)
    codes, scales, factor = o.quantize_linear_input(x, d, base=.875, residual=1.125, gain=1.25)
    p = gpu_quantize(x, d, repair=1, base=.875, res=1.125, gain=1.25)
    assert np.float32(p.factor.item()) == factor
    assert np.array_equal(as_np(p.codes), codes) and np.array_equal(as_np(p.scales), scales)


def test_online_selector_mask_matches_oracle_ranking():
    m, k, na = 384, 2048, 4
    x = o.synthetic_activation(m, k, 8)
    sens = (np.random.default_rng(2).random(k) + 0.5).astype(np.float32)
    scores, _ = o.residual_scores(x, None, sens)
    want = o.choose_blocks(scores, na)
    p = gpu_quantize(x, repair=3, na=na, sensitivity=torch.from_numpy(sens).cuda())
    got = p.mask.cpu().numpy()
    assert got.sum(1).tolist() == [na] * 3
    # float32 summation order may flip only blocks whose scores are within rounding of the cut
    for i in range(3):
        diff = np.flatnonzero(got[i] != want[i])
        if diff.size:
            cut = np.sort(scores[i])[-na]
            assert np.all(np.abs(scores[i][diff] - cut) <= 1e-4 * cut)
    # residual bytes are valid under the mask (the reference compares only there)
    codes, scales, _ = o.quantize_linear_input(x, rows_padded=m)
    assert np.array_equal(as_np(p.codes), codes)


@pytest.mark.parametrize('energy', [0.5, 0.75])
def test_online_selector_energy_prefix_stop(energy):
    """The energy-prefix stop: a K128 block is kept only while the blocks ranked before it hold less than `energy`
    of the row block's total score (thunderworld_fp4/_sparse_pack.py:54-60), so fewer than `na` blocks may be kept."""
    m, k, na = 300, 1024, 4
    x = o.synthetic_activation(m, k, 12)
    x[:, :128] *= 6                                   # one dominant block: the prefix stops early
    x = o.bf16_round(x)
    sens = (np.random.default_rng(4).random(k) + 0.5).astype(np.float32)
    scores, _ = o.residual_scores(x, None, sens)
    want = o.choose_blocks(scores, na, energy)
    p = gpu_quantize(x, repair=3, na=na, sensitivity=torch.from_numpy(sens).cuda(), energy=energy)
    got = p.mask.cpu().numpy()
    assert (got.sum(1) <= na).all() and (want.sum(1) < na).any()
    assert np.array_equal(got, want)


def test_bounded_wait_runs_out_and_is_reported():
    """A wait that nothing will ever satisfy ends after its cycle limit with a status code, and the GPU goes on
    working: no trap, no hang, nothing left in flight."""
    from thunderworld_b200 import ops
    ops.reset_device_status()
    assert ops.device_status() == 0
    status = ops.selftest_bounded_wait(limit_cycles=500_000)
    assert status == 8                                # TW_ERR_TIMEOUT
    from thunderworld_b200 import _lib
    assert b'wait ran out' in _lib.load().tw_status(status)
    ops.reset_device_status()
    assert ops.device_status() == 0
    x = o.synthetic_activation(64, 256, 1)
    codes, _, _ = o.quantize_linear_input(x, rows_padded=64)
    assert np.array_equal(as_np(gpu_quantize(x, repair=1).codes), codes)     # the context is intact


def test_rejects_bad_arguments():
    from thunderworld_b200 import ops
    with pytest.raises(ValueError):
        ops.quantize(torch.zeros(4, 100, device='cuda', dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        ops.quantize(torch.zeros(0, 128, device='cuda', dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        ops.quantize(torch.zeros(4, 128, device='cuda', dtype=torch.float16))
