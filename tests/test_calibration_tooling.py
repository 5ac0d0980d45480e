"""Calibration-side tooling (CPU): prescale proposals, outlier proposal and the encoder that honours it, budget
allocator, asset export / load with manifest. The facts checked are the ones the reference's own CPU tests pin
(packages/fp4-repair/tests/test_compute_budget.py:72-116); the encoder is also checked bit for bit against the
reference-run fixtures and the numpy oracle."""
import numpy as np
import pytest
import torch
from oracle import nvfp4_oracle as o
from test_oracle_golden import load
from thunderworld_b200.cosmos import calibration as cal
from thunderworld_b200.cosmos.allocation import allocate
from thunderworld_b200.cosmos.assets import compact, expand, export_assets, load_assets


def test_prescale_direction_and_mandatory_outliers():
    torch.manual_seed(4)
    w = torch.randn(128, 256).bfloat16()
    rms = torch.linspace(.1, 5, 256)
    names = []
    for name, d in cal.prescale_candidates(rms, w):
        names.append(name)
        assert d.min() >= 1 / 16 and d.max() <= 16
        x = torch.randn(3, 256)
        torch.testing.assert_close((x * d) @ (w.float() / d).T, x @ w.float().T, atol=1e-4, rtol=1e-4)
    assert names[0] == 'identity' and names[-1] == 'legacy_orientation' and len(names) == 7
    w[0, 0] = 100
    remove, mandatory = cal.outlier_mask(w, torch.ones(256), rms, [0], 2.)
    assert remove.reshape(128, 16, 16).sum(-1).max() <= 1
    assert not remove[:, 128:].any() and mandatory == (0,)
    c, s, g = cal.quantize_weight(w, torch.ones(256), remove=remove)
    decoded = cal.decode(c, s, g)
    assert decoded[0, 0, 0] == 0 and decoded[1, 0, 0] > 90
    asset = dict(codes=c, scales=s, factor=g, score=torch.ones(1, 2), mandatory_w_blocks=mandatory)
    with pytest.raises(ValueError):
        compact(asset, [])
    restored = expand(compact(asset, [0]), [0])
    assert torch.equal(restored['codes'][0], c[0])
    with pytest.raises(ValueError):
        expand(compact(asset, [0]), [1])
    with pytest.raises(ValueError):
        cal.outlier_mask(w, torch.ones(256), rms, [0], 2.5)
    assert cal.outlier_mask(w, torch.ones(256), rms, [0], None)[1] == ()
    assert cal.panel_objective([1., 3.]) == 2.75


@pytest.mark.parametrize('case', ['plain', 'outlier', 'calib_a', 'ties', 'zeros'])
def test_cpu_encoder_matches_reference_fixtures(golden_dir, case):
    g = load(golden_dir, 'quantize_linear.npz')[case]
    y = (torch.from_numpy(g['x']) * torch.from_numpy(g['d'])).bfloat16().float()
    codes, scales, factor = cal.quantize_weight(y, torch.ones(y.shape[1]), base=float(g['base']), residual=float(g['res']))
    assert np.float32(factor.item()) == g['factor']
    assert np.array_equal(codes.numpy(), g['codes']) and np.array_equal(scales.view(torch.uint8).numpy(), g['scales'])
    assert np.array_equal(cal.decode(codes, scales, factor).numpy(), g['decoded'])
    oc, osb, of = o.quantize_weight(g['x'] * g['d'], None, base=float(g['base']), residual=float(g['res']))
    assert np.array_equal(codes.numpy(), oc) and np.array_equal(scales.view(torch.uint8).numpy(), osb)


def test_allocator_grow_prune_hard_cap_and_combination_loss():
    groups = {f'g{i}': [dict(id=0, base_mma=100, mma=100, loss=10.), dict(id=1, base_mma=100, mma=110, loss=8.),
                        dict(id=2, base_mma=100, mma=125, loss=9.),            # dominated combination
                        dict(id=3, base_mma=100, mma=150, loss=3.)] for i in range(4)}
    for direction in ('grow', 'prune'):
        for budget in (1., 1.125, 1.25, 1.5):
            result = allocate(groups, budget, direction=direction)
            assert result['total_mma'] <= result['base_mma'] * budget
            assert all(c['id'] != 2 for c in result['assignments'].values())
    assert allocate(groups, 1.5)['total_mma'] == 600                             # everything at id 3 fits exactly
    with pytest.raises(ValueError):
        allocate(groups, 1.5, direction='sideways')
    with pytest.raises(ValueError):
        allocate({'g': []}, 1.5)


def test_restricted_allocation_filters_before_pareto_pruning():
    group = [dict(id=0, base_mma=100, mma=100, loss=10., a_blocks=0, w_blocks=[]),
             dict(id=1, base_mma=100, mma=110, loss=8., a_blocks=1, w_blocks=[]),
             dict(id=2, base_mma=100, mma=105, loss=7., a_blocks=0, w_blocks=[0])]
    assert allocate({'op': group}, 1.125, preference='a')['assignments']['op']['id'] == 1
    assert allocate({'op': group}, 1.125, preference='w')['assignments']['op']['id'] == 2


def test_asset_export_manifest_and_hash_checks(tmp_path):
    torch.manual_seed(1)
    w = torch.randn(256, 256).bfloat16()
    c, s, g = cal.quantize_weight(w, torch.ones(256))
    asset = dict(codes=c, scales=s, factor=g, prescale=torch.ones(256), score=torch.rand(2, 2), bias=None)
    folder = tmp_path / 'assets'
    manifest = export_assets(folder, {'blocks.0.qkv': asset}, model_identity='toy', targets=['blocks.0.qkv'],
                             support={'blocks.0.qkv': [0, 3]})
    assert manifest['complete'] and list(manifest['modules']) == ['blocks.0.qkv']
    back = load_assets(folder, model_identity='toy', required={'blocks.0.qkv': [3]})
    assert torch.equal(back['blocks.0.qkv']['codes'][0], c[0])
    with pytest.raises(ValueError):
        load_assets(folder, model_identity='other')
    with pytest.raises(ValueError):
        load_assets(folder, model_identity='toy', required={'blocks.0.qkv': [1]})
    path = folder / manifest['modules']['blocks.0.qkv']['file']
    path.write_bytes(path.read_bytes() + b'x')
    with pytest.raises(ValueError):
        load_assets(folder, model_identity='toy')
    with pytest.raises(FileExistsError):
        export_assets(folder, {}, model_identity='toy')
