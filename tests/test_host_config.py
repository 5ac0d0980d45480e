"""CPU tests of the host-side mirror of the reference's configuration, plan and ledger modules.
The facts asserted are the ones the reference's own CPU tests pin
(packages/fp4-repair/tests/test_config.py, test_compute_budget.py)."""
import itertools
import json
import pytest
import torch
from thunderworld_b200.config import (PRESETS, InferenceConfig, LinearRepairConfig, RepairConfig, RepairPolicy,
                                      RepairRule, preset)
from thunderworld_b200.head_finding import config_from_head_scores, make_repair_mask, policy_from_head_atlas
from thunderworld_b200.cosmos.budget import RepairPlan, attention_cost, compile_request, linear_cost
from thunderworld_b200.cosmos.settings import TIERS, LinearSpec, RunConfig, phase
from thunderworld_b200.cosmos.assets import compact, expand
from thunderworld_b200.cosmos import trees


@pytest.mark.parametrize('name', PRESETS)
def test_presets_round_trip(name):
    config = preset(name)
    assert RepairConfig.from_dict(json.loads(json.dumps(config.to_dict()))) == config


@pytest.mark.parametrize('kwargs', [{'coverage': float('nan')}, {'coverage': True}, {'coverage': 1.1}, {'query_tile': 48},
                                    {'terms': 1}, {'head_budgets': [(0, .2), (0, .5)]}, {'head_budgets': [(-1, .2)]},
                                    {'splits': 3}, {'lazy_p': 1}, {'head_quotas': ()}, {'pv_terms': 5}])
def test_invalid_repair_config(kwargs):
    with pytest.raises(ValueError):
        RepairConfig(**kwargs)


def test_independent_sections_and_cost():
    c = InferenceConfig.from_dict({'ffn': {'coverage': 1}, 'attention': {'coverage': .5, 'head_budgets': [[1, 0], [2, 1]]},
                                   'attention_projection': {'coverage': .25}})
    assert c.ffn.output_counts(256, 512) == (4, 4)
    assert c.attention.head_counts(3, 512) == (2, 0, 4)
    assert c.attention_projection.output_counts(256, 512) == (1, 1)
    assert InferenceConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c
    assert c.attention.cost(3, 512)['matrix_product_multiplier'] == 2
    with pytest.raises(ValueError):
        InferenceConfig.from_dict({'other': {}})


def test_head_scores_policy_and_atlas():
    high = config_from_head_scores([.2, .9, .9, .1], protected_count=1, coverage=.25, protected_coverage=1)
    assert high.head_counts(4, 512) == (1, 4, 1, 1)
    p = RepairPolicy(rules=(RepairRule(high, layers=(2,), steps=(3, 5)),))
    assert p.resolve(layer=2, step=3) == high
    assert p.resolve(layer=2, step=5) == p.default
    with pytest.raises(ValueError):
        p.resolve(layer=2)
    with pytest.raises(ValueError):
        RepairConfig(head_budgets=((9, .5),)).head_counts(2, 128)
    with pytest.raises(ValueError):
        LinearRepairConfig().output_counts(129, 256)
    atlas = {'layers': [{'layer': 0, 'compiled_q_fp8_heads': [1, 3]}, {'layer': 2, 'compiled_q_fp8_heads': [0]}]}
    policy = policy_from_head_atlas(atlas, coverage=.25, protected_coverage=1)
    assert policy.resolve(layer=0).head_counts(4, 512) == (1, 4, 1, 4)
    assert policy.resolve(layer=2).head_counts(4, 512) == (4, 1, 1, 1)
    assert policy.resolve(layer=1).head_counts(4, 512) == (1, 1, 1, 1)
    with pytest.raises(ValueError):
        policy_from_head_atlas({'layers': atlas['layers'] * 2})
    mask = make_repair_mask(300, 500, 2, {1: [(2, 3), (0, 0)]}, device='cpu')
    assert mask.shape == (2, 3, 4) and mask.sum() == 2 and mask[1, 2, 3]
    with pytest.raises(ValueError):
        make_repair_mask(300, 500, 2, {1: [(3, 0)]}, device='cpu')


@pytest.mark.parametrize('m', [129, 416])
@pytest.mark.parametrize('bm', [32, 64, 128])
def test_linear_ledger_exact_and_cross_bound(m, bm):
    weights = (0, 1, 3, 5, 6)
    bound = linear_cost(m, 256, 512, bm=bm, a_blocks=2, w_blocks=weights, cross=True)
    for chosen in itertools.combinations(range(4), 2):
        exact = linear_cost(m, 256, 512, bm=bm, a_blocks=2, w_blocks=weights, cross=True,
                            a_support=[chosen] * ((m + 127) // 128))
        assert exact['total_mma'] <= bound['total_mma']
    full = linear_cost(m, 256, 512, bm=bm, a_blocks=4, w_blocks=range(8), cross=True)
    assert full['total_mma'] == 4 * full['base_mma']
    base = linear_cost(m, 256, 512, bm=bm)
    assert base['total_mma'] == base['base_mma']
    assert base['padded_base_mma'] == 2 * ((m + bm - 1) // bm * bm - m) * 256 * 512
    with pytest.raises(ValueError):
        linear_cost(m, 200, 512)
    with pytest.raises(ValueError):
        linear_cost(m, 256, 512, w_blocks=(1, 1))


def test_attention_ledger():
    base = attention_cost(129, 416, 4, 2, qk_counts=[0] * 4, pv_counts=[0] * 4)
    full = attention_cost(129, 416, 4, 2, qk_counts=[4] * 4, pv_counts=[4] * 4, qk_terms=4, pv_terms=4)
    assert full['total_mma'] == 4 * base['total_mma']
    partial = attention_cost(129, 416, 4, 2, qk_counts=[1, 0, 2, 4], pv_counts=[0, 1, 0, 1])
    assert partial['mma_by_dtype']['bf16']['selector'] == 4 * 2 * 2 * 16 * 32 * 128
    assert partial['gqa_support_union_upper'][0]['k_blocks_upper'] == 2
    mask = [[[False] * 4 for _ in range(2)] for _ in range(4)]
    exact = attention_cost(129, 416, 4, 2, explicit_masks={'qk': mask, 'pv': mask})
    assert exact['total_mma'] == base['total_mma']


def test_request_budget_is_global_and_fails_closed():
    rows = []
    for branch in range(2):
        for ph in range(4):
            rows.append({**linear_cost(129, 128, 128, a_blocks=1 if ph == 0 else 0), 'name': 'linear', 'branch': branch, 'phase': ph})
            rows.append({**attention_cost(129, 128, 1, 1), 'name': '0', 'branch': branch, 'phase': ph})
    result = compile_request(rows, 1.125, expected_modules=['linear'], expected_layers=['0'])
    assert result['feasible'] and result['rows'][0]['calls'] == 7
    with pytest.raises(ValueError, match='exceeded'):
        compile_request(rows, 1.)
    with pytest.raises(ValueError):
        compile_request(rows[:-1], 1.5)
    with pytest.raises(ValueError):
        compile_request(rows + rows[:1], 1.5)


def test_specs_tiers_and_run_config_round_trip():
    spec = LinearSpec(0, 0, True, activation_blocks=1, weight_support=(0, 2))
    assert spec.counts(256, 256) == (1, 2)
    with pytest.raises(ValueError):
        spec.counts(128, 128)
    with pytest.raises(ValueError):
        LinearSpec(0, 0, True)
    assert TIERS['four'].cross and TIERS['base'].counts(256, 256) == (0, 0)
    cfg = RepairConfig(head_quotas=(0, 1), pv_head_quotas=(2, 0), pv_terms=4)
    assert cfg.head_counts(2, 129) == (0, 1) and cfg.pv_counts(2, 129) == (2, 0)
    with pytest.raises(ValueError):
        cfg.pv_counts(2, 128)
    run = RunConfig(compute_budget=1.25, ffn=spec, tensor_parallel=2)
    assert RunConfig.from_dict(json.loads(json.dumps(run.to_dict()))) == run
    assert run.fingerprint != RunConfig().fingerprint
    with pytest.raises(ValueError):
        RunConfig(compute_budget=1.3)
    with pytest.raises(ValueError):
        RunConfig(budget_plan='plan.json')
    assert [phase(s, 35) for s in (0, 6, 7, 17, 18, 27, 28, 34)] == [0, 0, 1, 1, 2, 2, 3, 3]


def plan_value():
    linears = {f'{b}|{p}|blk.q': {'a_blocks': 1, 'w_blocks': [0, 3], 'cross': False} for b in range(2) for p in range(4)}
    attention = {f'{b}|{p}|0': {'qk_counts': [1, 0], 'pv_counts': [0, 1], 'qk_terms': 3, 'pv_terms': 2} for b in range(2) for p in range(4)}
    attention['1|3|0'] = {'full_attention': True}
    attention['1|2|0'] = {'qk_fractions': [.5, 0.], 'pv_fractions': [0., .25]}
    return dict(schema_version=1, budget=1.5, steps=35, phases=[0, 7, 18, 28, 35], task='i2v', linears=linears, attention=attention)


def test_plan_lookup_fails_closed(tmp_path):
    path = tmp_path / 'plan.json'
    path.write_text(json.dumps(plan_value()))
    plan = RepairPlan.load(path)
    spec = plan.linear('i2v', 0, 1, 'blk.q')
    assert spec.activation_blocks == 1 and spec.weight_support == (0, 3) and not spec.cross
    with pytest.raises(KeyError):
        plan.linear('i2v', 0, 1, 'missing')
    with pytest.raises(ValueError):
        plan.linear('t2v', 0, 1, 'blk.q')
    cfg = plan.attention_config('i2v', 0, 0, 0, RepairConfig())
    assert cfg.head_quotas == (1, 0) and cfg.pv_head_quotas == (0, 1) and cfg.pv_terms == 2 and cfg.sparse_pack
    assert plan.attention_config('i2v', 1, 3, 0, RepairConfig()).coverage == 1.
    frac = plan.attention_config('i2v', 1, 2, 0, RepairConfig())
    assert frac.head_budgets == ((0, .5), (1, 0.)) and frac.pv_head_budgets == ((0, 0.), (1, .25))
    assert len(plan.fingerprint) == 64
    for broken in ({'steps': 30}, {'budget': 3.}, {'task': ''}, {'schema_version': 2}):
        with pytest.raises(ValueError):
            RepairPlan({**plan_value(), **broken})


def test_w1_support_compact_expand_round_trip():
    torch.manual_seed(0)
    nb, kb = 2, 3
    asset = dict(codes=torch.randint(0, 255, (2, nb * 128, kb * 64), dtype=torch.uint8),
                 scales=torch.randint(0, 120, (2, nb * 128, kb * 8), dtype=torch.uint8).view(torch.float8_e4m3fn),
                 factor=torch.tensor(.01), prescale=torch.ones(kb * 128), score=torch.rand(nb, kb), bias=None)
    keep = [0, 4, 5]
    small = compact(asset, keep)
    assert small['storage_schema'] == 2 and small['codes_residual'].shape == (3, 128, 64)
    back = expand(small, keep)
    tiles = torch.zeros(nb * kb, dtype=torch.bool); tiles[keep] = True
    grid = tiles.reshape(nb, kb).repeat_interleave(128, 0)
    assert torch.equal(back['codes'][0], asset['codes'][0])
    assert torch.equal(back['codes'][1], asset['codes'][1] * grid.repeat_interleave(64, 1))
    assert torch.equal(back['scales'][1].view(torch.uint8), asset['scales'][1].view(torch.uint8) * grid.repeat_interleave(8, 1))
    with pytest.raises(ValueError):
        expand(small, [0, 1])
    by_score = compact(asset, .5)
    assert by_score['storage_schema'] == 1 and len(by_score['residual_indices']) == 3
    assert set(by_score['residual_indices'].tolist()) == set(torch.argsort(asset['score'].flatten(), descending=True)[:3].tolist())
    with pytest.raises(ValueError):
        expand(by_score, .75)
    with pytest.raises(ValueError):
        compact({**asset, 'mandatory_w_blocks': (1,)}, [0, 4])


def test_tree_signature_clone_copy():
    a = {'x': torch.zeros(2, 3), 'meta': (1, 'cond', None), 'list': [torch.ones(4)]}
    b = trees.clone_tree(a)
    assert trees.signature(a) == trees.signature(b) and b['x'] is not a['x']
    b['x'].fill_(7); b['list'][0].fill_(5)
    trees.copy_tree(a, b)
    assert float(a['x'].sum()) == 42 and float(a['list'][0].sum()) == 20
    assert trees.signature({'x': torch.zeros(2, 3)}) != trees.signature({'x': torch.zeros(3, 2)})
    with pytest.raises(TypeError):
        trees.signature(object())


def test_cfg_parallel_rank_compiles_its_own_branch():
    """A CFG-parallel rank runs branch 1 of the plan as its only branch: its rows carry the plan's branch
    index, the ledger it proves counts one branch."""
    from thunderworld_b200.cosmos.engine import StepEngine
    from thunderworld_b200.cosmos.settings import RunConfig
    engine = StepEngine(RunConfig(compute_budget=2.), branches=1)
    engine._branch_offset = 1
    for ph in range(4):
        row = linear_cost(256, 256, 512, a_blocks=2, w_blocks=(0, 3))
        engine.rows[('linear', 'proj', 1, ph)] = {**row, 'name': 'proj', 'branch': 1, 'phase': ph}
        att = attention_cost(256, 256, 2, 2, qk_counts=[1, 1], pv_counts=[1, 1])
        engine.rows[('attention', '0', 1, ph)] = {**att, 'name': '0', 'branch': 1, 'phase': ph}
    ledger = engine.compile_budget()
    assert ledger['feasible'] and ledger['total_mma'] <= 2 * ledger['base_mma']


def test_bench_topology_splits_cfg_branches_first():
    """The benchmark's layout per GPU count: one GPU, then one CFG branch per GPU, then tensor parallelism inside
    each branch; `--cfg-parallel 1` forces tensor parallelism alone."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'bench.py')
    spec = importlib.util.spec_from_file_location('bench_module_for_test', path)
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert [bench.step_topology(n, 0) for n in (1, 2, 4, 8)] == [(1, 1), (1, 2), (2, 2), (4, 2)]
    assert [bench.step_topology(n, 1) for n in (2, 4)] == [(2, 1), (4, 1)]
