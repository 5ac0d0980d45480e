"""DiT step on the repaired operators under the step engine: CUDA-Graph replay equals eager execution
bit for bit over a multi-phase plan, the ledger proves the budget, unwarmed shapes raise
(reference integration test: packages/fp4-repair/tests/test_compute_cuda.py:103-157)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def tiny_plan(cfg, budget=2.0):
    from thunderworld_b200.cosmos.budget import RepairPlan
    h, f = cfg.hidden // 128, cfg.ffn // 128
    lattice = {'qkv': (3 * h, h), 'out': (h, h), 'up': (f, h), 'down': (h, f)}
    rng = np.random.default_rng(0)
    linears, attention = {}, {}
    for b in range(2):
        for p in range(4):
            for i in range(cfg.blocks):
                for part, (nb, kb) in lattice.items():
                    tiles = sorted(int(t) for t in rng.permutation(nb * kb)[:(nb * kb) // 4]) if p % 2 == 0 else []
                    linears[f'{b}|{p}|blocks.{i}.{part}'] = {'a_blocks': [0, 1, kb // 2, kb][p] if kb > 1 else p % 2,
                                                              'w_blocks': tiles, 'cross': False}
                attention[f'{b}|{p}|{i}'] = {'qk_counts': [p % 2] * cfg.heads, 'pv_counts': [1 - p % 2] * cfg.heads}
    return RepairPlan(dict(schema_version=1, budget=budget, steps=35, phases=[0, 7, 18, 28, 35], task='t2v',
                           linears=linears, attention=attention))


def build(execution, plan_budget=2.0):
    from thunderworld_b200.cosmos.dit import DiTConfig, DiTModel
    from thunderworld_b200.cosmos.engine import StepEngine
    from thunderworld_b200.cosmos.settings import RunConfig
    cfg = DiTConfig(hidden=256, heads=2, ffn=512, blocks=2, seed=1)
    plan = tiny_plan(cfg, plan_budget)
    engine = StepEngine(RunConfig(compute_budget=plan_budget, execution=execution), plan=plan)
    model = DiTModel(cfg, engine)
    return cfg, engine, model


def make_inputs(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(2, 200, cfg.hidden, generator=g).bfloat16().cuda()
    mod = (torch.randn(2, cfg.blocks, 6, cfg.hidden, generator=g) * 0.1).bfloat16().cuda()
    return x, mod


def test_graph_replay_equals_eager_over_a_four_phase_plan():
    cfg, eager_engine, eager_model = build('eager')
    _, graph_engine, graph_model = build('graph')
    x, mod = make_inputs(cfg, 0)
    for engine, model in ((eager_engine, eager_model), (graph_engine, graph_model)):
        seen = engine.warm_schedule(model, x=x, mod=mod)
        assert len(seen) == 8                               # 2 branches x 4 phases
        ledger = engine.compile_budget()
        assert ledger['feasible'] and ledger['total_mma'] <= 2 * ledger['base_mma']
    outs = []
    for call in range(70):                                  # 35 steps x 2 branches
        xi, modi = make_inputs(cfg, call % 3)
        a = eager_engine(eager_model, x=xi, mod=modi)
        b = graph_engine(graph_model, x=xi, mod=modi)
        assert torch.equal(a, b), call
        outs.append(b)
    assert len(graph_engine.graphs) == 8
    assert torch.isfinite(outs[-1].float()).all()
    assert outs[0].data_ptr() != outs[3].data_ptr()         # outputs own their storage
    assert graph_engine.device_status() == 0
    with pytest.raises(RuntimeError, match='Unwarmed'):
        eager_engine(eager_model, x=x[:, :100].contiguous(), mod=mod)


def test_budget_check_fails_closed():
    cfg, engine, model = build('eager', plan_budget=1.125)
    engine.warm_schedule(model, *[], **dict(zip(('x', 'mod'), make_inputs(cfg, 0))))
    with pytest.raises(ValueError, match='exceeded'):
        engine.compile_budget()


def test_repaired_step_tracks_the_unquantized_model():
    """Sanity of the whole block arithmetic: full repair stays close to a bf16 torch forward of the
    same weights (loose bound; operator-level parity is tested against the oracle elsewhere)."""
    from thunderworld_b200.cosmos.dit import DiTConfig, DiTModel, rms_norm, rope_tables, apply_rope
    from thunderworld_b200.cosmos.engine import StepEngine
    from thunderworld_b200.cosmos.settings import LinearSpec, RunConfig
    from thunderworld_b200.config import RepairConfig, RepairPolicy
    from thunderworld_b200 import parallel
    cfg = DiTConfig(hidden=256, heads=2, ffn=512, blocks=1, seed=2)
    run = RunConfig(execution='eager', ffn=LinearSpec(1., 1.), projection=LinearSpec(1., 1.),
                    attention=RepairPolicy(RepairConfig(coverage=1., terms=3)))
    engine = StepEngine(run)
    model = DiTModel(cfg, engine)
    x, mod = make_inputs(cfg, 5)
    engine.warm_schedule(model, x=x, mod=mod)
    y = engine(model, x=x, mod=mod).float()
    # reference forward in fp32 with the same seeded weights
    gen = torch.Generator(device='cpu').manual_seed(cfg.seed * 100003)
    w = {k: (torch.randn(n, kk, generator=gen) * 0.02).bfloat16().float().cuda() for k, (n, kk) in
         (('qkv', (768, 256)), ('out', (256, 256)), ('up', (512, 256)), ('down', (256, 512)))}
    xf, m = x.float(), mod[:, 0].float()
    s1, c1, g1, s2, c2, g2 = m.unbind(1)
    hcur = rms_norm(xf) * (1 + c1[:, None]) + s1[:, None]
    q, k, v = (hcur @ w['qkv'].T).reshape(2, 200, 3, 2, 128).unbind(2)
    cos, sin = rope_tables(200, 'cuda')
    q, k = apply_rope(rms_norm(q), cos, sin), apply_rope(rms_norm(k), cos, sin)
    att = torch.softmax(torch.einsum('bshd,bthd->bhst', q, k) / 128 ** .5, -1)
    a = torch.einsum('bhst,bthd->bshd', att, v).reshape(2, 200, 256)
    xf = xf + g1[:, None] * (a @ w['out'].T)
    hcur = rms_norm(xf) * (1 + c2[:, None]) + s2[:, None]
    xf = xf + g2[:, None] * (torch.nn.functional.gelu(hcur @ w['up'].T, approximate='tanh') @ w['down'].T)
    want = rms_norm(xf)
    rel = float((y - want).norm() / want.norm())
    assert rel < 0.05, rel
