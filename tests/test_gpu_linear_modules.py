"""GPU tests of the module-level operator surface: FP4Linear and RepairLinear against the oracle
(tolerance: relative L2 <= 1e-3 against the fp32-accumulated, bf16-rounded emulation)."""
from types import SimpleNamespace
import numpy as np
import pytest
import torch
from oracle import nvfp4_oracle as o

pytestmark = pytest.mark.gpu
TOL = 1e-3


def as_np(t):
    return (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).cpu().numpy()


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def test_fp4linear_full_repair_with_bias_and_prescale():
    from thunderworld_b200.linear import FP4Linear
    from thunderworld_b200.config import LinearRepairConfig
    m, n, k = 200, 256, 384
    x = o.synthetic_activation(m, k, 1)
    w = o.synthetic_weight(n, k, 1)
    d = (np.random.default_rng(0).random(k) + 0.5).astype(np.float32)
    bias = o.bf16_round(np.random.default_rng(1).standard_normal(n).astype(np.float32))
    layer = FP4Linear.from_float(torch.from_numpy(w).cuda().bfloat16(), prescale=torch.from_numpy(d).cuda(),
                                 bias=torch.from_numpy(bias).cuda(), config=LinearRepairConfig(coverage=1.0))
    y = layer(torch.from_numpy(x).cuda().bfloat16().reshape(2, 100, k))
    assert y.shape == (2, 100, n)
    wc, wsb, wf = o.quantize_weight(w, d)
    assert np.array_equal(as_np(layer.weight_codes), wc[0]) and np.array_equal(as_np(layer.weight_scales), wsb[0])
    ac, asb, af = o.quantize_linear_input(x, d, rows_padded=208)
    want = o.repair_linear(ac, asb, af, wc, wsb, wf, m, a_full=True, bias=bias)
    assert rel_l2(y.float().cpu().numpy().reshape(m, n), want) <= TOL
    with pytest.raises(ValueError):
        layer(torch.zeros(4, 100, device='cuda', dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        layer(torch.zeros(4, k, device='cuda', dtype=torch.bfloat16, requires_grad=True))


def test_fp4linear_explicit_mask_per_output_block():
    from thunderworld_b200.linear import FP4Linear
    m, n, k = 300, 384, 512
    x = o.synthetic_activation(m, k, 2)
    w = o.synthetic_weight(n, k, 2)
    layer = FP4Linear.from_float(torch.from_numpy(w).cuda().bfloat16())
    mask = np.random.default_rng(3).random((3, 3, 4)) < 0.5
    y = layer(torch.from_numpy(x).cuda().bfloat16(), repair_mask=torch.from_numpy(mask).cuda())
    wc, wsb, wf = o.quantize_weight(w)
    ac, asb, af = o.quantize_linear_input(x, rows_padded=304)
    ac, asb = o.zero_unselected_residual(ac, asb, mask.any(1))
    want = np.concatenate([o.repair_linear(ac, asb, af, wc[:, nb * 128:(nb + 1) * 128], wsb[:, nb * 128:(nb + 1) * 128], wf, m,
                                           a_mask=mask[:, nb]) for nb in range(3)], axis=1)
    assert rel_l2(y.float().cpu().numpy(), want) <= TOL
    with pytest.raises(ValueError):
        layer(torch.from_numpy(x).cuda().bfloat16(), repair_mask=torch.zeros(3, 3, 3, device='cuda', dtype=torch.bool))


def torch_block_rank(x, prescale, m, k):
    """The sampled-energy ranking in plain torch (the checker of the CUDA activation_rank kernel): eight rows and
    eight columns (every 16th) of bf16(x*d) per 128x128 block, stable descending argsort."""
    mb, kb = (m + 127) // 128, k // 128
    rows = (torch.arange(mb, device=x.device)[:, None] * 128 + torch.arange(8, device=x.device)[None, :] * 16)
    rows = rows.clamp_max(m - 1).reshape(-1)
    sample = (x[rows][:, ::16].float() * prescale[::16]).bfloat16().float()
    energy = sample.square().reshape(mb, 8, kb, 8).sum((1, 3))
    order = torch.argsort(energy, dim=1, descending=True, stable=True)
    rank = torch.empty_like(order)
    rank.scatter_(1, order, torch.arange(kb, device=x.device).expand(mb, kb))
    return rank.int()


@pytest.mark.parametrize('m,k', [(256, 1024), (300, 2048), (129, 24576)])
def test_activation_rank_kernel_matches_torch_ranking(m, k):
    from thunderworld_b200 import ops
    x = torch.from_numpy(o.synthetic_activation(m, k, 6)).cuda().bfloat16()
    d = (torch.rand(k, device='cuda') * 1.5 + .5)
    for prescale in (None, d):
        got = ops.activation_rank(x, prescale)
        want = torch_block_rank(x, torch.ones(k, device='cuda') if prescale is None else prescale, m, k)
        assert got.shape == want.shape and got.dtype == torch.int32
        assert sorted(got[0].tolist()) == list(range(k // 128))
        # float32 summation order may swap blocks of (nearly) equal energy
        assert (got != want).float().mean() < 0.02


def test_fp4linear_explicit_mask_with_256_wide_outputs():
    """An explicit [M128, N128, K128] mask with N a multiple of 256: one A support per output block, which only
    the 128-wide tiles can honour."""
    from thunderworld_b200.linear import FP4Linear
    from thunderworld_b200.config import LinearRepairConfig
    m, n, k = 384, 512, 512
    x = o.synthetic_activation(m, k, 9)
    w = o.synthetic_weight(n, k, 9)
    layer = FP4Linear.from_float(torch.from_numpy(w).cuda().bfloat16(), config=LinearRepairConfig(coverage=0.5))
    mask = np.random.default_rng(9).random((3, 4, 4)) < 0.4
    y = layer(torch.from_numpy(x).cuda().bfloat16(), repair_mask=torch.from_numpy(mask).cuda())
    wc, wsb, wf = o.quantize_weight(w)
    ac, asb, af = o.quantize_linear_input(x, rows_padded=384)
    ac, asb = o.zero_unselected_residual(ac, asb, mask.any(1))
    want = np.concatenate([o.repair_linear(ac, asb, af, wc[:, nb * 128:(nb + 1) * 128], wsb[:, nb * 128:(nb + 1) * 128], wf, m,
                                           a_mask=mask[:, nb]) for nb in range(4)], axis=1)
    assert rel_l2(y.float().cpu().numpy(), want) <= TOL


def test_fp4linear_partial_coverage_uses_sampled_ranking():
    from thunderworld_b200.linear import FP4Linear, sampled_block_rank
    from thunderworld_b200.config import LinearRepairConfig
    m, n, k = 256, 256, 1024
    x = torch.from_numpy(o.synthetic_activation(m, k, 4)).cuda().bfloat16()
    w = torch.from_numpy(o.synthetic_weight(n, k, 4)).cuda().bfloat16()
    layer = FP4Linear.from_float(w, config=LinearRepairConfig(coverage=0.5, output_budgets=((1, 0.25),)))
    rank = sampled_block_rank(x, layer.prescale, m, k)
    assert sorted(rank[0].tolist()) == list(range(8))
    mask = (rank[:, None, :] < torch.tensor([4, 2], device='cuda')[None, :, None]).contiguous()
    assert torch.equal(layer(x), layer(x, repair_mask=mask))


def make_plan(name, nb, kb):
    from thunderworld_b200.cosmos.budget import RepairPlan
    linears = {}
    for b in range(2):
        for p in range(4):
            linears[f'{b}|{p}|{name}'] = {'a_blocks': [0, 1, 2, kb][p], 'w_blocks': [[], [1, 5], [0, 1, 2, 7], [3]][p],
                                          'cross': p == 2}
    return RepairPlan(dict(schema_version=1, budget=2., steps=35, phases=[0, 7, 18, 28, 35], task='t', linears=linears,
                           attention={}))


def test_repair_linear_follows_the_plan_per_phase():
    from thunderworld_b200.cosmos.linears import RepairLinear
    from thunderworld_b200.cosmos.settings import LinearSpec
    m, n, k = 260, 256, 512
    nb, kb = n // 128, k // 128
    torch.manual_seed(0)
    source = torch.nn.Linear(k, n, bias=True)
    source.weight.data = torch.from_numpy(o.synthetic_weight(n, k, 5))
    plan = make_plan('blk.proj', nb, kb)
    state = SimpleNamespace(phase=0)
    recorded = []
    controller = SimpleNamespace(budget_plan=plan, warming=True, config=SimpleNamespace(activation_repair_energy=1.),
                                 linear_spec=lambda name, default: plan.linear('t', 0, state.phase, name),
                                 record_linear=lambda *a: recorded.append(a))
    layer = RepairLinear(source, controller, 'blk.proj', LinearSpec(0, 0))
    assert layer.weight_union == [0, 1, 2, 3, 5, 7] and layer.asset['storage_schema'] == 2
    x = torch.from_numpy(o.synthetic_activation(m, k, 6)).cuda().bfloat16()
    warm = []
    for ph in range(4):
        state.phase = ph
        warm.append(layer(x))
    assert len(recorded) == 4 and len(layer.ops) == 4
    controller.warming = False
    w = o.bf16_round(source.weight.detach().numpy())
    wc, wsb, wf = o.quantize_weight(w)
    bias = o.bf16_round(source.bias.detach().numpy())
    sens = (w.astype(np.float64) ** 2).sum(0).astype(np.float32)
    ac, asb, af = o.quantize_linear_input(x.float().cpu().numpy(), rows_padded=272)
    scores, _ = o.residual_scores(x.float().cpu().numpy(), None, sens)
    for ph in range(4):
        state.phase = ph
        y = layer(x)
        assert torch.equal(y, warm[ph])
        row = plan.linears[f'0|{ph}|blk.proj']
        na = row['a_blocks']
        op = layer.bound
        mask = op.am.cpu().numpy() if 0 < na < kb else None
        if mask is not None:
            assert mask.sum(1).tolist() == [na] * 3
            want_mask = o.choose_blocks(scores, na)
            assert (mask != want_mask).sum() <= 2          # float32 summation order near ties
        # the bias joins the fp32 accumulator before the single bf16 rounding (TwRepairIO.bias)
        want = o.repair_linear(ac, asb, af, wc, wsb, wf, m, a_mask=mask, a_full=na == kb, w_tiles=row['w_blocks'],
                               cross=row['cross'], bias=bias, round_bf16=True)
        assert rel_l2(y.float().cpu().numpy(), want) <= TOL, ph
    # all operators share W0 and the union bank
    ops_ = list(layer.ops.values())
    assert all(op.wc.data_ptr() == ops_[0].wc.data_ptr() for op in ops_)
    assert all(op.wr.data_ptr() == ops_[1].wr.data_ptr() for op in ops_[1:])
    state.phase = 0
    with pytest.raises(RuntimeError, match='Unwarmed'):
        layer(x[:100])
