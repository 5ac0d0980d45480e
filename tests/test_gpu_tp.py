"""Tensor-parallel DiT step on two GPUs (NCCL): TP2 output against the single-GPU output of the same
seeded model. With full (or no) A repair the sharded quantizer produces the same bytes as the
unsharded one (global factor); what differs is that each rank rounds its partial sum of a row-split
layer to bf16 before the all-reduce (two roundings of larger partials instead of one of the total).
Bound: relative L2 <= 4e-3 after two blocks.

Second case: a row-split (K divided) linear under a 2x issued-work plan. Each shard quantizes its K half with
the global activation factor, selects its own A1 blocks (quota ceil(a / tp) per shard) with the online
residual-sensitivity selector and issues the plan's W1 tiles that fall into its half. The check feeds the
oracle the per-shard operands, the masks the shards realised (also compared with the oracle's own selection)
and the per-shard tile lists, rounds each partial to bf16 as the ranks do, and sums. Needs two GPUs; skipped
otherwise."""
import os
import socket
import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _run(rank, world, port, results):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        from thunderworld_b200 import parallel
        from thunderworld_b200.cosmos.dit import DiTConfig, DiTModel
        from thunderworld_b200.cosmos.engine import StepEngine
        from thunderworld_b200.cosmos.settings import LinearSpec, RunConfig
        from thunderworld_b200.config import RepairConfig, RepairPolicy
        cfg = DiTConfig(hidden=512, heads=4, ffn=1024, blocks=2, seed=3)
        run = RunConfig(execution='graph', ffn=LinearSpec(1., 1.), projection=LinearSpec(1., 1.),
                        attention=RepairPolicy(RepairConfig(coverage=1., terms=3)), tensor_parallel=world)
        g = torch.Generator().manual_seed(0)
        x = torch.randn(2, 300, cfg.hidden, generator=g).bfloat16().cuda()
        mod = (torch.randn(2, cfg.blocks, 6, cfg.hidden, generator=g) * 0.1).bfloat16().cuda()
        outs = {}
        for name, topo in (('tp', parallel.make_topology(tp_size=world)), ('single', parallel.Topology())):
            engine = StepEngine(run, topo=topo)
            model = DiTModel(cfg, engine, topo)
            engine.warm_schedule(model, x=x, mod=mod)
            a = engine(model, x=x, mod=mod)
            b = engine(model, x=x, mod=mod)               # replay of the captured graph (incl. NCCL)
            assert torch.equal(a, b)
            outs[name] = a.float()
            assert engine.device_status() == 0
            # captured graphs hold NCCL kernels: drop them before the communicator is torn down
            engine.graphs.clear()
            del model, engine
            torch.cuda.synchronize()
        rel = float((outs['tp'] - outs['single']).norm() / outs['single'].norm())
        results[rank] = rel
    finally:
        dist.destroy_process_group()


def _run_plan(rank, world, port, results):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        from oracle import nvfp4_oracle as o
        from thunderworld_b200 import parallel
        from thunderworld_b200.cosmos.budget import RepairPlan
        from thunderworld_b200.cosmos.dit import DiTConfig, DiTModel
        from thunderworld_b200.cosmos.engine import StepEngine
        from thunderworld_b200.cosmos.settings import RunConfig
        cfg = DiTConfig(hidden=512, heads=4, ffn=1024, blocks=1, seed=5)
        h, f = cfg.hidden // 128, cfg.ffn // 128
        lattice = {'qkv': (3 * h, h), 'out': (h, h), 'up': (f, h), 'down': (h, f)}
        rng = np.random.default_rng(11)
        linears, tiles_of = {}, {}
        for part, (nb, kb) in lattice.items():
            tiles_of[part] = sorted(int(t) for t in rng.permutation(nb * kb)[:nb * kb // 2])
            row = {'a_blocks': kb // 2, 'w_blocks': tiles_of[part], 'cross': False}
            for b in range(2):
                for ph in range(4):
                    linears[f'{b}|{ph}|blocks.0.{part}'] = row
        plan = RepairPlan(dict(schema_version=1, budget=2., steps=35, phases=[0, 7, 18, 28, 35], task='t2v',
                               linears=linears, attention={}))
        topo = parallel.make_topology(tp_size=world)
        engine = StepEngine(RunConfig(compute_budget=2.), plan=plan, topo=topo, branches=1)
        block = DiTModel(cfg, engine, topo).blocks[0]
        m, nb, kb = 300, h, f
        width = cfg.ffn // world
        u = torch.from_numpy(o.synthetic_activation(m, cfg.ffn, seed=4)).bfloat16()
        local = u[:, rank * width:(rank + 1) * width].contiguous().cuda()
        engine.warming = True
        y = block._row_split(block.down, local)
        engine.warming = False
        torch.cuda.synchronize()
        assert engine.device_status() == 0
        op = block.down.bound
        assert op.na == -(-(kb // 2) // world)                 # the A quota is divided with the K blocks
        masks = [torch.empty_like(op.am) for _ in range(world)]
        dist.all_gather(masks, op.am.contiguous())
        outs = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(outs, y.contiguous())
        assert all(torch.equal(outs[0], t) for t in outs)      # every rank holds the same reduced output
        if rank == 0:
            # the full weight of the seeded block, drawn in the order qkv, out, up, down
            gen = torch.Generator(device='cpu').manual_seed(cfg.seed * 100003)
            make = lambda n, k: (torch.randn(n, k, generator=gen) * 0.02).bfloat16()
            weight = [make(3 * cfg.hidden, cfg.hidden), make(cfg.hidden, cfg.hidden), make(cfg.ffn, cfg.hidden),
                      make(cfg.hidden, cfg.ffn)][3].float().numpy()
            x = u.float().numpy()
            factor = o.tensor_factor(o.scaled_input(x))        # global: max over both halves
            total = np.zeros((m, cfg.hidden), np.float32)
            for r in range(world):
                xs, ws = x[:, r * width:(r + 1) * width], weight[:, r * width:(r + 1) * width]
                ac, asb, _ = o.quantize_linear_input(xs, factor=factor)
                wc, wsb, wf = o.quantize_weight(ws)
                sens = (ws.astype(np.float64) ** 2).sum(0)
                scores, _ = o.residual_scores(xs, None, sens, factor=factor)
                chosen = o.choose_blocks(scores, op.na)
                realised = masks[r].cpu().numpy()
                assert realised.sum(1).tolist() == [op.na] * realised.shape[0]
                assert np.array_equal(realised, chosen), (r, realised, chosen)
                tiles = parallel.remap_tiles(tiles_of['down'], nb, kb, world, r, 'row')
                assert len(tiles) > 0
                total += o.repair_linear(ac, asb, factor, wc, wsb, wf, m, a_mask=realised, w_tiles=tiles)
            want = o.bf16_round(total)
            got = y.float().cpu().numpy()
            results['rel'] = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    finally:
        dist.destroy_process_group()


def _run_rows(rank, world, port, results):
    """One batch entry under TP2 and a 2x plan: the row-sharded (reduce-scatter / all-gather of packed bytes) execution
    gives the same bits as the all-reduce execution, for a token count that leaves padding rows in the last shard."""
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port), NCCL_NVLS_ENABLE='0')
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        from thunderworld_b200 import parallel
        from thunderworld_b200.cosmos.budget import RepairPlan
        from thunderworld_b200.cosmos.dit import DiTConfig, DiTModel
        from thunderworld_b200.cosmos.engine import StepEngine
        from thunderworld_b200.cosmos.settings import RunConfig
        cfg = DiTConfig(hidden=512, heads=4, ffn=1024, blocks=2, seed=7)
        h, f = cfg.hidden // 128, cfg.ffn // 128
        lattice = {'qkv': (3 * h, h), 'out': (h, h), 'up': (f, h), 'down': (h, f)}
        rng = np.random.default_rng(5)
        linears = {}
        for i in range(cfg.blocks):
            for part, (nb, kb) in lattice.items():
                row = {'a_blocks': kb // 2, 'w_blocks': sorted(int(t) for t in rng.permutation(nb * kb)[:nb * kb // 2]), 'cross': False}
                for b in range(2):
                    for ph in range(4):
                        linears[f'{b}|{ph}|blocks.{i}.{part}'] = row
        plan = RepairPlan(dict(schema_version=1, budget=2., steps=35, phases=[0, 7, 18, 28, 35], task='t2v',
                               linears=linears, attention={}))
        g = torch.Generator().manual_seed(0)
        outs = {}
        for tokens in (300, 512):                              # 300: the second shard holds 44 rows and 212 padding rows
            x = torch.randn(1, tokens, cfg.hidden, generator=g).bfloat16().cuda()
            mod = (torch.randn(1, cfg.blocks, 6, cfg.hidden, generator=g) * 0.1).bfloat16().cuda()
            for name, sharded in (('rows', True), ('allreduce', False)):
                topo = parallel.make_topology(tp_size=world)
                engine = StepEngine(RunConfig(compute_budget=2.), plan=plan, topo=topo, branches=1)
                model = DiTModel(cfg, engine, topo)
                model.row_sharded = sharded
                engine.warm_schedule(model, x=x, mod=mod)
                a = engine(model, x=x, mod=mod)
                b = engine(model, x=x, mod=mod)               # graph replay, collectives inside
                assert torch.equal(a, b)
                assert engine.device_status() == 0
                outs[name] = a.clone()
                engine.graphs.clear()
                del model, engine
                torch.cuda.synchronize()
            assert outs['rows'].shape == (1, tokens, cfg.hidden)
            assert torch.isfinite(outs['rows'].float()).all()
            results[(rank, tokens)] = bool(torch.equal(outs['rows'], outs['allreduce']))
    finally:
        dist.destroy_process_group()


def _launch(target, results):
    ctx = mp.get_context('spawn')
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0)); port = s.getsockname()[1]
    procs = [ctx.Process(target=target, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:                                       # never leave a rank behind holding the GPUs
        p.kill()
        p.join()
    assert not stuck, 'a rank did not finish within the time limit'
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_tp2_matches_single_gpu():
    results = mp.get_context('spawn').Manager().dict()
    _launch(_run, results)
    assert len(results) == 2 and all(rel <= 4e-3 for rel in results.values()), dict(results)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_tp2_row_split_under_a_2x_plan_matches_the_oracle_with_per_shard_masks():
    results = mp.get_context('spawn').Manager().dict()
    _launch(_run_plan, results)
    # each partial is within 1e-3 of its oracle; the sum of two bf16-rounded partials is rounded once more
    assert 'rel' in results and results['rel'] <= 2e-3, dict(results)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_tp2_row_sharded_step_equals_the_allreduce_step_bit_for_bit():
    results = mp.get_context('spawn').Manager().dict()
    _launch(_run_rows, results)
    assert len(results) == 4 and all(results.values()), dict(results)


def test_shard_factor_is_an_ieee_division_on_the_device():
    """max|x| / 2688 computed by the tensor-parallel helper equals the correctly rounded float32 quotient that the
    unsharded quantizer kernel (and the CPU reference) produce; 66 / 2688 is a peak where multiplying by the
    rounded reciprocal lands one ulp away."""
    from thunderworld_b200 import parallel
    peaks = np.concatenate([np.float32([66., 1., 447.5, 3e-3]), np.random.default_rng(0).uniform(1e-2, 500, 4096)]).astype(np.float32)
    for p in peaks[:64]:
        got = parallel.factor_of_peak(torch.tensor([p], device='cuda'))
        assert got.dtype == torch.float32 and got.shape == ()
        assert np.float32(got.item()) == np.float32(p) / np.float32(2688.), p
    assert float(parallel.factor_of_peak(torch.zeros(1, device='cuda'))) == 1.
