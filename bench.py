"""Benchmark of the selective-FP4-repair hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--budget 2.0|1.5|1.0]
                  [--workload auto|step|projections|attention]

Default workload (`auto`): one Cosmos3-Nano-shaped DiT denoise step (28 blocks, hidden 4096, 32 heads x 128,
FFN 16384, 3840 tokens x CFG 2, seeded 2x issued-work plan) replayed as one CUDA Graph, the same work at every
GPU count (strong scaling): N = 1 one GPU; N = 2 tensor parallel over 2 (column-split QKV / FFN-up, row-split
out-proj / FFN-down with NCCL all-reduces inside the graph); N = 4 TP2 x CFG2 (each CFG branch on its own GPU
pair); N = 8 TP4 x CFG2. `value` is effective TFLOP/s on issued FP4 work of the step over all ranks,
`ms_per_step` the denoise-step time. Beside it, every rank also runs the Cosmos3-Edge-shaped projection set
(M = 7680 tokens; QKV 6144x2048, out-proj 2048x2048, FFN-up 8192x2048, FFN-down 2048x8192: online activation
quantizer with A1 block selection, then the fused repair GEMM with the seeded W1 tile plan, FFN-down with the
A1W1 cross term) as independent replicas: that is where the dominant kernel is timed alone (`roofline`),
where outputs are checked against the CPU oracle (`parity`) and what `projection_set` reports.
`--workload projections` makes the projection set the headline (weak scaling over replicas).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_TOKENS = 7680
PROJECTIONS = (('qkv', 6144, 2048), ('out', 2048, 2048), ('ffn_up', 8192, 2048), ('ffn_down', 2048, 8192))
NOMINAL_FP4_TFLOPS = 9000.0
# dram__bytes_read.sum + dram__bytes_write.sum of the four fused_kernel<256> launches of one step (M = 7680,
# 2x plan), from the one-pass full-size ncu capture summarised under profiles/ (bytes per launch, by layer).
NCU_TRAFFIC_BY_LAYER = {'qkv': 66.3e6, 'out': 18.8e6, 'ffn_up': 99.5e6, 'ffn_down': 83.7e6}
NCU_TRAFFIC_BYTES_PER_LAUNCH = sum(NCU_TRAFFIC_BY_LAYER.values()) / len(NCU_TRAFFIC_BY_LAYER)


def plan_for(name, n, k, budget, seed):
    """Issued-work plan of one layer: A quota, W1 tile ids, cross. 1.5x: a = KB/4 and 25 % of the
    W tiles; 2x: a = KB/2 and 50 %. FFN-down adds the cross term and trims W tiles (highest ids
    first) until the provable bound 1 + a/KB + w/(NB*KB) + cross_bound <= budget holds."""
    kb, nb = k // 128, n // 128
    if budget <= 1.0:                     # base W4A4: no repair term
        return 0, [], False
    frac = 0.25 if budget < 1.75 else 0.5
    na = int(kb * frac)
    rng = np.random.default_rng(seed + 7919)
    tiles = sorted(int(t) for t in rng.permutation(nb * kb)[:int(round(frac * nb * kb))])
    cross = name == 'ffn_down'
    if cross:
        def ratio(ts):
            counts = np.bincount(np.array(ts, dtype=np.int64) % kb, minlength=kb) if ts else np.zeros(kb, int)
            bound = int(np.sort(counts)[::-1][:na].sum())
            return 1 + na / kb + len(ts) / (nb * kb) + bound / (nb * kb)
        while tiles and ratio(tiles) > budget:
            tiles = tiles[:-1]
    return na, tiles, cross


class Layer:
    """One projection: offline weights + plan + preallocated activation."""

    def __init__(self, name, n, k, m, budget, seed, device):
        import torch
        from thunderworld_b200.native import Native, quantize_weight
        self.name, self.n, self.k, self.m = name, n, k, m
        self.na, self.tiles, self.cross = plan_for(name, n, k, budget, seed)
        kb, nb, mb = k // 128, n // 128, (m + 127) // 128
        gen = torch.Generator(device='cpu').manual_seed(seed)
        x = torch.randn(m, k, generator=gen)
        cols = torch.randperm(k, generator=gen)[:max(1, round(0.005 * k))]
        x[:, cols] *= 20
        self.x_host = x.bfloat16().pin_memory()
        self.x = self.x_host.to(device, non_blocking=True)
        w = (torch.randn(n, k, generator=gen) * 0.02).bfloat16().to(device)
        wc, ws, wg = quantize_weight(w)
        self.weights = (wc, ws, wg)                                               # both planes, for the parity check
        am = torch.zeros(mb, kb, dtype=torch.bool); am[:, :self.na] = True       # placeholder support, rewritten online
        wm = torch.zeros(nb * kb, dtype=torch.bool); wm[self.tiles] = True
        self.op = Native(wc, ws, wg, torch.ones(k, device=device), am.repeat_interleave(128, 1).to(device),
                         wm.reshape(nb, kb).repeat_interleave(128, 0).repeat_interleave(128, 1).to(device),
                         cross=self.cross)
        self.sens = (w.float() ** 2).sum(0).contiguous()                          # selector weights: sum_n W^2
        self.out = torch.empty(m, n, device=device, dtype=torch.bfloat16)
        self.out_host = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()
        self.packed = None
        del w

    def quantize(self, x):
        from thunderworld_b200 import ops
        if self.na == 0:
            self.packed = ops.quantize(x, None, repair=0, wg=self.op.wg, out=self.packed)
        else:
            self.packed = ops.quantize(x, None, repair=3, na=self.na, sensitivity=self.sens, mask=self.op.am,
                                       wg=self.op.wg, out=self.packed)
        return self.packed

    def gemm(self, x):
        return self.op.run_packed(x, self.packed, out=self.out)

    def issued_flops(self):
        """Issued FP4 FLOPs with the realised A support (M is a multiple of 128: no padding)."""
        from thunderworld_b200.cosmos.budget import linear_cost
        support = [row.nonzero().flatten().tolist() for row in self.op.am.cpu()]
        return linear_cost(self.m, self.n, self.k, a_blocks=self.na, w_blocks=self.tiles, cross=self.cross,
                           a_support=support)['total_mma']


def layer_parity(layer, blocks):
    """Checks one projection of the timed workload against the CPU oracle on the given M128 row blocks, at full
    N and K (output rows are independent given the packed bytes, so a few blocks cost seconds on the host):
    the quantizer's bytes of those rows (bit-exact, given the tensor factor the GPU reduced over all rows), the
    selector's realised support of those blocks (equal to the oracle's ranking except blocks whose score lies
    within float32 rounding of the cut) and the fused GEMM output (relative L2 against the decoded fp32
    emulation fed with the GPU's own bytes and realised mask). Returns a dict; raises nothing."""
    import torch
    from oracle import nvfp4_oracle as o
    u8 = lambda t: (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).cpu().numpy()
    op, pk = layer.op, layer.packed
    kb = layer.k // 128
    rows = torch.cat([torch.arange(b * 128, min((b + 1) * 128, layer.m)) for b in blocks]).to(layer.x.device)
    codes, scales = u8(pk.codes[:, rows]), u8(pk.scales[:, rows])
    factor = pk.factor.item()
    x_rows = layer.x[rows].float().cpu().numpy()
    oc, osb, _ = o.quantize_linear_input(x_rows, factor=factor, rows_padded=len(rows))
    bytes_equal = bool(np.array_equal(oc[:codes.shape[0]], codes) and np.array_equal(osb[:scales.shape[0]], scales))
    mask = None
    mask_ok = True
    if layer.na:
        mask = op.am[torch.as_tensor(blocks, device=op.am.device)].cpu().numpy()
        scores, _ = o.residual_scores(x_rows, None, layer.sens.cpu().numpy(), factor=factor)
        want = o.choose_blocks(scores, layer.na)
        for i in range(len(blocks)):
            diff = np.flatnonzero(mask[i] != want[i])
            cut = np.sort(scores[i])[-layer.na]
            mask_ok &= bool(mask[i].sum() == layer.na and np.all(np.abs(scores[i][diff] - cut) <= 1e-4 * cut))
    wc, ws, wg = layer.weights
    want = o.repair_linear(codes, scales, factor, u8(wc), u8(ws), wg.item(), len(rows), a_mask=mask,
                           a_full=layer.na == kb, w_tiles=layer.tiles, cross=layer.cross)
    got = layer.out[rows].float().cpu().numpy()
    rel = float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))
    return {'layer': layer.name, 'rows': int(len(rows)), 'rel_l2': rel, 'packed_bytes_bit_exact': bytes_equal,
            'selector_matches_oracle': bool(mask_ok), 'finite': bool(np.isfinite(got).all())}


class ClockSampler(threading.Thread):
    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag = index, [], set(), False
        self.max_mhz = None

    def run(self):
        fields = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
                  'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')
        names = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')
        while not self.stop_flag:
            try:
                out = subprocess.run(['nvidia-smi', f'--query-gpu={fields}', '--format=csv,noheader,nounits', '-i',
                                      str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                parts = [p.strip() for p in out.split(',')]
                self.samples.append(float(parts[0])); self.max_mhz = float(parts[1])
                for name, val in zip(names, parts[2:]):
                    if val.lower().startswith('active'):
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.05)

    def result(self):
        return {'sm_mhz': float(np.median(self.samples)) if self.samples else None, 'sm_max_mhz': self.max_mhz,
                'reasons': sorted(self.reasons), 'samples': len(self.samples)}


def cpu_baseline(budget, threads, sample_rows=1536, shape=None):
    """The reference's PyTorch FP4 emulation of the same path on the host cores (threaded torch restatement,
    oracle/torch_emulation.py): quantize + select + decoded fp32 matmuls per term, on a bounded sample (the
    first `sample_rows` rows of one QKV projection)."""
    import torch
    from oracle import torch_emulation as te
    from oracle import nvfp4_oracle as o
    torch.set_num_threads(max(1, threads))          # explicit: torchrun exports OMP_NUM_THREADS=1
    name, n, k = shape or PROJECTIONS[0]
    na, tiles, cross = plan_for(name, n, k, budget, 0)
    x = torch.from_numpy(o.synthetic_activation(sample_rows, k, 0))
    w = torch.from_numpy(o.synthetic_weight(n, k, 0))
    wc, ws, wf = te.quantize(w)                     # offline in the real path: not timed
    sens = (w.double() ** 2).sum(0).float()
    t0 = time.perf_counter()
    ac, asc, af = te.quantize(x)
    mask = te.select_blocks(x, af, ac[0], asc[0], sens, na) if na else None
    te.repair_linear(ac, asc, af, wc, ws, wf, sample_rows, a_mask=mask, w_tiles=tiles, cross=cross)
    dt = time.perf_counter() - t0
    flops = o.issued_flops(sample_rows, n, k, a_mask=None if mask is None else mask.numpy(), w_tiles=tiles, cross=cross)
    terms = 1 + (na > 0) + (len(tiles) > 0) + (cross and na > 0 and len(tiles) > 0)
    return flops / dt / 1e12, dt, (f'{sample_rows} rows of the {name} projection ({n}x{k}): quantize + select + '
                                   f'{terms}-term decoded fp32 matmul, torch CPU emulation on {threads} threads')


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_reference(args):
    """The reference arm: the CPU emulation of the path on all host threads; rank 0 alone runs it."""
    if int(os.environ.get('RANK', '0')) != 0:
        return
    threads = host_threads()
    step_mode = args.workload in ('auto', 'step')
    shape = ('qkv', 3 * 4096, 4096) if step_mode else None
    for _ in range(args.warmup):
        cpu_baseline(args.budget, threads, 256, shape)
    vals, times, sample = [], [], ''
    for _ in range(args.steps):
        v, dt, sample = cpu_baseline(args.budget, threads, 1536, shape)
        vals.append(v); times.append(dt)
    value = float(np.mean(vals))
    config = step_config(args, max(args.gpus, 1)) if step_mode else workload_config(args.budget, 1)
    line = {'metric': METRIC_STEP if step_mode else METRIC_PROJ, 'impl': 'reference', 'value': value,
            'unit': 'TFLOP/s', 'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': float(np.mean(times)) * 1e3, 'higher_is_better': True,
            'scaling': 'strong' if step_mode else 'weak', 'vs_baseline': None,
            'dtype': 'nvfp4 emulated in fp32 (e2m1 x ue4m3 decoded, fp32 matmul)', 'data': 'synthetic',
            'config': config,
            'cpu_baseline': {'value': value, 'unit': 'TFLOP/s', 'cores': threads, 'kind': 'port', 'sample': sample},
            'e2e': {'value': value, 'unit': 'TFLOP/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0}}
    print(json.dumps(line))


METRIC_PROJ = 'repaired NVFP4 GEMM effective TFLOPS on issued FP4 work'
METRIC_STEP = 'repaired NVFP4 GEMM effective TFLOPS on issued FP4 work (DiT denoise step)'


def step_topology(world, cfg_parallel):
    """(tp, cfg) for a world size: the two CFG branches are independent and split first (no collective inside the
    step); tensor parallelism divides each branch from four GPUs on."""
    cfg = cfg_parallel or (2 if world >= 2 else 1)
    return world // cfg, cfg


def step_config(args, world):
    tp, cfg = step_topology(world, args.cfg_parallel)
    blocks = args.blocks or {'nano': 28, 'super': 48}[args.model]
    return {'workload': f'{args.model}-shaped DiT denoise step: {blocks} blocks, {args.tokens} tokens x CFG 2, '
                        f'{args.budget}x issued-work plan, one CUDA Graph replay per step',
            'budget': args.budget, 'parallelism': f'tp{tp} x cfg{cfg}',
            'l2': 'per-step working set (weights ~2.9 GB at tp1, activations 63 MB per tensor) exceeds the 126 MB L2'}


def workload_config(budget, world, m=M_TOKENS, layers='qkv,out,ffn_up,ffn_down'):
    return {'workload': f'cosmos3-edge projection set, M={m}, layers {layers}, '
                        f'{budget}x issued-work plan, cross term on FFN-down',
            'budget': budget, 'replicas': world, 'parallelism': f'dp{world}',
            'l2': 'per-step working set ~0.55 GB (activations, packed planes, outputs) exceeds the 126 MB L2'}


def step_plan(cfg, budget, seed=0):
    """Seeded issued-work plan of a DiT: per layer a = KB/2 (KB/4 at 1.5x) and 50 % (25 %) of the W1 tiles,
    the same for both CFG branches and all four phases; attention quotas cover the same fraction of key tiles."""
    from thunderworld_b200.cosmos.budget import RepairPlan
    h, f = cfg.hidden // 128, cfg.ffn // 128
    lattice = {'qkv': (3 * h, h), 'out': (h, h), 'up': (f, h), 'down': (h, f)}
    frac = 0. if budget <= 1. else (0.25 if budget < 1.75 else 0.5)
    rng = np.random.default_rng(seed)
    linears, attention = {}, {}
    for i in range(cfg.blocks):
        for part, (nb, kb) in lattice.items():
            tiles = sorted(int(t) for t in rng.permutation(nb * kb)[:int(frac * nb * kb)])
            row = {'a_blocks': int(frac * kb), 'w_blocks': tiles, 'cross': False}
            for b in range(2):
                for ph in range(4):
                    linears[f'{b}|{ph}|blocks.{i}.{part}'] = row
    return RepairPlan(dict(schema_version=1, budget=max(budget, 1.), steps=35, phases=[0, 7, 18, 28, 35], task='t2v',
                           linears=linears, attention={})), frac


def measure_step(args, device, rank, world, dist):
    """DiT denoise step (Nano- or Super-shaped synthetic DiT): one CUDA Graph replay per step, CFG batch 2 (split
    over GPU groups when cfg > 1), tensor parallel inside a group. Returns the rank-0 result dictionary."""
    import torch
    from thunderworld_b200 import _lib, parallel
    from thunderworld_b200.config import RepairConfig, RepairPolicy
    from thunderworld_b200.cosmos import dit
    from thunderworld_b200.cosmos.engine import StepEngine
    from thunderworld_b200.cosmos.settings import RunConfig
    tp, cfg_par = step_topology(world, args.cfg_parallel)
    topo = parallel.make_topology(tp_size=tp, cfg_size=cfg_par) if world > 1 else parallel.Topology()
    base = {'nano': dit.NANO, 'super': dit.SUPER}[args.model]
    cfg = dit.DiTConfig(base.hidden, base.heads, base.ffn, args.blocks or base.blocks)
    plan, frac = step_plan(cfg, args.budget)
    nt = (args.tokens + 127) // 128
    quota = max(0, int(nt * frac) - 1)          # one tile less than the fraction: leaves room for the selector's own MMAs
    local_heads = cfg.heads // topo.tp_size
    run = RunConfig(compute_budget=max(args.budget, 1.),
                    attention=RepairPolicy(RepairConfig(coverage=0., head_quotas=(quota,) * local_heads, terms=3)))
    engine = StepEngine(run, plan=plan, topo=topo, branches=1)
    engine._branch_offset = topo.cfg_rank if cfg_par > 1 else 0
    model = dit.DiTModel(cfg, engine, topo, device)
    model.row_sharded = args.tp_row_sharded
    batch = 2 // cfg_par
    g = torch.Generator().manual_seed(0)
    x_all = torch.randn(2, args.tokens, cfg.hidden, generator=g)
    cols = torch.randperm(cfg.hidden, generator=g)[:max(1, round(0.005 * cfg.hidden))]
    x_all[..., cols] *= 20
    mod_all = (torch.randn(2, cfg.blocks, 6, cfg.hidden, generator=g) * 0.1).bfloat16()
    first = topo.cfg_rank * batch if cfg_par > 1 else 0
    x_host = x_all[first:first + batch].bfloat16().contiguous().pin_memory()
    mod_host = mod_all[first:first + batch].contiguous().pin_memory()
    x, mod = x_host.to(device), mod_host.to(device)
    calls0 = _lib.calls
    engine.warm_schedule(model, x=x, mod=mod)
    calls_per_step = _lib.calls - calls0          # C-ABI kernel calls of one eager pass = launches captured per step
    ledger = engine.compile_budget() if args.budget > 1. else None
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def replay():
        engine.reset_request()
        return engine(model, x=x, mod=mod)

    for _ in range(max(args.warmup, 3)):
        replay()
    barrier()
    sampler = ClockSampler(device.index)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        replay()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    sampler.stop_flag = True
    # end to end: pinned host inputs in, the step's output back to pinned host memory, every step
    out_host = torch.empty_like(x_host).pin_memory()
    for _ in range(0 if args.no_e2e else 2):
        x.copy_(x_host, non_blocking=True); mod.copy_(mod_host, non_blocking=True)
        out_host.copy_(replay(), non_blocking=True)
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record(stream)
    for _ in range(0 if args.no_e2e else args.steps):
        x.copy_(x_host, non_blocking=True); mod.copy_(mod_host, non_blocking=True)
        out_host.copy_(replay(), non_blocking=True)
    s1.record(stream)
    barrier()
    ms_e2e = max(s0.elapsed_time(s1), 1e-9) / args.steps
    # sustained: at least three seconds of back-to-back replays with the SM clock sampled underneath
    sustained = None
    if world == 1 and not args.no_sustained:
        sus = ClockSampler(device.index)
        sus.start()
        n_sus = max(args.steps, int(3000. / ms) + 1)
        u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        u0.record(stream)
        for _ in range(n_sus):
            replay()
        u1.record(stream)
        torch.cuda.synchronize()
        sus.stop_flag = True
        sus.join(timeout=2)
        sustained = {'ms_per_step': u0.elapsed_time(u1) / n_sus, 'steps': n_sus, 'seconds': u0.elapsed_time(u1) / 1e3,
                     'sm_mhz_median': sus.result()['sm_mhz'], 'reasons': sus.result()['reasons']}
    times = torch.tensor([ms, ms_e2e], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(times[0]), float(times[1])
    sampler.join(timeout=2)
    status = engine.device_status()
    rows = list(engine.rows.values())
    # one (branch, phase) of the schedule = the work of one step; attention rows are per batch entry
    issued = sum(r['total_mma'] * (batch if r['kind'] == 'attention' else 1) for r in rows
                 if r['phase'] == 0 and r['branch'] == engine._branch_offset) * topo.tp_size * cfg_par
    result = {'ms': ms, 'ms_e2e': ms_e2e, 'issued': issued, 'clocks': sampler.result(), 'status': status,
              'h2d': (x_host.numel() + mod_host.numel()) * 2, 'd2h': out_host.numel() * 2, 'calls_per_step': calls_per_step,
              'ledger_ratio': None if ledger is None else ledger['ratio'], 'sustained': sustained,
              'parallelism': f'tp{topo.tp_size} x cfg{cfg_par}',
              'collectives': None if topo.tp_size == 1 else
              f'per block: 2 x all_reduce(SUM) of bf16 [{batch * args.tokens}, {cfg.hidden}] and 2 x 4-byte all_reduce(MAX), NCCL, inside the graph'}
    if sustained is not None:
        sustained['value'] = issued / 1e12 / (sustained['ms_per_step'] * 1e-3)
    # the captured graphs hold NCCL kernels: they go before anything tears the communicator down
    engine.graphs.clear()
    del model, engine
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return result


def measure_projections(args, device, rank, world, dist):
    """The projection set on this rank's GPU (replicas under N > 1): whole-set throughput, the fused kernel timed
    alone (roofline), the oracle check of the outputs and the host-buffer (end-to-end) throughput."""
    import torch
    from thunderworld_b200 import ops
    chosen = args.layers.split(',')
    layers = [Layer(name, n, k, args.m_tokens, args.budget, seed, device)
              for seed, (name, n, k) in enumerate(PROJECTIONS) if name in chosen]
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream()

    def step():
        for layer in layers:
            layer.quantize(layer.x)
            layer.gemm(layer.x)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    flops_step = sum(layer.issued_flops() for layer in layers)

    # The denoise step runs under CUDA Graph capture in the runtime this path serves, so the step is
    # captured once and replayed: launches cost no host time inside the timed region.
    side = torch.cuda.Stream()
    g_step = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_step, stream=side):
        step()
    g_gemm = {}
    for layer in layers:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            layer.gemm(layer.x)
        g_gemm[layer.name] = g
    for _ in range(3):
        g_step.replay()
    barrier()

    sampler = ClockSampler(device.index)
    sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record(stream)
    for _ in range(args.steps):
        g_step.replay()
    t1.record(stream)
    barrier()
    ms = t0.elapsed_time(t1)

    # the dominant kernel alone: one launch per layer per step, events around each launch. A spin
    # kernel first lets the host queue everything, so no launch latency sits between the events.
    gemm_events = []
    torch.cuda._sleep(int(2e8))
    for _ in range(args.steps):
        for layer in layers:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            g_gemm[layer.name].replay()
            e1.record(stream)
            gemm_events.append((layer.name, e0, e1))
    barrier()
    sampler.stop_flag = True
    if ops.device_status(device) != 0:
        raise RuntimeError('device status word reports a bounded-wait timeout')
    # outputs of the timed workload against the CPU oracle (after the timed region; rank 0 only)
    parity = None
    if rank == 0 and not args.no_parity:
        g_step.replay()
        torch.cuda.synchronize()
        mb = (args.m_tokens + 127) // 128
        checks = [layer_parity(layer, sorted({0, mb - 1})) for layer in layers]
        parity = {'rel_l2': max(c['rel_l2'] for c in checks), 'rows': sum(c['rows'] for c in checks),
                  'tolerance': 1e-3, 'packed_bytes_bit_exact': all(c['packed_bytes_bit_exact'] for c in checks),
                  'selector_matches_oracle': all(c['selector_matches_oracle'] for c in checks),
                  'against': 'CPU oracle (decoded fp32 emulation), first and last M128 row block of every layer at full N and K',
                  'layers': checks}

    # end to end: pinned host inputs in, outputs back to pinned host memory, every step. The copies run on
    # their own streams (PCIe is full duplex): a layer's upload overlaps the previous layer's quantizer + GEMM
    # and the download of the layer before that. Each layer keeps one device input and one device output, so
    # its upload waits for its previous use to be computed and its compute waits for its previous output to
    # be downloaded.
    g_layer = {}
    for layer in layers:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            layer.quantize(layer.x)
            layer.gemm(layer.x)
        g_layer[layer.name] = g
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    uploaded = {layer.name: torch.cuda.Event() for layer in layers}
    computed = {layer.name: torch.cuda.Event() for layer in layers}
    downloaded = {layer.name: torch.cuda.Event() for layer in layers}
    for layer in layers:
        computed[layer.name].record(stream)
        downloaded[layer.name].record(stream)

    def step_e2e():
        for layer in layers:
            up.wait_event(computed[layer.name])
            with torch.cuda.stream(up):
                layer.x.copy_(layer.x_host, non_blocking=True)
                uploaded[layer.name].record(up)
            stream.wait_event(uploaded[layer.name])
            stream.wait_event(downloaded[layer.name])
            g_layer[layer.name].replay()
            computed[layer.name].record(stream)
            down.wait_event(computed[layer.name])
            with torch.cuda.stream(down):
                layer.out_host.copy_(layer.out, non_blocking=True)
                downloaded[layer.name].record(down)

    def drain_e2e():
        for layer in layers:
            stream.wait_event(downloaded[layer.name])

    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(0 if args.no_e2e else 2):
        step_e2e()
    drain_e2e()
    barrier()
    s0.record(stream)
    for _ in range(0 if args.no_e2e else args.steps):
        step_e2e()
    drain_e2e()
    s1.record(stream)
    barrier()
    ms_e2e = max(s0.elapsed_time(s1), 1e-9)

    times = torch.tensor([ms, ms_e2e], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(times[0]), float(times[1])
    sampler.join(timeout=2)

    per_layer = {}
    for name, e0, e1 in gemm_events:
        per_layer.setdefault(name, []).append(e0.elapsed_time(e1))
    flops_by_layer = {layer.name: layer.issued_flops() for layer in layers}
    gemm_ms = sum(sum(v) for v in per_layer.values())
    gemm_launches = sum(len(v) for v in per_layer.values())
    achieved = sum(flops_by_layer[n_] * len(v) for n_, v in per_layer.items()) / (gemm_ms * 1e-3) / 1e12
    fp4_peak = measured_fp4_peak()
    full = args.m_tokens == M_TOKENS and args.budget == 2.0 and args.layers == 'qkv,out,ffn_up,ffn_down'
    roofline = {'bound': 'tensor', 'kernel': 'fused_kernel (tcgen05 mxf4nvf4 repair GEMM), timed alone on the projection set',
                'achieved': achieved, 'peak': NOMINAL_FP4_TFLOPS, 'unit': 'TFLOP/s', 'frac': achieved / NOMINAL_FP4_TFLOPS,
                'peak_source': 'nominal dense FP4 (MEASURED_PEAKS.json holds no FP4 figure)',
                'peak_measured': fp4_peak, 'frac_measured': achieved / fp4_peak['burst_tflops'] if fp4_peak else None,
                'traffic': NCU_TRAFFIC_BYTES_PER_LAUNCH if full else None,
                'traffic_unit': 'bytes per launch (ncu dram read + write, mean of the four layers)',
                'launches': gemm_launches, 'avg_launch_ms': gemm_ms / gemm_launches,
                'per_layer_tflops': {n_: flops_by_layer[n_] / (np.mean(v) * 1e-3) / 1e12 for n_, v in per_layer.items()},
                'gemm_share_of_projection_set': gemm_ms / ms}
    result = {'value': world * flops_step * args.steps / (ms * 1e-3) / 1e12, 'ms_per_step': ms / args.steps,
              'e2e_value': world * flops_step * args.steps / (ms_e2e * 1e-3) / 1e12, 'e2e_ms_per_step': ms_e2e / args.steps,
              'h2d': sum(l.x_host.numel() * 2 for l in layers), 'd2h': sum(l.out_host.numel() * 2 for l in layers),
              'launches_per_step': len(layers) * 4, 'clocks': sampler.result(), 'roofline': roofline, 'parity': parity}
    del layers, g_step, g_gemm, g_layer
    torch.cuda.empty_cache()
    return result


def measured_fp4_peak():
    """Dense NVFP4 GEMM peak measured on this pool's B200 by baseline/fp4_peak_probe.py (cuBLASLt through
    torch._scaled_mm, 8192^3): the figures of the committed summary profiles/fp4_peak_probe.md."""
    return {'burst_tflops': 5863.4, 'sustained_tflops': 5240.5, 'sustained_sm_mhz_median': 1305.0,
            'how': 'cuBLASLt NVFP4 8192^3 via torch._scaled_mm: best of 10 / back to back for 3.4 s'}


def run_attention(args):
    """Streaming FP4 attention workload: batch 2 (CFG) x heads x seq x 128, self- and
    cross-attention (512 text keys), base and 50 % / 3-term repair; time includes packing and selection."""
    import torch
    from thunderworld_b200 import RepairConfig
    from thunderworld_b200.runtime import _forward
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(0)
    B, H, S = 2, args.att_heads, args.tokens
    results = {}
    for name, sk in (('self', S), ('cross', 512)):
        mk = lambda s_: (torch.randn(B, s_, H, 128, generator=g) * (torch.rand(H, generator=g) * 1.5 + .5)[None, None, :, None]).bfloat16().cuda()
        q, k, v = mk(S), mk(sk), mk(sk)
        for label, cfg in (('base', RepairConfig(coverage=0.)), ('repair50_terms3', RepairConfig(coverage=.5, terms=3))):
            quotas = (torch.tensor(cfg.head_counts(H, sk), device='cuda', dtype=torch.int32),
                      torch.tensor(cfg.pv_counts(H, sk), device='cuda', dtype=torch.int32))
            for _ in range(3):
                _forward(q, k, v, cfg, None, quotas)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                held = _forward(q, k, v, cfg, None, quotas)
            for _ in range(max(args.warmup, 3)):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            nt = (sk + 127) // 128
            issued = 4 * B * H * S * nt * 128 * 128 * (1 + (cfg.terms - 1) * sum(cfg.head_counts(H, sk)) / (H * nt))
            results[f'{name}_{label}'] = {'ms': ms, 'issued_tflop': issued / 1e12, 'tflops': issued / 1e12 / (ms * 1e-3)}
    best = results['self_base']
    print(json.dumps({'metric': 'streaming FP4 attention effective TFLOPS on issued FP4 work', 'value': best['tflops'],
                      'unit': 'TFLOP/s', 'n_gpus': 1, 'steps': args.steps, 'warmup': max(args.warmup, 3),
                      'ms_per_step': best['ms'], 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
                      'dtype': 'nvfp4 (e2m1 x ue4m3, fp32 softmax)', 'data': 'synthetic',
                      'config': {'workload': f'streaming attention: batch 2 x {H} heads x seq {S} x 128, cross 512 keys'},
                      'cases': results,
                      'roofline': {'bound': 'tensor', 'achieved': best['tflops'], 'peak': NOMINAL_FP4_TFLOPS, 'unit': 'TFLOP/s',
                                   'frac': best['tflops'] / NOMINAL_FP4_TFLOPS, 'traffic': None}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', default='ours')
    ap.add_argument('--budget', type=float, default=2.0)
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-parity', action='store_true', help='skip the oracle check of the outputs (profiling runs)')
    ap.add_argument('--no-e2e', action='store_true', help='skip the host-buffer timing (profiling runs)')
    ap.add_argument('--no-sustained', action='store_true', help='skip the three-second sustained run of the step')
    ap.add_argument('--m-tokens', type=int, default=M_TOKENS, help='rows per projection (smaller for profiler captures)')
    ap.add_argument('--layers', default='qkv,out,ffn_up,ffn_down', help='subset of the projection set')
    ap.add_argument('--workload', default='auto', choices=('auto', 'projections', 'step', 'attention'))
    ap.add_argument('--model', default='nano', choices=('nano', 'super'))
    ap.add_argument('--tp-row-sharded', action='store_true', help='tensor-parallel step: keep the residual stream row-sharded (reduce-scatter / all-gather of packed bytes) instead of all-reducing the row-split outputs')
    ap.add_argument('--blocks', type=int, default=0, help='override the number of DiT blocks (step workload)')
    ap.add_argument('--tokens', type=int, default=3840)
    ap.add_argument('--cfg-parallel', type=int, default=0, help='CFG groups (0: 2 from two GPUs on, else 1; 1 forces tensor parallelism only)')
    ap.add_argument('--att-heads', type=int, default=32)
    args = ap.parse_args()
    if args.impl == 'reference':
        return run_reference(args)
    if args.workload == 'attention':
        return run_attention(args)

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get('RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    if not torch.cuda.is_available():
        raise RuntimeError('bench.py needs a CUDA device: the product path has no CPU fallback')
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    if world > 1:
        os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
        dist.init_process_group('nccl', device_id=device)

    proj = measure_projections(args, device, rank, world, dist) if args.workload in ('auto', 'projections') else None
    step = measure_step(args, device, rank, world, dist) if args.workload in ('auto', 'step') else None
    if step is not None and step['status'] != 0:
        raise RuntimeError('device status word reports a bounded-wait timeout')

    if rank == 0:
        common = {'higher_is_better': True, 'vs_baseline': None, 'n_gpus': world, 'steps': args.steps,
                  'warmup': max(args.warmup, 3), 'dtype': 'nvfp4 (e2m1 x ue4m3, fp32 accumulate)', 'data': 'synthetic'}
        if step is not None:
            line = {'metric': METRIC_STEP, 'value': step['issued'] / 1e12 / (step['ms'] * 1e-3), 'unit': 'TFLOP/s', **common,
                    'ms_per_step': step['ms'], 'scaling': 'strong', 'config': step_config(args, world),
                    'denoise_step_ms': step['ms'], 'issued_tflop_per_step': step['issued'] / 1e12,
                    'ledger_ratio': step['ledger_ratio'], 'collectives': step['collectives'],
                    'e2e': {'value': step['issued'] / 1e12 / (step['ms_e2e'] * 1e-3), 'unit': 'TFLOP/s',
                            'h2d_bytes_per_step': step['h2d'], 'd2h_bytes_per_step': step['d2h'],
                            'ms_per_step': step['ms_e2e'], 'bytes_are': 'per rank'},
                    'gpu_launches': args.steps * step['calls_per_step'],
                    'gpu_launches_are': 'C-ABI kernel calls per rank captured in the step graph x steps (each call launches >= 1 kernel)',
                    'clocks': step['clocks'], 'sustained': step['sustained']}
            if proj is not None:
                line['roofline'] = proj['roofline']
                line['parity'] = proj['parity']
                line['projection_set'] = {'value': proj['value'], 'unit': 'TFLOP/s', 'ms_per_step': proj['ms_per_step'],
                                          'replicas': world, 'config': workload_config(args.budget, world, args.m_tokens, args.layers),
                                          'e2e': {'value': proj['e2e_value'], 'ms_per_step': proj['e2e_ms_per_step'],
                                                  'h2d_bytes_per_step': proj['h2d'], 'd2h_bytes_per_step': proj['d2h']},
                                          'clocks': proj['clocks']}
        else:
            line = {'metric': METRIC_PROJ, 'value': proj['value'], 'unit': 'TFLOP/s', **common,
                    'ms_per_step': proj['ms_per_step'], 'scaling': 'weak',
                    'config': workload_config(args.budget, world, args.m_tokens, args.layers),
                    'e2e': {'value': proj['e2e_value'], 'unit': 'TFLOP/s', 'h2d_bytes_per_step': proj['h2d'],
                            'd2h_bytes_per_step': proj['d2h'], 'ms_per_step': proj['e2e_ms_per_step']},
                    'gpu_launches': args.steps * proj['launches_per_step'], 'clocks': proj['clocks'],
                    'roofline': proj['roofline'], 'parity': proj['parity']}
        if world == 1 and not args.no_cpu_baseline:
            shape = ('qkv', 3 * 4096, 4096) if step is not None else None
            v, dt, sample = cpu_baseline(args.budget, host_threads(), 1536, shape)
            line['cpu_baseline'] = {'value': v, 'unit': 'TFLOP/s', 'cores': host_threads(), 'kind': 'port',
                                    'sample': sample, 'seconds': dt}
        print(json.dumps(line), flush=True)
    if world > 1:
        # NCCL teardown after graph capture has blocked before: leave once every rank is done
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == '__main__':
    main()
