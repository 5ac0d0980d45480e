"""Step engine: the controller the repaired modules talk to, the (branch, phase) repair schedule, the
issued-work ledger and whole-step CUDA Graph capture / replay.

Graph-capture contract of the reference's JointEngine (packages/fp4-repair/src/thunderworld_fp4/
cosmos/engine.py): step and CFG branch are host counters (`divmod(call, branches)`, :316); phases follow
`settings.phase`; one graph per (branch, schedule, argument signature) is captured after eager warm-up
passes on cloned static arguments (:321-345) and replayed with `copy_tree` in / `clone_tree` out
(:351-353); an operator that was not warmed raises (:165, :350); with a budget plan the observed rows are
compiled into the request ledger and the budget is proved before capture (:247-305). The diffusers
module swap and attention-processor hook of the reference have no counterpart: models built from
`RepairLinear` call `engine.attend` directly.
"""
import torch
from .. import ops
from ..config import RepairConfig
from ..runtime import _forward as attention_forward
from . import trees
from .budget import PHASES, attention_cost, compile_request, linear_cost
from .settings import RunConfig, phase as phase_of


class StepEngine:
    def __init__(self, config=None, plan=None, task='t2v', topo=None, steps=35, branches=2):
        self.config = config or RunConfig()
        self.budget_plan = plan
        self.task, self.steps, self.branches = task, steps, branches
        self.topo = topo
        self.warming = False
        self.call = 0
        self.model = None
        self.graphs = {}
        self.pool = None
        self.rows = {}                 # (kind, name, branch, phase) -> ledger row
        self.linears = {}              # name -> (split, tile_map, tp)
        self.attention_layers = set()
        self._quotas = {}
        self._branch_offset = 0        # CFG-parallel ranks run one fixed branch

    # ---- controller protocol used by RepairLinear -------------------------------------------------
    def register_linear(self, name, split, tile_map, tp):
        self.linears[name] = (split, tile_map, tp)

    @property
    def position(self):
        step, branch = divmod(self.call, self.branches)
        return step, branch + self._branch_offset, phase_of(step, self.steps)

    def linear_spec(self, name, default):
        if self.budget_plan is None:
            return self.config.ffn if ('.up' in name or '.down' in name) else self.config.projection
        _, branch, ph = self.position
        spec = self.budget_plan.linear(self.task, branch, ph, name)
        split, tile_map, tp = self.linears.get(name, ('none', None, 1))
        if tile_map is None:
            return spec
        blocks = spec.activation_blocks
        if split == 'row':             # K blocks are divided: the A quota is divided with them (per-shard selection)
            blocks = -(-blocks // tp)
        from .settings import LinearSpec
        support = tuple(tile_map(spec.weight_support))
        cross = spec.cross and bool(blocks) and bool(support)
        return LinearSpec(0, 0, cross, activation_blocks=blocks, weight_support=support)

    def record_linear(self, name, shape, n, spec, op):
        _, branch, ph = self.position
        m, k = int(shape[0]), int(shape[1])
        row = linear_cost(m, n, k, a_blocks=op.na, w_blocks=op.weight_ids, cross=bool(op.cross))
        self.rows[('linear', name, branch, ph)] = {**row, 'name': name, 'branch': branch, 'phase': ph}

    # ---- attention -------------------------------------------------------------------------------
    def attention_config(self, layer):
        step, branch, ph = self.position
        default = self.config.attention.resolve(layer=layer, step=step, branch=str(branch)) \
            if self.config.attention.rules else self.config.attention.default
        if self.budget_plan is not None and self.budget_plan.attention:
            return self.budget_plan.attention_config(self.task, branch, ph, layer, default)
        return default

    def attend(self, layer, q, k, v):
        cfg = self.attention_config(layer)
        h, n, m = q.shape[2], k.shape[1], q.shape[1]
        key = (cfg, h, n, q.device)
        if key not in self._quotas:
            if not self.warming:
                raise RuntimeError(f'Unwarmed attention layer {layer}: {(m, n, h)}')
            self._quotas[key] = (torch.tensor(cfg.head_counts(h, n), device=q.device, dtype=torch.int32),
                                 torch.tensor(cfg.pv_counts(h, n), device=q.device, dtype=torch.int32))
        if self.warming:
            _, branch, ph = self.position
            row = attention_cost(m, n, h, k.shape[2], bm=128, qk_counts=cfg.head_counts(h, n), pv_counts=cfg.pv_counts(h, n),
                                 qk_terms=cfg.terms, pv_terms=cfg.pv_terms or cfg.terms)
            self.rows[('attention', str(layer), branch, ph)] = {**row, 'name': str(layer), 'branch': branch, 'phase': ph}
            self.attention_layers.add(str(layer))
        out, _, held = attention_forward(q, k, v, cfg, None, self._quotas[key], False)
        return out

    # ---- schedule, ledger, graphs ----------------------------------------------------------------
    def schedule_key(self):
        """What distinguishes the work of this call: CFG branch and, under a plan, the denoise phase."""
        _, branch, ph = self.position
        return (branch, ph if self.budget_plan is not None or self.config.attention.rules else 0)

    def reset_request(self):
        self.call = 0

    def compile_budget(self):
        """Prove total <= budget * base over the whole request from the rows observed while warming.
        Rows exist for the (branch, phase) pairs that were run; missing pairs fail closed."""
        if self.config.compute_budget is None:
            raise ValueError('no compute budget configured')
        modules = sorted({name for kind, name, _, _ in self.rows if kind == 'linear'})
        layers = sorted({name for kind, name, _, _ in self.rows if kind == 'attention'})
        # a CFG-parallel rank runs one fixed branch of the plan: its ledger counts that branch as its only one
        rows = [{**row, 'branch': row['branch'] - self._branch_offset} for row in self.rows.values()]
        return compile_request(rows, self.config.compute_budget, steps=self.steps,
                               branches=self.branches, expected_modules=modules, expected_layers=layers)

    def warm_schedule(self, model, **kwargs):
        """Discovery pass: run one eager call per distinct (branch, phase) so that every operator and
        ledger row exists before any graph is captured."""
        saved = self.call
        self.warming = True
        try:
            seen = set()
            for step in range(self.steps):
                for branch in range(self.branches):
                    self.call = step * self.branches + branch
                    key = self.schedule_key()
                    if key not in seen:
                        seen.add(key)
                        model(**kwargs)
        finally:
            self.warming = False
            self.call = saved
        return seen

    def __call__(self, model, **kwargs):
        """One denoiser call of the request: replay (capturing first if needed) and advance the counters."""
        if self.config.execution == 'eager':
            out = model(**kwargs)
            self.call += 1
            return out
        key = (id(model), self.schedule_key(), trees.signature(kwargs), torch.cuda.current_stream().cuda_stream)
        if key not in self.graphs:
            static = trees.clone_tree(kwargs)
            self.warming = True
            try:
                for _ in range(2):
                    model(**static)
            finally:
                self.warming = False
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            if self.pool is None:
                self.pool = torch.cuda.graph_pool_handle()
            with torch.cuda.graph(graph, pool=self.pool):
                output = model(**static)
            self.graphs[key] = (graph, static, output)
        graph, static, output = self.graphs[key]
        trees.copy_tree(static, kwargs)
        graph.replay()
        self.call += 1
        return trees.clone_tree(output)

    def device_status(self):
        return ops.device_status()
