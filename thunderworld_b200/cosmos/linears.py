"""`RepairLinear`: the module that replaces every generation `nn.Linear` in the joint-inference runtime
(reference: packages/fp4-repair/src/thunderworld_fp4/cosmos/linears.py:55-265). It owns the offline asset
(W0/W1 planes, factor, prescale, tile scores, selector weights), builds one operator per
(rows, repair spec) while the controller is warming, shares W0 between them and keeps the W1 tiles of a
budget plan in one union bank addressed through `wloc`. The launch-table search of the reference has no
counterpart: there is one sm_100a kernel configuration per shape.

Controller protocol (duck-typed, as in the reference): `linear_spec(name, default) -> LinearSpec`,
`warming: bool`, `record_linear(name, shape, n, spec, op)`, optional `budget_plan` (RepairPlan) and
`config` (RunConfig: activation_repair_energy).
"""
import json
import torch
from .. import ops
from ..linear import sampled_block_rank
from ..native import Native, quantize_weight
from .assets import compact, expand


class RepairLinear(torch.nn.Module):
    def __init__(self, source, controller, name, spec, asset=None, tile_map=None, sensitivity=None):
        super().__init__()
        # sensitivity: selector weights [K] to use instead of the column energy of `source` (a column-split shard
        # passes the energy of the whole weight, so that every rank selects what the unsharded layer selects)
        # tile_map: plan tile ids of the full layer -> ids of this (tensor-parallel) shard's lattice
        self.tile_map = tile_map
        self.in_features, self.out_features = source.in_features, source.out_features
        self.controller, self.name, self.default = controller, name, spec
        self.repair_energy = getattr(getattr(controller, 'config', None), 'activation_repair_energy', 1.)
        n, k = self.out_features, self.in_features
        if n % 128 or k % 128:
            raise ValueError(f'Unsupported FP4 projection {name}: {n}x{k}')
        plan = getattr(controller, 'budget_plan', None)
        if asset is None:
            w = source.weight.detach().cuda().bfloat16().contiguous()
            codes, scales, factor = quantize_weight(w)
            # residual magnitude per tile: deterministic offline fallback score for W1 selection
            score = scales[1].float().reshape(n // 128, 128, k // 128, 8).square().sum((1, 3))
            asset = dict(codes=codes.cpu(), scales=scales.cpu(), factor=factor.cpu(), prescale=torch.ones(k),
                         identity_prescale=True, score=score.cpu(), bias=None if source.bias is None else source.bias.detach().cpu())
            if plan is not None:
                asset.update(selector='residual_sensitivity', activation_sensitivity=(
                    w.float().square().sum(0) if sensitivity is None else sensitivity.float()).cpu())
        # with a plan only the union of W1 tiles any phase/branch selects is kept
        self.weight_union = None
        if plan is not None:
            self.weight_union = self._plan_union(plan)
            self.asset = compact(asset, self.weight_union)
        else:
            self.asset = asset
        self.register_buffer('bias', None if asset['bias'] is None else asset['bias'].cuda().bfloat16())
        self.register_buffer('sensitivity', asset.get('activation_sensitivity', torch.ones(k)).float().cuda())
        self.ops, self.bound, self.weight_bank = {}, None, None

    def _plan_union(self, plan):
        ids = set()
        for key, row in plan.linears.items():
            if key.split('|', 2)[-1] == self.name:
                ids.update(self.tile_map(row['w_blocks']) if self.tile_map else row['w_blocks'])
        return sorted(ids)

    def export(self):
        return expand(self.asset, self.weight_union) if self.weight_union is not None else self.asset

    def prepare_shape(self, m, spec):
        """Build (or fetch) the operator for `m` rows under `spec`. Host work only; called while warming."""
        key = (m, spec.key)
        if key in self.ops:
            self.bound = self.ops[key]
            return
        n, k = self.out_features, self.in_features
        mb, kb, nb = ops.cdiv(m, 128), k // 128, n // 128
        a = self.export()
        c, s, g, d = (a[x].cuda() for x in ('codes', 'scales', 'factor', 'prescale'))
        na, nw = spec.counts(n, k)
        if self.repair_energy != 1 and 0 < na < kb and a.get('selector') != 'residual_sensitivity':
            raise ValueError('Adaptive A repair requires an offline residual-sensitivity asset')
        scores = a['score'].flatten()
        if spec.weight_support is None:
            ids = torch.argsort(scores, descending=True, stable=True)[:nw]
        else:
            ids = torch.tensor(spec.weight_support, dtype=torch.long)
        if not set(a.get('mandatory_w_blocks', ())).issubset(ids.tolist()):
            raise ValueError('Policy disables mandatory outlier W1 support')
        selected = torch.zeros(nb * kb, dtype=torch.bool)
        selected[ids] = True
        wm = selected.reshape(nb, kb).repeat_interleave(128, 0).repeat_interleave(128, 1).cuda()
        am = torch.ones((mb, k), device='cuda', dtype=torch.bool)
        op = Native(c, s, g, d.float(), am, wm, bm=128, interleave=True, cross=spec.cross)
        # W0 (and its atom-layout scales) is shared by every (m, A, cross) variant; W1 by equal W support
        for (_, old_key), previous in self.ops.items():
            for name in ('wc', 'ws', 'wg', 'd', 'ws_swz'):
                setattr(op, name, getattr(previous, name))
            old = json.loads(old_key)
            same_support = old.get('weight_support') == (list(spec.weight_support) if spec.weight_support is not None else None)
            if old['weight'] == spec.weight and same_support:
                for name in ('wr', 'wrs', 'wi', 'off', 'wrs_swz', '_bank_key'):
                    setattr(op, name, getattr(previous, name))
            break
        plan = getattr(self.controller, 'budget_plan', None)
        if plan is not None:
            if self.weight_bank is None:
                union = self._plan_union(plan)
                union_ids = torch.tensor(union, device=c.device, dtype=torch.long)
                tiles_c = c[1].reshape(nb, 128, kb, 64).permute(0, 2, 1, 3).reshape(-1, 128, 64)
                tiles_s = s[1].view(torch.uint8).reshape(nb, 128, kb, 8).permute(0, 2, 1, 3).reshape(-1, 128, 8)
                self.weight_bank = (tiles_c[union_ids].contiguous(),
                                    tiles_s[union_ids].contiguous().view(torch.float8_e4m3fn),
                                    {v: i for i, v in enumerate(union)})
            op.wr, op.wrs, positions = self.weight_bank
            op.wloc = torch.tensor([positions[i] for i in sorted(ids.tolist())], device=c.device, dtype=torch.int32)
            op.shared_bank = not op.dense_w
            op.hasw = bool(len(ids))
        op.na = na
        op.weight_ids = tuple(ids.tolist())
        op.am = op.union = torch.full((mb, kb), na == kb, device='cuda', dtype=torch.bool)
        self.ops[key] = op
        self.bound = op

    def _pack(self, x, factor=None, mask=None, out=None):
        """Quantize x [rows, k] for the bound operator. The A1 support of a partial repair is written into `mask`
        (default: the operator's own [ceil(rows/128), k/128]); `out`: preallocated planes (ops.Packed)."""
        op = self.bound
        m, k = x.shape
        kb = k // 128
        mask = op.am if mask is None else mask
        base, res = self.asset.get('activation_scale', (1., 1.))
        identity = bool(self.asset.get('identity_prescale', False))
        common = dict(wg=op.wg, base=base, res=res, out=out)
        d = None if identity else op.d               # an identity prescale is bf16(x * 1) = x: skip the multiply
        if self.asset.get('selector') == 'residual_sensitivity' and 0 < op.na < kb:
            # online current-residual selection: mask written in place, then read by the GEMM
            return ops.quantize(x, d, repair=3, na=op.na, sensitivity=self.sensitivity, mask=mask,
                                factor=factor if identity else None, energy=self.repair_energy, **common)
        if 0 < op.na < kb:                           # sampled-energy selector of assets without sensitivities
            mask.copy_(sampled_block_rank(x, op.d, m, k) < op.na)
        mode = 0 if op.na == 0 else (1 if op.na == kb else 2)
        use_factor = factor if (base, res) == (1., 1.) else None
        return ops.quantize(x, d, repair=mode, mask=mask if mode == 2 else None, factor=use_factor, **common)

    def _compute(self, x, factor=None, packed=None, activation=None, out=None):
        if packed is None:
            packed = self._pack(x, factor)
        # the bias is added in fp32 before the single bf16 rounding of the epilogue (TwRepairIO.bias)
        return self.bound.run_packed(x, packed, out=out, bias=self.bias, activation=activation, want_stats=activation is not None)

    def pack_shard(self, x_rows, factor, rows, total_rows, topo):
        """Row-sharded input of a column-split layer: quantize this rank's `x_rows` [valid, k] (valid <= rows, the
        shard's padded height, a multiple of 128) with the tensor-wide `factor`, then all-gather the packed planes,
        the atom-layout scales and the A1 support of every shard. Returns the Packed of all `total_rows` rows; the
        operator's own support (`bound.am`) is overwritten with the gathered one. Called after `prepare`."""
        op = self.bound
        k = self.in_features
        kb = k // 128
        if not self.asset.get('identity_prescale', False) or self.asset.get('activation_scale', (1., 1.)) != (1., 1.):
            raise ValueError('row-sharded packing needs the tensor factor from the producer: identity prescale only')
        dev = self.sensitivity.device
        planes = 1 if op.na == 0 else 2
        tp = topo.tp_size
        local = ops.Packed(torch.empty((planes, rows, k // 2), device=dev, dtype=torch.uint8),
                           torch.empty((planes, rows, k // 16), device=dev, dtype=torch.float8_e4m3fn), factor, rows,
                           torch.empty((planes, rows, k // 16), device=dev, dtype=torch.uint8),
                           torch.empty((), device=dev, dtype=torch.float32), None)
        partial = 0 < op.na < kb
        local_mask = torch.zeros((rows // 128, kb), device=dev, dtype=torch.bool) if partial else None
        valid = x_rows.shape[0]
        if valid:
            self._pack(x_rows, factor, mask=None if local_mask is None else local_mask[:ops.cdiv(valid, 128)], out=local)
        full = ops.Packed(torch.empty((planes, rows * tp, k // 2), device=dev, dtype=torch.uint8),
                          torch.empty((planes, rows * tp, k // 16), device=dev, dtype=torch.float8_e4m3fn), factor, rows * tp,
                          torch.empty((planes, rows * tp, k // 16), device=dev, dtype=torch.uint8), local.alpha, None)
        pieces = []
        for plane in range(planes):
            pieces += [(full.codes[plane], local.codes[plane]), (full.scales[plane], local.scales[plane]),
                       (full.scales_swz[plane], local.scales_swz[plane])]
        if partial:
            gathered = torch.empty((rows * tp // 128, kb), device=dev, dtype=torch.bool)
            pieces.append((gathered, local_mask))
        from .. import parallel
        parallel.all_gather_rows(pieces, topo)
        if partial:
            op.am.copy_(gathered[:op.am.shape[0]])
        return full

    def prepare(self, rows):
        """Controller bookkeeping of forward() for `rows` input rows without running anything: binds (while warming:
        builds and records) the operator of the current repair spec."""
        c = self.controller
        spec = c.linear_spec(self.name, self.default)
        key = (rows, spec.key)
        if c.warming:
            self.prepare_shape(rows, spec)
            c.record_linear(self.name, (rows, self.in_features), self.out_features, spec, self.bound)
        elif key not in self.ops:
            raise RuntimeError(f'Unwarmed projection {self.name}: {key}')
        else:
            self.bound = self.ops[key]

    def run_rows(self, rows, packed, activation=None):
        """GEMM of the bound operator on `rows` rows of an already packed (gathered) activation."""
        shape_only = torch.empty((rows, 0), device=packed.codes.device, dtype=torch.bfloat16)
        return self.bound.run_packed(shape_only, packed, bias=self.bias, activation=activation, want_stats=activation is not None)

    def forward(self, x, *, factor=None, packed=None, activation=None, out=None):
        """activation='gelu_tanh': the activation is applied in the GEMM epilogue and the call returns
        (y, stats) with stats = (max|y| / 2688, max|y|), as ops.activate_with_factor(..., return_stats=True) would."""
        shape = x.shape
        flat = x.reshape(-1, self.in_features).contiguous()
        self.prepare(len(flat))
        if activation is not None:
            y, stats = self._compute(flat, factor, packed, activation)
            return y.reshape(*shape[:-1], self.out_features), stats
        return self._compute(flat, factor, packed, out=out).reshape(*shape[:-1], self.out_features)
