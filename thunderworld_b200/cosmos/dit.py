"""A DiT denoiser built from the repaired operators, for the step-level configurations: RMSNorm ->
AdaLN modulation -> QKV (repaired linear) -> per-head RMSNorm -> FP4 attention -> out-proj -> gated
residual -> RMSNorm -> AdaLN -> FFN-up (GELU) -> FFN-down -> gated residual.

The reference runs the diffusers Cosmos3 transformer (absent here); its per-layer dataflow is the one
spelled out in thunderworld_fp4/cosmos/ar_cache.py:72-107. Every projection is a `RepairLinear`, attention
goes through the engine's `attend`; norms, modulation, GELU and the gated residuals are the fused
pointwise producers of `ops` (one pass each, the tensor factor of the next quantizer reduced in the same
pass, as the reference does with activate_with_factor / pack_with_factor, thunderworld_fp4/_fusion.py:26-42).

Tensor parallelism: QKV and FFN-up are column-split (heads shard with them, attention needs no
exchange); out-proj and FFN-down are row-split, their activations are quantized under the global
factor (4-byte MAX all-reduce) and their partial outputs summed with one all-reduce each.
"""
from dataclasses import dataclass
import torch
from .. import ops, parallel
from .linears import RepairLinear
from .settings import LinearSpec


@dataclass(frozen=True)
class DiTConfig:
    hidden: int = 4096
    heads: int = 32
    ffn: int = 16384
    blocks: int = 28
    head_dim: int = 128
    qk_norm: bool = True
    rope: bool = True
    seed: int = 0

    def __post_init__(self):
        if self.heads * self.head_dim != self.hidden or self.head_dim != 128:
            raise ValueError('hidden must equal heads * 128')
        if self.hidden % 128 or self.ffn % 128:
            raise ValueError('hidden and ffn must be multiples of 128')


NANO = DiTConfig(4096, 32, 16384, 28)      # Cosmos3-Nano-shaped step: 28 blocks, hidden 4096, 32 heads, FFN 16384
SUPER = DiTConfig(6144, 48, 24576, 48)     # Cosmos3-Super-shaped step: 48 blocks, hidden 6144, 48 heads, FFN 24576


class _Source:
    """Minimal stand-in for nn.Linear handed to RepairLinear."""

    def __init__(self, weight):
        self.weight, self.bias = weight, None
        self.out_features, self.in_features = weight.shape


def rope_tables(tokens, device, head_dim=128, theta=10000.0):
    """cos / sin tables [tokens, head_dim] (float32) of a rotary position embedding over the token index; the two
    halves of a head row rotate together (rotate-half convention of thunderworld_fp4/cosmos/pipeline_tuning.py:42-55)."""
    inv = theta ** (-torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim)
    ang = torch.arange(tokens, dtype=torch.float32)[:, None] * inv[None, :]
    ang = torch.cat([ang, ang], -1)
    return ang.cos().contiguous().to(device), ang.sin().contiguous().to(device)


def apply_rope(x, cos, sin):
    """Plain torch rotate-half RoPE in the dtype of x (reference arithmetic for tests)."""
    d = x.shape[-1]
    rot = torch.cat([-x[..., d // 2:], x[..., :d // 2]], -1)
    return x * cos[:, None, :].to(x.dtype) + rot * sin[:, None, :].to(x.dtype)


def rms_norm(x, eps=1e-6):
    """Plain torch RMSNorm (reference arithmetic for tests; the model runs ops.rms_norm)."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)).to(x.dtype)


class DiTBlock(torch.nn.Module):
    def __init__(self, cfg, index, controller, topo, device):
        super().__init__()
        self.cfg, self.index, self.controller, self.topo = cfg, index, controller, topo
        tp, r = topo.tp_size, topo.tp_rank
        gen = torch.Generator(device='cpu').manual_seed(cfg.seed * 100003 + index)
        make = lambda n, k: (torch.randn(n, k, generator=gen) * 0.02).bfloat16().to(device)
        h, f = cfg.hidden, cfg.ffn
        nb_h, kb_h, nb_f = h // 128, h // 128, f // 128
        self.local_heads = cfg.heads // tp
        full = {'qkv': make(3 * h, h), 'out': make(h, h), 'up': make(f, h), 'down': make(h, f)}
        shards = {'qkv': parallel.shard_qkv(full['qkv'], cfg.heads, tp, r), 'out': parallel.shard_rows(full['out'], tp, r),
                  'up': parallel.shard_columns(full['up'], tp, r), 'down': parallel.shard_rows(full['down'], tp, r)}
        lattice = {'qkv': (3 * nb_h, kb_h, 'qkv'), 'out': (nb_h, kb_h, 'row'), 'up': (nb_f, kb_h, 'column'),
                   'down': (nb_h, nb_f, 'row')}
        self.split = {}
        for part, w in shards.items():
            name = f'blocks.{index}.{part}'
            nb, kb, split = lattice[part]
            tile_map = self._tile_map(nb, kb, split, tp, r, cfg.heads)
            controller.register_linear(name, split, tile_map, tp)
            self.split[part] = split
            # column-split shards rank A1 blocks with the column energy of the whole weight: the same support on
            # every rank, and the one the unsharded layer selects
            energy = full[part].float().square().sum(0) if split in ('column', 'qkv') and tp > 1 else None
            setattr(self, part, RepairLinear(_Source(w.contiguous()), controller, name, LinearSpec(), tile_map=tile_map,
                                             sensitivity=energy))
        del full, shards

    @staticmethod
    def _tile_map(nb, kb, split, tp, r, heads):
        if tp == 1:
            return None
        if split == 'qkv':          # N blocks = [q heads | k heads | v heads], one block per head
            per = heads // tp

            def qkv_map(ids):
                out = []
                for t in ids:
                    b, k = divmod(t, kb)
                    which, head = divmod(b, heads)
                    if r * per <= head < (r + 1) * per:
                        out.append((which * per + head - r * per) * kb + k)
                return sorted(out)
            return qkv_map
        return lambda ids: parallel.remap_tiles(ids, nb, kb, tp, r, split)

    def controller_tables(self, tokens, device):
        """Rotary tables of this sequence length, built once (before graph capture, in the warm-up pass)."""
        cache = self.__dict__.setdefault('_rope', {})
        if (tokens, device) not in cache:
            cache[(tokens, device)] = rope_tables(tokens, device)
        return cache[(tokens, device)]

    def _row_split(self, layer, x, stats=None):
        """Row-split linear: global activation factor, local GEMM, summed partial outputs.
        stats = (factor, max|x|) of the local shard when its producer reduced them."""
        if self.topo.tp_size == 1:
            return layer(x) if stats is None else layer(x, factor=stats[0])
        if stats is None:
            factor = parallel.global_factor(x, self.topo)
        else:
            factor = parallel.global_factor_from_peak(stats[1:2].clone(), self.topo)
        return parallel.allreduce_sum(layer(x, factor=factor), self.topo)

    def _gathered_input(self, layer, x_rows, stats, rows, tokens):
        """Row-sharded producer -> column-split layer: global factor from the shards' maxima, local quantization,
        all-gather of the packed bytes. Returns the Packed activation of all tokens."""
        layer.prepare(tokens)
        factor = parallel.global_factor_from_peak(stats[1:2].clone(), self.topo)
        return layer.pack_shard(x_rows, factor, rows, tokens, self.topo)

    def _row_split_scatter(self, layer, x, rows_padded, stats=None):
        """Row-split linear whose partial sums are reduce-scattered over token rows: returns this rank's summed rows
        [rows_padded / tp, hidden]."""
        if stats is None:
            factor = parallel.global_factor(x, self.topo)
        else:
            factor = parallel.global_factor_from_peak(stats[1:2].clone(), self.topo)
        y = layer(x, factor=factor)                              # [tokens, hidden] partial sums
        if rows_padded != y.shape[0]:
            padded = torch.zeros((rows_padded, y.shape[1]), device=y.device, dtype=y.dtype)
            padded[:y.shape[0]] = y
            y = padded
        return parallel.reduce_scatter_rows(y, self.topo)

    def forward_rows(self, x_rows, mod, tokens):
        """Sequence-parallel form of forward() for one batch entry under tensor parallelism: `x_rows`
        [rows, hidden] is this rank's share of the residual stream (rows = padded tokens / tp, whole M128 blocks;
        rows past the end of the sequence are padding), updated in place. Pointwise producers and the quantizer run
        on the shard; packed bytes are all-gathered in front of the column-split layers and the partial sums of the
        row-split layers are reduce-scattered. Same bits as forward() on the all-reduce path."""
        rows, h = x_rows.shape
        _, first, valid = parallel.shard_rows_of(tokens, self.topo)
        rows_padded = rows * self.topo.tp_size
        shift1, scale1, gate1, shift2, scale2, gate2 = mod.unbind(0)
        live = x_rows[:valid].unsqueeze(0)                       # [1, valid, hidden] view: padding rows never enter a maximum
        y, stats = ops.rms_norm(live, shift=shift1, scale=scale1, want_factor=True, return_stats=True)
        packed = self._gathered_input(self.qkv, y[0], stats, rows, tokens)
        qkv = self.qkv.run_rows(tokens, packed).reshape(1, tokens, 3, self.local_heads, 128)
        q, k, v = qkv.unbind(2)
        if self.cfg.rope:
            cos, sin = self.controller_tables(tokens, x_rows.device)
            q = ops.rope_heads(q, cos, sin, norm=self.cfg.qk_norm)
            k = ops.rope_heads(k, cos, sin, norm=self.cfg.qk_norm)
        elif self.cfg.qk_norm:
            q, k = ops.rms_norm_heads(q), ops.rms_norm_heads(k)
        a = self.controller.attend(self.index, q, k, v).reshape(tokens, self.local_heads * 128)
        part = self._row_split_scatter(self.out, a, rows_padded)
        ops.gate_residual_(x_rows.unsqueeze(0), gate1, part.unsqueeze(0))
        y, stats = ops.rms_norm(live, shift=shift2, scale=scale2, want_factor=True, return_stats=True)
        packed = self._gathered_input(self.up, y[0], stats, rows, tokens)
        u, ustats = self.up.run_rows(tokens, packed, activation='gelu_tanh')
        part = self._row_split_scatter(self.down, u, rows_padded, ustats)
        ops.gate_residual_(x_rows.unsqueeze(0), gate2, part.unsqueeze(0))
        return x_rows

    def forward(self, x, mod):
        """x bf16 [batch, tokens, hidden], updated in place; mod [6, batch, hidden] contiguous."""
        b, s, h = x.shape
        shift1, scale1, gate1, shift2, scale2, gate2 = mod.unbind(0)
        y, f = ops.rms_norm(x, shift=shift1, scale=scale1, want_factor=True)
        qkv = self.qkv(y, factor=f).reshape(b, s, 3, self.local_heads, 128)
        q, k, v = qkv.unbind(2)
        if self.cfg.rope:
            # q/k head norm and rotary embedding in one pass over q and one over k (the reference's dataflow:
            # q/k norm -> RoPE -> attention, thunderworld_fp4/cosmos/ar_cache.py:72-107)
            cos, sin = self.controller_tables(s, x.device)
            q = ops.rope_heads(q, cos, sin, norm=self.cfg.qk_norm)
            k = ops.rope_heads(k, cos, sin, norm=self.cfg.qk_norm)
        elif self.cfg.qk_norm:
            q, k = ops.rms_norm_heads(q), ops.rms_norm_heads(k)
        a = self.controller.attend(self.index, q, k, v).reshape(b, s, self.local_heads * 128)
        ops.gate_residual_(x, gate1, self._row_split(self.out, a))
        y, f = ops.rms_norm(x, shift=shift2, scale=scale2, want_factor=True)
        u, stats = self.up(y, factor=f, activation='gelu_tanh')      # GELU and max|u| come out of the GEMM epilogue
        return ops.gate_residual_(x, gate2, self._row_split(self.down, u, stats))


class DiTModel(torch.nn.Module):
    def __init__(self, cfg, controller, topo=None, device='cuda'):
        super().__init__()
        self.cfg = cfg
        self.topo = topo or parallel.Topology()
        # tensor-parallel runs of one batch entry may keep the residual stream row-sharded (forward_rows); off by
        # default: with two shards the extra collectives cost more than the halved pointwise work saves
        self.row_sharded = False
        self.blocks = torch.nn.ModuleList(DiTBlock(cfg, i, controller, self.topo, device) for i in range(cfg.blocks))

    def forward(self, x, mod):
        """x bf16 [batch, tokens, hidden]; mod bf16 [batch, blocks, 6, hidden] (AdaLN shift/scale/gate)."""
        mods = mod.permute(1, 2, 0, 3).contiguous()           # [blocks, 6, batch, hidden]
        topo = self.topo
        if topo.tp_size > 1 and x.shape[0] == 1 and self.row_sharded:
            # the residual stream lives row-sharded between the projections (see DiTBlock.forward_rows)
            tokens, hidden = x.shape[1], x.shape[2]
            rows, first, valid = parallel.shard_rows_of(tokens, topo)
            mine = torch.zeros((rows, hidden), device=x.device, dtype=x.dtype)
            mine[:valid] = x[0, first:first + valid]
            for i, block in enumerate(self.blocks):
                block.forward_rows(mine, mods[i], tokens)
            mine = ops.rms_norm(mine.unsqueeze(0))[0]
            full = torch.empty((rows * topo.tp_size, hidden), device=x.device, dtype=x.dtype)
            parallel.all_gather_rows([(full, mine)], topo)
            return full[:tokens].unsqueeze(0)
        x = x.clone()                                         # blocks update the residual stream in place
        for i, block in enumerate(self.blocks):
            x = block(x, mods[i])
        return ops.rms_norm(x)
