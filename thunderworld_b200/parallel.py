"""Tensor-parallel and CFG-parallel plumbing over torch.distributed (NCCL on GPUs, gloo in CPU tests).

The reference has no sharded execution (its two-GPU mode places whole branches on different devices,
tools/contribution_study/super_runtime.py:74-102); this module is what the sharded projections need:

* column split (QKV, FFN-up): rows of W0/W1, i.e. N128 blocks, are divided; the activation and its
  packed planes are replicated, so every rank quantizes the same bytes;
* row split (out-proj, FFN-down): K128 blocks are divided; the tensor-wide activation factor must be the
  global one, so ranks exchange max|x| (4 bytes, MAX) before quantizing, and partial outputs are summed;
* W1 tile ids `nb*KB + kb` of a plan are remapped to the shard's own lattice;
* CFG split: ranks are arranged as [cfg][tp]; each CFG group runs one of the cond / uncond branches;
* row sharding of the residual stream between the projections (sequence parallelism): the partial sums of a
  row-split layer are reduce-scattered over token rows instead of all-reduced, every rank runs the pointwise
  producers and the quantizer on its rows only, and the packed bytes (0.56 B per element instead of 2) are
  all-gathered for the next column-split layer. Shards are whole M128 row blocks, so block-wise selection and
  the atom-layout scales of a shard are exactly the corresponding part of the unsharded result.
"""
from dataclasses import dataclass
import torch
import torch.distributed as dist


@dataclass
class Topology:
    """Rank layout of one node: world = cfg_size * tp_size, rank = cfg_rank * tp_size + tp_rank."""
    rank: int = 0
    world: int = 1
    tp_size: int = 1
    cfg_size: int = 1
    tp_group: object = None
    cfg_group: object = None

    @property
    def tp_rank(self):
        return self.rank % self.tp_size

    @property
    def cfg_rank(self):
        return self.rank // self.tp_size


def make_topology(tp_size=None, cfg_size=1):
    """Build TP and CFG sub-groups from the default process group (every rank must call this)."""
    if not dist.is_available() or not dist.is_initialized():
        return Topology()
    world, rank = dist.get_world_size(), dist.get_rank()
    tp_size = world // cfg_size if tp_size is None else tp_size
    if tp_size * cfg_size != world:
        raise ValueError(f'world size {world} != tp {tp_size} x cfg {cfg_size}')
    tp_group = cfg_group = None
    for c in range(cfg_size):
        ranks = list(range(c * tp_size, (c + 1) * tp_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            tp_group = g
    for t in range(tp_size):
        ranks = [c * tp_size + t for c in range(cfg_size)]
        g = dist.new_group(ranks)
        if rank in ranks:
            cfg_group = g
    return Topology(rank, world, tp_size, cfg_size, tp_group, cfg_group)


def block_range(blocks, parts, index):
    """Contiguous share [start, stop) of `blocks` lattice blocks for shard `index` of `parts`."""
    if blocks % parts:
        raise ValueError(f'{blocks} blocks do not divide over {parts} shards')
    per = blocks // parts
    return index * per, (index + 1) * per


def shard_columns(weight, parts, index):
    """Column split of a linear: rows (output features) of W [N, K], on N128 boundaries."""
    start, stop = block_range(weight.shape[0] // 128, parts, index)
    return weight[start * 128:stop * 128]


def shard_rows(weight, parts, index):
    """Row split of a linear: input features (K) of W [N, K], on K128 boundaries."""
    start, stop = block_range(weight.shape[1] // 128, parts, index)
    return weight[:, start * 128:stop * 128]


def shard_qkv(weight, heads, parts, index, head_dim=128):
    """Column split of a fused QKV weight [3*heads*head_dim, K] that keeps q, k and v of the shard's
    heads together: rows = [q heads of the shard | k heads | v heads]."""
    if heads % parts:
        raise ValueError('heads must divide over the tensor-parallel shards')
    per = heads // parts
    w = weight.reshape(3, heads, head_dim, weight.shape[1])
    return w[:, index * per:(index + 1) * per].reshape(3 * per * head_dim, weight.shape[1])


def remap_tiles(tile_ids, nb, kb, parts, index, split):
    """W1 tile ids of the full layer -> ids inside shard `index` (tiles of other shards dropped).
    split = 'column' (N blocks divided) or 'row' (K blocks divided)."""
    out = []
    if split == 'column':
        start, stop = block_range(nb, parts, index)
        for t in tile_ids:
            b, k = divmod(t, kb)
            if start <= b < stop:
                out.append((b - start) * kb + k)
    elif split == 'row':
        start, stop = block_range(kb, parts, index)
        width = stop - start
        for t in tile_ids:
            b, k = divmod(t, kb)
            if start <= k < stop:
                out.append(b * width + (k - start))
    else:
        raise ValueError('split must be column or row')
    return sorted(out)


def allreduce_sum(x, topo):
    if topo.tp_size > 1:
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=topo.tp_group)
    return x


_DIVISOR = {}


def factor_of_peak(peak):
    """max|x| -> max|x| / 2688 (1.0 for zero) with an IEEE division. The divisor is a tensor on purpose: torch
    turns division of a CUDA tensor by a Python number into a multiplication by the rounded reciprocal, which
    is off by one ulp for some peaks and would make a shard's packed bytes differ from the unsharded
    quantizer's (which divides)."""
    key = (peak.device, peak.dtype)
    if key not in _DIVISOR:
        _DIVISOR[key] = torch.full((1,), 2688., device=peak.device, dtype=peak.dtype)
    return torch.where(peak > 0, peak / _DIVISOR[key], torch.ones_like(peak)).reshape(())


def global_factor(x_local, topo):
    """Tensor-wide NVFP4 factor max|x| / 2688 (1.0 for an all-zero tensor) of an activation whose K
    dimension is divided over the tensor-parallel group: one 4-byte MAX all-reduce."""
    peak = x_local.abs().amax().float().reshape(1)
    if topo.tp_size > 1:
        dist.all_reduce(peak, op=dist.ReduceOp.MAX, group=topo.tp_group)
    return factor_of_peak(peak)


def global_factor_from_peak(peak, topo):
    """Same, starting from the shard's max|x| (1-element float32 tensor, overwritten) that the producer of x
    already reduced."""
    if topo.tp_size > 1:
        dist.all_reduce(peak, op=dist.ReduceOp.MAX, group=topo.tp_group)
    return factor_of_peak(peak)


def guide(branch_output, scale, topo):
    """Classifier-free guidance across the CFG split: CFG rank 0 holds the conditional output, rank 1 the
    unconditional one; every rank gets  uncond + scale * (cond - uncond)  after one all-gather of
    [tokens, hidden] over its CFG group (ranks of the same tensor-parallel index)."""
    if topo.cfg_size == 1:
        return branch_output
    if topo.cfg_size != 2:
        raise ValueError('guidance combines exactly two branches')
    both = [torch.empty_like(branch_output) for _ in range(2)]
    dist.all_gather(both, branch_output.contiguous(), group=topo.cfg_group)
    return both[1] + scale * (both[0] - both[1])


# ---- row sharding of the residual stream (sequence parallelism) -----------------------------------------------
def padded_rows(m, tp):
    """Rows of the token dimension rounded up so that every shard is a whole number of M128 blocks."""
    step = 128 * tp
    return -(-m // step) * step


def shard_rows_of(m, topo):
    """(rows per shard, first row, valid rows) of this rank's share of m token rows."""
    per = padded_rows(m, topo.tp_size) // topo.tp_size
    first = topo.tp_rank * per
    return per, first, max(0, min(per, m - first))


def _backend(group):
    return dist.get_backend(group) if dist.is_initialized() else None


def reduce_scatter_rows(partial, topo):
    """partial [padded rows, hidden] (this rank's partial sums, padding rows zero) -> this rank's summed rows
    [padded rows / tp, hidden]."""
    per = partial.shape[0] // topo.tp_size
    if _backend(topo.tp_group) == 'nccl':
        out = torch.empty((per, partial.shape[1]), device=partial.device, dtype=partial.dtype)
        dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM, group=topo.tp_group)
        return out
    total = partial.clone()                                   # backends without reduce-scatter (CPU tests)
    dist.all_reduce(total, op=dist.ReduceOp.SUM, group=topo.tp_group)
    return total[topo.tp_rank * per:(topo.tp_rank + 1) * per].contiguous()


def all_gather_rows(pieces, topo):
    """pieces: list of (full, local) tensor pairs; full = concatenation of every rank's `local` along dim 0.
    On NCCL all pieces travel in one grouped launch."""
    bytes_of = lambda t: t.view(torch.uint8) if t.dtype in (torch.bool, torch.float8_e4m3fn) else t
    pairs = [(bytes_of(f), bytes_of(l.contiguous())) for f, l in pieces]
    if _backend(topo.tp_group) == 'nccl':
        with dist._coalescing_manager(group=topo.tp_group, device=pairs[0][0].device, async_ops=False):
            for full, local in pairs:
                dist.all_gather_into_tensor(full, local, group=topo.tp_group)
    else:
        for full, local in pairs:
            parts = [torch.empty_like(local) for _ in range(topo.tp_size)]
            dist.all_gather(parts, local, group=topo.tp_group)
            full.copy_(torch.cat(parts, 0))
