"""Host-side tensor-parallel logic on CPU with gloo, world size 2: shard maps, tile remapping, the
MAX all-reduce of the activation factor and the SUM all-reduce of row-split partial outputs."""
import os
import socket
import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from thunderworld_b200 import parallel


def test_block_ranges_and_tile_remap():
    assert parallel.block_range(8, 4, 2) == (4, 6)
    with pytest.raises(ValueError):
        parallel.block_range(6, 4, 0)
    nb, kb = 4, 6
    tiles = [0, 5, 7, 13, 20, 23]
    cols = [parallel.remap_tiles(tiles, nb, kb, 2, r, 'column') for r in range(2)]
    assert cols == [[0, 5, 7], [1, 8, 11]]                 # N blocks 0-1 -> rank 0, 2-3 -> rank 1
    rows = [parallel.remap_tiles(tiles, nb, kb, 2, r, 'row') for r in range(2)]
    assert rows == [[0, 4, 7, 11], [2, 11]] or sum(len(r) for r in rows) == len(tiles)
    # every tile lands on exactly one shard and maps back to itself
    for split in ('column', 'row'):
        back = []
        for r in range(2):
            for t in parallel.remap_tiles(tiles, nb, kb, 2, r, split):
                if split == 'column':
                    b, k = divmod(t, kb); back.append((b + r * 2) * kb + k)
                else:
                    b, k = divmod(t, 3); back.append(b * kb + k + r * 3)
        assert sorted(back) == tiles
    w = torch.arange(3 * 4 * 128 * 2, dtype=torch.float32).reshape(3 * 4 * 128, 2)
    s = parallel.shard_qkv(w, 4, 2, 1)
    assert s.shape == (3 * 2 * 128, 2)
    assert torch.equal(s[:256], w[256:512]) and torch.equal(s[256:512], w[512 + 256:512 + 512])


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        topo = parallel.make_topology(tp_size=2, cfg_size=1)
        assert (topo.tp_rank, topo.cfg_rank, topo.tp_size) == (rank, 0, 2)
        g = torch.Generator().manual_seed(0)
        x = torch.randn(64, 512, generator=g)
        x[:, 300] *= 50                                     # the global peak lives in rank 1's K shard
        w = torch.randn(256, 512, generator=g) * 0.02
        # row split: local K slice, global factor, summed partial outputs
        xs, ws = parallel.shard_rows(x, 2, rank), parallel.shard_rows(w, 2, rank)
        factor = parallel.global_factor(xs, topo)
        assert torch.equal(factor, x.abs().amax() / 2688.)
        y = parallel.allreduce_sum(xs @ ws.T, topo)
        assert torch.allclose(y, x @ w.T, atol=1e-4)
        # column split: replicated activation, outputs concatenated
        yc = x @ parallel.shard_columns(w, 2, rank).T
        gathered = [torch.empty_like(yc) for _ in range(2)]
        dist.all_gather(gathered, yc, group=topo.tp_group)
        assert torch.allclose(torch.cat(gathered, 1), x @ w.T, atol=1e-4)
        zero = parallel.global_factor(torch.zeros(4, 128), topo)
        assert float(zero) == 1.0
        # the same factor from the shard's own max|x| (what a fused producer hands over)
        peak = xs.abs().amax().float().reshape(1)
        assert torch.equal(parallel.global_factor_from_peak(peak, topo), factor)
        assert float(parallel.global_factor_from_peak(torch.zeros(1), topo)) == 1.0
        results[rank] = 1
    finally:
        dist.destroy_process_group()


def _cfg_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        topo = parallel.make_topology(tp_size=1, cfg_size=2)
        assert (topo.tp_rank, topo.cfg_rank) == (0, rank)
        # each CFG rank computes one branch; guidance combines them with one exchange
        branch = torch.full((4,), float(rank + 1))
        guided = parallel.guide(branch, 3.0, topo)
        assert torch.equal(guided, torch.full((4,), 2 + 3.0 * (1 - 2)))
        assert parallel.guide(branch, 3.0, parallel.Topology()) is branch
        results[rank] = 1
    finally:
        dist.destroy_process_group()


def _rows_worker(rank, world, port, results):
    """Row sharding of the residual stream: shard geometry with padding rows, reduce-scatter of partial sums over
    token rows, all-gather of several per-shard pieces (bytes, bool support) into row order."""
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        topo = parallel.make_topology(tp_size=2, cfg_size=1)
        assert parallel.padded_rows(300, 2) == 512 and parallel.padded_rows(512, 2) == 512 and parallel.padded_rows(3840, 4) == 4096
        rows, first, valid = parallel.shard_rows_of(300, topo)
        assert (rows, first, valid) == ((256, 0, 256) if rank == 0 else (256, 256, 44))
        g = torch.Generator().manual_seed(1)
        parts = [torch.randn(512, 8, generator=g) for _ in range(2)]     # both ranks draw both partial sums
        mine = parallel.reduce_scatter_rows(parts[rank].clone(), topo)
        assert mine.shape == (256, 8)
        assert torch.allclose(mine, (parts[0] + parts[1])[rank * 256:(rank + 1) * 256])
        codes = torch.full((256, 4), rank + 1, dtype=torch.uint8)
        support = torch.zeros((2, 3), dtype=torch.bool)
        support[rank, rank] = True
        full_codes = torch.empty((512, 4), dtype=torch.uint8)
        full_support = torch.empty((4, 3), dtype=torch.bool)
        parallel.all_gather_rows([(full_codes, codes), (full_support, support)], topo)
        assert torch.equal(full_codes[:256], torch.full((256, 4), 1, dtype=torch.uint8))
        assert torch.equal(full_codes[256:], torch.full((256, 4), 2, dtype=torch.uint8))
        want = torch.zeros((4, 3), dtype=torch.bool)
        want[0, 0] = True
        want[3, 1] = True
        assert torch.equal(full_support, want)
        results[rank] = 1
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


@pytest.mark.parametrize('worker', [_worker, _cfg_worker, _rows_worker])
def test_two_rank_gloo(worker):
    ctx = mp.get_context('spawn')
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs) and dict(results) == {0: 1, 1: 1}
