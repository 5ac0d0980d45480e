"""GPU parity of the fused repair GEMM against the decoded fp32 emulation of the oracle.

Tolerance: relative L2 <= 1e-3 against the oracle's fp32-accumulated, bf16-rounded output (the
kernel accumulates the same products in fp32 in a different order and rounds to bf16 once).
The packed operands fed to the oracle are the GPU's own bytes, which test_gpu_quantize checks
bit for bit."""
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


def build(m, n, k, seed, a_fraction, w_fraction, cross=False):
    from thunderworld_b200.native import Native, quantize_weight
    x = torch.from_numpy(o.synthetic_activation(m, k, seed)).cuda().bfloat16()
    w = torch.from_numpy(o.synthetic_weight(n, k, seed)).cuda().bfloat16()
    wc, ws, wg = quantize_weight(w)
    mb, kb, nb = (m + 127) // 128, k // 128, n // 128
    rng = np.random.default_rng(seed)
    na = int(round(a_fraction * kb))
    am = np.zeros((mb, kb), bool)
    for i in range(mb):
        am[i, rng.permutation(kb)[:na]] = True
    tiles = o.seeded_tiles(nb, kb, w_fraction, seed)
    wm = np.zeros((nb, kb), bool)
    wm.flat[tiles] = True
    am_t = torch.from_numpy(np.repeat(am, 128, 1)).cuda()
    wm_t = torch.from_numpy(np.repeat(np.repeat(wm, 128, 0), 128, 1)).cuda()
    op = Native(wc, ws, wg, torch.ones(k, device='cuda'), am_t, wm_t, cross=cross)
    return op, x, (wc, ws, wg), am, tiles


def oracle_output(op, x, weights, packed, am, tiles, cross):
    wc, ws, wg = weights
    m = x.shape[0]
    full = op.na == op.k // 128
    return o.repair_linear(as_np(packed.codes), as_np(packed.scales), packed.factor.item(), as_np(wc), as_np(ws),
                           wg.item(), m, a_mask=None if op.na == 0 else am, a_full=full, w_tiles=tiles, cross=cross)


CASES = [
    # m, n, k, a_fraction, w_fraction, cross
    (128, 256, 256, 0.0, 0.0, False),       # plain W4A4, one tile
    (300, 256, 512, 0.0, 0.0, False),       # M tail
    (256, 384, 512, 0.0, 0.0, False),       # N = 3 x 128 -> 128-wide tiles
    (416, 512, 1024, 1.0, 0.0, False),      # full A1
    (416, 512, 1024, 0.5, 0.0, False),      # masked A1
    (384, 512, 1024, 0.0, 0.25, False),     # W1 tiles only
    (129, 256, 768, 0.5, 0.5, False),       # three terms, M tail of one row
    (384, 768, 1024, 0.5, 0.5, True),       # four terms with cross, 128-wide tiles
    (512, 1024, 2048, 0.25, 0.25, True),
    (256, 256, 256, 1.0, 1.0, True),        # dense W1 addressing
    (130, 256, 24576, 0.25, 0.25, False),   # the largest supported K (192 blocks: the Super-shaped FFN-down)
    (9600, 512, 256, 0.5, 0.5, False),      # 150 tiles on 148 SMs: two rounds of the persistent schedule
]


@pytest.mark.parametrize('m,n,k,af,wf,cross', CASES)
def test_fused_matches_oracle(m, n, k, af, wf, cross):
    from thunderworld_b200 import ops
    op, x, weights, am, tiles = build(m, n, k, 11, af, wf, cross)
    packed = op.pack(x)
    y = op.run_packed(x, packed)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    want = oracle_output(op, x, weights, packed, am, tiles, cross)
    got = y.float().cpu().numpy()
    assert got.shape == (m, n)
    assert np.isfinite(got).all()
    assert rel_l2(got, want) <= TOL, rel_l2(got, want)


def test_config0_full_size_and_deterministic():
    """The single repaired linear layer workload: M=3840, K=N=2048, full A1, 64 of 256 W1 tiles."""
    op, x, weights, am, tiles = build(3840, 2048, 2048, 0, 1.0, 0.25, False)
    assert len(tiles) == 64
    packed = op.pack(x)
    y1 = op.run_packed(x, packed)
    y2 = op.run_packed(x, packed)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    want = oracle_output(op, x, weights, packed, am, tiles, False)
    assert rel_l2(y1.float().cpu().numpy(), want) <= TOL


@pytest.mark.parametrize('budget', [2.0, 1.5])
@pytest.mark.parametrize('index', [0, 1, 2, 3])
def test_projection_set_layers_at_benchmark_shape(index, budget):
    """The four projections the benchmark times (M = 7680; QKV 6144x2048, out 2048x2048, FFN-up 8192x2048,
    FFN-down 2048x8192 with the cross term), built exactly as the benchmark builds them: online A1 selection
    (repair mode 3) writes the support the GEMM reads in the same stream. Checked against the oracle on the
    first, middle and last M128 row block at full N and K; tolerance 1e-3 on the output, bytes bit-exact."""
    import bench
    from thunderworld_b200 import ops
    name, n, k = bench.PROJECTIONS[index]
    layer = bench.Layer(name, n, k, bench.M_TOKENS, budget, index, torch.device('cuda', 0))
    layer.quantize(layer.x)
    layer.gemm(layer.x)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    mb = bench.M_TOKENS // 128
    res = bench.layer_parity(layer, [0, mb // 2, mb - 1])
    assert res['packed_bytes_bit_exact'] and res['selector_matches_oracle'] and res['finite'], res
    assert res['rel_l2'] <= TOL, res


PAIR_CASES = [
    (256, 256, 256, 0.0, 0.0, False),       # one pair tile, base only
    (300, 512, 1024, 0.5, 0.5, True),       # three row blocks: the last pair's peer has no rows
    (512, 1024, 2048, 0.25, 0.25, True),
    (1024, 512, 768, 1.0, 0.0, False),      # full A1, odd number of K128 blocks
    (640, 768, 512, 0.5, 1.0, True),        # dense W1 addressing
    (130, 256, 24576, 0.25, 0.25, False),   # the largest supported K
    (9728, 512, 256, 0.5, 0.5, False),      # more pair tiles than resident pairs
]


@pytest.mark.parametrize('m,n,k,af,wf,cross', PAIR_CASES)
def test_pair_kernel_matches_single_cta_kernel_and_oracle(m, n, k, af, wf, cross):
    """The CTA-pair kernel (tcgen05 cta_group::2) issues the same MMAs in the same order per output element as
    the single-CTA kernel (the A1 blocks it adds for the union of two supports are zeros), so the two agree bit
    for bit; both are within the tolerance of the oracle."""
    from thunderworld_b200 import ops
    op, x, weights, am, tiles = build(m, n, k, 23, af, wf, cross)
    packed = op.pack(x)
    op.kernel = 1
    single = op.run_packed(x, packed)
    op.kernel = 2
    pair = op.run_packed(x, packed)
    pair2 = op.run_packed(x, packed)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.isfinite(pair.float()).all()
    assert torch.equal(pair, pair2)
    assert torch.equal(pair, single)
    want = oracle_output(op, x, weights, packed, am, tiles, cross)
    assert rel_l2(pair.float().cpu().numpy(), want) <= TOL


def test_linearity_in_alpha_and_zero_activation():
    """Size-independent properties: zero input gives exact zeros; the output scales with alpha."""
    op, x, weights, am, tiles = build(256, 512, 512, 3, 0.5, 0.5, True)
    y0 = op(torch.zeros_like(x))
    assert float(y0.abs().max()) == 0.0
    packed = op.pack(x)
    y = op.run_packed(x, packed)
    packed.alpha.mul_(2.0)
    y2 = op.run_packed(x, packed)
    torch.cuda.synchronize()
    assert torch.equal(y2.float(), y.float() * 2)


def test_mask_is_read_at_run_time_under_graph_replay():
    """Capture once, then change the input and the A-support in place; replay equals eager
    (reference: tests/test_cuda.py:95-104, experiments/cutlass_fused_repair/test_fused.py:55-62)."""
    op, x, weights, am, tiles = build(384, 512, 1024, 3, 0.5, 0.25, False)
    static_x = x.clone()
    for _ in range(2):
        op(static_x)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = op(static_x)
    new_x = torch.from_numpy(o.synthetic_activation(384, 1024, 99)).cuda().bfloat16()
    static_x.copy_(new_x)
    new_mask = torch.roll(op.am, 1, 1)
    op.am.copy_(new_mask); op.union.copy_(new_mask)
    graph.replay()
    torch.cuda.synchronize()
    eager = op(new_x)
    assert torch.equal(out, eager)


@pytest.mark.parametrize('m,n,k,a_fraction,w_fraction,with_bias', [
    (300, 512, 512, 0.5, 0.5, True),        # M tail: rows beyond m (gelu(bias) != 0 there) must not reach the maximum
    (256, 384, 512, 0.0, 0.0, False),       # 128-wide tiles
    (1000, 1024, 1024, 0.5, 0.25, False),   # several tiles per CTA
])
def test_fused_activation_epilogue_matches_the_separate_activation_pass(m, n, k, a_fraction, w_fraction, with_bias):
    """GELU in the GEMM epilogue = activate_with_factor applied to the plain GEMM output, bit for bit, and the
    (factor, max) pair equals the one the separate pass reduces."""
    from thunderworld_b200 import ops
    op, x, _, am, _ = build(m, n, k, 11, a_fraction, w_fraction)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(1)) * 0.5).bfloat16().cuda() if with_bias else None
    packed = op.pack(x)
    plain = op.run_packed(x, packed, bias=bias)
    want, want_stats = ops.activate_with_factor(plain, mode='gelu_tanh', return_stats=True)
    got, stats = op.run_packed(x, packed, bias=bias, activation='gelu_tanh', want_stats=True)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert torch.equal(stats, want_stats), (stats, want_stats)
    again, stats2 = op.run_packed(x, packed, bias=bias, activation='gelu_tanh', want_stats=True)   # scratch was left zeroed
    assert torch.equal(stats2, want_stats) and torch.equal(again, got)
    only = op.run_packed(x, packed, bias=bias, activation='gelu_tanh')                              # without the reduction
    assert torch.equal(only, got)
    assert ops.device_status() == 0


def test_fused_activation_argument_checks():
    op, x, _, _, _ = build(256, 512, 512, 3, 0.0, 0.0)
    packed = op.pack(x)
    with pytest.raises(ValueError):
        op.run_packed(x, packed, activation='relu2')
    with pytest.raises(ValueError):
        op.run_packed(x, packed, want_stats=True)
    op.kernel = 2                                            # the CTA-pair kernel has no activation epilogue
    with pytest.raises(RuntimeError):
        op.run_packed(x, packed, activation='gelu_tanh')
