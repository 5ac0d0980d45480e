"""Pointwise producers (activation, RMSNorm + modulation, head norm, gated residual) against the oracle.

relu^2, a*b and the gated residual are bit-exact (float32 arithmetic with one bf16 rounding, as in the
reference's pointwise_amax, thunderworld_fp4/_fusion.py:15-24); the factor is bit-exact with them. GELU and
the norms go through approximate transcendental / a different summation order: stated tolerances below.
"""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu
TOL_L2 = 2e-3            # relative L2 of bf16 outputs whose last-bit rounding may differ
TOL_ULP = 2 ** -7        # one bf16 ulp, relative


def _dev(a):
    return torch.from_numpy(np.asarray(a, np.float32)).bfloat16().cuda()


def _host(t):
    return t.float().cpu().numpy()


def _rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize('shape', [(3, 128), (1920, 8192), (7, 40)])
@pytest.mark.parametrize('mode', ['relu2', 'mul'])
def test_activate_bit_exact(shape, mode):
    from thunderworld_b200 import ops
    rng = np.random.default_rng(1)
    a = O.bf16_round(rng.standard_normal(shape).astype(np.float32) * 3)
    b = O.bf16_round(rng.standard_normal(shape).astype(np.float32)) if mode == 'mul' else None
    want, factor = O.activate_with_factor(a, b)
    for _ in range(2):                                   # the scratch must come back zeroed
        y, f = ops.activate_with_factor(_dev(a), None if b is None else _dev(b))
        assert np.array_equal(_host(y).view(np.uint32), want.view(np.uint32))
        assert np.float32(f.item()).view(np.uint32) == np.float32(factor).view(np.uint32)


def test_activate_zero_tensor_factor_is_one():
    from thunderworld_b200 import ops
    y, f = ops.activate_with_factor(torch.zeros(16, 128, device='cuda', dtype=torch.bfloat16))
    assert f.item() == 1.0 and not y.any()


def test_gelu_tanh():
    from thunderworld_b200 import ops
    rng = np.random.default_rng(2)
    a = O.bf16_round(rng.standard_normal((512, 1024)).astype(np.float32) * 2)
    want, factor = O.activate_with_factor(a, mode='gelu_tanh')
    y, f = ops.activate_with_factor(_dev(a), mode='gelu_tanh')
    got = _host(y)
    assert _rel(got, want) < TOL_L2
    assert np.all(np.abs(got - want) <= TOL_ULP * np.abs(want) + 1e-3)
    assert abs(f.item() - factor) <= TOL_ULP * factor


@pytest.mark.parametrize('hidden', [128, 2048, 4096, 6144])
@pytest.mark.parametrize('modulated', [False, True])
def test_rms_norm(hidden, modulated):
    from thunderworld_b200 import ops
    rng = np.random.default_rng(hidden)
    batch, tokens = 2, 96
    x = O.bf16_round(rng.standard_normal((batch, tokens, hidden)).astype(np.float32) * 2)
    w = O.bf16_round(1 + 0.1 * rng.standard_normal(hidden).astype(np.float32))
    shift = O.bf16_round(0.1 * rng.standard_normal((batch, hidden)).astype(np.float32)) if modulated else None
    scale = O.bf16_round(0.1 * rng.standard_normal((batch, hidden)).astype(np.float32)) if modulated else None
    want, factor = O.rms_norm(x, w, 1e-6, shift, scale)
    y, f = ops.rms_norm(_dev(x), _dev(w), 1e-6, shift=None if shift is None else _dev(shift),
                        scale=None if scale is None else _dev(scale), want_factor=True)
    got = _host(y)
    assert _rel(got, want) < TOL_L2
    assert np.all(np.abs(got - want) <= TOL_ULP * np.abs(want) + 1e-6)
    assert abs(f.item() - factor) <= TOL_ULP * factor
    # without weight and factor
    want2, _ = O.rms_norm(x, None, 1e-6)
    assert _rel(_host(ops.rms_norm(_dev(x))), want2) < TOL_L2


def test_rms_norm_feeds_the_quantizer_factor():
    """The fused factor equals what the quantizer reduces itself, so packed bytes are identical."""
    from thunderworld_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(1, 256, 2048, device='cuda').bfloat16()
    y, f = ops.rms_norm(x, want_factor=True)
    own = ops.quantize(y.reshape(256, 2048), repair=1)
    given = ops.quantize(y.reshape(256, 2048), repair=1, factor=f.reshape(()))
    assert own.factor.item() == f.item()
    assert torch.equal(own.codes, given.codes) and torch.equal(own.scales.view(torch.uint8), given.scales.view(torch.uint8))


def test_rms_norm_heads_strided_view():
    from thunderworld_b200 import ops
    torch.manual_seed(1)
    qkv = torch.randn(2, 200, 3, 4, 128, device='cuda').bfloat16()
    for part in range(2):
        view = qkv[:, :, part]
        y = ops.rms_norm_heads(view)
        want, _ = O.rms_norm(_host(view))
        assert y.is_contiguous() and y.shape == view.shape
        assert _rel(_host(y), want) < TOL_L2


def test_gate_residual_bit_exact():
    from thunderworld_b200 import ops
    rng = np.random.default_rng(3)
    x = O.bf16_round(rng.standard_normal((2, 300, 512)).astype(np.float32))
    y = O.bf16_round(rng.standard_normal((2, 300, 512)).astype(np.float32))
    g = O.bf16_round(rng.standard_normal((2, 512)).astype(np.float32))
    want = O.gate_residual(x, g, y)
    xd = _dev(x)
    out = ops.gate_residual_(xd, _dev(g), _dev(y))
    assert out.data_ptr() == xd.data_ptr()
    assert np.array_equal(_host(out).view(np.uint32), want.view(np.uint32))


def test_argument_errors():
    from thunderworld_b200 import ops
    a = torch.zeros(4, 128, device='cuda', dtype=torch.float32)
    with pytest.raises(ValueError):
        ops.activate_with_factor(a)
    b = torch.zeros(4, 129, device='cuda', dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):                   # n % 8 != 0 -> status from the C ABI
        ops.activate_with_factor(b)


@pytest.mark.parametrize('table_dtype', [torch.float32, torch.bfloat16])
def test_rope_heads_bit_exact_and_fused_with_head_norm(table_dtype):
    """Exact-rounding RoPE: bit for bit against the oracle; running it after the head norm in the same kernel gives
    the bytes of the two kernels run one after the other; strided q / k views of a fused QKV output are accepted."""
    from thunderworld_b200 import ops
    from thunderworld_b200.cosmos.dit import rope_tables
    g = torch.Generator().manual_seed(3)
    b, s, h = 2, 75, 3
    qkv = torch.randn(b, s, 3, h, 128, generator=g).bfloat16().cuda()
    cos, sin = (t.to(table_dtype) for t in rope_tables(s, 'cuda'))
    q = qkv[:, :, 0]                                              # strided view [b, s, h, 128]
    got = ops.rope_heads(q, cos, sin)
    want = O.rope(q.float().cpu().numpy(), np.tile(cos.float().cpu().numpy(), (b, 1)).reshape(b, s, 128)[0],
                  sin.float().cpu().numpy())
    assert np.array_equal(got.float().cpu().numpy(), want)
    fused = ops.rope_heads(q, cos, sin, norm=True)
    two = ops.rope_heads(ops.rms_norm_heads(q), cos, sin)
    assert torch.equal(fused, two)
    with pytest.raises(ValueError):
        ops.rope_heads(q, cos[:, :64].contiguous(), sin[:, :64].contiguous())
