"""CPU checks of the pointwise restatements against plain torch (bf16 eager semantics of the reference's
pointwise_amax: float32 op, one rounding)."""
import numpy as np
import torch

from oracle import nvfp4_oracle as O


def test_relu2_and_mul_match_torch_float32_then_bf16():
    torch.manual_seed(0)
    a = torch.randn(64, 256).bfloat16()
    b = torch.randn(64, 256).bfloat16()
    relu2 = (a.float().clamp_min(0) ** 2).bfloat16().float().numpy()
    mul = (a.float() * b.float()).bfloat16().float().numpy()
    y, f = O.activate_with_factor(a.float().numpy())
    assert np.array_equal(y, relu2) and f == np.float32(np.abs(relu2).max() / np.float32(2688.))
    y, _ = O.activate_with_factor(a.float().numpy(), b.float().numpy())
    assert np.array_equal(y, mul)
    assert O.activate_with_factor(np.zeros((2, 8), np.float32))[1] == 1.0


def test_gelu_and_norm_match_torch():
    torch.manual_seed(1)
    a = torch.randn(32, 512).bfloat16()
    want = torch.nn.functional.gelu(a.float(), approximate='tanh').bfloat16().float().numpy()
    y, _ = O.activate_with_factor(a.float().numpy(), mode='gelu_tanh')
    assert np.mean(y != want) < 0.01 and np.allclose(y, want, rtol=2 ** -7, atol=1e-6)
    x = torch.randn(2, 16, 256).bfloat16()
    w = (1 + 0.1 * torch.randn(256)).bfloat16()
    xf = x.float()
    want = (w.float() * (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + 1e-6))).bfloat16().float().numpy()
    y, _ = O.rms_norm(x.float().numpy(), w.float().numpy(), 1e-6)
    assert np.mean(y != want) < 0.01 and np.allclose(y, want, rtol=2 ** -7, atol=1e-6)


def test_gate_residual_matches_float32_fma():
    torch.manual_seed(2)
    x, y = torch.randn(2, 8, 64).bfloat16(), torch.randn(2, 8, 64).bfloat16()
    g = torch.randn(2, 64).bfloat16()
    want = torch.addcmul(x.double(), g.double()[:, None], y.double()).float().bfloat16().float().numpy()
    assert np.array_equal(O.gate_residual(x.float().numpy(), g.float().numpy(), y.float().numpy()), want)


def test_rope_matches_bf16_torch_arithmetic():
    """The reference's RoPE kernel reproduces PyTorch's bf16 evaluation, which materialises both bf16 products before
    the bf16 addition (cosmos/pipeline_tuning.py:53-55); the oracle must equal that evaluation bit for bit."""
    import torch
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 17, 3, 128, generator=g).bfloat16()
    ang = torch.rand(17, 128, generator=g) * 6
    cos, sin = ang.cos().bfloat16(), ang.sin().bfloat16()
    rot = torch.cat([-x[..., 64:], x[..., :64]], -1)
    want = x * cos[:, None, :] + rot * sin[:, None, :]                      # bf16 mul, bf16 mul, bf16 add
    got = O.rope(x.float().numpy(), cos.float().numpy(), sin.float().numpy())
    assert np.array_equal(got, want.float().numpy())
