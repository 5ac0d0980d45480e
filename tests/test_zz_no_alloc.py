"""tw_quantize_static: the quantizer for hosts that may not allocate device memory.

Some callers (a plugin living inside another framework's memory plan, a loop that must not allocate
after start-up) cannot hand the quantizer a scratch buffer. This entry point keeps its scratch in a fixed
array inside the library. The test calls it through the C ABI twice in a row, with different inputs, and
requires the same bytes as the ordinary entry point (bit-exact, like every other quantizer test). The file
name sorts last so that a run stopping at the first failure has already run everything else."""
import ctypes
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def run(entry, x, mask, sens, na, workspace):
    from thunderworld_b200 import _lib
    lib = _lib.load()
    m, k = x.shape
    mp, mb = (m + 15) // 16 * 16, (m + 127) // 128
    dev = x.device
    out = dict(codes=torch.zeros((2, mp, k // 2), device=dev, dtype=torch.uint8),
               scales=torch.zeros((2, mp, k // 16), device=dev, dtype=torch.uint8),
               swz=torch.zeros((2, mb * 128, k // 16), device=dev, dtype=torch.uint8),
               factor=torch.zeros((), device=dev, dtype=torch.float32), mask=mask)
    args = _lib.QuantizeArgs(x.data_ptr(), None, sens.data_ptr(), out['factor'].data_ptr(), None, None,
                             out['codes'].data_ptr(), out['scales'].data_ptr(), out['swz'].data_ptr(), mask.data_ptr(),
                             None if workspace is None else workspace.data_ptr(), m, k, mp, 3, na, 0, 1., 1., 1., 1.)
    status = getattr(lib, entry)(ctypes.byref(args), torch.cuda.current_stream().cuda_stream)
    assert status == 0, lib.tw_status(status)
    torch.cuda.synchronize()
    return out


def test_static_scratch_entry_matches_workspace_entry_twice():
    from oracle import nvfp4_oracle as o
    from thunderworld_b200 import _lib
    lib = _lib.load()
    for seed, (m, k, na) in enumerate([(300, 1024, 3), (640, 512, 1)]):
        x = torch.from_numpy(o.synthetic_activation(m, k, 40 + seed)).cuda().bfloat16()
        sens = torch.rand(k, device='cuda') + 0.5
        mb, kb = (m + 127) // 128, k // 128
        ws = torch.zeros(lib.tw_quantize_workspace(m, k), device='cuda', dtype=torch.uint8)
        want = run('tw_quantize', x, torch.zeros((mb, kb), device='cuda', dtype=torch.bool), sens, na, ws)
        got = run('tw_quantize_static', x, torch.zeros((mb, kb), device='cuda', dtype=torch.bool), sens, na, None)
        for key in ('codes', 'scales', 'swz', 'factor', 'mask'):
            assert torch.equal(got[key], want[key]), key
        assert int(got['mask'].sum()) == mb * na


def test_static_scratch_entry_rejects_oversized_problems():
    from thunderworld_b200 import _lib
    lib = _lib.load()
    limit = lib.tw_quantize_static_max_tiles()
    m, k = 128 * 129, 128 * 128                     # 129 * 128 tiles > 16384
    assert (m // 128) * (k // 128) > limit
    args = _lib.QuantizeArgs(1, None, None, 1, None, None, 1, 1, None, None, None, m, k, m, 0, 0, 0, 1., 1., 1., 1.)
    status = lib.tw_quantize_static(ctypes.byref(args), None)
    assert status != 0 and b'maximum' in lib.tw_status(status)
