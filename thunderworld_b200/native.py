"""Repaired linear operator over packed NVFP4 weights: host-side mirror of the reference's
`Native` (packages/fp4-repair/src/thunderworld_fp4/_native.py:73-121) and of its CUTLASS bridge
`CutlassFused` (thunderworld_fp4/cutlass/backend.py:15-71), backed by the sm_100a fused kernel.

Same constructor arguments, attributes and call protocol: `pack(x)`, `run_packed(x, packed)`,
`__call__(x)`; `am`, `union`, `na`, `wr`, `wrs`, `wi`, `off`, `wloc`, `shared_bank`, `dense_w`
may be replaced by a caller that manages a shared W1 bank (thunderworld_fp4/cosmos/linears.py:118-144).
"""
import torch
from . import ops


class Native:
    def __init__(self, wc, ws, wg, d, am, wm, b=128, cross=False, bm=128, interleave=True, num_warps=4,
                 num_stages=1, split_k=1):
        if b != 128 or bm not in (32, 64, 128):
            raise ValueError('the sm_100a kernel works on the K128 lattice with 128-row tiles')
        if split_k != 1:
            raise ValueError('split-K is not used on sm_100a: one accumulator per output tile')
        if not wc.is_cuda:
            raise ValueError('packed weights must be on a CUDA device')
        ops.require_sm100(wc.device)
        if am.dtype != torch.bool or wm.dtype != torch.bool:
            raise ValueError('repair supports must be boolean')
        self.b, self.bm, self.interleave, self.cross, self.d = b, 128, True, bool(cross), d
        self.split_k = 1
        self.wc = wc[0].contiguous().clone()
        self.ws = ws[0].contiguous().clone()
        self.wg = wg
        self.n, self.k = self.wc.shape[0], self.wc.shape[1] * 2
        if self.n % 128 or self.k % 128:
            raise ValueError('N and K must be multiples of 128')
        kb, nb = self.k // 128, self.n // 128
        # activation support: all host inspection happens here, offline
        self.am = am.reshape(-1, kb, 128).any(-1).contiguous()
        counts = self.am.sum(-1)
        if not bool((counts == counts[0]).all()):
            raise ValueError('every M128 row block must select the same number of K blocks')
        self.na = int(counts[0])
        self.ai = self.am.nonzero()[:, 1].reshape(self.am.shape[0], self.na).int().contiguous()
        self.union = self.am.clone()
        # weight support: CSR over N128 blocks, tiles gathered into a bank
        tiles = wm.reshape(nb, 128, kb, 128).any((1, 3))
        pairs = tiles.nonzero()
        self.hasw = bool(pairs.numel())
        self.dense_w = bool(tiles.all())
        self.off = torch.cat([torch.zeros(1, device=wc.device, dtype=torch.int32),
                              tiles.sum(-1).int().cumsum(0).int()]).contiguous()
        self.wi = pairs[:, 1].int().contiguous()
        self.wloc = self.wi
        self.shared_bank = False
        code_tiles = wc[1].reshape(nb, 128, kb, 64).permute(0, 2, 1, 3)
        scale_tiles = ws[1].view(torch.uint8).reshape(nb, 128, kb, 8).permute(0, 2, 1, 3)
        self.wr = code_tiles[pairs[:, 0], pairs[:, 1]].contiguous()
        self.wrs = scale_tiles[pairs[:, 0], pairs[:, 1]].contiguous().view(torch.float8_e4m3fn)
        self._prepare_layouts()

    def _prepare_layouts(self):
        """Atom-layout copies of the offline scales (done once; the reference does the same for W0 in
        CutlassFused.__init__, cutlass/backend.py:29)."""
        self.ws_swz = ops.swizzle(self.ws)
        self._bank_key = None
        self.wrs_swz = None
        self._refresh_bank()

    def _refresh_bank(self):
        key = (self.wrs.data_ptr(), tuple(self.wrs.shape)) if self.hasw else None
        if key != self._bank_key:
            self.wrs_swz = ops.swizzle(self.wrs.reshape(-1, 8)) if self.hasw and self.wrs.numel() else None
            self._bank_key = key

    def pack(self, x, **kw):
        repair = 0 if self.na == 0 else (1 if self.na == self.k // 128 else 2)
        return ops.quantize(x, self.d, repair=repair, mask=self.union if repair == 2 else None, wg=self.wg, **kw)

    def run_packed(self, x, packed, out=None, bias=None, activation=None, want_stats=False):
        m = x.shape[0]
        self._refresh_bank()
        if not isinstance(packed, ops.Packed):
            raise TypeError('run_packed expects the Packed result of pack()')
        return ops.fused_gemm(m, self.n, self.k, packed, self.wc, self.ws_swz, packed.alpha, na=self.na,
                              mask=self.am, wr=self.wr if self.hasw else None, wrs_swz=self.wrs_swz, wi=self.wi,
                              off=self.off, wloc=self.wloc, cross=self.cross, shared=self.shared_bank,
                              dense=self.dense_w, ws=self.ws, wrs=self.wrs if self.hasw else None, out=out,
                              kernel=getattr(self, 'kernel', 0), bias=bias, activation=activation, want_stats=want_stats)

    def __call__(self, x):
        if x.ndim != 2 or x.shape[1] != self.k or x.shape[0] <= 0 or ops.cdiv(x.shape[0], 128) != self.am.shape[0]:
            raise ValueError('activation shape must match the prepared M128 support and K')
        if x.dtype != torch.bfloat16 or x.device != self.wc.device or not x.is_contiguous():
            raise ValueError('expected contiguous BF16 activation on the packed-weight device')
        return self.run_packed(x, self.pack(x))

    @property
    def residual_weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.wr, self.wrs, self.wi, self.off)) if self.hasw else 0


def quantize_weight(weight, prescale=None):
    """Offline W0/W1 preparation on the GPU: the activation packer applied to W / prescale
    (reference: cosmos/linears.py:64-73; CPU twin calibration.py:44-54). Returns codes [2,N,K/2],
    scales [2,N,K/16] (E4M3), factor."""
    if weight.ndim != 2 or weight.dtype != torch.bfloat16 or not weight.is_cuda:
        raise ValueError('offline weight must be BF16 CUDA [N,K]')
    w = weight if prescale is None else (weight.float() / prescale).bfloat16()
    p = ops.quantize(w.contiguous(), None, repair=1)
    n = weight.shape[0]
    return p.codes[:, :n].contiguous(), p.scales[:, :n].contiguous(), p.factor
