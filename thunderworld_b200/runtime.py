"""Attention boundary: validation, online packing, tile selection, the streaming FP4 kernel and an
optional per-operator CUDA Graph cache. Mirrors the reference's runtime
(packages/fp4-repair/src/thunderworld_fp4/runtime.py: _validate :11-29, _forward :32-108,
fp4_attention :111-122, FP4Attention :128-194) on the sm_100a kernels.

Input and output layout is [1, sequence, heads, 128] BF16 (sequence stride free). Attention is
non-causal and unmasked; a repair mask selects residual work, it never removes an edge. One difference
from the reference: a leading batch dimension larger than one is accepted and processed as independent
problems (the CFG cond/uncond pair), with one mask per batch entry when masks are given.
"""
from collections import OrderedDict
from contextlib import nullcontext
from threading import RLock
import ctypes
import torch
from . import _lib, ops
from .config import RepairConfig, RepairPolicy


def _validate(q, k, v):
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v)):
        raise TypeError('q, k, v must be tensors')
    if any(t.ndim != 4 for t in (q, k, v)):
        raise ValueError('expected [batch, sequence, heads, 128] Q/K/V')
    if q.shape[0] != k.shape[0] or k.shape != v.shape:
        raise ValueError('batch sizes and K/V shapes must match')
    if any(t.shape[-1] != 128 or t.stride(-1) != 1 for t in (q, k, v)):
        raise ValueError('head dimension must be 128 with contiguous last dimension')
    if min(q.shape[:3]) <= 0 or min(k.shape[:3]) <= 0 or q.shape[2] % k.shape[2]:
        raise ValueError('nonempty sequences/heads and an integer GQA ratio are required')
    if any(t.dtype != torch.bfloat16 for t in (q, k, v)):
        raise ValueError('Q/K/V must be BF16 inputs; FP4 quantization is online')
    if not q.is_cuda or k.device != q.device or v.device != q.device:
        raise ValueError('Q/K/V must be on the same CUDA device')
    if any(t.stride(1) % 8 or t.stride(2) % 8 for t in (q, k, v)):
        raise ValueError('token and head strides must be multiples of 8 elements')
    ops.require_sm100(q.device)
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v)):
        raise RuntimeError('inference-only backend: use torch.inference_mode()')


class PackedRows:
    """One packed operand (Q, K or V of one batch entry)."""

    def __init__(self, x, rows_padded, repair, transpose_v=False, need_energy=False):
        rows, heads = x.shape[0], x.shape[1]
        dev = x.device
        planes = 2 if repair else 1
        blocks = ops.cdiv(rows_padded, 128)
        self.codes = torch.empty((planes, heads * rows_padded, 64), device=dev, dtype=torch.uint8)
        self.scales = torch.empty((planes, heads * rows_padded, 8), device=dev, dtype=torch.float8_e4m3fn)
        # every byte of an atom is written by the packer for rows below rows_padded: padding atoms exist only
        # when rows_padded is not a multiple of 128, and only then the buffer has to start zeroed
        make = torch.zeros if rows_padded % 128 else torch.empty
        self.scales_swz = make((planes, heads, blocks, 1024), device=dev, dtype=torch.uint8)
        self.factors = torch.empty((heads * rows_padded,), device=dev, dtype=torch.float32)
        self.energy = torch.empty((heads, blocks, 8), device=dev, dtype=torch.float32) if need_energy else None
        args = _lib.PackRowsArgs(x.data_ptr(), self.codes.data_ptr(), self.scales.data_ptr(), self.scales_swz.data_ptr(),
                                 self.factors.data_ptr(), None if self.energy is None else self.energy.data_ptr(),
                                 x.stride(0), x.stride(1), rows, heads, rows_padded, int(repair), int(transpose_v),
                                 int(need_energy))
        _lib.check(_lib.load().tw_pack_rows(ctypes.byref(args), torch.cuda.current_stream(dev).cuda_stream))


def pack_inputs(q, k, v, repair=True, need_energy=False, terms=3, pv_repair=None, pv_terms=None):
    """q [M,H,128], k/v [N,HK,128] views -> (PackedRows q, k, v, mp, np)."""
    m, n = q.shape[0], k.shape[0]
    mp, np_ = ops.cdiv(m, 16) * 16, ops.cdiv(n, 128) * 128
    pv_repair = repair if pv_repair is None else pv_repair
    pv_terms = terms if pv_terms is None else pv_terms
    pq = PackedRows(q, mp, repair)
    pk = PackedRows(k, np_, repair and terms >= 3)
    pv = PackedRows(v, np_, pv_repair and pv_terms >= 3, transpose_v=True, need_energy=need_energy)
    return pq, pk, pv, mp, np_


def _forward_one(q, k, v, config, repair_mask, counts_tensor, return_mask, out):
    """One batch entry. q [M,H,128], k/v [N,HK,128] (strided views), out [M,H,128] contiguous."""
    lib = _lib.load()
    dev = q.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    m, n, h, hk = q.shape[0], k.shape[0], q.shape[1], k.shape[1]
    nt, mt = ops.cdiv(n, 128), ops.cdiv(m, 128)
    counts = config.head_counts(h, n)
    pv_counts = config.pv_counts(h, n)
    separate = config.separate_pv
    pv_terms = config.pv_terms or config.terms
    mask_shape = (h, mt, nt)
    flags = pv_flags = None
    if repair_mask is not None:
        if (tuple(repair_mask.shape) != mask_shape or repair_mask.dtype != torch.bool or repair_mask.device != dev
                or not repair_mask.is_contiguous()):
            raise ValueError(f'repair_mask must be contiguous CUDA bool {mask_shape}')
        # True selects repair; False still executes every dense FP4 base product
        flags = torch.where(repair_mask, config.terms, 1).to(torch.int32)
        pv_flags = torch.where(repair_mask, pv_terms, 1).to(torch.int32) if separate else flags
        repair, full, pv_repair, pv_full, selection = True, False, True, False, False
    else:
        repair, full = any(counts), all(c == nt for c in counts)
        pv_repair, pv_full = any(pv_counts), all(c == nt for c in pv_counts)
        if not separate:
            pv_repair, pv_full = repair, full
        selection = (repair and not full) or (separate and pv_repair and not pv_full)
    pq, pk, pv, mp, np_ = pack_inputs(q, k, v, repair, selection, config.terms, pv_repair, pv_terms)
    keepalive = [pq, pk, pv]
    if selection:
        if counts_tensor is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError('head quotas must be resident before capture: use FP4Attention or an explicit repair_mask')
            counts_tensor = (torch.tensor(counts, device=dev, dtype=torch.int32),
                             torch.tensor(pv_counts, device=dev, dtype=torch.int32))
        flags = torch.empty(mask_shape, device=dev, dtype=torch.int32)
        pv_flags = torch.empty(mask_shape, device=dev, dtype=torch.int32) if separate else flags
        args = _lib.SelectArgs(q.data_ptr(), k.data_ptr(), pv.energy.data_ptr(), flags.data_ptr(),
                               pv_flags.data_ptr() if separate else None, counts_tensor[0].data_ptr(),
                               counts_tensor[1].data_ptr() if separate else None, q.stride(0), q.stride(1), k.stride(0),
                               k.stride(1), m, n, h, hk, config.terms, pv_terms)
        _lib.check(lib.tw_select_tiles(ctypes.byref(args), stream))
        keepalive.append(counts_tensor)
    ws = ops._workspace(dev, lib.tw_attention_workspace(m, n, h, hk), 'a')
    args = _lib.AttentionArgs(pq.codes.data_ptr(), pk.codes.data_ptr(), pv.codes.data_ptr(), pq.scales_swz.data_ptr(),
                              pk.scales_swz.data_ptr(), pv.scales_swz.data_ptr(), pq.factors.data_ptr(),
                              pk.factors.data_ptr(), pv.factors.data_ptr(), None if flags is None else flags.data_ptr(),
                              None if pv_flags is None else pv_flags.data_ptr(), out.data_ptr(), ws.data_ptr(),
                              m, n, h, hk, mp, np_, int(repair), int(full), config.terms, int(pv_repair), int(pv_full),
                              pv_terms)
    _lib.check(lib.tw_attention(ctypes.byref(args), stream))
    keepalive += [flags, pv_flags]
    selected = None
    if return_mask:
        if flags is not None:
            selected = flags > 1
            if separate:
                selected = torch.stack((selected, pv_flags > 1))
        else:
            selected = torch.full(mask_shape, full, device=dev, dtype=torch.bool)
            if separate:
                selected = torch.stack((selected, torch.full(mask_shape, pv_full, device=dev, dtype=torch.bool)))
    return selected, keepalive


_side_streams = {}


def _side_stream(device, index):
    key = (device, index)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device)
    return _side_streams[key]


def _forward(q, k, v, config, repair_mask=None, counts_tensor=None, return_mask=False):
    _validate(q, k, v)
    if not isinstance(config, RepairConfig):
        raise TypeError('config must be RepairConfig')
    batch = q.shape[0]
    out = torch.empty(tuple(q.shape), device=q.device, dtype=q.dtype)
    masks, keep = [], []
    # Batch entries are independent problems (CFG cond / uncond). Entry 0 runs on the caller's stream, the
    # others on side streams that fork from it and join it again, so that the tail of one entry's
    # attention grid (960 CTAs = 6.5 waves of 148) is filled by the next entry's CTAs. The fork / join is
    # made of events only, which a CUDA Graph capture of the caller's stream records as parallel branches.
    main = torch.cuda.current_stream(q.device)
    fork = None
    if batch > 1:
        fork = torch.cuda.Event()
        fork.record(main)
    for b in range(batch):
        mask_b = None
        if repair_mask is not None:
            mask_b = repair_mask if batch == 1 and repair_mask.ndim == 3 else repair_mask[b]
        if b == 0:
            selected, held = _forward_one(q[b], k[b], v[b], config, mask_b, counts_tensor, return_mask, out[b])
        else:
            side = _side_stream(q.device, b)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                selected, held = _forward_one(q[b], k[b], v[b], config, mask_b, counts_tensor, return_mask, out[b])
                join = torch.cuda.Event()
                join.record(side)
            main.wait_event(join)
        masks.append(selected)
        keep.append(held)
    selected = None
    if return_mask:
        selected = masks[0] if batch == 1 else torch.stack(masks)
    return out, selected, keep


def fp4_attention(q, k, v, config=None, *, repair_mask=None, return_mask=False):
    """Non-causal, unmasked GQA attention with Q, K, V and P in NVFP4 and selective residual repair.
    An explicit boolean `repair_mask` [heads, ceil(M/128), ceil(N/128)] overrides coverage and quotas."""
    cuda = isinstance(q, torch.Tensor) and q.is_cuda
    with torch.cuda.device(q.device) if cuda else nullcontext():
        out, selected, _ = _forward(q, k, v, config or RepairConfig(), repair_mask, return_mask=return_mask)
    return (out, selected) if return_mask else out


class FP4Attention:
    """Attention operator with an optional CUDA Graph cache keyed by stream, shapes and resolved
    configuration. Every call copies the current inputs (and mask) into the cached buffers, replays,
    and returns output that owns its storage. Layer / step / CFG-branch context is explicit."""

    def __init__(self, config=None, *, policy=None, graph_cache_size=2):
        if config is not None and policy is not None:
            raise ValueError('choose config or policy')
        if type(graph_cache_size) is not int or graph_cache_size < 0:
            raise ValueError('graph_cache_size must be a nonnegative integer')
        self.policy = policy or RepairPolicy(default=config or RepairConfig())
        if not isinstance(self.policy, RepairPolicy):
            raise TypeError('policy must be RepairPolicy')
        self.graph_cache_size = graph_cache_size
        self._cache = OrderedDict()
        self._lock = RLock()

    def clear(self):
        with self._lock:
            for entry in self._cache.values():
                entry['stream'].synchronize()
            self._cache.clear()

    def _quotas(self, config, q, k):
        dev = q.device
        return (torch.tensor(config.head_counts(q.shape[2], k.shape[1]), device=dev, dtype=torch.int32),
                torch.tensor(config.pv_counts(q.shape[2], k.shape[1]), device=dev, dtype=torch.int32))

    def __call__(self, q, k, v, *, layer=None, step=None, branch=None, repair_mask=None, return_mask=False):
        config = self.policy.resolve(layer=layer, step=step, branch=branch)
        _validate(q, k, v)
        with torch.cuda.device(q.device):
            if not self.graph_cache_size or torch.cuda.is_current_stream_capturing():
                out, selected, _ = _forward(q, k, v, config, repair_mask, self._quotas(config, q, k)
                                            if not torch.cuda.is_current_stream_capturing() else None, return_mask)
                return (out, selected) if return_mask else out
            stream = torch.cuda.current_stream(q.device)
            key = (q.device, stream.cuda_stream, tuple(q.shape), tuple(k.shape), config, repair_mask is not None,
                   return_mask)
            with self._lock:
                if repair_mask is not None:
                    expected = (q.shape[2], ops.cdiv(q.shape[1], 128), ops.cdiv(k.shape[1], 128))
                    lead = () if q.shape[0] == 1 and repair_mask.ndim == 3 else (q.shape[0],)
                    if (repair_mask.dtype != torch.bool or repair_mask.device != q.device
                            or tuple(repair_mask.shape) != lead + expected or not repair_mask.is_contiguous()):
                        raise ValueError(f'repair_mask must be contiguous CUDA bool {lead + expected}')
                if key not in self._cache:
                    if len(self._cache) >= self.graph_cache_size:
                        _, previous = self._cache.popitem(last=False)
                        previous['stream'].synchronize()
                    buffers = tuple(t.contiguous().clone() for t in (q, k, v))
                    mask_buffer = repair_mask.clone() if repair_mask is not None else None
                    quotas = self._quotas(config, q, k)
                    for _ in range(2):
                        _forward(*buffers, config, mask_buffer, quotas, return_mask)
                    torch.cuda.synchronize(q.device)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        output, selected, held = _forward(*buffers, config, mask_buffer, quotas, return_mask)
                    self._cache[key] = dict(buffers=buffers, mask=mask_buffer, graph=graph, output=output,
                                            selected=selected, stream=stream, quotas=quotas, held=held)
                else:
                    self._cache.move_to_end(key)
                entry = self._cache[key]
                for source, target in zip((q, k, v), entry['buffers']):
                    target.copy_(source)
                if entry['mask'] is not None:
                    entry['mask'].copy_(repair_mask)
                entry['graph'].replay()
                result = entry['output'].clone()
                return (result, entry['selected'].clone()) if return_mask else result
