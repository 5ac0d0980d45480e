"""Times the reference project's own tcgen05 fused repair GEMM ("reference-sm100", built by
baseline/build_reference_sm100.py) beside this repository's tw_fused on the Cosmos3-Edge-shaped projection
set (M = 7680; QKV 6144x2048, out 2048x2048, FFN-up 8192x2048, FFN-down 2048x8192) at the base, 1.5x and 2x
issued-work plans. Both kernels get byte-identical packed operands (this repository's quantizer output, the
selector's realised mask, the same W1 bank) through the same C ABI; only the scale-layout pointers differ
(the reference reads row-major residual scales, tw_fused reads atom-layout ones).

    python baseline/reference_sm100.py [--steps 20] [--out FILE.json]

Protocol: every (layer, kernel) launch is captured in its own CUDA Graph; per round all launches are queued
behind a spin kernel and bracketed by CUDA events; the layers rotate so consecutive launches of one kernel
do not find their operands in L2. One GPU only.
"""
import argparse
import ctypes
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
REF_LIB = os.path.join(ROOT, 'baseline', '_ref', 'libtw_ref_sm100.so')


class RefIO(ctypes.Structure):
    """RepairIO of tools/thor_handoff/sm110_repair_collective.cuh:6-11."""
    _fields_ = [(n, ctypes.c_void_p) for n in ('ac', 'ascale', 'wc', 'ws', 'wr', 'wrs', 'wi', 'off', 'wloc', 'mask')] + \
               [(n, ctypes.c_int) for n in ('m', 'mp', 'n', 'k', 'na', 'hasw', 'cross', 'shared', 'dense', 'bank_blocks')]


def load_reference():
    lib = ctypes.CDLL(REF_LIB)
    lib.tw_workspace.argtypes = [ctypes.c_int] * 3; lib.tw_workspace.restype = ctypes.c_size_t
    lib.tw_fused.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p] * 8 + [ctypes.POINTER(RefIO)]; lib.tw_fused.restype = ctypes.c_int
    lib.tw_status.argtypes = [ctypes.c_int]; lib.tw_status.restype = ctypes.c_char_p
    return lib


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--m-tokens', type=int, default=7680)
    ap.add_argument('--budgets', default='1.0,1.5,2.0')
    ap.add_argument('--out', default=os.path.join(ROOT, 'gpurun_out', 'reference_sm100.json'))
    args = ap.parse_args()
    import numpy as np
    import torch
    import bench
    if not os.path.exists(REF_LIB):
        print(json.dumps({'impl': 'reference-sm100', 'unavailable': 'baseline/_ref/libtw_ref_sm100.so is not built'}))
        return
    ref = load_reference()
    dev = torch.device('cuda', 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream()
    ptr = lambda t: None if t is None else t.data_ptr()
    results = {}
    for budget in [float(b) for b in args.budgets.split(',')]:
        layers = [bench.Layer(name, n, k, args.m_tokens, budget, seed, dev) for seed, (name, n, k) in enumerate(bench.PROJECTIONS)]
        graphs, outs, flops = {}, {}, {}
        side = torch.cuda.Stream()
        for layer in layers:
            op, m = layer.op, layer.m
            layer.quantize(layer.x)
            for _ in range(2):
                layer.gemm(layer.x)
            torch.cuda.synchronize()
            flops[layer.name] = layer.issued_flops()
            pk = layer.packed
            ws_ref = torch.zeros(max(1, ref.tw_workspace(m, op.n, op.k)), device=dev, dtype=torch.uint8)
            out_ref = torch.empty(m, op.n, device=dev, dtype=torch.bfloat16)
            hasw = bool(op.hasw)
            empty_i = torch.zeros(1, device=dev, dtype=torch.int32)
            io = RefIO(ptr(pk.codes), ptr(pk.scales), ptr(op.wc), ptr(op.ws), ptr(op.wr) if hasw else ptr(op.wc),
                       ptr(op.wrs) if hasw else ptr(op.ws), ptr(op.wi) if hasw else ptr(empty_i), ptr(op.off),
                       ptr(op.wloc) if hasw else ptr(empty_i), ptr(op.am), m, pk.mp, op.n, op.k, int(op.na), int(hasw),
                       int(op.cross), 0, int(op.dense_w), int(op.wr.shape[0]) if hasw else 0)

            def call_ref(io=io, pk=pk, op=op, out_ref=out_ref, ws_ref=ws_ref, m=m):
                st = ref.tw_fused(m, op.n, op.k, pk.codes.data_ptr(), op.wc.data_ptr(), pk.scales_swz[0].data_ptr(),
                                  op.ws_swz.data_ptr(), out_ref.data_ptr(), pk.alpha.data_ptr(), ws_ref.data_ptr(),
                                  torch.cuda.current_stream().cuda_stream, ctypes.byref(io))
                if st:
                    raise RuntimeError('reference tw_fused: ' + ref.tw_status(st).decode())
            for _ in range(2):
                call_ref()
            torch.cuda.synchronize()
            ours = layer.out.float()
            theirs = out_ref.float()
            rel = float((ours - theirs).norm() / theirs.norm())
            g_ref, g_ours = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_ref, stream=side):
                call_ref()
            with torch.cuda.graph(g_ours, stream=side):
                layer.gemm(layer.x)
            graphs[layer.name] = {'reference': g_ref, 'ours': g_ours}
            outs[layer.name] = {'rel_l2_ours_vs_reference': rel, 'keep': (io, out_ref, ws_ref, empty_i)}
        ev = {layer.name: {'reference': [], 'ours': []} for layer in layers}
        for impl in ('reference', 'ours'):
            for _ in range(3):
                for layer in layers:
                    graphs[layer.name][impl].replay()
            torch.cuda.synchronize()
            torch.cuda._sleep(int(2e8))
            for _ in range(args.steps):
                for layer in layers:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    graphs[layer.name][impl].replay()
                    e1.record(stream)
                    ev[layer.name][impl].append((e0, e1))
            torch.cuda.synchronize()
        table = {}
        for layer in layers:
            row = {'issued_gflop': flops[layer.name] / 1e9, 'rel_l2_ours_vs_reference': outs[layer.name]['rel_l2_ours_vs_reference']}
            for impl in ('reference', 'ours'):
                us = float(np.median([a.elapsed_time(b) for a, b in ev[layer.name][impl]])) * 1e3
                row[impl + '_us'] = us
                row[impl + '_tflops'] = flops[layer.name] / (us * 1e-6) / 1e12
            row['speedup'] = row['reference_us'] / row['ours_us']
            table[layer.name] = row
        results[str(budget)] = table
        del layers, graphs, outs
        torch.cuda.empty_cache()
    line = {'impl': 'reference-sm100 vs ours', 'm': args.m_tokens, 'steps': args.steps, 'results': results}
    os.makedirs(os.path.dirname(args.out), exist_ok=True)
    with open(args.out, 'w') as f:
        json.dump(line, f, indent=1)
    print(json.dumps(line))


if __name__ == '__main__':
    main()
