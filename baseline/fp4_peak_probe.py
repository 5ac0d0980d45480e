"""Dense NVFP4 GEMM peak probe: the library path (cuBLASLt through torch._scaled_mm, float4_e2m1fn_x2 operands
with E4M3 block scales in the 128x4 atom layout) at 8192^3, as a burst (best of 10) and sustained (back to
back for ~3 s, median SM clock sampled with nvidia-smi). This is the measured denominator beside the nominal
9 PFLOP/s figure; it is a baseline script, not part of the product path.

    python baseline/fp4_peak_probe.py [--size 8192] [--out FILE.json]
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def sample_clock(stop, samples):
    while not stop.is_set():
        try:
            out = subprocess.run(['nvidia-smi', '--query-gpu=clocks.sm,power.draw', '--format=csv,noheader,nounits', '-i', '0'],
                                 capture_output=True, text=True, timeout=5).stdout.strip().split(',')
            samples.append((float(out[0]), float(out[1])))
        except Exception:
            pass
        time.sleep(0.1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--size', type=int, default=8192)
    ap.add_argument('--out', default=os.path.join(ROOT, 'gpurun_out', 'fp4_peak.json'))
    args = ap.parse_args()
    import numpy as np
    import torch
    n = args.size
    line = {'probe': 'dense NVFP4 GEMM via torch._scaled_mm', 'size': n}
    try:
        torch.cuda.set_device(0)
        a = torch.randint(0, 256, (n, n // 2), device='cuda', dtype=torch.uint8).view(torch.float4_e2m1fn_x2)
        b = torch.randint(0, 256, (n, n // 2), device='cuda', dtype=torch.uint8).view(torch.float4_e2m1fn_x2)
        rows = (n + 127) // 128 * 128
        cols = (n // 16 + 3) // 4 * 4
        sa = torch.full((rows * cols,), 0.5, device='cuda').to(torch.float8_e4m3fn)
        sb = torch.full((rows * cols,), 0.5, device='cuda').to(torch.float8_e4m3fn)
        run = lambda: torch._scaled_mm(a, b.t(), sa, sb, out_dtype=torch.bfloat16)
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        flops = 2.0 * n * n * n
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); run(); e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        line['burst_tflops'] = flops / (best * 1e-3) / 1e12
        stop, samples = threading.Event(), []
        th = threading.Thread(target=sample_clock, args=(stop, samples), daemon=True); th.start()
        iters = max(10, int(3.0 / (best * 1e-3)))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            run()
        e1.record(); torch.cuda.synchronize()
        stop.set(); th.join(timeout=2)
        line['sustained_tflops'] = flops * iters / (e0.elapsed_time(e1) * 1e-3) / 1e12
        line['sustained_seconds'] = e0.elapsed_time(e1) * 1e-3
        if samples:
            line['sm_mhz_median'] = float(np.median([s[0] for s in samples]))
            line['power_w_max'] = float(max(s[1] for s in samples))
    except Exception as exc:                                    # the library path may be absent in this torch build
        line['unavailable'] = f'{type(exc).__name__}: {exc}'[:300]
    os.makedirs(os.path.dirname(args.out), exist_ok=True)
    with open(args.out, 'w') as f:
        json.dump(line, f, indent=1)
    print(json.dumps(line))


if __name__ == '__main__':
    main()
