"""Build recipe for the "reference-sm100" baseline: the reference project's own tcgen05 fused repair GEMM
(tools/thor_handoff/cutlass_sm110_fused.cu + sm110_repair_collective.cuh, CUTLASS arch::Sm100 collectives),
compiled unmodified for sm_100a from the sources where they lie in the reference checkout.

    python baseline/build_reference_sm100.py [reference_root]

Output: baseline/_ref/libtw_ref_sm100.so (git-ignored; exports tw_workspace, tw_fused, tw_status with the
reference's RepairIO). Needs the CUTLASS headers vendored by the flashinfer package, the same header source
the reference's own build script uses (packages/fp4-repair/src/thunderworld_fp4/cutlass/build.py:23-27).
Baseline harness only: the product library never links or loads it. Single-GPU use only.
"""
import hashlib
import json
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / '_ref' / 'libtw_ref_sm100.so'


def cutlass_include():
    import flashinfer
    root = Path(flashinfer.__file__).resolve().parent / 'data' / 'cutlass'
    return [root / 'include', root / 'tools' / 'util' / 'include']


def build(reference_root='/root/reference'):
    src = Path(reference_root) / 'tools' / 'thor_handoff' / 'cutlass_sm110_fused.cu'
    if not src.exists():
        raise FileNotFoundError(f'{src}: the reference checkout is needed to build this baseline')
    OUT.parent.mkdir(parents=True, exist_ok=True)
    nvcc = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    cmd = [nvcc, '-std=c++17', '-O3', '--expt-relaxed-constexpr', '--expt-extended-lambda',
           '-gencode', 'arch=compute_100a,code=sm_100a', '--shared', '-Xcompiler=-fPIC',
           *[f'-I{p}' for p in cutlass_include()], f'-I{src.parent}', '-o', str(OUT), str(src)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode:
        raise RuntimeError(proc.stderr[-4000:])
    meta = {'backend': 'reference cutlass-sm110-fused-mainloop compiled for sm_100a', 'tile': [128, 128, 128],
            'source_sha256': hashlib.sha256(src.read_bytes()).hexdigest(),
            'collective_sha256': hashlib.sha256((src.parent / 'sm110_repair_collective.cuh').read_bytes()).hexdigest(),
            'library_sha256': hashlib.sha256(OUT.read_bytes()).hexdigest()}
    OUT.with_suffix('.build.json').write_text(json.dumps(meta, indent=1))
    return OUT


if __name__ == '__main__':
    print(build(*sys.argv[1:2]))
