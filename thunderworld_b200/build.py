"""Offline nvcc build of libtwb200.so (sm_100a only), in-tree next to this file.

Mirrors the reference's offline artifact build
(packages/fp4-repair/src/thunderworld_fp4/cutlass/build.py:31-40): a plain shared
library with a C ABI, no pybind/ATen dependency, plus a `.build.json` holding the
source and binary hashes that the loader re-checks.
"""
import hashlib
import json
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / 'csrc'
LIB = HERE / 'libtwb200.so'
META = HERE / 'libtwb200.build.json'
SOURCES = ('tw_api.cu', 'tw_quantize.cu', 'tw_fused.cu', 'tw_fused_pair.cu', 'tw_attention.cu', 'tw_pointwise.cu')
HEADERS = ('tw_common.cuh', '../../include/twb200.h')
FLAGS = ['-std=c++17', '-O3', '-lineinfo', '-gencode', 'arch=compute_100a,code=sm_100a',
         '--shared', '-Xcompiler=-fPIC', '-Xptxas=-v']


def _sha(paths):
    h = hashlib.sha256()
    for p in paths:
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def source_hash():
    files = [CSRC / s for s in SOURCES if (CSRC / s).exists()] + [(CSRC / h).resolve() for h in HEADERS]
    return _sha(files)


def nvcc_path():
    return shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'


def build(force=False, verbose=False):
    """Compile when sources changed (or `force`). Returns the library path."""
    want = source_hash()
    if not force and LIB.exists() and META.exists():
        meta = json.loads(META.read_text())
        if meta.get('sources_sha256') == want and meta.get('library_sha256') == _sha([LIB]):
            return LIB
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    cmd = [nvcc_path(), *FLAGS, '-o', str(LIB), *srcs, '-lcuda']
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode:
        print(proc.stdout, proc.stderr)
    if proc.returncode:
        raise RuntimeError('nvcc failed:\n' + proc.stderr[-4000:])
    (HERE / 'libtwb200.ptxas.txt').write_text(proc.stderr)
    META.write_text(json.dumps({'backend': 'twb200-sm100a', 'sources_sha256': want,
                                'library_sha256': _sha([LIB]), 'flags': FLAGS}, indent=1))
    return LIB


if __name__ == '__main__':
    import sys
    print(build(force='--force' in sys.argv, verbose=True))
