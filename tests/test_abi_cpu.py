"""The C-ABI library without a GPU: it loads, exports every function include/twb200.h declares, its ctypes mirrors
have the layout a C compiler gives the header's structs, and the pure host entry points and the argument checks that
precede any CUDA call answer. Nothing here launches a kernel."""
import ctypes
import os
import re
import shutil
import subprocess
import pytest
from thunderworld_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, 'include', 'twb200.h')


def declared_functions():
    text = re.sub(r'/\*.*?\*/', '', open(HEADER).read(), flags=re.S)
    return sorted(set(re.findall(r'\b(tw_[a-z0-9_]+)\s*\(', text)))


def test_library_loads_and_exports_every_declared_function():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 20
    assert set(names) == set(_lib.EXPORTS)
    for name in names:
        assert hasattr(lib, name), name
    assert lib.tw_abi_version() == 3
    texts = [lib.tw_status(code) for code in range(0, 16)]
    assert all(t for t in texts) and texts[0] == b'success'
    assert lib.tw_status(12345) == b'unknown status'


def test_pure_host_entry_points():
    lib = _lib.load()
    assert lib.tw_fused_tile_n(6144) == 256 and lib.tw_fused_tile_n(384) == 128 and lib.tw_fused_tile_n(128) == 128
    assert lib.tw_workspace(7680, 6144, 2048) >= 4
    assert lib.tw_quantize_workspace(7680, 2048) >= 256 + 60 * 16 * 4
    assert lib.tw_quantize_static_max_tiles() == 16384
    assert lib.tw_attention_workspace(3840, 3840, 32, 32) >= 4


def test_null_arguments_are_refused_before_any_device_call():
    lib = _lib.load()
    assert lib.tw_quantize(None, None) != 0
    assert lib.tw_quantize(ctypes.byref(_lib.QuantizeArgs()), None) != 0
    assert lib.tw_fused(128, 128, 128, None, None, None, None, None, None, None, None, None) != 0
    assert lib.tw_pack_rows(None, None) != 0 and lib.tw_select_tiles(None, None) != 0 and lib.tw_attention(None, None) != 0
    assert lib.tw_activate(None, None, None, None, None, 0, 0, None) != 0
    assert lib.tw_rope_heads(None, None, 0, 0, 0, 0, None, None, 0, 0, 0, 0., None) != 0
    assert lib.tw_gate_residual(None, None, None, 0, 0, 0, None) != 0


STRUCTS = {'TwQuantizeArgs': _lib.QuantizeArgs, 'TwRepairIO': _lib.RepairIO, 'TwPackRowsArgs': _lib.PackRowsArgs,
           'TwSelectArgs': _lib.SelectArgs, 'TwAttentionArgs': _lib.AttentionArgs}
# ctypes field name -> header field name where they differ
RENAMED = {('TwRepairIO', 'ascale'): 'as'}


@pytest.mark.skipif(shutil.which('gcc') is None, reason='gcc not available')
def test_ctypes_mirrors_have_the_header_layout(tmp_path):
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', 'int main(void) {']
    for cname, mirror in STRUCTS.items():
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for field, _ in mirror._fields_:
            cfield = RENAMED.get((cname, field), field)
            lines.append(f'  printf("{cname} {field} %zu\\n", offsetof({cname}, {cfield}));')
    lines += ['  return 0;', '}']
    src = tmp_path / 'layout.c'
    src.write_text('\n'.join(lines))
    exe = tmp_path / 'layout'
    subprocess.run(['gcc', '-std=c11', '-o', str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    seen = 0
    for line in out.splitlines():
        cname, field, value = line.split()
        mirror = STRUCTS[cname]
        want = ctypes.sizeof(mirror) if field == 'size' else getattr(mirror, field).offset
        assert int(value) == want, line
        seen += 1
    assert seen == sum(len(m._fields_) + 1 for m in STRUCTS.values())
