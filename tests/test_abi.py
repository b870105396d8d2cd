"""The C-ABI library loads, exports every symbol include/miniattn.h declares, its parameter
block has the layout the ctypes mirror assumes, and argument validation rejects bad calls
before anything touches the GPU.  Runs without a CUDA device."""
import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "miniattn.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(miniattn_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = declared_functions()
    assert "miniattn_fwd" in names and "miniattn_last_error_string" in names


def test_library_exports_every_declared_symbol():
    from miniattn import _lib
    for name in declared_functions():
        assert hasattr(_lib.lib, name), f"{name} declared in miniattn.h but not exported"


def test_version_string():
    import miniattn
    assert "sm_100a" in miniattn.version()


def test_struct_layouts_match_c(tmp_path):
    """Compile the header as plain C and compare sizeof/offsetof of every struct with its ctypes mirror."""
    from miniattn import _lib
    pairs = [("MiniAttnFwdParams", _lib.FwdParams), ("MiniAttnInt8Params", _lib.Int8Params),
             ("MiniAttnMergeParams", _lib.MergeParams), ("MiniAttnPlanInfo", _lib.PlanInfo),
             ("MiniAttnPlanPiece", _lib.PlanPiece)]
    src = tmp_path / "layout.c"
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void){"]
    for cname, mirror in pairs:
        lines.append(f'printf("%zu\\n", sizeof({cname}));')
        for f in mirror._fields_:
            lines.append(f'printf("%zu\\n", offsetof({cname}, {f[0]}));')
    lines.append("return 0;}")
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", str(src), "-o", str(exe)], check=True)
    out = iter(subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split())
    for cname, mirror in pairs:
        assert int(next(out)) == C.sizeof(mirror), cname
        for f in mirror._fields_:
            assert int(next(out)) == getattr(mirror, f[0]).offset, (cname, f[0])


def _params(**kw):
    from miniattn import _lib
    p = _lib.FwdParams()
    p.q = p.k = p.v = p.o = 0x1000  # never dereferenced: validation fails first
    p.B, p.Hq, p.Hkv, p.Nq, p.Nk, p.D = 1, 2, 2, 128, 128, 128
    for s in (p.q_stride, p.k_stride, p.v_stride, p.o_stride):
        s[:] = (2 * 128 * 128, 128 * 128, 128)
    for k, v in kw.items():
        if isinstance(v, tuple):
            getattr(p, k)[:] = v
        else:
            setattr(p, k, v)
    return p


@pytest.mark.parametrize(
    "kw, code, text",
    [
        (dict(dtype=7), -2, "dtype"),
        (dict(D=80), -2, "head dim"),
        (dict(carry_in=1), -1, "carry is null"),
        (dict(carry_out=1, carry=0x1010), -1, "256-byte aligned"),
        (dict(carry_out=1, carry=0x1000, kernel=1), -2, "warp-specialised"),
        (dict(carry_in=3, carry=0x1000), -1, "0 or 1"),
        (dict(carry_out=1, carry=0x1000, carry_tile0=1), -1, "exceed carry_tiles"),
        (dict(carry_out=1, carry=0x1000, carry_tile0=2, carry_tiles=2), -1, "exceed carry_tiles"),
        (dict(Nq=-1), -1, "negative"),
        (dict(Hkv=3), -1, "multiple of Hkv"),
        (dict(causal=2), -1, "causal"),
        (dict(kernel=9), -1, "kernel"),
        (dict(q=0), -1, "q is null"),
        (dict(o=0x1004), -1, "aligned"),
        (dict(k_stride=(128 * 128, 128 * 128, 130)), -1, "multiple of 8"),
        (dict(v_stride=(128 * 128, 128 * 128, 64)), -1, "smaller than D"),
    ],
)
def test_validation_rejects(kw, code, text):
    from miniattn import _lib
    rc = _lib.lib.miniattn_fwd(C.byref(_params(**kw)), None)
    assert rc == code
    assert text in _lib.last_error()


def test_null_params_and_empty_problem():
    from miniattn import _lib
    assert _lib.lib.miniattn_fwd(None, None) == -1
    assert _lib.lib.miniattn_fwd(C.byref(_params(B=0)), None) == 0   # empty output: no launch
    assert _lib.lib.miniattn_fwd(C.byref(_params(Nq=0)), None) == 0
    assert _lib.last_error() == ""


def test_python_surface_rejects_bad_tensors():
    """Mirrors the reference launcher's TORCH_CHECKs (flash_attention.cu:41-80): RuntimeError."""
    import torch
    import miniattn
    q = torch.zeros(1, 2, 128, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        miniattn.flash_attn_fwd(q, q, q)
    with pytest.raises(RuntimeError, match="layout"):
        miniattn.flash_attn_fwd(q, q, q, layout="hbnd")


def test_selftest_rejects_bad_limit():
    from miniattn import _lib
    assert _lib.lib.miniattn_selftest_wait(None, 1000, None) == -1
    assert _lib.lib.miniattn_selftest_wait(0x1000, 0, None) == -1


def test_check_status_names_the_waits():
    from miniattn import _lib
    assert _lib.lib.miniattn_check_status(0) == 0 and _lib.last_error() == ""
    assert _lib.lib.miniattn_check_status((1 << 6) | 1) == _lib.EDEVICE_WAIT
    assert "another CTA" in _lib.last_error() and "tile load" in _lib.last_error()
    assert _lib.lib.miniattn_check_status(1 << 30) == _lib.EDEVICE_WAIT and "self-test" in _lib.last_error()


def test_carry_bytes():
    from miniattn import _lib
    p = _params(Nq=300, D=96)          # 3 Q tiles x 2 heads, state kept at the kernel's head dim 128
    assert _lib.lib.miniattn_fwd_carry_bytes(C.byref(p)) == 1 * 2 * 3 * 128 * (128 * 4 + 8)
    assert _lib.lib.miniattn_fwd_carry_bytes(C.byref(_params(D=80))) == -2
