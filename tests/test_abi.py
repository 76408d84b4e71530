"""CPU checks of the drop-in boundary: the shared library loads without a GPU
and exports every symbol include/mamba_b200.h declares; the ctypes argument
struct matches the C layout; compute calls refuse to run without CUDA."""
import ctypes
import os
import re
import subprocess
import tempfile

import pytest

import mamba_rs_b200 as mb
from mamba_rs_b200 import ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "mamba_b200.h")


def declared_symbols():
    src = open(HEADER).read()
    return sorted(set(re.findall(r"MAMBA_B200_API\s+[\w\s\*]+?\b(mamba_b200_\w+)\s*\(", src)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for s in ("mamba_b200_init", "mamba_b200_destroy", "mamba_b200_last_error",
              "mamba_b200_sscan_fwd", "mamba_b200_ssm_scan_fwd_nosave"):
        assert s in syms


def test_library_exports_every_declared_symbol():
    lib = ffi.lib()
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} declared in the header but not exported"


def test_args_struct_matches_c_layout():
    """Compile a tiny C program against the header and compare sizeof/offsetof
    with the ctypes Structure (what a Rust #[repr(C)] mirror must also match)."""
    structs = {"mamba_b200_sscan_fwd_args": ffi.SscanFwdArgs}
    for extra in ("mamba_b200_sscan_bwd_args", "mamba_b200_sscan_step_args",
                  "mamba_b200_conv1d_args", "mamba_b200_m3_ssd_args", "mamba_b200_m3_ssd_bwd_args"):
        cls = getattr(ffi, "".join(p.capitalize() for p in extra.replace("mamba_b200_", "").split("_")), None)
        if cls is not None and extra in open(HEADER).read():
            structs[extra] = cls
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void){"]
    for cname, cls in structs.items():
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            lines.append(f'printf("{cname}.{fname} %zu\\n", offsetof({cname}, {fname}));')
    lines.append("return 0;}")
    with tempfile.TemporaryDirectory() as td:
        src = os.path.join(td, "t.c")
        open(src, "w").write("\n".join(lines))
        exe = os.path.join(td, "t")
        subprocess.check_call(["gcc", "-std=c11", "-o", exe, src])
        out = subprocess.check_output([exe]).decode().split("\n")
    got = dict(l.rsplit(" ", 1) for l in out if l)
    for cname, cls in structs.items():
        assert int(got[cname]) == ctypes.sizeof(cls), cname
        for fname, _ in cls._fields_:
            assert int(got[f"{cname}.{fname}"]) == getattr(cls, fname).offset, (cname, fname)


def test_compute_refuses_cpu_tensors():
    import torch
    x = torch.zeros(1, 4, 8)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        mb.selective_scan_fwd(x, x, torch.zeros(1, 4, 4), torch.zeros(1, 4, 4), torch.zeros(8, 4),
                              torch.zeros(8))


def test_init_fails_loudly_without_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(RuntimeError, match="mamba_b200_init"):
        ffi.Handle(0)
