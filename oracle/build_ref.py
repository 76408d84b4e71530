"""Compiles the reference's OWN CUDA kernels, from the sources where they lie
in a mounted mamba-rs tree, into oracle/_ref/*.cubin (checker only, never part
of the product; oracle/_ref/ is git-ignored).  The reference builds these files
with NVRTC at run time (src/mamba_ssm/gpu/kernels.rs:451-545, options
--fmad=true --extra-device-vectorization); here nvcc does the same offline for
sm_100a.  No reference source is copied into this repository.

    python oracle/build_ref.py /path/to/mamba-rs      (or MAMBA_RS_REFERENCE=/path/to/mamba-rs)
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
ENV_REF = "MAMBA_RS_REFERENCE"
FILES = ["mamba_ssm_parallel.cu", "mamba_ssm.cu", "conv1d.cu", "mamba3_chunked.cu", "mamba3_ssd.cu", "mamba3_ops.cu"]


def build_ref(ref_root: str = "", verbose: bool = False) -> bool:
    """ref_root: the mounted mamba-rs tree; empty = the MAMBA_RS_REFERENCE environment
    variable; nothing is built when neither names a tree."""
    ref_root = ref_root or os.environ.get(ENV_REF, "")
    kdir = os.path.join(ref_root, "kernels")
    if not ref_root or not os.path.isdir(kdir):
        if verbose:
            print(f"no reference tree at {ref_root!r}: oracle/_ref not built")
        return False
    os.makedirs(OUT, exist_ok=True)
    procs = []
    for f in FILES:
        src = os.path.join(kdir, f)
        dst = os.path.join(OUT, f.replace(".cu", ".cubin"))
        if os.path.exists(dst) and os.path.getmtime(dst) >= os.path.getmtime(src):
            continue
        cmd = ["nvcc", "-cubin", "-gencode", "arch=compute_100a,code=sm_100a", "--fmad=true",
               "-extra-device-vectorization", "-O3", "-I", kdir,
               # the reference prepends the typed prelude to every module before NVRTC
               # (src/mamba_ssm/gpu/kernels.rs:455-480)
               "-include", os.path.join(kdir, "_typed_prelude.cuh"), "-o", dst, src]
        procs.append((f, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    ok = True
    for f, p in procs:
        out, _ = p.communicate()
        if p.returncode:
            ok = False
            sys.stderr.write(f"reference kernel {f} did not compile:\n{out.decode()[:2000]}\n")
    return ok


if __name__ == "__main__":
    build_ref(sys.argv[1] if len(sys.argv) > 1 else "", verbose=True)
    print(sorted(os.listdir(OUT)) if os.path.isdir(OUT) else "nothing built")
