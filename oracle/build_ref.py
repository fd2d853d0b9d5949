"""Build the unmodified reference CUDA extensions for sm_100 into ``oracle/_ref/`` (test infrastructure).

The reference ships no sm_100 build: its ``setup.py`` rejects every architecture outside
{8.0, 8.6, 8.7, 8.9, 9.0} (setup.py:52,105-112) and wants a visible GPU (setup.py:123-137).
Nothing in its CUDA sources is architecture-locked, though: the sm80 / sm89 ``mma.sync`` kernels
compile for ``compute_100``. This recipe therefore leaves ``setup.py`` alone and compiles the
reference's own translation units, from where they lie, with the flags of setup.py:56-66 and the
one ``-gencode`` pair that setup.py:154-165 would have produced for a 10.0 device:

    csrc/qattn/pybind.cpp, qk_int_sv_f16_cuda_sm80.cu, qk_int_sv_f8_cuda_sm89.cu
    + the explicit instantiations written by instantiations_sm80|sm89/autogen.py  -> _qattn
    csrc/fused/pybind.cpp, fused.cu                                               -> _fused

(the sm90 ``wgmma`` kernel is left out exactly as setup.py leaves it out without a 9.0 device).
The instantiation generators write next to themselves, so they are run from a scratch copy.
The reference's Python package is copied beside the two built modules so that
``sys.path.insert(0, "oracle/_ref"); import spas_sage_attn`` gives the reference API on a machine
that has no reference checkout. Everything lands under ``oracle/_ref/`` (git-ignored).

Only tests, the golden-fixture generator and the benchmark's reference leg may use the result;
the product never imports it.

Usage:  python oracle/build_ref.py [--reference /path/to/SpargeAttn] [--jobs 8]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"


def sh(cmd: list[str], log: Path) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        log.write_text(" ".join(cmd) + "\n" + r.stdout)
        raise RuntimeError(f"failed: {' '.join(cmd[:3])} ... see {log}\n{r.stdout[-2000:]}")


def build(reference: Path, jobs: int) -> Path:
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    csrc = reference / "csrc"
    gen = OUT / "gen"
    obj = OUT / "obj"
    pkg = OUT / "spas_sage_attn"
    for d in (gen, obj, pkg):
        d.mkdir(parents=True, exist_ok=True)

    # explicit template instantiations (setup.py:172-174), generated in a scratch copy
    inst: list[tuple[Path, Path]] = []
    for arch in ("sm80", "sm89"):
        src_dir = csrc / "qattn" / f"instantiations_{arch}"
        dst_dir = gen / f"instantiations_{arch}"
        dst_dir.mkdir(exist_ok=True)
        shutil.copy(src_dir / "autogen.py", dst_dir / "autogen.py")
        subprocess.run([sys.executable, str(dst_dir / "autogen.py")], check=True, stdout=subprocess.DEVNULL)
        # the generated files include "../<kernel>.cuh": resolved through -I <reference dir of the generator>
        inst += [(p, src_dir) for p in sorted(dst_dir.glob("*.cu"))]

    abi = 1 if torch._C._GLIBCXX_USE_CXX11_ABI else 0
    tinc = [f"-I{p}" for p in include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    nvcc = ["nvcc", "-O3", "-std=c++17", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
            "--use_fast_math", "-diag-suppress=174", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
            "-gencode", "arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC", f"-I{csrc}"]
    cxx = ["g++", "-O3", "-std=c++17", "-fPIC", "-fopenmp", "-DENABLE_BF16", "-DSAGE2PP_ENABLED", "-w",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-I{csrc}", "-I/usr/local/cuda/include"]

    tasks: list[tuple[list[str], Path]] = []

    def add(src: Path, name: str, module: str, extra: list[str]) -> Path:
        o = obj / (name + ".o")
        if not o.exists() or o.stat().st_mtime < src.stat().st_mtime:
            base = cxx if src.suffix == ".cpp" else nvcc
            tasks.append((base + tinc + extra + [f"-DTORCH_EXTENSION_NAME={module}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                                                 "-c", str(src), "-o", str(o)], o))
        return o

    q_objs = [add(csrc / "qattn" / "pybind.cpp", "qattn_pybind", "_qattn", []),
              add(csrc / "qattn" / "qk_int_sv_f16_cuda_sm80.cu", "qattn_sm80_host", "_qattn", []),
              add(csrc / "qattn" / "qk_int_sv_f8_cuda_sm89.cu", "qattn_sm89_host", "_qattn", [])]
    q_objs += [add(p, p.parent.name + "_" + p.stem, "_qattn", [f"-I{inc}"]) for p, inc in inst]
    f_objs = [add(csrc / "fused" / "pybind.cpp", "fused_pybind", "_fused", []),
              add(csrc / "fused" / "fused.cu", "fused_cu", "_fused", [])]

    print(f"compiling {len(tasks)} translation units with {jobs} jobs", flush=True)
    with ThreadPoolExecutor(jobs) as ex:
        list(ex.map(lambda t: sh(t[0], t[1].with_suffix(".log")), tasks))

    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    libs = [f"-L{p}" for p in library_paths("cuda")] + ["-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python",
                                                         "-lc10_cuda", "-ltorch_cuda", "-lcudart", "-lcuda", "-lgomp"]
    for name, objs in (("_qattn", q_objs), ("_fused", f_objs)):
        sh(["g++", "-shared", "-o", str(pkg / (name + suffix))] + [str(o) for o in objs] + libs, obj / (name + ".link.log"))
    for py in (reference / "spas_sage_attn").glob("*.py"):
        dst = pkg / py.name
        if dst.exists():
            dst.chmod(0o644)
        shutil.copyfile(py, dst)
    return pkg


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 8)
    a = ap.parse_args()
    ref = Path(a.reference)
    if not (ref / "csrc" / "qattn").is_dir():
        print(f"no reference checkout at {ref}: nothing built")
        return
    print("built", build(ref, a.jobs))


if __name__ == "__main__":
    main()
