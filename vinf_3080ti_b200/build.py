"""Builds libvinf_b200.so (the C-ABI library) for sm_100a with nvcc, in-tree.

    python -m vinf_3080ti_b200.build [--force] [--jobs N] [--define NAME[=VALUE] ...] [--out PATH]

--define passes -DNAME[=VALUE] to every translation unit: the kernels' experiment switches (VQM_ABLATE_STEP: the matvec
pipeline without the decoders; VQM_PURE_COMPUTE: the decoders without copies and waits; VQM_NO_SCALE_PASS / VQM_NO_DOT:
without one of the two passes of the tuned K-quant decoders; VQM_TC5_ABLATE=<bits>: the prompt GEMM without decode /
activation copies / proxy fence / everything but the MMA loop) give the ablation timings quoted in profiles/; their
results are wrong on purpose.  VQM_TC5_SHAPE=<n> selects another block shape of the prompt GEMM (results stay right).
Such a build goes to --out (objects beside it) and is loaded with VINF_B200_LIB=<path>.

Two translation units per GGUF type (the matvec kernel instantiations, plain and with the fused prologues) plus the small kernels and the
runtime; objects go to csrc/build/, the library next to this file.  Cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = CSRC / "build"
LIB = HERE / "libvinf_b200.so"

TYPES = [(0, "F32"), (1, "F16"), (8, "Q8_0"), (10, "Q2_K"), (11, "Q3_K"), (12, "Q4_K"), (13, "Q5_K"), (14, "Q6_K"),
         (16, "IQ2_XXS"), (17, "IQ2_XS"), (18, "IQ3_XXS"), (20, "IQ4_NL"), (21, "IQ3_S"), (22, "IQ2_S"), (23, "IQ4_XS")]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return found


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) +
                  [HERE.parent / "include" / "vinf_b200.h"])


def up_to_date() -> bool:
    if not LIB.exists():
        return False
    built = LIB.stat().st_mtime
    return all(src.stat().st_mtime <= built for src in _sources())


EXTRA_DEFINES: list[str] = []


def _compile(job: tuple[str, list[str], Path]) -> tuple[str, str]:
    name, extra, obj = job
    src = CSRC / name
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, *EXTRA_DEFINES, "-c", str(src), "-o", str(obj)]
    env = dict(os.environ)
    env.pop("CC", None)  # nvcc picks its host compiler from PATH
    env.pop("CXX", None)
    done = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if done.returncode != 0:
        raise RuntimeError(f"nvcc failed for {name} {extra}:\n{done.stdout}\n{done.stderr}")
    return obj.name, done.stdout + done.stderr


def build(force: bool = False, jobs: int | None = None, verbose: bool = False, defines: list[str] | None = None, out: Path | None = None) -> Path:
    global OBJ, LIB
    if defines or out:
        if out is None:
            raise ValueError("an experimental build (--define) needs --out, it must not replace the library")
        LIB = Path(out).resolve()
        OBJ = LIB.parent / (LIB.stem + "_obj")
        EXTRA_DEFINES[:] = [f"-D{d}" for d in (defines or [])]
        force = True
    if not force and up_to_date():
        return LIB
    OBJ.mkdir(parents=True, exist_ok=True)
    work: list[tuple[str, list[str], Path]] = [
        ("vqm_matvec_type.cu", [f"-DVQM_TYPE={tid}", f"-DVQM_TYPE_NAME={tname}"], OBJ / f"matvec_{tname}.o")
        for tid, tname in TYPES
    ]
    # the same kernels with the fused prologues / residual add compiled in (vqm_qmv_fused)
    work += [("vqm_matvec_type.cu", [f"-DVQM_TYPE={tid}", f"-DVQM_TYPE_NAME={tname}", "-DVQM_FUSED=1"], OBJ / f"matvec_fused_{tname}.o")
             for tid, tname in TYPES]
    work.append(("vqm_aux.cu", [], OBJ / "aux.o"))
    work.append(("vqm_probe.cu", [], OBJ / "probe.o"))
    work.append(("vqm_gemm.cu", [], OBJ / "gemm.o"))
    work.append(("vqm_gemm_tc5.cu", [], OBJ / "gemm_tc5.o"))
    work.append(("vqm_runtime.cu", [], OBJ / "runtime.o"))
    jobs = jobs or min(len(work), os.cpu_count() or 4)
    logs = []
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        for name, log in pool.map(_compile, work):
            logs.append(f"== {name}\n{log}")
    (OBJ / "ptxas.log").write_text("\n".join(logs))
    if verbose:
        print("\n".join(logs))
    cmd = [_nvcc(), "-shared", "-o", str(LIB), *[str(obj) for _, _, obj in work]]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    done = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if done.returncode != 0:
        raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--define", action="append", default=[], metavar="NAME[=VALUE]")
    ap.add_argument("--out", default=None)
    ns = ap.parse_args()
    print(build(ns.force, ns.jobs, ns.verbose, ns.define, ns.out))
    sys.exit(0)
