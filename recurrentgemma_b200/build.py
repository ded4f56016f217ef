"""Builds recurrentgemma_b200/librgk.so from csrc/*.cu with nvcc for sm_100a (in-tree).

    python -m recurrentgemma_b200.build [--force] [--verbose] [--checks]

nvcc cross-compiles without a GPU.  Objects go to recurrentgemma_b200/build/, the shared library
next to the package so that ``recurrentgemma_b200._lib`` finds it.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "librgk.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
  for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
    if cand and os.path.exists(cand):
      return cand
  raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _sources():
  return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps():
  return (glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) +
          glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h")))


def _stale(target: str, inputs) -> bool:
  if not os.path.exists(target):
    return True
  t = os.path.getmtime(target)
  return any(os.path.getmtime(i) > t for i in inputs)


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool, checks: bool = False) -> str:
  cmd = [nvcc, *NVCC_FLAGS, *(["-DRGK_CHECKS"] if checks else []), "-c", src, "-o", obj]
  r = subprocess.run(cmd, capture_output=True, text=True)
  if r.returncode != 0:
    raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
  with open(obj + ".ptxas.txt", "w") as f:
    f.write(r.stderr)
  if verbose:
    sys.stderr.write(r.stderr)
  return obj


def build_library(force: bool = False, verbose: bool = False, checks: bool = False) -> str:
  """Compiles every .cu under csrc/ and links librgk.so; returns its path.  checks=True builds
  librgk_checks.so instead: the same library with -DRGK_CHECKS, in which computed indices of the
  look-back records, states and outputs are range-checked (a bad one raises the status word to -8
  and the access is skipped; nothing traps)."""
  nvcc = _nvcc()
  os.makedirs(OBJ_DIR, exist_ok=True)
  deps = _deps()
  jobs = []
  objs = []
  lib_path = LIB_PATH[:-3] + "_checks.so" if checks else LIB_PATH
  for src in _sources():
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + (".checks.o" if checks else ".o"))
    objs.append(obj)
    if force or _stale(obj, [src, *deps]):
      jobs.append((src, obj))
  with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
    for fut in [ex.submit(_compile_one, nvcc, s, o, verbose, checks) for s, o in jobs]:
      fut.result()
  if force or jobs or _stale(lib_path, objs):
    cmd = [nvcc, "-shared", "-o", lib_path, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
           "-lcudart_static"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
      raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
  return lib_path


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--force", action="store_true")
  ap.add_argument("--verbose", action="store_true")
  ap.add_argument("--checks", action="store_true",
                  help="build librgk_checks.so (-DRGK_CHECKS: range-checked indices) instead")
  args = ap.parse_args()
  print(build_library(args.force, args.verbose, args.checks))


if __name__ == "__main__":
  main()
