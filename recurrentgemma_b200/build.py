"""Builds recurrentgemma_b200/librgk.so from csrc/*.cu with nvcc for sm_100a (in-tree).

    python -m recurrentgemma_b200.build [--force] [--verbose]

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


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool) -> str:
  cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
  r = subprocess.run(cmd, capture_output=True, text=True)
  if r.returncode != 0:
    raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
  with open(obj + ".ptxas.txt", "w") as f:
    f.write(r.stderr)
  if verbose:
    sys.stderr.write(r.stderr)
  return obj


def build_library(force: bool = False, verbose: bool = False) -> str:
  """Compiles every .cu under csrc/ and links librgk.so; returns its path."""
  nvcc = _nvcc()
  os.makedirs(OBJ_DIR, exist_ok=True)
  deps = _deps()
  jobs = []
  objs = []
  for src in _sources():
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    objs.append(obj)
    if force or _stale(obj, [src, *deps]):
      jobs.append((src, obj))
  with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
    for fut in [ex.submit(_compile_one, nvcc, s, o, verbose) for s, o in jobs]:
      fut.result()
  if force or jobs or _stale(LIB_PATH, objs):
    cmd = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
           "-lcudart_static"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
      raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
  return LIB_PATH


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--force", action="store_true")
  ap.add_argument("--verbose", action="store_true")
  args = ap.parse_args()
  print(build_library(args.force, args.verbose))


if __name__ == "__main__":
  main()
