"""In-tree build of liblewi_moe.so for sm_100a (explicit nvcc; the .so lands next to this file)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "lewi_moe.cu")
OUT = os.path.join(HERE, "liblewi_moe.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _sources():
  csrc = os.path.join(HERE, "csrc")
  inc = os.path.join(os.path.dirname(HERE), "include")
  files = [os.path.join(csrc, f) for f in sorted(os.listdir(csrc))]
  files += [os.path.join(inc, f) for f in sorted(os.listdir(inc))]
  return files


def is_stale():
  if not os.path.exists(OUT):
    return True
  t = os.path.getmtime(OUT)
  return any(os.path.getmtime(f) > t for f in _sources())


def build(force=False, verbose=False):
  """Compile the CUDA library if it is missing or older than its sources.  Returns the .so path."""
  if not force and not is_stale():
    return OUT
  nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
  cmd = [nvcc, *NVCC_FLAGS, "-o", OUT, SRC]
  if verbose:
    cmd.insert(1, "-Xptxas")
    cmd.insert(2, "-v")
  res = subprocess.run(cmd, capture_output=True, text=True)
  if res.returncode != 0:
    raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
  if verbose:
    print(res.stderr)
  return OUT


if __name__ == "__main__":
  print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
