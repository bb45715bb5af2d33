"""The jax.ffi shim without JAX: its XLA-free core compiles and links against the library (so every call matches
include/lewi_moe.h), the handler layer type-checks against a stand-in of jaxlib's FFI header (handler signatures equal
their bindings), and the Python side names exactly the handlers the C++ side defines."""
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "lewi_surge_b200", "csrc")
GXX = shutil.which("g++")
CUDA_INC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")


@pytest.mark.skipif(GXX is None, reason="no g++")
def test_xla_free_core_compiles_and_links(tmp_path):
  from lewi_surge_b200 import build
  build.build()
  out = tmp_path / "libffi_core.so"
  res = subprocess.run([GXX, "-std=c++17", "-Wall", "-Werror", "-shared", "-fPIC", os.path.join(CSRC, "ffi_core.cc"),
                        "-L" + os.path.join(ROOT, "lewi_surge_b200"), "-llewi_moe", "-Wl,--no-undefined", "-o", str(out)],
                       capture_output=True, text=True)
  assert res.returncode == 0, res.stderr
  syms = subprocess.run(["nm", "-D", "--defined-only", str(out)], capture_output=True, text=True).stdout
  for name in ("sort_indices", "gather_rows", "ragged_dot_fwd", "ragged_dot_dlhs", "ragged_dot_drhs", "moe_fwd", "moe_bwd",
               "causal_conv1d_fwd", "causal_conv1d_bwd", "gdn_chunk_fwd", "gdn_chunk_bwd"):
    assert re.search(rf"lewi_ffi\d+{name}", syms), name


@pytest.mark.skipif(GXX is None or not os.path.exists(os.path.join(CUDA_INC, "cuda_runtime.h")), reason="no g++ / CUDA headers")
def test_handler_layer_type_checks_against_the_stand_in_header():
  res = subprocess.run([GXX, "-std=c++17", "-fsyntax-only", "-I" + os.path.join(ROOT, "tests", "stubs"), "-I" + CUDA_INC,
                        os.path.join(CSRC, "ffi_xla.cc")], capture_output=True, text=True)
  assert res.returncode == 0, res.stderr


def test_python_side_registers_the_handlers_the_cxx_side_defines():
  from lewi_surge_b200 import jax_ops
  src = open(os.path.join(CSRC, "ffi_xla.cc")).read()
  defined = re.findall(r"XLA_FFI_DEFINE_HANDLER_SYMBOL\((lewi_ffi_[a-z0-9_]+),", src)
  assert sorted(defined) == sorted(jax_ops._TARGETS)
  used = set(re.findall(r'ffi_call\(\s*"(lewi_ffi_[a-z0-9_]+)"', open(jax_ops.__file__).read()))
  assert used == set(defined)


def test_jax_ops_imports_without_jax_and_fails_loudly_when_used():
  from lewi_surge_b200 import jax_ops
  try:
    import jax  # noqa: F401
    pytest.skip("JAX is installed here")
  except ImportError:
    pass
  with pytest.raises(ImportError):
    jax_ops.install(num_experts=64)
