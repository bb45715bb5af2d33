"""Generates tests/golden/causal_conv.npz by RUNNING the reference's shift-add convolution.

  python tests/golden/make_golden_seqmix.py /path/to/reference

`_fast_call` (modal/fast_conv.py:14-31) is a method patched onto flax's `nnx.Conv`; flax is not installable here, so
the function definition alone is taken out of the parsed source with `ast` and executed with the NumPy stand-in for
`jax.numpy` (jax_numpy_shim.py) and a plain object carrying the attributes the function reads.  Nothing is copied.
"""
import ast
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import jax_numpy_shim  # noqa: E402


def bf16_round(a):
  u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
  return ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32).reshape(a.shape)


def main(ref_root):
  jax = jax_numpy_shim.install()
  path = os.path.join(ref_root, "modal", "fast_conv.py")
  tree = ast.parse(open(path).read())
  fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "_fast_call"]
  ns = {"jnp": jax.numpy, "_orig_call": None}
  exec(compile(ast.Module(body=fn, type_ignores=[]), path, "exec"), ns)
  rng = np.random.default_rng(77)
  out = {}
  for name, (b, t, c, k) in {"a": (2, 50, 64, 4), "b": (1, 33, 16, 3)}.items():
    x = bf16_round(rng.standard_normal((b, t, c)).astype(np.float32))
    w = bf16_round((rng.standard_normal((k, 1, c)) * 0.5).astype(np.float32))
    conv = types.SimpleNamespace(kernel_size=(k,), feature_group_count=c, in_features=c, out_features=c, padding="CAUSAL",
                                 bias=None, kernel_dilation=1, strides=1, dtype=np.float32,
                                 kernel=types.SimpleNamespace(value=w.view(jax_numpy_shim.Arr)))
    y = ns["_fast_call"](conv, x.view(jax_numpy_shim.Arr))
    out.update({f"{name}_x": x, f"{name}_w": w, f"{name}_y": np.asarray(y, np.float32)})
  np.savez_compressed(os.path.join(HERE, "causal_conv.npz"), **out)
  print("wrote causal_conv.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
  if len(sys.argv) != 2:
    raise SystemExit("usage: python tests/golden/make_golden_seqmix.py <path to a checkout of the reference repository>")
  main(sys.argv[1])
