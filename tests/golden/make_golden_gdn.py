"""Generates tests/golden/gdn_chunk.npz by RUNNING the reference's chunked gated delta rule.

  python tests/golden/make_golden_gdn.py /path/to/reference

`fast_chunk_gated_delta_rule` and `_inv_unit_lower` (modal/gdn_fast.py:21-113) are taken out of the parsed source
with `ast` (the module itself imports JAX at its top) and executed over NumPy stand-ins for the `jnp` / `lax` names
they use.  The stand-ins keep JAX's dtype rules where they matter: a product of two bfloat16 arrays is accumulated in
float32 and rounded to bfloat16, `lax.scan` threads the carry and stacks the per-step outputs.  Nothing is copied.
"""
import ast
import os
import sys
import types

import ml_dtypes
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BF16 = ml_dtypes.bfloat16


def bf16_round(a):
  return np.asarray(a, np.float32).astype(BF16).astype(np.float32)


def _matmul(a, b, precision=None):
  a, b = np.asarray(a), np.asarray(b)
  if a.dtype == BF16 and b.dtype == BF16:
    return (a.astype(np.float32) @ b.astype(np.float32)).astype(BF16)
  return a.astype(np.float32) @ b.astype(np.float32)


def _solve_triangular(a, b, lower=True, unit_diagonal=True):
  return np.linalg.solve(np.asarray(a, np.float64), np.asarray(b, np.float64)).astype(np.float32)


def _scan(body, init, xs, unroll=1):
  carry, outs = init, []
  for i in range(xs[0].shape[0]):
    carry, o = body(carry, tuple(x[i] for x in xs))
    outs.append(o)
  return carry, np.stack(outs)


def namespace():
  jnp = types.SimpleNamespace(
      eye=np.eye, broadcast_to=np.broadcast_to, matmul=_matmul, float32=np.float32, bfloat16=BF16, array=np.array,
      pad=np.pad, cumsum=np.cumsum, tril=np.tril, ones=np.ones, where=np.where, exp=np.exp, zeros=np.zeros)
  lax = types.SimpleNamespace(rsqrt=lambda x: (1.0 / np.sqrt(x)).astype(np.float32), scan=_scan)
  jax = types.SimpleNamespace(lax=lax, scipy=types.SimpleNamespace(linalg=types.SimpleNamespace(solve_triangular=_solve_triangular)))
  return dict(jax=jax, jnp=jnp, lax=lax, PREC=None, UNROLL=1, _orig=None)


def main(ref_root):
  path = os.path.join(ref_root, "modal", "gdn_fast.py")
  tree = ast.parse(open(path).read())
  keep = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in ("_inv_unit_lower", "fast_chunk_gated_delta_rule")]
  rng = np.random.default_rng(123)
  out = {}
  for name, (b, s, h, kd, vd, with_state) in {"a": (2, 150, 2, 64, 64, False), "b": (1, 128, 3, 32, 64, True)}.items():
    n = lambda *shape: rng.standard_normal(shape).astype(np.float32)
    q, k, v = bf16_round(n(b, s, h, kd)), bf16_round(n(b, s, h, kd) / np.sqrt(kd) * 2), bf16_round(n(b, s, h, vd))
    g = -np.abs(n(b, s, h)) * 0.3                              # log-decay, never positive
    beta = bf16_round(1 / (1 + np.exp(-n(b, s, h))))           # write strength in (0, 1)
    h0 = bf16_round(n(b, h, kd, vd) * 0.1) if with_state else None
    res = {}
    for inv in ("solve", "neumann"):
      ns = namespace()
      ns["INV"] = inv
      exec(compile(ast.Module(body=keep, type_ignores=[]), path, "exec"), ns)
      o, hf = ns["fast_chunk_gated_delta_rule"](q.astype(BF16), k.astype(BF16), v.astype(BF16), g, beta.astype(BF16),
                                                chunk_size=64, initial_state=h0, compute_dtype=BF16)
      res[inv] = (np.asarray(o, np.float32), None if hf is None else np.asarray(hf, np.float32))
    assert np.abs(res["solve"][0] - res["neumann"][0]).max() <= 2e-2 * np.abs(res["solve"][0]).max()
    out.update({f"{name}_q": q, f"{name}_k": k, f"{name}_v": v, f"{name}_g": g, f"{name}_beta": beta,
                f"{name}_o": res["solve"][0], f"{name}_o_neumann": res["neumann"][0]})
    if with_state:
      out.update({f"{name}_h0": h0, f"{name}_h_final": res["solve"][1]})
  np.savez_compressed(os.path.join(HERE, "gdn_chunk.npz"), **out)
  print("wrote gdn_chunk.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
  if len(sys.argv) != 2:
    raise SystemExit("usage: python tests/golden/make_golden_gdn.py <path to a checkout of the reference repository>")
  main(sys.argv[1])
