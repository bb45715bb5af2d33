"""Generates tests/golden/*.npz by RUNNING the reference's own pure-array MoE code.

  python tests/golden/make_golden.py /path/to/reference

The reference's `modal/moe_permute.py` and `modal/padded_gmm.py` are imported from the reference tree
(never copied) under the NumPy stand-in of `jax_numpy_shim.py`, because real JAX is not installable
where this runs.  With `CFG["enabled"] = False` every reference function takes its XLA (pure jnp)
branch, which is the executable specification the CUDA kernels and the oracle must match.
Inputs are seeded NumPy arrays with the shapes of the reference's unit test
(modal/test_moe_permute.py:20,37: n=64, E=16, k in {6,12}; d=128 keeps the fixtures small).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import jax_numpy_shim  # noqa: E402


def bf16_round(a):
  u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
  return ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32).reshape(a.shape)


def main(ref_root):
  jax = jax_numpy_shim.install()
  sys.path.insert(0, os.path.join(ref_root, "modal"))
  import moe_permute as mp
  import padded_gmm as pg
  mp.CFG["enabled"] = False
  E, n, d = 16, 64, 128
  for case, (k, bf16) in enumerate([(6, False), (12, True)]):
    rng = np.random.default_rng(100 + case)
    prep = bf16_round if bf16 else (lambda a: a.astype(np.float32))
    x = prep(rng.standard_normal((n, d)).astype(np.float32))
    sel = np.argsort(-rng.standard_normal((n, E)), axis=1, kind="stable")[:, :k].astype(np.int32)
    flat = sel.reshape(-1)
    w = jax.nn.softmax(rng.standard_normal((n, k)).astype(np.float32), axis=1)
    m = n * k
    y = prep(rng.standard_normal((m, d)).astype(np.float32))
    g = prep(rng.standard_normal((n, d)).astype(np.float32))
    idx = (rng.permutation(m) % n).astype(np.int32)
    scale = rng.standard_normal(m).astype(np.float32)
    A = lambda a: np.asarray(a).view(jax_numpy_shim.Arr)
    order_a, pos_a = mp.sort_indices(A(flat), E, "argsort")
    order_c, pos_c = mp.sort_indices(A(flat), E, "count")
    pos2 = np.asarray(pos_a).reshape(n, k)
    out = dict(
        k=k, bf16=int(bf16), x=x, flat=flat, w=np.asarray(w), y=y, g=g, idx=idx, scale=scale,
        order_argsort=np.asarray(order_a), pos_argsort=np.asarray(pos_a),
        order_count=np.asarray(order_c), pos_count=np.asarray(pos_c),
        gather_rows=np.asarray(mp.gather_rows(A(x), A(idx))),
        gather_rows_scale=np.asarray(mp.gather_rows(A(x), A(idx), A(scale))),
        gather_reduce=np.asarray(mp.gather_reduce(A(y), A(pos2), None, np.float32)),
        gather_reduce_w=np.asarray(mp.gather_reduce(A(y), A(pos2), A(np.asarray(w)), np.float32)),
        gather_dot=np.asarray(mp.gather_dot(A(y), A(pos2), A(g))),
        ref_dispatch=np.asarray(mp.ref_dispatch(A(x), A(flat))),
        ref_combine=np.asarray(mp.ref_combine(A(y), A(flat), A(np.asarray(w)))),
        moe_block_tanh=np.asarray(mp.moe_block(A(x), A(flat), A(np.asarray(w)),
                                               lambda r: np.tanh(np.asarray(r, np.float32)).view(jax_numpy_shim.Arr),
                                               use_kernels=False)),
    )
    np.savez_compressed(os.path.join(HERE, f"moe_permute_k{k}_{'bf16' if bf16 else 'f32'}.npz"), **out)
    print("wrote case", k, bf16, {a: np.asarray(b).shape for a, b in out.items() if hasattr(b, "shape")})
  # padded_ragged_dot on the group sizes of the reference's own known-answer check (modal/te_run.py:72)
  gs = np.array([5, 0, 9, 3, 7, 1, 6, 4], np.int32)
  mrows = int(gs.sum()) + 3
  rng = np.random.default_rng(7)
  a = bf16_round(rng.standard_normal((mrows, 64)).astype(np.float32))
  b = bf16_round(rng.standard_normal((8, 64, 64)).astype(np.float32))
  res = dict(gs=gs, a=a, b=b)
  for factor in (2.0, 1.0):
    pg.FACTOR = factor
    res[f"out_factor{int(factor)}"] = np.asarray(pg.padded_ragged_dot(np.asarray(a).view(jax_numpy_shim.Arr),
                                                                      np.asarray(b).view(jax_numpy_shim.Arr),
                                                                      np.asarray(gs).view(jax_numpy_shim.Arr)))
  np.savez_compressed(os.path.join(HERE, "padded_ragged_dot_te_shapes.npz"), **res)
  print("wrote padded_ragged_dot", {a_: b_.shape for a_, b_ in res.items()})


if __name__ == "__main__":
  if len(sys.argv) != 2:
    raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference repository>")
  main(sys.argv[1])
