"""Generates tests/golden/*.npz by RUNNING the reference's own pure-array MoE code.

  python tests/golden/make_golden.py /path/to/reference

The reference's `modal/moe_permute.py` and `modal/padded_gmm.py` are imported from the reference tree
(never copied) under the NumPy stand-in of `jax_numpy_shim.py`, because real JAX is not installable
where this runs.  With `CFG["enabled"] = False` every reference function takes its XLA (pure jnp)
branch, which is the executable specification the CUDA kernels and the oracle must match.  The backward
functions the reference registers with `defvjp` (`_dispatch_bwd`, `_combine_bwd`, `_permute_rows_bwd`:
modal/moe_permute.py:282-329; `_perm_gather_bwd`: modal/padded_gmm.py:35-39) are called through the `fwd` / `bwd`
pair the stand-in keeps, so gradients are pinned by the reference's own code as well.
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
    # backward passes exactly as jax.custom_vjp would run them: residuals from fwd, cotangents into bwd
    gy = prep(rng.standard_normal((m, d)).astype(np.float32))          # cotangent of dispatch / permute_rows outputs
    gc = rng.standard_normal((n, d)).astype(np.float32)                # cotangent of combine's float32 output
    perm = rng.permutation(m).astype(np.int32)
    _, res_d = mp.dispatch.fwd(A(x), order_a, pos_a)
    dispatch_dx = mp.dispatch.bwd(res_d, A(gy))[0]
    comb_out, res_c = mp.combine.fwd(A(y), order_a, pos_a, A(np.asarray(w)))
    combine_dy, _, _, combine_dw = mp.combine.bwd(res_c, A(gc))
    perm_out, res_p = mp.permute_rows.fwd(A(y), A(perm))
    permute_dx = mp.permute_rows.bwd(res_p, A(gy))[0]
    out = dict(
        gy=gy, gc=gc, perm=perm, dispatch_dx=np.asarray(dispatch_dx, np.float32),
        combine_fwd=np.asarray(comb_out), combine_dy=np.asarray(combine_dy, np.float32),
        combine_dw=np.asarray(combine_dw, np.float32), permute_fwd=np.asarray(perm_out, np.float32),
        permute_dx=np.asarray(permute_dx, np.float32),
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
  b = bf16_round(rng.standard_normal((8, 64, 48)).astype(np.float32))   # K=64, N=48 as in modal/te_run.py:73
  res = dict(gs=gs, a=a, b=b)
  for factor in (2.0, 1.0):
    pg.FACTOR = factor
    res[f"out_factor{int(factor)}"] = np.asarray(pg.padded_ragged_dot(np.asarray(a).view(jax_numpy_shim.Arr),
                                                                      np.asarray(b).view(jax_numpy_shim.Arr),
                                                                      np.asarray(gs).view(jax_numpy_shim.Arr)))
  # _perm_gather and its registered backward on the row <-> slot maps padded_ragged_dot builds for factor 2
  e, c = 8, 16
  starts = np.cumsum(gs) - gs
  rows = np.arange(mrows, dtype=np.int32)
  expert = np.minimum(np.searchsorted(np.cumsum(gs), rows, side="right"), e - 1).astype(np.int32)
  pos = rows - starts[expert]
  slot = np.where((rows < gs.sum()) & (pos < c), expert * c + pos, e * c).astype(np.int32)
  se, sc = np.arange(e * c, dtype=np.int32) // c, np.arange(e * c, dtype=np.int32) % c
  src = np.where(sc < np.minimum(gs[se], c), starts[se] + sc, mrows).astype(np.int32)
  V = lambda v: np.asarray(v).view(jax_numpy_shim.Arr)
  buf, res_g = pg._perm_gather.fwd(V(a), V(src), V(slot))
  gbuf = bf16_round(rng.standard_normal(np.asarray(buf).shape).astype(np.float32))
  res.update(pg_src=src, pg_slot=slot, pg_fwd=np.asarray(buf, np.float32), pg_g=gbuf,
             pg_bwd=np.asarray(pg._perm_gather.bwd(res_g, V(gbuf))[0], np.float32))
  np.savez_compressed(os.path.join(HERE, "padded_ragged_dot_te_shapes.npz"), **res)
  print("wrote padded_ragged_dot", {a_: b_.shape for a_, b_ in res.items()})


if __name__ == "__main__":
  if len(sys.argv) != 2:
    raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference repository>")
  main(sys.argv[1])
