"""A NumPy stand-in for the few `jax` names the reference's pure-array MoE code uses.

Real JAX cannot be installed where the golden vectors are generated, so `make_golden.py` runs the
reference's own source files (`modal/moe_permute.py`, `modal/padded_gmm.py`) with these modules in
`sys.modules`.  Every function maps to the NumPy call with the meaning JAX documents for it:
`jnp.argsort` is stable, `jnp.take(..., mode="clip")` clips indices, `x.at[i].set(v)` is a functional
scatter-set, `jax.custom_vjp` objects call their primal function.  Nothing here is used by the product.
"""
import sys
import types

import numpy as np

try:
  import ml_dtypes
  _bf16 = ml_dtypes.bfloat16
except Exception:  # noqa: BLE001
  _bf16 = np.float32


class Arr(np.ndarray):
  """ndarray with the functional `.at[idx].set(v)` update."""

  @property
  def at(self):
    return _At(self)


class _At:
  def __init__(self, a):
    self.a = a

  def __getitem__(self, idx):
    a = self.a

    class _Set:
      def set(self, v):
        out = np.array(a, copy=True)
        out[np.asarray(idx)] = np.asarray(v)
        return out.view(Arr)
    return _Set()


def _wrap(fn):
  def f(*args, **kw):
    args = [np.asarray(a) if isinstance(a, np.ndarray) else a for a in args]
    out = fn(*args, **kw)
    return out.view(Arr) if isinstance(out, np.ndarray) else out
  return f


def _take(a, idx, axis=0, mode=None):
  a, idx = np.asarray(a), np.asarray(idx)
  if mode == "clip":
    idx = np.clip(idx, 0, a.shape[axis] - 1)
  return np.take(a, idx, axis=axis).view(Arr)


def _argsort(a, axis=-1, **kw):
  return np.argsort(np.asarray(a), axis=axis, kind="stable").astype(np.int32).view(Arr)


def _einsum(spec, *ops, precision=None, preferred_element_type=None):
  out = np.einsum(spec, *[np.asarray(o, np.float32) for o in ops])
  return out.astype(preferred_element_type or np.float32).view(Arr)


def _one_hot(x, n, dtype=np.float32):
  return (np.asarray(x)[..., None] == np.arange(n)).astype(dtype).view(Arr)


def _softmax(x, axis=-1):
  x = np.asarray(x, np.float32)
  e = np.exp(x - x.max(axis=axis, keepdims=True))
  return (e / e.sum(axis=axis, keepdims=True)).view(Arr)


def _searchsorted(a, v, side="left"):
  return np.searchsorted(np.asarray(a), np.asarray(v), side=side).astype(np.int32).view(Arr)


class _CustomVjp:
  def __init__(self, fn, nondiff_argnums=()):
    self.fn = fn

  def __call__(self, *a, **k):
    return self.fn(*a, **k)

  def defvjp(self, fwd, bwd):
    self.fwd, self.bwd = fwd, bwd


def _ragged_dot(lhs, rhs, group_sizes, **kw):
  lhs, rhs = np.asarray(lhs, np.float32), np.asarray(rhs, np.float32)
  out = np.zeros((lhs.shape[0], rhs.shape[2]), np.float32)
  s = 0
  for e, c in enumerate(np.asarray(group_sizes)):
    out[s:s + c] = lhs[s:s + c] @ rhs[e]
    s += c
  return out.view(Arr)


def install():
  jnp = types.ModuleType("jax.numpy")
  for name in ("zeros", "ones", "arange", "cumsum", "concatenate", "minimum", "maximum", "where", "sum", "tanh",
               "take_along_axis", "array_equal", "empty", "reshape", "abs", "exp", "pad"):
    setattr(jnp, name, _wrap(getattr(np, name)))
  jnp.take, jnp.argsort, jnp.einsum, jnp.searchsorted = _take, _argsort, _einsum, _searchsorted
  jnp.float32, jnp.int32, jnp.uint32, jnp.uint16, jnp.float16, jnp.bfloat16 = (np.float32, np.int32, np.uint32,
                                                                               np.uint16, np.float16, _bf16)
  jnp.dtype = np.dtype
  jnp.asarray = lambda a, dtype=None: np.asarray(a, dtype).view(Arr)
  lax = types.ModuleType("jax.lax")
  lax.ragged_dot = _ragged_dot
  lax.bitcast_convert_type = lambda a, t: np.asarray(a).view(t).view(Arr)
  lax.fori_loop = None
  nn = types.ModuleType("jax.nn")
  nn.one_hot, nn.softmax = _one_hot, _softmax
  jax = types.ModuleType("jax")
  jax.numpy, jax.lax, jax.nn = jnp, lax, nn
  jax.custom_vjp = _CustomVjp
  jax.jit = lambda f, **k: f
  jax.devices = lambda: [types.SimpleNamespace(platform="cpu")]
  jax.named_scope = lambda name: __import__("contextlib").nullcontext()
  exp = types.ModuleType("jax.experimental")
  pallas = types.ModuleType("jax.experimental.pallas")
  tpu = types.ModuleType("jax.experimental.pallas.tpu")
  tpu.InterpretParams = lambda: None
  exp.pallas, pallas.tpu = pallas, tpu
  jax.experimental = exp
  sys.modules.update({"jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.nn": nn, "jax.experimental": exp,
                      "jax.experimental.pallas": pallas, "jax.experimental.pallas.tpu": tpu})
  return jax
