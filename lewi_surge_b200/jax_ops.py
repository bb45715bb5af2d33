"""JAX-facing operators: `jax.ffi` custom calls with `custom_vjp` wrappers that keep the signatures of the
reference's `moe_permute` / `padded_gmm` functions, and `install()` which patches MaxText exactly where the
reference does (modal/moe_permute.py:386-436, modal/padded_gmm.py:72-76).

JAX is imported lazily: this module can be imported without it (the torch-facing mirror is `ops.py`).  It needs
`liblewi_moe_ffi.so` (csrc/ffi_xla.cc built against jaxlib's FFI headers).  COMPILE-UNVERIFIED: neither JAX nor
jaxlib could be installed where this repository was built; all numerics are validated through the same C entry
points via ctypes.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
FFI_LIB = os.path.join(HERE, "liblewi_moe_ffi.so")
BLOCK = 128
CFG = {"num_experts": None, "registered": False}
_TARGETS = ("lewi_ffi_sort_indices", "lewi_ffi_gather_rows", "lewi_ffi_gather_reduce", "lewi_ffi_gather_dot",
            "lewi_ffi_ragged_dot_fwd", "lewi_ffi_ragged_dot_dlhs", "lewi_ffi_ragged_dot_drhs")


def _register():
  """Load the FFI library and register its handlers once (idempotent)."""
  if CFG["registered"]:
    return
  import jax
  if not os.path.exists(FFI_LIB):
    raise RuntimeError(f"{FFI_LIB} not built: compile csrc/ffi_xla.cc against jax.ffi.include_dir() first. "
                       "There is no fallback path.")
  ctypes.CDLL(os.path.join(HERE, "liblewi_moe.so"), mode=ctypes.RTLD_GLOBAL)
  lib = ctypes.CDLL(FFI_LIB)
  for name in _TARGETS:
    jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(lib, name)), platform="CUDA")
  CFG["registered"] = True


def _core():
  from . import _lib
  return _lib.load()


def _check_rows(x):
  if x.ndim != 2 or (x.shape[1] * x.dtype.itemsize) % 16 != 0:
    raise ValueError("lewi_surge_b200: rows must be 2-D with a multiple of 16 bytes per row (no fallback path)")


def gather_rows(x, idx, scale=None, idx_div=1, scale_by_idx=False):
  """out[i] = x[idx[i]] (* scale[i]) -- signature of modal/moe_permute.py:116."""
  import jax
  import jax.numpy as jnp
  _register()
  _check_rows(x)
  sc = scale.astype(jnp.float32) if scale is not None else jnp.zeros((0,), jnp.float32)
  call = jax.ffi.ffi_call("lewi_ffi_gather_rows", jax.ShapeDtypeStruct((idx.shape[0], x.shape[1]), x.dtype))
  return call(x, idx.astype(jnp.int32), sc, has_scale=scale is not None, idx_div=int(idx_div),
              scale_by_idx=bool(scale_by_idx))


def gather_reduce(y, pos, w=None, out_dtype=None):
  """out[t] = sum_j w[t,j] * y[pos[t,j]] -- signature of modal/moe_permute.py:214."""
  import jax
  import jax.numpy as jnp
  _register()
  _check_rows(y)
  out_dtype = out_dtype or y.dtype
  ww = w.astype(jnp.float32) if w is not None else jnp.zeros((0, 0), jnp.float32)
  call = jax.ffi.ffi_call("lewi_ffi_gather_reduce", jax.ShapeDtypeStruct((pos.shape[0], y.shape[1]), out_dtype))
  return call(y, pos.astype(jnp.int32), ww, has_w=w is not None)


def gather_dot(y, pos, g):
  """out[t,j] = <g[t], y[pos[t,j]]> -- signature of modal/moe_permute.py:228."""
  import jax
  import jax.numpy as jnp
  _register()
  call = jax.ffi.ffi_call("lewi_ffi_gather_dot", jax.ShapeDtypeStruct(pos.shape, jnp.float32))
  return call(y, pos.astype(jnp.int32), g.astype(y.dtype))


def sort_indices(flat_experts, num_experts=None, method=None):
  """(order, pos) of the stable sort by expert id -- signature of modal/moe_permute.py:240."""
  import jax
  import jax.numpy as jnp
  del method
  _register()
  e = num_experts or CFG["num_experts"]
  m = flat_experts.shape[0]
  ws = int(_core().lewi_route_workspace_bytes(m, e))
  call = jax.ffi.ffi_call("lewi_ffi_sort_indices", (jax.ShapeDtypeStruct((m,), jnp.int32), jax.ShapeDtypeStruct((m,), jnp.int32),
                                                    jax.ShapeDtypeStruct((ws,), jnp.uint8)))
  order, pos, _ = call(flat_experts.astype(jnp.int32), num_experts=int(e))
  return order, pos


def _make_vjp_ops():
  """Builds dispatch / combine / permute_rows / ragged_dot with the reference's gather-only backward passes."""
  import jax
  import jax.numpy as jnp

  @jax.custom_vjp
  def dispatch(x, order, pos):
    k = order.shape[0] // x.shape[0]
    return gather_rows(x, order, idx_div=k)

  def dispatch_fwd(x, order, pos):
    return dispatch(x, order, pos), (order, pos, jnp.empty((x.shape[0], 0), x.dtype))

  def dispatch_bwd(res, g):
    order, pos, carrier = res
    n = carrier.shape[0]
    return gather_reduce(g, pos.reshape(n, order.shape[0] // n), None, carrier.dtype), None, None

  dispatch.defvjp(dispatch_fwd, dispatch_bwd)

  @jax.custom_vjp
  def combine(y, order, pos, w):
    n, k = w.shape
    return gather_reduce(y, pos.reshape(n, k), w, jnp.float32)

  def combine_fwd(y, order, pos, w):
    return combine(y, order, pos, w), (y, order, pos, w)

  def combine_bwd(res, g):
    y, order, pos, w = res
    n, k = w.shape
    dy = gather_rows(g.astype(y.dtype), order, w.reshape(-1), idx_div=k, scale_by_idx=True)
    dw = gather_dot(y, pos.reshape(n, k), g).astype(w.dtype)
    return dy, None, None, dw

  combine.defvjp(combine_fwd, combine_bwd)

  @jax.custom_vjp
  def permute_rows(x, idx):
    return gather_rows(x, idx)

  def permute_fwd(x, idx):
    return permute_rows(x, idx), idx

  def permute_bwd(idx, g):
    inv = jnp.zeros_like(idx).at[idx].set(jnp.arange(idx.shape[0], dtype=idx.dtype))
    return gather_rows(g, inv), None

  permute_rows.defvjp(permute_fwd, permute_bwd)

  def _shapes(m, k, n, e):
    mpad = int(_core().lewi_padded_rows_bound(m, e, BLOCK))
    i32 = lambda *s: jax.ShapeDtypeStruct(s, jnp.int32)
    b16 = lambda *s: jax.ShapeDtypeStruct(s, jnp.bfloat16)
    return mpad, i32, b16

  @jax.custom_vjp
  def ragged_dot_core(lhs, rhs, gs):
    return _ragged_fwd(lhs, rhs, gs)[0]

  def _ragged_fwd(lhs, rhs, gs):
    m, k = lhs.shape
    e, _, n = rhs.shape
    mpad, i32, b16 = _shapes(m, k, n, e)
    call = jax.ffi.ffi_call("lewi_ffi_ragged_dot_fwd",
                            (b16(m, n), i32(e + 1), i32(mpad // BLOCK), i32(1), i32(mpad), i32(m), b16(mpad, k), b16(mpad, n)))
    return call(lhs.astype(jnp.bfloat16), rhs.astype(jnp.bfloat16), gs.astype(jnp.int32))

  def ragged_fwd(lhs, rhs, gs):
    out, pad_offsets, block_expert, n_blocks, rop, por, lhs_pad, _ = _ragged_fwd(lhs, rhs, gs)
    return out, (rhs.astype(jnp.bfloat16), pad_offsets, block_expert, n_blocks, rop, por, lhs_pad, lhs.dtype, rhs.dtype)

  def ragged_bwd(res, g):
    rhs, pad_offsets, block_expert, n_blocks, rop, por, lhs_pad, ldt, rdt = res
    m, n = g.shape
    e, k, _ = rhs.shape
    mpad = lhs_pad.shape[0]
    b16 = lambda *s: jax.ShapeDtypeStruct(s, jnp.bfloat16)
    dlhs, g_pad, _ = jax.ffi.ffi_call("lewi_ffi_ragged_dot_dlhs", (b16(m, k), b16(mpad, n), b16(mpad, k)))(
        g.astype(jnp.bfloat16), rhs, block_expert, n_blocks, rop, por)
    drhs = jax.ffi.ffi_call("lewi_ffi_ragged_dot_drhs", jax.ShapeDtypeStruct((e, k, n), jnp.float32))(lhs_pad, g_pad,
                                                                                                      pad_offsets)
    return dlhs.astype(ldt), drhs.astype(rdt), None

  ragged_dot_core.defvjp(ragged_fwd, ragged_bwd)
  return dispatch, combine, permute_rows, ragged_dot_core


def install(mode="full", num_experts=None, tile=None, sort=None, factor=None, probe=True, patch_ragged_dot=True):
  """Patch `jax.lax.ragged_dot` and `maxtext.layers.moe` (0.2.5); call BEFORE `import maxtext` is used.

  Same arguments as the reference's installers; `tile`, `sort`, `factor`, `probe` are accepted and ignored
  (block size is 128, the sort is a counting sort, the layout is dropless, there is no packing to probe).
  """
  import jax
  import jax.numpy as jnp
  del tile, sort, factor, probe
  _register()
  if num_experts:
    CFG["num_experts"] = int(num_experts)
  dispatch, combine, permute_rows, ragged_dot_core = _make_vjp_ops()
  orig_ragged_dot = jax.lax.ragged_dot

  def ragged_dot(lhs, rhs, group_sizes, precision=None, preferred_element_type=None, **kw):
    # same guard as modal/padded_gmm.py:46-48: other forms go to the original op
    if lhs.ndim != 2 or rhs.ndim != 3 or kw.get("group_offset") is not None:
      return orig_ragged_dot(lhs, rhs, group_sizes, precision=precision, preferred_element_type=preferred_element_type, **kw)
    out = ragged_dot_core(lhs, rhs, group_sizes)
    return out.astype(preferred_element_type or lhs.dtype)

  if patch_ragged_dot:
    jax.lax.ragged_dot = ragged_dot

  import maxtext.layers.moe as moe  # pylint: disable=import-outside-toplevel

  def _route_activations(inputs, selected_experts):
    flat = selected_experts.reshape(-1)
    order, pos = sort_indices(flat, CFG["num_experts"])
    with jax.named_scope("moe_permute_dispatch"):
      return dispatch(inputs, order, pos)

  def _sort_activations(inputs, sort_idx, use_custom_vjp=True):
    del use_custom_vjp
    with jax.named_scope("moe_permute_sort"):
      return permute_rows(inputs, sort_idx.astype(jnp.int32))

  moe._route_activations = _route_activations  # pylint: disable=protected-access
  moe._sort_activations = _sort_activations  # pylint: disable=protected-access

  if mode == "full":
    orig_unpermute = moe.RoutedMoE.unpermute

    def unpermute(self, intermediate, sorted_selected_experts, weights, batch_size, sequence_length,
                  use_custom_sort_vjp=True, group_sizes=None, topk_argsort_indices=None, **kw):
      simple = (not kw.get("tc_routing")
                and not (self.config.use_ragged_sort and self.config.use_ring_of_experts)
                and self.config.decoder_block != moe.ctypes.DecoderBlockType.LLAMA4
                and not isinstance(intermediate, moe.qpl.QArray))
      if not simple:
        return orig_unpermute(self, intermediate, sorted_selected_experts, weights, batch_size, sequence_length,
                              use_custom_sort_vjp, group_sizes, topk_argsort_indices, **kw)
      order = sorted_selected_experts.astype(jnp.int32)
      m = order.shape[0]
      pos = jnp.zeros((m,), jnp.int32).at[order].set(jnp.arange(m, dtype=jnp.int32))
      w = jnp.reshape(weights, (-1, self.num_experts_per_tok)).astype(jnp.float32)
      with jax.named_scope("moe_permute_combine"):
        out = combine(intermediate, order, pos, w)
      return out.reshape(batch_size, sequence_length, -1).astype(self.dtype)

    moe.RoutedMoE.unpermute = unpermute
  print(f"[lewi_surge_b200] installed mode={mode} block={BLOCK} num_experts={CFG['num_experts']} "
        f"(sm_100a kernels behind jax.ffi)", flush=True)
