"""JAX-facing operators: `jax.ffi` custom calls with `custom_vjp` wrappers that keep the signatures of the
reference's `moe_permute` / `padded_gmm` functions, a fused `moe_layer`, and `install()` which patches MaxText at the
reference's patch points (modal/moe_permute.py:386-436, modal/padded_gmm.py:72-76).

JAX is imported lazily: this module can be imported without it (the torch-facing mirror is `ops.py` / `layer.py`).
It needs `liblewi_moe_ffi.so`: csrc/ffi_xla.cc + csrc/ffi_core.cc built against jaxlib's FFI headers.  NOT RUN
ANYWHERE YET: neither JAX nor jaxlib could be installed where this repository was built.  What is checked without
JAX: the XLA-free core compiles and links against the library, and the handler layer type-checks against a stand-in
of the FFI header (tests/test_ffi_compile.py); all numerics are validated through the same C entry points via ctypes.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
FFI_LIB = os.path.join(HERE, "liblewi_moe_ffi.so")
BLOCK = 128
CFG = {"num_experts": None, "registered": False}
_TARGETS = ("lewi_ffi_sort_indices", "lewi_ffi_gather_rows", "lewi_ffi_gather_reduce", "lewi_ffi_gather_dot",
            "lewi_ffi_ragged_dot_fwd", "lewi_ffi_ragged_dot_dlhs", "lewi_ffi_ragged_dot_drhs", "lewi_ffi_moe_fwd",
            "lewi_ffi_moe_bwd", "lewi_ffi_causal_conv1d_fwd", "lewi_ffi_causal_conv1d_bwd", "lewi_ffi_gdn_chunk_fwd",
            "lewi_ffi_gdn_chunk_bwd")


def _register():
  """Load the FFI library and register its handlers once (idempotent)."""
  if CFG["registered"]:
    return
  import jax
  if not os.path.exists(FFI_LIB):
    raise RuntimeError(f"{FFI_LIB} not built: compile csrc/ffi_xla.cc and csrc/ffi_core.cc against "
                       "jax.ffi.include_dir() first.  There is no fallback path.")
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


# ----------------------------------------------------------------------------------- per-op custom calls


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


class _Ops:
  """The differentiable operators, built once JAX is importable.  Residuals hold JAX values only: dtypes travel as
  zero-size carrier arrays (the reference's trick, modal/moe_permute.py:277-279), never as Python objects."""

  def __init__(self):
    import jax
    import jax.numpy as jnp
    self.jax, self.jnp = jax, jnp
    carrier = lambda a: jnp.empty((a.shape[0], 0), a.dtype)

    # dispatch: rows grouped by expert; backward = unweighted gather-reduce (modal/moe_permute.py:270-289)
    def dispatch(x, order, pos):
      return gather_rows(x, order, idx_div=order.shape[0] // x.shape[0])
    self.dispatch = jax.custom_vjp(dispatch)
    self.dispatch.defvjp(
        lambda x, order, pos: (dispatch(x, order, pos), (order, pos, carrier(x))),
        lambda res, g: (gather_reduce(g, res[1].reshape(res[2].shape[0], -1), None, res[2].dtype), None, None))

    # combine: weighted sum of each token's k rows in f32; backward = scaled gather + gather-dot (:292-312)
    def combine(y, order, pos, w):
      return gather_reduce(y, pos.reshape(w.shape), w, jnp.float32)

    def combine_bwd(res, g):
      y, order, pos, w = res
      k = w.shape[1]
      dy = gather_rows(g.astype(y.dtype), order, w.reshape(-1), idx_div=k, scale_by_idx=True)
      return dy, None, None, gather_dot(y, pos.reshape(w.shape), g).astype(w.dtype)
    self.combine = jax.custom_vjp(combine)
    self.combine.defvjp(lambda y, order, pos, w: (combine(y, order, pos, w), (y, order, pos, w)), combine_bwd)

    # permute_rows: x[idx] for a permutation; backward gathers through the inverse permutation (:315-329)
    def permute_rows(x, idx):
      return gather_rows(x, idx)

    def permute_bwd(idx, g):
      inverse = jnp.zeros_like(idx).at[idx].set(jnp.arange(idx.shape[0], dtype=idx.dtype))
      return gather_rows(g, inverse), None
    self.permute_rows = jax.custom_vjp(permute_rows)
    self.permute_rows.defvjp(lambda x, idx: (permute_rows(x, idx), idx), permute_bwd)

    self.ragged_dot = jax.custom_vjp(lambda lhs, rhs, gs: self._ragged_call(lhs, rhs, gs)[0])
    self.ragged_dot.defvjp(self._ragged_fwd, self._ragged_bwd)

  # ragged_dot: gather -> grouped GEMM -> gather, forward and backward (modal/padded_gmm.py:45-69 made dropless)
  def _ragged_call(self, lhs, rhs, gs):
    jax, jnp = self.jax, self.jnp
    m, k = lhs.shape
    e, _, n = rhs.shape
    mpad = int(_core().lewi_padded_rows_bound(m, e, BLOCK))
    i32 = lambda *s: jax.ShapeDtypeStruct(s, jnp.int32)
    b16 = lambda *s: jax.ShapeDtypeStruct(s, jnp.bfloat16)
    call = jax.ffi.ffi_call("lewi_ffi_ragged_dot_fwd",
                            (b16(m, n), i32(e + 1), i32(mpad // BLOCK), i32(1), i32(mpad), i32(m), b16(mpad, k), b16(mpad, n)))
    return call(lhs.astype(jnp.bfloat16), rhs.astype(jnp.bfloat16), gs.astype(jnp.int32))

  def _ragged_fwd(self, lhs, rhs, gs):
    jnp = self.jnp
    out, pad_offsets, block_expert, n_blocks, rop, por, lhs_pad, _ = self._ragged_call(lhs, rhs, gs)
    residual = (rhs.astype(jnp.bfloat16), pad_offsets, block_expert, n_blocks, rop, por, lhs_pad,
                jnp.empty((0,), lhs.dtype), jnp.empty((0,), rhs.dtype))
    return out, residual

  def _ragged_bwd(self, res, g):
    jax, jnp = self.jax, self.jnp
    rhs, pad_offsets, block_expert, n_blocks, rop, por, lhs_pad, lhs_like, rhs_like = res
    m, n = g.shape
    e, k, _ = rhs.shape
    mpad = lhs_pad.shape[0]
    b16 = lambda *s: jax.ShapeDtypeStruct(s, jnp.bfloat16)
    dlhs, g_pad, _ = jax.ffi.ffi_call("lewi_ffi_ragged_dot_dlhs", (b16(m, k), b16(mpad, n), b16(mpad, k)))(
        g.astype(jnp.bfloat16), rhs, pad_offsets, block_expert, n_blocks, rop, por)
    scratch = max(int(_core().lewi_grouped_gemm_tn_workspace_bytes(mpad, k, n, e, 0)), 16)
    drhs, _ = jax.ffi.ffi_call("lewi_ffi_ragged_dot_drhs", (jax.ShapeDtypeStruct((e, k, n), jnp.float32),
                                                            jax.ShapeDtypeStruct((scratch,), jnp.uint8)))(lhs_pad, g_pad, pad_offsets)
    return dlhs.astype(lhs_like.dtype), drhs.astype(rhs_like.dtype), None


_OPS = None


def _ops():
  global _OPS
  if _OPS is None:
    _register()
    _OPS = _Ops()
  return _OPS


def dispatch(x, order, pos):
  """Signature of modal/moe_permute.py:271."""
  return _ops().dispatch(x, order, pos)


def combine(y, order, pos, w):
  """Signature of modal/moe_permute.py:293."""
  return _ops().combine(y, order, pos, w)


def permute_rows(x, idx):
  """Signature of modal/moe_permute.py:316."""
  return _ops().permute_rows(x, idx)


def padded_ragged_dot(lhs, rhs, group_sizes, precision=None, preferred_element_type=None, **kw):
  """Drop-in for `jax.lax.ragged_dot` with the signature of modal/padded_gmm.py:45 (dropless layout)."""
  del precision
  if lhs.ndim != 2 or rhs.ndim != 3 or kw.get("group_offset") is not None:
    raise ValueError("lewi_surge_b200.padded_ragged_dot: only lhs [M,K], rhs [E,K,N] without group_offset")
  return _ops().ragged_dot(lhs, rhs, group_sizes).astype(preferred_element_type or lhs.dtype)


te_ragged_dot = padded_ragged_dot


# ----------------------------------------------------------------------------------- the fused layer


def moe_layer(x, w_router, w_gate, w_up, w_down, ws_gate=None, ws_up=None, ws_down=None, w_sg=None, router_bias=None, *,
              k, aux_weight=0.0):
  """The whole MoE layer as ONE custom call each way: (out [T,d], aux_loss [1]) = layer(x; weights).

  Weight orientation is MaxText's (modal/stage2.py:338-345).  Differentiable in x and every weight through
  `lewi_ffi_moe_bwd`; `aux_weight` adds the gradient of `aux_weight * aux_loss` to the router (aux_loss itself is
  returned as a value without gradient)."""
  import jax
  import jax.numpy as jnp
  _register()
  t, d = x.shape
  e, _, f = w_gate.shape
  has_shared, has_gate, has_bias = ws_gate is not None, w_sg is not None, router_bias is not None
  fs = ws_gate.shape[1] if has_shared else 0
  core = _core()
  res_bytes = int(core.lewi_moe_residual_layout(t, d, e, f, int(k), fs, int(has_gate), None))
  ws_bytes = int(core.lewi_moe_workspace_bytes(t, d, e, f, int(k), fs, int(has_gate)))
  empty16 = jnp.zeros((0, 0), jnp.bfloat16)
  empty32 = jnp.zeros((0,), jnp.float32)
  u8 = lambda n: jax.ShapeDtypeStruct((max(n, 16),), jnp.uint8)
  like = lambda a, dt=None: jax.ShapeDtypeStruct(a.shape, dt or a.dtype)
  attrs = dict(k=int(k), has_bias=has_bias, has_gate=has_gate)

  def operands(xv, wr, wg, wu, wd, sg, su, sd, gate, bias):
    b16 = lambda a: a.astype(jnp.bfloat16)
    return (b16(xv), wr.astype(jnp.float32), bias.astype(jnp.float32) if has_bias else empty32, b16(wg), b16(wu), b16(wd),
            b16(sg) if has_shared else empty16, b16(su) if has_shared else empty16, b16(sd) if has_shared else empty16,
            gate.astype(jnp.float32) if has_gate else empty32)

  def forward(*args):
    ops = operands(*args)
    out, aux, residual, _ = jax.ffi.ffi_call(
        "lewi_ffi_moe_fwd", (jax.ShapeDtypeStruct((t, d), jnp.bfloat16), jax.ShapeDtypeStruct((1,), jnp.float32),
                             u8(res_bytes), u8(ws_bytes)))(*ops, **attrs)
    return (out.astype(x.dtype), aux), (ops, residual)

  @jax.custom_vjp
  def layer(*args):
    return forward(*args)[0]

  def backward(saved, cot):
    ops, residual = saved
    g_out, _ = cot
    xv, wr, bias, wg, wu, wd, sg, su, sd, gate = ops
    z16 = jax.ShapeDtypeStruct((0, 0), jnp.bfloat16)
    z32 = jax.ShapeDtypeStruct((0,), jnp.float32)
    outs = jax.ffi.ffi_call(
        "lewi_ffi_moe_bwd",
        (like(xv), like(wr), like(bias) if has_bias else z32, like(wg), like(wu), like(wd),
         like(sg) if has_shared else z16, like(su) if has_shared else z16, like(sd) if has_shared else z16,
         like(gate) if has_gate else z32, u8(ws_bytes)))(
             g_out.astype(jnp.bfloat16), xv, wr, wg, wu, wd, sg, su, sd, gate, residual, aux_grad=float(aux_weight), **attrs)
    dx, dwr, dbias, dwg, dwu, dwd, dsg, dsu, dsd, dgate, _ = outs
    grads = (dx.astype(x.dtype), dwr.astype(w_router.dtype), dwg.astype(w_gate.dtype), dwu.astype(w_up.dtype),
             dwd.astype(w_down.dtype), dsg.astype(ws_gate.dtype) if has_shared else None,
             dsu.astype(ws_up.dtype) if has_shared else None, dsd.astype(ws_down.dtype) if has_shared else None,
             dgate.astype(w_sg.dtype) if has_gate else None, dbias.astype(router_bias.dtype) if has_bias else None)
    return grads

  layer.defvjp(forward, backward)
  return layer(x, w_router, w_gate, w_up, w_down, ws_gate, ws_up, ws_down, w_sg, router_bias)


# ----------------------------------------------------------------------------------- MaxText patch


class MaxTextPatch:
  """The three callables the reference swaps into `maxtext.layers.moe` (0.2.5), kept together with the originals so
  that the patch can be undone.  Signatures are MaxText's; see modal/moe_permute.py:399-433 for the reference bodies."""

  def __init__(self, moe_module, mode):
    self.moe, self.mode = moe_module, mode
    self.saved = {}

  def route_activations(self, inputs, selected_experts):
    import jax
    order, pos = sort_indices(selected_experts.reshape(-1), CFG["num_experts"])
    with jax.named_scope("moe_permute_dispatch"):
      return dispatch(inputs, order, pos)

  def sort_activations(self, inputs, sort_idx, use_custom_vjp=True):
    import jax
    import jax.numpy as jnp
    del use_custom_vjp
    with jax.named_scope("moe_permute_sort"):
      return permute_rows(inputs, sort_idx.astype(jnp.int32))

  def _plain_dropless_case(self, block, intermediate, kw):
    """Whether this call is the plain dropless case the kernels cover; the special routings (tc_routing, ragged sort
    with ring of experts, the LLAMA4 block, quantised activations) stay with MaxText's own unpermute."""
    moe, cfg = self.moe, block.config
    if kw.get("tc_routing"):
      return False
    if cfg.use_ragged_sort and cfg.use_ring_of_experts:
      return False
    if cfg.decoder_block == moe.ctypes.DecoderBlockType.LLAMA4:
      return False
    return not isinstance(intermediate, moe.qpl.QArray)

  def make_unpermute(self):
    import jax
    import jax.numpy as jnp
    original = self.saved["unpermute"]
    patch = self

    def unpermute(self, intermediate, sorted_selected_experts, weights, batch_size, sequence_length,
                  use_custom_sort_vjp=True, group_sizes=None, topk_argsort_indices=None, **kw):
      if not patch._plain_dropless_case(self, intermediate, kw):
        return original(self, intermediate, sorted_selected_experts, weights, batch_size, sequence_length,
                        use_custom_sort_vjp, group_sizes, topk_argsort_indices, **kw)
      order = sorted_selected_experts.astype(jnp.int32)
      slots = order.shape[0]
      pos = jnp.zeros((slots,), jnp.int32).at[order].set(jnp.arange(slots, dtype=jnp.int32))   # inverse permutation
      w = jnp.reshape(weights, (-1, self.num_experts_per_tok)).astype(jnp.float32)
      with jax.named_scope("moe_permute_combine"):
        out = combine(intermediate, order, pos, w)
      return out.reshape(batch_size, sequence_length, -1).astype(self.dtype)

    return unpermute

  def apply(self):
    moe = self.moe
    self.saved.update(route=moe._route_activations, sort=moe._sort_activations, unpermute=moe.RoutedMoE.unpermute)  # pylint: disable=protected-access
    moe._route_activations = self.route_activations  # pylint: disable=protected-access
    moe._sort_activations = self.sort_activations  # pylint: disable=protected-access
    if self.mode == "full":
      moe.RoutedMoE.unpermute = self.make_unpermute()
    return self

  def restore(self):
    moe = self.moe
    moe._route_activations, moe._sort_activations = self.saved["route"], self.saved["sort"]  # pylint: disable=protected-access
    moe.RoutedMoE.unpermute = self.saved["unpermute"]


def install(mode="full", num_experts=None, tile=None, sort=None, factor=None, probe=True, patch_ragged_dot=True):
  """Patch `jax.lax.ragged_dot` and `maxtext.layers.moe` (0.2.5); call BEFORE `import maxtext` is used, like the
  reference's installers (modal/padded_gmm.py:12).  Same arguments as theirs; `tile`, `sort`, `factor`, `probe` are
  accepted and ignored (the block size is 128, the sort is a counting sort, the layout is dropless, there is no packing
  to probe).  Returns the `MaxTextPatch` (its `restore()` undoes the MaxText part)."""
  import jax
  del tile, sort, factor, probe
  _register()
  if num_experts:
    CFG["num_experts"] = int(num_experts)
  if patch_ragged_dot:
    stock = jax.lax.ragged_dot

    def ragged_dot(lhs, rhs, group_sizes, precision=None, preferred_element_type=None, **kw):
      # forms the kernels do not cover go to the stock op, as in modal/padded_gmm.py:46-48
      if lhs.ndim != 2 or rhs.ndim != 3 or kw.get("group_offset") is not None:
        return stock(lhs, rhs, group_sizes, precision=precision, preferred_element_type=preferred_element_type, **kw)
      return padded_ragged_dot(lhs, rhs, group_sizes, preferred_element_type=preferred_element_type)

    jax.lax.ragged_dot = ragged_dot
  import maxtext.layers.moe as moe  # pylint: disable=import-outside-toplevel
  patch = MaxTextPatch(moe, mode).apply()
  print(f"[lewi_surge_b200] installed mode={mode} block={BLOCK} num_experts={CFG['num_experts']} "
        f"(sm_100a kernels behind jax.ffi)", flush=True)
  return patch


# ----------------------------------------------------------------------------------- sequence mixing beside the layer


def causal_conv1d(x, w):
  """y[b,t,c] = sum_j w[j,0,c] * x[b, t-(K-1)+j, c]: the causal depthwise convolution of `_fast_call`
  (modal/fast_conv.py:14-31), x [B,T,C], w [K,1,C]; differentiable."""
  import jax
  import jax.numpy as jnp
  _register()

  def run(xv, wv):
    call = jax.ffi.ffi_call("lewi_ffi_causal_conv1d_fwd", jax.ShapeDtypeStruct(xv.shape, jnp.bfloat16))
    return call(xv, wv)

  def forward(xv, wv):
    return run(xv, wv), (xv, wv)

  def backward(saved, gy):
    xv, wv = saved
    b, t, c = xv.shape
    ws = int(_core().lewi_causal_conv1d_workspace_bytes(b, t, c, wv.shape[0]))
    call = jax.ffi.ffi_call("lewi_ffi_causal_conv1d_bwd", (jax.ShapeDtypeStruct(xv.shape, jnp.bfloat16),
                                                           jax.ShapeDtypeStruct(wv.shape, jnp.float32),
                                                           jax.ShapeDtypeStruct((max(ws, 1),), jnp.uint8)))
    dx, dw, _ = call(xv, wv, gy.astype(jnp.bfloat16))
    return dx, dw.astype(wv.dtype)

  op = jax.custom_vjp(run)
  op.defvjp(forward, backward)
  return op(x.astype(jnp.bfloat16), w.astype(jnp.bfloat16)).astype(x.dtype)


def chunk_gated_delta_rule(query, key, value, g, beta, chunk_size=64, initial_state=None, use_qk_norm_in_gdn=False,
                           cp_axis=None, compute_dtype=None):
  """Signature of the reference's `fast_chunk_gated_delta_rule` (modal/gdn_fast.py:37-38) for compute_dtype = bfloat16,
  chunks of 64 and no context parallelism; the q/k normalisation, when asked for, stays in JAX in front of the call as
  in the reference (:43-46).  Returns (o in query's dtype, final state in bf16 or None).  Differentiable."""
  import jax
  import jax.numpy as jnp
  _register()
  if cp_axis is not None or chunk_size != 64 or (compute_dtype is not None and compute_dtype != jnp.bfloat16):
    raise ValueError("lewi_surge_b200: chunk_gated_delta_rule covers chunk_size 64, bfloat16, no context parallelism "
                     "(no fallback path)")
  out_dtype = query.dtype
  if use_qk_norm_in_gdn:
    from maxtext.layers.normalizations import l2norm  # pylint: disable=import-outside-toplevel
    query, key = l2norm(query, dim=-1, eps=1e-6), l2norm(key, dim=-1, eps=1e-6)
  has_state = initial_state is not None
  b, s, h, kd = key.shape
  vd = value.shape[-1]
  core = _core()
  fwd_bytes = int(core.lewi_gdn_chunk_workspace_bytes(b, s, h, kd, vd))
  bwd_bytes = int(core.lewi_gdn_chunk_bwd_workspace_bytes(b, s, h, kd, vd))
  state_shape = (b, h, kd, vd)

  def call_fwd(q, k, v, gg, bb, h0):
    call = jax.ffi.ffi_call("lewi_ffi_gdn_chunk_fwd", (jax.ShapeDtypeStruct((b, s, h, vd), jnp.bfloat16),
                                                       jax.ShapeDtypeStruct(state_shape, jnp.float32),
                                                       jax.ShapeDtypeStruct((fwd_bytes,), jnp.uint8)))
    return call(q, k, v, gg, bb, h0, has_state=has_state)

  def run(q, k, v, gg, bb, h0):
    o, hf, _ = call_fwd(q, k, v, gg, bb, h0)
    return o, hf

  def forward(q, k, v, gg, bb, h0):
    o, hf, saved = call_fwd(q, k, v, gg, bb, h0)
    return (o, hf), (q, k, v, gg, bb, h0, saved)

  def backward(res, cot):
    q, k, v, gg, bb, h0, saved = res
    d_o, d_hf = cot
    call = jax.ffi.ffi_call("lewi_ffi_gdn_chunk_bwd", (jax.ShapeDtypeStruct(q.shape, jnp.bfloat16),
                                                       jax.ShapeDtypeStruct(k.shape, jnp.bfloat16),
                                                       jax.ShapeDtypeStruct(v.shape, jnp.bfloat16),
                                                       jax.ShapeDtypeStruct(gg.shape, jnp.float32),
                                                       jax.ShapeDtypeStruct(bb.shape, jnp.bfloat16),
                                                       jax.ShapeDtypeStruct(state_shape, jnp.float32),
                                                       jax.ShapeDtypeStruct((bwd_bytes,), jnp.uint8)))
    dq, dk, dv, dg, db, dh0, _ = call(q, k, v, gg, bb, h0, d_o.astype(jnp.bfloat16), d_hf.astype(jnp.float32), saved,
                                      has_state=has_state, has_dstate=True)
    return dq, dk, dv, dg, db, (dh0 if has_state else jnp.zeros_like(h0))

  op = jax.custom_vjp(run)
  op.defvjp(forward, backward)
  h0 = initial_state.astype(jnp.float32) if has_state else jnp.zeros((0,), jnp.float32)
  o, hf = op(query.astype(jnp.bfloat16), key.astype(jnp.bfloat16), value.astype(jnp.bfloat16), g.astype(jnp.float32),
             beta.astype(jnp.bfloat16), h0)
  return o.astype(out_dtype), (hf.astype(jnp.bfloat16) if has_state else None)


def install_seqmix(conv=True, gdn=True):
  """Patch the two sequence-mixing spots the reference patches: flax `nnx.Conv.__call__` for causal depthwise 1-D
  convolutions (modal/fast_conv.py:34-36; every other convolution goes to the original call, as there) and
  `maxtext.models.qwen3.jax_chunk_gated_delta_rule` (modal/gdn_fast.py:116-124; context-parallel calls go to the
  original, as there)."""
  _register()
  if conv:
    from flax import nnx  # pylint: disable=import-outside-toplevel
    stock = nnx.Conv.__call__

    def conv_call(self, inputs, **kwargs):
      k = self.kernel_size if isinstance(self.kernel_size, (tuple, list)) else (self.kernel_size,)
      depthwise = self.feature_group_count == self.in_features == self.out_features
      plain = (len(k) == 1 and depthwise and self.padding == "CAUSAL" and inputs.ndim == 3
               and (self.bias is None or self.bias.value is None)
               and getattr(self, "kernel_dilation", 1) in (1, (1,), None) and getattr(self, "strides", 1) in (1, (1,), None))
      if not plain or inputs.shape[-1] % 8 != 0:
        return stock(self, inputs, **kwargs)
      dtype = self.dtype or inputs.dtype
      return causal_conv1d(inputs.astype(dtype), self.kernel.value.astype(dtype))

    nnx.Conv.__call__ = conv_call
  if gdn:
    import maxtext.models.qwen3 as q3  # pylint: disable=import-outside-toplevel
    stock_gdn = q3.jax_chunk_gated_delta_rule

    def gdn_call(query, key, value, g, beta, chunk_size=64, initial_state=None, use_qk_norm_in_gdn=False, cp_axis=None,
                 **kw):
      if cp_axis is not None or chunk_size != 64 or key.shape[-1] > 128 or value.shape[-1] > 128:
        return stock_gdn(query, key, value, g, beta, chunk_size=chunk_size, initial_state=initial_state,
                         use_qk_norm_in_gdn=use_qk_norm_in_gdn, cp_axis=cp_axis, **kw)
      return chunk_gated_delta_rule(query, key, value, g, beta, chunk_size, initial_state, use_qk_norm_in_gdn)

    q3.jax_chunk_gated_delta_rule = gdn_call
  print(f"[lewi_surge_b200] sequence mixing: conv={conv} gated delta rule={gdn} (sm_100a kernels behind jax.ffi)", flush=True)
