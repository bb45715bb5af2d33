"""Host-side mirror of the reference's MoE operators, backed by the sm_100a kernels.

Same names, argument meaning and shapes as ``modal/moe_permute.py`` (gather_rows, gather_reduce,
gather_dot, sort_indices, dispatch, combine, permute_rows, moe_block, CFG, install) and
``modal/padded_gmm.py`` / ``modal/te_gmm.py`` (a drop-in ``ragged_dot``).  Arrays are torch CUDA
tensors (device memory and streams only); differentiable ops are ``torch.autograd.Function`` s whose
backward passes have the reference's gather-only structure (``_dispatch_bwd``, ``_combine_bwd``,
``_permute_rows_bwd``: modal/moe_permute.py:282-329).

Unlike the reference there is no fallback: a shape the kernels cannot take raises ``LewiError``.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import BF16, F32, LewiError, check, ptr, stream

BLOCK = 128

# Same keys as the reference's CFG (modal/moe_permute.py:32-40) where they still mean something.
CFG = {
    "enabled": True,      # kept for signature compatibility; False raises (there is no second path)
    "tile": BLOCK,        # rows per padded block
    "sort": "count",      # the kernels implement the counting sort; "argsort" gives the same result
    "num_experts": None,
}


def _dt(t):
  if t.dtype == torch.bfloat16:
    return BF16
  if t.dtype == torch.float32:
    return F32
  raise LewiError(f"unsupported dtype {t.dtype}: the kernels take bfloat16 or float32")


def _i32(t):
  return t if t.dtype == torch.int32 else t.to(torch.int32)


def padded_rows_bound(m, num_experts, block=BLOCK):
  return int(_lib.load().lewi_padded_rows_bound(int(m), int(num_experts), int(block)))


def route_workspace(num_slots, num_experts, device):
  n = int(_lib.load().lewi_route_workspace_bytes(int(num_slots), int(num_experts)))
  return torch.empty(max(n, 256), dtype=torch.uint8, device=device)


# ----------------------------------------------------------------------------------- kernels


def gather_rows(x, idx, scale=None, *, idx_div=1, scale_by_idx=False, out=None, n_rows_dev=None, rows_per_unit=1):
  """out[i] = x[idx[i]] (* scale[i]).  x: (N, D), idx: (M,) int32, scale: (M,) f32 or None -> (M, D) x.dtype.

  Reference: gather_rows, modal/moe_permute.py:116-158.  A negative index gives a zero row.
  """
  lib = _lib.load()
  idx = _i32(idx).contiguous()
  x = x.contiguous()
  m, d = idx.shape[0], x.shape[1]
  if out is None:
    out = torch.empty((m, d), dtype=x.dtype, device=x.device)
  if scale is not None:
    scale = scale.to(torch.float32).contiguous()
  if m == 0:
    return out
  check(lib.lewi_gather_rows(stream(), ptr(x), ptr(idx), ptr(scale), ptr(out), x.shape[0], m, d, _dt(x),
                             int(idx_div), int(bool(scale_by_idx)), ptr(n_rows_dev), int(rows_per_unit)),
        "lewi_gather_rows")
  return out


def dispatch_rows(x, pad_pos, row_slot, *, out=None, n_rows_dev=None, rows_per_unit=1):
  """out[pad_pos[t,j]] = x[t]; padded rows without a slot become zero rows.  x: (T, D) bf16, pad_pos: (T, k) int32,
  row_slot: (Mpad,) int32 -> (Mpad, D).  Equals ``gather_rows(x, row_slot, idx_div=k)`` (the dispatch of
  modal/moe_permute.py:399-404), reading every token row once."""
  lib = _lib.load()
  t, k = pad_pos.shape
  d = x.shape[1]
  rows = row_slot.shape[0]
  if out is None:
    out = torch.empty((rows, d), dtype=x.dtype, device=x.device)
  if x.dtype != torch.bfloat16:
    raise LewiError("dispatch_rows takes bfloat16 rows")
  check(lib.lewi_dispatch_rows(stream(), ptr(x.contiguous()), ptr(_i32(pad_pos).contiguous()), ptr(_i32(row_slot).contiguous()),
                               ptr(out), t, k, d, rows, ptr(n_rows_dev), int(rows_per_unit)), "lewi_dispatch_rows")
  return out


def gather_reduce(y, pos, w=None, out_dtype=None, *, add0=None, add1=None, out=None):
  """out[t] = sum_j w[t,j] * y[pos[t,j]] in f32.  y: (M, D), pos: (N, k) int32, w: (N, k) or None -> (N, D).

  Reference: gather_reduce, modal/moe_permute.py:214-225.
  """
  lib = _lib.load()
  out_dtype = out_dtype or y.dtype
  pos = _i32(pos).contiguous()
  y = y.contiguous()
  n, k = pos.shape
  d = y.shape[1]
  if w is not None:
    w = w.to(torch.float32).contiguous()
  if out is None:
    out = torch.empty((n, d), dtype=out_dtype, device=y.device)
  for a in (add0, add1):
    if a is not None and a.dtype != y.dtype:
      raise LewiError("addends must have the dtype of y")
  if n == 0:
    return out
  check(lib.lewi_gather_reduce(stream(), ptr(y), ptr(pos), ptr(w), ptr(add0), ptr(add1), ptr(out), n, k, d, _dt(y),
                               _dt(out), y.shape[0]), "lewi_gather_reduce")
  return out


def gather_dot(y, pos, g):
  """out[t, j] = <g[t], y[pos[t,j]]> in f32.  y: (M, D), pos: (N, k), g: (N, D) -> (N, k) f32.

  Reference: gather_dot, modal/moe_permute.py:228-234.
  """
  lib = _lib.load()
  pos = _i32(pos).contiguous()
  y = y.contiguous()
  g = g.to(y.dtype).contiguous()
  n, k = pos.shape
  out = torch.empty((n, k), dtype=torch.float32, device=y.device)
  if n == 0:
    return out
  check(lib.lewi_gather_dot(stream(), ptr(y), ptr(pos), ptr(g), ptr(out), n, k, y.shape[1], _dt(y), y.shape[0]),
        "lewi_gather_dot")
  return out


def sort_indices(flat_experts, num_experts=None, method=None):
  """Stable sort of the N*k expert slots by expert id -> (order, pos).

  Reference: sort_indices, modal/moe_permute.py:240-264.  Both reference methods give the same
  result; the kernel is a counting sort, so ``num_experts`` is required.
  """
  del method
  num_experts = num_experts or CFG["num_experts"]
  if num_experts is None:
    raise LewiError("sort_indices needs num_experts (argument or CFG['num_experts'])")
  lib = _lib.load()
  flat = _i32(flat_experts).contiguous()
  m = flat.shape[0]
  order = torch.empty(m, dtype=torch.int32, device=flat.device)
  pos = torch.empty(m, dtype=torch.int32, device=flat.device)
  if m == 0:
    return order, pos
  ws = route_workspace(m, num_experts, flat.device)
  check(lib.lewi_sort_indices(stream(), ptr(flat), m, int(num_experts), 0, ptr(order), ptr(pos), None, None, None,
                              None, None, None, None, ptr(ws), ws.numel()), "lewi_sort_indices")
  return order, pos


# ----------------------------------------------------------------------------------- differentiable ops


class _Dispatch(torch.autograd.Function):
  """x: (N, D) -> (N*k, D), row p = x[order[p] // k].  Backward: gather_reduce(g, pos) (no x saved)."""

  @staticmethod
  def forward(ctx, x, order, pos):
    n = x.shape[0]
    k = order.shape[0] // n
    ctx.save_for_backward(pos)
    ctx.n, ctx.k, ctx.dtype = n, k, x.dtype
    return gather_rows(x, order, idx_div=k)

  @staticmethod
  def backward(ctx, g):
    (pos,) = ctx.saved_tensors
    return gather_reduce(g.contiguous(), pos.view(ctx.n, ctx.k), None, ctx.dtype), None, None


class _Combine(torch.autograd.Function):
  """y: (N*k, D) sorted rows, w: (N, k) -> (N, D) f32.  Backward: scaled gather (dy) and gather_dot (dw)."""

  @staticmethod
  def forward(ctx, y, order, pos, w):
    n, k = w.shape
    ctx.save_for_backward(y, order, pos, w)
    return gather_reduce(y, pos.view(n, k), w, torch.float32)

  @staticmethod
  def backward(ctx, g):
    y, order, pos, w = ctx.saved_tensors
    n, k = w.shape
    gy = g.to(y.dtype).contiguous()
    # dy[p] = w_flat[order[p]] * g[order[p] // k]
    dy = gather_rows(gy, order, w.reshape(-1), idx_div=k, scale_by_idx=True)
    dw = gather_dot(y, pos.view(n, k), gy).to(w.dtype)
    return dy, None, None, dw


class _PermuteRows(torch.autograd.Function):
  """x[idx] for a permutation idx; backward gathers with the inverse permutation."""

  @staticmethod
  def forward(ctx, x, idx):
    ctx.save_for_backward(idx)
    return gather_rows(x, idx)

  @staticmethod
  def backward(ctx, g):
    (idx,) = ctx.saved_tensors
    inv = torch.empty_like(idx)
    inv[idx.long()] = torch.arange(idx.shape[0], dtype=idx.dtype, device=idx.device)
    return gather_rows(g.contiguous(), inv), None


def dispatch(x, order, pos):
  """Reference: dispatch, modal/moe_permute.py:270-289."""
  return _Dispatch.apply(x, _i32(order), _i32(pos))


def combine(y, order, pos, w):
  """Reference: combine, modal/moe_permute.py:292-312."""
  return _Combine.apply(y, _i32(order), _i32(pos), w)


def permute_rows(x, idx):
  """Reference: permute_rows, modal/moe_permute.py:315-329."""
  return _PermuteRows.apply(x, _i32(idx))


def moe_block(x, flat_experts, w, expert_fn, use_kernels=True):
  """dispatch -> expert_fn(rows) -> combine.  Reference: moe_block, modal/moe_permute.py:348-353."""
  if not use_kernels:
    raise LewiError("there is no second (XLA-style) path in this library; the oracle lives in the tests")
  order, pos = sort_indices(flat_experts, CFG["num_experts"])
  return combine(expert_fn(dispatch(x, order, pos)), order, pos, w)


# ----------------------------------------------------------------------------------- grouped GEMM


def group_tables(group_sizes, m, block=BLOCK):
  """Padded-block tables for rows that are already sorted by expert (see lewi_group_tables)."""
  lib = _lib.load()
  gs = _i32(group_sizes).contiguous()
  e = gs.shape[0]
  mpad = padded_rows_bound(m, e, block)
  dev = gs.device
  pad_offsets = torch.empty(e + 1, dtype=torch.int32, device=dev)
  block_expert = torch.empty(max(mpad // block, 1), dtype=torch.int32, device=dev)
  n_blocks = torch.empty(1, dtype=torch.int32, device=dev)
  row_of_padded = torch.empty(max(mpad, 1), dtype=torch.int32, device=dev)
  padded_of_row = torch.empty(max(m, 1), dtype=torch.int32, device=dev)
  check(lib.lewi_group_tables(stream(), ptr(gs), m, e, block, ptr(pad_offsets), ptr(block_expert), ptr(n_blocks),
                              ptr(row_of_padded), ptr(padded_of_row)), "lewi_group_tables")
  return dict(pad_offsets=pad_offsets, block_expert=block_expert, n_blocks=n_blocks,
              row_of_padded=row_of_padded[:mpad], padded_of_row=padded_of_row[:m], mpad=mpad)


def grouped_gemm_nn(a, b, block_expert, n_blocks, out_dtype=torch.bfloat16, row_scale=None, out=None, pad_offsets=None):
  """out[r] = a[r] . b[expert of r's block];  a (rows, K), b (E, K, N).  With ``pad_offsets`` the CTA-pair kernel runs."""
  lib = _lib.load()
  rows, k = a.shape
  e, _, n = b.shape
  if out is None:
    out = torch.empty((rows, n), dtype=out_dtype, device=a.device)
  check(lib.lewi_grouped_gemm_nn(stream(), ptr(a), ptr(b), ptr(out), ptr(row_scale), ptr(block_expert),
                                 ptr(n_blocks), ptr(pad_offsets), rows, k, n, e, _dt(out)), "lewi_grouped_gemm_nn")
  return out


def grouped_gemm_nt(a, b, block_expert, n_blocks, out_dtype=torch.bfloat16, row_scale=None, out=None, pad_offsets=None):
  """out[r] = a[r] . b[expert]^T;  a (rows, K), b (E, N, K)."""
  lib = _lib.load()
  rows, k = a.shape
  e, n, _ = b.shape
  if out is None:
    out = torch.empty((rows, n), dtype=out_dtype, device=a.device)
  check(lib.lewi_grouped_gemm_nt(stream(), ptr(a), ptr(b), ptr(out), ptr(row_scale), ptr(block_expert),
                                 ptr(n_blocks), ptr(pad_offsets), rows, k, n, e, _dt(out)), "lewi_grouped_gemm_nt")
  return out


def grouped_gemm_tn(a, b, pad_offsets, num_experts, out_dtype=torch.bfloat16, out=None, out2=None, split=False):
  """out[e] = a[rows of e]^T . b[rows of e];  a (rows, Ma), b (rows, Nb) -> (E, Ma, Nb).

  With ``split`` the product's columns are written as two (E, Ma, Nb/2) tensors.  Long contractions are cut into
  parts (one group: evenly; several experts: only the experts far above the mean) that are summed in a fixed order.
  """
  lib = _lib.load()
  ma, nb = a.shape[1], b.shape[1]
  rows = a.shape[0]
  if split:
    if out is None:
      out = torch.empty((num_experts, ma, nb // 2), dtype=out_dtype, device=a.device)
    if out2 is None:
      out2 = torch.empty((num_experts, ma, nb // 2), dtype=out_dtype, device=a.device)
  elif out is None:
    out = torch.empty((num_experts, ma, nb), dtype=out_dtype, device=a.device)
  ws_bytes = int(lib.lewi_grouped_gemm_tn_workspace_bytes(rows, ma, nb, int(num_experts), int(bool(split))))
  ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device) if ws_bytes > 0 else None
  check(lib.lewi_grouped_gemm_tn(stream(), ptr(a), ptr(b), ptr(out), ptr(out2), ptr(pad_offsets), rows, ma, nb,
                                 int(num_experts), _dt(out), ptr(ws), ws_bytes), "lewi_grouped_gemm_tn")
  return (out, out2) if split else out


class _RaggedDot(torch.autograd.Function):
  """Dropless grouped GEMM with the reference's gather -> batched GEMM -> gather structure.

  Reference: padded_ragged_dot, modal/padded_gmm.py:45-69 (and te_ragged_dot, modal/te_gmm.py:12-19
  for the dropless semantics): rows of lhs are sorted by expert, group g multiplies rhs[g], rows past
  sum(group_sizes) yield zeros.  Both the forward and the backward only gather (never scatter).
  """

  @staticmethod
  def forward(ctx, lhs, rhs, group_sizes):
    m, _ = lhs.shape
    e = rhs.shape[0]
    t = group_tables(group_sizes, m)
    a = lhs.to(torch.bfloat16).contiguous()
    b = rhs.to(torch.bfloat16).contiguous()
    buf = gather_rows(a, t["row_of_padded"])
    out_pad = grouped_gemm_nn(buf, b, t["block_expert"], t["n_blocks"], pad_offsets=t["pad_offsets"])
    out = gather_rows(out_pad, t["padded_of_row"])
    ctx.save_for_backward(buf, b, t["row_of_padded"], t["padded_of_row"], t["block_expert"], t["n_blocks"],
                          t["pad_offsets"])
    ctx.e, ctx.lhs_dtype, ctx.rhs_dtype = e, lhs.dtype, rhs.dtype
    return out.to(lhs.dtype)

  @staticmethod
  def backward(ctx, g):
    buf, b, row_of_padded, padded_of_row, block_expert, n_blocks, pad_offsets = ctx.saved_tensors
    g_pad = gather_rows(g.to(torch.bfloat16).contiguous(), row_of_padded)
    # dlhs = g . rhs[e]^T: rhs [E,K,N] read as the K-major operand with contraction over N
    dl_pad = grouped_gemm_nt(g_pad, b, block_expert, n_blocks, pad_offsets=pad_offsets)
    dlhs = gather_rows(dl_pad, padded_of_row)
    drhs = grouped_gemm_tn(buf, g_pad, pad_offsets, ctx.e, out_dtype=torch.float32)
    return dlhs.to(ctx.lhs_dtype), drhs.to(ctx.rhs_dtype), None


def ragged_dot(lhs, rhs, group_sizes, precision=None, preferred_element_type=None, **kw):
  """Drop-in for ``jax.lax.ragged_dot`` as patched by the reference (modal/padded_gmm.py:45)."""
  del precision, preferred_element_type
  if lhs.dim() != 2 or rhs.dim() != 3 or kw.get("group_offset") is not None:
    raise LewiError("ragged_dot: only lhs [M,K], rhs [E,K,N] without group_offset is supported")
  return _RaggedDot.apply(lhs, rhs, _i32(group_sizes))


padded_ragged_dot = ragged_dot
te_ragged_dot = ragged_dot


def install(mode="full", tile=None, sort=None, num_experts=None, factor=None, probe=True):
  """Record the configuration the way the reference's installers do and load the CUDA library.

  Reference: install, modal/moe_permute.py:386-436 and modal/padded_gmm.py:72-76.  The MaxText patch
  itself lives in ``jax_ops.install`` (it needs JAX); this call configures the torch-facing operators.
  """
  del probe, factor
  if tile and int(tile) != BLOCK:
    raise LewiError(f"the padded-block size is fixed at {BLOCK} rows")
  if sort:
    CFG["sort"] = sort
  if num_experts:
    CFG["num_experts"] = int(num_experts)
  _lib.load()
  print(f"[lewi_surge_b200] installed mode={mode} block={BLOCK} sort={CFG['sort']} "
        f"num_experts={CFG['num_experts']} (sm_100a kernels, C ABI v{_lib.load().lewi_version()})", flush=True)
