"""CPU restatement (NumPy) of the reference's MoE-layer math.  TEST INFRASTRUCTURE ONLY.

This file is the checker for the CUDA path.  It is never imported by the product
package; only tests, the smoke check and the benchmark's CPU-baseline leg use it.

What is pinned and what is not
------------------------------
* sort / dispatch / combine / permute and their gradients restate
  ``modal/moe_permute.py:240-353`` and are pinned by golden vectors produced by running
  that file's own pure-array functions (see ``tests/golden/make_golden.py``).
* dropless ``ragged_dot`` semantics follow the known-answer check in
  ``modal/te_run.py:68-80`` (empty group, tail rows past ``sum(group_sizes)``); the
  capacity layout follows ``modal/padded_gmm.py:45-69`` and is pinned the same way.
* Router softmax/top-k/renormalise, the SwiGLU expert and the shared expert live in the
  third-party package ``maxtext==0.2.5`` (``maxtext.layers.moe.RoutedMoE``), whose source
  is not part of the reference tree.  They are restated from the reference's
  configuration (``configs/stage1.yml:33-41``: top-6, ``norm_topk_prob``) and weight
  layouts (``modal/stage2.py:338-345``, ``tools/grow_7b.py:104-112``) and cross-checked
  against the Hugging Face ``qwen3_5_moe`` block in the tests: PARITY UNPINNED for these.

Precision policy: inputs are bf16 values held in float32; all arithmetic is float32 (float64
for the soft-max ordering), no intermediate rounding unless asked for.
"""
from __future__ import annotations

import math

import numpy as np

__all__ = [
    "bf16_round", "rel_err", "softmax", "router_topk", "router_topk_bwd", "aux_loss", "aux_loss_bwd",
    "sort_indices", "block_layout", "padded_rows_bound",
    "gather_rows", "gather_reduce", "gather_dot",
    "dispatch", "dispatch_bwd", "combine", "combine_bwd", "permute_rows", "permute_rows_bwd",
    "ref_dispatch", "ref_combine", "moe_block",
    "ragged_dot", "ragged_dot_bwd", "padded_ragged_dot",
    "silu", "dsilu", "swiglu_experts_fwd", "swiglu_experts_bwd",
    "moe_layer_fwd", "moe_layer_bwd", "make_inputs", "zipf_bias",
]


# ----------------------------------------------------------------------------- helpers


def bf16_round(a):
  """Round float32 values to the nearest bfloat16 (ties to even); result stays float32."""
  a = np.ascontiguousarray(a, dtype=np.float32)
  u = a.view(np.uint32).astype(np.uint64)
  rounded = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
  out = rounded.view(np.float32).reshape(a.shape).copy()
  nan = np.isnan(a)
  if nan.any():
    out[nan] = np.nan
  return out


def rel_err(got, want):
  """The reference's error metric: max|got-want| / (max|want| + 1e-6) (modal/test_moe_permute.py:31)."""
  got = np.asarray(got, np.float64)
  want = np.asarray(want, np.float64)
  if got.shape != want.shape:
    return float("inf")
  if want.size == 0:
    return 0.0
  return float(np.abs(got - want).max() / (np.abs(want).max() + 1e-6))


# ----------------------------------------------------------------------------- router


def softmax(logits):
  """float32 soft-max over the last axis (max-subtracted)."""
  l = np.asarray(logits, np.float32)
  z = l - l.max(axis=-1, keepdims=True)
  e = np.exp(z, dtype=np.float32)
  return (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)


def router_topk(logits, k):
  """softmax -> top-k -> renormalise (configs/stage1.yml:36-37: num_experts_per_tok, norm_topk_prob).

  Selection order is by probability descending, lower expert index first on ties, which is
  what ``lax.top_k`` documents.  The ordering is decided in float64 so that two different
  float32 logits never collide; this equals ordering by (logit desc, index asc).
  Returns (idx int32 [T,k], w float32 [T,k], probs float32 [T,E]).
  """
  l = np.asarray(logits, np.float32)
  t, e = l.shape
  p = softmax(l)
  l64 = l.astype(np.float64)
  p64 = np.exp(l64 - l64.max(axis=-1, keepdims=True))
  # stable argsort of -p64 => descending probability, ascending index on ties
  idx = np.argsort(-p64, axis=-1, kind="stable")[:, :k].astype(np.int32)
  v = np.take_along_axis(p, idx, axis=-1)
  w = (v / v.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)
  return idx, w, p


def router_topk_bwd(logits, idx, dw):
  """Gradient of the renormalised top-k weights with respect to the logits.

  w_j = p_j / S, S = sum of the selected p; p = softmax(logits).
  """
  l = np.asarray(logits, np.float32)
  p = softmax(l).astype(np.float64)
  dw = np.asarray(dw, np.float64)
  v = np.take_along_axis(p, idx.astype(np.int64), axis=-1)
  s = v.sum(axis=-1, keepdims=True)
  w = v / s
  dv = (dw - (dw * w).sum(axis=-1, keepdims=True)) / s
  dp = np.zeros_like(p)
  np.put_along_axis(dp, idx.astype(np.int64), dv, axis=-1)
  dl = p * (dp - (p * dp).sum(axis=-1, keepdims=True))
  return dl.astype(np.float32)


def aux_loss(probs, idx, num_experts):
  """Load-balance loss E * sum_e f_e * P_e (configs/stage1.yml:41 weights it by 1e-3).

  f_e = fraction of the T*k routed slots that chose expert e, P_e = mean router probability.
  """
  t, k = idx.shape
  counts = np.bincount(idx.reshape(-1), minlength=num_experts).astype(np.float64)
  f = counts / float(t * k)
  pm = np.asarray(probs, np.float64).mean(axis=0)
  return float(num_experts * (f * pm).sum())


# ----------------------------------------------------------------------------- sort + layout


def sort_indices(flat_experts, num_experts=None, method="argsort"):
  """Stable sort of the N*k slots by expert id (modal/moe_permute.py:240-264).

  order[p] = slot at sorted position p, pos[i] = sorted position of slot i.
  method "count" restates the chunked one-hot counting sort of lines 252-264.
  """
  flat = np.asarray(flat_experts).astype(np.int32)
  m = flat.shape[0]
  if method == "argsort" or num_experts is None:
    order = np.argsort(flat, kind="stable").astype(np.int32)
    pos = np.argsort(order, kind="stable").astype(np.int32)
    return order, pos
  e = int(num_experts)
  chunk = 2048 if m % 2048 == 0 else m
  if m == 0:
    return np.zeros((0,), np.int32), np.zeros((0,), np.int32)
  onehot = (flat[:, None] == np.arange(e, dtype=np.int32)[None, :]).astype(np.int32).reshape(m // chunk, chunk, e)
  local = np.cumsum(onehot, axis=1)
  totals = local[:, -1, :]
  carry = np.cumsum(totals, axis=0) - totals
  counts = totals.sum(axis=0)
  offsets = np.cumsum(counts) - counts
  rank = (local + carry[:, None, :]).reshape(m, e) - 1
  rank = np.take_along_axis(rank, flat[:, None].astype(np.int64), axis=1)[:, 0]
  pos = (offsets[flat] + rank).astype(np.int32)
  order = np.zeros((m,), np.int32)
  order[pos] = np.arange(m, dtype=np.int32)
  return order, pos


def padded_rows_bound(m, num_experts, block=128):
  """Static upper bound on padded rows: every group rounded up to a multiple of ``block``."""
  return (m + num_experts * (block - 1)) // block * block


def block_layout(flat_experts, num_experts, block=128):
  """Dropless padded-block layout: each expert's group starts on a multiple of ``block`` rows.

  Returns a dict with
    counts[E], offsets[E+1] (unpadded exclusive prefix), pad_offsets[E+1] (padded prefix),
    n_blocks, block_expert[NBmax] (-1 past n_blocks), order[M], pos[M] (unpadded, as sort_indices),
    pad_pos[M] (padded row of slot i), row_slot[Mpad] (slot stored in padded row r, -1 = padding).
  """
  flat = np.asarray(flat_experts).astype(np.int32)
  m = flat.shape[0]
  e = int(num_experts)
  counts = np.bincount(flat, minlength=e).astype(np.int32)
  offsets = np.zeros(e + 1, np.int32)
  offsets[1:] = np.cumsum(counts)
  padded = (counts + block - 1) // block * block
  pad_offsets = np.zeros(e + 1, np.int32)
  pad_offsets[1:] = np.cumsum(padded)
  mpad = padded_rows_bound(m, e, block)
  nbmax = mpad // block
  n_blocks = int(pad_offsets[-1] // block)
  block_expert = np.full(nbmax, -1, np.int32)
  for ex in range(e):
    block_expert[pad_offsets[ex] // block: pad_offsets[ex + 1] // block] = ex
  order, pos = sort_indices(flat)
  rank = pos - offsets[flat]
  pad_pos = (pad_offsets[flat] + rank).astype(np.int32)
  row_slot = np.full(mpad, -1, np.int32)
  row_slot[pad_pos] = np.arange(m, dtype=np.int32)
  return dict(counts=counts, offsets=offsets, pad_offsets=pad_offsets, n_blocks=n_blocks,
              block_expert=block_expert, order=order, pos=pos, pad_pos=pad_pos, row_slot=row_slot,
              mpad=mpad, nbmax=nbmax)


# ----------------------------------------------------------------------------- gathers


def gather_rows(x, idx, scale=None, out_bf16=False):
  """out[i] = x[idx[i]] (* scale[i], multiplied in float32) (modal/moe_permute.py:116-121).

  A negative index yields a zero row (the padded layout's empty rows).
  """
  x = np.asarray(x, np.float32)
  idx = np.asarray(idx).astype(np.int64)
  out = x[np.clip(idx, 0, max(x.shape[0] - 1, 0))] if x.shape[0] else np.zeros((idx.shape[0],) + x.shape[1:], np.float32)
  out = np.where((idx >= 0)[:, None], out, np.float32(0))
  if scale is not None:
    out = out * np.asarray(scale, np.float32)[:, None]
  return bf16_round(out) if out_bf16 else out.astype(np.float32)


def gather_reduce(y, pos, w=None, out_bf16=False):
  """out[t] = sum_j w[t,j] * y[pos[t,j]] in float32 (modal/moe_permute.py:214-225)."""
  y = np.asarray(y, np.float32)
  n, k = pos.shape
  g = y[np.asarray(pos).astype(np.int64).reshape(-1)].reshape(n, k, -1)
  if w is not None:
    g = g * np.asarray(w, np.float32)[:, :, None]
  out = g.sum(axis=1, dtype=np.float32)
  return bf16_round(out) if out_bf16 else out


def gather_dot(y, pos, g):
  """out[t,j] = <g[t], y[pos[t,j]]> in float32 (modal/moe_permute.py:228-234)."""
  y = np.asarray(y, np.float32)
  n, k = pos.shape
  rows = y[np.asarray(pos).astype(np.int64).reshape(-1)].reshape(n, k, -1)
  return np.einsum("nkd,nd->nk", rows, np.asarray(g, np.float32)).astype(np.float32)


# ----------------------------------------------------------------------------- differentiable ops


def dispatch(x, order, pos):
  """x [N,D] -> [N*k,D], row p = x[order[p] // k] (modal/moe_permute.py:270-274)."""
  k = order.shape[0] // x.shape[0]
  return gather_rows(x, order // k)


def dispatch_bwd(g, order, pos, n):
  """Gradient of dispatch: gather_reduce(g, pos) without weights (modal/moe_permute.py:282-286)."""
  k = order.shape[0] // n
  return gather_reduce(g, pos.reshape(n, k), None)


def combine(y, order, pos, w):
  """out[t] = sum_j w[t,j] y[pos[t,j]] in float32 (modal/moe_permute.py:292-296)."""
  n, k = w.shape
  return gather_reduce(y, pos.reshape(n, k), w)


def combine_bwd(g, y, order, pos, w):
  """(dy, dw) of combine (modal/moe_permute.py:303-309)."""
  n, k = w.shape
  w_sorted = np.asarray(w, np.float32).reshape(-1)[order]
  dy = gather_rows(g, order // k, w_sorted)
  dw = gather_dot(y, pos.reshape(n, k), g)
  return dy, dw


def permute_rows(x, idx):
  """x[idx] for a permutation idx (modal/moe_permute.py:315-318)."""
  return gather_rows(x, idx)


def permute_rows_bwd(g, idx):
  """Gradient of permute_rows: gather with the inverse permutation (modal/moe_permute.py:325-326)."""
  return gather_rows(g, np.argsort(idx, kind="stable"))


def ref_dispatch(x, flat_experts):
  """modal/moe_permute.py:335-338."""
  k = flat_experts.shape[0] // x.shape[0]
  order = np.argsort(flat_experts, kind="stable")
  return np.asarray(x, np.float32)[order // k]


def ref_combine(y, flat_experts, w):
  """modal/moe_permute.py:341-345."""
  n, k = w.shape
  pos = np.argsort(np.argsort(flat_experts, kind="stable"), kind="stable")
  rows = np.asarray(y, np.float32)[pos].reshape(n, k, -1)
  return np.einsum("nkd,nk->nd", rows, np.asarray(w, np.float32)).astype(np.float32)


def moe_block(x, flat_experts, w, expert_fn):
  """dispatch -> expert_fn -> combine (modal/moe_permute.py:348-353, reference branch)."""
  return ref_combine(expert_fn(ref_dispatch(x, flat_experts)), flat_experts, w)


# ----------------------------------------------------------------------------- grouped GEMM


def ragged_dot(lhs, rhs, group_sizes):
  """Dropless grouped GEMM: row r of group g -> lhs[r] @ rhs[g]; rows past sum(group_sizes) -> 0.

  Semantics of ``jax.lax.ragged_dot`` as exercised by modal/te_run.py:68-80.
  """
  lhs = np.asarray(lhs, np.float32)
  rhs = np.asarray(rhs, np.float32)
  gs = np.asarray(group_sizes).astype(np.int64)
  out = np.zeros((lhs.shape[0], rhs.shape[2]), np.float32)
  s = 0
  for e, c in enumerate(gs):
    if c:
      out[s:s + c] = lhs[s:s + c] @ rhs[e]
    s += c
  return out


def ragged_dot_bwd(dout, lhs, rhs, group_sizes):
  """(dlhs, drhs) of ragged_dot.  Empty groups get an all-zero drhs; tail rows a zero dlhs."""
  lhs = np.asarray(lhs, np.float32)
  rhs = np.asarray(rhs, np.float32)
  dout = np.asarray(dout, np.float32)
  gs = np.asarray(group_sizes).astype(np.int64)
  dl = np.zeros_like(lhs)
  dr = np.zeros_like(rhs)
  s = 0
  for e, c in enumerate(gs):
    if c:
      dl[s:s + c] = dout[s:s + c] @ rhs[e].T
      dr[e] = lhs[s:s + c].T @ dout[s:s + c]
    s += c
  return dl, dr


def padded_ragged_dot(lhs, rhs, group_sizes, factor=2.0):
  """Fixed-capacity variant (modal/padded_gmm.py:45-69): rows past capacity C yield zeros."""
  lhs = np.asarray(lhs, np.float32)
  rhs = np.asarray(rhs, np.float32)
  m, k = lhs.shape
  e, _, n = rhs.shape
  c = int(math.ceil(m / e * factor))
  c = max(8, (c + 7) // 8 * 8)
  gs = np.asarray(group_sizes).astype(np.int32)
  starts = np.cumsum(gs) - gs
  rows = np.arange(m, dtype=np.int32)
  expert = np.minimum(np.searchsorted(np.cumsum(gs), rows, side="right"), e - 1).astype(np.int32)
  pos = rows - starts[expert]
  valid = (rows < gs.sum()) & (pos < c)
  slot = np.where(valid, expert * c + pos, e * c)
  se = np.arange(e * c, dtype=np.int32) // c
  sc = np.arange(e * c, dtype=np.int32) % c
  src = np.where(sc < np.minimum(gs[se], c), starts[se] + sc, m)
  lhs_ext = np.concatenate([lhs, np.zeros((1, k), np.float32)], axis=0)
  buf = lhs_ext[np.clip(src, 0, m)].reshape(e, c, k)
  out = np.einsum("eck,ekn->ecn", buf, rhs).reshape(e * c, n)
  out_ext = np.concatenate([out, np.zeros((1, n), np.float32)], axis=0)
  return out_ext[np.clip(slot, 0, e * c)]


# ----------------------------------------------------------------------------- SwiGLU experts


def silu(g):
  g = np.asarray(g, np.float32)
  return (g / (1.0 + np.exp(-g, dtype=np.float32))).astype(np.float32)


def dsilu(g):
  g = np.asarray(g, np.float32)
  s = (1.0 / (1.0 + np.exp(-g, dtype=np.float32))).astype(np.float32)
  return (s * (1.0 + g * (1.0 - s))).astype(np.float32)


def swiglu_experts_fwd(xs, w_gate, w_up, w_down, group_sizes):
  """Per expert group: h = silu(x Wg) * (x Wu); y = h Wd.

  Weight orientation: wi_0/wi_1 [E,d,f], wo [E,f,d] (modal/stage2.py:338-341; shapes as
  benchmarked in modal/gemm_bench.py:33-35).  Returns (y, g, u, h).
  """
  g = ragged_dot(xs, w_gate, group_sizes)
  u = ragged_dot(xs, w_up, group_sizes)
  h = silu(g) * u
  y = ragged_dot(h, w_down, group_sizes)
  return y, g, u, h


def swiglu_experts_bwd(dy, xs, w_gate, w_up, w_down, group_sizes, g, u, h):
  """Gradients of swiglu_experts_fwd: (dxs, dWg, dWu, dWd)."""
  dh, dwd = ragged_dot_bwd(dy, h, w_down, group_sizes)
  dg = dh * u * dsilu(g)
  du = dh * silu(g)
  dx1, dwg = ragged_dot_bwd(dg, xs, w_gate, group_sizes)
  dx2, dwu = ragged_dot_bwd(du, xs, w_up, group_sizes)
  return dx1 + dx2, dwg, dwu, dwd


# ----------------------------------------------------------------------------- whole layer


def moe_layer_fwd(x, w_router, w_gate, w_up, w_down, ws_gate, ws_up, ws_down, k,
                  router_bias=None, shared_gate=None, logits=None):
  """Full MoE layer forward in float32.  Returns (out [T,d], cache dict).

  router -> top-k -> dispatch (sorted, dropless) -> SwiGLU experts -> weighted combine, plus one
  always-on shared SwiGLU expert (configs/stage1.yml:32-37).  ``shared_gate`` ([d] vector) turns on
  the Hugging Face twin's sigmoid gate on the shared expert; None means gate == 1.
  ``logits`` overrides the router GEMM (used to feed the device's own logits to the checker).
  """
  x = np.asarray(x, np.float32)
  t, d = x.shape
  e = w_gate.shape[0]
  if logits is None:
    logits = x @ np.asarray(w_router, np.float32)
    if router_bias is not None:
      logits = logits + np.asarray(router_bias, np.float32)[None, :]
  logits = np.asarray(logits, np.float32)
  idx, w, p = router_topk(logits, k)
  flat = idx.reshape(-1)
  order, pos = sort_indices(flat)
  gs = np.bincount(flat, minlength=e).astype(np.int32)
  xs = dispatch(x, order, pos)
  y, g, u, h = swiglu_experts_fwd(xs, w_gate, w_up, w_down, gs)
  routed = combine(y, order, pos, w)
  sg = x @ np.asarray(ws_gate, np.float32)
  su = x @ np.asarray(ws_up, np.float32)
  sh = silu(sg) * su
  sy = sh @ np.asarray(ws_down, np.float32)
  if shared_gate is not None:
    zs = x @ np.asarray(shared_gate, np.float32)
    gate = (1.0 / (1.0 + np.exp(-zs))).astype(np.float32)
    out = routed + gate[:, None] * sy
  else:
    gate = None
    out = routed + sy
  cache = dict(logits=logits, idx=idx, w=w, p=p, order=order, pos=pos, gs=gs, xs=xs, y=y, g=g, u=u, h=h,
               sg=sg, su=su, sh=sh, sy=sy, gate=gate, routed=routed)
  return out.astype(np.float32), cache


def aux_loss_bwd(probs, idx, num_experts):
  """Gradient of aux_loss with respect to the LOGITS [T,E]; the token fractions f_e are constants
  (they come from an arg-max), so only the mean probabilities carry gradient."""
  p = np.asarray(probs, np.float64)
  t, k = idx.shape
  counts = np.bincount(idx.reshape(-1), minlength=num_experts).astype(np.float64)
  c = num_experts * counts / float(t * k) / float(t)          # d loss / d p[t,e], the same for every token
  return (p * (c[None, :] - (p * c[None, :]).sum(axis=-1, keepdims=True))).astype(np.float32)


def moe_layer_bwd(dout, x, w_router, w_gate, w_up, w_down, ws_gate, ws_up, ws_down, k, cache,
                  shared_gate=None, aux_weight=0.0):
  """Gradients of moe_layer_fwd for every differentiable input (plus ``aux_weight`` times the load-balance loss).

  Structure is the reference's gather-only backward (modal/moe_permute.py:282-309):
  dy = scaled gather of dout, dw = gather_dot, dx = gather_reduce.
  """
  x = np.asarray(x, np.float32)
  dout = np.asarray(dout, np.float32)
  c = cache
  t, d = x.shape
  dy, dw = combine_bwd(dout, c["y"], c["order"], c["pos"], c["w"])
  dxs, dwg, dwu, dwd = swiglu_experts_bwd(dy, c["xs"], w_gate, w_up, w_down, c["gs"], c["g"], c["u"], c["h"])
  dx = dispatch_bwd(dxs, c["order"], c["pos"], t)
  # shared expert
  if shared_gate is not None:
    gate = c["gate"]
    dsy = dout * gate[:, None]
    dgate = (dout * c["sy"]).sum(axis=1)
    dzs = dgate * gate * (1.0 - gate)
    dshared_gate = x.T @ dzs
    dx = dx + dzs[:, None] * np.asarray(shared_gate, np.float32)[None, :]
  else:
    dsy = dout
    dshared_gate = None
  dsh = dsy @ np.asarray(ws_down, np.float32).T
  dws_down = c["sh"].T @ dsy
  dsg = dsh * c["su"] * dsilu(c["sg"])
  dsu = dsh * silu(c["sg"])
  dws_gate = x.T @ dsg
  dws_up = x.T @ dsu
  dx = dx + dsg @ np.asarray(ws_gate, np.float32).T + dsu @ np.asarray(ws_up, np.float32).T
  # router
  dlogits = router_topk_bwd(c["logits"], c["idx"], dw)
  if aux_weight:
    dlogits = dlogits + np.float32(aux_weight) * aux_loss_bwd(c["p"], c["idx"], w_gate.shape[0])
  dw_router = x.T @ dlogits
  drouter_bias = dlogits.sum(axis=0)
  dx = dx + dlogits @ np.asarray(w_router, np.float32).T
  return dict(dx=dx.astype(np.float32), dw_router=dw_router.astype(np.float32), drouter_bias=drouter_bias,
              dw_gate=dwg, dw_up=dwu, dw_down=dwd, dws_gate=dws_gate.astype(np.float32),
              dws_up=dws_up.astype(np.float32), dws_down=dws_down.astype(np.float32),
              dshared_gate=dshared_gate, shared_gate_in=shared_gate, dw=dw, dlogits=dlogits)


# ----------------------------------------------------------------------------- synthetic inputs


def zipf_bias(num_experts, seed=0, s=1.2, scale=2.0):
  """Per-expert logit bias b_e = scale * ln(1 / rank_e**s) over a seeded random permutation of experts."""
  rng = np.random.default_rng(seed + 1000)
  rank = rng.permutation(num_experts) + 1
  return (scale * np.log(1.0 / rank.astype(np.float64) ** s)).astype(np.float32)


def make_inputs(t, d, e, f, fs, seed=0):
  """Seeded synthetic layer inputs with the benchmark's shapes and distributions.

  x, dout ~ N(0,1) rounded to bf16; router weight float32 ~ N(0,0.02); expert and shared-expert
  weights ~ N(0,0.02) rounded to bf16.  All arrays are float32 holding those values.
  """
  rng = np.random.default_rng(seed)
  n = lambda *shape, std=1.0: (rng.standard_normal(shape, dtype=np.float32) * np.float32(std))
  return dict(
      x=bf16_round(n(t, d)),
      w_router=n(d, e, std=0.02),
      w_gate=bf16_round(n(e, d, f, std=0.02)),
      w_up=bf16_round(n(e, d, f, std=0.02)),
      w_down=bf16_round(n(e, f, d, std=0.02)),
      ws_gate=bf16_round(n(d, fs, std=0.02)),
      ws_up=bf16_round(n(d, fs, std=0.02)),
      ws_down=bf16_round(n(fs, d, std=0.02)),
      dout=bf16_round(n(t, d)),
  )
