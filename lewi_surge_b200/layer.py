"""The whole MoE layer, forward and backward, as one sequence of kernel launches.

Forward (reference call stack: router -> top-k -> `_route_activations` -> three `ragged_dot` s ->
`unpermute`, see modal/moe_permute.py:399-433 and modal/padded_gmm.py:45-69):

  logits  = x . W_r                                   lewi_router_logits
  tables  = softmax/top-k/renorm + stable sort        lewi_router_topk
  xs      = rows of x in padded-block order           lewi_gather_rows      (dispatch)
  gu, h   = SwiGLU(xs . Wg[e], xs . Wu[e])            lewi_grouped_gemm_gateup_swiglu
  ys      = h . Wd[e]                                 lewi_grouped_gemm_nn
  shared expert on all tokens (same two kernels, one group)
  out[t]  = sum_j w[t,j] ys[row(t,j)] + shared[t]     lewi_gather_reduce    (combine)

Backward is gather-only like the reference's (modal/moe_permute.py:282-309): dy by a scaled gather,
dw by gather_dot, dx by gather_reduce; weight gradients are per-expert transposed GEMMs over the
padded rows (padding rows are exact zeros, so they add nothing).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import check, ptr, stream
from . import ops

BLOCK = ops.BLOCK

_HOOK = None


def set_profile_hook(fn):
  """fn(name) is called after every kernel launch of the layer (used to drop CUDA events); None disables."""
  global _HOOK
  _HOOK = fn


def _mark(name):
  if _HOOK is not None:
    _HOOK(name)


# The shared expert depends only on x (forward) / dout (backward), so it runs on a side stream next to the
# memory-bound routing and gather kernels of the routed path and is joined before the combine.
OVERLAP_SHARED = True
# Carry the router weight through h (the down projection then yields weighted outputs and the combine needs no
# weights), scale dh by it in the dH epilogue and take the routing-weight gradient from that epilogue instead of a
# separate gather_dot pass.
FUSED_EPILOGUE = True
# Additionally pick the rows of x / dout inside the GEMM producer warp instead of materialising permuted copies.
# Correct (bit-identical) but measured 3-5x slower on B200: one producer warp cannot keep enough 16-byte copies in
# flight, and TMA gather4 moves only ~85 rows per microsecond per SM.  Kept for experiments, off by default.
FUSED_GATHER = False
_SIDE = {}


def _side_stream(device):
  st = _SIDE.get(device)
  if st is None:
    st = _SIDE[device] = torch.cuda.Stream(device=device)
  return st


class _Fork:
  """Runs a block on the side stream after everything already queued on the current one."""

  def __init__(self, device, enabled):
    self.enabled = enabled
    self.main = torch.cuda.current_stream(device)
    self.side = _side_stream(device) if enabled else None
    self.ctx = None

  def __enter__(self):
    if self.enabled:
      self.side.wait_stream(self.main)
      self.ctx = torch.cuda.stream(self.side)
      self.ctx.__enter__()
      _mark("side_begin")
    return self

  def __exit__(self, *exc):
    if self.enabled:
      self.ctx.__exit__(*exc)
    return False

  def join(self, *tensors):
    """Makes the current stream wait for the side stream; `tensors` were produced there and are used here."""
    if self.enabled:
      self.main.wait_stream(self.side)
      for t in tensors:
        if t is not None:
          t.record_stream(self.main)


@dataclass
class MoEWeights:
  """Parameter tensors in the reference's orientation (modal/stage2.py:338-345).

  w_router [d,E] f32 (experts on the last axis); w_gate, w_up [E,d,f] (wi_0, wi_1), w_down [E,f,d] (wo),
  shared expert ws_gate, ws_up [d,fs], ws_down [fs,d]; all expert weights bf16.
  """
  w_router: torch.Tensor
  w_gate: torch.Tensor
  w_up: torch.Tensor
  w_down: torch.Tensor
  ws_gate: Optional[torch.Tensor] = None
  ws_up: Optional[torch.Tensor] = None
  ws_down: Optional[torch.Tensor] = None
  router_bias: Optional[torch.Tensor] = None


@dataclass
class RouteTables:
  topk_idx: torch.Tensor
  topk_w: torch.Tensor
  counts: torch.Tensor
  offsets: torch.Tensor
  pad_offsets: torch.Tensor
  block_expert: torch.Tensor
  n_blocks: torch.Tensor
  order: torch.Tensor
  pos: torch.Tensor
  pad_pos: torch.Tensor
  row_slot: torch.Tensor
  probs_sum: torch.Tensor
  mpad: int


def router_logits(x, w_router, bias=None, tensor_cores=True):
  lib = _lib.load()
  t, d = x.shape
  e = w_router.shape[1]
  logits = torch.empty((t, e), dtype=torch.float32, device=x.device)
  ws_bytes = int(lib.lewi_router_logits_workspace_bytes(d, e)) if tensor_cores else 0
  ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes > 0 else None
  check(lib.lewi_router_logits(stream(), ptr(x), ptr(w_router), ptr(bias), ptr(logits), t, d, e, ptr(ws), ws_bytes),
        "lewi_router_logits")
  return logits


def router_topk(logits, k, block=BLOCK):
  """softmax -> top-k -> renormalise + stable sort of the T*k slots + padded-block tables."""
  lib = _lib.load()
  t, e = logits.shape
  m = t * k
  dev = logits.device
  mpad = ops.padded_rows_bound(m, e, block)
  i32 = dict(dtype=torch.int32, device=dev)
  tb = RouteTables(
      topk_idx=torch.empty((t, k), **i32), topk_w=torch.empty((t, k), dtype=torch.float32, device=dev),
      counts=torch.empty(e, **i32), offsets=torch.empty(e + 1, **i32), pad_offsets=torch.empty(e + 1, **i32),
      block_expert=torch.empty(max(mpad // block, 1), **i32), n_blocks=torch.empty(1, **i32),
      order=torch.empty(max(m, 1), **i32)[:m], pos=torch.empty(max(m, 1), **i32)[:m],
      pad_pos=torch.empty(max(m, 1), **i32)[:m], row_slot=torch.empty(max(mpad, 1), **i32)[:mpad],
      probs_sum=torch.empty(e, dtype=torch.float32, device=dev), mpad=mpad)
  ws = ops.route_workspace(m, e, dev)
  check(lib.lewi_router_topk(stream(), ptr(logits), t, e, k, block, ptr(tb.topk_idx), ptr(tb.topk_w), ptr(tb.counts),
                             ptr(tb.offsets), ptr(tb.pad_offsets), ptr(tb.block_expert), ptr(tb.n_blocks),
                             ptr(tb.order), ptr(tb.pos), ptr(tb.pad_pos), ptr(tb.row_slot), ptr(tb.probs_sum),
                             ptr(ws), ws.numel()), "lewi_router_topk")
  return tb


def router_topk_bwd(logits, topk_idx, dw, want_f32=True, want_bf16=False, dw_partial=None, pad_pos=None):
  """dlogits (f32 and/or bf16).  ``dw`` [T,k], or its pieces ``dw_partial`` [rows,parts] + ``pad_pos``; in
  the latter case the summed dw is returned as a third value."""
  lib = _lib.load()
  t, e = logits.shape
  k = topk_idx.shape[1]
  dl = torch.empty_like(logits) if want_f32 else None
  dlb = torch.empty((t, e), dtype=torch.bfloat16, device=logits.device) if want_bf16 else None
  if dw_partial is None:
    check(lib.lewi_router_topk_bwd(stream(), ptr(logits), ptr(topk_idx), ptr(dw.contiguous()), ptr(dl), ptr(dlb), t, e, k),
          "lewi_router_topk_bwd")
    return dl, dlb
  dw_out = torch.empty((t, k), dtype=torch.float32, device=logits.device)
  check(lib.lewi_router_topk_bwd_partial(stream(), ptr(logits), ptr(topk_idx), None, ptr(dw_partial),
                                         dw_partial.shape[1], ptr(pad_pos), ptr(dw_out), ptr(dl), ptr(dlb), t, e, k),
        "lewi_router_topk_bwd_partial")
  return dl, dlb, dw_out


def cast_bf16(src):
  lib = _lib.load()
  dst = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
  check(lib.lewi_cast_f32_to_bf16(stream(), ptr(src.contiguous()), ptr(dst), src.numel()), "lewi_cast_f32_to_bf16")
  return dst


def gateup_swiglu(xs, w_gate, w_up, block_expert, n_blocks, want_gu=True, pad_offsets=None, row_idx=None, idx_div=1,
                  rows=None, h_scale_src=None, scale_idx=None):
  """(gu [rows,2f], h [rows,f]) = fused gate/up projection + SwiGLU over the padded rows.

  With ``row_idx`` the dispatch gather is fused in: ``xs`` is the unpermuted source, padded row r reads
  ``xs[row_idx[r] // idx_div]`` and ``rows`` is the padded row count; ``h_scale_src[row_idx[r]]`` scales h."""
  lib = _lib.load()
  e, d, f = w_gate.shape
  src_rows = xs.shape[0]
  rows = src_rows if row_idx is None else int(rows)
  gu = torch.empty((rows, 2 * f), dtype=torch.bfloat16, device=xs.device) if want_gu else None
  h = torch.empty((rows, f), dtype=torch.bfloat16, device=xs.device)
  check(lib.lewi_grouped_gemm_gateup_swiglu_gather(stream(), ptr(xs), ptr(row_idx), int(idx_div), src_rows,
                                                   ptr(scale_idx), ptr(h_scale_src), ptr(w_gate), ptr(w_up), ptr(gu), ptr(h),
                                                   ptr(block_expert), ptr(n_blocks), ptr(pad_offsets), rows, d, f, e),
        "lewi_grouped_gemm_gateup_swiglu")
  return gu, h


def dh_dswiglu(dys, w_down, gu, block_expert, n_blocks, pad_offsets=None, row_idx=None, idx_div=1, scale_src=None,
               want_dw_partial=False, scale_idx=None):
  """dgu [rows,2f] = SwiGLU'(gu) applied to dh = dys . w_down[e]^T.

  With ``row_idx`` the upstream-gradient gather is fused in (``dys`` is the unpermuted [T,d] gradient),
  ``scale_src[row_idx[r]]`` multiplies dh, and ``want_dw_partial`` also returns the routing-weight
  gradient pieces [rows, parts] f32."""
  lib = _lib.load()
  e, f, d = w_down.shape
  rows = gu.shape[0]
  dgu = torch.empty((rows, 2 * f), dtype=torch.bfloat16, device=dys.device)
  dwp = None
  if want_dw_partial:
    dwp = torch.empty((rows, int(lib.lewi_dw_partial_parts(f))), dtype=torch.float32, device=dys.device)
  check(lib.lewi_grouped_gemm_dh_dswiglu_gather(stream(), ptr(dys), ptr(row_idx), int(idx_div), dys.shape[0],
                                                ptr(scale_idx), ptr(scale_src), ptr(dwp), ptr(w_down), ptr(gu), ptr(dgu),
                                                ptr(block_expert), ptr(n_blocks), ptr(pad_offsets), rows, d, f, e),
        "lewi_grouped_gemm_dh_dswiglu")
  return (dgu, dwp) if want_dw_partial else dgu


def dx_from_dgu(dgu, w_gate, w_up, block_expert, n_blocks, pad_offsets=None):
  lib = _lib.load()
  rows = dgu.shape[0]
  e, d, f = w_gate.shape
  dxs = torch.empty((rows, d), dtype=torch.bfloat16, device=dgu.device)
  check(lib.lewi_grouped_gemm_dx(stream(), ptr(dgu), ptr(w_gate), ptr(w_up), ptr(dxs), ptr(block_expert),
                                 ptr(n_blocks), ptr(pad_offsets), rows, d, f, e), "lewi_grouped_gemm_dx")
  return dxs


@dataclass
class LayerCache:
  x: torch.Tensor
  logits: torch.Tensor
  tables: RouteTables
  xs: torch.Tensor
  gu: torch.Tensor
  h: torch.Tensor
  ys: torch.Tensor
  gus: Optional[torch.Tensor]
  hs: Optional[torch.Tensor]
  k: int
  fused: bool = False


def moe_layer_fwd(x, w: MoEWeights, k, logits=None):
  """x [T,d] bf16 -> (out [T,d] bf16, cache).  ``logits`` (f32 [T,E]) replaces the router GEMM."""
  t, d = x.shape
  if logits is None:
    logits = router_logits(x, w.w_router, w.router_bias)
    _mark("router_logits")
  gus = hs = ysh = None
  fork = _Fork(x.device, OVERLAP_SHARED and w.ws_gate is not None)
  if w.ws_gate is not None:
    with fork:
      gus, hs = gateup_swiglu(x, w.ws_gate[None], w.ws_up[None], None, None)
      _mark("shared_gateup_swiglu")
      ysh = ops.grouped_gemm_nn(hs, w.ws_down[None], None, None)
      _mark("shared_down")
  tb = router_topk(logits, k)
  _mark("router_topk")
  # dispatch: padded row r holds token row_slot[r] // k (zero row where row_slot[r] < 0)
  fused = FUSED_EPILOGUE or FUSED_GATHER
  wflat = tb.topk_w.view(-1)
  if FUSED_GATHER:
    # rows of x are picked by the producer warp; h carries the router weight, so ys is already weighted
    xs = None
    gu, h = gateup_swiglu(x, w.w_gate, w.w_up, tb.block_expert, tb.n_blocks, pad_offsets=tb.pad_offsets,
                          row_idx=tb.row_slot, idx_div=k, rows=tb.mpad, h_scale_src=wflat)
  else:
    xs = torch.empty((tb.mpad, d), dtype=x.dtype, device=x.device)
    ops.gather_rows(x, tb.row_slot, idx_div=k, out=xs, n_rows_dev=tb.n_blocks, rows_per_unit=BLOCK)
    _mark("dispatch_gather")
    gu, h = gateup_swiglu(xs, w.w_gate, w.w_up, tb.block_expert, tb.n_blocks, pad_offsets=tb.pad_offsets,
                          scale_idx=tb.row_slot if fused else None, h_scale_src=wflat if fused else None)
  _mark("gemm_gateup_swiglu")
  ys = ops.grouped_gemm_nn(h, w.w_down, tb.block_expert, tb.n_blocks, pad_offsets=tb.pad_offsets)
  _mark("gemm_down")
  fork.join(gus, hs, ysh)
  out = ops.gather_reduce(ys, tb.pad_pos.view(t, k), None if fused else tb.topk_w, x.dtype, add0=ysh)
  _mark("combine_gather_reduce")
  return out, LayerCache(x=x, logits=logits, tables=tb, xs=xs, gu=gu, h=h, ys=ys, gus=gus, hs=hs, k=k, fused=fused)


def moe_layer_bwd(dout, w: MoEWeights, c: LayerCache):
  """Gradients for x and every weight, given dout [T,d] bf16."""
  x, tb, k = c.x, c.tables, c.k
  t, d = x.shape
  e = w.w_gate.shape[0]
  dout = dout.contiguous()
  pad_pos = tb.pad_pos.view(t, k)
  # shared expert backward: needs only dout, x and its own saved activations -> side stream
  dxsh = None
  shared_grads = {}
  fork = _Fork(x.device, OVERLAP_SHARED and w.ws_gate is not None)
  if w.ws_gate is not None:
    with fork:
      dgus = dh_dswiglu(dout, w.ws_down[None], c.gus, None, None)
      _mark("shared_dh_dswiglu")
      dws_down = ops.grouped_gemm_tn(c.hs, dout, None, 1, out_dtype=w.ws_down.dtype)[0]
      _mark("shared_dw_down")
      dxsh = dx_from_dgu(dgus, w.ws_gate[None], w.ws_up[None], None, None)
      _mark("shared_dx")
      dws_gate, dws_up = ops.grouped_gemm_tn(x, dgus, None, 1, out_dtype=w.ws_gate.dtype, split=True)
      _mark("shared_dw_gateup")
      shared_grads = dict(dws_gate=dws_gate[0], dws_up=dws_up[0], dws_down=dws_down)
  dw = dw_partial = None
  wflat = tb.topk_w.view(-1)
  if c.fused and c.xs is not None:
    # unscaled gather of dout into padded order; the router weight scales dh in the dH epilogue, which also emits
    # the pieces of the routing-weight gradient <dout[t], y[row]> = sum_n dh[row,n] * h[row,n]
    dys = torch.empty_like(c.ys)
    ops.gather_rows(dout, tb.row_slot, idx_div=k, out=dys, n_rows_dev=tb.n_blocks, rows_per_unit=BLOCK)
    _mark("combine_bwd_gather")
    dgu, dw_partial = dh_dswiglu(dys, w.w_down, c.gu, tb.block_expert, tb.n_blocks, pad_offsets=tb.pad_offsets,
                                 scale_idx=tb.row_slot, scale_src=wflat, want_dw_partial=True)
    _mark("gemm_dh_dswiglu")
    dw_down = ops.grouped_gemm_tn(c.h, dys, tb.pad_offsets, e, out_dtype=w.w_down.dtype)
    _mark("gemm_dw_down")
    dxs = dx_from_dgu(dgu, w.w_gate, w.w_up, tb.block_expert, tb.n_blocks, pad_offsets=tb.pad_offsets)
    _mark("gemm_dx")
    dw_gate, dw_up = ops.grouped_gemm_tn(c.xs, dgu, tb.pad_offsets, e, out_dtype=w.w_gate.dtype, split=True)
    _mark("gemm_dw_gateup")
  elif c.fused:
    # dout rows are picked by the producer warps
    dgu, dw_partial = dh_dswiglu(dout, w.w_down, c.gu, tb.block_expert, tb.n_blocks, pad_offsets=tb.pad_offsets,
                                 row_idx=tb.row_slot, idx_div=k, scale_src=wflat, want_dw_partial=True)
    _mark("gemm_dh_dswiglu")
    dw_down = ops.grouped_gemm_tn(c.h, dout, tb.pad_offsets, e, out_dtype=w.w_down.dtype, row_idx=tb.row_slot,
                                  idx_div=k, gather_b=True, rows=tb.mpad)
    _mark("gemm_dw_down")
    dxs = dx_from_dgu(dgu, w.w_gate, w.w_up, tb.block_expert, tb.n_blocks, pad_offsets=tb.pad_offsets)
    _mark("gemm_dx")
    dw_gate, dw_up = ops.grouped_gemm_tn(x, dgu, tb.pad_offsets, e, out_dtype=w.w_gate.dtype, split=True,
                                         row_idx=tb.row_slot, idx_div=k, gather_a=True, rows=tb.mpad)
    _mark("gemm_dw_gateup")
  else:
    # combine backward: dw = <g, y>, dy = w * g (scaled gather into padded order)
    dw = ops.gather_dot(c.ys, pad_pos, dout)
    _mark("combine_bwd_gather_dot")
    dys = torch.empty_like(c.ys)
    ops.gather_rows(dout, tb.row_slot, tb.topk_w.view(-1), idx_div=k, scale_by_idx=True, out=dys,
                    n_rows_dev=tb.n_blocks, rows_per_unit=BLOCK)
    _mark("combine_bwd_scaled_gather")
    # experts backward
    dgu = dh_dswiglu(dys, w.w_down, c.gu, tb.block_expert, tb.n_blocks, pad_offsets=tb.pad_offsets)
    _mark("gemm_dh_dswiglu")
    dw_down = ops.grouped_gemm_tn(c.h, dys, tb.pad_offsets, e, out_dtype=w.w_down.dtype)
    _mark("gemm_dw_down")
    dxs = dx_from_dgu(dgu, w.w_gate, w.w_up, tb.block_expert, tb.n_blocks, pad_offsets=tb.pad_offsets)
    _mark("gemm_dx")
    dw_gate, dw_up = ops.grouped_gemm_tn(c.xs, dgu, tb.pad_offsets, e, out_dtype=w.w_gate.dtype, split=True)
    _mark("gemm_dw_gateup")
  grads = dict(dw_gate=dw_gate, dw_up=dw_up, dw_down=dw_down, dw=dw)
  grads.update(shared_grads)
  # router backward
  if dw_partial is not None:
    _, dlb, dw = router_topk_bwd(c.logits, tb.topk_idx, None, want_f32=False, want_bf16=True, dw_partial=dw_partial,
                                 pad_pos=tb.pad_pos)
    grads["dw"] = dw
  else:
    _, dlb = router_topk_bwd(c.logits, tb.topk_idx, dw, want_f32=False, want_bf16=True)
  _mark("router_topk_bwd")
  w_r_bf16 = cast_bf16(w.w_router)                                  # [d,E] = K-major operand over E
  dx_r = ops.grouped_gemm_nt(dlb, w_r_bf16[None], None, None)        # [T,d] = dlogits . W_r^T
  _mark("router_dx")
  dw_router = ops.grouped_gemm_tn(x, dlb, None, 1, out_dtype=torch.float32)[0]   # [d,E] = x^T . dlogits
  _mark("router_dw")
  grads.update(dw_router=dw_router, dlogits_bf16=dlb)
  fork.join(dxsh, *shared_grads.values())
  # dispatch backward: dx[t] = sum_j dxs[row(t,j)] (+ shared-expert and router terms)
  grads["dx"] = ops.gather_reduce(dxs, pad_pos, None, x.dtype, add0=dxsh, add1=dx_r)
  _mark("dispatch_bwd_gather_reduce")
  return grads


def moe_layer_step_host(x_host, dout_host, w: MoEWeights, k, out_host, dx_host, bufs=None):
  """One forward+backward with HOST activations: copies x and the upstream gradient in from (pinned)
  host memory, runs the layer, copies the output and dx back.  Weight gradients stay on the device
  (they feed the optimizer there).  Returns the gradient dict; everything is asynchronous with respect to the
  host and ordered on the current stream, so synchronise it before reading the host buffers.

  With a `bufs` dict that is passed again on later calls the device buffers are kept, the forward and the
  backward pass are each recorded into a CUDA graph on the second call (the first one runs eagerly and sets
  kernel attributes), the upstream gradient is copied in on a second stream while the forward pass runs and the
  output is copied out while the backward pass runs: of the four PCIe transfers only x (before) and dx (after)
  are exposed."""
  dev = w.w_gate.device
  if bufs is None:
    bufs = {}
  xd = bufs.get("x")
  if xd is None or xd.shape != x_host.shape or bufs.get("k") != k:
    bufs.clear()
    xd = bufs["x"] = torch.empty(x_host.shape, dtype=x_host.dtype, device=dev)
    bufs["dout"] = torch.empty(dout_host.shape, dtype=dout_host.dtype, device=dev)
    bufs["k"] = k
    bufs["copy_stream"] = torch.cuda.Stream(dev)
    bufs["calls"] = 0
  gd, cp = bufs["dout"], bufs["copy_stream"]
  main = torch.cuda.current_stream(dev)
  bufs["calls"] += 1

  if bufs["calls"] == 2 and "graphs" not in bufs:
    hook = _HOOK
    set_profile_hook(None)
    try:
      fwd, bwd = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
      with torch.cuda.graph(fwd):
        out, cache = moe_layer_fwd(xd, w, k)
      with torch.cuda.graph(bwd, pool=fwd.pool()):
        grads = moe_layer_bwd(gd, w, cache)
      bufs["graphs"] = (fwd, bwd, out, grads)
    except Exception:   # a step that cannot be captured keeps running eagerly
      bufs["graphs"] = None
    finally:
      set_profile_hook(hook)

  graphs = bufs.get("graphs")
  xd.copy_(x_host, non_blocking=True)
  start = main.record_event()
  with torch.cuda.stream(cp):
    cp.wait_event(start)   # the previous step no longer reads the upstream-gradient buffer
    gd.copy_(dout_host, non_blocking=True)
    dout_in = cp.record_event()
  if graphs:
    fwd, bwd, out, grads = graphs
    fwd.replay()
  else:
    out, cache = moe_layer_fwd(xd, w, k)
  fwd_done = main.record_event()
  with torch.cuda.stream(cp):
    cp.wait_event(fwd_done)
    out_host.copy_(out, non_blocking=True)
    out_back = cp.record_event()
  main.wait_event(dout_in)
  if graphs:
    bwd.replay()
  else:
    grads = moe_layer_bwd(gd, w, cache)
  dx_host.copy_(grads["dx"], non_blocking=True)
  main.wait_event(out_back)
  return grads


class CapturedStep:
  """A step function (fixed shapes, fixed input buffers) recorded once into a CUDA graph and replayed.

  Queuing one forward+backward eagerly takes the host 0.6 ms on an idle core and several milliseconds on a busy
  one, which can exceed the 3 ms the GPU needs; a replay is one call.  `fn` must have run at least once before
  (first calls set kernel attributes), must read its inputs from the same tensors every time, and must not
  synchronise with the host.  Calling the object replays the graph and returns the tensors `fn` returned during
  capture (they are overwritten by every replay)."""

  def __init__(self, fn, keep_profile_hook=False):
    self.graph = torch.cuda.CUDAGraph()
    hook = _HOOK
    if not keep_profile_hook:
      set_profile_hook(None)   # ordinary timing events cannot be recorded into a graph (external ones can)
    try:
      with torch.cuda.graph(self.graph):
        self.result = fn()
    finally:
      set_profile_hook(hook)

  def __call__(self):
    self.graph.replay()
    return self.result


class _MoELayerFn(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, k, w_router, w_gate, w_up, w_down, ws_gate, ws_up, ws_down, router_bias):
    w = MoEWeights(w_router, w_gate, w_up, w_down, ws_gate, ws_up, ws_down, router_bias)
    out, cache = moe_layer_fwd(x, w, k)
    ctx.w, ctx.cache = w, cache
    return out

  @staticmethod
  def backward(ctx, g):
    gr = moe_layer_bwd(g, ctx.w, ctx.cache)
    return (gr["dx"], None, gr["dw_router"], gr["dw_gate"], gr["dw_up"], gr["dw_down"], gr.get("dws_gate"),
            gr.get("dws_up"), gr.get("dws_down"), None)


def moe_layer(x, w: MoEWeights, k):
  """Differentiable MoE layer: out = routed experts + shared expert (bf16 in, bf16 out)."""
  return _MoELayerFn.apply(x, k, w.w_router, w.w_gate, w.w_up, w.w_down, w.ws_gate, w.ws_up, w.ws_down,
                           w.router_bias)
