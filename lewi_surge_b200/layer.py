"""The whole MoE layer, forward and backward: a thin caller of `lewi_moe_fwd` / `lewi_moe_bwd`.

The launch sequence itself lives behind the C ABI (csrc/lewi_moe.cu); it replaces, in the reference, router ->
top-k -> `_route_activations` -> three `ragged_dot`s -> `unpermute` (modal/moe_permute.py:399-433,
modal/padded_gmm.py:45-69) and their gather-only gradients (modal/moe_permute.py:282-309):

  logits  = x . W_r                                   router GEMM (f32-exact on the tensor cores)
  tables  = softmax/top-k/renorm + stable sort        lewi_router_topk
  xs      = rows of x in padded-block order           lewi_gather_rows      (dispatch)
  gu, h   = SwiGLU(xs . Wg[e], xs . Wu[e]) * w        gate/up GEMM, router weight folded into h
  ys      = h . Wd[e]                                 down GEMM
  shared expert on all tokens (same kernels, one group; optional sigmoid gate)
  out[t]  = sum_j ys[row(t,j)] + shared[t]            lewi_gather_reduce    (combine)

This module owns what a host framework owns: the residual and workspace buffers (torch tensors as device memory),
the side stream the shared expert runs on, and CUDA-graph capture of a step.  The per-kernel wrappers further down
are what the expert-parallel layer composes.
"""
from __future__ import annotations

import ctypes
import weakref
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import check, ptr, stream
from . import ops

BLOCK = ops.BLOCK

_HOOK = None
_C_HOOK = None   # keeps the ctypes callback object alive while it is installed


def set_profile_hook(fn):
  """fn(name, stream_ptr) is called after every kernel launch of the layer (used to drop CUDA events on that
  stream); None disables."""
  global _HOOK, _C_HOOK
  _HOOK = fn
  lib = _lib.load()
  if fn is None:
    lib.lewi_moe_set_mark_callback(None)
    _C_HOOK = None
    return
  cb_type = ctypes.CFUNCTYPE(None, ctypes.c_char_p, ctypes.c_void_p)
  _C_HOOK = cb_type(lambda name, st: fn(name.decode(), st or 0))
  lib.lewi_moe_set_mark_callback(ctypes.cast(_C_HOOK, ctypes.c_void_p))


def _mark(name):
  if _HOOK is not None:
    _HOOK(name, stream())


# The shared expert depends only on x (forward) / dout (backward), so it runs on a side stream next to the
# memory-bound routing and gather kernels of the routed path and is joined before the combine.
OVERLAP_SHARED = True
_SIDE = {}


def _side_stream(device):
  st = _SIDE.get(device)
  if st is None:
    st = _SIDE[device] = torch.cuda.Stream(device=device)
  return st


@dataclass
class MoEWeights:
  """Parameter tensors in the reference's orientation (modal/stage2.py:338-345).

  w_router [d,E] f32 (experts on the last axis); w_gate, w_up [E,d,f] (wi_0, wi_1), w_down [E,f,d] (wo),
  shared expert ws_gate, ws_up [d,fs], ws_down [fs,d]; all expert weights bf16.  router_bias f32 [E] (optional),
  w_sg f32 [d] (optional): sigmoid gate on the shared expert as in the Hugging Face twin (tools/grow_7b.py:85).
  """
  w_router: torch.Tensor
  w_gate: torch.Tensor
  w_up: torch.Tensor
  w_down: torch.Tensor
  ws_gate: Optional[torch.Tensor] = None
  ws_up: Optional[torch.Tensor] = None
  ws_down: Optional[torch.Tensor] = None
  router_bias: Optional[torch.Tensor] = None
  w_sg: Optional[torch.Tensor] = None


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


def router_topk(logits, k, block=BLOCK, aux_loss=None):
  """softmax -> top-k -> renormalise + stable sort of the T*k slots + padded-block tables.  ``aux_loss`` (f32 [1],
  optional) receives the unweighted load-balance loss."""
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
                             ptr(aux_loss), ptr(ws), ws.numel()), "lewi_router_topk")
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


def gateup_swiglu(xs, w_gate, w_up, block_expert, n_blocks, want_gu=True, pad_offsets=None, h_scale_src=None,
                  scale_idx=None):
  """(gu [rows,2f], h [rows,f]) = fused gate/up projection + SwiGLU over the padded rows; with ``h_scale_src`` h is
  multiplied by ``h_scale_src[scale_idx[r]]`` (``scale_idx`` None: by ``h_scale_src[r]``)."""
  lib = _lib.load()
  e, d, f = w_gate.shape
  rows = xs.shape[0]
  gu = torch.empty((rows, 2 * f), dtype=torch.bfloat16, device=xs.device) if want_gu else None
  h = torch.empty((rows, f), dtype=torch.bfloat16, device=xs.device)
  check(lib.lewi_grouped_gemm_gateup_swiglu_scaled(stream(), ptr(xs), ptr(scale_idx), ptr(h_scale_src), ptr(w_gate),
                                                   ptr(w_up), ptr(gu), ptr(h), ptr(block_expert), ptr(n_blocks),
                                                   ptr(pad_offsets), rows, d, f, e),
        "lewi_grouped_gemm_gateup_swiglu")
  return gu, h


def dh_dswiglu(dys, w_down, gu, block_expert, n_blocks, pad_offsets=None, scale_src=None, want_dw_partial=False,
               scale_idx=None):
  """dgu [rows,2f] = SwiGLU'(gu) applied to dh = dys . w_down[e]^T.  ``scale_src[scale_idx[r]]`` multiplies dh, and
  ``want_dw_partial`` also returns the routing-weight gradient pieces [rows, parts] f32."""
  lib = _lib.load()
  e, f, d = w_down.shape
  rows = gu.shape[0]
  dgu = torch.empty((rows, 2 * f), dtype=torch.bfloat16, device=dys.device)
  dwp = None
  if want_dw_partial:
    dwp = torch.empty((rows, int(lib.lewi_dw_partial_parts(f))), dtype=torch.float32, device=dys.device)
  check(lib.lewi_grouped_gemm_dh_dswiglu_scaled(stream(), ptr(dys), ptr(scale_idx), ptr(scale_src), ptr(dwp), ptr(w_down),
                                                ptr(gu), ptr(dgu), ptr(block_expert), ptr(n_blocks), ptr(pad_offsets),
                                                rows, d, f, e),
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


_RES_NAMES = ("logits", "topk_idx", "topk_w", "counts", "offsets", "pad_offsets", "n_blocks", "probs_sum", "block_expert",
              "order", "pos", "pad_pos", "row_slot", "xs", "gu", "h", "gus", "hs", "gate")
_WORKSPACE = {}   # device -> grow-only scratch shared by every layer call on that device
_PREPARED = {}    # id of a router-weight tensor -> (weak reference to it, its version counter, prepared bf16 pieces)


def _workspace(nbytes, device):
  ws = _WORKSPACE.get(device)
  if ws is None or ws.numel() < nbytes:
    ws = _WORKSPACE[device] = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
  return ws


def _prepared_router(w_router):
  """bf16 pieces of the f32 router weight, converted once per weight tensor and version (in-place updates bump the
  version).  The entry is tied to the tensor OBJECT: another tensor that happens to reuse its memory converts anew."""
  key = id(w_router)
  hit = _PREPARED.get(key)
  if hit is not None and hit[0]() is w_router and hit[1] == w_router._version:
    return hit[2]
  lib = _lib.load()
  d, e = w_router.shape
  buf = torch.empty(int(lib.lewi_moe_router_prepared_bytes(d, e)), dtype=torch.uint8, device=w_router.device)
  check(lib.lewi_moe_prepare_router(stream(), ptr(w_router), ptr(buf), d, e), "lewi_moe_prepare_router")
  for k_ in [k_ for k_, v in _PREPARED.items() if v[0]() is None]:   # drop entries of tensors that no longer exist
    del _PREPARED[k_]
  _PREPARED[key] = (weakref.ref(w_router), w_router._version, buf)
  return buf


@dataclass
class LayerCache:
  """What the backward pass needs: the inputs' dimensions and the residual buffer `lewi_moe_fwd` filled."""
  x: torch.Tensor
  k: int
  dims: tuple                 # (T, d, E, f, k, fs)
  residual: torch.Tensor      # uint8, layout of lewi_moe_residual_layout
  offsets: tuple
  aux_loss: torch.Tensor      # f32 [1], unweighted load-balance loss

  def item(self, name, dtype, shape):
    i = _RES_NAMES.index(name)
    n = 1
    for v in shape:
      n *= v
    n_bytes = n * torch.empty((), dtype=dtype).element_size()
    return self.residual[self.offsets[i]:self.offsets[i] + n_bytes].view(dtype).view(*shape)

  @property
  def logits(self):
    t, _, e = self.dims[:3]
    return self.item("logits", torch.float32, (t, e))

  @property
  def tables(self):
    t, d, e, f, k, fs = self.dims
    m = t * k
    mpad = ops.padded_rows_bound(m, e, BLOCK)
    i32, f32 = torch.int32, torch.float32
    return RouteTables(
        topk_idx=self.item("topk_idx", i32, (t, k)), topk_w=self.item("topk_w", f32, (t, k)),
        counts=self.item("counts", i32, (e,)), offsets=self.item("offsets", i32, (e + 1,)),
        pad_offsets=self.item("pad_offsets", i32, (e + 1,)), block_expert=self.item("block_expert", i32, (max(mpad // BLOCK, 1),)),
        n_blocks=self.item("n_blocks", i32, (1,)), order=self.item("order", i32, (m,)), pos=self.item("pos", i32, (m,)),
        pad_pos=self.item("pad_pos", i32, (m,)), row_slot=self.item("row_slot", i32, (mpad,)),
        probs_sum=self.item("probs_sum", f32, (e,)), mpad=mpad)


def _dims(x, w: MoEWeights, k):
  t, d = x.shape
  e, _, f = w.w_gate.shape
  fs = w.ws_gate.shape[1] if w.ws_gate is not None else 0
  return int(t), int(d), int(e), int(f), int(k), int(fs)


def _streams(device, shared):
  side = _side_stream(device).cuda_stream if (OVERLAP_SHARED and shared) else None
  return stream(), side


def moe_layer_fwd(x, w: MoEWeights, k, prepared=True):
  """x [T,d] bf16 -> (out [T,d] bf16, cache).  ``prepared`` reuses the converted router weight across calls."""
  lib = _lib.load()
  dims = _dims(x, w, k)
  t, d, e, f, _, fs = dims
  gate = w.w_sg is not None
  off = (ctypes.c_int64 * 20)()
  res_bytes = int(lib.lewi_moe_residual_layout(*dims, int(gate), off))
  if res_bytes < 0:
    check(res_bytes, "lewi_moe_residual_layout")
  ws_bytes = int(lib.lewi_moe_workspace_bytes(*dims, int(gate)))
  dev = x.device
  residual = torch.empty(max(res_bytes, 256), dtype=torch.uint8, device=dev)
  ws = _workspace(ws_bytes, dev)
  out = torch.empty_like(x)
  aux = torch.empty(1, dtype=torch.float32, device=dev)
  prep = _prepared_router(w.w_router) if prepared else None
  main, side = _streams(dev, fs > 0)
  check(lib.lewi_moe_fwd(main, side, ptr(x), ptr(w.w_router), ptr(w.router_bias), ptr(prep), ptr(w.w_gate), ptr(w.w_up),
                         ptr(w.w_down), ptr(w.ws_gate), ptr(w.ws_up), ptr(w.ws_down), ptr(w.w_sg), ptr(out), ptr(aux),
                         ptr(residual), residual.numel(), ptr(ws), ws.numel(), *dims), "lewi_moe_fwd")
  return out, LayerCache(x=x, k=k, dims=dims, residual=residual, offsets=tuple(off), aux_loss=aux)


def moe_layer_bwd(dout, w: MoEWeights, c: LayerCache, aux_grad=0.0, wgrad_dtype=None, want_bias_grad=None, prepared=True):
  """Gradients for x and every weight, given dout [T,d] bf16.  ``aux_grad`` = load-balance loss weight times the
  upstream gradient of that loss (0: the loss does not contribute)."""
  lib = _lib.load()
  dims = c.dims
  t, d, e, f, k, fs = dims
  dev = dout.device
  dout = dout.contiguous()
  wdt = wgrad_dtype or w.w_gate.dtype
  new = lambda like, dt=None: torch.empty(like.shape, dtype=dt or wdt, device=dev)
  g = dict(dx=torch.empty_like(c.x), dw_router=new(w.w_router, torch.float32), dw_gate=new(w.w_gate), dw_up=new(w.w_up),
           dw_down=new(w.w_down), dw=torch.empty((t, k), dtype=torch.float32, device=dev))
  if fs > 0:
    g.update(dws_gate=new(w.ws_gate), dws_up=new(w.ws_up), dws_down=new(w.ws_down))
  if w.w_sg is not None:
    g["dw_sg"] = new(w.w_sg, torch.float32)
  if want_bias_grad if want_bias_grad is not None else w.router_bias is not None:
    g["drouter_bias"] = torch.empty(e, dtype=torch.float32, device=dev)
  ws = _workspace(int(lib.lewi_moe_workspace_bytes(*dims, int(w.w_sg is not None))), dev)
  prep = _prepared_router(w.w_router) if prepared else None
  main, side = _streams(dev, fs > 0)
  check(lib.lewi_moe_bwd(main, side, ptr(dout), ptr(c.x), ptr(w.w_router), ptr(prep), ptr(w.w_gate), ptr(w.w_up),
                         ptr(w.w_down), ptr(w.ws_gate), ptr(w.ws_up), ptr(w.ws_down), ptr(w.w_sg), ptr(c.residual),
                         c.residual.numel(), ptr(ws), ws.numel(), ptr(g["dx"]), ptr(g["dw_router"]),
                         ptr(g.get("drouter_bias")), ptr(g["dw_gate"]), ptr(g["dw_up"]), ptr(g["dw_down"]),
                         ptr(g.get("dws_gate")), ptr(g.get("dws_up")), ptr(g.get("dws_down")), ptr(g.get("dw_sg")),
                         ptr(g["dw"]), float(aux_grad), _lib.F32 if wdt == torch.float32 else _lib.BF16, *dims),
        "lewi_moe_bwd")
  return g


class HostPipeline:
  """Steps on HOST activations with the PCIe copies hidden behind the compute of neighbouring steps.

  `make_step(x_dev, dout_dev)` must return a callable that runs one forward+backward reading those two fixed device
  tensors and returns (out, dx) device tensors (typically a `CapturedStep`).  `step(x_host, dout_host, out_host,
  dx_host)` then queues, without blocking the host:
    copy-in stream   x, dout: pinned host -> one of two device staging sets (runs while the previous step computes);
    compute stream   staging -> the step's input tensors, the step itself, its results -> one of two staging sets;
    copy-out stream  results: staging -> pinned host (runs while the next step computes).
  PCIe is full duplex, so in steady state a step costs max(compute, copy in, copy out) instead of their sum.  Every
  step's inputs are copied in and every step's results are copied out; `drain()` waits for all of it.  The host
  buffers of a step must stay untouched until `drain()` (or two further `step` calls) returned.
  """

  def __init__(self, make_step, tokens, d, device, dtype=torch.bfloat16):
    mk = lambda: torch.empty((tokens, d), dtype=dtype, device=device)
    self.x, self.dout = mk(), mk()
    self.run = make_step(self.x, self.dout)
    self.in_x, self.in_g = [mk(), mk()], [mk(), mk()]
    self.out_y, self.out_dx = [mk(), mk()], [mk(), mk()]
    self.h2d, self.d2h = torch.cuda.Stream(device), torch.cuda.Stream(device)
    self.in_free = [None, None]    # staging set i may be overwritten by the next copy in
    self.out_free = [None, None]   # result set i has been copied out
    self.device = device
    self.n = 0
    self.holder = {}

  @property
  def grads(self):
    """The weight gradients of the most recent step (device tensors), when the step function publishes them."""
    return self.holder.get("grads")

  def step(self, x_host, dout_host, out_host, dx_host):
    i = self.n & 1
    main = torch.cuda.current_stream(self.device)
    with torch.cuda.stream(self.h2d):
      if self.in_free[i] is not None:
        self.h2d.wait_event(self.in_free[i])
      self.in_x[i].copy_(x_host, non_blocking=True)
      self.in_g[i].copy_(dout_host, non_blocking=True)
      arrived = self.h2d.record_event()
    main.wait_event(arrived)
    self.x.copy_(self.in_x[i])
    self.dout.copy_(self.in_g[i])
    self.in_free[i] = main.record_event()
    out, dx = self.run()
    if self.out_free[i] is not None:
      main.wait_event(self.out_free[i])
    self.out_y[i].copy_(out)
    self.out_dx[i].copy_(dx)
    done = main.record_event()
    with torch.cuda.stream(self.d2h):
      self.d2h.wait_event(done)
      out_host.copy_(self.out_y[i], non_blocking=True)
      dx_host.copy_(self.out_dx[i], non_blocking=True)
      self.out_free[i] = self.d2h.record_event()
    self.n += 1

  def drain(self):
    self.d2h.synchronize()
    torch.cuda.current_stream(self.device).synchronize()


def host_pipeline(w: MoEWeights, k, tokens, graph=True):
  """A `HostPipeline` over this layer: forward + backward of `tokens` tokens per step; weight gradients stay on the
  device (`pipeline.grads`, overwritten by every step)."""
  dev = w.w_gate.device
  d = w.w_gate.shape[1]
  holder = {}

  def make_step(x, dout):
    def step():
      out, cache = moe_layer_fwd(x, w, k)
      holder["grads"] = moe_layer_bwd(dout, w, cache)
      return out, holder["grads"]["dx"]
    step()                        # first call: kernel attributes, workspace, converted router weight
    return CapturedStep(step) if graph else step

  pipe = HostPipeline(make_step, tokens, d, dev)
  pipe.holder = holder
  return pipe


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
  def forward(ctx, x, k, aux_weight, w_router, w_gate, w_up, w_down, ws_gate, ws_up, ws_down, router_bias, w_sg):
    w = MoEWeights(w_router, w_gate, w_up, w_down, ws_gate, ws_up, ws_down, router_bias, w_sg)
    out, cache = moe_layer_fwd(x, w, k)
    ctx.w, ctx.cache, ctx.aux_weight = w, cache, float(aux_weight)
    ctx.mark_non_differentiable(cache.aux_loss)
    return out, cache.aux_loss

  @staticmethod
  def backward(ctx, g, _g_aux):
    gr = moe_layer_bwd(g, ctx.w, ctx.cache, aux_grad=ctx.aux_weight)
    return (gr["dx"], None, None, gr["dw_router"], gr["dw_gate"], gr["dw_up"], gr["dw_down"], gr.get("dws_gate"),
            gr.get("dws_up"), gr.get("dws_down"), gr.get("drouter_bias"), gr.get("dw_sg"))


def moe_layer(x, w: MoEWeights, k, aux_weight=0.0):
  """Differentiable MoE layer: out = routed experts + shared expert (bf16 in, bf16 out).

  Returns (out, aux_loss): aux_loss is the unweighted load-balance loss (f32 [1], not differentiable by itself).
  With ``aux_weight`` (the reference's load_balance_loss_weight, configs/stage1.yml:41) the backward pass adds the
  gradient of ``aux_weight * aux_loss`` to the router, i.e. it behaves as if that term were part of the scalar the
  caller differentiates."""
  return _MoELayerFn.apply(x, k, aux_weight, w.w_router, w.w_gate, w.w_up, w.w_down, w.ws_gate, w.ws_up, w.ws_down,
                           w.router_bias, w.w_sg)
