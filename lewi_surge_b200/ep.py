"""Expert parallelism: experts sharded across the GPUs of one node, tokens stay data-parallel.

Rank g owns experts [g*E/G, (g+1)*E/G) and T_local tokens.  Because the routed slots are sorted by
global expert id (sort_indices of the reference, modal/moe_permute.py:240-264), a rank's sorted rows are
already contiguous by destination rank, so dispatch and combine are one all-to-all each way with
per-destination split sizes taken from the expert histogram:

  forward   route -> sorted rows -> all-to-all (rows + their expert ids) -> regroup received rows into
            padded blocks per local expert -> SwiGLU grouped GEMMs -> back to received order ->
            all-to-all back -> weighted combine (+ shared expert, computed while the all-to-all runs)
  backward  mirrors it: scaled gather of dout -> all-to-all -> expert backward -> all-to-all back ->
            gather-reduce into dx.  Expert weight gradients stay with their owner; the router and the
            shared expert are replicated, so their gradients are local (summing them across ranks is
            the data-parallel all-reduce of the surrounding trainer).

The reference never ran expert parallelism (configs/stage1.yml:102 keeps ici_expert_parallelism at 1);
this is the build's own design for an NVSwitch node.  Collectives are torch.distributed calls (NCCL on
GPUs, gloo in the CPU tests); received rows land in this GPU's own memory before any kernel reads them.
All math goes through a backend object: `CudaBackend` (the sm_100a kernels) in production; the tests
inject a CPU stand-in to exercise the exchange logic under gloo.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

BLOCK = 128


def expert_owner_splits(counts, world):
  """Rows this rank sends to each destination: sums of `counts[E]` over each owner's expert range."""
  e = counts.shape[-1]
  return counts.reshape(*counts.shape[:-1], world, e // world).sum(-1)


@dataclass
class Plan:
  send_splits: list          # rows sent to each rank (and received back in combine)
  recv_splits: list          # rows received from each rank
  n_recv: int


def make_plan(counts_all, rank, world):
  """counts_all [G,E] (expert histogram of every rank, on the host) -> split sizes for this rank."""
  per_owner = expert_owner_splits(counts_all, world)          # [G(src), G(dst)]
  send = [int(v) for v in per_owner[rank].tolist()]
  recv = [int(v) for v in per_owner[:, rank].tolist()]
  return Plan(send, recv, sum(recv))


class CudaBackend:
  """The production math: every call lands in liblewi_moe.so."""

  def __init__(self):
    from . import layer, ops
    self.layer, self.ops = layer, ops

  def route(self, x, w_router, bias, k):
    logits = self.layer.router_logits(x, w_router, bias)
    tb = self.layer.router_topk(logits, k)
    return logits, tb

  def sort_padded(self, flat_e, num_experts):
    """Stable sort of received rows by local expert + padded-block tables."""
    from . import _lib
    lib = _lib.load()
    flat = flat_e.contiguous()
    m = flat.shape[0]
    dev = flat.device
    mpad = self.ops.padded_rows_bound(m, num_experts, BLOCK)
    i32 = dict(dtype=torch.int32, device=dev)
    t = dict(pad_offsets=torch.zeros(num_experts + 1, **i32), block_expert=torch.full((max(mpad // BLOCK, 1),), -1, **i32),
             n_blocks=torch.zeros(1, **i32), pad_pos=torch.empty(max(m, 1), **i32)[:m],
             row_slot=torch.full((max(mpad, 1),), -1, **i32)[:mpad], counts=torch.zeros(num_experts, **i32), mpad=mpad)
    if m > 0:
      ws = self.ops.route_workspace(m, num_experts, dev)
      _lib.check(lib.lewi_sort_indices(_lib.stream(), _lib.ptr(flat), m, num_experts, BLOCK, None, None,
                                       _lib.ptr(t["counts"]), None, _lib.ptr(t["pad_offsets"]), _lib.ptr(t["block_expert"]),
                                       _lib.ptr(t["n_blocks"]), _lib.ptr(t["pad_pos"]), _lib.ptr(t["row_slot"]),
                                       _lib.ptr(ws), ws.numel()), "lewi_sort_indices")
    return t

  def gather_rows(self, x, idx, scale=None, idx_div=1, scale_by_idx=False, n_out=None):
    return self.ops.gather_rows(x, idx, scale, idx_div=idx_div, scale_by_idx=scale_by_idx)

  def gather_reduce(self, y, pos, w, out_dtype, add0=None, add1=None):
    return self.ops.gather_reduce(y, pos, w, out_dtype, add0=add0, add1=add1)

  def gather_dot(self, y, pos, g):
    return self.ops.gather_dot(y, pos, g)

  def experts_fwd(self, xs_pad, w_gate, w_up, w_down, t):
    gu, h = self.layer.gateup_swiglu(xs_pad, w_gate, w_up, t["block_expert"], t["n_blocks"], pad_offsets=t["pad_offsets"])
    ys = self.ops.grouped_gemm_nn(h, w_down, t["block_expert"], t["n_blocks"], pad_offsets=t["pad_offsets"])
    return gu, h, ys

  def experts_bwd(self, dys_pad, xs_pad, gu, h, w_gate, w_up, w_down, t):
    e = w_gate.shape[0]
    dgu = self.layer.dh_dswiglu(dys_pad, w_down, gu, t["block_expert"], t["n_blocks"], pad_offsets=t["pad_offsets"])
    dw_down = self.ops.grouped_gemm_tn(h, dys_pad, t["pad_offsets"], e, out_dtype=w_down.dtype)
    dxs = self.layer.dx_from_dgu(dgu, w_gate, w_up, t["block_expert"], t["n_blocks"], pad_offsets=t["pad_offsets"])
    dw_gate, dw_up = self.ops.grouped_gemm_tn(xs_pad, dgu, t["pad_offsets"], e, out_dtype=w_gate.dtype, split=True)
    return dxs, dw_gate, dw_up, dw_down

  def shared_fwd(self, x, ws_gate, ws_up, ws_down):
    gus, hs = self.layer.gateup_swiglu(x, ws_gate[None], ws_up[None], None, None)
    return gus, hs, self.ops.grouped_gemm_nn(hs, ws_down[None], None, None)

  def shared_bwd(self, dout, x, gus, hs, ws_gate, ws_up, ws_down):
    dgus = self.layer.dh_dswiglu(dout, ws_down[None], gus, None, None)
    dws_down = self.ops.grouped_gemm_tn(hs, dout, None, 1, out_dtype=ws_down.dtype)[0]
    dxsh = self.layer.dx_from_dgu(dgus, ws_gate[None], ws_up[None], None, None)
    dws_gate, dws_up = self.ops.grouped_gemm_tn(x, dgus, None, 1, out_dtype=ws_gate.dtype, split=True)
    return dxsh, dws_gate[0], dws_up[0], dws_down

  def router_bwd(self, x, logits, topk_idx, dw, w_router):
    _, dlb = self.layer.router_topk_bwd(logits, topk_idx, dw, want_f32=False, want_bf16=True)
    dx_r = self.ops.grouped_gemm_nt(dlb, self.layer.cast_bf16(w_router)[None], None, None)
    dw_router = self.ops.grouped_gemm_tn(x, dlb, None, 1, out_dtype=torch.float32)[0]
    return dx_r, dw_router

  def zero_rows(self, n, d, like):
    return torch.empty((n, d), dtype=like.dtype, device=like.device)


class ExpertParallelLayer:
  """MoE layer with experts sharded over `group`.  `w` holds this rank's LOCAL expert weights
  (w_gate/w_up [E/G,d,f], w_down [E/G,f,d]) and replicated router / shared-expert weights."""

  def __init__(self, w, k, num_experts, group=None, backend=None):
    self.w, self.k, self.e = w, k, num_experts
    self.group = group
    self.world = dist.get_world_size(group)
    self.rank = dist.get_rank(group)
    if num_experts % self.world != 0:
      raise ValueError("num_experts must be divisible by the number of ranks")
    self.e_local = num_experts // self.world
    if w.w_gate.shape[0] != self.e_local:
      raise ValueError(f"expected {self.e_local} local experts, got {w.w_gate.shape[0]}")
    self.be = backend or CudaBackend()

  # -- collectives --------------------------------------------------------------------------------
  def _all_to_all_rows(self, rows, in_splits, out_splits, async_op=False):
    out = self.be.zero_rows(sum(out_splits), rows.shape[1], rows) if rows.dim() == 2 else \
        torch.empty(sum(out_splits), dtype=rows.dtype, device=rows.device)
    work = dist.all_to_all_single(out, rows.contiguous(), out_splits, in_splits, group=self.group, async_op=async_op)
    return out, work

  def _exchange_counts(self, counts):
    """All ranks' expert histograms, on the host (one small device->host copy per step)."""
    gathered = torch.empty(self.world * self.e, dtype=counts.dtype, device=counts.device)
    dist.all_gather_into_tensor(gathered, counts.contiguous().view(-1), group=self.group)
    return gathered.view(self.world, self.e).cpu()

  # -- forward / backward ---------------------------------------------------------------------------
  def forward(self, x):
    be, w, k = self.be, self.w, self.k
    t_loc = x.shape[0]
    logits, tb = be.route(x, w.w_router, w.router_bias, k)
    plan = make_plan(self._exchange_counts(tb.counts), self.rank, self.world)
    # rows sorted by global expert = contiguous by owner rank
    xs_sorted = be.gather_rows(x, tb.order, idx_div=k)
    e_sorted = tb.topk_idx.reshape(-1)[tb.order.long()]   # expert id of every sorted row (4 bytes per row)
    xs_recv, work_x = self._all_to_all_rows(xs_sorted, plan.send_splits, plan.recv_splits, async_op=True)
    e_recv, work_e = self._all_to_all_rows(e_sorted.contiguous(), plan.send_splits, plan.recv_splits, async_op=True)
    # the shared expert runs while the rows are in flight
    shared = be.shared_fwd(x, w.ws_gate, w.ws_up, w.ws_down) if w.ws_gate is not None else None
    work_e.wait()
    work_x.wait()
    lt = be.sort_padded(e_recv - self.rank * self.e_local, self.e_local)
    xs_pad = be.gather_rows(xs_recv, lt["row_slot"])
    gu, h, ys_pad = be.experts_fwd(xs_pad, w.w_gate, w.w_up, w.w_down, lt)
    ys_recv = be.gather_rows(ys_pad, lt["pad_pos"])
    ys_sorted, work_y = self._all_to_all_rows(ys_recv, plan.recv_splits, plan.send_splits, async_op=True)
    work_y.wait()
    out = be.gather_reduce(ys_sorted, tb.pos.view(t_loc, k), tb.topk_w, x.dtype,
                           add0=shared[2] if shared is not None else None)
    cache = dict(x=x, logits=logits, tb=tb, plan=plan, lt=lt, xs_pad=xs_pad, gu=gu, h=h, ys_sorted=ys_sorted,
                 shared=shared)
    return out, cache

  def backward(self, dout, c):
    be, w, k = self.be, self.w, self.k
    x, tb, plan, lt = c["x"], c["tb"], c["plan"], c["lt"]
    t_loc = x.shape[0]
    pos2 = tb.pos.view(t_loc, k)
    dout = dout.contiguous()
    dys_sorted = be.gather_rows(dout, tb.order, tb.topk_w.reshape(-1), idx_div=k, scale_by_idx=True)
    dys_recv, work = self._all_to_all_rows(dys_sorted, plan.send_splits, plan.recv_splits, async_op=True)
    # overlapped with the all-to-all: routing-weight gradient and the shared expert's backward
    dw = be.gather_dot(c["ys_sorted"], pos2, dout)
    grads = dict(dw=dw)
    dxsh = None
    if c["shared"] is not None:
      gus, hs, _ = c["shared"]
      dxsh, grads["dws_gate"], grads["dws_up"], grads["dws_down"] = be.shared_bwd(dout, x, gus, hs, w.ws_gate, w.ws_up,
                                                                                  w.ws_down)
    work.wait()
    dys_pad = be.gather_rows(dys_recv, lt["row_slot"])
    dxs_pad, grads["dw_gate"], grads["dw_up"], grads["dw_down"] = be.experts_bwd(dys_pad, c["xs_pad"], c["gu"], c["h"],
                                                                                 w.w_gate, w.w_up, w.w_down, lt)
    dxs_recv = be.gather_rows(dxs_pad, lt["pad_pos"])
    dxs_sorted, work = self._all_to_all_rows(dxs_recv, plan.recv_splits, plan.send_splits, async_op=True)
    dx_r, grads["dw_router"] = be.router_bwd(x, c["logits"], tb.topk_idx, dw, w.w_router)
    work.wait()
    grads["dx"] = be.gather_reduce(dxs_sorted, pos2, None, x.dtype, add0=dxsh, add1=dx_r)
    return grads

  def step(self, x, dout):
    out, cache = self.forward(x)
    return out, self.backward(dout, cache)


# ======================================================================================================
# Peer-memory variant: dispatch / combine are single kernels whose stores / loads cross NVLink directly.
# ======================================================================================================


class _DevBuf:
  """Device memory from lewi_ep_alloc that exposes itself to torch through __cuda_array_interface__."""

  def __init__(self, nbytes, device_index):
    import ctypes
    from . import _lib
    self.lib = _lib.load()
    self.nbytes = int(nbytes)
    out = ctypes.c_void_p()
    _lib.check(self.lib.lewi_ep_alloc(self.nbytes, ctypes.byref(out)), "lewi_ep_alloc")
    self.ptr = out.value
    self.device_index = device_index
    self.__cuda_array_interface__ = {"shape": (self.nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 2}

  def tensor(self, shape, dtype):
    t = torch.as_tensor(self, device=torch.device("cuda", self.device_index))
    return t.view(dtype).view(*shape)

  def ipc_handle(self):
    import ctypes
    from . import _lib
    buf = ctypes.create_string_buffer(64)
    _lib.check(self.lib.lewi_ep_ipc_export(self.ptr, buf), "lewi_ep_ipc_export")
    return bytes(buf.raw)


class _SymmetricBuffer:
  """One buffer of the same size on every rank, each rank holding device pointers to all of them."""

  def __init__(self, nbytes, group, device):
    import ctypes
    from . import _lib
    lib = _lib.load()
    self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
    self.local = _DevBuf(nbytes, device.index)
    handles = [None] * self.world
    dist.all_gather_object(handles, self.local.ipc_handle(), group=group)
    self.ptrs = []
    for r, h in enumerate(handles):
      if r == self.rank:
        self.ptrs.append(self.local.ptr)
      else:
        out = ctypes.c_void_p()
        _lib.check(lib.lewi_ep_ipc_import(ctypes.create_string_buffer(h, 64), ctypes.byref(out)), "lewi_ep_ipc_import")
        self.ptrs.append(out.value)
    self.c_ptrs = (ctypes.c_void_p * self.world)(*self.ptrs)   # host array handed to the C entry points


class ExpertParallelP2P:
  """Expert-parallel MoE layer whose dispatch and combine are kernels over peer memory.

  Every rank routes its own tokens and all-gathers the expert histogram (the only data-dependent
  collective, 4*E bytes per rank); `lewi_ep_plan` turns it into row offsets on every owner.  Rows are then
  pushed straight into the owners' padded buffers (`lewi_ep_push_rows`), the owners run the grouped GEMMs in
  place, and the sources pull and sum their results (`lewi_ep_pull_reduce`).  The backward pass pushes the
  upstream gradient rows the same way and pulls dx and the routing-weight gradient pieces.  Ordering between
  ranks is a one-element all-reduce on the compute stream (stream-ordered: it completes on a rank only when
  every rank has reached it, i.e. has finished the kernels queued before it).  No host synchronisation.

  `capacity` bounds the rows a rank can receive as a multiple of its own routed rows (M = T*k); the buffers are
  allocated once for that bound.  More rows than that raise LEWI_STATUS_EP_OVERFLOW (rows are dropped, not
  written out of bounds).
  """

  def __init__(self, w, k, num_experts, tokens, d, group=None, capacity=None):
    from . import _lib, layer, ops
    self.lib, self.layer, self.ops, self._lib = _lib.load(), layer, ops, _lib
    self.w, self.k, self.e, self.d, self.t = w, k, num_experts, d, tokens
    self.group = group
    self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
    if num_experts % self.world != 0:
      raise ValueError("num_experts must be divisible by the number of ranks")
    if self.world > 8:
      raise ValueError("at most 8 ranks (one NVSwitch node)")
    self.el = num_experts // self.world
    self.f = w.w_gate.shape[2]
    self.dev = w.w_gate.device
    self.m = tokens * k
    cap = float(capacity) if capacity is not None else min(float(self.world), 2.0)
    rows = int(self.m * cap)
    self.rmax = (rows + self.el * (BLOCK - 1)) // BLOCK * BLOCK
    self.parts = int(self.lib.lewi_dw_partial_parts(self.f))
    bf = torch.bfloat16
    sb = lambda nbytes: _SymmetricBuffer(nbytes, group, self.dev)
    self.s_x, self.s_w = sb(self.rmax * d * 2), sb(self.rmax * 4)
    self.s_ys, self.s_dy, self.s_dxs = sb(self.rmax * d * 2), sb(self.rmax * d * 2), sb(self.rmax * d * 2)
    self.s_dwp = sb(self.rmax * self.parts * 4)
    self.recv_x = self.s_x.local.tensor((self.rmax, d), bf)
    self.recv_w = self.s_w.local.tensor((self.rmax,), torch.float32)
    self.ys = self.s_ys.local.tensor((self.rmax, d), bf)
    self.recv_dy = self.s_dy.local.tensor((self.rmax, d), bf)
    self.dxs = self.s_dxs.local.tensor((self.rmax, d), bf)
    self.dwp = self.s_dwp.local.tensor((self.rmax, self.parts), torch.float32)
    i32 = dict(dtype=torch.int32, device=self.dev)
    self.counts_all = torch.zeros(self.world * num_experts, **i32)
    self.dst_base = torch.zeros(num_experts, **i32)
    self.pad_offsets = torch.zeros(self.el + 1, **i32)
    self.valid_end = torch.zeros(self.el, **i32)
    self.n_blocks = torch.zeros(1, **i32)
    self.block_expert = torch.zeros(self.rmax // BLOCK, **i32)
    self.recv_rows = torch.zeros(1, **i32)
    self.slot_rank = torch.zeros(self.m, **i32)
    self.slot_row = torch.zeros(self.m, **i32)
    self._flag = torch.zeros(1, dtype=torch.float32, device=self.dev)
    self.recv_w.zero_()
    torch.cuda.synchronize(self.dev)
    dist.barrier(group=group)

  def _sync_ranks(self):
    dist.all_reduce(self._flag, group=self.group)

  def forward(self, x):
    lib, L, ops, _lib, w, k = self.lib, self.layer, self.ops, self._lib, self.w, self.k
    st, ptr, check = _lib.stream, _lib.ptr, _lib.check
    t, d = x.shape
    logits = L.router_logits(x, w.w_router, w.router_bias)
    tb = L.router_topk(logits, k)
    dist.all_gather_into_tensor(self.counts_all, tb.counts, group=self.group)
    check(lib.lewi_ep_plan(st(), ptr(self.counts_all), self.world, self.e, self.rank, BLOCK, self.rmax, ptr(self.dst_base),
                           ptr(self.pad_offsets), ptr(self.valid_end), ptr(self.n_blocks), ptr(self.block_expert),
                           ptr(self.recv_rows)), "lewi_ep_plan")
    self._sync_ranks()   # every rank is done reading the buffers of the previous step
    check(lib.lewi_ep_push_rows(st(), ptr(x), ptr(tb.order), ptr(tb.topk_idx), ptr(tb.offsets), ptr(self.dst_base),
                                ptr(tb.topk_w), self.s_x.c_ptrs, self.s_w.c_ptrs, ptr(self.slot_rank), ptr(self.slot_row),
                                self.m, k, d, self.e, self.world, self.rmax, t), "lewi_ep_push_rows")
    check(lib.lewi_ep_zero_pad(st(), ptr(self.recv_x), ptr(self.valid_end), ptr(self.pad_offsets), self.el, d, self.rmax),
          "lewi_ep_zero_pad")
    # the shared expert needs nothing from other ranks: it fills the time the rows are in flight
    shared = None
    if w.ws_gate is not None:
      gus, hs = L.gateup_swiglu(x, w.ws_gate[None], w.ws_up[None], None, None)
      shared = (gus, hs, ops.grouped_gemm_nn(hs, w.ws_down[None], None, None))
    self._sync_ranks()   # all rows have arrived
    po = self.pad_offsets
    gu, h = L.gateup_swiglu(self.recv_x, w.w_gate, w.w_up, self.block_expert, self.n_blocks, pad_offsets=po,
                            h_scale_src=self.recv_w)
    ops.grouped_gemm_nn(h, w.w_down, self.block_expert, self.n_blocks, pad_offsets=po, out=self.ys)
    self._sync_ranks()   # all expert outputs are written
    out = torch.empty_like(x)
    check(lib.lewi_ep_pull_reduce(st(), self.s_ys.c_ptrs, ptr(self.slot_rank), ptr(self.slot_row),
                                  ptr(shared[2]) if shared else None, None, ptr(out), t, k, d, self.world, self.rmax),
          "lewi_ep_pull_reduce")
    return out, dict(x=x, logits=logits, tb=tb, gu=gu, h=h, shared=shared)

  def backward(self, dout, c):
    lib, L, ops, _lib, w, k = self.lib, self.layer, self.ops, self._lib, self.w, self.k
    st, ptr, check = _lib.stream, _lib.ptr, _lib.check
    x, tb = c["x"], c["tb"]
    t, d = x.shape
    dout = dout.contiguous()
    check(lib.lewi_ep_push_rows(st(), ptr(dout), ptr(tb.order), ptr(tb.topk_idx), ptr(tb.offsets), ptr(self.dst_base),
                                None, self.s_dy.c_ptrs, None, None, None, self.m, k, d, self.e, self.world, self.rmax, t),
          "lewi_ep_push_rows")
    check(lib.lewi_ep_zero_pad(st(), ptr(self.recv_dy), ptr(self.valid_end), ptr(self.pad_offsets), self.el, d, self.rmax),
          "lewi_ep_zero_pad")
    grads = {}
    dxsh = None
    if c["shared"] is not None:
      gus, hs, _ = c["shared"]
      dgus = L.dh_dswiglu(dout, w.ws_down[None], gus, None, None)
      grads["dws_down"] = ops.grouped_gemm_tn(hs, dout, None, 1, out_dtype=w.ws_down.dtype)[0]
      dxsh = L.dx_from_dgu(dgus, w.ws_gate[None], w.ws_up[None], None, None)
      g1, g2 = ops.grouped_gemm_tn(x, dgus, None, 1, out_dtype=w.ws_gate.dtype, split=True)
      grads["dws_gate"], grads["dws_up"] = g1[0], g2[0]
    self._sync_ranks()   # all upstream-gradient rows have arrived
    po = self.pad_offsets
    lib_parts = self.parts
    dgu = torch.empty((self.rmax, 2 * self.f), dtype=torch.bfloat16, device=self.dev)
    check(lib.lewi_grouped_gemm_dh_dswiglu_gather(st(), ptr(self.recv_dy), None, 1, self.rmax, None, ptr(self.recv_w),
                                                  ptr(self.dwp), ptr(w.w_down), ptr(c["gu"]), ptr(dgu),
                                                  ptr(self.block_expert), ptr(self.n_blocks), ptr(po), self.rmax, d, self.f,
                                                  self.el), "lewi_grouped_gemm_dh_dswiglu")
    grads["dw_down"] = ops.grouped_gemm_tn(c["h"], self.recv_dy, po, self.el, out_dtype=w.w_down.dtype)
    check(lib.lewi_grouped_gemm_dx(st(), ptr(dgu), ptr(w.w_gate), ptr(w.w_up), ptr(self.dxs), ptr(self.block_expert),
                                   ptr(self.n_blocks), ptr(po), self.rmax, d, self.f, self.el), "lewi_grouped_gemm_dx")
    grads["dw_gate"], grads["dw_up"] = ops.grouped_gemm_tn(self.recv_x, dgu, po, self.el, out_dtype=w.w_gate.dtype,
                                                           split=True)
    self._sync_ranks()   # dxs and the routing-weight gradient pieces are written everywhere
    dw = torch.empty((t, k), dtype=torch.float32, device=self.dev)
    check(lib.lewi_ep_pull_dw(st(), self.s_dwp.c_ptrs, ptr(self.slot_rank), ptr(self.slot_row), ptr(dw), self.m,
                              lib_parts, self.world, self.rmax), "lewi_ep_pull_dw")
    grads["dw"] = dw
    _, dlb = L.router_topk_bwd(c["logits"], tb.topk_idx, dw, want_f32=False, want_bf16=True)
    dx_r = ops.grouped_gemm_nt(dlb, L.cast_bf16(w.w_router)[None], None, None)
    grads["dw_router"] = ops.grouped_gemm_tn(x, dlb, None, 1, out_dtype=torch.float32)[0]
    dx = torch.empty_like(x)
    check(lib.lewi_ep_pull_reduce(st(), self.s_dxs.c_ptrs, ptr(self.slot_rank), ptr(self.slot_row), ptr(dxsh), ptr(dx_r),
                                  ptr(dx), t, k, d, self.world, self.rmax), "lewi_ep_pull_reduce")
    grads["dx"] = dx
    return grads

  def step(self, x, dout):
    out, cache = self.forward(x)
    return out, self.backward(dout, cache)
