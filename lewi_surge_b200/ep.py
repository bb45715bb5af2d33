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


def range_bounds(num_local_experts, phases, weights=None):
  """Boundaries of the ranges of local experts one pass works through: `phases` ranges of equal size, or sizes in the
  proportion of `weights` (a short first range lets the GEMMs start early, a short last one shortens the tail in which
  only the exchange runs).  Every range gets at least one expert; ranges that would be empty are dropped."""
  if weights is None:
    weights = [1.0] * phases
  weights = [float(v) for v in weights]
  if not weights or min(weights) <= 0:
    raise ValueError("range weights must be positive")
  total, acc, bounds = sum(weights), 0.0, [0]
  for v in weights:
    acc += v
    b = min(num_local_experts, max(bounds[-1] + 1, int(round(num_local_experts * acc / total))))
    if b > bounds[-1]:
      bounds.append(b)
  bounds[-1] = num_local_experts
  return bounds


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

  def free(self):
    if self.ptr:
      self.lib.lewi_ep_free(self.ptr)
      self.ptr = None


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

  def close(self):
    """Unmaps the peers' buffers and frees this rank's own (call on every rank, after a barrier)."""
    from . import _lib
    lib = _lib.load()
    for r, p in enumerate(self.ptrs):
      if r != self.rank and p:
        lib.lewi_ep_ipc_release(p)
    self.ptrs = []
    self.local.free()


class ExpertParallelP2P:
  """Expert-parallel MoE layer whose dispatch and combine are kernels over peer memory.

  Every rank routes its own tokens and shares its expert histogram (4*E bytes, stored into every peer's table);
  `lewi_ep_plan` turns the histograms into row offsets on every owner.  Rows are then pushed straight into the
  owners' padded buffers together with their return address (`lewi_ep_push_rows`), the owners run the grouped
  GEMMs in place and every output row goes back into the source's slot-ordered buffer, where the combine is a sum
  over k consecutive rows: by default straight from the epilogue of the down-projection (and dx) GEMM
  (`lewi_grouped_gemm_nn_return`, `lewi_grouped_gemm_dx_return`: a tile's rows travel while the next tile is being
  multiplied), or with `fused_return=False` by a transfer kernel of its own (`lewi_ep_return_rows`).  The backward
  pass moves the upstream gradient rows, dx and the routing-weight gradient pieces the same way; the weight
  gradients of all ranges are one pair of GEMM launches after the last range (`dw_deferred`).

  `return_sms=(fwd, bwd)`: those return GEMMs cannot finish before their rows have crossed the links, so they get a
  share of the SMs (`lewi_set_gemm_cta_limit`) and a stream of their own, and the next range's first GEMM (gate/up,
  dH) runs beside them on the remaining SMs instead of after them.

  `unique_push=True` sends a token once per destination RANK instead of once per slot (top-6 over 8 ranks: 3.9
  instead of 5.25 rows per token on the links): the owner copies the row to the padded rows of its experts
  (`lewi_ep_local_rows`) before a range's GEMMs.  With `combined_return=True` the owner also adds up a token's local
  expert outputs and returns one partial row per token (`lewi_ep_combine_return`); the source adds the partial rows
  of the ranks it used.  Both are off by default: at 2 GPUs they measured slower than the slot-wise exchange.

  The local experts are worked on in `phases` ranges.  The exchange kernels run on their own stream and are small
  enough to share an SM with a grouped-GEMM CTA, so the rows of range p+1 arrive, and the outputs of range p-1
  leave, while the GEMMs of range p run.  (More than one range needs the CTA-pair GEMM kernels, which find a row
  block's expert from pad_offsets alone.)

  Ordering between ranks (`sync`): "flags" uses `lewi_ep_barrier`, a one-warp kernel that exchanges epoch flags
  through peer memory with a bounded wait; "nccl" uses a one-element all-reduce.  Both are stream-ordered: a rank
  passes only when every rank has finished the kernels queued before it.  No host synchronisation.

  `capacity` bounds the rows a rank can receive as a multiple of its own routed rows (M = T*k); the buffers are
  allocated once for that bound.  The default is the number of ranks: even if every token of every rank chose this
  rank's experts nothing is dropped, like the reference (configs/stage1.yml: capacity_factor -1).  A smaller value
  saves memory; rows beyond it are then dropped (never written out of bounds) and the device status gets
  LEWI_STATUS_EP_OVERFLOW, which `overflowed()` reads: check it after a step when running with a reduced capacity.
  """

  BARRIER_TIMEOUT_MS = 4000

  def __init__(self, w, k, num_experts, tokens, d, group=None, capacity=None, phases=None, sync="flags",
               exchange_threads=(0, 0), dw_down_last=True, range_weights=None, dw_deferred=True,
               fused_return=True, unique_push=False, combined_return=None, return_sms=None, router_tail=False):
    from . import _lib, layer, ops
    self.lib, self.layer, self.ops, self._lib = _lib.load(), layer, ops, _lib
    self.w, self.k, self.e, self.d, self.t = w, k, num_experts, d, tokens
    self.group = group
    self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
    if num_experts % self.world != 0:
      raise ValueError("num_experts must be divisible by the number of ranks")
    if self.world > 8:
      raise ValueError("at most 8 ranks (one NVSwitch node)")
    if sync not in ("flags", "nccl"):
      raise ValueError("sync must be 'flags' or 'nccl'")
    self.sync = sync
    self.fwd_threads, self.bwd_threads = (int(v) for v in exchange_threads)   # CTA size of the exchange kernels (0: largest)
    self.dw_down_last = bool(dw_down_last)
    self.el = num_experts // self.world
    self.f = w.w_gate.shape[2]
    self.dev = w.w_gate.device
    self.m = tokens * k
    want = int(phases) if phases is not None else (1 if self.world == 1 else 4)
    self.phases = max(1, min(want, self.el))
    self.bounds = range_bounds(self.el, self.phases, range_weights)
    self.phases = len(self.bounds) - 1
    # weight gradients of all ranges as one pair of launches after the last range's dx (or range by range)
    self.dw_deferred = bool(dw_deferred)
    # The router backward on the caller's stream after the weight-gradient GEMMs (default), or right after the last
    # barrier on the exchange stream, beside them.  The second form saves 0.05 ms in an eagerly queued step, but replayed
    # as a CUDA graph at 4 GPUs it measured between 3.96 and 5.77 ms per step against 3.76 ms for the first on the same
    # box: off by default.
    self.router_tail = bool(router_tail)
    # A token travels once per destination rank (and is copied to its experts' padded rows by the owner) instead of
    # once per slot; with combined_return the owner also adds up the token's local expert outputs and returns one
    # partial row per token.  Otherwise rows return per slot: as the epilogue of the GEMM that makes them (down
    # projection, dx), or by a transfer kernel of its own.
    self.unique_push = bool(unique_push)
    self.combined_return = self.unique_push if combined_return is None else bool(combined_return)
    if self.combined_return and not self.unique_push:
      raise ValueError("combined_return needs unique_push")
    self.fused_return = bool(fused_return) and not self.combined_return
    if self.phases > 8:
      raise ValueError("at most 8 ranges")
    # > 0: the GEMMs whose epilogues send rows home (they run at the speed of the links) get this many SMs and a
    # stream of their own, and the next range's first GEMM runs beside them on the other SMs.  One number, or one for
    # the forward pass (down projection beside gate/up) and one for the backward pass (dx beside dH).
    # Default with more than one rank: 64 of 148 SMs in the forward pass, 80 in the backward pass (dx is the heavier
    # GEMM); measured 3.82 -> 3.61 ms at 4 GPUs, 3.47 -> 3.41 ms at 2.
    if return_sms is None:
      sms = self._sm_count()
      return_sms = (64 * sms // 148 & ~1, 80 * sms // 148 & ~1) if self.world > 1 else 0
    pair = tuple(return_sms) if isinstance(return_sms, (tuple, list)) else (return_sms,)
    pair = (pair * 2)[:2]
    self.return_sms = tuple(int(v) for v in pair) if self.fused_return and self.phases > 1 else (0, 0)
    for v in self.return_sms:
      if v < 0 or v == 1 or v >= self._sm_count() - 1:
        raise ValueError("return_sms must leave SMs to both GEMMs")
    cap = float(capacity) if capacity is not None else float(self.world)
    rows = int(self.m * cap)
    self.rmax = (rows + self.el * (BLOCK - 1)) // BLOCK * BLOCK
    self.parts = int(self.lib.lewi_dw_partial_parts(self.f))
    bf, f32 = torch.bfloat16, torch.float32
    i32 = dict(dtype=torch.int32, device=self.dev)
    sb = lambda nbytes: _SymmetricBuffer(nbytes, group, self.dev)
    # written by peers: received rows, their router weights and return addresses; returned rows in slot order
    self.s_x, self.s_w, self.s_ret = sb(self.rmax * d * 2), sb(self.rmax * 4), sb(self.rmax * 4)
    self.s_dy = sb(self.rmax * d * 2)
    self.s_yslot, self.s_dxslot = sb(max(self.m, 1) * d * 2), sb(max(self.m, 1) * d * 2)
    self.s_dwslot = sb(max(self.m, 1) * self.parts * 4)
    self.s_counts, self.s_flags = sb(self.world * num_experts * 4), sb(self.world * 4)
    self.recv_x = self.s_x.local.tensor((self.rmax, d), bf)
    self.recv_w = self.s_w.local.tensor((self.rmax,), f32)
    self.ret = self.s_ret.local.tensor((self.rmax,), torch.int32)
    self.recv_dy = self.s_dy.local.tensor((self.rmax, d), bf)
    self.y_slot = self.s_yslot.local.tensor((max(self.m, 1), d), bf)[:self.m]
    self.dx_slot = self.s_dxslot.local.tensor((max(self.m, 1), d), bf)[:self.m]
    self.dw_slot = self.s_dwslot.local.tensor((max(self.m, 1), self.parts), f32)[:self.m]
    self.counts_all = self.s_counts.local.tensor((self.world * num_experts,), torch.int32)
    self.flags = self.s_flags.local.tensor((self.world,), torch.int32)
    # local to the owner
    if not self.fused_return:
      self.ys = torch.empty((self.rmax, d), dtype=bf, device=self.dev)
      self.dxs = torch.empty((self.rmax, d), dtype=bf, device=self.dev)
    if self.unique_push:
      import ctypes
      G, T = self.world, tokens
      self.umax = max(G * T, 1)   # every token of every rank may come here: nothing is dropped
      self.s_ux = sb(self.umax * d * 2)
      self.s_rowu, self.s_urows = sb(self.rmax * 4), sb(self.umax * k * 4)
      self.s_umeta, self.s_uret = sb(self.umax * 4), sb(self.umax * 4)
      self.s_ucounts = sb(G * G * 4)
      self.ux = self.s_ux.local.tensor((self.umax, d), bf)
      self.rowu = self.s_rowu.local.tensor((self.rmax,), torch.int32)
      self.urows = self.s_urows.local.tensor((self.umax, k), torch.int32)
      self.umeta = self.s_umeta.local.tensor((self.umax,), torch.int32)
      self.uret = self.s_uret.local.tensor((self.umax,), torch.int32)
      self.ucount_all = self.s_ucounts.local.tensor((G * G,), torch.int32)
      self.info = torch.zeros((max(T, 1), G), **i32)
      self.uidx = torch.zeros((max(T, 1), G), **i32)
      self.comb = torch.zeros((max(T, 1), G), **i32)
      self.ucount, self.usrc_base, self.utotal = torch.zeros(G, **i32), torch.zeros(G, **i32), torch.zeros(1, **i32)
      self.uws = torch.zeros(max(int(self.lib.lewi_ep_unique_workspace_bytes(T, G)), 4) // 4, **i32)
      self.c_bounds = (ctypes.c_int32 * len(self.bounds))(*self.bounds)
      self.rowu.fill_(-1)
      self.ucount_all.zero_()
      if self.combined_return:
        self.s_yrecv, self.s_dxrecv = sb(self.umax * d * 2), sb(self.umax * d * 2)
        self.y_recv = self.s_yrecv.local.tensor((self.umax, d), bf)
        self.dx_recv = self.s_dxrecv.local.tensor((self.umax, d), bf)
    self.dwp = torch.zeros((self.rmax, self.parts), dtype=f32, device=self.dev)
    self.dst_base = torch.zeros(num_experts, **i32)
    self.pad_offsets = torch.zeros(self.el + 1, **i32)
    self.valid_end = torch.zeros(self.el, **i32)
    self.n_blocks = torch.zeros(1, **i32)
    self.block_expert = torch.zeros(self.rmax // BLOCK, **i32)
    self.recv_rows = torch.zeros(1, **i32)
    self.slot_ids = torch.arange(max(self.m, 1), **i32)[:self.m].view(tokens, k)
    self._flag = torch.zeros(1, dtype=f32, device=self.dev)
    self._epoch = torch.zeros(1, **i32)   # barriers passed so far, counted on the device
    # Exchange kernels and whatever orders them between ranks run on their own stream, the GEMMs on the caller's.
    self.comm = torch.cuda.Stream(self.dev)
    self.gemm2 = torch.cuda.Stream(self.dev) if max(self.return_sms) > 0 else None
    self.recv_w.zero_()
    self.ret.fill_(-1)
    self.flags.zero_()
    self.counts_all.zero_()
    torch.cuda.synchronize(self.dev)
    dist.barrier(group=group)

  def overflowed(self):
    """Synchronises and reports whether a receive buffer was too small since the last status read (rows dropped).
    Any other device-side problem raises."""
    status = self._lib.last_status()
    if status & ~self._lib.STATUS_EP_OVERFLOW:
      raise self._lib.LewiError(f"device status {status}")
    return bool(status & self._lib.STATUS_EP_OVERFLOW)

  def close(self):
    """Releases the peer mappings and this rank's exchange buffers.  Collective: every rank calls it."""
    torch.cuda.synchronize(self.dev)
    dist.barrier(group=self.group)
    for name in ("s_x", "s_w", "s_ret", "s_dy", "s_yslot", "s_dxslot", "s_dwslot", "s_counts", "s_flags", "s_ux", "s_rowu",
                 "s_urows", "s_umeta", "s_uret", "s_ucounts", "s_yrecv", "s_dxrecv"):
      buf = getattr(self, name, None)
      if buf is not None:
        buf.close()
        setattr(self, name, None)
    for view in ("recv_x", "recv_w", "ret", "recv_dy", "y_slot", "dx_slot", "dw_slot", "counts_all", "flags", "ux", "rowu",
                 "urows", "umeta", "uret", "ucount_all", "y_recv", "dx_recv"):
      setattr(self, view, None)   # these pointed into the freed buffers
    dist.barrier(group=self.group)

  def _sm_count(self):
    return torch.cuda.get_device_properties(self.w.w_gate.device).multi_processor_count

  def _split_gemms(self, first, second, mark_done, p, sms):
    """The two GEMMs of range p: `first` (compute-bound) on the caller's stream, `second` (its epilogue stores to peers)
    after it — in line, or with `sms` > 0 on the second GEMM stream with that many CTAs while the caller's stream goes
    on with the next range's `first` on the other SMs.  The first range's `first` and the last range's `second` have
    nothing beside them and take the whole GPU."""
    if sms <= 0 or self.gemm2 is None:
      first()
      second()
      mark_done()
      return
    main = torch.cuda.current_stream(self.dev)
    try:
      self.lib.lewi_set_gemm_cta_limit(self._sm_count() - sms if p > 0 else 0)
      first()
      ready = main.record_event()
      self.lib.lewi_set_gemm_cta_limit(sms if p + 1 < self.phases else 0)
      with torch.cuda.stream(self.gemm2):
        self.gemm2.wait_event(ready)
        self.layer._mark("side_begin")
        second()
        mark_done(self.gemm2)
    finally:
      self.lib.lewi_set_gemm_cta_limit(0)

  def _sync_ranks(self):
    """Barrier between the ranks in the order of the current stream."""
    if self.sync == "nccl":
      dist.all_reduce(self._flag, group=self.group)
      return
    self._lib.check(self.lib.lewi_ep_barrier(self._lib.stream(), self.s_flags.c_ptrs, self._lib.ptr(self.flags),
                                             self._lib.ptr(self._epoch), self.rank, self.world, self.BARRIER_TIMEOUT_MS),
                    "lewi_ep_barrier")

  def _range(self, p):
    """(lo, hi, pad_offsets, block_expert, n_blocks) of local-expert range p."""
    lo, hi = self.bounds[p], self.bounds[p + 1]
    if self.phases == 1:
      return lo, hi, self.pad_offsets, self.block_expert, self.n_blocks
    # a sub-range has no block table of its own: the CTA-pair kernels read pad_offsets alone
    return lo, hi, self.pad_offsets[lo:hi + 1], None, None

  def _overlap_mode(self, on):
    """While a pass is queued the GEMM CTAs leave room on their SMs for one thin exchange CTA each."""
    self.lib.lewi_set_sm_sharing(1 if on else 0)

  def forward(self, x):
    self._overlap_mode(True)
    try:
      return self._forward(x)
    finally:
      self._overlap_mode(False)

  def _pipeline(self, push, gemms, give_back, first=None, last=None, tail=None):
    """Issue order of one pass.  On the exchange stream: push 0, push 1, then for every range p >= 1 push p+1 followed
    by the return of range p-1, last the return of the final range and a barrier.  On the caller's stream: the GEMMs of
    range p once its rows have arrived.  So while range p is being multiplied, range p+1 is arriving and range p-1 is
    on its way back.  `first` runs on the caller's stream while the first rows are in flight, `last` while the final
    range is on its way back, `tail` on the exchange stream right after the final barrier (work that needs what came
    back but not what `last` computes).  Returns with the caller's stream waiting for the final barrier and `tail`."""
    L, P = self.layer, self.phases
    main, comm = torch.cuda.current_stream(self.dev), self.comm
    arrived, done = {}, {}

    def do_push(p):
      with torch.cuda.stream(comm):
        push(p)
        self._sync_ranks()   # the rows of this range have arrived everywhere
        L._mark("ep_barrier")
        arrived[p] = comm.record_event()

    def do_return(p):
      with torch.cuda.stream(comm):
        comm.wait_event(done[p])
        L._mark("side_begin")
        give_back(p)

    do_push(0)
    if P > 1:
      do_push(1)
    if first is not None:
      first()   # work of the caller's stream that needs no rows from other ranks
    for p in range(P):
      if p >= 1:
        if p + 1 < P:
          do_push(p + 1)
        do_return(p - 1)
      main.wait_event(arrived[p])
      L._mark("step_begin")
      gemms(p, lambda stream=None, p=p: done.__setitem__(p, (stream or main).record_event()))
    do_return(P - 1)
    with torch.cuda.stream(comm):
      self._sync_ranks()   # everything is back at its source
      L._mark("ep_barrier")
      if tail is not None:
        tail()
      returned = comm.record_event()
    if last is not None:
      last()
    main.wait_event(returned)
    L._mark("step_begin")

  def _forward(self, x):
    lib, L, ops, _lib, w, k = self.lib, self.layer, self.ops, self._lib, self.w, self.k
    st, ptr, check = _lib.stream, _lib.ptr, _lib.check
    t, d = x.shape
    f, G = self.f, self.world
    main, comm = torch.cuda.current_stream(self.dev), self.comm
    logits = L.router_logits(x, w.w_router, w.router_bias)
    L._mark("router_logits")
    self.last_logits = logits
    tb = L.router_topk(logits, k)
    self.last_topk_idx = tb.topk_idx
    L._mark("router_topk")
    routed = main.record_event()
    with torch.cuda.stream(comm):
      comm.wait_event(routed)
      L._mark("side_begin")
      if self.unique_push:
        check(lib.lewi_ep_unique_tables(st(), ptr(tb.topk_idx), t, k, self.e, G, self.c_bounds, self.phases,
                                        ptr(self.info), ptr(self.uidx), ptr(self.comb), ptr(self.ucount), ptr(self.uws),
                                        self.uws.numel() * 4), "lewi_ep_unique_tables")
        check(lib.lewi_ep_put_i32(st(), ptr(self.ucount), self.s_ucounts.c_ptrs, self.rank * G, G, G), "lewi_ep_put_i32")
        L._mark("ep_unique_tables")
      check(lib.lewi_ep_put_i32(st(), ptr(tb.counts), self.s_counts.c_ptrs, self.rank * self.e, self.e, G),
            "lewi_ep_put_i32")
      L._mark("ep_put_counts")
      self._sync_ranks()   # histograms are everywhere; every rank is done with the buffers of the previous step
      L._mark("ep_barrier")
      check(lib.lewi_ep_plan(st(), ptr(self.counts_all), G, self.e, self.rank, BLOCK, self.rmax, ptr(self.dst_base),
                             ptr(self.pad_offsets), ptr(self.valid_end), ptr(self.n_blocks), ptr(self.block_expert),
                             ptr(self.recv_rows)), "lewi_ep_plan")
      L._mark("ep_plan")
      check(lib.lewi_ep_zero_pad(st(), ptr(self.recv_x), ptr(self.ret), ptr(self.valid_end), ptr(self.pad_offsets),
                                 self.el, d, self.rmax), "lewi_ep_zero_pad")
      L._mark("ep_zero_pad")
      if self.unique_push:
        check(lib.lewi_ep_unique_plan(st(), ptr(self.ucount_all), G, self.rank, self.umax, ptr(self.usrc_base),
                                      ptr(self.utotal)), "lewi_ep_unique_plan")
        check(lib.lewi_ep_zero_pad(st(), ptr(self.recv_x), ptr(self.rowu), ptr(self.valid_end), ptr(self.pad_offsets),
                                   self.el, d, self.rmax), "lewi_ep_zero_pad")
        check(lib.lewi_ep_unique_meta(st(), ptr(tb.topk_idx), ptr(tb.topk_w), ptr(tb.pos), ptr(tb.offsets),
                                      ptr(self.dst_base), ptr(self.info), ptr(self.uidx), ptr(self.usrc_base),
                                      self.s_w.c_ptrs, self.s_ret.c_ptrs, self.s_rowu.c_ptrs, self.s_urows.c_ptrs,
                                      self.s_umeta.c_ptrs, self.s_uret.c_ptrs, self.rank, t, k, self.e, G, self.rmax,
                                      self.umax), "lewi_ep_unique_meta")
        L._mark("ep_unique_meta")
    gu = torch.empty((self.rmax, 2 * f), dtype=torch.bfloat16, device=self.dev)
    h = torch.empty((self.rmax, f), dtype=torch.bfloat16, device=self.dev)
    shared = []

    def push(p):
      if self.unique_push:
        check(lib.lewi_ep_push_unique(st(), ptr(x), ptr(self.info), ptr(self.uidx), ptr(self.usrc_base), self.s_ux.c_ptrs,
                                      self.rank, t, d, G, p if self.phases > 1 else -1, self.umax, self.fwd_threads),
              "lewi_ep_push_unique")
      else:
        check(lib.lewi_ep_push_rows(st(), ptr(x), ptr(tb.order), ptr(tb.topk_idx), ptr(tb.offsets), ptr(self.dst_base),
                                    ptr(tb.topk_w), self.s_x.c_ptrs, self.s_w.c_ptrs, self.s_ret.c_ptrs, self.rank, self.m,
                                    k, d, self.e, G, self.rmax, t, self.bounds[p], self.bounds[p + 1], self.fwd_threads),
              "lewi_ep_push_rows")
      L._mark("ep_push_x")

    def gemms(p, mark_done):
      lo, hi, po, be, nb = self._range(p)
      if self.unique_push:   # the received rows go to the padded rows of this range's experts
        check(lib.lewi_ep_local_rows(st(), ptr(self.ux), ptr(self.rowu), ptr(self.pad_offsets), lo, hi, ptr(self.recv_x), d,
                                     self.rmax, self.umax), "lewi_ep_local_rows")
        L._mark("ep_local_rows_x")
      def gate_up():
        check(lib.lewi_grouped_gemm_gateup_swiglu_scaled(st(), ptr(self.recv_x), None, ptr(self.recv_w),
                                                         ptr(w.w_gate[lo:hi]), ptr(w.w_up[lo:hi]), ptr(gu), ptr(h), ptr(be),
                                                         ptr(nb), ptr(po), self.rmax, d, f, hi - lo),
              "lewi_grouped_gemm_gateup_swiglu")
        L._mark("gemm_gateup_swiglu")

      def down():
        if self.fused_return:
          check(lib.lewi_grouped_gemm_nn_return(st(), ptr(h), ptr(w.w_down[lo:hi]), ptr(self.ret), self.s_yslot.c_ptrs, G,
                                                self.m, ptr(be), ptr(nb), ptr(po), self.rmax, f, d, hi - lo),
                "lewi_grouped_gemm_nn_return")
        else:
          ops.grouped_gemm_nn(h, w.w_down[lo:hi], be, nb, pad_offsets=po, out=self.ys)
        L._mark("gemm_down")

      self._split_gemms(gate_up, down, mark_done, p, self.return_sms[0])

    def give_back(p):
      if self.fused_return:
        return   # the rows left with the GEMM's epilogue
      if self.combined_return:
        check(lib.lewi_ep_combine_return(st(), ptr(self.ys), ptr(self.urows), ptr(self.umeta), ptr(self.uret),
                                         ptr(self.utotal), p if self.phases > 1 else -1, self.s_yrecv.c_ptrs, k, d, G,
                                         self.rmax, self.umax, self.fwd_threads), "lewi_ep_combine_return")
        L._mark("ep_combine_return_y")
        return
      check(lib.lewi_ep_return_rows(st(), ptr(self.ys), None, ptr(self.ret), ptr(self.pad_offsets), self.bounds[p],
                                    self.bounds[p + 1], self.s_yslot.c_ptrs, None, d, self.parts, G, self.m, self.rmax,
                                    self.fwd_threads), "lewi_ep_return_rows")
      L._mark("ep_return_y")

    def shared_expert():   # needs nothing from other ranks: it fills the time the first rows are in flight
      if w.ws_gate is None:
        return
      gus, hs = L.gateup_swiglu(x, w.ws_gate[None], w.ws_up[None], None, None)
      L._mark("shared_gateup_swiglu")
      shared.extend((gus, hs, ops.grouped_gemm_nn(hs, w.ws_down[None], None, None)))
      L._mark("shared_down")

    self._pipeline(push, gemms, give_back, first=shared_expert)
    if self.combined_return:   # one partial row per rank the token went to
      out = ops.gather_reduce(self.y_recv, self.comb[:t], None, x.dtype, add0=shared[2] if shared else None)
    else:
      out = ops.gather_reduce(self.y_slot, self.slot_ids, None, x.dtype, add0=shared[2] if shared else None)
    L._mark("combine_reduce")
    return out, dict(x=x, logits=logits, tb=tb, gu=gu, h=h, shared=tuple(shared) or None)

  def backward(self, dout, c):
    self._overlap_mode(True)
    try:
      return self._backward(dout, c)
    finally:
      self._overlap_mode(False)

  def _backward(self, dout, c):
    lib, L, ops, _lib, w, k = self.lib, self.layer, self.ops, self._lib, self.w, self.k
    st, ptr, check = _lib.stream, _lib.ptr, _lib.check
    x, tb = c["x"], c["tb"]
    t, d = x.shape
    f, G = self.f, self.world
    main, comm = torch.cuda.current_stream(self.dev), self.comm
    dout = dout.contiguous()
    ready = main.record_event()
    with torch.cuda.stream(comm):
      comm.wait_event(ready)
      L._mark("side_begin")
      if not self.unique_push:   # (the owner's local copy writes the zero rows itself)
        check(lib.lewi_ep_zero_pad(st(), ptr(self.recv_dy), None, ptr(self.valid_end), ptr(self.pad_offsets), self.el, d,
                                   self.rmax), "lewi_ep_zero_pad")
        L._mark("ep_zero_pad")
    grads = {}
    dxsh = []

    def shared_expert():
      if c["shared"] is None:
        return
      gus, hs, _ = c["shared"]
      dgus = L.dh_dswiglu(dout, w.ws_down[None], gus, None, None)
      L._mark("shared_dh_dswiglu")
      grads["dws_down"] = ops.grouped_gemm_tn(hs, dout, None, 1, out_dtype=w.ws_down.dtype)[0]
      L._mark("shared_dw_down")
      dxsh.append(L.dx_from_dgu(dgus, w.ws_gate[None], w.ws_up[None], None, None))
      L._mark("shared_dx")
      g1, g2 = ops.grouped_gemm_tn(x, dgus, None, 1, out_dtype=w.ws_gate.dtype, split=True)
      L._mark("shared_dw_gateup")
      grads["dws_gate"], grads["dws_up"] = g1[0], g2[0]

    dgu = torch.empty((self.rmax, 2 * f), dtype=torch.bfloat16, device=self.dev)
    grads["dw_down"] = torch.empty_like(w.w_down)
    grads["dw_gate"], grads["dw_up"] = torch.empty_like(w.w_gate), torch.empty_like(w.w_up)

    def push(p):
      if self.unique_push:
        check(lib.lewi_ep_push_unique(st(), ptr(dout), ptr(self.info), ptr(self.uidx), ptr(self.usrc_base),
                                      self.s_ux.c_ptrs, self.rank, t, d, G, p if self.phases > 1 else -1, self.umax,
                                      self.bwd_threads), "lewi_ep_push_unique")
      else:
        check(lib.lewi_ep_push_rows(st(), ptr(dout), ptr(tb.order), ptr(tb.topk_idx), ptr(tb.offsets), ptr(self.dst_base),
                                    None, self.s_dy.c_ptrs, None, None, self.rank, self.m, k, d, self.e, G, self.rmax, t,
                                    self.bounds[p], self.bounds[p + 1], self.bwd_threads), "lewi_ep_push_rows")
      L._mark("ep_push_dout")

    def gemms(p, mark_done):
      lo, hi, po, be, nb = self._range(p)
      if self.unique_push:
        check(lib.lewi_ep_local_rows(st(), ptr(self.ux), ptr(self.rowu), ptr(self.pad_offsets), lo, hi, ptr(self.recv_dy),
                                     d, self.rmax, self.umax), "lewi_ep_local_rows")
        L._mark("ep_local_rows_dout")
      def dh():
        check(lib.lewi_grouped_gemm_dh_dswiglu_scaled(st(), ptr(self.recv_dy), None, ptr(self.recv_w),
                                                      ptr(self.dwp), ptr(w.w_down[lo:hi]), ptr(c["gu"]), ptr(dgu), ptr(be),
                                                      ptr(nb), ptr(po), self.rmax, d, f, hi - lo),
              "lewi_grouped_gemm_dh_dswiglu")
        L._mark("gemm_dh_dswiglu")

      def dx():
        if self.fused_return:
          check(lib.lewi_grouped_gemm_dx_return(st(), ptr(dgu), ptr(w.w_gate[lo:hi]), ptr(w.w_up[lo:hi]), ptr(self.ret),
                                                self.s_dxslot.c_ptrs, G, self.m, ptr(be), ptr(nb), ptr(po), self.rmax, d, f,
                                                hi - lo), "lewi_grouped_gemm_dx_return")
        else:
          check(lib.lewi_grouped_gemm_dx(st(), ptr(dgu), ptr(w.w_gate[lo:hi]), ptr(w.w_up[lo:hi]), ptr(self.dxs), ptr(be),
                                         ptr(nb), ptr(po), self.rmax, d, f, hi - lo), "lewi_grouped_gemm_dx")
        L._mark("gemm_dx")

      self._split_gemms(dh, dx, mark_done, p, self.return_sms[1])   # (the other ranks do not wait for the weight gradients)
      if not self.dw_deferred:
        weight_grads(lo, hi, po)

    def weight_grads(lo, hi, po):
      def dw_down():
        ops.grouped_gemm_tn(c["h"], self.recv_dy, po, hi - lo, out=grads["dw_down"][lo:hi])
        L._mark("gemm_dw_down")

      def dw_gateup():
        ops.grouped_gemm_tn(self.recv_x, dgu, po, hi - lo, out=grads["dw_gate"][lo:hi], out2=grads["dw_up"][lo:hi],
                            split=True)
        L._mark("gemm_dw_gateup")

      # A return of dx rows shares the SMs with these.  dW_down (few tiles, long contraction) was measured 3x slower
      # beside it, dW_gate|up 1.1x: the robust one goes first.
      for gemm in ((dw_gateup, dw_down) if self.dw_down_last else (dw_down, dw_gateup)):
        gemm()

    def all_weight_grads():
      # One pair of launches over every local expert: each has enough tiles to fill the GPU (a range of a few experts
      # does not), and they run while the last range's dx rows travel home.
      if self.dw_deferred:
        weight_grads(0, self.el, self.pad_offsets)

    def give_back(p):
      # fused: the dx rows left with the GEMM's epilogue; only the routing-weight gradient pieces remain
      rows_too = not (self.fused_return or self.combined_return)
      check(lib.lewi_ep_return_rows(st(), ptr(self.dxs) if rows_too else None, ptr(self.dwp), ptr(self.ret),
                                    ptr(self.pad_offsets), self.bounds[p], self.bounds[p + 1],
                                    self.s_dxslot.c_ptrs if rows_too else None, self.s_dwslot.c_ptrs, d,
                                    self.parts, G, self.m, self.rmax, self.bwd_threads), "lewi_ep_return_rows")
      L._mark("ep_return_dx" if rows_too else "ep_return_dw")
      if self.combined_return:
        check(lib.lewi_ep_combine_return(st(), ptr(self.dxs), ptr(self.urows), ptr(self.umeta), ptr(self.uret),
                                         ptr(self.utotal), p if self.phases > 1 else -1, self.s_dxrecv.c_ptrs, k, d, G,
                                         self.rmax, self.umax, self.bwd_threads), "lewi_ep_combine_return")
        L._mark("ep_combine_return_dx")

    router = {}

    def router_backward():
      # needs the routing-weight gradient pieces that came back, nothing of the weight-gradient GEMMs: it runs on the
      # exchange stream beside them.  (Its outputs are allocated on that stream; every later use of the stream starts
      # by waiting for an event of the caller's stream, so the allocator cannot hand their memory out too early.)
      _, dlb, dw = L.router_topk_bwd(c["logits"], tb.topk_idx, None, want_f32=False, want_bf16=True,
                                     dw_partial=self.dw_slot, pad_pos=self.slot_ids)
      L._mark("router_topk_bwd")
      grads["dw"] = dw
      router["dx"] = ops.grouped_gemm_nt(dlb, L.cast_bf16(w.w_router)[None], None, None)
      L._mark("router_dx")
      grads["dw_router"] = ops.grouped_gemm_tn(x, dlb, None, 1, out_dtype=torch.float32)[0]
      L._mark("router_dw")

    self._pipeline(push, gemms, give_back, first=shared_expert, last=all_weight_grads,
                   tail=router_backward if self.router_tail else None)
    if not self.router_tail:
      router_backward()
    dx_r = router["dx"]
    if self.combined_return:
      grads["dx"] = ops.gather_reduce(self.dx_recv, self.comb[:t], None, x.dtype, add0=dxsh[0] if dxsh else None, add1=dx_r)
    else:
      grads["dx"] = ops.gather_reduce(self.dx_slot, self.slot_ids, None, x.dtype, add0=dxsh[0] if dxsh else None,
                                      add1=dx_r)
    L._mark("combine_bwd_reduce")
    return grads

  def step(self, x, dout):
    out, cache = self.forward(x)
    return out, self.backward(dout, cache)

  def exchange_summary(self, topk_idx):
    """Rows this rank sends to OTHER ranks per pass for the routing `topk_idx` [T,k] (global expert ids), counted both
    ways: once per (token, expert) slot and once per (token, destination rank); and the mode this layer runs in.
    Synchronises (reads a few numbers back)."""
    ranks = (topk_idx // self.el).to(torch.int64)
    away = ranks != self.rank
    per_rank = torch.zeros((topk_idx.shape[0], self.world), dtype=torch.bool, device=topk_idx.device)
    per_rank.scatter_(1, ranks, True)
    per_rank[:, self.rank] = False
    slots, unique = int(away.sum().item()), int(per_rank.sum().item())
    row_bytes = 2 * self.d
    return dict(push="unique" if self.unique_push else "slots",
                back="combined" if self.combined_return else ("fused" if self.fused_return else "kernel"),
                ranges=self.phases, rows_sent_per_slot=slots, rows_sent_once_per_rank=unique,
                push_bytes_per_pass=(unique if self.unique_push else slots) * row_bytes,
                return_bytes_per_pass=(unique if self.combined_return else slots) * row_bytes)
