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
