"""Host-side mirror of the reference's sequence-mixing patches, backed by the sm_100a kernels.

`causal_conv1d(x, w)` is the causal depthwise 1-D convolution the reference rewrites as shift-adds
(`_fast_call`, modal/fast_conv.py:14-31): x [B,T,C] bf16, w [K,1,C] (the flax kernel layout) -> y [B,T,C].
Differentiable through `torch.autograd`; no fallback path.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import LewiError, check, ptr, stream


class _CausalConv1d(torch.autograd.Function):

  @staticmethod
  def forward(ctx, x, w):
    lib = _lib.load()
    if x.dim() != 3 or w.dim() != 3 or w.shape[1] != 1 or w.shape[2] != x.shape[2]:
      raise LewiError("causal_conv1d: x [B,T,C] and a depthwise kernel w [K,1,C] are required")
    if x.dtype != torch.bfloat16:
      raise LewiError("causal_conv1d takes bfloat16 activations")
    x = x.contiguous()
    wb = w.to(torch.bfloat16).contiguous()
    b, t, c = x.shape
    y = torch.empty_like(x)
    check(lib.lewi_causal_conv1d_fwd(stream(), ptr(x), ptr(wb), ptr(y), b, t, c, w.shape[0]), "lewi_causal_conv1d_fwd")
    ctx.save_for_backward(x, wb)
    ctx.w_dtype = w.dtype
    return y

  @staticmethod
  def backward(ctx, g):
    lib = _lib.load()
    x, wb = ctx.saved_tensors
    b, t, c = x.shape
    k = wb.shape[0]
    g = g.contiguous()
    dx = torch.empty_like(x)
    dw = torch.empty((k, 1, c), dtype=torch.float32, device=x.device)
    ws_bytes = int(lib.lewi_causal_conv1d_workspace_bytes(b, t, c, k))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device)
    check(lib.lewi_causal_conv1d_bwd(stream(), ptr(x), ptr(wb), ptr(g), ptr(dx), ptr(dw), _lib.F32, ptr(ws), ws_bytes, b, t,
                                     c, k), "lewi_causal_conv1d_bwd")
    return dx, dw.to(ctx.w_dtype)


def causal_conv1d(x, w):
  """y[b,t,c] = sum_j w[j,0,c] * x[b, t-(K-1)+j, c] (zero before the sequence starts).  Reference:
  `_fast_call`, modal/fast_conv.py:14-31."""
  return _CausalConv1d.apply(x, w)


class _ChunkGatedDeltaRule(torch.autograd.Function):
  """o, final state = chunked gated delta rule; the backward pass is `lewi_gdn_chunk_bwd`."""

  @staticmethod
  def forward(ctx, q, k, v, g, beta, h0):
    lib = _lib.load()
    b, s, h, kd = k.shape
    vd = v.shape[-1]
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    gf = g.to(torch.float32).contiguous()
    bb = beta.to(torch.bfloat16).contiguous()
    o = torch.empty((b, s, h, vd), dtype=torch.bfloat16, device=q.device)
    h0f = h0.to(torch.float32).contiguous() if h0 is not None else None
    hf = torch.empty((b, h, kd, vd), dtype=torch.float32, device=q.device)
    ws_bytes = int(lib.lewi_gdn_chunk_workspace_bytes(b, s, h, kd, vd))
    if ws_bytes < 0:
      check(ws_bytes, "lewi_gdn_chunk_workspace_bytes")
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    check(lib.lewi_gdn_chunk_fwd(stream(), ptr(q), ptr(k), ptr(v), ptr(gf), ptr(bb), ptr(h0f), ptr(o), ptr(hf), ptr(ws),
                                 ws_bytes, b, s, h, kd, vd), "lewi_gdn_chunk_fwd")
    ctx.save_for_backward(q, k, v, gf, bb, h0f, ws)
    ctx.set_materialize_grads(False)   # an output nobody differentiates arrives as None, not as a tensor of zeros
    ctx.in_dtypes = (g.dtype, beta.dtype, h0.dtype if h0 is not None else None)
    return o, hf

  @staticmethod
  def backward(ctx, d_o, d_hf):
    lib = _lib.load()
    q, k, v, gf, bb, h0f, ws = ctx.saved_tensors
    b, s, h, kd = k.shape
    vd = v.shape[-1]
    d_o = d_o.to(torch.bfloat16).contiguous() if d_o is not None else torch.zeros_like(v)
    d_hf = d_hf.to(torch.float32).contiguous() if d_hf is not None else None
    bws_bytes = int(lib.lewi_gdn_chunk_bwd_workspace_bytes(b, s, h, kd, vd))
    if bws_bytes < 0:
      check(bws_bytes, "lewi_gdn_chunk_bwd_workspace_bytes")
    bws = torch.empty(bws_bytes, dtype=torch.uint8, device=q.device)
    dq, dk, dv, db = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(bb)
    dg = torch.empty_like(gf)
    dh0 = torch.empty_like(h0f) if h0f is not None else None
    check(lib.lewi_gdn_chunk_bwd(stream(), ptr(q), ptr(k), ptr(v), ptr(gf), ptr(bb), ptr(h0f), ptr(d_o), ptr(d_hf), ptr(ws),
                                 ws.numel(), ptr(bws), bws_bytes, ptr(dq), ptr(dk), ptr(dv), ptr(dg), ptr(db), ptr(dh0), b,
                                 s, h, kd, vd), "lewi_gdn_chunk_bwd")
    g_dt, b_dt, h_dt = ctx.in_dtypes
    return dq, dk, dv, dg.to(g_dt), db.to(b_dt), (dh0.to(h_dt) if dh0 is not None else None)


def chunk_gated_delta_rule(query, key, value, g, beta, chunk_size=64, initial_state=None):
  """The chunked gated delta rule with the signature of the reference's `fast_chunk_gated_delta_rule`
  (modal/gdn_fast.py:37): query, key [B,S,H,K], value [B,S,H,V] bf16, g [B,S,H] (log decay), beta [B,S,H]; returns
  (o [B,S,H,V] bf16, final state [B,H,K,V] bf16 or None when no initial state was given, as the reference does).
  Differentiable through `torch.autograd` in q, k, v, g, beta and the initial state (head dimensions up to 128)."""
  if chunk_size != 64:
    raise LewiError("chunk_gated_delta_rule: the kernels work in chunks of 64 tokens")
  if query.dtype != torch.bfloat16 or key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16:
    raise LewiError("chunk_gated_delta_rule takes bfloat16 q, k, v")
  o, hf = _ChunkGatedDeltaRule.apply(query, key, value, g, beta, initial_state)
  return o, (hf.to(torch.bfloat16) if initial_state is not None else None)
