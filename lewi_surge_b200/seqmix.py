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


def chunk_gated_delta_rule(query, key, value, g, beta, chunk_size=64, initial_state=None):
  """Forward of the chunked gated delta rule with the signature of the reference's
  `fast_chunk_gated_delta_rule` (modal/gdn_fast.py:37): query, key [B,S,H,K], value [B,S,H,V] bf16, g [B,S,H]
  (log decay), beta [B,S,H]; returns (o [B,S,H,V] bf16, final state [B,H,K,V] bf16 or None when no initial state
  was given, as the reference does).  Not differentiable (no backward kernel)."""
  lib = _lib.load()
  if chunk_size != 64:
    raise LewiError("chunk_gated_delta_rule: the kernels work in chunks of 64 tokens")
  if query.dtype != torch.bfloat16 or key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16:
    raise LewiError("chunk_gated_delta_rule takes bfloat16 q, k, v")
  b, s, h, kd = key.shape
  vd = value.shape[-1]
  q, k, v = query.contiguous(), key.contiguous(), value.contiguous()
  gf = g.to(torch.float32).contiguous()
  bb = beta.to(torch.bfloat16).contiguous()
  o = torch.empty((b, s, h, vd), dtype=torch.bfloat16, device=q.device)
  h0 = initial_state.to(torch.float32).contiguous() if initial_state is not None else None
  hf = torch.empty((b, h, kd, vd), dtype=torch.float32, device=q.device) if initial_state is not None else None
  ws_bytes = int(lib.lewi_gdn_chunk_workspace_bytes(b, s, h, kd, vd))
  if ws_bytes < 0:
    check(ws_bytes, "lewi_gdn_chunk_workspace_bytes")
  ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
  check(lib.lewi_gdn_chunk_fwd(stream(), ptr(q), ptr(k), ptr(v), ptr(gf), ptr(bb), ptr(h0), ptr(o), ptr(hf), ptr(ws), ws_bytes,
                               b, s, h, kd, vd), "lewi_gdn_chunk_fwd")
  return o, (hf.to(torch.bfloat16) if hf is not None else None)
