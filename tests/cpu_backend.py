"""CPU stand-in for lewi_surge_b200.ep.CudaBackend, built on the oracle.  TEST ONLY: it lets the
expert-parallel exchange logic run under gloo on machines without a GPU."""
from types import SimpleNamespace

import numpy as np
import torch

import oracle as O


def _t(a, dtype=torch.float32):
  return torch.from_numpy(np.ascontiguousarray(a)).to(dtype)


class CpuBackend:

  def route(self, x, w_router, bias, k):
    logits = x.numpy() @ w_router.numpy()
    if bias is not None:
      logits = logits + bias.numpy()[None]
    idx, w, p = O.router_topk(logits, k)
    e = w_router.shape[1]
    order, pos = O.sort_indices(idx.reshape(-1), e)
    tb = SimpleNamespace(topk_idx=_t(idx, torch.int32), topk_w=_t(w), order=_t(order, torch.int32), pos=_t(pos, torch.int32),
                         counts=_t(np.bincount(idx.reshape(-1), minlength=e), torch.int32))
    return _t(logits), tb

  def sort_padded(self, flat_e, num_experts):
    L = O.block_layout(flat_e.numpy(), num_experts, 128)
    return dict(pad_offsets=_t(L["pad_offsets"], torch.int32), block_expert=_t(L["block_expert"], torch.int32),
                n_blocks=torch.tensor([L["n_blocks"]], dtype=torch.int32), pad_pos=_t(L["pad_pos"], torch.int32),
                row_slot=_t(L["row_slot"], torch.int32), counts=_t(L["counts"], torch.int32), mpad=L["mpad"])

  def gather_rows(self, x, idx, scale=None, idx_div=1, scale_by_idx=False, n_out=None):
    raw = idx.numpy().astype(np.int64)
    src = np.where(raw >= 0, raw // idx_div, -1)
    sc = None
    if scale is not None:
      s = scale.numpy()
      sc = s[np.clip(raw, 0, None)] if scale_by_idx else s
    return _t(O.gather_rows(x.numpy(), src, sc))

  def gather_reduce(self, y, pos, w, out_dtype, add0=None, add1=None):
    out = O.gather_reduce(y.numpy(), pos.numpy(), None if w is None else w.numpy())
    for a in (add0, add1):
      if a is not None:
        out = out + a.numpy()
    return _t(out)

  def gather_dot(self, y, pos, g):
    return _t(O.gather_dot(y.numpy(), pos.numpy(), g.numpy()))

  @staticmethod
  def _gs(t):
    po = t["pad_offsets"].numpy()
    return po, t["counts"].numpy()

  def experts_fwd(self, xs_pad, w_gate, w_up, w_down, t):
    po, cnt = self._gs(t)
    x = xs_pad.numpy()
    gu = np.zeros((x.shape[0], 2 * w_gate.shape[2]), np.float32)
    h = np.zeros((x.shape[0], w_gate.shape[2]), np.float32)
    ys = np.zeros_like(x)
    f = w_gate.shape[2]
    for e in range(w_gate.shape[0]):
      s = slice(po[e], po[e] + cnt[e])
      g, u = x[s] @ w_gate[e].numpy(), x[s] @ w_up[e].numpy()
      gu[s, :f], gu[s, f:] = g, u
      h[s] = O.silu(g) * u
      ys[s] = h[s] @ w_down[e].numpy()
    return _t(gu), _t(h), _t(ys)

  def experts_bwd(self, dys_pad, xs_pad, gu, h, w_gate, w_up, w_down, t):
    po, cnt = self._gs(t)
    f = w_gate.shape[2]
    dy, x, gu, h = dys_pad.numpy(), xs_pad.numpy(), gu.numpy(), h.numpy()
    dxs = np.zeros_like(x)
    dwg, dwu, dwd = (np.zeros(tuple(w.shape), np.float32) for w in (w_gate, w_up, w_down))
    for e in range(w_gate.shape[0]):
      s = slice(po[e], po[e] + cnt[e])
      dh = dy[s] @ w_down[e].numpy().T
      g, u = gu[s, :f], gu[s, f:]
      dg, du = dh * u * O.dsilu(g), dh * O.silu(g)
      dwd[e] = h[s].T @ dy[s]
      dwg[e], dwu[e] = x[s].T @ dg, x[s].T @ du
      dxs[s] = dg @ w_gate[e].numpy().T + du @ w_up[e].numpy().T
    return _t(dxs), _t(dwg), _t(dwu), _t(dwd)

  def shared_fwd(self, x, ws_gate, ws_up, ws_down):
    g, u = x.numpy() @ ws_gate.numpy(), x.numpy() @ ws_up.numpy()
    h = O.silu(g) * u
    return _t(np.concatenate([g, u], 1)), _t(h), _t(h @ ws_down.numpy())

  def shared_bwd(self, dout, x, gus, hs, ws_gate, ws_up, ws_down):
    fs = ws_gate.shape[1]
    g, u = gus.numpy()[:, :fs], gus.numpy()[:, fs:]
    dh = dout.numpy() @ ws_down.numpy().T
    dg, du = dh * u * O.dsilu(g), dh * O.silu(g)
    dx = dg @ ws_gate.numpy().T + du @ ws_up.numpy().T
    return _t(dx), _t(x.numpy().T @ dg), _t(x.numpy().T @ du), _t(hs.numpy().T @ dout.numpy())

  def router_bwd(self, x, logits, topk_idx, dw, w_router):
    dl = O.router_topk_bwd(logits.numpy(), topk_idx.numpy(), dw.numpy())
    return _t(dl @ w_router.numpy().T), _t(x.numpy().T @ dl)

  def zero_rows(self, n, d, like):
    return torch.empty((n, d), dtype=like.dtype)
