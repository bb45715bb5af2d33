"""Weight-layout adapters for the MoE layer: MaxText parameter tree <-> `MoEWeights` <-> Hugging Face tensors, and
the reference's two growth recipes expressed on the layer's own layout.

Layouts (one MoE layer):
  MaxText tree (modal/stage2.py:338-345)       `mlp/routed_experts/gate/kernel` [d,E] (experts on the LAST axis),
                                               `mlp/routed_experts/wi_0`, `wi_1` [E,d,f], `wo` [E,f,d],
                                               `mlp/shared_expert/wi_0/kernel`, `wi_1/kernel` [d,fs], `wo/kernel` [fs,d]
  this library (`layer.MoEWeights`)            the same orientation: no transposition between MaxText and the kernels
  Hugging Face qwen3_5_moe (tools/grow_7b.py:104-112, kaggle/stage2/conv_wrapper.py:32-39)
                                               `mlp.gate.weight` [E,H], `mlp.experts.gate_up_proj` [E,2I,H] (rows 0..I-1
                                               gate, I..2I-1 up), `mlp.experts.down_proj` [E,H,I],
                                               `mlp.shared_expert.{gate,up,down}_proj.weight` [I_s,H] / [H,I_s],
                                               `mlp.shared_expert_gate.weight` [1,H]
All functions work on NumPy arrays or torch tensors of any device (plain indexing, concatenation, transposition);
nothing here launches a kernel, so the module is testable on a CPU.
"""
from __future__ import annotations

import numpy as np

MAXTEXT_KEYS = {
    "w_router": "mlp/routed_experts/gate/kernel",
    "w_gate": "mlp/routed_experts/wi_0",
    "w_up": "mlp/routed_experts/wi_1",
    "w_down": "mlp/routed_experts/wo",
    "ws_gate": "mlp/shared_expert/wi_0/kernel",
    "ws_up": "mlp/shared_expert/wi_1/kernel",
    "ws_down": "mlp/shared_expert/wo/kernel",
}
HF_KEYS = ("mlp.gate.weight", "mlp.experts.gate_up_proj", "mlp.experts.down_proj", "mlp.shared_expert.gate_proj.weight",
           "mlp.shared_expert.up_proj.weight", "mlp.shared_expert.down_proj.weight", "mlp.shared_expert_gate.weight")


def _is_torch(a):
  return type(a).__module__.startswith("torch")


def _cat(parts, axis):
  if _is_torch(parts[0]):
    import torch
    return torch.cat(list(parts), dim=axis)
  return np.concatenate(list(parts), axis=axis)


def _swap(a, i, j):
  return a.transpose(i, j) if _is_torch(a) else np.swapaxes(a, i, j)


def _contig(a):
  return a.contiguous() if _is_torch(a) else np.ascontiguousarray(a)


def _walk(tree, path):
  node = tree
  for part in path.split("/"):
    node = node[part]
  return node


def from_maxtext(tree, prefix=""):
  """One layer's arrays out of a MaxText parameter tree (nested dicts, keys as in modal/stage2.py:338-345) as a dict
  with `MoEWeights` field names.  The orientation is already the kernels'; a missing shared expert gives no ws_* keys."""
  out = {}
  for name, key in MAXTEXT_KEYS.items():
    try:
      out[name] = _walk(tree, prefix + key if not prefix or prefix.endswith("/") else prefix + "/" + key)
    except (KeyError, TypeError):
      if not name.startswith("ws_"):
        raise KeyError(f"MaxText tree has no {key!r}") from None
  return out


def to_maxtext(w):
  """Inverse of from_maxtext: nested dicts keyed like the MaxText tree, from a dict / object with MoEWeights fields."""
  get = (lambda n: w.get(n)) if isinstance(w, dict) else (lambda n: getattr(w, n, None))
  tree = {}
  for name, key in MAXTEXT_KEYS.items():
    val = get(name)
    if val is None:
      continue
    node = tree
    parts = key.split("/")
    for part in parts[:-1]:
      node = node.setdefault(part, {})
    node[parts[-1]] = val
  return tree


def from_hf(sd, prefix=""):
  """Hugging Face tensors of one `Qwen3_5MoeSparseMoeBlock` (tools/grow_7b.py:104-112) -> dict with MoEWeights field
  names.  gate_up_proj [E,2I,H] splits into gate rows 0..I-1 and up rows I..2I-1, each transposed to [E,H,I];
  down_proj [E,H,I] -> [E,I,H]; gate.weight [E,H] -> [H,E]; shared_expert_gate.weight [1,H] -> w_sg [H]."""
  g = lambda k: sd[prefix + k]
  gu = g("mlp.experts.gate_up_proj")
  i = gu.shape[1] // 2
  out = {
      "w_router": _contig(_swap(g("mlp.gate.weight"), 0, 1)),
      "w_gate": _contig(_swap(gu[:, :i, :], 1, 2)),
      "w_up": _contig(_swap(gu[:, i:, :], 1, 2)),
      "w_down": _contig(_swap(g("mlp.experts.down_proj"), 1, 2)),
  }
  if prefix + "mlp.shared_expert.gate_proj.weight" in sd:
    out["ws_gate"] = _contig(_swap(g("mlp.shared_expert.gate_proj.weight"), 0, 1))
    out["ws_up"] = _contig(_swap(g("mlp.shared_expert.up_proj.weight"), 0, 1))
    out["ws_down"] = _contig(_swap(g("mlp.shared_expert.down_proj.weight"), 0, 1))
  if prefix + "mlp.shared_expert_gate.weight" in sd:
    out["w_sg"] = _contig(g("mlp.shared_expert_gate.weight")[0])
  return out


def to_hf(w, prefix=""):
  """Inverse of from_hf."""
  get = (lambda n: w.get(n)) if isinstance(w, dict) else (lambda n: getattr(w, n, None))
  sd = {
      prefix + "mlp.gate.weight": _contig(_swap(get("w_router"), 0, 1)),
      prefix + "mlp.experts.gate_up_proj": _contig(_cat([_swap(get("w_gate"), 1, 2), _swap(get("w_up"), 1, 2)], 1)),
      prefix + "mlp.experts.down_proj": _contig(_swap(get("w_down"), 1, 2)),
  }
  if get("ws_gate") is not None:
    sd[prefix + "mlp.shared_expert.gate_proj.weight"] = _contig(_swap(get("ws_gate"), 0, 1))
    sd[prefix + "mlp.shared_expert.up_proj.weight"] = _contig(_swap(get("ws_up"), 0, 1))
    sd[prefix + "mlp.shared_expert.down_proj.weight"] = _contig(_swap(get("ws_down"), 0, 1))
  if get("w_sg") is not None:
    sd[prefix + "mlp.shared_expert_gate.weight"] = get("w_sg")[None]
  return sd


def grow_experts(w, expert_mult=2, noise=1e-3, seed=0):
  """The expert half of the reference's net2net growth (`grow_tree`, modal/stage2.py:318-348): every expert tensor is
  followed by `expert_mult - 1` noisy copies of the whole stack (noise = `noise` x the tensor's standard deviation,
  drawn in the order wi_0, wi_1, wo, gate as the tree is walked), the router kernel grows the same way along its
  expert (last) axis.  Expert e and expert e + E start out as near-twins, so the layer's output barely moves.
  NumPy arrays in, NumPy arrays out; shared-expert weights pass through."""
  rng = np.random.default_rng(seed)
  get = (lambda n: w.get(n)) if isinstance(w, dict) else (lambda n: getattr(w, n, None))
  out = {n: get(n) for n in ("ws_gate", "ws_up", "ws_down", "w_sg", "router_bias") if get(n) is not None}

  def grown(a, axis):
    a = np.asarray(a)
    sd = float(np.std(a.astype(np.float32))) + 1e-8
    copies = [a] + [a + (rng.standard_normal(a.shape) * noise * sd).astype(a.dtype) for _ in range(expert_mult - 1)]
    return np.concatenate(copies, axis=axis)

  # the reference visits dict keys in insertion order of the MaxText tree: gate kernel first, then wi_0, wi_1, wo
  out["w_router"] = grown(get("w_router"), -1)
  for name in ("w_gate", "w_up", "w_down"):
    out[name] = grown(get(name), 0)
  if "router_bias" in out:
    out["router_bias"] = np.concatenate([np.asarray(out["router_bias"])] * expert_mult)
  return out


def merge_expert_pairs(w, usage=None, eps=0.5):
  """The reference's expert merge to half as many experts of twice the width (`merge_experts`,
  tools/grow_7b.py:84-112), on this library's layout: experts are paired (adjacent pairs, or by `usage`: i-th most
  used with i-th least used), the pair's gate / up columns are concatenated ([E,d,f] -> [E/2,d,2f] = [a | b]), the
  down rows likewise with the second expert's scaled by `eps` ([E,f,d] -> [E/2,2f,d] = [a ; eps*b]), and the router
  keeps the first ("strong") expert's column."""
  get = (lambda n: w.get(n)) if isinstance(w, dict) else (lambda n: getattr(w, n, None))
  wg, wu, wd, wr = (np.asarray(get(n)) for n in ("w_gate", "w_up", "w_down", "w_router"))
  e = wg.shape[0]
  if e % 2:
    raise ValueError("merge_expert_pairs needs an even number of experts")
  if usage is not None:
    order = np.argsort(-np.asarray(usage))
    sa, sb = order[: e // 2], order[e // 2:][::-1]
  else:
    idx = np.arange(e)
    sa, sb = idx[0::2], idx[1::2]
  out = {n: get(n) for n in ("ws_gate", "ws_up", "ws_down", "w_sg") if get(n) is not None}
  out["w_gate"] = np.concatenate([wg[sa], wg[sb]], axis=2)
  out["w_up"] = np.concatenate([wu[sa], wu[sb]], axis=2)
  out["w_down"] = np.concatenate([wd[sa], (wd[sb].astype(np.float32) * eps).astype(wd.dtype)], axis=1)
  out["w_router"] = wr[:, sa]
  if get("router_bias") is not None:
    out["router_bias"] = np.asarray(get("router_bias"))[sa]
  return out
