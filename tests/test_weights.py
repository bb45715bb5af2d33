"""Weight-layout adapters and growth recipes (CPU only), pinned to outputs of the reference's own functions
(tests/golden/make_golden_weights.py ran `grow_tree` of modal/stage2.py and `merge_experts` of tools/grow_7b.py)."""
import os

import numpy as np
import pytest
import torch

from lewi_surge_b200 import weights as W

HERE = os.path.dirname(os.path.abspath(__file__))
Z = np.load(os.path.join(HERE, "golden", "weight_growth.npz"))


def small_layer(rng, e=6, d=8, f=4, fs=6):
  n = lambda *s: rng.standard_normal(s).astype(np.float32)
  return dict(w_router=n(d, e), w_gate=n(e, d, f), w_up=n(e, d, f), w_down=n(e, f, d), ws_gate=n(d, fs), ws_up=n(d, fs),
              ws_down=n(fs, d), w_sg=n(d))


def test_maxtext_tree_round_trip():
  w = small_layer(np.random.default_rng(0))
  del w["w_sg"]
  tree = W.to_maxtext(w)
  assert tree["mlp"]["routed_experts"]["gate"]["kernel"].shape == (8, 6)        # experts on the last axis
  assert tree["mlp"]["routed_experts"]["wi_0"].shape == (6, 8, 4) and tree["mlp"]["routed_experts"]["wo"].shape == (6, 4, 8)
  back = W.from_maxtext(tree)
  assert set(back) == set(w) and all(back[k] is w[k] for k in w)                 # no copy, no transposition
  del tree["mlp"]["shared_expert"]
  assert "ws_gate" not in W.from_maxtext(tree)
  with pytest.raises(KeyError):
    W.from_maxtext({"mlp": {}})


@pytest.mark.parametrize("as_torch", [False, True])
def test_hf_round_trip_and_orientation(as_torch):
  w = small_layer(np.random.default_rng(1))
  if as_torch:
    w = {k: torch.from_numpy(v) for k, v in w.items()}
  sd = W.to_hf(w, prefix="model.layers.0.")
  assert tuple(sd["model.layers.0.mlp.gate.weight"].shape) == (6, 8)
  assert tuple(sd["model.layers.0.mlp.experts.gate_up_proj"].shape) == (6, 8, 8)      # [E, 2I, H]
  assert tuple(sd["model.layers.0.mlp.experts.down_proj"].shape) == (6, 8, 4)         # [E, H, I]
  assert tuple(sd["model.layers.0.mlp.shared_expert_gate.weight"].shape) == (1, 8)
  # rows 0..I-1 of gate_up_proj are the gate projection (tools/grow_7b.py:104)
  a = np.asarray(sd["model.layers.0.mlp.experts.gate_up_proj"])
  assert np.array_equal(a[:, :4, :], np.swapaxes(np.asarray(w["w_gate"]), 1, 2))
  back = W.from_hf(sd, prefix="model.layers.0.")
  for k in w:
    assert np.array_equal(np.asarray(back[k]), np.asarray(w[k])), k


def test_layouts_compute_the_same_layer():
  """The oracle's layer on MoEWeights-layout arrays equals the Hugging Face formulas on to_hf's tensors."""
  import oracle as O
  w = small_layer(np.random.default_rng(2), e=4)
  x = np.random.default_rng(3).standard_normal((5, 8)).astype(np.float32)
  out, c = O.moe_layer_fwd(x, w["w_router"], w["w_gate"], w["w_up"], w["w_down"], w["ws_gate"], w["ws_up"], w["ws_down"], 2,
                           shared_gate=w["w_sg"])
  sd = W.to_hf(w)
  probs = O.softmax(x @ sd["mlp.gate.weight"].T)
  want = np.zeros_like(x)
  for t in range(5):
    for j in range(2):
      e = c["idx"][t, j]
      gu = sd["mlp.experts.gate_up_proj"][e] @ x[t]
      h = O.silu(gu[:4]) * gu[4:]
      want[t] += c["w"][t, j] * (sd["mlp.experts.down_proj"][e] @ h)
    hs = O.silu(sd["mlp.shared_expert.gate_proj.weight"] @ x[t]) * (sd["mlp.shared_expert.up_proj.weight"] @ x[t])
    gate = 1 / (1 + np.exp(-(sd["mlp.shared_expert_gate.weight"][0] @ x[t])))
    want[t] += gate * (sd["mlp.shared_expert.down_proj.weight"] @ hs)
  assert np.allclose(probs.argsort(1)[:, -2:][:, ::-1], c["idx"])
  assert O.rel_err(out, want) <= 1e-5


def test_grow_experts_equals_the_reference_grow_tree():
  """Expert doubling with noise: bit-identical to `grow_tree` (modal/stage2.py:318-348) on its scanned layout.  The
  layer-cycle duplication grow_tree does first is not part of the MoE layer; it is redone here with plain indexing."""
  import ml_dtypes
  bf = ml_dtypes.bfloat16
  def dup_cycle(a, zero_new=False, cyc=1):
    a = a.astype(bf)
    new = a.take([cyc], axis=1).copy()
    if zero_new:
      new[:] = 0
    return np.concatenate([a.take(range(cyc + 1), axis=1), new, a.take(range(cyc + 1, a.shape[1]), axis=1)], axis=1)
  w = dict(w_router=dup_cycle(Z["gt_in_gate"]), w_gate=dup_cycle(Z["gt_in_wi_0"]), w_up=dup_cycle(Z["gt_in_wi_1"]),
           w_down=dup_cycle(Z["gt_in_wo"], zero_new=True))
  g = W.grow_experts(w, expert_mult=2, noise=1e-3, seed=5)
  for mine, ref in (("w_router", "gt_out_gate"), ("w_gate", "gt_out_wi_0"), ("w_up", "gt_out_wi_1"), ("w_down", "gt_out_wo")):
    assert np.array_equal(np.asarray(g[mine], np.float32), Z[ref]), mine
  e = Z["gt_in_wi_0"].shape[0]
  assert g["w_gate"].shape[0] == 2 * e and g["w_router"].shape[-1] == 2 * e
  # twins: expert e + E is expert e plus noise of relative size 1e-3
  a = np.asarray(g["w_gate"], np.float32)
  assert 0 < np.abs(a[e:] - a[:e]).max() < 0.05 * np.abs(a).max()


@pytest.mark.parametrize("pairs", ["adjacent", "usage"])
def test_merge_expert_pairs_equals_the_reference_merge(pairs):
  """Pair-merge to E/2 experts of width 2I: through from_hf / to_hf it reproduces `merge_experts`
  (tools/grow_7b.py:84-112) exactly, for adjacent pairs and for usage-ranked pairs."""
  sd = {"mlp.gate.weight": Z[f"me_{pairs}_gate_in"], "mlp.experts.gate_up_proj": Z[f"me_{pairs}_gate_up_in"],
        "mlp.experts.down_proj": Z[f"me_{pairs}_down_in"]}
  usage = Z["me_usage_counts"] if pairs == "usage" else None
  merged = W.to_hf(W.merge_expert_pairs(W.from_hf(sd), usage=usage, eps=0.5))
  assert np.array_equal(merged["mlp.experts.gate_up_proj"], Z[f"me_{pairs}_gate_up"])
  assert np.array_equal(merged["mlp.experts.down_proj"], Z[f"me_{pairs}_down"])
  assert np.array_equal(merged["mlp.gate.weight"], Z[f"me_{pairs}_gate"])
  with pytest.raises(ValueError):
    W.merge_expert_pairs(dict(w_router=np.zeros((4, 3)), w_gate=np.zeros((3, 4, 2)), w_up=np.zeros((3, 4, 2)), w_down=np.zeros((3, 2, 4))))
