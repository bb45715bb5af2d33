"""The CPU oracle against independent statements of the same math (no GPU).

* index ops against the reference's own checks (modal/test_moe_permute.py:50-91): both sort methods
  agree exactly, pos is the inverse of order, the custom backward passes equal autograd of the
  reference formulas;
* dropless ragged_dot on the known-answer shapes of modal/te_run.py:68-80 (empty group, tail rows);
* the capacity layout of modal/padded_gmm.py equals the dropless result when nothing overflows and
  zeroes overflowing rows;
* the analytic whole-layer backward against torch autograd of the same forward;
* router / SwiGLU / shared expert against the Hugging Face qwen3_5_moe block (second opinion).
"""
import numpy as np
import pytest
import torch

import oracle as O
from util import rand_routing, softmax_np

E = 16


@pytest.mark.parametrize("k", [6, 12])
@pytest.mark.parametrize("n", [64, 60, 2048 * 2 // 6 * 6 // 6])
def test_sort_methods_agree_and_invert(k, n):
  rng = np.random.default_rng(k * 7 + n)
  flat = rand_routing(rng, n, E, k).reshape(-1)
  o1, p1 = O.sort_indices(flat, E, "argsort")
  o2, p2 = O.sort_indices(flat, E, "count")
  assert np.array_equal(o1, o2) and np.array_equal(p1, p2)
  assert np.array_equal(o1[p1], np.arange(flat.size))
  s = flat[o1]
  assert np.all(np.diff(s) >= 0)
  same = np.diff(s) == 0
  assert np.all(np.diff(o1)[same] > 0)  # stable: slot order kept inside an expert


def test_count_sort_chunked_path():
  rng = np.random.default_rng(3)
  flat = rng.integers(0, E, size=4096).astype(np.int32)  # multiple of 2048 -> two chunks with carry
  o1, p1 = O.sort_indices(flat, E, "argsort")
  o2, p2 = O.sort_indices(flat, E, "count")
  assert np.array_equal(o1, o2) and np.array_equal(p1, p2)


def test_block_layout_invariants():
  rng = np.random.default_rng(0)
  flat = rng.integers(0, 8, size=1000).astype(np.int32)
  flat[flat == 3] = 4  # expert 3 is empty
  L = O.block_layout(flat, 8, 128)
  assert L["counts"][3] == 0 and L["pad_offsets"][3] == L["pad_offsets"][4]
  assert np.all(L["pad_offsets"] % 128 == 0)
  assert L["mpad"] == (1000 + 8 * 127) // 128 * 128
  live = L["block_expert"][: L["n_blocks"]]
  assert np.all(live >= 0) and np.all(np.diff(live) >= 0) and np.all(L["block_expert"][L["n_blocks"]:] == -1)
  # slot <-> padded row is a bijection on valid entries; padded order keeps the sorted order
  assert np.array_equal(L["row_slot"][L["pad_pos"]], np.arange(1000))
  assert (L["row_slot"] >= 0).sum() == 1000
  valid_rows = np.nonzero(L["row_slot"] >= 0)[0]
  assert np.array_equal(L["row_slot"][valid_rows], L["order"])
  for r in valid_rows[:50]:
    assert L["block_expert"][r // 128] == flat[L["row_slot"][r]]


@pytest.mark.parametrize("k", [6, 12])
def test_dispatch_combine_backward_match_autograd(k):
  n, d = 64, 32
  rng = np.random.default_rng(k)
  x = rng.standard_normal((n, d)).astype(np.float32)
  flat = rand_routing(rng, n, E, k).reshape(-1)
  w = softmax_np(rng.standard_normal((n, k)).astype(np.float32))
  g = rng.standard_normal((n, d)).astype(np.float32)
  order, pos = O.sort_indices(flat, E)
  # forward through the oracle's ops equals the reference branch
  y = np.tanh(O.dispatch(x, order, pos))
  out = O.combine(y, order, pos, w)
  ref = O.moe_block(x, flat, w, np.tanh)
  assert O.rel_err(out, ref) <= 1e-6
  # autograd of the reference formulas
  xt = torch.tensor(x, requires_grad=True)
  wt = torch.tensor(w, requires_grad=True)
  ot = torch.as_tensor(np.argsort(flat, kind="stable"))
  pt = torch.as_tensor(np.argsort(np.argsort(flat, kind="stable"), kind="stable"))
  yt = torch.tanh(xt[ot // k])
  outt = torch.einsum("nkd,nk->nd", yt[pt].reshape(n, k, d), wt)
  (outt * torch.tensor(g)).sum().backward()
  dy, dw = O.combine_bwd(g, y, order, pos, w)
  dx = O.dispatch_bwd(dy * (1 - y * y), order, pos, n)
  assert O.rel_err(dx, xt.grad.numpy()) <= 1e-5
  assert O.rel_err(dw, wt.grad.numpy()) <= 1e-5
  # permute_rows gradient (modal/test_moe_permute.py:84-87)
  perm = rng.permutation(n * k).astype(np.int32)
  gy = rng.standard_normal((n * k, d)).astype(np.float32)
  ytt = torch.tensor(y, requires_grad=True)
  (ytt[torch.as_tensor(perm).long()] * torch.tensor(gy)).sum().backward()
  assert O.rel_err(O.permute_rows_bwd(gy, perm), ytt.grad.numpy()) <= 1e-6


def te_case():
  """Shapes of the reference's known-answer check (modal/te_run.py:72-73)."""
  gs = np.array([5, 0, 9, 3, 7, 1, 6, 4], np.int32)
  s = int(gs.sum())
  m = s + 3
  rng = np.random.default_rng(0)
  a = O.bf16_round(rng.standard_normal((m, 64)).astype(np.float32))
  b = O.bf16_round(rng.standard_normal((8, 64, 48)).astype(np.float32))
  return gs, s, m, a, b


def test_ragged_dot_known_answer_shapes():
  gs, s, m, a, b = te_case()
  out = O.ragged_dot(a, b, gs)
  assert np.all(out[s:] == 0)
  at = torch.tensor(a, requires_grad=True)
  bt = torch.tensor(b, requires_grad=True)
  rows = torch.repeat_interleave(torch.arange(8), torch.as_tensor(gs).long())
  ref = torch.einsum("mk,mkn->mn", at[:s], bt[rows])
  assert O.rel_err(out[:s], ref.detach().numpy()) <= 1e-5
  (ref ** 2).sum().backward()
  dl, dr = O.ragged_dot_bwd(np.concatenate([2 * out[:s], np.zeros((3, 48), np.float32)]), a, b, gs)
  assert O.rel_err(dl[:s], at.grad.numpy()[:s]) <= 1e-5 and np.all(dl[s:] == 0)
  assert O.rel_err(dr, bt.grad.numpy()) <= 1e-5
  assert np.all(dr[1] == 0)  # the empty group's weight gradient is exactly zero


def test_capacity_layout_matches_dropless_without_overflow_and_drops_with():
  gs, s, m, a, b = te_case()
  full = O.ragged_dot(a, b, gs)
  # factor 2: C = max(8, ceil8(ceil(38/8*2))) = 16 >= max group (9): nothing dropped
  assert O.rel_err(O.padded_ragged_dot(a, b, gs, factor=2.0), full) <= 1e-6
  # factor 1: C = 8 < 9: the 9th row of group 2 is dropped -> zeros
  out = O.padded_ragged_dot(a, b, gs, factor=1.0)
  dropped = 5 + 0 + 8
  assert np.all(out[dropped] == 0)
  keep = np.ones(m, bool)
  keep[dropped] = False
  assert O.rel_err(out[keep], full[keep]) <= 1e-6


def small_layer(seed=0, t=96, d=64, e=8, f=64, fs=64, k=3):
  inp = O.make_inputs(t, d, e, f, fs, seed)
  # larger router weights so that routing is not near-uniform
  inp["w_router"] = inp["w_router"] * 20
  return inp, k


def torch_layer(inp, k, idx):
  """Independent torch statement of the forward with the routing decision fixed to idx."""
  T = {n: torch.tensor(v, dtype=torch.float64, requires_grad=True) for n, v in inp.items() if n != "dout"}
  x = T["x"]
  p = torch.softmax(x @ T["w_router"], dim=-1)
  it = torch.as_tensor(idx).long()
  v = torch.gather(p, 1, it)
  w = v / v.sum(-1, keepdim=True)
  out = torch.zeros_like(x)
  for j in range(k):
    e = it[:, j]
    g = torch.einsum("td,tdf->tf", x, T["w_gate"][e])
    u = torch.einsum("td,tdf->tf", x, T["w_up"][e])
    y = torch.einsum("tf,tfd->td", torch.nn.functional.silu(g) * u, T["w_down"][e])
    out = out + w[:, j:j + 1] * y
  sh = (torch.nn.functional.silu(x @ T["ws_gate"]) * (x @ T["ws_up"])) @ T["ws_down"]
  return out + sh, T


def test_layer_forward_and_analytic_backward_match_autograd():
  inp, k = small_layer()
  args = [inp[n] for n in ("x", "w_router", "w_gate", "w_up", "w_down", "ws_gate", "ws_up", "ws_down")]
  out, cache = O.moe_layer_fwd(*args, k)
  ref, T = torch_layer(inp, k, cache["idx"])
  assert O.rel_err(out, ref.detach().numpy()) <= 1e-5
  (ref * torch.tensor(inp["dout"], dtype=torch.float64)).sum().backward()
  g = O.moe_layer_bwd(inp["dout"], *args, k, cache)
  names = dict(dx="x", dw_router="w_router", dw_gate="w_gate", dw_up="w_up", dw_down="w_down",
               dws_gate="ws_gate", dws_up="ws_up", dws_down="ws_down")
  for gn, pn in names.items():
    assert O.rel_err(g[gn], T[pn].grad.numpy()) <= 2e-5, gn


def test_router_selection_rule_and_weights():
  rng = np.random.default_rng(1)
  logits = rng.standard_normal((512, 64)).astype(np.float32)
  logits[0, 5] = logits[0, 9] = logits[0].max() + 1.0  # exact tie -> lower index first
  idx, w, p = O.router_topk(logits, 6)
  assert idx[0, 0] == 5 and idx[0, 1] == 9
  # selection == ordering by (logit desc, index asc)
  key = np.argsort(-logits.astype(np.float64), axis=1, kind="stable")[:, :6]
  assert np.array_equal(idx, key.astype(np.int32))
  assert np.allclose(w.sum(1), 1.0, atol=1e-6)
  tv, ti = torch.topk(torch.softmax(torch.tensor(logits), -1), 6)
  clear = np.ones(512, bool)
  clear[0] = False
  assert np.array_equal(idx[clear], ti.numpy()[clear])
  assert O.rel_err(w[clear], (tv / tv.sum(-1, keepdim=True)).numpy()[clear]) <= 1e-6


def test_router_backward_matches_autograd():
  rng = np.random.default_rng(2)
  logits = rng.standard_normal((128, 32)).astype(np.float32)
  idx, w, p = O.router_topk(logits, 4)
  dw = rng.standard_normal((128, 4)).astype(np.float32)
  lt = torch.tensor(logits, dtype=torch.float64, requires_grad=True)
  v = torch.gather(torch.softmax(lt, -1), 1, torch.as_tensor(idx).long())
  ((v / v.sum(-1, keepdim=True)) * torch.tensor(dw, dtype=torch.float64)).sum().backward()
  assert O.rel_err(O.router_topk_bwd(logits, idx, dw), lt.grad.numpy()) <= 1e-5


def test_against_huggingface_qwen3_5_moe_block():
  """Second opinion on router, SwiGLU experts and shared expert: the HF twin of the MaxText block.

  The HF block multiplies the shared expert by sigmoid(x . w_sg); the oracle's optional
  ``shared_gate`` reproduces that, and a zero gate weight gives sigmoid(0) = 0.5 exactly.
  """
  mod = pytest.importorskip("transformers.models.qwen3_5_moe.modeling_qwen3_5_moe")
  cfg_mod = pytest.importorskip("transformers.models.qwen3_5_moe.configuration_qwen3_5_moe")
  t, d, e, f, fs, k = 64, 32, 8, 16, 16, 3
  try:
    cfg = cfg_mod.Qwen3_5MoeTextConfig(hidden_size=d, num_experts=e, num_experts_per_tok=k, moe_intermediate_size=f,
                                       shared_expert_intermediate_size=fs, norm_topk_prob=True)
    blk = mod.Qwen3_5MoeSparseMoeBlock(cfg).float().eval()
  except Exception as ex:  # constructor signature differs between transformers versions
    pytest.skip(f"cannot build the HF block in this transformers version: {ex!r}")
  inp = O.make_inputs(t, d, e, f, fs, seed=4)
  inp["w_router"] = inp["w_router"] * 30
  sd = blk.state_dict()
  want = {
      "gate.weight": inp["w_router"].T,                                       # [E,H]   (tools/grow_7b.py:110)
      "experts.gate_up_proj": np.concatenate([inp["w_gate"].transpose(0, 2, 1), inp["w_up"].transpose(0, 2, 1)], 1),
      "experts.down_proj": inp["w_down"].transpose(0, 2, 1),                  # [E,H,I] (tools/grow_7b.py:104-109)
      "shared_expert.gate_proj.weight": inp["ws_gate"].T,
      "shared_expert.up_proj.weight": inp["ws_up"].T,
      "shared_expert.down_proj.weight": inp["ws_down"].T,
  }
  rng = np.random.default_rng(9)
  sgate = (rng.standard_normal(d) * 0.5).astype(np.float32)
  want["shared_expert_gate.weight"] = sgate[None, :]
  for name, val in want.items():
    if name not in sd or tuple(sd[name].shape) != tuple(val.shape):
      pytest.skip(f"HF parameter {name} missing or shaped {tuple(sd.get(name, torch.empty(0)).shape)} != {val.shape}")
    sd[name] = torch.tensor(np.ascontiguousarray(val))
  blk.load_state_dict(sd)
  with torch.no_grad():
    res = blk(torch.tensor(inp["x"])[None])
  hf = (res[0] if isinstance(res, tuple) else res).reshape(t, d).numpy()
  args = [inp[n] for n in ("x", "w_router", "w_gate", "w_up", "w_down", "ws_gate", "ws_up", "ws_down")]
  out, _ = O.moe_layer_fwd(*args, k, shared_gate=sgate)
  assert O.rel_err(out, hf) <= 1e-4


def test_aux_loss_uniform_is_one():
  e, t, k = 8, 64, 2
  probs = np.full((t, e), 1.0 / e, np.float32)
  idx = (np.arange(t * k) % e).reshape(t, k).astype(np.int32)
  assert abs(O.aux_loss(probs, idx, e) - 1.0) < 1e-6


def test_aux_loss_backward_matches_autograd():
  """aux = E * sum_e f_e * mean_t softmax(logits)[t,e] with the token fractions f_e held constant."""
  rng = np.random.default_rng(3)
  t, e, k = 96, 16, 3
  logits = rng.standard_normal((t, e)).astype(np.float32)
  idx, w, p = O.router_topk(logits, k)
  lt = torch.tensor(logits, dtype=torch.float64, requires_grad=True)
  f = torch.tensor(np.bincount(idx.reshape(-1), minlength=e) / float(t * k))
  loss = e * (f * torch.softmax(lt, -1).mean(0)).sum()
  assert abs(float(loss) - O.aux_loss(p, idx, e)) <= 1e-6
  loss.backward()
  assert O.rel_err(O.aux_loss_bwd(p, idx, e), lt.grad.numpy()) <= 1e-5


def test_layer_backward_with_gate_bias_and_aux_matches_autograd():
  """The optional terms of the whole-layer backward (sigmoid gate on the shared expert, router bias, load-balance
  loss) against torch autograd of the same forward."""
  inp, k = small_layer()
  names = ("x", "w_router", "w_gate", "w_up", "w_down", "ws_gate", "ws_up", "ws_down")
  args = [inp[n] for n in names]
  rng = np.random.default_rng(11)
  t, d = inp["x"].shape
  e = inp["w_gate"].shape[0]
  bias = (rng.standard_normal(e) * 0.3).astype(np.float32)
  sgate = (rng.standard_normal(d) * 0.2).astype(np.float32)
  aux_w = 0.3
  out, cache = O.moe_layer_fwd(*args, k, router_bias=bias, shared_gate=sgate)
  g = O.moe_layer_bwd(inp["dout"], *args, k, cache, shared_gate=sgate, aux_weight=aux_w)
  T = {n: torch.tensor(inp[n], dtype=torch.float64, requires_grad=True) for n in names}
  tb = torch.tensor(bias, dtype=torch.float64, requires_grad=True)
  tg = torch.tensor(sgate, dtype=torch.float64, requires_grad=True)
  x = T["x"]
  probs = torch.softmax(x @ T["w_router"] + tb, -1)
  idx = torch.as_tensor(cache["idx"]).long()
  v = torch.gather(probs, 1, idx)
  wts = v / v.sum(-1, keepdim=True)
  routed = torch.zeros_like(x)
  for j in range(k):
    ex = idx[:, j]
    h = torch.nn.functional.silu(torch.einsum("td,tdf->tf", x, T["w_gate"][ex])) * torch.einsum("td,tdf->tf", x, T["w_up"][ex])
    routed = routed + wts[:, j:j + 1] * torch.einsum("tf,tfd->td", h, T["w_down"][ex])
  sh = (torch.nn.functional.silu(x @ T["ws_gate"]) * (x @ T["ws_up"])) @ T["ws_down"]
  ref = routed + torch.sigmoid(x @ tg)[:, None] * sh
  assert O.rel_err(out, ref.detach().numpy()) <= 1e-5
  f = torch.tensor(np.bincount(cache["idx"].reshape(-1), minlength=e) / float(t * k))
  total = (ref * torch.tensor(inp["dout"], dtype=torch.float64)).sum() + aux_w * e * (f * probs.mean(0)).sum()
  total.backward()
  pairs = dict(dx="x", dw_router="w_router", dw_gate="w_gate", dw_up="w_up", dw_down="w_down", dws_gate="ws_gate",
               dws_up="ws_up", dws_down="ws_down")
  for gn, pn in pairs.items():
    assert O.rel_err(g[gn], T[pn].grad.numpy()) <= 2e-5, gn
  assert O.rel_err(g["drouter_bias"], tb.grad.numpy()) <= 2e-5
  assert O.rel_err(g["dshared_gate"], tg.grad.numpy()) <= 2e-5


def test_bf16_round():
  a = np.array([1.0, 1.00390625, 1.005859375, -3.14159, 1e-30, 65504.0], np.float32)
  got = O.bf16_round(a)
  want = torch.tensor(a).to(torch.bfloat16).float().numpy()
  assert np.array_equal(got, want)
