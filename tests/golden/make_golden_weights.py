"""Generates tests/golden/weight_growth.npz by RUNNING the reference's own weight-surgery functions.

  python tests/golden/make_golden_weights.py /path/to/reference

`grow_tree` (modal/stage2.py:318-348) and `merge_experts` / `pairing` (tools/grow_7b.py:84-112) sit in scripts whose
module level needs packages and files that do not exist here, so only those function definitions (and the constants
they read) are taken out of the parsed source with `ast` and executed; nothing is copied into this repository.
Inputs are small seeded arrays in the layouts the functions expect.
"""
import ast
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def functions_from(path, names):
  """Compiles the named top-level functions / assignments of a source file into a fresh namespace."""
  tree = ast.parse(open(path).read())
  keep = [n for n in tree.body
          if (isinstance(n, ast.FunctionDef) and n.name in names)
          or (isinstance(n, ast.Assign) and any(isinstance(t, ast.Name) and t.id in names for t in n.targets))]
  ns = {"np": np}
  exec(compile(ast.Module(body=keep, type_ignores=[]), path, "exec"), ns)
  return ns


def main(ref_root):
  rng = np.random.default_rng(31)
  # ---- grow_tree: scanned MaxText layout, axis 1 = layer cycle; experts on axis 0 (router: last axis)
  ns = functions_from(os.path.join(ref_root, "modal", "stage2.py"), {"grow_tree", "ZERO_OUT"})
  e, cyc, d, f = 4, 3, 8, 6
  n = lambda *s: rng.standard_normal(s).astype(np.float32)
  routed = {"gate": {"kernel": n(d, cyc, e)}, "wi_0": n(e, cyc, d, f), "wi_1": n(e, cyc, d, f), "wo": n(e, cyc, f, d)}
  tree = {"decoder": {"layers": {"mlp": {"routed_experts": routed}}}}
  grown = ns["grow_tree"](tree, dup_cycle=1, expert_mult=2, noise=1e-3, seed=5)
  g = grown["decoder"]["layers"]["mlp"]["routed_experts"]
  out = {"gt_in_gate": routed["gate"]["kernel"], "gt_in_wi_0": routed["wi_0"], "gt_in_wi_1": routed["wi_1"],
         "gt_in_wo": routed["wo"],
         "gt_out_gate": np.asarray(g["gate"]["kernel"], np.float32), "gt_out_wi_0": np.asarray(g["wi_0"], np.float32),
         "gt_out_wi_1": np.asarray(g["wi_1"], np.float32), "gt_out_wo": np.asarray(g["wo"], np.float32)}
  # ---- merge_experts: Hugging Face layout of one layer
  E, I, H = 6, 4, 5
  for pairs in ("adjacent", "usage"):
    usage = {"0": rng.permutation(E).astype(np.float64).tolist()} if pairs == "usage" else None
    ns2 = functions_from(os.path.join(ref_root, "tools", "grow_7b.py"), {"merge_experts", "pairing"})
    ns2.update(E=E, I=I, EPS=0.5, USAGE=usage)
    gu, dn, gate = n(E, 2 * I, H), n(E, H, I), n(E, H)
    out.update({f"me_{pairs}_gate_up_in": gu, f"me_{pairs}_down_in": dn, f"me_{pairs}_gate_in": gate,
                f"me_{pairs}_gate_up": ns2["merge_experts"]("x.mlp.experts.gate_up_proj", gu, 0),
                f"me_{pairs}_down": ns2["merge_experts"]("x.mlp.experts.down_proj", dn, 0),
                f"me_{pairs}_gate": ns2["merge_experts"]("x.mlp.gate.weight", gate, 0)})
    if usage is not None:
      out["me_usage_counts"] = np.asarray(usage["0"])
  np.savez_compressed(os.path.join(HERE, "weight_growth.npz"), **out)
  print("wrote weight_growth.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
  if len(sys.argv) != 2:
    raise SystemExit("usage: python tests/golden/make_golden_weights.py <path to a checkout of the reference repository>")
  main(sys.argv[1])
