"""bench.py without a GPU: the reference arm's JSON line, the rank that stays silent, and the work table."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _run(extra_env=None, *flags):
  env = dict(os.environ)
  env.update(extra_env or {})
  return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--config", "config1",
                         "--tokens", "256", "--steps", "1", "--warmup", "0", *flags],
                        capture_output=True, text=True, env=env, timeout=300)


def test_reference_arm_line():
  res = _run()
  assert res.returncode == 0, res.stderr
  lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
  assert len(lines) == 1
  j = json.loads(lines[0])
  assert j["impl"] == "reference" and j["unit"] == "tokens/s" and j["higher_is_better"] is True
  assert j["metric"] == "moe_layer_fwd_bwd_tokens_per_s" and j["value"] > 0 and j["vs_baseline"] is None
  assert j["cpu_baseline"]["kind"] == "port" and j["cpu_baseline"]["value"] == j["value"] and j["cpu_baseline"]["cores"] >= 1
  assert j["e2e"] == {"value": j["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
  assert "workload" in j["config"] and "model" not in j["config"]


def test_reference_arm_other_ranks_stay_silent():
  res = _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}, "--gpus", "2")
  assert res.returncode == 0 and res.stdout.strip() == ""


def test_own_arm_needs_a_gpu():
  import torch
  if torch.cuda.is_available():
    pytest.skip("a GPU is present")
  res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1"], capture_output=True, text=True,
                       timeout=300)
  assert res.returncode != 0 and "CUDA" in (res.stderr + res.stdout)   # no CPU path for the kernels


def test_work_table_adds_up_to_the_layer():
  import bench
  c = dict(bench.CONFIGS["config2"])
  work = bench.kernel_work(c)
  single = ("router_logits", "gemm_gateup_swiglu", "gemm_down", "shared_gateup_swiglu", "shared_down", "gemm_dh_dswiglu",
            "gemm_dw_down", "gemm_dx", "gemm_dw_gateup", "shared_dh_dswiglu", "shared_dw_down", "shared_dx",
            "shared_dw_gateup", "router_dx", "router_dw")
  flops = sum(work[n][1] for n in single if work[n][0] == "tensor")
  assert abs(flops - bench.layer_flops(c)) / bench.layer_flops(c) < 0.02
  assert all(work[n][0] == "nvlink" and work[n][1] == 0 for n in ("ep_push_x", "ep_return_dx"))   # one GPU: nothing leaves
  w8 = bench.kernel_work(c, world=8)
  assert w8["ep_push_x"][1] == c["T"] * c["k"] * 2 * c["d"] * 7 / 8


def test_exchange_flags_map_to_layer_arguments():
  import argparse
  import bench
  ns = lambda **kw: argparse.Namespace(ep_push=None, ep_return=None, ep_range_weights=None, ep_return_sms=None, **kw)
  assert bench.ep_exchange_mode(ns()) == {}
  a = ns()
  a.ep_push, a.ep_return = "unique", "combined"
  assert bench.ep_exchange_mode(a) == {"unique_push": True, "fused_return": False, "combined_return": True}
  a.ep_push, a.ep_return = "slots", "kernel"
  assert bench.ep_exchange_mode(a) == {"unique_push": False, "fused_return": False, "combined_return": False}
  a.ep_range_weights = "1,3,3,1"
  assert bench.ep_range_weights(a) == [1.0, 3.0, 3.0, 1.0] and bench.ep_range_weights(ns()) is None


def test_exchange_summary_counts_rows_both_ways():
  import types
  import torch
  from lewi_surge_b200 import ep
  me = types.SimpleNamespace(el=4, rank=1, world=4, d=8, unique_push=True, combined_return=False, fused_return=True,
                             phases=2)
  idx = torch.tensor([[0, 1, 5, 6], [4, 5, 6, 7], [12, 13, 0, 8]])
  got = ep.ExpertParallelP2P.exchange_summary(me, idx)
  # token 0: experts 0,1 on rank 0 (one row once per rank, two per slot); token 1 stays home; token 2: ranks 3,3,0,2
  assert got["rows_sent_per_slot"] == 6 and got["rows_sent_once_per_rank"] == 4
  assert got["push_bytes_per_pass"] == 4 * 16 and got["return_bytes_per_pass"] == 6 * 16
  assert (got["push"], got["back"]) == ("unique", "fused")
