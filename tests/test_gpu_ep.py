"""Expert-parallel layer on real GPUs, one process per GPU: the NCCL all-to-all version and the peer-memory version
(one exchange per pass, pipelined over ranges of experts, with either way of ordering the ranks), against the
single-GPU layer on the concatenated batch (which the other tests pin to the oracle).  World size 1 runs on one
GPU; the rest needs at least 2."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
NAMES = ("x", "w_router", "w_gate", "w_up", "w_down", "ws_gate", "ws_up", "ws_down")


def _free_port():
  s = socket.socket()
  s.bind(("127.0.0.1", 0))
  p = s.getsockname()[1]
  s.close()
  return p


def _worker(rank, world, port, cfg, out_dir, impl="nccl"):
  sys.path.insert(0, HERE)
  sys.path.insert(0, os.path.dirname(HERE))
  os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
  import torch.distributed as dist
  torch.cuda.set_device(rank)
  dev = torch.device("cuda", rank)
  dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
  try:
    import oracle as O
    from lewi_surge_b200 import ep, _lib
    from lewi_surge_b200.layer import MoEWeights
    t, d, e, f, fs, k = cfg
    inp = O.make_inputs(t * world, d, e, f, fs, seed=5)
    inp["w_router"] = inp["w_router"] * 5
    el = e // world
    tt = lambda a, dt=torch.bfloat16: torch.from_numpy(np.ascontiguousarray(a)).to(dev, dt)
    w = MoEWeights(tt(inp["w_router"], torch.float32), tt(inp["w_gate"][rank * el:(rank + 1) * el]),
                   tt(inp["w_up"][rank * el:(rank + 1) * el]), tt(inp["w_down"][rank * el:(rank + 1) * el]),
                   tt(inp["ws_gate"]), tt(inp["ws_up"]), tt(inp["ws_down"]))
    if impl.startswith("p2p"):
      # "p2p": one exchange per pass; "p2p-phased": pipelined over ranges of local experts; "p2p-nccl": ranks
      # ordered by a one-element all-reduce instead of the flag barrier
      # "p2p-ranges": uneven ranges, the weight gradients range by range and the way back as a kernel of its own; the
      # others compute the weight gradients once at the end and send rows back from the GEMM epilogues
      # "p2p-unique": a token travels once per destination rank and one partial row per token comes back;
      # "p2p-unique-slots": once per rank on the way out, per slot from the GEMM epilogues on the way back
      # "p2p-split": the GEMMs that send rows home run on 48 SMs beside the next range's first GEMM
      phases = {"p2p": 1, "p2p-phased": 4, "p2p-nccl": 2, "p2p-ranges": 3, "p2p-unique": 4, "p2p-unique-slots": 2,
                "p2p-split": 4}[impl]
      lay = ep.ExpertParallelP2P(w, k, e, t, d, phases=phases, sync="nccl" if impl == "p2p-nccl" else "flags",
                                 range_weights=[1, 2, 1] if impl == "p2p-ranges" else None,
                                 dw_deferred=impl != "p2p-ranges", fused_return=impl != "p2p-ranges",
                                 unique_push=impl.startswith("p2p-unique"),
                                 combined_return=impl == "p2p-unique", return_sms=48 if impl == "p2p-split" else 0,
                                 router_tail=impl == "p2p-nccl")   # (one variant keeps the router backward on the exchange stream)
    else:
      lay = ep.ExpertParallelLayer(w, k, e)
    sl = slice(rank * t, (rank + 1) * t)
    xr, gr = tt(inp["x"][sl]), tt(inp["dout"][sl])
    out, grads = lay.step(xr, gr)
    if impl.startswith("p2p"):     # a second step over the same buffers must give the same answer
      out2, grads2 = lay.step(xr, gr)
      assert torch.equal(out, out2) and torch.equal(grads["dx"], grads2["dx"])
    assert _lib.last_status() == 0
    if impl.startswith("p2p"):
      assert not lay.overflowed()
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), out=out.float().cpu().numpy(),
             **{n: g.float().cpu().numpy() for n, g in grads.items()})
    dist.barrier()
  finally:
    dist.destroy_process_group()


@pytest.mark.parametrize("impl", ["p2p", "p2p-phased", "p2p-ranges", "p2p-unique", "p2p-unique-slots", "p2p-split"])
def test_peer_memory_layer_on_one_gpu(cuda, tmp_path, impl):
  """World size 1: the push / return kernels, the plan and the barrier run against this GPU's own buffers."""
  _check(cuda, tmp_path, (512, 256, 16, 128, 128, 4), 1, impl)


@pytest.mark.parametrize("impl", ["nccl", "p2p", "p2p-phased", "p2p-nccl", "p2p-ranges", "p2p-unique", "p2p-unique-slots", "p2p-split"])
@pytest.mark.parametrize("cfg", [(512, 256, 16, 128, 128, 4), (1024, 1024, 64, 512, 512, 6)])
def test_expert_parallel_matches_single_gpu(cuda, tmp_path, cfg, impl):
  world = min(torch.cuda.device_count(), 4)
  if world < 2:
    pytest.skip("needs at least 2 GPUs")
  _check(cuda, tmp_path, cfg, world, impl)


def _check(cuda, tmp_path, cfg, world, impl):
  import torch.multiprocessing as mp
  import oracle as O
  from lewi_surge_b200 import layer
  mp.spawn(_worker, args=(world, _free_port(), cfg, str(tmp_path), impl), nprocs=world, join=True)
  t, d, e, f, fs, k = cfg
  inp = O.make_inputs(t * world, d, e, f, fs, seed=5)
  inp["w_router"] = inp["w_router"] * 5
  tt = lambda a, dt=torch.bfloat16: torch.from_numpy(np.ascontiguousarray(a)).to(cuda, dt)
  w = layer.MoEWeights(tt(inp["w_router"], torch.float32), *(tt(inp[n]) for n in NAMES[2:]))
  out, cache = layer.moe_layer_fwd(tt(inp["x"]), w, k)
  g = layer.moe_layer_bwd(tt(inp["dout"]), w, cache)
  res = [np.load(tmp_path / f"r{r}.npz") for r in range(world)]
  el = e // world
  f32 = lambda v: v.float().cpu().numpy()
  # same kernels, same routing; only summation orders of the combine differ -> tight tolerance
  assert O.rel_err(np.concatenate([r["out"] for r in res]), f32(out)) <= 1e-2
  assert O.rel_err(np.concatenate([r["dx"] for r in res]), f32(g["dx"])) <= 1e-2
  for name in ("dw_gate", "dw_up", "dw_down"):
    for r in range(world):
      assert O.rel_err(res[r][name], f32(g[name])[r * el:(r + 1) * el]) <= 1e-2, (name, r)
  for name in ("dw_router", "dws_gate", "dws_up", "dws_down"):
    assert O.rel_err(sum(r[name] for r in res), f32(g[name])) <= 1e-2, name
