"""Times the two sequence-mixing operators on one GPU: `python -m lewi_surge_b200.seqmix_bench [--b 8 --s 4096 ...]`.

Prints one line per operator (forward, forward+backward) from CUDA events around `--steps` calls after two warm-up
calls.  With `--steps` small it is also the program to put under a profiler."""
from __future__ import annotations

import argparse

import torch

from . import seqmix


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--b", type=int, default=8)
  ap.add_argument("--s", type=int, default=4096)
  ap.add_argument("--h", type=int, default=8)
  ap.add_argument("--k", type=int, default=128)
  ap.add_argument("--v", type=int, default=128)
  ap.add_argument("--channels", type=int, default=4096, help="channels of the causal convolution")
  ap.add_argument("--taps", type=int, default=4)
  ap.add_argument("--steps", type=int, default=10)
  ap.add_argument("--only", choices=["gdn", "conv"], default=None)
  a = ap.parse_args()
  dev = torch.device("cuda:0")
  gen = torch.Generator(device=dev).manual_seed(0)
  rn = lambda *shape: torch.randn(*shape, generator=gen, device=dev)

  def timed(fn):
    for _ in range(2):
      fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
      fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / a.steps

  if a.only in (None, "gdn"):
    q = rn(a.b, a.s, a.h, a.k).bfloat16().requires_grad_(True)
    k = (rn(a.b, a.s, a.h, a.k) / a.k ** 0.5 * 2).bfloat16().requires_grad_(True)
    v = rn(a.b, a.s, a.h, a.v).bfloat16().requires_grad_(True)
    g = (-torch.rand(a.b, a.s, a.h, generator=gen, device=dev) * 0.3).requires_grad_(True)
    beta = torch.rand(a.b, a.s, a.h, generator=gen, device=dev).bfloat16().requires_grad_(True)
    d_o = rn(a.b, a.s, a.h, a.v).bfloat16()
    with torch.no_grad():
      fwd = timed(lambda: seqmix.chunk_gated_delta_rule(q, k, v, g, beta))
    both = timed(lambda: seqmix.chunk_gated_delta_rule(q, k, v, g, beta)[0].backward(d_o))
    print(f"gated delta rule B={a.b} S={a.s} H={a.h} K={a.k} V={a.v}: forward {fwd:.3f} ms, forward+backward {both:.3f} ms "
          f"({a.b * a.s / both / 1e3:.2f} M tokens/s)")
  if a.only in (None, "conv"):
    x = rn(a.b, a.s, a.channels).bfloat16().requires_grad_(True)
    w = (rn(a.taps, 1, a.channels) * 0.5).requires_grad_(True)
    gy = rn(a.b, a.s, a.channels).bfloat16()
    with torch.no_grad():
      fwd = timed(lambda: seqmix.causal_conv1d(x, w))
    both = timed(lambda: torch.autograd.grad(seqmix.causal_conv1d(x, w), (x, w), gy))
    nbytes = 2 * a.b * a.s * a.channels * 2
    print(f"causal conv B={a.b} T={a.s} C={a.channels} taps={a.taps}: forward {fwd:.4f} ms ({nbytes / fwd / 1e6:.0f} GB/s), "
          f"forward+backward {both:.4f} ms")


if __name__ == "__main__":
  main()
