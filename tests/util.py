"""Helpers shared by the tests: numpy <-> torch conversion and the reference's error metric."""
import numpy as np
import torch

from oracle import bf16_round, rel_err  # noqa: F401


def to_dev(a, dtype, device):
  """numpy array (float32 values) -> torch tensor of `dtype` on `device`."""
  t = torch.from_numpy(np.ascontiguousarray(a))
  return t.to(device=device, dtype=dtype).contiguous()


def to_np(t):
  """torch tensor -> numpy (bf16 goes through float32)."""
  if t.dtype == torch.bfloat16:
    t = t.float()
  return t.detach().cpu().numpy()


def rand_routing(rng, n, e, k):
  """Top-k expert ids without repeats per token (modal/test_moe_permute.py:23-26)."""
  logits = rng.standard_normal((n, e)).astype(np.float32)
  return np.argsort(-logits, axis=1, kind="stable")[:, :k].astype(np.int32)


def softmax_np(a):
  a = a - a.max(axis=-1, keepdims=True)
  e = np.exp(a)
  return (e / e.sum(axis=-1, keepdims=True)).astype(np.float32)
