"""The workspace-free router entry point, lewi_router_topk_static, against lewi_router_topk.

Some callers cannot give the library a scratch buffer and must not allocate (a handler inside a
compiled XLA program, a serving runtime with a fixed memory budget).  For them the library carries a
fixed 4 MiB scratch array of its own.  This test drives the entry point through the C ABI exactly as
such a caller would -- ctypes, raw device addresses, no workspace -- and requires bit-identical
outputs to the ordinary entry point, twice in a row (the shared array keeps the first call's
contents, so the second call proves nothing stale is read).  It lives in a file that sorts last so
that a run stopping at the first failure has already executed every other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FIELDS = ("topk_idx", "topk_w", "counts", "offsets", "pad_offsets", "block_expert", "n_blocks", "order", "pos",
          "pad_pos", "row_slot", "probs_sum")


def call_static(lib, logits, k, block=128):
  """Calls lewi_router_topk_static with freshly made output tensors; returns them by name."""
  from lewi_surge_b200 import _lib, ops
  t, e = logits.shape
  m = t * k
  dev = logits.device
  mpad = ops.padded_rows_bound(m, e, block)
  i32 = dict(dtype=torch.int32, device=dev)
  out = dict(topk_idx=torch.empty((t, k), **i32), topk_w=torch.empty((t, k), dtype=torch.float32, device=dev),
             counts=torch.empty(e, **i32), offsets=torch.empty(e + 1, **i32), pad_offsets=torch.empty(e + 1, **i32),
             block_expert=torch.empty(mpad // block, **i32), n_blocks=torch.empty(1, **i32), order=torch.empty(m, **i32),
             pos=torch.empty(m, **i32), pad_pos=torch.empty(m, **i32), row_slot=torch.empty(mpad, **i32),
             probs_sum=torch.empty(e, dtype=torch.float32, device=dev))
  rc = lib.lewi_router_topk_static(_lib.stream(), _lib.ptr(logits), t, e, k, block, *(_lib.ptr(out[n]) for n in FIELDS))
  return rc, out


def test_static_scratch_variant_matches_workspace_variant_twice(cuda):
  from lewi_surge_b200 import _lib, layer
  lib = _lib.load()
  assert lib.lewi_router_topk_static_max_bytes() == 4 * 1024 * 1024
  g = torch.Generator(device="cpu").manual_seed(123)
  cases = [(4096, 64, 6), (1000, 128, 8)]          # the second call reuses the array the first one dirtied
  for t, e, k in cases:
    logits = torch.randn((t, e), generator=g, dtype=torch.float32).to(cuda)
    want = layer.router_topk(logits, k)
    rc, got = call_static(lib, logits, k)
    assert rc == 0, lib.lewi_error_string(rc)
    assert _lib.last_status() == 0
    for name in FIELDS:
      w = getattr(want, name)
      n = got[name].numel()
      assert torch.equal(got[name].reshape(-1), w.reshape(-1)[:n]), name
    # and directly against the CPU restatement of the router and of the reference's stable slot sort
    import oracle as O
    idx, wts, _ = O.router_topk(logits.cpu().numpy(), k)
    lay = O.block_layout(idx.reshape(-1), e)
    assert np.array_equal(got["topk_idx"].cpu().numpy(), idx)
    assert O.rel_err(got["topk_w"].cpu().numpy(), wts) <= 1e-5
    for name in ("counts", "offsets", "pad_offsets", "order", "pos", "pad_pos", "row_slot"):
      assert np.array_equal(got[name].cpu().numpy(), lay[name]), name
  # and once more on the first shape: same answer after the array has held other data
  logits = torch.randn((4096, 64), generator=torch.Generator(device="cpu").manual_seed(123), dtype=torch.float32).to(cuda)
  want = layer.router_topk(logits, 6)
  rc, got = call_static(lib, logits, 6)
  assert rc == 0
  for name in FIELDS:
    n = got[name].numel()
    assert torch.equal(got[name].reshape(-1), getattr(want, name).reshape(-1)[:n]), name


def test_static_scratch_variant_rejects_oversized_problem(cuda):
  from lewi_surge_b200 import _lib
  lib = _lib.load()
  t, e, k = 65536, 128, 8     # needs more than 4 MiB of scratch
  assert lib.lewi_route_workspace_bytes(t * k, e) > lib.lewi_router_topk_static_max_bytes()
  logits = torch.zeros((t, e), dtype=torch.float32, device=cuda)
  rc, _ = call_static(lib, logits, k)
  assert rc == -6
  assert b"built-in scratch" in lib.lewi_error_string(rc)
