"""ctypes binding of liblewi_moe.so (the C ABI declared in include/lewi_moe.h).

There is no fallback: if the CUDA library is missing or a call is rejected, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblewi_moe.so")

BF16, F32 = 0, 1
STATUS_WAIT_TIMEOUT, STATUS_BAD_INDEX, STATUS_EP_OVERFLOW = 1, 2, 4

P = c_void_p  # every device pointer crosses the boundary as an integer address

# name -> (restype, argtypes); mirrors include/lewi_moe.h one to one
SIGNATURES = {
    "lewi_version": (c_int, []),
    "lewi_error_string": (c_char_p, [c_int]),
    "lewi_launch_count": (c_int64, []),
    "lewi_last_status": (c_int, [P]),
    "lewi_padded_rows_bound": (c_int64, [c_int64, c_int, c_int]),
    "lewi_route_workspace_bytes": (c_int64, [c_int64, c_int]),
    "lewi_router_logits_workspace_bytes": (c_int64, [c_int, c_int]),
    "lewi_router_logits": (c_int, [P, P, P, P, P, c_int64, c_int, c_int, P, c_int64]),
    "lewi_router_topk": (c_int, [P, P, c_int64, c_int, c_int, c_int, P, P, P, P, P, P, P, P, P, P, P, P, P, P, c_int64]),
    "lewi_router_topk_static_max_bytes": (c_int64, []),
    "lewi_router_topk_static": (c_int, [P, P, c_int64, c_int, c_int, c_int, P, P, P, P, P, P, P, P, P, P, P, P]),
    "lewi_sort_indices": (c_int, [P, P, c_int64, c_int, c_int, P, P, P, P, P, P, P, P, P, P, c_int64]),
    "lewi_router_topk_bwd": (c_int, [P, P, P, P, P, P, c_int64, c_int, c_int]),
    "lewi_cast_f32_to_bf16": (c_int, [P, P, P, c_int64]),
    "lewi_router_topk_bwd_partial": (c_int, [P, P, P, P, P, c_int, P, P, P, P, c_int64, c_int, c_int]),
    "lewi_router_bias_grad_workspace_bytes": (c_int64, [c_int64, c_int]),
    "lewi_router_topk_bwd_full": (c_int, [P, P, P, P, P, c_int, P, P, P, P, c_int64, c_int, c_int, P, c_float, P, P, c_int64]),
    "lewi_grouped_gemm_gateup_swiglu_scaled": (c_int, [P, P, P, P, P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int]),
    "lewi_dw_partial_parts": (c_int, [c_int]),
    "lewi_grouped_gemm_dh_dswiglu_scaled": (c_int, [P, P, P, P, P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int]),
    "lewi_group_tables": (c_int, [P, P, c_int64, c_int, c_int, P, P, P, P, P]),
    "lewi_gather_rows": (c_int, [P, P, P, P, P, c_int64, c_int64, c_int, c_int, c_int, c_int, P, c_int]),
    "lewi_dispatch_rows": (c_int, [P, P, P, P, P, c_int64, c_int, c_int, c_int64, P, c_int]),
    "lewi_gather_reduce": (c_int, [P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int, c_int, c_int64]),
    "lewi_gather_dot": (c_int, [P, P, P, P, P, c_int64, c_int, c_int, c_int, c_int64]),
    "lewi_grouped_gemm_nn": (c_int, [P, P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int, c_int]),
    "lewi_grouped_gemm_nt": (c_int, [P, P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int, c_int]),
    "lewi_grouped_gemm_tn": (c_int, [P, P, P, P, P, P, c_int64, c_int, c_int, c_int, c_int, P, c_int64]),
    "lewi_grouped_gemm_tn_workspace_bytes": (c_int64, [c_int64, c_int, c_int, c_int, c_int]),
    "lewi_grouped_gemm_gateup_swiglu": (c_int, [P, P, P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int]),
    "lewi_grouped_gemm_dh_dswiglu": (c_int, [P, P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int]),
    "lewi_grouped_gemm_dx": (c_int, [P, P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int]),
    "lewi_ep_unique_workspace_bytes": (c_int64, [c_int64, c_int]),
    "lewi_ep_unique_tables": (c_int, [P, P, c_int64, c_int, c_int, c_int, P, c_int, P, P, P, P, P, c_int64]),
    "lewi_ep_unique_plan": (c_int, [P, P, c_int, c_int, c_int64, P, P]),
    "lewi_ep_unique_meta": (c_int, [P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, c_int, c_int64, c_int, c_int, c_int,
                                    c_int64, c_int64]),
    "lewi_ep_push_unique": (c_int, [P, P, P, P, P, P, c_int, c_int64, c_int, c_int, c_int, c_int64, c_int]),
    "lewi_ep_local_rows": (c_int, [P, P, P, P, c_int, c_int, P, c_int, c_int64, c_int64]),
    "lewi_ep_combine_return": (c_int, [P, P, P, P, P, P, c_int, P, c_int, c_int, c_int, c_int64, c_int64, c_int]),
    "lewi_set_gemm_cta_limit": (c_int, [c_int]),
    "lewi_gdn_chunk_bwd_workspace_bytes": (c_int64, [c_int, c_int, c_int, c_int, c_int]),
    "lewi_gdn_chunk_bwd": (c_int, [P, P, P, P, P, P, P, P, P, P, c_int64, P, c_int64, P, P, P, P, P, P, c_int, c_int, c_int,
                                   c_int, c_int]),
    "lewi_grouped_gemm_nn_return": (c_int, [P, P, P, P, P, c_int, c_int64, P, P, P, c_int64, c_int, c_int, c_int]),
    "lewi_grouped_gemm_dx_return": (c_int, [P, P, P, P, P, P, c_int, c_int64, P, P, P, c_int64, c_int, c_int, c_int]),
    "lewi_causal_conv1d_workspace_bytes": (c_int64, [c_int, c_int, c_int, c_int]),
    "lewi_causal_conv1d_fwd": (c_int, [P, P, P, P, c_int, c_int, c_int, c_int]),
    "lewi_causal_conv1d_bwd": (c_int, [P, P, P, P, P, P, c_int, P, c_int64, c_int, c_int, c_int, c_int]),
    "lewi_gdn_chunk_workspace_bytes": (c_int64, [c_int, c_int, c_int, c_int, c_int]),
    "lewi_gdn_chunk_fwd": (c_int, [P, P, P, P, P, P, P, P, P, P, c_int64, c_int, c_int, c_int, c_int, c_int]),
    "lewi_moe_residual_layout": (c_int64, [c_int64, c_int, c_int, c_int, c_int, c_int, c_int, P]),
    "lewi_moe_workspace_bytes": (c_int64, [c_int64, c_int, c_int, c_int, c_int, c_int, c_int]),
    "lewi_moe_router_prepared_bytes": (c_int64, [c_int, c_int]),
    "lewi_moe_prepare_router": (c_int, [P, P, P, c_int, c_int]),
    "lewi_moe_fwd": (c_int, [P] * 16 + [c_int64, P, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int]),
    "lewi_moe_bwd": (c_int, [P] * 14 + [c_int64, P, c_int64] + [P] * 11 + [c_float, c_int, c_int64, c_int, c_int, c_int, c_int, c_int]),
    "lewi_moe_set_mark_callback": (c_int, [P]),
    "lewi_ep_alloc": (c_int, [c_int64, P]),
    "lewi_ep_free": (c_int, [P]),
    "lewi_ep_ipc_export": (c_int, [P, P]),
    "lewi_ep_ipc_import": (c_int, [P, P]),
    "lewi_ep_ipc_release": (c_int, [P]),
    "lewi_ep_plan": (c_int, [P, P, c_int, c_int, c_int, c_int, c_int64, P, P, P, P, P, P]),
    "lewi_ep_push_rows": (c_int, [P, P, P, P, P, P, P, P, P, P, c_int, c_int64, c_int, c_int, c_int, c_int, c_int64, c_int64,
                                  c_int, c_int, c_int]),
    "lewi_ep_return_rows": (c_int, [P, P, P, P, P, c_int, c_int, P, P, c_int, c_int, c_int, c_int64, c_int64, c_int]),
    "lewi_ep_zero_pad": (c_int, [P, P, P, P, P, c_int, c_int, c_int64]),
    "lewi_set_sm_sharing": (c_int, [c_int]),
    "lewi_ep_put_i32": (c_int, [P, P, P, c_int64, c_int, c_int]),
    "lewi_ep_barrier": (c_int, [P, P, P, P, c_int, c_int, c_int64]),
    "lewi_set_cta_pair": (c_int, [c_int]),
}

_lib = None


class LewiError(RuntimeError):
  pass


def load():
  """Load the shared library once and set the prototypes.  Raises if it has not been built."""
  global _lib
  if _lib is not None:
    return _lib
  if not os.path.exists(LIB_PATH):
    raise LewiError(
        f"{LIB_PATH} not found: build it first (python -m lewi_surge_b200.build). There is no CPU fallback.")
  lib = ctypes.CDLL(LIB_PATH)
  for name, (res, args) in SIGNATURES.items():
    fn = getattr(lib, name)
    fn.restype = res
    fn.argtypes = args
  _lib = lib
  return lib


def check(rc, what):
  if rc != 0:
    msg = load().lewi_error_string(int(rc)).decode()
    raise LewiError(f"{what}: {msg} (code {rc})")


def ptr(t):
  """Device address of a torch tensor (None -> null)."""
  if t is None:
    return None
  if not t.is_cuda:
    raise LewiError("expected a CUDA tensor: the kernels have no CPU path")
  if not t.is_contiguous():
    raise LewiError("expected a contiguous tensor")
  return t.data_ptr()


def stream():
  import torch
  return torch.cuda.current_stream().cuda_stream


def last_status():
  """Synchronise the current stream, return and clear the device status word."""
  rc = load().lewi_last_status(stream())
  if rc < 0:
    check(rc, "lewi_last_status")
  return rc
