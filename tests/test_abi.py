"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "lewi_moe.h")


def declared_symbols():
  src = open(HEADER).read()
  src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
  return sorted(set(re.findall(r"\b(lewi_[a-z0-9_]+)\s*\(", src)))


@pytest.fixture(scope="module")
def lib():
  from lewi_surge_b200 import build, _lib
  build.build()
  return _lib.load()


def test_header_declares_entry_points():
  syms = declared_symbols()
  for must in ("lewi_router_topk", "lewi_sort_indices", "lewi_gather_rows", "lewi_gather_reduce", "lewi_gather_dot",
               "lewi_grouped_gemm_nn", "lewi_grouped_gemm_nt", "lewi_grouped_gemm_tn",
               "lewi_grouped_gemm_gateup_swiglu", "lewi_grouped_gemm_dh_dswiglu", "lewi_grouped_gemm_dx"):
    assert must in syms


def test_every_declared_symbol_is_exported(lib):
  raw = ctypes.CDLL(os.path.join(ROOT, "lewi_surge_b200", "liblewi_moe.so"))
  for name in declared_symbols():
    assert hasattr(raw, name), f"{name} declared in include/lewi_moe.h but not exported"


def test_binding_table_matches_header(lib):
  from lewi_surge_b200 import _lib
  assert sorted(_lib.SIGNATURES) == declared_symbols()


def header_prototypes():
  """name -> (return kind, [parameter kinds]) parsed from the header; kinds: P pointer, i int, l int64_t, f float."""
  src = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
  kinds = {"int": "i", "int64_t": "l", "float": "f"}
  out = {}
  for ret, name, params in re.findall(r"\b(int64_t|int|const char\s*\*)\s+(lewi_[a-z0-9_]+)\s*\((.*?)\)\s*;", src, flags=re.S):
    plist = []
    for prm in [q.strip() for q in params.split(",")]:
      if prm in ("void", ""):
        continue
      if "*" in prm or "(" in prm:
        plist.append("P")
      else:
        plist.append(kinds[prm.split()[-2] if len(prm.split()) > 1 else prm])
    out[name] = ("P" if "*" in ret else kinds[ret], plist)
  return out


def test_binding_argument_types_match_header(lib):
  """Every ctypes prototype has the header's parameter count and kinds (catches drift of either side)."""
  from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
  from lewi_surge_b200 import _lib
  kind = {c_void_p: "P", c_int: "i", c_int64: "l", c_float: "f", c_char_p: "P"}
  # function-pointer parameters span a comma in the header; they are checked by count of their own
  skip = {"lewi_moe_set_mark_callback"}
  protos = header_prototypes()
  for name, (res, args) in _lib.SIGNATURES.items():
    if name in skip:
      continue
    want_res, want_args = protos[name]
    assert kind[res] == want_res, name
    assert [kind[a] for a in args] == want_args, name


def test_host_only_entry_points(lib):
  assert lib.lewi_version() >= 100
  assert lib.lewi_padded_rows_bound(196608, 128, 128) == (196608 + 128 * 127) // 128 * 128
  assert lib.lewi_padded_rows_bound(-1, 128, 128) < 0
  assert lib.lewi_route_workspace_bytes(24576, 64) > 0
  assert b"workspace" in lib.lewi_error_string(-3)


def test_argument_rejection_without_gpu(lib):
  # null pointers and bad sizes are rejected before any CUDA call
  assert lib.lewi_gather_rows(None, None, None, None, None, 1, 1, 8, 0, 1, 0, None, 1) == -1
  assert lib.lewi_router_topk(None, None, 4, 8, 2, 128, None, None, None, None, None, None, None, None, None, None,
                              None, None, None, None, 0) == -1
  assert lib.lewi_grouped_gemm_nn(None, None, None, None, None, None, None, None, 128, 64, 64, 1, 0) == -1
  assert lib.lewi_grouped_gemm_tn(None, None, None, None, None, None, 128, 64, 64, 1, 0, None, 0) == -1
  assert lib.lewi_grouped_gemm_nn(None, 16, 16, 16, None, None, None, None, 128, 60, 64, 1, 0) == -2  # K % 8


def test_group_table_guards_without_gpu(lib):
  """Several experts need block_expert, or pad_offsets with CTA pairs; the pair kernels' per-expert table in shared
  memory holds 512 experts.  Both are rejected before anything is launched (16 stands in for non-null pointers)."""
  nn = lambda be, po, e: lib.lewi_grouped_gemm_nn(None, 16, 16, 16, None, be, None, po, 1024, 64, 64, e, 0)
  assert nn(None, 16, 513) == -5          # pad_offsets with more experts than the table holds
  assert nn(None, None, 4) == -2          # no way to find a block's expert
  lib.lewi_set_cta_pair(0)
  try:
    assert nn(None, 16, 4) == -2          # pad_offsets alone needs the CTA-pair kernels
  finally:
    lib.lewi_set_cta_pair(1)
  gu = lambda be, po, e: lib.lewi_grouped_gemm_gateup_swiglu(None, 16, 16, 16, 16, 16, be, None, po, 1024, 64, 64, e)
  assert gu(None, 16, 513) == -5 and gu(None, None, 4) == -2
  assert lib.lewi_grouped_gemm_dx(None, 16, 16, 16, 16, None, None, 16, 1024, 64, 64, 600) == -5


def test_layer_layout_functions_without_gpu(lib):
  import ctypes
  from lewi_surge_b200 import _lib
  off = (ctypes.c_int64 * 20)()
  total = lib.lewi_moe_residual_layout(4096, 1024, 64, 512, 6, 512, 0, off)
  assert total == off[19] > 0 and list(off) == sorted(off) and all(o % 256 == 0 for o in off)
  assert off[18] == off[19]               # no gate: that item is empty
  assert lib.lewi_moe_residual_layout(4096, 1024, 64, 512, 6, 512, 1, off) > total
  assert lib.lewi_moe_workspace_bytes(4096, 1024, 64, 512, 6, 512, 0) > 0
  assert lib.lewi_moe_workspace_bytes(4096, 0, 64, 512, 6, 512, 0) == -1
  assert lib.lewi_moe_router_prepared_bytes(1024, 64) == 4 * 1024 * 64 * 2
  # null pointers are rejected before any CUDA call
  assert lib.lewi_moe_fwd(*([None] * 16), 0, None, 0, 4096, 1024, 64, 512, 6, 512) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
  from lewi_surge_b200 import _lib
  monkeypatch.setattr(_lib, "_lib", None)
  monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
  with pytest.raises(_lib.LewiError):
    _lib.load()
