// liblewi_moe.so: C ABI over the sm_100a kernels (declarations and contracts: include/lewi_moe.h).
#include "common.cuh"
#include "ep.cuh"
#include "gather.cuh"
#include "grouped_gemm.cuh"
#include "router_gemm.cuh"
#include "routing.cuh"

#include <cstring>
#include <mutex>

using namespace lewi;

// Scratch for lewi_router_topk_static(): lives in the library image, so every GPU that loads the
// library holds these bytes until the process exits.  Host code must not pass this name to a kernel:
// on the host it is only a handle; the device address comes from cudaGetSymbolAddress().
#define LEWI_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
static __device__ __align__(256) unsigned char g_route_static_scratch[LEWI_STATIC_SCRATCH_BYTES];

namespace {

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" {

int lewi_version(void) { return 100; }

const char* lewi_error_string(int code) {
  switch (code) {
    case LEWI_OK: return "ok";
    case LEWI_ERR_ARG: return "bad argument (null pointer, non-positive size or unknown dtype)";
    case LEWI_ERR_SHAPE: return "shape not supported by the kernels";
    case LEWI_ERR_WORKSPACE: return "workspace missing or too small";
    case LEWI_ERR_CUDA: return "CUDA call failed at launch";
    case LEWI_ERR_LIMIT: return "size beyond a compiled-in maximum";
    case LEWI_ERR_STATIC_SCRATCH:
      return "problem too large for the built-in scratch of lewi_router_topk_static (see "
             "lewi_router_topk_static_max_bytes); use lewi_router_topk with a caller-supplied workspace";
    default: return "unknown error code";
  }
}

int64_t lewi_launch_count(void) { return launch_counter(); }

int lewi_last_status(void* stream) {
  if (cudaStreamSynchronize(as_stream(stream)) != cudaSuccess) return LEWI_ERR_CUDA;
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return LEWI_ERR_CUDA;
  if (v != 0 && cudaMemcpyToSymbol(g_status, &zero, sizeof(int)) != cudaSuccess) return LEWI_ERR_CUDA;
  return v;
}

int64_t lewi_padded_rows_bound(int64_t m, int num_experts, int block) {
  if (m < 0 || num_experts <= 0 || block <= 0) return LEWI_ERR_ARG;
  return (m + (int64_t)num_experts * (block - 1)) / block * block;
}

int64_t lewi_route_workspace_bytes(int64_t num_slots, int num_experts) {
  if (num_slots < 0 || num_experts <= 0) return LEWI_ERR_ARG;
  const int64_t chunks = (num_slots + 127) / 128 + 1;
  const int64_t bytes = chunks * num_experts * 8 + (int64_t)(num_experts + 1) * 4;
  return (bytes + 255) / 256 * 256;
}

// ------------------------------------------------------------------------------------------------ router

int lewi_router_topk(void* stream, const float* logits, int64_t T, int E, int k, int block, int32_t* topk_idx,
                     float* topk_w, int32_t* counts, int32_t* offsets, int32_t* pad_offsets,
                     int32_t* block_expert, int32_t* n_blocks, int32_t* order, int32_t* pos, int32_t* pad_pos,
                     int32_t* row_slot, float* probs_sum, void* workspace, int64_t workspace_bytes) {
  if (!logits || !topk_idx || !topk_w || T < 0 || E <= 0 || k <= 0) return LEWI_ERR_ARG;
  if (k > E || k > kMaxTopK) return LEWI_ERR_LIMIT;
  if (block > 0 && (!pad_offsets || !block_expert || !n_blocks)) return LEWI_ERR_ARG;
  return route_common(as_stream(stream), logits, nullptr, T, T * k, E, k, block, topk_idx, topk_w, counts, offsets,
                      pad_offsets, block_expert, n_blocks, order, pos, pad_pos, row_slot, probs_sum, workspace,
                      workspace_bytes);
}

int64_t lewi_router_topk_static_max_bytes(void) { return LEWI_STATIC_SCRATCH_BYTES; }

int lewi_router_topk_static(void* stream, const float* logits, int64_t T, int E, int k, int block,
                            int32_t* topk_idx, float* topk_w, int32_t* counts, int32_t* offsets,
                            int32_t* pad_offsets, int32_t* block_expert, int32_t* n_blocks, int32_t* order,
                            int32_t* pos, int32_t* pad_pos, int32_t* row_slot, float* probs_sum) {
  if (!logits || !topk_idx || !topk_w || T < 0 || E <= 0 || k <= 0) return LEWI_ERR_ARG;
  if (k > E || k > kMaxTopK) return LEWI_ERR_LIMIT;
  if (block > 0 && (!pad_offsets || !block_expert || !n_blocks)) return LEWI_ERR_ARG;
  // The problem must fit the built-in scratch; nothing is launched otherwise.
  const int64_t need = lewi_route_workspace_bytes(T * k, E);
  if (need < 0 || need > (int64_t)LEWI_STATIC_SCRATCH_BYTES) return LEWI_ERR_STATIC_SCRATCH;
  // One-time set-up per device, done with that device current: resolve the device address of the array.
  static std::mutex mu;
  static void* dev_ptr[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return LEWI_ERR_CUDA;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev_ptr[dev] == nullptr) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_route_static_scratch) != cudaSuccess || p == nullptr) {
        (void)cudaGetLastError();
        return LEWI_ERR_CUDA;
      }
      dev_ptr[dev] = p;
    }
    scratch = dev_ptr[dev];
  }
  return route_common(as_stream(stream), logits, nullptr, T, T * k, E, k, block, topk_idx, topk_w, counts, offsets,
                      pad_offsets, block_expert, n_blocks, order, pos, pad_pos, row_slot, probs_sum, scratch,
                      LEWI_STATIC_SCRATCH_BYTES);
}

int lewi_sort_indices(void* stream, const int32_t* flat_experts, int64_t M, int E, int block, int32_t* order,
                      int32_t* pos, int32_t* counts, int32_t* offsets, int32_t* pad_offsets, int32_t* block_expert,
                      int32_t* n_blocks, int32_t* pad_pos, int32_t* row_slot, void* workspace,
                      int64_t workspace_bytes) {
  if (!flat_experts || M < 0 || E <= 0) return LEWI_ERR_ARG;
  if (block > 0 && pad_offsets && (!block_expert || !n_blocks)) return LEWI_ERR_ARG;
  return route_common(as_stream(stream), nullptr, flat_experts, 0, M, E, 1, pad_offsets ? block : 0, nullptr,
                      nullptr, counts, offsets, pad_offsets, block_expert, n_blocks, order, pos, pad_pos, row_slot,
                      nullptr, workspace, workspace_bytes);
}

int lewi_router_topk_bwd(void* stream, const float* logits, const int32_t* topk_idx, const float* dw,
                         float* dlogits, void* dlogits_bf16, int64_t T, int E, int k) {
  return lewi_router_topk_bwd_partial(stream, logits, topk_idx, dw, nullptr, 0, nullptr, nullptr, dlogits, dlogits_bf16,
                                      T, E, k);
}

int lewi_router_topk_bwd_partial(void* stream, const float* logits, const int32_t* topk_idx, const float* dw,
                                 const float* dw_partial, int dw_parts, const int32_t* pad_pos, float* dw_out,
                                 float* dlogits, void* dlogits_bf16, int64_t T, int E, int k) {
  if (!logits || !topk_idx || (!dw && !dw_partial) || (!dlogits && !dlogits_bf16) || T < 0 || E <= 0 || k <= 0)
    return LEWI_ERR_ARG;
  if (dw_partial != nullptr && (dw_parts <= 0 || pad_pos == nullptr)) return LEWI_ERR_ARG;
  __nv_bfloat16* dlb = reinterpret_cast<__nv_bfloat16*>(dlogits_bf16);
  if (E > kMaxExperts || k > kMaxTopK || k > E) return LEWI_ERR_LIMIT;
  if (T == 0) return LEWI_OK;
  const int grid = gather_grid(T);
  cudaStream_t st = as_stream(stream);
  if (E <= 64) router_topk_bwd_kernel<2><<<grid, 256, 0, st>>>(logits, topk_idx, dw, dw_partial, dw_parts, pad_pos, dw_out, dlogits, dlb, T, E, k);
  else if (E <= 128) router_topk_bwd_kernel<4><<<grid, 256, 0, st>>>(logits, topk_idx, dw, dw_partial, dw_parts, pad_pos, dw_out, dlogits, dlb, T, E, k);
  else if (E <= 256) router_topk_bwd_kernel<8><<<grid, 256, 0, st>>>(logits, topk_idx, dw, dw_partial, dw_parts, pad_pos, dw_out, dlogits, dlb, T, E, k);
  else router_topk_bwd_kernel<16><<<grid, 256, 0, st>>>(logits, topk_idx, dw, dw_partial, dw_parts, pad_pos, dw_out, dlogits, dlb, T, E, k);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_cast_f32_to_bf16(void* stream, const float* src, void* dst, int64_t n) {
  if (!src || !dst || n < 0) return LEWI_ERR_ARG;
  if (n == 0) return LEWI_OK;
  long long grid = (n + 255) / 256;
  if (grid > (long long)num_sms() * 8) grid = (long long)num_sms() * 8;
  cast_f32_bf16_kernel<<<(int)grid, 256, 0, as_stream(stream)>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), n);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_group_tables(void* stream, const int32_t* group_sizes, int64_t M, int E, int block, int32_t* pad_offsets,
                      int32_t* block_expert, int32_t* n_blocks, int32_t* row_of_padded, int32_t* padded_of_row) {
  if (!group_sizes || !pad_offsets || !block_expert || !n_blocks || !row_of_padded || !padded_of_row || M < 0 ||
      E <= 0 || block <= 0)
    return LEWI_ERR_ARG;
  if (E > kMaxExperts) return LEWI_ERR_LIMIT;
  const long long mpad = (M + (long long)E * (block - 1)) / block * block;
  const int nbmax = (int)(mpad / block);
  long long work = mpad > M ? mpad : M;
  int grid = (int)((work + 255) / 256);
  if (grid < 1) grid = 1;
  if (grid > num_sms() * 8) grid = num_sms() * 8;
  group_tables_kernel<<<grid, 256, 0, as_stream(stream)>>>(group_sizes, M, E, block, mpad, nbmax, pad_offsets,
                                                           block_expert, n_blocks, row_of_padded, padded_of_row);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

// ------------------------------------------------------------------------------------------------ gathers

int lewi_gather_rows(void* stream, const void* x, const int32_t* idx, const float* scale, void* out, int64_t n_src,
                     int64_t m, int d, int dtype, int idx_div, int scale_by_idx, const int32_t* n_rows_dev,
                     int rows_per_unit) {
  if (!x || !idx || !out || n_src < 0 || m < 0 || d <= 0) return LEWI_ERR_ARG;
  if (dtype != LEWI_BF16 && dtype != LEWI_F32) return LEWI_ERR_ARG;
  if (!aligned16(x) || !aligned16(out)) return LEWI_ERR_SHAPE;
  const int vpl = pick_vpl(d, dtype == LEWI_BF16 ? 2 : 4);
  if (vpl == 0) return LEWI_ERR_SHAPE;
  if (m == 0) return LEWI_OK;
  const int grid = gather_grid(m);
  cudaStream_t st = as_stream(stream);
  if (dtype == LEWI_BF16) {
    LEWI_DISPATCH_VPL(vpl, (gather_rows_kernel<__nv_bfloat16, VPL><<<grid, kGatherThreads, 0, st>>>(
                               reinterpret_cast<const __nv_bfloat16*>(x), idx, scale,
                               reinterpret_cast<__nv_bfloat16*>(out), n_src, m, d, idx_div, scale_by_idx, n_rows_dev,
                               rows_per_unit)));
  } else {
    LEWI_DISPATCH_VPL(vpl, (gather_rows_kernel<float, VPL><<<grid, kGatherThreads, 0, st>>>(
                               reinterpret_cast<const float*>(x), idx, scale, reinterpret_cast<float*>(out), n_src, m,
                               d, idx_div, scale_by_idx, n_rows_dev, rows_per_unit)));
  }
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_gather_reduce(void* stream, const void* y, const int32_t* pos, const float* w, const void* add0,
                       const void* add1, void* out, int64_t n, int k, int d, int in_dtype, int out_dtype,
                       int64_t n_y_rows) {
  if (!y || !pos || !out || n < 0 || k <= 0 || d <= 0 || n_y_rows < 0) return LEWI_ERR_ARG;
  if ((in_dtype != LEWI_BF16 && in_dtype != LEWI_F32) || (out_dtype != LEWI_BF16 && out_dtype != LEWI_F32))
    return LEWI_ERR_ARG;
  if (k > kWarp) return LEWI_ERR_LIMIT;
  if (!aligned16(y) || !aligned16(out) || !aligned16(add0) || !aligned16(add1)) return LEWI_ERR_SHAPE;
  const int vpl = pick_vpl(d, in_dtype == LEWI_BF16 ? 2 : 4);
  if (vpl == 0) return LEWI_ERR_SHAPE;
  if (n == 0) return LEWI_OK;
  const int grid = gather_grid(n);
  cudaStream_t st = as_stream(stream);
#define LEWI_GR(TI, TO)                                                                                         \
  LEWI_DISPATCH_VPL(vpl, (gather_reduce_kernel<TI, TO, VPL><<<grid, kGatherThreads, 0, st>>>(                   \
                             reinterpret_cast<const TI*>(y), pos, w, reinterpret_cast<const TI*>(add0),         \
                             reinterpret_cast<const TI*>(add1), reinterpret_cast<TO*>(out), n, k, d, n_y_rows)))
  if (in_dtype == LEWI_BF16 && out_dtype == LEWI_BF16) { LEWI_GR(__nv_bfloat16, __nv_bfloat16); }
  else if (in_dtype == LEWI_BF16) { LEWI_GR(__nv_bfloat16, float); }
  else if (out_dtype == LEWI_BF16) { LEWI_GR(float, __nv_bfloat16); }
  else { LEWI_GR(float, float); }
#undef LEWI_GR
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_gather_dot(void* stream, const void* y, const int32_t* pos, const void* g, float* out, int64_t n, int k,
                    int d, int dtype, int64_t n_y_rows) {
  if (!y || !pos || !g || !out || n < 0 || k <= 0 || d <= 0 || n_y_rows < 0) return LEWI_ERR_ARG;
  if (dtype != LEWI_BF16 && dtype != LEWI_F32) return LEWI_ERR_ARG;
  if (k > kWarp) return LEWI_ERR_LIMIT;
  if (!aligned16(y) || !aligned16(g)) return LEWI_ERR_SHAPE;
  const int vpl = pick_vpl(d, dtype == LEWI_BF16 ? 2 : 4);
  if (vpl == 0) return LEWI_ERR_SHAPE;
  if (n == 0) return LEWI_OK;
  const int grid = gather_grid(n);
  cudaStream_t st = as_stream(stream);
  if (dtype == LEWI_BF16) {
    LEWI_DISPATCH_VPL(vpl, (gather_dot_kernel<__nv_bfloat16, VPL><<<grid, kGatherThreads, 0, st>>>(
                               reinterpret_cast<const __nv_bfloat16*>(y), pos, reinterpret_cast<const __nv_bfloat16*>(g),
                               out, n, k, d, n_y_rows)));
  } else {
    LEWI_DISPATCH_VPL(vpl, (gather_dot_kernel<float, VPL><<<grid, kGatherThreads, 0, st>>>(
                               reinterpret_cast<const float*>(y), pos, reinterpret_cast<const float*>(g), out, n, k, d,
                               n_y_rows)));
  }
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

// ------------------------------------------------------------------------------------------------ grouped GEMMs

namespace {

int g_debug_flags = 0;

struct RowGroupArgs {
  const int32_t* block_expert;
  const int32_t* n_blocks;
  const int32_t* pad_offsets;
  int64_t rows;
  int E;
};

// The CTA-pair kernels derive a row block's expert from pad_offsets; the single-CTA ones read
// block_expert.  One group (no tables at all) works with both.
inline bool use_pair(const RowGroupArgs& r) {
  if (!gg::pair_mode()) return false;
  if (r.block_expert != nullptr && r.pad_offsets == nullptr) return false;
  const long long nb = (r.rows + gg::BM - 1) / gg::BM;
  return (nb + r.E) / 2 + 1 < 65535;   // pair prefixes are kept as 16-bit counts
}

inline int check_rows(const RowGroupArgs& r) {
  if (r.rows < 0 || r.E <= 0) return LEWI_ERR_ARG;
  if (r.rows > 0x7fffff00LL) return LEWI_ERR_LIMIT;
  return LEWI_OK;
}

inline void fill_common(gg::Args& a, const RowGroupArgs& r) {
  a.out = nullptr;
  a.out2 = nullptr;
  a.gu = nullptr;
  a.row_scale = nullptr;
  a.block_expert = r.block_expert;
  a.n_blocks = r.n_blocks;
  a.pad_offsets = r.pad_offsets;
  a.rows = r.rows;
  a.n_blocks_host = (int)((r.rows + gg::BM - 1) / gg::BM);
  if (use_pair(r)) a.n_blocks_host = (int)((a.n_blocks_host + r.E + 1) / 2);   // bound on row-block pairs
  a.K = 0;
  a.N = 0;
  a.Ma = 0;
  a.E = r.E;
  a.kb_split = 1 << 30;
  a.k2_offset = 0;
  a.kb_total = 0;
  a.out_f32 = 0;
  a.a_k_wrap = 0;
  a.k_splits = 1;
  a.partial = nullptr;
  a.col_bias = nullptr;
  a.scale_src = nullptr;
  a.scale_idx = nullptr;
  a.dw_partial = nullptr;
  a.dw_parts = 0;
  a.ga_ptr = nullptr;
  a.gb_ptr = nullptr;
  a.ga_ld = 0;
  a.gb_ld = 0;
  a.g_idx = nullptr;
  a.g_div = 1;
  a.g_src_rows = 0;
  a.dbg = g_debug_flags;
}

// Number of contraction parts for a TN product with `tiles0` output tiles (1 = no split).
inline int tn_pick_splits(long long tiles0, int64_t rows) {
  const int sms = num_sms();
  if (tiles0 <= 0 || tiles0 * 2 > sms) return 1;
  long long s = (sms + tiles0 - 1) / tiles0;
  const long long kb_total = (rows + gg::BK - 1) / gg::BK;
  if (s > kb_total / 4) s = kb_total / 4;
  if (s > 64) s = 64;
  return s < 1 ? 1 : (int)s;
}

}  // namespace

int64_t lewi_router_logits_workspace_bytes(int d, int E) {
  if (d <= 0 || E <= 0) return LEWI_ERR_ARG;
  return ((int64_t)3 * d * E * 2 + 255) / 256 * 256;
}

int lewi_router_logits(void* stream, const void* x, const float* w_router, const float* bias, float* logits,
                       int64_t T, int d, int E, void* workspace, int64_t workspace_bytes) {
  if (!x || !w_router || !logits || T < 0 || d <= 0 || E <= 0) return LEWI_ERR_ARG;
  if (T == 0) return LEWI_OK;
  cudaStream_t st = as_stream(stream);
  const bool tensor_path = workspace != nullptr && workspace_bytes >= (int64_t)3 * d * E * 2 && d % 64 == 0 &&
                           E % 64 == 0 && aligned16(x) && aligned16(workspace) && aligned16(logits) &&
                           T <= 0x7fffff00LL;
  if (!tensor_path) {
    dim3 grid((unsigned)((T + kRgTile - 1) / kRgTile), (unsigned)((E + kRgTile - 1) / kRgTile));
    router_logits_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), w_router, bias, logits, T,
                                               d, E);
    LEWI_CHECK_LAUNCH();
    return LEWI_OK;
  }
  // f32 weight = hi + mid + lo (three bf16 pieces, 24 mantissa bits); x is bf16, so every product is
  // exact in f32 and the tensor cores accumulate in f32: logits = [x x x] . [hi; mid; lo].
  __nv_bfloat16* w3 = reinterpret_cast<__nv_bfloat16*>(workspace);
  const long long n = (long long)d * E;
  long long sgrid = (n + 255) / 256;
  if (sgrid > (long long)num_sms() * 8) sgrid = (long long)num_sms() * 8;
  split3_bf16_kernel<<<(int)sgrid, 256, 0, st>>>(w_router, w3, n);
  LEWI_CHECK_LAUNCH();
  CUtensorMap ta, tb;
  if (!gg::make_map(&ta, x, (uint64_t)d, (uint64_t)T, 0, 64, 128)) return LEWI_ERR_CUDA;
  if (!gg::make_map(&tb, w3, (uint64_t)E, (uint64_t)3 * d, 1, 64, 64)) return LEWI_ERR_CUDA;
  RowGroupArgs r{nullptr, nullptr, nullptr, T, 1};
  const bool pair = use_pair(r);
  gg::Args a;
  fill_common(a, r);
  a.out = logits;
  a.K = 3 * d;
  a.kb_total = 3 * d / gg::BK;
  a.N = E;
  a.out_f32 = 1;
  a.a_k_wrap = d;
  a.col_bias = bias;
  const long long tiles = (long long)a.n_blocks_host * ((E + gg::BN - 1) / gg::BN);
  return gg::launch_auto<gg::NN, gg::PLAIN>(pair, st, ta, tb, tb, a, tiles);
}

int lewi_grouped_gemm_nn(void* stream, const void* a_ptr, const void* b_ptr, void* out, const float* row_scale,
                         const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows,
                         int K, int N, int E, int out_dtype) {
  if (!a_ptr || !b_ptr || !out || K <= 0 || N <= 0) return LEWI_ERR_ARG;
  if (out_dtype != LEWI_BF16 && out_dtype != LEWI_F32) return LEWI_ERR_ARG;
  RowGroupArgs r{block_expert, n_blocks, pad_offsets, rows, E};
  const bool pair = use_pair(r);
  if (int rc = check_rows(r)) return rc;
  if (K % 8 != 0 || N % 8 != 0 || !aligned16(a_ptr) || !aligned16(b_ptr) || !aligned16(out)) return LEWI_ERR_SHAPE;
  if (rows == 0) return LEWI_OK;
  CUtensorMap ta, tb;
  if (!gg::make_map(&ta, a_ptr, (uint64_t)K, (uint64_t)rows, 0, 64, 128)) return LEWI_ERR_CUDA;
  if (!gg::make_map(&tb, b_ptr, (uint64_t)N, (uint64_t)K, (uint64_t)E, 64, 64)) return LEWI_ERR_CUDA;
  gg::Args a;
  fill_common(a, r);
  a.out = out;
  a.row_scale = row_scale;
  a.K = K;
  a.kb_total = (K + gg::BK - 1) / gg::BK;
  a.N = N;
  a.out_f32 = out_dtype == LEWI_F32;
  const long long tiles = (long long)a.n_blocks_host * ((N + gg::BN - 1) / gg::BN);
  return gg::launch_auto<gg::NN, gg::PLAIN>(pair, as_stream(stream), ta, tb, tb, a, tiles);
}

int lewi_grouped_gemm_nt(void* stream, const void* a_ptr, const void* b_ptr, void* out, const float* row_scale,
                         const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows,
                         int K, int N, int E, int out_dtype) {
  if (!a_ptr || !b_ptr || !out || K <= 0 || N <= 0) return LEWI_ERR_ARG;
  if (out_dtype != LEWI_BF16 && out_dtype != LEWI_F32) return LEWI_ERR_ARG;
  RowGroupArgs r{block_expert, n_blocks, pad_offsets, rows, E};
  const bool pair = use_pair(r);
  if (int rc = check_rows(r)) return rc;
  if (K % 8 != 0 || N % 8 != 0 || !aligned16(a_ptr) || !aligned16(b_ptr) || !aligned16(out)) return LEWI_ERR_SHAPE;
  if (rows == 0) return LEWI_OK;
  CUtensorMap ta, tb;
  if (!gg::make_map(&ta, a_ptr, (uint64_t)K, (uint64_t)rows, 0, 64, 128)) return LEWI_ERR_CUDA;
  if (!gg::make_map(&tb, b_ptr, (uint64_t)K, (uint64_t)N, (uint64_t)E, 64, pair ? 128 : 256)) return LEWI_ERR_CUDA;
  gg::Args a;
  fill_common(a, r);
  a.out = out;
  a.row_scale = row_scale;
  a.K = K;
  a.kb_total = (K + gg::BK - 1) / gg::BK;
  a.N = N;
  a.out_f32 = out_dtype == LEWI_F32;
  const long long tiles = (long long)a.n_blocks_host * ((N + gg::BN - 1) / gg::BN);
  return gg::launch_auto<gg::NT, gg::PLAIN>(pair, as_stream(stream), ta, tb, tb, a, tiles);
}

int64_t lewi_grouped_gemm_tn_workspace_bytes(int64_t rows, int Ma, int Nb, int E, int split_out) {
  if (rows < 0 || Ma <= 0 || Nb <= 0 || E <= 0) return LEWI_ERR_ARG;
  const long long n_tiles = split_out ? 2LL * ((Nb / 2 + gg::BN - 1) / gg::BN) : (Nb + gg::BN - 1) / gg::BN;
  const int tm = gg::pair_mode() ? 2 * gg::BM : gg::BM;
  const long long tiles0 = (long long)E * ((Ma + tm - 1) / tm) * n_tiles;
  const int s = tn_pick_splits(tiles0 * (gg::pair_mode() ? 2 : 1), rows);
  return s > 1 ? (int64_t)s * E * Ma * Nb * 4 : 0;
}

int lewi_grouped_gemm_tn(void* stream, const void* a_ptr, const void* b_ptr, void* out, void* out2,
                         const int32_t* pad_offsets, int64_t rows, int Ma, int Nb, int E, int out_dtype,
                         void* workspace, int64_t workspace_bytes) {
  return lewi_grouped_gemm_tn_gather(stream, a_ptr, b_ptr, out, out2, pad_offsets, rows, Ma, Nb, E, out_dtype, workspace,
                                     workspace_bytes, nullptr, 1, 0, 0, 0);
}

int lewi_grouped_gemm_tn_gather(void* stream, const void* a_ptr, const void* b_ptr, void* out, void* out2,
                                const int32_t* pad_offsets, int64_t rows, int Ma, int Nb, int E, int out_dtype,
                                void* workspace, int64_t workspace_bytes, const int32_t* row_idx, int idx_div,
                                int64_t src_rows, int gather_a, int gather_b) {
  if (!a_ptr || !b_ptr || !out || Ma <= 0 || Nb <= 0 || rows < 0 || E <= 0) return LEWI_ERR_ARG;
  if ((gather_a || gather_b) && (!row_idx || idx_div <= 0 || src_rows <= 0 || src_rows > 0x7fffffffLL))
    return LEWI_ERR_ARG;
  if (out_dtype != LEWI_BF16 && out_dtype != LEWI_F32) return LEWI_ERR_ARG;
  if (rows > 0x7fffff00LL) return LEWI_ERR_LIMIT;
  if (Ma % 8 != 0 || Nb % 8 != 0 || !aligned16(a_ptr) || !aligned16(b_ptr) || !aligned16(out) || !aligned16(out2) ||
      !aligned16(workspace))
    return LEWI_ERR_SHAPE;
  if (out2 != nullptr && (Nb / 2) % 8 != 0) return LEWI_ERR_SHAPE;
  if (pad_offsets == nullptr && E != 1) return LEWI_ERR_ARG;
  RowGroupArgs r{nullptr, nullptr, nullptr, rows, E};
  const bool pair = gg::pair_mode();
  gg::Args a;
  fill_common(a, r);
  a.out = out;
  a.out2 = out2;
  a.pad_offsets = pad_offsets;
  a.N = Nb;
  a.Ma = Ma;
  a.out_f32 = out_dtype == LEWI_F32;
  const long long n_tiles = out2 ? 2LL * ((Nb / 2 + gg::BN - 1) / gg::BN) : (Nb + gg::BN - 1) / gg::BN;
  const int tm = pair ? 2 * gg::BM : gg::BM;
  const long long tiles0 = (long long)E * ((Ma + tm - 1) / tm) * n_tiles;
  cudaStream_t st = as_stream(stream);
  if (rows == 0) {
    // no rows at all: the product is all zeros
    const size_t esz = out_dtype == LEWI_F32 ? 4 : 2;
    const size_t half = out2 ? (size_t)Nb / 2 : (size_t)Nb;
    if (cudaMemsetAsync(out, 0, (size_t)E * Ma * half * esz, st) != cudaSuccess) return LEWI_ERR_CUDA;
    if (out2 && cudaMemsetAsync(out2, 0, (size_t)E * Ma * half * esz, st) != cudaSuccess) return LEWI_ERR_CUDA;
    return LEWI_OK;
  }
  int splits = 1;
  if (workspace != nullptr) {
    splits = tn_pick_splits(tiles0 * (pair ? 2 : 1), rows);
    const long long per = (long long)E * Ma * Nb * 4;
    if ((long long)splits * per > workspace_bytes) splits = (int)(workspace_bytes / per);
    if (splits < 2) splits = 1;
  }
  a.k_splits = splits;
  a.partial = splits > 1 ? reinterpret_cast<float*>(workspace) : nullptr;
  CUtensorMap ta, tb;
  if (!gg::make_map(&ta, a_ptr, (uint64_t)Ma, (uint64_t)(gather_a ? src_rows : rows), 0, 64, 64))
    return LEWI_ERR_CUDA;
  if (!gg::make_map(&tb, b_ptr, (uint64_t)Nb, (uint64_t)(gather_b ? src_rows : rows), 0, 64, 64))
    return LEWI_ERR_CUDA;
  if (gather_a || gather_b) {   // the contraction rows of that operand are picked through row_idx
    a.g_idx = row_idx;
    a.g_div = idx_div;
    a.g_src_rows = (int)src_rows;
    if (gather_a) { a.ga_ptr = a_ptr; a.ga_ld = Ma; }
    if (gather_b) { a.gb_ptr = b_ptr; a.gb_ld = Nb; }
  }
  if (int rc = gg::launch_auto<gg::TN, gg::TNOUT>(pair, st, ta, tb, tb, a, tiles0 * splits)) return rc;
  if (splits > 1) {
    const long long total4 = (long long)E * Ma * Nb / 4;
    long long grid = (total4 + 255) / 256;
    if (grid > (long long)num_sms() * 8) grid = (long long)num_sms() * 8;
    gg::tn_reduce_kernel<<<(int)grid, 256, 0, st>>>(a.partial, splits, (long long)E * Ma, Nb, out, out2, a.out_f32);
    LEWI_CHECK_LAUNCH();
  }
  return LEWI_OK;
}

int lewi_grouped_gemm_gateup_swiglu(void* stream, const void* xs, const void* w_gate, const void* w_up, void* gu,
                                    void* h, const int32_t* block_expert, const int32_t* n_blocks,
                                    const int32_t* pad_offsets, int64_t rows, int d, int f, int E) {
  return lewi_grouped_gemm_gateup_swiglu_gather(stream, xs, nullptr, 1, rows, nullptr, nullptr, w_gate, w_up, gu, h,
                                                block_expert, n_blocks, pad_offsets, rows, d, f, E);
}

int lewi_grouped_gemm_gateup_swiglu_gather(void* stream, const void* xs, const int32_t* row_idx, int idx_div,
                                           int64_t src_rows, const int32_t* scale_idx, const float* h_scale_src,
                                           const void* w_gate,
                                           const void* w_up, void* gu, void* h, const int32_t* block_expert,
                                           const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows, int d,
                                           int f, int E) {
  if (!xs || !w_gate || !w_up || !h || d <= 0 || f <= 0) return LEWI_ERR_ARG;
  if (row_idx != nullptr && (idx_div <= 0 || src_rows <= 0 || src_rows > 0x7fffffffLL)) return LEWI_ERR_ARG;
  if (scale_idx == nullptr) scale_idx = row_idx;   // still null: the scale table is indexed by the padded row itself
  RowGroupArgs r{block_expert, n_blocks, pad_offsets, rows, E};
  const bool pair = use_pair(r);
  if (int rc = check_rows(r)) return rc;
  if (d % 8 != 0 || f % 8 != 0 || !aligned16(xs) || !aligned16(w_gate) || !aligned16(w_up) || !aligned16(gu) ||
      !aligned16(h))
    return LEWI_ERR_SHAPE;
  if (rows == 0) return LEWI_OK;
  CUtensorMap ta, tb, tb2;
  if (!gg::make_map(&ta, xs, (uint64_t)d, (uint64_t)(row_idx ? src_rows : rows), 0, 64, 128))
    return LEWI_ERR_CUDA;
  if (!gg::make_map(&tb, w_gate, (uint64_t)f, (uint64_t)d, (uint64_t)E, 64, 64)) return LEWI_ERR_CUDA;
  if (!gg::make_map(&tb2, w_up, (uint64_t)f, (uint64_t)d, (uint64_t)E, 64, 64)) return LEWI_ERR_CUDA;
  gg::Args a;
  fill_common(a, r);
  if (row_idx != nullptr) {   // rows of xs are picked through row_idx instead of being materialised first
    a.ga_ptr = xs;
    a.ga_ld = d;
    a.g_idx = row_idx;
    a.g_div = idx_div;
    a.g_src_rows = (int)src_rows;
  }
  a.scale_src = h_scale_src;
  a.scale_idx = scale_idx;
  a.out = h;
  a.out2 = gu;
  a.K = d;
  a.kb_total = (d + gg::BK - 1) / gg::BK;
  a.N = f;
  const long long tiles = (long long)a.n_blocks_host * ((f + gg::BN / 2 - 1) / (gg::BN / 2));
  return gg::launch_auto<gg::NN, gg::SWIGLU>(pair, as_stream(stream), ta, tb, tb2, a, tiles);
}

int lewi_grouped_gemm_dh_dswiglu(void* stream, const void* dys, const void* w_down, const void* gu, void* dgu,
                                 const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets,
                                 int64_t rows, int d, int f, int E) {
  return lewi_grouped_gemm_dh_dswiglu_gather(stream, dys, nullptr, 1, rows, nullptr, nullptr, nullptr, w_down, gu, dgu,
                                             block_expert, n_blocks, pad_offsets, rows, d, f, E);
}

int lewi_dw_partial_parts(int f) { return f > 0 ? 2 * ((f + gg::BN - 1) / gg::BN) : LEWI_ERR_ARG; }

int lewi_grouped_gemm_dh_dswiglu_gather(void* stream, const void* dys, const int32_t* row_idx, int idx_div,
                                        int64_t src_rows, const int32_t* scale_idx, const float* scale_src,
                                        float* dw_partial,
                                        const void* w_down, const void* gu, void* dgu, const int32_t* block_expert,
                                        const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows, int d,
                                        int f, int E) {
  if (!dys || !w_down || !gu || !dgu || d <= 0 || f <= 0) return LEWI_ERR_ARG;
  if (row_idx != nullptr && (idx_div <= 0 || src_rows <= 0 || src_rows > 0x7fffffffLL)) return LEWI_ERR_ARG;
  if (scale_idx == nullptr) scale_idx = row_idx;   // still null: the scale table is indexed by the padded row itself
  RowGroupArgs r{block_expert, n_blocks, pad_offsets, rows, E};
  const bool pair = use_pair(r);
  if (int rc = check_rows(r)) return rc;
  if (d % 8 != 0 || f % 8 != 0 || !aligned16(dys) || !aligned16(w_down) || !aligned16(gu) || !aligned16(dgu))
    return LEWI_ERR_SHAPE;
  if (rows == 0) return LEWI_OK;
  CUtensorMap ta, tb;
  if (!gg::make_map(&ta, dys, (uint64_t)d, (uint64_t)(row_idx ? src_rows : rows), 0, 64, 128))
    return LEWI_ERR_CUDA;
  // w_down [E,f,d]: as the K-major B operand of dh[rows,f] = dys[rows,d] . w_down[e]^T
  if (!gg::make_map(&tb, w_down, (uint64_t)d, (uint64_t)f, (uint64_t)E, 64, pair ? 128 : 256)) return LEWI_ERR_CUDA;
  gg::Args a;
  fill_common(a, r);
  if (row_idx != nullptr) {
    a.ga_ptr = dys;
    a.ga_ld = d;
    a.g_idx = row_idx;
    a.g_div = idx_div;
    a.g_src_rows = (int)src_rows;
  }
  a.scale_src = scale_src;
  a.scale_idx = scale_idx;
  a.dw_partial = dw_partial;
  a.dw_parts = lewi_dw_partial_parts(f);
  a.out = dgu;
  a.gu = reinterpret_cast<const __nv_bfloat16*>(gu);
  a.K = d;
  a.kb_total = (d + gg::BK - 1) / gg::BK;
  a.N = f;
  // the epilogue reads g|u and writes dg|du as tiles of 32 rows x 64 columns of the [rows][2][f] tensors
  CUtensorMap tgu, tdgu;
  if (!gg::make_map(&tgu, gu, (uint64_t)f, 2, (uint64_t)rows, 64, 1, 32)) return LEWI_ERR_CUDA;
  if (!gg::make_map(&tdgu, dgu, (uint64_t)f, 2, (uint64_t)rows, 64, 1, 32)) return LEWI_ERR_CUDA;
  const long long tiles = (long long)a.n_blocks_host * ((f + gg::BN - 1) / gg::BN);
  return gg::launch_auto<gg::NT, gg::DSWIGLU>(pair, as_stream(stream), ta, tb, tb, a, tiles, &tgu, &tdgu);
}

int lewi_grouped_gemm_dx(void* stream, const void* dgu, const void* w_gate, const void* w_up, void* dxs,
                         const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets,
                         int64_t rows, int d, int f, int E) {
  if (!dgu || !w_gate || !w_up || !dxs || d <= 0 || f <= 0) return LEWI_ERR_ARG;
  RowGroupArgs r{block_expert, n_blocks, pad_offsets, rows, E};
  const bool pair = use_pair(r);
  if (int rc = check_rows(r)) return rc;
  if (d % 8 != 0 || f % 8 != 0 || !aligned16(dgu) || !aligned16(w_gate) || !aligned16(w_up) || !aligned16(dxs))
    return LEWI_ERR_SHAPE;
  if (rows == 0) return LEWI_OK;
  CUtensorMap ta, tb, tb2;
  if (!gg::make_map(&ta, dgu, (uint64_t)(2 * f), (uint64_t)rows, 0, 64, 128)) return LEWI_ERR_CUDA;
  // w_gate/w_up [E,d,f]: K-major B operands (contraction over f) of dxs[rows,d]
  if (!gg::make_map(&tb, w_gate, (uint64_t)f, (uint64_t)d, (uint64_t)E, 64, pair ? 128 : 256)) return LEWI_ERR_CUDA;
  if (!gg::make_map(&tb2, w_up, (uint64_t)f, (uint64_t)d, (uint64_t)E, 64, pair ? 128 : 256)) return LEWI_ERR_CUDA;
  gg::Args a;
  fill_common(a, r);
  a.out = dxs;
  a.K = 2 * f;
  a.N = d;
  a.kb_split = (f + gg::BK - 1) / gg::BK;
  a.k2_offset = f;
  a.kb_total = 2 * a.kb_split;
  const long long tiles = (long long)a.n_blocks_host * ((d + gg::BN - 1) / gg::BN);
  return gg::launch_auto<gg::NT, gg::PLAIN>(pair, as_stream(stream), ta, tb, tb2, a, tiles);
}

// Bring-up hook: override the shared-memory descriptor geometry (bytes).  A value of 0 keeps the
// current setting.  Not part of the drop-in surface.
// ------------------------------------------------------------------------------------------------ expert parallel

int lewi_ep_alloc(int64_t bytes, void** out_host) {
  if (bytes <= 0 || !out_host) return LEWI_ERR_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return LEWI_ERR_CUDA;
  }
  *out_host = p;
  return LEWI_OK;
}

int lewi_ep_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? LEWI_OK : LEWI_ERR_CUDA; }

int lewi_ep_ipc_export(void* ptr, void* handle64_host) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!ptr || !handle64_host) return LEWI_ERR_ARG;
  if (cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64_host), ptr) != cudaSuccess) {
    (void)cudaGetLastError();
    return LEWI_ERR_CUDA;
  }
  return LEWI_OK;
}

int lewi_ep_ipc_import(const void* handle64_host, void** out_host) {
  if (!handle64_host || !out_host) return LEWI_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64_host, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    (void)cudaGetLastError();
    return LEWI_ERR_CUDA;
  }
  *out_host = p;
  return LEWI_OK;
}

int lewi_ep_ipc_release(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? LEWI_OK : LEWI_ERR_CUDA; }

namespace {
// The exchange kernels use no shared memory; without this the SMs they run on are switched to an L1-heavy
// split, and a GEMM CTA (which needs the largest shared-memory split) could not join them until they drain.
inline void prefer_shared_carveout(const void* kern, bool* done) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || done[dev]) return;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) !=
      cudaSuccess)
    (void)cudaGetLastError();
  done[dev] = true;
}

inline bool fill_peers(PeerPtrs& pp, void* const* host, int G, bool required) {
  for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = nullptr;
  if (host == nullptr) return !required;
  for (int i = 0; i < G; ++i) {
    if (host[i] == nullptr) return false;
    pp.p[i] = host[i];
  }
  return true;
}
}  // namespace

int lewi_ep_plan(void* stream, const int32_t* counts_all, int G, int E, int me, int block, int64_t rmax_pad,
                 int32_t* dst_base, int32_t* pad_offsets, int32_t* valid_end, int32_t* n_blocks,
                 int32_t* block_expert, int32_t* recv_rows) {
  if (!counts_all || !dst_base || !pad_offsets || !valid_end || !n_blocks || !recv_rows) return LEWI_ERR_ARG;
  if (G <= 0 || G > kMaxPeers || E <= 0 || E % G != 0 || me < 0 || me >= G || block <= 0 || rmax_pad <= 0)
    return LEWI_ERR_ARG;
  if (E > kMaxExperts) return LEWI_ERR_LIMIT;
  static bool carve[64] = {false};
  prefer_shared_carveout(reinterpret_cast<const void*>(ep_plan_kernel), carve);
  ep_plan_kernel<<<1, 1024, 0, as_stream(stream)>>>(counts_all, G, E, me, block, rmax_pad, (int)(rmax_pad / block),
                                                    dst_base, pad_offsets, valid_end, n_blocks, block_expert,
                                                    recv_rows);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_ep_push_rows(void* stream, const void* x, const int32_t* order, const int32_t* flat_expert,
                      const int32_t* offsets, const int32_t* dst_base, const float* slot_w,
                      void* const* peers_rows_host, void* const* peers_w_host, void* const* peers_ret_host, int me,
                      int64_t M, int k, int d, int E, int G, int64_t rmax_pad, int64_t T, int el_lo, int el_hi,
                      int threads) {
  if (!x || !order || !flat_expert || !offsets || !dst_base || M < 0 || k <= 0 || d <= 0 || T < 0) return LEWI_ERR_ARG;
  if (G <= 0 || G > kMaxPeers || E <= 0 || E % G != 0 || me < 0 || me >= G || d % 8 != 0) return LEWI_ERR_ARG;
  if (el_lo < 0 || el_hi > E / G || el_lo > el_hi) return LEWI_ERR_ARG;
  if (M >= (1ll << kEpSlotBits)) return LEWI_ERR_LIMIT;
  if (threads == 0) threads = kEpThreads;
  if (threads < 32 || threads > kEpThreads || threads % 32 != 0) return LEWI_ERR_ARG;
  PeerPtrs rows, w, ret;
  if (!fill_peers(rows, peers_rows_host, G, true)) return LEWI_ERR_ARG;
  if (!fill_peers(w, peers_w_host, G, slot_w != nullptr)) return LEWI_ERR_ARG;
  if (!fill_peers(ret, peers_ret_host, G, false)) return LEWI_ERR_ARG;
  if (M == 0 || el_lo == el_hi) return LEWI_OK;
  static bool carve[64] = {false};
  prefer_shared_carveout(reinterpret_cast<const void*>(ep_push_rows_kernel), carve);
  ep_push_rows_kernel<<<num_sms(), threads, 0, as_stream(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), order, flat_expert, offsets, dst_base, slot_w, rows, w, ret, M, k, d, E / G,
      G, rmax_pad, T, el_lo, el_hi, me);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_ep_return_rows(void* stream, const void* rows, const float* pieces, const int32_t* ret,
                        const int32_t* pad_offsets, int el_lo, int el_hi, void* const* peers_slot_rows_host,
                        void* const* peers_slot_pieces_host, int d, int parts, int G, int64_t M, int64_t rmax_pad,
                        int threads) {
  if (!ret || !pad_offsets || (!rows && !pieces) || d <= 0 || d % 8 != 0 || G <= 0 || G > kMaxPeers || M < 0)
    return LEWI_ERR_ARG;
  if (el_lo < 0 || el_lo > el_hi || (pieces && parts <= 0)) return LEWI_ERR_ARG;
  if (threads == 0) threads = kEpThreads;
  if (threads < 32 || threads > kEpThreads || threads % 32 != 0) return LEWI_ERR_ARG;
  PeerPtrs pr, pp;
  if (!fill_peers(pr, peers_slot_rows_host, G, rows != nullptr)) return LEWI_ERR_ARG;
  if (!fill_peers(pp, peers_slot_pieces_host, G, pieces != nullptr)) return LEWI_ERR_ARG;
  if (el_lo == el_hi) return LEWI_OK;
  static bool carve[64] = {false};
  prefer_shared_carveout(reinterpret_cast<const void*>(ep_return_rows_kernel), carve);
  ep_return_rows_kernel<<<num_sms(), threads, 0, as_stream(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(rows), pieces, ret, pad_offsets, el_lo, el_hi, pr, pp, d, parts, G, M,
      rmax_pad);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_ep_zero_pad(void* stream, void* buf, int32_t* ret, const int32_t* valid_end, const int32_t* pad_offsets,
                     int E_local, int d, int64_t rmax_pad) {
  if (!buf || !valid_end || !pad_offsets || E_local <= 0 || d <= 0 || d % 8 != 0) return LEWI_ERR_ARG;
  static bool carve[64] = {false};
  prefer_shared_carveout(reinterpret_cast<const void*>(ep_zero_pad_kernel), carve);
  ep_zero_pad_kernel<<<E_local, 256, 0, as_stream(stream)>>>(reinterpret_cast<__nv_bfloat16*>(buf), ret, valid_end,
                                                             pad_offsets, d, rmax_pad);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_ep_put_i32(void* stream, const int32_t* src, void* const* peers_dst_host, int64_t dst_offset, int n, int G) {
  if (!src || n < 0 || dst_offset < 0 || G <= 0 || G > kMaxPeers) return LEWI_ERR_ARG;
  PeerPtrs pd;
  if (!fill_peers(pd, peers_dst_host, G, true)) return LEWI_ERR_ARG;
  if (n == 0) return LEWI_OK;
  static bool carve[64] = {false};
  prefer_shared_carveout(reinterpret_cast<const void*>(ep_put_i32_kernel), carve);
  ep_put_i32_kernel<<<1, 256, 0, as_stream(stream)>>>(src, pd, dst_offset, n, G);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_ep_barrier(void* stream, void* const* peers_flags_host, int32_t* my_flags, int32_t* epoch_counter, int me,
                    int G, int64_t timeout_ms) {
  if (!my_flags || !epoch_counter || G <= 0 || G > kMaxPeers || me < 0 || me >= G || timeout_ms <= 0 || timeout_ms > 10000)
    return LEWI_ERR_ARG;
  PeerPtrs pf;
  if (!fill_peers(pf, peers_flags_host, G, true)) return LEWI_ERR_ARG;
  static bool carve[64] = {false};
  prefer_shared_carveout(reinterpret_cast<const void*>(ep_barrier_kernel), carve);
  ep_barrier_kernel<<<1, 32, 0, as_stream(stream)>>>(pf, my_flags, epoch_counter, me, G,
                                                     (unsigned long long)timeout_ms * 1000000ull);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_set_sm_sharing(int on) {
  gg::sm_sharing() = on != 0;
  return LEWI_OK;
}

// Bring-up hook: 0 forces the single-CTA (cta_group::1) GEMM kernels, 1 (default) allows CTA pairs.
int lewi_debug_set_cta_pair(int on) {
  gg::pair_mode() = on != 0;
  return LEWI_OK;
}

// Bring-up hook: timing experiments that switch off parts of the GEMM kernels (results become wrong).
int lewi_debug_set_flags(int flags) {
  g_debug_flags = flags & 7;
  route_wide() = (flags & 8) != 0;
  return LEWI_OK;
}

int lewi_debug_set_desc(int k_lbo, int k_sbo, int k_step, int mn_lbo, int mn_sbo, int mn_step) {
  gg::DescGeometry& g = gg::desc_geometry();
  if (k_lbo > 0) g.k_lbo = (uint32_t)k_lbo;
  if (k_sbo > 0) g.k_sbo = (uint32_t)k_sbo;
  if (k_step > 0) g.k_step = (uint32_t)k_step;
  if (mn_lbo > 0) g.mn_lbo = (uint32_t)mn_lbo;
  if (mn_sbo > 0) g.mn_sbo = (uint32_t)mn_sbo;
  if (mn_step > 0) g.mn_step = (uint32_t)mn_step;
  return LEWI_OK;
}

}  // extern "C"
