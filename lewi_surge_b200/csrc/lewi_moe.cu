// liblewi_moe.so: C ABI over the sm_100a kernels (declarations and contracts: include/lewi_moe.h).
#include "common.cuh"
#include "ep.cuh"
#include "ep_unique.cuh"
#include "gather.cuh"
#include "grouped_gemm.cuh"
#include "moe_layer.cuh"
#include "router_gemm.cuh"
#include "routing.cuh"
#include "seqmix.cuh"
#include "seqmix_bwd.cuh"

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
                     int32_t* row_slot, float* probs_sum, float* aux_loss, void* workspace,
                     int64_t workspace_bytes) {
  if (!logits || !topk_idx || !topk_w || T < 0 || E <= 0 || k <= 0) return LEWI_ERR_ARG;
  if (k > E || k > kMaxTopK) return LEWI_ERR_LIMIT;
  if (block > 0 && (!pad_offsets || !block_expert || !n_blocks)) return LEWI_ERR_ARG;
  if (aux_loss != nullptr && probs_sum == nullptr) return LEWI_ERR_ARG;
  return route_common(as_stream(stream), logits, nullptr, T, T * k, E, k, block, topk_idx, topk_w, counts, offsets,
                      pad_offsets, block_expert, n_blocks, order, pos, pad_pos, row_slot, probs_sum, workspace,
                      workspace_bytes, aux_loss);
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
  return lewi_router_topk_bwd_full(stream, logits, topk_idx, dw, nullptr, 0, nullptr, nullptr, dlogits, dlogits_bf16, T, E,
                                   k, nullptr, 0.f, nullptr, nullptr, 0);
}

int lewi_router_topk_bwd_partial(void* stream, const float* logits, const int32_t* topk_idx, const float* dw,
                                 const float* dw_partial, int dw_parts, const int32_t* pad_pos, float* dw_out,
                                 float* dlogits, void* dlogits_bf16, int64_t T, int E, int k) {
  return lewi_router_topk_bwd_full(stream, logits, topk_idx, dw, dw_partial, dw_parts, pad_pos, dw_out, dlogits,
                                   dlogits_bf16, T, E, k, nullptr, 0.f, nullptr, nullptr, 0);
}

int64_t lewi_router_bias_grad_workspace_bytes(int64_t T, int E) {
  if (T < 0 || E <= 0) return LEWI_ERR_ARG;
  return ((int64_t)gather_grid(T > 0 ? T : 1) * E * 4 + 255) / 256 * 256;
}

int lewi_router_topk_bwd_full(void* stream, const float* logits, const int32_t* topk_idx, const float* dw,
                              const float* dw_partial, int dw_parts, const int32_t* pad_pos, float* dw_out,
                              float* dlogits, void* dlogits_bf16, int64_t T, int E, int k, const int32_t* counts,
                              float aux_grad, float* d_bias, void* workspace, int64_t workspace_bytes) {
  if (!logits || !topk_idx || (!dw && !dw_partial) || (!dlogits && !dlogits_bf16) || T < 0 || E <= 0 || k <= 0)
    return LEWI_ERR_ARG;
  if (dw_partial != nullptr && (dw_parts <= 0 || pad_pos == nullptr)) return LEWI_ERR_ARG;
  __nv_bfloat16* dlb = reinterpret_cast<__nv_bfloat16*>(dlogits_bf16);
  if (E > kMaxExperts || k > kMaxTopK || k > E) return LEWI_ERR_LIMIT;
  cudaStream_t st = as_stream(stream);
  if (T == 0) {
    if (d_bias != nullptr && cudaMemsetAsync(d_bias, 0, (size_t)E * 4, st) != cudaSuccess) return LEWI_ERR_CUDA;
    return LEWI_OK;
  }
  const int grid = gather_grid(T);
  float* bias_partial = nullptr;
  if (d_bias != nullptr) {
    if (workspace == nullptr || workspace_bytes < (int64_t)grid * E * 4) return LEWI_ERR_WORKSPACE;
    bias_partial = reinterpret_cast<float*>(workspace);
  }
  // load-balance loss E * sum_e (counts_e / M)(probs_sum_e / T): d/dp[t,e] = E * counts_e / (M * T), times aux_grad
  const float aux_coef = counts != nullptr ? aux_grad * (float)E / ((float)(T * k) * (float)T) : 0.f;
  const int32_t* cnt = (counts != nullptr && aux_grad != 0.f) ? counts : nullptr;
#define LEWI_RTB(ER)                                                                                                  \
  router_topk_bwd_kernel<ER><<<grid, 256, 0, st>>>(logits, topk_idx, dw, dw_partial, dw_parts, pad_pos, dw_out, dlogits, \
                                                   dlb, T, E, k, cnt, aux_coef, bias_partial)
  if (E <= 64) LEWI_RTB(2);
  else if (E <= 128) LEWI_RTB(4);
  else if (E <= 256) LEWI_RTB(8);
  else LEWI_RTB(16);
#undef LEWI_RTB
  LEWI_CHECK_LAUNCH();
  if (d_bias != nullptr) {
    col_sum_reduce_kernel<<<E, 256, 0, st>>>(bias_partial, grid, E, d_bias);
    LEWI_CHECK_LAUNCH();
  }
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

int lewi_dispatch_rows(void* stream, const void* x, const int32_t* pos, const int32_t* row_slot, void* out, int64_t T,
                       int k, int d, int64_t out_rows, const int32_t* n_rows_dev, int rows_per_unit) {
  if (!x || !pos || !row_slot || !out || T < 0 || k <= 0 || d <= 0 || out_rows < 0) return LEWI_ERR_ARG;
  if (k > kWarp) return LEWI_ERR_LIMIT;
  if (!aligned16(x) || !aligned16(out)) return LEWI_ERR_SHAPE;
  const int vpl = pick_vpl(d, 2);
  if (vpl == 0) return LEWI_ERR_SHAPE;
  if (out_rows == 0) return LEWI_OK;
  const int grid = gather_grid(T > out_rows / kWarp ? T : out_rows / kWarp + 1);
  cudaStream_t st = as_stream(stream);
  LEWI_DISPATCH_VPL(vpl, (dispatch_rows_kernel<VPL><<<grid, kGatherThreads, 0, st>>>(
                             reinterpret_cast<const __nv_bfloat16*>(x), pos, row_slot,
                             reinterpret_cast<__nv_bfloat16*>(out), T, k, d, out_rows, n_rows_dev, rows_per_unit)));
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
  // the CTA-pair kernels keep a per-expert prefix table in shared memory that is sized for kMaxExperts
  if (r.pad_offsets != nullptr && r.E > kMaxExperts) return LEWI_ERR_LIMIT;
  // several groups need a way to find a row block's expert: block_expert (single-CTA kernels) or
  // pad_offsets with the CTA-pair kernels; pad_offsets alone is not enough when pairs are unavailable
  if (r.E > 1 && r.block_expert == nullptr && (r.pad_offsets == nullptr || !use_pair(r))) return LEWI_ERR_SHAPE;
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
  a.r1_row = nullptr;
  a.r1_col = nullptr;
  a.tn_part_rows = 0;
  a.scale_src = nullptr;
  a.scale_idx = nullptr;
  a.dw_partial = nullptr;
  a.ret = nullptr;
  a.ret_slots = 0;
  a.ret_ranks = 0;
  for (int g = 0; g < gg::kRetRanks; ++g) a.ret_out[g] = nullptr;
  a.dw_parts = 0;
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

namespace {
// logits = [x x x] . [hi; mid; lo] on the tensor cores; w3 holds the three bf16 pieces of the f32 weight.
int router_logits_tensor(cudaStream_t st, const void* x, const void* w3, const float* bias, float* logits, int64_t T,
                         int d, int E) {
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
  CUtensorMap tc;
  if (!gg::make_out_map(&tc, logits, (uint64_t)E, (uint64_t)T, 0, true)) return LEWI_ERR_CUDA;
  const long long tiles = (long long)a.n_blocks_host * ((E + gg::BN - 1) / gg::BN);
  return gg::launch_auto<gg::NN, gg::PLAIN>(pair, st, ta, tb, tb, a, tiles, &tc);
}

inline bool router_tensor_ok(const void* x, const float* logits, int64_t T, int d, int E) {
  return d % 64 == 0 && E % 64 == 0 && aligned16(x) && aligned16(logits) && T <= 0x7fffff00LL;
}
}  // namespace

int lewi_router_logits(void* stream, const void* x, const float* w_router, const float* bias, float* logits,
                       int64_t T, int d, int E, void* workspace, int64_t workspace_bytes) {
  if (!x || !w_router || !logits || T < 0 || d <= 0 || E <= 0) return LEWI_ERR_ARG;
  if (T == 0) return LEWI_OK;
  cudaStream_t st = as_stream(stream);
  const bool tensor_path = workspace != nullptr && workspace_bytes >= (int64_t)3 * d * E * 2 && aligned16(workspace) &&
                           router_tensor_ok(x, logits, T, d, E);
  if (!tensor_path) {
    dim3 grid((unsigned)((T + kRgTile - 1) / kRgTile), (unsigned)((E + kRgTile - 1) / kRgTile));
    router_logits_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), w_router, bias, logits, T,
                                               d, E);
    LEWI_CHECK_LAUNCH();
    return LEWI_OK;
  }
  // f32 weight = hi + mid + lo (three bf16 pieces, 24 mantissa bits); x is bf16, so every product is
  // exact in f32 and the tensor cores accumulate in f32.
  __nv_bfloat16* w3 = reinterpret_cast<__nv_bfloat16*>(workspace);
  const long long n = (long long)d * E;
  long long sgrid = (n + 255) / 256;
  if (sgrid > (long long)num_sms() * 8) sgrid = (long long)num_sms() * 8;
  split3_bf16_kernel<<<(int)sgrid, 256, 0, st>>>(w_router, w3, nullptr, n);
  LEWI_CHECK_LAUNCH();
  return router_logits_tensor(st, x, w3, bias, logits, T, d, E);
}

namespace {
// Where the rows of a product go when they are not stored as a tensor (gg::SCATTER).
struct ReturnTable {
  const int32_t* ret;
  void* const* out_host;   // [ranks] device pointers (this GPU's or peers'), host array
  int ranks;
  int64_t slots;
};

inline int fill_return(gg::Args& a, const ReturnTable& rt, int row_elems) {
  if (!rt.ret || !rt.out_host || rt.ranks < 1 || rt.ranks > gg::kRetRanks || rt.slots < 0 ||
      rt.slots > (1LL << gg::kRetSlotBits))
    return LEWI_ERR_ARG;
  if (row_elems % 8 != 0) return LEWI_ERR_SHAPE;
  a.ret = rt.ret;
  a.ret_ranks = rt.ranks;
  a.ret_slots = rt.slots;
  for (int g = 0; g < gg::kRetRanks; ++g) {
    a.ret_out[g] = g < rt.ranks ? rt.out_host[g] : nullptr;
    if (g < rt.ranks && (!a.ret_out[g] || !aligned16(a.ret_out[g]))) return LEWI_ERR_ARG;
  }
  return LEWI_OK;
}

int grouped_gemm_nn_impl(void* stream, const void* a_ptr, const void* b_ptr, void* out, const float* row_scale,
                         const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows,
                         int K, int N, int E, int out_dtype, const ReturnTable* rt);
}  // namespace

int lewi_grouped_gemm_nn(void* stream, const void* a_ptr, const void* b_ptr, void* out, const float* row_scale,
                         const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows,
                         int K, int N, int E, int out_dtype) {
  if (!out) return LEWI_ERR_ARG;
  return grouped_gemm_nn_impl(stream, a_ptr, b_ptr, out, row_scale, block_expert, n_blocks, pad_offsets, rows, K, N, E,
                              out_dtype, nullptr);
}

int lewi_grouped_gemm_nn_return(void* stream, const void* a_ptr, const void* b_ptr, const int32_t* ret,
                                void* const* out_ptrs_host, int ranks, int64_t out_rows, const int32_t* block_expert,
                                const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows, int K, int N, int E) {
  const ReturnTable rt{ret, out_ptrs_host, ranks, out_rows};
  return grouped_gemm_nn_impl(stream, a_ptr, b_ptr, nullptr, nullptr, block_expert, n_blocks, pad_offsets, rows, K, N, E,
                              LEWI_BF16, &rt);
}

namespace {
int grouped_gemm_nn_impl(void* stream, const void* a_ptr, const void* b_ptr, void* out, const float* row_scale,
                         const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows,
                         int K, int N, int E, int out_dtype, const ReturnTable* rt) {
  if (!a_ptr || !b_ptr || (!out && !rt) || K <= 0 || N <= 0) return LEWI_ERR_ARG;
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
  if (rt != nullptr) {
    if (int rc = fill_return(a, *rt, N)) return rc;
    return gg::launch_auto<gg::NN, gg::SCATTER>(pair, as_stream(stream), ta, tb, tb, a, tiles);
  }
  CUtensorMap tc;
  if (!gg::make_out_map(&tc, out, (uint64_t)N, (uint64_t)rows, 0, a.out_f32 != 0)) return LEWI_ERR_CUDA;
  return gg::launch_auto<gg::NN, gg::PLAIN>(pair, as_stream(stream), ta, tb, tb, a, tiles, &tc);
}
}  // namespace

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
  CUtensorMap tc;
  if (!gg::make_out_map(&tc, out, (uint64_t)N, (uint64_t)rows, 0, a.out_f32 != 0)) return LEWI_ERR_CUDA;
  const long long tiles = (long long)a.n_blocks_host * ((N + gg::BN - 1) / gg::BN);
  return gg::launch_auto<gg::NT, gg::PLAIN>(pair, as_stream(stream), ta, tb, tb, a, tiles, &tc);
}

namespace {
// Several experts: rows per contraction part.  Twice the mean group (so balanced routing never splits an expert and
// only the heavy experts of a skewed batch are cut), a multiple of 64, at least 512.
inline int tn_part_rows(int64_t rows, int E) {
  long long r = 2 * ((rows + E - 1) / E);
  if (r < 512) r = 512;
  r = (r + gg::BK - 1) / gg::BK * gg::BK;
  return r > 0x3fffffc0LL ? 0x3fffffc0 : (int)r;
}
// Slots of `partial` the ragged split can need: parts of multi-part experts, laid out with a stride of two per extra
// part (see decode_tile), plus the run of the last such expert.
inline long long tn_ragged_slots(int64_t rows, int E) {
  const int R = tn_part_rows(rows, E);
  return 2 * (rows / R) + 2;
}
}  // namespace

int64_t lewi_grouped_gemm_tn_workspace_bytes(int64_t rows, int Ma, int Nb, int E, int split_out) {
  if (rows < 0 || Ma <= 0 || Nb <= 0 || E <= 0) return LEWI_ERR_ARG;
  if (E > 1) return (int64_t)tn_ragged_slots(rows, E) * Ma * Nb * 4;
  const long long n_tiles = split_out ? 2LL * ((Nb / 2 + gg::BN - 1) / gg::BN) : (Nb + gg::BN - 1) / gg::BN;
  const int tm = gg::pair_mode() ? 2 * gg::BM : gg::BM;
  const long long tiles0 = (long long)E * ((Ma + tm - 1) / tm) * n_tiles;
  const int s = tn_pick_splits(tiles0 * (gg::pair_mode() ? 2 : 1), rows);
  return s > 1 ? (int64_t)s * E * Ma * Nb * 4 : 0;
}

int lewi_grouped_gemm_tn(void* stream, const void* a_ptr, const void* b_ptr, void* out, void* out2,
                         const int32_t* pad_offsets, int64_t rows, int Ma, int Nb, int E, int out_dtype,
                         void* workspace, int64_t workspace_bytes) {
  if (!a_ptr || !b_ptr || !out || Ma <= 0 || Nb <= 0 || rows < 0 || E <= 0) return LEWI_ERR_ARG;
  if (out_dtype != LEWI_BF16 && out_dtype != LEWI_F32) return LEWI_ERR_ARG;
  if (rows > 0x7fffff00LL) return LEWI_ERR_LIMIT;
  if (E > kMaxExperts) return LEWI_ERR_LIMIT;
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
  const bool f32 = a.out_f32 != 0;
  const long long n_tiles = out2 ? 2LL * ((Nb / 2 + gg::BN - 1) / gg::BN) : (Nb + gg::BN - 1) / gg::BN;
  const int tm = pair ? 2 * gg::BM : gg::BM;
  const long long per_e = (long long)((Ma + tm - 1) / tm) * n_tiles;
  cudaStream_t st = as_stream(stream);
  const size_t half = out2 ? (size_t)Nb / 2 : (size_t)Nb;
  if (rows == 0) {
    // no rows at all: the product is all zeros
    const size_t esz = f32 ? 4 : 2;
    if (cudaMemsetAsync(out, 0, (size_t)E * Ma * half * esz, st) != cudaSuccess) return LEWI_ERR_CUDA;
    if (out2 && cudaMemsetAsync(out2, 0, (size_t)E * Ma * half * esz, st) != cudaSuccess) return LEWI_ERR_CUDA;
    return LEWI_OK;
  }
  const long long per_bytes = (long long)Ma * Nb * 4;
  long long max_tiles = (long long)E * per_e;
  int splits = 1, part_rows = 0;
  long long slots = 0;
  if (workspace != nullptr && E > 1) {
    // ragged split: heavy experts are cut into parts of part_rows rows, summed afterwards in part order
    const long long units = rows / tn_part_rows(rows, E) + E;
    slots = tn_ragged_slots(rows, E);
    if (slots * per_bytes <= workspace_bytes && units < 65535) {
      part_rows = tn_part_rows(rows, E);
      a.n_blocks_host = (int)units;
      max_tiles = units * per_e;
    }
  } else if (workspace != nullptr) {
    splits = tn_pick_splits(per_e * (pair ? 2 : 1), rows);
    if ((long long)splits * per_bytes > workspace_bytes) splits = (int)(workspace_bytes / per_bytes);
    if (splits < 2) splits = 1;
    slots = splits > 1 ? splits : 0;
    max_tiles = per_e * splits;
  }
  a.k_splits = splits;
  a.tn_part_rows = part_rows;
  a.partial = (splits > 1 || part_rows > 0) ? reinterpret_cast<float*>(workspace) : nullptr;
  CUtensorMap ta, tb, tp, tc, td;
  if (!gg::make_map(&ta, a_ptr, (uint64_t)Ma, (uint64_t)rows, 0, 64, 64)) return LEWI_ERR_CUDA;
  if (!gg::make_map(&tb, b_ptr, (uint64_t)Nb, (uint64_t)rows, 0, 64, 64)) return LEWI_ERR_CUDA;
  if (!gg::make_out_map(&tc, out, (uint64_t)half, (uint64_t)Ma, (uint64_t)E, f32)) return LEWI_ERR_CUDA;
  if (out2 != nullptr && !gg::make_out_map(&td, out2, (uint64_t)half, (uint64_t)Ma, (uint64_t)E, f32)) return LEWI_ERR_CUDA;
  if (a.partial != nullptr && !gg::make_out_map(&tp, a.partial, (uint64_t)Nb, (uint64_t)Ma, (uint64_t)slots, true))
    return LEWI_ERR_CUDA;
  if (int rc = gg::launch_auto<gg::TN, gg::TNOUT>(pair, st, ta, tb, a.partial ? tp : tb, a, max_tiles, &tc,
                                                   out2 ? &td : &tc))
    return rc;
  if (splits > 1) {
    const long long total4 = (long long)E * Ma * Nb / 4;
    long long grid = (total4 + 255) / 256;
    if (grid > (long long)num_sms() * 8) grid = (long long)num_sms() * 8;
    gg::tn_reduce_kernel<<<(int)grid, 256, 0, st>>>(a.partial, splits, (long long)E * Ma, Nb, out, out2, a.out_f32);
    LEWI_CHECK_LAUNCH();
  } else if (part_rows > 0) {
    long long gx = ((long long)Ma * Nb / 4 + 255) / 256;
    if (gx > 32) gx = 32;
    gg::tn_reduce_ragged_kernel<<<dim3((unsigned)gx, (unsigned)E), 256, 0, st>>>(a.partial, pad_offsets, E, part_rows, Ma, Nb,
                                                                                 out, out2, a.out_f32);
    LEWI_CHECK_LAUNCH();
  }
  return LEWI_OK;
}

int lewi_grouped_gemm_gateup_swiglu(void* stream, const void* xs, const void* w_gate, const void* w_up, void* gu,
                                    void* h, const int32_t* block_expert, const int32_t* n_blocks,
                                    const int32_t* pad_offsets, int64_t rows, int d, int f, int E) {
  return lewi_grouped_gemm_gateup_swiglu_scaled(stream, xs, nullptr, nullptr, w_gate, w_up, gu, h, block_expert, n_blocks,
                                                pad_offsets, rows, d, f, E);
}

int lewi_grouped_gemm_gateup_swiglu_scaled(void* stream, const void* xs, const int32_t* scale_idx,
                                           const float* h_scale_src, const void* w_gate, const void* w_up, void* gu,
                                           void* h, const int32_t* block_expert, const int32_t* n_blocks,
                                           const int32_t* pad_offsets, int64_t rows, int d, int f, int E) {
  if (!xs || !w_gate || !w_up || !h || d <= 0 || f <= 0) return LEWI_ERR_ARG;
  RowGroupArgs r{block_expert, n_blocks, pad_offsets, rows, E};
  if (int rc = check_rows(r)) return rc;
  const bool pair = use_pair(r);
  if (d % 8 != 0 || f % 8 != 0 || !aligned16(xs) || !aligned16(w_gate) || !aligned16(w_up) || !aligned16(gu) ||
      !aligned16(h))
    return LEWI_ERR_SHAPE;
  if (rows == 0) return LEWI_OK;
  CUtensorMap ta, tb, tb2;
  if (!gg::make_map(&ta, xs, (uint64_t)d, (uint64_t)rows, 0, 64, 128)) return LEWI_ERR_CUDA;
  if (!gg::make_map(&tb, w_gate, (uint64_t)f, (uint64_t)d, (uint64_t)E, 64, 64)) return LEWI_ERR_CUDA;
  if (!gg::make_map(&tb2, w_up, (uint64_t)f, (uint64_t)d, (uint64_t)E, 64, 64)) return LEWI_ERR_CUDA;
  gg::Args a;
  fill_common(a, r);
  a.scale_src = h_scale_src;
  a.scale_idx = scale_idx;
  a.out = h;
  a.out2 = gu;
  a.K = d;
  a.kb_total = (d + gg::BK - 1) / gg::BK;
  a.N = f;
  CUtensorMap th, tgu;
  if (!gg::make_out_map(&th, h, (uint64_t)f, (uint64_t)rows, 0, false)) return LEWI_ERR_CUDA;
  if (gu != nullptr && !gg::make_map(&tgu, gu, (uint64_t)f, 2, (uint64_t)rows, 64, 1, 32)) return LEWI_ERR_CUDA;
  const long long tiles = (long long)a.n_blocks_host * ((f + gg::BN / 2 - 1) / (gg::BN / 2));
  return gg::launch_auto<gg::NN, gg::SWIGLU>(pair, as_stream(stream), ta, tb, tb2, a, tiles, &th, gu ? &tgu : &th);
}

int lewi_grouped_gemm_dh_dswiglu(void* stream, const void* dys, const void* w_down, const void* gu, void* dgu,
                                 const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets,
                                 int64_t rows, int d, int f, int E) {
  return lewi_grouped_gemm_dh_dswiglu_scaled(stream, dys, nullptr, nullptr, nullptr, w_down, gu, dgu, block_expert,
                                             n_blocks, pad_offsets, rows, d, f, E);
}

int lewi_dw_partial_parts(int f) { return f > 0 ? 2 * ((f + gg::BN - 1) / gg::BN) : LEWI_ERR_ARG; }

int lewi_grouped_gemm_dh_dswiglu_scaled(void* stream, const void* dys, const int32_t* scale_idx, const float* scale_src,
                                        float* dw_partial, const void* w_down, const void* gu, void* dgu,
                                        const int32_t* block_expert, const int32_t* n_blocks,
                                        const int32_t* pad_offsets, int64_t rows, int d, int f, int E) {
  if (!dys || !w_down || !gu || !dgu || d <= 0 || f <= 0) return LEWI_ERR_ARG;
  RowGroupArgs r{block_expert, n_blocks, pad_offsets, rows, E};
  if (int rc = check_rows(r)) return rc;
  const bool pair = use_pair(r);
  if (d % 8 != 0 || f % 8 != 0 || !aligned16(dys) || !aligned16(w_down) || !aligned16(gu) || !aligned16(dgu))
    return LEWI_ERR_SHAPE;
  if (rows == 0) return LEWI_OK;
  CUtensorMap ta, tb;
  if (!gg::make_map(&ta, dys, (uint64_t)d, (uint64_t)rows, 0, 64, 128)) return LEWI_ERR_CUDA;
  // w_down [E,f,d]: as the K-major B operand of dh[rows,f] = dys[rows,d] . w_down[e]^T
  if (!gg::make_map(&tb, w_down, (uint64_t)d, (uint64_t)f, (uint64_t)E, 64, pair ? 128 : 256)) return LEWI_ERR_CUDA;
  gg::Args a;
  fill_common(a, r);
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

namespace {
int grouped_gemm_dx_impl(void* stream, const void* dgu, const void* w_gate, const void* w_up, void* dxs,
                         const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets,
                         int64_t rows, int d, int f, int E, const float* r1_row, const float* r1_col,
                         const ReturnTable* rt = nullptr);

// Shared expert: dxs = dgu . [Wg | Wu]^T (+ dz[t] * w_sg[c], the input gradient through the gate) for one group.
int moe_dx_rank1(void* stream, const void* dgu, const void* w_gate, const void* w_up, void* dxs, const float* dz,
                 const float* w_sg, int64_t T, int d, int fs) {
  return grouped_gemm_dx_impl(stream, dgu, w_gate, w_up, dxs, nullptr, nullptr, nullptr, T, d, fs, 1, dz,
                              dz != nullptr ? w_sg : nullptr);
}
}  // namespace

int lewi_grouped_gemm_dx(void* stream, const void* dgu, const void* w_gate, const void* w_up, void* dxs,
                         const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets,
                         int64_t rows, int d, int f, int E) {
  if (!dxs) return LEWI_ERR_ARG;
  return grouped_gemm_dx_impl(stream, dgu, w_gate, w_up, dxs, block_expert, n_blocks, pad_offsets, rows, d, f, E, nullptr,
                              nullptr);
}

int lewi_grouped_gemm_dx_return(void* stream, const void* dgu, const void* w_gate, const void* w_up, const int32_t* ret,
                                void* const* out_ptrs_host, int ranks, int64_t out_rows, const int32_t* block_expert,
                                const int32_t* n_blocks, const int32_t* pad_offsets, int64_t rows, int d, int f, int E) {
  const ReturnTable rt{ret, out_ptrs_host, ranks, out_rows};
  return grouped_gemm_dx_impl(stream, dgu, w_gate, w_up, nullptr, block_expert, n_blocks, pad_offsets, rows, d, f, E,
                              nullptr, nullptr, &rt);
}

namespace {
int grouped_gemm_dx_impl(void* stream, const void* dgu, const void* w_gate, const void* w_up, void* dxs,
                         const int32_t* block_expert, const int32_t* n_blocks, const int32_t* pad_offsets,
                         int64_t rows, int d, int f, int E, const float* r1_row, const float* r1_col,
                         const ReturnTable* rt) {
  if (!dgu || !w_gate || !w_up || (!dxs && !rt) || d <= 0 || f <= 0) return LEWI_ERR_ARG;
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
  a.r1_row = r1_row;
  a.r1_col = r1_col;
  a.K = 2 * f;
  a.N = d;
  a.kb_split = (f + gg::BK - 1) / gg::BK;
  a.k2_offset = f;
  a.kb_total = 2 * a.kb_split;
  const long long tiles = (long long)a.n_blocks_host * ((d + gg::BN - 1) / gg::BN);
  if (rt != nullptr) {
    if (int rc = fill_return(a, *rt, d)) return rc;
    return gg::launch_auto<gg::NT, gg::SCATTER>(pair, as_stream(stream), ta, tb, tb2, a, tiles);
  }
  CUtensorMap tc;
  if (!gg::make_out_map(&tc, dxs, (uint64_t)d, (uint64_t)rows, 0, false)) return LEWI_ERR_CUDA;
  return gg::launch_auto<gg::NT, gg::PLAIN>(pair, as_stream(stream), ta, tb, tb2, a, tiles, &tc);
}
}  // namespace

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

// ---- one row per (token, destination rank)

namespace {
inline bool fill_bounds(EpBounds& bd, const int32_t* bounds_host, int n_ranges, int El) {
  if (!bounds_host || n_ranges < 1 || n_ranges > kEpMaxRanges) return false;
  bd.n = n_ranges;
  for (int i = 0; i <= kEpMaxRanges; ++i) bd.b[i] = El;
  for (int i = 0; i <= n_ranges; ++i) {
    if (bounds_host[i] < 0 || bounds_host[i] > El || (i > 0 && bounds_host[i] < bounds_host[i - 1])) return false;
    bd.b[i] = bounds_host[i];
  }
  return bounds_host[0] == 0 && bounds_host[n_ranges] == El;
}
inline int unique_chunks(int64_t T) { return (int)((T + kEpUniqueChunk - 1) / kEpUniqueChunk); }
}  // namespace

int64_t lewi_ep_unique_workspace_bytes(int64_t T, int G) {
  if (T < 0 || G <= 0 || G > kMaxPeers) return LEWI_ERR_ARG;
  return (int64_t)(unique_chunks(T) > 0 ? unique_chunks(T) : 1) * G * 4;
}

int lewi_ep_unique_tables(void* stream, const int32_t* topk_idx, int64_t T, int k, int E, int G,
                          const int32_t* bounds_host, int n_ranges, int32_t* info, int32_t* uidx, int32_t* comb,
                          int32_t* ucount, void* workspace, int64_t workspace_bytes) {
  if (!topk_idx || !info || !uidx || !comb || !ucount || !workspace || T < 0 || k <= 0 || k > kMaxTopK) return LEWI_ERR_ARG;
  if (G <= 0 || G > kMaxPeers || E <= 0 || E % G != 0) return LEWI_ERR_ARG;
  if ((long long)T * G > (1LL << kEpSlotBits)) return LEWI_ERR_LIMIT;
  if (workspace_bytes < lewi_ep_unique_workspace_bytes(T, G)) return LEWI_ERR_WORKSPACE;
  EpBounds bd;
  if (!fill_bounds(bd, bounds_host, n_ranges, E / G)) return LEWI_ERR_ARG;
  cudaStream_t st = as_stream(stream);
  if (T == 0) {
    if (cudaMemsetAsync(ucount, 0, (size_t)G * 4, st) != cudaSuccess) return LEWI_ERR_CUDA;
    return LEWI_OK;
  }
  const int chunks = unique_chunks(T);
  int32_t* chunk_cnt = reinterpret_cast<int32_t*>(workspace);
  ep_unique_info_kernel<<<chunks, 256, 0, st>>>(topk_idx, T, k, E / G, G, bd, info, chunk_cnt);
  LEWI_CHECK_LAUNCH();
  ep_unique_rank_kernel<<<chunks, 256, 0, st>>>(info, chunk_cnt, T, G, uidx, comb, ucount);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_ep_unique_plan(void* stream, const int32_t* ucount_all, int G, int me, int64_t umax, int32_t* usrc_base,
                        int32_t* utotal) {
  if (!ucount_all || !usrc_base || !utotal || G <= 0 || G > kMaxPeers || me < 0 || me >= G || umax < 0) return LEWI_ERR_ARG;
  ep_unique_plan_kernel<<<1, 32, 0, as_stream(stream)>>>(ucount_all, G, me, umax, usrc_base, utotal);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_ep_unique_meta(void* stream, const int32_t* topk_idx, const float* topk_w, const int32_t* pos,
                        const int32_t* offsets, const int32_t* dst_base, const int32_t* info, const int32_t* uidx,
                        const int32_t* usrc_base, void* const* peers_w_host, void* const* peers_ret_host,
                        void* const* peers_rowu_host, void* const* peers_urows_host, void* const* peers_umeta_host,
                        void* const* peers_uret_host, int me, int64_t T, int k, int E, int G, int64_t rmax_pad,
                        int64_t umax) {
  if (!topk_idx || !topk_w || !pos || !offsets || !dst_base || !info || !uidx || !usrc_base) return LEWI_ERR_ARG;
  if (T < 0 || k <= 0 || k > kMaxTopK || G <= 0 || G > kMaxPeers || E <= 0 || E % G != 0 || me < 0 || me >= G)
    return LEWI_ERR_ARG;
  if ((long long)T * G > (1LL << kEpSlotBits) || (long long)T * k > (1LL << kEpSlotBits)) return LEWI_ERR_LIMIT;
  EpUniqueMeta a;
  if (!fill_peers(a.w, peers_w_host, G, true) || !fill_peers(a.ret, peers_ret_host, G, true) ||
      !fill_peers(a.rowu, peers_rowu_host, G, true) || !fill_peers(a.urows, peers_urows_host, G, true) ||
      !fill_peers(a.umeta, peers_umeta_host, G, true) || !fill_peers(a.uret, peers_uret_host, G, true))
    return LEWI_ERR_ARG;
  if (T == 0) return LEWI_OK;
  a.topk_idx = topk_idx; a.topk_w = topk_w; a.pos = pos; a.offsets = offsets; a.dst_base = dst_base;
  a.info = info; a.uidx = uidx; a.usrc_base = usrc_base;
  a.T = T; a.rmax = rmax_pad; a.umax = umax; a.k = k; a.El = E / G; a.G = G; a.me = me;
  long long grid = (T * G + 255) / 256;
  if (grid > (long long)num_sms() * 8) grid = (long long)num_sms() * 8;
  ep_unique_meta_kernel<<<(int)grid, 256, 0, as_stream(stream)>>>(a);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_ep_push_unique(void* stream, const void* x, const int32_t* info, const int32_t* uidx, const int32_t* usrc_base,
                        void* const* peers_ux_host, int me, int64_t T, int d, int G, int group, int64_t umax,
                        int threads) {
  if (!x || !info || !uidx || !usrc_base || T < 0 || d <= 0 || d % 8 != 0 || G <= 0 || G > kMaxPeers || me < 0 || me >= G)
    return LEWI_ERR_ARG;
  if (group >= kEpMaxRanges) return LEWI_ERR_ARG;
  if (threads == 0) threads = kEpThreads;
  if (threads < 32 || threads > kEpThreads || threads % 32 != 0) return LEWI_ERR_ARG;
  PeerPtrs ux;
  if (!fill_peers(ux, peers_ux_host, G, true)) return LEWI_ERR_ARG;
  if (T == 0) return LEWI_OK;
  static bool carve[64] = {false};
  prefer_shared_carveout(reinterpret_cast<const void*>(ep_push_unique_kernel), carve);
  ep_push_unique_kernel<<<num_sms(), threads, 0, as_stream(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(x), info, uidx,
                                                                    usrc_base, ux, T, d, G, me, group, umax);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_ep_local_rows(void* stream, const void* ux, const int32_t* rowu, const int32_t* pad_offsets, int el_lo, int el_hi,
                       void* out, int d, int64_t rmax_pad, int64_t umax) {
  if (!ux || !rowu || !pad_offsets || !out || d <= 0 || el_lo < 0 || el_lo > el_hi) return LEWI_ERR_ARG;
  const int vpl = pick_vpl(d, 2);
  if (vpl == 0 || !aligned16(ux) || !aligned16(out)) return LEWI_ERR_SHAPE;
  if (el_lo == el_hi) return LEWI_OK;
  const int grid = num_sms() * 8;
  LEWI_DISPATCH_VPL(vpl, ep_local_rows_kernel<VPL><<<grid, 256, 0, as_stream(stream)>>>(
                             reinterpret_cast<const __nv_bfloat16*>(ux), rowu, pad_offsets, el_lo, el_hi,
                             reinterpret_cast<__nv_bfloat16*>(out), d, rmax_pad, umax));
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_ep_combine_return(void* stream, const void* rows, const int32_t* urows, const int32_t* umeta,
                           const int32_t* uret, const int32_t* utotal, int group, void* const* peers_out_host, int k,
                           int d, int G, int64_t rmax_pad, int64_t out_rows, int threads) {
  if (!rows || !urows || !umeta || !uret || !utotal || k <= 0 || k > kMaxTopK || d <= 0 || d % 8 != 0 || G <= 0 ||
      G > kMaxPeers || out_rows < 0 || out_rows > (1LL << kEpSlotBits))
    return LEWI_ERR_ARG;
  if (group >= kEpMaxRanges) return LEWI_ERR_ARG;
  if (threads == 0) threads = kEpThreads;
  if (threads < 32 || threads > kEpThreads || threads % 32 != 0) return LEWI_ERR_ARG;
  PeerPtrs out;
  if (!fill_peers(out, peers_out_host, G, true)) return LEWI_ERR_ARG;
  static bool carve[64] = {false};
  prefer_shared_carveout(reinterpret_cast<const void*>(ep_combine_return_kernel), carve);
  ep_combine_return_kernel<<<num_sms(), threads, 0, as_stream(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(rows), urows, umeta, uret, utotal, group, out, k, d, G, rmax_pad, out_rows);
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


// ------------------------------------------------------------------------------------------------ sequence mixing

#define LEWI_DISPATCH_TAPS(K_VALUE, ...)                    \
  switch (K_VALUE) {                                        \
    case 1: { constexpr int KT = 1; __VA_ARGS__; } break;   \
    case 2: { constexpr int KT = 2; __VA_ARGS__; } break;   \
    case 3: { constexpr int KT = 3; __VA_ARGS__; } break;   \
    case 4: { constexpr int KT = 4; __VA_ARGS__; } break;   \
    case 5: { constexpr int KT = 5; __VA_ARGS__; } break;   \
    case 6: { constexpr int KT = 6; __VA_ARGS__; } break;   \
    case 7: { constexpr int KT = 7; __VA_ARGS__; } break;   \
    default: { constexpr int KT = 8; __VA_ARGS__; } break;  \
  }

int64_t lewi_causal_conv1d_workspace_bytes(int B, int T, int C, int K) {
  if (B <= 0 || T <= 0 || C <= 0 || K <= 0) return LEWI_ERR_ARG;
  const int64_t runs = (T + kConvRun - 1) / kConvRun;
  return ((int64_t)B * runs * K * C * 4 + 255) / 256 * 256;
}

int lewi_causal_conv1d_fwd(void* stream, const void* x, const void* w, void* y, int B, int T, int C, int K) {
  if (!x || !w || !y || B <= 0 || T <= 0 || C <= 0 || K <= 0) return LEWI_ERR_ARG;
  if (K > kConvMaxTaps) return LEWI_ERR_LIMIT;
  if (C % 8 != 0 || !aligned16(x) || !aligned16(w) || !aligned16(y)) return LEWI_ERR_SHAPE;
  const dim3 grid((unsigned)((C / 8 + kConvThreads - 1) / kConvThreads), (unsigned)((T + kConvRun - 1) / kConvRun), (unsigned)B);
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16* yb = reinterpret_cast<__nv_bfloat16*>(y);
  cudaStream_t st = as_stream(stream);
  LEWI_DISPATCH_TAPS(K, (causal_conv1d_kernel<false, KT><<<grid, kConvThreads, 0, st>>>(xb, wb, yb, B, T, C)));
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int lewi_causal_conv1d_bwd(void* stream, const void* x, const void* w, const void* g, void* dx, void* dw, int dw_dtype,
                           void* workspace, int64_t workspace_bytes, int B, int T, int C, int K) {
  if (!x || !w || !g || (!dx && !dw) || B <= 0 || T <= 0 || C <= 0 || K <= 0) return LEWI_ERR_ARG;
  if (dw_dtype != LEWI_BF16 && dw_dtype != LEWI_F32) return LEWI_ERR_ARG;
  if (K > kConvMaxTaps) return LEWI_ERR_LIMIT;
  if (C % 8 != 0 || !aligned16(x) || !aligned16(w) || !aligned16(g) || !aligned16(dx) || !aligned16(workspace))
    return LEWI_ERR_SHAPE;
  const int runs = (T + kConvRun - 1) / kConvRun;
  if (dw != nullptr && (workspace == nullptr || workspace_bytes < (int64_t)B * runs * K * C * 4)) return LEWI_ERR_WORKSPACE;
  cudaStream_t st = as_stream(stream);
  const dim3 grid((unsigned)((C / 8 + kConvThreads - 1) / kConvThreads), (unsigned)runs, (unsigned)B);
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wb = reinterpret_cast<const __nv_bfloat16*>(w);
  const __nv_bfloat16* gb = reinterpret_cast<const __nv_bfloat16*>(g);
  if (dx != nullptr) {
    __nv_bfloat16* dxb = reinterpret_cast<__nv_bfloat16*>(dx);
    LEWI_DISPATCH_TAPS(K, (causal_conv1d_kernel<true, KT><<<grid, kConvThreads, 0, st>>>(gb, wb, dxb, B, T, C)));
    LEWI_CHECK_LAUNCH();
  }
  if (dw != nullptr) {
    float* partial = reinterpret_cast<float*>(workspace);
    LEWI_DISPATCH_TAPS(K, (causal_conv1d_dw_kernel<KT><<<grid, kConvThreads, 0, st>>>(xb, gb, partial, B, T, C)));
    LEWI_CHECK_LAUNCH();
    const int n = K * C;
    conv_dw_reduce_kernel<<<(n + 255) / 256, 256, 0, st>>>(partial, B * runs, n,
                                                          dw_dtype == LEWI_BF16 ? reinterpret_cast<__nv_bfloat16*>(dw) : nullptr,
                                                          dw_dtype == LEWI_F32 ? reinterpret_cast<float*>(dw) : nullptr);
    LEWI_CHECK_LAUNCH();
  }
  return LEWI_OK;
}

int64_t lewi_gdn_chunk_workspace_bytes(int B, int S, int H, int K, int V) {
  if (B <= 0 || S <= 0 || H <= 0 || K <= 0 || V <= 0) return LEWI_ERR_ARG;
  const int64_t n = (S + kGdnChunk - 1) / kGdnChunk;
  return ((int64_t)B * n * H * gdn_chunk_ws_bytes(K, V) + 255) / 256 * 256;
}

int lewi_gdn_chunk_fwd(void* stream, const void* q, const void* k, const void* v, const float* g, const void* beta,
                       const float* h0, void* o, float* h_final, void* workspace, int64_t workspace_bytes, int B, int S,
                       int H, int K, int V) {
  if (!q || !k || !v || !g || !beta || !o || !workspace || B <= 0 || S <= 0 || H <= 0 || K <= 0 || V <= 0) return LEWI_ERR_ARG;
  if (K > kGdnMaxDim || V > 4 * kGdnMaxDim) return LEWI_ERR_LIMIT;
  if (K % 8 != 0 || V % 8 != 0) return LEWI_ERR_SHAPE;
  if (workspace_bytes < lewi_gdn_chunk_workspace_bytes(B, S, H, K, V)) return LEWI_ERR_WORKSPACE;
  GdnDims D{B, S, H, K, V, (S + kGdnChunk - 1) / kGdnChunk};
  // 64 state columns per scan CTA when 32 would need more than one wave of CTAs (and the state has that many columns)
  const long long ctas32 = (long long)B * H * ((V + 31) / 32);
  const int vb = (V % 64 == 0 && ctas32 > num_sms()) ? 64 : 32;
  const size_t smem_a = gdn_prep_smem_bytes(K, V), smem_b = gdn_scan_smem_bytes(K, vb);
  static bool attr_set[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return LEWI_ERR_CUDA;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(gdn_chunk_scan_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(gdn_chunk_scan_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) {
      (void)cudaGetLastError();
      return LEWI_ERR_CUDA;
    }
    attr_set[dev] = true;
  }
  if (smem_a > 200 * 1024 || smem_b > 200 * 1024) return LEWI_ERR_LIMIT;
  cudaStream_t st = as_stream(stream);
  const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kb = reinterpret_cast<const __nv_bfloat16*>(k);
  gdn_chunk_prep_kernel<<<dim3((unsigned)D.N, (unsigned)H, (unsigned)B), kGdnThreads, smem_a, st>>>(
      qb, kb, reinterpret_cast<const __nv_bfloat16*>(v), g, reinterpret_cast<const __nv_bfloat16*>(beta),
      reinterpret_cast<uint8_t*>(workspace), D);
  LEWI_CHECK_LAUNCH();
  const dim3 grid((unsigned)((V + vb - 1) / vb), (unsigned)H, (unsigned)B);
  if (vb == 64)
    gdn_chunk_scan_kernel<64><<<grid, kGdnThreads, smem_b, st>>>(qb, kb, reinterpret_cast<const uint8_t*>(workspace), h0,
                                                              reinterpret_cast<__nv_bfloat16*>(o), h_final, D);
  else
    gdn_chunk_scan_kernel<32><<<grid, kGdnThreads, smem_b, st>>>(qb, kb, reinterpret_cast<const uint8_t*>(workspace), h0,
                                                              reinterpret_cast<__nv_bfloat16*>(o), h_final, D);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

int64_t lewi_gdn_chunk_bwd_workspace_bytes(int B, int S, int H, int K, int V) {
  if (B <= 0 || S <= 0 || H <= 0 || K <= 0 || V <= 0) return LEWI_ERR_ARG;
  GdnDims D{B, S, H, K, V, (S + kGdnChunk - 1) / kGdnChunk};
  return gdn_bwd_ws(D).total;
}

int lewi_gdn_chunk_bwd(void* stream, const void* q, const void* k, const void* v, const float* g, const void* beta,
                       const float* h0, const void* d_o, const float* dh_final, const void* fwd_workspace,
                       int64_t fwd_workspace_bytes, void* workspace, int64_t workspace_bytes, void* dq, void* dk, void* dv,
                       float* dg, void* dbeta, float* dh0, int B, int S, int H, int K, int V) {
  if (!q || !k || !v || !g || !beta || !d_o || !fwd_workspace || !workspace || !dq || !dk || !dv || !dg || !dbeta)
    return LEWI_ERR_ARG;
  if (B <= 0 || S <= 0 || H <= 0 || K <= 0 || V <= 0) return LEWI_ERR_ARG;
  if (K > kGdnBwdMaxDim || V > kGdnBwdMaxDim) return LEWI_ERR_LIMIT;
  if (K % 8 != 0 || V % 8 != 0) return LEWI_ERR_SHAPE;
  if (fwd_workspace_bytes < lewi_gdn_chunk_workspace_bytes(B, S, H, K, V)) return LEWI_ERR_WORKSPACE;
  if (workspace_bytes < lewi_gdn_chunk_bwd_workspace_bytes(B, S, H, K, V)) return LEWI_ERR_WORKSPACE;
  GdnDims D{B, S, H, K, V, (S + kGdnChunk - 1) / kGdnChunk};
  const size_t smem_a = gdn_bwd_scan_smem_bytes(K), smem_b = gdn_bwd_chunk_smem_bytes(K, V);
  if (smem_a > 220 * 1024 || smem_b > 220 * 1024) return LEWI_ERR_LIMIT;
  static bool attr_set[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return LEWI_ERR_CUDA;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gdn_bwd_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(gdn_bwd_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess) {
      (void)cudaGetLastError();
      return LEWI_ERR_CUDA;
    }
    attr_set[dev] = true;
  }
  cudaStream_t st = as_stream(stream);
  const __nv_bfloat16* qb = reinterpret_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kb = reinterpret_cast<const __nv_bfloat16*>(k);
  const uint8_t* fws = reinterpret_cast<const uint8_t*>(fwd_workspace);
  uint8_t* bws = reinterpret_cast<uint8_t*>(workspace);
  (void)g;   // the forward workspace holds the cumulative decay of every chunk
  gdn_bwd_scan_kernel<<<dim3((unsigned)((V + kGdnBwdVB - 1) / kGdnBwdVB), (unsigned)H, (unsigned)B), kGdnThreads, smem_a, st>>>(
      qb, kb, fws, h0, reinterpret_cast<const __nv_bfloat16*>(d_o), dh_final, bws, dh0, D);
  LEWI_CHECK_LAUNCH();
  gdn_bwd_chunk_kernel<<<dim3((unsigned)D.N, (unsigned)H, (unsigned)B), kGdnThreads, smem_b, st>>>(
      qb, kb, reinterpret_cast<const __nv_bfloat16*>(v), reinterpret_cast<const __nv_bfloat16*>(beta), fws, bws,
      reinterpret_cast<__nv_bfloat16*>(dq), reinterpret_cast<__nv_bfloat16*>(dk), reinterpret_cast<__nv_bfloat16*>(dv), dg,
      reinterpret_cast<__nv_bfloat16*>(dbeta), D);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

// ------------------------------------------------------------------------------------------------ whole layer

int64_t lewi_moe_residual_layout(int64_t T, int d, int E, int f, int k, int fs, int has_gate, int64_t* offsets_host) {
  moe::Dims D;
  if (!moe::make_dims(D, T, d, E, f, k, fs, has_gate)) return LEWI_ERR_ARG;
  int64_t off[LEWI_MOE_RES_COUNT + 1];
  moe::residual_layout(D, off);
  if (offsets_host != nullptr) memcpy(offsets_host, off, sizeof(off));
  return off[LEWI_MOE_RES_COUNT];
}

int64_t lewi_moe_workspace_bytes(int64_t T, int d, int E, int f, int k, int fs, int has_gate) {
  moe::Dims D;
  if (!moe::make_dims(D, T, d, E, f, k, fs, has_gate)) return LEWI_ERR_ARG;
  moe::Workspace W;
  moe::workspace_layout(D, W);
  return W.total;
}

int lewi_moe_set_mark_callback(void (*fn)(const char*, void*)) {
  moe::mark_fn() = fn;
  return LEWI_OK;
}

int64_t lewi_moe_router_prepared_bytes(int d, int E) {
  if (d <= 0 || E <= 0) return LEWI_ERR_ARG;
  return (int64_t)4 * d * E * 2;
}

int lewi_moe_prepare_router(void* stream, const float* w_router, void* prepared, int d, int E) {
  if (!w_router || !prepared || d <= 0 || E <= 0) return LEWI_ERR_ARG;
  __nv_bfloat16* w3 = reinterpret_cast<__nv_bfloat16*>(prepared);
  const long long n = (long long)d * E;
  long long sgrid = (n + 255) / 256;
  if (sgrid > (long long)num_sms() * 8) sgrid = (long long)num_sms() * 8;
  split3_bf16_kernel<<<(int)sgrid, 256, 0, as_stream(stream)>>>(w_router, w3, w3 + 3 * n, n);
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

#define LEWI_TRY(call)            \
  do {                            \
    const int rc_ = (call);       \
    if (rc_ != LEWI_OK) return rc_; \
  } while (0)

int lewi_moe_fwd(void* stream, void* side_stream, const void* x, const float* w_router, const float* router_bias,
                 const void* router_prepared, const void* w_gate, const void* w_up, const void* w_down,
                 const void* ws_gate, const void* ws_up, const void* ws_down, const float* w_sg, void* out,
                 float* aux_loss, void* residual, int64_t residual_bytes, void* workspace, int64_t workspace_bytes,
                 int64_t T, int d, int E, int f, int k, int fs) {
  if (!x || !w_router || !w_gate || !w_up || !w_down || !out || !residual || !workspace) return LEWI_ERR_ARG;
  if (fs > 0 && (!ws_gate || !ws_up || !ws_down)) return LEWI_ERR_ARG;
  if (fs == 0 && w_sg != nullptr) return LEWI_ERR_ARG;
  moe::Dims D;
  if (!moe::make_dims(D, T, d, E, f, k, fs, w_sg != nullptr)) return LEWI_ERR_ARG;
  if (E > kMaxExperts || k > kMaxTopK || k > E) return LEWI_ERR_LIMIT;
  if (d % 8 != 0 || f % 8 != 0 || fs % 8 != 0 || !aligned16(residual) || !aligned16(workspace)) return LEWI_ERR_SHAPE;
  int64_t ro[LEWI_MOE_RES_COUNT + 1];
  moe::residual_layout(D, ro);
  moe::Workspace W;
  moe::workspace_layout(D, W);
  if (residual_bytes < ro[LEWI_MOE_RES_COUNT] || workspace_bytes < W.total) return LEWI_ERR_WORKSPACE;
  if (T == 0) return LEWI_OK;
  uint8_t* R = reinterpret_cast<uint8_t*>(residual);
  uint8_t* Wk = reinterpret_cast<uint8_t*>(workspace);
  auto res = [&](int i) { return R + ro[i]; };
  cudaStream_t st = as_stream(stream), sd = as_stream(side_stream);
  const bool shared = fs > 0;
  const bool fork = shared && side_stream != nullptr && side_stream != stream;
  moe::Events* ev = fork ? moe::events() : nullptr;
  if (fork && ev == nullptr) return LEWI_ERR_CUDA;
  void* sh_stream = fork ? side_stream : stream;

  float* logits = reinterpret_cast<float*>(res(LEWI_MOE_RES_LOGITS));
  int32_t* topk_idx = reinterpret_cast<int32_t*>(res(LEWI_MOE_RES_TOPK_IDX));
  float* topk_w = reinterpret_cast<float*>(res(LEWI_MOE_RES_TOPK_W));
  int32_t* pad_offsets = reinterpret_cast<int32_t*>(res(LEWI_MOE_RES_PAD_OFFSETS));
  int32_t* block_expert = reinterpret_cast<int32_t*>(res(LEWI_MOE_RES_BLOCK_EXPERT));
  int32_t* n_blocks = reinterpret_cast<int32_t*>(res(LEWI_MOE_RES_N_BLOCKS));
  int32_t* pad_pos = reinterpret_cast<int32_t*>(res(LEWI_MOE_RES_PAD_POS));
  int32_t* row_slot = reinterpret_cast<int32_t*>(res(LEWI_MOE_RES_ROW_SLOT));
  float* gate = D.gate ? reinterpret_cast<float*>(res(LEWI_MOE_RES_GATE)) : nullptr;
  void* ysh = shared ? Wk + W.ysh : nullptr;

  // the shared expert needs only x: on the side stream it runs beside the memory-bound routing and dispatch
  if (fork) {
    if (cudaEventRecord(ev->fork_fwd, st) != cudaSuccess || cudaStreamWaitEvent(sd, ev->fork_fwd, 0) != cudaSuccess)
      return LEWI_ERR_CUDA;
    moe::mark("side_begin", sh_stream);
  }
  auto shared_fwd = [&]() -> int {
    if (D.gate) {
      moe::shared_gate_fwd_kernel<<<gather_grid(T), 256, 0, as_stream(sh_stream)>>>(
          reinterpret_cast<const __nv_bfloat16*>(x), w_sg, gate, T, d);
      LEWI_CHECK_LAUNCH();
      moe::mark("shared_gate", sh_stream);
    }
    // with a gate, hs (and so the shared output) is stored already multiplied by it
    LEWI_TRY(lewi_grouped_gemm_gateup_swiglu_scaled(sh_stream, x, nullptr, gate, ws_gate, ws_up, res(LEWI_MOE_RES_GUS),
                                                    res(LEWI_MOE_RES_HS), nullptr, nullptr, nullptr, T, d, fs, 1));
    moe::mark("shared_gateup_swiglu", sh_stream);
    LEWI_TRY(lewi_grouped_gemm_nn(sh_stream, res(LEWI_MOE_RES_HS), ws_down, ysh, nullptr, nullptr, nullptr, nullptr, T, fs,
                                  d, 1, LEWI_BF16));
    moe::mark("shared_down", sh_stream);
    return LEWI_OK;
  };
  if (shared && fork) LEWI_TRY(shared_fwd());

  // router
  const bool tensor_router = router_tensor_ok(x, logits, T, d, E);
  if (tensor_router) {
    const void* w3 = router_prepared;
    if (w3 == nullptr) {
      LEWI_TRY(lewi_moe_prepare_router(stream, w_router, Wk + W.w3, d, E));
      w3 = Wk + W.w3;
    }
    LEWI_TRY(router_logits_tensor(st, x, w3, router_bias, logits, T, d, E));
  } else {
    LEWI_TRY(lewi_router_logits(stream, x, w_router, router_bias, logits, T, d, E, nullptr, 0));
  }
  moe::mark("router_logits", stream);
  {
  moe::Range nvtx_sort("moe_permute_sort");
  LEWI_TRY(lewi_router_topk(stream, logits, T, E, k, moe::kBlock, topk_idx, topk_w,
                            reinterpret_cast<int32_t*>(res(LEWI_MOE_RES_COUNTS)),
                            reinterpret_cast<int32_t*>(res(LEWI_MOE_RES_OFFSETS)), pad_offsets, block_expert, n_blocks,
                            reinterpret_cast<int32_t*>(res(LEWI_MOE_RES_ORDER)),
                            reinterpret_cast<int32_t*>(res(LEWI_MOE_RES_POS)), pad_pos, row_slot,
                            reinterpret_cast<float*>(res(LEWI_MOE_RES_PROBS_SUM)), aux_loss, Wk + W.route,
                            lewi_route_workspace_bytes(D.M, E)));
  moe::mark("router_topk", stream);
  }
  {
  // dispatch: padded row r holds token row_slot[r] / k (zero row where row_slot[r] < 0), written in token order
  moe::Range nvtx_dispatch("moe_permute_dispatch");
  LEWI_TRY(lewi_dispatch_rows(stream, x, pad_pos, row_slot, res(LEWI_MOE_RES_XS), T, k, d, D.Mpad, n_blocks, moe::kBlock));
  moe::mark("dispatch_gather", stream);
  }
  // h carries the router weight of its row, so the down projection yields weighted outputs
  LEWI_TRY(lewi_grouped_gemm_gateup_swiglu_scaled(stream, res(LEWI_MOE_RES_XS), row_slot, topk_w, w_gate, w_up,
                                                  res(LEWI_MOE_RES_GU), res(LEWI_MOE_RES_H), block_expert, n_blocks,
                                                  pad_offsets, D.Mpad, d, f, E));
  moe::mark("gemm_gateup_swiglu", stream);
  LEWI_TRY(lewi_grouped_gemm_nn(stream, res(LEWI_MOE_RES_H), w_down, Wk + W.ys, nullptr, block_expert, n_blocks,
                                pad_offsets, D.Mpad, f, d, E, LEWI_BF16));
  moe::mark("gemm_down", stream);
  if (shared && !fork) LEWI_TRY(shared_fwd());
  if (fork) {
    if (cudaEventRecord(ev->join_fwd, sd) != cudaSuccess || cudaStreamWaitEvent(st, ev->join_fwd, 0) != cudaSuccess)
      return LEWI_ERR_CUDA;
  }
  // combine: out[t] = sum_j ys[pad_pos[t,j]] + shared[t]
  moe::Range nvtx_combine("moe_permute_combine");
  LEWI_TRY(lewi_gather_reduce(stream, Wk + W.ys, pad_pos, nullptr, ysh, nullptr, out, T, k, d, LEWI_BF16, LEWI_BF16,
                              D.Mpad));
  moe::mark("combine_gather_reduce", stream);
  return LEWI_OK;
}

int lewi_moe_bwd(void* stream, void* side_stream, const void* dout, const void* x, const float* w_router,
                 const void* router_prepared, const void* w_gate, const void* w_up, const void* w_down,
                 const void* ws_gate, const void* ws_up, const void* ws_down, const float* w_sg, const void* residual,
                 int64_t residual_bytes, void* workspace, int64_t workspace_bytes, void* dx, float* dw_router,
                 float* d_router_bias, void* dw_gate, void* dw_up, void* dw_down, void* dws_gate, void* dws_up,
                 void* dws_down, float* dw_sg, float* dw_topk, float aux_grad, int wgrad_dtype, int64_t T, int d, int E,
                 int f, int k, int fs) {
  if (!dout || !x || !w_router || !w_gate || !w_up || !w_down || !residual || !workspace) return LEWI_ERR_ARG;
  if (!dx || !dw_router || !dw_gate || !dw_up || !dw_down) return LEWI_ERR_ARG;
  if (fs > 0 && (!ws_gate || !ws_up || !ws_down || !dws_gate || !dws_up || !dws_down)) return LEWI_ERR_ARG;
  if ((w_sg != nullptr) != (dw_sg != nullptr) || (fs == 0 && w_sg != nullptr)) return LEWI_ERR_ARG;
  if (wgrad_dtype != LEWI_BF16 && wgrad_dtype != LEWI_F32) return LEWI_ERR_ARG;
  moe::Dims D;
  if (!moe::make_dims(D, T, d, E, f, k, fs, w_sg != nullptr)) return LEWI_ERR_ARG;
  if (E > kMaxExperts || k > kMaxTopK || k > E) return LEWI_ERR_LIMIT;
  if (d % 8 != 0 || f % 8 != 0 || fs % 8 != 0 || E % 8 != 0 || !aligned16(residual) || !aligned16(workspace))
    return LEWI_ERR_SHAPE;
  int64_t ro[LEWI_MOE_RES_COUNT + 1];
  moe::residual_layout(D, ro);
  moe::Workspace W;
  moe::workspace_layout(D, W);
  if (residual_bytes < ro[LEWI_MOE_RES_COUNT] || workspace_bytes < W.total) return LEWI_ERR_WORKSPACE;
  cudaStream_t st = as_stream(stream), sd = as_stream(side_stream);
  const size_t wsz = wgrad_dtype == LEWI_F32 ? 4 : 2;
  if (T == 0) {   // no tokens: every weight gradient is zero
    if (cudaMemsetAsync(dw_router, 0, (size_t)d * E * 4, st) != cudaSuccess ||
        cudaMemsetAsync(dw_gate, 0, (size_t)E * d * f * wsz, st) != cudaSuccess ||
        cudaMemsetAsync(dw_up, 0, (size_t)E * d * f * wsz, st) != cudaSuccess ||
        cudaMemsetAsync(dw_down, 0, (size_t)E * d * f * wsz, st) != cudaSuccess)
      return LEWI_ERR_CUDA;
    if (fs > 0 && (cudaMemsetAsync(dws_gate, 0, (size_t)d * fs * wsz, st) != cudaSuccess ||
                   cudaMemsetAsync(dws_up, 0, (size_t)d * fs * wsz, st) != cudaSuccess ||
                   cudaMemsetAsync(dws_down, 0, (size_t)d * fs * wsz, st) != cudaSuccess))
      return LEWI_ERR_CUDA;
    if (dw_sg && cudaMemsetAsync(dw_sg, 0, (size_t)d * 4, st) != cudaSuccess) return LEWI_ERR_CUDA;
    if (d_router_bias && cudaMemsetAsync(d_router_bias, 0, (size_t)E * 4, st) != cudaSuccess) return LEWI_ERR_CUDA;
    return LEWI_OK;
  }
  const uint8_t* R = reinterpret_cast<const uint8_t*>(residual);
  uint8_t* Wk = reinterpret_cast<uint8_t*>(workspace);
  auto res = [&](int i) { return R + ro[i]; };
  const bool shared = fs > 0;
  // the side stream takes the shared expert and, once dH has left the routing-weight gradient pieces, the router
  const bool fork = side_stream != nullptr && side_stream != stream;
  moe::Events* ev = fork ? moe::events() : nullptr;
  if (fork && ev == nullptr) return LEWI_ERR_CUDA;
  void* sh_stream = fork ? side_stream : stream;

  const float* logits = reinterpret_cast<const float*>(res(LEWI_MOE_RES_LOGITS));
  const int32_t* topk_idx = reinterpret_cast<const int32_t*>(res(LEWI_MOE_RES_TOPK_IDX));
  const float* topk_w = reinterpret_cast<const float*>(res(LEWI_MOE_RES_TOPK_W));
  const int32_t* counts = reinterpret_cast<const int32_t*>(res(LEWI_MOE_RES_COUNTS));
  const int32_t* pad_offsets = reinterpret_cast<const int32_t*>(res(LEWI_MOE_RES_PAD_OFFSETS));
  const int32_t* block_expert = reinterpret_cast<const int32_t*>(res(LEWI_MOE_RES_BLOCK_EXPERT));
  const int32_t* n_blocks = reinterpret_cast<const int32_t*>(res(LEWI_MOE_RES_N_BLOCKS));
  const int32_t* pad_pos = reinterpret_cast<const int32_t*>(res(LEWI_MOE_RES_PAD_POS));
  const int32_t* row_slot = reinterpret_cast<const int32_t*>(res(LEWI_MOE_RES_ROW_SLOT));
  const float* gate = D.gate ? reinterpret_cast<const float*>(res(LEWI_MOE_RES_GATE)) : nullptr;
  void* dxsh = shared ? Wk + W.dxsh : nullptr;
  float* dz = D.gate ? reinterpret_cast<float*>(Wk + W.dz) : nullptr;

  // shared expert backward: needs only dout, x and its own saved activations
  if (fork) {
    if (cudaEventRecord(ev->fork_bwd, st) != cudaSuccess || cudaStreamWaitEvent(sd, ev->fork_bwd, 0) != cudaSuccess)
      return LEWI_ERR_CUDA;
    moe::mark("side_begin", sh_stream);
  }
  auto shared_bwd = [&]() -> int {
    float* dwps = D.gate ? reinterpret_cast<float*>(Wk + W.dwps) : nullptr;
    // dh is scaled by the gate; the epilogue also leaves <dout[t], ungated shared output[t]> in pieces
    LEWI_TRY(lewi_grouped_gemm_dh_dswiglu_scaled(sh_stream, dout, nullptr, gate, dwps, ws_down, res(LEWI_MOE_RES_GUS),
                                                 Wk + W.dgus, nullptr, nullptr, nullptr, T, d, fs, 1));
    moe::mark("shared_dh_dswiglu", sh_stream);
    if (D.gate) {
      float* partial = reinterpret_cast<float*>(Wk + W.colsum);
      const int nparts = moe::colsum_parts(T);
      moe::shared_gate_bwd_kernel<<<nparts, 256, 0, as_stream(sh_stream)>>>(
          reinterpret_cast<const __nv_bfloat16*>(x), dwps, D.parts_s, gate, dz, partial, T, d);
      LEWI_CHECK_LAUNCH();
      col_sum_reduce_kernel<<<d, 256, 0, as_stream(sh_stream)>>>(partial, nparts, d, dw_sg);
      LEWI_CHECK_LAUNCH();
      moe::mark("shared_gate_bwd", sh_stream);
    }
    LEWI_TRY(lewi_grouped_gemm_tn(sh_stream, res(LEWI_MOE_RES_HS), dout, dws_down, nullptr, nullptr, T, fs, d, 1,
                                  wgrad_dtype, W.tn_s_bytes > 0 ? Wk + W.tn_s : nullptr, W.tn_s_bytes));
    moe::mark("shared_dw_down", sh_stream);
    LEWI_TRY(moe_dx_rank1(sh_stream, Wk + W.dgus, ws_gate, ws_up, dxsh, dz, w_sg, T, d, fs));
    moe::mark("shared_dx", sh_stream);
    LEWI_TRY(lewi_grouped_gemm_tn(sh_stream, x, Wk + W.dgus, dws_gate, dws_up, nullptr, T, d, 2 * fs, 1, wgrad_dtype,
                                  W.tn_s_bytes > 0 ? Wk + W.tn_s : nullptr, W.tn_s_bytes));
    moe::mark("shared_dw_gateup", sh_stream);
    return LEWI_OK;
  };
  if (shared && fork) LEWI_TRY(shared_bwd());

  // combine backward: dout rows into padded order (the same dispatch); the router weight scales dh in the dH epilogue,
  // which also emits the pieces of the routing-weight gradient <dout[t], y[row]>
  LEWI_TRY(lewi_dispatch_rows(stream, dout, pad_pos, row_slot, Wk + W.dys, T, k, d, D.Mpad, n_blocks, moe::kBlock));
  moe::mark("combine_bwd_gather", stream);
  LEWI_TRY(lewi_grouped_gemm_dh_dswiglu_scaled(stream, Wk + W.dys, row_slot, topk_w, reinterpret_cast<float*>(Wk + W.dwp),
                                               w_down, res(LEWI_MOE_RES_GU), Wk + W.dgu, block_expert, n_blocks, pad_offsets,
                                               D.Mpad, d, f, E));
  moe::mark("gemm_dh_dswiglu", stream);
  // Router backward: three small launches that need the pieces dH left behind and nothing else of the routed experts.
  // On the side stream they run beside the three big GEMMs below instead of after them.
  auto router_bwd = [&]() -> int {
    LEWI_TRY(lewi_router_topk_bwd_full(sh_stream, logits, topk_idx, nullptr, reinterpret_cast<const float*>(Wk + W.dwp),
                                       D.parts, pad_pos, dw_topk, nullptr, Wk + W.dlb, T, E, k, counts, aux_grad,
                                       d_router_bias, Wk + W.bias, W.bias_bytes));
    moe::mark("router_topk_bwd", sh_stream);
    const __nv_bfloat16* w_r_bf16 = reinterpret_cast<const __nv_bfloat16*>(router_prepared);
    if (w_r_bf16 == nullptr) {
      LEWI_TRY(lewi_cast_f32_to_bf16(sh_stream, w_router, Wk + W.w3, (int64_t)d * E));
      w_r_bf16 = reinterpret_cast<const __nv_bfloat16*>(Wk + W.w3);
    } else {
      w_r_bf16 += (size_t)3 * d * E;
    }
    // dx_r [T,d] = dlogits . W_r^T  (W_r [d,E] is the K-major operand over E)
    LEWI_TRY(lewi_grouped_gemm_nt(sh_stream, Wk + W.dlb, w_r_bf16, Wk + W.dx_r, nullptr, nullptr, nullptr, nullptr, T, E, d,
                                  1, LEWI_BF16));
    moe::mark("router_dx", sh_stream);
    // dW_r [d,E] = x^T . dlogits
    LEWI_TRY(lewi_grouped_gemm_tn(sh_stream, x, Wk + W.dlb, dw_router, nullptr, nullptr, T, d, E, 1, LEWI_F32,
                                  W.tn_r_bytes > 0 ? Wk + W.tn_r : nullptr, W.tn_r_bytes));
    moe::mark("router_dw", sh_stream);
    return LEWI_OK;
  };
  if (fork) {
    if (cudaEventRecord(ev->dh_done, st) != cudaSuccess || cudaStreamWaitEvent(sd, ev->dh_done, 0) != cudaSuccess)
      return LEWI_ERR_CUDA;
    LEWI_TRY(router_bwd());
  }
  LEWI_TRY(lewi_grouped_gemm_tn(stream, res(LEWI_MOE_RES_H), Wk + W.dys, dw_down, nullptr, pad_offsets, D.Mpad, f, d, E,
                                wgrad_dtype, W.tn_e_bytes > 0 ? Wk + W.tn_e : nullptr, W.tn_e_bytes));
  moe::mark("gemm_dw_down", stream);
  LEWI_TRY(lewi_grouped_gemm_dx(stream, Wk + W.dgu, w_gate, w_up, Wk + W.dxs, block_expert, n_blocks, pad_offsets, D.Mpad,
                                d, f, E));
  moe::mark("gemm_dx", stream);
  LEWI_TRY(lewi_grouped_gemm_tn(stream, res(LEWI_MOE_RES_XS), Wk + W.dgu, dw_gate, dw_up, pad_offsets, D.Mpad, d, 2 * f, E,
                                wgrad_dtype, W.tn_e_bytes > 0 ? Wk + W.tn_e : nullptr, W.tn_e_bytes));
  moe::mark("gemm_dw_gateup", stream);
  if (!fork) {
    LEWI_TRY(router_bwd());
    if (shared) LEWI_TRY(shared_bwd());
  }
  if (fork) {
    if (cudaEventRecord(ev->join_bwd, sd) != cudaSuccess || cudaStreamWaitEvent(st, ev->join_bwd, 0) != cudaSuccess)
      return LEWI_ERR_CUDA;
  }
  // dispatch backward: dx[t] = sum_j dxs[pad_pos[t,j]] + shared-expert and router terms
  LEWI_TRY(lewi_gather_reduce(stream, Wk + W.dxs, pad_pos, nullptr, dxsh, Wk + W.dx_r, dx, T, k, d, LEWI_BF16, LEWI_BF16,
                              D.Mpad));
  moe::mark("dispatch_bwd_gather_reduce", stream);
  return LEWI_OK;
}

int lewi_set_gemm_cta_limit(int n) {
  if (n < 0 || n == 1) return LEWI_ERR_ARG;
  gg::cta_limit() = n;
  return LEWI_OK;
}

// A/B switch: 0 forces the single-CTA (cta_group::1) GEMM kernels, 1 (default) allows CTA pairs.
int lewi_set_cta_pair(int on) {
  gg::pair_mode() = on != 0;
  return LEWI_OK;
}

}  // extern "C"
