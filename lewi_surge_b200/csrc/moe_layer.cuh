// The whole MoE layer behind two entry points: lewi_moe_fwd / lewi_moe_bwd queue the complete launch sequence
// (router, dispatch, SwiGLU expert GEMMs, shared expert, combine and every gradient) on the caller's stream(s).
// The caller owns the output, one residual buffer (what the backward pass needs from the forward pass) and one
// workspace (transient); nothing is allocated and the host is never synchronised, so both calls can be captured
// into a CUDA graph.  The sequence replaces, in the reference, router -> `_route_activations` -> three
// `ragged_dot`s -> `unpermute` (modal/moe_permute.py:399-433, modal/padded_gmm.py:45-69) and their gradients.
#pragma once

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"
#include "gather.cuh"

namespace lewi {
namespace moe {

constexpr int kBlock = 128;

inline int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

struct Dims {
  int64_t T;
  int d, E, f, k, fs;
  bool gate;
  int64_t M, Mpad;
  int parts, parts_s;
};

inline bool make_dims(Dims& D, int64_t T, int d, int E, int f, int k, int fs, int has_gate) {
  if (T < 0 || d <= 0 || E <= 0 || f <= 0 || k <= 0 || fs < 0) return false;
  D.T = T; D.d = d; D.E = E; D.f = f; D.k = k; D.fs = fs;
  D.gate = has_gate != 0 && fs > 0;
  D.M = T * k;
  D.Mpad = lewi_padded_rows_bound(D.M, E, kBlock);
  D.parts = lewi_dw_partial_parts(f);
  D.parts_s = fs > 0 ? lewi_dw_partial_parts(fs) : 0;
  return true;
}

// Residual buffer: item i lives at byte offset off[i]; off[LEWI_MOE_RES_COUNT] is the total size.
inline void residual_layout(const Dims& D, int64_t* off) {
  int64_t sz[LEWI_MOE_RES_COUNT];
  const int64_t nb = D.Mpad / kBlock > 0 ? D.Mpad / kBlock : 1;
  sz[LEWI_MOE_RES_LOGITS] = D.T * D.E * 4;
  sz[LEWI_MOE_RES_TOPK_IDX] = D.M * 4;
  sz[LEWI_MOE_RES_TOPK_W] = D.M * 4;
  sz[LEWI_MOE_RES_COUNTS] = (int64_t)D.E * 4;
  sz[LEWI_MOE_RES_OFFSETS] = (int64_t)(D.E + 1) * 4;
  sz[LEWI_MOE_RES_PAD_OFFSETS] = (int64_t)(D.E + 1) * 4;
  sz[LEWI_MOE_RES_N_BLOCKS] = 4;
  sz[LEWI_MOE_RES_PROBS_SUM] = (int64_t)D.E * 4;
  sz[LEWI_MOE_RES_BLOCK_EXPERT] = nb * 4;
  sz[LEWI_MOE_RES_ORDER] = D.M * 4;
  sz[LEWI_MOE_RES_POS] = D.M * 4;
  sz[LEWI_MOE_RES_PAD_POS] = D.M * 4;
  sz[LEWI_MOE_RES_ROW_SLOT] = D.Mpad * 4;
  sz[LEWI_MOE_RES_XS] = D.Mpad * D.d * 2;
  sz[LEWI_MOE_RES_GU] = D.Mpad * 2 * D.f * 2;
  sz[LEWI_MOE_RES_H] = D.Mpad * D.f * 2;
  sz[LEWI_MOE_RES_GUS] = D.T * 2 * D.fs * 2;
  sz[LEWI_MOE_RES_HS] = D.T * D.fs * 2;
  sz[LEWI_MOE_RES_GATE] = D.gate ? D.T * 4 : 0;
  int64_t run = 0;
  for (int i = 0; i < LEWI_MOE_RES_COUNT; ++i) {
    off[i] = run;
    run += align256(sz[i]);
  }
  off[LEWI_MOE_RES_COUNT] = run;
}

// Workspace: transient buffers of one forward or one backward call (the two share the space).
struct Workspace {
  int64_t w3, route, ys, ysh;                                               // forward
  int64_t dys, dgu, dxs, dwp, dlb, dx_r, dgus, dwps, dxsh, dz, colsum;      // backward
  int64_t tn_e, tn_e_bytes, tn_s, tn_s_bytes, tn_r, tn_r_bytes, bias, bias_bytes;
  int64_t total;
};

inline int colsum_parts(int64_t T) { return (int)((T + 127) / 128); }

inline void workspace_layout(const Dims& D, Workspace& W) {
  int64_t run = 0;
  auto take = [&](int64_t bytes) {
    const int64_t at = run;
    run += align256(bytes > 0 ? bytes : 0);
    return at;
  };
  W.w3 = take((int64_t)4 * D.d * D.E * 2);   // three split pieces + the rounded bf16 copy of the router weight
  const int64_t fwd0 = run;
  W.route = take(lewi_route_workspace_bytes(D.M, D.E));
  W.ys = take(D.Mpad * D.d * 2);
  W.ysh = take(D.T * D.d * 2);
  const int64_t fwd_end = run;
  run = fwd0;
  W.dys = take(D.Mpad * D.d * 2);
  W.dgu = take(D.Mpad * 2 * D.f * 2);
  W.dxs = take(D.Mpad * D.d * 2);
  W.dwp = take(D.Mpad * D.parts * 4);
  W.dlb = take(D.T * D.E * 2);
  W.dx_r = take(D.T * D.d * 2);
  W.dgus = take(D.T * 2 * D.fs * 2);
  W.dwps = take(D.gate ? D.T * D.parts_s * 4 : 0);
  W.dxsh = take(D.T * D.d * 2);
  W.dz = take(D.gate ? D.T * 4 : 0);
  W.colsum = take(D.gate ? (int64_t)colsum_parts(D.T) * D.d * 4 : 0);
  // weight-gradient GEMMs that cut their contraction: routed experts (ragged split), shared expert, router
  const int64_t e1 = lewi_grouped_gemm_tn_workspace_bytes(D.Mpad, D.d, 2 * D.f, D.E, 1);
  const int64_t e2 = lewi_grouped_gemm_tn_workspace_bytes(D.Mpad, D.f, D.d, D.E, 0);
  W.tn_e_bytes = e1 > e2 ? e1 : e2;
  W.tn_e = take(W.tn_e_bytes);
  int64_t s1 = 0, s2 = 0;
  if (D.fs > 0) {
    s1 = lewi_grouped_gemm_tn_workspace_bytes(D.T, D.d, 2 * D.fs, 1, 1);
    s2 = lewi_grouped_gemm_tn_workspace_bytes(D.T, D.fs, D.d, 1, 0);
  }
  W.tn_s_bytes = s1 > s2 ? s1 : s2;
  W.tn_s = take(W.tn_s_bytes);
  W.tn_r_bytes = lewi_grouped_gemm_tn_workspace_bytes(D.T, D.d, D.E, 1, 0);
  W.tn_r = take(W.tn_r_bytes);
  W.bias_bytes = lewi_router_bias_grad_workspace_bytes(D.T, D.E);
  W.bias = take(W.bias_bytes);
  W.total = run > fwd_end ? run : fwd_end;
}

// ------------------------------------------------------------------------------------------------ small kernels

// gate[t] = sigmoid(<x[t], w[:]>): the optional gate of the shared expert (one warp per token).
__global__ void __launch_bounds__(256) shared_gate_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                              const float* __restrict__ w, float* __restrict__ gate,
                                                              long long T, int d) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long t = warp0; t < T; t += n_warps) {
    float acc = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
      const uint4 v = ld_nc_v4(x + t * d + c);
      float f[8];
      Elem<__nv_bfloat16>::unpack(v, f);
#pragma unroll
      for (int q = 0; q < 8; ++q) acc = fmaf(f[q], w[c + q], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) gate[t] = 1.0f / (1.0f + __expf(-acc));
  }
}

// dz[t] = (sum_p pieces[t,p]) * gate[t] * (1 - gate[t]);  partial[b, c] = sum over the 128 tokens of CTA b of
// x[t,c] * dz[t] (tokens added in index order).  The pieces are <dout[t], shared_out[t]> as the dSwiGLU epilogue
// leaves them.
__global__ void __launch_bounds__(256) shared_gate_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                              const float* __restrict__ pieces, int parts,
                                                              const float* __restrict__ gate, float* __restrict__ dz,
                                                              float* __restrict__ partial, long long T, int d) {
  __shared__ float s_dz[128];
  const long long t0 = (long long)blockIdx.x * 128;
  if (threadIdx.x < 128) {
    const long long t = t0 + threadIdx.x;
    float v = 0.f;
    if (t < T) {
      for (int p = 0; p < parts; ++p) v += pieces[t * parts + p];
      const float g = gate[t];
      v *= g * (1.0f - g);
      dz[t] = v;
    }
    s_dz[threadIdx.x] = v;
  }
  __syncthreads();
  const int n_tok = (int)min(128LL, T - t0);
  for (int c = threadIdx.x * 2; c < d; c += 512) {
    float a0 = 0.f, a1 = 0.f;
    for (int i = 0; i < n_tok; ++i) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + (t0 + i) * d + c);
      a0 = fmaf(__low2float(v), s_dz[i], a0);
      a1 = fmaf(__high2float(v), s_dz[i], a1);
    }
    partial[(long long)blockIdx.x * d + c] = a0;
    partial[(long long)blockIdx.x * d + c + 1] = a1;
  }
}

// Per-device events that tie the side stream to the main one (created once, never destroyed).
struct Events {
  cudaEvent_t fork_fwd, join_fwd, fork_bwd, join_bwd, dh_done;
  bool ok;
};

inline Events* events() {
  static Events ev[64];
  static bool made[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!made[dev]) {
    Events& e = ev[dev];
    e.ok = cudaEventCreateWithFlags(&e.fork_fwd, cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&e.join_fwd, cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&e.fork_bwd, cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&e.join_bwd, cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&e.dh_done, cudaEventDisableTiming) == cudaSuccess;
    made[dev] = true;
  }
  return ev[dev].ok ? &ev[dev] : nullptr;
}

// NVTX range on the host thread around the launches of one stage, named like the reference's profiler scopes
// (`jax.named_scope("moe_permute_dispatch" / "moe_permute_sort" / "moe_permute_combine")`,
// modal/moe_permute.py:403,408,431), so that timelines of the two implementations line up.
struct Range {
  explicit Range(const char* name) { nvtxRangePushA(name); }
  ~Range() { nvtxRangePop(); }
  Range(const Range&) = delete;
  Range& operator=(const Range&) = delete;
};

typedef void (*MarkFn)(const char*, void*);
inline MarkFn& mark_fn() {
  static MarkFn fn = nullptr;
  return fn;
}
inline void mark(const char* name, void* stream) {
  if (mark_fn() != nullptr) mark_fn()(name, stream);
}

}  // namespace moe
}  // namespace lewi
