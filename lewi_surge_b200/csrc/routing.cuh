// Router post-processing and the stable counting sort of routed slots.
//
// Three launches, no atomics whose order could vary, so every integer output is reproducible:
//   1. route_chunk_kernel   one CTA per chunk of slots: (soft-max + top-k + renormalise when fed
//                           logits) and a per-chunk histogram of expert ids;
//   2. route_scan_kernel    one CTA: prefix over chunks per expert, prefix over experts, padded
//                           offsets, block table;
//   3. route_rank_kernel    one CTA per chunk: stable rank of every slot inside its expert group ->
//                           pos / order / padded row / slot-of-row.
// The result equals sort_indices() of the reference (modal/moe_permute.py:240-264): a stable sort
// of slots i = t*k + j by expert id, order[p] = slot at sorted position p, pos = inverse of order.
#pragma once

#include "common.cuh"

namespace lewi {

constexpr int kRouteThreads = 256;
constexpr int kRouteWarps = kRouteThreads / kWarp;
constexpr int kRouteChunkTokens = 128;  // tokens per chunk when fed logits
constexpr int kSortChunkSlots = 1024;   // slots per chunk when fed expert ids
constexpr int kMaxExperts = 512;
constexpr int kMaxTopK = 32;

__device__ __forceinline__ uint32_t float_order_key(float v) {
  uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  return v;
}

// Per-warp histogram of s_e[begin, end) into run[E] (a row private to this warp).
__device__ __forceinline__ void warp_histogram(const int* s_e, int begin, int end, int* run, int lane) {
  for (int base = begin; base < end; base += kWarp) {
    int i = base + lane;
    int e = (i < end) ? s_e[i] : -1;
    unsigned mask = __match_any_sync(0xffffffffu, e);
    int leader = __ffs(mask) - 1;
    if (e >= 0 && lane == leader) run[e] += __popc(mask);
    __syncwarp();
  }
}

// ER = experts held per lane (E <= 32*ER); NT = tokens a warp works on at once.  The soft-max and the k rounds of
// arg-max are chains of dependent shuffles; NT independent chains side by side keep the warp's issue slots busy
// while one of them waits.  Token i of the group is rows[i] (null: no such token); its results are the same bits
// whatever NT is.
template <int ER, int NT>
__device__ __forceinline__ void warp_softmax_topk(const float* const (&rows)[NT], int E, int k, int lane,
                                                  int (&out_idx)[NT], float (&out_w)[NT], float (&p)[NT][ER]) {
  float l[NT][ER];
  float mx[NT], sum[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
#pragma unroll
    for (int r = 0; r < ER; ++r) {
      const int e = lane + r * kWarp;
      l[i][r] = (e < E && rows[i] != nullptr) ? rows[i][e] : -INFINITY;
    }
  }
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    mx[i] = -INFINITY;
#pragma unroll
    for (int r = 0; r < ER; ++r) mx[i] = fmaxf(mx[i], l[i][r]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
    for (int i = 0; i < NT; ++i) mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], o));
  }
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    sum[i] = 0.f;
#pragma unroll
    for (int r = 0; r < ER; ++r) {
      const int e = lane + r * kWarp;
      p[i][r] = (e < E && rows[i] != nullptr) ? expf(l[i][r] - mx[i]) : 0.f;
      sum[i] += p[i][r];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
    for (int i = 0; i < NT; ++i) sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], o);
  }
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const float inv = 1.0f / sum[i];
#pragma unroll
    for (int r = 0; r < ER; ++r) p[i][r] *= inv;
  }

  // k rounds of warp arg-max on (logit descending, index ascending).
  unsigned long long key[NT][ER];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
#pragma unroll
    for (int r = 0; r < ER; ++r) {
      const int e = lane + r * kWarp;
      key[i][r] = (e < E && rows[i] != nullptr)
                      ? ((unsigned long long)float_order_key(l[i][r]) << 32) | (unsigned)(0xFFFFFFFFu - (unsigned)e)
                      : 0ull;
    }
  }
  float vsum[NT], my_v[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    vsum[i] = 0.f;
    my_v[i] = 0.f;
    out_idx[i] = 0;
  }
  for (int j = 0; j < k; ++j) {
    unsigned long long best[NT];
    float best_p[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      best[i] = 0ull;
      best_p[i] = 0.f;
#pragma unroll
      for (int r = 0; r < ER; ++r) {
        if (key[i][r] > best[i]) {
          best[i] = key[i][r];
          best_p[i] = p[i][r];
        }
      }
    }
    unsigned long long win[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) win[i] = best[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, win[i], o);
        win[i] = other > win[i] ? other : win[i];
      }
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int e_win = (int)(0xFFFFFFFFu - (unsigned)(win[i] & 0xFFFFFFFFull));
      const int owner = e_win & (kWarp - 1);
      const float v = __shfl_sync(0xffffffffu, best_p[i], owner);
      if (lane == owner) {
#pragma unroll
        for (int r = 0; r < ER; ++r)
          if (key[i][r] == win[i]) key[i][r] = 0ull;
      }
      vsum[i] += v;
      if (lane == j) {
        my_v[i] = v;
        out_idx[i] = e_win;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NT; ++i) out_w[i] = my_v[i] / vsum[i];
}

struct RouteChunkArgs {
  const float* logits;        // [T,E] or null
  const int32_t* flat_in;     // [M] or null (when logits == null)
  int32_t* topk_idx;          // [T,k] (written when logits != null)
  float* topk_w;              // [T,k]
  int32_t* chunk_hist;        // [n_chunks, E]
  float* chunk_probs;         // [n_chunks, E] or null
  int32_t* row_slot;          // [mpad] or null: filled with -1 here
  long long num_slots;        // M
  long long mpad;
  int E, k, chunk_slots;
};

template <int ER>
__global__ void __launch_bounds__(kRouteThreads) route_chunk_kernel(RouteChunkArgs a) {
  extern __shared__ int s_mem[];
  int* s_e = s_mem;                                 // [chunk_slots]
  int* s_run = s_mem + a.chunk_slots;               // [kRouteWarps][E]
  float* s_prob = reinterpret_cast<float*>(s_run + kRouteWarps * a.E);  // [kRouteWarps][E]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long chunk = blockIdx.x;
  const long long slot0 = chunk * a.chunk_slots;
  const int n_slots = (int)min((long long)a.chunk_slots, a.num_slots - slot0);

  const int nthreads = blockDim.x, nwarps = blockDim.x >> 5;
  for (int i = tid; i < kRouteWarps * a.E; i += nthreads) s_run[i] = 0;
  if (a.row_slot != nullptr) {
    for (long long r = (long long)blockIdx.x * nthreads + tid; r < a.mpad; r += (long long)gridDim.x * nthreads)
      a.row_slot[r] = -1;
  }

  if (a.logits != nullptr) {
    float pacc[ER];
#pragma unroll
    for (int r = 0; r < ER; ++r) pacc[r] = 0.f;
    const int n_tok = n_slots / a.k;
    const long long tok0 = slot0 / a.k;
    // a warp takes NT of its tokens (warp, warp + nwarps, ...) at a time; fewer when a lane holds many experts
    constexpr int NT = ER <= 4 ? 4 : (ER <= 8 ? 2 : 1);
    for (int t0 = warp; t0 < n_tok; t0 += nwarps * NT) {
      const float* rows[NT];
      float p[NT][ER];
      int idx[NT];
      float w[NT];
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int t = t0 + i * nwarps;
        rows[i] = t < n_tok ? a.logits + (tok0 + t) * a.E : nullptr;
      }
      warp_softmax_topk<ER, NT>(rows, a.E, a.k, lane, idx, w, p);
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int t = t0 + i * nwarps;
        if (t >= n_tok) continue;
#pragma unroll
        for (int r = 0; r < ER; ++r) pacc[r] += p[i][r];
        if (lane < a.k) {
          const long long s = (tok0 + t) * a.k + lane;
          a.topk_idx[s] = idx[i];
          a.topk_w[s] = w[i];
          s_e[t * a.k + lane] = idx[i];
        }
      }
    }
    if (a.chunk_probs != nullptr) {
      // warps w, w+8, w+16, ... fold their column sums into row w % 8 one after the other (fixed order)
      for (int round = 0; round * kRouteWarps < nwarps; ++round) {
        if (warp / kRouteWarps == round) {
#pragma unroll
          for (int r = 0; r < ER; ++r) {
            int e = lane + r * kWarp;
            if (e < a.E) {
              float* dst = &s_prob[(warp % kRouteWarps) * a.E + e];
              *dst = (round == 0 ? 0.f : *dst) + pacc[r];
            }
          }
        }
        __syncthreads();
      }
    }
  } else {
    for (int i = tid; i < n_slots; i += nthreads) {
      int e = a.flat_in[slot0 + i];
      if (e < 0 || e >= a.E) {
        raise_status(LEWI_STATUS_BAD_INDEX);
        e = -1;
      }
      s_e[i] = e;
    }
  }
  __syncthreads();

  const int spw = ((a.chunk_slots + kRouteWarps - 1) / kRouteWarps + kWarp - 1) / kWarp * kWarp;
  if (warp < kRouteWarps) {
    const int begin = min(warp * spw, n_slots), end = min(begin + spw, n_slots);
    warp_histogram(s_e, begin, end, s_run + warp * a.E, lane);
  }
  __syncthreads();
  for (int e = tid; e < a.E; e += nthreads) {
    int tot = 0;
#pragma unroll
    for (int w = 0; w < kRouteWarps; ++w) tot += s_run[w * a.E + e];
    a.chunk_hist[chunk * a.E + e] = tot;
    if (a.logits != nullptr && a.chunk_probs != nullptr) {
      float ps = 0.f;
      const int rows = min(nwarps, kRouteWarps);
      for (int w = 0; w < rows; ++w) ps += s_prob[w * a.E + e];
      a.chunk_probs[chunk * a.E + e] = ps;
    }
  }
}

struct RouteScanArgs {
  int32_t* chunk_hist;   // [n_chunks, E] in: histogram, out: exclusive prefix over chunks
  const float* chunk_probs;  // or null
  int32_t* counts;       // [E] or null
  int32_t* offsets;      // [E+1] (required: the rank kernel reads it)
  int32_t* pad_offsets;  // [E+1] or null
  int32_t* block_expert; // [nbmax] or null
  int32_t* n_blocks;     // [1] or null
  float* probs_sum;      // [E] or null
  float* aux_loss;       // [1] or null: E * sum_e (counts_e / num_slots) * (probs_sum_e / num_tokens)
  long long num_slots, num_tokens;
  int n_chunks, E, block, nbmax;
};

constexpr int kScanThreads = 1024;

__global__ void __launch_bounds__(kScanThreads) route_scan_kernel(RouteScanArgs a) {
  __shared__ int s_part[kScanThreads];
  __shared__ int s_cnt[kMaxExperts];
  __shared__ int s_off[kMaxExperts + 1];
  __shared__ int s_pad[kMaxExperts + 1];
  __shared__ float s_ps[kMaxExperts];
  const int tid = threadIdx.x;
  // parts: each expert's chunk range is split among P threads (P a power of two).
  int P = 1;
  while (P * 2 * a.E <= kScanThreads) P *= 2;
  const int e = tid % a.E, part = tid / a.E;
  const bool active = part < P;
  const int per = (a.n_chunks + P - 1) / P;
  const int c0 = min(part * per, a.n_chunks), c1 = min(c0 + per, a.n_chunks);
  int tot = 0;
  if (active) {
    for (int c = c0; c < c1; ++c) tot += a.chunk_hist[(long long)c * a.E + e];
  }
  s_part[tid] = active ? tot : 0;
  __syncthreads();
  if (active) {
    int base = 0;
    for (int q = 0; q < part; ++q) base += s_part[q * a.E + e];
    int run = base;
    for (int c = c0; c < c1; ++c) {
      long long i = (long long)c * a.E + e;
      int h = a.chunk_hist[i];
      a.chunk_hist[i] = run;
      run += h;
    }
    if (part == P - 1) s_cnt[e] = run;
  }
  __syncthreads();
  if (tid == 0) {
    int off = 0, pad = 0;
    for (int x = 0; x < a.E; ++x) {
      s_off[x] = off;
      s_pad[x] = pad;
      off += s_cnt[x];
      if (a.block > 0) pad += (s_cnt[x] + a.block - 1) / a.block * a.block;
    }
    s_off[a.E] = off;
    s_pad[a.E] = pad;
    if (a.n_blocks != nullptr && a.block > 0) a.n_blocks[0] = pad / a.block;
  }
  __syncthreads();
  for (int x = tid; x <= a.E; x += kScanThreads) {
    a.offsets[x] = s_off[x];
    if (a.pad_offsets != nullptr) a.pad_offsets[x] = s_pad[x];
    if (x < a.E && a.counts != nullptr) a.counts[x] = s_cnt[x];
  }
  if (a.block_expert != nullptr && a.block > 0) {
    const int nb = s_pad[a.E] / a.block;
    for (int b = tid; b < a.nbmax; b += kScanThreads) {
      int val = -1;
      if (b < nb) {
        int row = b * a.block;
        int lo = 0, hi = a.E;  // largest x with s_pad[x] <= row
        while (hi - lo > 1) {
          int mid = (lo + hi) >> 1;
          if (s_pad[mid] <= row) lo = mid; else hi = mid;
        }
        val = lo;
      }
      a.block_expert[b] = val;
    }
  }
  if (a.probs_sum != nullptr && a.chunk_probs != nullptr) {
    // same (expert, part) split as the histogram; parts are added in a fixed order
    __syncthreads();
    float ps = 0.f;
    if (active) {
      for (int c = c0; c < c1; ++c) ps += a.chunk_probs[(long long)c * a.E + e];
    }
    s_part[tid] = __float_as_int(active ? ps : 0.f);
    __syncthreads();
    if (tid < a.E) {
      float tot_p = 0.f;
      for (int q = 0; q < P; ++q) tot_p += __int_as_float(s_part[q * a.E + tid]);
      a.probs_sum[tid] = tot_p;
      s_ps[tid] = tot_p;
    }
    if (a.aux_loss != nullptr) {
      // load-balance loss: one thread adds the E terms in index order, so the value is reproducible
      __syncthreads();
      if (tid == 0) {
        float acc = 0.f;
        for (int x = 0; x < a.E; ++x) acc += (float)s_cnt[x] * s_ps[x];
        const float denom = (float)a.num_slots * (float)a.num_tokens;
        a.aux_loss[0] = denom > 0.f ? acc * (float)a.E / denom : 0.f;
      }
    }
  }
}

struct RouteRankArgs {
  const int32_t* flat;        // [M] expert id per slot
  const int32_t* chunk_base;  // [n_chunks, E] exclusive prefix over chunks
  const int32_t* offsets;     // [E+1]
  const int32_t* pad_offsets; // [E+1] or null
  int32_t* order;             // [M] or null
  int32_t* pos;               // [M] or null
  int32_t* pad_pos;           // [M] or null
  int32_t* row_slot;          // [mpad] or null
  long long num_slots;
  int E, chunk_slots;
};

__global__ void __launch_bounds__(kRouteThreads) route_rank_kernel(RouteRankArgs a) {
  extern __shared__ int s_mem[];
  int* s_e = s_mem;                    // [chunk_slots]
  int* s_run = s_mem + a.chunk_slots;  // [kRouteWarps][E]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long chunk = blockIdx.x;
  const long long slot0 = chunk * a.chunk_slots;
  const int n_slots = (int)min((long long)a.chunk_slots, a.num_slots - slot0);
  for (int i = tid; i < kRouteWarps * a.E; i += kRouteThreads) s_run[i] = 0;
  for (int i = tid; i < n_slots; i += kRouteThreads) {
    int e = a.flat[slot0 + i];
    s_e[i] = (e < 0 || e >= a.E) ? -1 : e;
  }
  __syncthreads();
  const int spw = ((a.chunk_slots + kRouteWarps - 1) / kRouteWarps + kWarp - 1) / kWarp * kWarp;
  const int begin = min(warp * spw, n_slots), end = min(begin + spw, n_slots);
  warp_histogram(s_e, begin, end, s_run + warp * a.E, lane);
  __syncthreads();
  // exclusive prefix over warps, seeded with the prefix over earlier chunks
  for (int e = tid; e < a.E; e += kRouteThreads) {
    int run = a.chunk_base[chunk * a.E + e];
#pragma unroll
    for (int w = 0; w < kRouteWarps; ++w) {
      int c = s_run[w * a.E + e];
      s_run[w * a.E + e] = run;
      run += c;
    }
  }
  __syncthreads();
  int* run = s_run + warp * a.E;
  for (int base = begin; base < end; base += kWarp) {
    int i = base + lane;
    int e = (i < end) ? s_e[i] : -1;
    unsigned mask = __match_any_sync(0xffffffffu, e);
    int leader = __ffs(mask) - 1;
    int rank = 0;
    if (e >= 0) rank = run[e] + __popc(mask & ((1u << lane) - 1u));
    __syncwarp();
    if (e >= 0 && lane == leader) run[e] += __popc(mask);
    __syncwarp();
    if (e >= 0) {
      long long slot = slot0 + i;
      int p = a.offsets[e] + rank;
      if (a.pos != nullptr) a.pos[slot] = p;
      if (a.order != nullptr) a.order[p] = (int)slot;
      if (a.pad_offsets != nullptr) {
        int pp = a.pad_offsets[e] + rank;
        if (a.pad_pos != nullptr) a.pad_pos[slot] = pp;
        if (a.row_slot != nullptr) a.row_slot[pp] = (int)slot;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Backward of softmax -> top-k -> renormalise.  One warp per token.
template <int ER>
__global__ void __launch_bounds__(256) router_topk_bwd_kernel(const float* __restrict__ logits,
                                                              const int32_t* __restrict__ topk_idx,
                                                              const float* __restrict__ dw,
                                                              const float* __restrict__ dw_partial, int dw_parts,
                                                              const int32_t* __restrict__ pad_pos,
                                                              float* __restrict__ dw_out,
                                                              float* __restrict__ dlogits,
                                                              __nv_bfloat16* __restrict__ dlogits_bf16, long long T,
                                                              int E, int k, const int32_t* __restrict__ counts,
                                                              float aux_coef, float* __restrict__ bias_partial) {
  __shared__ float s_bias[kMaxExperts];
  const int lane = threadIdx.x & 31;
  const long long warp_global = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  // gradient of the load-balance loss with respect to the soft-max probabilities of any token: the token
  // fractions are constants, so dL/dp[t,e] = aux_coef * counts[e]
  float cvec[ER], bias_acc[ER];
#pragma unroll
  for (int r = 0; r < ER; ++r) {
    const int e = lane + r * kWarp;
    cvec[r] = (counts != nullptr && e < E) ? aux_coef * (float)counts[e] : 0.f;
    bias_acc[r] = 0.f;
  }
  for (long long t = warp_global; t < T; t += n_warps) {
    const float* row = logits + t * E;
    float l[ER], p[ER];
    float mx = -INFINITY;
#pragma unroll
    for (int r = 0; r < ER; ++r) {
      int e = lane + r * kWarp;
      l[r] = (e < E) ? row[e] : -INFINITY;
      mx = fmaxf(mx, l[r]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int r = 0; r < ER; ++r) {
      int e = lane + r * kWarp;
      p[r] = (e < E) ? expf(l[r] - mx) : 0.f;
      sum += p[r];
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int r = 0; r < ER; ++r) p[r] *= inv;
    int my_e = 0;
    float my_v = 0.f, my_dw = 0.f;
    if (lane < k) {
      my_e = topk_idx[t * k + lane];
      my_e = min(max(my_e, 0), E - 1);
      my_v = expf(row[my_e] - mx) * inv;
      if (dw != nullptr) {
        my_dw = dw[t * k + lane];
      } else {  // the routing-weight gradient arrives as per-row pieces written by the dH GEMM's epilogue
        const long long pr = pad_pos[t * k + lane];
        for (int p = 0; p < dw_parts; ++p) my_dw += dw_partial[pr * dw_parts + p];
      }
      if (dw_out != nullptr) dw_out[t * k + lane] = my_dw;
    }
    const float S = warp_sum(my_v);
    const float wj = my_v / S;
    const float dot = warp_sum(my_dw * wj);
    const float dv = (lane < k) ? (my_dw - dot) / S : 0.f;
    const float pdp = warp_sum(my_v * dv);
    float dl[ER];
    float pc = 0.f;
    if (counts != nullptr) {
#pragma unroll
      for (int r = 0; r < ER; ++r) pc += p[r] * cvec[r];
      pc = warp_sum(pc);
    }
#pragma unroll
    for (int r = 0; r < ER; ++r) dl[r] = -p[r] * pdp + p[r] * (cvec[r] - pc);
    for (int j = 0; j < k; ++j) {
      int ej = __shfl_sync(0xffffffffu, my_e, j);
      float dvj = __shfl_sync(0xffffffffu, dv, j);
      if ((ej & (kWarp - 1)) == lane) {
#pragma unroll
        for (int r = 0; r < ER; ++r)
          if ((ej >> 5) == r) dl[r] += p[r] * dvj;
      }
    }
#pragma unroll
    for (int r = 0; r < ER; ++r) {
      int e = lane + r * kWarp;
      if (e < E) {
        if (dlogits != nullptr) dlogits[t * E + e] = dl[r];
        if (dlogits_bf16 != nullptr) dlogits_bf16[t * E + e] = __float2bfloat16_rn(dl[r]);
      }
      bias_acc[r] += dl[r];
    }
  }
  if (bias_partial != nullptr) {
    // column sums of dlogits over this CTA's tokens: warps fold in one after the other (fixed order)
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int w = 0; w < nwarps; ++w) {
      if (warp == w) {
#pragma unroll
        for (int r = 0; r < ER; ++r) {
          const int e = lane + r * kWarp;
          if (e < E) s_bias[e] = (w == 0 ? 0.f : s_bias[e]) + bias_acc[r];
        }
      }
      __syncthreads();
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) bias_partial[(long long)blockIdx.x * E + e] = s_bias[e];
  }
}

// out[c] = sum over parts of partial[part, c]; one CTA per column group, fixed summation order.
__global__ void __launch_bounds__(256) col_sum_reduce_kernel(const float* __restrict__ partial, int n_parts, int n_cols,
                                                             float* __restrict__ out) {
  __shared__ float s_red[256];
  const int c = blockIdx.x;
  float acc = 0.f;
  for (int p = threadIdx.x; p < n_parts; p += blockDim.x) acc += partial[(long long)p * n_cols + c];
  s_red[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) s_red[threadIdx.x] += s_red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[c] = s_red[0];
}

// ------------------------------------------------------------------------------------------------
// Row tables for a drop-in ragged_dot: rows already sorted by expert, group_sizes given.
__global__ void __launch_bounds__(256) group_tables_kernel(const int32_t* __restrict__ gs, long long M, int E,
                                                           int block, long long mpad, int nbmax,
                                                           int32_t* pad_offsets, int32_t* block_expert,
                                                           int32_t* n_blocks, int32_t* row_of_padded,
                                                           int32_t* padded_of_row) {
  __shared__ int s_off[kMaxExperts + 1];
  __shared__ int s_pad[kMaxExperts + 1];
  if (threadIdx.x == 0) {
    int off = 0, pad = 0;
    for (int x = 0; x < E; ++x) {
      s_off[x] = off;
      s_pad[x] = pad;
      int c = max(gs[x], 0);
      off += c;
      pad += (c + block - 1) / block * block;
    }
    s_off[E] = off;
    s_pad[E] = pad;
  }
  __syncthreads();
  const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long gstride = (long long)gridDim.x * blockDim.x;
  if (blockIdx.x == 0) {
    for (int x = threadIdx.x; x <= E; x += blockDim.x) pad_offsets[x] = s_pad[x];
    if (threadIdx.x == 0) n_blocks[0] = s_pad[E] / block;
  }
  const int nb = s_pad[E] / block;
  for (long long b = gtid; b < nbmax; b += gstride) {
    int val = -1;
    if (b < nb) {
      int row = (int)b * block, lo = 0, hi = E;
      while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (s_pad[mid] <= row) lo = mid; else hi = mid;
      }
      val = lo;
    }
    block_expert[b] = val;
  }
  for (long long r = gtid; r < mpad; r += gstride) {
    int val = -1;
    if (r < s_pad[E]) {
      int lo = 0, hi = E;
      while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (s_pad[mid] <= r) lo = mid; else hi = mid;
      }
      int local = (int)r - s_pad[lo];
      int cnt = s_off[lo + 1] - s_off[lo];
      if (local < cnt) val = s_off[lo] + local;
    }
    row_of_padded[r] = val;
  }
  for (long long m = gtid; m < M; m += gstride) {
    int val = -1;
    if (m < s_off[E]) {
      int lo = 0, hi = E;  // largest x with s_off[x] <= m and non-empty group containing m
      while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (s_off[mid] <= m) lo = mid; else hi = mid;
      }
      val = s_pad[lo] + ((int)m - s_off[lo]);
    }
    padded_of_row[m] = val;
  }
}

// f32 -> bf16 (round to nearest even), grid-stride.
__global__ void __launch_bounds__(256) cast_f32_bf16_kernel(const float* __restrict__ src,
                                                            __nv_bfloat16* __restrict__ dst, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}

// f32 -> three bf16 pieces with hi + mid + lo == w to 24 mantissa bits; dst is [3][n].  `rounded` (optional, [n])
// receives hi alone: the weight rounded to bf16.
__global__ void __launch_bounds__(256) split3_bf16_kernel(const float* __restrict__ src,
                                                          __nv_bfloat16* __restrict__ dst,
                                                          __nv_bfloat16* __restrict__ rounded, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float w = src[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(w);
    const float r1 = w - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(mid);
    dst[i] = hi;
    if (rounded != nullptr) rounded[i] = hi;
    dst[n + i] = mid;
    dst[2 * n + i] = __float2bfloat16_rn(r2);
  }
}

// ------------------------------------------------------------------------------------------------ host

inline int route_n_chunks(long long num_slots, int chunk_slots) {
  return (int)((num_slots + chunk_slots - 1) / chunk_slots);
}

template <int ER>
inline void launch_route_chunk(cudaStream_t st, const RouteChunkArgs& a, int n_chunks, size_t smem) {
  route_chunk_kernel<ER><<<n_chunks, kRouteThreads, smem, st>>>(a);
}

inline int route_common(cudaStream_t st, const float* logits, const int32_t* flat_in, long long T, long long M,
                        int E, int k, int block, int32_t* topk_idx, float* topk_w, int32_t* counts,
                        int32_t* offsets, int32_t* pad_offsets, int32_t* block_expert, int32_t* n_blocks,
                        int32_t* order, int32_t* pos, int32_t* pad_pos, int32_t* row_slot, float* probs_sum,
                        void* ws, long long ws_bytes, float* aux_loss = nullptr) {
  if (E <= 0 || E > kMaxExperts) return LEWI_ERR_LIMIT;
  if (M > 0x7fffffffLL) return LEWI_ERR_LIMIT;
  const int chunk_slots = logits ? kRouteChunkTokens * k : kSortChunkSlots;
  const int n_chunks = route_n_chunks(M, chunk_slots);
  const long long need = (long long)n_chunks * E * 8 + (long long)(E + 1) * 4;
  if (ws == nullptr || ws_bytes < need) return LEWI_ERR_WORKSPACE;
  int32_t* chunk_hist = reinterpret_cast<int32_t*>(ws);
  float* chunk_probs = reinterpret_cast<float*>(chunk_hist + (long long)n_chunks * E);
  int32_t* ws_offsets = reinterpret_cast<int32_t*>(chunk_probs + (long long)n_chunks * E);
  if (offsets == nullptr) offsets = ws_offsets;
  const bool padded = block > 0 && pad_offsets != nullptr;
  const long long mpad = padded ? (M + (long long)E * (block - 1)) / block * block : 0;
  const int nbmax = padded ? (int)(mpad / block) : 0;
  RouteChunkArgs ca;
  ca.logits = logits;
  ca.flat_in = flat_in;
  ca.topk_idx = topk_idx;
  ca.topk_w = topk_w;
  ca.chunk_hist = chunk_hist;
  ca.chunk_probs = (logits && probs_sum) ? chunk_probs : nullptr;
  ca.row_slot = padded ? row_slot : nullptr;
  ca.num_slots = M;
  ca.mpad = mpad;
  ca.E = E;
  ca.k = k;
  ca.chunk_slots = chunk_slots;
  const size_t smem = (size_t)chunk_slots * 4 + (size_t)kRouteWarps * E * 8;
  if (n_chunks > 0) {
    if (logits) {
      if (E <= 64) launch_route_chunk<2>(st, ca, n_chunks, smem);
      else if (E <= 128) launch_route_chunk<4>(st, ca, n_chunks, smem);
      else if (E <= 256) launch_route_chunk<8>(st, ca, n_chunks, smem);
      else launch_route_chunk<16>(st, ca, n_chunks, smem);
    } else {
      launch_route_chunk<1>(st, ca, n_chunks, smem);
    }
    LEWI_CHECK_LAUNCH();
  } else if (padded && row_slot != nullptr && mpad > 0) {
    cudaMemsetAsync(row_slot, 0xff, (size_t)mpad * 4, st);
  }
  RouteScanArgs sa;
  sa.chunk_hist = chunk_hist;
  sa.chunk_probs = ca.chunk_probs;
  sa.counts = counts;
  sa.offsets = offsets;
  sa.pad_offsets = padded ? pad_offsets : nullptr;
  sa.block_expert = padded ? block_expert : nullptr;
  sa.n_blocks = padded ? n_blocks : nullptr;
  sa.probs_sum = probs_sum;
  sa.aux_loss = (logits && probs_sum) ? aux_loss : nullptr;
  sa.num_slots = M;
  sa.num_tokens = T;
  sa.n_chunks = n_chunks;
  sa.E = E;
  sa.block = padded ? block : 0;
  sa.nbmax = nbmax;
  route_scan_kernel<<<1, kScanThreads, 0, st>>>(sa);
  LEWI_CHECK_LAUNCH();
  if (n_chunks > 0) {
    RouteRankArgs ra;
    ra.flat = logits ? topk_idx : flat_in;
    ra.chunk_base = chunk_hist;
    ra.offsets = offsets;
    ra.pad_offsets = padded ? pad_offsets : nullptr;
    ra.order = order;
    ra.pos = pos;
    ra.pad_pos = padded ? pad_pos : nullptr;
    ra.row_slot = padded ? row_slot : nullptr;
    ra.num_slots = M;
    ra.E = E;
    ra.chunk_slots = chunk_slots;
    route_rank_kernel<<<n_chunks, kRouteThreads, (size_t)chunk_slots * 4 + (size_t)kRouteWarps * E * 4, st>>>(ra);
    LEWI_CHECK_LAUNCH();
  }
  return LEWI_OK;
}

}  // namespace lewi
