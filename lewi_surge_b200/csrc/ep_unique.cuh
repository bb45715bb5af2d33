// Expert-parallel exchange that moves a token ONCE per destination rank.
//
// A token whose k experts live on fewer than k ranks is sent once to each of those ranks instead of once per
// (token, expert) slot: top-6 over 2 / 4 / 8 ranks sends 0.99 / 2.5 / 3.9 rows per token across NVLink instead of
// 3 / 4.5 / 5.25.  The owner copies a received row to the padded rows of its local experts (local memory), runs the
// grouped GEMMs as usual, adds up a token's local expert outputs (they already carry the routing weights) and sends
// ONE partial row per token back; the source adds the partial rows of the ranks it sent the token to.
//
// Per source rank (tokens t, destinations r):
//   info[t,r]   -1 if t is not sent to r, else (first range | last range << 8) of t's experts on r, where a "range" is
//               one of the groups of local experts the exchange is pipelined over (bounds);
//   uidx[t,r]   rank of t among the tokens this source sends to r, in token order ("unique index"), or -1;
//   comb[t,r]   r*T + uidx[t,r], the row of the source's return buffer [G*T, d] in which r's partial row lands, or -1.
// Per owner: unique rows of source s start at ubase[s] = sum of ucount_all[s' < s][me] in its buffer ux [G*T, d];
//   rowu[row]   unique row that padded row `row` is a copy of (-1: padding);
//   urows[u,j]  padded rows of unique row u (-1 padded to k), umeta[u] its last range, uret[u] = source << 28 |
//               row of the source's return buffer.
// Rows whose first range is p are pushed as group p, so the GEMMs of range p can start once groups <= p have
// arrived; partial rows whose last range is p go back as soon as the GEMMs of range p are done.
#pragma once

#include "common.cuh"
#include "ep.cuh"

namespace lewi {

constexpr int kEpMaxRanges = 8;
constexpr int kEpUniqueChunk = 1024;   // tokens per CTA of the table kernels

struct EpBounds {
  int n;                        // number of ranges
  int b[kEpMaxRanges + 1];      // range p = local experts [b[p], b[p+1])
};

__device__ __forceinline__ int ep_range_of(const EpBounds& bd, int el) {
  int p = 0;
#pragma unroll
  for (int i = 1; i < kEpMaxRanges; ++i) p += (i < bd.n && el >= bd.b[i]) ? 1 : 0;
  return p;
}

// Pass 1: info[t,r] and the number of tokens of every chunk that go to r.
__global__ void __launch_bounds__(256) ep_unique_info_kernel(const int32_t* __restrict__ topk_idx, long long T, int k,
                                                             int El, int G, EpBounds bd, int32_t* __restrict__ info,
                                                             int32_t* __restrict__ chunk_cnt) {
  __shared__ int s_cnt[kMaxPeers];
  if (threadIdx.x < kMaxPeers) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  const long long t0 = (long long)blockIdx.x * kEpUniqueChunk;
  for (int i = threadIdx.x; i < kEpUniqueChunk; i += blockDim.x) {
    const long long t = t0 + i;
    if (t >= T) break;
    // first / last range per destination, 4 bits each (0xF = none)
    uint32_t lo = 0xFFFFFFFFu, hi = 0u, sent = 0u;
    for (int j = 0; j < k; ++j) {
      const int e = topk_idx[t * k + j];
      if (e < 0 || e >= El * G) {
        raise_status(LEWI_STATUS_BAD_INDEX);
        continue;
      }
      const int r = e / El;
      const uint32_t p = (uint32_t)ep_range_of(bd, e - r * El);
      const int sh = r * 4;
      if (p < ((lo >> sh) & 0xFu)) lo = (lo & ~(0xFu << sh)) | (p << sh);
      if (!((sent >> r) & 1u) || p > ((hi >> sh) & 0xFu)) hi = (hi & ~(0xFu << sh)) | (p << sh);
      sent |= 1u << r;
    }
    for (int r = 0; r < G; ++r) {
      const bool on = (sent >> r) & 1u;
      info[t * G + r] = on ? (int)(((lo >> (r * 4)) & 0xFu) | (((hi >> (r * 4)) & 0xFu) << 8)) : -1;
      if (on) atomicAdd(&s_cnt[r], 1);   // a count: the order of the additions does not matter
    }
  }
  __syncthreads();
  if (threadIdx.x < G) chunk_cnt[(long long)blockIdx.x * G + threadIdx.x] = s_cnt[threadIdx.x];
}

// Pass 2: uidx / comb in token order, and the totals ucount[r].
__global__ void __launch_bounds__(256) ep_unique_rank_kernel(const int32_t* __restrict__ info,
                                                             const int32_t* __restrict__ chunk_cnt, long long T, int G,
                                                             int32_t* __restrict__ uidx, int32_t* __restrict__ comb,
                                                             int32_t* __restrict__ ucount) {
  __shared__ int s_base[kMaxPeers];
  __shared__ int s_warp[8][kMaxPeers];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < G) {
    int b = 0;
    for (int c = 0; c < (int)blockIdx.x; ++c) b += chunk_cnt[(long long)c * G + tid];
    s_base[tid] = b;
    if (blockIdx.x == gridDim.x - 1) ucount[tid] = b + chunk_cnt[(long long)blockIdx.x * G + tid];
  }
  __syncthreads();
  const long long t0 = (long long)blockIdx.x * kEpUniqueChunk;
  for (int round = 0; round < kEpUniqueChunk / 256; ++round) {
    const long long t = t0 + round * 256 + tid;
    int mine[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      const bool on = r < G && t < T && info[t * G + r] >= 0;
      const unsigned m = __ballot_sync(0xffffffffu, on);
      mine[r] = on ? __popc(m & ((1u << lane) - 1u)) : -1;
      if (lane == 0) s_warp[warp][r] = __popc(m);
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      if (r >= G || t >= T) continue;
      int before = s_base[r];
      for (int w = 0; w < warp; ++w) before += s_warp[w][r];
      const int u = mine[r] >= 0 ? before + mine[r] : -1;
      uidx[t * G + r] = u;
      comb[t * G + r] = u >= 0 ? (int)(r * T + u) : -1;
    }
    __syncthreads();
    if (tid < G) {
      int tot = 0;
      for (int w = 0; w < 8; ++w) tot += s_warp[w][tid];
      s_base[tid] += tot;
    }
    __syncthreads();
  }
}

// From everybody's ucount (ucount_all [G,G], row = source): where this rank's unique rows start in every owner's
// buffer (usrc_base [G]) and how many unique rows this rank receives (utotal).
__global__ void __launch_bounds__(32) ep_unique_plan_kernel(const int32_t* __restrict__ ucount_all, int G, int me,
                                                            long long umax, int32_t* __restrict__ usrc_base,
                                                            int32_t* __restrict__ utotal) {
  const int r = threadIdx.x;
  if (r < G) {
    int b = 0;
    for (int s = 0; s < me; ++s) b += ucount_all[s * G + r];
    usrc_base[r] = b;
  }
  if (r == 0) {
    long long tot = 0;
    for (int s = 0; s < G; ++s) tot += ucount_all[s * G + me];
    if (tot > umax) raise_status(LEWI_STATUS_EP_OVERFLOW);
    utotal[0] = (int)min(tot, umax);
  }
}

struct EpUniqueMeta {
  const int32_t* topk_idx;   // [T,k]
  const float* topk_w;       // [T,k]
  const int32_t* pos;        // [M] sorted position of slot
  const int32_t* offsets;    // [E+1] first sorted position of expert e
  const int32_t* dst_base;   // [E] first row, on e's owner, of this rank's rows for e
  const int32_t* info;       // [T,G]
  const int32_t* uidx;       // [T,G]
  const int32_t* usrc_base;  // [G]
  PeerPtrs w, ret, rowu, urows, umeta, uret;   // the owners' tables
  long long T, rmax, umax;
  int k, El, G, me;
};

// One thread per (token, destination): everything the owner needs to know about the token's rows except the row.
__global__ void __launch_bounds__(256) ep_unique_meta_kernel(EpUniqueMeta a) {
  const long long n = a.T * a.G;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / a.G;
    const int r = (int)(i - t * a.G);
    const int nf = a.info[i];
    if (nf < 0) continue;
    const long long u = (long long)a.usrc_base[r] + a.uidx[i];
    if (u >= a.umax) continue;   // overflow, reported by the plan kernel
    int32_t* urows = reinterpret_cast<int32_t*>(a.urows.p[r]) + u * a.k;
    int n_rows = 0;
    for (int j = 0; j < a.k; ++j) {
      const long long slot = t * a.k + j;
      const int e = a.topk_idx[slot];
      if (e < r * a.El || e >= (r + 1) * a.El) continue;
      const long long row = (long long)a.dst_base[e] + (a.pos[slot] - a.offsets[e]);
      if (row < 0 || row >= a.rmax) continue;   // capacity overflow, reported by the plan kernel
      reinterpret_cast<float*>(a.w.p[r])[row] = a.topk_w[slot];
      reinterpret_cast<int32_t*>(a.ret.p[r])[row] = (a.me << kEpSlotBits) | (int)slot;
      reinterpret_cast<int32_t*>(a.rowu.p[r])[row] = (int)u;
      urows[n_rows++] = (int)row;
    }
    for (; n_rows < a.k; ++n_rows) urows[n_rows] = -1;
    reinterpret_cast<int32_t*>(a.umeta.p[r])[u] = (nf >> 8) & 0xFF;
    reinterpret_cast<int32_t*>(a.uret.p[r])[u] = (a.me << kEpSlotBits) | (int)(r * a.T + a.uidx[i]);
  }
}

// Rows of group `group` (tokens whose first range on the destination is `group`; negative: all) go to the owners'
// unique-row buffers.  Thin like the other exchange kernels; the same batching: a lane looks up one (token,
// destination) pair, the warp then copies up to 32 rows.  Consecutive pairs go to consecutive destinations.
__global__ void __launch_bounds__(kEpThreads, 6) ep_push_unique_kernel(
    const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ info, const int32_t* __restrict__ uidx,
    const int32_t* __restrict__ usrc_base, PeerPtrs peer_ux, long long T, int d, int G, int me, int group,
    long long umax) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / 8;
  const long long total = T * G;
  for (long long base = warp0 * kWarp; base < total; base += n_warps * kWarp) {
    const long long j = base + lane;
    int my_r = -1, my_tok = 0, my_row = 0;
    if (j < total) {
      const long long t = j / G;
      const int r = (int)((me + 1 + j % G) % G);
      const int nf = info[t * G + r];
      if (nf >= 0 && (group < 0 || (nf & 0xFF) == group)) {
        const long long u = (long long)usrc_base[r] + uidx[t * G + r];
        if (u < umax) {
          my_r = r;
          my_tok = (int)t;
          my_row = (int)u;
        }
      }
    }
    for (int i = 0; i < kWarp; ++i) {
      const int r = __shfl_sync(0xffffffffu, my_r, i);
      const long long tok = __shfl_sync(0xffffffffu, my_tok, i);
      const long long row = __shfl_sync(0xffffffffu, my_row, i);
      if (r < 0) continue;
      ep_copy_row(x + tok * d, reinterpret_cast<__nv_bfloat16*>(peer_ux.p[r]) + row * d, nvec, lane);
    }
  }
}

// Owner, local memory only: padded rows [pad_offsets[el_lo], pad_offsets[el_hi]) become copies of their unique rows
// (zero rows where rowu < 0).
template <int VPL>
__global__ void __launch_bounds__(256) ep_local_rows_kernel(const __nv_bfloat16* __restrict__ ux,
                                                            const int32_t* __restrict__ rowu,
                                                            const int32_t* __restrict__ pad_offsets, int el_lo, int el_hi,
                                                            __nv_bfloat16* __restrict__ out, int d, long long rmax,
                                                            long long umax) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / 8;
  const long long r0 = pad_offsets[el_lo], r1 = min((long long)pad_offsets[el_hi], rmax);
  for (long long row = r0 + warp0; row < r1; row += n_warps) {
    const long long u = rowu[row];
    if (u >= umax) {
      if (lane == 0) raise_status(LEWI_STATUS_BAD_INDEX);
      continue;
    }
    uint4 v[VPL];
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      const int vi = lane + c * kWarp;
      v[c] = make_uint4(0, 0, 0, 0);
      if (u >= 0 && vi < nvec) v[c] = ld_nc_v4(reinterpret_cast<const uint4*>(ux + u * d) + vi);
    }
#pragma unroll
    for (int c = 0; c < VPL; ++c) {
      const int vi = lane + c * kWarp;
      if (vi < nvec) st_v4(reinterpret_cast<uint4*>(out + row * d) + vi, v[c]);
    }
  }
}

// Owner: partial row of unique row u = sum of its padded rows of `rows` (f32), sent as bf16 to the row of the
// source's return buffer named by uret[u]; only unique rows whose last range is `group` (negative: all).  Thin: one
// 16-byte piece per lane at a time.
__global__ void __launch_bounds__(kEpThreads, 6) ep_combine_return_kernel(
    const __nv_bfloat16* __restrict__ rows, const int32_t* __restrict__ urows, const int32_t* __restrict__ umeta,
    const int32_t* __restrict__ uret, const int32_t* __restrict__ utotal, int group, PeerPtrs peer_out, int k, int d,
    int G, long long rmax, long long out_rows) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / 8;
  const long long n_u = utotal[0];
  for (long long base = warp0 * kWarp; base < n_u; base += n_warps * kWarp) {
    const long long mine = base + lane;
    int my_code = -1;
    if (mine < n_u && (group < 0 || umeta[mine] == group)) {
      my_code = uret[mine];
      const int src = my_code >> kEpSlotBits;
      const long long dst = my_code & ((1 << kEpSlotBits) - 1);
      if (my_code < 0 || src >= G || dst >= out_rows) {
        raise_status(LEWI_STATUS_BAD_INDEX);
        my_code = -1;
      }
    }
    for (unsigned todo = __ballot_sync(0xffffffffu, my_code >= 0); todo != 0; todo &= todo - 1) {
      const int i = __ffs(todo) - 1;
      const int code = __shfl_sync(0xffffffffu, my_code, i);
      const long long u = base + i;
      const int my_row = lane < k ? urows[u * k + lane] : -1;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(peer_out.p[code >> kEpSlotBits]) +
                           (long long)(code & ((1 << kEpSlotBits) - 1)) * d;
      for (int v0 = 0; v0 < nvec; v0 += kWarp) {   // uniform trip count: the shuffles below need the whole warp
        const int vi = v0 + lane;
        float acc[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = 0.f;
        for (int j = 0; j < k; ++j) {
          const long long row = __shfl_sync(0xffffffffu, my_row, j);
          if (row < 0 || row >= rmax || vi >= nvec) continue;
          float f[8];
          Elem<__nv_bfloat16>::unpack(ld_nc_v4(reinterpret_cast<const uint4*>(rows + row * d) + vi), f);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] += f[q];
        }
        if (vi < nvec) st_v4(reinterpret_cast<uint4*>(dst) + vi, Elem<__nv_bfloat16>::pack(acc));
      }
    }
  }
}

}  // namespace lewi
