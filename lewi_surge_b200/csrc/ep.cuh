// Expert-parallel dispatch / combine as kernels over peer memory (NVLink loads and stores).
//
// Rank g owns experts [g*El, (g+1)*El).  After the ranks have exchanged their expert histograms
// (counts_all [G,E], a tiny all-gather), every rank can compute where its rows live on the owner:
//   owner layout   rows of local expert el from all sources, source-major inside the expert, each expert
//                  padded to a multiple of 128 rows (the layout the grouped GEMMs consume);
//   dst_base[e]    first row, in the owner's buffer, of THIS rank's rows for global expert e.
// Dispatch is then one gather kernel whose stores go straight into the owners' buffers, together with a
// return address per row (source rank and slot); the owners send expert outputs back the same way, with
// stores into the source's slot-ordered buffer, where the combine is a sum over k consecutive rows.
// Stores only cross NVLink (a store holds no register while in flight, a load does), and the kernels
// are "thin": one CTA of 256 threads and at most 40 registers per SM, no shared memory, so that a CTA of
// these fits on an SM beside a resident grouped-GEMM CTA whichever of the two arrives first; transfers of one
// range of experts then overlap the GEMMs of another.  (Giving the exchange 16-32 SMs of its own, with the GEMM
// grids shrunk by as many, was measured slower in every arrangement tried.)  Ordering between ranks is either a
// stream-ordered collective issued by the host code or the flag barrier below.  Plain loads/stores only (no
// multimem, no TMA).
#pragma once

#include "common.cuh"
#include "gather.cuh"
#include "routing.cuh"

namespace lewi {

constexpr int kMaxPeers = 8;

struct PeerPtrs {
  void* p[kMaxPeers];
};

// One CTA.  counts_all [G,E]; outputs as described above.
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int32_t* __restrict__ counts_all, int G, int E, int me,
                                                       int block, long long rmax_pad, int nbmax,
                                                       int32_t* dst_base, int32_t* pad_offsets, int32_t* valid_end,
                                                       int32_t* n_blocks, int32_t* block_expert,
                                                       int32_t* recv_rows) {
  __shared__ int s_total[kMaxExperts];   // rows of expert e over all sources
  __shared__ int s_before[kMaxExperts];  // rows of expert e from sources < me
  __shared__ int s_pad[kMaxExperts + 1]; // padded start of expert e on ITS owner
  const int El = E / G;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, bef = 0;
    for (int s = 0; s < G; ++s) {
      const int c = counts_all[s * E + e];
      tot += c;
      if (s < me) bef += c;
    }
    s_total[e] = tot;
    s_before[e] = bef;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int first = (e / El) * El;   // first expert of e's owner
    int pad = 0;
    for (int x = first; x < e; ++x) pad += (s_total[x] + block - 1) / block * block;
    s_pad[e] = pad;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) dst_base[e] = s_pad[e] + s_before[e];
  // this rank as owner
  const int e0 = me * El;
  for (int el = threadIdx.x; el <= El; el += blockDim.x) {
    int v;
    if (el < El) {
      v = s_pad[e0 + el];
      valid_end[el] = v + s_total[e0 + el];
    } else {
      const int last = e0 + El - 1;
      v = s_pad[last] + (s_total[last] + block - 1) / block * block;
    }
    pad_offsets[el] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int last = e0 + El - 1;
    const long long total_pad = s_pad[last] + (s_total[last] + block - 1) / block * block;
    if (total_pad > rmax_pad) raise_status(LEWI_STATUS_EP_OVERFLOW);
    n_blocks[0] = (int)(min(total_pad, rmax_pad) / block);
    int rows = 0;
    for (int el = 0; el < El; ++el) rows += s_total[e0 + el];
    recv_rows[0] = rows;
  }
  if (block_expert != nullptr) {
    const int last = e0 + El - 1;
    const int nb = (s_pad[last] + (s_total[last] + block - 1) / block * block) / block;
    for (int b = threadIdx.x; b < nbmax; b += blockDim.x) {
      int val = -1;
      if (b < nb) {
        const int row = b * block;
        int lo = 0, hi = El;
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (s_pad[e0 + mid] <= row) lo = mid; else hi = mid;
        }
        val = lo;
      }
      block_expert[b] = val;
    }
  }
}

__device__ __forceinline__ unsigned long long ep_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

constexpr int kEpThreads = 256;      // 8 warps x 40 registers: what is left beside a GEMM CTA (12 warps measured no faster)
constexpr int kEpChunk = 4;          // 16-byte vectors per lane and pass
constexpr int kEpSlotBits = 28;      // return address = source rank << 28 | slot

__device__ __forceinline__ void ep_copy_row(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                            int nvec, int lane) {
  for (int c0 = 0; c0 < nvec; c0 += kEpChunk * kWarp) {
    uint4 v[kEpChunk];
#pragma unroll
    for (int c = 0; c < kEpChunk; ++c) {
      const int vi = c0 + lane + c * kWarp;
      v[c] = make_uint4(0, 0, 0, 0);
      if (vi < nvec) v[c] = ld_nc_v4(reinterpret_cast<const uint4*>(src) + vi);
    }
#pragma unroll
    for (int c = 0; c < kEpChunk; ++c) {
      const int vi = c0 + lane + c * kWarp;
      if (vi < nvec) st_v4(reinterpret_cast<uint4*>(dst) + vi, v[c]);
    }
  }
}

// Dispatch: sorted position p of this rank (slot order[p], token order[p]/k, expert e) goes to row
// dst_base[e] + (p - offsets[e]) of the owner's buffer.  Only the positions of local experts [el_lo, el_hi) of
// every owner are visited (they are contiguous per owner in the sorted order).  With the row go, optionally,
// the slot's router weight and its return address.
// A warp takes 32 rows at a time: each lane looks up one row's token, owner and destination row (three dependent
// table reads, paid once per 32 rows instead of once per row) and stores that row's weight and return address;
// then the whole warp copies the 32 rows one after the other.  Consecutive rows of a batch go to consecutive
// destinations, starting at this rank's right-hand neighbour, so at any moment every rank is sending to all the
// others and no destination's ingress port is everybody's target.
__global__ void __launch_bounds__(kEpThreads, 6) ep_push_rows_kernel(
    const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ order, const int32_t* __restrict__ flat_expert,
    const int32_t* __restrict__ offsets, const int32_t* __restrict__ dst_base, const float* __restrict__ slot_w,
    PeerPtrs peer_rows, PeerPtrs peer_w, PeerPtrs peer_ret, long long m, int k, int d, int El, int G,
    long long rmax_pad, long long n_tokens, int el_lo, int el_hi, int me) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / 8;
  long long longest = 0;
  for (int r = 0; r < G; ++r) {
    const long long len = (long long)offsets[r * El + el_hi] - offsets[r * El + el_lo];
    longest = max(longest, len);
  }
  const long long total = longest * G;
  for (long long base = warp0 * kWarp; base < total; base += n_warps * kWarp) {
    const long long j = base + lane;
    int my_r = -1, my_tok = 0, my_row = 0;
    if (j < total) {
      const int r = (int)((me + 1 + j % G) % G);
      const long long p = (long long)offsets[r * El + el_lo] + j / G;
      if (p < min((long long)offsets[r * El + el_hi], m)) {
        const int slot = order[p];
        bool ok = slot >= 0 && slot < m;
        int e = 0;
        if (ok) {
          e = flat_expert[slot];
          ok = e >= r * El + el_lo && e < r * El + el_hi && slot / k < n_tokens;
        }
        if (!ok) {
          raise_status(LEWI_STATUS_BAD_INDEX);
        } else {
          const long long row = (long long)dst_base[e] + (p - offsets[e]);
          if (row >= 0 && row < rmax_pad) {   // beyond: capacity overflow, reported by the plan kernel
            my_r = r;
            my_tok = slot / k;
            my_row = (int)row;
            if (slot_w != nullptr) reinterpret_cast<float*>(peer_w.p[r])[row] = slot_w[slot];
            if (peer_ret.p[r] != nullptr) reinterpret_cast<int32_t*>(peer_ret.p[r])[row] = (me << kEpSlotBits) | slot;
          }
        }
      }
    }
    for (int i = 0; i < kWarp; ++i) {
      const int r = __shfl_sync(0xffffffffu, my_r, i);
      const long long tok = __shfl_sync(0xffffffffu, my_tok, i);
      const long long row = __shfl_sync(0xffffffffu, my_row, i);
      if (r < 0) continue;
      ep_copy_row(x + tok * d, reinterpret_cast<__nv_bfloat16*>(peer_rows.p[r]) + row * d, nvec, lane);
    }
  }
}

// Owner side: rows [pad_offsets[el_lo], pad_offsets[el_hi]) go back to where they came from: row r to row
// `slot` of the source rank's slot-ordered buffer, and (optionally) its `parts` routing-weight gradient
// pieces to the source's [slots, parts] buffer.  Padding rows carry the return address -1.  Same batching as
// the push kernel: a lane reads one row's return address (and sends its pieces), the warp then copies 32 rows.
__global__ void __launch_bounds__(kEpThreads, 6) ep_return_rows_kernel(
    const __nv_bfloat16* __restrict__ rows, const float* __restrict__ pieces, const int32_t* __restrict__ ret,
    const int32_t* __restrict__ pad_offsets, int el_lo, int el_hi, PeerPtrs peer_slot_rows, PeerPtrs peer_slot_pieces,
    int d, int parts, int G, long long m_slots, long long rmax_pad) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = d / 8;
  const long long r0 = pad_offsets[el_lo], r1 = min((long long)pad_offsets[el_hi], rmax_pad);
  for (long long base = r0 + warp0 * kWarp; base < r1; base += n_warps * kWarp) {
    const long long r = base + lane;
    int my_src = -1, my_slot = 0;
    if (r < r1) {
      const int code = ret[r];
      if (code >= 0) {
        const int src = code >> kEpSlotBits;
        const int slot = code & ((1 << kEpSlotBits) - 1);
        if (src >= G || slot >= m_slots) {
          raise_status(LEWI_STATUS_BAD_INDEX);
        } else {
          my_src = src;
          my_slot = slot;
          if (pieces != nullptr)
            for (int q = 0; q < parts; ++q)
              reinterpret_cast<float*>(peer_slot_pieces.p[src])[(long long)slot * parts + q] = pieces[r * parts + q];
        }
      }
    }
    if (rows == nullptr) continue;
    for (int i = 0; i < kWarp; ++i) {
      const int src = __shfl_sync(0xffffffffu, my_src, i);
      const long long slot = __shfl_sync(0xffffffffu, my_slot, i);
      if (src < 0) continue;
      ep_copy_row(rows + (base + i) * d, reinterpret_cast<__nv_bfloat16*>(peer_slot_rows.p[src]) + slot * d, nvec, lane);
    }
  }
}

// Owner side: the unused tail of every expert's last block must be zero rows (and have no return address).
__global__ void __launch_bounds__(256) ep_zero_pad_kernel(__nv_bfloat16* buf, int32_t* __restrict__ ret,
                                                          const int32_t* __restrict__ valid_end,
                                                          const int32_t* __restrict__ pad_offsets, int d,
                                                          long long rmax_pad) {
  const int el = blockIdx.x;
  const long long r0 = valid_end[el], r1 = min((long long)pad_offsets[el + 1], rmax_pad);
  const long long n16 = (r1 > r0 ? (r1 - r0) : 0) * d / 8;
  uint4* base = reinterpret_cast<uint4*>(buf + r0 * d);
  for (long long i = threadIdx.x; i < n16; i += blockDim.x) base[i] = make_uint4(0, 0, 0, 0);
  if (ret != nullptr)
    for (long long r = r0 + threadIdx.x; r < r1; r += blockDim.x) ret[r] = -1;
}

// Small all-gather by stores: src[0..n) goes to element dst_offset of every peer's buffer.
__global__ void __launch_bounds__(256) ep_put_i32_kernel(const int32_t* __restrict__ src, PeerPtrs dst, long long dst_offset,
                                                         int n, int G) {
  for (int g = 0; g < G; ++g) {
    int32_t* out = reinterpret_cast<int32_t*>(dst.p[g]) + dst_offset;
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[i] = src[i];
  }
}

// Barrier between the ranks, in stream order, without a collective library: thread g tells rank g that
// this rank has reached `epoch` (a store into g's flag array, after a system-scope fence that orders it
// behind this GPU's earlier peer stores), then waits until rank g has said the same here.  One tiny
// CTA: it fits beside whatever else is resident, so it never waits for a free SM.  The wait is bounded:
// after `timeout_ns` it records LEWI_STATUS_WAIT_TIMEOUT and returns.  Every rank must run the same
// sequence of barriers (each counts them in its own epoch_counter); no other kernel of the same GPU is ever
// waited for.
__global__ void __launch_bounds__(32) ep_barrier_kernel(PeerPtrs peer_flags, volatile int32_t* my_flags,
                                                        int32_t* epoch_counter, int me, int G,
                                                        unsigned long long timeout_ns) {
  const int g = threadIdx.x;
  // the epoch lives on the device (every rank counts its own barriers), so that a captured graph can be replayed
  int epoch = 0;
  if (g == 0) {
    epoch = *epoch_counter + 1;
    *epoch_counter = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  if (g >= G) return;
  __threadfence_system();
  int32_t* remote = reinterpret_cast<int32_t*>(peer_flags.p[g]) + me;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const unsigned long long t0 = ep_timer_ns();
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(my_flags + g) : "memory");
    if (v - epoch >= 0) break;
    if (ep_timer_ns() - t0 > timeout_ns) {
      raise_status(LEWI_STATUS_WAIT_TIMEOUT);
      break;
    }
    __nanosleep(200);
  }
  __threadfence_system();
}

}  // namespace lewi
