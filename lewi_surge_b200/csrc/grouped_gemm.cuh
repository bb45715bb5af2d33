// Grouped GEMMs over the padded-block layout on the 5th-generation tensor cores.
//
// One persistent, warp-specialised kernel per (operand-major, epilogue) combination:
//   warp 0      TMA producer: tiled cp.async.bulk.tensor loads (128-byte swizzle, no multicast)
//               into a shared-memory ring (4 stages of 48 KB per CTA, or 6 of 32 KB per CTA of a pair);
//   warp 1      allocates TMEM and issues tcgen05.mma (128 x 256 x 16, bf16 in, f32 accumulate)
//               from one thread; accumulators are double-buffered in TMEM (2 x 256 columns);
//   warps 2-9   epilogue: tcgen05.ld the accumulator (thread = row; two warps share a TMEM lane
//               quarter and split the columns), fuse SwiGLU / its derivative / the router-weight
//               scale, store bf16 or f32 rows.
// A 128-row block of the padded layout belongs to exactly one expert, so a tile never straddles
// two weight matrices; the tile scheduler walks tiles (block, n-tile) read from the device-side
// block table, and empty experts simply own no tiles.
//
// Every wait is bounded (tcgen05.cuh: mbar_wait): when one runs out the CTA raises the device
// status, every role leaves its loop, TMEM is released and the kernel returns.
#pragma once

#include "common.cuh"
#include "tcgen05.cuh"

namespace lewi {
namespace gg {

constexpr int BM = 128;       // rows per CTA tile (= routing block)
constexpr int BN = 256;       // accumulator columns per tile (MMA N)
constexpr int BK = 64;        // contraction elements per stage (128 bytes of bf16)
constexpr int DATA_BYTES = 224 * 1024;         // operand ring + epilogue staging of one CTA
constexpr int EPI_WARPS = 8;      // two warps per TMEM lane quarter, each takes half of the columns
// Every epilogue warp moves its output (and the dSwiGLU epilogue also its g|u input) as TMA tiles of 32 rows x
// 128 bytes (128-byte swizzle, 4 KB).  It owns two such tiles of staging, three under the SwiGLU epilogue, which
// stores g, u and h of the same columns.  The operand ring gets the rest.
constexpr int TILE_BYTES = 4096;
__host__ __device__ constexpr int staging_per_warp(int epi) { return epi == 1 /* SWIGLU */ ? 3 * TILE_BYTES : 2 * TILE_BYTES; }
__host__ __device__ constexpr int ring_bytes(int epi) { return DATA_BYTES - EPI_WARPS * staging_per_warp(epi); }
constexpr int A_BYTES = BM * BK * 2;           // 16 KB
constexpr int CHUNK_BYTES = 64 * BK * 2;       // 8 KB: one [64 k][64 mn] box of an MN-major operand
// One CTA per tile (cta_group::1): B is 256 x 64 = 32 KB, 3 stages of 48 KB (2 under the SwiGLU epilogue).
// A CTA pair per 256-row tile (cta_group::2): each CTA holds its own 128 rows of A and HALF of B
// (128 x 64 = 16 KB), 5 stages of 32 KB (4 under SwiGLU); the tensor cores of both SMs read both halves.
template <bool PAIR, int EPI = 0> struct Cfg {
  static constexpr int B_BYTES = PAIR ? BN * BK : BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = ring_bytes(EPI) / STAGE_BYTES;
};
constexpr int MAX_STAGES = 5;
constexpr int PAIR_PREFIX_BYTES = 1040;        // uint16 prefix per expert (E <= 512): row-block pairs (NN/NT) or contraction parts (TN)
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int TMEM_COLS = 512;
constexpr int EPI_BAR_BYTES = 64;        // one mbarrier per epilogue warp (TMA loads of the dSwiGLU epilogue)
// 230,736 bytes.  An SM has 233,472 and every resident CTA reserves 1,024 of them, so exactly one more CTA that
// uses no shared memory (a gather or exchange kernel from another stream) fits beside a GEMM CTA.  That is why
// there is no slack for aligning the ring: the kernel asks for a 1024-byte aligned base and checks it.
constexpr size_t SMEM_BYTES = (size_t)DATA_BYTES + 256 /*barriers*/ + PAIR_PREFIX_BYTES + EPI_BAR_BYTES;

enum Major { NN = 0, NT = 1, TN = 2 };
enum Epi { PLAIN = 0, SWIGLU = 1, DSWIGLU = 2, TNOUT = 3, SCATTER = 4 };
constexpr int kRetSlotBits = 28;   // return address of a row = rank << 28 | row in that rank's buffer
constexpr int kRetRanks = 8;

struct Args {
  void* out;                    // PLAIN: [rows,N]; SWIGLU: h [rows,f]; DSWIGLU: dgu [rows,2f]; TNOUT: [E,Ma,Nb(/2)]
  void* out2;                   // SWIGLU: gu [rows,2f] or null; TNOUT: second half or null
  const __nv_bfloat16* gu;      // DSWIGLU input
  const float* row_scale;       // PLAIN: optional f32 per row
  const int32_t* block_expert;  // [blocks] or null (single group)
  const int32_t* n_blocks;      // device count of live blocks or null
  const int32_t* pad_offsets;   // TN: [E+1] or null
  long long rows;               // rows of the row-indexed operand(s)
  int n_blocks_host;            // bound on / value of the block count
  int K;                        // contraction extent (NN, NT); unused for TN
  int N;                        // output columns (SWIGLU/DSWIGLU: f); TN: Nb
  int Ma;                       // TN: rows of the output
  int E;
  int kb_split;                 // NT with two B tensors: k-blocks >= kb_split read the second one ...
  int k2_offset;                // ... and the A operand's k coordinate restarts at this column
  int kb_total;                 // NN / NT: 64-wide contraction steps per tile
  int out_f32;                  // PLAIN / TNOUT: 1 = f32 output, 0 = bf16
  int a_k_wrap;                 // NN: if > 0 the A operand's k coordinate wraps at this extent
  int k_splits;                 // TN: the contraction of every output tile is cut into this many parts
  float* partial;               // TN with k_splits > 1: f32 partial products [k_splits, E, Ma, N]
  const float* col_bias;        // PLAIN: optional f32 per output column
  const float* r1_row;          // PLAIN: optional rank-one term added to the product: out[r,n] += r1_row[r] * r1_col[n]
  const float* r1_col;
  int tn_part_rows;             // TN over several experts: > 0 cuts an expert's contraction into parts of this many rows
                                // (a multiple of 64); experts with more than one part go through `partial`
  const int32_t* scale_idx;     // SWIGLU / DSWIGLU: padded row -> index into scale_src (negative: scale 0; null: the row itself)
  const float* scale_src;       // SWIGLU / DSWIGLU: optional f32 table indexed by scale_idx[row] (router weight of the
                                // row's slot); SWIGLU stores h * scale, DSWIGLU multiplies dh by it
  float* dw_partial;            // DSWIGLU: optional [rows, dw_parts] f32, sum over this warp's columns of
  int dw_parts;                 //   dh_unscaled * silu(g) * u  (= pieces of the routing-weight gradient)
  // SCATTER: the bf16 product [rows, N] is not stored as a tensor: row r goes to row (ret[r] & slot mask) of
  // ret_out[ret[r] >> kRetSlotBits], a [ret_slots, N] buffer in this GPU's or a peer's memory; negative: not stored
  const int32_t* ret;
  void* ret_out[kRetRanks];
  long long ret_slots;
  int ret_ranks;
  uint64_t desc_hi_a, desc_hi_b;
  uint32_t kstep_a, kstep_b;    // bytes to advance the descriptor start per 16-wide k step
  uint32_t idesc;
};

__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// ---- epilogue output.  A thread owns one row of the accumulator (TMEM lane = row).  Rows are written into a
// staging tile of 32 rows x 128 bytes in the layout a 128-byte-swizzled TMA box has in shared memory (16-byte piece
// q of row r sits at r*128 + ((q ^ (r & 7)) << 4)); one lane then stores the tile with cp.async.bulk.tensor, which
// writes whole 128-byte lines and clips rows and columns that lie outside the tensor.
__device__ __forceinline__ void tile_put16(uint8_t* tile, int lane, int piece, uint4 v) {
  *reinterpret_cast<uint4*>(tile + lane * 128 + ((piece ^ (lane & 7)) << 4)) = v;
}
// 32 floats of this lane's row -> bf16 pieces [piece0, piece0 + 4) of the tile
__device__ __forceinline__ void tile_put_bf16x32(uint8_t* tile, int lane, int piece0, const float* v) {
#pragma unroll
  for (int q = 0; q < 4; ++q)
    tile_put16(tile, lane, piece0 + q,
               make_uint4(pack_bf16(v[q * 8 + 0], v[q * 8 + 1]), pack_bf16(v[q * 8 + 2], v[q * 8 + 3]),
                          pack_bf16(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16(v[q * 8 + 6], v[q * 8 + 7])));
}
// 32 floats of this lane's row -> the whole tile as f32
__device__ __forceinline__ void tile_put_f32x32(uint8_t* tile, int lane, const float* v) {
#pragma unroll
  for (int q = 0; q < 8; ++q)
    tile_put16(tile, lane, q,
               make_uint4(__float_as_uint(v[q * 4]), __float_as_uint(v[q * 4 + 1]), __float_as_uint(v[q * 4 + 2]),
                          __float_as_uint(v[q * 4 + 3])));
}

// One warp's staging tiles, used round-robin.  acquire() hands out the next tile once the TMA store that last
// read it has finished reading; commit(...) is called after the warp has filled the tile.
template <int NBUF>
struct TileStager {
  uint8_t* base;
  uint32_t n;
  __device__ __forceinline__ uint8_t* acquire(int lane) {
    if (lane == 0 && n >= NBUF) ptx::bulk_wait_read_n<NBUF - 1>();
    __syncwarp();
    return base + (n % NBUF) * TILE_BYTES;
  }
  __device__ __forceinline__ void store2d(int lane, const void* tmap, uint8_t* tile, int c0, int c1) {
    ptx::fence_proxy_async();   // the tile was written through the generic proxy, the store reads it through the async one
    __syncwarp();
    if (lane == 0) {
      ptx::tma_store_2d(tmap, ptx::smem_u32(tile), c0, c1);
      ptx::bulk_commit();
    }
    ++n;
  }
  __device__ __forceinline__ void store3d(int lane, const void* tmap, uint8_t* tile, int c0, int c1, int c2) {
    ptx::fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      ptx::tma_store_3d(tmap, ptx::smem_u32(tile), c0, c1, c2);
      ptx::bulk_commit();
    }
    ++n;
  }
};

struct Tile {
  int e;        // expert
  int second;   // pair mode, NN/NT: 1 if the second 128-row block of the pair belongs to the same expert
  int row0;     // first row of the row-indexed operand (NN/NT: A rows; TN: first contraction row)
  int m0;       // TN: first output row
  int n0;       // first accumulator column in output coordinates (SWIGLU: first h column)
  int nlim;     // columns >= nlim are not stored by this tile
  int kb0;      // first 64-wide contraction step of this tile
  int kb;       // number of 64-wide contraction steps
  int split;    // TN: slot of this part in `partial`, or -1 when the tile is stored straight to the output
};

// Row-block pairs (pair mode, NN/NT): expert e owns ceil(blocks_e / 2) pairs; pp[e] is the exclusive
// prefix of those counts (uint16 in shared memory).  Pair p belongs to the largest e with pp[e] <= p.
template <int MAJOR, int EPI, bool PAIR>
__device__ __forceinline__ Tile decode_tile(const Args& a, int tile, int n_tiles_n, const uint16_t* pp) {
  Tile t;
  t.second = 1;
  if constexpr (MAJOR == TN) {
    constexpr int TM = PAIR ? 2 * BM : BM;
    const int m_tiles = (a.Ma + TM - 1) / TM;
    const int per_e = m_tiles * n_tiles_n;
    int part, n_parts, part_kb;   // this tile's contraction part, the parts of its expert, 64-row steps per part
    if (a.tn_part_rows > 0) {
      // ragged split: pp[e] = exclusive prefix of the experts' part counts (every expert has at least one part)
      const int unit = tile / per_e;
      tile -= unit * per_e;
      int lo = 0, hi = a.E;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((int)pp[mid] <= unit) lo = mid; else hi = mid;
      }
      t.e = lo;
      part = unit - (int)pp[lo];
      n_parts = (int)pp[lo + 1] - (int)pp[lo];
      part_kb = a.tn_part_rows / BK;
      // parts of multi-part experts live in `partial`; expert e's run of slots starts at 2 * (pp[e] - e), which is
      // twice the number of extra parts before it and therefore never overlaps the next run
      t.split = n_parts > 1 ? 2 * ((int)pp[lo] - lo) + part : -1;
    } else {
      part = tile % a.k_splits;
      tile /= a.k_splits;
      t.e = tile / per_e;
      tile -= t.e * per_e;
      n_parts = a.k_splits;
      part_kb = 0;
      t.split = a.k_splits > 1 ? part * a.E + t.e : -1;
    }
    const int rem = tile;
    t.m0 = (rem / n_tiles_n) * TM;
    const int nt = rem % n_tiles_n;
    if (a.out2 != nullptr) {  // two column halves, tiled separately so that no tile straddles them
      const int half = a.N / 2, per_half = n_tiles_n / 2;
      const int which = nt / per_half;
      t.n0 = which * half + (nt - which * per_half) * BN;
      t.nlim = (which + 1) * half;
    } else {
      t.n0 = nt * BN;
      t.nlim = a.N;
    }
    int r0 = 0;
    long long r1 = a.rows;
    if (a.pad_offsets != nullptr) {
      r0 = a.pad_offsets[t.e];
      r1 = a.pad_offsets[t.e + 1];
    }
    t.row0 = r0;
    const int kb_total = (int)((r1 - r0 + BK - 1) / BK);
    if (part_kb == 0) part_kb = (kb_total + n_parts - 1) / n_parts;
    t.kb0 = part * part_kb;
    t.kb = max(0, min(part_kb, kb_total - t.kb0));
  } else {
    const int unit = tile / n_tiles_n;   // row block (one CTA) or pair of row blocks (CTA pair)
    const int nt = tile - unit * n_tiles_n;
    t.m0 = 0;
    t.n0 = nt * (EPI == SWIGLU ? BN / 2 : BN);
    t.nlim = a.N;
    t.kb0 = 0;
    t.split = 0;
    t.kb = a.kb_total;
    if constexpr (PAIR) {
      if (a.pad_offsets != nullptr) {
        int lo = 0, hi = a.E;  // largest e with pp[e] <= unit
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if ((int)pp[mid] <= unit) lo = mid; else hi = mid;
        }
        t.e = lo;
        const int first = a.pad_offsets[lo] / BM + 2 * (unit - (int)pp[lo]);
        t.row0 = first * BM;
        t.second = (first + 1) * BM < a.pad_offsets[lo + 1];
      } else {
        t.e = 0;
        t.row0 = unit * 2 * BM;
        t.second = (long long)t.row0 + BM < a.rows;
      }
    } else {
      t.e = a.block_expert ? a.block_expert[unit] : 0;
      t.row0 = unit * BM;
      if (t.e < 0 || t.e >= a.E) {  // corrupted table: skip the tile's work but keep the roles in step
        t.e = 0;
        t.kb = 0;
      }
    }
  }
  return t;
}

// 144 registers per thread: the register file is split over the SM's four schedulers (16,384 each), three of this
// CTA's ten warps land on one scheduler, and 3 x 144 x 32 leaves it room for two 40-register warps of an exchange
// CTA from another stream.  At the 168 the compiler would take by itself nothing else fits on the SM.  The
// dSwiGLU epilogue spills under that cap (measured 0.09 ms per step), so that kernel keeps 168 and shares nothing.
#ifndef LEWI_GEMM_MAX_REGS
#define LEWI_GEMM_MAX_REGS 144
#endif
constexpr int max_regs(int epi) { return epi == 2 /* DSWIGLU */ ? 168 : LEWI_GEMM_MAX_REGS; }

template <int MAJOR, int EPI, bool PAIR>
__global__ void __maxnreg__(max_regs(EPI))
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_c,
                    const __grid_constant__ CUtensorMap tm_d, const Args a) {
  constexpr int STAGES = Cfg<PAIR, EPI>::STAGES;
  constexpr int STAGE_BYTES = Cfg<PAIR, EPI>::STAGE_BYTES;
  constexpr int RING_BYTES = ring_bytes(EPI);
  constexpr int B_CHUNKS = PAIR ? 2 : 4;   // 64-column boxes of an MN-major B operand held by one CTA
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = ptx::smem_u32(smem_raw);
  if ((smem_base & 1023u) != 0) {   // 128-byte swizzled tiles need it; nothing has been set up yet, so just leave
    if (threadIdx.x == 0) raise_status(LEWI_STATUS_SMEM_LAYOUT);
    return;
  }
  const uint32_t bar_base = smem_base + DATA_BYTES;
  // barrier layout (8 bytes each): full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[2], drain
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * MAX_STAGES + 4);
  uint8_t* generic_base = smem_raw;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(generic_base + DATA_BYTES + 160);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(generic_base + DATA_BYTES + 168);
  uint16_t* pair_prefix = reinterpret_cast<uint16_t*>(generic_base + DATA_BYTES + 256);
  auto epi_bar = [&](int w) { return bar_base + 256u + PAIR_PREFIX_BYTES + 8u * w; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = PAIR ? ptx::cluster_ctarank() : 0u;   // 0 = leader of the pair
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);    // one arrival posts the TMA byte count
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(tfull_bar(b), 1);
      ptx::mbar_init(tempty_bar(b), PAIR ? 2 * EPI_WARPS : EPI_WARPS);
    }
    ptx::mbar_init(drain_bar, 1);
    for (int w = 0; w < EPI_WARPS; ++w) ptx::mbar_init(epi_bar(w), 1);
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tensormap(&tm_a);
    ptx::prefetch_tensormap(&tm_b);
    if constexpr (EPI == SWIGLU || MAJOR == NT) ptx::prefetch_tensormap(&tm_b2);
    ptx::prefetch_tensormap(&tm_c);
    ptx::prefetch_tensormap(&tm_d);
  }
  int n_units = 0;  // NN/NT: row blocks (or pairs of row blocks) to process
  if constexpr (MAJOR == TN) {
    if (a.tn_part_rows > 0 && threadIdx.x == 32) {  // exclusive prefix of the experts' contraction-part counts
      int run = 0;
      for (int e = 0; e < a.E; ++e) {
        pair_prefix[e] = (uint16_t)run;
        const int rows_e = a.pad_offsets[e + 1] - a.pad_offsets[e];
        run += max(1, (rows_e + a.tn_part_rows - 1) / a.tn_part_rows);
      }
      pair_prefix[a.E] = (uint16_t)min(run, 65535);
    }
  } else {
    if constexpr (PAIR) {
      if (a.pad_offsets != nullptr) {
        if (threadIdx.x == 32) {  // exclusive prefix of ceil(blocks_e / 2); a few hundred adds at most
          int run = 0;
          for (int e = 0; e < a.E; ++e) {
            pair_prefix[e] = (uint16_t)run;
            const int nb = (a.pad_offsets[e + 1] - a.pad_offsets[e]) / BM;
            run += (nb + 1) >> 1;
          }
          pair_prefix[a.E] = (uint16_t)min(run, 65535);
        }
      }
    }
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) ptx::cluster_sync();   // both CTAs' barriers exist before anything remote touches them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile range
  int n_tiles_n, total_tiles;
  if constexpr (MAJOR == TN) {
    constexpr int TM = PAIR ? 2 * BM : BM;
    n_tiles_n = a.out2 != nullptr ? 2 * ((a.N / 2 + BN - 1) / BN) : (a.N + BN - 1) / BN;
    const int per_e = ((a.Ma + TM - 1) / TM) * n_tiles_n;
    total_tiles = a.tn_part_rows > 0 ? min((int)pair_prefix[a.E], a.n_blocks_host) * per_e : a.E * per_e * a.k_splits;
  } else {
    const int bn_out = (EPI == SWIGLU) ? BN / 2 : BN;
    n_tiles_n = (a.N + bn_out - 1) / bn_out;
    if constexpr (PAIR) {
      if (a.pad_offsets != nullptr) n_units = pair_prefix[a.E];
      else n_units = (int)((a.rows + 2 * BM - 1) / (2 * BM));
      n_units = min(n_units, a.n_blocks_host);
    } else {
      n_units = a.n_blocks_host;
      if (a.n_blocks != nullptr) n_units = min(n_units, max(a.n_blocks[0], 0));
    }
    total_tiles = n_units * n_tiles_n;
  }
  const int tile_first = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tile_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  // in pair mode every load credits the LEADER's full barrier
  auto full_target = [&](int s) { return PAIR ? ptx::map_to_cta(full_bar(s), 0) : full_bar(s); };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer warp
    // Lane 0 posts the byte count of a stage and issues its tiled TMA loads.
    uint32_t it = 0;
    bool ok = true;
    if (lane == 0) {
      for (int tile = tile_first; ok && tile < total_tiles; tile += tile_step) {
        const Tile t = decode_tile<MAJOR, EPI, PAIR>(a, tile, n_tiles_n, pair_prefix);
        for (int kb = 0; kb < t.kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!ptx::mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES;
          const int nb0 = t.n0 + (PAIR ? (int)cta_rank * (BN / 2) : 0);   // first B column/row held by this CTA
          constexpr uint32_t cta_bytes = A_BYTES + Cfg<PAIR, EPI>::B_BYTES;
          // in pair mode both CTAs bring the same TMA byte count to the leader's barrier
          if (leader) ptx::mbar_expect_tx(full_bar(s), PAIR ? 2 * cta_bytes : cta_bytes);
          const uint32_t fb = full_target(s);
          auto load2 = [&](uint32_t dst, const CUtensorMap* tm, int c0, int c1) {
            if constexpr (PAIR) ptx::tma_load_2d_pair(dst, tm, fb, c0, c1); else ptx::tma_load_2d(dst, tm, fb, c0, c1);
          };
          auto load3 = [&](uint32_t dst, const CUtensorMap* tm, int c0, int c1, int c2) {
            if constexpr (PAIR) ptx::tma_load_3d_pair(dst, tm, fb, c0, c1, c2); else ptx::tma_load_3d(dst, tm, fb, c0, c1, c2);
          };
          if constexpr (MAJOR == TN) {
            const int r = t.row0 + (t.kb0 + kb) * BK;
            const int ma0 = t.m0 + (int)cta_rank * BM;
#pragma unroll
            for (int c = 0; c < 2; ++c) load2(sa + c * CHUNK_BYTES, &tm_a, ma0 + 64 * c, r);
#pragma unroll
            for (int c = 0; c < B_CHUNKS; ++c) load2(sb + c * CHUNK_BYTES, &tm_b, nb0 + 64 * c, r);
          } else {
            int ka = kb * BK;
            if constexpr (MAJOR == NN) {
              if (a.a_k_wrap > 0) ka %= a.a_k_wrap;
            } else {
              if (kb >= a.kb_split) ka = a.k2_offset + (kb - a.kb_split) * BK;
            }
            load2(sa, &tm_a, ka, t.row0 + (int)cta_rank * BM);
            if constexpr (MAJOR == NN) {
              if constexpr (EPI == SWIGLU) {
                if constexpr (PAIR) {  // the leader's half of B is the gate tile, the peer's half the up tile
                  const CUtensorMap* tm = leader ? &tm_b : &tm_b2;
#pragma unroll
                  for (int c = 0; c < 2; ++c) load3(sb + c * CHUNK_BYTES, tm, t.n0 + 64 * c, kb * BK, t.e);
                } else {
#pragma unroll
                  for (int c = 0; c < 2; ++c) load3(sb + c * CHUNK_BYTES, &tm_b, t.n0 + 64 * c, kb * BK, t.e);
#pragma unroll
                  for (int c = 0; c < 2; ++c) load3(sb + (2 + c) * CHUNK_BYTES, &tm_b2, t.n0 + 64 * c, kb * BK, t.e);
                }
              } else {
#pragma unroll
                for (int c = 0; c < B_CHUNKS; ++c) load3(sb + c * CHUNK_BYTES, &tm_b, nb0 + 64 * c, kb * BK, t.e);
              }
            } else {  // NT
              if (kb < a.kb_split) load3(sb, &tm_b, kb * BK, nb0, t.e);
              else load3(sb, &tm_b2, (kb - a.kb_split) * BK, nb0, t.e);
            }
          }
        }
      }
      if (*abort_flag && leader) {
        // give the copies already issued a bounded chance to land before shared memory is released
        const uint32_t first = it > STAGES ? it - STAGES : 0;
        for (uint32_t j = first; j < it; ++j) {
          const unsigned long long t0 = ptx::globaltimer_ns();
          while (!ptx::mbar_try_wait(full_bar(j % STAGES), (j / STAGES) & 1u)) {
            if (ptx::globaltimer_ns() - t0 > 2000000ull) break;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only in pair mode)
    if (lane == 0 && leader) {
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int tile = tile_first; ok && tile < total_tiles; tile += tile_step) {
        const Tile t = decode_tile<MAJOR, EPI, PAIR>(a, tile, n_tiles_n, pair_prefix);
        if (t.kb == 0) continue;
        const uint32_t acc = acc_it & 1u, acc_ph = (acc_it >> 1) & 1u;
        if (!ptx::mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!ptx::mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES;
#pragma unroll
          for (int j = 0; j < BK / 16; ++j) {
            const uint64_t da = ptx::smem_desc(a.desc_hi_a, sa + j * a.kstep_a);
            const uint64_t db = ptx::smem_desc(a.desc_hi_b, sb + j * a.kstep_b);
            if constexpr (PAIR) ptx::mma_bf16_pair(d_tmem, da, db, a.idesc, (kb > 0 || j > 0) ? 1u : 0u);
            else ptx::mma_bf16(d_tmem, da, db, a.idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          if constexpr (PAIR) ptx::mma_commit_pair(empty_bar(s), 3);
          else ptx::mma_commit(empty_bar(s));
        }
        if (!ok) break;
        if constexpr (PAIR) ptx::mma_commit_pair(tfull_bar(acc), 3);
        else ptx::mma_commit(tfull_bar(acc));
        ++acc_it;
      }
      if (*abort_flag) {
        // wait (bounded) until the tensor core has finished what was issued
        if constexpr (PAIR) ptx::mma_commit_pair(drain_bar, 1);
        else ptx::mma_commit(drain_bar);
        const unsigned long long t0 = ptx::globaltimer_ns();
        while (!ptx::mbar_try_wait(drain_bar, 0)) {
          if (ptx::globaltimer_ns() - t0 > 2000000ull) break;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int lane_grp = warp & 3;           // TMEM lanes 32*lane_grp .. +31 are readable by this warp
    const int col_half = (warp - 2) >> 2;    // which half of the tile's columns this warp stores
    uint8_t* stage = generic_base + RING_BYTES + (warp - 2) * staging_per_warp(EPI);
    uint32_t acc_it = 0;
    [[maybe_unused]] uint32_t epi_phase = 0;
    [[maybe_unused]] TileStager<2> out2buf{stage, 0};
    bool ok = true;
    for (int tile = tile_first; ok && tile < total_tiles; tile += tile_step) {
      const Tile t = decode_tile<MAJOR, EPI, PAIR>(a, tile, n_tiles_n, pair_prefix);
      const bool has_acc = t.kb > 0;
      // first row (of the output tensor) handled by this warp and how many of its 32 rows exist
      const long long wrow0 = (MAJOR == TN ? (long long)t.m0 : (long long)t.row0) + (long long)cta_rank * BM + lane_grp * 32;
      const long long row_lim = MAJOR == TN ? (long long)a.Ma : a.rows;
      int rows_valid = (int)max(0LL, min(32LL, row_lim - wrow0));
      if (MAJOR != TN && cta_rank == 1 && !t.second) rows_valid = 0;   // this CTA's block belongs to the next expert
      const int n_end = t.nlim;

      // DSWIGLU: this warp's 32 rows x 128 columns of g and u arrive, and dg and du leave, as TMA tiles of 32 rows x
      // 64 columns in the warp's two staging tiles: [g tile | u tile], results written in place.
      // Lane 0 issues the copies; the first pair of loads is in flight before the accumulator is waited for.
      [[maybe_unused]] const uint32_t tile_g = ptx::smem_u32(stage), tile_u = tile_g + TILE_BYTES;
      [[maybe_unused]] auto dsw_load = [&](int n) {
        if (lane == 0) {
          ptx::bulk_wait_read();   // the stores of the previous half have finished reading the staging tiles
          ptx::mbar_expect_tx(epi_bar(warp - 2), 2 * TILE_BYTES);
          ptx::tma_load_3d(tile_g, &tm_c, epi_bar(warp - 2), n, 0, (int)wrow0);
          ptx::tma_load_3d(tile_u, &tm_c, epi_bar(warp - 2), n, 1, (int)wrow0);
        }
      };
      if constexpr (EPI == DSWIGLU) {
        if (rows_valid > 0 && t.n0 + col_half * 128 < n_end) dsw_load(t.n0 + col_half * 128);
      }

      // What the epilogue needs per row besides the accumulator is fetched now, while the tensor cores still work on
      // the tile: the row's scale (a dependent pair of loads under SWIGLU / DSWIGLU), rank-one factor or destination.
      [[maybe_unused]] float row_sc = 1.0f, row_r1 = 0.f;
      [[maybe_unused]] unsigned long long my_dst = 0;
      if (lane < rows_valid) {
        if constexpr (EPI == PLAIN) {
          if (a.row_scale != nullptr) row_sc = a.row_scale[wrow0 + lane];
          if (a.r1_row != nullptr) row_r1 = a.r1_row[wrow0 + lane];
        } else if constexpr (EPI == SWIGLU || EPI == DSWIGLU) {
          if (a.scale_src != nullptr) {
            const long long gi = a.scale_idx != nullptr ? (long long)a.scale_idx[wrow0 + lane] : wrow0 + lane;
            row_sc = gi >= 0 ? a.scale_src[gi] : 0.f;
          }
        } else if constexpr (EPI == SCATTER) {
          const int code = a.ret[wrow0 + lane];
          if (code >= 0) {
            const int rank = code >> kRetSlotBits;
            const long long slot = code & ((1 << kRetSlotBits) - 1);
            if (rank < a.ret_ranks && slot < a.ret_slots)
              my_dst = reinterpret_cast<unsigned long long>(a.ret_out[rank]) + (unsigned long long)slot * a.N * 2;
            else
              raise_status(LEWI_STATUS_BAD_INDEX);
          }
        }
      } else if constexpr (EPI == SWIGLU || EPI == DSWIGLU) {
        if (a.scale_src != nullptr) row_sc = 0.f;
      }

      uint32_t acc = 0;
      bool acc_held = false;
      // The accumulator goes back to the MMA warp as soon as this warp has read its last piece of it, before that
      // piece is converted and stored.
      auto release_acc = [&]() {
        if (!acc_held) return;
        acc_held = false;
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar(acc), 0));
          else ptx::mbar_arrive(tempty_bar(acc));
        }
      };
      if (has_acc) {
        acc_held = true;
        acc = acc_it & 1u;
        const uint32_t acc_ph = (acc_it >> 1) & 1u;
        const bool got = ptx::mbar_wait(tfull_bar(acc), acc_ph, abort_flag);
        __syncwarp();
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        ptx::tc_fence_after();
      }
      const uint32_t t_addr = tmem_base + acc * BN + ((uint32_t)(lane_grp * 32) << 16);

      if constexpr (EPI == PLAIN) {
        // out [rows, N] through tm_c: bf16 tiles of 64 columns or f32 tiles of 32 columns
        if (rows_valid > 0) {
          const float sc = row_sc, r1 = row_r1;
          uint8_t* buf = nullptr;
#pragma unroll 1
          for (int c = col_half * 4; c < col_half * 4 + 4; ++c) {
            const int n = t.n0 + c * 32;
            if (n >= n_end) break;  // uniform across the warp
            const int cv = min(32, a.N - n);
            uint32_t r[32];
            float v[32];
            if (has_acc) {
              ptx::tmem_ld_32x32(t_addr + c * 32, r);
              ptx::tmem_ld_wait();
              if (c == col_half * 4 + 3 || n + 32 >= n_end) release_acc();
            }
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = has_acc ? __uint_as_float(r[q]) * sc : 0.f;
            if (a.col_bias != nullptr) {
#pragma unroll
              for (int q = 0; q < 32; ++q) v[q] += (q < cv) ? a.col_bias[n + q] : 0.f;
            }
            if (a.r1_row != nullptr) {
#pragma unroll
              for (int q = 0; q < 32; ++q) v[q] += (q < cv) ? r1 * a.r1_col[n + q] : 0.f;
            }
            if (a.out_f32) {
              buf = out2buf.acquire(lane);
              tile_put_f32x32(buf, lane, v);
              out2buf.store2d(lane, &tm_c, buf, n, (int)wrow0);
            } else {
              if ((c & 1) == 0) buf = out2buf.acquire(lane);
              tile_put_bf16x32(buf, lane, (c & 1) * 4, v);
              // a 64-column tile is complete after its odd 32-column block, or when the row ends inside it
              if ((c & 1) == 1 || n + 32 >= n_end) out2buf.store2d(lane, &tm_c, buf, n - (c & 1) * 32, (int)wrow0);
            }
          }
        }
      } else if constexpr (EPI == SWIGLU) {
        // h [rows, f] through tm_c, gu [rows][2][f] through tm_d; this warp owns 64 h columns: three 4 KB tiles
        const int f = a.N;
        const int n64 = t.n0 + col_half * 64;
        if (rows_valid > 0 && n64 < n_end) {
          const float hsc = row_sc;
          if (lane == 0) ptx::bulk_wait_read();   // the previous tile's three stores have read the staging tiles
          __syncwarp();
          uint8_t* buf_g = stage;
          uint8_t* buf_u = stage + TILE_BYTES;
          uint8_t* buf_h = stage + 2 * TILE_BYTES;
#pragma unroll 1
          for (int b = 0; b < 2; ++b) {
            const int c = col_half * 2 + b;
            if (t.n0 + c * 32 >= n_end) break;
            uint32_t rg[32], ru[32];
            if (has_acc) {
              ptx::tmem_ld_32x32(t_addr + c * 32, rg);
              ptx::tmem_ld_32x32(t_addr + BN / 2 + c * 32, ru);
              ptx::tmem_ld_wait();
            }
            float g[32], u[32];
#pragma unroll
            for (int q = 0; q < 32; ++q) {
              g[q] = has_acc ? __uint_as_float(rg[q]) : 0.f;
              u[q] = has_acc ? __uint_as_float(ru[q]) : 0.f;
            }
            if (a.out2 != nullptr) {
              tile_put_bf16x32(buf_g, lane, b * 4, g);
              tile_put_bf16x32(buf_u, lane, b * 4, u);
            }
#pragma unroll
            for (int q = 0; q < 32; ++q) g[q] = g[q] * fast_sigmoid(g[q]) * u[q] * hsc;
            tile_put_bf16x32(buf_h, lane, b * 4, g);
          }
          ptx::fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            if (a.out2 != nullptr) {
              ptx::tma_store_3d(&tm_d, ptx::smem_u32(buf_g), n64, 0, (int)wrow0);
              ptx::tma_store_3d(&tm_d, ptx::smem_u32(buf_u), n64, 1, (int)wrow0);
            }
            ptx::tma_store_2d(&tm_c, ptx::smem_u32(buf_h), n64, (int)wrow0);
            ptx::bulk_commit();
          }
        }
      } else if constexpr (EPI == DSWIGLU) {
        const int f = a.N;
        const float dsc = row_sc;
        float dw_acc = 0.f;
        uint8_t* my_g = stage + lane * 128;   // this lane's row of the swizzled g tile; the u tile is 4 KB further
#pragma unroll 1
        for (int hf = 0; hf < 2 && ok; ++hf) {
          const int nh = t.n0 + col_half * 128 + hf * 64;
          if (rows_valid == 0 || nh >= n_end) break;   // uniform across the warp
          if (hf == 1) dsw_load(nh);
          const bool got = ptx::mbar_wait(epi_bar(warp - 2), epi_phase, abort_flag);
          epi_phase ^= 1u;
          __syncwarp();
          if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
#pragma unroll 1
          for (int b = 0; b < 2; ++b) {
            const int c = col_half * 4 + hf * 2 + b;
            float g[32], u[32];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int off = ((b * 4 + q) ^ (lane & 7)) << 4;
              const uint4 pg = *reinterpret_cast<const uint4*>(my_g + off);
              const uint4 pu = *reinterpret_cast<const uint4*>(my_g + TILE_BYTES + off);
              g[q * 8 + 0] = bf16_lo(pg.x); g[q * 8 + 1] = bf16_hi(pg.x); g[q * 8 + 2] = bf16_lo(pg.y); g[q * 8 + 3] = bf16_hi(pg.y);
              g[q * 8 + 4] = bf16_lo(pg.z); g[q * 8 + 5] = bf16_hi(pg.z); g[q * 8 + 6] = bf16_lo(pg.w); g[q * 8 + 7] = bf16_hi(pg.w);
              u[q * 8 + 0] = bf16_lo(pu.x); u[q * 8 + 1] = bf16_hi(pu.x); u[q * 8 + 2] = bf16_lo(pu.y); u[q * 8 + 3] = bf16_hi(pu.y);
              u[q * 8 + 4] = bf16_lo(pu.z); u[q * 8 + 5] = bf16_hi(pu.z); u[q * 8 + 6] = bf16_lo(pu.w); u[q * 8 + 7] = bf16_hi(pu.w);
            }
            uint32_t r[32];
            if (has_acc) {
              ptx::tmem_ld_32x32(t_addr + c * 32, r);
              ptx::tmem_ld_wait();
            }
#pragma unroll
            for (int q = 0; q < 32; ++q) {
              const float dh0 = has_acc ? __uint_as_float(r[q]) : 0.f;
              const float sg = fast_sigmoid(g[q]);
              dw_acc = fmaf(dh0, g[q] * sg * u[q], dw_acc);
              const float dh = dh0 * dsc;
              const float du = dh * g[q] * sg;
              g[q] = dh * u[q] * sg * (1.0f + g[q] * (1.0f - sg));
              u[q] = du;
            }
            tile_put_bf16x32(stage, lane, b * 4, g);
            tile_put_bf16x32(stage + TILE_BYTES, lane, b * 4, u);
          }
          ptx::fence_proxy_async();   // the tiles were written through the generic proxy, the store reads them through the async one
          __syncwarp();
          if (lane == 0) {
            ptx::tma_store_3d(&tm_d, tile_g, nh, 0, (int)wrow0);
            ptx::tma_store_3d(&tm_d, tile_u, nh, 1, (int)wrow0);
            ptx::bulk_commit();
          }
        }
        if (a.dw_partial != nullptr && lane < rows_valid) {
          const int part = (t.n0 / BN) * 2 + col_half;
          if (part < a.dw_parts) a.dw_partial[(wrow0 + lane) * a.dw_parts + part] = dw_acc;
        }
      } else if constexpr (EPI == SCATTER) {
        // Every lane looks up where its row goes; the warp then fills a 64-column staging tile and stores it row by
        // row, 8 lanes per 128-byte row piece and 4 rows per instruction, with plain 16-byte stores (the destination
        // may be a peer's memory: the rows travel while the tensor cores work on the next tile).
        if (rows_valid > 0) {
#pragma unroll 1
          for (int c = col_half * 4; c < col_half * 4 + 4; ++c) {
            const int n = t.n0 + c * 32;
            if (n >= n_end) break;  // uniform across the warp
            uint32_t r[32];
            float v[32];
            if (has_acc) {
              ptx::tmem_ld_32x32(t_addr + c * 32, r);
              ptx::tmem_ld_wait();
              if (c == col_half * 4 + 3 || n + 32 >= n_end) release_acc();
            }
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = has_acc ? __uint_as_float(r[q]) : 0.f;
            uint8_t* buf = stage + ((c >> 1) & 1) * TILE_BYTES;
            tile_put_bf16x32(buf, lane, (c & 1) * 4, v);
            if ((c & 1) == 1 || n + 32 >= n_end) {
              __syncwarp();
              const int nb = n - (c & 1) * 32;   // first column of the staging tile
              const int piece = lane & 7;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int row = i * 4 + (lane >> 3);
                const unsigned long long dst = __shfl_sync(0xffffffffu, my_dst, row);
                if (dst != 0 && nb + piece * 8 < a.N) {
                  const uint4 val = *reinterpret_cast<const uint4*>(buf + row * 128 + ((piece ^ (row & 7)) << 4));
                  st_v4(reinterpret_cast<void*>(dst + (unsigned long long)(nb + piece * 8) * 2), val);
                }
              }
              __syncwarp();
            }
          }
        }
      } else {  // TNOUT
        // straight to the output ([E, Ma, N] through tm_c, or its two column halves through tm_c / tm_d), or one part
        // of an expert's product as f32 into `partial` ([slots, Ma, N] through tm_b2)
        if (rows_valid > 0) {
          const int half = a.out2 != nullptr ? a.N / 2 : a.N;
          const bool to_partial = t.split >= 0;
          const bool f32_out = to_partial || a.out_f32;
          uint8_t* buf = nullptr;
#pragma unroll 1
          for (int c = col_half * 4; c < col_half * 4 + 4; ++c) {
            const int n = t.n0 + c * 32;
            if (n >= n_end) break;
            uint32_t r[32];
            float v[32];
            if (has_acc) {
              ptx::tmem_ld_32x32(t_addr + c * 32, r);
              ptx::tmem_ld_wait();
              if (c == col_half * 4 + 3 || n + 32 >= n_end) release_acc();
            }
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] = has_acc ? __uint_as_float(r[q]) : 0.f;
            const CUtensorMap* tm = to_partial ? &tm_b2 : (n < half ? &tm_c : &tm_d);
            const int z = to_partial ? t.split : t.e;
            const int ncol = to_partial ? n : (n < half ? n : n - half);
            if (f32_out) {
              buf = out2buf.acquire(lane);
              tile_put_f32x32(buf, lane, v);
              out2buf.store3d(lane, tm, buf, ncol, (int)wrow0, z);
            } else {
              if ((c & 1) == 0) buf = out2buf.acquire(lane);
              tile_put_bf16x32(buf, lane, (c & 1) * 4, v);
              if ((c & 1) == 1 || n + 32 >= n_end) out2buf.store3d(lane, tm, buf, ncol - (c & 1) * 32, (int)wrow0, z);
            }
          }
        }
      }

      if (has_acc) {
        release_acc();   // (warps without rows or columns of this tile have not read it)
        ++acc_it;
      }
    }
    if (lane == 0) ptx::bulk_wait_all();   // this warp's last tile stores are complete before the CTA can exit
  }

  ptx::tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) ptx::cluster_sync();   // neither CTA leaves while the other may still touch its memory
  if (warp == 1) {
    __syncwarp();
    ptx::tc_fence_after();
    if constexpr (PAIR) ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Sums the k_splits partial products of a TN GEMM and writes the result in the output dtype.
__global__ void __launch_bounds__(256) tn_reduce_kernel(const float* __restrict__ partial, int splits, long long e_ma,
                                                        int N, void* out, void* out2, int out_f32) {
  const int half = out2 != nullptr ? N / 2 : N;
  const long long total4 = e_ma * N / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = reinterpret_cast<const float4*>(partial)[i];
    for (int s = 1; s < splits; ++s) {
      const float4 v = reinterpret_cast<const float4*>(partial)[i + (long long)s * total4];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const long long flat = i * 4;
    const long long r = flat / N;
    const int n = (int)(flat - r * N);
    void* base = n < half ? out : out2;
    const long long off = r * half + (n < half ? n : n - half);
    if (out_f32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off) = acc;
    } else {
      uint2 pk = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(base) + off) = pk;
    }
  }
}

// Ragged split (tn_part_rows > 0): sums the parts of every expert that has more than one, in part order, and writes
// the expert's product in the output dtype.  grid = (column chunks, E); experts with one part were stored directly.
__global__ void __launch_bounds__(256) tn_reduce_ragged_kernel(const float* __restrict__ partial,
                                                               const int32_t* __restrict__ pad_offsets, int E,
                                                               int part_rows, long long ma, int N, void* out, void* out2,
                                                               int out_f32) {
  __shared__ int s_base;
  const int e = blockIdx.y;
  const int rows_e = pad_offsets[e + 1] - pad_offsets[e];
  const int n_parts = (rows_e + part_rows - 1) / part_rows;
  if (n_parts <= 1) return;
  if (threadIdx.x == 0) {
    int extra = 0;   // parts beyond the first of all experts before e
    for (int x = 0; x < e; ++x) {
      const int r = pad_offsets[x + 1] - pad_offsets[x];
      extra += max(1, (r + part_rows - 1) / part_rows) - 1;
    }
    s_base = 2 * extra;
  }
  __syncthreads();
  const long long per = ma * N;               // elements of one expert's product
  const long long total4 = per / 4;
  const float4* src = reinterpret_cast<const float4*>(partial) + (long long)s_base * total4;
  const int half = out2 != nullptr ? N / 2 : N;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = src[i];
    for (int p = 1; p < n_parts; ++p) {
      const float4 v = src[i + (long long)p * total4];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const long long flat = i * 4;
    const long long r = flat / N;
    const int n = (int)(flat - r * N);
    void* base = n < half ? out : out2;
    const long long off = ((long long)e * ma + r) * half + (n < half ? n : n - half);
    if (out_f32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off) = acc;
    } else {
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(base) + off) =
          make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
  }
}

// ------------------------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// bf16 (or f32) tensor [d2][d1][d0] (d0 contiguous); box [b2][b1][b0]; rank 2 when d2 == 0.
inline bool make_map(CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0,
                     uint32_t b1, uint32_t b2 = 1, bool f32 = false) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || d0 == 0 || d1 == 0) return false;
  const uint64_t esz = f32 ? 4 : 2;
  cuuint64_t dims[3] = {d0, d1, d2 ? d2 : 1};
  cuuint64_t strides[2] = {d0 * esz, d0 * d1 * esz};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  const cuuint32_t rank = d2 ? 3 : 2;
  CUresult r = fn(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank,
                  const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Tensor map of an epilogue output [d2][rows][cols]: boxes of 32 rows x 128 bytes (64 bf16 or 32 f32 columns).
inline bool make_out_map(CUtensorMap* m, const void* ptr, uint64_t cols, uint64_t rows, uint64_t d2, bool f32) {
  return make_map(m, ptr, cols, rows, d2, f32 ? 32 : 64, 32, 1, f32);
}

// Shared-memory matrix-descriptor geometry (bytes) of the two operand layouts, both 128-byte swizzled.
struct DescGeometry {
  uint32_t k_lbo = 16, k_sbo = 1024, k_step = 32;          // K-major operand: rows of 128 bytes, 8-row groups 1 KB apart
  uint32_t mn_lbo = CHUNK_BYTES, mn_sbo = 1024, mn_step = 2048;  // MN-major operand: [64 k][64 mn] boxes 8 KB apart
};

// Whether the CTA-pair (cta_group::2) kernels are used where the arguments allow it.
inline bool& pair_mode() {
  static bool on = true;
  return on;
}

// Whether a GEMM CTA leaves its SM's last kilobytes of shared memory to a CTA of another kernel (see SMEM_BYTES).
// Off: the launch asks for 1 KB it does not use, so a GEMM CTA has its SM to itself.
inline bool& sm_sharing() {
  static bool on = false;
  return on;
}
constexpr size_t SMEM_EXCLUSIVE_PAD = 1024;

// Upper bound on the CTAs of the GEMM launches that follow (0: one per SM).  Two GEMMs launched on different streams
// with limits that add up to the SM count run side by side, each on its share of the GPU.
inline int& cta_limit() {
  static int n = 0;
  return n;
}

template <int MAJOR, int EPI, bool PAIR>
inline int launch(cudaStream_t st, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, Args a,
                  long long max_tiles, const CUtensorMap& tc, const CUtensorMap& td) {
  static bool attr_set[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return LEWI_ERR_CUDA;
  auto kern = grouped_gemm_kernel<MAJOR, EPI, PAIR>;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(SMEM_BYTES + SMEM_EXCLUSIVE_PAD)) != cudaSuccess) {
      (void)cudaGetLastError();
      return LEWI_ERR_CUDA;
    }
    attr_set[dev] = true;
  }
  const DescGeometry g;
  const bool a_mn = MAJOR == TN, b_mn = MAJOR != NT;
  a.desc_hi_a = a_mn ? ptx::smem_desc_hi_sw128(g.mn_lbo, g.mn_sbo) : ptx::smem_desc_hi_sw128(g.k_lbo, g.k_sbo);
  a.desc_hi_b = b_mn ? ptx::smem_desc_hi_sw128(g.mn_lbo, g.mn_sbo) : ptx::smem_desc_hi_sw128(g.k_lbo, g.k_sbo);
  a.kstep_a = a_mn ? g.mn_step : g.k_step;
  a.kstep_b = b_mn ? g.mn_step : g.k_step;
  a.idesc = ptx::instr_desc_bf16(PAIR ? 2 * BM : BM, BN, a_mn ? 1 : 0, b_mn ? 1 : 0);
  if (max_tiles <= 0) return LEWI_OK;
  const size_t smem = SMEM_BYTES + (sm_sharing() ? 0 : SMEM_EXCLUSIVE_PAD);
  long long grid = num_sms();
  if (cta_limit() > 0 && grid > cta_limit()) grid = cta_limit();
  if constexpr (PAIR) {
    grid &= ~1LL;
    if (grid > 2 * max_tiles) grid = 2 * max_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, ta, tb, tb2, tc, td, a) != cudaSuccess) {
      (void)cudaGetLastError();
      return LEWI_ERR_CUDA;
    }
  } else {
    if (grid > max_tiles) grid = max_tiles;
    kern<<<(int)grid, THREADS, smem, st>>>(ta, tb, tb2, tc, td, a);
  }
  LEWI_CHECK_LAUNCH();
  return LEWI_OK;
}

// Picks the CTA-pair kernel when enabled, else the single-CTA one.
template <int MAJOR, int EPI>
// tc / td: tensor maps of the epilogue's tiled outputs (dSwiGLU: its g|u input and dg|du output).
inline int launch_auto(bool pair, cudaStream_t st, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2,
                       const Args& a, long long max_tiles, const CUtensorMap* tc = nullptr,
                       const CUtensorMap* td = nullptr) {
  const CUtensorMap& c = tc != nullptr ? *tc : ta;
  const CUtensorMap& d = td != nullptr ? *td : ta;
  if (pair) return launch<MAJOR, EPI, true>(st, ta, tb, tb2, a, max_tiles, c, d);
  return launch<MAJOR, EPI, false>(st, ta, tb, tb2, a, max_tiles, c, d);
}

}  // namespace gg
}  // namespace lewi
