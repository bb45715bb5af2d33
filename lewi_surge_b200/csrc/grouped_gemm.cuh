// Grouped GEMMs over the padded-block layout on the 5th-generation tensor cores.
//
// One persistent, warp-specialised kernel per (operand-major, epilogue) combination:
//   warp 0      TMA producer: tiled cp.async.bulk.tensor loads (128-byte swizzle, no multicast)
//               into a 4-stage shared-memory ring;
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
// The dSwiGLU epilogue moves its g|u and dg|du blocks with TMA and needs 8 KB of staging per warp (two 32-row x
// 128-byte swizzled tiles); the others transpose 32x32 blocks through 4 KB.  The ring gets the rest.
__host__ __device__ constexpr int staging_per_warp(int epi) { return epi == 2 /* DSWIGLU */ ? 8192 : 4096; }
__host__ __device__ constexpr int ring_bytes(int epi) { return DATA_BYTES - EPI_WARPS * staging_per_warp(epi); }
constexpr int A_BYTES = BM * BK * 2;           // 16 KB
constexpr int CHUNK_BYTES = 64 * BK * 2;       // 8 KB: one [64 k][64 mn] box of an MN-major operand
// One CTA per tile (cta_group::1): B is 256 x 64 = 32 KB, 4 stages of 48 KB (3 under the dSwiGLU epilogue).
// A CTA pair per 256-row tile (cta_group::2): each CTA holds its own 128 rows of A and HALF of B
// (128 x 64 = 16 KB), 6 stages of 32 KB (5 under dSwiGLU); the tensor cores of both SMs read both halves.
template <bool PAIR, int EPI = 0> struct Cfg {
  static constexpr int B_BYTES = PAIR ? BN * BK : BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = ring_bytes(EPI) / STAGE_BYTES;
};
constexpr int MAX_STAGES = 6;
constexpr int PAIR_PREFIX_BYTES = 1040;        // uint16 prefix of row-block pairs per expert (E <= 512)
constexpr int GATHER_ROWS_BYTES = 512;         // source-row numbers of the tile being gathered
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int TMEM_COLS = 512;
constexpr int EPI_BAR_BYTES = 64;        // one mbarrier per epilogue warp (TMA loads of the dSwiGLU epilogue)
// 231,248 bytes.  An SM has 233,472 and every resident CTA reserves 1,024 of them, so exactly one more CTA that
// uses no shared memory (a gather or exchange kernel from another stream) fits beside a GEMM CTA.  That is why
// there is no slack for aligning the ring: the kernel asks for a 1024-byte aligned base and checks it.
constexpr size_t SMEM_BYTES = (size_t)DATA_BYTES + 256 /*barriers*/ + PAIR_PREFIX_BYTES + GATHER_ROWS_BYTES + EPI_BAR_BYTES;

enum Major { NN = 0, NT = 1, TN = 2 };
enum Epi { PLAIN = 0, SWIGLU = 1, DSWIGLU = 2, TNOUT = 3 };

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
  const int32_t* scale_idx;     // SWIGLU / DSWIGLU: padded row -> index into scale_src (negative: scale 0; null: the row itself)
  const float* scale_src;       // SWIGLU / DSWIGLU: optional f32 table indexed by scale_idx[row] (router weight of the
                                // row's slot); SWIGLU stores h * scale, DSWIGLU multiplies dh by it
  float* dw_partial;            // DSWIGLU: optional [rows, dw_parts] f32, sum over this warp's columns of
  int dw_parts;                 //   dh_unscaled * silu(g) * u  (= pieces of the routing-weight gradient)
  const void* ga_ptr;           // gathered A operand (bf16 rows picked through g_idx) or null: A comes through tm_a
  const void* gb_ptr;           // TN only: gathered B operand or null
  long long ga_ld, gb_ld;       // row strides (elements) of the gathered sources
  const int32_t* g_idx;         // padded row -> source index (negative = zero row)
  int g_div;                    // source row = index / g_div (slot -> token)
  int g_src_rows;               // rows of the gathered source (indices beyond it give zero rows)
  int dbg;                      // bring-up experiments only (0 in production): 1 no global I/O in the epilogue,
                                // 2 epilogue only hands the accumulator back, 4 the producer skips the B operand
  uint64_t desc_hi_a, desc_hi_b;
  uint32_t kstep_a, kstep_b;    // bytes to advance the descriptor start per 16-wide k step
  uint32_t idesc;
};

__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// ---- epilogue I/O.  A thread owns one row of the accumulator (TMEM lane = row), but a warp-wide
// store of "my row's 16 bytes" would touch 32 different lines.  Blocks of 32 rows x 32 columns are
// therefore transposed through a small swizzled staging buffer in shared memory so that every
// global load/store instruction covers whole 64- or 128-byte row segments.

// 32 x 32 f32 (one row per lane) -> bf16 rows of 64 bytes.  `base` points at (first row of the warp,
// first column of the block); rows >= rows_valid and 8-column groups >= cols_valid are skipped.
__device__ __forceinline__ void warp_store32_bf16(uint8_t* stage, int lane, const float* v, __nv_bfloat16* base,
                                                  long long ld, int rows_valid, int cols_valid) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 pk = make_uint4(pack_bf16(v[q * 8 + 0], v[q * 8 + 1]), pack_bf16(v[q * 8 + 2], v[q * 8 + 3]),
                          pack_bf16(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16(v[q * 8 + 6], v[q * 8 + 7]));
    *reinterpret_cast<uint4*>(stage + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) = pk;
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 8 + (lane >> 2), seg = lane & 3;
    const uint4 pk = *reinterpret_cast<const uint4*>(stage + r * 64 + ((seg ^ ((r >> 1) & 3)) << 4));
    if (r < rows_valid && seg * 8 < cols_valid) st_v4(base + r * ld + seg * 8, pk);
  }
  __syncwarp();
}

// 32 x 32 f32 (one row per lane) -> f32 rows of 128 bytes.
__device__ __forceinline__ void warp_store32_f32(uint8_t* stage, int lane, const float* v, float* base, long long ld,
                                                 int rows_valid, int cols_valid) {
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    uint4 pk = make_uint4(__float_as_uint(v[q * 4]), __float_as_uint(v[q * 4 + 1]), __float_as_uint(v[q * 4 + 2]),
                          __float_as_uint(v[q * 4 + 3]));
    *reinterpret_cast<uint4*>(stage + lane * 128 + ((q ^ (lane & 7)) << 4)) = pk;
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3), seg = lane & 7;
    const uint4 pk = *reinterpret_cast<const uint4*>(stage + r * 128 + ((seg ^ (r & 7)) << 4));
    if (r < rows_valid && seg * 4 < cols_valid) st_v4(base + r * ld + seg * 4, pk);
  }
  __syncwarp();
}

// Coalesced read of a 32 x 32 bf16 block into registers (4 x 16 bytes per lane, not yet transposed).
__device__ __forceinline__ void warp_fetch32_bf16(int lane, const __nv_bfloat16* base, long long ld, int rows_valid,
                                                  int cols_valid, uint4 (&t)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 8 + (lane >> 2), seg = lane & 3;
    t[i] = make_uint4(0, 0, 0, 0);
    if (r < rows_valid && seg * 8 < cols_valid) t[i] = ld_nc_v4(base + r * ld + seg * 8);
  }
}
// Registers of warp_fetch32_bf16 -> staging -> this lane's own row as 32 floats.
__device__ __forceinline__ void warp_own_row32_bf16(uint8_t* stage, int lane, const uint4 (&t)[4], float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 8 + (lane >> 2), seg = lane & 3;
    *reinterpret_cast<uint4*>(stage + r * 64 + ((seg ^ ((r >> 1) & 3)) << 4)) = t[i];
  }
  __syncwarp();
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint4 pk = *reinterpret_cast<const uint4*>(stage + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4));
    v[q * 8 + 0] = bf16_lo(pk.x); v[q * 8 + 1] = bf16_hi(pk.x);
    v[q * 8 + 2] = bf16_lo(pk.y); v[q * 8 + 3] = bf16_hi(pk.y);
    v[q * 8 + 4] = bf16_lo(pk.z); v[q * 8 + 5] = bf16_hi(pk.z);
    v[q * 8 + 6] = bf16_lo(pk.w); v[q * 8 + 7] = bf16_hi(pk.w);
  }
  __syncwarp();
}

struct Tile {
  int e;        // expert
  int second;   // pair mode, NN/NT: 1 if the second 128-row block of the pair belongs to the same expert
  int row0;     // first row of the row-indexed operand (NN/NT: A rows; TN: first contraction row)
  int m0;       // TN: first output row
  int n0;       // first accumulator column in output coordinates (SWIGLU: first h column)
  int nlim;     // columns >= nlim are not stored by this tile
  int kb0;      // first 64-wide contraction step of this tile
  int kb;       // number of 64-wide contraction steps
  int split;    // TN: index of the contraction part
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
    t.split = tile % a.k_splits;
    tile /= a.k_splits;
    t.e = tile / per_e;
    const int rem = tile - t.e * per_e;
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
    const int per = (kb_total + a.k_splits - 1) / a.k_splits;
    t.kb0 = t.split * per;
    t.kb = max(0, min(per, kb_total - t.kb0));
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
  auto gfull_bar = [&](int s) { return bar_base + 176u + 8u * s; };   // peer CTA: its own gathered rows of stage s
  uint8_t* generic_base = smem_raw;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(generic_base + DATA_BYTES + 160);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(generic_base + DATA_BYTES + 168);
  uint16_t* pair_prefix = reinterpret_cast<uint16_t*>(generic_base + DATA_BYTES + 256);
  int* gather_rows = reinterpret_cast<int*>(generic_base + DATA_BYTES + 256 + PAIR_PREFIX_BYTES);   // [128] source rows
  auto epi_bar = [&](int w) { return bar_base + 256u + PAIR_PREFIX_BYTES + GATHER_ROWS_BYTES + 8u * w; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = PAIR ? ptx::cluster_ctarank() : 0u;   // 0 = leader of the pair
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    const bool gathering = a.ga_ptr != nullptr || a.gb_ptr != nullptr;
    for (int s = 0; s < STAGES; ++s) {
      // one arrival posts the TMA byte count; gathering adds this CTA's 32 lanes and, in pair mode, one
      // forwarded arrival for the peer's lanes
      ptx::mbar_init(full_bar(s), 1 + (gathering ? 32 + (PAIR ? 1 : 0) : 0));
      ptx::mbar_init(empty_bar(s), 1);
      ptx::mbar_init(gfull_bar(s), 32);
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
    if constexpr (EPI == DSWIGLU) {
      ptx::prefetch_tensormap(&tm_c);
      ptx::prefetch_tensormap(&tm_d);
    }
  }
  int n_units = 0;  // NN/NT: row blocks (or pairs of row blocks) to process
  if constexpr (MAJOR != TN) {
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
    total_tiles = a.E * ((a.Ma + TM - 1) / TM) * n_tiles_n * a.k_splits;
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
    // Lane 0 posts the byte count and issues the tiled TMA loads.  A gathered operand (its rows are picked
    // through an index table instead of being materialised first) is copied by all 32 lanes with 16-byte
    // cp.async into the same 128-byte-swizzled layout a tiled TMA load would have written: row j of a tile
    // sits at j*128 bytes and its 16-byte piece c at ((c ^ (j & 7)) << 4).  Rows that do not exist
    // (padding, rows past the group) are zero-filled.  Each lane then lets the hardware arrive on the
    // stage's barrier when its copies have landed (cp.async.mbarrier.arrive.noinc), so nothing waits here.
    const bool gather_a = a.ga_ptr != nullptr, gather_b = a.gb_ptr != nullptr;
    const bool gathering = gather_a || gather_b;
    const int src_rows = a.g_src_rows;
    uint32_t it = 0;
    bool ok = true;
    auto src_of = [&](int v) {
      if (v < 0) return -1;
      v /= a.g_div;
      return v < src_rows ? v : -1;
    };
    const int piece = lane & 7, rsub = lane >> 3;
    for (int tile = tile_first; ok && tile < total_tiles; tile += tile_step) {
      const Tile t = decode_tile<MAJOR, EPI, PAIR>(a, tile, n_tiles_n, pair_prefix);
      // TN: queue of the next stages' row indices (lanes 0-15 hold four consecutive k-rows each)
      [[maybe_unused]] int4 q0 = make_int4(-1, -1, -1, -1), q1 = q0, q2 = q0, q3 = q0;
      [[maybe_unused]] long long tn_r_end = 0;
      auto tn_idx = [&](int kb) {
        const long long r = (long long)t.row0 + (long long)(t.kb0 + kb) * BK + 4 * (lane & 15);
        int4 v = make_int4(-1, -1, -1, -1);
        if (lane < 16 && kb < t.kb) {
          if (r + 3 < tn_r_end) {
            v = *reinterpret_cast<const int4*>(a.g_idx + r);
          } else {
            if (r < tn_r_end) v.x = a.g_idx[r];
            if (r + 1 < tn_r_end) v.y = a.g_idx[r + 1];
            if (r + 2 < tn_r_end) v.z = a.g_idx[r + 2];
          }
        }
        return v;
      };
      if (gathering) {
        if constexpr (MAJOR != TN) {
          // source rows of this CTA's 128 tile rows -> shared memory (lane writes rows 4*lane .. +3)
          const long long r = (long long)t.row0 + (long long)cta_rank * BM + 4 * lane;
          int4 v = make_int4(-1, -1, -1, -1);
          if (r + 3 < a.rows) {
            v = *reinterpret_cast<const int4*>(a.g_idx + r);
          } else {
            if (r < a.rows) v.x = a.g_idx[r];
            if (r + 1 < a.rows) v.y = a.g_idx[r + 1];
            if (r + 2 < a.rows) v.z = a.g_idx[r + 2];
          }
          __syncwarp();
          *reinterpret_cast<int4*>(gather_rows + 4 * lane) = make_int4(src_of(v.x), src_of(v.y), src_of(v.z), src_of(v.w));
          __syncwarp();
        } else {
          tn_r_end = a.pad_offsets != nullptr ? (long long)a.pad_offsets[t.e + 1] : a.rows;
          q0 = tn_idx(0); q1 = tn_idx(1); q2 = tn_idx(2); q3 = tn_idx(3);
        }
      }
      for (int kb = 0; kb < t.kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1u;
        bool got = true;
        if (lane == 0 || gathering) got = ptx::mbar_wait(empty_bar(s), ph ^ 1u, abort_flag);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES;
        const bool skip_b = (a.dbg & 4) != 0;
        const int nb0 = t.n0 + (PAIR ? (int)cta_rank * (BN / 2) : 0);   // first B column/row held by this CTA
        if (lane == 0) {
          const uint32_t cta_bytes = (gather_a ? 0 : A_BYTES) + ((skip_b || gather_b) ? 0 : Cfg<PAIR, EPI>::B_BYTES);
          // in pair mode the peer gathers the same operands, so both CTAs bring the same TMA byte count
          if (leader) ptx::mbar_expect_tx(full_bar(s), PAIR ? 2 * cta_bytes : cta_bytes);
          const uint32_t fb = full_target(s);
          auto load2 = [&](uint32_t dst, const CUtensorMap* tm, int c0, int c1) {
            if constexpr (PAIR) ptx::tma_load_2d_pair(dst, tm, fb, c0, c1); else ptx::tma_load_2d(dst, tm, fb, c0, c1);
          };
          auto load3 = [&](uint32_t dst, const CUtensorMap* tm, int c0, int c1, int c2) {
            if (skip_b) return;   // every 3-D load is a B-operand load
            if constexpr (PAIR) ptx::tma_load_3d_pair(dst, tm, fb, c0, c1, c2); else ptx::tma_load_3d(dst, tm, fb, c0, c1, c2);
          };
          if constexpr (MAJOR == TN) {
            const int r = t.row0 + (t.kb0 + kb) * BK;
            const int ma0 = t.m0 + (int)cta_rank * BM;
            if (!gather_a) {
#pragma unroll
              for (int c = 0; c < 2; ++c) load2(sa + c * CHUNK_BYTES, &tm_a, ma0 + 64 * c, r);
            }
            if (!gather_b && !skip_b) {
#pragma unroll
              for (int c = 0; c < B_CHUNKS; ++c) load2(sb + c * CHUNK_BYTES, &tm_b, nb0 + 64 * c, r);
            }
          } else {
            int ka = kb * BK;
            if constexpr (MAJOR == NN) {
              if (a.a_k_wrap > 0) ka %= a.a_k_wrap;
            } else {
              if (kb >= a.kb_split) ka = a.k2_offset + (kb - a.kb_split) * BK;
            }
            if (!gather_a) load2(sa, &tm_a, ka, t.row0 + (int)cta_rank * BM);
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
        if (gathering) {
          if constexpr (MAJOR != TN) {
            // A tile [128 rows][64 k]
            const int col = kb * BK + piece * 8;
            const bool col_ok = col < a.K;
            const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(a.ga_ptr);
#pragma unroll 8
            for (int i = 0; i < 32; ++i) {
              const int j = i * 4 + rsub;
              const int sr = gather_rows[j];
              const bool v = sr >= 0 && col_ok;
              const __nv_bfloat16* src = v ? base + (long long)sr * a.ga_ld + col : base;
              ptx::cp_async16(sa + j * 128 + ((piece ^ (j & 7)) << 4), src, v);
            }
          } else {
            // MN-major chunks [64 k-rows][64 columns]: k-row j of the stage is padded row r0 + j
            __syncwarp();
            if (lane < 16) *reinterpret_cast<int4*>(gather_rows + 4 * lane) = make_int4(src_of(q0.x), src_of(q0.y), src_of(q0.z), src_of(q0.w));
            q0 = q1; q1 = q2; q2 = q3; q3 = tn_idx(kb + 4);
            __syncwarp();
            auto gather_chunks = [&](uint32_t dst0, int n_chunks, const void* ptr, long long ld, int col0, int width) {
              const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(ptr);
              for (int c = 0; c < n_chunks; ++c) {
                const int col = col0 + 64 * c + piece * 8;
                const bool col_ok = col < width;
#pragma unroll 8
                for (int i = 0; i < 16; ++i) {
                  const int j = i * 4 + rsub;
                  const int sr = gather_rows[j];
                  const bool v = sr >= 0 && col_ok;
                  const __nv_bfloat16* src = v ? base + (long long)sr * ld + col : base;
                  ptx::cp_async16(dst0 + c * CHUNK_BYTES + j * 128 + ((piece ^ (j & 7)) << 4), src, v);
                }
              }
            };
            if (gather_a) gather_chunks(sa, 2, a.ga_ptr, a.ga_ld, t.m0 + (int)cta_rank * BM, a.Ma);
            if (gather_b && !skip_b) gather_chunks(sb, B_CHUNKS, a.gb_ptr, a.gb_ld, nb0, a.N);
          }
          // the hardware arrives for this lane once its copies above have landed
          ptx::cp_async_arrive_noinc((PAIR && !leader) ? gfull_bar(s) : full_bar(s));
        }
      }
    }
    if (gathering) ptx::cp_async_wait<0>();   // nothing of this warp is in flight when shared memory is released
    if (lane == 0 && *abort_flag && leader) {
      // give the copies already issued a bounded chance to land before shared memory is released
      const uint32_t first = it > STAGES ? it - STAGES : 0;
      for (uint32_t j = first; j < it; ++j) {
        const unsigned long long t0 = ptx::globaltimer_ns();
        while (!ptx::mbar_try_wait(full_bar(j % STAGES), (j / STAGES) & 1u)) {
          if (ptx::globaltimer_ns() - t0 > 2000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only in pair mode)
    const bool gathering = a.ga_ptr != nullptr || a.gb_ptr != nullptr;
    if (PAIR && lane == 0 && !leader && gathering) {
      // Peer CTA: its gathered rows are announced on its own barrier (cp.async can only arrive locally);
      // this otherwise idle thread forwards each completed stage to the leader's full barrier.
      uint32_t it = 0;
      bool ok = true;
      for (int tile = tile_first; ok && tile < total_tiles; tile += tile_step) {
        const Tile t = decode_tile<MAJOR, EPI, PAIR>(a, tile, n_tiles_n, pair_prefix);
        for (int kb = 0; kb < t.kb; ++kb, ++it) {
          const int s = it % STAGES;
          if (!ptx::mbar_wait(gfull_bar(s), (it / STAGES) & 1u, abort_flag)) { ok = false; break; }
          ptx::fence_proxy_async();
          ptx::mbar_arrive_cluster(ptx::map_to_cta(full_bar(s), 0));
        }
      }
    }
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
          if (gathering) ptx::fence_proxy_async();   // cp.async wrote through the generic proxy, the MMA reads through the async one
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
    bool ok = true;
    for (int tile = tile_first; ok && tile < total_tiles; tile += tile_step) {
      const Tile t = decode_tile<MAJOR, EPI, PAIR>(a, tile, n_tiles_n, pair_prefix);
      const bool has_acc = t.kb > 0;
      // first row (of the output tensor) handled by this warp and how many of its 32 rows exist
      const long long wrow0 = (MAJOR == TN ? (long long)t.m0 : (long long)t.row0) + (long long)cta_rank * BM + lane_grp * 32;
      const long long row_lim = MAJOR == TN ? (long long)a.Ma : a.rows;
      int rows_valid = (int)max(0LL, min(32LL, row_lim - wrow0));
      if (MAJOR != TN && cta_rank == 1 && !t.second) rows_valid = 0;   // this CTA's block belongs to the next expert
      if (a.dbg & 3) rows_valid = 0;
      const int n_end = (a.dbg & 2) ? 0 : t.nlim;

      // DSWIGLU: this warp's 32 rows x 128 columns of g and u arrive, and dg and du leave, as TMA tiles of 32 rows x
      // 64 columns (128-byte swizzle) in the warp's 8 KB of staging: [g tile | u tile], results written in place.
      // Lane 0 issues the copies; the first pair of loads is in flight before the accumulator is waited for.
      [[maybe_unused]] const uint32_t tile_g = ptx::smem_u32(stage), tile_u = tile_g + 4096;
      [[maybe_unused]] auto dsw_load = [&](int n) {
        if (lane == 0) {
          ptx::bulk_wait_read();   // the stores of the previous half have finished reading the staging tiles
          ptx::mbar_expect_tx(epi_bar(warp - 2), 8192);
          ptx::tma_load_3d(tile_g, &tm_c, epi_bar(warp - 2), n, 0, (int)wrow0);
          ptx::tma_load_3d(tile_u, &tm_c, epi_bar(warp - 2), n, 1, (int)wrow0);
        }
      };
      if constexpr (EPI == DSWIGLU) {
        if (rows_valid > 0 && t.n0 + col_half * 128 < n_end) dsw_load(t.n0 + col_half * 128);
      }

      uint32_t acc = 0;
      if (has_acc) {
        acc = acc_it & 1u;
        const uint32_t acc_ph = (acc_it >> 1) & 1u;
        const bool got = ptx::mbar_wait(tfull_bar(acc), acc_ph, abort_flag);
        __syncwarp();
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        ptx::tc_fence_after();
      }
      const uint32_t t_addr = tmem_base + acc * BN + ((uint32_t)(lane_grp * 32) << 16);

      if constexpr (EPI == PLAIN) {
        const long long grow = wrow0 + lane;
        const float sc = (a.row_scale != nullptr && lane < rows_valid) ? a.row_scale[grow] : 1.0f;
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
          }
#pragma unroll
          for (int q = 0; q < 32; ++q) v[q] = has_acc ? __uint_as_float(r[q]) * sc : 0.f;
          if (a.col_bias != nullptr) {
#pragma unroll
            for (int q = 0; q < 32; ++q) v[q] += (q < cv) ? a.col_bias[n + q] : 0.f;
          }
          if (a.out_f32) warp_store32_f32(stage, lane, v, reinterpret_cast<float*>(a.out) + wrow0 * a.N + n, a.N, rows_valid, cv);
          else warp_store32_bf16(stage, lane, v, reinterpret_cast<__nv_bfloat16*>(a.out) + wrow0 * a.N + n, a.N, rows_valid, cv);
        }
      } else if constexpr (EPI == SWIGLU) {
        const int f = a.N;
        float hsc = 1.0f;
        if (a.scale_src != nullptr) {
          hsc = 0.f;
          if (lane < rows_valid) {
            const long long gi = a.scale_idx != nullptr ? (long long)a.scale_idx[wrow0 + lane] : wrow0 + lane;
            if (gi >= 0) hsc = a.scale_src[gi];
          }
        }
#pragma unroll 1
        for (int c = col_half * 2; c < col_half * 2 + 2; ++c) {
          const int n = t.n0 + c * 32;
          if (n >= n_end) break;
          const int cv = min(32, f - n);
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
            __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(a.out2) + wrow0 * (2LL * f);
            warp_store32_bf16(stage, lane, g, gu + n, 2LL * f, rows_valid, cv);
            warp_store32_bf16(stage, lane, u, gu + f + n, 2LL * f, rows_valid, cv);
          }
#pragma unroll
          for (int q = 0; q < 32; ++q) g[q] = g[q] * fast_sigmoid(g[q]) * u[q] * hsc;
          warp_store32_bf16(stage, lane, g, reinterpret_cast<__nv_bfloat16*>(a.out) + wrow0 * f + n, f, rows_valid, cv);
        }
      } else if constexpr (EPI == DSWIGLU) {
        const int f = a.N;
        float dsc = 1.0f, dw_acc = 0.f;
        if (a.scale_src != nullptr) {
          dsc = 0.f;
          if (lane < rows_valid) {
            const long long gi = a.scale_idx != nullptr ? (long long)a.scale_idx[wrow0 + lane] : wrow0 + lane;
            if (gi >= 0) dsc = a.scale_src[gi];
          }
        }
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
              const uint4 pu = *reinterpret_cast<const uint4*>(my_g + 4096 + off);
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
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int off = ((b * 4 + q) ^ (lane & 7)) << 4;
              *reinterpret_cast<uint4*>(my_g + off) =
                  make_uint4(pack_bf16(g[q * 8 + 0], g[q * 8 + 1]), pack_bf16(g[q * 8 + 2], g[q * 8 + 3]),
                             pack_bf16(g[q * 8 + 4], g[q * 8 + 5]), pack_bf16(g[q * 8 + 6], g[q * 8 + 7]));
              *reinterpret_cast<uint4*>(my_g + 4096 + off) =
                  make_uint4(pack_bf16(u[q * 8 + 0], u[q * 8 + 1]), pack_bf16(u[q * 8 + 2], u[q * 8 + 3]),
                             pack_bf16(u[q * 8 + 4], u[q * 8 + 5]), pack_bf16(u[q * 8 + 6], u[q * 8 + 7]));
            }
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
      } else {  // TNOUT
        const int half = a.out2 != nullptr ? a.N / 2 : a.N;
#pragma unroll 1
        for (int c = col_half * 4; c < col_half * 4 + 4; ++c) {
          const int n = t.n0 + c * 32;
          if (n >= n_end) break;
          const int cv = min(32, t.nlim - n);
          uint32_t r[32];
          float v[32];
          if (has_acc) {
            ptx::tmem_ld_32x32(t_addr + c * 32, r);
            ptx::tmem_ld_wait();
          }
#pragma unroll
          for (int q = 0; q < 32; ++q) v[q] = has_acc ? __uint_as_float(r[q]) : 0.f;
          if (a.k_splits > 1) {
            float* dst = a.partial + (((long long)t.split * a.E + t.e) * a.Ma + wrow0) * a.N + n;
            warp_store32_f32(stage, lane, v, dst, a.N, rows_valid, cv);
          } else {
            void* base = (n < half) ? a.out : a.out2;
            const long long off = ((long long)t.e * a.Ma + wrow0) * half + (n < half ? n : n - half);
            if (a.out_f32) warp_store32_f32(stage, lane, v, reinterpret_cast<float*>(base) + off, half, rows_valid, cv);
            else warp_store32_bf16(stage, lane, v, reinterpret_cast<__nv_bfloat16*>(base) + off, half, rows_valid, cv);
          }
        }
      }

      if (has_acc) {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar(acc), 0));
          else ptx::mbar_arrive(tempty_bar(acc));
        }
        ++acc_it;
      }
    }
    if constexpr (EPI == DSWIGLU) {
      if (lane == 0) ptx::bulk_wait_all();   // this warp's last tile stores are complete before the CTA can exit
    }
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

// bf16 tensor [d2][d1][d0] (d0 contiguous); box [b2][b1][b0]; rank 2 when d2 == 0.
inline bool make_map(CUtensorMap* m, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0,
                     uint32_t b1, uint32_t b2 = 1) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || d0 == 0 || d1 == 0) return false;
  cuuint64_t dims[3] = {d0, d1, d2 ? d2 : 1};
  cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  const cuuint32_t rank = d2 ? 3 : 2;
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Descriptor geometry (bytes).  Overridable for bring-up through lewi_debug_set_desc().
struct DescGeometry {
  uint32_t k_lbo = 16, k_sbo = 1024, k_step = 32;          // K-major operand, 128-byte swizzle
  uint32_t mn_lbo = CHUNK_BYTES, mn_sbo = 1024, mn_step = 2048;  // MN-major operand
};
inline DescGeometry& desc_geometry() {
  static DescGeometry g;
  return g;
}

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
  const DescGeometry& g = desc_geometry();
  const bool a_mn = MAJOR == TN, b_mn = MAJOR != NT;
  a.desc_hi_a = a_mn ? ptx::smem_desc_hi_sw128(g.mn_lbo, g.mn_sbo) : ptx::smem_desc_hi_sw128(g.k_lbo, g.k_sbo);
  a.desc_hi_b = b_mn ? ptx::smem_desc_hi_sw128(g.mn_lbo, g.mn_sbo) : ptx::smem_desc_hi_sw128(g.k_lbo, g.k_sbo);
  a.kstep_a = a_mn ? g.mn_step : g.k_step;
  a.kstep_b = b_mn ? g.mn_step : g.k_step;
  a.idesc = ptx::instr_desc_bf16(PAIR ? 2 * BM : BM, BN, a_mn ? 1 : 0, b_mn ? 1 : 0);
  if (max_tiles <= 0) return LEWI_OK;
  const size_t smem = SMEM_BYTES + (sm_sharing() ? 0 : SMEM_EXCLUSIVE_PAD);
  long long grid = num_sms();
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
// tc / td: tensor maps of the epilogue's own tiled input and output (dSwiGLU: g|u and dg|du); unused otherwise.
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
