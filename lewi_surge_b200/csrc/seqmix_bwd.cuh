// Chunked gated delta rule, backward.  Forward definitions and notation: seqmix.cuh.
//
// The roundings to bf16 of the forward pass are kept in the values and treated as the identity in the derivative
// (what automatic differentiation of the reference's forward does with its casts).  Per chunk, with
//   kb = bf16(k beta), vb = bf16(v beta), E = exp(gcs), D_ij = exp(gcs_i - gcs_j), kg = kb E, qE = q E,
//   kd = k exp(gcs_last - gcs), S = strict(bf16(kb k^T) D), A = (I + S)^-1, u = bf16(A vb), w = bf16(A kg),
//   attn = lower(bf16(q k^T) D), v_new = u - w h_in,
// and the upstream gradients do (of o) and dh (of the state after the chunk):
//   dv_new = attn^T do + kd dh                      dh_in = qE^T do + dh exp(gcs_last) - w^T dv_new
//   dattn  = lower(do v_new^T)                      dqE = do h_in^T      dkd = v_new dh^T      dw = -dv_new h_in^T
//   dq = (dqE E + (dattn D) k) scale                dk = dkd exp(gcs_last - gcs) + (dattn D)^T q + dP^T kb + dkb beta
//   dA = dv_new vb^T + dw kg^T                      dvb = A^T dv_new     dkg = A^T dw
//   dS = -strict(A^T dA A^T)    dP = dS D           dkb = dkg E + dP k
//   dv = dvb beta               dbeta = rowsum(dkb k) + rowsum(dvb v)
//   dgcs = rowsum(dqE qE) - rowsum(dkd kd) + rowsum(G) - colsum(G) + rowsum(dkg kg)      with G = dattn attn + dS S,
//   dgcs_last += exp(gcs_last) <dh, h_in> + sum(dkd kd);        dg = reverse cumulative sum of dgcs inside the chunk.
//
// Kernel 1 (one CTA per batch, head and 32 state columns) first runs the forward recurrence again to store the state
// at the start of every chunk, then walks the chunks backwards with dh in shared memory.  Everything that contracts
// over the state's columns (dqE, dkd, dw, dattn, <dh, h_in>) leaves it as one partial per column block; kernel 2
// (one CTA per chunk and head) adds the partials in a fixed order and does the rest.  No atomics.
#pragma once

#include "seqmix.cuh"

constexpr int kGdnBwdVB = 32;          // state columns per CTA of kernel 1
constexpr int kGdnBwdMaxDim = 128;     // head dimensions the register tiles are sized for (K, V <= 128)

// A thread's tile of a 64-row product: rows row0 + 4*tr + i (i < 4), columns tc + 16*j (j < NJ).
// acc[i][j] += sum over x in [x0, x1) of fa(i, x) * fb(j, x); sums run over x ascending.
template <int NJ, class FA, class FB>
__device__ __forceinline__ void gdn_tile_mm(float (&acc)[4][NJ], int x0, int x1, FA fa, FB fb) {
  for (int x = x0; x < x1; ++x) {
    float a[4], b[NJ];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = fa(i, x);
#pragma unroll
    for (int j = 0; j < NJ; ++j) b[j] = fb(j, x);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < NJ; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// The same tile when both operands are contiguous along the contraction: four steps per iteration through 16-byte
// loads (fa4 / fb4 return elements x .. x+3, x a multiple of 4), added in ascending x.
template <int NJ, class FA, class FB>
__device__ __forceinline__ void gdn_tile_mm_x4(float (&acc)[4][NJ], int x0, int x1, FA fa4, FB fb4) {
  for (int x = x0; x < x1; x += 4) {
    float4 a[4], b[NJ];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = fa4(i, x);
#pragma unroll
    for (int j = 0; j < NJ; ++j) b[j] = fb4(j, x);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
        acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
        acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
        acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
      }
  }
}

template <int NJ>
__device__ __forceinline__ void gdn_tile_zero(float (&acc)[4][NJ]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < NJ; ++j) acc[i][j] = 0.f;
}

// sum over the 16 lanes that share a tile row (lanes with the same tr are 16 consecutive lanes of a warp)
__device__ __forceinline__ float gdn_row16_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct GdnBwdWs {   // byte offsets into the backward workspace
  long long hs, du, pq, pk, pw, pat, pgl, total;
  int slices;
};

__host__ __device__ inline GdnBwdWs gdn_bwd_ws(const GdnDims& D) {
  GdnBwdWs w;
  const long long C = kGdnChunk;
  const long long chunks = (long long)D.B * D.N * D.H;
  w.slices = (D.V + kGdnBwdVB - 1) / kGdnBwdVB;
  long long run = 0;
  auto take = [&](long long bytes) {
    const long long at = run;
    run += (bytes + 255) / 256 * 256;
    return at;
  };
  w.hs = take(chunks * D.K * D.V * 4);                 // state at the start of every chunk [B,N,H,K,V]
  w.du = take(chunks * C * D.V * 4);                   // dv_new [B,N,H,C,V]
  w.pq = take(w.slices * chunks * C * D.K * 4);        // partials per column block: dqE, dkd, dw [slices][B,N,H,C,K]
  w.pk = take(w.slices * chunks * C * D.K * 4);
  w.pw = take(w.slices * chunks * C * D.K * 4);
  w.pat = take(w.slices * chunks * C * C * 4);         // dattn [slices][B,N,H,C,C]
  w.pgl = take(w.slices * chunks * 4);                 // exp(gcs_last) <dh, h_in> [slices][B,N,H]
  w.total = run;
  return w;
}

inline size_t gdn_bwd_scan_smem_bytes(int K) {
  const int C = kGdnChunk, KP = K + 1, VBP = kGdnBwdVB + 4;
  return (size_t)(2 * K * VBP + 3 * C * KP + 3 * C * VBP + C * (C + 1) + 3 * C + 32) * 4;
}

__global__ void __launch_bounds__(kGdnThreads) gdn_bwd_scan_kernel(const __nv_bfloat16* __restrict__ q,
                                                                   const __nv_bfloat16* __restrict__ k,
                                                                   const uint8_t* __restrict__ fws,
                                                                   const float* __restrict__ h0,
                                                                   const __nv_bfloat16* __restrict__ d_o,
                                                                   const float* __restrict__ dh_final,
                                                                   uint8_t* __restrict__ bws, float* __restrict__ dh0,
                                                                   GdnDims D) {
  extern __shared__ float gdn_smem[];
  // rows of the [*, VB] arrays are 36 floats apart: 16-byte aligned for the 4-wide loads of the products that contract
  // over the columns, and the 8 lanes of one 16-byte load phase (rows tc .. tc+7) fall on 8 different bank groups
  constexpr int C = kGdnChunk, VB = kGdnBwdVB, VBP = VB + 4;
  const int K = D.K, V = D.V, KP = K + 1;
  float* sH = gdn_smem;               // [K][VBP]   forward state, later dh
  float* sHin = sH + K * VBP;         // [K][VBP]   state at the start of the current chunk
  float* sQ = sHin + K * VBP;         // [C][KP]    q exp(gcs)
  float* sK = sQ + C * KP;            // [C][KP]    k exp(gcs_last - gcs)
  float* sW = sK + C * KP;            // [C][KP]    w
  float* sVn = sW + C * KP;           // [C][VBP]   u, then v_new
  float* sDo = sVn + C * VBP;         // [C][VBP]   do
  float* sDv = sDo + C * VBP;         // [C][VBP]   dv_new
  float* sAt = sDv + C * VBP;         // [C][C+1]   attn
  float* sG = sAt + C * (C + 1);      // [C]
  float* sEq = sG + C;                // [C] exp(gcs)
  float* sEk = sEq + C;               // [C] exp(gcs_last - gcs)
  float* sRed = sEk + C;              // [32] block reduction
  const int vb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tr = tid >> 4, tc = tid & 15;
  const int v0 = vb * VB;
  const float scale = gdn_round_bf16(rsqrtf((float)K));
  const GdnBwdWs W = gdn_bwd_ws(D);
  const long long chunks = (long long)D.B * D.N * D.H;
  float* hs = reinterpret_cast<float*>(bws + W.hs);
  float* du_out = reinterpret_cast<float*>(bws + W.du);
  float* pq = reinterpret_cast<float*>(bws + W.pq) + (long long)vb * chunks * C * K;
  float* pk = reinterpret_cast<float*>(bws + W.pk) + (long long)vb * chunks * C * K;
  float* pw = reinterpret_cast<float*>(bws + W.pw) + (long long)vb * chunks * C * K;
  float* pat = reinterpret_cast<float*>(bws + W.pat) + (long long)vb * chunks * C * C;
  float* pgl = reinterpret_cast<float*>(bws + W.pgl) + (long long)vb * chunks;

  // loads of one chunk: gcs and the decay factors, k (with its decay), w, u; optionally q (with its decay), attn, do
  auto load_chunk = [&](int n, bool backward) {
    const long long tok0 = (long long)n * C;
    const uint8_t* cw = fws + (((long long)b * D.N + n) * D.H + h) * gdn_chunk_ws_bytes(K, V);
    const __nv_bfloat16* u_in = reinterpret_cast<const __nv_bfloat16*>(cw);
    const __nv_bfloat16* w_in = u_in + C * V;
    const float* attn_in = reinterpret_cast<const float*>(w_in + C * K);
    const float* gcs_in = attn_in + C * C;
    __syncthreads();   // the previous chunk is done with every buffer
    if (tid < C) {
      const float gc = gcs_in[tid], gl = gcs_in[C - 1];
      sG[tid] = gc;
      sEq[tid] = __expf(gc);
      sEk[tid] = __expf(gl - gc);
    }
    __syncthreads();
    const int kv8 = K / 8;   // K is a multiple of 8: 16-byte pieces of the bf16 rows
    for (int i = tid; i < C * kv8; i += kGdnThreads) {
      const int r = i / kv8, c = (i - r * kv8) * 8;
      const long long t = tok0 + r;
      uint4 kraw = make_uint4(0, 0, 0, 0), qraw = make_uint4(0, 0, 0, 0);
      if (t < D.S) {
        const long long off = (((long long)b * D.S + t) * D.H + h) * K + c;
        kraw = *reinterpret_cast<const uint4*>(k + off);
        if (backward) qraw = *reinterpret_cast<const uint4*>(q + off);
      }
      const uint4 wraw = *reinterpret_cast<const uint4*>(w_in + r * K + c);
      float kf[8], qf[8], wf[8];
      lewi::Elem<__nv_bfloat16>::unpack(kraw, kf);
      lewi::Elem<__nv_bfloat16>::unpack(qraw, qf);
      lewi::Elem<__nv_bfloat16>::unpack(wraw, wf);
      const float eq = sEq[r], ek = sEk[r];
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        sQ[r * KP + c + x] = gdn_round_bf16(qf[x] * scale) * eq;
        sK[r * KP + c + x] = kf[x] * ek;
        sW[r * KP + c + x] = wf[x];
      }
    }
    for (int i = tid; i < C * VB; i += kGdnThreads) {
      const int r = i / VB, c = i - r * VB;
      const long long t = tok0 + r;
      const bool live = v0 + c < V;
      sVn[r * VBP + c] = live ? __bfloat162float(u_in[r * V + v0 + c]) : 0.f;
      if (backward)
        sDo[r * VBP + c] = (live && t < D.S) ? __bfloat162float(d_o[(((long long)b * D.S + t) * D.H + h) * V + v0 + c]) : 0.f;
    }
    if (backward) {
      for (int i = tid; i < C * C; i += kGdnThreads) {
        const int r = i / C, c = i - r * C;
        sAt[r * (C + 1) + c] = attn_in[i];
      }
    }
    __syncthreads();
  };
  // v_new = u - w state, in place over u (a thread owns the elements it reads and writes)
  auto make_vnew = [&](const float* state) {
    float acc[4][2];
    gdn_tile_zero(acc);
    gdn_tile_mm<2>(acc, 0, K, [&](int i, int x) { return sW[(tr * 4 + i) * KP + x]; },
                   [&](int j, int x) { return state[x * VBP + tc + 16 * j]; });
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) sVn[(tr * 4 + i) * VBP + tc + 16 * j] -= acc[i][j];
  };

  // ---- pass 1: the forward recurrence again, storing the state at the start of every chunk
  for (int i = tid; i < K * VB; i += kGdnThreads) {
    const int r = i / VB, c = i - r * VB;
    sH[r * VBP + c] = (h0 != nullptr && v0 + c < V) ? h0[(((long long)b * D.H + h) * K + r) * V + v0 + c] : 0.f;
  }
  for (int n = 0; n < D.N; ++n) {
    load_chunk(n, false);
    float* hs_n = hs + (((long long)b * D.N + n) * D.H + h) * K * V;
    for (int i = tid; i < K * VB; i += kGdnThreads) {
      const int r = i / VB, c = i - r * VB;
      if (v0 + c < V) hs_n[(long long)r * V + v0 + c] = sH[r * VBP + c];
    }
    make_vnew(sH);
    __syncthreads();
    const float dec = __expf(sG[C - 1]);
    for (int row0 = 0; row0 < K; row0 += 64) {
      float acc[4][2];
      gdn_tile_zero(acc);
      gdn_tile_mm<2>(acc, 0, C, [&](int i, int x) { const int kr = row0 + tr * 4 + i; return kr < K ? sK[x * KP + kr] : 0.f; },
                     [&](int j, int x) { return sVn[x * VBP + tc + 16 * j]; });
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kr = row0 + tr * 4 + i;
        if (kr >= K) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float* cell = &sH[kr * VBP + tc + 16 * j];
          *cell = *cell * dec + acc[i][j];   // every element of the state has one owner here
        }
      }
    }
  }

  // ---- pass 2: chunks in reverse, dh in sH
  __syncthreads();
  for (int i = tid; i < K * VB; i += kGdnThreads) {
    const int r = i / VB, c = i - r * VB;
    sH[r * VBP + c] = (dh_final != nullptr && v0 + c < V) ? dh_final[(((long long)b * D.H + h) * K + r) * V + v0 + c] : 0.f;
  }
  for (int n = D.N - 1; n >= 0; --n) {
    load_chunk(n, true);
    const long long chunk = ((long long)b * D.N + n) * D.H + h;
    const float* hs_n = hs + chunk * K * V;
    for (int i = tid; i < K * VB; i += kGdnThreads) {
      const int r = i / VB, c = i - r * VB;
      sHin[r * VBP + c] = v0 + c < V ? hs_n[(long long)r * V + v0 + c] : 0.f;
    }
    __syncthreads();
    make_vnew(sHin);
    __syncthreads();
    // dv_new = attn^T do + kd dh
    {
      float acc[4][2];
      gdn_tile_zero(acc);
      gdn_tile_mm<2>(acc, 0, C, [&](int i, int x) { return sAt[x * (C + 1) + tr * 4 + i]; },
                     [&](int j, int x) { return sDo[x * VBP + tc + 16 * j]; });
      gdn_tile_mm<2>(acc, 0, K, [&](int i, int x) { return sK[(tr * 4 + i) * KP + x]; },
                     [&](int j, int x) { return sH[x * VBP + tc + 16 * j]; });
      float* du_n = du_out + chunk * C * V;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int r = tr * 4 + i, c = tc + 16 * j;
          sDv[r * VBP + c] = acc[i][j];
          if (v0 + c < V) du_n[(long long)r * V + v0 + c] = acc[i][j];
        }
    }
    __syncthreads();
    // what contracts over this CTA's columns leaves as a partial: dqE = do h_in^T, dkd = v_new dh^T, dw = -dv_new h_in^T
    // (one product at a time: three sets of 32 accumulators at once did not fit the register file)
    for (int col0 = 0; col0 < K; col0 += 128) {
      for (int which = 0; which < 3; ++which) {
        const float* lhs = which == 0 ? sDo : (which == 1 ? sVn : sDv);
        const float* rhs = which == 1 ? sH : sHin;
        float* dst = which == 0 ? pq : (which == 1 ? pk : pw);
        const float sign = which == 2 ? -1.f : 1.f;
        float acc[4][8];
        gdn_tile_zero(acc);
        gdn_tile_mm_x4<8>(acc, 0, VB,
                          [&](int i, int x) { return *reinterpret_cast<const float4*>(&lhs[(tr * 4 + i) * VBP + x]); },
                          [&](int j, int x) {
                            const int kk = col0 + tc + 16 * j;
                            return kk < K ? *reinterpret_cast<const float4*>(&rhs[kk * VBP + x]) : make_float4(0.f, 0.f, 0.f, 0.f);
                          });
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int r = tr * 4 + i, kk = col0 + tc + 16 * j;
            if (kk < K) dst[(chunk * C + r) * K + kk] = sign * acc[i][j];
          }
      }
    }
    // dattn = lower(do v_new^T)
    {
      float acc[4][4];
      gdn_tile_zero(acc);
      gdn_tile_mm_x4<4>(acc, 0, VB,
                        [&](int i, int x) { return *reinterpret_cast<const float4*>(&sDo[(tr * 4 + i) * VBP + x]); },
                        [&](int j, int x) { return *reinterpret_cast<const float4*>(&sVn[(tc + 16 * j) * VBP + x]); });
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = tr * 4 + i, c = tc + 16 * j;
          pat[(chunk * C + r) * C + c] = c <= r ? acc[i][j] : 0.f;
        }
    }
    // exp(gcs_last) <dh, h_in> over this CTA's columns: fixed-order block sum
    {
      float part = 0.f;
      for (int i = tid; i < K * VB; i += kGdnThreads) {
        const int r = i / VB, c = i - r * VB;
        part = fmaf(sH[r * VBP + c], sHin[r * VBP + c], part);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if (lane == 0) sRed[warp] = part;
      __syncthreads();
      if (tid == 0) {
        float tot = 0.f;
        for (int w8 = 0; w8 < kGdnThreads / 32; ++w8) tot += sRed[w8];
        pgl[chunk] = tot * __expf(sG[C - 1]);
      }
    }
    // dh_in = qE^T do + dh exp(gcs_last) - w^T dv_new  (every thread has read the old dh above: barrier first)
    __syncthreads();
    const float dec = __expf(sG[C - 1]);
    for (int row0 = 0; row0 < K; row0 += 64) {
      float acc[4][2], sub[4][2];
      gdn_tile_zero(acc);
      gdn_tile_zero(sub);
      gdn_tile_mm<2>(acc, 0, C, [&](int i, int x) { const int kr = row0 + tr * 4 + i; return kr < K ? sQ[x * KP + kr] : 0.f; },
                     [&](int j, int x) { return sDo[x * VBP + tc + 16 * j]; });
      gdn_tile_mm<2>(sub, 0, C, [&](int i, int x) { const int kr = row0 + tr * 4 + i; return kr < K ? sW[x * KP + kr] : 0.f; },
                     [&](int j, int x) { return sDv[x * VBP + tc + 16 * j]; });
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kr = row0 + tr * 4 + i;
        if (kr >= K) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float* cell = &sH[kr * VBP + tc + 16 * j];
          *cell = *cell * dec + acc[i][j] - sub[i][j];
        }
      }
    }
  }
  __syncthreads();
  if (dh0 != nullptr) {
    for (int i = tid; i < K * VB; i += kGdnThreads) {
      const int r = i / VB, c = i - r * VB;
      if (v0 + c < V) dh0[(((long long)b * D.H + h) * K + r) * V + v0 + c] = sH[r * VBP + c];
    }
  }
}

inline size_t gdn_bwd_chunk_smem_bytes(int K, int V) {
  const int C = kGdnChunk, KP = K + 1, WP = (K > V ? K : V) + 1;
  return (size_t)(2 * C * KP + 2 * C * WP + 4 * C * (C + 1) + 8 * C) * 4;
}

__global__ void __launch_bounds__(kGdnThreads, 1) gdn_bwd_chunk_kernel(const __nv_bfloat16* __restrict__ q,
                                                                    const __nv_bfloat16* __restrict__ k,
                                                                    const __nv_bfloat16* __restrict__ v,
                                                                    const __nv_bfloat16* __restrict__ beta,
                                                                    const uint8_t* __restrict__ fws,
                                                                    const uint8_t* __restrict__ bws,
                                                                    __nv_bfloat16* __restrict__ dq,
                                                                    __nv_bfloat16* __restrict__ dk,
                                                                    __nv_bfloat16* __restrict__ dv, float* __restrict__ dg,
                                                                    __nv_bfloat16* __restrict__ dbeta, GdnDims D) {
  extern __shared__ float gdn_smem[];
  constexpr int C = kGdnChunk, CP = C + 1;
  const int K = D.K, V = D.V, KP = K + 1, VP = max(K, V) + 1;   // VP: row stride of the two areas that hold [C,V] and [C,K] data in turn
  float* sK = gdn_smem;               // [C][KP]  k
  float* sQ = sK + C * KP;            // [C][KP]  scaled q, later dw
  float* sV = sQ + C * KP;            // [C][VP]  vb, later kb
  float* sU = sV + C * VP;            // [C][VP]  dv_new
  float* sA = sU + C * VP;            // [C][CP]  A
  float* sS = sA + C * CP;            // [C][CP]  S
  float* sT = sS + C * CP;            // [C][CP]  dattn D, later dA, later dS / dP
  float* sX = sT + C * CP;            // [C][CP]  scratch: G, A^T dA, dS S
  float* sG = sX + C * CP;            // [C] gcs
  float* sB = sG + C;                 // [C] beta
  float* sE = sB + C;                 // [C] exp(gcs)
  float* sEk = sE + C;                // [C] exp(gcs_last - gcs)
  // every accumulator below has ONE writing thread per element, so the sums do not depend on timing:
  float* sDgA = sEk + C;              // [C] dgcs, the terms thread r adds (row and column sums of [C,C] matrices)
  float* sDgB = sDgA + C;             // [C] dgcs, the terms the first lane of a tile row adds (row sums of [C,K] tiles)
  float* sDb = sDgB + C;              // [C] dbeta (first lane of a tile row)
  float* sTmp = sDb + C;              // [C] rowsum(dkd kd)
  const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int tr = tid >> 4, tc = tid & 15;
  const long long tok0 = (long long)n * C;
  const float scale = gdn_round_bf16(rsqrtf((float)K));
  const GdnBwdWs W = gdn_bwd_ws(D);
  const long long chunks = (long long)D.B * D.N * D.H;
  const long long chunk = ((long long)b * D.N + n) * D.H + h;
  const uint8_t* cw = fws + chunk * gdn_chunk_ws_bytes(K, V);
  const float* attn_in = reinterpret_cast<const float*>(cw + (long long)C * V * 2 + (long long)C * K * 2);
  const float* gcs_in = attn_in + C * C;
  const float* du_in = reinterpret_cast<const float*>(bws + W.du) + chunk * C * V;
  const float* pq = reinterpret_cast<const float*>(bws + W.pq) + chunk * C * K;
  const float* pk = reinterpret_cast<const float*>(bws + W.pk) + chunk * C * K;
  const float* pw = reinterpret_cast<const float*>(bws + W.pw) + chunk * C * K;
  const float* pat = reinterpret_cast<const float*>(bws + W.pat) + chunk * C * C;
  const float* pgl = reinterpret_cast<const float*>(bws + W.pgl) + chunk;
  const long long pstride_k = chunks * C * K, pstride_c = chunks * C * C;
  auto tok_off = [&](int r) { return ((long long)b * D.S + tok0 + r) * D.H + h; };
  auto live = [&](int r) { return tok0 + r < D.S; };
  // fixed-order sum of the column blocks' partials
  auto psum = [&](const float* p, long long stride, long long at) {
    float s = p[at];
    for (int sl = 1; sl < W.slices; ++sl) s += p[at + sl * stride];
    return s;
  };

  // the same sum for four adjacent elements (16-byte loads; every partial array starts on a 256-byte boundary and the
  // extents are multiples of 8)
  auto psum4 = [&](const float* p, long long stride, long long at) {
    float4 s4 = *reinterpret_cast<const float4*>(p + at);
    for (int sl = 1; sl < W.slices; ++sl) {
      const float4 t4 = *reinterpret_cast<const float4*>(p + at + sl * stride);
      s4.x += t4.x; s4.y += t4.y; s4.z += t4.z; s4.w += t4.w;
    }
    return s4;
  };

  // ---- loads (16-byte pieces: the loops below are short enough for their loads to be in flight together)
  {
    const int kv8 = K / 8;
#pragma unroll 4
    for (int i = tid; i < C * kv8; i += kGdnThreads) {
      const int r = i / kv8, c = (i - r * kv8) * 8;
      uint4 kraw = make_uint4(0, 0, 0, 0), qraw = make_uint4(0, 0, 0, 0);
      if (live(r)) {
        kraw = *reinterpret_cast<const uint4*>(k + tok_off(r) * K + c);
        qraw = *reinterpret_cast<const uint4*>(q + tok_off(r) * K + c);
      }
      float kf[8], qf[8];
      lewi::Elem<__nv_bfloat16>::unpack(kraw, kf);
      lewi::Elem<__nv_bfloat16>::unpack(qraw, qf);
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        sK[r * KP + c + x] = kf[x];
        sQ[r * KP + c + x] = gdn_round_bf16(qf[x] * scale);
      }
    }
  }
  if (tid < C) {
    const float gc = gcs_in[tid];
    sG[tid] = gc;
    sB[tid] = live(tid) ? __bfloat162float(beta[tok_off(tid)]) : 0.f;
    sE[tid] = __expf(gc);
    sEk[tid] = __expf(gcs_in[C - 1] - gc);
    sDgA[tid] = 0.f;
    sDgB[tid] = 0.f;
    sDb[tid] = 0.f;
  }
  __syncthreads();
  auto kb_at = [&](int r, int x) { return gdn_round_bf16(sK[r * KP + x] * sB[r]); };

  // ---- S = strict(bf16(kb k^T) D) and A = (I + S)^-1, as in the forward pass
  {
    float acc[4][4];
    gdn_tile_zero(acc);
    if (tc <= tr * 4 + 3)
      gdn_tile_mm<4>(acc, 0, K, [&](int i, int x) { return kb_at(tr * 4 + i, x); },
                     [&](int j, int x) { return sK[(tc + 16 * j) * KP + x]; });
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = tr * 4 + i, c = tc + 16 * j;
        sS[r * CP + c] = c < r ? gdn_round_bf16(acc[i][j]) * __expf(sG[r] - sG[c]) : 0.f;
      }
  }
  __syncthreads();
  if (tid < C) {
    const int c = tid;
    float colv[C];
#pragma unroll
    for (int i = 0; i < C; ++i) {
      float acc = i == c ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) acc = fmaf(-sS[i * CP + j], colv[j], acc);
      colv[i] = i < c ? 0.f : acc;
      sA[i * CP + c] = colv[i];
    }
  }
  // ---- dattn (sum of the partials), G = dattn attn, then dattn D in place
#pragma unroll 2
  for (int i4 = tid; i4 < C * C / 4; i4 += kGdnThreads) {
    const int r = i4 / (C / 4), c0 = (i4 - r * (C / 4)) * 4;
    const float4 da4 = psum4(pat, pstride_c, (long long)i4 * 4);
    const float4 at4 = *reinterpret_cast<const float4*>(attn_in + i4 * 4);
    const float da[4] = {da4.x, da4.y, da4.z, da4.w}, at[4] = {at4.x, at4.y, at4.z, at4.w};
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int c = c0 + x;
      const float d = c <= r ? da[x] : 0.f;
      sX[r * CP + c] = d * at[x];
      sT[r * CP + c] = c <= r ? d * __expf(sG[r] - sG[c]) : 0.f;
    }
  }
  // dqE and dkd (sums of the partials) wait in the two areas that vb and dv_new take over later
  {
    const int k4 = K / 4;
#pragma unroll 2
    for (int i4 = tid; i4 < C * k4; i4 += kGdnThreads) {
      const int r = i4 / k4, c0 = (i4 - r * k4) * 4;
      const float4 a4 = psum4(pq, pstride_k, (long long)i4 * 4), b4 = psum4(pk, pstride_k, (long long)i4 * 4);
      sV[r * VP + c0] = a4.x; sV[r * VP + c0 + 1] = a4.y; sV[r * VP + c0 + 2] = a4.z; sV[r * VP + c0 + 3] = a4.w;
      sU[r * VP + c0] = b4.x; sU[r * VP + c0 + 1] = b4.y; sU[r * VP + c0 + 2] = b4.z; sU[r * VP + c0 + 3] = b4.w;
    }
  }
  __syncthreads();
  if (tid < C) {   // rowsum(G) - colsum(G)
    float rs = 0.f, cs = 0.f;
    for (int j = 0; j < C; ++j) {
      rs += sX[tid * CP + j];
      cs += sX[j * CP + tid];
    }
    sDgA[tid] += rs - cs;
  }
  // ---- [C,K] tiles kept in registers to the end: dk and dkb
  float dk_acc[4][8], dkb_acc[4][8];
  gdn_tile_zero(dk_acc);
  gdn_tile_zero(dkb_acc);
  {
    // dq = (dqE E + (dattn D) k) scale;  dgcs += rowsum(dqE qE)
    float acc[4][8];
    gdn_tile_zero(acc);
    gdn_tile_mm<8>(acc, 0, C, [&](int i, int x) { return sT[(tr * 4 + i) * CP + x]; },
                   [&](int j, int x) { const int c = tc + 16 * j; return c < K ? sK[x * KP + c] : 0.f; });
    // dk = dkd exp(gcs_last - gcs) + (dattn D)^T q;  dgcs -= rowsum(dkd kd)
    gdn_tile_mm<8>(dk_acc, 0, C, [&](int i, int x) { return sT[x * CP + tr * 4 + i]; },
                   [&](int j, int x) { const int c = tc + 16 * j; return c < K ? sQ[x * KP + c] : 0.f; });
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = tr * 4 + i;
      float rq = 0.f, rk = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = tc + 16 * j;
        if (c >= K) continue;
        const float dqe = sV[r * VP + c], dkd = sU[r * VP + c];
        acc[i][j] = fmaf(dqe, sE[r], acc[i][j]);
        rq = fmaf(dqe, sQ[r * KP + c] * sE[r], rq);
        dk_acc[i][j] = fmaf(dkd, sEk[r], dk_acc[i][j]);
        rk = fmaf(dkd, sK[r * KP + c] * sEk[r], rk);
        if (live(r)) dq[tok_off(r) * K + c] = __float2bfloat16_rn(acc[i][j] * scale);
      }
      rq = gdn_row16_sum(rq);
      rk = gdn_row16_sum(rk);
      if (tc == 0) {
        sDgB[r] += rq - rk;
        sTmp[r] = rk;
      }
    }
  }
  __syncthreads();
  if (tid == C - 1) {   // dgcs_last += exp(gcs_last) <dh, h_in> + sum(dkd kd)
    float tot = psum(pgl, chunks, 0);
    for (int r = 0; r < C; ++r) tot += sTmp[r];
    sDgA[C - 1] += tot;
  }
  // ---- dw (partials) over q's place, vb and dv_new
  {
    const int k4 = K / 4, v8 = V / 8;
#pragma unroll 2
    for (int i4 = tid; i4 < C * k4; i4 += kGdnThreads) {
      const int r = i4 / k4, c0 = (i4 - r * k4) * 4;
      const float4 w4 = psum4(pw, pstride_k, (long long)i4 * 4);
      sQ[r * KP + c0] = w4.x; sQ[r * KP + c0 + 1] = w4.y; sQ[r * KP + c0 + 2] = w4.z; sQ[r * KP + c0 + 3] = w4.w;
    }
#pragma unroll 2
    for (int i8 = tid; i8 < C * v8; i8 += kGdnThreads) {
      const int r = i8 / v8, c0 = (i8 - r * v8) * 8;
      const uint4 vraw = live(r) ? *reinterpret_cast<const uint4*>(v + tok_off(r) * V + c0) : make_uint4(0, 0, 0, 0);
      const float4 u0 = *reinterpret_cast<const float4*>(du_in + (long long)r * V + c0);
      const float4 u1 = *reinterpret_cast<const float4*>(du_in + (long long)r * V + c0 + 4);
      float vf[8];
      lewi::Elem<__nv_bfloat16>::unpack(vraw, vf);
      const float uu[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        sV[r * VP + c0 + x] = gdn_round_bf16(vf[x] * sB[r]);
        sU[r * VP + c0 + x] = uu[x];
      }
    }
  }
  __syncthreads();
  // ---- dA = dv_new vb^T + dw kg^T  (over dattn D, which is no longer needed)
  {
    float acc[4][4];
    gdn_tile_zero(acc);
    gdn_tile_mm<4>(acc, 0, V, [&](int i, int x) { return sU[(tr * 4 + i) * VP + x]; },
                   [&](int j, int x) { return sV[(tc + 16 * j) * VP + x]; });
    gdn_tile_mm<4>(acc, 0, K, [&](int i, int x) { return sQ[(tr * 4 + i) * KP + x]; },
                   [&](int j, int x) { const int c = tc + 16 * j; return kb_at(c, x) * sE[c]; });
    __syncthreads();   // every thread is done reading dattn D
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) sT[(tr * 4 + i) * CP + tc + 16 * j] = acc[i][j];
  }
  // ---- dvb = A^T dv_new: dv = dvb beta, dbeta += rowsum(dvb v)
  for (int col0 = 0; col0 < V; col0 += 128) {
    float acc[4][8];
    gdn_tile_zero(acc);
    gdn_tile_mm<8>(acc, 0, C, [&](int i, int x) { return sA[x * CP + tr * 4 + i]; },
                   [&](int j, int x) { const int c = col0 + tc + 16 * j; return c < V ? sU[x * VP + c] : 0.f; });
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = tr * 4 + i;
      float rb = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = col0 + tc + 16 * j;
        if (c >= V || !live(r)) continue;
        const float vv = __bfloat162float(v[tok_off(r) * V + c]);
        rb = fmaf(acc[i][j], vv, rb);
        dv[tok_off(r) * V + c] = __float2bfloat16_rn(acc[i][j] * sB[r]);
      }
      rb = gdn_row16_sum(rb);
      if (tc == 0) sDb[r] += rb;
    }
  }
  // ---- dkg = A^T dw: dkb = dkg E, dgcs += rowsum(dkg kg)
  {
    float acc[4][8];
    gdn_tile_zero(acc);
    gdn_tile_mm<8>(acc, 0, C, [&](int i, int x) { return sA[x * CP + tr * 4 + i]; },
                   [&](int j, int x) { const int c = tc + 16 * j; return c < K ? sQ[x * KP + c] : 0.f; });
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = tr * 4 + i;
      float rg = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = tc + 16 * j;
        if (c >= K) continue;
        dkb_acc[i][j] = acc[i][j] * sE[r];
        rg = fmaf(acc[i][j], kb_at(r, c) * sE[r], rg);
      }
      rg = gdn_row16_sum(rg);
      if (tc == 0) sDgB[r] += rg;
    }
  }
  __syncthreads();
  // ---- dS = -strict(A^T dA A^T): first A^T dA, then times A^T
  {
    float acc[4][4];
    gdn_tile_zero(acc);
    gdn_tile_mm<4>(acc, 0, C, [&](int i, int x) { return sA[x * CP + tr * 4 + i]; },
                   [&](int j, int x) { return sT[x * CP + tc + 16 * j]; });
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) sX[(tr * 4 + i) * CP + tc + 16 * j] = acc[i][j];
  }
  __syncthreads();
  {
    float acc[4][4];
    gdn_tile_zero(acc);
    gdn_tile_mm<4>(acc, 0, C, [&](int i, int x) { return sX[(tr * 4 + i) * CP + x]; },
                   [&](int j, int x) { return sA[(tc + 16 * j) * CP + x]; });
    // (dA is no longer needed: every thread finished reading it before the barrier above)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = tr * 4 + i, c = tc + 16 * j;
        sT[r * CP + c] = c < r ? -acc[i][j] : 0.f;   // dS
      }
  }
  __syncthreads();
  // G = dS S -> dgcs; dP = dS D in place; kb over vb's place
  for (int i = tid; i < C * C; i += kGdnThreads) {
    const int r = i / C, c = i - r * C;
    const float ds = sT[r * CP + c];
    sX[r * CP + c] = ds * sS[r * CP + c];
    sT[r * CP + c] = c < r ? ds * __expf(sG[r] - sG[c]) : 0.f;
  }
  for (int i = tid; i < C * K; i += kGdnThreads) {
    const int r = i / K, c = i - r * K;
    sV[r * VP + c] = kb_at(r, c);
  }
  __syncthreads();
  if (tid < C) {
    float rs = 0.f, cs = 0.f;
    for (int j = 0; j < C; ++j) {
      rs += sX[tid * CP + j];
      cs += sX[j * CP + tid];
    }
    sDgA[tid] += rs - cs;
  }
  // ---- dkb += dP k;  dk += dP^T kb + dkb beta;  dbeta += rowsum(dkb k)
  gdn_tile_mm<8>(dkb_acc, 0, C, [&](int i, int x) { return sT[(tr * 4 + i) * CP + x]; },
                 [&](int j, int x) { const int c = tc + 16 * j; return c < K ? sK[x * KP + c] : 0.f; });
  gdn_tile_mm<8>(dk_acc, 0, C, [&](int i, int x) { return sT[x * CP + tr * 4 + i]; },
                 [&](int j, int x) { const int c = tc + 16 * j; return c < K ? sV[x * VP + c] : 0.f; });
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = tr * 4 + i;
    float rb = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = tc + 16 * j;
      if (c >= K) continue;
      rb = fmaf(dkb_acc[i][j], sK[r * KP + c], rb);
      if (live(r)) dk[tok_off(r) * K + c] = __float2bfloat16_rn(dk_acc[i][j] + dkb_acc[i][j] * sB[r]);
    }
    rb = gdn_row16_sum(rb);
    if (tc == 0) sDb[r] += rb;
  }
  __syncthreads();
  // ---- dg = reverse cumulative sum of dgcs; dbeta
  if (tid == 0) {
    float run = 0.f;
    for (int r = C - 1; r >= 0; --r) {
      run += sDgA[r] + sDgB[r];
      if (live(r)) dg[tok_off(r)] = run;
    }
  }
  if (tid < C && live(tid)) dbeta[tok_off(tid)] = __float2bfloat16_rn(sDb[tid]);
}
