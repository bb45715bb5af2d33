// Sequence-mixing helpers of the Gated-DeltaNet block that sits beside the MoE layer in the reference's decoder.
// Causal depthwise 1-D convolution (the reference replaces flax's `nnx.Conv(padding="CAUSAL", groups=C)` by K
// shifted multiply-adds, modal/fast_conv.py:14-31):
//   y[b,t,c] = sum_{j<K} w[j,c] * x[b, t-(K-1)+j, c]          (x before the start of the sequence is zero)
// and its gradients
//   dx[b,t,c] = sum_{j<K} w[j,c] * g[b, t+(K-1)-j, c]          (g past the end of the sequence is zero)
//   dw[j,c]   = sum_{b,t} g[b,t,c] * x[b, t-(K-1)+j, c].
// Pure HBM streaming: a thread owns 8 channels (16 bytes) of a run of consecutive time steps and slides a window of
// K vectors through registers, so x is read once (plus K-1 halo steps per run) and y written once.  Products and
// sums are float32, rounded to bf16 once at the end.
#pragma once

#include "common.cuh"
#include "gather.cuh"

namespace lewi {

constexpr int kConvMaxTaps = 8;
constexpr int kConvRun = 32;      // time steps per thread
constexpr int kConvThreads = 128;

// KT = number of taps, a compile-time constant so that the sliding window lives in registers.
template <int KT>
struct ConvTaps {
  float w[KT][8];
};

template <int KT>
__device__ __forceinline__ void conv_load_taps(ConvTaps<KT>& taps, const __nv_bfloat16* __restrict__ w, int C, int c0) {
  constexpr int K = KT;
#pragma unroll
  for (int j = 0; j < KT; ++j) {
    if (j < K) {
      float f[8];
      Elem<__nv_bfloat16>::unpack(ld_nc_v4(w + (long long)j * C + c0), f);
#pragma unroll
      for (int q = 0; q < 8; ++q) taps.w[j][q] = f[q];
    }
  }
}

// REVERSE = false: forward (window looks back in time); true: the input gradient (window looks ahead, taps flipped).
template <bool REVERSE, int KT>
__global__ void __launch_bounds__(kConvThreads) causal_conv1d_kernel(const __nv_bfloat16* __restrict__ x,
                                                                     const __nv_bfloat16* __restrict__ w,
                                                                     __nv_bfloat16* __restrict__ y, int B, int T, int C) {
  constexpr int K = KT;
  const int cvec = C / 8;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;      // channel vector
  if (v >= cvec) return;
  const int c0 = v * 8;
  const int run = blockIdx.y, b = blockIdx.z;
  const int t0 = run * kConvRun;
  ConvTaps<KT> taps;
  conv_load_taps<KT>(taps, w, C, c0);
  const __nv_bfloat16* xb = x + (long long)b * T * C + c0;
  __nv_bfloat16* yb = y + (long long)b * T * C + c0;
  float win[KT][8];   // win[i] = input at offset i of the current window
  auto fetch = [&](int t, float* dst) {
    if (t >= 0 && t < T) {
      Elem<__nv_bfloat16>::unpack(ld_nc_v4(xb + (long long)t * C), dst);
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) dst[q] = 0.f;
    }
  };
  // forward: output t reads inputs t-(K-1) .. t, tap j at window slot j
  // reverse: output t reads inputs t .. t+(K-1), input t+i meets tap K-1-i
#pragma unroll
  for (int i = 0; i < KT; ++i)
    if (i < K - 1) fetch(REVERSE ? t0 + i : t0 - (K - 1) + i, win[i]);
  const int t_end = min(t0 + kConvRun, T);
  for (int t = t0; t < t_end; ++t) {
    fetch(REVERSE ? t + (K - 1) : t, win[K - 1]);
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.f;
#pragma unroll
    for (int i = 0; i < KT; ++i) {
      if (i < K) {
        const int j = REVERSE ? K - 1 - i : i;
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = fmaf(taps.w[j][q], win[i][q], acc[q]);
      }
    }
    st_v4(yb + (long long)t * C, Elem<__nv_bfloat16>::pack(acc));
#pragma unroll
    for (int i = 0; i < KT - 1; ++i)
      if (i < K - 1) {
#pragma unroll
        for (int q = 0; q < 8; ++q) win[i][q] = win[i + 1][q];
      }
  }
}

// partial[(b * runs + run), j, c] = sum over the run's time steps of g[b,t,c] * x[b, t-(K-1)+j, c]
template <int KT>
__global__ void __launch_bounds__(kConvThreads) causal_conv1d_dw_kernel(const __nv_bfloat16* __restrict__ x,
                                                                        const __nv_bfloat16* __restrict__ g,
                                                                        float* __restrict__ partial, int B, int T, int C) {
  constexpr int K = KT;
  const int cvec = C / 8;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= cvec) return;
  const int c0 = v * 8;
  const int run = blockIdx.y, b = blockIdx.z;
  const int t0 = run * kConvRun;
  const __nv_bfloat16* xb = x + (long long)b * T * C + c0;
  const __nv_bfloat16* gb = g + (long long)b * T * C + c0;
  float win[KT][8], acc[KT][8];
#pragma unroll
  for (int j = 0; j < KT; ++j)
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[j][q] = 0.f;
  auto fetch = [&](int t, float* dst) {
    if (t >= 0 && t < T) {
      Elem<__nv_bfloat16>::unpack(ld_nc_v4(xb + (long long)t * C), dst);
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) dst[q] = 0.f;
    }
  };
#pragma unroll
  for (int i = 0; i < KT; ++i)
    if (i < K - 1) fetch(t0 - (K - 1) + i, win[i]);
  const int t_end = min(t0 + kConvRun, T);
  for (int t = t0; t < t_end; ++t) {
    fetch(t, win[K - 1]);
    float gv[8];
    Elem<__nv_bfloat16>::unpack(ld_nc_v4(gb + (long long)t * C), gv);
#pragma unroll
    for (int j = 0; j < KT; ++j)
      if (j < K) {
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[j][q] = fmaf(gv[q], win[j][q], acc[j][q]);
      }
#pragma unroll
    for (int i = 0; i < KT - 1; ++i)
      if (i < K - 1) {
#pragma unroll
        for (int q = 0; q < 8; ++q) win[i][q] = win[i + 1][q];
      }
  }
  const long long part = (long long)b * gridDim.y + run;
#pragma unroll
  for (int j = 0; j < KT; ++j)
    if (j < K) {
      float* dst = partial + (part * K + j) * C + c0;
      *reinterpret_cast<float4*>(dst) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
    }
}

// out[i] (bf16) = sum over parts of partial[part, i]; the parts of a column are added in index order.
__global__ void __launch_bounds__(256) conv_dw_reduce_kernel(const float* __restrict__ partial, int n_parts, int n,
                                                             __nv_bfloat16* __restrict__ out_bf16, float* __restrict__ out_f32) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = 0.f;
  for (int p = 0; p < n_parts; ++p) acc += partial[(long long)p * n + i];
  if (out_f32 != nullptr) out_f32[i] = acc;
  if (out_bf16 != nullptr) out_bf16[i] = __float2bfloat16_rn(acc);
}

}  // namespace lewi

// =====================================================================================================
// Chunked gated delta rule, forward (the reference's `fast_chunk_gated_delta_rule`, modal/gdn_fast.py:37-113).
//
// Per (batch, head) the state h [K,V] follows  h <- h*exp(g_t) + k_t (x) beta_t (v_t - k_t^T h),  o_t = q_t^T h.
// Tokens are processed in chunks of 64 (WY form): with gcs = cumsum(g) inside the chunk,
//   S    = strict_lower( bf16(k_beta k^T) * exp(gcs_i - gcs_j) ),   A = (I + S)^-1,
//   u    = bf16(A v_beta),   w = bf16(A (k_beta * exp(gcs))),
//   attn = lower( bf16(q k^T) * exp(gcs_i - gcs_j) )
// depend on one chunk only (kernel 1, one CTA per chunk and head), and the recurrence over chunks
//   v_new = u - w h;   o = (q exp(gcs)) h + attn v_new;   h <- h exp(gcs_last) + (k exp(gcs_last - gcs))^T v_new
// is independent per column of h, so kernel 2 runs one CTA per (batch, head, 32 columns of V) over the chunks in
// order with its slice of h in shared memory.  The roundings to bf16 are the ones JAX applies in the reference for
// compute_dtype = bfloat16; everything that involves g or the state is float32, like the reference at its default
// precision.  All products run on the CUDA cores in float32.
// =====================================================================================================

constexpr int kGdnChunk = 64;
constexpr int kGdnThreads = 256;
constexpr int kGdnMaxDim = 128;

__device__ __forceinline__ float gdn_round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct GdnDims {
  int B, S, H, K, V, N;   // N = chunks per sequence
};

// workspace of one (b, n, h) chunk: u bf16 [64,V] | w bf16 [64,K] | attn f32 [64,64] | gcs f32 [64]
inline size_t gdn_prep_smem_bytes(int K, int V) {
  const int C = kGdnChunk, KP = K + 1, VP = V + 1;
  const int QP = KP > VP ? (KP > C + 1 ? KP : C + 1) : (VP > C + 1 ? VP : C + 1);
  return (size_t)(C * KP + C * QP + C * (C + 1) + 3 * C) * 4;
}
inline size_t gdn_scan_smem_bytes(int K, int vb) {
  const int C = kGdnChunk, KP = K + 1;
  return (size_t)(K * vb + 3 * C * KP + C * vb + C * (C + 1) + 3 * C) * 4;
}

__host__ __device__ inline long long gdn_chunk_ws_bytes(int K, int V) {
  return (long long)kGdnChunk * V * 2 + (long long)kGdnChunk * K * 2 + (long long)kGdnChunk * kGdnChunk * 4 + kGdnChunk * 4;
}

__global__ void __launch_bounds__(kGdnThreads) gdn_chunk_prep_kernel(const __nv_bfloat16* __restrict__ q,
                                                                     const __nv_bfloat16* __restrict__ k,
                                                                     const __nv_bfloat16* __restrict__ v,
                                                                     const float* __restrict__ g,
                                                                     const __nv_bfloat16* __restrict__ beta,
                                                                     uint8_t* __restrict__ ws, GdnDims D) {
  extern __shared__ float gdn_smem[];
  constexpr int C = kGdnChunk;
  const int K = D.K, V = D.V, KP = K + 1, VP = V + 1;
  // k * beta (rounded to bf16) is recomputed from k wherever it is needed instead of being kept: with one array less
  // two CTAs fit on an SM, and the phases in which few threads work (prefix sum, substitution) overlap another CTA.
  float* sK = gdn_smem;                 // [C][KP]   k
  float* sQ = sK + C * KP;              // [C][QP]   scaled q, later A while it is built, later v * beta
  const int QP = max(max(KP, VP), C + 1);   // the area also holds A [C][C+1] during the substitution
  float* sS = sQ + C * QP;              // [C][C+1]  S, then A
  float* sG = sS + C * (C + 1);         // [C] gcs
  float* sB = sG + C;                   // [C] beta
  float* sE = sB + C;                   // [C] exp(gcs)
  const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const long long tok0 = (long long)n * C;
  const float scale = gdn_round_bf16(rsqrtf((float)K));
  // loads (tokens past the end of the sequence are zero rows with g = 0, beta = 0)
  if ((K & 7) == 0) {   // 16-byte pieces of the bf16 rows
    const int kv8 = K / 8;
    for (int i = tid; i < C * kv8; i += kGdnThreads) {
      const int r = i / kv8, c = (i - r * kv8) * 8;
      const long long t = tok0 + r;
      uint4 kq[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
      if (t < D.S) {
        const long long off = (((long long)b * D.S + t) * D.H + h) * K + c;
        kq[0] = *reinterpret_cast<const uint4*>(k + off);
        kq[1] = *reinterpret_cast<const uint4*>(q + off);
      }
      float kf[8], qf[8];
      lewi::Elem<__nv_bfloat16>::unpack(kq[0], kf);
      lewi::Elem<__nv_bfloat16>::unpack(kq[1], qf);
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        sK[r * KP + c + x] = kf[x];
        sQ[r * QP + c + x] = gdn_round_bf16(qf[x] * scale);
      }
    }
  } else {
    for (int i = tid; i < C * K; i += kGdnThreads) {
      const int r = i / K, c = i - r * K;
      const long long t = tok0 + r;
      float kv = 0.f, qv = 0.f;
      if (t < D.S) {
        const long long off = (((long long)b * D.S + t) * D.H + h) * K + c;
        kv = __bfloat162float(k[off]);
        qv = gdn_round_bf16(__bfloat162float(q[off]) * scale);
      }
      sK[r * KP + c] = kv;
      sQ[r * QP + c] = qv;
    }
  }
  if (tid < C) {
    const long long t = tok0 + tid;
    sG[tid] = t < D.S ? g[((long long)b * D.S + t) * D.H + h] : 0.f;
    sB[tid] = t < D.S ? __bfloat162float(beta[((long long)b * D.S + t) * D.H + h]) : 0.f;
  }
  __syncthreads();
  if (tid == 0) {   // inclusive prefix sum of g in index order (64 adds)
    float run = 0.f;
    for (int i = 0; i < C; ++i) {
      run += sG[i];
      sG[i] = run;
    }
  }
  __syncthreads();
  if (tid < C) sE[tid] = __expf(sG[tid]);
  uint8_t* my_ws = ws + (((long long)b * D.N + n) * D.H + h) * gdn_chunk_ws_bytes(K, V);
  __nv_bfloat16* u_out = reinterpret_cast<__nv_bfloat16*>(my_ws);
  __nv_bfloat16* w_out = u_out + C * V;
  float* attn_out = reinterpret_cast<float*>(w_out + C * K);
  float* gcs_out = attn_out + C * C;
  // S (strictly lower) and the in-chunk attention (lower, diagonal included).  Register tiles: a thread owns rows
  // 4*tr .. 4*tr+3 and columns tc, tc+16, tc+32, tc+48 (neighbouring lanes read neighbouring rows of k: no bank
  // conflicts with the odd row stride), 32 fused multiply-adds per 12 shared-memory loads; sums run over x ascending.
  {
    const int tr = tid >> 4, tc = tid & 15;
    float s_acc[4][4], a_acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        s_acc[i][j] = 0.f;
        a_acc[i][j] = 0.f;
      }
    if (tc <= tr * 4 + 3) {   // otherwise every element of the tile lies above the diagonal
      const float b4[4] = {sB[tr * 4], sB[tr * 4 + 1], sB[tr * 4 + 2], sB[tr * 4 + 3]};
      for (int x = 0; x < K; ++x) {
        float kb[4], qq[4], kc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          kb[i] = gdn_round_bf16(sK[(tr * 4 + i) * KP + x] * b4[i]);
          qq[i] = sQ[(tr * 4 + i) * QP + x];
          kc[i] = sK[(tc + 16 * i) * KP + x];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            s_acc[i][j] = fmaf(kb[i], kc[j], s_acc[i][j]);
            a_acc[i][j] = fmaf(qq[i], kc[j], a_acc[i][j]);
          }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = tr * 4 + i, c = tc + 16 * j;
        float sv = 0.f, av = 0.f;
        if (c <= r) {
          const float dec = __expf(sG[r] - sG[c]);
          sv = c < r ? gdn_round_bf16(s_acc[i][j]) * dec : 0.f;
          av = gdn_round_bf16(a_acc[i][j]) * dec;
        }
        sS[r * (C + 1) + c] = sv;
        attn_out[r * C + c] = av;
      }
  }
  if (tid < C) gcs_out[tid] = sG[tid];
  __syncthreads();
  // A = (I + S)^-1 by forward substitution; thread c owns column c of A and needs nobody else's column
  // (A[i,c] = delta_ic - sum_{j<i} S[i,j] A[j,c]); the column lives in the sQ area, which is free again
  float* sA = sQ;   // [C][C+1]
  __syncthreads();
  if (tid < C) {
    // the column stays in registers (both loops unrolled); terms with j < c multiply an exact zero, so the sum equals
    // the one that starts at j = c
    const int c = tid;
    float colv[C];
#pragma unroll
    for (int i = 0; i < C; ++i) {
      float acc = i == c ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) acc = fmaf(-sS[i * (C + 1) + j], colv[j], acc);
      colv[i] = i < c ? 0.f : acc;
      sA[i * (C + 1) + c] = colv[i];
    }
  }
  __syncthreads();
  // move A into sS, free the sQ area for v_beta
  for (int i = tid; i < C * C; i += kGdnThreads) {
    const int r = i / C, c = i - r * C;
    sS[r * (C + 1) + c] = sA[r * (C + 1) + c];
  }
  __syncthreads();
  if ((V & 7) == 0) {
    const int vv8 = V / 8;
    for (int i = tid; i < C * vv8; i += kGdnThreads) {
      const int r = i / vv8, c = (i - r * vv8) * 8;
      const long long t = tok0 + r;
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (t < D.S) raw = *reinterpret_cast<const uint4*>(v + (((long long)b * D.S + t) * D.H + h) * V + c);
      float vf[8];
      lewi::Elem<__nv_bfloat16>::unpack(raw, vf);
      const float br = sB[r];
#pragma unroll
      for (int x = 0; x < 8; ++x) sQ[r * QP + c + x] = gdn_round_bf16(vf[x] * br);
    }
  } else {
    for (int i = tid; i < C * V; i += kGdnThreads) {
      const int r = i / V, c = i - r * V;
      const long long t = tok0 + r;
      float vv = 0.f;
      if (t < D.S) vv = __bfloat162float(v[(((long long)b * D.S + t) * D.H + h) * V + c]);
      sQ[r * QP + c] = gdn_round_bf16(vv * sB[r]);
    }
  }
  __syncthreads();
  // u = A v_beta, w = A (k_beta exp(gcs)); A is lower triangular with exact zeros above the diagonal, so a tile of
  // four rows sums j up to its last row.  A thread owns rows 4*tr .. 4*tr+3 and columns tc + 16*i of a 128-column
  // block: 32 fused multiply-adds per 12 shared-memory loads, sums over j ascending.
  {
    const int tr = tid >> 4, tc = tid & 15;
    for (int pass = 0; pass < 2; ++pass) {
      const float* src = pass == 0 ? sQ : sK;           // v_beta, then k (made k_beta exp(gcs) below)
      const int ld = pass == 0 ? QP : KP, width = pass == 0 ? V : K;
      __nv_bfloat16* dst = pass == 0 ? u_out : w_out;
      for (int cb = 0; cb < width; cb += 128) {
        float acc[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[i][c] = 0.f;
        for (int j = 0; j <= tr * 4 + 3; ++j) {
          float av[4], xv[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) av[i] = sS[(tr * 4 + i) * (C + 1) + j];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const int col = cb + tc + 16 * c;
            xv[c] = col < width ? src[j * ld + col] : 0.f;
          }
          if (pass == 1) {
            const float bj = sB[j], ej = sE[j];
#pragma unroll
            for (int c = 0; c < 8; ++c) xv[c] = gdn_round_bf16(xv[c] * bj) * ej;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[i][c] = fmaf(av[i], xv[c], acc[i][c]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const int col = cb + tc + 16 * c;
            if (col < width) dst[(tr * 4 + i) * width + col] = __float2bfloat16_rn(acc[i][c]);
          }
      }
    }
  }
}

// VB = state columns per CTA: 32 (more CTAs) or 64 (half as many CTAs, twice the multiply-adds per shared-memory load).
template <int VB>
__global__ void __launch_bounds__(kGdnThreads) gdn_chunk_scan_kernel(const __nv_bfloat16* __restrict__ q,
                                                                     const __nv_bfloat16* __restrict__ k,
                                                                     const uint8_t* __restrict__ ws,
                                                                     const float* __restrict__ h0,
                                                                     __nv_bfloat16* __restrict__ o,
                                                                     float* __restrict__ h_final, GdnDims D) {
  extern __shared__ float gdn_smem[];
  constexpr int C = kGdnChunk;
  constexpr int CG = VB / 4;                 // groups of 4 adjacent columns
  constexpr int RG = kGdnThreads / CG;       // row groups
  constexpr int RPT = C / RG;                // chunk rows per thread
  const int K = D.K, V = D.V, KP = K + 1;
  float* sH = gdn_smem;               // [K][VB]      this CTA's columns of the state
  float* sQ = sH + K * VB;            // [C][KP]      q exp(gcs)
  float* sK = sQ + C * KP;            // [C][KP]      k, later k exp(gcs_last - gcs)
  float* sW = sK + C * KP;            // [C][KP]      w
  float* sVn = sW + C * KP;           // [C][VB]      u, then v_new
  float* sAt = sVn + C * VB;          // [C][C+1]     in-chunk attention
  float* sG = sAt + C * (C + 1);      // [C]
  float* sEq = sG + C;                // [C] exp(gcs)
  float* sEk = sEq + C;               // [C] exp(gcs_last - gcs)
  const int vb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int v0 = vb * VB;
  const float scale = gdn_round_bf16(rsqrtf((float)K));
  for (int i = tid; i < K * VB; i += kGdnThreads) {
    const int r = i / VB, c = i - r * VB;
    sH[i] = (h0 != nullptr && v0 + c < V) ? h0[(((long long)b * D.H + h) * K + r) * V + v0 + c] : 0.f;
  }
  for (int n = 0; n < D.N; ++n) {
    const long long tok0 = (long long)n * C;
    const uint8_t* cw = ws + (((long long)b * D.N + n) * D.H + h) * gdn_chunk_ws_bytes(K, V);
    const __nv_bfloat16* u_in = reinterpret_cast<const __nv_bfloat16*>(cw);
    const __nv_bfloat16* w_in = u_in + C * V;
    const float* attn_in = reinterpret_cast<const float*>(w_in + C * K);
    const float* gcs_in = attn_in + C * C;
    __syncthreads();   // the previous chunk is done with every buffer
    if (tid < C) {
      const float gc = gcs_in[tid], gl = gcs_in[C - 1];
      sG[tid] = gc;
      sEq[tid] = __expf(gc);        // q rows carry exp(gcs)
      sEk[tid] = __expf(gl - gc);   // k rows carry exp(gcs_last - gcs)
    }
    __syncthreads();
    const float g_last = sG[C - 1];
    if ((K & 7) == 0) {   // 16-byte pieces of the bf16 rows
      const int kv8 = K / 8;
      for (int i = tid; i < C * kv8; i += kGdnThreads) {
        const int r = i / kv8, c = (i - r * kv8) * 8;
        const long long t = tok0 + r;
        uint4 kq[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
        if (t < D.S) {
          const long long off = (((long long)b * D.S + t) * D.H + h) * K + c;
          kq[0] = *reinterpret_cast<const uint4*>(k + off);
          kq[1] = *reinterpret_cast<const uint4*>(q + off);
        }
        const uint4 wv = *reinterpret_cast<const uint4*>(w_in + r * K + c);
        float kf[8], qf[8], wf[8];
        lewi::Elem<__nv_bfloat16>::unpack(kq[0], kf);
        lewi::Elem<__nv_bfloat16>::unpack(kq[1], qf);
        lewi::Elem<__nv_bfloat16>::unpack(wv, wf);
        const float eq = sEq[r], ek = sEk[r];
#pragma unroll
        for (int x = 0; x < 8; ++x) {
          sQ[r * KP + c + x] = gdn_round_bf16(qf[x] * scale) * eq;
          sK[r * KP + c + x] = kf[x] * ek;
          sW[r * KP + c + x] = wf[x];
        }
      }
    } else {
      for (int i = tid; i < C * K; i += kGdnThreads) {
        const int r = i / K, c = i - r * K;
        const long long t = tok0 + r;
        float kv = 0.f, qv = 0.f;
        if (t < D.S) {
          const long long off = (((long long)b * D.S + t) * D.H + h) * K + c;
          kv = __bfloat162float(k[off]);
          qv = gdn_round_bf16(__bfloat162float(q[off]) * scale);
        }
        sQ[r * KP + c] = qv * sEq[r];
        sK[r * KP + c] = kv * sEk[r];
        sW[r * KP + c] = __bfloat162float(w_in[i]);
      }
    }
    for (int i = tid; i < C * VB; i += kGdnThreads) {
      const int r = i / VB, c = i - r * VB;
      sVn[i] = v0 + c < V ? __bfloat162float(u_in[r * V + v0 + c]) : 0.f;
    }
    for (int i = tid; i < C * C; i += kGdnThreads) {
      const int r = i / C, c = i - r * C;
      sAt[r * (C + 1) + c] = attn_in[i];
    }
    __syncthreads();
    // Register tiles: a thread owns 4 adjacent state columns (c0..c0+3) and RPT adjacent rows of the chunk's 64; of the
    // state's K rows it owns rows rg, rg+RG, ...  Every sum runs over its index in ascending order.
    const int c0 = (tid % CG) * 4, rg = tid / CG;
    const int r0 = rg * RPT;
    float vn[RPT][4], acc_o[RPT][4];
#pragma unroll
    for (int x = 0; x < RPT; ++x)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        vn[x][c] = 0.f;
        acc_o[x][c] = 0.f;
      }
    // w h and (q exp(gcs)) h with the OLD state
    for (int kk = 0; kk < K; ++kk) {
      const float4 hv = *reinterpret_cast<const float4*>(&sH[kk * VB + c0]);
      const float h4[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
      for (int x = 0; x < RPT; ++x) {
        const float wv = sW[(r0 + x) * KP + kk], qv = sQ[(r0 + x) * KP + kk];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          vn[x][c] = fmaf(wv, h4[c], vn[x][c]);
          acc_o[x][c] = fmaf(qv, h4[c], acc_o[x][c]);
        }
      }
    }
    // v_new = u - w h, written over u (a thread reads and writes only its own elements)
#pragma unroll
    for (int x = 0; x < RPT; ++x) {
      float4* cell = reinterpret_cast<float4*>(&sVn[(r0 + x) * VB + c0]);
      const float4 u4 = *cell;
      *cell = make_float4(u4.x - vn[x][0], u4.y - vn[x][1], u4.z - vn[x][2], u4.w - vn[x][3]);
    }
    __syncthreads();
    // o = (q exp(gcs)) h + attn v_new
    for (int j = 0; j < C; ++j) {
      const float4 vj = *reinterpret_cast<const float4*>(&sVn[j * VB + c0]);
      const float v4[4] = {vj.x, vj.y, vj.z, vj.w};
#pragma unroll
      for (int x = 0; x < RPT; ++x) {
        const float av = sAt[(r0 + x) * (C + 1) + j];
#pragma unroll
        for (int c = 0; c < 4; ++c) acc_o[x][c] = fmaf(av, v4[c], acc_o[x][c]);
      }
    }
#pragma unroll
    for (int x = 0; x < RPT; ++x) {
      const long long t = tok0 + r0 + x;
      if (t >= D.S) continue;
      __nv_bfloat16* dst = o + (((long long)b * D.S + t) * D.H + h) * V + v0 + c0;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (v0 + c0 + c < V) dst[c] = __float2bfloat16_rn(acc_o[x][c]);
    }
    // h <- h exp(gcs_last) + (k exp(gcs_last - gcs))^T v_new: state rows rg, rg + RG, ... of this thread's 4 columns
    const float dec = __expf(g_last);
    for (int kr0 = rg; kr0 < K; kr0 += 4 * RG) {
      float acc[4][4];
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int kr = kr0 + y * RG;
        const float4 hv = kr < K ? *reinterpret_cast<const float4*>(&sH[kr * VB + c0]) : make_float4(0.f, 0.f, 0.f, 0.f);
        acc[y][0] = hv.x * dec; acc[y][1] = hv.y * dec; acc[y][2] = hv.z * dec; acc[y][3] = hv.w * dec;
      }
      for (int i = 0; i < C; ++i) {
        const float4 vi = *reinterpret_cast<const float4*>(&sVn[i * VB + c0]);
        const float v4[4] = {vi.x, vi.y, vi.z, vi.w};
#pragma unroll
        for (int y = 0; y < 4; ++y) {
          const int kr = kr0 + y * RG;
          const float kv = kr < K ? sK[i * KP + kr] : 0.f;
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[y][c] = fmaf(kv, v4[c], acc[y][c]);
        }
      }
      // every element of the state has one owner in this phase; others read it after the barrier at the top of the
      // next chunk
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int kr = kr0 + y * RG;
        if (kr < K) *reinterpret_cast<float4*>(&sH[kr * VB + c0]) = make_float4(acc[y][0], acc[y][1], acc[y][2], acc[y][3]);
      }
    }
  }
  __syncthreads();
  if (h_final != nullptr) {
    for (int i = tid; i < K * VB; i += kGdnThreads) {
      const int r = i / VB, c = i - r * VB;
      if (v0 + c < V) h_final[(((long long)b * D.H + h) * K + r) * V + v0 + c] = sH[i];
    }
  }
}
