// XLA-free core of the jax.ffi shim: every handler of ffi_xla.cc reads pointers, extents and attributes out of its
// call frame and forwards them to one of these functions, which only know plain pointers and sizes and call the
// C ABI of liblewi_moe.so (include/lewi_moe.h).  This translation unit compiles with any C++17 compiler and needs no
// JAX, so the argument lists are checked against the header wherever the library itself is built.
#pragma once

#include <cstdint>

#include "../../include/lewi_moe.h"

namespace lewi_ffi {

constexpr int kBlock = 128;

// Extents of one MoE layer call, read off the operand shapes by the handlers.
struct MoeDims {
  int64_t T;
  int d, E, f, k, fs;
  bool has_bias, has_gate;
};

int sort_indices(void* stream, const int32_t* flat, int64_t m, int num_experts, int32_t* order, int32_t* pos,
                 void* scratch, int64_t scratch_bytes);
int gather_rows(void* stream, const void* x, int64_t n_src, int d, int dtype, const int32_t* idx, int64_t m,
                const float* scale, void* out, int idx_div, bool scale_by_idx);
int gather_reduce(void* stream, const void* y, int64_t n_y_rows, int d, int in_dtype, const int32_t* pos, int64_t n, int k,
                  const float* w, void* out, int out_dtype);
int gather_dot(void* stream, const void* y, int64_t n_y_rows, int d, int dtype, const int32_t* pos, int64_t n, int k,
               const void* g, float* out);

// ragged_dot: lhs [m,k] bf16 sorted by expert, rhs [e,k,n] bf16, group_sizes [e].  The tables and the two padded
// buffers are results of the forward call (XLA owns them) and inputs of the two backward calls.
int ragged_dot_fwd(void* stream, const void* lhs, const void* rhs, const int32_t* group_sizes, int64_t m, int k, int n,
                   int e, void* out, int32_t* pad_offsets, int32_t* block_expert, int32_t* n_blocks,
                   int32_t* row_of_padded, int32_t* padded_of_row, void* lhs_pad, void* out_pad);
int ragged_dot_dlhs(void* stream, const void* g, const void* rhs, const int32_t* pad_offsets, const int32_t* block_expert,
                    const int32_t* n_blocks, const int32_t* row_of_padded, const int32_t* padded_of_row, int64_t m,
                    int64_t mpad, int k, int n, int e, void* dlhs, void* g_pad, void* dl_pad);
int ragged_dot_drhs(void* stream, const void* lhs_pad, const void* g_pad, const int32_t* pad_offsets, int64_t mpad, int k,
                    int n, int e, float* drhs, void* scratch, int64_t scratch_bytes);
int64_t ragged_dot_drhs_scratch_bytes(int64_t mpad, int k, int n, int e);

// The whole layer (lewi_moe_fwd / lewi_moe_bwd).  Null pointers stand for absent optional operands.
int64_t moe_residual_bytes(const MoeDims& D);
int64_t moe_workspace_bytes(const MoeDims& D);
int moe_fwd(void* stream, const MoeDims& D, const void* x, const float* w_router, const float* router_bias,
            const void* w_gate, const void* w_up, const void* w_down, const void* ws_gate, const void* ws_up,
            const void* ws_down, const float* w_sg, void* out, float* aux_loss, void* residual, int64_t residual_bytes,
            void* workspace, int64_t workspace_bytes);
int moe_bwd(void* stream, const MoeDims& D, const void* dout, const void* x, const float* w_router, const void* w_gate,
            const void* w_up, const void* w_down, const void* ws_gate, const void* ws_up, const void* ws_down,
            const float* w_sg, const void* residual, int64_t residual_bytes, void* workspace, int64_t workspace_bytes,
            void* dx, float* dw_router, float* d_router_bias, void* dw_gate, void* dw_up, void* dw_down, void* dws_gate,
            void* dws_up, void* dws_down, float* dw_sg, float aux_grad, int wgrad_dtype);

// Sequence mixing beside the layer: the causal depthwise convolution and the chunked gated delta rule, each with its
// gradient.  Scratch sizes come from the library; XLA allocates them as extra results.
int64_t causal_conv1d_scratch_bytes(int b, int t, int c, int k);
int causal_conv1d_fwd(void* stream, const void* x, const void* w, void* y, int b, int t, int c, int k);
int causal_conv1d_bwd(void* stream, const void* x, const void* w, const void* g, void* dx, float* dw, void* scratch,
                      int64_t scratch_bytes, int b, int t, int c, int k);
int64_t gdn_chunk_fwd_scratch_bytes(int b, int s, int h, int k, int v);
int64_t gdn_chunk_bwd_scratch_bytes(int b, int s, int h, int k, int v);
int gdn_chunk_fwd(void* stream, const void* q, const void* k, const void* v, const float* g, const void* beta,
                  const float* h0, void* o, float* h_final, void* saved, int64_t saved_bytes, int b, int s, int h, int kd,
                  int vd);
int gdn_chunk_bwd(void* stream, const void* q, const void* k, const void* v, const float* g, const void* beta,
                  const float* h0, const void* d_o, const float* dh_final, const void* saved, int64_t saved_bytes,
                  void* scratch, int64_t scratch_bytes, void* dq, void* dk, void* dv, float* dg, void* dbeta, float* dh0,
                  int b, int s, int h, int kd, int vd);

}  // namespace lewi_ffi
