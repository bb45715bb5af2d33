// See ffi_core.h.  Build (no CUDA or JAX headers needed):
//   g++ -std=c++17 -shared -fPIC -Iinclude lewi_surge_b200/csrc/ffi_core.cc -Llewi_surge_b200 -llewi_moe -o libffi_core.so
#include "ffi_core.h"

namespace lewi_ffi {

int sort_indices(void* stream, const int32_t* flat, int64_t m, int num_experts, int32_t* order, int32_t* pos,
                 void* scratch, int64_t scratch_bytes) {
  return lewi_sort_indices(stream, flat, m, num_experts, 0, order, pos, nullptr, nullptr, nullptr, nullptr, nullptr,
                           nullptr, nullptr, scratch, scratch_bytes);
}

int gather_rows(void* stream, const void* x, int64_t n_src, int d, int dtype, const int32_t* idx, int64_t m,
                const float* scale, void* out, int idx_div, bool scale_by_idx) {
  return lewi_gather_rows(stream, x, idx, scale, out, n_src, m, d, dtype, idx_div, scale_by_idx ? 1 : 0, nullptr, 1);
}

int gather_reduce(void* stream, const void* y, int64_t n_y_rows, int d, int in_dtype, const int32_t* pos, int64_t n, int k,
                  const float* w, void* out, int out_dtype) {
  return lewi_gather_reduce(stream, y, pos, w, nullptr, nullptr, out, n, k, d, in_dtype, out_dtype, n_y_rows);
}

int gather_dot(void* stream, const void* y, int64_t n_y_rows, int d, int dtype, const int32_t* pos, int64_t n, int k,
               const void* g, float* out) {
  return lewi_gather_dot(stream, y, pos, g, out, n, k, d, dtype, n_y_rows);
}

int ragged_dot_fwd(void* stream, const void* lhs, const void* rhs, const int32_t* group_sizes, int64_t m, int k, int n,
                   int e, void* out, int32_t* pad_offsets, int32_t* block_expert, int32_t* n_blocks,
                   int32_t* row_of_padded, int32_t* padded_of_row, void* lhs_pad, void* out_pad) {
  const int64_t mpad = lewi_padded_rows_bound(m, e, kBlock);
  if (int rc = lewi_group_tables(stream, group_sizes, m, e, kBlock, pad_offsets, block_expert, n_blocks, row_of_padded,
                                 padded_of_row))
    return rc;
  if (int rc = lewi_gather_rows(stream, lhs, row_of_padded, nullptr, lhs_pad, m, mpad, k, LEWI_BF16, 1, 0, n_blocks, kBlock))
    return rc;
  if (int rc = lewi_grouped_gemm_nn(stream, lhs_pad, rhs, out_pad, nullptr, block_expert, n_blocks, pad_offsets, mpad, k, n,
                                    e, LEWI_BF16))
    return rc;
  return lewi_gather_rows(stream, out_pad, padded_of_row, nullptr, out, mpad, m, n, LEWI_BF16, 1, 0, nullptr, 1);
}

int ragged_dot_dlhs(void* stream, const void* g, const void* rhs, const int32_t* pad_offsets, const int32_t* block_expert,
                    const int32_t* n_blocks, const int32_t* row_of_padded, const int32_t* padded_of_row, int64_t m,
                    int64_t mpad, int k, int n, int e, void* dlhs, void* g_pad, void* dl_pad) {
  if (int rc = lewi_gather_rows(stream, g, row_of_padded, nullptr, g_pad, m, mpad, n, LEWI_BF16, 1, 0, n_blocks, kBlock))
    return rc;
  // rhs [e,k,n] read as the K-major operand [e, N' = k, K' = n] of g . rhs^T
  if (int rc = lewi_grouped_gemm_nt(stream, g_pad, rhs, dl_pad, nullptr, block_expert, n_blocks, pad_offsets, mpad, n, k, e,
                                    LEWI_BF16))
    return rc;
  return lewi_gather_rows(stream, dl_pad, padded_of_row, nullptr, dlhs, mpad, m, k, LEWI_BF16, 1, 0, nullptr, 1);
}

int64_t ragged_dot_drhs_scratch_bytes(int64_t mpad, int k, int n, int e) {
  return lewi_grouped_gemm_tn_workspace_bytes(mpad, k, n, e, 0);
}

int ragged_dot_drhs(void* stream, const void* lhs_pad, const void* g_pad, const int32_t* pad_offsets, int64_t mpad, int k,
                    int n, int e, float* drhs, void* scratch, int64_t scratch_bytes) {
  return lewi_grouped_gemm_tn(stream, lhs_pad, g_pad, drhs, nullptr, pad_offsets, mpad, k, n, e, LEWI_F32,
                              scratch_bytes > 0 ? scratch : nullptr, scratch_bytes);
}

int64_t moe_residual_bytes(const MoeDims& D) {
  return lewi_moe_residual_layout(D.T, D.d, D.E, D.f, D.k, D.fs, D.has_gate ? 1 : 0, nullptr);
}

int64_t moe_workspace_bytes(const MoeDims& D) {
  return lewi_moe_workspace_bytes(D.T, D.d, D.E, D.f, D.k, D.fs, D.has_gate ? 1 : 0);
}

int moe_fwd(void* stream, const MoeDims& D, const void* x, const float* w_router, const float* router_bias,
            const void* w_gate, const void* w_up, const void* w_down, const void* ws_gate, const void* ws_up,
            const void* ws_down, const float* w_sg, void* out, float* aux_loss, void* residual, int64_t residual_bytes,
            void* workspace, int64_t workspace_bytes) {
  // one stream only: XLA hands a custom call a single stream, so the shared expert is queued in line
  return lewi_moe_fwd(stream, nullptr, x, w_router, D.has_bias ? router_bias : nullptr, nullptr, w_gate, w_up, w_down,
                      D.fs > 0 ? ws_gate : nullptr, D.fs > 0 ? ws_up : nullptr, D.fs > 0 ? ws_down : nullptr,
                      D.has_gate ? w_sg : nullptr, out, aux_loss, residual, residual_bytes, workspace, workspace_bytes, D.T,
                      D.d, D.E, D.f, D.k, D.fs);
}

int moe_bwd(void* stream, const MoeDims& D, const void* dout, const void* x, const float* w_router, const void* w_gate,
            const void* w_up, const void* w_down, const void* ws_gate, const void* ws_up, const void* ws_down,
            const float* w_sg, const void* residual, int64_t residual_bytes, void* workspace, int64_t workspace_bytes,
            void* dx, float* dw_router, float* d_router_bias, void* dw_gate, void* dw_up, void* dw_down, void* dws_gate,
            void* dws_up, void* dws_down, float* dw_sg, float aux_grad, int wgrad_dtype) {
  const bool sh = D.fs > 0;
  return lewi_moe_bwd(stream, nullptr, dout, x, w_router, nullptr, w_gate, w_up, w_down, sh ? ws_gate : nullptr,
                      sh ? ws_up : nullptr, sh ? ws_down : nullptr, D.has_gate ? w_sg : nullptr, residual, residual_bytes,
                      workspace, workspace_bytes, dx, dw_router, D.has_bias ? d_router_bias : nullptr, dw_gate, dw_up, dw_down,
                      sh ? dws_gate : nullptr, sh ? dws_up : nullptr, sh ? dws_down : nullptr, D.has_gate ? dw_sg : nullptr,
                      nullptr, aux_grad, wgrad_dtype, D.T, D.d, D.E, D.f, D.k, D.fs);
}

int64_t causal_conv1d_scratch_bytes(int b, int t, int c, int k) { return lewi_causal_conv1d_workspace_bytes(b, t, c, k); }

int causal_conv1d_fwd(void* stream, const void* x, const void* w, void* y, int b, int t, int c, int k) {
  return lewi_causal_conv1d_fwd(stream, x, w, y, b, t, c, k);
}

int causal_conv1d_bwd(void* stream, const void* x, const void* w, const void* g, void* dx, float* dw, void* scratch,
                      int64_t scratch_bytes, int b, int t, int c, int k) {
  return lewi_causal_conv1d_bwd(stream, x, w, g, dx, dw, LEWI_F32, scratch, scratch_bytes, b, t, c, k);
}

int64_t gdn_chunk_fwd_scratch_bytes(int b, int s, int h, int k, int v) { return lewi_gdn_chunk_workspace_bytes(b, s, h, k, v); }
int64_t gdn_chunk_bwd_scratch_bytes(int b, int s, int h, int k, int v) {
  return lewi_gdn_chunk_bwd_workspace_bytes(b, s, h, k, v);
}

int gdn_chunk_fwd(void* stream, const void* q, const void* k, const void* v, const float* g, const void* beta,
                  const float* h0, void* o, float* h_final, void* saved, int64_t saved_bytes, int b, int s, int h, int kd,
                  int vd) {
  return lewi_gdn_chunk_fwd(stream, q, k, v, g, beta, h0, o, h_final, saved, saved_bytes, b, s, h, kd, vd);
}

int gdn_chunk_bwd(void* stream, const void* q, const void* k, const void* v, const float* g, const void* beta,
                  const float* h0, const void* d_o, const float* dh_final, const void* saved, int64_t saved_bytes,
                  void* scratch, int64_t scratch_bytes, void* dq, void* dk, void* dv, float* dg, void* dbeta, float* dh0,
                  int b, int s, int h, int kd, int vd) {
  return lewi_gdn_chunk_bwd(stream, q, k, v, g, beta, h0, d_o, dh_final, saved, saved_bytes, scratch, scratch_bytes, dq, dk,
                            dv, dg, dbeta, dh0, b, s, h, kd, vd);
}

}  // namespace lewi_ffi
