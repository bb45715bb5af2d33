// XLA FFI handlers over the C ABI of liblewi_moe.so.  Compiled only where jaxlib's headers exist:
//   nvcc -shared -Xcompiler -fPIC -std=c++17 -I$(python -c "import jax; print(jax.ffi.include_dir())") \
//        -Iinclude lewi_surge_b200/csrc/ffi_xla.cc -Llewi_surge_b200 -llewi_moe -o liblewi_moe_ffi.so
// Each handler reads device pointers, dimensions and the CUDA stream from the call frame and forwards
// to the entry point of the same name; a non-zero return code becomes an ffi::Error.  All scratch is
// passed in as extra result buffers, so XLA owns every allocation.
#include <cstdint>

#include "../../include/lewi_moe.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error Check(int rc, const char* what) {
  if (rc == 0) return ffi::Error::Success();
  return ffi::Error(ffi::ErrorCode::kInvalidArgument, std::string(what) + ": " + lewi_error_string(rc));
}

int DType(ffi::DataType t) { return t == ffi::DataType::F32 ? LEWI_F32 : LEWI_BF16; }

// sort_indices(flat_experts[M], num_experts) -> order[M], pos[M]; scratch u8[workspace]
ffi::Error SortIndices(cudaStream_t stream, ffi::Buffer<ffi::S32> flat, ffi::ResultBuffer<ffi::S32> order,
                       ffi::ResultBuffer<ffi::S32> pos, ffi::ResultBuffer<ffi::U8> scratch, int32_t num_experts) {
  const int64_t m = flat.element_count();
  return Check(lewi_sort_indices(stream, flat.typed_data(), m, num_experts, 0, order->typed_data(), pos->typed_data(),
                                 nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, scratch->typed_data(),
                                 (int64_t)scratch->element_count()),
               "lewi_sort_indices");
}

// gather_rows(x[N,D], idx[M], scale[M] or empty) -> out[M,D]
ffi::Error GatherRows(cudaStream_t stream, ffi::AnyBuffer x, ffi::Buffer<ffi::S32> idx, ffi::Buffer<ffi::F32> scale,
                      ffi::Result<ffi::AnyBuffer> out, bool has_scale, int32_t idx_div, bool scale_by_idx) {
  const auto dims = x.dimensions();
  return Check(lewi_gather_rows(stream, x.untyped_data(), idx.typed_data(), has_scale ? scale.typed_data() : nullptr,
                                out->untyped_data(), dims[0], idx.element_count(), (int)dims[1], DType(x.element_type()),
                                idx_div, scale_by_idx ? 1 : 0, nullptr, 1),
               "lewi_gather_rows");
}

// gather_reduce(y[M,D], pos[N,k], w[N,k] or empty) -> out[N,D]
ffi::Error GatherReduce(cudaStream_t stream, ffi::AnyBuffer y, ffi::Buffer<ffi::S32> pos, ffi::Buffer<ffi::F32> w,
                        ffi::Result<ffi::AnyBuffer> out, bool has_w) {
  const auto yd = y.dimensions();
  const auto pd = pos.dimensions();
  return Check(lewi_gather_reduce(stream, y.untyped_data(), pos.typed_data(), has_w ? w.typed_data() : nullptr, nullptr,
                                  nullptr, out->untyped_data(), pd[0], (int)pd[1], (int)yd[1], DType(y.element_type()),
                                  DType(out->element_type()), yd[0]),
               "lewi_gather_reduce");
}

// gather_dot(y[M,D], pos[N,k], g[N,D]) -> out[N,k] f32
ffi::Error GatherDot(cudaStream_t stream, ffi::AnyBuffer y, ffi::Buffer<ffi::S32> pos, ffi::AnyBuffer g,
                     ffi::ResultBuffer<ffi::F32> out) {
  const auto yd = y.dimensions();
  const auto pd = pos.dimensions();
  return Check(lewi_gather_dot(stream, y.untyped_data(), pos.typed_data(), g.untyped_data(), out->typed_data(), pd[0],
                               (int)pd[1], (int)yd[1], DType(y.element_type()), yd[0]),
               "lewi_gather_dot");
}

// ragged_dot forward: lhs[M,K] bf16 (sorted by expert), rhs[E,K,N] bf16, group_sizes[E] -> out[M,N] bf16.
// Scratch results: tables (pad_offsets[E+1], block_expert[Mpad/128], n_blocks[1], row_of_padded[Mpad],
// padded_of_row[M]) and the two padded buffers lhs_pad[Mpad,K], out_pad[Mpad,N].
ffi::Error RaggedDotFwd(cudaStream_t stream, ffi::Buffer<ffi::BF16> lhs, ffi::Buffer<ffi::BF16> rhs,
                        ffi::Buffer<ffi::S32> gs, ffi::ResultBuffer<ffi::BF16> out, ffi::ResultBuffer<ffi::S32> pad_offsets,
                        ffi::ResultBuffer<ffi::S32> block_expert, ffi::ResultBuffer<ffi::S32> n_blocks,
                        ffi::ResultBuffer<ffi::S32> row_of_padded, ffi::ResultBuffer<ffi::S32> padded_of_row,
                        ffi::ResultBuffer<ffi::BF16> lhs_pad, ffi::ResultBuffer<ffi::BF16> out_pad) {
  const int64_t m = lhs.dimensions()[0];
  const int k = (int)lhs.dimensions()[1], e = (int)rhs.dimensions()[0], n = (int)rhs.dimensions()[2];
  const int64_t mpad = lewi_padded_rows_bound(m, e, 128);
  if (int rc = lewi_group_tables(stream, gs.typed_data(), m, e, 128, pad_offsets->typed_data(), block_expert->typed_data(),
                                 n_blocks->typed_data(), row_of_padded->typed_data(), padded_of_row->typed_data()))
    return Check(rc, "lewi_group_tables");
  if (int rc = lewi_gather_rows(stream, lhs.typed_data(), row_of_padded->typed_data(), nullptr, lhs_pad->typed_data(), m,
                                mpad, k, LEWI_BF16, 1, 0, n_blocks->typed_data(), 128))
    return Check(rc, "lewi_gather_rows");
  if (int rc = lewi_grouped_gemm_nn(stream, lhs_pad->typed_data(), rhs.typed_data(), out_pad->typed_data(), nullptr,
                                    block_expert->typed_data(), n_blocks->typed_data(), mpad, k, n, e, LEWI_BF16))
    return Check(rc, "lewi_grouped_gemm_nn");
  return Check(lewi_gather_rows(stream, out_pad->typed_data(), padded_of_row->typed_data(), nullptr, out->typed_data(),
                                mpad, m, n, LEWI_BF16, 1, 0, nullptr, 1),
               "lewi_gather_rows");
}

// dlhs = g . rhs[e]^T over the tables saved by the forward: g[M,N], rhs[E,K,N] -> dlhs[M,K]
ffi::Error RaggedDotDlhs(cudaStream_t stream, ffi::Buffer<ffi::BF16> g, ffi::Buffer<ffi::BF16> rhs,
                         ffi::Buffer<ffi::S32> block_expert, ffi::Buffer<ffi::S32> n_blocks,
                         ffi::Buffer<ffi::S32> row_of_padded, ffi::Buffer<ffi::S32> padded_of_row,
                         ffi::ResultBuffer<ffi::BF16> dlhs, ffi::ResultBuffer<ffi::BF16> g_pad,
                         ffi::ResultBuffer<ffi::BF16> dl_pad) {
  const int64_t m = g.dimensions()[0], mpad = row_of_padded.element_count();
  const int n = (int)g.dimensions()[1], e = (int)rhs.dimensions()[0], k = (int)rhs.dimensions()[1];
  if (int rc = lewi_gather_rows(stream, g.typed_data(), row_of_padded.typed_data(), nullptr, g_pad->typed_data(), m, mpad,
                                n, LEWI_BF16, 1, 0, n_blocks.typed_data(), 128))
    return Check(rc, "lewi_gather_rows");
  // rhs [E,K,N] read as the K-major operand [E, N'=K, K'=N] of g . rhs^T
  if (int rc = lewi_grouped_gemm_nt(stream, g_pad->typed_data(), rhs.typed_data(), dl_pad->typed_data(), nullptr,
                                    block_expert.typed_data(), n_blocks.typed_data(), mpad, n, k, e, LEWI_BF16))
    return Check(rc, "lewi_grouped_gemm_nt");
  return Check(lewi_gather_rows(stream, dl_pad->typed_data(), padded_of_row.typed_data(), nullptr, dlhs->typed_data(),
                                mpad, m, k, LEWI_BF16, 1, 0, nullptr, 1),
               "lewi_gather_rows");
}

// drhs[e] = lhs_pad[rows of e]^T . g_pad[rows of e]  -> [E,K,N] f32
ffi::Error RaggedDotDrhs(cudaStream_t stream, ffi::Buffer<ffi::BF16> lhs_pad, ffi::Buffer<ffi::BF16> g_pad,
                         ffi::Buffer<ffi::S32> pad_offsets, ffi::ResultBuffer<ffi::F32> drhs) {
  const int64_t mpad = lhs_pad.dimensions()[0];
  const int k = (int)lhs_pad.dimensions()[1], n = (int)g_pad.dimensions()[1];
  const int e = (int)pad_offsets.element_count() - 1;
  return Check(lewi_grouped_gemm_tn(stream, lhs_pad.typed_data(), g_pad.typed_data(), drhs->typed_data(), nullptr,
                                    pad_offsets.typed_data(), mpad, k, n, e, LEWI_F32, nullptr, 0),
               "lewi_grouped_gemm_tn");
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(lewi_ffi_sort_indices, SortIndices,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::U8>>()
                                  .Attr<int32_t>("num_experts"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(lewi_ffi_gather_rows, GatherRows,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::F32>>().Ret<ffi::AnyBuffer>()
                                  .Attr<bool>("has_scale").Attr<int32_t>("idx_div").Attr<bool>("scale_by_idx"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(lewi_ffi_gather_reduce, GatherReduce,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::F32>>().Ret<ffi::AnyBuffer>()
                                  .Attr<bool>("has_w"));
XLA_FFI_DEFINE_HANDLER_SYMBOL(lewi_ffi_gather_dot, GatherDot,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::AnyBuffer>().Ret<ffi::Buffer<ffi::F32>>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(lewi_ffi_ragged_dot_fwd, RaggedDotFwd,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::Buffer<ffi::BF16>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>().Arg<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::BF16>>()
                                  .Ret<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::S32>>()
                                  .Ret<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::BF16>>()
                                  .Ret<ffi::Buffer<ffi::BF16>>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(lewi_ffi_ragged_dot_dlhs, RaggedDotDlhs,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::Buffer<ffi::BF16>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>().Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
                                  .Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::BF16>>()
                                  .Ret<ffi::Buffer<ffi::BF16>>().Ret<ffi::Buffer<ffi::BF16>>());
XLA_FFI_DEFINE_HANDLER_SYMBOL(lewi_ffi_ragged_dot_drhs, RaggedDotDrhs,
                              ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::Buffer<ffi::BF16>>()
                                  .Arg<ffi::Buffer<ffi::BF16>>().Arg<ffi::Buffer<ffi::S32>>().Ret<ffi::Buffer<ffi::F32>>());
