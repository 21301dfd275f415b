// XLA FFI handlers that expose libgla_b200.so to JAX as custom calls (platform "CUDA").
//
// Built only when jaxlib is importable (python -m gla_jax_b200.build --with-jax), against the
// headers jax.ffi.include_dir() provides.  NOT EXERCISED: no environment with jax has been available
// to this library, so this file has been compiled and run nowhere yet.  Each handler unpacks the buffers
// and the stream and forwards to the C ABI of include/gla_b200.h; nothing else happens here.
// Residuals and workspaces are extra results so that XLA owns every allocation.
//
// Batching: the kernels take a leading batch axis natively, and the Python side calls with
// vmap_method="broadcast_all", so under jax.vmap (the reference maps chunk_gla over the batch this way,
// gla.py:1335) every operand arrives with extra leading axes; the handlers fold ALL leading axes into the
// batch size (the byte sizes of residuals and workspaces are linear in it).
#include <cstdint>
#include <string>

#include "xla/ffi/api/ffi.h"

#include "../../include/gla_b200.h"

namespace ffi = xla::ffi;

namespace {

// float32 and bfloat16 are the element types the library has kernels for; -1 for anything else, which
// Checked() below turns into an error instead of reading the buffer with the wrong element size.
int DtypeOf(ffi::DataType t) {
  return t == ffi::DataType::BF16 ? GLA_BF16 : t == ffi::DataType::F32 ? GLA_F32 : -1;
}
ffi::Error BadDtype(const char* what) {
  return ffi::Error(ffi::ErrorCode::kInvalidArgument, std::string(what) + ": element type must be float32 or bfloat16, and hidden, "
                                                                         "value, key and query must share it");
}
template <typename... Bufs>
bool SameSupportedDtype(const ffi::AnyBuffer& first, const Bufs&... rest) {
  if (DtypeOf(first.element_type()) < 0) return false;
  bool same = true;
  ((same = same && rest.element_type() == first.element_type()), ...);
  return same;
}

ffi::Error Status(int st, const char* what) {
  if (st == GLA_OK) return ffi::Error::Success();
  return ffi::Error(ffi::ErrorCode::kInvalidArgument, std::string(what) + ": " + gla_status_string(st));
}

// Shapes: value (..., T, H, D), hidden (..., H, D, D); every leading axis is batch.
struct Dims { int64_t B, T, H, D; };
Dims DimsOf(const ffi::AnyBuffer& value) {
  auto d = value.dimensions();
  const size_t n = d.size();
  if (n < 3) return {0, 0, 0, 0};          // rejected by the C ABI as bad dimensions
  int64_t B = 1;
  for (size_t i = 0; i + 3 < n; ++i) B *= d[i];
  return {B, d[n - 3], d[n - 2], d[n - 1]};
}

ffi::Error ChunkFwd(cudaStream_t stream, ffi::AnyBuffer hidden_init, ffi::Buffer<ffi::F32> log_fgate,
                    ffi::AnyBuffer value, ffi::AnyBuffer key, ffi::AnyBuffer query, int64_t chunk, int64_t impl,
                    ffi::Result<ffi::AnyBuffer> hidden_final, ffi::Result<ffi::AnyBuffer> out,
                    ffi::Result<ffi::AnyBuffer> saved, ffi::Result<ffi::AnyBuffer> workspace) {
  Dims s = DimsOf(value);
  if (!SameSupportedDtype(value, hidden_init, key, query)) return BadDtype("gla_chunk_fwd");
  return Status(gla_chunk_fwd(stream, s.B, s.T, s.H, s.D, chunk, DtypeOf(value.element_type()), (int)impl,
                              hidden_init.untyped_data(), log_fgate.typed_data(), value.untyped_data(),
                              key.untyped_data(), query.untyped_data(), hidden_final->untyped_data(),
                              out->untyped_data(), saved->untyped_data(), workspace->untyped_data(),
                              workspace->size_bytes()),
                "gla_chunk_fwd");
}

ffi::Error ChunkBwd(cudaStream_t stream, ffi::Buffer<ffi::F32> log_fgate, ffi::AnyBuffer value, ffi::AnyBuffer key,
                    ffi::AnyBuffer query, ffi::AnyBuffer saved, ffi::AnyBuffer dhidden_final, ffi::AnyBuffer dout,
                    int64_t chunk, int64_t impl, ffi::Result<ffi::AnyBuffer> dhidden_init,
                    ffi::Result<ffi::Buffer<ffi::F32>> dlog_fgate, ffi::Result<ffi::AnyBuffer> dvalue,
                    ffi::Result<ffi::AnyBuffer> dkey, ffi::Result<ffi::AnyBuffer> dquery,
                    ffi::Result<ffi::AnyBuffer> workspace) {
  Dims s = DimsOf(value);
  if (!SameSupportedDtype(value, key, query, dhidden_final, dout)) return BadDtype("gla_chunk_bwd");
  return Status(gla_chunk_bwd(stream, s.B, s.T, s.H, s.D, chunk, DtypeOf(value.element_type()), (int)impl,
                              log_fgate.typed_data(), value.untyped_data(), key.untyped_data(), query.untyped_data(),
                              saved.untyped_data(), dhidden_final.untyped_data(), dout.untyped_data(),
                              dhidden_init->untyped_data(), dlog_fgate->typed_data(), dvalue->untyped_data(),
                              dkey->untyped_data(), dquery->untyped_data(), workspace->untyped_data(),
                              workspace->size_bytes()),
                "gla_chunk_bwd");
}

ffi::Error RecurrentFwd(cudaStream_t stream, ffi::AnyBuffer hidden_init, ffi::Buffer<ffi::F32> log_fgate,
                        ffi::AnyBuffer value, ffi::AnyBuffer key, ffi::AnyBuffer query, int64_t reverse,
                        ffi::Result<ffi::AnyBuffer> hidden_final, ffi::Result<ffi::AnyBuffer> out) {
  Dims s = DimsOf(value);
  if (!SameSupportedDtype(value, hidden_init, key, query) || DtypeOf(out->element_type()) < 0) return BadDtype("gla_recurrent_fwd");
  return Status(gla_recurrent_fwd(stream, s.B, s.T, s.H, s.D, DtypeOf(value.element_type()),
                                  hidden_init.untyped_data(), log_fgate.typed_data(), value.untyped_data(),
                                  key.untyped_data(), query.untyped_data(), hidden_final->untyped_data(),
                                  out->untyped_data(), DtypeOf(out->element_type()), (int)reverse),
                "gla_recurrent_fwd");
}

ffi::Error RecurrentBwd(cudaStream_t stream, ffi::AnyBuffer hidden_init, ffi::Buffer<ffi::F32> log_fgate,
                        ffi::AnyBuffer value, ffi::AnyBuffer key, ffi::AnyBuffer query, ffi::AnyBuffer dhidden_final,
                        ffi::AnyBuffer dout, int64_t reverse, ffi::Result<ffi::AnyBuffer> dhidden_init,
                        ffi::Result<ffi::Buffer<ffi::F32>> dlog_fgate, ffi::Result<ffi::AnyBuffer> dvalue,
                        ffi::Result<ffi::AnyBuffer> dkey, ffi::Result<ffi::AnyBuffer> dquery,
                        ffi::Result<ffi::AnyBuffer> workspace) {
  Dims s = DimsOf(value);
  if (!SameSupportedDtype(value, hidden_init, key, query, dhidden_final) || DtypeOf(dout.element_type()) < 0)
    return BadDtype("gla_recurrent_bwd");
  return Status(gla_recurrent_bwd(stream, s.B, s.T, s.H, s.D, DtypeOf(value.element_type()),
                                  hidden_init.untyped_data(), log_fgate.typed_data(), value.untyped_data(),
                                  key.untyped_data(), query.untyped_data(), dhidden_final.untyped_data(),
                                  dout.untyped_data(), DtypeOf(dout.element_type()), dhidden_init->untyped_data(),
                                  dlog_fgate->typed_data(), dvalue->untyped_data(), dkey->untyped_data(),
                                  dquery->untyped_data(), (int)reverse, workspace->untyped_data(),
                                  workspace->size_bytes()),
                "gla_recurrent_bwd");
}

// src viewed as (..., T, D) with every leading axis folded into N; init (..., D) or an empty buffer for "no init".
ffi::Error Cumsum(cudaStream_t stream, ffi::AnyBuffer src, ffi::AnyBuffer init, int64_t reverse,
                  ffi::Result<ffi::AnyBuffer> dst) {
  auto d = src.dimensions();
  const size_t n = d.size();
  if (n < 2 || DtypeOf(src.element_type()) < 0 || DtypeOf(dst->element_type()) < 0) return BadDtype("gla_cumsum");
  int64_t N = 1;
  for (size_t i = 0; i + 2 < n; ++i) N *= d[i];
  const void* ip = init.element_count() == 0 ? nullptr : init.untyped_data();
  if (ip != nullptr && init.element_type() != src.element_type()) return BadDtype("gla_cumsum");
  return Status(gla_cumsum(stream, N, d[n - 2], d[n - 1], src.untyped_data(), ip, dst->untyped_data(), (int)reverse,
                           DtypeOf(src.element_type()), DtypeOf(dst->element_type())),
                "gla_cumsum");
}

// log_fgate (..., T, K) float32, kv (..., T, K, V), every leading axis folded into the batch; init buffers may be empty.
ffi::Error RnnScan(cudaStream_t stream, ffi::Buffer<ffi::F32> log_fgate, ffi::AnyBuffer kv,
                   ffi::Buffer<ffi::F32> init_log_fgate, ffi::AnyBuffer init_kv, int64_t reverse, int64_t last_only,
                   ffi::Result<ffi::Buffer<ffi::F32>> out_log, ffi::Result<ffi::AnyBuffer> out_state) {
  auto d = kv.dimensions();
  const size_t n = d.size();
  if (n < 3 || DtypeOf(kv.element_type()) < 0 || out_state->element_type() != kv.element_type()) return BadDtype("gla_rnn_scan");
  int64_t Bn = 1;
  for (size_t i = 0; i + 3 < n; ++i) Bn *= d[i];
  const bool has_init = init_kv.element_count() != 0;
  if (has_init && init_kv.element_type() != kv.element_type()) return BadDtype("gla_rnn_scan");
  return Status(gla_rnn_scan(stream, Bn, d[n - 3], d[n - 2], d[n - 1], log_fgate.typed_data(), kv.untyped_data(),
                             has_init ? init_log_fgate.typed_data() : nullptr,
                             has_init ? init_kv.untyped_data() : nullptr, out_log->typed_data(),
                             out_state->untyped_data(), (int)reverse, (int)last_only, DtypeOf(kv.element_type())),
                "gla_rnn_scan");
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    GlaChunkFwd, ChunkFwd,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>().Arg<ffi::Buffer<ffi::F32>>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Attr<int64_t>("chunk").Attr<int64_t>("impl")
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    GlaChunkBwd, ChunkBwd,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::Buffer<ffi::F32>>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Attr<int64_t>("chunk").Attr<int64_t>("impl").Ret<ffi::AnyBuffer>().Ret<ffi::Buffer<ffi::F32>>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    GlaRecurrentFwd, RecurrentFwd,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>().Arg<ffi::Buffer<ffi::F32>>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Attr<int64_t>("reverse")
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    GlaRecurrentBwd, RecurrentBwd,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>().Arg<ffi::Buffer<ffi::F32>>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Attr<int64_t>("reverse").Ret<ffi::AnyBuffer>().Ret<ffi::Buffer<ffi::F32>>().Ret<ffi::AnyBuffer>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    GlaCumsum, Cumsum,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Attr<int64_t>("reverse").Ret<ffi::AnyBuffer>());

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    GlaRnnScan, RnnScan,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::Buffer<ffi::F32>>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::Buffer<ffi::F32>>().Arg<ffi::AnyBuffer>().Attr<int64_t>("reverse").Attr<int64_t>("last_only")
        .Ret<ffi::Buffer<ffi::F32>>().Ret<ffi::AnyBuffer>());
