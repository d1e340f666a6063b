// XLA FFI handlers over the bsx C ABI: the custom-call targets a JAX binding of
// brainstate's event-connection layers registers (jax.ffi.register_ffi_target) in place
// of brainevent's Numba/Warp/Pallas kernels.  One handler per product that
// brainstate/nn/_event_fixedprob.py:202-205,249-252 and _event_linear.py:99-100 reach,
// plus the two reverse-mode products pinned by _event_fixedprob_test.py:56-88.
//
// Compiled only where the XLA FFI headers exist (they ship inside jaxlib:
// `python -c "import jax.ffi; print(jax.ffi.include_dir())"`):
//
//   g++ -O2 -fPIC -shared -std=c++17 -I <jax.ffi.include_dir()> -I include \
//       -I /usr/local/cuda/include ffi/bsx_ffi.cc -o libbsx_ffi.so -L brainstate_b200 -lbsx
//
// Conventions shared by all handlers:
//  - operands may carry any number of leading batch dimensions; all but the last
//    dimension are folded into the batch the C ABI takes (this is also what makes
//    jax.vmap with vmap_method="expand_dims"/"broadcast_all" a single launch);
//  - the connectivity arrives as (indices int32 [n_pre, K] or [nnz], indptr int32/int64 [n_pre+1]
//    or [0] for the fixed-number layout, weights f32 [1] or same shape as indices);
//  - scratch memory is an extra result buffer XLA allocates, sized at trace time with the
//    bsx_*_workspace_bytes functions: nothing is allocated inside a handler;
//  - the work is enqueued on XLA's stream; a negative bsx status becomes an ffi::Error
//    carrying bsx_last_error_string().
#if __has_include("xla/ffi/api/ffi.h")
#include <cstdint>

#include <cuda_runtime_api.h>

#include "bsx.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error Status(int rc) {
  if (rc >= 0) return ffi::Error::Success();
  return ffi::Error::Internal(bsx_last_error_string());
}

// Last dimension, and the product of all others (the folded batch).
struct Folded {
  int64_t batch, n;
};
template <typename Buf>
Folded Fold(const Buf& b) {
  auto dims = b.dimensions();
  if (dims.size() == 0) return {1, 1};
  const int64_t n = dims[dims.size() - 1];
  return {n ? static_cast<int64_t>(b.element_count()) / n : 0, n};
}

int SpikeFormat(ffi::DataType t, bool* ok) {
  *ok = true;
  switch (t) {
    case ffi::DataType::PRED:
    case ffi::DataType::U8:
      return BSX_SPK_BOOL8;
    case ffi::DataType::F32:
      return BSX_SPK_F32;
    case ffi::DataType::U32:
    case ffi::DataType::S32:
      return BSX_SPK_BITS32;      // packed words; the caller says so by passing integers
    default:
      *ok = false;
      return 0;
  }
}

// bsx_conn_t from the three connectivity operands.
bool MakeConn(ffi::AnyBuffer indices, ffi::AnyBuffer indptr, ffi::AnyBuffer weights, int64_t n_pre, int64_t n_post,
              bsx_conn_t* c) {
  if (indices.element_type() != ffi::DataType::S32 || weights.element_type() != ffi::DataType::F32) return false;
  c->n_pre = n_pre;
  c->n_post = n_post;
  c->nnz = static_cast<int64_t>(indices.element_count());
  c->indices = static_cast<const int32_t*>(indices.untyped_data());
  c->weights = static_cast<const float*>(weights.untyped_data());
  c->hetero = weights.element_count() == indices.element_count() && indices.element_count() > 1;
  if (indptr.element_count() == 0) {
    c->indptr = nullptr;
    c->indptr_is_64 = 0;
    c->conn_num = n_pre ? c->nnz / n_pre : 0;
  } else {
    if (indptr.element_type() != ffi::DataType::S32 && indptr.element_type() != ffi::DataType::S64) return false;
    c->indptr = indptr.untyped_data();
    c->indptr_is_64 = indptr.element_type() == ffi::DataType::S64;
    c->conn_num = 0;
  }
  return true;
}

// y = EventArray(spk) @ conn   (event = 1)   or   y = x @ conn   (event = 0, float x)
ffi::Error VecmatImpl(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer indices, ffi::AnyBuffer indptr,
                      ffi::AnyBuffer weights, ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> scratch,
                      int64_t n_post, bool event) {
  const Folded f = Fold(x);
  bsx_conn_t c;
  if (!MakeConn(indices, indptr, weights, f.n, n_post, &c)) return ffi::Error::InvalidArgument("bsx: bad connectivity operands");
  float* y = static_cast<float*>(out->untyped_data());
  if (!event) {
    if (x.element_type() != ffi::DataType::F32) return ffi::Error::InvalidArgument("bsx: float vecmat takes f32");
    return Status(bsx_float_vecmat(&c, static_cast<const float*>(x.untyped_data()), f.batch, y, 0,
                                   scratch->untyped_data(), scratch->size_bytes(), stream));
  }
  bool ok;
  const int fmt = SpikeFormat(x.element_type(), &ok);
  if (!ok) return ffi::Error::InvalidArgument("bsx: spikes must be bool, uint8, float32 or packed 32-bit words");
  if (fmt == BSX_SPK_BITS32) c.n_pre = indptr.element_count() ? static_cast<int64_t>(indptr.element_count()) - 1
                                                                : indices.dimensions()[0];
  return Status(bsx_event_vecmat(&c, x.untyped_data(), fmt, f.batch, y, 0, scratch->untyped_data(),
                                 scratch->size_bytes(), stream));
}

// y = conn @ EventArray(s)  (event = 1, deterministic gather)  or  y = conn @ v  (event = 0)
ffi::Error MatvecImpl(cudaStream_t stream, ffi::AnyBuffer v, ffi::AnyBuffer indices, ffi::AnyBuffer indptr,
                      ffi::AnyBuffer weights, ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> scratch,
                      int64_t n_pre, bool event) {
  const Folded f = Fold(v);
  bsx_conn_t c;
  if (!MakeConn(indices, indptr, weights, n_pre, f.n, &c)) return ffi::Error::InvalidArgument("bsx: bad connectivity operands");
  float* y = static_cast<float*>(out->untyped_data());
  if (!event) {
    if (v.element_type() != ffi::DataType::F32) return ffi::Error::InvalidArgument("bsx: float matvec takes f32");
    return Status(bsx_float_matvec(&c, static_cast<const float*>(v.untyped_data()), f.batch, y, stream));
  }
  bool ok;
  const int fmt = SpikeFormat(v.element_type(), &ok);
  if (!ok || fmt == BSX_SPK_BITS32) return ffi::Error::InvalidArgument("bsx: spikes must be bool, uint8 or float32");
  return Status(bsx_event_matvec(&c, v.untyped_data(), fmt, f.batch, y, scratch->untyped_data(), scratch->size_bytes(),
                                 stream));
}

// Cotangents of y = x @ conn: dx (batch, n_pre) and dw (shape of the weights).
ffi::Error VjpImpl(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer ct, ffi::AnyBuffer indices, ffi::AnyBuffer indptr,
                   ffi::AnyBuffer weights, ffi::Result<ffi::AnyBuffer> dx, ffi::Result<ffi::AnyBuffer> dw,
                   ffi::Result<ffi::AnyBuffer> scratch, bool event) {
  const Folded fx = Fold(x), fc = Fold(ct);
  if (fx.batch != fc.batch) return ffi::Error::InvalidArgument("bsx: x and ct disagree on the batch");
  bsx_conn_t c;
  if (!MakeConn(indices, indptr, weights, fx.n, fc.n, &c)) return ffi::Error::InvalidArgument("bsx: bad connectivity operands");
  bool ok;
  const int fmt = SpikeFormat(x.element_type(), &ok);
  if (!ok || fmt == BSX_SPK_BITS32) return ffi::Error::InvalidArgument("bsx: the primal input must be bool, uint8 or float32");
  if (ct.element_type() != ffi::DataType::F32) return ffi::Error::InvalidArgument("bsx: the cotangent must be float32");
  float* pdx = dx->element_count() ? static_cast<float*>(dx->untyped_data()) : nullptr;
  float* pdw = dw->element_count() ? static_cast<float*>(dw->untyped_data()) : nullptr;
  const float* pct = static_cast<const float*>(ct.untyped_data());
  if (fx.batch >= 4)
    return Status(bsx_vecmat_vjp_batched(&c, x.untyped_data(), fmt, event, pct, fx.batch, pdx, pdw, scratch->untyped_data(),
                                         scratch->size_bytes(), stream));
  return Status(bsx_vecmat_vjp(&c, x.untyped_data(), fmt, event, pct, fx.batch, pdx, pdw, stream));
}

// y = EventArray(spk) @ W for a dense row-major W (n_pre, n_post).
ffi::Error DenseEventImpl(cudaStream_t stream, ffi::AnyBuffer spk, ffi::Buffer<ffi::F32> weight,
                          ffi::Result<ffi::Buffer<ffi::F32>> out) {
  const Folded f = Fold(spk);
  auto wd = weight.dimensions();
  if (wd.size() != 2 || wd[0] != f.n) return ffi::Error::InvalidArgument("bsx: weight must be (n_pre, n_post)");
  bool ok;
  const int fmt = SpikeFormat(spk.element_type(), &ok);
  if (!ok || fmt == BSX_SPK_BITS32) return ffi::Error::InvalidArgument("bsx: spikes must be bool, uint8 or float32");
  return Status(bsx_dense_event_vecmat(spk.untyped_data(), fmt, weight.typed_data(), f.batch, wd[0], wd[1],
                                       out->typed_data(), stream));
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(bsx_ffi_vecmat, VecmatImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // x or spikes
                                  .Arg<ffi::AnyBuffer>()   // indices
                                  .Arg<ffi::AnyBuffer>()   // indptr (empty: fixed-number layout)
                                  .Arg<ffi::AnyBuffer>()   // weights
                                  .Ret<ffi::AnyBuffer>()   // y
                                  .Ret<ffi::AnyBuffer>()   // scratch
                                  .Attr<int64_t>("n_post")
                                  .Attr<bool>("event"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(bsx_ffi_matvec, MatvecImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int64_t>("n_pre")
                                  .Attr<bool>("event"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(bsx_ffi_vecmat_vjp, VjpImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // primal input
                                  .Arg<ffi::AnyBuffer>()   // output cotangent
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()   // dx (empty: not wanted)
                                  .Ret<ffi::AnyBuffer>()   // dw (empty: not wanted)
                                  .Ret<ffi::AnyBuffer>()   // scratch
                                  .Attr<bool>("event"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(bsx_ffi_dense_event_vecmat, DenseEventImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::F32>>()
                                  .Ret<ffi::Buffer<ffi::F32>>());

#endif  // __has_include("xla/ffi/api/ffi.h")
