// XLA FFI handlers that put the C ABI of libsc_b200.so behind the reference's JAX primitives on the
// CUDA platform.
//
// NOT PART OF THE DEFAULT BUILD.  The XLA FFI headers (xla/ffi/api/ffi.h, shipped inside jaxlib)
// are not available where this library is developed, so this file has never been compiled; it is
// kept as the exact binding a maintainer adds once jaxlib is present:
//
//   g++ -std=c++17 -O2 -fPIC -shared -DSC_HAVE_XLA_FFI -I$(python -c "import jax.ffi; print(jax.ffi.include_dir())")
//       -I include -I /usr/local/cuda/include sc_xla_ffi.cc -L. -lsc_b200 -lcudart -o libsc_b200_ffi.so
//
// and in Python (replacing the MLIR lowerings to the libtpu custom calls "SparseDenseMatmulOp" and
// "SparseDenseMatmulGradOpWithOptimizerUpdate" of
// jax_tpu_embedding/sparsecore/lib/core/primitives/sparse_dense_matmul_csr.py:114-207,
// sparse_dense_matmul_grad_with_sgd.py:98-238, ..._adagrad.py:119-292, ..._adam.py:144-405):
//
//   lib = ctypes.CDLL("libsc_b200_ffi.so")
//   for name in ("sc_b200_fwd", "sc_b200_grad_sgd", "sc_b200_grad_adagrad", "sc_b200_grad_adam"):
//     jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(lib, name)), platform="CUDA")
//   # forward:  jax.ffi.ffi_call("sc_b200_fwd", jax.ShapeDtypeStruct((device_batch_size, dim), jnp.float32))(
//   #               row_pointers, embedding_ids, sample_ids, gains, table, device_batch_size=..., num_sc_per_device=...)
//   # backward: jax.ffi.ffi_call("sc_b200_grad_adagrad", (table_type, accumulator_type),
//   #               input_output_aliases={4: 0, 5: 1})(row_pointers, embedding_ids, sample_ids, gains, table,
//   #               accumulator, activations_grad, learning_rate, num_sc_per_device=..., clip_min=..., clip_max=...)
//
// The gradient handlers update the table and the slot variables in place.  With the aliases above XLA
// hands the operand buffers over as result buffers; without them the handlers first copy operand to
// result.  The update body that the TPU custom call receives as a called computation
// (sparse_dense_matmul_grad_with_adagrad.py:266-275) has no counterpart: the optimizer is chosen by the
// handler and its hyper-parameters travel as scalar operands.
//
// Scope: all shards of the stacked table are addressable from the calling device, i.e. the operands
// carry [num_scs * rows_per_shard, dim] tables (one GPU, or "virtual devices").  Row-sharded tables over
// several processes use peer-mapped shard pointers (sc_fwd_item_t.local_shard, sc_grad_item_t.sources),
// which XLA buffers cannot express; that path stays behind the Python operators.
#ifdef SC_HAVE_XLA_FFI

#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <limits>
#include <string>

#include "sc_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error status_to_error(int32_t status) {
  if (status == SC_OK) return ffi::Error::Success();
  char message[512];
  sc_last_error(message, sizeof message);
  const ffi::ErrorCode code = (status == SC_INVALID_ARGUMENT || status == SC_ID_LIMIT_EXCEEDED)
                                  ? ffi::ErrorCode::kInvalidArgument
                                  : (status == SC_UNSUPPORTED ? ffi::ErrorCode::kUnimplemented : ffi::ErrorCode::kInternal);
  return ffi::Error(code, std::string(sc_status_name(status)) + ": " + message);
}

// Geometry of one call from the operand shapes and the two topology attributes, as the Python
// operators derive it (lib/core/primitives/_ops.py, class Geometry).
ffi::Error make_csr(const ffi::Buffer<ffi::S32>& row_pointers, const ffi::Buffer<ffi::S32>& ids,
                    const ffi::Buffer<ffi::S32>& sample_ids, const ffi::Buffer<ffi::F32>& gains,
                    const ffi::Buffer<ffi::F32>& table, int64_t device_batch_size, int64_t num_sc_per_device,
                    int64_t global_device_count, sc_csr_t* csr) {
  const int64_t num_scs = num_sc_per_device * global_device_count;
  if (num_sc_per_device <= 0 || global_device_count <= 0 || num_scs > SC_MAX_SHARDS)
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "bad num_sc_per_device / global_device_count");
  const auto dims = table.dimensions();
  if (dims.size() != 2 || dims[0] % num_scs != 0)
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "embedding_table must be [num_scs * rows_per_shard, dim]");
  csr->row_pointers = row_pointers.typed_data();
  csr->embedding_ids = ids.typed_data();
  csr->sample_ids = sample_ids.typed_data();
  csr->gains = gains.typed_data();
  csr->coo_buffer_size = static_cast<int32_t>(ids.element_count());
  csr->num_sc_per_device = static_cast<int32_t>(num_sc_per_device * global_device_count);  // all devices' slices are local
  csr->num_scs = static_cast<int32_t>(num_scs);
  csr->device_batch_size = static_cast<int32_t>(device_batch_size * global_device_count);
  csr->dim = static_cast<int32_t>(dims[1]);
  csr->max_ids_per_sample = 0;
  csr->rows_per_shard = dims[0] / num_scs;
  return ffi::Error::Success();
}

void shard_pointers(float* base, const sc_csr_t& csr, float** out) {
  for (int g = 0; g < csr.num_scs; ++g) out[g] = base + static_cast<int64_t>(g) * csr.rows_per_shard * csr.dim;
}

ffi::Error FwdImpl(cudaStream_t stream, ffi::ScratchAllocator scratch, ffi::Buffer<ffi::S32> row_pointers,
                   ffi::Buffer<ffi::S32> ids, ffi::Buffer<ffi::S32> sample_ids, ffi::Buffer<ffi::F32> gains,
                   ffi::Buffer<ffi::F32> table, ffi::ResultBuffer<ffi::F32> activations, int64_t device_batch_size,
                   int64_t num_sc_per_device, int64_t global_device_count) {
  sc_csr_t csr;
  if (ffi::Error e = make_csr(row_pointers, ids, sample_ids, gains, table, device_batch_size, num_sc_per_device,
                              global_device_count, &csr); e.failure())
    return e;
  float* shards[SC_MAX_SHARDS];
  shard_pointers(table.typed_data(), csr, shards);
  const size_t bytes = sc_sparse_dense_matmul_fwd_workspace_bytes(&csr);
  auto workspace = scratch.Allocate(bytes);
  if (!workspace.has_value()) return ffi::Error(ffi::ErrorCode::kResourceExhausted, "no scratch memory for the lookup");
  return status_to_error(sc_sparse_dense_matmul_fwd(&csr, shards, activations->typed_data(), *workspace, bytes, stream));
}

// Common part of the gradient handlers.  `tables[k]` / `results[k]`: table, slot 0, slot 1.
ffi::Error GradCommon(cudaStream_t stream, ffi::ScratchAllocator& scratch, const sc_csr_t& csr, const float* activation_grad,
                      int optimizer, const float* hyper, int num_hyper, float clip_min, float clip_max, int num_arrays,
                      const ffi::Buffer<ffi::F32>* const* operands, ffi::Result<ffi::Buffer<ffi::F32>>* const* results) {
  float* shards[3][SC_MAX_SHARDS];
  for (int k = 0; k < num_arrays; ++k) {
    float* dst = (*results[k])->typed_data();
    const float* src = operands[k]->typed_data();
    if (dst != src) {  // the call was made without input_output_aliases: update a copy
      if (cudaMemcpyAsync(dst, src, operands[k]->size_bytes(), cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
        return ffi::Error(ffi::ErrorCode::kInternal, "copy of an embedding variable failed");
    }
    shard_pointers(dst, csr, shards[k]);
  }
  sc_optimizer_t opt;
  opt.optimizer = optimizer;
  for (int i = 0; i < 8; ++i) opt.hyper[i] = i < num_hyper ? hyper[i] : 0.0f;
  opt.clip_min = clip_min;
  opt.clip_max = clip_max;
  const size_t bytes = sc_sparse_dense_matmul_grad_workspace_bytes(&csr);
  auto workspace = scratch.Allocate(bytes);
  if (!workspace.has_value()) return ffi::Error(ffi::ErrorCode::kResourceExhausted, "no scratch memory for the update");
  return status_to_error(sc_sparse_dense_matmul_grad(&csr, activation_grad, shards[0], num_arrays > 1 ? shards[1] : nullptr,
                                                     num_arrays > 2 ? shards[2] : nullptr, &opt, *workspace, bytes, stream));
}

// Scalar hyper-parameters are device operands in the reference's primitives (learning_rate is a traced
// value); the handlers read them with one small copy on the call's stream.
ffi::Error read_scalars(cudaStream_t stream, const ffi::Buffer<ffi::F32>* const* scalars, int count, float* out) {
  for (int i = 0; i < count; ++i)
    if (cudaMemcpyAsync(out + i, scalars[i]->typed_data(), sizeof(float), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
      return ffi::Error(ffi::ErrorCode::kInternal, "reading a hyper-parameter failed");
  if (cudaStreamSynchronize(stream) != cudaSuccess) return ffi::Error(ffi::ErrorCode::kInternal, "stream synchronisation failed");
  return ffi::Error::Success();
}

float bound_or_nan(float v, bool set) { return set ? v : std::numeric_limits<float>::quiet_NaN(); }

#define SC_FFI_CSR_ARGS                                                                                     \
  ffi::Buffer<ffi::S32> row_pointers, ffi::Buffer<ffi::S32> ids, ffi::Buffer<ffi::S32> sample_ids,          \
      ffi::Buffer<ffi::F32> gains

ffi::Error GradSgdImpl(cudaStream_t stream, ffi::ScratchAllocator scratch, SC_FFI_CSR_ARGS, ffi::Buffer<ffi::F32> table,
                       ffi::Buffer<ffi::F32> activation_grad, ffi::Buffer<ffi::F32> learning_rate,
                       ffi::ResultBuffer<ffi::F32> table_out, int64_t num_sc_per_device, int64_t global_device_count,
                       float clip_min, float clip_max, bool has_clip_min, bool has_clip_max) {
  sc_csr_t csr;
  const int64_t batch = activation_grad.dimensions()[0] / global_device_count;
  if (ffi::Error e = make_csr(row_pointers, ids, sample_ids, gains, table, batch, num_sc_per_device, global_device_count, &csr);
      e.failure())
    return e;
  float hyper[1];
  const ffi::Buffer<ffi::F32>* scalars[] = {&learning_rate};
  if (ffi::Error e = read_scalars(stream, scalars, 1, hyper); e.failure()) return e;
  const ffi::Buffer<ffi::F32>* operands[] = {&table};
  ffi::Result<ffi::Buffer<ffi::F32>>* results[] = {&table_out};
  return GradCommon(stream, scratch, csr, activation_grad.typed_data(), SC_OPT_SGD, hyper, 1, bound_or_nan(clip_min, has_clip_min),
                    bound_or_nan(clip_max, has_clip_max), 1, operands, results);
}

ffi::Error GradAdagradImpl(cudaStream_t stream, ffi::ScratchAllocator scratch, SC_FFI_CSR_ARGS, ffi::Buffer<ffi::F32> table,
                           ffi::Buffer<ffi::F32> accumulator, ffi::Buffer<ffi::F32> activation_grad,
                           ffi::Buffer<ffi::F32> learning_rate, ffi::ResultBuffer<ffi::F32> table_out,
                           ffi::ResultBuffer<ffi::F32> accumulator_out, int64_t num_sc_per_device,
                           int64_t global_device_count, float clip_min, float clip_max, bool has_clip_min,
                           bool has_clip_max) {
  sc_csr_t csr;
  const int64_t batch = activation_grad.dimensions()[0] / global_device_count;
  if (ffi::Error e = make_csr(row_pointers, ids, sample_ids, gains, table, batch, num_sc_per_device, global_device_count, &csr);
      e.failure())
    return e;
  float hyper[1];
  const ffi::Buffer<ffi::F32>* scalars[] = {&learning_rate};
  if (ffi::Error e = read_scalars(stream, scalars, 1, hyper); e.failure()) return e;
  const ffi::Buffer<ffi::F32>* operands[] = {&table, &accumulator};
  ffi::Result<ffi::Buffer<ffi::F32>>* results[] = {&table_out, &accumulator_out};
  return GradCommon(stream, scratch, csr, activation_grad.typed_data(), SC_OPT_ADAGRAD, hyper, 1,
                    bound_or_nan(clip_min, has_clip_min), bound_or_nan(clip_max, has_clip_max), 2, operands, results);
}

// Operand order of the reference's Adam primitive: ..., table, momentum, velocity, activations_grad, alpha_t, beta_1,
// beta_2, epsilon_hat (sparse_dense_matmul_grad_with_adam.py:41-75).
ffi::Error GradAdamImpl(cudaStream_t stream, ffi::ScratchAllocator scratch, SC_FFI_CSR_ARGS, ffi::Buffer<ffi::F32> table,
                        ffi::Buffer<ffi::F32> momentum, ffi::Buffer<ffi::F32> velocity, ffi::Buffer<ffi::F32> activation_grad,
                        ffi::Buffer<ffi::F32> alpha_t, ffi::Buffer<ffi::F32> beta_1, ffi::Buffer<ffi::F32> beta_2,
                        ffi::Buffer<ffi::F32> epsilon_hat, ffi::ResultBuffer<ffi::F32> table_out,
                        ffi::ResultBuffer<ffi::F32> momentum_out, ffi::ResultBuffer<ffi::F32> velocity_out,
                        int64_t num_sc_per_device, int64_t global_device_count, float clip_min, float clip_max,
                        bool has_clip_min, bool has_clip_max) {
  sc_csr_t csr;
  const int64_t batch = activation_grad.dimensions()[0] / global_device_count;
  if (ffi::Error e = make_csr(row_pointers, ids, sample_ids, gains, table, batch, num_sc_per_device, global_device_count, &csr);
      e.failure())
    return e;
  float hyper[4];
  const ffi::Buffer<ffi::F32>* scalars[] = {&alpha_t, &beta_1, &beta_2, &epsilon_hat};
  if (ffi::Error e = read_scalars(stream, scalars, 4, hyper); e.failure()) return e;
  const ffi::Buffer<ffi::F32>* operands[] = {&table, &momentum, &velocity};
  ffi::Result<ffi::Buffer<ffi::F32>>* results[] = {&table_out, &momentum_out, &velocity_out};
  return GradCommon(stream, scratch, csr, activation_grad.typed_data(), SC_OPT_ADAM, hyper, 4,
                    bound_or_nan(clip_min, has_clip_min), bound_or_nan(clip_max, has_clip_max), 3, operands, results);
}

#define SC_FFI_BIND_CSR()                    \
  ffi::Ffi::Bind()                           \
      .Ctx<ffi::PlatformStream<cudaStream_t>>() \
      .Ctx<ffi::ScratchAllocator>()          \
      .Arg<ffi::Buffer<ffi::S32>>()          \
      .Arg<ffi::Buffer<ffi::S32>>()          \
      .Arg<ffi::Buffer<ffi::S32>>()          \
      .Arg<ffi::Buffer<ffi::F32>>()

#define SC_FFI_GRAD_ATTRS()                        \
  .Attr<int64_t>("num_sc_per_device")              \
      .Attr<int64_t>("global_device_count")        \
      .Attr<float>("clip_min")                     \
      .Attr<float>("clip_max")                     \
      .Attr<bool>("has_clip_min")                  \
      .Attr<bool>("has_clip_max")

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(sc_b200_fwd, FwdImpl,
                              SC_FFI_BIND_CSR()
                                  .Arg<ffi::Buffer<ffi::F32>>()   // embedding_table
                                  .Ret<ffi::Buffer<ffi::F32>>()   // activations
                                  .Attr<int64_t>("device_batch_size")
                                  .Attr<int64_t>("num_sc_per_device")
                                  .Attr<int64_t>("global_device_count"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(sc_b200_grad_sgd, GradSgdImpl,
                              SC_FFI_BIND_CSR()
                                  .Arg<ffi::Buffer<ffi::F32>>()   // 4: embedding_table   -> result 0
                                  .Arg<ffi::Buffer<ffi::F32>>()   // activations_grad
                                  .Arg<ffi::Buffer<ffi::F32>>()   // learning_rate
                                  .Ret<ffi::Buffer<ffi::F32>>() SC_FFI_GRAD_ATTRS());

XLA_FFI_DEFINE_HANDLER_SYMBOL(sc_b200_grad_adagrad, GradAdagradImpl,
                              SC_FFI_BIND_CSR()
                                  .Arg<ffi::Buffer<ffi::F32>>()   // 4: embedding_table   -> result 0
                                  .Arg<ffi::Buffer<ffi::F32>>()   // 5: accumulator       -> result 1
                                  .Arg<ffi::Buffer<ffi::F32>>()   // activations_grad
                                  .Arg<ffi::Buffer<ffi::F32>>()   // learning_rate
                                  .Ret<ffi::Buffer<ffi::F32>>()
                                  .Ret<ffi::Buffer<ffi::F32>>() SC_FFI_GRAD_ATTRS());

XLA_FFI_DEFINE_HANDLER_SYMBOL(sc_b200_grad_adam, GradAdamImpl,
                              SC_FFI_BIND_CSR()
                                  .Arg<ffi::Buffer<ffi::F32>>()   // 4: embedding_table   -> result 0
                                  .Arg<ffi::Buffer<ffi::F32>>()   // 5: momentum          -> result 1
                                  .Arg<ffi::Buffer<ffi::F32>>()   // 6: velocity          -> result 2
                                  .Arg<ffi::Buffer<ffi::F32>>()   // activations_grad
                                  .Arg<ffi::Buffer<ffi::F32>>()   // alpha_t
                                  .Arg<ffi::Buffer<ffi::F32>>()   // beta_1
                                  .Arg<ffi::Buffer<ffi::F32>>()   // beta_2
                                  .Arg<ffi::Buffer<ffi::F32>>()   // epsilon_hat
                                  .Ret<ffi::Buffer<ffi::F32>>()
                                  .Ret<ffi::Buffer<ffi::F32>>()
                                  .Ret<ffi::Buffer<ffi::F32>>() SC_FFI_GRAD_ATTRS());

#endif  // SC_HAVE_XLA_FFI
