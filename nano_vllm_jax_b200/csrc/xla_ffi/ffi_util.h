// Helpers shared by the XLA-FFI handlers (api_version 1, the plain C API of xla/ffi/api/c_api.h).
//
// NOT COMPILED BY THE BUILD: the XLA FFI header ships with jaxlib (`jax.ffi.include_dir()`), and JAX is not
// installed where this library is built and measured.  `nano_vllm_jax_b200/kernels/jax_ffi.py` compiles this
// directory into libnvj_b200_xla.so on first use when JAX is present.
//
// The conventions are those of the reference's handlers (nanovllm_jax/kernels/csrc/fp32_kv_append.cu):
//   * answer the metadata-extension probe with the API version and the command-buffer-compatible trait, and
//     return success without touching the operands (:786-799, :1565-1568);
//   * only the execute stage is served (:68-71);
//   * operands and results are XLA_FFI_Buffer; a wrong dtype, rank or dimension is INVALID_ARGUMENT (:17-27, :72-155);
//   * the stream comes from XLA_FFI_Stream_Get (:1575-1583); kernels are launched on it and nothing synchronises;
//   * results that alias an operand (the caches) are written through the RESULT buffers (:1589-1590);
//   * a launch failure is INTERNAL (:1621-1625).
#pragma once

#include <cstdint>
#include <cstring>
#include <string>

#include "xla/ffi/api/c_api.h"

#include "nvj_b200.h"

namespace nvj_xla {

inline XLA_FFI_Error* MakeError(const XLA_FFI_Api* api, XLA_FFI_Error_Code code, const std::string& message) {
  XLA_FFI_Error_Create_Args args;
  args.struct_size = XLA_FFI_Error_Create_Args_STRUCT_SIZE;
  args.extension_start = nullptr;
  args.message = message.c_str();
  args.errc = code;
  return api->XLA_FFI_Error_Create(&args);
}

inline XLA_FFI_Error* Invalid(XLA_FFI_CallFrame* frame, const std::string& message) {
  return MakeError(frame->api, XLA_FFI_Error_Code_INVALID_ARGUMENT, message);
}

// True when the call is the metadata probe: the metadata has been filled in and the handler must return nullptr.
inline bool AnswerMetadataProbe(XLA_FFI_CallFrame* frame) {
  XLA_FFI_Extension_Base* extension = frame->extension_start;
  if (extension == nullptr || extension->type != XLA_FFI_Extension_Metadata) return false;
  XLA_FFI_Metadata* metadata = reinterpret_cast<XLA_FFI_Metadata_Extension*>(extension)->metadata;
  metadata->api_version.major_version = XLA_FFI_API_MAJOR;
  metadata->api_version.minor_version = XLA_FFI_API_MINOR;
  metadata->traits = XLA_FFI_HANDLER_TRAITS_COMMAND_BUFFER_COMPATIBLE;  // no allocation, no sync: capturable
  metadata->state_type_id = XLA_FFI_UNKNOWN_TYPE_ID;
  return true;
}

// Execute stage with exactly `num_args` (or num_args + optional) buffer operands and `num_rets` buffer results.
inline XLA_FFI_Error* CheckFrame(XLA_FFI_CallFrame* frame, const char* name, int64_t num_args, int64_t optional_args,
                                 int64_t num_rets) {
  const std::string n(name);
  if (frame->stage != XLA_FFI_ExecutionStage_EXECUTE) return Invalid(frame, n + " only supports the execute stage");
  if (frame->args.size < num_args || frame->args.size > num_args + optional_args)
    return Invalid(frame, n + ": wrong number of operands");
  if (frame->rets.size != num_rets) return Invalid(frame, n + ": wrong number of results");
  for (int64_t i = 0; i < frame->args.size; ++i)
    if (frame->args.types[i] != XLA_FFI_ArgType_BUFFER) return Invalid(frame, n + ": operands must be buffers");
  for (int64_t i = 0; i < frame->rets.size; ++i)
    if (frame->rets.types[i] != XLA_FFI_RetType_BUFFER) return Invalid(frame, n + ": results must be buffers");
  return nullptr;
}

inline XLA_FFI_Buffer* Arg(XLA_FFI_CallFrame* frame, int64_t i) {
  return i < frame->args.size ? reinterpret_cast<XLA_FFI_Buffer*>(frame->args.args[i]) : nullptr;
}
inline XLA_FFI_Buffer* Ret(XLA_FFI_CallFrame* frame, int64_t i) {
  return reinterpret_cast<XLA_FFI_Buffer*>(frame->rets.rets[i]);
}

inline bool Is(const XLA_FFI_Buffer* b, XLA_FFI_DataType dtype, int64_t rank) {
  return b != nullptr && b->dtype == dtype && b->rank == rank;
}
inline bool IsI32(const XLA_FFI_Buffer* b, int64_t rank) { return Is(b, XLA_FFI_DataType_S32, rank); }

// nvj_dtype of a floating-point buffer, or -1.
inline int FloatDtype(const XLA_FFI_Buffer* b) {
  if (b == nullptr) return -1;
  switch (b->dtype) {
    case XLA_FFI_DataType_BF16: return NVJ_BF16;
    case XLA_FFI_DataType_F16: return NVJ_F16;
    case XLA_FFI_DataType_F32: return NVJ_F32;
    default: return -1;
  }
}

inline int64_t Elements(const XLA_FFI_Buffer* b) {
  int64_t n = 1;
  for (int64_t i = 0; i < b->rank; ++i) n *= b->dims[i];
  return n;
}

inline bool SameShape(const XLA_FFI_Buffer* a, const XLA_FFI_Buffer* b) {
  if (a->rank != b->rank || a->dtype != b->dtype) return false;
  for (int64_t i = 0; i < a->rank; ++i)
    if (a->dims[i] != b->dims[i]) return false;
  return true;
}

// A scalar attribute by name (`jax.ffi.ffi_call(...)(*operands, layer_id=np.int32(3))`); false when absent.
inline bool ScalarAttr(XLA_FFI_CallFrame* frame, const char* name, XLA_FFI_DataType dtype, void* value, size_t bytes) {
  const size_t len = std::strlen(name);
  for (int64_t i = 0; i < frame->attrs.size; ++i) {
    const XLA_FFI_ByteSpan* key = frame->attrs.names[i];
    if (key->len != len || std::memcmp(key->ptr, name, len) != 0) continue;
    if (frame->attrs.types[i] != XLA_FFI_AttrType_SCALAR) return false;
    const XLA_FFI_Scalar* scalar = reinterpret_cast<const XLA_FFI_Scalar*>(frame->attrs.attrs[i]);
    if (scalar->dtype != dtype) return false;
    std::memcpy(value, scalar->value, bytes);
    return true;
  }
  return false;
}
inline bool IntAttr(XLA_FFI_CallFrame* frame, const char* name, int32_t* value) {
  return ScalarAttr(frame, name, XLA_FFI_DataType_S32, value, sizeof(int32_t));
}
inline bool FloatAttr(XLA_FFI_CallFrame* frame, const char* name, float* value) {
  return ScalarAttr(frame, name, XLA_FFI_DataType_F32, value, sizeof(float));
}

inline XLA_FFI_Error* GetStream(XLA_FFI_CallFrame* frame, nvj_stream_t* stream) {
  XLA_FFI_Stream_Get_Args args;
  args.struct_size = XLA_FFI_Stream_Get_Args_STRUCT_SIZE;
  args.extension_start = nullptr;
  args.ctx = frame->ctx;
  args.stream = nullptr;
  if (XLA_FFI_Error* error = frame->api->XLA_FFI_Stream_Get(&args)) return error;
  *stream = args.stream;
  return nullptr;
}

// nvj status -> XLA error (nullptr for NVJ_OK).
inline XLA_FFI_Error* FromStatus(XLA_FFI_CallFrame* frame, const char* name, int status) {
  if (status == NVJ_OK) return nullptr;
  const XLA_FFI_Error_Code code = status == NVJ_ERR_LAUNCH ? XLA_FFI_Error_Code_INTERNAL
                                  : status == NVJ_ERR_UNSUPPORTED ? XLA_FFI_Error_Code_UNIMPLEMENTED
                                                                  : XLA_FFI_Error_Code_INVALID_ARGUMENT;
  return MakeError(frame->api, code, std::string(name) + ": " + nvj_status_string(status));
}

}  // namespace nvj_xla

// Common opening of every handler: probe, frame check, stream.
#define NVJ_XLA_PROLOGUE(NAME, NUM_ARGS, OPTIONAL_ARGS, NUM_RETS)                                          \
  if (nvj_xla::AnswerMetadataProbe(frame)) return nullptr;                                                 \
  if (frame->extension_start != nullptr) return nullptr;                                                   \
  if (XLA_FFI_Error* error = nvj_xla::CheckFrame(frame, NAME, NUM_ARGS, OPTIONAL_ARGS, NUM_RETS)) return error; \
  nvj_stream_t stream = nullptr;                                                                           \
  if (XLA_FFI_Error* error = nvj_xla::GetStream(frame, &stream)) return error
