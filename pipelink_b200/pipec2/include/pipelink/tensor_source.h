// The handle a tensor export's `produce` callable returns and a generated import adapter unpacks:
// where the exported tensor lives, as one 64-bit word. A provider never publishes its placement
// through the consumer's parameter list; it returns pl::source_of(pointer) for a shared-memory or
// register-frame export and pl::source_of_tmem(address) for a tensor-memory one, and the adapter
// the link generated for the connection reads it according to the export's declared placement
// (the reference's handle of the same name: docs/reference/tensor-imports.md "Callable ABI").
#pragma once
#include <stdint.h>

struct pipelink_tensor_source {
  uint64_t bits;
};

#ifdef __CUDACC__
__device__ __forceinline__ const void* pipelink_source_pointer(pipelink_tensor_source s) {
  return reinterpret_cast<const void*>(s.bits);
}
__device__ __forceinline__ uint32_t pipelink_source_tmem(pipelink_tensor_source s) { return static_cast<uint32_t>(s.bits); }
namespace pl {
__device__ __forceinline__ pipelink_tensor_source source_of(const void* p) {
  return pipelink_tensor_source{reinterpret_cast<uint64_t>(p)};
}
__device__ __forceinline__ pipelink_tensor_source source_of_tmem(uint32_t address) { return pipelink_tensor_source{address}; }
}  // namespace pl
#endif
