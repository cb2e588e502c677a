// Stage hello.caller: one four-warp role owns a grid-stride loop and calls through the trampoline
// of the call channel `scale`; the link generates the trampoline's body from the two declarations
// (the reference's caller: docs/reference/annotations.md:68-74, examples/hello-callable/src/caller.cu).
#include "hello.cuh"

extern "C" __device__ float pipelink_call_scale(float value);
extern "C" __device__ void hello_call(const void* params, unsigned variant);
PL_STAGE("hello.caller", "1.0.0");
PL_PARAMS(HelloCallerParams, input, output, count);
PL_ROLE(call, hello_call, 4);
PL_CALL(scale, pipelink_call_scale, pl::produce, "call");

#ifndef PIPELINK_EMIT
extern "C" __device__ void hello_call(const void* raw_params, unsigned) {
  const HelloCallerParams& p = *static_cast<const HelloCallerParams*>(raw_params);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.count; i += stride)
    p.output[i] = pipelink_call_scale(p.input[i]);
}
#endif
