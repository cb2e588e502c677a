// Stage hello.provider: a role-less stage that only provides a callable. `hello_scale` runs on the
// threads of whichever role calls it through the call channel `scale` (the reference's provider of
// its first tutorial: docs/reference/annotations.md:60-66, examples/hello-callable/src/provider.cu).
#include "hello.cuh"

extern "C" __device__ float hello_scale(float value);
PL_STAGE("hello.provider", "1.0.0");
PL_NO_PARAMS();
PL_EXPORT(scale, hello_scale);
PL_CALL(scale, hello_scale, pl::consume, "scale");

#ifndef PIPELINK_EMIT
extern "C" __device__ float hello_scale(float value) { return value * 2.0f; }
#endif
