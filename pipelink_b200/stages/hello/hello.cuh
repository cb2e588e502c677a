// Shared by the two hello stages: the caller's params block (the kernel parameter bytes of the
// linked image) and nothing else; the provider has no params and no role.
#pragma once
#include <stdint.h>
#include <pipelink/stage.hpp>

struct HelloCallerParams {
  const float* input;
  float* output;
  long long count;
};
