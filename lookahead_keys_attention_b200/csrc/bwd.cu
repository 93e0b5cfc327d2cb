#include "common.cuh"
using namespace castle;
extern "C" size_t castle_bwd_workspace_bytes(const castle_problem_t*) { return 0; }
extern "C" int castle_bwd(const castle_problem_t*, const castle_tensor_t*, const castle_tensor_t*, const castle_tensor_t*,
                          const castle_tensor_t*, const castle_tensor_t*, const castle_tensor_t*, const castle_tensor_t*,
                          const castle_tensor_t*, const float*, const float*, const castle_tensor_t*,
                          const castle_tensor_t*, const castle_tensor_t*, const castle_tensor_t*, const castle_tensor_t*,
                          const castle_tensor_t*, void*, size_t, int32_t*, void*) {
  return reject("castle_bwd: not built");
}
