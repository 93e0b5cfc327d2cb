// Version and error-text entry points of the C ABI.
#include "common.cuh"

namespace castle {
char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}
}  // namespace castle

extern "C" int castle_abi_version(void) { return CASTLE_ABI_VERSION; }
extern "C" const char* castle_last_error(void) { return castle::last_error_buf(); }
