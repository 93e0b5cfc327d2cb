// Version and error-text entry points of the C ABI.
#include "common.cuh"

namespace castle {
char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}
KernelEvents& kernel_events(int which) {
  static KernelEvents ev[3];  // process-wide: torch runs backward passes on its own worker thread
  return ev[which];
}
}  // namespace castle

extern "C" int castle_abi_version(void) { return CASTLE_ABI_VERSION; }
extern "C" const char* castle_last_error(void) { return castle::last_error_buf(); }
extern "C" int castle_set_kernel_events(int32_t which, void* start_event, void* stop_event) {
  if (which < 0 || which > 2) return castle::reject("castle_set_kernel_events: which %d out of range", which);
  castle::kernel_events(which).start = (cudaEvent_t)start_event;
  castle::kernel_events(which).stop = (cudaEvent_t)stop_event;
  return 0;
}
