// Status plumbing of the C ABI: per-thread error text and the version query.
#include "common.cuh"

namespace b200lut {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace b200lut

extern "C" int b200lut_version(void) { return 100; }

extern "C" const char* b200lut_last_error(void) { return b200lut::error_buffer(); }
