// What ingest.cc needs from the rest of the library (error text), so that the file can be built
// on its own with -fsanitize=address,undefined for tests/test_ingest_cpu.py.
#include "common.h"

namespace gearb {
std::string &last_error() {
  static thread_local std::string text;
  return text;
}
int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  last_error() = buf;
  return code;
}
}  // namespace gearb

extern "C" const char *gearb_last_error(void) { return gearb::last_error().c_str(); }
