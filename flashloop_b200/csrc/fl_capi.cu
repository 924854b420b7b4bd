// Error reporting shared by all entry points.
#include <cstring>

#include "fl_common.cuh"

namespace fl {

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
}

}  // namespace fl

extern "C" const char* fl_last_error(void) { return fl::g_error; }

extern "C" int fl_version(void) { return 1; }
