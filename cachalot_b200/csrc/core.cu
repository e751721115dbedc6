// Library-wide state: the per-thread error message and the version.
#include "common.cuh"

namespace cachalot {
static thread_local char g_error[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof g_error, fmt, ap);
  va_end(ap);
}
}  // namespace cachalot

extern "C" const char* cachalot_last_error(void) { return cachalot::g_error; }
// 2: cachalot_group_rows takes cachalot_group_rows_scratch_ints() of scratch; rows-level prefill, combine and peer sum added
extern "C" int cachalot_version(void) { return 2; }
