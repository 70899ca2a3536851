// Host helpers shared by the translation units of the library.
#pragma once

namespace xf {
// printf-style setter of the calling thread's last-error text (read by xf_last_error_string()).
void set_error(const char* fmt, ...);
const char* last_error();
}  // namespace xf
