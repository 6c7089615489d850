// Shared by the translation units of libmps_b200.so; not part of the public ABI.
#pragma once
namespace mps {
// Records a printf-style message for mps_last_error() on this thread and returns `code`.
int fail(int code, const char *fmt, ...);
}  // namespace mps
