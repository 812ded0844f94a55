// Shared by the translation units of the library; not part of the public ABI.
#pragma once

namespace ckl {

// Records `fmt` as the calling thread's last error (what ckl_last_error() returns) and
// returns `code`, so a failing path can `return set_error(CKL_ERR_..., "...", ...)`.
int set_error(int code, const char* fmt, ...);

}  // namespace ckl
