// Shared host-side helpers of the C ABI (error reporting).
#pragma once

namespace ph {

// Records a printf-style message as the calling thread's last error and
// returns `code`, so call sites can write `return fail(PH_ERR_..., "...")`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();
const char* last_error();

unsigned long long lcg_skip_host(unsigned long long s, unsigned long long n);

}  // namespace ph
