// Shared host-side helpers of the C ABI (error reporting).
#pragma once
#include <cstddef>

namespace ph {

// Records a printf-style message as the calling thread's last error and
// returns `code`, so call sites can write `return fail(PH_ERR_..., "...")`.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();
const char* last_error();

// Bytes of the rounded f16 copies of f32-stored A [M,K] and B [K,N] (each padded to 256 bytes).
size_t gemm_staging_bytes(long long M, long long N, long long K);

unsigned long long lcg_skip_host(unsigned long long s, unsigned long long n);

}  // namespace ph
