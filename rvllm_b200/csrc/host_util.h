// Host-side helpers shared by the C-ABI translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// Records a thread-local error message (printf-style) and returns `code`.
int rv_fail(int code, const char* fmt, ...);
// Checks the launch that was just enqueued; returns 0 or RVLLM_E_LAUNCH with the reason recorded.
int rv_launched(const char* what);
inline bool rv_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline uint32_t rv_umin(uint32_t a, uint32_t b) { return a < b ? a : b; }
inline uint32_t rv_umax(uint32_t a, uint32_t b) { return a > b ? a : b; }
