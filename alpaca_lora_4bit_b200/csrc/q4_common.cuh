// Shared device helpers and host-side error plumbing for the q4b200 kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/q4b200.h"

namespace q4 {

// ---- host-side error reporting -------------------------------------------------------------
// Thread-local message returned by q4_last_error_string().
char* err_buf();
int fail(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
// 0 if the current device is sm_100, else Q4_E_DEVICE (cached per device).
int check_device();
// Number of SMs of the current device (cached).
int sm_count();

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- device helpers --------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }

// SiLU as every kernel of the library computes it (the fused gate_up epilogue and the element-wise SwiGLU kernel
// must agree to the bit).
// Approximate reciprocal and exponential (2 ulp each): the result is rounded to fp16 right away, and an IEEE
// division costs more instructions than the rest of an epilogue's work per element.
__device__ __forceinline__ float silu_f(float v) { return __fdividef(v, 1.f + __expf(-v)); }

// Streaming 128-bit load that does not allocate in L1 (weights are read exactly once).
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// (a & mask) | bits as ONE three-input logic instruction.  Written in C++ with two literal constants
// the expression compiles to two instructions (the instruction has room for a single immediate);
// here both constants are register operands, loaded once outside the loops that use them.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t bits) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(bits));
  return d;
}

// 128-bit read-only load that the compiler may not move: used where a load is issued early on
// purpose (a prefetch) and must not sink down to its first use.
__device__ __forceinline__ int4 ldg_pinned_int4(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Two exact small integers as a half2, taken from the same byte lane of two packed words.
//   byte b (0..3) of `lo` and of `hi` each hold two 4-bit levels; `odd` selects the high nibble.
// The byte pair is gathered with one PRMT; the low nibble is turned into 1024+q by OR-ing the
// fp16 exponent 0x6400 and removed with an exact subtraction; the high nibble gives 1024+16q,
// brought back with one exact fused multiply-add by 1/16 (constants only, no data-dependent
// rounding).  Result: (q(lo), q(hi)) as exact fp16 integers in 0..15.
template <int BYTE, bool ODD>
__device__ __forceinline__ __half2 nibble_pair(uint32_t lo, uint32_t hi) {
  // selector nibble i picks output byte i (0-3 from `lo`, 4-7 from `hi`); bytes 1 and 3 are
  // masked away below, so only output bytes 0 and 2 matter.
  constexpr uint32_t sel = BYTE | ((BYTE + 4) << 8);
  uint32_t u = prmt(lo, hi, sel);
  if (!ODD) {
    uint32_t v = and_or(u, 0x000F000Fu, 0x64006400u);
    return __hsub2(as_h2(v), as_h2(0x64006400u));
  } else {
    uint32_t v = and_or(u, 0x00F000F0u, 0x64006400u);
    return __hfma2(as_h2(v), as_h2(0x2C002C00u) /* 1/16 */, as_h2(0xD400D400u) /* -64 */);
  }
}

#endif  // __CUDACC__

}  // namespace q4
