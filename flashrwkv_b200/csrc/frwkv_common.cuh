// Shared helpers of the frwkv_b200 kernels: error reporting, 16-bit io types, the
// retention transform, small PTX wrappers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "frwkv_b200.h"

namespace frwkv {

// ---- error reporting (thread-local message, negative return codes) -----------------------
void set_error(const char* fmt, ...);
void clear_error();

inline int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  set_error("%s", buf);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    return fail(FRWKV_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
  }
  return FRWKV_OK;
}

#define FRWKV_REQUIRE(cond, ...)                              \
  do {                                                        \
    if (!(cond)) return ::frwkv::fail(FRWKV_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

// true when every pointer (null pointers, i.e. absent optional arguments, aside) is a multiple of 32 bytes: the kernels
// move token rows and state tiles as 16- and 32-byte vectors, and a misaligned one would fault on the device
inline bool aligned32() { return true; }
template <typename... Rest>
inline bool aligned32(const void* p, Rest... rest) {
  return (reinterpret_cast<uintptr_t>(p) & 31u) == 0 && aligned32(rest...);
}

// ---- 16-bit io -----------------------------------------------------------------------------
template <typename T>
struct Io16;

template <>
struct Io16<__half> {
  using pair = __half2;
  static __device__ __forceinline__ float2 unpack(uint32_t bits) {
    return __half22float2(*reinterpret_cast<const __half2*>(&bits));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float load(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ __half store(float x) { return __float2half_rn(x); }
};

template <>
struct Io16<__nv_bfloat16> {
  using pair = __nv_bfloat162;
  // a bf16 is the upper half of the fp32 with the same value: unpack with shifts
  static __device__ __forceinline__ float2 unpack(uint32_t bits) {
    return make_float2(__uint_as_float(bits << 16), __uint_as_float(bits & 0xffff0000u));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ __nv_bfloat16 store(float x) { return __float2bfloat16_rn(x); }
};

// ---- retention transform -------------------------------------------------------------------
// w = exp(-exp(-0.5) * sigmoid(x)), in the reference's exp2 form
// (csrc/sm120/tmix/wkv7/recurrent_decay.cuh:18-22 of the reference).  The hot kernels evaluate it 64 times per
// (token, head), so it is six instructions: ex2.approx (relative error 2^-22), one add, rcp.approx (1 ulp) and two
// multiplies; the result is within 3e-7 relative of the correctly rounded value, far inside every tolerance here.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float retention(float decay_logit) {
  // clamp keeps 1 + 2^(-x log2 e) finite for very negative logits (sigmoid -> 0, w -> 1)
  const float e = ex2_approx(fminf(-1.4426950408889634f * decay_logit, 126.0f));
  return ex2_approx(-0.8750387749145276f * rcp_approx(1.0f + e));
}

// d log(w) / dx = -exp(-0.5) * s * (1 - s), s = sigmoid(x) (recurrent_decay.cuh:27-32).
__device__ __forceinline__ float retention_log_derivative(float decay_logit) {
  const float s = 1.0f / (1.0f + exp2f(-1.4426950408889634f * decay_logit));
  return -0.6065306597126334f * s * (1.0f - s);
}

// fp16-state contract: the rounded retention increment half(w - 1 + dither) of one key channel; the dither is the
// signed 32-bit product phase * 2654435769 scaled by 2^-41 (tests/tmix/wkv7/test.py:249-258 of the reference).
__device__ __forceinline__ float delta_of(float logit, uint32_t phase) {
  const float w = retention(logit);
  const float dither = __int2float_rn((int)(phase * 2654435769u)) * 4.547473508864641e-13f;
  return __half2float(__float2half_rn((w - 1.0f) + dither));
}

__device__ __forceinline__ float quiet_nan() { return __int_as_float(0x7fffffff); }

// ---- programmatic dependent launch -------------------------------------------------------------------------------
// The short kernels of a decode step run back to back in one stream and each is bound by launch latency rather than
// by its work.  A kernel launched with launch_chained() may start while its predecessor is still running; it calls
// chain_begin() first, which lets ITS successor be scheduled early and then waits until everything before it in the
// stream has completed and is visible.  Nothing that a predecessor may write is read, and nothing at all is written,
// before that wait (the projection kernels fetch weights, which are constants, between chain_release() and
// chain_wait()).  Both instructions do nothing in a kernel launched the ordinary way.
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_begin() {
  chain_release();
  chain_wait();
}

bool chained_launch_enabled();  // false when FRWKV_DISABLE_CHAINED_LAUNCH=1 (for comparisons)

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KernelArgs>(args)...);
}

// 32-byte global accesses (sm_100: one request instead of two).  A thread that owns a token row reads or writes a
// run of its own row, so the lanes of a warp touch 32 different lines; the tag lookups, one per line and request,
// are what such accesses cost, and half as many requests cost half as much.  Addresses must be 32-byte aligned.
__device__ __forceinline__ void ldg256(const void* p, uint4& a, uint4& b) {
  asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w), "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
               : "l"(p));
}
__device__ __forceinline__ void stg256(void* p, const uint4& a, const uint4& b) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
               "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}

}  // namespace frwkv
