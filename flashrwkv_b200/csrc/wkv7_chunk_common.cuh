// Helpers shared by the chunked WKV7 kernels (fused forward / adjoint scan, chunk-parallel backward): access to
// chunk-major operand tiles, the warp-uniform bounded wait and 16-bit unpacking.
#pragma once

#include "frwkv_common.cuh"
#include "umma.cuh"

namespace frwkv {
namespace chunk {

__device__ __forceinline__ float4 ld4(const unsigned char* base, uint32_t off) {
  return *reinterpret_cast<const float4*>(base + off);
}
__device__ __forceinline__ float ld1(const unsigned char* base, uint32_t off) {
  return *reinterpret_cast<const float*>(base + off);
}
__device__ __forceinline__ void st4(unsigned char* base, uint32_t off, float4 v) {
  *reinterpret_cast<float4*>(base + off) = v;
}
__device__ __forceinline__ void st1(unsigned char* base, uint32_t off, float v) {
  *reinterpret_cast<float*>(base + off) = v;
}
__device__ __forceinline__ uint32_t tile_off(uint32_t cs, int row, int col) {
  return uint32_t(col >> 2) * cs + uint32_t(row) * 16 + uint32_t(col & 3) * 4;
}
__device__ __forceinline__ uint32_t tf32_bits(float x) { return __float_as_uint(umma::to_tf32(x)); }

// Bounded wait with one answer per warp: the tensor-memory loads and stores that follow are warp-collective, so a
// warp either does its epilogue as a whole or skips it as a whole.  Once a wait has run out no later one is tried.
__device__ __forceinline__ bool wait_warp(uint64_t* mbar, uint32_t parity, bool ok) {
  if (ok) ok = umma::mbar_wait_suspended(mbar, parity);
  return __all_sync(0xffffffffu, ok) != 0;
}

template <typename io_t>
__device__ __forceinline__ void unpack8(uint4 u, float (&f)[8]) {
  using IO = Io16<io_t>;
  float2 p;
  p = IO::unpack(u.x); f[0] = p.x; f[1] = p.y;
  p = IO::unpack(u.y); f[2] = p.x; f[3] = p.y;
  p = IO::unpack(u.z); f[4] = p.x; f[5] = p.y;
  p = IO::unpack(u.w); f[6] = p.x; f[7] = p.y;
}

}  // namespace chunk
}  // namespace frwkv
