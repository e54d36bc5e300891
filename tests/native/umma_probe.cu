// Test-only probes of the sm_100a tensor-core path (built into tests/native/libfrwkv_probe.so, never into the
// product library).  Each entry point runs one small kernel through the same inline-PTX helpers and tile formats
// that the WKV7 chunk kernels use (csrc/umma.cuh), so that a descriptor encoding, a tensor-memory layout or the
// bounded-wait give-up path can be checked against a host computation in isolation.
//
// Return value of every entry point: 0, a positive cudaError_t, or -4 when a bounded wait ran out.
#include <cuda_runtime.h>

#include <cstdint>

#include "umma.cuh"

namespace {

using namespace frwkv;

constexpr int kM = 128;
constexpr int kK = 64;

__device__ __forceinline__ void put_tile(unsigned char* tile, int chunk_stride, int row, int col, float x) {
  *reinterpret_cast<float*>(tile + (col >> 2) * chunk_stride + row * 16 + (col & 3) * 4) = umma::to_tf32(x);
}

// D[m][n] = sum_k A[m][k] * B[n][k]; A is [128][64], B is [N][64], D is [128][N] (row-major, global).
// a_in_tmem == 0: A staged in shared memory as a chunk-major tile.
// a_in_tmem == 1: A written to tensor memory with tcgen05.st (thread = row) and read from there by the MMA.
__global__ __launch_bounds__(128, 1) void umma_probe_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                            float* __restrict__ Dout, int N, int a_chunk_stride,
                                                            int b_chunk_stride, int a_in_tmem,
                                                            int* __restrict__ error_flag) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t mbar;
  __shared__ uint32_t tmem_base_holder;
  unsigned char* a_tile = smem;
  unsigned char* b_tile = smem + 65536;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;

  if (!a_in_tmem)
    for (int e = tid; e < kM * kK; e += 128) put_tile(a_tile, a_chunk_stride, e / kK, e % kK, A[e]);
  for (int e = tid; e < N * kK; e += 128) put_tile(b_tile, b_chunk_stride, e / kK, e % kK, B[e]);
  if (tid == 0) {
    umma::mbar_init(&mbar, 1);
    umma::mbar_fence_init();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_base_holder, 256);
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_base_holder;
  const uint32_t lane_base = uint32_t(warp * 32) << 16;
  const uint32_t a_tmem = tmem + 128;  // columns 128..191 hold A when a_in_tmem

  if (a_in_tmem) {
    for (int c0 = 0; c0 < kK; c0 += 32) {
      uint32_t v[32];
      for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(umma::to_tf32(A[tid * kK + c0 + j]));
      umma::tmem_st32(a_tmem + lane_base + c0, v);
    }
    umma::tmem_st_wait();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
  }

  if (tid == 0) {
    const uint32_t idesc = umma::idesc_tf32(kM, N);
    const uint32_t a_addr = umma::smem_u32(a_tile), b_addr = umma::smem_u32(b_tile);
    for (int ks = 0; ks < kK / 8; ++ks) {
      const uint64_t bdesc = umma::desc_k_major(b_addr + ks * umma::kstep_k_major(b_chunk_stride), b_chunk_stride);
      if (a_in_tmem)
        umma::mma_tf32_ts(tmem, a_tmem + 8 * ks, bdesc, idesc, ks > 0 ? 1u : 0u);
      else
        umma::mma_tf32_ss(tmem, umma::desc_k_major(a_addr + ks * umma::kstep_k_major(a_chunk_stride), a_chunk_stride),
                          bdesc, idesc, ks > 0 ? 1u : 0u);
    }
    umma::mma_commit(&mbar);
  }
  const bool ok = umma::mbar_wait(&mbar, 0);
  umma::fence_after_sync();
  if (!ok) {
    if (tid == 0) atomicExch(error_flag, 1);
  } else {
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t v[32];
      umma::tmem_ld32(tmem + lane_base + c0, v);
      umma::tmem_ld_wait();
      for (int j = 0; j < 32; ++j) Dout[tid * N + c0 + j] = __uint_as_float(v[j]);
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, 256);
}

// Every thread writes 32 words to its tensor-memory lane, reads them back doubled (load, modify, store in
// place, load again): pins the register <-> tensor-memory path used for operands that stay in tensor memory.
__global__ __launch_bounds__(128, 1) void tmem_roundtrip_kernel(const uint32_t* __restrict__ in,
                                                                uint32_t* __restrict__ out) {
  __shared__ uint32_t tmem_base_holder;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (warp == 0) umma::tmem_alloc(&tmem_base_holder, 64);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_base_holder;
  const uint32_t addr = tmem + (uint32_t(warp * 32) << 16) + 32;  // columns 32..63 of this thread's lane
  uint32_t v[32];
  for (int j = 0; j < 32; ++j) v[j] = in[tid * 32 + j];
  umma::tmem_st32(addr, v);
  umma::tmem_st_wait();
  uint32_t u[32];
  umma::tmem_ld32(addr, u);
  umma::tmem_ld_wait();
  for (int j = 0; j < 32; ++j) u[j] = 2 * u[j];
  umma::tmem_st32(addr, u);
  umma::tmem_st_wait();
  umma::tmem_ld32(addr, v);
  umma::tmem_ld_wait();
  for (int j = 0; j < 32; ++j) out[tid * 32 + j] = v[j];
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, 64);
}

// A wait on a barrier at which nothing ever arrives: the bounded wait must give up after `limit` polls, the
// kernel records that and returns normally.
__global__ void bounded_wait_kernel(uint32_t limit, int* __restrict__ flag, unsigned long long* __restrict__ polls) {
  __shared__ uint64_t mbar;
  if (threadIdx.x == 0) {
    umma::mbar_init(&mbar, 1);
    umma::mbar_fence_init();
  }
  __syncthreads();
  const long long t0 = clock64();
  const bool ok = umma::mbar_wait(&mbar, 0, limit);
  const long long t1 = clock64();
  const int all_ok = __syncthreads_and(ok ? 1 : 0);
  if (threadIdx.x == 0) {
    *flag = all_ok ? 0 : 1;
    *polls = (unsigned long long)(t1 - t0);
  }
}

}  // namespace

extern "C" int frwkv_probe_umma(const float* a, const float* b, float* d, int n, int a_chunk_stride,
                                int b_chunk_stride, int a_in_tmem, int32_t* error_flag, cudaStream_t stream) {
  if (!a || !b || !d || !error_flag || (n != 64 && n != 128)) return (int)cudaErrorInvalidValue;
  if (a_chunk_stride % 16 != 0 || a_chunk_stride < 128 * 16 || 16 * a_chunk_stride > 65536) return (int)cudaErrorInvalidValue;
  if (b_chunk_stride % 16 != 0 || b_chunk_stride < n * 16 || 16 * b_chunk_stride > 65536) return (int)cudaErrorInvalidValue;
  const int smem_bytes = 65536 + 65536;
  cudaError_t err = cudaFuncSetAttribute(umma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (err != cudaSuccess) return (int)err;
  umma_probe_kernel<<<1, 128, smem_bytes, stream>>>(a, b, d, n, a_chunk_stride, b_chunk_stride, a_in_tmem, error_flag);
  return (int)cudaGetLastError();
}

extern "C" int frwkv_probe_tmem_roundtrip(const uint32_t* in, uint32_t* out, cudaStream_t stream) {
  if (!in || !out) return (int)cudaErrorInvalidValue;
  tmem_roundtrip_kernel<<<1, 128, 0, stream>>>(in, out);
  return (int)cudaGetLastError();
}

// Synchronous on purpose (test code): returns -4 when the wait gave up, 0 if the barrier completed (it cannot).
extern "C" int frwkv_probe_bounded_wait(uint32_t limit, int32_t* flag_dev, unsigned long long* cycles_dev,
                                        cudaStream_t stream) {
  if (!flag_dev || !cycles_dev) return (int)cudaErrorInvalidValue;
  bounded_wait_kernel<<<1, 128, 0, stream>>>(limit, flag_dev, cycles_dev);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return (int)err;
  err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) return (int)err;
  int flag = 0;
  err = cudaMemcpy(&flag, flag_dev, sizeof(int), cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) return (int)err;
  return flag != 0 ? -4 : 0;
}
