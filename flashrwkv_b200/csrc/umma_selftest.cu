// Diagnostic entry point: one tcgen05.mma product through the same descriptor helpers
// and shared-memory tile formats the WKV7 chunk kernels use.  It exists so that every
// tile size and chunk stride can be checked against a host matrix product in isolation.
#include "frwkv_common.cuh"
#include "umma.cuh"

namespace frwkv {
namespace {

constexpr int kM = 128;
constexpr int kK = 64;

// D[m][n] = sum_k A[m][k] * B[n][k]; A is [128][64], B is [N][64], D is [128][N] (row-major, global).
__global__ __launch_bounds__(128, 1) void umma_selftest_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                               float* __restrict__ Dout, int N,
                                                               int a_chunk_stride, int b_chunk_stride,
                                                               int a_raw_shift, int* __restrict__ error_flag) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t mbar;
  __shared__ uint32_t tmem_base_holder;
  unsigned char* a_tile = smem;
  unsigned char* b_tile = smem + 65536;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;

  // place A as a chunk-major tile: row = m, col = k
  for (int e = tid; e < kM * kK; e += 128) {
    const int row = e / kK, col = e % kK;
    *reinterpret_cast<float*>(a_tile + (col >> 2) * a_chunk_stride + row * 16 + (col & 3) * 4) =
        umma::to_tf32(A[e]);
  }
  if (a_raw_shift >= 0) {
    // layout probe: every 32-bit word of the A region holds (word index >> shift) & 2047, so that with a
    // one-hot B the output names the word the tensor core read for each (m, k)
    for (int i = tid; i < 16384; i += 128)
      reinterpret_cast<float*>(a_tile)[i] = float((i >> a_raw_shift) & 2047);
  }
  for (int e = tid; e < N * kK; e += 128) {
    const int row = e / kK, col = e % kK;
    *reinterpret_cast<float*>(b_tile + (col >> 2) * b_chunk_stride + row * 16 + (col & 3) * 4) =
        umma::to_tf32(B[e]);
  }
  if (tid == 0) {
    umma::mbar_init(&mbar, 1);
    umma::mbar_fence_init();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_base_holder, 128);
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_base_holder;

  if (tid == 0) {
    const uint32_t idesc = umma::idesc_tf32(kM, N);
    const uint32_t a_addr = umma::smem_u32(a_tile), b_addr = umma::smem_u32(b_tile);
    for (int ks = 0; ks < kK / 8; ++ks) {
      umma::mma_tf32_ss(tmem, umma::desc_k_major(a_addr + ks * umma::kstep_k_major(a_chunk_stride), a_chunk_stride),
                        umma::desc_k_major(b_addr + ks * umma::kstep_k_major(b_chunk_stride), b_chunk_stride), idesc,
                        ks > 0 ? 1u : 0u);
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
      umma::tmem_ld32(tmem + (uint32_t(warp * 32) << 16) + c0, v);
      umma::tmem_ld_wait();
      for (int j = 0; j < 32; ++j) Dout[tid * N + c0 + j] = __uint_as_float(v[j]);
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, 128);
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_selftest_umma(const float* a, const float* b, float* d, int n, int a_chunk_stride,
                                   int b_chunk_stride, int a_raw_shift,
                                   int32_t* error_flag, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(a && b && d && error_flag, "selftest_umma: null pointer argument");
  FRWKV_REQUIRE(n == 64 || n == 128, "selftest_umma: n must be 64 or 128");
  FRWKV_REQUIRE(a_chunk_stride % 16 == 0 && a_chunk_stride >= 128 * 16 && 16 * a_chunk_stride <= 65536,
                "selftest_umma: bad a_chunk_stride");
  FRWKV_REQUIRE(b_chunk_stride % 16 == 0 && b_chunk_stride >= n * 16 && 16 * b_chunk_stride <= 32768,
                "selftest_umma: bad b_chunk_stride");
  const int smem_bytes = 65536 + 32768;
  cudaError_t err = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (err != cudaSuccess) return fail(FRWKV_ERR_CUDA, "selftest_umma: %s", cudaGetErrorString(err));
  umma_selftest_kernel<<<1, 128, smem_bytes, reinterpret_cast<cudaStream_t>(stream)>>>(
      a, b, d, n, a_chunk_stride, b_chunk_stride, a_raw_shift, error_flag);
  return check_launch("umma_selftest_kernel");
}
