// Shared declarations of the TMix projection kernels (tmix_linear.cu: small-row and cp.async tensor-core kernels;
// tmix_gemm_tma.cu: the TMA-fed persistent tensor-core GEMM).
#pragma once

#include "frwkv_common.cuh"

namespace frwkv {

constexpr int kMaxProblems = 4;

struct LinearProblem {
  const void* x;        // [M][K]
  const void* w;        // [N][K] (w_kn == 0, the reference's original layout) or [K][N] (w_kn == 1, its runtime layout)
  void* y;              // [M][N]
  const void* v;        // epilogue 1: [M][N]
  const void* v_first;  // epilogue 1: [M][N]
  const void* v0;       // epilogue 1: [N]
  int n, k, act, epilogue;
  int w_kn = 0;
};
struct LinearGroup {
  LinearProblem p[kMaxProblems];
};

__device__ __forceinline__ float apply_act(float x, int act) {
  if (act == 1) return tanhf(x);
  if (act == 2) return 1.f / (1.f + __expf(-x));
  return x;
}

template <typename io_t>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  using IO = Io16<io_t>;
  float2 t;
  t = IO::unpack(u.x); f[0] = t.x; f[1] = t.y;
  t = IO::unpack(u.y); f[2] = t.x; f[3] = t.y;
  t = IO::unpack(u.z); f[4] = t.x; f[5] = t.y;
  t = IO::unpack(u.w); f[6] = t.x; f[7] = t.y;
}

// epilogue of one output element (row m, column n) with accumulator acc
template <typename io_t>
__device__ __forceinline__ float finish(const LinearProblem& pr, float acc, int m, int n) {
  if (pr.epilogue == 1) {  // v + (v_first - v) * sigmoid(v0 + acc)
    const long long o = (long long)m * pr.n + n;
    const float vv = Io16<io_t>::load(static_cast<const io_t*>(pr.v) + o);
    const float vf = Io16<io_t>::load(static_cast<const io_t*>(pr.v_first) + o);
    const float z = Io16<io_t>::load(static_cast<const io_t*>(pr.v0) + n) + acc;
    return fmaf(vf - vv, 1.f / (1.f + __expf(-z)), vv);
  }
  return acc;
}

// kind::f16 tcgen05.mma, A and B from shared memory, fp32 accumulator in tensor memory
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// instruction descriptor of kind::f16: fp32 accumulate, A K-major, fp16 (0) or bf16 (1) inputs; bit 16 set = the B
// operand is MN-major (its tile holds rows of the contraction index: a [K][N] weight as it lies in memory)
__host__ __device__ constexpr uint32_t idesc_f16(bool bf16, int M, int N, bool b_mn_major = false) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

// stores the last row of every sequence in its shift-state slot (tmix_elementwise.cu)
int launch_shift_state_update(const void* x, void* shift_state_pool, const int* cu_seqlens, const int* state_indices,
                              const int* metadata_status, int num_sequences, int channels, int io_dtype,
                              cudaStream_t stream);

// The TMA-fed GEMM takes a group whose problems all have act == 0 and 16-byte aligned x / w rows.
// Returns FRWKV_OK, or a negative code with the message set.
bool linear_tma_usable(const LinearGroup& g, int count, int M);
int launch_linear_tma(const LinearGroup& g, int count, int M, int io_dtype, int* error_flag, cudaStream_t stream);

}  // namespace frwkv
