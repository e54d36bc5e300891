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

// ---- small-row products ("skinny") --------------------------------------------------------------------------------------
// grid = (column blocks, problems); dynamic shared memory = M * K fp32 values of x (activation applied): unpacking the
// 16-bit x once per CTA instead of once per weight row is what keeps M = 4..8 bound by the weight stream rather than
// by instruction issue.  Long rows (K >= 256): a warp owns two output columns at a time (sixteen 16-byte weight
// loads in flight per lane, every x value used twice) and reduces with shuffles.  Short rows (rank-out,
// K = rank): eight lanes share a column.
// Output columns a warp works on at a time (long rows) and 16-byte weight pieces per column and lane in flight at once.
// Two columns keep 128 CTAs busy on a 2048-wide projection; four columns halve the shared-memory reads of x but leave
// 64 CTAs to pull the weights, and the layer took twice as long (measured): the kernel lives on SMs pulling in parallel.
constexpr int kSkinnyCols = 2;
constexpr int kSkinnyDepth = 8;

// The first block of weight pieces of a warp's first column group.  Weights are constants, so a kernel fetches them
// before it waits for its predecessors in the stream and before it stages x: the DRAM round trip of the weight
// stream then overlaps the tail of the previous kernel and the staging.
struct SkinnyPrefetch {
  uint4 q[kSkinnyCols][kSkinnyDepth];
};
template <typename io_t>
__device__ __forceinline__ void skinny_prefetch(const void* weight, int N, int K, SkinnyPrefetch& pf, int vblock,
                                                int vgrid) {
  (void)vgrid;
  if (K < 256) return;
  const int lane = threadIdx.x & 31, kv = K >> 3;
  const int n = kSkinnyCols * (vblock * (blockDim.x >> 5) + (threadIdx.x >> 5));
  if (n >= N) return;
  const io_t* w = static_cast<const io_t*>(weight);
#pragma unroll
  for (int col = 0; col < kSkinnyCols; ++col) {
    const uint4* wrow = reinterpret_cast<const uint4*>(w + (long long)(n + col) * K);
#pragma unroll
    for (int j = 0; j < kSkinnyDepth; ++j) {
      const int c = lane + 32 * j;
      if (c < kv) pf.q[col][j] = __ldg(wrow + c);
    }
  }
}

// the products of one CTA: xs / xs_hi hold x as fp32 (see linear_skinny_kernel)
template <typename io_t, int M>
__device__ __forceinline__ void skinny_products(const LinearProblem& pr, const float4* xs, const float4* xs_hi,
                                                const SkinnyPrefetch& pf, int vblock, int vgrid) {
  using IO = Io16<io_t>;
  const int K = pr.k, N = pr.n, kv = K >> 3;
  const io_t* w = static_cast<const io_t*>(pr.w);
  io_t* y = static_cast<io_t*>(pr.y);
  if (K >= 256) {
    const int lane = threadIdx.x & 31;
    const int warps_total = vgrid * (blockDim.x >> 5);
    // N is a multiple of 8, so a group of kSkinnyCols columns starting at a multiple of kSkinnyCols is always complete
    const int n_first = kSkinnyCols * (vblock * (blockDim.x >> 5) + (threadIdx.x >> 5));
    for (int n = n_first; n < N; n += kSkinnyCols * warps_total) {
      // accumulators as fp32 pairs (even | odd elements of a piece): one fma.rn.f32x2 per two multiply-adds
      float2 acc[kSkinnyCols][M];
#pragma unroll
      for (int col = 0; col < kSkinnyCols; ++col) {
#pragma unroll
        for (int m = 0; m < M; ++m) acc[col][m] = make_float2(0.f, 0.f);
      }
      // all weight loads of a block (kSkinnyCols x kSkinnyDepth pieces per lane) are issued before the first one is used
      for (int cb = lane; cb < kv; cb += 32 * kSkinnyDepth) {
        uint4 q[kSkinnyCols][kSkinnyDepth];
        const bool fetched = (n == n_first && cb == lane);  // this block came in with skinny_prefetch
#pragma unroll
        for (int col = 0; col < kSkinnyCols; ++col) {
          const uint4* wrow = reinterpret_cast<const uint4*>(w + (long long)(n + col) * K);
#pragma unroll
          for (int j = 0; j < kSkinnyDepth; ++j) {
            const int c = cb + 32 * j;
            if (c < kv) q[col][j] = fetched ? pf.q[col][j] : __ldg(wrow + c);
          }
        }
#pragma unroll
        for (int j = 0; j < kSkinnyDepth; ++j) {
          const int c = cb + 32 * j;
          if (c < kv) {
            float2 wv[kSkinnyCols][4];
#pragma unroll
            for (int col = 0; col < kSkinnyCols; ++col) {
              wv[col][0] = IO::unpack(q[col][j].x); wv[col][1] = IO::unpack(q[col][j].y);
              wv[col][2] = IO::unpack(q[col][j].z); wv[col][3] = IO::unpack(q[col][j].w);
            }
#pragma unroll
            for (int m = 0; m < M; ++m) {
              const float4 xa = xs[m * kv + c], xb = xs_hi[m * kv + c];
              const float2 x0 = make_float2(xa.x, xa.y), x1 = make_float2(xa.z, xa.w);
              const float2 x2 = make_float2(xb.x, xb.y), x3 = make_float2(xb.z, xb.w);
#pragma unroll
              for (int col = 0; col < kSkinnyCols; ++col)
                acc[col][m] = __ffma2_rn(wv[col][0], x0, __ffma2_rn(wv[col][1], x1,
                                         __ffma2_rn(wv[col][2], x2, __ffma2_rn(wv[col][3], x3, acc[col][m]))));
            }
          }
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float t[kSkinnyCols];
#pragma unroll
        for (int col = 0; col < kSkinnyCols; ++col) {
          t[col] = acc[col][m].x + acc[col][m].y;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) t[col] += __shfl_xor_sync(0xffffffffu, t[col], o);
        }
        if (lane == 0) {
#pragma unroll
          for (int col = 0; col < kSkinnyCols; col += 2)
            *reinterpret_cast<uint32_t*>(y + (long long)m * N + n + col) =
                IO::pack(finish<io_t>(pr, t[col], m, n + col), finish<io_t>(pr, t[col + 1], m, n + col + 1));
        }
      }
    }
  } else {
    // short rows (rank-out, K = rank): eight lanes share a column, a warp works on four columns at a time
    const int lane = threadIdx.x & 31, sub = lane & 7, grp = lane >> 3;
    const int warps_total = vgrid * (blockDim.x >> 5);
    for (int n0 = 4 * (vblock * (blockDim.x >> 5) + (threadIdx.x >> 5)); n0 < N; n0 += 4 * warps_total) {
      const int n = n0 + grp;  // N is a multiple of 8: all four columns exist
      float2 acc[M];
#pragma unroll
      for (int m = 0; m < M; ++m) acc[m] = make_float2(0.f, 0.f);
      const uint4* wrow = reinterpret_cast<const uint4*>(w + (long long)n * K);
      for (int c = sub; c < kv; c += 8) {
        const uint4 q = __ldg(wrow + c);
        const float2 a0 = IO::unpack(q.x), a1 = IO::unpack(q.y), a2 = IO::unpack(q.z), a3 = IO::unpack(q.w);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float4 xa = xs[m * kv + c], xb = xs_hi[m * kv + c];
          acc[m] = __ffma2_rn(a0, make_float2(xa.x, xa.y),
                              __ffma2_rn(a1, make_float2(xa.z, xa.w),
                                         __ffma2_rn(a2, make_float2(xb.x, xb.y),
                                                    __ffma2_rn(a3, make_float2(xb.z, xb.w), acc[m]))));
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float t = acc[m].x + acc[m].y;
        t += __shfl_xor_sync(0xffffffffu, t, 1);
        t += __shfl_xor_sync(0xffffffffu, t, 2);
        t += __shfl_xor_sync(0xffffffffu, t, 4);
        if (sub == 0) y[(long long)m * N + n] = IO::store(finish<io_t>(pr, t, m, n));
      }
    }
  }
}

// The block index and grid size are arguments (vblock of vgrid CTAs share one problem's columns), so that a persistent
// kernel can give each projection a share of its CTAs.

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
// the same GEMM with the token shift applied to x while it is staged (tmix_gemm_tma.cu)
int launch_linear_tma_shift(const LinearGroup& g, int count, int M, int io_dtype, const void* const* mix,
                            const void* shift_pool, const int* row_prev_slot, int* error_flag, cudaStream_t stream);

}  // namespace frwkv
