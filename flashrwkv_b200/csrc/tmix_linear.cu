// TMix projections: y[M][N] = act(x)[M][K] * W[N][K]^T (+ value-residual epilogue), grouped so that the three or four
// low-rank projections of a TMix layer (decay / a / gate / value-residual) go out in one launch.
//
// Two kernels, picked by the row count:
//   * M <= 8 ("skinny", decode): weight-bandwidth bound.  x is staged once per CTA in shared memory as fp32 with the
//     activation applied; every weight element is read exactly once with 16-byte loads.  For long rows (K >= 256) a
//     warp owns two output columns at a time and reduces with shuffles; for short rows (rank-out) eight lanes own one.
//   * M > 8: tcgen05 tensor-core GEMM (kind::f16, fp32 accumulate in tensor memory).  Problems without an activation
//     on x go to the TMA-fed persistent kernel of tmix_gemm_tma.cu; the kernel here (128 x 64 output tile per CTA, K in
//     blocks of 64 through a 4-stage cp.async pipeline into chunk-major tiles, see umma.cuh) applies tanh / sigmoid
//     to the staged x tile and so serves the rank-out projections.
// Weights are in the reference's "original" layout [N][K] (K contiguous).
//
// Replaces linear_wag[v]_rank_in_f16_kernel / linear_wag[v]_rank_out_f16_kernel
// (csrc/sm120/tmix/linear/infer_fp16_forward_varlen.cu:916-1233), the linear_orig_* / linear_t_* GEMV-class kernels
// (:133-786) and the cublasGemmEx / cublasLtMatmul calls (:1403-1446,1687-1777) of the reference.

#include <cstdlib>

#include "tmix_linear.cuh"
#include "umma.cuh"

namespace frwkv {
namespace {

template <typename io_t, int M>
__global__ __launch_bounds__(256) void linear_skinny_kernel(LinearGroup group) {
  using IO = Io16<io_t>;
  extern __shared__ __align__(16) unsigned char xs_raw[];
  const LinearProblem& pr = group.p[blockIdx.y];
  chain_release();
  SkinnyPrefetch pf;
  skinny_prefetch<io_t>(pr.w, pr.n, pr.k, pf, blockIdx.x, gridDim.x);
  chain_wait();
  const int kv = pr.k >> 3;
  // fp32 x as two planes of float4: plane 0 holds elements 8c..8c+3 of row m at [m*kv + c], plane 1 elements 8c+4..8c+7
  // (consecutive lanes then read consecutive 16-byte words: no bank conflicts)
  float4* xs = reinterpret_cast<float4*>(xs_raw);
  float4* xs_hi = xs + M * kv;
  for (int i = threadIdx.x; i < M * kv; i += blockDim.x) {
    float f[8];
    unpack8<io_t>(__ldg(reinterpret_cast<const uint4*>(pr.x) + i), f);
    if (pr.act != 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = apply_act(f[e], pr.act);
    }
    xs[i] = make_float4(f[0], f[1], f[2], f[3]);
    xs_hi[i] = make_float4(f[4], f[5], f[6], f[7]);
  }
  __syncthreads();
  skinny_products<io_t, M>(pr, xs, xs_hi, pf, blockIdx.x, gridDim.x);
}

// ---- token shift fused into the projections (decode) -------------------------------------------------------------
// y_j = (x + (prev - x) * mix_j) W_j^T for up to eight projections of the same rows x in one launch: the six-way
// token-shift interpolation (mix6) happens while x is staged, in fp32, instead of in a kernel of its own that writes
// six [M, C] tensors for the projections to read back.  prev is the previous row of the same sequence, or the
// sequence's shift state for its first row.  The shift states are updated by a separate small kernel afterwards
// (every CTA here reads them).  grid = (column blocks, projections).
constexpr int kMaxShiftProjections = 8;
struct ShiftProjection {
  const void* mix;  // [C]
  const void* w;    // [N][C]
  void* y;          // [M][N]
  int n;
};
struct ShiftProjectGroup {
  ShiftProjection p[kMaxShiftProjections];
};

template <typename io_t, int M>
__global__ __launch_bounds__(256) void shift_project_kernel(ShiftProjectGroup group, const io_t* __restrict__ x,
                                                            const io_t* __restrict__ shift_pool,
                                                            const int* __restrict__ cu_seqlens,
                                                            const int* __restrict__ state_indices,
                                                            const int* __restrict__ status, int num_sequences, int C) {
  using IO = Io16<io_t>;
  extern __shared__ __align__(16) unsigned char xs_raw[];
  __shared__ const io_t* prev_row[M];
  const ShiftProjection& sp = group.p[blockIdx.y];
  chain_release();
  SkinnyPrefetch pf;
  skinny_prefetch<io_t>(sp.w, sp.n, C, pf, blockIdx.x, gridDim.x);
  chain_wait();
  const int kv = C >> 3;
  io_t* y = static_cast<io_t*>(sp.y);
  if (status != nullptr && status[0] != 0) {  // fail closed: NaN outputs
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * sp.n; i += gridDim.x * blockDim.x)
      y[i] = IO::store(quiet_nan());
    return;
  }
  if (threadIdx.x < M) {
    const int row = threadIdx.x;
    int seq = 0;
    while (seq + 1 < num_sequences && cu_seqlens[seq + 1] <= row) ++seq;  // at most eight rows: a linear search
    prev_row[row] = row == cu_seqlens[seq] ? shift_pool + (long long)state_indices[seq] * C
                                           : x + (long long)(row - 1) * C;
  }
  __syncthreads();
  float4* xs = reinterpret_cast<float4*>(xs_raw);
  float4* xs_hi = xs + M * kv;
  const uint4* mixv = reinterpret_cast<const uint4*>(sp.mix);
  for (int c = threadIdx.x; c < kv; c += blockDim.x) {
    uint4 rx[M], rp[M];
    const uint4 rm = __ldg(mixv + c);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      rx[m] = __ldg(reinterpret_cast<const uint4*>(x) + m * kv + c);
      rp[m] = __ldg(reinterpret_cast<const uint4*>(prev_row[m]) + c);
    }
    float mf[8];
    unpack8<io_t>(rm, mf);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float xf[8], pf8[8];
      unpack8<io_t>(rx[m], xf);
      unpack8<io_t>(rp[m], pf8);
#pragma unroll
      for (int e = 0; e < 8; ++e) xf[e] = fmaf(pf8[e] - xf[e], mf[e], xf[e]);
      xs[m * kv + c] = make_float4(xf[0], xf[1], xf[2], xf[3]);
      xs_hi[m * kv + c] = make_float4(xf[4], xf[5], xf[6], xf[7]);
    }
  }
  __syncthreads();
  const LinearProblem pr{x, sp.w, sp.y, nullptr, nullptr, nullptr, sp.n, C, 0, 0};
  skinny_products<io_t, M>(pr, xs, xs_hi, pf, blockIdx.x, gridDim.x);
}

// ---- tensor-core kernel -----------------------------------------------------------------------------------
constexpr int kBM = 128, kBN = 64, kBK = 64, kStages = 4;
// Loads run kAhead k-blocks in front of the MMA.  A stage is refilled only once the MMA that read it has completed; with
// kAhead = kStages - 2 that MMA is two k-blocks old, so the wait never stalls on the MMA issued just before it.
constexpr int kAhead = kStages - 2;
constexpr uint32_t kCsA = kBM * 16 + 16;  // chunk stride of the A stage tile (128 rows), padded against bank conflicts
constexpr uint32_t kCsB = kBN * 16 + 16;
constexpr uint32_t kStageBytes = 8 * kCsA + 8 * kCsB;
constexpr uint32_t kTcSmem = kStages * kStageBytes;

template <typename io_t>
__global__ __launch_bounds__(128, 2) void linear_tc_kernel(LinearGroup group, int M, int* __restrict__ error_flag) {
  using IO = Io16<io_t>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t done_bar[kStages];
  __shared__ uint32_t tmem_holder;
  const LinearProblem& pr = group.p[blockIdx.z];
  const int K = pr.k, N = pr.n;
  const int n0 = blockIdx.x * kBN, m0 = blockIdx.y * kBM;
  if (n0 >= N) return;  // problems of one group may have different widths
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < kStages; ++i) umma::mbar_init(&done_bar[i], 1);
    umma::mbar_fence_init();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_holder, 64);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_holder;
  const uint32_t sbase = umma::smem_u32(smem);
  const io_t* x = static_cast<const io_t*>(pr.x);
  const io_t* w = static_cast<const io_t*>(pr.w);
  const int KB = (K + kBK - 1) / kBK;
  constexpr bool is_bf16 = sizeof(typename IO::pair) == 4 && !__is_same(io_t, __half);
  const uint32_t idesc = (1u << 4) | ((is_bf16 ? 1u : 0u) << 7) | ((is_bf16 ? 1u : 0u) << 10) |
                         (uint32_t(kBN >> 3) << 17) | (uint32_t(kBM >> 4) << 24);

  auto load_stage = [&](int kb) {
    const uint32_t st = sbase + uint32_t(kb % kStages) * kStageBytes;
    const int k0 = kb * kBK;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = i * 128 + tid, r = idx >> 3, c = idx & 7;
      const bool in = (m0 + r < M) && (k0 + 8 * c < K);
      const io_t* src = in ? x + (long long)(m0 + r) * K + k0 + 8 * c : x;
      umma::cp_async16(st + uint32_t(c) * kCsA + r * 16, src, in ? 16u : 0u);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = i * 128 + tid, r = idx >> 3, c = idx & 7;
      const bool in = (n0 + r < N) && (k0 + 8 * c < K);
      const io_t* src = in ? w + (long long)(n0 + r) * K + k0 + 8 * c : w;
      umma::cp_async16(st + 8 * kCsA + uint32_t(c) * kCsB + r * 16, src, in ? 16u : 0u);
    }
  };

  bool ok = true;
#pragma unroll
  for (int s = 0; s < kAhead; ++s) {
    if (s < KB) load_stage(s);
    umma::cp_async_commit();
  }
  for (int kb = 0; kb < KB; ++kb) {
    const int pre = kb + kAhead;
    if (pre < KB) {
      const int old = pre - kStages;  // k-block whose MMA last read the stage about to be refilled
      if (old >= 0) ok = umma::mbar_wait(&done_bar[old % kStages], (old / kStages) & 1) && ok;
      load_stage(pre);
    }
    umma::cp_async_commit();
    asm volatile("cp.async.wait_group %0;" ::"n"(kAhead) : "memory");
    unsigned char* st = smem + uint32_t(kb % kStages) * kStageBytes;
    if (pr.act != 0) {  // activation on the A operand: each thread transforms the chunks it copied itself
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = i * 128 + tid, r = idx >> 3, c = idx & 7;
        uint4* q = reinterpret_cast<uint4*>(st + uint32_t(c) * kCsA + r * 16);
        float f[8];
        unpack8<io_t>(*q, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = apply_act(f[e], pr.act);
        *q = make_uint4(IO::pack(f[0], f[1]), IO::pack(f[2], f[3]), IO::pack(f[4], f[5]), IO::pack(f[6], f[7]));
      }
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      umma::fence_after_sync();
      const uint32_t a_addr = sbase + uint32_t(kb % kStages) * kStageBytes, b_addr = a_addr + 8 * kCsA;
#pragma unroll
      for (int ks = 0; ks < kBK / 16; ++ks)
        mma_f16_ss(tmem, umma::desc_k_major(a_addr + ks * 2 * kCsA, kCsA), umma::desc_k_major(b_addr + ks * 2 * kCsB, kCsB),
                   idesc, (kb > 0 || ks > 0) ? 1u : 0u);
      umma::mma_commit(&done_bar[kb % kStages]);
    }
  }
  ok = umma::mbar_wait(&done_bar[(KB - 1) % kStages], ((KB - 1) / kStages) & 1) && ok;
  umma::fence_after_sync();
  if (ok) {
    const int m = m0 + warp * 32 + (tid & 31);
    io_t* y = static_cast<io_t*>(pr.y);
#pragma unroll 1
    for (int c0 = 0; c0 < kBN; c0 += 32) {
      uint32_t u[32];
      umma::tmem_ld32(tmem + (uint32_t(warp * 32) << 16) + c0, u);
      umma::tmem_ld_wait();
      if (m < M) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          const int n = n0 + c0 + j;
          if (n < N) {
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = finish<io_t>(pr, __uint_as_float(u[j + e]), m, n + e);
            *reinterpret_cast<uint4*>(y + (long long)m * N + n) =
                make_uint4(IO::pack(o[0], o[1]), IO::pack(o[2], o[3]), IO::pack(o[4], o[5]), IO::pack(o[6], o[7]));
          }
        }
      }
    }
  } else {  // a wait ran out: the tile reads as NaN, not as stale memory
    if (tid == 0 && error_flag != nullptr) atomicExch(error_flag, 3);
    const int m = m0 + warp * 32 + (tid & 31);
    io_t* y = static_cast<io_t*>(pr.y);
    for (int n = n0; m < M && n < n0 + kBN && n < N; ++n) y[(long long)m * N + n] = IO::store(quiet_nan());
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, 64);
}

// ---- small-row kernel for a weight in the runtime layout [K][N] ---------------------------------------------------
// A CTA owns 64 output columns: lane l of every warp the columns 2 l, 2 l + 1 (one 128-byte row segment per warp and
// k), the eight warps split K (k = warp, warp + 8, ...) and their partial sums meet in shared memory.  x is staged
// as fp32 with the activation applied, as in the kernel above.  Fewer CTAs pull the weights than in the original
// layout (N / 64), which is the price of reading this layout in place.
template <typename io_t, int M>
__global__ __launch_bounds__(256) void linear_kn_skinny_kernel(const LinearProblem pr) {
  using IO = Io16<io_t>;
  extern __shared__ float xs_kn[];           // [M][K]
  __shared__ float2 part[8][M][32];
  const int K = pr.k, N = pr.n, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const io_t* x = static_cast<const io_t*>(pr.x);
  for (int e = tid; e < M * K; e += 256) xs_kn[e] = apply_act(IO::load(x + e), pr.act);
  __syncthreads();
  const int n = 64 * blockIdx.x + 2 * lane;
  const io_t* w = static_cast<const io_t*>(pr.w);
  float2 acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = make_float2(0.f, 0.f);
  if (n < N) {
#pragma unroll 4
    for (int k = warp; k < K; k += 8) {
      const float2 wv = IO::unpack(__ldg(reinterpret_cast<const uint32_t*>(w + (long long)k * N + n)));
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float xv = xs_kn[m * K + k];
        acc[m].x = fmaf(xv, wv.x, acc[m].x);
        acc[m].y = fmaf(xv, wv.y, acc[m].y);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) part[warp][m][lane] = acc[m];
  __syncthreads();
  for (int e = tid; e < M * 32; e += 256) {
    const int m = e >> 5, l = e & 31, col = 64 * blockIdx.x + 2 * l;
    if (col < N) {
      float2 t = part[0][m][l];
#pragma unroll
      for (int wv = 1; wv < 8; ++wv) {
        t.x += part[wv][m][l].x;
        t.y += part[wv][m][l].y;
      }
      *reinterpret_cast<uint32_t*>(static_cast<io_t*>(pr.y) + (long long)m * N + col) =
          IO::pack(finish<io_t>(pr, t.x, m, col), finish<io_t>(pr, t.y, m, col + 1));
    }
  }
}

template <typename io_t>
int launch_linear_kn_skinny(const LinearProblem& pr, int M, cudaStream_t stream) {
  const size_t smem = (size_t)M * pr.k * 4;
  const dim3 grid((pr.n + 63) / 64);
#define FRWKV_KN(MM)                                                                                          \
  case MM: {                                                                                                  \
    if (smem > 24 * 1024) { /* the static partial-sum array takes up to 16 KB of the default 48 KB */        \
      cudaError_t e = cudaFuncSetAttribute(linear_kn_skinny_kernel<io_t, MM>,                                 \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "tmix_linear: %s", cudaGetErrorString(e));            \
    }                                                                                                         \
    linear_kn_skinny_kernel<io_t, MM><<<grid, 256, smem, stream>>>(pr);                                       \
    break;                                                                                                    \
  }
  switch (M) {
    FRWKV_KN(1) FRWKV_KN(2) FRWKV_KN(3) FRWKV_KN(4) FRWKV_KN(5) FRWKV_KN(6) FRWKV_KN(7) FRWKV_KN(8)
  }
#undef FRWKV_KN
  return check_launch("linear_kn_skinny_kernel");
}

template <typename io_t>
int launch_linear(const LinearGroup& g, int count, int M, int max_n, int max_k, int* error_flag, cudaStream_t stream) {
  if (M <= 8) {
    const size_t smem = (size_t)M * max_k * 4;
    const int blocks = max_k >= 256 ? (max_n + 8 * kSkinnyCols - 1) / (8 * kSkinnyCols) : (max_n + 31) / 32;
    dim3 grid(blocks < 1 ? 1 : blocks, count);
#define FRWKV_SKINNY(MM)                                                                                      \
  case MM: {                                                                                                  \
    if (smem > 48 * 1024) {                                                                                   \
      cudaError_t e = cudaFuncSetAttribute(linear_skinny_kernel<io_t, MM>,                                    \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
      if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "tmix_linear: %s", cudaGetErrorString(e));            \
    }                                                                                                         \
    launch_chained(linear_skinny_kernel<io_t, MM>, grid, dim3(256), smem, stream, g);                                         \
    break;                                                                                                    \
  }
    switch (M) {
      FRWKV_SKINNY(1) FRWKV_SKINNY(2) FRWKV_SKINNY(3) FRWKV_SKINNY(4)
      FRWKV_SKINNY(5) FRWKV_SKINNY(6) FRWKV_SKINNY(7) FRWKV_SKINNY(8)
    }
#undef FRWKV_SKINNY
    return check_launch("linear_skinny_kernel");
  }
  cudaError_t e = cudaFuncSetAttribute(linear_tc_kernel<io_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem);
  if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "tmix_linear: %s", cudaGetErrorString(e));
  dim3 grid((max_n + kBN - 1) / kBN, (M + kBM - 1) / kBM, count);
  linear_tc_kernel<io_t><<<grid, 128, kTcSmem, stream>>>(g, M, error_flag);
  return check_launch("linear_tc_kernel");
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_tmix_linear_grouped(const frwkv_linear_problem* problems, int count, int m, int io_dtype,
                                         int32_t* error_flag, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(problems != nullptr, "tmix_linear: null pointer argument");
  FRWKV_REQUIRE(count >= 1 && count <= kMaxProblems, "tmix_linear: 1..4 problems per call");
  FRWKV_REQUIRE(m > 0, "tmix_linear: row count must be positive");
  LinearGroup g;
  int max_n = 0, max_k = 0;
  for (int i = 0; i < count; ++i) {
    const frwkv_linear_problem& p = problems[i];
    FRWKV_REQUIRE(p.x && p.weight && p.y, "tmix_linear: null pointer in problem %d", i);
    FRWKV_REQUIRE(p.n > 0 && p.k > 0 && p.n % 8 == 0 && p.k % 8 == 0,
                  "tmix_linear: feature counts must be positive multiples of 8 (problem %d: n=%d k=%d)", i, p.n, p.k);
    FRWKV_REQUIRE(p.act >= 0 && p.act <= 2 && p.epilogue >= 0 && p.epilogue <= 1, "tmix_linear: bad act/epilogue code");
    if (p.epilogue == 1) FRWKV_REQUIRE(p.v && p.v_first && p.v0, "tmix_linear: value-residual epilogue needs v, v_first, v0");
    g.p[i] = LinearProblem{p.x, p.weight, p.y, p.v, p.v_first, p.v0, p.n, p.k, p.act, p.epilogue};
    max_n = p.n > max_n ? p.n : max_n;
    max_k = p.k > max_k ? p.k : max_k;
  }
  for (int i = count; i < kMaxProblems; ++i) g.p[i] = g.p[0];
  if (m <= 8) FRWKV_REQUIRE((size_t)m * max_k * 4 <= 200 * 1024, "tmix_linear: K too large for the small-row kernel");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype != FRWKV_DTYPE_BF16 && io_dtype != FRWKV_DTYPE_FP16)
    return fail(FRWKV_ERR_UNSUPPORTED, "tmix_linear: tensors must be float16 or bfloat16");
  if (linear_tma_usable(g, count, m)) return launch_linear_tma(g, count, m, io_dtype, error_flag, s);
  if (io_dtype == FRWKV_DTYPE_BF16) return launch_linear<__nv_bfloat16>(g, count, m, max_n, max_k, error_flag, s);
  if (io_dtype == FRWKV_DTYPE_FP16) return launch_linear<__half>(g, count, m, max_n, max_k, error_flag, s);
  return fail(FRWKV_ERR_UNSUPPORTED, "tmix_linear: tensors must be float16 or bfloat16");
}

// row m -> the shift-state slot that holds its predecessor when m is the first row of its sequence, else -1; -2 in
// every row when the metadata failed validation (the consumer then writes NaN)
namespace frwkv {
namespace {
__global__ void row_prev_slot_kernel(const int* __restrict__ cu_seqlens, const int* __restrict__ state_indices,
                                     const int* __restrict__ status, int num_sequences, int total_rows,
                                     int* __restrict__ out) {
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= total_rows) return;
  if (status != nullptr && status[0] != 0) { out[m] = -2; return; }
  int lo = 0, hi = num_sequences;  // largest s with cu_seqlens[s] <= m
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu_seqlens[mid] <= m) lo = mid; else hi = mid;
  }
  out[m] = cu_seqlens[lo] == m ? state_indices[lo] : -1;
}
}  // namespace
}  // namespace frwkv

extern "C" int frwkv_tmix_shift_project_gemm(const void* x, void* shift_state_pool, const int32_t* cu_seqlens,
                                             const int32_t* state_indices, const int32_t* metadata_status,
                                             const frwkv_shift_projection* projections, int count, int total_rows,
                                             int num_sequences, int channels, int io_dtype, int32_t* row_workspace,
                                             int32_t* error_flag, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(x && shift_state_pool && cu_seqlens && state_indices && projections && row_workspace,
                "tmix_shift_project_gemm: null pointer argument");
  FRWKV_REQUIRE(count >= 1 && count <= kMaxShiftProjections, "tmix_shift_project_gemm: 1..8 projections per call");
  FRWKV_REQUIRE(total_rows > 8, "tmix_shift_project_gemm: more than 8 rows (fewer: frwkv_tmix_shift_project_varlen)");
  FRWKV_REQUIRE(num_sequences >= 1 && num_sequences <= total_rows, "tmix_shift_project_gemm: bad sequence count");
  FRWKV_REQUIRE(channels >= 64 && channels % 8 == 0, "tmix_shift_project_gemm: channel count must be a multiple of 8");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  row_prev_slot_kernel<<<(total_rows + 255) / 256, 256, 0, s>>>(cu_seqlens, state_indices, metadata_status, num_sequences,
                                                                  total_rows, row_workspace);
  int rc = check_launch("row_prev_slot_kernel");
  if (rc != FRWKV_OK) return rc;
  for (int first = 0; first < count; first += kMaxProblems) {
    const int n = count - first < kMaxProblems ? count - first : kMaxProblems;
    LinearGroup g;
    const void* mix[kMaxProblems] = {nullptr, nullptr, nullptr, nullptr};
    for (int i = 0; i < n; ++i) {
      const frwkv_shift_projection& p = projections[first + i];
      FRWKV_REQUIRE(p.mix && p.weight && p.y, "tmix_shift_project_gemm: null pointer in projection %d", first + i);
      FRWKV_REQUIRE(p.n > 0 && p.n % 8 == 0, "tmix_shift_project_gemm: output width must be a positive multiple of 8");
      g.p[i] = LinearProblem{x, p.weight, p.y, nullptr, nullptr, nullptr, p.n, channels, 0, 0};
      mix[i] = p.mix;
    }
    for (int i = n; i < kMaxProblems; ++i) g.p[i] = g.p[0];
    if (!linear_tma_usable(g, n, total_rows))
      return fail(FRWKV_ERR_UNSUPPORTED, "tmix_shift_project_gemm: x, weights and mix vectors must be 16-byte aligned");
    rc = launch_linear_tma_shift(g, n, total_rows, io_dtype, mix, shift_state_pool, row_workspace, error_flag, s);
    if (rc != FRWKV_OK) return rc;
  }
  // every launch above has read the shift states: now they take each sequence's last row
  return launch_shift_state_update(x, shift_state_pool, cu_seqlens, state_indices, metadata_status, num_sequences,
                                   channels, io_dtype, s);
}

extern "C" int frwkv_tmix_shift_project_varlen(const void* x, void* shift_state_pool, const int32_t* cu_seqlens,
                                               const int32_t* state_indices, const int32_t* metadata_status,
                                               const frwkv_shift_projection* projections, int count, int total_rows,
                                               int num_sequences, int channels, int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(x && shift_state_pool && cu_seqlens && state_indices && projections,
                "tmix_shift_project: null pointer argument");
  FRWKV_REQUIRE(count >= 1 && count <= kMaxShiftProjections, "tmix_shift_project: 1..8 projections per call");
  FRWKV_REQUIRE(total_rows >= 1 && total_rows <= 8, "tmix_shift_project: 1..8 rows (more rows: mix6, then the GEMM)");
  FRWKV_REQUIRE(num_sequences >= 1 && num_sequences <= total_rows, "tmix_shift_project: bad sequence count");
  FRWKV_REQUIRE(channels >= 256 && channels % 8 == 0, "tmix_shift_project: channel count must be a multiple of 8, >= 256");
  FRWKV_REQUIRE((size_t)total_rows * channels * 4 <= 200 * 1024, "tmix_shift_project: too many channels");
  ShiftProjectGroup g;
  int max_n = 0;
  for (int i = 0; i < count; ++i) {
    const frwkv_shift_projection& p = projections[i];
    FRWKV_REQUIRE(p.mix && p.weight && p.y, "tmix_shift_project: null pointer in projection %d", i);
    FRWKV_REQUIRE(p.n > 0 && p.n % 8 == 0, "tmix_shift_project: output width must be a positive multiple of 8");
    g.p[i] = ShiftProjection{p.mix, p.weight, p.y, p.n};
    max_n = p.n > max_n ? p.n : max_n;
  }
  for (int i = count; i < kMaxShiftProjections; ++i) g.p[i] = g.p[0];
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)total_rows * channels * 4;
  const dim3 grid((max_n + 8 * kSkinnyCols - 1) / (8 * kSkinnyCols), count);
#define FRWKV_SHIFT_PROJECT(T, MM)                                                                                 \
  case MM: {                                                                                                       \
    if (smem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(shift_project_kernel<T, MM>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                             \
      if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "tmix_shift_project: %s", cudaGetErrorString(e));          \
    }                                                                                                              \
    launch_chained(shift_project_kernel<T, MM>, grid, dim3(256), smem, s, g, static_cast<const T*>(x),             \
                   static_cast<const T*>(shift_state_pool), cu_seqlens, state_indices, metadata_status,            \
                   num_sequences, channels);                                                                       \
    break;                                                                                                         \
  }
#define FRWKV_SHIFT_PROJECT_ALL(T)                                                                   \
  switch (total_rows) {                                                                              \
    FRWKV_SHIFT_PROJECT(T, 1) FRWKV_SHIFT_PROJECT(T, 2) FRWKV_SHIFT_PROJECT(T, 3) FRWKV_SHIFT_PROJECT(T, 4) \
    FRWKV_SHIFT_PROJECT(T, 5) FRWKV_SHIFT_PROJECT(T, 6) FRWKV_SHIFT_PROJECT(T, 7) FRWKV_SHIFT_PROJECT(T, 8) \
  }
  if (io_dtype == FRWKV_DTYPE_BF16) {
    FRWKV_SHIFT_PROJECT_ALL(__nv_bfloat16)
  } else if (io_dtype == FRWKV_DTYPE_FP16) {
    FRWKV_SHIFT_PROJECT_ALL(__half)
  } else {
    return fail(FRWKV_ERR_UNSUPPORTED, "tmix_shift_project: tensors must be float16 or bfloat16");
  }
#undef FRWKV_SHIFT_PROJECT_ALL
#undef FRWKV_SHIFT_PROJECT
  int rc = check_launch("shift_project_kernel");
  if (rc != FRWKV_OK) return rc;
  return launch_shift_state_update(x, shift_state_pool, cu_seqlens, state_indices, metadata_status, num_sequences,
                                   channels, io_dtype, s);
}

// One projection with the weight in the reference's runtime layout [k][n] (read in place: the small-row kernel above
// for m <= 8, the TMA-fed GEMM with an MN-major B operand for more rows; there the activation must be 0).
extern "C" int frwkv_tmix_linear_runtime_layout(const frwkv_linear_problem* problem, int m, int io_dtype,
                                                int32_t* error_flag, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(problem != nullptr && problem->x && problem->weight && problem->y, "tmix_linear: null pointer argument");
  const frwkv_linear_problem& p = *problem;
  FRWKV_REQUIRE(m > 0 && p.n > 0 && p.k > 0 && p.n % 8 == 0 && p.k % 8 == 0,
                "tmix_linear: sizes must be positive, feature counts multiples of 8");
  FRWKV_REQUIRE(p.act >= 0 && p.act <= 2 && p.epilogue >= 0 && p.epilogue <= 1, "tmix_linear: bad act/epilogue code");
  if (p.epilogue == 1) FRWKV_REQUIRE(p.v && p.v_first && p.v0, "tmix_linear: value-residual epilogue needs v, v_first, v0");
  LinearGroup g;
  g.p[0] = LinearProblem{p.x, p.weight, p.y, p.v, p.v_first, p.v0, p.n, p.k, p.act, p.epilogue, 1};
  for (int i = 1; i < kMaxProblems; ++i) g.p[i] = g.p[0];
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype != FRWKV_DTYPE_BF16 && io_dtype != FRWKV_DTYPE_FP16)
    return fail(FRWKV_ERR_UNSUPPORTED, "tmix_linear: tensors must be float16 or bfloat16");
  if (m <= 8 && ((size_t)m * p.k * 4 <= 200 * 1024 || p.act != 0)) {
    FRWKV_REQUIRE((size_t)m * p.k * 4 <= 200 * 1024, "tmix_linear: K too large for the small-row kernel");
    return io_dtype == FRWKV_DTYPE_BF16 ? launch_linear_kn_skinny<__nv_bfloat16>(g.p[0], m, s)
                                        : launch_linear_kn_skinny<__half>(g.p[0], m, s);
  }
  if (p.act != 0)
    return fail(FRWKV_ERR_UNSUPPORTED, "tmix_linear: a runtime-layout weight with more than 8 rows takes no activation "
                                       "(apply it to x first)");
  if (!linear_tma_usable(g, 1, m))
    return fail(FRWKV_ERR_UNSUPPORTED, "tmix_linear: runtime-layout weights need 16-byte aligned tensors");
  return launch_linear_tma(g, 1, m, io_dtype, error_flag, s);
}
