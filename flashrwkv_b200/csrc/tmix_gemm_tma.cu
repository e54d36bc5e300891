// TMix projections for many rows: y[M][N] = x[M][K] * W[N][K]^T as a persistent, warp-specialised tensor-core GEMM.
//
//   warp 0 (one lane)  producer: TMA tile loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of a 128 x 64 block of x
//                      and a BN x 64 block of W per pipeline stage, completion counted on the stage's "full" mbarrier
//   warp 1 (one lane)  MMA issuer: four tcgen05.mma (kind::f16, K = 16 each) per stage into one of two accumulators
//                      in tensor memory; tcgen05.commit releases the stage ("empty") and, after the last K block,
//                      hands the accumulator to the epilogue ("acc_full")
//   warps 2..5         epilogue: tcgen05.ld of the finished accumulator (each warp its 32 lanes), optional
//                      value-residual gate, 16-bit stores; then "acc_empty" lets the issuer reuse the accumulator
// so loads, tensor-core work and the epilogue of consecutive tiles overlap.  CTAs walk the output tiles of all problems
// of the group (tile = blockIdx.x, + gridDim.x, ...).  Every wait is bounded: on a time-out the role sets the error
// flag and leaves its loop, the others run into their own limits, and the kernel still frees its tensor memory.
//
// Operand tiles are exactly what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B: row r of a tile is 128 bytes (64 values
// of K) at byte offset 128 r, its 16-byte pieces XOR-permuted by (r mod 8).  The matching shared-memory descriptor is
// "K-major, 128-byte swizzle": stride byte offset 1024 (eight rows), start address advanced by 32 bytes per K = 16.
//
// A weight in the runtime layout [K][N] is loaded as it lies: per stage BN / 64 boxes of 64 (N) x 64 (K), i.e. tiles whose
// 128-byte rows run along N and are indexed by k.  That is the "MN-major, 128-byte swizzle" operand form: eight k rows
// (1024 bytes) per group, 64-column groups one box (8192 bytes) apart, start address advanced by 16 rows per K = 16.
//
// Replaces the cublasGemmEx / cublasLtMatmul calls of the reference's projections
// (csrc/sm120/tmix/linear/infer_fp16_forward_varlen.cu:1403-1446,1687-1777,2817-2900).

#include <cuda.h>

#include "tmix_linear.cuh"
#include "umma.cuh"

namespace frwkv {
namespace {

constexpr int kBM = 128, kBK = 64;
constexpr uint32_t kABytes = kBM * kBK * 2;  // 16 KB
constexpr int kGemmThreads = 192;

// kShift: the A operand is the token-shifted x, x + (prev - x) * mix, made in shared memory by four extra warps from
// the x tile and the tile of the rows before (a second TMA load of the same map, one row up) before the MMA reads it.
template <int BN, bool kShift>
struct Cfg {
  static constexpr uint32_t kBBytes = BN * kBK * 2;
  static constexpr uint32_t kPrevBytes = kShift ? kABytes : 0;
  static constexpr uint32_t kStageBytes = kABytes + kPrevBytes + kBBytes;
  static constexpr int kPlain = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kStages = kShift ? (BN == 256 ? 3 : (BN == 128 ? 4 : 5)) : kPlain;
  static constexpr uint32_t kSmem = kStages * kStageBytes + 1024;  // + slack to align the tiles to 1024 bytes
  static constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulators (a power of two >= 32)
  static constexpr int kThreads = kShift ? kGemmThreads + 128 : kGemmThreads;
};

struct GemmParams {
  CUtensorMap map_x[kMaxProblems];
  CUtensorMap map_w[kMaxProblems];
  LinearGroup group;
  const void* mix[kMaxProblems];     // kShift: the token-shift vector [K] of each problem
  const void* shift_pool;            // kShift: [slots][K], the row before the first row of a sequence
  const int* row_prev_slot;          // kShift: [M], the slot for a sequence's first row, -1 for every other row
  int tile_begin[kMaxProblems + 1];  // first tile index of each problem
  int tiles_m;                       // row tiles (the same for all problems)
  int count, M;
};

// K-major operand tile with 128-byte swizzle: [0,14) address >> 4, [16,30) leading offset (unused, 1),
// [32,46) stride offset 1024 >> 4, [46,48) version 1, [61,64) layout 2 = SWIZZLE_128B
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr) {
  return uint64_t((addr & 0x3ffffu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
         (uint64_t(2) << 61);
}

// MN-major operand tile with 128-byte swizzle (rows = contraction index, 64 N values per row): leading offset = the
// distance between 64-column groups (one box), stride offset = eight rows
__device__ __forceinline__ uint64_t desc_mn_sw128(uint32_t addr) {
  return uint64_t((addr & 0x3ffffu) >> 4) | (uint64_t(8192 >> 4) << 16) | (uint64_t(1024 >> 4) << 32) |
         (uint64_t(1) << 46) | (uint64_t(2) << 61);
}

__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint64_t* mbar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_dst),
      "l"(map), "r"(x), "r"(y), "r"(umma::smem_u32(mbar))
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* mbar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(umma::smem_u32(mbar)) : "memory");
}

template <typename io_t, int BN, bool kShift>
__global__ __launch_bounds__(Cfg<BN, kShift>::kThreads, 1) void linear_tma_kernel(const __grid_constant__ GemmParams prm,
                                                                                  int* __restrict__ error_flag) {
  using IO = Io16<io_t>;
  using C = Cfg<BN, kShift>;
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t full_bar[C::kStages], empty_bar[C::kStages], ready_bar[C::kStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_holder;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t tiles_base = (umma::smem_u32(smem_raw) + 1023u) & ~1023u;

  if (tid == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      umma::mbar_init(&full_bar[i], 1);
      umma::mbar_init(&empty_bar[i], 1);
      umma::mbar_init(&ready_bar[i], 4);  // one arrival per transform warp
    }
    for (int i = 0; i < 2; ++i) {
      umma::mbar_init(&acc_full[i], 1);
      umma::mbar_init(&acc_empty[i], 4);
    }
    umma::mbar_fence_init();
  }
  if (warp == 1) umma::tmem_alloc(&tmem_holder, C::kTmemCols);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_holder;
  const int total_tiles = prm.tile_begin[prm.count];
  bool ok = true;

  // tile -> (problem, first row, first column); rows vary fastest so that concurrent CTAs share a block of W
  const auto locate = [&](int tile, int& z, int& m0, int& n0) {
    z = 0;
    while (z + 1 < prm.count && tile >= prm.tile_begin[z + 1]) ++z;
    const int local = tile - prm.tile_begin[z];
    m0 = (local % prm.tiles_m) * kBM;
    n0 = (local / prm.tiles_m) * BN;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int z, m0, n0;
        locate(tile, z, m0, n0);
        const int KB = (prm.group.p[z].k + kBK - 1) / kBK;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          if (!umma::mbar_wait(&empty_bar[s], ph ^ 1u)) { ok = false; break; }
          umma::mbar_expect_tx(&full_bar[s], C::kStageBytes);
          const uint32_t a_dst = tiles_base + s * C::kStageBytes;
          tma_load_2d(a_dst, &prm.map_x[z], kb * kBK, m0, &full_bar[s]);
          // the rows before: the same map one row up (row -1 of the first tile reads as zeros and is never used:
          // row 0 starts a sequence)
          if (kShift) tma_load_2d(a_dst + kABytes, &prm.map_x[z], kb * kBK, m0 - 1, &full_bar[s]);
          const uint32_t b_dst = a_dst + kABytes + C::kPrevBytes;
          if (prm.group.p[z].w_kn) {
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, &prm.map_w[z], n0 + 64 * j, kb * kBK, &full_bar[s]);
          } else {
            tma_load_2d(b_dst, &prm.map_w[z], kb * kBK, n0, &full_bar[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr bool is_bf16 = !__is_same(io_t, __half);
      uint32_t it = 0, t = 0;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++t) {
        int z, m0, n0;
        locate(tile, z, m0, n0);
        const int KB = (prm.group.p[z].k + kBK - 1) / kBK;
        const bool w_kn = prm.group.p[z].w_kn != 0;
        const uint32_t idesc = idesc_f16(is_bf16, kBM, BN, w_kn);
        const uint32_t acc = t & 1u, aph = (t >> 1) & 1u;
        if (!umma::mbar_wait(&acc_empty[acc], aph ^ 1u)) { ok = false; break; }
        umma::fence_after_sync();
        const uint32_t d_tmem = tmem + acc * BN;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          if (!umma::mbar_wait(kShift ? &ready_bar[s] : &full_bar[s], ph)) { ok = false; break; }
          umma::fence_after_sync();
          const uint32_t a_addr = tiles_base + s * C::kStageBytes, b_addr = a_addr + kABytes + C::kPrevBytes;
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks)
            mma_f16_ss(d_tmem, desc_sw128(a_addr + ks * 32),
                       w_kn ? desc_mn_sw128(b_addr + ks * 2048) : desc_sw128(b_addr + ks * 32), idesc,
                       (kb > 0 || ks > 0) ? 1u : 0u);
          umma::mma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
        }
        if (ok) umma::mma_commit(&acc_full[acc]);
      }
    }
  } else if (kShift && warp >= 6) {
    // ---- token shift: A <- x + (prev - x) * mix, in place in the x tile ---------------------------------------------
    // Thread t of the 128 takes the 16-byte piece at position t % 8 of rows t / 8 + 16 i (i = 0..7): consecutive lanes,
    // consecutive pieces.  TMA's 128-byte swizzle has put the logical piece (t % 8) ^ (row % 8) there, the same for
    // all eight rows of a thread, so its eight mix values per k-block are one 16-byte load.
    const int t = tid - kGemmThreads, pos = t & 7, sub = t >> 3;
    const int piece = pos ^ (sub & 7);  // logical 16-byte piece (eight k values) of these rows
    unsigned char* tiles = smem_raw + (tiles_base - umma::smem_u32(smem_raw));
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int z, m0, n0;
      locate(tile, z, m0, n0);
      const int K = prm.group.p[z].k, KB = (K + kBK - 1) / kBK;
      const io_t* mix = static_cast<const io_t*>(prm.mix[z]);
      int slot[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int m = m0 + sub + 16 * i;
        slot[i] = m < prm.M ? __ldg(prm.row_prev_slot + m) : -1;
      }
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
        if (!__all_sync(0xffffffffu, umma::mbar_wait(&full_bar[s], ph))) { ok = false; break; }
        const int k0 = kb * kBK + 8 * piece;
        if (k0 < K) {  // pieces beyond K are zero in x and stay zero
          float mf[8];
          unpack8<io_t>(__ldg(reinterpret_cast<const uint4*>(mix + k0)), mf);
          unsigned char* a_tile = tiles + s * C::kStageBytes;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t off = uint32_t(sub + 16 * i) * 128u + uint32_t(pos) * 16u;
            uint4* xa = reinterpret_cast<uint4*>(a_tile + off);
            uint4 pv = *reinterpret_cast<const uint4*>(a_tile + kABytes + off);
            if (slot[i] >= 0)
              pv = __ldg(reinterpret_cast<const uint4*>(static_cast<const io_t*>(prm.shift_pool) + (long long)slot[i] * K + k0));
            float xf[8], pf[8];
            unpack8<io_t>(*xa, xf);
            unpack8<io_t>(pv, pf);
#pragma unroll
            for (int e = 0; e < 8; ++e) xf[e] = slot[i] == -2 ? quiet_nan() : fmaf(pf[e] - xf[e], mf[e], xf[e]);  // -2: bad metadata
            *xa = make_uint4(IO::pack(xf[0], xf[1]), IO::pack(xf[2], xf[3]), IO::pack(xf[4], xf[5]), IO::pack(xf[6], xf[7]));
          }
        }
        umma::fence_async_smem();  // generic writes before the tensor core's reads of the tile
        __syncwarp();
        if (lane == 0) mbar_arrive(&ready_bar[s]);
      }
    }
  } else {
    const uint32_t quarter = warp & 3u;  // the tensor-memory lanes this warp may read: 32 * (warp % 4) ..
    uint32_t t = 0;
    int tile = blockIdx.x;
    for (; tile < total_tiles && ok; tile += gridDim.x, ++t) {
      int z, m0, n0;
      locate(tile, z, m0, n0);
      const LinearProblem& pr = prm.group.p[z];
      const uint32_t acc = t & 1u, aph = (t >> 1) & 1u;
      // warp-uniform outcome: the tensor-memory loads below need the whole warp
      if (!__all_sync(0xffffffffu, umma::mbar_wait(&acc_full[acc], aph))) { ok = false; break; }
      umma::fence_after_sync();
      const int m = m0 + 32 * quarter + lane;
      io_t* y = static_cast<io_t*>(pr.y);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t u[32];
        umma::tmem_ld32(tmem + ((32u * quarter) << 16) + acc * BN + c0, u);
        umma::tmem_ld_wait();
        if (m < prm.M) {
#pragma unroll
          for (int jj = 0; jj < 32; jj += 8) {
            const int n = n0 + c0 + jj;
            if (n < pr.n) {  // n and N are multiples of 8
              float o[8];
              if (pr.epilogue == 1) {  // value-residual gate, its three operands as 16-byte pieces
                const long long at = (long long)m * pr.n + n;
                float vv[8], vf[8], z0[8];
                unpack8<io_t>(*reinterpret_cast<const uint4*>(static_cast<const io_t*>(pr.v) + at), vv);
                unpack8<io_t>(*reinterpret_cast<const uint4*>(static_cast<const io_t*>(pr.v_first) + at), vf);
                unpack8<io_t>(*reinterpret_cast<const uint4*>(static_cast<const io_t*>(pr.v0) + n), z0);
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  o[e] = fmaf(vf[e] - vv[e], 1.f / (1.f + __expf(-(z0[e] + __uint_as_float(u[jj + e])))), vv[e]);
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(u[jj + e]);
              }
              *reinterpret_cast<uint4*>(y + (long long)m * pr.n + n) =
                  make_uint4(IO::pack(o[0], o[1]), IO::pack(o[2], o[3]), IO::pack(o[4], o[5]), IO::pack(o[6], o[7]));
            }
          }
        }
      }
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
    // a wait ran out: the tile it was for and the tiles this CTA never got to read as NaN, not as stale memory
    for (; !ok && tile < total_tiles; tile += gridDim.x) {
      int z, m0, n0;
      locate(tile, z, m0, n0);
      const LinearProblem& pr = prm.group.p[z];
      const int m = m0 + 32 * quarter + lane;
      io_t* y = static_cast<io_t*>(pr.y);
      for (int n = n0; m < prm.M && n < n0 + BN && n < pr.n; ++n) y[(long long)m * pr.n + n] = IO::store(quiet_nan());
    }
  }
  if (!ok) {
    if (error_flag != nullptr) atomicExch(error_flag, 5);
    // give copies and MMAs that may still be in flight time to finish before the shared and tensor memory go away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  __syncwarp();
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 1) umma::tmem_dealloc(tmem, C::kTmemCols);
}

// ---- host side -----------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static const EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// [rows][K] 16-bit matrix, boxes of 64 (K) x box_rows, 128-byte swizzle, zero fill outside
bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows, bool bf16) {
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return encode_tiled()(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                        const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [K][N] 16-bit matrix (runtime-layout weight), boxes of 64 (N) x 64 (K), 128-byte swizzle, zero fill outside
bool make_map_kn(CUtensorMap* map, const void* base, int K, int N, bool bf16) {
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};
  const cuuint64_t strides[1] = {(cuuint64_t)N * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)kBK};
  const cuuint32_t elem[2] = {1, 1};
  return encode_tiled()(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                        const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename io_t, int BN, bool kShift>
int launch_bn(GemmParams& prm, bool bf16, int sm_count, int* error_flag, cudaStream_t stream) {
  int tiles = 0;
  for (int z = 0; z < prm.count; ++z) {
    const LinearProblem& p = prm.group.p[z];
    prm.tile_begin[z] = tiles;
    tiles += prm.tiles_m * ((p.n + BN - 1) / BN);
    const bool w_ok = p.w_kn ? make_map_kn(&prm.map_w[z], p.w, p.k, p.n, bf16)
                             : make_map(&prm.map_w[z], p.w, p.n, p.k, BN, bf16);
    if (!make_map(&prm.map_x[z], p.x, prm.M, p.k, kBM, bf16) || !w_ok)
      return fail(FRWKV_ERR_CUDA, "tmix_linear: cuTensorMapEncodeTiled failed (problem %d)", z);
  }
  for (int z = prm.count; z <= kMaxProblems; ++z) prm.tile_begin[z] = tiles;
  using C = Cfg<BN, kShift>;
  cudaError_t e = cudaFuncSetAttribute(linear_tma_kernel<io_t, BN, kShift>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)C::kSmem);
  if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "tmix_linear: %s", cudaGetErrorString(e));
  const int grid = tiles < sm_count ? tiles : sm_count;
  linear_tma_kernel<io_t, BN, kShift><<<grid, C::kThreads, C::kSmem, stream>>>(prm, error_flag);
  return check_launch("linear_tma_kernel");
}

template <typename io_t, bool kShift>
int launch_typed(const LinearGroup& g, int count, int M, bool bf16, const void* const* mix, const void* shift_pool,
                 const int* row_prev_slot, int* error_flag, cudaStream_t stream) {
  int device = 0, sm_count = 0;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
  if (sm_count <= 0) sm_count = 1;
  GemmParams prm;
  prm.group = g;
  prm.count = count;
  prm.M = M;
  for (int z = 0; z < kMaxProblems; ++z) prm.mix[z] = (kShift && z < count) ? mix[z] : nullptr;
  prm.shift_pool = shift_pool;
  prm.row_prev_slot = row_prev_slot;
  prm.tiles_m = (M + kBM - 1) / kBM;
  // the widest tile that still gives every SM a tile (wide tiles read x fewer times)
  const auto tiles_for = [&](int bn) {
    int t = 0;
    for (int z = 0; z < count; ++z) t += prm.tiles_m * ((g.p[z].n + bn - 1) / bn);
    return t;
  };
  if (tiles_for(256) >= sm_count) return launch_bn<io_t, 256, kShift>(prm, bf16, sm_count, error_flag, stream);
  if (tiles_for(128) >= sm_count) return launch_bn<io_t, 128, kShift>(prm, bf16, sm_count, error_flag, stream);
  return launch_bn<io_t, 64, kShift>(prm, bf16, sm_count, error_flag, stream);
}

}  // namespace

bool linear_tma_usable(const LinearGroup& g, int count, int M) {
  if (M <= 8 || encode_tiled() == nullptr) return false;
  for (int z = 0; z < count; ++z) {
    const LinearProblem& p = g.p[z];
    if (p.act != 0) return false;  // the activation on x needs a pass over the staged tile: cp.async kernel
    if ((reinterpret_cast<uintptr_t>(p.x) & 15u) || (reinterpret_cast<uintptr_t>(p.w) & 15u)) return false;
    if (p.k % 8 != 0 || p.n % 8 != 0) return false;
  }
  return true;
}

int launch_linear_tma(const LinearGroup& g, int count, int M, int io_dtype, int* error_flag, cudaStream_t stream) {
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_typed<__nv_bfloat16, false>(g, count, M, true, nullptr, nullptr, nullptr, error_flag, stream);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_typed<__half, false>(g, count, M, false, nullptr, nullptr, nullptr, error_flag, stream);
  return fail(FRWKV_ERR_UNSUPPORTED, "tmix_linear: tensors must be float16 or bfloat16");
}

// y_z = (x + (prev - x) * mix_z) W_z^T for up to four projections of the same rows x: mix[z] is [K]; prev is the row
// before, or shift_pool[row_prev_slot[m]] where row m starts a sequence (row_prev_slot[m] >= 0)
int launch_linear_tma_shift(const LinearGroup& g, int count, int M, int io_dtype, const void* const* mix,
                            const void* shift_pool, const int* row_prev_slot, int* error_flag, cudaStream_t stream) {
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_typed<__nv_bfloat16, true>(g, count, M, true, mix, shift_pool, row_prev_slot, error_flag, stream);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_typed<__half, true>(g, count, M, false, mix, shift_pool, row_prev_slot, error_flag, stream);
  return fail(FRWKV_ERR_UNSUPPORTED, "tmix_linear: tensors must be float16 or bfloat16");
}

}  // namespace frwkv
