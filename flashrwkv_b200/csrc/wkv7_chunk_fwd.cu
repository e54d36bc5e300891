// Chunked WKV7 forward on the tcgen05 tensor cores (head size 64, chunk length <= 64).
//
// Per (chunk, head) with chunk-start state S0 (K x V), tokens t = 0..L-1, per-key cumulative decay
// g_t = prod_{s<=t} w_s (g_{-1} = 1), the recurrence  S_t = diag(w_t) S_{t-1} + b_t (S_{t-1}^T a_t)^T + k_t v_t^T,
// y_t = S_t^T r_t  collapses to two affine maps of S0:
//     Y  = E S0 + F          (L x V)        S_L = M S0 + N        (K x V)
// with  A~ = a*g_{t-1}, R~ = r*g_t, B~ = b/g_t, K~ = k/g_t, B^ = B~*g_L, K^ = K~*g_L  (all L x K) and
//     A_ab = strict_lower(A~ B~^T)  A_ak = strict_lower(A~ K~^T)  A_rb = lower(R~ B~^T)  A_rk = lower(R~ K~^T)
//     T = (I - A_ab)^-1,  P = T A~,  Q = T A_ak V
//     E = R~ + A_rb P,  F = A_rb Q + A_rk V,  M = diag(g_L) + B^^T P,  N = B^^T Q + K^^T V.
//
// Kernel 1 (build, persistent CTAs over the (chunk, head) items, all chunks independent) forms [E;M] and [F;N] with five
// tcgen05.mma (kind::tf32, fp32 accumulate in tensor memory) products; the 64 x 64 unit-triangular inverse
// is done in fp32 on the CUDA cores (one thread per column of T).  Operands are rounded to tf32 once, with
// round-to-nearest, when they are written to shared memory.  Results go to a workspace laid out exactly as
// kernel 2's shared-memory operands.
// Kernel 2 (scan, one CTA per (sequence, head)) walks the chunks in order: per chunk one 128 x 64 x 64 MMA
// [Y; S'] = [E;M] S + [F;N], with the 64 KB of [E;M],[F;N] brought in by double-buffered bulk copies.
//
// Every tensor-core operand is a "chunk-major tile" with contraction over the tile's columns (see umma.cuh);
// where the producing thread owns a column rather than a row it writes 4-byte words, and the tile's chunk
// stride is padded by 16 bytes so those writes stay bank-conflict free.
//
// Replaces the reference's SIMT chunk family: infer_chunk_bf16_k1/k2
// (csrc/sm120/tmix/wkv7/infer_chunk_bf16_forward_varlen.cu:42-266) and build_transforms / scan_boundaries /
// emit_outputs (csrc/sm90/rl_infctx/wkv7/rl_infctx_chunk_fp32io16_forward.cu:317-538,
// rl_infctx_chunk_fp32io16_backward.cu:45-127), and the forward of statetune / pretrain
// (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_forward.cu:32-130).

#include "frwkv_common.cuh"
#include "umma.cuh"

namespace frwkv {
namespace {

constexpr int kL = 64;  // maximum chunk length
constexpr int kD = 64;
constexpr uint32_t kCS128 = 2048;   // chunk stride of a 128-row tile written row-wise
constexpr uint32_t kCS128P = 2064;  // ... of a 128-row tile that also receives column-wise (4-byte) writes
constexpr uint32_t kCS64P = 1040;   // ... of a 64-row tile with column-wise writes
constexpr uint32_t kWsTile = 32768; // bytes of one workspace tile ([E;M] or [F;N]) per (chunk, head)

// ---- build kernel shared-memory map -------------------------------------------------------------
constexpr uint32_t kOffX1 = 0;                       // [A~ ; R~]          128 rows x K, stride 2048
constexpr uint32_t kOffX2 = kOffX1 + 16 * kCS128;    // [B~ ; K~]  -> [A_ak ; -] -> [P | Q]^T   (reused in turn)
constexpr uint32_t kOffRB = kOffX2 + 16 * kCS128;    // [A_rb ; B^^T]      128 rows x s, stride 2064
constexpr uint32_t kOffRK = kOffRB + 16 * kCS128P;   // [A_rk ; K^^T]
constexpr uint32_t kOffAZ = kOffRK + 16 * kCS128P;   // [A~^T ; Z^T]       128 rows x s
constexpr uint32_t kOffTT = kOffAZ + 16 * kCS128P;   // T (rows t, cols s) 64 rows, stride 1040
constexpr uint32_t kOffVT = kOffTT + 16 * kCS64P;    // V^T (rows v, cols s)
constexpr uint32_t kOffSC = kOffVT + 16 * kCS64P;    // scratch: g[t][k] (stride 1040), later A_ab[t][s] (row stride 272)
constexpr uint32_t kScratchBytes = 64 * 272;
constexpr uint32_t kBuildSmem = kOffSC + kScratchBytes;  // 215,296 bytes
constexpr uint32_t kAabRow = 272;
constexpr uint32_t kOffOutEM = kOffX2;  // output staging: [E;M] (32 KB, chunk stride 2048) over the dead P|Q tile,
constexpr uint32_t kOffOutFN = kOffVT;  // [F;N] over V^T and the scratch area
static_assert(kOffSC + kScratchBytes - kOffVT >= kWsTile && kOffVT % 128 == 0, "the [F;N] staging area must fit");

__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(umma::smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ float4 ld4(const unsigned char* base, uint32_t off) {
  return *reinterpret_cast<const float4*>(base + off);
}
__device__ __forceinline__ void st4(unsigned char* base, uint32_t off, float4 v) {
  *reinterpret_cast<float4*>(base + off) = v;
}
__device__ __forceinline__ void st1(unsigned char* base, uint32_t off, float v) {
  *reinterpret_cast<float*>(base + off) = v;
}
// offset of (row, col) in a chunk-major tile
__device__ __forceinline__ uint32_t tile_off(uint32_t cs, int row, int col) {
  return uint32_t(col >> 2) * cs + uint32_t(row) * 16 + uint32_t(col & 3) * 4;
}

// one 128 x N x 64 product: 8 K-steps of tcgen05.mma, A and B chunk-major tiles contracted over their columns
__device__ __forceinline__ void issue_mma(uint32_t d_tmem, uint32_t a_addr, uint32_t a_cs, uint32_t b_addr,
                                          uint32_t b_cs, int n, bool accumulate_first) {
  const uint32_t idesc = umma::idesc_tf32(128, n);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    umma::mma_tf32_ss(d_tmem, umma::desc_k_major(a_addr + ks * 2 * a_cs, a_cs),
                      umma::desc_k_major(b_addr + ks * 2 * b_cs, b_cs), idesc, (ks > 0 || accumulate_first) ? 1u : 0u);
  }
}

__device__ __forceinline__ float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }

// =================================================================================================
// Kernel 1: build [E;M] and [F;N] for every (chunk, head)
// Persistent: each CTA walks (chunk, head) items blockIdx.x, blockIdx.x + gridDim.x, ... so that the
// tensor-memory allocation and the barriers are set up once per SM.  512 threads: the per-item work is a
// chain of short phases separated by barriers, so it is latency- not throughput-bound and wants four
// warps per scheduler.  Thread roles:
//   operand phases : t = tid % 64 (token), part = tid / 64: hsel = part % 2 picks the tensor group
//                    (0: a, b   1: r, k, v), quarter = part / 2 picks 16 of the 64 key channels;
//   epilogues      : warp w reads tensor-memory lanes 32*(w%4).. (row m = 32*(w%4) + lane) and the
//                    32 accumulator columns starting at 32*(w/4).
// =================================================================================================
constexpr int kBuildThreads = 512;

template <typename io_t>
__global__ __launch_bounds__(kBuildThreads, 1) void wkv7_chunk_build_kernel(
    const int* __restrict__ chunk_starts, const int* __restrict__ chunk_ends, const int* __restrict__ metadata_status,
    const io_t* __restrict__ r_ptr, const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr,
    const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr, const io_t* __restrict__ b_ptr,
    const io_t* __restrict__ bias_ptr, unsigned char* __restrict__ workspace, int num_heads, int num_items,
    int* __restrict__ error_flag) {
  using IO = Io16<io_t>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t mbar[4];
  __shared__ uint32_t tmem_holder;
  if (metadata_status != nullptr && metadata_status[0] != 0) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t = tid & 63, part = tid >> 6, hsel = part & 1, quarter = part >> 1;
  const int m = 32 * (warp & 3) + lane;  // accumulator row of this thread
  const int colq = warp >> 2;            // accumulator column quarter of this thread
  const int mt = m & 63;                 // token (rows 0..63) or key channel (rows 64..127) of that row
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) umma::mbar_init(&mbar[i], 1);
    umma::mbar_fence_init();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_holder, 256);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_holder;
  const uint32_t sbase = umma::smem_u32(smem);
  const uint32_t lane_base = uint32_t(32 * (warp & 3)) << 16;
  const uint32_t tcol = uint32_t(t >> 2), tsub = uint32_t(t & 3) * 4;
  bool ok = true;
  bool stores_in_flight = false;  // thread 0 only
  uint32_t parity = 0;

  // Stage the 16-bit token rows of an item in shared memory with cp.async (rows past the end of a short chunk are
  // zero-filled).  The staging slots are the parts of RB / RK / AZ / TT that the item's own operands do not occupy
  // until later phases, so the copies for the NEXT item start as soon as the last product of the current one has
  // completed and overlap its final epilogue.  Slot of the 16-byte piece (token t, key channels 8c..8c+7):
  //   a : RB chunk c, row t        r : RB chunk 8 + c, row t       b : RK chunk c, row t      k : RK chunk 8 + c, row t
  //   v : AZ chunk c, row 64 + t   w : TT region, slot [c][t]
  // Thread i copies piece (t, c) = (i / 8, i % 8) of each tensor: eight consecutive lanes fetch one whole 128-byte
  // row, so a warp's copy instruction is four full-line requests (one piece per lane of 32 different rows would be
  // 32 half-used sector requests, and the request rate, not bandwidth, then bounds the staging).  The consumers
  // read other threads' pieces, behind the barrier that follows the wait.
  auto stage_item = [&](int it) {
    const int ch = it / num_heads, hd = it % num_heads;
    const int tt0 = chunk_starts[ch];
    const int ln = min(max(chunk_ends[ch] - tt0, 1), kL);
    const int st = tid >> 3, sc = tid & 7;
    const uint32_t nbytes = (st < ln) ? 16u : 0u;
    const long long rw = ((long long)(tt0 + min(st, ln - 1)) * num_heads + hd) * kD + 8 * sc;
    umma::cp_async16(sbase + kOffRB + uint32_t(sc) * kCS128P + st * 16, a_ptr + rw, nbytes);
    umma::cp_async16(sbase + kOffRB + uint32_t(8 + sc) * kCS128P + st * 16, r_ptr + rw, nbytes);
    umma::cp_async16(sbase + kOffRK + uint32_t(sc) * kCS128P + st * 16, b_ptr + rw, nbytes);
    umma::cp_async16(sbase + kOffRK + uint32_t(8 + sc) * kCS128P + st * 16, k_ptr + rw, nbytes);
    umma::cp_async16(sbase + kOffAZ + uint32_t(sc) * kCS128P + 1024 + st * 16, v_ptr + rw, nbytes);
    umma::cp_async16(sbase + kOffTT + uint32_t(sc) * 1024 + st * 16, w_ptr + rw, nbytes);
    umma::cp_async_commit();
  };
  if ((int)blockIdx.x < num_items) stage_item(blockIdx.x);

  for (int item = blockIdx.x; item < num_items; item += gridDim.x, parity ^= 1u) {
    const int chunk = item / num_heads, head = item % num_heads;
    const int t0 = chunk_starts[chunk];
    const int len = min(max(chunk_ends[chunk] - t0, 1), kL);
    const bool valid = t < len;

    umma::cp_async_wait_all();  // this thread's share of the staged rows has landed; the barrier below covers the rest
    // the previous item's output tiles leave shared memory by bulk copies: they must have been read before this item
    // overwrites the scratch area (next phase) and the P|Q tile (operand phase)
    if (tid == 0 && stores_in_flight) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    __syncthreads();
    // ---- per-step retention for key channels 8*part .. 8*part+7 -> scratch [kc][t][4] ---------------
    {
      float x[8];
      if (valid) {
        const uint4 u = *reinterpret_cast<const uint4*>(smem + kOffTT + uint32_t(part) * 1024 + t * 16);
        float2 f;
        f = IO::unpack(u.x); x[0] = f.x; x[1] = f.y;
        f = IO::unpack(u.y); x[2] = f.x; x[3] = f.y;
        f = IO::unpack(u.z); x[4] = f.x; x[5] = f.y;
        f = IO::unpack(u.w); x[6] = f.x; x[7] = f.y;
        if (bias_ptr != nullptr) {
          const uint4 bu = __ldg(reinterpret_cast<const uint4*>(bias_ptr + head * kD + 8 * part));
          f = IO::unpack(bu.x); x[0] += f.x; x[1] += f.y;
          f = IO::unpack(bu.y); x[2] += f.x; x[3] += f.y;
          f = IO::unpack(bu.z); x[4] += f.x; x[5] += f.y;
          f = IO::unpack(bu.w); x[6] += f.x; x[7] += f.y;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = retention(x[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = 1.f;
      }
      const uint32_t o = kOffSC + uint32_t(2 * part) * kCS64P + t * 16;
      st4(smem, o, make_float4(x[0], x[1], x[2], x[3]));
      st4(smem, o + kCS64P, make_float4(x[4], x[5], x[6], x[7]));
    }
    __syncthreads();
    // Pull the NEXT item's token rows into L2 now (one 128-byte line per thread: 6 tensors x 64 rows); the cp.async
    // staging at the end of this item then finds them there.  A cp.async that misses L2 holds its issue slot for the
    // whole DRAM round trip, which cost the last phase of every item more than its arithmetic.
    if (tid < 6 * kL && item + (int)gridDim.x < num_items) {
      const int nit = item + gridDim.x, nch = nit / num_heads, nhd = nit % num_heads;
      const int nt0 = chunk_starts[nch];
      const int nln = min(max(chunk_ends[nch] - nt0, 1), kL);
      const int which = tid >> 6, row = tid & 63;
      if (row < nln) {
        const io_t* base = which == 0 ? a_ptr : which == 1 ? r_ptr : which == 2 ? b_ptr : which == 3 ? k_ptr
                                                                       : which == 4 ? v_ptr : w_ptr;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + ((long long)(nt0 + row) * num_heads + nhd) * kD));
      }
    }
    // ---- cumulative decay g_t[k] down each key column: 128 threads, two per column ---------------------
    // (rows 0..31 and 32..63 are scanned separately, then the lower half is scaled by the upper total)
    if (tid < 128) {
      const int kcol = tid & 63, hh = tid >> 6;
      float col[32];
      const uint32_t base = kOffSC + (kcol >> 2) * kCS64P + (kcol & 3) * 4 + uint32_t(32 * hh) * 16;
#pragma unroll
      for (int i = 0; i < 32; ++i) col[i] = *reinterpret_cast<const float*>(smem + base + i * 16);
      float run = 1.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        run *= col[i];
        col[i] = run;
      }
      if (hh == 0) {
#pragma unroll
        for (int i = 0; i < 32; ++i) st1(smem, base + i * 16, col[i]);
      }
      // named barrier over the 128 scanning threads only
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (hh == 1) {
        const float top = *reinterpret_cast<const float*>(smem + base - 16);  // g_31[k]
#pragma unroll
        for (int i = 0; i < 32; ++i) st1(smem, base + i * 16, col[i] * top);
      }
    }
    __syncthreads();
    // ---- operands (one code path for both groups), key channels 16*quarter .. 16*quarter+15 --------------
    //   X1[64*hsel + t] = p * (hsel ? g_t : g_{t-1})      p = a | r
    //   X2[64*hsel + t] = q / g_t                         q = b | k
    //   (RB | RK) rows 64 + k, col t = q / g_t * g_L      (B^^T | K^^T)
    //   group 0: AZ rows k, col t = a * g_{t-1}  (A~^T);  group 1: VT rows v, col t = v
    float diag_gl = 0.f;  // g_L[k] for the threads that later own row k of M
    if (m >= 64) diag_gl = *reinterpret_cast<const float*>(smem + kOffSC + tile_off(kCS64P, 63, mt));
    {
      const uint32_t o3 = (hsel == 0 ? kOffRB : kOffRK) + tcol * kCS128P + tsub + 64 * 16;
      const uint32_t o4 = hsel == 0 ? kOffAZ + tcol * kCS128P + tsub : kOffVT + tcol * kCS64P + tsub;
      const uint32_t oscale = kOffSC + uint32_t(hsel == 0 ? max(t - 1, 0) : t) * 16;
      const bool first_row = (hsel == 0 && t == 0);
      const uint32_t stage01 = uint32_t(8 * hsel) * kCS128P + t * 16;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int kc = 4 * quarter + i;
        const uint32_t so = uint32_t(kc >> 1) * kCS128P + uint32_t(kc & 1) * 8;
        const uint2 u0 = *reinterpret_cast<const uint2*>(smem + kOffRB + stage01 + so);
        const uint2 u1 = *reinterpret_cast<const uint2*>(smem + kOffRK + stage01 + so);
        uint2 u2 = make_uint2(0u, 0u);
        if (hsel == 1) u2 = *reinterpret_cast<const uint2*>(smem + kOffAZ + 1024 + t * 16 + so);
        const float4 g = ld4(smem, kOffSC + kc * kCS64P + t * 16);
        const float4 gl = ld4(smem, kOffSC + kc * kCS64P + 63 * 16);
        float4 sc = ld4(smem, oscale + kc * kCS64P);
        if (first_row) sc = make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 inv = make_float4(rcp_approx(g.x), rcp_approx(g.y), rcp_approx(g.z), rcp_approx(g.w));
        const float2 p01 = IO::unpack(u0.x), p23 = IO::unpack(u0.y);
        const float2 q01 = IO::unpack(u1.x), q23 = IO::unpack(u1.y);
        const float2 v01 = IO::unpack(u2.x), v23 = IO::unpack(u2.y);
        const float4 p = umma::to_tf32(mul4(make_float4(p01.x, p01.y, p23.x, p23.y), sc));
        const float4 q = mul4(make_float4(q01.x, q01.y, q23.x, q23.y), inv);
        const float4 qh = umma::to_tf32(mul4(q, gl));
        const float4 x4 = hsel == 0 ? p : make_float4(v01.x, v01.y, v23.x, v23.y);
        st4(smem, kOffX1 + kc * kCS128 + (64 * hsel + t) * 16, p);
        st4(smem, kOffX2 + kc * kCS128 + (64 * hsel + t) * 16, umma::to_tf32(q));
        const uint32_t a3 = o3 + uint32_t(4 * kc) * 16, a4 = o4 + uint32_t(4 * kc) * 16;
        st1(smem, a3, qh.x); st1(smem, a3 + 16, qh.y); st1(smem, a3 + 32, qh.z); st1(smem, a3 + 48, qh.w);
        st1(smem, a4, x4.x); st1(smem, a4 + 16, x4.y); st1(smem, a4 + 32, x4.z); st1(smem, a4 + 48, x4.w);
      }
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();

    // ---- MMA 1: [A~;R~] [B~;K~]^T  ->  rows t: [A_ab | A_ak], rows 64+t: [A_rb | A_rk] -----------
    if (tid == 0) {
      issue_mma(tmem, sbase + kOffX1, kCS128, sbase + kOffX2, kCS128, 128, false);
      umma::mma_commit(&mbar[0]);
    }
    ok = __all_sync(0xffffffffu, umma::mbar_wait(&mbar[0], parity) && ok) != 0;  // one answer per warp
    umma::fence_after_sync();
    if (ok) {
      uint32_t u[32];
      umma::tmem_ld32(tmem + lane_base + 32 * colq, u);
      umma::tmem_ld_wait();
      const int s0 = 32 * (colq & 1);
      const int limit = (m < 64) ? mt : mt + 1;  // keep s < t (strict) or s <= t
      if (m < 64 && colq < 2) {                  // A_ab -> fp32 scratch for the inverse
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          st4(smem, kOffSC + mt * kAabRow + (s0 + j) * 4,
              make_float4(s0 + j < limit ? __uint_as_float(u[j]) : 0.f,
                          s0 + j + 1 < limit ? __uint_as_float(u[j + 1]) : 0.f,
                          s0 + j + 2 < limit ? __uint_as_float(u[j + 2]) : 0.f,
                          s0 + j + 3 < limit ? __uint_as_float(u[j + 3]) : 0.f));
      } else {
        // A_ak -> X2 region rows t; A_rb -> RB rows t; A_rk -> RK rows t
        const uint32_t base = (m < 64) ? kOffX2 : (colq < 2 ? kOffRB : kOffRK);
        const uint32_t cs = (m < 64) ? kCS128 : kCS128P;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          st4(smem, base + uint32_t((s0 + j) >> 2) * cs + mt * 16,
              umma::to_tf32(make_float4(s0 + j < limit ? __uint_as_float(u[j]) : 0.f,
                                        s0 + j + 1 < limit ? __uint_as_float(u[j + 1]) : 0.f,
                                        s0 + j + 2 < limit ? __uint_as_float(u[j + 2]) : 0.f,
                                        s0 + j + 3 < limit ? __uint_as_float(u[j + 3]) : 0.f)));
      }
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();

    // ---- MMA 2: Z = A_ak V (rows 0..63 of the product; rows 64..127 of the A tile are don't-care) ----
    if (tid == 0) {
      issue_mma(tmem + 128, sbase + kOffX2, kCS128, sbase + kOffVT, kCS64P, 64, false);
      umma::mma_commit(&mbar[1]);
    }
    {
      // T = (I - A_ab)^-1 on the CUDA cores in fp32, by 16 x 16 blocks (all 512 threads).  A_ab is strictly lower
      // triangular, so T is unit lower triangular and
      //   T_ii = (I - A_ii)^-1                                   (16 right-looking steps, one thread per column)
      //   T_ib = T_ii * sum_{k=b..i-1} A_ik T_kb   for i > b      (small products, one block anti-diagonal at a time)
      // T is built unrounded in the TT tile (row t, col s); the inner sums W live in the still unused Z^T half of AZ.
      const auto tt_off = [](int row, int col) { return kOffTT + uint32_t(col >> 2) * kCS64P + uint32_t(row) * 16 + uint32_t(col & 3) * 4; };
      const auto w_off = [](int row, int col) { return kOffAZ + uint32_t(col >> 2) * kCS128P + 1024 + uint32_t(row) * 16 + uint32_t(col & 3) * 4; };
      if (tid < 64) {
        const int blk = tid >> 4, jj = tid & 15;
        const uint32_t ablk = kOffSC + uint32_t(16 * blk) * kAabRow + uint32_t(16 * blk) * 4;
        float acc[16];
#pragma unroll
        for (int rr = 0; rr < 16; ++rr) acc[rr] = 0.f;
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const float xq = acc[q] + (q == jj ? 1.f : 0.f);
          st1(smem, tt_off(16 * blk + q, 16 * blk + jj), xq);
#pragma unroll
          for (int rr = q + 1; rr < 16; ++rr)
            acc[rr] = fmaf(*reinterpret_cast<const float*>(smem + ablk + rr * kAabRow + q * 4), xq, acc[rr]);
        }
      } else {
        // zero the six blocks above the diagonal (1536 elements over 448 threads)
        for (int e = tid - 64; e < 6 * 256; e += kBuildThreads - 64) {
          const int ub = e >> 8, rr = (e >> 4) & 15, cc = e & 15;
          // ub -> (row block, col block) with col block > row block: (0,1)(0,2)(0,3)(1,2)(1,3)(2,3)
          const int rb = ub < 3 ? 0 : (ub < 5 ? 1 : 2);
          const int cb = ub < 3 ? ub + 1 : (ub < 5 ? ub - 1 : 3);
          st1(smem, tt_off(16 * rb + rr, 16 * cb + cc), 0.f);
        }
      }
      __syncthreads();
#pragma unroll 1
      for (int dg = 1; dg < 4; ++dg) {
        const int nblk = 4 - dg;  // blocks (i, b) = (b + dg, b), b = 0 .. nblk-1
        // W_ib = sum_{k=b..i-1} A_ik T_kb
        for (int e = tid; e < nblk * 256; e += kBuildThreads) {
          const int bb = e >> 8, rr = (e >> 4) & 15, cc = e & 15;
          const int ib = bb + dg;
          const uint32_t arow = kOffSC + uint32_t(16 * ib + rr) * kAabRow;
          float acc = 0.f;
          for (int kq = 4 * bb; kq < 4 * ib; ++kq) {  // groups of four columns of A / rows of T
            const float4 a4 = ld4(smem, arow + kq * 16);
            acc = fmaf(a4.x, *reinterpret_cast<const float*>(smem + tt_off(4 * kq + 0, 16 * bb + cc)), acc);
            acc = fmaf(a4.y, *reinterpret_cast<const float*>(smem + tt_off(4 * kq + 1, 16 * bb + cc)), acc);
            acc = fmaf(a4.z, *reinterpret_cast<const float*>(smem + tt_off(4 * kq + 2, 16 * bb + cc)), acc);
            acc = fmaf(a4.w, *reinterpret_cast<const float*>(smem + tt_off(4 * kq + 3, 16 * bb + cc)), acc);
          }
          st1(smem, w_off(16 * ib + rr, 16 * bb + cc), acc);
        }
        __syncthreads();
        // T_ib = T_ii W_ib
        for (int e = tid; e < nblk * 256; e += kBuildThreads) {
          const int bb = e >> 8, rr = (e >> 4) & 15, cc = e & 15;
          const int ib = bb + dg;
          float acc = 0.f;
#pragma unroll
          for (int q = 0; q < 16; ++q)
            acc = fmaf(*reinterpret_cast<const float*>(smem + tt_off(16 * ib + rr, 16 * ib + q)),
                       *reinterpret_cast<const float*>(smem + w_off(16 * ib + q, 16 * bb + cc)), acc);
          st1(smem, tt_off(16 * ib + rr, 16 * bb + cc), acc);
        }
        __syncthreads();
      }
      // the tensor core truncates: round T to tf32 (eight elements per thread)
      {
        const int row = tid & 63, c0 = (tid >> 6) * 8;
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          const uint32_t o = tt_off(row, c0 + cc);
          st1(smem, o, umma::to_tf32(*reinterpret_cast<const float*>(smem + o)));
        }
      }
    }
    if (m < 64 && colq < 2) {
      // warps 0, 1, 4, 5: Z^T -> AZ rows 64 + v, col t (32 value columns per warp)
      ok = __all_sync(0xffffffffu, umma::mbar_wait(&mbar[1], parity) && ok) != 0;  // one answer per warp
      umma::fence_after_sync();
      if (ok) {
        const uint32_t o = kOffAZ + uint32_t(mt >> 2) * kCS128P + uint32_t(mt & 3) * 4 + 64 * 16;
        uint32_t u[32];
        umma::tmem_ld32(tmem + 128 + lane_base + 32 * colq, u);
        umma::tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < 32; ++jj)
          st1(smem, o + (32 * colq + jj) * 16, umma::to_tf32(__uint_as_float(u[jj])));
      }
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();

    // ---- MMA 3: [A~^T ; Z^T] T^T -> rows j: P[.][j] (j < 64) and Q[.][j-64], columns t -------------
    if (tid == 0) {
      issue_mma(tmem + 192, sbase + kOffAZ, kCS128P, sbase + kOffTT, kCS64P, 64, false);
      umma::mma_commit(&mbar[2]);
    }
    ok = __all_sync(0xffffffffu, umma::mbar_wait(&mbar[2], parity) && ok) != 0;  // one answer per warp
    umma::fence_after_sync();
    if (ok && colq < 2) {  // warps 0..7, 32 of the 64 columns each
      uint32_t u[32];
      umma::tmem_ld32(tmem + 192 + lane_base + 32 * colq, u);
      umma::tmem_ld_wait();
#pragma unroll
      for (int jj = 0; jj < 32; jj += 4)
        st4(smem, kOffX2 + uint32_t((32 * colq + jj) >> 2) * kCS128 + m * 16,
            umma::to_tf32(make_float4(__uint_as_float(u[jj]), __uint_as_float(u[jj + 1]),
                                      __uint_as_float(u[jj + 2]), __uint_as_float(u[jj + 3]))));
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();

    // ---- MMA 4 + 5: [A_rb ; B^^T] [P|Q]  (+)  [A_rk ; K^^T] V into columns 64..127 ------------------
    if (tid == 0) {
      issue_mma(tmem, sbase + kOffRB, kCS128P, sbase + kOffX2, kCS128, 128, false);
      issue_mma(tmem + 64, sbase + kOffRK, kCS128P, sbase + kOffVT, kCS64P, 64, true);
      umma::mma_commit(&mbar[3]);
    }
    ok = __all_sync(0xffffffffu, umma::mbar_wait(&mbar[3], parity) && ok) != 0;  // one answer per warp
    umma::fence_after_sync();
    if (ok && item + (int)gridDim.x < num_items) stage_item(item + gridDim.x);
    if (ok) {
      // [E;M] and [F;N] are laid down in shared memory exactly as the workspace wants them ([E;M] over the P|Q tile,
      // [F;N] over V^T and the scratch area, all dead by now) and leave with two bulk copies that drain while the
      // next item starts.
      uint32_t u[32];
      umma::tmem_ld32(tmem + lane_base + 32 * colq, u);
      umma::tmem_ld_wait();
      const int cb = 32 * (colq & 1);
      if (colq < 2) {
#pragma unroll
        for (int jj = 0; jj < 32; jj += 4) {
          float4 val = make_float4(__uint_as_float(u[jj]), __uint_as_float(u[jj + 1]), __uint_as_float(u[jj + 2]),
                                   __uint_as_float(u[jj + 3]));
          const int c = cb + jj;
          if (m < 64) {  // E = R~ + A_rb P
            const float4 rt = ld4(smem, kOffX1 + uint32_t(c >> 2) * kCS128 + (64 + mt) * 16);
            val.x += rt.x; val.y += rt.y; val.z += rt.z; val.w += rt.w;
          } else {       // M = diag(g_L) + B^^T P
            val.x += (mt == c) ? diag_gl : 0.f;
            val.y += (mt == c + 1) ? diag_gl : 0.f;
            val.z += (mt == c + 2) ? diag_gl : 0.f;
            val.w += (mt == c + 3) ? diag_gl : 0.f;
          }
          st4(smem, kOffOutEM + uint32_t(c >> 2) * kCS128 + m * 16, umma::to_tf32(val));
        }
      } else {
#pragma unroll
        for (int jj = 0; jj < 32; jj += 4)
          st4(smem, kOffOutFN + uint32_t((cb + jj) >> 2) * kCS128 + m * 16,
              make_float4(__uint_as_float(u[jj]), __uint_as_float(u[jj + 1]), __uint_as_float(u[jj + 2]),
                          __uint_as_float(u[jj + 3])));
      }
    }
    // every thread is done with this item's shared memory and accumulators before the next item starts
    umma::fence_async_smem();
    umma::fence_before_sync();
    ok = __syncthreads_and(ok) != 0;
    umma::fence_after_sync();
    if (!ok) break;
    if (tid == 0) {
      unsigned char* ws = workspace + (size_t)item * (2 * kWsTile);
      bulk_s2g(ws, smem + kOffOutEM, kWsTile);
      bulk_s2g(ws + kWsTile, smem + kOffOutFN, kWsTile);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      stores_in_flight = true;
    }
  }
  if (!ok && tid == 0 && error_flag != nullptr) atomicExch(error_flag, 1);
  if (tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // output tiles are out before shared memory goes
  umma::cp_async_wait_all();
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, 256);
}

// =================================================================================================
// Kernel 2: scan the chunks of one (sequence, head):  [Y; S'] = [E;M] S + [F;N]
// =================================================================================================
constexpr uint32_t kScanStage = 2 * kWsTile;             // [E;M] then [F;N]
constexpr uint32_t kScanOffST = 2 * kScanStage;          // S^T (rows v, cols k), stride 1040
constexpr uint32_t kScanSmem = kScanOffST + 16 * kCS64P; // 147,712 bytes

template <typename io_t>
__global__ __launch_bounds__(128, 1) void wkv7_chunk_scan_kernel(
    const int* __restrict__ seq_chunk_offsets, const int* __restrict__ chunk_starts, const int* __restrict__ chunk_ends,
    const int* __restrict__ state_indices, const int* __restrict__ metadata_status, float* __restrict__ state_pool,
    const unsigned char* __restrict__ workspace, io_t* __restrict__ y_ptr, float* __restrict__ y32_ptr,
    float* __restrict__ boundary, int num_heads, long long output_elements, float scale, int* __restrict__ error_flag) {
  using IO = Io16<io_t>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full_bar[2];
  __shared__ uint64_t mma_bar;
  __shared__ uint32_t tmem_holder;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (metadata_status != nullptr && metadata_status[0] != 0) {
    const io_t nan16 = IO::store(quiet_nan());
    for (long long i = (long long)blockIdx.x * 128 + tid; i < output_elements; i += (long long)gridDim.x * 128) {
      y_ptr[i] = nan16;
      if (y32_ptr != nullptr) y32_ptr[i] = quiet_nan();
    }
    return;
  }
  const int seq = blockIdx.x / num_heads, head = blockIdx.x % num_heads;
  const int c_begin = seq_chunk_offsets[seq], c_end = seq_chunk_offsets[seq + 1];
  const int slot = state_indices != nullptr ? state_indices[seq] : seq;
  float* state = state_pool + ((long long)slot * num_heads + head) * (kD * kD);

  if (tid == 0) {
    umma::mbar_init(&full_bar[0], 1);
    umma::mbar_init(&full_bar[1], 1);
    umma::mbar_init(&mma_bar, 1);
    umma::mbar_fence_init();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_holder, 128);
  __syncthreads();
  if (tid == 0) {
    for (int i = 0; i < 2 && c_begin + i < c_end; ++i) {
      const unsigned char* src = workspace + ((size_t)(c_begin + i) * num_heads + head) * kScanStage;
      umma::mbar_expect_tx(&full_bar[i], kScanStage);
      umma::bulk_g2s(smem + i * kScanStage, src, kScanStage, &full_bar[i]);
    }
  }
  // initial state: thread 64 + k owns key row k
  if (tid >= 64) {
    const int kk = tid - 64;
    const uint32_t o = kScanOffST + uint32_t(kk >> 2) * kCS64P + uint32_t(kk & 3) * 4;
    float* bnd = boundary != nullptr && c_begin < c_end
                     ? boundary + ((long long)c_begin * num_heads + head) * (kD * kD) + kk * kD
                     : nullptr;
#pragma unroll
    for (int v4 = 0; v4 < 16; ++v4) {
      const float4 s = *reinterpret_cast<const float4*>(state + kk * kD + 4 * v4);
      if (bnd != nullptr) *reinterpret_cast<float4*>(bnd + 4 * v4) = s;
      st1(smem, o + (4 * v4 + 0) * 16, umma::to_tf32(s.x));
      st1(smem, o + (4 * v4 + 1) * 16, umma::to_tf32(s.y));
      st1(smem, o + (4 * v4 + 2) * 16, umma::to_tf32(s.z));
      st1(smem, o + (4 * v4 + 3) * 16, umma::to_tf32(s.w));
    }
  }
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_holder;
  const uint32_t sbase = umma::smem_u32(smem);
  const uint32_t lane_base = uint32_t(warp * 32) << 16;
  bool ok = true;

  for (int c = c_begin; c < c_end && ok; ++c) {
    const int it = c - c_begin, stage = it & 1;
    const uint32_t acc = tmem + 64 * stage;
    unsigned char* st = smem + stage * kScanStage;
    // one verdict for the whole CTA on every wait: nobody runs on alone into the barriers and tensor-memory loads below
    ok = __syncthreads_and(umma::mbar_wait(&full_bar[stage], (it >> 1) & 1) ? 1 : 0) != 0;
    if (!ok) break;
    if (tid == 0) {
      umma::fence_after_sync();
      issue_mma(acc, sbase + stage * kScanStage, kCS128, sbase + kScanOffST, kCS64P, 64, false);
      umma::mma_commit(&mma_bar);
    }
    ok = __syncthreads_and(umma::mbar_wait(&mma_bar, it & 1) ? 1 : 0) != 0;
    umma::fence_after_sync();
    if (!ok) break;
    const int t0 = chunk_starts[c];
    const int len = min(max(chunk_ends[c] - t0, 0), kL);
    if (tid >= 64) {
      // rows 64..127 of the product: S' = M S + N, this thread owns key row kk
      const int kk = tid - 64;
      const bool last = (c + 1 == c_end);
      float* dst = last ? state + kk * kD
                        : (boundary != nullptr ? boundary + ((long long)(c + 1) * num_heads + head) * (kD * kD) + kk * kD
                                               : nullptr);
      const uint32_t o = kScanOffST + uint32_t(kk >> 2) * kCS64P + uint32_t(kk & 3) * 4;
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t u[32];
        umma::tmem_ld32(acc + lane_base + c0, u);
        umma::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 n4 = ld4(st, kWsTile + uint32_t((c0 + j) >> 2) * kCS128 + tid * 16);
          const float4 s = make_float4(__uint_as_float(u[j]) + n4.x, __uint_as_float(u[j + 1]) + n4.y,
                                       __uint_as_float(u[j + 2]) + n4.z, __uint_as_float(u[j + 3]) + n4.w);
          if (dst != nullptr) *reinterpret_cast<float4*>(dst + c0 + j) = s;
          if (!last) {
            st1(smem, o + (c0 + j + 0) * 16, umma::to_tf32(s.x));
            st1(smem, o + (c0 + j + 1) * 16, umma::to_tf32(s.y));
            st1(smem, o + (c0 + j + 2) * 16, umma::to_tf32(s.z));
            st1(smem, o + (c0 + j + 3) * 16, umma::to_tf32(s.w));
          }
        }
      }
    } else {
      // rows 0..63: Y = scale * (E S + F), this thread owns token t
      const int t = tid;
      const long long row = ((long long)(t0 + t) * num_heads + head) * kD;
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t u[32];
        umma::tmem_ld32(acc + lane_base + c0, u);
        umma::tmem_ld_wait();
        if (t < len) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            const float4 f0 = ld4(st, kWsTile + uint32_t((c0 + j) >> 2) * kCS128 + tid * 16);
            const float4 f1 = ld4(st, kWsTile + uint32_t((c0 + j + 4) >> 2) * kCS128 + tid * 16);
            float o[8];
            o[0] = scale * (__uint_as_float(u[j + 0]) + f0.x); o[1] = scale * (__uint_as_float(u[j + 1]) + f0.y);
            o[2] = scale * (__uint_as_float(u[j + 2]) + f0.z); o[3] = scale * (__uint_as_float(u[j + 3]) + f0.w);
            o[4] = scale * (__uint_as_float(u[j + 4]) + f1.x); o[5] = scale * (__uint_as_float(u[j + 5]) + f1.y);
            o[6] = scale * (__uint_as_float(u[j + 6]) + f1.z); o[7] = scale * (__uint_as_float(u[j + 7]) + f1.w);
            uint4 packed;
            packed.x = IO::pack(o[0], o[1]); packed.y = IO::pack(o[2], o[3]);
            packed.z = IO::pack(o[4], o[5]); packed.w = IO::pack(o[6], o[7]);
            *reinterpret_cast<uint4*>(y_ptr + row + c0 + j) = packed;
            if (y32_ptr != nullptr) {
              *reinterpret_cast<float4*>(y32_ptr + row + c0 + j) = make_float4(o[0], o[1], o[2], o[3]);
              *reinterpret_cast<float4*>(y32_ptr + row + c0 + j + 4) = make_float4(o[4], o[5], o[6], o[7]);
            }
          }
        }
      }
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // this stage's tiles are consumed: refill it with the chunk after next
    if (tid == 0 && c + 2 < c_end) {
      const unsigned char* src = workspace + ((size_t)(c + 2) * num_heads + head) * kScanStage;
      umma::mbar_expect_tx(&full_bar[stage], kScanStage);
      umma::bulk_g2s(st, src, kScanStage, &full_bar[stage]);
    }
  }
  if (!ok) {
    // fail closed: the rows of this (sequence, head) read as NaN; copies and products that may still be in flight get
    // time to land before the shared and tensor memory go away
    if (tid == 0 && error_flag != nullptr) atomicExch(error_flag, 2);
    const io_t nan16 = IO::store(quiet_nan());
    const int tb = chunk_starts[c_begin], te = chunk_ends[c_end - 1];
    for (long long e = (long long)tb * kD + tid; e < (long long)te * kD; e += blockDim.x) {
      const long long at = ((e / kD) * num_heads + head) * kD + (e % kD);
      y_ptr[at] = nan16;
      if (y32_ptr != nullptr) y32_ptr[at] = quiet_nan();
    }
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, 128);
}

template <typename io_t>
int launch_chunk_forward(const int* seq_chunk_offsets, const int* chunk_starts, const int* chunk_ends,
                         const int* state_indices, const int* status, float* state_pool, const void* r, const void* w,
                         const void* k, const void* v, const void* a, const void* b, const void* bias, void* y,
                         float* y32, float* boundary, void* workspace, int* error_flag, int total_tokens,
                         int num_sequences, int num_chunks, int num_heads, float scale, cudaStream_t stream) {
  // the shared-memory opt-in and the SM count are looked up once per device and instantiation, not on every call
  static bool opted_in[64] = {};
  static int sm_counts[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
    return fail(FRWKV_ERR_CUDA, "wkv7_chunk_forward: cannot identify the current device");
  if (!opted_in[device]) {
    cudaError_t e1 = cudaFuncSetAttribute(wkv7_chunk_build_kernel<io_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)kBuildSmem);
    cudaError_t e2 = cudaFuncSetAttribute(wkv7_chunk_scan_kernel<io_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)kScanSmem);
    if (e1 != cudaSuccess || e2 != cudaSuccess)
      return fail(FRWKV_ERR_CUDA, "wkv7_chunk_forward: cannot reserve shared memory: %s",
                  cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    cudaDeviceGetAttribute(&sm_counts[device], cudaDevAttrMultiProcessorCount, device);
    opted_in[device] = true;
  }
  const int sm_count = sm_counts[device];
  const int num_items = num_chunks * num_heads;
  const int build_grid = sm_count > 0 && sm_count < num_items ? sm_count : num_items;
  wkv7_chunk_build_kernel<io_t><<<(unsigned)build_grid, kBuildThreads, kBuildSmem, stream>>>(
      chunk_starts, chunk_ends, status, static_cast<const io_t*>(r), static_cast<const io_t*>(w),
      static_cast<const io_t*>(k), static_cast<const io_t*>(v), static_cast<const io_t*>(a),
      static_cast<const io_t*>(b), static_cast<const io_t*>(bias), static_cast<unsigned char*>(workspace), num_heads,
      num_items, error_flag);
  int rc = check_launch("wkv7_chunk_build_kernel");
  if (rc != FRWKV_OK) return rc;
  wkv7_chunk_scan_kernel<io_t><<<(unsigned)(num_sequences * num_heads), 128, kScanSmem, stream>>>(
      seq_chunk_offsets, chunk_starts, chunk_ends, state_indices, status, state_pool,
      static_cast<const unsigned char*>(workspace), static_cast<io_t*>(y), y32, boundary, num_heads,
      (long long)total_tokens * num_heads * kD, scale, error_flag);
  return check_launch("wkv7_chunk_scan_kernel");
}

}  // namespace
}  // namespace frwkv

extern "C" size_t frwkv_wkv7_chunk_workspace_bytes(int num_chunks, int num_heads) {
  if (num_chunks <= 0 || num_heads <= 0) return 0;
  return (size_t)num_chunks * (size_t)num_heads * (size_t)(2 * frwkv::kWsTile);
}

extern "C" int frwkv_wkv7_chunk_fp32io16_forward(
    const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends,
    const int32_t* state_indices, const int32_t* metadata_status, float* state_pool, const void* r,
    const void* decay_logits, const void* k, const void* v, const void* a, const void* b, const void* decay_bias,
    void* y, float* y_fp32, float* boundary, void* workspace, size_t workspace_bytes, int32_t* error_flag,
    int total_tokens, int num_sequences, int num_chunks, int num_heads, int head_size, int io_dtype, float scale,
    frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(seq_chunk_offsets && chunk_starts && chunk_ends && state_pool && r && decay_logits && k && v && a &&
                    b && y && workspace,
                "wkv7_chunk_forward: null pointer argument");
  FRWKV_REQUIRE(total_tokens > 0 && num_sequences > 0 && num_chunks > 0 && num_heads > 0,
                "wkv7_chunk_forward: sizes must be positive");
  if (head_size != 64) return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_chunk_forward: head size %d is not built (only 64)", head_size);
  FRWKV_REQUIRE(workspace_bytes >= frwkv_wkv7_chunk_workspace_bytes(num_chunks, num_heads),
                "wkv7_chunk_forward: workspace too small (%zu bytes given)", workspace_bytes);
  FRWKV_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 127) == 0, "wkv7_chunk_forward: workspace must be 128-byte aligned");
  FRWKV_REQUIRE((long long)num_chunks * num_heads <= 0x7fffffffLL, "wkv7_chunk_forward: too many (chunk, head) pairs");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_chunk_forward<__nv_bfloat16>(seq_chunk_offsets, chunk_starts, chunk_ends, state_indices,
                                               metadata_status, state_pool, r, decay_logits, k, v, a, b, decay_bias, y,
                                               y_fp32, boundary, workspace, error_flag, total_tokens, num_sequences,
                                               num_chunks, num_heads, scale, s);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_chunk_forward<__half>(seq_chunk_offsets, chunk_starts, chunk_ends, state_indices, metadata_status,
                                        state_pool, r, decay_logits, k, v, a, b, decay_bias, y, y_fp32, boundary,
                                        workspace, error_flag, total_tokens, num_sequences, num_chunks, num_heads,
                                        scale, s);
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_chunk_forward: token tensors must be float16 or bfloat16");
}

// ---------------------------------------------------------------------------------------------------------
// Chunked forward for callers that must not allocate device memory.
//
// Some hosts hand the whole device to fixed pools when they start (state pools, activation arenas) and forbid
// any later cudaMalloc: an inference server that has sized its pools to the last megabyte, a real-time loop in
// which an allocation could stall the device, a plain C host with no caching allocator behind it.  For them the
// [E;M] / [F;N] workspace of the build and scan kernels lives in a fixed array inside this library instead of in
// memory the caller provides.  The array costs kNoAllocBytes on every GPU that loads the library, for the life
// of the process, so it is kept modest: it covers kNoAllocMaxItems (chunk, head) pairs per call, e.g. 256 tokens
// of 64 heads, or 1024 tokens of 16 heads.
//
// The array name is only a handle on the host side; the device address comes from cudaGetSymbolAddress, looked
// up once per device (on the first call made with that device current - do that first call outside any stream
// capture) and cached.  Every call uses the same array: two calls whose kernels overlap on the GPU (different
// streams) would overwrite each other's tiles, so callers must order them.  Nothing in the array has to start at
// zero - the build kernel writes every tile before the scan kernel reads it - so the contents left by the
// previous call are harmless.
// ---------------------------------------------------------------------------------------------------------
namespace frwkv {
namespace {
constexpr int kNoAllocMaxItems = 256;
constexpr size_t kNoAllocBytes = (size_t)kNoAllocMaxItems * 2 * kWsTile;  // 16 MiB
constexpr int kNoAllocMaxDevices = 64;
}  // namespace
}  // namespace frwkv

static __device__ __align__(256) unsigned char g_noalloc_workspace[frwkv::kNoAllocBytes];

static void* noalloc_workspace_for_current_device(int* status) {
  static void* cached[frwkv::kNoAllocMaxDevices] = {};
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= frwkv::kNoAllocMaxDevices) {
    *status = frwkv::fail(FRWKV_ERR_CUDA, "wkv7_chunk_forward_noalloc: cannot identify the current device");
    return nullptr;
  }
  void* ptr = __atomic_load_n(&cached[device], __ATOMIC_ACQUIRE);
  if (ptr == nullptr) {
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_noalloc_workspace);
    if (err != cudaSuccess || ptr == nullptr) {
      *status = frwkv::fail(FRWKV_ERR_CUDA, "wkv7_chunk_forward_noalloc: cudaGetSymbolAddress failed: %s",
                            cudaGetErrorString(err));
      return nullptr;
    }
    __atomic_store_n(&cached[device], ptr, __ATOMIC_RELEASE);  // racing first calls store the same address
  }
  return ptr;
}

extern "C" size_t frwkv_wkv7_chunk_noalloc_max_items(void) { return (size_t)frwkv::kNoAllocMaxItems; }

extern "C" int frwkv_wkv7_chunk_fp32io16_forward_noalloc(
    const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends,
    const int32_t* state_indices, const int32_t* metadata_status, float* state_pool, const void* r,
    const void* decay_logits, const void* k, const void* v, const void* a, const void* b, const void* decay_bias,
    void* y, float* y_fp32, float* boundary, int32_t* error_flag, int total_tokens, int num_sequences, int num_chunks,
    int num_heads, int head_size, int io_dtype, float scale, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(num_chunks > 0 && num_heads > 0, "wkv7_chunk_forward_noalloc: sizes must be positive");
  FRWKV_REQUIRE((long long)num_chunks * num_heads <= kNoAllocMaxItems,
                "wkv7_chunk_forward_noalloc: %d chunks x %d heads exceeds the built-in workspace of %d (chunk, head) "
                "pairs; split the batch or use frwkv_wkv7_chunk_fp32io16_forward with your own workspace",
                num_chunks, num_heads, kNoAllocMaxItems);
  int status = FRWKV_OK;
  void* workspace = noalloc_workspace_for_current_device(&status);
  if (workspace == nullptr) return status;
  return frwkv_wkv7_chunk_fp32io16_forward(seq_chunk_offsets, chunk_starts, chunk_ends, state_indices, metadata_status,
                                           state_pool, r, decay_logits, k, v, a, b, decay_bias, y, y_fp32, boundary,
                                           workspace, kNoAllocBytes, error_flag, total_tokens, num_sequences,
                                           num_chunks, num_heads, head_size, io_dtype, scale, stream);
}
