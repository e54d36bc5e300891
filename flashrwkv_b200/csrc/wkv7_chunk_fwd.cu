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
// Kernel 1 (build, one CTA per (chunk, head), all chunks in parallel) forms [E;M] and [F;N] with five
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

template <typename io_t>
__device__ __forceinline__ void load_row_half(const io_t* p, bool valid, float (&out)[32]) {
  // 32 consecutive 16-bit values (64 bytes) -> fp32
  using IO = Io16<io_t>;
  if (valid) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 u = __ldg(q + i);
      float2 f;
      f = IO::unpack(u.x); out[8 * i + 0] = f.x; out[8 * i + 1] = f.y;
      f = IO::unpack(u.y); out[8 * i + 2] = f.x; out[8 * i + 3] = f.y;
      f = IO::unpack(u.z); out[8 * i + 4] = f.x; out[8 * i + 5] = f.y;
      f = IO::unpack(u.w); out[8 * i + 6] = f.x; out[8 * i + 7] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) out[i] = 0.f;
  }
}

template <typename io_t>
__device__ __forceinline__ void load_row_raw(const io_t* p, bool valid, uint32_t (&out)[32]) {
  // 64 consecutive 16-bit values kept packed (two per register)
  if (valid) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 u = __ldg(q + i);
      out[4 * i] = u.x; out[4 * i + 1] = u.y; out[4 * i + 2] = u.z; out[4 * i + 3] = u.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) out[i] = 0u;
  }
}

template <typename io_t>
__device__ __forceinline__ float4 unpack4(const uint32_t (&raw)[32], int kc) {
  using IO = Io16<io_t>;
  const float2 lo = IO::unpack(raw[2 * kc]), hi = IO::unpack(raw[2 * kc + 1]);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

__device__ __forceinline__ float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }

// =================================================================================================
// Kernel 1: build [E;M] and [F;N] for every (chunk, head)
// =================================================================================================
template <typename io_t>
__global__ __launch_bounds__(128, 1) void wkv7_chunk_build_kernel(
    const int* __restrict__ chunk_starts, const int* __restrict__ chunk_ends, const int* __restrict__ metadata_status,
    const io_t* __restrict__ r_ptr, const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr,
    const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr, const io_t* __restrict__ b_ptr,
    const io_t* __restrict__ bias_ptr, unsigned char* __restrict__ workspace, int num_heads,
    int* __restrict__ error_flag) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t mbar[4];
  __shared__ uint32_t tmem_holder;
  if (metadata_status != nullptr && metadata_status[0] != 0) return;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int t = tid & 63, hsel = tid >> 6;
  const int chunk = blockIdx.x / num_heads, head = blockIdx.x % num_heads;
  const int t0 = chunk_starts[chunk];
  const int len = min(max(chunk_ends[chunk] - t0, 0), kL);
  const bool valid = t < len;
  const long long row = ((long long)(t0 + t) * num_heads + head) * kD;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) umma::mbar_init(&mbar[i], 1);
    umma::mbar_fence_init();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_holder, 256);

  // ---- issue the token loads early: group 0 owns a and b, group 1 owns r, k and v ---------------
  uint32_t raw0[32], raw1[32], raw2[32];
  if (hsel == 0) {
    load_row_raw(a_ptr + row, valid, raw0);
    load_row_raw(b_ptr + row, valid, raw1);
  } else {
    load_row_raw(r_ptr + row, valid, raw0);
    load_row_raw(k_ptr + row, valid, raw1);
    load_row_raw(v_ptr + row, valid, raw2);
  }
  // ---- per-step retention for this thread's half of the key channels ---------------------------
  {
    float x[32];
    load_row_half(w_ptr + row + 32 * hsel, valid, x);
    if (bias_ptr != nullptr) {
      float bx[32];
      load_row_half(bias_ptr + head * kD + 32 * hsel, true, bx);
#pragma unroll
      for (int i = 0; i < 32; ++i) x[i] += bx[i];
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float4 w4;
      w4.x = valid ? retention(x[4 * c]) : 1.f;
      w4.y = valid ? retention(x[4 * c + 1]) : 1.f;
      w4.z = valid ? retention(x[4 * c + 2]) : 1.f;
      w4.w = valid ? retention(x[4 * c + 3]) : 1.f;
      st4(smem, kOffSC + (8 * hsel + c) * kCS64P + t * 16, w4);
    }
  }
  __syncthreads();
  // ---- cumulative decay g_t[k] down each key column (threads 0..63 own one column each) ---------
  if (tid < 64) {
    float col[64];
    const uint32_t base = kOffSC + (tid >> 2) * kCS64P + (tid & 3) * 4;
#pragma unroll
    for (int i = 0; i < 64; ++i) col[i] = *reinterpret_cast<const float*>(smem + base + i * 16);
    float run = 1.f;
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      run *= col[i];
      st1(smem, base + i * 16, run);
    }
  }
  __syncthreads();
  // ---- operands -------------------------------------------------------------------------------
  float diag_gl = 0.f;  // g_L[k] for the thread that later owns row k of M
  if (tid >= 64) diag_gl = *reinterpret_cast<const float*>(smem + kOffSC + tile_off(kCS64P, 63, tid - 64));
#pragma unroll
  for (int kc = 0; kc < 16; ++kc) {
    const float4 g = ld4(smem, kOffSC + kc * kCS64P + t * 16);
    const float4 gl = ld4(smem, kOffSC + kc * kCS64P + 63 * 16);
    const float4 inv = make_float4(__frcp_rn(g.x), __frcp_rn(g.y), __frcp_rn(g.z), __frcp_rn(g.w));
    const uint32_t tcol = uint32_t(t >> 2), tsub = uint32_t(t & 3) * 4;
    if (hsel == 0) {
      float4 gp = make_float4(1.f, 1.f, 1.f, 1.f);
      if (t > 0) gp = ld4(smem, kOffSC + kc * kCS64P + (t - 1) * 16);
      const float4 at = umma::to_tf32(mul4(unpack4<io_t>(raw0, kc), gp));
      const float4 bt = mul4(unpack4<io_t>(raw1, kc), inv);
      const float4 bh = umma::to_tf32(mul4(bt, gl));
      st4(smem, kOffX1 + kc * kCS128 + t * 16, at);
      st4(smem, kOffX2 + kc * kCS128 + t * 16, umma::to_tf32(bt));
      // A~^T (rows k, col t) and B^^T (rows 64 + k, col t)
      const uint32_t oa = kOffAZ + tcol * kCS128P + tsub + uint32_t(4 * kc) * 16;
      st1(smem, oa, at.x); st1(smem, oa + 16, at.y); st1(smem, oa + 32, at.z); st1(smem, oa + 48, at.w);
      const uint32_t ob = kOffRB + tcol * kCS128P + tsub + uint32_t(64 + 4 * kc) * 16;
      st1(smem, ob, bh.x); st1(smem, ob + 16, bh.y); st1(smem, ob + 32, bh.z); st1(smem, ob + 48, bh.w);
    } else {
      const float4 rt = umma::to_tf32(mul4(unpack4<io_t>(raw0, kc), g));
      const float4 kt = mul4(unpack4<io_t>(raw1, kc), inv);
      const float4 kh = umma::to_tf32(mul4(kt, gl));
      const float4 vv = unpack4<io_t>(raw2, kc);
      st4(smem, kOffX1 + kc * kCS128 + (64 + t) * 16, rt);
      st4(smem, kOffX2 + kc * kCS128 + (64 + t) * 16, umma::to_tf32(kt));
      const uint32_t ok = kOffRK + tcol * kCS128P + tsub + uint32_t(64 + 4 * kc) * 16;
      st1(smem, ok, kh.x); st1(smem, ok + 16, kh.y); st1(smem, ok + 32, kh.z); st1(smem, ok + 48, kh.w);
      const uint32_t ov = kOffVT + tcol * kCS64P + tsub + uint32_t(4 * kc) * 16;
      st1(smem, ov, vv.x); st1(smem, ov + 16, vv.y); st1(smem, ov + 32, vv.z); st1(smem, ov + 48, vv.w);
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

  // ---- MMA 1: [A~;R~] [B~;K~]^T  ->  rows t: [A_ab | A_ak], rows 64+t: [A_rb | A_rk] -----------
  if (tid == 0) {
    issue_mma(tmem, sbase + kOffX1, kCS128, sbase + kOffX2, kCS128, 128, false);
    umma::mma_commit(&mbar[0]);
  }
  ok = umma::mbar_wait(&mbar[0], 0) && ok;
  umma::fence_after_sync();
  if (ok) {
#pragma unroll
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t u[32];
      umma::tmem_ld32(tmem + lane_base + c0, u);
      umma::tmem_ld_wait();
      const int s0 = c0 & 63;
      float f[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int s = s0 + j;
        const bool keep = (tid < 64) ? (s < t) : (s <= t);
        f[j] = keep ? __uint_as_float(u[j]) : 0.f;
      }
      if (tid < 64 && c0 < 64) {  // A_ab -> fp32 scratch for the inverse
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          st4(smem, kOffSC + t * kAabRow + (s0 + j) * 4, make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]));
      } else {
        // A_ak -> X2 region rows t; A_rb -> RB rows t; A_rk -> RK rows t
        const uint32_t base = (tid < 64) ? kOffX2 : (c0 < 64 ? kOffRB : kOffRK);
        const uint32_t cs = (tid < 64) ? kCS128 : kCS128P;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          st4(smem, base + uint32_t((s0 + j) >> 2) * cs + t * 16,
              umma::to_tf32(make_float4(f[j], f[j + 1], f[j + 2], f[j + 3])));
      }
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
  if (tid >= 64) {
    // T = (I - A_ab)^-1, one column per thread: T[t][j] = [t == j] + sum_{s<t} A_ab[t][s] T[s][j]
    const int j = tid - 64;
    float col[64];
#pragma unroll
    for (int tt = 0; tt < 64; ++tt) {
      float acc0 = (tt == j) ? 1.f : 0.f, acc1 = 0.f;
#pragma unroll
      for (int s4 = 0; s4 < (tt + 3) / 4; ++s4) {
        const float4 a4 = ld4(smem, kOffSC + tt * kAabRow + s4 * 16);
        if (4 * s4 + 0 < tt) acc0 = fmaf(a4.x, col[4 * s4 + 0], acc0);
        if (4 * s4 + 1 < tt) acc1 = fmaf(a4.y, col[4 * s4 + 1], acc1);
        if (4 * s4 + 2 < tt) acc0 = fmaf(a4.z, col[4 * s4 + 2], acc0);
        if (4 * s4 + 3 < tt) acc1 = fmaf(a4.w, col[4 * s4 + 3], acc1);
      }
      col[tt] = acc0 + acc1;
    }
    const uint32_t o = kOffTT + uint32_t(j >> 2) * kCS64P + uint32_t(j & 3) * 4;
#pragma unroll
    for (int tt = 0; tt < 64; ++tt) st1(smem, o + tt * 16, umma::to_tf32(col[tt]));
  } else {
    ok = umma::mbar_wait(&mbar[1], 0) && ok;
    umma::fence_after_sync();
    if (ok) {
      // Z^T -> AZ rows 64 + v, col t
      const uint32_t o = kOffAZ + uint32_t(t >> 2) * kCS128P + uint32_t(t & 3) * 4 + 64 * 16;
#pragma unroll
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t u[32];
        umma::tmem_ld32(tmem + 128 + lane_base + c0, u);
        umma::tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) st1(smem, o + (c0 + jj) * 16, umma::to_tf32(__uint_as_float(u[jj])));
      }
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
  ok = umma::mbar_wait(&mbar[2], 0) && ok;
  umma::fence_after_sync();
  if (ok) {
#pragma unroll
    for (int c0 = 0; c0 < 64; c0 += 32) {
      uint32_t u[32];
      umma::tmem_ld32(tmem + 192 + lane_base + c0, u);
      umma::tmem_ld_wait();
#pragma unroll
      for (int jj = 0; jj < 32; jj += 4)
        st4(smem, kOffX2 + uint32_t((c0 + jj) >> 2) * kCS128 + tid * 16,
            umma::to_tf32(make_float4(__uint_as_float(u[jj]), __uint_as_float(u[jj + 1]),
                                      __uint_as_float(u[jj + 2]), __uint_as_float(u[jj + 3]))));
    }
  }
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();

  // ---- MMA 4 + 5: [A_rb ; B^^T] [P|Q]  (+)  [A_rk ; K^^T] V into columns 64..127 ----------------------
  if (tid == 0) {
    issue_mma(tmem, sbase + kOffRB, kCS128P, sbase + kOffX2, kCS128, 128, false);
    issue_mma(tmem + 64, sbase + kOffRK, kCS128P, sbase + kOffVT, kCS64P, 64, true);
    umma::mma_commit(&mbar[3]);
  }
  ok = umma::mbar_wait(&mbar[3], 0) && ok;
  umma::fence_after_sync();
  if (ok) {
    unsigned char* ws = workspace + (size_t)blockIdx.x * (2 * kWsTile);
#pragma unroll
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t u[32];
      umma::tmem_ld32(tmem + lane_base + c0, u);
      umma::tmem_ld_wait();
#pragma unroll
      for (int jj = 0; jj < 32; jj += 4) {
        float4 val = make_float4(__uint_as_float(u[jj]), __uint_as_float(u[jj + 1]), __uint_as_float(u[jj + 2]),
                                 __uint_as_float(u[jj + 3]));
        const int c = c0 + jj;
        if (c < 64) {
          if (tid < 64) {  // E = R~ + A_rb P
            const float4 rt = ld4(smem, kOffX1 + uint32_t(c >> 2) * kCS128 + (64 + t) * 16);
            val.x += rt.x; val.y += rt.y; val.z += rt.z; val.w += rt.w;
          } else {         // M = diag(g_L) + B^^T P
            const int kk = tid - 64;
            if (kk == c) val.x += diag_gl;
            if (kk == c + 1) val.y += diag_gl;
            if (kk == c + 2) val.z += diag_gl;
            if (kk == c + 3) val.w += diag_gl;
          }
          st4(ws, uint32_t(c >> 2) * kCS128 + tid * 16, umma::to_tf32(val));
        } else {
          st4(ws, kWsTile + uint32_t((c - 64) >> 2) * kCS128 + tid * 16, val);
        }
      }
    }
  }
  if (!ok && tid == 0 && error_flag != nullptr) atomicExch(error_flag, 1);
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
    ok = umma::mbar_wait(&full_bar[stage], (it >> 1) & 1);
    if (!ok) break;
    if (tid == 0) {
      umma::fence_after_sync();
      issue_mma(acc, sbase + stage * kScanStage, kCS128, sbase + kScanOffST, kCS64P, 64, false);
      umma::mma_commit(&mma_bar);
    }
    ok = umma::mbar_wait(&mma_bar, it & 1);
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
  if (!ok && tid == 0 && error_flag != nullptr) atomicExch(error_flag, 2);
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
  {
    cudaError_t e1 = cudaFuncSetAttribute(wkv7_chunk_build_kernel<io_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)kBuildSmem);
    cudaError_t e2 = cudaFuncSetAttribute(wkv7_chunk_scan_kernel<io_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)kScanSmem);
    if (e1 != cudaSuccess || e2 != cudaSuccess)
      return fail(FRWKV_ERR_CUDA, "wkv7_chunk_forward: cannot reserve shared memory: %s",
                  cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
  }
  wkv7_chunk_build_kernel<io_t><<<(unsigned)(num_chunks * num_heads), 128, kBuildSmem, stream>>>(
      chunk_starts, chunk_ends, status, static_cast<const io_t*>(r), static_cast<const io_t*>(w),
      static_cast<const io_t*>(k), static_cast<const io_t*>(v), static_cast<const io_t*>(a),
      static_cast<const io_t*>(b), static_cast<const io_t*>(bias), static_cast<unsigned char*>(workspace), num_heads,
      error_flag);
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
