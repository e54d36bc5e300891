// Helpers shared by the chunked WKV7 kernels (fused forward / adjoint scan, chunk-parallel backward): access to
// chunk-major operand tiles, the warp-uniform bounded wait, 16-bit unpacking, and the blocked triangular inverse.
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

// T' = (I - A)^-1 - I for the strictly lower triangular 64 x 64 A in the scratch, in fp32, by 16 x 16 blocks:
// T_ii = (I - A_ii)^-1 (one thread per column, 16 right-looking steps), then the off-diagonal blocks in two levels
// (inside the 32 x 32 halves, then the 32 x 32 block below them).  A block product is done by 32 threads with 2 x 4
// register tiles and 16-byte operand reads (rows of A and of T, four adjacent columns of T and W).  Ends with T'
// rounded to tf32 in rows 0..63 of the tile and zeros in rows 64..127 (the second operand half of MMA 3).  Contains barriers.
__device__ __forceinline__ void fma_2x4(float (&acc)[2][4], const float4& a0, const float4& a1, const float4& t0,
                                        const float4& t1, const float4& t2, const float4& t3) {
  const float a[2][4] = {{a0.x, a0.y, a0.z, a0.w}, {a1.x, a1.y, a1.z, a1.w}};
  const float t[4][4] = {{t0.x, t0.y, t0.z, t0.w}, {t1.x, t1.y, t1.z, t1.w}, {t2.x, t2.y, t2.z, t2.w},
                         {t3.x, t3.y, t3.z, t3.w}};
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) acc[r][cc] = fmaf(a[r][k], t[k][cc], acc[r][cc]);
}

// kGroupThreads = 0: every thread of the CTA calls it and the barriers are CTA-wide.  kGroupThreads = 256: only
// threads 0..255 call it (barriers on named barrier 1) and the other warps are free to do something else meanwhile.
template <uint32_t kScratch, uint32_t kTile, uint32_t kCST, bool kTransposed, int kGroupThreads = 0>
__device__ __forceinline__ void inverse_blocked(unsigned char* smem, int tid) {
  static_assert(kGroupThreads == 0 || kGroupThreads == 256, "the last pass uses threads 0..255");
  const auto group_sync = [] {
    if (kGroupThreads == 0) __syncthreads();
    else asm volatile("bar.sync 1, %0;" ::"n"(kGroupThreads) : "memory");
  };
  // A: fp32 scratch at kScratch, row t = 256 bytes, 16-byte pieces permuted by the row pair (see aab_off);
  // T (then T' or T'^T) in rows 0..63 of the 128-row tile at kTile (chunk stride kCST), scratch W in rows 64..127
  const auto aab_off = [](int t, int s4) { return kScratch + uint32_t(t) * 256 + uint32_t((s4 ^ ((t >> 1) & 7)) * 16); };
  const auto aab = [&](const unsigned char* sm, int t, int sc) { return ld1(sm, aab_off(t, sc >> 2) + (sc & 3) * 4); };
  const auto t_off = [](int row, int col) { return kTile + tile_off(kCST, row, col); };
  const auto w_off = [](int row, int col) { return kTile + tile_off(kCST, 64 + row, col); };
  if (tid < 64) {
    const int blk = tid >> 4, jj = tid & 15;
    float acc[16];
#pragma unroll
    for (int rr = 0; rr < 16; ++rr) acc[rr] = 0.f;
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      const float xq = acc[q] + (q == jj ? 1.f : 0.f);
      st1(smem, t_off(16 * blk + q, 16 * blk + jj), xq);
#pragma unroll
      for (int rr = q + 1; rr < 16; ++rr) acc[rr] = fmaf(aab(smem, 16 * blk + rr, 16 * blk + q), xq, acc[rr]);
    }
  }
  group_sync();
  const int warp = tid >> 5, sub = tid & 31;
  const int rp = sub >> 2, cq = sub & 3;  // rows 2 rp, 2 rp + 1 and columns 4 cq .. 4 cq + 3 of a 16 x 16 block
  // One 16 x 16 x 16 block product per warp: acc += L[rows lr .. lr + 15][k] * R[k][columns rc .. rc + 15], k = 0..15.
  // L is a block of A (scratch; lc = its first column), of T or of W (tile rows 0..63 / 64..127); R a block of T or W.
  enum { kFromA = 0, kFromT = 1, kFromW = 2 };
  const auto product = [&](float (&acc)[2][4], int lkind, int lr, int lc, int rkind, int rr, int rc) {
    const int row = lr + 2 * rp, col = rc + 4 * cq;
#pragma unroll 2
    for (int kq = 0; kq < 4; ++kq) {
      float4 l0, l1;
      if (lkind == kFromA) {
        l0 = ld4(smem, aab_off(row, (lc >> 2) + kq));
        l1 = ld4(smem, aab_off(row + 1, (lc >> 2) + kq));
      } else {
        const uint32_t base0 = lkind == kFromT ? t_off(row, lc + 4 * kq) : w_off(row, lc + 4 * kq);
        l0 = ld4(smem, base0);
        l1 = ld4(smem, base0 + 16);  // the next row of the same 16-byte column chunk
      }
      const uint32_t r0 = rkind == kFromT ? t_off(rr + 4 * kq, col) : w_off(rr + 4 * kq, col);
      fma_2x4(acc, l0, l1, ld4(smem, r0), ld4(smem, r0 + 16), ld4(smem, r0 + 32), ld4(smem, r0 + 48));
    }
  };
  const auto store = [&](bool to_t, int r0, int c0, const float (&acc)[2][4]) {
    const uint32_t o = to_t ? t_off(r0 + 2 * rp, c0 + 4 * cq) : w_off(r0 + 2 * rp, c0 + 4 * cq);
    st4(smem, o, make_float4(acc[0][0], acc[0][1], acc[0][2], acc[0][3]));
    st4(smem, o + 16, make_float4(acc[1][0], acc[1][1], acc[1][2], acc[1][3]));
  };
  // Two levels instead of one block anti-diagonal at a time: first the off-diagonal blocks inside the two 32 x 32
  // halves, T_10 = T_11 (A_10 T_00) and T_32 = T_33 (A_32 T_22); then the 32 x 32 block below,
  // T_lo = T22' (A21' T11') with T11' = [T_00 0; T_10 T_11], T22' = [T_22 0; T_32 T_33], one warp per 16 x 16 block.
  // Four barrier-separated steps in place of six.  W block (i, j) lives in tile rows 64 + 16 i .., columns 16 j ...
  // ---- step 1a: W(0,0) = A_10 T_00, W(0,1) = A_32 T_22 ----------------------------------------------------------
  if (warp < 2) {
    float acc[2][4] = {};
    const int j = 32 * warp;  // block column 0 or 2
    product(acc, kFromA, j + 16, j, kFromT, j, j);
    store(false, 0, 16 * warp, acc);
  }
  group_sync();
  // ---- step 1b: T_10 = T_11 W(0,0), T_32 = T_33 W(0,1) -----------------------------------------------------------
  if (warp < 2) {
    float acc[2][4] = {};
    const int j = 32 * warp;
    product(acc, kFromT, j + 16, j + 16, kFromW, 0, 16 * warp);
    store(true, j + 16, j, acc);
  }
  group_sync();
  // ---- step 2a: W' = A21' T11': W'_p0 = A_{2+p,0} T_00 + A_{2+p,1} T_10, W'_p1 = A_{2+p,1} T_11; W'_pj in W(1+p, j) ---
  if (warp < 4) {
    float acc[2][4] = {};
    const int p = warp >> 1, j = warp & 1;
    if (j == 0) {
      product(acc, kFromA, 32 + 16 * p, 0, kFromT, 0, 0);
      product(acc, kFromA, 32 + 16 * p, 16, kFromT, 16, 0);
    } else {
      product(acc, kFromA, 32 + 16 * p, 16, kFromT, 16, 16);
    }
    store(false, 16 * (1 + p), 16 * j, acc);
  }
  group_sync();
  // ---- step 2b: T_lo = T22' W': T_2j = T_22 W'_0j, T_3j = T_32 W'_0j + T_33 W'_1j ----------------------------------
  if (warp < 4) {
    float acc[2][4] = {};
    const int i = warp >> 1, j = warp & 1;
    if (i == 0) {
      product(acc, kFromT, 32, 32, kFromW, 16, 16 * j);
    } else {
      product(acc, kFromT, 48, 32, kFromW, 16, 16 * j);
      product(acc, kFromT, 48, 48, kFromW, 32, 16 * j);
    }
    store(true, 32 + 16 * i, 16 * j, acc);
  }
  group_sync();
  {
    // T' = T - I, rounded; everything on and above the diagonal is zero (the blocks above it were never written).
    // kTransposed: the tile ends as T'^T (rows and columns exchanged through registers, behind a barrier).
    const int row = tid & 63, c4 = (tid >> 6) & 3;
    float4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int col = 16 * c4 + 4 * i;
      v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tid < 256 && col < row) {
        v[i] = umma::to_tf32(ld4(smem, t_off(row, col)));
        if (col + 1 >= row) v[i].y = 0.f;
        if (col + 2 >= row) v[i].z = 0.f;
        if (col + 3 >= row) v[i].w = 0.f;
      }
    }
    if (kTransposed) group_sync();
    if (tid < 256) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = 16 * c4 + 4 * i;
        if (kTransposed) {
          st1(smem, t_off(col, row), v[i].x);
          st1(smem, t_off(col + 1, row), v[i].y);
          st1(smem, t_off(col + 2, row), v[i].z);
          st1(smem, t_off(col + 3, row), v[i].w);
        } else {
          st4(smem, t_off(row, col), v[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int piece = tid + i * 256;  // 16 chunks x 64 rows of 16 bytes
        st4(smem, kTile + uint32_t(piece >> 6) * kCST + 1024 + uint32_t(piece & 63) * 16, make_float4(0.f, 0.f, 0.f, 0.f));
      }
    }
  }
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
