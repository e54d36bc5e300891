// One RWKV-7 TMix layer for a decode batch (one token per sequence, at most 8 rows) as ONE persistent kernel.
//
// The unfused operator sequence is seven launches (token shift + r / k / v / rank-in projections, shift-state update,
// rank-out projections with the value-residual gate, kk_a_gate, the WKV7 step, lnx_rkvres_xg, the output projection);
// at one to eight rows each of them is bound by its launch and its fixed dependency chain, not by the 38 MB of weights
// the layer streams.  Here one CTA per SM stays resident for the whole layer (cooperative launch) and the stages are
// separated by grid-wide barriers:
//   stage 1   token shift in fp32 while x is staged; r, k, v (C x C) and the four rank-in products; every projection
//             gets a share of the CTAs in proportion to its weight bytes, so all weight streams are in flight at once.
//             The weight rows arrive through a ring of cp.async.bulk copies per warp (two rows per copy), which keeps
//             ~190 KB per SM in flight
//   stage 2   rank-out products: tanh(fw) w2, fa a2, sigmoid(fg) g2, fv v2 with the value-residual gate; a CTA's
//             weight rows are copied to shared memory while it waits at the barrier before; the shift states take x
//   stage 3   per (row, head): kk_a_gate, the WKV7 state update and output, lnx_rkvres_xg; one CTA per unit; the
//             state tile and the channel vectors of a CTA's first unit are requested when the kernel starts
//   stage 4   the output projection; its first weight rows are requested before stage 3
// Intermediate tensors are rounded to the 16-bit io type at exactly the points where the separate operators round
// them, so the result equals the operator sequence up to summation order.
//
// Grid barrier: a counter per barrier in global memory; thread 0 of a CTA arrives (fence, atomic add) and polls with
// an acquire load and a bounded number of sleeps; the last CTA to finish the kernel zeroes the counters again.  If a
// wait runs out, the CTA raises the error flag, fills its share of the output with NaN and leaves.
//
// No counterpart in the reference (its layer is the operator sequence: csrc/sm120/tmix/{mix6,linear,kk_a_gate,
// wkv7,lnx_rkvres_xg}); the arithmetic of every stage is that of the separate kernels in tmix_linear.cu,
// tmix_elementwise.cu and wkv7_recurrent.cu.

#include "tmix_linear.cuh"
#include "umma.cuh"

namespace frwkv {
namespace {

constexpr int kLayerThreads = 256;
constexpr unsigned kBarrierPolls = 1u << 20;  // x >= 64 ns per poll: gives up after roughly a tenth of a second

struct DecodeLayerParams {
  const void* x;        // [M][C]
  const void* v_first;  // [M][C]
  void* shift_pool;     // [slots][C]
  float* state_pool;    // [slots][H][64][64]
  const void* mix[6];   // x_r, x_w, x_k, x_v, x_a, x_g  [C]
  const void* w_r; const void* w_k; const void* w_v; const void* w_o;  // [C][C]
  const void* w1[4];    // decay, a, gate, value-residual rank-in  [R][C]
  const void* w2[4];    // ... rank-out [C][R]
  int rank[4];
  const void* k_k; const void* a0; const void* k_a; const void* r_k; const void* ln_w; const void* ln_b; const void* v0;
  void* out;            // [M][C]
  void* r; void* k; void* v;                        // intermediates, 16-bit [M][C]
  void* f[4];                                       // rank-in results [M][R]
  void* wl; void* a12; void* g; void* vres; void* z;  // [M][C]
  const int* state_indices;
  const int* status;
  unsigned* barrier;    // 4 counters (three grid barriers, the exit count): zero before a launch and after it
  int* error_flag;
  int first1[8];        // stage 1: first CTA of each of the 7 projections (r, k, v, rank-in w / a / g / v), then the grid size
  int first2[5];        // stage 2: ... of the 4 rank-out projections
  int depth;            // bulk-copy slots per warp (2..4)
  uint32_t ring_bytes;  // size of the ring
  int C, H;
  float eps;
};

__device__ __forceinline__ float sigmoid_exact(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float warp_total(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// every thread of the CTA calls it; returns false (for all threads) if the wait ran out
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned expected) {
  __syncthreads();
  int ok = 1;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    unsigned seen = 0, polls = 0;
    for (;;) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
      if (seen >= expected) break;
      if (++polls > kBarrierPolls) { ok = 0; break; }
      __nanosleep(64);
    }
  }
  return __syncthreads_and(ok) != 0;
}

// ---- weight rows through a bulk-copy ring -----------------------------------------------------------------------------
// The long projections (K = C) are bound by how many bytes a resident CTA keeps in flight.  Register-staged loads give
// 8 warps x 16 x 512 B = 64 KB per SM with a gap after every pass; here every warp owns `depth` slots of shared memory,
// each filled by one cp.async.bulk of two adjacent weight rows (completion on the slot's mbarrier), and refills a slot
// as soon as it has consumed it, so the copy engine keeps depth x 8 x 2 rows per SM on their way while the warps
// multiply.  A CTA takes a contiguous range of row pairs; warp w the pairs w, w + 8, ... of that range.
struct RowRing {
  const unsigned char* w;  // weight matrix [N][K], 16-bit
  int g_begin, g_end;      // this CTA's row pairs
  uint32_t pair_bytes;     // 2 * K * 2
  int depth;               // slots per warp
};

__device__ __forceinline__ RowRing make_ring(const void* w, int N, int K, int vblock, int vgrid, int depth) {
  const int pairs = N >> 1;
  return RowRing{static_cast<const unsigned char*>(w), (int)((long long)pairs * vblock / vgrid),
                 (int)((long long)pairs * (vblock + 1) / vgrid), uint32_t(K) * 4u, depth};
}

// lane 0 of every warp requests the warp's first `depth` pairs
__device__ __forceinline__ void ring_start(const RowRing& rg, unsigned char* ring, uint64_t* mbar) {
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) != 0) return;
  for (int i = 0; i < rg.depth; ++i) {
    const int g = rg.g_begin + warp + 8 * i;
    if (g >= rg.g_end) break;
    uint64_t* bar = mbar + warp * 4 + i;
    umma::mbar_expect_tx(bar, rg.pair_bytes);
    umma::bulk_g2s(ring + (size_t)(warp * rg.depth + i) * rg.pair_bytes, rg.w + (size_t)g * rg.pair_bytes, rg.pair_bytes, bar);
  }
}

// y[m][n] = finish(sum_k xs[m][k] W[n][k]) for the CTA's rows; xs / xs_hi: the fp32 planes of the staged rows of x.
// Returns false if a wait ran out (uniform over the warp).
template <typename io_t, int M>
__device__ __forceinline__ bool ring_products(const RowRing& rg, const LinearProblem& pr, const float4* xs,
                                              const float4* xs_hi, unsigned char* ring, uint64_t* mbar) {
  using IO = Io16<io_t>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, kv = pr.k >> 3, N = pr.n;
  io_t* y = static_cast<io_t*>(pr.y);
  for (int i = 0;; ++i) {
    const int g = rg.g_begin + warp + 8 * i;
    if (g >= rg.g_end) break;
    const int slot = i % rg.depth;
    uint64_t* bar = mbar + warp * 4 + slot;
    if (!umma::mbar_wait(bar, (uint32_t)(i / rg.depth) & 1u)) return false;
    const uint4* row0 = reinterpret_cast<const uint4*>(ring + (size_t)(warp * rg.depth + slot) * rg.pair_bytes);
    const uint4* row1 = row0 + kv;
    float2 acc0[M], acc1[M];
#pragma unroll
    for (int m = 0; m < M; ++m) { acc0[m] = make_float2(0.f, 0.f); acc1[m] = make_float2(0.f, 0.f); }
    for (int c = lane; c < kv; c += 32) {
      const uint4 q0 = row0[c], q1 = row1[c];
      const float2 a0 = IO::unpack(q0.x), a1 = IO::unpack(q0.y), a2 = IO::unpack(q0.z), a3 = IO::unpack(q0.w);
      const float2 b0 = IO::unpack(q1.x), b1 = IO::unpack(q1.y), b2 = IO::unpack(q1.z), b3 = IO::unpack(q1.w);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float4 xa = xs[m * kv + c], xb = xs_hi[m * kv + c];
        const float2 x0 = make_float2(xa.x, xa.y), x1 = make_float2(xa.z, xa.w);
        const float2 x2 = make_float2(xb.x, xb.y), x3 = make_float2(xb.z, xb.w);
        acc0[m] = __ffma2_rn(a0, x0, __ffma2_rn(a1, x1, __ffma2_rn(a2, x2, __ffma2_rn(a3, x3, acc0[m]))));
        acc1[m] = __ffma2_rn(b0, x0, __ffma2_rn(b1, x1, __ffma2_rn(b2, x2, __ffma2_rn(b3, x3, acc1[m]))));
      }
    }
    __syncwarp();  // every lane has read the slot: it may be refilled
    if (lane == 0) {
      const int g2 = g + 8 * rg.depth;
      if (g2 < rg.g_end) {
        umma::mbar_expect_tx(bar, rg.pair_bytes);
        umma::bulk_g2s(ring + (size_t)(warp * rg.depth + slot) * rg.pair_bytes, rg.w + (size_t)g2 * rg.pair_bytes,
                       rg.pair_bytes, bar);
      }
    }
    const int n = 2 * g;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float t0 = acc0[m].x + acc0[m].y, t1 = acc1[m].x + acc1[m].y;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        t0 += __shfl_xor_sync(0xffffffffu, t0, o);
        t1 += __shfl_xor_sync(0xffffffffu, t1, o);
      }
      if (lane == 0)
        *reinterpret_cast<uint32_t*>(y + (long long)m * N + n) =
            IO::pack(finish<io_t>(pr, t0, m, n), finish<io_t>(pr, t1, m, n + 1));
    }
  }
  return true;
}

// Rank-out products (K = rank <= 512, rows of a few hundred bytes): eight lanes share an output column and a warp works on
// sixteen columns at a time (four per lane group), so that every lane has 4 x ceil(K / 64) independent 16-byte weight
// loads in flight instead of one column's worth.  A CTA takes the contiguous columns [n_begin, n_end); with kStaged
// their weight rows have been copied to shared memory beforehand.  xs / xs_hi as in ring_products.
template <typename io_t, int M, bool kStaged>
__device__ __forceinline__ void rank_out_products(const LinearProblem& pr, const float4* xs, const float4* xs_hi,
                                                  int n_begin, int n_end, const unsigned char* staged) {
  using IO = Io16<io_t>;
  const int K = pr.k, N = pr.n, kv = K >> 3;
  // the CTA's columns [n_begin, n_end): from global memory, or from the copy of exactly those rows in shared memory
  const io_t* w = kStaged ? reinterpret_cast<const io_t*>(staged) - (long long)n_begin * K : static_cast<const io_t*>(pr.w);
  io_t* y = static_cast<io_t*>(pr.y);
  const int lane = threadIdx.x & 31, sub = lane & 7, grp = lane >> 3;
  for (int n0 = n_begin + 16 * (threadIdx.x >> 5); n0 < n_end; n0 += 16 * (blockDim.x >> 5)) {
    float2 acc[4][M];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int m = 0; m < M; ++m) acc[u][m] = make_float2(0.f, 0.f);
    }
    // N is a multiple of 8, not of 16: the last block of a matrix may hold only the first two lane groups' columns
    const uint4* wrow[4];
    bool live[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int n = n0 + 4 * u + grp;
      live[u] = n < n_end;
      wrow[u] = reinterpret_cast<const uint4*>(w + (long long)(live[u] ? n : n_begin) * K);
    }
#pragma unroll 2
    for (int c = sub; c < kv; c += 8) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) q[u] = kStaged ? wrow[u][c] : __ldg(wrow[u] + c);
      float4 xa[M], xb[M];
#pragma unroll
      for (int m = 0; m < M; ++m) { xa[m] = xs[m * kv + c]; xb[m] = xs_hi[m * kv + c]; }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 a0 = IO::unpack(q[u].x), a1 = IO::unpack(q[u].y), a2 = IO::unpack(q[u].z), a3 = IO::unpack(q[u].w);
#pragma unroll
        for (int m = 0; m < M; ++m)
          acc[u][m] = __ffma2_rn(a0, make_float2(xa[m].x, xa[m].y),
                                 __ffma2_rn(a1, make_float2(xa[m].z, xa[m].w),
                                            __ffma2_rn(a2, make_float2(xb[m].x, xb[m].y),
                                                       __ffma2_rn(a3, make_float2(xb[m].z, xb[m].w), acc[u][m]))));
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int n = n0 + 4 * u + grp;
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float t = acc[u][m].x + acc[u][m].y;
        t += __shfl_xor_sync(0xffffffffu, t, 1);
        t += __shfl_xor_sync(0xffffffffu, t, 2);
        t += __shfl_xor_sync(0xffffffffu, t, 4);
        if (sub == 0 && live[u]) y[(long long)m * N + n] = IO::store(finish<io_t>(pr, t, m, n));
      }
    }
  }
}

template <typename io_t, int M>
__global__ __launch_bounds__(kLayerThreads, 1) void tmix_decode_layer_kernel(const DecodeLayerParams p) {
  using IO = Io16<io_t>;
  extern __shared__ __align__(16) unsigned char xs_raw[];
  __shared__ float hv[7][64];    // stage 3: r, w, k', v, -kk, kk a, y of one head
  __shared__ float part[4][64];
  const int C = p.C, kv = C >> 3, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, grid = gridDim.x;
  io_t* out = static_cast<io_t*>(p.out);
  if (p.status != nullptr && p.status[0] != 0) {  // fail closed (uniform over the grid: no barrier is entered)
    for (int i = cta * kLayerThreads + tid; i < M * C; i += grid * kLayerThreads) out[i] = IO::store(quiet_nan());
    return;
  }
  float4* xs = reinterpret_cast<float4*>(xs_raw);
  unsigned char* ring = xs_raw + (size_t)M * C * 4;  // after the staged rows of x
  __shared__ uint64_t mbar1[8 * 4], mbar4[8 * 4], state_bar, w2_bar;
  __shared__ __align__(128) float s_state[64 * 64];  // the state tile of this CTA's first stage-3 unit, fetched at once
  if (tid < 64) umma::mbar_init(tid < 32 ? &mbar1[tid] : &mbar4[tid - 32], 1);
  if (tid == 64) umma::mbar_init(&state_bar, 1);
  if (tid == 65) umma::mbar_init(&w2_bar, 1);
  umma::mbar_fence_init();
  __syncthreads();
  bool ok = true;
  // the per-channel vectors of this CTA's first stage-3 unit are constants too: warp 0 asks for them now
  uint32_t pre[6] = {0u, 0u, 0u, 0u, 0u, 0u};
  if (warp == 0 && cta < M * p.H) {
    const int c = (cta % p.H) * 64 + 2 * lane;
    const void* const vecs[6] = {p.k_k, p.a0, p.k_a, p.r_k, p.ln_w, p.ln_b};
#pragma unroll
    for (int i = 0; i < 6; ++i) pre[i] = __ldg(reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(vecs[i]) + c));
  }
  if (tid == 0 && cta < M * p.H) {
    const int m = cta / p.H, h = cta % p.H;
    umma::mbar_expect_tx(&state_bar, 64 * 64 * 4);
    umma::bulk_g2s(s_state, p.state_pool + ((long long)p.state_indices[m] * p.H + h) * 4096, 64 * 64 * 4, &state_bar);
  }

  // ---- stage 1: token shift + r / k / v / rank-in projections ---------------------------------------------------
  {
    int j = 0;
    while (j < 6 && cta >= p.first1[j + 1]) ++j;
    const int vblock = cta - p.first1[j], vgrid = p.first1[j + 1] - p.first1[j];
    const void* w = j == 0 ? p.w_r : j == 1 ? p.w_k : j == 2 ? p.w_v : p.w1[j - 3];
    void* y = j == 0 ? p.r : j == 1 ? p.k : j == 2 ? p.v : p.f[j - 3];
    const int n = j < 3 ? C : p.rank[j - 3];
    const int mix_id = j == 0 ? 0 : j == 1 ? 2 : j == 2 ? 3 : j == 3 ? 1 : j == 4 ? 4 : j == 5 ? 5 : 3;
    const RowRing rg = make_ring(w, n, C, vblock, vgrid, p.depth);
    ring_start(rg, ring, mbar1);
    float4* xs_hi = xs + M * kv;
    const uint4* mixv = reinterpret_cast<const uint4*>(p.mix[mix_id]);
    for (int c = tid; c < kv; c += kLayerThreads) {
      float mf[8];
      unpack8<io_t>(__ldg(mixv + c), mf);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float xf[8], pv[8];
        unpack8<io_t>(__ldg(reinterpret_cast<const uint4*>(p.x) + m * kv + c), xf);
        unpack8<io_t>(__ldg(reinterpret_cast<const uint4*>(p.shift_pool) + (long long)p.state_indices[m] * kv + c), pv);
#pragma unroll
        for (int e = 0; e < 8; ++e) xf[e] = fmaf(pv[e] - xf[e], mf[e], xf[e]);
        xs[m * kv + c] = make_float4(xf[0], xf[1], xf[2], xf[3]);
        xs_hi[m * kv + c] = make_float4(xf[4], xf[5], xf[6], xf[7]);
      }
    }
    __syncthreads();
    const LinearProblem pr{p.x, w, y, nullptr, nullptr, nullptr, n, C, 0, 0};
    ok = ring_products<io_t, M>(rg, pr, xs, xs_hi, ring, mbar1);
  }
  // this CTA's rank-out share: projection j2, columns [n2_begin, n2_end) (multiples of 8).  The weights are constants:
  // their rows are requested now, into the ring's memory (stage 1 has consumed it), and arrive while the CTA waits at
  // the barrier.
  int j2 = 0;
  while (j2 < 3 && cta >= p.first2[j2 + 1]) ++j2;
  const int vb2 = cta - p.first2[j2], vg2 = p.first2[j2 + 1] - p.first2[j2];
  const int n2_begin = 8 * (int)((long long)(C >> 3) * vb2 / vg2), n2_end = 8 * (int)((long long)(C >> 3) * (vb2 + 1) / vg2);
  const uint32_t w2_bytes = uint32_t(n2_end - n2_begin) * uint32_t(p.rank[j2]) * 2u;
  const bool w2_staged = w2_bytes > 0 && w2_bytes <= p.ring_bytes;
  __syncthreads();  // every warp is done with its slots
  if (tid == 0 && w2_staged) {
    umma::mbar_expect_tx(&w2_bar, w2_bytes);
    umma::bulk_g2s(ring, static_cast<const unsigned char*>(p.w2[j2]) + (size_t)n2_begin * p.rank[j2] * 2, w2_bytes, &w2_bar);
  }
  ok = grid_barrier(&p.barrier[0], grid) && __syncthreads_and(ok ? 1 : 0) != 0;

  // ---- stage 2: rank-out projections (+ value-residual gate); the shift states take x ---------------------------
  if (ok) {
    if (cta < M) {
      const uint4* src = reinterpret_cast<const uint4*>(p.x) + cta * kv;
      uint4* dst = reinterpret_cast<uint4*>(p.shift_pool) + (long long)p.state_indices[cta] * kv;
      for (int c = tid; c < kv; c += kLayerThreads) dst[c] = src[c];
    }
    const int j = j2, rk = p.rank[j], rkv = rk >> 3;
    const int act = j == 0 ? 1 : j == 2 ? 2 : 0;
    void* y = j == 0 ? p.wl : j == 1 ? p.a12 : j == 2 ? p.g : p.vres;
    float4* xs_hi = xs + M * rkv;
    for (int i = tid; i < M * rkv; i += kLayerThreads) {
      float f[8];
      unpack8<io_t>(*(reinterpret_cast<const uint4*>(p.f[j]) + i), f);  // written in stage 1: a plain (coherent) load
      if (act != 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = apply_act(f[e], act);
      }
      xs[i] = make_float4(f[0], f[1], f[2], f[3]);
      xs_hi[i] = make_float4(f[4], f[5], f[6], f[7]);
    }
    __syncthreads();
    const LinearProblem pr{p.f[j], p.w2[j], y, j == 3 ? p.v : nullptr, j == 3 ? p.v_first : nullptr,
                           j == 3 ? p.v0 : nullptr, C, rk, 0, j == 3 ? 1 : 0};
    if (w2_staged) {
      if (!umma::mbar_wait(&w2_bar, 0)) ok = false;
      if (ok) rank_out_products<io_t, M, true>(pr, xs, xs_hi, n2_begin, n2_end, ring);
    } else {
      rank_out_products<io_t, M, false>(pr, xs, xs_hi, n2_begin, n2_end, nullptr);
    }
    ok = grid_barrier(&p.barrier[1], grid) && __syncthreads_and(ok ? 1 : 0) != 0;
  }

  // ---- stage 3: per (row, head): kk_a_gate, WKV7 step, lnx_rkvres_xg ------------------------------------------------
  const RowRing rg_o = make_ring(p.w_o, C, C, cta, grid, p.depth);
  if (ok) {
    ring_start(rg_o, ring, mbar4);  // constants: on their way while the heads are worked on
    const int units = M * p.H;
    for (int unit = cta; unit < units; unit += grid) {
      const int m = unit / p.H, h = unit % p.H;
      const long long o = (long long)m * C + h * 64 + 2 * lane;
      const int c = h * 64 + 2 * lane;
      if (warp == 0) {
        const float2 kx = IO::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.k) + o));
        const bool first = unit == cta;
        const float2 kkv = IO::unpack(first ? pre[0] : __ldg(reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.k_k) + c)));
        const float2 a0v = IO::unpack(first ? pre[1] : __ldg(reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.a0) + c)));
        const float2 a12v = IO::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.a12) + o));
        const float2 kav = IO::unpack(first ? pre[2] : __ldg(reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.k_a) + c)));
        const float2 q = make_float2(kx.x * kkv.x, kx.y * kkv.y);
        const float2 gt = make_float2(sigmoid_exact(a0v.x + a12v.x), sigmoid_exact(a0v.y + a12v.y));
        const float nrm = fmaxf(sqrtf(warp_total(fmaf(q.x, q.x, q.y * q.y))), 1e-12f);
        const float n0 = q.x / nrm, n1 = q.y / nrm;
        // rounded as the separate kk_a_gate operator rounds its three outputs
        const float2 nk = IO::unpack(IO::pack(kx.x * (1.f + (gt.x - 1.f) * kav.x), kx.y * (1.f + (gt.y - 1.f) * kav.y)));
        const float2 na = IO::unpack(IO::pack(-n0, -n1));
        const float2 nb = IO::unpack(IO::pack(n0 * gt.x, n1 * gt.y));
        hv[2][2 * lane] = nk.x; hv[2][2 * lane + 1] = nk.y;
        hv[4][2 * lane] = na.x; hv[4][2 * lane + 1] = na.y;
        hv[5][2 * lane] = nb.x; hv[5][2 * lane + 1] = nb.y;
      } else if (warp == 1) {
        const float2 rx = IO::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.r) + o));
        const float2 wx = IO::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.wl) + o));
        const float2 vx = IO::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.vres) + o));
        hv[0][2 * lane] = rx.x; hv[0][2 * lane + 1] = rx.y;
        hv[1][2 * lane] = retention(wx.x); hv[1][2 * lane + 1] = retention(wx.y);
        hv[3][2 * lane] = vx.x; hv[3][2 * lane + 1] = vx.y;
      }
      // state tile: thread (value column vc, key group kq) holds S[16 kq + i][vc]
      const int vc = tid & 63, kq = tid >> 6;
      float* sp = p.state_pool + ((long long)p.state_indices[m] * p.H + h) * 4096 + (16 * kq) * 64 + vc;
      float S[16];
      if (unit == cta) {  // the tile requested when the kernel started
        if (!umma::mbar_wait(&state_bar, 0)) ok = false;
#pragma unroll
        for (int i = 0; i < 16; ++i) S[i] = s_state[(16 * kq + i) * 64 + vc];
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) S[i] = sp[i * 64];
      }
      __syncthreads();
      float sa = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) sa = fmaf(hv[4][16 * kq + i], S[i], sa);
      part[kq][vc] = sa;
      __syncthreads();
      sa = (part[0][vc] + part[1][vc]) + (part[2][vc] + part[3][vc]);
      __syncthreads();
      const float vv = hv[3][vc];
      float y = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int kc = 16 * kq + i;
        S[i] = fmaf(hv[1][kc], S[i], fmaf(hv[5][kc], sa, hv[2][kc] * vv));
        y = fmaf(hv[0][kc], S[i], y);
        sp[i * 64] = S[i];
      }
      part[kq][vc] = y;
      __syncthreads();
      if (kq == 0)  // rounded as the recurrent operator rounds its output
        hv[6][vc] = IO::unpack(IO::pack((part[0][vc] + part[1][vc]) + (part[2][vc] + part[3][vc]), 0.f)).x;
      __syncthreads();
      if (warp == 0) {  // lnx_rkvres_xg on the rounded y
        const float2 xv = make_float2(hv[6][2 * lane], hv[6][2 * lane + 1]);
        const bool first = unit == cta;
        const float2 rk = IO::unpack(first ? pre[3] : __ldg(reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.r_k) + c)));
        float dot = fmaf(hv[0][2 * lane] * hv[2][2 * lane], rk.x, hv[0][2 * lane + 1] * hv[2][2 * lane + 1] * rk.y);
        const float mean = warp_total(xv.x + xv.y) * (1.f / 64.f);
        const float d0 = xv.x - mean, d1 = xv.y - mean;
        const float var = warp_total(fmaf(d0, d0, d1 * d1)) * (1.f / 64.f);
        dot = warp_total(dot);
        const float rstd = rsqrtf(var + p.eps);
        const float2 gv = IO::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.g) + o));
        const float2 wv = IO::unpack(first ? pre[4] : __ldg(reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.ln_w) + c)));
        const float2 bv = IO::unpack(first ? pre[5] : __ldg(reinterpret_cast<const uint32_t*>(static_cast<const io_t*>(p.ln_b) + c)));
        *reinterpret_cast<uint32_t*>(static_cast<io_t*>(p.z) + o) =
            IO::pack((d0 * rstd * wv.x + bv.x + dot * hv[3][2 * lane]) * gv.x,
                     (d1 * rstd * wv.y + bv.y + dot * hv[3][2 * lane + 1]) * gv.y);
      }
      __syncthreads();  // hv and part are reused by the next unit
    }
    ok = grid_barrier(&p.barrier[2], grid) && __syncthreads_and(ok ? 1 : 0) != 0;
  }

  // ---- stage 4: output projection ------------------------------------------------------------------------------------
  if (ok) {
    float4* xs_hi = xs + M * kv;
    for (int i = tid; i < M * kv; i += kLayerThreads) {
      float f[8];
      unpack8<io_t>(*(reinterpret_cast<const uint4*>(p.z) + i), f);
      xs[i] = make_float4(f[0], f[1], f[2], f[3]);
      xs_hi[i] = make_float4(f[4], f[5], f[6], f[7]);
    }
    __syncthreads();
    const LinearProblem pr{p.z, p.w_o, p.out, nullptr, nullptr, nullptr, C, C, 0, 0};
    ok = __syncthreads_and(ring_products<io_t, M>(rg_o, pr, xs, xs_hi, ring, mbar4) ? 1 : 0) != 0;
  }
  if (!ok) {
    if (tid == 0 && p.error_flag != nullptr) atomicExch(p.error_flag, 5);
    for (int i = cta * kLayerThreads + tid; i < M * C; i += grid * kLayerThreads) out[i] = IO::store(quiet_nan());
  }
  // the last CTA to get here puts the counters back to zero for the next launch
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(&p.barrier[3], 1u) == (unsigned)grid - 1u) {
      p.barrier[0] = 0u; p.barrier[1] = 0u; p.barrier[2] = 0u;
      __threadfence();
      p.barrier[3] = 0u;
    }
  }
}

// first CTA of each of `count` projections: one CTA each, the rest in proportion to the weight bytes
void split_ctas(int grid, const long long* weight, int count, int* first) {
  long long total = 0, cum = 0;
  for (int i = 0; i < count; ++i) total += weight[i];
  const int left = grid - count;
  first[0] = 0;
  for (int i = 0; i < count; ++i) {
    cum += weight[i];
    first[i + 1] = (i + 1) + (int)((left * cum + total / 2) / total);
  }
  first[count] = grid;
}

template <typename io_t, int M>
int launch_layer(DecodeLayerParams& p, cudaStream_t stream) {
  static bool ready[64] = {};
  static int sm_counts[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
    return fail(FRWKV_ERR_CUDA, "tmix_decode_layer: cannot identify the current device");
  // the staged rows of x (fp32), then the bulk-copy ring: 8 warps x depth slots of two weight rows
  const size_t xs_bytes = (size_t)M * p.C * 4, pair_bytes = (size_t)p.C * 4;
  int depth = (int)((204 * 1024 - xs_bytes) / (8 * pair_bytes));  // 227 KB less the static arrays (one state tile)
  depth = depth > 4 ? 4 : depth;
  if (depth < 2) return fail(FRWKV_ERR_UNSUPPORTED, "tmix_decode_layer: rows x channels too large for one CTA");
  p.depth = depth;
  p.ring_bytes = (uint32_t)((size_t)8 * depth * pair_bytes);
  const size_t smem = xs_bytes + (size_t)8 * depth * pair_bytes;
  if (!ready[device]) {
    int cooperative = 0;
    cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device);
    if (!cooperative) return fail(FRWKV_ERR_UNSUPPORTED, "tmix_decode_layer: the device has no cooperative launch");
    cudaDeviceGetAttribute(&sm_counts[device], cudaDevAttrMultiProcessorCount, device);
    ready[device] = true;
  }
  // (the attribute is per kernel instantiation: set it whenever the request exceeds the default)
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(tmix_decode_layer_kernel<io_t, M>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "tmix_decode_layer: %s", cudaGetErrorString(e));
  }
  const int grid = sm_counts[device];
  if (grid < 16) return fail(FRWKV_ERR_UNSUPPORTED, "tmix_decode_layer: needs at least 16 SMs");
  const long long w1[7] = {p.C, p.C, p.C, p.rank[0], p.rank[1], p.rank[2], p.rank[3]};
  const long long w2[4] = {p.rank[0], p.rank[1], p.rank[2], p.rank[3]};
  split_ctas(grid, w1, 7, p.first1);
  split_ctas(grid, w2, 4, p.first2);
  void* args[] = {&p};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(tmix_decode_layer_kernel<io_t, M>), dim3(grid),
                                              dim3(kLayerThreads), args, smem, stream);
  if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "tmix_decode_layer: %s", cudaGetErrorString(e));
  return check_launch("tmix_decode_layer_kernel");
}

template <typename io_t>
int launch_layer_rows(DecodeLayerParams& p, int rows, cudaStream_t stream) {
  switch (rows) {
    case 1: return launch_layer<io_t, 1>(p, stream);
    case 2: return launch_layer<io_t, 2>(p, stream);
    case 3: return launch_layer<io_t, 3>(p, stream);
    case 4: return launch_layer<io_t, 4>(p, stream);
    case 5: return launch_layer<io_t, 5>(p, stream);
    case 6: return launch_layer<io_t, 6>(p, stream);
    case 7: return launch_layer<io_t, 7>(p, stream);
    case 8: return launch_layer<io_t, 8>(p, stream);
  }
  return fail(FRWKV_ERR_INVALID_ARGUMENT, "tmix_decode_layer: 1..8 rows");
}

}  // namespace
}  // namespace frwkv

extern "C" size_t frwkv_tmix_decode_layer_workspace_bytes(int rows, int channels, const int* rank) {
  if (rows <= 0 || channels <= 0 || rank == nullptr) return 0;
  size_t ranks = 0;
  for (int i = 0; i < 4; ++i) ranks += (size_t)(rank[i] > 0 ? rank[i] : 0);
  return ((size_t)8 * rows * channels + (size_t)rows * ranks) * 2;
}

extern "C" int frwkv_tmix_decode_layer_forward(const frwkv_tmix_decode_layer_args* args, const int32_t* state_indices,
                                               const int32_t* metadata_status, int rows, int channels, int num_heads,
                                               float ln_eps, int io_dtype, int32_t* error_flag, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(args != nullptr && state_indices != nullptr, "tmix_decode_layer: null pointer argument");
  const frwkv_tmix_decode_layer_args& a = *args;
  FRWKV_REQUIRE(a.x && a.v_first && a.shift_state_pool && a.state_pool && a.w_r && a.w_k && a.w_v && a.w_o && a.k_k &&
                    a.a0 && a.k_a && a.r_k && a.ln_w && a.ln_b && a.v0 && a.out && a.workspace && a.barrier,
                "tmix_decode_layer: null pointer in the argument block");
  for (int i = 0; i < 6; ++i) FRWKV_REQUIRE(a.mix[i] != nullptr, "tmix_decode_layer: null mix vector %d", i);
  for (int i = 0; i < 4; ++i) {
    FRWKV_REQUIRE(a.w1[i] && a.w2[i], "tmix_decode_layer: null low-rank weight %d", i);
    FRWKV_REQUIRE(a.rank[i] >= 8 && a.rank[i] % 8 == 0 && a.rank[i] <= channels,
                  "tmix_decode_layer: ranks must be multiples of 8 in [8, C]");
  }
  FRWKV_REQUIRE(rows >= 1 && rows <= 8, "tmix_decode_layer: 1..8 rows (one token per sequence)");
  FRWKV_REQUIRE(channels >= 256 && channels % 64 == 0 && num_heads * 64 == channels,
                "tmix_decode_layer: head size 64, C = 64 H >= 256");
  FRWKV_REQUIRE((size_t)rows * channels * 4 <= 200 * 1024, "tmix_decode_layer: rows x channels too large for one CTA");
  DecodeLayerParams p{};
  p.x = a.x; p.v_first = a.v_first; p.shift_pool = a.shift_state_pool; p.state_pool = a.state_pool;
  for (int i = 0; i < 6; ++i) p.mix[i] = a.mix[i];
  p.w_r = a.w_r; p.w_k = a.w_k; p.w_v = a.w_v; p.w_o = a.w_o;
  for (int i = 0; i < 4; ++i) { p.w1[i] = a.w1[i]; p.w2[i] = a.w2[i]; p.rank[i] = a.rank[i]; }
  p.k_k = a.k_k; p.a0 = a.a0; p.k_a = a.k_a; p.r_k = a.r_k; p.ln_w = a.ln_w; p.ln_b = a.ln_b; p.v0 = a.v0;
  p.out = a.out;
  unsigned char* ws = static_cast<unsigned char*>(a.workspace);
  const size_t mc = (size_t)rows * channels * 2;
  p.r = ws; p.k = ws + mc; p.v = ws + 2 * mc; p.wl = ws + 3 * mc; p.a12 = ws + 4 * mc; p.g = ws + 5 * mc;
  p.vres = ws + 6 * mc; p.z = ws + 7 * mc;
  size_t off = 8 * mc;
  for (int i = 0; i < 4; ++i) { p.f[i] = ws + off; off += (size_t)rows * a.rank[i] * 2; }
  p.state_indices = state_indices; p.status = metadata_status;
  p.barrier = a.barrier; p.error_flag = error_flag;
  p.C = channels; p.H = num_heads; p.eps = ln_eps;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype == FRWKV_DTYPE_BF16) return launch_layer_rows<__nv_bfloat16>(p, rows, s);
  if (io_dtype == FRWKV_DTYPE_FP16) return launch_layer_rows<__half>(p, rows, s);
  return fail(FRWKV_ERR_UNSUPPORTED, "tmix_decode_layer: tensors must be float16 or bfloat16");
}
