// Training-side TMix glue around the chunked WKV7 kernel, forward and backward, on dense [B, T, C] 16-bit tensors:
//
//   a_gate         y = sigmoid(a0 + a12)
//   vres_gate      y = v + (v_first - v) * sigmoid(v0 + v12)
//   mix6           y_j = x + (x[t-1] - x) * m_j, j = r, w, k, v, a, g; the row before t = 0 is zero
//   kk_pre         kk = normalize(k * k_k) per head (eps 1e-12); (k * (1 + (a - 1) * k_a), -kk, kk * a)
//   lnx_rkvres_xg  (LayerNorm_head(x) * w + b + (sum_head r * k * r_k) * v) * g, eps 64e-5
//
// Every pass is bound by HBM traffic, so the kernels are organised around 16-byte accesses: a thread owns eight
// adjacent channels, a head of D channels is D / 8 adjacent lanes of one warp (per-head sums are xor-shuffles inside
// that lane group), a warp covers 256 channels (512 contiguous bytes per row and tensor).  The rows are cut into
// contiguous slabs, one CTA of four warps per (channel tile of 256, slab); each warp walks its own quarter of the slab
// row by row.  The passes that also produce a gradient of a [C] parameter (a sum over all B * T rows) keep the column
// sums in registers along the walk, add the four warps in shared memory in a fixed order and write one fp32 partial
// per CTA; reduce_partials_kernel adds the slabs in a fixed order.  The parameter gradients are therefore
// bit-reproducible; the reference accumulates them with fp32 atomics.  Walking contiguous rows also hands mix6 its
// previous row in registers, so x is read once.
//
// Replaces csrc/sm90/tmix/{a_gate,vres_gate,mix6,kk_pre,lnx_rkvres_xg}/pretrain_bf16_{forward,backward}.cu.

#include <cstdlib>

#include "frwkv_common.cuh"

namespace frwkv {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kTileCols = 32 * 8;  // channels of one CTA: every warp covers all of them, for its own rows
constexpr float kNormalizeEps = 1.0e-12f;
constexpr float kLnxEps = 64e-5f;

// ex2.approx and rcp.approx (relative error about 2^-22 each): four instructions instead of the two dozen of an exact
// division, which would make the sigmoid passes instruction-bound; the result is rounded to 16 bits anyway.
__device__ __forceinline__ float sigmoidf_(float x) {
  return rcp_approx(1.f + ex2_approx(fminf(-1.4426950408889634f * x, 126.0f)));
}

template <typename io_t>
__device__ __forceinline__ void load8(const io_t* p, float (&f)[8]) {
  using IO = Io16<io_t>;
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  float2 t;
  t = IO::unpack(u.x); f[0] = t.x; f[1] = t.y;
  t = IO::unpack(u.y); f[2] = t.x; f[3] = t.y;
  t = IO::unpack(u.z); f[4] = t.x; f[5] = t.y;
  t = IO::unpack(u.w); f[6] = t.x; f[7] = t.y;
}

template <typename io_t>
__device__ __forceinline__ void store8(io_t* p, const float (&f)[8]) {
  using IO = Io16<io_t>;
  uint4 u;
  u.x = IO::pack(f[0], f[1]);
  u.y = IO::pack(f[2], f[3]);
  u.z = IO::pack(f[4], f[5]);
  u.w = IO::pack(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ void zero8(float (&f)[8]) {
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] = 0.f;
}

// sum over the kLanes adjacent lanes that hold one head
template <int kLanes>
__device__ __forceinline__ float head_sum(float v) {
#pragma unroll
  for (int o = kLanes / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// The rows of this warp and the eight channels of this lane in a (channel tile, slab) grid.  row_begin >= row_end for
// a warp past the last row.
struct Walk {
  long long row_begin, row_end;
  int col;
  bool active;
};
__device__ __forceinline__ Walk my_walk(long long rows, int channels, int rows_per_warp) {
  Walk w;
  w.col = (blockIdx.x * 32 + (threadIdx.x & 31)) * 8;
  w.active = w.col < channels;
  w.row_begin = ((long long)blockIdx.y * kWarps + (threadIdx.x >> 5)) * rows_per_warp;
  w.row_end = w.row_begin + rows_per_warp < rows ? w.row_begin + rows_per_warp : rows;
  return w;
}

// Adds the column sums of the CTA's four warps (warp 0 + 1 + 2 + 3, in that order) and writes the CTA's partial:
// workspace[v][slab][channel].  Every thread of the CTA calls it.
template <int V>
__device__ __forceinline__ void store_partials(float* workspace, int channels, const Walk& w, float (&acc)[V][8]) {
  __shared__ float4 buf[kWarps - 1][2 * V][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp > 0) {
#pragma unroll
    for (int v = 0; v < V; ++v) {
      buf[warp - 1][2 * v][lane] = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
      buf[warp - 1][2 * v + 1][lane] = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
    }
  }
  __syncthreads();
  if (warp != 0 || !w.active) return;
#pragma unroll
  for (int v = 0; v < V; ++v) {
#pragma unroll
    for (int j = 0; j < kWarps - 1; ++j) {
      const float4 lo = buf[j][2 * v][lane], hi = buf[j][2 * v + 1][lane];
      acc[v][0] += lo.x; acc[v][1] += lo.y; acc[v][2] += lo.z; acc[v][3] += lo.w;
      acc[v][4] += hi.x; acc[v][5] += hi.y; acc[v][6] += hi.z; acc[v][7] += hi.w;
    }
    float* p = workspace + ((long long)v * gridDim.y + blockIdx.y) * channels + w.col;
    *reinterpret_cast<float4*>(p) = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
  }
}

struct ReduceTargets {
  void* out[6];
};

// out[v][c] = sum over slabs of workspace[v][slab][c], slabs in ascending order, four interleaved chains
template <typename io_t>
__global__ __launch_bounds__(256) void reduce_partials_kernel(const float* __restrict__ workspace, ReduceTargets targets,
                                                              int slabs, int channels, int vectors) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= (long long)vectors * channels) return;
  const int vec = (int)(i / channels), c = (int)(i % channels);
  const float* p = workspace + (long long)vec * slabs * channels + c;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int s = 0;
  for (; s + 4 <= slabs; s += 4) {
    s0 += p[(long long)s * channels];
    s1 += p[(long long)(s + 1) * channels];
    s2 += p[(long long)(s + 2) * channels];
    s3 += p[(long long)(s + 3) * channels];
  }
  for (; s < slabs; ++s) s0 += p[(long long)s * channels];
  void* dst = targets.out[0];
#pragma unroll
  for (int j = 1; j < 6; ++j)
    if (vec == j) dst = targets.out[j];
  static_cast<io_t*>(dst)[c] = Io16<io_t>::store((s0 + s1) + (s2 + s3));
}

// ---- a_gate --------------------------------------------------------------------------------------------------------
// Rows whose loads a lane of the a_gate kernels keeps in flight together.  Measured at B=8, T=4096, C=4096 (forward /
// backward): 2 rows 100 / 162 us, 4 rows 100 / 213 us (the registers of four rows cost the backward three of its seven
// CTAs per SM).
#ifndef FRWKV_GATE_ROWS
#define FRWKV_GATE_ROWS 2
#endif
constexpr int kGateRows = FRWKV_GATE_ROWS;
template <typename io_t>
__global__ __launch_bounds__(kThreads) void a_gate_forward_kernel(const io_t* __restrict__ a0,
                                                                  const io_t* __restrict__ a12, io_t* __restrict__ out,
                                                                  long long rows, int channels, int rows_per_warp) {
  const Walk w = my_walk(rows, channels, rows_per_warp);
  if (!w.active) return;
  float z0[8];
  load8(a0 + w.col, z0);
  for (long long row = w.row_begin; row < w.row_end; row += kGateRows) {  // kGateRows rows' loads in flight together
    const long long at = row * channels + w.col;
    float t[kGateRows][8];
#pragma unroll
    for (int u = 0; u < kGateRows; ++u)
      if (row + u < w.row_end) load8(a12 + at + u * (long long)channels, t[u]);
#pragma unroll
    for (int u = 0; u < kGateRows; ++u) {
      if (row + u < w.row_end) {
#pragma unroll
        for (int e = 0; e < 8; ++e) t[u][e] = sigmoidf_(z0[e] + t[u][e]);
        store8(out + at + u * (long long)channels, t[u]);
      }
    }
  }
}

template <typename io_t>
__global__ __launch_bounds__(kThreads) void a_gate_backward_kernel(const io_t* __restrict__ grad_out,
                                                                   const io_t* __restrict__ a0,
                                                                   const io_t* __restrict__ a12,
                                                                   io_t* __restrict__ grad_a12,
                                                                   float* __restrict__ workspace, long long rows,
                                                                   int channels, int rows_per_warp) {
  const Walk w = my_walk(rows, channels, rows_per_warp);
  float acc[1][8];
  zero8(acc[0]);
  if (w.active) {
    float z0[8];
    load8(a0 + w.col, z0);
    for (long long row = w.row_begin; row < w.row_end; row += kGateRows) {  // kGateRows rows' loads in flight together
      const long long at = row * channels + w.col;
      float z[kGateRows][8], g[kGateRows][8];
#pragma unroll
      for (int u = 0; u < kGateRows; ++u) {
        if (row + u < w.row_end) {
          load8(a12 + at + u * (long long)channels, z[u]);
          load8(grad_out + at + u * (long long)channels, g[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < kGateRows; ++u) {
        if (row + u < w.row_end) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float y = sigmoidf_(z0[e] + z[u][e]);
            g[u][e] *= y * (1.f - y);
            acc[0][e] += g[u][e];
          }
          store8(grad_a12 + at + u * (long long)channels, g[u]);
        }
      }
    }
  }
  store_partials<1>(workspace, channels, w, acc);
}

// ---- vres_gate -----------------------------------------------------------------------------------------------------
template <typename io_t>
__global__ __launch_bounds__(kThreads) void vres_gate_backward_kernel(
    const io_t* __restrict__ grad_out, const io_t* __restrict__ v, const io_t* __restrict__ v_first,
    const io_t* __restrict__ v0, const io_t* __restrict__ v12, io_t* __restrict__ grad_v,
    io_t* __restrict__ grad_v_first, io_t* __restrict__ grad_v12, float* __restrict__ workspace, long long rows,
    int channels, int rows_per_warp) {
  const Walk w = my_walk(rows, channels, rows_per_warp);
  float acc[1][8];
  zero8(acc[0]);
  if (w.active) {
    float z0[8];
    load8(v0 + w.col, z0);
    for (long long row = w.row_begin; row < w.row_end; row += 2) {  // two rows' loads in flight together
      const long long at = row * channels + w.col;
      const bool second = row + 1 < w.row_end;
      float g[2][8], a[2][8], f[2][8], z[2][8];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u == 1 && !second) break;
        const long long au = at + u * (long long)channels;
        load8(grad_out + au, g[u]);
        load8(v + au, a[u]);
        load8(v_first + au, f[u]);
        load8(v12 + au, z[u]);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u == 1 && !second) break;
        const long long au = at + u * (long long)channels;
        float gz[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float sg = sigmoidf_(z0[e] + z[u][e]);
          gz[e] = g[u][e] * (f[u][e] - a[u][e]) * sg * (1.f - sg);
          acc[0][e] += gz[e];
          f[u][e] = g[u][e] * sg;          // grad of v_first
          a[u][e] = g[u][e] - f[u][e];     // grad of v
        }
        store8(grad_v + au, a[u]);
        store8(grad_v_first + au, f[u]);
        store8(grad_v12 + au, gz);
      }
    }
  }
  store_partials<1>(workspace, channels, w, acc);
}

// ---- mix6 ----------------------------------------------------------------------------------------------------------
struct Six {
  const void* in[6];
  void* out[6];
  // StateTune form (all null in the pretrain form): the row before t = 0 is initial[b] instead of zero, the last row
  // of every sequence is also written to final_shift[b]; in the backward grad_final[b] joins the gradient of that last
  // row and grad_initial[b] receives the shifted term of row t = 0.  All [B][C].
  const void* initial = nullptr;
  void* final_shift = nullptr;
  const void* grad_final = nullptr;
  void* grad_initial = nullptr;
};

// The six mix vectors of the CTA's 256 channels as fp32 in shared memory (all four warps walk the same channels; a
// lane reads its own eight values, no bank conflict).  Every thread of the CTA calls it.
using MixTable = float4[6][2][32];
template <typename io_t>
__device__ __forceinline__ void stage_mix(MixTable& table, const void* const* vectors, const Walk& w) {
  if (threadIdx.x < 32 && w.active) {
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      float f[8];
      load8(static_cast<const io_t*>(vectors[j]) + w.col, f);
      table[j][0][threadIdx.x] = make_float4(f[0], f[1], f[2], f[3]);
      table[j][1][threadIdx.x] = make_float4(f[4], f[5], f[6], f[7]);
    }
  }
  __syncthreads();
}
// volatile: the compiler would otherwise keep all 48 loop-invariant values in registers, which is what the table is
// there to avoid
__device__ __forceinline__ float4 lds_volatile(const float4* p) {
  float4 v;
  asm volatile("ld.volatile.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"((unsigned)__cvta_generic_to_shared(p)));
  return v;
}
__device__ __forceinline__ void read_mix(const MixTable& table, int j, float (&m)[8]) {
  const float4 lo = lds_volatile(&table[j][0][threadIdx.x & 31]), hi = lds_volatile(&table[j][1][threadIdx.x & 31]);
  m[0] = lo.x; m[1] = lo.y; m[2] = lo.z; m[3] = lo.w;
  m[4] = hi.x; m[5] = hi.y; m[6] = hi.z; m[7] = hi.w;
}

// Rows are b * T + t; a slab may cross sequence boundaries, the row before t = 0 is zero.  The next row's x is
// requested before the current row's six stores, so that a warp always has a read in flight.
template <typename io_t>
__global__ __launch_bounds__(kThreads) void mix6_forward_kernel(const io_t* __restrict__ x, Six mix, long long rows,
                                                                int seq_len, int channels, int rows_per_warp) {
  __shared__ MixTable m_s;
  const Walk w = my_walk(rows, channels, rows_per_warp);
  stage_mix<io_t>(m_s, mix.in, w);
  if (!w.active || w.row_begin >= w.row_end) return;
  float prev[8], cur[8], next[8];
  int t = (int)(w.row_begin % seq_len);
  long long b = w.row_begin / seq_len;
  const io_t* initial = static_cast<const io_t*>(mix.initial);
  io_t* final_shift = static_cast<io_t*>(mix.final_shift);
  if (t != 0) load8(x + (w.row_begin - 1) * channels + w.col, prev);
  load8(x + w.row_begin * channels + w.col, cur);
  for (long long row = w.row_begin; row < w.row_end; ++row) {
    const long long at = row * channels + w.col;
    if (row + 1 < w.row_end) load8(x + at + channels, next);
    if (t == 0) {
      if (initial != nullptr) load8(initial + b * channels + w.col, prev);
      else zero8(prev);
    }
    float xx[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) xx[e] = prev[e] - cur[e];
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      float y[8], m[8];
      read_mix(m_s, j, m);
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = fmaf(xx[e], m[e], cur[e]);
      store8(static_cast<io_t*>(mix.out[j]) + at, y);
    }
    if (t == seq_len - 1 && final_shift != nullptr) store8(final_shift + b * channels + w.col, cur);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      prev[e] = cur[e];
      cur[e] = next[e];
    }
    if (++t == seq_len) {
      t = 0;
      ++b;
    }
  }
}

// grad_x[t] = sum_j g_j[t] (1 - m_j) + sum_j g_j[t+1] m_j (second term only inside the sequence);
// grad_m_j = sum_rows g_j (x[t-1] - x[t]).  mix.in = the six upstream gradients, mix.out = the six mix vectors.
// kShift = false (pretrain form) compiles the shift-state pointers away: with them the walk spills and runs a quarter
// slower.
template <typename io_t, bool kShift>
__device__ __forceinline__ void mix6_backward_walk(const io_t* __restrict__ x, const Six& mix,
                                                   io_t* __restrict__ grad_x, float (&dm)[6][8], const Walk& w,
                                                   const MixTable& m_s, long long rows, int seq_len, int channels) {
  float prev[8], carry[8];
  int t = (int)(w.row_begin % seq_len);
  long long b = w.row_begin / seq_len;
  const io_t* initial = kShift ? static_cast<const io_t*>(mix.initial) : nullptr;
  const io_t* grad_final = kShift ? static_cast<const io_t*>(mix.grad_final) : nullptr;
  io_t* grad_initial = kShift ? static_cast<io_t*>(mix.grad_initial) : nullptr;
  if (t != 0) load8(x + (w.row_begin - 1) * channels + w.col, prev);
  zero8(carry);
  for (long long row = w.row_begin; row < w.row_end; ++row) {
    const long long at = row * channels + w.col;
    float cur[8], xx[8], direct[8], shifted[8];
    load8(x + at, cur);
    zero8(direct);
    zero8(shifted);
    if (t == 0) {
      if (initial != nullptr) load8(initial + b * channels + w.col, prev);
      else zero8(prev);
    }
    if (t == seq_len - 1 && grad_final != nullptr) load8(grad_final + b * channels + w.col, direct);
#pragma unroll
    for (int e = 0; e < 8; ++e) xx[e] = prev[e] - cur[e];
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      float g[8], m[8];
      load8(static_cast<const io_t*>(mix.in[j]) + at, g);
      read_mix(m_s, j, m);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dm[j][e] = fmaf(g[e], xx[e], dm[j][e]);
        shifted[e] = fmaf(g[e], m[e], shifted[e]);
        direct[e] += g[e];
      }
    }
    if (row > w.row_begin) {  // the previous row is complete once this row's shifted term is known
#pragma unroll
      for (int e = 0; e < 8; ++e) carry[e] += t != 0 ? shifted[e] : 0.f;
      store8(grad_x + at - channels, carry);
    }
    if (t == 0 && grad_initial != nullptr) store8(grad_initial + b * channels + w.col, shifted);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      carry[e] = direct[e] - shifted[e];
      prev[e] = cur[e];
    }
    if (++t == seq_len) {
      t = 0;
      ++b;
    }
  }
  if (w.row_end < rows && t != 0) {  // the slab's last row takes its shifted term from the next slab's first row
    const long long at = w.row_end * channels + w.col;
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      float g[8], m[8];
      load8(static_cast<const io_t*>(mix.in[j]) + at, g);
      read_mix(m_s, j, m);
#pragma unroll
      for (int e = 0; e < 8; ++e) carry[e] = fmaf(g[e], m[e], carry[e]);
    }
  }
  store8(grad_x + (w.row_end - 1) * channels + w.col, carry);
}

template <typename io_t, int kMinCtas, bool kShift>
__global__ __launch_bounds__(kThreads, kMinCtas) void mix6_backward_kernel(const io_t* __restrict__ x, Six mix,
                                                                 io_t* __restrict__ grad_x,
                                                                 float* __restrict__ workspace, long long rows,
                                                                 int seq_len, int channels, int rows_per_warp) {
  __shared__ MixTable m_s;
  const Walk w = my_walk(rows, channels, rows_per_warp);
  stage_mix<io_t>(m_s, mix.out, w);
  float dm[6][8];
#pragma unroll
  for (int j = 0; j < 6; ++j) zero8(dm[j]);
  if (w.active && w.row_begin < w.row_end)
    mix6_backward_walk<io_t, kShift>(x, mix, grad_x, dm, w, m_s, rows, seq_len, channels);
  store_partials<6>(workspace, channels, w, dm);
}

// ---- kk_pre --------------------------------------------------------------------------------------------------------
// A head is kLanes = D / 8 adjacent lanes.  Lanes past the last channel keep running the row loop with their loads and
// stores switched off so that the full-mask shuffles stay converged.

template <typename io_t, int kLanes>
__global__ __launch_bounds__(kThreads) void kk_pre_forward_kernel(
    const io_t* __restrict__ k, const io_t* __restrict__ k_k, const io_t* __restrict__ a, const io_t* __restrict__ k_a,
    io_t* __restrict__ new_k, io_t* __restrict__ neg_kk, io_t* __restrict__ kka, float* __restrict__ inv_norm,
    long long rows, int channels, int rows_per_warp) {
  const Walk w = my_walk(rows, channels, rows_per_warp);
  const int heads = channels / (kLanes * 8), head = w.col / (kLanes * 8);
  float ks[8], ka[8];
  zero8(ks);
  zero8(ka);
  if (w.active) {
    load8(k_k + w.col, ks);
    load8(k_a + w.col, ka);
  }
  for (long long row = w.row_begin; row < w.row_end; ++row) {
    const long long at = row * channels + w.col;
    float kv[8], av[8], u[8];
    zero8(kv);
    zero8(av);
    if (w.active) {
      load8(k + at, kv);
      load8(a + at, av);
    }
    float sq = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      u[e] = kv[e] * ks[e];
      sq = fmaf(u[e], u[e], sq);
    }
    const float inv = 1.f / fmaxf(sqrtf(head_sum<kLanes>(sq)), kNormalizeEps);
    if (!w.active) continue;
    if ((threadIdx.x & (kLanes - 1)) == 0) inv_norm[row * heads + head] = inv;
    float o0[8], o1[8], o2[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float kk = u[e] * inv;
      o0[e] = kv[e] * fmaf(av[e], ka[e], 1.f - ka[e]);
      o1[e] = -kk;
      o2[e] = kk * av[e];
    }
    store8(new_k + at, o0);
    store8(neg_kk + at, o1);
    store8(kka + at, o2);
  }
}

// d kk / d u = inv (I - kk kk^T) while the norm is above eps, inv * I below it (the clamp has no gradient).
template <typename io_t, int kLanes>
__global__ __launch_bounds__(kThreads) void kk_pre_backward_kernel(
    const io_t* __restrict__ g_new_k, const io_t* __restrict__ g_neg_kk, const io_t* __restrict__ g_kka,
    const io_t* __restrict__ k, const io_t* __restrict__ k_k, const io_t* __restrict__ a, const io_t* __restrict__ k_a,
    const float* __restrict__ inv_norm, io_t* __restrict__ grad_k, io_t* __restrict__ grad_a,
    float* __restrict__ workspace, long long rows, int channels, int rows_per_warp) {
  const Walk w = my_walk(rows, channels, rows_per_warp);
  const int heads = channels / (kLanes * 8), head = w.col / (kLanes * 8);
  float ks[8], ka[8], acc[2][8];  // acc: d k_k, d k_a
  zero8(ks);
  zero8(ka);
  zero8(acc[0]);
  zero8(acc[1]);
  if (w.active) {
    load8(k_k + w.col, ks);
    load8(k_a + w.col, ka);
  }
  for (long long row = w.row_begin; row < w.row_end; ++row) {
    const long long at = row * channels + w.col;
    float kv[8], av[8], gn[8], gneg[8], gka[8], kk[8], gkk[8];
    zero8(kv);
    zero8(av);
    zero8(gn);
    zero8(gneg);
    zero8(gka);
    float inv = 0.f;
    if (w.active) {
      load8(k + at, kv);
      load8(a + at, av);
      load8(g_new_k + at, gn);
      load8(g_neg_kk + at, gneg);
      load8(g_kka + at, gka);
      inv = __ldg(inv_norm + row * heads + head);
    }
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      kk[e] = kv[e] * ks[e] * inv;
      gkk[e] = fmaf(gka[e], av[e], -gneg[e]);
      dot = fmaf(kk[e], gkk[e], dot);
    }
    dot = head_sum<kLanes>(dot);
    if (!w.active) continue;
    if (!(inv < 1.f / kNormalizeEps)) dot = 0.f;
    float gk[8], ga[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float gu = inv * fmaf(-kk[e], dot, gkk[e]);
      gk[e] = fmaf(gn[e], fmaf(av[e], ka[e], 1.f - ka[e]), gu * ks[e]);
      ga[e] = fmaf(gn[e] * kv[e], ka[e], gka[e] * kk[e]);
      acc[0][e] = fmaf(gu, kv[e], acc[0][e]);
      acc[1][e] = fmaf(gn[e] * kv[e], av[e] - 1.f, acc[1][e]);
    }
    store8(grad_k + at, gk);
    store8(grad_a + at, ga);
  }
  store_partials<2>(workspace, channels, w, acc);
}

// ---- lnx_rkvres_xg -------------------------------------------------------------------------------------------------
template <typename io_t, int kLanes>
__global__ __launch_bounds__(kThreads) void lnx_forward_kernel(
    const io_t* __restrict__ x, const io_t* __restrict__ r, const io_t* __restrict__ k, const io_t* __restrict__ v,
    const io_t* __restrict__ r_k, const io_t* __restrict__ weight, const io_t* __restrict__ bias,
    const io_t* __restrict__ g, io_t* __restrict__ out, float* __restrict__ mean_out, float* __restrict__ rstd_out,
    long long rows, int channels, int rows_per_warp) {
  constexpr float kInvD = 1.f / (kLanes * 8);
  const Walk w = my_walk(rows, channels, rows_per_warp);
  const int heads = channels / (kLanes * 8), head = w.col / (kLanes * 8);
  float rk[8], wt[8], bs[8];
  zero8(rk);
  zero8(wt);
  zero8(bs);
  if (w.active) {
    load8(r_k + w.col, rk);
    load8(weight + w.col, wt);
    load8(bias + w.col, bs);
  }
  for (long long row = w.row_begin; row < w.row_end; ++row) {
    const long long at = row * channels + w.col;
    float xv[8], rv[8], kv[8], vv[8], gv[8];
    zero8(xv);
    zero8(rv);
    zero8(kv);
    if (w.active) {
      load8(x + at, xv);
      load8(r + at, rv);
      load8(k + at, kv);
      load8(v + at, vv);
      load8(g + at, gv);
    }
    float sum = 0.f, s = 0.f, sq = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      sum += xv[e];
      s = fmaf(rv[e] * kv[e], rk[e], s);
    }
    const float mean = head_sum<kLanes>(sum) * kInvD;
    s = head_sum<kLanes>(s);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      xv[e] -= mean;
      sq = fmaf(xv[e], xv[e], sq);
    }
    const float rstd = rsqrtf(head_sum<kLanes>(sq) * kInvD + kLnxEps);
    if (!w.active) continue;
    if ((threadIdx.x & (kLanes - 1)) == 0) {
      mean_out[row * heads + head] = mean;
      rstd_out[row * heads + head] = rstd;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) xv[e] = (fmaf(xv[e] * rstd, wt[e], bs[e]) + s * vv[e]) * gv[e];
    store8(out + at, xv);
  }
}

template <typename io_t, int kLanes>
__global__ __launch_bounds__(kThreads) void lnx_backward_kernel(
    const io_t* __restrict__ grad_out, const io_t* __restrict__ x, const io_t* __restrict__ r,
    const io_t* __restrict__ k, const io_t* __restrict__ v, const io_t* __restrict__ r_k,
    const io_t* __restrict__ weight, const io_t* __restrict__ bias, const io_t* __restrict__ g,
    const float* __restrict__ mean_in, const float* __restrict__ rstd_in, io_t* __restrict__ grad_x,
    io_t* __restrict__ grad_r, io_t* __restrict__ grad_k, io_t* __restrict__ grad_v, io_t* __restrict__ grad_g,
    float* __restrict__ workspace, long long rows, int channels, int rows_per_warp) {
  constexpr float kInvD = 1.f / (kLanes * 8);
  const Walk w = my_walk(rows, channels, rows_per_warp);
  const int heads = channels / (kLanes * 8), head = w.col / (kLanes * 8);
  float rk[8], wt[8], bs[8], acc[3][8];  // acc: d r_k, d weight, d bias
  zero8(rk);
  zero8(wt);
  zero8(bs);
  zero8(acc[0]);
  zero8(acc[1]);
  zero8(acc[2]);
  if (w.active) {
    load8(r_k + w.col, rk);
    load8(weight + w.col, wt);
    load8(bias + w.col, bs);
  }
  for (long long row = w.row_begin; row < w.row_end; ++row) {
    const long long at = row * channels + w.col;
    float go[8], xh[8], rv[8], kv[8], vv[8], gv[8];
    zero8(go);
    zero8(xh);
    zero8(rv);
    zero8(kv);
    zero8(vv);
    zero8(gv);
    float mean = 0.f, rstd = 0.f;
    if (w.active) {
      load8(grad_out + at, go);
      load8(x + at, xh);
      load8(r + at, rv);
      load8(k + at, kv);
      load8(v + at, vv);
      load8(g + at, gv);
      mean = __ldg(mean_in + row * heads + head);
      rstd = __ldg(rstd_in + row * heads + head);
    }
    float s = 0.f, gs = 0.f, m1 = 0.f, m2 = 0.f;
    float gy[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      xh[e] = (xh[e] - mean) * rstd;
      gy[e] = go[e] * gv[e];
      s = fmaf(rv[e] * kv[e], rk[e], s);
      gs = fmaf(gy[e], vv[e], gs);
      const float gxh = gy[e] * wt[e];
      m1 += gxh;
      m2 = fmaf(gxh, xh[e], m2);
    }
    s = head_sum<kLanes>(s);
    gs = head_sum<kLanes>(gs);
    m1 = head_sum<kLanes>(m1) * kInvD;
    m2 = head_sum<kLanes>(m2) * kInvD;
    if (!w.active) continue;
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      o[e] = go[e] * (fmaf(xh[e], wt[e], bs[e]) + s * vv[e]);  // grad of g
      acc[1][e] = fmaf(gy[e], xh[e], acc[1][e]);
      acc[2][e] += gy[e];
      acc[0][e] = fmaf(gs * rv[e], kv[e], acc[0][e]);
    }
    store8(grad_g + at, o);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = rstd * (fmaf(gy[e], wt[e], -m1) - xh[e] * m2);
    store8(grad_x + at, o);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = gs * kv[e] * rk[e];
    store8(grad_r + at, o);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = gs * rv[e] * rk[e];
    store8(grad_k + at, o);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = gy[e] * s;
    store8(grad_v + at, o);
  }
  store_partials<3>(workspace, channels, w, acc);
}

// ---- host side -----------------------------------------------------------------------------------------------------
struct Plan {
  int col_tiles, slabs, rows_per_warp;
};
// One wave: as many CTAs as are resident at once (ctas_per_sm of this kernel on every SM), so that no second, partly
// filled wave follows; a slab is four warps' rows and holds at least one row.
Plan make_plan(long long rows, int channels, int ctas_per_sm, int sms) {
  Plan p;
  p.col_tiles = (channels + kTileCols - 1) / kTileCols;
  long long slabs = (long long)sms * ctas_per_sm / p.col_tiles;
  const long long most = (rows + kWarps - 1) / kWarps;
  if (slabs > most) slabs = most;
  if (slabs < 1) slabs = 1;
  p.rows_per_warp = (int)((rows + slabs * kWarps - 1) / (slabs * kWarps));
  p.slabs = (int)((rows + (long long)p.rows_per_warp * kWarps - 1) / ((long long)p.rows_per_warp * kWarps));
  return p;
}
constexpr int kMaxCtasPerSm = 16;  // 2048 threads
int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        n <= 0)
      n = 148;
    sms = n;
  }
  return sms;
}
// the slab count never exceeds this one, whatever the kernel
long long max_slabs(long long rows, int channels) { return make_plan(rows, channels, kMaxCtasPerSm, sm_count()).slabs; }

// Launches a row-walking kernel (its last parameter is rows_per_warp) on one wave of CTAs and returns the plan used.
template <typename... KArgs, typename... Args>
Plan launch_walk(void (*kernel)(KArgs...), long long rows, int channels, cudaStream_t s, Args... args) {
  int resident = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, kThreads, 0) != cudaSuccess || resident < 1)
    resident = 4;
  if (resident > kMaxCtasPerSm) resident = kMaxCtasPerSm;
  const Plan plan = make_plan(rows, channels, resident, sm_count());
  kernel<<<dim3(plan.col_tiles, plan.slabs), kThreads, 0, s>>>(args..., plan.rows_per_warp);
  return plan;
}

template <typename io_t>
int reduce_partials(const float* workspace, const ReduceTargets& targets, const Plan& plan, int channels, int vectors,
                    cudaStream_t s) {
  const long long n = (long long)vectors * channels;
  reduce_partials_kernel<io_t><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(workspace, targets, plan.slabs, channels,
                                                                          vectors);
  return check_launch("reduce_partials_kernel");
}

int check_dense(const char* name, long long rows, int channels, long long workspace_floats, int vectors) {
  if (rows <= 0 || channels <= 0) return fail(FRWKV_ERR_INVALID_ARGUMENT, "%s: sizes must be positive", name);
  if (channels % 8 != 0) return fail(FRWKV_ERR_INVALID_ARGUMENT, "%s: channel count must be a multiple of 8", name);
  if (rows > 0x7fffffffLL) return fail(FRWKV_ERR_INVALID_ARGUMENT, "%s: too many rows", name);
  if (vectors > 0 && workspace_floats < (long long)vectors * max_slabs(rows, channels) * channels)
    return fail(FRWKV_ERR_INVALID_ARGUMENT, "%s: workspace is smaller than frwkv_pretrain_workspace_floats", name);
  return FRWKV_OK;
}

int check_heads(const char* name, int channels, int head_size) {
  if (head_size != 64 && head_size != 128 && head_size != 256)
    return fail(FRWKV_ERR_INVALID_ARGUMENT, "%s: head_size must be one of 64, 128, or 256", name);
  if (channels % head_size != 0)
    return fail(FRWKV_ERR_INVALID_ARGUMENT, "%s: channel count must be divisible by head_size", name);
  return FRWKV_OK;
}

}  // namespace
}  // namespace frwkv

#define FRWKV_TRAIN_IO(io_dtype, NAME, ...)                                                      \
  if ((io_dtype) == FRWKV_DTYPE_BF16) {                                                          \
    using io_t = __nv_bfloat16;                                                                  \
    __VA_ARGS__                                                                                  \
  } else if ((io_dtype) == FRWKV_DTYPE_FP16) {                                                   \
    using io_t = __half;                                                                         \
    __VA_ARGS__                                                                                  \
  } else {                                                                                       \
    return ::frwkv::fail(FRWKV_ERR_UNSUPPORTED, NAME ": tensors must be float16 or bfloat16");   \
  }
// the head size picks the lane count of a head: 8, 16 or 32
#define FRWKV_TRAIN_LANES(head_size, ...)          \
  if ((head_size) == 64) {                         \
    constexpr int kLanes = 8;                      \
    __VA_ARGS__                                    \
  } else if ((head_size) == 128) {                 \
    constexpr int kLanes = 16;                     \
    __VA_ARGS__                                    \
  } else {                                         \
    constexpr int kLanes = 32;                     \
    __VA_ARGS__                                    \
  }
#define P(T, ptr) static_cast<T*>(ptr)
#define CP(T, ptr) static_cast<const T*>(ptr)

extern "C" long long frwkv_pretrain_workspace_floats(long long rows, int channels, int vectors) {
  if (rows <= 0 || channels <= 0 || vectors <= 0) return 0;
  return (long long)vectors * frwkv::max_slabs(rows, channels) * channels;
}

extern "C" int frwkv_pretrain_a_gate_forward(const void* a0, const void* a12, void* out, long long rows, int channels,
                                             int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(a0 && a12 && out, "pretrain_a_gate: null pointer argument");
  if (int rc = check_dense("pretrain_a_gate", rows, channels, 0, 0)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_TRAIN_IO(io_dtype, "pretrain_a_gate", {
    launch_walk(a_gate_forward_kernel<io_t>, rows, channels, s, CP(io_t, a0), CP(io_t, a12), P(io_t, out), rows,
                channels);
    return check_launch("a_gate_forward_kernel");
  })
}

extern "C" int frwkv_pretrain_a_gate_backward(const void* grad_out, const void* a0, const void* a12, void* grad_a0,
                                              void* grad_a12, float* workspace, long long workspace_floats,
                                              long long rows, int channels, int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(grad_out && a0 && a12 && grad_a0 && grad_a12 && workspace, "pretrain_a_gate: null pointer argument");
  if (int rc = check_dense("pretrain_a_gate", rows, channels, workspace_floats, 1)) return rc;
  Plan plan;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  ReduceTargets targets{{grad_a0}};
  FRWKV_TRAIN_IO(io_dtype, "pretrain_a_gate", {
    plan = launch_walk(a_gate_backward_kernel<io_t>, rows, channels, s, 
        CP(io_t, grad_out), CP(io_t, a0), CP(io_t, a12), P(io_t, grad_a12), workspace, rows, channels);
    if (int rc = check_launch("a_gate_backward_kernel")) return rc;
    return reduce_partials<io_t>(workspace, targets, plan, channels, 1, s);
  })
}

extern "C" int frwkv_pretrain_vres_gate_backward(const void* grad_out, const void* v, const void* v_first,
                                                 const void* v0, const void* v12, void* grad_v, void* grad_v_first,
                                                 void* grad_v0, void* grad_v12, float* workspace,
                                                 long long workspace_floats, long long rows, int channels,
                                                 int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(grad_out && v && v_first && v0 && v12 && grad_v && grad_v_first && grad_v0 && grad_v12 && workspace,
                "pretrain_vres_gate: null pointer argument");
  if (int rc = check_dense("pretrain_vres_gate", rows, channels, workspace_floats, 1)) return rc;
  Plan plan;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  ReduceTargets targets{{grad_v0}};
  FRWKV_TRAIN_IO(io_dtype, "pretrain_vres_gate", {
    plan = launch_walk(vres_gate_backward_kernel<io_t>, rows, channels, s, 
        CP(io_t, grad_out), CP(io_t, v), CP(io_t, v_first), CP(io_t, v0), CP(io_t, v12), P(io_t, grad_v),
        P(io_t, grad_v_first), P(io_t, grad_v12), workspace, rows, channels);
    if (int rc = check_launch("vres_gate_backward_kernel")) return rc;
    return reduce_partials<io_t>(workspace, targets, plan, channels, 1, s);
  })
}

static int mix6_forward_impl(const void* x, const void* initial, const void* const* mix, void* const* out,
                             void* final_shift, long long batch, int seq_len, int channels, int io_dtype,
                             frwkv_stream_t stream) {
  using namespace frwkv;
  FRWKV_REQUIRE(x && mix && out, "pretrain_mix6: null pointer argument");
  FRWKV_REQUIRE(batch > 0 && seq_len > 0, "pretrain_mix6: sizes must be positive");
  const long long rows = batch * seq_len;
  if (int rc = check_dense("pretrain_mix6", rows, channels, 0, 0)) return rc;
  Six six;
  for (int j = 0; j < 6; ++j) {
    FRWKV_REQUIRE(mix[j] && out[j], "pretrain_mix6: null pointer argument");
    six.in[j] = mix[j];
    six.out[j] = out[j];
  }
  six.initial = initial;
  six.final_shift = final_shift;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_TRAIN_IO(io_dtype, "pretrain_mix6", {
    launch_walk(mix6_forward_kernel<io_t>, rows, channels, s, CP(io_t, x), six, rows, seq_len,
                                                                                   channels);
    return check_launch("mix6_forward_kernel");
  })
}

extern "C" int frwkv_pretrain_mix6_forward(const void* x, const void* const* mix, void* const* out, long long batch,
                                           int seq_len, int channels, int io_dtype, frwkv_stream_t stream) {
  frwkv::clear_error();
  return mix6_forward_impl(x, nullptr, mix, out, nullptr, batch, seq_len, channels, io_dtype, stream);
}

extern "C" int frwkv_statetune_mix6_forward(const void* x, const void* initial_shift, const void* const* mix,
                                            void* const* out, void* final_shift, long long batch, int seq_len,
                                            int channels, int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(initial_shift && final_shift, "statetune_mix6: null pointer argument");
  return mix6_forward_impl(x, initial_shift, mix, out, final_shift, batch, seq_len, channels, io_dtype, stream);
}

static int mix6_backward_impl(const void* const* grad_out, const void* grad_final, const void* x, const void* initial,
                              const void* const* mix, void* grad_x, void* grad_initial, void* const* grad_mix,
                              float* workspace, long long workspace_floats, long long batch, int seq_len,
                              int channels, int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  FRWKV_REQUIRE(grad_out && x && mix && grad_x && grad_mix && workspace, "pretrain_mix6: null pointer argument");
  FRWKV_REQUIRE(batch > 0 && seq_len > 0, "pretrain_mix6: sizes must be positive");
  const long long rows = batch * seq_len;
  if (int rc = check_dense("pretrain_mix6", rows, channels, workspace_floats, 6)) return rc;
  Six six;
  ReduceTargets targets;
  for (int j = 0; j < 6; ++j) {
    FRWKV_REQUIRE(grad_out[j] && mix[j] && grad_mix[j], "pretrain_mix6: null pointer argument");
    six.in[j] = grad_out[j];
    six.out[j] = const_cast<void*>(mix[j]);
    targets.out[j] = grad_mix[j];
  }
  six.initial = initial;
  six.grad_final = grad_final;
  six.grad_initial = grad_initial;
  Plan plan;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_TRAIN_IO(io_dtype, "pretrain_mix6", {
    // register budget of the walk: 3 CTAs per SM (168 registers, a few spilled words); 2 CTAs without spills measured
    // slower
    const bool shift = initial != nullptr;  // StateTune form
    if (shift)
      plan = launch_walk(mix6_backward_kernel<io_t, 3, true>, rows, channels, s, CP(io_t, x), six, P(io_t, grad_x),
                         workspace, rows, seq_len, channels);
    else
      plan = launch_walk(mix6_backward_kernel<io_t, 3, false>, rows, channels, s, CP(io_t, x), six, P(io_t, grad_x),
                         workspace, rows, seq_len, channels);
    if (int rc = check_launch("mix6_backward_kernel")) return rc;
    return reduce_partials<io_t>(workspace, targets, plan, channels, 6, s);
  })
}

extern "C" int frwkv_pretrain_mix6_backward(const void* const* grad_out, const void* x, const void* const* mix,
                                            void* grad_x, void* const* grad_mix, float* workspace,
                                            long long workspace_floats, long long batch, int seq_len, int channels,
                                            int io_dtype, frwkv_stream_t stream) {
  frwkv::clear_error();
  return mix6_backward_impl(grad_out, nullptr, x, nullptr, mix, grad_x, nullptr, grad_mix, workspace, workspace_floats,
                            batch, seq_len, channels, io_dtype, stream);
}

extern "C" int frwkv_statetune_mix6_backward(const void* const* grad_out, const void* grad_final_shift, const void* x,
                                             const void* initial_shift, const void* const* mix, void* grad_x,
                                             void* grad_initial_shift, void* const* grad_mix, float* workspace,
                                             long long workspace_floats, long long batch, int seq_len, int channels,
                                             int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(grad_final_shift && initial_shift && grad_initial_shift, "statetune_mix6: null pointer argument");
  return mix6_backward_impl(grad_out, grad_final_shift, x, initial_shift, mix, grad_x, grad_initial_shift, grad_mix,
                            workspace, workspace_floats, batch, seq_len, channels, io_dtype, stream);
}

extern "C" int frwkv_pretrain_kk_pre_forward(const void* k, const void* k_k, const void* a, const void* k_a,
                                             void* new_k, void* neg_kk, void* kka, float* inv_norm, long long rows,
                                             int channels, int head_size, int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(k && k_k && a && k_a && new_k && neg_kk && kka && inv_norm, "pretrain_kk_pre: null pointer argument");
  if (int rc = check_dense("pretrain_kk_pre", rows, channels, 0, 0)) return rc;
  if (int rc = check_heads("pretrain_kk_pre", channels, head_size)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_TRAIN_IO(io_dtype, "pretrain_kk_pre", {
    FRWKV_TRAIN_LANES(head_size, {
      launch_walk(kk_pre_forward_kernel<io_t, kLanes>, rows, channels, s, 
          CP(io_t, k), CP(io_t, k_k), CP(io_t, a), CP(io_t, k_a), P(io_t, new_k), P(io_t, neg_kk), P(io_t, kka),
          inv_norm, rows, channels);
    })
    return check_launch("kk_pre_forward_kernel");
  })
}

extern "C" int frwkv_pretrain_kk_pre_backward(const void* grad_new_k, const void* grad_neg_kk, const void* grad_kka,
                                              const void* k, const void* k_k, const void* a, const void* k_a,
                                              const float* inv_norm, void* grad_k, void* grad_k_k, void* grad_a,
                                              void* grad_k_a, float* workspace, long long workspace_floats,
                                              long long rows, int channels, int head_size, int io_dtype,
                                              frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(grad_new_k && grad_neg_kk && grad_kka && k && k_k && a && k_a && inv_norm && grad_k && grad_k_k &&
                    grad_a && grad_k_a && workspace,
                "pretrain_kk_pre: null pointer argument");
  if (int rc = check_dense("pretrain_kk_pre", rows, channels, workspace_floats, 2)) return rc;
  if (int rc = check_heads("pretrain_kk_pre", channels, head_size)) return rc;
  Plan plan;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  ReduceTargets targets{{grad_k_k, grad_k_a}};
  FRWKV_TRAIN_IO(io_dtype, "pretrain_kk_pre", {
    FRWKV_TRAIN_LANES(head_size, {
      plan = launch_walk(kk_pre_backward_kernel<io_t, kLanes>, rows, channels, s, 
          CP(io_t, grad_new_k), CP(io_t, grad_neg_kk), CP(io_t, grad_kka), CP(io_t, k), CP(io_t, k_k), CP(io_t, a),
          CP(io_t, k_a), inv_norm, P(io_t, grad_k), P(io_t, grad_a), workspace, rows, channels);
    })
    if (int rc = check_launch("kk_pre_backward_kernel")) return rc;
    return reduce_partials<io_t>(workspace, targets, plan, channels, 2, s);
  })
}

extern "C" int frwkv_pretrain_lnx_rkvres_xg_forward(const void* x, const void* r, const void* k, const void* v,
                                                    const void* r_k, const void* weight, const void* bias,
                                                    const void* g, void* out, float* mean, float* rstd,
                                                    long long rows, int channels, int head_size, int io_dtype,
                                                    frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(x && r && k && v && r_k && weight && bias && g && out && mean && rstd,
                "pretrain_lnx_rkvres_xg: null pointer argument");
  if (int rc = check_dense("pretrain_lnx_rkvres_xg", rows, channels, 0, 0)) return rc;
  if (int rc = check_heads("pretrain_lnx_rkvres_xg", channels, head_size)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_TRAIN_IO(io_dtype, "pretrain_lnx_rkvres_xg", {
    FRWKV_TRAIN_LANES(head_size, {
      launch_walk(lnx_forward_kernel<io_t, kLanes>, rows, channels, s, 
          CP(io_t, x), CP(io_t, r), CP(io_t, k), CP(io_t, v), CP(io_t, r_k), CP(io_t, weight), CP(io_t, bias),
          CP(io_t, g), P(io_t, out), mean, rstd, rows, channels);
    })
    return check_launch("lnx_forward_kernel");
  })
}

extern "C" int frwkv_pretrain_lnx_rkvres_xg_backward(
    const void* grad_out, const void* x, const void* r, const void* k, const void* v, const void* r_k,
    const void* weight, const void* bias, const void* g, const float* mean, const float* rstd, void* grad_x,
    void* grad_r, void* grad_k, void* grad_v, void* grad_r_k, void* grad_weight, void* grad_bias, void* grad_g,
    float* workspace, long long workspace_floats, long long rows, int channels, int head_size, int io_dtype,
    frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(grad_out && x && r && k && v && r_k && weight && bias && g && mean && rstd && grad_x && grad_r &&
                    grad_k && grad_v && grad_r_k && grad_weight && grad_bias && grad_g && workspace,
                "pretrain_lnx_rkvres_xg: null pointer argument");
  if (int rc = check_dense("pretrain_lnx_rkvres_xg", rows, channels, workspace_floats, 3)) return rc;
  if (int rc = check_heads("pretrain_lnx_rkvres_xg", channels, head_size)) return rc;
  Plan plan;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  ReduceTargets targets{{grad_r_k, grad_weight, grad_bias}};
  FRWKV_TRAIN_IO(io_dtype, "pretrain_lnx_rkvres_xg", {
    FRWKV_TRAIN_LANES(head_size, {
      plan = launch_walk(lnx_backward_kernel<io_t, kLanes>, rows, channels, s, 
          CP(io_t, grad_out), CP(io_t, x), CP(io_t, r), CP(io_t, k), CP(io_t, v), CP(io_t, r_k), CP(io_t, weight),
          CP(io_t, bias), CP(io_t, g), mean, rstd, P(io_t, grad_x), P(io_t, grad_r), P(io_t, grad_k), P(io_t, grad_v),
          P(io_t, grad_g), workspace, rows, channels);
    })
    if (int rc = check_launch("lnx_backward_kernel")) return rc;
    return reduce_partials<io_t>(workspace, targets, plan, channels, 3, s);
  })
}

#undef P
#undef CP
