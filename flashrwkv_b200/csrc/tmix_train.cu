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
// that lane group), a CTA of 128 threads covers 1024 channels.  The passes that also produce a gradient of a [C]
// parameter (a sum over all B * T rows) cut the rows into contiguous slabs, one CTA per (channel tile, slab): a
// thread walks its slab row by row with the column sums in registers and writes one fp32 partial per slab, and
// reduce_partials_kernel adds the slabs in a fixed order.  The parameter gradients are therefore bit-reproducible;
// the reference accumulates them with fp32 atomics.  Walking contiguous rows also hands mix6 its previous row in
// registers, so x is read once.
//
// Replaces csrc/sm90/tmix/{a_gate,vres_gate,mix6,kk_pre,lnx_rkvres_xg}/pretrain_bf16_{forward,backward}.cu.

#include "frwkv_common.cuh"

namespace frwkv {
namespace {

constexpr int kThreads = 128;
constexpr int kTileCols = kThreads * 8;
constexpr float kNormalizeEps = 1.0e-12f;
constexpr float kLnxEps = 64e-5f;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

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

// The slab of rows and the eight channels of this thread in a (channel tile, slab) grid.
struct Walk {
  long long row_begin, row_end;
  int col;
  bool active;
};
__device__ __forceinline__ Walk my_walk(long long rows, int channels, int rows_per_slab) {
  Walk w;
  w.col = (blockIdx.x * kThreads + threadIdx.x) * 8;
  w.active = w.col < channels;
  w.row_begin = (long long)blockIdx.y * rows_per_slab;
  w.row_end = w.row_begin + rows_per_slab < rows ? w.row_begin + rows_per_slab : rows;
  return w;
}
__device__ __forceinline__ void store_partial(float* workspace, int vec, int channels, int col, const float (&f)[8]) {
  float* p = workspace + ((long long)vec * gridDim.y + blockIdx.y) * channels + col;
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
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
template <typename io_t>
__global__ __launch_bounds__(256) void a_gate_forward_kernel(const io_t* __restrict__ a0, const io_t* __restrict__ a12,
                                                             io_t* __restrict__ out, long long vec_total,
                                                             int vec_per_row) {
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < vec_total; i += (long long)gridDim.x * 256) {
    float z[8], t[8];
    load8(a0 + (i % vec_per_row) * 8, z);
    load8(a12 + i * 8, t);
#pragma unroll
    for (int e = 0; e < 8; ++e) t[e] = sigmoidf_(z[e] + t[e]);
    store8(out + i * 8, t);
  }
}

template <typename io_t>
__global__ __launch_bounds__(kThreads) void a_gate_backward_kernel(const io_t* __restrict__ grad_out,
                                                                   const io_t* __restrict__ a0,
                                                                   const io_t* __restrict__ a12,
                                                                   io_t* __restrict__ grad_a12,
                                                                   float* __restrict__ workspace, long long rows,
                                                                   int channels, int rows_per_slab) {
  const Walk w = my_walk(rows, channels, rows_per_slab);
  if (!w.active) return;
  float z0[8], acc[8];
  load8(a0 + w.col, z0);
  zero8(acc);
#pragma unroll 2
  for (long long row = w.row_begin; row < w.row_end; ++row) {
    const long long at = row * channels + w.col;
    float z[8], g[8];
    load8(a12 + at, z);
    load8(grad_out + at, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float y = sigmoidf_(z0[e] + z[e]);
      g[e] *= y * (1.f - y);
      acc[e] += g[e];
    }
    store8(grad_a12 + at, g);
  }
  store_partial(workspace, 0, channels, w.col, acc);
}

// ---- vres_gate -----------------------------------------------------------------------------------------------------
template <typename io_t>
__global__ __launch_bounds__(kThreads) void vres_gate_backward_kernel(
    const io_t* __restrict__ grad_out, const io_t* __restrict__ v, const io_t* __restrict__ v_first,
    const io_t* __restrict__ v0, const io_t* __restrict__ v12, io_t* __restrict__ grad_v,
    io_t* __restrict__ grad_v_first, io_t* __restrict__ grad_v12, float* __restrict__ workspace, long long rows,
    int channels, int rows_per_slab) {
  const Walk w = my_walk(rows, channels, rows_per_slab);
  if (!w.active) return;
  float z0[8], acc[8];
  load8(v0 + w.col, z0);
  zero8(acc);
#pragma unroll 2
  for (long long row = w.row_begin; row < w.row_end; ++row) {
    const long long at = row * channels + w.col;
    float g[8], a[8], f[8], z[8], gz[8];
    load8(grad_out + at, g);
    load8(v + at, a);
    load8(v_first + at, f);
    load8(v12 + at, z);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float s = sigmoidf_(z0[e] + z[e]);
      gz[e] = g[e] * (f[e] - a[e]) * s * (1.f - s);
      acc[e] += gz[e];
      f[e] = g[e] * s;         // grad of v_first
      a[e] = g[e] - f[e];      // grad of v
    }
    store8(grad_v + at, a);
    store8(grad_v_first + at, f);
    store8(grad_v12 + at, gz);
  }
  store_partial(workspace, 0, channels, w.col, acc);
}

// ---- mix6 ----------------------------------------------------------------------------------------------------------
struct Six {
  const void* in[6];
  void* out[6];
};

// Rows are b * T + t; a slab may cross sequence boundaries, the row before t = 0 is zero.
template <typename io_t>
__global__ __launch_bounds__(kThreads) void mix6_forward_kernel(const io_t* __restrict__ x, Six mix, long long rows,
                                                                int seq_len, int channels, int rows_per_slab) {
  const Walk w = my_walk(rows, channels, rows_per_slab);
  if (!w.active || w.row_begin >= w.row_end) return;
  float m[6][8], prev[8];
#pragma unroll
  for (int j = 0; j < 6; ++j) load8(static_cast<const io_t*>(mix.in[j]) + w.col, m[j]);
  int t = (int)(w.row_begin % seq_len);
  if (t != 0) load8(x + (w.row_begin - 1) * channels + w.col, prev);
  for (long long row = w.row_begin; row < w.row_end; ++row) {
    const long long at = row * channels + w.col;
    float cur[8], xx[8];
    load8(x + at, cur);
#pragma unroll
    for (int e = 0; e < 8; ++e) xx[e] = (t != 0 ? prev[e] : 0.f) - cur[e];
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      float y[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = fmaf(xx[e], m[j][e], cur[e]);
      store8(static_cast<io_t*>(mix.out[j]) + at, y);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) prev[e] = cur[e];
    if (++t == seq_len) t = 0;
  }
}

// grad_x[t] = sum_j g_j[t] (1 - m_j) + sum_j g_j[t+1] m_j (second term only inside the sequence);
// grad_m_j = sum_rows g_j (x[t-1] - x[t]).  mix.in = the six upstream gradients, mix.out = the six mix vectors.
template <typename io_t>
__global__ __launch_bounds__(kThreads) void mix6_backward_kernel(const io_t* __restrict__ x, Six mix,
                                                                 io_t* __restrict__ grad_x,
                                                                 float* __restrict__ workspace, long long rows,
                                                                 int seq_len, int channels, int rows_per_slab) {
  const Walk w = my_walk(rows, channels, rows_per_slab);
  if (!w.active || w.row_begin >= w.row_end) return;
  float m[6][8], dm[6][8], prev[8], carry[8];
#pragma unroll
  for (int j = 0; j < 6; ++j) {
    load8(static_cast<const io_t*>(mix.out[j]) + w.col, m[j]);
    zero8(dm[j]);
  }
  int t = (int)(w.row_begin % seq_len);
  if (t != 0) load8(x + (w.row_begin - 1) * channels + w.col, prev);
  zero8(carry);
  for (long long row = w.row_begin; row < w.row_end; ++row) {
    const long long at = row * channels + w.col;
    float cur[8], xx[8], direct[8], shifted[8];
    load8(x + at, cur);
    zero8(direct);
    zero8(shifted);
#pragma unroll
    for (int e = 0; e < 8; ++e) xx[e] = (t != 0 ? prev[e] : 0.f) - cur[e];
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      float g[8];
      load8(static_cast<const io_t*>(mix.in[j]) + at, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dm[j][e] = fmaf(g[e], xx[e], dm[j][e]);
        shifted[e] = fmaf(g[e], m[j][e], shifted[e]);
        direct[e] += g[e];
      }
    }
    if (row > w.row_begin) {  // the previous row is complete once this row's shifted term is known
#pragma unroll
      for (int e = 0; e < 8; ++e) carry[e] += t != 0 ? shifted[e] : 0.f;
      store8(grad_x + at - channels, carry);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      carry[e] = direct[e] - shifted[e];
      prev[e] = cur[e];
    }
    if (++t == seq_len) t = 0;
  }
  if (w.row_end < rows && t != 0) {  // the slab's last row takes its shifted term from the next slab's first row
    const long long at = w.row_end * channels + w.col;
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      float g[8];
      load8(static_cast<const io_t*>(mix.in[j]) + at, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) carry[e] = fmaf(g[e], m[j][e], carry[e]);
    }
  }
  store8(grad_x + (w.row_end - 1) * channels + w.col, carry);
#pragma unroll
  for (int j = 0; j < 6; ++j) store_partial(workspace, j, channels, w.col, dm[j]);
}

// ---- kk_pre --------------------------------------------------------------------------------------------------------
// A head is kLanes = D / 8 adjacent lanes.  Lanes past the last channel keep running the row loop with their loads and
// stores switched off so that the full-mask shuffles stay converged; a warp with no channel at all leaves at once.
__device__ __forceinline__ bool warp_has_channels(int channels) {
  return (blockIdx.x * kThreads + (threadIdx.x & ~31)) * 8 < channels;
}

template <typename io_t, int kLanes>
__global__ __launch_bounds__(kThreads) void kk_pre_forward_kernel(
    const io_t* __restrict__ k, const io_t* __restrict__ k_k, const io_t* __restrict__ a, const io_t* __restrict__ k_a,
    io_t* __restrict__ new_k, io_t* __restrict__ neg_kk, io_t* __restrict__ kka, float* __restrict__ inv_norm,
    long long rows, int channels, int rows_per_slab) {
  const Walk w = my_walk(rows, channels, rows_per_slab);
  if (!warp_has_channels(channels)) return;
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
    float* __restrict__ workspace, long long rows, int channels, int rows_per_slab) {
  const Walk w = my_walk(rows, channels, rows_per_slab);
  if (!warp_has_channels(channels)) return;
  const int heads = channels / (kLanes * 8), head = w.col / (kLanes * 8);
  float ks[8], ka[8], dks[8], dka[8];
  zero8(ks);
  zero8(ka);
  zero8(dks);
  zero8(dka);
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
      dks[e] = fmaf(gu, kv[e], dks[e]);
      dka[e] = fmaf(gn[e] * kv[e], av[e] - 1.f, dka[e]);
    }
    store8(grad_k + at, gk);
    store8(grad_a + at, ga);
  }
  if (w.active) {
    store_partial(workspace, 0, channels, w.col, dks);
    store_partial(workspace, 1, channels, w.col, dka);
  }
}

// ---- lnx_rkvres_xg -------------------------------------------------------------------------------------------------
template <typename io_t, int kLanes>
__global__ __launch_bounds__(kThreads) void lnx_forward_kernel(
    const io_t* __restrict__ x, const io_t* __restrict__ r, const io_t* __restrict__ k, const io_t* __restrict__ v,
    const io_t* __restrict__ r_k, const io_t* __restrict__ weight, const io_t* __restrict__ bias,
    const io_t* __restrict__ g, io_t* __restrict__ out, float* __restrict__ mean_out, float* __restrict__ rstd_out,
    long long rows, int channels, int rows_per_slab) {
  constexpr float kInvD = 1.f / (kLanes * 8);
  const Walk w = my_walk(rows, channels, rows_per_slab);
  if (!warp_has_channels(channels)) return;
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
    float* __restrict__ workspace, long long rows, int channels, int rows_per_slab) {
  constexpr float kInvD = 1.f / (kLanes * 8);
  const Walk w = my_walk(rows, channels, rows_per_slab);
  if (!warp_has_channels(channels)) return;
  const int heads = channels / (kLanes * 8), head = w.col / (kLanes * 8);
  float rk[8], wt[8], bs[8], drk[8], dwt[8], dbs[8];
  zero8(rk);
  zero8(wt);
  zero8(bs);
  zero8(drk);
  zero8(dwt);
  zero8(dbs);
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
      dwt[e] = fmaf(gy[e], xh[e], dwt[e]);
      dbs[e] += gy[e];
      drk[e] = fmaf(gs * rv[e], kv[e], drk[e]);
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
  if (w.active) {
    store_partial(workspace, 0, channels, w.col, drk);
    store_partial(workspace, 1, channels, w.col, dwt);
    store_partial(workspace, 2, channels, w.col, dbs);
  }
}

// ---- host side -----------------------------------------------------------------------------------------------------
struct Plan {
  int col_tiles, slabs, rows_per_slab;
};
// About eight CTAs of 128 threads per SM; every slab holds at least one row.
Plan make_plan(long long rows, int channels) {
  Plan p;
  p.col_tiles = (channels + kTileCols - 1) / kTileCols;
  long long slabs = (148 * 8 + p.col_tiles - 1) / p.col_tiles;
  if (slabs > rows) slabs = rows;
  if (slabs < 1) slabs = 1;
  p.rows_per_slab = (int)((rows + slabs - 1) / slabs);
  p.slabs = (int)((rows + p.rows_per_slab - 1) / p.rows_per_slab);
  return p;
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
  if (vectors > 0 && workspace_floats < (long long)vectors * make_plan(rows, channels).slabs * channels)
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
  return (long long)vectors * frwkv::make_plan(rows, channels).slabs * channels;
}

extern "C" int frwkv_pretrain_a_gate_forward(const void* a0, const void* a12, void* out, long long rows, int channels,
                                             int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(a0 && a12 && out, "pretrain_a_gate: null pointer argument");
  if (int rc = check_dense("pretrain_a_gate", rows, channels, 0, 0)) return rc;
  const long long vec_total = rows * (channels / 8);
  long long blocks = (vec_total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_TRAIN_IO(io_dtype, "pretrain_a_gate", {
    a_gate_forward_kernel<io_t><<<(unsigned)blocks, 256, 0, s>>>(CP(io_t, a0), CP(io_t, a12), P(io_t, out), vec_total,
                                                                 channels / 8);
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
  const Plan plan = make_plan(rows, channels);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  ReduceTargets targets{{grad_a0}};
  FRWKV_TRAIN_IO(io_dtype, "pretrain_a_gate", {
    a_gate_backward_kernel<io_t><<<dim3(plan.col_tiles, plan.slabs), kThreads, 0, s>>>(
        CP(io_t, grad_out), CP(io_t, a0), CP(io_t, a12), P(io_t, grad_a12), workspace, rows, channels,
        plan.rows_per_slab);
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
  const Plan plan = make_plan(rows, channels);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  ReduceTargets targets{{grad_v0}};
  FRWKV_TRAIN_IO(io_dtype, "pretrain_vres_gate", {
    vres_gate_backward_kernel<io_t><<<dim3(plan.col_tiles, plan.slabs), kThreads, 0, s>>>(
        CP(io_t, grad_out), CP(io_t, v), CP(io_t, v_first), CP(io_t, v0), CP(io_t, v12), P(io_t, grad_v),
        P(io_t, grad_v_first), P(io_t, grad_v12), workspace, rows, channels, plan.rows_per_slab);
    if (int rc = check_launch("vres_gate_backward_kernel")) return rc;
    return reduce_partials<io_t>(workspace, targets, plan, channels, 1, s);
  })
}

extern "C" int frwkv_pretrain_mix6_forward(const void* x, const void* const* mix, void* const* out, long long batch,
                                           int seq_len, int channels, int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
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
  const Plan plan = make_plan(rows, channels);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_TRAIN_IO(io_dtype, "pretrain_mix6", {
    mix6_forward_kernel<io_t><<<dim3(plan.col_tiles, plan.slabs), kThreads, 0, s>>>(CP(io_t, x), six, rows, seq_len,
                                                                                   channels, plan.rows_per_slab);
    return check_launch("mix6_forward_kernel");
  })
}

extern "C" int frwkv_pretrain_mix6_backward(const void* const* grad_out, const void* x, const void* const* mix,
                                            void* grad_x, void* const* grad_mix, float* workspace,
                                            long long workspace_floats, long long batch, int seq_len, int channels,
                                            int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
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
  const Plan plan = make_plan(rows, channels);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_TRAIN_IO(io_dtype, "pretrain_mix6", {
    mix6_backward_kernel<io_t><<<dim3(plan.col_tiles, plan.slabs), kThreads, 0, s>>>(
        CP(io_t, x), six, P(io_t, grad_x), workspace, rows, seq_len, channels, plan.rows_per_slab);
    if (int rc = check_launch("mix6_backward_kernel")) return rc;
    return reduce_partials<io_t>(workspace, targets, plan, channels, 6, s);
  })
}

extern "C" int frwkv_pretrain_kk_pre_forward(const void* k, const void* k_k, const void* a, const void* k_a,
                                             void* new_k, void* neg_kk, void* kka, float* inv_norm, long long rows,
                                             int channels, int head_size, int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(k && k_k && a && k_a && new_k && neg_kk && kka && inv_norm, "pretrain_kk_pre: null pointer argument");
  if (int rc = check_dense("pretrain_kk_pre", rows, channels, 0, 0)) return rc;
  if (int rc = check_heads("pretrain_kk_pre", channels, head_size)) return rc;
  const Plan plan = make_plan(rows, channels);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_TRAIN_IO(io_dtype, "pretrain_kk_pre", {
    FRWKV_TRAIN_LANES(head_size, {
      kk_pre_forward_kernel<io_t, kLanes><<<dim3(plan.col_tiles, plan.slabs), kThreads, 0, s>>>(
          CP(io_t, k), CP(io_t, k_k), CP(io_t, a), CP(io_t, k_a), P(io_t, new_k), P(io_t, neg_kk), P(io_t, kka),
          inv_norm, rows, channels, plan.rows_per_slab);
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
  const Plan plan = make_plan(rows, channels);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  ReduceTargets targets{{grad_k_k, grad_k_a}};
  FRWKV_TRAIN_IO(io_dtype, "pretrain_kk_pre", {
    FRWKV_TRAIN_LANES(head_size, {
      kk_pre_backward_kernel<io_t, kLanes><<<dim3(plan.col_tiles, plan.slabs), kThreads, 0, s>>>(
          CP(io_t, grad_new_k), CP(io_t, grad_neg_kk), CP(io_t, grad_kka), CP(io_t, k), CP(io_t, k_k), CP(io_t, a),
          CP(io_t, k_a), inv_norm, P(io_t, grad_k), P(io_t, grad_a), workspace, rows, channels, plan.rows_per_slab);
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
  const Plan plan = make_plan(rows, channels);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_TRAIN_IO(io_dtype, "pretrain_lnx_rkvres_xg", {
    FRWKV_TRAIN_LANES(head_size, {
      lnx_forward_kernel<io_t, kLanes><<<dim3(plan.col_tiles, plan.slabs), kThreads, 0, s>>>(
          CP(io_t, x), CP(io_t, r), CP(io_t, k), CP(io_t, v), CP(io_t, r_k), CP(io_t, weight), CP(io_t, bias),
          CP(io_t, g), P(io_t, out), mean, rstd, rows, channels, plan.rows_per_slab);
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
  const Plan plan = make_plan(rows, channels);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  ReduceTargets targets{{grad_r_k, grad_weight, grad_bias}};
  FRWKV_TRAIN_IO(io_dtype, "pretrain_lnx_rkvres_xg", {
    FRWKV_TRAIN_LANES(head_size, {
      lnx_backward_kernel<io_t, kLanes><<<dim3(plan.col_tiles, plan.slabs), kThreads, 0, s>>>(
          CP(io_t, grad_out), CP(io_t, x), CP(io_t, r), CP(io_t, k), CP(io_t, v), CP(io_t, r_k), CP(io_t, weight),
          CP(io_t, bias), CP(io_t, g), mean, rstd, P(io_t, grad_x), P(io_t, grad_r), P(io_t, grad_k), P(io_t, grad_v),
          P(io_t, grad_g), workspace, rows, channels, plan.rows_per_slab);
    })
    if (int rc = check_launch("lnx_backward_kernel")) return rc;
    return reduce_partials<io_t>(workspace, targets, plan, channels, 3, s);
  })
}

#undef P
#undef CP
