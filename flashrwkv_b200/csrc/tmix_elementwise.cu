// TMix elementwise / per-head kernels (bandwidth-bound; 16-byte vector accesses, fp32 arithmetic):
//   mix6          out_j = x + (prev - x) * mix_j, j = r,w,k,v,a,g; prev = previous packed row, or the shift-state
//                 slot at a sequence start; the slot takes the sequence's last row
//   kk_a_gate     kk = normalize(k*k_k) per head; a = sigmoid(a0 + a12); k' = k*(1 + (a-1)*k_a); -> (k', -kk, kk*a)
//   lnx_rkvres_xg (GroupNorm_head(x)*weight + bias + (sum_d r k r_k) v) * g
//   vres_gate     v + (v_first - v) * sigmoid(v0 + v12)
// They replace tmix_mix6_kernel (csrc/sm120/tmix/mix6/infer_fp16_forward_varlen.cu:75-188),
// tmix_kk_a_gate_kernel (csrc/sm120/tmix/kk_a_gate/infer_fp16_forward_varlen.cu:52-210),
// tmix_lnx_rkvres_xg_kernel (csrc/sm120/tmix/lnx_rkvres_xg/infer_fp16_forward_varlen.cu:133-244) and
// tmix_vres_gate_kernel (csrc/sm120/tmix/vres_gate/infer_fp16_forward_varlen.cu:47-93) of the reference.

#include "frwkv_common.cuh"

namespace frwkv {
namespace {

template <typename io_t>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  using IO = Io16<io_t>;
  float2 t;
  t = IO::unpack(u.x); f[0] = t.x; f[1] = t.y;
  t = IO::unpack(u.y); f[2] = t.x; f[3] = t.y;
  t = IO::unpack(u.z); f[4] = t.x; f[5] = t.y;
  t = IO::unpack(u.w); f[6] = t.x; f[7] = t.y;
}
template <typename io_t>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  using IO = Io16<io_t>;
  return make_uint4(IO::pack(f[0], f[1]), IO::pack(f[2], f[3]), IO::pack(f[4], f[5]), IO::pack(f[6], f[7]));
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- mix6 ------------------------------------------------------------------------------------------
// One CTA per packed row.  Thread 0 finds the row's sequence by binary search over cu_seqlens.  When the row is
// both first and last of its sequence (decode) the shift slot is rewritten here, each thread overwriting exactly
// the elements it read; longer sequences get their slot from mix6_shift_update_kernel afterwards, because the
// CTA of a sequence's first row may not have read the slot yet when its last row is processed.
struct Mix6Vectors {
  const void* p[6];  // x_r, x_w, x_k, x_v, x_a, x_g, each [C]
};

template <typename io_t>
__global__ void mix6_kernel(const io_t* __restrict__ x, io_t* __restrict__ shift_pool, Mix6Vectors mix6,
                            const int* __restrict__ cu_seqlens, const int* __restrict__ state_indices,
                            const int* __restrict__ status, io_t* __restrict__ out, int num_sequences,
                            long long total_rows, int C) {
  chain_begin();
  const long long row = blockIdx.x;
  const int vecs = C >> 3;
  if (status != nullptr && status[0] != 0) {
    const uint32_t nan2 = Io16<io_t>::pack(quiet_nan(), quiet_nan());
    const uint4 nanv = make_uint4(nan2, nan2, nan2, nan2);
    for (int j = 0; j < 6; ++j)
      for (int i = threadIdx.x; i < vecs; i += blockDim.x)
        reinterpret_cast<uint4*>(out + ((long long)j * total_rows + row) * C)[i] = nanv;
    return;
  }
  __shared__ int s_first, s_last, s_slot;
  if (threadIdx.x == 0) {
    int lo = 0, hi = num_sequences;  // largest s with cu[s] <= row
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if ((long long)cu_seqlens[mid] <= row) lo = mid; else hi = mid;
    }
    s_first = ((long long)cu_seqlens[lo] == row);
    s_last = ((long long)cu_seqlens[lo + 1] == row + 1);
    s_slot = state_indices[lo];
  }
  __syncthreads();
  const bool first = s_first != 0, last = s_last != 0;
  const uint4* cur = reinterpret_cast<const uint4*>(x + row * C);
  const uint4* prev = first ? reinterpret_cast<const uint4*>(shift_pool + (long long)s_slot * C)
                            : reinterpret_cast<const uint4*>(x + (row - 1) * C);
  for (int i = threadIdx.x; i < vecs; i += blockDim.x) {
    const uint4 cu4 = cur[i];
    float c[8], p[8];
    unpack8<io_t>(cu4, c);
    unpack8<io_t>(prev[i], p);
#pragma unroll
    for (int e = 0; e < 8; ++e) p[e] -= c[e];
#pragma unroll
    for (int j = 0; j < 6; ++j) {
      float m[8], o[8];
      unpack8<io_t>(__ldg(reinterpret_cast<const uint4*>(mix6.p[j]) + i), m);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = fmaf(p[e], m[e], c[e]);
      reinterpret_cast<uint4*>(out + ((long long)j * total_rows + row) * C)[i] = pack8<io_t>(o);
    }
    if (first && last) reinterpret_cast<uint4*>(shift_pool + (long long)s_slot * C)[i] = cu4;
  }
}

template <typename io_t>
__global__ void mix6_shift_update_kernel(const io_t* __restrict__ x, io_t* __restrict__ shift_pool,
                                         const int* __restrict__ cu_seqlens, const int* __restrict__ state_indices,
                                         const int* __restrict__ status, int C, int min_len) {
  chain_begin();
  if (status != nullptr && status[0] != 0) return;
  const int s = blockIdx.x;
  const int t0 = cu_seqlens[s], t1 = cu_seqlens[s + 1];
  if (t1 - t0 < min_len) return;  // after mix6_kernel (min_len = 2): it has stored the rows of one-token sequences
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)(t1 - 1) * C);
  uint4* dst = reinterpret_cast<uint4*>(shift_pool + (long long)state_indices[s] * C);
  for (int i = threadIdx.x; i < (C >> 3); i += blockDim.x) dst[i] = src[i];
}

// ---- per-(row, head) kernels: one warp per head; a lane holds P = head_size / 64 pairs of channels, pair p at
// channels 64 p + 2 lane (every load of the warp is one contiguous 128-byte segment) ----------------------------------
template <typename io_t, int P>
__global__ void kk_a_gate_kernel(const io_t* __restrict__ k, const io_t* __restrict__ k_k, const io_t* __restrict__ a0,
                                 const io_t* __restrict__ a12, const io_t* __restrict__ k_a, io_t* __restrict__ new_k,
                                 io_t* __restrict__ neg_kk, io_t* __restrict__ kka, long long units, int H) {
  chain_begin();
  using IO = Io16<io_t>;
  constexpr int kHead = 64 * P;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= units) return;
  const int lane = threadIdx.x & 31;
  const int head = (int)(unit % H);
  float2 kv[P], q[P], g[P], kav[P];
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < P; ++p) {
    const long long o = unit * kHead + 64 * p + 2 * lane;
    const int c = head * kHead + 64 * p + 2 * lane;
    kv[p] = IO::unpack(*reinterpret_cast<const uint32_t*>(k + o));
    const float2 kkv = IO::unpack(*reinterpret_cast<const uint32_t*>(k_k + c));
    const float2 a0v = IO::unpack(*reinterpret_cast<const uint32_t*>(a0 + c));
    const float2 a12v = IO::unpack(*reinterpret_cast<const uint32_t*>(a12 + o));
    kav[p] = IO::unpack(*reinterpret_cast<const uint32_t*>(k_a + c));
    q[p] = make_float2(kv[p].x * kkv.x, kv[p].y * kkv.y);
    g[p] = make_float2(sigmoidf_(a0v.x + a12v.x), sigmoidf_(a0v.y + a12v.y));
    ss = fmaf(q[p].x, q[p].x, fmaf(q[p].y, q[p].y, ss));
  }
  const float nrm = fmaxf(sqrtf(warp_sum(ss)), 1e-12f);
#pragma unroll
  for (int p = 0; p < P; ++p) {
    const long long o = unit * kHead + 64 * p + 2 * lane;
    const float n0 = q[p].x / nrm, n1 = q[p].y / nrm;
    *reinterpret_cast<uint32_t*>(new_k + o) =
        IO::pack(kv[p].x * (1.f + (g[p].x - 1.f) * kav[p].x), kv[p].y * (1.f + (g[p].y - 1.f) * kav[p].y));
    *reinterpret_cast<uint32_t*>(neg_kk + o) = IO::pack(-n0, -n1);
    *reinterpret_cast<uint32_t*>(kka + o) = IO::pack(n0 * g[p].x, n1 * g[p].y);
  }
}

template <typename io_t, int P>
__global__ void lnx_rkvres_xg_kernel(const io_t* __restrict__ x, const io_t* __restrict__ r, const io_t* __restrict__ k,
                                     const io_t* __restrict__ v, const io_t* __restrict__ r_k,
                                     const io_t* __restrict__ weight, const io_t* __restrict__ bias,
                                     const io_t* __restrict__ g, io_t* __restrict__ out, long long units, int H,
                                     float eps) {
  chain_begin();
  using IO = Io16<io_t>;
  constexpr int kHead = 64 * P;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= units) return;
  const int lane = threadIdx.x & 31;
  const int head = (int)(unit % H);
  float2 xv[P];
  float sum = 0.f, dot = 0.f;
#pragma unroll
  for (int p = 0; p < P; ++p) {
    const long long o = unit * kHead + 64 * p + 2 * lane;
    const int c = head * kHead + 64 * p + 2 * lane;
    xv[p] = IO::unpack(*reinterpret_cast<const uint32_t*>(x + o));
    const float2 rv = IO::unpack(*reinterpret_cast<const uint32_t*>(r + o));
    const float2 kv = IO::unpack(*reinterpret_cast<const uint32_t*>(k + o));
    const float2 rk = IO::unpack(*reinterpret_cast<const uint32_t*>(r_k + c));
    sum += xv[p].x + xv[p].y;
    dot = fmaf(rv.x * kv.x, rk.x, fmaf(rv.y * kv.y, rk.y, dot));
  }
  const float mean = warp_sum(sum) * (1.f / kHead);
  float sq = 0.f;
#pragma unroll
  for (int p = 0; p < P; ++p) {
    const float d0 = xv[p].x - mean, d1 = xv[p].y - mean;
    sq = fmaf(d0, d0, fmaf(d1, d1, sq));
  }
  const float var = warp_sum(sq) * (1.f / kHead);
  dot = warp_sum(dot);
  const float rstd = rsqrtf(var + eps);
#pragma unroll
  for (int p = 0; p < P; ++p) {
    const long long o = unit * kHead + 64 * p + 2 * lane;
    const int c = head * kHead + 64 * p + 2 * lane;
    const float2 vv = IO::unpack(*reinterpret_cast<const uint32_t*>(v + o));
    const float2 gv = IO::unpack(*reinterpret_cast<const uint32_t*>(g + o));
    const float2 wv = IO::unpack(*reinterpret_cast<const uint32_t*>(weight + c));
    const float2 bv = IO::unpack(*reinterpret_cast<const uint32_t*>(bias + c));
    const float d0 = xv[p].x - mean, d1 = xv[p].y - mean;
    *reinterpret_cast<uint32_t*>(out + o) = IO::pack((d0 * rstd * wv.x + bv.x + dot * vv.x) * gv.x,
                                                     (d1 * rstd * wv.y + bv.y + dot * vv.y) * gv.y);
  }
}

// out = x + vec (fp32 sum, one rounding): one 4-byte pair per thread and step, row index from the grid-stride counter
// so that any even channel count works (the recurrence's pre-add-vector helper; replaces recurrent_add_vec_kernel,
// csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu:83-124).
template <typename io_t>
__global__ void add_vec_kernel(const io_t* __restrict__ x, const io_t* __restrict__ vec, io_t* __restrict__ out,
                               long long pair_total, int pairs_per_row) {
  using IO = Io16<io_t>;
  chain_begin();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < pair_total;
       i += (long long)gridDim.x * blockDim.x) {
    const float2 a = IO::unpack(reinterpret_cast<const uint32_t*>(x)[i]);
    const float2 b = IO::unpack(__ldg(reinterpret_cast<const uint32_t*>(vec) + (i % pairs_per_row)));
    reinterpret_cast<uint32_t*>(out)[i] = IO::pack(a.x + b.x, a.y + b.y);
  }
}

template <typename io_t>
__global__ void vres_gate_kernel(const io_t* __restrict__ v, const io_t* __restrict__ v_first,
                                 const io_t* __restrict__ v0, const io_t* __restrict__ v12, io_t* __restrict__ out,
                                 long long vec_total, int vecs_per_row) {
  chain_begin();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vec_total;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8], f[8], z[8], t[8];
    unpack8<io_t>(reinterpret_cast<const uint4*>(v)[i], a);
    unpack8<io_t>(reinterpret_cast<const uint4*>(v_first)[i], f);
    unpack8<io_t>(reinterpret_cast<const uint4*>(v12)[i], t);
    unpack8<io_t>(__ldg(reinterpret_cast<const uint4*>(v0) + (i % vecs_per_row)), z);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = fmaf(f[e] - a[e], sigmoidf_(z[e] + t[e]), a[e]);
    reinterpret_cast<uint4*>(out)[i] = pack8<io_t>(a);
  }
}

template <typename io_t>
__global__ void act_kernel(const io_t* __restrict__ x, io_t* __restrict__ out, long long vec_total, int act) {
  chain_begin();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vec_total;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8];
    unpack8<io_t>(reinterpret_cast<const uint4*>(x)[i], a);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = act == 1 ? tanhf(a[e]) : sigmoidf_(a[e]);
    reinterpret_cast<uint4*>(out)[i] = pack8<io_t>(a);
  }
}

}  // namespace
}  // namespace frwkv

#define FRWKV_DISPATCH_IO(io_dtype, NAME, ...)                                                   \
  if ((io_dtype) == FRWKV_DTYPE_BF16) {                                                          \
    using io_t = __nv_bfloat16;                                                                  \
    __VA_ARGS__                                                                                  \
  } else if ((io_dtype) == FRWKV_DTYPE_FP16) {                                                   \
    using io_t = __half;                                                                         \
    __VA_ARGS__                                                                                  \
  } else {                                                                                       \
    return ::frwkv::fail(FRWKV_ERR_UNSUPPORTED, NAME ": tensors must be float16 or bfloat16");   \
  }

namespace frwkv {
int launch_shift_state_update(const void* x, void* shift_state_pool, const int* cu_seqlens, const int* state_indices,
                              const int* metadata_status, int num_sequences, int channels, int io_dtype,
                              cudaStream_t s) {
  const int threads = channels / 8 >= 256 ? 256 : (channels / 8 >= 128 ? 128 : 64);
  FRWKV_DISPATCH_IO(io_dtype, "tmix_shift_update", {
    launch_chained(mix6_shift_update_kernel<io_t>, dim3((unsigned)num_sequences), dim3(threads), 0, s,
                   static_cast<const io_t*>(x), static_cast<io_t*>(shift_state_pool), cu_seqlens, state_indices,
                   metadata_status, channels, 1);
    return check_launch("mix6_shift_update_kernel");
  })
}
}  // namespace frwkv

extern "C" int frwkv_tmix_mix6_forward_varlen(const void* x, void* shift_state_pool, const void* x_r, const void* x_w,
                                              const void* x_k, const void* x_v, const void* x_a, const void* x_g,
                                              const int32_t* cu_seqlens, const int32_t* state_indices,
                                              const int32_t* metadata_status, void* out, int total_rows,
                                              int num_sequences, int channels, int max_seqlen, int io_dtype,
                                              frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(x && shift_state_pool && x_r && x_w && x_k && x_v && x_a && x_g && cu_seqlens && state_indices && out,
                "tmix_mix6: null pointer argument");
  const Mix6Vectors mix6{{x_r, x_w, x_k, x_v, x_a, x_g}};
  FRWKV_REQUIRE(total_rows > 0 && num_sequences > 0 && channels > 0, "tmix_mix6: sizes must be positive");
  FRWKV_REQUIRE(channels % 8 == 0, "tmix_mix6: channel count must be a multiple of 8");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int threads = channels / 8 >= 256 ? 256 : (channels / 8 >= 128 ? 128 : 64);
  FRWKV_DISPATCH_IO(io_dtype, "tmix_mix6", {
    launch_chained(mix6_kernel<io_t>, dim3((unsigned)total_rows), dim3(threads), 0, s, 
        static_cast<const io_t*>(x), static_cast<io_t*>(shift_state_pool), mix6, cu_seqlens,
        state_indices, metadata_status, static_cast<io_t*>(out), num_sequences, (long long)total_rows, channels);
    int rc = check_launch("mix6_kernel");
    if (rc != FRWKV_OK) return rc;
    if (max_seqlen != 1) {  // unknown (<= 0) or longer than one token: some slot may still need its last row
      launch_chained(mix6_shift_update_kernel<io_t>, dim3((unsigned)num_sequences), dim3(threads), 0, s, 
          static_cast<const io_t*>(x), static_cast<io_t*>(shift_state_pool), cu_seqlens, state_indices,
          metadata_status, channels, 2);
      return check_launch("mix6_shift_update_kernel");
    }
    return FRWKV_OK;
  })
}

extern "C" int frwkv_tmix_kk_a_gate_forward_varlen(const void* k, const void* k_k, const void* a0, const void* a12,
                                                   const void* k_a, void* new_k, void* neg_kk, void* kka,
                                                   long long total_rows, int channels, int head_size, int io_dtype,
                                                   frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(k && k_k && a0 && a12 && k_a && new_k && neg_kk && kka, "tmix_kk_a_gate: null pointer argument");
  FRWKV_REQUIRE(total_rows > 0 && channels > 0, "tmix_kk_a_gate: sizes must be positive");
  if (head_size != 64 && head_size != 128 && head_size != 256)
    return fail(FRWKV_ERR_UNSUPPORTED, "tmix_kk_a_gate: head size must be 64, 128, or 256, got %d", head_size);
  FRWKV_REQUIRE(channels % head_size == 0, "tmix_kk_a_gate: channels must be a multiple of head_size");
  const int H = channels / head_size;
  const long long units = total_rows * H;
  const long long blocks = (units + 7) / 8;
  FRWKV_REQUIRE(blocks <= 0x7fffffffLL, "tmix_kk_a_gate: too many rows");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_DISPATCH_IO(io_dtype, "tmix_kk_a_gate", {
    const dim3 grid((unsigned)blocks), block(256);
    const io_t *kp = static_cast<const io_t*>(k), *kkp = static_cast<const io_t*>(k_k), *a0p = static_cast<const io_t*>(a0),
               *a12p = static_cast<const io_t*>(a12), *kap = static_cast<const io_t*>(k_a);
    io_t *o1 = static_cast<io_t*>(new_k), *o2 = static_cast<io_t*>(neg_kk), *o3 = static_cast<io_t*>(kka);
    if (head_size == 64) launch_chained(kk_a_gate_kernel<io_t, 1>, grid, block, 0, s, kp, kkp, a0p, a12p, kap, o1, o2, o3, units, H);
    else if (head_size == 128) launch_chained(kk_a_gate_kernel<io_t, 2>, grid, block, 0, s, kp, kkp, a0p, a12p, kap, o1, o2, o3, units, H);
    else launch_chained(kk_a_gate_kernel<io_t, 4>, grid, block, 0, s, kp, kkp, a0p, a12p, kap, o1, o2, o3, units, H);
    return check_launch("kk_a_gate_kernel");
  })
}

extern "C" int frwkv_tmix_lnx_rkvres_xg_forward_varlen(const void* x, const void* r, const void* k, const void* v,
                                                       const void* r_k, const void* weight, const void* bias,
                                                       const void* g, void* out, long long total_rows, int channels,
                                                       int head_size, float eps, int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(x && r && k && v && r_k && weight && bias && g && out, "tmix_lnx_rkvres_xg: null pointer argument");
  FRWKV_REQUIRE(total_rows > 0 && channels > 0, "tmix_lnx_rkvres_xg: sizes must be positive");
  if (head_size != 64 && head_size != 128 && head_size != 256)
    return fail(FRWKV_ERR_UNSUPPORTED, "tmix_lnx_rkvres_xg: head size must be 64, 128, or 256, got %d", head_size);
  FRWKV_REQUIRE(channels % head_size == 0, "tmix_lnx_rkvres_xg: channels must be a multiple of head_size");
  const int H = channels / head_size;
  const long long units = total_rows * H;
  const long long blocks = (units + 7) / 8;
  FRWKV_REQUIRE(blocks <= 0x7fffffffLL, "tmix_lnx_rkvres_xg: too many rows");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_DISPATCH_IO(io_dtype, "tmix_lnx_rkvres_xg", {
    const dim3 grid((unsigned)blocks), block(256);
    const io_t *xp = static_cast<const io_t*>(x), *rp = static_cast<const io_t*>(r), *kp = static_cast<const io_t*>(k),
               *vp = static_cast<const io_t*>(v), *rkp = static_cast<const io_t*>(r_k),
               *wp = static_cast<const io_t*>(weight), *bp = static_cast<const io_t*>(bias),
               *gp = static_cast<const io_t*>(g);
    io_t* op = static_cast<io_t*>(out);
    if (head_size == 64) launch_chained(lnx_rkvres_xg_kernel<io_t, 1>, grid, block, 0, s, xp, rp, kp, vp, rkp, wp, bp, gp, op, units, H, eps);
    else if (head_size == 128) launch_chained(lnx_rkvres_xg_kernel<io_t, 2>, grid, block, 0, s, xp, rp, kp, vp, rkp, wp, bp, gp, op, units, H, eps);
    else launch_chained(lnx_rkvres_xg_kernel<io_t, 4>, grid, block, 0, s, xp, rp, kp, vp, rkp, wp, bp, gp, op, units, H, eps);
    return check_launch("lnx_rkvres_xg_kernel");
  })
}

extern "C" int frwkv_tmix_vres_gate_forward_varlen(const void* v, const void* v_first, const void* v0, const void* v12,
                                                   void* out, long long total_rows, int channels, int io_dtype,
                                                   frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(v && v_first && v0 && v12 && out, "tmix_vres_gate: null pointer argument");
  FRWKV_REQUIRE(total_rows > 0 && channels > 0, "tmix_vres_gate: sizes must be positive");
  FRWKV_REQUIRE(channels % 8 == 0, "tmix_vres_gate: channel count must be a multiple of 8");
  const long long vec_total = total_rows * (channels / 8);
  long long blocks = (vec_total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_DISPATCH_IO(io_dtype, "tmix_vres_gate", {
    launch_chained(vres_gate_kernel<io_t>, dim3((unsigned)blocks), dim3(256), 0, s, 
        static_cast<const io_t*>(v), static_cast<const io_t*>(v_first), static_cast<const io_t*>(v0),
        static_cast<const io_t*>(v12), static_cast<io_t*>(out), vec_total, channels / 8);
    return check_launch("vres_gate_kernel");
  })
}

extern "C" int frwkv_recurrent_add_vec_forward(const void* x, const void* vec, void* out, long long total_rows,
                                               int channels, int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(x && vec && out, "recurrent_add_vec: null pointer argument");
  FRWKV_REQUIRE(total_rows > 0 && channels > 0 && channels % 2 == 0,
                "recurrent_add_vec: x must have packed shape [total_tokens,C] with even C");
  const long long pair_total = total_rows * (channels / 2);
  long long blocks = (pair_total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_DISPATCH_IO(io_dtype, "recurrent_add_vec", {
    launch_chained(add_vec_kernel<io_t>, dim3((unsigned)blocks), dim3(256), 0, s, static_cast<const io_t*>(x),
                   static_cast<const io_t*>(vec), static_cast<io_t*>(out), pair_total, channels / 2);
    return check_launch("add_vec_kernel");
  })
}

extern "C" int frwkv_tmix_act_forward(const void* x, void* out, long long elements, int act, int io_dtype,
                                      frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(x && out, "tmix_act: null pointer argument");
  FRWKV_REQUIRE(elements > 0 && elements % 8 == 0, "tmix_act: element count must be a positive multiple of 8");
  FRWKV_REQUIRE(act == 1 || act == 2, "tmix_act: act must be 1 (tanh) or 2 (sigmoid)");
  const long long vec_total = elements / 8;
  long long blocks = (vec_total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  FRWKV_DISPATCH_IO(io_dtype, "tmix_act", {
    launch_chained(act_kernel<io_t>, dim3((unsigned)blocks), dim3(256), 0, s, static_cast<const io_t*>(x), static_cast<io_t*>(out), vec_total, act);
    return check_launch("act_kernel");
  })
}
