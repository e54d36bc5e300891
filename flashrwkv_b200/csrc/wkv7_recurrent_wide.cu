// WKV7 recurrence for head sizes 128 and 256 (fp32 state pool updated in place).
//
// One CTA per (sequence, head, block of 128 value columns).  Thread (c, q) = (tid % 128, tid / 128) keeps the 64 state
// values S[64 q + i][v0 + c], i = 0..63, in registers for the whole sequence; a warp's state loads and stores are 128
// contiguous bytes per key row.  Per token the D-vectors (r, w, k, a, b; w through the retention transform) are staged
// in shared memory and read as broadcast float4s; the key-direction sums  sa = S^T a  and  y = S'^T r  are finished
// across the D/64 row slabs through a small table in shared memory.  Value-column blocks of one head never exchange
// data, so a head of 256 is simply two CTAs.
//
// The head-size-64 kernels (wkv7_recurrent.cu) are the tuned ones; this kernel carries the same arithmetic to the
// reference's other head sizes.  Replaces the D = 128 / 256 instantiations of wkv_fp32_v2_kernel
// (csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cu:90-275, dispatch :384-446).

#include "frwkv_common.cuh"

namespace frwkv {
namespace {

constexpr int kCols = 128;  // value columns per CTA

template <typename io_t, int D>
__global__ __launch_bounds__(kCols* (D / 64), 1) void wkv7_recurrent_wide_kernel(
    const int* __restrict__ cu_seqlens, const int* __restrict__ state_indices,
    const int* __restrict__ metadata_status, float* __restrict__ state_pool, const io_t* __restrict__ r_ptr,
    const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr, const io_t* __restrict__ v_ptr,
    const io_t* __restrict__ a_ptr, const io_t* __restrict__ b_ptr, const io_t* __restrict__ bias_ptr,
    io_t* __restrict__ y_ptr, float* __restrict__ y32_ptr, int num_heads, long long output_elements, float scale) {
  using IO = Io16<io_t>;
  constexpr int kSlabs = D / 64, kThreads = kCols * kSlabs, kColBlocks = D / kCols;
  chain_begin();
  if (metadata_status != nullptr && metadata_status[0] != 0) {  // fail closed: NaN output, state untouched
    const io_t nan16 = IO::store(quiet_nan());
    for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < output_elements;
         i += (long long)gridDim.x * kThreads) {
      y_ptr[i] = nan16;
      if (y32_ptr != nullptr) y32_ptr[i] = quiet_nan();
    }
    return;
  }
  __shared__ __align__(16) float vec_s[5][D];          // r, w, k, a, b of the current token
  __shared__ float part_s[kSlabs][kCols];              // per-slab partial sums of sa, then of y
  const int c = threadIdx.x % kCols, q = threadIdx.x / kCols;
  const int cb = blockIdx.x % kColBlocks;
  const long long seq_head = blockIdx.x / kColBlocks;
  const int head = (int)(seq_head % num_heads), seq = (int)(seq_head / num_heads);
  const int col = cb * kCols + c;
  const int t_begin = cu_seqlens[seq], t_end = cu_seqlens[seq + 1];
  float* sbase = state_pool + ((long long)state_indices[seq] * num_heads + head) * ((long long)D * D) +
                 (long long)(64 * q) * D + col;
  float S[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) S[i] = sbase[(long long)i * D];

  for (int t = t_begin; t < t_end; ++t) {
    const long long tb = ((long long)t * num_heads + head) * D;
    __syncthreads();  // the previous token's vectors and partial sums are no longer read
    for (int e = threadIdx.x; e < D; e += kThreads) {
      float x = IO::load(w_ptr + tb + e);
      if (bias_ptr != nullptr) x += IO::load(bias_ptr + head * D + e);
      vec_s[0][e] = IO::load(r_ptr + tb + e);
      vec_s[1][e] = retention(x);
      vec_s[2][e] = IO::load(k_ptr + tb + e);
      vec_s[3][e] = IO::load(a_ptr + tb + e);
      vec_s[4][e] = IO::load(b_ptr + tb + e);
    }
    const float vv = IO::load(v_ptr + tb + col);
    __syncthreads();
    float sa = 0.f;
#pragma unroll
    for (int i = 0; i < 64; i += 4) {
      const float4 a4 = *reinterpret_cast<const float4*>(&vec_s[3][64 * q + i]);
      sa = fmaf(a4.x, S[i], fmaf(a4.y, S[i + 1], fmaf(a4.z, S[i + 2], fmaf(a4.w, S[i + 3], sa))));
    }
    part_s[q][c] = sa;
    __syncthreads();
    sa = 0.f;
#pragma unroll
    for (int j = 0; j < kSlabs; ++j) sa += part_s[j][c];
    __syncthreads();  // everyone has the total before the table is reused for y
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < 64; i += 4) {
      const float4 w4 = *reinterpret_cast<const float4*>(&vec_s[1][64 * q + i]);
      const float4 b4 = *reinterpret_cast<const float4*>(&vec_s[4][64 * q + i]);
      const float4 k4 = *reinterpret_cast<const float4*>(&vec_s[2][64 * q + i]);
      const float4 r4 = *reinterpret_cast<const float4*>(&vec_s[0][64 * q + i]);
      S[i] = fmaf(w4.x, S[i], fmaf(b4.x, sa, k4.x * vv));
      S[i + 1] = fmaf(w4.y, S[i + 1], fmaf(b4.y, sa, k4.y * vv));
      S[i + 2] = fmaf(w4.z, S[i + 2], fmaf(b4.z, sa, k4.z * vv));
      S[i + 3] = fmaf(w4.w, S[i + 3], fmaf(b4.w, sa, k4.w * vv));
      y = fmaf(r4.x, S[i], fmaf(r4.y, S[i + 1], fmaf(r4.z, S[i + 2], fmaf(r4.w, S[i + 3], y))));
    }
    part_s[q][c] = y;
    __syncthreads();
    if (q == 0) {
      y = 0.f;
#pragma unroll
      for (int j = 0; j < kSlabs; ++j) y += part_s[j][c];
      y *= scale;
      y_ptr[tb + col] = IO::store(y);
      if (y32_ptr != nullptr) y32_ptr[tb + col] = y;
    }
  }
#pragma unroll
  for (int i = 0; i < 64; ++i) sbase[(long long)i * D] = S[i];
}

template <typename io_t, int D>
int launch_wide(const int* cu, const int* idx, const int* status, float* state, const void* r, const void* w,
                const void* k, const void* v, const void* a, const void* b, const void* bias, void* y, float* y32,
                int total_tokens, int num_sequences, int num_heads, float scale, cudaStream_t stream) {
  const long long blocks = (long long)num_sequences * num_heads * (D / kCols);
  if (blocks > 0x7fffffffLL) return fail(FRWKV_ERR_INVALID_ARGUMENT, "wkv7_recurrent: too many (sequence, head) pairs");
  launch_chained(wkv7_recurrent_wide_kernel<io_t, D>, dim3((unsigned)blocks), dim3(kCols * (D / 64)), 0, stream, cu, idx,
                 status, state, static_cast<const io_t*>(r), static_cast<const io_t*>(w), static_cast<const io_t*>(k),
                 static_cast<const io_t*>(v), static_cast<const io_t*>(a), static_cast<const io_t*>(b),
                 static_cast<const io_t*>(bias), static_cast<io_t*>(y), y32, num_heads,
                 (long long)total_tokens * num_heads * D, scale);
  return check_launch("wkv7_recurrent_wide_kernel");
}

}  // namespace

int launch_recurrent_wide(const int* cu, const int* idx, const int* status, float* state, const void* r, const void* w,
                          const void* k, const void* v, const void* a, const void* b, const void* bias, void* y,
                          float* y32, int total_tokens, int num_sequences, int num_heads, int head_size, int io_dtype,
                          float scale, cudaStream_t stream) {
#define FRWKV_WIDE(T, DD)                                                                                          \
  return launch_wide<T, DD>(cu, idx, status, state, r, w, k, v, a, b, bias, y, y32, total_tokens, num_sequences, \
                            num_heads, scale, stream)
  if (io_dtype == FRWKV_DTYPE_BF16 && head_size == 128) FRWKV_WIDE(__nv_bfloat16, 128);
  if (io_dtype == FRWKV_DTYPE_BF16 && head_size == 256) FRWKV_WIDE(__nv_bfloat16, 256);
  if (io_dtype == FRWKV_DTYPE_FP16 && head_size == 128) FRWKV_WIDE(__half, 128);
  if (io_dtype == FRWKV_DTYPE_FP16 && head_size == 256) FRWKV_WIDE(__half, 256);
#undef FRWKV_WIDE
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_recurrent: token tensors must be float16 or bfloat16");
}

}  // namespace frwkv
