// WKV7 recurrence for head sizes 128 and 256, on an fp32 or an fp16 state pool (updated in place).
//
// One CTA per (sequence, head, block of 128 value columns).  Thread (c, q) = (tid % 128, tid / 128) keeps the 64 state
// values S[64 q + i][v0 + c], i = 0..63, in registers for the whole sequence; a warp's state loads and stores are 128
// contiguous bytes per key row.  Per token the D-vectors (r, w, k, a, b; w through the retention transform) are staged
// in shared memory and read as broadcast float4s; the key-direction sums  sa = S^T a  and  y = S'^T r  are finished
// across the D/64 row slabs through a small table in shared memory.  Value-column blocks of one head never exchange
// data, so a head of 256 is simply two CTAs.
//
// On an fp16 pool (state_t = __half) the state values live in registers as the fp32 copies of fp16 numbers and every
// token rounds them once: S' = half(S + S * delta + b * sa + k * v) with delta = half(w - 1 + dither), the dither
// phase head * D + key channel + elapsed[slot] + token offset; the output comes from the rounded state.  The elapsed
// counters are only read.
//
// The head-size-64 kernels (wkv7_recurrent.cu, wkv7_recurrent_fp16.cu) are the tuned ones; this kernel carries the
// same arithmetic to the reference's other head sizes.  Replaces the D = 128 / 256 instantiations of
// wkv_fp32_v2_kernel (csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cu:90-275, dispatch :384-446) and
// of the fp16-state kernel families (csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu:503-1076).

#include "frwkv_common.cuh"

namespace frwkv {
namespace {

constexpr int kCols = 128;  // value columns per CTA

__device__ __forceinline__ float state_load(const float* p) { return *p; }
__device__ __forceinline__ float state_load(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void state_store(float* p, float x) { *p = x; }
__device__ __forceinline__ void state_store(__half* p, float x) { *p = __float2half_rn(x); }

template <typename io_t, typename state_t, int D>
__global__ __launch_bounds__(kCols* (D / 64), 1) void wkv7_recurrent_wide_kernel(
    const int* __restrict__ cu_seqlens, const int* __restrict__ state_indices,
    const int* __restrict__ metadata_status, const int* __restrict__ elapsed_pool, state_t* __restrict__ state_pool,
    const io_t* __restrict__ r_ptr,
    const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr, const io_t* __restrict__ v_ptr,
    const io_t* __restrict__ a_ptr, const io_t* __restrict__ b_ptr, const io_t* __restrict__ bias_ptr,
    io_t* __restrict__ y_ptr, float* __restrict__ y32_ptr, int num_heads, long long output_elements, float scale) {
  using IO = Io16<io_t>;
  constexpr bool kHalfState = sizeof(state_t) == 2;
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
  const int slot = state_indices[seq];
  state_t* sbase = state_pool + ((long long)slot * num_heads + head) * ((long long)D * D) + (long long)(64 * q) * D + col;
  uint32_t phase = 0;
  if constexpr (kHalfState) phase = (uint32_t)(head * D) + (uint32_t)elapsed_pool[slot];
  float S[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) S[i] = state_load(sbase + (long long)i * D);

  for (int t = t_begin; t < t_end; ++t) {
    const long long tb = ((long long)t * num_heads + head) * D;
    __syncthreads();  // the previous token's vectors and partial sums are no longer read
    for (int e = threadIdx.x; e < D; e += kThreads) {
      float x = IO::load(w_ptr + tb + e);
      if (bias_ptr != nullptr) x += IO::load(bias_ptr + head * D + e);
      vec_s[0][e] = IO::load(r_ptr + tb + e);
      // retention w on an fp32 pool, the rounded increment w - 1 + dither on an fp16 pool
      vec_s[1][e] = kHalfState ? delta_of(x, phase + (uint32_t)e + (uint32_t)(t - t_begin)) : retention(x);
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
      if constexpr (kHalfState) {  // same order of operations as the head-size-64 fp16 kernels
        S[i] = __half2float(__float2half_rn(fmaf(S[i], w4.x, S[i]) + fmaf(b4.x, sa, k4.x * vv)));
        S[i + 1] = __half2float(__float2half_rn(fmaf(S[i + 1], w4.y, S[i + 1]) + fmaf(b4.y, sa, k4.y * vv)));
        S[i + 2] = __half2float(__float2half_rn(fmaf(S[i + 2], w4.z, S[i + 2]) + fmaf(b4.z, sa, k4.z * vv)));
        S[i + 3] = __half2float(__float2half_rn(fmaf(S[i + 3], w4.w, S[i + 3]) + fmaf(b4.w, sa, k4.w * vv)));
      } else {
        S[i] = fmaf(w4.x, S[i], fmaf(b4.x, sa, k4.x * vv));
        S[i + 1] = fmaf(w4.y, S[i + 1], fmaf(b4.y, sa, k4.y * vv));
        S[i + 2] = fmaf(w4.z, S[i + 2], fmaf(b4.z, sa, k4.z * vv));
        S[i + 3] = fmaf(w4.w, S[i + 3], fmaf(b4.w, sa, k4.w * vv));
      }
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
  for (int i = 0; i < 64; ++i) state_store(sbase + (long long)i * D, S[i]);
}

template <typename io_t, typename state_t, int D>
int launch_wide(const int* cu, const int* idx, const int* status, const int* elapsed, state_t* state, const void* r,
                const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias, void* y,
                float* y32, int total_tokens, int num_sequences, int num_heads, float scale, cudaStream_t stream) {
  const long long blocks = (long long)num_sequences * num_heads * (D / kCols);
  if (blocks > 0x7fffffffLL) return fail(FRWKV_ERR_INVALID_ARGUMENT, "wkv7_recurrent: too many (sequence, head) pairs");
  launch_chained(wkv7_recurrent_wide_kernel<io_t, state_t, D>, dim3((unsigned)blocks), dim3(kCols * (D / 64)), 0, stream,
                 cu, idx, status, elapsed, state, static_cast<const io_t*>(r), static_cast<const io_t*>(w),
                 static_cast<const io_t*>(k), static_cast<const io_t*>(v), static_cast<const io_t*>(a),
                 static_cast<const io_t*>(b), static_cast<const io_t*>(bias), static_cast<io_t*>(y), y32, num_heads,
                 (long long)total_tokens * num_heads * D, scale);
  return check_launch("wkv7_recurrent_wide_kernel");
}

template <typename io_t, int D>
int launch_wide_state(const int* cu, const int* idx, const int* status, const int* elapsed, void* state, const void* r,
                      const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias,
                      void* y, float* y32, int total_tokens, int num_sequences, int num_heads, float scale,
                      cudaStream_t stream) {
  if (elapsed != nullptr)
    return launch_wide<io_t, __half, D>(cu, idx, status, elapsed, static_cast<__half*>(state), r, w, k, v, a, b, bias, y,
                                        y32, total_tokens, num_sequences, num_heads, scale, stream);
  return launch_wide<io_t, float, D>(cu, idx, status, nullptr, static_cast<float*>(state), r, w, k, v, a, b, bias, y,
                                     y32, total_tokens, num_sequences, num_heads, scale, stream);
}

}  // namespace

// elapsed == nullptr: fp32 state pool; otherwise an fp16 pool with its elapsed counters (dither phase).
int launch_recurrent_wide(const int* cu, const int* idx, const int* status, const int* elapsed, void* state,
                          const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                          const void* bias, void* y, float* y32, int total_tokens, int num_sequences, int num_heads,
                          int head_size, int io_dtype, float scale, cudaStream_t stream) {
#define FRWKV_WIDE(T, DD)                                                                                         \
  return launch_wide_state<T, DD>(cu, idx, status, elapsed, state, r, w, k, v, a, b, bias, y, y32, total_tokens, \
                                  num_sequences, num_heads, scale, stream)
  if (io_dtype == FRWKV_DTYPE_BF16 && head_size == 128) FRWKV_WIDE(__nv_bfloat16, 128);
  if (io_dtype == FRWKV_DTYPE_BF16 && head_size == 256) FRWKV_WIDE(__nv_bfloat16, 256);
  if (io_dtype == FRWKV_DTYPE_FP16 && head_size == 128) FRWKV_WIDE(__half, 128);
  if (io_dtype == FRWKV_DTYPE_FP16 && head_size == 256) FRWKV_WIDE(__half, 256);
#undef FRWKV_WIDE
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_recurrent: token tensors must be float16 or bfloat16");
}

}  // namespace frwkv
