// Block-level add + LayerNorm in front of the TMix group, optionally with the token shift (mix6) fused behind it.
//
//   sum  = x + residual                      (rounded to the 16-bit io type: this is the tensor the caller keeps)
//   norm = (sum - mean) * rsqrt(var + eps) * weight + bias     (mean / biased variance of the rounded sum, fp32)
//   mix_j = norm + (prev - norm) * x_j       (prev = shift state of the row's sequence; one-token sequences only)
//
// One CTA per row; the row lives in shared memory as fp32 between the three sweeps (sum, centred squares, output),
// so global memory is read once and written once per tensor.  These rows are a few KB: the kernels are bound by
// launch latency, which is why the fused form exists and why they take part in the chained launches.
//
// Replaces tmix_layer_norm / tmix_add_layer_norm / tmix_add_last_layer_norm / tmix_add
// (flashrwkv2/tmix/normalization/__init__.py:31-90 of the reference, kernels in csrc/sm120/tmix/normalization/) and
// tmix_mix6_add_layer_norm_forward_varlen (flashrwkv2/tmix/mix6/__init__.py:103-199; contract pinned by
// tests/tmix/mix6/test.py:312-368 and tests/tmix/normalization/test.py:17-88).

#include "frwkv_common.cuh"

namespace frwkv {
namespace {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < (kNormThreads >> 5) ? scratch[lane] : 0.f;
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return __shfl_sync(0xffffffffu, t, 0);
}

struct MixVectors {
  const void* v[6];
};

// kMix: after the normalisation, interpolate with the row's shift state six ways and store the normalised row as the
// new shift state (every sequence has exactly one row: row == sequence).
template <typename io_t, bool kMix>
__global__ __launch_bounds__(kNormThreads) void add_layer_norm_kernel(
    const io_t* __restrict__ x, const io_t* __restrict__ residual, const io_t* __restrict__ weight,
    const io_t* __restrict__ bias, io_t* __restrict__ sum_out, io_t* __restrict__ norm_out, MixVectors mix,
    io_t* __restrict__ shift_pool, const int* __restrict__ state_indices, const int* __restrict__ status,
    io_t* __restrict__ mix_out, long long rows, int C, float eps) {
  chain_begin();
  using IO = Io16<io_t>;
  extern __shared__ __align__(16) float row_s[];  // [C]
  __shared__ float red[kNormThreads >> 5];
  const long long row = blockIdx.x;
  const int kv = C >> 3;
  const bool bad = kMix && status != nullptr && status[0] != 0;
  if (bad) {  // fail closed: NaN outputs, shift state untouched
    const uint32_t nan2 = IO::pack(quiet_nan(), quiet_nan());
    const uint4 nanv = make_uint4(nan2, nan2, nan2, nan2);
    for (int c = threadIdx.x; c < kv; c += kNormThreads) {
      if (sum_out != nullptr) reinterpret_cast<uint4*>(sum_out + row * C)[c] = nanv;
      for (int j = 0; j < 6; ++j) reinterpret_cast<uint4*>(mix_out + ((long long)j * rows + row) * C)[c] = nanv;
    }
    return;
  }
  // sweep 1: the (rounded) sum, kept as fp32 in shared memory
  float part = 0.f;
  for (int c = threadIdx.x; c < kv; c += kNormThreads) {
    const uint4 ux = __ldg(reinterpret_cast<const uint4*>(x + row * C) + c);
    float f[8];
    {
      float2 t;
      t = IO::unpack(ux.x); f[0] = t.x; f[1] = t.y;
      t = IO::unpack(ux.y); f[2] = t.x; f[3] = t.y;
      t = IO::unpack(ux.z); f[4] = t.x; f[5] = t.y;
      t = IO::unpack(ux.w); f[6] = t.x; f[7] = t.y;
    }
    if (residual != nullptr) {
      const uint4 ur = __ldg(reinterpret_cast<const uint4*>(residual + row * C) + c);
      float2 t;
      t = IO::unpack(ur.x); f[0] += t.x; f[1] += t.y;
      t = IO::unpack(ur.y); f[2] += t.x; f[3] += t.y;
      t = IO::unpack(ur.z); f[4] += t.x; f[5] += t.y;
      t = IO::unpack(ur.w); f[6] += t.x; f[7] += t.y;
      const uint4 us = make_uint4(IO::pack(f[0], f[1]), IO::pack(f[2], f[3]), IO::pack(f[4], f[5]), IO::pack(f[6], f[7]));
      if (sum_out != nullptr) reinterpret_cast<uint4*>(sum_out + row * C)[c] = us;
      // statistics are those of the rounded sum, the tensor the caller sees
      t = IO::unpack(us.x); f[0] = t.x; f[1] = t.y;
      t = IO::unpack(us.y); f[2] = t.x; f[3] = t.y;
      t = IO::unpack(us.z); f[4] = t.x; f[5] = t.y;
      t = IO::unpack(us.w); f[6] = t.x; f[7] = t.y;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      row_s[8 * c + e] = f[e];
      part += f[e];
    }
  }
  if (weight == nullptr) return;  // plain add
  const float mean = block_sum(part, red) / (float)C;
  // sweep 2: centred squares (each thread revisits the elements it wrote itself)
  part = 0.f;
  for (int c = threadIdx.x; c < kv; c += kNormThreads) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float d = row_s[8 * c + e] - mean;
      part = fmaf(d, d, part);
    }
  }
  const float rstd = rsqrtf(block_sum(part, red) / (float)C + eps);
  // sweep 3: normalise, round, and (kMix) interpolate with the shift state
  const int slot = kMix ? state_indices[row] : 0;
  for (int c = threadIdx.x; c < kv; c += kNormThreads) {
    const uint4 uw = __ldg(reinterpret_cast<const uint4*>(weight) + c);
    const uint4 ub = __ldg(reinterpret_cast<const uint4*>(bias) + c);
    float w[8], b[8], n[8];
    {
      float2 t;
      t = IO::unpack(uw.x); w[0] = t.x; w[1] = t.y; t = IO::unpack(uw.y); w[2] = t.x; w[3] = t.y;
      t = IO::unpack(uw.z); w[4] = t.x; w[5] = t.y; t = IO::unpack(uw.w); w[6] = t.x; w[7] = t.y;
      t = IO::unpack(ub.x); b[0] = t.x; b[1] = t.y; t = IO::unpack(ub.y); b[2] = t.x; b[3] = t.y;
      t = IO::unpack(ub.z); b[4] = t.x; b[5] = t.y; t = IO::unpack(ub.w); b[6] = t.x; b[7] = t.y;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) n[e] = fmaf((row_s[8 * c + e] - mean) * rstd, w[e], b[e]);
    const uint4 un = make_uint4(IO::pack(n[0], n[1]), IO::pack(n[2], n[3]), IO::pack(n[4], n[5]), IO::pack(n[6], n[7]));
    if (norm_out != nullptr) reinterpret_cast<uint4*>(norm_out + row * C)[c] = un;
    if (kMix) {
      {  // the interpolation starts from the rounded normalised row, as if it had been stored and read back
        float2 t;
        t = IO::unpack(un.x); n[0] = t.x; n[1] = t.y; t = IO::unpack(un.y); n[2] = t.x; n[3] = t.y;
        t = IO::unpack(un.z); n[4] = t.x; n[5] = t.y; t = IO::unpack(un.w); n[6] = t.x; n[7] = t.y;
      }
      uint4* state = reinterpret_cast<uint4*>(shift_pool + (long long)slot * C) + c;
      const uint4 up = *state;
      float p[8];
      {
        float2 t;
        t = IO::unpack(up.x); p[0] = t.x; p[1] = t.y; t = IO::unpack(up.y); p[2] = t.x; p[3] = t.y;
        t = IO::unpack(up.z); p[4] = t.x; p[5] = t.y; t = IO::unpack(up.w); p[6] = t.x; p[7] = t.y;
      }
#pragma unroll
      for (int j = 0; j < 6; ++j) {
        const uint4 um = __ldg(reinterpret_cast<const uint4*>(mix.v[j]) + c);
        float m[8], o[8];
        float2 t;
        t = IO::unpack(um.x); m[0] = t.x; m[1] = t.y; t = IO::unpack(um.y); m[2] = t.x; m[3] = t.y;
        t = IO::unpack(um.z); m[4] = t.x; m[5] = t.y; t = IO::unpack(um.w); m[6] = t.x; m[7] = t.y;
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = fmaf(p[e] - n[e], m[e], n[e]);
        reinterpret_cast<uint4*>(mix_out + ((long long)j * rows + row) * C)[c] =
            make_uint4(IO::pack(o[0], o[1]), IO::pack(o[2], o[3]), IO::pack(o[4], o[5]), IO::pack(o[6], o[7]));
      }
      *state = un;  // this row is the only reader of its slot (slots are unique): no hazard
    }
  }
}

template <typename io_t, bool kMix>
int launch_norm(const void* x, const void* residual, const void* weight, const void* bias, void* sum_out, void* norm_out,
                const MixVectors& mix, void* shift_pool, const int* state_indices, const int* status, void* mix_out,
                long long rows, int channels, float eps, cudaStream_t s) {
  const size_t smem = (size_t)channels * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_layer_norm_kernel<io_t, kMix>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "tmix_layer_norm: %s", cudaGetErrorString(e));
  }
  launch_chained(add_layer_norm_kernel<io_t, kMix>, dim3((unsigned)rows), dim3(kNormThreads), smem, s,
                 static_cast<const io_t*>(x), static_cast<const io_t*>(residual), static_cast<const io_t*>(weight),
                 static_cast<const io_t*>(bias), static_cast<io_t*>(sum_out), static_cast<io_t*>(norm_out), mix,
                 static_cast<io_t*>(shift_pool), state_indices, status, static_cast<io_t*>(mix_out), rows, channels, eps);
  return check_launch("add_layer_norm_kernel");
}

int check_norm_sizes(const char* what, long long rows, int channels, float eps, bool needs_eps) {
  FRWKV_REQUIRE(rows > 0 && rows <= 0x7fffffffLL && channels > 0, "%s: sizes must be positive", what);
  FRWKV_REQUIRE(channels % 8 == 0, "%s: channel count must be a multiple of 8", what);
  FRWKV_REQUIRE((size_t)channels * 4 <= 200 * 1024, "%s: at most 51200 channels", what);
  if (needs_eps) FRWKV_REQUIRE(eps > 0.f && eps - eps == 0.f, "%s: eps must be finite and positive", what);
  return FRWKV_OK;
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_tmix_add_layer_norm_forward(const void* x, const void* residual, const void* weight,
                                                 const void* bias, void* sum_out, void* norm_out, long long rows,
                                                 int channels, float eps, int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(x != nullptr, "tmix_layer_norm: null pointer argument");
  FRWKV_REQUIRE((weight == nullptr) == (bias == nullptr), "tmix_layer_norm: weight and bias go together");
  FRWKV_REQUIRE(weight != nullptr || (residual != nullptr && sum_out != nullptr),
                "tmix_layer_norm: without weight and bias the call is a plain add and needs residual and sum_out");
  FRWKV_REQUIRE(weight == nullptr || norm_out != nullptr, "tmix_layer_norm: norm_out is required");
  FRWKV_REQUIRE(sum_out == nullptr || residual != nullptr, "tmix_layer_norm: sum_out needs residual");
  int rc = check_norm_sizes("tmix_layer_norm", rows, channels, eps, weight != nullptr);
  if (rc != FRWKV_OK) return rc;
  const MixVectors none{};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_norm<__nv_bfloat16, false>(x, residual, weight, bias, sum_out, norm_out, none, nullptr, nullptr, nullptr,
                                             nullptr, rows, channels, eps, s);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_norm<__half, false>(x, residual, weight, bias, sum_out, norm_out, none, nullptr, nullptr, nullptr,
                                      nullptr, rows, channels, eps, s);
  return fail(FRWKV_ERR_UNSUPPORTED, "tmix_layer_norm: tensors must be float16 or bfloat16");
}

extern "C" int frwkv_tmix_mix6_add_layer_norm_forward(const void* x, const void* residual, const void* weight,
                                                      const void* bias, const void* x_r, const void* x_w,
                                                      const void* x_k, const void* x_v, const void* x_a,
                                                      const void* x_g, void* shift_state_pool,
                                                      const int32_t* state_indices, const int32_t* metadata_status,
                                                      void* sum_out, void* mix_out, int rows, int channels, float eps,
                                                      int io_dtype, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(x && residual && weight && bias && x_r && x_w && x_k && x_v && x_a && x_g && shift_state_pool &&
                    state_indices && sum_out && mix_out,
                "tmix_mix6_add_layer_norm: null pointer argument");
  int rc = check_norm_sizes("tmix_mix6_add_layer_norm", rows, channels, eps, true);
  if (rc != FRWKV_OK) return rc;
  const MixVectors mix{{x_r, x_w, x_k, x_v, x_a, x_g}};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_norm<__nv_bfloat16, true>(x, residual, weight, bias, sum_out, nullptr, mix, shift_state_pool,
                                            state_indices, metadata_status, mix_out, rows, channels, eps, s);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_norm<__half, true>(x, residual, weight, bias, sum_out, nullptr, mix, shift_state_pool, state_indices,
                                     metadata_status, mix_out, rows, channels, eps, s);
  return fail(FRWKV_ERR_UNSUPPORTED, "tmix_mix6_add_layer_norm: tensors must be float16 or bfloat16");
}
