// Dense training layout: the state after every 16 tokens, [B][H][T/16][key][value] fp32, as the reference's
// pretraining forward leaves it for its backward (forward_kernel_preload,
// csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cu:32-97, the `s_` stores at :85-92).
//
// The chunked forward has already produced the state at the start of every 64-token chunk and the row
// sa_t = S_{t-1}^T a_t of every token.  With sa known the recurrence has no reduction left,
//     S_t[k][v] = w_t[k] S_{t-1}[k][v] + b_t[k] sa_t[v] + k_t[k] v_t[v],
// so every (chunk, head) is advanced independently and element-wise: one CTA per (chunk, head), 256 threads, each
// thread 4 keys x 4 values of the state in registers, 16 tokens staged in shared memory at a time.  HBM-bound on
// the checkpoint stores (16 KB per 16 tokens and head, against 1.6 KB of token data read).
#include "frwkv_common.cuh"

namespace frwkv {
namespace {

constexpr int kD = 64;
constexpr int kGroup = 16;  // tokens between checkpoints
constexpr int kThreads = 256;

template <typename io_t>
__global__ __launch_bounds__(kThreads, 4) void dense_checkpoints_kernel(
    const float* __restrict__ boundary, const float* __restrict__ state_dot_a, const io_t* __restrict__ decay_logits,
    const io_t* __restrict__ k_, const io_t* __restrict__ v_, const io_t* __restrict__ b_,
    float* __restrict__ checkpoints, int tokens, int heads, int chunks_per_sequence) {
  __shared__ __align__(16) float s_w[kGroup][kD], s_b[kGroup][kD], s_k[kGroup][kD], s_v[kGroup][kD], s_sa[kGroup][kD];
  const int c = blockIdx.x, h = blockIdx.y, bi = blockIdx.z;
  const int tid = threadIdx.x;
  const int v0 = (tid & 15) * 4;  // four consecutive value columns
  const int k0 = tid >> 4;        // keys k0, k0 + 16, k0 + 32, k0 + 48

  float S[4][4];
  {
    const float* src = boundary + ((long long)(bi * chunks_per_sequence + c) * heads + h) * (kD * kD);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 x = *reinterpret_cast<const float4*>(src + (k0 + 16 * q) * kD + v0);
      S[q][0] = x.x; S[q][1] = x.y; S[q][2] = x.z; S[q][3] = x.w;
    }
  }
  const int first = c * 64;
  const int groups = min(4, (tokens - first) / kGroup);
  const int groups_total = tokens / kGroup;
  float* out = checkpoints + ((long long)(bi * heads + h) * groups_total + first / kGroup) * (kD * kD);

  for (int g = 0; g < groups; ++g) {
    const long long tok0 = (long long)bi * tokens + first + g * kGroup;
    __syncthreads();
    {  // stage 16 tokens: thread -> token tid / 16, four channels (tid % 16) * 4
      const int tt = tid >> 4, ch = (tid & 15) * 4;
      const long long off = ((tok0 + tt) * heads + h) * kD + ch;
      const uint2 wb = *reinterpret_cast<const uint2*>(decay_logits + off);
      const uint2 bb = *reinterpret_cast<const uint2*>(b_ + off);
      const uint2 kb = *reinterpret_cast<const uint2*>(k_ + off);
      const uint2 vb = *reinterpret_cast<const uint2*>(v_ + off);
      float2 lo, hi;
      lo = Io16<io_t>::unpack(wb.x); hi = Io16<io_t>::unpack(wb.y);
      *reinterpret_cast<float4*>(&s_w[tt][ch]) =
          make_float4(retention(lo.x), retention(lo.y), retention(hi.x), retention(hi.y));
      lo = Io16<io_t>::unpack(bb.x); hi = Io16<io_t>::unpack(bb.y);
      *reinterpret_cast<float4*>(&s_b[tt][ch]) = make_float4(lo.x, lo.y, hi.x, hi.y);
      lo = Io16<io_t>::unpack(kb.x); hi = Io16<io_t>::unpack(kb.y);
      *reinterpret_cast<float4*>(&s_k[tt][ch]) = make_float4(lo.x, lo.y, hi.x, hi.y);
      lo = Io16<io_t>::unpack(vb.x); hi = Io16<io_t>::unpack(vb.y);
      *reinterpret_cast<float4*>(&s_v[tt][ch]) = make_float4(lo.x, lo.y, hi.x, hi.y);
      *reinterpret_cast<float4*>(&s_sa[tt][ch]) = *reinterpret_cast<const float4*>(state_dot_a + off);
    }
    __syncthreads();
#pragma unroll 4
    for (int tt = 0; tt < kGroup; ++tt) {
      const float4 sa = *reinterpret_cast<const float4*>(&s_sa[tt][v0]);
      const float4 vv = *reinterpret_cast<const float4*>(&s_v[tt][v0]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int key = k0 + 16 * q;
        const float w = s_w[tt][key], bk = s_b[tt][key], kk = s_k[tt][key];
        S[q][0] = fmaf(S[q][0], w, fmaf(bk, sa.x, kk * vv.x));
        S[q][1] = fmaf(S[q][1], w, fmaf(bk, sa.y, kk * vv.y));
        S[q][2] = fmaf(S[q][2], w, fmaf(bk, sa.z, kk * vv.z));
        S[q][3] = fmaf(S[q][3], w, fmaf(bk, sa.w, kk * vv.w));
      }
    }
    float* dst = out + (long long)g * (kD * kD);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      *reinterpret_cast<float4*>(dst + (k0 + 16 * q) * kD + v0) = make_float4(S[q][0], S[q][1], S[q][2], S[q][3]);
  }
}

template <typename io_t>
int launch_checkpoints(const float* boundary, const float* state_dot_a, const void* decay_logits, const void* k,
                       const void* v, const void* b, float* checkpoints, int batch, int tokens, int heads,
                       cudaStream_t stream) {
  const int per = (tokens + 63) / 64;
  dense_checkpoints_kernel<io_t><<<dim3(per, heads, batch), kThreads, 0, stream>>>(
      boundary, state_dot_a, static_cast<const io_t*>(decay_logits), static_cast<const io_t*>(k),
      static_cast<const io_t*>(v), static_cast<const io_t*>(b), checkpoints, tokens, heads, per);
  return check_launch("wkv7_dense_checkpoints");
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_wkv7_dense_checkpoints(const float* boundary, const float* state_dot_a, const void* decay_logits,
                                            const void* k, const void* v, const void* b, float* checkpoints, int batch,
                                            int tokens, int num_heads, int head_size, int io_dtype,
                                            frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(boundary && state_dot_a && decay_logits && k && v && b && checkpoints,
                "wkv7_dense_checkpoints: null pointer argument");
  FRWKV_REQUIRE(batch > 0 && tokens > 0 && num_heads > 0, "wkv7_dense_checkpoints: sizes must be positive");
  FRWKV_REQUIRE(tokens % 16 == 0, "wkv7_dense_checkpoints: tokens must be a multiple of 16");
  FRWKV_REQUIRE(batch <= 65535 && num_heads <= 65535, "wkv7_dense_checkpoints: batch and heads must be <= 65535");
  if (head_size != 64)
    return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_dense_checkpoints: head size %d is not built (only 64)", head_size);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_checkpoints<__nv_bfloat16>(boundary, state_dot_a, decay_logits, k, v, b, checkpoints, batch, tokens,
                                             num_heads, s);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_checkpoints<__half>(boundary, state_dot_a, decay_logits, k, v, b, checkpoints, batch, tokens,
                                      num_heads, s);
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_dense_checkpoints: token tensors must be float16 or bfloat16");
}
