// WKV7 recurrence with an fp16 state pool updated in place (head size 64): half the state traffic of the fp32 path.
//
// Per token, with the fp16 state S (key row k, value column v) of one (sequence, head):
//     delta[k] = half( exp(-e^-0.5 sigmoid(logit[k] + bias[k])) - 1 + dither )      (the retention as a rounded increment)
//     sa[v]    = sum_k a[k] S[k,v]
//     S'[k,v]  = half( S + S delta[k] + b[k] sa[v] + k[k] v[v] )                   (fp32 arithmetic, one rounding)
//     y[v]     = scale * sum_k r[k] S'[k,v]                                          (from the ROUNDED new state)
// dither = int32( uint32(phase) * 2654435769 ) * 2^-41 with phase = head*64 + k + elapsed[slot] + (token's index in its
// sequence): a deterministic +-2^-10 perturbation that decorrelates the rounding of delta from step to step.  The kernel
// reads the per-slot elapsed counters and never advances them (the caller does, with the advance entry points).
//
// Two kernels share the per-token step:
//   * wkv7_fp16_register_kernel: any packed batch; one warp per half (32 value columns) of a (sequence, head), state in
//     registers as fp32 copies of the fp16 values for the whole sequence;
//   * wkv7_fp16_decode_kernel: batches of one token per sequence; persistent CTAs stream the 8 KB state tiles, two
//     adjacent heads at a time, through a shared-memory ring with bulk copies (loader warp, storer lane, seven pairs of
//     consumer warps), as the fp32 decode kernel does with its 16 KB tiles.
// Lane layout in both: lane = kg*8 + vq holds key rows [16 kg, 16 kg + 16) of value columns [4 vq, 4 vq + 4) of its half.
//
// Replaces the reference's fp16-state family (csrc/sm120/tmix/wkv7/infer_recurrent_fp16_forward_varlen.cu; contract
// restated by rwkv7_fp16_reference, tests/tmix/wkv7/test.py:216-277, and docs/kernel_api.md:85-91,109-123).

#include <cstdlib>

#include "frwkv_common.cuh"
#include "umma.cuh"

namespace frwkv {
// head sizes 128 and 256 (wkv7_recurrent_wide.cu); elapsed != nullptr selects the fp16 pool
int launch_recurrent_wide(const int* cu, const int* idx, const int* status, const int* elapsed, void* state,
                          const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                          const void* bias, void* y, float* y32, int total_tokens, int num_sequences, int num_heads,
                          int head_size, int io_dtype, float scale, cudaStream_t stream);
namespace {

constexpr int kD = 64;

__device__ __forceinline__ void ld16h(const void* p, uint32_t (&w)[8], bool global) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
  const uint4 lo = global ? __ldg(q) : *q, hi = global ? __ldg(q + 1) : *(q + 1);
  w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w;
  w[4] = hi.x; w[5] = hi.y; w[6] = hi.z; w[7] = hi.w;
}
__device__ __forceinline__ float4 half4_to_float4(uint2 u) {
  const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
// round four fp32 values to fp16; returns the packed halves and leaves the rounded values in q
__device__ __forceinline__ uint2 round_half4(float4& q) {
  const __half2 lo = __floats2half2_rn(q.x, q.y), hi = __floats2half2_rn(q.z, q.w);
  const float2 flo = __half22float2(lo), fhi = __half22float2(hi);
  q = make_float4(flo.x, flo.y, fhi.x, fhi.y);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  return u;
}

struct Out4 {
  float o0, o1, o2, o3;
};

// One token on this lane's 16 x 4 piece (fp32 copies of fp16 values in s).  tok_* point at the 64-value rows of this
// (token, head); `global` says whether they are global (register kernel) or shared (decode kernel) memory.  On return
// s holds the rounded new state (exactly representable in fp16); when tile_rows is given, each new row is also
// written there as fp16 (row stride 64 values).
template <typename io_t>
__device__ __forceinline__ Out4 token_step_fp16(float4 (&s)[16], __half* tile_rows, const io_t* tok_r,
                                                const io_t* tok_w, const io_t* tok_k, const io_t* tok_v,
                                                const io_t* tok_a, const io_t* tok_b, const io_t* bias_row,
                                                uint32_t phase0, int row0, int col0, float scale, bool global) {
  using IO = Io16<io_t>;
  const int lane = threadIdx.x & 31;
  // delta of this lane group's 16 key rows: each of the 8 lanes that share the rows computes two and the group
  // exchanges them by shuffle
  float dl[16];
  {
    const int vq = lane & 7;
    const uint32_t xw = global ? __ldg(reinterpret_cast<const uint32_t*>(tok_w + row0 + 2 * vq))
                               : *reinterpret_cast<const uint32_t*>(tok_w + row0 + 2 * vq);
    float2 x = IO::unpack(xw);
    if (bias_row != nullptr) {
      const float2 bx = IO::unpack(__ldg(reinterpret_cast<const uint32_t*>(bias_row + row0 + 2 * vq)));
      x.x += bx.x;
      x.y += bx.y;
    }
    const float d_lo = delta_of(x.x, phase0 + (uint32_t)(row0 + 2 * vq));
    const float d_hi = delta_of(x.y, phase0 + (uint32_t)(row0 + 2 * vq + 1));
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      dl[2 * p] = __shfl_sync(0xffffffffu, d_lo, (lane & 24) + p);
      dl[2 * p + 1] = __shfl_sync(0xffffffffu, d_hi, (lane & 24) + p);
    }
  }
  uint32_t rr[8], aa[8], bb[8], kk[8];
  ld16h(tok_a + row0, aa, global);
  ld16h(tok_b + row0, bb, global);
  ld16h(tok_k + row0, kk, global);
  ld16h(tok_r + row0, rr, global);
  const uint2 vraw = global ? __ldg(reinterpret_cast<const uint2*>(tok_v + col0))
                            : *reinterpret_cast<const uint2*>(tok_v + col0);
  float sa0 = 0.f, sa1 = 0.f, sa2 = 0.f, sa3 = 0.f;
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const float2 a2 = IO::unpack(aa[p]);
    const float4 q0 = s[2 * p], q1 = s[2 * p + 1];
    sa0 = fmaf(a2.x, q0.x, fmaf(a2.y, q1.x, sa0)); sa1 = fmaf(a2.x, q0.y, fmaf(a2.y, q1.y, sa1));
    sa2 = fmaf(a2.x, q0.z, fmaf(a2.y, q1.z, sa2)); sa3 = fmaf(a2.x, q0.w, fmaf(a2.y, q1.w, sa3));
  }
#pragma unroll
  for (int m = 8; m <= 16; m <<= 1) {
    sa0 += __shfl_xor_sync(0xffffffffu, sa0, m); sa1 += __shfl_xor_sync(0xffffffffu, sa1, m);
    sa2 += __shfl_xor_sync(0xffffffffu, sa2, m); sa3 += __shfl_xor_sync(0xffffffffu, sa3, m);
  }
  const float2 v01 = IO::unpack(vraw.x), v23 = IO::unpack(vraw.y);
  float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const float2 b2 = IO::unpack(bb[p]), k2 = IO::unpack(kk[p]), r2 = IO::unpack(rr[p]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float bi = h ? b2.y : b2.x, ki = h ? k2.y : k2.x, ri = h ? r2.y : r2.x, di = dl[2 * p + h];
      float4 q = s[2 * p + h];
      q.x = fmaf(q.x, di, q.x) + fmaf(bi, sa0, ki * v01.x);
      q.y = fmaf(q.y, di, q.y) + fmaf(bi, sa1, ki * v01.y);
      q.z = fmaf(q.z, di, q.z) + fmaf(bi, sa2, ki * v23.x);
      q.w = fmaf(q.w, di, q.w) + fmaf(bi, sa3, ki * v23.y);
      const uint2 enc = round_half4(q);
      if (tile_rows != nullptr) *reinterpret_cast<uint2*>(tile_rows + (2 * p + h) * kD) = enc;
      s[2 * p + h] = q;
      y0 = fmaf(ri, q.x, y0); y1 = fmaf(ri, q.y, y1); y2 = fmaf(ri, q.z, y2); y3 = fmaf(ri, q.w, y3);
    }
  }
#pragma unroll
  for (int m = 8; m <= 16; m <<= 1) {
    y0 += __shfl_xor_sync(0xffffffffu, y0, m); y1 += __shfl_xor_sync(0xffffffffu, y1, m);
    y2 += __shfl_xor_sync(0xffffffffu, y2, m); y3 += __shfl_xor_sync(0xffffffffu, y3, m);
  }
  Out4 out;
  out.o0 = scale * y0; out.o1 = scale * y1; out.o2 = scale * y2; out.o3 = scale * y3;
  return out;
}

template <typename io_t>
__device__ __forceinline__ void fill_nan(io_t* y_ptr, long long output_elements, int threads) {
  const io_t nan16 = Io16<io_t>::store(quiet_nan());
  for (long long i = (long long)blockIdx.x * threads + threadIdx.x; i < output_elements;
       i += (long long)gridDim.x * threads)
    y_ptr[i] = nan16;
}

// ---- any packed batch: state in registers --------------------------------------------------------------------------
constexpr int kRegWarps = 4;

template <typename io_t>
__global__ __launch_bounds__(kRegWarps * 32, 4) void wkv7_fp16_register_kernel(
    const int* __restrict__ cu_seqlens, const int* __restrict__ state_indices, const int* __restrict__ metadata_status,
    const int* __restrict__ elapsed_pool, __half* __restrict__ state_pool, const io_t* __restrict__ r_ptr,
    const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr, const io_t* __restrict__ v_ptr,
    const io_t* __restrict__ a_ptr, const io_t* __restrict__ b_ptr, const io_t* __restrict__ bias_ptr,
    io_t* __restrict__ y_ptr, long long num_units, int num_heads, long long output_elements, float scale) {
  using IO = Io16<io_t>;
  chain_begin();
  if (metadata_status != nullptr && metadata_status[0] != 0) {  // fail closed: NaN output, state untouched
    fill_nan(y_ptr, output_elements, kRegWarps * 32);
    return;
  }
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * kRegWarps + (threadIdx.x >> 5);
  if (unit >= num_units) return;
  const int vhalf = (int)(unit & 1);
  const long long seq_head = unit >> 1;
  const int head = (int)(seq_head % num_heads), seq = (int)(seq_head / num_heads);
  const int kg = lane >> 3, vq = lane & 7, row0 = kg * 16, col0 = vhalf * 32 + vq * 4;
  const int t_begin = cu_seqlens[seq], t_end = cu_seqlens[seq + 1];
  const int slot = state_indices[seq];
  const uint32_t phase_base = (uint32_t)(head * kD) + (uint32_t)elapsed_pool[slot];
  __half* sbase = state_pool + ((long long)slot * num_heads + head) * (kD * kD) + row0 * kD + col0;
  float4 s[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) s[i] = half4_to_float4(*reinterpret_cast<const uint2*>(sbase + i * kD));
  const io_t* bias_row = bias_ptr != nullptr ? bias_ptr + head * kD : nullptr;
  for (int t = t_begin; t < t_end; ++t) {
    const long long tb = ((long long)t * num_heads + head) * kD;
    const Out4 o = token_step_fp16<io_t>(s, nullptr, r_ptr + tb, w_ptr + tb, k_ptr + tb, v_ptr + tb, a_ptr + tb,
                                         b_ptr + tb, bias_row, phase_base + (uint32_t)(t - t_begin), row0, col0, scale,
                                         true);
    if (kg == 0) *reinterpret_cast<uint2*>(y_ptr + tb + col0) = make_uint2(IO::pack(o.o0, o.o1), IO::pack(o.o2, o.o3));
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float4 q = s[i];  // already fp16 values: the conversion is exact
    *reinterpret_cast<uint2*>(sbase + i * kD) = round_half4(q);
  }
}

// ---- decode: persistent CTAs, bulk-copy ring ----------------------------------------------------------------------------
// A stage holds kT state tiles of adjacent heads of one sequence (adjacent in the pool and in the token tensors) and
// their token rows: [kT x 8 KB tiles][6 vectors x kT x 128 B].  Two tiles per stage halve the number of bulk copies per
// byte: with 8 KB copies the per-copy latency of the copy pipeline, not DRAM bandwidth, bounds the kernel.
constexpr int kTileBytes = kD * kD * 2;  // 8 KB
constexpr int kTokBytes = 6 * kD * 2;    // r, w, k, v, a, b rows of one (token, head)
constexpr int kConsumerPairs = 7;
constexpr int kDecodeThreads = 32 * (2 + 2 * kConsumerPairs);
constexpr int kMetaUnits = 512;          // units per CTA whose metadata is staged in shared memory

template <int kT>
struct RingCfg {
  static constexpr int kStages = 24 / kT;
  static constexpr int kStageBytes = kT * (kTileBytes + kTokBytes);
  static constexpr int kSmem = kStages * kStageBytes;  // 215,040
  // a consumer pair's first unit must find its stage in the stage's first phase (a wait for the second fill of a
  // fresh barrier returns at once): no more pairs work than there are stages
  static constexpr int kActivePairs = kStages < kConsumerPairs ? kStages : kConsumerPairs;
};

__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(umma::smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* mbar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(umma::smem_u32(mbar)) : "memory");
}

template <typename io_t, int kT>
__global__ __launch_bounds__(kDecodeThreads, 1) void wkv7_fp16_decode_kernel(
    const int* __restrict__ state_indices, const int* __restrict__ metadata_status,
    const int* __restrict__ elapsed_pool, __half* __restrict__ state_pool, const io_t* __restrict__ r_ptr,
    const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr, const io_t* __restrict__ v_ptr,
    const io_t* __restrict__ a_ptr, const io_t* __restrict__ b_ptr, const io_t* __restrict__ bias_ptr,
    io_t* __restrict__ y_ptr, int num_units, int num_heads, long long output_elements, float scale, int reverse,
    int* __restrict__ error_flag) {
  using IO = Io16<io_t>;
  using R = RingCfg<kT>;
  constexpr int kStages = R::kStages, kStageBytes = R::kStageBytes;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full_bar[kStages], done_bar[kStages], empty_bar[kStages];
  chain_begin();  // the counter kernel of the step before may still be running: nothing is read before this returns
  // state slot and elapsed counter of this CTA's first kMetaUnits units, fetched by all threads before the pipeline
  // starts: the loader, the storer and the consumers would otherwise each wait for two dependent global loads per unit
  __shared__ int slot_s[kMetaUnits], elapsed_s[kMetaUnits];
  const int units_per_seq = num_heads / kT;
  // i-th unit of this CTA; `reverse` walks the pool from the other end (a caller that alternates it between decode
  // steps finds the tiles it touched last, still in L2, first)
  const auto unit_of = [&](int i) {
    const int fwd = blockIdx.x + i * gridDim.x;
    return reverse ? num_units - 1 - fwd : fwd;
  };
  if (metadata_status != nullptr && metadata_status[0] != 0) {
    fill_nan(y_ptr, output_elements, kDecodeThreads);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      umma::mbar_init(&full_bar[i], 1 + 32);  // the tiles' expect_tx arrival + one arrival per loader lane
      umma::mbar_init(&done_bar[i], 2);
      umma::mbar_init(&empty_bar[i], 1);
    }
    umma::mbar_fence_init();
  }
  const int my_units = ((int)blockIdx.x < num_units) ? (num_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  for (int i = threadIdx.x; i < min(my_units, kMetaUnits); i += kDecodeThreads) {
    const int slot = state_indices[unit_of(i) / units_per_seq];
    slot_s[i] = slot;
    elapsed_s[i] = elapsed_pool[slot];
  }
  __syncthreads();
  const auto slot_of = [&](int i) { return i < kMetaUnits ? slot_s[i] : state_indices[unit_of(i) / units_per_seq]; };
  bool ok = true;

  if (warp == 0) {
    // loader (whole warp).  Lane 0 brings the state tiles in with one bulk copy; the 6 x kT token rows of 128 bytes go
    // as 16-byte cp.async pieces spread over the lanes (a bulk copy per row would cost the copy engine a descriptor
    // each).  Each lane's pieces count on the stage's "full" barrier through cp.async.mbarrier.arrive.noinc.
    for (int i = 0; i < my_units && ok; ++i) {
      const int st = i % kStages;
      if (i >= kStages) ok = umma::mbar_wait(&empty_bar[st], ((i / kStages) - 1) & 1);
      if (!ok) break;
      const int unit = unit_of(i);
      const int seq = unit / units_per_seq, head0 = kT * (unit % units_per_seq);
      const long long tb = ((long long)seq * num_heads + head0) * kD;  // one token per sequence
      unsigned char* stage = smem + st * kStageBytes;
      if (lane == 0) {
        const __half* src = state_pool + ((long long)slot_of(i) * num_heads + head0) * (kD * kD);
        umma::mbar_expect_tx(&full_bar[st], kT * kTileBytes);
        umma::bulk_g2s(stage, src, kT * kTileBytes, &full_bar[st]);
      }
      const uint32_t rows = umma::smem_u32(stage + kT * kTileBytes);
#pragma unroll
      for (int p = lane; p < 48 * kT; p += 32) {  // piece p: vector p / (8 kT), 16-byte piece p % (8 kT) of its kT rows
        const int vec = p / (8 * kT), within = p % (8 * kT);
        const io_t* src = vec == 0 ? r_ptr : vec == 1 ? w_ptr : vec == 2 ? k_ptr : vec == 3 ? v_ptr : vec == 4 ? a_ptr : b_ptr;
        umma::cp_async16(rows + p * 16, src + tb + 8 * within, 16u);
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(umma::smem_u32(&full_bar[st])) : "memory");
    }
  } else if (warp == 1) {
    if (lane == 0) {  // storer
      for (int i = 0; i < my_units && ok; ++i) {
        const int st = i % kStages;
        ok = umma::mbar_wait(&done_bar[st], (i / kStages) & 1);
        if (!ok) break;
        const int head0 = kT * (unit_of(i) % units_per_seq);
        __half* dst = state_pool + ((long long)slot_of(i) * num_heads + head0) * (kD * kD);
        bulk_s2g(dst, smem + st * kStageBytes, kT * kTileBytes);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        // at most one store may still be reading shared memory: the stage of unit i-1 is free again
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        if (i >= 1) mbar_arrive(&empty_bar[(i - 1) % kStages]);
      }
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      if (my_units > 0 && ok) mbar_arrive(&empty_bar[(my_units - 1) % kStages]);
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // all state writes are complete before exit
    }
  } else {
    const int pair = (warp - 2) >> 1, vhalf = (warp - 2) & 1;
    const int kg = lane >> 3, vq = lane & 7;
    const int row0 = kg * 16, col0 = vhalf * 32 + vq * 4;
    for (int i = pair < R::kActivePairs ? pair : my_units; i < my_units && ok; i += R::kActivePairs) {
      const int st = i % kStages;
      const int unit = unit_of(i);
      const int seq = unit / units_per_seq, head0 = kT * (unit % units_per_seq);
      const uint32_t elapsed = (uint32_t)(i < kMetaUnits ? elapsed_s[i] : elapsed_pool[slot_of(i)]);
      ok = umma::mbar_wait(&full_bar[st], (i / kStages) & 1);
      if (!ok) {
        // fail closed: this pair's remaining units read as NaN; it never reports them done, so the storer gives
        // up as well and their state tiles keep the values they had
        for (int j = i; j < my_units; j += R::kActivePairs) {
          const int u2 = unit_of(j);
          if (kg == 0)
            for (int t = 0; t < kT; ++t) {
              const long long tb = ((long long)(u2 / units_per_seq) * num_heads + kT * (u2 % units_per_seq) + t) * kD;
              const io_t nan16 = IO::store(quiet_nan());
              for (int e = 0; e < 4; ++e) y_ptr[tb + col0 + e] = nan16;
            }
        }
        break;
      }
      unsigned char* stage = smem + st * kStageBytes;
      const io_t* tok = reinterpret_cast<const io_t*>(stage + kT * kTileBytes);  // vector j of tile t at (j*kT + t)*64
#pragma unroll 1
      for (int t = 0; t < kT; ++t) {
        const int head = head0 + t;
        __half* tile_rows = reinterpret_cast<__half*>(stage + t * kTileBytes) + row0 * kD + col0;
        float4 s[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) s[j] = half4_to_float4(*reinterpret_cast<const uint2*>(tile_rows + j * kD));
        const Out4 o = token_step_fp16<io_t>(s, tile_rows, tok + (0 * kT + t) * kD, tok + (1 * kT + t) * kD,
                                             tok + (2 * kT + t) * kD, tok + (3 * kT + t) * kD, tok + (4 * kT + t) * kD,
                                             tok + (5 * kT + t) * kD, bias_ptr != nullptr ? bias_ptr + head * kD : nullptr,
                                             (uint32_t)(head * kD) + elapsed, row0, col0, scale, false);
        if (kg == 0) {
          const long long tb = ((long long)seq * num_heads + head) * kD;
          *reinterpret_cast<uint2*>(y_ptr + tb + col0) = make_uint2(IO::pack(o.o0, o.o1), IO::pack(o.o2, o.o3));
        }
      }
      umma::fence_async_smem();  // the bulk store reads what this warp just wrote
      __syncwarp();
      if (lane == 0) mbar_arrive(&done_bar[st]);
    }
  }
  if (!ok && lane == 0 && error_flag != nullptr) atomicOr(error_flag, FRWKV_META_WAIT_TIMEOUT);
}

// ---- elapsed counters ---------------------------------------------------------------------------------------------------
__global__ void advance_all_kernel(int* __restrict__ elapsed, long long n, int amount) {
  chain_begin();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    elapsed[i] = (int)((unsigned)elapsed[i] + (unsigned)amount);  // wraps like the 32-bit phase
}
__global__ void advance_varlen_kernel(int* __restrict__ elapsed_pool, const int* __restrict__ cu_seqlens,
                                      const int* __restrict__ state_indices, const int* __restrict__ metadata_status,
                                      int num_sequences) {
  chain_begin();
  if (metadata_status != nullptr && metadata_status[0] != 0) return;  // fail closed: counters untouched
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < num_sequences; i += gridDim.x * blockDim.x) {
    const int slot = state_indices[i];
    elapsed_pool[slot] = (int)((unsigned)elapsed_pool[slot] + (unsigned)(cu_seqlens[i + 1] - cu_seqlens[i]));
  }
}

template <typename io_t>
int launch_fp16(const int* cu, const int* idx, const int* status, const int* elapsed, __half* state, const void* r,
                const void* w, const void* k, const void* v, const void* a, const void* b, const void* bias, void* y,
                int total_tokens, int num_sequences, int num_heads, int max_seqlen, float scale, int reverse,
                cudaStream_t stream) {
  const long long out_elems = (long long)total_tokens * num_heads * kD;
  const int tiles = num_sequences * num_heads;
  if (max_seqlen == 1 && total_tokens == num_sequences && tiles >= 1024) {
    int device = 0, sm_count = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
#define FRWKV_FP16_DECODE(KT)                                                                                     \
  {                                                                                                               \
    cudaError_t e = cudaFuncSetAttribute(wkv7_fp16_decode_kernel<io_t, KT>,                                       \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, RingCfg<KT>::kSmem);        \
    if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "wkv7_recurrent_fp16: %s", cudaGetErrorString(e));          \
    const int units = tiles / KT;                                                                                 \
    const int grid = sm_count > 0 && sm_count < units ? sm_count : units;                                         \
    launch_chained(wkv7_fp16_decode_kernel<io_t, KT>, dim3((unsigned)grid), dim3(kDecodeThreads),                 \
                   (size_t)RingCfg<KT>::kSmem, stream, idx, status, elapsed, state, static_cast<const io_t*>(r),  \
                   static_cast<const io_t*>(w), static_cast<const io_t*>(k), static_cast<const io_t*>(v),         \
                   static_cast<const io_t*>(a), static_cast<const io_t*>(b), static_cast<const io_t*>(bias),      \
                   static_cast<io_t*>(y), units, num_heads, out_elems, scale, reverse, const_cast<int*>(status)); \
  }
    // two adjacent heads per stage (16 KB copies, twelve stages); four per stage (32 KB copies, six stages) measured
    // slower at 256 x 32 tiles: 29.8 us per launch against 24.4 us
    if (num_heads % 2 == 0) FRWKV_FP16_DECODE(2)
    else FRWKV_FP16_DECODE(1)
#undef FRWKV_FP16_DECODE
    return check_launch("wkv7_fp16_decode_kernel");
  }
  const long long units = (long long)tiles * 2;
  const long long blocks = (units + kRegWarps - 1) / kRegWarps;
  launch_chained(wkv7_fp16_register_kernel<io_t>, dim3((unsigned)blocks), dim3(kRegWarps * 32), 0, stream, cu, idx, status,
                 elapsed, state, static_cast<const io_t*>(r), static_cast<const io_t*>(w), static_cast<const io_t*>(k),
                 static_cast<const io_t*>(v), static_cast<const io_t*>(a), static_cast<const io_t*>(b),
                 static_cast<const io_t*>(bias), static_cast<io_t*>(y), units, num_heads, out_elems, scale);
  return check_launch("wkv7_fp16_register_kernel");
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_wkv7_recurrent_fp16_forward_varlen(
    const int32_t* cu_seqlens, const int32_t* state_indices, const int32_t* metadata_status,
    const int32_t* elapsed_state_pool, void* state_pool, const void* r, const void* decay_logits, const void* k,
    const void* v, const void* a, const void* b, const void* decay_bias, void* y, int total_tokens, int num_sequences,
    int num_heads, int head_size, int max_seqlen, int io_dtype, float scale, int flags, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(cu_seqlens && state_indices && elapsed_state_pool && state_pool && r && decay_logits && k && v && a &&
                    b && y,
                "wkv7_recurrent_fp16: null pointer argument");
  FRWKV_REQUIRE(total_tokens > 0 && num_sequences > 0 && num_heads > 0, "wkv7_recurrent_fp16: sizes must be positive");
  FRWKV_REQUIRE(num_sequences <= 65535, "wkv7_recurrent_fp16: at most 65535 sequences per call");
  if (head_size == 128 || head_size == 256)  // the general kernel; the kernels of this file are the tuned head-size-64 ones
    return launch_recurrent_wide(cu_seqlens, state_indices, metadata_status, elapsed_state_pool, state_pool, r,
                                 decay_logits, k, v, a, b, decay_bias, y, nullptr, total_tokens, num_sequences, num_heads,
                                 head_size, io_dtype, scale, reinterpret_cast<cudaStream_t>(stream));
  if (head_size != 64)
    return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_recurrent_fp16: head size must be 64, 128, or 256, got %d", head_size);
  FRWKV_REQUIRE((long long)num_sequences * num_heads * 2 <= 0x7fffffffLL, "wkv7_recurrent_fp16: too many units");
  FRWKV_REQUIRE(scale == scale && scale - scale == 0.f, "wkv7_recurrent_fp16: scale must be finite");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int reverse = (flags & FRWKV_RECURRENT_REVERSE_ORDER) ? 1 : 0;
  __half* st = static_cast<__half*>(state_pool);
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_fp16<__nv_bfloat16>(cu_seqlens, state_indices, metadata_status, elapsed_state_pool, st, r,
                                      decay_logits, k, v, a, b, decay_bias, y, total_tokens, num_sequences, num_heads,
                                      max_seqlen, scale, reverse, s);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_fp16<__half>(cu_seqlens, state_indices, metadata_status, elapsed_state_pool, st, r, decay_logits, k, v,
                               a, b, decay_bias, y, total_tokens, num_sequences, num_heads, max_seqlen, scale, reverse,
                               s);
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_recurrent_fp16: token tensors must be float16 or bfloat16");
}

extern "C" int frwkv_recurrent_fp16_advance_i32(int32_t* elapsed_state, long long count, int amount,
                                                frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(elapsed_state != nullptr && count > 0, "recurrent_fp16_advance: a non-empty counter array is required");
  const long long blocks = (count + 255) / 256;
  launch_chained(advance_all_kernel, dim3((unsigned)(blocks > 1024 ? 1024 : blocks)), dim3(256), 0,
                 reinterpret_cast<cudaStream_t>(stream), elapsed_state, count, amount);
  return check_launch("advance_all_kernel");
}

extern "C" int frwkv_recurrent_fp16_advance_i32_varlen(int32_t* elapsed_state_pool, const int32_t* cu_seqlens,
                                                       const int32_t* state_indices, const int32_t* metadata_status,
                                                       int num_sequences, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(elapsed_state_pool && cu_seqlens && state_indices, "recurrent_fp16_advance_varlen: null pointer argument");
  FRWKV_REQUIRE(num_sequences > 0, "recurrent_fp16_advance_varlen: sizes must be positive");
  const int blocks = (num_sequences + 255) / 256;
  launch_chained(advance_varlen_kernel, dim3((unsigned)blocks), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
                 elapsed_state_pool, cu_seqlens, state_indices, metadata_status, num_sequences);
  return check_launch("advance_varlen_kernel");
}
