// WKV7 recurrence over packed sequences, fp32 state pool updated in place (head size 64).
//
// Work decomposition.  One warp owns one half (32 value columns) of one
// (sequence, head) state for the whole sequence; the two halves of a head never
// exchange data, so there is no shared memory and no block-level barrier.
// Inside the warp, lane = kg*8 + vq: the lane holds key rows [16*kg, 16*kg+16)
// of value columns [4*vq, 4*vq+4) -- 16 float4 registers.  A row segment of the
// eight lanes with equal kg is 128 contiguous bytes, so every state load and
// store instruction moves four full 128-byte lines, and the 16 independent
// 128-bit loads per lane are issued back to back before the first use.
//
// One sweep per token.  With S' = diag(w) S + b sa^T + k v^T,
//     y / scale = S'^T r = S^T (w*r) + (b.r) sa + (k.r) v,
// so both matrix-vector products (S^T a and S^T (w*r)) read the OLD state in the
// same pass; the key-direction sums finish with two xor-shuffles (over kg), then
// the update streams out of the registers.  A decode step (one token per
// sequence) therefore reads and writes each state element exactly once.
//
// Replaces wkv_fp32_v2_kernel / wkv_fp32_v2_small_warp_kernel of the reference
// (csrc/sm120/tmix/wkv7/infer_recurrent_fp32io16_forward_varlen.cu:90-275).

#include "frwkv_common.cuh"
#include "umma.cuh"

namespace frwkv {
// head sizes 128 and 256 (wkv7_recurrent_wide.cu)
int launch_recurrent_wide(const int* cu, const int* idx, const int* status, const int* elapsed, void* state,
                          const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                          const void* bias, void* y, float* y32, int total_tokens, int num_sequences, int num_heads,
                          int head_size, int io_dtype, float scale, cudaStream_t stream);
namespace {
// Decode batches with more (sequence, head) tiles than this take the bulk-copy ring kernel, smaller ones the register
// kernel.  Measured per launch in a CUDA graph (H = 32, register / ring): 1024 tiles 6.9 / 8.5 us, 2048 10.3 / 12.2,
// 3072 14.4 / 16.5, 4096 20.8 / 21.2, 5120 30.5 / 27.6, 6144 38.0 / 32.4, 8192 50.1 / 43.5.  Up to 4096 tiles the
// state (64 MB) stays in the 126 MB L2 between steps and the ring's fill and drain is pure overhead; beyond that the
// step streams from HBM and the ring's deeper queue of copies wins.
constexpr long long kRingMinTiles = 4608;


constexpr int kD = 64;
constexpr int kWarpsPerBlock = 4;
constexpr int kThreads = kWarpsPerBlock * 32;

__device__ __forceinline__ void load16(const void* p, uint32_t (&w)[8]) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
  const uint4 lo = __ldg(q), hi = __ldg(q + 1);
  w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w;
  w[4] = hi.x; w[5] = hi.y; w[6] = hi.z; w[7] = hi.w;
}

struct StepOut {
  float sa0, sa1, sa2, sa3;  // S_{t-1}^T a for this lane's four value columns
  float o0, o1, o2, o3;      // scale * S_t^T r for the same columns
};

// One token of the recurrence on this lane's 16 x 4 piece of the state (rows row0.., columns col0..); tb is the
// element offset of (token, head) in the packed token tensors.  Returns the complete (all key rows) sums.
// kNeedOutput = false (the training-side replay) leaves out r and everything that only the output needs.
template <typename io_t, bool kNeedOutput>
__device__ __forceinline__ StepOut token_step(float4 (&s)[16], const io_t* __restrict__ r_ptr,
                                              const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr,
                                              const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr,
                                              const io_t* __restrict__ b_ptr, const io_t* __restrict__ bias_ptr,
                                              long long tb, int head, int row0, int col0, float scale) {
  using IO = Io16<io_t>;
  const int lane = threadIdx.x & 31;
  uint32_t rr[8], kk[8], aa[8], bb[8];
  // retention of this lane group's 16 key rows: each of the eight lanes that share the rows computes two of them and
  // the group exchanges them by shuffle (three special-function instructions per value: all sixteen on every lane
  // would make that unit, not the FMAs, the limit of the step)
  const int vq = lane & 7;
  float2 wx = IO::unpack(__ldg(reinterpret_cast<const uint32_t*>(w_ptr + tb + row0 + 2 * vq)));
  load16(a_ptr + tb + row0, aa);
  if (kNeedOutput) load16(r_ptr + tb + row0, rr);
  load16(b_ptr + tb + row0, bb);
  load16(k_ptr + tb + row0, kk);
  const uint2 vraw = __ldg(reinterpret_cast<const uint2*>(v_ptr + tb + col0));

  float wv[16];
  {
    if (bias_ptr != nullptr) {
      const float2 bx = IO::unpack(__ldg(reinterpret_cast<const uint32_t*>(bias_ptr + head * kD + row0 + 2 * vq)));
      wx.x += bx.x;
      wx.y += bx.y;
    }
    const float w_lo = retention(wx.x), w_hi = retention(wx.y);
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      wv[2 * p] = __shfl_sync(0xffffffffu, w_lo, (lane & 24) + p);
      wv[2 * p + 1] = __shfl_sync(0xffffffffu, w_hi, (lane & 24) + p);
    }
  }

  // The four value columns of a lane travel as two pairs: fma.rn.f32x2 does two multiply-adds per instruction, each
  // rounded as the scalar one would be, so the results are the bits of the scalar form.
  float2 sa01 = make_float2(0.f, 0.f), sa23 = sa01, y01 = sa01, y23 = sa01;
  float br = 0.f, kr = 0.f;
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const float2 a2 = IO::unpack(aa[p]);
    float2 r2 = make_float2(0.f, 0.f);
    if (kNeedOutput) {
      r2 = IO::unpack(rr[p]);
      const float2 b2 = IO::unpack(bb[p]), k2 = IO::unpack(kk[p]);
      br = fmaf(b2.x, r2.x, br);
      br = fmaf(b2.y, r2.y, br);
      kr = fmaf(k2.x, r2.x, kr);
      kr = fmaf(k2.y, r2.y, kr);
    }
    {
      const float4 q = s[2 * p];
      const float2 ax = make_float2(a2.x, a2.x);
      sa01 = __ffma2_rn(ax, make_float2(q.x, q.y), sa01);
      sa23 = __ffma2_rn(ax, make_float2(q.z, q.w), sa23);
      if (kNeedOutput) {
        const float wr = wv[2 * p] * r2.x;
        const float2 wr2 = make_float2(wr, wr);
        y01 = __ffma2_rn(wr2, make_float2(q.x, q.y), y01);
        y23 = __ffma2_rn(wr2, make_float2(q.z, q.w), y23);
      }
    }
    {
      const float4 q = s[2 * p + 1];
      const float2 ay = make_float2(a2.y, a2.y);
      sa01 = __ffma2_rn(ay, make_float2(q.x, q.y), sa01);
      sa23 = __ffma2_rn(ay, make_float2(q.z, q.w), sa23);
      if (kNeedOutput) {
        const float wr = wv[2 * p + 1] * r2.y;
        const float2 wr2 = make_float2(wr, wr);
        y01 = __ffma2_rn(wr2, make_float2(q.x, q.y), y01);
        y23 = __ffma2_rn(wr2, make_float2(q.z, q.w), y23);
      }
    }
  }
  float sa0 = sa01.x, sa1 = sa01.y, sa2 = sa23.x, sa3 = sa23.y;
  float y0 = y01.x, y1 = y01.y, y2 = y23.x, y3 = y23.y;
  // finish the key-direction sums across the four row groups (lane bits 3 and 4)
#pragma unroll
  for (int m = 8; m <= 16; m <<= 1) {
    sa0 += __shfl_xor_sync(0xffffffffu, sa0, m); sa1 += __shfl_xor_sync(0xffffffffu, sa1, m);
    sa2 += __shfl_xor_sync(0xffffffffu, sa2, m); sa3 += __shfl_xor_sync(0xffffffffu, sa3, m);
    if (kNeedOutput) {
      y0 += __shfl_xor_sync(0xffffffffu, y0, m); y1 += __shfl_xor_sync(0xffffffffu, y1, m);
      y2 += __shfl_xor_sync(0xffffffffu, y2, m); y3 += __shfl_xor_sync(0xffffffffu, y3, m);
      br += __shfl_xor_sync(0xffffffffu, br, m); kr += __shfl_xor_sync(0xffffffffu, kr, m);
    }
  }
  const float2 v01 = IO::unpack(vraw.x), v23 = IO::unpack(vraw.y);
  sa01 = make_float2(sa0, sa1);
  sa23 = make_float2(sa2, sa3);

#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const float2 b2 = IO::unpack(bb[p]), k2 = IO::unpack(kk[p]);
    {
      float4 q = s[2 * p];
      const float2 wi = make_float2(wv[2 * p], wv[2 * p]), bx = make_float2(b2.x, b2.x), kx = make_float2(k2.x, k2.x);
      const float2 lo = __ffma2_rn(wi, make_float2(q.x, q.y), __ffma2_rn(bx, sa01, __fmul2_rn(kx, v01)));
      const float2 hi = __ffma2_rn(wi, make_float2(q.z, q.w), __ffma2_rn(bx, sa23, __fmul2_rn(kx, v23)));
      s[2 * p] = make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    {
      float4 q = s[2 * p + 1];
      const float2 wi = make_float2(wv[2 * p + 1], wv[2 * p + 1]), by = make_float2(b2.y, b2.y), ky = make_float2(k2.y, k2.y);
      const float2 lo = __ffma2_rn(wi, make_float2(q.x, q.y), __ffma2_rn(by, sa01, __fmul2_rn(ky, v01)));
      const float2 hi = __ffma2_rn(wi, make_float2(q.z, q.w), __ffma2_rn(by, sa23, __fmul2_rn(ky, v23)));
      s[2 * p + 1] = make_float4(lo.x, lo.y, hi.x, hi.y);
    }
  }
  StepOut out;
  out.sa0 = sa0; out.sa1 = sa1; out.sa2 = sa2; out.sa3 = sa3;
  out.o0 = scale * fmaf(kr, v01.x, fmaf(br, sa0, y0));
  out.o1 = scale * fmaf(kr, v01.y, fmaf(br, sa1, y1));
  out.o2 = scale * fmaf(kr, v23.x, fmaf(br, sa2, y2));
  out.o3 = scale * fmaf(kr, v23.y, fmaf(br, sa3, y3));
  return out;
}

// kReplay = true turns the kernel into the training-side "replay": units are (chunk, head, half), the state is
// read from the chunk-start boundary tensor and never written back, and instead of being discarded the per-token
// S^T a vectors (state_dot_a) and the states after every 16th token of a chunk (checkpoints for the backward
// pass) are stored.  cu_seqlens / state_indices then hold chunk_starts / chunk_ends.
// kDirect (decode of a batch whose sequence i is token i and owns state slot i, as a host-checked ticket has
// established): neither table is read, and the status word is asked for together with the state tile instead of one
// round trip ahead of it; the kernel is then one dependent round trip shorter, which shows when a launch is a few
// hundred tiles and bound by that chain.
template <typename io_t, bool kReplay, bool kDirect = false>
__global__ __launch_bounds__(kThreads, 4) void wkv7_recurrent_d64_kernel(
    const int* __restrict__ cu_seqlens, const int* __restrict__ state_indices,
    const int* __restrict__ metadata_status, float* __restrict__ state_pool,
    const io_t* __restrict__ r_ptr, const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr,
    const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr, const io_t* __restrict__ b_ptr,
    const io_t* __restrict__ bias_ptr, io_t* __restrict__ y_ptr, float* __restrict__ y32_ptr,
    float* __restrict__ sa_ptr, float* __restrict__ ckpt_ptr, long long num_units, int num_heads,
    long long output_elements, float scale) {
  using IO = Io16<io_t>;
  chain_begin();
  const int lane = threadIdx.x & 31;
  const long long unit_raw = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const bool active = unit_raw < num_units;
  const long long unit = active ? unit_raw : 0;
  const int vhalf = (int)(unit & 1);
  const long long seq_head = unit >> 1;
  const int head = (int)(seq_head % num_heads);
  const int seq = (int)(seq_head / num_heads);
  const int kg = lane >> 3, vq = lane & 7;
  const int row0 = kg * 16;
  const int col0 = vhalf * 32 + vq * 4;
  // the status word and the sequence's metadata are requested together (one round trip, not two in a row: in a decode
  // step of a few hundred tiles the kernel is a chain of dependent loads)
  const int status0 = (!kReplay && metadata_status != nullptr) ? metadata_status[0] : 0;
  const int t_begin = kDirect ? seq : cu_seqlens[seq];
  const int t_end = kDirect ? seq + 1 : (kReplay ? state_indices[seq] : cu_seqlens[seq + 1]);
  const int slot = (kReplay || kDirect) ? seq : state_indices[seq];
  float4 s[16];
  float* sbase = state_pool + ((long long)slot * num_heads + head) * (kD * kD) + row0 * kD + col0;
  if (kDirect) {  // the tile's address needs no table: its loads leave with the status word's
#pragma unroll
    for (int i = 0; i < 16; ++i) s[i] = *reinterpret_cast<const float4*>(sbase + i * kD);
  }
  if (status0 != 0) {
    // fail closed: NaN output, state untouched
    const io_t nan16 = IO::store(quiet_nan());
    for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < output_elements;
         i += (long long)gridDim.x * kThreads) {
      y_ptr[i] = nan16;
      if (y32_ptr != nullptr) y32_ptr[i] = quiet_nan();
    }
    return;
  }
  if (!active) return;

  if (!kDirect) {
#pragma unroll
    for (int i = 0; i < 16; ++i) s[i] = *reinterpret_cast<const float4*>(sbase + i * kD);
  }

  for (int t = t_begin; t < t_end; ++t) {
    const long long tb = ((long long)t * num_heads + head) * kD;
    const StepOut st = token_step<io_t, !kReplay>(s, r_ptr, w_ptr, k_ptr, v_ptr, a_ptr, b_ptr, bias_ptr, tb, head, row0, col0, scale);
    if (kReplay) {
      if (kg == 0) *reinterpret_cast<float4*>(sa_ptr + tb + col0) = make_float4(st.sa0, st.sa1, st.sa2, st.sa3);
      const int done = t - t_begin + 1;
      if (ckpt_ptr != nullptr && (done & 15) == 0 && t + 1 < t_end) {
        float* cbase = ckpt_ptr + (((long long)seq * 3 + (done >> 4) - 1) * num_heads + head) * (kD * kD) +
                       row0 * kD + col0;
#pragma unroll
        for (int i = 0; i < 16; ++i) *reinterpret_cast<float4*>(cbase + i * kD) = s[i];
      }
    } else if (kg == 0) {
      uint2 packed;
      packed.x = IO::pack(st.o0, st.o1);
      packed.y = IO::pack(st.o2, st.o3);
      *reinterpret_cast<uint2*>(y_ptr + tb + col0) = packed;
      if (y32_ptr != nullptr) {
        *reinterpret_cast<float4*>(y32_ptr + tb + col0) = make_float4(st.o0, st.o1, st.o2, st.o3);
      }
    }
  }

  if (!kReplay) {
#pragma unroll
    for (int i = 0; i < 16; ++i) *reinterpret_cast<float4*>(sbase + i * kD) = s[i];
  }
}

// ---------------------------------------------------------------------------------------------------------
// Decode kernel (every sequence has one token): persistent CTAs that stream the 16 KB state tiles through a
// shared-memory ring with bulk copies, so that loads and stores stay in flight independently of the arithmetic.
//   warp 0 (one lane)  : loader  - waits for a free stage, cp.async.bulk global -> shared, completion on full[stage]
//   warp 1 (one lane)  : storer  - waits for done[stage] (both halves updated), cp.async.bulk shared -> global,
//                                  and hands a stage back (empty[stage]) once its store has finished reading it
//   warps 2..15        : seven pairs of consumer warps (as many of them work as there are stages); a pair owns one
//                        stage at a time, one warp per half of a tile, and runs the same per-token step as the register
//                        kernel on float4s read from the staged tile(s)
// CTA b owns the units (kT adjacent heads of a sequence) b, b + gridDim.x, ...; its i-th unit uses stage i % kStages.
// ---------------------------------------------------------------------------------------------------------
// 2: six stages of two adjacent heads (32 KB bulk copies), 42.97 us per launch at 256 x 32 tiles;
// 1: thirteen stages of one tile (16 KB copies), 45.0 us.  Odd head counts always take 1.
constexpr int kDecodeTilesPerStage = 2;
constexpr int kTileBytes = kD * kD * 4;
constexpr int kTokBytes = 6 * kD * 2;  // r, w, k, v, a, b rows of one (token, head)
constexpr int kConsumerPairs = 7;
constexpr int kDecodeThreads = 32 * (2 + 2 * kConsumerPairs);

// A stage holds the state tiles of kT adjacent heads of one sequence (adjacent in the pool and in the token tensors) and
// their token rows: [kT x 16 KB tiles][6 vectors x kT x 128 B].  Bigger bulk copies amortise the per-copy latency of
// the copy pipeline; fewer stages remain for the same shared memory.
template <int kT>
struct RingCfg {
  static constexpr int kStages = 13 / kT;
  static constexpr int kStageBytes = kT * (kTileBytes + kTokBytes);
  static constexpr int kSmem = kStages * kStageBytes;
};

__device__ __forceinline__ void bulk_s2g(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(umma::smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* mbar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(umma::smem_u32(mbar)) : "memory");
}
__device__ __forceinline__ void lds16(const unsigned char* p, uint32_t (&w)[8]) {
  const uint4 lo = *reinterpret_cast<const uint4*>(p), hi = *reinterpret_cast<const uint4*>(p + 16);
  w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w;
  w[4] = hi.x; w[5] = hi.y; w[6] = hi.z; w[7] = hi.w;
}

// One token on a staged tile: same arithmetic as token_step, but the state stays in shared memory (read twice,
// written once) and the token vectors come from the stage's token area (vector j at tok + j * vstride bytes), so the
// consumer needs few registers and touches no global memory except for the output.
template <typename io_t>
__device__ __forceinline__ StepOut tile_step_smem(float* __restrict__ tbase, const unsigned char* __restrict__ tok,
                                                  int vstride, const io_t* __restrict__ bias_ptr, int head, int row0,
                                                  int col0, float scale) {
  using IO = Io16<io_t>;
  const int lane = threadIdx.x & 31;
  // retention of this lane group's 16 key rows: each of the 8 lanes that share the rows computes two of them and
  // the group exchanges them by shuffle (the transform is the expensive part of the step)
  float wv[16];
  {
    const int vq = lane & 7;
    float2 x = IO::unpack(*reinterpret_cast<const uint32_t*>(tok + 1 * vstride + (row0 + 2 * vq) * 2));
    if (bias_ptr != nullptr) {
      const float2 bx = IO::unpack(__ldg(reinterpret_cast<const uint32_t*>(bias_ptr + head * kD + row0 + 2 * vq)));
      x.x += bx.x;
      x.y += bx.y;
    }
    const float w_lo = retention(x.x), w_hi = retention(x.y);
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      wv[2 * p] = __shfl_sync(0xffffffffu, w_lo, (lane & 24) + p);
      wv[2 * p + 1] = __shfl_sync(0xffffffffu, w_hi, (lane & 24) + p);
    }
  }
  uint32_t rr[8], aa[8];
  lds16(tok + 0 * vstride + row0 * 2, rr);
  lds16(tok + 4 * vstride + row0 * 2, aa);
  const uint2 vraw = *reinterpret_cast<const uint2*>(tok + 3 * vstride + col0 * 2);
  float sa0 = 0.f, sa1 = 0.f, sa2 = 0.f, sa3 = 0.f, y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f, br = 0.f, kr = 0.f;
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const float2 a2 = IO::unpack(aa[p]), r2 = IO::unpack(rr[p]);
    const float2 b2 = IO::unpack(*reinterpret_cast<const uint32_t*>(tok + 5 * vstride + (row0 + 2 * p) * 2));
    const float2 k2 = IO::unpack(*reinterpret_cast<const uint32_t*>(tok + 2 * vstride + (row0 + 2 * p) * 2));
    br = fmaf(b2.x, r2.x, fmaf(b2.y, r2.y, br));
    kr = fmaf(k2.x, r2.x, fmaf(k2.y, r2.y, kr));
    const float4 q0 = *reinterpret_cast<const float4*>(tbase + (2 * p) * kD);
    const float4 q1 = *reinterpret_cast<const float4*>(tbase + (2 * p + 1) * kD);
    const float wr0 = wv[2 * p] * r2.x, wr1 = wv[2 * p + 1] * r2.y;
    sa0 = fmaf(a2.x, q0.x, fmaf(a2.y, q1.x, sa0)); sa1 = fmaf(a2.x, q0.y, fmaf(a2.y, q1.y, sa1));
    sa2 = fmaf(a2.x, q0.z, fmaf(a2.y, q1.z, sa2)); sa3 = fmaf(a2.x, q0.w, fmaf(a2.y, q1.w, sa3));
    y0 = fmaf(wr0, q0.x, fmaf(wr1, q1.x, y0)); y1 = fmaf(wr0, q0.y, fmaf(wr1, q1.y, y1));
    y2 = fmaf(wr0, q0.z, fmaf(wr1, q1.z, y2)); y3 = fmaf(wr0, q0.w, fmaf(wr1, q1.w, y3));
  }
#pragma unroll
  for (int m = 8; m <= 16; m <<= 1) {
    sa0 += __shfl_xor_sync(0xffffffffu, sa0, m); sa1 += __shfl_xor_sync(0xffffffffu, sa1, m);
    sa2 += __shfl_xor_sync(0xffffffffu, sa2, m); sa3 += __shfl_xor_sync(0xffffffffu, sa3, m);
    y0 += __shfl_xor_sync(0xffffffffu, y0, m); y1 += __shfl_xor_sync(0xffffffffu, y1, m);
    y2 += __shfl_xor_sync(0xffffffffu, y2, m); y3 += __shfl_xor_sync(0xffffffffu, y3, m);
    br += __shfl_xor_sync(0xffffffffu, br, m); kr += __shfl_xor_sync(0xffffffffu, kr, m);
  }
  const float2 v01 = IO::unpack(vraw.x), v23 = IO::unpack(vraw.y);
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const float2 b2 = IO::unpack(*reinterpret_cast<const uint32_t*>(tok + 5 * vstride + (row0 + 2 * p) * 2));
    const float2 k2 = IO::unpack(*reinterpret_cast<const uint32_t*>(tok + 2 * vstride + (row0 + 2 * p) * 2));
    float4 q0 = *reinterpret_cast<const float4*>(tbase + (2 * p) * kD);
    float4 q1 = *reinterpret_cast<const float4*>(tbase + (2 * p + 1) * kD);
    const float w0 = wv[2 * p], w1 = wv[2 * p + 1];
    q0.x = fmaf(w0, q0.x, fmaf(b2.x, sa0, k2.x * v01.x)); q0.y = fmaf(w0, q0.y, fmaf(b2.x, sa1, k2.x * v01.y));
    q0.z = fmaf(w0, q0.z, fmaf(b2.x, sa2, k2.x * v23.x)); q0.w = fmaf(w0, q0.w, fmaf(b2.x, sa3, k2.x * v23.y));
    q1.x = fmaf(w1, q1.x, fmaf(b2.y, sa0, k2.y * v01.x)); q1.y = fmaf(w1, q1.y, fmaf(b2.y, sa1, k2.y * v01.y));
    q1.z = fmaf(w1, q1.z, fmaf(b2.y, sa2, k2.y * v23.x)); q1.w = fmaf(w1, q1.w, fmaf(b2.y, sa3, k2.y * v23.y));
    *reinterpret_cast<float4*>(tbase + (2 * p) * kD) = q0;
    *reinterpret_cast<float4*>(tbase + (2 * p + 1) * kD) = q1;
  }
  StepOut out;
  out.sa0 = sa0; out.sa1 = sa1; out.sa2 = sa2; out.sa3 = sa3;
  out.o0 = scale * fmaf(kr, v01.x, fmaf(br, sa0, y0));
  out.o1 = scale * fmaf(kr, v01.y, fmaf(br, sa1, y1));
  out.o2 = scale * fmaf(kr, v23.x, fmaf(br, sa2, y2));
  out.o3 = scale * fmaf(kr, v23.y, fmaf(br, sa3, y3));
  return out;
}

template <typename io_t, int kT>
__global__ __launch_bounds__(kDecodeThreads, 1) void wkv7_decode_pipelined_kernel(
    const int* __restrict__ state_indices, const int* __restrict__ metadata_status, float* __restrict__ state_pool,
    const io_t* __restrict__ r_ptr, const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr,
    const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr, const io_t* __restrict__ b_ptr,
    const io_t* __restrict__ bias_ptr, io_t* __restrict__ y_ptr, float* __restrict__ y32_ptr, int num_units,
    int num_heads, long long output_elements, float scale, int reverse, int* __restrict__ error_flag) {
  using IO = Io16<io_t>;
  using R = RingCfg<kT>;
  constexpr int kStages = R::kStages, kStageBytes = R::kStageBytes;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full_bar[kStages], done_bar[kStages], empty_bar[kStages];
  const int units_per_seq = num_heads / kT;
  // i-th unit (kT adjacent heads of one sequence) of this CTA.  `reverse` walks the pool from the other end: a caller
  // that alternates it between consecutive decode steps finds the tiles it touched last (still in the 126 MB L2) first.
  const auto unit_of = [&](int i) {
    const int fwd = blockIdx.x + i * gridDim.x;
    return reverse ? num_units - 1 - fwd : fwd;
  };
  if (metadata_status != nullptr && metadata_status[0] != 0) {
    const io_t nan16 = IO::store(quiet_nan());
    for (long long i = (long long)blockIdx.x * kDecodeThreads + threadIdx.x; i < output_elements;
         i += (long long)gridDim.x * kDecodeThreads) {
      y_ptr[i] = nan16;
      if (y32_ptr != nullptr) y32_ptr[i] = quiet_nan();
    }
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      umma::mbar_init(&full_bar[i], 1);
      umma::mbar_init(&done_bar[i], 2);
      umma::mbar_init(&empty_bar[i], 1);
    }
    umma::mbar_fence_init();
  }
  __syncthreads();
  const int my_units = ((int)blockIdx.x < num_units) ? (num_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < my_units && ok; ++i) {
        const int st = i % kStages;
        if (i >= kStages) ok = umma::mbar_wait(&empty_bar[st], ((i / kStages) - 1) & 1);
        if (!ok) break;
        const int unit = unit_of(i);
        const int seq = unit / units_per_seq, head0 = kT * (unit % units_per_seq);
        const float* src = state_pool + ((long long)state_indices[seq] * num_heads + head0) * (kD * kD);
        const long long tb = ((long long)seq * num_heads + head0) * kD;  // one token per sequence: token == sequence
        unsigned char* stage = smem + st * kStageBytes;
        unsigned char* rows = stage + kT * kTileBytes;
        umma::mbar_expect_tx(&full_bar[st], kStageBytes);
        umma::bulk_g2s(stage, src, kT * kTileBytes, &full_bar[st]);
        umma::bulk_g2s(rows + 0 * kT * 128, r_ptr + tb, kT * 128, &full_bar[st]);
        umma::bulk_g2s(rows + 1 * kT * 128, w_ptr + tb, kT * 128, &full_bar[st]);
        umma::bulk_g2s(rows + 2 * kT * 128, k_ptr + tb, kT * 128, &full_bar[st]);
        umma::bulk_g2s(rows + 3 * kT * 128, v_ptr + tb, kT * 128, &full_bar[st]);
        umma::bulk_g2s(rows + 4 * kT * 128, a_ptr + tb, kT * 128, &full_bar[st]);
        umma::bulk_g2s(rows + 5 * kT * 128, b_ptr + tb, kT * 128, &full_bar[st]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int i = 0; i < my_units && ok; ++i) {
        const int st = i % kStages;
        ok = umma::mbar_wait(&done_bar[st], (i / kStages) & 1);
        if (!ok) break;
        const int unit = unit_of(i);
        const int seq = unit / units_per_seq, head0 = kT * (unit % units_per_seq);
        float* dst = state_pool + ((long long)state_indices[seq] * num_heads + head0) * (kD * kD);
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
    // A pair's first unit must use a stage in its first phase: a wait for the SECOND fill of a fresh barrier (parity 1)
    // returns at once.  So no more pairs work than there are stages.
    constexpr int kActivePairs = kStages < kConsumerPairs ? kStages : kConsumerPairs;
    for (int i = pair < kActivePairs ? pair : my_units; i < my_units && ok; i += kActivePairs) {
      const int st = i % kStages;
      const int unit = unit_of(i);
      const int seq = unit / units_per_seq, head0 = kT * (unit % units_per_seq);
      ok = umma::mbar_wait(&full_bar[st], (i / kStages) & 1);
      if (!ok) {
        // fail closed: this pair's remaining units read as NaN; it never reports them done, so the storer gives
        // up as well and their state tiles keep the values they had
        for (int j = i; j < my_units; j += kActivePairs) {
          const int u2 = unit_of(j);
          if (kg == 0)
            for (int t = 0; t < kT; ++t) {
              const long long tb = ((long long)(u2 / units_per_seq) * num_heads + kT * (u2 % units_per_seq) + t) * kD;
              const io_t nan16 = IO::store(quiet_nan());
              for (int e = 0; e < 4; ++e) {
                y_ptr[tb + col0 + e] = nan16;
                if (y32_ptr != nullptr) y32_ptr[tb + col0 + e] = quiet_nan();
              }
            }
        }
        break;
      }
      unsigned char* stage = smem + st * kStageBytes;
#pragma unroll 1
      for (int t = 0; t < kT; ++t) {
        const int head = head0 + t;
        const StepOut o = tile_step_smem<io_t>(reinterpret_cast<float*>(stage + t * kTileBytes) + row0 * kD + col0,
                                               stage + kT * kTileBytes + t * 128, kT * 128, bias_ptr, head, row0, col0,
                                               scale);
        if (kg == 0) {
          const long long tb = ((long long)seq * num_heads + head) * kD;
          uint2 packed;
          packed.x = IO::pack(o.o0, o.o1);
          packed.y = IO::pack(o.o2, o.o3);
          *reinterpret_cast<uint2*>(y_ptr + tb + col0) = packed;
          if (y32_ptr != nullptr) *reinterpret_cast<float4*>(y32_ptr + tb + col0) = make_float4(o.o0, o.o1, o.o2, o.o3);
        }
      }
      umma::fence_async_smem();  // the bulk store reads what this warp just wrote
      __syncwarp();
      if (lane == 0) mbar_arrive(&done_bar[st]);
    }
  }
  if (!ok && lane == 0 && error_flag != nullptr) atomicOr(error_flag, FRWKV_META_WAIT_TIMEOUT);
}

template <typename io_t>
int launch(const int* cu, const int* idx, const int* status, float* state, const void* r,
           const void* w, const void* k, const void* v, const void* a, const void* b,
           const void* bias, void* y, float* y32, int total_tokens, int num_sequences, int num_heads,
           float scale, bool direct, cudaStream_t stream) {
  const long long units = (long long)num_sequences * num_heads * 2;
  const long long blocks = (units + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (direct) {
    launch_chained(wkv7_recurrent_d64_kernel<io_t, false, true>, dim3((unsigned)blocks), dim3(kThreads), 0, stream,
        cu, idx, status, state, static_cast<const io_t*>(r), static_cast<const io_t*>(w),
        static_cast<const io_t*>(k), static_cast<const io_t*>(v), static_cast<const io_t*>(a),
        static_cast<const io_t*>(b), static_cast<const io_t*>(bias), static_cast<io_t*>(y), y32, nullptr, nullptr,
        units, num_heads, (long long)total_tokens * num_heads * kD, scale);
    return check_launch("wkv7_recurrent_d64_kernel<direct>");
  }
  launch_chained(wkv7_recurrent_d64_kernel<io_t, false>, dim3((unsigned)blocks), dim3(kThreads), 0, stream,
      cu, idx, status, state, static_cast<const io_t*>(r), static_cast<const io_t*>(w),
      static_cast<const io_t*>(k), static_cast<const io_t*>(v), static_cast<const io_t*>(a),
      static_cast<const io_t*>(b), static_cast<const io_t*>(bias), static_cast<io_t*>(y), y32, nullptr, nullptr,
      units, num_heads, (long long)total_tokens * num_heads * kD, scale);
  return check_launch("wkv7_recurrent_d64_kernel");
}

template <typename io_t>
int launch_decode(const int* idx, const int* status, float* state, const void* r, const void* w, const void* k,
                  const void* v, const void* a, const void* b, const void* bias, void* y, float* y32,
                  int num_sequences, int num_heads, float scale, int reverse, cudaStream_t stream) {
  // the SM count and the shared-memory opt-in are looked up once per device and kernel, not on every launch
  static int sm_counts[64] = {};
  static bool opted_in[64][2] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
    return fail(FRWKV_ERR_CUDA, "wkv7_recurrent: cannot identify the current device");
  if (sm_counts[device] == 0) cudaDeviceGetAttribute(&sm_counts[device], cudaDevAttrMultiProcessorCount, device);
  const int sm_count = sm_counts[device];
  const int tiles = num_sequences * num_heads;
#define FRWKV_DECODE(KT)                                                                                          \
  {                                                                                                               \
    if (!opted_in[device][KT - 1]) {                                                                              \
      cudaError_t e = cudaFuncSetAttribute(wkv7_decode_pipelined_kernel<io_t, KT>,                                \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, RingCfg<KT>::kSmem);      \
      if (e != cudaSuccess) return fail(FRWKV_ERR_CUDA, "wkv7_recurrent: %s", cudaGetErrorString(e));             \
      opted_in[device][KT - 1] = true;                                                                            \
    }                                                                                                             \
    const int units = tiles / KT;                                                                                 \
    const int grid = sm_count > 0 && sm_count < units ? sm_count : units;                                         \
    wkv7_decode_pipelined_kernel<io_t, KT><<<grid, kDecodeThreads, RingCfg<KT>::kSmem, stream>>>(                 \
        idx, status, state, static_cast<const io_t*>(r), static_cast<const io_t*>(w), static_cast<const io_t*>(k), \
        static_cast<const io_t*>(v), static_cast<const io_t*>(a), static_cast<const io_t*>(b),                    \
        static_cast<const io_t*>(bias), static_cast<io_t*>(y), y32, units, num_heads,                             \
        (long long)num_sequences * num_heads * kD, scale, reverse, const_cast<int*>(status));                     \
  }
  if (kDecodeTilesPerStage == 2 && num_heads % 2 == 0) FRWKV_DECODE(2) else FRWKV_DECODE(1)
#undef FRWKV_DECODE
  return check_launch("wkv7_decode_pipelined_kernel");
}

template <typename io_t>
int launch_replay(const int* chunk_starts, const int* chunk_ends, const float* boundary, const void* r, const void* w,
                  const void* k, const void* v, const void* a, const void* b, const void* bias, float* sa, float* ckpt,
                  int num_chunks, int num_heads, cudaStream_t stream) {
  const long long units = (long long)num_chunks * num_heads * 2;
  const long long blocks = (units + kWarpsPerBlock - 1) / kWarpsPerBlock;
  wkv7_recurrent_d64_kernel<io_t, true><<<(unsigned)blocks, kThreads, 0, stream>>>(
      chunk_starts, chunk_ends, nullptr, const_cast<float*>(boundary), static_cast<const io_t*>(r),
      static_cast<const io_t*>(w), static_cast<const io_t*>(k), static_cast<const io_t*>(v),
      static_cast<const io_t*>(a), static_cast<const io_t*>(b), static_cast<const io_t*>(bias), nullptr, nullptr, sa,
      ckpt, units, num_heads, 0, 1.0f);
  return check_launch("wkv7_recurrent_d64_kernel<replay>");
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_wkv7_recurrent_fp32io16_forward_varlen(
    const int32_t* cu_seqlens, const int32_t* state_indices, const int32_t* metadata_status,
    float* state_pool, const void* r, const void* decay_logits, const void* k, const void* v,
    const void* a, const void* b, const void* decay_bias, void* y, float* y_fp32,
    int total_tokens, int num_sequences, int num_heads, int head_size, int max_seqlen,
    int io_dtype, float scale, frwkv_stream_t stream) {
  return frwkv_wkv7_recurrent_fp32io16_forward_varlen_ex(cu_seqlens, state_indices, metadata_status, state_pool, r,
                                                         decay_logits, k, v, a, b, decay_bias, y, y_fp32, total_tokens,
                                                         num_sequences, num_heads, head_size, max_seqlen, io_dtype,
                                                         scale, 0, stream);
}

extern "C" int frwkv_wkv7_recurrent_fp32io16_forward_varlen_ex(
    const int32_t* cu_seqlens, const int32_t* state_indices, const int32_t* metadata_status,
    float* state_pool, const void* r, const void* decay_logits, const void* k, const void* v,
    const void* a, const void* b, const void* decay_bias, void* y, float* y_fp32,
    int total_tokens, int num_sequences, int num_heads, int head_size, int max_seqlen,
    int io_dtype, float scale, int flags, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(cu_seqlens && state_indices && state_pool && r && decay_logits && k && v && a && b && y,
                "wkv7_recurrent: null pointer argument");
  FRWKV_REQUIRE(total_tokens > 0 && num_heads > 0, "wkv7_recurrent: sizes must be positive");
  FRWKV_REQUIRE(num_sequences > 0 && num_sequences <= 65535,
                "wkv7_recurrent: state_indices must contain 1..65535 sequences");
  if (head_size == 128 || head_size == 256)  // the general kernel; the tuned ones below are for head size 64
    return launch_recurrent_wide(cu_seqlens, state_indices, metadata_status, nullptr, state_pool, r, decay_logits, k, v, a, b,
                                 decay_bias, y, y_fp32, total_tokens, num_sequences, num_heads, head_size, io_dtype,
                                 scale, reinterpret_cast<cudaStream_t>(stream));
  if (head_size != 64) {
    return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_recurrent: head size must be 64, 128, or 256, got %d", head_size);
  }
  const long long blocks = ((long long)num_sequences * num_heads * 2 + 3) / 4;
  FRWKV_REQUIRE(blocks <= 0x7fffffffLL, "wkv7_recurrent: too many (sequence, head) pairs");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // decode (one token per sequence, known from the caller's validated metadata) with enough tiles to keep a
  // persistent grid busy takes the bulk-copy pipelined kernel; everything else the register kernel
  const bool decode = max_seqlen == 1 && total_tokens == num_sequences &&
                      (long long)num_sequences * num_heads >= kRingMinTiles && (long long)num_sequences * num_heads <= 0x7fffffffLL;
  if (decode && io_dtype == FRWKV_DTYPE_BF16)
    return launch_decode<__nv_bfloat16>(state_indices, metadata_status, state_pool, r, decay_logits, k, v, a, b,
                                        decay_bias, y, y_fp32, num_sequences, num_heads, scale, flags & 1, s);
  if (decode && io_dtype == FRWKV_DTYPE_FP16)
    return launch_decode<__half>(state_indices, metadata_status, state_pool, r, decay_logits, k, v, a, b, decay_bias,
                                 y, y_fp32, num_sequences, num_heads, scale, flags & 1, s);
  // one token per sequence, sequence i in slot i, on the caller's word: the register kernel reads neither table
  const bool direct = (flags & FRWKV_RECURRENT_DIRECT_SLOTS) != 0 && max_seqlen == 1 && total_tokens == num_sequences;
  if (io_dtype == FRWKV_DTYPE_BF16) {
    return launch<__nv_bfloat16>(cu_seqlens, state_indices, metadata_status, state_pool, r, decay_logits, k,
                                 v, a, b, decay_bias, y, y_fp32, total_tokens, num_sequences, num_heads,
                                 scale, direct, s);
  }
  if (io_dtype == FRWKV_DTYPE_FP16) {
    return launch<__half>(cu_seqlens, state_indices, metadata_status, state_pool, r, decay_logits, k, v, a,
                          b, decay_bias, y, y_fp32, total_tokens, num_sequences, num_heads, scale, direct, s);
  }
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_recurrent: token tensors must be float16 or bfloat16");
}

extern "C" int frwkv_wkv7_chunk_replay(const int32_t* chunk_starts, const int32_t* chunk_ends, const float* boundary,
                                       const void* r, const void* decay_logits, const void* k, const void* v,
                                       const void* a, const void* b, const void* decay_bias, float* state_dot_a,
                                       float* checkpoints, int num_chunks, int num_heads, int head_size, int io_dtype,
                                       frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(chunk_starts && chunk_ends && boundary && r && decay_logits && k && v && a && b && state_dot_a,
                "wkv7_chunk_replay: null pointer argument");
  FRWKV_REQUIRE(num_chunks > 0 && num_heads > 0, "wkv7_chunk_replay: sizes must be positive");
  if (head_size != 64) return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_chunk_replay: head size %d is not built (only 64)", head_size);
  FRWKV_REQUIRE(((long long)num_chunks * num_heads * 2 + 3) / 4 <= 0x7fffffffLL, "wkv7_chunk_replay: too many chunks");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_replay<__nv_bfloat16>(chunk_starts, chunk_ends, boundary, r, decay_logits, k, v, a, b, decay_bias,
                                        state_dot_a, checkpoints, num_chunks, num_heads, s);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_replay<__half>(chunk_starts, chunk_ends, boundary, r, decay_logits, k, v, a, b, decay_bias,
                                 state_dot_a, checkpoints, num_chunks, num_heads, s);
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_chunk_replay: token tensors must be float16 or bfloat16");
}
