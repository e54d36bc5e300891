// Chunked WKV7 forward as ONE kernel: a CTA owns a (sequence, head) pair, keeps its fp32 state on chip and walks
// the sequence's chunks (<= 64 tokens, head size 64) in order.  Nothing but the token rows, the outputs and the
// optional per-chunk boundary states / state_dot_a rows touches HBM: no per-chunk workspace.
//
// Per chunk with start state S0 (K x V), tokens t = 0..L-1, cumulative decay g_t = prod_{s<=t} w_s (g_{-1} = 1):
//     A~ = a*g_{t-1}   R~ = r*g_t   B~ = b/g_t   K~ = k/g_t   B^ = B~*g_L   K^ = K~*g_L              (L x K)
//     [A_ab | A_ak ; A_rb | A_rk] = [A~ ; R~] [B~ ; K~]^T, masked (strictly lower for A_a*, lower for A_r*)
//     X  = A~ S0 + A_ak V          U = (I - A_ab)^-1 X   (rows u_t = S_{t-1}^T a_t, the reference's state_dot_a)
//     Y  = scale * (R~ S0 + A_rk V + A_rb U)
//     S' = diag(g_L) (S0 + B~^T U + K~^T V)
//
// Tensor memory carries the operands from one product to the next (row i of a matrix = lane i):
//     XA  (64 columns)  lanes 0..63 A~, lanes 64..127 R~            written with tcgen05.st, operand A of MMA 1 and 2
//     D1  (128 columns) result of MMA 1; masked and rounded in place; the A_ab block (needed only by the solve, which
//                       reads it from shared memory) is replaced by B~^T, after MMA 2 the A_ak block by K~^T and the
//                       A_rk block by zeros, so that D1 as a whole is operand A of MMA 3:
//                       [B~^T | K~^T ; A_rb | 0] [U ; V].  B~^T and K~^T are columns of the [B~;K~] tile read back
//                       from shared memory by the thread that owns the lane.
//     DA  (64 columns)  MMA 2: XA S0 + D1[:,64:128] V  = [X ; R~ S0 + A_rk V]
//     DC  (= XA's columns, free by then)  MMA 3:  [B~^T U + K~^T V ; A_rb U]
// All products are tcgen05.mma kind::tf32 with fp32 accumulation; operands are rounded to tf32 (nearest) once.  The
// B operands contract over tokens or keys that their producers own as rows, so they are written transposed with
// 4-byte stores into 64-row tiles whose chunk stride (1040 bytes) keeps those stores free of bank conflicts.  The
// unit-triangular system (I - A_ab) U = X is solved in fp32 on the CUDA cores by blocked forward substitution (one
// thread per value column and block of 16 tokens); the inverse is never formed.  The state stays in fp32 registers;
// only its rounded copy is an operand.
//
// 256 threads, 105 KB of shared memory and 256 tensor-memory columns per CTA: two CTAs share an SM, so one CTA's
// barrier-separated phases overlap the other's.  The loop body is kept small on purpose (rolled loops, 16-column
// tensor-memory transfers): a first version whose body was 170 KB of unrolled code ran five times slower, bound by
// instruction fetch.
//
// Replaces the same reference kernels as wkv7_chunk_fwd.cu (which remains the path for batches with too few
// (sequence, head) pairs to fill the GPU this way): csrc/sm120/tmix/wkv7/infer_chunk_bf16_forward_varlen.cu:42-266,
// csrc/sm90/rl_infctx/wkv7/rl_infctx_chunk_fp32io16_forward.cu:317-538, and the forward halves of
// csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_forward.cu:32-130 (boundary and state_dot_a outputs).

#include "wkv7_chunk_common.cuh"

namespace frwkv {
namespace {

using namespace chunk;

constexpr int kL = 64;
constexpr int kD = 64;
constexpr int kThreads = 256;
constexpr uint32_t kCSB = 2064;   // chunk stride of [B~;K~]  (128 rows, written row-wise, read back column-wise)
constexpr uint32_t kCS64 = 1040;  // ... of the 64-row transposed tiles and of g

constexpr uint32_t kOffG = 0;                        // g[t][k], chunk-major, 16 x 1040
constexpr uint32_t kOffX2 = kOffG + 16 * kCS64;      // [B~;K~], later X^T -> U^T (fp32, 64-row tile) during the solve
constexpr uint32_t kOffUV = kOffX2 + 16 * kCSB;      // [U^T | V^T]: 32 chunks x 1040; the U half first holds A_ab^T
constexpr uint32_t kOffS = kOffUV + 32 * kCS64;      // S0^T
constexpr uint32_t kOffW = kOffS + 16 * kCS64;       // the chunk's decay logits as they are in HBM: [64][64] 16-bit
constexpr uint32_t kFusedSmem = kOffW + kL * kD * 2; // 107,776 bytes
static_assert(kOffX2 % 128 == 0 && kOffUV % 128 == 0 && kOffS % 128 == 0 && kOffW % 128 == 0,
              "tile bases must stay 128-byte aligned");
static_assert(64 * 256 <= 16 * kCS64, "the A_ab scratch must fit the U half");
// The token rows of the next chunk are staged as they are in HBM over the [B~;K~] and [U^T|V^T] tiles, which are
// free between a chunk's last product and the next chunk's operand phase: five tiles of 64 rows, rows padded by 16
// bytes so that the threads of a warp, which read consecutive rows, hit different banks.
constexpr uint32_t kRawRow16 = 144;
constexpr uint32_t kRawA = kOffX2, kRawR = kRawA + 64 * kRawRow16, kRawB = kRawR + 64 * kRawRow16,
                   kRawV = kRawB + 64 * kRawRow16, kRawK = kRawV + 64 * kRawRow16;
static_assert(kRawK + 64 * kRawRow16 <= kOffS, "the staged rows must fit the two free tiles");
static_assert(2 * (kFusedSmem + 1024) <= 233472, "two CTAs must fit one SM");

constexpr uint32_t kColXA = 0, kColD1 = 64, kColDA = 192, kColDC = 0, kTmemCols = 256;

// kAdj = false: the forward recurrence.  kAdj = true: the same kernel walks every sequence BACKWARDS (last chunk
// first, last token of a chunk first) and makes its key rows itself: this is how the backward pass gets the adjoint of
// the state at every chunk boundary, because that adjoint obeys a recurrence of the same form
//     G_{t-1} = diag(w_t) G_t + a_t (G_t^T b_t)^T + k^_t dy_t^T,      k^_t = scale (w_t * r_t + (b_t . r_t) a_t)
// (the forward one with a and b exchanged, k^ for k, dy for v, run in reverse time).  The launcher passes b as a,
// a as b and dy as v; k^ comes from the staged r, a and b rows and the decay w_t = g_t / g_{t-1}; outputs y /
// state_dot_a are not produced, `boundary[c]` receives the adjoint that enters chunk c from the future and the state
// slot ends as the gradient of the initial state.
template <typename io_t, bool kAdj>
__global__ __launch_bounds__(kThreads, 2) void wkv7_chunk_fused_kernel(
    const int* __restrict__ seq_chunk_offsets, const int* __restrict__ chunk_starts, const int* __restrict__ chunk_ends,
    const int* __restrict__ state_indices, const int* __restrict__ metadata_status, float* __restrict__ state_pool,
    const io_t* __restrict__ r_ptr, const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr,
    const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr, const io_t* __restrict__ b_ptr,
    const io_t* __restrict__ bias_ptr, io_t* __restrict__ y_ptr,
    float* __restrict__ y32_ptr, float* __restrict__ boundary, float* __restrict__ sda_ptr, int num_heads,
    int num_units, long long output_elements, float scale, int* __restrict__ error_flag) {
  using IO = Io16<io_t>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t mbar[3];
  __shared__ uint32_t tmem_holder;
  __shared__ float seg_total[4][64];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (metadata_status != nullptr && metadata_status[0] != 0) {
    const io_t nan16 = IO::store(quiet_nan());
    for (long long i = (long long)blockIdx.x * kThreads + tid; y_ptr != nullptr && i < output_elements;
         i += (long long)gridDim.x * kThreads) {
      y_ptr[i] = nan16;
      if (y32_ptr != nullptr) y32_ptr[i] = quiet_nan();
    }
    return;
  }
  const int m = 32 * (warp & 3) + lane;  // tensor-memory lane / operand row of this thread
  const int half = warp >> 2;            // which 32 of 64 columns (64 of 128) this thread handles
  const int mt = m & 63;                 // token (or key channel) of that row
  const bool low = m < 64;               // lanes 0..63: A~ / B~ rows, later key rows; lanes 64..127: R~ / K~ / V, Y rows
  const int c0 = 32 * half;
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 3; ++i) umma::mbar_init(&mbar[i], 1);
    umma::mbar_fence_init();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_holder, kTmemCols);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_holder;
  const uint32_t sbase = umma::smem_u32(smem);
  const uint32_t lane_base = uint32_t(32 * (warp & 3)) << 16;
  const uint32_t idesc128 = umma::idesc_tf32(128, 128), idesc64 = umma::idesc_tf32(128, 64);
  const long long row_stride = (long long)num_heads * kD;
  bool ok = true;
  uint32_t parity = 0;

  // packed row of the i-th token a chunk [tt0, tt0 + ln) is walked in
  const auto token_row = [](int tt0, int ln, int i) { return kAdj ? tt0 + ln - 1 - i : tt0 + i; };

  // the decay logits of a chunk travel by cp.async one chunk ahead (two 16-byte pieces per thread; rows past the
  // end of a short chunk are zero-filled and not used)
  auto stage_w = [&](int chunk, long long head_off) {
    const int tt0 = chunk_starts[chunk];
    const int ln = min(max(chunk_ends[chunk] - tt0, 1), kL);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int piece = tid + i * kThreads, rowi = piece >> 3, part = piece & 7;
      umma::cp_async16(sbase + kOffW + piece * 16,
                       w_ptr + (long long)token_row(tt0, ln, min(rowi, ln - 1)) * row_stride + head_off + 8 * part,
                       rowi < ln ? 16u : 0u);
    }
    umma::cp_async_commit();
  };

  // The a, r, b, k and v rows of a chunk, copied as 16-byte pieces with eight consecutive lanes per row: whole 128-byte
  // lines per request.  Read straight into registers by the thread that owns
  // a row, the same rows cost a tag lookup per lane and request, which made the loads the longest stall of a chunk.
  auto stage_rows = [&](int tt0, int ln, long long head_off) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int piece = tid + i * kThreads, which = piece >> 9, rowi = (piece >> 3) & 63, part = piece & 7;
      const io_t* base = which == 0 ? a_ptr : which == 1 ? r_ptr : which == 2 ? b_ptr : v_ptr;
      umma::cp_async16(sbase + kRawA + which * (64 * kRawRow16) + rowi * kRawRow16 + part * 16,
                       base + (long long)token_row(tt0, ln, min(rowi, ln - 1)) * row_stride + head_off + 8 * part,
                       rowi < ln ? 16u : 0u);
    }
    if (!kAdj) {  // the adjoint run makes its key rows from the r, a and b rows
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int piece = tid + i * kThreads, rowi = piece >> 3, part = piece & 7;
        umma::cp_async16(sbase + kRawK + rowi * kRawRow16 + part * 16,
                         k_ptr + (long long)token_row(tt0, ln, min(rowi, ln - 1)) * row_stride + head_off + 8 * part,
                         rowi < ln ? 16u : 0u);
      }
    }
    umma::cp_async_commit();
  };

  // g[t][k] of a chunk: (1) thread (token, 16 channels): retention of the staged logits, row-wise into the g tile;
  // (2) thread (key channel, 16-token segment): running product down the column, segment totals, prefix fix-up.
  // Runs one chunk ahead of its use (while the tensor core does MMA 1 of the previous chunk) and starts the copy of
  // the logits of the chunk after.  Contains barriers: every thread calls it.
  auto compute_g = [&](int chunk, int chunk_after, long long head_off) {  // chunk_after < 0: none
    const int ln = min(max(chunk_ends[chunk] - chunk_starts[chunk], 1), kL);
    umma::cp_async_wait_all();
    __syncthreads();
    {
      const int t = tid >> 2, q = tid & 3;
      float x[16];
      unpack8<io_t>(*reinterpret_cast<const uint4*>(smem + kOffW + t * 128 + q * 32), *reinterpret_cast<float(*)[8]>(&x[0]));
      unpack8<io_t>(*reinterpret_cast<const uint4*>(smem + kOffW + t * 128 + q * 32 + 16), *reinterpret_cast<float(*)[8]>(&x[8]));
      if (bias_ptr != nullptr) {
        float bz[16];
        unpack8<io_t>(__ldg(reinterpret_cast<const uint4*>(bias_ptr + head_off + 16 * q)), *reinterpret_cast<float(*)[8]>(&bz[0]));
        unpack8<io_t>(__ldg(reinterpret_cast<const uint4*>(bias_ptr + head_off + 16 * q + 8)), *reinterpret_cast<float(*)[8]>(&bz[8]));
#pragma unroll
        for (int e = 0; e < 16; ++e) x[e] += bz[e];
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) x[e] = t < ln ? retention(x[e]) : 1.f;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        st4(smem, kOffG + (4 * q + i) * kCS64 + t * 16, make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]));
    }
    __syncthreads();
    if (chunk_after >= 0) stage_w(chunk_after, head_off);  // everybody has read this chunk's logits
    {
      const int kcol = tid & 63, seg = tid >> 6;
      const uint32_t gcol = kOffG + uint32_t(kcol >> 2) * kCS64 + uint32_t(kcol & 3) * 4 + uint32_t(16 * seg) * 16;
      float pr[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) pr[i] = ld1(smem, gcol + i * 16);
#pragma unroll
      for (int i = 1; i < 16; ++i) pr[i] *= pr[i - 1];
      seg_total[seg][kcol] = pr[15];
      __syncthreads();
      float mult = 1.f;
      if (seg > 0) mult = seg_total[0][kcol];
      if (seg > 1) mult *= seg_total[1][kcol];
      if (seg > 2) mult *= seg_total[2][kcol];
#pragma unroll
      for (int i = 0; i < 16; ++i) st1(smem, gcol + i * 16, pr[i] * mult);
    }
    __syncthreads();
  };

  for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
    const int seq = unit / num_heads, head = unit % num_heads;
    const int c_begin = seq_chunk_offsets[seq], c_end = seq_chunk_offsets[seq + 1];
    if (c_begin >= c_end) continue;
    const int slot = state_indices != nullptr ? state_indices[seq] : seq;
    float* state = state_pool + ((long long)slot * num_heads + head) * (kD * kD);
    const long long head_off = (long long)head * kD;
    const int n_chunks = c_end - c_begin, c_step = kAdj ? -1 : 1, c_first = kAdj ? c_end - 1 : c_begin;
    stage_w(c_first, head_off);
    {
      const int ft0 = chunk_starts[c_first];
      stage_rows(ft0, min(max(chunk_ends[c_first] - ft0, 1), kL), head_off);
    }

    // ---- this unit's state: row mt, columns c0..c0+31 in registers (fp32) and, transposed and rounded, in S0^T ----
    float S[32];
    if (low) {
      float* bnd = boundary != nullptr ? boundary + ((long long)c_first * num_heads + head) * (kD * kD) + mt * kD + c0
                                       : nullptr;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 s = *reinterpret_cast<const float4*>(state + mt * kD + c0 + j);
        if (bnd != nullptr) *reinterpret_cast<float4*>(bnd + j) = s;
        S[j] = s.x; S[j + 1] = s.y; S[j + 2] = s.z; S[j + 3] = s.w;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) st1(smem, kOffS + tile_off(kCS64, c0 + j, mt), umma::to_tf32(S[j]));
    }
    compute_g(c_first, n_chunks > 1 ? c_first + c_step : -1, head_off);

    int next_t0 = chunk_starts[c_first], next_end = chunk_ends[c_first];
    for (int nc = 0; nc < n_chunks; ++nc, parity ^= 1u) {
      const int c = c_first + nc * c_step;
      const bool has_next = nc + 1 < n_chunks;
      const int t0 = next_t0;
      const int len = min(max(next_end - t0, 1), kL);
      if (has_next) {  // the next chunk's bounds are on their way while this one is worked on
        next_t0 = chunk_starts[c + c_step];
        next_end = chunk_ends[c + c_step];
      }
      // ---- this thread's operand rows, from the staged tiles (rows past the end of a short chunk were zero-filled) --
      const bool valid = mt < len;
      uint4 praw[4], qraw[4], vraw[4];
      float b_dot_r = 0.f;  // adjoint run, lanes 64..127: (b_t . r_t) over the row's 64 channels
      umma::cp_async_wait_all();
      __syncthreads();
      {
        const uint32_t rp = (low ? kRawA : kRawR) + mt * kRawRow16 + c0 * 2;
        // q rows: b for lanes 0..63; k for lanes 64..127, or in the adjoint run the row of the a operand again, from
        // which (with r) the modified key is made
        const uint32_t rq = (low || kAdj ? kRawB : kRawK) + mt * kRawRow16 + c0 * 2;
        const uint32_t rv = kRawV + mt * kRawRow16 + c0 * 2;
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          praw[i] = *reinterpret_cast<const uint4*>(smem + rp + 16 * i);
          qraw[i] = *reinterpret_cast<const uint4*>(smem + rq + 16 * i);
          vraw[i] = !low ? *reinterpret_cast<const uint4*>(smem + rv + 16 * i) : zero;
        }
        if (kAdj && !low) {
          // the launcher passed the true b as this kernel's a operand: its staged tile times the r tile, whole rows
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float bf[8], rf[8];
            unpack8<io_t>(*reinterpret_cast<const uint4*>(smem + kRawA + mt * kRawRow16 + 16 * i), bf);
            unpack8<io_t>(*reinterpret_cast<const uint4*>(smem + kRawR + mt * kRawRow16 + 16 * i), rf);
#pragma unroll
            for (int e = 0; e < 8; ++e) b_dot_r = fmaf(bf[e], rf[e], b_dot_r);
          }
        }
      }
      __syncthreads();  // the staged tiles have been read: the operand tiles may go over them

      // ---- operands: XA -> tensor memory, [B~;K~] and V^T -> shared memory -------------------------------------
      const float g_last = low ? ld1(smem, kOffG + tile_off(kCS64, 63, mt)) : 0.f;  // g_L of key row mt
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float pf[8], qf[8];
        unpack8<io_t>(praw[i], pf);
        unpack8<io_t>(qraw[i], qf);
        uint32_t xa[8];
#pragma unroll
        for (int hq = 0; hq < 2; ++hq) {
          const int kc = (c0 >> 2) + 2 * i + hq;  // 16-byte column chunk of g / of the tiles
          const float4 g = ld4(smem, kOffG + kc * kCS64 + mt * 16);
          float4 sc = g;                          // R~ = r * g_t
          if (low) sc = mt > 0 ? ld4(smem, kOffG + kc * kCS64 + (mt - 1) * 16) : make_float4(1.f, 1.f, 1.f, 1.f);
          const int e = 4 * hq;
          if (kAdj && !low) {
            // the adjoint run's key k^ = scale (w r + (b . r) a), with w_t = g_t / g_{t-1}; qf holds the a channels
            const float4 gp = mt > 0 ? ld4(smem, kOffG + kc * kCS64 + (mt - 1) * 16) : make_float4(1.f, 1.f, 1.f, 1.f);
            qf[e + 0] = scale * fmaf(b_dot_r, qf[e + 0], g.x * rcp_approx(gp.x) * pf[e + 0]);
            qf[e + 1] = scale * fmaf(b_dot_r, qf[e + 1], g.y * rcp_approx(gp.y) * pf[e + 1]);
            qf[e + 2] = scale * fmaf(b_dot_r, qf[e + 2], g.z * rcp_approx(gp.z) * pf[e + 2]);
            qf[e + 3] = scale * fmaf(b_dot_r, qf[e + 3], g.w * rcp_approx(gp.w) * pf[e + 3]);
          }
          // products in pairs (mul.rn.f32x2: two per instruction, the scalar bits)
          const float2 p01 = __fmul2_rn(make_float2(pf[e + 0], pf[e + 1]), make_float2(sc.x, sc.y));
          const float2 p23 = __fmul2_rn(make_float2(pf[e + 2], pf[e + 3]), make_float2(sc.z, sc.w));
          xa[e + 0] = tf32_bits(p01.x);  // rows past the end of a short chunk were loaded as zeros
          xa[e + 1] = tf32_bits(p01.y);
          xa[e + 2] = tf32_bits(p23.x);
          xa[e + 3] = tf32_bits(p23.y);
          const float2 q01 = __fmul2_rn(make_float2(qf[e + 0], qf[e + 1]), make_float2(rcp_approx(g.x), rcp_approx(g.y)));
          const float2 q23 = __fmul2_rn(make_float2(qf[e + 2], qf[e + 3]), make_float2(rcp_approx(g.z), rcp_approx(g.w)));
          st4(smem, kOffX2 + kc * kCSB + m * 16, umma::to_tf32(make_float4(q01.x, q01.y, q23.x, q23.y)));
        }
        umma::tmem_st8(tmem + kColXA + lane_base + c0 + 8 * i, xa);
        if (!low) {
          float vf[8];
          unpack8<io_t>(vraw[i], vf);
          const uint32_t o = kOffUV + uint32_t(16 + (mt >> 2)) * kCS64 + uint32_t(mt & 3) * 4 + (c0 + 8 * i) * 16;
#pragma unroll
          for (int e = 0; e < 8; ++e) st1(smem, o + e * 16, vf[e]);
        }
      }
      umma::tmem_st_wait();
      // pull the next chunk's operand rows into L2 (its decay logits are already on their way to shared memory)
      if (has_next) {
        const int nt0 = next_t0, nlen = next_end - nt0;
        for (int e = tid; e < 5 * kL; e += kThreads) {
          const int which = e >> 6, rowi = e & 63;
          if (rowi < nlen) {
            const io_t* base = which == 0 ? a_ptr : which == 1 ? r_ptr : which == 2 ? b_ptr : which == 3 ? k_ptr : v_ptr;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(base + (long long)(nt0 + rowi) * row_stride + head_off));
          }
        }
      }
      umma::fence_async_smem();
      umma::fence_before_sync();
      __syncthreads();
      umma::fence_after_sync();

      // ---- MMA 1: D1 = XA [B~;K~]^T ------------------------------------------------------------------------------
      if (tid == 0) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_tf32_ts(tmem + kColD1, tmem + kColXA + 8 * ks,
                            umma::desc_k_major(sbase + kOffX2 + ks * 2 * kCSB, kCSB), idesc128, ks > 0 ? 1u : 0u);
        umma::mma_commit(&mbar[0]);
      }
      if (has_next)  // g of this chunk has been consumed (barrier above)
        compute_g(c + c_step, nc + 2 < n_chunks ? c + 2 * c_step : -1, head_off);
      ok = wait_warp(&mbar[0], parity, ok);
      umma::fence_after_sync();
      // ---- epilogue 1: mask; A_ab -> fp32 scratch, the other three blocks rounded in place -----------------------
      if (ok) {
        const int limit = low ? mt : mt + 1;  // keep s < t (strict) or s <= t
#pragma unroll 1
        for (int hb = 0; hb < 4; ++hb) {
          uint32_t u[16];
          const uint32_t taddr = tmem + kColD1 + lane_base + 64 * half + 16 * hb;
          umma::tmem_ld16(taddr, u);
          umma::tmem_ld_wait();
          const int s0 = 16 * hb;
          if (low && half == 0) {
            // A_ab^T: element [s][t] at 256 s + 4 t bytes (the lanes of a warp are consecutive t: consecutive words)
#pragma unroll
            for (int j = 0; j < 16; ++j)
              st1(smem, kOffUV + uint32_t(s0 + j) * 256 + uint32_t(mt) * 4, s0 + j < limit ? __uint_as_float(u[j]) : 0.f);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) u[j] = s0 + j < limit ? tf32_bits(__uint_as_float(u[j])) : 0u;
            umma::tmem_st16(taddr, u);
          }
        }
        umma::tmem_st_wait();
      }
      umma::fence_before_sync();
      __syncthreads();
      umma::fence_after_sync();

      // ---- MMA 2: DA = XA S0 + D1[:,64:128] V ------------------------------------------------------------------
      if (tid == 0) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_tf32_ts(tmem + kColDA, tmem + kColXA + 8 * ks,
                            umma::desc_k_major(sbase + kOffS + ks * 2 * kCS64, kCS64), idesc64, ks > 0 ? 1u : 0u);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma::mma_tf32_ts(tmem + kColDA, tmem + kColD1 + 64 + 8 * ks,
                            umma::desc_k_major(sbase + kOffUV + (16 + 2 * ks) * kCS64, kCS64), idesc64, 1u);
        umma::mma_commit(&mbar[1]);
      }
      // Meanwhile the key rows of MMA 3's operand: lane k gets column k of the [B~;K~] tile.  B~^T goes over the A_ab
      // block at once (every reader of that block passed the barrier above); K~^T waits in registers for MMA 2,
      // which still reads the A_ak block it will replace.
      uint32_t kt[32];
      if (low) {
        const uint32_t colk = kOffX2 + uint32_t(mt >> 2) * kCSB + uint32_t(mt & 3) * 4;
#pragma unroll 1
        for (int hb = 0; hb < 2; ++hb) {
          uint32_t bt[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) bt[j] = __float_as_uint(ld1(smem, colk + (c0 + 16 * hb + j) * 16));
          umma::tmem_st16(tmem + kColD1 + lane_base + c0 + 16 * hb, bt);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) kt[j] = __float_as_uint(ld1(smem, colk + (64 + c0 + j) * 16));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) kt[j] = 0u;  // lanes 64..127: zeros over A_rk (A_rk V is already part of DA)
      }
      ok = wait_warp(&mbar[1], parity, ok);
      umma::fence_after_sync();
      umma::tmem_st32(tmem + kColD1 + 64 + lane_base + c0, kt);
      umma::tmem_st_wait();
      umma::fence_before_sync();
      __syncthreads();  // the [B~;K~] tile has been read: X^T may go over it
      // ---- epilogue 2: X^T (fp32, unrounded) -> shared memory, over the [B~;K~] tile --------------------------------
      umma::fence_after_sync();
      if (ok && low) {
#pragma unroll 1
        for (int hb = 0; hb < 2; ++hb) {
          uint32_t u[16];
          umma::tmem_ld16(tmem + kColDA + lane_base + c0 + 16 * hb, u);
          umma::tmem_ld_wait();
          const uint32_t o = kOffX2 + uint32_t(mt >> 2) * kCS64 + uint32_t(mt & 3) * 4 + (c0 + 16 * hb) * 16;
#pragma unroll
          for (int j = 0; j < 16; ++j) st1(smem, o + j * 16, __uint_as_float(u[j]));
        }
      }
      __syncthreads();
      // ---- U = (I - A_ab)^-1 X by blocked forward substitution in fp32, U_t = X_t + sum_{s < t} A_ab[t][s] U_s.
      //      Thread (value column v, block j) holds rows 16 j .. 16 j + 15 of column v.  From the first block to the
      //      last: the owners of block jb finish it (a 16 x 16 triangular solve in registers) and publish it; the owners
      //      of later blocks fold it in (a 16 x 16 update).  T = (I - A_ab)^-1 is never formed. ---------------------------
      {
        const int v = tid & 63, j = tid >> 6;
        float x[16];
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {
          const float4 q = ld4(smem, kOffX2 + (4 * j + c4) * kCS64 + v * 16);
          x[4 * c4] = q.x; x[4 * c4 + 1] = q.y; x[4 * c4 + 2] = q.z; x[4 * c4 + 3] = q.w;
        }
#pragma unroll 1
        for (int jb = 0; jb < 4; ++jb) {
          if (j == jb) {
            const uint32_t acol = kOffUV + uint32_t(16 * jb) * 256 + uint32_t(16 * jb) * 4;  // A_ab^T[16 jb][16 jb]
#pragma unroll
            for (int tt = 0; tt < 15; ++tt) {
              const float xt = x[tt];
#pragma unroll
              for (int q4 = (tt + 1) >> 2; q4 < 4; ++q4) {
                const float4 a4 = ld4(smem, acol + tt * 256 + q4 * 16);  // A_ab[16 jb + 4 q4 ..][16 jb + tt]
                if (4 * q4 > tt) x[4 * q4] = fmaf(a4.x, xt, x[4 * q4]);
                if (4 * q4 + 1 > tt) x[4 * q4 + 1] = fmaf(a4.y, xt, x[4 * q4 + 1]);
                if (4 * q4 + 2 > tt) x[4 * q4 + 2] = fmaf(a4.z, xt, x[4 * q4 + 2]);
                x[4 * q4 + 3] = fmaf(a4.w, xt, x[4 * q4 + 3]);
              }
            }
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4)
              st4(smem, kOffX2 + (4 * j + c4) * kCS64 + v * 16, make_float4(x[4 * c4], x[4 * c4 + 1], x[4 * c4 + 2], x[4 * c4 + 3]));
          }
          __syncthreads();
          if (j > jb) {
            float xb[16];
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              const float4 q = ld4(smem, kOffX2 + (4 * jb + c4) * kCS64 + v * 16);
              xb[4 * c4] = q.x; xb[4 * c4 + 1] = q.y; xb[4 * c4 + 2] = q.z; xb[4 * c4 + 3] = q.w;
            }
            const uint32_t acol = kOffUV + uint32_t(16 * jb) * 256 + uint32_t(16 * j) * 4;  // A_ab^T[16 jb][16 j]
            // two multiply-adds per instruction (fma.rn.f32x2): this fold is bound by instruction issue
            float2 xp[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) xp[e] = make_float2(x[2 * e], x[2 * e + 1]);
#pragma unroll
            for (int tt = 0; tt < 16; ++tt) {
              const float2 bb = make_float2(xb[tt], xb[tt]);
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                const float4 a4 = ld4(smem, acol + tt * 256 + q4 * 16);
                xp[2 * q4] = __ffma2_rn(make_float2(a4.x, a4.y), bb, xp[2 * q4]);
                xp[2 * q4 + 1] = __ffma2_rn(make_float2(a4.z, a4.w), bb, xp[2 * q4 + 1]);
              }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) { x[2 * e] = xp[e].x; x[2 * e + 1] = xp[e].y; }
          }
        }
        // every block has been read and A_ab^T with it: U rows -> state_dot_a (optional), U^T rounded over A_ab^T
        if (ok) {
          if (sda_ptr != nullptr) {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (16 * j + e < len)
                sda_ptr[(long long)token_row(t0, len, 16 * j + e) * row_stride + head_off + v] = x[e];
          }
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4)
            st4(smem, kOffUV + (4 * j + c4) * kCS64 + v * 16,
                umma::to_tf32(make_float4(x[4 * c4], x[4 * c4 + 1], x[4 * c4 + 2], x[4 * c4 + 3])));
        }
      }
      umma::fence_async_smem();
      umma::fence_before_sync();
      __syncthreads();
      umma::fence_after_sync();

      // ---- MMA 3: DC = D1 [U ; V] ---------------------------------------------------------------------------------
      if (tid == 0) {
#pragma unroll
        for (int ks = 0; ks < 16; ++ks)
          umma::mma_tf32_ts(tmem + kColDC, tmem + kColD1 + 8 * ks,
                            umma::desc_k_major(sbase + kOffUV + ks * 2 * kCS64, kCS64), idesc64, ks > 0 ? 1u : 0u);
        umma::mma_commit(&mbar[2]);
      }
      ok = wait_warp(&mbar[2], parity, ok);
      umma::fence_after_sync();
      // the last product has read its tiles: the next chunk's rows start their way into them
      if (has_next && ok) stage_rows(next_t0, min(max(next_end - next_t0, 1), kL), head_off);
      // ---- epilogue 3: Y rows out; S' = g_L (S + DC) -> registers, S0^T, boundary / state pool ----------------------
      if (ok) {
        uint32_t u[32];
        umma::tmem_ld32(tmem + kColDC + lane_base + c0, u);
        if (low) {
          umma::tmem_ld_wait();
          const bool last = !has_next;
          float* dst = last ? state + mt * kD + c0
                            : (boundary != nullptr
                                   ? boundary + ((long long)(c + c_step) * num_heads + head) * (kD * kD) + mt * kD + c0
                                   : nullptr);
#pragma unroll
          for (int j = 0; j < 32; j += 2) {  // two state values per instruction, the scalar bits
            const float2 t = __fmul2_rn(make_float2(g_last, g_last),
                                        __fadd2_rn(make_float2(S[j], S[j + 1]),
                                                   make_float2(__uint_as_float(u[j]), __uint_as_float(u[j + 1]))));
            S[j] = t.x;
            S[j + 1] = t.y;
          }
          if (dst != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; j += 8)
              stg256(dst + j, make_uint4(__float_as_uint(S[j]), __float_as_uint(S[j + 1]), __float_as_uint(S[j + 2]), __float_as_uint(S[j + 3])),
                     make_uint4(__float_as_uint(S[j + 4]), __float_as_uint(S[j + 5]), __float_as_uint(S[j + 6]), __float_as_uint(S[j + 7])));
          }
          if (!last) {
#pragma unroll
            for (int j = 0; j < 32; ++j) st1(smem, kOffS + tile_off(kCS64, c0 + j, mt), umma::to_tf32(S[j]));
          }
        } else {
          uint32_t u2[32];
          umma::tmem_ld32(tmem + kColDA + lane_base + c0, u2);
          umma::tmem_ld_wait();
          if (valid && y_ptr != nullptr) {
            const long long row = (long long)token_row(t0, len, mt) * row_stride + head_off + c0;
#pragma unroll
            for (int j = 0; j < 32; j += 16) {
              uint4 packed[2];
#pragma unroll
              for (int h8 = 0; h8 < 2; ++h8) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  o[e] = scale * (__uint_as_float(u[j + 8 * h8 + e]) + __uint_as_float(u2[j + 8 * h8 + e]));
                packed[h8].x = IO::pack(o[0], o[1]); packed[h8].y = IO::pack(o[2], o[3]);
                packed[h8].z = IO::pack(o[4], o[5]); packed[h8].w = IO::pack(o[6], o[7]);
                if (y32_ptr != nullptr)
                  stg256(y32_ptr + row + j + 8 * h8,
                         make_uint4(__float_as_uint(o[0]), __float_as_uint(o[1]), __float_as_uint(o[2]), __float_as_uint(o[3])),
                         make_uint4(__float_as_uint(o[4]), __float_as_uint(o[5]), __float_as_uint(o[6]), __float_as_uint(o[7])));
              }
              stg256(y_ptr + row + j, packed[0], packed[1]);
            }
          }
        }
      }
      umma::fence_async_smem();
      umma::fence_before_sync();
      ok = __syncthreads_and(ok ? 1 : 0) != 0;  // one verdict for the whole CTA: nobody walks on alone
      umma::fence_after_sync();
      if (!ok) {
        // fail closed: the rows of this (sequence, head) read as NaN, its state slot keeps the value it had
        const io_t nan16 = IO::store(quiet_nan());
        const int tb = chunk_starts[c_begin], te = chunk_ends[c_end - 1];
        for (long long e = (long long)tb * kD + tid; y_ptr != nullptr && e < (long long)te * kD; e += kThreads) {
          const long long at = (e / kD) * row_stride + head_off + (e % kD);
          y_ptr[at] = nan16;
          if (y32_ptr != nullptr) y32_ptr[at] = quiet_nan();
        }
        break;
      }
    }
  }
  if (!ok && tid == 0 && error_flag != nullptr) atomicExch(error_flag, 3);
  umma::cp_async_wait_all();
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, kTmemCols);
}

struct DeviceInfo {
  int sm_count = 0;
  bool attr_set[4] = {false, false, false, false};
};

DeviceInfo* device_info() {
  static DeviceInfo info[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
  DeviceInfo* d = &info[device];
  if (d->sm_count == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) return nullptr;
    d->sm_count = n;
  }
  return d;
}

template <typename io_t, bool kAdj>
int launch_fused(const int* sco, const int* cs, const int* ce, const int* state_indices, const int* status,
                 float* state_pool, const void* r, const void* w, const void* k, const void* v, const void* a,
                 const void* b, const void* bias, void* y, float* y32, float* boundary, float* sda,
                 int* error_flag, int total_tokens, int num_sequences, int num_heads, float scale, int which,
                 cudaStream_t stream) {
  DeviceInfo* info = device_info();
  if (info == nullptr) return fail(FRWKV_ERR_CUDA, "wkv7_chunk_fused_forward: cannot query the current device");
  if (!info->attr_set[which]) {
    cudaError_t e = cudaFuncSetAttribute(wkv7_chunk_fused_kernel<io_t, kAdj>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kFusedSmem);
    if (e != cudaSuccess)
      return fail(FRWKV_ERR_CUDA, "wkv7_chunk_fused_forward: cannot reserve shared memory: %s", cudaGetErrorString(e));
    info->attr_set[which] = true;
  }
  const int units = num_sequences * num_heads;
  const int grid = units < 2 * info->sm_count ? units : 2 * info->sm_count;
  wkv7_chunk_fused_kernel<io_t, kAdj><<<(unsigned)grid, kThreads, kFusedSmem, stream>>>(
      sco, cs, ce, state_indices, status, state_pool, static_cast<const io_t*>(r), static_cast<const io_t*>(w),
      static_cast<const io_t*>(k), static_cast<const io_t*>(v), static_cast<const io_t*>(a),
      static_cast<const io_t*>(b), static_cast<const io_t*>(bias), static_cast<io_t*>(y), y32, boundary, sda,
      num_heads, units, (long long)total_tokens * num_heads * kD, scale, error_flag);
  return check_launch("wkv7_chunk_fused_kernel");
}

}  // namespace
}  // namespace frwkv

// The fused form runs one CTA per (sequence, head) and takes the same time for any number of pairs up to one per SM;
// the two-kernel form spreads the chunks of few sequences over the GPU and its time grows with the pairs.  Measured
// at T = 4096 (and the same ratios at T = 1024): 64 pairs 0.51 ms against the fused form's 0.60 ms, 96 pairs 0.70 ms
// against 0.60 ms.
extern "C" int frwkv_wkv7_chunk_prefers_fused(int num_sequences, int num_heads) {
  return (long long)num_sequences * num_heads >= 80 ? 1 : 0;
}

extern "C" int frwkv_wkv7_chunk_fused_fp32io16_forward(
    const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends,
    const int32_t* state_indices, const int32_t* metadata_status, float* state_pool, const void* r,
    const void* decay_logits, const void* k, const void* v, const void* a, const void* b, const void* decay_bias,
    void* y, float* y_fp32, float* boundary, float* state_dot_a, int32_t* error_flag, int total_tokens,
    int num_sequences, int num_chunks, int num_heads, int head_size, int io_dtype, float scale,
    frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(seq_chunk_offsets && chunk_starts && chunk_ends && state_pool && r && decay_logits && k && v && a &&
                    b && y,
                "wkv7_chunk_fused_forward: null pointer argument");
  FRWKV_REQUIRE(total_tokens > 0 && num_sequences > 0 && num_chunks > 0 && num_heads > 0,
                "wkv7_chunk_fused_forward: sizes must be positive");
  FRWKV_REQUIRE(aligned32(state_pool, r, decay_logits, k, v, a, b, decay_bias, y, y_fp32, boundary, state_dot_a),
                "wkv7_chunk_fused_forward: tensor pointers must be 32-byte aligned");
  if (head_size != 64)
    return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_chunk_fused_forward: head size %d is not built (only 64)", head_size);
  FRWKV_REQUIRE((long long)num_sequences * num_heads <= 0x7fffffffLL,
                "wkv7_chunk_fused_forward: too many (sequence, head) pairs");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_fused<__nv_bfloat16, false>(seq_chunk_offsets, chunk_starts, chunk_ends, state_indices,
                                              metadata_status, state_pool, r, decay_logits, k, v, a, b, decay_bias,
                                              y, y_fp32, boundary, state_dot_a, error_flag, total_tokens,
                                              num_sequences, num_heads, scale, 0, s);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_fused<__half, false>(seq_chunk_offsets, chunk_starts, chunk_ends, state_indices, metadata_status,
                                       state_pool, r, decay_logits, k, v, a, b, decay_bias, y, y_fp32,
                                       boundary, state_dot_a, error_flag, total_tokens, num_sequences, num_heads,
                                       scale, 1, s);
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_chunk_fused_forward: token tensors must be float16 or bfloat16");
}

// ---- adjoint of the state at every chunk boundary (first stage of the chunked backward) -----------------------------
extern "C" int frwkv_wkv7_adjoint_scan(const int32_t* seq_chunk_offsets, const int32_t* chunk_starts,
                                       const int32_t* chunk_ends, const void* r, const void* decay_logits,
                                       const void* a, const void* b, const void* decay_bias, const void* grad_output,
                                       float* grad_state, float* boundary_adjoint, int32_t* error_flag,
                                       const int32_t* metadata_status, int total_tokens, int num_sequences,
                                       int num_chunks, int num_heads, int head_size, int io_dtype, float scale,
                                       frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(seq_chunk_offsets && chunk_starts && chunk_ends && r && decay_logits && a && b && grad_output &&
                    grad_state && boundary_adjoint,
                "wkv7_adjoint_scan: null pointer argument");
  FRWKV_REQUIRE(total_tokens > 0 && num_sequences > 0 && num_chunks > 0 && num_heads > 0,
                "wkv7_adjoint_scan: sizes must be positive");
  FRWKV_REQUIRE(aligned32(r, decay_logits, a, b, decay_bias, grad_output, grad_state, boundary_adjoint),
                "wkv7_adjoint_scan: tensor pointers must be 32-byte aligned");
  if (head_size != 64)
    return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_adjoint_scan: head size %d is not built (only 64)", head_size);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // the forward kernel in reverse time with a and b exchanged and dy for v; it makes its key rows
  // k^ = scale (w r + (b . r) a) itself, from the rows it has staged
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_fused<__nv_bfloat16, true>(seq_chunk_offsets, chunk_starts, chunk_ends, nullptr, metadata_status,
                                             grad_state, r, decay_logits, /*k: unused*/ r, grad_output, /*a=*/b,
                                             /*b=*/a, decay_bias, nullptr, nullptr, boundary_adjoint, nullptr,
                                             error_flag, total_tokens, num_sequences, num_heads, scale, 2, s);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_fused<__half, true>(seq_chunk_offsets, chunk_starts, chunk_ends, nullptr, metadata_status,
                                      grad_state, r, decay_logits, /*k: unused*/ r, grad_output, /*a=*/b, /*b=*/a,
                                      decay_bias, nullptr, nullptr, boundary_adjoint, nullptr, error_flag,
                                      total_tokens, num_sequences, num_heads, scale, 3, s);
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_adjoint_scan: token tensors must be float16 or bfloat16");
}
