// Chunk-parallel WKV7 backward on the tcgen05 tensor cores (head size 64, chunks of <= 64 tokens).
//
// Second stage of the chunked backward.  The first stage (frwkv_wkv7_adjoint_scan) has left, for every chunk, the
// adjoint G = dL/dS at the chunk's END; the forward has left the chunk-start state S0 (boundary) and the rows
// U = state_dot_a.  With those every (chunk, head) is independent: a persistent CTA takes one at a time and produces
// the six token gradients of its rows.  With the forward's quantities per chunk (g_t cumulative decay, g_L its last row)
//     A~ = a*g_{t-1}  R~ = r*g_t  B~ = b/g_t  K~ = k/g_t,   [A_ab|A_ak ; A_rb|A_rk] = mask([A~;R~][B~;K~]^T),
//     T = (I - A_ab)^-1,   X = A~ S0 + A_ak V,  U = T X,  Y' = R~ S0 + A_rk V + A_rb U,  S_L = g_L (S0 + B~^T U + K~^T V)
// and dY' = scale * dy, G^ = g_L * G (rows scaled), the adjoints are
//     dU = A_rb^T dY' + B~ G^            dX = T^T dU            dV = A_rk^T dY' + K~ G^ + A_ak^T dX
//     [dA_ab|dA_ak ; dA_rb|dA_rk] = mask([dX;dY'] [U;V]^T)                                       =: DD
//     [dA~ ; dR~] = [dX;dY'] S0^T + DD [B~;K~]          [dB~ ; dK~] = mask(DD^T) [A~;R~] + [U;V] G^^T
//     da = dA~ g_{t-1}   dr = dR~ g_t   db = dB~ / g_t   dk = dK~ / g_t
//     dlog w_s = sum_{t>=s} ( dr_t r_t - db_t b_t - dk_t k_t + da_{t+1} a_{t+1} ) + sum_v G S_L     (per key channel)
//     dlogit = dlog w * retention_log_derivative(logit).
// Every contraction is a tcgen05.mma kind::tf32 with fp32 accumulation.  Token x token matrices come straight from
// row tiles ([x;y][u;v]^T needs no transposition) and stay in tensor memory, masked in place, as the A operand of
// the next product; contractions over tokens take their B operand from tiles written transposed ([feature][token]).
// Transposed token x token matrices are not transposed but computed: D1T = [B~;K~][A~;R~]^T, DDT = [U;V][dX;dY']^T.
// T is never formed: dX = T^T dU is the solution of (I - A_ab)^T dX = dU, found in fp32 by blocked back substitution
// (256 threads, one per (value column, block of 16 tokens)), which costs a third of inverting and multiplying.
// [dX;dY'] and [U;V] enter the later products as shared-memory row tiles (both operands from shared memory).
//
// Tensor-memory columns (512):  XA [A~;R~]            |  XB [B~;K~] -> OUT1 [dA~;dR~]  |  D1 (A_ab) -> DD
//                               D1T -> DDT            |  DUV [dU;dV] -> OUT2 [dB~;dK~]
// 512 threads (warp w: lanes 32 (w % 4).., column group w / 4), one CTA per SM, ~221 KB of shared memory.
//
// Replaces the reference's serial backward kernels: csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_backward.cu:49-255
// and cuda_backward_v3 of csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cu:163-291.

#include "wkv7_chunk_common.cuh"

namespace frwkv {
namespace {

using namespace chunk;

constexpr int kL = 64;
constexpr int kD = 64;
constexpr int kBwdThreads = 512;
constexpr uint32_t kCS128 = 2064;  // chunk stride of the 128-row tiles
constexpr uint32_t kCS64 = 1040;   // ... of the 64-row tiles

constexpr uint32_t kOffGT = 0;                         // g[t][k]
constexpr uint32_t kOffRA = kOffGT + 16 * kCS64;       // B~ rows -> A_ab (fp32, rows 0..63) -> [U;V] rows
constexpr uint32_t kOffRB = kOffRA + 16 * kCS128;      // [A~;R~] rows -> [dX;dY'] rows
constexpr uint32_t kOffTBK = kOffRB + 16 * kCS128;     // [B~^T | K~^T]  rows k, columns (s | 64 + s)
constexpr uint32_t kOffTAR = kOffTBK + 32 * kCS64;     // [A~^T | R~^T]
constexpr uint32_t kOffTDY = kOffTAR + 32 * kCS64;     // dY'^T [v][t] -> dU^T -> dX^T; at the end  db * b
constexpr uint32_t kOffTG = kOffTDY + 16 * kCS64;      // G^^T [v][k];                 at the end  dr * r, then dlogit
constexpr uint32_t kOffNG = kOffTG + 16 * kCS64;       // G^ [k][v];                   at the end  dk * k
constexpr uint32_t kOffNS = kOffNG + 16 * kCS64;       // S0 [k][v];                   at the end  da * a
constexpr uint32_t kOffW = kOffNS + 16 * kCS64;        // the chunk's decay logits [64][64] 16-bit
constexpr uint32_t kBwdSmem = kOffW + kL * kD * 2;
static_assert(kOffRA % 128 == 0 && kOffRB % 128 == 0 && kOffTBK % 128 == 0 && kOffTAR % 128 == 0 && kOffTDY % 128 == 0 &&
                  kOffTG % 128 == 0 && kOffNG % 128 == 0 && kOffNS % 128 == 0 && kOffW % 128 == 0,
              "tile bases must stay 128-byte aligned");
static_assert(kBwdSmem + 2048 <= 232448, "the CTA must fit one SM's shared memory");
// The a, r, b, k and dy rows of the next item are staged as they are in HBM over the [dX;dY'] and [B~^T|K~^T] tiles,
// which are free from the fourth product group on: five tiles of 64 rows, rows padded by 16 bytes so that the threads
// of a warp, which read consecutive rows, hit different banks.
constexpr uint32_t kRawRow = 144;
constexpr uint32_t kRawBase = kOffRB;
constexpr uint32_t kRawW = kRawBase + 5 * 64 * kRawRow;  // the staged decay logits, 128 bytes per row
static_assert(kRawW + kL * kD * 2 <= kOffTAR, "the staged rows must fit the two free tiles");

constexpr uint32_t kColXA = 0, kColXB = 64, kColD1 = 128, kColD1T = 256, kColDUV = 384;
constexpr uint32_t kColOUT1 = kColXB, kColDD = kColD1, kColDDT = kColD1T, kColOUT2 = kColDUV;

template <typename io_t>
__global__ __launch_bounds__(kBwdThreads, 1) void wkv7_chunk_backward_kernel(
    const int* __restrict__ seq_chunk_offsets, const int* __restrict__ chunk_starts, const int* __restrict__ chunk_ends,
    const float* __restrict__ final_state, const float* __restrict__ boundary, const float* __restrict__ adjoint,
    const float* __restrict__ sda_ptr, const io_t* __restrict__ r_ptr, const io_t* __restrict__ w_ptr,
    const io_t* __restrict__ k_ptr, const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr,
    const io_t* __restrict__ b_ptr, const io_t* __restrict__ bias_ptr, const io_t* __restrict__ dy_ptr,
    io_t* __restrict__ dr_ptr, io_t* __restrict__ dw_ptr, io_t* __restrict__ dk_ptr, io_t* __restrict__ dv_ptr,
    io_t* __restrict__ da_ptr, io_t* __restrict__ db_ptr, int num_sequences, int num_heads, int num_items, float scale,
    int* __restrict__ error_flag, const int* __restrict__ metadata_status, long long output_elements) {
  using IO = Io16<io_t>;
  if (metadata_status != nullptr && metadata_status[0] != 0) {  // bad chunk tables: fail closed, touch nothing else
    const io_t nan16 = IO::store(quiet_nan());
    for (long long i = (long long)blockIdx.x * kBwdThreads + threadIdx.x; i < output_elements;
         i += (long long)gridDim.x * kBwdThreads) {
      dr_ptr[i] = nan16; dw_ptr[i] = nan16; dk_ptr[i] = nan16; dv_ptr[i] = nan16; da_ptr[i] = nan16; db_ptr[i] = nan16;
    }
    return;
  }
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t mbar[5];
  __shared__ uint32_t tmem_holder;
  __shared__ float seg_total[8][64];
  __shared__ float end_sum[64];  // sum_v G S_L per key channel
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m = 32 * (warp & 3) + lane;  // tensor-memory lane / operand row of this thread
  const int cg = warp >> 2;              // column group: 16 of 64 columns, 32 of 128
  const int mt = m & 63;                 // token of that row
  const bool low = m < 64;               // lanes 0..63: a / b / dX / U rows; lanes 64..127: r / k / dY' / V rows
  const int ch0 = 16 * cg;               // this thread's 16 channels
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 5; ++i) umma::mbar_init(&mbar[i], 1);
    umma::mbar_fence_init();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_holder, 512);
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

  // (first token, length, sequence, last chunk of its sequence?) of an item.  The next item's are requested while the
  // current one is worked on, so that no item starts by waiting for its chunk tables.
  struct ItemMeta { int t0, len, seq; bool last; };
  auto item_meta = [&](int item) {
    ItemMeta im;
    const int ch = item / num_heads;
    im.t0 = chunk_starts[ch];
    im.len = min(max(chunk_ends[ch] - im.t0, 1), kL);
    int lo = 0, hi = num_sequences;  // largest s with seq_chunk_offsets[s] <= ch
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (seq_chunk_offsets[mid] <= ch) lo = mid; else hi = mid;
    }
    im.seq = lo;
    im.last = ch + 1 == seq_chunk_offsets[lo + 1];
    return im;
  };
  // The a, r, b, k, dy rows and the decay logits of an item travel by cp.async one item ahead, as 16-byte pieces with
  // eight consecutive lanes per row (whole 128-byte lines per request; read straight into registers by the thread
  // that owns a row they cost a tag lookup per lane).  The logits sit behind the five padded tiles, 128 bytes per row,
  // and move to their own tile when the item starts (they are read again at its end).
  auto stage_rows = [&](int item, const ItemMeta& im) {
    const long long hoff = (long long)(item % num_heads) * kD;
    const int rowi = tid >> 3, part = tid & 7;
    const long long at = (long long)(im.t0 + min(rowi, im.len - 1)) * row_stride + hoff + 8 * part;
    const uint32_t bytes = rowi < im.len ? 16u : 0u;
#pragma unroll
    for (int i = 0; i < 5; ++i) {
      const io_t* base = i == 0 ? a_ptr : i == 1 ? r_ptr : i == 2 ? b_ptr : i == 3 ? k_ptr : dy_ptr;
      umma::cp_async16(sbase + kRawBase + i * (64 * kRawRow) + rowi * kRawRow + part * 16, base + at, bytes);
    }
    umma::cp_async16(sbase + kRawW + tid * 16, w_ptr + at, bytes);
    umma::cp_async_commit();
  };
  ItemMeta cur = item_meta(min((int)blockIdx.x, num_items - 1));
  if ((int)blockIdx.x < num_items) stage_rows(blockIdx.x, cur);

  for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, parity ^= 1u) {
    const int chunk = item / num_heads, head = item % num_heads;
    const int t0 = cur.t0, len = cur.len, seq = cur.seq;
    const bool last_of_seq = cur.last;
    const long long head_off = (long long)head * kD;
    const bool valid = mt < len;
    const float* s_end = last_of_seq ? final_state + ((long long)seq * num_heads + head) * (kD * kD)
                                     : boundary + ((long long)(chunk + 1) * num_heads + head) * (kD * kD);
    const float* s_start = boundary + ((long long)chunk * num_heads + head) * (kD * kD);
    const float* g_end = adjoint + ((long long)chunk * num_heads + head) * (kD * kD);
    const long long row = (long long)(t0 + min(mt, len - 1)) * row_stride + head_off + ch0;

    // ---- this thread's rows: 16 channels of (a, b) or (r, k, dy), from the staged tiles (rows past the end of a short
    //      chunk were zero-filled) ----------------------------------------------------------------------------------------
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    uint4 praw[2], qraw[2], draw[2];
    umma::cp_async_wait_all();
    __syncthreads();
    {
      const uint32_t at = kRawBase + uint32_t(mt) * kRawRow + uint32_t(ch0) * 2;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        praw[i] = *reinterpret_cast<const uint4*>(smem + at + (low ? 0 : 1) * (64 * kRawRow) + 16 * i);
        qraw[i] = *reinterpret_cast<const uint4*>(smem + at + (low ? 2 : 3) * (64 * kRawRow) + 16 * i);
        draw[i] = !low ? *reinterpret_cast<const uint4*>(smem + at + 4 * (64 * kRawRow) + 16 * i) : zero4;
      }
      // the previous item has read its logits for the last time (the barrier above): this item's take their place
      // for the decay gradient at the end; the decay tile below reads the staged copy
      *reinterpret_cast<uint4*>(smem + kOffW + tid * 16) = *reinterpret_cast<const uint4*>(smem + kRawW + tid * 16);
    }
    const bool has_next = item + (int)gridDim.x < num_items;
    // ---- g[t][k] (as in the forward kernel; threads 0..255 work) ------------------------------------------------
    if (tid < 256) {
      const int t = tid >> 2, q = tid & 3;
      float x[16];
      unpack8<io_t>(*reinterpret_cast<const uint4*>(smem + kRawW + t * 128 + q * 32), *reinterpret_cast<float(*)[8]>(&x[0]));
      unpack8<io_t>(*reinterpret_cast<const uint4*>(smem + kRawW + t * 128 + q * 32 + 16), *reinterpret_cast<float(*)[8]>(&x[8]));
      if (bias_ptr != nullptr) {
        float bz[16];
        unpack8<io_t>(__ldg(reinterpret_cast<const uint4*>(bias_ptr + head_off + 16 * q)), *reinterpret_cast<float(*)[8]>(&bz[0]));
        unpack8<io_t>(__ldg(reinterpret_cast<const uint4*>(bias_ptr + head_off + 16 * q + 8)), *reinterpret_cast<float(*)[8]>(&bz[8]));
#pragma unroll
        for (int e = 0; e < 16; ++e) x[e] += bz[e];
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) x[e] = t < len ? retention(x[e]) : 1.f;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        st4(smem, kOffGT + (4 * q + i) * kCS64 + t * 16, make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]));
    }
    __syncthreads();
    {
      const int kcol = tid & 63, seg = (tid >> 6) & 3;
      const uint32_t gcol = kOffGT + uint32_t(kcol >> 2) * kCS64 + uint32_t(kcol & 3) * 4 + uint32_t(16 * seg) * 16;
      float pr[16];
      if (tid < 256) {
#pragma unroll
        for (int i = 0; i < 16; ++i) pr[i] = ld1(smem, gcol + i * 16);
#pragma unroll
        for (int i = 1; i < 16; ++i) pr[i] *= pr[i - 1];
        seg_total[seg][kcol] = pr[15];
      }
      __syncthreads();
      if (tid < 256) {
        float mult = 1.f;
        if (seg > 0) mult = seg_total[0][kcol];
        if (seg > 1) mult *= seg_total[1][kcol];
        if (seg > 2) mult *= seg_total[2][kcol];
#pragma unroll
        for (int i = 0; i < 16; ++i) st1(smem, gcol + i * 16, pr[i] * mult);
      }
    }
    __syncthreads();
    // ---- operands: A forms to tensor memory, row tiles and transposed tiles to shared memory --------------------
      float dyv[16];  // dY' of this thread's row and channels (lanes 64..127), kept for the [dX;dY'] row tile
    {
      float pf[16], qf[16];
      unpack8<io_t>(praw[0], *reinterpret_cast<float(*)[8]>(&pf[0]));
      unpack8<io_t>(praw[1], *reinterpret_cast<float(*)[8]>(&pf[8]));
      unpack8<io_t>(qraw[0], *reinterpret_cast<float(*)[8]>(&qf[0]));
      unpack8<io_t>(qraw[1], *reinterpret_cast<float(*)[8]>(&qf[8]));
      unpack8<io_t>(draw[0], *reinterpret_cast<float(*)[8]>(&dyv[0]));
      unpack8<io_t>(draw[1], *reinterpret_cast<float(*)[8]>(&dyv[8]));
      uint32_t xa[16], xb[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kc = 4 * cg + j;  // 16-byte column chunk (4 channels)
        const float4 g = ld4(smem, kOffGT + kc * kCS64 + mt * 16);
        float4 sc = g;              // R~ = r * g_t
        if (low) sc = mt > 0 ? ld4(smem, kOffGT + kc * kCS64 + (mt - 1) * 16) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 p4 = umma::to_tf32(make_float4(pf[4 * j] * sc.x, pf[4 * j + 1] * sc.y, pf[4 * j + 2] * sc.z,
                                                    pf[4 * j + 3] * sc.w));
        const float4 q4 = umma::to_tf32(make_float4(qf[4 * j] * rcp_approx(g.x), qf[4 * j + 1] * rcp_approx(g.y),
                                                    qf[4 * j + 2] * rcp_approx(g.z), qf[4 * j + 3] * rcp_approx(g.w)));
        xa[4 * j] = __float_as_uint(p4.x); xa[4 * j + 1] = __float_as_uint(p4.y);
        xa[4 * j + 2] = __float_as_uint(p4.z); xa[4 * j + 3] = __float_as_uint(p4.w);
        xb[4 * j] = __float_as_uint(q4.x); xb[4 * j + 1] = __float_as_uint(q4.y);
        xb[4 * j + 2] = __float_as_uint(q4.z); xb[4 * j + 3] = __float_as_uint(q4.w);
        st4(smem, kOffRB + kc * kCS128 + m * 16, p4);           // [A~;R~] rows (B operand of D1T)
        if (low) st4(smem, kOffRA + kc * kCS128 + m * 16, q4);  // B~ rows (B operand of D1)
        // transposed: row = channel, column = this thread's token (second half of the columns for lanes 64..127)
        const uint32_t tcol = uint32_t(m >> 2) * kCS64 + uint32_t(m & 3) * 4 + uint32_t(4 * kc) * 16;
        st1(smem, kOffTAR + tcol, p4.x); st1(smem, kOffTAR + tcol + 16, p4.y);
        st1(smem, kOffTAR + tcol + 32, p4.z); st1(smem, kOffTAR + tcol + 48, p4.w);
        st1(smem, kOffTBK + tcol, q4.x); st1(smem, kOffTBK + tcol + 16, q4.y);
        st1(smem, kOffTBK + tcol + 32, q4.z); st1(smem, kOffTBK + tcol + 48, q4.w);
      }
      umma::tmem_st16(tmem + kColXA + lane_base + ch0, xa);
      umma::tmem_st16(tmem + kColXB + lane_base + ch0, xb);
      if (!low) {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          dyv[e] = umma::to_tf32(scale * dyv[e]);
          st1(smem, kOffTDY + tile_off(kCS64, ch0 + e, mt), dyv[e]);  // dY'^T [v][t]
        }
      }
    }
    umma::tmem_st_wait();
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- D1 = XA B~^T (only its A_ab block is used) and D1T = XB [A~;R~]^T ---------------------------------------
    if (tid == 0) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma::mma_tf32_ts(tmem + kColD1, tmem + kColXA + 8 * ks,
                          umma::desc_k_major(sbase + kOffRA + ks * 2 * kCS128, kCS128), idesc64, ks > 0 ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma::mma_tf32_ts(tmem + kColD1T, tmem + kColXB + 8 * ks,
                          umma::desc_k_major(sbase + kOffRB + ks * 2 * kCS128, kCS128), idesc128, ks > 0 ? 1u : 0u);
      umma::mma_commit(&mbar[0]);
    }
    // meanwhile the three state tiles: G^ = g_L * G in both orientations, S0, and the end term sum_v G S_L.  Warp w
    // takes keys 4 w .. 4 w + 3: lane (key kq = lane % 4, value chunk c = lane / 4) reads 16 bytes of each tile row
    // half, so that a load covers whole 128-byte lines; the transposed tile is written as 16-byte pieces after a
    // 4 x 4 exchange among the four lanes of a value chunk.
    {
      const int kq = lane & 3, c = lane >> 2;
      const int k0 = 4 * warp, kk = k0 + kq;
      const float gl = ld1(smem, kOffGT + tile_off(kCS64, 63, kk));
      float4 gv[2], sv[2], zv[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int at = kk * kD + 32 * h + 4 * c;
        gv[h] = __ldg(reinterpret_cast<const float4*>(g_end + at));
        sv[h] = __ldg(reinterpret_cast<const float4*>(s_end + at));
        zv[h] = __ldg(reinterpret_cast<const float4*>(s_start + at));
      }
      float e = 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        e += gv[h].x * sv[h].x + gv[h].y * sv[h].y + gv[h].z * sv[h].z + gv[h].w * sv[h].w;
        const int vc = 8 * h + c;  // 16-byte column chunk of the value index
        float4 hg = umma::to_tf32(make_float4(gl * gv[h].x, gl * gv[h].y, gl * gv[h].z, gl * gv[h].w));
        st4(smem, kOffNG + uint32_t(vc) * kCS64 + kk * 16, hg);
        st4(smem, kOffNS + uint32_t(vc) * kCS64 + kk * 16, umma::to_tf32(zv[h]));
        {  // afterwards lane kq holds G^[k0 .. k0 + 3][v] for v = 4 vc + kq
          const bool odd = (kq & 1) != 0, hi = (kq & 2) != 0;
          float s0 = odd ? hg.x : hg.y, s1 = odd ? hg.z : hg.w;
          float r0 = __shfl_xor_sync(0xffffffffu, s0, 1), r1 = __shfl_xor_sync(0xffffffffu, s1, 1);
          if (odd) { hg.x = r0; hg.z = r1; } else { hg.y = r0; hg.w = r1; }
          s0 = hi ? hg.x : hg.z; s1 = hi ? hg.y : hg.w;
          r0 = __shfl_xor_sync(0xffffffffu, s0, 2); r1 = __shfl_xor_sync(0xffffffffu, s1, 2);
          if (hi) { hg.x = r0; hg.y = r1; } else { hg.z = r0; hg.w = r1; }
        }
        st4(smem, kOffTG + uint32_t(k0 >> 2) * kCS64 + uint32_t(4 * vc + kq) * 16, hg);
      }
      // the end term of key kk: the eight lanes of the key added in a fixed order
      e += __shfl_xor_sync(0xffffffffu, e, 4);
      e += __shfl_xor_sync(0xffffffffu, e, 8);
      e += __shfl_xor_sync(0xffffffffu, e, 16);
      if (c == 0) end_sum[kk] = e;
    }
    ok = wait_warp(&mbar[0], parity, ok);
    umma::fence_after_sync();
    // D1T masked in place: its element [s][t] is kept for t > s (columns 0..63: products with A~) or t >= s (columns
    // 64..127: with R~).  A_ab -> fp32, as rows 0..63 of the [U;V] tile (B~ rows, consumed); dY' rows -> rows 64..127
    // of the [dX;dY'] tile ([A~;R~] rows, consumed).
    if (ok) {
      const bool mask_d1t = !low || cg >= 2;  // the A_ab^T block (lanes 0..63, columns 0..63) is never used
      if (mask_d1t) {
        uint32_t ut[32];
        const uint32_t taddr = tmem + kColD1T + lane_base + 32 * cg;
        umma::tmem_ld32(taddr, ut);
        umma::tmem_ld_wait();
        const int tbase = (32 * cg) & 63;
        const int first = cg >= 2 ? mt : mt + 1;  // smallest kept t
#pragma unroll
        for (int j = 0; j < 32; ++j) ut[j] = tbase + j >= first ? tf32_bits(__uint_as_float(ut[j])) : 0u;
        umma::tmem_st32(taddr, ut);
      }
      if (low) {
        uint32_t u[16];
        umma::tmem_ld16(tmem + kColD1 + lane_base + ch0, u);
        umma::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          const int s = ch0 + j;
          st4(smem, kOffRA + uint32_t(s >> 2) * kCS128 + uint32_t(mt) * 16,
              make_float4(s < mt ? __uint_as_float(u[j]) : 0.f, s + 1 < mt ? __uint_as_float(u[j + 1]) : 0.f,
                          s + 2 < mt ? __uint_as_float(u[j + 2]) : 0.f, s + 3 < mt ? __uint_as_float(u[j + 3]) : 0.f));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          st4(smem, kOffRB + (4 * cg + j) * kCS128 + m * 16,
              make_float4(dyv[4 * j], dyv[4 * j + 1], dyv[4 * j + 2], dyv[4 * j + 3]));
      }
      umma::tmem_st_wait();
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- DUV = D1T[:,64:128] dY' + XB G^  ->  [dU ; A_rk^T dY' + K~ G^] -------------------------------------------------
    if (tid == 0) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma::mma_tf32_ts(tmem + kColDUV, tmem + kColD1T + 64 + 8 * ks,
                          umma::desc_k_major(sbase + kOffTDY + ks * 2 * kCS64, kCS64), idesc64, ks > 0 ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma::mma_tf32_ts(tmem + kColDUV, tmem + kColXB + 8 * ks,
                          umma::desc_k_major(sbase + kOffTG + ks * 2 * kCS64, kCS64), idesc64, 1u);
      umma::mma_commit(&mbar[1]);
    }
    // this thread's 16 channels of its U row (fp32, four pieces) or V row (16-bit, two pieces)
    uint4 uvraw[4];
    {
      const uint4* up = low ? reinterpret_cast<const uint4*>(sda_ptr + row) : reinterpret_cast<const uint4*>(v_ptr + row);
#pragma unroll
      for (int i = 0; i < 4; ++i) uvraw[i] = zero4;
      if (valid) {
        ldg256(up, uvraw[0], uvraw[1]);
        if (low) ldg256(up + 2, uvraw[2], uvraw[3]);
      }
    }
    ok = wait_warp(&mbar[1], parity, ok);
    umma::fence_after_sync();
    // ---- dU^T -> shared memory (over dY'^T, consumed), unrounded: the solve below works in fp32 -------------------------
    if (ok && low) {
      uint32_t u[16];
      umma::tmem_ld16(tmem + kColDUV + lane_base + ch0, u);
      umma::tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 16; ++e) st1(smem, kOffTDY + tile_off(kCS64, ch0 + e, mt), __uint_as_float(u[e]));
    }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- dX = (I - A_ab)^-T dU by blocked back substitution in fp32, dX_s = dU_s + sum_{t > s} A_ab[t][s] dX_t.
    //      Thread (column v, block j) of warps 0..7 holds rows 16 j .. 16 j + 15 of column v.  From the last block to
    //      the first: the owners of block jb finish it (a 16 x 16 triangular solve in registers) and publish it; the
    //      owners of earlier blocks fold it in (a 16 x 16 update).  The other warps meanwhile pull the next item's
    //      rows into L2. --------------------------------------------------------------------------------------------------
    if (warp < 8) {
      const int v = tid & 63, j = tid >> 6;
      float x[16];
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const float4 q = ld4(smem, kOffTDY + (4 * j + c4) * kCS64 + v * 16);
        x[4 * c4] = q.x; x[4 * c4 + 1] = q.y; x[4 * c4 + 2] = q.z; x[4 * c4 + 3] = q.w;
      }
#pragma unroll 1
      for (int jb = 3; jb >= 0; --jb) {
        if (j == jb) {
          const uint32_t arow = kOffRA + uint32_t(4 * jb) * kCS128 + uint32_t(16 * jb) * 16;  // A_ab[16 jb][16 jb]
#pragma unroll
          for (int tt = 15; tt >= 1; --tt) {
            const float xt = x[tt];
#pragma unroll
            for (int s4 = 0; 4 * s4 < tt; ++s4) {
              const float4 a4 = ld4(smem, arow + s4 * kCS128 + tt * 16);
              x[4 * s4] = fmaf(a4.x, xt, x[4 * s4]);
              if (4 * s4 + 1 < tt) x[4 * s4 + 1] = fmaf(a4.y, xt, x[4 * s4 + 1]);
              if (4 * s4 + 2 < tt) x[4 * s4 + 2] = fmaf(a4.z, xt, x[4 * s4 + 2]);
              if (4 * s4 + 3 < tt) x[4 * s4 + 3] = fmaf(a4.w, xt, x[4 * s4 + 3]);
            }
          }
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4)
            st4(smem, kOffTDY + (4 * j + c4) * kCS64 + v * 16, make_float4(x[4 * c4], x[4 * c4 + 1], x[4 * c4 + 2], x[4 * c4 + 3]));
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (j < jb) {
          float xb[16];
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const float4 q = ld4(smem, kOffTDY + (4 * jb + c4) * kCS64 + v * 16);
            xb[4 * c4] = q.x; xb[4 * c4 + 1] = q.y; xb[4 * c4 + 2] = q.z; xb[4 * c4 + 3] = q.w;
          }
          const uint32_t arow = kOffRA + uint32_t(4 * j) * kCS128 + uint32_t(16 * jb) * 16;  // A_ab[16 jb][16 j]
          // two multiply-adds per instruction (fma.rn.f32x2): this fold is bound by instruction issue
          float2 xp[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) xp[e] = make_float2(x[2 * e], x[2 * e + 1]);
#pragma unroll
          for (int tt = 0; tt < 16; ++tt) {
            const float2 bb = make_float2(xb[tt], xb[tt]);
#pragma unroll
            for (int s4 = 0; s4 < 4; ++s4) {
              const float4 a4 = ld4(smem, arow + s4 * kCS128 + tt * 16);
              xp[2 * s4] = __ffma2_rn(make_float2(a4.x, a4.y), bb, xp[2 * s4]);
              xp[2 * s4 + 1] = __ffma2_rn(make_float2(a4.z, a4.w), bb, xp[2 * s4 + 1]);
            }
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) { x[2 * e] = xp[e].x; x[2 * e + 1] = xp[e].y; }
        }
      }
      // every block has been read: dX^T, rounded, over dU^T, and the dX rows into rows 0..63 of the [dX;dY'] tile
#pragma unroll
      for (int e = 0; e < 16; ++e) x[e] = umma::to_tf32(x[e]);
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4)
        st4(smem, kOffTDY + (4 * j + c4) * kCS64 + v * 16, make_float4(x[4 * c4], x[4 * c4 + 1], x[4 * c4 + 2], x[4 * c4 + 3]));
      const uint32_t col = kOffRB + uint32_t(v >> 2) * kCS128 + uint32_t(v & 3) * 4 + uint32_t(16 * j) * 16;
#pragma unroll
      for (int e = 0; e < 16; ++e) st1(smem, col + e * 16, x[e]);
    } else if (warp >= 8 && has_next) {
      // pull the next item's rows into L2
      const int u = tid - 256;
      const int nit = item + gridDim.x, nch = nit / num_heads, nhd = nit % num_heads;
      const int num_chunks_total = num_items / num_heads;
      const int nt0 = chunk_starts[nch], nlen = chunk_ends[nch] - nt0;
      for (int e = u; e < 8 * kL; e += 256) {
        const int which = e >> 6, rowi = e & 63;
        if (rowi < nlen) {
          const long long at = (long long)(nt0 + rowi) * row_stride + (long long)nhd * kD;
          if (which < 7) {
            const io_t* base = which == 0 ? a_ptr : which == 1 ? r_ptr : which == 2 ? b_ptr : which == 3 ? k_ptr
                               : which == 4 ? v_ptr : which == 5 ? dy_ptr : w_ptr;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(base + at));
          } else {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(sda_ptr + at));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(sda_ptr + at + 32));
          }
        }
      }
      // ... and its three 16 KB state tiles (chunk-start state, chunk-end adjoint; the chunk-end state where it is the
      // next boundary, which is all but the last chunk of a sequence): 128 lines of 128 bytes each
      for (int e = u; e < 384; e += 256) {
        const int which = e >> 7, line = e & 127;
        const float* base = nullptr;
        if (which == 0) base = boundary + ((long long)nch * num_heads + nhd) * (kD * kD);
        if (which == 1) base = adjoint + ((long long)nch * num_heads + nhd) * (kD * kD);
        if (which == 2 && nch + 1 < num_chunks_total) base = boundary + ((long long)(nch + 1) * num_heads + nhd) * (kD * kD);
        if (base != nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(base + 32 * line));
      }
    }
    // this thread's 16 channels of its U row or V row, rounded as operands; the V rows go to rows 64..127 of the
    // [U;V] tile now, the U rows (over A_ab) once the solve has read it
    float uv[16];
    {
      if (low) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uv[4 * i] = __uint_as_float(uvraw[i].x); uv[4 * i + 1] = __uint_as_float(uvraw[i].y);
          uv[4 * i + 2] = __uint_as_float(uvraw[i].z); uv[4 * i + 3] = __uint_as_float(uvraw[i].w);
        }
      } else {
        unpack8<io_t>(uvraw[0], *reinterpret_cast<float(*)[8]>(&uv[0]));
        unpack8<io_t>(uvraw[1], *reinterpret_cast<float(*)[8]>(&uv[8]));
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) uv[e] = umma::to_tf32(uv[e]);
      if (!low) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          st4(smem, kOffRA + (4 * cg + j) * kCS128 + m * 16, make_float4(uv[4 * j], uv[4 * j + 1], uv[4 * j + 2], uv[4 * j + 3]));
      }
    }
    __syncthreads();
    if (low) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        st4(smem, kOffRA + (4 * cg + j) * kCS128 + m * 16, make_float4(uv[4 * j], uv[4 * j + 1], uv[4 * j + 2], uv[4 * j + 3]));
    }
    // the next item's chunk-table entries: requested here, with no other load of this thread in flight, used at the end
    const ItemMeta nxt = has_next ? item_meta(item + gridDim.x) : cur;
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- dV: DUV += D1T[:,0:64] dX;   DD = [dX;dY'] [U;V]^T ---------------------------------------------------------
    if (tid == 0) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma::mma_tf32_ts(tmem + kColDUV, tmem + kColD1T + 8 * ks,
                          umma::desc_k_major(sbase + kOffTDY + ks * 2 * kCS64, kCS64), idesc64, 1u);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma::mma_tf32_ss(tmem + kColDD, umma::desc_k_major(sbase + kOffRB + ks * 2 * kCS128, kCS128),
                          umma::desc_k_major(sbase + kOffRA + ks * 2 * kCS128, kCS128), idesc128, ks > 0 ? 1u : 0u);
      umma::mma_commit(&mbar[2]);
    }
    ok = wait_warp(&mbar[2], parity, ok);
    umma::fence_after_sync();
    if (ok) {
      uint32_t u[16], ud[32];
      const uint32_t taddr = tmem + kColDD + lane_base + 32 * cg;
      if (!low) umma::tmem_ld16(tmem + kColDUV + lane_base + ch0, u);
      umma::tmem_ld32(taddr, ud);
      umma::tmem_ld_wait();
      // DD masked in place: element [t][s] kept for s < t (rows of dX) or s <= t (rows of dY')
      {
        const int sbase_col = (32 * cg) & 63;
        const int limit = low ? mt : mt + 1;
#pragma unroll
        for (int j = 0; j < 32; ++j) ud[j] = sbase_col + j < limit ? tf32_bits(__uint_as_float(ud[j])) : 0u;
        umma::tmem_st32(taddr, ud);
      }
      if (!low && valid) {  // dV rows out
        uint4 p0, p1;
        p0.x = IO::pack(__uint_as_float(u[0]), __uint_as_float(u[1])); p0.y = IO::pack(__uint_as_float(u[2]), __uint_as_float(u[3]));
        p0.z = IO::pack(__uint_as_float(u[4]), __uint_as_float(u[5])); p0.w = IO::pack(__uint_as_float(u[6]), __uint_as_float(u[7]));
        p1.x = IO::pack(__uint_as_float(u[8]), __uint_as_float(u[9])); p1.y = IO::pack(__uint_as_float(u[10]), __uint_as_float(u[11]));
        p1.z = IO::pack(__uint_as_float(u[12]), __uint_as_float(u[13])); p1.w = IO::pack(__uint_as_float(u[14]), __uint_as_float(u[15]));
        uint4* dst = reinterpret_cast<uint4*>(dv_ptr + row);
        stg256(dst, p0, p1);
      }
      umma::tmem_st_wait();
    }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- DDT = [U;V] [dX;dY']^T;   OUT1 = [dX;dY'] S0^T + DD [B~;K~]  ->  [dA~ ; dR~] --------------------------------
    if (tid == 0) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma::mma_tf32_ss(tmem + kColDDT, umma::desc_k_major(sbase + kOffRA + ks * 2 * kCS128, kCS128),
                          umma::desc_k_major(sbase + kOffRB + ks * 2 * kCS128, kCS128), idesc128, ks > 0 ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma::mma_tf32_ss(tmem + kColOUT1, umma::desc_k_major(sbase + kOffRB + ks * 2 * kCS128, kCS128),
                          umma::desc_k_major(sbase + kOffNS + ks * 2 * kCS64, kCS64), idesc64, ks > 0 ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < 16; ++ks)
        umma::mma_tf32_ts(tmem + kColOUT1, tmem + kColDD + 8 * ks,
                          umma::desc_k_major(sbase + kOffTBK + ks * 2 * kCS64, kCS64), idesc64, 1u);
      umma::mma_commit(&mbar[3]);
    }
    // this thread's a or r channels again (asked for twice rather than held in registers across the solve)
    uint4 praw2[2];
    {
      const uint4* pp = reinterpret_cast<const uint4*>((low ? a_ptr : r_ptr) + row);
      praw2[0] = zero4; praw2[1] = zero4;
      if (valid) ldg256(pp, praw2[0], praw2[1]);
    }
    ok = wait_warp(&mbar[3], parity, ok);
    umma::fence_after_sync();
    // the [dX;dY'] and [B~^T|K~^T] tiles have been read for the last time: the next item's rows start their way in
    if (ok && has_next) stage_rows(item + gridDim.x, nxt);
    // ---- DDT masked in place ([s][t] kept for t > s in the dX columns, t >= s in the dY' columns); da, dr out ------
    if (ok) {
      uint32_t u[16];
      {
        uint32_t ut[32];
        const uint32_t taddr = tmem + kColDDT + lane_base + 32 * cg;
        umma::tmem_ld32(taddr, ut);
        umma::tmem_ld16(tmem + kColOUT1 + lane_base + ch0, u);
        umma::tmem_ld_wait();
        const int tbase = (32 * cg) & 63;
        const int first = cg >= 2 ? mt : mt + 1;
#pragma unroll
        for (int j = 0; j < 32; ++j) ut[j] = tbase + j >= first ? tf32_bits(__uint_as_float(ut[j])) : 0u;
        umma::tmem_st32(taddr, ut);
      }
      // lanes 0..63: da = dA~ g_{t-1}; lanes 64..127: dr = dR~ g_t; the products da * a and dr * r go to shared memory
      // for the decay gradient, over the S0 tile and the G^^T tile (both read only by products that have completed)
      float pf[16];
      unpack8<io_t>(praw2[0], *reinterpret_cast<float(*)[8]>(&pf[0]));
      unpack8<io_t>(praw2[1], *reinterpret_cast<float(*)[8]>(&pf[8]));
      float gr[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kc = 4 * cg + j;
        float4 sc = make_float4(1.f, 1.f, 1.f, 1.f);
        if (!low) sc = ld4(smem, kOffGT + kc * kCS64 + mt * 16);
        else if (mt > 0) sc = ld4(smem, kOffGT + kc * kCS64 + (mt - 1) * 16);
        gr[4 * j] = __uint_as_float(u[4 * j]) * sc.x; gr[4 * j + 1] = __uint_as_float(u[4 * j + 1]) * sc.y;
        gr[4 * j + 2] = __uint_as_float(u[4 * j + 2]) * sc.z; gr[4 * j + 3] = __uint_as_float(u[4 * j + 3]) * sc.w;
        st4(smem, (low ? kOffNS : kOffTG) + kc * kCS64 + mt * 16,
            make_float4(gr[4 * j] * pf[4 * j], gr[4 * j + 1] * pf[4 * j + 1], gr[4 * j + 2] * pf[4 * j + 2],
                        gr[4 * j + 3] * pf[4 * j + 3]));
      }
      if (valid) {
        uint4 p0, p1;
        p0.x = IO::pack(gr[0], gr[1]); p0.y = IO::pack(gr[2], gr[3]); p0.z = IO::pack(gr[4], gr[5]); p0.w = IO::pack(gr[6], gr[7]);
        p1.x = IO::pack(gr[8], gr[9]); p1.y = IO::pack(gr[10], gr[11]); p1.z = IO::pack(gr[12], gr[13]); p1.w = IO::pack(gr[14], gr[15]);
        uint4* dst = reinterpret_cast<uint4*>((low ? da_ptr : dr_ptr) + row);
        stg256(dst, p0, p1);
      }
      umma::tmem_st_wait();
    }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- OUT2 = DDT [A~;R~] + [U;V] G^^T  ->  [dB~ ; dK~] --------------------------------------------------------------
    if (tid == 0) {
#pragma unroll
      for (int ks = 0; ks < 16; ++ks)
        umma::mma_tf32_ts(tmem + kColOUT2, tmem + kColDDT + 8 * ks,
                          umma::desc_k_major(sbase + kOffTAR + ks * 2 * kCS64, kCS64), idesc64, ks > 0 ? 1u : 0u);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma::mma_tf32_ss(tmem + kColOUT2, umma::desc_k_major(sbase + kOffRA + ks * 2 * kCS128, kCS128),
                          umma::desc_k_major(sbase + kOffNG + ks * 2 * kCS64, kCS64), idesc64, 1u);
      umma::mma_commit(&mbar[4]);
    }
    uint4 qraw2[2];  // ... and its b or k channels
    {
      const uint4* qp = reinterpret_cast<const uint4*>((low ? b_ptr : k_ptr) + row);
      qraw2[0] = zero4; qraw2[1] = zero4;
      if (valid) ldg256(qp, qraw2[0], qraw2[1]);
    }
    ok = wait_warp(&mbar[4], parity, ok);
    umma::fence_after_sync();
    // lanes 0..63: db = dB~ / g_s; lanes 64..127: dk = dK~ / g_s; products db * b, dk * k to shared memory
    if (ok) {
      uint32_t u[16];
      umma::tmem_ld16(tmem + kColOUT2 + lane_base + ch0, u);
      umma::tmem_ld_wait();
      float qf[16];
      unpack8<io_t>(qraw2[0], *reinterpret_cast<float(*)[8]>(&qf[0]));
      unpack8<io_t>(qraw2[1], *reinterpret_cast<float(*)[8]>(&qf[8]));
      float gr[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kc = 4 * cg + j;
        const float4 g = ld4(smem, kOffGT + kc * kCS64 + mt * 16);
        gr[4 * j] = __uint_as_float(u[4 * j]) * rcp_approx(g.x); gr[4 * j + 1] = __uint_as_float(u[4 * j + 1]) * rcp_approx(g.y);
        gr[4 * j + 2] = __uint_as_float(u[4 * j + 2]) * rcp_approx(g.z); gr[4 * j + 3] = __uint_as_float(u[4 * j + 3]) * rcp_approx(g.w);
        st4(smem, (low ? kOffTDY : kOffNG) + kc * kCS64 + mt * 16,
            make_float4(gr[4 * j] * qf[4 * j], gr[4 * j + 1] * qf[4 * j + 1], gr[4 * j + 2] * qf[4 * j + 2],
                        gr[4 * j + 3] * qf[4 * j + 3]));
      }
      if (valid) {
        uint4 p0, p1;
        p0.x = IO::pack(gr[0], gr[1]); p0.y = IO::pack(gr[2], gr[3]); p0.z = IO::pack(gr[4], gr[5]); p0.w = IO::pack(gr[6], gr[7]);
        p1.x = IO::pack(gr[8], gr[9]); p1.y = IO::pack(gr[10], gr[11]); p1.z = IO::pack(gr[12], gr[13]); p1.w = IO::pack(gr[14], gr[15]);
        uint4* dst = reinterpret_cast<uint4*>((low ? db_ptr : dk_ptr) + row);
        stg256(dst, p0, p1);
      }
    }
    __syncthreads();
    // ---- decay gradient: thread (key channel, 8-token segment): D_t = dr r - db b - dk k + (da a)_{t+1}, plus the end
    //      term at the chunk's last token; suffix sums over t; times dlog w / dlogit -----------------------------------
    {
      const int kcol = tid & 63, seg = tid >> 6;
      const uint32_t col = uint32_t(kcol >> 2) * kCS64 + uint32_t(kcol & 3) * 4;
      float dsum[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int t = 8 * seg + i;
        float d = ld1(smem, kOffTG + col + t * 16) - ld1(smem, kOffTDY + col + t * 16) - ld1(smem, kOffNG + col + t * 16);
        if (t + 1 < kL) d += ld1(smem, kOffNS + col + (t + 1) * 16);
        if (t == len - 1) {
          d += end_sum[kcol];
        }
        dsum[i] = t < len ? d : 0.f;
      }
#pragma unroll
      for (int i = 6; i >= 0; --i) dsum[i] += dsum[i + 1];
      seg_total[seg][kcol] = dsum[0];
      __syncthreads();
      float later = 0.f;
      for (int s2 = seg + 1; s2 < 8; ++s2) later += seg_total[s2][kcol];
      const float bias = bias_ptr != nullptr ? IO::load(bias_ptr + head_off + kcol) : 0.f;
      const io_t* wraw = reinterpret_cast<const io_t*>(smem + kOffW) + kcol;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int t = 8 * seg + i;
        st1(smem, kOffTG + col + t * 16, (dsum[i] + later) * retention_log_derivative(IO::load(wraw + t * kD) + bias));
      }
    }
    __syncthreads();
    {
      // dlogit rows out: thread (token, 8 channels)
      const int t = tid >> 3, c8 = tid & 7;
      if (t < len) {
        const float4 x0 = ld4(smem, kOffTG + (2 * c8) * kCS64 + t * 16), x1 = ld4(smem, kOffTG + (2 * c8 + 1) * kCS64 + t * 16);
        uint4 pk;
        pk.x = IO::pack(x0.x, x0.y); pk.y = IO::pack(x0.z, x0.w); pk.z = IO::pack(x1.x, x1.y); pk.w = IO::pack(x1.z, x1.w);
        *reinterpret_cast<uint4*>(dw_ptr + (long long)(t0 + t) * row_stride + head_off + 8 * c8) = pk;
      }
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    umma::fence_after_sync();
    cur = nxt;
    if (!ok) {
      // fail closed: the gradients of this item's rows read as NaN
      const io_t nan16 = IO::store(quiet_nan());
      io_t* outs[6] = {dr_ptr, dw_ptr, dk_ptr, dv_ptr, da_ptr, db_ptr};
      for (int e = tid; e < len * kD; e += kBwdThreads)
        for (int o = 0; o < 6; ++o) outs[o][(long long)(t0 + e / kD) * row_stride + head_off + e % kD] = nan16;
    }
  }
  if (!ok && tid == 0 && error_flag != nullptr) atomicExch(error_flag, 5);
  umma::cp_async_wait_all();
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, 512);
}

template <typename io_t>
int launch_chunk_backward(const int* sco, const int* cs, const int* ce, const float* final_state, const float* boundary,
                          const float* adjoint, const float* sda, const void* r, const void* w, const void* k,
                          const void* v, const void* a, const void* b, const void* bias, const void* dy, void* dr,
                          void* dw, void* dk, void* dv, void* da, void* db, int num_sequences, int num_chunks,
                          int num_heads, float scale, int* error_flag, const int* metadata_status, int total_tokens,
                          int which, cudaStream_t stream) {
  static bool opted_in[64][2] = {};
  static int sm_counts[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64)
    return fail(FRWKV_ERR_CUDA, "wkv7_chunk_backward: cannot identify the current device");
  if (!opted_in[device][which]) {
    cudaError_t e = cudaFuncSetAttribute(wkv7_chunk_backward_kernel<io_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kBwdSmem);
    if (e != cudaSuccess)
      return fail(FRWKV_ERR_CUDA, "wkv7_chunk_backward: cannot reserve shared memory: %s", cudaGetErrorString(e));
    cudaDeviceGetAttribute(&sm_counts[device], cudaDevAttrMultiProcessorCount, device);
    opted_in[device][which] = true;
  }
  const int items = num_chunks * num_heads;
  const int grid = sm_counts[device] > 0 && sm_counts[device] < items ? sm_counts[device] : items;
  using T = io_t;
  wkv7_chunk_backward_kernel<T><<<(unsigned)grid, kBwdThreads, kBwdSmem, stream>>>(
      sco, cs, ce, final_state, boundary, adjoint, sda, static_cast<const T*>(r), static_cast<const T*>(w),
      static_cast<const T*>(k), static_cast<const T*>(v), static_cast<const T*>(a), static_cast<const T*>(b),
      static_cast<const T*>(bias), static_cast<const T*>(dy), static_cast<T*>(dr), static_cast<T*>(dw),
      static_cast<T*>(dk), static_cast<T*>(dv), static_cast<T*>(da), static_cast<T*>(db), num_sequences, num_heads, items,
      scale, error_flag, metadata_status, (long long)total_tokens * num_heads * kD);
  return check_launch("wkv7_chunk_backward_kernel");
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_wkv7_chunk_backward(
    const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends, const float* final_state,
    const float* boundary, const float* boundary_adjoint, const float* state_dot_a, const void* r,
    const void* decay_logits, const void* k, const void* v, const void* a, const void* b, const void* decay_bias,
    const void* grad_output, void* grad_r, void* grad_decay_logits, void* grad_k, void* grad_v, void* grad_a, void* grad_b,
    int32_t* error_flag, const int32_t* metadata_status, int total_tokens, int num_sequences, int num_chunks,
    int num_heads, int head_size, int io_dtype, float scale, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(seq_chunk_offsets && chunk_starts && chunk_ends && final_state && boundary && boundary_adjoint &&
                    state_dot_a && r && decay_logits && k && v && a && b && grad_output && grad_r && grad_decay_logits &&
                    grad_k && grad_v && grad_a && grad_b,
                "wkv7_chunk_backward: null pointer argument");
  FRWKV_REQUIRE(num_sequences > 0 && num_chunks > 0 && num_heads > 0 && total_tokens > 0,
                "wkv7_chunk_backward: sizes must be positive");
  FRWKV_REQUIRE(aligned32(final_state, boundary, boundary_adjoint, state_dot_a, r, decay_logits, k, v, a, b, decay_bias,
                          grad_output, grad_r, grad_decay_logits, grad_k, grad_v, grad_a, grad_b),
                "wkv7_chunk_backward: tensor pointers must be 32-byte aligned");
  if (head_size != 64)
    return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_chunk_backward: head size %d is not built (only 64)", head_size);
  FRWKV_REQUIRE((long long)num_chunks * num_heads <= 0x7fffffffLL, "wkv7_chunk_backward: too many (chunk, head) pairs");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (io_dtype == FRWKV_DTYPE_BF16)
    return launch_chunk_backward<__nv_bfloat16>(seq_chunk_offsets, chunk_starts, chunk_ends, final_state, boundary,
                                                boundary_adjoint, state_dot_a, r, decay_logits, k, v, a, b, decay_bias,
                                                grad_output, grad_r, grad_decay_logits, grad_k, grad_v, grad_a, grad_b,
                                                num_sequences, num_chunks, num_heads, scale, error_flag, metadata_status,
                                                total_tokens, 0, s);
  if (io_dtype == FRWKV_DTYPE_FP16)
    return launch_chunk_backward<__half>(seq_chunk_offsets, chunk_starts, chunk_ends, final_state, boundary,
                                         boundary_adjoint, state_dot_a, r, decay_logits, k, v, a, b, decay_bias,
                                         grad_output, grad_r, grad_decay_logits, grad_k, grad_v, grad_a, grad_b,
                                         num_sequences, num_chunks, num_heads, scale, error_flag, metadata_status,
                                         total_tokens, 1, s);
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_chunk_backward: token tensors must be float16 or bfloat16");
}
