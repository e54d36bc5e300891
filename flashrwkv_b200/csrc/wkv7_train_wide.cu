// WKV7 training (forward with saved tensors, backward with all seven gradients) for head sizes 128 and 256.
//
// These sizes keep the plain recurrence (the head-size-64 operators are the chunked tensor-core kernels):
//   forward      one CTA per (sequence, head, block of 128 value columns), thread (c, q) holds the 64 state values
//                S[64 q + i][v0 + c] in registers for the whole sequence (the layout of wkv7_recurrent_wide.cu) and
//                additionally writes the state at the start of every chunk (boundary), the row sa_t = S_{t-1}^T a_t of
//                every token (state_dot_a) and, for the dense op library, the state after every 16 tokens.
//   checkpoints  with sa known the update S_t = diag(w) S + b sa^T + k v^T has no reduction left, so the state after
//                tokens 16 / 32 / 48 of every chunk is rebuilt element-wise from the chunk's boundary state, all
//                (chunk, head, column block) units in parallel.  The backward re-anchors on them.
//   backward     one CTA per (sequence, head, block of 64 value columns), D threads; thread (rg, cg) = (j / 4, j % 4)
//                owns rows 4 rg .. 4 rg + 3 and 16 of the 64 columns of the state slice S and of its adjoint G.
//                Tokens are walked in reverse; per token
//                    G += scale r (x) dy;   dr = scale S_t dy;   dk = G v;   db = G sa;       (row sums)
//                    dv = G^T k;   dsa = G^T b;                                               (column sums)
//                    S_{t-1} = (S_t - k v^T - b sa^T) / w;   dw = rowsum(G * S_{t-1});   da = S_{t-1} dsa;
//                    G = diag(w) G + a dsa^T.
//                Undoing the update amplifies rounding by 1/w per step, so S is re-anchored every <= 16 tokens.
//                Column sums (dv, dsa) are complete inside a CTA.  Row sums run over all D value columns, i.e. over
//                the D / 64 CTAs of a head: each writes its partial sums as fp32 to a workspace, in a fixed place.
//   reduce       adds the D / 64 partials in a fixed order (bit-reproducible), applies d w / d logit to dw, rounds.
//
// Replaces, for D = 128 / 256, forward_kernel_split64 / backward_kernel_split64 / the tiled256 backward
// (csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cu:110-150,293-478) and the wide instantiations of the
// StateTune kernels (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_forward.cu,
// csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_backward.cu:317-502) of the reference.

#include "frwkv_common.cuh"

namespace frwkv {
namespace {

constexpr int kFwdCols = 128;  // value columns per CTA, forward and checkpoints
constexpr int kBwdCols = 64;   // value columns per CTA, backward

// r, retention(w), k, a, b of one token into shared memory (D values each); called by every thread of the CTA
template <typename io_t, int D>
__device__ __forceinline__ void stage_vectors(float (*vec_s)[D], const io_t* r_ptr, const io_t* w_ptr,
                                              const io_t* k_ptr, const io_t* a_ptr, const io_t* b_ptr, long long tb,
                                              int threads) {
  using IO = Io16<io_t>;
  for (int e = threadIdx.x; e < D; e += threads) {
    vec_s[0][e] = r_ptr != nullptr ? IO::load(r_ptr + tb + e) : 0.f;
    vec_s[1][e] = retention(IO::load(w_ptr + tb + e));
    vec_s[2][e] = IO::load(k_ptr + tb + e);
    vec_s[3][e] = a_ptr != nullptr ? IO::load(a_ptr + tb + e) : 0.f;
    vec_s[4][e] = IO::load(b_ptr + tb + e);
  }
}

// ---- forward ---------------------------------------------------------------------------------------------------------
template <typename io_t, int D>
__global__ __launch_bounds__(kFwdCols*(D / 64), 1) void train_wide_forward_kernel(
    const int* __restrict__ seq_chunk_offsets, const int* __restrict__ chunk_starts, const int* __restrict__ chunk_ends,
    float* __restrict__ state, const io_t* __restrict__ r_ptr, const io_t* __restrict__ w_ptr,
    const io_t* __restrict__ k_ptr, const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr,
    const io_t* __restrict__ b_ptr, io_t* __restrict__ y_ptr, float* __restrict__ boundary,
    float* __restrict__ state_dot_a, float* __restrict__ dense_checkpoints, int dense_groups, int num_heads,
    float scale, const int* __restrict__ status) {
  using IO = Io16<io_t>;
  constexpr int kSlabs = D / 64, kThreads = kFwdCols * kSlabs, kColBlocks = D / kFwdCols;
  __shared__ __align__(16) float vec_s[5][D];
  __shared__ float part_s[kSlabs][kFwdCols];
  if (status != nullptr && status[0] != 0) return;  // bad chunk tables: touch nothing (the host side poisons the outputs)
  const int c = threadIdx.x % kFwdCols, q = threadIdx.x / kFwdCols;
  const int cb = blockIdx.x % kColBlocks;
  const long long seq_head = blockIdx.x / kColBlocks;
  const int head = (int)(seq_head % num_heads), seq = (int)(seq_head / num_heads);
  const int col = cb * kFwdCols + c;
  const long long tile = (long long)(64 * q) * D + col;  // this thread's first element inside a D x D state
  float* sbase = state + seq_head * ((long long)D * D) + tile;
  float S[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) S[i] = sbase[(long long)i * D];
  int seq_token = 0;  // index of the token inside its sequence (dense checkpoints)
  for (int ch = seq_chunk_offsets[seq]; ch < seq_chunk_offsets[seq + 1]; ++ch) {
    const int t0 = chunk_starts[ch], t1 = chunk_ends[ch];
    if (boundary != nullptr) {
      float* dst = boundary + ((long long)ch * num_heads + head) * ((long long)D * D) + tile;
#pragma unroll
      for (int i = 0; i < 64; ++i) dst[(long long)i * D] = S[i];
    }
    for (int t = t0; t < t1; ++t, ++seq_token) {
      const long long tb = ((long long)t * num_heads + head) * D;
      __syncthreads();  // the previous token's vectors and partial sums are no longer read
      stage_vectors<io_t, D>(vec_s, r_ptr, w_ptr, k_ptr, a_ptr, b_ptr, tb, kThreads);
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
      if (q == 0 && state_dot_a != nullptr) state_dot_a[tb + col] = sa;
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
        y_ptr[tb + col] = IO::store(y * scale);
      }
      if (dense_checkpoints != nullptr && (seq_token & 15) == 15) {
        float* dst = dense_checkpoints + (seq_head * dense_groups + (seq_token >> 4)) * ((long long)D * D) + tile;
#pragma unroll
        for (int i = 0; i < 64; ++i) dst[(long long)i * D] = S[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 64; ++i) sbase[(long long)i * D] = S[i];
}

// ---- checkpoints: state after tokens 16 / 32 / 48 of every chunk, [Cn][3][H][D][D] ---------------------------------------
template <typename io_t, int D>
__global__ __launch_bounds__(kFwdCols*(D / 64), 1) void train_wide_checkpoints_kernel(
    const int* __restrict__ chunk_starts, const int* __restrict__ chunk_ends, const float* __restrict__ boundary,
    const float* __restrict__ state_dot_a, const io_t* __restrict__ w_ptr, const io_t* __restrict__ k_ptr,
    const io_t* __restrict__ v_ptr, const io_t* __restrict__ b_ptr, float* __restrict__ checkpoints, int num_heads,
    const int* __restrict__ status) {
  using IO = Io16<io_t>;
  if (status != nullptr && status[0] != 0) return;
  constexpr int kSlabs = D / 64, kThreads = kFwdCols * kSlabs, kColBlocks = D / kFwdCols;
  __shared__ __align__(16) float vec_s[5][D];
  const int c = threadIdx.x % kFwdCols, q = threadIdx.x / kFwdCols;
  const int cb = blockIdx.x % kColBlocks;
  const long long chunk_head = blockIdx.x / kColBlocks;
  const int head = (int)(chunk_head % num_heads), ch = (int)(chunk_head / num_heads);
  const int col = cb * kFwdCols + c;
  const long long tile = (long long)(64 * q) * D + col;
  const int t0 = chunk_starts[ch], len = chunk_ends[ch] - t0;
  if (len <= 16) return;  // no checkpoint inside this chunk (uniform over the CTA)
  const float* src = boundary + chunk_head * ((long long)D * D) + tile;
  float S[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) S[i] = src[(long long)i * D];
  const int last = 16 * ((len - 1) / 16);  // tokens before the last checkpoint that is needed
  for (int rel = 0; rel < last; ++rel) {
    const long long tb = ((long long)(t0 + rel) * num_heads + head) * D;
    __syncthreads();
    stage_vectors<io_t, D>(vec_s, nullptr, w_ptr, k_ptr, nullptr, b_ptr, tb, kThreads);
    const float vv = IO::load(v_ptr + tb + col), sa = state_dot_a[tb + col];
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 64; i += 4) {
      const float4 w4 = *reinterpret_cast<const float4*>(&vec_s[1][64 * q + i]);
      const float4 b4 = *reinterpret_cast<const float4*>(&vec_s[4][64 * q + i]);
      const float4 k4 = *reinterpret_cast<const float4*>(&vec_s[2][64 * q + i]);
      S[i] = fmaf(w4.x, S[i], fmaf(b4.x, sa, k4.x * vv));
      S[i + 1] = fmaf(w4.y, S[i + 1], fmaf(b4.y, sa, k4.y * vv));
      S[i + 2] = fmaf(w4.z, S[i + 2], fmaf(b4.z, sa, k4.z * vv));
      S[i + 3] = fmaf(w4.w, S[i + 3], fmaf(b4.w, sa, k4.w * vv));
    }
    if ((rel & 15) == 15) {
      float* dst = checkpoints + (((long long)ch * 3 + (rel >> 4)) * num_heads + head) * ((long long)D * D) + tile;
#pragma unroll
      for (int i = 0; i < 64; ++i) dst[(long long)i * D] = S[i];
    }
  }
}

// ---- backward --------------------------------------------------------------------------------------------------------
enum { kPartDr = 0, kPartDk = 1, kPartDb = 2, kPartDw = 3, kPartDa = 4, kPartCount = 5 };

__device__ __forceinline__ float group_sum4(float x) {  // over the four adjacent lanes that share a row group
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

// partials: [kPartCount][D / 64][elements] fp32, elements = total_tokens * num_heads * D
template <typename io_t, int D>
__global__ __launch_bounds__(D, 1) void train_wide_backward_kernel(
    const int* __restrict__ seq_chunk_offsets, const int* __restrict__ chunk_starts, const int* __restrict__ chunk_ends,
    const float* __restrict__ final_state, const float* __restrict__ boundary, const float* __restrict__ checkpoints,
    const float* __restrict__ state_dot_a, const io_t* __restrict__ r_ptr, const io_t* __restrict__ w_ptr,
    const io_t* __restrict__ k_ptr, const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr,
    const io_t* __restrict__ b_ptr, const io_t* __restrict__ dy_ptr, const float* __restrict__ grad_final_state,
    io_t* __restrict__ dv_ptr, float* __restrict__ dS0_ptr, float* __restrict__ partials, long long elements,
    int num_heads, float scale, const int* __restrict__ status) {
  using IO = Io16<io_t>;
  constexpr int kBlocks = D / kBwdCols, kRowGroups = D / 4;
  if (status != nullptr && status[0] != 0) return;
  __shared__ __align__(16) float vec_s[5][D];                    // r, w, k, a, b of the current token
  __shared__ __align__(16) float col_s[3][kBwdCols];             // v, dy, sa of this CTA's columns
  __shared__ __align__(16) float part_dv[kRowGroups][kBwdCols + 4];
  __shared__ __align__(16) float part_dsa[kRowGroups][kBwdCols + 4];
  __shared__ __align__(16) float dsa_s[kBwdCols];
  const int j = threadIdx.x;
  const int rg = j >> 2, cg = j & 3, row0 = 4 * rg, colb = 4 * cg;
  // tile column c4 + e (c4 = 0, 4, 8, 12; e = 0..3) is column colb + 4 * c4 + e of the CTA's 64
  const int vb = blockIdx.x % kBlocks;
  const long long seq_head = blockIdx.x / kBlocks;
  const int head = (int)(seq_head % num_heads), seq = (int)(seq_head / num_heads);
  const int c_begin = seq_chunk_offsets[seq], c_end = seq_chunk_offsets[seq + 1];
  const long long DD = (long long)D * D;
  const long long slice = (long long)kBwdCols * vb;  // first column of this CTA inside a D x D state
  const auto tile_ptr = [&](const float* base, int rr, int c4) { return base + (long long)(row0 + rr) * D + slice + colb + 4 * c4; };

  float S[4][16], G[4][16];
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
#pragma unroll
    for (int c4 = 0; c4 < 16; c4 += 4) {
      float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
      if (grad_final_state != nullptr) g = *reinterpret_cast<const float4*>(tile_ptr(grad_final_state + seq_head * DD, rr, c4));
      G[rr][c4] = g.x; G[rr][c4 + 1] = g.y; G[rr][c4 + 2] = g.z; G[rr][c4 + 3] = g.w;
      S[rr][c4] = 0.f; S[rr][c4 + 1] = 0.f; S[rr][c4 + 2] = 0.f; S[rr][c4 + 3] = 0.f;
    }
  }
  float* part = partials + (long long)vb * elements;  // + which * kBlocks * elements + token offset + row
  const long long part_stride = (long long)kBlocks * elements;

  for (int ch = c_end - 1; ch >= c_begin; --ch) {
    const int t0 = chunk_starts[ch], len = chunk_ends[ch] - t0;
    for (int rel = len - 1; rel >= 0; --rel) {
      const int t = t0 + rel;
      const long long tb = ((long long)t * num_heads + head) * D;
      __syncthreads();  // the previous token's vectors, tables and dsa are no longer read
      stage_vectors<io_t, D>(vec_s, r_ptr, w_ptr, k_ptr, a_ptr, b_ptr, tb, D);
      if (j < kBwdCols) {
        col_s[0][j] = IO::load(v_ptr + tb + slice + j);
        col_s[1][j] = dy_ptr != nullptr ? IO::load(dy_ptr + tb + slice + j) : 0.f;
        col_s[2][j] = state_dot_a[tb + slice + j];
      }
      if (rel == len - 1 || (rel & 15) == 15) {  // re-anchor S on the saved state that follows this token
        const int q = rel >> 4;
        const float* anchor;
        if (16 * (q + 1) < len) anchor = checkpoints + (((long long)ch * 3 + q) * num_heads + head) * DD;
        else if (ch + 1 < c_end) anchor = boundary + ((long long)(ch + 1) * num_heads + head) * DD;
        else anchor = final_state + seq_head * DD;
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
#pragma unroll
          for (int c4 = 0; c4 < 16; c4 += 4) {
            const float4 s = *reinterpret_cast<const float4*>(tile_ptr(anchor, rr, c4));
            S[rr][c4] = s.x; S[rr][c4 + 1] = s.y; S[rr][c4 + 2] = s.z; S[rr][c4 + 3] = s.w;
          }
        }
      }
      __syncthreads();
      // ---- phase 1: G += scale r (x) dy, then every sum that uses G_t and S_t ------------------------------------------
      float rs[4], kr[4], br[4], dr[4], dk[4], db[4];
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) {
        rs[rr] = scale * vec_s[0][row0 + rr]; kr[rr] = vec_s[2][row0 + rr]; br[rr] = vec_s[4][row0 + rr];
        dr[rr] = 0.f; dk[rr] = 0.f; db[rr] = 0.f;
      }
#pragma unroll
      for (int c4 = 0; c4 < 16; c4 += 4) {
        const float4 vv = *reinterpret_cast<const float4*>(&col_s[0][colb + 4 * c4]);
        const float4 dy = *reinterpret_cast<const float4*>(&col_s[1][colb + 4 * c4]);
        const float4 sa = *reinterpret_cast<const float4*>(&col_s[2][colb + 4 * c4]);
        const float v4[4] = {vv.x, vv.y, vv.z, vv.w}, dy4[4] = {dy.x, dy.y, dy.z, dy.w}, sa4[4] = {sa.x, sa.y, sa.z, sa.w};
        float dvp[4] = {0.f, 0.f, 0.f, 0.f}, dsap[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float g = fmaf(rs[rr], dy4[e], G[rr][c4 + e]);
            G[rr][c4 + e] = g;
            dr[rr] = fmaf(S[rr][c4 + e], dy4[e], dr[rr]);
            dk[rr] = fmaf(g, v4[e], dk[rr]);
            db[rr] = fmaf(g, sa4[e], db[rr]);
            dvp[e] = fmaf(g, kr[rr], dvp[e]);
            dsap[e] = fmaf(g, br[rr], dsap[e]);
          }
        }
        *reinterpret_cast<float4*>(&part_dv[rg][colb + 4 * c4]) = make_float4(dvp[0], dvp[1], dvp[2], dvp[3]);
        *reinterpret_cast<float4*>(&part_dsa[rg][colb + 4 * c4]) = make_float4(dsap[0], dsap[1], dsap[2], dsap[3]);
      }
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) {
        dr[rr] = scale * group_sum4(dr[rr]); dk[rr] = group_sum4(dk[rr]); db[rr] = group_sum4(db[rr]);
      }
      if (cg == 0) {
        *reinterpret_cast<float4*>(part + kPartDr * part_stride + tb + row0) = make_float4(dr[0], dr[1], dr[2], dr[3]);
        *reinterpret_cast<float4*>(part + kPartDk * part_stride + tb + row0) = make_float4(dk[0], dk[1], dk[2], dk[3]);
        *reinterpret_cast<float4*>(part + kPartDb * part_stride + tb + row0) = make_float4(db[0], db[1], db[2], db[3]);
      }
      __syncthreads();
      // ---- column sums over all D key rows: dsa (idx < 64) and dv (idx >= 64) ----------------------------------------
      if (j < 2 * kBwdCols) {
        const int col = j & (kBwdCols - 1);
        const float(*tab)[kBwdCols + 4] = j < kBwdCols ? part_dsa : part_dv;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 4
        for (int g = 0; g < kRowGroups; g += 4) {
          s0 += tab[g][col]; s1 += tab[g + 1][col]; s2 += tab[g + 2][col]; s3 += tab[g + 3][col];
        }
        const float total = (s0 + s1) + (s2 + s3);
        if (j < kBwdCols) dsa_s[col] = total;
        else if (dv_ptr != nullptr) dv_ptr[tb + slice + col] = IO::store(total);
      }
      __syncthreads();
      // ---- phase 2: undo the state update, the sums that use S_{t-1}, then the adjoint step --------------------------
      float wr[4], ar[4], iw[4], dw[4], da[4];
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) {
        wr[rr] = vec_s[1][row0 + rr]; ar[rr] = vec_s[3][row0 + rr]; iw[rr] = 1.f / wr[rr];
        dw[rr] = 0.f; da[rr] = 0.f;
      }
#pragma unroll
      for (int c4 = 0; c4 < 16; c4 += 4) {
        const float4 vv = *reinterpret_cast<const float4*>(&col_s[0][colb + 4 * c4]);
        const float4 sa = *reinterpret_cast<const float4*>(&col_s[2][colb + 4 * c4]);
        const float4 dd = *reinterpret_cast<const float4*>(&dsa_s[colb + 4 * c4]);
        const float v4[4] = {vv.x, vv.y, vv.z, vv.w}, sa4[4] = {sa.x, sa.y, sa.z, sa.w}, d4[4] = {dd.x, dd.y, dd.z, dd.w};
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float sp = fmaf(-br[rr], sa4[e], fmaf(-kr[rr], v4[e], S[rr][c4 + e])) * iw[rr];
            S[rr][c4 + e] = sp;
            dw[rr] = fmaf(G[rr][c4 + e], sp, dw[rr]);
            da[rr] = fmaf(sp, d4[e], da[rr]);
            G[rr][c4 + e] = fmaf(wr[rr], G[rr][c4 + e], ar[rr] * d4[e]);
          }
        }
      }
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) { dw[rr] = group_sum4(dw[rr]); da[rr] = group_sum4(da[rr]); }
      if (cg == 0) {
        *reinterpret_cast<float4*>(part + kPartDw * part_stride + tb + row0) = make_float4(dw[0], dw[1], dw[2], dw[3]);
        *reinterpret_cast<float4*>(part + kPartDa * part_stride + tb + row0) = make_float4(da[0], da[1], da[2], da[3]);
      }
    }
  }
  if (dS0_ptr != nullptr) {
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
#pragma unroll
      for (int c4 = 0; c4 < 16; c4 += 4)
        *reinterpret_cast<float4*>(dS0_ptr + seq_head * DD + (long long)(row0 + rr) * D + slice + colb + 4 * c4) =
            make_float4(G[rr][c4], G[rr][c4 + 1], G[rr][c4 + 2], G[rr][c4 + 3]);
    }
  }
}

// adds the D / 64 partials of every row sum in a fixed order; dw gets d w / d logit = w dlog(w)/dx
template <typename io_t, int D>
__global__ void train_wide_reduce_kernel(const float* __restrict__ partials, long long elements,
                                         const io_t* __restrict__ w_ptr, io_t* __restrict__ dr_ptr,
                                         io_t* __restrict__ dw_ptr, io_t* __restrict__ dk_ptr,
                                         io_t* __restrict__ da_ptr, io_t* __restrict__ db_ptr,
                                         const int* __restrict__ status) {
  using IO = Io16<io_t>;
  if (status != nullptr && status[0] != 0) return;
  constexpr int kBlocks = D / kBwdCols;
  const long long part_stride = (long long)kBlocks * elements;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < elements;
       e += (long long)gridDim.x * blockDim.x) {
    float sum[kPartCount];
#pragma unroll
    for (int which = 0; which < kPartCount; ++which) {
      float s = 0.f;
#pragma unroll
      for (int vb = 0; vb < kBlocks; ++vb) s += partials[which * part_stride + vb * elements + e];
      sum[which] = s;
    }
    if (dr_ptr != nullptr) dr_ptr[e] = IO::store(sum[kPartDr]);
    if (dk_ptr != nullptr) dk_ptr[e] = IO::store(sum[kPartDk]);
    if (db_ptr != nullptr) db_ptr[e] = IO::store(sum[kPartDb]);
    if (da_ptr != nullptr) da_ptr[e] = IO::store(sum[kPartDa]);
    if (dw_ptr != nullptr) {
      const float x = IO::load(w_ptr + e);
      dw_ptr[e] = IO::store(sum[kPartDw] * retention(x) * retention_log_derivative(x));
    }
  }
}

template <typename io_t, int D>
int launch_forward(const int* sco, const int* cs, const int* ce, float* state, const void* r, const void* w,
                   const void* k, const void* v, const void* a, const void* b, void* y, float* boundary, float* sda,
                   float* dense_checkpoints, int dense_groups, int num_sequences, int num_heads, float scale,
                   const int* status, cudaStream_t stream) {
  const long long blocks = (long long)num_sequences * num_heads * (D / kFwdCols);
  if (blocks > 0x7fffffffLL) return fail(FRWKV_ERR_INVALID_ARGUMENT, "wkv7_train_wide: too many (sequence, head) pairs");
  train_wide_forward_kernel<io_t, D><<<(unsigned)blocks, kFwdCols*(D / 64), 0, stream>>>(
      sco, cs, ce, state, static_cast<const io_t*>(r), static_cast<const io_t*>(w), static_cast<const io_t*>(k),
      static_cast<const io_t*>(v), static_cast<const io_t*>(a), static_cast<const io_t*>(b), static_cast<io_t*>(y),
      boundary, sda, dense_checkpoints, dense_groups, num_heads, scale, status);
  return check_launch("train_wide_forward_kernel");
}

template <typename io_t, int D>
int launch_backward(const int* sco, const int* cs, const int* ce, const float* final_state, const float* boundary,
                    const float* sda, const void* r, const void* w, const void* k, const void* v, const void* a,
                    const void* b, const void* dy, const float* grad_final_state, void* dr, void* dw, void* dk, void* dv,
                    void* da, void* db, float* dS0, float* workspace, long long total_tokens, int num_sequences,
                    int num_chunks, int num_heads, float scale, const int* status, cudaStream_t stream) {
  const long long DD = (long long)D * D;
  const long long elements = total_tokens * num_heads * D;
  float* checkpoints = workspace;                                       // [Cn][3][H][D][D]
  float* partials = workspace + (long long)num_chunks * 3 * num_heads * DD;  // [5][D / 64][elements]
  const long long cp_blocks = (long long)num_chunks * num_heads * (D / kFwdCols);
  const long long bw_blocks = (long long)num_sequences * num_heads * (D / kBwdCols);
  if (cp_blocks > 0x7fffffffLL || bw_blocks > 0x7fffffffLL)
    return fail(FRWKV_ERR_INVALID_ARGUMENT, "wkv7_train_wide: too many (chunk, head) pairs");
  train_wide_checkpoints_kernel<io_t, D><<<(unsigned)cp_blocks, kFwdCols*(D / 64), 0, stream>>>(
      cs, ce, boundary, sda, static_cast<const io_t*>(w), static_cast<const io_t*>(k), static_cast<const io_t*>(v),
      static_cast<const io_t*>(b), checkpoints, num_heads, status);
  int rc = check_launch("train_wide_checkpoints_kernel");
  if (rc != FRWKV_OK) return rc;
  train_wide_backward_kernel<io_t, D><<<(unsigned)bw_blocks, D, 0, stream>>>(
      sco, cs, ce, final_state, boundary, checkpoints, sda, static_cast<const io_t*>(r), static_cast<const io_t*>(w),
      static_cast<const io_t*>(k), static_cast<const io_t*>(v), static_cast<const io_t*>(a),
      static_cast<const io_t*>(b), static_cast<const io_t*>(dy), grad_final_state, static_cast<io_t*>(dv), dS0, partials,
      elements, num_heads, scale, status);
  rc = check_launch("train_wide_backward_kernel");
  if (rc != FRWKV_OK) return rc;
  const long long want = (elements + 255) / 256;
  train_wide_reduce_kernel<io_t, D><<<(unsigned)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream>>>(
      partials, elements, static_cast<const io_t*>(w), static_cast<io_t*>(dr), static_cast<io_t*>(dw),
      static_cast<io_t*>(dk), static_cast<io_t*>(da), static_cast<io_t*>(db), status);
  return check_launch("train_wide_reduce_kernel");
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_wkv7_train_wide_forward(const int32_t* seq_chunk_offsets, const int32_t* chunk_starts,
                                             const int32_t* chunk_ends, float* state, const void* r,
                                             const void* decay_logits, const void* k, const void* v, const void* a,
                                             const void* b, void* y, float* boundary, float* state_dot_a,
                                             float* dense_checkpoints, int dense_groups,
                                             const int32_t* metadata_status, int num_sequences, int num_heads,
                                             int head_size, int io_dtype, float scale, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(seq_chunk_offsets && chunk_starts && chunk_ends && state && r && decay_logits && k && v && a && b && y,
                "wkv7_train_wide_forward: null pointer argument");
  FRWKV_REQUIRE(num_sequences > 0 && num_heads > 0, "wkv7_train_wide_forward: sizes must be positive");
  FRWKV_REQUIRE(dense_checkpoints == nullptr || dense_groups > 0, "wkv7_train_wide_forward: dense_groups must be positive");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define FRWKV_WF(T, DD)                                                                                               \
  return launch_forward<T, DD>(seq_chunk_offsets, chunk_starts, chunk_ends, state, r, decay_logits, k, v, a, b, y,    \
                               boundary, state_dot_a, dense_checkpoints, dense_groups, num_sequences, num_heads, scale,      \
                               metadata_status, s)
  if (io_dtype == FRWKV_DTYPE_BF16 && head_size == 128) FRWKV_WF(__nv_bfloat16, 128);
  if (io_dtype == FRWKV_DTYPE_BF16 && head_size == 256) FRWKV_WF(__nv_bfloat16, 256);
  if (io_dtype == FRWKV_DTYPE_FP16 && head_size == 128) FRWKV_WF(__half, 128);
  if (io_dtype == FRWKV_DTYPE_FP16 && head_size == 256) FRWKV_WF(__half, 256);
#undef FRWKV_WF
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_train_wide_forward: head size 128 or 256 and float16 / bfloat16 tokens only");
}

extern "C" size_t frwkv_wkv7_train_wide_workspace_floats(long long total_tokens, int num_chunks, int num_heads,
                                                         int head_size) {
  if (total_tokens <= 0 || num_chunks <= 0 || num_heads <= 0 || (head_size != 128 && head_size != 256)) return 0;
  const size_t dd = (size_t)head_size * head_size;
  return (size_t)num_chunks * 3 * num_heads * dd +
         (size_t)5 * (head_size / 64) * (size_t)total_tokens * num_heads * head_size;
}

extern "C" int frwkv_wkv7_train_wide_backward(
    const int32_t* seq_chunk_offsets, const int32_t* chunk_starts, const int32_t* chunk_ends, const float* final_state,
    const float* boundary, const float* state_dot_a, const void* r, const void* decay_logits, const void* k,
    const void* v, const void* a, const void* b, const void* grad_output, const float* grad_final_state, void* grad_r,
    void* grad_decay_logits, void* grad_k, void* grad_v, void* grad_a, void* grad_b, float* grad_initial_state,
    float* workspace, const int32_t* metadata_status, long long total_tokens, int num_sequences, int num_chunks,
    int num_heads, int head_size, int io_dtype, float scale, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(seq_chunk_offsets && chunk_starts && chunk_ends && final_state && boundary && state_dot_a && r &&
                    decay_logits && k && v && a && b && workspace,
                "wkv7_train_wide_backward: null pointer argument");
  FRWKV_REQUIRE(total_tokens > 0 && num_sequences > 0 && num_chunks > 0 && num_heads > 0,
                "wkv7_train_wide_backward: sizes must be positive");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define FRWKV_WB(T, DD)                                                                                                \
  return launch_backward<T, DD>(seq_chunk_offsets, chunk_starts, chunk_ends, final_state, boundary, state_dot_a, r,    \
                                decay_logits, k, v, a, b, grad_output, grad_final_state, grad_r, grad_decay_logits,    \
                                grad_k, grad_v, grad_a, grad_b, grad_initial_state, workspace, total_tokens,           \
                                num_sequences, num_chunks, num_heads, scale, metadata_status, s)
  if (io_dtype == FRWKV_DTYPE_BF16 && head_size == 128) FRWKV_WB(__nv_bfloat16, 128);
  if (io_dtype == FRWKV_DTYPE_BF16 && head_size == 256) FRWKV_WB(__nv_bfloat16, 256);
  if (io_dtype == FRWKV_DTYPE_FP16 && head_size == 128) FRWKV_WB(__half, 128);
  if (io_dtype == FRWKV_DTYPE_FP16 && head_size == 256) FRWKV_WB(__half, 256);
#undef FRWKV_WB
  return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_train_wide_backward: head size 128 or 256 and float16 / bfloat16 tokens only");
}
