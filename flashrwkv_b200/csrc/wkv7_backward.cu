// WKV7 backward: gradients of r, decay logits, k, v, a, b and of the initial state (head size 64).
//
// One CTA of 64 threads per (sequence, head) walks the tokens in reverse.  The state S and the adjoint G = dL/dS
// (both 64 x 64, key row x value column) live in registers as 4 x 16 tiles: thread (rg, cg) = (tid / 4, tid % 4) owns
// rows 4 rg .. 4 rg + 3 and the columns 16 q + 4 cg + e (q, e = 0..3) of both.  (Measured: 4 x 8 tiles on 128 threads
// hide latency better but execute 1.7 times the instructions per token, the reductions and the per-row set-up being
// paid per warp, and come out slower.)  Per token
//     G   += scale r (x) dy
//     dr[k] = scale S_t[k,:].dy      dk[k] = G[k,:].v      db[k] = G[k,:].sa             (row sums)
//     dv[v] = G[:,v].k               dsa[v] = G[:,v].b                                   (column sums)
//     S_{t-1}[k,:] = (S_t[k,:] - k[k] v - b[k] sa) / w[k]
//     dw[k] = G[k,:].S_{t-1}[k,:]    dlogit[k] = dw[k] w[k] dlog(w)/dx                   da[k] = S_{t-1}[k,:].dsa
//     G    = diag(w) G + a (x) dsa
// Row sums finish with two shuffles over the four column groups (adjacent lanes); column sums go through a
// 16 x 64 table of partials in shared memory that thread v adds up.  A shared-memory read of a token vector feeds
// 4 (column vectors) to 16 (row vectors) multiply-adds per element, which keeps the kernel bound by the FMA pipe
// rather than by shared-memory bandwidth, and one copy of G serves both orientations.  The 16-bit token vectors and
// sa are copied to shared memory as they are with cp.async, two tokens ahead of their use (three slots), so that no
// register holds data in flight and global latency stays off the per-token chain.
//
// The state is walked backwards by undoing the update, which amplifies rounding by 1/w per step, so it is
// re-anchored from saved states at least every 16 tokens: the chunk-start boundaries of the forward pass, the
// final state, and the 16-token checkpoints written by the replay kernel; sa = S_{t-1}^T a comes from the
// replay kernel as well (state_dot_a).
//
// Replaces backward_kernel_preload (csrc/sm90/tmix/wkv7/pretrain_recurrent_bf16_forward.cu:163-291) and
// statetune_recurrent_fp32io16_backward_kernel (csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_backward.cu:49-255)
// of the reference.

#include "frwkv_common.cuh"
#include "umma.cuh"

namespace frwkv {
namespace {

constexpr int kD = 64;

constexpr int kTR = 4;   // rows of a thread's tile
constexpr int kTC = 16;  // columns of a thread's tile
constexpr int kCG = kD / kTC;  // column groups (lanes that share a row group)
constexpr int kBwdThreads = (kD / kTR) * kCG;  // 64

// one token as it lies in global memory: seven 16-bit vectors and the fp32 sa = S_{t-1}^T a
template <typename io_t>
struct __align__(16) RawToken {
  io_t vec[7][kD];  // r, decay logit, k, v, a, b, dy
  float sa[kD];
};
enum { kVecR = 0, kVecX = 1, kVecK = 2, kVecV = 3, kVecA = 4, kVecB = 5, kVecDy = 6 };

// walks the tokens of one sequence backwards through its chunk table (empty chunks are skipped)
struct TokenCursor {
  int c, t, t0, len;
  bool valid;
};

// packed fp32 pairs: one fma.rn.f32x2 does two multiply-adds per issue slot
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 dup(float x) { return make_float2(x, x); }

__device__ __forceinline__ float group_sum(float x) {  // over the kCG adjacent lanes of a row group
#pragma unroll
  for (int m = 1; m < kCG; m <<= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
  return x;
}
__device__ __forceinline__ void ld4f(float (&d)[4], const float* p) {
  const float4 q = *reinterpret_cast<const float4*>(p);
  d[0] = q.x; d[1] = q.y; d[2] = q.z; d[3] = q.w;
}
__device__ __forceinline__ void ld4p(float2 (&d)[2], const float* p) {  // four floats as two pairs
  const float4 q = *reinterpret_cast<const float4*>(p);
  d[0] = make_float2(q.x, q.y); d[1] = make_float2(q.z, q.w);
}

template <typename io_t>
__device__ __forceinline__ void ld4h(float (&d)[4], const io_t* p) {  // four consecutive 16-bit values
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 lo = Io16<io_t>::unpack(u.x), hi = Io16<io_t>::unpack(u.y);
  d[0] = lo.x; d[1] = lo.y; d[2] = hi.x; d[3] = hi.y;
}

template <typename io_t>
__device__ __forceinline__ void ld4hp(float2 (&d)[2], const io_t* p) {  // four 16-bit values as two fp32 pairs
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  d[0] = Io16<io_t>::unpack(u.x); d[1] = Io16<io_t>::unpack(u.y);
}

template <typename io_t>
__device__ __forceinline__ void store_rows4(io_t* base, const float (&x)[4]) {
  using IO = Io16<io_t>;
  *reinterpret_cast<uint2*>(base) = make_uint2(IO::pack(x[0], x[1]), IO::pack(x[2], x[3]));
}

template <typename io_t>
__global__ __launch_bounds__(kBwdThreads, 4) void wkv7_backward_kernel(
    const int* __restrict__ seq_chunk_offsets, const int* __restrict__ chunk_starts, const int* __restrict__ chunk_ends,
    const float* __restrict__ final_state, const float* __restrict__ boundary, const float* __restrict__ checkpoints,
    const float* __restrict__ state_dot_a, const io_t* __restrict__ r_ptr, const io_t* __restrict__ w_ptr,
    const io_t* __restrict__ k_ptr, const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr,
    const io_t* __restrict__ b_ptr, const io_t* __restrict__ dy_ptr, const float* __restrict__ grad_final_state,
    io_t* __restrict__ dr_ptr, io_t* __restrict__ dw_ptr, io_t* __restrict__ dk_ptr, io_t* __restrict__ dv_ptr,
    io_t* __restrict__ da_ptr, io_t* __restrict__ db_ptr, float* __restrict__ dS0_ptr, int num_heads, float scale) {
  using IO = Io16<io_t>;
  __shared__ RawToken<io_t> raw[3];
  __shared__ __align__(16) float w_s[kD];            // retention of the current token
  __shared__ __align__(16) float part_dv[16][kD + 4];   // column-sum partials, one row per row group (padded: the
  __shared__ __align__(16) float part_dsa[16][kD + 4];  // 16-byte writes of a warp then spread over all banks)
  __shared__ __align__(16) float dsa_s[kD];
  const int j = threadIdx.x;
  const int rg = j / kCG, cg = j % kCG, row0 = kTR * rg;
  static_assert(kBwdThreads / kCG * kTR == kD && kCG * kTC == kD, "the thread tiles must cover the 64 x 64 state");
  // tile column c4 + e (c4 = 0, 4, ...) is matrix column colb + kCG * c4 + e: the column groups interleave in 16-byte
  // units, so the lanes of a row group read contiguous bytes of a token vector (no bank conflicts)
  const int colb = 4 * cg;
  const int seq = blockIdx.x / num_heads, head = blockIdx.x % num_heads;
  const int c_begin = seq_chunk_offsets[seq], c_end = seq_chunk_offsets[seq + 1];
  const long long sh = ((long long)seq * num_heads + head) * (kD * kD);

  // ---- token cursor and the cp.async staging ------------------------------------------------------------------
  const auto settle = [&](TokenCursor& u) {  // make u point at the last token of chunk u.c or of an earlier one
    u.valid = false;
    while (u.c >= c_begin) {
      u.t0 = chunk_starts[u.c];
      u.len = chunk_ends[u.c] - u.t0;
      if (u.len > 0) { u.t = u.t0 + u.len - 1; u.valid = true; return; }
      --u.c;
    }
  };
  const auto retreat = [&](TokenCursor& u) {
    if (!u.valid) return;
    if (u.t > u.t0) { --u.t; return; }
    --u.c;
    settle(u);
  };
  // a token is 72 pieces of 16 bytes: 8 for each of the seven 16-bit vectors, then 16 of sa.  Thread j copies piece j
  // and, when there are fewer than 72 threads, piece j + kBwdThreads (always a piece of sa).
  static_assert(kBwdThreads >= 56 && 2 * kBwdThreads >= 72, "the second piece of a thread must be one of sa");
  const io_t* first_src = nullptr;  // source vector of the first piece (nullptr: sa, or a missing grad_output)
  switch (j >> 3) {
    case kVecR: first_src = r_ptr; break;
    case kVecX: first_src = w_ptr; break;
    case kVecK: first_src = k_ptr; break;
    case kVecV: first_src = v_ptr; break;
    case kVecA: first_src = a_ptr; break;
    case kVecB: first_src = b_ptr; break;
    case kVecDy: first_src = dy_ptr; break;
    default: break;
  }
  const auto stage = [&](const TokenCursor& u, int slot) {  // always commits a group, possibly an empty one
    if (u.valid) {
      const long long off = ((long long)u.t * num_heads + head) * kD;
      if (j < 56) {
        // a missing grad_output reads as zeros (source size 0 zero-fills the destination)
        const io_t* src = first_src != nullptr ? first_src + off + 8 * (j & 7) : r_ptr;
        umma::cp_async16(umma::smem_u32(&raw[slot].vec[j >> 3][8 * (j & 7)]), src, first_src != nullptr ? 16u : 0u);
      } else if (j < 72) {
        umma::cp_async16(umma::smem_u32(&raw[slot].sa[4 * (j - 56)]), state_dot_a + off + 4 * (j - 56), 16u);
      }
      if (j + kBwdThreads >= 56 && j + kBwdThreads < 72)
        umma::cp_async16(umma::smem_u32(&raw[slot].sa[4 * (j + kBwdThreads - 56)]),
                         state_dot_a + off + 4 * (j + kBwdThreads - 56), 16u);
    }
    umma::cp_async_commit();
  };

  // tiles as fp32 pairs along the columns: pair index 2 * (c4 / 4) + {0, 1} holds tile columns c4 + {0,1} | {2,3}
  float2 S[kTR][kTC / 2], G[kTR][kTC / 2];
#pragma unroll
  for (int rr = 0; rr < kTR; ++rr) {
#pragma unroll
    for (int c4 = 0; c4 < kTC; c4 += 4) {
      if (grad_final_state != nullptr) {
        ld4p(*reinterpret_cast<float2(*)[2]>(&G[rr][c4 / 2]), grad_final_state + sh + (row0 + rr) * kD + colb + kCG * c4);
      } else {
        G[rr][c4 / 2] = make_float2(0.f, 0.f); G[rr][c4 / 2 + 1] = make_float2(0.f, 0.f);
      }
    }
  }

  TokenCursor cur{c_end - 1, 0, 0, 0, false}, ahead;
  settle(cur);
  ahead = cur;
  stage(ahead, 0);
  retreat(ahead);
  stage(ahead, 1);
  int slot = 0;
  for (; cur.valid; retreat(cur), slot = slot == 2 ? 0 : slot + 1) {
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // this token's pieces (the next token's may be in flight)
    const int t = cur.t, c = cur.c, rel = t - cur.t0;
    if (rel == cur.len - 1 || (rel & 15) == 15) {
      // last token of a group of <= 16: re-anchor S on the saved state that follows it
      const int q = rel >> 4;
      const float* anchor;
      if (16 * (q + 1) < cur.len) anchor = checkpoints + (((long long)c * 3 + q) * num_heads + head) * (kD * kD);
      else if (c + 1 < c_end) anchor = boundary + ((long long)(c + 1) * num_heads + head) * (kD * kD);
      else anchor = final_state + sh;
#pragma unroll
      for (int rr = 0; rr < kTR; ++rr) {
#pragma unroll
        for (int c4 = 0; c4 < kTC; c4 += 4)
          ld4p(*reinterpret_cast<float2(*)[2]>(&S[rr][c4 / 2]), anchor + (row0 + rr) * kD + colb + kCG * c4);
      }
    }
    const long long tok_off = ((long long)t * num_heads + head) * kD;
    const RawToken<io_t>& ts = raw[slot];
    __syncthreads();  // every thread's pieces of this token have landed; the previous token is done with,
    retreat(ahead);   // so its slot takes the token two steps ahead
    stage(ahead, slot == 0 ? 2 : slot - 1);
    for (int i = j; i < kD; i += kBwdThreads) w_s[i] = retention(IO::load(&ts.vec[kVecX][i]));
    // ---- phase 1: G += scale r (x) dy, then every sum that uses G_t and S_t -------------------------------
    float rs[kTR], kr[kTR], br[kTR];
    ld4h<io_t>(rs, &ts.vec[kVecR][row0]); ld4h<io_t>(kr, &ts.vec[kVecK][row0]); ld4h<io_t>(br, &ts.vec[kVecB][row0]);
    float2 rs2[kTR], kr2[kTR], br2[kTR], dr2[kTR], dk2[kTR], db2[kTR];
#pragma unroll
    for (int rr = 0; rr < kTR; ++rr) {
      rs2[rr] = dup(rs[rr] * scale); kr2[rr] = dup(kr[rr]); br2[rr] = dup(br[rr]);
      dr2[rr] = dup(0.f); dk2[rr] = dup(0.f); db2[rr] = dup(0.f);
    }
#pragma unroll
    for (int c4 = 0; c4 < kTC; c4 += 4) {
      float2 dy2[2], v2[2], sa2[2], dvp[2], dsap[2];
      ld4hp<io_t>(dy2, &ts.vec[kVecDy][colb + kCG * c4]); ld4hp<io_t>(v2, &ts.vec[kVecV][colb + kCG * c4]);
      ld4p(sa2, ts.sa + colb + kCG * c4);
      dvp[0] = dup(0.f); dvp[1] = dup(0.f); dsap[0] = dup(0.f); dsap[1] = dup(0.f);
#pragma unroll
      for (int rr = 0; rr < kTR; ++rr) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float2 g = fma2(rs2[rr], dy2[h], G[rr][c4 / 2 + h]);
          G[rr][c4 / 2 + h] = g;
          dr2[rr] = fma2(S[rr][c4 / 2 + h], dy2[h], dr2[rr]);
          dk2[rr] = fma2(g, v2[h], dk2[rr]);
          db2[rr] = fma2(g, sa2[h], db2[rr]);
          dvp[h] = fma2(g, kr2[rr], dvp[h]);
          dsap[h] = fma2(g, br2[rr], dsap[h]);
        }
      }
      *reinterpret_cast<float4*>(&part_dv[rg][colb + kCG * c4]) = make_float4(dvp[0].x, dvp[0].y, dvp[1].x, dvp[1].y);
      *reinterpret_cast<float4*>(&part_dsa[rg][colb + kCG * c4]) = make_float4(dsap[0].x, dsap[0].y, dsap[1].x, dsap[1].y);
    }
    float dr[kTR], dk[kTR], db[kTR];
#pragma unroll
    for (int rr = 0; rr < kTR; ++rr) {
      dr[rr] = scale * group_sum(dr2[rr].x + dr2[rr].y);
      dk[rr] = group_sum(dk2[rr].x + dk2[rr].y);
      db[rr] = group_sum(db2[rr].x + db2[rr].y);
    }
    if (cg == 0) {
      if (dr_ptr != nullptr) store_rows4<io_t>(dr_ptr + tok_off + row0, dr);
      if (dk_ptr != nullptr) store_rows4<io_t>(dk_ptr + tok_off + row0, dk);
      if (db_ptr != nullptr) store_rows4<io_t>(db_ptr + tok_off + row0, db);
    }
    __syncthreads();
    // ---- column sums: the 16 partials of dsa (idx < 64) and of dv (idx >= 64) for each column -------------------
#pragma unroll
    for (int idx = j; idx < 2 * kD; idx += kBwdThreads) {
      const int col = idx & (kD - 1);
      const float(*part)[kD + 4] = idx < kD ? part_dsa : part_dv;
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int g = 0; g < 16; g += 4) {
        s0 += part[g][col]; s1 += part[g + 1][col]; s2 += part[g + 2][col]; s3 += part[g + 3][col];
      }
      const float total = (s0 + s1) + (s2 + s3);
      if (idx < kD) dsa_s[col] = total;
      else if (dv_ptr != nullptr) dv_ptr[tok_off + col] = IO::store(total);
    }
    __syncthreads();
    // ---- phase 2: undo the state update, the sums that use S_{t-1}, then the adjoint step ------------------
    float wr[kTR], ar[kTR];
    ld4f(wr, w_s + row0); ld4h<io_t>(ar, &ts.vec[kVecA][row0]);
    float2 wr2[kTR], ar2[kTR], iw2[kTR], nk2[kTR], nb2[kTR], dw2[kTR], da2[kTR];
#pragma unroll
    for (int rr = 0; rr < kTR; ++rr) {
      wr2[rr] = dup(wr[rr]); ar2[rr] = dup(ar[rr]); iw2[rr] = dup(1.f / wr[rr]);
      nk2[rr] = dup(-kr[rr]); nb2[rr] = dup(-br[rr]);
      dw2[rr] = dup(0.f); da2[rr] = dup(0.f);
    }
#pragma unroll
    for (int c4 = 0; c4 < kTC; c4 += 4) {
      float2 v2[2], sa2[2], d2[2];
      ld4hp<io_t>(v2, &ts.vec[kVecV][colb + kCG * c4]); ld4p(sa2, ts.sa + colb + kCG * c4); ld4p(d2, dsa_s + colb + kCG * c4);
#pragma unroll
      for (int rr = 0; rr < kTR; ++rr) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float2 sp = mul2(fma2(nb2[rr], sa2[h], fma2(nk2[rr], v2[h], S[rr][c4 / 2 + h])), iw2[rr]);
          S[rr][c4 / 2 + h] = sp;
          dw2[rr] = fma2(G[rr][c4 / 2 + h], sp, dw2[rr]);
          da2[rr] = fma2(sp, d2[h], da2[rr]);
          G[rr][c4 / 2 + h] = fma2(wr2[rr], G[rr][c4 / 2 + h], mul2(ar2[rr], d2[h]));
        }
      }
    }
    float dw[kTR], da[kTR];
#pragma unroll
    for (int rr = 0; rr < kTR; ++rr) { dw[rr] = group_sum(dw2[rr].x + dw2[rr].y); da[rr] = group_sum(da2[rr].x + da2[rr].y); }
    if (cg == 0) {
      if (da_ptr != nullptr) store_rows4<io_t>(da_ptr + tok_off + row0, da);
      if (dw_ptr != nullptr) {
        float xr[kTR];
        ld4h<io_t>(xr, &ts.vec[kVecX][row0]);
#pragma unroll
        for (int rr = 0; rr < kTR; ++rr) dw[rr] *= wr[rr] * retention_log_derivative(xr[rr]);
        store_rows4<io_t>(dw_ptr + tok_off + row0, dw);
      }
    }
    // Hazards.  raw[slot] is refilled after the first barrier of the next iteration, which every thread passes only
    // when it is done with this token; w_s, the partial tables and dsa_s are rewritten after that same barrier.
  }
  umma::cp_async_wait_all();
  if (dS0_ptr != nullptr) {
#pragma unroll
    for (int rr = 0; rr < kTR; ++rr) {
#pragma unroll
      for (int c4 = 0; c4 < kTC; c4 += 4)
        *reinterpret_cast<float4*>(dS0_ptr + sh + (row0 + rr) * kD + colb + kCG * c4) =
            make_float4(G[rr][c4 / 2].x, G[rr][c4 / 2].y, G[rr][c4 / 2 + 1].x, G[rr][c4 / 2 + 1].y);
    }
  }
}

}  // namespace
}  // namespace frwkv

extern "C" int frwkv_wkv7_backward(const int32_t* seq_chunk_offsets, const int32_t* chunk_starts,
                                   const int32_t* chunk_ends, const float* final_state, const float* boundary,
                                   const float* checkpoints, const float* state_dot_a, const void* r,
                                   const void* decay_logits, const void* k, const void* v, const void* a, const void* b,
                                   const void* grad_output, const float* grad_final_state, void* grad_r,
                                   void* grad_decay_logits, void* grad_k, void* grad_v, void* grad_a, void* grad_b,
                                   float* grad_initial_state, int num_sequences, int num_heads, int head_size,
                                   int io_dtype, float scale, frwkv_stream_t stream) {
  using namespace frwkv;
  clear_error();
  FRWKV_REQUIRE(seq_chunk_offsets && chunk_starts && chunk_ends && final_state && boundary && checkpoints &&
                    state_dot_a && r && decay_logits && k && v && a && b,
                "wkv7_backward: null pointer argument");
  FRWKV_REQUIRE(num_sequences > 0 && num_heads > 0, "wkv7_backward: sizes must be positive");
  if (head_size != 64) return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_backward: head size %d is not built (only 64)", head_size);
  FRWKV_REQUIRE((long long)num_sequences * num_heads <= 0x7fffffffLL, "wkv7_backward: too many (sequence, head) pairs");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)(num_sequences * num_heads);
#define FRWKV_BWD(T)                                                                                               \
  wkv7_backward_kernel<T><<<grid, kBwdThreads, 0, s>>>(                                                                     \
      seq_chunk_offsets, chunk_starts, chunk_ends, final_state, boundary, checkpoints, state_dot_a,                \
      static_cast<const T*>(r), static_cast<const T*>(decay_logits), static_cast<const T*>(k),                     \
      static_cast<const T*>(v), static_cast<const T*>(a), static_cast<const T*>(b),                                \
      static_cast<const T*>(grad_output), grad_final_state, static_cast<T*>(grad_r), static_cast<T*>(grad_decay_logits), \
      static_cast<T*>(grad_k), static_cast<T*>(grad_v), static_cast<T*>(grad_a), static_cast<T*>(grad_b),          \
      grad_initial_state, num_heads, scale)
  if (io_dtype == FRWKV_DTYPE_BF16) {
    FRWKV_BWD(__nv_bfloat16);
  } else if (io_dtype == FRWKV_DTYPE_FP16) {
    FRWKV_BWD(__half);
  } else {
    return fail(FRWKV_ERR_UNSUPPORTED, "wkv7_backward: token tensors must be float16 or bfloat16");
  }
#undef FRWKV_BWD
  return check_launch("wkv7_backward_kernel");
}
