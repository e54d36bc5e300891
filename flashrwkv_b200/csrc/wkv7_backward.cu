// WKV7 backward: gradients of r, decay logits, k, v, a, b and of the initial state (head size 64).
//
// One CTA of 64 threads per (sequence, head) walks the tokens in reverse.  Thread j keeps three 64-vectors in
// registers: row j of the state S, row j of the adjoint G = dL/dS, and column j of G.  With both orientations of G
// at hand every reduction of the adjoint equations is private to one thread:
//     G   += scale r (x) dy
//     dr[j] = scale S_t[j,:].dy      dk[j] = G[j,:].v      db[j] = G[j,:].sa             (rows)
//     dv[j] = G[:,j].k               dsa[j] = G[:,j].b                                   (columns)
//     S_{t-1}[j,:] = (S_t[j,:] - k[j] v - b[j] sa) / w[j]
//     dw[j] = G[j,:].S_{t-1}[j,:]    dlogit[j] = dw[j] w[j] dlog(w)/dx                   da[j] = S_{t-1}[j,:].dsa
//     G    = diag(w) G + a (x) dsa
// and only the 64-vector dsa crosses threads (through shared memory, one barrier).  Per-token vectors are staged
// in double-buffered shared memory one token ahead.
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

namespace frwkv {
namespace {

constexpr int kD = 64;

struct TokenRegs {
  float r, x, k, v, a, b, dy, sa;
};

template <typename io_t>
__device__ __forceinline__ TokenRegs load_token(const io_t* r, const io_t* w, const io_t* k, const io_t* v,
                                                const io_t* a, const io_t* b, const io_t* dy, const float* sa,
                                                long long off) {
  using IO = Io16<io_t>;
  TokenRegs t;
  t.r = IO::load(r + off); t.x = IO::load(w + off); t.k = IO::load(k + off); t.v = IO::load(v + off);
  t.a = IO::load(a + off); t.b = IO::load(b + off);
  t.dy = dy != nullptr ? IO::load(dy + off) : 0.f;
  t.sa = sa[off];
  return t;
}

// shared vectors of one token: r, w, k, v, a, b, dy, sa (each 64 floats)
struct __align__(16) TokenSmem {
  float r[kD], w[kD], k[kD], v[kD], a[kD], b[kD], dy[kD], sa[kD];
};

__device__ __forceinline__ float dot64(const float (&x)[kD], const float* __restrict__ vec) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
  for (int i = 0; i < kD; i += 4) {
    const float4 q = *reinterpret_cast<const float4*>(vec + i);
    a0 = fmaf(x[i], q.x, a0); a1 = fmaf(x[i + 1], q.y, a1); a2 = fmaf(x[i + 2], q.z, a2); a3 = fmaf(x[i + 3], q.w, a3);
  }
  return (a0 + a1) + (a2 + a3);
}

template <typename io_t>
__global__ __launch_bounds__(64, 4) void wkv7_backward_kernel(
    const int* __restrict__ seq_chunk_offsets, const int* __restrict__ chunk_starts, const int* __restrict__ chunk_ends,
    const float* __restrict__ final_state, const float* __restrict__ boundary, const float* __restrict__ checkpoints,
    const float* __restrict__ state_dot_a, const io_t* __restrict__ r_ptr, const io_t* __restrict__ w_ptr,
    const io_t* __restrict__ k_ptr, const io_t* __restrict__ v_ptr, const io_t* __restrict__ a_ptr,
    const io_t* __restrict__ b_ptr, const io_t* __restrict__ dy_ptr, const float* __restrict__ grad_final_state,
    io_t* __restrict__ dr_ptr, io_t* __restrict__ dw_ptr, io_t* __restrict__ dk_ptr, io_t* __restrict__ dv_ptr,
    io_t* __restrict__ da_ptr, io_t* __restrict__ db_ptr, float* __restrict__ dS0_ptr, int num_heads, float scale) {
  using IO = Io16<io_t>;
  __shared__ TokenSmem tok[2];
  __shared__ __align__(16) float dsa_s[kD];
  const int j = threadIdx.x;
  const int seq = blockIdx.x / num_heads, head = blockIdx.x % num_heads;
  const int c_begin = seq_chunk_offsets[seq], c_end = seq_chunk_offsets[seq + 1];
  const long long sh = ((long long)seq * num_heads + head) * (kD * kD);

  float Srow[kD], Grow[kD], Gcol[kD];
  if (grad_final_state != nullptr) {
#pragma unroll
    for (int i = 0; i < kD; i += 4) {
      const float4 q = *reinterpret_cast<const float4*>(grad_final_state + sh + j * kD + i);
      Grow[i] = q.x; Grow[i + 1] = q.y; Grow[i + 2] = q.z; Grow[i + 3] = q.w;
    }
#pragma unroll
    for (int i = 0; i < kD; ++i) Gcol[i] = grad_final_state[sh + i * kD + j];
  } else {
#pragma unroll
    for (int i = 0; i < kD; ++i) { Grow[i] = 0.f; Gcol[i] = 0.f; }
  }

  for (int c = c_end - 1; c >= c_begin; --c) {
    const int t0 = chunk_starts[c];
    const int len = chunk_ends[c] - t0;
    for (int q = (len - 1) >> 4; q >= 0; --q) {
      const int sub_begin = t0 + 16 * q;
      const int sub_end = min(sub_begin + 16, t0 + len);
      // state after the last token of this group of <= 16 tokens
      const float* anchor;
      if (16 * (q + 1) < len) anchor = checkpoints + (((long long)c * 3 + q) * num_heads + head) * (kD * kD);
      else if (c + 1 < c_end) anchor = boundary + ((long long)(c + 1) * num_heads + head) * (kD * kD);
      else anchor = final_state + sh;
#pragma unroll
      for (int i = 0; i < kD; i += 4) {
        const float4 s4 = *reinterpret_cast<const float4*>(anchor + j * kD + i);
        Srow[i] = s4.x; Srow[i + 1] = s4.y; Srow[i + 2] = s4.z; Srow[i + 3] = s4.w;
      }
      TokenRegs cur = load_token<io_t>(r_ptr, w_ptr, k_ptr, v_ptr, a_ptr, b_ptr, dy_ptr, state_dot_a,
                                       ((long long)(sub_end - 1) * num_heads + head) * kD + j);
      for (int t = sub_end - 1; t >= sub_begin; --t) {
        const long long off = ((long long)t * num_heads + head) * kD + j;
        TokenSmem& ts = tok[t & 1];
        const float wj = retention(cur.x);
        ts.r[j] = cur.r; ts.w[j] = wj; ts.k[j] = cur.k; ts.v[j] = cur.v;
        ts.a[j] = cur.a; ts.b[j] = cur.b; ts.dy[j] = cur.dy; ts.sa[j] = cur.sa;
        const TokenRegs me = cur;
        if (t > sub_begin) cur = load_token<io_t>(r_ptr, w_ptr, k_ptr, v_ptr, a_ptr, b_ptr, dy_ptr, state_dot_a, off - (long long)num_heads * kD);
        __syncthreads();
        // G += scale r (x) dy  (both orientations), then the reductions that use G_t and S_t
        const float srj = scale * me.r, sdyj = scale * me.dy;
        float dr = 0.f, dk = 0.f, db = 0.f, dv = 0.f, dsa = 0.f;
#pragma unroll
        for (int i = 0; i < kD; i += 4) {
          const float4 dy4 = *reinterpret_cast<const float4*>(ts.dy + i);
          const float4 r4 = *reinterpret_cast<const float4*>(ts.r + i);
          const float4 v4 = *reinterpret_cast<const float4*>(ts.v + i);
          const float4 sa4 = *reinterpret_cast<const float4*>(ts.sa + i);
          const float4 k4 = *reinterpret_cast<const float4*>(ts.k + i);
          const float4 b4 = *reinterpret_cast<const float4*>(ts.b + i);
          Grow[i] = fmaf(srj, dy4.x, Grow[i]); Grow[i + 1] = fmaf(srj, dy4.y, Grow[i + 1]);
          Grow[i + 2] = fmaf(srj, dy4.z, Grow[i + 2]); Grow[i + 3] = fmaf(srj, dy4.w, Grow[i + 3]);
          Gcol[i] = fmaf(r4.x, sdyj, Gcol[i]); Gcol[i + 1] = fmaf(r4.y, sdyj, Gcol[i + 1]);
          Gcol[i + 2] = fmaf(r4.z, sdyj, Gcol[i + 2]); Gcol[i + 3] = fmaf(r4.w, sdyj, Gcol[i + 3]);
          dr = fmaf(Srow[i], dy4.x, fmaf(Srow[i + 1], dy4.y, fmaf(Srow[i + 2], dy4.z, fmaf(Srow[i + 3], dy4.w, dr))));
          dk = fmaf(Grow[i], v4.x, fmaf(Grow[i + 1], v4.y, fmaf(Grow[i + 2], v4.z, fmaf(Grow[i + 3], v4.w, dk))));
          db = fmaf(Grow[i], sa4.x, fmaf(Grow[i + 1], sa4.y, fmaf(Grow[i + 2], sa4.z, fmaf(Grow[i + 3], sa4.w, db))));
          dv = fmaf(Gcol[i], k4.x, fmaf(Gcol[i + 1], k4.y, fmaf(Gcol[i + 2], k4.z, fmaf(Gcol[i + 3], k4.w, dv))));
          dsa = fmaf(Gcol[i], b4.x, fmaf(Gcol[i + 1], b4.y, fmaf(Gcol[i + 2], b4.z, fmaf(Gcol[i + 3], b4.w, dsa))));
        }
        dsa_s[j] = dsa;
        __syncthreads();
        // undo the state update for row j, then the reductions that use S_{t-1}, then the adjoint step
        const float inv_w = 1.f / wj;
        float dw = 0.f, da = 0.f;
#pragma unroll
        for (int i = 0; i < kD; i += 4) {
          const float4 v4 = *reinterpret_cast<const float4*>(ts.v + i);
          const float4 sa4 = *reinterpret_cast<const float4*>(ts.sa + i);
          const float4 d4 = *reinterpret_cast<const float4*>(dsa_s + i);
          const float4 w4 = *reinterpret_cast<const float4*>(ts.w + i);
          const float4 a4 = *reinterpret_cast<const float4*>(ts.a + i);
          Srow[i] = (Srow[i] - me.k * v4.x - me.b * sa4.x) * inv_w;
          Srow[i + 1] = (Srow[i + 1] - me.k * v4.y - me.b * sa4.y) * inv_w;
          Srow[i + 2] = (Srow[i + 2] - me.k * v4.z - me.b * sa4.z) * inv_w;
          Srow[i + 3] = (Srow[i + 3] - me.k * v4.w - me.b * sa4.w) * inv_w;
          dw = fmaf(Grow[i], Srow[i], fmaf(Grow[i + 1], Srow[i + 1], fmaf(Grow[i + 2], Srow[i + 2], fmaf(Grow[i + 3], Srow[i + 3], dw))));
          da = fmaf(Srow[i], d4.x, fmaf(Srow[i + 1], d4.y, fmaf(Srow[i + 2], d4.z, fmaf(Srow[i + 3], d4.w, da))));
          Grow[i] = fmaf(wj, Grow[i], me.a * d4.x); Grow[i + 1] = fmaf(wj, Grow[i + 1], me.a * d4.y);
          Grow[i + 2] = fmaf(wj, Grow[i + 2], me.a * d4.z); Grow[i + 3] = fmaf(wj, Grow[i + 3], me.a * d4.w);
          Gcol[i] = fmaf(w4.x, Gcol[i], a4.x * dsa); Gcol[i + 1] = fmaf(w4.y, Gcol[i + 1], a4.y * dsa);
          Gcol[i + 2] = fmaf(w4.z, Gcol[i + 2], a4.z * dsa); Gcol[i + 3] = fmaf(w4.w, Gcol[i + 3], a4.w * dsa);
        }
        if (dr_ptr != nullptr) dr_ptr[off] = IO::store(scale * dr);
        if (dk_ptr != nullptr) dk_ptr[off] = IO::store(dk);
        if (db_ptr != nullptr) db_ptr[off] = IO::store(db);
        if (dv_ptr != nullptr) dv_ptr[off] = IO::store(dv);
        if (da_ptr != nullptr) da_ptr[off] = IO::store(da);
        if (dw_ptr != nullptr) dw_ptr[off] = IO::store(dw * wj * retention_log_derivative(me.x));
        // tok[t & 1] and dsa_s are rewritten two / one tokens later, each time behind a barrier
      }
    }
  }
  if (dS0_ptr != nullptr) {
#pragma unroll
    for (int i = 0; i < kD; i += 4)
      *reinterpret_cast<float4*>(dS0_ptr + sh + j * kD + i) = make_float4(Grow[i], Grow[i + 1], Grow[i + 2], Grow[i + 3]);
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
  wkv7_backward_kernel<T><<<grid, 64, 0, s>>>(                                                                     \
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
