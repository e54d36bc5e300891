/*
 * CPU oracle for the RWKV-7 WKV7 time-mix path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic that the FlashRWKV2 reference
 * pins with its own pure-PyTorch test oracles.  It is the checker for the CUDA
 * kernels of this repository and the timed CPU baseline; it is never part of
 * the product path (only tests/, the smoke check and the benchmark's CPU
 * baseline may load it).
 *
 * Parity is pinned: tests/golden/ holds vectors produced by the reference's own
 * oracles, and tests/test_oracle_golden.py checks every function below against
 * them.
 *
 * Reference locations restated here (paths inside the reference project):
 *   retention transform   csrc/sm120/tmix/wkv7/recurrent_decay.cuh:10-32
 *   forward recurrence    tests/tmix/wkv7/test.py:157-213
 *   fp16-state recurrence tests/tmix/wkv7/test.py:216-277 (rounded retention increment, dither, elapsed phase)
 *                         tests/tmix/wkv7/statetune/test.py:39-87 (boundaries, state_dot_a)
 *   backward (adjoint)    csrc/sm90/tmix/wkv7/statetune_recurrent_fp32io16_backward.cu:139-254
 *                         (checked here against autograd of the forward oracle)
 *   mix6                  tests/tmix/mix6/test.py:231-278
 *   kk_a_gate             tests/tmix/kk_a_gate/test.py:52-74
 *   lnx_rkvres_xg         tests/tmix/lnx_rkvres_xg/test.py:36-66
 *   vres_gate             tests/tmix/vres_gate/test.py:15-26
 *
 * State convention: S[k][v] (key row, value column), per (sequence, head),
 * stored [slot][H][D][D] row-major.  Token tensors are packed [N][H][D] fp32
 * (callers upcast 16-bit inputs once, so the oracle sees exactly the rounded
 * values the kernels see).
 *
 * acc_t selects the accumulation type: the *_f32 entry points accumulate in
 * float like the reference kernels, the *_f64 ones in double for a tighter
 * truth.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define DECAY_RATE 0.6065306597126334 /* exp(-0.5) */

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* w = exp(-exp(-0.5) * sigmoid(x))   (recurrent_decay.cuh:18-22 in exp2 form) */
static inline double retention_d(double x) {
  return exp(-DECAY_RATE / (1.0 + exp(-x)));
}
static inline float retention_f(float x) {
  return expf(-(float)DECAY_RATE / (1.0f + expf(-x)));
}
/* d log(w) / dx = -exp(-0.5) * s * (1 - s)   (recurrent_decay.cuh:27-32) */
static inline double retention_dlog_d(double x) {
  double s = 1.0 / (1.0 + exp(-x));
  return -DECAY_RATE * s * (1.0 - s);
}

void oracle_retention_f32(const float* x, float* w, int64_t n) {
  for (int64_t i = 0; i < n; ++i) w[i] = retention_f(x[i]);
}

/* ------------------------------------------------------------------------- */
/* Forward recurrence over packed sequences.                                   */
/*   sa_t[v]  = sum_k a_t[k] S[k][v]                                           */
/*   S[k][v]  = w_t[k] S[k][v] + b_t[k] sa_t[v] + k_t[k] v_t[v]                */
/*   y_t[v]   = scale * sum_k r_t[k] S[k][v]      (updated state)              */
/* chunk tables (optional): sequence s owns chunks                             */
/*   [seq_chunk_offsets[s], seq_chunk_offsets[s+1]); chunk c covers tokens     */
/*   [chunk_starts[c], chunk_ends[c]); boundary[c] = state before chunk c.     */
/* If seq_chunk_offsets is NULL the token range of sequence s is               */
/*   [cu_seqlens[s], cu_seqlens[s+1]).                                         */
/* ------------------------------------------------------------------------- */
#define DEFINE_FORWARD(NAME, acc_t, RET)                                        \
  void NAME(const int32_t* cu_seqlens, const int32_t* state_indices,            \
            const int32_t* seq_chunk_offsets, const int32_t* chunk_starts,      \
            const int32_t* chunk_ends, int B, int H, int D, float* state_pool,  \
            const float* r, const float* logits, const float* k,                \
            const float* v, const float* a, const float* b,                     \
            const float* decay_bias, float scale, float* y, float* boundary,    \
            float* state_dot_a) {                                               \
    const int64_t DD = (int64_t)D * D;                                          \
    _Pragma("omp parallel for collapse(2) schedule(dynamic)")                   \
    for (int s = 0; s < B; ++s) {                                               \
      for (int h = 0; h < H; ++h) {                                             \
        acc_t* S = (acc_t*)malloc(sizeof(acc_t) * DD);                          \
        acc_t* sa = (acc_t*)malloc(sizeof(acc_t) * D);                          \
        acc_t* w = (acc_t*)malloc(sizeof(acc_t) * D);                           \
        const int slot = state_indices ? state_indices[s] : s;                  \
        float* Sg = state_pool + ((int64_t)slot * H + h) * DD;                  \
        for (int64_t i = 0; i < DD; ++i) S[i] = (acc_t)Sg[i];                   \
        int c0 = 0, c1 = 1;                                                     \
        if (seq_chunk_offsets) {                                                \
          c0 = seq_chunk_offsets[s];                                            \
          c1 = seq_chunk_offsets[s + 1];                                        \
        }                                                                       \
        for (int c = c0; c < c1; ++c) {                                         \
          int t0, t1;                                                           \
          if (seq_chunk_offsets) {                                              \
            t0 = chunk_starts[c];                                               \
            t1 = chunk_ends[c];                                                 \
            if (boundary) {                                                     \
              float* Bd = boundary + ((int64_t)c * H + h) * DD;                 \
              for (int64_t i = 0; i < DD; ++i) Bd[i] = (float)S[i];             \
            }                                                                   \
          } else {                                                              \
            t0 = cu_seqlens[s];                                                 \
            t1 = cu_seqlens[s + 1];                                             \
          }                                                                     \
          for (int t = t0; t < t1; ++t) {                                       \
            const int64_t base = ((int64_t)t * H + h) * D;                      \
            for (int i = 0; i < D; ++i) {                                       \
              acc_t x = (acc_t)logits[base + i];                                \
              if (decay_bias) x += (acc_t)decay_bias[(int64_t)h * D + i];       \
              w[i] = RET(x);                                                    \
            }                                                                   \
            for (int j = 0; j < D; ++j) sa[j] = 0;                              \
            for (int i = 0; i < D; ++i) {                                       \
              const acc_t ai = (acc_t)a[base + i];                              \
              const acc_t* Si = S + (int64_t)i * D;                             \
              for (int j = 0; j < D; ++j) sa[j] += ai * Si[j];                  \
            }                                                                   \
            if (state_dot_a)                                                    \
              for (int j = 0; j < D; ++j) state_dot_a[base + j] = (float)sa[j]; \
            acc_t ytmp[256];                                                    \
            for (int j = 0; j < D; ++j) ytmp[j] = 0;                            \
            for (int i = 0; i < D; ++i) {                                       \
              const acc_t wi = w[i], bi = (acc_t)b[base + i];                   \
              const acc_t ki = (acc_t)k[base + i], ri = (acc_t)r[base + i];     \
              acc_t* Si = S + (int64_t)i * D;                                   \
              for (int j = 0; j < D; ++j) {                                     \
                const acc_t u = wi * Si[j] + bi * sa[j] +                       \
                                ki * (acc_t)v[base + j];                        \
                Si[j] = u;                                                      \
                ytmp[j] += ri * u;                                              \
              }                                                                 \
            }                                                                   \
            for (int j = 0; j < D; ++j)                                         \
              y[base + j] = (float)((acc_t)scale * ytmp[j]);                    \
          }                                                                     \
        }                                                                       \
        for (int64_t i = 0; i < DD; ++i) Sg[i] = (float)S[i];                   \
        free(S);                                                                \
        free(sa);                                                               \
        free(w);                                                                \
      }                                                                         \
    }                                                                           \
  }

DEFINE_FORWARD(oracle_wkv7_forward_f32, float, retention_f)
DEFINE_FORWARD(oracle_wkv7_forward_f64, double, retention_d)

/* ------------------------------------------------------------------------- */
/* Forward recurrence on an fp16 state pool (tests/tmix/wkv7/test.py:216-277   */
/* of the reference), fp32 arithmetic in the reference's order of operations:  */
/*   phase    = h*D + k + elapsed[slot] + (t - first token of the sequence)    */
/*   dither   = (float)(int32)((uint32)phase * 2654435769) * 2^-41             */
/*   delta[k] = half(exp(-e^-0.5 sigmoid(logit[k] + bias[k])) - 1 + dither)    */
/*   sa[v]    = sum_k a[k] S[k][v]                                             */
/*   S[k][v]  = half(S + S*delta[k] + b[k]*sa[v] + k[k]*v[v])                  */
/*   y[v]     = half(scale * sum_k r[k] S[k][v])        (rounded new state)    */
/* state_pool holds IEEE binary16 values; y receives the fp16-rounded outputs  */
/* as floats.  The elapsed counters are read, never advanced.                  */
/* ------------------------------------------------------------------------- */
void oracle_wkv7_fp16_forward(const int32_t* cu_seqlens, const int32_t* state_indices,
                              const int32_t* elapsed, int B, int H, int D, _Float16* state_pool,
                              const float* r, const float* logits, const float* k, const float* v,
                              const float* a, const float* b, const float* decay_bias, float scale,
                              float* y) {
  const int64_t DD = (int64_t)D * D;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int s = 0; s < B; ++s) {
    for (int h = 0; h < H; ++h) {
      float* S = (float*)malloc(sizeof(float) * DD);
      float* sa = (float*)malloc(sizeof(float) * D);
      float* delta = (float*)malloc(sizeof(float) * D);
      const int slot = state_indices ? state_indices[s] : s;
      _Float16* Sg = state_pool + ((int64_t)slot * H + h) * DD;
      for (int64_t i = 0; i < DD; ++i) S[i] = (float)Sg[i];
      const int t0 = cu_seqlens[s], t1 = cu_seqlens[s + 1];
      for (int t = t0; t < t1; ++t) {
        const int64_t base = ((int64_t)t * H + h) * D;
        for (int i = 0; i < D; ++i) {
          float x = logits[base + i];
          if (decay_bias) x += decay_bias[(int64_t)h * D + i];
          const float w = expf(-(float)DECAY_RATE * (1.0f / (1.0f + expf(-x))));
          const uint32_t phase = (uint32_t)(h * D + i) + (uint32_t)elapsed[slot] + (uint32_t)(t - t0);
          const float dither = (float)(int32_t)(phase * 2654435769u) * 4.547473508864641e-13f;
          delta[i] = (float)(_Float16)((w - 1.0f) + dither);
        }
        for (int j = 0; j < D; ++j) sa[j] = 0.f;
        for (int i = 0; i < D; ++i) {
          const float ai = a[base + i];
          for (int j = 0; j < D; ++j) sa[j] += ai * S[(int64_t)i * D + j];
        }
        float ytmp[256];
        for (int j = 0; j < D; ++j) ytmp[j] = 0.f;
        for (int i = 0; i < D; ++i) {
          float* Si = S + (int64_t)i * D;
          const float di = delta[i], bi = b[base + i], ki = k[base + i], ri = r[base + i];
          for (int j = 0; j < D; ++j) {
            const float u = (float)(_Float16)(((Si[j] + Si[j] * di) + bi * sa[j]) + ki * v[base + j]);
            Si[j] = u;
            ytmp[j] += ri * u;
          }
        }
        for (int j = 0; j < D; ++j) y[base + j] = (float)(_Float16)(scale * ytmp[j]);
      }
      for (int64_t i = 0; i < DD; ++i) Sg[i] = (_Float16)S[i];
      free(S);
      free(sa);
      free(delta);
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Backward of the forward above for dense equal-length sequences             */
/* ([B][T][H][D] == packed with cu_seqlens = arange*T), double accumulation.  */
/* Inputs: S0 [B][H][D][D], tokens, dy [N][H][D], dSfinal (nullable).         */
/* Outputs: dr, dlogits, dk, dv, da, db [N][H][D] and dS0 [B][H][D][D].       */
/* The forward states are recomputed and kept (T*D*D doubles per head), so    */
/* this is for test-sized T only.  Adjoint equations:                         */
/*   G += scale r_t (x) dy_t ; dr = scale S_t dy ; dk = G v ; db = G sa       */
/*   dv = G^T k ; dsa = G^T b ; dw = rowsum(G * S_{t-1})                      */
/*   dlogit = dw * w * dlogw/dx ; da = S_{t-1} dsa ; G = diag(w) G + a(x)dsa  */
/* ------------------------------------------------------------------------- */
void oracle_wkv7_backward_f64(const int32_t* cu_seqlens, int B, int H, int D,
                              const float* S0, const float* r,
                              const float* logits, const float* k,
                              const float* v, const float* a, const float* b,
                              const float* decay_bias, float scale,
                              const float* dy, const float* dSfinal, float* dr,
                              float* dlogits, float* dk, float* dv, float* da,
                              float* db, float* dS0) {
  const int64_t DD = (int64_t)D * D;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int s = 0; s < B; ++s) {
    for (int h = 0; h < H; ++h) {
      const int t0 = cu_seqlens[s], t1 = cu_seqlens[s + 1];
      const int T = t1 - t0;
      double* St = (double*)malloc(sizeof(double) * DD * (T + 1));
      double* sa = (double*)malloc(sizeof(double) * D * T);
      double* w = (double*)malloc(sizeof(double) * D * T);
      double* G = (double*)malloc(sizeof(double) * DD);
      double* dsa = (double*)malloc(sizeof(double) * D);
      const float* S0g = S0 + ((int64_t)s * H + h) * DD;
      for (int64_t i = 0; i < DD; ++i) St[i] = S0g[i];
      for (int t = 0; t < T; ++t) {
        const int64_t base = ((int64_t)(t0 + t) * H + h) * D;
        const double* P = St + (int64_t)t * DD;
        double* Q = St + (int64_t)(t + 1) * DD;
        double* sat = sa + (int64_t)t * D;
        double* wt = w + (int64_t)t * D;
        for (int i = 0; i < D; ++i) {
          double x = logits[base + i];
          if (decay_bias) x += decay_bias[(int64_t)h * D + i];
          wt[i] = retention_d(x);
        }
        for (int j = 0; j < D; ++j) sat[j] = 0;
        for (int i = 0; i < D; ++i)
          for (int j = 0; j < D; ++j) sat[j] += (double)a[base + i] * P[i * D + j];
        for (int i = 0; i < D; ++i)
          for (int j = 0; j < D; ++j)
            Q[i * D + j] = wt[i] * P[i * D + j] + (double)b[base + i] * sat[j] +
                           (double)k[base + i] * (double)v[base + j];
      }
      if (dSfinal) {
        const float* g = dSfinal + ((int64_t)s * H + h) * DD;
        for (int64_t i = 0; i < DD; ++i) G[i] = g[i];
      } else {
        for (int64_t i = 0; i < DD; ++i) G[i] = 0;
      }
      for (int t = T - 1; t >= 0; --t) {
        const int64_t base = ((int64_t)(t0 + t) * H + h) * D;
        const double* P = St + (int64_t)t * DD;       /* S_{t-1} */
        const double* Q = St + (int64_t)(t + 1) * DD; /* S_t */
        const double* sat = sa + (int64_t)t * D;
        const double* wt = w + (int64_t)t * D;
        for (int i = 0; i < D; ++i) {
          double acc = 0;
          for (int j = 0; j < D; ++j) {
            G[i * D + j] += (double)scale * r[base + i] * dy[base + j];
            acc += Q[i * D + j] * dy[base + j];
          }
          dr[base + i] = (float)((double)scale * acc);
        }
        for (int j = 0; j < D; ++j) dsa[j] = 0;
        double dvj[256];
        for (int j = 0; j < D; ++j) dvj[j] = 0;
        for (int i = 0; i < D; ++i) {
          double gk = 0, gb = 0, gw = 0;
          for (int j = 0; j < D; ++j) {
            const double g = G[i * D + j];
            gk += g * v[base + j];
            gb += g * sat[j];
            gw += g * P[i * D + j];
            dvj[j] += g * k[base + i];
            dsa[j] += g * b[base + i];
          }
          dk[base + i] = (float)gk;
          db[base + i] = (float)gb;
          double x = logits[base + i];
          if (decay_bias) x += decay_bias[(int64_t)h * D + i];
          dlogits[base + i] = (float)(gw * wt[i] * retention_dlog_d(x));
        }
        for (int j = 0; j < D; ++j) dv[base + j] = (float)dvj[j];
        for (int i = 0; i < D; ++i) {
          double acc = 0;
          for (int j = 0; j < D; ++j) acc += P[i * D + j] * dsa[j];
          da[base + i] = (float)acc;
        }
        for (int i = 0; i < D; ++i)
          for (int j = 0; j < D; ++j)
            G[i * D + j] = wt[i] * G[i * D + j] + (double)a[base + i] * dsa[j];
      }
      if (dS0) {
        float* g = dS0 + ((int64_t)s * H + h) * DD;
        for (int64_t i = 0; i < DD; ++i) g[i] = (float)G[i];
      }
      free(St);
      free(sa);
      free(w);
      free(G);
      free(dsa);
    }
  }
}

/* ------------------------------------------------------------------------- */
/* TMix elementwise pieces (fp32 in, fp32 out; callers round to 16 bits).     */
/* ------------------------------------------------------------------------- */

/* out_j = x + (prev - x) * mix_j ; prev = previous packed row, or the shift   */
/* state slot at a sequence start; the slot then takes the last row.           */
void oracle_mix6(const float* x, float* shift_pool, const float* mix /*[6][C]*/,
                 const int32_t* cu_seqlens, const int32_t* state_indices,
                 int B, int C, float* out /*[6][N][C]*/, int64_t N) {
  for (int s = 0; s < B; ++s) {
    const int t0 = cu_seqlens[s], t1 = cu_seqlens[s + 1];
    float* slot = shift_pool + (int64_t)state_indices[s] * C;
    for (int t = t0; t < t1; ++t) {
      const float* prev = (t == t0) ? slot : x + (int64_t)(t - 1) * C;
      const float* cur = x + (int64_t)t * C;
      for (int j = 0; j < 6; ++j)
        for (int c = 0; c < C; ++c)
          out[((int64_t)j * N + t) * C + c] =
              cur[c] + (prev[c] - cur[c]) * mix[(int64_t)j * C + c];
    }
    memcpy(slot, x + (int64_t)(t1 - 1) * C, sizeof(float) * C);
  }
}

/* kk = normalize(k * k_k) per head (eps 1e-12 on the norm);                   */
/* a = sigmoid(a0 + a12); new_k = k * (1 + (a - 1) * k_a);                     */
/* returns new_k, -kk, kk * a.                                                 */
void oracle_kk_a_gate(const float* k, const float* k_k, const float* a0,
                      const float* a12, const float* k_a, int64_t N, int H,
                      int D, float* new_k, float* neg_kk, float* kka) {
  const int C = H * D;
  for (int64_t n = 0; n < N; ++n)
    for (int h = 0; h < H; ++h) {
      const int64_t o = n * C + (int64_t)h * D;
      double ss = 0;
      for (int i = 0; i < D; ++i) {
        double q = (double)k[o + i] * k_k[h * D + i];
        ss += q * q;
      }
      double nrm = sqrt(ss);
      if (nrm < 1e-12) nrm = 1e-12;
      for (int i = 0; i < D; ++i) {
        const int c = h * D + i;
        double kk = (double)k[o + i] * k_k[c] / nrm;
        double av = 1.0 / (1.0 + exp(-((double)a0[c] + a12[o + i])));
        new_k[o + i] = (float)(k[o + i] * (1.0 + (av - 1.0) * k_a[c]));
        neg_kk[o + i] = (float)(-kk);
        kka[o + i] = (float)(kk * av);
      }
    }
}

/* per-head GroupNorm of x (biased variance, eps) * weight + bias              */
/*   + (sum_d r k r_k) * v, all times g.                                       */
void oracle_lnx_rkvres_xg(const float* x, const float* r, const float* k,
                          const float* v, const float* r_k, const float* weight,
                          const float* bias, const float* g, int64_t N, int H,
                          int D, double eps, float* out) {
  const int C = H * D;
  for (int64_t n = 0; n < N; ++n)
    for (int h = 0; h < H; ++h) {
      const int64_t o = n * C + (int64_t)h * D;
      double mean = 0, var = 0, dot = 0;
      for (int i = 0; i < D; ++i) mean += x[o + i];
      mean /= D;
      for (int i = 0; i < D; ++i) {
        double d = x[o + i] - mean;
        var += d * d;
        dot += (double)r[o + i] * k[o + i] * r_k[h * D + i];
      }
      var /= D;
      const double rstd = 1.0 / sqrt(var + eps);
      for (int i = 0; i < D; ++i) {
        const int c = h * D + i;
        double nx = (x[o + i] - mean) * rstd * weight[c] + bias[c];
        out[o + i] = (float)((nx + dot * v[o + i]) * g[o + i]);
      }
    }
}

/* v + (v_first - v) * sigmoid(v0 + v12) */
void oracle_vres_gate(const float* v, const float* v_first, const float* v0,
                      const float* v12, int64_t N, int C, float* out) {
  for (int64_t n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c) {
      const int64_t o = n * C + c;
      double gate = 1.0 / (1.0 + exp(-((double)v0[c] + v12[o])));
      out[o] = (float)(v[o] + ((double)v_first[o] - v[o]) * gate);
    }
}

/* y[M][N] = act(x)[M][K] @ W[N][K]^T ; act: 0 none, 1 tanh, 2 sigmoid.        */
void oracle_linear_nt(const float* x, const float* w, int64_t M, int N, int K,
                      int act, float* y) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    double* ax = (double*)malloc(sizeof(double) * K);
    for (int q = 0; q < K; ++q) {
      double xv = x[m * K + q];
      ax[q] = act == 1 ? tanh(xv) : act == 2 ? 1.0 / (1.0 + exp(-xv)) : xv;
    }
    for (int n = 0; n < N; ++n) {
      double acc = 0;
      const float* wr = w + (int64_t)n * K;
      for (int q = 0; q < K; ++q) acc += ax[q] * wr[q];
      y[m * N + n] = (float)acc;
    }
    free(ax);
  }
}
