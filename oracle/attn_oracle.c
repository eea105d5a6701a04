/*
 * attn_oracle.c — CPU restatement of Tyr's attention path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing the product ships may call into this file:
 * it is the checker for the tests, the smoke check and the CPU-baseline leg of
 * the benchmark.  The arithmetic of the reference path lives in a third-party
 * dependency that is not vendored in the reference tree: LibTorch/ATen
 * `scaled_dot_product_attention` (the reference pins LibTorch 2.9.1 for CPU
 * builds, Readme.md:37,53 and .github/workflows/ci.yml:12).  This file restates
 * the published algorithm and is pinned against outputs of that same ATen
 * operator (torch 2.11 in this image) stored under tests/golden/, and against
 * closed-form cases.  The reference's own tests hold no golden vectors for
 * attention (fixtures are generated at run time, Examples/GPU/FixtureRunner.lean:22-39).
 *
 * What each function follows:
 *   tyr_oracle_sdpa        softmax(Q K^T * scale + mask) V on fp32 data, the formula of the
 *                          reference's fixture generator (Examples/GPU/RunFlashAttn.lean:30-48);
 *                          GQA head map of repeat_interleave (cc/src/tyr.cpp:3931-3938);
 *                          causal mask "col > row is masked" (cc/src/tyr.cpp:3990-3991);
 *                          LSE = log(sum(exp(scaled scores))) (RunFlashAttn.lean:45-48).
 *   tyr_oracle_sdpa_window the same with the causal sliding-window mask of
 *                          lean_torch_sdpa_gqa_window (cc/src/tyr.cpp:3953-4018).
 *   tyr_oracle_sdpa_keymask the same with the key padding mask of lean_torch_sdpa_gqa_mask
 *                          (cc/src/tyr.cpp:4024-4095).
 *   tyr_oracle_sdpa_online the running max / running sum form of
 *                          Tyr/GPU/Codegen/Macros.lean:121-163 with fp32 state.
 *   tyr_oracle_sdpa_backward  gradients of the direct form with respect to Q, K and V for a given dO,
 *                          the derivative LibTorch autograd supplies to the reference
 *                          (cc/src/tyr.cpp:2111-2122), written as in
 *                          Tyr/GPU/Kernels/MhaH100.lean:196-344: d = rowsum(dO*O),
 *                          dV = P^T dO, dP = dO V^T, dS = scale * P * (dP - d), dQ = dS K, dK = dS^T Q.
 *   tyr_oracle_merge2      LSE merge of two partial results,
 *                          Tyr/GPU/Kernels/RingAttn.lean:164-180.
 *   tyr_oracle_bf16_round  round-to-nearest-even fp32 -> bf16 -> fp32, the quantisation the
 *                          reference applies to inputs before its fp32 check (RunFlashAttn.lean:30-36).
 *
 * Layout: contiguous row-major [B, H, S, D] fp32.  Accumulation is in double, so
 * the result is the correctly rounded fp32 answer to well below 1e-6 relative.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int tyr_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void tyr_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

void tyr_oracle_bf16_round(const float* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t u;
    memcpy(&u, &in[i], 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
      u |= 0x00400000u; /* quiet NaN */
    } else {
      u += 0x7fffu + ((u >> 16) & 1u);
    }
    u &= 0xffff0000u;
    memcpy(&out[i], &u, 4);
  }
}

/* Direct form.  Returns 0, or -1 on bad arguments.  window > 0 adds the sliding-window mask of
 * lean_torch_sdpa_gqa_window (cc/src/tyr.cpp:3986-3996): key j is also hidden from query i
 * when i - j >= window; that entry point always combines it with the causal mask. */
static int sdpa_direct(const float* q, const float* k, const float* v, float* o, float* lse, int B,
                       int Hq, int Hkv, int Sq, int Skv, int D, int is_causal, float scale,
                       int window, const uint8_t* key_mask) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || D <= 0 || Hq % Hkv != 0) return -1;
  const int g = Hq / Hkv; /* query head h reads KV head h / g */
  const int64_t rows = (int64_t)B * Hq * Sq;
  int failed = 0;
#pragma omp parallel
  {
    double* s = (double*)malloc(sizeof(double) * (size_t)Skv);
    double* acc = (double*)malloc(sizeof(double) * (size_t)D);
    if (!s || !acc) {
#pragma omp atomic write
      failed = 1;
    } else {
#pragma omp for schedule(dynamic, 16)
      for (int64_t r = 0; r < rows; ++r) {
        const int i = (int)(r % Sq);
        const int h = (int)((r / Sq) % Hq);
        const int b = (int)(r / ((int64_t)Sq * Hq));
        const float* qr = q + r * D;
        const float* kb = k + ((int64_t)b * Hkv + h / g) * (int64_t)Skv * D;
        const float* vb = v + ((int64_t)b * Hkv + h / g) * (int64_t)Skv * D;
        const int n = is_causal ? (i + 1 < Skv ? i + 1 : Skv) : Skv; /* keys j <= i */
        const int j0 = (window > 0 && i - window + 1 > 0) ? i - window + 1 : 0; /* i - j < window */
        double mx = -INFINITY;
        for (int j = j0; j < n; ++j) {
          const float* kr = kb + (int64_t)j * D;
          double dot = 0.0;
          for (int d = 0; d < D; ++d) dot += (double)qr[d] * (double)kr[d];
          s[j] = dot * (double)scale;
          if (key_mask && key_mask[(int64_t)b * Skv + j] == 0) s[j] = -INFINITY; /* padding key */
          if (s[j] > mx) mx = s[j];
        }
        double sum = 0.0;
        for (int d = 0; d < D; ++d) acc[d] = 0.0;
        for (int j = j0; j < n; ++j) {
          const double p = (s[j] == -INFINITY) ? 0.0 : exp(s[j] - mx);
          sum += p;
          const float* vr = vb + (int64_t)j * D;
          for (int d = 0; d < D; ++d) acc[d] += p * (double)vr[d];
        }
        for (int d = 0; d < D; ++d) o[r * D + d] = (float)(acc[d] / sum);
        if (lse) lse[r] = (float)(mx + log(sum));
      }
    }
    free(s);
    free(acc);
  }
  return failed ? -1 : 0;
}

int tyr_oracle_sdpa(const float* q, const float* k, const float* v, float* o, float* lse, int B,
                    int Hq, int Hkv, int Sq, int Skv, int D, int is_causal, float scale) {
  return sdpa_direct(q, k, v, o, lse, B, Hq, Hkv, Sq, Skv, D, is_causal, scale, 0, NULL);
}

int tyr_oracle_sdpa_window(const float* q, const float* k, const float* v, float* o, float* lse,
                           int B, int Hq, int Hkv, int S, int D, float scale, int window) {
  if (window <= 0) return -1;
  return sdpa_direct(q, k, v, o, lse, B, Hq, Hkv, S, S, D, 1, scale, window, NULL);
}

/* Padding mask of lean_torch_sdpa_gqa_mask (cc/src/tyr.cpp:4024-4095): key_mask [B, S] bytes,
 * 0 = padding key hidden from every query, combined with the causal mask when is_causal.
 * A query that sees no key gets 0/0 = NaN, as ATen's softmax over all -inf does. */
int tyr_oracle_sdpa_keymask(const float* q, const float* k, const float* v, float* o, float* lse,
                            int B, int Hq, int Hkv, int S, int D, int is_causal, float scale,
                            const uint8_t* key_mask) {
  if (!key_mask) return -1;
  return sdpa_direct(q, k, v, o, lse, B, Hq, Hkv, S, S, D, is_causal, scale, 0, key_mask);
}

/* Online form with fp32 state, keys visited in blocks of `block` (Macros.lean:121-163):
 *   prevMax = rowMax; rowMax = max(rowMax, max(scores)); scale = exp(prevMax - rowMax);
 *   out *= scale; rowSum *= scale; scores = exp(scores - rowMax); rowSum += sum(scores);
 *   out += scores V;  finally out /= rowSum, lse = log(rowSum) + rowMax. */
int tyr_oracle_sdpa_online(const float* q, const float* k, const float* v, float* o, float* lse,
                           int B, int Hq, int Hkv, int Sq, int Skv, int D, int is_causal,
                           float scale, int block) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || D <= 0 || Hq % Hkv != 0 ||
      block <= 0 || block > 4096)
    return -1;
  const int g = Hq / Hkv;
  const int64_t rows = (int64_t)B * Hq * Sq;
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t r = 0; r < rows; ++r) {
    const int i = (int)(r % Sq);
    const int h = (int)((r / Sq) % Hq);
    const int b = (int)(r / ((int64_t)Sq * Hq));
    const float* qr = q + r * D;
    const float* kb = k + ((int64_t)b * Hkv + h / g) * (int64_t)Skv * D;
    const float* vb = v + ((int64_t)b * Hkv + h / g) * (int64_t)Skv * D;
    const int n = is_causal ? (i + 1 < Skv ? i + 1 : Skv) : Skv;
    float row_max = -INFINITY, row_sum = 0.f;
    float out[1024];
    float sc[4096];
    if (D > 1024) continue;
    for (int d = 0; d < D; ++d) out[d] = 0.f;
    for (int j0 = 0; j0 < n; j0 += block) {
      const int nb = (n - j0 < block) ? n - j0 : block;
      const float prev_max = row_max;
      for (int j = 0; j < nb; ++j) {
        const float* kr = kb + (int64_t)(j0 + j) * D;
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot += qr[d] * kr[d];
        sc[j] = dot * scale;
        if (sc[j] > row_max) row_max = sc[j];
      }
      const float resc = (prev_max == -INFINITY) ? 0.f : expf(prev_max - row_max);
      for (int d = 0; d < D; ++d) out[d] *= resc;
      row_sum *= resc;
      for (int j = 0; j < nb; ++j) {
        sc[j] = expf(sc[j] - row_max);
        row_sum += sc[j];
        const float* vr = vb + (int64_t)(j0 + j) * D;
        for (int d = 0; d < D; ++d) out[d] += sc[j] * vr[d];
      }
    }
    for (int d = 0; d < D; ++d) o[r * D + d] = out[d] / row_sum;
    if (lse) lse[r] = logf(row_sum) + row_max;
  }
  return 0;
}

/* Backward of the direct form in double precision.  One (batch, KV head) per task: dK and dV
 * of a KV head sum over the Hq / Hkv query heads that share it (the derivative of
 * repeat_interleave, cc/src/tyr.cpp:3931-3938).  Returns 0, or -1 on bad arguments. */
static int sdpa_backward_direct(const float* q, const float* k, const float* v, const float* d_o,
                                float* d_q, float* d_k, float* d_v, int B, int Hq, int Hkv, int Sq,
                                int Skv, int D, int is_causal, float scale, int window,
                                const uint8_t* key_mask) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Sq <= 0 || Skv <= 0 || D <= 0 || Hq % Hkv != 0) return -1;
  const int g = Hq / Hkv;
  const int64_t tasks = (int64_t)B * Hkv;
  int failed = 0;
#pragma omp parallel
  {
    double* p = (double*)malloc(sizeof(double) * (size_t)Skv);
    double* dp = (double*)malloc(sizeof(double) * (size_t)Skv);
    double* o = (double*)malloc(sizeof(double) * (size_t)D);
    double* dk = (double*)malloc(sizeof(double) * (size_t)Skv * D);
    double* dv = (double*)malloc(sizeof(double) * (size_t)Skv * D);
    double* dq = (double*)malloc(sizeof(double) * (size_t)D);
    if (!p || !dp || !o || !dk || !dv || !dq) {
#pragma omp atomic write
      failed = 1;
    } else {
#pragma omp for schedule(dynamic, 1)
      for (int64_t t = 0; t < tasks; ++t) {
        const int b = (int)(t / Hkv), hk = (int)(t % Hkv);
        const float* kb = k + t * (int64_t)Skv * D;
        const float* vb = v + t * (int64_t)Skv * D;
        for (int64_t x = 0; x < (int64_t)Skv * D; ++x) dk[x] = dv[x] = 0.0;
        for (int hh = 0; hh < g; ++hh) {
          const int h = hk * g + hh;
          for (int i = 0; i < Sq; ++i) {
            const int64_t r = ((int64_t)b * Hq + h) * Sq + i;
            const float* qr = q + r * D;
            const float* gr = d_o + r * D;
            const int n = is_causal ? (i + 1 < Skv ? i + 1 : Skv) : Skv; /* keys j <= i */
            const int j0 = (window > 0 && i - window + 1 > 0) ? i - window + 1 : 0; /* i - j < window */
            double mx = -INFINITY, sum = 0.0, delta = 0.0;
            for (int j = j0; j < n; ++j) {
              double dot = 0.0;
              for (int d = 0; d < D; ++d) dot += (double)qr[d] * (double)kb[(int64_t)j * D + d];
              p[j] = dot * (double)scale;
              if (key_mask && key_mask[(int64_t)b * Skv + j] == 0) p[j] = -INFINITY; /* padding key */
              if (p[j] > mx) mx = p[j];
            }
            for (int j = j0; j < n; ++j) {
              p[j] = (p[j] == -INFINITY) ? 0.0 : exp(p[j] - mx);
              sum += p[j];
            }
            for (int d = 0; d < D; ++d) o[d] = 0.0;
            for (int j = j0; j < n; ++j) {
              p[j] /= sum; /* softmax row */
              double g_dot_v = 0.0;
              for (int d = 0; d < D; ++d) {
                o[d] += p[j] * (double)vb[(int64_t)j * D + d];
                g_dot_v += (double)gr[d] * (double)vb[(int64_t)j * D + d];
              }
              dp[j] = g_dot_v; /* dP = dO V^T */
            }
            for (int d = 0; d < D; ++d) delta += (double)gr[d] * o[d]; /* d = rowsum(dO * O) */
            for (int d = 0; d < D; ++d) dq[d] = 0.0;
            for (int j = j0; j < n; ++j) {
              const double ds = (double)scale * p[j] * (dp[j] - delta);
              for (int d = 0; d < D; ++d) {
                dv[(int64_t)j * D + d] += p[j] * (double)gr[d];         /* dV = P^T dO */
                dq[d] += ds * (double)kb[(int64_t)j * D + d];           /* dQ = dS K */
                dk[(int64_t)j * D + d] += ds * (double)qr[d];           /* dK = dS^T Q */
              }
            }
            for (int d = 0; d < D; ++d) d_q[r * D + d] = (float)dq[d];
          }
        }
        for (int64_t x = 0; x < (int64_t)Skv * D; ++x) {
          d_k[t * (int64_t)Skv * D + x] = (float)dk[x];
          d_v[t * (int64_t)Skv * D + x] = (float)dv[x];
        }
      }
    }
    free(p);
    free(dp);
    free(o);
    free(dk);
    free(dv);
    free(dq);
  }
  return failed ? -1 : 0;
}

int tyr_oracle_sdpa_backward(const float* q, const float* k, const float* v, const float* d_o,
                             float* d_q, float* d_k, float* d_v, int B, int Hq, int Hkv, int Sq,
                             int Skv, int D, int is_causal, float scale) {
  return sdpa_backward_direct(q, k, v, d_o, d_q, d_k, d_v, B, Hq, Hkv, Sq, Skv, D, is_causal, scale, 0, NULL);
}

/* The same under the sliding-window mask (window > 0, always with the causal mask, cc/src/tyr.cpp:3986-3996)
 * and / or the key padding mask (key_mask [B, Skv] bytes, 0 = padding key, cc/src/tyr.cpp:4063-4086). */
int tyr_oracle_sdpa_backward_masked(const float* q, const float* k, const float* v, const float* d_o,
                                    float* d_q, float* d_k, float* d_v, int B, int Hq, int Hkv, int Sq,
                                    int Skv, int D, int is_causal, float scale, int window,
                                    const uint8_t* key_mask) {
  return sdpa_backward_direct(q, k, v, d_o, d_q, d_k, d_v, B, Hq, Hkv, Sq, Skv, D,
                              (is_causal || window > 0) ? 1 : 0, scale, window, key_mask);
}

/* L = Lr + log(1 + exp(Lb - Lr));  O = Or*exp(Lr - L) + Ob*exp(Lb - L)
 * (RingAttn.lean:164-180), evaluated with the larger LSE as Lr so that exp never overflows. */
void tyr_oracle_merge2(const float* o_a, const float* lse_a, const float* o_b, const float* lse_b,
                       float* o_out, float* lse_out, int64_t rows, int D) {
  for (int64_t r = 0; r < rows; ++r) {
    const double la = lse_a[r], lb = lse_b[r];
    const double hi = la > lb ? la : lb, lo = la > lb ? lb : la;
    const double L = (hi == -INFINITY) ? -INFINITY : hi + log1p(exp(lo - hi));
    const double wa = (la == -INFINITY) ? 0.0 : exp(la - L), wb = (lb == -INFINITY) ? 0.0 : exp(lb - L);
    for (int d = 0; d < D; ++d)
      o_out[r * D + d] = (float)((double)o_a[r * D + d] * wa + (double)o_b[r * D + d] * wb);
    lse_out[r] = (float)L;
  }
}

/* Prologue of the attention call on fp32 data, per (batch, token, head) row:
 *   RMSNorm over the head vector, x * rsqrt(mean(x^2) + eps) * weight
 *     (applyHeadNorm, Tyr/Model/Qwen/Attention.lean:73-98); skipped when weight == NULL;
 *   rotary embedding on the two halves of the vector,
 *     [x1, x2] -> [x1*cos - x2*sin, x1*sin + x2*cos] with cos/sin rows indexed by position
 *     (lean_torch_apply_rotary_emb, cc/src/tyr.cpp:3824-3861); skipped when cos == NULL;
 *   the layout change [B,S,H,D] -> [B,H,S,D] (transpose_for_attention, cc/src/tyr.cpp:2402-2414)
 *   written at row positions[b] + s of out [B,H,cap,D], which for a KV cache is the
 *   slice_scatter of the new rows (cc/src/tyr.cpp:2261-2277) done in place. */
void tyr_oracle_qk_prologue(const float* x, const float* weight, const float* cs, const float* sn,
                            const int32_t* positions, int position0, float* out, int B, int S, int H,
                            int D, int cap, float eps) {
  const int half = D / 2;
  for (int b = 0; b < B; ++b)
    for (int s = 0; s < S; ++s)
      for (int h = 0; h < H; ++h) {
        const float* xr = x + (((int64_t)b * S + s) * H + h) * D;
        const int pos = (positions ? positions[b] : position0) + s;
        float* orow = out + (((int64_t)b * H + h) * cap + pos) * D;
        double inv = 1.0;
        if (weight) {
          double ss = 0.0;
          for (int d = 0; d < D; ++d) ss += (double)xr[d] * xr[d];
          inv = 1.0 / sqrt(ss / D + (double)eps);
        }
        for (int i = 0; i < half; ++i) {
          double a = xr[i], c = xr[half + i];
          if (weight) {
            a *= inv * weight[i];
            c *= inv * weight[half + i];
          }
          if (cs) {
            const double co = cs[(int64_t)pos * half + i], si = sn[(int64_t)pos * half + i];
            const double y1 = a * co - c * si, y2 = a * si + c * co;
            a = y1;
            c = y2;
          }
          orow[i] = (float)a;
          orow[half + i] = (float)c;
        }
      }
}

/* The same prologue with Flux's rotary form in place of the rotate-half one
 * (flux.applyRope, Tyr/Model/Flux/RoPE.lean:71-96): the head vector is read as D/2
 * INTERLEAVED pairs (x_2i, x_2i+1) and pair i of position `pos` is multiplied by the 2x2
 * matrix pe[b][pos][i]: out_2i+c = pe[i][c][0]*x_2i + pe[i][c][1]*x_2i+1.  pe is
 * [n_tables, max_pos, D/2, 2, 2]; batch element b reads table b * pe_batch_stride / (max_pos*2D),
 * i.e. `pe + b * pe_batch_stride` (0: one shared table).  RMSNorm as above when weight != NULL
 * (QKNorm.forward, Tyr/Model/Flux/QKNorm.lean:32-39). */
void tyr_oracle_qk_prologue_pe(const float* x, const float* weight, const float* pe, int64_t pe_batch_stride,
                               const int32_t* positions, int position0, float* out, int B, int S, int H,
                               int D, int cap, float eps) {
  for (int b = 0; b < B; ++b)
    for (int s = 0; s < S; ++s)
      for (int h = 0; h < H; ++h) {
        const float* xr = x + (((int64_t)b * S + s) * H + h) * D;
        const int pos = (positions ? positions[b] : position0) + s;
        float* orow = out + (((int64_t)b * H + h) * cap + pos) * D;
        const float* tab = pe + b * pe_batch_stride + (int64_t)pos * 2 * D;
        double inv = 1.0;
        if (weight) {
          double ss = 0.0;
          for (int d = 0; d < D; ++d) ss += (double)xr[d] * xr[d];
          inv = 1.0 / sqrt(ss / D + (double)eps);
        }
        for (int i = 0; i < D / 2; ++i) {
          double x0 = xr[2 * i], x1 = xr[2 * i + 1];
          if (weight) {
            x0 *= inv * weight[2 * i];
            x1 *= inv * weight[2 * i + 1];
          }
          orow[2 * i] = (float)(tab[4 * i] * x0 + tab[4 * i + 1] * x1);
          orow[2 * i + 1] = (float)(tab[4 * i + 2] * x0 + tab[4 * i + 3] * x1);
        }
      }
}
