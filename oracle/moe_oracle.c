/*
 * CPU oracle for the Qwen3 MoE layer (gate -> top-k -> softmax over the kept
 * logits -> expert SwiGLU FFN -> slot-ordered weighted sum).
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the algorithm of
 * the reference project's own CPU implementation so that the CUDA path can be
 * checked against it.  Nothing in the shipped library links or calls it; only
 * the tests, the smoke check and the cpu_baseline / reference legs of the
 * benchmark may load it, and there only as the checker or the timed baseline.
 *
 * Parity status: PINNED.  tests/test_oracle.py compares every function here,
 * bit for bit, with the reference's own headers compiled from where they lie
 * (oracle/_ref, built by oracle/Makefile) and with the golden vectors under
 * tests/golden/ that were generated from that build.
 *
 * Each function names the reference file:line it follows (paths relative to
 * the reference project root).  All arithmetic is fp32 in the reference's
 * order, except the softmax, which the reference evaluates in double.
 * Compile without fast-math and without FMA contraction (see the Makefile):
 * the reference accumulates `acc += a*b` with a rounded product.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* C[M,N] = A[M,K] * B[N,K]^T, fp32, k strictly sequential per output.
 * Follows test/singleGPU/cpp/moe/reference/refGemm.h:11-29. */
void oracle_gemm_nt(const float* A, const float* B, float* C, int M, int N,
                    int K) {
  for (int i = 0; i < M; ++i) {
    const float* a = A + (size_t)i * (size_t)K;
    float* c = C + (size_t)i * (size_t)N;
    for (int j = 0; j < N; ++j) {
      const float* b = B + (size_t)j * (size_t)K;
      float acc = 0.0f;
      for (int k = 0; k < K; ++k) acc += a[k] * b[k];
      c[j] = acc;
    }
  }
}

/* Same GEMM with B stored as bf16 (the upper 16 bits of the fp32 value).  A bf16 value
 * widens to fp32 exactly, so the result equals oracle_gemm_nt on the widened B bit for bit;
 * the benchmark's multi-rank parity check uses it to share one bf16 copy of all expert
 * weights between the ranks instead of an fp32 copy per rank. */
static float bf16_bits_to_f32(unsigned short b) {
  union {
    unsigned int u;
    float f;
  } v;
  v.u = (unsigned int)b << 16;
  return v.f;
}

void oracle_gemm_nt_bw(const float* A, const unsigned short* B, float* C, int M, int N,
                       int K) {
  for (int i = 0; i < M; ++i) {
    const float* a = A + (size_t)i * (size_t)K;
    float* c = C + (size_t)i * (size_t)N;
    for (int j = 0; j < N; ++j) {
      const unsigned short* b = B + (size_t)j * (size_t)K;
      float acc = 0.0f;
      for (int k = 0; k < K; ++k) acc += a[k] * bf16_bits_to_f32(b[k]);
      c[j] = acc;
    }
  }
}

/* Per-row top-k by insertion: descending values, strict '>' so that among
 * equal values the lower column index stays first.
 * Follows test/singleGPU/cpp/moe/reference/refTopk.h:17-67. */
void oracle_topk_rows(const float* in, int rows, int cols, float* out_vals,
                      int* out_idx, int topk) {
  for (int r = 0; r < rows; ++r) {
    const float* row = in + (size_t)r * (size_t)cols;
    float* tv = out_vals + (size_t)r * (size_t)topk;
    int* ti = out_idx + (size_t)r * (size_t)topk;
    for (int t = 0; t < topk; ++t) {
      tv[t] = -FLT_MAX; /* numeric_limits<float>::lowest() */
      ti[t] = -1;
    }
    for (int c = 0; c < cols; ++c) {
      const float v = row[c];
      int pos = topk;
      for (int t = 0; t < topk; ++t) {
        if (v > tv[t]) {
          pos = t;
          break;
        }
      }
      if (pos == topk) continue;
      for (int t = topk - 1; t > pos; --t) {
        tv[t] = tv[t - 1];
        ti[t] = ti[t - 1];
      }
      tv[pos] = v;
      ti[pos] = c;
    }
  }
}

/* In-place per-row softmax with a running max, evaluated in double and cast
 * back to float.
 * Follows test/singleGPU/cpp/moe/reference/refSoftmax.h:15-52. */
void oracle_softmax_rows(float* data, int rows, int cols) {
  if (rows == 0 || cols == 0) return;
  for (int r = 0; r < rows; ++r) {
    float* row = data + (size_t)r * (size_t)cols;
    double maxv = (double)row[0];
    double sum = 1.0;
    for (int j = 1; j < cols; ++j) {
      double x = (double)row[j];
      if (x > maxv) {
        double d = exp(maxv - x);
        sum = sum * d + 1.0;
        maxv = x;
      } else {
        sum += exp(x - maxv);
      }
    }
    if (sum <= 0.0) {
      float inv = (float)(1.0 / (double)cols);
      for (int j = 0; j < cols; ++j) row[j] = inv;
    } else {
      for (int j = 0; j < cols; ++j) {
        double e = exp((double)row[j] - maxv);
        row[j] = (float)(e / sum);
      }
    }
  }
}

/* Gate: logits = tokens * Wg^T, top-k, softmax over the kept logits.
 * `logits_out` (may be NULL) receives the fp32 logits [T,E].
 * Follows test/singleGPU/cpp/moe/reference/refMoeGate.h:16-33. */
void oracle_gate(const float* tokens, const float* gate_w, int T, int E, int H,
                 int topk, float* topk_w, int* topk_idx, float* logits_out) {
  float* logits = logits_out;
  if (!logits) logits = (float*)malloc((size_t)T * (size_t)E * sizeof(float));
  oracle_gemm_nt(tokens, gate_w, logits, T, E, H);
  oracle_topk_rows(logits, T, E, topk_w, topk_idx, topk);
  oracle_softmax_rows(topk_w, T, topk);
  if (!logits_out) free(logits);
}

/* Follows refExpertFFN1.h:12-22 (sigmoid_stable<float>). */
static float sigmoid_stable(float x) {
  if (x >= 0.0f) {
    float e = expf(-x);
    return 1.0f / (1.0f + e);
  } else {
    float e = expf(x);
    return e / (1.0f + e);
  }
}

/* out[rows,I] = silu(x W1^T) * (x W3^T) with W13 = [2I,H]: rows 0..I-1 are the
 * gate projection (left half of the GEMM output), rows I..2I-1 the up
 * projection.  Follows refExpertFFN1.h:31-48 (refSiluMul) and :51-65. */
static void ffn1_any(const float* tokens, const void* w13, int wbf16, int rows, int H, int I,
                     float* out) {
  float* g = (float*)malloc((size_t)rows * 2u * (size_t)I * sizeof(float));
  if (wbf16)
    oracle_gemm_nt_bw(tokens, (const unsigned short*)w13, g, rows, 2 * I, H);
  else
    oracle_gemm_nt(tokens, (const float*)w13, g, rows, 2 * I, H);
  for (int r = 0; r < rows; ++r) {
    const float* a = g + (size_t)r * 2u * (size_t)I;
    const float* b = a + I;
    float* o = out + (size_t)r * (size_t)I;
    for (int c = 0; c < I; ++c) {
      float s = sigmoid_stable(a[c]);
      o[c] = a[c] * s * b[c];
    }
  }
  free(g);
}

void oracle_ffn1(const float* tokens, const float* w13, int rows, int H, int I,
                 float* out) {
  ffn1_any(tokens, w13, 0, rows, H, I, out);
}

/* One token through gate-selected experts; stage buffers are optional.
 * act_out [K,I]: SwiGLU activations per slot; y_out [K,H]: unscaled FFN2 rows.
 * Follows refFullMoe.h:36-66 (the body of the per-token loop). */
static void moe_one_token(const float* x, const void* w13, const void* w2, int wbf16,
                          const float* gate_scores, const int* experts, int E,
                          int H, int topk, int I, float* out, float* act_out,
                          float* y_out, float* act_tmp, float* y_tmp) {
  for (int d = 0; d < H; ++d) out[d] = 0.0f;
  for (int k = 0; k < topk; ++k) {
    const int e = experts[k];
    const float score = gate_scores[k];
    float* act = act_out ? act_out + (size_t)k * (size_t)I : act_tmp;
    float* y = y_out ? y_out + (size_t)k * (size_t)H : y_tmp;
    if (e < 0 || e >= E || w13 == NULL) {
      if (act_out) memset(act, 0, (size_t)I * sizeof(float));
      if (y_out) memset(y, 0, (size_t)H * sizeof(float));
      continue;
    }
    const size_t esz = wbf16 ? 2u : 4u;
    const char* w13e = (const char*)w13 + (size_t)e * (size_t)H * (size_t)(2 * I) * esz;
    const char* w2e = (const char*)w2 + (size_t)e * (size_t)H * (size_t)I * esz;
    ffn1_any(x, w13e, wbf16, 1, H, I, act);
    if (wbf16)
      oracle_gemm_nt_bw(act, (const unsigned short*)w2e, y, 1, H, I);
    else
      oracle_gemm_nt(act, (const float*)w2e, y, 1, H, I);
    for (int d = 0; d < H; ++d) out[d] += y[d] * score;
  }
}

typedef struct {
  const float *tokens, *tw;
  const void *w13, *w2;
  int wbf16;
  const int* ti;
  float *out, *act_out, *y_out;
  int T, E, H, topk, I;
  int tid, nthreads;
} moe_job_t;

/* Tokens are independent; thread `tid` takes tokens tid, tid+n, tid+2n, ... */
static void* moe_worker(void* arg) {
  const moe_job_t* j = (const moe_job_t*)arg;
  float* act_tmp = (float*)malloc((size_t)j->I * sizeof(float));
  float* y_tmp = (float*)malloc((size_t)j->H * sizeof(float));
  for (int t = j->tid; t < j->T; t += j->nthreads) {
    moe_one_token(
        j->tokens + (size_t)t * (size_t)j->H, j->w13, j->w2, j->wbf16,
        j->tw + (size_t)t * (size_t)j->topk, j->ti + (size_t)t * (size_t)j->topk,
        j->E, j->H, j->topk, j->I, j->out + (size_t)t * (size_t)j->H,
        j->act_out ? j->act_out + (size_t)t * (size_t)j->topk * (size_t)j->I : NULL,
        j->y_out ? j->y_out + (size_t)t * (size_t)j->topk * (size_t)j->H : NULL,
        act_tmp, y_tmp);
  }
  free(act_tmp);
  free(y_tmp);
  return NULL;
}

/* Full layer.  out [T,H]; optional stage outputs: topk_w/topk_idx [T,K],
 * act_out [T,K,I], y_out [T,K,H] (any may be NULL).  `threads` > 1 splits the
 * independent token loop over that many POSIX threads; results do not depend
 * on it.  Follows test/singleGPU/cpp/moe/reference/refFullMoe.h:9-69. */
static void full_moe_any(const float* tokens, const float* gate_w, const void* w13,
                         const void* w2, int wbf16, int T, int E, int H, int topk, int I,
                         float* out, float* topk_w_out, int* topk_idx_out,
                         float* act_out, float* y_out, int threads) {
  if (T <= 0) return;
  float* tw = topk_w_out ? topk_w_out
                         : (float*)malloc((size_t)T * (size_t)topk * sizeof(float));
  int* ti = topk_idx_out ? topk_idx_out
                         : (int*)malloc((size_t)T * (size_t)topk * sizeof(int));
  oracle_gate(tokens, gate_w, T, E, H, topk, tw, ti, NULL);
  if (threads < 1) threads = 1;
  if (threads > T) threads = T;
  moe_job_t* jobs = (moe_job_t*)malloc((size_t)threads * sizeof(moe_job_t));
  pthread_t* th = (pthread_t*)malloc((size_t)threads * sizeof(pthread_t));
  for (int i = 0; i < threads; ++i) {
    moe_job_t j = {tokens, tw, w13, w2, wbf16, ti, out, act_out, y_out,
                   T,      E,  H,   topk, I,    i,  threads};
    jobs[i] = j;
  }
  for (int i = 1; i < threads; ++i) pthread_create(&th[i], NULL, moe_worker, &jobs[i]);
  moe_worker(&jobs[0]);
  for (int i = 1; i < threads; ++i) pthread_join(th[i], NULL);
  free(jobs);
  free(th);
  if (!topk_w_out) free(tw);
  if (!topk_idx_out) free(ti);
}

void oracle_full_moe(const float* tokens, const float* gate_w, const float* w13,
                     const float* w2, int T, int E, int H, int topk, int I,
                     float* out, float* topk_w_out, int* topk_idx_out,
                     float* act_out, float* y_out, int threads) {
  full_moe_any(tokens, gate_w, w13, w2, 0, T, E, H, topk, I, out, topk_w_out, topk_idx_out, act_out,
               y_out, threads);
}

/* The full layer with the expert weights stored as bf16 (see oracle_gemm_nt_bw): same results
 * as oracle_full_moe on the widened weights. */
void oracle_full_moe_bw(const float* tokens, const float* gate_w, const unsigned short* w13,
                        const unsigned short* w2, int T, int E, int H, int topk, int I,
                        float* out, float* topk_w_out, int* topk_idx_out, int threads) {
  full_moe_any(tokens, gate_w, w13, w2, 1, T, E, H, topk, I, out, topk_w_out, topk_idx_out, NULL, NULL,
               threads);
}

/* Host cores available to this process. */
int oracle_max_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n < 1 ? 1 : (int)n;
}

/* The reference's test-input stream: libc rand() seeded once with 7907, each
 * value lo + (rand()/RAND_MAX)*(hi-lo) in float arithmetic.  Successive calls
 * continue the same stream (tokens, gate, FFN1, FFN2 weights in that order).
 * Follows test/common/utils.h:9,62-86 and test/common/moeTools.h:45-69. */
void oracle_rand_uniform_fill(float* dst, size_t n, float lo, float hi,
                              int reseed) {
  if (reseed) srand(7907u);
  for (size_t i = 0; i < n; ++i) {
    float r01 = (float)rand() / (float)RAND_MAX;
    dst[i] = lo + r01 * (hi - lo);
  }
}
