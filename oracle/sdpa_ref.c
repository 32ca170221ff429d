/*
 * Plain-C restatement of the attention math, fp64 accumulation. TEST INFRASTRUCTURE ONLY:
 * tests/ and bench.py's CPU-baseline leg may load it as a checker; the product never does.
 *
 * Follows the reference's test oracle attention_ref
 * (test/torch_ops/test_scaled_dot_product_attention.py:78-161): scores = (q*scale) k^T,
 * bottom-right causal mask col > row + Lk - Lq (:69), GQA by repeating each KV head over
 * Hq/Hkv consecutive query heads (:119-120), softmax, rows without a visible key give 0
 * (:143-147), out = P v. logsumexp is the natural log of the row sum of exp(scores), the
 * quantity mha_varlen_fwd returns (FlashAttention_internal.cpp:129). The backward is the
 * analytic gradient of that forward (what the reference tests obtain by autograd, :1018-1075):
 *   dV = P^T dO, dP = dO V^T, dS = P o (dP - rowsum(P o dP)), dQ = scale dS K, dK = scale dS^T Q.
 * Tensors are contiguous fp32: q/out/dout/dq [B,Hq,Lq,D], k/v/dk/dv [B,Hkv,Lk,D], lse [B,Hq,Lq].
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

static int visible(int causal, int i, int j, int lq, int lk) { return !causal || j <= i + lk - lq; }

void sdpa_ref_forward(const float* q, const float* k, const float* v, float* out, float* lse, int B,
                      int Hq, int Hkv, int Lq, int Lk, int D, float scale, int causal) {
  const int g = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    for (int h = 0; h < Hq; ++h) {
      double* s = (double*)malloc(sizeof(double) * (size_t)Lk);
      double* acc = (double*)malloc(sizeof(double) * (size_t)D);
      const float* kb = k + ((size_t)b * Hkv + h / g) * Lk * D;
      const float* vb = v + ((size_t)b * Hkv + h / g) * Lk * D;
      for (int i = 0; i < Lq; ++i) {
        const float* qi = q + (((size_t)b * Hq + h) * Lq + i) * D;
        double mx = -INFINITY;
        for (int j = 0; j < Lk; ++j) {
          if (!visible(causal, i, j, Lq, Lk)) { s[j] = -INFINITY; continue; }
          double d = 0.0;
          for (int c = 0; c < D; ++c) d += (double)qi[c] * (double)scale * (double)kb[(size_t)j * D + c];
          s[j] = d;
          if (d > mx) mx = d;
        }
        double sum = 0.0;
        memset(acc, 0, sizeof(double) * (size_t)D);
        if (mx > -INFINITY) {
          for (int j = 0; j < Lk; ++j) {
            if (s[j] == -INFINITY) continue;
            const double p = exp(s[j] - mx);
            sum += p;
            for (int c = 0; c < D; ++c) acc[c] += p * (double)vb[(size_t)j * D + c];
          }
        }
        float* oi = out + (((size_t)b * Hq + h) * Lq + i) * D;
        for (int c = 0; c < D; ++c) oi[c] = (float)(sum > 0.0 ? acc[c] / sum : 0.0);
        lse[((size_t)b * Hq + h) * Lq + i] = (float)(sum > 0.0 ? mx + log(sum) : INFINITY);
      }
      free(s);
      free(acc);
    }
  }
}

void sdpa_ref_backward(const float* q, const float* k, const float* v, const float* dout, float* dq,
                       float* dk, float* dv, int B, int Hq, int Hkv, int Lq, int Lk, int D,
                       float scale, int causal) {
  const int g = Hq / Hkv;
  memset(dk, 0, sizeof(float) * (size_t)B * Hkv * Lk * D);
  memset(dv, 0, sizeof(float) * (size_t)B * Hkv * Lk * D);
  /* parallel over (batch, kv head): the query heads of one group accumulate into the same dk/dv */
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    for (int hk = 0; hk < Hkv; ++hk) {
      double* p = (double*)malloc(sizeof(double) * (size_t)Lk);
      double* dp = (double*)malloc(sizeof(double) * (size_t)Lk);
      double* dkd = (double*)calloc((size_t)Lk * D, sizeof(double));
      double* dvd = (double*)calloc((size_t)Lk * D, sizeof(double));
      const float* kb = k + ((size_t)b * Hkv + hk) * Lk * D;
      const float* vb = v + ((size_t)b * Hkv + hk) * Lk * D;
      for (int h = hk * g; h < (hk + 1) * g; ++h) {
        for (int i = 0; i < Lq; ++i) {
          const size_t row = (((size_t)b * Hq + h) * Lq + i) * D;
          const float* qi = q + row;
          const float* doi = dout + row;
          double mx = -INFINITY;
          for (int j = 0; j < Lk; ++j) {
            if (!visible(causal, i, j, Lq, Lk)) { p[j] = -INFINITY; continue; }
            double d = 0.0;
            for (int c = 0; c < D; ++c) d += (double)qi[c] * (double)scale * (double)kb[(size_t)j * D + c];
            p[j] = d;
            if (d > mx) mx = d;
          }
          double sum = 0.0;
          for (int j = 0; j < Lk; ++j) {
            p[j] = (p[j] == -INFINITY || mx == -INFINITY) ? 0.0 : exp(p[j] - mx);
            sum += p[j];
          }
          double delta = 0.0;
          for (int j = 0; j < Lk; ++j) {
            p[j] = sum > 0.0 ? p[j] / sum : 0.0;
            double d = 0.0;
            for (int c = 0; c < D; ++c) d += (double)doi[c] * (double)vb[(size_t)j * D + c];
            dp[j] = d;
            delta += p[j] * d;
          }
          float* dqi = dq + row;
          for (int c = 0; c < D; ++c) dqi[c] = 0.f;
          double dqa[512];
          for (int c = 0; c < D; ++c) dqa[c] = 0.0;
          for (int j = 0; j < Lk; ++j) {
            if (p[j] == 0.0) continue;
            const double ds = p[j] * (dp[j] - delta) * (double)scale;
            for (int c = 0; c < D; ++c) {
              dqa[c] += ds * (double)kb[(size_t)j * D + c];
              dkd[(size_t)j * D + c] += ds * (double)qi[c];
              dvd[(size_t)j * D + c] += p[j] * (double)doi[c];
            }
          }
          for (int c = 0; c < D; ++c) dqi[c] = (float)dqa[c];
        }
      }
      float* dkb = dk + ((size_t)b * Hkv + hk) * Lk * D;
      float* dvb = dv + ((size_t)b * Hkv + hk) * Lk * D;
      for (size_t x = 0; x < (size_t)Lk * D; ++x) {
        dkb[x] = (float)dkd[x];
        dvb[x] = (float)dvd[x];
      }
      free(p);
      free(dp);
      free(dkd);
      free(dvd);
    }
  }
}
