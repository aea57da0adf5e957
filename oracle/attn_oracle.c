/*
 * attn_oracle.c — CPU restatement of the reference's attention semantics.
 * TEST INFRASTRUCTURE ONLY: tests, the smoke check and the benchmark's CPU
 * baseline leg may call this; no product path does.
 *
 * What it restates (dsuarez01/minfer-python):
 *   src/minfer/kernels/refs.py:53-55   flash_attn = scaled_dot_product_attention
 *       (Q, K, V, attn_mask=mask), default scale 1/sqrt(head_dim), bool mask with
 *       True = attend
 *   test/kernels.py:253-255            grouped-query expansion of K/V with
 *       repeat_interleave(n_rep, dim=1): query head h reads kv head h / n_rep
 *   test/kernels.py:242                causal mask  j <= i
 * The arithmetic itself lives in PyTorch ATen's SDPA (torch 2.10.0 pinned in
 * the reference's uv.lock:601-602), which is not part of the reference tree;
 * this file restates the published definition
 *     out = softmax(q k^T * scale + mask) v
 * with double-precision accumulation.  Rows with no visible key give zeros,
 * which is what torch's CPU SDPA returns for them.
 *
 * Layout: contiguous fp32 q,out [B,H,Lq,D]; k,v [B,Hkv,Lk,D]; mask (optional)
 * bytes [B,1,Lq,Lk]; lens (optional) int32 [B] limits keys to [0, lens[b]).
 * Only query rows [row0, row1) are computed (others left untouched), so a
 * test can check row blocks of a large problem.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

int attn_oracle_f32(const float* q, const float* k, const float* v, const uint8_t* mask, const int32_t* lens,
                    float* out, int B, int H, int Hkv, int Lq, int Lk, int D, float scale, int causal, int row0,
                    int row1) {
  if (B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || Lq <= 0 || Lk <= 0 || D <= 0) return 1;
  if (row0 < 0) row0 = 0;
  if (row1 > Lq) row1 = Lq;
  const int group = H / Hkv;
  const int off = Lk - Lq;
  if (scale == 0.0f) scale = (float)(1.0 / sqrt((double)D));
  const long nrows = (long)B * H * (row1 - row0);
  int fail = 0;
#pragma omp parallel
  {
    double* s = (double*)malloc(sizeof(double) * (size_t)Lk);
    double* acc = (double*)malloc(sizeof(double) * (size_t)D);
    if (!s || !acc) {
#pragma omp atomic write
      fail = 1;
    } else {
#pragma omp for schedule(dynamic, 16)
      for (long idx = 0; idx < nrows; ++idx) {
        const int i = row0 + (int)(idx % (row1 - row0));
        const int h = (int)((idx / (row1 - row0)) % H);
        const int b = (int)(idx / ((long)(row1 - row0) * H));
        const int kvh = h / group;
        const float* qr = q + (((size_t)b * H + h) * Lq + i) * D;
        const float* kb = k + ((size_t)b * Hkv + kvh) * (size_t)Lk * D;
        const float* vb = v + ((size_t)b * Hkv + kvh) * (size_t)Lk * D;
        const uint8_t* mr = mask ? mask + ((size_t)b * Lq + i) * Lk : NULL;
        int lim = Lk;
        if (lens) lim = lens[b] < Lk ? lens[b] : Lk;
        double mx = -INFINITY;
        for (int j = 0; j < Lk; ++j) {
          int vis = j < lim;
          if (causal && j > i + off) vis = 0;
          if (mr && !mr[j]) vis = 0;
          if (!vis) {
            s[j] = -INFINITY;
            continue;
          }
          double d = 0.0;
          const float* kr = kb + (size_t)j * D;
          for (int e = 0; e < D; ++e) d += (double)qr[e] * (double)kr[e];
          s[j] = d * (double)scale;
          if (s[j] > mx) mx = s[j];
        }
        float* o = out + (((size_t)b * H + h) * Lq + i) * D;
        if (mx == -INFINITY) {
          for (int e = 0; e < D; ++e) o[e] = 0.0f;
          continue;
        }
        double l = 0.0;
        for (int e = 0; e < D; ++e) acc[e] = 0.0;
        for (int j = 0; j < Lk; ++j) {
          if (s[j] == -INFINITY) continue;
          const double p = exp(s[j] - mx);
          l += p;
          const float* vr = vb + (size_t)j * D;
          for (int e = 0; e < D; ++e) acc[e] += p * (double)vr[e];
        }
        for (int e = 0; e < D; ++e) o[e] = (float)(acc[e] / l);
      }
    }
    free(s);
    free(acc);
  }
  return fail ? 2 : 0;
}
