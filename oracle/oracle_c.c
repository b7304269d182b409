/*
 * Plain-C restatement of the two hot paths.  TEST INFRASTRUCTURE ONLY: built
 * into oracle/_build/liboracle.so and loaded by tests (single-threaded: gcc has no OpenMP
 * runtime in this image); the product library never links or calls it.
 *
 * GEMM follows the reference's index arithmetic a[i*K+k], b[k*N+j], c[i*N+j]
 * (kernels/gemm/pkg/gemm_unified/csrc/auto/gemm_0.cu:12-20) with fp32
 * accumulation.  FMHA follows the blocked online-softmax recurrences of
 * kernels/fmha/pkg/fmha_unified/csrc/semi/fmha_2_nv.cu:173-208 (running max m,
 * running sum l, rescale of O by exp(m_old - m_new)) and the final O / l of
 * :283, with the GQA mapping of :36,42-45, in fp32 instead of the reference's
 * fp16 statistics.  Keys at index >= kv_len are masked (the reference's
 * `k_idx > decode_length`, :181, leaves one key too many; not reproduced).
 *
 * Parity of this file is pinned through oracle.py's golden fixtures
 * (tests/golden/): tests compare it with them.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while (!(man & 0x400u));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static inline float bf16_to_f32(uint16_t h) {
  uint32_t bits = (uint32_t)h << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static void widen(const uint16_t* src, float* dst, size_t n, int is_bf16) {
  for (long i = 0; i < (long)n; ++i) dst[i] = is_bf16 ? bf16_to_f32(src[i]) : f16_to_f32(src[i]);
}

/* c[M,N] (fp32) = a[M,K] . b[K,N]; a, b are 16-bit (fp16 or bf16) bit patterns. */
int oracle_gemm(const uint16_t* a, const uint16_t* b, float* c, int M, int N, int K, int is_bf16) {
  float* af = (float*)malloc((size_t)M * K * sizeof(float));
  float* bf = (float*)malloc((size_t)K * N * sizeof(float));
  if (!af || !bf) {
    free(af);
    free(bf);
    return -1;
  }
  widen(a, af, (size_t)M * K, is_bf16);
  widen(b, bf, (size_t)K * N, is_bf16);
  for (int i = 0; i < M; ++i) {
    float* ci = c + (size_t)i * N;
    for (int j = 0; j < N; ++j) ci[j] = 0.f;
    for (int k = 0; k < K; ++k) {
      const float aik = af[(size_t)i * K + k];
      const float* bk = bf + (size_t)k * N;
      for (int j = 0; j < N; ++j) ci[j] += aik * bk[j];
    }
  }
  free(af);
  free(bf);
  return 0;
}

/*
 * o[B,Hq,Sq,D] (fp32) from contiguous 16-bit q [B,Hq,Sq,D], k, v [B,Hkv,Skv,D].
 * kv_lens: int32[B] or NULL (= Skv).  causal: key j visible to query i when
 * j <= i + (len - Sq).  Key blocks of 64 as in the reference kernels.
 */
int oracle_fmha(const uint16_t* q, const uint16_t* k, const uint16_t* v, float* o, int B, int Hq, int Hkv, int Sq,
                int Skv, int D, int causal, const int32_t* kv_lens, int is_bf16) {
  const int group = Hq / Hkv;
  const float scale = 1.0f / sqrtf((float)D);
  enum { BLK = 64 };
  int rc = 0;
  for (int b = 0; b < B; ++b) {
    for (int h = 0; h < Hq; ++h) {
      const int n = kv_lens ? kv_lens[b] : Skv;
      const int hk = h / group;
      const uint16_t* kh = k + ((size_t)b * Hkv + hk) * (size_t)Skv * D;
      const uint16_t* vh = v + ((size_t)b * Hkv + hk) * (size_t)Skv * D;
      float* qf = (float*)malloc((size_t)D * sizeof(float));
      float* acc = (float*)malloc((size_t)D * sizeof(float));
      if (!qf || !acc) {
        rc = -1;
        free(qf);
        free(acc);
        continue;
      }
      for (int i = 0; i < Sq; ++i) {
        const uint16_t* qi = q + (((size_t)b * Hq + h) * Sq + i) * D;
        float* oi = o + (((size_t)b * Hq + h) * Sq + i) * D;
        for (int d = 0; d < D; ++d) {
          qf[d] = is_bf16 ? bf16_to_f32(qi[d]) : f16_to_f32(qi[d]);
          acc[d] = 0.f;
        }
        float m = -INFINITY, l = 0.f;
        const int last = causal ? i + (n - Sq) : n - 1; /* last visible key */
        const int hi = last < n - 1 ? last : n - 1;
        for (int j0 = 0; j0 <= hi; j0 += BLK) {
          const int j1 = j0 + BLK <= hi + 1 ? j0 + BLK : hi + 1;
          float s[BLK];
          float bmax = -INFINITY;
          for (int j = j0; j < j1; ++j) {
            const uint16_t* kj = kh + (size_t)j * D;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot += qf[d] * (is_bf16 ? bf16_to_f32(kj[d]) : f16_to_f32(kj[d]));
            s[j - j0] = dot * scale;
            if (s[j - j0] > bmax) bmax = s[j - j0];
          }
          const float m_new = m > bmax ? m : bmax;
          const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
          float rowsum = 0.f;
          for (int d = 0; d < D; ++d) acc[d] *= alpha;
          for (int j = j0; j < j1; ++j) {
            const float p = expf(s[j - j0] - m_new);
            rowsum += p;
            const uint16_t* vj = vh + (size_t)j * D;
            for (int d = 0; d < D; ++d) acc[d] += p * (is_bf16 ? bf16_to_f32(vj[d]) : f16_to_f32(vj[d]));
          }
          l = alpha * l + rowsum;
          m = m_new;
        }
        for (int d = 0; d < D; ++d) oi[d] = l > 0.f ? acc[d] / l : 0.f;
      }
      free(qf);
      free(acc);
    }
  }
  return rc;
}
