/* Oracle, plain C -- TEST INFRASTRUCTURE, never on the product path.
 *
 * An independent restatement of the reference's numeric check
 * (backend/node/run_tma.py:67: fp32 matmul of the fp16 operands, C = A . Bt^T) as a triple
 * loop, with its own fp16 decoder, so the numpy oracle (oracle/gemm_ref.py) is checked by
 * code that shares nothing with it.  Also the sampled exact check of
 * backend/node/cublas_q7.cpp:26,91-97 on the index-hash inputs.
 *
 * Build: make -C oracle   ->  oracle/liboracle_gemm.so
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

static float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do { man <<= 1; e++; } while (!(man & 0x400u));
      bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3ffu) << 13;
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | man << 13;
  } else {
    bits = sign | (exp + 127 - 15) << 23 | man << 13;
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* C[m,n] = A[m,k] . Bt[n,k]^T, fp16 bit patterns in, fp32 out, fp32 accumulation in k order */
void oracle_gemm_f16_f32(const uint16_t* a, const uint16_t* bt, float* c, int m, int n, int k) {
  for (int i = 0; i < m; i++)
    for (int j = 0; j < n; j++) {
      float acc = 0.0f;
      const uint16_t *ra = a + (size_t)i * k, *rb = bt + (size_t)j * k;
      for (int p = 0; p < k; p++) acc += half_to_float(ra[p]) * half_to_float(rb[p]);
      c[(size_t)i * n + j] = acc;
    }
}

/* same, accumulated in double: the bound the fp32 results are compared with on uniform inputs */
void oracle_gemm_f16_f64(const uint16_t* a, const uint16_t* bt, double* c, int m, int n, int k) {
  for (int i = 0; i < m; i++)
    for (int j = 0; j < n; j++) {
      double acc = 0.0;
      const uint16_t *ra = a + (size_t)i * k, *rb = bt + (size_t)j * k;
      for (int p = 0; p < k; p++) acc += (double)half_to_float(ra[p]) * (double)half_to_float(rb[p]);
      c[(size_t)i * n + j] = acc;
    }
}

static int hash_val(uint64_t i, uint64_t salt) { return (int)(((i * 2654435761ull + salt) >> 13) % 7) - 3; }

/* entries of the index-hash inputs (salt 1 for A, 7 for Bt) */
void oracle_hash_fill(int16_t* out, size_t count, uint64_t salt) {
  for (size_t i = 0; i < count; i++) out[i] = (int16_t)hash_val(i, salt);
}

/* exact value of C[i,j] on the index-hash inputs */
long oracle_hash_entry(int i, int j, int k) {
  long ref = 0;
  for (int p = 0; p < k; p++) ref += (long)hash_val((uint64_t)i * k + p, 1) * hash_val((uint64_t)j * k + p, 7);
  return ref;
}

/* number of the 64 sampled entries of c that differ from the exact value */
int oracle_hash_sampled_wrong(const float* c, int m, int n, int k) {
  int bad = 0;
  for (int s = 0; s < 64; s++) {
    int i = (int)((s * 7919ull + 13) % m), j = (int)((s * 104729ull + 5) % n);
    if ((double)c[(size_t)i * n + j] != (double)oracle_hash_entry(i, j, k)) bad++;
  }
  return bad;
}
