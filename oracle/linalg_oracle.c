/* CPU oracle for the IMEX hot path — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * See linalg_oracle.h for what it restates and which reference files each
 * function follows.  Build: gcc -O2 -ffp-contract=off -fno-fast-math
 * (mulf and addf must stay two separately rounded operations). */
#include "linalg_oracle.h"

#include <float.h>
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
#define ORACLE_CLONES __attribute__((target_clones("avx2", "default")))
#else
#define ORACLE_CLONES
#endif

/* ------------------------------------------------------------------------
 * 16-bit floats.  bf16 -> f32 is bits<<16 (ImexRunnerUtils.cpp:165-169);
 * f16 -> f32 is exact; f32 -> 16-bit rounds to nearest even (what
 * arith.truncf and the bf16(float)/f16(float) constructors of upstream
 * Float16bits do). */
float oracle_bf16_to_f32(uint16_t bits) {
  uint32_t u = (uint32_t)bits << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t oracle_f32_to_bf16(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) /* NaN: keep quiet bit */
    return (uint16_t)((u >> 16) | 0x0040u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

float oracle_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while (!(man & 0x400u));
      man &= 0x3ffu;
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t oracle_f32_to_f16(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  uint32_t a = u & 0x7fffffffu;
  if (a > 0x7f800000u)
    return (uint16_t)(sign | 0x7e00u);
  if (a >= 0x47800000u) /* >= 65536 -> inf (65520 rounds up too, below) */
    return (uint16_t)(sign | 0x7c00u);
  if (a < 0x33000000u) /* < 2^-25 -> 0 */
    return sign;
  int32_t e = (int32_t)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;
  int shift;
  uint32_t base;
  if (e < -14) { /* subnormal half */
    shift = 13 + (-14 - e);
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(e + 15) << 10;
    m &= 0x7fffffu;
  }
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u)))
    ++q;
  uint32_t r = base + q; /* mantissa carry rolls into the exponent */
  if (r >= 0x7c00u)
    r = 0x7c00u;
  return (uint16_t)(sign | r);
}

void oracle_round_to_bf16(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    dst[i] = oracle_f32_to_bf16(src[i]);
}

void oracle_round_to_f16(const float *src, uint16_t *dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    dst[i] = oracle_f32_to_f16(src[i]);
}

/* ------------------------------------------------------------------------
 * matmul */
void oracle_matmul_f32_loops(const float *A, const float *B, float *C,
                             int64_t M, int64_t N, int64_t K) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j)
      for (int64_t k = 0; k < K; ++k) {
        float p = A[i * K + k] * B[k * N + j];
        volatile float *c = &C[i * N + j]; /* load/store per point, as the loops do */
        *c = *c + p;
      }
}

ORACLE_CLONES
static void matmul_row_block_f32(const float *A, const float *B, float *C,
                                 int64_t i0, int64_t i1, int64_t N, int64_t K) {
  for (int64_t i = i0; i < i1; ++i) {
    float *restrict c = C + i * N;
    for (int64_t k = 0; k < K; ++k) {
      const float a = A[i * K + k];
      const float *restrict b = B + k * N;
      for (int64_t j = 0; j < N; ++j) {
        float p = a * b[j];
        c[j] = c[j] + p;
      }
    }
  }
}

/* Rows are independent, so splitting them over threads changes no result. */
typedef struct {
  const float *A, *B;
  float *C;
  int64_t i0, i1, N, K;
} RowJob;

static void *row_job_main(void *p) {
  RowJob *j = (RowJob *)p;
  matmul_row_block_f32(j->A, j->B, j->C, j->i0, j->i1, j->N, j->K);
  return NULL;
}

static int oracle_threads(void) {
  const char *e = getenv("ORACLE_THREADS");
  long n = e ? strtol(e, NULL, 10) : sysconf(_SC_NPROCESSORS_ONLN);
  if (n < 1)
    n = 1;
  if (n > 64)
    n = 64;
  return (int)n;
}

void oracle_matmul_f32_fast(const float *A, const float *B, float *C,
                            int64_t M, int64_t N, int64_t K) {
  int nt = oracle_threads();
  if (nt > M)
    nt = M > 0 ? (int)M : 1;
  pthread_t tid[64];
  RowJob job[64];
  for (int t = 0; t < nt; ++t) {
    job[t] = (RowJob){A, B, C, M * t / nt, M * (t + 1) / nt, N, K};
    if (t == nt - 1 || pthread_create(&tid[t], NULL, row_job_main, &job[t]) != 0) {
      row_job_main(&job[t]);
      tid[t] = 0;
    }
  }
  for (int t = 0; t < nt - 1; ++t)
    if (tid[t])
      pthread_join(tid[t], NULL);
}

static inline float x16_to_f32(uint16_t v, int is_bf16) {
  return is_bf16 ? oracle_bf16_to_f32(v) : oracle_f16_to_f32(v);
}

void oracle_matmul_x16_f32_loops(const uint16_t *A, const uint16_t *B,
                                 float *C, int64_t M, int64_t N, int64_t K,
                                 int is_bf16) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j)
      for (int64_t k = 0; k < K; ++k) {
        float a = x16_to_f32(A[i * K + k], is_bf16);
        float b = x16_to_f32(B[k * N + j], is_bf16);
        float p = a * b;
        volatile float *c = &C[i * N + j];
        *c = *c + p;
      }
}

void oracle_matmul_x16_f32_rows(const uint16_t *A, const uint16_t *B, float *C,
                                int64_t row0, int64_t nrows, int64_t N,
                                int64_t K, int is_bf16) {
  /* B extended once; extension is exact so per-element arithmetic is the
   * same as extending inside the loop. */
  float *Bf = (float *)malloc((size_t)K * (size_t)N * sizeof(float));
  float *Af = (float *)malloc((size_t)nrows * (size_t)K * sizeof(float));
  if (!Bf || !Af)
    abort();
  for (int64_t k = 0; k < K; ++k)
    for (int64_t j = 0; j < N; ++j)
      Bf[k * N + j] = x16_to_f32(B[k * N + j], is_bf16);
  for (int64_t i = 0; i < nrows; ++i)
    for (int64_t k = 0; k < K; ++k)
      Af[i * K + k] = x16_to_f32(A[(row0 + i) * K + k], is_bf16);
  oracle_matmul_f32_fast(Af, Bf, C, nrows, N, K);
  free(Af);
  free(Bf);
}

void oracle_matmul_x16_f32_fast(const uint16_t *A, const uint16_t *B, float *C,
                                int64_t M, int64_t N, int64_t K, int is_bf16) {
  oracle_matmul_x16_f32_rows(A, B, C, 0, M, N, K, is_bf16);
}

void oracle_bias_add_f32(float *C, const float *bias, int64_t M, int64_t N) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j)
      C[i * N + j] = C[i * N + j] + bias[j];
}

/* ------------------------------------------------------------------------
 * elementwise */
void oracle_relu_f32(const float *x, float *y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    float v = x[i];
    int ugt = !(v <= 0.0f); /* unordered-or-greater: NaN passes through */
    y[i] = ugt ? v : 0.0f;
  }
}

void oracle_silu_f32(const float *x, float *y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    float v = x[i];
    float e = expf(-v);
    float d = e + 1.0f;
    float s = 1.0f / d;
    y[i] = s * v;
  }
}

void oracle_epilogue_f32(float *c, int64_t n, int epilogue) {
  if (epilogue == ORACLE_EPI_RELU)
    oracle_relu_f32(c, c, n);
  else if (epilogue == ORACLE_EPI_SILU)
    oracle_silu_f32(c, c, n);
}

static inline float maximumf_(float a, float b);

/* ------------------------------------------------------------------------
 * attention forward, as the reference test's cpu_impl computes it */
typedef struct {
  const uint16_t *Q, *K, *V;
  uint16_t *O;
  int64_t r0, r1, n_ctx, d_head;
  float sm_scale;
  int is_bf16;
} AttnJob;

static void *attn_job_main(void *arg) {
  AttnJob *a = (AttnJob *)arg;
  const int64_t n = a->n_ctx, d = a->d_head;
  const float log2e = 1.442695040888963f;
  float *s = (float *)malloc(sizeof(float) * (size_t)n);
  float *q = (float *)malloc(sizeof(float) * (size_t)d);
  float *pv = (float *)malloc(sizeof(float) * (size_t)d);
  for (int64_t row = a->r0; row < a->r1; ++row) {
    const int64_t head = row / n, base = head * n;
    for (int64_t k = 0; k < d; ++k)
      q[k] = x16_to_f32(a->Q[row * d + k], a->is_bf16);
    for (int64_t j = 0; j < n; ++j) {
      float acc = 0.0f;
      const uint16_t *kr = a->K + (base + j) * d;
      for (int64_t k = 0; k < d; ++k) {
        float t = q[k] * x16_to_f32(kr[k], a->is_bf16);
        acc = acc + t;
      }
      s[j] = acc * a->sm_scale;
    }
    float mx = -INFINITY;
    for (int64_t j = 0; j < n; ++j)
      mx = maximumf_(mx, s[j]);
    for (int64_t j = 0; j < n; ++j) {
      float t = s[j] - mx;
      float t1 = t * log2e;
      s[j] = exp2f(t1);
    }
    float sum = 0.0f;
    for (int64_t j = 0; j < n; ++j)
      sum = sum + s[j];
    for (int64_t j = 0; j < n; ++j)
      s[j] = s[j] / sum;
    for (int64_t c = 0; c < d; ++c)
      pv[c] = 0.0f;
    for (int64_t j = 0; j < n; ++j) { /* same per-(row, c) order as the k loop of the test */
      const float p = a->is_bf16 ? oracle_bf16_to_f32(oracle_f32_to_bf16(s[j]))
                                 : oracle_f16_to_f32(oracle_f32_to_f16(s[j]));
      const uint16_t *vr = a->V + (base + j) * d;
      for (int64_t c = 0; c < d; ++c) {
        float t = p * x16_to_f32(vr[c], a->is_bf16);
        pv[c] = t + pv[c];
      }
    }
    for (int64_t c = 0; c < d; ++c)
      a->O[row * d + c] = a->is_bf16 ? oracle_f32_to_bf16(pv[c]) : oracle_f32_to_f16(pv[c]);
  }
  free(s);
  free(q);
  free(pv);
  return NULL;
}

void oracle_attention_fwd_x16(const uint16_t *Q, const uint16_t *K, const uint16_t *V, uint16_t *O,
                              int64_t heads, int64_t n_ctx, int64_t d_head, float sm_scale,
                              int is_bf16) {
  const int64_t rows = heads * n_ctx;
  int nt = oracle_threads();
  if (nt > rows)
    nt = rows > 0 ? (int)rows : 1;
  pthread_t tid[64];
  AttnJob job[64];
  for (int t = 0; t < nt; ++t) {
    job[t] = (AttnJob){Q, K, V, O, rows * t / nt, rows * (t + 1) / nt, n_ctx, d_head, sm_scale, is_bf16};
    if (t == nt - 1 || pthread_create(&tid[t], NULL, attn_job_main, &job[t]) != 0) {
      attn_job_main(&job[t]);
      tid[t] = 0;
    }
  }
  for (int t = 0; t < nt - 1; ++t)
    if (tid[t])
      pthread_join(tid[t], NULL);
}

/* ------------------------------------------------------------------------
 * single elementwise generics in the IR's element type */
static inline float minimumf_(float a, float b) {
  if (a != a || b != b)
    return NAN;
  if (a < b)
    return a;
  if (b < a)
    return b;
  return signbit(a) ? a : b; /* minimumf(+0,-0) = -0 */
}

float oracle_round_as(float v, int dtype) {
  if (dtype == ORACLE_DT_BF16)
    return oracle_bf16_to_f32(oracle_f32_to_bf16(v));
  if (dtype == ORACLE_DT_F16)
    return oracle_f16_to_f32(oracle_f32_to_f16(v));
  return v;
}

int oracle_unary(int op, int dtype, const float *x, float *y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    float v = x[i], r;
    switch (op) {
    case ORACLE_OP_NEGF: r = -v; break;
    case ORACLE_OP_ABSF: r = fabsf(v); break;
    case ORACLE_OP_LOG: r = logf(v); break;
    case ORACLE_OP_EXP: r = expf(v); break;
    case ORACLE_OP_SQRT: r = sqrtf(v); break;
    case ORACLE_OP_RSQRT: r = 1.0f / sqrtf(v); break;
    case ORACLE_OP_TANH: r = tanhf(v); break;
    case ORACLE_OP_RELU: r = !(v <= 0.0f) ? v : 0.0f; break; /* cmpf ugt ; select */
    default: return -1;
    }
    y[i] = oracle_round_as(r, dtype);
  }
  return 0;
}

int oracle_binary(int op, int dtype, const float *a, const float *b, float *y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    float r;
    switch (op) {
    case ORACLE_OP_ADDF: r = a[i] + b[i]; break;
    case ORACLE_OP_SUBF: r = a[i] - b[i]; break;
    case ORACLE_OP_MULF: r = a[i] * b[i]; break;
    case ORACLE_OP_DIVF: r = a[i] / b[i]; break;
    case ORACLE_OP_MAXIMUMF: r = maximumf_(a[i], b[i]); break;
    case ORACLE_OP_MINIMUMF: r = minimumf_(a[i], b[i]); break;
    default: return -1;
    }
    y[i] = oracle_round_as(r, dtype);
  }
  return 0;
}

void oracle_reduce_leading_as(int dtype, const float *x, float *y, int64_t lead, int64_t inner) {
  for (int64_t j = 0; j < inner; ++j)   /* d0: the output element */
    for (int64_t i = 0; i < lead; ++i)  /* d1: the reduction */
      y[j] = oracle_round_as(y[j] + x[i * inner + j], dtype);
}

/* ------------------------------------------------------------------------
 * softmax: the chain of generics with its full-size temporaries */
static inline float maximumf_(float a, float b) {
  if (a != a || b != b)
    return NAN;
  if (a > b)
    return a;
  if (b > a)
    return b;
  return signbit(a) ? b : a; /* maximumf(+0,-0) = +0 */
}

void oracle_softmax_f32(const float *x, float *y, int64_t rows, int64_t cols,
                        int flavour) {
  float *mx = (float *)malloc((size_t)(rows > 0 ? rows : 1) * sizeof(float));
  float *sm = (float *)malloc((size_t)(rows > 0 ? rows : 1) * sizeof(float));
  float *t = (float *)malloc((size_t)(rows * cols > 0 ? rows * cols : 1) * sizeof(float));
  if (!mx || !sm || !t)
    abort();
  for (int64_t r = 0; r < rows; ++r)
    mx[r] = flavour == ORACLE_SOFTMAX_PLAIDML ? -INFINITY : -FLT_MAX;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) {
      float in = x[r * cols + c], out = mx[r];
      if (flavour == ORACLE_SOFTMAX_PLAIDML)
        mx[r] = (in > out) ? in : out; /* cmpf ogt in,out ; select in,out */
      else
        mx[r] = maximumf_(in, out);
    }
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c)
      t[r * cols + c] = x[r * cols + c] - mx[r];
  for (int64_t i = 0; i < rows * cols; ++i)
    t[i] = expf(t[i]);
  for (int64_t r = 0; r < rows; ++r)
    sm[r] = 0.0f;
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) {
      volatile float *s = &sm[r];
      *s = t[r * cols + c] + *s;
    }
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c)
      y[r * cols + c] = t[r * cols + c] / sm[r];
  free(t);
  free(sm);
  free(mx);
}

/* ------------------------------------------------------------------------
 * reductions */
void oracle_reduce_rows_f32(const float *x, float *y, int64_t rows,
                            int64_t cols) {
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < cols; ++c) {
      volatile float *o = &y[r];
      *o = *o + x[r * cols + c];
    }
}

void oracle_reduce_leading_f32(const float *x, float *y, int64_t lead,
                               int64_t inner) {
  for (int64_t i = 0; i < inner; ++i)
    for (int64_t l = 0; l < lead; ++l) {
      volatile float *o = &y[i];
      *o = *o + x[l * inner + i];
    }
}

void oracle_reduce_all_f32(const float *x, float *y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    volatile float *o = y;
    *o = *o + x[i];
  }
}

/* ------------------------------------------------------------------------
 * transpose */
void oracle_transpose2d_b32(const uint32_t *x, uint32_t *y, int64_t rows,
                            int64_t cols) {
  for (int64_t i = 0; i < rows; ++i)
    for (int64_t j = 0; j < cols; ++j)
      y[j * rows + i] = x[i * cols + j];
}

void oracle_transpose2d_b16(const uint16_t *x, uint16_t *y, int64_t rows,
                            int64_t cols) {
  for (int64_t i = 0; i < rows; ++i)
    for (int64_t j = 0; j < cols; ++j)
      y[j * rows + i] = x[i * cols + j];
}

void oracle_transpose3d_b32(const uint32_t *x, uint32_t *y, const int64_t *dims,
                            const int *perm) {
  int64_t od[3] = {dims[perm[0]], dims[perm[1]], dims[perm[2]]};
  int64_t idx[3];
  for (idx[0] = 0; idx[0] < dims[0]; ++idx[0])
    for (idx[1] = 0; idx[1] < dims[1]; ++idx[1])
      for (idx[2] = 0; idx[2] < dims[2]; ++idx[2]) {
        int64_t o0 = idx[perm[0]], o1 = idx[perm[1]], o2 = idx[perm[2]];
        y[(o0 * od[1] + o1) * od[2] + o2] =
            x[(idx[0] * dims[1] + idx[1]) * dims[2] + idx[2]];
      }
}

/* ------------------------------------------------------------------------
 * seeded inputs */
static inline uint64_t splitmix64_(uint64_t z) {
  z += 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}

void oracle_fill_uniform_f32(float *v, int64_t n, uint64_t seed, int64_t first,
                             float lo, float hi) {
  const float span = hi - lo;
  for (int64_t i = 0; i < n; ++i) {
    uint64_t h = splitmix64_((uint64_t)(first + i) + seed * 0x9E3779B97F4A7C15ULL);
    float u = (float)(uint32_t)(h >> 40) * (1.0f / 16777216.0f);
    float p = u * span;
    v[i] = lo + p;
  }
}

/* ------------------------------------------------------------------------
 * comparisons */
int oracle_allclose_f32(const float *got, const float *ref, int64_t n) {
  const float atol = 1e-04f, rtol = 1e-03f;
  for (int64_t i = 0; i < n; ++i)
    if (!(fabsf(got[i] - ref[i]) <= atol + rtol * fabsf(ref[i])))
      return 0;
  return 1;
}

double oracle_max_rel_err_f32(const float *got, const float *ref, int64_t n,
                              double floor_abs) {
  double worst = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    double d = fabs((double)got[i] - (double)ref[i]);
    double den = fabs((double)ref[i]);
    if (den < floor_abs)
      den = floor_abs;
    double r = (d == 0.0) ? 0.0 : d / den;
    if (r != r)
      return INFINITY;
    if (r > worst)
      worst = r;
  }
  return worst;
}

double oracle_rel_frobenius_f32(const float *got, const float *ref, int64_t n) {
  double num = 0.0, den = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    double d = (double)got[i] - (double)ref[i];
    num += d * d;
    den += (double)ref[i] * (double)ref[i];
  }
  if (den == 0.0)
    return num == 0.0 ? 0.0 : INFINITY;
  return sqrt(num / den);
}
