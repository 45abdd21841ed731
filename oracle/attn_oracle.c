/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement, in plain C, of the reference's
 * scaled-dot-product attention arithmetic.  Only tests, the smoke check and
 * the CPU-baseline leg of the benchmark may load this file; the product path
 * never does.
 *
 * The reference computes attention as a chain of generic fp32 CPU ops
 * (src/Function/FuncNNLayer.h:231-266):
 *   scores = matmul(Q, transpose(K))          src/Operation/OpLinalgCpu.h:138-150
 *   scores *= scale                           src/Operation/OpElemWiseCpu.h:395-403
 *   scores += bias (0 / -inf / additive)      src/Function/FuncNNLayer.h:241-260
 *   P = softmax(scores, -1)                   src/Operation/OpNNLayerCpu.h:16-64
 *   O = matmul(P, V)                          src/Operation/OpLinalgCpu.h:138-150
 * Each step below keeps the reference's loop and accumulation order (gemm sums
 * over the contraction index in ascending order in a float accumulator; the
 * softmax takes max from -FLT_MAX, sums expf() sequentially and multiplies by
 * a float reciprocal that is formed in double), so the forward output is
 * bit-identical to the reference's CPU fp32 path when both are compiled
 * without FMA contraction.
 *
 * The reference has no attention backward (FuncNNLayer.h:267 traps).  Its
 * gradient is defined by its differentiable primitives composed per (b,h)
 * slice: linear -> mul -> add -> softmax -> linear, whose backward rules are
 *   FuncLinear::backward   src/Function/FuncNNLayer.h:20-34
 *   FuncMul::backward      src/Function/FuncElemWise.h:113-123
 *   FuncAdd::backward      src/Function/FuncElemWise.h:77-87
 *   softmaxBackward        src/Operation/OpNNLayerCpu.h:78-109
 * oracle_sdpa_bwd restates exactly that chain.
 *
 * Grouped-query attention follows op::repeatInterleave(kv, group, 1)
 * (src/Operation/OpTransformCpu.h:399-442): query head h reads kv head
 * h / group.  Per-sequence lengths follow the reference's boolean-mask path
 * (FuncNNLayer.h:249-252): key j participates iff j < kv_len[b].
 *
 * Layout: every tensor is dense row-major [B, H, S, D], D innermost
 * (src/Tensor/TensorImpl.cpp:13-31).
 *
 * Pinned against: the three known-answer cases of
 * test/test_function.cpp:393-419, and the reference's own CPU code compiled
 * from its sources (see ref_shim.cpp and the Makefile in this directory).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <stdatomic.h>

/* bias_kind values */
#define ORACLE_BIAS_NONE 0
#define ORACLE_BIAS_CAUSAL 1 /* keep j <= i, top-left aligned for any L,S */
#define ORACLE_BIAS_ADDITIVE 2 /* float bias with broadcast strides */

typedef struct {
  int64_t B, Hq, Hkv, L, S, D;
  int32_t bias_kind;
  float scale;
  const int32_t* kv_lens;  /* [B] or NULL */
  const float* bias;       /* additive bias or NULL */
  int64_t bias_stride[4];  /* element strides over (b, h, l, s); 0 = broadcast */
} oracle_dims;

/* c[m,n] (+)= a[m,k] * b, with the reference's ikj loop and flags. */
static void gemm_ref(float* c, const float* a, const float* b, int64_t m, int64_t k, int64_t n, int transA,
                     int transB) {
  memset(c, 0, (size_t)(m * n) * sizeof(float));
  for (int64_t i = 0; i < m; i++) {
    for (int64_t p = 0; p < k; p++) {
      float aVal = transA ? a[p * m + i] : a[i * k + p];
      for (int64_t j = 0; j < n; j++) {
        float bVal = transB ? b[j * k + p] : b[p * n + j];
        c[i * n + j] += aVal * bVal;
      }
    }
  }
}

/* Scaled, biased scores of one (b, h) slice into s[L,S]. */
static void slice_scores(const oracle_dims* d, int64_t b, int64_t h, const float* q, const float* k, float* kT,
                         float* s) {
  const int64_t L = d->L, S = d->S, D = d->D;
  /* op::transpose(key, -2, -1) materialises K^T [D,S] */
  for (int64_t j = 0; j < S; j++)
    for (int64_t x = 0; x < D; x++) kT[x * S + j] = k[j * D + x];
  gemm_ref(s, q, kT, L, D, S, 0, 0);
  for (int64_t i = 0; i < L * S; i++) s[i] *= d->scale;
  if (d->bias_kind == ORACLE_BIAS_CAUSAL) {
    for (int64_t i = 0; i < L; i++)
      for (int64_t j = 0; j < S; j++) s[i * S + j] += (j <= i) ? 0.0f : -INFINITY;
  } else if (d->bias_kind == ORACLE_BIAS_ADDITIVE && d->bias) {
    const int64_t* st = d->bias_stride;
    for (int64_t i = 0; i < L; i++)
      for (int64_t j = 0; j < S; j++) s[i * S + j] += d->bias[b * st[0] + h * st[1] + i * st[2] + j * st[3]];
  }
  if (d->kv_lens) {
    int64_t len = d->kv_lens[b];
    for (int64_t i = 0; i < L; i++)
      for (int64_t j = 0; j < S; j++) s[i * S + j] += (j < len) ? 0.0f : -INFINITY;
  }
}

/* Row softmax in place; optionally returns log-sum-exp per row. */
static void slice_softmax(float* s, int64_t L, int64_t S, float* lse) {
  for (int64_t i = 0; i < L; i++) {
    float* row = s + i * S;
    float maxVal = -FLT_MAX;
    for (int64_t j = 0; j < S; j++)
      if (row[j] > maxVal) maxVal = row[j];
    float sum = 0;
    for (int64_t j = 0; j < S; j++) {
      float e = expf(row[j] - maxVal);
      row[j] = e;
      sum += e;
    }
    float invSum = (float)(1.0 / sum);
    for (int64_t j = 0; j < S; j++) row[j] *= invSum;
    if (lse) lse[i] = (float)((double)maxVal + log((double)sum));
  }
}

/* ---- slice workers: (b,h) slices are independent, so threads only change
 * wall time, never a result. ---- */

static int g_threads = 1;

void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
int oracle_num_threads(void) { return g_threads; }

typedef struct {
  const oracle_dims* d;
  const float *q, *k, *v, *dout;
  float *out, *lse, *dq, *dk, *dv;
  atomic_llong next;
  atomic_int fail;
  int is_bwd;
} job_t;

static void fwd_worker(job_t* jb) {
  const oracle_dims* d = jb->d;
  const int64_t L = d->L, S = d->S, D = d->D, g = d->Hq / d->Hkv;
  const int64_t slices = d->B * d->Hq;
  float* s = (float*)malloc((size_t)(L * S) * sizeof(float));
  float* kT = (float*)malloc((size_t)(D * S) * sizeof(float));
  if (!s || !kT) {
    atomic_store(&jb->fail, 1);
  } else {
    for (;;) {
      int64_t u = atomic_fetch_add(&jb->next, 1);
      if (u >= slices) break;
      int64_t b = u / d->Hq, h = u % d->Hq, hk = h / g;
      const float* qs = jb->q + (b * d->Hq + h) * L * D;
      const float* ks = jb->k + (b * d->Hkv + hk) * S * D;
      const float* vs = jb->v + (b * d->Hkv + hk) * S * D;
      slice_scores(d, b, h, qs, ks, kT, s);
      slice_softmax(s, L, S, jb->lse ? jb->lse + u * L : NULL);
      gemm_ref(jb->out + u * L * D, s, vs, L, S, D, 0, 0);
    }
  }
  free(s);
  free(kT);
}

static void bwd_worker(job_t* jb) {
  const oracle_dims* d = jb->d;
  const int64_t L = d->L, S = d->S, D = d->D, g = d->Hq / d->Hkv;
  const int64_t groups = d->B * d->Hkv;
  float *dq = jb->dq, *dk = jb->dk, *dv = jb->dv;
  float* p = (float*)malloc((size_t)(L * S) * sizeof(float));
  float* dp = (float*)malloc((size_t)(L * S) * sizeof(float));
  float* kT = (float*)malloc((size_t)(D * S) * sizeof(float));
  float* vT = (float*)malloc((size_t)(D * S) * sizeof(float));
  float* tmp = (float*)malloc((size_t)(S * D) * sizeof(float));
  if (!p || !dp || !kT || !vT || !tmp) {
    atomic_store(&jb->fail, 1);
  } else {
    for (;;) {
      int64_t u = atomic_fetch_add(&jb->next, 1);
      if (u >= groups) break;
      int64_t b = u / d->Hkv, hk = u % d->Hkv;
      const float* ks = jb->k + u * S * D;
      const float* vs = jb->v + u * S * D;
      if (dk) memset(dk + u * S * D, 0, (size_t)(S * D) * sizeof(float));
      if (dv) memset(dv + u * S * D, 0, (size_t)(S * D) * sizeof(float));
      for (int64_t x = 0; x < D; x++)
        for (int64_t j = 0; j < S; j++) vT[x * S + j] = vs[j * D + x];
      for (int64_t r = 0; r < g; r++) {
        int64_t h = hk * g + r;
        const float* qs = jb->q + (b * d->Hq + h) * L * D;
        const float* dos = jb->dout + (b * d->Hq + h) * L * D;
        slice_scores(d, b, h, qs, ks, kT, p);
        slice_softmax(p, L, S, NULL);
        /* o = linear(p, vT): dIn = g . W  ->  dP[L,S] = dO[L,D] . vT[D,S] */
        gemm_ref(dp, dos, vT, L, D, S, 0, 0);
        /* dW = g^T . In  ->  dvT[D,S] = dO^T . P ; handed back transposed */
        if (dv) {
          float* dvT = kT; /* kT is free again after slice_scores */
          gemm_ref(dvT, dos, p, D, L, S, 1, 0);
          for (int64_t j = 0; j < S; j++)
            for (int64_t x = 0; x < D; x++) dv[u * S * D + j * D + x] += dvT[x * S + j];
        }
        /* softmax backward: dS = P * (dP - sum_j P_j dP_j) */
        for (int64_t i = 0; i < L; i++) {
          float sum = 0;
          for (int64_t j = 0; j < S; j++) sum += p[i * S + j] * dp[i * S + j];
          for (int64_t j = 0; j < S; j++) dp[i * S + j] = p[i * S + j] * (dp[i * S + j] - sum);
        }
        /* add: pass-through.  mul by the scale scalar. */
        for (int64_t i = 0; i < L * S; i++) dp[i] *= d->scale;
        /* s = linear(q, k): dq = dS . K ; dk = dS^T . Q */
        if (dq) gemm_ref(dq + (b * d->Hq + h) * L * D, dp, ks, L, S, D, 0, 0);
        if (dk) {
          gemm_ref(tmp, dp, qs, S, L, D, 1, 0);
          for (int64_t i = 0; i < S * D; i++) dk[u * S * D + i] += tmp[i];
        }
      }
    }
  }
  free(p);
  free(dp);
  free(kT);
  free(vT);
  free(tmp);
}

static void* worker_entry(void* arg) {
  job_t* jb = (job_t*)arg;
  if (jb->is_bwd)
    bwd_worker(jb);
  else
    fwd_worker(jb);
  return NULL;
}

static int run_job(job_t* jb, int64_t units) {
  int n = g_threads;
  if ((int64_t)n > units) n = (int)units;
  if (n <= 1) {
    worker_entry(jb);
  } else {
    pthread_t th[256];
    int started = 0;
    for (int i = 0; i < n - 1; i++)
      if (pthread_create(&th[started], NULL, worker_entry, jb) == 0) started++;
    worker_entry(jb);
    for (int i = 0; i < started; i++) pthread_join(th[i], NULL);
  }
  return atomic_load(&jb->fail) ? -1 : 0;
}

/*
 * Forward.  q [B,Hq,L,D]; k,v [B,Hkv,S,D]; out [B,Hq,L,D]; lse [B,Hq,L] or
 * NULL.  Returns 0, or -1 on bad arguments / allocation failure.
 */
int oracle_sdpa_fwd(const oracle_dims* d, const float* q, const float* k, const float* v, float* out, float* lse) {
  if (!d || !q || !k || !v || !out) return -1;
  if (d->Hkv <= 0 || d->Hq % d->Hkv) return -1;
  job_t jb;
  memset(&jb, 0, sizeof(jb));
  jb.d = d, jb.q = q, jb.k = k, jb.v = v, jb.out = out, jb.lse = lse;
  atomic_init(&jb.next, 0);
  atomic_init(&jb.fail, 0);
  return run_job(&jb, d->B * d->Hq);
}

/*
 * Backward through the composed chain.  dout [B,Hq,L,D]; dq [B,Hq,L,D];
 * dk, dv [B,Hkv,S,D].  With Hq > Hkv the gradients of the query heads that
 * share a kv head are summed in ascending head order (the gradient of
 * repeatInterleave).  Any of dq/dk/dv may be NULL.
 */
int oracle_sdpa_bwd(const oracle_dims* d, const float* q, const float* k, const float* v, const float* dout,
                    float* dq, float* dk, float* dv) {
  if (!d || !q || !k || !v || !dout) return -1;
  if (d->Hkv <= 0 || d->Hq % d->Hkv) return -1;
  job_t jb;
  memset(&jb, 0, sizeof(jb));
  jb.d = d, jb.q = q, jb.k = k, jb.v = v, jb.dout = dout, jb.dq = dq, jb.dk = dk, jb.dv = dv;
  jb.is_bwd = 1;
  atomic_init(&jb.next, 0);
  atomic_init(&jb.fail, 0);
  return run_job(&jb, d->B * d->Hkv);
}
