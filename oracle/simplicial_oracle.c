/* CPU oracle for 2-simplicial attention, loop form.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's `simplicial/reference.py:8-76`
 * (`two_simplicial_attention_reference`): for every query row, a double loop over the K1 window
 * and the K2 window, weight = exp(scale * sum_d q*k1*k2), output = sum(weight * v1*v2) /
 * (sum(weight) + 1e-8).  The backward is the analytic derivative of that expression, i.e. what
 * torch autograd produces when run through the reference function.
 *
 * It is the checker and the timed CPU baseline; the shipped library never links or calls it.
 * Parity status: pinned against outputs of the unmodified reference (tests/golden).
 *
 * Differences from the reference text, all deliberate:
 *  - windows are (i-w, i]  (the operator's convention; the reference loop called with w-1,
 *    `reference.py:41-45`);
 *  - K/V may have fewer heads than Q (grouped heads): query head h reads KV head h / (H / Hkv),
 *    equal to the reference applied to repeat_interleave-expanded K/V;
 *  - K1/V1 (K2/V2) may carry halo1 (halo2) leading rows that precede query row 0;
 *  - accumulation is in double, the exponent is taken relative to the row maximum (the reference
 *    takes exp(score) directly, `reference.py:65`, and overflows for scores above ~88).
 *
 * Tensors are contiguous fp32: q, o, dO, dq [B,N,H,D]; k1, v1, dk1, dv1 [B,N+halo1,Hkv,D];
 * k2, v2, dk2, dv2 [B,N+halo2,Hkv,D]; lse [B,H,N].
 * Build: gcc -O3 -march=x86-64-v3 -fopenmp -shared -fPIC (see oracle/Makefile).
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
    int B, N, H, Hkv, D;
    int w1, w2;
    int halo1, halo2;
    float scale, k2_bias, v2_bias;
} sa_oracle_dims;

static inline int imax(int a, int b) { return a > b ? a : b; }

int sa_oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the number of OpenMP threads the loops use (a launcher may have exported OMP_NUM_THREADS=1). */
void sa_oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* One query row: fills o_row[D] and returns the natural-log softmax denominator.
 * `p_out` (may be NULL) receives the normalised weights, laid out [j - j_lo][k - k_lo]. */
static double row_forward(const sa_oracle_dims *p, const float *qrow, const float *k1h, const float *k2h,
                          const float *v1h, const float *v2h, long kv_stride, int i, double *o_row,
                          double *p_out, double *scratch /* D + D + w1*w2 */) {
    const int D = p->D;
    const int j_hi = i + p->halo1, j_lo = imax(0, j_hi - p->w1 + 1);
    const int k_hi = i + p->halo2, k_lo = imax(0, k_hi - p->w2 + 1);
    const int nj = j_hi - j_lo + 1, nk = k_hi - k_lo + 1;
    double *a = scratch, *t = scratch + D, *s = scratch + 2 * D;
    double m = -INFINITY;
    for (int k = k_lo; k <= k_hi; ++k) {
        const float *k2r = k2h + (long)k * kv_stride;
        for (int d = 0; d < D; ++d) a[d] = (double)qrow[d] * ((double)k2r[d] + p->k2_bias) * p->scale;
        for (int j = j_lo; j <= j_hi; ++j) {
            const float *k1r = k1h + (long)j * kv_stride;
            double acc = 0.0;
            for (int d = 0; d < D; ++d) acc += a[d] * (double)k1r[d];   /* reference.py:63 */
            s[(long)(j - j_lo) * nk + (k - k_lo)] = acc;
            if (acc > m) m = acc;
        }
    }
    double total = 0.0;
    for (long e = 0; e < (long)nj * nk; ++e) { s[e] = exp(s[e] - m); total += s[e]; }  /* reference.py:64 */
    /* reference.py:74 divides by (total_weight + 1e-8) with un-shifted weights; shifted by m the
       epsilon becomes 1e-8 * exp(-m). */
    const double denom = total + 1e-8 * exp(-m);
    for (int d = 0; d < D; ++d) o_row[d] = 0.0;
    for (int k = k_lo; k <= k_hi; ++k) {
        const float *v2r = v2h + (long)k * kv_stride;
        for (int d = 0; d < D; ++d) t[d] = 0.0;
        for (int j = j_lo; j <= j_hi; ++j) {
            const float *v1r = v1h + (long)j * kv_stride;
            const double w = s[(long)(j - j_lo) * nk + (k - k_lo)];
            for (int d = 0; d < D; ++d) t[d] += w * (double)v1r[d];
        }
        for (int d = 0; d < D; ++d) o_row[d] += t[d] * ((double)v2r[d] + p->v2_bias);   /* reference.py:67-70 */
    }
    for (int d = 0; d < D; ++d) o_row[d] /= denom;
    if (p_out) for (long e = 0; e < (long)nj * nk; ++e) p_out[e] = s[e] / denom;
    return m + log(denom);
}

/* Forward for query rows [row_begin, row_end) of every (b, h).  o: [B,N,H,D], lse: [B,H,N];
 * rows outside the range are left untouched. */
int sa_oracle_forward(const sa_oracle_dims *p, const float *q, const float *k1, const float *k2,
                      const float *v1, const float *v2, float *o, float *lse, int row_begin, int row_end) {
    const int B = p->B, N = p->N, H = p->H, Hkv = p->Hkv, D = p->D;
    if (H % Hkv != 0 || row_begin < 0 || row_end > N) return 1;
    const int g = H / Hkv;
    const long kv_stride = (long)Hkv * D;
    const long n1 = N + p->halo1, n2 = N + p->halo2;
    const long rows = row_end - row_begin;
    const long tasks = (long)B * H * rows;
#pragma omp parallel
    {
        double *scratch = (double *)malloc(sizeof(double) * (3 * (size_t)D + (size_t)p->w1 * p->w2));
        double *orow = scratch + 2 * D + (size_t)p->w1 * p->w2;
#pragma omp for schedule(dynamic, 16)
        for (long task = 0; task < tasks; ++task) {
            const int i = row_begin + (int)(task % rows);
            const int h = (int)((task / rows) % H);
            const int b = (int)(task / rows / H);
            const int hk = h / g;
            const float *qrow = q + (((long)b * N + i) * H + h) * D;
            const double l = row_forward(p, qrow, k1 + (long)b * n1 * kv_stride + (long)hk * D,
                                         k2 + (long)b * n2 * kv_stride + (long)hk * D,
                                         v1 + (long)b * n1 * kv_stride + (long)hk * D,
                                         v2 + (long)b * n2 * kv_stride + (long)hk * D, kv_stride, i, orow,
                                         NULL, scratch);
            float *orow_out = o + (((long)b * N + i) * H + h) * D;
            for (int d = 0; d < D; ++d) orow_out[d] = (float)orow[d];
            if (lse) lse[((long)b * H + h) * N + i] = (float)l;
        }
        free(scratch);
    }
    return 0;
}

/* Backward of sum(O * dO) for query rows [row_begin, row_end): ADDS the contributions of those
 * rows into dq, dk1, dk2, dv1, dv2 (callers zero them first).  With the full row range this is
 * the complete gradient; with a sub-range it is that range's share, which is what a sequence
 * shard computes.  Derivation from reference.py:63-74 with P = weight / total:
 *   Delta_i = dO_i . O_i;  dP_ijk = dO_i . (v1_j * v2_k);  dS = P * (dP - Delta)
 *   dq_i  += scale * dS * k1_j * k2_k      dk1_j += scale * dS * q_i * k2_k
 *   dk2_k += scale * dS * q_i * k1_j       dv1_j += P * dO_i * v2_k      dv2_k += P * dO_i * v1_j
 */
int sa_oracle_backward(const sa_oracle_dims *p, const float *q, const float *k1, const float *k2,
                       const float *v1, const float *v2, const float *dO, float *dq, float *dk1, float *dk2,
                       float *dv1, float *dv2, int row_begin, int row_end) {
    const int B = p->B, N = p->N, H = p->H, Hkv = p->Hkv, D = p->D;
    if (H % Hkv != 0 || row_begin < 0 || row_end > N) return 1;
    const int g = H / Hkv;
    const long kv_stride = (long)Hkv * D;
    const long n1 = N + p->halo1, n2 = N + p->halo2;
    const int CH = 32;                                /* query rows per task */
    const long rows = row_end - row_begin;
    const long chunks = (rows + CH - 1) / CH;
    const long tasks = (long)B * H * chunks;
#pragma omp parallel
    {
        const size_t w12 = (size_t)p->w1 * p->w2;
        const size_t r1 = (size_t)CH + p->w1, r2 = (size_t)CH + p->w2;
        double *scratch = (double *)malloc(sizeof(double) * (3 * (size_t)D + w12));
        double *orow = (double *)malloc(sizeof(double) * D);
        double *pw = (double *)malloc(sizeof(double) * w12);
        double *l_dk1 = (double *)malloc(sizeof(double) * r1 * D * 2);
        double *l_dv1 = l_dk1 + r1 * D;
        double *l_dk2 = (double *)malloc(sizeof(double) * r2 * D * 2);
        double *l_dv2 = l_dk2 + r2 * D;
        double *dqrow = (double *)malloc(sizeof(double) * D * 3);
        double *c = dqrow + D, *u = dqrow + 2 * D;
#pragma omp for schedule(dynamic, 1)
        for (long task = 0; task < tasks; ++task) {
            const int ch = (int)(task % chunks);
            const int h = (int)((task / chunks) % H);
            const int b = (int)(task / chunks / H);
            const int hk = h / g;
            const int i0 = row_begin + ch * CH, i1 = (i0 + CH < row_end) ? i0 + CH : row_end;
            const float *k1h = k1 + (long)b * n1 * kv_stride + (long)hk * D;
            const float *v1h = v1 + (long)b * n1 * kv_stride + (long)hk * D;
            const float *k2h = k2 + (long)b * n2 * kv_stride + (long)hk * D;
            const float *v2h = v2 + (long)b * n2 * kv_stride + (long)hk * D;
            /* local accumulators cover buffer rows [base1, base1 + r1) of K1/V1 and likewise for K2/V2 */
            const int base1 = imax(0, i0 + p->halo1 - p->w1 + 1);
            const int base2 = imax(0, i0 + p->halo2 - p->w2 + 1);
            memset(l_dk1, 0, sizeof(double) * r1 * D * 2);
            memset(l_dk2, 0, sizeof(double) * r2 * D * 2);
            for (int i = i0; i < i1; ++i) {
                const float *qrow = q + (((long)b * N + i) * H + h) * D;
                const float *dorow = dO + (((long)b * N + i) * H + h) * D;
                row_forward(p, qrow, k1h, k2h, v1h, v2h, kv_stride, i, orow, pw, scratch);
                double delta = 0.0;
                for (int d = 0; d < D; ++d) delta += (double)dorow[d] * orow[d];
                const int j_hi = i + p->halo1, j_lo = imax(0, j_hi - p->w1 + 1);
                const int k_hi = i + p->halo2, k_lo = imax(0, k_hi - p->w2 + 1);
                const int nk = k_hi - k_lo + 1;
                for (int d = 0; d < D; ++d) dqrow[d] = 0.0;
                for (int k = k_lo; k <= k_hi; ++k) {
                    const float *k2r = k2h + (long)k * kv_stride, *v2r = v2h + (long)k * kv_stride;
                    double *gk2 = l_dk2 + (size_t)(k - base2) * D, *gv2 = l_dv2 + (size_t)(k - base2) * D;
                    /* c = dO * (v2 + bias), u = q * (k2 + bias) */
                    for (int d = 0; d < D; ++d) {
                        c[d] = (double)dorow[d] * ((double)v2r[d] + p->v2_bias);
                        u[d] = (double)qrow[d] * ((double)k2r[d] + p->k2_bias);
                    }
                    for (int j = j_lo; j <= j_hi; ++j) {
                        const float *k1r = k1h + (long)j * kv_stride, *v1r = v1h + (long)j * kv_stride;
                        double *gk1 = l_dk1 + (size_t)(j - base1) * D, *gv1 = l_dv1 + (size_t)(j - base1) * D;
                        const double P = pw[(long)(j - j_lo) * nk + (k - k_lo)];
                        double dP = 0.0;
                        for (int d = 0; d < D; ++d) dP += c[d] * (double)v1r[d];
                        const double dS = P * (dP - delta) * p->scale;
                        for (int d = 0; d < D; ++d) {
                            const double k1d = k1r[d], v1d = v1r[d];
                            dqrow[d] += dS * k1d * ((double)k2r[d] + p->k2_bias);
                            gk1[d] += dS * u[d];
                            gk2[d] += dS * (double)qrow[d] * k1d;
                            gv1[d] += P * c[d];
                            gv2[d] += P * (double)dorow[d] * v1d;
                        }
                    }
                }
                float *dqo = dq + (((long)b * N + i) * H + h) * D;
                for (int d = 0; d < D; ++d) dqo[d] += (float)dqrow[d];
            }
#pragma omp critical
            {
                for (size_t r = 0; r < r1 && (long)(base1 + r) < n1; ++r) {
                    float *o1 = dk1 + (((long)b * n1 + base1 + (long)r) * Hkv + hk) * D;
                    float *o2 = dv1 + (((long)b * n1 + base1 + (long)r) * Hkv + hk) * D;
                    for (int d = 0; d < D; ++d) { o1[d] += (float)l_dk1[r * D + d]; o2[d] += (float)l_dv1[r * D + d]; }
                }
                for (size_t r = 0; r < r2 && (long)(base2 + r) < n2; ++r) {
                    float *o1 = dk2 + (((long)b * n2 + base2 + (long)r) * Hkv + hk) * D;
                    float *o2 = dv2 + (((long)b * n2 + base2 + (long)r) * Hkv + hk) * D;
                    for (int d = 0; d < D; ++d) { o1[d] += (float)l_dk2[r * D + d]; o2[d] += (float)l_dv2[r * D + d]; }
                }
            }
        }
        free(scratch); free(orow); free(pw); free(l_dk1); free(l_dk2); free(dqrow);
    }
    return 0;
}
