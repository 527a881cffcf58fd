/*
 * CPU oracle for the native Field recurrence. TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C, double-precision, step-by-step restatement of the
 * reference's Field read:
 *   forward   reference_field_read      (field_only_v4_chunked_triton_wiki100.py:392-416)
 *             gate math                  (same file :400-406 and :493-501)
 *             displaced readout          (same file :408-416 and :605-617)
 *   backward  dual recurrence and gate   (same file :794-909)
 *             derivatives
 * It is the checker for the CUDA kernels. Nothing in the shipped library
 * calls it; only the test-suite, the smoke check and the CPU-baseline leg of
 * the benchmark load it.
 *
 * Parity status: pinned. The fixtures under tests/golden/ were produced by
 * importing the reference's own Python module and running
 * reference_field_read plus autograd; tests/test_oracle_golden.py holds this
 * oracle to those fixtures.
 *
 * Layouts (identical to the reference's tensors, channel fastest):
 *   raw        [B, L, 3C]  planes z_r | z_i | z_v
 *   read       [B, L, 4C]  planes Re s | Im s | Re d | Im d
 *   grad_read  [B, L, 4C]
 *   grad_raw   [B, L, 3C]
 *   state      [B, 2C]     planes Re s | Im s
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#define FIELD_VAC_MAX 0.90 /* VAC_MAX, field_only_v4_chunked_triton_wiki100.py:68 */
#define CBLK 16            /* channels walked together so a cache line is used whole */

static double sigmoid_d(double x) { return 1.0 / (1.0 + exp(-x)); }

/*
 * Forward. state_in may be NULL (the reference always starts from zero,
 * field_only_v4_chunked_triton_wiki100.py:535-536). state_out may be NULL.
 * Follows :400-416: inj = tanh(z_r) + i tanh(z_i); v = 0.9 sigmoid(z_v);
 * a = (1 - v) lambda; b = gamma v inj; s_t = a s_{t-1} + b;
 * d_t = v lambda s_{t-1}.
 */
int field_oracle_forward(const float *raw, const float *tr, const float *ti,
                         const float *gamma, const double *state_in,
                         double *read, double *state_out, int B, int L, int C)
{
    if (B < 0 || L < 0 || C <= 0) return 1;
    const int nblk = (C + CBLK - 1) / CBLK;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b) {
        for (int blk = 0; blk < nblk; ++blk) {
            const int c0 = blk * CBLK;
            const int cn = (C - c0 < CBLK) ? (C - c0) : CBLK;
            double sr[CBLK], si[CBLK];
            for (int j = 0; j < cn; ++j) {
                sr[j] = state_in ? state_in[(size_t)b * 2 * C + c0 + j] : 0.0;
                si[j] = state_in ? state_in[(size_t)b * 2 * C + C + c0 + j] : 0.0;
            }
            for (int t = 0; t < L; ++t) {
                const float *z = raw + ((size_t)b * L + t) * 3 * C;
                double *o = read + ((size_t)b * L + t) * 4 * C;
                for (int j = 0; j < cn; ++j) {
                    const int c = c0 + j;
                    const double lr = tr[c], li = ti[c], gm = gamma[c];
                    const double ir = tanh((double)z[c]);
                    const double ii = tanh((double)z[C + c]);
                    const double v = FIELD_VAC_MAX * sigmoid_d((double)z[2 * C + c]);
                    const double keep = 1.0 - v;
                    const double mr = lr * sr[j] - li * si[j]; /* lambda * s_{t-1} */
                    const double mi = lr * si[j] + li * sr[j];
                    const double nr = keep * mr + gm * v * ir;
                    const double ni = keep * mi + gm * v * ii;
                    o[c] = nr;
                    o[C + c] = ni;
                    o[2 * C + c] = v * mr;
                    o[3 * C + c] = v * mi;
                    sr[j] = nr;
                    si[j] = ni;
                }
            }
            if (state_out) {
                for (int j = 0; j < cn; ++j) {
                    state_out[(size_t)b * 2 * C + c0 + j] = sr[j];
                    state_out[(size_t)b * 2 * C + C + c0 + j] = si[j];
                }
            }
        }
    }
    return 0;
}

/*
 * Backward. Recomputes the forward states, then walks time in reverse with the
 * dual recurrence of field_only_v4_chunked_triton_wiki100.py:794-909:
 *   G_t      = u_t + carry_t                       (:818-829, carry_{L-1} = grad_state_out or 0)
 *   da       = G_t conj(s_{t-1}),  db = G_t        (:858-861)
 *   carry_{t-1} = conj(a_t) G_t + v_t conj(lambda) gd_t            (:863-864, :874-879)
 *   dv       = -(lr da_r + li da_i) + gamma (inj . G) + gd . (lambda s_{t-1})   (:866, :880-883)
 *   dlambda += keep da + v gd conj(s_{t-1});  dgamma += v (inj . G)           (:867-872, :884-886)
 *   dz_r = gamma v G_r (1 - inj_r^2), dz_i likewise, dz_v = dv 0.9 sig (1 - sig)  (:888-890)
 * grad_tr / grad_ti / grad_gamma are sums over batch and time (:1098-1105).
 * grad_state_out and grad_state_in may be NULL.
 */
int field_oracle_backward(const float *raw, const float *tr, const float *ti,
                          const float *gamma, const double *state_in,
                          const float *grad_read, const double *grad_state_out,
                          double *grad_raw, double *grad_tr, double *grad_ti,
                          double *grad_gamma, double *grad_state_in,
                          int B, int L, int C)
{
    if (B < 0 || L < 0 || C <= 0) return 1;
    const int nblk = (C + CBLK - 1) / CBLK;
    /* per-batch partials so the reduction order does not depend on threads */
    double *part = (double *)calloc((size_t)(B > 0 ? B : 1) * 3 * C, sizeof(double));
    if (!part) return 2;
    int fail = 0;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b) {
        for (int blk = 0; blk < nblk; ++blk) {
            const int c0 = blk * CBLK;
            const int cn = (C - c0 < CBLK) ? (C - c0) : CBLK;
            /* prev[t][j] = s_{t-1} for this channel block */
            double *prev = (double *)malloc((size_t)(L > 0 ? L : 1) * 2 * CBLK * sizeof(double));
            if (!prev) {
#pragma omp atomic write
                fail = 1;
                continue;
            }
            double sr[CBLK], si[CBLK];
            for (int j = 0; j < cn; ++j) {
                sr[j] = state_in ? state_in[(size_t)b * 2 * C + c0 + j] : 0.0;
                si[j] = state_in ? state_in[(size_t)b * 2 * C + C + c0 + j] : 0.0;
            }
            for (int t = 0; t < L; ++t) {
                const float *z = raw + ((size_t)b * L + t) * 3 * C;
                for (int j = 0; j < cn; ++j) {
                    const int c = c0 + j;
                    prev[((size_t)t * 2) * CBLK + j] = sr[j];
                    prev[((size_t)t * 2 + 1) * CBLK + j] = si[j];
                    const double lr = tr[c], li = ti[c], gm = gamma[c];
                    const double ir = tanh((double)z[c]);
                    const double ii = tanh((double)z[C + c]);
                    const double v = FIELD_VAC_MAX * sigmoid_d((double)z[2 * C + c]);
                    const double keep = 1.0 - v;
                    const double mr = lr * sr[j] - li * si[j];
                    const double mi = lr * si[j] + li * sr[j];
                    sr[j] = keep * mr + gm * v * ir;
                    si[j] = keep * mi + gm * v * ii;
                }
            }
            double cr[CBLK], ci[CBLK], dtr[CBLK], dti[CBLK], dgm[CBLK];
            for (int j = 0; j < cn; ++j) {
                cr[j] = grad_state_out ? grad_state_out[(size_t)b * 2 * C + c0 + j] : 0.0;
                ci[j] = grad_state_out ? grad_state_out[(size_t)b * 2 * C + C + c0 + j] : 0.0;
                dtr[j] = dti[j] = dgm[j] = 0.0;
            }
            for (int t = L - 1; t >= 0; --t) {
                const float *z = raw + ((size_t)b * L + t) * 3 * C;
                const float *g = grad_read + ((size_t)b * L + t) * 4 * C;
                double *o = grad_raw + ((size_t)b * L + t) * 3 * C;
                for (int j = 0; j < cn; ++j) {
                    const int c = c0 + j;
                    const double lr = tr[c], li = ti[c], gm = gamma[c];
                    const double ir = tanh((double)z[c]);
                    const double ii = tanh((double)z[C + c]);
                    const double sg = sigmoid_d((double)z[2 * C + c]);
                    const double v = FIELD_VAC_MAX * sg;
                    const double keep = 1.0 - v;
                    const double pr = prev[((size_t)t * 2) * CBLK + j];
                    const double pi = prev[((size_t)t * 2 + 1) * CBLK + j];
                    const double Gr = (double)g[c] + cr[j];
                    const double Gi = (double)g[C + c] + ci[j];
                    const double gdr = g[2 * C + c], gdi = g[3 * C + c];
                    const double ar = keep * lr, ai = keep * li;
                    const double mr = lr * pr - li * pi;
                    const double mi = lr * pi + li * pr;
                    const double dar = Gr * pr + Gi * pi;
                    const double dai = -Gr * pi + Gi * pr;
                    const double common_b = ir * Gr + ii * Gi;
                    const double dv = -lr * dar - li * dai + gm * common_b
                                      + gdr * mr + gdi * mi;
                    dtr[j] += keep * dar + v * (gdr * pr + gdi * pi);
                    dti[j] += keep * dai + v * (-gdr * pi + gdi * pr);
                    dgm[j] += v * common_b;
                    o[c] = gm * v * Gr * (1.0 - ir * ir);
                    o[C + c] = gm * v * Gi * (1.0 - ii * ii);
                    o[2 * C + c] = dv * FIELD_VAC_MAX * sg * (1.0 - sg);
                    cr[j] = ar * Gr + ai * Gi + v * (lr * gdr + li * gdi);
                    ci[j] = -ai * Gr + ar * Gi + v * (-li * gdr + lr * gdi);
                }
            }
            for (int j = 0; j < cn; ++j) {
                part[((size_t)b * 3 + 0) * C + c0 + j] = dtr[j];
                part[((size_t)b * 3 + 1) * C + c0 + j] = dti[j];
                part[((size_t)b * 3 + 2) * C + c0 + j] = dgm[j];
                if (grad_state_in) {
                    grad_state_in[(size_t)b * 2 * C + c0 + j] = cr[j];
                    grad_state_in[(size_t)b * 2 * C + C + c0 + j] = ci[j];
                }
            }
            free(prev);
        }
    }
    for (int c = 0; c < C; ++c) {
        double a = 0.0, bb = 0.0, g = 0.0;
        for (int b = 0; b < B; ++b) {
            a += part[((size_t)b * 3 + 0) * C + c];
            bb += part[((size_t)b * 3 + 1) * C + c];
            g += part[((size_t)b * 3 + 2) * C + c];
        }
        grad_tr[c] = a;
        grad_ti[c] = bb;
        grad_gamma[c] = g;
    }
    free(part);
    return fail ? 2 : 0;
}

/*
 * Affine summary of a whole span per (batch, channel): s_out = A s_in + Bv,
 * composed step by step as in field_only_v4_chunked_triton_wiki100.py:503-509.
 * summary is [B, 4, C] with planes Re A | Im A | Re Bv | Im Bv. Used to check
 * the sequence-sharded forward, where spans exchange exactly this pair.
 */
int field_oracle_span_summary(const float *raw, const float *tr, const float *ti,
                              const float *gamma, double *summary,
                              int B, int L, int C)
{
    if (B < 0 || L < 0 || C <= 0) return 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; ++b) {
        for (int c = 0; c < C; ++c) {
            double Ar = 1.0, Ai = 0.0, Br = 0.0, Bi = 0.0;
            const double lr = tr[c], li = ti[c], gm = gamma[c];
            for (int t = 0; t < L; ++t) {
                const float *z = raw + ((size_t)b * L + t) * 3 * C;
                const double ir = tanh((double)z[c]);
                const double ii = tanh((double)z[C + c]);
                const double v = FIELD_VAC_MAX * sigmoid_d((double)z[2 * C + c]);
                const double ar = (1.0 - v) * lr, ai = (1.0 - v) * li;
                const double nBr = ar * Br - ai * Bi + gm * v * ir;
                const double nBi = ar * Bi + ai * Br + gm * v * ii;
                const double nAr = ar * Ar - ai * Ai;
                const double nAi = ar * Ai + ai * Ar;
                Ar = nAr; Ai = nAi; Br = nBr; Bi = nBi;
            }
            double *s = summary + (size_t)b * 4 * C;
            s[c] = Ar; s[C + c] = Ai; s[2 * C + c] = Br; s[3 * C + c] = Bi;
        }
    }
    return 0;
}
