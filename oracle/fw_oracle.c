/*
 * CPU oracle for the fast-weight recurrences (decay rule "LFW" and delta rule "DFW").
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It restates, step by step and in float64,
 * the algorithm of the reference's TorchScript implementation so that the CUDA kernels can
 * be checked against it.  Only tests, the smoke check and the benchmark's CPU-baseline leg
 * may call it; the library never does.
 *
 * Reference statements followed here (paths inside the reference project):
 *   decay rule forward ............ t2fw/torch.py:21-28
 *   decay rule backward ........... autograd of the above; the same per-step algebra is
 *                                   spelled out in t2fw/csrc/lfw_kernel.cu:85-100 (state
 *                                   gradient scan) and t2fw/csrc/lfw.cpp:84-93 (the six
 *                                   gradients as contractions of S_t, R_t and R_t*S_{t-1})
 *   delta rule forward ............ t2fw/torch.py:44-52
 *   delta rule backward ........... t2fw/torch.py:84-143 (t2dfw_torch_bw)
 *
 * Parity pinned: the functions below are compared in tests against golden vectors produced
 * by importing the reference's own t2fw/torch.py (tests/golden/make_golden.py).
 *
 * Layout: all arrays are dense row-major float64.
 *   x, f, out, dx, df ......... [B, T, D]
 *   q, k, fk, dq, dk, dfk ..... [B, T, K]
 *   s0, s_final, ds0 .......... [B, D, K]
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC (see oracle/build_oracle.py).
 */
#include <stdlib.h>
#include <string.h>
#include <stdint.h>

#define ORACLE_SEG 128 /* steps whose states are kept at once in the backward passes */

/* ------------------------------------------------------------------------------------ */
/* decay rule:  S_t = (f_t fk_t^T) .* S_{t-1} + x_t k_t^T ;  o_t = S_t q_t                */
/* ------------------------------------------------------------------------------------ */

static void lfw_step(double *S, const double *x, const double *f, const double *k,
                     const double *fk, int D, int K)
{
    for (int d = 0; d < D; ++d) {
        double *row = S + (size_t)d * K;
        for (int c = 0; c < K; ++c)
            row[c] = row[c] * (f[d] * fk[c]) + x[d] * k[c];
    }
}

void t2fw_oracle_lfw_forward(const double *x, const double *f, const double *q,
                             const double *k, const double *fk, const double *s0,
                             int64_t B, int64_t T, int64_t D, int64_t K,
                             double *out, double *s_final)
{
#pragma omp parallel for schedule(dynamic)
    for (int64_t b = 0; b < B; ++b) {
        double *S = (double *)malloc(sizeof(double) * D * K);
        memcpy(S, s0 + b * D * K, sizeof(double) * D * K);
        for (int64_t t = 0; t < T; ++t) {
            const size_t od = (size_t)(b * T + t) * D, ok = (size_t)(b * T + t) * K;
            lfw_step(S, x + od, f + od, k + ok, fk + ok, (int)D, (int)K);
            for (int64_t d = 0; d < D; ++d) {
                double acc = 0.0;
                for (int64_t c = 0; c < K; ++c) acc += S[d * K + c] * q[ok + c];
                out[od + d] = acc;
            }
        }
        memcpy(s_final + b * D * K, S, sizeof(double) * D * K);
        free(S);
    }
}

/*
 * Backward of the decay rule for upstream gradients g_out [B,T,D] (w.r.t. outputs) and
 * g_state [B,D,K] (w.r.t. the final state).  With R_t the gradient w.r.t. S_t:
 *   R_t  = g_out_t q_t^T + (f_{t+1} fk_{t+1}^T) .* R_{t+1},   R_T += g_state
 *   dq_t = S_t^T g_out_t      dx_t = R_t k_t        dk_t = R_t^T x_t
 *   W_t  = R_t .* S_{t-1}     df_t = W_t fk_t       dfk_t = W_t^T f_t
 *   ds0  = (f_1 fk_1^T) .* R_1
 * States are recomputed segment by segment from stored segment-start states.
 */
void t2fw_oracle_lfw_backward(const double *g_out, const double *g_state,
                              const double *x, const double *f, const double *q,
                              const double *k, const double *fk, const double *s0,
                              int64_t B, int64_t T, int64_t D, int64_t K,
                              double *dx, double *df, double *dq, double *dk,
                              double *dfk, double *ds0)
{
    const int64_t DK = D * K;
    const int64_t nseg = (T + ORACLE_SEG - 1) / ORACLE_SEG;
#pragma omp parallel for schedule(dynamic)
    for (int64_t b = 0; b < B; ++b) {
        double *seg0 = (double *)malloc(sizeof(double) * DK * (nseg > 0 ? nseg : 1));
        double *hist = (double *)malloc(sizeof(double) * DK * (ORACLE_SEG + 1));
        double *R = (double *)malloc(sizeof(double) * DK);
        double *S = (double *)malloc(sizeof(double) * DK);
        /* forward sweep: remember the state at the start of every segment */
        memcpy(S, s0 + b * DK, sizeof(double) * DK);
        for (int64_t t = 0; t < T; ++t) {
            if (t % ORACLE_SEG == 0) memcpy(seg0 + (t / ORACLE_SEG) * DK, S, sizeof(double) * DK);
            const size_t od = (size_t)(b * T + t) * D, ok = (size_t)(b * T + t) * K;
            lfw_step(S, x + od, f + od, k + ok, fk + ok, (int)D, (int)K);
        }
        memcpy(R, g_state + b * DK, sizeof(double) * DK);
        /* R currently holds the part of R_t that arrives from the future */
        for (int64_t sg = nseg - 1; sg >= 0; --sg) {
            const int64_t t0 = sg * ORACLE_SEG;
            const int64_t t1 = (t0 + ORACLE_SEG < T) ? t0 + ORACLE_SEG : T;
            /* hist[j] = state before step t0+j; hist[t1-t0] = state after step t1-1 */
            memcpy(hist, seg0 + sg * DK, sizeof(double) * DK);
            for (int64_t t = t0; t < t1; ++t) {
                double *nxt = hist + (t - t0 + 1) * DK;
                memcpy(nxt, hist + (t - t0) * DK, sizeof(double) * DK);
                const size_t od = (size_t)(b * T + t) * D, ok = (size_t)(b * T + t) * K;
                lfw_step(nxt, x + od, f + od, k + ok, fk + ok, (int)D, (int)K);
            }
            for (int64_t t = t1 - 1; t >= t0; --t) {
                const size_t od = (size_t)(b * T + t) * D, ok = (size_t)(b * T + t) * K;
                const double *Sprev = hist + (t - t0) * DK;
                const double *Scur = hist + (t - t0 + 1) * DK;
                for (int64_t c = 0; c < K; ++c) { dq[ok + c] = 0; dk[ok + c] = 0; dfk[ok + c] = 0; }
                for (int64_t d = 0; d < D; ++d) {
                    double sdx = 0, sdf = 0;
                    const double go = g_out[od + d];
                    for (int64_t c = 0; c < K; ++c) {
                        const double r = R[d * K + c] + go * q[ok + c];      /* R_t */
                        const double w = r * Sprev[d * K + c];               /* W_t */
                        dq[ok + c] += Scur[d * K + c] * go;
                        sdx += r * k[ok + c];
                        dk[ok + c] += r * x[od + d];
                        sdf += w * fk[ok + c];
                        dfk[ok + c] += w * f[od + d];
                        R[d * K + c] = r * (f[od + d] * fk[ok + c]);         /* flows to S_{t-1} */
                    }
                    dx[od + d] = sdx;
                    df[od + d] = sdf;
                }
            }
        }
        memcpy(ds0 + b * DK, R, sizeof(double) * DK);
        free(seg0); free(hist); free(R); free(S);
    }
}

/* ------------------------------------------------------------------------------------ */
/* delta rule:  o_t = S_{t-1} q_t ; delta_t = v_t - S_{t-1} k_t ; S_t = S_{t-1} + delta_t k_t^T */
/* ------------------------------------------------------------------------------------ */

void t2fw_oracle_dfw_forward(const double *q, const double *k, const double *v,
                             const double *s0, int64_t B, int64_t T, int64_t D, int64_t M,
                             double *out, double *s_final, double *delta /* may be NULL */)
{
#pragma omp parallel for schedule(dynamic)
    for (int64_t b = 0; b < B; ++b) {
        double *S = (double *)malloc(sizeof(double) * D * M);
        memcpy(S, s0 + b * D * M, sizeof(double) * D * M);
        for (int64_t t = 0; t < T; ++t) {
            const size_t od = (size_t)(b * T + t) * D, om = (size_t)(b * T + t) * M;
            for (int64_t d = 0; d < D; ++d) {
                double so = 0, sk = 0;
                for (int64_t m = 0; m < M; ++m) {
                    so += S[d * M + m] * q[om + m];
                    sk += S[d * M + m] * k[om + m];
                }
                out[od + d] = so;
                const double dl = v[od + d] - sk;
                if (delta) delta[od + d] = dl;
                for (int64_t m = 0; m < M; ++m) S[d * M + m] += dl * k[om + m];
            }
        }
        memcpy(s_final + b * D * M, S, sizeof(double) * D * M);
        free(S);
    }
}

/*
 * Backward of the delta rule.  With G_t the gradient w.r.t. S_t (G_T = g_state):
 *   dv_t   = G_t k_t
 *   dq_t   = S_{t-1}^T g_out_t
 *   dk_t   = G_t^T delta_t - S_{t-1}^T dv_t
 *   G_{t-1} = G_t - dv_t k_t^T + g_out_t q_t^T ,   ds0 = G_0
 * The states S_{t-1} are recomputed forward from stored segment starts (the reference walks
 * them backwards from the final state, t2fw/torch.py:116; both give the same values).
 */
void t2fw_oracle_dfw_backward(const double *g_out, const double *g_state,
                              const double *q, const double *k, const double *v,
                              const double *s0, int64_t B, int64_t T, int64_t D, int64_t M,
                              double *dq, double *dk, double *dv, double *ds0)
{
    const int64_t DM = D * M;
    const int64_t nseg = (T + ORACLE_SEG - 1) / ORACLE_SEG;
#pragma omp parallel for schedule(dynamic)
    for (int64_t b = 0; b < B; ++b) {
        double *seg0 = (double *)malloc(sizeof(double) * DM * (nseg > 0 ? nseg : 1));
        double *hist = (double *)malloc(sizeof(double) * DM * (ORACLE_SEG + 1));
        double *dlt = (double *)malloc(sizeof(double) * D * ORACLE_SEG);
        double *G = (double *)malloc(sizeof(double) * DM);
        double *S = (double *)malloc(sizeof(double) * DM);
        memcpy(S, s0 + b * DM, sizeof(double) * DM);
        for (int64_t t = 0; t < T; ++t) {
            if (t % ORACLE_SEG == 0) memcpy(seg0 + (t / ORACLE_SEG) * DM, S, sizeof(double) * DM);
            const size_t od = (size_t)(b * T + t) * D, om = (size_t)(b * T + t) * M;
            for (int64_t d = 0; d < D; ++d) {
                double sk = 0;
                for (int64_t m = 0; m < M; ++m) sk += S[d * M + m] * k[om + m];
                const double dl = v[od + d] - sk;
                for (int64_t m = 0; m < M; ++m) S[d * M + m] += dl * k[om + m];
            }
        }
        memcpy(G, g_state + b * DM, sizeof(double) * DM);
        for (int64_t sg = nseg - 1; sg >= 0; --sg) {
            const int64_t t0 = sg * ORACLE_SEG;
            const int64_t t1 = (t0 + ORACLE_SEG < T) ? t0 + ORACLE_SEG : T;
            memcpy(hist, seg0 + sg * DM, sizeof(double) * DM);
            for (int64_t t = t0; t < t1; ++t) {
                const double *cur = hist + (t - t0) * DM;
                double *nxt = hist + (t - t0 + 1) * DM;
                const size_t od = (size_t)(b * T + t) * D, om = (size_t)(b * T + t) * M;
                for (int64_t d = 0; d < D; ++d) {
                    double sk = 0;
                    for (int64_t m = 0; m < M; ++m) sk += cur[d * M + m] * k[om + m];
                    const double dl = v[od + d] - sk;
                    dlt[(t - t0) * D + d] = dl;
                    for (int64_t m = 0; m < M; ++m) nxt[d * M + m] = cur[d * M + m] + dl * k[om + m];
                }
            }
            for (int64_t t = t1 - 1; t >= t0; --t) {
                const size_t od = (size_t)(b * T + t) * D, om = (size_t)(b * T + t) * M;
                const double *Sprev = hist + (t - t0) * DM;
                for (int64_t m = 0; m < M; ++m) { dq[om + m] = 0; dk[om + m] = 0; }
                for (int64_t d = 0; d < D; ++d) {
                    double sdv = 0;
                    for (int64_t m = 0; m < M; ++m) sdv += G[d * M + m] * k[om + m];
                    dv[od + d] = sdv;
                    const double go = g_out[od + d];
                    const double dl = dlt[(t - t0) * D + d];
                    for (int64_t m = 0; m < M; ++m) {
                        dq[om + m] += Sprev[d * M + m] * go;
                        dk[om + m] += G[d * M + m] * dl - Sprev[d * M + m] * sdv;
                        G[d * M + m] += go * q[om + m] - sdv * k[om + m];
                    }
                }
            }
        }
        memcpy(ds0 + b * DM, G, sizeof(double) * DM);
        free(seg0); free(hist); free(dlt); free(G); free(S);
    }
}
