/*
 * CPU oracle for the Mamba-3 SISO SSD scan (trapezoidal recurrence).  TEST
 * INFRASTRUCTURE ONLY — see the header of m1_oracle.c; the same rules and the
 * same parity-pin status apply (the reference is Rust, its tests hold no
 * golden vectors for this path; pinned on properties, unpinned at bit level).
 *
 * Boundary: the inputs exactly as the reference's chunked kernels consume them
 * (kernels/mamba3_chunked.cu:57-115, :346-419): x [B,T,nh*hd] (V), K and Q
 * [B,T,nh,N] after bias + RoPE, dt [B,T,nh] after softplus, trap [B,T,nh]
 * after sigmoid, adt = A*dt [B,T,nh], D [nh].
 *
 * Definition (sequential), src/mamba3_siso/cpu/forward.rs:85-138, :385-415:
 *   alpha = exp(adt), beta = alpha*dt*(1-trap), gamma = trap*dt
 *   h[p,n] = alpha*h[p,n] + (beta*v_prev[p])*k_prev[n] + (gamma*x[p])*k[n]
 *   y[p]   = sum_n h[p,n]*q[n] + D*x[p]
 * with k_prev / v_prev the previous step's k and x (the carried k_state /
 * v_state), evaluated with the reference's fused multiply-adds.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

float orc_fast_exp_scalar(float x); /* m1_oracle.c, src/ops/fast_math.rs:53-74 */

typedef struct {
    int B, T, nh, hd, N;
} OrcM3Shape;

/* Sequential forward; states are in/out: ssm [B,nh,hd,N], kst [B,nh,N], vst [B,nh,hd].
 * h_all (optional) [B,(T+1),nh,hd,N] keeps every state (slot 0 = entering). */
ORC_API int orc_m3_ssd_fwd(const OrcM3Shape *s, const float *x, const float *K, const float *Q,
                           const float *dt, const float *trap, const float *adt, const float *Dh,
                           float *ssm, float *kst, float *vst, float *y, float *h_all) {
    const size_t T = s->T, nh = s->nh, hd = s->hd, N = s->N, di = nh * hd;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < s->B; b++)
        for (int h = 0; h < s->nh; h++) {
            float *st = ssm + ((size_t)b * nh + h) * hd * N;
            float *kp = kst + ((size_t)b * nh + h) * N;
            float *vp = vst + ((size_t)b * nh + h) * hd;
            if (h_all) memcpy(h_all + (((size_t)b * (T + 1)) * nh + h) * hd * N, st, sizeof(float) * hd * N);
            for (size_t t = 0; t < T; t++) {
                const size_t th = ((size_t)b * T + t) * nh + h;
                const float alpha = orc_fast_exp_scalar(adt[th]);
                const float beta = alpha * dt[th] * (1.0f - trap[th]);
                const float gamma = trap[th] * dt[th];
                const float *kc = K + th * N, *qc = Q + th * N;
                const float *xc = x + ((size_t)b * T + t) * di + (size_t)h * hd;
                for (size_t p = 0; p < hd; p++) {
                    const float bv = beta * vp[p], gx = gamma * xc[p];
                    float *sp = st + p * N;
                    float acc = 0.0f;
                    for (size_t n = 0; n < N; n++) {
                        sp[n] = fmaf(alpha, sp[n], fmaf(bv, kp[n], gx * kc[n]));
                        acc = fmaf(sp[n], qc[n], acc);
                    }
                    y[((size_t)b * T + t) * di + (size_t)h * hd + p] = fmaf(Dh[h], xc[p], acc);
                }
                memcpy(kp, kc, sizeof(float) * N);
                memcpy(vp, xc, sizeof(float) * hd);
                if (h_all)
                    memcpy(h_all + (((size_t)b * (T + 1) + t + 1) * nh + h) * hd * N, st,
                           sizeof(float) * hd * N);
            }
        }
    return 0;
}

/* f64 shadow of the same definition (libm exp). */
ORC_API int orc_m3_ssd_fwd_f64(const OrcM3Shape *s, const double *x, const double *K, const double *Q,
                               const double *dt, const double *trap, const double *adt,
                               const double *Dh, double *y) {
    const size_t T = s->T, nh = s->nh, hd = s->hd, N = s->N, di = nh * hd;
    for (int b = 0; b < s->B; b++)
        for (size_t h = 0; h < nh; h++) {
            double *st = (double *)calloc(hd * N, sizeof(double));
            double *kp = (double *)calloc(N, sizeof(double));
            double *vp = (double *)calloc(hd, sizeof(double));
            for (size_t t = 0; t < T; t++) {
                const size_t th = ((size_t)b * T + t) * nh + h;
                const double alpha = exp(adt[th]), beta = alpha * dt[th] * (1.0 - trap[th]),
                             gamma = trap[th] * dt[th];
                const double *kc = K + th * N, *qc = Q + th * N, *xc = x + ((size_t)b * T + t) * di + h * hd;
                for (size_t p = 0; p < hd; p++) {
                    double acc = 0.0;
                    for (size_t n = 0; n < N; n++) {
                        st[p * N + n] = alpha * st[p * N + n] + beta * vp[p] * kp[n] + gamma * xc[p] * kc[n];
                        acc += st[p * N + n] * qc[n];
                    }
                    y[((size_t)b * T + t) * di + h * hd + p] = acc + Dh[h] * xc[p];
                }
                memcpy(kp, kc, sizeof(double) * N);
                memcpy(vp, xc, sizeof(double) * hd);
            }
            free(st); free(kp); free(vp);
        }
    return 0;
}

/*
 * Backward (BPTT) of the sequential definition from zero entering state,
 * src/mamba3_siso/cpu/backward.rs:178-268 (the RoPE / bias / norm parts of that
 * loop lie outside this boundary).  Outputs, all overwritten except dD (+=):
 *   dx [B,T,nh*hd], dK, dQ [B,T,nh,N], d_alpha, d_beta, d_gamma [B,T,nh], and
 *   their chain through alpha = exp(adt), beta = alpha*dt*(1-trap), gamma =
 *   trap*dt: d_adt, d_dt, d_trap [B,T,nh].
 */
ORC_API int orc_m3_ssd_bwd(const OrcM3Shape *s, const float *x, const float *K, const float *Q,
                           const float *dt, const float *trap, const float *adt, const float *Dh,
                           const float *dy, float *dx, float *dK, float *dQ, float *d_alpha,
                           float *d_beta, float *d_gamma, float *d_adt, float *d_dt, float *d_trap,
                           float *dD) {
    const size_t B = s->B, T = s->T, nh = s->nh, hd = s->hd, N = s->N, di = nh * hd;
    OrcM3Shape one = *s;
    memset(dx, 0, sizeof(float) * B * T * di);
    memset(dK, 0, sizeof(float) * B * T * nh * N);
    for (size_t b = 0; b < B; b++) {
        float *ssm = (float *)calloc(nh * hd * N, sizeof(float));
        float *kst = (float *)calloc(nh * N, sizeof(float));
        float *vst = (float *)calloc(nh * hd, sizeof(float));
        float *yb = (float *)malloc(sizeof(float) * T * di);
        float *h_all = (float *)malloc(sizeof(float) * (T + 1) * nh * hd * N);
        float *d_h = (float *)calloc(nh * hd * N, sizeof(float));
        one.B = 1;
        orc_m3_ssd_fwd(&one, x + b * T * di, K + b * T * nh * N, Q + b * T * nh * N, dt + b * T * nh,
                       trap + b * T * nh, adt + b * T * nh, Dh, ssm, kst, vst, yb, h_all);
        for (size_t t = T; t-- > 0;)
            for (size_t h = 0; h < nh; h++) {
                const size_t th = (b * T + t) * nh + h;
                const float alpha = orc_fast_exp_scalar(adt[th]);
                const float beta = alpha * dt[th] * (1.0f - trap[th]);
                const float gamma = trap[th] * dt[th];
                const float *kc = K + th * N, *qc = Q + th * N;
                const float *kp = t ? K + (th - nh) * N : NULL;
                float da = 0.0f, db = 0.0f, dg = 0.0f;
                float *dq = dQ + th * N;
                for (size_t n = 0; n < N; n++) dq[n] = 0.0f;
                for (size_t p = 0; p < hd; p++) {
                    const size_t xi = (b * T + t) * di + h * hd + p;
                    const float xv = x[xi], dyv = dy[xi];
                    const float vprev = t ? x[xi - di] : 0.0f;
                    dD[h] += dyv * xv;
                    const float *hc = h_all + (((t + 1) * nh + h) * hd + p) * N;
                    const float *hp = h_all + ((t * nh + h) * hd + p) * N;
                    float *dh = d_h + (h * hd + p) * N;
                    for (size_t n = 0; n < N; n++) {
                        dh[n] += dyv * qc[n];
                        dq[n] += dyv * hc[n];
                    }
                    float dxv = Dh[h] * dyv;
                    for (size_t n = 0; n < N; n++) {
                        const float g = dh[n];
                        const float kpn = kp ? kp[n] : 0.0f;
                        da += g * hp[n];
                        db += g * vprev * kpn;
                        dg += g * xv * kc[n];
                        if (t) {
                            dx[xi - di] += g * beta * kpn;
                            dK[(th - nh) * N + n] += g * beta * vprev;
                        }
                        dxv += g * gamma * kc[n];
                        dK[th * N + n] += g * gamma * xv;
                        dh[n] = alpha * g;
                    }
                    dx[xi] += dxv;
                }
                d_alpha[th] = da; d_beta[th] = db; d_gamma[th] = dg;
                d_adt[th] = alpha * da + beta * db;
                d_dt[th] = alpha * (1.0f - trap[th]) * db + trap[th] * dg;
                d_trap[th] = -alpha * dt[th] * db + dt[th] * dg;
            }
        free(ssm); free(kst); free(vst); free(yb); free(h_all); free(d_h);
    }
    return 0;
}

/*
 * Chunked reformulation of the forward for a stateless window (zero entering
 * state), as kernels/mamba3_chunked.cu:1-46 states it, in plain f32 loops:
 *   gamma_t = dt_t*trap_t, sgamma_t = dt_{t+1}(1-trap_{t+1}) (0 at the last step),
 *   scale_t = gamma_t + sgamma_t, dA = per-chunk inclusive cumsum of adt,
 *   y_t = exp(dA_t) q_t.S_in + sum_{s<t} exp(dA_t-dA_s) scale_s (q_t.k_s) v_s
 *         + (D + gamma_t q_t.k_t) v_t,
 *   S_out = exp(dA_end) S_in + sum_t exp(dA_end-dA_t) scale_t v_t k_t^T.
 * Used to check that the reformulation equals the sequential definition.
 */
ORC_API int orc_m3_ssd_fwd_chunked(const OrcM3Shape *s, int CS, const float *x, const float *K,
                                   const float *Q, const float *dt, const float *trap,
                                   const float *adt, const float *Dh, float *y, float *final_state) {
    const size_t T = s->T, nh = s->nh, hd = s->hd, N = s->N, di = nh * hd;
    float *dA = (float *)malloc(sizeof(float) * CS);
    float *sc = (float *)malloc(sizeof(float) * CS);
    float *gm = (float *)malloc(sizeof(float) * CS);
    for (int b = 0; b < s->B; b++)
        for (size_t h = 0; h < nh; h++) {
            float *S = (float *)calloc(hd * N, sizeof(float));
            float *Sn = (float *)malloc(sizeof(float) * hd * N);
            for (size_t c0 = 0; c0 < T; c0 += CS) {
                const size_t len = (c0 + CS <= T) ? (size_t)CS : T - c0;
                float run = 0.0f;
                for (size_t i = 0; i < len; i++) {
                    const size_t th = ((size_t)b * T + c0 + i) * nh + h;
                    run += adt[th];
                    dA[i] = run;
                    gm[i] = dt[th] * trap[th];
                    float sg = 0.0f;
                    if (c0 + i + 1 < T) sg = dt[th + nh] * (1.0f - trap[th + nh]);
                    sc[i] = gm[i] + sg;
                }
                for (size_t i = 0; i < len; i++) {
                    const size_t th = ((size_t)b * T + c0 + i) * nh + h;
                    const float *q = Q + th * N;
                    const float ed = orc_fast_exp_scalar(dA[i]);
                    for (size_t p = 0; p < hd; p++) {
                        float acc = 0.0f;
                        for (size_t n = 0; n < N; n++) acc += q[n] * S[p * N + n];
                        acc *= ed;
                        for (size_t j = 0; j < i; j++) {
                            const size_t tj = ((size_t)b * T + c0 + j) * nh + h;
                            float qk = 0.0f;
                            for (size_t n = 0; n < N; n++) qk += q[n] * K[tj * N + n];
                            acc += orc_fast_exp_scalar(dA[i] - dA[j]) * sc[j] * qk *
                                   x[((size_t)b * T + c0 + j) * di + h * hd + p];
                        }
                        float qkd = 0.0f;
                        for (size_t n = 0; n < N; n++) qkd += q[n] * K[th * N + n];
                        const float xv = x[((size_t)b * T + c0 + i) * di + h * hd + p];
                        y[((size_t)b * T + c0 + i) * di + h * hd + p] = acc + (Dh[h] + gm[i] * qkd) * xv;
                    }
                }
                const float eend = orc_fast_exp_scalar(dA[len - 1]);
                for (size_t i = 0; i < hd * N; i++) Sn[i] = eend * S[i];
                for (size_t i = 0; i < len; i++) {
                    const size_t th = ((size_t)b * T + c0 + i) * nh + h;
                    const float w = orc_fast_exp_scalar(dA[len - 1] - dA[i]) * sc[i];
                    for (size_t p = 0; p < hd; p++) {
                        const float wv = w * x[((size_t)b * T + c0 + i) * di + h * hd + p];
                        for (size_t n = 0; n < N; n++) Sn[p * N + n] += wv * K[th * N + n];
                    }
                }
                memcpy(S, Sn, sizeof(float) * hd * N);
            }
            if (final_state) memcpy(final_state + ((size_t)b * nh + h) * hd * N, S, sizeof(float) * hd * N);
            free(S); free(Sn);
        }
    free(dA); free(sc); free(gm);
    return 0;
}
