/*
 * CPU oracle for the Mamba-1 selective-scan path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped library links, loads or calls this file; it is the
 * checker the parity tests, the smoke check and the CPU-baseline leg of the
 * benchmark compare the CUDA path against.
 *
 * It restates, in plain C and in the reference's own f32 operation order, the
 * CPU implementation of silvermpx/mamba-rs v0.5.3.  Every function cites the
 * reference file:line it follows.  The reference is Rust and cannot be built
 * in an image without cargo, and its test-suite stores no golden vectors for
 * this path (all of its checks are property / tolerance tests), so:
 *
 *   PARITY PIN STATUS: pinned against the reference's own test PROPERTIES
 *   (fast_exp accuracy and edge cases of src/ops/fast_math.rs:263-341, the
 *   step == batched == prefill identities of tests/prefill.rs:90-168, the
 *   f64 finite-difference gradient check of tests/grad_oracle.rs) and, on a
 *   GPU box, against the reference's own CUDA kernels compiled unchanged from
 *   its sources (oracle/_ref): scan forward (parallel and sequential), scan
 *   backward (ssm_parallel_scan_bwd_*, ssm_backward_local_* and the four
 *   reducers), conv1d forward and backward, within 1e-4 (f32) / 2e-2 (16-bit
 *   storage).  Bit-level parity with a build of the Rust CPU code itself is
 *   UNPINNED.
 *
 * Build: make -C oracle   (gcc -O2 -ffp-contract=off: Rust never contracts
 * a*b+c into an fma, so neither may the C compiler.)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* fast_exp: Cephes degree-7 exp, src/ops/fast_math.rs:17-74 (scalar) and    */
/* :187-257 (AVX2+FMA 8-wide form used by fast_exp_inplace on x86_64).       */
/* ------------------------------------------------------------------------ */
static const float EXP_HI = 88.37626f, EXP_LO = -88.37626f;
static const float LOG2EF = 1.44269504088896341f;
static const float LN2_HI = 0.6933594f, LN2_LO = -2.1219444e-4f;
static const float CP0 = 1.987569e-4f, CP1 = 1.3982e-3f, CP2 = 8.333452e-3f,
                   CP3 = 4.16658e-2f, CP4 = 1.666667e-1f, CP5 = 0.5f;

/* src/ops/fast_math.rs:38-51 — round to nearest even via the 2^23 trick. */
static inline float roundeven_f(float x) {
    const float MAGIC = 8388608.0f;
    volatile float t;
    if (x >= 0.0f) {
        if (x >= MAGIC) return x;
        t = x + MAGIC;
        return t - MAGIC;
    }
    if (-x >= MAGIC) return x;
    t = x - MAGIC;
    return t + MAGIC;
}

static inline float pow2n_bits(float n) {
    int32_t ni = (int32_t)n;
    uint32_t bits = (uint32_t)(ni + 127) << 23;
    float r;
    memcpy(&r, &bits, 4);
    return r;
}

/* src/ops/fast_math.rs:53-74 — scalar form: every mul and add rounds. */
ORC_API float orc_fast_exp_scalar(float x) {
    if (x < EXP_LO) x = EXP_LO;
    if (x > EXP_HI) x = EXP_HI;
    float n = roundeven_f(x * LOG2EF);
    float r = x - n * LN2_HI - n * LN2_LO;
    float r2 = r * r;
    float p = CP0;
    p = p * r + CP1;
    p = p * r + CP2;
    p = p * r + CP3;
    p = p * r + CP4;
    p = p * r + CP5;
    p = p * r2 + r + 1.0f;
    return p * pow2n_bits(n);
}

/* src/ops/fast_math.rs:213-252 — one lane of the AVX2 body: the range
 * reduction uses separate mul/sub, the polynomial uses fused multiply-add. */
ORC_API float orc_fast_exp_simd_lane(float x) {
    if (x < EXP_LO) x = EXP_LO; /* _mm256_max_ps then _mm256_min_ps */
    if (x > EXP_HI) x = EXP_HI;
    float n = roundeven_f(x * LOG2EF);
    float r = (x - n * LN2_HI) - n * LN2_LO;
    float r2 = r * r;
    float p = fmaf(CP0, r, CP1);
    p = fmaf(p, r, CP2);
    p = fmaf(p, r, CP3);
    p = fmaf(p, r, CP4);
    p = fmaf(p, r, CP5);
    p = fmaf(p, r2, r);
    p = p + 1.0f;
    return p * pow2n_bits(n);
}

/* src/ops/fast_math.rs:82-107 — in-place slice exp: 8-wide SIMD body and a
 * scalar tail (the x86_64 dispatch with AVX2+FMA present). */
ORC_API void orc_fast_exp_inplace(float *buf, long n) {
    long body = (n / 8) * 8;
    for (long i = 0; i < body; i++) buf[i] = orc_fast_exp_simd_lane(buf[i]);
    for (long i = body; i < n; i++) buf[i] = orc_fast_exp_scalar(buf[i]);
}

/* softplus with threshold 20: src/mamba_ssm/cpu/prefill.rs:593-599 */
static inline float softplus_ref(float v) {
    return v <= 20.0f ? log1pf(orc_fast_exp_scalar(v)) : v;
}
/* conv-side SiLU: prefill.rs:222-224  (val / (1 + exp(-val))) */
static inline float silu_div(float v) { return v / (1.0f + orc_fast_exp_scalar(-v)); }
/* gate-side SiLU: prefill.rs:506-508  (g * (1 / (1 + exp(-g)))) */
static inline float silu_mul(float g) { return g * (1.0f / (1.0f + orc_fast_exp_scalar(-g))); }

/* ------------------------------------------------------------------------ */
/* Fused-op view of the path.  All tensors f32; storage-dtype rounding of    */
/* the inputs is applied by the caller before the call, so the oracle and    */
/* the CUDA kernel see identical values.                                     */
/* ------------------------------------------------------------------------ */
typedef struct {
    int B, T, D, N, K;      /* K = 0: no conv, x is already u            */
    long ld_x, ld_delta, ld_z, ld_bc, ld_y; /* row strides (elements)     */
    int delta_softplus;     /* 1: delta input is raw (bias included)     */
    int has_z;              /* 1: multiply by silu(z)                    */
} OrcM1Shape;

/*
 * Forward of the fused op for one sample b (the reference treats samples
 * independently; prefill_batch, prefill.rs:702-727).
 *   conv + SiLU      : prefill.rs:178-225 (shift register == bulk form)
 *   softplus         : prefill.rs:593-599
 *   recurrence       : prefill.rs:241-315 / cpu/forward.rs:235-283
 *   D skip + gating  : prefill.rs:303-306, :646-655
 * conv_state is the GPU-convention full window [D,K] oldest->newest
 * (kernels/conv1d.cu:30-35); ssm_state [D,N] is h0 in, h_T out.
 * Optional outputs (may be NULL): u_out[T,D], dl_out[T,D] (post-softplus),
 * pc_out[T,D] (conv pre-activation), yssm_out[T,D] (pre-gate y), h_all
 * [(T+1),D,N] with slot 0 = h0 (kernels/mamba_ssm.cu:261-293).
 */
static void m1_fwd_sample(const OrcM1Shape *s, const float *x, const float *delta,
                          const float *Bm, const float *Cm, const float *z,
                          const float *a_neg, const float *Dp, const float *conv_w,
                          const float *conv_b, float *conv_state, float *ssm_state,
                          float *y, float *u_out, float *dl_out, float *pc_out,
                          float *yssm_out, float *h_all, int d_begin, int d_end,
                          int train_form) {
    const int T = s->T, D = s->D, N = s->N, K = s->K;
    float *da = (float *)malloc(sizeof(float) * (size_t)(N > 8 ? N : 8));
    if (h_all)
        memcpy(h_all + (size_t)d_begin * N, ssm_state + (size_t)d_begin * N,
               sizeof(float) * (size_t)(d_end - d_begin) * N);
    for (int d = d_begin; d < d_end; d++) {
        float *reg = K ? conv_state + (size_t)d * K : NULL;
        float *h = ssm_state + (size_t)d * N;
        for (int t = 0; t < T; t++) {
            float u;
            if (K) {
                for (int k = 0; k < K - 1; k++) reg[k] = reg[k + 1];
                reg[K - 1] = x[(size_t)t * s->ld_x + d];
                float val = conv_b[d];
                for (int k = 0; k < K; k++) val += reg[k] * conv_w[(size_t)d * K + k];
                if (pc_out) pc_out[(size_t)t * D + d] = val;
                u = silu_div(val);
            } else {
                u = x[(size_t)t * s->ld_x + d];
            }
            float dl = delta[(size_t)t * s->ld_delta + d];
            if (s->delta_softplus) dl = softplus_ref(dl);
            if (u_out) u_out[(size_t)t * D + d] = u;
            if (dl_out) dl_out[(size_t)t * D + d] = dl;
            float du = dl * u;
            for (int n = 0; n < N; n++) da[n] = dl * a_neg[(size_t)d * N + n];
            /* prefill.rs:287 exponentiates d_state * SSM_BLOCK lanes at once (always a
             * multiple of 8: every lane takes the AVX2 form); the training forward
             * (cpu/forward.rs:246-249) exponentiates the d_state values of one channel
             * (AVX2 body, scalar tail). */
            if (train_form) orc_fast_exp_inplace(da, N);
            else for (int n = 0; n < N; n++) da[n] = orc_fast_exp_simd_lane(da[n]);
            const float *Bt = Bm + (size_t)t * s->ld_bc;
            const float *Ct = Cm + (size_t)t * s->ld_bc;
            float acc = 0.0f;
            for (int n = 0; n < N; n++) {
                float hn = da[n] * h[n] + du * Bt[n];
                h[n] = hn;
                acc += hn * Ct[n];
            }
            if (h_all) memcpy(h_all + ((size_t)(t + 1) * D + d) * N, h, sizeof(float) * N);
            float yv = acc + Dp[d] * u;
            if (yssm_out) yssm_out[(size_t)t * D + d] = yv;
            if (s->has_z) yv *= silu_mul(z[(size_t)t * s->ld_z + d]);
            y[(size_t)t * s->ld_y + d] = yv;
        }
    }
    free(da);
}

ORC_API int orc_m1_fused_fwd(const OrcM1Shape *s, const float *x, const float *delta,
                             const float *Bm, const float *Cm, const float *z,
                             const float *a_neg, const float *Dp, const float *conv_w,
                             const float *conv_b, float *conv_state, float *ssm_state,
                             float *y, float *u_out, float *dl_out, float *h_all) {
    const size_t T = s->T, D = s->D, N = s->N;
    const int DB = 8; /* channels per task: SSM_BLOCK, prefill.rs:234 */
    const int nblk = (s->D + DB - 1) / DB;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < s->B; b++)
      for (int blk = 0; blk < nblk; blk++) {
        int d_begin = blk * DB, d_end = d_begin + DB < s->D ? d_begin + DB : s->D;
        m1_fwd_sample(s, x + b * T * s->ld_x, delta + b * T * s->ld_delta,
                      Bm + b * T * s->ld_bc, Cm + b * T * s->ld_bc,
                      s->has_z ? z + b * T * s->ld_z : NULL, a_neg, Dp, conv_w, conv_b,
                      s->K ? conv_state + b * D * s->K : NULL, ssm_state + b * D * N,
                      y + b * T * s->ld_y, u_out ? u_out + b * T * D : NULL,
                      dl_out ? dl_out + b * T * D : NULL, NULL, NULL,
                      h_all ? h_all + b * (T + 1) * D * N : NULL, d_begin, d_end, 0);
      }
    return 0;
}

/*
 * Backward of the fused op (BPTT), following src/mamba_ssm/cpu/backward.rs:
 *   gating backward  :62-82      d_y = dg*silu(z), d_z = dg*y*silu'(z)
 *   SSM BPTT         :84-150     reverse t; d_D, d_u, d_delta, d_B, d_C, d_a_log
 *   softplus backward:152-166
 *   SiLU + conv bwd  :228-274 with backward_ops.rs:22-58 (shift-register carry)
 * Activations are recomputed by m1_fwd_sample (the reference reads its saved
 * tape; the values are the same).  dg = gradient w.r.t. the op output.
 * d_u_extra (may be NULL) is added to d_u before the SiLU/conv backward: the
 * reference adds the x_proj GEMM's input gradient there (backward.rs:210-226).
 * Per-sample outputs are overwritten: d_x[B,T,D] (d_u when K==0),
 * d_delta[B,T,D] (w.r.t. raw when delta_softplus), d_z[B,T,D], dB/dC[B,T,N].
 * Parameter gradients are accumulated (+=) over samples in sample order:
 * dA_log[D,N], dD[D], dconv_w[D,K], dconv_b[D].
 */
ORC_API int orc_m1_fused_bwd(const OrcM1Shape *s, const float *x, const float *delta,
                             const float *Bm, const float *Cm, const float *z,
                             const float *a_neg, const float *Dp, const float *conv_w,
                             const float *conv_b, const float *conv_state0,
                             const float *ssm_state0, const float *dg,
                             const float *d_u_extra, float *d_x, float *d_delta,
                             float *d_z, float *dBm, float *dCm, float *dA_log, float *dD,
                             float *dconv_w, float *dconv_b) {
    const size_t T = s->T, D = s->D, N = s->N, K = s->K;
    OrcM1Shape sp = *s;
    sp.ld_y = (long)D;
    for (int b = 0; b < s->B; b++) {
        float *cs = K ? (float *)malloc(sizeof(float) * D * K) : NULL;
        float *hs = (float *)malloc(sizeof(float) * D * N);
        if (K) {
            if (conv_state0) memcpy(cs, conv_state0 + b * D * K, sizeof(float) * D * K);
            else memset(cs, 0, sizeof(float) * D * K);
        }
        if (ssm_state0) memcpy(hs, ssm_state0 + b * D * N, sizeof(float) * D * N);
        else memset(hs, 0, sizeof(float) * D * N);
        float *yg = (float *)malloc(sizeof(float) * T * D);
        float *u = (float *)malloc(sizeof(float) * T * D);
        float *dl = (float *)malloc(sizeof(float) * T * D);
        float *pc = (float *)malloc(sizeof(float) * T * D);
        float *ys = (float *)malloc(sizeof(float) * T * D);
        float *h_all = (float *)malloc(sizeof(float) * (T + 1) * D * N);
        float *d_y = (float *)malloc(sizeof(float) * T * D);
        float *d_u = (float *)calloc(T * D, sizeof(float));
        float *d_h = (float *)calloc(D * N, sizeof(float));
        const float *xb = x + b * T * s->ld_x, *db = delta + b * T * s->ld_delta;
        const float *Bb = Bm + b * T * s->ld_bc, *Cb = Cm + b * T * s->ld_bc;
        const float *zb = s->has_z ? z + b * T * s->ld_z : NULL;
        m1_fwd_sample(&sp, xb, db, Bb, Cb, zb, a_neg, Dp, conv_w, conv_b, cs, hs, yg, u, dl,
                      pc, ys, h_all, 0, (int)D, 1);
        const float *dgb = dg + b * T * D;
        /* gating backward, backward.rs:62-82 */
        for (size_t i = 0; i < T * D; i++) {
            size_t t = i / D, d = i % D;
            if (s->has_z) {
                float zz = zb[t * s->ld_z + d];
                float gpost = silu_mul(zz);
                d_y[i] = dgb[i] * gpost;
                float sg = 1.0f / (1.0f + orc_fast_exp_scalar(-zz));
                float sgrad = sg * (1.0f + zz * (1.0f - sg));
                d_z[b * T * D + i] = dgb[i] * ys[i] * sgrad;
            } else {
                d_y[i] = dgb[i];
                if (d_z) d_z[b * T * D + i] = 0.0f;
            }
        }
        /* SSM BPTT, backward.rs:84-150 */
        for (size_t tt = T; tt-- > 0;) {
            float *dBt = dBm + (b * T + tt) * N, *dCt = dCm + (b * T + tt) * N;
            for (size_t n = 0; n < N; n++) dBt[n] = dCt[n] = 0.0f;
            const float *hp = h_all + tt * D * N, *hc = h_all + (tt + 1) * D * N;
            for (size_t d = 0; d < D; d++) {
                float dl_d = dl[tt * D + d], u_d = u[tt * D + d], dy_d = d_y[tt * D + d];
                dD[d] += dy_d * u_d;
                float ddl = 0.0f, duacc = 0.0f;
                duacc += dy_d * Dp[d];
                for (size_t n = 0; n < N; n++) {
                    size_t idx = d * N + n;
                    float a = a_neg[idx];
                    /* saved da_exp is the SIMD-form exp for N>=8 lanes and the
                     * scalar form in the tail (forward.rs:246-249). */
                    float da = ((long)n < ((long)N / 8) * 8) ? orc_fast_exp_simd_lane(dl_d * a)
                                                             : orc_fast_exp_scalar(dl_d * a);
                    float b_n = Bb[tt * s->ld_bc + n], c_n = Cb[tt * s->ld_bc + n];
                    d_h[idx] += dy_d * c_n;
                    float dh = d_h[idx];
                    ddl += dh * (a * da * hp[idx] + u_d * b_n);
                    duacc += dh * dl_d * b_n;
                    dBt[n] += dh * dl_d * u_d;
                    dCt[n] += dy_d * hc[idx];
                    dA_log[idx] += dh * da * dl_d * a * hp[idx];
                    d_h[idx] = da * dh;
                }
                d_u[tt * D + d] = duacc;
                /* softplus backward, backward.rs:152-166 */
                if (s->delta_softplus) {
                    float raw = db[tt * s->ld_delta + d];
                    if (raw <= 20.0f) ddl *= 1.0f / (1.0f + orc_fast_exp_scalar(-raw));
                }
                d_delta[b * T * D + tt * D + d] = ddl;
            }
        }
        if (d_u_extra)
            for (size_t i = 0; i < T * D; i++) d_u[i] += d_u_extra[b * T * D + i];
        if (!K) {
            memcpy(d_x + b * T * D, d_u, sizeof(float) * T * D);
        } else {
            /* SiLU backward + conv backward with carry, backward.rs:228-274 */
            float *carry = (float *)calloc(D * (K > 1 ? K - 1 : 1), sizeof(float));
            float *win = (float *)malloc(sizeof(float) * K);
            for (size_t tt = T; tt-- > 0;) {
                for (size_t d = 0; d < D; d++) {
                    float p = pc[tt * D + d];
                    float sg = 1.0f / (1.0f + orc_fast_exp_scalar(-p));
                    float dco = d_u[tt * D + d] * sg * (1.0f + p * (1.0f - sg));
                    /* window consumed at time tt: x[tt-K+1..tt], earlier taps
                     * come from the entering conv state (conv1d.cu:326-359). */
                    for (size_t k = 0; k < K; k++) {
                        long src = (long)tt - (long)(K - 1) + (long)k;
                        if (src >= 0) win[k] = xb[(size_t)src * s->ld_x + d];
                        else {
                            long j = (long)K + src; /* index into entering window */
                            win[k] = conv_state0 ? conv_state0[(b * D + d) * K + j] : 0.0f;
                        }
                    }
                    dconv_b[d] += dco;
                    for (size_t k = 0; k < K; k++) dconv_w[d * K + k] += dco * win[k];
                    float dx = dco * conv_w[d * K + K - 1];
                    if (K > 1) {
                        size_t cst = K - 1;
                        float *c = carry + d * cst;
                        dx += c[0];
                        for (size_t k = 0; k + 1 < cst; k++)
                            c[k] = c[k + 1] + dco * conv_w[d * K + K - 2 - k];
                        c[cst - 1] = dco * conv_w[d * K];
                    }
                    d_x[b * T * D + tt * D + d] = dx;
                }
            }
            free(carry);
            free(win);
        }
        free(cs); free(hs); free(yg); free(u); free(dl); free(pc); free(ys);
        free(h_all); free(d_y); free(d_u); free(d_h);
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* f64 shadow of the fused forward (libm exp/log1p, no fast paths): the      */
/* "truth" both the f32 oracle and the CUDA kernel are measured against,     */
/* after the template of tests/grad_oracle.rs:159-230 (forward_f64).         */
/* ------------------------------------------------------------------------ */
ORC_API int orc_m1_fused_fwd_f64(const OrcM1Shape *s, const double *x, const double *delta,
                                 const double *Bm, const double *Cm, const double *z,
                                 const double *a_neg, const double *Dp, const double *conv_w,
                                 const double *conv_b, double *conv_state,
                                 double *ssm_state, double *y) {
    const size_t T = s->T, D = s->D, N = s->N, K = s->K;
#pragma omp parallel for schedule(static)
    for (int b = 0; b < s->B; b++) {
        for (size_t d = 0; d < D; d++) {
            double *reg = K ? conv_state + (b * D + d) * K : NULL;
            double *h = ssm_state + (b * D + d) * N;
            for (size_t t = 0; t < T; t++) {
                double u;
                if (K) {
                    for (size_t k = 0; k + 1 < K; k++) reg[k] = reg[k + 1];
                    reg[K - 1] = x[(b * T + t) * s->ld_x + d];
                    double val = conv_b[d];
                    for (size_t k = 0; k < K; k++) val += reg[k] * conv_w[d * K + k];
                    u = val / (1.0 + exp(-val));
                } else u = x[(b * T + t) * s->ld_x + d];
                double dl = delta[(b * T + t) * s->ld_delta + d];
                if (s->delta_softplus && dl <= 20.0) dl = log1p(exp(dl));
                double acc = 0.0;
                for (size_t n = 0; n < N; n++) {
                    double hn = exp(dl * a_neg[d * N + n]) * h[n] +
                                dl * u * Bm[(b * T + t) * s->ld_bc + n];
                    h[n] = hn;
                    acc += hn * Cm[(b * T + t) * s->ld_bc + n];
                }
                double yv = acc + Dp[d] * u;
                if (s->has_z) {
                    double zz = z[(b * T + t) * s->ld_z + d];
                    yv *= zz / (1.0 + exp(-zz));
                }
                y[(b * T + t) * s->ld_y + d] = yv;
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------ */
/* T = 1 decode step of the fused op, src/mamba_ssm/cpu/inference.rs:117-196 */
/* (conv dot BEFORE shift: history taps, then x*w[K-1], then bias), on the   */
/* GPU-convention full-window conv state (slot 0 is the dead/oldest entry).  */
/* ------------------------------------------------------------------------ */
ORC_API int orc_m1_step(const OrcM1Shape *s, const float *x, const float *delta,
                        const float *Bm, const float *Cm, const float *z, const float *a_neg,
                        const float *Dp, const float *conv_w, const float *conv_b,
                        float *conv_state, float *ssm_state, float *y) {
    const size_t D = s->D, N = s->N, K = s->K;
    float *da = (float *)malloc(sizeof(float) * (N > 8 ? N : 8));
    for (int b = 0; b < s->B; b++)
        for (size_t d = 0; d < D; d++) {
            float u;
            if (K) {
                float *reg = conv_state + (b * D + d) * K; /* reg[1..K) = history */
                float val = 0.0f;
                for (size_t k = 0; k + 1 < K; k++) val += reg[k + 1] * conv_w[d * K + k];
                float xv = x[b * s->ld_x + d];
                val += xv * conv_w[d * K + K - 1];
                val += conv_b[d];
                for (size_t k = 0; k + 1 < K; k++) reg[k] = reg[k + 1];
                reg[K - 1] = xv;
                u = val * (1.0f / (1.0f + orc_fast_exp_scalar(-val)));
            } else u = x[b * s->ld_x + d];
            float dl = delta[b * s->ld_delta + d];
            if (s->delta_softplus) dl = dl > 20.0f ? dl : log1pf(orc_fast_exp_scalar(dl));
            float du = dl * u;
            for (size_t n = 0; n < N; n++) da[n] = dl * a_neg[d * N + n];
            orc_fast_exp_inplace(da, (long)N);
            float *h = ssm_state + (b * D + d) * N;
            float acc = 0.0f;
            for (size_t n = 0; n < N; n++) {
                h[n] = da[n] * h[n] + du * Bm[b * s->ld_bc + n];
                acc += h[n] * Cm[b * s->ld_bc + n];
            }
            acc += Dp[d] * u;
            if (s->has_z) acc *= silu_mul(z[b * s->ld_z + d]);
            y[b * s->ld_y + d] = acc;
        }
    free(da);
    return 0;
}

/* ------------------------------------------------------------------------ */
/* Seeded weights: src/weights.rs:107-160 (init), :224-250 (LCG, Kaiming,    */
/* inv_softplus).  Flat per-layer blocks in the order the reference draws.   */
/* ------------------------------------------------------------------------ */
typedef struct {
    int d_model, n_layers, d_state, d_conv, expand, dt_rank, input_dim;
} OrcM1Config;

static uint64_t lcg_next(uint64_t *st) {
    *st = *st * 6364136223846793005ULL + 1442695040888963407ULL;
    return *st;
}
static float lcg_f32(uint64_t *st) { return (float)(lcg_next(st) >> 40) / (float)(1ULL << 24); }
static void kaiming(float *w, size_t n, int fan_in, uint64_t *st) {
    float bound = sqrtf(3.0f / (float)fan_in);
    for (size_t i = 0; i < n; i++) w[i] = -bound + 2.0f * bound * lcg_f32(st);
}

/* Per-layer parameter block sizes, in this order:
 * norm_weight[dm] in_proj_w[dm*2di] conv_w[di*K] conv_b[di] x_proj_w[di*xd]
 * dt_proj_w[dr*di] dt_proj_b[di] a_log[di*N] a_neg[di*N] d_param[di] out_proj_w[di*dm] */
ORC_API long orc_m1_layer_floats(const OrcM1Config *c) {
    long dm = c->d_model, di = (long)c->expand * dm, N = c->d_state, K = c->d_conv,
         dr = c->dt_rank, xd = dr + 2 * N;
    return dm + dm * 2 * di + di * K + di + di * xd + dr * di + di + di * N + di * N + di + di * dm;
}
ORC_API long orc_m1_weights_floats(const OrcM1Config *c) {
    long dm = c->d_model;
    return (long)c->input_dim * dm + dm + c->n_layers * orc_m1_layer_floats(c) + dm;
}

typedef struct {
    float *norm_w, *in_proj_w, *conv_w, *conv_b, *x_proj_w, *dt_proj_w, *dt_proj_b, *a_log,
        *a_neg, *d_param, *out_proj_w;
} LayerView;

static LayerView layer_view(const OrcM1Config *c, float *base) {
    long dm = c->d_model, di = (long)c->expand * dm, N = c->d_state, K = c->d_conv,
         dr = c->dt_rank, xd = dr + 2 * N;
    LayerView v;
    v.norm_w = base; base += dm;
    v.in_proj_w = base; base += dm * 2 * di;
    v.conv_w = base; base += di * K;
    v.conv_b = base; base += di;
    v.x_proj_w = base; base += di * xd;
    v.dt_proj_w = base; base += dr * di;
    v.dt_proj_b = base; base += di;
    v.a_log = base; base += di * N;
    v.a_neg = base; base += di * N;
    v.d_param = base; base += di;
    v.out_proj_w = base;
    return v;
}

/* Layout of the flat weight buffer: input_proj_w[in*dm] input_proj_b[dm]
 * layer blocks ... norm_f[dm].  weights.rs:107-160. */
ORC_API int orc_m1_weights_init(const OrcM1Config *c, uint64_t seed, float *w) {
    long dm = c->d_model, di = (long)c->expand * dm, N = c->d_state, K = c->d_conv,
         dr = c->dt_rank, xd = dr + 2 * N;
    uint64_t st = seed;
    memset(w, 0, sizeof(float) * (size_t)orc_m1_weights_floats(c));
    kaiming(w, (size_t)c->input_dim * dm, c->input_dim, &st);
    float *p = w + (long)c->input_dim * dm + dm;
    float log_min = logf(0.001f), log_max = logf(0.1f);
    for (int l = 0; l < c->n_layers; l++, p += orc_m1_layer_floats(c)) {
        LayerView v = layer_view(c, p);
        for (long i = 0; i < dm; i++) v.norm_w[i] = 1.0f;
        kaiming(v.in_proj_w, (size_t)(dm * 2 * di), (int)dm, &st);
        kaiming(v.conv_w, (size_t)(di * K), (int)K, &st);
        kaiming(v.x_proj_w, (size_t)(di * xd), (int)di, &st);
        kaiming(v.dt_proj_w, (size_t)(dr * di), (int)dr, &st);
        for (long i = 0; i < di; i++) {
            float dt = expf(lcg_f32(&st) * (log_max - log_min) + log_min);
            v.dt_proj_b[i] = dt > 20.0f ? dt : logf(expf(dt) - 1.0f);
        }
        for (long d = 0; d < di; d++)
            for (long n = 0; n < N; n++) {
                v.a_log[d * N + n] = logf((float)(n + 1));
                v.a_neg[d * N + n] = -expf(v.a_log[d * N + n]); /* weights.rs compute_a_neg */
            }
        for (long i = 0; i < di; i++) v.d_param[i] = 1.0f;
        kaiming(v.out_proj_w, (size_t)(di * dm), (int)di, &st);
    }
    for (long i = 0; i < dm; i++) p[i] = 1.0f;
    return 0;
}

/* Row-major GEMM y[M,Nn] = bias + x[M,Kk] @ w[Kk,Nn] in the k-outer order of
 * the reference's scalar fallback, src/ops/blas.rs:132-148. */
static void gemm_ref(float *y, const float *x, const float *w, const float *bias, long M,
                     long Kk, long Nn) {
    for (long r = 0; r < M; r++) {
        float *yr = y + r * Nn;
        if (bias) memcpy(yr, bias, sizeof(float) * (size_t)Nn);
        else memset(yr, 0, sizeof(float) * (size_t)Nn);
        for (long k = 0; k < Kk; k++) {
            float xv = x[r * Kk + k];
            const float *wr = w + k * Nn;
            for (long j = 0; j < Nn; j++) yr[j] += xv * wr[j];
        }
    }
}

/*
 * Full-sequence backbone prefill of ONE sample, following
 * forward_mamba_backbone_prefill_mode, src/mamba_ssm/cpu/prefill.rs:420-696.
 * conv_state here is the GPU-convention [L][D,K] window (slot 0 dead,
 * prefill.rs:524-529); ssm_state [L][D,N].  Optional per-layer taps for
 * parity: y_gated[L][T,D] (input of out_proj), and the fused-op inputs
 * x_branch/z as proj[L][T,2D], delta_raw[L][T,D], xdbl[L][T,xd].
 */
ORC_API int orc_m1_prefill(const OrcM1Config *c, const float *w, const float *input, int T,
                           float *conv_state, float *ssm_state, float *out, float *tap_proj,
                           float *tap_delta_raw, float *tap_xdbl, float *tap_gated) {
    long dm = c->d_model, di = (long)c->expand * dm, N = c->d_state, K = c->d_conv,
         dr = c->dt_rank, xd = dr + 2 * N;
    const float eps = 1e-5f; /* RMS_NORM_EPS, fast_math.rs:17 */
    float *post = (float *)malloc(sizeof(float) * T * dm);
    float *proj = (float *)malloc(sizeof(float) * T * 2 * di);
    float *u = (float *)malloc(sizeof(float) * T * di);
    float *xdbl = (float *)malloc(sizeof(float) * T * xd);
    float *dtin = (float *)malloc(sizeof(float) * T * dr);
    float *draw = (float *)malloc(sizeof(float) * T * di);
    float *yg = (float *)malloc(sizeof(float) * T * di);
    float *o = (float *)malloc(sizeof(float) * T * dm);
    gemm_ref(out, input, w, w + (long)c->input_dim * dm, T, c->input_dim, dm);
    const float *p = w + (long)c->input_dim * dm + dm;
    for (int l = 0; l < c->n_layers; l++, p += orc_m1_layer_floats(c)) {
        LayerView v = layer_view(c, (float *)p);
        for (long t = 0; t < T; t++) { /* F1 RMSNorm, prefill.rs:473-487 */
            const float *src = out + t * dm;
            float ss = 0.0f;
            for (long i = 0; i < dm; i++) ss += src[i] * src[i];
            float inv = 1.0f / sqrtf(ss / (float)dm + eps);
            for (long i = 0; i < dm; i++) post[t * dm + i] = src[i] * inv * v.norm_w[i];
        }
        gemm_ref(proj, post, v.in_proj_w, NULL, T, dm, 2 * di); /* F2 */
        /* F4a conv + SiLU on the x branch to get u for x_proj (prefill.rs:531-564) */
        OrcM1Shape s = {1, T, (int)di, (int)N, (int)K, 2 * di, di, 2 * di, xd, di, 1, 1};
        float *cs = conv_state + (long)l * di * K, *hs = ssm_state + (long)l * di * N;
        float *cs_tmp = (float *)malloc(sizeof(float) * di * K);
        memcpy(cs_tmp, cs, sizeof(float) * di * K);
        for (long d = 0; d < di; d++) {
            float *reg = cs_tmp + d * K;
            for (long t = 0; t < T; t++) {
                for (long k = 0; k < K - 1; k++) reg[k] = reg[k + 1];
                reg[K - 1] = proj[t * 2 * di + d];
                float val = v.conv_b[d];
                for (long k = 0; k < K; k++) val += reg[k] * v.conv_w[d * K + k];
                u[t * di + d] = silu_div(val);
            }
        }
        free(cs_tmp);
        gemm_ref(xdbl, u, v.x_proj_w, NULL, T, di, xd); /* F4b */
        for (long t = 0; t < T; t++) memcpy(dtin + t * dr, xdbl + t * xd, sizeof(float) * dr);
        gemm_ref(draw, dtin, v.dt_proj_w, v.dt_proj_b, T, dr, di); /* F4c (pre-softplus) */
        if (tap_proj) memcpy(tap_proj + (long)l * T * 2 * di, proj, sizeof(float) * T * 2 * di);
        if (tap_delta_raw) memcpy(tap_delta_raw + (long)l * T * di, draw, sizeof(float) * T * di);
        if (tap_xdbl) memcpy(tap_xdbl + (long)l * T * xd, xdbl, sizeof(float) * T * xd);
        /* F4a(again, carrying the real state)+F4c softplus+F4d+F4e: the fused op */
        m1_fwd_sample(&s, proj, draw, xdbl + dr, xdbl + dr + N, proj + di, v.a_neg, v.d_param,
                      v.conv_w, v.conv_b, cs, hs, yg, NULL, NULL, NULL, NULL, NULL, 0, (int)di, 0);
        if (tap_gated) memcpy(tap_gated + (long)l * T * di, yg, sizeof(float) * T * di);
        gemm_ref(o, yg, v.out_proj_w, NULL, T, di, dm); /* F5 */
        for (long i = 0; i < T * dm; i++) out[i] += o[i]; /* F6 */
    }
    for (long t = 0; t < T; t++) { /* norm_f at every position, prefill.rs:685-695 */
        float *row = out + t * dm;
        float ss = 0.0f;
        for (long i = 0; i < dm; i++) ss += row[i] * row[i];
        float inv = 1.0f / sqrtf(ss / (float)dm + eps);
        for (long i = 0; i < dm; i++) row[i] *= inv * p[i];
    }
    free(post); free(proj); free(u); free(xdbl); free(dtin); free(draw); free(yg); free(o);
    return 0;
}

/* Batch of independent samples, one task per sample (prefill_batch,
 * prefill.rs:702-727).  Returns the number of threads used. */
ORC_API int orc_m1_prefill_batch(const OrcM1Config *c, const float *w, const float *input,
                                 int B, int T, float *conv_state, float *ssm_state,
                                 float *out) {
    long dm = c->d_model, di = (long)c->expand * dm, L = c->n_layers;
    int nthreads = 1;
#pragma omp parallel
    {
#ifdef _OPENMP
#pragma omp single
        nthreads = omp_get_num_threads();
#endif
#pragma omp for schedule(dynamic, 1)
        for (int b = 0; b < B; b++)
            orc_m1_prefill(c, w, input + (long)b * T * c->input_dim, T,
                           conv_state + (long)b * L * di * c->d_conv,
                           ssm_state + (long)b * L * di * c->d_state,
                           out + (long)b * T * dm, NULL, NULL, NULL, NULL);
    }
    return nthreads;
}

/* Sets the OpenMP team size for later calls (a launcher such as torchrun exports
 * OMP_NUM_THREADS=1 to its workers; the CPU baseline wants every host core). */
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------ */
/* Standalone conv1d + SiLU over a sequence and its backward, for the        */
/* kernels that run the conv as a separate launch.                           */
/*   forward : prefill.rs:178-225 (== cpu/forward.rs:157-191)                */
/*   backward: cpu/backward.rs:228-274 + backward_ops.rs:22-58               */
/* conv_state [B,D,K] is the GPU-convention window, in/out for the forward,  */
/* the ENTERING window for the backward.  dW/db accumulate (+=).             */
/* ------------------------------------------------------------------------ */
ORC_API int orc_conv1d_fwd(int B, int T, int D, int K, const float *x, long ld_x,
                           const float *w, const float *bias, float *conv_state, float *u) {
    for (int b = 0; b < B; b++)
        for (int d = 0; d < D; d++) {
            float *reg = conv_state + ((size_t)b * D + d) * K;
            for (int t = 0; t < T; t++) {
                for (int k = 0; k < K - 1; k++) reg[k] = reg[k + 1];
                reg[K - 1] = x[((size_t)b * T + t) * ld_x + d];
                float val = bias[d];
                for (int k = 0; k < K; k++) val += reg[k] * w[(size_t)d * K + k];
                u[((size_t)b * T + t) * D + d] = silu_div(val);
            }
        }
    return 0;
}

ORC_API int orc_conv1d_bwd(int B, int T, int D, int K, const float *x, long ld_x,
                           const float *w, const float *bias, const float *conv_state0,
                           const float *d_u, float *d_x, float *dW, float *db) {
    float *carry = (float *)malloc(sizeof(float) * (size_t)D * (K > 1 ? K - 1 : 1));
    float *win = (float *)malloc(sizeof(float) * (size_t)K);
    for (int b = 0; b < B; b++) {
        memset(carry, 0, sizeof(float) * (size_t)D * (K > 1 ? K - 1 : 1));
        for (int t = T - 1; t >= 0; t--)
            for (int d = 0; d < D; d++) {
                for (int k = 0; k < K; k++) {
                    long src = (long)t - (K - 1) + k;
                    if (src >= 0) win[k] = x[((size_t)b * T + src) * ld_x + d];
                    else win[k] = conv_state0 ? conv_state0[((size_t)b * D + d) * K + K + src] : 0.0f;
                }
                float p = bias[d];
                for (int k = 0; k < K; k++) p += win[k] * w[(size_t)d * K + k];
                float sg = 1.0f / (1.0f + orc_fast_exp_scalar(-p));
                float dco = d_u[((size_t)b * T + t) * D + d] * sg * (1.0f + p * (1.0f - sg));
                db[d] += dco;
                for (int k = 0; k < K; k++) dW[(size_t)d * K + k] += dco * win[k];
                float dx = dco * w[(size_t)d * K + K - 1];
                if (K > 1) {
                    int cst = K - 1;
                    float *c = carry + (size_t)d * cst;
                    dx += c[0];
                    for (int k = 0; k + 1 < cst; k++) c[k] = c[k + 1] + dco * w[(size_t)d * K + K - 2 - k];
                    c[cst - 1] = dco * w[(size_t)d * K];
                }
                d_x[((size_t)b * T + t) * D + d] = dx;
            }
    }
    free(carry);
    free(win);
    return 0;
}
