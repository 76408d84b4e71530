/*
 * libmamba_b200 — precompiled sm_100a kernels for the selective-scan hot path
 * of mamba-rs, behind a plain C ABI.
 *
 * The reference (silvermpx/mamba-rs v0.5.3) has no FFI on this path: it
 * compiles kernels/*.cu with NVRTC at start-up and launches `CudaFunction`s by
 * name (src/mamba_ssm/gpu/kernels.rs:547-564, :581-810;
 * src/mamba3_siso/gpu/kernels.rs:201-391).  Each entry point below names the
 * reference kernels / launch sites it replaces.  Conventions kept from that
 * boundary (src/mamba_ssm/gpu/buffers.rs:12-19,:142-147, forward_mixed.rs:150-155):
 *   - every pointer is a DEVICE pointer owned by the caller; nothing here
 *     allocates, frees or synchronises; launches are asynchronous on `stream`
 *     (a CUstream / cudaStream_t passed as void*);
 *   - activations are stored as f32 / f16 / bf16 (`dtype`), all arithmetic,
 *     recurrent state, a_neg, D, and every gradient accumulator is f32
 *     (kernels/mamba_ssm.cu:573-578, src/mamba_ssm/gpu/dtype.rs:12-28);
 *   - row strides (`ld_*`) are in ELEMENTS, so B/C can be read in place from
 *     xdbl[B*T, dt_rank+2N] and x/z from proj[B*T, 2*d_inner];
 *   - return value 0 = ok, negative = argument error (nothing was launched);
 *     mamba_b200_last_error() describes the last failure of the handle.
 */
#ifndef MAMBA_B200_H
#define MAMBA_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MAMBA_B200_API __attribute__((visibility("default")))
#else
#define MAMBA_B200_API
#endif

#define MAMBA_B200_F32 0  /* WeightDtype::F32  */
#define MAMBA_B200_F16 1  /* WeightDtype::F16  */
#define MAMBA_B200_BF16 2 /* WeightDtype::Bf16 */

#define MAMBA_B200_OK 0
#define MAMBA_B200_ERR_ARG (-1)     /* null / misaligned / out-of-range argument */
#define MAMBA_B200_ERR_SHAPE (-2)   /* unsupported shape (d_state > 256, d_conv > 8 ...) */
#define MAMBA_B200_ERR_CUDA (-3)    /* a CUDA runtime / driver call failed */
#define MAMBA_B200_ERR_DEVICE (-4)  /* not an sm_100 device */
#define MAMBA_B200_ERR_KERNEL (-5)  /* a kernel reported a bounded-wait timeout */

/* Create / destroy a per-device handle.  Replaces MambaKernels::new /
 * Mamba3Kernels::new (NVRTC compile + PTX cache, src/mamba_ssm/gpu/kernels.rs:451-545):
 * the cubins are linked into this library, nothing is compiled at run time.
 * init makes `device` current, raises the dynamic shared-memory limits of the
 * kernels and allocates one 4-byte device status word (the only allocation
 * the library ever makes). */
MAMBA_B200_API int mamba_b200_init(int device, void** handle);
MAMBA_B200_API int mamba_b200_destroy(void* handle);
MAMBA_B200_API const char* mamba_b200_last_error(void* handle);
/* Synchronously reads the device status word (bounded waits that gave up).
 * Returns 0 or MAMBA_B200_ERR_KERNEL.  Not graph-capturable; optional. */
MAMBA_B200_API int mamba_b200_check_status(void* handle, void* stream);
/* Diagnostic with no counterpart in the reference: launches one tiny kernel whose only
 * thread waits, for at most max_polls (1..100000) polls, on a barrier that nothing
 * signals.  The wait gives up, the kernel returns normally, and the next
 * mamba_b200_check_status reports MAMBA_B200_ERR_KERNEL once and clears the word:
 * the path every bounded wait of the library takes when it runs out. */
MAMBA_B200_API int mamba_b200_selftest_wait_timeout(void* handle, void* stream, int max_polls);

/*
 * Mamba-1 fused forward:
 *   [causal depthwise conv1d + SiLU] -> softplus(delta) -> selective scan
 *   -> + D*u -> * SiLU(z)
 * One launch replaces, per layer, conv1d_burnin_forward[_nosave]_{dt}
 * (kernels/conv1d.cu:161-359), softplus_copy / softplus_forward_{dt}
 * (kernels/elementwise.cu:305-313, kernels/activations.cu:34-52),
 * gather_bc_cols_{dt} (kernels/elementwise.cu:291-303),
 * ssm_parallel_scan_fwd[_nosave]_{dt} / ssm_burnin_forward[_nosave]_{dt}
 * (kernels/mamba_ssm_parallel.cu:265-1145, kernels/mamba_ssm.cu:232-455) and
 * the gate multiply elementwise_mul_{dt} (kernels/elementwise.cu:132-138);
 * launch sites src/mamba_ssm/gpu/forward_mixed.rs:500-717, prefill.rs:767-961.
 */
typedef struct mamba_b200_sscan_fwd_args {
    int dtype;           /* MAMBA_B200_F32 / F16 / BF16: storage of x, delta, B, C, z, y, u_out */
    int B, T, D, N;      /* batch, seq_len, d_inner, d_state (N <= 256) */
    const void* x;       /* [B*T, ld_x]: u, or the pre-conv x branch when conv_w != NULL */
    long long ld_x;
    const void* delta;   /* [B*T, ld_delta]: dt_proj output (bias included) */
    long long ld_delta;
    int delta_softplus;  /* 1: apply softplus (threshold 20) in-kernel; 0: delta is final */
    const void* Bm;      /* [B*T, ld_bc], N used columns */
    const void* Cm;      /* [B*T, ld_bc] */
    long long ld_bc;
    const void* z;       /* [B*T, ld_z] gate input, or NULL */
    long long ld_z;
    int z_mode;          /* 0: no gate; 1: y *= SiLU(z); 2: y *= z (z already holds SiLU(gate)) */
    const float* a_neg;  /* [D, N]  (-exp(a_log)) */
    const float* Dp;     /* [D] */
    const float* conv_w; /* [D, K] or NULL (no conv: x is u) */
    const float* conv_b; /* [D] (required with conv_w) */
    float* conv_state;   /* [B, D, K] window oldest->newest, in/out; NULL = zeros in, not written */
    int K;               /* d_conv, 1..8 (ignored when conv_w == NULL) */
    float* ssm_state;    /* [B, D, N] h0 in / h_T out; NULL = zeros in, not written */
    void* y;             /* [B*T, ld_y] output */
    long long ld_y;
    void* u_out;         /* optional [B*T, ld_u]: SiLU(conv(x)) for the x_proj GEMM */
    long long ld_u;
    float* chunk_states; /* optional training save: [B, ceil(T/save_stride), D, N], the state
                            ENTERING each block of save_stride steps (replaces h_saved) */
    int save_stride;     /* 32 or 64 when chunk_states != NULL; 32 is the backward's fast setting */
    void* workspace;     /* optional caller-owned scratch, 256-byte aligned, or NULL.  With it, a
                            launch whose batch x channels cannot fill the GPU is cut along the
                            sequence into up to 16 segments that run side by side (a first pass
                            for the segments' leaving states, an exact carry, then the full pass);
                            without it the sequence is always walked by one CTA per channel tile. */
    long long workspace_bytes; /* >= mamba_b200_sscan_fwd_workspace_bytes(B,T,D,N) uses every segment */
} mamba_b200_sscan_fwd_args;

MAMBA_B200_API long long mamba_b200_sscan_fwd_workspace_bytes(int B, int T, int D, int N);
MAMBA_B200_API int mamba_b200_sscan_fwd(void* handle, void* stream, const mamba_b200_sscan_fwd_args* args);

/*
 * Reference-compatible unfused entry point: same argument list and meaning as
 * ssm_parallel_scan_fwd_nosave_{f32,bf16,f16}
 * (kernels/mamba_ssm_parallel.cu:544-553, :969-980; launch
 * src/mamba_ssm/gpu/prefill.rs:913, forward.rs:940-958) and, equally, of
 * ssm_burnin_forward_nosave_{dt} (kernels/mamba_ssm.cu:304-400).
 *   h[B,D,N] f32 in/out, y_out[B,T,D], delta (already softplus'ed), u, B, C
 *   [B,T,N] contiguous, a_neg[D,N], D[D].
 */
MAMBA_B200_API int mamba_b200_ssm_scan_fwd_nosave(void* handle, void* stream, int dtype, float* h, void* y_out,
                                   const void* delta, const void* u, const void* B,
                                   const void* C, const float* a_neg, const float* D, int batch,
                                   int T, int d_inner, int d_state);

/*
 * The saving forward and the backward with the reference kernels' own buffers, for a
 * call-site swap without re-plumbing the trainer's activations:
 *   mamba_b200_ssm_scan_fwd_save : argument list of ssm_parallel_scan_fwd_{dt} /
 *       ssm_burnin_forward_{dt} (kernels/mamba_ssm_parallel.cu:265-276, :777-790,
 *       kernels/mamba_ssm.cu:232-246; launch src/mamba_ssm/gpu/forward_mixed.rs:632-702).
 *       h_saved is the reference's [batch, T+1, d_inner, d_state] f32 buffer; only its
 *       rows 0, 32, 64, ... (the states entering each 32-step block) are written, which is
 *       all mamba_b200_ssm_scan_bwd reads.  The reference's own backward kernels need
 *       every row: pair this forward with this backward, not with theirs.
 *   mamba_b200_ssm_scan_bwd : replaces ssm_parallel_scan_bwd_{dt} / ssm_backward_local_{dt}
 *       AND the four reducers ssm_reduce_d_{B,C,D,a_log} in one call
 *       (kernels/mamba_ssm_parallel.cu:1182-1200, kernels/mamba_ssm.cu:466-763; launch
 *       src/mamba_ssm/gpu/backward_mixed.rs:205-348).  Same inputs in the same order; the
 *       [B,T,D,N] d_B_local / d_C_local and the per-sample d_D_local / d_a_log_local
 *       partials do not exist here, so the outputs are the reducers' outputs:
 *       d_B, d_C [batch, T, d_state] f32 (overwritten), d_D [d_inner], d_a_log
 *       [d_inner, d_state] f32 (+=), plus a caller workspace of
 *       mamba_b200_sscan_bwd_workspace_bytes(batch, T, d_inner, d_state) bytes.
 *   mamba_b200_conv1d_fwd_nosave : argument list of conv1d_burnin_forward_nosave_{dt}
 *       (kernels/conv1d.cu:284-296; launch src/mamba_ssm/gpu/prefill.rs:788).
 * The saving conv forward and the conv backward have no such twin: the reference's pair
 * exchanges post_conv [B,T,D] and conv_states [B,T,D,K] (kernels/conv1d.cu:326-338,
 * :459-470), which this library never materialises; mamba_b200_conv1d_bwd takes x itself.
 */
MAMBA_B200_API int mamba_b200_ssm_scan_fwd_save(void* handle, void* stream, int dtype, float* h, void* y_out,
                                 float* h_saved, const void* delta, const void* u, const void* B,
                                 const void* C, const float* a_neg, const float* D, int batch, int T,
                                 int d_inner, int d_state);
MAMBA_B200_API int mamba_b200_ssm_scan_bwd(void* handle, void* stream, int dtype, const float* h_saved,
                            const void* delta, const void* u, const void* B, const void* C,
                            const float* a_neg, const float* D, const void* dy, void* d_delta, void* d_u,
                            float* d_B, float* d_C, float* d_D, float* d_a_log, int batch, int T, int d_inner,
                            int d_state, void* workspace, long long workspace_bytes);
MAMBA_B200_API int mamba_b200_conv1d_fwd_nosave(void* handle, void* stream, int dtype, void* u_out, float* state,
                                 const void* x_branch, const float* weight, const float* bias, int batch,
                                 int T, int d_inner, int d_conv);

/*
 * Mamba-1 fused backward (BPTT) by recomputation.  One call replaces, per layer,
 * gating_backward_{dt} (kernels/elementwise.cu:191-233), the B/C gather,
 * ssm_parallel_scan_bwd_{dt} / ssm_backward_local_{dt}
 * (kernels/mamba_ssm_parallel.cu:1182-1532, kernels/mamba_ssm.cu:466-662), the four
 * reducers ssm_reduce_d_{B,C,D,a_log} (kernels/mamba_ssm.cu:667-763) and
 * softplus_backward (kernels/activations.cu:68-104); launch sites
 * src/mamba_ssm/gpu/backward_mixed.rs:162-425.  It reads the block-boundary
 * states the training-mode forward saved (chunk_states) instead of h_saved
 * [B,(T+1),D,N] and never materialises the [B,T,D,N] dB/dC partials.
 *   overwritten: d_u, d_delta (w.r.t. the raw input when delta_softplus), d_z
 *                (storage dtype), dBm, dCm [B,T,N] f32
 *   accumulated (+=, grad-arena convention of backward_mixed.rs:331-347):
 *                dA_log [D,N], dD [D] f32
 * The conv1d backward is a separate entry point because the reference adds the
 * x_proj GEMM's input gradient to d_u in between (backward_mixed.rs:350-580).
 */
typedef struct mamba_b200_sscan_bwd_args {
    int dtype;
    int B, T, D, N;        /* N <= 256; N <= 16 (every shipped Mamba-1 model) takes the tuned kernels */
    const void* u;         /* [B*T, ld_u] scan input (post conv + SiLU) */
    long long ld_u;
    const void* delta;     /* as given to the forward */
    long long ld_delta;
    int delta_softplus;
    const void* Bm;
    const void* Cm;
    long long ld_bc;
    const void* z;
    long long ld_z;
    int z_mode;
    const float* a_neg;
    const float* Dp;
    const float* chunk_states; /* [B, ceil(T/save_stride), D, N] from the forward */
    int save_stride;           /* 32 or 64, as given to the forward; 32 is the native setting, a
                                  stride-64 save is first rebuilt to stride 32 (about 20 % slower) */
    const void* dy;            /* [B*T, ld_dy] gradient w.r.t. the forward output */
    long long ld_dy;
    void* d_u;
    long long ld_du;
    void* d_delta;
    long long ld_ddelta;
    void* d_z;                 /* required when z_mode != 0 */
    long long ld_dz;
    float* dBm;                /* [B*T, N] contiguous */
    float* dCm;
    float* dA_log;             /* [D, N], += */
    float* dD;                 /* [D], += */
    void* workspace;           /* caller-owned scratch, 256-byte aligned */
    long long workspace_bytes; /* >= mamba_b200_sscan_bwd_workspace_bytes(B,T,D,N) */
} mamba_b200_sscan_bwd_args;

MAMBA_B200_API long long mamba_b200_sscan_bwd_workspace_bytes(int B, int T, int D, int N);
MAMBA_B200_API int mamba_b200_sscan_bwd(void* handle, void* stream, const mamba_b200_sscan_bwd_args* args);

/*
 * Decode step (T = 1): conv step + SiLU, softplus(delta), SSM step, D skip and
 * gate in one launch.  Replaces conv1d_step_forward_silu_{dt}
 * (kernels/conv1d.cu:85-115), softplus_forward_{dt} and
 * ssm_step_forward_gather_gate_{dt} (kernels/mamba_ssm.cu:180-227); launch sites
 * src/mamba_ssm/gpu/inference.rs:1062-1215.  Rows are [B, ld]; B and C are
 * read in place from xdbl.  conv_state / ssm_state are updated in place.
 */
typedef struct mamba_b200_sscan_step_args {
    int dtype;
    int B, D, N;
    const void* x;        /* [B, ld_x]: pre-conv x when conv_w != NULL, else u */
    long long ld_x;
    const void* delta;    /* [B, ld_delta] */
    long long ld_delta;
    int delta_softplus;
    const void* Bm;       /* [B, ld_bc] */
    const void* Cm;
    long long ld_bc;
    const void* z;        /* [B, ld_z] or NULL */
    long long ld_z;
    int z_mode;           /* 0 none, 1 SiLU(z), 2 z is the ready gate */
    const float* a_neg;
    const float* Dp;
    const float* conv_w;  /* [D, K] or NULL */
    const float* conv_b;
    float* conv_state;    /* [B, D, K], required with conv_w */
    int K;
    float* ssm_state;     /* [B, D, N], required */
    void* y;              /* [B, ld_y] */
    long long ld_y;
    void* u_out;          /* optional [B, ld_u] */
    long long ld_u;
} mamba_b200_sscan_step_args;

MAMBA_B200_API int mamba_b200_sscan_step(void* handle, void* stream, const mamba_b200_sscan_step_args* args);

/*
 * Standalone depthwise causal conv1d + SiLU over a sequence, forward and
 * backward.  In the layer pipeline u must exist before the x_proj GEMM that
 * produces B, C and delta, so the conv runs as its own launch ahead of the scan.
 *   forward : replaces conv1d_burnin_forward[_nosave]_{dt} (kernels/conv1d.cu:161-359;
 *             src/mamba_ssm/gpu/forward_mixed.rs:500-537, prefill.rs:788); writes u and
 *             updates conv_state in place.  Nothing is saved for the backward.
 *   backward: replaces conv1d_burnin_backward_{dt} + two reduce_sum_axis0 launches
 *             (kernels/conv1d.cu:373-515, backward_mixed.rs:580-659); recomputes the
 *             pre-activation from x; d_x overwritten, dconv_w / dconv_b accumulated
 *             (+=) through per-(sample, time chunk) partials added in a fixed order.
 *             conv_state is the window that ENTERED the forward (NULL = zeros).
 */
typedef struct mamba_b200_conv1d_args {
    int dtype;
    int B, T, D, K;        /* K = d_conv, 1..8 */
    const void* x;         /* [B*T, ld_x] pre-conv x branch */
    long long ld_x;
    const float* conv_w;   /* [D, K] */
    const float* conv_b;   /* [D] */
    float* conv_state;     /* [B, D, K]; forward: in/out (NULL = zeros in, not written) */
    void* u;               /* forward output [B*T, ld_u] */
    long long ld_u;
    const void* d_u;       /* backward: gradient w.r.t. u [B*T, ld_du] */
    long long ld_du;
    void* d_x;             /* backward output [B*T, ld_dx] */
    long long ld_dx;
    float* dconv_w;        /* [D, K], += */
    float* dconv_b;        /* [D], += */
    void* workspace;       /* backward scratch */
    long long workspace_bytes; /* >= mamba_b200_conv1d_bwd_workspace_bytes(B,T,D,K) */
} mamba_b200_conv1d_args;

MAMBA_B200_API int mamba_b200_conv1d_fwd(void* handle, void* stream, const mamba_b200_conv1d_args* args);
MAMBA_B200_API long long mamba_b200_conv1d_bwd_workspace_bytes(int B, int T, int D, int K);
MAMBA_B200_API int mamba_b200_conv1d_bwd(void* handle, void* stream, const mamba_b200_conv1d_args* args);

/*
 * Mamba-3 SISO SSD scan (trapezoidal recurrence), forward.  Inputs are exactly
 * what the reference's chunked kernels consume: one call replaces
 * m3_preprocess_chunks, m3_dA_cumsum, m3_chunk_state_fwd, m3_state_passing_fwd,
 * m3_chunk_scan_fwd and m3_writeback_parallel_states
 * (kernels/mamba3_chunked.cu:57-419, :1050-1242; src/mamba3_siso/gpu/forward.rs:258-421),
 * and, with carry_in = 1, m3_burnin_fwd[_nosave] (kernels/mamba3_ssd.cu:229-546).
 *   x [B,T,nh*hd], K, Q [B,T,nh,N] (after bias + RoPE), y [B,T,nh*hd]: storage dtype
 *   dt (after softplus), trap (after sigmoid), adt = A*dt: [B,T,nh] f32; Dh [nh] f32
 *   ssm_state [B,nh,hd,N], k_state [B,nh,N], v_state [B,nh,hd] f32: written with
 *   the state after the window (NULL = not written); read first when carry_in = 1.
 * 16-bit storage with hd <= 64 and N <= 128 (multiples of 8; tiles are padded to
 * 64 / 128 columns with zeros inside the kernel, so the reference's own limits
 * hd 32, N 64 are covered) and no carried state runs the chunked form on tcgen05
 * tensor cores with the running state in TMEM (no chunk-state or K_scaled tensors
 * in HBM); every other case runs the sequential definition.
 * hd and N are not limited to the reference's hd <= 32, N <= 64
 * (src/mamba3_siso/config.rs:66-99); N <= 128.
 */
typedef struct mamba_b200_m3_ssd_args {
    int dtype;
    int B, T, nh, hd, N;
    const void* x;
    const void* K;
    const void* Q;
    const float* dt;
    const float* trap;
    const float* adt;
    const float* Dh;
    void* y;
    float* ssm_state;
    float* k_state;
    float* v_state;
    int carry_in;         /* 1: continue from the given state (sequential kernel) */
    int force_sequential; /* 1: never take the tensor-core path (for comparison) */
    /* Optional (Bn != NULL; tensor-core path only, else MAMBA_B200_ERR_SHAPE): the per-head
     * K and Q are built inside the kernel and K, Q above are ignored.  Replaces
     * bc_bias_add (kernels/mamba3_ops.cu:279-310), m3_angle_dt_fwd_seq (:400-440) and
     * rope_fwd (:575-640) and the two [B,T,nh,N] tensors they write
     * (src/mamba3_siso/cpu/forward.rs:336-375 is the definition):
     *   K[t,h,:] = rope(Bn[t,g,:] + b_bias[h,:], angle[t,h,:]), g = h / (nh / ng); Q from Cn, c_bias
     *   angle[t,h,a] = (angle_state[h,a] + sum_{s<=t} angle_vel[s,a] * dt[s,h]) mod 2 pi
     *   rope rotates the pairs (2a, 2a+1), a < n_angles; the other columns pass through.
     * Bn, Cn [B,T,ng,N] storage dtype (after BCNorm); b_bias, c_bias [nh,N] f32;
     * angle_vel [B,T,n_angles] f32 = tanh(angles_raw) * pi (the head-independent factor the
     * reference hoists, forward.rs:318-325); angle_state [B,nh,n_angles] f32, read and
     * overwritten with the angle after the window (NULL: zero in, not written).
     * n_angles a multiple of 4, 2 * n_angles <= N.  The in-chunk sums run in f32, the
     * angle entering each 128-step chunk is carried in f64. */
    const void* Bn;
    const void* Cn;
    const float* b_bias;
    const float* c_bias;
    const float* angle_vel;
    float* angle_state;
    int ng;
    int n_angles;
} mamba_b200_m3_ssd_args;

MAMBA_B200_API int mamba_b200_m3_ssd_fwd(void* handle, void* stream, const mamba_b200_m3_ssd_args* args);

/*
 * Mamba-3 SISO SSD scan, backward through a window that started from a zero
 * state.  One call replaces the scan part of the reference's backward:
 * m3_extract_da_cs_sum, m3_dqkv (with its dD reduce), and the d(dt), d(trap),
 * d(adt) terms that m3_ddt_dtrap / m3_final_grads derive from the scan
 * (kernels/mamba3_chunked.cu:439-1035; src/mamba3_siso/gpu/backward.rs:235-457);
 * same gradients as m3_ssd_backward_seq (kernels/mamba3_ssd.cu:558-808).
 * The states entering each 32-step chunk are recomputed into the workspace, so
 * the forward saves nothing.
 *   inputs as for the forward, plus dy [B,T,nh*hd] (storage dtype)
 *   dx [B,T,nh*hd] storage dtype (overwritten); dK, dQ [B,T,nh,N] f32 (overwritten)
 *   d_adt, d_dt, d_trap [B,T,nh] f32 (overwritten; d_dt is the direct path only,
 *   the caller adds A * d_adt as the reference does); dD [nh] f32, +=
 * hd <= 64, N <= 128.
 */
typedef struct mamba_b200_m3_ssd_bwd_args {
    int dtype;
    int B, T, nh, hd, N;
    const void* x;
    const void* K;
    const void* Q;
    const float* dt;
    const float* trap;
    const float* adt;
    const float* Dh;
    const void* dy;
    void* dx;
    float* dK;
    float* dQ;
    float* d_adt;
    float* d_dt;
    float* d_trap;
    float* dD;
    void* workspace;           /* 256-byte aligned */
    long long workspace_bytes; /* >= mamba_b200_m3_ssd_bwd_workspace_bytes(...) */
} mamba_b200_m3_ssd_bwd_args;

/* Upper bound over every dtype (the f32 CUDA-core kernel parks f32 states every 32
 * steps); _for(dtype, ...) is what a call with that storage dtype needs when its
 * tensors are 16-byte aligned: far less for the tensor-core geometry (16-bit, hd 64,
 * N 128: 16-bit state tiles every 128 steps). */
MAMBA_B200_API long long mamba_b200_m3_ssd_bwd_workspace_bytes(int B, int T, int nh, int hd, int N);
MAMBA_B200_API long long mamba_b200_m3_ssd_bwd_workspace_bytes_for(int dtype, int B, int T, int nh, int hd, int N);
MAMBA_B200_API int mamba_b200_m3_ssd_bwd(void* handle, void* stream, const mamba_b200_m3_ssd_bwd_args* args);

/*
 * conv1d backward for callers that cannot allocate: identical to
 * mamba_b200_conv1d_bwd, except that the partial-sum scratch is a fixed 16 MiB
 * array inside the library (workspace / workspace_bytes in `args` are ignored).
 * This entry point has no counterpart in the reference.
 *
 * It is meant for an engine that must not create device memory on this path:
 * one that handed all of its memory to an arena sized before this kernel's
 * scratch was known, or one that runs beside latency-critical streams, which a
 * cudaMalloc would stall because it synchronises the device (and which can
 * simply fail when another allocator owns the remaining memory).  The call
 * makes no cudaMalloc / cudaFree and calls no allocating library routine.
 *
 *   - Limit: B * ceil(T/64) * D * (K+1) * 4 bytes must not exceed
 *     mamba_b200_conv1d_bwd_static_max_bytes() (16 MiB); larger problems are
 *     refused with MAMBA_B200_ERR_SHAPE and a message, nothing is launched.
 *   - Every GPU that loads the library holds the 16 MiB until the process exits.
 *   - The first call on a device looks up the array's device address (with the
 *     caller's current device, which must be the one `stream` belongs to); make
 *     that first call before starting any stream capture.
 *   - All calls on a device share the array: two calls whose kernels can overlap
 *     on the GPU (different streams, no ordering) race.  Nothing needs clearing
 *     between calls; each call overwrites every partial it later reads.
 *   - `handle` may be NULL (failures are then reported by return code alone).
 */
MAMBA_B200_API long long mamba_b200_conv1d_bwd_static_max_bytes(void);
MAMBA_B200_API int mamba_b200_conv1d_bwd_static(void* handle, void* stream, const mamba_b200_conv1d_args* args);

/*
 * Residual add + RMSNorm in one pass, forward and backward.  Between two layers the
 * reference launches residual_add_f32_{dt} (kernels/elementwise.cu:367-377; f32
 * residual stream += the 16-bit out_proj output) and then rmsnorm_forward_f32in_{dt}
 * (kernels/norms.cu:126-168) on the stream it has just written
 * (src/mamba_ssm/gpu/forward_mixed.rs:433-480, :745-758).
 *   forward : residual [rows, dim] f32 += branch [rows, dim] (storage dtype; NULL = no
 *             add); y [rows, dim] (storage dtype) = residual / rms * scale; rms_out [rows]
 *             (NULL = not kept) is what the backward needs.  rms = sqrt(mean(x^2) + eps),
 *             replaced by 1 when it is not finite (the reference's guard).
 *   backward: replaces rmsnorm_backward_f32in_{dt} (kernels/norms.cu:323-367), the
 *             [rows, dim] d_scale partials and their reduce_sum_axis0, and the add of dx
 *             into the residual gradient: d_residual [rows, dim] f32 += dx;
 *             d_scale [dim] f32 += sum over rows (per-CTA partials in the workspace,
 *             added in CTA order: no atomics).  x is the residual the forward normalised.
 * dim <= 16384.
 */
MAMBA_B200_API int mamba_b200_residual_rmsnorm_fwd(void* handle, void* stream, int dtype, float* residual,
                                    const void* branch, const float* scale, void* y, float* rms_out,
                                    int rows, int dim, float eps);
MAMBA_B200_API long long mamba_b200_residual_rmsnorm_bwd_workspace_bytes(int rows, int dim);
MAMBA_B200_API int mamba_b200_residual_rmsnorm_bwd(void* handle, void* stream, int dtype, const void* dy,
                                    const float* x, const float* scale, const float* rms_saved,
                                    float* d_residual, float* d_scale, int rows, int dim, void* workspace,
                                    long long workspace_bytes);

/*
 * The ends of a training step on the device.  The reference trainer receives its input
 * rows and the output gradient from the host (src/mamba_ssm/gpu/trainer.rs:437-481) and
 * its language-model wrapper keeps a [vocab, d_model] table for both the embedding and
 * the tied head (src/module/gpu_lm.rs:560-679); these three launches have no kernel
 * counterpart there except AdamW.
 *   embedding_gather: out [rows, dim] f32 (the residual stream) = table[ids[r], :]
 *             (table in the storage dtype; an id outside [0, vocab) gives a zero row).
 *   softmax_xent    : per row of logits [rows, ld] (V used columns, storage dtype):
 *             loss_rows[r] = logsumexp(l) - l[target]; with d_logits != NULL also
 *             d_logits = (softmax(l) - onehot(target)) * grad_scale.  target < 0 marks a
 *             row that does not count (loss 0, zero gradient).  One read of the logits,
 *             one write of the gradient when a row fits shared memory (V * size <= 208 KB).
 *   adamw_step      : adamw_step_f32_capturable (kernels/adamw.cu:30-61; decoupled decay,
 *             bias_factors = {1/(1-beta1^t), 1/(1-beta2^t)} in a 2-float DEVICE buffer so the
 *             launch can sit in a captured graph) fused with the reference's separate
 *             master -> compute cast (trainer.rs:1453-1475): param_lp (f16 / bf16, may be
 *             NULL) receives the updated parameter in the compute dtype.
 */
MAMBA_B200_API int mamba_b200_embedding_gather(void* handle, void* stream, int dtype, const void* table,
                                const int* ids, float* out, long long rows, int dim, int vocab);
MAMBA_B200_API int mamba_b200_softmax_xent(void* handle, void* stream, int dtype, const void* logits,
                            const int* targets, float* loss_rows, void* dlogits, float grad_scale,
                            long long rows, int V, long long ld);
MAMBA_B200_API int mamba_b200_adamw_step(void* handle, void* stream, float* param, const float* grad, float* m,
                          float* v, float lr, float beta1, float beta2, float eps, float weight_decay,
                          const float* bias_factors, void* param_lp, int lp_dtype, long long n);

#ifdef __cplusplus
}
#endif
#endif /* MAMBA_B200_H */
