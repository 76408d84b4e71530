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
 *     (a CUstream / cudaStream_t passed as void*) and are graph-capturable;
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
    int save_stride;     /* multiple of 64 when chunk_states != NULL */
} mamba_b200_sscan_fwd_args;

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

#ifdef __cplusplus
}
#endif
#endif /* MAMBA_B200_H */
