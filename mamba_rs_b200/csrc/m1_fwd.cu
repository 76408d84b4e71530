// Mamba-1 fused selective-scan forward for sm_100a.
// Host side of the fused forward: argument validation, TMA descriptors, variant
// selection and launch.  The kernels live in m1_fwd_kernel.cuh.
#include <stdlib.h>

#include "m1_fwd_kernel.cuh"

namespace mb200 {

struct FwdTable {
    FwdVariant v[3][kMaxFwdVariants];
    int n[3];
};

static const FwdTable& fwd_table() {
    static FwdTable t;
    static bool init = false;
    if (!init) {
        memset(&t, 0, sizeof(t));
#ifndef MB200_FWD_BF16_ONLY
        t.n[MAMBA_B200_F32] = fwd_variants_f32(t.v[MAMBA_B200_F32]);
        t.n[MAMBA_B200_F16] = fwd_variants_f16(t.v[MAMBA_B200_F16]);
#endif
        t.n[MAMBA_B200_BF16] = fwd_variants_bf16(t.v[MAMBA_B200_BF16]);
        init = true;
    }
    return t;
}

int m1_fwd_configure(Ctx* c) {
    const FwdTable& t = fwd_table();
    for (int dt = 0; dt < 3; ++dt)
        for (int i = 0; i < t.n[dt]; ++i)
            for (int f = 0; f < 8; ++f)
                if (t.v[dt][i].fn[f] && t.v[dt][i].smem <= 227 * 1024)
                    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(
                                            reinterpret_cast<const void*>(t.v[dt][i].fn[f]),
                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(t.v[dt][i].smem)));
    return MAMBA_B200_OK;
}

static int launch_fwd(Ctx* c, cudaStream_t stream, const mamba_b200_sscan_fwd_args& a) {
    if (!dtype_ok(a.dtype)) return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: bad dtype %d", a.dtype);
    if (a.B < 0 || a.T < 0 || a.D <= 0 || a.N <= 0)
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: bad dims B=%d T=%d D=%d N=%d", a.B, a.T, a.D, a.N);
    if (a.N > 256) return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_fwd: d_state %d > 256", a.N);
    if (a.B == 0 || a.T == 0) return MAMBA_B200_OK;
    if (a.B > 65535) return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_fwd: batch %d > 65535", a.B);
    if (!a.x || !a.delta || !a.Bm || !a.Cm || !a.a_neg || !a.Dp || !a.y)
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: null required pointer");
    if (a.z_mode < 0 || a.z_mode > 2 || (a.z_mode && !a.z))
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: z_mode %d with z=%p", a.z_mode, a.z);
    if (a.conv_w && (!a.conv_b || a.K < 1 || a.K > kKMax))
        return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_fwd: d_conv %d outside 1..%d or null bias", a.K, kKMax);
    if (a.ld_x < a.D || a.ld_delta < a.D || a.ld_y < a.D || a.ld_bc < a.N ||
        (a.z_mode && a.ld_z < a.D) || (a.u_out && a.ld_u < a.D))
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: a row stride is smaller than its row");
    const size_t es = dtype_size(a.dtype);
    auto misaligned = [&](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) % es) != 0; };
    if (misaligned(a.x) || misaligned(a.delta) || misaligned(a.Bm) || misaligned(a.Cm) ||
        misaligned(a.y) || (a.z && misaligned(a.z)) || (a.u_out && misaligned(a.u_out)))
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: pointer not aligned to its element size");

    const FwdTable& tab = fwd_table();
    const FwdVariant* vs = tab.v[a.dtype];
    const FwdVariant* v = nullptr;
    for (int i = 0; i < tab.n[a.dtype]; ++i)
        if (vs[i].ns * vs[i].lpc >= a.N) { v = &vs[i]; break; }
    if (!v) return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_fwd: no variant for d_state %d", a.N);
    if (a.chunk_states && (a.save_stride <= 0 || a.save_stride % v->tc != 0 || a.save_stride > 64))
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: save_stride %d must be 32 or 64", a.save_stride);

    FwdParams p;
    memset(&p, 0, sizeof(p));
    p.x = a.x; p.dl = a.delta; p.z = a.z_mode ? a.z : nullptr; p.bm = a.Bm; p.cm = a.Cm;
    p.y = a.y; p.u_out = a.conv_w ? a.u_out : nullptr;
    p.ld_x = a.ld_x; p.ld_dl = a.ld_delta; p.ld_z = a.ld_z; p.ld_bc = a.ld_bc; p.ld_y = a.ld_y;
    p.ld_u = a.ld_u;
    p.a_neg = a.a_neg; p.Dp = a.Dp; p.conv_w = a.conv_w; p.conv_b = a.conv_b;
    p.conv_state = a.conv_w ? a.conv_state : nullptr;
    p.ssm_state = a.ssm_state; p.chunk_states = a.chunk_states;
    p.B = a.B; p.T = a.T; p.D = a.D; p.N = a.N; p.K = a.conv_w ? a.K : 0;
    p.delta_softplus = a.delta_softplus; p.z_mode = a.z_mode;
    p.save_stride = a.chunk_states ? a.save_stride : 1;
    p.status = c->d_status;
    p.u_vec = (a.u_out && (a.ld_u % 2 == 0) && (reinterpret_cast<uintptr_t>(a.u_out) % (2 * es) == 0)) ? 1 : 0;
    unsigned m = 0;
    // The y tile must not alias rows of other tensors the same CTA still reads
    // through TMA; in-place use (y == x) is served by the plain-store path.
    if (make_tmap_3d(c, &p.tm_x, a.dtype, a.x, a.ld_x, a.D, a.T, a.B, v->dt, v->tc)) m |= kTmaX;
    if (make_tmap_3d(c, &p.tm_dl, a.dtype, a.delta, a.ld_delta, a.D, a.T, a.B, v->dt, v->tc)) m |= kTmaDl;
    if (a.z_mode && make_tmap_3d(c, &p.tm_z, a.dtype, a.z, a.ld_z, a.D, a.T, a.B, v->dt, v->tc)) m |= kTmaZ;
    if (!a.z_mode) m |= kTmaZ;  // nothing to load
    if (make_tmap_3d(c, &p.tm_b, a.dtype, a.Bm, a.ld_bc, a.N, a.T, a.B, a.N, v->tc)) m |= kTmaB;
    if (make_tmap_3d(c, &p.tm_c, a.dtype, a.Cm, a.ld_bc, a.N, a.T, a.B, a.N, v->tc)) m |= kTmaC;
    if (make_tmap_3d(c, &p.tm_y, a.dtype, a.y, a.ld_y, a.D, a.T, a.B, v->dt, v->tc)) m |= kTmaY;
    p.tma_mask = m;

    const int flags = (a.delta_softplus ? 1 : 0) | (a.z_mode ? 2 : 0) | (a.conv_w ? 4 : 0);
    FwdKernelFn fn = v->fn[flags];
    if (!fn || v->smem > 227 * 1024)
        return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_fwd: no kernel for dtype %d flags %d d_state %d",
                    a.dtype, flags, a.N);
    // Time segments: when batch x channel tiles cannot even give every warp
    // scheduler one warp (small-batch prefill), split the sequence; each extra
    // segment replays the earlier ones for its entering state (about half the
    // cost of a full chunk), so at most 3 segments.  Measured on B200: no gain
    // once the schedulers hold 2-3 warps each (the kernel is then bound by
    // instruction throughput, and replay only adds instructions).
    const long long tiles = static_cast<long long>((a.D + v->dt - 1) / v->dt) * a.B;
    const long long warps = tiles * (v->threads / 32);
    const int nchunks = (a.T + v->tc - 1) / v->tc;
    int segs = 1;
    const char* env = getenv("MAMBA_B200_FWD_SEGMENTS");
    if (env && atoi(env) > 0) segs = atoi(env);
    else {
        const long long want = 4ll * c->sm_count;  // one warp per scheduler at least
        while (segs < 3 && warps * segs < want && nchunks >= 8 * (segs + 1)) ++segs;
    }
    if (segs > nchunks) segs = nchunks > 0 ? nchunks : 1;
    p.seg_chunks = segs > 1 ? (nchunks + segs - 1) / segs : 0;
    if (segs > 1) segs = (nchunks + p.seg_chunks - 1) / p.seg_chunks;
    dim3 grid((a.D + v->dt - 1) / v->dt, a.B, segs);
    fn<<<grid, v->threads, v->smem, stream>>>(p);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}

}  // namespace mb200

using namespace mb200;

extern "C" MAMBA_B200_API int mamba_b200_sscan_fwd(void* handle, void* stream, const mamba_b200_sscan_fwd_args* args) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!args) return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: null args");
    return launch_fwd(c, static_cast<cudaStream_t>(stream), *args);
}

extern "C" MAMBA_B200_API int mamba_b200_ssm_scan_fwd_nosave(void* handle, void* stream, int dtype, float* h,
                                              void* y_out, const void* delta, const void* u,
                                              const void* B, const void* C, const float* a_neg,
                                              const float* D, int batch, int T, int d_inner,
                                              int d_state) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    mamba_b200_sscan_fwd_args a;
    memset(&a, 0, sizeof(a));
    a.dtype = dtype; a.B = batch; a.T = T; a.D = d_inner; a.N = d_state;
    a.x = u; a.ld_x = d_inner; a.delta = delta; a.ld_delta = d_inner; a.delta_softplus = 0;
    a.Bm = B; a.Cm = C; a.ld_bc = d_state; a.z_mode = 0;
    a.a_neg = a_neg; a.Dp = D; a.ssm_state = h; a.y = y_out; a.ld_y = d_inner;
    return launch_fwd(c, static_cast<cudaStream_t>(stream), a);
}
