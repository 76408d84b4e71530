// Mamba-1 fused selective-scan forward for sm_100a.
// Host side of the fused forward: argument validation, TMA descriptors, variant
// selection, the time-segment plan and launch.  The kernels live in
// m1_fwd_kernel.cuh.
#include "m1_fwd_kernel.cuh"

namespace mb200 {

constexpr int kMaxSegments = 16;

struct FwdTable {
    FwdVariant v[3][kMaxFwdVariants];
    int n[3];
};

// Built once, under the thread-safe initialisation of a function-local static.
static const FwdTable& fwd_table() {
    static const FwdTable table = [] {
        FwdTable t;
        memset(&t, 0, sizeof(t));
        t.n[MAMBA_B200_F32] = fwd_variants_f32(t.v[MAMBA_B200_F32]);
        t.n[MAMBA_B200_F16] = fwd_variants_f16(t.v[MAMBA_B200_F16]);
        t.n[MAMBA_B200_BF16] = fwd_variants_bf16(t.v[MAMBA_B200_BF16]);
        return t;
    }();
    return table;
}

int m1_fwd_configure(Ctx* c) {
    const FwdTable& t = fwd_table();
    for (int dt = 0; dt < 3; ++dt)
        for (int i = 0; i < t.n[dt]; ++i)
            for (int f = 0; f < 16; ++f)
                if (t.v[dt][i].fn[f] && t.v[dt][i].smem <= 227 * 1024)
                    MB200_CUDA_CHECK(c, cudaFuncSetAttribute(
                                            reinterpret_cast<const void*>(t.v[dt][i].fn[f]),
                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(t.v[dt][i].smem)));
    return MAMBA_B200_OK;
}

// Segment hand-over: slot s of seg_states arrives holding the state segment s
// leaves when started from zero (segment 0: from the real entering state) and
// leaves holding the true state at the end of segment s, i.e. the one segment
// s + 1 starts from.  A segment's decay is exp(a * sum of its deltas): the carry
// costs one exp2 per state and segment.
__global__ void sscan_seg_carry_kernel(float* seg_states, const float* seg_sumdl, const float* a_neg,
                                       int B, int S, int D, int N) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= static_cast<long long>(B) * D * N) return;
    const int n = static_cast<int>(i % N);
    const int d = static_cast<int>((i / N) % D);
    const int b = static_cast<int>(i / (static_cast<long long>(N) * D));
    const float a2 = a_neg[static_cast<long long>(d) * N + n] * kLog2e;
    float run = seg_states[((static_cast<long long>(b) * S + 0) * D + d) * N + n];
    for (int s = 1; s + 1 < S; ++s) {
        const long long at = ((static_cast<long long>(b) * S + s) * D + d) * N + n;
        const float sum = seg_sumdl[(static_cast<long long>(b) * S + s) * D + d];
        run = fmaf(ex2(a2 * sum), run, seg_states[at]);
        seg_states[at] = run;
    }
}

static size_t fwd_ws_bytes(int B, int D, int N, int segs, size_t* o_sum, size_t* o_h0, size_t* o_c0) {
    auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
    size_t off = al(sizeof(float) * static_cast<size_t>(B) * segs * D * N);
    *o_sum = off;
    off += al(sizeof(float) * static_cast<size_t>(B) * segs * D);
    *o_h0 = off;
    off += al(sizeof(float) * static_cast<size_t>(B) * D * N);
    *o_c0 = off;
    off += al(sizeof(float) * static_cast<size_t>(B) * D * kKMax);
    return off;
}

static bool overlaps(const void* a, size_t na, const void* b, size_t nb) {
    const uintptr_t x = reinterpret_cast<uintptr_t>(a), y = reinterpret_cast<uintptr_t>(b);
    return a && b && x < y + nb && y < x + na;
}

static int launch_fwd(Ctx* c, cudaStream_t stream, const mamba_b200_sscan_fwd_args& a, long long cs_ld_b = 0,
                      long long cs_ld_k = 0) {
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
    // With the conv fused, a chunk re-reads the rows of x just before it: y (or u_out)
    // written over x would be read back as input.
    const size_t span_x = (static_cast<size_t>(a.B) * a.T - 1) * a.ld_x * es + a.D * es;
    if (a.conv_w && (overlaps(a.x, span_x, a.y, (static_cast<size_t>(a.B) * a.T - 1) * a.ld_y * es + a.D * es) ||
                     (a.u_out && overlaps(a.x, span_x, a.u_out,
                                          (static_cast<size_t>(a.B) * a.T - 1) * a.ld_u * es + a.D * es))))
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: with the conv fused, y and u_out must not overlap x");

    const FwdTable& tab = fwd_table();
    const FwdVariant* vs = tab.v[a.dtype];
    const FwdVariant* v = nullptr;
    for (int i = 0; i < tab.n[a.dtype]; ++i)
        if (vs[i].ns * vs[i].lpc >= a.N) { v = &vs[i]; break; }
    if (!v) return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_fwd: no variant for d_state %d", a.N);
    if (a.chunk_states && (a.save_stride <= 0 || a.save_stride % 32 != 0 || a.save_stride > 64))
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
    p.conv_in = p.conv_state; p.ssm_in = p.ssm_state;
    p.B = a.B; p.T = a.T; p.D = a.D; p.N = a.N; p.K = a.conv_w ? a.K : 0;
    p.z_mode = a.z_mode;
    p.save_stride = a.chunk_states ? a.save_stride : 1;
    if (a.chunk_states) {  // default: dense [B, ceil(T / stride), D, N]
        p.cs_ld_k = cs_ld_k ? cs_ld_k : static_cast<long long>(a.D) * a.N;
        p.cs_ld_b = cs_ld_b ? cs_ld_b : p.cs_ld_k * ((a.T + a.save_stride - 1) / a.save_stride);
    }
    p.status = c->d_status;
    unsigned m = 0;
    const int xrows = a.conv_w ? v->tc + kHaloRows : v->tc;
    if (make_tmap_3d(c, &p.tm_x, a.dtype, a.x, a.ld_x, a.D, a.T, a.B, v->dt, xrows)) m |= kTmaX;
    if (make_tmap_3d(c, &p.tm_dl, a.dtype, a.delta, a.ld_delta, a.D, a.T, a.B, v->dt, v->tc)) m |= kTmaDl;
    if (a.z_mode && make_tmap_3d(c, &p.tm_z, a.dtype, a.z, a.ld_z, a.D, a.T, a.B, v->dt, v->tc)) m |= kTmaZ;
    if (make_tmap_3d(c, &p.tm_b, a.dtype, a.Bm, a.ld_bc, a.N, a.T, a.B, a.N, v->tc)) m |= kTmaB;
    if (make_tmap_3d(c, &p.tm_c, a.dtype, a.Cm, a.ld_bc, a.N, a.T, a.B, a.N, v->tc)) m |= kTmaC;
    p.tma_mask = m;

    const int flags = (a.delta_softplus ? 1 : 0) | (a.z_mode ? 2 : 0) | (a.conv_w ? 4 : 0);
    FwdKernelFn fn = v->fn[flags];
    FwdKernelFn fn_state = v->fn[8 | (flags & 5)];
    if (!fn || !fn_state || v->smem > 227 * 1024)
        return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_fwd: no kernel for dtype %d flags %d d_state %d",
                    a.dtype, flags, a.N);

    // Time segments.  When batch x channel tiles leave warp schedulers idle
    // (small-batch prefill) and the caller lent a workspace, the sequence is cut
    // into S segments that run side by side: a first launch walks segments
    // 0 .. S-2 for their leaving states only (segment s > 0 from a zero state,
    // keeping the sum of its deltas), a small kernel chains them into the true
    // entering states, and the second launch runs every segment in full.
    const int tiles = (a.D + v->dt - 1) / v->dt;
    const long long warps = static_cast<long long>(tiles) * a.B * (v->threads / 32 - 1);
    const int nchunks = (a.T + v->tc - 1) / v->tc;
    int segs = 1;
    if (a.workspace && a.workspace_bytes > 0) {
        const long long want = 8ll * c->sm_count;  // two warps per scheduler
        while (segs < kMaxSegments && warps * segs < want && nchunks / (segs * 2) >= 4) segs *= 2;
        size_t o1, o2, o3;
        while (segs > 1 && fwd_ws_bytes(a.B, a.D, a.N, segs, &o1, &o2, &o3) > static_cast<size_t>(a.workspace_bytes))
            segs /= 2;
        if (segs > 1 && reinterpret_cast<uintptr_t>(a.workspace) % 256)
            return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: workspace must be 256-byte aligned");
    }
    dim3 grid(tiles, a.B, 1);
    if (segs > 1) {
        p.seg_chunks = (nchunks + segs - 1) / segs;
        segs = (nchunks + p.seg_chunks - 1) / p.seg_chunks;
    }
    if (segs > 1) {
        size_t o_sum, o_h0, o_c0;
        fwd_ws_bytes(a.B, a.D, a.N, segs, &o_sum, &o_h0, &o_c0);
        unsigned char* ws = static_cast<unsigned char*>(a.workspace);
        p.seg_states = reinterpret_cast<float*>(ws);
        p.seg_sumdl = reinterpret_cast<float*>(ws + o_sum);
        grid.z = segs;
        FwdParams p1 = p;  // state-only pass: also keeps the entering states for the second pass
        p1.ssm_copy = reinterpret_cast<float*>(ws + o_h0);
        p1.conv_copy = p.K ? reinterpret_cast<float*>(ws + o_c0) : nullptr;
        fn_state<<<grid, v->threads, v->smem, stream>>>(p1);
        MB200_CUDA_CHECK(c, cudaGetLastError());
        const long long n = static_cast<long long>(a.B) * a.D * a.N;
        sscan_seg_carry_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
            p.seg_states, p.seg_sumdl, a.a_neg, a.B, segs, a.D, a.N);
        MB200_CUDA_CHECK(c, cudaGetLastError());
        // segment 0 of the second pass reads the copies: the last segment overwrites the
        // caller's state arrays while other segments may still be starting
        p.ssm_in = p1.ssm_copy;
        p.conv_in = p1.conv_copy;
    }
    fn<<<grid, v->threads, v->smem, stream>>>(p);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}

}  // namespace mb200

using namespace mb200;

extern "C" MAMBA_B200_API long long mamba_b200_sscan_fwd_workspace_bytes(int B, int T, int D, int N) {
    (void)T;
    if (B <= 0 || D <= 0 || N <= 0 || N > 256) return 0;
    size_t o1, o2, o3;
    return static_cast<long long>(fwd_ws_bytes(B, D, N, kMaxSegments, &o1, &o2, &o3));
}

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

extern "C" MAMBA_B200_API int mamba_b200_ssm_scan_fwd_save(void* handle, void* stream, int dtype, float* h,
                                                           void* y_out, float* h_saved, const void* delta,
                                                           const void* u, const void* B, const void* C,
                                                           const float* a_neg, const float* D, int batch, int T,
                                                           int d_inner, int d_state) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!h_saved) return fail(c, MAMBA_B200_ERR_ARG, "ssm_scan_fwd_save: null h_saved");
    mamba_b200_sscan_fwd_args a;
    memset(&a, 0, sizeof(a));
    a.dtype = dtype; a.B = batch; a.T = T; a.D = d_inner; a.N = d_state;
    a.x = u; a.ld_x = d_inner; a.delta = delta; a.ld_delta = d_inner; a.delta_softplus = 0;
    a.Bm = B; a.Cm = C; a.ld_bc = d_state; a.z_mode = 0;
    a.a_neg = a_neg; a.Dp = D; a.ssm_state = h; a.y = y_out; a.ld_y = d_inner;
    // rows 0, 32, 64, ... of h_saved [batch, T+1, d_inner, d_state]
    a.chunk_states = h_saved; a.save_stride = 32;
    const long long row = static_cast<long long>(d_inner) * d_state;
    return launch_fwd(c, static_cast<cudaStream_t>(stream), a, row * (static_cast<long long>(T) + 1), 32 * row);
}
