// Mamba-1 fused selective-scan forward for sm_100a.
//
// One CTA owns (sample b, a tile of DT channels) and walks the sequence in
// chunks of TC steps.  Per chunk:
//   load   : TMA (cp.async.bulk.tensor.3d) brings the x / delta / z / B / C tiles
//            of chunk c+1 into the other shared-memory stage while chunk c runs;
//   stage 1: every thread, mapped over (t, channel pair): conv1d + SiLU,
//            softplus(delta), SiLU(z), D skip -> f32 staging in shared memory;
//   stage 2: thread = (group of CH channels, slice of NS states): the
//            recurrence h = exp(delta*a)*h + delta*u*B, y = <h, C>, with h in
//            registers and packed f32x2 arithmetic, reduced over the LPC lanes
//            that share a channel; the lane with slice 0 applies gate and skip
//            and writes the output tile;
//   store  : TMA store of the y tile (clipped at T and D).
// HBM is touched once per input and once per output element.
#include <string.h>

#include <type_traits>

#include "common.cuh"
#include "internal.h"

namespace mb200 {

constexpr int kKMax = 8;  // widest supported d_conv

struct FwdParams {
    CUtensorMap tm_x, tm_dl, tm_z, tm_b, tm_c, tm_y;
    const void *x, *dl, *z, *bm, *cm;
    void *y, *u_out;
    long long ld_x, ld_dl, ld_z, ld_bc, ld_y, ld_u;
    const float *a_neg, *Dp, *conv_w, *conv_b;
    float *conv_state, *ssm_state, *chunk_states;
    int B, T, D, N, K;
    int delta_softplus, z_mode, save_stride;
    int u_vec;          // u_out rows allow paired stores
    unsigned tma_mask;  // bit0 x, bit1 delta, bit2 z, bit3 B, bit4 C, bit5 y
    int* status;
};

enum : unsigned { kTmaX = 1, kTmaDl = 2, kTmaZ = 4, kTmaB = 8, kTmaC = 16, kTmaY = 32 };

template <typename Tact, int CH_, int NS_, int LPC_, int WARPS_, int TC_>
struct FwdTraits {
    static constexpr int CH = CH_, NS = NS_, LPC = LPC_, WARPS = WARPS_, TC = TC_;
    static constexpr int THREADS = WARPS * 32;
    static constexpr int G = THREADS / LPC;  // channel groups per CTA
    static constexpr int DT = G * CH;        // channels per CTA
    static constexpr int NP = NS * LPC;      // padded d_state
    static constexpr size_t al(size_t v) { return (v + 127) & ~size_t(127); }
    static constexpr size_t RAW_ACT = al(sizeof(Tact) * TC * DT);
    static constexpr size_t RAW_BC = al(sizeof(Tact) * TC * NP);
    static constexpr size_t STAGE = 3 * RAW_ACT + 2 * RAW_BC;
    static constexpr size_t OFF_RAW = 0;
    static constexpr size_t OFF_A1 = OFF_RAW + 2 * STAGE;                     // float2 (delta, du)
    static constexpr size_t OFF_A2 = OFF_A1 + al(sizeof(float2) * TC * DT);   // float2 (gate, skip)
    static constexpr size_t OFF_BS = OFF_A2 + al(sizeof(float2) * TC * DT);   // f32 B [TC][NP]
    static constexpr size_t OFF_CS = OFF_BS + al(sizeof(float) * TC * NP);    // f32 C [TC][NP]
    static constexpr size_t OFF_OUT = OFF_CS + al(sizeof(float) * TC * NP);   // Tact y [TC][DT]
    static constexpr size_t OFF_HALO = OFF_OUT + RAW_ACT;                     // f32 [kKMax][DT]
    static constexpr size_t OFF_CW = OFF_HALO + al(sizeof(float) * kKMax * DT);  // f32 [kKMax][DT]
    static constexpr size_t OFF_CB = OFF_CW + al(sizeof(float) * kKMax * DT);    // f32 [DT]
    static constexpr size_t OFF_DP = OFF_CB + al(sizeof(float) * DT);            // f32 [DT]
    static constexpr size_t OFF_BAR = OFF_DP + al(sizeof(float) * DT);           // 2 mbarriers
    static constexpr size_t SMEM = OFF_BAR + 128;
    static_assert(DT % 2 == 0, "channel tile must be even");
    static_assert(NS % 4 == 0, "state slice must be a multiple of 4");
    static_assert((LPC & (LPC - 1)) == 0 && LPC <= 32, "LPC must be a power of two");
};

// Plain-load path for one tile (used when a tensor breaks a TMA layout rule).
template <typename Tact>
__device__ __forceinline__ void load_tile_plain(Tact* dst, const Tact* src, long long ld, int b,
                                                int T, int t0, int c0, int cols, int rows,
                                                int box_cols, int nthreads) {
    const Tact zero = from_f<Tact>(0.0f);
    for (int i = threadIdx.x; i < rows * box_cols; i += nthreads) {
        int r = i / box_cols, c = i - r * box_cols;
        int t = t0 + r, col = c0 + c;
        Tact v = zero;
        if (t < T && col < cols) v = src[(static_cast<long long>(b) * T + t) * ld + col];
        dst[i] = v;
    }
}

template <typename Tr, typename Tact>
__global__ void __launch_bounds__(Tr::THREADS)
sscan_fwd_kernel(const __grid_constant__ FwdParams p) {
    constexpr int CH = Tr::CH, NS = Tr::NS, LPC = Tr::LPC, TC = Tr::TC, DT = Tr::DT, NP = Tr::NP,
                  G = Tr::G, THREADS = Tr::THREADS;
    extern __shared__ __align__(128) unsigned char smem[];
    float2* A1 = reinterpret_cast<float2*>(smem + Tr::OFF_A1);
    float2* A2 = reinterpret_cast<float2*>(smem + Tr::OFF_A2);
    float* Bs = reinterpret_cast<float*>(smem + Tr::OFF_BS);
    float* Cs = reinterpret_cast<float*>(smem + Tr::OFF_CS);
    Tact* out_t = reinterpret_cast<Tact*>(smem + Tr::OFF_OUT);
    float* halo = reinterpret_cast<float*>(smem + Tr::OFF_HALO);
    float* cw_s = reinterpret_cast<float*>(smem + Tr::OFF_CW);
    float* cb_s = reinterpret_cast<float*>(smem + Tr::OFF_CB);
    float* dp_s = reinterpret_cast<float*>(smem + Tr::OFF_DP);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Tr::OFF_BAR);

    const int tid = threadIdx.x;
    const int b = blockIdx.y;
    const int d0 = blockIdx.x * DT;
    const int T = p.T, D = p.D, N = p.N, K = p.conv_w ? p.K : 0;
    const int nchunks = (T + TC - 1) / TC;
    const unsigned load_mask = p.tma_mask & (kTmaX | kTmaDl | kTmaZ | kTmaB | kTmaC);
    const bool has_z = p.z_mode != 0;

    auto raw_x = [&](int s) { return reinterpret_cast<Tact*>(smem + Tr::OFF_RAW + s * Tr::STAGE); };
    auto raw_dl = [&](int s) {
        return reinterpret_cast<Tact*>(smem + Tr::OFF_RAW + s * Tr::STAGE + Tr::RAW_ACT);
    };
    auto raw_z = [&](int s) {
        return reinterpret_cast<Tact*>(smem + Tr::OFF_RAW + s * Tr::STAGE + 2 * Tr::RAW_ACT);
    };
    auto raw_b = [&](int s) {
        return reinterpret_cast<Tact*>(smem + Tr::OFF_RAW + s * Tr::STAGE + 3 * Tr::RAW_ACT);
    };
    auto raw_c = [&](int s) {
        return reinterpret_cast<Tact*>(smem + Tr::OFF_RAW + s * Tr::STAGE + 3 * Tr::RAW_ACT +
                                       Tr::RAW_BC);
    };

    // Bytes one stage receives through TMA (full boxes: out-of-range parts are
    // zero-filled and still counted).
    uint32_t tx_bytes = 0;
    if (load_mask & kTmaX) tx_bytes += sizeof(Tact) * TC * DT;
    if (load_mask & kTmaDl) tx_bytes += sizeof(Tact) * TC * DT;
    if (has_z && (load_mask & kTmaZ)) tx_bytes += sizeof(Tact) * TC * DT;
    if (load_mask & kTmaB) tx_bytes += sizeof(Tact) * TC * N;
    if (load_mask & kTmaC) tx_bytes += sizeof(Tact) * TC * N;

    auto issue_loads = [&](int c) {  // one thread
        const int s = c & 1, t0 = c * TC;
        if (tx_bytes == 0) return;
        mbar_expect_tx(&bars[s], tx_bytes);
        if (load_mask & kTmaX) tma_load_3d(raw_x(s), &p.tm_x, &bars[s], d0, t0, b);
        if (load_mask & kTmaDl) tma_load_3d(raw_dl(s), &p.tm_dl, &bars[s], d0, t0, b);
        if (has_z && (load_mask & kTmaZ)) tma_load_3d(raw_z(s), &p.tm_z, &bars[s], d0, t0, b);
        if (load_mask & kTmaB) tma_load_3d(raw_b(s), &p.tm_b, &bars[s], 0, t0, b);
        if (load_mask & kTmaC) tma_load_3d(raw_c(s), &p.tm_c, &bars[s], 0, t0, b);
    };

    if (tid == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        fence_barrier_init();
    }
    // Per-channel constants of the tile and the entering conv window.
    for (int i = tid; i < DT; i += THREADS) {
        int d = d0 + i;
        dp_s[i] = d < D ? p.Dp[d] : 0.0f;
        cb_s[i] = (K && d < D) ? p.conv_b[d] : 0.0f;
        for (int k = 0; k < kKMax; ++k) {
            cw_s[k * DT + i] = (k < K && d < D) ? p.conv_w[static_cast<long long>(d) * K + k] : 0.0f;
            float hv = 0.0f;
            if (k < K && d < D && p.conv_state)
                hv = p.conv_state[(static_cast<long long>(b) * D + d) * K + k];
            halo[k * DT + i] = hv;
        }
    }
    __syncthreads();
    if (tid == 0 && nchunks > 0) issue_loads(0);

    // ---- stage-2 ownership: CH channels x NS states per thread ----
    const int grp = tid / LPC, part = tid % LPC;
    const int n0 = part * NS;
    float2 h[CH][NS / 2];
    float2 a2[CH][NS / 2];  // a_neg * log2(e)
    bool geo_local = true;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int d = d0 + grp * CH + c;
        float av[NS], hv[NS];
#pragma unroll
        for (int j = 0; j < NS; ++j) {
            const int n = n0 + j;
            const bool ok = d < D && n < N;
            av[j] = ok ? p.a_neg[static_cast<long long>(d) * N + n] * kLog2e : 0.0f;
            hv[j] = (ok && p.ssm_state) ? p.ssm_state[(static_cast<long long>(b) * D + d) * N + n]
                                        : 0.0f;
        }
        // Arithmetic-progression test a[n] = a[n0] + (n-n0)*step, to 4 ulp: then
        // exp(delta*a[n]) = E * R^(n-n0) needs two exp2 per step instead of NS.
        const float step = av[1] - av[0];
#pragma unroll
        for (int j = 2; j < NS; ++j) {
            const float pred = fmaf(static_cast<float>(j), step, av[0]);
            if (fabsf(av[j] - pred) > 4.8e-7f * fabsf(av[j])) geo_local = false;
        }
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) {
            a2[c][j] = make_float2(av[2 * j], av[2 * j + 1]);
            h[c][j] = make_float2(hv[2 * j], hv[2 * j + 1]);
        }
    }
    const bool geo = __syncthreads_and(geo_local ? 1 : 0) != 0;

    const long long save_chunks = p.chunk_states ? (T + p.save_stride - 1) / p.save_stride : 0;

    for (int c = 0; c < nchunks; ++c) {
        const int s = c & 1, t0 = c * TC;
        const int nv = min(TC, T - t0);
        if (tid == 0 && c + 1 < nchunks) issue_loads(c + 1);
        // Tensors that could not be described to TMA: cooperative plain loads.
        if (load_mask != (kTmaX | kTmaDl | kTmaZ | kTmaB | kTmaC)) {
            if (!(load_mask & kTmaX))
                load_tile_plain(raw_x(s), static_cast<const Tact*>(p.x), p.ld_x, b, T, t0, d0, D, TC,
                                DT, THREADS);
            if (!(load_mask & kTmaDl))
                load_tile_plain(raw_dl(s), static_cast<const Tact*>(p.dl), p.ld_dl, b, T, t0, d0, D,
                                TC, DT, THREADS);
            if (has_z && !(load_mask & kTmaZ))
                load_tile_plain(raw_z(s), static_cast<const Tact*>(p.z), p.ld_z, b, T, t0, d0, D, TC,
                                DT, THREADS);
            if (!(load_mask & kTmaB))
                load_tile_plain(raw_b(s), static_cast<const Tact*>(p.bm), p.ld_bc, b, T, t0, 0, N,
                                TC, N, THREADS);
            if (!(load_mask & kTmaC))
                load_tile_plain(raw_c(s), static_cast<const Tact*>(p.cm), p.ld_bc, b, T, t0, 0, N,
                                TC, N, THREADS);
            __syncthreads();
        }
        if (tx_bytes) mbar_wait(&bars[s], (c >> 1) & 1, p.status);

        // ---------------- stage 1: elementwise prologue ----------------
        {
            const Tact* rx = raw_x(s);
            const Tact* rd = raw_dl(s);
            const Tact* rz = raw_z(s);
            for (int i = tid; i < TC * (DT / 2); i += THREADS) {
                const int r = i / (DT / 2), dl_ = (i - r * (DT / 2)) * 2;
                float2 u;
                if (K) {
                    float2 acc = make_float2(cb_s[dl_], cb_s[dl_ + 1]);
                    for (int k = 0; k < K; ++k) {
                        const int rr = r - (K - 1) + k;
                        float2 xv = rr >= 0 ? ld_pair(rx + rr * DT + dl_)
                                            : make_float2(halo[(K + rr) * DT + dl_],
                                                          halo[(K + rr) * DT + dl_ + 1]);
                        acc = fma2(xv, make_float2(cw_s[k * DT + dl_], cw_s[k * DT + dl_ + 1]), acc);
                    }
                    u = make_float2(siluf_fast(acc.x), siluf_fast(acc.y));
                    if (p.u_out && r < nv) {
                        Tact* up = static_cast<Tact*>(p.u_out) +
                                   (static_cast<long long>(b) * T + t0 + r) * p.ld_u + d0 + dl_;
                        if (d0 + dl_ + 1 < D && p.u_vec) st_pair(up, u);
                        else {
                            if (d0 + dl_ < D) up[0] = from_f<Tact>(u.x);
                            if (d0 + dl_ + 1 < D) up[1] = from_f<Tact>(u.y);
                        }
                    }
                } else {
                    u = ld_pair(rx + r * DT + dl_);
                }
                float2 dl = ld_pair(rd + r * DT + dl_);
                if (p.delta_softplus) dl = make_float2(softplusf_fast(dl.x), softplusf_fast(dl.y));
                const float2 du = mul2(dl, u);
                float2 g = make_float2(1.0f, 1.0f);
                if (has_z) {
                    g = ld_pair(rz + r * DT + dl_);
                    if (p.z_mode == 1) g = make_float2(siluf_fast(g.x), siluf_fast(g.y));
                }
                const float2 skip = mul2(mul2(make_float2(dp_s[dl_], dp_s[dl_ + 1]), u), g);
                // staging index [r][c][grp]: channel = grp*CH + c
                const int g0 = dl_ / CH, c0 = dl_ % CH;
                const int g1 = (dl_ + 1) / CH, c1 = (dl_ + 1) % CH;
                A1[(r * CH + c0) * G + g0] = make_float2(dl.x, du.x);
                A1[(r * CH + c1) * G + g1] = make_float2(dl.y, du.y);
                A2[(r * CH + c0) * G + g0] = make_float2(g.x, skip.x);
                A2[(r * CH + c1) * G + g1] = make_float2(g.y, skip.y);
            }
            // B / C -> f32, zero-padded to NP columns.
            const Tact* rb = raw_b(s);
            const Tact* rc = raw_c(s);
            for (int i = tid; i < TC * NP; i += THREADS) {
                const int r = i / NP, n = i - r * NP;
                Bs[i] = n < N ? to_f(rb[r * N + n]) : 0.0f;
                Cs[i] = n < N ? to_f(rc[r * N + n]) : 0.0f;
            }
        }
        if (tid == 0) tma_wait_read0();  // previous y tile fully read before it is rewritten
        __syncthreads();

        // Conv window hand-over: the K most recent x values per channel.
        if (K) {
            const Tact* rx = raw_x(s);
            for (int i = tid; i < DT; i += THREADS) {
                float nw[kKMax];
                for (int k = 0; k < K; ++k) {
                    const int rr = nv - K + k;  // row of the chunk, or negative -> old window
                    nw[k] = rr >= 0 ? to_f(rx[rr * DT + i]) : halo[(K + rr) * DT + i];
                }
                for (int k = 0; k < K; ++k) halo[k * DT + i] = nw[k];
            }
        }
        // Training save: state entering each block of save_stride steps.
        if (p.chunk_states && (t0 % p.save_stride) == 0) {
            const long long sc = t0 / p.save_stride;
#pragma unroll
            for (int cc = 0; cc < CH; ++cc) {
                const int d = d0 + grp * CH + cc;
#pragma unroll
                for (int j = 0; j < NS; ++j) {
                    const int n = n0 + j;
                    if (d < D && n < N)
                        p.chunk_states[((static_cast<long long>(b) * save_chunks + sc) * D + d) * N + n] =
                            (j & 1) ? h[cc][j / 2].y : h[cc][j / 2].x;
                }
            }
        }

        // ---------------- stage 2: recurrence + epilogue ----------------
        auto run = [&](auto geo_tag) {
            constexpr bool GEO = decltype(geo_tag)::value;
#pragma unroll 2
            for (int r = 0; r < nv; ++r) {
                float2 Bv[NS / 2], Cv[NS / 2];
#pragma unroll
                for (int j = 0; j < NS / 4; ++j) {
                    const float4 bb = *reinterpret_cast<const float4*>(Bs + r * NP + n0 + 4 * j);
                    const float4 cc = *reinterpret_cast<const float4*>(Cs + r * NP + n0 + 4 * j);
                    Bv[2 * j] = make_float2(bb.x, bb.y);
                    Bv[2 * j + 1] = make_float2(bb.z, bb.w);
                    Cv[2 * j] = make_float2(cc.x, cc.y);
                    Cv[2 * j + 1] = make_float2(cc.z, cc.w);
                }
                float yv[CH];
#pragma unroll
                for (int cc = 0; cc < CH; ++cc) {
                    const float2 dd = A1[(r * CH + cc) * G + grp];  // (delta, delta*u)
                    const float2 du2 = splat2(dd.y);
                    float2 y2 = make_float2(0.0f, 0.0f);
                    if (GEO) {
                        const float E = ex2(dd.x * a2[cc][0].x);
                        const float R = ex2(dd.x * (a2[cc][0].y - a2[cc][0].x));
                        float2 e = make_float2(E, E * R);
                        const float2 r2 = splat2(R * R);
#pragma unroll
                        for (int j = 0; j < NS / 2; ++j) {
                            h[cc][j] = fma2(e, h[cc][j], mul2(du2, Bv[j]));
                            y2 = fma2(h[cc][j], Cv[j], y2);
                            e = mul2(e, r2);
                        }
                    } else {
                        const float2 dl2 = splat2(dd.x);
#pragma unroll
                        for (int j = 0; j < NS / 2; ++j) {
                            const float2 xa = mul2(dl2, a2[cc][j]);
                            const float2 e = make_float2(ex2(xa.x), ex2(xa.y));
                            h[cc][j] = fma2(e, h[cc][j], mul2(du2, Bv[j]));
                            y2 = fma2(h[cc][j], Cv[j], y2);
                        }
                    }
                    float y = y2.x + y2.y;
#pragma unroll
                    for (int m = 1; m < LPC; m <<= 1) y += __shfl_xor_sync(0xffffffffu, y, m);
                    yv[cc] = y;
                }
                if (part == 0) {
#pragma unroll
                    for (int cc = 0; cc < CH; ++cc) {
                        const float2 gs = A2[(r * CH + cc) * G + grp];  // (gate, D*u*gate)
                        yv[cc] = fmaf(yv[cc], gs.x, gs.y);
                    }
                    Tact* o = out_t + r * DT + grp * CH;
                    if (CH % 2 == 0) {
#pragma unroll
                        for (int cc = 0; cc < CH; cc += 2) st_pair(o + cc, make_float2(yv[cc], yv[cc + 1]));
                    } else {
#pragma unroll
                        for (int cc = 0; cc < CH; ++cc) o[cc] = from_f<Tact>(yv[cc]);
                    }
                }
            }
        };
        if (geo) run(std::true_type{});
        else run(std::false_type{});

        // ---------------- store the y tile ----------------
        if (p.tma_mask & kTmaY) {
            fence_proxy_async();
            __syncthreads();
            if (tid == 0) {
                tma_store_3d(&p.tm_y, out_t, d0, t0, b);
                tma_commit();
            }
        } else {
            __syncthreads();
            Tact* yb = static_cast<Tact*>(p.y);
            for (int i = tid; i < nv * DT; i += THREADS) {
                const int r = i / DT, cidx = i - r * DT;
                if (d0 + cidx < D)
                    yb[(static_cast<long long>(b) * T + t0 + r) * p.ld_y + d0 + cidx] = out_t[i];
            }
            __syncthreads();
        }
    }

    // Final recurrent state and conv window.
    if (p.ssm_state) {
#pragma unroll
        for (int cc = 0; cc < CH; ++cc) {
            const int d = d0 + grp * CH + cc;
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                const int n = n0 + j;
                if (d < D && n < N)
                    p.ssm_state[(static_cast<long long>(b) * D + d) * N + n] =
                        (j & 1) ? h[cc][j / 2].y : h[cc][j / 2].x;
            }
        }
    }
    if (K && p.conv_state) {
        __syncthreads();
        for (int i = tid; i < DT; i += THREADS) {
            const int d = d0 + i;
            if (d < D)
                for (int k = 0; k < K; ++k)
                    p.conv_state[(static_cast<long long>(b) * D + d) * K + k] = halo[k * DT + i];
        }
    }
    if (tid == 0) tma_wait_read0();  // shared memory must outlive the last bulk store
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef void (*FwdKernelFn)(const FwdParams);

struct FwdVariant {
    int ns, lpc, dt, tc, threads;
    size_t smem[3];     // by dtype
    FwdKernelFn fn[3];  // by dtype
};

template <int CH, int NS, int LPC, int WARPS, int TC>
static FwdVariant make_variant() {
    using T0 = FwdTraits<float, CH, NS, LPC, WARPS, TC>;
    using T1 = FwdTraits<__half, CH, NS, LPC, WARPS, TC>;
    using T2 = FwdTraits<__nv_bfloat16, CH, NS, LPC, WARPS, TC>;
    FwdVariant v;
    v.ns = NS; v.lpc = LPC; v.dt = T0::DT; v.tc = TC; v.threads = T0::THREADS;
    v.smem[MAMBA_B200_F32] = T0::SMEM;
    v.smem[MAMBA_B200_F16] = T1::SMEM;
    v.smem[MAMBA_B200_BF16] = T2::SMEM;
    v.fn[MAMBA_B200_F32] = sscan_fwd_kernel<T0, float>;
    v.fn[MAMBA_B200_F16] = sscan_fwd_kernel<T1, __half>;
    v.fn[MAMBA_B200_BF16] = sscan_fwd_kernel<T2, __nv_bfloat16>;
    return v;
}

#ifndef MB200_FWD_CH
#define MB200_FWD_CH 2
#endif
#ifndef MB200_FWD_WARPS
#define MB200_FWD_WARPS 4
#endif
#ifndef MB200_FWD_TC
#define MB200_FWD_TC 16
#endif

// Variants by padded d_state: slice of 8 states per lane, LPC lanes per channel
// (d_state <= 4 uses a 4-state slice).
static const FwdVariant* fwd_variants(int* count) {
    static FwdVariant v[7];
    static bool init = false;
    if (!init) {
        v[0] = make_variant<MB200_FWD_CH, 4, 1, MB200_FWD_WARPS, MB200_FWD_TC>();
        v[1] = make_variant<MB200_FWD_CH, 8, 1, MB200_FWD_WARPS, MB200_FWD_TC>();
        v[2] = make_variant<MB200_FWD_CH, 8, 2, MB200_FWD_WARPS, MB200_FWD_TC>();
        v[3] = make_variant<MB200_FWD_CH, 8, 4, MB200_FWD_WARPS, MB200_FWD_TC>();
        v[4] = make_variant<MB200_FWD_CH, 8, 8, MB200_FWD_WARPS, MB200_FWD_TC>();
        v[5] = make_variant<MB200_FWD_CH, 8, 16, MB200_FWD_WARPS, MB200_FWD_TC>();
        v[6] = make_variant<MB200_FWD_CH, 8, 32, MB200_FWD_WARPS, MB200_FWD_TC>();
        init = true;
    }
    *count = 7;
    return v;
}

int m1_fwd_configure(Ctx* c) {
    int n = 0;
    const FwdVariant* v = fwd_variants(&n);
    for (int i = 0; i < n; ++i)
        for (int dt = 0; dt < 3; ++dt)
            MB200_CUDA_CHECK(c, cudaFuncSetAttribute(reinterpret_cast<const void*>(v[i].fn[dt]),
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     static_cast<int>(v[i].smem[dt])));
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

    int nv = 0;
    const FwdVariant* vs = fwd_variants(&nv);
    const FwdVariant* v = nullptr;
    for (int i = 0; i < nv; ++i)
        if (vs[i].ns * vs[i].lpc >= a.N) { v = &vs[i]; break; }
    if (!v) return fail(c, MAMBA_B200_ERR_SHAPE, "sscan_fwd: no variant for d_state %d", a.N);
    if (a.chunk_states && (a.save_stride <= 0 || a.save_stride % v->tc != 0))
        return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: save_stride %d is not a multiple of %d",
                    a.save_stride, v->tc);

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

    dim3 grid((a.D + v->dt - 1) / v->dt, a.B);
    v->fn[a.dtype]<<<grid, v->threads, v->smem[a.dtype], stream>>>(p);
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}

}  // namespace mb200

using namespace mb200;

extern "C" int mamba_b200_sscan_fwd(void* handle, void* stream, const mamba_b200_sscan_fwd_args* args) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!args) return fail(c, MAMBA_B200_ERR_ARG, "sscan_fwd: null args");
    return launch_fwd(c, static_cast<cudaStream_t>(stream), *args);
}

extern "C" int mamba_b200_ssm_scan_fwd_nosave(void* handle, void* stream, int dtype, float* h,
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
