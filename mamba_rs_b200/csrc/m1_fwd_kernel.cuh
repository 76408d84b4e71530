// Mamba-1 fused selective-scan forward for sm_100a.
//
// One CTA owns (sample b, a tile of DT channels, a time segment) and walks its
// steps in chunks of TC.  The CTA is CW consumer warps plus one producer warp;
// no block-wide barrier exists in the loop, the warps meet on mbarriers only:
//
//   producer : TMA (cp.async.bulk.tensor.3d, no multicast) brings the x / delta
//              / z / B / C tiles of chunk c+STAGES-1 into a ring of shared-memory
//              stages (full[s] signals arrival), and widens the landed B / C
//              tiles to zero-padded f32 rows once per CTA (bcfull[s]);
//   consumers: LPC lanes own one channel, NS states each, in registers for the
//              whole sequence.  Per block of RB = 4 steps the lanes of a channel
//              split the elementwise work by step (conv1d + SiLU, softplus(delta),
//              SiLU(z), D skip), exchange (delta, delta*u) with shuffles, run
//              h = exp(delta*a)*h + delta*u*B, y = <h, C> in packed f32x2, combine
//              their partial y and store the finished rows straight to global
//              memory; empty[s] hands the stage back.
//
// HBM is touched once per input and once per output element (the fused conv
// re-reads an 8-row halo per chunk, mostly from L2).
#pragma once
#include <string.h>

#include <type_traits>
#include <utility>

#include "common.cuh"
#include "internal.h"

namespace mb200 {

constexpr int kKMax = 8;       // widest supported d_conv
constexpr int kHaloRows = 8;   // rows of x before the chunk kept in the tile (>= kKMax - 1)

struct FwdParams {
    CUtensorMap tm_x, tm_dl, tm_z, tm_b, tm_c;
    const void *x, *dl, *z, *bm, *cm;
    void *y, *u_out;
    long long ld_x, ld_dl, ld_z, ld_bc, ld_y, ld_u;
    const float *a_neg, *Dp, *conv_w, *conv_b;
    float *conv_state, *ssm_state, *chunk_states;   // conv / ssm state: written at the end
    long long cs_ld_b, cs_ld_k;   // saved state k of sample b starts at chunk_states + b*cs_ld_b + k*cs_ld_k
    const float *conv_in, *ssm_in;                  // entering conv window / state (read)
    float *conv_copy, *ssm_copy;  // state-only pass, segment 0: keeps the entering state for the second pass
    // Time segments (grid.z > 1): segment s > 0 starts from seg_states[b][s-1] and
    // reads no conv / ssm state; a state-only launch writes its leaving state and
    // the sum of its deltas per channel instead of y.
    float* seg_states;   // [B][segments][D][N]
    float* seg_sumdl;    // [B][segments][D] (state-only launch)
    int seg_chunks;      // chunks per segment (0: one segment)
    int B, T, D, N, K;
    int z_mode, save_stride;
    unsigned tma_mask;  // bit0 x, bit1 delta, bit2 z, bit3 B, bit4 C
    int* status;
};

enum : unsigned { kTmaX = 1, kTmaDl = 2, kTmaZ = 4, kTmaB = 8, kTmaC = 16 };

template <typename Tact, int NS_, int LPC_, int CW_, int TC_, int STAGES_>
struct FwdTraits {
    static constexpr int NS = NS_, LPC = LPC_, CW = CW_, TC = TC_, STAGES = STAGES_;
    static constexpr int THREADS = (CW + 1) * 32;
    static constexpr int CHW = 32 / LPC;      // channels per consumer warp
    static constexpr int DT = CW * CHW;       // channels per CTA
    static constexpr int NP = NS * LPC;       // padded d_state
    static constexpr int RB = 4;              // steps per block of the hot loop
    static constexpr int OWN = LPC >= RB ? 1 : RB / LPC;  // elementwise rows a lane owns per block
    static constexpr size_t al(size_t v) { return (v + 127) & ~size_t(127); }
    static constexpr size_t X_TILE = al(sizeof(Tact) * (TC + kHaloRows) * DT);
    static constexpr size_t ACT = al(sizeof(Tact) * TC * DT);
    static constexpr size_t RAW_BC = al(sizeof(Tact) * TC * NP);
    static constexpr size_t WIDE = al(sizeof(float) * TC * NP);
    static constexpr size_t OFF_X = 0, OFF_DL = X_TILE, OFF_Z = OFF_DL + ACT, OFF_RB = OFF_Z + ACT,
                            OFF_RC = OFF_RB + RAW_BC, OFF_WB = OFF_RC + RAW_BC, OFF_WC = OFF_WB + WIDE,
                            STAGE = OFF_WC + WIDE;
    static constexpr size_t OFF_BAR = STAGES * STAGE;  // full, empty, bcfull: 3 * STAGES mbarriers
    static constexpr size_t SMEM = OFF_BAR + 128;
    static_assert(NS == 8 || NS == 16, "a lane holds 8 or 16 states");
    static_assert((LPC & (LPC - 1)) == 0 && LPC <= 32, "LPC must be a power of two");
    static_assert(TC % RB == 0, "chunk must be a whole number of blocks");
    static_assert(3 * STAGES * 8 <= 128, "barrier area");
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// sigmoid through one MUFU op (tanh), 2^-11 relative error: 16-bit storage only.
__device__ __forceinline__ float sigmoid_tanh(float v) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * v));
    return fmaf(t, 0.5f, 0.5f);
}
template <bool HALF>
__device__ __forceinline__ float silu_sel(float v) {
    if constexpr (HALF) return v * sigmoid_tanh(v);
    else return siluf_fast(v);
}
// softplus for 16-bit storage: ln(1 + e) straight from the MUFU pipe (the small-e
// series of softplusf_fast buys accuracy far below the storage rounding here).
template <bool HALF>
__device__ __forceinline__ float softplus_sel(float v) {
    if constexpr (HALF) {
        const float e = ex2(fminf(v, 20.0f) * kLog2e);
        const float r = lg2(1.0f + e) * kLn2;
        return v > 20.0f ? v : r;
    } else {
        return softplusf_fast(v);
    }
}

// FLAGS (compile-time, so that the hot block is one branch-free basic block):
//   bit0 softplus on delta, bit1 gate present, bit2 conv1d + SiLU on x,
//   bit3 state-only pass (no y: leaves the segment's final state and delta sum).
template <typename Tr, typename Tact, int FLAGS>
__global__ void __launch_bounds__(Tr::THREADS)
sscan_fwd_kernel(const __grid_constant__ FwdParams p) {
    constexpr bool kSoftplus = (FLAGS & 1) != 0, kStateOnly = (FLAGS & 8) != 0;
    constexpr bool kGate = (FLAGS & 2) != 0 && !kStateOnly, kConv = (FLAGS & 4) != 0;
    constexpr int NS = Tr::NS, LPC = Tr::LPC, TC = Tr::TC, DT = Tr::DT, NP = Tr::NP, CW = Tr::CW,
                  STAGES = Tr::STAGES, RB = Tr::RB, OWN = Tr::OWN, CHW = Tr::CHW;
    constexpr bool kHalf = sizeof(Tact) == 2;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + Tr::OFF_BAR);
    uint64_t* empty = full + STAGES;
    uint64_t* bcfull = empty + STAGES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.y;
    const int d0 = blockIdx.x * DT;
    const int T = p.T, D = p.D, N = p.N, K = kConv ? p.K : 0;
    const int nchunks_all = (T + TC - 1) / TC;
    const int seg = blockIdx.z, nseg = gridDim.z;
    const int c_begin = p.seg_chunks > 0 ? min(nchunks_all, seg * p.seg_chunks) : 0;
    const int c_end = (p.seg_chunks > 0 && seg + 1 < nseg) ? min(nchunks_all, (seg + 1) * p.seg_chunks)
                                                           : nchunks_all;
    const int nch = c_end - c_begin;  // chunks this CTA walks
    if (kStateOnly && seg == nseg - 1) return;  // nothing follows the last segment
    const unsigned load_mask = p.tma_mask;
    const bool use_z = kGate;

    auto stage = [&](int s) { return smem + static_cast<size_t>(s) * Tr::STAGE; };

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CW * 32);
            mbar_init(&bcfull[s], 32);
        }
        fence_barrier_init();
    }
    __syncthreads();

    // =========================== producer warp ===========================
    if (warp == CW) {
        uint32_t tx_bytes = 0;
        if (load_mask & kTmaX) tx_bytes += sizeof(Tact) * (kConv ? TC + kHaloRows : TC) * DT;
        if (load_mask & kTmaDl) tx_bytes += sizeof(Tact) * TC * DT;
        if (use_z && (load_mask & kTmaZ)) tx_bytes += sizeof(Tact) * TC * DT;
        if (load_mask & kTmaB) tx_bytes += sizeof(Tact) * TC * N;
        if (!kStateOnly && (load_mask & kTmaC)) tx_bytes += sizeof(Tact) * TC * N;
        const Tact zero = from_f<Tact>(0.0f);
        // Copies one [rows x cols] tile with plain loads (a tensor that breaks a TMA
        // layout rule): out-of-range elements become zero, as TMA would fill them.
        auto plain = [&](Tact* dst, const void* src, long long ld, int t_first, int rows, int c_first,
                         int box_cols, int cols_total) {
            const Tact* g = static_cast<const Tact*>(src);
            for (int i = lane; i < rows * box_cols; i += 32) {
                const int r = i / box_cols, cc = i - r * box_cols;
                const int t = t_first + r, col = c_first + cc;
                Tact v = zero;
                if (t >= 0 && t < T && col < cols_total) v = g[(static_cast<long long>(b) * T + t) * ld + col];
                dst[i] = v;
            }
        };
        auto issue = [&](int c) {  // whole warp
            const int s = c % STAGES, t0 = (c_begin + c) * TC;
            unsigned char* st = stage(s);
            Tact* xs = reinterpret_cast<Tact*>(st + Tr::OFF_X);
            const int xr0 = kConv ? t0 - kHaloRows : t0;
            Tact* xdst = kConv ? xs : xs + kHaloRows * DT;
            const bool any_plain = (load_mask & (kTmaX | kTmaDl | kTmaB)) != (kTmaX | kTmaDl | kTmaB) ||
                                   (use_z && !(load_mask & kTmaZ)) || (!kStateOnly && !(load_mask & kTmaC));
            if (any_plain) {
                if (!(load_mask & kTmaX)) plain(xdst, p.x, p.ld_x, xr0, kConv ? TC + kHaloRows : TC, d0, DT, D);
                if (!(load_mask & kTmaDl))
                    plain(reinterpret_cast<Tact*>(st + Tr::OFF_DL), p.dl, p.ld_dl, t0, TC, d0, DT, D);
                if (use_z && !(load_mask & kTmaZ))
                    plain(reinterpret_cast<Tact*>(st + Tr::OFF_Z), p.z, p.ld_z, t0, TC, d0, DT, D);
                if (!(load_mask & kTmaB))
                    plain(reinterpret_cast<Tact*>(st + Tr::OFF_RB), p.bm, p.ld_bc, t0, TC, 0, N, N);
                if (!kStateOnly && !(load_mask & kTmaC))
                    plain(reinterpret_cast<Tact*>(st + Tr::OFF_RC), p.cm, p.ld_bc, t0, TC, 0, N, N);
                __syncwarp();
            }
            if (lane == 0) {
                // one arrival completes the phase once every TMA byte has landed
                mbar_expect_tx(&full[s], tx_bytes);
                if (load_mask & kTmaX) tma_load_3d(xdst, &p.tm_x, &full[s], d0, xr0, b);
                if (load_mask & kTmaDl) tma_load_3d(st + Tr::OFF_DL, &p.tm_dl, &full[s], d0, t0, b);
                if (use_z && (load_mask & kTmaZ)) tma_load_3d(st + Tr::OFF_Z, &p.tm_z, &full[s], d0, t0, b);
                if (load_mask & kTmaB) tma_load_3d(st + Tr::OFF_RB, &p.tm_b, &full[s], 0, t0, b);
                if (!kStateOnly && (load_mask & kTmaC)) tma_load_3d(st + Tr::OFF_RC, &p.tm_c, &full[s], 0, t0, b);
            }
        };
        int issued = 0, widened = 0;
        bool ok = true;
        for (; issued < nch && issued < STAGES - 1; ++issued) issue(issued);
        for (int c = 0; c < nch && ok; ++c) {
            const int s = c % STAGES;
            ok = mbar_wait(&full[s], (c / STAGES) & 1, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            widened = c + 1;
            // B / C rows of the chunk as zero-padded f32 [TC][NP]
            {
                const Tact* rb = reinterpret_cast<const Tact*>(stage(s) + Tr::OFF_RB);
                const Tact* rc = reinterpret_cast<const Tact*>(stage(s) + Tr::OFF_RC);
                float4* wb = reinterpret_cast<float4*>(stage(s) + Tr::OFF_WB);
                float4* wc = reinterpret_cast<float4*>(stage(s) + Tr::OFF_WC);
                constexpr int Q = NP / 4;
                for (int i = lane; i < TC * Q; i += 32) {
                    const int r = i / Q, n = (i - r * Q) * 4;
                    float vb[4], vc[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const bool in = n + j < N;
                        vb[j] = in ? to_f(rb[r * N + n + j]) : 0.0f;
                        vc[j] = (in && !kStateOnly) ? to_f(rc[r * N + n + j]) : 0.0f;
                    }
                    wb[i] = make_float4(vb[0], vb[1], vb[2], vb[3]);
                    if (!kStateOnly) wc[i] = make_float4(vc[0], vc[1], vc[2], vc[3]);
                }
            }
            mbar_arrive(&bcfull[s]);
            // refill the stage chunk c-1 used, once every consumer has left it
            if (issued < nch) {
                if (c >= 1) {
                    ok = mbar_wait(&empty[(c - 1) % STAGES], ((c - 1) / STAGES) & 1, p.status);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                issue(issued++);
            }
        }
        // After a wait that gave up, the bulk copies still in flight must land before
        // the CTA may leave (its shared memory is their destination).
        for (int c = widened; c < issued; ++c) mbar_wait(&full[c % STAGES], (c / STAGES) & 1, p.status);
        return;
    }

    // =========================== consumer warps ===========================
    const int colw = lane / LPC, part = lane % LPC;   // channel within the warp, state slice
    const int col = warp * CHW + colw;
    const int d = d0 + col;
    const bool d_ok = d < D;
    const int n0 = part * NS;
    const int lane_base = lane & ~(LPC - 1);
    float2 h[NS / 2], a2[NS / 2];  // a2 = a_neg * log2(e)
    bool geo_local = true;
    {
        float av[NS], hv[NS];
        const float* h0 = nullptr;
        if (seg == 0) h0 = p.ssm_in ? p.ssm_in + (static_cast<long long>(b) * D) * N : nullptr;
        else if (!kStateOnly) h0 = p.seg_states + ((static_cast<long long>(b) * nseg + (seg - 1)) * D) * N;
        // (a state-only segment after the first starts from zero)
#pragma unroll
        for (int j = 0; j < NS; ++j) {
            const int n = n0 + j;
            const bool okn = d_ok && n < N;
            av[j] = okn ? p.a_neg[static_cast<long long>(d) * N + n] * kLog2e : 0.0f;
            hv[j] = (okn && h0) ? h0[static_cast<long long>(d) * N + n] : 0.0f;
            if (kStateOnly && seg == 0 && okn && p.ssm_copy)
                p.ssm_copy[(static_cast<long long>(b) * D + d) * N + n] = hv[j];
        }
        // Arithmetic-progression test a[n] = a[n0] + (n-n0)*step, to 4 ulp: then
        // exp(delta*a[n]) = E * R^(n-n0) and a step needs 2 exp2 instead of NS.
        const float step = av[1] - av[0];
#pragma unroll
        for (int j = 2; j < NS; ++j) {
            const float pred = fmaf(static_cast<float>(j), step, av[0]);
            if (fabsf(av[j] - pred) > 4.8e-7f * fabsf(av[j])) geo_local = false;
        }
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) {
            a2[j] = make_float2(av[2 * j], av[2 * j + 1]);
            h[j] = make_float2(hv[2 * j], hv[2 * j + 1]);
        }
    }
    const bool geo = __all_sync(0xffffffffu, geo_local ? 1 : 0) != 0;  // per warp
    const float a2_first = a2[0].x, a2_step = a2[0].y - a2[0].x;
    const float Dd = d_ok ? p.Dp[d] : 0.0f;
    // conv taps aligned to the END of an 8-tap window: w8[j] multiplies x[t - 7 + j]
    float w8[kKMax];
    float cb = 0.0f;
#pragma unroll
    for (int j = 0; j < kKMax; ++j) {
        const int k = j - (kKMax - K);
        w8[j] = (kConv && k >= 0 && d_ok) ? p.conv_w[static_cast<long long>(d) * K + k] : 0.0f;
    }
    if (kConv && d_ok) cb = p.conv_b[d];
    if (kConv && kStateOnly && seg == 0 && p.conv_copy && part == 0 && d_ok)
        for (int k = 0; k < K; ++k)
            p.conv_copy[(static_cast<long long>(b) * D + d) * K + k] =
                p.conv_in ? p.conv_in[(static_cast<long long>(b) * D + d) * K + k] : 0.0f;
    const bool gate_is_silu = p.z_mode == 1;
    float sum_dl = 0.0f;  // state-only pass: sum of this segment's deltas (owner rows only)

    Tact* yg = static_cast<Tact*>(p.y);
    Tact* ug = static_cast<Tact*>(p.u_out);

    struct Elem {
        float dl, du, g, sk;
    };
    // What the recurrence of one row needs from the elementwise stage, in every lane of
    // the channel: with an arithmetic-progression a_neg the two seeds of the decay tree
    // (p0 = R = exp2(delta * step), p1 = E = exp2(delta * a_first)), otherwise delta
    // itself (p0); and delta * u.
    struct Prep {
        float p0, p1, du;
    };

    bool alive = true;
    for (int c = 0; c < nch; ++c) {
        const int s = c % STAGES, t0 = (c_begin + c) * TC;
        const int nv = min(TC, T - t0);
        {
            bool ok = mbar_wait(&full[s], (c / STAGES) & 1, p.status);
            ok = ok && mbar_wait(&bcfull[s], (c / STAGES) & 1, p.status);
            alive = __all_sync(0xffffffffu, ok);
            if (!alive) break;
        }
        unsigned char* st = stage(s);
        const Tact* xt = reinterpret_cast<const Tact*>(st + Tr::OFF_X) + kHaloRows * DT + col;  // row 0 of the chunk
        const Tact* rd = reinterpret_cast<const Tact*>(st + Tr::OFF_DL) + col;
        const Tact* rz = reinterpret_cast<const Tact*>(st + Tr::OFF_Z) + col;
        const float* Bp = reinterpret_cast<const float*>(st + Tr::OFF_WB) + n0;
        const float* Cp = reinterpret_cast<const float*>(st + Tr::OFF_WC) + n0;

        // Training save: state entering each block of save_stride steps.
        if (!kStateOnly && p.chunk_states && (t0 % p.save_stride) == 0) {
            const long long sc = t0 / p.save_stride;
            float* dst = p.chunk_states + b * p.cs_ld_b + sc * p.cs_ld_k + static_cast<long long>(d) * N;
#pragma unroll
            for (int j = 0; j < NS; ++j)
                if (d_ok && n0 + j < N) dst[n0 + j] = (j & 1) ? h[j / 2].y : h[j / 2].x;
        }

        // Elementwise stage of one timestep (row r of the chunk).  SLOW: the first
        // rows of the sequence, whose conv taps reach into the carried window.
        auto elem = [&](auto slow_tag, int r) -> Elem {
            constexpr bool SLOW = decltype(slow_tag)::value;
            (void)SLOW;
            float u;
            if constexpr (kConv) {
                float acc = cb;
#pragma unroll
                for (int j = 0; j < kKMax; ++j) {
                    float xv = to_f(xt[(r - (kKMax - 1) + j) * DT]);
                    if constexpr (SLOW) {
                        const int tg = t0 + r - (kKMax - 1) + j;  // global step of this tap
                        const int k = j - (kKMax - K);
                        if (tg < 0)
                            xv = (k >= 0 && d_ok && p.conv_in && K + tg >= 0)
                                     ? p.conv_in[(static_cast<long long>(b) * D + d) * K + K + tg]
                                     : 0.0f;
                    }
                    acc = fmaf(xv, w8[j], acc);  // w8[j] == 0 outside the K-tap window
                }
                u = silu_sel<kHalf>(acc);
                if (!kStateOnly && ug && d_ok)
                    ug[(static_cast<long long>(b) * T + t0 + r) * p.ld_u + d] = from_f<Tact>(u);
            } else {
                u = to_f(xt[r * DT]);
            }
            float dv = to_f(rd[r * DT]);
            if (kSoftplus) dv = softplus_sel<kHalf>(dv);
            float gv = 1.0f;
            if (kGate) {
                const float zv = to_f(rz[r * DT]);
                const float sz = silu_sel<kHalf>(zv);
                gv = gate_is_silu ? sz : zv;  // select, not a branch
            }
            Elem o;
            o.dl = dv;
            o.du = dv * u;
            o.g = gv;
            o.sk = Dd * u * gv;
            return o;
        };
        // Elementwise work this lane owns in the block starting at row r0: rows
        // r0 + part, r0 + part + LPC, ... (one row, clamped, when LPC >= RB).
        auto elem_block = [&](int r0, Elem* out) {
#pragma unroll
            for (int k = 0; k < OWN; ++k) {
                const int r = LPC >= RB ? r0 + min(part, RB - 1) : r0 + k * LPC + part;
                out[k] = elem(std::false_type{}, r);
            }
        };
        auto prep_row = [&](auto geo_tag, float dli, float dui) -> Prep {
            constexpr bool GEO = decltype(geo_tag)::value;
            Prep q;
            q.du = dui;
            if (GEO) {
                q.p0 = ex2(dli * a2_step);
                q.p1 = ex2(dli * a2_first);
            } else {
                q.p0 = dli;
                q.p1 = 0.0f;
            }
            return q;
        };
        // (delta, delta*u) of every row of a block from the lanes that own the rows
        auto prep_block = [&](auto geo_tag, const Elem* el, Prep* pp) {
#pragma unroll
            for (int i = 0; i < RB; ++i) {
                const int owner = LPC >= RB ? i : i % LPC, k = LPC >= RB ? 0 : i / LPC;
                float dli = el[k].dl, dui = el[k].du;
                if (LPC > 1) {
                    dli = __shfl_sync(0xffffffffu, dli, lane_base + owner);
                    dui = __shfl_sync(0xffffffffu, dui, lane_base + owner);
                }
                pp[i] = prep_row(geo_tag, dli, dui);
            }
        };
        // exp(delta * a) for the NS states of this lane
        auto decays = [&](auto geo_tag, const Prep& q, float2* e) {
            constexpr bool GEO = decltype(geo_tag)::value;
            if (GEO) {
                // e[j] = (E R^(2j), E R^(2j+1)): product tree of depth 3 (4 with 16 states)
                const float R = q.p0, E0 = q.p1;
                const float R2 = R * R, R4 = R2 * R2;
                const float2 r2 = splat2(R2), r4 = splat2(R4);
                e[0] = make_float2(E0, E0 * R);
                e[1] = mul2(e[0], r2);
                e[2] = mul2(e[0], r4);
                e[3] = mul2(e[1], r4);
                if constexpr (NS == 16) {
                    const float2 r8 = splat2(R4 * R4);
#pragma unroll
                    for (int j = 0; j < 4; ++j) e[4 + j] = mul2(e[j], r8);
                }
            } else {
                const float2 dl2 = splat2(q.p0);
#pragma unroll
                for (int j = 0; j < NS / 2; ++j) {
                    const float2 xa = mul2(dl2, a2[j]);
                    e[j] = make_float2(ex2(xa.x), ex2(xa.y));
                }
            }
        };
        // one step of the recurrence; returns this lane's partial y
        auto step = [&](auto geo_tag, const Prep& q, int r) -> float {
            float4 bq[NS / 4];
#pragma unroll
            for (int v = 0; v < NS / 4; ++v) bq[v] = *reinterpret_cast<const float4*>(Bp + r * NP + 4 * v);
            float2 e[NS / 2];
            decays(geo_tag, q, e);
            const float2 du2 = splat2(q.du);
#pragma unroll
            for (int v = 0; v < NS / 4; ++v) {
                h[2 * v] = fma2(e[2 * v], h[2 * v], mul2(du2, make_float2(bq[v].x, bq[v].y)));
                h[2 * v + 1] = fma2(e[2 * v + 1], h[2 * v + 1], mul2(du2, make_float2(bq[v].z, bq[v].w)));
            }
            if (kStateOnly) return 0.0f;
            float4 cq[NS / 4];
#pragma unroll
            for (int v = 0; v < NS / 4; ++v) cq[v] = *reinterpret_cast<const float4*>(Cp + r * NP + 4 * v);
            // two independent fma chains
            float2 ya = mul2(h[0], make_float2(cq[0].x, cq[0].y));
            float2 yb = mul2(h[1], make_float2(cq[0].z, cq[0].w));
#pragma unroll
            for (int v = 1; v < NS / 4; ++v) {
                ya = fma2(h[2 * v], make_float2(cq[v].x, cq[v].y), ya);
                yb = fma2(h[2 * v + 1], make_float2(cq[v].z, cq[v].w), yb);
            }
            const float2 y2 = add2(ya, yb);
            return y2.x + y2.y;
        };
        // Rows beyond d_inner are computed on zero-filled tiles and never stored.  The
        // store is predicated in PTX: a branch around it would put a convergence
        // barrier into the hot block for every row.
        auto store_y = [&](int r, float v) {
            Tact* ptr = yg + (static_cast<long long>(b) * T + t0 + r) * p.ld_y + d;
            const Tact tv = from_f<Tact>(v);
            if constexpr (sizeof(Tact) == 2) {
                unsigned short bits;
                memcpy(&bits, &tv, 2);
                asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %2, 0;\n\t@q st.global.b16 [%0], %1;\n\t}" ::"l"(ptr),
                             "h"(bits), "r"(static_cast<int>(d_ok))
                             : "memory");
            } else {
                float fv;
                memcpy(&fv, &tv, 4);
                asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.s32 q, %2, 0;\n\t@q st.global.f32 [%0], %1;\n\t}" ::"l"(ptr),
                             "f"(fv), "r"(static_cast<int>(d_ok))
                             : "memory");
            }
        };
        // A full block of RB rows starting at r0: el holds the elementwise values of the
        // rows this lane owns, pp what every row's recurrence needs.
        auto block = [&](auto geo_tag, int r0, const Elem* el, const Prep* pp) {
            float yp[RB];
#pragma unroll
            for (int i = 0; i < RB; ++i) yp[i] = step(geo_tag, pp[i], r0 + i);
            if (kStateOnly) {
#pragma unroll
                for (int k = 0; k < OWN; ++k)
                    if (LPC < RB || part < RB) sum_dl += el[k].dl;
                return;
            }
            if constexpr (LPC == 1) {
#pragma unroll
                for (int i = 0; i < RB; ++i) store_y(r0 + i, fmaf(yp[i], el[i].g, el[i].sk));
            } else if constexpr (LPC == 2) {
                // rows 2k (owner part 0) and 2k+1 (part 1): each lane sends the partial
                // the other one finishes; one shuffle per row pair
#pragma unroll
                for (int k = 0; k < RB / 2; ++k) {
                    const float send = part ? yp[2 * k] : yp[2 * k + 1];
                    const float mine = part ? yp[2 * k + 1] : yp[2 * k];
                    const float y = mine + __shfl_xor_sync(0xffffffffu, send, 1);
                    store_y(r0 + 2 * k + part, fmaf(y, el[k].g, el[k].sk));
                }
            } else {
#pragma unroll
                for (int i = 0; i < RB; ++i) {
                    const int owner = LPC >= RB ? i : i % LPC, k = LPC >= RB ? 0 : i / LPC;
                    float y = yp[i];
#pragma unroll
                    for (int m = 1; m < LPC; m <<= 1) y += __shfl_xor_sync(0xffffffffu, y, m);
                    if (part == owner) store_y(r0 + i, fmaf(y, el[k].g, el[k].sk));
                }
            }
        };
        // One row, every lane doing its own elementwise work (sequence start with a
        // carried conv window; ragged last chunk).
        auto single = [&](auto geo_tag, int r) {
            const Elem e1 = elem(std::true_type{}, r);
            float y = step(geo_tag, prep_row(geo_tag, e1.dl, e1.du), r);
            if (kStateOnly) {
                if (part == 0) sum_dl += e1.dl;
                return;
            }
#pragma unroll
            for (int m = 1; m < LPC; m <<= 1) y += __shfl_xor_sync(0xffffffffu, y, m);
            if (part == 0) store_y(r, fmaf(y, e1.g, e1.sk));
        };
        auto run = [&](auto geo_tag) {
            // rows whose conv window reaches before step 0 take the one-row path
            int r_fast = 0;
            if (kConv && t0 < kKMax - 1) r_fast = min(nv, ((kKMax - 1 - t0) + RB - 1) / RB * RB);
            for (int r = 0; r < r_fast; ++r) single(geo_tag, r);
            const int r_full = r_fast + (nv - r_fast) / RB * RB;  // end of the whole blocks
            // Three stages run interleaved, each on its own block of rows, so that no
            // instruction waits on the chain before it:
            //   elementwise of block k+2 | shuffles + decay seeds of block k+1 |
            //   recurrence and output of block k.
            // Full unrolling is kept to the kernels that carry the throughput (d_state <= 16,
            // no fused conv, not the state-only pass): it multiplies their code size by 8.
            constexpr bool kUnroll = LPC <= 2 && !kConv && !kStateOnly;
            if (kUnroll && r_fast == 0 && nv == TC) {
                // a whole chunk: fully unrolled, the stage hand-over is register renaming
                constexpr int NB = TC / RB;
                Elem el[NB + 2][OWN];
                Prep pp[NB + 1][RB];
                elem_block(0, el[0]);
                elem_block(RB, el[1]);
                prep_block(geo_tag, el[0], pp[0]);
#pragma unroll
                for (int k = 0; k < NB; ++k) {
                    if (k + 2 < NB) elem_block((k + 2) * RB, el[k + 2]);
                    if (k + 1 < NB) prep_block(geo_tag, el[k + 1], pp[k + 1]);
                    block(geo_tag, k * RB, el[k], pp[k]);
                }
            } else if (r_full > r_fast) {
                // ragged chunk: a rolled loop; past the last block the early stages redo
                // the last one (clamped row)
                const int r_last = r_full - RB;
                Elem e0[OWN], e1[OWN], e2[OWN];
                Prep p0[RB], p1[RB];
                elem_block(r_fast, e0);
                elem_block(min(r_fast + RB, r_last), e1);
                prep_block(geo_tag, e0, p0);
#pragma unroll 1
                for (int r0 = r_fast; r0 < r_full; r0 += RB) {
                    elem_block(min(r0 + 2 * RB, r_last), e2);
                    prep_block(geo_tag, e1, p1);
                    block(geo_tag, r0, e0, p0);
#pragma unroll
                    for (int k = 0; k < OWN; ++k) {
                        e0[k] = e1[k];
                        e1[k] = e2[k];
                    }
#pragma unroll
                    for (int i = 0; i < RB; ++i) p0[i] = p1[i];
                }
            }
            for (int r = r_full; r < nv; ++r) single(geo_tag, r);
        };
        if (geo) run(std::true_type{});
        else run(std::false_type{});

        // Conv window after the sequence: the K most recent inputs, oldest first.
        if (kConv && !kStateOnly && p.conv_state && c == nch - 1 && seg == nseg - 1 && part == 0 && d_ok) {
            float nw[kKMax];
#pragma unroll
            for (int k = 0; k < kKMax; ++k) {
                const int tg = T - K + k;  // global step held by slot k
                float v = 0.0f;
                if (k < K) {
                    if (tg >= 0) v = to_f(xt[(tg - t0) * DT]);
                    else v = p.conv_in ? p.conv_in[(static_cast<long long>(b) * D + d) * K + K + tg] : 0.0f;
                }
                nw[k] = v;
            }
#pragma unroll
            for (int k = 0; k < kKMax; ++k)
                if (k < K) p.conv_state[(static_cast<long long>(b) * D + d) * K + k] = nw[k];
        }
        mbar_arrive(&empty[s]);  // every lane: its reads of the stage are done
    }

    if (!alive) return;
    // Final recurrent state (the last segment's), or the segment hand-over.
    float* hout = nullptr;
    if (kStateOnly) hout = p.seg_states + ((static_cast<long long>(b) * nseg + seg) * D) * N;
    else if (p.ssm_state && seg == nseg - 1) hout = p.ssm_state + (static_cast<long long>(b) * D) * N;
    if (hout) {
#pragma unroll
        for (int j = 0; j < NS; ++j) {
            const int n = n0 + j;
            if (d_ok && n < N) hout[static_cast<long long>(d) * N + n] = (j & 1) ? h[j / 2].y : h[j / 2].x;
        }
    }
    if (kStateOnly) {
        // owners of the elementwise rows hold partial sums: add them over the channel's lanes
#pragma unroll
        for (int m = 1; m < LPC; m <<= 1) sum_dl += __shfl_xor_sync(0xffffffffu, sum_dl, m);
        if (part == 0 && d_ok) p.seg_sumdl[(static_cast<long long>(b) * nseg + seg) * D + d] = sum_dl;
    }
}

typedef void (*FwdKernelFn)(const FwdParams);

struct FwdVariant {
    int ns, lpc, dt, tc, threads;
    size_t smem;          // dynamic shared memory of this dtype's layout
    FwdKernelFn fn[16];   // by FLAGS
};

template <typename Tr, typename Tact, int... F>
static void fill_flags(FwdKernelFn* out, std::integer_sequence<int, F...>) {
    ((out[F] = sscan_fwd_kernel<Tr, Tact, F>), ...);
}

// Chunk length by storage size: 32 steps of 16-bit tiles, 16 steps of f32 tiles keep
// a CTA near 58 KB of shared memory at d_state 16, so three CTAs share an SM; 16
// steps at d_state > 128, whose B / C rows alone fill the stages.
template <typename Tact, int NS, int LPC, int CW>
static FwdVariant make_variant() {
    using Tr = FwdTraits<Tact, NS, LPC, CW, (sizeof(Tact) == 2 && NS * LPC < 256) ? 32 : 16, 3>;
    FwdVariant v;
    memset(&v, 0, sizeof(v));
    v.ns = NS; v.lpc = LPC; v.dt = Tr::DT; v.tc = Tr::TC; v.threads = Tr::THREADS;
    v.smem = Tr::SMEM;
    // FLAGS 0-7: softplus / gate / conv combinations; 8, 9, 12, 13: state-only passes
    fill_flags<Tr, Tact>(v.fn, std::integer_sequence<int, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 12, 13>{});
    return v;
}

// Variants of one storage dtype, ordered by padded d_state (8 states per lane).
template <typename Tact>
static int build_fwd_variants(FwdVariant* v) {
    int n = 0;
    v[n++] = make_variant<Tact, 8, 1, 4>();    // d_state <= 8
    v[n++] = make_variant<Tact, 8, 2, 4>();    // <= 16
    v[n++] = make_variant<Tact, 8, 4, 4>();    // <= 32
    v[n++] = make_variant<Tact, 8, 8, 4>();    // <= 64
    v[n++] = make_variant<Tact, 8, 16, 8>();   // <= 128
    v[n++] = make_variant<Tact, 8, 32, 8>();   // <= 256
    return n;
}

constexpr int kMaxFwdVariants = 8;
// One translation unit per storage dtype defines its table (parallel builds).
int fwd_variants_f32(FwdVariant* v);
int fwd_variants_f16(FwdVariant* v);
int fwd_variants_bf16(FwdVariant* v);

}  // namespace mb200
