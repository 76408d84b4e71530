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
#pragma once
#include <string.h>

#include <type_traits>
#include <utility>

#include "common.cuh"
#include "internal.h"

namespace mb200 {

constexpr int kKMax = 8;  // widest supported d_conv

#ifndef MB200_FWD_F32BC
#define MB200_FWD_F32BC 1
#endif

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
    int seg_chunks;     // chunks per time segment (grid.z segments); 0 = one segment
    unsigned tma_mask;  // bit0 x, bit1 delta, bit2 z, bit3 B, bit4 C, bit5 y
    int* status;
};

enum : unsigned { kTmaX = 1, kTmaDl = 2, kTmaZ = 4, kTmaB = 8, kTmaC = 16, kTmaY = 32 };

template <typename Tact, int NS_, int LPC_, int WARPS_, int TC_>
struct FwdTraits {
    static constexpr int NS = NS_, LPC = LPC_, WARPS = WARPS_, TC = TC_;
    static constexpr int THREADS = WARPS * 32;
    static constexpr int DT = THREADS / LPC;  // channels per CTA (one lane group per channel)
    static constexpr int NP = NS * LPC;       // padded d_state
    static constexpr int STAGES = 3;
    // 16-bit B / C are widened to f32 once per chunk and CTA (every lane of the
    // CTA would otherwise repeat the widening at each step); large d_state keeps
    // the storage dtype to bound shared memory.
    static constexpr bool F32BC = MB200_FWD_F32BC && sizeof(Tact) == 2 && NS_ * LPC_ <= 64;
    using Tbc = typename std::conditional<F32BC, float, Tact>::type;
    static constexpr size_t al(size_t v) { return (v + 127) & ~size_t(127); }
    static constexpr size_t RAW_ACT = al(sizeof(Tact) * TC * DT);
    static constexpr size_t RAW_BC = al(sizeof(Tact) * TC * NP);
    static constexpr size_t STAGE = 3 * RAW_ACT + 2 * RAW_BC;
    static constexpr size_t OFF_RAW = 0;
    static constexpr size_t BC_COPY = al(sizeof(Tbc) * TC * NP);
    static constexpr size_t OFF_BS = OFF_RAW + STAGES * STAGE;  // B [TC][NP] widened / zero-padded copy
    static constexpr size_t OFF_CS = OFF_BS + BC_COPY;          // C [TC][NP]
    static constexpr size_t OFF_OUT = OFF_CS + BC_COPY;         // 2 x Tact y [TC][DT]
    static constexpr size_t OFF_HALO = OFF_OUT + 2 * RAW_ACT;                // f32 conv window [kKMax][DT]
    static constexpr size_t OFF_BAR = OFF_HALO + al(sizeof(float) * kKMax * DT);  // STAGES mbarriers
    static constexpr size_t SMEM = OFF_BAR + 128;
    // Timesteps per block of the hot loop, and how the per-(t, channel)
    // elementwise work is spread: with 2 or 4 lanes per channel each lane does
    // it for the rows r = part (mod LPC) of a block and the results are
    // exchanged with shuffles; otherwise every lane repeats it.
    static constexpr int RB = 4;
    static constexpr bool SHARE = (LPC == 2 || LPC == 4);
    static constexpr int OWN = SHARE ? RB / LPC : RB;
    static_assert(NS == 4 || NS == 8 || NS == 16, "state slice must be 4, 8 or 16");
    static_assert((LPC & (LPC - 1)) == 0 && LPC <= 32, "LPC must be a power of two");
    static_assert(TC % 4 == 0, "chunk must be a multiple of the 4-step block");
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

template <typename To, typename Ti>
__device__ __forceinline__ To bc_cast(Ti v) {
    if constexpr (std::is_same<To, Ti>::value) return v;
    else return to_f(v);
}

// FLAGS (compile-time, so that the hot block is one branch-free basic block):
//   bit0 softplus on delta, bit1 gate present, bit2 conv1d + SiLU on x.
template <typename Tr, typename Tact, int FLAGS>
__global__ void __launch_bounds__(Tr::THREADS)
sscan_fwd_kernel(const __grid_constant__ FwdParams p) {
    constexpr bool kSoftplus = (FLAGS & 1) != 0, kGate = (FLAGS & 2) != 0, kConv = (FLAGS & 4) != 0;
    constexpr int NS = Tr::NS, LPC = Tr::LPC, TC = Tr::TC, DT = Tr::DT, NP = Tr::NP,
                  THREADS = Tr::THREADS, STAGES = Tr::STAGES;
    constexpr int RB = Tr::RB, OWN = Tr::OWN;
    constexpr bool SHARE = Tr::SHARE;
    extern __shared__ __align__(128) unsigned char smem[];
    using Tbc = typename Tr::Tbc;
    constexpr bool F32BC = Tr::F32BC;
    Tbc* Bs = reinterpret_cast<Tbc*>(smem + Tr::OFF_BS);
    Tbc* Cs = reinterpret_cast<Tbc*>(smem + Tr::OFF_CS);
    float* halo = reinterpret_cast<float*>(smem + Tr::OFF_HALO);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Tr::OFF_BAR);

    const int tid = threadIdx.x;
    const int b = blockIdx.y;
    const int d0 = blockIdx.x * DT;
    const int T = p.T, D = p.D, N = p.N, K = kConv ? p.K : 0;
    const int nchunks = (T + TC - 1) / TC;
    // Time segments: CTA z produces y for chunks [c_begin, c_end) and first
    // replays chunks [0, c_begin) without output (state only) to get its
    // entering state.  That costs extra arithmetic but multiplies the number
    // of warps in flight when batch x channels alone cannot fill the GPU.
    const int c_begin = p.seg_chunks > 0 ? min(nchunks, static_cast<int>(blockIdx.z) * p.seg_chunks) : 0;
    const int c_end = (p.seg_chunks > 0 && blockIdx.z + 1 < gridDim.z)
                          ? min(nchunks, (static_cast<int>(blockIdx.z) + 1) * p.seg_chunks)
                          : nchunks;
    const bool last_seg = blockIdx.z + 1 == gridDim.z;
    const unsigned load_mask = p.tma_mask & (kTmaX | kTmaDl | kTmaZ | kTmaB | kTmaC);
    constexpr bool has_z = kGate;
    const bool gate_is_silu = p.z_mode == 1;

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
    auto out_tile = [&](int s) { return reinterpret_cast<Tact*>(smem + Tr::OFF_OUT + s * Tr::RAW_ACT); };

    // Bytes one stage receives through TMA (full boxes: out-of-range parts are
    // zero-filled and still counted).
    uint32_t tx_bytes = 0;
    if (load_mask & kTmaX) tx_bytes += sizeof(Tact) * TC * DT;
    if (load_mask & kTmaDl) tx_bytes += sizeof(Tact) * TC * DT;
    if (has_z && (load_mask & kTmaZ)) tx_bytes += sizeof(Tact) * TC * DT;
    if (load_mask & kTmaB) tx_bytes += sizeof(Tact) * TC * N;
    if (load_mask & kTmaC) tx_bytes += sizeof(Tact) * TC * N;

    const uint32_t z_bytes = (has_z && (load_mask & kTmaZ)) ? sizeof(Tact) * TC * DT : 0;
    auto issue_loads = [&](int c) {  // one thread
        const int s = c % STAGES, t0 = c * TC;
        if (tx_bytes == 0) return;
        const bool replay = c < c_begin;  // the gate input is not needed to rebuild the state
        mbar_expect_tx(&bars[s], replay ? tx_bytes - z_bytes : tx_bytes);
        if (load_mask & kTmaX) tma_load_3d(raw_x(s), &p.tm_x, &bars[s], d0, t0, b);
        if (load_mask & kTmaDl) tma_load_3d(raw_dl(s), &p.tm_dl, &bars[s], d0, t0, b);
        if (z_bytes && !replay) tma_load_3d(raw_z(s), &p.tm_z, &bars[s], d0, t0, b);
        if (load_mask & kTmaB) tma_load_3d(raw_b(s), &p.tm_b, &bars[s], 0, t0, b);
        if (load_mask & kTmaC) tma_load_3d(raw_c(s), &p.tm_c, &bars[s], 0, t0, b);
    };

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (tid == 0) {
        if (c_end > 0) issue_loads(0);
        if (c_end > 1) issue_loads(1);
    }

    // ---- ownership: LPC lanes per channel, NS states per lane ----
    // Up to 16 states live in one lane (LPC = 1: no shuffles, no divergence);
    // larger d_state spreads a channel over LPC lanes that all repeat the cheap
    // per-(t, channel) elementwise work and reduce y with shuffles.
    const int col = tid / LPC, part = tid % LPC;
    const int d = d0 + col;
    const bool d_ok = d < D;
    const int n0 = part * NS;
    float2 h[NS / 2];
    float2 a2[NS / 2];  // a_neg * log2(e)
    bool geo_local = true;
    {
        float av[NS], hv[NS];
#pragma unroll
        for (int j = 0; j < NS; ++j) {
            const int n = n0 + j;
            const bool ok = d_ok && n < N;
            av[j] = ok ? p.a_neg[static_cast<long long>(d) * N + n] * kLog2e : 0.0f;
            hv[j] = (ok && p.ssm_state) ? p.ssm_state[(static_cast<long long>(b) * D + d) * N + n]
                                        : 0.0f;
        }
        // Arithmetic-progression test a[n] = a[n0] + (n-n0)*step, to 4 ulp: then
        // exp(delta*a[n]) = E * R^(n-n0) and a step needs 2-3 exp2 instead of NS.
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
    const float a2_mid = a2[NS / 4].x;  // second seed of the power chain (NS == 16)
    (void)a2_mid;
    const float Dd = d_ok ? p.Dp[d] : 0.0f;
    // conv taps in registers; the window of the K most recent x values per
    // channel (oldest -> newest) lives in shared memory between chunks.
    float cw[kKMax];
    float cb = 0.0f;
#pragma unroll
    for (int k = 0; k < kKMax; ++k)
        cw[k] = (k < K && d_ok) ? p.conv_w[static_cast<long long>(d) * K + k] : 0.0f;
    if (K && d_ok) cb = p.conv_b[d];
    if (kConv) {
        for (int i = tid; i < kKMax * DT; i += THREADS) {
            const int k = i / DT, cc = i - k * DT;
            float hv = 0.0f;
            if (k < K && d0 + cc < D && p.conv_state)
                hv = p.conv_state[(static_cast<long long>(b) * D + d0 + cc) * K + k];
            halo[i] = hv;
        }
        __syncthreads();
    }
    const int lane_base = (tid & 31) & ~(LPC - 1);  // lane holding slice 0 of this channel

    const long long save_chunks = p.chunk_states ? (T + p.save_stride - 1) / p.save_stride : 0;

    // Per-timestep values produced by the elementwise stage.
    struct Elem {
        float dl, du, g, sk;
    };

    for (int c = 0; c < c_end; ++c) {
        const int s = c % STAGES, t0 = c * TC;
        const int nv = min(TC, T - t0);
        const bool replay = c < c_begin;
        if (tid == 0 && c + 2 < c_end) issue_loads(c + 2);
        // Tensors that could not be described to TMA: cooperative plain loads.
        const bool any_plain = load_mask != (kTmaX | kTmaDl | kTmaZ | kTmaB | kTmaC);
        if (any_plain) {
            if (!(load_mask & kTmaX))
                load_tile_plain(raw_x(s), static_cast<const Tact*>(p.x), p.ld_x, b, T, t0, d0, D, TC,
                                DT, THREADS);
            if (!(load_mask & kTmaDl))
                load_tile_plain(raw_dl(s), static_cast<const Tact*>(p.dl), p.ld_dl, b, T, t0, d0, D,
                                TC, DT, THREADS);
            if (has_z && !replay && !(load_mask & kTmaZ))
                load_tile_plain(raw_z(s), static_cast<const Tact*>(p.z), p.ld_z, b, T, t0, d0, D, TC,
                                DT, THREADS);
            if (!(load_mask & kTmaB))
                load_tile_plain(raw_b(s), static_cast<const Tact*>(p.bm), p.ld_bc, b, T, t0, 0, N,
                                TC, N, THREADS);
            if (!(load_mask & kTmaC))
                load_tile_plain(raw_c(s), static_cast<const Tact*>(p.cm), p.ld_bc, b, T, t0, 0, N,
                                TC, N, THREADS);
        }
        // the y buffer written in this iteration was last stored two chunks ago:
        // wait until that bulk store has finished reading it (one store may stay
        // in flight); the barrier that follows orders this before any write.
        if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        if (tx_bytes) mbar_wait(&bars[s], (c / STAGES) & 1, p.status);
        __syncthreads();

        // B / C: 16-bit tiles are widened to f32 once per chunk (F32BC); otherwise the
        // recurrence reads the landed tile in its storage dtype, and only a d_state
        // that is not a whole number of lane slices needs a zero-padded copy.
        const bool padded = N != NP;
        if (F32BC && !padded) {
            const uint4* rb = reinterpret_cast<const uint4*>(raw_b(s));
            const uint4* rc = reinterpret_cast<const uint4*>(raw_c(s));
            for (int i = tid; i < TC * NP / 8; i += THREADS) {
                StateVec<Tact, 8> vb, vc;
                vb.load(reinterpret_cast<const Tact*>(rb + i));
                vc.load(reinterpret_cast<const Tact*>(rc + i));
                float4* ob = reinterpret_cast<float4*>(Bs) + 2 * i;
                float4* oc = reinterpret_cast<float4*>(Cs) + 2 * i;
                const float2 b0 = vb.pair(0), b1 = vb.pair(1), b2 = vb.pair(2), b3 = vb.pair(3);
                const float2 c0 = vc.pair(0), c1 = vc.pair(1), c2 = vc.pair(2), c3 = vc.pair(3);
                ob[0] = make_float4(b0.x, b0.y, b1.x, b1.y);
                ob[1] = make_float4(b2.x, b2.y, b3.x, b3.y);
                oc[0] = make_float4(c0.x, c0.y, c1.x, c1.y);
                oc[1] = make_float4(c2.x, c2.y, c3.x, c3.y);
            }
            __syncthreads();
        } else if (F32BC || padded) {
            const Tact* rb = raw_b(s);
            const Tact* rc = raw_c(s);
            for (int i = tid; i < TC * NP; i += THREADS) {
                const int r = i / NP, n = i - r * NP;
                Bs[i] = n < N ? bc_cast<Tbc>(rb[r * N + n]) : bc_cast<Tbc>(from_f<Tact>(0.0f));
                Cs[i] = n < N ? bc_cast<Tbc>(rc[r * N + n]) : bc_cast<Tbc>(from_f<Tact>(0.0f));
            }
            __syncthreads();
        }

        // Training save: state entering each block of save_stride steps.
        if (p.chunk_states && !replay && (t0 % p.save_stride) == 0) {
            const long long sc = t0 / p.save_stride;
#pragma unroll
            for (int j = 0; j < NS; ++j) {
                const int n = n0 + j;
                if (d_ok && n < N)
                    p.chunk_states[((static_cast<long long>(b) * save_chunks + sc) * D + d) * N + n] =
                        (j & 1) ? h[j / 2].y : h[j / 2].x;
            }
        }

        const Tact* rx = raw_x(s) + col;
        const Tact* rd = raw_dl(s) + col;
        const Tact* rz = raw_z(s) + col;
        const float* hl = halo + col;
        Tact* ot = out_tile(c & 1) + col;
        const Tbc* Bp = ((F32BC || padded) ? Bs : reinterpret_cast<const Tbc*>(raw_b(s))) + n0;
        const Tbc* Cp = ((F32BC || padded) ? Cs : reinterpret_cast<const Tbc*>(raw_c(s))) + n0;

        // Elementwise stage of one timestep (row r of the chunk).
        auto elem = [&](auto replay_tag, int r) -> Elem {
            constexpr bool RP = decltype(replay_tag)::value;
            float u;
            if (kConv) {
                float acc = cb;
#pragma unroll
                for (int k = 0; k < kKMax; ++k) {
                    // tap k reads x[r - (K-1) + k]: this chunk's tile, or the window
                    // carried from the previous chunk for the first K-1 rows.
                    const int rr = r - (K - 1) + k;
                    const float a = to_f(rx[max(rr, 0) * DT]);
                    const float w = hl[min(max(K + rr, 0), kKMax - 1) * DT];
                    acc = fmaf(rr >= 0 ? a : w, cw[k], acc);  // cw[k] == 0 for k >= K
                }
                u = siluf_fast(acc);
                if (!RP && p.u_out && d_ok)
                    static_cast<Tact*>(p.u_out)[(static_cast<long long>(b) * T + t0 + r) * p.ld_u + d] =
                        from_f<Tact>(u);
            } else {
                u = to_f(rx[r * DT]);
            }
            float dv = to_f(rd[r * DT]);
            if (kSoftplus) dv = softplusf_fast(dv);
            float gv = 1.0f;
            if (kGate && !RP) {
                const float zv = to_f(rz[r * DT]);
                const float sz = siluf_fast(zv);
                gv = gate_is_silu ? sz : zv;  // select, not a branch
            }
            Elem o;
            o.dl = dv;
            o.du = dv * u;
            o.g = gv;
            o.sk = Dd * u * gv;
            return o;
        };
        // Elementwise work this lane owns in the block starting at row r0.
        auto elem_block = [&](auto replay_tag, int r0, Elem* out) {
#pragma unroll
            for (int k = 0; k < OWN; ++k) out[k] = elem(replay_tag, SHARE ? r0 + k * LPC + part : r0 + k);
        };

        // Recurrence of the block at row r0 (NB = RB), or of the single row r0
        // (NB = 1, ragged last chunk; `el` then holds that row for every lane).
        auto recur = [&](auto geo_tag, auto replay_tag, auto nb_tag, int r0, const Elem* el) {
            constexpr bool GEO = decltype(geo_tag)::value;
            constexpr bool RP = decltype(replay_tag)::value;
            constexpr int NB = decltype(nb_tag)::value;
            constexpr bool SH = SHARE && NB == RB;
            StateVec<Tbc, NS> Bq[NB], Cq[NB];
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                Bq[i].load(Bp + (r0 + i) * NP);
                if (!RP) Cq[i].load(Cp + (r0 + i) * NP);
            }
            float yo[NB];
#pragma unroll
            for (int i = 0; i < NB; ++i) {
                // (delta, delta*u) of row i: from the lane that owns the row
                const int k = SH ? i / LPC : i;
                float dli = el[k].dl, dui = el[k].du;
                if (SH) {
                    dli = __shfl_sync(0xffffffffu, dli, lane_base + (i % LPC));
                    dui = __shfl_sync(0xffffffffu, dui, lane_base + (i % LPC));
                }
                float2 e[NS / 2];
                if (GEO) {
                    // e[j] = (E R^(2j), E R^(2j+1)): product tree of depth <= 3,
                    // re-seeded at the middle state when NS == 16.
                    const float R = ex2(dli * a2_step);
                    const float R2 = R * R;
                    const float2 r2 = splat2(R2), r4 = splat2(R2 * R2);
                    const float E0 = ex2(dli * a2_first);
                    e[0] = make_float2(E0, E0 * R);
                    e[1] = mul2(e[0], r2);
                    if (NS >= 8) {
                        e[2] = mul2(e[0], r4);
                        e[3] = mul2(e[1], r4);
                    }
                    if (NS == 16) {
                        const float E1 = ex2(dli * a2_mid);
                        e[4] = make_float2(E1, E1 * R);
                        e[5] = mul2(e[4], r2);
                        e[6] = mul2(e[4], r4);
                        e[7] = mul2(e[5], r4);
                    }
                } else {
                    const float2 dl2 = splat2(dli);
#pragma unroll
                    for (int j = 0; j < NS / 2; ++j) {
                        const float2 xa = mul2(dl2, a2[j]);
                        e[j] = make_float2(ex2(xa.x), ex2(xa.y));
                    }
                }
                const float2 du2 = splat2(dui);
                float2 dub[NS / 2];
#pragma unroll
                for (int j = 0; j < NS / 2; ++j) dub[j] = mul2(du2, Bq[i].pair(j));
#pragma unroll
                for (int j = 0; j < NS / 2; ++j) h[j] = fma2(e[j], h[j], dub[j]);
                if (RP) continue;  // state only
                // y = <h, C>: two independent fma chains
                float2 ya = mul2(h[0], Cq[i].pair(0));
                float2 yb = mul2(h[1], Cq[i].pair(1));
#pragma unroll
                for (int j = 1; j < NS / 4; ++j) {
                    ya = fma2(h[2 * j], Cq[i].pair(2 * j), ya);
                    yb = fma2(h[2 * j + 1], Cq[i].pair(2 * j + 1), yb);
                }
                const float2 y2 = add2(ya, yb);
                float y = y2.x + y2.y;
#pragma unroll
                for (int m = 1; m < LPC; m <<= 1) y += __shfl_xor_sync(0xffffffffu, y, m);
                // gate and skip are applied by the lane that owns the row
                yo[i] = fmaf(y, el[k].g, el[k].sk);
            }
            // Stores after every load of the block.
            if (!RP) {
#pragma unroll
                for (int i = 0; i < NB; ++i)
                    if (part == (SH ? i % LPC : 0)) ot[(r0 + i) * DT] = from_f<Tact>(yo[i]);
            }
        };
        auto run = [&](auto geo_tag, auto replay_tag) {
            if (nv == TC) {
                Elem cur[OWN], nxt[OWN];
                elem_block(replay_tag, 0, cur);
                // Every iteration but the last also does the elementwise work of the
                // following block; it is independent of this block's recurrence and
                // sits in the same basic block, so the two interleave.
#pragma unroll 1
                for (int r0 = 0; r0 < TC - RB; r0 += RB) {
                    elem_block(replay_tag, r0 + RB, nxt);
                    recur(geo_tag, replay_tag, std::integral_constant<int, RB>{}, r0, cur);
#pragma unroll
                    for (int k = 0; k < OWN; ++k) cur[k] = nxt[k];
                }
                recur(geo_tag, replay_tag, std::integral_constant<int, RB>{}, TC - RB, cur);
            } else {
#pragma unroll 1
                for (int r0 = 0; r0 < nv; ++r0) {
                    Elem one = elem(replay_tag, r0);  // every lane: no sharing on the ragged tail
                    recur(geo_tag, replay_tag, std::integral_constant<int, 1>{}, r0, &one);
                }
            }
        };
        if (replay) {
            if (geo) run(std::true_type{}, std::true_type{});
            else run(std::false_type{}, std::true_type{});
        } else {
            if (geo) run(std::true_type{}, std::false_type{});
            else run(std::false_type{}, std::false_type{});
        }

        // ---------------- store the y tile ----------------
        if (replay) {
            __syncthreads();  // every reader of this stage is done before it is refilled
        } else if (p.tma_mask & kTmaY) {
            fence_proxy_async();
            __syncthreads();
            if (tid == 0) {
                tma_store_3d(&p.tm_y, out_tile(c & 1), d0, t0, b);
                tma_commit();
            }
        } else {
            __syncthreads();
            Tact* yb = static_cast<Tact*>(p.y);
            const Tact* o = out_tile(c & 1);
            for (int i = tid; i < nv * DT; i += THREADS) {
                const int r = i / DT, cidx = i - r * DT;
                if (d0 + cidx < D)
                    yb[(static_cast<long long>(b) * T + t0 + r) * p.ld_y + d0 + cidx] = o[i];
            }
        }
        // Conv window hand-over: the K most recent x values per channel.  Readers
        // of the old window finished before the barrier above; the next chunk's
        // first read comes after its own barrier.
        if (kConv) {
            const Tact* rxs = raw_x(s);
            for (int i = tid; i < DT; i += THREADS) {
                float nw[kKMax];
#pragma unroll
                for (int k = 0; k < kKMax; ++k) {
                    const int rr = nv - K + k;  // row of this chunk, or negative: old window
                    nw[k] = (k < K) ? (rr >= 0 ? to_f(rxs[max(rr, 0) * DT + i])
                                               : halo[min(max(K + rr, 0), kKMax - 1) * DT + i])
                                    : 0.0f;
                }
#pragma unroll
                for (int k = 0; k < kKMax; ++k) halo[k * DT + i] = nw[k];
            }
            __syncthreads();  // the window is read by other threads in the next chunk
        }
    }

    // Final recurrent state and conv window.
    if (p.ssm_state && last_seg) {
#pragma unroll
        for (int j = 0; j < NS; ++j) {
            const int n = n0 + j;
            if (d_ok && n < N)
                p.ssm_state[(static_cast<long long>(b) * D + d) * N + n] =
                    (j & 1) ? h[j / 2].y : h[j / 2].x;
        }
    }
    if (kConv && p.conv_state && last_seg) {
        __syncthreads();
        for (int i = tid; i < DT; i += THREADS)
            if (d0 + i < D)
                for (int k = 0; k < K; ++k)
                    p.conv_state[(static_cast<long long>(b) * D + d0 + i) * K + k] = halo[k * DT + i];
    }
    if (tid == 0) tma_wait_read0();  // shared memory must outlive the last bulk store
}

typedef void (*FwdKernelFn)(const FwdParams);

struct FwdVariant {
    int ns, lpc, dt, tc, threads;
    size_t smem;          // dynamic shared memory of this dtype's layout
    FwdKernelFn fn[8];    // by FLAGS
};

#ifndef MB200_FWD_WARPS
#define MB200_FWD_WARPS 2
#endif
#ifndef MB200_FWD_TC
#define MB200_FWD_TC 32
#endif

template <typename Tr, typename Tact, int... F>
static void fill_flags(FwdKernelFn* out, std::integer_sequence<int, F...>) {
    ((out[F] = sscan_fwd_kernel<Tr, Tact, F>), ...);
}

template <typename Tact, int NS, int LPC>
static FwdVariant make_variant() {
    using Tr = FwdTraits<Tact, NS, LPC, MB200_FWD_WARPS, MB200_FWD_TC>;
    FwdVariant v;
    memset(&v, 0, sizeof(v));
    v.ns = NS; v.lpc = LPC; v.dt = Tr::DT; v.tc = Tr::TC; v.threads = Tr::THREADS;
    v.smem = Tr::SMEM;
#ifdef MB200_FWD_TUNING  // tuning builds: compat (0) and fused-no-conv (3) only
    fill_flags<Tr, Tact>(v.fn, std::integer_sequence<int, 0, 3>{});
#else
    fill_flags<Tr, Tact>(v.fn, std::make_integer_sequence<int, 8>{});
#endif
    return v;
}

// Variants of one storage dtype, ordered by padded d_state: up to 16 states per
// lane; above that LPC lanes share a channel.
template <typename Tact>
static int build_fwd_variants(FwdVariant* v) {
    int n = 0;
#ifndef MB200_FWD_TUNING
    v[n++] = make_variant<Tact, 4, 1>();
    v[n++] = make_variant<Tact, 8, 1>();
#endif
#if defined(MB200_FWD_NS16)
    v[n++] = make_variant<Tact, 16, 1>();
#elif defined(MB200_FWD_NS4)
    v[n++] = make_variant<Tact, 4, 4>();
#else
    v[n++] = make_variant<Tact, 8, 2>();
#endif
#ifndef MB200_FWD_TUNING
    v[n++] = make_variant<Tact, 16, 2>();
    v[n++] = make_variant<Tact, 16, 4>();
    v[n++] = make_variant<Tact, 16, 8>();
    v[n++] = make_variant<Tact, 16, 16>();
#endif
    return n;
}

constexpr int kMaxFwdVariants = 8;
// One translation unit per storage dtype defines its table (parallel builds).
int fwd_variants_f32(FwdVariant* v);
int fwd_variants_f16(FwdVariant* v);
int fwd_variants_bf16(FwdVariant* v);

}  // namespace mb200
