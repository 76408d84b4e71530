// Mamba-1 selective-scan backward, two lanes per channel (8 < d_state <= 16).
//
// Same algorithm as sscan_bwd_kernel (recomputation from the state entering
// each block of S steps), laid out for occupancy and issue rate:
//   * a channel is owned by two lanes (8 states each, lanes l and l+16 of a
//     warp) and a CTA is ONE warp = 16 channels, so twice as many warps exist
//     as with one lane per channel; the CTA needs ~19 KB of shared memory
//     (16-bit storage, S = 32) instead of ~100 KB, so every CTA of a
//     model-sized launch is resident at once (no second wave, ~10 warps per SM)
//     and nothing in the kernel needs more than a warp-level barrier;
//   * sub-blocks are 4 steps long and their 8 states x 4 steps stay in
//     REGISTERS between the forward and the reverse sweep (no shared-memory
//     round trip for h_t); the kernel is capped at 168 registers so that three
//     warps fit each scheduler's 16K-register file (12 per SM);
//   * all state arithmetic is packed f32x2;
//   * softplus(delta) and dy*gate are computed once per block into shared
//     memory, 16-bit B / C are widened once per block;
//   * dB_t / dC_t are reduced over the warp's 16 channels by a recursive-halving
//     shuffle butterfly (15 shuffles) that leaves one of the 32 sums in each
//     lane: one coalesced 128-byte store per step into the per-channel-tile
//     partials;
//   * du / ddelta / dz leave as 32-byte segments straight from registers; rows are
//     finished in pairs (lanes 0-15 the even row, lanes 16-31 the odd one), so the
//     elementwise output code runs once per two rows without divergence.
// Results differ from the one-lane kernel only by summation order.
#pragma once
#include <string.h>

#include <type_traits>

#include "common.cuh"
#include "internal.h"

namespace mb200 {

// Steps per sub-block of the reverse sweep, and the register cap that lets 11-12
// one-warp CTAs share an SM (both found by measurement on B200).
constexpr int kBwd2SubBlock = 4;
constexpr int kBwd2MaxRegs = 168;

struct BwdParams {
    CUtensorMap tm_u, tm_dl, tm_z, tm_dy, tm_b, tm_c, tm_du, tm_ddl, tm_dz;
    const void *u, *dl, *z, *dy, *bm, *cm;
    void *du, *ddl, *dz;
    long long ld_u, ld_dl, ld_z, ld_dy, ld_bc, ld_du, ld_ddl, ld_dz;
    const float *a_neg, *Dp, *chunk_states;
    // saved state k of sample b starts at chunk_states + b * cs_ld_b + k * cs_ld_k
    // ([B, blocks, D, N] from the fused forward; rows 0, S, 2S... of the reference's
    // h_saved [B, T+1, D, N] through the compat entry point)
    long long cs_ld_b, cs_ld_k;
    float *part_bc;  // [B][tiles][T][2N]
    float *part_a;   // [B][D][N]
    float *part_d;   // [B][D]
    int B, T, D, N, S;
    int z_mode;
    unsigned tma_mask;  // bit per tensor map, in declaration order
    int* status;
};

enum : unsigned {
    kBU = 1, kBDl = 2, kBZ = 4, kBDy = 8, kBB = 16, kBC = 32, kBDu = 64, kBDdl = 128, kBDz = 256
};

typedef void (*BwdKernelFn)(const BwdParams);

template <typename Tact>
__device__ __forceinline__ void bwd_load_plain(Tact* dst, const Tact* src, long long ld, int b, int T,
                                               int t0, int c0, int cols, int rows, int box_cols,
                                               int nthreads = 32) {
    const Tact zero = from_f<Tact>(0.0f);
    for (int i = threadIdx.x; i < rows * box_cols; i += nthreads) {
        int r = i / box_cols, c = i - r * box_cols;
        int t = t0 + r, col = c0 + c;
        Tact v = zero;
        if (t < T && col < cols) v = src[(static_cast<long long>(b) * T + t) * ld + col];
        dst[i] = v;
    }
}

template <typename Tact, int S>
struct Bwd2Traits {
    static constexpr int DT = 16, THREADS = 32, SB = kBwd2SubBlock, NSUB = S / SB, NP = 16;
    static constexpr size_t al(size_t v) { return (v + 127) & ~size_t(127); }
    static constexpr size_t mx(size_t a, size_t b) { return a > b ? a : b; }
    static constexpr size_t ACT = al(sizeof(Tact) * S * DT);
    static constexpr size_t BCR = al(sizeof(Tact) * S * NP);
    // One stage of inputs.  The raw B / C tiles are dead once widened, so the
    // states entering sub-blocks 1.. (sub-block 0 starts from the saved chunk
    // state, re-read from global memory) share their bytes.
    static constexpr size_t OFF_BF = 4 * ACT;                                     // f32 B [S][16]
    static constexpr size_t OFF_CF = OFF_BF + sizeof(float) * S * NP;             // f32 C [S][16]
    static constexpr size_t OFF_DLS = OFF_CF + sizeof(float) * S * NP;            // f32 delta [S][16]
    static constexpr size_t OFF_GY = OFF_DLS + sizeof(float) * S * DT;            // f32 dy*gate [S][16]
    static constexpr size_t OFF_RAWB = OFF_GY + sizeof(float) * S * DT;           // Tact B [S][N]
    static constexpr size_t OFF_RAWC = OFF_RAWB + BCR;                            // Tact C [S][N]
    static constexpr size_t OFF_ENT = OFF_RAWB;                                   // f32 [NSUB-1][8][32]
    static constexpr size_t OFF_BAR = OFF_ENT + mx(2 * BCR, sizeof(float) * (NSUB - 1) * 8 * THREADS);
    static constexpr size_t SMEM = OFF_BAR + 128;
    static_assert(SB % 2 == 0, "rows are finished in pairs");
};

// FLAGS: bit0 softplus on delta, bit1 gate present.
template <typename Tact, int S, int FLAGS>
__global__ void __maxnreg__(kBwd2MaxRegs) sscan_bwd2_kernel(const __grid_constant__ BwdParams p) {
    using Tr = Bwd2Traits<Tact, S>;
    constexpr bool kSoftplus = (FLAGS & 1) != 0, kGate = (FLAGS & 2) != 0;
    constexpr int DT = 16, SB = Tr::SB, NSUB = Tr::NSUB, NP = 16, THREADS = 32;
    extern __shared__ __align__(128) unsigned char smem[];
    float* Bf = reinterpret_cast<float*>(smem + Tr::OFF_BF);
    float* Cf = reinterpret_cast<float*>(smem + Tr::OFF_CF);
    float2* ent = reinterpret_cast<float2*>(smem + Tr::OFF_ENT);  // [NSUB-1][4][32], sub-blocks 1..
    float* dls = reinterpret_cast<float*>(smem + Tr::OFF_DLS);
    float* gy = reinterpret_cast<float*>(smem + Tr::OFF_GY);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Tr::OFF_BAR);
    const int tid = threadIdx.x, lane = tid;
    const int part = lane >> 4, chl = lane & 15;
    const int col = chl;  // channel within the CTA's tile
    const int b = blockIdx.y, tile = blockIdx.x, d0 = tile * DT, d = d0 + col;
    const int n0 = part * 8;
    const int T = p.T, D = p.D, N = p.N;
    const bool d_ok = d < D;
    const int nblk = (T + S - 1) / S;
    const bool gate_is_silu = p.z_mode == 1;

    auto st_u = [&](int s) { return reinterpret_cast<Tact*>(smem + 0 * s); };
    auto st_dl = [&](int s) { return reinterpret_cast<Tact*>(smem + 0 * s + Tr::ACT); };
    auto st_z = [&](int s) { return reinterpret_cast<Tact*>(smem + 0 * s + 2 * Tr::ACT); };
    auto st_dy = [&](int s) { return reinterpret_cast<Tact*>(smem + 0 * s + 3 * Tr::ACT); };
    auto st_b = [&](int s) { return reinterpret_cast<Tact*>(smem + 0 * s + Tr::OFF_RAWB); };
    auto st_c = [&](int s) { return reinterpret_cast<Tact*>(smem + 0 * s + Tr::OFF_RAWC); };
    Tact* g_du = static_cast<Tact*>(p.du);
    Tact* g_ddl = static_cast<Tact*>(p.ddl);
    Tact* g_dz = static_cast<Tact*>(p.dz);

    const unsigned lm = p.tma_mask;
    uint32_t tx_bytes = 0;
    if (lm & kBU) tx_bytes += sizeof(Tact) * S * DT;
    if (lm & kBDl) tx_bytes += sizeof(Tact) * S * DT;
    if (kGate && (lm & kBZ)) tx_bytes += sizeof(Tact) * S * DT;
    if (lm & kBDy) tx_bytes += sizeof(Tact) * S * DT;
    if (lm & kBB) tx_bytes += sizeof(Tact) * S * N;
    if (lm & kBC) tx_bytes += sizeof(Tact) * S * N;
    const unsigned all_loads = kBU | kBDl | kBZ | kBDy | kBB | kBC;
    const bool any_plain = (lm & all_loads) != all_loads;

    auto issue = [&](int k, int s) {  // one thread
        const int t0 = k * S;
        if (!tx_bytes) return;
        mbar_expect_tx(&bars[s], tx_bytes);
        if (lm & kBU) tma_load_3d(st_u(s), &p.tm_u, &bars[s], d0, t0, b);
        if (lm & kBDl) tma_load_3d(st_dl(s), &p.tm_dl, &bars[s], d0, t0, b);
        if (kGate && (lm & kBZ)) tma_load_3d(st_z(s), &p.tm_z, &bars[s], d0, t0, b);
        if (lm & kBDy) tma_load_3d(st_dy(s), &p.tm_dy, &bars[s], d0, t0, b);
        if (lm & kBB) tma_load_3d(st_b(s), &p.tm_b, &bars[s], 0, t0, b);
        if (lm & kBC) tma_load_3d(st_c(s), &p.tm_c, &bars[s], 0, t0, b);
    };

    if (tid == 0) {
        mbar_init(&bars[0], 1);
        fence_barrier_init();
    }
    __syncwarp();

    // per-lane constants: 8 states of one channel
    float2 a2[4];
    bool geo_local = true;
    {
        float av[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            av[j] = (d_ok && n0 + j < N) ? p.a_neg[static_cast<long long>(d) * N + n0 + j] * kLog2e : 0.0f;
        const float step = av[1] - av[0];
#pragma unroll
        for (int j = 2; j < 8; ++j)
            if (fabsf(av[j] - fmaf(static_cast<float>(j), step, av[0])) > 4.8e-7f * fabsf(av[j])) geo_local = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) a2[j] = make_float2(av[2 * j], av[2 * j + 1]);
    }
    const bool geo = __all_sync(0xffffffffu, geo_local ? 1 : 0) != 0;
    const float a2_first = a2[0].x, a2_step = a2[0].y - a2[0].x;
    const float Dd = d_ok ? p.Dp[d] : 0.0f;

    // exp2(delta * a2[j]) for the lane's 8 states
    auto decay = [&](auto geo_tag, float dlv, float2* e) {
        if (decltype(geo_tag)::value) {
            const float R = ex2(dlv * a2_step);
            const float R2 = R * R;
            const float2 r2 = splat2(R2), r4 = splat2(R2 * R2);
            const float E0 = ex2(dlv * a2_first);
            e[0] = make_float2(E0, E0 * R);
            e[1] = mul2(e[0], r2);
            e[2] = mul2(e[0], r4);
            e[3] = mul2(e[1], r4);
        } else {
            const float2 dl2 = splat2(dlv);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 xa = mul2(dl2, a2[j]);
                e[j] = make_float2(ex2(xa.x), ex2(xa.y));
            }
        }
    };

    float2 dh[4], accA[4];
    float accD = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) dh[j] = accA[j] = make_float2(0.0f, 0.0f);

    auto run_blocks = [&](auto geo_tag) {
        for (int it = 0; it < nblk; ++it) {
            const int k = nblk - 1 - it, s = 0, t0 = k * S;
            const int nv = min(S, T - t0);
            // One stage: the previous block's readers finished at the warp barrier that
            // ended it; other resident CTAs cover this load's latency.
            if (tid == 0) issue(k, 0);
            if (any_plain) {
                if (!(lm & kBU)) bwd_load_plain(st_u(s), static_cast<const Tact*>(p.u), p.ld_u, b, T, t0, d0, D, S, DT, THREADS);
                if (!(lm & kBDl)) bwd_load_plain(st_dl(s), static_cast<const Tact*>(p.dl), p.ld_dl, b, T, t0, d0, D, S, DT, THREADS);
                if (kGate && !(lm & kBZ)) bwd_load_plain(st_z(s), static_cast<const Tact*>(p.z), p.ld_z, b, T, t0, d0, D, S, DT, THREADS);
                if (!(lm & kBDy)) bwd_load_plain(st_dy(s), static_cast<const Tact*>(p.dy), p.ld_dy, b, T, t0, d0, D, S, DT, THREADS);
                if (!(lm & kBB)) bwd_load_plain(st_b(s), static_cast<const Tact*>(p.bm), p.ld_bc, b, T, t0, 0, N, S, N, THREADS);
                if (!(lm & kBC)) bwd_load_plain(st_c(s), static_cast<const Tact*>(p.cm), p.ld_bc, b, T, t0, 0, N, S, N, THREADS);
            }
            if (tx_bytes) mbar_wait(&bars[0], it & 1, p.status);
            __syncwarp();

            // ---- 1. per-block elementwise caches ----
            {
                const Tact* rd = st_dl(s);
                const Tact* rdy = st_dy(s);
                const Tact* rz = st_z(s);
                for (int i = tid; i < S * DT; i += THREADS) {
                    const float v = to_f(rd[i]);
                    dls[i] = kSoftplus ? softplusf_fast(v) : v;
                    float g = to_f(rdy[i]);
                    if (kGate) {
                        const float zv = to_f(rz[i]);
                        g *= gate_is_silu ? siluf_fast(zv) : zv;
                    }
                    gy[i] = g;
                }
                const Tact* rb = st_b(s);
                const Tact* rc = st_c(s);
                for (int i = tid; i < S * NP; i += THREADS) {
                    const int r = i / NP, n = i - r * NP;
                    Bf[i] = n < N ? to_f(rb[r * N + n]) : 0.0f;
                    Cf[i] = n < N ? to_f(rc[r * N + n]) : 0.0f;
                }
            }
            __syncwarp();

            const Tact* ru = st_u(s) + col;
            const float* rdl = dls + col;
            const float* rgy = gy + col;
            const float* Bp = Bf + n0;
            const float* Cp = Cf + n0;

            auto fwd_step = [&](int r, float2* h) {
                const float dlv = rdl[r * DT], duv = dlv * to_f(ru[r * DT]);
                float2 e[4];
                decay(geo_tag, dlv, e);
                StateVec<float, 8> Bq;
                Bq.load(Bp + r * NP);
                const float2 du2 = splat2(duv);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = fma2(e[j], h[j], mul2(du2, Bq.pair(j)));
            };

            // ---- 2. state entering each sub-block ----
            const float* cs = p.chunk_states + b * p.cs_ld_b + k * p.cs_ld_k +
                              static_cast<long long>(d_ok ? d : 0) * N + n0;
            auto load_entry = [&](int sb, float2* h) {
                if (sb == 0) {
                    float hv[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) hv[j] = (d_ok && n0 + j < N) ? cs[j] : 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) h[j] = make_float2(hv[2 * j], hv[2 * j + 1]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) h[j] = ent[((sb - 1) * 4 + j) * THREADS + tid];
                }
            };
            float2 h[4];
            load_entry(0, h);
            const int nsub = (nv + SB - 1) / SB;
            for (int sb = 1; sb < nsub; ++sb) {
#pragma unroll
                for (int i = 0; i < SB; ++i) fwd_step((sb - 1) * SB + i, h);
#pragma unroll
                for (int j = 0; j < 4; ++j) ent[((sb - 1) * 4 + j) * THREADS + tid] = h[j];
            }

            // ---- 3. sub-blocks, last to first ----
            for (int sb = nsub - 1; sb >= 0; --sb) {
                const int r_lo = sb * SB;
                float2 hs[SB][4];  // h after step i of the sub-block
                load_entry(sb, h);
#pragma unroll
                for (int i = 0; i < SB; ++i) {
                    fwd_step(r_lo + i, h);
#pragma unroll
                    for (int j = 0; j < 4; ++j) hs[i][j] = h[j];
                }
                float* pbc = p.part_bc + (((static_cast<long long>(b) * gridDim.x + tile) * T) + t0 + r_lo) * 32 +
                             ((chl & 8) ? 16 : 0) + n0 + (chl & 7);
                float hB = 0.0f, hA = 0.0f, hY = 0.0f;  // sums of the odd row of a pair
#pragma unroll
                for (int i = SB - 1; i >= 0; --i) {
                    const int r = r_lo + i;
                    const float dlv = rdl[r * DT], uv = to_f(ru[r * DT]), dyp = rgy[r * DT];
                    const float duv = dlv * uv;
                    float2 e[4];
                    decay(geo_tag, dlv, e);
                    StateVec<float, 8> Bq, Cq;
                    Bq.load(Bp + r * NP);
                    Cq.load(Cp + r * NP);
                    float2 hp[4];
                    if (i > 0) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) hp[j] = hs[i - 1][j];
                    } else {
                        load_entry(sb, hp);
                    }
                    const float2 dyp2 = splat2(dyp), du2 = splat2(duv), dl2 = splat2(dlv);
                    float2 sB2 = make_float2(0.0f, 0.0f), sA2 = sB2, ys2 = sB2;
                    float2 rB[4], rC[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 c = Cq.pair(j);
                        dh[j] = fma2(dyp2, c, dh[j]);
                        sB2 = fma2(dh[j], Bq.pair(j), sB2);
                        const float2 dhda = mul2(dh[j], e[j]);
                        const float2 w = mul2(dhda, hp[j]);
                        sA2 = fma2(a2[j], w, sA2);
                        accA[j] = fma2(dl2, w, accA[j]);
                        rB[j] = mul2(dh[j], du2);
                        rC[j] = mul2(dyp2, hs[i][j]);
                        ys2 = fma2(hs[i][j], c, ys2);
                        dh[j] = dhda;
                    }
                    float sB = sB2.x + sB2.y, sA = sA2.x + sA2.y, ys = ys2.x + ys2.y;
                    sB += __shfl_xor_sync(0xffffffffu, sB, 16);
                    sA += __shfl_xor_sync(0xffffffffu, sA, 16);
                    if (kGate) ys += __shfl_xor_sync(0xffffffffu, ys, 16);
                    // Elementwise outputs, two rows at a time: the sums of the odd row wait
                    // for the even row below it, then lanes 0-15 finish the even row and
                    // lanes 16-31 the odd one with the same instructions.
                    if (i & 1) {
                        hB = sB; hA = sA; hY = ys;
                    } else {
                        const int rm = r + part;
                        const float mB = part ? hB : sB, mA = part ? hA : sA, mY = part ? hY : ys;
                        const float m_dl = rdl[rm * DT], m_u = to_f(ru[rm * DT]), m_dyp = rgy[rm * DT];
                        const bool row_ok = d_ok && rm < nv;
                        const long long grow = static_cast<long long>(b) * T + t0 + rm;
                        if (row_ok) g_du[grow * p.ld_du + d] = from_f<Tact>(fmaf(m_dyp, Dd, m_dl * mB));
                        accD = fmaf(m_dyp, m_u, accD);
                        if (kGate) {
                            const float zv = to_f(st_z(s)[rm * DT + col]);
                            const float dyv = to_f(st_dy(s)[rm * DT + col]);
                            const float sg = sigmoidf_fast(zv);
                            const float dsilu = sg * fmaf(zv, 1.0f - sg, 1.0f);
                            // pre-gate output and the gate, kernels/elementwise.cu:191-233
                            if (row_ok)
                                g_dz[grow * p.ld_dz + d] = from_f<Tact>(dyv * fmaf(Dd, m_u, mY) * (gate_is_silu ? dsilu : 1.0f));
                        }
                        float ddl = fmaf(mA, kLn2, m_u * mB);
                        if (kSoftplus) {
                            const float raw = to_f(st_dl(s)[rm * DT + col]);
                            ddl *= raw > 20.0f ? 1.0f : sigmoidf_fast(raw);  // activations.cu:68-104
                        }
                        if (row_ok) g_ddl[grow * p.ld_ddl + d] = from_f<Tact>(ddl);
                    }
                    // sum over the 16 channels of this half-warp: recursive halving, lane
                    // chl ends with element chl of (dB[n0..n0+7] | dC[n0..n0+7]).
                    float red[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        red[2 * j] = rB[j].x; red[2 * j + 1] = rB[j].y;
                        red[8 + 2 * j] = rC[j].x; red[8 + 2 * j + 1] = rC[j].y;
                    }
#pragma unroll
                    for (int st = 0; st < 4; ++st) {
                        const int m = 8 >> st;  // lane distance and number of elements kept
                        const bool upper = (chl & m) != 0;
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            if (q < m) {
                                const float send = upper ? red[q] : red[q + m];
                                const float keep = upper ? red[q + m] : red[q];
                                red[q] = keep + __shfl_xor_sync(0xffffffffu, send, m);
                            }
                        }
                    }
                    if (r < nv) pbc[i * 32] = red[0];
                }
            }

            __syncwarp();  // every reader of the stage is done before it is refilled
        }
    };
    if (geo) run_blocks(std::true_type{});
    else run_blocks(std::false_type{});

    // per-sample parameter-gradient partials
    accD += __shfl_xor_sync(0xffffffffu, accD, 16);
    if (d_ok) {
        if (part == 0) p.part_d[static_cast<long long>(b) * D + d] = accD;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (n0 + j < N)
                p.part_a[(static_cast<long long>(b) * D + d) * N + n0 + j] =
                    ((j & 1) ? accA[j / 2].y : accA[j / 2].x) * p.a_neg[static_cast<long long>(d) * N + n0 + j];
    }
}

template <typename Tact>
static void fill_bwd2(BwdKernelFn (*fn)[4], size_t* smem) {
    fn[0][0] = sscan_bwd2_kernel<Tact, 32, 0>;
    fn[0][1] = sscan_bwd2_kernel<Tact, 32, 1>;
    fn[0][2] = sscan_bwd2_kernel<Tact, 32, 2>;
    fn[0][3] = sscan_bwd2_kernel<Tact, 32, 3>;
    fn[1][0] = sscan_bwd2_kernel<Tact, 64, 0>;
    fn[1][1] = sscan_bwd2_kernel<Tact, 64, 1>;
    fn[1][2] = sscan_bwd2_kernel<Tact, 64, 2>;
    fn[1][3] = sscan_bwd2_kernel<Tact, 64, 3>;
    smem[0] = Bwd2Traits<Tact, 32>::SMEM;
    smem[1] = Bwd2Traits<Tact, 64>::SMEM;
}

// [stride index: 0 = 32, 1 = 64][flags]; one translation unit per storage dtype
void bwd2_kernels_f32(BwdKernelFn (*fn)[4], size_t* smem);
void bwd2_kernels_f16(BwdKernelFn (*fn)[4], size_t* smem);
void bwd2_kernels_bf16(BwdKernelFn (*fn)[4], size_t* smem);

}  // namespace mb200
