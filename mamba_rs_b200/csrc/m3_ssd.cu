// Mamba-3 SISO SSD scan (trapezoidal recurrence) forward for sm_100a.
//
// Two kernels behind one entry point:
//  * m3_ssd_fwd_tc_kernel — chunked form on the 5th-generation tensor cores
//    (tcgen05.mma, accumulators in TMEM) for 16-bit storage, headdim 64,
//    d_state 128: per (sample, head) one CTA walks 128-step chunks and keeps
//    the running state S^T [N x hd] f32 resident in TMEM, so the entering states
//    never touch HBM (the reference writes [B, chunks, nh, hd, N] f32 of them).
//    Per chunk: G = Q K^T, decay/causal mask in registers, Y1 = M V,
//    Y2 = Q S_in^T, S^T <- exp(dA_end) S^T + K^T (w o V).
//  * m3_ssd_seq_kernel — the sequential definition (one thread per
//    (sample, head, p), state in registers) for every other shape / dtype and
//    whenever a recurrent state is carried in.
#include <string.h>

#include <type_traits>

#include "common.cuh"
#include "internal.h"
#include "m3_tc.cuh"

namespace mb200 {

struct M3Params {
    // tensor-core kernel: Q (or Cn), K (or Bn) and x as [128 x 64] swizzled sub-tile maps
    CUtensorMap tm_q, tm_k, tm_v;
    CUtensorMap tm_adt, tm_dt, tm_trap;  // [B,T,nh] f32, boxes of 4 heads x 129 rows
    int sc_tma;                          // 1: the three maps above are valid (nheads % 4 == 0)
    int wide_y;                          // 1: y rows leave as 256-bit stores
    const void *x, *K, *Q;
    const float *dt, *trap, *adt, *Dh;
    void* y;
    float *ssm_state, *k_state, *v_state;  // in/out (may be null: zero in, not written)
    int B, T, nh, hd, N;
    int carry_in;  // 1: the state buffers hold a state to continue from
    // Optional: K and Q built inside the tensor-core kernel from the group-level
    // B / C after BCNorm, the per-head biases and RoPE (Bn == nullptr: K, Q are read).
    const void *Bn, *Cn;            // [B,T,ng,N] storage dtype
    const float *b_bias, *c_bias;   // [nh,N]
    const float* angle_vel;         // [B,T,n_angles]: tanh(angles_raw) * pi
    float* angle_state;             // [B,nh,n_angles] in/out (may be null: zero in, not written)
    int ng, n_angles;
    int* status;
};

// ---------------------------------------------------------------------------
// Sequential definition, src/mamba3_siso/cpu/forward.rs:85-138 / kernels/mamba3_ssd.cu:229-348:
//   h = alpha h + (beta v_prev) k_prev + (gamma x) k ;  y = <h, q> + D x
// grid (nh, B), block hd threads (rounded up to a warp); k, q, k_prev staged in
// shared memory per step.
// ---------------------------------------------------------------------------
template <typename Tact, int NMAX>
__global__ void m3_ssd_seq_kernel(const M3Params p) {
    extern __shared__ float sm[];
    float* ks = sm;                // [2][N] current / previous k
    float* qs = sm + 2 * p.N;      // [N]
    const int h = blockIdx.x, b = blockIdx.y, pp = threadIdx.x;
    const int N = p.N, hd = p.hd, nh = p.nh, T = p.T;
    const bool act = pp < hd;
    float st[NMAX];
#pragma unroll
    for (int n = 0; n < NMAX; ++n) st[n] = 0.0f;
    float vprev = 0.0f;
    if (p.carry_in) {
        if (act) {
#pragma unroll
            for (int n = 0; n < NMAX; ++n)
                if (n < N) st[n] = p.ssm_state[((static_cast<long long>(b) * nh + h) * hd + pp) * N + n];
            vprev = p.v_state[(static_cast<long long>(b) * nh + h) * hd + pp];
        }
        for (int n = threadIdx.x; n < N; n += blockDim.x)
            ks[N + n] = p.k_state[(static_cast<long long>(b) * nh + h) * N + n];
    } else {
        for (int n = threadIdx.x; n < N; n += blockDim.x) ks[N + n] = 0.0f;
    }
    const Tact* xb = static_cast<const Tact*>(p.x);
    const Tact* Kb = static_cast<const Tact*>(p.K);
    const Tact* Qb = static_cast<const Tact*>(p.Q);
    Tact* yb = static_cast<Tact*>(p.y);
    const float Dv = p.Dh[h];
    for (int t = 0; t < T; ++t) {
        const long long th = (static_cast<long long>(b) * T + t) * nh + h;
        const int cur = t & 1, prv = cur ^ 1;  // ks[cur] <- k_t ; ks[prv] holds k_{t-1}
        __syncthreads();
        for (int n = threadIdx.x; n < N; n += blockDim.x) {
            ks[cur * N + n] = to_f(Kb[th * N + n]);
            qs[n] = to_f(Qb[th * N + n]);
        }
        __syncthreads();
        const float alpha = ex2(p.adt[th] * kLog2e);
        const float beta = alpha * p.dt[th] * (1.0f - p.trap[th]);
        const float gamma = p.trap[th] * p.dt[th];
        if (act) {
            const float xv = to_f(xb[(static_cast<long long>(b) * T + t) * nh * hd + h * hd + pp]);
            const float bv = beta * vprev, gx = gamma * xv;
            float acc = 0.0f;
            const float* kc = ks + cur * N;
            const float* kp = ks + prv * N;
#pragma unroll
            for (int n = 0; n < NMAX; ++n)
                if (n < N) {
                    st[n] = fmaf(alpha, st[n], fmaf(bv, kp[n], gx * kc[n]));
                    acc = fmaf(st[n], qs[n], acc);
                }
            yb[(static_cast<long long>(b) * T + t) * nh * hd + h * hd + pp] = from_f<Tact>(fmaf(Dv, xv, acc));
            vprev = xv;
        }
    }
    // T == 0 leaves the state untouched; otherwise ks[(T-1)&1] holds the last k.
    if (T > 0) {
        if (p.ssm_state && act) {
#pragma unroll
            for (int n = 0; n < NMAX; ++n)
                if (n < N) p.ssm_state[((static_cast<long long>(b) * nh + h) * hd + pp) * N + n] = st[n];
        }
        if (p.v_state && act) p.v_state[(static_cast<long long>(b) * nh + h) * hd + pp] = vprev;
        __syncthreads();
        if (p.k_state)
            for (int n = threadIdx.x; n < N; n += blockDim.x)
                p.k_state[(static_cast<long long>(b) * nh + h) * N + n] = ks[((T - 1) & 1) * N + n];
    }
}

// ---------------------------------------------------------------------------
// tcgen05 / TMEM chunked kernel.  hd = 64, N = 128, chunk = 128, 256 threads.
// ---------------------------------------------------------------------------
namespace tc {

constexpr int CS = 128, HD = 64, NS = 128;
// Shared-memory operand tiles are 128-byte-swizzled [rows x 64] sub-tiles (m3_tc.cuh); TMA
// lands Q, K and V in that form.  One CTA per SM.  Q, K and V are double-buffered: the
// copies of chunk c + 1 are issued (one thread, five boxes) before chunk c is touched, so a
// whole chunk of work hides their latency -- with single buffers, two CTAs per SM and
// 16-byte asynchronous copies, 7.6 of the 11.5 us a chunk took were spent waiting for its
// tiles.  M has its own tile; one more tile holds w o V for the state update and then the
// 16-bit copy of the new state for the next chunk's Y2; then f32 vectors, barriers.
constexpr uint32_t kQ0 = 0, kK0 = 65536, kV0 = 131072, kQKStride = 32768, kVStride = 16384;
constexpr uint32_t kM = 163840, kVw = 196608, kS = 196608;
// f32 dA[128], scale[128], gamma[128], dA*log2(e)[128], dt[128] per chunk, two sets: a chunk's
// set is written while slower threads may still read the previous chunk's
constexpr uint32_t kVec = 212992, kVecSet = 5 * 128;
// K / Q generation: the angle entering the chunk, f64 [64]; this head's B / C biases [2][128]
constexpr uint32_t kCarry = kVec + 2 * kVecSet * 4, kBias = kCarry + 64 * 8;
// per-row adt, dt, trap of a chunk (dt and trap with the row after it), two buffers,
// filled by 4-byte asynchronous copies
// [3][129 rows][4 heads] f32; a TMA destination has to start on a 128-byte boundary
constexpr uint32_t kStage = kBias + 2 * 128 * 4, kStageArr = 17 * 128;
static_assert(kStage % 128 == 0 && kStageArr >= 129 * 16, "scalar staging");
constexpr uint32_t kBar = kStage + 3 * kStageArr + 16, kTmemSlot = kBar + 48;
constexpr uint32_t kSmem = kTmemSlot + 16;
// TMEM columns: G; Y1; Y2; S^T.
constexpr uint32_t cG = 0, cY1 = 256, cY2 = 320, cS = 384, kTmemCols = 512;

// GEN: build the K and Q tiles of a chunk in the kernel instead of reading them:
//   K[t,h,:] = rope(Bn[t,g,:] + b_bias[h,:], angle[t,h,:]),  Q likewise from Cn / c_bias,
//   angle[t,h,a] = (angle_in[h,a] + sum_{s<=t} angle_vel[s,a] * dt[s,h]) mod 2 pi
// (src/mamba3_siso/cpu/forward.rs:336-375; kernels/mamba3_ops.cu:279-310, :400-440,
// :575-640).  The in-chunk sums run in f32 (shuffle scans over the rows), the angle
// entering a chunk is carried in f64.
template <typename Th, bool GEN>
__global__ void __launch_bounds__(256, 1) m3_ssd_fwd_tc_kernel(const __grid_constant__ M3Params p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    // two threads per step: thread (row, half) owns row `row` of the chunk (TMEM lane
    // `row`) and half of that row's columns in every elementwise stage
    const int tid = threadIdx.x & 127, half = threadIdx.x >> 7, warp = (threadIdx.x >> 5) & 3;
    const int lane = threadIdx.x & 31, wfull = threadIdx.x >> 5;
    const int h = blockIdx.x, b = blockIdx.y;
    const int T = p.T, nh = p.nh;
    // headdim <= 64 and d_state <= 128 (multiples of 8): the tiles keep their full
    // size and the missing columns are zero-filled, so every product is unchanged.
    const int hdv = p.hd, nsv = p.N;
    constexpr uint32_t fmt = std::is_same<Th, __nv_bfloat16>::value ? 1u : 0u;
    float* vec = reinterpret_cast<float*>(smem + kVec);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBar);
    uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + kTmemSlot);
    const uint32_t sbase = smem_u32(smem);

    uint64_t* full = bars + 2;  // tiles of buffer 0 / 1 have landed (TMA)
    if (threadIdx.x == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        mbar_init(bars + 4, 1);
        fence_barrier_init();
    }
    double* carry = reinterpret_cast<double*>(smem + kCarry);
    float* bias_sm = reinterpret_cast<float*>(smem + kBias);
    if (GEN) {
        if (threadIdx.x < 64) {
            const int a = threadIdx.x;
            const float v = (a < p.n_angles && p.angle_state)
                                ? p.angle_state[(static_cast<long long>(b) * nh + h) * p.n_angles + a] : 0.0f;
            carry[a] = static_cast<double>(v);
        }
        const float* bsrc = half ? p.c_bias : p.b_bias;
        bias_sm[half * 128 + tid] = tid < nsv ? bsrc[static_cast<long long>(h) * nsv + tid] : 0.0f;
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tslot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *tslot;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);  // this warp's 32 lanes

    const Th* xg = static_cast<const Th*>(p.x);
    Th* yg = static_cast<Th*>(p.y);
    const Th* Kg = static_cast<const Th*>(p.K);
    const float Dv = p.Dh[h];
    const int nchunks = (T + CS - 1) / CS;
    bool ok = true;

    // Per-row scalars of chunk c into stage `st`: inclusive cumsum of adt, scale, gamma.
    // Per-row adt, dt, trap of the next chunk (dt and trap with the row after it) are staged in
    // shared memory while the current chunk runs.  As register loads they were drained by every
    // proxy fence of the chunk (0.18 ms of 0.45 ms at 32 heads, where they are 128-byte-strided
    // words); a fence waits for 4-byte asynchronous copies too.  TMA copies are not waited for:
    // with nheads % 4 == 0 one thread fetches [129 rows x 4 heads] boxes; otherwise the copies
    // are issued where the next fence is furthest away.
    uint64_t* scf = bars + 4;
    const int hcol = h & 3;
    auto stage_scalars = [&](int c) {
        if (c >= nchunks) return;
        if (p.sc_tma) {
            if (threadIdx.x == 0) {
                mbar_expect_tx(scf, 3 * 129 * 16);
                tma_load_3d(smem + kStage, &p.tm_adt, scf, h & ~3, c * CS, b);
                tma_load_3d(smem + kStage + kStageArr, &p.tm_dt, scf, h & ~3, c * CS, b);
                tma_load_3d(smem + kStage + 2 * kStageArr, &p.tm_trap, scf, h & ~3, c * CS, b);
            }
        } else {
            if (threadIdx.x <= CS) {
                float* st = reinterpret_cast<float*>(smem + kStage) + threadIdx.x * 4 + hcol;
                const int t = c * CS + threadIdx.x;
                const long long th = (static_cast<long long>(b) * T + t) * nh + h;
                if (t < T) {
                    cp_async4(st, p.adt + th);
                    cp_async4(st + kStageArr / 4, p.dt + th);
                    cp_async4(st + 2 * kStageArr / 4, p.trap + th);
                } else {
                    st[0] = st[kStageArr / 4] = st[2 * kStageArr / 4] = 0.0f;
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
    };
    auto scalars = [&](int c, int st) {
        float* dA = vec + st * kVecSet;
        float* scl = dA + 128;
        float* gam = dA + 256;
        if (p.sc_tma) {
            ok = mbar_wait(scf, c & 1, p.status) && ok;
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();  // every thread's staged words of this chunk are in shared memory
        }
        const float* stg = reinterpret_cast<const float*>(smem + kStage) + hcol;
        const float a = stg[tid * 4], dtr = stg[kStageArr / 4 + tid * 4], g = dtr * stg[2 * kStageArr / 4 + tid * 4];
        const float s = g + stg[kStageArr / 4 + tid * 4 + 4] * (1.0f - stg[2 * kStageArr / 4 + tid * 4 + 4]);
        float run = a;
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
            const float o = __shfl_up_sync(0xffffffffu, run, m);
            if (lane >= m) run += o;
        }
        // warp totals in the 112 spare bytes behind the first staging array
        float* wtot = reinterpret_cast<float*>(smem + kStage + 129 * 16);
        if (lane == 31) wtot[warp] = run;
        gam[tid] = g;
        scl[tid] = s;
        if (GEN) dA[512 + tid] = dtr;
        __syncthreads();
        const float w0 = wtot[0], w1 = wtot[1], w2 = wtot[2];
        const float off = (warp > 0 ? w0 : 0.0f) + (warp > 1 ? w1 : 0.0f) + (warp > 2 ? w2 : 0.0f);
        dA[tid] = run + off;
        dA[384 + tid] = (run + off) * kLog2e;
        // (the barrier ahead of the first MMA group publishes these rows)
    };


    // K and Q tiles of chunk c from the group-level rows (GEN only): TMA lands the raw Bn / Cn
    // rows of this head's group in the K / Q tiles and gen_apply rewrites them in place.
    // Thread (lane, warp w) owns the 16-byte pieces j = w and w + 8 of the rows lane,
    // lane + 32, lane + 64, lane + 96.  The angle of (row, a) is the angle entering the chunk
    // (f64, shared memory) plus an inclusive sum over the rows: a warp shuffle scan inside each
    // block of 32 rows and a running prefix over the four blocks, which the same thread owns.
    // this thread's angle velocities of the chunk that gen_apply rewrites next (loaded a
    // chunk ahead, like the per-row scalars)
    float4 velr[4][2];
    auto load_vel = [&](int c) {
        const int t0 = c * CS, nv = min(CS, T - t0), na = p.n_angles;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int j = wfull + 8 * q, row = lane + 32 * i;
                velr[i][q] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (c < nchunks && 4 * j < na && row < nv)
                    velr[i][q] = __ldg(reinterpret_cast<const float4*>(
                        p.angle_vel + (static_cast<long long>(b) * T + t0 + row) * na + 4 * j));
            }
    };
    auto gen_apply = [&](int c, int buf) {
        const int t0 = c * CS, nv = min(CS, T - t0);
        const int na = p.n_angles;
        constexpr double kTwoPi64 = 6.283185307179586, kInvTwoPi64 = 0.15915494309189535;
        const bool rot0 = 4 * wfull < na, rot1 = 4 * (wfull + 8) < na;
        float ang[4][2][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = lane + 32 * i;
            const float dtr = row < nv ? vec[(c & 1) * kVecSet + 512 + row] : 0.0f;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                ang[i][q][0] = velr[i][q].x * dtr; ang[i][q][1] = velr[i][q].y * dtr;
                ang[i][q][2] = velr[i][q].z * dtr; ang[i][q][3] = velr[i][q].w * dtr;
            }
        }
        // inclusive sums over the 32 rows of each block: every value advances together
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    if (q ? rot1 : rot0) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float o = __shfl_up_sync(0xffffffffu, ang[i][q][e], m);
                            if (lane >= m) ang[i][q][e] += o;
                        }
                    }
        }
        // entering angle + the blocks before; the chunk's total goes into the f64 carry
#pragma unroll
        for (int q = 0; q < 2; ++q)
            if (q ? rot1 : rot0) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int a = 4 * (wfull + 8 * q) + e;
                    const double cin = carry[a];
                    float run = static_cast<float>(cin), tot = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float bt = __shfl_sync(0xffffffffu, ang[i][q][e], 31);
                        ang[i][q][e] += run;
                        run += bt;
                        tot += bt;
                    }
                    double sacc = cin + static_cast<double>(tot);
                    sacc -= kTwoPi64 * floor(sacc * kInvTwoPi64);
                    __syncwarp();
                    if (lane == 0) carry[a] = sacc;
                }
            }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int row = lane + 32 * i;
            const bool rok = row < nv;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int j = wfull + 8 * q;
                const bool rot = q ? rot1 : rot0;
                float sn[4], cs[4];
                if (rot) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // to [-pi, pi] before the fast sine / cosine
                        float x = ang[i][q][e];
                        const float turns = rintf(x * 0.15915494309189535f);
                        x = fmaf(turns, -6.2831854820251465f, x);
                        x = fmaf(turns, 1.7484555e-7f, x);
                        __sincosf(x, &sn[e], &cs[e]);
                    }
                }
                if (8 * j < nsv && rok) {
#pragma unroll
                    for (int which = 0; which < 2; ++which) {
                        uint4* pp = reinterpret_cast<uint4*>(smem + (which ? kQ0 : kK0) + buf * kQKStride +
                                                             sw_chunk(row, j));
                        const uint4 raw = *pp;
                        const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
                        const float4 b0 = *reinterpret_cast<const float4*>(bias_sm + which * 128 + 8 * j);
                        const float4 b1 = *reinterpret_cast<const float4*>(bias_sm + which * 128 + 8 * j + 4);
                        const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                        uint32_t ow[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = unpack2<Th>(rw[e]);
                            float v0 = f.x + bv[2 * e], v1 = f.y + bv[2 * e + 1];
                            if (rot) {
                                const float r0 = cs[e] * v0 - sn[e] * v1, r1 = sn[e] * v0 + cs[e] * v1;
                                v0 = r0; v1 = r1;
                            }
                            ow[e] = pack2<Th>(v0, v1);
                        }
                        *pp = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    }
                }
            }
        }
    };

    // One elected thread issues the five boxes of a chunk (Q and K: two 64-column sub-tiles
    // each, V: one); rows past the end of the sequence and columns past the head's width
    // arrive as zeros.
    auto issue_tiles = [&](int c) {
        if (threadIdx.x == 0) {
            const int buf = c & 1, t0 = c * CS;
            const int hq = GEN ? h / (nh / p.ng) : h;
            mbar_expect_tx(&full[buf], 2 * kQKStride + kVStride);
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
                tma_load_4d(smem + kQ0 + buf * kQKStride + sub * kSwSub, &p.tm_q, &full[buf], 64 * sub, hq, t0, b);
                tma_load_4d(smem + kK0 + buf * kQKStride + sub * kSwSub, &p.tm_k, &full[buf], 64 * sub, hq, t0, b);
            }
            tma_load_4d(smem + kV0 + buf * kVStride, &p.tm_v, &full[buf], 0, h, t0, b);
        }
    };
    issue_tiles(0);
    stage_scalars(0);
    if (GEN) load_vel(0);

    for (int c = 0; c < nchunks; ++c) {
        const int t0 = c * CS, nv = min(CS, T - t0);
        const bool row_ok = tid < nv;
        const float* dA = vec + (c & 1) * kVecSet;
        const float* scl = dA + 128;
        const float* gam = dA + 256;
        const uint32_t tQ = kQ0 + (c & 1) * kQKStride, tK = kK0 + (c & 1) * kQKStride, tV = kV0 + (c & 1) * kVStride;
        // ---- 1. copies of the next chunk's tiles into the other buffers (their last readers,
        //         the MMAs of chunk c - 1, have completed); per-row scalars; this chunk's tiles ----
        if (c + 1 < nchunks) issue_tiles(c + 1);
        scalars(c, c & 1);
        ok = mbar_wait(&full[c & 1], (c >> 1) & 1, p.status) && ok;
        if (GEN) {
            gen_apply(c, c & 1);
            fence_proxy_async();  // the rewritten K / Q pieces, before the tensor core reads them
        }
        fence_before();
        __syncthreads();
        // A proxy fence waits for this thread's outstanding asynchronous copies (measured:
        // 1500 cycles when the staged scalars were issued ahead of one), so they start here,
        // with the MMA wait and the mask stage between them and the next fence.
        stage_scalars(c + 1);
        // ---- 2. G = Q K^T (and Y2 = Q S_in^T for c > 0) ----
        if (threadIdx.x == 0) {
            fence_after();
            const uint32_t idG = instr_desc(fmt, 0, 0, 128), idY = instr_desc(fmt, 0, 1, 64);
#pragma unroll
            for (int k = 0; k < NS / 16; ++k)
                mma(tmem + cG, desc_sw_k(sbase + tQ, k), desc_sw_k(sbase + tK, k), idG, k > 0);
            if (c > 0) {
#pragma unroll
                for (int k = 0; k < NS / 16; ++k)  // N = p, K = n
                    mma(tmem + cY2, desc_sw_k(sbase + tQ, k), desc_sw_mn(sbase + kS, k), idY, k > 0);
            }
            commit(&bars[0]);
        }
        ok = mbar_wait(&bars[0], c & 1, p.status) && ok;
        fence_after();
        // ---- 3. decay / causal mask -> M (over the Q tile); w o V (over the old state
        //         copy); rescale the running state ----
        {
            {
                const float wt = row_ok ? ex2((dA[nv - 1] - dA[tid]) * kLog2e) * scl[tid] : 0.0f;
#pragma unroll
                for (int j = half * (HD / 16); j < (half + 1) * (HD / 16); ++j) {
                    const uint4 v = *reinterpret_cast<const uint4*>(smem + tV + sw_chunk(tid, j));
                    uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const float2 f = unpack2<Th>(w4[q4]);
                        w4[q4] = pack2<Th>(f.x * wt, f.y * wt);
                    }
                    *reinterpret_cast<uint4*>(smem + kVw + sw_chunk(tid, j)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                }
            }
            const float* dAl = dA + 384;  // dA * log2(e)
            const float dAlt = dAl[tid], gt = gam[tid];
            // One 32-column block of row `tid`.  Blocks left of the diagonal block need no
            // mask; rows and columns past the end of the sequence need none either (their
            // V rows are zero and their y rows are never stored).
            auto mask_block = [&](auto diag_tag, int q4) {
                constexpr bool DIAG = decltype(diag_tag)::value;
                float g[32];
                tmem_ld32(lane_addr + cG + q4 * 32, g);
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    const float4 da4 = *reinterpret_cast<const float4*>(dAl + q4 * 32 + i);
                    const float4 sc4 = *reinterpret_cast<const float4*>(scl + q4 * 32 + i);
                    const float dav[4] = {da4.x, da4.y, da4.z, da4.w}, scv[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
                    float m[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float v = g[i + u] * scv[u] * ex2(dAlt - dav[u]);
                        if (DIAG) {
                            const int s = q4 * 32 + i + u;
                            if (s > tid) v = 0.0f;
                            else if (s == tid) v = fmaf(g[i + u], gt, Dv);
                        }
                        m[u] = v;
                    }
                    packed[i / 2] = pack2<Th>(m[0], m[1]);
                    packed[i / 2 + 1] = pack2<Th>(m[2], m[3]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<uint4*>(smem + kM + sw_chunk(tid, q4 * 4 + j)) =
                        make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
            };
            for (int q4 = 2 * half; q4 < 2 * half + 2; ++q4) {
                if (q4 > warp) {  // wholly above the diagonal for every row of this warp
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *reinterpret_cast<uint4*>(smem + kM + sw_chunk(tid, q4 * 4 + j)) = make_uint4(0, 0, 0, 0);
                } else if (q4 == warp) {
                    mask_block(std::true_type{}, q4);
                } else {
                    mask_block(std::false_type{}, q4);
                }
            }
            if (c > 0) {  // S^T row `tid` (state index n = tid) *= exp(dA_end)
                const float e_end = ex2(dA[nv - 1] * kLog2e);
                float sv[32];
                tmem_ld32(lane_addr + cS + half * 32, sv);
#pragma unroll
                for (int i = 0; i < 32; ++i) sv[i] *= e_end;
                tmem_st32(lane_addr + cS + half * 32, sv);
            }
        }
        fence_proxy_async();
        fence_before();
        __syncthreads();
        // register loads issued here have the longest run before the next proxy fence
        if (GEN) load_vel(c + 1);
        // ---- 4. Y1 = M V ;  S^T += K^T (w o V) ----
        if (threadIdx.x == 0) {
            fence_after();
            const uint32_t idY = instr_desc(fmt, 0, 1, 64), idS = instr_desc(fmt, 1, 1, 64);
#pragma unroll
            for (int k = 0; k < CS / 16; ++k)  // N = p, K = s
                mma(tmem + cY1, desc_sw_k(sbase + kM, k), desc_sw_mn(sbase + tV, k), idY, k > 0);
#pragma unroll
            for (int k = 0; k < CS / 16; ++k)  // M = n, N = p, K = t
                mma(tmem + cS, desc_sw_mn(sbase + tK, k), desc_sw_mn(sbase + kVw, k), idS, c > 0 || k > 0);
            commit(&bars[1]);
        }
        ok = mbar_wait(&bars[1], c & 1, p.status) && ok;
        fence_after();
        // ---- 5. epilogue: y row; 16-bit copy of the new state for the next chunk ----
        {
            const float e_t = ex2(dA[tid] * kLog2e);
            const int q2 = half;
            float y1[32], y2[32];
            if (c > 0) {
                tmem_ld32x2(lane_addr + cY1 + q2 * 32, y1, lane_addr + cY2 + q2 * 32, y2);
#pragma unroll
                for (int i = 0; i < 32; ++i) y1[i] = fmaf(e_t, y2[i], y1[i]);
            } else {
                tmem_ld32(lane_addr + cY1 + q2 * 32, y1);
            }
            uint4 yo[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                yo[j] = make_uint4(pack2<Th>(y1[8 * j], y1[8 * j + 1]), pack2<Th>(y1[8 * j + 2], y1[8 * j + 3]),
                                   pack2<Th>(y1[8 * j + 4], y1[8 * j + 5]), pack2<Th>(y1[8 * j + 6], y1[8 * j + 7]));
            float sv[32];
            tmem_ld32(lane_addr + cS + q2 * 32, sv);
            if (c + 1 < nchunks) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<uint4*>(smem + kS + sw_chunk(tid, q2 * 4 + j)) =
                        make_uint4(pack2<Th>(sv[8 * j], sv[8 * j + 1]), pack2<Th>(sv[8 * j + 2], sv[8 * j + 3]),
                                   pack2<Th>(sv[8 * j + 4], sv[8 * j + 5]), pack2<Th>(sv[8 * j + 6], sv[8 * j + 7]));
            } else if (p.ssm_state) {  // final state [b, h, p, n], n = tid
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (q2 * 32 + i < hdv && tid < nsv)
                        p.ssm_state[((static_cast<long long>(b) * nh + h) * hdv + q2 * 32 + i) * nsv + tid] = sv[i];
            }
            fence_proxy_async();  // the state copy, before the next chunk's Y2 reads it
            // y rows leave after the fence: a proxy fence waits for the thread's outstanding
            // global stores too, and the next one is most of a chunk away
            if (row_ok) {
                Th* yrow = yg + (static_cast<long long>(b) * T + t0 + tid) * nh * hdv + h * hdv + q2 * 32;
                if (p.wide_y) {  // headdim a multiple of 16, y 32-byte aligned
#pragma unroll
                    for (int j = 0; j < 4; j += 2)
                        if (q2 * 32 + 8 * j < hdv) store32b(yrow + 8 * j, yo[j], yo[j + 1], true);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (q2 * 32 + 8 * j < hdv) *reinterpret_cast<uint4*>(yrow + 8 * j) = yo[j];
                }
            }
        }
        // no barrier here: the next chunk writes the other set of per-row vectors, and every tile,
        // TMEM column and the state copy it touches is ordered by its own barriers
    }
    fence_before();
    __syncthreads();
    fence_after();
    // last inputs of the window (kernels/mamba3_chunked.cu:289-330)
    if (T > 0) {
        const long long last = static_cast<long long>(b) * T + (T - 1);
        if (GEN) {
            // the last K row is still in its tile; fold the last chunk's sums into the angle
            const int lr = T - 1 - (nchunks - 1) * CS;
            if (p.k_state && half == 0 && tid < nsv)
                p.k_state[(static_cast<long long>(b) * nh + h) * nsv + tid] =
                    to_f(*reinterpret_cast<const Th*>(smem + kK0 + ((nchunks - 1) & 1) * kQKStride +
                                                     sw_chunk(lr, tid >> 3) + (tid & 7) * 2));
            if (p.angle_state && threadIdx.x < p.n_angles)
                p.angle_state[(static_cast<long long>(b) * nh + h) * p.n_angles + threadIdx.x] =
                    static_cast<float>(carry[threadIdx.x]);
        } else if (p.k_state && half == 0 && tid < nsv)
            p.k_state[(static_cast<long long>(b) * nh + h) * nsv + tid] = to_f(Kg[(last * nh + h) * nsv + tid]);
        if (p.v_state && half == 0 && tid < hdv)
            p.v_state[(static_cast<long long>(b) * nh + h) * hdv + tid] = to_f(xg[last * nh * hdv + h * hdv + tid]);
    }
    __syncthreads();
    if (threadIdx.x < 32)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    (void)ok;
}

}  // namespace tc

int m3_configure(Ctx* c) {
    const void* fns[4] = {reinterpret_cast<const void*>(tc::m3_ssd_fwd_tc_kernel<__nv_bfloat16, false>),
                          reinterpret_cast<const void*>(tc::m3_ssd_fwd_tc_kernel<__half, false>),
                          reinterpret_cast<const void*>(tc::m3_ssd_fwd_tc_kernel<__nv_bfloat16, true>),
                          reinterpret_cast<const void*>(tc::m3_ssd_fwd_tc_kernel<__half, true>)};
    for (const void* fn : fns)
        MB200_CUDA_CHECK(c, cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::kSmem));
    return MAMBA_B200_OK;
}

template <typename Tact>
static void launch_seq(const M3Params& p, cudaStream_t st) {
    dim3 grid(p.nh, p.B);
    const int threads = ((p.hd + 31) / 32) * 32;
    const size_t smem = sizeof(float) * 3 * p.N;
    if (p.N <= 16) m3_ssd_seq_kernel<Tact, 16><<<grid, threads, smem, st>>>(p);
    else if (p.N <= 32) m3_ssd_seq_kernel<Tact, 32><<<grid, threads, smem, st>>>(p);
    else if (p.N <= 64) m3_ssd_seq_kernel<Tact, 64><<<grid, threads, smem, st>>>(p);
    else m3_ssd_seq_kernel<Tact, 128><<<grid, threads, smem, st>>>(p);
}

}  // namespace mb200

using namespace mb200;

extern "C" MAMBA_B200_API int mamba_b200_m3_ssd_fwd(void* handle, void* stream,
                                                    const mamba_b200_m3_ssd_args* ap) {
    Ctx* c = static_cast<Ctx*>(handle);
    if (!c) return MAMBA_B200_ERR_ARG;
    if (!ap) return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_fwd: null args");
    const mamba_b200_m3_ssd_args& a = *ap;
    if (!dtype_ok(a.dtype)) return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_fwd: bad dtype %d", a.dtype);
    if (a.B < 0 || a.T < 0 || a.nh <= 0 || a.hd <= 0 || a.N <= 0)
        return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_fwd: bad dims");
    if (a.hd > 1024 || a.N > 128)
        return fail(c, MAMBA_B200_ERR_SHAPE, "m3_ssd_fwd: headdim %d > 1024 or d_state %d > 128", a.hd, a.N);
    if (a.B == 0 || a.T == 0) return MAMBA_B200_OK;
    if (a.B > 65535) return fail(c, MAMBA_B200_ERR_SHAPE, "m3_ssd_fwd: batch %d > 65535", a.B);
    const bool gen = a.Bn != nullptr;
    if (!a.x || (!gen && (!a.K || !a.Q)) || !a.dt || !a.trap || !a.adt || !a.Dh || !a.y)
        return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_fwd: null required pointer");
    if (gen) {
        if (!a.Cn || !a.b_bias || !a.c_bias || a.ng <= 0 || a.nh % a.ng != 0 || a.n_angles < 0 ||
            (a.n_angles > 0 && !a.angle_vel))
            return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_fwd: K/Q generation needs Bn, Cn, both biases, ngroups "
                                                "dividing nheads and angle_vel when n_angles > 0");
        if (a.n_angles % 4 != 0 || 2 * a.n_angles > a.N)
            return fail(c, MAMBA_B200_ERR_SHAPE, "m3_ssd_fwd: n_angles %d must be a multiple of 4 and <= d_state / 2",
                        a.n_angles);
    }
    if (a.carry_in && (!a.ssm_state || !a.k_state || !a.v_state))
        return fail(c, MAMBA_B200_ERR_ARG, "m3_ssd_fwd: carry_in needs all three state buffers");
    M3Params p;
    memset(&p, 0, sizeof(p));
    p.x = a.x; p.K = a.K; p.Q = a.Q; p.dt = a.dt; p.trap = a.trap; p.adt = a.adt; p.Dh = a.Dh; p.y = a.y;
    p.ssm_state = a.ssm_state; p.k_state = a.k_state; p.v_state = a.v_state;
    p.B = a.B; p.T = a.T; p.nh = a.nh; p.hd = a.hd; p.N = a.N; p.carry_in = a.carry_in;
    p.Bn = a.Bn; p.Cn = a.Cn; p.b_bias = a.b_bias; p.c_bias = a.c_bias; p.angle_vel = a.angle_vel;
    p.angle_state = a.angle_state; p.ng = a.ng; p.n_angles = a.n_angles;
    p.status = c->d_status;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    bool tensor_core = a.dtype != MAMBA_B200_F32 && a.hd <= tc::HD && a.hd % 8 == 0 && a.N <= tc::NS &&
                       a.N % 8 == 0 && !a.carry_in &&
                       !a.force_sequential && al16(a.x) && al16(a.y) &&
                       (gen ? al16(a.Bn) && al16(a.Cn) && al16(a.angle_vel) : al16(a.K) && al16(a.Q));
    // the tile maps; when the driver refuses one (no encoder, a stride beyond its range) the
    // sequential kernel takes the call
    tensor_core = tensor_core &&
                  make_tmap_head_tile(c, &p.tm_q, a.dtype, gen ? a.Cn : a.Q, a.N, gen ? a.ng : a.nh, a.T, a.B) &&
                  make_tmap_head_tile(c, &p.tm_k, a.dtype, gen ? a.Bn : a.K, a.N, gen ? a.ng : a.nh, a.T, a.B) &&
                  make_tmap_head_tile(c, &p.tm_v, a.dtype, a.x, a.hd, a.nh, a.T, a.B);
    if (gen && !tensor_core)
        return fail(c, MAMBA_B200_ERR_SHAPE, "m3_ssd_fwd: K/Q generation runs on the tensor-core path only (16-bit "
                                              "storage, headdim <= 64, d_state <= 128, multiples of 8, no carried "
                                              "state, 16-byte aligned tensors)");
    if (tensor_core) {
        p.wide_y = a.hd % 16 == 0 && reinterpret_cast<uintptr_t>(a.y) % 32 == 0;
        p.sc_tma = a.nh % 4 == 0 &&
                   make_tmap_3d(c, &p.tm_adt, MAMBA_B200_F32, a.adt, a.nh, a.nh, a.T, a.B, 4, 129) &&
                   make_tmap_3d(c, &p.tm_dt, MAMBA_B200_F32, a.dt, a.nh, a.nh, a.T, a.B, 4, 129) &&
                   make_tmap_3d(c, &p.tm_trap, MAMBA_B200_F32, a.trap, a.nh, a.nh, a.T, a.B, 4, 129);
        dim3 grid(a.nh, a.B);
        if (a.dtype == MAMBA_B200_BF16) {
            if (gen) tc::m3_ssd_fwd_tc_kernel<__nv_bfloat16, true><<<grid, 256, tc::kSmem, st>>>(p);
            else tc::m3_ssd_fwd_tc_kernel<__nv_bfloat16, false><<<grid, 256, tc::kSmem, st>>>(p);
        } else {
            if (gen) tc::m3_ssd_fwd_tc_kernel<__half, true><<<grid, 256, tc::kSmem, st>>>(p);
            else tc::m3_ssd_fwd_tc_kernel<__half, false><<<grid, 256, tc::kSmem, st>>>(p);
        }
    } else {
        if (a.dtype == MAMBA_B200_F32) launch_seq<float>(p, st);
        else if (a.dtype == MAMBA_B200_F16) launch_seq<__half>(p, st);
        else launch_seq<__nv_bfloat16>(p, st);
    }
    MB200_CUDA_CHECK(c, cudaGetLastError());
    return MAMBA_B200_OK;
}
