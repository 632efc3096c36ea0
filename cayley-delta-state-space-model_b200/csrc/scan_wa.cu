// Fused scan with warp-autonomous chains: the Gram blocks of a 32-token sub-block come from the tcgen05
// tensor cores (TMA-staged bf16 tiles, fp32 accumulators in tensor memory), everything that depends on the
// running state stays inside the warp that owns the head.
// Shapes: bf16 storage, state_dim N = 2, head_dim D = chunk C in {64, 128}, H a multiple of 4.
//
// A thread block owns the same chunk of FOUR heads and walks it in 32-token sub-blocks; UMMA tile row
// 32 j + t is token t of head j's sub-block and compute warp j owns head j.  Per sub-block:
//   G = K K^T, P = Q K^T                : one full-width UMMA (M = N = 128) per 16-column k-step; head j reads its
//                                         own 32 x 32 diagonal block (lanes 32 j.., columns 32 j..).  The blocks
//                                         depend on nothing but the tiles, so the producer warp issues them as soon
//                                         as a tile has landed, a step ahead of the compute warps.
//   kappa, rho = K S^T, Q S^T           : products with the running states (local state z, correction r;
//                                         bf16 hi + lo columns), warp-level mma.sync on the warp's own 32
//                                         tile rows (ldmatrix straight from the swizzled TMA tile) with the
//                                         state held in the warp's registers in fragment layout.  |q_t|^2 comes
//                                         from the same Q fragments (diagonal of Q Q^T).
//   solve / read-out                    : unit-lower-triangular 32 x 32 systems by substitution through
//                                         warp shuffles, rows from tcgen05.ld (thread = token = TMEM lane).
//   S <- W_31 S + K^T Omega             : warp-level mma.sync again (ldmatrix.trans of the same K rows),
//                                         accumulating onto the decayed state registers.
// A step of a warp therefore contains no hand-off to another warp: the only barriers are "tile landed",
// "Gram blocks done" and the releases of tiles and tensor memory back to the producer.  Buffers: two K tiles
// (the update at the end of a step still reads the tile while the next one lands), one Q tile (handed back
// right after rho and |q|, a fifth into the step), one set of tensor-memory columns (handed back once the
// rows are in registers).
//
// Reference semantics (intra_chunk_scan.cu:100-195, exact_correction.cu:89-150): z starts at zero at the
// chunk start, r starts from the chunk's carry (bf16, from the carry pass), the correction is read before
// its step.  Algebra per sub-block with incoming states z0, r0:
//   u  = T beta (v - W kappa_z),  x = T beta W kappa_r,  T = (I + M)^-1,  M[t,i] = beta_t Gamma[t,i] G[t,i]
//   y_t = W_t rho_z,t + sum_{i<=t} Gamma[t,i] P[t,i] u_i + W0_t rho_r,t - sum_{i<t} Gamma0[t,i] P[t,i] x_i
//   z_end = W_31 z0 + sum_i Gamma[31,i] u_i k_i,   r_end = W_31 r0 - sum_i Gamma[31,i] x_i k_i
// (W, W0: inclusive / exclusive prefix products of a inside the sub-block.)
#include "cdssm_common.cuh"
#include "sm100_ptx.cuh"

namespace cdssm {
using namespace sm100;

namespace wa {

constexpr int kSub = 32;
constexpr int kThreads = 160;
constexpr uint32_t kSlab = 128 * 128;   // bytes of 128 tile rows x 64 bf16 columns

template <int kD>
struct Dims {
    static constexpr int kSlabs = kD / 64;
    static constexpr uint32_t kTile = kSlabs * kSlab;
    static constexpr int kKs = kD / 16;         // 16-column k-steps of a row
    static constexpr int kSteps = kD / kSub;    // sub-blocks per chunk (chunk = head_dim)
};

template <int kD, bool kOutput>
struct __align__(1024) Smem {
    uint8_t k[2][Dims<kD>::kTile];                 // rows 32 j + t: token t of head j (TMA, double buffered)
    uint8_t q[kOutput ? Dims<kD>::kTile : 1024];
    float scr[4][32 * 12];                         // per warp: kappa[4], rho[4] of token t at 12 t (transposition)
    float qs[4][32];                               // per warp: |q_t|^2
    float om[4][4 * 32];                           // per warp: omega[n'][t]
    uint64_t full_k[2], full_q, mma_g, mma_p, taken, q_free, k_free[2], drain;
    uint32_t tmem_base;
    int abort_flag;
};

template <bool kOutput>
struct Cols {   // tensor-memory columns: G (and P) of one step, 128 columns each: head j's block at column 32 j
    static constexpr uint32_t kTotal = kOutput ? 256 : 128;
    static constexpr uint32_t kG = 0, kP = 128;
};

struct Args {
    const uint4* rec;            // per (token, head) record from the dynamics pre-pass
    float* ws_gamma;             // (B,NC,H,2): written by the local pass
    float* ws_state;             // (B,NC,H,2,D): local pass writes z_{C-1}; the output pass reads the carry s_c
    __nv_bfloat16* y;
    int* status;
    unsigned long long wait_ns;  // limit of every device-side wait
    int withhold;                // test hook: the producer issues nothing, so the first wait runs out
    float shortcut_scale;
    int B, L, H, NC;
    int HG, items;               // head groups of four; items = B * NC * HG (one chunk of four heads each)
};

#ifdef CDSSM_WA_TRACE   // performance debugging builds only: clock stamps of one warp's steps
__device__ long long g_trace[32 * 16];
#define WA_STAMP(idx) do { if (blockIdx.x == 0 && J == 1 && tl == 0 && g >= 8 && g < 40) g_trace[(g - 8) * 16 + (idx)] = clock64(); } while (0)
#define WA_PSTAMP(n, idx) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (n) >= 8 && (n) < 40) g_trace[((n) - 8) * 16 + (idx)] = clock64(); } while (0)
#else
#define WA_STAMP(idx) do { } while (0)
#define WA_PSTAMP(n, idx) do { } while (0)
#endif

struct cplx { float r, i; };
__device__ __forceinline__ cplx cmul(cplx a, cplx b) { return {a.r * b.r - a.i * b.i, a.r * b.i + a.i * b.r}; }
__device__ __forceinline__ cplx cshfl(cplx v, int src) {
    return {__shfl_sync(0xffffffffu, v.r, src), __shfl_sync(0xffffffffu, v.i, src)};
}
__device__ __forceinline__ float bfr(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

struct ItemPos {   // chunk c of heads h0 .. h0 + 3 of batch row b
    int b, c, h0;
};
__device__ __forceinline__ ItemPos item_pos(const Args& a, int item) {
    ItemPos p;
    p.h0 = (item % a.HG) * 4;
    p.c = (item / a.HG) % a.NC;
    p.b = item / (a.HG * a.NC);
    return p;
}

// Record of one (token, head): {a_re | a_im | vg_re, vg_im | beta, sel_C}: the transition as two floats (bf16
// values like the reference's storage unless the caller asked for a float32 transition), the rest as bf16
// pairs.  Layout (B, blocks of 32 tokens, H, 32): the 32 tokens of a head's
// sub-block are contiguous, so a warp fetches its step with one 512-byte load.
__device__ __forceinline__ size_t rec_index(const Args& a, int steps, int b, int c, int sub, int hd, int tl) {
    return ((((size_t)b * a.NC + c) * steps + sub) * a.H + hd) * kSub + tl;
}

// ------------------------------------------------------------------------------------------
// Producer warp: TMA loads and the Gram UMMAs, strictly in step order.  The block's work is a flat sequence
// of sub-block steps g; step g uses K slot g & 1, the single Q buffer and the single set of tensor-memory columns.
// ------------------------------------------------------------------------------------------
template <int kD, bool kOutput>
__device__ __forceinline__ void producer(Smem<kD, kOutput>& sm, const CUtensorMap* tmK, const CUtensorMap* tmQ,
                                         const Args& a) {
    using DM = Dims<kD>;
    using TC = Cols<kOutput>;
    constexpr int kSteps = DM::kSteps;
    volatile int* ab = &sm.abort_flag;
    const uint32_t tm = sm.tmem_base;
    constexpr uint32_t idesc = umma_idesc_bf16(128, 128, false, false);
    const int n_items = ((int)blockIdx.x < a.items) ? (a.items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int NS = n_items * kSteps;
    if (NS == 0) return;
    // loads requested whose completion this warp has not observed yet (drained if the kernel gives up)
    int pend_k[2] = {-1, -1}, pend_q = -1;   // parity of the pending phase, -1: none
    int code = 0;
    auto load_tile = [&](uint8_t* dst, const CUtensorMap* tmap, uint64_t* bar, int g) {
        const ItemPos p = item_pos(a, (int)blockIdx.x + (g / kSteps) * (int)gridDim.x);
        const int l0 = p.c * kD + (g % kSteps) * kSub;
        if (elect_one_sync()) {
            mbar_arrive_expect_tx(bar, DM::kTile);
#pragma unroll 1
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int s = 0; s < DM::kSlabs; s++)
                    tma_load_4d(dst + s * kSlab + j * kSub * 128, tmap, bar, 64 * s, p.h0 + j, l0, p.b);
        }
        __syncwarp();
    };
    auto wait = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, mbar_wait_suspend(bar, parity, ab, a.wait_ns));
    };
    const uint32_t lK[2] = {desc_lo_sw128(smem_u32(sm.k[0]), 16), desc_lo_sw128(smem_u32(sm.k[1]), 16)};
    const uint32_t lQ = desc_lo_sw128(smem_u32(sm.q), 16);
    constexpr uint32_t kSlabJump = (kSlab >> 4) - 8;   // from the fourth k-step of a slab to the next slab
    // G = K K^T / P = Q K^T of step g: one UMMA (N = 128) per 16-column k-step.  All four heads' rows against
    // all four heads' rows; only the 32 x 32 diagonal blocks are read (head j: lanes 32 j.., columns 32 j..).
    // A single full-width UMMA reads its operands once per k-step and takes less tensor-pipe and
    // shared-memory time than lane-masked half-width ones, although three quarters of its output go unused.
    auto issue_g = [&](int g) {
        tc_fence_after();
        uint32_t ak = lK[g & 1];
#pragma unroll 1
        for (int j = 0; j < DM::kKs; j++) {
            umma_bf16_elect(tm + TC::kG, ak, ak, idesc, j);
            ak += ((j & 3) == 3) ? 2 + kSlabJump : 2;
        }
        umma_commit_elect(&sm.mma_g);
    };
    auto issue_p = [&](int g) {
        tc_fence_after();
        uint32_t ak = lK[g & 1], aq = lQ;
#pragma unroll 1
        for (int j = 0; j < DM::kKs; j++) {
            umma_bf16_elect(tm + TC::kP, aq, ak, idesc, j);
            const uint32_t adv = ((j & 3) == 3) ? 2 + kSlabJump : 2;
            ak += adv;
            aq += adv;
        }
        umma_commit_elect(&sm.mma_p);
    };
    if (!a.withhold) {
        load_tile(sm.k[0], tmK, &sm.full_k[0], 0); pend_k[0] = 0;
        if (kOutput) { load_tile(sm.q, tmQ, &sm.full_q, 0); pend_q = 0; }
        if (NS > 1) { load_tile(sm.k[1], tmK, &sm.full_k[1], 1); pend_k[1] = 0; }
        do {
            if (!wait(&sm.full_k[0], 0)) { code = 1; break; }
            pend_k[0] = -1;
            issue_g(0);
            if (kOutput) {
                if (!wait(&sm.full_q, 0)) { code = 2; break; }
                pend_q = -1;
                issue_p(0);
            }
            for (int g = 0; g < NS; g++) {
                const int n = g + 1;   // the step whose Gram blocks are issued in this iteration
                if (n < NS) {
                    if (kOutput) {   // every warp has taken rho and |q| of step g from the Q tile (and P has read it)
                        if (!wait(&sm.q_free, g & 1)) { code = 3; break; }
                        load_tile(sm.q, tmQ, &sm.full_q, n); pend_q = n & 1;
                    }
                    // every warp has G and P of step g in registers
                    if (!wait(&sm.taken, g & 1)) { code = 6; break; }
                    if (!wait(&sm.full_k[n & 1], (n >> 1) & 1)) { code = 4; break; }
                    pend_k[n & 1] = -1;
                    issue_g(n);
                    if (kOutput) {
                        if (!wait(&sm.full_q, n & 1)) { code = 5; break; }
                        WA_PSTAMP(n, 13);
                        pend_q = -1;
                        issue_p(n);
                        WA_PSTAMP(n, 14);
                    }
                }
                if (g + 2 < NS) {   // K slot of step g is free once every warp has finished its state update
                    if (!wait(&sm.k_free[g & 1], (g >> 1) & 1)) { code = 7; break; }
                    WA_PSTAMP(g + 2, 15);
                    load_tile(sm.k[g & 1], tmK, &sm.full_k[g & 1], g + 2); pend_k[g & 1] = ((g + 2) >> 1) & 1;
                }
            }
        } while (0);
    } else {
        // test hook: nothing is issued; wait until a compute warp has given up (or the limit has passed)
        const uint64_t t0 = global_ns();
        while (!*ab && global_ns() - t0 < 2 * a.wait_ns) __nanosleep(256);
        code = *ab ? 0 : 9;
    }
    if (code || *ab) {
        *ab = 1;
        if (elect_one_sync()) {   // the lane that issues the UMMAs and the TMA loads
            if (code) atomicCAS(a.status, 0, 300 + code);
            umma_commit(&sm.drain);
            int never = 0;
            mbar_wait_ns(&sm.drain, 0, &never, a.wait_ns);
            if (pend_k[0] >= 0) mbar_wait_ns(&sm.full_k[0], pend_k[0], &never, a.wait_ns);
            if (pend_k[1] >= 0) mbar_wait_ns(&sm.full_k[1], pend_k[1], &never, a.wait_ns);
            if (pend_q >= 0) mbar_wait_ns(&sm.full_q, pend_q, &never, a.wait_ns);
        }
    }
    __syncwarp();
}

// ------------------------------------------------------------------------------------------
// Compute warps.
//
// Scaled unknowns.  With W_t = a_0 ... a_t (inside the sub-block) the decay between two tokens is the
// ratio Gamma[t,i] = W_t / W_i, so the system (I + M) u = b, M[t,i] = beta_t Gamma[t,i] G[t,i], becomes in
// u^_i = u_i / W_i the REAL unit-lower-triangular system
//     u^_t = b_t / W_t - beta_t sum_{i<t} G[t,i] u^_i
// with complex right-hand sides only, and the in-block read-out becomes two real-matrix products
//     sum_{i<t} P[t,i] Gamma[t,i] u_i = W_t sum_{i<t} P[t,i] u^_i   (correction: W0_t, before its step).
// One pass over the columns does both: per column four shuffles and eight FMAs.  The scaling needs
// 1 / W_t, so a sub-block whose |W| gets small (strong decay; the zero padding behind the sequence end)
// takes the slower walk that builds the decay products explicitly (robust_block).
// ------------------------------------------------------------------------------------------
struct Tok {   // per-token quantities of one sub-block step, prepared one step ahead
    cplx at, vg;        // a_t, vp-scaled value
    cplx viw;           // vg / D_t
    cplx D, D0;         // scaling of token t and of token t - 1
    cplx R, D31;        // reference product W_15 and D of the last token
    cplx W31;           // D31 R: product of a over the sub-block
    float be, sc;       // beta_t, sel_C gate
    bool fast;
};

// Unpacks the token's record and forms the decay scalings of the sub-block.  The scaled walk only needs
// ratios W_t / W_i of the prefix products W_t = a_0 ... a_t, so they are taken relative to the middle of the
// sub-block, D_t = W_t / W_15: lanes 0-15 hold the suffix product a_{t+1} ... a_15 = 1 / D_t, lanes 16-31 the
// prefix product a_16 ... a_t = D_t, and neither half leaves the float range unless one half alone decays by
// more than 1e-30 (then, or with the zero padding behind the sequence end, the explicit walk is taken).
__device__ __forceinline__ Tok prepare(const uint4& rec, int tl) {
    Tok k;
    k.at = {__uint_as_float(rec.x), __uint_as_float(rec.y)};
    k.vg = {bf_lo(rec.z), bf_hi(rec.z)};
    k.be = bf_lo(rec.w);
    k.sc = bf_hi(rec.w);
    const bool lo = tl < 16;
    // lanes < 16: exclusive suffix product inside the first half; lanes >= 16: inclusive prefix inside the second
    cplx X = k.at;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
        const cplx other = cshfl(X, lo ? tl + o : tl - o);
        const bool take = lo ? (tl + o < 16) : (tl - o >= 16);
        if (take) X = cmul(X, other);
    }
    const cplx incl0 = cshfl(X, 0);              // a_0 ... a_15 = W_15
    cplx E = cshfl(X, tl + 1);                   // first half: exclusive suffix = inclusive suffix of lane t + 1
    if (tl == 15) E = {1.f, 0.f};
    if (!lo) E = X;
    // E: 1 / D_t (first half) or D_t (second half); one complex reciprocal gives the other
    const float m = fmaxf(fabsf(E.r), fabsf(E.i));
    const bool in_range = m >= 1e-30f && m <= 1e30f;
    const float sc1 = __fdividef(1.f, m);
    const cplx En = {E.r * sc1, E.i * sc1};
    const float q = __fdividef(sc1, En.r * En.r + En.i * En.i);
    const cplx Einv = {En.r * q, -En.i * q};
    k.D = lo ? Einv : E;
    const cplx Dinv = lo ? E : Einv;
    k.viw = cmul(k.vg, Dinv);
    k.R = incl0;
    k.D31 = cshfl(k.D, 31);
    k.D0 = cshfl(k.D, tl - 1);                   // lane 0 never uses it (W0 = 1 there)
    const float mr = fmaxf(fabsf(incl0.r), fabsf(incl0.i));
    k.fast = __all_sync(0xffffffffu, in_range && mr >= 1e-30f && mr <= 1e30f);
    k.W31 = cmul(k.D31, k.R);                    // both factors are plain products of a: valid for any a
    return k;
}

struct BlockOut {   // what a sub-block walk hands back
    cplx wh, xh;    // omega columns: Gamma[31,t] u~_t and -Gamma[31,t] x~_t
    cplx ysum;      // read-out without the rho terms (before the |q|^-1 factor)
    cplx yW, yW0;   // factors of rho_z and rho_r in the read-out
    float pd;       // P_raw[t,t]
};

// The walk with explicit decay products (any a, including zeros): phases A (coefficients
// cc[i] = a_t Gamma0[t,i] G_raw[t,i], Gamma0 built leftwards from the diagonal), B (substitution for
// u~ = n u, x~ = n x) and C (in-block read-out; the correction is read before its step,
// exact_correction.cu:90-94).  Reads G / P from tensor memory itself, eight columns at a time.
template <bool kOutput>
__device__ __noinline__ BlockOut robust_block(uint32_t tg, uint32_t tp, int tl, cplx at, cplx vg, float be, float nt,
                                              cplx kz, cplx kr) {
    const float bnn = be * nt * nt;
    cplx W = at, S = at;   // inclusive prefix / suffix products of a over the sub-block
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        cplx up = {__shfl_up_sync(0xffffffffu, W.r, o), __shfl_up_sync(0xffffffffu, W.i, o)};
        cplx dn = {__shfl_down_sync(0xffffffffu, S.r, o), __shfl_down_sync(0xffffffffu, S.i, o)};
        if (tl >= o) W = cmul(W, up);
        if (tl + o < 32) S = cmul(S, dn);
    }
    cplx W0 = {__shfl_up_sync(0xffffffffu, W.r, 1), __shfl_up_sync(0xffffffffu, W.i, 1)};
    if (tl == 0) W0 = {1.f, 0.f};
    cplx V = {__shfl_down_sync(0xffffffffu, S.r, 1), __shfl_down_sync(0xffffffffu, S.i, 1)};
    if (tl == 31) V = {1.f, 0.f};
    cplx cc[32];   // indexed with run-time group numbers on purpose: local memory, this walk is rarely taken
    {
        cplx cur = {1.f, 0.f};
#pragma unroll 1
        for (int grp = 3; grp >= 0; grp--) {
            float g8[8];
            tmem_ld8(tg + grp * 8, g8);
#pragma unroll
            for (int e = 7; e >= 0; e--) {
                const int i = grp * 8 + e;
                const cplx ai = cshfl(at, i);
                const bool on = i < tl;
                const cplx fg = cmul(at, cur);
                cc[i] = {on ? fg.r * g8[e] : 0.f, on ? fg.i * g8[e] : 0.f};
                const cplx nx = cmul(cur, ai);
                cur = {on ? nx.r : cur.r, on ? nx.i : cur.i};
            }
        }
    }
    const cplx wkz = cmul(W, kz), wkr = cmul(W, kr);
    cplx cw = {nt * be * (vg.r - nt * wkz.r), nt * be * (vg.i - nt * wkz.i)};
    cplx cx = {nt * be * nt * wkr.r, nt * be * nt * wkr.i};
#pragma unroll 1
    for (int grp = 0; grp < 4; grp++) {
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int i = grp * 8 + e;
            const float cr_ = bnn * cc[i].r, ci_ = bnn * cc[i].i;
            const cplx uw = cshfl(cw, i), ux = cshfl(cx, i);
            cw.r -= cr_ * uw.r - ci_ * uw.i;
            cw.i -= cr_ * uw.i + ci_ * uw.r;
            cx.r -= cr_ * ux.r - ci_ * ux.i;
            cx.i -= cr_ * ux.i + ci_ * ux.r;
        }
    }
    BlockOut o;
    o.wh = cmul(V, cw);
    const cplx xv = cmul(V, cx);
    o.xh = {-xv.r, -xv.i};
    o.ysum = {0.f, 0.f};
    o.pd = 0.f;
    o.yW = W;
    o.yW0 = W0;
    if (kOutput) {
        cplx yin = {0.f, 0.f};
        float pd = 0.f;
        cplx cur = {1.f, 0.f};
#pragma unroll 1
        for (int grp = 3; grp >= 0; grp--) {
            float p8[8];
            tmem_ld8(tp + grp * 8, p8);
#pragma unroll
            for (int e = 7; e >= 0; e--) {
                const int i = grp * 8 + e;
                const cplx ai = cshfl(at, i);
                const cplx uw = cshfl(cw, i), ux = cshfl(cx, i);
                const bool on = i < tl;
                pd = (i == tl) ? p8[e] : pd;
                const cplx au = cmul(at, uw);
                const cplx ee = cmul(cur, cplx{au.r - ux.r, au.i - ux.i});
                const float pi = on ? p8[e] : 0.f;
                yin.r += pi * ee.r;
                yin.i += pi * ee.i;
                const cplx nx = cmul(cur, ai);
                cur = {on ? nx.r : cur.r, on ? nx.i : cur.i};
            }
        }
        o.ysum = {pd * cw.r + yin.r, pd * cw.i + yin.i};
        o.pd = pd;
    }
    return o;
}

// x[idx] for a lane-dependent idx in 0 .. 31 without run-time register indexing: a binary tree of selects
__device__ __forceinline__ float pick32(const float (&x)[32], int idx) {
    float a[16], b[8], c[4];
#pragma unroll
    for (int j = 0; j < 16; j++) a[j] = (idx & 1) ? x[2 * j + 1] : x[2 * j];
#pragma unroll
    for (int j = 0; j < 8; j++) b[j] = (idx & 2) ? a[2 * j + 1] : a[2 * j];
#pragma unroll
    for (int j = 0; j < 4; j++) c[j] = (idx & 4) ? b[2 * j + 1] : b[2 * j];
    const float d0 = (idx & 8) ? c[1] : c[0], d1 = (idx & 8) ? c[3] : c[2];
    return (idx & 16) ? d1 : d0;
}

// bf16 pair for an mma operand from two fp32 values split as x = hi + lo with hi = x truncated to bf16 (exact
// in fp32, so lo = x - hi is exact too) and lo truncated to bf16 in turn: hi + lo carries 16 significant bits.
// low = false gives the pair of high parts, low = true the pair of low parts.  Truncation keeps the whole split
// on the integer and FMA pipes (mask, subtract, byte permute) - no conversion instructions.
__device__ __forceinline__ uint32_t split_pack(float x0, float x1, bool low) {
    const uint32_t m = low ? 0xffff0000u : 0u;
    const float r0 = x0 - __uint_as_float(__float_as_uint(x0) & m);
    const float r1 = x1 - __uint_as_float(__float_as_uint(x1) & m);
    return __byte_perm(__float_as_uint(r0), __float_as_uint(r1), 0x7632);   // {r1[31:16], r0[31:16]}
}

template <int kD, bool kOutput>
__device__ __forceinline__ void compute(Smem<kD, kOutput>& sm, const Args& a) {
    using DM = Dims<kD>;
    using TC = Cols<kOutput>;
    constexpr int kKs = DM::kKs, kSteps = DM::kSteps;
    volatile int* ab = &sm.abort_flag;
    const int t = threadIdx.x, J = t >> 5, tl = t & 31;
    // fragment coordinates of this lane: state row n' = grp >> 1 (z_re, z_im, r_re, r_im), bf16 part grp & 1
    const int grp = tl >> 2, tig = tl & 3, np = grp >> 1;
    const bool low = (grp & 1) != 0;
    const int H = a.H, L = a.L;
    const uint32_t tlane = sm.tmem_base + ((uint32_t)(J * 32) << 16) + 32 * J;
    const int n_items = ((int)blockIdx.x < a.items) ? (a.items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int NS = n_items * kSteps;
    if (NS == 0) return;
    auto wait = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, mbar_wait_suspend(bar, parity, ab, a.wait_ns));
    };
    int code = 0;
    // State of the warp's head in fragment layout: S[ks][e] is row n', column 16 ks + 2 tig + (e & 1) + 8 (e >> 1)
    float S[kKs][4];
    cplx gam = {1.f, 0.f};
    float* scr = sm.scr[J];
    float* qs = sm.qs[J];
    float* om = sm.om[J];
    // ldmatrix addressing inside a tile: lane l supplies row (l & 7) + 8 ((l >> 3) & 1) of a 16-row group and
    // the 16-byte piece (l >> 4) of a 16-column k-step; pieces are swizzled with the row (128-byte swizzle)
    const int lrow = (tl & 7) + ((tl >> 3) & 1) * 8;
    const uint32_t row_off[2] = {(uint32_t)(J * 32 + lrow) * 128u, (uint32_t)(J * 32 + 16 + lrow) * 128u};
    const uint32_t sw = (uint32_t)(lrow & 7), piece = (uint32_t)(tl >> 4);
    auto frag_addr = [&](uint32_t tile, int mt, int ks) {
        return tile + (uint32_t)(ks >> 2) * kSlab + row_off[mt] + ((((uint32_t)(ks & 3) * 2 + piece) ^ sw) << 4);
    };
    const uint32_t ktile[2] = {smem_u32(sm.k[0]), smem_u32(sm.k[1])};
    const uint32_t qtile = smem_u32(sm.q);

    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    ItemPos cur = item_pos(a, blockIdx.x), nxi = cur;
    Tok tk;
    {
        const bool valid = cur.c * kD + tl < L;
        const uint4 first = valid ? __ldg(a.rec + rec_index(a, kSteps, cur.b, cur.c, 0, cur.h0 + J, tl)) : zero4;
        tk = prepare(first, tl);
    }
    for (int g = 0; g < NS; g++) {
        const int st = g & 1;
        const uint32_t ph2 = (g >> 1) & 1;
        const int step = g % kSteps;
        if (step == 0) {
            if (g > 0) cur = nxi;
            nxi = item_pos(a, (int)blockIdx.x + (g / kSteps + 1) * (int)gridDim.x);
        }
        const int l = cur.c * kD + step * kSub + tl, hd = cur.h0 + J;
        const bool valid = l < L;
        const size_t unit = ((size_t)cur.b * a.NC + cur.c) * H + hd;   // workspace slot of this head's chunk
        if (step == 0) {   // states at the chunk start: z = 0, r = the chunk's carry
            const float* s = a.ws_state + unit * 2 * kD + (size_t)(np & 1) * kD;
#pragma unroll
            for (int ks = 0; ks < kKs; ks++) {
                float2 v0 = make_float2(0.f, 0.f), v1 = v0;
                if (kOutput && np >= 2) {
                    v0 = *reinterpret_cast<const float2*>(s + 16 * ks + 2 * tig);
                    v1 = *reinterpret_cast<const float2*>(s + 16 * ks + 8 + 2 * tig);
                }
                S[ks][0] = v0.x; S[ks][1] = v0.y; S[ks][2] = v1.x; S[ks][3] = v1.y;
            }
            gam = {1.f, 0.f};
        }
        // ---- fetch the record of step g + 1 (the next item's first sub-block after this item's last)
        uint4 rec = zero4;
        if (g + 1 < NS) {
            const ItemPos& np_ = (step + 1 < kSteps) ? cur : nxi;
            const int nsub = (step + 1) % kSteps;
            if (np_.c * kD + nsub * kSub + tl < L)
                rec = __ldg(a.rec + rec_index(a, kSteps, np_.b, np_.c, nsub, np_.h0 + J, tl));
        }
        const cplx at = tk.at, vg = tk.vg;
        const float be = tk.be;
        WA_STAMP(0);
        // ---- rho = Q S^T, |q|^2 = diag(Q Q^T), kappa = K S^T on this warp's 32 tile rows.  The Q tile goes first
        // and is handed back at once: its single buffer is what the next step's load is waiting for.
        uint32_t bfrag[kKs][2];
#pragma unroll
        for (int ks = 0; ks < kKs; ks++) {
            bfrag[ks][0] = split_pack(S[ks][0], S[ks][1], low);
            bfrag[ks][1] = split_pack(S[ks][2], S[ks][3], low);
        }
        WA_STAMP(12);
        float ak[2][4], aq[2][4], qa[2][4], qb[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int e = 0; e < 4; e++) ak[mt][e] = aq[mt][e] = qa[mt][e] = qb[mt][e] = 0.f;
        if (kOutput) {
            if (!wait(&sm.full_q, g & 1)) { code = 12; break; }
            WA_STAMP(1);
            // fragments of k-step ks + 1 are requested before the products of k-step ks are issued
            uint32_t fq[2][2][4];
            ldsm_x4(frag_addr(qtile, 0, 0), fq[0][0]);
            ldsm_x4(frag_addr(qtile, 1, 0), fq[0][1]);
#pragma unroll
            for (int ks = 0; ks < kKs; ks++) {
                const int cb = ks & 1, nb = cb ^ 1;
                if (ks + 1 < kKs) {
                    ldsm_x4(frag_addr(qtile, 0, ks + 1), fq[nb][0]);
                    ldsm_x4(frag_addr(qtile, 1, ks + 1), fq[nb][1]);
                }
#pragma unroll
                for (int mt = 0; mt < 2; mt++) {
                    mma_bf16_m16n8k16(aq[mt], fq[cb][mt], bfrag[ks][0], bfrag[ks][1]);
                    mma_bf16_m16n8k16(qa[mt], fq[cb][mt], fq[cb][mt][0], fq[cb][mt][2]);   // rows x tokens 0-7
                    mma_bf16_m16n8k16(qb[mt], fq[cb][mt], fq[cb][mt][1], fq[cb][mt][3]);   // rows x tokens 8-15
                }
            }
            // P of this step was issued a step ago: it has long finished reading the Q tile
            if (!wait(&sm.mma_p, g & 1)) { code = 14; break; }
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.q_free);
        }
        if (!wait(&sm.full_k[st], ph2)) { code = 11; break; }
        if (!kOutput) WA_STAMP(1);
        {
            uint32_t fa[2][2][4];
            ldsm_x4(frag_addr(ktile[st], 0, 0), fa[0][0]);
            ldsm_x4(frag_addr(ktile[st], 1, 0), fa[0][1]);
#pragma unroll
            for (int ks = 0; ks < kKs; ks++) {
                const int cb = ks & 1, nb = cb ^ 1;
                if (ks + 1 < kKs) {
                    ldsm_x4(frag_addr(ktile[st], 0, ks + 1), fa[nb][0]);
                    ldsm_x4(frag_addr(ktile[st], 1, ks + 1), fa[nb][1]);
                }
                mma_bf16_m16n8k16(ak[0], fa[cb][0], bfrag[ks][0], bfrag[ks][1]);
                mma_bf16_m16n8k16(ak[1], fa[cb][1], bfrag[ks][0], bfrag[ks][1]);
            }
        }
        WA_STAMP(2);
        // accumulator element (row grp / grp + 8, column 2 tig + {0, 1}): columns are {hi, lo} of state row tig
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            scr[(16 * mt + grp) * 12 + tig] = ak[mt][0] + ak[mt][1];
            scr[(16 * mt + grp + 8) * 12 + tig] = ak[mt][2] + ak[mt][3];
            if (kOutput) {
                scr[(16 * mt + grp) * 12 + 4 + tig] = aq[mt][0] + aq[mt][1];
                scr[(16 * mt + grp + 8) * 12 + 4 + tig] = aq[mt][2] + aq[mt][3];
                if (tig == (grp >> 1)) {   // the diagonal of the 16 x 16 block sits with this lane
                    qs[16 * mt + grp] = (grp & 1) ? qa[mt][1] : qa[mt][0];
                    qs[16 * mt + grp + 8] = (grp & 1) ? qb[mt][3] : qb[mt][2];
                }
            }
        }
        __syncwarp();
        const float4 kap = *reinterpret_cast<const float4*>(scr + tl * 12);
        float4 rho = make_float4(0.f, 0.f, 0.f, 0.f);
        float mt_ = 0.f;
        if (kOutput) {
            rho = *reinterpret_cast<const float4*>(scr + tl * 12 + 4);
            mt_ = rsqrtf(qs[tl] + kEps);
        }
        const cplx kz = {kap.x, kap.y}, kr = {kap.z, kap.w};
        WA_STAMP(3);
        // ---- Gram rows of the own head from tensor memory: |k_t|^-1 from the diagonal
        if (!wait(&sm.mma_g, g & 1)) { code = 13; break; }
        tc_fence_after();
        WA_STAMP(4);
        const uint32_t tg = tlane + TC::kG, tp = tlane + TC::kP;
        float gs[32], p[32];
        tmem_ld32(tg, gs);
        WA_STAMP(5);
        float pd = 0.f;
        const float gd = pick32(gs, tl);
        const float nt = rsqrtf(gd + kEps);
        const float bnn = be * nt * nt;
        BlockOut o;
        if (tk.fast) {
            if (kOutput) tmem_ld32(tp, p);
            tc_fence_before();
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.taken);   // G and P are in registers, rho and |q| have been taken from the Q tile
#pragma unroll
            for (int i = 0; i < 32; i++) gs[i] *= -bnn;
            const cplx rkz = cmul(tk.R, kz);
            cplx cw = {nt * be * (tk.viw.r - nt * rkz.r), nt * be * (tk.viw.i - nt * rkz.i)};
            if (kOutput) {
                const cplx rkr = cmul(tk.R, kr);
                cplx cx = {nt * be * nt * rkr.r, nt * be * nt * rkr.i};
                pd = pick32(p, tl);
                cplx accu = {0.f, 0.f}, accx = {0.f, 0.f};
                WA_STAMP(6);
                // column i: the finished unknown of token i goes to the tokens behind it (rows t > i only)
#pragma unroll
                for (int i = 0; i < 31; i++) {
                    const cplx uw = cshfl(cw, i), ux = cshfl(cx, i);
                    if (tl > i) {
                        cw.r = fmaf(gs[i], uw.r, cw.r);
                        cw.i = fmaf(gs[i], uw.i, cw.i);
                        cx.r = fmaf(gs[i], ux.r, cx.r);
                        cx.i = fmaf(gs[i], ux.i, cx.i);
                        accu.r = fmaf(p[i], uw.r, accu.r);
                        accu.i = fmaf(p[i], uw.i, accu.i);
                        accx.r = fmaf(p[i], ux.r, accx.r);
                        accx.i = fmaf(p[i], ux.i, accx.i);
                    }
                }
                WA_STAMP(7);
                const cplx xv = cmul(tk.D31, cx);
                o.xh = {-xv.r, -xv.i};
                // y = D (R rho_z + pd u^ + accu) + D0 (R rho_r - accx); lane 0: W0 = 1, the carried correction itself
                const cplx yl = cmul(tk.D, cplx{pd * cw.r + accu.r, pd * cw.i + accu.i});
                cplx yc = cmul(tk.D0, cplx{-accx.r, -accx.i});
                if (tl == 0) yc = {0.f, 0.f};
                o.ysum = {yl.r + yc.r, yl.i + yc.i};
                o.yW = cmul(tk.D, tk.R);
                o.yW0 = cmul(tk.D0, tk.R);
                if (tl == 0) o.yW0 = {1.f, 0.f};
                o.pd = pd;
            } else {
                WA_STAMP(6);
#pragma unroll
                for (int i = 0; i < 31; i++) {
                    const cplx uw = cshfl(cw, i);
                    if (tl > i) {
                        cw.r = fmaf(gs[i], uw.r, cw.r);
                        cw.i = fmaf(gs[i], uw.i, cw.i);
                    }
                }
                WA_STAMP(7);
                o.xh = {0.f, 0.f};
            }
            o.wh = cmul(tk.D31, cw);
        } else {
            o = robust_block<kOutput>(tg, tp, tl, at, vg, be, nt, kz, kr);
            tc_fence_before();
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.taken);
        }
        // ---- read-out
        if (kOutput) {
            const cplx rz = cmul(o.yW, cplx{rho.x, rho.y});
            const cplx rr = cmul(o.yW0, cplx{rho.z, rho.w});
            float yr = mt_ * (o.ysum.r + rz.r + rr.r), yi = mt_ * (o.ysum.i + rz.i + rr.i);
            if (a.shortcut_scale != 0.f) {   // block.py:202-208
                const float qk = mt_ * nt * o.pd;
                yr += a.shortcut_scale * qk * qk * vg.r;
                yi += a.shortcut_scale * qk * qk * vg.i;
            }
            if (valid) {
                __nv_bfloat162 ov = __floats2bfloat162_rn(bfr(yr) * tk.sc, bfr(yi) * tk.sc);
                *reinterpret_cast<__nv_bfloat162*>(a.y + (((size_t)cur.b * L + l) * H + hd) * 2) = ov;
            }
        }
        WA_STAMP(8);
        // ---- state update S <- W_31 S + Omega K: not needed after the last sub-block of the output pass
        const cplx W31 = tk.W31;
        if (!kOutput || step + 1 < kSteps) {
            om[tl] = o.wh.r;
            om[32 + tl] = o.wh.i;
            if (kOutput) {
                om[64 + tl] = o.xh.r;
                om[96 + tl] = o.xh.i;
            }
            __syncwarp();
            // A fragments: row grp (and its duplicate) carries the high parts of omega[n'], row grp + 8 the low parts
            uint32_t fo[2][4];
#pragma unroll
            for (int kk = 0; kk < 2; kk++) {
                float2 x0 = make_float2(0.f, 0.f), x1 = x0;
                if (kOutput || np < 2) {
                    x0 = *reinterpret_cast<const float2*>(om + np * 32 + 16 * kk + 2 * tig);
                    x1 = *reinterpret_cast<const float2*>(om + np * 32 + 16 * kk + 8 + 2 * tig);
                }
                fo[kk][0] = split_pack(x0.x, x0.y, false);
                fo[kk][1] = split_pack(x0.x, x0.y, true);
                fo[kk][2] = split_pack(x1.x, x1.y, false);
                fo[kk][3] = split_pack(x1.x, x1.y, true);
            }
            WA_STAMP(9);
            // decay: complex product with W_31; the other part of the complex row sits eight lanes away
            const float wr = W31.r, wi = (np & 1) ? W31.i : -W31.i;
#pragma unroll
            for (int ks = 0; ks < kKs; ks++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float other = __shfl_xor_sync(0xffffffffu, S[ks][e], 8);
                    S[ks][e] = wr * S[ks][e] + wi * other;
                }
            uint32_t fb[2][2][4];
            ldsm_x4_trans(frag_addr(ktile[st], 0, 0), fb[0][0]);
            ldsm_x4_trans(frag_addr(ktile[st], 1, 0), fb[0][1]);
#pragma unroll
            for (int ks = 0; ks < kKs; ks++) {
                const int cb = ks & 1, nb = cb ^ 1;
                if (ks + 1 < kKs) {
                    ldsm_x4_trans(frag_addr(ktile[st], 0, ks + 1), fb[nb][0]);
                    ldsm_x4_trans(frag_addr(ktile[st], 1, ks + 1), fb[nb][1]);
                }
                float c0[4] = {S[ks][0], S[ks][1], 0.f, 0.f}, c1[4] = {S[ks][2], S[ks][3], 0.f, 0.f};
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    mma_bf16_m16n8k16(c0, fo[kk], fb[cb][kk][0], fb[cb][kk][1]);
                    mma_bf16_m16n8k16(c1, fo[kk], fb[cb][kk][2], fb[cb][kk][3]);
                }
                S[ks][0] = c0[0] + c0[2]; S[ks][1] = c0[1] + c0[3];
                S[ks][2] = c1[0] + c1[2]; S[ks][3] = c1[1] + c1[3];
            }
            gam = cmul(W31, gam);
        }
        __syncwarp();
        WA_STAMP(10);
        if (tl == 0) mbar_arrive(&sm.k_free[st]);
        if (!kOutput && step + 1 == kSteps) {
            // the carry pass consumes these as the reference's bf16 cum_A[:, -1] / local_h[:, -1]
            if (!low && np < 2) {
                float* s = a.ws_state + unit * 2 * kD + (size_t)np * kD;
#pragma unroll
                for (int ks = 0; ks < kKs; ks++) {
                    *reinterpret_cast<float2*>(s + 16 * ks + 2 * tig) = make_float2(bfr(S[ks][0]), bfr(S[ks][1]));
                    *reinterpret_cast<float2*>(s + 16 * ks + 8 + 2 * tig) = make_float2(bfr(S[ks][2]), bfr(S[ks][3]));
                }
            }
            if (tl == 0) {
                a.ws_gamma[unit * 2] = bfr(gam.r);
                a.ws_gamma[unit * 2 + 1] = bfr(gam.i);
            }
        }
        if (g + 1 < NS) tk = prepare(rec, tl);
        WA_STAMP(11);
    }
    if (code && tl == 0) atomicCAS(a.status, 0, 200 + code);
}

template <int kD, bool kOutput>
__global__ void __launch_bounds__(kThreads, kOutput ? 2 : (kD == 128 ? 3 : 4))
scan_wa_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ, const Args a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    Smem<kD, kOutput>& sm = *reinterpret_cast<Smem<kD, kOutput>*>(smem_raw);
    const int warp = threadIdx.x >> 5;
    if ((smem_u32(smem_raw) & 1023u) != 0) {   // the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicCAS(a.status, 0, 399);
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(&sm.full_k[0], 1); mbar_init(&sm.full_k[1], 1); mbar_init(&sm.full_q, 1);
        mbar_init(&sm.mma_g, 1); mbar_init(&sm.mma_p, 1); mbar_init(&sm.taken, 4); mbar_init(&sm.q_free, 4);
        mbar_init(&sm.k_free[0], 4); mbar_init(&sm.k_free[1], 4);
        mbar_init(&sm.drain, 1);
        sm.abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 4) tmem_alloc(&sm.tmem_base, Cols<kOutput>::kTotal);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp < 4) {
        compute<kD, kOutput>(sm, a);
    } else {
        if (threadIdx.x == 128) {
            prefetch_tmap(&tmK);
            if (kOutput) prefetch_tmap(&tmQ);
        }
        __syncwarp();
        producer<kD, kOutput>(sm, &tmK, &tmQ, a);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        tmem_dealloc(sm.tmem_base, Cols<kOutput>::kTotal);
    }
}

// ------------------------------------------------------------------------------------------
// Dynamics pre-pass: one thread per (token, head), heads fastest (the gate rows are read coalesced).
// dynamics_fused.cu:64-139 and the vp scale of block.py:194-195, every result rounded to bf16 like the
// reference's stores.  Both scan passes read the 16-byte records instead of repeating the transcendental
// chain inside their sequential walks.
// ------------------------------------------------------------------------------------------
struct DynArgs {
    const __nv_bfloat16 *v, *gate_raw;
    const float *log_dt_scale, *rope_freqs;
    uint4* rec;
    DynConsts dc;
    int B, L, H, NB, pos0, segs;   // NB: 32-token blocks per batch row (chunks padded to full length)
    int fp32_decay;                // 0: the transition is rounded to bf16 like the reference's A_bar store
};
__global__ void __launch_bounds__(256) wa_dynamics_kernel(const DynArgs a) {
    using T = __nv_bfloat16;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)a.B * a.L * a.H;
    if (idx >= total) return;
    const int hd = (int)(idx % a.H);
    const long long bl = idx / a.H;
    const int l = (int)(bl % a.L), b = (int)(bl / a.L);
    const int H = a.H;
    const T* gr = a.gate_raw + (size_t)bl * (size_t)(7 * H);
    const float lds = a.log_dt_scale[hd], freq = a.rope_freqs[hd];
    const float pos = (float)(l + a.pos0 + (b % a.segs) * a.L);
    const float g0 = IO<T>::ld(gr + hd), g1 = IO<T>::ld(gr + H + hd);
    DynShared ds = dyn_shared<true>(g0, g1, IO<T>::ld(gr + 2 * H + hd), IO<T>::ld(gr + 3 * H + hd),
                                    IO<T>::ld(gr + 4 * H + hd), IO<T>::ld(gr + 5 * H + hd), IO<T>::ld(gr + 6 * H + hd),
                                    lds, freq, pos, a.dc);
    float ar, ai, vp;
    dyn_pair<true>(g0, g1, freq, pos, ds, ar, ai, vp);
    vp = bfr(vp);
    if (!a.fp32_decay) {
        ar = bfr(ar);
        ai = bfr(ai);
    }
    const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(a.v + ((size_t)bl * H + hd) * 2);
    uint4 r;
    r.x = __float_as_uint(ar);
    r.y = __float_as_uint(ai);
    r.z = pack2(__low2float(v2) * vp, __high2float(v2) * vp);
    r.w = pack2(ds.beta, ds.sel_c);
    a.rec[(((size_t)b * a.NB + (l >> 5)) * H + hd) * kSub + (l & 31)] = r;
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static const EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(p);
        return static_cast<EncodeTiledFn>(nullptr);
    }();
    return fn;
}

// (B, L, H, D) bf16 tensor viewed as 4-D (D, H, L, B); box = 64 columns x 1 head x 32 positions.
static bool make_tile_map(CUtensorMap* m, const void* base, int B, int L, int H, int D) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)H * D * 2, (cuuint64_t)L * H * D * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)kSub, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

#ifdef CDSSM_WA_TRACE
static int g_grid_override = 0;
#endif
template <int kD, bool kOutput>
static int launch_pass(const CUtensorMap& tmK, const CUtensorMap& tmQ, const Args& a, int sms, cudaStream_t st) {
    constexpr int kBlocksPerSm = kOutput ? 2 : (kD == 128 ? 3 : 4);
    const size_t smem = sizeof(Smem<kD, kOutput>);
    if (int rc = check_cuda(cudaFuncSetAttribute(scan_wa_kernel<kD, kOutput>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem)))
        return rc;
    long long resident = (long long)kBlocksPerSm * sms;
#ifdef CDSSM_WA_TRACE
    if (g_grid_override > 0) resident = g_grid_override;
#endif
    const int grid = (int)(a.items < resident ? a.items : resident);
    scan_wa_kernel<kD, kOutput><<<grid, kThreads, smem, st>>>(tmK, tmQ, a);
    return check_launch();
}

}  // namespace wa

#ifdef CDSSM_WA_TRACE
extern "C" __attribute__((visibility("default"))) void cdssm_b200_wa_trace_grid(int n) { wa::g_grid_override = n; }
extern "C" __attribute__((visibility("default"))) int cdssm_b200_wa_trace_read(long long* host) {
    return (int)cudaMemcpyFromSymbol(host, wa::g_trace, sizeof(wa::g_trace));
}
#endif

bool scan_wa_supported(int D, int N, int C, int H, int dtype) {
    return dtype == CDSSM_BF16 && N == 2 && D == C && (D == 64 || D == 128) && H % 4 == 0;
}

size_t scan_wa_record_bytes(int B, int L, int H, int C) {
    const size_t NC = ((size_t)L + C - 1) / C;
    return (size_t)B * NC * C * H * sizeof(uint4);
}

// Dynamics pre-pass: fills rec (scan_wa_record_bytes bytes) for both scan passes.
int scan_wa_dynamics(const void* v, const void* gate_raw, const float* log_dt_scale, const float* rope_freqs,
                     void* rec, const DynConsts& dc, int B, int L, int H, int C, int pos0, int segs, int fp32_decay,
                     cudaStream_t st) {
    wa::DynArgs d;
    d.v = static_cast<const __nv_bfloat16*>(v);
    d.gate_raw = static_cast<const __nv_bfloat16*>(gate_raw);
    d.log_dt_scale = log_dt_scale; d.rope_freqs = rope_freqs;
    d.rec = static_cast<uint4*>(rec);
    d.dc = dc;
    d.B = B; d.L = L; d.H = H; d.NB = ((L + C - 1) / C) * (C / wa::kSub); d.pos0 = pos0; d.segs = segs;
    d.fp32_decay = fp32_decay;
    const long long total = (long long)B * L * H;
    wa::wa_dynamics_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(d);
    return check_launch();
}

// One pass of the warp-autonomous tensor-core scan over every chunk.  output = false: local pass (fills
// ws_state / ws_gamma for the carry pass); output = true: reads the carries from ws_state, writes y.
// status: one int in device memory, set by a bounded wait that ran out (not cleared here).
int scan_wa_pass(bool output, const void* q, const void* k, const void* rec, float* ws_gamma, float* ws_state, void* y,
                 int* status, float shortcut_scale, int B, int L, int H, int D, unsigned long long wait_ns, int withhold,
                 cudaStream_t st) {
    using namespace wa;
    CUtensorMap tmK, tmQ;
    if (!make_tile_map(&tmK, k, B, L, H, D) || !make_tile_map(&tmQ, output ? q : k, B, L, H, D)) return CDSSM_ERR_CUDA;
    int dev = 0, sms = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev))) return rc;
    if (int rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev))) return rc;
    Args a;
    a.rec = static_cast<const uint4*>(rec);
    a.ws_gamma = ws_gamma; a.ws_state = ws_state;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.status = status;
    a.wait_ns = wait_ns ? wait_ns : 400ull * 1000 * 1000;
    a.withhold = withhold;
    a.shortcut_scale = shortcut_scale;
    a.B = B; a.L = L; a.H = H; a.NC = (L + D - 1) / D;
    a.HG = H / 4;
    const long long items = (long long)B * a.NC * a.HG;
    if (items > 0x7fffffff / 8) return CDSSM_ERR_UNSUPPORTED;
    a.items = (int)items;
    if (D == 128) return output ? launch_pass<128, true>(tmK, tmQ, a, sms, st) : launch_pass<128, false>(tmK, tmQ, a, sms, st);
    return output ? launch_pass<64, true>(tmK, tmQ, a, sms, st) : launch_pass<64, false>(tmK, tmQ, a, sms, st);
}

}  // namespace cdssm
