// Fused CD-SSM scan on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), single pass over
// HBM.  Shapes: bf16 storage, state_dim N = 2 (one complex pair), head_dim D = chunk C = 128.
//
// One CTA walks one (batch, head) sequence chunk by chunk.  Per chunk of C tokens (k_t, q_t rows
// of the raw bf16 tiles, n_t / m_t their inverse norms, a_t the complex decay, beta_t, v_t):
//   G[t,i] = k_t.k_i and P[t,i] = q_t.k_i   : two C x C x D contractions on the tensor cores,
//                                             operands staged by TMA (128-byte swizzle), fp32
//                                             accumulators in tensor memory, in two column halves;
//   kappa_t = k_t.s, rho_t = q_t.s          : skinny UMMAs against the carry s (bf16, as the
//                                             reference rounds chunk_states);
//   (I + M) w = beta v,  (I + M) x = beta gamma kappa,  M[t,i] = beta_t Gamma[t,i] G[t,i]
//                                           : the chunk-local delta rule and the correction as two
//                                             triangular solves sharing M; Gamma[t,i] = prod a_r,
//                                             i < r <= t, is separable across 32-token blocks
//                                             (prefix x block products x suffix, all |.| <= 1, no
//                                             division), so only the 32 x 32 diagonal blocks need a
//                                             sequential substitution (warp shuffles), everything
//                                             else is real-matrix x complex-vector FMAs on rows
//                                             read straight from tensor memory;
//   y_t = (z_t + r_t).q_t                   : from P, w, x, rho (correction taken before step t);
//   l = sum_i Gamma[C-1,i] w_i k_i          : a third skinny UMMA (K tile as MN-major operand);
//   s <- bf16(gamma_C) s + bf16(l)          : the reference's decay-only carry.
// The algebra restates intra_chunk_scan.cu:100-195, inter_chunk_scan.cu:52-84 and
// exact_correction.cu:89-150 chunk-wise; dynamics and normalisation are fused as in scan_simt.cu
// (k and q enter the tensor cores un-normalised, the inverse norms scale the fp32 results).
//
// Roles: warps 0-3 (one thread per token / per TMEM lane) do the CUDA-core work; warp 4 issues
// TMA and UMMA.  All waits are bounded; a wait that runs out sets the status word, and every role
// unwinds through the common exit where tensor memory is freed.
#include "cdssm_common.cuh"
#include "sm100_ptx.cuh"

namespace cdssm {
using namespace sm100;

constexpr int kTcC = 128, kTcD = 128;
constexpr int kTcComputeThreads = 128, kTcThreads = 160;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColG = 0, kColP = 64, kColKappa = 128, kColRho = 144, kColEll = 160;
constexpr uint32_t kSlabBytes = kTcC * 128;        // 64 bf16 columns of 128 rows, 128 B per row
constexpr uint32_t kTileBytes = 2 * kSlabBytes;    // 32 KB: one K or Q chunk tile

struct __align__(1024) TcSmem {
    uint8_t k[2][kTileBytes];     // K tile, double buffered (TMA)
    uint8_t q[kTileBytes];        // Q tile (TMA)
    uint8_t s_tile[4096];         // UMMA B operand: rows 0,1 = bf16(s_re), bf16(s_im) over d
    uint8_t o_tile[4096];         // UMMA B operand: rows 0..3 = omega re/im hi, re/im lo over tokens
    float4 wx[kTcC];              // per token: V_t n_t w_t (xy) and V_t n_t x_t (zw)
    float2 a[2][kTcC];            // per token decay a_t (double buffered by chunk parity)
    float2 bp[2][4];              // product of a over each 32-token block
    uint64_t full_k[2], full_q, mma_gp0, mma_kr, mma_gp1, mma_ell;
    uint64_t gp0_free, gp1_free, s_ready, omega_ready, blk_done[3], bp_ready, drain;
    uint32_t tmem_base;
    int abort_flag;
};

struct TcArgs {
    const __nv_bfloat16 *v, *gate_raw;
    const float *log_dt_scale, *rope_freqs, *h0;
    __nv_bfloat16* y;
    float* final_state;
    int* status;                  // device word: 0 ok, else the code of the wait that ran out
    long long* trace;             // optional: per-phase clock64 stamps of CTA 0 (performance debugging)
    DynConsts dc;
    float shortcut_scale;
    int B, L, H, NC, pos0, segs;
};

struct cplx { float r, i; };
__device__ __forceinline__ cplx cmul(cplx a, cplx b) { return {a.r * b.r - a.i * b.i, a.r * b.i + a.i * b.r}; }
__device__ __forceinline__ cplx cshfl(cplx v, int src) {
    return {__shfl_sync(0xffffffffu, v.r, src), __shfl_sync(0xffffffffu, v.i, src)};
}

// ------------------------------------------------------------------------------------------
// Producer warp (one elected lane): TMA loads and UMMA issue for one sequence.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_producer(TcSmem& sm, const CUtensorMap* tmK, const CUtensorMap* tmQ,
                                            const TcArgs& a, int b, int hd) {
    volatile int* ab = &sm.abort_flag;
    const uint32_t tm = sm.tmem_base;
    constexpr uint32_t idesc_gp = umma_idesc_bf16(128, 64, false, false);
    constexpr uint32_t idesc_sk = umma_idesc_bf16(128, 16, false, false);
    constexpr uint32_t idesc_el = umma_idesc_bf16(128, 16, true, false);
    const uint32_t kaddr[2] = {smem_u32(sm.k[0]), smem_u32(sm.k[1])};
    const uint32_t qaddr = smem_u32(sm.q), saddr = smem_u32(sm.s_tile), oaddr = smem_u32(sm.o_tile);
    bool pend_k[2] = {false, false}, pend_q = false;   // TMA issued, not yet waited for
    int code = 0;

    auto load_k = [&](int c) {
        const int st = c & 1;
        mbar_arrive_expect_tx(&sm.full_k[st], kTileBytes);
        tma_load_4d(sm.k[st], tmK, &sm.full_k[st], 0, hd, c * kTcC, b);
        tma_load_4d(sm.k[st] + kSlabBytes, tmK, &sm.full_k[st], 64, hd, c * kTcC, b);
        pend_k[st] = true;
    };
    auto load_q = [&](int c) {
        mbar_arrive_expect_tx(&sm.full_q, kTileBytes);
        tma_load_4d(sm.q, tmQ, &sm.full_q, 0, hd, c * kTcC, b);
        tma_load_4d(sm.q + kSlabBytes, tmQ, &sm.full_q, 64, hd, c * kTcC, b);
        pend_q = true;
    };
    // K-major operand, k-step j of 8 (16 bf16 = 32 bytes each; 4 steps per 64-column slab)
    auto kmaj = [](uint32_t base, uint32_t slab_bytes, int j, uint32_t row_off) {
        return umma_desc_sw128(base + (uint32_t)(j >> 2) * slab_bytes + (uint32_t)(j & 3) * 32 + row_off, 16, 1024);
    };

    load_k(0);
    load_q(0);
    if (a.NC > 1) load_k(1);

    // Event loop: every task of every chunk is issued as soon as what it depends on has happened,
    // so the Gram UMMAs of chunk c+1 and the TMA refills run under chunk c's CUDA-core work.
    // A task's barrier is only polled before the event that could complete its NEXT phase has been
    // triggered (each such event depends on the task itself), so parity tests cannot alias.
    const int NC = a.NC;
    int i_gp0 = 0, i_kr = 0, i_gp1 = 0, i_lq = 1, i_ell = 0, i_lk = 2;
    bool k_ok = false, q_ok = false;              // tiles of chunk i_gp0 have landed
    const uint64_t t0 = global_ns();
    uint64_t last = t0;
    uint32_t idle = 0;
    auto par = [](int c) { return (uint32_t)(c & 1); };
    while (i_ell < NC) {
        bool progress = false;
        if (i_gp0 < NC) {   // pass 0: G[:, 0:64] = K K[0:64]^T ; P[:, 0:64] = Q K[0:64]^T
            const int c = i_gp0, st = c & 1;
            if (!k_ok && mbar_test(&sm.full_k[st], (c >> 1) & 1)) { k_ok = true; pend_k[st] = false; }
            if (!q_ok && mbar_test(&sm.full_q, par(c))) { q_ok = true; pend_q = false; }
            if (k_ok && q_ok && (c == 0 || mbar_test(&sm.gp1_free, par(c - 1)))) {
                tc_fence_after();
#pragma unroll 1
    #pragma unroll 1
            for (int j = 0; j < 8; j++)
                    umma_bf16(tm + kColG, kmaj(kaddr[st], kSlabBytes, j, 0), kmaj(kaddr[st], kSlabBytes, j, 0), idesc_gp, j > 0);
#pragma unroll 1
    #pragma unroll 1
            for (int j = 0; j < 8; j++)
                    umma_bf16(tm + kColP, kmaj(qaddr, kSlabBytes, j, 0), kmaj(kaddr[st], kSlabBytes, j, 0), idesc_gp, j > 0);
                umma_commit(&sm.mma_gp0);
                if (a.trace && blockIdx.x == 0 && c < 8) a.trace[(c * 5 + 4) * 16 + 0] = clock64();
                i_gp0++; k_ok = q_ok = false; progress = true;
            }
        }
        if (i_kr < i_gp0 && mbar_test(&sm.s_ready, par(i_kr))) {   // kappa = K s^T, rho = Q s^T
            const int st = i_kr & 1;
            tc_fence_after();
#pragma unroll 1
            for (int j = 0; j < 8; j++)
                umma_bf16(tm + kColKappa, kmaj(kaddr[st], kSlabBytes, j, 0), kmaj(saddr, 2048, j, 0), idesc_sk, j > 0);
#pragma unroll 1
            for (int j = 0; j < 8; j++)
                umma_bf16(tm + kColRho, kmaj(qaddr, kSlabBytes, j, 0), kmaj(saddr, 2048, j, 0), idesc_sk, j > 0);
            umma_commit(&sm.mma_kr);
            if (a.trace && blockIdx.x == 0 && i_kr < 8) a.trace[(i_kr * 5 + 4) * 16 + 1] = clock64();
            i_kr++; progress = true;
        }
        if (i_gp1 < i_kr && mbar_test(&sm.gp0_free, par(i_gp1))) {   // pass 1: columns 64..127
            const int st = i_gp1 & 1;
            tc_fence_after();
#pragma unroll 1
            for (int j = 0; j < 8; j++)
                umma_bf16(tm + kColG, kmaj(kaddr[st], kSlabBytes, j, 0), kmaj(kaddr[st], kSlabBytes, j, 64 * 128), idesc_gp, j > 0);
#pragma unroll 1
            for (int j = 0; j < 8; j++)
                umma_bf16(tm + kColP, kmaj(qaddr, kSlabBytes, j, 0), kmaj(kaddr[st], kSlabBytes, j, 64 * 128), idesc_gp, j > 0);
            umma_commit(&sm.mma_gp1);
            if (a.trace && blockIdx.x == 0 && i_gp1 < 8) a.trace[(i_gp1 * 5 + 4) * 16 + 2] = clock64();
            i_gp1++; progress = true;
        }
        // the Q tile is free once pass 1 (and, issued before it, rho) of its chunk have completed
        if (i_lq <= i_gp1 && i_lq <= NC && mbar_test(&sm.mma_gp1, par(i_lq - 1))) {
            if (i_lq < NC) load_q(i_lq);
            i_lq++; progress = true;
        }
        // l = K^T omega : A = K tile read MN-major (M = d: two 64-wide groups 16 KB apart; K = tokens,
        // 16 per step = 2 KB), B = omega tile (16 rows x 128 tokens, K-major)
        if (i_ell < i_gp1 && mbar_test(&sm.omega_ready, par(i_ell))) {
            const int st = i_ell & 1;
            tc_fence_after();
#pragma unroll 1
            for (int j = 0; j < 8; j++)
                umma_bf16(tm + kColEll, umma_desc_sw128(kaddr[st] + (uint32_t)j * 2048, kSlabBytes, 1024),
                          kmaj(oaddr, 2048, j, 0), idesc_el, j > 0);
            umma_commit(&sm.mma_ell);
            if (a.trace && blockIdx.x == 0 && i_ell < 8) a.trace[(i_ell * 5 + 4) * 16 + 3] = clock64();
            i_ell++; progress = true;
        }
        // the K stage of chunk c is free once l_c has completed
        if (i_lk - 2 < i_ell && i_lk - 2 < NC && mbar_test(&sm.mma_ell, par(i_lk - 2))) {
            if (i_lk < NC) load_k(i_lk);
            i_lk++; progress = true;
        }
        if (progress) {
            last = global_ns();
        } else if ((++idle & 7) != 0) {
            __nanosleep(32);          // do not steal issue slots from the compute warp on this scheduler
        } else if (*ab || global_ns() - last > kWaitLimitNs) {
            code = 1 + (i_gp0 > i_kr) + 2 * (i_kr > i_gp1) + 4 * (i_gp1 > i_ell);
            *ab = 1;
            break;
        }
    }
    if (code) {
        atomicCAS(a.status, 0, 100 + code);
        // let copies and UMMAs in flight land before shared and tensor memory are released
        umma_commit(&sm.drain);
        int never = 0;
        mbar_wait(&sm.drain, 0, &never);
        if (pend_k[0]) mbar_wait(&sm.full_k[0], 0, &never), mbar_wait(&sm.full_k[0], 1, &never);
        if (pend_k[1]) mbar_wait(&sm.full_k[1], 0, &never), mbar_wait(&sm.full_k[1], 1, &never);
        if (pend_q) mbar_wait(&sm.full_q, 0, &never), mbar_wait(&sm.full_q, 1, &never);
    }
}

// Element (row n, column kk) of a 16-row K-major bf16 operand tile with 128-byte swizzle:
// 64 columns per 2 KB slab, 16-byte chunk index XORed with (row mod 8).
__device__ __forceinline__ uint32_t small_tile_off(int n, int kk) {
    return (uint32_t)(kk >> 6) * 2048u + (uint32_t)n * 128u + (uint32_t)((((kk & 63) >> 3) ^ (n & 7)) << 4) +
           (uint32_t)(kk & 7) * 2u;
}
__device__ __forceinline__ void st_bf16(uint8_t* tile, uint32_t off, float x) {
    *reinterpret_cast<__nv_bfloat16*>(tile + off) = __float2bfloat16_rn(x);
}
__device__ __forceinline__ float bfr(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// all lanes of a warp wait; the outcome is made warp-uniform
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* ab) {
    const bool ok = mbar_wait(bar, parity, ab);
    return __all_sync(0xffffffffu, ok);
}

// ------------------------------------------------------------------------------------------
// Compute warps: thread t owns token t of the chunk (TMEM lane t) and column d = t of the carry.
// ------------------------------------------------------------------------------------------
struct TokenCtx {          // per-token quantities of one chunk, produced by tc_prologue
    cplx at, vg, W, W0, V, gpre, gsuf, gall, bp1, bp2;
    float be, sc, mt;
    bool valid;
};

// Everything of chunk c that does not depend on the carry or on tensor memory: dynamics of token t
// (dynamics_fused.cu:64-139; vp scale of block.py:194-195), the in-block prefix / suffix products
// of a, the block products, and |q_t|^-1 from the Q tile row.
__device__ __noinline__ bool tc_prologue(TcSmem& sm, const TcArgs& a, int b, int hd, int c, float lds,
                                            float freq, TokenCtx& x) {
    using T = __nv_bfloat16;
    volatile int* ab = &sm.abort_flag;
    const int t = threadIdx.x, J = t >> 5, tl = t & 31, H = a.H, L = a.L;
    const int l = c * kTcC + t;
    x.valid = l < L;
    x.at = {0.f, 0.f};
    x.vg = {0.f, 0.f};
    x.be = 0.f;
    x.sc = 0.f;
    if (x.valid) {
        const size_t bl = (size_t)b * L + l;
        const T* gr = a.gate_raw + bl * (size_t)(7 * H);
        const float pos = (float)(l + a.pos0 + (b % a.segs) * L);
        DynShared ds = dyn_shared<true>(IO<T>::ld(gr + hd), IO<T>::ld(gr + H + hd), IO<T>::ld(gr + 2 * H + hd),
                                        IO<T>::ld(gr + 3 * H + hd), IO<T>::ld(gr + 4 * H + hd),
                                        IO<T>::ld(gr + 5 * H + hd), IO<T>::ld(gr + 6 * H + hd), lds, freq, pos, a.dc);
        float vp;
        dyn_pair<true>(IO<T>::ld(gr + hd), IO<T>::ld(gr + H + hd), freq, pos, ds, x.at.r, x.at.i, vp);
        x.at.r = bfr(x.at.r);
        x.at.i = bfr(x.at.i);
        vp = bfr(vp);
        x.be = bfr(ds.beta);
        x.sc = bfr(ds.sel_c);
        const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(a.v + (bl * H + hd) * 2);
        x.vg.r = bfr(__low2float(v2) * vp);
        x.vg.i = bfr(__high2float(v2) * vp);
    }
    const int pb = c & 1;                                  // a / bp are double buffered by chunk parity
    sm.a[pb][t] = make_float2(x.at.r, x.at.i);
    cplx W = x.at, S = x.at;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        cplx up = {__shfl_up_sync(0xffffffffu, W.r, o), __shfl_up_sync(0xffffffffu, W.i, o)};
        cplx dn = {__shfl_down_sync(0xffffffffu, S.r, o), __shfl_down_sync(0xffffffffu, S.i, o)};
        if (tl >= o) W = cmul(W, up);
        if (tl + o < 32) S = cmul(S, dn);
    }
    x.W = W;
    x.W0 = {__shfl_up_sync(0xffffffffu, W.r, 1), __shfl_up_sync(0xffffffffu, W.i, 1)};
    x.V = {__shfl_down_sync(0xffffffffu, S.r, 1), __shfl_down_sync(0xffffffffu, S.i, 1)};
    if (tl == 0) x.W0 = {1.f, 0.f};
    if (tl == 31) { x.V = {1.f, 0.f}; sm.bp[pb][J] = make_float2(W.r, W.i); }
    __syncwarp();
    if (tl == 0) mbar_arrive(&sm.bp_ready);
    // |q_t|^-1 from the Q tile row (swizzled 16-byte chunks) while the other warps catch up
    if (!warp_wait(&sm.full_q, c & 1, ab)) return false;
    float qq = 0.f;
#pragma unroll
    for (int sl = 0; sl < 2; sl++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint4 r = *reinterpret_cast<const uint4*>(sm.q + sl * kSlabBytes + t * 128 + ((j ^ (t & 7)) << 4));
            float f[8];
            unpack8(r, f);
#pragma unroll
            for (int e = 0; e < 8; e++) qq += f[e] * f[e];
        }
    x.mt = rsqrtf(qq + kEps);
    if (!warp_wait(&sm.bp_ready, c & 1, ab)) return false;
    cplx bpv[4];
#pragma unroll
    for (int i = 0; i < 4; i++) bpv[i] = {sm.bp[pb][i].x, sm.bp[pb][i].y};
    x.gpre = {1.f, 0.f};
    x.gsuf = {1.f, 0.f};
    x.gall = {1.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if (i < J) x.gpre = cmul(x.gpre, bpv[i]);
        if (i > J) x.gsuf = cmul(x.gsuf, bpv[i]);
        x.gall = cmul(x.gall, bpv[i]);
    }
    x.bp1 = bpv[1];
    x.bp2 = bpv[2];
    return true;
}

#define TC_STAMP(idx) do { if (a.trace && blockIdx.x == 0 && tl == 0 && c < 8) a.trace[(c * 5 + J) * 16 + (idx)] = clock64(); } while (0)
__device__ __forceinline__ void tc_compute(TcSmem& sm, const TcArgs& a, int b, int hd) {
    volatile int* ab = &sm.abort_flag;
    const int t = threadIdx.x, J = t >> 5, tl = t & 31;
    const int H = a.H, L = a.L;
    const uint32_t tlane = sm.tmem_base + ((uint32_t)(J * 32) << 16);
    const float lds = a.log_dt_scale[hd], freq = a.rope_freqs[hd];
    int code = 0;

    // carry column d = t: s = h0 (or 0); publish bf16(s) as the first UMMA operand
    float s_re = 0.f, s_im = 0.f;
    if (a.h0) {
        const float* h = a.h0 + ((size_t)b * H + hd) * 2 * kTcD;
        s_re = h[t];
        s_im = h[kTcD + t];
    }
    st_bf16(sm.s_tile, small_tile_off(0, t), s_re);
    st_bf16(sm.s_tile, small_tile_off(1, t), s_im);
    fence_proxy_async();
    tc_fence_before();
    __syncwarp();
    if (tl == 0) mbar_arrive(&sm.s_ready);

    TokenCtx x;
    if (!tc_prologue(sm, a, b, hd, 0, lds, freq, x)) code = 10;

    for (int c = 0; c < a.NC && !code; c++) {
        const uint32_t ph = c & 1;
        const int l = c * kTcC + t;
        const cplx at = x.at, vg = x.vg, W = x.W, W0 = x.W0, V = x.V;
        const float be = x.be, mt = x.mt;
        TC_STAMP(0);
        // ---- off-diagonal column blocks I < J.  Loops over groups of eight columns stay rolled and
        // read tensor memory with a run-time column address: the fully unrolled form of this kernel was
        // 110 KB of straight-line code and stalled on instruction fetch.
        cplx agw = {0, 0}, agx = {0, 0}, apw = {0, 0}, apx = {0, 0};
        bool fail = false;
        for (int I = 0; I < J; I++) {
            if (!warp_wait(I < 2 ? &sm.mma_gp0 : &sm.mma_gp1, ph, ab)) { code = 13; fail = true; break; }
            tc_fence_after();
            if (!warp_wait(&sm.blk_done[I], ph, ab)) { code = 14; fail = true; break; }
            if (I > 0) {
                const cplx bpI = I == 1 ? x.bp1 : x.bp2;
                agw = cmul(agw, bpI); agx = cmul(agx, bpI); apw = cmul(apw, bpI); apx = cmul(apx, bpI);
            }
#pragma unroll 1
            for (int grp = 0; grp < 4; grp++) {
                float g8[8], p8[8];
                tmem_ld8x2(tlane + kColG + (I & 1) * 32 + grp * 8, g8, tlane + kColP + (I & 1) * 32 + grp * 8, p8);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const float4 wx = sm.wx[I * 32 + grp * 8 + e];
                    agw.r += g8[e] * wx.x; agw.i += g8[e] * wx.y; agx.r += g8[e] * wx.z; agx.i += g8[e] * wx.w;
                    apw.r += p8[e] * wx.x; apw.i += p8[e] * wx.y; apx.r += p8[e] * wx.z; apx.i += p8[e] * wx.w;
                }
            }
            if (I == 1 && J >= 2) {   // warps 2, 3: last read of the first column half
                tc_fence_before();
                __syncwarp();
                if (tl == 0) mbar_arrive(&sm.gp0_free);
            }
        }
        if (fail) break;
        TC_STAMP(2);
        // ---- diagonal block J: P[t, 32J..] into registers, G[t, 32J..] streamed through phase A
        if (!warp_wait(J < 2 ? &sm.mma_gp0 : &sm.mma_gp1, ph, ab)) { code = 13; break; }
        tc_fence_after();
        float p[32];
        tmem_ld32(tlane + kColP + (J & 1) * 32, p);
        float pd = 0.f;
#pragma unroll
        for (int i = 0; i < 32; i++) pd = (i == tl) ? p[i] : pd;
        // Phase A (no dependence on other lanes): coefficients of the unit-lower-triangular system
        // for the unknowns u = n w and x~ = n x,
        //   u_t = n_t b_t - sum_{i<t} cc[i] u_i,  cc[i] = beta_t n_t^2 a_t Gamma0[t,i] G_raw[t,i],
        // Gamma0[t,i] = prod a_r, i < r <= t-1, built leftwards from the diagonal (0 for i >= t).
        // n_t = |k_t|^-1 comes from the Gram diagonal, so the scalar factor is applied afterwards.
        cplx cc[32];
        float gd = 0.f;
        {
            cplx cur = {1.f, 0.f};
#pragma unroll 1
            for (int grp = 3; grp >= 0; grp--) {
                if (grp < 3) {
#pragma unroll
                    for (int k = 31; k >= 8; k--) cc[k] = cc[k - 8];
                }
                float g8[8];
                tmem_ld8(tlane + kColG + (J & 1) * 32 + grp * 8, g8);
#pragma unroll
                for (int e = 7; e >= 0; e--) {
                    const int i = grp * 8 + e;
                    const float2 ai = sm.a[ph][J * 32 + i];
                    const bool on = i < tl;
                    gd = (i == tl) ? g8[e] : gd;
                    const cplx fg = cmul(at, cur);
                    cc[e] = {on ? fg.r * g8[e] : 0.f, on ? fg.i * g8[e] : 0.f};
                    const cplx nx = cmul(cur, cplx{ai.x, ai.y});
                    cur = {on ? nx.r : cur.r, on ? nx.i : cur.i};
                }
            }
        }
        // every TMEM read of this chunk's G/P is done
        tc_fence_before();
        __syncwarp();
        if (tl == 0) {
            if (J < 2) mbar_arrive(&sm.gp0_free);
            mbar_arrive(&sm.gp1_free);
        }
        const float nt = rsqrtf(gd + kEps);                  // |k_t|^-1
        const float bnn = be * nt * nt;
        TC_STAMP(3);
        // ---- kappa_t = k_t.s, rho_t = q_t.s (raw rows; scaled by the norms)
        if (!warp_wait(&sm.mma_kr, ph, ab)) { code = 12; break; }
        tc_fence_after();
        TC_STAMP(1);
        float kr4[4], rr4[4];
        tmem_ld4(tlane + kColKappa, kr4);
        tmem_ld4(tlane + kColRho, rr4);
        const cplx kap = {kr4[0], kr4[1]}, rho = {rr4[0], rr4[1]};
        const cplx gam = cmul(x.gpre, W), gam_prev = cmul(x.gpre, W0);
        const cplx wagw = cmul(W, agw), wagx = cmul(W, agx);
        const cplx gk = cmul(gam, kap);
        cplx cw = {nt * be * (vg.r - nt * wagw.r), nt * be * (vg.i - nt * wagw.i)};
        cplx cx = {nt * be * (nt * gk.r - nt * wagx.r), nt * be * (nt * gk.i - nt * wagx.i)};
        // Phase B: the sequential substitution, eight steps per rolled iteration; the coefficient
        // queue is rotated so that the unrolled body always reads slots 0..7.
#pragma unroll 1
        for (int grp = 0; grp < 4; grp++) {
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const int i = grp * 8 + e;
                const cplx uw = cshfl(cw, i), ux = cshfl(cx, i);
                const float cr_ = bnn * cc[e].r, ci_ = bnn * cc[e].i;
                cw.r -= cr_ * uw.r - ci_ * uw.i;
                cw.i -= cr_ * uw.i + ci_ * uw.r;
                cx.r -= cr_ * ux.r - ci_ * ux.i;
                cx.i -= cr_ * ux.i + ci_ * ux.r;
            }
#pragma unroll
            for (int k = 0; k < 24; k++) cc[k] = cc[k + 8];
        }
        TC_STAMP(4);
        // ---- publish V n w, V n x for the later blocks; omega = Gamma[C-1,t] n_t w_t for l
        const cplx wh = cmul(V, cw), xh = cmul(V, cx);
        sm.wx[t] = make_float4(wh.r, wh.i, xh.r, xh.i);
        const cplx om = cmul(x.gsuf, wh);
        {
            const float hr = bfr(om.r), hi = bfr(om.i);
            st_bf16(sm.o_tile, small_tile_off(0, t), hr);
            st_bf16(sm.o_tile, small_tile_off(1, t), hi);
            st_bf16(sm.o_tile, small_tile_off(2, t), om.r - hr);
            st_bf16(sm.o_tile, small_tile_off(3, t), om.i - hi);
        }
        fence_proxy_async();
        __syncwarp();
        if (tl == 0) {
            if (J < 3) mbar_arrive(&sm.blk_done[J]);
            mbar_arrive(&sm.omega_ready);
        }
        // Phase C (off the other warps' critical path): in-block part of the read-out,
        // sum_{i<t} P_raw[t,i] Gamma0[t,i] (a_t u_i - x~_i); columns taken from the top of a rotating queue
        cplx yin = {0.f, 0.f};
        {
            cplx cur = {1.f, 0.f};
#pragma unroll 1
            for (int grp = 3; grp >= 0; grp--) {
#pragma unroll
                for (int e = 7; e >= 0; e--) {
                    const int i = grp * 8 + e;
                    const float2 ai = sm.a[ph][J * 32 + i];
                    const cplx uw = cshfl(cw, i), ux = cshfl(cx, i);
                    const bool on = i < tl;
                    const cplx au = cmul(at, uw);
                    const cplx ee = cmul(cur, cplx{au.r - ux.r, au.i - ux.i});
                    const float pi = on ? p[24 + e] : 0.f;
                    yin.r += pi * ee.r;
                    yin.i += pi * ee.i;
                    const cplx nx = cmul(cur, cplx{ai.x, ai.y});
                    cur = {on ? nx.r : cur.r, on ? nx.i : cur.i};
                }
#pragma unroll
                for (int k = 31; k >= 8; k--) p[k] = p[k - 8];
            }
        }
        // ---- read-out: local + correction taken before the step (exact_correction.cu:90-94)
        {
            const cplx apwa = cmul(at, apw);
            const cplx off = cmul(W0, cplx{apwa.r - apx.r, apwa.i - apx.i});
            const cplx car = cmul(gam_prev, rho);
            float yr = mt * (pd * cw.r + yin.r + off.r + car.r);
            float yi = mt * (pd * cw.i + yin.i + off.i + car.i);
            if (a.shortcut_scale != 0.f) {   // block.py:202-208
                const float qk = mt * nt * pd;
                yr += a.shortcut_scale * qk * qk * vg.r;
                yi += a.shortcut_scale * qk * qk * vg.i;
            }
            if (x.valid) {
                __nv_bfloat162 o = __floats2bfloat162_rn(bfr(yr) * x.sc, bfr(yi) * x.sc);
                *reinterpret_cast<__nv_bfloat162*>(a.y + (((size_t)b * L + l) * H + hd) * 2) = o;
            }
        }
        TC_STAMP(5);
        // ---- next chunk's carry-independent work runs under the l UMMA
        const cplx gall = x.gall;
        if (c + 1 < a.NC && !tc_prologue(sm, a, b, hd, c + 1, lds, freq, x)) { code = 10; break; }
        // ---- carry: s <- bf16(gamma_C) s + bf16(l)   (inter_chunk_scan.cu:73-83 on bf16 inputs)
        TC_STAMP(6);
        if (!warp_wait(&sm.mma_ell, ph, ab)) { code = 15; break; }
        tc_fence_after();
        TC_STAMP(7);
        float e4[4];
        tmem_ld4(tlane + kColEll, e4);
        {
            const float lr = bfr(e4[0] + e4[2]), li = bfr(e4[1] + e4[3]);
            const float cr = bfr(gall.r), ci = bfr(gall.i);
            const float nr = cr * s_re - ci * s_im + lr;
            const float ni = cr * s_im + ci * s_re + li;
            s_re = nr;
            s_im = ni;
        }
        st_bf16(sm.s_tile, small_tile_off(0, t), s_re);
        st_bf16(sm.s_tile, small_tile_off(1, t), s_im);
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (tl == 0) mbar_arrive(&sm.s_ready);
        TC_STAMP(8);
    }
    if (code) {
        if (tl == 0) atomicCAS(a.status, 0, 200 + code);
    } else if (a.final_state) {
        float* fs = a.final_state + ((size_t)b * H + hd) * 2 * kTcD;
        fs[t] = s_re;
        fs[kTcD + t] = s_im;
    }
}

__global__ void __launch_bounds__(kTcThreads, 2)
scan_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ, const TcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    TcSmem& sm = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int b = blockIdx.x / a.H, hd = blockIdx.x % a.H;
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        mbar_init(&sm.full_k[0], 1); mbar_init(&sm.full_k[1], 1); mbar_init(&sm.full_q, 1);
        mbar_init(&sm.mma_gp0, 1); mbar_init(&sm.mma_kr, 1); mbar_init(&sm.mma_gp1, 1); mbar_init(&sm.mma_ell, 1);
        mbar_init(&sm.gp0_free, 4); mbar_init(&sm.gp1_free, 4); mbar_init(&sm.s_ready, 4);
        mbar_init(&sm.omega_ready, 4);
        mbar_init(&sm.blk_done[0], 1); mbar_init(&sm.blk_done[1], 1); mbar_init(&sm.blk_done[2], 1);
        mbar_init(&sm.bp_ready, 4);
        mbar_init(&sm.drain, 1);
        sm.abort_flag = 0;
        fence_barrier_init();
    }
    // the unused rows of the two small operand tiles stay zero for the whole kernel
    for (int i = threadIdx.x; i < 2 * 4096 / 16; i += kTcThreads)
        reinterpret_cast<uint4*>(sm.s_tile)[i] = make_uint4(0, 0, 0, 0);   // s_tile and o_tile are adjacent
    if (warp == 4) tmem_alloc(&sm.tmem_base, kTmemCols);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp < 4) {
        tc_compute(sm, a, b, hd);
    } else if (threadIdx.x == kTcComputeThreads) {
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmQ);
        tc_producer(sm, &tmK, &tmQ, a, b, hd);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        tmem_dealloc(sm.tmem_base, kTmemCols);
    }
}


// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// (B, L, H, D) bf16 tensor viewed as 4-D (D, H, L, B); box = 64 columns x 1 head x 128 positions.
static bool make_tile_map(CUtensorMap* m, const void* base, int B, int L, int H) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)kTcD, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)kTcD * 2, (cuuint64_t)H * kTcD * 2, (cuuint64_t)L * H * kTcD * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)kTcC, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static long long* g_trace = nullptr;
void scan_tc_set_trace(long long* p) { g_trace = p; }

bool scan_tc_supported(int D, int N, int C, int dtype) {
    return dtype == CDSSM_BF16 && N == 2 && D == kTcD && C == kTcC;
}

// status: one int in device memory, zeroed here on the stream before the launch.
int scan_fused_tc(const void* q, const void* k, const void* v, const void* gate_raw, const float* log_dt_scale,
                  const float* rope_freqs, const float* h0, void* y, float* final_state, int* status,
                  const DynConsts& dc, float shortcut_scale, int B, int L, int H, int pos0, int segs,
                  cudaStream_t st) {
    CUtensorMap tmK, tmQ;
    if (!make_tile_map(&tmK, k, B, L, H) || !make_tile_map(&tmQ, q, B, L, H)) return CDSSM_ERR_CUDA;
    const size_t smem = sizeof(TcSmem) + 1024;
    constexpr int kMaxDevices = 64;
    static bool attr_of_device[kMaxDevices] = {false};   // the shared-memory opt-in is per device
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev))) return rc;
    if (dev < 0 || dev >= kMaxDevices) return CDSSM_ERR_UNSUPPORTED;
    if (!attr_of_device[dev]) {
        if (int rc = check_cuda(cudaFuncSetAttribute(scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)))
            return rc;
        attr_of_device[dev] = true;
    }
    if (int rc = check_cuda(cudaMemsetAsync(status, 0, sizeof(int), st))) return rc;
    TcArgs a;
    a.v = static_cast<const __nv_bfloat16*>(v);
    a.gate_raw = static_cast<const __nv_bfloat16*>(gate_raw);
    a.log_dt_scale = log_dt_scale; a.rope_freqs = rope_freqs; a.h0 = h0;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.final_state = final_state; a.status = status; a.trace = g_trace;
    a.dc = dc; a.shortcut_scale = shortcut_scale;
    a.B = B; a.L = L; a.H = H; a.NC = (L + kTcC - 1) / kTcC; a.pos0 = pos0; a.segs = segs;
    scan_tc_kernel<<<B * H, kTcThreads, smem, st>>>(tmK, tmQ, a);
    return check_launch();
}

}  // namespace cdssm
