// Tensor-core output pass with four independent chains per CTA (tcgen05 + TMEM + TMA).
// Shapes: bf16 storage, state_dim N = 2, head_dim D = 128, chunk C = 128, H a multiple of 4.
//
// The single-chain kernel in scan_tc.cu keeps one warp at a time on the critical path.  Here a CTA
// owns the same chunk of FOUR heads; the chunk is walked in 32-token sub-blocks and every compute
// warp owns one head: UMMA tile row 32 j + t is token t of head j's sub-block.  Per sub-block:
//   G_j = K_j K_j^T, P_j = Q_j K_j^T     : the 32 x 32 diagonal blocks only - one UMMA per head with
//                                          N = 32 and every output lane but the head's own masked
//                                          off (disable_output_lane), so all four heads share 32 + 32
//                                          TMEM columns;
//   kappa, rho = K S^T, Q S^T            : products with the running states (local state z and
//                                          correction r of each head, bf16 hi + lo rows) - they
//                                          replace all off-diagonal work of the chunk form;
//   solve / read-out                     : each warp solves its own unit-lower-triangular 32 x 32
//                                          systems (local + correction) by substitution through warp
//                                          shuffles and reads y out, with rows from tcgen05.ld;
//   S <- gamma S + K^T Omega             : state update as one UMMA (K tile as MN-major operand),
//                                          thread d applies it to column d of all four heads' states.
// The four warps never wait for one another except at the UMMA hand-offs, so four chains per CTA and
// two CTAs per SM are in flight.  Reference semantics: z starts at zero at the chunk start, r starts
// from the chunk's carry (bf16, from the carry pass), the correction is read before its step.
// Algebra per sub-block with incoming states z0, r0 (restating intra_chunk_scan.cu:100-195 and
// exact_correction.cu:89-150):
//   u  = T beta (v - W kappa_z),  x = T beta W kappa_r,  T = (I + M)^-1,  M[t,i] = beta_t Gamma[t,i] G[t,i]
//   y_t = W_t rho_z,t + sum_{i<=t} Gamma[t,i] P[t,i] u_i + W0_t rho_r,t - sum_{i<t} Gamma0[t,i] P[t,i] x_i
//   z_end = W_31 z0 + sum_i V_i u_i k_i,   r_end = W_31 r0 - sum_i V_i x_i k_i
// (W, W0: inclusive / exclusive prefix products of a inside the sub-block, V: exclusive suffix.)
#include "cdssm_common.cuh"
#include "sm100_ptx.cuh"

namespace cdssm {
using namespace sm100;

namespace tc4 {

constexpr int kC = 128, kD = 128, kSub = 32, kSteps = kC / kSub;
constexpr int kThreads = 160;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColG = 0, kColP = 32, kColKappa = 64, kColRho = 96, kColUp = 128;
constexpr uint32_t kSlab = 128 * 128;          // 64 bf16 columns x 128 rows
constexpr uint32_t kTile = 2 * kSlab;          // 32 KB
constexpr uint32_t kSmallSlab = 32 * 128;      // 32-row operand tiles: 4 KB per 64 columns
constexpr uint32_t kSmallTile = 2 * kSmallSlab;

struct __align__(1024) Smem {
    uint8_t k[2][kTile];        // rows 32 j + t: token t of head j (TMA, double buffered)
    uint8_t q[kTile];
    uint8_t s_tile[kSmallTile]; // rows 8 j + {z_re hi, lo, z_im hi, lo, r_re hi, lo, r_im hi, lo}, columns d
    uint8_t o_tile[kSmallTile]; // rows 8 j + {uz_re hi, lo, uz_im hi, lo, ur_re hi, lo, ur_im hi, lo}, columns = tile rows
    __nv_bfloat162 a[kC];       // a_t of tile row r (a is a bf16 pair in the reference's storage)
    float2 bp[2][4];            // product of a over the sub-block, per head, by step parity
    uint64_t full_k[2], full_q, mma_gp, mma_kr, mma_up, gp_free, s_ready, omega_ready, bp_ready, drain;
    uint32_t tmem_base;
    int abort_flag;
};

struct Args {
    const __nv_bfloat16 *v, *gate_raw;
    const float *log_dt_scale, *rope_freqs;
    float* ws_gamma;             // (B,NC,H,2): written by the local pass
    float* ws_state;             // (B,NC,H,2,D): local pass writes z_{C-1}; the output pass reads the carry s_c
    __nv_bfloat16* y;
    int* status;
    long long* trace;
    DynConsts dc;
    float shortcut_scale;
    int B, L, H, NC, pos0, segs;
    int HG, items;               // head groups of four; items = B * NC * HG (one chunk of four heads each)
};

struct cplx { float r, i; };
__device__ __forceinline__ cplx cmul(cplx a, cplx b) { return {a.r * b.r - a.i * b.i, a.r * b.i + a.i * b.r}; }
__device__ __forceinline__ cplx cshfl(cplx v, int src) {
    return {__shfl_sync(0xffffffffu, v.r, src), __shfl_sync(0xffffffffu, v.i, src)};
}
__device__ __forceinline__ float bfr(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// element (row n, column kk) of a 32-row K-major bf16 operand tile with 128-byte swizzle
__device__ __forceinline__ uint32_t small_off(int n, int kk) {
    return (uint32_t)(kk >> 6) * kSmallSlab + (uint32_t)n * 128u + (uint32_t)((((kk & 63) >> 3) ^ (n & 7)) << 4) +
           (uint32_t)(kk & 7) * 2u;
}
__device__ __forceinline__ void st_hi_lo(uint8_t* tile, int n, int kk, float x) {
    const __nv_bfloat16 hi = __float2bfloat16_rn(x);
    *reinterpret_cast<__nv_bfloat16*>(tile + small_off(n, kk)) = hi;
    *reinterpret_cast<__nv_bfloat16*>(tile + small_off(n + 1, kk)) = __float2bfloat16_rn(x - __bfloat162float(hi));
}
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* ab) {
    const bool ok = mbar_wait(bar, parity, ab);
    return __all_sync(0xffffffffu, ok);
}

// D[tmem] (+)= A * B with every output lane outside [32*unit, 32*unit + 32) disabled
__device__ __forceinline__ void umma_bf16_unit(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               bool accumulate, int unit) {
    const uint32_t m0 = unit == 0 ? 0u : 0xffffffffu, m1 = unit == 1 ? 0u : 0xffffffffu;
    const uint32_t m2 = unit == 2 ? 0u : 0xffffffffu, m3 = unit == 3 ? 0u : 0xffffffffu;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate), "r"(m0), "r"(m1), "r"(m2),
          "r"(m3)
        : "memory");
}


// ------------------------------------------------------------------------------------------
// Producer (one elected lane of warp 4): TMA and UMMA issue, event driven.  The CTA's work is a flat
// sequence of sub-block steps g = 0 .. 4 * n_items - 1; item (g >> 2) is chunk c of heads h0 .. h0 + 3
// of batch row b.  Every barrier completes once per step, so its parity is that of g.
// ------------------------------------------------------------------------------------------
template <bool kOutput>
__device__ __forceinline__ void producer(Smem& sm, const CUtensorMap* tmK, const CUtensorMap* tmQ, const Args& a) {
    volatile int* ab = &sm.abort_flag;
    const uint32_t tm = sm.tmem_base;
    constexpr uint32_t idesc32 = umma_idesc_bf16(128, 32, false, false);
    constexpr uint32_t idesc_up = umma_idesc_bf16(128, 32, true, false);
    const uint32_t kaddr[2] = {smem_u32(sm.k[0]), smem_u32(sm.k[1])};
    const uint32_t qaddr = smem_u32(sm.q), saddr = smem_u32(sm.s_tile), oaddr = smem_u32(sm.o_tile);
    bool pend_k[2] = {false, false}, pend_q = false;
    int code = 0;
    const int n_items = ((int)blockIdx.x < a.items) ? (a.items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int NS = n_items * kSteps;
    auto load_tile = [&](uint8_t* dst, const CUtensorMap* tmap, uint64_t* bar, int g) {
        const int item = (int)blockIdx.x + (g >> 2) * (int)gridDim.x;
        const int h0 = (item % a.HG) * 4, c = (item / a.HG) % a.NC, b = item / (a.HG * a.NC);
        const int l0 = c * kC + (g & 3) * kSub;
        mbar_arrive_expect_tx(bar, kTile);
#pragma unroll 1
        for (int j = 0; j < 4; j++) {
            tma_load_4d(dst + j * kSub * 128, tmap, bar, 0, h0 + j, l0, b);
            tma_load_4d(dst + kSlab + j * kSub * 128, tmap, bar, 64, h0 + j, l0, b);
        }
    };
    auto kmaj = [](uint32_t base, uint32_t slab_bytes, int j, uint32_t row_off) {
        return umma_desc_sw128(base + (uint32_t)(j >> 2) * slab_bytes + (uint32_t)(j & 3) * 32 + row_off, 16, 1024);
    };
    if (NS > 0) {
        load_tile(sm.k[0], tmK, &sm.full_k[0], 0); pend_k[0] = true;
        if (kOutput) { load_tile(sm.q, tmQ, &sm.full_q, 0); pend_q = true; }
        load_tile(sm.k[1], tmK, &sm.full_k[1], 1); pend_k[1] = true;
    }
    int i_gp = 0, i_kr = 0, i_up = 0, i_lq = 1, i_lk = 2;
    bool k_ok = false, q_ok = !kOutput;
    uint64_t last = global_ns();
    uint32_t idle = 0;
    auto par = [](int n) { return (uint32_t)(n & 1); };
    while (i_up < NS) {
        bool progress = false;
        if (i_gp < NS) {   // diagonal Gram blocks of step i_gp
            const int n = i_gp, st = n & 1;
            if (!k_ok && mbar_test(&sm.full_k[st], (n >> 1) & 1)) { k_ok = true; pend_k[st] = false; }
            if (!q_ok && mbar_test(&sm.full_q, par(n))) { q_ok = true; pend_q = false; }
            if (k_ok && q_ok && (n == 0 || mbar_test(&sm.gp_free, par(n - 1)))) {
                tc_fence_after();
#pragma unroll 1
                for (int u = 0; u < 4; u++) {
#pragma unroll 1
                    for (int j = 0; j < 8; j++)
                        umma_bf16_unit(tm + kColG, kmaj(kaddr[st], kSlab, j, 0),
                                       kmaj(kaddr[st], kSlab, j, u * kSub * 128), idesc32, j > 0, u);
                    if (kOutput) {
#pragma unroll 1
                        for (int j = 0; j < 8; j++)
                            umma_bf16_unit(tm + kColP, kmaj(qaddr, kSlab, j, 0),
                                           kmaj(kaddr[st], kSlab, j, u * kSub * 128), idesc32, j > 0, u);
                    }
                }
                umma_commit(&sm.mma_gp);
                i_gp++; k_ok = false; q_ok = !kOutput; progress = true;
            }
        }
        if (i_kr < i_gp && mbar_test(&sm.s_ready, par(i_kr))) {   // kappa = K S^T, rho = Q S^T
            const int st = i_kr & 1;
            tc_fence_after();
#pragma unroll 1
            for (int j = 0; j < 8; j++)
                umma_bf16(tm + kColKappa, kmaj(kaddr[st], kSlab, j, 0), kmaj(saddr, kSmallSlab, j, 0), idesc32, j > 0);
            if (kOutput) {
#pragma unroll 1
                for (int j = 0; j < 8; j++)
                    umma_bf16(tm + kColRho, kmaj(qaddr, kSlab, j, 0), kmaj(saddr, kSmallSlab, j, 0), idesc32, j > 0);
            }
            umma_commit(&sm.mma_kr);
            i_kr++; progress = true;
        }
        // Q tile of step n is free once its UMMAs have completed (mma_kr is committed after mma_gp of the
        // same step, so it covers both) and every warp has read |q| from it (gp_free follows that read)
        if (kOutput && i_lq <= i_kr && i_lq <= NS && mbar_test(&sm.mma_kr, par(i_lq - 1)) &&
            mbar_test(&sm.gp_free, par(i_lq - 1))) {
            if (i_lq < NS) { load_tile(sm.q, tmQ, &sm.full_q, i_lq); pend_q = true; }
            i_lq++; progress = true;
        }
        // state update: A = K tile read MN-major (M = d, two 64-wide groups 16 KB apart; K = tile rows,
        // 16 per instruction = 2 KB), B = omega tile (32 rows x 128 tile rows)
        // (issued only once the completion of the previous update has been observed below, so that the
        // mma_up barrier is never more than one phase ahead of what this loop tests)
        if (i_up < i_kr && i_lk - 2 >= i_up && mbar_test(&sm.omega_ready, par(i_up))) {
            const int st = i_up & 1;
            tc_fence_after();
#pragma unroll 1
            for (int j = 0; j < 8; j++)
                umma_bf16(tm + kColUp, umma_desc_sw128(kaddr[st] + (uint32_t)j * 2048, kSlab, 1024),
                          kmaj(oaddr, kSmallSlab, j, 0), idesc_up, j > 0);
            umma_commit(&sm.mma_up);
            i_up++; progress = true;
        }
        if (i_lk - 2 < i_up && i_lk - 2 < NS && mbar_test(&sm.mma_up, par(i_lk - 2))) {
            if (i_lk < NS) { load_tile(sm.k[i_lk & 1], tmK, &sm.full_k[i_lk & 1], i_lk); pend_k[i_lk & 1] = true; }
            i_lk++; progress = true;
        }
        if (progress) {
            last = global_ns();
        } else if ((++idle & 7) != 0) {
            __nanosleep(32);
        } else if (*ab || global_ns() - last > kWaitLimitNs) {
            code = 1 + (i_gp > i_kr) + 2 * (i_kr > i_up);
            *ab = 1;
            break;
        }
    }
    if (code) {
        atomicCAS(a.status, 0, 300 + code);
        umma_commit(&sm.drain);
        int never = 0;
        mbar_wait(&sm.drain, 0, &never);
        if (pend_k[0]) mbar_wait(&sm.full_k[0], 0, &never), mbar_wait(&sm.full_k[0], 1, &never);
        if (pend_k[1]) mbar_wait(&sm.full_k[1], 0, &never), mbar_wait(&sm.full_k[1], 1, &never);
        if (pend_q) mbar_wait(&sm.full_q, 0, &never), mbar_wait(&sm.full_q, 1, &never);
    }
}

// ------------------------------------------------------------------------------------------
// Compute warps.  Thread t = 32 j + tl is token tl of head j's sub-block (TMEM lane t) and, for the state
// hand-off, column d = t of all four heads' states.
// kOutput = false: local pass - z only; writes z_{C-1} and the chunk's decay product for the carry pass.
// kOutput = true : output pass - z and r (r starts from the chunk's carry), writes y.
// ------------------------------------------------------------------------------------------
#define TC4_STAMP(idx) do { if (a.trace && blockIdx.x == 0 && tl == 0 && g < 16) a.trace[(g * 4 + J) * 8 + (idx)] = clock64(); } while (0)
template <bool kOutput>
__device__ __forceinline__ void compute(Smem& sm, const Args& a) {
    using T = __nv_bfloat16;
    volatile int* ab = &sm.abort_flag;
    const int t = threadIdx.x, J = t >> 5, tl = t & 31;
    const int H = a.H, L = a.L;
    const uint32_t tlane = sm.tmem_base + ((uint32_t)(J * 32) << 16);
    int code = 0;
    cplx Sz[4], Sr[4], gam[4];
    int g = 0;   // flat step index
    for (int item = blockIdx.x; item < a.items && !code; item += gridDim.x) {
        const int h0 = (item % a.HG) * 4, c = (item / a.HG) % a.NC, b = item / (a.HG * a.NC);
        const int hd = h0 + J;
        const float lds = a.log_dt_scale[hd], freq = a.rope_freqs[hd];
        const size_t unit0 = ((size_t)b * a.NC + c) * H + h0;   // workspace slot of head h0 (one pair per head)
        // ---- states at the chunk start, column d = t of every head
#pragma unroll
        for (int u = 0; u < 4; u++) {
            Sz[u] = {0.f, 0.f};
            Sr[u] = {0.f, 0.f};
            gam[u] = {1.f, 0.f};
            if (kOutput) {
                const float* s = a.ws_state + (unit0 + u) * 2 * kD;
                Sr[u] = {s[t], s[kD + t]};
            }
        }
        for (int step = 0; step < kSteps && !code; step++, g++) {
            const uint32_t ph = g & 1;
            // ---- publish the states for kappa / rho of this step
#pragma unroll
            for (int u = 0; u < 4; u++) {
                st_hi_lo(sm.s_tile, 8 * u + 0, t, Sz[u].r);
                st_hi_lo(sm.s_tile, 8 * u + 2, t, Sz[u].i);
                if (kOutput) {
                    st_hi_lo(sm.s_tile, 8 * u + 4, t, Sr[u].r);
                    st_hi_lo(sm.s_tile, 8 * u + 6, t, Sr[u].i);
                }
            }
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.s_ready);
            TC4_STAMP(0);
            // ---- dynamics of this thread's token (dynamics_fused.cu:64-139; vp scale of block.py:194-195)
            const int l = c * kC + step * kSub + tl;
            const bool valid = l < L;
            cplx at = {0.f, 0.f}, vg = {0.f, 0.f};
            float be = 0.f, sc = 0.f;
            if (valid) {
                const size_t bl = (size_t)b * L + l;
                const T* gr = a.gate_raw + bl * (size_t)(7 * H);
                const float pos = (float)(l + a.pos0 + (b % a.segs) * L);
                DynShared ds = dyn_shared<true>(IO<T>::ld(gr + hd), IO<T>::ld(gr + H + hd), IO<T>::ld(gr + 2 * H + hd),
                                                IO<T>::ld(gr + 3 * H + hd), IO<T>::ld(gr + 4 * H + hd),
                                                IO<T>::ld(gr + 5 * H + hd), IO<T>::ld(gr + 6 * H + hd), lds, freq, pos,
                                                a.dc);
                float vp;
                dyn_pair<true>(IO<T>::ld(gr + hd), IO<T>::ld(gr + H + hd), freq, pos, ds, at.r, at.i, vp);
                at.r = bfr(at.r);
                at.i = bfr(at.i);
                vp = bfr(vp);
                be = bfr(ds.beta);
                sc = bfr(ds.sel_c);
                const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(a.v + (bl * H + hd) * 2);
                vg.r = bfr(__low2float(v2) * vp);
                vg.i = bfr(__high2float(v2) * vp);
            }
            sm.a[t] = __floats2bfloat162_rn(at.r, at.i);
            cplx W = at, S = at;   // inclusive prefix / suffix products of a over the sub-block
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                cplx up = {__shfl_up_sync(0xffffffffu, W.r, o), __shfl_up_sync(0xffffffffu, W.i, o)};
                cplx dn = {__shfl_down_sync(0xffffffffu, S.r, o), __shfl_down_sync(0xffffffffu, S.i, o)};
                if (tl >= o) W = cmul(W, up);
                if (tl + o < 32) S = cmul(S, dn);
            }
            cplx W0 = {__shfl_up_sync(0xffffffffu, W.r, 1), __shfl_up_sync(0xffffffffu, W.i, 1)};
            cplx V = {__shfl_down_sync(0xffffffffu, S.r, 1), __shfl_down_sync(0xffffffffu, S.i, 1)};
            if (tl == 0) W0 = {1.f, 0.f};
            if (tl == 31) { V = {1.f, 0.f}; sm.bp[ph][J] = make_float2(W.r, W.i); }
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.bp_ready);
            // ---- |q_t|^-1 from the Q tile row (swizzled 16-byte pieces)
            float mt = 0.f;
            if (kOutput) {
                if (!warp_wait(&sm.full_q, ph, ab)) { code = 11; break; }
                float qq = 0.f;
#pragma unroll
                for (int sl = 0; sl < 2; sl++)
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint4 r = *reinterpret_cast<const uint4*>(sm.q + sl * kSlab + t * 128 + ((j ^ (t & 7)) << 4));
                        float f[8];
                        unpack8(r, f);
#pragma unroll
                        for (int e = 0; e < 8; e++) qq += f[e] * f[e];
                    }
                mt = rsqrtf(qq + kEps);
            }
            TC4_STAMP(1);
            // ---- diagonal block: P[t, :] into registers, G[t, :] streamed through phase A
            if (!warp_wait(&sm.mma_gp, ph, ab)) { code = 13; break; }
            tc_fence_after();
            float p[32];
            float pd = 0.f;
            if (kOutput) {
                tmem_ld32(tlane + kColP, p);
#pragma unroll
                for (int i = 0; i < 32; i++) pd = (i == tl) ? p[i] : pd;
            }
            // Phase A (no dependence on other lanes): coefficients of the unit-lower-triangular system for
            // u~ = n u and x~ = n x:  u~_t = rhs_t - sum_{i<t} beta_t n_t^2 cc[i] u~_i,
            // cc[i] = a_t Gamma0[t,i] G_raw[t,i],  Gamma0[t,i] = prod a_r, i < r <= t-1, built leftwards
            // from the diagonal (0 for i >= t).  n_t = |k_t|^-1 comes from the Gram diagonal.
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
                    tmem_ld8(tlane + kColG + grp * 8, g8);
#pragma unroll
                    for (int e = 7; e >= 0; e--) {
                        const int i = grp * 8 + e;
                        const float2 ai = __bfloat1622float2(sm.a[J * 32 + i]);
                        const bool on = i < tl;
                        gd = (i == tl) ? g8[e] : gd;
                        const cplx fg = cmul(at, cur);
                        cc[e] = {on ? fg.r * g8[e] : 0.f, on ? fg.i * g8[e] : 0.f};
                        const cplx nx = cmul(cur, cplx{ai.x, ai.y});
                        cur = {on ? nx.r : cur.r, on ? nx.i : cur.i};
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.gp_free);   // every read of this step's G / P / Q row is done
            const float nt = rsqrtf(gd + kEps);      // |k_t|^-1
            const float bnn = be * nt * nt;
            TC4_STAMP(2);
            // ---- kappa_t = k_t . z0 | r0, rho_t = q_t . z0 | r0 (raw rows; hi + lo parts summed)
            if (!warp_wait(&sm.mma_kr, ph, ab)) { code = 12; break; }
            tc_fence_after();
            TC4_STAMP(3);
            float k8[8], r8[8];
            if (kOutput) {
                tmem_ld8x2(tlane + kColKappa + 8 * J, k8, tlane + kColRho + 8 * J, r8);
            } else {
                tmem_ld8(tlane + kColKappa + 8 * J, k8);
            }
            const cplx wkz = cmul(W, cplx{k8[0] + k8[1], k8[2] + k8[3]});
            cplx cw = {nt * be * (vg.r - nt * wkz.r), nt * be * (vg.i - nt * wkz.i)};
            cplx cx = {0.f, 0.f};
            if (kOutput) {
                const cplx wkr = cmul(W, cplx{k8[4] + k8[5], k8[6] + k8[7]});
                cx = {nt * be * nt * wkr.r, nt * be * nt * wkr.i};
            }
            // Phase B: the sequential substitution, eight columns per rolled iteration; the coefficient
            // queue is rotated so that the unrolled body always reads slots 0..7.
#pragma unroll 1
            for (int grp = 0; grp < 4; grp++) {
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const int i = grp * 8 + e;
                    const float cr_ = bnn * cc[e].r, ci_ = bnn * cc[e].i;
                    const cplx uw = cshfl(cw, i);
                    cw.r -= cr_ * uw.r - ci_ * uw.i;
                    cw.i -= cr_ * uw.i + ci_ * uw.r;
                    if (kOutput) {
                        const cplx ux = cshfl(cx, i);
                        cx.r -= cr_ * ux.r - ci_ * ux.i;
                        cx.i -= cr_ * ux.i + ci_ * ux.r;
                    }
                }
#pragma unroll
                for (int k = 0; k < 24; k++) cc[k] = cc[k + 8];
            }
            TC4_STAMP(4);
            // ---- omega columns of the state update: z += sum_t V_t u~_t k_t, r -= sum_t V_t x~_t k_t
            {
                const cplx wh = cmul(V, cw);
                st_hi_lo(sm.o_tile, 8 * J + 0, t, wh.r);
                st_hi_lo(sm.o_tile, 8 * J + 2, t, wh.i);
                if (kOutput) {
                    const cplx xh = cmul(V, cx);
                    st_hi_lo(sm.o_tile, 8 * J + 4, t, -xh.r);
                    st_hi_lo(sm.o_tile, 8 * J + 6, t, -xh.i);
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.omega_ready);
            if (kOutput) {
                // Phase C: in-block part of the read-out, sum_{i<t} P_raw[t,i] Gamma0[t,i] (a_t u~_i - x~_i);
                // the correction is read before its step (exact_correction.cu:90-94)
                cplx yin = {0.f, 0.f};
                {
                    cplx cur = {1.f, 0.f};
#pragma unroll 1
                    for (int grp = 3; grp >= 0; grp--) {
#pragma unroll
                        for (int e = 7; e >= 0; e--) {
                            const int i = grp * 8 + e;
                            const float2 ai = __bfloat1622float2(sm.a[J * 32 + i]);
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
                const cplx yz = cmul(W, cplx{r8[0] + r8[1], r8[2] + r8[3]});
                const cplx yr0 = cmul(W0, cplx{r8[4] + r8[5], r8[6] + r8[7]});
                float yr = mt * (pd * cw.r + yin.r + yz.r + yr0.r);
                float yi = mt * (pd * cw.i + yin.i + yz.i + yr0.i);
                if (a.shortcut_scale != 0.f) {   // block.py:202-208
                    const float qk = mt * nt * pd;
                    yr += a.shortcut_scale * qk * qk * vg.r;
                    yi += a.shortcut_scale * qk * qk * vg.i;
                }
                if (valid) {
                    __nv_bfloat162 o = __floats2bfloat162_rn(bfr(yr) * sc, bfr(yi) * sc);
                    *reinterpret_cast<__nv_bfloat162*>(a.y + (((size_t)b * L + l) * H + hd) * 2) = o;
                }
            }
            TC4_STAMP(5);
            // ---- state hand-off: S <- BP S + K^T omega, column d = t of every head
            if (!warp_wait(&sm.bp_ready, ph, ab)) { code = 14; break; }
            if (!warp_wait(&sm.mma_up, ph, ab)) { code = 15; break; }
            tc_fence_after();
            TC4_STAMP(6);
            if (!kOutput || step + 1 < kSteps) {
                float up[32];
                tmem_ld32(tlane + kColUp, up);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const cplx bpu = {sm.bp[ph][u].x, sm.bp[ph][u].y};
                    const cplx nz = cmul(bpu, Sz[u]);
                    Sz[u] = {nz.r + up[8 * u] + up[8 * u + 1], nz.i + up[8 * u + 2] + up[8 * u + 3]};
                    if (kOutput) {
                        const cplx nr = cmul(bpu, Sr[u]);
                        Sr[u] = {nr.r + up[8 * u + 4] + up[8 * u + 5], nr.i + up[8 * u + 6] + up[8 * u + 7]};
                    } else {
                        gam[u] = cmul(bpu, gam[u]);
                    }
                }
            }
            tc_fence_before();
            TC4_STAMP(7);
        }
        if (!kOutput && !code) {
            // the carry pass consumes these as the reference's bf16 cum_A[:, -1] / local_h[:, -1]
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float* s = a.ws_state + (unit0 + u) * 2 * kD;
                s[t] = bfr(Sz[u].r);
                s[kD + t] = bfr(Sz[u].i);
            }
            if (t < 4) {
                cplx gm = gam[0];
                if (t == 1) gm = gam[1];
                if (t == 2) gm = gam[2];
                if (t == 3) gm = gam[3];
                a.ws_gamma[(unit0 + t) * 2] = bfr(gm.r);
                a.ws_gamma[(unit0 + t) * 2 + 1] = bfr(gm.i);
            }
        }
    }
    if (code && tl == 0) atomicCAS(a.status, 0, 200 + code);
}

template <bool kOutput>
__global__ void __launch_bounds__(kThreads, 2)
scan_tc4_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ, const Args a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
    const int warp = threadIdx.x >> 5;
    if ((smem_u32(smem_raw) & 1023u) != 0) {   // the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicCAS(a.status, 0, 399);
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(&sm.full_k[0], 1); mbar_init(&sm.full_k[1], 1); mbar_init(&sm.full_q, 1);
        mbar_init(&sm.mma_gp, 1); mbar_init(&sm.mma_kr, 1); mbar_init(&sm.mma_up, 1);
        mbar_init(&sm.gp_free, 4); mbar_init(&sm.s_ready, 4); mbar_init(&sm.omega_ready, 4);
        mbar_init(&sm.bp_ready, 4);
        mbar_init(&sm.drain, 1);
        sm.abort_flag = 0;
        fence_barrier_init();
    }
    // rows of the two small operand tiles that a pass does not write stay zero for the whole kernel
    for (int i = threadIdx.x; i < 2 * (int)kSmallTile / 16; i += kThreads)
        reinterpret_cast<uint4*>(sm.s_tile)[i] = make_uint4(0, 0, 0, 0);   // s_tile and o_tile are adjacent
    if (warp == 4) tmem_alloc(&sm.tmem_base, kTmemCols);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp < 4) {
        compute<kOutput>(sm, a);
    } else if (threadIdx.x == 128) {
        prefetch_tmap(&tmK);
        if (kOutput) prefetch_tmap(&tmQ);
        producer<kOutput>(sm, &tmK, &tmQ, a);
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

// (B, L, H, D) bf16 tensor viewed as 4-D (D, H, L, B); box = 64 columns x 1 head x 32 positions.
static bool make_tile_map(CUtensorMap* m, const void* base, int B, int L, int H) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)kD * 2, (cuuint64_t)H * kD * 2, (cuuint64_t)L * H * kD * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)kSub, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static long long* g_trace = nullptr;

}  // namespace tc4

void scan_tc4_set_trace(long long* p) { tc4::g_trace = p; }

bool scan_tc4_supported(int D, int N, int C, int H, int dtype) {
    return dtype == CDSSM_BF16 && N == 2 && D == tc4::kD && C == tc4::kC && H % 4 == 0;
}

// One pass of the four-chain tensor-core scan over every chunk.  output = false: local pass (fills
// ws_state / ws_gamma for the carry pass); output = true: reads the carries from ws_state, writes y.
// status: one int in device memory, set by a bounded wait that ran out (not cleared here).
int scan_tc4_pass(bool output, const void* q, const void* k, const void* v, const void* gate_raw,
                  const float* log_dt_scale, const float* rope_freqs, float* ws_gamma, float* ws_state, void* y,
                  int* status, const DynConsts& dc, float shortcut_scale, int B, int L, int H, int pos0, int segs,
                  cudaStream_t st) {
    using namespace tc4;
    CUtensorMap tmK, tmQ;
    if (!make_tile_map(&tmK, k, B, L, H) || !make_tile_map(&tmQ, output ? q : k, B, L, H)) return CDSSM_ERR_CUDA;
    const size_t smem = sizeof(Smem);
    static bool attr = false;
    static int sms = 0;
    if (!attr) {
        if (int rc = check_cuda(cudaFuncSetAttribute(scan_tc4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)))
            return rc;
        if (int rc = check_cuda(cudaFuncSetAttribute(scan_tc4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)))
            return rc;
        int dev = 0;
        if (int rc = check_cuda(cudaGetDevice(&dev))) return rc;
        if (int rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev))) return rc;
        attr = true;
    }
    Args a;
    a.v = static_cast<const __nv_bfloat16*>(v);
    a.gate_raw = static_cast<const __nv_bfloat16*>(gate_raw);
    a.log_dt_scale = log_dt_scale; a.rope_freqs = rope_freqs;
    a.ws_gamma = ws_gamma; a.ws_state = ws_state;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.status = status; a.trace = g_trace;
    a.dc = dc; a.shortcut_scale = shortcut_scale;
    a.B = B; a.L = L; a.H = H; a.NC = (L + kC - 1) / kC; a.pos0 = pos0; a.segs = segs;
    a.HG = H / 4;
    const long long items = (long long)B * a.NC * a.HG;
    if (items > 0x7fffffff / 8) return CDSSM_ERR_UNSUPPORTED;
    a.items = (int)items;
    const int grid = (int)(items < 2LL * sms ? items : 2LL * sms);
    if (output) scan_tc4_kernel<true><<<grid, kThreads, smem, st>>>(tmK, tmQ, a);
    else scan_tc4_kernel<false><<<grid, kThreads, smem, st>>>(tmK, tmQ, a);
    return check_launch();
}

}  // namespace cdssm
