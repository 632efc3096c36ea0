// Fused scan on the tensor cores with four independent chains per thread block (tcgen05 + TMEM + TMA):
// a local pass and an output pass around the CUDA-core carry pass, fed by a dynamics pre-pass.
// Shapes: bf16 storage, state_dim N = 2, head_dim D = 128, chunk C = 128, H a multiple of 4.
//
// The single-chain kernel in scan_tc.cu keeps one warp at a time on the critical path.  Here a block
// owns the same chunk of FOUR heads; the chunk is walked in 32-token sub-blocks and every compute
// warp owns one head: UMMA tile row 32 j + t is token t of head j's sub-block.  Per sub-block:
//   G_j = K_j K_j^T, P_j = Q_j K_j^T     : the 32 x 32 diagonal blocks only - one UMMA (N = 64) per pair
//                                          of heads with every output lane but the pair's 64 masked off
//                                          (disable_output_lane), so the four heads share 64 + 64 TMEM
//                                          columns;
//   kappa, rho = K S^T, Q S^T            : products with the running states (local state z and
//                                          correction r of each head, bf16 hi + lo rows) - they
//                                          replace all off-diagonal work of the chunk form;
//   solve / read-out                     : each warp solves its own unit-lower-triangular 32 x 32
//                                          systems (local + correction) by substitution through warp
//                                          shuffles and reads y out, with rows from tcgen05.ld;
//   S <- W_31 S + K^T Omega              : state update as one UMMA (K tile as MN-major operand),
//                                          thread d applies it to column d of all four heads' states.
// The four warps never wait for one another except at the UMMA hand-offs, so four chains per block and
// two (output pass) or three (local pass) blocks per SM are in flight.  Reference semantics: z starts at
// zero at the chunk start, r starts from the chunk's carry (bf16, from the carry pass), the correction is
// read before its step.
// Algebra per sub-block with incoming states z0, r0 (restating intra_chunk_scan.cu:100-195 and
// exact_correction.cu:89-150):
//   u  = T beta (v - W kappa_z),  x = T beta W kappa_r,  T = (I + M)^-1,  M[t,i] = beta_t Gamma[t,i] G[t,i]
//   y_t = W_t rho_z,t + sum_{i<=t} Gamma[t,i] P[t,i] u_i + W0_t rho_r,t - sum_{i<t} Gamma0[t,i] P[t,i] x_i
//   z_end = W_31 z0 + sum_i Gamma[31,i] u_i k_i,   r_end = W_31 r0 - sum_i Gamma[31,i] x_i k_i
// (W, W0: inclusive / exclusive prefix products of a inside the sub-block.)  The comment above compute()
// says how the decay products are scaled out of the triangular system.
#include "cdssm_common.cuh"
#include "sm100_ptx.cuh"
#include <cstdlib>

namespace cdssm {
using namespace sm100;

namespace tc4 {

constexpr int kC = 128, kD = 128, kSub = 32, kSteps = kC / kSub;
constexpr int kThreads = 160;
constexpr uint32_t kSlab = 128 * 128;          // 64 bf16 columns x 128 rows
constexpr uint32_t kTile = 2 * kSlab;          // 32 KB

// Sizes that differ between the two passes.  The local pass carries only z (4 operand rows per head instead
// of 8, half the tensor-memory columns) and needs no Q tile, so three of its thread blocks fit on an SM.
template <bool kOutput>
struct Cfg {
    static constexpr int kRows = kOutput ? 8 : 4;               // state / omega operand rows per head (hi + lo)
    static constexpr int kN = 4 * kRows;                        // rows of the two small operand tiles
    static constexpr uint32_t kSmallSlab = kN * 128;            // bytes per 64 columns
    static constexpr uint32_t kSmallTile = 2 * kSmallSlab;
    static constexpr uint32_t kTmemCols = kOutput ? 256 : 128;
    // G and P: 64 columns each - a pair of heads per UMMA, a thread reads the 32 columns of its own head
    static constexpr uint32_t kColG = 0, kColP = 64;
    static constexpr uint32_t kColKappa = kOutput ? 128 : 64, kColRho = 160, kColUp = kOutput ? 192 : 80;
    static constexpr int kBlocksPerSm = kOutput ? 2 : 3;
};

template <bool kOutput>
struct Smem;
template <>
struct __align__(1024) Smem<true> {
    uint8_t k[2][kTile];        // rows 32 j + t: token t of head j (TMA, double buffered)
    uint8_t q[kTile];
    uint8_t s_tile[Cfg<true>::kSmallTile]; // rows 8 j + {z_re hi, lo, z_im hi, lo, r_re hi, lo, r_im hi, lo}, columns d
    uint8_t o_tile[Cfg<true>::kSmallTile]; // rows 8 j + {uz_re hi, lo, uz_im hi, lo, ur_re hi, lo, ur_im hi, lo}, columns = tile rows
    __nv_bfloat162 a[kC];       // a_t of tile row r (a is a bf16 pair in the reference's storage)
    float2 bp[2][4];            // product of a over the sub-block, per head, by step parity
    uint64_t full_k[2], full_q, mma_g, mma_p, mma_kr, mma_up, g_free, p_free, s_ready, omega_ready, bp_ready, drain;
    uint32_t tmem_base;
    int abort_flag;
};
template <>
struct __align__(1024) Smem<false> {
    uint8_t k[2][kTile];
    uint8_t s_tile[Cfg<false>::kSmallTile]; // rows 4 j + {z_re hi, lo, z_im hi, lo}, columns d
    uint8_t o_tile[Cfg<false>::kSmallTile]; // rows 4 j + {uz_re hi, lo, uz_im hi, lo}, columns = tile rows
    uint8_t q[16];              // never used: keeps the code of the two passes the same
    __nv_bfloat162 a[kC];
    float2 bp[2][4];
    uint64_t full_k[2], full_q, mma_g, mma_p, mma_kr, mma_up, g_free, p_free, s_ready, omega_ready, bp_ready, drain;
    uint32_t tmem_base;
    int abort_flag;
};

struct Args {
    const uint4* rec;            // per (token, head) record from the dynamics pre-pass (see tc4_dynamics_kernel)
    float* ws_gamma;             // (B,NC,H,2): written by the local pass
    float* ws_state;             // (B,NC,H,2,D): local pass writes z_{C-1}; the output pass reads the carry s_c
    __nv_bfloat16* y;
    int* status;
    long long* trace;
    int trace_g0, trace_block;   // debugging: first traced step and the traced block
    float shortcut_scale;
    int B, L, H, NC;
    int HG, items;               // head groups of four; items = B * NC * HG (one chunk of four heads each)
};

struct cplx { float r, i; };
__device__ __forceinline__ cplx cmul(cplx a, cplx b) { return {a.r * b.r - a.i * b.i, a.r * b.i + a.i * b.r}; }
__device__ __forceinline__ cplx cshfl(cplx v, int src) {
    return {__shfl_sync(0xffffffffu, v.r, src), __shfl_sync(0xffffffffu, v.i, src)};
}
__device__ __forceinline__ float bfr(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// element (row n, column kk) of a small K-major bf16 operand tile with 128-byte swizzle (slab: bytes per 64 columns)
__device__ __forceinline__ uint32_t small_off(uint32_t slab, int n, int kk) {
    return (uint32_t)(kk >> 6) * slab + (uint32_t)n * 128u + (uint32_t)((((kk & 63) >> 3) ^ (n & 7)) << 4) +
           (uint32_t)(kk & 7) * 2u;
}
__device__ __forceinline__ void st_hi_lo(uint8_t* tile, uint32_t slab, int n, int kk, float x) {
    const __nv_bfloat16 hi = __float2bfloat16_rn(x);
    *reinterpret_cast<__nv_bfloat16*>(tile + small_off(slab, n, kk)) = hi;
    *reinterpret_cast<__nv_bfloat16*>(tile + small_off(slab, n + 1, kk)) = __float2bfloat16_rn(x - __bfloat162float(hi));
}
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* ab) {
    const bool ok = mbar_wait(bar, parity, ab);
    return __all_sync(0xffffffffu, ok);
}



// The producer warp runs its event loop with all 32 lanes (warp-uniform values keep the descriptors in
// uniform registers); only one elected lane issues each asynchronous instruction.
// Every shared-memory descriptor used here has the same upper word (stride between eight-row groups
// 1024 bytes, Blackwell descriptor version, 128-byte swizzle), so only the lower word (start address and
// leading-dimension offset, both in 16-byte units) is carried around and advanced.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
    return ((smem_addr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ void umma_lo_e(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t.reg .b64 ad, bd;\n\t"
        "mov.b64 ad, {%1, %5};\n\t"
        "mov.b64 bd, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], ad, bd, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(acc), "r"(kDescHi)
        : "memory");
}
__device__ __forceinline__ void umma_lo_unit_e(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                               uint32_t acc, uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3) {
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t.reg .b64 ad, bd;\n\t"
        "mov.b64 ad, {%1, %9};\n\t"
        "mov.b64 bd, {%2, %9};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], ad, bd, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(acc), "r"(m0), "r"(m1), "r"(m2), "r"(m3), "r"(kDescHi)
        : "memory");
}
__device__ __forceinline__ void umma_commit_e(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t e;
    asm volatile(
        "{\n\t.reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, e;\n\t}"
        : "=r"(e));
    return e != 0;
}
__device__ __forceinline__ bool warp_test(uint64_t* bar, uint32_t parity) {
    return __all_sync(0xffffffffu, mbar_test(bar, parity));
}

// ------------------------------------------------------------------------------------------
// Producer (one elected lane of warp 4): TMA and UMMA issue, event driven.  The CTA's work is a flat
// sequence of sub-block steps g = 0 .. 4 * n_items - 1; item (g >> 2) is chunk c of heads h0 .. h0 + 3
// of batch row b.  Every barrier completes once per step, so its parity is that of g.
// ------------------------------------------------------------------------------------------
template <bool kOutput>
__device__ __forceinline__ void producer(Smem<kOutput>& sm, const CUtensorMap* tmK, const CUtensorMap* tmQ, const Args& a) {
    using C = Cfg<kOutput>;
    volatile int* ab = &sm.abort_flag;
    const uint32_t tm = sm.tmem_base;
    constexpr uint32_t idesc_s = umma_idesc_bf16(128, C::kN, false, false);   // kappa / rho: N = state rows
    constexpr uint32_t idesc64 = umma_idesc_bf16(128, 64, false, false);
    constexpr uint32_t idesc_up = umma_idesc_bf16(128, C::kN, true, false);
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
        if (elect_one()) {
            mbar_arrive_expect_tx(bar, kTile);
#pragma unroll 1
            for (int j = 0; j < 4; j++) {
                tma_load_4d(dst + j * kSub * 128, tmap, bar, 0, h0 + j, l0, b);
                tma_load_4d(dst + kSlab + j * kSub * 128, tmap, bar, 64, h0 + j, l0, b);
            }
        }
        __syncwarp();
    };
    if (NS > 0) {
        load_tile(sm.k[0], tmK, &sm.full_k[0], 0); pend_k[0] = true;
        if (kOutput) { load_tile(sm.q, tmQ, &sm.full_q, 0); pend_q = true; }
        load_tile(sm.k[1], tmK, &sm.full_k[1], 1); pend_k[1] = true;
    }
    // Lower descriptor words of the operands at k-step 0.  A k-step is 32 bytes (+2); after four of them the
    // next 64-column slab starts (K-major tiles).  The MN-major K tile advances 16 tile rows = 2 KB per step.
    const uint32_t lK[2] = {desc_lo(kaddr[0], 16), desc_lo(kaddr[1], 16)};
    const uint32_t lKt[2] = {desc_lo(kaddr[0], kSlab), desc_lo(kaddr[1], kSlab)};
    const uint32_t lQ = desc_lo(qaddr, 16), lS = desc_lo(saddr, 16), lO = desc_lo(oaddr, 16);
    constexpr uint32_t kBigJump = (kSlab >> 4) - 8, kSmallJump = (C::kSmallSlab >> 4) - 8;
    // Progress counters: UMMA groups issued (G, P, kappa / rho, state update) and tiles requested.
    int i_g = 0, i_p = 0, i_kr = 0, i_up = 0, i_lq = 1, i_lk = 2;
    bool k_ok = false, q_ok = false;   // the K tile of step i_g / the Q tile of step i_p has landed
    uint64_t last = global_ns();
    uint32_t idle = 0;
#define TC4_PSTAMP(n, idx) do { if (a.trace && (threadIdx.x & 31) == 0 && blockIdx.x == a.trace_block && (n) >= a.trace_g0 && (n) < a.trace_g0 + 16) a.trace[(((n) - a.trace_g0) * 5 + 4) * 16 + (idx)] = clock64(); } while (0)
    auto par = [](int n) { return (uint32_t)(n & 1); };
    // Tasks in order of urgency: the state update and kappa / rho sit on the compute warps' critical path; the
    // tile loads and the Gram blocks of the NEXT step do not.  G (needs only the K tile) and P (needs the Q
    // tile, whose single buffer is refilled late) are separate tasks so that G is never held back by Q.
    while (i_up < NS) {
        bool progress = false;
        // state update: A = K tile read MN-major (M = d, two 64-wide groups 16 KB apart; K = tile rows,
        // 16 per instruction = 2 KB), B = omega tile (32 rows x 128 tile rows).  Issued only once the
        // completion of the previous update has been observed (i_lk), so that the mma_up barrier is never
        // more than one phase ahead of what this loop tests.
        if (i_up < i_kr && i_lk - 2 >= i_up && warp_test(&sm.omega_ready, par(i_up))) {
            const int st = i_up & 1;
            tc_fence_after();
            {
                uint32_t al = lKt[st], bl = lO;
#pragma unroll 1
                for (int j = 0; j < 8; j++) {
                    umma_lo_e(tm + C::kColUp, al, bl, idesc_up, j);
                    al += 2048 >> 4;
                    bl += (j == 3) ? 2 + kSmallJump : 2;
                }
            }
            umma_commit_e(&sm.mma_up);
            TC4_PSTAMP(i_up, 3);
            i_up++; progress = true;
        } else if (i_kr < i_g && (!kOutput || i_kr < i_p) && warp_test(&sm.s_ready, par(i_kr))) {
            // kappa = K S^T, rho = Q S^T (G and P of the step have been issued, so its tiles have landed)
            const int st = i_kr & 1;
            tc_fence_after();
            {
                uint32_t ak = lK[st], aq = lQ, bl = lS;
#pragma unroll 1
                for (int j = 0; j < 8; j++) {
                    umma_lo_e(tm + C::kColKappa, ak, bl, idesc_s, j);
                    if (kOutput) umma_lo_e(tm + C::kColRho, aq, bl, idesc_s, j);
                    const uint32_t big = (j == 3) ? 2 + kBigJump : 2;
                    ak += big;
                    aq += big;
                    bl += (j == 3) ? 2 + kSmallJump : 2;
                }
            }
            umma_commit_e(&sm.mma_kr);
            TC4_PSTAMP(i_kr, 2);
            i_kr++; progress = true;
        } else if (i_lk - 2 < i_up && i_lk - 2 < NS && warp_test(&sm.mma_up, par(i_lk - 2))) {
            // the K stage of step n is free once its state update has completed
            if (i_lk < NS) { TC4_PSTAMP(i_lk, 5); load_tile(sm.k[i_lk & 1], tmK, &sm.full_k[i_lk & 1], i_lk); pend_k[i_lk & 1] = true; }
            i_lk++; progress = true;
        } else if (kOutput && i_lq <= i_kr && i_lq <= NS && warp_test(&sm.mma_kr, par(i_lq - 1)) &&
                   warp_test(&sm.p_free, par(i_lq - 1))) {
            // Q tile of step n is free once its UMMAs have completed (rho is committed after P of the same step,
            // so mma_kr covers both) and the compute warps have taken |q| from it (before p_free)
            if (i_lq < NS) { TC4_PSTAMP(i_lq, 4); load_tile(sm.q, tmQ, &sm.full_q, i_lq); pend_q = true; }
            i_lq++; progress = true;
        } else {
            if (kOutput && i_p < NS && i_p < i_g) {   // P = Q K^T of step i_p, the diagonal blocks of both pairs of heads
                if (!q_ok && warp_test(&sm.full_q, par(i_p))) { q_ok = true; pend_q = false; }
                if (q_ok && (i_p == 0 || warp_test(&sm.p_free, par(i_p - 1)))) {
                    const int st = i_p & 1;
                    tc_fence_after();
                    uint32_t ak = lK[st], aq = lQ;
                    constexpr uint32_t r2 = 2 * (kSub * 128 >> 4), all = 0xffffffffu;
#pragma unroll 1
                    for (int j = 0; j < 8; j++) {
                        umma_lo_unit_e(tm + C::kColP, aq, ak, idesc64, j, 0u, 0u, all, all);
                        umma_lo_unit_e(tm + C::kColP, aq, ak + r2, idesc64, j, all, all, 0u, 0u);
                        const uint32_t big = (j == 3) ? 2 + kBigJump : 2;
                        ak += big;
                        aq += big;
                    }
                    umma_commit_e(&sm.mma_p);
                    TC4_PSTAMP(i_p, 1);
                    i_p++; q_ok = false; progress = true;
                }
            }
            if (!progress && i_g < NS) {   // G = K K^T of step i_g, likewise
                const int st = i_g & 1;
                if (!k_ok && warp_test(&sm.full_k[st], (i_g >> 1) & 1)) { k_ok = true; pend_k[st] = false; }
                if (k_ok && (i_g == 0 || warp_test(&sm.g_free, par(i_g - 1)))) {
                    tc_fence_after();
                    TC4_PSTAMP(i_g, 0);
                    uint32_t ak = lK[st];
                    constexpr uint32_t r2 = 2 * (kSub * 128 >> 4), all = 0xffffffffu;
#pragma unroll 1
                    for (int j = 0; j < 8; j++) {
                        umma_lo_unit_e(tm + C::kColG, ak, ak, idesc64, j, 0u, 0u, all, all);
                        umma_lo_unit_e(tm + C::kColG, ak, ak + r2, idesc64, j, all, all, 0u, 0u);
                        ak += (j == 3) ? 2 + kBigJump : 2;
                    }
                    umma_commit_e(&sm.mma_g);
                    i_g++; k_ok = false; progress = true;
                }
            }
        }
        if (progress) {
            last = global_ns();
        } else if ((++idle & 7) != 0) {
            __nanosleep(200);
        } else if (__any_sync(0xffffffffu, *ab || global_ns() - last > kWaitLimitNs)) {
            code = 1 + (i_g > i_kr) + 2 * (i_kr > i_up);
            *ab = 1;
            break;
        }
    }
    if (code && elect_one()) {   // the lane that issued the UMMAs and the TMA loads
        atomicCAS(a.status, 0, 300 + code);
        umma_commit(&sm.drain);
        int never = 0;
        mbar_wait(&sm.drain, 0, &never);
        if (pend_k[0]) mbar_wait(&sm.full_k[0], 0, &never), mbar_wait(&sm.full_k[0], 1, &never);
        if (pend_k[1]) mbar_wait(&sm.full_k[1], 0, &never), mbar_wait(&sm.full_k[1], 1, &never);
        if (pend_q) mbar_wait(&sm.full_q, 0, &never), mbar_wait(&sm.full_q, 1, &never);
    }
    __syncwarp();
}

// ------------------------------------------------------------------------------------------
// Compute warps.  Thread t = 32 j + tl is token tl of head j's sub-block (TMEM lane t) and, for the state
// hand-off, column d = t of all four heads' states.
// kOutput = false: local pass - z only; writes z_{C-1} and the chunk's decay product for the carry pass.
// kOutput = true : output pass - z and r (r starts from the chunk's carry), writes y.
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
// Record of one (token, head), written by the dynamics pre-pass: {a_re, a_im | vg_re, vg_im | beta, sel_C | -}
// as bf16 pairs (all of them are bf16 values in the reference's storage).  Layout (B, NC*4, H, 32 tokens):
// the 32 tokens of a head's sub-block are contiguous, so a warp fetches its step with one 512-byte load.
__device__ __forceinline__ size_t rec_index(const Args& a, int b, int c, int sub, int hd, int tl) {
    return ((((size_t)b * a.NC + c) * kSteps + sub) * a.H + hd) * kSub + tl;
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

struct BlockOut {   // what a sub-block walk hands back
    cplx wh, xh;    // omega columns: Gamma[31,t] u~_t and -Gamma[31,t] x~_t
    cplx ysum;      // pd u~_t + in-block read-out + W rho_z + W0 rho_r (before the |q|^-1 factor)
    // used by the three-blocks-per-SM variant only:
    float pd;       // P_raw[t,t]
    bool ok;        // false: a bounded wait ran out
    cplx W, W0;     // inclusive / exclusive prefix product of a at this token
};

// The walk with explicit decay products (any a, including zeros): phases A (coefficients
// cc[i] = a_t Gamma0[t,i] G_raw[t,i], Gamma0 built leftwards from the diagonal), B (substitution for
// u~ = n u, x~ = n x) and C (in-block read-out; the correction is read before its step,
// exact_correction.cu:90-94).  Reads G / P from tensor memory itself.
template <bool kOutput>
__device__ __forceinline__ BlockOut robust_block(const Smem<kOutput>& sm, uint32_t tlane, int J, int tl, cplx at, cplx vg, float be,
                                             float nt, cplx kz, cplx kr, cplx rz, cplx rr) {
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
    // cc is indexed with run-time group numbers on purpose: it lives in local memory, so this rarely taken
    // walk does not compete for registers with the scaled walk it is inlined next to.
    cplx cc[32];
    {
        cplx cur = {1.f, 0.f};
#pragma unroll 1
        for (int grp = 3; grp >= 0; grp--) {
            float g8[8];
            tmem_ld8(tlane + Cfg<kOutput>::kColG + 32 * (J & 1) + grp * 8, g8);
#pragma unroll
            for (int e = 7; e >= 0; e--) {
                const int i = grp * 8 + e;
                const float2 ai = __bfloat1622float2(sm.a[J * 32 + i]);
                const bool on = i < tl;
                const cplx fg = cmul(at, cur);
                cc[i] = {on ? fg.r * g8[e] : 0.f, on ? fg.i * g8[e] : 0.f};
                const cplx nx = cmul(cur, cplx{ai.x, ai.y});
                cur = {on ? nx.r : cur.r, on ? nx.i : cur.i};
            }
        }
    }
    const cplx wkz = cmul(W, kz);
    cplx cw = {nt * be * (vg.r - nt * wkz.r), nt * be * (vg.i - nt * wkz.i)};
    cplx cx = {0.f, 0.f};
    if (kOutput) {
        const cplx wkr = cmul(W, kr);
        cx = {nt * be * nt * wkr.r, nt * be * nt * wkr.i};
    }
#pragma unroll 1
    for (int grp = 0; grp < 4; grp++) {
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int i = grp * 8 + e;
            const float cr_ = bnn * cc[i].r, ci_ = bnn * cc[i].i;
            const cplx uw = cshfl(cw, i);
            cw.r -= cr_ * uw.r - ci_ * uw.i;
            cw.i -= cr_ * uw.i + ci_ * uw.r;
            if (kOutput) {
                const cplx ux = cshfl(cx, i);
                cx.r -= cr_ * ux.r - ci_ * ux.i;
                cx.i -= cr_ * ux.i + ci_ * ux.r;
            }
        }
    }
    BlockOut o;
    o.wh = cmul(V, cw);
    o.xh = {0.f, 0.f};
    o.ysum = {0.f, 0.f};
    if (kOutput) {
        const cplx xv = cmul(V, cx);
        o.xh = {-xv.r, -xv.i};
        cplx yin = {0.f, 0.f};
        float pd = 0.f;
        cplx cur = {1.f, 0.f};
#pragma unroll 1
        for (int grp = 3; grp >= 0; grp--) {
            float p8[8];
            tmem_ld8(tlane + Cfg<kOutput>::kColP + 32 * (J & 1) + grp * 8, p8);
#pragma unroll
            for (int e = 7; e >= 0; e--) {
                const int i = grp * 8 + e;
                const float2 ai = __bfloat1622float2(sm.a[J * 32 + i]);
                const cplx uw = cshfl(cw, i), ux = cshfl(cx, i);
                const bool on = i < tl;
                pd = (i == tl) ? p8[e] : pd;
                const cplx au = cmul(at, uw);
                const cplx ee = cmul(cur, cplx{au.r - ux.r, au.i - ux.i});
                const float pi = on ? p8[e] : 0.f;
                yin.r += pi * ee.r;
                yin.i += pi * ee.i;
                const cplx nx = cmul(cur, cplx{ai.x, ai.y});
                cur = {on ? nx.r : cur.r, on ? nx.i : cur.i};
            }
        }
        const cplx yz = cmul(W, rz), yr0 = cmul(W0, rr);
        o.ysum = {pd * cw.r + yin.r + yz.r + yr0.r, pd * cw.i + yin.i + yz.i + yr0.i};
    }
    return o;
}

#define TC4_STAMP(idx) do { if (a.trace && blockIdx.x == a.trace_block && tl == 0 && g >= a.trace_g0 && g < a.trace_g0 + 16) a.trace[((g - a.trace_g0) * 5 + J) * 16 + (idx)] = clock64(); } while (0)

struct Tok {   // per-token quantities of one sub-block step, prepared one step ahead
    cplx at, vg;        // a_t, vp-scaled value
    cplx viw;           // vg / D_t
    cplx D, D0;         // scaling of token t (see prepare) and of token t - 1
    cplx R, D31;        // reference product W_15 and D of the last token: W_31 = D31 R
    float be, sc;       // beta_t, sel_C gate
    bool fast;
};
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

// Unpacks the token's record and forms the decay scalings of the sub-block.  The scaled walk only needs
// ratios W_t / W_i of the prefix products W_t = a_0 ... a_t, so they are taken relative to the middle of the
// sub-block, D_t = W_t / W_15: lanes 0-15 hold the suffix product a_{t+1} ... a_15 = 1 / D_t, lanes 16-31 the
// prefix product a_16 ... a_t = D_t, and neither half leaves the float range unless one half alone decays by
// more than 1e-30 (then, or with the zero padding behind the sequence end, the explicit walk is taken).
// Publishes a_t and the block product W_31 for step g (read by all threads in the state hand-off).
template <class SmemT>
__device__ __forceinline__ Tok prepare(SmemT& sm, const uint4& rec, int g, int J, int tl) {
    Tok k;
    k.at = {bf_lo(rec.x), bf_hi(rec.x)};
    k.vg = {bf_lo(rec.y), bf_hi(rec.y)};
    k.be = bf_lo(rec.z);
    k.sc = bf_hi(rec.z);
    sm.a[threadIdx.x] = *reinterpret_cast<const __nv_bfloat162*>(&rec.x);
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
    if (tl == 31) {
        const cplx bp = cmul(k.D, incl0);        // W_31
        sm.bp[g & 1][J] = make_float2(bp.r, bp.i);
    }
    __syncwarp();
    if (tl == 0) mbar_arrive(&sm.bp_ready);
    return k;
}

template <bool kOutput>
__device__ __forceinline__ void compute(Smem<kOutput>& sm, const Args& a) {
    using C = Cfg<kOutput>;
    constexpr int R = C::kRows;
    volatile int* ab = &sm.abort_flag;
    const int t = threadIdx.x, J = t >> 5, tl = t & 31;
    const int H = a.H, L = a.L;
    const uint32_t tlane = sm.tmem_base + ((uint32_t)(J * 32) << 16);
    const int n_items = ((int)blockIdx.x < a.items) ? (a.items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int NS = n_items * kSteps;
    if (NS == 0) return;
    int code = 0;
    cplx Sz[4], Sr[4], gam[4];
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    ItemPos cur = item_pos(a, blockIdx.x), nxi = cur;
    Tok tk;
    {
        const bool valid = cur.c * kC + tl < L;
        const uint4 first = valid ? __ldg(a.rec + rec_index(a, cur.b, cur.c, 0, cur.h0 + J, tl)) : zero4;
        tk = prepare(sm, first, 0, J, tl);
    }
    for (int g = 0; g < NS && !code; g++) {
        const uint32_t ph = g & 1;
        const int step = g & 3;
        if (step == 0) {
            if (g > 0) cur = nxi;
            nxi = item_pos(a, (int)blockIdx.x + ((g >> 2) + 1) * (int)gridDim.x);
        }
        const int l = cur.c * kC + step * kSub + tl, hd = cur.h0 + J;
        const bool valid = l < L;
        const size_t unit0 = ((size_t)cur.b * a.NC + cur.c) * H + cur.h0;   // workspace slot of head h0
        if (step == 0) {   // states at the chunk start, column d = t of every head
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
        }
        // ---- publish the states for kappa / rho of this step
        TC4_STAMP(11);
#pragma unroll
        for (int u = 0; u < 4; u++) {
            st_hi_lo(sm.s_tile, C::kSmallSlab, R * u + 0, t, Sz[u].r);
            st_hi_lo(sm.s_tile, C::kSmallSlab, R * u + 2, t, Sz[u].i);
            if (kOutput) {
                st_hi_lo(sm.s_tile, C::kSmallSlab, R * u + 4, t, Sr[u].r);
                st_hi_lo(sm.s_tile, C::kSmallSlab, R * u + 6, t, Sr[u].i);
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (tl == 0) mbar_arrive(&sm.s_ready);
        TC4_STAMP(0);
        // ---- fetch the record of step g + 1 (the next item's first sub-block after this item's last)
        uint4 rec = zero4;
        if (g + 1 < NS) {
            const ItemPos& np = (step + 1 < kSteps) ? cur : nxi;
            const int nsub = (step + 1) & 3;
            if (np.c * kC + nsub * kSub + tl < L) rec = __ldg(a.rec + rec_index(a, np.b, np.c, nsub, np.h0 + J, tl));
        }
        const cplx at = tk.at, vg = tk.vg;
        const float be = tk.be;
        TC4_STAMP(2);
        // ---- |q_t|^-1 from the Q tile row (swizzled 16-byte pieces): the compute warps have time for it while
        // they wait for UMMAs, and the tensor pipe is the busier resource
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
                    for (int e = 0; e < 8; e++) qq = fmaf(f[e], f[e], qq);
                }
            mt = rsqrtf(qq + kEps);
        }
        // ---- Gram rows of the own head: |k_t|^-1 from the diagonal
        if (!warp_wait(&sm.mma_g, ph, ab)) { code = 13; break; }
        tc_fence_after();
        TC4_STAMP(3);
        float gs[32], p[32];
        float pd = 0.f;
        tmem_ld32(tlane + C::kColG + 32 * (J & 1), gs);
        float gd = 0.f;
#pragma unroll
        for (int i = 0; i < 32; i++) gd = (i == tl) ? gs[i] : gd;
        const float nt = rsqrtf(gd + kEps);
        const float bnn = be * nt * nt;
        BlockOut o;
        if (tk.fast) {
            tc_fence_before();
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.g_free);   // G is in registers
            // coefficients of the real system, zero on and above the diagonal
#pragma unroll
            for (int i = 0; i < 32; i++) gs[i] = (i < tl) ? -bnn * gs[i] : 0.f;
            if (kOutput) {
                if (!warp_wait(&sm.mma_p, ph, ab)) { code = 16; break; }
                tc_fence_after();
                tmem_ld32(tlane + C::kColP + 32 * (J & 1), p);
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    pd = (i == tl) ? p[i] : pd;
                    p[i] = (i < tl) ? p[i] : 0.f;
                }
            }
            if (kOutput) {
                tc_fence_before();
                __syncwarp();
                if (tl == 0) mbar_arrive(&sm.p_free);   // P is in registers, |q| has been taken from the Q tile
            }
            if (!warp_wait(&sm.mma_kr, ph, ab)) { code = 12; break; }
            tc_fence_after();
            TC4_STAMP(4);
            float k8[8], r8[8];
            if (kOutput) tmem_ld8x2(tlane + C::kColKappa + 8 * J, k8, tlane + C::kColRho + 8 * J, r8);
            else tmem_ld4(tlane + C::kColKappa + 4 * J, k8);
            const cplx rkz = cmul(tk.R, cplx{k8[0] + k8[1], k8[2] + k8[3]});
            cplx cw = {nt * be * (tk.viw.r - nt * rkz.r), nt * be * (tk.viw.i - nt * rkz.i)};
            cplx cx = {0.f, 0.f}, accu = {0.f, 0.f}, accx = {0.f, 0.f};
            if (kOutput) {
                const cplx rkr = cmul(tk.R, cplx{k8[4] + k8[5], k8[6] + k8[7]});
                cx = {nt * be * nt * rkr.r, nt * be * nt * rkr.i};
            }
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const cplx uw = cshfl(cw, i);
                cw.r = fmaf(gs[i], uw.r, cw.r);
                cw.i = fmaf(gs[i], uw.i, cw.i);
                if (kOutput) {
                    const cplx ux = cshfl(cx, i);
                    cx.r = fmaf(gs[i], ux.r, cx.r);
                    cx.i = fmaf(gs[i], ux.i, cx.i);
                    accu.r = fmaf(p[i], uw.r, accu.r);
                    accu.i = fmaf(p[i], uw.i, accu.i);
                    accx.r = fmaf(p[i], ux.r, accx.r);
                    accx.i = fmaf(p[i], ux.i, accx.i);
                }
            }
            o.wh = cmul(tk.D31, cw);
            if (kOutput) {
                const cplx xv = cmul(tk.D31, cx);
                o.xh = {-xv.r, -xv.i};
                const cplx rz = cmul(tk.R, cplx{r8[0] + r8[1], r8[2] + r8[3]});
                const cplx rr = cmul(tk.R, cplx{r8[4] + r8[5], r8[6] + r8[7]});
                const cplx yl = cmul(tk.D, cplx{rz.r + pd * cw.r + accu.r, rz.i + pd * cw.i + accu.i});
                cplx yc = cmul(tk.D0, cplx{rr.r - accx.r, rr.i - accx.i});
                if (tl == 0) yc = {r8[4] + r8[5], r8[6] + r8[7]};   // W0 = 1: the carried correction itself
                o.ysum = {yl.r + yc.r, yl.i + yc.i};
            }
        } else {
            if (kOutput) {
                tmem_ld32(tlane + C::kColP + 32 * (J & 1), p);
#pragma unroll
                for (int i = 0; i < 32; i++) pd = (i == tl) ? p[i] : pd;
            }
            if (!warp_wait(&sm.mma_kr, ph, ab)) { code = 12; break; }
            tc_fence_after();
            float k8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, r8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (kOutput) tmem_ld8x2(tlane + C::kColKappa + 8 * J, k8, tlane + C::kColRho + 8 * J, r8);
            else tmem_ld4(tlane + C::kColKappa + 4 * J, k8);
            if (kOutput) { if (!warp_wait(&sm.mma_p, ph, ab)) { code = 16; break; } tc_fence_after(); }
            o = robust_block<kOutput>(sm, tlane, J, tl, at, vg, be, nt, cplx{k8[0] + k8[1], k8[2] + k8[3]},
                                      cplx{k8[4] + k8[5], k8[6] + k8[7]}, cplx{r8[0] + r8[1], r8[2] + r8[3]},
                                      cplx{r8[4] + r8[5], r8[6] + r8[7]});
            tc_fence_before();
            __syncwarp();
            if (tl == 0) { mbar_arrive(&sm.g_free); if (kOutput) mbar_arrive(&sm.p_free); }
        }
        TC4_STAMP(5);
        // ---- omega columns of the state update: z += sum_t Gamma[31,t] u~_t k_t, r -= sum_t Gamma[31,t] x~_t k_t
        st_hi_lo(sm.o_tile, C::kSmallSlab, R * J + 0, t, o.wh.r);
        st_hi_lo(sm.o_tile, C::kSmallSlab, R * J + 2, t, o.wh.i);
        if (kOutput) {
            st_hi_lo(sm.o_tile, C::kSmallSlab, R * J + 4, t, o.xh.r);
            st_hi_lo(sm.o_tile, C::kSmallSlab, R * J + 6, t, o.xh.i);
        }
        fence_proxy_async();
        __syncwarp();
        if (tl == 0) mbar_arrive(&sm.omega_ready);
        if (kOutput) {
            float yr = mt * o.ysum.r, yi = mt * o.ysum.i;
            if (a.shortcut_scale != 0.f) {   // block.py:202-208
                const float qk = mt * nt * pd;
                yr += a.shortcut_scale * qk * qk * vg.r;
                yi += a.shortcut_scale * qk * qk * vg.i;
            }
            if (valid) {
                __nv_bfloat162 ov = __floats2bfloat162_rn(bfr(yr) * tk.sc, bfr(yi) * tk.sc);
                *reinterpret_cast<__nv_bfloat162*>(a.y + (((size_t)cur.b * L + l) * H + hd) * 2) = ov;
            }
        }
        TC4_STAMP(1);
        // ---- the next step's token while the state-update UMMA runs.  This step's block products are waited
        // for first: prepare() arrives on the same barrier for the next step, and a wait must never be two
        // phases behind its barrier.
        if (!warp_wait(&sm.bp_ready, ph, ab)) { code = 14; break; }
        if (g + 1 < NS) tk = prepare(sm, rec, g + 1, J, tl);
        TC4_STAMP(8);
        // ---- state hand-off: S <- BP S + K^T omega, column d = t of every head
        if (!warp_wait(&sm.mma_up, ph, ab)) { code = 15; break; }
        tc_fence_after();
        TC4_STAMP(6);
        if (!kOutput || step + 1 < kSteps) {
            float up[32];
            if (kOutput) tmem_ld32(tlane + C::kColUp, up);
            else tmem_ld16(tlane + C::kColUp, up);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const cplx bpu = {sm.bp[ph][u].x, sm.bp[ph][u].y};
                const cplx nz = cmul(bpu, Sz[u]);
                Sz[u] = {nz.r + up[R * u] + up[R * u + 1], nz.i + up[R * u + 2] + up[R * u + 3]};
                if (kOutput) {
                    const cplx nr = cmul(bpu, Sr[u]);
                    Sr[u] = {nr.r + up[R * u + 4] + up[R * u + 5], nr.i + up[R * u + 6] + up[R * u + 7]};
                } else {
                    gam[u] = cmul(bpu, gam[u]);
                }
            }
        }
        tc_fence_before();
        TC4_STAMP(7);
        if (!kOutput && step + 1 == kSteps) {
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

// ==========================================================================================
// Output pass, three thread blocks per SM.
//
// The output pass above is held to two blocks per SM by its three 32 KB tiles (K of this step, K of the
// next, Q) and its 224 tensor-memory columns.  This variant lives on two tile buffers and 128 columns:
//   * K of step g sits in tile[g & 1], Q of step g in the other buffer.  Q is only needed for the read-out
//     side (P, rho, |q|), K for the solve (G, kappa) and the state update: once P, rho and |q| of step g are
//     done, K of step g + 1 is fetched into Q's buffer (early enough for G of the next step), and once the
//     state update of step g has completed, Q of step g + 1 is fetched into K's buffer (it lands a couple of
//     thousand cycles into step g + 1, which is when the solve has been set up and P is needed).
//   * G and P take turns in the same 64 columns (P is issued when every warp has its G row in registers),
//     kappa and the state update share 32 columns (the update is read before the next states are published),
//     rho has 32 of its own and is read after the substitution loop.
//   * the states (operand of kappa / rho) and the omega columns (operand of the update) take turns in one
//     small tile, so every token thread writes its whole omega column (its head's eight values and zeros).
// ==========================================================================================
struct __align__(1024) Smem3 {
    uint8_t tile[2][kTile];
    uint8_t so_tile[Cfg<true>::kSmallTile];
    __nv_bfloat162 a[kC];
    float2 bp[2][4];
    uint64_t full_k, full_q, mma_g, mma_p, mma_k, mma_r, mma_up, g_free, p_free, r_free, s_ready, omega_ready,
        bp_ready, drain;
    uint32_t tmem_base;
    int abort_flag;
};
constexpr uint32_t k3TmemCols = 128, k3ColGP = 0, k3ColKU = 64, k3ColRho = 96;

__device__ __forceinline__ void producer3(Smem3& sm, const CUtensorMap* tmK, const CUtensorMap* tmQ, const Args& a) {
    using C = Cfg<true>;
    volatile int* ab = &sm.abort_flag;
    const uint32_t tm = sm.tmem_base;
    constexpr uint32_t idesc_s = umma_idesc_bf16(128, C::kN, false, false);
    constexpr uint32_t idesc64 = umma_idesc_bf16(128, 64, false, false);
    constexpr uint32_t idesc_up = umma_idesc_bf16(128, C::kN, true, false);
    const uint32_t taddr[2] = {smem_u32(sm.tile[0]), smem_u32(sm.tile[1])};
    const uint32_t soaddr = smem_u32(sm.so_tile);
    bool pend_k = false, pend_q = false;
    int code = 0;
    const int n_items = ((int)blockIdx.x < a.items) ? (a.items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int NS = n_items * kSteps;
    auto load_tile = [&](uint8_t* dst, const CUtensorMap* tmap, uint64_t* bar, int g) {
        const int item = (int)blockIdx.x + (g >> 2) * (int)gridDim.x;
        const int h0 = (item % a.HG) * 4, c = (item / a.HG) % a.NC, b = item / (a.HG * a.NC);
        const int l0 = c * kC + (g & 3) * kSub;
        if (elect_one()) {
            mbar_arrive_expect_tx(bar, kTile);
#pragma unroll 1
            for (int j = 0; j < 4; j++) {
                tma_load_4d(dst + j * kSub * 128, tmap, bar, 0, h0 + j, l0, b);
                tma_load_4d(dst + kSlab + j * kSub * 128, tmap, bar, 64, h0 + j, l0, b);
            }
        }
        __syncwarp();
    };
    if (NS > 0) {
        load_tile(sm.tile[0], tmK, &sm.full_k, 0); pend_k = true;
        load_tile(sm.tile[1], tmQ, &sm.full_q, 0); pend_q = true;
    }
    const uint32_t lT[2] = {desc_lo(taddr[0], 16), desc_lo(taddr[1], 16)};        // K-major tile operands
    const uint32_t lTt[2] = {desc_lo(taddr[0], kSlab), desc_lo(taddr[1], kSlab)}; // MN-major (state update)
    const uint32_t lSO = desc_lo(soaddr, 16);
    constexpr uint32_t kBigJump = (kSlab >> 4) - 8, kSmallJump = (C::kSmallSlab >> 4) - 8;
    // UMMA groups issued (G, P, kappa, rho, state update) and the next tile loads (K / Q of step i_lk / i_lq)
    int i_g = 0, i_p = 0, i_k = 0, i_r = 0, i_up = 0, i_lk = 1, i_lq = 1;
    bool k_ok = false, q_ok = false;   // the K tile of step i_g / the Q tile of step i_p has landed
    uint64_t last = global_ns();
    uint32_t idle = 0;
    auto par = [](int n) { return (uint32_t)(n & 1); };
    while (i_up < NS) {
        bool progress = false;
        if (i_up < i_k && i_lq > i_up && warp_test(&sm.omega_ready, par(i_up))) {
            // state update (issued only once the completion of the previous one has been observed by the Q
            // reload below, so that mma_up is never more than one phase ahead of what this loop tests)
            tc_fence_after();
            uint32_t al = lTt[i_up & 1], bl = lSO;
#pragma unroll 1
            for (int j = 0; j < 8; j++) {
                umma_lo_e(tm + k3ColKU, al, bl, idesc_up, j);
                al += 2048 >> 4;
                bl += (j == 3) ? 2 + kSmallJump : 2;
            }
            umma_commit_e(&sm.mma_up);
            i_up++; progress = true;
        } else if (i_k < i_g && warp_test(&sm.s_ready, par(i_k))) {
            // kappa = K S^T (G of the step has been issued, so its K tile has landed)
            tc_fence_after();
            uint32_t ak = lT[i_k & 1], bl = lSO;
#pragma unroll 1
            for (int j = 0; j < 8; j++) {
                umma_lo_e(tm + k3ColKU, ak, bl, idesc_s, j);
                ak += (j == 3) ? 2 + kBigJump : 2;
                bl += (j == 3) ? 2 + kSmallJump : 2;
            }
            umma_commit_e(&sm.mma_k);
            i_k++; progress = true;
        } else if (i_r < i_p && i_r < i_k && (i_r == 0 || warp_test(&sm.r_free, par(i_r - 1)))) {
            // rho = Q S^T (P of the step has been issued: its Q tile has landed; kappa of the step has been
            // issued: its states are published)
            tc_fence_after();
            uint32_t aq = lT[(i_r + 1) & 1], bl = lSO;
#pragma unroll 1
            for (int j = 0; j < 8; j++) {
                umma_lo_e(tm + k3ColRho, aq, bl, idesc_s, j);
                aq += (j == 3) ? 2 + kBigJump : 2;
                bl += (j == 3) ? 2 + kSmallJump : 2;
            }
            umma_commit_e(&sm.mma_r);
            i_r++; progress = true;
        } else if (i_lq <= NS && i_lq <= i_up && warp_test(&sm.mma_up, par(i_lq - 1))) {
            // the update of step n - 1 has completed: its K buffer takes the Q tile of step n
            if (i_lq < NS) { load_tile(sm.tile[(i_lq + 1) & 1], tmQ, &sm.full_q, i_lq); pend_q = true; }
            i_lq++; progress = true;
        } else if (i_lk <= NS && i_lk <= i_r && i_lk <= i_p && warp_test(&sm.mma_r, par(i_lk - 1)) &&
                   warp_test(&sm.mma_p, par(i_lk - 1)) && warp_test(&sm.p_free, par(i_lk - 1))) {
            // P, rho and |q| of step n - 1 are done: its Q buffer takes the K tile of step n
            if (i_lk < NS) { load_tile(sm.tile[i_lk & 1], tmK, &sm.full_k, i_lk); pend_k = true; }
            i_lk++; progress = true;
        } else {
            if (i_p < NS && i_p < i_g) {   // P = Q K^T of step i_p into the columns its G has been read from
                if (!q_ok && warp_test(&sm.full_q, par(i_p))) { q_ok = true; pend_q = false; }
                if (q_ok && warp_test(&sm.g_free, par(i_p))) {
                    tc_fence_after();
                    uint32_t ak = lT[i_p & 1], aq = lT[(i_p + 1) & 1];
                    constexpr uint32_t r2 = 2 * (kSub * 128 >> 4), all = 0xffffffffu;
#pragma unroll 1
                    for (int j = 0; j < 8; j++) {
                        umma_lo_unit_e(tm + k3ColGP, aq, ak, idesc64, j, 0u, 0u, all, all);
                        umma_lo_unit_e(tm + k3ColGP, aq, ak + r2, idesc64, j, all, all, 0u, 0u);
                        const uint32_t big = (j == 3) ? 2 + kBigJump : 2;
                        ak += big;
                        aq += big;
                    }
                    umma_commit_e(&sm.mma_p);
                    i_p++; q_ok = false; progress = true;
                }
            }
            if (!progress && i_g < NS) {   // G = K K^T of step i_g into the columns the previous P has been read from
                if (!k_ok && warp_test(&sm.full_k, par(i_g))) { k_ok = true; pend_k = false; }
                if (k_ok && (i_g == 0 || warp_test(&sm.p_free, par(i_g - 1)))) {
                    tc_fence_after();
                    uint32_t ak = lT[i_g & 1];
                    constexpr uint32_t r2 = 2 * (kSub * 128 >> 4), all = 0xffffffffu;
#pragma unroll 1
                    for (int j = 0; j < 8; j++) {
                        umma_lo_unit_e(tm + k3ColGP, ak, ak, idesc64, j, 0u, 0u, all, all);
                        umma_lo_unit_e(tm + k3ColGP, ak, ak + r2, idesc64, j, all, all, 0u, 0u);
                        ak += (j == 3) ? 2 + kBigJump : 2;
                    }
                    umma_commit_e(&sm.mma_g);
                    i_g++; k_ok = false; progress = true;
                }
            }
        }
        if (progress) {
            last = global_ns();
        } else if ((++idle & 7) != 0) {
            __nanosleep(200);
        } else if (__any_sync(0xffffffffu, *ab || global_ns() - last > kWaitLimitNs)) {
            code = 1 + (i_g > i_k) + 2 * (i_k > i_up);
            *ab = 1;
            break;
        }
    }
    if (code && elect_one()) {   // the lane that issued the UMMAs and the TMA loads
        atomicCAS(a.status, 0, 400 + code);
        umma_commit(&sm.drain);
        int never = 0;
        mbar_wait(&sm.drain, 0, &never);
        if (pend_k) mbar_wait(&sm.full_k, 0, &never), mbar_wait(&sm.full_k, 1, &never);
        if (pend_q) mbar_wait(&sm.full_q, 0, &never), mbar_wait(&sm.full_q, 1, &never);
    }
    __syncwarp();
}

// The explicit walk for this variant: G and P arrive one after the other in the same columns, so it reports
// G as read after phase A and waits for P before phase C.
__device__ __forceinline__ BlockOut robust_block3(Smem3& sm, uint32_t tcol, uint32_t ph, int J, int tl, cplx at, cplx vg,
                                                  float be, float nt, cplx kz, cplx kr) {
    volatile int* ab = &sm.abort_flag;
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
    cplx cc[32];   // run-time indexed on purpose: local memory (see robust_block)
    {
        cplx cur = {1.f, 0.f};
#pragma unroll 1
        for (int grp = 3; grp >= 0; grp--) {
            float g8[8];
            tmem_ld8(tcol + grp * 8, g8);
#pragma unroll
            for (int e = 7; e >= 0; e--) {
                const int i = grp * 8 + e;
                const float2 ai = __bfloat1622float2(sm.a[J * 32 + i]);
                const bool on = i < tl;
                const cplx fg = cmul(at, cur);
                cc[i] = {on ? fg.r * g8[e] : 0.f, on ? fg.i * g8[e] : 0.f};
                const cplx nx = cmul(cur, cplx{ai.x, ai.y});
                cur = {on ? nx.r : cur.r, on ? nx.i : cur.i};
            }
        }
    }
    tc_fence_before();
    __syncwarp();
    if (tl == 0) mbar_arrive(&sm.g_free);
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
    o.ok = warp_wait(&sm.mma_p, ph, ab);
    if (!o.ok) return o;
    tc_fence_after();
    cplx yin = {0.f, 0.f};
    float pd = 0.f;
    cplx cur = {1.f, 0.f};
#pragma unroll 1
    for (int grp = 3; grp >= 0; grp--) {
        float p8[8];
        tmem_ld8(tcol + grp * 8, p8);
#pragma unroll
        for (int e = 7; e >= 0; e--) {
            const int i = grp * 8 + e;
            const float2 ai = __bfloat1622float2(sm.a[J * 32 + i]);
            const cplx uw = cshfl(cw, i), ux = cshfl(cx, i);
            const bool on = i < tl;
            pd = (i == tl) ? p8[e] : pd;
            const cplx au = cmul(at, uw);
            const cplx ee = cmul(cur, cplx{au.r - ux.r, au.i - ux.i});
            const float pi = on ? p8[e] : 0.f;
            yin.r += pi * ee.r;
            yin.i += pi * ee.i;
            const cplx nx = cmul(cur, cplx{ai.x, ai.y});
            cur = {on ? nx.r : cur.r, on ? nx.i : cur.i};
        }
    }
    // W rho_z + W0 rho_r is added by the caller, which reads rho after this walk
    o.ysum = {pd * cw.r + yin.r, pd * cw.i + yin.i};
    o.pd = pd;
    // the caller needs W and W0 for that: hand them back in place of the unused fields
    o.W = W;
    o.W0 = W0;
    return o;
}

__device__ __forceinline__ void compute3(Smem3& sm, const Args& a) {
    using C = Cfg<true>;
    volatile int* ab = &sm.abort_flag;
    const int t = threadIdx.x, J = t >> 5, tl = t & 31;
    const int H = a.H, L = a.L;
    const uint32_t tlane = sm.tmem_base + ((uint32_t)(J * 32) << 16);
    const uint32_t tcol = tlane + k3ColGP + 32 * (J & 1);
    const int n_items = ((int)blockIdx.x < a.items) ? (a.items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int NS = n_items * kSteps;
    if (NS == 0) return;
    int code = 0;
    cplx Sz[4], Sr[4];
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    ItemPos cur = item_pos(a, blockIdx.x), nxi = cur;
    Tok tk;
    {
        const bool valid = cur.c * kC + tl < L;
        const uint4 first = valid ? __ldg(a.rec + rec_index(a, cur.b, cur.c, 0, cur.h0 + J, tl)) : zero4;
        tk = prepare(sm, first, 0, J, tl);
    }
    for (int g = 0; g < NS && !code; g++) {
        const uint32_t ph = g & 1;
        const int step = g & 3;
        if (step == 0) {
            if (g > 0) cur = nxi;
            nxi = item_pos(a, (int)blockIdx.x + ((g >> 2) + 1) * (int)gridDim.x);
        }
        const int l = cur.c * kC + step * kSub + tl, hd = cur.h0 + J;
        const bool valid = l < L;
        const size_t unit0 = ((size_t)cur.b * a.NC + cur.c) * H + cur.h0;   // workspace slot of head h0
        if (step == 0) {   // states at the chunk start, column d = t of every head
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float* s = a.ws_state + (unit0 + u) * 2 * kD;
                Sz[u] = {0.f, 0.f};
                Sr[u] = {s[t], s[kD + t]};
            }
        }
        // ---- publish the states for kappa / rho of this step (the omega columns of the previous step have
        // been consumed: this thread has seen its state update complete)
#pragma unroll
        for (int u = 0; u < 4; u++) {
            st_hi_lo(sm.so_tile, C::kSmallSlab, 8 * u + 0, t, Sz[u].r);
            st_hi_lo(sm.so_tile, C::kSmallSlab, 8 * u + 2, t, Sz[u].i);
            st_hi_lo(sm.so_tile, C::kSmallSlab, 8 * u + 4, t, Sr[u].r);
            st_hi_lo(sm.so_tile, C::kSmallSlab, 8 * u + 6, t, Sr[u].i);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (tl == 0) mbar_arrive(&sm.s_ready);
        TC4_STAMP(0);
        // ---- fetch the record of step g + 1 (the next item's first sub-block after this item's last)
        uint4 rec = zero4;
        if (g + 1 < NS) {
            const ItemPos& np = (step + 1 < kSteps) ? cur : nxi;
            const int nsub = (step + 1) & 3;
            if (np.c * kC + nsub * kSub + tl < L) rec = __ldg(a.rec + rec_index(a, np.b, np.c, nsub, np.h0 + J, tl));
        }
        const cplx at = tk.at, vg = tk.vg;
        const float be = tk.be;
        // ---- Gram row of the own head: |k_t|^-1 from its diagonal
        TC4_STAMP(2);
        if (!warp_wait(&sm.mma_g, ph, ab)) { code = 13; break; }
        tc_fence_after();
        TC4_STAMP(3);
        float gs[32], p[32];
        float pd = 0.f, mt = 0.f;
        tmem_ld32(tcol, gs);
        if (tk.fast) {   // G is in registers: P may take its columns (the explicit walk reads G again itself)
            tc_fence_before();
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.g_free);
        }
        float gd = 0.f;
#pragma unroll
        for (int i = 0; i < 32; i++) gd = (i == tl) ? gs[i] : gd;
        const float nt = rsqrtf(gd + kEps);
        const float bnn = be * nt * nt;
        // ---- kappa_t = k_t . z0 | r0 (raw rows; hi + lo parts summed)
        if (!warp_wait(&sm.mma_k, ph, ab)) { code = 12; break; }
        tc_fence_after();
        TC4_STAMP(4);
        float k8[8];
        tmem_ld8(tlane + k3ColKU + 8 * J, k8);
        const cplx kz = {k8[0] + k8[1], k8[2] + k8[3]}, kr = {k8[4] + k8[5], k8[6] + k8[7]};
        BlockOut o;
        cplx yW = {0.f, 0.f}, yW0 = {0.f, 0.f};   // factors of rho_z and rho_r in the read-out
        if (tk.fast) {
#pragma unroll
            for (int i = 0; i < 32; i++) gs[i] = (i < tl) ? -bnn * gs[i] : 0.f;
            const cplx rkz = cmul(tk.R, kz), rkr = cmul(tk.R, kr);
            cplx cw = {nt * be * (tk.viw.r - nt * rkz.r), nt * be * (tk.viw.i - nt * rkz.i)};
            cplx cx = {nt * be * nt * rkr.r, nt * be * nt * rkr.i};
            // ---- |q_t|^-1 from the Q tile row (swizzled 16-byte pieces); the Q tile lands late in this variant
            TC4_STAMP(9);
            if (!warp_wait(&sm.full_q, ph, ab)) { code = 11; break; }
            TC4_STAMP(10);
            {
                const uint8_t* qt = sm.tile[(g + 1) & 1];
                float qq = 0.f, qq2 = 0.f;
#pragma unroll 2
                for (int c16 = 0; c16 < 16; c16++) {
                    const uint4 r = *reinterpret_cast<const uint4*>(qt + (c16 >> 3) * kSlab + t * 128 + (((c16 & 7) ^ (t & 7)) << 4));
                    float f[8];
                    unpack8(r, f);
#pragma unroll
                    for (int e = 0; e < 4; e++) { qq = fmaf(f[e], f[e], qq); qq2 = fmaf(f[4 + e], f[4 + e], qq2); }
                }
                mt = rsqrtf(qq + qq2 + kEps);
            }
            TC4_STAMP(12);
            if (!warp_wait(&sm.mma_p, ph, ab)) { code = 16; break; }
            tc_fence_after();
            TC4_STAMP(13);
            tmem_ld32(tcol, p);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                pd = (i == tl) ? p[i] : pd;
                p[i] = (i < tl) ? p[i] : 0.f;
            }
            tc_fence_before();
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.p_free);   // P is in registers, |q| has been taken from the Q tile
            cplx accu = {0.f, 0.f}, accx = {0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const cplx uw = cshfl(cw, i), ux = cshfl(cx, i);
                cw.r = fmaf(gs[i], uw.r, cw.r);
                cw.i = fmaf(gs[i], uw.i, cw.i);
                cx.r = fmaf(gs[i], ux.r, cx.r);
                cx.i = fmaf(gs[i], ux.i, cx.i);
                accu.r = fmaf(p[i], uw.r, accu.r);
                accu.i = fmaf(p[i], uw.i, accu.i);
                accx.r = fmaf(p[i], ux.r, accx.r);
                accx.i = fmaf(p[i], ux.i, accx.i);
            }
            o.wh = cmul(tk.D31, cw);
            const cplx xv = cmul(tk.D31, cx);
            o.xh = {-xv.r, -xv.i};
            // y = D (R rho_z + pd u^ + accu) + D0 (R rho_r - accx); lane 0: W0 = 1, the carried correction itself
            const cplx yl = cmul(tk.D, cplx{pd * cw.r + accu.r, pd * cw.i + accu.i});
            cplx yc = cmul(tk.D0, cplx{-accx.r, -accx.i});
            if (tl == 0) yc = {0.f, 0.f};
            o.ysum = {yl.r + yc.r, yl.i + yc.i};
            yW = cmul(tk.D, tk.R);
            yW0 = cmul(tk.D0, tk.R);
            if (tl == 0) yW0 = {1.f, 0.f};
        } else {
            if (!warp_wait(&sm.full_q, ph, ab)) { code = 11; break; }
            {
                const uint8_t* qt = sm.tile[(g + 1) & 1];
                float qq = 0.f;
#pragma unroll 1
                for (int c16 = 0; c16 < 16; c16++) {
                    const uint4 r = *reinterpret_cast<const uint4*>(qt + (c16 >> 3) * kSlab + t * 128 + (((c16 & 7) ^ (t & 7)) << 4));
                    float f[8];
                    unpack8(r, f);
#pragma unroll
                    for (int e = 0; e < 8; e++) qq = fmaf(f[e], f[e], qq);
                }
                mt = rsqrtf(qq + kEps);
            }
            o = robust_block3(sm, tcol, ph, J, tl, at, vg, be, nt, kz, kr);
            if (!o.ok) { code = 17; break; }
            pd = o.pd;
            yW = o.W;
            yW0 = o.W0;
            tc_fence_before();
            __syncwarp();
            if (tl == 0) mbar_arrive(&sm.p_free);
        }
        // ---- rho_t = q_t . z0 | r0; once it has completed, nothing reads the published states any more and
        // the tile can take the omega columns
        TC4_STAMP(5);
        if (!warp_wait(&sm.mma_r, ph, ab)) { code = 18; break; }
        tc_fence_after();
        float r8[8];
        tmem_ld8(tlane + k3ColRho + 8 * J, r8);
        tc_fence_before();
        __syncwarp();
        if (tl == 0) mbar_arrive(&sm.r_free);
        // ---- omega column of this token: the head's eight values, zeros in the other heads' rows
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const bool mine = u == J;
            st_hi_lo(sm.so_tile, C::kSmallSlab, 8 * u + 0, t, mine ? o.wh.r : 0.f);
            st_hi_lo(sm.so_tile, C::kSmallSlab, 8 * u + 2, t, mine ? o.wh.i : 0.f);
            st_hi_lo(sm.so_tile, C::kSmallSlab, 8 * u + 4, t, mine ? o.xh.r : 0.f);
            st_hi_lo(sm.so_tile, C::kSmallSlab, 8 * u + 6, t, mine ? o.xh.i : 0.f);
        }
        fence_proxy_async();
        __syncwarp();
        if (tl == 0) mbar_arrive(&sm.omega_ready);
        {
            const cplx rz = cmul(yW, cplx{r8[0] + r8[1], r8[2] + r8[3]});
            const cplx rr = cmul(yW0, cplx{r8[4] + r8[5], r8[6] + r8[7]});
            float yr = mt * (o.ysum.r + rz.r + rr.r), yi = mt * (o.ysum.i + rz.i + rr.i);
            if (a.shortcut_scale != 0.f) {   // block.py:202-208
                const float qk = mt * nt * pd;
                yr += a.shortcut_scale * qk * qk * vg.r;
                yi += a.shortcut_scale * qk * qk * vg.i;
            }
            if (valid) {
                __nv_bfloat162 ov = __floats2bfloat162_rn(bfr(yr) * tk.sc, bfr(yi) * tk.sc);
                *reinterpret_cast<__nv_bfloat162*>(a.y + (((size_t)cur.b * L + l) * H + hd) * 2) = ov;
            }
        }
        // ---- the next step's token while the state-update UMMA runs (this step's block products are waited for
        // first: prepare() arrives on the same barrier for the next step)
        TC4_STAMP(1);
        if (!warp_wait(&sm.bp_ready, ph, ab)) { code = 14; break; }
        if (g + 1 < NS) tk = prepare(sm, rec, g + 1, J, tl);
        // ---- state hand-off: S <- W_31 S + K^T omega, column d = t of every head
        TC4_STAMP(8);
        if (!warp_wait(&sm.mma_up, ph, ab)) { code = 15; break; }
        tc_fence_after();
        TC4_STAMP(6);
        if (step + 1 < kSteps) {
            float up[32];
            tmem_ld32(tlane + k3ColKU, up);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const cplx bpu = {sm.bp[ph][u].x, sm.bp[ph][u].y};
                const cplx nz = cmul(bpu, Sz[u]), nr = cmul(bpu, Sr[u]);
                Sz[u] = {nz.r + up[8 * u] + up[8 * u + 1], nz.i + up[8 * u + 2] + up[8 * u + 3]};
                Sr[u] = {nr.r + up[8 * u + 4] + up[8 * u + 5], nr.i + up[8 * u + 6] + up[8 * u + 7]};
            }
        }
        tc_fence_before();
        TC4_STAMP(7);
    }
    if (code && tl == 0) atomicCAS(a.status, 0, 500 + code);
}

__global__ void __launch_bounds__(kThreads, 3)
scan_tc4_out3_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ, const Args a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    Smem3& sm = *reinterpret_cast<Smem3*>(smem_raw);
    const int warp = threadIdx.x >> 5;
    if ((smem_u32(smem_raw) & 1023u) != 0) {   // the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicCAS(a.status, 0, 399);
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(&sm.full_k, 1); mbar_init(&sm.full_q, 1);
        mbar_init(&sm.mma_g, 1); mbar_init(&sm.mma_p, 1); mbar_init(&sm.mma_k, 1); mbar_init(&sm.mma_r, 1);
        mbar_init(&sm.mma_up, 1);
        mbar_init(&sm.g_free, 4); mbar_init(&sm.p_free, 4); mbar_init(&sm.r_free, 4);
        mbar_init(&sm.s_ready, 4); mbar_init(&sm.omega_ready, 4); mbar_init(&sm.bp_ready, 4);
        mbar_init(&sm.drain, 1);
        sm.abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 4) tmem_alloc(&sm.tmem_base, k3TmemCols);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp < 4) {
        compute3(sm, a);
    } else {
        if (threadIdx.x == 128) {
            prefetch_tmap(&tmK);
            prefetch_tmap(&tmQ);
        }
        __syncwarp();
        producer3(sm, &tmK, &tmQ, a);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        tmem_dealloc(sm.tmem_base, k3TmemCols);
    }
}

template <bool kOutput>
__global__ void __launch_bounds__(kThreads, Cfg<kOutput>::kBlocksPerSm)
scan_tc4_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ, const Args a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    Smem<kOutput>& sm = *reinterpret_cast<Smem<kOutput>*>(smem_raw);
    const int warp = threadIdx.x >> 5;
    if ((smem_u32(smem_raw) & 1023u) != 0) {   // the swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicCAS(a.status, 0, 399);
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(&sm.full_k[0], 1); mbar_init(&sm.full_k[1], 1); mbar_init(&sm.full_q, 1);
        mbar_init(&sm.mma_g, 1); mbar_init(&sm.mma_p, 1); mbar_init(&sm.mma_kr, 1); mbar_init(&sm.mma_up, 1);
        mbar_init(&sm.g_free, 4); mbar_init(&sm.p_free, 4); mbar_init(&sm.s_ready, 4); mbar_init(&sm.omega_ready, 4);
        mbar_init(&sm.bp_ready, 4);
        mbar_init(&sm.drain, 1);
        sm.abort_flag = 0;
        fence_barrier_init();
    }
    // rows of the two small operand tiles that a pass does not write stay zero for the whole kernel
    for (int i = threadIdx.x; i < 2 * (int)Cfg<kOutput>::kSmallTile / 16; i += kThreads)
        reinterpret_cast<uint4*>(sm.s_tile)[i] = make_uint4(0, 0, 0, 0);   // s_tile and o_tile are adjacent
    if (warp == 4) tmem_alloc(&sm.tmem_base, Cfg<kOutput>::kTmemCols);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp < 4) {
        compute<kOutput>(sm, a);
    } else {
        if (threadIdx.x == 128) {
            prefetch_tmap(&tmK);
            if (kOutput) prefetch_tmap(&tmQ);
        }
        __syncwarp();
        producer<kOutput>(sm, &tmK, &tmQ, a);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        tmem_dealloc(sm.tmem_base, Cfg<kOutput>::kTmemCols);
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
    int B, L, H, NC, pos0, segs;
};
__global__ void __launch_bounds__(256) tc4_dynamics_kernel(const DynArgs a) {
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
    const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(a.v + ((size_t)bl * H + hd) * 2);
    uint4 r;
    r.x = pack2(ar, ai);
    r.y = pack2(__low2float(v2) * vp, __high2float(v2) * vp);
    r.z = pack2(ds.beta, ds.sel_c);
    r.w = 0u;
    const int c = l / kC, sub = (l % kC) / kSub, tl = l % kSub;
    a.rec[((((size_t)b * a.NC + c) * kSteps + sub) * H + hd) * kSub + tl] = r;
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

size_t scan_tc4_record_bytes(int B, int L, int H) {
    const size_t NC = ((size_t)L + tc4::kC - 1) / tc4::kC;
    return (size_t)B * NC * tc4::kC * H * sizeof(uint4);
}

// Dynamics pre-pass: fills rec (scan_tc4_record_bytes bytes) for both scan passes.
int scan_tc4_dynamics(const void* v, const void* gate_raw, const float* log_dt_scale, const float* rope_freqs,
                      void* rec, const DynConsts& dc, int B, int L, int H, int pos0, int segs, cudaStream_t st) {
    tc4::DynArgs d;
    d.v = static_cast<const __nv_bfloat16*>(v);
    d.gate_raw = static_cast<const __nv_bfloat16*>(gate_raw);
    d.log_dt_scale = log_dt_scale; d.rope_freqs = rope_freqs;
    d.rec = static_cast<uint4*>(rec);
    d.dc = dc;
    d.B = B; d.L = L; d.H = H; d.NC = (L + tc4::kC - 1) / tc4::kC; d.pos0 = pos0; d.segs = segs;
    const long long total = (long long)B * L * H;
    tc4::tc4_dynamics_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(d);
    return check_launch();
}

// One pass of the four-chain tensor-core scan over every chunk.  output = false: local pass (fills
// ws_state / ws_gamma for the carry pass); output = true: reads the carries from ws_state, writes y
// (two_blocks: the variant with three tile buffers and two blocks per SM).
// status: one int in device memory, set by a bounded wait that ran out (not cleared here).
int scan_tc4_pass(bool output, bool two_blocks, const void* q, const void* k, const void* rec, float* ws_gamma,
                  float* ws_state, void* y, int* status, float shortcut_scale, int B, int L, int H, cudaStream_t st) {
    using namespace tc4;
    CUtensorMap tmK, tmQ;
    if (!make_tile_map(&tmK, k, B, L, H) || !make_tile_map(&tmQ, output ? q : k, B, L, H)) return CDSSM_ERR_CUDA;
    const size_t smem = output ? sizeof(Smem<true>) : sizeof(Smem<false>);
    // the opt-in to more than 48 KB of dynamic shared memory and the SM count are per device
    constexpr int kMaxDevices = 64;
    static int sms_of_device[kMaxDevices] = {0};
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev))) return rc;
    if (dev < 0 || dev >= kMaxDevices) return CDSSM_ERR_UNSUPPORTED;
    if (sms_of_device[dev] == 0) {
        if (int rc = check_cuda(cudaFuncSetAttribute(scan_tc4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     (int)sizeof(Smem<true>))))
            return rc;
        if (int rc = check_cuda(cudaFuncSetAttribute(scan_tc4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     (int)sizeof(Smem<false>))))
            return rc;
        if (int rc = check_cuda(cudaFuncSetAttribute(scan_tc4_out3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     (int)sizeof(Smem3))))
            return rc;
        int n = 0;
        if (int rc = check_cuda(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev))) return rc;
        sms_of_device[dev] = n;
    }
    const int sms = sms_of_device[dev];
    Args a;
    a.rec = static_cast<const uint4*>(rec);
    a.ws_gamma = ws_gamma; a.ws_state = ws_state;
    a.y = static_cast<__nv_bfloat16*>(y);
    a.status = status; a.trace = g_trace;
    a.trace_g0 = 0; a.trace_block = 0;
    if (g_trace) {   // performance debugging only: which 16 steps of which block are stamped
        if (const char* e = getenv("CDSSM_TC4_TRACE_G0")) a.trace_g0 = atoi(e);
        if (const char* e = getenv("CDSSM_TC4_TRACE_BLOCK")) a.trace_block = atoi(e);
    }
    a.shortcut_scale = shortcut_scale;
    a.B = B; a.L = L; a.H = H; a.NC = (L + kC - 1) / kC;
    a.HG = H / 4;
    const long long items = (long long)B * a.NC * a.HG;
    if (items > 0x7fffffff / 8) return CDSSM_ERR_UNSUPPORTED;
    a.items = (int)items;
    const bool three = output && !two_blocks;   // the output pass on two tile buffers, three blocks per SM
    const long long resident = (long long)(!output ? Cfg<false>::kBlocksPerSm : three ? 3 : Cfg<true>::kBlocksPerSm) * sms;
    const int grid = (int)(items < resident ? items : resident);
    if (three) scan_tc4_out3_kernel<<<grid, kThreads, sizeof(Smem3), st>>>(tmK, tmQ, a);
    else if (output) scan_tc4_kernel<true><<<grid, kThreads, smem, st>>>(tmK, tmQ, a);
    else scan_tc4_kernel<false><<<grid, kThreads, smem, st>>>(tmK, tmQ, a);
    return check_launch();
}

}  // namespace cdssm
