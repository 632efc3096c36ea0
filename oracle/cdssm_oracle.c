/*
 * CPU restatement of the CD-SSM scan path.  TEST INFRASTRUCTURE ONLY: it is the checker
 * for the CUDA kernels (tests/, the smoke check) and the timed CPU baseline of the bench.
 * The product library never links, imports or calls anything in this file.
 *
 * Every function restates, in plain fp32 C, the arithmetic of one reference CUDA kernel
 * or one piece of reference Python glue; the reference location is cited per function.
 * The reference has no CPU path and no tests (cdssm/ops.py:10 imports the CUDA extension
 * only), so this restatement is pinned against the reference kernels themselves, compiled
 * unmodified for sm_100 and run on a B200 (tests/golden/ holds their outputs).
 *
 * Tensors are float32 arrays in the reference's layouts.  round_bf16 is a bit mask that says
 * which of the reference's bfloat16 stores are emulated (round-to-nearest-even at the same
 * point):
 *   1  scan inputs: dynamics outputs, normalised k/q, the vp-scaled v
 *   2  per-token state stores: local_h, cum_A, corrections, Y = local_h + correction, shortcut
 *   4  per-chunk carry: cum_A and local_h of the last step of a chunk, chunk_states
 *   8  outputs: the read-out and its sel_C product
 *  16  modifier (not a reference behaviour): A_bar is NOT rounded although bit 1 is set - the transition stays
 *      float32 between the dynamics and the scan.  The reference's bfloat16 A_bar puts |a| above 1 by rounding
 *      for slowly rotating heads, and its carry (inter_chunk_scan.cu:73-83: decay only, no erasure) then grows
 *      without bound over some 1e5 tokens; this bit states the same algorithm without that growth.
 * 15 is the reference as it runs (everything bfloat16 between kernels); 0 is the fp32
 * statement of the same algorithm; 13 is "bfloat16 inputs and outputs, fp32 state".
 * Transcendentals use libm, the reference uses --use_fast_math intrinsics: results agree to
 * a few fp32 ulp, not bit for bit.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_MAX_N 32      /* common.cuh:34 */
#define ORC_MAX_D 128     /* common.cuh:35 */
#define ORC_EPS 1e-6f     /* common.cuh:142 */

static inline float bf16r(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    u &= 0xffff0000u;
    memcpy(&x, &u, 4);
    return x;
}
static inline float rnd(float x, int on) { return on ? bf16r(x) : x; }
#define R_IN 1
#define R_STATE 2
#define R_CARRY 4
#define R_OUT 8
#define R_KEEP_A 16

float orc_bf16_round(float x) { return bf16r(x); }

/* common.cuh:82-91 */
static inline float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
static inline float softplusf_(float x) { return x > 20.0f ? x : logf(1.0f + expf(x)); }
static inline float siluf_(float x) { return x / (1.0f + expf(-x)); }

/* ------------------------------------------------------------------------------------
 * Fused dynamics.  dynamics_fused.cu:50-139, cayley_math.cuh:51-99.
 * gate_raw (B,L,(N+5)*H): segments alpha_0.., omega_0.., sel_B, sel_C, sel_dt, beta, r_gate,
 * each H wide.  Outputs A_bar (B,L,H,N), vp (B,L,H,N/2), beta (B,L,H), sel_C (B,L,H).
 * pos0 is added to the position l (the reference always has pos0 = 0).
 * ---------------------------------------------------------------------------------- */
void orc_dynamics(const float* gate_raw, const float* log_dt_scale, const float* rope_freqs,
                  float gating_c, float omega_thresh, float adt_delta, float adt_smoothness,
                  float adt_eps, int B, int L, int H, int N, int pos0, int round_bf16,
                  float* A_bar, float* vp_scale, float* beta_out, float* selC_out) {
    const int NH = N / 2, G = N + 5;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int l = 0; l < L; l++) {
            const float* g = gate_raw + ((size_t)b * L + l) * (size_t)(G * H);
            for (int h = 0; h < H; h++) {
                const float* sc = g + N * H;
                float sel_B = sc[0 * H + h], sel_C = sc[1 * H + h], sel_dt = sc[2 * H + h];
                float beta_raw = sc[3 * H + h], r_raw = sc[4 * H + h];
                float r_gate = sigmoidf_(r_raw);
                float freq = rope_freqs[h];
                float pos = (float)(l + pos0);
                float alpha0 = softplusf_(g[0 * H + h]);
                float omega0 = g[NH * H + h] + pos * freq;
                float dt_scale = softplusf_(log_dt_scale[h]);
                float w0 = fabsf(omega0);
                float dt_raw = dt_scale / (alpha0 + w0 + adt_eps);
                float dt_max = (2.0f - adt_delta) / (alpha0 + adt_eps);
                float blend = sigmoidf_((omega_thresh - w0) / adt_smoothness);
                float dt_cap = fminf(dt_raw, dt_max);
                float dt = blend * dt_cap + (1.0f - blend) * dt_raw + softplusf_(sel_dt);
                size_t blh = ((size_t)b * L + l) * H + h;
                for (int j = 0; j < NH; j++) {
                    float alpha = fmaxf(softplusf_(g[j * H + h]), 0.0f);
                    float omega = g[(NH + j) * H + h] + pos * freq;
                    float tau = dt * 0.5f, ta = tau * alpha, tw = tau * omega;
                    float nr = 1.0f - ta, ni = tw, dr = 1.0f + ta, di = -tw;
                    float denom = fmaf(dr, dr, di * di) + ORC_EPS;
                    float inv_d = 1.0f / denom;
                    float mu_re = (nr * dr + ni * di) * inv_d;
                    float mu_im = (ni * dr - nr * di) * inv_d;
                    float numer = fmaf(1.0f - ta, 1.0f - ta, tw * tw);
                    float den2 = fmaf(1.0f + ta, 1.0f + ta, tw * tw);
                    float eig = fmaxf(numer / (den2 + ORC_EPS), 1e-8f);
                    float scale = powf(eig, (gating_c * r_gate - 1.0f) / 2.0f);
                    A_bar[blh * N + 2 * j] = rnd(mu_re * scale, (round_bf16 & R_IN) && !(round_bf16 & R_KEEP_A));
                    A_bar[blh * N + 2 * j + 1] = rnd(-mu_im * scale, (round_bf16 & R_IN) && !(round_bf16 & R_KEEP_A));
                    float eff = powf(eig, gating_c * r_gate);
                    float vp = fminf(sqrtf(fmaxf(1.0f - eff, ORC_EPS)), 1.0f);
                    vp_scale[blh * NH + j] = rnd(vp, round_bf16 & R_IN);
                }
                beta_out[blh] = rnd(sigmoidf_(beta_raw) * sigmoidf_(sel_B), round_bf16 & R_IN);
                selC_out[blh] = rnd(sigmoidf_(sel_C), round_bf16 & R_IN);
            }
        }
}

/* L2 normalisation of K and Q rows.  normalize_kq.cu:46-79 (x * rsqrt(sum x^2 + 1e-6)). */
void orc_normalize_kq(const float* K, const float* Q, size_t rows, int D, int round_bf16,
                      float* K_out, float* Q_out) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++) {
        const float* k = K + r * D;
        const float* q = Q + r * D;
        float sk = 0.f, sq = 0.f;
        for (int d = 0; d < D; d++) { sk += k[d] * k[d]; sq += q[d] * q[d]; }
        float ik = 1.0f / sqrtf(sk + ORC_EPS), iq = 1.0f / sqrtf(sq + ORC_EPS);
        for (int d = 0; d < D; d++) {
            K_out[r * D + d] = rnd(k[d] * ik, round_bf16 & R_IN);
            Q_out[r * D + d] = rnd(q[d] * iq, round_bf16 & R_IN);
        }
    }
}

/* One delta-rule step on the (N,D) state.  intra_chunk_scan.cu:117-167:
 * u = h k ; h -= beta u k^T ; rotate row pairs by (re,im) ; (optionally) h += beta v k^T. */
static inline void step_state(float* h, const float* a, const float* k, const float* v,
                              float beta, int N, int D, int inject) {
    float u[ORC_MAX_N];
    for (int s = 0; s < N; s++) {
        float acc = 0.f;
        for (int d = 0; d < D; d++) acc += h[s * D + d] * k[d];
        u[s] = acc;
    }
    for (int s = 0; s < N; s++)
        for (int d = 0; d < D; d++) h[s * D + d] -= beta * u[s] * k[d];
    for (int j = 0; j < N / 2; j++) {
        float re = a[2 * j], im = a[2 * j + 1];
        float* hr = h + (2 * j) * D;
        float* hi = h + (2 * j + 1) * D;
        for (int d = 0; d < D; d++) {
            float x = hr[d], y = hi[d];
            hr[d] = re * x - im * y;
            hi[d] = re * y + im * x;
        }
    }
    if (inject)
        for (int s = 0; s < N; s++)
            for (int d = 0; d < D; d++) h[s * D + d] += beta * v[s] * k[d];
}

/* Intra-chunk scan from a zero state.  intra_chunk_scan.cu:86-195.
 * A (BNC,C,H,N), K (BNC,C,H,D), V (BNC,C,H,N), beta (BNC,C,H)
 * -> local_h (BNC,C,H,N,D), cum_A (BNC,C,H,N). */
void orc_intra_chunk(const float* A, const float* K, const float* V, const float* beta,
                     int BNC, int C, int H, int D, int N, int round_bf16,
                     float* local_h, float* cum_A) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int c = 0; c < BNC; c++)
        for (int hd = 0; hd < H; hd++) {
            float h[ORC_MAX_N * ORC_MAX_D];
            float cA[ORC_MAX_N];
            memset(h, 0, sizeof(float) * N * D);
            for (int s = 0; s < N; s += 2) { cA[s] = 1.f; cA[s + 1] = 0.f; }
            for (int t = 0; t < C; t++) {
                size_t row = ((size_t)c * C + t) * H + hd;
                const float* a = A + row * N;
                step_state(h, a, K + row * D, V + row * N, beta[row], N, D, 1);
                const int ron = (round_bf16 & R_STATE) || ((round_bf16 & R_CARRY) && t == C - 1);
                float* out = local_h + row * (size_t)N * D;
                for (int i = 0; i < N * D; i++) out[i] = rnd(h[i], ron);
                for (int j = 0; j < N / 2; j++) {
                    float ar = a[2 * j], ai = a[2 * j + 1], cr = cA[2 * j], ci = cA[2 * j + 1];
                    cA[2 * j] = ar * cr - ai * ci;
                    cA[2 * j + 1] = ar * ci + ai * cr;
                }
                for (int s = 0; s < N; s++) cum_A[row * N + s] = rnd(cA[s], ron);
            }
        }
}

/* Inter-chunk carry: emit s, then s = total_A (*) s + final_local_h (complex diagonal, no
 * erasure).  inter_chunk_scan.cu:48-84.  total_A (B,NC,H,N), flh/out (B,NC,H,N,D).
 * s0 (B,H,N,D) may be NULL (the reference always starts from zero); s_final (B,H,N,D) may be
 * NULL (the reference discards the carry after the last chunk). */
void orc_inter_chunk(const float* total_A, const float* flh, const float* s0, int B, int NC,
                     int H, int D, int N, int round_bf16, float* chunk_states, float* s_final) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int hd = 0; hd < H; hd++) {
            float s[ORC_MAX_N * ORC_MAX_D];
            if (s0) memcpy(s, s0 + ((size_t)b * H + hd) * N * D, sizeof(float) * N * D);
            else memset(s, 0, sizeof(float) * N * D);
            for (int k = 0; k < NC; k++) {
                size_t idx = ((size_t)b * NC + k) * H + hd;
                float* out = chunk_states + idx * (size_t)N * D;
                for (int i = 0; i < N * D; i++) out[i] = rnd(s[i], round_bf16 & R_CARRY);
                const float* a = total_A + idx * N;
                const float* f = flh + idx * (size_t)N * D;
                for (int j = 0; j < N / 2; j++) {
                    float re = a[2 * j], im = a[2 * j + 1];
                    for (int d = 0; d < D; d++) {
                        float sr = s[(2 * j) * D + d], si = s[(2 * j + 1) * D + d];
                        s[(2 * j) * D + d] = re * sr - im * si + f[(2 * j) * D + d];
                        s[(2 * j + 1) * D + d] = re * si + im * sr + f[(2 * j + 1) * D + d];
                    }
                }
            }
            if (s_final) memcpy(s_final + ((size_t)b * H + hd) * N * D, s, sizeof(float) * N * D);
        }
}

/* Correction pass: h = chunk_state; for t: store h, then erase + rotate (no injection).
 * exact_correction.cu:83-150.  A (B,NC,C,H,N), K (B,NC,C,H,D), beta (B,NC,C,H),
 * chunk_states (B,NC,H,N,D) -> corrections (B,NC,C,H,N,D). */
void orc_exact_correction(const float* A, const float* K, const float* beta,
                          const float* chunk_states, int B, int NC, int C, int H, int D, int N,
                          int round_bf16, float* corrections) {
    const int BNC = B * NC;
#pragma omp parallel for collapse(2) schedule(static)
    for (int c = 0; c < BNC; c++)
        for (int hd = 0; hd < H; hd++) {
            float h[ORC_MAX_N * ORC_MAX_D];
            memcpy(h, chunk_states + ((size_t)c * H + hd) * N * D, sizeof(float) * N * D);
            for (int t = 0; t < C; t++) {
                size_t row = ((size_t)c * C + t) * H + hd;
                float* out = corrections + row * (size_t)N * D;
                for (int i = 0; i < N * D; i++) out[i] = rnd(h[i], round_bf16 & R_STATE);
                step_state(h, A + row * N, K + row * D, NULL, beta[row], N, D, 0);
            }
        }
}

/* Causal depthwise 4-tap conv + bias + SiLU.  conv1d_silu.cu:48-89.
 * x,out (B,L,Dm); weight (Dm,4); bias (Dm). */
void orc_conv1d_silu(const float* x, const float* w, const float* bias, int B, int L, int Dm,
                     int round_bf16, float* out) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int l = 0; l < L; l++)
            for (int d = 0; d < Dm; d++) {
                const float* xb = x + (size_t)b * L * Dm + d;
                float x0 = l >= 3 ? xb[(size_t)(l - 3) * Dm] : 0.f;
                float x1 = l >= 2 ? xb[(size_t)(l - 2) * Dm] : 0.f;
                float x2 = l >= 1 ? xb[(size_t)(l - 1) * Dm] : 0.f;
                float x3 = xb[(size_t)l * Dm];
                float y = w[d * 4 + 0] * x0 + w[d * 4 + 1] * x1 + w[d * 4 + 2] * x2 +
                          w[d * 4 + 3] * x3 + bias[d];
                out[((size_t)b * L + l) * Dm + d] = rnd(siluf_(y), round_bf16 != 0);
            }
}

/* ------------------------------------------------------------------------------------
 * The whole path as the reference block runs it, materialising every intermediate:
 *   dynamics (block.py:181-186) -> normalise (block.py:189-190) -> vp scale (block.py:194-195)
 *   -> pad/chunk (ssd.py:56-80) -> intra (ssd.py:83) -> inter (ssd.py:90-94)
 *   -> correction (ssd.py:98-100) -> Y = local_h + correction (ssd.py:102)
 *   -> shortcut (block.py:202-205) -> read-out einsum (block.py:208) -> sel_C gate (block.py:211).
 * q,k (B,L,H,D) un-normalised; v (B,L,H,N) before the vp scale; y (B,L,H,N).
 * h0 (B,H,N,D) or NULL is the carry into the first chunk; final_state (B,H,N,D) or NULL gets
 * the carry after the last chunk (both are extensions: the reference starts from zero and
 * discards the last carry, inter_chunk_scan.cu:48-84).
 * Returns 0, or -1 on allocation failure / bad sizes.
 * ---------------------------------------------------------------------------------- */
int orc_scan_reference(const float* q, const float* k, const float* v, const float* gate_raw,
                       const float* log_dt_scale, const float* rope_freqs, float gating_c,
                       float omega_thresh, float adt_delta, float adt_smoothness, float adt_eps,
                       float shortcut_scale, const float* h0, int B, int L, int H, int D, int N,
                       int C, int pos0, int round_bf16, float* y, float* final_state) {
    if (N > ORC_MAX_N || D > ORC_MAX_D || (N & 1) || C < 1) return -1;
    const int NH = N / 2;
    const int NC = (L + C - 1) / C, Lp = NC * C;
    const size_t T = (size_t)B * L * H, Tp = (size_t)B * Lp * H;
    float* A = malloc(sizeof(float) * T * N);
    float* vp = malloc(sizeof(float) * T * NH);
    float* be = malloc(sizeof(float) * T);
    float* sc = malloc(sizeof(float) * T);
    float* kn = malloc(sizeof(float) * T * D);
    float* qn = malloc(sizeof(float) * T * D);
    float* Ap = calloc(Tp * N, sizeof(float));
    float* Kp = calloc(Tp * D, sizeof(float));
    float* Vp = calloc(Tp * N, sizeof(float));
    float* bp = calloc(Tp, sizeof(float));
    float* lh = malloc(sizeof(float) * Tp * N * D);
    float* cA = malloc(sizeof(float) * Tp * N);
    float* co = malloc(sizeof(float) * Tp * N * D);
    float* tA = malloc(sizeof(float) * (size_t)B * NC * H * N);
    float* fl = malloc(sizeof(float) * (size_t)B * NC * H * N * D);
    float* cs = malloc(sizeof(float) * (size_t)B * NC * H * N * D);
    int rc = -1;
    if (!A || !vp || !be || !sc || !kn || !qn || !Ap || !Kp || !Vp || !bp || !lh || !cA || !co ||
        !tA || !fl || !cs)
        goto done;
    orc_dynamics(gate_raw, log_dt_scale, rope_freqs, gating_c, omega_thresh, adt_delta,
                 adt_smoothness, adt_eps, B, L, H, N, pos0, round_bf16, A, vp, be, sc);
    orc_normalize_kq(k, q, T, D, round_bf16, kn, qn);
    /* pad to a multiple of C with zeros (ssd.py:60-67); V_gated = V * repeat(vp, 2) */
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int l = 0; l < L; l++) {
            size_t src = ((size_t)b * L + l) * H, dst = ((size_t)b * Lp + l) * H;
            memcpy(Ap + dst * N, A + src * N, sizeof(float) * H * N);
            memcpy(Kp + dst * D, kn + src * D, sizeof(float) * H * D);
            memcpy(bp + dst, be + src, sizeof(float) * H);
            for (int h = 0; h < H; h++)
                for (int s = 0; s < N; s++)
                    Vp[(dst + h) * N + s] = rnd(v[(src + h) * N + s] * vp[(src + h) * NH + s / 2], round_bf16 & R_IN);
        }
    orc_intra_chunk(Ap, Kp, Vp, bp, B * NC, C, H, D, N, round_bf16, lh, cA);
    /* total_A = cum_A[:, :, -1], final_local_h = local_h[:, :, -1]  (ssd.py:90-91) */
    for (int c = 0; c < B * NC; c++)
        for (int h = 0; h < H; h++) {
            size_t row = ((size_t)c * C + (C - 1)) * H + h, idx = (size_t)c * H + h;
            memcpy(tA + idx * N, cA + row * N, sizeof(float) * N);
            memcpy(fl + idx * N * D, lh + row * (size_t)N * D, sizeof(float) * N * D);
        }
    orc_inter_chunk(tA, fl, h0, B, NC, H, D, N, round_bf16, cs, final_state);
    orc_exact_correction(Ap, Kp, bp, cs, B, NC, C, H, D, N, round_bf16, co);
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int l = 0; l < L; l++)
            for (int h = 0; h < H; h++) {
                size_t src = ((size_t)b * L + l) * H + h, row = ((size_t)b * Lp + l) * H + h;
                const float* kk = kn + src * D;
                const float* qq = qn + src * D;
                float qk = 0.f;
                for (int d = 0; d < D; d++) qk += qq[d] * kk[d];
                const int rs = round_bf16 & R_STATE;
                qk = rnd(qk, rs);
                for (int s = 0; s < N; s++) {
                    const float* l_ = lh + (row * N + s) * D;
                    const float* c_ = co + (row * N + s) * D;
                    float vg = Vp[row * N + s];
                    float t1 = rnd(qk * vg, rs);
                    float acc = 0.f;
                    for (int d = 0; d < D; d++) {
                        float Y = rnd(l_[d] + c_[d], rs);
                        if (shortcut_scale != 0.f) {
                            float sh = rnd(t1 * kk[d], rs);
                            Y = rnd(Y + rnd(shortcut_scale * sh, rs), rs);
                        }
                        acc += Y * qq[d];
                    }
                    float r = rnd(acc, round_bf16 & R_OUT);
                    y[src * N + s] = rnd(r * sc[src], round_bf16 & R_OUT);
                }
            }
    rc = 0;
done:
    free(A); free(vp); free(be); free(sc); free(kn); free(qn); free(Ap); free(Kp); free(Vp);
    free(bp); free(lh); free(cA); free(co); free(tA); free(fl); free(cs);
    return rc;
}

/* ------------------------------------------------------------------------------------
 * The plain sequential recurrence (one intra_chunk_scan.cu:117-167 step per token, no chunk
 * boundaries), with the same fused dynamics, normalisation, vp scale, shortcut and read-out.
 * Inside the first chunk the reference equals this recurrence; the one-token decode step is
 * defined by it.  state (B,H,N,D) is updated in place; y (B,L,H,N).
 * ---------------------------------------------------------------------------------- */
int orc_scan_recurrent(const float* q, const float* k, const float* v, const float* gate_raw,
                       const float* log_dt_scale, const float* rope_freqs, float gating_c,
                       float omega_thresh, float adt_delta, float adt_smoothness, float adt_eps,
                       float shortcut_scale, float* state, int B, int L, int H, int D, int N,
                       int pos0, int round_bf16, float* y) {
    if (N > ORC_MAX_N || D > ORC_MAX_D || (N & 1)) return -1;
    const int NH = N / 2;
    const size_t T = (size_t)B * L * H;
    float* A = malloc(sizeof(float) * T * N);
    float* vp = malloc(sizeof(float) * T * NH);
    float* be = malloc(sizeof(float) * T);
    float* sc = malloc(sizeof(float) * T);
    float* kn = malloc(sizeof(float) * T * D);
    float* qn = malloc(sizeof(float) * T * D);
    int rc = -1;
    if (!A || !vp || !be || !sc || !kn || !qn) goto done;
    orc_dynamics(gate_raw, log_dt_scale, rope_freqs, gating_c, omega_thresh, adt_delta,
                 adt_smoothness, adt_eps, B, L, H, N, pos0, round_bf16, A, vp, be, sc);
    orc_normalize_kq(k, q, T, D, round_bf16, kn, qn);
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < B; b++)
        for (int h = 0; h < H; h++) {
            float* st = state + ((size_t)b * H + h) * N * D;
            for (int l = 0; l < L; l++) {
                size_t row = ((size_t)b * L + l) * H + h;
                float vg[ORC_MAX_N];
                for (int s = 0; s < N; s++) vg[s] = rnd(v[row * N + s] * vp[row * NH + s / 2], round_bf16 & R_IN);
                step_state(st, A + row * N, kn + row * D, vg, be[row], N, D, 1);
                float qk = 0.f;
                for (int d = 0; d < D; d++) qk += qn[row * D + d] * kn[row * D + d];
                for (int s = 0; s < N; s++) {
                    float acc = 0.f;
                    for (int d = 0; d < D; d++) acc += st[s * D + d] * qn[row * D + d];
                    acc += shortcut_scale * qk * qk * vg[s];
                    y[row * N + s] = rnd(rnd(acc, round_bf16 & R_OUT) * sc[row], round_bf16 & R_OUT);
                }
            }
        }
    rc = 0;
done:
    free(A); free(vp); free(be); free(sc); free(kn); free(qn);
    return rc;
}

/* Size of the OpenMP team (test and benchmark infrastructure).  A launcher such as torch.distributed.run
 * exports OMP_NUM_THREADS=1 to its children; the CPU baseline asks for the host threads it may really use
 * and reports the team size it got.  Without OpenMP both return 1. */
#ifdef _OPENMP
#include <omp.h>
int orc_set_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
    int got = 1;
#pragma omp parallel
    {
#pragma omp single
        got = omp_get_num_threads();
    }
    return got;
}
#else
int orc_set_threads(int n) { (void)n; return 1; }
#endif
