// Backward kernels of the six operators (the reference's: dynamics_fused.cu:145-387, normalize_kq.cu:89-163,
// intra_chunk_scan.cu:215-553, inter_chunk_scan.cu:89-196, exact_correction.cu:169-383, conv1d_silu.cu:94-219).
// The gradients are derived from this library's own forward kernels by the chain rule, in fp32 (complex notation for
// the state row pairs), and checked against a float64 oracle that is itself checked by finite differences.
#include "cdssm_common.cuh"

namespace cdssm {

// (softplus'(x) = sigmoid(x); the x > 20 branch of the forward has slope 1 = sigmoid(x) to seven digits)

// ---------------------------------------------------------------- dynamics backward
// One thread per (token, head), heads fastest.  Recomputes the forward scalars, then walks the graph backwards:
//   per pair:   (A_re, A_im, vp) <- (mu, e, cr);  mu, e <- (ta, tw);  (ta, tw) <- (alpha_j, omega_j, dt)
//   shared:     dt <- (alpha_0, |omega_0|, log_dt_scale, sel_dt);  cr <- r_gate;  beta, sel_C <- their gates
// grad_log_dt_scale (H) is a sum over all tokens: per-block partial sums in shared memory, one atomic per head
// and block.
template <typename T>
__global__ void __launch_bounds__(256)
dynamics_bwd_kernel(const T* __restrict__ gA, const T* __restrict__ gvp, const T* __restrict__ gbeta,
                    const T* __restrict__ gselc, const T* __restrict__ gate_raw,
                    const float* __restrict__ log_dt_scale, const float* __restrict__ rope_freqs,
                    T* __restrict__ ggate, float* __restrict__ glds, DynConsts c, long long total, int H, int N, int L,
                    int pos0) {
    constexpr bool kFast = IO<T>::kBf16;
    extern __shared__ float part[];                 // H partial sums of grad_log_dt_scale
    for (int i = threadIdx.x; i < H; i += blockDim.x) part[i] = 0.f;
    __syncthreads();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) {
        const int h = (int)(idx % H);
        const long long bl = idx / H;
        const int NH = N >> 1;
        const long long gbase = bl * (long long)((N + 5) * H);
        const T* g = gate_raw + gbase;
        const T* sc = g + N * H;
        T* og = ggate + gbase;
        T* osc = og + N * H;
        const float freq = rope_freqs[h], pos = (float)((int)(bl % L) + pos0);
        // ---- forward scalars of the head (cdssm_math.cuh: dyn_shared)
        const float selB_raw = IO<T>::ld(sc + h), selC_raw = IO<T>::ld(sc + H + h), seldt_raw = IO<T>::ld(sc + 2 * H + h);
        const float beta_raw = IO<T>::ld(sc + 3 * H + h), r_raw = IO<T>::ld(sc + 4 * H + h);
        const float a0_raw = IO<T>::ld(g + h), w0_raw = IO<T>::ld(g + NH * H + h);
        const float lds = log_dt_scale[h];
        const float r = sigmoidf_<kFast>(r_raw);
        const float alpha0 = softplusf_<kFast>(a0_raw);
        const float w0 = w0_raw + pos * freq, w0a = fabsf(w0);
        const float s = softplusf_<kFast>(lds);
        const float cf = alpha0 + w0a + c.adt_eps;
        const float dt_raw = div_<kFast>(s, cf);
        const float am = alpha0 + c.adt_eps;
        const float dt_max = div_<kFast>(2.0f - c.adt_delta, am);
        const float blend = sigmoidf_<kFast>(div_<kFast>(c.omega_thresh - w0a, c.adt_smoothness));
        const bool capped = dt_raw > dt_max;
        const float dt = blend * fminf(dt_raw, dt_max) + (1.0f - blend) * dt_raw + softplusf_<kFast>(seldt_raw);
        const float cr = c.gating_c * r, x = (cr - 1.0f) * 0.5f, tau = 0.5f * dt;
        // ---- pairs
        float g_dt = 0.f, g_r = 0.f, g_a0_extra = 0.f, g_w0_extra = 0.f;
        for (int j = 0; j < NH; j++) {
            const float aj_raw = IO<T>::ld(g + j * H + h);
            const float alpha = fmaxf(softplusf_<kFast>(aj_raw), 0.0f);
            const float omega = IO<T>::ld(g + (NH + j) * H + h) + pos * freq;
            const float ta = tau * alpha, tw = tau * omega;
            const float den = (1.0f + ta) * (1.0f + ta) + tw * tw + kEps, iden = 1.0f / den;
            const float P = (1.0f - ta) * (1.0f + ta) - tw * tw;          // numerator of Re mu
            const float mu_re = P * iden, mu_im = 2.0f * tw * iden;
            const float num2 = (1.0f - ta) * (1.0f - ta) + tw * tw;
            const float e_raw = num2 * iden;
            const bool e_free = e_raw > 1e-8f;                            // the clamp passes the gradient through
            const float e = fmaxf(e_raw, 1e-8f), le = log_<kFast>(e);
            const float scale = exp_<kFast>(x * le), eff = exp_<kFast>(cr * le);
            const float vp2 = 1.0f - eff;
            const float uA_re = IO<T>::ld(gA + idx * N + 2 * j), uA_im = IO<T>::ld(gA + idx * N + 2 * j + 1);
            const float uvp = IO<T>::ld(gvp + idx * NH + j);
            // vp = min(sqrt(max(1 - eff, eps)), 1): gradient only where neither clamp is active
            float g_eff = 0.f;
            if (vp2 > kEps && vp2 < 1.0f) g_eff = -0.5f * uvp * rsqrtf(vp2);
            // A = (mu_re, -mu_im) * scale
            const float g_scale = uA_re * mu_re - uA_im * mu_im;
            const float g_mu_re = uA_re * scale, g_mu_im = -uA_im * scale;
            // scale = e^x, eff = e^cr
            const float g_e = e_free ? (g_scale * x * scale + g_eff * cr * eff) / e : 0.f;
            g_r += (0.5f * g_scale * scale + g_eff * eff) * le * c.gating_c;
            // quotient rules: e = num2 / den, mu_re = P / den, mu_im = 2 tw / den
            const float g_den = -(g_e * e_raw + g_mu_re * mu_re + g_mu_im * mu_im) * iden;
            const float g_ta = g_e * iden * (-2.0f * (1.0f - ta)) + g_mu_re * iden * (-2.0f * ta) + g_den * 2.0f * (1.0f + ta);
            const float g_tw = g_e * iden * (2.0f * tw) + g_mu_re * iden * (-2.0f * tw) + g_mu_im * iden * 2.0f + g_den * 2.0f * tw;
            // ta = tau alpha, tw = tau omega, tau = dt / 2
            g_dt += 0.5f * (g_ta * alpha + g_tw * omega);
            float ga = g_ta * tau * sigmoidf_<kFast>(aj_raw), gw = g_tw * tau;
            if (j == 0) { g_a0_extra = ga; g_w0_extra = gw; }             // completed below with the dt path
            else {
                IO<T>::st(og + j * H + h, ga);
                IO<T>::st(og + (NH + j) * H + h, gw);
            }
        }
        // ---- adaptive time step: dt = blend min(dt_raw, dt_max) + (1 - blend) dt_raw + softplus(sel_dt)
        const float g_dt_raw = g_dt * (capped ? 1.0f - blend : 1.0f);
        const float g_dt_max = capped ? g_dt * blend : 0.f;
        const float g_blend = g_dt * (fminf(dt_raw, dt_max) - dt_raw);
        const float g_s = g_dt_raw / cf, g_cf = -g_dt_raw * dt_raw / cf;
        const float g_w0a = g_cf - g_blend * blend * (1.0f - blend) / c.adt_smoothness;
        const float g_alpha0 = g_cf - g_dt_max * dt_max / am;
        IO<T>::st(og + h, g_a0_extra + g_alpha0 * sigmoidf_<kFast>(a0_raw));
        IO<T>::st(og + NH * H + h, g_w0_extra + (w0 >= 0.f ? g_w0a : -g_w0a));
        // ---- gates
        const float sb = sigmoidf_<kFast>(selB_raw), sbe = sigmoidf_<kFast>(beta_raw), scg = sigmoidf_<kFast>(selC_raw);
        const float ub = IO<T>::ld(gbeta + idx), uc = IO<T>::ld(gselc + idx);
        IO<T>::st(osc + h, ub * sbe * sb * (1.0f - sb));
        IO<T>::st(osc + H + h, uc * scg * (1.0f - scg));
        IO<T>::st(osc + 2 * H + h, g_dt * sigmoidf_<kFast>(seldt_raw));
        IO<T>::st(osc + 3 * H + h, ub * sb * sbe * (1.0f - sbe));
        IO<T>::st(osc + 4 * H + h, g_r * r * (1.0f - r));
        atomicAdd(&part[h], g_s * sigmoidf_<kFast>(lds));
    }
    __syncthreads();
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        if (part[i] != 0.f) atomicAdd(glds + i, part[i]);
}

// ---------------------------------------------------------------- normalise backward
// x_hat = x * n, n = rsqrt(|x|^2 + eps):  grad_x = n * (g - x_hat * (g . x_hat)) up to the eps term of n.
// One warp per row pair, like the forward.
template <typename T>
__global__ void __launch_bounds__(256)
normalize_kq_bwd_kernel(const T* __restrict__ gKo, const T* __restrict__ gQo, const T* __restrict__ K,
                        const T* __restrict__ Q, T* __restrict__ gK, T* __restrict__ gQ, long long rows, int D) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const long long o = row * D;
    float sk = 0.f, sq = 0.f, dk = 0.f, dq = 0.f;
    for (int d = lane; d < D; d += 32) {
        const float a = IO<T>::ld(K + o + d), b = IO<T>::ld(Q + o + d);
        sk += a * a;
        sq += b * b;
        dk += a * IO<T>::ld(gKo + o + d);
        dq += b * IO<T>::ld(gQo + o + d);
    }
    sk = warp_sum(sk); sq = warp_sum(sq); dk = warp_sum(dk); dq = warp_sum(dq);
    const float nk = rsqrtf(sk + kEps), nq = rsqrtf(sq + kEps);
    const float ck = dk * nk * nk, cq = dq * nq * nq;      // (g . x_hat) * n
    for (int d = lane; d < D; d += 32) {
        IO<T>::st(gK + o + d, nk * (IO<T>::ld(gKo + o + d) - IO<T>::ld(K + o + d) * ck));
        IO<T>::st(gQ + o + d, nq * (IO<T>::ld(gQo + o + d) - IO<T>::ld(Q + o + d) * cq));
    }
}

// ---------------------------------------------------------------- scan-side backward kernels
// All three walk their recurrence backwards with the forward's SAVED outputs as the state before each step (like
// the reference: intra_chunk_scan.cu:268-540, exact_correction.cu:230-375, inter_chunk_scan.cu:115-190), one warp
// per (.., head, complex pair), lanes over the head dimension (up to four columns per lane).  Complex notation: a
// state row pair is z in C^D, the stored A pair multiplies it as a complex number, k is real.  For p = a e the
// gradients are G_a = sum_d G_p conj(e) and G_e = conj(a) G_p.  grad_K and grad_beta sum over the pairs of a head:
// float32 outputs, accumulated with atomics (zeroed by the launcher).
constexpr int kBwdCols = 4;   // D <= 128

struct cf { float r, i; };
__device__ __forceinline__ cf cmulf(cf a, cf b) { return {a.r * b.r - a.i * b.i, a.r * b.i + a.i * b.r}; }
__device__ __forceinline__ cf cmulc(cf a, cf b) { return {a.r * b.r + a.i * b.i, a.i * b.r - a.r * b.i}; }   // a conj(b)
__device__ __forceinline__ cf wsum(cf v) { return {warp_sum(v.r), warp_sum(v.i)}; }

// One reverse step shared by the intra-chunk and the correction walk: given G (gradient of the state AFTER the
// step, z_t = a e [+ beta v k], e = z' - beta u k, u = z' . k), the state before the step z', and the step's
// inputs, returns the gradient of z' and accumulates the input gradients.
template <bool kInject>
__device__ __forceinline__ void reverse_step(cf (&G)[kBwdCols], const cf (&zp)[kBwdCols], const float (&k)[kBwdCols],
                                             cf a, cf v, float beta, int ncols, cf& gA, cf& gV, float& gB,
                                             float (&gK)[kBwdCols]) {
    cf u = {0.f, 0.f}, s = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kBwdCols; i++) {
        u.r += zp[i].r * k[i]; u.i += zp[i].i * k[i];
        s.r += G[i].r * k[i];  s.i += G[i].i * k[i];
    }
    u = wsum(u);
    s = wsum(s);
    cf ga = {0.f, 0.f}, w = {0.f, 0.f};
    cf Ge[kBwdCols];
#pragma unroll
    for (int i = 0; i < kBwdCols; i++) {
        const cf e = {zp[i].r - beta * u.r * k[i], zp[i].i - beta * u.i * k[i]};
        const cf t = cmulc(G[i], e);
        ga.r += t.r; ga.i += t.i;
        Ge[i] = cmulc(G[i], a);                    // conj(a) G  ==  G conj(a)
        w.r += Ge[i].r * k[i]; w.i += Ge[i].i * k[i];
    }
    gA = wsum(ga);
    w = wsum(w);
    gB = -(w.r * u.r + w.i * u.i);
    gV = {0.f, 0.f};
    if (kInject) {
        gV = {beta * s.r, beta * s.i};
        gB += s.r * v.r + s.i * v.i;
    }
    const cf Gu = {-beta * w.r, -beta * w.i};
#pragma unroll
    for (int i = 0; i < kBwdCols; i++) {
        float g = -beta * (Ge[i].r * u.r + Ge[i].i * u.i) + Gu.r * zp[i].r + Gu.i * zp[i].i;
        if (kInject) g += beta * (G[i].r * v.r + G[i].i * v.i);
        gK[i] = g;
        G[i] = {Ge[i].r + Gu.r * k[i], Ge[i].i + Gu.i * k[i]};
    }
    (void)ncols;
}

// kIntra: intra-chunk scan backward (grad of local_h and cum_A in; grad A, K, V, beta out).
// !kIntra: correction backward (grad of corrections in; grad A, K, beta and grad chunk_states out).
// units = chunks (BNC resp. B*NC); A (units,C,H,N), K (units,C,H,D), V (units,C,H,N), beta (units,C,H);
// saved (units,C,H,N,D) = local_h resp. corrections; g_saved likewise; cum_A / g_cum_A (units,C,H,N) (intra only).
template <typename T, bool kIntra>
__global__ void __launch_bounds__(128)
chunk_walk_bwd_kernel(const T* __restrict__ g_saved, const T* __restrict__ g_cumA, const T* __restrict__ A,
                      const T* __restrict__ K, const T* __restrict__ V, const T* __restrict__ beta,
                      const T* __restrict__ saved, const T* __restrict__ cumA, T* __restrict__ gA_out,
                      float* __restrict__ gK_out, T* __restrict__ gV_out, float* __restrict__ gB_out,
                      T* __restrict__ gS_out, long long units, int C, int H, int D, int N, int g_first) {
    const int NP = N >> 1;
    const long long wid = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (wid >= units * H * NP) return;
    const int lane = threadIdx.x & 31;
    const int j = (int)(wid % NP);
    const int h = (int)((wid / NP) % H);
    const long long m = wid / ((long long)NP * H);
    cf G[kBwdCols], Gc = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kBwdCols; i++) G[i] = {0.f, 0.f};
    for (int t = C - 1; t >= 0; t--) {
        const long long row = (m * C + t) * H + h;                 // (unit, t, head)
        const long long srow = row * N + 2 * j;                    // pair j of the N-vectors
        const long long drow = srow * D;                           // pair j of the (N, D) state
        float k[kBwdCols];
        cf zp[kBwdCols];
        const long long prow = ((m * C + t - 1) * H + h) * N + 2 * j;
#pragma unroll
        for (int i = 0; i < kBwdCols; i++) {
            const int d = lane + 32 * i;
            const bool on = d < D;
            k[i] = on ? IO<T>::ld(K + row * D + d) : 0.f;
            if (kIntra) {
                // upstream gradient of the state AFTER step t; the state before it is the saved local_h[t-1]
                if (on) { G[i].r += IO<T>::ld(g_saved + drow + d); G[i].i += IO<T>::ld(g_saved + drow + D + d); }
                zp[i] = (on && t > 0) ? cf{IO<T>::ld(saved + prow * D + d), IO<T>::ld(saved + prow * D + D + d)} : cf{0.f, 0.f};
            } else {
                // the saved corrections[t] IS the state before step t
                zp[i] = on ? cf{IO<T>::ld(saved + drow + d), IO<T>::ld(saved + drow + D + d)} : cf{0.f, 0.f};
                // reference order: the upstream gradient of corrections[t] joins BEFORE step t is walked back
                // (exact_correction.cu:219-223), as if corrections[t] were the state after the step
                if (g_first && on) { G[i].r += IO<T>::ld(g_saved + drow + d); G[i].i += IO<T>::ld(g_saved + drow + D + d); }
            }
        }
        const cf a = {IO<T>::ld(A + srow), IO<T>::ld(A + srow + 1)};
        const cf v = kIntra ? cf{IO<T>::ld(V + srow), IO<T>::ld(V + srow + 1)} : cf{0.f, 0.f};
        const float be = IO<T>::ld(beta + row);
        cf gA, gV;
        float gB, gK[kBwdCols];
        reverse_step<kIntra>(G, zp, k, a, v, be, D, gA, gV, gB, gK);
        // reference order also reproduces the reference's grad_beta, which sums an already block-reduced value over
        // its D threads once more (exact_correction.cu:347-359): D times the derivative
        if (!kIntra && g_first) gB *= (float)D;
        if (kIntra) {   // cum_A[t] = a cum_A[t-1]
            Gc.r += IO<T>::ld(g_cumA + srow);
            Gc.i += IO<T>::ld(g_cumA + srow + 1);
            const cf cp = t > 0 ? cf{IO<T>::ld(cumA + prow), IO<T>::ld(cumA + prow + 1)} : cf{1.f, 0.f};
            const cf t1 = cmulc(Gc, cp);
            gA.r += t1.r; gA.i += t1.i;
            Gc = cmulc(Gc, a);
        } else if (!g_first) {
            // the output corrections[t] is the state before step t: its upstream gradient joins here
#pragma unroll
            for (int i = 0; i < kBwdCols; i++) {
                const int d = lane + 32 * i;
                if (d < D) { G[i].r += IO<T>::ld(g_saved + drow + d); G[i].i += IO<T>::ld(g_saved + drow + D + d); }
            }
        }
        if (lane == 0) {
            IO<T>::st(gA_out + srow, gA.r);
            IO<T>::st(gA_out + srow + 1, gA.i);
            if (kIntra) { IO<T>::st(gV_out + srow, gV.r); IO<T>::st(gV_out + srow + 1, gV.i); }
            atomicAdd(gB_out + row, gB);
        }
#pragma unroll
        for (int i = 0; i < kBwdCols; i++) {
            const int d = lane + 32 * i;
            if (d < D) atomicAdd(gK_out + row * D + d, gK[i]);
        }
    }
    if (!kIntra) {   // gradient of the chunk state the walk started from
        const long long so = ((m * H + h) * N + 2 * j) * D;
#pragma unroll
        for (int i = 0; i < kBwdCols; i++) {
            const int d = lane + 32 * i;
            if (d < D) { IO<T>::st(gS_out + so + d, G[i].r); IO<T>::st(gS_out + so + D + d, G[i].i); }
        }
    }
}

// Inter-chunk carry backward: s_{c+1} = A_c s_c + h_c, outputs s_c.  One warp per (batch, head, pair).
template <typename T>
__global__ void __launch_bounds__(128)
inter_chunk_bwd_kernel(const T* __restrict__ g_states, const T* __restrict__ total_A, const T* __restrict__ states,
                       T* __restrict__ gA_out, T* __restrict__ gH_out, int B, int NC, int H, int D, int N) {
    const int NP = N >> 1;
    const long long wid = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (wid >= (long long)B * H * NP) return;
    const int lane = threadIdx.x & 31;
    const int j = (int)(wid % NP);
    const int h = (int)((wid / NP) % H);
    const long long b = wid / ((long long)NP * H);
    cf G[kBwdCols];
#pragma unroll
    for (int i = 0; i < kBwdCols; i++) G[i] = {0.f, 0.f};
    for (int c = NC - 1; c >= 0; c--) {
        const long long srow = ((b * NC + c) * H + h) * N + 2 * j;
        const long long drow = srow * D;
        const cf a = {IO<T>::ld(total_A + srow), IO<T>::ld(total_A + srow + 1)};
        cf ga = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < kBwdCols; i++) {
            const int d = lane + 32 * i;
            if (d < D) {
                IO<T>::st(gH_out + drow + d, G[i].r);
                IO<T>::st(gH_out + drow + D + d, G[i].i);
                const cf s = {IO<T>::ld(states + drow + d), IO<T>::ld(states + drow + D + d)};
                const cf t = cmulc(G[i], s);
                ga.r += t.r; ga.i += t.i;
                const cf n = cmulc(G[i], a);
                G[i] = {n.r + IO<T>::ld(g_states + drow + d), n.i + IO<T>::ld(g_states + drow + D + d)};
            }
        }
        ga = wsum(ga);
        if (lane == 0) { IO<T>::st(gA_out + srow, ga.r); IO<T>::st(gA_out + srow + 1, ga.i); }
    }
}

// conv1d + SiLU backward: one thread per (batch row, segment of kSeg positions, channel).  pre-activations are
// recomputed; grad_x[t] needs the gradient of the pre-activations t .. t+3, so the walk runs three positions past
// the segment.  grad_w (Dm,4) and grad_bias (Dm): float32, accumulated with atomics (zeroed by the launcher).
template <typename T, int kSeg>
__global__ void __launch_bounds__(128)
conv1d_silu_bwd_kernel(const T* __restrict__ g_out, const T* __restrict__ x, const T* __restrict__ w,
                       const T* __restrict__ bias, T* __restrict__ gx, float* __restrict__ gw, float* __restrict__ gb,
                       int L, int Dm) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= Dm) return;
    const int l0 = blockIdx.y * kSeg;
    const long long base = (long long)blockIdx.z * L * Dm + d;
    const float w0 = IO<T>::ld(w + d * 4), w1 = IO<T>::ld(w + d * 4 + 1), w2 = IO<T>::ld(w + d * 4 + 2),
                w3 = IO<T>::ld(w + d * 4 + 3), bv = IO<T>::ld(bias + d);
    auto X = [&](int l) { return (l >= 0 && l < L) ? IO<T>::ld(x + base + (long long)l * Dm) : 0.f; };
    float x0 = X(l0 - 3), x1 = X(l0 - 2), x2 = X(l0 - 1);
    float p0 = 0.f, p1 = 0.f, p2 = 0.f;       // gradients of the three previous pre-activations
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, ab = 0.f;
    const int lend = min(l0 + kSeg, L);
    for (int u = l0; u < lend + 3; u++) {
        float gp = 0.f;
        const float x3 = X(u);
        if (u < L) {
            const float pre = w0 * x0 + w1 * x1 + w2 * x2 + w3 * x3 + bv;
            const float sg = sigmoidf_<false>(pre);
            gp = IO<T>::ld(g_out + base + (long long)u * Dm) * sg * (1.0f + pre * (1.0f - sg));
            if (u < lend) { a0 += gp * x0; a1 += gp * x1; a2 += gp * x2; a3 += gp * x3; ab += gp; }
        }
        // x[u-3] feeds pre[u-3] (w3), pre[u-2] (w2), pre[u-1] (w1), pre[u] (w0)
        const int t = u - 3;
        if (t >= l0 && t < lend) IO<T>::st(gx + base + (long long)t * Dm, w3 * p0 + w2 * p1 + w1 * p2 + w0 * gp);
        p0 = p1; p1 = p2; p2 = gp;
        x0 = x1; x1 = x2; x2 = x3;
    }
    atomicAdd(gw + d * 4, a0); atomicAdd(gw + d * 4 + 1, a1); atomicAdd(gw + d * 4 + 2, a2); atomicAdd(gw + d * 4 + 3, a3);
    atomicAdd(gb + d, ab);
}

}  // namespace cdssm

using namespace cdssm;

#define DISPATCH_DTYPE(dtype, ...)                                 \
    if ((dtype) == CDSSM_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else if ((dtype) == CDSSM_F32) { using T = float; __VA_ARGS__; }     \
    else return CDSSM_ERR_BAD_ARG;

extern "C" int cdssm_b200_dynamics_bwd(const void* grad_A_bar, const void* grad_vp_scale, const void* grad_beta,
                                       const void* grad_sel_C, const void* gate_raw, const float* log_dt_scale,
                                       const float* rope_freqs, void* grad_gate_raw, float* grad_log_dt_scale,
                                       float gating_c, float omega_thresh, float adt_delta, float adt_smoothness,
                                       float adt_eps, int B, int L, int H, int N, int pos0, int dtype, void* stream) {
    if (!grad_A_bar || !grad_vp_scale || !grad_beta || !grad_sel_C || !gate_raw || !log_dt_scale || !rope_freqs ||
        !grad_gate_raw || !grad_log_dt_scale)
        return CDSSM_ERR_BAD_ARG;
    if (B < 0 || L < 0 || H <= 0 || N <= 0 || (N & 1)) return CDSSM_ERR_BAD_ARG;
    if (N > kMaxStateDim || H > 8192) return CDSSM_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (int rc = check_cuda(cudaMemsetAsync(grad_log_dt_scale, 0, sizeof(float) * H, st))) return rc;
    const long long total = (long long)B * L * H;
    if (total == 0) return CDSSM_OK;
    DynConsts c{gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps};
    const unsigned blocks = (unsigned)((total + 255) / 256);
    DISPATCH_DTYPE(dtype, (dynamics_bwd_kernel<T><<<blocks, 256, sizeof(float) * H, st>>>(
                              (const T*)grad_A_bar, (const T*)grad_vp_scale, (const T*)grad_beta, (const T*)grad_sel_C,
                              (const T*)gate_raw, log_dt_scale, rope_freqs, (T*)grad_gate_raw, grad_log_dt_scale, c,
                              total, H, N, L, pos0)));
    return check_launch();
}

extern "C" int cdssm_b200_normalize_kq_bwd(const void* grad_K_out, const void* grad_Q_out, const void* K, const void* Q,
                                           void* grad_K, void* grad_Q, int64_t rows, int D, int dtype, void* stream) {
    if (!grad_K_out || !grad_Q_out || !K || !Q || !grad_K || !grad_Q || rows < 0 || D <= 0) return CDSSM_ERR_BAD_ARG;
    if (rows == 0) return CDSSM_OK;
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    DISPATCH_DTYPE(dtype, (normalize_kq_bwd_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>(
                              (const T*)grad_K_out, (const T*)grad_Q_out, (const T*)K, (const T*)Q, (T*)grad_K,
                              (T*)grad_Q, rows, D)));
    return check_launch();
}

static int check_bwd_dims(int C, int H, int D, int N) {
    if (C <= 0 || H <= 0 || D <= 0 || N <= 0 || (N & 1)) return CDSSM_ERR_BAD_ARG;
    if (N > kMaxStateDim || D > 32 * kBwdCols) return CDSSM_ERR_UNSUPPORTED;
    return CDSSM_OK;
}

extern "C" int cdssm_b200_intra_chunk_scan_bwd(const void* grad_local_h, const void* grad_cum_A, const void* A,
                                               const void* K, const void* V, const void* beta, const void* local_h,
                                               const void* cum_A, void* grad_A, float* grad_K, void* grad_V,
                                               float* grad_beta, int BNC, int C, int H, int D, int N, int dtype,
                                               void* stream) {
    if (!grad_local_h || !grad_cum_A || !A || !K || !V || !beta || !local_h || !cum_A || !grad_A || !grad_K ||
        !grad_V || !grad_beta || BNC < 0)
        return CDSSM_ERR_BAD_ARG;
    if (int rc = check_bwd_dims(C, H, D, N)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const long long rows = (long long)BNC * C * H;
    if (rows == 0) return CDSSM_OK;
    if (int rc = check_cuda(cudaMemsetAsync(grad_K, 0, sizeof(float) * rows * D, st))) return rc;
    if (int rc = check_cuda(cudaMemsetAsync(grad_beta, 0, sizeof(float) * rows, st))) return rc;
    const long long warps = (long long)BNC * H * (N / 2);
    DISPATCH_DTYPE(dtype, (chunk_walk_bwd_kernel<T, true><<<(unsigned)((warps + 3) / 4), 128, 0, st>>>(
                              (const T*)grad_local_h, (const T*)grad_cum_A, (const T*)A, (const T*)K, (const T*)V,
                              (const T*)beta, (const T*)local_h, (const T*)cum_A, (T*)grad_A, grad_K, (T*)grad_V,
                              grad_beta, nullptr, BNC, C, H, D, N, 0)));
    return check_launch();
}

extern "C" int cdssm_b200_exact_correction_bwd(const void* grad_corrections, const void* A, const void* K,
                                               const void* beta, const void* corrections, void* grad_A,
                                               float* grad_K, float* grad_beta, void* grad_states, int B, int NC,
                                               int C, int H, int D, int N, int reference_order, int dtype,
                                               void* stream) {
    if (!grad_corrections || !A || !K || !beta || !corrections || !grad_A || !grad_K || !grad_beta || !grad_states ||
        B < 0 || NC < 0)
        return CDSSM_ERR_BAD_ARG;
    if (int rc = check_bwd_dims(C, H, D, N)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const long long units = (long long)B * NC, rows = units * C * H;
    if (rows == 0) return CDSSM_OK;
    if (int rc = check_cuda(cudaMemsetAsync(grad_K, 0, sizeof(float) * rows * D, st))) return rc;
    if (int rc = check_cuda(cudaMemsetAsync(grad_beta, 0, sizeof(float) * rows, st))) return rc;
    const long long warps = units * H * (N / 2);
    DISPATCH_DTYPE(dtype, (chunk_walk_bwd_kernel<T, false><<<(unsigned)((warps + 3) / 4), 128, 0, st>>>(
                              (const T*)grad_corrections, nullptr, (const T*)A, (const T*)K, nullptr, (const T*)beta,
                              (const T*)corrections, nullptr, (T*)grad_A, grad_K, nullptr, grad_beta,
                              (T*)grad_states, units, C, H, D, N, reference_order ? 1 : 0)));
    return check_launch();
}

extern "C" int cdssm_b200_inter_chunk_scan_bwd(const void* grad_chunk_states, const void* total_A,
                                               const void* chunk_states, void* grad_total_A,
                                               void* grad_final_local_h, int B, int NC, int H, int D, int N,
                                               int dtype, void* stream) {
    if (!grad_chunk_states || !total_A || !chunk_states || !grad_total_A || !grad_final_local_h || B < 0 || NC < 0)
        return CDSSM_ERR_BAD_ARG;
    if (int rc = check_bwd_dims(1, H, D, N)) return rc;
    const long long warps = (long long)B * H * (N / 2);
    if (warps == 0 || NC == 0) return CDSSM_OK;
    DISPATCH_DTYPE(dtype, (inter_chunk_bwd_kernel<T><<<(unsigned)((warps + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
                              (const T*)grad_chunk_states, (const T*)total_A, (const T*)chunk_states,
                              (T*)grad_total_A, (T*)grad_final_local_h, B, NC, H, D, N)));
    return check_launch();
}

extern "C" int cdssm_b200_conv1d_silu_bwd(const void* grad_out, const void* x, const void* weight, const void* bias,
                                          void* grad_x, float* grad_weight, float* grad_bias, int B, int L, int Dm,
                                          int dtype, void* stream) {
    if (!grad_out || !x || !weight || !bias || !grad_x || !grad_weight || !grad_bias || B < 0 || L < 0 || Dm <= 0)
        return CDSSM_ERR_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    if (int rc = check_cuda(cudaMemsetAsync(grad_weight, 0, sizeof(float) * Dm * 4, st))) return rc;
    if (int rc = check_cuda(cudaMemsetAsync(grad_bias, 0, sizeof(float) * Dm, st))) return rc;
    if (B == 0 || L == 0) return CDSSM_OK;
    if (B > 65535) return CDSSM_ERR_UNSUPPORTED;
    constexpr int kSeg = 64;
    dim3 grid((Dm + 127) / 128, (L + kSeg - 1) / kSeg, B);
    if (grid.y > 65535) return CDSSM_ERR_UNSUPPORTED;
    DISPATCH_DTYPE(dtype, (conv1d_silu_bwd_kernel<T, kSeg><<<grid, 128, 0, st>>>(
                              (const T*)grad_out, (const T*)x, (const T*)weight, (const T*)bias, (T*)grad_x,
                              grad_weight, grad_bias, L, Dm)));
    return check_launch();
}
