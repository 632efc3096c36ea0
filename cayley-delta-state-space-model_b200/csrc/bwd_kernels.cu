// Backward kernels of the two memory-bound operators: the fused dynamics and the K/Q normalisation.
// (The reference's are dynamics_fused.cu:145-387 and normalize_kq.cu:89-163; the gradients here are derived from
// this library's own forward in cdssm_math.cuh by the chain rule, stage by stage, in fp32.  The four scan-side
// backward kernels are not built.)
#include "cdssm_common.cuh"

namespace cdssm {

// d/dx of sigmoid and softplus (softplus'(x) = sigmoid(x); the x > 20 branch of the forward has slope 1 = sigmoid(x)
// to seven digits)
template <bool kFast> __device__ __forceinline__ float dsigmoid_(float s) { return s * (1.0f - s); }

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
