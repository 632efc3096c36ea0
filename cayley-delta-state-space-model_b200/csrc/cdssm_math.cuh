// Device-side math shared by every kernel of the CD-SSM scan path.
//
// The formulas restate the reference's (cdssm/csrc/include/common.cuh:82-91 for the
// activations, cdssm/csrc/include/cayley_math.cuh:51-99 for the Cayley map,
// cdssm/csrc/kernels/dynamics_fused.cu:64-139 for the gate pipeline).  The reference is built
// with --use_fast_math, so its expf/logf/powf and '/' are the fast intrinsics; the bfloat16
// instantiations here call those intrinsics explicitly (kFast) and their outputs agree with
// the reference's bit for bit almost everywhere.  The float32 instantiations use the accurate
// library functions instead, to stay within 1e-4 of an fp32 restatement over long sequences.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cdssm {

constexpr int kMaxStateDim = 32;   // N: even, N/2 complex pairs per head (common.cuh:34)
constexpr int kMaxHeadDim = 128;   // D (common.cuh:35)
constexpr float kEps = 1e-6f;      // common.cuh:142

// ---- storage types: bf16 (the reference's only I/O type) and fp32 ------------------------
template <typename T> struct IO;
template <> struct IO<__nv_bfloat16> {
    static constexpr bool kBf16 = true;
    static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void st(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
    // value as the reference would see it after a bf16 store
    static __device__ __forceinline__ float rnd(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <> struct IO<float> {
    static constexpr bool kBf16 = false;
    static __device__ __forceinline__ float ld(const float* p) { return *p; }
    static __device__ __forceinline__ void st(float* p, float x) { *p = x; }
    static __device__ __forceinline__ float rnd(float x) { return x; }
};

template <bool kFast> __device__ __forceinline__ float exp_(float x) { return kFast ? __expf(x) : expf(x); }
template <bool kFast> __device__ __forceinline__ float log_(float x) { return kFast ? __logf(x) : logf(x); }
template <bool kFast> __device__ __forceinline__ float pow_(float x, float y) { return kFast ? __powf(x, y) : powf(x, y); }
template <bool kFast> __device__ __forceinline__ float div_(float a, float b) { return kFast ? __fdividef(a, b) : a / b; }

template <bool kFast> __device__ __forceinline__ float sigmoidf_(float x) {
    return div_<kFast>(1.0f, 1.0f + exp_<kFast>(-x));
}
template <bool kFast> __device__ __forceinline__ float softplusf_(float x) {
    return x > 20.0f ? x : log_<kFast>(1.0f + exp_<kFast>(x));
}
template <bool kFast> __device__ __forceinline__ float siluf_(float x) {
    return div_<kFast>(x, 1.0f + exp_<kFast>(-x));
}

struct DynConsts {
    float gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps;
};

// Per-(token, head) quantities shared by all complex pairs of the head.
struct DynShared {
    float dt, cr, beta, sel_c;   // cr = gating_c * sigmoid(r_gate)
};

// dynamics_fused.cu:64-96,133-139.  alpha0_raw/omega0_raw are pair 0's gates; pos is the
// absolute position of the token.
template <bool kFast>
__device__ __forceinline__ DynShared dyn_shared(float alpha0_raw, float omega0_raw, float sel_B,
                                                float sel_C, float sel_dt, float beta_raw,
                                                float r_raw, float log_dt_scale, float freq,
                                                float pos, const DynConsts& c) {
    DynShared o;
    float r_gate = sigmoidf_<kFast>(r_raw);
    float alpha0 = softplusf_<kFast>(alpha0_raw);
    float w0 = fabsf(omega0_raw + pos * freq);
    float dt_scale = softplusf_<kFast>(log_dt_scale);
    float dt_raw = div_<kFast>(dt_scale, alpha0 + w0 + c.adt_eps);
    float dt_max = div_<kFast>(2.0f - c.adt_delta, alpha0 + c.adt_eps);
    float blend = sigmoidf_<kFast>(div_<kFast>(c.omega_thresh - w0, c.adt_smoothness));
    float dt_cap = fminf(dt_raw, dt_max);
    o.dt = blend * dt_cap + (1.0f - blend) * dt_raw + softplusf_<kFast>(sel_dt);
    o.cr = c.gating_c * r_gate;
    o.beta = sigmoidf_<kFast>(beta_raw) * sigmoidf_<kFast>(sel_B);
    o.sel_c = sigmoidf_<kFast>(sel_C);
    return o;
}

// One complex pair: Cayley map of lambda = -alpha + i*omega with tau = dt/2, stored as the
// conjugate, scaled by |mu|^(c*r - 1); vp = sqrt(1 - |mu|^(2*c*r)).
// dynamics_fused.cu:98-131, cayley_math.cuh:51-99.
template <bool kFast>
__device__ __forceinline__ void dyn_pair(float alpha_raw, float omega_raw, float freq, float pos,
                                         const DynShared& s, float& a_re, float& a_im, float& vp) {
    float alpha = fmaxf(softplusf_<kFast>(alpha_raw), 0.0f);
    float omega = omega_raw + pos * freq;
    float tau = s.dt * 0.5f, ta = tau * alpha, tw = tau * omega;
    float nr = 1.0f - ta, ni = tw, dr = 1.0f + ta, di = -tw;
    float denom = __fmaf_rn(dr, dr, di * di) + kEps;
    float inv_d = __fdiv_rn(1.0f, denom);
    float mu_re = (nr * dr + ni * di) * inv_d;
    float mu_im = (ni * dr - nr * di) * inv_d;
    float numer = __fmaf_rn(1.0f - ta, 1.0f - ta, tw * tw);
    float den2 = __fmaf_rn(1.0f + ta, 1.0f + ta, tw * tw);
    float eig = fmaxf(div_<kFast>(numer, den2 + kEps), 1e-8f);
    float scale = pow_<kFast>(eig, (s.cr - 1.0f) / 2.0f);
    a_re = mu_re * scale;
    a_im = -mu_im * scale;
    float eff = pow_<kFast>(eig, s.cr);
    vp = fminf(sqrtf(fmaxf(1.0f - eff, kEps)), 1.0f);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 16-byte vector of eight bfloat16 values <-> eight floats.
__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

template <typename T> struct Vec8;   // eight consecutive elements
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float* f) {
        unpack8(*reinterpret_cast<const uint4*>(p), f);
    }
    static __device__ __forceinline__ void st(__nv_bfloat16* p, const float* f) {
        uint4 r;
        r.x = pack2(f[0], f[1]); r.y = pack2(f[2], f[3]); r.z = pack2(f[4], f[5]); r.w = pack2(f[6], f[7]);
        *reinterpret_cast<uint4*>(p) = r;
    }
};
template <> struct Vec8<float> {
    static __device__ __forceinline__ void ld(const float* p, float* f) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    static __device__ __forceinline__ void st(float* p, const float* f) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
};

}  // namespace cdssm
