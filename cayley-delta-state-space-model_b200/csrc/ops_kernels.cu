// The six operator-level forward kernels behind the reference's cdssm/ops.py classes.
//
// These keep the reference's operator boundaries (and therefore its HBM traffic: the
// (B,L,H,N,D) tensors are materialised) so that cdssm/models/ssd.py and block.py can run on
// them unchanged.  The measured path is the fused one (scan_wa.cu, scan_simt.cu); these exist for the
// strict drop-in and as building blocks of the parity tests.
//
// Thread mappings differ from the reference's (one block of D threads per (chunk, head) with
// two block barriers per step):
//   * the complex pairs of a head never interact (each pair owns two state rows; the erase
//     uses a per-row dot product), so the sequential kernels run one WARP per
//     (chunk, head, pair): the per-step reduction is a warp shuffle, no barrier at all;
//   * the dynamics kernel maps consecutive threads to consecutive heads so that every gate
//     segment is read coalesced.
#include "cdssm_common.cuh"

namespace cdssm {

// ---------------------------------------------------------------- dynamics
template <typename T>
__global__ void __launch_bounds__(256)
dynamics_fwd_kernel(const T* __restrict__ gate_raw, const float* __restrict__ log_dt_scale,
                    const float* __restrict__ rope_freqs, T* __restrict__ A_bar,
                    T* __restrict__ vp_scale, T* __restrict__ beta, T* __restrict__ sel_C,
                    DynConsts c, long long total, int H, int N, int L, int pos0) {
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int h = (int)(idx % H);
    const long long bl = idx / H;
    const int l = (int)(bl % L);
    const int NH = N >> 1;
    const T* g = gate_raw + bl * (long long)((N + 5) * H);
    const T* sc = g + N * H;
    const float freq = rope_freqs[h];
    const float pos = (float)(l + pos0);
    DynShared s = dyn_shared<IO<T>::kBf16>(IO<T>::ld(g + h), IO<T>::ld(g + NH * H + h), IO<T>::ld(sc + h),
                             IO<T>::ld(sc + H + h), IO<T>::ld(sc + 2 * H + h),
                             IO<T>::ld(sc + 3 * H + h), IO<T>::ld(sc + 4 * H + h),
                             log_dt_scale[h], freq, pos, c);
    for (int j = 0; j < NH; j++) {
        float a_re, a_im, vp;
        dyn_pair<IO<T>::kBf16>(IO<T>::ld(g + j * H + h), IO<T>::ld(g + (NH + j) * H + h), freq, pos, s, a_re,
                 a_im, vp);
        IO<T>::st(A_bar + idx * N + 2 * j, a_re);
        IO<T>::st(A_bar + idx * N + 2 * j + 1, a_im);
        IO<T>::st(vp_scale + idx * NH + j, vp);
    }
    IO<T>::st(beta + idx, s.beta);
    IO<T>::st(sel_C + idx, s.sel_c);
}

// ---------------------------------------------------------------- normalise
// One warp per row pair (K row and Q row of the same token-head).
template <typename T>
__global__ void __launch_bounds__(256)
normalize_kq_fwd_kernel(const T* __restrict__ K, const T* __restrict__ Q, T* __restrict__ Ko,
                        T* __restrict__ Qo, long long rows, int D) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const T* k = K + row * D;
    const T* q = Q + row * D;
    float sk = 0.f, sq = 0.f;
    for (int d = lane; d < D; d += 32) {
        float a = IO<T>::ld(k + d), b = IO<T>::ld(q + d);
        sk += a * a;
        sq += b * b;
    }
    sk = warp_sum(sk);
    sq = warp_sum(sq);
    const float ik = rsqrtf(sk + kEps), iq = rsqrtf(sq + kEps);
    for (int d = lane; d < D; d += 32) {
        IO<T>::st(Ko + row * D + d, IO<T>::ld(k + d) * ik);
        IO<T>::st(Qo + row * D + d, IO<T>::ld(q + d) * iq);
    }
}

// ---------------------------------------------------------------- intra-chunk scan
// One warp per (chunk, head, pair).  Lane owns columns lane, lane+32, ... of the pair's two rows.
template <typename T, bool kInject>
__global__ void __launch_bounds__(128)
chunk_walk_kernel(const T* __restrict__ A, const T* __restrict__ K, const T* __restrict__ V,
                  const T* __restrict__ beta, const T* __restrict__ init,  // correction: carry in
                  T* __restrict__ states,   // local_h or corrections (units,C,H,N,D)
                  T* __restrict__ cum_A,    // intra only
                  long long units, int C, int H, int D, int N) {
    const int NH = N >> 1;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= units * H * NH) return;
    const int lane = threadIdx.x & 31;
    const int j = (int)(w % NH);
    const int hd = (int)((w / NH) % H);
    const long long c = w / ((long long)NH * H);
    constexpr int kCols = kMaxHeadDim / 32;
    float zr[kCols], zi[kCols];
#pragma unroll
    for (int i = 0; i < kCols; i++) {
        zr[i] = 0.f;
        zi[i] = 0.f;
        if (!kInject) {
            const int d = lane + 32 * i;
            if (d < D) {
                const T* p = init + ((c * H + hd) * N + 2 * j) * (long long)D + d;
                zr[i] = IO<T>::ld(p);
                zi[i] = IO<T>::ld(p + D);
            }
        }
    }
    float cr = 1.f, ci = 0.f;
    for (int t = 0; t < C; t++) {
        const long long row = (c * C + t) * H + hd;
        if (!kInject) {  // correction stores the state BEFORE the step (exact_correction.cu:90-94)
            T* out = states + (row * N + 2 * j) * (long long)D;
#pragma unroll
            for (int i = 0; i < kCols; i++) {
                const int d = lane + 32 * i;
                if (d < D) {
                    IO<T>::st(out + d, zr[i]);
                    IO<T>::st(out + D + d, zi[i]);
                }
            }
        }
        const float a_re = IO<T>::ld(A + row * N + 2 * j), a_im = IO<T>::ld(A + row * N + 2 * j + 1);
        const float b = IO<T>::ld(beta + row);
        float kk[kCols], ur = 0.f, ui = 0.f;
#pragma unroll
        for (int i = 0; i < kCols; i++) {
            const int d = lane + 32 * i;
            kk[i] = d < D ? IO<T>::ld(K + row * D + d) : 0.f;
            ur += zr[i] * kk[i];
            ui += zi[i] * kk[i];
        }
        ur = warp_sum(ur);
        ui = warp_sum(ui);
        float vr = 0.f, vi = 0.f;
        if (kInject) {
            vr = IO<T>::ld(V + row * N + 2 * j);
            vi = IO<T>::ld(V + row * N + 2 * j + 1);
        }
#pragma unroll
        for (int i = 0; i < kCols; i++) {
            float er = zr[i] - b * ur * kk[i];
            float ei = zi[i] - b * ui * kk[i];
            float nr = a_re * er - a_im * ei;
            float ni = a_re * ei + a_im * er;
            if (kInject) {
                nr += b * vr * kk[i];
                ni += b * vi * kk[i];
            }
            zr[i] = nr;
            zi[i] = ni;
        }
        if (kInject) {  // local scan stores the state AFTER the step (intra_chunk_scan.cu:169-173)
            T* out = states + (row * N + 2 * j) * (long long)D;
#pragma unroll
            for (int i = 0; i < kCols; i++) {
                const int d = lane + 32 * i;
                if (d < D) {
                    IO<T>::st(out + d, zr[i]);
                    IO<T>::st(out + D + d, zi[i]);
                }
            }
            const float nr = a_re * cr - a_im * ci, ni = a_re * ci + a_im * cr;
            cr = nr;
            ci = ni;
            if (lane == 0) {
                IO<T>::st(cum_A + row * N + 2 * j, cr);
                IO<T>::st(cum_A + row * N + 2 * j + 1, ci);
            }
        }
    }
}

// ---------------------------------------------------------------- inter-chunk carry
// One thread per (b, h, pair, d); serial over the chunks (inter_chunk_scan.cu:52-84).
template <typename T>
__global__ void __launch_bounds__(128)
inter_chunk_fwd_kernel(const T* __restrict__ total_A, const T* __restrict__ flh,
                       T* __restrict__ chunk_states, int B, int NC, int H, int D, int N) {
    const int NH = N >> 1;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)B * H * NH * D) return;
    const int d = (int)(idx % D);
    const int j = (int)((idx / D) % NH);
    const int hd = (int)((idx / ((long long)D * NH)) % H);
    const int b = (int)(idx / ((long long)D * NH * H));
    float sr = 0.f, si = 0.f;
    for (int k = 0; k < NC; k++) {
        const long long u = ((long long)b * NC + k) * H + hd;
        const long long o = (u * N + 2 * j) * (long long)D + d;
        IO<T>::st(chunk_states + o, sr);
        IO<T>::st(chunk_states + o + D, si);
        const float re = IO<T>::ld(total_A + u * N + 2 * j), im = IO<T>::ld(total_A + u * N + 2 * j + 1);
        const float fr = IO<T>::ld(flh + o), fi = IO<T>::ld(flh + o + D);
        const float nr = re * sr - im * si + fr;
        const float ni = re * si + im * sr + fi;
        sr = nr;
        si = ni;
    }
}

// ---------------------------------------------------------------- conv1d + SiLU
// One thread per channel, walking kSeg consecutive positions with the 3-deep history in
// registers (the reference re-reads the three neighbours from global for every output).
template <typename T, int kSeg>
__global__ void __launch_bounds__(128)
conv1d_silu_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                       T* __restrict__ out, int L, int Dm) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= Dm) return;
    const int l0 = blockIdx.y * kSeg;
    const long long base = (long long)blockIdx.z * L * Dm + d;
    const float w0 = IO<T>::ld(w + d * 4), w1 = IO<T>::ld(w + d * 4 + 1), w2 = IO<T>::ld(w + d * 4 + 2),
                w3 = IO<T>::ld(w + d * 4 + 3), bv = IO<T>::ld(bias + d);
    float x0 = l0 >= 3 ? IO<T>::ld(x + base + (long long)(l0 - 3) * Dm) : 0.f;
    float x1 = l0 >= 2 ? IO<T>::ld(x + base + (long long)(l0 - 2) * Dm) : 0.f;
    float x2 = l0 >= 1 ? IO<T>::ld(x + base + (long long)(l0 - 1) * Dm) : 0.f;
    const int lend = min(l0 + kSeg, L);
    for (int l = l0; l < lend; l++) {
        const float x3 = IO<T>::ld(x + base + (long long)l * Dm);
        const float yv = w0 * x0 + w1 * x1 + w2 * x2 + w3 * x3 + bv;
        IO<T>::st(out + base + (long long)l * Dm, siluf_<IO<T>::kBf16>(yv));
        x0 = x1;
        x1 = x2;
        x2 = x3;
    }
}

// ---------------------------------------------------------------- carries into consecutive segments
// One thread per (b, h, pair, d): carry_in[g] = s; s <- decay[g] (*) s + carry_out[g], g = 0..S-1.
// Segment g of batch element b is found at index b*batch_stride + g*seg_stride (in segments), so the
// same kernel serves segments stored as consecutive batch rows and summaries gathered rank by rank.
__global__ void __launch_bounds__(128)
compose_carries_kernel(const float* __restrict__ decay, const float* __restrict__ carry_out,
                       const float* __restrict__ h0, float* __restrict__ carry_in,
                       float* __restrict__ final_state, float* __restrict__ total_decay, int B, int S, int H,
                       int D, int N, long long batch_stride, long long seg_stride) {
    const int NH = N >> 1;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)B * H * NH * D) return;
    const int d = (int)(idx % D);
    const int j = (int)((idx / D) % NH);
    const int hd = (int)((idx / ((long long)D * NH)) % H);
    const int b = (int)(idx / ((long long)D * NH * H));
    const long long so = (((long long)b * H + hd) * N + 2 * j) * D + d;
    float sr = 0.f, si = 0.f, pr = 1.f, pi = 0.f;
    if (h0) { sr = h0[so]; si = h0[so + D]; }
    for (int g = 0; g < S; g++) {
        const long long seg = (long long)b * batch_stride + (long long)g * seg_stride;
        const long long o = ((seg * H + hd) * N + 2 * j) * D + d;
        if (carry_in) { carry_in[o] = sr; carry_in[o + D] = si; }
        const float re = decay[(seg * H + hd) * N + 2 * j], im = decay[(seg * H + hd) * N + 2 * j + 1];
        const float nr = re * sr - im * si + carry_out[o];
        const float ni = re * si + im * sr + carry_out[o + D];
        sr = nr;
        si = ni;
        const float qr = re * pr - im * pi, qi = re * pi + im * pr;
        pr = qr;
        pi = qi;
    }
    if (final_state) { final_state[so] = sr; final_state[so + D] = si; }
    if (total_decay && d == 0) {
        total_decay[((long long)b * H + hd) * N + 2 * j] = pr;
        total_decay[((long long)b * H + hd) * N + 2 * j + 1] = pi;
    }
}

}  // namespace cdssm

using namespace cdssm;

#define DISPATCH_DTYPE(dtype, ...)                                 \
    if ((dtype) == CDSSM_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else if ((dtype) == CDSSM_F32) { using T = float; __VA_ARGS__; }     \
    else return CDSSM_ERR_BAD_ARG;

extern "C" int cdssm_b200_dynamics_fwd(const void* gate_raw, const float* log_dt_scale,
                                       const float* rope_freqs, void* A_bar, void* vp_scale,
                                       void* beta, void* sel_C, float gating_c, float omega_thresh,
                                       float adt_delta, float adt_smoothness, float adt_eps, int B,
                                       int L, int H, int N, int pos0, int dtype, void* stream) {
    if (!gate_raw || !log_dt_scale || !rope_freqs || !A_bar || !vp_scale || !beta || !sel_C)
        return CDSSM_ERR_BAD_ARG;
    if (B < 0 || L < 0 || H <= 0 || N <= 0 || (N & 1)) return CDSSM_ERR_BAD_ARG;
    if (N > kMaxStateDim) return CDSSM_ERR_UNSUPPORTED;
    const long long total = (long long)B * L * H;
    if (total == 0) return CDSSM_OK;
    DynConsts c{gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps};
    const unsigned blocks = (unsigned)((total + 255) / 256);
    DISPATCH_DTYPE(dtype, (dynamics_fwd_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>(
                              (const T*)gate_raw, log_dt_scale, rope_freqs, (T*)A_bar,
                              (T*)vp_scale, (T*)beta, (T*)sel_C, c, total, H, N, L, pos0)));
    return check_launch();
}

extern "C" int cdssm_b200_normalize_kq_fwd(const void* K, const void* Q, void* K_out, void* Q_out,
                                           int64_t rows, int D, int dtype, void* stream) {
    if (!K || !Q || !K_out || !Q_out || rows < 0 || D <= 0) return CDSSM_ERR_BAD_ARG;
    if (rows == 0) return CDSSM_OK;
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    DISPATCH_DTYPE(dtype, (normalize_kq_fwd_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>(
                              (const T*)K, (const T*)Q, (T*)K_out, (T*)Q_out, rows, D)));
    return check_launch();
}

static int check_scan_dims(int C, int H, int D, int N) {
    if (C <= 0 || H <= 0 || D <= 0 || N <= 0 || (N & 1)) return CDSSM_ERR_BAD_ARG;
    if (N > kMaxStateDim || D > kMaxHeadDim) return CDSSM_ERR_UNSUPPORTED;
    return CDSSM_OK;
}

extern "C" int cdssm_b200_intra_chunk_scan_fwd(const void* A, const void* K, const void* V,
                                               const void* beta, void* local_h, void* cum_A,
                                               int BNC, int C, int H, int D, int N, int dtype,
                                               void* stream) {
    if (!A || !K || !V || !beta || !local_h || !cum_A || BNC < 0) return CDSSM_ERR_BAD_ARG;
    if (int rc = check_scan_dims(C, H, D, N)) return rc;
    const long long warps = (long long)BNC * H * (N / 2);
    if (warps == 0) return CDSSM_OK;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    DISPATCH_DTYPE(dtype, (chunk_walk_kernel<T, true><<<blocks, 128, 0, (cudaStream_t)stream>>>(
                              (const T*)A, (const T*)K, (const T*)V, (const T*)beta, nullptr,
                              (T*)local_h, (T*)cum_A, BNC, C, H, D, N)));
    return check_launch();
}

extern "C" int cdssm_b200_exact_correction_fwd(const void* A, const void* K, const void* beta,
                                               const void* chunk_states, void* corrections, int B,
                                               int NC, int C, int H, int D, int N, int dtype,
                                               void* stream) {
    if (!A || !K || !beta || !chunk_states || !corrections || B < 0 || NC < 0)
        return CDSSM_ERR_BAD_ARG;
    if (int rc = check_scan_dims(C, H, D, N)) return rc;
    const long long units = (long long)B * NC;
    const long long warps = units * H * (N / 2);
    if (warps == 0) return CDSSM_OK;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    DISPATCH_DTYPE(dtype, (chunk_walk_kernel<T, false><<<blocks, 128, 0, (cudaStream_t)stream>>>(
                              (const T*)A, (const T*)K, nullptr, (const T*)beta,
                              (const T*)chunk_states, (T*)corrections, nullptr, units, C, H, D, N)));
    return check_launch();
}

extern "C" int cdssm_b200_inter_chunk_scan_fwd(const void* total_A, const void* final_local_h,
                                               void* chunk_states, int B, int NC, int H, int D,
                                               int N, int dtype, void* stream) {
    if (!total_A || !final_local_h || !chunk_states || B < 0 || NC < 0) return CDSSM_ERR_BAD_ARG;
    if (int rc = check_scan_dims(1, H, D, N)) return rc;
    const long long threads = (long long)B * H * (N / 2) * D;
    if (threads == 0 || NC == 0) return CDSSM_OK;
    const unsigned blocks = (unsigned)((threads + 127) / 128);
    DISPATCH_DTYPE(dtype, (inter_chunk_fwd_kernel<T><<<blocks, 128, 0, (cudaStream_t)stream>>>(
                              (const T*)total_A, (const T*)final_local_h, (T*)chunk_states, B, NC,
                              H, D, N)));
    return check_launch();
}

extern "C" int cdssm_b200_conv1d_silu_fwd(const void* x, const void* weight, const void* bias,
                                          void* out, int B, int L, int Dm, int dtype,
                                          void* stream) {
    if (!x || !weight || !bias || !out || B < 0 || L < 0 || Dm <= 0) return CDSSM_ERR_BAD_ARG;
    if (B == 0 || L == 0) return CDSSM_OK;
    if (B > 65535) return CDSSM_ERR_UNSUPPORTED;
    constexpr int kSeg = 32;
    dim3 grid((Dm + 127) / 128, (L + kSeg - 1) / kSeg, B);
    if (grid.y > 65535) return CDSSM_ERR_UNSUPPORTED;
    DISPATCH_DTYPE(dtype, (conv1d_silu_fwd_kernel<T, kSeg><<<grid, 128, 0, (cudaStream_t)stream>>>(
                              (const T*)x, (const T*)weight, (const T*)bias, (T*)out, L, Dm)));
    return check_launch();
}

extern "C" int cdssm_b200_compose_carries(const float* decay, const float* carry_out, const float* h0,
                                          float* carry_in, float* final_state, float* total_decay, int B,
                                          int S, int H, int D, int N, int64_t batch_stride,
                                          int64_t seg_stride, void* stream) {
    if (!decay || !carry_out || B < 0 || S < 0) return CDSSM_ERR_BAD_ARG;
    if (int rc = check_scan_dims(1, H, D, N)) return rc;
    const long long threads = (long long)B * H * (N / 2) * D;
    if (threads == 0) return CDSSM_OK;
    compose_carries_kernel<<<(unsigned)((threads + 127) / 128), 128, 0, (cudaStream_t)stream>>>(
        decay, carry_out, h0, carry_in, final_state, total_decay, B, S, H, D, N, batch_stride, seg_stride);
    return check_launch();
}
