// Fused CD-SSM scan on CUDA cores (the general path: any even N <= 32, D <= 128, C <= 256,
// bf16 or fp32 storage).
//
// Reference chunk semantics (cdssm/models/ssd.py:56-111 over intra_chunk_scan.cu:100-195,
// inter_chunk_scan.cu:52-84, exact_correction.cu:89-150), per head and complex pair:
//   z_t : local state, zero at the start of every chunk, delta-rule step per token;
//   s_c : carry into chunk c,  s_{c+1} = gamma_c * s_c + z_{C-1}   (decay product only);
//   r_t : correction, r_0 = s_c, erase+rotate per token, taken BEFORE step t;
//   y_t = sel_C * ((z_t + r_t) . q_t + shortcut).
// Nothing of size (B,L,H,N,D) is stored.  Three launches:
//   local pass  : per (chunk, head, pair) walk z only -> gamma_c and z_{C-1}  (workspace)
//   carry pass  : per (batch, head, pair, d) serial over chunks -> s_c in place of z_{C-1}
//   output pass : per (chunk, head, pair) walk z and r together, read out y
// The local pass re-reads k, v and the gates (about half of the algorithmic bytes).  scan_wa.cu holds the
// tensor-core local and output pass for the shapes it supports; the carry pass here serves both.
//
// Thread mapping: eight lanes own one (chunk, head, pair) unit, each lane D/8 contiguous
// columns of the two state rows, so a k/q row is fetched with 16-byte loads and a dot product
// costs three shuffles.  The sixteen units of a block are consecutive (head, pair) of one chunk
// wherever H*N/2 allows, which makes the strided gate and v reads of a block contiguous.
// The dynamics of a chunk are computed once per unit into shared memory before the walk.
#include "cdssm_common.cuh"
#include <atomic>

namespace cdssm {

constexpr int kLanesPerUnit = 8;
constexpr int kUnitsPerBlock = 16;
constexpr int kSimtThreads = kLanesPerUnit * kUnitsPerBlock;   // 128
constexpr int kMaxChunk = 256;

template <int kLanes = 8>
__device__ __forceinline__ float group_sum(float v) {   // sum over the kLanes (8 or 16) lanes of a unit
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    if (kLanes == 16) v += __shfl_xor_sync(0xffffffffu, v, 8);
    return v;
}

// Raw (storage-typed) slice of one row: kCols contiguous columns starting at g*kCols.
template <typename T, int kCols> struct RowSlice;
template <int kCols> struct RowSlice<__nv_bfloat16, kCols> {
    uint4 v[kCols / 8];
    __device__ __forceinline__ void load(const __nv_bfloat16* row, int g, int D, bool vec) {
        if (vec) {
            const uint4* p = reinterpret_cast<const uint4*>(row + g * kCols);
#pragma unroll
            for (int i = 0; i < kCols / 8; i++) v[i] = __ldg(p + i);
        } else {
            unsigned short* s = reinterpret_cast<unsigned short*>(v);
#pragma unroll
            for (int i = 0; i < kCols; i++) {
                const int d = g * kCols + i;
                s[i] = d < D ? __ldg(reinterpret_cast<const unsigned short*>(row) + d) : (unsigned short)0;
            }
        }
    }
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < kCols / 8; i++) v[i] = make_uint4(0, 0, 0, 0);
    }
    __device__ __forceinline__ void get(float* f) const {
#pragma unroll
        for (int i = 0; i < kCols / 8; i++) unpack8(v[i], f + 8 * i);
    }
};
template <int kCols> struct RowSlice<float, kCols> {
    float4 v[kCols / 4];
    __device__ __forceinline__ void load(const float* row, int g, int D, bool vec) {
        if (vec) {
            const float4* p = reinterpret_cast<const float4*>(row + g * kCols);
#pragma unroll
            for (int i = 0; i < kCols / 4; i++) v[i] = __ldg(p + i);
        } else {
            float* s = reinterpret_cast<float*>(v);
#pragma unroll
            for (int i = 0; i < kCols; i++) {
                const int d = g * kCols + i;
                s[i] = d < D ? __ldg(row + d) : 0.f;
            }
        }
    }
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < kCols / 4; i++) v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __device__ __forceinline__ void get(float* f) const {
        const float* s = reinterpret_cast<const float*>(v);
#pragma unroll
        for (int i = 0; i < kCols; i++) f[i] = s[i];
    }
};

// x * rsqrt(sum x^2 + 1e-6) over the unit's row, rounded like the reference's K_norm/Q_norm
// store (normalize_kq.cu:72-79).
template <typename T, int kCols>
__device__ __forceinline__ void normalise(float* f) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kCols; i++) ss += f[i] * f[i];
    const float inv = rsqrtf(group_sum(ss) + kEps);
#pragma unroll
    for (int i = 0; i < kCols; i++) f[i] = IO<T>::rnd(f[i] * inv);
}

struct ScanArgs {
    const void *q, *k, *v, *gate_raw;
    const float *log_dt_scale, *rope_freqs, *h0;
    void* y;
    float *final_state, *tail_state;
    float* total_decay;   // (B,H,N) or NULL: product over the chunks of the (rounded) chunk decays
    int segs;             // batch rows are `segs` consecutive segments of longer sequences
    int run_local;        // 0: the workspace already holds this input's local pass
    int run_output;       // 0: stop after the carry pass (another kernel writes y)
    int publish;          // 0: summary only, the carry pass leaves the local results in place
    int fp32_decay;       // 1: the transition a_t keeps float32 precision (the reference stores it as bf16)
    float* ws_gamma;   // (B,NC,H,NP,2)
    float* ws_state;   // (B,NC,H,NP,2,D): z_{C-1} after the local pass, s_c after the carry pass
    DynConsts dc;
    float shortcut_scale;
    int B, L, H, D, N, C, NC, pos0;
    long long units;   // B*NC*H*NP
};

// Shared-memory staging of one chunk's per-token scalars for the 16 units of a block.
struct ChunkScalars {
    float *a_re, *a_im, *beta, *v_re, *v_im, *sel_c;   // each [kUnitsPerBlock][C]
    __device__ ChunkScalars(float* base, int C, int units_per_block = kUnitsPerBlock) {
        const int n = units_per_block * C;
        a_re = base; a_im = base + n; beta = base + 2 * n; v_re = base + 3 * n;
        v_im = base + 4 * n; sel_c = base + 5 * n;
    }
};

// Dynamics of the unit's chunk: lane g handles tokens g, g+8, ...  (dynamics_fused.cu:64-139
// and the vp scale of block.py:194-195).  Padded positions (l >= L) get a = k = v = beta = 0
// like the reference's zero padding (ssd.py:60-67).
template <typename T, int kLanes>
__device__ __forceinline__ void stage_dynamics(const ScanArgs& a, ChunkScalars& sm, int ul, int g,
                                               int b, int c, int hd, int j) {
    const T* gate = static_cast<const T*>(a.gate_raw);
    const T* vv = static_cast<const T*>(a.v);
    const int NH = a.N >> 1, H = a.H;
    const float lds = a.log_dt_scale[hd], freq = a.rope_freqs[hd];
    for (int t = g; t < a.C; t += kLanes) {
        const int l = c * a.C + t;
        float ar = 0.f, ai = 0.f, be = 0.f, vr = 0.f, vi = 0.f, sc = 0.f;
        if (l < a.L) {
            const long long bl = (long long)b * a.L + l;
            const T* gr = gate + bl * (long long)((a.N + 5) * H);
            const T* s5 = gr + a.N * H;
            const float pos = (float)(l + a.pos0 + (b % a.segs) * a.L);
            DynShared ds = dyn_shared<IO<T>::kBf16>(IO<T>::ld(gr + hd), IO<T>::ld(gr + NH * H + hd),
                                      IO<T>::ld(s5 + hd), IO<T>::ld(s5 + H + hd),
                                      IO<T>::ld(s5 + 2 * H + hd), IO<T>::ld(s5 + 3 * H + hd),
                                      IO<T>::ld(s5 + 4 * H + hd), lds, freq, pos, a.dc);
            float vp;
            dyn_pair<IO<T>::kBf16>(IO<T>::ld(gr + j * H + hd), IO<T>::ld(gr + (NH + j) * H + hd), freq, pos, ds,
                     ar, ai, vp);
            if (!a.fp32_decay) {
                ar = IO<T>::rnd(ar);
                ai = IO<T>::rnd(ai);
            }
            vp = IO<T>::rnd(vp);
            be = IO<T>::rnd(ds.beta);
            sc = IO<T>::rnd(ds.sel_c);
            const T* vrow = vv + (bl * H + hd) * a.N + 2 * j;
            vr = IO<T>::rnd(IO<T>::ld(vrow) * vp);
            vi = IO<T>::rnd(IO<T>::ld(vrow + 1) * vp);
        }
        const int o = ul * a.C + t;
        sm.a_re[o] = ar; sm.a_im[o] = ai; sm.beta[o] = be;
        sm.v_re[o] = vr; sm.v_im[o] = vi; sm.sel_c[o] = sc;
    }
}

// kOutput = false: local pass (z only).  kOutput = true: output pass (z, r, read-out).
template <typename T, int kCols, int kLanes, bool kOutput>
__global__ void __launch_bounds__(kSimtThreads, kOutput ? (kCols == 16 ? 4 : 6) : 1)
scan_walk_kernel(const ScanArgs a) {
    constexpr int kUnits = kSimtThreads / kLanes;       // units per block
    extern __shared__ float smem[];
    ChunkScalars sm(smem, a.C, kUnits);
    const int ul = threadIdx.x / kLanes;                 // unit within the block
    const int g = threadIdx.x % kLanes;                  // lane within the unit
    long long u = (long long)blockIdx.x * kUnits + ul;
    const bool active = u < a.units;
    if (!active) u = a.units - 1;                        // keep the lane in the shuffles
    const int NH = a.N >> 1, D = a.D, C = a.C, H = a.H;
    const int j = (int)(u % NH);
    const int hd = (int)((u / NH) % H);
    const int c = (int)((u / ((long long)NH * H)) % a.NC);
    const int b = (int)(u / ((long long)NH * H * a.NC));
    const bool vec = (D == kCols * kLanes);              // rows are 16-byte aligned slices

    stage_dynamics<T, kLanes>(a, sm, ul, g, b, c, hd, j);
    __syncwarp();

    const int Lc = min(C, a.L - c * C);                  // valid tokens of this chunk
    const T* kbase = static_cast<const T*>(a.k) + (((long long)b * a.L + (long long)c * C) * H + hd) * D;
    const T* qbase = static_cast<const T*>(a.q) + (((long long)b * a.L + (long long)c * C) * H + hd) * D;
    const long long rstride = (long long)H * D;

    // State columns are held as pairs: every element-wise operation of the step is a packed
    // fp32x2 instruction (Blackwell FFMA2 / FMUL2), which halves the issue slots of a kernel that
    // is bound by instruction issue.
    constexpr int kP = kCols / 2;
    float2 zr[kP], zi[kP], rr[kP], ri[kP];
#pragma unroll
    for (int i = 0; i < kP; i++) { zr[i] = zi[i] = rr[i] = ri[i] = make_float2(0.f, 0.f); }
    const long long sidx = ((((long long)b * a.NC + c) * H + hd) * NH + j);
    if (kOutput) {
        const float* s = a.ws_state + sidx * 2 * D;
#pragma unroll
        for (int i = 0; i < kP; i++) {
            const int d = g * kCols + 2 * i;
            if (d < D) { rr[i].x = s[d]; ri[i].x = s[D + d]; }
            if (d + 1 < D) { rr[i].y = s[d + 1]; ri[i].y = s[D + d + 1]; }
        }
    }
    float cr = 1.f, ci = 0.f;

    RowSlice<T, kCols> kraw, qraw;
    kraw.load(kbase, g, D, vec);
    if (kOutput) qraw.load(qbase, g, D, vec);
    const int so = ul * C;
    // The four units of a warp may sit in different chunks (a full one and the ragged last one):
    // every lane walks the warp's longest chunk so that the shuffles stay warp-wide; beyond its
    // own Lc a unit sees the zero padding of the reference (a = k = v = beta = 0, ssd.py:60-67).
    const int Lw = __reduce_max_sync(0xffffffffu, Lc);
    for (int t = 0; t < Lw; t++) {
        float2 kk[kP], qq[kP];
        kraw.get(reinterpret_cast<float*>(kk));
        if (kOutput) qraw.get(reinterpret_cast<float*>(qq));
        if (t + 1 < Lc) {
            kraw.load(kbase + (long long)(t + 1) * rstride, g, D, vec);
            if (kOutput) qraw.load(qbase + (long long)(t + 1) * rstride, g, D, vec);
        } else {
            kraw.zero();
            if (kOutput) qraw.zero();
        }
        const float a_re = sm.a_re[so + t], a_im = sm.a_im[so + t], be = sm.beta[so + t];
        const float vr = sm.v_re[so + t], vi = sm.v_im[so + t];
        // The rows stay raw; the normalisation (normalize_kq.cu:46-79) enters through the scalars
        // ik = |k|^-1, iq = |q|^-1:  k^ = ik k, q^ = iq q.  Every dot product of the step is taken
        // against the state BEFORE the update, so all reductions are issued together; the
        // post-step read-out follows from  z' = a z + Kz k  =>  z'.q = a (z.q) + Kz (k.q).
        // (The reference rounds k^ and q^ to bf16 before use; here they keep fp32 precision.)
        const float2 zero2 = make_float2(0.f, 0.f);
        float2 skk2 = zero2, zkr2 = zero2, zki2 = zero2;
#pragma unroll
        for (int i = 0; i < kP; i++) {
            skk2 = __ffma2_rn(kk[i], kk[i], skk2);
            zkr2 = __ffma2_rn(zr[i], kk[i], zkr2);
            zki2 = __ffma2_rn(zi[i], kk[i], zki2);
        }
        float skk = skk2.x + skk2.y, zkr = zkr2.x + zkr2.y, zki = zki2.x + zki2.y;
        float sqq = 0.f, kq = 0.f, zqr = 0.f, zqi = 0.f, rkr = 0.f, rki = 0.f, rqr = 0.f, rqi = 0.f;
        if (kOutput) {
            float2 sqq2 = zero2, kq2 = zero2, zqr2 = zero2, zqi2 = zero2, rkr2 = zero2, rki2 = zero2,
                   rqr2 = zero2, rqi2 = zero2;
#pragma unroll
            for (int i = 0; i < kP; i++) {
                sqq2 = __ffma2_rn(qq[i], qq[i], sqq2);
                kq2 = __ffma2_rn(kk[i], qq[i], kq2);
                zqr2 = __ffma2_rn(zr[i], qq[i], zqr2);
                zqi2 = __ffma2_rn(zi[i], qq[i], zqi2);
                rkr2 = __ffma2_rn(rr[i], kk[i], rkr2);
                rki2 = __ffma2_rn(ri[i], kk[i], rki2);
                rqr2 = __ffma2_rn(rr[i], qq[i], rqr2);
                rqi2 = __ffma2_rn(ri[i], qq[i], rqi2);
            }
            sqq = sqq2.x + sqq2.y; kq = kq2.x + kq2.y; zqr = zqr2.x + zqr2.y; zqi = zqi2.x + zqi2.y;
            rkr = rkr2.x + rkr2.y; rki = rki2.x + rki2.y; rqr = rqr2.x + rqr2.y; rqi = rqi2.x + rqi2.y;
        }
        skk = group_sum<kLanes>(skk); zkr = group_sum<kLanes>(zkr); zki = group_sum<kLanes>(zki);
        if (kOutput) {
            sqq = group_sum<kLanes>(sqq); kq = group_sum<kLanes>(kq); zqr = group_sum<kLanes>(zqr); zqi = group_sum<kLanes>(zqi);
            rkr = group_sum<kLanes>(rkr); rki = group_sum<kLanes>(rki); rqr = group_sum<kLanes>(rqr); rqi = group_sum<kLanes>(rqi);
        }
        const float ik = rsqrtf(skk + kEps);
        const float bik = be * ik, bik2 = bik * ik;
        // z' = a (z - beta (z.k^) k^) + beta v k^ = a z + Kz k
        const float czr = bik2 * zkr, czi = bik2 * zki;
        const float Kzr = bik * vr - (a_re * czr - a_im * czi);
        const float Kzi = bik * vi - (a_re * czi + a_im * czr);
        const float2 are2 = make_float2(a_re, a_re), aim2 = make_float2(a_im, a_im), nim2 = make_float2(-a_im, -a_im);
        {
            const float2 kzr2 = make_float2(Kzr, Kzr), kzi2 = make_float2(Kzi, Kzi);
#pragma unroll
            for (int i = 0; i < kP; i++) {
                const float2 x = zr[i], y = zi[i];
                zr[i] = __ffma2_rn(kzr2, kk[i], __ffma2_rn(are2, x, __fmul2_rn(nim2, y)));
                zi[i] = __ffma2_rn(kzi2, kk[i], __ffma2_rn(are2, y, __fmul2_rn(aim2, x)));
            }
        }
        const float ncr = a_re * cr - a_im * ci, nci = a_re * ci + a_im * cr;
        cr = ncr;
        ci = nci;
        if (kOutput) {
            const float iq = rsqrtf(sqq + kEps);
            // correction is read BEFORE its step (exact_correction.cu:90-94), the local state after
            float yr = iq * (rqr + a_re * zqr - a_im * zqi + Kzr * kq);
            float yi = iq * (rqi + a_re * zqi + a_im * zqr + Kzi * kq);
            // r' = a (r - beta (r.k^) k^) = a r + Kr k
            const float crr = bik2 * rkr, cri = bik2 * rki;
            const float Krr = -(a_re * crr - a_im * cri), Kri = -(a_re * cri + a_im * crr);
            const float2 krr2 = make_float2(Krr, Krr), kri2 = make_float2(Kri, Kri);
#pragma unroll
            for (int i = 0; i < kP; i++) {
                const float2 x = rr[i], y = ri[i];
                rr[i] = __ffma2_rn(krr2, kk[i], __ffma2_rn(are2, x, __fmul2_rn(nim2, y)));
                ri[i] = __ffma2_rn(kri2, kk[i], __ffma2_rn(are2, y, __fmul2_rn(aim2, x)));
            }
            if (a.shortcut_scale != 0.f) {   // block.py:202-208: sum_d shortcut[s,d] q[d] = (q^.k^)^2 v[s]
                const float qk = iq * ik * kq;
                const float f = a.shortcut_scale * qk * qk;
                yr += f * vr;
                yi += f * vi;
            }
            if (g == 0) {   // v slots of this step are consumed: reuse them to stage y
                const float sc = sm.sel_c[so + t];
                sm.v_re[so + t] = IO<T>::rnd(IO<T>::rnd(yr) * sc);
                sm.v_im[so + t] = IO<T>::rnd(IO<T>::rnd(yi) * sc);
            }
            if (a.tail_state != nullptr && c * C + t == a.L - 1 && active) {
                float* ts = a.tail_state + (((long long)b * H + hd) * a.N + 2 * j) * D;
#pragma unroll
                for (int i = 0; i < kP; i++) {
                    const int d = g * kCols + 2 * i;
                    if (d < D) { ts[d] = zr[i].x + rr[i].x; ts[D + d] = zi[i].x + ri[i].x; }
                    if (d + 1 < D) { ts[d + 1] = zr[i].y + rr[i].y; ts[D + d + 1] = zi[i].y + ri[i].y; }
                }
            }
        }
    }
    if (!kOutput) {
        if (Lc < C) {   // zero padding wipes the local state and the decay product
#pragma unroll
            for (int i = 0; i < kP; i++) { zr[i] = zi[i] = make_float2(0.f, 0.f); }
            cr = 0.f;
            ci = 0.f;
        }
        if (active) {
            // the carry pass consumes these as the reference's bf16 cum_A[:, -1] / local_h[:, -1]
            float* s = a.ws_state + sidx * 2 * D;
#pragma unroll
            for (int i = 0; i < kP; i++) {
                const int d = g * kCols + 2 * i;
                if (d < D) { s[d] = IO<T>::rnd(zr[i].x); s[D + d] = IO<T>::rnd(zi[i].x); }
                if (d + 1 < D) { s[d + 1] = IO<T>::rnd(zr[i].y); s[D + d + 1] = IO<T>::rnd(zi[i].y); }
            }
            if (g == 0) {
                a.ws_gamma[sidx * 2] = IO<T>::rnd(cr);
                a.ws_gamma[sidx * 2 + 1] = IO<T>::rnd(ci);
            }
        }
    } else {
        __syncwarp();
        if (active) {
            T* y = static_cast<T*>(a.y);
            for (int t = g; t < Lc; t += kLanes) {
                T* o = y + (((long long)b * a.L + c * C + t) * H + hd) * a.N + 2 * j;
                IO<T>::st(o, sm.v_re[so + t]);
                IO<T>::st(o + 1, sm.v_im[so + t]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// "Exact" semantics: the plain sequential recurrence over the whole sequence (what the reference's
// chunked scan equals inside its first chunk, and what the one-token decode step continues),
//   z_t = a_t (z_{t-1} - beta_t (z_{t-1}.k^_t) k^_t) + beta_t v_t k^_t,  y_t = sel_C (z_t.q^_t + shortcut),
// with z_{-1} = h0.  One 8-lane unit walks one (batch, head, pair) sequence from start to end; the
// dynamics are staged in shared memory kMaxChunk tokens at a time.  Parallel over B*H*N/2 only.
template <typename T, int kCols>
__global__ void __launch_bounds__(kSimtThreads)
scan_recurrent_kernel(const ScanArgs a) {
    constexpr int kLanes = kLanesPerUnit, kP = kCols / 2;
    extern __shared__ float smem[];
    const int CS = a.C;                                   // staging length (tokens per stage)
    ChunkScalars sm(smem, CS);
    const int ul = threadIdx.x / kLanes, g = threadIdx.x % kLanes;
    long long u = (long long)blockIdx.x * kUnitsPerBlock + ul;
    const bool active = u < a.units;
    if (!active) u = a.units - 1;
    const int NH = a.N >> 1, D = a.D, H = a.H;
    const int j = (int)(u % NH);
    const int hd = (int)((u / NH) % H);
    const int b = (int)(u / ((long long)NH * H));
    const bool vec = (D == kCols * kLanes);
    const long long rstride = (long long)H * D;
    float2 zr[kP], zi[kP];
    {
        const float* h = a.h0 ? a.h0 + (((long long)b * H + hd) * a.N + 2 * j) * D : nullptr;
#pragma unroll
        for (int i = 0; i < kP; i++) {
            const int d = g * kCols + 2 * i;
            zr[i] = make_float2(h && d < D ? h[d] : 0.f, h && d + 1 < D ? h[d + 1] : 0.f);
            zi[i] = make_float2(h && d < D ? h[D + d] : 0.f, h && d + 1 < D ? h[D + d + 1] : 0.f);
        }
    }
    const int so = ul * CS;
    for (int c = 0; c < a.NC; c++) {
        __syncwarp();
        stage_dynamics<T, kLanes>(a, sm, ul, g, b, c, hd, j);
        __syncwarp();
        const int Lc = min(CS, a.L - c * CS);
        const T* kbase = static_cast<const T*>(a.k) + (((long long)b * a.L + (long long)c * CS) * H + hd) * D;
        const T* qbase = static_cast<const T*>(a.q) + (((long long)b * a.L + (long long)c * CS) * H + hd) * D;
        RowSlice<T, kCols> kraw, qraw;
        kraw.load(kbase, g, D, vec);
        qraw.load(qbase, g, D, vec);
        for (int t = 0; t < Lc; t++) {
            float2 kk[kP], qq[kP];
            kraw.get(reinterpret_cast<float*>(kk));
            qraw.get(reinterpret_cast<float*>(qq));
            if (t + 1 < Lc) {
                kraw.load(kbase + (long long)(t + 1) * rstride, g, D, vec);
                qraw.load(qbase + (long long)(t + 1) * rstride, g, D, vec);
            }
            const float a_re = sm.a_re[so + t], a_im = sm.a_im[so + t], be = sm.beta[so + t];
            const float vr = sm.v_re[so + t], vi = sm.v_im[so + t];
            const float2 zero2 = make_float2(0.f, 0.f);
            float2 skk2 = zero2, sqq2 = zero2, kq2 = zero2, zkr2 = zero2, zki2 = zero2, zqr2 = zero2, zqi2 = zero2;
#pragma unroll
            for (int i = 0; i < kP; i++) {
                skk2 = __ffma2_rn(kk[i], kk[i], skk2);
                sqq2 = __ffma2_rn(qq[i], qq[i], sqq2);
                kq2 = __ffma2_rn(kk[i], qq[i], kq2);
                zkr2 = __ffma2_rn(zr[i], kk[i], zkr2);
                zki2 = __ffma2_rn(zi[i], kk[i], zki2);
                zqr2 = __ffma2_rn(zr[i], qq[i], zqr2);
                zqi2 = __ffma2_rn(zi[i], qq[i], zqi2);
            }
            const float skk = group_sum(skk2.x + skk2.y), sqq = group_sum(sqq2.x + sqq2.y);
            const float kq = group_sum(kq2.x + kq2.y);
            const float zkr = group_sum(zkr2.x + zkr2.y), zki = group_sum(zki2.x + zki2.y);
            const float zqr = group_sum(zqr2.x + zqr2.y), zqi = group_sum(zqi2.x + zqi2.y);
            const float ik = rsqrtf(skk + kEps), iq = rsqrtf(sqq + kEps);
            const float bik = be * ik, bik2 = bik * ik;
            const float czr = bik2 * zkr, czi = bik2 * zki;
            const float Kzr = bik * vr - (a_re * czr - a_im * czi);
            const float Kzi = bik * vi - (a_re * czi + a_im * czr);
            const float2 are2 = make_float2(a_re, a_re), aim2 = make_float2(a_im, a_im), nim2 = make_float2(-a_im, -a_im);
            const float2 kzr2 = make_float2(Kzr, Kzr), kzi2 = make_float2(Kzi, Kzi);
#pragma unroll
            for (int i = 0; i < kP; i++) {
                const float2 x = zr[i], y = zi[i];
                zr[i] = __ffma2_rn(kzr2, kk[i], __ffma2_rn(are2, x, __fmul2_rn(nim2, y)));
                zi[i] = __ffma2_rn(kzi2, kk[i], __ffma2_rn(are2, y, __fmul2_rn(aim2, x)));
            }
            float yr = iq * (a_re * zqr - a_im * zqi + Kzr * kq);
            float yi = iq * (a_re * zqi + a_im * zqr + Kzi * kq);
            if (a.shortcut_scale != 0.f) {
                const float qk = iq * ik * kq;
                yr += a.shortcut_scale * qk * qk * vr;
                yi += a.shortcut_scale * qk * qk * vi;
            }
            if (g == 0) {
                const float sc = sm.sel_c[so + t];
                sm.v_re[so + t] = IO<T>::rnd(IO<T>::rnd(yr) * sc);
                sm.v_im[so + t] = IO<T>::rnd(IO<T>::rnd(yi) * sc);
            }
        }
        __syncwarp();
        if (active) {
            T* y = static_cast<T*>(a.y);
            for (int t = g; t < Lc; t += kLanes) {
                T* o = y + (((long long)b * a.L + c * CS + t) * H + hd) * a.N + 2 * j;
                IO<T>::st(o, sm.v_re[so + t]);
                IO<T>::st(o + 1, sm.v_im[so + t]);
            }
        }
    }
    if (active && a.final_state) {
        float* fs = a.final_state + (((long long)b * H + hd) * a.N + 2 * j) * D;
#pragma unroll
        for (int i = 0; i < kP; i++) {
            const int d = g * kCols + 2 * i;
            if (d < D) { fs[d] = zr[i].x; fs[D + d] = zi[i].x; }
            if (d + 1 < D) { fs[d + 1] = zr[i].y; fs[D + d + 1] = zi[i].y; }
        }
    }
}

template <typename T, int kCols>
static int launch_recurrent(ScanArgs a, cudaStream_t st) {
    a.C = a.L < 128 ? a.L : 128;                          // staging length only: no chunk semantics here
    a.NC = (a.L + a.C - 1) / a.C;
    a.segs = 1;
    a.units = (long long)a.B * a.H * (a.N / 2);
    const size_t smem = (size_t)6 * kUnitsPerBlock * a.C * sizeof(float);
    const unsigned blocks = (unsigned)((a.units + kUnitsPerBlock - 1) / kUnitsPerBlock);
    scan_recurrent_kernel<T, kCols><<<blocks, kSimtThreads, smem, st>>>(a);
    return check_launch();
}

// Carry pass: s_0 = h0 (or 0); for every chunk: publish s_c, then s <- gamma_c * s + z_{C-1}.
// One thread per (b, h, pair, d).  Chunks are taken eight at a time so that the loads of a
// batch are in flight together (the recurrence itself is two FMAs per chunk).
template <typename T>
__global__ void __launch_bounds__(128)
scan_carry_kernel(const ScanArgs a) {
    const int NH = a.N >> 1, D = a.D, H = a.H, NC = a.NC;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)a.B * H * NH * D) return;
    const int d = (int)(idx % D);
    const int j = (int)((idx / D) % NH);
    const int hd = (int)((idx / ((long long)D * NH)) % H);
    const int b = (int)(idx / ((long long)D * NH * H));
    const long long so = (((long long)b * H + hd) * a.N + 2 * j) * D + d;
    float sr = 0.f, si = 0.f, dr = 1.f, di = 0.f;
    if (a.h0) { sr = a.h0[so]; si = a.h0[so + D]; }
    const long long cstride = (long long)H * NH;            // units per chunk index
    const long long u0 = ((long long)b * NC * H + hd) * NH + j;
    constexpr int kBatch = 8;
    for (int c0 = 0; c0 < NC; c0 += kBatch) {
        float gr[kBatch], gi[kBatch], lr[kBatch], li[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; i++) {
            if (c0 + i < NC) {
                const long long u = u0 + (long long)(c0 + i) * cstride;
                gr[i] = a.ws_gamma[u * 2];
                gi[i] = a.ws_gamma[u * 2 + 1];
                lr[i] = a.ws_state[u * 2 * D + d];
                li[i] = a.ws_state[u * 2 * D + D + d];
            }
        }
#pragma unroll
        for (int i = 0; i < kBatch; i++) {
            if (c0 + i < NC) {
                const long long u = u0 + (long long)(c0 + i) * cstride;
                if (a.publish) {
                    a.ws_state[u * 2 * D + d] = IO<T>::rnd(sr);       // chunk_states store
                    a.ws_state[u * 2 * D + D + d] = IO<T>::rnd(si);
                }
                const float nr = gr[i] * sr - gi[i] * si + lr[i];
                const float ni = gr[i] * si + gi[i] * sr + li[i];
                sr = nr;
                si = ni;
                const float pr = gr[i] * dr - gi[i] * di, pi = gr[i] * di + gi[i] * dr;
                dr = pr;
                di = pi;
            }
        }
    }
    if (a.final_state) { a.final_state[so] = sr; a.final_state[so + D] = si; }
    if (a.total_decay && d == 0) {
        float* td = a.total_decay + ((long long)b * H + hd) * a.N + 2 * j;
        td[0] = dr;
        td[1] = di;
    }
}

template <typename T, int kCols, int kLanes>
static int launch_simt(const ScanArgs& a, cudaStream_t st) {
    constexpr int kUnits = kSimtThreads / kLanes;
    const size_t smem = (size_t)6 * kUnits * a.C * sizeof(float);
    if (smem > 48 * 1024) {   // opt in to more than 48 KB of dynamic shared memory
        if (int rc = check_cuda(cudaFuncSetAttribute(scan_walk_kernel<T, kCols, kLanes, false>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)))
            return rc;
        if (int rc = check_cuda(cudaFuncSetAttribute(scan_walk_kernel<T, kCols, kLanes, true>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)))
            return rc;
    }
    const unsigned blocks = (unsigned)((a.units + kUnits - 1) / kUnits);
    if (a.run_local) {
        scan_walk_kernel<T, kCols, kLanes, false><<<blocks, kSimtThreads, smem, st>>>(a);
        if (int rc = check_launch()) return rc;
    }
    const long long th = (long long)a.B * a.H * (a.N / 2) * a.D;
    scan_carry_kernel<T><<<(unsigned)((th + 127) / 128), 128, 0, st>>>(a);
    if (int rc = check_launch()) return rc;
    if (a.y == nullptr || !a.run_output) return CDSSM_OK;   // summary only, or y comes from another kernel
    scan_walk_kernel<T, kCols, kLanes, true><<<blocks, kSimtThreads, smem, st>>>(a);
    return check_launch();
}

// Column split: D <= 64 -> 8 lanes x 8 columns; D <= 128 -> 8 lanes x 16 columns, or (wide) 16 lanes x 8
// columns, which halves the state registers per thread and doubles the resident warps - measured
// slower on B200 (10.8 ms against 8.9 ms at the benchmark size: the per-unit scalar work and the extra
// shuffle stage cost more than the occupancy gains), so the narrow split is the one used.
int scan_fused_simt(const ScanArgs& a, int dtype, bool wide, cudaStream_t st) {
    const int cols = (a.D + kLanesPerUnit - 1) / kLanesPerUnit;
    if (dtype == CDSSM_BF16) {
        if (cols <= 8) return launch_simt<__nv_bfloat16, 8, 8>(a, st);
        return wide ? launch_simt<__nv_bfloat16, 8, 16>(a, st) : launch_simt<__nv_bfloat16, 16, 8>(a, st);
    }
    if (cols <= 8) return launch_simt<float, 8, 8>(a, st);
    return wide ? launch_simt<float, 8, 16>(a, st) : launch_simt<float, 16, 8>(a, st);
}

}  // namespace cdssm

namespace cdssm {
// ---------------------------------------------------------------------------------------------
// One-token decode step.  Eight lanes per (batch, head, pair): dynamics for position `pos`,
// normalise q/k, one delta-rule step on the fp32 state in place, read-out.  One pass over the
// state (read + write), everything else is a few hundred bytes per head.
struct DecodeArgs {
    float* state;
    float *corr, *carry, *gamma;   // reference-compatible step only: correction, carry (B,H,N,D), chunk decay (B,H,N)
    int C;                         // chunk length of the reference-compatible step
    const void *q, *k, *v, *gate_raw;
    long long k_stride, v_stride;  // elements between the batch rows of k and v (column slices of a wider projection)
    long long q_stride, g_stride;  // the same for q and gate_raw (plain step only)
    const void *v_first, *mix;     // plain step only, or NULL: v <- lerp(v_first, v, mix[head]) (value residual)
    const float *log_dt_scale, *rope_freqs;
    void* y;
    DynConsts dc;
    float shortcut_scale;
    int B, H, D, N, pos;
    const int* pos_dev;   // if not NULL the position is read from device memory (graph replay)
    long long units;   // B*H*NP
};

template <typename T, int kCols>
__global__ void __launch_bounds__(kSimtThreads)
decode_step_kernel(const DecodeArgs a) {
    const int g = threadIdx.x % kLanesPerUnit;
    long long u = (long long)blockIdx.x * kUnitsPerBlock + threadIdx.x / kLanesPerUnit;
    const bool active = u < a.units;
    if (!active) u = a.units - 1;
    const int NH = a.N >> 1, D = a.D, H = a.H;
    const int j = (int)(u % NH);
    const int hd = (int)((u / NH) % H);
    const long long b = u / ((long long)NH * H);
    const bool vec = (D == kCols * kLanesPerUnit);
    const long long bh = b * H + hd;

    RowSlice<T, kCols> kraw, qraw;
    kraw.load(static_cast<const T*>(a.k) + b * a.k_stride + (long long)hd * D, g, D, vec);
    qraw.load(static_cast<const T*>(a.q) + b * a.q_stride + (long long)hd * D, g, D, vec);
    float* st = a.state + (bh * a.N + 2 * j) * D;
    float zr[kCols], zi[kCols];
    if (vec) {
#pragma unroll
        for (int i = 0; i < kCols / 4; i++) {
            const float4 x = *reinterpret_cast<const float4*>(st + g * kCols + 4 * i);
            const float4 w = *reinterpret_cast<const float4*>(st + D + g * kCols + 4 * i);
            zr[4 * i] = x.x; zr[4 * i + 1] = x.y; zr[4 * i + 2] = x.z; zr[4 * i + 3] = x.w;
            zi[4 * i] = w.x; zi[4 * i + 1] = w.y; zi[4 * i + 2] = w.z; zi[4 * i + 3] = w.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < kCols; i++) {
            const int d = g * kCols + i;
            zr[i] = d < D ? st[d] : 0.f;
            zi[i] = d < D ? st[D + d] : 0.f;
        }
    }
    // dynamics (every lane of the unit computes the same scalars; dynamics_fused.cu:64-139)
    const T* gr = static_cast<const T*>(a.gate_raw) + b * a.g_stride;
    const T* s5 = gr + a.N * H;
    const float freq = a.rope_freqs[hd], pos = (float)(a.pos_dev ? *a.pos_dev : a.pos);
    DynShared ds = dyn_shared<IO<T>::kBf16>(IO<T>::ld(gr + hd), IO<T>::ld(gr + NH * H + hd), IO<T>::ld(s5 + hd),
                              IO<T>::ld(s5 + H + hd), IO<T>::ld(s5 + 2 * H + hd),
                              IO<T>::ld(s5 + 3 * H + hd), IO<T>::ld(s5 + 4 * H + hd),
                              a.log_dt_scale[hd], freq, pos, a.dc);
    float a_re, a_im, vp;
    dyn_pair<IO<T>::kBf16>(IO<T>::ld(gr + j * H + hd), IO<T>::ld(gr + (NH + j) * H + hd), freq, pos, ds, a_re, a_im, vp);
    a_re = IO<T>::rnd(a_re);
    a_im = IO<T>::rnd(a_im);
    vp = IO<T>::rnd(vp);
    const float be = IO<T>::rnd(ds.beta), sc = IO<T>::rnd(ds.sel_c);
    const T* vrow = static_cast<const T*>(a.v) + b * a.v_stride + (long long)hd * a.N + 2 * j;
    float v0 = IO<T>::ld(vrow), v1 = IO<T>::ld(vrow + 1);
    if (a.v_first) {   // value residual across layers (block.py:167-171), rounded like the eager lerp's output
        const T* f = static_cast<const T*>(a.v_first) + bh * a.N + 2 * j;
        const float w = IO<T>::ld(static_cast<const T*>(a.mix) + hd), f0 = IO<T>::ld(f), f1 = IO<T>::ld(f + 1);
        const float d0 = v0 - f0, d1 = v1 - f1;
        v0 = IO<T>::rnd(fabsf(w) < 0.5f ? f0 + w * d0 : v0 - d0 * (1.f - w));
        v1 = IO<T>::rnd(fabsf(w) < 0.5f ? f1 + w * d1 : v1 - d1 * (1.f - w));
    }
    const float vr = IO<T>::rnd(v0 * vp), vi = IO<T>::rnd(v1 * vp);

    float kk[kCols], qq[kCols];
    kraw.get(kk);
    qraw.get(qq);
    normalise<T, kCols>(kk);
    normalise<T, kCols>(qq);
    float ur = 0.f, ui = 0.f;
#pragma unroll
    for (int i = 0; i < kCols; i++) { ur += zr[i] * kk[i]; ui += zi[i] * kk[i]; }
    ur = be * group_sum(ur);
    ui = be * group_sum(ui);
    const float ivr = be * vr, ivi = be * vi;
    float yr = 0.f, yi = 0.f;
#pragma unroll
    for (int i = 0; i < kCols; i++) {
        const float er = zr[i] - ur * kk[i], ei = zi[i] - ui * kk[i];
        zr[i] = a_re * er - a_im * ei + ivr * kk[i];
        zi[i] = a_re * ei + a_im * er + ivi * kk[i];
        yr += zr[i] * qq[i];
        yi += zi[i] * qq[i];
    }
    yr = group_sum(yr);
    yi = group_sum(yi);
    if (a.shortcut_scale != 0.f) {
        float qk = 0.f;
#pragma unroll
        for (int i = 0; i < kCols; i++) qk += qq[i] * kk[i];
        qk = group_sum(qk);
        const float f = a.shortcut_scale * qk * qk;
        yr += f * vr;
        yi += f * vi;
    }
    if (!active) return;
    if (vec) {
#pragma unroll
        for (int i = 0; i < kCols / 4; i++) {
            *reinterpret_cast<float4*>(st + g * kCols + 4 * i) =
                make_float4(zr[4 * i], zr[4 * i + 1], zr[4 * i + 2], zr[4 * i + 3]);
            *reinterpret_cast<float4*>(st + D + g * kCols + 4 * i) =
                make_float4(zi[4 * i], zi[4 * i + 1], zi[4 * i + 2], zi[4 * i + 3]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < kCols; i++) {
            const int d = g * kCols + i;
            if (d < D) { st[d] = zr[i]; st[D + d] = zi[i]; }
        }
    }
    if (g == 0) {
        T* o = static_cast<T*>(a.y) + bh * a.N + 2 * j;
        IO<T>::st(o, IO<T>::rnd(yr) * sc);
        IO<T>::st(o + 1, IO<T>::rnd(yi) * sc);
    }
}

// The decode step that reproduces the reference's CHUNKED scan token by token (its outputs beyond the first
// chunk are not those of the plain recurrence): per (batch, head) the local state z (zero at every chunk start),
// the correction r (starts from the rounded carry, erase + rotate only, read before its step), the carry s
// and the cumulative decay of the current chunk.  Position pos counts from the sequence start; chunks are
// C tokens.  Same thread mapping as decode_step_kernel.
template <typename T, int kCols>
__global__ void __launch_bounds__(kSimtThreads)
decode_step_ref_kernel(const DecodeArgs a) {
    const int g = threadIdx.x % kLanesPerUnit;
    long long u = (long long)blockIdx.x * kUnitsPerBlock + threadIdx.x / kLanesPerUnit;
    const bool active = u < a.units;
    if (!active) u = a.units - 1;
    const int NH = a.N >> 1, D = a.D, H = a.H;
    const int j = (int)(u % NH);
    const int hd = (int)((u / NH) % H);
    const long long b = u / ((long long)NH * H);
    const bool vec = (D == kCols * kLanesPerUnit);
    const long long bh = b * H + hd;

    RowSlice<T, kCols> kraw, qraw;
    kraw.load(static_cast<const T*>(a.k) + bh * D, g, D, vec);
    qraw.load(static_cast<const T*>(a.q) + bh * D, g, D, vec);
    const long long so = (bh * a.N + 2 * j) * D;
    float* st = a.state + so;
    float* ct = a.corr + so;
    float zr[kCols], zi[kCols], rr[kCols], ri[kCols];
    if (vec) {
#pragma unroll
        for (int i = 0; i < kCols / 4; i++) {
            const float4 x = *reinterpret_cast<const float4*>(st + g * kCols + 4 * i);
            const float4 w = *reinterpret_cast<const float4*>(st + D + g * kCols + 4 * i);
            zr[4 * i] = x.x; zr[4 * i + 1] = x.y; zr[4 * i + 2] = x.z; zr[4 * i + 3] = x.w;
            zi[4 * i] = w.x; zi[4 * i + 1] = w.y; zi[4 * i + 2] = w.z; zi[4 * i + 3] = w.w;
            const float4 p = *reinterpret_cast<const float4*>(ct + g * kCols + 4 * i);
            const float4 r = *reinterpret_cast<const float4*>(ct + D + g * kCols + 4 * i);
            rr[4 * i] = p.x; rr[4 * i + 1] = p.y; rr[4 * i + 2] = p.z; rr[4 * i + 3] = p.w;
            ri[4 * i] = r.x; ri[4 * i + 1] = r.y; ri[4 * i + 2] = r.z; ri[4 * i + 3] = r.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < kCols; i++) {
            const int d = g * kCols + i;
            zr[i] = d < D ? st[d] : 0.f;
            zi[i] = d < D ? st[D + d] : 0.f;
            rr[i] = d < D ? ct[d] : 0.f;
            ri[i] = d < D ? ct[D + d] : 0.f;
        }
    }
    // dynamics (every lane of the unit computes the same scalars; dynamics_fused.cu:64-139)
    const T* gr = static_cast<const T*>(a.gate_raw) + b * (long long)((a.N + 5) * H);
    const T* s5 = gr + a.N * H;
    const float freq = a.rope_freqs[hd], pos = (float)(a.pos_dev ? *a.pos_dev : a.pos);
    DynShared ds = dyn_shared<IO<T>::kBf16>(IO<T>::ld(gr + hd), IO<T>::ld(gr + NH * H + hd), IO<T>::ld(s5 + hd),
                              IO<T>::ld(s5 + H + hd), IO<T>::ld(s5 + 2 * H + hd),
                              IO<T>::ld(s5 + 3 * H + hd), IO<T>::ld(s5 + 4 * H + hd),
                              a.log_dt_scale[hd], freq, pos, a.dc);
    float a_re, a_im, vp;
    dyn_pair<IO<T>::kBf16>(IO<T>::ld(gr + j * H + hd), IO<T>::ld(gr + (NH + j) * H + hd), freq, pos, ds, a_re, a_im, vp);
    a_re = IO<T>::rnd(a_re);
    a_im = IO<T>::rnd(a_im);
    vp = IO<T>::rnd(vp);
    const float be = IO<T>::rnd(ds.beta), sc = IO<T>::rnd(ds.sel_c);
    const T* vrow = static_cast<const T*>(a.v) + bh * a.N + 2 * j;
    const float vr = IO<T>::rnd(IO<T>::ld(vrow) * vp), vi = IO<T>::rnd(IO<T>::ld(vrow + 1) * vp);

    float kk[kCols], qq[kCols];
    kraw.get(kk);
    qraw.get(qq);
    normalise<T, kCols>(kk);
    normalise<T, kCols>(qq);
    float ur = 0.f, ui = 0.f, wr = 0.f, wi = 0.f;
#pragma unroll
    for (int i = 0; i < kCols; i++) {
        ur += zr[i] * kk[i]; ui += zi[i] * kk[i];
        wr += rr[i] * kk[i]; wi += ri[i] * kk[i];
    }
    ur = be * group_sum(ur);
    ui = be * group_sum(ui);
    wr = be * group_sum(wr);
    wi = be * group_sum(wi);
    const float ivr = be * vr, ivi = be * vi;
    float yr = 0.f, yi = 0.f;
#pragma unroll
    for (int i = 0; i < kCols; i++) {
        const float er = zr[i] - ur * kk[i], ei = zi[i] - ui * kk[i];
        zr[i] = a_re * er - a_im * ei + ivr * kk[i];
        zi[i] = a_re * ei + a_im * er + ivi * kk[i];
        // the correction is read BEFORE its step (exact_correction.cu:90-94), then erased and rotated
        yr += (zr[i] + rr[i]) * qq[i];
        yi += (zi[i] + ri[i]) * qq[i];
        const float cr = rr[i] - wr * kk[i], ci = ri[i] - wi * kk[i];
        rr[i] = a_re * cr - a_im * ci;
        ri[i] = a_re * ci + a_im * cr;
    }
    yr = group_sum(yr);
    yi = group_sum(yi);
    if (a.shortcut_scale != 0.f) {
        float qk = 0.f;
#pragma unroll
        for (int i = 0; i < kCols; i++) qk += qq[i] * kk[i];
        qk = group_sum(qk);
        const float f = a.shortcut_scale * qk * qk;
        yr += f * vr;
        yi += f * vi;
    }
    if (!active) return;
    // cumulative decay of the chunk; at the chunk's last token the carry takes the (rounded) chunk results, the
    // local state restarts from zero and the correction from the (rounded) carry (inter_chunk_scan.cu:52-84)
    float* gm = a.gamma + bh * a.N + 2 * j;
    const float g0 = gm[0], g1 = gm[1];
    float gr_ = a_re * g0 - a_im * g1, gi_ = a_re * g1 + a_im * g0;
    const int posi = a.pos_dev ? *a.pos_dev : a.pos;
    if (posi % a.C == a.C - 1) {
        float* cy = a.carry + so;
        const float dr = IO<T>::rnd(gr_), di = IO<T>::rnd(gi_);
#pragma unroll
        for (int i = 0; i < kCols; i++) {
            const int d = g * kCols + i;
            if (d < D) {
                const float sr = cy[d], si = cy[D + d];
                const float nr = dr * sr - di * si + IO<T>::rnd(zr[i]), ni = dr * si + di * sr + IO<T>::rnd(zi[i]);
                cy[d] = nr;
                cy[D + d] = ni;
                rr[i] = IO<T>::rnd(nr);
                ri[i] = IO<T>::rnd(ni);
            }
            zr[i] = 0.f;
            zi[i] = 0.f;
        }
        gr_ = 1.f;
        gi_ = 0.f;
    }
    if (g == 0) { gm[0] = gr_; gm[1] = gi_; }
    if (vec) {
#pragma unroll
        for (int i = 0; i < kCols / 4; i++) {
            *reinterpret_cast<float4*>(st + g * kCols + 4 * i) =
                make_float4(zr[4 * i], zr[4 * i + 1], zr[4 * i + 2], zr[4 * i + 3]);
            *reinterpret_cast<float4*>(st + D + g * kCols + 4 * i) =
                make_float4(zi[4 * i], zi[4 * i + 1], zi[4 * i + 2], zi[4 * i + 3]);
            *reinterpret_cast<float4*>(ct + g * kCols + 4 * i) =
                make_float4(rr[4 * i], rr[4 * i + 1], rr[4 * i + 2], rr[4 * i + 3]);
            *reinterpret_cast<float4*>(ct + D + g * kCols + 4 * i) =
                make_float4(ri[4 * i], ri[4 * i + 1], ri[4 * i + 2], ri[4 * i + 3]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < kCols; i++) {
            const int d = g * kCols + i;
            if (d < D) { st[d] = zr[i]; st[D + d] = zi[i]; ct[d] = rr[i]; ct[D + d] = ri[i]; }
        }
    }
    if (g == 0) {
        T* o = static_cast<T*>(a.y) + bh * a.N + 2 * j;
        IO<T>::st(o, IO<T>::rnd(yr) * sc);
        IO<T>::st(o + 1, IO<T>::rnd(yi) * sc);
    }
}

template <typename T, int kCols>
static int launch_decode(const DecodeArgs& a, cudaStream_t st) {
    const unsigned blocks = (unsigned)((a.units + kUnitsPerBlock - 1) / kUnitsPerBlock);
    if (a.corr) decode_step_ref_kernel<T, kCols><<<blocks, kSimtThreads, 0, st>>>(a);
    else decode_step_kernel<T, kCols><<<blocks, kSimtThreads, 0, st>>>(a);
    return check_launch();
}

}  // namespace cdssm

using namespace cdssm;

namespace cdssm {
unsigned long long wait_limit_ns();   // c_abi.cu
// scan_wa.cu
bool scan_wa_supported(int D, int N, int C, int H, int dtype);
size_t scan_wa_record_bytes(int B, int L, int H, int C);
int scan_wa_dynamics(const void* v, const void* gate_raw, const float* log_dt_scale, const float* rope_freqs,
                     void* rec, const DynConsts& dc, int B, int L, int H, int C, int pos0, int segs, int fp32_decay,
                     cudaStream_t st);
int scan_wa_pass(bool output, const void* q, const void* k, const void* rec, float* ws_gamma, float* ws_state, void* y,
                 int* status, float shortcut_scale, int B, int L, int H, int D, unsigned long long wait_ns, int withhold,
                 cudaStream_t st);
}

static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

extern "C" size_t cdssm_b200_scan_fused_workspace_bytes(int B, int L, int H, int D, int N, int C) {
    if (B <= 0 || L <= 0 || H <= 0 || D <= 0 || N <= 0 || (N & 1) || C <= 0) return 0;
    const size_t NC = ((size_t)L + C - 1) / C;
    const size_t units = (size_t)B * NC * H * (N / 2);
    size_t bytes = 256 + align256(units * 2 * sizeof(float)) + align256(units * 2 * D * sizeof(float));
    // per-token records of the four-chain tensor-core kernels (the data type is not known here)
    if (scan_wa_supported(D, N, C, H, CDSSM_BF16)) bytes += align256(scan_wa_record_bytes(B, L, H, C));
    return bytes;
}

extern "C" int cdssm_b200_scan_fused_status(const void* workspace, int* status_host, void* stream) {
    if (!workspace || !status_host) return CDSSM_ERR_BAD_ARG;
    if (int rc = check_cuda(cudaMemcpyAsync(status_host, workspace, sizeof(int), cudaMemcpyDeviceToHost,
                                            (cudaStream_t)stream)))
        return rc;
    if (int rc = check_cuda(cudaStreamSynchronize((cudaStream_t)stream))) return rc;
    return *status_host == 0 ? CDSSM_OK : CDSSM_ERR_TIMEOUT;
}

static int scan_fused_impl(const void* q, const void* k, const void* v, const void* gate_raw,
                           const float* log_dt_scale, const float* rope_freqs, const float* h0, void* y,
                           float* final_state, float* tail_state, float* total_decay, bool summary_only,
                           void* workspace, size_t workspace_bytes, float gating_c, float omega_thresh,
                           float adt_delta, float adt_smoothness, float adt_eps, float shortcut_scale,
                           int B, int L, int H, int D, int N, int C, int pos0, int segs, int dtype,
                           int flags, void* stream) {
    if (summary_only) { q = k; y = nullptr; tail_state = nullptr; }
    if (!q || !k || !v || !gate_raw || !log_dt_scale || !rope_freqs || (!y && !summary_only))
        return CDSSM_ERR_BAD_ARG;
    if (segs < 1 || (B > 0 && B % segs)) return CDSSM_ERR_BAD_ARG;
    if (B < 0 || L < 0 || H <= 0 || D <= 0 || N <= 0 || (N & 1) || C <= 0) return CDSSM_ERR_BAD_ARG;
    if (dtype != CDSSM_BF16 && dtype != CDSSM_F32) return CDSSM_ERR_BAD_ARG;
    if (((uintptr_t)q | (uintptr_t)k) & 15) return CDSSM_ERR_BAD_ARG;   // 16-byte row loads
    if (N > kMaxStateDim || D > kMaxHeadDim || C > kMaxChunk) return CDSSM_ERR_UNSUPPORTED;
    if (B == 0 || L == 0) return CDSSM_OK;
    const size_t need = cdssm_b200_scan_fused_workspace_bytes(B, L, H, D, N, C);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255)) return CDSSM_ERR_WORKSPACE;
    // first 256 bytes of the workspace: status word of the tensor-core kernel's bounded waits
    int* status = static_cast<int*>(workspace);
    if (int rc = check_cuda(cudaMemsetAsync(status, 0, sizeof(int), (cudaStream_t)stream))) return rc;
    workspace = static_cast<char*>(workspace) + 256;
    if ((flags & CDSSM_SCAN_EXACT) && (summary_only || segs != 1)) return CDSSM_ERR_UNSUPPORTED;
    ScanArgs a;
    a.q = q; a.k = k; a.v = v; a.gate_raw = gate_raw;
    a.log_dt_scale = log_dt_scale; a.rope_freqs = rope_freqs; a.h0 = h0;
    a.y = y; a.final_state = final_state; a.tail_state = tail_state;
    a.total_decay = total_decay; a.segs = segs;
    a.run_local = (flags & CDSSM_SCAN_REUSE_LOCAL) ? 0 : 1;
    a.run_output = 1;
    a.publish = summary_only ? 0 : 1;
    a.fp32_decay = (flags & CDSSM_SCAN_FP32_DECAY) ? 1 : 0;
    a.dc = DynConsts{gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps};
    a.shortcut_scale = shortcut_scale;
    a.B = B; a.L = L; a.H = H; a.D = D; a.N = N; a.C = C; a.pos0 = pos0;
    a.NC = (L + C - 1) / C;
    a.units = (long long)B * a.NC * H * (N / 2);
    a.ws_gamma = static_cast<float*>(workspace);
    a.ws_state = reinterpret_cast<float*>(static_cast<char*>(workspace) +
                                          align256((size_t)a.units * 2 * sizeof(float)));
    if (flags & CDSSM_SCAN_EXACT) {
        // the recurrent state after the last token is both the "carry" and the tail state
        const int cols = (D + kLanesPerUnit - 1) / kLanesPerUnit;
        cudaStream_t st = (cudaStream_t)stream;
        float* extra = tail_state;
        if (!a.final_state) { a.final_state = tail_state; extra = nullptr; }
        int rc;
        if (dtype == CDSSM_BF16) rc = cols <= 8 ? launch_recurrent<__nv_bfloat16, 8>(a, st) : launch_recurrent<__nv_bfloat16, 16>(a, st);
        else rc = cols <= 8 ? launch_recurrent<float, 8>(a, st) : launch_recurrent<float, 16>(a, st);
        if (rc == CDSSM_OK && extra && a.final_state)
            rc = check_cuda(cudaMemcpyAsync(extra, a.final_state, sizeof(float) * (size_t)B * H * N * D,
                                            cudaMemcpyDeviceToDevice, st));
        return rc;
    }
    // Warp-autonomous tensor-core passes (scan_wa.cu) for the local and the output pass, with the CUDA-core
    // carry pass between them: the default wherever the shapes allow.  (Bits 256 / 512 keep the CUDA-core
    // local / output pass: used by the tests to check each tensor-core pass alone.)
    // (the tensor-core passes read v and write y as 4-byte pairs: buffers that are only 2-byte aligned, which
    // the contract allows, stay on the CUDA-core kernels)
    const bool pair_aligned = ((((uintptr_t)v) | ((uintptr_t)y)) & 3) == 0;
    const bool wa_ok = tail_state == nullptr && pair_aligned && scan_wa_supported(D, N, C, H, dtype);
    const bool wa_asked = (flags & CDSSM_SCAN_TENSOR_CORE_WA) != 0;
    if (!(flags & CDSSM_SCAN_FORCE_SIMT) && (wa_asked || wa_ok)) {
        if (!wa_ok) return CDSSM_ERR_UNSUPPORTED;
        cudaStream_t st = (cudaStream_t)stream;
        const bool tc_local = !(flags & CDSSM_SCAN_KEEP_SIMT_LOCAL), tc_output = !(flags & CDSSM_SCAN_KEEP_SIMT_OUTPUT);
        const int withhold = (flags & CDSSM_SCAN_TEST_WITHHOLD) ? 1 : 0;
        const unsigned long long limit = wait_limit_ns();
        void* rec = reinterpret_cast<char*>(a.ws_state) + align256((size_t)a.units * 2 * D * sizeof(float));
        if (int rc = scan_wa_dynamics(v, gate_raw, log_dt_scale, rope_freqs, rec, a.dc, B, L, H, C, pos0, segs,
                                      a.fp32_decay, st))
            return rc;
        if (a.run_local && tc_local) {
            if (int rc = scan_wa_pass(false, q, k, rec, a.ws_gamma, a.ws_state, nullptr, status, shortcut_scale, B, L, H,
                                      D, limit, withhold, st))
                return rc;
            a.run_local = 0;
        }
        a.run_output = tc_output ? 0 : 1;
        if (int rc = scan_fused_simt(a, dtype, false, st)) return rc;   // carry pass (+ whatever was kept)
        if (!tc_output || summary_only) return CDSSM_OK;
        return scan_wa_pass(true, q, k, rec, a.ws_gamma, a.ws_state, y, status, shortcut_scale, B, L, H, D, limit,
                            withhold, st);
    }
    return scan_fused_simt(a, dtype, false, (cudaStream_t)stream);
}

static int decode_step_impl(float* state, const void* q, const void* k, const void* v,
                            const void* gate_raw, const float* log_dt_scale, const float* rope_freqs,
                            void* y, float gating_c, float omega_thresh, float adt_delta,
                            float adt_smoothness, float adt_eps, float shortcut_scale, int B, int H, int D,
                            int N, int pos, const int* pos_dev, int dtype, void* stream, float* corr = nullptr,
                            float* carry = nullptr, float* gamma = nullptr, int C = 0, long long k_stride = 0,
                            long long v_stride = 0, const void* v_first = nullptr, const void* mix = nullptr,
                            long long q_stride = 0, long long g_stride = 0) {
    if (!state || !q || !k || !v || !gate_raw || !log_dt_scale || !rope_freqs || !y)
        return CDSSM_ERR_BAD_ARG;
    if (corr && (!carry || !gamma || C <= 0 || (((uintptr_t)corr | (uintptr_t)carry) & 15))) return CDSSM_ERR_BAD_ARG;
    if (B < 0 || H <= 0 || D <= 0 || N <= 0 || (N & 1)) return CDSSM_ERR_BAD_ARG;
    if (dtype != CDSSM_BF16 && dtype != CDSSM_F32) return CDSSM_ERR_BAD_ARG;
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)state) & 15) return CDSSM_ERR_BAD_ARG;
    if (N > kMaxStateDim || D > kMaxHeadDim) return CDSSM_ERR_UNSUPPORTED;
    if (B == 0) return CDSSM_OK;
    DecodeArgs a;
    a.state = state; a.q = q; a.k = k; a.v = v; a.gate_raw = gate_raw;
    a.corr = corr; a.carry = carry; a.gamma = gamma; a.C = C;
    a.k_stride = k_stride ? k_stride : (long long)H * D;
    a.v_stride = v_stride ? v_stride : (long long)H * N;
    a.v_first = v_first; a.mix = mix;
    a.q_stride = q_stride ? q_stride : (long long)H * D;
    a.g_stride = g_stride ? g_stride : (long long)(N + 5) * H;
    {
        const long long es = dtype == CDSSM_F32 ? 4 : 2;
        const bool vec_rows = D == 64 || D == 128;                             // 16-byte row loads of k and q
        if (vec_rows && (((a.k_stride | a.q_stride) * es) & 15)) return CDSSM_ERR_BAD_ARG;
        if (a.q_stride < (long long)H * D || a.g_stride < (long long)(N + 5) * H) return CDSSM_ERR_BAD_ARG;
        if (a.k_stride < (long long)H * D || a.v_stride < (long long)H * N) return CDSSM_ERR_BAD_ARG;
        if ((v_first != nullptr) != (mix != nullptr)) return CDSSM_ERR_BAD_ARG;
        if (corr && (v_first || k_stride || v_stride || q_stride || g_stride)) return CDSSM_ERR_UNSUPPORTED;
    }
    a.log_dt_scale = log_dt_scale; a.rope_freqs = rope_freqs; a.y = y;
    a.dc = DynConsts{gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps};
    a.shortcut_scale = shortcut_scale;
    a.B = B; a.H = H; a.D = D; a.N = N; a.pos = pos; a.pos_dev = pos_dev;
    a.units = (long long)B * H * (N / 2);
    const int cols = (D + kLanesPerUnit - 1) / kLanesPerUnit;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == CDSSM_BF16)
        return cols <= 8 ? launch_decode<__nv_bfloat16, 8>(a, st) : launch_decode<__nv_bfloat16, 16>(a, st);
    return cols <= 8 ? launch_decode<float, 8>(a, st) : launch_decode<float, 16>(a, st);
}

extern "C" int cdssm_b200_scan_fused_fwd(const void* q, const void* k, const void* v,
                                         const void* gate_raw, const float* log_dt_scale,
                                         const float* rope_freqs, const float* h0, void* y,
                                         float* final_state, float* tail_state, void* workspace,
                                         size_t workspace_bytes, float gating_c,
                                         float omega_thresh, float adt_delta, float adt_smoothness,
                                         float adt_eps, float shortcut_scale, int B, int L, int H,
                                         int D, int N, int C, int pos0, int dtype, int flags,
                                         void* stream) {
    return scan_fused_impl(q, k, v, gate_raw, log_dt_scale, rope_freqs, h0, y, final_state, tail_state,
                           nullptr, false, workspace, workspace_bytes, gating_c, omega_thresh, adt_delta,
                           adt_smoothness, adt_eps, shortcut_scale, B, L, H, D, N, C, pos0, 1, dtype, flags,
                           stream);
}

extern "C" int cdssm_b200_scan_fused_segmented_fwd(const void* q, const void* k, const void* v,
                                                   const void* gate_raw, const float* log_dt_scale,
                                                   const float* rope_freqs, const float* h0, void* y,
                                                   float* final_state, void* workspace,
                                                   size_t workspace_bytes, float gating_c,
                                                   float omega_thresh, float adt_delta,
                                                   float adt_smoothness, float adt_eps,
                                                   float shortcut_scale, int B, int L, int H, int D, int N,
                                                   int C, int pos0, int segs, int dtype, int flags,
                                                   void* stream) {
    return scan_fused_impl(q, k, v, gate_raw, log_dt_scale, rope_freqs, h0, y, final_state, nullptr,
                           nullptr, false, workspace, workspace_bytes, gating_c, omega_thresh, adt_delta,
                           adt_smoothness, adt_eps, shortcut_scale, B, L, H, D, N, C, pos0, segs, dtype,
                           flags, stream);
}

extern "C" int cdssm_b200_scan_summary_fwd(const void* k, const void* v, const void* gate_raw,
                                           const float* log_dt_scale, const float* rope_freqs,
                                           const float* h0, float* carry_out, float* total_decay,
                                           void* workspace, size_t workspace_bytes, float gating_c,
                                           float omega_thresh, float adt_delta, float adt_smoothness,
                                           float adt_eps, int B, int L, int H, int D, int N, int C, int pos0,
                                           int segs, int dtype, int flags, void* stream) {
    if (!carry_out || !total_decay) return CDSSM_ERR_BAD_ARG;
    if (flags & ~CDSSM_SCAN_FP32_DECAY) return CDSSM_ERR_BAD_ARG;   // the only option that applies to a summary
    return scan_fused_impl(nullptr, k, v, gate_raw, log_dt_scale, rope_freqs, h0, nullptr, carry_out,
                           nullptr, total_decay, true, workspace, workspace_bytes, gating_c, omega_thresh,
                           adt_delta, adt_smoothness, adt_eps, 0.f, B, L, H, D, N, C, pos0, segs, dtype,
                           flags, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the fused scan.
//
// Some hosts of this library cannot hand it a workspace: an inference server whose memory pool
// already owns every byte of the device, a plugin that runs inside somebody else's framework and
// is not allowed to call the CUDA allocator (cudaMalloc synchronises the whole device and would
// stall the other streams of that process), or an embedding whose allocator is simply not reachable
// from where the scan is called.  For them the scratch of the three-launch scan lives in a
// file-scope device array that the module carries itself: kNoAllocScratchBytes on every GPU that
// loads the library, for as long as the process lives.
//
// In host code the array's name is only a handle for the symbol, not a device pointer; the device
// address is looked up once per device with cudaGetSymbolAddress (with that device current) and it
// is this address that the kernels receive.
constexpr size_t kNoAllocScratchBytes = 16u << 20;   // 16 MiB
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
constexpr int kNoAllocMaxDevices = 64;
static std::atomic<void*> g_noalloc_scratch_of_device[kNoAllocMaxDevices];   // device address of the array, per device

extern "C" size_t cdssm_b200_scan_fused_noalloc_max_bytes(void) { return kNoAllocScratchBytes; }

extern "C" int cdssm_b200_scan_fused_fwd_noalloc(const void* q, const void* k, const void* v,
                                                 const void* gate_raw, const float* log_dt_scale,
                                                 const float* rope_freqs, const float* h0, void* y,
                                                 float* final_state, float* tail_state, float gating_c,
                                                 float omega_thresh, float adt_delta,
                                                 float adt_smoothness, float adt_eps,
                                                 float shortcut_scale, int B, int L, int H, int D, int N,
                                                 int C, int pos0, int dtype, int flags, void* stream) {
    if (B <= 0 || L <= 0) {   // nothing to do, but still validate like the allocating entry point
        return cdssm_b200_scan_fused_fwd(q, k, v, gate_raw, log_dt_scale, rope_freqs, h0, y, final_state,
                                         tail_state, nullptr, 0, gating_c, omega_thresh, adt_delta,
                                         adt_smoothness, adt_eps, shortcut_scale, B, L, H, D, N, C, pos0,
                                         dtype, flags, stream);
    }
    const size_t need = cdssm_b200_scan_fused_workspace_bytes(B, L, H, D, N, C);
    if (need == 0) return CDSSM_ERR_BAD_ARG;
    if (need > kNoAllocScratchBytes) return CDSSM_ERR_WORKSPACE;   // beyond the built-in scratch
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev))) return rc;
    if (dev < 0 || dev >= kNoAllocMaxDevices) return CDSSM_ERR_UNSUPPORTED;
    void* scratch = g_noalloc_scratch_of_device[dev].load(std::memory_order_acquire);
    if (scratch == nullptr) {
        // one-time set-up for this device (do it before any stream capture begins); two host threads that
        // race here both look up the same address
        if (int rc = check_cuda(cudaGetSymbolAddress(&scratch, g_noalloc_scratch))) return rc;
        g_noalloc_scratch_of_device[dev].store(scratch, std::memory_order_release);
    }
    // Nothing in the scratch has to start at zero except the status word, which the scan itself
    // clears on the stream; gamma/state slots are all written by the local pass before they are read.
    return cdssm_b200_scan_fused_fwd(q, k, v, gate_raw, log_dt_scale, rope_freqs, h0, y, final_state,
                                     tail_state, scratch, kNoAllocScratchBytes, gating_c,
                                     omega_thresh, adt_delta, adt_smoothness, adt_eps, shortcut_scale, B, L,
                                     H, D, N, C, pos0, dtype, flags, stream);
}

extern "C" int cdssm_b200_scan_fused_noalloc_status(int* status_host, void* stream) {
    if (!status_host) return CDSSM_ERR_BAD_ARG;
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev))) return rc;
    if (dev < 0 || dev >= kNoAllocMaxDevices) return CDSSM_ERR_UNSUPPORTED;
    void* p = g_noalloc_scratch_of_device[dev].load(std::memory_order_acquire);
    if (!p) return CDSSM_ERR_BAD_ARG;   // no allocation-free call has run on this device yet
    return cdssm_b200_scan_fused_status(p, status_host, stream);
}

extern "C" int cdssm_b200_decode_step(float* state, const void* q, const void* k, const void* v,
                                      const void* gate_raw, const float* log_dt_scale,
                                      const float* rope_freqs, void* y, float gating_c,
                                      float omega_thresh, float adt_delta, float adt_smoothness,
                                      float adt_eps, float shortcut_scale, int B, int H, int D,
                                      int N, int pos, int dtype, void* stream) {
    return decode_step_impl(state, q, k, v, gate_raw, log_dt_scale, rope_freqs, y, gating_c, omega_thresh,
                            adt_delta, adt_smoothness, adt_eps, shortcut_scale, B, H, D, N, pos, nullptr,
                            dtype, stream);
}

extern "C" int cdssm_b200_decode_step_at(float* state, const void* q, const void* k, const void* v,
                                         const void* gate_raw, const float* log_dt_scale,
                                         const float* rope_freqs, void* y, float gating_c,
                                         float omega_thresh, float adt_delta, float adt_smoothness,
                                         float adt_eps, float shortcut_scale, int B, int H, int D, int N,
                                         const int* pos_dev, int dtype, void* stream) {
    if (!pos_dev) return CDSSM_ERR_BAD_ARG;
    return decode_step_impl(state, q, k, v, gate_raw, log_dt_scale, rope_freqs, y, gating_c, omega_thresh,
                            adt_delta, adt_smoothness, adt_eps, shortcut_scale, B, H, D, N, 0, pos_dev,
                            dtype, stream);
}

extern "C" int cdssm_b200_decode_step_strided(float* state, const void* q, int64_t q_row_stride, const void* k,
                                              int64_t k_row_stride, const void* v, int64_t v_row_stride,
                                              const void* v_first, const void* mix, const void* gate_raw,
                                              int64_t gate_row_stride, const float* log_dt_scale,
                                              const float* rope_freqs, void* y, float gating_c, float omega_thresh,
                                              float adt_delta, float adt_smoothness, float adt_eps,
                                              float shortcut_scale, int B, int H, int D, int N, int pos,
                                              const int* pos_dev, int dtype, void* stream) {
    if (k_row_stride <= 0 || v_row_stride <= 0 || q_row_stride <= 0 || gate_row_stride <= 0) return CDSSM_ERR_BAD_ARG;
    return decode_step_impl(state, q, k, v, gate_raw, log_dt_scale, rope_freqs, y, gating_c, omega_thresh,
                            adt_delta, adt_smoothness, adt_eps, shortcut_scale, B, H, D, N, pos, pos_dev, dtype,
                            stream, nullptr, nullptr, nullptr, 0, k_row_stride, v_row_stride, v_first, mix, q_row_stride,
                            gate_row_stride);
}

extern "C" int cdssm_b200_decode_step_reference(float* local_state, float* correction, float* carry, float* chunk_decay,
                                                const void* q, const void* k, const void* v, const void* gate_raw,
                                                const float* log_dt_scale, const float* rope_freqs, void* y,
                                                float gating_c, float omega_thresh, float adt_delta,
                                                float adt_smoothness, float adt_eps, float shortcut_scale, int B,
                                                int H, int D, int N, int C, int pos, const int* pos_dev, int dtype,
                                                void* stream) {
    if (!correction || !carry || !chunk_decay || C <= 0 || pos < 0) return CDSSM_ERR_BAD_ARG;
    return decode_step_impl(local_state, q, k, v, gate_raw, log_dt_scale, rope_freqs, y, gating_c, omega_thresh,
                            adt_delta, adt_smoothness, adt_eps, shortcut_scale, B, H, D, N, pos, pos_dev, dtype,
                            stream, correction, carry, chunk_decay, C);
}
