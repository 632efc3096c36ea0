// The memory-bound steps either side of the scan inside a CD-SSM block, one kernel each instead of the
// handful of elementwise kernels an eager framework launches for them:
//   RMSNorm                                   cdssm/models/modules.py:37-53
//   GroupNorm -> * silu(z) -> + D * x_conv    cdssm/models/block.py:213-224
//   one-token depthwise conv + SiLU on a cached three-row history (the decode-time form of conv1d_silu.cu:25-90)
// Arithmetic in fp32; with bf16 storage every intermediate is rounded where the reference's eager bf16
// operations round it, so the fused result equals the unfused one bit for bit except for the reduction order
// of the statistics.
#include "cdssm_common.cuh"

namespace cdssm {

// ---------------------------------------------------------------- RMSNorm
// One warp per row: out = rnd(rnd(x * rsqrt(mean x^2 + eps)) * w)   (modules.py:50-53)
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out, long long rows, int d,
                   float eps) {
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const T* xr = x + row * d;
    float ss = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
        float f[8];
        Vec8<T>::ld(xr + c, f);
#pragma unroll
        for (int e = 0; e < 8; e++) ss += f[e] * f[e];
    }
    const float rms = rsqrtf(warp_sum(ss) / (float)d + eps);
    T* orow = out + row * d;
    for (int c = lane * 8; c < d; c += 256) {
        float f[8], g[8];
        Vec8<T>::ld(xr + c, f);
        Vec8<T>::ld(w + c, g);
#pragma unroll
        for (int e = 0; e < 8; e++) f[e] = IO<T>::rnd(f[e] * rms) * g[e];
        Vec8<T>::st(orow + c, f);
    }
}

// Few rows (a decode step: one row per sequence): one block per row, so that a row's loads are spread over 256
// threads instead of one warp's dependent loop.  Same arithmetic; the sum of squares is reduced in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_row_block_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out, int d, float eps) {
    const T* xr = x + (long long)blockIdx.x * d;
    T* orow = out + (long long)blockIdx.x * d;
    __shared__ float sh[8];
    float ss = 0.f;
    for (int c = threadIdx.x * 8; c < d; c += 2048) {
        float f[8];
        Vec8<T>::ld(xr + c, f);
#pragma unroll
        for (int e = 0; e < 8; e++) ss += f[e] * f[e];
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += sh[i];
    const float rms = rsqrtf(tot / (float)d + eps);
    for (int c = threadIdx.x * 8; c < d; c += 2048) {
        float f[8], g[8];
        Vec8<T>::ld(xr + c, f);
        Vec8<T>::ld(w + c, g);
#pragma unroll
        for (int e = 0; e < 8; e++) f[e] = IO<T>::rnd(f[e] * rms) * g[e];
        Vec8<T>::st(orow + c, f);
    }
}

// ---------------------------------------------------------------- GroupNorm statistics over a whole sequence
// The reference normalises (B, d_inner, L): each group's statistics run over its channels AND all positions
// (block.py:216-222).  Two stages, both with a fixed summation order (deterministic): blocks of di / 8 threads
// read whole rows (coalesced 16-byte vectors, thread = eight channels) of a tile of positions and leave the
// tile's (sum, sum of squares) per group; a second, tiny launch adds the tiles in double precision.
constexpr int kGnTileRows = 32;
constexpr int kGnMaxTiles = 512;
static int gn_tiles(int L) {
    const int t = (L + kGnTileRows - 1) / kGnTileRows;
    return t < 1 ? 1 : (t > kGnMaxTiles ? kGnMaxTiles : t);
}

template <typename T>
__global__ void __launch_bounds__(1024)
groupnorm_partial_kernel(const T* __restrict__ y, float* __restrict__ partial, int L, int di, int groups, int tiles) {
    const int b = blockIdx.x / tiles, tile = blockIdx.x % tiles;
    const int rows = (L + tiles - 1) / tiles;
    const int l0 = tile * rows, l1 = min(L, l0 + rows);
    const int cg = di / groups, tpg = cg / 8;
    const T* base = y + ((long long)b * L) * di + threadIdx.x * 8;
    float s = 0.f, q = 0.f;
    for (int l = l0; l < l1; l++) {
        float f[8];
        Vec8<T>::ld(base + (long long)l * di, f);
#pragma unroll
        for (int e = 0; e < 8; e++) { s += f[e]; q = fmaf(f[e], f[e], q); }
    }
    __shared__ float sh[2][1024];
    sh[0][threadIdx.x] = s;
    sh[1][threadIdx.x] = q;
    __syncthreads();
    if ((int)threadIdx.x < groups) {
        float ts = 0.f, tq = 0.f;
        for (int i = 0; i < tpg; i++) { ts += sh[0][threadIdx.x * tpg + i]; tq += sh[1][threadIdx.x * tpg + i]; }
        float* o = partial + (((long long)b * tiles + tile) * groups + threadIdx.x) * 2;
        o[0] = ts;
        o[1] = tq;
    }
}

__global__ void __launch_bounds__(128)
groupnorm_finalize_kernel(const float* __restrict__ partial, float* __restrict__ stats, int total, int L, int cg,
                          int groups, int tiles, float eps) {
    const int i = blockIdx.x * 4 + (threadIdx.x >> 5);     // (batch row, group): one warp each
    if (i >= total) return;
    const int lane = threadIdx.x & 31;
    const int b = i / groups, grp = i % groups;
    double s = 0.0, q = 0.0;
    for (int t = lane; t < tiles; t += 32) {               // lane-strided, then a fixed shuffle tree: deterministic
        const float* p = partial + (((long long)b * tiles + t) * groups + grp) * 2;
        s += (double)p[0];
        q += (double)p[1];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o);
        q += __shfl_xor_sync(0xffffffffu, q, o);
    }
    if (lane == 0) {
        const double n = (double)L * cg, mean = s / n;
        const double var = fmax(q / n - mean * mean, 0.0);
        stats[2 * i] = (float)mean;
        stats[2 * i + 1] = (float)(1.0 / sqrt(var + (double)eps));
    }
}

// ---------------------------------------------------------------- GroupNorm + gate + skip
// One block per token, one thread per eight channels.  stats == NULL: statistics per token and group (the
// causal form used with a decode cache); otherwise mean / rstd of the token's (batch row, group) from
// groupnorm_stats_kernel.  out = rnd(rnd(rnd(GN(y)) * rnd(silu(z))) + rnd(D * x_conv))   (block.py:216-224)
template <typename T>
__global__ void __launch_bounds__(1024)
groupnorm_gate_fwd_kernel(const T* __restrict__ y, const float* __restrict__ stats, const T* __restrict__ gn_w,
                          const T* __restrict__ gn_b, const T* __restrict__ z, long long z_row_stride,
                          const T* __restrict__ skip, const T* __restrict__ x_conv, T* __restrict__ out, int L,
                          int di, int groups, float eps) {
    const long long row = blockIdx.x;
    const int c = threadIdx.x * 8;
    const int cg = di / groups, tpg = cg / 8;          // threads per group
    const int grp = threadIdx.x / tpg;
    float f[8];
    Vec8<T>::ld(y + row * di + c, f);
    float mean, rstd;
    if (stats == nullptr) {
        __shared__ float sh[2][1024];
        float ps = 0.f, pq = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) { ps += f[e]; pq += f[e] * f[e]; }
        sh[0][threadIdx.x] = ps;
        sh[1][threadIdx.x] = pq;
        __syncthreads();
        float s = 0.f, q = 0.f;
        for (int i = 0; i < tpg; i++) { s += sh[0][grp * tpg + i]; q += sh[1][grp * tpg + i]; }
        mean = s / (float)cg;
        rstd = rsqrtf(fmaxf(q / (float)cg - mean * mean, 0.f) + eps);
    } else {
        const long long b = row / L;
        mean = stats[2 * (b * groups + grp)];
        rstd = stats[2 * (b * groups + grp) + 1];
    }
    float gw[8], gb[8], zz[8], sk[8], xc[8];
    Vec8<T>::ld(gn_w + c, gw);
    Vec8<T>::ld(gn_b + c, gb);
    Vec8<T>::ld(z + row * z_row_stride + c, zz);
    Vec8<T>::ld(skip + c, sk);
    Vec8<T>::ld(x_conv + row * di + c, xc);
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const float n = IO<T>::rnd((f[e] - mean) * rstd * gw[e] + gb[e]);
        const float g = IO<T>::rnd(siluf_<IO<T>::kBf16>(zz[e]));
        f[e] = IO<T>::rnd(n * g) + IO<T>::rnd(sk[e] * xc[e]);
    }
    Vec8<T>::st(out + row * di + c, f);
}

// The same with statistics given, kRows tokens per block: the per-channel parameters are loaded once and the
// loads of all rows are in flight together.
template <typename T, int kRows>
__global__ void __launch_bounds__(1024)
groupnorm_gate_rows_kernel(const T* __restrict__ y, const float* __restrict__ stats, const T* __restrict__ gn_w,
                           const T* __restrict__ gn_b, const T* __restrict__ z, long long z_row_stride,
                           const T* __restrict__ skip, const T* __restrict__ x_conv, T* __restrict__ out,
                           long long rows, int L, int di, int groups) {
    const long long r0 = (long long)blockIdx.x * kRows;
    const int c = threadIdx.x * 8;
    const int grp = threadIdx.x / ((di / groups) / 8);
    float f[kRows][8], zz[kRows][8], xc[kRows][8], mean[kRows], rstd[kRows];
#pragma unroll
    for (int r = 0; r < kRows; r++) {
        const long long row = r0 + r < rows ? r0 + r : rows - 1;
        Vec8<T>::ld(y + row * di + c, f[r]);
        Vec8<T>::ld(z + row * z_row_stride + c, zz[r]);
        Vec8<T>::ld(x_conv + row * di + c, xc[r]);
        const long long b = row / L;
        mean[r] = stats[2 * (b * groups + grp)];
        rstd[r] = stats[2 * (b * groups + grp) + 1];
    }
    float gw[8], gb[8], sk[8];
    Vec8<T>::ld(gn_w + c, gw);
    Vec8<T>::ld(gn_b + c, gb);
    Vec8<T>::ld(skip + c, sk);
#pragma unroll
    for (int r = 0; r < kRows; r++) {
        if (r0 + r >= rows) break;
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float n = IO<T>::rnd((f[r][e] - mean[r]) * rstd[r] * gw[e] + gb[e]);
            const float g = IO<T>::rnd(siluf_<IO<T>::kBf16>(zz[r][e]));
            f[r][e] = IO<T>::rnd(n * g) + IO<T>::rnd(sk[e] * xc[r][e]);
        }
        Vec8<T>::st(out + (r0 + r) * di + c, f[r]);
    }
}

// ---------------------------------------------------------------- one-token conv + SiLU on a cached history
// hist (B,3,Dm): the last three inputs of the causal 4-tap depthwise conv, updated in place.
template <typename T>
__global__ void __launch_bounds__(256)
conv1d_silu_step_kernel(const T* __restrict__ x, long long x_row_stride, T* __restrict__ hist,
                        const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ out, int B, int Dm) {
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= (long long)B * Dm) return;
    const int d = (int)(idx % Dm);
    const long long b = idx / Dm;
    T* h = hist + b * 3 * Dm + d;
    const float x0 = IO<T>::ld(h), x1 = IO<T>::ld(h + Dm), x2 = IO<T>::ld(h + 2 * Dm);
    const float x3 = IO<T>::ld(x + b * x_row_stride + d);
    const float yv = IO<T>::ld(w + d * 4) * x0 + IO<T>::ld(w + d * 4 + 1) * x1 + IO<T>::ld(w + d * 4 + 2) * x2 +
                     IO<T>::ld(w + d * 4 + 3) * x3 + IO<T>::ld(bias + d);
    IO<T>::st(out + b * Dm + d, siluf_<IO<T>::kBf16>(yv));
    IO<T>::st(h, x1);
    IO<T>::st(h + Dm, x2);
    IO<T>::st(h + 2 * Dm, x3);
}

// Eight channels per thread (16-byte accesses of x, the history rows and the output; the 4 taps of a channel are
// 8 contiguous bytes of the (Dm,1,4) weight).
template <typename T>
__global__ void __launch_bounds__(256)
conv1d_silu_step_vec_kernel(const T* __restrict__ x, long long x_row_stride, T* __restrict__ hist,
                            const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ out, int B, int Dm) {
    const int v8 = Dm / 8;
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= (long long)B * v8) return;
    const int d = (int)(idx % v8) * 8;
    const long long b = idx / v8;
    T* h = hist + b * 3 * Dm + d;
    float x0[8], x1[8], x2[8], x3[8], bi[8], wa[8], wb[8], wc[8], wd[8], y[8];
    Vec8<T>::ld(h, x0);
    Vec8<T>::ld(h + Dm, x1);
    Vec8<T>::ld(h + 2 * Dm, x2);
    Vec8<T>::ld(x + b * x_row_stride + d, x3);
    Vec8<T>::ld(bias + d, bi);
    Vec8<T>::ld(w + d * 4, wa);          // taps of channels d, d + 1
    Vec8<T>::ld(w + d * 4 + 8, wb);      // d + 2, d + 3
    Vec8<T>::ld(w + d * 4 + 16, wc);
    Vec8<T>::ld(w + d * 4 + 24, wd);
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const float* ww = (e < 2 ? wa : e < 4 ? wb : e < 6 ? wc : wd) + (e & 1) * 4;
        y[e] = siluf_<IO<T>::kBf16>(ww[0] * x0[e] + ww[1] * x1[e] + ww[2] * x2[e] + ww[3] * x3[e] + bi[e]);
    }
    Vec8<T>::st(out + b * Dm + d, y);
    Vec8<T>::st(h, x1);
    Vec8<T>::st(h + Dm, x2);
    Vec8<T>::st(h + 2 * Dm, x3);
}

}  // namespace cdssm

using namespace cdssm;

#define DISPATCH_DTYPE(dtype, ...)                                 \
    if ((dtype) == CDSSM_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else if ((dtype) == CDSSM_F32) { using T = float; __VA_ARGS__; }     \
    else return CDSSM_ERR_BAD_ARG;

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int cdssm_b200_rmsnorm_fwd(const void* x, const void* weight, void* out, int64_t rows, int d, float eps,
                                      int dtype, void* stream) {
    if (!x || !weight || !out || rows < 0 || d <= 0) return CDSSM_ERR_BAD_ARG;
    if (d % 8 || !aligned16(x) || !aligned16(weight) || !aligned16(out)) return CDSSM_ERR_UNSUPPORTED;
    if (rows == 0) return CDSSM_OK;
    if (rows <= 2048) {   // one block per row
        DISPATCH_DTYPE(dtype, (rmsnorm_row_block_kernel<T><<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
                                  (const T*)x, (const T*)weight, (T*)out, d, eps)));
        return check_launch();
    }
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    DISPATCH_DTYPE(dtype, (rmsnorm_fwd_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>(
                              (const T*)x, (const T*)weight, (T*)out, rows, d, eps)));
    return check_launch();
}

static int check_gn(int di, int groups) {
    if (di <= 0 || groups <= 0 || di % groups) return CDSSM_ERR_BAD_ARG;
    if ((di / groups) % 8 || di / 8 > 1024) return CDSSM_ERR_UNSUPPORTED;
    return CDSSM_OK;
}

extern "C" size_t cdssm_b200_groupnorm_stats_floats(int B, int L, int groups) {
    if (B <= 0 || L <= 0 || groups <= 0) return 0;
    return (size_t)B * groups * 2 * (size_t)(1 + gn_tiles(L));
}

extern "C" int cdssm_b200_groupnorm_stats(const void* y, float* stats, int B, int L, int di, int groups, float eps,
                                          int dtype, void* stream) {
    if (!y || !stats || B < 0 || L < 0) return CDSSM_ERR_BAD_ARG;
    if (int rc = check_gn(di, groups)) return rc;
    if (!aligned16(y) || groups > di / 8) return CDSSM_ERR_UNSUPPORTED;
    if (B == 0 || L == 0) return CDSSM_OK;
    const int tiles = gn_tiles(L);
    float* partial = stats + (size_t)B * groups * 2;       // the tiles' sums live behind the results
    DISPATCH_DTYPE(dtype, (groupnorm_partial_kernel<T><<<(unsigned)(B * tiles), di / 8, 0, (cudaStream_t)stream>>>(
                              (const T*)y, partial, L, di, groups, tiles)));
    if (int rc = check_launch()) return rc;
    const int total = B * groups;
    groupnorm_finalize_kernel<<<(unsigned)((total + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
        partial, stats, total, L, di / groups, groups, tiles, eps);
    return check_launch();
}

extern "C" int cdssm_b200_groupnorm_gate_fwd(const void* y, const float* stats, const void* gn_weight,
                                             const void* gn_bias, const void* z, int64_t z_row_stride,
                                             const void* skip, const void* x_conv, void* out, int B, int L, int di,
                                             int groups, float eps, int dtype, void* stream) {
    if (!y || !gn_weight || !gn_bias || !z || !skip || !x_conv || !out || B < 0 || L < 0) return CDSSM_ERR_BAD_ARG;
    if (int rc = check_gn(di, groups)) return rc;
    const size_t es = dtype == CDSSM_F32 ? 4 : 2;
    if (!aligned16(y) || !aligned16(z) || !aligned16(x_conv) || !aligned16(out) || !aligned16(gn_weight) ||
        !aligned16(gn_bias) || !aligned16(skip) || (z_row_stride * es) % 16)
        return CDSSM_ERR_UNSUPPORTED;
    const long long rows = (long long)B * L;
    if (rows == 0) return CDSSM_OK;
    if (rows > 0x7fffffffLL) return CDSSM_ERR_UNSUPPORTED;
    if (stats != nullptr && rows >= 4096) {
        constexpr int kRows = 4;
        DISPATCH_DTYPE(dtype, (groupnorm_gate_rows_kernel<T, kRows><<<(unsigned)((rows + kRows - 1) / kRows), di / 8, 0,
                                                                      (cudaStream_t)stream>>>(
                                  (const T*)y, stats, (const T*)gn_weight, (const T*)gn_bias, (const T*)z, z_row_stride,
                                  (const T*)skip, (const T*)x_conv, (T*)out, rows, L, di, groups)));
        return check_launch();
    }
    DISPATCH_DTYPE(dtype, (groupnorm_gate_fwd_kernel<T><<<(unsigned)rows, di / 8, 0, (cudaStream_t)stream>>>(
                              (const T*)y, stats, (const T*)gn_weight, (const T*)gn_bias, (const T*)z, z_row_stride,
                              (const T*)skip, (const T*)x_conv, (T*)out, L, di, groups, eps)));
    return check_launch();
}

extern "C" int cdssm_b200_conv1d_silu_step(const void* x, int64_t x_row_stride, void* hist, const void* weight,
                                           const void* bias, void* out, int B, int Dm, int dtype, void* stream) {
    if (!x || !hist || !weight || !bias || !out || B < 0 || Dm <= 0) return CDSSM_ERR_BAD_ARG;
    if (B == 0) return CDSSM_OK;
    const size_t es = dtype == CDSSM_F32 ? 4 : 2;
    if (Dm % 8 == 0 && aligned16(x) && aligned16(hist) && aligned16(weight) && aligned16(bias) && aligned16(out) &&
        (x_row_stride * es) % 16 == 0) {
        const long long nv = (long long)B * (Dm / 8);
        DISPATCH_DTYPE(dtype, (conv1d_silu_step_vec_kernel<T><<<(unsigned)((nv + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
                                  (const T*)x, x_row_stride, (T*)hist, (const T*)weight, (const T*)bias, (T*)out, B, Dm)));
        return check_launch();
    }
    const long long n = (long long)B * Dm;
    DISPATCH_DTYPE(dtype, (conv1d_silu_step_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
                              (const T*)x, x_row_stride, (T*)hist, (const T*)weight, (const T*)bias, (T*)out, B, Dm)));
    return check_launch();
}
