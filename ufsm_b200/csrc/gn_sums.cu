/* GroupNorm statistics of MX tensors: lp_gn_sums_mx (src/nn_lp.h:175) and the finalise step (src/nn_elem.cu:5-11).

   A sum lives in a slot of three 64-bit words.  The slot is a data format of the reference interface, written by these entry points and
   read by the caller's other kernels (src/gnacc.cuh:9-27), so its meaning is the reference's: words 0 and 1 are one 128-bit two's
   complement integer in units of 2^-64 (word 0 the low half, i.e. the fraction; word 1 the whole part), word 2 counts contributions that
   were not finite or reached 2^62, after which the sum reads as NaN.  Blocks add into it with integer atomics, so the words do not
   depend on the order in which blocks finish.

   Inside a block the sums are exact as well, for any realistic tensor.  A lane owns eight channels of its rows (mx_rows.cuh).  Where these
   lie in one group (C / G a multiple of 8) it adds the row's eight codes in fp32, which is exact: MX-fp8 codes are multiples of 2^-9 below
   2^9, so the partial sums need 21 bits; the squares of the codes go through fp64 fma, and one fp64 fma per row and sum applies the row's power-of-two scale (squared for the squares).  Otherwise it keeps fp64 sums per channel.  Lanes, then warps, are combined in fp64. */
#include "mx_rows.cuh"

namespace {

/* v, rounded down to a multiple of 2^-64, added to slot i */
__device__ __forceinline__ void slot_add(double *base, size_t i, double v) {
    unsigned long long *w = (unsigned long long *)base + 3 * i;
    const unsigned long long bits = (unsigned long long)__double_as_longlong(v);
    const int ex = (int)((bits >> 52) & 0x7ffu);
    if (ex >= 1023 + 62) { atomicAdd(&w[2], 1ull); return; }                  /* NaN, inf, or 2^62 and beyond */
    if (ex == 0) return;                                                       /* zero (fp64 subnormals are below 2^-64) */
    /* |v| = m 2^(ex - 1075) = m 2^sh units of 2^-64, m the 53-bit significand */
    const unsigned long long m = (bits & 0xfffffffffffffull) | (1ull << 52);
    const int sh = ex - 1075 + 64;
    unsigned long long lo, hi; bool cut = false;
    if (sh >= 64) { lo = 0ull; hi = m << (sh - 64); }
    else if (sh > 0) { lo = m << sh; hi = m >> (64 - sh); }
    else if (sh > -53) { lo = m >> -sh; hi = 0ull; cut = (m & ((1ull << -sh) - 1ull)) != 0ull; }
    else { lo = 0ull; hi = 0ull; cut = true; }
    if (bits >> 63) {                                                          /* negative: round away from zero, then negate */
        if (cut) { lo++; if (!lo) hi++; }
        lo = ~lo + 1ull; hi = ~hi + (lo == 0ull ? 1ull : 0ull);
    }
    if (lo) { const unsigned long long old = atomicAdd(&w[0], lo); if (old + lo < old) hi++; }
    if (hi) atomicAdd(&w[1], hi);
}
__device__ __forceinline__ double slot_get(const double *base, size_t i) {
    const unsigned long long *w = (const unsigned long long *)base + 3 * i;
    if (w[2]) return __longlong_as_double(0x7ff8000000000000ll);
    return __ll2double_rn((long long)w[1]) + __ull2double_rn(w[0]) * 5.42101086242752217e-20;     /* 2^-64 */
}

/* block = (run of voxels, 32-channel block, sample); ONE: a lane's eight channels share a group */
template <int BITS, bool ONE>
__global__ void __launch_bounds__(256) gn_sums_rows_k(const uint8_t *__restrict__ x, int N, int C, int G, size_t S, double *sums, size_t v0, size_t v1, int n0) {
    const int nb = (C + 31) / 32, blk = blockIdx.y, n = n0 + (int)blockIdx.z, q = threadIdx.x & 3, ph = threadIdx.x >> 2, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int RB = BITS == 8 ? 32 : 16, NA = ONE ? 1 : 8;
    size_t q0 = S * blockIdx.x / gridDim.x, q1 = S * (blockIdx.x + 1) / gridDim.x;
    if (q0 < v0) q0 = v0;
    if (q1 > v1) q1 = v1;
    const uint8_t *xs = x + (size_t)N * nb * S * RB;
    const size_t rbase = ((size_t)n * nb + blk) * S;
    double s1[NA], s2[NA];
#pragma unroll
    for (int k = 0; k < NA; k++) { s1[k] = 0.0; s2[k] = 0.0; }
    for (size_t vb = q0; vb < q1; vb += 256) {
        uint2 raw[4]; unsigned sb[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const size_t v = vb + u * 64 + ph;
            raw[u] = make_uint2(0u, 0u); sb[u] = 127u;             /* rows past the end count as zeros */
            if (v < q1) { raw[u] = qrow_ld<BITS>(x, rbase + v, q); sb[u] = __ldg(xs + rbase + v); }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            float2 r[4];
            if (ONE) {
                qrow_dec<BITS>(raw[u], 1.f, r);                   /* the bare codes */
                const float2 h01 = __fadd2_rn(r[0], r[1]), h23 = __fadd2_rn(r[2], r[3]), h = __fadd2_rn(h01, h23);
                const float t1 = h.x + h.y;
                double t2 = 0.0;
#pragma unroll
                for (int j = 0; j < 4; j++) { const double px = (double)r[j].x, py = (double)r[j].y; t2 = fma(px, px, t2); t2 = fma(py, py, t2); }
                const double f = (double)mx_scale(sb[u]);
                s1[0] = fma((double)t1, f, s1[0]); s2[0] = fma(t2, f * f, s2[0]);
            } else {
                qrow_dec<BITS>(raw[u], mx_scale(sb[u]), r);
#pragma unroll
                for (int k = 0; k < 8; k++) { const double p = (double)((k & 1) ? r[k >> 1].y : r[k >> 1].x); s1[k] += p; s2[k] = fma(p, p, s2[k]); }
            }
        }
    }
    /* lanes of equal q (same channels), then the eight warps */
    __shared__ double w1[8][4][NA], w2[8][4][NA];
#pragma unroll
    for (int k = 0; k < NA; k++) {
        double a = s1[k], b = s2[k];
#pragma unroll
        for (int o = 16; o >= 4; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
        if (lane < 4) { w1[warp][q][k] = a; w2[warp][q][k] = b; }
    }
    __syncthreads();
    if (threadIdx.x < 4 * NA) {
        const int qq = threadIdx.x / NA, k = threadIdx.x % NA, ch = blk * 32 + qq * 8 + (ONE ? 0 : k);
        if (ch < C) {
            double a = 0.0, b = 0.0;
#pragma unroll
            for (int w = 0; w < 8; w++) { a += w1[w][qq][k]; b += w2[w][qq][k]; }
            const size_t o = 2 * ((size_t)n * G + ch / (C / G));
            slot_add(sums, o, a); slot_add(sums, o + 1, b);
        }
    }
}

/* the same sums of a plane-major fp32 tensor [N][C][S] (a conv's unrounded accumulators): block = (run of voxels, channel, sample); fp64 sums
   (a square of an fp32 value is exact in fp64), a fixed-order reduction in the block, one slot addition per sum */
__global__ void __launch_bounds__(256) gn_sums_pm32_k(const float *__restrict__ x, int C, int G, size_t S, double *sums, size_t v0, size_t v1) {
    const int c = blockIdx.y, n = blockIdx.z;
    size_t q0 = S * blockIdx.x / gridDim.x, q1 = S * (blockIdx.x + 1) / gridDim.x;
    if (q0 < v0) q0 = v0;
    if (q1 > v1) q1 = v1;
    const float *p = x + ((size_t)n * C + c) * S;
    double a = 0.0, b = 0.0;
    for (size_t v = q0 + threadIdx.x; v < q1; v += 256) { const double t = (double)__ldg(p + v); a += t; b = fma(t, t, b); }
    __shared__ double sa[256], sb[256];
    sa[threadIdx.x] = a; sb[threadIdx.x] = b;
    __syncthreads();
    for (int h = 128; h > 0; h >>= 1) {
        if ((int)threadIdx.x < h) { sa[threadIdx.x] += sa[threadIdx.x + h]; sb[threadIdx.x] += sb[threadIdx.x + h]; }
        __syncthreads();
    }
    if (threadIdx.x == 0 && q1 > q0) { const size_t o = 2 * ((size_t)n * G + c / (C / G)); slot_add(sums, o, sa[0]); slot_add(sums, o + 1, sb[0]); }
}

__global__ void gn_finalize_k(const double *sums, int NG, size_t len, float eps, float *mean, float *rstd) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= NG) return;
    const double m = slot_get(sums, 2 * (size_t)i) / (double)len, v = slot_get(sums, 2 * (size_t)i + 1) / (double)len - m * m;
    mean[i] = (float)m;
    rstd[i] = (float)(1.0 / sqrt((v > 0.0 ? v : 0.0) + (double)eps));
}

}   // namespace

/* (sum, sum of squares) per (sample, group) of the decoded values of an MX tensor (xdt 3 MX-fp8, 4 MX-fp4; reference layout; 16 channels
   or fewer in rows of 8 / 16) over the voxels [v0, v1), added to the slots sums[2 (n G + g)], sums[2 (n G + g) + 1] (3 x 8 bytes each; the caller zeroes them
   before the first part).  Returns 0, or -1 for a combination this library (or the reference: G > 64, C % G != 0) does not cover. */
extern "C" int lp_gn_sums_mx_n(const void *x, int xdt, int N, int C, int G, size_t S, double *sums, size_t v0, size_t v1, int n0, int cnt) {
    if (!umx_ready("lp_gn_sums_mx")) return -1;
    if ((xdt != UMX_MX8 && xdt != UMX_MX4) || C < 1 || G < 1 || G > 64 || C % G || n0 < 0 || n0 + cnt > N) return -1;
    if (cnt <= 0 || v1 <= v0 || !S) return 0;
    if (C <= 16) {                                             /* rows of 8 / 16 channels: the same codes and scale in 32-wide rows, zeros behind them */
        const int xb = xdt == UMX_MX8 ? 8 : 4;
        void *wide = umx_ws(3, umx_mx_bytes32(xb, N, C, S));
        if (!wide) return -1;
        umx_mx_rewidth(x, xb, N, C, S, wide, 1);
        x = wide;
    }
    const int nb = (C + 31) / 32;
    /* runs of about 2048 voxels of S (eight trips a block; a block ends in 2 x 4 or 2 x 32 slot additions), fewer where that leaves
       the machine short of blocks, never under 256 voxels */
    const size_t ny = (size_t)nb * cnt, fill = (8 * 148 + ny - 1) / ny, most = (S + 255) / 256;
    size_t runs = (S + 2047) / 2048;
    if (runs < fill) runs = fill;
    if (runs > most) runs = most;
    if (runs > 65535) runs = 65535;
    const dim3 grid((unsigned)runs, (unsigned)nb, (unsigned)cnt);
    const bool one = (C / G) % 8 == 0;
    const uint8_t *xq = (const uint8_t *)x;
    if (xdt == UMX_MX8) { if (one) gn_sums_rows_k<8, true><<<grid, 256>>>(xq, N, C, G, S, sums, v0, v1, n0); else gn_sums_rows_k<8, false><<<grid, 256>>>(xq, N, C, G, S, sums, v0, v1, n0); }
    else { if (one) gn_sums_rows_k<4, true><<<grid, 256>>>(xq, N, C, G, S, sums, v0, v1, n0); else gn_sums_rows_k<4, false><<<grid, 256>>>(xq, N, C, G, S, sums, v0, v1, n0); }
    g_umx_launches++;
    UMX_CK("lp_gn_sums_mx");
    return 0;
}
/* the same for a plane-major fp32 tensor (the unrounded output of a conv: split_t.stored_stats == 0, src/nn_lp.h:37) */
int umx_gn_sums_pm32(const float *x, int N, int C, int G, size_t S, double *sums, size_t v0, size_t v1) {
    if (!umx_ready("umx_gn_sums_pm32")) return -1;
    if (G < 1 || G > 64 || C % G || C > 65535 || N > 65535) return -1;
    if (N <= 0 || v1 <= v0 || !S) return 0;
    size_t runs = (S + 8191) / 8192; if (runs > 4096) runs = 4096;
    gn_sums_pm32_k<<<dim3((unsigned)runs, (unsigned)C, (unsigned)N), 256>>>(x, C, G, S, sums, v0, v1);
    g_umx_launches++;
    UMX_CK("umx_gn_sums_pm32");
    return 0;
}
extern "C" int lp_gn_sums_mx(const void *x, int xdt, int N, int C, int G, size_t S, double *sums, size_t v0, size_t v1) {
    return lp_gn_sums_mx_n(x, xdt, N, C, G, S, sums, v0, v1, 0, N);
}
/* mean and 1 / sqrt(max(var, 0) + eps) of NG (sample, group) pairs of len elements each from their slots */
extern "C" void umx_gn_finalize(const double *sums, int NG, size_t len, float eps, float *mean, float *rstd) {
    if (!umx_ready("umx_gn_finalize") || NG < 1) return;
    gn_finalize_k<<<(NG + 127) / 128, 128>>>(sums, NG, len, eps, mean, rstd);
    g_umx_launches++;
    UMX_CK("umx_gn_finalize");
}
