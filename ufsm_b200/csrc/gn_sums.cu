/* GroupNorm statistics of MX tensors: lp_gn_sums_mx (src/nn_lp.h:175, src/lp_mx_gnsums.cu:9-106) and the finalise step
   (gn_finalize_k, src/nn_elem.cu:5-11).

   A sum lives in a slot of three 64-bit words, the reference's exact fixed point (src/gnacc.cuh:9-27): word 0 the fraction in units of
   2^-64, word 1 the signed integer part (two's complement together with word 0), word 2 a count of non-finite contributions.  Blocks add
   their partial sums with integer atomics, so the result does not depend on the order in which blocks finish.  Inside a block the
   arithmetic is fp64 in a fixed order (per thread over its rows, then lanes, then warps): decoded MX values are products of a 4- or
   2-bit mantissa and a power of two, so the fp64 sums of values and squares carry no rounding error for any realistic tensor. */
#include "mx_common.cuh"

namespace {

__device__ __forceinline__ void slot_add(double *base, size_t i, double v) {
    unsigned long long *w = (unsigned long long *)base + 3 * i;
    if (!(fabs(v) < 4.611686018427387904e18)) { atomicAdd(&w[2], 1ull); return; }      /* NaN, inf, or beyond 2^62: the sum reads as NaN */
    const double fl = floor(v);
    const unsigned long long frac = (unsigned long long)((v - fl) * 18446744073709551616.0);   /* [0, 1) scaled by 2^64, exact */
    const long long whole = (long long)fl;
    if (frac) { const unsigned long long old = atomicAdd(&w[0], frac); if (old + frac < old) atomicAdd(&w[1], 1ull); }   /* carry */
    if (whole) atomicAdd(&w[1], (unsigned long long)whole);
}
__device__ __forceinline__ double slot_get(const double *base, size_t i) {
    const unsigned long long *w = (const unsigned long long *)base + 3 * i;
    if (w[2]) return __longlong_as_double(0x7ff8000000000000ll);
    return (double)(long long)w[1] + (double)w[0] * 5.42101086242752217e-20;
}

/* block = (voxel slab, 32-channel block, sample); two threads a row (16 channels each), rows 128 apart */
template <int BITS>
__global__ void __launch_bounds__(256) gn_sums_k(const uint8_t *__restrict__ x, int N, int C, int G, size_t S, double *sums, size_t v0, size_t v1, int n0) {
    const int nb = (C + 31) / 32, blk = blockIdx.y, n = n0 + (int)blockIdx.z, h = threadIdx.x & 1, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int RB = BITS == 8 ? 32 : 16;
    size_t q0 = S * blockIdx.x / gridDim.x, q1 = S * (blockIdx.x + 1) / gridDim.x;
    if (q0 < v0) q0 = v0;
    if (q1 > v1) q1 = v1;
    const uint8_t *sc = x + (size_t)N * nb * S * RB;
    const size_t rbase = ((size_t)n * nb + blk) * S;
    double s1[16], s2[16];
#pragma unroll
    for (int k = 0; k < 16; k++) { s1[k] = 0.0; s2[k] = 0.0; }
    for (size_t q = q0 + (threadIdx.x >> 1); q < q1; q += 128) {
        const size_t ri = rbase + q;
        const float fx = mx_scale(__ldg(sc + ri));
        if (BITS == 8) {
            const uint4 t = __ldg((const uint4 *)(x + ri * 32 + 16 * h));
            const unsigned wd[4] = {t.x, t.y, t.z, t.w};
            float r[16];
#pragma unroll
            for (int j = 0; j < 4; j++) dec_e4m3x4(wd[j], r + 4 * j);
#pragma unroll
            for (int k = 0; k < 16; k++) { const double v = (double)(r[k] * fx); s1[k] += v; s2[k] = fma(v, v, s2[k]); }
        } else {
            const uint2 t = __ldg((const uint2 *)(x + ri * 16 + 8 * h));
            const unsigned wd[2] = {t.x, t.y};
            float r[16];
#pragma unroll
            for (int j = 0; j < 2; j++) dec_e2m1x8(wd[j], r + 8 * j);
#pragma unroll
            for (int k = 0; k < 16; k++) { const double v = (double)(r[k] * fx); s1[k] += v; s2[k] = fma(v, v, s2[k]); }
        }
    }
    __shared__ double w1[8][32], w2[8][32];
#pragma unroll
    for (int k = 0; k < 16; k++) {
        double a = s1[k], b = s2[k];
#pragma unroll
        for (int o = 16; o >= 2; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
        if (lane < 2) { w1[warp][16 * h + k] = a; w2[warp][16 * h + k] = b; }
    }
    __syncthreads();
    const int ch = blk * 32 + (int)threadIdx.x;
    if (threadIdx.x < 32 && ch < C) {
        double a = 0.0, b = 0.0;
#pragma unroll
        for (int w = 0; w < 8; w++) { a += w1[w][threadIdx.x]; b += w2[w][threadIdx.x]; }
        const size_t o = 2 * ((size_t)n * G + ch / (C / G));
        slot_add(sums, o, a); slot_add(sums, o + 1, b);
    }
}

__global__ void gn_finalize_k(const double *sums, int NG, size_t len, float eps, float *mean, float *rstd) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= NG) return;
    const double m = slot_get(sums, 2 * (size_t)i) / (double)len, v = slot_get(sums, 2 * (size_t)i + 1) / (double)len - m * m;
    mean[i] = (float)m;
    rstd[i] = (float)(1.0 / sqrt((v > 0.0 ? v : 0.0) + (double)eps));
}

}   // namespace

/* (sum, sum of squares) per (sample, group) of the decoded values of an MX tensor (xdt 3 MX-fp8, 4 MX-fp4; reference layout, more than 16
   channels) over the voxels [v0, v1), added to the slots sums[2 (n G + g)], sums[2 (n G + g) + 1] (3 x 8 bytes each; the caller zeroes them
   before the first part).  Returns 0, or -1 for a combination this library (or the reference: G > 64, C % G != 0) does not cover. */
extern "C" int lp_gn_sums_mx_n(const void *x, int xdt, int N, int C, int G, size_t S, double *sums, size_t v0, size_t v1, int n0, int cnt) {
    if (!umx_ready("lp_gn_sums_mx")) return -1;
    if ((xdt != UMX_MX8 && xdt != UMX_MX4) || C <= 16 || G < 1 || G > 64 || C % G || n0 < 0 || n0 + cnt > N) return -1;
    if (cnt <= 0 || v1 <= v0 || !S) return 0;
    const int nb = (C + 31) / 32;
    /* slabs of about 4096 voxels, at least about 160 blocks in all, at least 512 voxels each, at most 1024 per (block, sample) */
    const size_t ny = (size_t)nb * cnt;
    size_t slabs = S / 4096; const size_t want = (160 + ny - 1) / ny, most = S / 512 > 0 ? S / 512 : 1;
    if (slabs < want) slabs = want;
    if (slabs > most) slabs = most;
    if (slabs > 1024) slabs = 1024;
    const dim3 grid((unsigned)slabs, (unsigned)nb, (unsigned)cnt);
    if (xdt == UMX_MX8) gn_sums_k<8><<<grid, 256>>>((const uint8_t *)x, N, C, G, S, sums, v0, v1, n0);
    else gn_sums_k<4><<<grid, 256>>>((const uint8_t *)x, N, C, G, S, sums, v0, v1, n0);
    g_umx_launches++;
    UMX_CK("lp_gn_sums_mx");
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
