/* Elementwise operators of the reference interface on MX tensors (32-wide rows, reference layout):
     lp_up2_fwd_mx        exact-2x trilinear upsample, optionally of silu(gn(x))      (src/nn_lp.h:136, src/lp_mx_gn.cu:32-72, 151-173)
     lp_conv1_fwd_mx      1^3 conv with fp32 weights to fp32 plane-major logits        (src/nn_lp.h:138, src/lp_mx_conv1.cu:4-22, 422-444)
     lp_conv1_fwd_mx_h16  the same with fp16 logits                                      (src/nn_lp.h:139)
   The arithmetic order is the reference's: the upsample adds its eight terms with fma in (z, y, x) order, near neighbour first; the 1^3
   conv starts from the bias and adds w[co][ci] x[ci] with fma in ascending ci.  Both are bit-equal to a CPU evaluation of that order when no
   GroupNorm is asked for; with gnp_t.G != 0 the input goes through silu(fma(x, a, b)) first (accurate expf; see gn_apply.cu). */
#include "mx_common.cuh"
#include <cuda_fp16.h>

namespace {

/* row i of an MX tensor (BITS bits) decoded to 32 floats */
template <int BITS> __device__ __forceinline__ void load_row32(const uint8_t *__restrict__ x, const uint8_t *__restrict__ sc, size_t i, float *r) {
    const float fx = mx_scale(__ldg(sc + i));
    if (BITS == 8) {
        const uint4 t0 = __ldg((const uint4 *)(x + i * 32)), t1 = __ldg((const uint4 *)(x + i * 32 + 16));
        const unsigned wd[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
        for (int j = 0; j < 8; j++) dec_e4m3x4(wd[j], r + 4 * j);
    } else {
        const uint4 t0 = __ldg((const uint4 *)(x + i * 16));
        const unsigned wd[4] = {t0.x, t0.y, t0.z, t0.w};
#pragma unroll
        for (int j = 0; j < 4; j++) dec_e2m1x8(wd[j], r + 8 * j);
    }
#pragma unroll
    for (int k = 0; k < 32; k++) r[k] *= fx;
}
__device__ __forceinline__ float silu_ab(float x, float a, float b) { const float u = __fmaf_rn(x, a, b); return __fdiv_rn(u, __fadd_rn(1.f, expf(-u))); }

/* grid (fine voxels / 256, sample x block) */
template <int BX, int BY>
__global__ void __launch_bounds__(256) up2_mx_k(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int N, int C, int D, int H, int W, gnp_t gp) {
    const int nb = (C + 31) / 32, Do = 2 * D, Ho = 2 * H, Wo = 2 * W;
    const size_t S = (size_t)D * H * W, So = 8 * S;
    const int nbk = blockIdx.y, n = nbk / nb, blk = nbk % nb;
    __shared__ float ca[32], cb[32];
    if (threadIdx.x < 32) {
        const int c = blk * 32 + (int)threadIdx.x;
        float a = 1.f, b = 0.f;
        if (gp.G && c < C) { const int ng = n * gp.G + c / (C / gp.G); a = __fmul_rn(gp.rstd[ng], gp.gamma[c]); b = __fmaf_rn(-gp.mean[ng], a, gp.beta[c]); }
        ca[threadIdx.x] = a; cb[threadIdx.x] = b;
    }
    __syncthreads();
    const size_t vo = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (vo >= So) return;
    const int fx = (int)(vo % Wo), fy = (int)((vo / Wo) % Ho), fz = (int)(vo / ((size_t)Wo * Ho));
    /* per axis the two source voxels of fine coordinate f on a grid of n: the coarse voxel under it (weight 3/4) and that voxel's
       neighbour on f's side, clamped to the grid (weight 1/4) */
    auto under = [](int f) { return f >> 1; };
    auto beside = [](int f, int n) { const int t = (f >> 1) + ((f & 1) ? 1 : -1); return t < 0 ? 0 : (t >= n ? n - 1 : t); };
    const int sz[2] = {under(fz), beside(fz, D)}, sy[2] = {under(fy), beside(fy, H)}, sx[2] = {under(fx), beside(fx, W)};
    constexpr int RBX = BX == 8 ? 32 : 16, RBY = BY == 8 ? 32 : 16;
    const uint8_t *sc = x + (size_t)N * nb * S * RBX;
    const int kmax = min(32, C - blk * 32);
    float acc[32];
#pragma unroll
    for (int k = 0; k < 32; k++) acc[k] = 0.f;
    /* the eight corners in (z, y, x) order, nearest first on each axis; one fma per corner and channel */
#pragma unroll
    for (int t = 0; t < 8; t++) {
        const int iz = t >> 2, iy = (t >> 1) & 1, ix = t & 1;
        const float w3 = (iz ? 0.25f : 0.75f) * (iy ? 0.25f : 0.75f) * (ix ? 0.25f : 0.75f);
        float r[32];
        load_row32<BX>(x, sc, (size_t)nbk * S + ((size_t)sz[iz] * H + sy[iy]) * W + sx[ix], r);
        if (gp.G) {
#pragma unroll
            for (int k = 0; k < 32; k++) if (k < kmax) r[k] = silu_ab(r[k], ca[k], cb[k]);
        }
#pragma unroll
        for (int k = 0; k < 32; k++) acc[k] = __fmaf_rn(w3, r[k], acc[k]);
    }
    unsigned wq[8];
    const unsigned sb = mx_encode_row32<BY>(acc, wq);
    const size_t i = (size_t)nbk * So + vo;
    *(uint4 *)(y + i * RBY) = make_uint4(wq[0], wq[1], wq[2], wq[3]);
    if (BY == 8) *(uint4 *)(y + i * 32 + 16) = make_uint4(wq[4], wq[5], wq[6], wq[7]);
    y[(size_t)N * nb * So * RBY + i] = (uint8_t)sb;
}

/* one thread per voxel; weights [ci][16] and the GroupNorm coefficients [n][ci] in shared memory */
template <int BITS, typename YT>
__global__ void __launch_bounds__(256) conv1_mx_k(const uint8_t *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b, YT *__restrict__ y,
                                                  int N, int Ci, int Co, size_t S, gnp_t gp) {
    extern __shared__ __align__(16) float c1s[];
    float *sw = c1s; float2 *sab = (float2 *)(c1s + (size_t)16 * Ci);
    const int nb = (Ci + 31) / 32;
    for (int i = threadIdx.x; i < 16 * Ci; i += blockDim.x) { const int ci = i >> 4, co = i & 15; sw[i] = co < Co ? w[(size_t)co * Ci + ci] : 0.f; }
    if (gp.G) for (int i = threadIdx.x; i < N * Ci; i += blockDim.x) {
        const int n = i / Ci, ci = i % Ci, ng = n * gp.G + ci / (Ci / gp.G);
        const float a = __fmul_rn(gp.rstd[ng], gp.gamma[ci]);
        sab[i] = make_float2(a, __fmaf_rn(-gp.mean[ng], a, gp.beta[ci]));
    }
    __syncthreads();
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= (size_t)N * S) return;
    const int n = (int)(i / S); const size_t v = i % S;
    constexpr int RB = BITS == 8 ? 32 : 16;
    const uint8_t *sc = x + (size_t)N * nb * S * RB;
    float acc[16];
#pragma unroll
    for (int co = 0; co < 16; co++) acc[co] = (b && co < Co) ? b[co] : 0.f;
    for (int blk = 0; blk < nb; blk++) {
        float r[32];
        load_row32<BITS>(x, sc, ((size_t)n * nb + blk) * S + v, r);
        const int kmax = min(32, Ci - blk * 32);
#pragma unroll
        for (int k = 0; k < 32; k++) {
            if (k < kmax) {
                const int ci = blk * 32 + k;
                const float xv = gp.G ? silu_ab(r[k], sab[n * Ci + ci].x, sab[n * Ci + ci].y) : r[k];
                const float4 *wr = (const float4 *)(sw + 16 * ci);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float4 t = wr[q];
                    acc[4 * q] = __fmaf_rn(t.x, xv, acc[4 * q]); acc[4 * q + 1] = __fmaf_rn(t.y, xv, acc[4 * q + 1]);
                    acc[4 * q + 2] = __fmaf_rn(t.z, xv, acc[4 * q + 2]); acc[4 * q + 3] = __fmaf_rn(t.w, xv, acc[4 * q + 3]);
                }
            }
        }
    }
#pragma unroll
    for (int co = 0; co < 16; co++) if (co < Co) {
        const size_t o = ((size_t)n * Co + co) * S + v;
        if (sizeof(YT) == 4) ((float *)y)[o] = acc[co]; else ((__half *)y)[o] = __float2half_rn(acc[co]);
    }
}

void gp_check(const char *fn, gnp_t gp, int C) {
    if (gp.G && (gp.ns > 1 || gp.zs || gp.zo || gp.zhw)) { fprintf(stderr, "%s: slab-local GroupNorm (gnp_t.ns / zs / zo / zhw) is not built in this library\n", fn); abort(); }
    if (gp.G && (gp.G < 1 || C % gp.G)) { fprintf(stderr, "%s: %d channels in %d groups\n", fn, C, gp.G); abort(); }
}

template <typename YT> void conv1_fwd(const char *fn, const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, YT *y, gnp_t gp) {
    if (!umx_ready(fn)) return;
    if (xdt != UMX_MX8 && xdt != UMX_MX4) { fprintf(stderr, "%s: input dtype %d is not MX\n", fn, xdt); abort(); }
    if (xs.c <= 16) { fprintf(stderr, "%s: an input of 16 channels or fewer (8 / 16-wide MX rows) is not built in this library\n", fn); abort(); }
    gp_check(fn, gp, xs.c);
    const size_t S = (size_t)xs.d * xs.h * xs.w;
    if (cout > 16 && cout % 16 == 0 && xs.n == 1) {     /* more outputs: passes of 16, as the reference */
        for (int c0 = 0; c0 < cout; c0 += 16) conv1_fwd<YT>(fn, x, xdt, xs, w + (size_t)c0 * xs.c, b ? b + c0 : nullptr, 16, y + (size_t)c0 * S, gp);
        return;
    }
    if (cout < 1 || cout > 16) { fprintf(stderr, "%s: cout %d > 16\n", fn, cout); abort(); }
    const size_t smem = (size_t)16 * xs.c * 4 + (gp.G ? (size_t)xs.n * xs.c * 8 : 0);
    if (smem > 48 * 1024) { fprintf(stderr, "%s: %d samples of %d channels need more shared memory than this kernel has\n", fn, xs.n, xs.c); abort(); }
    const size_t rows = (size_t)xs.n * S;
    if (!rows) return;
    const unsigned blocks = (unsigned)((rows + 255) / 256);
    if (xdt == UMX_MX8) conv1_mx_k<8, YT><<<blocks, 256, smem>>>((const uint8_t *)x, w, b, y, xs.n, xs.c, cout, S, gp);
    else conv1_mx_k<4, YT><<<blocks, 256, smem>>>((const uint8_t *)x, w, b, y, xs.n, xs.c, cout, S, gp);
    g_umx_launches++;
    UMX_CK(fn);
}

}   // namespace

extern "C" void lp_up2_fwd_mx(const void *x, int xdt, shape5 xs, void *y, int ydt, gnp_t gp) {
    const char *fn = "lp_up2_fwd_mx";
    if (!umx_ready(fn)) return;
    if ((xdt != UMX_MX8 && xdt != UMX_MX4) || (ydt != UMX_MX8 && ydt != UMX_MX4)) { fprintf(stderr, "%s: dtypes %d -> %d are not MX\n", fn, xdt, ydt); abort(); }
    if (xs.c <= 16) { fprintf(stderr, "%s: 16 channels or fewer (8 / 16-wide MX rows) is not built in this library\n", fn); abort(); }
    gp_check(fn, gp, xs.c);
    const size_t So = 8 * (size_t)xs.d * xs.h * xs.w;
    if (!So || !xs.n) return;
    const dim3 grid((unsigned)((So + 255) / 256), (unsigned)(xs.n * ((xs.c + 31) / 32)));
    const uint8_t *xq = (const uint8_t *)x; uint8_t *yq = (uint8_t *)y;
    if (xdt == UMX_MX4) { if (ydt == UMX_MX4) up2_mx_k<4, 4><<<grid, 256>>>(xq, yq, xs.n, xs.c, xs.d, xs.h, xs.w, gp); else up2_mx_k<4, 8><<<grid, 256>>>(xq, yq, xs.n, xs.c, xs.d, xs.h, xs.w, gp); }
    else { if (ydt == UMX_MX4) up2_mx_k<8, 4><<<grid, 256>>>(xq, yq, xs.n, xs.c, xs.d, xs.h, xs.w, gp); else up2_mx_k<8, 8><<<grid, 256>>>(xq, yq, xs.n, xs.c, xs.d, xs.h, xs.w, gp); }
    g_umx_launches++;
    UMX_CK(fn);
}
extern "C" void lp_conv1_fwd_mx(const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, float *y, gnp_t gp) {
    conv1_fwd<float>("lp_conv1_fwd_mx", x, xdt, xs, w, b, cout, y, gp);
}
extern "C" void lp_conv1_fwd_mx_h16(const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, void *y, gnp_t gp) {
    conv1_fwd<__half>("lp_conv1_fwd_mx_h16", x, xdt, xs, w, b, cout, (__half *)y, gp);
}
