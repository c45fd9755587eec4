/* y = quantise(silu(groupnorm(x))) on MX tensors: lp_gn_silu_apply_mx (src/nn_lp.h:134, src/lp_mx_gn.cu:4-31), and the same pass with the
   coefficient form of the convs' input transform (a = rstd gamma, b = beta - mean a, v = fma(x, a, b): make_chan / act_ab,
   src/lp_common.cuh:244-261, 474-482), which the conv entry points run ahead of the conv when gnp_t.G != 0.

   The reference evaluates SiLU with approximate intrinsics (__expf, or tanh.approx in the fused staging: about 2^-11 relative); here it
   is v / (1 + expf(-v)) with the accurate expf and an IEEE division, so that the result agrees with a CPU evaluation of the definition to
   an ulp or two and MX codes differ from that evaluation's only where a value sits on a rounding boundary. */
#include "mx_common.cuh"
#include <cuda_fp16.h>

namespace {

/* XK: 8 / 4 MX input of that many bits, 0 fp32 plane-major, 2 fp16 plane-major.  FORM 0: ((x - mean) rstd) gamma + beta; 1: fma(x, a, b).
   One thread per 32-channel row (sample, block, voxel). */
template <int XK, int BY, int FORM>
__global__ void __launch_bounds__(256) gn_silu_apply_k(const void *__restrict__ xv, uint8_t *__restrict__ y, int N, int C, int G, size_t S,
                                                       const float *__restrict__ gamma, const float *__restrict__ beta, const float *__restrict__ mean, const float *__restrict__ rstd, int y_split) {
    const int nb = (C + 31) / 32, cpg = C / G;
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= (size_t)N * nb * S) return;
    const size_t v = i % S;
    const int blk = (int)((i / S) % nb), n = (int)(i / (S * nb));
    float r[32];
    if (XK == 8) {
        const uint8_t *x = (const uint8_t *)xv;
        const float fx = mx_scale(x[(size_t)N * nb * S * 32 + i]);
        const uint4 t0 = *(const uint4 *)(x + i * 32), t1 = *(const uint4 *)(x + i * 32 + 16);
        const unsigned wd[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
        for (int j = 0; j < 8; j++) dec_e4m3x4(wd[j], r + 4 * j);
#pragma unroll
        for (int k = 0; k < 32; k++) r[k] *= fx;
    } else if (XK == 4) {
        const uint8_t *x = (const uint8_t *)xv;
        const float fx = mx_scale(x[(size_t)N * nb * S * 16 + i]);
        const uint4 t0 = *(const uint4 *)(x + i * 16);
        const unsigned wd[4] = {t0.x, t0.y, t0.z, t0.w};
#pragma unroll
        for (int j = 0; j < 4; j++) dec_e2m1x8(wd[j], r + 8 * j);
#pragma unroll
        for (int k = 0; k < 32; k++) r[k] *= fx;
    } else {
#pragma unroll
        for (int k = 0; k < 32; k++) {
            const int c = blk * 32 + k;
            const size_t o = ((size_t)n * C + c) * S + v;
            r[k] = c < C ? (XK == 0 ? ((const float *)xv)[o] : __half2float(((const __half *)xv)[o])) : 0.f;
        }
    }
#pragma unroll
    for (int k = 0; k < 32; k++) {
        const int c = blk * 32 + k;
        if (c < C) {
            const int ng = n * G + c / cpg;
            float u;
            if (FORM == 0) u = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(r[k], mean[ng]), rstd[ng]), gamma[c]), beta[c]);
            else { const float a = __fmul_rn(rstd[ng], gamma[c]), b = __fmaf_rn(-mean[ng], a, beta[c]); u = __fmaf_rn(r[k], a, b); }
            r[k] = __fdiv_rn(u, __fadd_rn(1.f, expf(-u)));
        } else r[k] = 0.f;
    }
    unsigned w[8];
    const unsigned sb = mx_encode_row32<BY>(r, w);
    if (BY == 8) {
        if (y_split) {
            const size_t nbk = i / S;
            *(uint4 *)(y + ((nbk * 2 + 0) * S + v) * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            *(uint4 *)(y + ((nbk * 2 + 1) * S + v) * 16) = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
            *(uint4 *)(y + i * 32) = make_uint4(w[0], w[1], w[2], w[3]);
            *(uint4 *)(y + i * 32 + 16) = make_uint4(w[4], w[5], w[6], w[7]);
        }
        y[(size_t)N * nb * S * 32 + i] = (uint8_t)sb;
    } else {
        *(uint4 *)(y + i * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        y[(size_t)N * nb * S * 16 + i] = (uint8_t)sb;
    }
}

template <int XK, int BY>
void launch_form(int form, unsigned blocks, const void *x, uint8_t *y, int N, int C, int G, size_t S, const float *gamma, const float *beta, const float *mean, const float *rstd, int y_split) {
    if (form == 0) gn_silu_apply_k<XK, BY, 0><<<blocks, 256>>>(x, y, N, C, G, S, gamma, beta, mean, rstd, y_split);
    else gn_silu_apply_k<XK, BY, 1><<<blocks, 256>>>(x, y, N, C, G, S, gamma, beta, mean, rstd, y_split);
}

}   // namespace

/* x: xdt 0 (fp32 plane-major), 2 (fp16 plane-major), 3 / 4 (MX, reference layout, 32-wide rows); y: MX of `bits` bits, `layout` as in
   umx_pm_to_mx32; form 0 / 1 as above.  Returns 0, -1 on an unsupported combination (the caller reports it). */
int umx_gn_silu_apply(const void *x, int xdt, int N, int C, size_t S, int G, const float *gamma, const float *beta, const float *mean, const float *rstd,
                      void *y, int bits, int layout, int form) {
    if (C <= 16 || G < 1 || C % G || (bits != 8 && bits != 4) || (xdt != UMX_F32 && xdt != UMX_F16 && xdt != UMX_MX8 && xdt != UMX_MX4)) return -1;
    const size_t rows = (size_t)N * ((C + 31) / 32) * S;
    if (!rows) return 0;
    const unsigned blocks = (unsigned)((rows + 255) / 256);
    const int ys = bits == 8 && layout == UMX_LAYOUT_SPLIT;
    uint8_t *yb = (uint8_t *)y;
#define UMX_GSA(XK) do { if (bits == 8) launch_form<XK, 8>(form, blocks, x, yb, N, C, G, S, gamma, beta, mean, rstd, ys); else launch_form<XK, 4>(form, blocks, x, yb, N, C, G, S, gamma, beta, mean, rstd, ys); } while (0)
    if (xdt == UMX_MX8) UMX_GSA(8); else if (xdt == UMX_MX4) UMX_GSA(4); else if (xdt == UMX_F16) UMX_GSA(2); else UMX_GSA(0);
#undef UMX_GSA
    g_umx_launches++;
    return 0;
}

extern "C" void lp_gn_silu_apply_mx(const void *x, int xdt, shape5 s, int G, const float *gamma, const float *beta, const float *mean, const float *rstd, void *y, int ydt) {
    if (!umx_ready("lp_gn_silu_apply_mx")) return;
    if (ydt != UMX_MX8 && ydt != UMX_MX4) { fprintf(stderr, "lp_gn_silu_apply_mx: output dtype %d is not MX\n", ydt); abort(); }
    if (umx_gn_silu_apply(x, xdt, s.n, s.c, (size_t)s.d * s.h * s.w, G, gamma, beta, mean, rstd, y, ydt == UMX_MX8 ? 8 : 4, UMX_LAYOUT_REF, 0) != 0) {
        fprintf(stderr, "lp_gn_silu_apply_mx: input dtype %d, %d channels in %d groups is not built in this library\n", xdt, s.c, G); abort();
    }
    UMX_CK("lp_gn_silu_apply_mx");
}
