/* y = quantise(silu(groupnorm(x))) on MX tensors: lp_gn_silu_apply_mx (src/nn_lp.h:134; arithmetic of src/lp_mx_gn.cu:4-31), and the same
   pass with the coefficient form of the convs' input transform (a = rstd gamma, b = beta - mean a, v = fma(x, a, b): make_chan / act_ab,
   src/lp_common.cuh:244-261, 474-482), which the conv entry points run ahead of the conv when gnp_t.G != 0.

   The reference evaluates SiLU with approximate intrinsics (__expf, or tanh.approx in the fused staging: about 2^-11 relative); here it
   is v * rcp(1 + ex2(-v log2 e)) with the two hardware approximations (silu_hw, mx_rows.cuh: about 1e-6 relative), so that MX codes
   differ from a CPU evaluation of the definition only where a value sits within that distance of a rounding boundary.  An exact expf
   and an IEEE division cost some 40 instructions an element and held this pass to a tenth of the memory rate.

   Four lanes a row (mx_rows.cuh), four rows a thread per trip with their loads issued together; a lane keeps the normalisation
   constants of its eight channels in registers for the whole run of voxels. */
#include "mx_rows.cuh"
#include <cuda_fp16.h>

namespace {

/* XK: 8 / 4 MX input of that many bits, 0 fp32 plane-major, 2 fp16 plane-major.  FORM 0: ((x - mean) rstd) gamma + beta; 1: fma(x, a, b).
   grid (runs of voxels, 32-channel blocks, samples) */
struct GnSlabs { int ns, zs, zo; size_t zhw; };             /* slab-local statistics (gnp_t.ns / zs / zo / zhw, src/nn_lp.h:15-18); ns 0: per sample */
template <int XK, int BY, int FORM, bool SL>
__global__ void __launch_bounds__(256) gn_silu_rows_k(const void *__restrict__ xv, uint8_t *__restrict__ y, int C, int G, size_t S,
                                                      const float *__restrict__ gamma, const float *__restrict__ beta, const float *__restrict__ mean, const float *__restrict__ rstd, int y_split,
                                                      int c_off, int cpg, const GnSlabs sl) {
    const int N = gridDim.z, nb = gridDim.y, blk = blockIdx.y, n = blockIdx.z, T = gridDim.x;
    const int q = threadIdx.x & 3, ph = threadIdx.x >> 2;
    constexpr int RBY = BY == 8 ? 32 : 16;
    const size_t nbk = (size_t)n * nb + blk, v0 = S * blockIdx.x / T, vend = S * (blockIdx.x + 1) / T;
    const uint8_t *xq = (const uint8_t *)xv;
    const uint8_t *xs = XK == 8 ? xq + (size_t)N * nb * S * 32 : xq + (size_t)N * nb * S * 16;
    uint8_t *ys = y + (size_t)N * nb * S * RBY;
    bool live[8];
#pragma unroll
    for (int k = 0; k < 8; k++) live[k] = blk * 32 + q * 8 + k < C;
    /* the block's run of voxels in pieces that lie in one statistics slab each (one piece when the statistics are per sample): plane z belongs
       to slab (z + zo) / zs clamped to [0, ns), whose statistics are row n ns + slab (gn_row, src/lp_slab.cuh:7-12) */
    for (size_t va = v0; va < vend;) {                       /* SL false: one trip, the loop folds away */
    int nr = n; size_t v1 = vend;
    if (SL) {
        int sb_ = ((int)(va / sl.zhw) + sl.zo) / sl.zs;
        sb_ = sb_ < 0 ? 0 : sb_ >= sl.ns ? sl.ns - 1 : sb_;
        nr = n * sl.ns + sb_;
        if (sb_ < sl.ns - 1) { const long long zb = (long long)(sb_ + 1) * sl.zs - sl.zo; if (zb > 0) v1 = min(vend, max(va + 1, (size_t)zb * sl.zhw)); }
    }
    /* per channel: FORM 0 (mean, rstd, gamma, beta) in (k0, k1, k2, k3); FORM 1 (a, b) in (k0, k1) */
    float2 k0[4], k1[4], k2[4], k3[4];                       /* FORM 0: k0 holds -mean */
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int c = blk * 32 + q * 8 + k;
        float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;
        if (live[k]) {
            const int cl = c_off + c, ng = nr * G + cl / cpg;      /* cl: the channel's index in the tensor the groups are counted over */
            if (FORM == 0) { t0 = -mean[ng]; t1 = rstd[ng]; t2 = gamma[cl]; t3 = beta[cl]; }
            else { t0 = __fmul_rn(rstd[ng], gamma[cl]); t1 = __fmaf_rn(-mean[ng], t0, beta[cl]); }
        }
        if (k & 1) { k0[k >> 1].y = t0; k1[k >> 1].y = t1; k2[k >> 1].y = t2; k3[k >> 1].y = t3; }
        else { k0[k >> 1].x = t0; k1[k >> 1].x = t1; k2[k >> 1].x = t2; k3[k >> 1].x = t3; }
    }
    for (size_t vb = va; vb < v1; vb += 256) {
        float2 r[4][4];
        if (XK == 8 || XK == 4) {
            uint2 raw[4]; unsigned sb[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const size_t v = vb + u * 64 + ph;
                raw[u] = make_uint2(0u, 0u); sb[u] = 127u;
                if (v < v1) { raw[u] = qrow_ld<(XK == 4 ? 4 : 8)>(xq, nbk * S + v, q); sb[u] = __ldg(xs + nbk * S + v); }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) qrow_dec<(XK == 4 ? 4 : 8)>(raw[u], mx_scale(sb[u]), r[u]);
        } else {
            /* plane-major source: eight lanes of a plane read eight consecutive voxels */
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const size_t v = vb + u * 64 + ph;
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const size_t o = ((size_t)n * C + blk * 32 + q * 8 + k) * S + v;
                    const float t = (live[k] && v < v1) ? (XK == 0 ? __ldg((const float *)xv + o) : __half2float(__ldg((const __half *)xv + o))) : 0.f;
                    if (k & 1) r[u][k >> 1].y = t; else r[u][k >> 1].x = t;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const size_t v = vb + u * 64 + ph;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 t;
                if (FORM == 0) t = __fadd2_rn(__fmul2_rn(__fmul2_rn(__fadd2_rn(r[u][j], k0[j]), k1[j]), k2[j]), k3[j]);     /* x + (-mean) is x - mean */
                else t = __ffma2_rn(r[u][j], k0[j], k1[j]);
                r[u][j] = make_float2(live[2 * j] ? silu_hw(t.x) : 0.f, live[2 * j + 1] ? silu_hw(t.y) : 0.f);
            }
            uint2 w;
            const unsigned sb = qrow_enc<BY>(r[u], w);       /* every lane, also those past the end of the run */
            if (v < v1) {
                if (BY == 8 && y_split) *(uint2 *)(y + ((nbk * 2 + (q >> 1)) * S + v) * 16 + (q & 1) * 8) = w;
                else qrow_st<BY>(y, nbk * S + v, q, w);
                if (q == 0) ys[nbk * S + v] = (uint8_t)sb;
            }
        }
    }
    if (!SL) break;
    va = v1;
    }
}

template <int XK, int BY>
void launch_form(int form, dim3 grid, const void *x, uint8_t *y, int C, int G, size_t S, const float *gamma, const float *beta, const float *mean, const float *rstd, int y_split, int c_off, int cpg, GnSlabs sl) {
    if (sl.ns) {
        if (form == 0) gn_silu_rows_k<XK, BY, 0, true><<<grid, 256>>>(x, y, C, G, S, gamma, beta, mean, rstd, y_split, c_off, cpg, sl);
        else gn_silu_rows_k<XK, BY, 1, true><<<grid, 256>>>(x, y, C, G, S, gamma, beta, mean, rstd, y_split, c_off, cpg, sl);
    } else if (form == 0) gn_silu_rows_k<XK, BY, 0, false><<<grid, 256>>>(x, y, C, G, S, gamma, beta, mean, rstd, y_split, c_off, cpg, sl);
    else gn_silu_rows_k<XK, BY, 1, false><<<grid, 256>>>(x, y, C, G, S, gamma, beta, mean, rstd, y_split, c_off, cpg, sl);
}

}   // namespace

/* x: xdt 0 (fp32 plane-major), 2 (fp16 plane-major), 3 / 4 (MX, reference layout, 32-wide rows); y: MX of `bits` bits, `layout` as in
   umx_pm_to_mx32; form 0 / 1 as above.  The tensor may be a channel segment of a larger one the G groups are counted over (a conv's
   concat input with one GroupNorm over both parts): its channel 0 is channel c_off of C_all (0, C for a whole tensor); gamma, beta,
   mean, rstd are the larger tensor's.  ns != 0: slab-local statistics, mean and rstd [N][ns][G], plane z = voxel / zhw of the tensor in slab
   (z + zo) / zs clamped to [0, ns) (gnp_t, src/nn_lp.h:15-18; zo may be negative here: a tensor that is a z range of the one the slabs are
   counted in).  Returns 0, -1 on an unsupported combination (the caller reports it). */
int umx_gn_silu_apply_seg_slabs(const void *x, int xdt, int N, int C, size_t S, int G, const float *gamma, const float *beta, const float *mean, const float *rstd,
                                void *y, int bits, int layout, int form, int c_off, int C_all, int ns, int zs, int zo, size_t zhw) {
    if (ns < 0 || (ns && (zs < 1 || !zhw || S % zhw))) return -1;
    const GnSlabs sl = {ns, zs, zo, zhw};
    if (C < 1 || G < 1 || C_all % G || c_off < 0 || c_off + C > C_all || (bits != 8 && bits != 4) || (xdt != UMX_F32 && xdt != UMX_F16 && xdt != UMX_MX8 && xdt != UMX_MX4)) return -1;
    const int cpg = C_all / G;
    const int nb = (C + 31) / 32;
    if (!N || !S) return 0;
    if (N > 65535 || nb > 65535) return -1;
    /* runs of about 2048 voxels (eight trips a block) */
    size_t T = (S + 2047) / 2048; if (T > 0x7fffffffu) return -1;
    const dim3 blocks((unsigned)T, (unsigned)nb, (unsigned)N);
    const int ys = bits == 8 && layout == UMX_LAYOUT_SPLIT;
    uint8_t *yb = (uint8_t *)y;
#define UMX_GSA(XK) do { if (bits == 8) launch_form<XK, 8>(form, blocks, x, yb, C, G, S, gamma, beta, mean, rstd, ys, c_off, cpg, sl); else launch_form<XK, 4>(form, blocks, x, yb, C, G, S, gamma, beta, mean, rstd, ys, c_off, cpg, sl); } while (0)
    if (xdt == UMX_MX8) UMX_GSA(8); else if (xdt == UMX_MX4) UMX_GSA(4); else if (xdt == UMX_F16) UMX_GSA(2); else UMX_GSA(0);
#undef UMX_GSA
    g_umx_launches++;
    return 0;
}
/* statistics per sample */
int umx_gn_silu_apply_seg(const void *x, int xdt, int N, int C, size_t S, int G, const float *gamma, const float *beta, const float *mean, const float *rstd,
                          void *y, int bits, int layout, int form, int c_off, int C_all) {
    return umx_gn_silu_apply_seg_slabs(x, xdt, N, C, S, G, gamma, beta, mean, rstd, y, bits, layout, form, c_off, C_all, 0, 0, 0, 0);
}
int umx_gn_silu_apply(const void *x, int xdt, int N, int C, size_t S, int G, const float *gamma, const float *beta, const float *mean, const float *rstd,
                      void *y, int bits, int layout, int form) {
    return umx_gn_silu_apply_seg(x, xdt, N, C, S, G, gamma, beta, mean, rstd, y, bits, layout, form, 0, C);
}

extern "C" void lp_gn_silu_apply_mx(const void *x, int xdt, shape5 s, int G, const float *gamma, const float *beta, const float *mean, const float *rstd, void *y, int ydt) {
    if (!umx_ready("lp_gn_silu_apply_mx")) return;
    if (ydt != UMX_MX8 && ydt != UMX_MX4) { fprintf(stderr, "lp_gn_silu_apply_mx: output dtype %d is not MX\n", ydt); abort(); }
    const size_t S = (size_t)s.d * s.h * s.w;
    const int ybits = ydt == UMX_MX8 ? 8 : 4;
    if (s.c <= 16 && s.c >= 1) {
        /* MX tensors of 16 channels or fewer are stored in rows of 8 / 16 (src/lp_common.cuh:132): widened into scratch, transformed there, narrowed */
        const void *xin = x;
        if (xdt == UMX_MX8 || xdt == UMX_MX4) {
            const int xb = xdt == UMX_MX8 ? 8 : 4;
            void *a = umx_ws(3, umx_mx_bytes32(xb, s.n, s.c, S));
            if (!a) return;
            umx_mx_rewidth(x, xb, s.n, s.c, S, a, 1);
            xin = a;
        }
        void *b = umx_ws(4, umx_mx_bytes32(ybits, s.n, s.c, S));
        if (!b) return;
        if (umx_gn_silu_apply(xin, xdt, s.n, s.c, S, G, gamma, beta, mean, rstd, b, ybits, UMX_LAYOUT_REF, 0) != 0) {
            fprintf(stderr, "lp_gn_silu_apply_mx: input dtype %d, %d channels in %d groups is not built in this library\n", xdt, s.c, G); abort();
        }
        umx_mx_rewidth(b, ybits, s.n, s.c, S, y, 0);
        UMX_CK("lp_gn_silu_apply_mx");
        return;
    }
    if (umx_gn_silu_apply(x, xdt, s.n, s.c, S, G, gamma, beta, mean, rstd, y, ybits, UMX_LAYOUT_REF, 0) != 0) {
        fprintf(stderr, "lp_gn_silu_apply_mx: input dtype %d, %d channels in %d groups is not built in this library\n", xdt, s.c, G); abort();
    }
    UMX_CK("lp_gn_silu_apply_mx");
}
