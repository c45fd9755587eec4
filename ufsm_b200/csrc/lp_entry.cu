/* The reference's conv entry points lp_conv_fwd_f8 / lp_conv_fwd_f4 / lp_conv_fwd_s2_f8 (src/nn_lp.h:53-54, 104) on top of the tcgen05
   conv: same signature, storage codes and error behaviour; the prepared weights are memoised under split_t.wkey as the reference's fp4
   kernel does (src/lp_f4fwd.cuh:748-770).  Of split_t (src/nn_lp.h:20-37): x2 / c_split / gp2 (concat input), up (the x part stored at
   half resolution and read as its trilinear upsample), y2 / o_split (split output), stored_stats with osum / Go / zlo / zhi (GroupNorm
   sums of the stored output), zi0 / Di, zw0 / zw1, yD / yzo (z range, z window, slab output), accum; sr / osr / o_pad stop with
   "not built". */
#include "mx_common.cuh"
#include <stdlib.h>
#include <string.h>

struct memo_t { unsigned wkey; const float *w, *b; int cout, cin, bits, dev; umx_conv *c; };
static memo_t g_memo[256];
static int g_nmemo = 0;

extern "C" void lp_wmemo_clear(void) {
    cudaDeviceSynchronize();
    for (int i = 0; i < g_nmemo; i++) umx_conv_free(g_memo[i].c);
    g_nmemo = 0;
}
int umx_gn_silu_apply(const void *x, int xdt, int N, int C, size_t S, int G, const float *gamma, const float *beta, const float *mean, const float *rstd,
                      void *y, int bits, int layout, int form);
/* the GroupNorm + SiLU input transform of a conv (gnp_t.G != 0): silu(fma(x, a, b)) quantised to the conv's MX format, into scratch, ahead
   of the conv (the reference applies it while staging the operand and quantises the staged rows the same way) */
int umx_gn_silu_apply_seg_slabs(const void *x, int xdt, int N, int C, size_t S, int G, const float *gamma, const float *beta, const float *mean, const float *rstd,
                                void *y, int bits, int layout, int form, int c_off, int C_all, int ns, int zs, int zo, size_t zhw);
/* slab-local statistics (gnp_t.ns != 0, src/nn_lp.h:15-18): the geometry must be that of the tensor */
static void slab_check(const char *fn, const gnp_t &gp, shape5 xs) {
    if (!gp.ns) return;
    if (gp.ns < 0 || gp.zs < 1 || gp.zo < 0 || gp.zo >= gp.zs || gp.zhw != xs.h * xs.w) {
        fprintf(stderr, "%s: slab-local GroupNorm with ns %d, zs %d, zo %d, zhw %d on planes of %d voxels\n", fn, gp.ns, gp.zs, gp.zo, gp.zhw, xs.h * xs.w); abort();
    }
}
static const void *gn_input(const char *fn, const void *x, int xbf, shape5 xs, gnp_t gp, int bits) {
    slab_check(fn, gp, xs);
    const size_t S = (size_t)xs.d * xs.h * xs.w;
    void *ws = umx_ws(2, umx_mx_bytes32(bits, xs.n, xs.c, S));
    if (!ws) return nullptr;
    if (umx_gn_silu_apply_seg_slabs(x, xbf, xs.n, xs.c, S, gp.G, gp.gamma, gp.beta, gp.mean, gp.rstd, ws, bits, UMX_LAYOUT_SPLIT, 1, 0, xs.c, gp.ns, gp.zs, gp.zo, (size_t)gp.zhw) != 0) {
        fprintf(stderr, "%s: the GroupNorm + SiLU input transform of a storage-%d tensor of %d channels in %d groups is not built in this library\n", fn, xbf, xs.c, gp.G); abort();
    }
    return ws;
}
int umx_gn_sums_pm32(const float *x, int N, int C, int G, size_t S, double *sums, size_t v0, size_t v1);
__global__ void f32_to_h16_k(const float *__restrict__ x, __half *__restrict__ y, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) y[i] = __float2half_rn(x[i]);
}
static void not_built(const char *fn, const char *what) { fprintf(stderr, "%s: %s is not built in this library\n", fn, what); abort(); }

/* ---- split_t: concat input, upsampled input segment, split output, output statistics ----
   These fields are served by composition: the conv's operand tensor is assembled in scratch from its segments, the conv runs on it,
   and a split output is dealt out of a scratch tensor.  The arithmetic is the reference's (its kernels do the same steps while
   staging: transform, blend, quantise rows of 32 channels to the MMA's format); the extra passes over memory are the price. */
int umx_gn_silu_apply_seg(const void *x, int xdt, int N, int C, size_t S, int G, const float *gamma, const float *beta, const float *mean, const float *rstd,
                          void *y, int bits, int layout, int form, int c_off, int C_all);
extern "C" void umx_pm_to_mx32_cat(const void *x, const void *x2, int c2, int dt, int N, int C, size_t S, void *y, int bits, int layout);
static inline int up32(int c) { return (c + 31) / 32 * 32; }

/* blocks [0, nb_src) of every sample of an MX tensor (reference layout) to blocks [b0, b0 + nb_src) of one with nb_dst blocks, or back */
static void mx_blocks_copy(uint8_t *dst, int nb_dst, int b0, const uint8_t *src, int nb_src, int N, size_t S, int bits, bool gather) {
    const size_t rb = bits == 8 ? 32 : 16;
    for (int n = 0; n < N; n++) {
        uint8_t *dc = dst + ((size_t)n * nb_dst + b0) * S * rb, *ds = dst + (size_t)N * nb_dst * S * rb + ((size_t)n * nb_dst + b0) * S;
        const uint8_t *sc = src + (size_t)n * nb_src * S * rb, *ss = src + (size_t)N * nb_src * S * rb + (size_t)n * nb_src * S;
        if (gather) {          /* dst is the small tensor */
            cudaMemcpyAsync((uint8_t *)sc, dc, (size_t)nb_src * S * rb, cudaMemcpyDeviceToDevice, 0);
            cudaMemcpyAsync((uint8_t *)ss, ds, (size_t)nb_src * S, cudaMemcpyDeviceToDevice, 0);
        } else {
            cudaMemcpyAsync(dc, sc, (size_t)nb_src * S * rb, cudaMemcpyDeviceToDevice, 0);
            cudaMemcpyAsync(ds, ss, (size_t)nb_src * S, cudaMemcpyDeviceToDevice, 0);
        }
    }
}
/* weights [co][ci][taps] and bias of the logical conv -> those of the conv on padded segments: input channel ci sits at ci (ci < cx) or
   cxp + ci - cx, output channel co at co (co < ox) or oxp + co - ox; rows and columns of the padding are zero */
__global__ void w_expand_k(const float *__restrict__ w, const float *__restrict__ b, float *__restrict__ wp, float *__restrict__ bp,
                           int co_n, int ci_n, int taps, int cx, int cxp, int cip, int ox, int oxp, int cop) {
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x, n = (size_t)cop * cip * taps;
    if (i < (size_t)cop) { const int p = (int)i, co = p < oxp ? (p < ox ? p : -1) : ox + p - oxp; bp[i] = (b && co >= 0 && co < co_n) ? b[co] : 0.f; }
    if (i >= n) return;
    const int t = (int)(i % taps), pi = (int)((i / taps) % cip), po = (int)(i / ((size_t)taps * cip));
    const int ci = pi < cxp ? (pi < cx ? pi : -1) : cx + pi - cxp, co = po < oxp ? (po < ox ? po : -1) : ox + po - oxp;
    wp[i] = (ci >= 0 && ci < ci_n && co >= 0 && co < co_n) ? w[((size_t)co * ci_n + ci) * taps + t] : 0.f;
}

extern "C" void umx_mx_rewidth(const void *x, int bits, int N, int C, size_t S, void *y, int to_wide);
static inline bool any_gn_(const gnp_t &gp, const split_t &sp) { return gp.G || sp.gp2.G; }

/* ---- z slabs (split_t.zi0 / Di, zw0 / zw1, yD / yzo) and accumulate ----
   A conv over a range of z planes is the same conv on a copy of the input planes it reads: planes [first, first + nz) of every
   (sample, channel block) of a tensor of depth D, zeros where the range leaves the tensor. */
struct tdesc { size_t rows, plane_b, sc_rows; int rb; };     /* rows of `plane_b` bytes per z plane; MX: as many scale rows of H W bytes per plane */
static tdesc tensor_desc(int bf, int N, int C, size_t hw) {
    tdesc t = {0, 0, 0, 0};
    if (bf == UMX_F16) { t.rows = (size_t)N * C; t.plane_b = hw * 2; }
    else {
        const int bits = bf == UMX_MX8 ? 8 : 4, bw = C <= 8 ? 8 : C <= 16 ? 16 : 32;
        t.rb = bw * bits / 8; t.rows = (size_t)N * ((C + bw - 1) / bw); t.plane_b = hw * t.rb; t.sc_rows = t.rows;
    }
    return t;
}
static size_t tensor_bytes(const tdesc &t, int D, size_t hw) { return t.rows * D * t.plane_b + t.sc_rows * D * hw; }
/* dst planes [dz, dz + nz) of depth Dd <- src planes [sz, sz + nz) of depth Ds (both ranges inside their tensors) */
static void planes_copy(void *dst, int Dd, int dz, const void *src, int Ds, int sz, int nz, const tdesc &t, size_t hw) {
    if (nz <= 0) return;
    cudaMemcpy2DAsync((uint8_t *)dst + (size_t)dz * t.plane_b, (size_t)Dd * t.plane_b, (const uint8_t *)src + (size_t)sz * t.plane_b, (size_t)Ds * t.plane_b, (size_t)nz * t.plane_b, t.rows, cudaMemcpyDeviceToDevice, 0);
    if (t.sc_rows) {
        const uint8_t *ss = (const uint8_t *)src + t.rows * Ds * t.plane_b; uint8_t *ds = (uint8_t *)dst + t.rows * Dd * t.plane_b;
        cudaMemcpy2DAsync(ds + (size_t)dz * hw, (size_t)Dd * hw, ss + (size_t)sz * hw, (size_t)Ds * hw, (size_t)nz * hw, t.sc_rows, cudaMemcpyDeviceToDevice, 0);
    }
}
static void *slab_of(int slot, const void *x, int bf, int N, int C, int D, size_t hw, int first, int nz) {
    const tdesc t = tensor_desc(bf, N, C, hw);
    void *s = umx_ws(slot, tensor_bytes(t, nz, hw));
    if (!s) return nullptr;
    cudaMemsetAsync(s, 0, tensor_bytes(t, nz, hw), 0);          /* zero codes under a zero scale byte: the value 0 */
    const int a = first < 0 ? 0 : first, e = first + nz > D ? D : first + nz;
    planes_copy(s, nz, a - first, x, D, a, e - a, t, hw);
    return s;
}
/* y (fp16 plane-major, n elements) += t */
__global__ void __launch_bounds__(256) h16_add_k(__half *__restrict__ y, const __half *__restrict__ t, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) y[i] = __float2half_rn(__fadd_rn(__half2float(y[i]), __half2float(t[i])));
}

static int conv_fwd(const char *fn, int bits, const void *x, int xbf, shape5 xs, const float *w, const float *b, int cout, void *y, int ybf, gnp_t gp, double *osum, int Go, split_t sp) {
    if (!umx_ready(fn)) return 0;
    if (sp.sr || sp.osr) not_built(fn, "stochastic rounding (split_t.sr / osr)");
    /* o_pad places the second output tensor's rows inside the reference's padded GEMM (src/nn_lp.h:32): here each output tensor has its own
       blocks whatever it says; the values the reference uses are accepted */
    if (sp.o_pad && !(sp.y2 && (sp.o_pad == 16 || sp.o_pad == (sp.o_split + 31) / 32 * 32))) { fprintf(stderr, "%s: split_t.o_pad %d with o_split %d\n", fn, (int)sp.o_pad, sp.o_split); abort(); }
    if (sp.accum) {
        /* y += conv: the conv into scratch, then one rounding of the fp16 sum (the reference adds in its epilogue, src/lp_common.cuh:1567-1571,
           and rounds once as well, but from the fp32 accumulator: the two can differ by the rounding of the conv's own fp16 result) */
        if (ybf != UMX_F16 || sp.y2 || osum) not_built(fn, "split_t.accum with an output that is not one fp16 plane-major tensor, or with output statistics");
        const int Dy = sp.yD ? sp.yD : xs.d;
        const size_t ny = (size_t)xs.n * cout * Dy * xs.h * xs.w;
        __half *t = (__half *)umx_ws(11, ny * 2);
        if (!t) return 0;
        if (sp.yD || sp.zw1) cudaMemsetAsync(t, 0, ny * 2, 0);     /* planes the conv does not write add nothing */
        split_t s2 = sp; s2.accum = 0;
        conv_fwd(fn, bits, x, xbf, xs, w, b, cout, t, ybf, gp, nullptr, 0, s2);
        size_t g = (ny + 255) / 256; if (g > 148u * 16u) g = 148u * 16u;
        if (ny) h16_add_k<<<(unsigned)g, 256>>>((__half *)y, t, ny);
        UMX_CK(fn);
        return 0;
    }
    if (sp.zi0 || sp.Di || sp.zw0 || sp.zw1 || sp.yD || sp.yzo) {
        if (sp.up) not_built(fn, "a z range / z window / slab output together with split_t.up");
        if ((sp.Di || sp.zi0) && sp.zw1) not_built(fn, "a z range and a z window in one call");
        if (ybf == UMX_H16B) not_built(fn, "a z range / z window with a blocked fp16 output");
        const size_t hw = (size_t)xs.h * xs.w;
        const int Din = sp.Di ? sp.Di : xs.d;                                   /* depth of the input tensors */
        const int z0 = sp.zw1 ? sp.zw0 : 0, z1 = sp.zw1 ? sp.zw1 : xs.d;         /* output planes of this launch, in the launch's own counting */
        if (z0 < 0 || z1 > xs.d || z1 <= z0) { fprintf(stderr, "%s: z window [%d, %d) of %d planes\n", fn, z0, z1, xs.d); abort(); }
        const int nz = z1 - z0, Dy = sp.yD ? sp.yD : xs.d, yz = z0 + sp.yzo;
        if (yz < 0 || yz + nz > Dy) { fprintf(stderr, "%s: output planes [%d, %d) of a depth-%d tensor\n", fn, yz, yz + nz, Dy); abort(); }
        const int Cx = sp.x2 ? sp.c_split : xs.c;
        /* the conv on nz + 2 planes: input planes z0 + zi0 - 1 .. z1 + zi0; its first and last output plane are thrown away */
        const int first = z0 + sp.zi0 - 1;
        const void *xa = slab_of(8, x, xbf, xs.n, Cx, Din, hw, first, nz + 2);
        if (!xa) return 0;
        split_t s2 = sp; s2.zi0 = s2.Di = s2.zw0 = s2.zw1 = s2.yD = s2.yzo = 0;
        if (gp.G || sp.gp2.G) {
            /* the transform belongs to the voxels of the tensor; the planes beyond its ends stay zero (the reference stages them as zeros): transform
               the slab here, clear those planes again, and hand the conv a plain MX tensor */
            if (sp.x2 || xs.c <= 16) not_built(fn, "a GroupNorm transform on a z range of a concat input or of 16 channels or fewer");
            const int mxf = bits == 8 ? UMX_MX8 : UMX_MX4;
            const tdesc tm = tensor_desc(mxf, xs.n, xs.c, hw);
            uint8_t *g = (uint8_t *)umx_ws(9, tensor_bytes(tm, nz + 2, hw));
            if (!g) return 0;
            slab_check(fn, gp, xs);                            /* local plane zl of the copy is plane zl + first of the tensor the slabs are counted in */
            if (umx_gn_silu_apply_seg_slabs(xa, xbf, xs.n, xs.c, (size_t)(nz + 2) * hw, gp.G, gp.gamma, gp.beta, gp.mean, gp.rstd, g, bits, UMX_LAYOUT_REF, 1, 0, xs.c,
                                            gp.ns, gp.zs, gp.zo + first, hw) != 0) not_built(fn, "this GroupNorm transform");
            const int lo = first < 0 ? -first : 0, hi = first + nz + 2 > Din ? first + nz + 2 - Din : 0;      /* planes before / after the tensor */
            for (int side = 0; side < 2; side++) {
                const int np = side ? hi : lo, p0 = side ? nz + 2 - hi : 0;
                if (!np) continue;
                cudaMemset2DAsync(g + (size_t)p0 * tm.plane_b, (size_t)(nz + 2) * tm.plane_b, 0, (size_t)np * tm.plane_b, tm.rows, 0);
                cudaMemset2DAsync(g + tm.rows * (nz + 2) * tm.plane_b + (size_t)p0 * hw, (size_t)(nz + 2) * hw, 0, (size_t)np * hw, tm.sc_rows, 0);
            }
            xa = g; xbf = mxf; gp.G = 0;
        }
        if (sp.x2) { s2.x2 = slab_of(9, sp.x2, xbf, xs.n, xs.c - Cx, Din, hw, z0 + sp.zi0 - 1, nz + 2); if (!s2.x2) return 0; }
        shape5 s5 = xs; s5.d = nz + 2;
        /* a split output: both parts through scratch tensors of nz + 2 planes; output statistics: the first and the last plane of the run are
           not output planes, so they join the planes the sums skip */
        const int Ox = sp.y2 ? sp.o_split : cout, O2 = cout - Ox;
        if (sp.y2 && (Ox < 1 || O2 < 1)) { fprintf(stderr, "%s: o_split %d of %d output channels\n", fn, Ox, cout); abort(); }
        const tdesc ty = tensor_desc(ybf, xs.n, Ox, hw), ty2 = tensor_desc(ybf, xs.n, sp.y2 ? O2 : 1, hw);
        void *t = umx_ws(10, tensor_bytes(ty, nz + 2, hw)), *t2 = nullptr;
        if (!t) return 0;
        if (sp.y2) { t2 = umx_ws(11, tensor_bytes(ty2, nz + 2, hw)); if (!t2) return 0; s2.y2 = t2; }
        if (osum) { s2.zlo = sp.zlo + 1; s2.zhi = sp.zhi + 1; }
        conv_fwd(fn, bits, xa, xbf, s5, w, b, cout, t, ybf, gp, osum, Go, s2);
        planes_copy(y, Dy, yz, t, nz + 2, 1, nz, ty, hw);
        if (sp.y2) planes_copy(sp.y2, Dy, yz, t2, nz + 2, 1, nz, ty2, hw);
        UMX_CK(fn);
        return 0;
    }
    if (sp.up && !sp.x2) { fprintf(stderr, "%s: split_t.up without x2\n", fn); abort(); }
    if (sp.gp2.G && !sp.x2) { fprintf(stderr, "%s: split_t.gp2 without x2\n", fn); abort(); }
    const int mxin = bits == 8 ? UMX_MX8 : UMX_MX4;
    const bool x_mx = xbf == UMX_MX8 || xbf == UMX_MX4;
    const int xb_bits = xbf == UMX_MX8 ? 8 : 4;
    const int Ci = xs.c, Cx = sp.x2 ? sp.c_split : Ci, C2 = Ci - Cx;
    if (sp.x2 && (Cx < 1 || C2 < 1)) { fprintf(stderr, "%s: c_split %d of %d input channels\n", fn, Cx, Ci); abort(); }
    if (sp.x2 && x_mx && (Cx <= 16 || C2 <= 16) && (any_gn_(gp, sp) || sp.up)) not_built(fn, "a transform of a concat input with a part of 16 channels or fewer (8 / 16-wide MX rows)");
    if (xbf != UMX_F16 && !x_mx) { fprintf(stderr, "%s: input storage %d (this entry takes fp16 plane-major or MX)\n", fn, xbf); abort(); }
    const bool any_gn = gp.G || sp.gp2.G;
    if (!any_gn && !sp.up && x_mx && xbf != mxin) { fprintf(stderr, "%s: an MX-fp%d input of an MX-fp%d conv needs a transform that requantises it\n", fn, xb_bits, bits); abort(); }
    if (sp.up && (!x_mx || ((xs.d | xs.h | xs.w) & 1))) not_built(fn, "split_t.up of a plane-major tensor or onto an odd grid");
    int out_mode, out_bits = 0;
    if (ybf == UMX_F16) out_mode = UMX_OUT_PM16;
    else if (ybf == UMX_MX8 || ybf == UMX_MX4) { out_mode = UMX_OUT_MXRAW; out_bits = ybf == UMX_MX8 ? 8 : 4; }
    else if (ybf == UMX_H16B) out_mode = UMX_OUT_H16B;
    else { fprintf(stderr, "%s: output storage %d\n", fn, ybf); abort(); }
    const bool narrow_out = out_mode == UMX_OUT_MXRAW && cout <= 16 && !sp.y2;      /* rows of 8 / 16 channels: written 32 wide into scratch, then narrowed */
    const int Ox = sp.y2 ? sp.o_split : cout, O2 = cout - Ox;
    if (sp.y2 && (Ox < 1 || O2 < 1)) { fprintf(stderr, "%s: o_split %d of %d output channels\n", fn, Ox, cout); abort(); }
    if (sp.y2 && out_mode == UMX_OUT_H16B) not_built(fn, "a split output in blocked fp16");
    if (osum || Go) {
        if (!osum || Go < 1) { fprintf(stderr, "%s: osum %p with %d groups\n", fn, (void *)osum, Go); abort(); }
        if (sp.stored_stats) {
            if (out_mode != UMX_OUT_MXRAW) not_built(fn, "statistics of a stored output that is not MX");
            if (sp.y2 && ((Ox & 31) || O2 <= 16)) not_built(fn, "output statistics of a split output whose first part does not end on a 32-channel block");
        } else if (sp.y2 || out_mode == UMX_OUT_H16B) not_built(fn, "statistics of the unrounded output (split_t.stored_stats 0) of a split or blocked fp16 output");
        if (Go > 64 || cout % Go) { fprintf(stderr, "%s: %d output channels in %d groups\n", fn, cout, Go); abort(); }
    }
    const size_t S = (size_t)xs.d * xs.h * xs.w;
    if (!S || !xs.n) return 0;

    /* ---- the operand tensor ---- */
    const void *xq = x; int cin = Ci, xflags = 0;
    const bool s2g = sp.x2 && sp.gp2.G;                       /* a GroupNorm per segment; otherwise gp counts its groups over all Ci channels */
    if (!sp.x2) {
        const void *xw = x;
        if (x_mx && Ci <= 16) {                                /* rows of 8 / 16 channels: the same codes and scale in a 32-wide row */
            void *ws = umx_ws(3, umx_mx_bytes32(xb_bits, xs.n, Ci, S));
            if (!ws) return 0;
            umx_mx_rewidth(x, xb_bits, xs.n, Ci, S, ws, 1);
            xw = xq = ws;
        }
        if (gp.G) { xq = gn_input(fn, xw, xbf, xs, gp, bits); if (!xq) return 0; xflags = UMX_X_SPLIT; }
        else if (xbf == UMX_F16) {
            void *ws = umx_ws(0, umx_mx_bytes32(bits, xs.n, Ci, S));
            if (!ws) return 0;
            umx_pm_to_mx32(x, UMX_F16, xs.n, Ci, S, ws, bits, UMX_LAYOUT_SPLIT);
            xq = ws; xflags = UMX_X_SPLIT;
        }
    } else if (!x_mx && !any_gn) {                             /* two plane-major tensors: quantised in one pass, blocks over the concatenated index */
        void *ws = umx_ws(0, umx_mx_bytes32(bits, xs.n, Ci, S));
        if (!ws) return 0;
        umx_pm_to_mx32_cat(x, sp.x2, Cx, UMX_F16, xs.n, Ci, S, ws, bits, UMX_LAYOUT_SPLIT);
        xq = ws; xflags = UMX_X_SPLIT;
    } else {
        /* segment by segment into an MX tensor of the conv's format (reference layout).  MX segments keep their own 32-channel blocks,
           the x part padded to whole blocks (the reference's "per-tensor 32-channel segments", src/lp_f8fwd.cuh:617-623) */
        if (!x_mx && (Cx & 31)) not_built(fn, "a GroupNorm transform of plane-major concat inputs split inside a 32-channel block");
        const int CxP = up32(Cx), nbA = CxP / 32, nbB = up32(C2) / 32, nbT = nbA + nbB;
        cin = nbT * 32;
        uint8_t *T = (uint8_t *)umx_ws(6, umx_mx_bytes32(bits, xs.n, cin, S));
        if (!T) return 0;
        for (int seg = 0; seg < 2; seg++) {
            const void *src = seg ? sp.x2 : x;
            const int C = seg ? C2 : Cx, nbs = seg ? nbB : nbA, b0 = seg ? nbA : 0;
            const gnp_t q = s2g ? (seg ? sp.gp2 : gp) : gp;
            const int c_off = s2g ? 0 : (seg ? Cx : 0), C_all = s2g ? C : Ci;
            const bool up = !seg && sp.up;
            const uint8_t *blocks = nullptr;
            if (up) {
                if (q.G && !s2g) not_built(fn, "split_t.up with one GroupNorm over both input parts");
                uint8_t *t = (uint8_t *)umx_ws(3, umx_mx_bytes32(bits, xs.n, C, S));
                if (!t) return 0;
                const shape5 cs = {xs.n, C, xs.d / 2, xs.h / 2, xs.w / 2};
                lp_up2_fwd_mx(src, xbf, cs, t, mxin, q);        /* silu(gn(coarse)) blended, quantised to the conv's rows */
                blocks = t;
            } else if (q.G) {
                uint8_t *t = (uint8_t *)umx_ws(3 + seg, umx_mx_bytes32(bits, xs.n, C, S));
                if (!t) return 0;
                slab_check(fn, q, xs);
                if (umx_gn_silu_apply_seg_slabs(src, xbf, xs.n, C, S, q.G, q.gamma, q.beta, q.mean, q.rstd, t, bits, UMX_LAYOUT_REF, 1, c_off, C_all, q.ns, q.zs, q.zo, (size_t)q.zhw) != 0) {
                    fprintf(stderr, "%s: the GroupNorm + SiLU input transform of a storage-%d segment of %d channels (%d groups over %d) is not built in this library\n", fn, xbf, C, q.G, C_all); abort();
                }
                blocks = t;
            } else if (x_mx) {
                if (xbf != mxin) { fprintf(stderr, "%s: an MX-fp%d input segment of an MX-fp%d conv without a transform\n", fn, xb_bits, bits); abort(); }
                blocks = (const uint8_t *)src;
                if (C <= 16) {                                 /* rows of 8 / 16 channels: the same codes and scale in a 32-wide row */
                    uint8_t *t = (uint8_t *)umx_ws(3 + seg, umx_mx_bytes32(bits, xs.n, C, S));
                    if (!t) return 0;
                    umx_mx_rewidth(src, bits, xs.n, C, S, t, 1);
                    blocks = t;
                }
            } else {
                uint8_t *t = (uint8_t *)umx_ws(3 + seg, umx_mx_bytes32(bits, xs.n, C, S));
                if (!t) return 0;
                umx_pm_to_mx32(src, UMX_F16, xs.n, C, S, t, bits, UMX_LAYOUT_REF);
                blocks = t;
            }
            mx_blocks_copy(T, nbT, b0, blocks, nbs, xs.n, S, bits, false);
        }
        xq = T;
    }

    /* ---- the conv on padded segments where a segment does not end on a block ---- */
    const bool pad_in = sp.x2 && cin != Ci, mx_split_out = sp.y2 && out_mode == UMX_OUT_MXRAW, pad_out = mx_split_out && (Ox & 31);
    const int OxP = pad_out ? up32(Ox) : Ox, cout_c = pad_out ? OxP + O2 : cout;
    int dev = 0; cudaGetDevice(&dev);
    umx_conv *c = nullptr; bool temp = true;
    if (sp.wkey) {
        for (int i = 0; i < g_nmemo; i++) { memo_t &m = g_memo[i]; if (m.wkey == sp.wkey && m.w == w && m.b == b && m.cout == cout_c && m.cin == cin && m.bits == bits && m.dev == dev) { c = m.c; break; } }
        temp = false;
    }
    if (!c) {
        const float *wc = w, *bc = b;
        if (pad_in || pad_out) {
            const size_t nw = (size_t)cout_c * cin * 27;
            float *wp = (float *)umx_ws(5, (nw + cout_c) * sizeof(float));     /* slot 5 is also the general kernel's K-split scratch: the weights are prepared (and the stream drained) before a launch asks for it */
            if (!wp) return 0;
            w_expand_k<<<(unsigned)((nw + 255) / 256), 256>>>(w, b, wp, wp + nw, cout, Ci, 27, pad_in ? Cx : Ci, pad_in ? up32(Cx) : Ci, cin, Ox, OxP, cout_c);
            wc = wp; bc = wp + nw;
        }
        c = umx_conv_create_dev(UMX_CONV3, wc, bc, cout_c, cin, bits);
        if (!c) return 0;
        if (sp.wkey && g_nmemo < 256) { memo_t m = {sp.wkey, w, b, cout_c, cin, bits, dev, c}; g_memo[g_nmemo++] = m; } else temp = true;
    }
    if (osum && !sp.stored_stats) {
        /* statistics of acc + bias before any rounding (the reference's epilogue sums its fp32 values, src/lp_common.cuh:1465-1598): the conv
           into a plane-major fp32 scratch tensor, exact sums of that, and the output tensor made from it (MX(acc + bias), or its fp16 rounding) */
        float *P = (float *)umx_ws(7, (size_t)xs.n * cout * S * 4);
        if (!P) return 0;
        umx_conv_fwd(c, xq, xs.n, xs.d, xs.h, xs.w, P, UMX_OUT_PM32, 0, 0, 0, nullptr, xflags);
        const size_t hw = (size_t)xs.h * xs.w, v0 = (size_t)sp.zlo * hw, v1 = S - (size_t)sp.zhi * hw;
        if (sp.zlo < 0 || sp.zhi < 0 || sp.zlo + sp.zhi > xs.d) { fprintf(stderr, "%s: zlo %d + zhi %d of %d planes\n", fn, sp.zlo, sp.zhi, xs.d); abort(); }
        if (umx_gn_sums_pm32(P, xs.n, cout, Go, S, osum, v0, v1) != 0) { fprintf(stderr, "%s: output statistics of %d channels in %d groups\n", fn, cout, Go); abort(); }
        if (out_mode == UMX_OUT_MXRAW) { if (out_bits == 8) lp_f32_to_mx8(P, xs.n, cout, S, y); else lp_f32_to_mx4(P, xs.n, cout, S, y); }
        else { const size_t ny = (size_t)xs.n * cout * S; size_t g = (ny + 255) / 256; if (g > 148u * 16u) g = 148u * 16u; f32_to_h16_k<<<(unsigned)g, 256>>>(P, (__half *)y, ny); }
    } else if (narrow_out) {
        void *t = umx_ws(4, umx_mx_bytes32(out_bits, xs.n, cout, S));
        if (!t) return 0;
        umx_conv_fwd(c, xq, xs.n, xs.d, xs.h, xs.w, t, out_mode, out_bits, 0, 0, nullptr, xflags);
        umx_mx_rewidth(t, out_bits, xs.n, cout, S, y, 0);
    } else if (!sp.y2) {
        umx_conv_fwd(c, xq, xs.n, xs.d, xs.h, xs.w, y, out_mode, out_bits, 0, 0, nullptr, xflags);   /* MX tensors of the reference interface keep the reference layout */
    } else if (out_mode == UMX_OUT_PM16) {
        __half *t = (__half *)umx_ws(4, (size_t)xs.n * cout * S * 2);
        if (!t) return 0;
        umx_conv_fwd(c, xq, xs.n, xs.d, xs.h, xs.w, t, out_mode, 0, 0, 0, nullptr, xflags);
        for (int n = 0; n < xs.n; n++) {
            cudaMemcpyAsync((__half *)y + (size_t)n * Ox * S, t + (size_t)n * cout * S, (size_t)Ox * S * 2, cudaMemcpyDeviceToDevice, 0);
            cudaMemcpyAsync((__half *)sp.y2 + (size_t)n * O2 * S, t + ((size_t)n * cout + Ox) * S, (size_t)O2 * S * 2, cudaMemcpyDeviceToDevice, 0);
        }
    } else {
        const int nb1 = up32(Ox) / 32, nb2 = up32(O2) / 32;
        uint8_t *t = (uint8_t *)umx_ws(4, umx_mx_bytes32(out_bits, xs.n, (nb1 + nb2) * 32, S));
        if (!t) return 0;
        umx_conv_fwd(c, xq, xs.n, xs.d, xs.h, xs.w, t, out_mode, out_bits, 0, 0, nullptr, xflags);
        for (int part = 0; part < 2; part++) {
            const int Cp = part ? O2 : Ox, nbp = part ? nb2 : nb1, b0 = part ? nb1 : 0;
            uint8_t *dst = (uint8_t *)(part ? sp.y2 : y);
            if (Cp > 16) { mx_blocks_copy(t, nb1 + nb2, b0, dst, nbp, xs.n, S, out_bits, true); continue; }
            uint8_t *one = (uint8_t *)umx_ws(7, umx_mx_bytes32(out_bits, xs.n, Cp, S));      /* a part of 16 channels or fewer is stored in rows of 8 / 16 */
            if (!one) return 0;
            mx_blocks_copy(t, nb1 + nb2, b0, one, 1, xs.n, S, out_bits, true);
            umx_mx_rewidth(one, out_bits, xs.n, Cp, S, dst, 0);
        }
        if (osum) {                                            /* Ox ends on a block: the scratch tensor is the cout-channel output */
            const size_t hw = (size_t)xs.h * xs.w, v0 = (size_t)sp.zlo * hw, v1 = S - (size_t)sp.zhi * hw;
            if (sp.zlo < 0 || sp.zhi < 0 || sp.zlo + sp.zhi > xs.d) { fprintf(stderr, "%s: zlo %d + zhi %d of %d planes\n", fn, sp.zlo, sp.zhi, xs.d); abort(); }
            if (lp_gn_sums_mx(t, ybf, xs.n, cout, Go, S, osum, v0, v1) != 0) { fprintf(stderr, "%s: output statistics of %d channels in %d groups\n", fn, cout, Go); abort(); }
        }
    }
    if (osum && !sp.y2 && sp.stored_stats) {
        /* statistics of the stored values (split_t.stored_stats) over the planes [zlo, D - zhi): exact sums into the caller's slots */
        const size_t hw = (size_t)xs.h * xs.w, v0 = (size_t)sp.zlo * hw, v1 = S - (size_t)sp.zhi * hw;
        if (sp.zlo < 0 || sp.zhi < 0 || sp.zlo + sp.zhi > xs.d) { fprintf(stderr, "%s: zlo %d + zhi %d of %d planes\n", fn, sp.zlo, sp.zhi, xs.d); abort(); }
        if (lp_gn_sums_mx(y, ybf, xs.n, cout, Go, S, osum, v0, v1) != 0) { fprintf(stderr, "%s: output statistics of %d channels in %d groups\n", fn, cout, Go); abort(); }
    }
    if (temp) { cudaDeviceSynchronize(); umx_conv_free(c); }
    UMX_CK(fn);
    return 0;
}
extern "C" int lp_conv_fwd_f8(const void *x, int xbf, shape5 xs, const float *w, const float *b, int cout, void *y, int ybf, gnp_t gp, double *osum, int Go, split_t sp) {
    return conv_fwd("lp_conv_fwd_f8", 8, x, xbf, xs, w, b, cout, y, ybf, gp, osum, Go, sp);
}
extern "C" int lp_conv_fwd_f4(const void *x, int xbf, shape5 xs, const float *w, const float *b, int cout, void *y, int ybf, gnp_t gp, double *osum, int Go, split_t sp) {
    return conv_fwd("lp_conv_fwd_f4", 4, x, xbf, xs, w, b, cout, y, ybf, gp, osum, Go, sp);
}

extern "C" int lp_conv_fwd_s2_f8(const void *x, int xbf, shape5 xs, const float *w, const float *b, int cout, void *y, int ybf, shape5 ys, gnp_t gp) {
    const char *fn = "lp_conv_fwd_s2_f8";
    if (!umx_ready(fn)) return 0;
    const bool x_mx = xbf == UMX_MX8 || xbf == UMX_MX4;
    if (xbf != UMX_F16 && !x_mx) { fprintf(stderr, "%s: input storage %d (this entry takes fp16 plane-major, MX-fp8 or MX-fp4)\n", fn, xbf); abort(); }
    if (ys.n != xs.n || ys.c != cout || ys.d != (xs.d + 1) / 2 || ys.h != (xs.h + 1) / 2 || ys.w != (xs.w + 1) / 2) {
        fprintf(stderr, "%s: output shape %d x %d x %d x %d x %d does not follow from the input\n", fn, ys.n, ys.c, ys.d, ys.h, ys.w); abort();
    }
    int out_mode, out_bits = 0;
    if (ybf == UMX_F16) out_mode = UMX_OUT_PM16;
    else if (ybf == UMX_MX8 || ybf == UMX_MX4) { out_mode = UMX_OUT_MXRAW; out_bits = ybf == UMX_MX8 ? 8 : 4; }
    else if (ybf == UMX_H16B) out_mode = UMX_OUT_H16B;
    else { fprintf(stderr, "%s: output storage %d\n", fn, ybf); abort(); }
    const size_t S = (size_t)xs.d * xs.h * xs.w, So = (size_t)ys.d * ys.h * ys.w;
    if (!S || !xs.n) return 0;
    /* An MX-fp4 input that needs no GroupNorm is multiplied as MX-fp4 (weights quantised to E2M1): the reference's conv_fwd_s2_f4_k /
       conv_fwd_s2_f4p_k cases (src/lp_s2.cu:652-716), reported by the return value 3.  Everything else computes in MX-fp8; a GroupNorm
       input is transformed and requantised to MX-fp8 first, as the reference's s2_prenorm_k path does (src/lp_s2.cu:733-744). */
    const int bits = (xbf == UMX_MX4 && !gp.G) ? 4 : 8;
    const void *xq = x; int xflags = 0;
    if (x_mx && xs.c <= 16) {                                  /* rows of 8 / 16 channels: the same codes and scale in a 32-wide row */
        const int xb = xbf == UMX_MX8 ? 8 : 4;
        void *ws = umx_ws(3, umx_mx_bytes32(xb, xs.n, xs.c, S));
        if (!ws) return 0;
        umx_mx_rewidth(x, xb, xs.n, xs.c, S, ws, 1);
        xq = ws;
    }
    if (gp.G) { xq = gn_input(fn, xq, xbf, xs, gp, 8); if (!xq) return 0; xflags = UMX_X_SPLIT; }
    else if (xbf == UMX_F16) {
        void *ws = umx_ws(0, umx_mx_bytes32(8, xs.n, xs.c, S));
        if (!ws) return 0;
        umx_pm_to_mx32(x, UMX_F16, xs.n, xs.c, S, ws, 8, UMX_LAYOUT_SPLIT);
        xq = ws; xflags = UMX_X_SPLIT;
    }
    /* an MX output of 16 channels or fewer is stored in rows of 8 / 16: the conv writes 32-wide rows into scratch, which are narrowed */
    const bool narrow = out_mode == UMX_OUT_MXRAW && cout <= 16;
    void *yq = y;
    if (narrow) { yq = umx_ws(4, umx_mx_bytes32(out_bits, xs.n, cout, So)); if (!yq) return 0; }
    umx_conv *c = umx_conv_create_dev(UMX_CONV3S2, w, b, cout, xs.c, bits);
    if (!c) return 0;
    umx_conv_fwd(c, xq, xs.n, xs.d, xs.h, xs.w, yq, out_mode, out_bits, 0, 0, nullptr, xflags);
    if (narrow) umx_mx_rewidth(yq, out_bits, xs.n, cout, So, y, 0);
    cudaDeviceSynchronize();
    umx_conv_free(c);
    return bits == 4 ? 3 : 0;
}
