/* The reference's conv entry points lp_conv_fwd_f8 / lp_conv_fwd_f4 / lp_conv_fwd_s2_f8 (src/nn_lp.h:53-54, 104) on top of the tcgen05
   conv: same signature, storage codes and error behaviour; the prepared weights are memoised under split_t.wkey as the reference's fp4
   kernel does (src/lp_f4fwd.cuh:748-770). */
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
static const void *gn_input(const char *fn, const void *x, int xbf, shape5 xs, gnp_t gp, int bits) {
    if (gp.ns > 1 || gp.zs || gp.zo || gp.zhw) { fprintf(stderr, "%s: slab-local GroupNorm (gnp_t.ns / zs / zo / zhw) is not built in this library\n", fn); abort(); }
    const size_t S = (size_t)xs.d * xs.h * xs.w;
    void *ws = umx_ws(2, umx_mx_bytes32(bits, xs.n, xs.c, S));
    if (!ws) return nullptr;
    if (umx_gn_silu_apply(x, xbf, xs.n, xs.c, S, gp.G, gp.gamma, gp.beta, gp.mean, gp.rstd, ws, bits, UMX_LAYOUT_SPLIT, 1) != 0) {
        fprintf(stderr, "%s: the GroupNorm + SiLU input transform of a storage-%d tensor of %d channels in %d groups is not built in this library\n", fn, xbf, xs.c, gp.G); abort();
    }
    return ws;
}
static void not_built(const char *fn, const char *what) { fprintf(stderr, "%s: %s is not built in this library\n", fn, what); abort(); }

static int conv_fwd(const char *fn, int bits, const void *x, int xbf, shape5 xs, const float *w, const float *b, int cout, void *y, int ybf, gnp_t gp, double *osum, int Go, split_t sp) {
    if (!umx_ready(fn)) return 0;
    if (osum || Go) not_built(fn, "output GroupNorm statistics (osum)");
    if (sp.x2 || sp.y2 || sp.accum || sp.gp2.G || sp.up || sp.yD || sp.sr || sp.osr || sp.zlo || sp.zhi || sp.stored_stats || sp.zi0 || sp.Di || sp.zw0 || sp.zw1 || sp.yzo || sp.c_split || sp.o_split || sp.o_pad)
        not_built(fn, "a non-zero split_t field other than wkey");
    if (xs.c <= 16) not_built(fn, "an input of 16 channels or fewer (8 / 16-wide MX rows)");
    const int mxin = bits == 8 ? UMX_MX8 : UMX_MX4;
    if (!gp.G && xbf != UMX_F16 && xbf != mxin) { fprintf(stderr, "%s: input storage %d (this entry takes fp16 plane-major or MX-fp%d)\n", fn, xbf, bits); abort(); }
    int out_mode, out_bits = 0;
    if (ybf == UMX_F16) out_mode = UMX_OUT_PM16;
    else if (ybf == UMX_MX8 || ybf == UMX_MX4) { out_mode = UMX_OUT_MXRAW; out_bits = ybf == UMX_MX8 ? 8 : 4; if (cout <= 16) not_built(fn, "an MX output of 16 channels or fewer"); }
    else if (ybf == UMX_H16B) out_mode = UMX_OUT_H16B;
    else { fprintf(stderr, "%s: output storage %d\n", fn, ybf); abort(); }
    const size_t S = (size_t)xs.d * xs.h * xs.w;
    const void *xq = x;
    if (gp.G) { xq = gn_input(fn, x, xbf, xs, gp, bits); if (!xq) return 0; xbf = UMX_F16; /* = already quantised into the split layout */ }
    else if (xbf == UMX_F16) {
        void *ws = umx_ws(0, umx_mx_bytes32(bits, xs.n, xs.c, S));
        if (!ws) return 0;
        umx_pm_to_mx32(x, UMX_F16, xs.n, xs.c, S, ws, bits, UMX_LAYOUT_SPLIT);
        xq = ws;
    }
    int dev = 0; cudaGetDevice(&dev);
    umx_conv *c = nullptr; bool temp = true;
    if (sp.wkey) {
        for (int i = 0; i < g_nmemo; i++) { memo_t &m = g_memo[i]; if (m.wkey == sp.wkey && m.w == w && m.b == b && m.cout == cout && m.cin == xs.c && m.bits == bits && m.dev == dev) { c = m.c; break; } }
        temp = false;
    }
    if (!c) {
        c = umx_conv_create_dev(UMX_CONV3, w, b, cout, xs.c, bits);
        if (!c) return 0;
        if (sp.wkey && g_nmemo < 256) { memo_t m = {sp.wkey, w, b, cout, xs.c, bits, dev, c}; g_memo[g_nmemo++] = m; } else temp = true;
    }
    umx_conv_fwd(c, xq, xs.n, xs.d, xs.h, xs.w, y, out_mode, out_bits, 0, 0, nullptr, xbf == UMX_F16 ? UMX_X_SPLIT : 0);   /* MX tensors of the reference interface keep the reference layout */
    if (temp) { cudaDeviceSynchronize(); umx_conv_free(c); }
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
    if (xs.c <= 16) not_built(fn, "an input of 16 channels or fewer (8 / 16-wide MX rows)");
    if (!gp.G && xbf != UMX_F16 && xbf != UMX_MX8) { fprintf(stderr, "%s: input storage %d (this entry takes fp16 plane-major or MX-fp8)\n", fn, xbf); abort(); }
    if (ys.n != xs.n || ys.c != cout || ys.d != (xs.d + 1) / 2 || ys.h != (xs.h + 1) / 2 || ys.w != (xs.w + 1) / 2) {
        fprintf(stderr, "%s: output shape %d x %d x %d x %d x %d does not follow from the input\n", fn, ys.n, ys.c, ys.d, ys.h, ys.w); abort();
    }
    int out_mode, out_bits = 0;
    if (ybf == UMX_F16) out_mode = UMX_OUT_PM16;
    else if (ybf == UMX_MX8 || ybf == UMX_MX4) { out_mode = UMX_OUT_MXRAW; out_bits = ybf == UMX_MX8 ? 8 : 4; if (cout <= 16) not_built(fn, "an MX output of 16 channels or fewer"); }
    else if (ybf == UMX_H16B) out_mode = UMX_OUT_H16B;
    else { fprintf(stderr, "%s: output storage %d\n", fn, ybf); abort(); }
    const size_t S = (size_t)xs.d * xs.h * xs.w;
    const void *xq = x;
    if (gp.G) { xq = gn_input(fn, x, xbf, xs, gp, 8); if (!xq) return 0; xbf = UMX_F16; }
    else if (xbf == UMX_F16) {
        void *ws = umx_ws(0, umx_mx_bytes32(8, xs.n, xs.c, S));
        if (!ws) return 0;
        umx_pm_to_mx32(x, UMX_F16, xs.n, xs.c, S, ws, 8, UMX_LAYOUT_SPLIT);
        xq = ws;
    }
    umx_conv *c = umx_conv_create_dev(UMX_CONV3S2, w, b, cout, xs.c, 8);
    if (!c) return 0;
    umx_conv_fwd(c, xq, xs.n, xs.d, xs.h, xs.w, y, out_mode, out_bits, 0, 0, nullptr, xbf == UMX_F16 ? UMX_X_SPLIT : 0);
    cudaDeviceSynchronize();
    umx_conv_free(c);
    return 0;
}
