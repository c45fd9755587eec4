/* CPU oracle for the MX block-scaled 3-D convolution forward path of ufsm.

   TEST INFRASTRUCTURE ONLY.  This file is the checker: the parity tests, the smoke test and the CPU-baseline leg of the
   benchmark call it; the product library never links, loads or calls it.

   It restates, in plain C with OpenMP, the arithmetic the reference defines for this path (citations are paths inside the
   ufsm source tree):
     block exponent            src/lp_common.cuh:492-500 (mx_exp), host twin tests/test_mx4_wide.c:123-128
     e4m3 / e2m1 encoders      src/mx_sw.cuh:16-52 (bit-exact twins of cvt.rn.satfinite), tests/test_mx4_wide.c:129-143
     element decoders          src/mx_sw.cuh:77-87
     activation row quantiser  src/lp_mxops.cuh:46-68 (mx_store_row_b), src/lp_mx_cvt.cu:9-19 (f32_to_mx_k)
     MX storage layout         src/lp_common.cuh:100-106, 132-134; sizes src/lp_mx_cvt.cu:6-7
     weight blocks             src/lp_f8fwd.cu:54-71 (prep_w8_k), src/lp_f4fwd.cu:53-66 (prep_w4_k)
     emulated-MX conv          src/nn_xnet.cu:128-232 (k_fq / fq_host), :370-390 (fp16 store + InstanceNorm sums)
     InstanceNorm coefficient  src/nn_xnet.cu:1565-1570 (k_in_coef)
     fused apply + requantise  src/nn_xnet.cu:1577-1620 (k_inq), LeakyReLU src/nn_xnet.cu:122-126 (act_f)
     transposed conv as GEMM   src/nn_xnet.cu:650-657, 688-697, 1775-1789
     conv index maps           tests/test_mx4_wide.c:176-198 (gather)
     Gaussian window blend     src/nn_ink3dext.cu:58-73, src/ink3dext.c:8

   Parity pin: the encoders, decoders and the block exponent are checked over strided and exhaustive sweeps against the
   reference's own src/mx_sw.cuh compiled from where it lies (oracle/ref_pin.cu -> oracle/_ref/libmxsw_ref.so) and against
   the golden vectors in tests/golden/ that were generated from that build.

   Layouts.  "Blocked" tensors hold 32-channel blocks: element (n, c, v) of an N x C x S tensor lives at
   ((n * nb + c / 32) * S + v) * 32 + c % 32 with nb = ceil(C / 32); padding channels are zero.  An MX tensor is the blocked
   code array (32 B rows for fp8, 16 B rows of nibble pairs for fp4, low nibble = even channel) followed by the scale plane
   sc[(n * nb + blk) * S + v] (UE8M0).  Plane-major tensors are [n][C][S]. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <stdio.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 h16;

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ scalar definitions */

/* exponent e of the block scale 2^e: the exponent of amax * (1 / qmax) rounded up, clamped to [-126, 126]; a NaN or inf amax gives
   128 (scale byte 0xFF).  src/lp_common.cuh:492-500 */
int orc_mx_exp(float amax, float inv_qmax) {
    const volatile float p = amax * inv_qmax;
    const uint32_t u = f2u(p);
    if ((u & 0x7fffffffu) >= 0x7f800000u) return 128;
    const int e = (int)((u >> 23) & 0xffu) - 127 + ((u & 0x7fffffu) != 0);
    return e < -126 ? -126 : e > 126 ? 126 : e;
}
/* 2^e built from the exponent bits with unsigned wrap-around, as the reference's exp2i (src/lp_common.cuh:501): e = 128 gives -inf */
static inline float exp2i(int e) { return u2f((uint32_t)(127 + e) << 23); }

/* e4m3, round to nearest even, saturating, NaN -> 0x7f.  Written from the format definition (bias 7, 3 mantissa bits, subnormal
   step 2^-9, largest finite 448), not from the reference's integer code, so that the pin against src/mx_sw.cuh:16-37 compares two
   independent formulations. */
unsigned orc_enc_e4m3(float x) {
    const uint32_t u = f2u(x), s = (u >> 24) & 0x80u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return 0x7fu;
    float ax = u2f(a);
    if (ax >= 448.f) return s | 0x7eu;
    int ex; frexpf(ax, &ex); ex -= 1;                       /* ax in [2^ex, 2^(ex+1)) (ax = 0: ex = -1) */
    if (ax == 0.f || ex < -6) ex = -6;
    const double q = ldexp(1.0, ex - 3);                     /* spacing of the binade */
    double k = nearbyint((double)ax / q);                    /* default rounding mode: ties to even */
    double v = k * q;
    if (v > 448.0) v = 448.0;
    if (v == 0.0) return s;
    int e2; const double m = frexp(v, &e2); e2 -= 1;        /* v = (2m) 2^e2 */
    if (e2 < -6) return s | (unsigned)(v / ldexp(1.0, -9)); /* subnormal: multiples of 2^-9 */
    return s | ((unsigned)(e2 + 7) << 3) | (unsigned)((2.0 * m - 1.0) * 8.0);
}
/* e2m1 nibble: grid {0, .5, 1, 1.5, 2, 3, 4, 6}, ties to the even code, saturating, NaN -> +6 (src/mx_sw.cuh:38-52) */
unsigned orc_enc_e2m1(float x) {
    static const float G[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    const uint32_t u = f2u(x), s = (u >> 28) & 8u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return 7u;
    const float ax = u2f(a);
    if (ax >= 6.f) return s | 7u;
    int i = 0; while (i < 7 && G[i + 1] <= ax) i++;
    const float lo = ax - G[i], hi = G[i + 1] - ax;          /* exact: grid differences of floats this close */
    if (lo < hi) return s | (unsigned)i;
    if (hi < lo) return s | (unsigned)(i + 1);
    return s | (unsigned)((i & 1) ? i + 1 : i);
}
float orc_dec_e4m3(unsigned b) {                             /* src/mx_sw.cuh:77-83 */
    const unsigned e = (b >> 3) & 15u, m = b & 7u;
    if ((b & 0x7fu) == 0x7fu) return u2f(0x7fc00000u | ((b & 0x80u) << 24));
    const float v = e ? ldexpf((float)(8u + m), (int)e - 10) : ldexpf((float)m, -9);
    return (b & 0x80u) ? -v : v;
}
float orc_dec_e2m1(unsigned n) {                             /* src/mx_sw.cuh:84-87 */
    static const float G[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    const float v = G[n & 7u];
    return (n & 8u) ? -v : v;
}
/* UE8M0 scale byte -> factor: 2^(b - 127); 0xFF decodes as +inf so a non-finite block stays non-finite (src/lp_common.cuh:100-106) */
float orc_dec_scale(unsigned b) { b &= 0xffu; return b == 0xffu ? INFINITY : b == 0 ? ldexpf(1.f, -127) : u2f(b << 23); }

void orc_enc_e4m3_n(const float *x, size_t n, uint8_t *y) { for (size_t i = 0; i < n; i++) y[i] = (uint8_t)orc_enc_e4m3(x[i]); }
void orc_enc_e2m1_n(const float *x, size_t n, uint8_t *y) { for (size_t i = 0; i < n; i++) y[i] = (uint8_t)orc_enc_e2m1(x[i]); }

float orc_h16_round(float f) { return (float)(h16)f; }
void orc_f32_to_h16(const float *x, size_t n, uint16_t *y) {
#pragma omp parallel for
    for (size_t i = 0; i < n; i++) { const h16 h = (h16)x[i]; memcpy(&y[i], &h, 2); }
}
void orc_h16_to_f32(const uint16_t *x, size_t n, float *y) {
#pragma omp parallel for
    for (size_t i = 0; i < n; i++) { h16 h; memcpy(&h, &x[i], 2); y[i] = (float)h; }
}

/* ------------------------------------------------------------------ row quantiser */

/* One row of bw <= 32 values -> codes and scale byte (src/lp_mxops.cuh:46-68): NaN-propagating amax over the magnitude bits,
   e = mx_exp, codes = encode(v * 2^-e), byte = e + 127.  codes: one byte per value (the caller packs nibbles). */
static inline uint8_t quant_row(const float *v, int bw, int bits, uint8_t *codes) {
    uint32_t am = 0;
    for (int k = 0; k < bw; k++) { const uint32_t a = f2u(v[k]) & 0x7fffffffu; if (a > am) am = a; }
    const int e = orc_mx_exp(u2f(am), bits == 4 ? 1.f / 6.f : 1.f / 448.f);
    const float m = exp2i(-e);
    for (int k = 0; k < bw; k++) {
        const volatile float t = v[k] * m;
        codes[k] = (uint8_t)(bits == 4 ? orc_enc_e2m1(t) : orc_enc_e4m3(t));
    }
    return (uint8_t)(e + 127);
}
static inline void dequant_row(const uint8_t *codes, uint8_t sc, int bw, int bits, float *v) {
    const float s = orc_dec_scale(sc);
    for (int k = 0; k < bw; k++) v[k] = (bits == 4 ? orc_dec_e2m1(codes[k]) : orc_dec_e4m3(codes[k])) * s;
}
/* rows of exactly 32 floats -> MX rows (32 B or 16 B) + scale bytes */
void orc_quant_rows32(const float *v, size_t rows, int bits, uint8_t *q, uint8_t *sc) {
#pragma omp parallel for
    for (size_t r = 0; r < rows; r++) {
        uint8_t c[32]; sc[r] = quant_row(v + r * 32, 32, bits, c);
        if (bits == 4) for (int k = 0; k < 16; k++) q[r * 16 + k] = (uint8_t)(c[2 * k] | (c[2 * k + 1] << 4));
        else memcpy(q + r * 32, c, 32);
    }
}
void orc_dequant_rows32(const uint8_t *q, const uint8_t *sc, size_t rows, int bits, float *v) {
#pragma omp parallel for
    for (size_t r = 0; r < rows; r++) {
        uint8_t c[32];
        if (bits == 4) for (int k = 0; k < 16; k++) { c[2 * k] = q[r * 16 + k] & 15u; c[2 * k + 1] = q[r * 16 + k] >> 4; }
        else memcpy(c, q + r * 32, 32);
        dequant_row(c, sc[r], 32, bits, v + r * 32);
    }
}

/* ------------------------------------------------------------------ MX storage (the reference's channel-blocked tensors) */

/* block width of a C-channel tensor: 8 / 16 / 32 (src/lp_common.cuh:132); bw_force > 0 overrides (the graph keeps every tensor at 32) */
static inline int mx_bw(int C, int bw_force) { return bw_force > 0 ? bw_force : C <= 8 ? 8 : C <= 16 ? 16 : 32; }
static inline int mx_nb(int C, int bw) { return (C + bw - 1) / bw; }
size_t orc_mx_bytes(int bits, int N, int C, size_t S, int bw_force) {
    const int bw = mx_bw(C, bw_force);
    return (size_t)N * mx_nb(C, bw) * S * (bw * bits / 8 + 1);
}
/* plane-major [n][C][S] fp32 (dt 0) or fp16 (dt 2) -> MX tensor (src/lp_mx_cvt.cu:9-19, 59-79) */
void orc_pm_to_mx(const void *x, int dt, int N, int C, size_t S, int bits, int bw_force, uint8_t *y) {
    const int bw = mx_bw(C, bw_force), nb = mx_nb(C, bw), rb = bw * bits / 8;
    uint8_t *sc = y + (size_t)N * nb * S * rb;
#pragma omp parallel for collapse(2)
    for (int nbk = 0; nbk < N * nb; nbk++) for (size_t v = 0; v < S; v++) {
        const int n = nbk / nb, blk = nbk % nb;
        float r[32]; uint8_t c[32];
        for (int k = 0; k < bw; k++) {
            const int ch = blk * bw + k;
            if (ch >= C) { r[k] = 0.f; continue; }
            const size_t i = ((size_t)n * C + ch) * S + v;
            if (dt == 2) { h16 h; memcpy(&h, (const uint16_t *)x + i, 2); r[k] = (float)h; } else r[k] = ((const float *)x)[i];
        }
        const size_t ri = (size_t)nbk * S + v;
        sc[ri] = quant_row(r, bw, bits, c);
        if (bits == 4) for (int k = 0; k < bw / 2; k++) y[ri * rb + k] = (uint8_t)(c[2 * k] | (c[2 * k + 1] << 4));
        else memcpy(y + ri * rb, c, bw);
    }
}
/* MX tensor -> plane-major fp32 (src/lp_mx_cvt.cu:429-447) */
void orc_mx_to_pm(const uint8_t *x, int bits, int N, int C, size_t S, int bw_force, float *y) {
    const int bw = mx_bw(C, bw_force), nb = mx_nb(C, bw), rb = bw * bits / 8;
    const uint8_t *sc = x + (size_t)N * nb * S * rb;
#pragma omp parallel for collapse(2)
    for (int nbk = 0; nbk < N * nb; nbk++) for (size_t v = 0; v < S; v++) {
        const int n = nbk / nb, blk = nbk % nb;
        const size_t ri = (size_t)nbk * S + v;
        uint8_t c[32]; float r[32];
        if (bits == 4) for (int k = 0; k < bw / 2; k++) { c[2 * k] = x[ri * rb + k] & 15u; c[2 * k + 1] = x[ri * rb + k] >> 4; }
        else memcpy(c, x + ri * rb, bw);
        dequant_row(c, sc[ri], bw, bits, r);
        for (int k = 0; k < bw; k++) { const int ch = blk * bw + k; if (ch < C) y[((size_t)n * C + ch) * S + v] = r[k]; }
    }
}
/* MX tensor with 32-wide blocks -> blocked fp32 [n][nb][S][32] (the operand of orc_conv_blocked) */
void orc_mx_to_blocked(const uint8_t *x, int bits, int N, int C, size_t S, float *y) {
    const size_t rows = (size_t)N * ((C + 31) / 32) * S;
    orc_dequant_rows32(x, x + rows * (bits == 4 ? 16 : 32), rows, bits, y);
}
/* blocked fp32 -> MX tensor with 32-wide blocks */
void orc_blocked_to_mx(const float *x, int bits, int N, int C, size_t S, uint8_t *y) {
    const size_t rows = (size_t)N * ((C + 31) / 32) * S;
    orc_quant_rows32(x, rows, bits, y, y + rows * (bits == 4 ? 16 : 32));
}
/* plane-major fp32 <-> blocked fp32 (padding channels zero) */
void orc_pm_to_blocked(const float *x, int N, int C, size_t S, float *y) {
    const int nb = (C + 31) / 32;
#pragma omp parallel for collapse(2)
    for (int nbk = 0; nbk < N * nb; nbk++) for (size_t v = 0; v < S; v++) {
        const int n = nbk / nb, blk = nbk % nb;
        for (int k = 0; k < 32; k++) { const int ch = blk * 32 + k; y[((size_t)nbk * S + v) * 32 + k] = ch < C ? x[((size_t)n * C + ch) * S + v] : 0.f; }
    }
}
void orc_blocked_to_pm(const float *x, int N, int C, size_t S, float *y) {
    const int nb = (C + 31) / 32;
#pragma omp parallel for collapse(2)
    for (int nc = 0; nc < N * C; nc++) for (size_t v = 0; v < S; v++) {
        const int n = nc / C, ch = nc % C;
        y[(size_t)nc * S + v] = x[(((size_t)n * nb + ch / 32) * S + v) * 32 + ch % 32];
    }
}

/* ------------------------------------------------------------------ weights */

/* fp32 weights -> MX blocks of 32 input channels per (tap, output row), the dequantised values the conv multiplies, and the codes and
   scale bytes (for bit comparisons with the device's weight preparation).
   layout 0: conv, PyTorch [co][ci][taps] (tap = (kz * k + ky) * k + kx), row = co             (src/lp_f8fwd.cu:54-71)
   layout 1: ConvTranspose3d k2 s2, PyTorch [ci][co][8], tap = abc = (a * 2 + b) * 2 + e         (src/nn_xnet.cu:650-657)
   wdq [taps][Cip][Cop] (Cip, Cop = Ci, Co rounded up to 32; padding zero), wq [taps][Cip / 32][Cop][32] one code per byte,
   ws [taps][Cip / 32][Cop].  Any of wdq / wq / ws may be NULL. */
void orc_prep_w(const float *w, int Co, int Ci, int taps, int bits, int layout, float *wdq, uint8_t *wq, uint8_t *ws) {
    const int Cip = (Ci + 31) / 32 * 32, Cop = (Co + 31) / 32 * 32, nch = Cip / 32;
#pragma omp parallel for collapse(2)
    for (int t = 0; t < taps; t++) for (int cop = 0; cop < Cop; cop++) for (int ch = 0; ch < nch; ch++) {
        float v[32], d[32]; uint8_t c[32];
        for (int k = 0; k < 32; k++) {
            const int ci = ch * 32 + k;
            v[k] = (cop < Co && ci < Ci) ? (layout ? w[((size_t)ci * Co + cop) * taps + t] : w[((size_t)cop * Ci + ci) * taps + t]) : 0.f;
        }
        const uint8_t sc = quant_row(v, 32, bits, c);
        dequant_row(c, sc, 32, bits, d);
        if (wdq) for (int k = 0; k < 32; k++) wdq[((size_t)t * Cip + ch * 32 + k) * Cop + cop] = d[k];
        if (wq) memcpy(wq + (((size_t)t * nch + ch) * Cop + cop) * 32, c, 32);
        if (ws) ws[((size_t)t * nch + ch) * Cop + cop] = sc;
    }
}

/* ------------------------------------------------------------------ convolutions on blocked fp32 operands */

/* y[n][cob][vo][32] = bias + sum over taps and input channels of x (blocked, dequantised) times wdq ([taps][Cip][Cop]), fp32
   accumulation (the products of MX values are exact in fp32, so only the summation order is a choice: taps outer, channels inner).
   k in {1, 2, 3}, stride in {1, 2}, zero padding pad.  Index map as tests/test_mx4_wide.c:176-198. */
static int g_order = 0;
/* summation order of the taps: 0 ascending, 1 descending.  Both are "fp32 accumulation of the same dequantised operands"; running a
   network both ways measures how far two correct implementations can drift apart through flipped roundings. */
void orc_set_tap_order(int descending) { g_order = descending; }
void orc_conv_blocked(const float *x, int N, int Ci, int D, int H, int W, const float *wdq, const float *bias, int Co,
                      int k, int stride, int pad, float *y) {
    const int Cip = (Ci + 31) / 32 * 32, Cop = (Co + 31) / 32 * 32, cbi = Cip / 32, cbo = Cop / 32;
    const int Do = (D + 2 * pad - k) / stride + 1, Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
    const size_t S = (size_t)D * H * W, So = (size_t)Do * Ho * Wo;
#pragma omp parallel for collapse(3) schedule(dynamic, 4)
    for (int n = 0; n < N; n++) for (int oz = 0; oz < Do; oz++) for (int oy = 0; oy < Ho; oy++) {
        float *acc = (float *)malloc((size_t)Cop * sizeof(float));
        for (int ox = 0; ox < Wo; ox++) {
            for (int c = 0; c < Cop; c++) acc[c] = 0.f;
            for (int tt = 0; tt < k * k * k; tt++) {
                const int tq = g_order ? k * k * k - 1 - tt : tt, kz = tq / (k * k), ky = (tq / k) % k, kx = tq % k;
                const int iz = oz * stride + kz - pad, iy = oy * stride + ky - pad, ix = ox * stride + kx - pad;
                if (iz < 0 || iz >= D || iy < 0 || iy >= H || ix < 0 || ix >= W) continue;
                const size_t iv = ((size_t)iz * H + iy) * W + ix;
                const int t = (kz * k + ky) * k + kx;
                for (int cb = 0; cb < cbi; cb++) {
                    const float *xr = x + (((size_t)n * cbi + cb) * S + iv) * 32;
                    const float *wr = wdq + ((size_t)t * Cip + cb * 32) * Cop;
                    for (int ci = 0; ci < 32; ci++) {
                        const float xv = xr[ci];
                        if (xv == 0.f) continue;
                        const float *wc = wr + (size_t)ci * Cop;
#pragma omp simd
                        for (int c = 0; c < Cop; c++) acc[c] += xv * wc[c];
                    }
                }
            }
            const size_t ov = ((size_t)oz * Ho + oy) * Wo + ox;
            for (int c = 0; c < Cop; c++)
                y[(((size_t)n * cbo + c / 32) * So + ov) * 32 + c % 32] = c < Co ? acc[c] + (bias ? bias[c] : 0.f) : 0.f;
        }
        free(acc);
    }
}
/* ConvTranspose3d k2 s2: y[n][o][2z+a][2y+b][2x+e] = bias[o] + sum_ci x[n][ci][z][y][x] wdq[abc][ci][o] (src/nn_xnet.cu:688-697) */
void orc_tconv_blocked(const float *x, int N, int Ci, int D, int H, int W, const float *wdq, const float *bias, int Co, float *y) {
    const int Cip = (Ci + 31) / 32 * 32, Cop = (Co + 31) / 32 * 32, cbi = Cip / 32, cbo = Cop / 32;
    const size_t S = (size_t)D * H * W, So = S * 8; const int Ho = 2 * H, Wo = 2 * W;
#pragma omp parallel for collapse(3) schedule(dynamic, 4)
    for (int n = 0; n < N; n++) for (int z = 0; z < D; z++) for (int yy = 0; yy < H; yy++) {
        float *acc = (float *)malloc((size_t)Cop * sizeof(float));
        for (int xx = 0; xx < W; xx++) for (int t = 0; t < 8; t++) {
            const size_t iv = ((size_t)z * H + yy) * W + xx;
            for (int c = 0; c < Cop; c++) acc[c] = 0.f;
            for (int cb = 0; cb < cbi; cb++) {
                const float *xr = x + (((size_t)n * cbi + cb) * S + iv) * 32;
                const float *wr = wdq + ((size_t)t * Cip + cb * 32) * Cop;
                for (int ci = 0; ci < 32; ci++) {
                    const float xv = xr[ci];
                    if (xv == 0.f) continue;
                    const float *wc = wr + (size_t)ci * Cop;
#pragma omp simd
                    for (int c = 0; c < Cop; c++) acc[c] += xv * wc[c];
                }
            }
            const size_t ov = ((size_t)(2 * z + (t >> 2)) * Ho + 2 * yy + ((t >> 1) & 1)) * Wo + 2 * xx + (t & 1);
            for (int c = 0; c < Cop; c++)
                y[(((size_t)n * cbo + c / 32) * So + ov) * 32 + c % 32] = c < Co ? acc[c] + (bias ? bias[c] : 0.f) : 0.f;
        }
        free(acc);
    }
}

/* ------------------------------------------------------------------ InstanceNorm + LeakyReLU + requantise */

void orc_round_h16(float *v, size_t n) {
#pragma omp parallel for
    for (size_t i = 0; i < n; i++) v[i] = (float)(h16)v[i];
}
/* sums [n][C][2] (sum, sum of squares) of a blocked tensor, fp64, voxels in order (src/nn_xnet.cu:370-390: sums of the stored
   fp16-rounded outputs; the caller rounds first) */
void orc_in_sums(const float *y, int N, int C, size_t S, double *sums) {
    const int nb = (C + 31) / 32;
#pragma omp parallel for
    for (int nc = 0; nc < N * C; nc++) {
        const int n = nc / C, c = nc % C; double s = 0, q = 0;
        const float *p = y + ((size_t)n * nb + c / 32) * S * 32 + c % 32;
        for (size_t v = 0; v < S; v++) { const double t = p[v * 32]; s += t; q += t * t; }
        sums[2 * (size_t)nc] = s; sums[2 * (size_t)nc + 1] = q;
    }
}
/* coef [n][C][2]: a = rstd gamma, b = beta - mean a (src/nn_xnet.cu:1565-1570) */
void orc_in_coef(const double *sums, int N, int C, double S, const float *gamma, const float *beta, float eps, float *coef) {
    for (int i = 0; i < N * C; i++) {
        const int c = i % C; const double m = sums[2 * i] / S, v = fmax(sums[2 * i + 1] / S - m * m, 0.0);
        const float rs = (float)(1.0 / sqrt(v + (double)eps)), a = rs * (gamma ? gamma[c] : 1.f);
        coef[2 * i] = a; coef[2 * i + 1] = fmaf(-(float)m, a, beta ? beta[c] : 0.f);   /* one rounding: the device compiler contracts the reference's expression */
    }
}
/* out = fp16(act(y a + b)) on a blocked tensor; act 2 = LeakyReLU 0.01, 0 = none.  One fused multiply-add, as the device compiler
   contracts the reference's expression (src/nn_xnet.cu:1601). */
void orc_in_apply(const float *y, const float *coef, int N, int C, size_t S, int act, float *out) {
    const int nb = (C + 31) / 32;
#pragma omp parallel for collapse(2)
    for (int nbk = 0; nbk < N * nb; nbk++) for (size_t v = 0; v < S; v++) {
        const int n = nbk / nb, blk = nbk % nb;
        for (int k = 0; k < 32; k++) {
            const int c = blk * 32 + k; const size_t i = ((size_t)nbk * S + v) * 32 + k;
            if (c >= C) { out[i] = 0.f; continue; }
            float f = fmaf(y[i], coef[2 * ((size_t)n * C + c)], coef[2 * ((size_t)n * C + c) + 1]);
            if (act == 2) f = f < 0.f ? 0.01f * f : f;
            out[i] = (float)(h16)f;
        }
    }
}
/* 2x2x2 space-to-depth of a blocked tensor: out block (tap * nb + blk) at coarse voxel (z, y, x) = in block blk at fine voxel
   (2z + a, 2y + b, 2x + e), tap = (a * 2 + b) * 2 + e.  A 2^3 stride-2 conv on the fine grid is a 1^3 conv on this tensor. */
void orc_s2d_blocked(const float *x, int N, int C, int D, int H, int W, float *y) {
    const int nb = (C + 31) / 32, Dc = D / 2, Hc = H / 2, Wc = W / 2; const size_t S = (size_t)D * H * W, Sc = S / 8;
#pragma omp parallel for collapse(2)
    for (int n = 0; n < N; n++) for (int tb = 0; tb < 8 * nb; tb++) {
        const int t = tb / nb, blk = tb % nb, a = t >> 2, b = (t >> 1) & 1, e = t & 1;
        for (int z = 0; z < Dc; z++) for (int yy = 0; yy < Hc; yy++) for (int xx = 0; xx < Wc; xx++) {
            const size_t vf = ((size_t)(2 * z + a) * H + 2 * yy + b) * W + 2 * xx + e, vc = ((size_t)z * Hc + yy) * Wc + xx;
            memcpy(y + (((size_t)n * 8 * nb + tb) * Sc + vc) * 32, x + (((size_t)n * nb + blk) * S + vf) * 32, 32 * sizeof(float));
        }
    }
}
/* copy the nb_src blocks of src into blocks [b0, b0 + nb_src) of dst (channel concat of blocked tensors) */
void orc_put_blocks(const float *src, int N, int nb_src, size_t S, float *dst, int nb_dst, int b0) {
    for (int n = 0; n < N; n++) for (int b = 0; b < nb_src; b++)
        memcpy(dst + ((size_t)n * nb_dst + b0 + b) * S * 32, src + ((size_t)n * nb_src + b) * S * 32, S * 32 * sizeof(float));
}
/* quantise then dequantise a blocked tensor in place: the values an MX consumer sees */
void orc_fake_quant_blocked(float *x, size_t rows, int bits) {
    uint8_t *q = (uint8_t *)malloc(rows * 33);
    orc_quant_rows32(x, rows, bits, q, q + rows * 32);
    orc_dequant_rows32(q, q + rows * 32, rows, bits, x);
    free(q);
}

/* ------------------------------------------------------------------ the benchmark's U-Net forward */

/* Five-level U-Net, widths cw[0..L), per level two 3^3 convs each followed by InstanceNorm(eps 1e-5, gamma 1, beta 0) + LeakyReLU 0.01,
   2^3 stride-2 down convs, ConvTranspose k2 s2 up, concat (up | skip), 1^3 head.  Every conv input is an MX tensor (bits_in[i] of
   conv i, 8 or 4, activations and weights alike).  Weights arrive as one flat fp32 array in forward order (see orc_unet_nweights);
   conv order: enc l c1, c2 (l = 0..L-1) with down l after enc l (l < L-1); then for l = L-2..0: up l, dec l c1, c2; head.
   x: [N][1][P^3] fp16 plane-major.  logits: [N][nh][P^3] fp32 plane-major (fp32 accumulators + bias of the head, not rounded).
   taps: optional callback to hand intermediate tensors to a test. */
typedef struct { int L; int cw[8]; int nh; int P; int bits_first, bits_mid, bits_last; } orc_unet_cfg;
typedef void (*orc_tap_fn)(void *ctx, const char *name, const float *blocked, int C, int D);

static size_t conv_nw(int co, int ci, int taps) { return (size_t)co * ci * taps + co; }   /* weights then bias */
size_t orc_unet_nweights(const orc_unet_cfg *c) {
    size_t n = 0;
    for (int l = 0; l < c->L; l++) {
        n += conv_nw(c->cw[l], l ? c->cw[l] : 1, 27) + conv_nw(c->cw[l], c->cw[l], 27);
        if (l < c->L - 1) n += conv_nw(c->cw[l + 1], c->cw[l], 8);
    }
    for (int l = c->L - 2; l >= 0; l--) n += conv_nw(c->cw[l], c->cw[l + 1], 8) + conv_nw(c->cw[l], 2 * c->cw[l], 27) + conv_nw(c->cw[l], c->cw[l], 27);
    return n + conv_nw(c->nh, c->cw[0], 1);
}
/* conv + fp16 store + IN + LeakyReLU -> fp16 blocked activation (fresh allocation) */
static float *conv_in_lrelu(const float *xin, int N, int Ci, int D, const float **wp, int Co, int bits, orc_tap_fn tap, void *ctx, const char *nm) {
    const size_t S = (size_t)D * D * D; const int Cip = (Ci + 31) / 32 * 32, Cop = (Co + 31) / 32 * 32;
    float *xq = (float *)malloc((size_t)N * Cip * S * 4); memcpy(xq, xin, (size_t)N * Cip * S * 4);
    orc_fake_quant_blocked(xq, (size_t)N * (Cip / 32) * S, bits);
    float *wdq = (float *)malloc((size_t)27 * Cip * Cop * 4);
    orc_prep_w(*wp, Co, Ci, 27, bits, 0, wdq, NULL, NULL);
    const float *bias = *wp + (size_t)Co * Ci * 27; *wp = bias + Co;
    float *y = (float *)malloc((size_t)N * Cop * S * 4);
    orc_conv_blocked(xq, N, Ci, D, D, D, wdq, bias, Co, 3, 1, 1, y);
    orc_round_h16(y, (size_t)N * Cop * S);
    if (tap) { char b[64]; snprintf(b, sizeof b, "%s.y", nm); tap(ctx, b, y, Co, D); }
    double *sums = (double *)malloc((size_t)N * Co * 2 * 8); float *coef = (float *)malloc((size_t)N * Co * 2 * 4);
    orc_in_sums(y, N, Co, S, sums); orc_in_coef(sums, N, Co, (double)S, NULL, NULL, 1e-5f, coef);
    orc_in_apply(y, coef, N, Co, S, 2, y);
    if (tap) { char b[64]; snprintf(b, sizeof b, "%s.a", nm); tap(ctx, b, y, Co, D); }
    free(xq); free(wdq); free(sums); free(coef);
    return y;
}
void orc_unet_forward(const orc_unet_cfg *c, const float *weights, const uint16_t *x16, int N, float *logits, orc_tap_fn tap, void *ctx) {
    const int L = c->L; const float *wp = weights;
    float *skip[8] = {0}; int Dl[8]; Dl[0] = c->P; for (int l = 1; l < L; l++) Dl[l] = Dl[l - 1] / 2;
    /* input: one channel, stored as a 32-wide block with 31 zero channels */
    size_t S = (size_t)c->P * c->P * c->P;
    float *xf = (float *)malloc((size_t)N * S * 4); orc_h16_to_f32(x16, (size_t)N * S, xf);
    float *cur = (float *)malloc((size_t)N * 32 * S * 4); orc_pm_to_blocked(xf, N, 1, S, cur); free(xf);
    int Ccur = 1; char nm[32];
    for (int l = 0; l < L; l++) {
        const int D = Dl[l], C = c->cw[l];
        snprintf(nm, sizeof nm, "enc%d.c1", l);
        float *a = conv_in_lrelu(cur, N, Ccur, D, &wp, C, (l == 0) ? c->bits_first : c->bits_mid, tap, ctx, nm); free(cur);
        snprintf(nm, sizeof nm, "enc%d.c2", l);
        float *b = conv_in_lrelu(a, N, C, D, &wp, C, c->bits_mid, tap, ctx, nm); free(a);
        if (l == L - 1) { cur = b; Ccur = C; break; }
        skip[l] = b;
        /* down: 2^3 stride-2 conv C -> cw[l+1], bias, fp16 store, no norm (its output feeds enc l+1 c1's quantiser) */
        S = (size_t)D * D * D; const int Cn = c->cw[l + 1], Cip = (C + 31) / 32 * 32, Cop = (Cn + 31) / 32 * 32;
        float *xq = (float *)malloc((size_t)N * Cip * S * 4); memcpy(xq, b, (size_t)N * Cip * S * 4);
        orc_fake_quant_blocked(xq, (size_t)N * (Cip / 32) * S, c->bits_mid);
        float *wdq = (float *)malloc((size_t)8 * Cip * Cop * 4); orc_prep_w(wp, Cn, C, 8, c->bits_mid, 0, wdq, NULL, NULL);
        const float *bias = wp + (size_t)Cn * C * 8; wp = bias + Cn;
        cur = (float *)malloc((size_t)N * Cop * (S / 8) * 4);
        orc_conv_blocked(xq, N, C, D, D, D, wdq, bias, Cn, 2, 2, 0, cur); orc_round_h16(cur, (size_t)N * Cop * (S / 8));
        if (tap) { snprintf(nm, sizeof nm, "down%d.y", l); tap(ctx, nm, cur, Cn, D / 2); }
        free(xq); free(wdq); Ccur = Cn;
    }
    for (int l = L - 2; l >= 0; l--) {
        const int D = Dl[l], C = c->cw[l], Cl = c->cw[l + 1], Dc = Dl[l + 1];
        const size_t Sc = (size_t)Dc * Dc * Dc; S = (size_t)D * D * D;
        const int Clp = (Cl + 31) / 32 * 32, Cp = (C + 31) / 32 * 32;
        float *xq = (float *)malloc((size_t)N * Clp * Sc * 4); memcpy(xq, cur, (size_t)N * Clp * Sc * 4); free(cur);
        orc_fake_quant_blocked(xq, (size_t)N * (Clp / 32) * Sc, c->bits_mid);
        float *wdq = (float *)malloc((size_t)8 * Clp * Cp * 4); orc_prep_w(wp, C, Cl, 8, c->bits_mid, 1, wdq, NULL, NULL);
        const float *bias = wp + (size_t)Cl * C * 8; wp = bias + C;
        float *up = (float *)malloc((size_t)N * Cp * S * 4);
        orc_tconv_blocked(xq, N, Cl, Dc, Dc, Dc, wdq, bias, C, up); orc_round_h16(up, (size_t)N * Cp * S);
        if (tap) { snprintf(nm, sizeof nm, "up%d.y", l); tap(ctx, nm, up, C, D); }
        free(xq); free(wdq);
        float *cat = (float *)malloc((size_t)N * 2 * Cp * S * 4);
        orc_put_blocks(up, N, Cp / 32, S, cat, 2 * Cp / 32, 0); orc_put_blocks(skip[l], N, Cp / 32, S, cat, 2 * Cp / 32, Cp / 32);
        free(up); free(skip[l]);
        snprintf(nm, sizeof nm, "dec%d.c1", l);
        float *a = conv_in_lrelu(cat, N, 2 * Cp, D, &wp, C, c->bits_mid, tap, ctx, nm); free(cat);
        snprintf(nm, sizeof nm, "dec%d.c2", l);
        cur = conv_in_lrelu(a, N, C, D, &wp, C, (l == 0) ? c->bits_last : c->bits_mid, tap, ctx, nm); free(a);
    }
    /* head: 1^3 conv cw[0] -> nh on the MX copy of the last activation; fp32 logits, plane-major */
    {
        S = (size_t)c->P * c->P * c->P; const int C = c->cw[0], Cp = (C + 31) / 32 * 32, nhp = (c->nh + 31) / 32 * 32;
        orc_fake_quant_blocked(cur, (size_t)N * (Cp / 32) * S, c->bits_last);
        float *wdq = (float *)malloc((size_t)Cp * nhp * 4); orc_prep_w(wp, c->nh, C, 1, c->bits_last, 0, wdq, NULL, NULL);
        const float *bias = wp + (size_t)c->nh * C;
        float *y = (float *)malloc((size_t)N * nhp * S * 4);
        orc_conv_blocked(cur, N, C, c->P, c->P, c->P, wdq, bias, c->nh, 1, 1, 0, y);
        orc_blocked_to_pm(y, N, c->nh, S, logits);
        free(y); free(wdq); free(cur);
    }
}

/* ------------------------------------------------------------------ sliding window */

/* Gaussian window weight of a P^3 patch: exp(-(i - P / 2)^2 / (2 sigma^2)) per axis with sigma = P / 8 and the integer centre P / 2
   (g1_init, src/nn_ink3dext.cu:48-56; src/ink3dext.c:8) */
void orc_gauss_window(int P, float *w1d) {
    const double s = P / 8.0, c = (double)(P / 2);
    for (int i = 0; i < P; i++) { const double d = (i - c) / s; w1d[i] = (float)exp(-0.5 * d * d); }
}
/* accumulate one patch: acc[ch][vol voxel] += w * logits, wsum[vol voxel] += w, for the patch with origin (z0, y0, x0) in a V^3 volume */
void orc_blend_add(const float *logits, int nh, int P, int V, int z0, int y0, int x0, const float *w1d, float *acc, float *wsum) {
    const size_t VS = (size_t)V * V * V, PS = (size_t)P * P * P;
#pragma omp parallel for
    for (int z = 0; z < P; z++) for (int y = 0; y < P; y++) for (int x = 0; x < P; x++) {
        const int gz = z0 + z, gy = y0 + y, gx = x0 + x;
        if (gz >= V || gy >= V || gx >= V) continue;
        const float w = w1d[z] * w1d[y] * w1d[x];
        const size_t gv = ((size_t)gz * V + gy) * V + gx, pv = ((size_t)z * P + y) * P + x;
        for (int c = 0; c < nh; c++) acc[(size_t)c * VS + gv] += w * logits[(size_t)c * PS + pv];
        wsum[gv] += w;
    }
}

/* The library's exact blend (its answer to the run-to-run changing fp32 atomics of k_i3_blend, src/nn_ink3dext.cu:58-73): a term is the
   exact product of the reference's fp32 window weight w1d[z] w1d[y] w1d[x] and the fp32 logit, rounded once to a multiple of 2^-46 and
   added as a 64-bit integer.  acc [nh][V^3], wsum [V^3]. */
void orc_blend_add_fx(const float *logits, int nh, int P, int V, int z0, int y0, int x0, const float *w1d, long long *acc, long long *wsum) {
    const size_t VS = (size_t)V * V * V, PS = (size_t)P * P * P;
#pragma omp parallel for
    for (int z = 0; z < P; z++) for (int y = 0; y < P; y++) for (int x = 0; x < P; x++) {
        const int gz = z0 + z, gy = y0 + y, gx = x0 + x;
        if (gz >= V || gy >= V || gx >= V) continue;
        const float w3 = (w1d[z] * w1d[y]) * w1d[x];
        const double w = (double)w3 * 70368744177664.0;
        const size_t gv = ((size_t)gz * V + gy) * V + gx, pv = ((size_t)z * P + y) * P + x;
        for (int c = 0; c < nh; c++) { const double t = w * (double)logits[(size_t)c * PS + pv]; acc[(size_t)c * VS + gv] += fabs(t) < 9.0e18 ? llrint(t) : 0; }
        wsum[gv] += llrint(w);
    }
}
/* the blended volume: l = (float)(sum / weight); fmt 2: fp16 logits; otherwise uint8 round(254 p), p = 1 / (1 + exp(-l)), 255 where nothing covers
   the voxel (k_i3_emit, src/nn_ink3dext.cu:77-100) */
void orc_emit_fx(const long long *acc, const long long *wsum, int nh, size_t nvox, int fmt, void *out) {
#pragma omp parallel for
    for (size_t v = 0; v < nvox; v++) for (int c = 0; c < nh; c++) {
        const size_t o = (size_t)c * nvox + v; const long long ws = wsum[v];
        const float l = ws > 0 ? (float)((double)acc[o] / (double)ws) : 0.f;
        if (fmt == 2) ((h16 *)out)[o] = (h16)l;
        else ((uint8_t *)out)[o] = ws > 0 ? (uint8_t)lrintf((1.f / (1.f + expf(-l))) * 254.f) : 255;
    }
}

/* ---- elementwise operators of the reference interface on dequantised tensors (plane-major fp32 [n][c][voxel]) ---- */

/* GroupNorm + SiLU of a tensor, or of a channel segment of a larger tensor the G groups are counted over (its channel 0 is channel
   c_off of C_all; gamma, beta, mean, rstd belong to the larger tensor).  form 0: ((x - mean) rstd) gamma + beta as lp_gn_silu_apply_mx
   (src/lp_mx_gn.cu:17); form 1: fma(x, a, b), a = rstd gamma, b = fma(-mean, a, beta), the conv operand's transform (make_chan / act_ab,
   src/lp_common.cuh:244-261, 474-476).  SiLU by its definition u / (1 + exp(-u)): the reference evaluates it with approximate
   intrinsics, so implementations are compared with this one under a tolerance. */
void orc_gn_silu(const float *x, int N, int C, size_t S, int G, const float *gamma, const float *beta, const float *mean, const float *rstd,
                 int form, int c_off, int C_all, float *y) {
    const int cpg = C_all / G;
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; n++)
        for (int c = 0; c < C; c++) {
            const int cl = c_off + c, ng = n * G + cl / cpg;
            const float a = rstd[ng] * gamma[cl], b = fmaf(-mean[ng], a, beta[cl]);
            const float *xp = x + ((size_t)n * C + c) * S; float *yp = y + ((size_t)n * C + c) * S;
            for (size_t v = 0; v < S; v++) {
                const float u = form == 0 ? (((xp[v] - mean[ng]) * rstd[ng]) * gamma[cl]) + beta[cl] : fmaf(xp[v], a, b);
                yp[v] = u / (1.f + expf(-u));
            }
        }
}

/* exact-2x trilinear upsample (align_corners false, edges clamped) with the reference's order of roundings (up2_mx_k,
   src/lp_mx_gn.cu:35-72; host blend of tests/test_mx4_wide.c:327-338): a fine voxel starts from zero and takes its eight coarse
   corners with one fma each, z outermost, x innermost, on every axis the corner under the fine voxel (weight 3/4) before its
   neighbour on the fine voxel's side (weight 1/4). */
void orc_up2(const float *x, int N, int C, int D, int H, int W, float *y) {
    const size_t S = (size_t)D * H * W;
#pragma omp parallel for collapse(2) schedule(static)
    for (int nc = 0; nc < N * C; nc++)
        for (int fz = 0; fz < 2 * D; fz++) {
            const float *xp = x + (size_t)nc * S; float *yp = y + (size_t)nc * 8 * S;
            for (int fy = 0; fy < 2 * H; fy++)
                for (int fx = 0; fx < 2 * W; fx++) {
                    int s[3][2]; const int f[3] = {fz, fy, fx}, lim[3] = {D, H, W};
                    for (int a = 0; a < 3; a++) {
                        const int t = (f[a] >> 1) + ((f[a] & 1) ? 1 : -1);
                        s[a][0] = f[a] >> 1; s[a][1] = t < 0 ? 0 : t >= lim[a] ? lim[a] - 1 : t;
                    }
                    float acc = 0.f;
                    for (int e = 0; e < 8; e++) {
                        const int iz = e >> 2, iy = (e >> 1) & 1, ix = e & 1;
                        const float w3 = (iz ? 0.25f : 0.75f) * (iy ? 0.25f : 0.75f) * (ix ? 0.25f : 0.75f);
                        acc = fmaf(w3, xp[((size_t)s[0][iz] * H + s[1][iy]) * W + s[2][ix]], acc);
                    }
                    yp[((size_t)fz * 2 * H + fy) * 2 * W + fx] = acc;
                }
        }
}

/* 1^3 conv with fp32 weights w [co][ci]: bias first, then one fma per input channel in ascending order (conv1_mx_k,
   src/lp_mx_conv1.cu:4-22) */
void orc_conv1(const float *x, const float *w, const float *b, int N, int Ci, int Co, size_t S, float *y) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; n++)
        for (int co = 0; co < Co; co++) {
            float *yp = y + ((size_t)n * Co + co) * S;
            for (size_t v = 0; v < S; v++) yp[v] = b ? b[co] : 0.f;
            for (int ci = 0; ci < Ci; ci++) {
                const float wv = w[(size_t)co * Ci + ci]; const float *xp = x + ((size_t)n * Ci + ci) * S;
                for (size_t v = 0; v < S; v++) yp[v] = fmaf(wv, xp[v], yp[v]);
            }
        }
}

/* The network input of the reference's predict (pred_in_mx_k, src/lp_mx_cvt.cu:29-41) before its MX rows: out [4][nz W W] plane-major,
   channel 0 the z-scored CT byte, 1 zero, 2 and 3 the unit direction (dy, dx) away from the scroll axis times `axis`, each rounded to
   the 16-bit input type (hd 2 fp16, 1 bf16, 0 none).  The radius is sqrtf(fmaf(dy, dy, dx dx)) + 1e-6f. */
static float round16(float v, int hd) {
    if (hd == 2) return (float)(h16)v;
    if (hd == 1) { uint32_t u; memcpy(&u, &v, 4); if ((u & 0x7fffffffu) > 0x7f800000u) u |= 0x00400000u; else u += 0x7fffu + ((u >> 16) & 1u); u &= 0xffff0000u; memcpy(&v, &u, 4); return v; }
    return v;
}
void orc_pred_input(const uint8_t *ct, int W, float mean, float isd, const float *dyo, const float *dxo, int axis, int z0, int nz, int hd, float *out) {
    const size_t S = (size_t)nz * W * W;
#pragma omp parallel for schedule(static)
    for (int zi = 0; zi < nz; zi++) {
        const int z = z0 + zi;
        for (int yy = 0; yy < W; yy++)
            for (int xx = 0; xx < W; xx++) {
                const size_t i = ((size_t)zi * W + yy) * W + xx;
                const float dy = dyo[z] + (float)yy, dx = dxo[z] + (float)xx;
                const float inv = axis ? (float)axis / (sqrtf(fmaf(dy, dy, dx * dx)) + 1e-6f) : 0.f;
                out[i] = round16(((float)ct[(size_t)z * W * W + (size_t)yy * W + xx] - mean) * isd, hd);
                out[S + i] = 0.f;
                out[2 * S + i] = round16(dy * inv, hd);
                out[3 * S + i] = round16(dx * inv, hd);
            }
    }
}
