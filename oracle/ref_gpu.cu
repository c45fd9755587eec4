/* Test infrastructure: the reference's own GPU code for this path, built from the reference tree where it lies, behind a few
   C entry points the parity tests call.  Nothing here is linked into the product library.

   Two reference units are built (see the Makefile beside this file):
     src/nn_xnet.cu    - included below as source text, so that this file can reach its file-scope statics: the emulated-MX switches
                         (UFSM_XNET_FQ: g_fq_a / g_fq_w, read from the environment once per process), the host weight rounding
                         fq_host, the InstanceNorm kernels k_in_coef / k_inq.  Its convolution is an fp16 mma.sync implicit GEMM that
                         runs on any sm_80+ device, sm_100 included; with UFSM_XNET_FQ = A,W it rounds activations (k_fq, per voxel and
                         32 channels) and weights (fq_host, per output row and 32 K) to MX values first (src/nn_xnet.cu:128-232,
                         582-597, 1467-1476): "the accuracy of an MX conv path, run on the fp16 kernels".
     src/lp_mx_cvt.cu  - compiled as its own object: lp_f32_to_mx8/4, lp_h16_to_mx8/4, lp_mx8/4_to_f32, the quantiser entry points of
                         src/nn_lp.h:110-118.  It needs three symbols from units that are not built here; they are defined below with
                         the meaning the reference gives them when the feature they serve is off.

   Tensors cross this boundary as host arrays: fp16 NDHWC activations (the xnet layout), PyTorch-order fp32 weights. */
#include "nn_xnet.cu"

/* ---- what src/lp_mx_cvt.cu expects from other reference units ---- */
thread_local cudaError_t g_lp_err = cudaSuccess;                       /* src/lp_f8fwd.cu:4: the thread's first launch error */
extern "C" void nn_err_post(int e, const char *file, int line, const char *what) {   /* src/nn_core.cu:244: process-wide error post */
    fprintf(stderr, "reference: CUDA error %d at %s:%d (%s)\n", e, file, line, what ? what : "");
}
int zw_win(int D, int *z0, int *z1) { (void)D; (void)z0; (void)z1; return 0; }   /* src/nn_bwd.cu:57: no z-window is set */

extern "C" {

int refgpu_init(int gpu) { return xnet_init(gpu); }
/* the emulated-MX formats of the convs from now on: a, w = 0 (off), 4 (e2m1) or 8 (e4m3), one ue8m0 scale per 32 */
void refgpu_set_fq(int a, int w) { g_fq_a = a; g_fq_w = w; g_fq_mask = -1; }
/* one block of n <= 32 weights rounded in place, as conv_upload does per 32 K of an output row */
void refgpu_fq_host(float *v, int n, int bits) { fq_host(v, n, bits); }

/* y = fp16(conv(x) + bias), k^3 taps, stride s, padding p; w [co][ci][k][k][k]; x [n][d][h][w][ci], y [n][do][ho][wo][co] fp16 on the host;
   st (optional): the reference's own InstanceNorm sums [n][co][2] of the stored y.  0 on success. */
int refgpu_conv(const float *w, const float *bias, int co, int ci, int k, int s, int p, const void *x, int n, int d, int h, int wd, void *y, double *st) {
    xconv c;
    if (xconv_init(&c, w, co, ci, k, k, k, s, s, s, p, p, p, nullptr, bias)) return -1;
    xt xin = xt_new(n, d, h, wd, ci);
    xh2d(xin.p, x, xt_numel(xin) * 2);
    double *std_ = nullptr;
    xt out = st ? xconv_fwd_st(&c, xin, &std_) : xconv_fwd(&c, xin, nullptr, XA_NONE);
    xnet_sync();
    const int rc = xnet_check("refgpu_conv");
    if (!rc) { xd2h(y, out.p, xt_numel(out) * 2); if (st) xd2h(st, std_, (size_t)n * co * 2 * sizeof(double)); }
    xfree_dev(std_); xt_free(&out); xt_free(&xin); xconv_free(&c);
    return rc;
}
/* ConvTranspose3d k2 s2: w [ci][co][2][2][2]; x [n][d][h][w][ci] -> y [n][2d][2h][2w][co].  The reference rounds the GEMM result to fp16
   before the shuffle kernel adds the bias (src/nn_xnet.cu:688-697), so only bias == NULL gives the single rounding of the fused path. */
int refgpu_tconv3(const float *w, const float *bias, int ci, int co, const void *x, int n, int d, int h, int wd, void *y) {
    xconv c;
    if (xtconv3_init(&c, w, ci, co, bias)) return -1;
    xt xin = xt_new(n, d, h, wd, ci);
    xh2d(xin.p, x, xt_numel(xin) * 2);
    xt out = xconv_fwd(&c, xin, nullptr, XA_NONE);
    xnet_sync();
    const int rc = xnet_check("refgpu_tconv3");
    if (!rc) xd2h(y, out.p, xt_numel(out) * 2);
    xt_free(&out); xt_free(&xin); xconv_free(&c);
    return rc;
}
/* InstanceNorm of a stored tensor from given sums: coef = k_in_coef(st) [n][C][2], then y = fp16(act(a y + b)) in place (k_inq with
   want_half, src/nn_xnet.cu:1565-1570, 1577-1620); y [n][S][C] fp16 on the host; gamma, beta [C] on the host */
int refgpu_in(const double *st, int n, int C, long long S, const float *gamma, const float *beta, float eps, float *coef, void *y, int act) {
    double *std_ = (double *)xmalloc_dev((size_t)n * C * 2 * sizeof(double));
    xh2d(std_, st, (size_t)n * C * 2 * sizeof(double));
    float *g = xdev_floats(gamma, C), *b = xdev_floats(beta, C);
    float *cf = xin_coef(std_, n, C, S, g, b, eps);
    xt t = xt_new(n, 1, 1, (int)S, C);
    xh2d(t.p, y, xt_numel(t) * 2);
    xin_apply(&t, cf, nullptr, nullptr, act, 1, 0);
    xnet_sync();
    const int rc = xnet_check("refgpu_in");
    if (!rc) { xd2h(coef, cf, (size_t)n * C * 2 * sizeof(float)); xd2h(y, t.p, xt_numel(t) * 2); }
    xt_free(&t); xfree_dev(cf); xfree_dev(g); xfree_dev(b); xfree_dev(std_);
    return rc;
}

/* the reference's quantiser entry points (src/lp_mx_cvt.cu:6-7, 59-79, 440-447) on host arrays: x plane-major [N][C][S] of dt 0 (fp32) or
   2 (fp16) -> y MX bytes; and back to fp32.  They run on the legacy default stream. */
size_t lp_mx8_bytes(int N, int C, size_t S);
size_t lp_mx4_bytes(int N, int C, size_t S);
void lp_f32_to_mx8(const float *x, int N, int C, size_t S, void *y);
void lp_f32_to_mx4(const float *x, int N, int C, size_t S, void *y);
void lp_h16_to_mx8(const void *x, int dt, int N, int C, size_t S, void *y);
void lp_h16_to_mx4(const void *x, int dt, int N, int C, size_t S, void *y);
void lp_mx8_to_f32(const void *x, int N, int C, size_t S, float *y);
void lp_mx4_to_f32(const void *x, int N, int C, size_t S, float *y);
size_t refgpu_mx_bytes(int bits, int N, int C, size_t S) { return bits == 8 ? lp_mx8_bytes(N, C, S) : lp_mx4_bytes(N, C, S); }
int refgpu_to_mx(int bits, const void *x, int dt, int N, int C, size_t S, void *y) {
    const size_t nx = (size_t)N * C * S * (dt == 0 ? 4 : 2), ny = refgpu_mx_bytes(bits, N, C, S);
    void *xd = nullptr, *yd = nullptr;
    if (cudaMalloc(&xd, nx) != cudaSuccess || cudaMalloc(&yd, ny) != cudaSuccess) { cudaFree(xd); return -1; }
    cudaMemcpy(xd, x, nx, cudaMemcpyHostToDevice); cudaMemset(yd, 0xEE, ny);
    if (dt == 0) (bits == 8 ? lp_f32_to_mx8 : lp_f32_to_mx4)((const float *)xd, N, C, S, yd);
    else (bits == 8 ? lp_h16_to_mx8 : lp_h16_to_mx4)(xd, dt, N, C, S, yd);
    const cudaError_t e = cudaDeviceSynchronize();
    cudaMemcpy(y, yd, ny, cudaMemcpyDeviceToHost);
    cudaFree(xd); cudaFree(yd);
    return e == cudaSuccess && g_lp_err == cudaSuccess ? 0 : -1;
}
int refgpu_mx_to_f32(int bits, const void *x, int N, int C, size_t S, float *y) {
    const size_t nx = refgpu_mx_bytes(bits, N, C, S), ny = (size_t)N * C * S * 4;
    void *xd = nullptr, *yd = nullptr;
    if (cudaMalloc(&xd, nx) != cudaSuccess || cudaMalloc(&yd, ny) != cudaSuccess) { cudaFree(xd); return -1; }
    cudaMemcpy(xd, x, nx, cudaMemcpyHostToDevice);
    (bits == 8 ? lp_mx8_to_f32 : lp_mx4_to_f32)(xd, N, C, S, (float *)yd);
    const cudaError_t e = cudaDeviceSynchronize();
    cudaMemcpy(y, yd, ny, cudaMemcpyDeviceToHost);
    cudaFree(xd); cudaFree(yd);
    return e == cudaSuccess && g_lp_err == cudaSuccess ? 0 : -1;
}

}   /* extern "C" */
