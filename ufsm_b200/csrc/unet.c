/* Host side (C23) of the benchmark's 3-D U-Net forward and of the sliding-window scheduler, on top of the C ABI of ufsm_mx.h.

   Network (the InstanceNorm / LeakyReLU / transposed-conv graph of the reference's ink U-Net, src/ink3dext_net.c:189-231, with
   the widths and layer list of the benchmark): per level two 3^3 convs, each conv -> fp16 store + InstanceNorm partial sums in
   the conv epilogue -> coefficients -> fused apply (affine, LeakyReLU 0.01, fp16 rounding, MX requantisation for the next conv).
   The second apply of an encoder level writes the skip half of the decoder's concat tensor directly and a space-to-depth copy
   that turns the 2^3 stride-2 down conv into a 1^3 GEMM; the transposed conv is a GEMM to 8 Cout columns whose epilogue scatters
   and requantises straight into the other half of the concat tensor (xtconv_cat_q, src/nn_xnet.cu:1775-1789).  Every tensor's MX
   format is that of the conv that reads it; MX-fp8 tensors are kept in the split layout (two 16-byte planes per block).  All buffers are allocated once at
   creation. */
#include "../../include/ufsm_mx.h"
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

void umx_u8_to_h16(const uint8_t *x, size_t n, void *y);
int umx_has_error(void);
void umx_h16_to_prob_u8(const void *x, size_t n, uint8_t *y);
void umx_blend_add_fx(const float *logits, int nh, int P, int V, int zlo, int zext, int z0, int y0, int x0, const float *w1d, long long *acc, long long *wsum);
void umx_emit_fx(const long long *acc, const long long *wsum, const uint8_t *mode, int want, int nh, int V, int zext, int za, int zb, int ya, int yb, int fmt, void *out);
void umx_copy2d_async(void *dst, size_t dpitch, const void *src, size_t spitch, size_t width, size_t height, int to_device, void *stream);
void umx_gather_u8_h16(const uint8_t *vol_dev, int V, int z, int y, int x, int P, void *out);
void umx_emit_rows_fx(const long long *acc, const long long *wsum, const int *zy_dev, long nrows, int nh, int V, int zext, int fmt, void *out);
void umx_rows_fx(long long *acc, long long *wsum, const int *zy_dev, long nrows, int nh, int V, int zext, int dir, long long *buf);
void umx_blend_add(const void *logits, int fmt, int nh, int P, int V, int zlo, int zext, int z0, int y0, int x0, const float *w1d, float *acc, float *wsum);
long umx_launch_count(void);

enum { MAXL = 8 };
struct umx_unet {
    umx_unet_cfg cfg; int maxN;
    umx_conv *enc1[MAXL], *enc2[MAXL], *down[MAXL], *up[MAXL], *dec1[MAXL], *dec2[MAXL], *head;
    int Dl[MAXL];
    void *ybuf;              /* blocked fp16 conv output, reused by every conv */
    double *part; float *coef;
    void *act[MAXL];         /* MX activation between the two convs of a level (encoder and decoder reuse it) */
    void *cat[MAXL];         /* MX concat (up | skip), 2 C_l channels; level L-1: the bottom activation, C channels */
    void *s2d[MAXL];         /* space-to-depth copy of the skip, the down conv's input */
    void *dn[MAXL];          /* MX output of down l-1 = input of enc l c1 (l >= 1) */
    void *dec[MAXL];         /* MX output of dec l c2 */
    void *x16, *xu8, *logits16;   /* staging for the host entry */
    /* the pipelined host entry: two slots of input bytes and fp16 logits, a copy-in and a copy-out stream, and per slot the events
       "input uploaded", "input consumed", "logits ready", "logits downloaded" */
    void *pxu8[2], *plog[2], *pprob[2], *s_in, *s_out, *ev_up[2], *ev_used[2], *ev_ready[2], *ev_down[2];
    long seq; int pipe_ok;
    long launches0;
};

static size_t cube(int d) { return (size_t)d * d * d; }
static size_t conv_nw(int co, int ci, int taps) { return (size_t)co * ci * taps + (size_t)co; }

size_t umx_unet_nweights(const umx_unet_cfg *c) {
    size_t n = 0;
    for (int l = 0; l < c->L; l++) {
        n += conv_nw(c->cw[l], l ? c->cw[l] : 1, 27) + conv_nw(c->cw[l], c->cw[l], 27);
        if (l < c->L - 1) n += conv_nw(c->cw[l + 1], c->cw[l], 8);
    }
    for (int l = c->L - 2; l >= 0; l--) n += conv_nw(c->cw[l], c->cw[l + 1], 8) + conv_nw(c->cw[l], 2 * c->cw[l], 27) + conv_nw(c->cw[l], c->cw[l], 27);
    return n + conv_nw(c->nh, c->cw[0], 1);
}
double umx_unet_flops(const umx_unet_cfg *c) {
    double f = 0; int D = c->P;
    int Dl[MAXL]; for (int l = 0; l < c->L; l++) { Dl[l] = D; D /= 2; }
    for (int l = 0; l < c->L; l++) {
        const double S = (double)cube(Dl[l]);
        f += 2.0 * S * 27 * ((l ? c->cw[l] : 1) * (double)c->cw[l] + (double)c->cw[l] * c->cw[l]);
        if (l < c->L - 1) f += 2.0 * (S / 8) * 8 * (double)c->cw[l] * c->cw[l + 1] * 2;   /* down l and up l */
        if (l < c->L - 1) f += 2.0 * S * 27 * (2.0 * c->cw[l] * c->cw[l] + (double)c->cw[l] * c->cw[l]);
    }
    return f + 2.0 * (double)cube(c->P) * c->cw[0] * c->nh;
}

static umx_conv *mk(int kind, const float **wp, int co, int ci, int taps, int bits) {
    const float *w = *wp, *b = w + (size_t)co * ci * taps;
    *wp = b + co;
    return umx_conv_create(kind, w, b, co, ci, bits);
}
void umx_unet_free(umx_unet *u) {
    if (!u) return;
    for (int l = 0; l < MAXL; l++) {
        umx_conv_free(u->enc1[l]); umx_conv_free(u->enc2[l]); umx_conv_free(u->down[l]); umx_conv_free(u->up[l]); umx_conv_free(u->dec1[l]); umx_conv_free(u->dec2[l]);
        nn_free(u->act[l]); nn_free(u->cat[l]); nn_free(u->s2d[l]); nn_free(u->dn[l]); nn_free(u->dec[l]);
    }
    umx_conv_free(u->head);
    nn_free(u->ybuf); nn_free(u->part); nn_free(u->coef); nn_free(u->x16); nn_free(u->xu8); nn_free(u->logits16);
    for (int k = 0; k < 2; k++) { nn_free(u->pxu8[k]); nn_free(u->plog[k]); nn_free(u->pprob[k]); umx_event_free(u->ev_up[k]); umx_event_free(u->ev_used[k]); umx_event_free(u->ev_ready[k]); umx_event_free(u->ev_down[k]); }
    umx_stream_free(u->s_in); umx_stream_free(u->s_out);
    free(u);
}
umx_unet *umx_unet_create(const umx_unet_cfg *cfg, const float *weights, int max_batch) {
    if (cfg->L < 2 || cfg->L > MAXL || max_batch < 1 || (cfg->P >> (cfg->L - 1)) < 1 || (cfg->P & ((1 << (cfg->L - 1)) - 1))) { fprintf(stderr, "umx_unet_create: bad configuration\n"); abort(); }
    for (int l = 0; l < cfg->L; l++) if (cfg->cw[l] % 32) { fprintf(stderr, "umx_unet_create: widths must be multiples of 32\n"); abort(); }
    umx_unet *u = calloc(1, sizeof *u);
    u->cfg = *cfg; u->maxN = max_batch;
    const int L = cfg->L, N = max_batch, bf = cfg->bits_first, bm = cfg->bits_mid, bl = cfg->bits_last;
    for (int l = 0, D = cfg->P; l < L; l++, D /= 2) u->Dl[l] = D;
    const float *wp = weights;
    for (int l = 0; l < L; l++) {
        u->enc1[l] = mk(UMX_CONV3, &wp, cfg->cw[l], l ? cfg->cw[l] : 1, 27, l ? bm : bf);
        u->enc2[l] = mk(UMX_CONV3, &wp, cfg->cw[l], cfg->cw[l], 27, bm);
        if (l < L - 1) u->down[l] = mk(UMX_DOWN2, &wp, cfg->cw[l + 1], cfg->cw[l], 8, bm);
    }
    for (int l = L - 2; l >= 0; l--) {
        u->up[l] = mk(UMX_TCONV2, &wp, cfg->cw[l], cfg->cw[l + 1], 8, bm);
        u->dec1[l] = mk(UMX_CONV3, &wp, cfg->cw[l], 2 * cfg->cw[l], 27, bm);
        u->dec2[l] = mk(UMX_CONV3, &wp, cfg->cw[l], cfg->cw[l], 27, l ? bm : bl);
    }
    u->head = mk(UMX_CONV1, &wp, cfg->nh, cfg->cw[0], 1, bl);
    /* buffers; every MX tensor is sized for 8-bit rows so one plan serves both formats */
    size_t ymax = 0, pmax = 0; int cmax = 0;
    for (int l = 0; l < L; l++) {
        const size_t S = cube(u->Dl[l]); const int C = cfg->cw[l];
        if ((size_t)C * S > ymax) ymax = (size_t)C * S;
        const size_t pd = umx_stats_doubles(N, C, u->Dl[l], u->Dl[l], u->Dl[l]); if (pd > pmax) pmax = pd;
        if (C > cmax) cmax = C;
        u->act[l] = nn_malloc(umx_mx_bytes32(8, N, C, S));
        u->cat[l] = nn_malloc(umx_mx_bytes32(8, N, l < L - 1 ? 2 * C : C, S));
        if (l < L - 1) { u->s2d[l] = nn_malloc(umx_mx_bytes32(8, N, 8 * C, S / 8)); u->dec[l] = nn_malloc(umx_mx_bytes32(8, N, C, S)); }
        if (l) u->dn[l] = nn_malloc(umx_mx_bytes32(8, N, C, S));
    }
    const size_t S0 = cube(cfg->P);
    u->ybuf = nn_malloc((size_t)N * ymax * 2);
    u->part = nn_malloc(pmax * sizeof(double));
    u->coef = nn_malloc((size_t)N * cmax * 2 * sizeof(float));
    u->x16 = nn_malloc((size_t)N * S0 * 2); u->xu8 = nn_malloc((size_t)N * S0);
    u->logits16 = nn_malloc((size_t)N * cfg->nh * S0 * 2);
    nn_sync();
    const char *e = nn_check();
    if (e) { fprintf(stderr, "umx_unet_create: %s\n", e); umx_unet_free(u); return nullptr; }
    u->launches0 = umx_launch_count();
    return u;
}
long umx_unet_launches(const umx_unet *u) { return umx_launch_count() - u->launches0; }

/* conv -> blocked fp16 + partial sums -> coefficients -> apply into q (and q_s2d) */
static void conv_norm(umx_unet *u, const umx_conv *c, const void *x, int xflag, int N, int C, int D, void *q, int bits, int nb_dst, int b0, void *q_s2d) {
    /* UMX_STATS_EPILOGUE=1 in the environment: InstanceNorm sums in the conv's epilogue (see umx_conv_fwd_norm); off by default */
    static int epi = -1;
    if (epi < 0) { const char *e = getenv("UMX_STATS_EPILOGUE"); epi = e && *e == '1'; }
    umx_conv_fwd_norm(c, x, N, D, D, D, u->ybuf, u->part, nullptr, nullptr, 1e-5f, u->coef, (xflag ? xflag : UMX_X_SPLIT) | (epi ? UMX_STATS_EPILOGUE : 0));
    umx_in_apply(u->ybuf, u->coef, N, C, D, D, D, 2, q, bits, nb_dst, b0, q_s2d, nullptr, UMX_LAYOUT_SPLIT);
}
enum { FMT_PROB8 = -8 };     /* forward(): the head writes probability bytes (UMX_OUT_PROB8) */
/* x_dev: the fp16 patches, or (x_u8) the CT bytes themselves, which the first conv reads as byte / 255 */
static int forward_x(umx_unet *u, const void *x_dev, int x_u8, int N, void *logits, int logits_fmt) {
    const umx_unet_cfg *c = &u->cfg; const int L = c->L, bm = c->bits_mid, bl = c->bits_last;
    if (N < 1 || N > u->maxN) { fprintf(stderr, "umx_unet_forward: batch %d outside 1..%d\n", N, u->maxN); abort(); }
    for (int l = 0; l < L; l++) {
        const int D = u->Dl[l], C = c->cw[l], nb = C / 32;
        /* the first conv takes the fp16 patch itself (UMX_X_H16: quantised on the way in) */
        conv_norm(u, u->enc1[l], l ? u->dn[l] : x_dev, l ? 0 : (x_u8 ? UMX_X_U8 : UMX_X_H16), N, C, D, u->act[l], bm, 0, 0, nullptr);
        if (l < L - 1) {
            conv_norm(u, u->enc2[l], u->act[l], 0, N, C, D, u->cat[l], bm, 2 * nb, nb, u->s2d[l]);
            umx_conv_fwd(u->down[l], u->s2d[l], N, D / 2, D / 2, D / 2, u->dn[l + 1], UMX_OUT_MX, bm, 0, 0, nullptr, UMX_X_SPLIT | UMX_Y_SPLIT);
        } else conv_norm(u, u->enc2[l], u->act[l], 0, N, C, D, u->cat[l], bm, 0, 0, nullptr);
    }
    const void *cur = u->cat[L - 1];
    for (int l = L - 2; l >= 0; l--) {
        const int D = u->Dl[l], C = c->cw[l], nb = C / 32, Dc = u->Dl[l + 1];
        umx_conv_fwd(u->up[l], cur, N, Dc, Dc, Dc, u->cat[l], UMX_OUT_MX, bm, 2 * nb, 0, nullptr, UMX_X_SPLIT | UMX_Y_SPLIT);
        conv_norm(u, u->dec1[l], u->cat[l], 0, N, C, D, u->act[l], l ? bm : bl, 0, 0, nullptr);
        conv_norm(u, u->dec2[l], u->act[l], 0, N, C, D, u->dec[l], l ? bm : bl, 0, 0, nullptr);
        cur = u->dec[l];
    }
    umx_conv_fwd(u->head, cur, N, c->P, c->P, c->P, logits, logits_fmt == UMX_F16 ? UMX_OUT_PM16 : logits_fmt == FMT_PROB8 ? UMX_OUT_PROB8 : UMX_OUT_PM32, 0, 0, 0, nullptr, UMX_X_SPLIT);
    return 0;
}
static int forward(umx_unet *u, const void *x_dev, int N, void *logits, int logits_fmt) { return forward_x(u, x_dev, 0, N, logits, logits_fmt); }
int umx_unet_forward(umx_unet *u, const void *x_dev, int N, float *logits_dev) { return forward(u, x_dev, N, logits_dev, UMX_F32); }
int umx_unet_forward_h16(umx_unet *u, const void *x_dev, int N, void *logits_dev) { return forward(u, x_dev, N, logits_dev, UMX_F16); }
/* uint8 CT patches on the host -> fp16 logits on the host: copy in, convert, forward, copy out */
int umx_unet_forward_host(umx_unet *u, const uint8_t *ct_host, int N, void *logits16_host) {
    const size_t S = cube(u->cfg.P);
    nn_h2d(u->xu8, ct_host, (size_t)N * S);
    forward_x(u, u->xu8, 1, N, u->logits16, UMX_F16);
    nn_d2h(logits16_host, u->logits16, (size_t)N * u->cfg.nh * S * 2);
    return nn_check() ? -1 : 0;
}
/* The same work, queued: returns once the copies and kernels are enqueued.  The upload of this call's patches and the download of its
   logits run on two copy streams and overlap the forward of the neighbouring calls (two slots, so at most two calls are in flight;
   a third waits on the device, not on the host).  ct_host and logits16_host should be pinned and must stay valid, and logits16_host
   unread, until umx_unet_wait returns.  0, or -1 with the message in lp_check(). */
static int pipe_init(umx_unet *u) {
    if (u->pipe_ok) return 0;
    const size_t S = cube(u->cfg.P);
    u->s_in = umx_stream_new(); u->s_out = umx_stream_new();
    for (int k = 0; k < 2; k++) {
        u->pxu8[k] = nn_malloc((size_t)u->maxN * S); u->plog[k] = nn_malloc((size_t)u->maxN * u->cfg.nh * S * 2); u->pprob[k] = nn_malloc((size_t)u->maxN * u->cfg.nh * S);
        u->ev_up[k] = umx_event_new(); u->ev_used[k] = umx_event_new(); u->ev_ready[k] = umx_event_new(); u->ev_down[k] = umx_event_new();
        if (!u->pxu8[k] || !u->plog[k] || !u->pprob[k] || !u->ev_up[k] || !u->ev_used[k] || !u->ev_ready[k] || !u->ev_down[k]) return -1;
    }
    if (!u->s_in || !u->s_out) return -1;
    u->pipe_ok = 1;
    return 0;
}
static int submit_host(umx_unet *u, const uint8_t *ct_host, int N, void *logits16_host, int as_u8) {
    if (N < 1 || N > u->maxN) { fprintf(stderr, "umx_unet_submit_host: batch %d outside 1..%d\n", N, u->maxN); abort(); }
    if (pipe_init(u)) return -1;
    const size_t S = cube(u->cfg.P);
    const int k = (int)(u->seq & 1);
    /* upload: the slot's bytes of two calls ago have been converted */
    umx_stream_wait(u->s_in, u->ev_used[k]);
    umx_copy_async(u->pxu8[k], ct_host, (size_t)N * S, 1, u->s_in);
    umx_event_record(u->ev_up[k], u->s_in);
    /* forward on the legacy default stream: after the upload, and after the slot's logits of two calls ago have left */
    umx_stream_wait(nullptr, u->ev_up[k]);
    umx_stream_wait(nullptr, u->ev_down[k]);
    /* the first conv reads the bytes itself and the head writes the probability bytes itself: no conversion pass on either side */
    if (as_u8) forward_x(u, u->pxu8[k], 1, N, u->pprob[k], FMT_PROB8); else forward_x(u, u->pxu8[k], 1, N, u->plog[k], UMX_F16);
    umx_event_record(u->ev_used[k], nullptr);          /* the slot's bytes have been read (by the first conv; recorded behind the forward) */
    umx_event_record(u->ev_ready[k], nullptr);
    /* download */
    umx_stream_wait(u->s_out, u->ev_ready[k]);
    if (as_u8) umx_copy_async(logits16_host, u->pprob[k], (size_t)N * u->cfg.nh * S, 0, u->s_out);
    else umx_copy_async(logits16_host, u->plog[k], (size_t)N * u->cfg.nh * S * 2, 0, u->s_out);
    umx_event_record(u->ev_down[k], u->s_out);
    u->seq++;
    return umx_has_error() ? -1 : 0;     /* launch errors latched so far; nothing here waits for the device (umx_unet_wait reports the rest) */
}
int umx_unet_submit_host(umx_unet *u, const uint8_t *ct_host, int N, void *logits16_host) { return submit_host(u, ct_host, N, logits16_host, 0); }
int umx_unet_submit_host_u8(umx_unet *u, const uint8_t *ct_host, int N, uint8_t *prob_host) { return submit_host(u, ct_host, N, prob_host, 1); }
int umx_unet_wait(umx_unet *u) {
    if (u->pipe_ok) { umx_stream_sync(u->s_in); umx_stream_sync(u->s_out); }
    nn_sync();
    return nn_check() ? -1 : 0;
}

/* ---------------- sliding window ---------------- */
umx_window umx_window_make(int V, int P, int overlap) {
    umx_window w = {V, P, overlap, 1, 1};
    const int stride = P - overlap;
    w.nper = V <= P ? 1 : (V - P + stride - 1) / stride + 1;
    w.npatch = w.nper * w.nper * w.nper;
    return w;
}
/* patch idx in (z, y, x) order; the last patch of an axis is pulled back so it ends at the volume's edge */
void umx_window_origin(const umx_window *w, int idx, int *z0, int *y0, int *x0) {
    const int stride = w->P - w->overlap, n = w->nper;
    const int iz = idx / (n * n), iy = (idx / n) % n, ix = idx % n;
    const int lim = w->V > w->P ? w->V - w->P : 0;
    *z0 = iz * stride < lim ? iz * stride : lim; *y0 = iy * stride < lim ? iy * stride : lim; *x0 = ix * stride < lim ? ix * stride : lim;
}
/* contiguous shares of the (z, y) patch rows: ranks get whole rows of nper patches, z-slab first (src/predict.c:2696-2717) */
void umx_window_share(const umx_window *w, int rank, int world, int *first, int *count) {
    const int rows = w->nper * w->nper, base = rows / world, extra = rows % world;
    const int r0 = rank * base + (rank < extra ? rank : extra), nr = base + (rank < extra ? 1 : 0);
    *first = r0 * w->nper; *count = nr * w->nper;
}
void umx_window_extent(const umx_window *w, int first, int count, int *zlo, int *zhi) {
    int z0, y0, x0, z1;
    if (count <= 0) { *zlo = 0; *zhi = 0; return; }
    umx_window_origin(w, first, &z0, &y0, &x0); umx_window_origin(w, first + count - 1, &z1, &y0, &x0);
    *zlo = z0; *zhi = (z1 + w->P < w->V ? z1 + w->P : w->V);
}
/* ---------------- the sliding window with exact blending and a share per rank ----------------
   A rank forwards its contiguous share of the (z, y) patch rows and blends the logits into 64-bit fixed-point accumulators on its device
   (umx_blend_add_fx: integer sums, so the result does not depend on the order, the batch or the partition).  A row (z, y) of the volume
   that only this rank's patches touch is final as soon as the rank's patch layer moves on: it is normalised and converted on the device
   and copied to the host while the next patches are forwarded.  A row that several ranks touch belongs to the lowest of them: the
   others hand their partial sums of it over (umx_wplan_pack on their side, umx_wplan_add on the owner's, the transport between the two
   devices is the caller's: a peer copy, a send / receive, or host memory), and umx_wplan_finish emits those rows last.  What crosses to
   the host is the finished volume, 1 or 2 bytes per voxel and head channel. */
enum { WP_MAXPEER = 64 };
typedef struct umx_wplan umx_wplan;
struct umx_wplan {
    umx_window w; int rank, world, first, count, zlo, zhi, nh;
    uint8_t *mode;                    /* host [zext][V]: 0 not touched by this rank, 1 this rank's alone, 2 this rank's, shared with higher ranks, 3 a lower rank's */
    long nsend[WP_MAXPEER], nrecv[WP_MAXPEER], nmine2; int *send_zy[WP_MAXPEER], *recv_zy[WP_MAXPEER], *mine2_zy;   /* (z - zlo, y) pairs in ascending order */
    long long *acc, *wsum; uint8_t *mode_dev; void *out_dev, *fin_dev; uint8_t *fin_host; float *logits; int out_fmt, batch; float *w1d; int *zy_dev; long zy_cap;
    void *ev_emit;
    /* the rank's planes of the volume on the device: uploaded piece by piece just ahead of the patches that read them (planes [zlo, zu)
       whole; of the current patch layer's new planes [ln0, ln1) the rows [yu0, yu)), each piece followed by an event of a ring of four */
    uint8_t *vol_dev; void *ev_vol[4]; int zu, lz0, ln0, ln1, yu0, yu, slot;
};
static void wp_rows_of_rank(const umx_window *w, int rank, int world, int *first, int *count) { umx_window_share(w, rank, world, first, count); }
umx_wplan *umx_wplan_create(const umx_window *w, int rank, int world, int nh) {
    if (world < 1 || world > WP_MAXPEER || rank < 0 || rank >= world || nh < 1) { fprintf(stderr, "umx_wplan_create: rank %d of %d (at most %d ranks)\n", rank, world, WP_MAXPEER); abort(); }
    umx_wplan *p = calloc(1, sizeof *p);
    p->w = *w; p->rank = rank; p->world = world; p->nh = nh;
    wp_rows_of_rank(w, rank, world, &p->first, &p->count);
    umx_window_extent(w, p->first, p->count, &p->zlo, &p->zhi);
    const int V = w->V, P = w->P, zext = p->zhi - p->zlo;
    if (zext <= 0) return p;
    /* which ranks touch a row (z, y) of this rank's extent: one bit a rank */
    uint64_t *mask = calloc((size_t)zext * V, sizeof *mask);
    for (int r = 0; r < world; r++) {
        int f, c; wp_rows_of_rank(w, r, world, &f, &c);
        for (int row = f / w->nper; row < (f + c) / w->nper; row++) {
            int z0, y0, x0; umx_window_origin(w, row * w->nper, &z0, &y0, &x0);
            const int za = z0 > p->zlo ? z0 : p->zlo, zb = (z0 + P < p->zhi ? z0 + P : p->zhi), yb = y0 + P < V ? y0 + P : V;
            for (int z = za; z < zb; z++) for (int y = y0; y < yb; y++) mask[(size_t)(z - p->zlo) * V + y] |= (uint64_t)1 << r;
        }
    }
    p->mode = malloc((size_t)zext * V);
    const uint64_t me = (uint64_t)1 << rank;
    for (int pass = 0; pass < 2; pass++) {       /* count, then fill */
        long ns[WP_MAXPEER] = {0}, nr[WP_MAXPEER] = {0}, n2 = 0;
        for (size_t i = 0; i < (size_t)zext * V; i++) {
            const uint64_t m = mask[i]; const int z = (int)(i / V), y = (int)(i % V);
            if (!(m & me)) { p->mode[i] = 0; continue; }
            const int owner = __builtin_ctzll(m);
            if (owner == rank) {
                p->mode[i] = m == me ? 1 : 2;
                if (m != me) {
                    if (pass) { p->mine2_zy[2 * n2] = z; p->mine2_zy[2 * n2 + 1] = y; }
                    n2++;
                    for (int r = rank + 1; r < world; r++) if (m >> r & 1) { if (pass) { p->recv_zy[r][2 * nr[r]] = z; p->recv_zy[r][2 * nr[r] + 1] = y; } nr[r]++; }
                }
            } else {
                p->mode[i] = 3;
                if (pass) { p->send_zy[owner][2 * ns[owner]] = z; p->send_zy[owner][2 * ns[owner] + 1] = y; }
                ns[owner]++;
            }
        }
        if (!pass) {
            p->nmine2 = n2; p->mine2_zy = malloc((size_t)(n2 ? n2 : 1) * 2 * sizeof(int));
            for (int r = 0; r < world; r++) {
                p->nsend[r] = ns[r]; p->nrecv[r] = nr[r];
                p->send_zy[r] = ns[r] ? malloc((size_t)ns[r] * 2 * sizeof(int)) : nullptr; p->recv_zy[r] = nr[r] ? malloc((size_t)nr[r] * 2 * sizeof(int)) : nullptr;
            }
        }
    }
    free(mask);
    return p;
}
void umx_wplan_free(umx_wplan *p) {
    if (!p) return;
    for (int r = 0; r < WP_MAXPEER; r++) { free(p->send_zy[r]); free(p->recv_zy[r]); }
    free(p->mine2_zy); free(p->mode);
    nn_free(p->acc); nn_free(p->wsum); nn_free(p->mode_dev); nn_free(p->out_dev); nn_free(p->fin_dev); nn_free(p->logits); nn_free(p->w1d); nn_free(p->zy_dev); umx_event_free(p->ev_emit);
    nn_free_host(p->fin_host);
    nn_free(p->vol_dev); for (int i = 0; i < 4; i++) umx_event_free(p->ev_vol[i]);
    free(p);
}
void umx_wplan_info(const umx_wplan *p, int *first, int *count, int *zlo, int *zhi) { *first = p->first; *count = p->count; *zlo = p->zlo; *zhi = p->zhi; }
/* rows this rank hands to `peer` (dir 0) or receives from it (dir 1); zy (optional, host): 2 ints a row, (z, y) in volume coordinates */
long umx_wplan_rows(const umx_wplan *p, int peer, int dir, int *zy) {
    if (peer < 0 || peer >= p->world) return 0;
    const long n = dir ? p->nrecv[peer] : p->nsend[peer]; const int *src = dir ? p->recv_zy[peer] : p->send_zy[peer];
    if (zy) for (long i = 0; i < n; i++) { zy[2 * i] = src[2 * i] + p->zlo; zy[2 * i + 1] = src[2 * i + 1]; }
    return n;
}
/* who has each row (z, y) of this rank's extent, mode [zhi - zlo][V]: 0 no patch of this rank touches it, 1 this rank's alone (delivered by
   umx_window_run_fx), 2 this rank's, shared with higher ranks (delivered by umx_wplan_finish), 3 a lower rank's (not delivered here) */
void umx_wplan_mode(const umx_wplan *p, uint8_t *mode) { if (p->mode) memcpy(mode, p->mode, (size_t)(p->zhi - p->zlo) * p->w.V); }
size_t umx_wplan_row_bytes(const umx_wplan *p) { return (size_t)(p->nh + 1) * p->w.V * sizeof(long long); }
static int *wp_zy_to_dev(umx_wplan *p, const int *zy, long n) {
    if (n > p->zy_cap) { nn_sync(); nn_free(p->zy_dev); p->zy_cap = n + n / 4 + 16; p->zy_dev = nn_malloc((size_t)p->zy_cap * 2 * sizeof(int)); if (!p->zy_dev) { p->zy_cap = 0; return nullptr; } }
    nn_h2d(p->zy_dev, zy, (size_t)n * 2 * sizeof(int));
    return p->zy_dev;
}
static int wp_alloc(umx_wplan *p, int out_fmt, int batch, size_t PS) {
    const int V = p->w.V, P = p->w.P, zext = p->zhi - p->zlo; const size_t plane = (size_t)V * V;
    if (!p->acc) {
        p->acc = nn_malloc((size_t)p->nh * zext * plane * 8); p->wsum = nn_malloc((size_t)zext * plane * 8);
        p->mode_dev = nn_malloc((size_t)zext * V); p->w1d = nn_malloc((size_t)P * 4); p->ev_emit = umx_event_new();
        p->vol_dev = nn_malloc((size_t)zext * plane); for (int i = 0; i < 4; i++) p->ev_vol[i] = umx_event_new();
        if (!p->acc || !p->wsum || !p->mode_dev || !p->w1d || !p->ev_emit || !p->vol_dev || !p->ev_vol[3]) return -1;
        float w1d_h[1024]; if (P > 1024) abort();
        { const double s = P / 8.0, c = (double)(P / 2);   /* the reference's centre: the integer P / 2 (g1_init, src/nn_ink3dext.cu:48-56) */
          for (int i = 0; i < P; i++) { const double d = (i - c) / s; w1d_h[i] = (float)exp(-0.5 * d * d); } }
        nn_h2d(p->w1d, w1d_h, (size_t)P * 4); nn_h2d(p->mode_dev, p->mode, (size_t)zext * V);
    }
    if (!p->out_dev || p->out_fmt != out_fmt) {
        const size_t el = out_fmt == UMX_F16 ? 2 : 1;
        nn_sync(); nn_free(p->out_dev); nn_free(p->fin_dev); nn_free_host(p->fin_host);
        p->out_dev = nn_malloc((size_t)p->nh * zext * plane * el); p->out_fmt = out_fmt;
        p->fin_dev = nn_malloc((size_t)(p->nmine2 ? p->nmine2 : 1) * p->nh * V * el); p->fin_host = nn_malloc_host((size_t)(p->nmine2 ? p->nmine2 : 1) * p->nh * V * el);
        if (!p->out_dev || !p->fin_dev || !p->fin_host) return -1;
    }
    if (p->batch < batch) {
        nn_sync(); nn_free(p->logits);
        p->logits = nn_malloc((size_t)batch * p->nh * PS * 4); p->batch = batch;
        if (!p->logits) { p->batch = 0; return -1; }
    }
    return nn_check() ? -1 : 0;
}
/* allocates what a run of this plan needs (the sums, the output image, staging buffers) so that umx_window_run_fx itself allocates nothing;
   optional: the run does it when it has not been done */
int umx_wplan_prepare(umx_wplan *p, umx_unet *u, int batch, int out_fmt) {
    if (p->zhi <= p->zlo) return 0;
    if (batch < 1) batch = 1; if (batch > u->maxN) batch = u->maxN;
    if (wp_alloc(p, out_fmt, batch, cube(p->w.P)) || pipe_init(u)) return -1;
    nn_sync();
    return nn_check() ? -1 : 0;
}
/* emit the rows that are this rank's alone in the box z in [za, zb) (planes of the extent), y in [ya, yb), and queue their copy to out_host
   [nh][zext][V][V] on the copy stream: per head channel one 2-D copy of (yb - ya) V contiguous elements a plane */
static void wp_emit_box(umx_unet *u, umx_wplan *p, int za, int zb, int ya, int yb, void *out_host) {
    if (zb <= za || yb <= ya) return;
    const int V = p->w.V, zext = p->zhi - p->zlo; const size_t plane = (size_t)V * V, el = p->out_fmt == UMX_F16 ? 2 : 1;
    umx_emit_fx(p->acc, p->wsum, p->mode_dev, 1, p->nh, V, zext, za, zb, ya, yb, p->out_fmt, p->out_dev);
    umx_event_record(p->ev_emit, nullptr);
    umx_stream_wait(u->s_out, p->ev_emit);
    for (int c = 0; c < p->nh; c++) {
        const size_t o = (((size_t)c * zext + za) * plane + (size_t)ya * V) * el;
        umx_copy2d_async((uint8_t *)out_host + o, plane * el, (uint8_t *)p->out_dev + o, plane * el, (size_t)(yb - ya) * V * el, (size_t)(zb - za), 0, u->s_out);
    }
}
/* issues the upload of what patch q reads of the volume and has not been uploaded yet: patches come in (z, y, x) order, so a layer's new
   planes are uploaded row range by row range as its patch rows come up (2-D copies on the copy stream; the host memory may be pageable) */
static void wp_upload(umx_unet *u, umx_wplan *p, const uint8_t *vol, int q) {
    const umx_window *w = &p->w; const int P = w->P, V = w->V; const size_t plane = (size_t)V * V;
    int z0, y0, x0; umx_window_origin(w, q, &z0, &y0, &x0);
    if (z0 != p->lz0) {
        if (p->lz0 >= 0 && p->yu0 == 0 && p->yu >= V && p->ln1 > p->zu) p->zu = p->ln1;      /* the layer before was uploaded in full */
        p->lz0 = z0; p->ln0 = z0 > p->zu ? z0 : p->zu; p->ln1 = z0 + P < p->zhi ? z0 + P : p->zhi;
        if (p->ln0 > p->ln1) p->ln0 = p->ln1;
        p->yu0 = p->yu = y0;
    }
    const int ye = y0 + P < V ? y0 + P : V;
    if (ye <= p->yu || p->ln1 <= p->ln0) return;
    const size_t off = (size_t)p->yu * V;
    umx_copy2d_async(p->vol_dev + (size_t)(p->ln0 - p->zlo) * plane + off, plane, vol + (size_t)p->ln0 * plane + off, plane, (size_t)(ye - p->yu) * V, (size_t)(p->ln1 - p->ln0), 1, u->s_in);
    p->yu = ye;
    p->slot = (p->slot + 1) & 3;
    umx_event_record(p->ev_vol[p->slot], u->s_in);
}
/* Forwards this rank's patches of the volume (vol_host: the V^3 uint8 volume; only the planes of the rank's extent are read), blends them,
   and delivers the rows that are this rank's alone to out_host [nh][zhi - zlo][V][V] (pinned), out_fmt UMX_F16 (blended logits) or UMX_U8OUT
   (round(254 sigmoid)).  Rows shared with other ranks are left to umx_wplan_pack / umx_wplan_add / umx_wplan_finish.  Returns 0, or -1 with
   the message in lp_check(). */
int umx_window_run_fx(umx_unet *u, umx_wplan *p, const uint8_t *vol, int batch, int out_fmt, void *out_host) {
    const umx_window *w = &p->w; const int P = w->P, V = w->V, nh = u->cfg.nh;
    if (P != u->cfg.P || nh != p->nh) { fprintf(stderr, "umx_window_run_fx: patch size %d / %d heads do not match the network's %d / %d\n", P, p->nh, u->cfg.P, nh); abort(); }
    if (batch < 1) batch = 1; if (batch > u->maxN) batch = u->maxN;
    const int zext = p->zhi - p->zlo; if (zext <= 0 || p->count <= 0) return 0;
    const size_t PS = cube(P), plane = (size_t)V * V;
    if (wp_alloc(p, out_fmt, batch, PS) || pipe_init(u)) return -1;
    float *logits = p->logits;
    nn_zero(p->acc, (size_t)nh * zext * plane * 8); nn_zero(p->wsum, (size_t)zext * plane * 8);
    /* emission: [ra, rb) the planes from the end of the previous layer's own planes to the origin of the next layer (no later layer touches
       them), lz the current layer's origin, y_done the first row of those planes not delivered yet */
    long j = 0; int lz = -1, ra = p->zlo, rb = p->zlo, y_done = 0, y_row = -1;
    p->zu = p->zlo; p->lz0 = -1; p->ln0 = p->ln1 = p->zlo; p->yu0 = p->yu = 0; p->slot = 0;
    const int last = p->first + p->count;
    for (int q = p->first; q < last; q += batch, j++) {
        const int nb = q + batch <= last ? batch : last - q;
        for (int i = 0; i < nb; i++) wp_upload(u, p, vol, q + i);       /* issued a batch ago by the look-ahead below, as a rule */
        umx_stream_wait(nullptr, p->ev_vol[p->slot]);
        for (int i = 0; i < nb; i++) {
            int z0, y0, x0; umx_window_origin(w, q + i, &z0, &y0, &x0);
            umx_gather_u8_h16(p->vol_dev, V, z0 - p->zlo, y0, x0, P, (uint8_t *)u->x16 + (size_t)i * PS * 2);
        }
        forward(u, u->x16, nb, logits, UMX_F32);
        for (int i = 0; i < batch && q + nb + i < last; i++) wp_upload(u, p, vol, q + nb + i);      /* while the GPU works on this batch */
        for (int i = 0; i < nb; i++) {
            int z0, y0, x0; umx_window_origin(w, q + i, &z0, &y0, &x0);
            if (z0 != lz) {           /* a new patch layer: what is left of the previous layer's own planes has had its last contribution from this rank */
                if (lz >= 0) { wp_emit_box(u, p, ra - p->zlo, rb - p->zlo, y_done, V, out_host); ra = rb; }
                lz = z0; y_done = 0; y_row = y0;
                const int nn2 = w->nper * w->nper, nxt = ((q + i) / nn2 + 1) * nn2;      /* the first patch of the next layer */
                rb = p->zhi;
                if (nxt < w->npatch) { int za, ya, xa; umx_window_origin(w, nxt, &za, &ya, &xa); if (za < rb) rb = za; }
                if (rb < ra) rb = ra;
            } else if (y0 != y_row) { /* a new patch row of the layer: the rows below its first row are complete in the layer's own planes */
                wp_emit_box(u, p, ra - p->zlo, rb - p->zlo, y_done, y0, out_host); y_done = y0; y_row = y0;
            }
            umx_blend_add_fx(logits + (size_t)i * nh * PS, nh, P, V, p->zlo, zext, z0, y0, x0, p->w1d, p->acc, p->wsum);
        }
    }
    wp_emit_box(u, p, ra - p->zlo, zext, y_done, V, out_host);
    umx_stream_sync(u->s_in); umx_stream_sync(u->s_out);
    nn_sync();
    return nn_check() ? -1 : 0;
}
/* this rank's partial sums of the rows it hands to `peer`, compact, into buf_dev (device, umx_wplan_rows(p, peer, 0, NULL) x umx_wplan_row_bytes bytes) */
int umx_wplan_pack(umx_wplan *p, int peer, void *buf_dev) {
    const long n = p->nsend[peer]; if (n <= 0) return 0;
    int *zy = wp_zy_to_dev(p, p->send_zy[peer], n); if (!zy) return -1;
    umx_rows_fx(p->acc, p->wsum, zy, n, p->nh, p->w.V, p->zhi - p->zlo, 0, buf_dev);
    nn_sync();
    return nn_check() ? -1 : 0;
}
/* adds the partial sums that `peer` packed for this rank (buf_dev on this rank's device) */
int umx_wplan_add(umx_wplan *p, int peer, const void *buf_dev) {
    const long n = p->nrecv[peer]; if (n <= 0) return 0;
    int *zy = wp_zy_to_dev(p, p->recv_zy[peer], n); if (!zy) return -1;
    umx_rows_fx(p->acc, p->wsum, zy, n, p->nh, p->w.V, p->zhi - p->zlo, 1, (void *)buf_dev);
    nn_sync();
    return nn_check() ? -1 : 0;
}
/* after every umx_wplan_add: the rows this rank shares with higher ranks, into out_host */
int umx_wplan_finish(umx_wplan *p, void *out_host) {
    const long n = p->nmine2; if (n <= 0) return 0;
    const int V = p->w.V, zext = p->zhi - p->zlo; const size_t el = p->out_fmt == UMX_F16 ? 2 : 1, plane = (size_t)V * V, rowb = (size_t)V * el;
    int *zy = wp_zy_to_dev(p, p->mine2_zy, n); if (!zy) return -1;
    void *cd = p->fin_dev; uint8_t *ch = p->fin_host;
    if (!cd || !ch) return -1;
    umx_emit_rows_fx(p->acc, p->wsum, zy, n, p->nh, V, zext, p->out_fmt, cd);
    nn_d2h(ch, cd, (size_t)n * p->nh * rowb);
    for (long r = 0; r < n; r++) for (int c = 0; c < p->nh; c++)
        memcpy((uint8_t *)out_host + (((size_t)c * zext + p->mine2_zy[2 * r]) * plane + (size_t)p->mine2_zy[2 * r + 1] * V) * el, ch + ((size_t)r * p->nh + c) * rowb, rowb);
    return nn_check() ? -1 : 0;
}
