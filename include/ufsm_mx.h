/* ufsm_mx: B200 (sm_100a) implementation of ufsm's MX block-scaled 3-D convolution forward path, behind a C ABI.

   Every pointer named "device" is CUDA device memory of the current device; all work is issued on the legacy default stream
   and is synchronous in that stream, as in the reference (src/nn.h:1-2).  CUDA errors are latched, not returned: lp_check()
   returns and clears the first message (src/lp_common.cuh:35-38, src/lp_f8wgrad.cu:140).  Invalid argument combinations print
   to stderr and abort(), as the reference's entry points do (src/lp_f8fwd.cu:28,35,44).  There is no CPU fallback: without a
   usable sm_100 device every compute entry latches an error.

   Storage types (xbf / ybf / dt codes of src/nn_lp.h:50-54): 0 fp32, 1 bf16, 2 fp16, plane-major [n][C][D][H][W];
   3 MX-fp8 (E4M3), 4 MX-fp4 (E2M1): channel-blocked codes data[n][blk][voxel][bw] (fp4: two nibbles a byte, low nibble first)
   followed by the UE8M0 scale plane sc[n][blk][voxel], bw = 8 / 16 / 32 for C <= 8 / <= 16 / larger (src/lp_common.cuh:100-106,
   132-134).  One addition: UMX_H16B (18) = fp16 in the same 32-channel blocking, [n][blk][voxel][32] halfs (NDHWC inside a
   block; exactly NDHWC when C <= 32), the form in which a conv hands its output to the InstanceNorm apply. */
#pragma once
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- types of the reference interface ---- */
typedef struct { int n, c, d, h, w; } shape5;                                              /* src/nn.h:21 */
typedef struct { const float *gamma, *beta, *mean, *rstd; int G; int zs, zo, ns, zhw; } gnp_t;   /* src/nn_lp.h:15; G == 0: no transform */
typedef struct { const void *x2; int c_split; void *y2; int o_split; int accum; gnp_t gp2; int16_t up, yD; unsigned sr; unsigned wkey;
                 int zlo, zhi; int stored_stats; unsigned osr; int16_t zi0, Di, o_pad, zw0, zw1, yzo; } split_t;   /* src/nn_lp.h:32 */
enum { UMX_F32 = 0, UMX_BF16 = 1, UMX_F16 = 2, UMX_MX8 = 3, UMX_MX4 = 4, UMX_H16B = 18 };
/* MX-fp8 code layouts.  REF: the reference's rows, [n][blk][voxel][32 B].  SPLIT: the same bytes as two 16-byte-wide planes per block,
   [n][blk][half][voxel][16 B]; a halo row of ten voxels is then 160 contiguous bytes, which is what makes the TMA staging of the conv
   efficient.  The graph keeps its fp8 tensors SPLIT; MX-fp4 rows are 16 bytes already, so both names mean the reference layout there.
   The scale plane follows the codes unchanged in either layout. */
enum { UMX_LAYOUT_REF = 0, UMX_LAYOUT_SPLIT = 1 };
enum { UMX_X_SPLIT = 1, UMX_Y_SPLIT = 2,     /* flags of umx_conv_fwd: the MX-fp8 input / output tensor is in the split layout */
       UMX_STATS_EPILOGUE = 4,               /* umx_conv_fwd_norm: take the InstanceNorm sums in the conv's epilogue where the kernel can (see there) */
       UMX_X_H16 = 8,                        /* x is the planar fp16 tensor [N][ci][D][H][W], not MX: the conv quantises it (UMX_CONV3 / UMX_CONV1) */
       UMX_X_U8 = 16 };                      /* x is a planar tensor of CT bytes, read as the fp16 values byte / 255 (umx_u8_to_h16), then as UMX_X_H16 */

/* ---- device runtime (src/nn.h:26-38: nn_init, nn_malloc, nn_free, nn_zero, nn_h2d, nn_d2h, nn_sync, nn_check) ---- */
int nn_init(int device);                 /* select the device, check it is sm_100; 0 on success */
void *nn_malloc(size_t bytes);
void nn_free(void *p);
void nn_zero(void *p, size_t bytes);
void nn_h2d(void *dst, const void *src, size_t bytes);
void nn_d2h(void *dst, const void *src, size_t bytes);
void nn_sync(void);
const char *nn_check(void);              /* NULL, or the first error since the last call (same latch as lp_check) */
const char *lp_check(void);              /* src/nn_lp.h:172 */
/* self-test of the kernels' bounded waits (no counterpart in the reference): a one-block kernel waits at most limit_clocks on a barrier nobody
   arrives on and gives up as a conv role would; 0 when it ran, and lp_check() then reports "bounded wait gave up" */
int umx_wait_selftest(long long limit_clocks);
void *umx_stream_new(void);               /* non-blocking copy stream, events and stream-ordered copies used by umx_unet_submit_host */
void umx_stream_free(void *stream);
void *umx_event_new(void);
void umx_event_free(void *ev);
void umx_event_record(void *ev, void *stream);           /* stream NULL: the legacy default stream */
void umx_stream_wait(void *stream, void *ev);
void umx_stream_sync(void *stream);
void umx_event_sync(void *ev);                           /* the host waits for the event */
void umx_copy_async(void *dst, const void *src, size_t bytes, int to_device, void *stream);
void umx_copy2d_async(void *dst, size_t dpitch, const void *src, size_t spitch, size_t width, size_t height, int to_device, void *stream);
void *nn_malloc_host(size_t bytes);      /* pinned host memory (cudaHostAlloc) for the window scheduler's staging buffers */
void nn_free_host(void *p);

/* timing with CUDA events on the stream the library launches on (the legacy default stream) */
void *umx_timer_new(void);
void umx_timer_start(void *t);           /* synchronises, then records the start event */
float umx_timer_stop_ms(void *t);        /* records the stop event, waits for it, returns the elapsed milliseconds */
void umx_timer_mark(void *t);            /* the same in two steps: record the stop event ... */
float umx_timer_read_ms(void *t);        /* ... wait for it and return the elapsed milliseconds */
void umx_timer_free(void *t);
/* between umx_prof_begin and umx_prof_end every conv kernel launch is bracketed by events: umx_prof_end returns the number of conv
   launches, their summed device time (ms) and their summed algorithmic FLOPs (2 x output voxels x C_in x C_out x taps) */
void umx_prof_begin(void);
int umx_prof_end(double *ms, double *flops);
int umx_prof_get(int i, double *ms, double *flops);   /* the i-th conv launch of the last profiled span; -1 past the end */

/* ---- MX storage and the quantiser (src/nn_lp.h:110-118, 126; kernels src/lp_mx_cvt.cu:9-19, 59-79, 429-447) ---- */
size_t lp_mx8_bytes(int N, int C, size_t S);
size_t lp_mx4_bytes(int N, int C, size_t S);
void lp_f32_to_mx8(const float *x, int N, int C, size_t S, void *y);                 /* x device fp32 [n][C][S] -> y device MX-fp8 */
void lp_f32_to_mx4(const float *x, int N, int C, size_t S, void *y);
void lp_h16_to_mx8(const void *x, int dt, int N, int C, size_t S, void *y);           /* dt 2 fp16 (1 bf16 aborts: not built) */
void lp_h16_to_mx4(const void *x, int dt, int N, int C, size_t S, void *y);
void lp_mx8_to_f32(const void *x, int N, int C, size_t S, float *y);
void lp_mx4_to_f32(const void *x, int N, int C, size_t S, float *y);
/* the same quantiser with 32-wide blocks whatever C (padding channels zero): the form the graph below keeps its tensors in */
size_t umx_mx_bytes32(int bits, int N, int C, size_t S);
void umx_pm_to_mx32(const void *x, int dt, int N, int C, size_t S, void *y, int bits, int layout);   /* dt 0 fp32 / 1 bf16 / 2 fp16 plane-major */
/* an MX tensor of C <= 16 channels (rows of 8 or 16 channels, src/lp_common.cuh:132-134) as the same tensor with 32-wide rows
   (to_wide) or back: the same codes and scale bytes, zeros behind them */
void umx_mx_rewidth(const void *x, int bits, int N, int C, size_t S, void *y, int to_wide);
/* src/nn_lp.h:164-165, src/lp_mx_cvt.cu:20-57: the network input of the reference's predict for planes [z0, z0 + nz) of a W x W CT
   window (device pointers): channel 0 (ct - mean) isd, 1 zero, 2 / 3 the unit (dy, dx) away from the scroll axis at (-dyo[z], -dxo[z])
   times axis (0: none), rounded to hd (2 fp16, 1 bf16, 0 fp32), stored as an MX tensor of 4 channels (8-wide rows) and depth nz */
void lp_pred_input_mx(const uint8_t *ct, int W, float mean, float isd, const float *dyo, const float *dxo, int axis, int z0, int nz, void *y, int hd, int bits);
void lp_pred_input_mx8(const uint8_t *ct, int W, float mean, float isd, const float *dyo, const float *dxo, int axis, int z0, int nz, void *y, int hd);
/* the same from two tensors, channels [0, c2) of the C from x and the rest from x2 (the concat input of split_t.x2 / c_split,
   src/nn_lp.h:20: rows of 32 channels over the concatenated index); x2 NULL: one tensor */
void umx_pm_to_mx32_cat(const void *x, const void *x2, int c2, int dt, int N, int C, size_t S, void *y, int bits, int layout);
void umx_mx32_to_f32(const void *x, int bits, int N, int C, size_t S, float *y, int layout);         /* -> plane-major fp32 */
void umx_mx_relayout(const void *src, int bits, int N, int C, size_t S, void *dst, int to_layout);   /* 32-wide MX tensor between the two layouts */
void umx_h16b_to_f32(const void *x, int N, int C, size_t S, float *y);                   /* blocked fp16 -> plane-major fp32 */

/* ---- 3x3x3 stride-1 pad-1 conv forward, the reference's entry points (src/nn_lp.h:53-54; src/lp_f8fwd.cu:26-52,
   src/lp_f4fwd.cu:30-51).  x: device, xbf 3 / 4 (MX; 16 channels or fewer in rows of 8 / 16) or 2 (fp16 plane-major, quantised to the
   conv's MX format first); w: device fp32 [cout][cin][27]; b: device fp32 [cout] or NULL; y: ybf 2 (fp16 plane-major), 3 / 4 (MX,
   acc + bias requantised per 32 output channels; 16 channels or fewer in rows of 8 / 16) or UMX_H16B.  lp_conv_fwd_f8 multiplies E4M3
   codes, lp_conv_fwd_f4 E2M1 codes; an MX input of the other format needs a transform that requantises it.  gp.G != 0: the GroupNorm +
   SiLU input transform silu(fma(x, rstd gamma, beta - mean rstd gamma)) (src/lp_common.cuh:244-261, 474-482), applied and quantised to
   the conv's format in a pass ahead of the conv (x may then be fp32 / fp16 plane-major or either MX format).
   split_t (src/nn_lp.h:20-41), served by passes into scratch around the conv: x2 / c_split (concat input; MX parts keep their own
   32-channel blocks, parts of 16 channels or fewer in rows of 8 / 16), gp2, up (the x part at half resolution, read as its trilinear 2x
   upsample), y2 / o_split / o_pad (split output, fp16 plane-major or MX, each part an MX tensor of its own rows), accum (fp16
   plane-major y += conv), osum / Go (exact GroupNorm sums over the planes [zlo, D - zhi): stored_stats 1, of the stored MX values, also of a split
   output whose first part ends on a 32-channel block; stored_stats 0, of acc + bias before rounding, through an fp32 copy of the output), zi0 / Di, zw0 / zw1, yD / yzo (z range, z window, output into a deeper
   tensor), wkey (prepared-weight memo).  What is not built prints "... is not built in this library" and aborts: stochastic rounding
   (sr / osr), osum of a stored output that is not MX or of the unrounded values of a split output, the z fields
   together with up, a transform of concat parts of 16 channels or fewer.  Returns 0. ---- */
int lp_conv_fwd_f8(const void *x, int xbf, shape5 xs, const float *w, const float *b, int cout, void *y, int ybf, gnp_t gp, double *osum, int Go, split_t sp);
int lp_conv_fwd_f4(const void *x, int xbf, shape5 xs, const float *w, const float *b, int cout, void *y, int ybf, gnp_t gp, double *osum, int Go, split_t sp);
void lp_wmemo_clear(void);               /* src/nn_lp.h:57: drop the prepared weights kept under split_t.wkey */
/* 3x3x3 stride-2 pad-1 conv forward (src/nn_lp.h:104; src/lp_s2.cu:647-754), fp32 accumulate.  x: xbf 3 (MX-fp8), 4 (MX-fp4) or 2 (fp16
   plane-major, quantised to MX-fp8 first); MX tensors of 16 channels or fewer in rows of 8 / 16; ys: the output shape, which must be
   ceil(xs / 2) per axis; y: ybf 2, 3, 4 or UMX_H16B as above (an MX output of 16 channels or fewer in rows of 8 / 16); gp as for
   lp_conv_fwd_f8.  An MX-fp4 input without a GroupNorm transform is multiplied in MX-fp4 (E2M1 weights; the cases of the reference's
   conv_fwd_s2_f4_k / conv_fwd_s2_f4p_k, here for every shape) and the call returns 3, the reference's "fp4 compute" report; every other
   call computes in E4M3 and returns 0.  Weights are prepared on every call, as in the reference. */
int lp_conv_fwd_s2_f8(const void *x, int xbf, shape5 xs, const float *w, const float *b, int cout, void *y, int ybf, shape5 ys, gnp_t gp);

/* ---- graph operators (the InstanceNorm / LeakyReLU / transposed-conv semantics of src/xnet.h:85-98) ---- */
enum { UMX_CONV3 = 0,      /* 3^3 stride 1 pad 1, w [co][ci][27]                         (xconv_init k3 s1 p1, src/nn_xnet.cu:615-637) */
       UMX_CONV1 = 1,      /* 1^3, w [co][ci]                                            (xhead, src/nn_xnet.cu:1751-1756) */
       UMX_DOWN2 = 2,      /* 2^3 stride 2 pad 0, w [co][ci][8]; input = space-to-depth copy (src/ink3dext_net.c:104-112) */
       UMX_TCONV2 = 3,     /* ConvTranspose3d k2 s2, w [ci][co][8]                       (xtconv3_init, src/nn_xnet.cu:650-662) */
       UMX_CONV3S2 = 4 };  /* 3^3 stride 2 pad 1, w [co][ci][27]; D, H, W of umx_conv_fwd are the input grid,
                              the output grid is ceil(D / 2) x ceil(H / 2) x ceil(W / 2)   (conv_fwd_s2_f8_k, conv_fwd_s2_f4_k, src/lp_s2.cu:23, 290, 647-754) */
enum { UMX_OUT_H16B = 0,   /* y = fp16(acc + bias), blocked fp16 */
       UMX_OUT_MX = 1,     /* y = MX(fp16(acc + bias)) into blocks [b0, ...) of an MX tensor with nb_dst blocks (xtconv_cat_q) */
       UMX_OUT_PM32 = 2,   /* y = acc + bias, plane-major fp32 [n][co][S] */
       UMX_OUT_PM16 = 3,   /* y = fp16(acc + bias), plane-major fp16 */
       UMX_OUT_MXRAW = 4,  /* y = MX(acc + bias) without the fp16 rounding (the lp epilogue, src/lp_common.cuh:1465-1536) */
       UMX_OUT_PROB8 = 5 };/* y = uint8 round(254 sigmoid(fp16(acc + bias))), plane-major [n][co][S]: the probability bytes of umx_h16_to_prob_u8 taken in
                              the conv's epilogue (UMX_CONV1 only: the network's head) */
typedef struct umx_conv umx_conv;
/* w, bias: host fp32 in PyTorch order (bias NULL: zero).  bits: 8 (E4M3) or 4 (E2M1) for weights and activations alike. */
umx_conv *umx_conv_create(int kind, const float *w, const float *bias, int co, int ci, int bits);
umx_conv *umx_conv_create_dev(int kind, const float *w_dev, const float *bias_dev, int co, int ci, int bits);   /* device weights */
void umx_conv_free(umx_conv *c);
/* x: MX tensor (32-wide blocks) of c->ci channels (UMX_DOWN2: the space-to-depth copy, 8 * ci channels at half resolution) on an
   N x D x H x W grid.  y per out_mode; nb_dst / b0: block count of the destination tensor and first block written (0, 0: the
   conv's own co).  part: optional device doubles for InstanceNorm partial sums (umx_stats_doubles), only with UMX_OUT_H16B.
   UMX_TCONV2 writes the 2D x 2H x 2W grid.  flags: UMX_X_SPLIT / UMX_Y_SPLIT (an fp8 input in the reference layout is re-laid into
   scratch first); UMX_X_H16: x is planar fp16 and is quantised to the conv's MX format on the way in (the values the quantiser gives;
   a 3^3 MX-fp8 conv of ONE input channel into at most 32 outputs with a UMX_OUT_H16B output runs as a tap-packed kernel that reads
   the fp16 tensor directly, the role of conv_fwd_f8s_k, src/lp_f8fwd.cuh:153-400; every other case is quantised into scratch first).
   Returns 0, or -1 after latching an error. */
int umx_conv_fwd(const umx_conv *c, const void *x, int N, int D, int H, int W, void *y, int out_mode, int out_bits, int nb_dst, int b0, double *part, int flags);
/* the conv with a blocked fp16 output followed by InstanceNorm: y as UMX_OUT_H16B and coef [N][co][2] = (a, b) of the stored values
   (k_in_coef, src/nn_xnet.cu:1565-1570), in one call; part: scratch of umx_stats_doubles doubles.  By default the sums are taken by the
   statistics pass over the stored tensor (fp64 in a fixed order: exact to the last bits, independent of batch size and block partition).
   With UMX_STATS_EPILOGUE the resident-weight 3^3 kernel takes them in its epilogue instead, as the reference's conv does (st_add,
   src/nn_xnet.cu:262-268, 370-390: fp32 partial sums per thread, then fp64 atomics, whose order changes from run to run).  Here they are
   fp64 sums of the stored fp16 values and of their squares, which are exact for a sample of any realistic size, so the coefficients are
   those of the pass, whatever the batch, the number of multiprocessors or the way the planes fall to the blocks.  The epilogue's extra
   work (a conversion and two fp64 operations per element) costs more than the pass saves on the benchmark's layers (measured: the
   level-0 conv goes from 72 to 120 us, the pass takes 33), which is why it is not the default. */
int umx_conv_fwd_norm(const umx_conv *c, const void *x, int N, int D, int H, int W, void *y, double *part, const float *gamma, const float *beta, float eps, float *coef, int flags);
size_t umx_stats_doubles(int N, int co, int D, int H, int W);   /* size of part for a conv output on that grid */
/* testing aid (no counterpart in the reference): at most `cap` thread blocks per column tile in the resident-weight 3^3 kernel (0: as many as
   the device holds), so that a small volume is cut into the several-planes-a-block pieces that otherwise only 64^3 and larger volumes see */
void umx_conv_r_block_cap(int cap);
int umx_conv_last_kernel(void);          /* which kernel the last umx_conv_fwd on this thread's process launched: 0 general, 1 resident-weight 3^3, 2 one-tap streaming, 3 tap-packed one-channel 3^3; -1 none yet */
/* coef [n][C][2] (device floats): a = gamma rstd, b = beta - mean a from the partial sums (k_in_coef, src/nn_xnet.cu:1565-1570);
   gamma / beta device arrays or NULL (1 / 0) */
void umx_in_coef(const double *part, int N, int C, int D, int H, int W, const float *gamma, const float *beta, float eps, float *coef);
/* the partial sums of a stored blocked-fp16 tensor y and the coefficients in one launch (part: scratch of umx_stats_doubles doubles); the
   same values as umx_conv_fwd's `part` followed by umx_in_coef up to fp64 summation order.  Calls on one device must not overlap. */
void umx_in_stats_coef(const void *y, int N, int C, int D, int H, int W, const float *gamma, const float *beta, float eps, double *part, float *coef);
/* No counterpart in the reference.  The same coefficients as umx_in_coef, computed from the stored blocked-fp16 tensor y itself
   (device, [n][blk][voxel][32] halfs) by a call that allocates nothing: for callers that must not touch the CUDA allocator (all memory
   already handed to their own pool, allocation forbidden after start-up, or a loop where cudaMalloc's device-wide synchronisation is
   not acceptable).  The partial sums live in a 4 MiB array built into the library's device image (one per GPU, held until exit), so
   N x 64 x roundup32(C) x 2 doubles must fit in 524288 (N = 1: C <= 4096; N = 8: C <= 512); larger sizes return -1 with a message in
   lp_check().  The first call on a device looks the array's address up.  All calls on a device
   share the array; calls that overlap on the GPU race, so issue them in order.  Returns 0 on success. */
int umx_in_coef_static(const void *y, int N, int C, int D, int H, int W, const float *gamma, const float *beta, float eps, float *coef);
/* y = fp16(act(x a + b)) requantised to MX (k_inq, src/nn_xnet.cu:1577-1620): x blocked fp16 [n][C][S]; act 2 = LeakyReLU 0.01,
   0 none; q: MX destination (bits) with nb_dst blocks, first block b0; q_s2d: optional second copy in 2x2x2 space-to-depth order
   (an MX tensor of 8 C channels on the half grid, the input of UMX_DOWN2) or NULL; h: optional blocked fp16 copy or NULL.
   coef NULL: identity (a = 1, b = 0).  layout: UMX_LAYOUT_REF / UMX_LAYOUT_SPLIT of q and q_s2d. */
void umx_in_apply(const void *x, const float *coef, int N, int C, int D, int H, int W, int act, void *q, int bits, int nb_dst, int b0, void *q_s2d, void *h, int layout);

/* ---- GroupNorm statistics of an MX tensor (src/nn_lp.h:175-176, src/lp_mx_gnsums.cu:9-106; finalise: src/nn_elem.cu:5-11).  x: device, xdt 3 / 4,
   reference layout (16 channels or fewer in rows of 8 / 16).  sums: device, 2 N G slots of 24 bytes (the reference's exact fixed point, src/gnacc.cuh:9-27:
   fraction in 2^-64, signed integer part, count of non-finite terms), zeroed by the caller; slot 2 (n G + g) takes the sum and the next one
   the sum of squares of group g of sample n over the voxels [v0, v1).  Returns 0, -1 when the combination is not covered (G > 64 or C % G != 0
   as in the reference).  umx_gn_finalize: mean and 1 / sqrt(max(var, 0) + eps) of NG groups of len elements. ---- */
/* y = MX(silu(groupnorm(x))) (src/nn_lp.h:134, src/lp_mx_gn.cu:4-31): x xdt 0 / 2 (fp32 / fp16 plane-major) or 3 / 4 (MX); y ydt 3 / 4; MX tensors of
   16 channels or fewer in rows of 8 / 16 (through a widened copy in scratch); mean, rstd per (sample, group).  SiLU is u * rcp(1 + ex2(-u log2 e))
   with the hardware approximations (about 1e-6 relative; the reference: __expf). */
void lp_gn_silu_apply_mx(const void *x, int xdt, shape5 s, int G, const float *gamma, const float *beta, const float *mean, const float *rstd, void *y, int ydt);
/* exact-2x trilinear upsample of an MX tensor (align_corners = false, edge clamp: 3/4 of the coarse voxel under the fine one, 1/4 of its neighbour
   on the fine voxel's side, per axis), the eight terms added with fma in (z, y, x) order; gp.G != 0: silu(gn(x)) is upsampled
   (src/nn_lp.h:136, src/lp_mx_gn.cu:32-72, 151-173).  xdt, ydt 3 / 4; y has the shape n x c x 2d x 2h x 2w; 16 channels or fewer in rows
   of 8 / 16 on both sides (through widened copies in scratch); gp.ns != 0: the statistics of the slab a coarse plane lies in. */
void lp_up2_fwd_mx(const void *x, int xdt, shape5 xs, void *y, int ydt, gnp_t gp);
/* 1^3 conv of an MX tensor with fp32 weights w [cout][cin] and bias b (or NULL): y [n][cout][S] fp32 (or fp16: _h16) = b + sum over ascending ci
   of w x with fma; cout <= 16, or a multiple of 16 for one sample; gp as above; an input of 16 channels or fewer in rows of 8 / 16
   (src/nn_lp.h:138-139, src/lp_mx_conv1.cu:4-22, 422-444). */
void lp_conv1_fwd_mx(const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, float *y, gnp_t gp);
void lp_conv1_fwd_mx_h16(const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, void *y, gnp_t gp);
/* src/nn_lp.h:140-141: the logits of voxels [vb, vb + nv) alone (nv 0: all) into planes of nv voxels (fp16) or of ly >= nv voxels (fp32, one
   sample; returns -1 for N != 1 or nv == 0 as the reference does): per voxel the bits of the whole-tensor entries */
void lp_conv1_fwd_mx_h16_r(const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, void *y, gnp_t gp, size_t vb, size_t nv);
int lp_conv1_fwd_mx_r(const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, float *y, gnp_t gp, size_t vb, size_t nv, size_t ly);
/* src/nn_lp.h:137: the upsample of the 32-channel blocks [b0, b0 + nbk) of x alone; y: an MX tensor of 32 nbk channels */
void lp_up2_fwd_mx_blocks(const void *x, int xdt, shape5 xs, int b0, int nbk, void *y, int ydt);
/* src/nn_lp.h:135, src/lp_mx_gn.cu:133-150: y += x for two MX tensors of the same format (dt 8 / 4 bits), rows re-encoded; sr (stochastic
   rounding) must be 0 */
void lp_add_mx(void *y, const void *x, shape5 s, int dt, unsigned sr);
int lp_gn_sums_mx(const void *x, int xdt, int N, int C, int G, size_t S, double *sums, size_t v0, size_t v1);
int lp_gn_sums_mx_n(const void *x, int xdt, int N, int C, int G, size_t S, double *sums, size_t v0, size_t v1, int n0, int cnt);
void umx_gn_finalize(const double *sums, int NG, size_t len, float eps, float *mean, float *rstd);

/* ---- the benchmark's U-Net (five levels 32/64/128/256/320, two 3^3 convs + InstanceNorm + LeakyReLU 0.01 a level, 2^3 stride-2
   down convs, ConvTranspose k2 s2 up, concat (up | skip), 1^3 head) and the sliding-window scheduler ---- */
typedef struct { int L; int cw[8]; int nh; int P; int bits_first, bits_mid, bits_last; } umx_unet_cfg;
typedef struct umx_unet umx_unet;
size_t umx_unet_nweights(const umx_unet_cfg *cfg);               /* floats of the flat weight array, forward order, each conv's bias after its weights */
umx_unet *umx_unet_create(const umx_unet_cfg *cfg, const float *weights_host, int max_batch);
void umx_unet_free(umx_unet *u);
/* x: device fp16 [N][1][P^3] (CT intensity / 255); logits: device fp32 [N][nh][P^3] (umx_unet_forward) or fp16 (.._h16).  0 on success. */
int umx_unet_forward(umx_unet *u, const void *x_dev, int N, float *logits_dev);
int umx_unet_forward_h16(umx_unet *u, const void *x_dev, int N, void *logits_dev);
/* the call a user of the library makes: uint8 CT patches [N][P^3] on the host (pinned or pageable) -> fp16 logits [N][nh][P^3] on the
   host; copies in, converts (x / 255 -> fp16), runs, copies out, synchronises.  0, or -1 with the message in lp_check(). */
int umx_unet_forward_host(umx_unet *u, const uint8_t *ct_host, int N, void *logits16_host);
/* the same work, queued: returns once copies and kernels are enqueued; the upload of this call's patches and the download of its logits
   overlap the forward of the neighbouring calls (two slots in flight).  Pinned host buffers, valid (and the logits unread) until
   umx_unet_wait returns.  No counterpart in the reference, whose predict overlaps I/O with a reader thread (src/predict.c:1772-1841). */
int umx_unet_submit_host(umx_unet *u, const uint8_t *ct_host, int N, void *logits16_host);
/* the same with the output as uint8 probabilities round(254 sigmoid(logit)) [N][nh][P^3], converted on the device: half the bytes back to the host */
int umx_unet_submit_host_u8(umx_unet *u, const uint8_t *ct_host, int N, uint8_t *prob_host);
int umx_unet_wait(umx_unet *u);
double umx_unet_flops(const umx_unet_cfg *cfg);                  /* 2 V_out C_in C_out taps summed over the convs, per patch */
long umx_unet_launches(const umx_unet *u);                       /* kernels launched by the library since this object was created */
long umx_launch_count(void);                                     /* kernels launched by the library in this process */
void umx_u8_to_h16(const uint8_t *x_dev, size_t n, void *y_dev); /* CT bytes -> fp16 x / 255 */
void umx_h16_to_prob_u8(const void *x_dev, size_t n, uint8_t *y_dev);   /* fp16 logits -> uint8 round(254 sigmoid), the probability bytes predict writes */
/* ---- the back end of the reference's predict on the device (src/nn.h:385, 871-885; src/nn_elem.cu:1096-1178): one head's logits of a
   D x W x W window -> probability bytes trunc(255 sigmoid(logit) + 0.5) where the CT voxel is material (0 elsewhere), the window's halo
   cropped (hz planes at either z end, halo voxels in y and x), written at (oz + z, oy + y, ox + x) of a device shard buffer [shard]^3 as
   far as that lies inside [0, ez) x [0, ey) x [0, ex).  lg: device fp32 logits, or fp16 after nn_set_logits_h16(1).  Material: ct >= the
   threshold of nn_set_pred_iso (default 1: CT != 0), or bit k of a mask made by nn_pred_ctmask(_t) (word k >> 5, bit k & 31).  The flag
   and the threshold are kept per device.  nn_pred_place_mz: the window is held from plane zoff on and only its planes [zlo, zhi) are placed. */
void nn_set_logits_h16(int on);
void nn_set_pred_iso(int t);
int nn_get_pred_iso(void);
void nn_pred_output(const float *lg, const uint8_t *ct, size_t n, uint8_t *out);             /* every voxel, no crop; material where ct != 0 */
void nn_pred_place(const float *lg, const uint8_t *ct, int W, int halo, int oz, int oy, int ox, int ez, int ey, int ex, int shard, uint8_t *dsh);
void nn_pred_place_d(const float *lg, const uint8_t *ct, int D, int W, int hz, int halo, int oz, int oy, int ox, int ez, int ey, int ex, int shard, uint8_t *dsh);
void nn_pred_ctmask(const uint8_t *ct, size_t n, uint32_t *bits);
void nn_pred_ctmask_t(const uint8_t *ct, size_t n, uint32_t *bits, int t);
void nn_pred_place_m(const float *lg, const uint32_t *bits, int W, int halo, int oz, int oy, int ox, int ez, int ey, int ex, int shard, uint8_t *dsh);
void nn_pred_place_m_d(const float *lg, const uint32_t *bits, int D, int W, int hz, int halo, int oz, int oy, int ox, int ez, int ey, int ex, int shard, uint8_t *dsh);
void nn_pred_place_mz(const float *lg, const uint32_t *bits, int W, int halo, int zlo, int zhi, int zoff, int oz, int oy, int ox, int ez, int ey, int ex, int shard, uint8_t *dsh);
/* the seam feather of the reference's predict (src/predict.c:282-333, there a host loop over downloaded windows) on the device.  Windows on a
   grid with interior S per axis; e: this window's prediction bytes over [0, S + B)^3 (interior plus B voxels of its upper halo); nb[d], d = 1..7:
   the spill of the window one step back along the axes of d's bits (bit 0 x, 1 y, 2 z), NULL where there is none: its z slab [B][S+B][S+B] if
   d has bit 2, else its y slab [S][B][S+B] if bit 1, else its x slab [S][S][B] (what umx_feather_keep stores of a window).  The interior voxels
   [oo, oo + on) per axis are written to out[(lz osh + ly) osh + lx]: e itself, except where a coordinate is below B, the weighted mean of e and
   the spills present with the weights prod (back ? 1 - u : u), u(j) = sin^2(pi / 2 (j + 0.5) / B), rounded as min(255, s / w + 0.5).  All
   pointers are device pointers.  Returns 0, -1 after latching an error. */
typedef struct { int S, B; const uint8_t *e; const uint8_t *nb[8]; int oo[3], on[3], osh; uint8_t *out; } umx_feather_t;
int umx_feather_blend(const umx_feather_t *f);
void umx_feather_keep(const uint8_t *e, int S, int B, uint8_t *zslab, uint8_t *yslab, uint8_t *xslab);
/* the reference's blend arithmetic, kept as an operator of its own: acc[c][z - zlo][y][x] = fma(w, logits[c][patch voxel], acc), wsum += w with
   the separable Gaussian window w1d (device, P floats) for the patch at (z0, y0, x0) of a V^3 volume; fmt UMX_F32 / UMX_F16 logits (k_i3_blend,
   src/nn_ink3dext.cu:58-73); fp32 sums, so the result depends on the order of the calls */
void umx_blend_add(const void *logits_dev, int fmt, int nh, int P, int V, int zlo, int zext, int z0, int y0, int x0, const float *w1d_dev, float *acc_dev, float *wsum_dev);

/* Sliding window over a V^3 uint8 volume (host): P^3 patches at stride P - overlap, Gaussian window sigma P / 8 about the integer centre
   P / 2, the (z, y) rows of the patch grid dealt to ranks in contiguous shares, z-slab first (src/predict.c:2696-2717; blend and emit
   src/nn_ink3dext.cu:48-73, 77-100).  A rank forwards its patches and blends them on its device into 64-bit fixed-point sums (a term is
   the exact product of the fp32 window weight and the fp32 logit rounded to a multiple of 2^-46; integer sums: the result does not
   depend on the order, the batch or the partition, which the reference's fp32 atomics cannot promise).  Rows (z, y) of the volume that
   only this rank's patches touch are normalised and converted on the device and copied to the host while later patches run; a row
   that several ranks touch belongs to the lowest of them: the others hand over their partial sums of it (umx_wplan_pack ->
   transport of the caller's choice -> umx_wplan_add), and umx_wplan_finish emits those rows.  What reaches the host is the finished
   volume: out [nh][zhi - zlo][V][V] of fp16 blended logits (UMX_F16) or of uint8 round(254 sigmoid(logit)), 255 where no patch covers
   a voxel (UMX_U8OUT; k_i3_emit).  With one rank nothing is shared and umx_window_run_fx alone delivers the whole volume. */
enum { UMX_U8OUT = 100 };
typedef struct { int V, P, overlap, nper, npatch; } umx_window;
umx_window umx_window_make(int V, int P, int overlap);
void umx_window_share(const umx_window *w, int rank, int world, int *first, int *count);      /* this rank's patches [first, first + count) in (z, y, x) order */
void umx_window_origin(const umx_window *w, int idx, int *z0, int *y0, int *x0);             /* the last patch of an axis is pulled back so that it ends at the volume's edge */
void umx_window_extent(const umx_window *w, int first, int count, int *zlo, int *zhi);
typedef struct umx_wplan umx_wplan;
umx_wplan *umx_wplan_create(const umx_window *w, int rank, int world, int nh);               /* host only: shares, ownership of the rows, exchange lists (at most 64 ranks) */
void umx_wplan_free(umx_wplan *p);
void umx_wplan_info(const umx_wplan *p, int *first, int *count, int *zlo, int *zhi);
long umx_wplan_rows(const umx_wplan *p, int peer, int dir, int *zy);                        /* rows handed to (dir 0) / received from (dir 1) `peer`; zy: optional, 2 ints a row (z, y), ascending */
void umx_wplan_mode(const umx_wplan *p, uint8_t *mode);                                     /* mode [zhi - zlo][V]: 0 not this rank's patches, 1 this rank's alone (umx_window_run_fx delivers it), 2 this rank's, shared (umx_wplan_finish), 3 a lower rank's */
size_t umx_wplan_row_bytes(const umx_wplan *p);                                             /* bytes of one exchanged row: (nh + 1) x V 64-bit sums */
int umx_wplan_prepare(umx_wplan *p, umx_unet *u, int batch, int out_fmt);                    /* optional: allocate everything a run needs ahead of it */
int umx_window_run_fx(umx_unet *u, umx_wplan *p, const uint8_t *vol_host, int batch, int out_fmt, void *out_host);
int umx_wplan_pack(umx_wplan *p, int peer, void *buf_dev);
int umx_wplan_add(umx_wplan *p, int peer, const void *buf_dev);
int umx_wplan_finish(umx_wplan *p, void *out_host);
/* the device operators underneath (acc [nh][zext][V][V], wsum [zext][V][V] 64-bit sums of an extent of zext planes from plane zlo) */
void umx_blend_add_fx(const float *logits_dev, int nh, int P, int V, int zlo, int zext, int z0, int y0, int x0, const float *w1d_dev, long long *acc_dev, long long *wsum_dev);
void umx_emit_fx(const long long *acc_dev, const long long *wsum_dev, const uint8_t *mode_dev, int want, int nh, int V, int zext, int za, int zb, int ya, int yb, int fmt, void *out_dev);
void umx_emit_rows_fx(const long long *acc_dev, const long long *wsum_dev, const int *zy_dev, long nrows, int nh, int V, int zext, int fmt, void *out_dev);
void umx_rows_fx(long long *acc_dev, long long *wsum_dev, const int *zy_dev, long nrows, int nh, int V, int zext, int dir, long long *buf_dev);

#ifdef __cplusplus
}
#endif
