/* Device-side pieces of the sliding-window path: the CT input conversion and the Gaussian-weighted blend of a patch's logits into
   the rank's accumulators (the role of k_i3_blend, src/nn_ink3dext.cu:58-73, in the reference).  HBM-bound elementwise passes. */
#include "mx_common.cuh"

__global__ void __launch_bounds__(256) u8_to_h16_k(const uint8_t *__restrict__ x, __half *__restrict__ y, size_t n) {
    pdl_trigger(); pdl_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        y[i] = __float2half_rn(__fdiv_rn((float)x[i], 255.f));
}
/* x: uint8 CT values on the device -> fp16 intensity x / 255 (one rounding of the exact quotient) */
extern "C" void umx_u8_to_h16(const uint8_t *x, size_t n, void *y) {
    if (!umx_ready("umx_u8_to_h16")) return;
    size_t g = (n + 255) / 256; if (g > 148u * 16u) g = 148u * 16u; if (!g) g = 1;
    umx_launch(u8_to_h16_k, dim3((unsigned)g), dim3(256), 0, x, (__half *)y, n);
    g_umx_launches++;
    UMX_CK("umx_u8_to_h16");
}
/* one P^3 patch at (z, y, x) of a uint8 volume slab on the device (planes of V x V voxels, z counted from the slab's first plane) -> fp16
   intensities x / 255, the patch contiguous; voxels beyond the volume's y / x extent read as zero.  Eight voxels of a row a thread when
   the rows allow 8-byte loads. */
__global__ void __launch_bounds__(256) gather_u8_h16_k(const uint8_t *__restrict__ vol, int V, int z, int y, int x, int P, __half *__restrict__ out, int vec) {
    pdl_trigger(); pdl_wait();
    const size_t plane = (size_t)V * V;
    if (vec) {
        const int P8 = P / 8; const size_t n8 = (size_t)P * P * P8;
        for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
            const int px = (int)(i % P8) * 8, py = (int)((i / P8) % P), pz = (int)(i / ((size_t)P8 * P));
            uint2 v = make_uint2(0u, 0u);
            if (y + py < V && x + px + 8 <= V) v = __ldg((const uint2 *)(vol + (size_t)(z + pz) * plane + (size_t)(y + py) * V + x + px));
            __half2 h[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const unsigned w = (k < 2 ? v.x : v.y) >> (16 * (k & 1));
                h[k] = __floats2half2_rn(__fdiv_rn((float)(w & 0xffu), 255.f), __fdiv_rn((float)((w >> 8) & 0xffu), 255.f));
            }
            *(uint4 *)(out + ((size_t)pz * P + py) * P + px) = *(const uint4 *)h;
        }
    } else {
        const size_t n = (size_t)P * P * P;
        for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
            const int px = (int)(i % P), py = (int)((i / P) % P), pz = (int)(i / ((size_t)P * P));
            const float v = (y + py < V && x + px < V) ? (float)vol[(size_t)(z + pz) * plane + (size_t)(y + py) * V + x + px] : 0.f;
            out[i] = __float2half_rn(__fdiv_rn(v, 255.f));
        }
    }
}
extern "C" void umx_gather_u8_h16(const uint8_t *vol_dev, int V, int z, int y, int x, int P, void *out) {
    if (!umx_ready("umx_gather_u8_h16")) return;
    const int vec = !((V | P | x) & 7) && x + P <= V && !((size_t)vol_dev & 7) && !((size_t)out & 15);
    size_t g = ((size_t)P * P * P / (vec ? 8 : 1) + 255) / 256; if (g > 148u * 16u) g = 148u * 16u; if (!g) g = 1;
    umx_launch(gather_u8_h16_k, dim3((unsigned)g), dim3(256), 0, vol_dev, V, z, y, x, P, (__half *)out, vec);
    g_umx_launches++;
    UMX_CK("umx_gather_u8_h16");
}
/* fp16 logits -> uint8 round(254 / (1 + exp(-l))): the per-patch form of the reference's probability output (pred_place_k, src/nn_elem.cu:1117-1125,
   rounds 255 p + 0.5 down; the blended path's k_i3_emit uses round(254 p), which is what this library uses throughout) */
__device__ __forceinline__ unsigned prob_u8(float l) { return (unsigned)__float2int_rn(__fmul_rn(__fdiv_rn(1.f, __fadd_rn(1.f, expf(-l))), 254.f)) & 0xffu; }
/* eight values a thread: one 16-byte load, one 8-byte store (x and y 16- and 8-byte aligned); the tail one by one */
__global__ void __launch_bounds__(256) h16_to_prob_u8_k(const __half *__restrict__ x, uint8_t *__restrict__ y, size_t n) {
    pdl_trigger(); pdl_wait();
    const size_t n8 = n / 8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = __ldg((const uint4 *)x + i);
        const __half2 *h = (const __half2 *)&v;
        unsigned w[2] = {0u, 0u};
#pragma unroll
        for (int k = 0; k < 4; k++) { const float2 f = __half22float2(h[k]); w[k >> 1] |= (prob_u8(f.x) | (prob_u8(f.y) << 8)) << (16 * (k & 1)); }
        ((uint2 *)y)[i] = make_uint2(w[0], w[1]);
    }
    for (size_t i = n8 * 8 + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) y[i] = (uint8_t)prob_u8(__half2float(x[i]));
}
__global__ void half_iota_k(unsigned short *h) { h[blockIdx.x * blockDim.x + threadIdx.x] = (unsigned short)(blockIdx.x * blockDim.x + threadIdx.x); }
/* the probability byte of every fp16 bit pattern (65536 bytes, made once per device by the pass itself): what a conv's epilogue looks its
   fp16 logit up in (UMX_OUT_PROB8) */
const uint8_t *umx_prob_table(void) {
    static uint8_t *tab[16];
    int d = 0; if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 16) return nullptr;
    if (tab[d]) return tab[d];
    unsigned short *h = (unsigned short *)nn_malloc(65536 * 2);
    uint8_t *t = (uint8_t *)nn_malloc(65536);
    if (!h || !t) { nn_free(h); nn_free(t); return nullptr; }
    half_iota_k<<<256, 256>>>(h);
    h16_to_prob_u8_k<<<32, 256>>>((const __half *)h, t, 65536);
    g_umx_launches += 2;
    cudaStreamSynchronize(0);
    UMX_CK("umx_prob_table");
    nn_free(h);
    tab[d] = t;
    return t;
}
extern "C" void umx_h16_to_prob_u8(const void *x, size_t n, uint8_t *y) {
    if (!umx_ready("umx_h16_to_prob_u8")) return;
    if (((size_t)x & 15) || ((size_t)y & 7)) { fprintf(stderr, "umx_h16_to_prob_u8: x must be 16-byte and y 8-byte aligned\n"); abort(); }
    size_t g = (n / 8 + 255) / 256; if (g > 148u * 16u) g = 148u * 16u; if (!g) g = 1;
    umx_launch(h16_to_prob_u8_k, dim3((unsigned)g), dim3(256), 0, (const __half *)x, y, n);
    g_umx_launches++;
    UMX_CK("umx_h16_to_prob_u8");
}
/* acc[c][z - zlo][y][x] += w(z) w(y) w(x) logits[c][patch voxel], wsum likewise, for the patch at (z0, y0, x0); one thread per patch
   voxel, channels looped (patches are added one launch at a time, so no two threads touch the same accumulator) */
template <typename T>
__global__ void __launch_bounds__(256) blend_add_k(const T *__restrict__ logits, int nh, int P, int V, int zlo, int zext, int z0, int y0, int x0,
                                                    const float *__restrict__ w1d, float *__restrict__ acc, float *__restrict__ wsum) {
    pdl_trigger(); pdl_wait();
    const size_t PS = (size_t)P * P * P, plane = (size_t)V * V, AS = plane * zext;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < PS; i += (size_t)gridDim.x * blockDim.x) {
        const int x = (int)(i % P), y = (int)((i / P) % P), z = (int)(i / ((size_t)P * P));
        const int gz = z0 + z - zlo, gy = y0 + y, gx = x0 + x;
        if (gz < 0 || gz >= zext || gy >= V || gx >= V) continue;
        const float w = __fmul_rn(__fmul_rn(w1d[z], w1d[y]), w1d[x]);
        const size_t gv = (size_t)gz * plane + (size_t)gy * V + gx;
        for (int c = 0; c < nh; c++) acc[(size_t)c * AS + gv] = __fmaf_rn(w, (float)logits[(size_t)c * PS + i], acc[(size_t)c * AS + gv]);
        wsum[gv] += w;
    }
}
extern "C" void umx_blend_add(const void *logits, int fmt, int nh, int P, int V, int zlo, int zext, int z0, int y0, int x0, const float *w1d, float *acc, float *wsum) {
    if (!umx_ready("umx_blend_add")) return;
    const size_t PS = (size_t)P * P * P; size_t g = (PS + 255) / 256; if (g > 148u * 16u) g = 148u * 16u;
    if (fmt == UMX_F16) umx_launch(blend_add_k<__half>, dim3((unsigned)g), dim3(256), 0, (const __half *)logits, nh, P, V, zlo, zext, z0, y0, x0, w1d, acc, wsum);
    else umx_launch(blend_add_k<float>, dim3((unsigned)g), dim3(256), 0, (const float *)logits, nh, P, V, zlo, zext, z0, y0, x0, w1d, acc, wsum);
    g_umx_launches++;
    UMX_CK("umx_blend_add");
}

/* ---- exact blending.  The reference adds w x logit in fp32 with atomics, in whatever order the threads arrive (k_i3_blend), so its sums change
   from run to run in the last bits.  Here a term is the exact product of the fp32 window weight and the fp32 logit, rounded once to a
   multiple of 2^-46 and added as a 64-bit integer: integer sums do not depend on the order of the patches, on the batch they were
   forwarded in or on which rank forwarded them, so the partial sums of two ranks add up to the single-rank sums bit for bit.
   (|sum| < 2^17; a weight is at least exp(-24) = 2^-34.6, so even the volume's corner voxels keep 11 significant bits of weight.) ---- */
#define UMX_FX_SCALE 70368744177664.0      /* 2^46 */
__global__ void __launch_bounds__(256) blend_fx_k(const float *__restrict__ logits, int nh, int P, int V, int zlo, int zext, int z0, int y0, int x0,
                                                   const float *__restrict__ w1d, long long *__restrict__ acc, long long *__restrict__ wsum) {
    pdl_trigger(); pdl_wait();
    const size_t PS = (size_t)P * P * P, plane = (size_t)V * V, AS = plane * zext;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < PS; i += (size_t)gridDim.x * blockDim.x) {
        const int x = (int)(i % P), y = (int)((i / P) % P), z = (int)(i / ((size_t)P * P));
        const int gz = z0 + z - zlo, gy = y0 + y, gx = x0 + x;
        if (gz < 0 || gz >= zext || gy >= V || gx >= V) continue;
        const double w = (double)__fmul_rn(__fmul_rn(w1d[z], w1d[y]), w1d[x]) * UMX_FX_SCALE;      /* the reference's fp32 weight, scaled */
        const size_t gv = (size_t)gz * plane + (size_t)gy * V + gx;
        for (int c = 0; c < nh; c++) {
            const double t = w * (double)logits[(size_t)c * PS + i];        /* exact: 24 x 24 bits, the scale a power of two */
            acc[(size_t)c * AS + gv] += fabs(t) < 9.0e18 ? __double2ll_rn(t) : 0ll;
        }
        wsum[gv] += __double2ll_rn(w);
    }
}
extern "C" void umx_blend_add_fx(const float *logits, int nh, int P, int V, int zlo, int zext, int z0, int y0, int x0, const float *w1d, long long *acc, long long *wsum) {
    if (!umx_ready("umx_blend_add_fx")) return;
    const size_t PS = (size_t)P * P * P; size_t g = (PS + 255) / 256; if (g > 148u * 16u) g = 148u * 16u;
    umx_launch(blend_fx_k, dim3((unsigned)g), dim3(256), 0, logits, nh, P, V, zlo, zext, z0, y0, x0, w1d, acc, wsum);
    g_umx_launches++;
    UMX_CK("umx_blend_add_fx");
}
/* the blended value of the rows (z, y) with mode[z][y] == want, z in [za, zb) of the accumulators' extent and y in [ya, yb): l = sum / weight (in fp64, rounded to
   fp32), then fmt UMX_F16: the logit as fp16; any other fmt (uint8): round(254 p) with p = 1 / (1 + exp(-l)), 255 where no patch covers the voxel
   (k_i3_emit, src/nn_ink3dext.cu:77-100).  out [nh][zext][V][V]. */
__global__ void __launch_bounds__(256) emit_fx_k(const long long *__restrict__ acc, const long long *__restrict__ wsum, const uint8_t *__restrict__ mode, int want,
                                                  int nh, int V, int zext, int za, int zb, int ya, int yb, int fmt, void *__restrict__ out) {
    pdl_trigger(); pdl_wait();
    const size_t plane = (size_t)V * V, AS = plane * zext, slab = (size_t)(yb - ya) * V, n = (size_t)(zb - za) * slab;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t zz = i / slab, gv = ((size_t)za + zz) * plane + (size_t)ya * V + (i - zz * slab);
        if (mode[gv / V] != want) continue;
        const long long ws = wsum[gv];
        for (int c = 0; c < nh; c++) {
            const size_t o = (size_t)c * AS + gv;
            const float l = ws > 0 ? (float)((double)acc[o] / (double)ws) : 0.f;
            if (fmt == UMX_F16) ((__half *)out)[o] = __float2half_rn(l);
            else ((uint8_t *)out)[o] = ws > 0 ? (uint8_t)__float2int_rn(__fmul_rn(__fdiv_rn(1.f, __fadd_rn(1.f, expf(-l))), 254.f)) : (uint8_t)255;
        }
    }
}
extern "C" void umx_emit_fx(const long long *acc, const long long *wsum, const uint8_t *mode, int want, int nh, int V, int zext, int za, int zb, int ya, int yb, int fmt, void *out) {
    if (!umx_ready("umx_emit_fx") || zb <= za || yb <= ya) return;
    const size_t n = (size_t)(zb - za) * (yb - ya) * V; size_t g = (n + 255) / 256; if (g > 148u * 32u) g = 148u * 32u;
    umx_launch(emit_fx_k, dim3((unsigned)g), dim3(256), 0, acc, wsum, mode, want, nh, V, zext, za, zb, ya, yb, fmt, out);
    g_umx_launches++;
    UMX_CK("umx_emit_fx");
}
/* the same values for a list of rows (z, y), compact: out [row][nh][V] */
__global__ void __launch_bounds__(256) emit_rows_fx_k(const long long *__restrict__ acc, const long long *__restrict__ wsum, const int *__restrict__ zy, long nrows, int nh, int V, int zext, int fmt, void *__restrict__ out) {
    pdl_trigger(); pdl_wait();
    const size_t plane = (size_t)V * V, AS = plane * zext, per = (size_t)nh * V, n = (size_t)nrows * per;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / per, k = i - r * per; const int c = (int)(k / V), x = (int)(k - (size_t)c * V);
        const size_t gv = (size_t)zy[2 * r] * plane + (size_t)zy[2 * r + 1] * V + x;
        const long long ws = wsum[gv];
        const float l = ws > 0 ? (float)((double)acc[(size_t)c * AS + gv] / (double)ws) : 0.f;
        if (fmt == UMX_F16) ((__half *)out)[i] = __float2half_rn(l);
        else ((uint8_t *)out)[i] = ws > 0 ? (uint8_t)__float2int_rn(__fmul_rn(__fdiv_rn(1.f, __fadd_rn(1.f, expf(-l))), 254.f)) : (uint8_t)255;
    }
}
extern "C" void umx_emit_rows_fx(const long long *acc, const long long *wsum, const int *zy_dev, long nrows, int nh, int V, int zext, int fmt, void *out) {
    if (!umx_ready("umx_emit_rows_fx") || nrows <= 0) return;
    const size_t n = (size_t)nrows * nh * V; size_t g = (n + 255) / 256; if (g > 148u * 32u) g = 148u * 32u;
    umx_launch(emit_rows_fx_k, dim3((unsigned)g), dim3(256), 0, acc, wsum, zy_dev, nrows, nh, V, zext, fmt, out);
    g_umx_launches++;
    UMX_CK("umx_emit_rows_fx");
}
/* rows (z, y) of the accumulators to or from a compact buffer buf [row][nh + 1][V] (the weight sum last): dir 0 copies the rows out, dir 1 adds
   the buffer's rows into the accumulators.  zy: device, 2 ints a row, z relative to the accumulators' first plane. */
__global__ void __launch_bounds__(256) rows_fx_k(long long *__restrict__ acc, long long *__restrict__ wsum, const int *__restrict__ zy, long nrows, int nh, int V, int zext, int dir, long long *__restrict__ buf) {
    pdl_trigger(); pdl_wait();
    const size_t plane = (size_t)V * V, AS = plane * zext, per = (size_t)(nh + 1) * V, n = (size_t)nrows * per;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / per, k = i - r * per; const int c = (int)(k / V), x = (int)(k - (size_t)c * V);
        const size_t gv = (size_t)zy[2 * r] * plane + (size_t)zy[2 * r + 1] * V + x;
        long long *cell = c < nh ? acc + (size_t)c * AS + gv : wsum + gv;
        if (dir) *cell += buf[i]; else buf[i] = *cell;
    }
}
extern "C" void umx_rows_fx(long long *acc, long long *wsum, const int *zy_dev, long nrows, int nh, int V, int zext, int dir, long long *buf) {
    if (!umx_ready("umx_rows_fx") || nrows <= 0) return;
    const size_t n = (size_t)nrows * (nh + 1) * V; size_t g = (n + 255) / 256; if (g > 148u * 32u) g = 148u * 32u;
    umx_launch(rows_fx_k, dim3((unsigned)g), dim3(256), 0, acc, wsum, zy_dev, nrows, nh, V, zext, dir, buf);
    g_umx_launches++;
    UMX_CK("umx_rows_fx");
}
extern "C" long umx_launch_count(void) { return g_umx_launches; }
extern "C" int umx_peek_device_error(void) { return umx_errflag_read(); }
