/* MX quantiser and inverse: plane-major fp32 / fp16 <-> channel-blocked MX-fp8 / MX-fp4 tensors.

   HBM-bound passes.  A thread owns one (n, block, voxel) row, so the amax that defines the row's scale is local: consecutive
   lanes own consecutive voxels, every channel plane is read in full sectors (32 lanes x 2 or 4 bytes), and a warp writes one
   contiguous run of rows (32 x 32 B or 32 x 16 B) plus 32 contiguous scale bytes.  Algorithmic bytes per element: read 4 or 2,
   write 1 + 1/32 (fp8) or 1/2 + 1/32 (fp4).  Semantics: src/lp_mx_cvt.cu:9-19, src/lp_mxops.cuh:46-68 of the reference. */
#include "mx_common.cuh"
#include <cuda_bf16.h>

__host__ __device__ static inline int mxbw(int C, int force) { return force > 0 ? force : C <= 8 ? 8 : C <= 16 ? 16 : 32; }

template <typename T> __device__ __forceinline__ float ld_as_f32(const T *p);
template <> __device__ __forceinline__ float ld_as_f32<float>(const float *p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld_as_f32<__half>(const __half *p) { return __half2float(__ldg(p)); }
template <> __device__ __forceinline__ float ld_as_f32<__nv_bfloat16>(const __nv_bfloat16 *p) { return __uint_as_float((unsigned)__ldg((const unsigned short *)p) << 16); }

/* grid = (voxel chunks, blocks, samples): no index division per row; consecutive threads take consecutive voxels, so the plane-major
   reads and the row writes are both coalesced.  Channels from c2 on come from a second tensor x2 of C - c2 channels (a conv's concat
   input, split_t.x2 / c_split of the reference: the 32-channel blocks run over the concatenated index); c2 = C without one. */
template <int BITS, typename TI, bool CAT>
__global__ void __launch_bounds__(256) pm_to_mx_k(const TI *__restrict__ x, uint8_t *__restrict__ y, int N, int C, size_t S, int bw, int split, const TI *__restrict__ x2, int c2) {
    pdl_trigger(); pdl_wait();
    const int nb = gridDim.y, blk = blockIdx.y, n = blockIdx.z, rb = bw * BITS / 8;
    const size_t rows = (size_t)N * nb * S, row0 = ((size_t)n * nb + blk) * S;
    uint8_t *sc = y + rows * rb;
    const TI *xb = x + ((size_t)n * c2 + (size_t)blk * bw) * S;                       /* channel k of the block: xb + k S while blk bw + k < c2 */
    const TI *xb2 = CAT ? x2 + ((ptrdiff_t)n * (C - c2) + (ptrdiff_t)blk * bw - c2) * (ptrdiff_t)S : nullptr;   /* and xb2 + k S from there on */
    const int nch = min(bw, C - blk * bw), k2 = c2 - blk * bw;
    for (size_t v = blockIdx.x * (size_t)blockDim.x + threadIdx.x; v < S; v += (size_t)gridDim.x * blockDim.x) {
        const size_t i = row0 + v;
        unsigned w[8]; unsigned sb;
        if (nch == 1) {
            /* a block with one real channel (a one-channel stem): the same bytes as the general path, without the 31 zero lanes */
            const float x0 = ld_as_f32((!CAT || 0 < k2 ? xb : xb2) + v);
            const int e = mx_exp(__uint_as_float(__float_as_uint(x0) & 0x7fffffffu), BITS == 4 ? 1.f / 6.f : 1.f / 448.f);
            const float m = exp2i(-e);
            sb = (unsigned)(e + 127) & 0xffu;
            const float z = 0.f * m;                     /* 0, or NaN for an inf / NaN block (scale byte 0xFF), as the general path gives */
            const unsigned zc = BITS == 8 ? cvt_e4m3x4(z, z, z, z) : cvt_e2m1x8((const float[8]){z, z, z, z, z, z, z, z}, 1.f);
#pragma unroll
            for (int k = 1; k < 8; k++) w[k] = zc;
            w[0] = BITS == 8 ? cvt_e4m3x4(x0 * m, z, z, z) : ((zc & ~0xfu) | (cvt_e2m1x2(x0 * m, z) & 0xfu));
        } else {
            float r[32];
#pragma unroll
            for (int k = 0; k < 32; k++) {
                if (CAT) r[k] = k < nch ? ld_as_f32((k < k2 ? xb : xb2) + (ptrdiff_t)k * (ptrdiff_t)S + v) : 0.f;
                else r[k] = k < nch ? ld_as_f32(xb + (size_t)k * S + v) : 0.f;
            }
            sb = mx_encode_row32<BITS>(r, w);
        }
        uint8_t *p = y + i * rb;
        if (BITS == 8) {
            if (bw == 32 && split) {   /* two 16-byte planes per block: [n][blk][half][voxel][16 B] */
                const size_t hp = ((size_t)n * nb + blk) * 2;
                *(uint4 *)(y + (hp * S + v) * 16) = make_uint4(w[0], w[1], w[2], w[3]); *(uint4 *)(y + ((hp + 1) * S + v) * 16) = make_uint4(w[4], w[5], w[6], w[7]);
            } else if (bw == 32) { ((uint4 *)p)[0] = make_uint4(w[0], w[1], w[2], w[3]); ((uint4 *)p)[1] = make_uint4(w[4], w[5], w[6], w[7]); }
            else if (bw == 16) ((uint4 *)p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            else ((uint2 *)p)[0] = make_uint2(w[0], w[1]);
        } else {
            if (bw == 32) ((uint4 *)p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            else if (bw == 16) ((uint2 *)p)[0] = make_uint2(w[0], w[1]);
            else ((unsigned *)p)[0] = w[0];
        }
        sc[i] = (uint8_t)sb;
    }
}
template <int BITS>
__global__ void __launch_bounds__(256) mx_to_pm_k(const uint8_t *__restrict__ x, float *__restrict__ y, int N, int C, size_t S, int bw, int split) {
    const int nb = (C + bw - 1) / bw, rb = bw * BITS / 8;
    const size_t rows = (size_t)N * nb * S;
    const uint8_t *sc = x + rows * rb;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows; i += (size_t)gridDim.x * blockDim.x) {
        const size_t v = i % S; const int blk = (int)((i / S) % nb), n = (int)(i / (S * nb));
        const float s = mx_scale(sc[i]);
        const uint8_t *p = x + i * rb;
        for (int k = 0; k < bw; k++) {
            const int c = blk * bw + k; if (c >= C) break;
            const float e = BITS == 8 ? dec_e4m3(split ? x[(((i / S) * 2 + (k >> 4)) * S + v) * 16 + (k & 15)] : p[k]) : dec_e2m1((p[k >> 1] >> ((k & 1) * 4)) & 15u);
            y[((size_t)n * C + c) * S + v] = e * s;
        }
    }
}
__global__ void __launch_bounds__(256) h16b_to_pm_k(const __half *__restrict__ x, float *__restrict__ y, int N, int C, size_t S) {
    const int nb = (C + 31) / 32;
    const size_t rows = (size_t)N * nb * S;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows; i += (size_t)gridDim.x * blockDim.x) {
        const size_t v = i % S; const int blk = (int)((i / S) % nb), n = (int)(i / (S * nb));
        for (int k = 0; k < 32; k++) { const int c = blk * 32 + k; if (c >= C) break; y[((size_t)n * C + c) * S + v] = __half2float(x[i * 32 + k]); }
    }
}

static unsigned grid_for(size_t rows) { size_t g = (rows + 255) / 256; return (unsigned)(g > 148u * 64u ? 148u * 64u : g ? g : 1); }

static void to_mx(const void *x, int dt, int N, int C, size_t S, void *y, int bits, int bwf, const char *who, int split = 0, const void *x2 = nullptr, int c2 = 0) {
    if (!umx_ready(who)) return;
    if (dt != 0 && dt != 1 && dt != 2) { fprintf(stderr, "%s: source type %d is not built (fp32, bf16 and fp16 only)\n", who, dt); abort(); }
    if (!x2) c2 = C;
    const int bw = mxbw(C, bwf);
    const int nb = (C + bw - 1) / bw;
    if (!S || !N) return;
    /* blocks per (block, sample): 16 per multiprocessor; a tensor of one channel (2 bytes read per 33 written: the network input) runs a
       third faster with two (measured: 31 against 42 us for 128^3) */
    const size_t cap = C == 1 ? 148u * 2u : 148u * 16u;
    size_t gx = (S + 255) / 256; if (gx > cap) gx = cap;
    const dim3 g((unsigned)gx, (unsigned)nb, (unsigned)N);
#define UMX_Q(B, T) do { if (x2) umx_launch(pm_to_mx_k<B, T, true>, g, dim3(256), 0, (const T *)x, (uint8_t *)y, N, C, S, bw, split, (const T *)x2, c2); \
                         else umx_launch(pm_to_mx_k<B, T, false>, g, dim3(256), 0, (const T *)x, (uint8_t *)y, N, C, S, bw, split, (const T *)x2, c2); } while (0)
    if (bits == 8) { if (dt == 2) UMX_Q(8, __half); else if (dt == 1) UMX_Q(8, __nv_bfloat16); else UMX_Q(8, float); }
    else { if (dt == 2) UMX_Q(4, __half); else if (dt == 1) UMX_Q(4, __nv_bfloat16); else UMX_Q(4, float); }
#undef UMX_Q
    g_umx_launches++;
    UMX_CK(who);
}
static void from_mx(const void *x, int N, int C, size_t S, float *y, int bits, int bwf, const char *who, int split = 0) {
    if (!umx_ready(who)) return;
    const int bw = mxbw(C, bwf);
    const size_t rows = (size_t)N * ((C + bw - 1) / bw) * S;
    if (bits == 8) mx_to_pm_k<8><<<grid_for(rows), 256>>>((const uint8_t *)x, y, N, C, S, bw, split);
    else mx_to_pm_k<4><<<grid_for(rows), 256>>>((const uint8_t *)x, y, N, C, S, bw, split);
    g_umx_launches++;
    UMX_CK(who);
}
extern "C" size_t lp_mx8_bytes(int N, int C, size_t S) { const int bw = mxbw(C, 0); return (size_t)N * ((C + bw - 1) / bw) * S * (bw + 1); }
extern "C" size_t lp_mx4_bytes(int N, int C, size_t S) { const int bw = mxbw(C, 0); return (size_t)N * ((C + bw - 1) / bw) * S * (bw / 2 + 1); }
extern "C" size_t umx_mx_bytes32(int bits, int N, int C, size_t S) { return (size_t)N * ((C + 31) / 32) * S * (32 * bits / 8 + 1); }
extern "C" void lp_f32_to_mx8(const float *x, int N, int C, size_t S, void *y) { to_mx(x, 0, N, C, S, y, 8, 0, "lp_f32_to_mx8"); }
extern "C" void lp_f32_to_mx4(const float *x, int N, int C, size_t S, void *y) { to_mx(x, 0, N, C, S, y, 4, 0, "lp_f32_to_mx4"); }
extern "C" void lp_h16_to_mx8(const void *x, int dt, int N, int C, size_t S, void *y) { to_mx(x, dt, N, C, S, y, 8, 0, "lp_h16_to_mx8"); }
extern "C" void lp_h16_to_mx4(const void *x, int dt, int N, int C, size_t S, void *y) { to_mx(x, dt, N, C, S, y, 4, 0, "lp_h16_to_mx4"); }
extern "C" void lp_mx8_to_f32(const void *x, int N, int C, size_t S, float *y) { from_mx(x, N, C, S, y, 8, 0, "lp_mx8_to_f32"); }
extern "C" void lp_mx4_to_f32(const void *x, int N, int C, size_t S, float *y) { from_mx(x, N, C, S, y, 4, 0, "lp_mx4_to_f32"); }
extern "C" void umx_pm_to_mx32(const void *x, int dt, int N, int C, size_t S, void *y, int bits, int layout) { to_mx(x, dt, N, C, S, y, bits, 32, "umx_pm_to_mx32", layout == UMX_LAYOUT_SPLIT && bits == 8); }
/* the same from two tensors: channels [0, c2) of the C from x, the rest from x2 */
extern "C" void umx_pm_to_mx32_cat(const void *x, const void *x2, int c2, int dt, int N, int C, size_t S, void *y, int bits, int layout) {
    if (x2 && (c2 < 1 || c2 >= C)) { fprintf(stderr, "umx_pm_to_mx32_cat: split at channel %d of %d\n", c2, C); abort(); }
    to_mx(x, dt, N, C, S, y, bits, 32, "umx_pm_to_mx32_cat", layout == UMX_LAYOUT_SPLIT && bits == 8, x2, c2);
}
extern "C" void umx_mx32_to_f32(const void *x, int bits, int N, int C, size_t S, float *y, int layout) { from_mx(x, N, C, S, y, bits, 32, "umx_mx32_to_f32", layout == UMX_LAYOUT_SPLIT && bits == 8); }
extern "C" void umx_h16b_to_f32(const void *x, int N, int C, size_t S, float *y) {
    if (!umx_ready("umx_h16b_to_f32")) return;
    h16b_to_pm_k<<<grid_for((size_t)N * ((C + 31) / 32) * S), 256>>>((const __half *)x, y, N, C, S);
    g_umx_launches++;
    UMX_CK("umx_h16b_to_f32");
}

/* MX-fp8 codes between the reference layout [n][blk][voxel][32 B] and the split layout [n][blk][half][voxel][16 B]; the scale plane is
   copied as it is.  One thread per 16-byte half row. */
__global__ void __launch_bounds__(256) relayout8_k(const uint4 *__restrict__ src, uint4 *__restrict__ dst, size_t rows, size_t S, int to_split) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows * 2; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i >> 1, h = i & 1, sp = ((r / S) * 2 + h) * S + r % S;       /* reference index i = 2 r + h; split index sp */
        if (to_split) dst[sp] = __ldg(src + i); else dst[i] = __ldg(src + sp);
    }
}
extern "C" void umx_mx_relayout(const void *src, int bits, int N, int C, size_t S, void *dst, int to_layout) {
    if (!umx_ready("umx_mx_relayout")) return;
    const size_t rows = (size_t)N * ((C + 31) / 32) * S, rb = bits == 8 ? 32 : 16;
    if (bits == 8) { relayout8_k<<<grid_for(rows * 2), 256>>>((const uint4 *)src, (uint4 *)dst, rows, S, to_layout == UMX_LAYOUT_SPLIT); g_umx_launches++; }
    else cudaMemcpyAsync(dst, src, rows * rb, cudaMemcpyDeviceToDevice, 0);
    cudaMemcpyAsync((uint8_t *)dst + rows * rb, (const uint8_t *)src + rows * rb, rows, cudaMemcpyDeviceToDevice, 0);
    UMX_CK("umx_mx_relayout");
}

/* MX tensors of 16 channels or fewer keep rows of 8 or 16 channels in the reference's storage (src/lp_common.cuh:132-134).  Such a row
   and the 32-wide row holding the same channels followed by zeros have the same amax, hence the same scale byte and the same codes:
   widening and narrowing are copies.  One thread per row. */
__global__ void __launch_bounds__(256) mx_rewidth_k(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, size_t rows, int rb_src, int rb_dst) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned *s = (const unsigned *)(src + i * rb_src); unsigned *d = (unsigned *)(dst + i * rb_dst);
        for (int k = 0; k < rb_dst / 4; k++) d[k] = k < rb_src / 4 ? __ldg(s + k) : 0u;
        dst[rows * rb_dst + i] = __ldg(src + rows * rb_src + i);
    }
}
/* x: an MX tensor of C <= 16 channels (one block of 8 or 16 a voxel) -> y: the same tensor with 32-wide rows (to_wide), or back */
extern "C" void umx_mx_rewidth(const void *x, int bits, int N, int C, size_t S, void *y, int to_wide) {
    if (!umx_ready("umx_mx_rewidth")) return;
    if (C < 1 || C > 16 || (bits != 8 && bits != 4)) { fprintf(stderr, "umx_mx_rewidth: %d channels, %d bits\n", C, bits); abort(); }
    const int bw = mxbw(C, 0), rn = bw * bits / 8, r32 = 32 * bits / 8;
    const size_t rows = (size_t)N * S;
    if (!rows) return;
    mx_rewidth_k<<<grid_for(rows), 256>>>((const uint8_t *)x, (uint8_t *)y, rows, to_wide ? rn : r32, to_wide ? r32 : rn);
    g_umx_launches++;
    UMX_CK("umx_mx_rewidth");
}

/* lp_pred_input_mx (src/nn_lp.h:164-165, src/lp_mx_cvt.cu:20-57): the network input of the reference's predict for window planes
   [z0, z0 + nz) of a W x W x depth CT window: channel 0 the z-scored CT byte, 1 zero, 2 and 3 the unit direction away from the scroll
   axis (dy, dx) (axis 0: zeros; -1 flips it), each rounded to the 16-bit input type (hd 2 fp16, 1 bf16, 0 none), stored as MX rows of
   one 8-channel block.  The radius is sqrt(fma(dy, dy, dx dx)) + 1e-6: the contraction a compiler picks for dy dy + dx dx, spelled out. */
template <int HD> __device__ __forceinline__ float round16(float v) {
    if (HD == 2) return __half2float(__float2half_rn(v));
    if (HD == 1) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}
template <int BITS, int HD>
__global__ void __launch_bounds__(256) pred_input_k(const uint8_t *__restrict__ ct, int W, float mean, float isd, const float *__restrict__ dyo, const float *__restrict__ dxo,
                                                    int axis, int z0, int nz, uint8_t *__restrict__ y) {
    const size_t S = (size_t)nz * W * W, i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= S) return;
    const int xx = (int)(i % W), yy = (int)((i / W) % W), z = z0 + (int)(i / ((size_t)W * W));
    const float dy = __fadd_rn(__ldg(dyo + z), (float)yy), dx = __fadd_rn(__ldg(dxo + z), (float)xx);
    const float inv = axis ? __fdiv_rn((float)axis, __fadd_rn(__fsqrt_rn(__fmaf_rn(dy, dy, __fmul_rn(dx, dx))), 1e-6f)) : 0.f;
    float r[32];
#pragma unroll
    for (int k = 0; k < 32; k++) r[k] = 0.f;
    r[0] = round16<HD>(__fmul_rn(__fsub_rn((float)__ldg(ct + (size_t)z * W * W + (size_t)yy * W + xx), mean), isd));
    r[2] = round16<HD>(__fmul_rn(dy, inv)); r[3] = round16<HD>(__fmul_rn(dx, inv));
    unsigned w[8];
    const unsigned sb = mx_encode_row32<BITS>(r, w);        /* channels 4..31 are zeros: the row's first 8 codes are the 8-wide row's */
    if (BITS == 8) *(uint2 *)(y + i * 8) = make_uint2(w[0], w[1]); else *(unsigned *)(y + i * 4) = w[0];
    y[S * (BITS == 8 ? 8 : 4) + i] = (uint8_t)sb;
}
extern "C" void lp_pred_input_mx(const uint8_t *ct, int W, float mean, float isd, const float *dyo, const float *dxo, int axis, int z0, int nz, void *y, int hd, int bits) {
    if (!umx_ready("lp_pred_input_mx")) return;
    if ((bits != 8 && bits != 4) || hd < 0 || hd > 2) { fprintf(stderr, "lp_pred_input_mx: %d bits, 16-bit type %d\n", bits, hd); abort(); }
    const size_t S = (size_t)(nz > 0 ? nz : 0) * W * W;
    if (!S) return;
    const unsigned g = (unsigned)((S + 255) / 256);
#define UMX_PI(B, H) pred_input_k<B, H><<<g, 256>>>(ct, W, mean, isd, dyo, dxo, axis, z0, nz, (uint8_t *)y)
    if (bits == 8) { if (hd == 2) UMX_PI(8, 2); else if (hd == 1) UMX_PI(8, 1); else UMX_PI(8, 0); }
    else { if (hd == 2) UMX_PI(4, 2); else if (hd == 1) UMX_PI(4, 1); else UMX_PI(4, 0); }
#undef UMX_PI
    g_umx_launches++;
    UMX_CK("lp_pred_input_mx");
}
extern "C" void lp_pred_input_mx8(const uint8_t *ct, int W, float mean, float isd, const float *dyo, const float *dxo, int axis, int z0, int nz, void *y, int hd) {
    lp_pred_input_mx(ct, W, mean, isd, dyo, dxo, axis, z0, nz, y, hd, 8);
}
