/* InstanceNorm coefficients from the conv epilogue's partial sums, and the fused apply: y = fp16(LeakyReLU(x a + b)) requantised
   to MX for the next conv.  HBM-bound: the apply reads 2 B and writes 1 + 1/32 B (fp8) or 1/2 + 1/32 B (fp4) per element (twice
   that when the space-to-depth copy for a down conv is also written).  Semantics: k_in_coef and k_inq of the reference
   (src/nn_xnet.cu:1565-1570, 1577-1620) with 32-channel UE8M0 blocks. */
#include "mx_common.cuh"

/* partial sums: part[((n * T + t) * Cop + c) * 2 + {0, 1}], T voxel chunks, Cop = C rounded up to 32.  One block per (c, n); the
   chunk sums are added in a fixed order (strided per thread, then a fixed tree), so the result does not depend on scheduling. */
__global__ void __launch_bounds__(256) in_coef_k(const double *__restrict__ part, int C, int Cop, int T, double S, const float *gamma, const float *beta, float eps, float *coef) {
    const int c = blockIdx.x, n = blockIdx.y;
    double s = 0.0, q = 0.0;
    for (int t = threadIdx.x; t < T; t += 256) { const double *p = part + (((size_t)n * T + t) * Cop + c) * 2; s += p[0]; q += p[1]; }
    __shared__ double ss[256], sq[256];
    ss[threadIdx.x] = s; sq[threadIdx.x] = q;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) { if ((int)threadIdx.x < o) { ss[threadIdx.x] += ss[threadIdx.x + o]; sq[threadIdx.x] += sq[threadIdx.x + o]; } __syncthreads(); }
    if (threadIdx.x == 0) {
        const double m = ss[0] / S, v = fmax(sq[0] / S - m * m, 0.0);
        const float rs = (float)(1.0 / sqrt(v + (double)eps)), a = __fmul_rn(rs, gamma ? gamma[c] : 1.f);
        coef[2 * ((size_t)n * C + c)] = a;
        coef[2 * ((size_t)n * C + c) + 1] = __fmaf_rn(-(float)m, a, beta ? beta[c] : 0.f);
    }
}
/* voxel chunks per (sample, channel) of the partial sums: about 2048 voxels each, at most 512 */
int umx_stats_chunks(int D, int H, int W) { const size_t S = (size_t)D * H * W; const size_t t = S / 2048; return t < 1 ? 1 : t > 512 ? 512 : (int)t; }

/* partial sums of chunk t of block blk of sample n of a blocked fp16 tensor: part[((n * T + t) * Cop + c) * 2 + {0, 1}].  A thread owns
   one channel and every eighth voxel of the chunk (a warp reads one voxel's 64-byte row); the eight phases are added in a fixed order.
   HBM-bound: reads 2 B per element. */
__global__ void __launch_bounds__(256) in_part_k(const __half *__restrict__ y, size_t S, int T, double *__restrict__ part) {
    const int t = blockIdx.x, blk = blockIdx.y, n = blockIdx.z, nb = gridDim.y, Cop = nb * 32;
    const int c = threadIdx.x & 31, ph = threadIdx.x >> 5;
    const size_t v0 = S * t / T, v1 = S * (t + 1) / T;
    const __half *p = y + ((size_t)n * nb + blk) * S * 32 + c;
    double s = 0.0, q = 0.0;
    size_t v = v0 + ph;
    for (; v + 24 < v1; v += 32) {   /* four loads in flight */
        const float x0 = __half2float(p[v * 32]), x1 = __half2float(p[(v + 8) * 32]), x2 = __half2float(p[(v + 16) * 32]), x3 = __half2float(p[(v + 24) * 32]);
        s += (double)x0; q += (double)x0 * x0; s += (double)x1; q += (double)x1 * x1; s += (double)x2; q += (double)x2 * x2; s += (double)x3; q += (double)x3 * x3;
    }
    for (; v < v1; v += 8) { const double x = (double)__half2float(p[v * 32]); s += x; q += x * x; }
    __shared__ double ss[8][32], sq[8][32];
    ss[ph][c] = s; sq[ph][c] = q;
    __syncthreads();
    if (ph == 0) {
        for (int k = 1; k < 8; k++) { s += ss[k][c]; q += sq[k][c]; }
        double *d = part + (((size_t)n * T + t) * Cop + blk * 32 + c) * 2;
        d[0] = s; d[1] = q;
    }
}
/* InstanceNorm partial sums of a stored blocked-fp16 conv output (what umx_conv_fwd runs after the conv when it is given `part`) */
void umx_in_part(const void *y, int N, int C, int D, int H, int W, double *part) {
    if (!umx_ready("umx_in_part")) return;
    const int T = umx_stats_chunks(D, H, W);
    in_part_k<<<dim3(T, (C + 31) / 32, N), 256>>>((const __half *)y, (size_t)D * H * W, T, part);
    g_umx_launches++;
    UMX_CK("umx_in_part");
}
extern "C" void umx_in_coef(const double *part, int N, int C, int D, int H, int W, const float *gamma, const float *beta, float eps, float *coef) {
    if (!umx_ready("umx_in_coef")) return;
    const int T = umx_stats_chunks(D, H, W), Cop = (C + 31) / 32 * 32;
    in_coef_k<<<dim3(C, N), 256>>>(part, C, Cop, T, (double)D * H * W, gamma, beta, eps, coef);
    g_umx_launches++;
    UMX_CK("umx_in_coef");
}

template <int BITS>
__global__ void __launch_bounds__(256) in_apply_k(const uint4 *__restrict__ x, const float2 *__restrict__ coef, int N, int C, int D, int H, int W, int act,
                                                  uint8_t *__restrict__ q, int nb_dst, int b0, uint8_t *__restrict__ q2, uint4 *__restrict__ hout, int split) {
    const int nb = (C + 31) / 32; const size_t S = (size_t)D * H * W, rows = (size_t)N * nb * S;
    constexpr int RB = 32 * BITS / 8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < rows; i += (size_t)gridDim.x * blockDim.x) {
        const size_t v = i % S; const int blk = (int)((i / S) % nb), n = (int)(i / (S * nb));
        uint4 raw[4];
#pragma unroll
        for (int j = 0; j < 4; j++) raw[j] = __ldg(x + i * 4 + j);
        const __half2 *hp = (const __half2 *)raw;
        float f[32];
#pragma unroll
        for (int k = 0; k < 16; k++) { const float2 t = __half22float2(hp[k]); f[2 * k] = t.x; f[2 * k + 1] = t.y; }
#pragma unroll
        for (int k = 0; k < 32; k++) {
            const int c = blk * 32 + k;
            float g = 0.f;
            if (c < C) {
                g = f[k];
                if (coef) { const float2 ab = __ldg(coef + (size_t)n * C + c); g = __fmaf_rn(g, ab.x, ab.y); }
                if (act == 2) g = g < 0.f ? __fmul_rn(0.01f, g) : g;
                g = __half2float(__float2half_rn(g));
            }
            f[k] = g;
        }
        if (hout) {
            uint4 o[4]; __half2 *op = (__half2 *)o;
#pragma unroll
            for (int k = 0; k < 16; k++) op[k] = __floats2half2_rn(f[2 * k], f[2 * k + 1]);
#pragma unroll
            for (int j = 0; j < 4; j++) hout[i * 4 + j] = o[j];
        }
        unsigned w[8];
        const unsigned sb = mx_encode_row32<BITS>(f, w);
        if (q) {
            const size_t ro = ((size_t)n * nb_dst + b0 + blk) * S + v;
            if (BITS == 8 && split) {
                const size_t hp = ((size_t)n * nb_dst + b0 + blk) * 2;
                *(uint4 *)(q + (hp * S + v) * 16) = make_uint4(w[0], w[1], w[2], w[3]); *(uint4 *)(q + ((hp + 1) * S + v) * 16) = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
                uint8_t *p = q + ro * RB;
                ((uint4 *)p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                if (BITS == 8) ((uint4 *)p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
            q[(size_t)N * nb_dst * S * RB + ro] = (uint8_t)sb;
        }
        if (q2) {   /* space-to-depth copy: block (tap * nb + blk) at the coarse voxel */
            const int xx = (int)(v % W), yy = (int)((v / W) % H), zz = (int)(v / ((size_t)W * H));
            const int tap = ((zz & 1) * 2 + (yy & 1)) * 2 + (xx & 1);
            const size_t Sc = S / 8, vc = ((size_t)(zz >> 1) * (H >> 1) + (yy >> 1)) * (W >> 1) + (xx >> 1);
            const size_t ro = ((size_t)n * 8 * nb + tap * nb + blk) * Sc + vc;
            if (BITS == 8 && split) {
                const size_t hp = ((size_t)n * 8 * nb + tap * nb + blk) * 2;
                *(uint4 *)(q2 + (hp * Sc + vc) * 16) = make_uint4(w[0], w[1], w[2], w[3]); *(uint4 *)(q2 + ((hp + 1) * Sc + vc) * 16) = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
                uint8_t *p = q2 + ro * RB;
                ((uint4 *)p)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                if (BITS == 8) ((uint4 *)p)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
            q2[(size_t)N * 8 * nb * Sc * RB + ro] = (uint8_t)sb;
        }
    }
}
extern "C" void umx_in_apply(const void *x, const float *coef, int N, int C, int D, int H, int W, int act, void *q, int bits, int nb_dst, int b0, void *q_s2d, void *h, int layout) {
    if (!umx_ready("umx_in_apply")) return;
    if (q_s2d && ((D | H | W) & 1)) { fprintf(stderr, "umx_in_apply: the space-to-depth copy needs even D, H, W\n"); abort(); }
    const int nb = (C + 31) / 32; if (!nb_dst) { nb_dst = nb; b0 = 0; }
    const size_t rows = (size_t)N * nb * D * H * W; size_t g = (rows + 255) / 256; if (g > 148u * 32u) g = 148u * 32u; if (!g) g = 1;
    if (bits == 8) in_apply_k<8><<<(unsigned)g, 256>>>((const uint4 *)x, (const float2 *)coef, N, C, D, H, W, act, (uint8_t *)q, nb_dst, b0, (uint8_t *)q_s2d, (uint4 *)h, layout == UMX_LAYOUT_SPLIT);
    else in_apply_k<4><<<(unsigned)g, 256>>>((const uint4 *)x, (const float2 *)coef, N, C, D, H, W, act, (uint8_t *)q, nb_dst, b0, (uint8_t *)q_s2d, (uint4 *)h, layout == UMX_LAYOUT_SPLIT);
    g_umx_launches++;
    UMX_CK("umx_in_apply");
}
