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
extern "C" void umx_in_coef(const double *part, int N, int C, int D, int H, int W, const float *gamma, const float *beta, float eps, float *coef);
/* voxel chunks per (sample, channel) of the partial sums: about 1024 voxels each, at most 512 */
int umx_stats_chunks(int D, int H, int W) { const size_t S = (size_t)D * H * W; const size_t t = S / 1024; return t < 1 ? 1 : t > 512 ? 512 : (int)t; }

/* partial sums of chunk t of block blk of sample n of a blocked fp16 tensor: part[((n * T + t) * Cop + c) * 2 + {0, 1}].  A thread owns
   eight channels (one 16-byte load) of every 64th voxel of the chunk, four loads in flight, so a warp reads 512 contiguous bytes per
   load; the 64 phases are added in a fixed order.  fp64 throughout: sums of fp16 values and of their squares are then exact to the
   last bits whatever the order.  HBM-bound: reads 2 B per element. */
/* tickets of the fused finalise: one counter per (sample, block); the block that draws the last ticket finalises and resets it */
__device__ unsigned g_stat_tickets[8192];

template <bool FINAL>
__global__ void __launch_bounds__(256) in_part_k(const uint4 *__restrict__ y, size_t S, int T, double *__restrict__ part,
                                                 int C, const float *gamma, const float *beta, float eps, float *coef) {
    pdl_trigger(); pdl_wait();
    const int t = blockIdx.x, blk = blockIdx.y, n = blockIdx.z, nb = gridDim.y, Cop = nb * 32;
    const int qd = threadIdx.x & 3, ph = threadIdx.x >> 2;
    const size_t v0 = S * t / T, v1 = S * (t + 1) / T;
    const uint4 *p = y + ((size_t)n * nb + blk) * S * 4 + qd;
    double s[8], q[8];
#pragma unroll
    for (int k = 0; k < 8; k++) { s[k] = 0.0; q[k] = 0.0; }
    auto add = [&](const uint4 &r) {
        const __half2 *h = (const __half2 *)&r;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 f = __half22float2(h[k]);
            const double a = (double)f.x, b = (double)f.y;
            s[2 * k] += a; q[2 * k] = fma(a, a, q[2 * k]); s[2 * k + 1] += b; q[2 * k + 1] = fma(b, b, q[2 * k + 1]);
        }
    };
    size_t v = v0 + ph;
    for (; v + 448 < v1; v += 512) {      /* eight loads in flight */
        const uint4 r0 = __ldg(p + v * 4), r1 = __ldg(p + (v + 64) * 4), r2 = __ldg(p + (v + 128) * 4), r3 = __ldg(p + (v + 192) * 4);
        const uint4 r4 = __ldg(p + (v + 256) * 4), r5 = __ldg(p + (v + 320) * 4), r6 = __ldg(p + (v + 384) * 4), r7 = __ldg(p + (v + 448) * 4);
        add(r0); add(r1); add(r2); add(r3); add(r4); add(r5); add(r6); add(r7);
    }
    for (; v + 192 < v1; v += 256) {
        const uint4 r0 = __ldg(p + v * 4), r1 = __ldg(p + (v + 64) * 4), r2 = __ldg(p + (v + 128) * 4), r3 = __ldg(p + (v + 192) * 4);
        add(r0); add(r1); add(r2); add(r3);
    }
    for (; v < v1; v += 64) { const uint4 r0 = __ldg(p + v * 4); add(r0); }
    __shared__ double ss[64][33], sq[64][33];
#pragma unroll
    for (int k = 0; k < 8; k++) { ss[ph][qd * 8 + k] = s[k]; sq[ph][qd * 8 + k] = q[k]; }
    __syncthreads();
    if (threadIdx.x < 64) {
        const int c = threadIdx.x & 31; double (*src)[33] = threadIdx.x < 32 ? ss : sq;
        double acc = 0.0;
        for (int k = 0; k < 64; k++) acc += src[k][c];
        part[(((size_t)n * T + t) * Cop + blk * 32 + c) * 2 + (threadIdx.x >> 5)] = acc;
    }
    if (!FINAL) return;
    /* the last block of this (sample, block) to finish turns the partial sums into coefficients: eight threads a channel add
       every eighth chunk, then the eight in order; the result does not depend on which block came last */
    __shared__ unsigned last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) { const unsigned tk = atomicAdd(&g_stat_tickets[n * nb + blk], 1u); last = tk == (unsigned)T - 1u; if (last) g_stat_tickets[n * nb + blk] = 0u; }
    __syncthreads();
    if (!last) return;
    __threadfence();
    {
        const int c = threadIdx.x & 31, g8 = threadIdx.x >> 5;
        double a0 = 0.0, a1 = 0.0;
        const double2 *pb = (const double2 *)part + ((size_t)n * T) * Cop + blk * 32 + c;
        int k = g8;
        for (; k + 24 < T; k += 32) {      /* four loads in flight; the order of the additions is fixed */
            const double2 p0 = __ldcg(pb + (size_t)k * Cop), p1 = __ldcg(pb + (size_t)(k + 8) * Cop), p2 = __ldcg(pb + (size_t)(k + 16) * Cop), p3 = __ldcg(pb + (size_t)(k + 24) * Cop);
            a0 += p0.x; a1 += p0.y; a0 += p1.x; a1 += p1.y; a0 += p2.x; a1 += p2.y; a0 += p3.x; a1 += p3.y;
        }
        for (; k < T; k += 8) { const double2 p0 = __ldcg(pb + (size_t)k * Cop); a0 += p0.x; a1 += p0.y; }
        ss[g8][c] = a0; sq[g8][c] = a1;
        __syncthreads();
        if (g8 == 0 && blk * 32 + c < C) {
            for (int k = 1; k < 8; k++) { a0 += ss[k][c]; a1 += sq[k][c]; }
            const int ch = blk * 32 + c;
            const double m = a0 / (double)S, v = fmax(a1 / (double)S - m * m, 0.0);
            const float rs = (float)(1.0 / sqrt(v + (double)eps)), ca = __fmul_rn(rs, gamma ? gamma[ch] : 1.f);
            coef[2 * ((size_t)n * C + ch)] = ca;
            coef[2 * ((size_t)n * C + ch) + 1] = __fmaf_rn(-(float)m, ca, beta ? beta[ch] : 0.f);
        }
    }
}
void umx_stat_tickets_reset(void) { void *p = nullptr; if (cudaGetSymbolAddress(&p, g_stat_tickets) == cudaSuccess && p) cudaMemset(p, 0, sizeof(unsigned) * 8192); }
/* InstanceNorm partial sums of a stored blocked-fp16 conv output (what umx_conv_fwd runs after the conv when it is given `part`) */
void umx_in_part(const void *y, int N, int C, int D, int H, int W, double *part) {
    if (!umx_ready("umx_in_part")) return;
    const int T = umx_stats_chunks(D, H, W);
    umx_launch(in_part_k<false>, dim3(T, (C + 31) / 32, N), dim3(256), 0, (const uint4 *)y, (size_t)D * H * W, T, part, C, (const float *)nullptr, (const float *)nullptr, 0.f, (float *)nullptr);
    g_umx_launches++;
    UMX_CK("umx_in_part");
}
/* statistics and coefficients of a stored blocked-fp16 tensor in one launch (part: scratch of umx_stats_doubles doubles).  Launches of
   this function on one device must not overlap (they share the ticket counters); on one stream they never do. */
extern "C" void umx_in_stats_coef(const void *y, int N, int C, int D, int H, int W, const float *gamma, const float *beta, float eps, double *part, float *coef) {
    if (!umx_ready("umx_in_stats_coef")) return;
    const int T = umx_stats_chunks(D, H, W), nb = (C + 31) / 32;
    if ((size_t)N * nb > 8192) { umx_in_part(y, N, C, D, H, W, part); umx_in_coef(part, N, C, D, H, W, gamma, beta, eps, coef); return; }
    umx_launch(in_part_k<true>, dim3(T, nb, N), dim3(256), 0, (const uint4 *)y, (size_t)D * H * W, T, part, C, gamma, beta, eps, coef);
    g_umx_launches++;
    UMX_CK("umx_in_stats_coef");
}
extern "C" void umx_in_coef(const double *part, int N, int C, int D, int H, int W, const float *gamma, const float *beta, float eps, float *coef) {
    if (!umx_ready("umx_in_coef")) return;
    const int T = umx_stats_chunks(D, H, W), Cop = (C + 31) / 32 * 32;
    in_coef_k<<<dim3(C, N), 256>>>(part, C, Cop, T, (double)D * H * W, gamma, beta, eps, coef);
    g_umx_launches++;
    UMX_CK("umx_in_coef");
}

/* NaN-propagating max of magnitudes in one instruction */
__device__ __forceinline__ float amax_nan(float a, float v) { float r; asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(fabsf(v))); return r; }

/* Four threads per voxel row, eight channels (one 16-byte load) each; a block walks a run of voxels of one (sample, block), so the
   sixteen coefficients a thread needs stay in registers.  The row's amax is combined with two shuffles.  grid = (voxel chunks,
   blocks, samples).  This pass is bound by instruction issue (about ten instructions an element for the affine map, the
   activation, two roundings and the MX encode), so the variants are compiled apart: COEF (affine map present), FULL (all 32
   channels of every block are real), S2D (second, space-to-depth destination). */
template <int BITS, bool COEF, bool FULL, bool S2D>
__global__ void __launch_bounds__(256) in_apply_k(const uint4 *__restrict__ x, const float2 *__restrict__ coef, int C, int D, int H, int W, int act,
                                                  uint8_t *__restrict__ q, int nb_dst, int b0, uint8_t *__restrict__ q2, uint4 *__restrict__ hout, int split, int T) {
    pdl_trigger(); pdl_wait();
    const int N = gridDim.z, nb = gridDim.y, blk = blockIdx.y, n = blockIdx.z;
    const size_t S = (size_t)D * H * W;
    const int qd = threadIdx.x & 3, ph = threadIdx.x >> 2;
    constexpr int RB = 32 * BITS / 8;
    float ca[8], cb[8]; bool live[8];
#pragma unroll
    for (int k = 0; k < 8; k++) {
        const int c = blk * 32 + qd * 8 + k;
        live[k] = FULL || c < C; ca[k] = 1.f; cb[k] = 0.f;
        if (COEF && live[k]) { const float2 ab = __ldg(coef + (size_t)n * C + c); ca[k] = ab.x; cb[k] = ab.y; }
    }
    const float slope = act == 2 ? 0.01f : 1.f;           /* LeakyReLU as max(g, slope g); slope 1 leaves g as it is */
    const int pow2 = S2D && !(W & (W - 1)) && !(H & (H - 1)), wsh = pow2 ? __ffs(W) - 1 : -1, hsh = pow2 ? __ffs(H) - 1 : 0;
    const unsigned v0 = (unsigned)(S * blockIdx.x / T), v1 = (unsigned)(S * (blockIdx.x + 1) / T);      /* S < 2^31: 32-bit voxel indices in the loop */
    const uint4 *xp = x + ((size_t)n * nb + blk) * S * 4 + qd;
    uint4 *hp_out = hout ? hout + ((size_t)n * nb + blk) * S * 4 + qd : nullptr;
    const size_t drow = (size_t)n * nb_dst + b0 + blk;
    /* destination of this thread's 8 (fp8) or 4 (fp4) code bytes of voxel v: base + v * stride */
    uint8_t *qb = nullptr; int qs = 0;
    if (q) {
        if (BITS == 8 && split) { qb = q + (drow * 2 + (qd >> 1)) * S * 16 + (qd & 1) * 8; qs = 16; }
        else if (BITS == 8) { qb = q + drow * S * 32 + qd * 8; qs = 32; }
        else { qb = q + drow * S * 16 + qd * 4; qs = 16; }
    }
    uint8_t *qsc = q ? q + (size_t)N * nb_dst * S * RB + drow * S : nullptr;
    for (unsigned vb = v0; vb < v1; vb += 256) {
        /* four rows a thread per trip, their loads issued together */
        uint4 raws[4];
#pragma unroll
        for (int u = 0; u < 4; u++) { const unsigned v = vb + u * 64 + ph; raws[u] = v < v1 ? __ldg(xp + (size_t)v * 4) : make_uint4(0u, 0u, 0u, 0u); }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const unsigned v = vb + u * 64 + ph; const bool ok = v < v1;      /* all 32 lanes stay for the shuffles */
            const __half2 *hp = (const __half2 *)&raws[u];
            uint4 o; __half2 *op = (__half2 *)&o;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float2 t = __half22float2(hp[k]);
                float g0 = t.x, g1 = t.y;
                if (COEF) { g0 = __fmaf_rn(g0, ca[2 * k], cb[2 * k]); g1 = __fmaf_rn(g1, ca[2 * k + 1], cb[2 * k + 1]); }
                g0 = fmaxf(g0, __fmul_rn(slope, g0)); g1 = fmaxf(g1, __fmul_rn(slope, g1));      /* LeakyReLU for 0 < slope <= 1 (NaN stays NaN) */
                if (!FULL) { if (!live[2 * k]) g0 = 0.f; if (!live[2 * k + 1]) g1 = 0.f; }
                op[k] = __floats2half2_rn(g0, g1);
            }
            if (hp_out && ok) hp_out[(size_t)v * 4] = o;
            /* amax of the stored fp16 values, NaN-propagating, taken on the halves (exact: the conversion to fp32 is monotonic) */
            __half2 a2 = __hmax2_nan(__hmax2_nan(__habs2(op[0]), __habs2(op[1])), __hmax2_nan(__habs2(op[2]), __habs2(op[3])));
            const __half a1 = __hmax_nan(__low2half(a2), __high2half(a2));
            unsigned am = __float_as_uint(__half2float(a1)) & 0x7fffffffu;
            am = max(am, __shfl_xor_sync(0xffffffffu, am, 1));
            am = max(am, __shfl_xor_sync(0xffffffffu, am, 2));
            const int e = mx_exp(__uint_as_float(am), BITS == 4 ? 1.f / 6.f : 1.f / 448.f);
            const unsigned sb = (unsigned)(e + 127) & 0xffu;
            unsigned w0, w1 = 0u;
            if (BITS == 8 && e >= -15 && e <= 14) {
                /* 2^-e is a normal fp16: scale the halves (exact, or below 2^-14 where E4M3 rounds to zero either way) and convert pairs */
                const unsigned mh = (unsigned)(15 - e) << 10, m2 = mh | (mh << 16);
                const __half2 mm = *(const __half2 *)&m2;
                unsigned short c0, c1, c2, c3;
                const __half2 s0 = __hmul2(op[0], mm), s1 = __hmul2(op[1], mm), s2 = __hmul2(op[2], mm), s3 = __hmul2(op[3], mm);
                asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(c0) : "r"(*(const unsigned *)&s0));
                asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(c1) : "r"(*(const unsigned *)&s1));
                asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(c2) : "r"(*(const unsigned *)&s2));
                asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(c3) : "r"(*(const unsigned *)&s3));
                w0 = (unsigned)c0 | ((unsigned)c1 << 16); w1 = (unsigned)c2 | ((unsigned)c3 << 16);
            } else {
                float f[8];
#pragma unroll
                for (int k = 0; k < 4; k++) { const float2 r = __half22float2(op[k]); f[2 * k] = r.x; f[2 * k + 1] = r.y; }
                const float m = exp2i(-e);
                if (BITS == 8) { w0 = cvt_e4m3x4(f[0] * m, f[1] * m, f[2] * m, f[3] * m); w1 = cvt_e4m3x4(f[4] * m, f[5] * m, f[6] * m, f[7] * m); }
                else w0 = cvt_e2m1x8(f, m);
            }
            if (!ok) continue;
            if (qb) {
                if (BITS == 8) *(uint2 *)(qb + (size_t)v * qs) = make_uint2(w0, w1); else *(unsigned *)(qb + (size_t)v * qs) = w0;
                if (qd == 0) qsc[v] = (uint8_t)sb;
            }
            if (S2D) {   /* space-to-depth copy: block (tap * nb + blk) at the coarse voxel */
                unsigned xx, yy, zz;
                if (wsh >= 0) { xx = v & ((1u << wsh) - 1u); const unsigned t1 = v >> wsh; yy = t1 & ((1u << hsh) - 1u); zz = t1 >> hsh; }      /* W and H powers of two */
                else { xx = v % (unsigned)W; const unsigned t1 = v / (unsigned)W; yy = t1 % (unsigned)H; zz = t1 / (unsigned)H; }
                const int tap = ((zz & 1) * 2 + (yy & 1)) * 2 + (xx & 1);
                const size_t Sc = S / 8, vc = ((size_t)(zz >> 1) * (H >> 1) + (yy >> 1)) * (W >> 1) + (xx >> 1);
                const size_t ro = (size_t)n * 8 * nb + tap * nb + blk;
                if (BITS == 8 && split) *(uint2 *)(q2 + ((ro * 2 + (qd >> 1)) * Sc + vc) * 16 + (qd & 1) * 8) = make_uint2(w0, w1);
                else if (BITS == 8) *(uint2 *)(q2 + (ro * Sc + vc) * 32 + qd * 8) = make_uint2(w0, w1);
                else *(unsigned *)(q2 + (ro * Sc + vc) * 16 + qd * 4) = w0;
                if (qd == 0) q2[(size_t)N * 8 * nb * Sc * RB + ro * Sc + vc] = (uint8_t)sb;
            }
        }
    }
}
template <int BITS, bool COEF, bool FULL>
static void in_apply_launch(dim3 grid, const void *x, const float *coef, int C, int D, int H, int W, int act, void *q, int nb_dst, int b0, void *q_s2d, void *h, int split, int T) {
    if (q_s2d) umx_launch(in_apply_k<BITS, COEF, FULL, true>, grid, dim3(256), 0, (const uint4 *)x, (const float2 *)coef, C, D, H, W, act, (uint8_t *)q, nb_dst, b0, (uint8_t *)q_s2d, (uint4 *)h, split, T);
    else umx_launch(in_apply_k<BITS, COEF, FULL, false>, grid, dim3(256), 0, (const uint4 *)x, (const float2 *)coef, C, D, H, W, act, (uint8_t *)q, nb_dst, b0, (uint8_t *)nullptr, (uint4 *)h, split, T);
}
extern "C" void umx_in_apply(const void *x, const float *coef, int N, int C, int D, int H, int W, int act, void *q, int bits, int nb_dst, int b0, void *q_s2d, void *h, int layout) {
    if (!umx_ready("umx_in_apply")) return;
    if (q_s2d && ((D | H | W) & 1)) { fprintf(stderr, "umx_in_apply: the space-to-depth copy needs even D, H, W\n"); abort(); }
    const int nb = (C + 31) / 32; if (!nb_dst) { nb_dst = nb; b0 = 0; }
    const size_t S = (size_t)D * H * W;
    if (S >= ((size_t)1 << 31)) { fprintf(stderr, "umx_in_apply: more than 2^31 voxels per sample\n"); abort(); }
    if (!S || !N) return;
    /* runs of about 1024 voxels, enough blocks to fill the machine */
    size_t T = (S + 1023) / 1024; if (T > 65535) T = 65535;
    const dim3 grid((unsigned)T, (unsigned)nb, (unsigned)N);
    const int split = layout == UMX_LAYOUT_SPLIT, full = (C & 31) == 0;
#define UMX_APPLY(B, CO, FU) in_apply_launch<B, CO, FU>(grid, x, coef, C, D, H, W, act, q, nb_dst, b0, q_s2d, h, split, (int)T)
    if (bits == 8) { if (coef) { if (full) UMX_APPLY(8, true, true); else UMX_APPLY(8, true, false); } else { if (full) UMX_APPLY(8, false, true); else UMX_APPLY(8, false, false); } }
    else { if (coef) { if (full) UMX_APPLY(4, true, true); else UMX_APPLY(4, true, false); } else { if (full) UMX_APPLY(4, false, true); else UMX_APPLY(4, false, false); } }
#undef UMX_APPLY
    g_umx_launches++;
    UMX_CK("umx_in_apply");
}
