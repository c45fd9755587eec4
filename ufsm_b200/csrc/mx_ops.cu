/* Elementwise operators of the reference interface on MX tensors (32-wide rows, reference layout):
     lp_up2_fwd_mx        exact-2x trilinear upsample, optionally of silu(gn(x))      (src/nn_lp.h:136; arithmetic of src/lp_mx_gn.cu:32-72)
     lp_conv1_fwd_mx      1^3 conv with fp32 weights to fp32 plane-major logits        (src/nn_lp.h:138; arithmetic of src/lp_mx_conv1.cu:4-22)
     lp_conv1_fwd_mx_h16  the same with fp16 logits                                      (src/nn_lp.h:139)
   What is kept of the reference is the order of the roundings, which fixes the bytes: a fine voxel is the sum of its eight coarse corners,
   one fma each onto a zero accumulator, z outermost and x innermost with the nearer corner first on every axis; a logit starts from its
   bias and takes w[co][ci] x[ci] with one fma per input channel in ascending order.  Both are bit-equal to a CPU evaluation of that order
   when no GroupNorm is asked for; with gnp_t.G != 0 the input goes through silu(fma(x, a, b)) first (silu_hw, mx_rows.cuh).

   The kernels are laid out for this machine.  The upsample works on the dual grid: the 2 x 2 x 2 fine voxels that lie between eight coarse
   neighbours all blend those same eight rows, so a block decodes (and activates) a halo tile of coarse rows once into shared memory, and
   four lanes a cell then march along z holding the two coarse planes of the cell in registers: four shared-memory rows fetched per eight
   rows written.  The 1^3 conv is one accumulator chain per (voxel, output) by definition, so a thread owns voxels; it takes two of them
   per trip against one broadcast read of the weights, and the output count is a template parameter in fours. */
#include "mx_rows.cuh"
#include <cuda_fp16.h>

namespace {

/* ---------------------------------------------------------------- upsample ---------------------------------------------------------------- */
constexpr int UZ = 4, UY = 4, UX = 16;                   /* dual cells of a block: 64 quads, each marching UZ cells */
constexpr int HZ = UZ + 1, HY = UY + 1, HX = UX + 1;     /* coarse rows staged: the cells' corners */
constexpr int UP2_ROWS = HZ * HY * HX;
constexpr size_t UP2_SMEM = (size_t)UP2_ROWS * 32 * sizeof(float);

__device__ __forceinline__ int clampi(int v, int hi) { return v < 0 ? 0 : (v > hi ? hi : v); }

/* Dual cell (a, b, c), a in [-1, D - 1] and likewise b, c, has the corners {a, a + 1} x {b, b + 1} x {c, c + 1} clamped to the grid and
   the fine voxels 2 a + 1 (nearer corner a) and 2 a + 2 (nearer corner a + 1) per axis; the first and last cell of an axis hold one
   fine voxel of the grid each.  A staged row lives at tile[8 s + f]: eight float4, lane q's channels at f = q ^ 4 (s & 1) and f ^ 4, so
   that two neighbouring rows read by eight lanes cover all the banks.
   grid (tiles, sample x block) */
/* slab-local statistics (gnp_t.ns != 0, src/nn_lp.h:15-18): the statistics row of sample n at plane z (gn_row, src/lp_slab.cuh:7-12) */
__device__ __forceinline__ int gn_row_of(const gnp_t &gp, int n, int z) {
    int s = (z + gp.zo) / gp.zs;
    s = s < 0 ? 0 : s >= gp.ns ? gp.ns - 1 : s;
    return n * gp.ns + s;
}
template <int BX, int BY, bool GN, bool SL>
__global__ void __launch_bounds__(256, 2) up2_dual_k(const uint8_t *__restrict__ x, uint8_t *__restrict__ y, int N, int C, int D, int H, int W, int tx, int ty, gnp_t gp, int nbx, int b0) {
    extern __shared__ __align__(16) float4 tile[];
    /* y has the nb blocks of its C channels; they are blocks [b0, b0 + nb) of x, which has nbx a sample */
    const int nb = (C + 31) / 32, nbk = blockIdx.y, n = nbk / nb, blk = nbk % nb;
    const size_t xrow0 = ((size_t)n * nbx + b0 + blk) * ((size_t)D * H * W);
    int t = blockIdx.x;
    const int c0 = (t % tx) * UX - 1; t /= tx;
    const int bb0 = (t % ty) * UY - 1, a0 = (t / ty) * UZ - 1;
    const int q = threadIdx.x & 3, quad = threadIdx.x >> 2;
    const size_t S = (size_t)D * H * W;
    constexpr int RBX = BX == 8 ? 32 : 16, RBY = BY == 8 ? 32 : 16;
    const uint8_t *xs = x + (size_t)N * nbx * S * RBX;

    float2 ca[4], cb[4]; bool live[8];
    if (GN) {
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int c = blk * 32 + q * 8 + k;
            float a = 1.f, b = 0.f;
            live[k] = c < C;
            if (live[k]) { const int ng = n * gp.G + c / (C / gp.G); a = __fmul_rn(gp.rstd[ng], gp.gamma[c]); b = __fmaf_rn(-gp.mean[ng], a, gp.beta[c]); }
            if (k & 1) { ca[k >> 1].y = a; cb[k >> 1].y = b; } else { ca[k >> 1].x = a; cb[k >> 1].x = b; }
        }
    }
    /* stage: loads of all trips first, then decode (+ activation) and store */
    constexpr int TRIPS = (UP2_ROWS + 63) / 64;
    uint2 raw[TRIPS]; unsigned sb[TRIPS];
#pragma unroll
    for (int u = 0; u < TRIPS; u++) {
        const int s = u * 64 + quad;
        raw[u] = make_uint2(0u, 0u); sb[u] = 127u;
        if (s < UP2_ROWS) {
            const int ix = s % HX, iy = (s / HX) % HY, iz = s / (HX * HY);
            const size_t row = xrow0 + ((size_t)clampi(a0 + iz, D - 1) * H + clampi(bb0 + iy, H - 1)) * W + clampi(c0 + ix, W - 1);
            raw[u] = qrow_ld<BX>(x, row, q); sb[u] = __ldg(xs + row);
        }
    }
#pragma unroll
    for (int u = 0; u < TRIPS; u++) {
        const int s = u * 64 + quad;
        float2 r[4];
        qrow_dec<BX>(raw[u], mx_scale(sb[u]), r);
        if (GN && SL && s < UP2_ROWS) {
            /* the coefficients of the slab this row's coarse plane lies in */
            const int nr = gn_row_of(gp, n, clampi(a0 + s / (HX * HY), D - 1));
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int c = blk * 32 + q * 8 + k;
                float a = 1.f, b = 0.f;
                if (live[k]) { const int ng = nr * gp.G + c / (C / gp.G); a = __fmul_rn(gp.rstd[ng], gp.gamma[c]); b = __fmaf_rn(-gp.mean[ng], a, gp.beta[c]); }
                if (k & 1) { ca[k >> 1].y = a; cb[k >> 1].y = b; } else { ca[k >> 1].x = a; cb[k >> 1].x = b; }
            }
        }
        if (GN) {
#pragma unroll
            for (int j = 0; j < 4; j++) { const float2 a2 = silu_ab2(r[j], ca[j], cb[j]); if (live[2 * j]) r[j].x = a2.x; if (live[2 * j + 1]) r[j].y = a2.y; }
        }
        if (s < UP2_ROWS) {
            const int f = q ^ ((s & 1) << 2);
            tile[8 * s + f] = make_float4(r[0].x, r[0].y, r[1].x, r[1].y);
            tile[8 * s + (f ^ 4)] = make_float4(r[2].x, r[2].y, r[3].x, r[3].y);
        }
    }
    __syncthreads();

    const int lb = quad / UX, lc = quad % UX;
    const int Do = 2 * D, Ho = 2 * H, Wo = 2 * W;
    const size_t So = 8 * S;                                /* below 2^31: voxel offsets inside a (sample, block) are 32-bit */
    /* the first fine voxel of the quad's cells on y and x, which of the two per axis lie in the grid, and this lane's store addresses
       for voxel 0 of its (sample, block): codes, and (lanes 0 and 1) the scale byte of the cell's first / second x voxel */
    const int fy0 = 2 * (bb0 + lb) + 1, fx0 = 2 * (c0 + lc) + 1;
    const bool vy[2] = {fy0 >= 0 && fy0 < Ho, fy0 + 1 < Ho}, vx[2] = {fx0 >= 0 && fx0 < Wo, fx0 + 1 < Wo};
    uint8_t *yq = y + (size_t)nbk * So * RBY + q * (RBY / 4);
    uint8_t *ysq = y + (size_t)N * nb * So * RBY + (size_t)nbk * So + (q & 1);
    const bool vs = q < 2 && vx[q & 1];
    float2 pl[2][2][2][4];                                  /* [plane of the cell][y corner][x corner][channel pair] */
    auto fetch = [&](int iz, float2 (*dst)[2][4]) {
#pragma unroll
        for (int j = 0; j < 2; j++)
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const int s = (iz * HY + lb + j) * HX + lc + i, f = q ^ ((s & 1) << 2);
                const float4 lo = tile[8 * s + f], hi = tile[8 * s + (f ^ 4)];
                dst[j][i][0] = make_float2(lo.x, lo.y); dst[j][i][1] = make_float2(lo.z, lo.w);
                dst[j][i][2] = make_float2(hi.x, hi.y); dst[j][i][3] = make_float2(hi.z, hi.w);
            }
    };
    fetch(0, pl[0]);
#pragma unroll
    for (int la = 0; la < UZ; la++) {
        /* the cell's lower plane sits in pl[la & 1], the upper one is fetched into the other half */
        fetch(la + 1, pl[(la + 1) & 1]);
        const int fz0 = 2 * (a0 + la) + 1;                  /* cells past the grid compute and store nothing: no early exit, the loop stays unrolled and pl in registers */
        const bool vz[2] = {fz0 >= 0 && fz0 < Do, fz0 + 1 < Do};
#pragma unroll
        for (int oz = 0; oz < 2; oz++)
#pragma unroll
            for (int oy = 0; oy < 2; oy++) {
                const bool okzy = vz[oz] && vy[oy];
                uint2 wq[2]; unsigned sq[2];
#pragma unroll
                for (int ox = 0; ox < 2; ox++) {
                    float2 acc[4];
#pragma unroll
                    for (int k = 0; k < 4; k++) acc[k] = make_float2(0.f, 0.f);
                    /* corner order: z outermost, the nearer corner first on each axis.  An odd fine coordinate (o = 0) is nearer to the
                       cell's lower corner, an even one (o = 1) to the upper */
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const int iz = e >> 2, iy = (e >> 1) & 1, ix = e & 1;
                        const float w3 = (iz ? 0.25f : 0.75f) * (iy ? 0.25f : 0.75f) * (ix ? 0.25f : 0.75f);
                        const float2 *src = pl[(la + (oz ^ iz)) & 1][oy ^ iy][ox ^ ix];
#pragma unroll
                        for (int k = 0; k < 4; k++) acc[k] = __ffma2_rn(make_float2(w3, w3), src[k], acc[k]);
                    }
                    sq[ox] = qrow_enc<BY>(acc, wq[ox]);
                }
                const int vo = ((fz0 + oz) * Ho + fy0 + oy) * Wo + fx0;                       /* meaningful only where stored */
                if (okzy && vx[0]) { if (BY == 8) *(uint2 *)(yq + (ptrdiff_t)vo * 32) = wq[0]; else *(unsigned *)(yq + (ptrdiff_t)vo * 16) = wq[0].x; }
                if (okzy && vx[1]) { if (BY == 8) *(uint2 *)(yq + (ptrdiff_t)(vo + 1) * 32) = wq[1]; else *(unsigned *)(yq + (ptrdiff_t)(vo + 1) * 16) = wq[1].x; }
                if (okzy && vs) ysq[vo] = (uint8_t)((q & 1) ? sq[1] : sq[0]);                 /* two lanes, two neighbouring scale bytes */
            }
    }
}

/* ---------------------------------------------------------------- 1^3 conv ---------------------------------------------------------------- */
/* grid (voxels / 512, sample); outputs co0 + [0, Co) of co_all; weights as [ci][4 CO4] and the sample's GroupNorm coefficients [ci] in
   shared memory, every read of them a broadcast */
template <int BITS, int CO4, bool GN, typename YT, bool SL = false>
__global__ void __launch_bounds__(256) conv1_vox_k(const uint8_t *__restrict__ x, const float *__restrict__ w, const float *__restrict__ bias, YT *__restrict__ y,
                                                   int N, int Ci, int Co, int co0, int co_all, size_t S, gnp_t gp, size_t vb, size_t nv, size_t ly) {
    extern __shared__ __align__(16) float4 c1sm[];
    float4 *sw = c1sm; float2 *sab = (float2 *)(c1sm + (size_t)Ci * CO4);
    constexpr int CO = 4 * CO4, RB = BITS == 8 ? 32 : 16, WORDS = RB / 4;
    const int nb = (Ci + 31) / 32, n = blockIdx.y;
    for (int i = threadIdx.x; i < Ci * CO; i += 256) { const int ci = i / CO, co = i % CO; ((float *)sw)[i] = co < Co ? w[(size_t)co * Ci + ci] : 0.f; }
    /* voxels [vb, vb + nv) of the S; logit planes of ly voxels */
    const size_t v0 = (size_t)blockIdx.x * 512 + threadIdx.x;
    const bool ok[2] = {v0 < nv, v0 + 256 < nv};
    int sof[2] = {0, 0};                                    /* SL: where the coefficient table of each of the thread's two voxels' slabs starts */
    if (GN && !SL) for (int ci = threadIdx.x; ci < Ci; ci += 256) {
        const int ng = n * gp.G + ci / (Ci / gp.G);
        const float a = __fmul_rn(gp.rstd[ng], gp.gamma[ci]);
        sab[ci] = make_float2(a, __fmaf_rn(-gp.mean[ng], a, gp.beta[ci]));
    }
    if (GN && SL) {
        /* one table per statistics slab the block's 512 voxels touch (the launcher has made room for them) */
        const size_t lo = vb + (size_t)blockIdx.x * 512, hi = min(lo + 511, vb + nv - 1);
        const int r_lo = gn_row_of(gp, n, (int)(lo / (size_t)gp.zhw)), r_hi = gn_row_of(gp, n, (int)(hi / (size_t)gp.zhw));
        for (int i = threadIdx.x; i < (r_hi - r_lo + 1) * Ci; i += 256) {
            const int ci = i % Ci, ng = (r_lo + i / Ci) * gp.G + ci / (Ci / gp.G);
            const float a = __fmul_rn(gp.rstd[ng], gp.gamma[ci]);
            sab[i] = make_float2(a, __fmaf_rn(-gp.mean[ng], a, gp.beta[ci]));
        }
#pragma unroll
        for (int u = 0; u < 2; u++) if (ok[u]) sof[u] = (gn_row_of(gp, n, (int)((vb + v0 + 256 * u) / (size_t)gp.zhw)) - r_lo) * Ci;
    }
    __syncthreads();
    const uint8_t *xs = x + (size_t)N * nb * S * RB;
    float acc[2][CO];                                       /* scalar fma: the packed form has the same pipe rate and needs the input twice */
#pragma unroll
    for (int co = 0; co < CO; co++) { const float b0 = (bias && co < Co) ? bias[co] : 0.f; acc[0][co] = b0; acc[1][co] = b0; }
    for (int blk = 0; blk < nb; blk++) {
        unsigned wd[2][WORDS]; float fx[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const size_t row = ((size_t)n * nb + blk) * S + vb + v0 + 256 * u;
#pragma unroll
            for (int j = 0; j < WORDS; j += 4) {
                const uint4 t4 = ok[u] ? __ldg((const uint4 *)(x + row * RB) + j / 4) : make_uint4(0u, 0u, 0u, 0u);
                wd[u][j] = t4.x; wd[u][j + 1] = t4.y; wd[u][j + 2] = t4.z; wd[u][j + 3] = t4.w;
            }
            fx[u] = mx_scale(ok[u] ? __ldg(xs + row) : 127u);
        }
        const int cend = min(32, Ci - blk * 32);
#pragma unroll
        for (int h = 0; h < 4; h++) {                       /* eight channels at a time */
            if (8 * h >= cend) break;
            float2 r[2][4];
#pragma unroll
            for (int u = 0; u < 2; u++) qrow_dec<BITS>(BITS == 8 ? make_uint2(wd[u][2 * h], wd[u][2 * h + 1]) : make_uint2(wd[u][h], 0u), fx[u], r[u]);
            auto chan = [&](int k) {
                const int ci = blk * 32 + 8 * h + k;
                float x0 = (k & 1) ? r[0][k >> 1].y : r[0][k >> 1].x, x1 = (k & 1) ? r[1][k >> 1].y : r[1][k >> 1].x;
                if (GN && !SL) { const float2 ab = sab[ci]; x0 = silu_hw(__fmaf_rn(x0, ab.x, ab.y)); x1 = silu_hw(__fmaf_rn(x1, ab.x, ab.y)); }
                if (GN && SL) { const float2 ab0 = sab[sof[0] + ci], ab1 = sab[sof[1] + ci]; x0 = silu_hw(__fmaf_rn(x0, ab0.x, ab0.y)); x1 = silu_hw(__fmaf_rn(x1, ab1.x, ab1.y)); }
#pragma unroll
                for (int j = 0; j < CO4; j++) {
                    const float4 t4 = sw[ci * CO4 + j];
                    acc[0][4 * j] = __fmaf_rn(t4.x, x0, acc[0][4 * j]); acc[0][4 * j + 1] = __fmaf_rn(t4.y, x0, acc[0][4 * j + 1]);
                    acc[0][4 * j + 2] = __fmaf_rn(t4.z, x0, acc[0][4 * j + 2]); acc[0][4 * j + 3] = __fmaf_rn(t4.w, x0, acc[0][4 * j + 3]);
                    acc[1][4 * j] = __fmaf_rn(t4.x, x1, acc[1][4 * j]); acc[1][4 * j + 1] = __fmaf_rn(t4.y, x1, acc[1][4 * j + 1]);
                    acc[1][4 * j + 2] = __fmaf_rn(t4.z, x1, acc[1][4 * j + 2]); acc[1][4 * j + 3] = __fmaf_rn(t4.w, x1, acc[1][4 * j + 3]);
                }
            };
            if (8 * h + 8 <= cend) {
#pragma unroll
                for (int k = 0; k < 8; k++) chan(k);
            } else {                                            /* the ragged end of the last block */
#pragma unroll
                for (int k = 0; k < 8; k++) if (8 * h + k < cend) chan(k);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < 2; u++)
#pragma unroll
        for (int co = 0; co < CO; co++) if (co < Co && ok[u]) {
            const size_t o = ((size_t)n * co_all + co0 + co) * ly + v0 + 256 * u;
            if (sizeof(YT) == 4) ((float *)y)[o] = acc[u][co]; else ((__half *)y)[o] = __float2half_rn(acc[u][co]);
        }
}

void gp_check(const char *fn, gnp_t gp, int C) {
    if (gp.G && gp.ns && (gp.ns < 0 || gp.zs < 1 || gp.zo < 0 || gp.zo >= gp.zs || gp.zhw < 1)) { fprintf(stderr, "%s: slab-local GroupNorm with ns %d, zs %d, zo %d, zhw %d\n", fn, gp.ns, gp.zs, gp.zo, gp.zhw); abort(); }
    if (gp.G && (gp.G < 1 || C % gp.G)) { fprintf(stderr, "%s: %d channels in %d groups\n", fn, C, gp.G); abort(); }
}

template <int BX, int BY, bool GN, bool SL = false> void up2_launch(dim3 grid, const uint8_t *x, uint8_t *y, shape5 xs, int tx, int ty, gnp_t gp, int nbx, int b0) {
    static bool sized = false;      /* per instantiation; the attribute belongs to the function, any device of this process */
    if (!sized) { cudaFuncSetAttribute(up2_dual_k<BX, BY, GN, SL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)UP2_SMEM); sized = true; }
    up2_dual_k<BX, BY, GN, SL><<<grid, 256, UP2_SMEM>>>(x, y, xs.n, xs.c, xs.d, xs.h, xs.w, tx, ty, gp, nbx, b0);
}
template <int BX, int BY> void up2_gn(dim3 grid, const uint8_t *x, uint8_t *y, shape5 xs, int tx, int ty, gnp_t gp, int nbx, int b0) {
    if (gp.G && gp.ns) up2_launch<BX, BY, true, true>(grid, x, y, xs, tx, ty, gp, nbx, b0);
    else if (gp.G) up2_launch<BX, BY, true>(grid, x, y, xs, tx, ty, gp, nbx, b0); else up2_launch<BX, BY, false>(grid, x, y, xs, tx, ty, gp, nbx, b0);
}

template <int BITS, int CO4, typename YT>
void conv1_launch(dim3 grid, size_t smem, const uint8_t *x, const float *w, const float *b, YT *y, int N, int Ci, int Co, int co0, int co_all, size_t S, gnp_t gp, size_t vb, size_t nv, size_t ly) {
    if (gp.G && gp.ns) conv1_vox_k<BITS, CO4, true, YT, true><<<grid, 256, smem>>>(x, w, b, y, N, Ci, Co, co0, co_all, S, gp, vb, nv, ly);
    else if (gp.G) conv1_vox_k<BITS, CO4, true, YT><<<grid, 256, smem>>>(x, w, b, y, N, Ci, Co, co0, co_all, S, gp, vb, nv, ly);
    else conv1_vox_k<BITS, CO4, false, YT><<<grid, 256, smem>>>(x, w, b, y, N, Ci, Co, co0, co_all, S, gp, vb, nv, ly);
}
template <int BITS, typename YT>
void conv1_co(int co4, dim3 grid, size_t smem, const uint8_t *x, const float *w, const float *b, YT *y, int N, int Ci, int Co, int co0, int co_all, size_t S, gnp_t gp, size_t vb, size_t nv, size_t ly) {
    switch (co4) {
    case 1: conv1_launch<BITS, 1, YT>(grid, smem, x, w, b, y, N, Ci, Co, co0, co_all, S, gp, vb, nv, ly); break;
    case 2: conv1_launch<BITS, 2, YT>(grid, smem, x, w, b, y, N, Ci, Co, co0, co_all, S, gp, vb, nv, ly); break;
    case 3: conv1_launch<BITS, 3, YT>(grid, smem, x, w, b, y, N, Ci, Co, co0, co_all, S, gp, vb, nv, ly); break;
    default: conv1_launch<BITS, 4, YT>(grid, smem, x, w, b, y, N, Ci, Co, co0, co_all, S, gp, vb, nv, ly); break;
    }
}

template <typename YT> void conv1_fwd(const char *fn, const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, YT *y, gnp_t gp, size_t vb = 0, size_t nv = 0, size_t ly = 0) {
    if (!umx_ready(fn)) return;
    if (xdt != UMX_MX8 && xdt != UMX_MX4) { fprintf(stderr, "%s: input dtype %d is not MX\n", fn, xdt); abort(); }
    if (xs.c < 1) { fprintf(stderr, "%s: %d input channels\n", fn, xs.c); abort(); }
    if (cout < 1 || (cout > 16 && cout % 16)) { fprintf(stderr, "%s: cout %d is neither 1..16 nor a multiple of 16\n", fn, cout); abort(); }
    if (xs.n > 65535) { fprintf(stderr, "%s: %d samples\n", fn, xs.n); abort(); }
    gp_check(fn, gp, xs.c);
    if (gp.G && gp.ns && gp.zhw != xs.h * xs.w) { fprintf(stderr, "%s: slab-local GroupNorm with zhw %d on planes of %d voxels\n", fn, gp.zhw, xs.h * xs.w); abort(); }
    const size_t S = (size_t)xs.d * xs.h * xs.w;
    if (!S || !xs.n) return;
    if (xs.c <= 16) {                                          /* rows of 8 / 16 channels (src/lp_common.cuh:132): the same codes and scale in 32-wide rows */
        const int xb = xdt == UMX_MX8 ? 8 : 4;
        void *wide = umx_ws(3, umx_mx_bytes32(xb, xs.n, xs.c, S));
        if (!wide) return;
        umx_mx_rewidth(x, xb, xs.n, xs.c, S, wide, 1);
        x = wide;
    }
    if (!nv) { vb = 0; nv = S; }
    if (!ly) ly = nv;
    if (vb + nv > S || ly < nv) { fprintf(stderr, "%s: voxels [%zu, %zu) of %zu into planes of %zu\n", fn, vb, vb + nv, S, ly); abort(); }
    const dim3 grid((unsigned)((nv + 511) / 512), (unsigned)xs.n);
    /* more than 16 outputs: passes of 16 over the same input (the reference's rule, src/lp_mx_conv1.cu:422-444) */
    for (int c0 = 0; c0 < cout; c0 += 16) {
        const int co = min(16, cout - c0), co4 = (co + 3) / 4;
        /* coefficient tables: one, or with slab-local statistics one per slab that 512 consecutive voxels can touch */
        const int ntab = !gp.G ? 0 : !gp.ns ? 1 : min(gp.ns, (int)((511 / (size_t)gp.zhw + 1) / (size_t)gp.zs) + 2);
        const size_t smem = (size_t)xs.c * co4 * 16 + (size_t)xs.c * 8 * ntab;
        if (smem > 48 * 1024) { fprintf(stderr, "%s: %d input channels need more shared memory than this kernel has\n", fn, xs.c); abort(); }
        const float *wp = w + (size_t)c0 * xs.c, *bp = b ? b + c0 : nullptr;
        if (xdt == UMX_MX8) conv1_co<8, YT>(co4, grid, smem, (const uint8_t *)x, wp, bp, y, xs.n, xs.c, co, c0, cout, S, gp, vb, nv, ly);
        else conv1_co<4, YT>(co4, grid, smem, (const uint8_t *)x, wp, bp, y, xs.n, xs.c, co, c0, cout, S, gp, vb, nv, ly);
        g_umx_launches++;
    }
    UMX_CK(fn);
}

}   // namespace

/* ys: the shape of the coarse tensor that y is the upsample of (its channels are blocks [b0, b0 + blocks of ys.c) of x, which has nbx) */
static void up2_fwd(const char *fn, const void *x, int xdt, shape5 ys, int nbx, int b0, void *y, int ydt, gnp_t gp) {
    if (!umx_ready(fn)) return;
    if ((xdt != UMX_MX8 && xdt != UMX_MX4) || (ydt != UMX_MX8 && ydt != UMX_MX4)) { fprintf(stderr, "%s: dtypes %d -> %d are not MX\n", fn, xdt, ydt); abort(); }
    gp_check(fn, gp, ys.c);
    if (gp.G && gp.ns && gp.zhw != ys.h * ys.w) { fprintf(stderr, "%s: slab-local GroupNorm with zhw %d on planes of %d voxels\n", fn, gp.zhw, ys.h * ys.w); abort(); }
    if (!ys.n || !ys.d || !ys.h || !ys.w) return;
    if ((size_t)ys.d * ys.h * ys.w >= ((size_t)1 << 28)) { fprintf(stderr, "%s: 2^31 fine voxels per sample or more\n", fn); abort(); }
    const int tx = (ys.w + 1 + UX - 1) / UX, ty = (ys.h + 1 + UY - 1) / UY, tz = (ys.d + 1 + UZ - 1) / UZ;      /* D + 1 dual cells an axis */
    const size_t tiles = (size_t)tx * ty * tz, nbk = (size_t)ys.n * ((ys.c + 31) / 32);
    if (tiles > 0x7fffffffu || nbk > 65535) { fprintf(stderr, "%s: %zu tiles x %zu (sample, block) pairs exceed the grid\n", fn, tiles, nbk); abort(); }
    const dim3 grid((unsigned)tiles, (unsigned)nbk);
    const uint8_t *xq = (const uint8_t *)x; uint8_t *yq = (uint8_t *)y;
    if (xdt == UMX_MX4) { if (ydt == UMX_MX4) up2_gn<4, 4>(grid, xq, yq, ys, tx, ty, gp, nbx, b0); else up2_gn<4, 8>(grid, xq, yq, ys, tx, ty, gp, nbx, b0); }
    else { if (ydt == UMX_MX4) up2_gn<8, 4>(grid, xq, yq, ys, tx, ty, gp, nbx, b0); else up2_gn<8, 8>(grid, xq, yq, ys, tx, ty, gp, nbx, b0); }
    g_umx_launches++;
    UMX_CK(fn);
}
extern "C" void lp_up2_fwd_mx(const void *x, int xdt, shape5 xs, void *y, int ydt, gnp_t gp) {
    if (xs.c <= 16 && xs.c >= 1 && (xdt == UMX_MX8 || xdt == UMX_MX4) && (ydt == UMX_MX8 || ydt == UMX_MX4)) {
        /* rows of 8 / 16 channels on either side: widened into scratch, blended there, narrowed */
        const int xb = xdt == UMX_MX8 ? 8 : 4, yb = ydt == UMX_MX8 ? 8 : 4;
        const size_t S = (size_t)xs.d * xs.h * xs.w;
        void *a = umx_ws(3, umx_mx_bytes32(xb, xs.n, xs.c, S)), *o = umx_ws(4, umx_mx_bytes32(yb, xs.n, xs.c, 8 * S));
        if (!a || !o || !S || !xs.n) return;
        umx_mx_rewidth(x, xb, xs.n, xs.c, S, a, 1);
        up2_fwd("lp_up2_fwd_mx", a, xdt, xs, 1, 0, o, ydt, gp);
        umx_mx_rewidth(o, yb, xs.n, xs.c, 8 * S, y, 0);
        return;
    }
    up2_fwd("lp_up2_fwd_mx", x, xdt, xs, (xs.c + 31) / 32, 0, y, ydt, gp);
}
/* src/nn_lp.h:137: the upsample of the 32-channel blocks [b0, b0 + nbk) of x alone; y an MX tensor of 32 nbk channels */
extern "C" void lp_up2_fwd_mx_blocks(const void *x, int xdt, shape5 xs, int b0, int nbk, void *y, int ydt) {
    const int nbx = (xs.c + 31) / 32;
    if (xs.c <= 16 || b0 < 0 || nbk < 1 || b0 + nbk > nbx) { fprintf(stderr, "lp_up2_fwd_mx_blocks: blocks %d + %d of %d channels\n", b0, nbk, xs.c); abort(); }
    shape5 ys = xs; ys.c = 32 * nbk;
    gnp_t none; memset(&none, 0, sizeof none);
    up2_fwd("lp_up2_fwd_mx_blocks", x, xdt, ys, nbx, b0, y, ydt, none);
}
extern "C" void lp_conv1_fwd_mx(const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, float *y, gnp_t gp) {
    conv1_fwd<float>("lp_conv1_fwd_mx", x, xdt, xs, w, b, cout, y, gp);
}
extern "C" void lp_conv1_fwd_mx_h16(const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, void *y, gnp_t gp) {
    conv1_fwd<__half>("lp_conv1_fwd_mx_h16", x, xdt, xs, w, b, cout, (__half *)y, gp);
}
/* src/nn_lp.h:140-141: the logits of voxels [vb, vb + nv) alone (nv 0: all), into planes of nv (fp16) or ly >= nv (fp32; 0: nv) voxels: the
   same arithmetic per voxel as the whole-tensor entries, so a voxel's logits are the same bits either way */
extern "C" void lp_conv1_fwd_mx_h16_r(const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, void *y, gnp_t gp, size_t vb, size_t nv) {
    conv1_fwd<__half>("lp_conv1_fwd_mx_h16_r", x, xdt, xs, w, b, cout, (__half *)y, gp, vb, nv, 0);
}
extern "C" int lp_conv1_fwd_mx_r(const void *x, int xdt, shape5 xs, const float *w, const float *b, int cout, float *y, gnp_t gp, size_t vb, size_t nv, size_t ly) {
    if (xs.n != 1 || !nv) return -1;
    conv1_fwd<float>("lp_conv1_fwd_mx_r", x, xdt, xs, w, b, cout, y, gp, vb, nv, ly);
    return 0;
}

/* lp_add_mx (src/nn_lp.h:135, src/lp_mx_gn.cu:133-150): y += x for two MX tensors of the same format, rows re-encoded (decoded y + decoded x
   in fp32, round to nearest; the reference's stochastic rounding, sr != 0, is not built).  Four lanes a row. */
namespace {
template <int BITS>
__global__ void __launch_bounds__(256) add_rows_k(uint8_t *__restrict__ y, const uint8_t *__restrict__ x, size_t rows) {
    constexpr int RB = BITS == 8 ? 32 : 16;
    const int q = threadIdx.x & 3;
    const uint8_t *xs = x + rows * RB; uint8_t *ys = y + rows * RB;
    for (size_t r0 = ((size_t)blockIdx.x * 256 + threadIdx.x) >> 2; r0 < ((rows + 63) & ~(size_t)63); r0 += (size_t)gridDim.x * 64) {
        const bool ok = r0 < rows;                           /* all lanes of a warp stay for the shuffles */
        const size_t r = ok ? r0 : 0;
        float2 a[4], b[4];
        qrow_dec<BITS>(qrow_ld<BITS>(y, r, q), mx_scale(ys[r]), a);
        qrow_dec<BITS>(qrow_ld<BITS>(x, r, q), mx_scale(__ldg(xs + r)), b);
#pragma unroll
        for (int j = 0; j < 4; j++) a[j] = __fadd2_rn(a[j], b[j]);
        uint2 w;
        const unsigned sb = qrow_enc<BITS>(a, w);
        if (ok) { qrow_st<BITS>(y, r, q, w); if (q == 0) ys[r] = (uint8_t)sb; }
    }
}
}   // namespace
extern "C" void lp_add_mx(void *y, const void *x, shape5 s, int dt, unsigned sr) {
    const char *fn = "lp_add_mx";
    if (!umx_ready(fn)) return;
    if (sr) { fprintf(stderr, "%s: stochastic rounding is not built in this library\n", fn); abort(); }
    if ((dt != 4 && dt != 8) || s.c < 1) { fprintf(stderr, "%s: %d bits, %d channels\n", fn, dt, s.c); abort(); }
    const size_t rows = (size_t)s.n * ((s.c + 31) / 32) * s.d * s.h * s.w;
    if (!rows) return;
    void *y_narrow = nullptr;
    if (s.c <= 16) {                                           /* rows of 8 / 16 channels: both tensors widened into scratch, the sum narrowed back */
        const size_t S = (size_t)s.d * s.h * s.w;
        void *a = umx_ws(3, umx_mx_bytes32(dt, s.n, s.c, S)), *b = umx_ws(4, umx_mx_bytes32(dt, s.n, s.c, S));
        if (!a || !b) return;
        umx_mx_rewidth(y, dt, s.n, s.c, S, a, 1);
        umx_mx_rewidth(x, dt, s.n, s.c, S, b, 1);
        y_narrow = y; y = a; x = b;
    }
    size_t g = (rows + 63) / 64; if (g > 148u * 16u) g = 148u * 16u;
    if (dt == 8) add_rows_k<8><<<(unsigned)g, 256>>>((uint8_t *)y, (const uint8_t *)x, rows);
    else add_rows_k<4><<<(unsigned)g, 256>>>((uint8_t *)y, (const uint8_t *)x, rows);
    g_umx_launches++;
    if (y_narrow) umx_mx_rewidth(y, dt, s.n, s.c, (size_t)s.d * s.h * s.w, y_narrow, 0);
    UMX_CK(fn);
}
