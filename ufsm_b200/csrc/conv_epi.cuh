/* Pieces shared by the conv kernels: the prepared-conv object and the epilogue of one 32-channel chunk of one voxel row. */
#pragma once
#include "mx_common.cuh"

struct umx_conv {
    int kind, co, ci, bits;
    int taps, nkb, nki, cop, cob_t, nt, ntiles_n, nst, items_max, ipq, nquad, w_stage_bytes;
    uint8_t *wpk; float *bias_p;
    uint8_t *wr;                    /* weight image of the z-marching kernel, or NULL */
    uint8_t *wp;                    /* weight image of the one-tap streaming kernel, or NULL */
    uint8_t *wstem;                 /* weight tile of the tap-packed one-channel kernel, or NULL */
};

struct EpiArgs {
    int N, D, H, W;                 /* the grid of GEMM rows */
    int cop;                        /* GEMM columns, padded to 32 */
    int out_mode, out_bits, nb_dst, b0, tconv, co_real, cob_t;   /* cob_t: blocks of one transposed-conv sub-voxel group */
    int y_split;                    /* MX-fp8 output in the split layout [n][blk][half][voxel][16 B] */
    void *y;
    const float *bias;              /* [cop] */
    const uint8_t *ptab;            /* UMX_OUT_PROB8: the probability byte of every fp16 bit pattern (65536 bytes) */
};

/* v: the 32 fp32 accumulators of GEMM row (n, z, oy, ox), 32-column block cb_g.  Adds the bias, rounds as the output mode asks (v keeps
   the values as stored, which is what the statistics are taken from) and writes the row if it lies inside the volume. */
__device__ __forceinline__ void epi_chunk(const EpiArgs &a, int n, int z, int oy, int ox, bool row_ok, int cb_g, float *v) {
    const size_t S = (size_t)a.D * a.H * a.W;
    {
        const float4 *bp = (const float4 *)(a.bias + cb_g * 32);
#pragma unroll
        for (int k = 0; k < 8; k++) { const float4 b = __ldg(bp + k); v[4 * k] = __fadd_rn(v[4 * k], b.x); v[4 * k + 1] = __fadd_rn(v[4 * k + 1], b.y); v[4 * k + 2] = __fadd_rn(v[4 * k + 2], b.z); v[4 * k + 3] = __fadd_rn(v[4 * k + 3], b.w); }
    }
    int ob = cb_g; size_t vo = ((size_t)z * a.H + oy) * a.W + ox; size_t So = S;
    if (a.tconv) {
        const int abc = cb_g / a.cob_t, Ho = 2 * a.H, Wo = 2 * a.W; ob = cb_g % a.cob_t; So = S * 8;
        vo = ((size_t)(2 * z + (abc >> 2)) * Ho + 2 * oy + ((abc >> 1) & 1)) * Wo + 2 * ox + (abc & 1);
    }
    if (a.out_mode == UMX_OUT_MX && a.out_bits == 8) {
        /* fp16 rounding, then the requantiser on the packed halves */
        if (!row_ok) return;
        __half2 h[16];
#pragma unroll
        for (int k = 0; k < 16; k++) h[k] = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
        unsigned w[8];
        const unsigned sbyte = mx_encode_row32_h8(h, w);
        uint8_t *yb = (uint8_t *)a.y;
        const size_t ro = ((size_t)n * a.nb_dst + a.b0 + ob) * So + vo;
        if (a.y_split) {
            const size_t hp = ((size_t)n * a.nb_dst + a.b0 + ob) * 2;
            *(uint4 *)(yb + (hp * So + vo) * 16) = make_uint4(w[0], w[1], w[2], w[3]); *(uint4 *)(yb + ((hp + 1) * So + vo) * 16) = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
            uint4 *dst = (uint4 *)(yb + ro * 32);
            dst[0] = make_uint4(w[0], w[1], w[2], w[3]); dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
        yb[(size_t)a.N * a.nb_dst * So * 32 + ro] = (uint8_t)sbyte;
        return;
    }
    if (a.out_mode != UMX_OUT_PM32 && a.out_mode != UMX_OUT_MXRAW) {
#pragma unroll
        for (int k = 0; k < 32; k++) v[k] = __half2float(__float2half_rn(v[k]));
    }
    if (!row_ok) return;
    const size_t ro = ((size_t)n * a.nb_dst + a.b0 + ob) * So + vo;
    if (a.out_mode == UMX_OUT_H16B) {
        uint4 o[4]; __half2 *op = (__half2 *)o;
#pragma unroll
        for (int k = 0; k < 16; k++) op[k] = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
        uint4 *dst = (uint4 *)a.y + ro * 4;
#pragma unroll
        for (int k = 0; k < 4; k++) dst[k] = o[k];
    } else if (a.out_mode == UMX_OUT_MX || a.out_mode == UMX_OUT_MXRAW) {
        unsigned w[8]; unsigned sbyte;
        uint8_t *yb = (uint8_t *)a.y;
        if (a.out_bits == 8) {
            sbyte = mx_encode_row32<8>(v, w);
            if (a.y_split) {
                const size_t hp = ((size_t)n * a.nb_dst + a.b0 + ob) * 2;
                *(uint4 *)(yb + (hp * So + vo) * 16) = make_uint4(w[0], w[1], w[2], w[3]); *(uint4 *)(yb + ((hp + 1) * So + vo) * 16) = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
                uint4 *dst = (uint4 *)(yb + ro * 32);
                dst[0] = make_uint4(w[0], w[1], w[2], w[3]); dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
            yb[(size_t)a.N * a.nb_dst * So * 32 + ro] = (uint8_t)sbyte;
        } else {
            sbyte = mx_encode_row32<4>(v, w);
            *(uint4 *)(yb + ro * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            yb[(size_t)a.N * a.nb_dst * So * 16 + ro] = (uint8_t)sbyte;
        }
    } else {
        for (int k = 0; k < 32; k++) {
            const int c = ob * 32 + k; if (c >= a.co_real) break;
            const size_t o = ((size_t)n * a.co_real + c) * So + vo;
            if (a.out_mode == UMX_OUT_PM32) ((float *)a.y)[o] = v[k]; else ((__half *)a.y)[o] = __float2half_rn(v[k]);
        }
    }
}

/* ---- weight preparation shared by the conv kernels: where GEMM row `row`, tap `tap`, K block `kb`, element k comes from ---- */
struct PrepArgs {
    const float *w; uint8_t *wpk; const float *bias; float *bias_p;
    int kind, co, ci, bits, cop, cob_t, nkb, nki, taps, nt, ntiles_n, nst, items_max, ipq, nquad, w_stage_bytes;
};
__device__ __forceinline__ float prep_src(const PrepArgs &p, int row, int tap, int kb, int k) {
    /* value of GEMM row `row`, tap `tap`, K block `kb`, element k (0 outside the real weights) */
    if (kb >= p.nkb) return 0.f;
    if (p.kind == UMX_CONV3) { const int ci = kb * 32 + k; return (row < p.co && ci < p.ci) ? p.w[((size_t)row * p.ci + ci) * 27 + tap] : 0.f; }
    if (p.kind == UMX_CONV1) { const int ci = kb * 32 + k; return (row < p.co && ci < p.ci) ? p.w[(size_t)row * p.ci + ci] : 0.f; }
    if (p.kind == UMX_CONV3S2) {   /* K block = tap * blocks(ci) + block; MX-fp4: the blocks of a tap padded to an even count (zero weights) */
        const int nb = (p.ci + 31) / 32, nbi = p.bits == 4 ? (nb + 1) / 2 * 2 : nb, t = kb / nbi, ci = (kb % nbi) * 32 + k;
        return (row < p.co && ci < p.ci) ? p.w[((size_t)row * p.ci + ci) * 27 + t] : 0.f;
    }
    if (p.kind == UMX_DOWN2) {   /* K block = sub-voxel tap * blocks(ci) + block */
        const int nbi = (p.ci + 31) / 32, t = kb / nbi, ci = (kb % nbi) * 32 + k;
        return (row < p.co && ci < p.ci) ? p.w[((size_t)row * p.ci + ci) * 8 + t] : 0.f;
    }
    /* UMX_TCONV2: row = abc * (32 cob_t) + o, w [ci][co][8] */
    const int abc = row / (32 * p.cob_t), o = row % (32 * p.cob_t), ci = kb * 32 + k;
    return (o < p.co && ci < p.ci) ? p.w[((size_t)ci * p.co + o) * 8 + abc] : 0.f;
}
