/* The network's first conv: 3^3, one input channel, up to 32 outputs (the role of the reference's tap-packed small-channel kernel
   conv_fwd_f8s_k, src/lp_f8fwd.cuh:153-400: K = taps x channels instead of one K block per tap).

   A 32-channel MX conv spends a whole K = 32 block per tap on one real channel: 27 MMAs a tile, and a 33-byte MX row a voxel as input.
   Here the 27 taps of the one channel are the K dimension of a single GEMM tile, [128 voxels] x [27 -> 32 taps] times [32 taps] x
   [32 outputs], and the input is the fp16 tensor itself.  The arithmetic is that of the MX conv: every input voxel is quantised
   to MX-fp8 by itself (a one-channel row: its own scale, mx_exp of |x|), every weight likewise (prep_w's block of one real channel), and
   the products of those values are accumulated in fp32.  An MX-fp8 value is a 4-bit significand times a power of two, which bf16 holds
   exactly, so the tile runs as a plain tcgen05.mma.kind::f16 on bf16 operands with exact products: the same result as the
   block-scaled path up to the order of the fp32 additions.

   A block walks runs of output planes of one 16 x 8 tile with three roles and two stages.  Four producer warps bring the input planes'
   18 x 10 halo tiles through the quantiser into a ring in shared memory (the loads run three planes ahead) and build the A tile of
   plane z ([K chunk][voxel][16 B], the canonical K-major layout; a thread keeps its voxel's taps of planes z - 1 and z in registers and
   reads only plane z + 1); one thread issues two MMAs (K = 16 each) and a commit; four epilogue warps take the accumulators out of
   TMEM (the bias is already in them: three K positions of A are 1 and B holds the fp32 bias there as three bf16 pieces), round to
   fp16 and pass the rows through shared memory so that they leave as 512-byte runs (as in the z-marching kernel).  Four blocks a
   multiprocessor hide the latencies of each other's short dependent chains.  Output: blocked fp16 [n][1][voxel][32]. */
#include "mx_common.cuh"
#include "tc_ptx.cuh"
#include "conv_epi.cuh"
#include <cuda_bf16.h>
#include <type_traits>

int umx_prof_open(double flops);
void umx_prof_close(int id);

namespace {

constexpr long long kWaitLimitS = 4000000000ll;

struct StemArgs {
    const void *x; uint8_t *y; const uint8_t *wb;      /* x: fp16 [N][D][H][W], or CT bytes read as fp16(byte / 255) (the U8 kernel) */
    int N, D, H, W, tiles_x, tiles; long long units; int *err;
};

/* x quantised to MX-fp8 as a row of one channel, as a number: e4m3(x 2^-e) 2^e with e = mx_exp(|x|); the code is decoded by the hardware
   conversion to fp16 (exact) and scaled by the power of two (exact).  An inf / NaN x (scale byte 0xFF in the MX tensor) gives NaN. */
__device__ __forceinline__ float fq_e4m3_one(float f) {
    const int e = mx_exp(__uint_as_float(__float_as_uint(f) & 0x7fffffffu), 1.f / 448.f);
    unsigned short code; unsigned h2;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(code) : "f"(0.f), "f"(f * exp2i(-e)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(code));
    const float v = __low2float(*(const __half2 *)&h2) * exp2i(e);
    return e == 128 ? __uint_as_float(0x7fc00000u) : v;
}
/* The same for an fp16 input, as bf16 bits.  There the rule collapses: the block scale puts |x| 2^-e into (224, 448], where E4M3 has four
   significant bits, never saturates and is never subnormal, so the value is x rounded to nearest-even at four significant bits (every
   finite fp16 value has been checked against the quantiser).  inf / NaN -> NaN. */
__device__ __forceinline__ unsigned short fq_h16_one(__half x, bool live) {
    const unsigned u = live ? __float_as_uint(__half2float(x)) : 0u;
    const unsigned r = (u + 0x7ffffu + ((u >> 20) & 1u)) >> 20;
    return (u & 0x7f800000u) == 0x7f800000u ? (unsigned short)0x7fc0 : (unsigned short)(r << 4);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

/* K layout of the tile: position 10 dz + 3 dy + dx holds tap (dz, dy, dx), positions 9, 19 and 29 hold 1 (B has the three pieces of the
   bias there), 30 and 31 are zero.  The ten positions of an input plane are five packed words, so a voxel's part of plane z + 1 is
   loaded once and serves as dz = 2, 1, 0 of three consecutive output planes by moving whole words. */
__device__ __forceinline__ void load_plane9(const unsigned short *p, int o, uint32_t *P) {
    unsigned short v[9];
#pragma unroll
    for (int dy = 0; dy < 3; dy++)
#pragma unroll
        for (int dx = 0; dx < 3; dx++) v[dy * 3 + dx] = p[o + dy * 10 + dx];
#pragma unroll
    for (int k = 0; k < 4; k++) P[k] = (uint32_t)v[2 * k] | ((uint32_t)v[2 * k + 1] << 16);
    P[4] = (uint32_t)v[8] | 0x3f800000u;
}
/* barrier 1 of the 128 producer threads, with an OR over their flags: every producer leaves its loop in the same iteration */
__device__ __forceinline__ uint32_t producers_sync_or(uint32_t flag) {
    uint32_t out;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(out) : "r"(flag) : "memory");
    return out;
}

struct StemRun { int n, zb, ze, x0, y0; };
__device__ __forceinline__ StemRun stem_run(const StemArgs &a, long long u, long long u1) {
    StemRun r;
    const long long col = u / a.D;
    r.zb = (int)(u - col * a.D); r.ze = (int)min((long long)a.D, (long long)r.zb + (u1 - u));
    r.n = (int)(col / a.tiles);
    const int txy = (int)(col - (long long)r.n * a.tiles);
    r.x0 = (txy % a.tiles_x) * 8; r.y0 = (txy / a.tiles_x) * 16;
    return r;
}
__device__ __forceinline__ void stem_raise(const StemArgs &a, volatile int *abort_s, int where, int pc) {
    if (atomicCAS(a.err, 0, 9) == 0) { a.err[1] = (int)blockIdx.x; a.err[2] = where; a.err[3] = pc; }
    *abort_s = 1;
}

constexpr int kStemThreads = 288, kStemBlocks = 4;           /* blocks a multiprocessor (registers: 56 a thread) */
/* Three roles, two stages (A tile and accumulator).  Warps 4-7 produce: input planes through the quantiser into the ring, the A tile of
   plane z from the ring, `full`.  One thread of warp 8 multiplies: waits `full` and the stage's accumulator to be free (`acce`), issues
   the two MMAs and a commit on `done`.  Warps 0-3 take the accumulators out (`done`), free them (`acce`) and store the rows.  `done` also
   tells the producers that the stage's A tile has been read.  Every wait is bounded; a wait that gives up raises the block's abort
   flag, which ends the other roles' waits, and records where in the error words. */
template <bool U8>
__global__ void __launch_bounds__(kStemThreads, kStemBlocks) conv_stem_k(const StemArgs a) {
    typedef typename std::conditional<U8, uint8_t, __half>::type XT;
    __shared__ unsigned short qtab[U8 ? 256 : 1];            /* U8: the quantised value (bf16 bits) of every CT byte */
    __shared__ __align__(128) uint8_t sA[2][8192];          /* per stage [4 K chunks][128 voxels][8 bf16] */
    __shared__ __align__(128) uint8_t sB[2048];             /* [4 K chunks][32 outputs][8 bf16] */
    __shared__ __align__(16) uint8_t stg_all[4 * 2048];     /* the epilogue warps' rows on their way out */
    __shared__ __align__(16) __nv_bfloat16 ring[4][192];    /* quantised input planes: 18 x 10 halo tiles, plane zp in slot (zp + 4) % 4 */
    __shared__ __align__(8) unsigned long long bars[6];     /* full[2], done[2], acce[2] */
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_mem;
    volatile int *abort_s = &abort_mem;
    const int warp = (int)threadIdx.x >> 5, lane = (int)threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(&bars[0]), bar_done = smem_u32(&bars[2]), bar_acce = smem_u32(&bars[4]);
    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; s++) { mbar_init(bar_full + 8 * s, 128); mbar_init(bar_done + 8 * s, 1); mbar_init(bar_acce + 8 * s, 4); }
        abort_mem = 0; fence_barrier_init();
    }
    if (threadIdx.x < 128) ((uint4 *)sB)[threadIdx.x] = __ldg((const uint4 *)a.wb + threadIdx.x);     /* layer constants: prepared and complete before any launch */
    if (U8 && threadIdx.x < 256) qtab[threadIdx.x] = fq_h16_one(__float2half_rn(__fdiv_rn((float)threadIdx.x, 255.f)), true);     /* the value umx_u8_to_h16 gives the byte */
    if (warp == 1) { tmem_alloc(smem_u32(&tmem_slot), 64); tmem_relinquish(); }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    pdl_trigger();
    pdl_wait();                                             /* activations are read and the output written from here on */

    const int D = a.D, H = a.H, W = a.W;
    const size_t S = (size_t)D * H * W;
    const long long u0 = a.units * blockIdx.x / gridDim.x, u1 = a.units * (blockIdx.x + 1) / gridDim.x;
    if (warp >= 4 && warp < 8) {
        /* ---- producers ---- */
        const int r = (int)threadIdx.x - 128, o = (r >> 3) * 10 + (r & 7);
        const int t0 = r, t1 = r + 128;
        const size_t HW = (size_t)H * W;
        uint32_t dead = 0; int pc = 0;
        for (long long u = u0; u < u1;) {
            const StemRun rn = stem_run(a, u, u1);
            const XT *xn = (const XT *)a.x + (size_t)rn.n * S;
            /* the halo tile of an input plane: 180 values, two a thread; plane z + 3 is requested while plane z is built */
            const int gy0 = rn.y0 - 1 + t0 / 10, gx0 = rn.x0 - 1 + t0 % 10, gy1 = rn.y0 - 1 + t1 / 10, gx1 = rn.x0 - 1 + t1 % 10;
            const bool in0 = gy0 >= 0 && gy0 < H && gx0 >= 0 && gx0 < W, in1 = t1 < 180 && gy1 >= 0 && gy1 < H && gx1 >= 0 && gx1 < W;
            /* every load is issued unconditionally from an address inside the tensor (positions outside the volume read the sample's first
               voxel) and masked when the value is used: nothing waits for a load at the place where it is issued */
            const XT *s0 = in0 ? xn + (ptrdiff_t)gy0 * W + gx0 : xn, *s1 = in1 ? xn + (ptrdiff_t)gy1 * W + gx1 : xn;
            auto fetch = [&](int zp, XT &v0, XT &v1) {
                const size_t zo = (size_t)min(max(zp, 0), D - 1) * HW;
                v0 = __ldg(s0 + zo); v1 = __ldg(s1 + zo);
            };
            auto quant = [&](XT v, bool live) -> unsigned short {
                if constexpr (U8) return live ? qtab[v] : (unsigned short)0; else return fq_h16_one(v, live);
            };
            auto put = [&](int zp, XT v0, XT v1) {
                const bool zin = zp >= 0 && zp < D;
                unsigned short *dst = (unsigned short *)ring[(zp + 4) & 3];
                dst[t0] = quant(v0, zin && in0);
                if (t1 < 180) dst[t1] = quant(v1, zin && in1);
            };
            XT a0, a1, b0, b1;
            fetch(rn.zb - 1, a0, a1); fetch(rn.zb, b0, b1);
            if (producers_sync_or(dead | (uint32_t)*abort_s)) break;     /* the previous run's last tile has been built: its ring slots are free */
            put(rn.zb - 1, a0, a1); put(rn.zb, b0, b1);
            fetch(rn.zb + 1, a0, a1); fetch(rn.zb + 2, b0, b1);          /* a: plane z + 1, b: plane z + 2 */
            bool out = false;
            uint32_t P0[5], P1[5], P2[5];                                /* the voxel's taps in planes z - 1, z, z + 1 */
            /* one plane; (v0, v1) holds the raw values of plane z + 1 and takes those of plane z + 3 as soon as they are used: the two register
               pairs alternate, so a value is never moved while its load is in flight */
            auto step = [&](int z, XT &v0, XT &v1) -> bool {
                put(z + 1, v0, v1);
                fetch(z + 3, v0, v1);
                if (producers_sync_or(dead | (uint32_t)*abort_s)) return true;
                const int s = pc & 1, k = pc >> 1;
                if (k > 0 && !mbar_wait(bar_done + 8 * s, (uint32_t)((k - 1) & 1), abort_s, kWaitLimitS)) { stem_raise(a, abort_s, 1, pc); dead = 1; pc++; return false; }
                if (z == rn.zb) { load_plane9((const unsigned short *)ring[(z + 3) & 3], o, P0); load_plane9((const unsigned short *)ring[z & 3], o, P1); }
                load_plane9((const unsigned short *)ring[(z + 1) & 3], o, P2);
                uint4 *dstA = (uint4 *)(sA[s] + (size_t)r * 16);
                dstA[0] = make_uint4(P0[0], P0[1], P0[2], P0[3]);
                dstA[128] = make_uint4(P0[4], P1[0], P1[1], P1[2]);
                dstA[256] = make_uint4(P1[3], P1[4], P2[0], P2[1]);
                dstA[384] = make_uint4(P2[2], P2[3], P2[4], 0u);
#pragma unroll
                for (int q = 0; q < 5; q++) { P0[q] = P1[q]; P1[q] = P2[q]; }
                fence_proxy_async();
                mbar_arrive(bar_full + 8 * s);
                pc++;
                return false;
            };
            for (int z = rn.zb; z < rn.ze; z += 2) {
                if (step(z, a0, a1)) { out = true; break; }
                if (z + 1 < rn.ze && step(z + 1, b0, b1)) { out = true; break; }
            }
            if (out) break;
            u += rn.ze - rn.zb;
        }
    } else if (warp == 8) {
        /* ---- the multiplying thread ---- */
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((32u >> 3) << 17) | ((128u >> 4) << 24);      /* fp32 accumulate, bf16 x bf16, N = 32, M = 128, both K-major */
            const uint64_t bd0 = smem_desc(smem_u32(sB), 512, 128), bd1 = smem_desc(smem_u32(sB) + 1024, 512, 128);
            const long long planes = u1 - u0;
            for (int pc = 0; pc < planes; pc++) {
                const int s = pc & 1, k = pc >> 1;
                if (!mbar_wait(bar_full + 8 * s, (uint32_t)(k & 1), abort_s, kWaitLimitS)) { stem_raise(a, abort_s, 2, pc); break; }
                if (k > 0 && !mbar_wait(bar_acce + 8 * s, (uint32_t)((k - 1) & 1), abort_s, kWaitLimitS)) { stem_raise(a, abort_s, 3, pc); break; }
                tc_fence_after();
                const uint32_t sa = smem_u32(sA[s]);
                umma_bf16(tmem + (uint32_t)(32 * s), smem_desc(sa, 2048, 128), bd0, idesc, 0u);
                umma_bf16(tmem + (uint32_t)(32 * s), smem_desc(sa + 4096, 2048, 128), bd1, idesc, 1u);
                umma_commit(bar_done + 8 * s);
            }
        }
    } else {
        /* ---- epilogue: warp q4 owns TMEM lanes [32 q4, 32 q4 + 32) = tile rows 4 q4 .. 4 q4 + 3; the rows pass through shared memory and leave
           as 512-byte runs (as in the z-marching kernel) ---- */
        const int q4 = warp;
        const int cl = (lane & 3) ^ ((lane >> 3) & 3);
        uint8_t *stg = stg_all + q4 * 2048, *stg_w = stg + lane * 64; const int swz = (lane >> 1) & 3;
        const uint8_t *stg_r = stg + (lane >> 2) * 64 + (lane & 3) * 16;
        const size_t plane_b = (size_t)H * W * 64, row_b = (size_t)W * 64;
        int pc = 0; bool dead = false;
        for (long long u = u0; u < u1 && !dead;) {
            const StemRun rn = stem_run(a, u, u1);
            const int sy = rn.y0 + q4 * 4;
            uint8_t *run_dst = a.y + (((size_t)rn.n * S + (size_t)sy * W + rn.x0 + (lane >> 2)) * 64) + cl * 16;
            for (int z = rn.zb; z < rn.ze; z++, pc++) {
                const int s = pc & 1, k = pc >> 1;
                if (!mbar_wait(bar_done + 8 * s, (uint32_t)(k & 1), abort_s, kWaitLimitS)) { stem_raise(a, abort_s, 4, pc); dead = true; break; }
                tc_fence_after();
                uint32_t rr[32];
                tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(32 * s), rr);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();                               /* the accumulators are in registers; the previous plane's rows have been read out of the staging buffer */
                if (lane == 0) mbar_arrive(bar_acce + 8 * s);
#pragma unroll
                for (int k4 = 0; k4 < 4; k4++) {            /* the bias came in through the GEMM: round and store */
                    __half2 h[4];
#pragma unroll
                    for (int t = 0; t < 4; t++) h[t] = __floats2half2_rn(__uint_as_float(rr[8 * k4 + 2 * t]), __uint_as_float(rr[8 * k4 + 2 * t + 1]));
                    *(uint4 *)(stg_w + ((k4 ^ swz) << 4)) = make_uint4(*(const uint32_t *)&h[0], *(const uint32_t *)&h[1], *(const uint32_t *)&h[2], *(const uint32_t *)&h[3]);
                }
                __syncwarp();
                uint8_t *pz = run_dst + (size_t)z * plane_b;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint4 v = *(const uint4 *)(stg_r + i * 512);
                    if (sy + i < H) *(uint4 *)(pz + (size_t)i * row_b) = v;
                }
            }
            u += rn.ze - rn.zb;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, 64); }
}

/* weights w [co][1][27] -> the B tile [4 K chunks][32 outputs][8 bf16], K as load_plane9 lays it out: each weight quantised as the one real channel of its
   32-channel block (src/lp_f8fwd.cu:54-71 with one channel: scale from |w| alone), as a number.  Rows 9, 19 and 29 carry the fp32 bias as
   three bf16 pieces whose sum is the bias exactly (A has ones there), so the accumulator leaves the tensor core with the bias in it. */
__global__ void prep_wstem_k(const float *__restrict__ w, const float *__restrict__ bias_p, uint8_t *__restrict__ wb, int co) {
    const int i = (int)threadIdx.x + (int)blockIdx.x * (int)blockDim.x;
    if (i >= 32 * 32) return;
    const int c = i >> 5, kk = i & 31, g = kk / 10, j = kk % 10;           /* K position kk: plane g, slot j (see load_plane9) */
    __nv_bfloat16 v = __float2bfloat16_rn(0.f);
    if (kk < 30 && j < 9) { if (c < co) v = __float2bfloat16_rn(fq_e4m3_one(w[(size_t)c * 27 + g * 9 + j])); }
    else if (kk < 30) {
        float rest = bias_p[c];
        for (int k = 0; ; k++) { v = __float2bfloat16_rn(rest); if (k == g) break; rest = __fsub_rn(rest, __bfloat162float(v)); }
    }
    ((__nv_bfloat16 *)wb)[((kk >> 3) * 32 + c) * 8 + (kk & 7)] = v;
}

}   // namespace

/* the B tile of a 3^3 conv with one input channel and at most 32 outputs in MX-fp8, or NULL */
uint8_t *umx_conv_stem_prepare(const umx_conv *c, const float *w_dev) {
    if (c->kind != UMX_CONV3 || c->ci != 1 || c->co > 32 || c->bits != 8) return nullptr;
    uint8_t *wb = (uint8_t *)nn_malloc(2048);
    if (!wb) return nullptr;
    prep_wstem_k<<<4, 256>>>(w_dev, c->bias_p, wb, c->co);
    g_umx_launches++;
    return wb;
}
/* y (blocked fp16, one block of 32 channels) = conv of the one-channel tensor x [N][D][H][W], fp16 or (src8) CT bytes read as fp16(byte / 255);
   1: this kernel does not take the shape */
int umx_conv_fwd_stem(const umx_conv *c, const void *x, int src8, int N, int D, int H, int W, void *y) {
    if (!c->wstem || (W & 7) || !N || !D || !H) return 1;
    StemArgs a; memset(&a, 0, sizeof a);
    a.x = x; a.y = (uint8_t *)y; a.wb = c->wstem;
    a.N = N; a.D = D; a.H = H; a.W = W; a.tiles_x = W / 8; a.tiles = a.tiles_x * ((H + 15) / 16); a.units = (long long)N * a.tiles * D;
    a.err = umx_errflag(); if (!a.err) return -1;
    static int slots_of[16];                                /* blocks of this kernel the device holds at once (three a multiprocessor: registers): looked up once per device */
    int dev = 0; cudaGetDevice(&dev); dev &= 15;
    if (!slots_of[dev]) { int sms = 148; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); slots_of[dev] = kStemBlocks * sms; }
    long long grid = slots_of[dev]; if (grid > a.units) grid = a.units;
    const int pid = umx_prof_open(2.0 * (double)N * D * H * W * 27.0 * c->co);
    if (src8) umx_launch(conv_stem_k<true>, dim3((unsigned)grid), dim3(kStemThreads), 0, a); else umx_launch(conv_stem_k<false>, dim3((unsigned)grid), dim3(kStemThreads), 0, a);
    umx_prof_close(pid);
    g_umx_launches++;
    UMX_CK("umx_conv_fwd_stem");
    return 0;
}
