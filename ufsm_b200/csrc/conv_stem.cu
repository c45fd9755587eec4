/* The network's first conv: 3^3, one input channel, up to 32 outputs (the role of the reference's tap-packed small-channel kernel
   conv_fwd_f8s_k, src/lp_f8fwd.cuh:153-400: K = taps x channels instead of one K block per tap).

   A 32-channel MX conv spends a whole K = 32 block per tap on one real channel: 27 MMAs a tile, and a 33-byte MX row a voxel as input.
   Here the 27 taps of the one channel are the K dimension of a single GEMM tile, [128 voxels] x [27 -> 32 taps] times [32 taps] x
   [32 outputs], and the input is the fp16 tensor itself.  The arithmetic is that of the MX conv: every input voxel is quantised
   to MX-fp8 by itself (a one-channel row: its own scale, mx_exp of |x|), every weight likewise (prep_w's block of one real channel), and
   the products of those values are accumulated in fp32.  An MX-fp8 value is a 4-bit significand times a power of two, which bf16 holds
   exactly, so the tile runs as a plain tcgen05.mma.kind::f16 on bf16 operands with exact products: the same result as the
   block-scaled path up to the order of the fp32 additions.

   A block walks runs of output planes of one 16 x 8 tile.  Per plane: four warps bring the next input plane's 18 x 10 halo through the
   quantiser into a three-plane ring in shared memory (while the other four finish the previous plane's epilogue), all eight build
   the A tile from the ring ([K chunk][voxel][16 B], the canonical K-major layout), one thread issues two MMAs (K = 16 each) and a
   commit, and warps 0-3 take the accumulators out of TMEM, add the bias, round to fp16 and pass the rows through shared memory so that
   they leave as 512-byte runs (the same epilogue as the z-marching kernel).  Output: blocked fp16 [n][1][voxel][32]. */
#include "mx_common.cuh"
#include "tc_ptx.cuh"
#include "conv_epi.cuh"
#include <cuda_bf16.h>

int umx_prof_open(double flops);
void umx_prof_close(int id);

namespace {

constexpr long long kWaitLimitS = 4000000000ll;

struct StemArgs {
    const __half *x; uint8_t *y; const uint8_t *wb;
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
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

/* the four 16-byte K chunks (taps 0-7, 8-15, 16-23, 24-26, then 1, 1, 1 for the three bias rows of B and two zeros) of the voxel whose halo origin is `o` in the ring planes p0, p1, p2
   (z - 1, z, z + 1); dst: the voxel's 16 bytes in chunk 0, the other chunks 2 KB apart */
__device__ __forceinline__ void build_row(const unsigned short *p0, const unsigned short *p1, const unsigned short *p2, int o, uint4 *dst) {
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
        unsigned short h2[2];
#pragma unroll
        for (int t = 0; t < 2; t++) {
            const int tap = j + t;
            h2[t] = tap < 30 ? (unsigned short)0x3f80 : (unsigned short)0;
            if (tap < 27) { const int dz = tap / 9, dy = (tap / 3) % 3, dx = tap % 3; h2[t] = (dz == 0 ? p0 : dz == 1 ? p1 : p2)[o + dy * 10 + dx]; }
        }
        w[j >> 1] = (uint32_t)h2[0] | ((uint32_t)h2[1] << 16);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) dst[128 * k] = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
}
/* barrier 1 of the 128 producer threads, with an OR over their flags: every producer leaves its loop in the same iteration */
__device__ __forceinline__ uint32_t producers_sync_or(uint32_t flag) {
    uint32_t out;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(out) : "r"(flag) : "memory");
    return out;
}

/* Bounded wait without a suspend-time hint: the hand-overs of this kernel are short (a tile, two MMAs), and a waiter parked with a
   long hint was seen to come back late */
__device__ __forceinline__ bool mbar_wait_now(uint32_t bar, uint32_t parity, volatile int *abort_flag, long long limit) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) return false;
    }
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

constexpr int kStemThreads = 288;
/* Three roles, two stages (A tile and accumulator).  Warps 4-7 produce: input planes through the quantiser into the ring, the A tile of
   plane z from the ring, `full`.  One thread of warp 8 multiplies: waits `full` and the stage's accumulator to be free (`acce`), issues
   the two MMAs and a commit on `done`.  Warps 0-3 take the accumulators out (`done`), free them (`acce`) and store the rows.  `done` also
   tells the producers that the stage's A tile has been read.  Every wait is bounded; a wait that gives up raises the block's abort
   flag, which ends the other roles' waits, and records where in the error words. */
__global__ void __launch_bounds__(kStemThreads, 3) conv_stem_k(const StemArgs a) {
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
            const __half *xn = a.x + (size_t)rn.n * S;
            /* the halo tile of an input plane: 180 values, two a thread; plane z + 3 is requested while plane z is built */
            const int gy0 = rn.y0 - 1 + t0 / 10, gx0 = rn.x0 - 1 + t0 % 10, gy1 = rn.y0 - 1 + t1 / 10, gx1 = rn.x0 - 1 + t1 % 10;
            const bool in0 = gy0 >= 0 && gy0 < H && gx0 >= 0 && gx0 < W, in1 = t1 < 180 && gy1 >= 0 && gy1 < H && gx1 >= 0 && gx1 < W;
            const __half *s0 = xn + (ptrdiff_t)gy0 * W + gx0, *s1 = xn + (ptrdiff_t)gy1 * W + gx1;
            const __half hz = __ushort_as_half((unsigned short)0);
            auto fetch = [&](int zp, __half &v0, __half &v1) {
                const bool zin = zp >= 0 && zp < D;
                v0 = (zin && in0) ? __ldg(s0 + (size_t)zp * HW) : hz;
                v1 = (zin && in1) ? __ldg(s1 + (size_t)zp * HW) : hz;
            };
            auto put = [&](int zp, __half v0, __half v1) {
                __nv_bfloat16 *dst = ring[(zp + 4) & 3];
                dst[t0] = __float2bfloat16_rn(fq_e4m3_one(__half2float(v0)));
                if (t1 < 180) dst[t1] = __float2bfloat16_rn(fq_e4m3_one(__half2float(v1)));
            };
            __half a0, a1, b0, b1, c0, c1;
            fetch(rn.zb - 1, a0, a1); fetch(rn.zb, b0, b1);
            if (producers_sync_or(dead | (uint32_t)*abort_s)) break;     /* the previous run's last tile has been built: its ring slots are free */
            put(rn.zb - 1, a0, a1); put(rn.zb, b0, b1);
            fetch(rn.zb + 1, a0, a1); fetch(rn.zb + 2, b0, b1);          /* a: plane z + 1, b: plane z + 2 */
            bool out = false;
            for (int z = rn.zb; z < rn.ze; z++, pc++) {
                put(z + 1, a0, a1);
                fetch(z + 3, c0, c1);
                a0 = b0; a1 = b1; b0 = c0; b1 = c1;
                if (producers_sync_or(dead | (uint32_t)*abort_s)) { out = true; break; }
                const int s = pc & 1, k = pc >> 1;
                if (k > 0 && !mbar_wait_now(bar_done + 8 * s, (uint32_t)((k - 1) & 1), abort_s, kWaitLimitS)) { stem_raise(a, abort_s, 1, pc); dead = 1; continue; }
                const unsigned short *p1 = (const unsigned short *)ring[z & 3], *p2 = (const unsigned short *)ring[(z + 1) & 3], *p0 = (const unsigned short *)ring[(z + 3) & 3];
                build_row(p0, p1, p2, o, (uint4 *)(sA[s] + (size_t)r * 16));
                fence_proxy_async();
                mbar_arrive(bar_full + 8 * s);
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
                if (!mbar_wait_now(bar_full + 8 * s, (uint32_t)(k & 1), abort_s, kWaitLimitS)) { stem_raise(a, abort_s, 2, pc); break; }
                if (k > 0 && !mbar_wait_now(bar_acce + 8 * s, (uint32_t)((k - 1) & 1), abort_s, kWaitLimitS)) { stem_raise(a, abort_s, 3, pc); break; }
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
                if (!mbar_wait_now(bar_done + 8 * s, (uint32_t)(k & 1), abort_s, kWaitLimitS)) { stem_raise(a, abort_s, 4, pc); dead = true; break; }
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

/* weights w [co][1][27] -> the B tile [4 K chunks][32 outputs][8 bf16], K = tap: each weight quantised as the one real channel of its
   32-channel block (src/lp_f8fwd.cu:54-71 with one channel: scale from |w| alone), as a number.  Rows 27-29 carry the fp32 bias as
   three bf16 pieces whose sum is the bias exactly (A has ones there), so the accumulator leaves the tensor core with the bias in it. */
__global__ void prep_wstem_k(const float *__restrict__ w, const float *__restrict__ bias_p, uint8_t *__restrict__ wb, int co) {
    const int i = (int)threadIdx.x + (int)blockIdx.x * (int)blockDim.x;
    if (i >= 32 * 32) return;
    const int c = i >> 5, tap = i & 31;
    __nv_bfloat16 v = __float2bfloat16_rn(0.f);
    if (tap < 27) { if (c < co) v = __float2bfloat16_rn(fq_e4m3_one(w[(size_t)c * 27 + tap])); }
    else if (tap < 30) {
        float rest = bias_p[c];
        for (int k = 27; ; k++) { v = __float2bfloat16_rn(rest); if (k == tap) break; rest = __fsub_rn(rest, __bfloat162float(v)); }
    }
    ((__nv_bfloat16 *)wb)[((tap >> 3) * 32 + c) * 8 + (tap & 7)] = v;
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
/* y (blocked fp16, one block of 32 channels) = conv of the fp16 one-channel tensor x [N][D][H][W]; 1: this kernel does not take the shape */
int umx_conv_fwd_stem(const umx_conv *c, const void *x16, int N, int D, int H, int W, void *y) {
    if (!c->wstem || (W & 7) || !N || !D || !H) return 1;
    StemArgs a; memset(&a, 0, sizeof a);
    a.x = (const __half *)x16; a.y = (uint8_t *)y; a.wb = c->wstem;
    a.N = N; a.D = D; a.H = H; a.W = W; a.tiles_x = W / 8; a.tiles = a.tiles_x * ((H + 15) / 16); a.units = (long long)N * a.tiles * D;
    a.err = umx_errflag(); if (!a.err) return -1;
    static int slots_of[16];                                /* blocks of this kernel the device holds at once (three a multiprocessor: registers): looked up once per device */
    int dev = 0; cudaGetDevice(&dev); dev &= 15;
    if (!slots_of[dev]) { int sms = 148; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); slots_of[dev] = 3 * sms; }
    long long grid = slots_of[dev]; if (grid > a.units) grid = a.units;
    const int pid = umx_prof_open(2.0 * (double)N * D * H * W * 27.0 * c->co);
    umx_launch(conv_stem_k, dim3((unsigned)grid), dim3(kStemThreads), 0, a);
    umx_prof_close(pid);
    g_umx_launches++;
    UMX_CK("umx_conv_fwd_stem");
    return 0;
}
