/* One-tap MX convs as a streaming GEMM: the 1^3 head, the 2^3 stride-2 down conv on a space-to-depth copy (K = 8 Cin) and the
   transposed conv (N = 8 Cout sub-voxel columns), for layers whose prepared weights fit in shared memory.  These layers move
   far more bytes than they compute, so the kernel is built around latency: persistent blocks (two a multiprocessor when shared
   memory allows), weights and B scale factors loaded once per block, and per job only what changes.

   GEMM rows are 128 consecutive voxels of the sample's linear voxel order.  In the split MX layout [plane][voxel][16 B] that is
   one contiguous 2 KB run per 16-byte-wide plane, so the A operand of a K item (32 fp8 or 64 fp4 channels) is one TMA box of
   256 x 2 eight-byte elements: [k half][128 rows][16 B], the canonical K-major no-swizzle operand (core matrices 128 B apart,
   halves 2 KB apart).  Rows past the end of the sample arrive as zeros.  The scale bytes of the same rows arrive as a second
   box (128 bytes x the stage's blocks) and one warp lays them out for tcgen05.cp.

   A job is (row tile, column tile of up to 64 GEMM columns); a stage is up to four K items of a job.  Jobs of a row tile are
   consecutive, so the tile is re-read from L2, not from HBM.  Accumulators alternate between TMEM slots; the epilogue is the
   generic one (bias, fp16 / MX / plane-major output, the transposed conv's scatter).

   Roles (384 threads): warp 0 lane 0 producer, warp 1 lane 0 MMA issue (the warp allocates TMEM), warp 2 scale layout, warp 3
   idle, warps 4-11 epilogue (two groups).  All waits are bounded as in conv_mx_k. */
#include "conv_epi.cuh"
#include "tc_ptx.cuh"
#include <stdlib.h>
#include <string.h>


namespace {

constexpr int kThreadsP = 384;
constexpr int kMaxSlotsP = 8;
constexpr long long kWaitLimitP = 4000000000ll;

struct ConvPArgs {
    int N, nkb, nki, bits, cop, ntp, ntiles, ngroups;
    long long S, rtiles_per_n, jobs;             /* voxels per sample, row tiles per sample, (row tile, column tile) jobs */
    int HW, W;
    int ring, stage_bytes, offSW, offSFA, sw_rows;
    int w_bytes, w_codes, nquad, nslot;
    int tmem_cols, sfa_base, sfb_base;
    int off_w, off_ring;
    const uint8_t *wp;
    EpiArgs e;
    int *err;
};

/* a wait gave up (its own limit, or another role's abort flag): the first to get here names the block; every role of that block then leaves
   where it stood (stage, barrier, parity), which the host prints */
__device__ __forceinline__ void raise_p(const ConvPArgs &a, volatile int *abort_flag, int code, int stage, uint32_t bar_off = 0, uint32_t parity = 0) {
    if (atomicCAS(a.err, 0, code) == 0) { a.err[1] = (int)blockIdx.x; a.err[2] = stage; a.err[3] = (int)threadIdx.x; __threadfence(); }
    if (((volatile int *)a.err)[1] == (int)blockIdx.x && code < 8) { int *d = a.err + 16 + 4 * code; d[0] = stage; d[1] = (int)bar_off; d[2] = (int)parity; d[3] = 1; }
    *abort_flag = 1;
    __threadfence_block();
}

/* EPI: the output mode known at compile time (0: any, read from the arguments; 1: plane-major fp32; 2: plane-major fp16; 3: MX-fp8 split
   layout; 4: the same through the transposed conv's scatter; 5, 6: MX-fp4 likewise), so that the epilogue's code is only what that mode needs */
template <int BITS, int EPI>
__global__ void __launch_bounds__(kThreadsP, 2) conv_mxp_k(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap maps, const ConvPArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint64_t *bars = (uint64_t *)smem_raw;
    uint32_t *tmem_slot = (uint32_t *)(smem_raw + 768);
    volatile int *abort_flag = (volatile int *)(smem_raw + 772);
    uint8_t *wsm = smem_raw + a.off_w, *stages = smem_raw + a.off_ring;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = a.ring, NS = a.nslot;
    const uint32_t bar_tma = smem_u32(bars), bar_sf = bar_tma + 8 * R, bar_empty = bar_tma + 16 * R, bar_accf = bar_tma + 24 * R, bar_acce = bar_accf + 8 * kMaxSlotsP, bar_w = bar_acce + 8 * kMaxSlotsP;
    constexpr int IPQ = BITS == 8 ? 4 : 2, NQ = 4 / IPQ;      /* K items a scale quad, quads a stage */

    if (threadIdx.x == 0) {
        for (int i = 0; i < R; i++) { mbar_init(bar_tma + 8 * i, 1); mbar_init(bar_sf + 8 * i, 1); mbar_init(bar_empty + 8 * i, 1); }
        for (int i = 0; i < kMaxSlotsP; i++) { mbar_init(bar_accf + 8 * i, 1); mbar_init(bar_acce + 8 * i, 8); }
        mbar_init(bar_w, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    pdl_trigger();
    if (threadIdx.x == 0) {
        /* the weight image is a constant of the layer: it may load while the previous kernel of the stream is still running */
        mbar_expect_tx(bar_w, (uint32_t)a.w_bytes);
        for (int o = 0; o < a.w_bytes; o += 32768) bulk_g2s(smem_u32(wsm + o), a.wp + o, (uint32_t)min(32768, a.w_bytes - o), bar_w);
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), (uint32_t)a.tmem_cols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const long long j0 = a.jobs * (long long)blockIdx.x / (long long)gridDim.x, j1 = a.jobs * ((long long)blockIdx.x + 1) / (long long)gridDim.x;

    if (warp == 0) {
        /* ---------------- producer ---------------- */
        if (lane == 0) {
            tma_prefetch_desc(&map0); tma_prefetch_desc(&maps);
            pdl_wait();      /* the only role that reads activations from global memory; every other role's data comes through this thread's loads,
                                so the weight load, the B scale copies and the zeroing of the accumulators overlap the previous kernel */
            int s = 0, ph = 0, it = 0; bool ok = true;
            /* job = (row tile, column tile), column tile fastest; the indices advance incrementally (no division per job) */
            int ntile = (int)(j0 % a.ntiles), n = (int)((j0 / a.ntiles) / a.rtiles_per_n), tin = (int)((j0 / a.ntiles) % a.rtiles_per_n);
            for (long long job = j0; job < j1 && ok; job++) {
                const int cx = tin * 256, pl0 = BITS == 8 ? n * a.nkb * 2 : n * a.nkb, cs = tin * 128, pls = n * a.nkb;
                for (int g = 0; g < a.ngroups; g++) {
                    if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, kWaitLimitP)) { raise_p(a, abort_flag, 1, it); ok = false; break; }
                    const int items = min(4, a.nki - 4 * g);
                    const uint32_t sb = smem_u32(stages + (size_t)s * a.stage_bytes), bar = bar_tma + 8 * s;
                    mbar_expect_tx(bar, (uint32_t)(items * 4096 + a.sw_rows * 128));
                    for (int j = 0; j < items; j++) tma_load_2d(sb + j * 4096, &map0, bar, cx, pl0 + 2 * (4 * g + j));
                    tma_load_2d(sb + a.offSW, &maps, bar, cs, pls + a.sw_rows * g);
                    it++; if (++s == R) { s = 0; ph ^= 1; }
                }
                if (++ntile == a.ntiles) { ntile = 0; if (++tin == (int)a.rtiles_per_n) { tin = 0; n++; } }
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issue ---------------- */
        if (lane == 0) {
            bool ok = mbar_wait(bar_w, 0, abort_flag, kWaitLimitP);
            if (!ok) raise_p(a, abort_flag, 6, 0);
            tc_fence_after();
            const uint32_t wbase = smem_u32(wsm), sf_hi = desc_hi(128), a_hi = desc_hi(128), b_hi = desc_hi(128);
            const uint32_t idesc_b = (BITS == 8 ? idesc_mxf8(0, 0, 0) : idesc_mxf4(0, 0, 0));
            if (ok) {
                const int nsf = a.ntiles * a.ngroups * NQ;
                for (int i = 0; i < nsf; i++) utccp_32x128b(tmem + a.sfb_base + i * 4, desc_make(desc_lo(wbase + a.w_codes + i * 512, 0), sf_hi));
            }
            const uint32_t a_lo0 = desc_lo(smem_u32(stages), 2048), a_step = (uint32_t)a.stage_bytes >> 4, sfa_off = (uint32_t)a.offSFA >> 4;
            const uint32_t b_lo0 = desc_lo(wbase, (uint32_t)a.ntp * 16), b_item = 2u * (uint32_t)a.ntp, b_tile = (uint32_t)a.nki * b_item;
            int s = 0, ph = 0, it = 0, slot = 0, sph = 0;
            long long job = j0; int ntile = (int)(j0 % a.ntiles);
            while (ok && job < j1) {
                const int n_cur = min(a.ntp, a.cop - ntile * a.ntp);
                const uint32_t idn = idesc_b | ((uint32_t)(n_cur >> 3) << 17), d = tmem + (uint32_t)(slot * a.ntp);
                if (!mbar_wait(bar_acce + 8 * slot, (uint32_t)(sph ^ 1), abort_flag, kWaitLimitP)) { raise_p(a, abort_flag, 7, it); break; }
                for (int g = 0; g < a.ngroups; g++) {
                    if (!mbar_wait(bar_sf + 8 * s, ph, abort_flag, kWaitLimitP)) { raise_p(a, abort_flag, 3, it); ok = false; break; }
                    if (!mbar_wait(bar_tma + 8 * s, ph, abort_flag, kWaitLimitP)) { raise_p(a, abort_flag, 2, it); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + (uint32_t)s * a_step, sfa_t = tmem + (uint32_t)a.sfa_base + ((uint32_t)it & 1u) * 8u;
                    const uint32_t sfb_t = tmem + (uint32_t)a.sfb_base + (uint32_t)((ntile * a.ngroups + g) * NQ * 4);
                    const uint32_t bb = b_lo0 + (uint32_t)ntile * b_tile + (uint32_t)(4 * g) * b_item;
                    const int items = min(4, a.nki - 4 * g);
#pragma unroll
                    for (int q = 0; q < NQ; q++) utccp_32x128b(sfa_t + 4 * q, desc_make((a_lo & 0xffffu) + sfa_off + 32u * q, sf_hi));
#pragma unroll
                    for (int j = 0; j < 4; j++) if (j < items) {
                        const int q = j / IPQ, id = (j % IPQ) * (4 / IPQ);
                        const uint32_t idesc = idn | ((uint32_t)id << 4) | ((uint32_t)id << 29), acc = (g == 0 && j == 0) ? 0u : 1u;
                        const uint64_t ad = desc_make(a_lo + (uint32_t)j * 256u, a_hi), bd = desc_make(bb + (uint32_t)j * b_item, b_hi);
                        if (BITS == 8) umma_mxf8(d, ad, bd, idesc, acc, sfa_t + 4 * q, sfb_t + 4 * q); else umma_mxf4(d, ad, bd, idesc, acc, sfa_t + 4 * q, sfb_t + 4 * q);
                    }
                    if (g == a.ngroups - 1) umma_commit(bar_accf + 8 * slot);
                    umma_commit(bar_empty + 8 * s);
                    it++; if (++s == R) { s = 0; ph ^= 1; }
                }
                if (++slot == NS) { slot = 0; sph ^= 1; }
                job++; if (++ntile == a.ntiles) ntile = 0;
            }
        }
    } else if (warp == 2) {
        /* ---------------- A scale layout: the window holds, per block of the stage, the scale bytes of the 128 rows ---------------- */
        int s = 0, ph = 0, it = 0; bool ok = true;
        const long long nst = (j1 - j0) * a.ngroups;
        for (long long i = 0; i < nst && ok; i++) {
            if (!mbar_wait(bar_tma + 8 * s, ph, abort_flag, kWaitLimitP)) { if (lane == 0) raise_p(a, abort_flag, 4, it); ok = false; break; }
            uint8_t *stg = stages + (size_t)s * a.stage_bytes;
            const uint8_t *sw = stg + a.offSW;
            uint32_t *sfa = (uint32_t *)(stg + a.offSFA);
#pragma unroll
            for (int q = 0; q < NQ; q++) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const uint8_t *p = sw + (q * 4) * 128 + c * 32 + lane;
                    sfa[q * 128 + lane * 4 + c] = (uint32_t)p[0] | ((uint32_t)p[128] << 8) | ((uint32_t)p[256] << 16) | ((uint32_t)p[384] << 24);
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sf + 8 * s);
            it++; if (++s == R) { s = 0; ph ^= 1; }
        }
    } else if (warp >= 4) {
        /* ---------------- epilogue: two groups of four warps; a job of two 32-column chunks gives one to each group, jobs of one chunk
           alternate between the groups.  Both groups wait for and release every accumulator slot. ---------------- */
        const int q4 = warp & 3, eg = (warp - 4) >> 2, r = q4 * 32 + lane;
        const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
        int slot = 0, sph = 0, pc = 0; bool dead = false;
        long long job = j0; int ntile = (int)(j0 % a.ntiles), n = (int)((j0 / a.ntiles) / a.rtiles_per_n), tin = (int)((j0 / a.ntiles) % a.rtiles_per_n);
        const unsigned Su = (unsigned)a.S, HWu = (unsigned)a.HW, Wu = (unsigned)a.W;
        for (; job < j1 && !dead; job++, pc++) {
            const int n_cur = min(a.ntp, a.cop - ntile * a.ntp), nchunk = n_cur >> 5;
            const bool mine = nchunk > 1 ? true : (pc & 1) == eg;
            const int jc = nchunk > 1 ? eg : 0;
            if (!mbar_wait(bar_accf + 8 * slot, (uint32_t)sph, abort_flag, kWaitLimitP)) { raise_p(a, abort_flag, 5, pc); dead = true; break; }
            tc_fence_after();
            if (EPI == 7) {
                /* probability bytes of a plane-major output of at most eight channels (the head): only those accumulator columns leave TMEM; the
                   byte of fp16(acc + bias) comes from the table of all 65536 fp16 values; a warp's 32 voxels are 32 consecutive bytes of a plane */
                uint32_t r8[8];
                if (mine) { tmem_ld8(tlane + (uint32_t)(slot * a.ntp), r8); tmem_ld_wait(); }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acce + 8 * slot);
                const unsigned vo = (unsigned)tin * 128u + (unsigned)r;
                if (mine && vo < Su) {
                    uint8_t *yo = (uint8_t *)a.e.y + (size_t)n * a.e.co_real * Su + vo;
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        if (k < a.e.co_real) {
                            const __half h = __float2half_rn(__fadd_rn(__uint_as_float(r8[k]), __ldg(a.e.bias + k)));
                            yo[(size_t)k * Su] = __ldg(a.e.ptab + __half_as_ushort(h));
                        }
                    }
                }
                if (++slot == NS) { slot = 0; sph ^= 1; }
                if (++ntile == a.ntiles) { ntile = 0; if (++tin == (int)a.rtiles_per_n) { tin = 0; n++; } }
                continue;
            }
            uint32_t rr[32];
            if (mine) { tmem_ld32(tlane + (uint32_t)(slot * a.ntp + jc * 32), rr); tmem_ld_wait(); }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acce + 8 * slot);     /* one arrival per warp: arrivals on one barrier serialise */
            if (mine) {
                const unsigned vo = (unsigned)tin * 128u + (unsigned)r;
                const bool row_ok = vo < Su;
                const unsigned zu = vo / HWu, rem = vo - zu * HWu, oyu = rem / Wu;
                float v[32];
#pragma unroll
                for (int k = 0; k < 32; k++) v[k] = __uint_as_float(rr[k]);
                EpiArgs e = a.e;
                if (EPI == 1) { e.out_mode = UMX_OUT_PM32; e.tconv = 0; }
                if (EPI == 2) { e.out_mode = UMX_OUT_PM16; e.tconv = 0; }
                if (EPI == 3) { e.out_mode = UMX_OUT_MX; e.out_bits = 8; e.y_split = 1; e.tconv = 0; }
                if (EPI == 4) { e.out_mode = UMX_OUT_MX; e.out_bits = 8; e.y_split = 1; e.tconv = 1; }
                if (EPI == 5) { e.out_mode = UMX_OUT_MX; e.out_bits = 4; e.tconv = 0; }
                if (EPI == 6) { e.out_mode = UMX_OUT_MX; e.out_bits = 4; e.tconv = 1; }
                epi_chunk(e, n, (int)zu, (int)oyu, (int)(rem - oyu * Wu), row_ok, ntile * (a.ntp >> 5) + jc, v);
            }
            if (++slot == NS) { slot = 0; sph ^= 1; }
            if (++ntile == a.ntiles) { ntile = 0; if (++tin == (int)a.rtiles_per_n) { tin = 0; n++; } }
        }
    }
    /* ---------------- teardown ---------------- */
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && warp == 0 && lane == 0) {
        for (int s = 0; s < R; s++) { const long long t0 = clock64(); while (!mbar_try(bar_tma + 8 * s, 0) && !mbar_try(bar_tma + 8 * s, 1) && clock64() - t0 < 20000000ll) { } }
        { const long long t0 = clock64(); while (!mbar_try(bar_w, 0) && clock64() - t0 < 20000000ll) { } }
    }
    if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, (uint32_t)a.tmem_cols); }
}

/* Weight image of the streaming kernel: codes [column tile][K item][k half][row of the tile][16 B], then the B scale bytes in the TMEM
   scale layout per (column tile, stage of four K items, scale quad): byte (lane, column, id) = row 32 column + lane, K item 4 g + id
   (fp8) or item 4 g + 2 q + id / 2, block id % 2 (fp4).  Quantisation per (row, 32 input channels) as the reference's prep_w8_k /
   prep_w4_k (src/lp_f8fwd.cu:54-71, src/lp_f4fwd.cu:53-66).  One thread per (column tile, K item, row). */
__global__ void __launch_bounds__(128) prep_wp_k(const PrepArgs p, uint8_t *wp, int ntp, int ntiles, int ngroups, int w_codes) {
    const int total = ntiles * p.nki * ntp, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int rl = i % ntp, ki = (i / ntp) % p.nki, nt_i = i / (ntp * p.nki), row = nt_i * ntp + rl;
    const bool live = row < p.cop;
    constexpr int dummy = 0; (void)dummy;
    unsigned w[8]; unsigned sb[2] = {127u, 127u};
    float v[32];
    if (p.bits == 8) {
#pragma unroll
        for (int k = 0; k < 32; k++) v[k] = live ? prep_src(p, row, 0, ki, k) : 0.f;
        sb[0] = mx_encode_row32<8>(v, w);
    } else {
        unsigned w4[4];
#pragma unroll
        for (int h = 0; h < 2; h++) {
#pragma unroll
            for (int k = 0; k < 32; k++) v[k] = live ? prep_src(p, row, 0, 2 * ki + h, k) : 0.f;
            sb[h] = mx_encode_row32<4>(v, w4);
#pragma unroll
            for (int t = 0; t < 4; t++) w[4 * h + t] = w4[t];
        }
    }
    if (!live) { sb[0] = 127u; sb[1] = 127u; }
    uint8_t *base = wp + ((size_t)(nt_i * p.nki + ki) * 2) * ntp * 16;
    *(uint4 *)(base + (size_t)rl * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    *(uint4 *)(base + (size_t)(ntp + rl) * 16) = make_uint4(w[4], w[5], w[6], w[7]);
    const int g = ki >> 2, j = ki & 3, l = rl & 31, c = rl >> 5, nq = p.bits == 8 ? 1 : 2;
    if (p.bits == 8) wp[w_codes + (size_t)((nt_i * ngroups + g) * nq) * 512 + l * 16 + c * 4 + j] = (uint8_t)sb[0];
    else { uint8_t *q = wp + w_codes + (size_t)((nt_i * ngroups + g) * nq + (j >> 1)) * 512 + l * 16 + c * 4 + (j & 1) * 2; q[0] = (uint8_t)sb[0]; q[1] = (uint8_t)sb[1]; }
}

}   // namespace

struct PGeo { int ntp, ntiles, ngroups, nq, w_codes, w_bytes; };
static int p_geometry(const umx_conv *c, PGeo *g) {
    if (c->kind == UMX_CONV3 || c->kind == UMX_CONV3S2) return 0;
    g->ntp = c->cop >= 64 ? 64 : 32; g->ntiles = (c->cop + g->ntp - 1) / g->ntp; g->ngroups = (c->nki + 3) / 4; g->nq = c->bits == 8 ? 1 : 2;
    g->w_codes = g->ntiles * c->nki * 2 * g->ntp * 16;
    g->w_bytes = g->w_codes + g->ntiles * g->ngroups * g->nq * 512;
    if (g->w_bytes > 150 * 1024) return 0;
    if (16 + g->ntiles * g->ngroups * g->nq * 4 + 2 * g->ntp > 512) return 0;
    return 1;
}
/* builds the weight image of the streaming kernel from device fp32 weights; NULL when the conv does not qualify */
uint8_t *umx_conv_p_prepare(const umx_conv *c, const float *w_dev) {
    PGeo g;
    if (!p_geometry(c, &g)) return nullptr;
    uint8_t *wp = (uint8_t *)nn_malloc((size_t)g.w_bytes);
    if (!wp) return nullptr;
    cudaMemset(wp, 127, (size_t)g.w_bytes);
    PrepArgs p; memset(&p, 0, sizeof p);
    p.w = w_dev; p.kind = c->kind; p.co = c->co; p.ci = c->ci; p.bits = c->bits; p.cop = c->cop; p.cob_t = c->cob_t; p.nkb = c->nkb; p.nki = c->nki; p.taps = 1;
    const int total = g.ntiles * c->nki * g.ntp;
    prep_wp_k<<<(total + 127) / 128, 128>>>(p, wp, g.ntp, g.ntiles, g.ngroups, g.w_codes);
    g_umx_launches++;
    return wp;
}
/* x: MX tensor (fp8 in the split layout).  Returns 1 when this kernel does not apply (the caller takes the general kernel), 0 after a
   launch, -1 on error. */
int umx_conv_fwd_p(const umx_conv *c, const void *x, void *enc_v, int N, int D, int H, int W, const EpiArgs &e) {
    typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    PGeo g; ConvPArgs a; memset(&a, 0, sizeof a);
    const size_t S = (size_t)D * H * W;
    if (!c->wp || !p_geometry(c, &g) || (S & 15) || S > (size_t)1 << 30) return 1;
    if (e.out_mode == UMX_OUT_PROB8 && (e.co_real > 8 || g.ntiles != 1 || e.tconv || !e.ptab)) return 1;     /* the probability epilogue is the head's: one column tile, at most eight channels */       /* the scale plane's rows must be multiples of 16 bytes */
    a.N = N; a.nkb = c->nkb; a.nki = c->nki; a.bits = c->bits; a.cop = c->cop; a.ntp = g.ntp; a.ntiles = g.ntiles; a.ngroups = g.ngroups;
    a.S = (long long)S; a.rtiles_per_n = (long long)((S + 127) / 128); a.jobs = (long long)N * a.rtiles_per_n * g.ntiles; a.HW = H * W; a.W = W;
    a.w_codes = g.w_codes; a.w_bytes = g.w_bytes; a.nquad = g.nq;
    a.sw_rows = c->bits == 8 ? 4 : 8;
    a.offSW = 4 * 4096; a.offSFA = a.offSW + 1024; a.stage_bytes = (a.offSFA + g.nq * 512 + 1023) & ~1023;
    a.off_w = 1024; a.off_ring = (a.off_w + a.w_bytes + 1023) & ~1023;
    const int sfb_cols = g.ntiles * g.ngroups * g.nq * 4;
    const int two = a.off_ring + 3 * a.stage_bytes <= 113 * 1024 && (256 - 16 - sfb_cols) / g.ntp >= 2;
    a.tmem_cols = two ? 256 : 512;
    a.nslot = (a.tmem_cols - 16 - sfb_cols) / g.ntp; if (a.nslot > kMaxSlotsP) a.nslot = kMaxSlotsP;
    if (a.nslot < 2) return 1;
    a.sfa_base = a.nslot * g.ntp; a.sfb_base = a.sfa_base + 16;
    a.ring = ((two ? 113 : 227) * 1024 - a.off_ring) / a.stage_bytes; if (a.ring > 8) a.ring = 8;
    if (a.ring < 2) return 1;
    CUtensorMap m0, ms; memset(&m0, 0, sizeof m0); memset(&ms, 0, sizeof ms);
    const int planes = N * c->nkb * (c->bits == 8 ? 2 : 1);
    {
        const cuuint64_t gd[2] = {(cuuint64_t)S * 2, (cuuint64_t)planes}, gs[1] = {(cuuint64_t)S * 16};
        const cuuint32_t box[2] = {256, 2}, es[2] = {1, 1};
        if (((encode_fn)enc_v)(&m0, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, (void *)x, gd, gs, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return 1;
        uint8_t *x_sc = (uint8_t *)x + (size_t)N * c->nkb * S * (c->bits == 8 ? 32 : 16);
        const cuuint64_t gd2[2] = {(cuuint64_t)S, (cuuint64_t)N * c->nkb}, gs2[1] = {(cuuint64_t)S};
        const cuuint32_t box2[2] = {128, (cuuint32_t)a.sw_rows};
        if (((encode_fn)enc_v)(&ms, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)x_sc, gd2, gs2, box2, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return 1;
    }
    a.wp = c->wp; a.e = e; a.err = umx_errflag();
    if (!a.err) return -1;
    int dev = 0, sms = 148; cudaGetDevice(&dev);
    { static int sms_of[16]; if (!sms_of[dev & 15]) { int v = 148; cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev); sms_of[dev & 15] = v; } sms = sms_of[dev & 15]; }   /* looked up once per device */
    static int attr_set[16];
    if (!attr_set[dev & 15]) {
        cudaError_t er = cudaSuccess;
#define UMX_P_ATTR(B, E) if (er == cudaSuccess) er = cudaFuncSetAttribute(conv_mxp_k<B, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)
        UMX_P_ATTR(8, 0); UMX_P_ATTR(8, 1); UMX_P_ATTR(8, 2); UMX_P_ATTR(8, 3); UMX_P_ATTR(8, 4); UMX_P_ATTR(8, 5); UMX_P_ATTR(8, 6); UMX_P_ATTR(8, 7);
        UMX_P_ATTR(4, 0); UMX_P_ATTR(4, 1); UMX_P_ATTR(4, 2); UMX_P_ATTR(4, 3); UMX_P_ATTR(4, 4); UMX_P_ATTR(4, 5); UMX_P_ATTR(4, 6); UMX_P_ATTR(4, 7);
#undef UMX_P_ATTR
        if (er != cudaSuccess) { umx_latch("umx_conv_fwd: shared memory attribute", er); return -1; }
        attr_set[dev & 15] = 1;
    }
    const long long slots = (long long)sms * (two ? 2 : 1);
    const int grid = (int)(a.jobs < slots ? a.jobs : slots);
    const size_t smem = (size_t)a.off_ring + (size_t)a.ring * a.stage_bytes;
    int epi = 0;
    if (e.out_mode == UMX_OUT_PM32 && !e.tconv) epi = 1;
    else if (e.out_mode == UMX_OUT_PM16 && !e.tconv) epi = 2;
    else if (e.out_mode == UMX_OUT_MX && e.out_bits == 8 && e.y_split) epi = e.tconv ? 4 : 3;
    else if (e.out_mode == UMX_OUT_MX && e.out_bits == 4) epi = e.tconv ? 6 : 5;
    else if (e.out_mode == UMX_OUT_PROB8) epi = 7;
#define UMX_P_GO(B, E) umx_launch(conv_mxp_k<B, E>, dim3(grid), dim3(kThreadsP), smem, m0, ms, a)
    if (c->bits == 8) { switch (epi) { case 1: UMX_P_GO(8, 1); break; case 2: UMX_P_GO(8, 2); break; case 3: UMX_P_GO(8, 3); break; case 4: UMX_P_GO(8, 4); break; case 5: UMX_P_GO(8, 5); break; case 6: UMX_P_GO(8, 6); break; case 7: UMX_P_GO(8, 7); break; default: UMX_P_GO(8, 0); } }
    else { switch (epi) { case 1: UMX_P_GO(4, 1); break; case 2: UMX_P_GO(4, 2); break; case 3: UMX_P_GO(4, 3); break; case 4: UMX_P_GO(4, 4); break; case 5: UMX_P_GO(4, 5); break; case 6: UMX_P_GO(4, 6); break; case 7: UMX_P_GO(4, 7); break; default: UMX_P_GO(4, 0); } }
#undef UMX_P_GO
    return 0;
}
