/* 3^3 MX conv forward, persistent z-marching kernel for layers whose prepared weights fit in shared memory (up to 64 output
   channels: the 32- and 64-channel levels, which hold most of the network's voxels).

   A block keeps the whole weight image (all taps, all input blocks) in shared memory and the B scale factors in TMEM, and walks
   jobs = (sample, z chunk, y tile, x tile).  Inside a job it marches along z.  Each input plane (one TMA halo load of the codes and
   one of the scale bytes per input block) is the A operand of nine MMAs, one per (dy, dx); the three dz taps that use the same
   shifted view are stacked along N: B rows are (dz, channel), and the accumulators of the three output planes z + 1, z, z - 1 sit
   in consecutive TMEM slots (slot = ring position of the plane, descending), so one MMA of N = 3 x channels updates all three.

   What bounds this kernel is not the tensor pipe but instruction issue: a lone thread runs dependent integer code at one
   instruction per four to five cycles, and an M = 128, N = 96, K = 32 MMA is only 48 cycles of tensor work.  So (1) the bookkeeping of
   a stage (TMEM columns, B rows, fresh accumulators, barriers to wait for and to commit) is worked out by the producer thread and
   handed over as a record next to the stage; (2) the MMA thread's steady-state path is eight straight-line MMAs whose operands are
   a base plus a constant; (3) the A scale factors are gathered from a TMA-staged window in shared memory, with no bounds logic
   (voxels outside the volume arrive as zero codes with scale byte 0); (4) InstanceNorm statistics are not taken here but by a
   separate bandwidth-bound pass; (5) two blocks share a multiprocessor when the weights are small enough, doubling the issue rate.

   Roles (256 threads): warp 0 lane 0 producer (records + TMA), warp 1 MMA issue (lane 0) and TMEM allocation, warps 2-3 scale
   gather (alternate stages), warps 4-7 epilogue.  All waits are bounded as in conv_mx_k. */
#include "conv_epi.cuh"
#include "tc_ptx.cuh"
#include <stdlib.h>
#include <string.h>

#ifdef UMX_KPROF
#define KP(...) __VA_ARGS__
#define KMAX(slot, dt, where) do { long long d_ = (dt); long long *q_ = a.prof + (size_t)blockIdx.x * 16 + (slot); if (d_ > q_[0]) { q_[0] = d_; q_[1] = (where); } } while (0)
#else
#define KP(...)
#endif

namespace {

constexpr int kThreadsR = 256;
constexpr int kMaxSlots = 12;
constexpr long long kWaitLimitR = 4000000000ll;

struct ConvRArgs {
    int N, D, H, W, nkb, nki, bits, nt;
    int tiles_x, tiles_y, zc, nzc, njobs;
    int ring, stage_bytes, offSW, offSFA;
    int w_bytes, w_codes, nquad, gt, goff1, goff2, nslot;
    int tmem_cols, sfa_base, sfb_base;           /* TMEM: accumulator slots from 0, two A scale buffers of 20 columns, B scales */
    int off_rec, off_w, off_ring;
    const uint8_t *wr;
    EpiArgs e;
    int *err;
    long long *prof;   /* cycle counters of block 0 when built with UMX_KPROF */
};

/* what the MMA thread does for one stage; written by the producer thread */
struct StageRec {
    uint32_t counts;          /* nseg0 | nseg << 8 | nwait << 16 | ncommit << 24 */
    uint32_t ki, last, pad0;
    uint32_t seg[2][4];       /* taps 1..8: TMEM column, N, B row offset, column offset of the B scale image */
    uint32_t seg0[3][4];      /* tap 0: the same, N | fresh << 16 */
    uint32_t wait[2][2];      /* accumulator-empty barriers to pass first: address, parity */
    uint32_t commit[2];       /* accumulator-full barriers to commit after the stage */
    uint32_t pad1[2];
};
static_assert(sizeof(StageRec) == 128, "stage record is 128 bytes");

__device__ __forceinline__ void raise_r(const ConvRArgs &a, volatile int *abort_flag, int code, int stage) {
    if (atomicCAS(a.err, 0, code) == 0) { a.err[1] = (int)blockIdx.x; a.err[2] = stage; a.err[3] = (int)threadIdx.x; }
    if (!*abort_flag) atomicCAS(a.err + 4 + code, 0, stage + 1);   /* which roles gave up on their own (not because another raised the flag), and where */
    *abort_flag = 1;
    __threadfence_block();
}
template <int BITS> __device__ __forceinline__ void mma_bs(uint32_t d, uint64_t ad, uint64_t bd, uint32_t idesc, uint32_t acc, uint32_t sfa, uint32_t sfb) {
    if (BITS == 8) umma_mxf8(d, ad, bd, idesc, acc, sfa, sfb); else umma_mxf4(d, ad, bd, idesc, acc, sfa, sfb);
}

template <int BITS>
__global__ void __launch_bounds__(kThreadsR, 2) conv_mxr_k(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap maps, const ConvRArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint64_t *bars = (uint64_t *)smem_raw;
    uint32_t *tmem_slot = (uint32_t *)(smem_raw + 768);
    volatile int *abort_flag = (volatile int *)(smem_raw + 772);
    StageRec *recs = (StageRec *)(smem_raw + a.off_rec);
    uint8_t *wsm = smem_raw + a.off_w, *stages = smem_raw + a.off_ring;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = a.ring, NS = a.nslot;
    /* barriers: tma[R] (codes + scale window landed), sf[R] (A scales laid out), empty[R], accumulator full / empty per slot, weights */
    const uint32_t bar_tma = smem_u32(bars), bar_sf = bar_tma + 8 * R, bar_empty = bar_tma + 16 * R, bar_accf = bar_tma + 24 * R, bar_acce = bar_accf + 8 * kMaxSlots, bar_w = bar_acce + 8 * kMaxSlots;
    const int tiles = a.tiles_x * a.tiles_y;
    constexpr int NQ = BITS == 8 ? 3 : 5;                  /* A scale quads per stage */
    constexpr uint32_t TX = 5760u + (BITS == 8 ? 576u : 1152u);

    if (threadIdx.x == 0) {
        for (int i = 0; i < R; i++) { mbar_init(bar_tma + 8 * i, 1); mbar_init(bar_sf + 8 * i, 1); mbar_init(bar_empty + 8 * i, 1); }
        for (int i = 0; i < kMaxSlots; i++) { mbar_init(bar_accf + 8 * i, 1); mbar_init(bar_acce + 8 * i, 128); }
        mbar_init(bar_w, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    KP(const long long ta0 = clock64();)
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), (uint32_t)a.tmem_cols); tmem_relinquish(); }
    KP(if (threadIdx.x == 32) { a.prof[(size_t)blockIdx.x * 16 + 14] = clock64() - ta0; })
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        /* ---------------- producer: stage records and TMA ---------------- */
        if (lane == 0) {
            tma_prefetch_desc(&map0); tma_prefetch_desc(&maps);
            mbar_expect_tx(bar_w, (uint32_t)a.w_bytes);
            for (int o = 0; o < a.w_bytes; o += 32768) bulk_g2s(smem_u32(wsm + o), a.wr + o, (uint32_t)min(32768, a.w_bytes - o), bar_w);
            int s = 0, ph = 0, it = 0, pcj = 0; bool ok = true;   /* pcj: ring position count of the job's first output plane */
            KP(long long p_wait = 0; const long long p_t0 = clock64();)
            for (int job = blockIdx.x; job < a.njobs && ok; job += gridDim.x) {
                const int txy = job % tiles, zci = (job / tiles) % a.nzc, n = job / (tiles * a.nzc);
                const int x0 = (txy % a.tiles_x) * 8, y0 = (txy / a.tiles_x) * 16;
                const int zb = zci * a.zc, ze = min(a.D, zb + a.zc), zlo = max(0, zb - 1), zhi = min(a.D - 1, ze);
                const bool last_job = job + (int)gridDim.x >= a.njobs;
                const int xa = ((x0 - 1) >> 4) << 4;             /* 16-aligned start of the 32-byte scale window (x0 = 0: -16, read as zeros) */
                for (int zi = zlo; zi <= zhi && ok; zi++) for (int ki = 0; ki < a.nki; ki++) {
                    KP(const long long pw0 = clock64();)
                    if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, kWaitLimitR)) { raise_r(a, abort_flag, 1, it); ok = false; break; }
                    KP(p_wait += clock64() - pw0; KMAX(0, clock64() - pw0, it);)
                    /* the record: planes z = zi + 1 - dz for dz = 0, 1, 2 that belong to the job, as runs of consecutive TMEM slots */
                    StageRec *r = recs + s;
                    uint32_t nseg0 = 0, nseg = 0, nwait = 0, ncommit = 0;
                    int prev_slot = -2; bool prev_fresh = false;
                    for (int dz = 0; dz < 3; dz++) {
                        const int z = zi + 1 - dz;
                        if (z < zb || z >= ze) continue;
                        const int pc = pcj + z - zb, slot = NS - 1 - pc % NS;
                        const bool fresh = ki == 0 && zi == max(z - 1, 0);
                        const uint32_t sfo = (uint32_t)(dz == 0 ? 0 : dz == 1 ? a.goff1 : a.goff2);
                        if (fresh) { r->wait[nwait][0] = bar_acce + 8 * slot; r->wait[nwait][1] = (uint32_t)(((pc / NS) & 1) ^ 1); nwait++; }
                        if (ki == a.nki - 1 && min(z + 1, a.D - 1) == zi) r->commit[ncommit++] = bar_accf + 8 * slot;
                        if (slot == prev_slot + 1) r->seg[nseg - 1][1] += (uint32_t)a.nt;
                        else { r->seg[nseg][0] = (uint32_t)(slot * a.nt); r->seg[nseg][1] = (uint32_t)a.nt; r->seg[nseg][2] = (uint32_t)(dz * a.nt); r->seg[nseg][3] = sfo; nseg++; }
                        if (slot == prev_slot + 1 && fresh == prev_fresh) r->seg0[nseg0 - 1][1] += (uint32_t)a.nt;
                        else { r->seg0[nseg0][0] = (uint32_t)(slot * a.nt); r->seg0[nseg0][1] = (uint32_t)a.nt | (fresh ? 0x10000u : 0u); r->seg0[nseg0][2] = (uint32_t)(dz * a.nt); r->seg0[nseg0][3] = sfo; nseg0++; }
                        prev_slot = slot; prev_fresh = fresh;
                    }
                    r->counts = nseg0 | (nseg << 8) | (nwait << 16) | (ncommit << 24);
                    r->ki = (uint32_t)ki; r->last = (last_job && zi == zhi && ki == a.nki - 1) ? 1u : 0u;
                    const uint32_t sb = smem_u32(stages + (size_t)s * a.stage_bytes), bar = bar_tma + 8 * s;
                    mbar_expect_tx(bar, TX);
                    /* codes: two 16-byte-wide planes (fp8: the halves of block ki; fp4: blocks 2 ki and 2 ki + 1), 18 rows of 10 voxels;
                       scale bytes: 18 rows of a 32-byte window per block */
                    tma_load_4d(sb, &map0, bar, (x0 - 1) * 16, y0 - 1, zi, BITS == 8 ? (n * a.nkb + ki) * 2 : n * a.nkb + 2 * ki);
                    tma_load_4d(sb + a.offSW, &maps, bar, xa, y0 - 1, zi, BITS == 8 ? n * a.nkb + ki : n * a.nkb + 2 * ki);
                    it++; if (++s == R) { s = 0; ph ^= 1; }
                }
                pcj += ze - zb;
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issue: follows the records; the common stage is straight-line code ---------------- */
        bool ok = mbar_wait(bar_w, 0, abort_flag, kWaitLimitR);
        if (!ok && lane == 0) raise_r(a, abort_flag, 6, 0);
        tc_fence_after();
        const uint32_t wbase = smem_u32(wsm), R3 = 3u * (uint32_t)a.nt, bstep = 2u * R3;
        const uint32_t a_hi = desc_hi(160), b_hi = desc_hi(128), b_lo0 = desc_lo(wbase, R3 * 16);
        const uint32_t idesc_b = (BITS == 8 ? idesc_mxf8(0, 0, 0) : idesc_mxf4(0, 0, 0));
        const uint32_t sfb_per_ki = (uint32_t)(a.nquad * a.gt * 4), sfb_per_q = (uint32_t)(a.gt * 4);
        const uint32_t sf_hi = desc_hi(128);                     /* scale blocks: 32 rows of 16 bytes, 8-row groups 128 bytes apart */
        if (ok && lane == 0) {
            /* the B scale factors of every (input block, tap quad, image, 128-row group): copied to TMEM once */
            const int nsf = a.nki * a.nquad * a.gt;
            for (int i = 0; i < nsf; i++) utccp_32x128b(tmem + a.sfb_base + i * 4, desc_make(desc_lo(wbase + a.w_codes + i * 512, 0), sf_hi));
        }
        __syncwarp();
        int s = 0, ph = 0, it = 0;
        KP(long long m_full = 0, m_acce = 0, m_issue = 0; const long long m_t0 = clock64();)
        while (ok) {
            KP(const long long mw0 = clock64();)
            if (!mbar_wait(bar_tma + 8 * s, ph, abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 2, it); ok = false; break; }
            if (!mbar_wait(bar_sf + 8 * s, ph, abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 3, it); ok = false; break; }
            KP(const long long mw1 = clock64(); m_full += mw1 - mw0; if (lane == 0) KMAX(2, mw1 - mw0, it);)
            const StageRec *r = recs + s;
            const uint4 h0 = *(const uint4 *)r;                  /* counts, ki, last */
            const uint32_t counts = h0.x, nwait = (counts >> 16) & 0xffu;
            if (nwait) {   /* a fresh plane's slot must have been drained by the epilogue */
                if (!mbar_wait(r->wait[0][0], r->wait[0][1], abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 7, it); ok = false; break; }
                if (nwait > 1 && !mbar_wait(r->wait[1][0], r->wait[1][1], abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 7, it); ok = false; break; }
            }
            tc_fence_after();
            KP(const long long mw2 = clock64(); m_acce += mw2 - mw1; if (lane == 0) KMAX(4, mw2 - mw1, it);)
            if (lane == 0) {
                const uint32_t sb = smem_u32(stages + (size_t)s * a.stage_bytes);
                const uint32_t sfa_t = tmem + (uint32_t)a.sfa_base + (uint32_t)(it & 1) * 20u;
                const uint32_t sf_lo = desc_lo(sb + a.offSFA, 0);
#pragma unroll
                for (int q = 0; q < NQ; q++) utccp_32x128b(sfa_t + 4 * q, desc_make(sf_lo + 32u * q, sf_hi));
                const uint32_t ki = h0.y, a_lo = desc_lo(sb, 2880), b_lo = b_lo0 + ki * 9u * bstep, sfb_t = tmem + (uint32_t)a.sfb_base + ki * sfb_per_ki;
                constexpr int IPQ = BITS == 8 ? 4 : 2;
                /* tap 0: up to three runs, a fresh accumulator starts with accumulate off */
                const uint32_t nseg0 = counts & 0xffu, nseg = (counts >> 8) & 0xffu;
                const uint64_t ad0 = desc_make(a_lo, a_hi);
                for (uint32_t k = 0; k < nseg0; k++) {
                    const uint4 g = *(const uint4 *)r->seg0[k];
                    mma_bs<BITS>(tmem + g.x, ad0, desc_make(b_lo + g.z, b_hi), idesc_b | (((g.y & 0xffffu) >> 3) << 17), (g.y >> 16) ? 0u : 1u, sfa_t, sfb_t + g.w);
                }
                /* taps 1..8: one run in the common case */
                const uint4 g0 = *(const uint4 *)r->seg[0];
                {
                    const uint32_t d = tmem + g0.x, idn = idesc_b | ((g0.y >> 3) << 17), bb = b_lo + g0.z, sfb0 = sfb_t + g0.w;
#pragma unroll
                    for (int j = 1; j < 9; j++) {
                        const int q = j / IPQ, id = (j % IPQ) * (4 / IPQ);
                        mma_bs<BITS>(d, desc_make(a_lo + (uint32_t)((j / 3) * 10 + j % 3), a_hi), desc_make(bb + (uint32_t)j * bstep, b_hi),
                                     idn | ((uint32_t)id << 4) | ((uint32_t)id << 29), 1u, sfa_t + 4 * q, sfb0 + (uint32_t)q * sfb_per_q);
                    }
                }
                if (nseg > 1) {   /* the window wraps around the slot ring: a second run */
                    const uint4 g1 = *(const uint4 *)r->seg[1];
                    const uint32_t d = tmem + g1.x, idn = idesc_b | ((g1.y >> 3) << 17), bb = b_lo + g1.z, sfb1 = sfb_t + g1.w;
#pragma unroll
                    for (int j = 1; j < 9; j++) {
                        const int q = j / IPQ, id = (j % IPQ) * (4 / IPQ);
                        mma_bs<BITS>(d, desc_make(a_lo + (uint32_t)((j / 3) * 10 + j % 3), a_hi), desc_make(bb + (uint32_t)j * bstep, b_hi),
                                     idn | ((uint32_t)id << 4) | ((uint32_t)id << 29), 1u, sfa_t + 4 * q, sfb1 + (uint32_t)q * sfb_per_q);
                    }
                }
                /* read what is still needed from the record first: the commit below hands the stage, record included, back to the producer */
                const uint32_t nc = counts >> 24, cb0 = r->commit[0], cb1 = r->commit[1];
                if (nc > 0) umma_commit(cb0);
                if (nc > 1) umma_commit(cb1);
                umma_commit(bar_empty + 8 * s);
            }
            __syncwarp();
            KP(m_issue += clock64() - mw2; if (lane == 0) KMAX(6, clock64() - mw2, it);)
            it++; if (++s == R) { s = 0; ph ^= 1; }
            if (h0.z) break;
        }
    } else if (warp < 4) {
        /* ---------------- A scale layout: warp 2 takes the even stages, warp 3 the odd ones ----------------
           The TMA left 18 rows of a 32-byte window of scale bytes (two windows for fp4); row r of the tile needs, for tap (dy, dx), the
           byte at window row r / 8 + dy, column r % 8 + dx + (x0 - 1 - xa).  Four rows per lane (one per TMEM column of the quad). */
        const int sfw = warp - 2;
        int it = 0, s = 0, ph = 0; bool ok = true;
        KP(long long g_wait = 0; const long long g_t0 = clock64();)
        for (int job = blockIdx.x; job < a.njobs && ok; job += gridDim.x) {
            const int txy = job % tiles, zci = (job / tiles) % a.nzc;
            const int x0 = (txy % a.tiles_x) * 8;
            const int zb = zci * a.zc, ze = min(a.D, zb + a.zc), zlo = max(0, zb - 1), zhi = min(a.D - 1, ze);
            const int xo = (x0 - 1) - (((x0 - 1) >> 4) << 4);     /* 7 or 15 */
            const int nst = (zhi - zlo + 1) * a.nki;
            for (int i = 0; i < nst && ok; i++) {
                const int my = (it & 1) == sfw, cs = s, cph = ph;
                it++; if (++s == R) { s = 0; ph ^= 1; }
                if (!my) continue;
                KP(const long long gw0 = clock64();)
                if (!mbar_wait(bar_tma + 8 * cs, cph, abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 4, it); ok = false; break; }
                KP(g_wait += clock64() - gw0; if (lane == 0) KMAX(8 + 2 * sfw, clock64() - gw0, it);)
                uint8_t *stg = stages + (size_t)cs * a.stage_bytes;
                const uint8_t *sw = stg + a.offSW;
                uint32_t *sfa = (uint32_t *)(stg + a.offSFA);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int r = q * 32 + lane;
                    const uint8_t *p = sw + (r >> 3) * 32 + (r & 7) + xo;
                    uint32_t wq[5] = {0, 0, 0, 0, 0};
#pragma unroll
                    for (int j = 0; j < 9; j++) {
                        const uint32_t b0 = p[(j / 3) * 32 + j % 3];
                        if (BITS == 8) wq[j >> 2] |= b0 << (8 * (j & 3));
                        else { const uint32_t b1 = p[576 + (j / 3) * 32 + j % 3]; wq[j >> 1] |= (b0 | (b1 << 8)) << (16 * (j & 1)); }
                    }
                    /* quad qd: word (lane, column) = row 32 * column + lane */
#pragma unroll
                    for (int qd = 0; qd < NQ; qd++) sfa[qd * 128 + lane * 4 + q] = wq[qd];
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sf + 8 * cs);
            }
        }
    } else {
        /* ---------------- epilogue: one output plane of one tile at a time ---------------- */
        const int q4 = warp & 3, r = q4 * 32 + lane, ry = r >> 3, rx = r & 7;
        const int nchunk = a.nt >> 5;
        int pcm = 0, pph = 0, pc = 0; bool dead = false;        /* pcm = plane count mod slots, pph = its wrap parity */
        KP(long long e_wait = 0; const long long e_t0 = clock64();)
        for (int job = blockIdx.x; job < a.njobs && !dead; job += gridDim.x) {
            const int txy = job % tiles, zci = (job / tiles) % a.nzc, n = job / (tiles * a.nzc);
            const int ox = (txy % a.tiles_x) * 8 + rx, oy = (txy / a.tiles_x) * 16 + ry;
            const bool row_ok = oy < a.H && ox < a.W;
            const int zb = zci * a.zc, ze = min(a.D, zb + a.zc);
            for (int z = zb; z < ze && !dead; z++, pc++) {
                const int slot = NS - 1 - pcm;
                KP(const long long ew0 = clock64();)
                if (!mbar_wait(bar_accf + 8 * slot, (uint32_t)pph, abort_flag, kWaitLimitR)) { raise_r(a, abort_flag, 5, pc); dead = true; break; }
                KP(e_wait += clock64() - ew0; if (threadIdx.x == 128) KMAX(12, clock64() - ew0, pc);)
                tc_fence_after();
                uint32_t rr[2][32];
                tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(slot * a.nt), rr[0]);
                if (nchunk > 1) tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(slot * a.nt + 32), rr[1]);
                tmem_ld_wait();
                tc_fence_before();
                mbar_arrive(bar_acce + 8 * slot);          /* the slot is free as soon as it is in registers */
#pragma unroll
                for (int jc = 0; jc < 2; jc++) if (jc < nchunk) {
                    float v[32];
#pragma unroll
                    for (int k = 0; k < 32; k++) v[k] = __uint_as_float(rr[jc][k]);
                    epi_chunk(a.e, n, z, oy, ox, row_ok, jc, v);
                }
                if (++pcm == NS) { pcm = 0; pph ^= 1; }
            }
        }
    }
    /* ---------------- teardown ---------------- */
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && warp == 0 && lane == 0) {
        /* after a give-up: let this thread's own copies in flight land (bounded) before the block's shared memory is released */
        for (int s = 0; s < R; s++) { const long long t0 = clock64(); while (!mbar_try(bar_tma + 8 * s, 0) && !mbar_try(bar_tma + 8 * s, 1) && clock64() - t0 < 20000000ll) { } }
        { const long long t0 = clock64(); while (!mbar_try(bar_w, 0) && clock64() - t0 < 20000000ll) { } }
    }
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, (uint32_t)a.tmem_cols); }
}

/* Weight image of the z-marching kernel: codes [input item][dy dx][k half][dz * nt + channel][16 B], then the B scale bytes in the TMEM
   scale layout per (input item, tap quad, first dz of the MMA, 128-row group): byte (lane, column, id) = row 128 g + 32 column + lane counted
   from that dz's first row, tap 4 q + id (fp8) or tap 2 q + id / 2, block id % 2 (fp4).  A block-scaled MMA wants its scale address on a
   4-column boundary of TMEM (a one-column offset faults with "misaligned address"), hence one re-based image per starting dz.
   Quantisation per (row, tap, 32 input channels) as the reference's prep_w8_k / prep_w4_k (src/lp_f8fwd.cu:54-71, src/lp_f4fwd.cu:53-66).
   One thread per (item, dy dx, dz, channel). */
__global__ void __launch_bounds__(128) prep_wr_k(const float *__restrict__ w, uint8_t *__restrict__ wr, int co, int ci, int bits, int nt, int nkb, int nki, int nquad, int gt, int goff1, int goff2, int w_codes) {
    const int total = nki * 9 * 3 * nt, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = i % nt, dz = (i / nt) % 3, j = (i / (3 * nt)) % 9, ki = i / (27 * nt);
    const int tap = dz * 9 + j, R3 = 3 * nt, row = dz * nt + c;
    unsigned wd[8], sb[2] = {127u, 127u};
    float v[32];
    if (bits == 8) {
#pragma unroll
        for (int k = 0; k < 32; k++) { const int cc = ki * 32 + k; v[k] = (c < co && cc < ci) ? w[((size_t)c * ci + cc) * 27 + tap] : 0.f; }
        sb[0] = mx_encode_row32<8>(v, wd);
    } else {
        unsigned w4[4];
#pragma unroll
        for (int h = 0; h < 2; h++) {
#pragma unroll
            for (int k = 0; k < 32; k++) { const int cc = (2 * ki + h) * 32 + k; v[k] = (c < co && cc < ci && 2 * ki + h < nkb) ? w[((size_t)c * ci + cc) * 27 + tap] : 0.f; }
            sb[h] = mx_encode_row32<4>(v, w4);
#pragma unroll
            for (int t = 0; t < 4; t++) wd[4 * h + t] = w4[t];
        }
    }
    uint8_t *base = wr + (size_t)(ki * 9 + j) * 2 * R3 * 16;
    *(uint4 *)(base + (size_t)row * 16) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
    *(uint4 *)(base + (size_t)(R3 + row) * 16) = make_uint4(wd[4], wd[5], wd[6], wd[7]);
    for (int d = 0; d <= dz; d++) {
        const int rr = row - d * nt, g = rr >> 7, col = (rr & 127) >> 5, l = rr & 31, gb = d == 0 ? 0 : d == 1 ? goff1 : goff2;
        if (bits == 8) wr[w_codes + ((ki * nquad + (j >> 2)) * gt + gb + g) * 512 + l * 16 + col * 4 + (j & 3)] = (uint8_t)sb[0];
        else { uint8_t *p = wr + w_codes + ((ki * nquad + (j >> 1)) * gt + gb + g) * 512 + l * 16 + col * 4 + (j & 1) * 2; p[0] = (uint8_t)sb[0]; p[1] = (uint8_t)sb[1]; }
    }
}

}   // namespace

/* geometry of the weight image; 0 when the z-marching kernel cannot run this conv (3^3 only, one column tile of at most 64 channels,
   codes + scales resident in shared memory, B scales resident in TMEM beside at least four accumulator slots) */
struct RGeo { int w_codes, w_bytes, gt, goff1, goff2, tmem_cols, nslot, sfa_base, sfb_base; };
static int r_geometry(const umx_conv *c, RGeo *g) {
    if (c->kind != UMX_CONV3 || c->ntiles_n != 1 || c->nt > 64) return 0;
    const int g0 = (3 * c->nt + 127) / 128, g1 = (2 * c->nt + 127) / 128, g2 = (c->nt + 127) / 128;
    g->goff1 = g0; g->goff2 = g0 + g1; g->gt = g0 + g1 + g2;
    g->w_codes = c->nki * 9 * 2 * 3 * c->nt * 16;
    g->w_bytes = g->w_codes + c->nki * c->nquad * g->gt * 512;
    if (g->w_bytes > 136 * 1024) return 0;
    const int sfb_cols = c->nki * c->nquad * g->gt * 4;
    /* 256 columns (two blocks a multiprocessor) when that leaves four slots, else the whole 512 */
    g->tmem_cols = (256 - 40 - sfb_cols) / c->nt >= 4 ? 256 : 512;
    g->nslot = (g->tmem_cols - 40 - sfb_cols) / c->nt;
    if (g->nslot > kMaxSlots) g->nslot = kMaxSlots;
    if (g->nslot < 4) return 0;
    g->sfa_base = g->nslot * c->nt; g->sfb_base = g->sfa_base + 40;
    return 1;
}
int umx_conv_r_fits(const umx_conv *c) { RGeo g; return r_geometry(c, &g); }
/* builds the weight image from device fp32 weights [co][ci][27]; called once when the conv is created */
uint8_t *umx_conv_r_prepare(const umx_conv *c, const float *w_dev) {
    RGeo g;
    if (!r_geometry(c, &g)) return nullptr;
    uint8_t *wr = (uint8_t *)nn_malloc((size_t)g.w_bytes);
    if (!wr) return nullptr;
    cudaMemset(wr, 127, (size_t)g.w_bytes);
    const int total = c->nki * 27 * c->nt;
    prep_wr_k<<<(total + 127) / 128, 128>>>(w_dev, wr, c->co, c->ci, c->bits, c->nt, c->nkb, c->nki, c->nquad, g.gt, g.goff1, g.goff2, g.w_codes);
    g_umx_launches++;
    return wr;
}
/* x: MX tensor (fp8 in the split layout); m0: tensor map over its codes; enc: the driver's tensor-map encoder (for the scale plane).
   Returns 1 when this kernel does not apply to the geometry (the caller then takes the general kernel), 0 after a launch, -1 on error. */
int umx_conv_fwd_r(const umx_conv *c, const void *x, const CUtensorMap *m0, void *enc_v, int N, int D, int H, int W, const EpiArgs &e) {
    typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    ConvRArgs a; memset(&a, 0, sizeof a);
    RGeo g;
    if (!r_geometry(c, &g) || !c->wr || (W & 15)) return 1;      /* the scale window needs rows that are multiples of 16 bytes */
    a.w_codes = g.w_codes; a.w_bytes = g.w_bytes; a.gt = g.gt; a.goff1 = g.goff1 * 4; a.goff2 = g.goff2 * 4;   /* TMEM column offsets of the dz >= 1, 2 images */
    a.tmem_cols = g.tmem_cols; a.nslot = g.nslot; a.sfa_base = g.sfa_base; a.sfb_base = g.sfb_base;
    a.N = N; a.D = D; a.H = H; a.W = W; a.nkb = c->nkb; a.nki = c->nki; a.bits = c->bits; a.nt = c->nt;
    a.tiles_x = (W + 7) / 8; a.tiles_y = (H + 15) / 16;
    a.nquad = c->nquad;
    /* the codes and the scale window are TMA destinations (128-byte aligned) */
    a.offSW = 5888; a.offSFA = a.offSW + (c->bits == 8 ? 640 : 1152);
    a.stage_bytes = (a.offSFA + c->nquad * 512 + 1023) & ~1023;
    a.off_rec = 1024; a.off_w = a.off_rec + 2048; a.off_ring = (a.off_w + a.w_bytes + 1023) & ~1023;
    int dev = 0, sms = 148; cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    /* two blocks a multiprocessor when shared memory (113 KB each) and TMEM (256 columns each) allow */
    const int two = g.tmem_cols == 256 && a.off_ring + 4 * a.stage_bytes <= 113 * 1024;
    const int room = (two ? 113 : 227) * 1024 - a.off_ring;
    a.ring = room / a.stage_bytes; if (a.ring > 12) a.ring = 12;
    if (a.ring < 3) return 1;
    const int slots = sms * (two ? 2 : 1);
    /* z chunk: the longest of 16, 12, 8, 6, 4, 3, 2, 1 planes that keeps the static round-robin over the blocks at least 93 % balanced */
    const int tiles = a.tiles_x * a.tiles_y; const int cand[8] = {16, 12, 8, 6, 4, 3, 2, 1};
    int best = 1; double best_eff = -1;
    for (int i = 0; i < 8; i++) {
        const int zc = cand[i] < D ? cand[i] : D, nzc = (D + zc - 1) / zc; const long jobs = (long)N * nzc * tiles;
        const long gsz = jobs < slots ? jobs : slots, rounds = (jobs + gsz - 1) / gsz;
        const double eff = (double)jobs / (double)(rounds * gsz) * (jobs < slots ? (double)jobs / slots : 1.0);
        if (eff >= 0.93) { best = zc; best_eff = eff; break; }
        if (eff > best_eff) { best_eff = eff; best = zc; }
    }
    a.zc = best; a.nzc = (D + a.zc - 1) / a.zc; a.njobs = N * a.nzc * tiles;
    const size_t S = (size_t)D * H * W;
    uint8_t *x_sc = (uint8_t *)x + (size_t)N * c->nkb * S * (c->bits == 8 ? 32 : 16);   /* the scale plane follows the codes in either layout */
    CUtensorMap ms; memset(&ms, 0, sizeof ms);
    {
        const cuuint64_t gd[4] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)D, (cuuint64_t)N * c->nkb};
        const cuuint64_t gs[3] = {(cuuint64_t)W, (cuuint64_t)W * H, (cuuint64_t)S};
        const cuuint32_t box[4] = {32, 18, 1, (cuuint32_t)(c->bits == 8 ? 1 : 2)}, es[4] = {1, 1, 1, 1};
        const CUresult r0 = ((encode_fn)enc_v)(&ms, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void *)x_sc, gd, gs, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r0 != CUDA_SUCCESS) return 1;                        /* e.g. a scale plane that is not 16-byte aligned: take the general kernel */
    }
    a.wr = c->wr; a.e = e; a.err = umx_errflag();
    if (!a.err) return -1;
    const size_t smem = (size_t)a.off_ring + (size_t)a.ring * a.stage_bytes;
    static int attr_set[16];
    if (!attr_set[dev & 15]) {
        cudaError_t er = cudaFuncSetAttribute(conv_mxr_k<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (er == cudaSuccess) er = cudaFuncSetAttribute(conv_mxr_k<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (er != cudaSuccess) { umx_latch("umx_conv_fwd: shared memory attribute", er); return -1; }
        attr_set[dev & 15] = 1;
    }
    const int grid = a.njobs < slots ? a.njobs : slots;
#ifdef UMX_KPROF
    a.prof = (long long *)umx_ws(7, (size_t)grid * 128); cudaMemset(a.prof, 0, (size_t)grid * 128);
#endif
    if (c->bits == 8) conv_mxr_k<8><<<grid, kThreadsR, smem>>>(*m0, ms, a); else conv_mxr_k<4><<<grid, kThreadsR, smem>>>(*m0, ms, a);
#ifdef UMX_KPROF
    { static long long hb[512 * 16]; cudaMemcpy(hb, a.prof, (size_t)grid * 128, cudaMemcpyDeviceToHost);
      const char *nm[8] = {"producer", "mma-full", "mma-slot", "mma-issue", "gather0", "gather1", "epilogue", "alloc"};
      for (int k = 0; k < 8; k++) { long long best = -1; int bb = 0; for (int b = 0; b < grid; b++) if (hb[b * 16 + 2 * k] > best) { best = hb[b * 16 + 2 * k]; bb = b; }
        if (best > 2000000) fprintf(stderr, "kprof: longest %s wait %lld cycles in block %d at %lld (grid %d jobs %d zc %d ring %d slots %d tmem %d nki %d nt %d)\n", nm[k], best, bb, hb[bb * 16 + 2 * k + 1], grid, a.njobs, a.zc, a.ring, a.nslot, a.tmem_cols, a.nki, a.nt); } }
#endif
    return 0;
}
