/* 3^3 MX conv forward, persistent z-marching variant for layers whose prepared weights fit in shared memory (up to 64 output
   channels here: the 32- and 64-channel levels, which hold most of the network's voxels).

   A block keeps the whole weight image (all taps, all input blocks) in shared memory and the B scale factors in TMEM, and walks
   jobs = (sample, z chunk, y tile, x tile).  Inside a job it marches along z: each input plane (one TMA halo load + one scale
   gather per input block) feeds up to 27 MMAs, nine taps for each of the three output planes it touches, so every activation byte
   is staged once per 128-voxel column instead of three times and nothing but activations streams through the ring.  Output planes
   accumulate in rotating TMEM buffers (4 x N columns); a plane is committed when its last input plane is done and the epilogue
   warps drain it while the MMAs go on with the next planes.

   Roles (320 threads): warp 0 lane 0 TMA producer, warp 1 MMA issue (lane 0) and TMEM allocation, warps 2-5 scale gather (one warp
   per stage, four stages in flight), warps 6-9 epilogue.  All waits are bounded as in conv_mx_k. */
#include "conv_epi.cuh"
#include "tc_ptx.cuh"
#include <stdlib.h>
#include <string.h>

namespace {

constexpr int kThreadsR = 320;
constexpr int kTmemColsR = 512;
constexpr int kSfaBase = 256, kSfbBase = 296;   /* TMEM columns: [0, 256) accumulators, [256, 296) two A scale buffers, [296, 512) B scales */
constexpr long long kWaitLimitR = 4000000000ll;

struct ConvRArgs {
    int N, D, H, W, nkb, nki, bits, nt;
    int tiles_x, tiles_y, zc, nzc, njobs;
    int ring, stage_bytes, offSFA;
    int w_bytes, w_stage_bytes, nst, ipq, nquad, nacc;
    int off_w, off_ring;
    const uint8_t *x_sc, *wpk;
    EpiArgs e;
    int *err;
    int dbg;
    long long *prof;
};

__device__ __forceinline__ void raise_r(const ConvRArgs &a, volatile int *abort_flag, int code, int stage) {
    if (atomicCAS(a.err, 0, code) == 0) { a.err[1] = (int)blockIdx.x; a.err[2] = stage; a.err[3] = (int)threadIdx.x; }
    *abort_flag = 1;
    __threadfence_block();
}

template <int BITS>
__global__ void __launch_bounds__(kThreadsR, 1) conv_mxr_k(const __grid_constant__ CUtensorMap map0, const ConvRArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint64_t *bars = (uint64_t *)smem_raw;
    uint32_t *tmem_slot = (uint32_t *)(smem_raw + 512);
    volatile int *abort_flag = (volatile int *)(smem_raw + 516);
    double *spart = (double *)(smem_raw + 1024);                 /* [2][quarter][chunk 2][lane][2] = 8 KB */
    uint8_t *wsm = smem_raw + a.off_w, *stages = smem_raw + a.off_ring;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = a.ring, NA = a.nacc;
    const uint32_t bar_tma = smem_u32(bars), bar_sf = bar_tma + 8 * R, bar_empty = bar_tma + 16 * R, bar_accf = bar_tma + 24 * R, bar_acce = bar_accf + 32, bar_w = bar_acce + 32;
    const int tiles = a.tiles_x * a.tiles_y;
    const size_t S = (size_t)a.D * a.H * a.W;

    if (threadIdx.x == 0) {
        for (int i = 0; i < R; i++) { mbar_init(bar_tma + 8 * i, 1); mbar_init(bar_sf + 8 * i, 1); mbar_init(bar_empty + 8 * i, 1); }
        for (int i = 0; i < 4; i++) { mbar_init(bar_accf + 8 * i, 1); mbar_init(bar_acce + 8 * i, 128); }
        mbar_init(bar_w, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), kTmemColsR); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        /* ---------------- TMA producer ---------------- */
        if (lane == 0) {
            tma_prefetch_desc(&map0);
            mbar_expect_tx(bar_w, (uint32_t)a.w_bytes);
            for (int o = 0; o < a.w_bytes; o += 32768) bulk_g2s(smem_u32(wsm + o), a.wpk + o, (uint32_t)min(32768, a.w_bytes - o), bar_w);
            int it = 0; bool ok = true;
            for (int job = blockIdx.x; job < a.njobs && ok; job += gridDim.x) {
                const int txy = job % tiles, zci = (job / tiles) % a.nzc, n = job / (tiles * a.nzc);
                const int x0 = (txy % a.tiles_x) * 8, y0 = (txy / a.tiles_x) * 16;
                const int zb = zci * a.zc, ze = min(a.D, zb + a.zc), zlo = max(0, zb - 1), zhi = min(a.D - 1, ze);
                for (int zi = zlo; zi <= zhi && ok; zi++) for (int ki = 0; ki < a.nki; ki++) {
                    const int s = it % R, ph = (it / R) & 1;
                    if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, kWaitLimitR)) { raise_r(a, abort_flag, 1, it); ok = false; break; }
                    const uint32_t sb = smem_u32(stages + (size_t)s * a.stage_bytes), bar = bar_tma + 8 * s;
                    if (a.dbg & 16) { mbar_arrive(bar); it++; continue; }
                    mbar_expect_tx(bar, 5760u);
                    /* two 16-byte-wide planes (fp8: the halves of block ki; fp4: blocks 2 ki and 2 ki + 1), 18 rows of 10 voxels each */
                    tma_load_4d(sb, &map0, bar, (x0 - 1) * 16, y0 - 1, zi, BITS == 8 ? (n * a.nkb + ki) * 2 : n * a.nkb + 2 * ki);
                    it++;
                }
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issue ---------------- */
        bool ok = mbar_wait(bar_w, 0, abort_flag, kWaitLimitR);
        if (!ok && lane == 0) raise_r(a, abort_flag, 6, 0);
        tc_fence_after();
        const uint32_t wbase = smem_u32(wsm);
        const uint32_t a_hi = desc_hi(160), b_hi = desc_hi(128), b_lo0 = desc_lo(wbase, (uint32_t)a.nt * 16), idesc0 = BITS == 8 ? idesc_mxf8(a.nt, 0, 0) : idesc_mxf4(a.nt, 0, 0);
        if (ok && lane == 0) {
            /* the B scale factors of every (input block, dz) stage: copied to TMEM once */
            for (int st = 0; st < a.nst; st++) for (int q = 0; q < a.nquad; q++)
                utccp_32x128b(tmem + kSfbBase + (st * a.nquad + q) * 4, smem_desc(wbase + st * a.w_stage_bytes + 9 * a.nt * 32 + q * 512, 0, 128));
        }
        __syncwarp();
        int it = 0, pc_base = 0;
        long long t_tma = 0, t_sf = 0, t_acce = 0, t_issue = 0, t_all0 = clock64(), t_f = 0, t_c1 = 0, t_c2 = 0, t_u = 0;
        for (int job = blockIdx.x; job < a.njobs && ok; job += gridDim.x) {
            const int zci = (job / tiles) % a.nzc;
            const int zb = zci * a.zc, ze = min(a.D, zb + a.zc), zlo = max(0, zb - 1), zhi = min(a.D - 1, ze);
            for (int zi = zlo; zi <= zhi && ok; zi++) for (int ki = 0; ki < a.nki && ok; ki++) {
                const int s = it % R, ph = (it / R) & 1;
                long long c0 = clock64();
                if (!mbar_wait(bar_tma + 8 * s, ph, abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 2, it); ok = false; break; }
                long long c1 = clock64(); t_tma += c1 - c0;
                if (!mbar_wait(bar_sf + 8 * s, ph, abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 3, it); ok = false; break; }
                c0 = clock64(); t_sf += c0 - c1;
                tc_fence_after();
                { const long long cf = clock64(); t_f += cf - c0; }
                const uint32_t sb = smem_u32(stages + (size_t)s * a.stage_bytes);
                const uint32_t sfa_t = tmem + kSfaBase + (it & 1) * 20;
                { const long long cu = clock64();
                if (lane == 0 && !(a.dbg & 32)) for (int q = 0; q < a.nquad; q++) utccp_32x128b(sfa_t + 4 * q, smem_desc(sb + a.offSFA + 512 * q, 0, 128));
                t_u += clock64() - cu; }
                for (int dz = 2; dz >= 0 && ok; dz--) {
                    const int z = zi + 1 - dz;
                    if (z < zb || z >= ze) continue;
                    const int pcz = pc_base + z - zb, buf = pcz % NA;
                    const bool first = ki == 0 && zi == max(z - 1, 0);
                    if (first) {   /* this plane's buffer must have been drained by the epilogue of the plane NA planes back */
                        const long long c2 = clock64();
                        if (!mbar_wait(bar_acce + 8 * buf, ((pcz / NA) & 1) ^ 1, abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 7, it); ok = false; break; }
                        tc_fence_after();
                        t_acce += clock64() - c2;
                    }
                    if (lane == 0 && !(a.dbg & 1)) {
                        const int st = ki * 3 + dz;
                        issue_items<BITS, 9, true>(tmem + buf * a.nt, desc_lo(sb, 2880), a_hi, b_lo0 + (uint32_t)(st * a.w_stage_bytes) / 16, b_hi, (uint32_t)a.nt * 2, 0,
                                                   idesc0, sfa_t, tmem + kSfbBase + st * a.nquad * 4, first, 9);
                    }
                }
                if (ok && lane == 0) {
                    const long long cc = clock64();
                    if (!(a.dbg & 128)) umma_commit(bar_empty + 8 * s); else mbar_arrive(bar_empty + 8 * s);
                    t_c1 += clock64() - cc;
                    if (ki == a.nki - 1) {   /* planes whose last input plane this was are complete */
                        const long long cd = clock64();
                        for (int z = zi - 1; z <= zi; z++) if (z >= zb && z < ze && min(z + 1, a.D - 1) == zi) { if (!(a.dbg & 128)) umma_commit(bar_accf + 8 * ((pc_base + z - zb) % NA)); else mbar_arrive(bar_accf + 8 * ((pc_base + z - zb) % NA)); }
                        t_c2 += clock64() - cd;
                    }
                }
                __syncwarp();
                t_issue += clock64() - c0;
                it++;
            }
            pc_base += ze - zb;
        }
        if (a.prof && blockIdx.x == 0 && lane == 0) { a.prof[0] = clock64() - t_all0; a.prof[1] = t_tma; a.prof[2] = t_sf; a.prof[3] = t_acce; a.prof[4] = t_issue; a.prof[5] = it; a.prof[11] = t_f; a.prof[12] = t_c1; a.prof[13] = t_c2; a.prof[14] = t_u; }
    } else if (warp < 6) {
        /* ---------------- scale gather: warp w takes the stages with it % 4 == w ---------------- */
        const int sfw = warp - 2;
        int it = 0; bool ok = true;
        for (int job = blockIdx.x; job < a.njobs && ok; job += gridDim.x) {
            const int txy = job % tiles, zci = (job / tiles) % a.nzc, n = job / (tiles * a.nzc);
            const int x0 = (txy % a.tiles_x) * 8, y0 = (txy / a.tiles_x) * 16;
            const int zb = zci * a.zc, ze = min(a.D, zb + a.zc), zlo = max(0, zb - 1), zhi = min(a.D - 1, ze);
            for (int zi = zlo; zi <= zhi && ok; zi++) for (int ki = 0; ki < a.nki; ki++, it++) {
                if ((it & 3) != sfw) continue;
                const int s = it % R, ph = (it / R) & 1;
                if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 4, it); ok = false; break; }
                uint32_t *sfa = (uint32_t *)(stages + (size_t)s * a.stage_bytes + a.offSFA);
                const uint8_t *sc0 = a.x_sc + ((size_t)n * a.nkb + (BITS == 8 ? ki : 2 * ki)) * S + (size_t)zi * a.H * a.W;
                const bool has1 = BITS == 4 && 2 * ki + 1 < a.nkb;
                if (!(a.dbg & 2))
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int r = q * 32 + lane, oy = y0 + (r >> 3), ox = x0 + (r & 7);
                    uint32_t wq[5] = {0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu};
#pragma unroll
                    for (int j = 0; j < 9; j++) {
                        const int iy = oy + j / 3 - 1, ix = ox + j % 3 - 1;
                        const bool in = iy >= 0 && iy < a.H && ix >= 0 && ix < a.W;
                        const size_t vox = (size_t)iy * a.W + ix;
                        if (BITS == 8) {
                            const unsigned b = in ? __ldg(sc0 + vox) : 127u;
                            wq[j >> 2] = (wq[j >> 2] & ~(0xffu << (8 * (j & 3)))) | (b << (8 * (j & 3)));
                        } else {
                            const unsigned b0 = in ? __ldg(sc0 + vox) : 127u, b1 = (in && has1) ? __ldg(sc0 + S + vox) : 127u;
                            const unsigned h = b0 | (b1 << 8);
                            wq[j >> 1] = (wq[j >> 1] & ~(0xffffu << (16 * (j & 1)))) | (h << (16 * (j & 1)));
                        }
                    }
#pragma unroll
                    for (int qd = 0; qd < (BITS == 8 ? 3 : 5); qd++) sfa[qd * 128 + lane * 4 + q] = wq[qd];
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sf + 8 * s);
            }
        }
    } else {
        /* ---------------- epilogue: one output plane of one tile at a time ---------------- */
        const int q4 = warp & 3, r = q4 * 32 + lane, ry = r >> 3, rx = r & 7;
        const int nchunk = a.nt >> 5, T = a.D * tiles, e128 = (int)threadIdx.x - 192;
        int pc = 0; bool dead = false;
        long long e_wait = 0, e_all0 = clock64();
        for (int job = blockIdx.x; job < a.njobs; job += gridDim.x) {
            const int txy = job % tiles, zci = (job / tiles) % a.nzc, n = job / (tiles * a.nzc);
            const int ox = (txy % a.tiles_x) * 8 + rx, oy = (txy / a.tiles_x) * 16 + ry;
            const bool row_ok = oy < a.H && ox < a.W;
            const int zb = zci * a.zc, ze = min(a.D, zb + a.zc);
            for (int z = zb; z < ze; z++, pc++) {
                const int buf = pc % NA;
                double *sp = spart + (pc & 1) * 512;
                const long long e0 = clock64();
                if (!dead && !mbar_wait(bar_accf + 8 * buf, (pc / NA) & 1, abort_flag, kWaitLimitR)) { raise_r(a, abort_flag, 5, pc); dead = true; }
                e_wait += clock64() - e0;
                if (!dead) {
                    tc_fence_after();
                    uint32_t rr[2][32];
                    if (!(a.dbg & 64)) tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(buf * a.nt), rr[0]);
                    if (nchunk > 1 && !(a.dbg & 64)) tmem_ld32(tmem + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(buf * a.nt + 32), rr[1]);
                    tmem_ld_wait();
                    tc_fence_before();
                    mbar_arrive(bar_acce + 8 * buf);       /* the buffer is free as soon as it is in registers */
#pragma unroll
                    for (int jc = 0; jc < 2; jc++) if (jc < nchunk) {
                        float v[32];
#pragma unroll
                        for (int k = 0; k < 32; k++) v[k] = __uint_as_float(rr[jc][k]);
                        if (!(a.dbg & 4)) epi_chunk(a.e, n, z, oy, ox, row_ok, jc, v);
                        if (a.e.part && !(a.dbg & 8)) {
                            double s1, s2;
                            epi_sums(v, row_ok, lane, s1, s2);
                            sp[((q4 * 2 + jc) * 32 + lane) * 2] = s1; sp[((q4 * 2 + jc) * 32 + lane) * 2 + 1] = s2;
                        }
                    }
                }
                if (a.e.part) {
                    /* reached by all 128 epilogue threads the same number of times, dead or not */
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (!dead && !*abort_flag && e128 < nchunk * 32) {
                        const int jc = e128 >> 5, l = e128 & 31;
                        double t1 = 0.0, t2 = 0.0;
#pragma unroll
                        for (int qq = 0; qq < 4; qq++) { t1 += sp[((qq * 2 + jc) * 32 + l) * 2]; t2 += sp[((qq * 2 + jc) * 32 + l) * 2 + 1]; }
                        double *dst = a.e.part + (((size_t)n * T + (size_t)z * tiles + txy) * a.e.cop + jc * 32 + l) * 2;
                        dst[0] = t1; dst[1] = t2;
                    }
                }
            }
        }
        if (a.prof && blockIdx.x == 0 && threadIdx.x == 192) { a.prof[8] = e_wait; a.prof[9] = clock64() - e_all0; a.prof[10] = pc; }
    }
    /* ---------------- teardown ---------------- */
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && warp == 0 && lane == 0) {
        for (int s = 0; s < R; s++) { const long long t0 = clock64(); while (!mbar_try(bar_tma + 8 * s, 0) && !mbar_try(bar_tma + 8 * s, 1) && clock64() - t0 < 20000000ll) { } }
        { const long long t0 = clock64(); while (!mbar_try(bar_w, 0) && clock64() - t0 < 20000000ll) { } }
    }
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, kTmemColsR); }
}

}   // namespace

/* 1 when the z-marching kernel can run this conv: 3^3, one column tile of at most 64 channels, weight image and B scales resident */
int umx_conv_r_fits(const umx_conv *c) {
    if (c->kind != UMX_CONV3 || c->ntiles_n != 1 || c->nt > 64) return 0;
    if ((size_t)c->nst * c->w_stage_bytes > 128 * 1024) return 0;
    if (c->nst * c->nquad * 4 > 512 - kSfbBase) return 0;
    return 1;
}
int umx_conv_fwd_r(const umx_conv *c, const void *x, const CUtensorMap *m0, int N, int D, int H, int W, const EpiArgs &e) {
    ConvRArgs a; memset(&a, 0, sizeof a);
    a.N = N; a.D = D; a.H = H; a.W = W; a.nkb = c->nkb; a.nki = c->nki; a.bits = c->bits; a.nt = c->nt;
    a.tiles_x = (W + 7) / 8; a.tiles_y = (H + 15) / 16;
    a.w_bytes = c->nst * c->w_stage_bytes; a.w_stage_bytes = c->w_stage_bytes; a.nst = c->nst; a.ipq = c->ipq; a.nquad = c->nquad; a.nacc = 4;
    a.offSFA = 2880 * 2;
    a.stage_bytes = (a.offSFA + c->nquad * 512 + 1023) & ~1023;
    a.off_w = 1024 + 8192; a.off_ring = (a.off_w + a.w_bytes + 1023) & ~1023;
    int dev = 0, sms = 148; cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int room = 227 * 1024 - a.off_ring;
    a.ring = room / a.stage_bytes; if (a.ring > 10) a.ring = 10;
    if (a.ring < 3) { umx_latch_msg("umx_conv_fwd: no room for the stage ring beside the resident weights"); return -1; }
    /* z chunk: the longest of 16, 12, 8, 6, 4, 3, 2, 1 planes that keeps the static round-robin over the blocks at least 93 % balanced */
    const int tiles = a.tiles_x * a.tiles_y; const int cand[8] = {16, 12, 8, 6, 4, 3, 2, 1};
    int best = 1; double best_eff = -1;
    for (int i = 0; i < 8; i++) {
        const int zc = cand[i] < D ? cand[i] : D, nzc = (D + zc - 1) / zc; const long jobs = (long)N * nzc * tiles;
        const long g = jobs < sms ? jobs : sms, rounds = (jobs + g - 1) / g;
        const double eff = (double)jobs / (double)(rounds * g) * (jobs < sms ? (double)jobs / sms : 1.0);
        if (eff >= 0.93) { best = zc; best_eff = eff; break; }
        if (eff > best_eff) { best_eff = eff; best = zc; }
    }
    a.zc = best; a.nzc = (D + a.zc - 1) / a.zc; a.njobs = N * a.nzc * tiles;
    const size_t S = (size_t)D * H * W;
    a.x_sc = (const uint8_t *)x + (size_t)N * c->nkb * S * (c->bits == 8 ? 32 : 16);   /* the scale plane follows the codes in either layout */
    a.wpk = c->wpk; a.e = e; a.err = umx_errflag();
    a.prof = nullptr;
    if (getenv("UMX_PROF")) { a.prof = (long long *)umx_ws(7, 256); cudaMemset(a.prof, 0, 256); }
    { const char *ev = getenv("UMX_DBG"); a.dbg = ev ? atoi(ev) : 0; if (ev && getenv("UMX_ZC")) { a.zc = atoi(getenv("UMX_ZC")); a.nzc = (D + a.zc - 1) / a.zc; a.njobs = N * a.nzc * tiles; } }
    if (!a.err) return -1;
    const size_t smem = (size_t)a.off_ring + (size_t)a.ring * a.stage_bytes;
    static int attr_set[16];
    if (!attr_set[dev & 15]) {
        cudaError_t er = cudaFuncSetAttribute(conv_mxr_k<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (er == cudaSuccess) er = cudaFuncSetAttribute(conv_mxr_k<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (er != cudaSuccess) { umx_latch("umx_conv_fwd: shared memory attribute", er); return -1; }
        attr_set[dev & 15] = 1;
    }
    const int grid = a.njobs < sms ? a.njobs : sms;
    if (c->bits == 8) conv_mxr_k<8><<<grid, kThreadsR, smem>>>(*m0, a); else conv_mxr_k<4><<<grid, kThreadsR, smem>>>(*m0, a);
    if (a.prof) { long long h[16]; cudaMemcpy(h, a.prof, 128, cudaMemcpyDeviceToHost); fprintf(stderr, "prof: mma total %lld tma %lld sf %lld acce %lld issue %lld stages %lld | epi wait %lld total %lld planes %lld | grid %d jobs %d zc %d ring %d | fence %lld commit1 %lld commit2 %lld utccp %lld\n", h[0], h[1], h[2], h[3], h[4], h[5], h[8], h[9], h[10], grid, a.njobs, a.zc, a.ring, h[11], h[12], h[13], h[14]); }
    return 0;
}
