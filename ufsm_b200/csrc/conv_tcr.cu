/* 3^3 MX conv forward, persistent z-marching kernel for layers whose prepared weights fit in shared memory (up to 64 output
   channels: the 32- and 64-channel levels, which hold most of the network's voxels).

   A block keeps the whole weight image (all taps, all input blocks) in shared memory and the B scale factors in TMEM, and owns a
   contiguous piece of the list of (sample, y-x tile, z) output planes; a piece is one to three runs along z.  Inside a run the
   block marches along z.  Each input plane (one TMA halo load of the codes and one of the scale bytes per input block) is the A
   operand of nine MMAs, one per (dy, dx); the three dz taps that use the same shifted view are stacked along N: B rows are
   (dz, channel), and the accumulators of the three output planes z + 1, z, z - 1 sit in consecutive TMEM slots (slot = ring
   position of the plane, descending), so one MMA of N = 3 x channels updates all three.  When that window wraps around the slot
   ring a stage issues two groups of MMAs.


   What bounds this kernel.  An M = 128, N = 96, K = 32 MMA occupies the tensor pipe for 56 clocks (48 of arithmetic; its 4 KB A tile and
   3 KB B tile exceed what shared memory delivers in 48), and one thread cannot issue tcgen05.mma faster than one per 54 clocks whatever
   N is; a scale copy or a commit costs the thread that issues it another 30 to 130 clocks while it takes next to nothing from the
   pipe.  So the MMA thread issues nothing but MMAs and one commit per stage, and every role's per-stage program is kept short: (1) the
   producer thread tracks slots and parities incrementally (no division) and hands the MMA thread a record with everything
   precomputed: TMEM addresses, the N field of the instruction descriptor, B descriptor and B scale addresses, the barriers to wait
   for; (2) the MMA thread's stage is three PTX blocks of three MMAs whose operands are a record field plus an immediate; (3)
   accumulators are never "fresh": the epilogue zeroes a slot after reading it, so every MMA accumulates; (4) the A scale factors are
   gathered from a TMA-staged window in shared memory with no bounds logic (voxels outside the volume arrive as zero codes with scale
   byte 0) and copied to TMEM by the scale warps themselves, whose commit is what the MMA thread waits for; (5) the MMA thread's single
   commit per stage lands on the stage's `empty` barrier; the scale warps, which wait for that barrier anyway before they reuse a TMEM
   scale buffer, pass the completion of output planes on to the epilogue's accumulator-full barriers; (6) two blocks share a
   multiprocessor when the weights are small enough: one block's waits are the other's issue time.

   Roles (256 threads): warp 0 lane 0 producer (records + TMA), warp 1 lane 0 MMA issue (the warp allocates TMEM), warps 2-3 scale
   layout, scale copies and completion relay (alternate stages), warps 4-7 epilogue.  All waits are bounded as in conv_mx_k. */
#include "conv_epi.cuh"
#include "tc_ptx.cuh"
#include <stdlib.h>
#include <string.h>


#define UMX_STR_(x) #x
#define UMX_STR(x) UMX_STR_(x)
/* operand numbers of the PTX blocks below: the five immediates of a tap follow one another */
#define UMX_ADD1(o) UMX_CAT(UMX_N1_, o)
#define UMX_ADD2(o) UMX_CAT(UMX_N2_, o)
#define UMX_ADD3(o) UMX_CAT(UMX_N3_, o)
#define UMX_ADD4(o) UMX_CAT(UMX_N4_, o)
#define UMX_CAT_(a, b) a##b
#define UMX_CAT(a, b) UMX_CAT_(a, b)
#define UMX_N1_8 9
#define UMX_N2_8 10
#define UMX_N3_8 11
#define UMX_N4_8 12
#define UMX_N1_13 14
#define UMX_N2_13 15
#define UMX_N3_13 16
#define UMX_N4_13 17
#define UMX_N1_18 19
#define UMX_N2_18 20
#define UMX_N3_18 21
#define UMX_N4_18 22

namespace {

constexpr int kThreadsR = 256;
constexpr int kMaxSlots = 12;
constexpr long long kWaitLimitR = 4000000000ll;

struct ConvRArgs {
    int N, D, H, W, nkb, nki, bits, nt;
    int tiles_x, tiles, ncol, gcol;              /* column tiles of nt channels; blocks per column tile */
    long long units;                             /* N x tiles x D output planes of one tile, split evenly over the grid */
    int ring, stage_bytes, offSW, offSFA;
    int w_bytes, w_codes, nquad, gt, goff1, goff2, nslot;
    int tmem_cols, sfa_base, sfa_cols, sfb_base; /* TMEM: accumulator slots from 0, two A scale buffers, B scales */
    int off_rec, off_bias, off_stage, off_w, off_ring;   /* off_stage: 2 KB per epilogue warp and 32-channel chunk, the fp16 output rows on their way to coalesced stores */
    int fast_h16;                                /* output is the fp16 blocked tensor of a plain conv: the short epilogue */
    /* InstanceNorm statistics taken in that epilogue (coef != NULL): fp64 sums of the stored fp16 values and of their squares, written once per
       sample and block into part [n][gcol][cop][2]; the last block of a column tile to finish adds the blocks' entries in block order and
       turns them into coefficients (a, b) per (sample, channel) */
    double *part; float *coef; const float *gamma, *beta; float eps; int cop, off_red;
    const uint8_t *wr;
    EpiArgs e;
    int *err;
};

/* what the MMA thread does for one stage; written by the producer thread */
struct StageRec {
    uint32_t d1, idn1, bb1, sfb1;      /* first group: TMEM accumulator address, instruction descriptor with N, B descriptor low word of tap 0, B scale address */
    uint32_t d2, idn2, bb2, sfb2;      /* second group when the window wraps (idn2 = 0: none) */
    uint32_t wait0, wait1;             /* accumulator-empty barriers to pass first: address | parity << 31 (0: none) */
    uint32_t commit0, commit1;         /* accumulator-full barriers to commit after the stage (0: none) */
    uint32_t last, pad[3];
};
static_assert(sizeof(StageRec) == 64, "stage record is 64 bytes");

/* a wait gave up (its own limit, or another role's abort flag): the first to get here names the block; every role of that block then leaves
   where it stood (stage, barrier, parity), which the host prints */
__device__ __forceinline__ void raise_r(const ConvRArgs &a, volatile int *abort_flag, int code, int stage, uint32_t bar_off = 0, uint32_t parity = 0) {
    if (atomicCAS(a.err, 0, code) == 0) { a.err[1] = (int)blockIdx.x; a.err[2] = stage; a.err[3] = (int)threadIdx.x; __threadfence(); }
    if (((volatile int *)a.err)[1] == (int)blockIdx.x && code < 8) { int *d = a.err + 16 + 4 * code; d[0] = stage; d[1] = (int)bar_off; d[2] = (int)parity; d[3] = 1; }
    *abort_flag = 1;
    __threadfence_block();
}
/* Three of the nine (dy, dx) MMAs of a group in one PTX block: tap j reads the A view a_lo + (j / 3) * 10 + j % 3 and the B image
   b_lo + j * BSTEP; the scale sets come in quads of four (fp8) or two (fp4) taps.  Everything that depends on the tap is an immediate, so
   between two MMAs the issuing thread runs a handful of independent integer instructions that the assembler is free to hoist: a lone
   thread runs dependent scalar code at four to five clocks an instruction, and every clock it spends between MMAs the tensor pipe idles. */
template <int BITS, int BSTEP, int SFBQ, int J0>
__device__ __forceinline__ void mma3(uint32_t d, uint32_t idn, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t sfa, uint32_t sfb) {
    constexpr int IPQ = BITS == 8 ? 4 : 2;
#define UMX_TAP(j) "n"(((j) / 3) * 10 + (j) % 3), "n"((j) * BSTEP), "n"(((((j) % IPQ) * (4 / IPQ)) << 4) | ((((j) % IPQ) * (4 / IPQ)) << 29)), "n"(4 * ((j) / IPQ)), "n"(((j) / IPQ) * SFBQ)
#define UMX_MMA_TEXT(KIND, o)                                                                                        \
    "add.u32 ta, %2, %" #o ";\n\tmov.b64 da, {ta, %3};\n\t"                                                         \
    "add.u32 tb, %4, %" UMX_STR(UMX_ADD1(o)) ";\n\tmov.b64 db, {tb, %5};\n\t"                                      \
    "or.b32 ti, %1, %" UMX_STR(UMX_ADD2(o)) ";\n\t"                                                                   \
    "add.u32 sa, %6, %" UMX_STR(UMX_ADD3(o)) ";\n\tadd.u32 sb, %7, %" UMX_STR(UMX_ADD4(o)) ";\n\t"                  \
    "tcgen05.mma.cta_group::1.kind::" KIND " [%0], da, db, ti, [sa], [sb], p;\n\t"
    if constexpr (BITS == 8) {
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 ta, tb, ti, sa, sb;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %1, 0;\n\t"
                     UMX_MMA_TEXT("mxf8f6f4.block_scale", 8) UMX_MMA_TEXT("mxf8f6f4.block_scale", 13) UMX_MMA_TEXT("mxf8f6f4.block_scale", 18) "}"
                     ::"r"(d), "r"(idn), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(sfa), "r"(sfb), UMX_TAP(J0), UMX_TAP(J0 + 1), UMX_TAP(J0 + 2) : "memory");
    } else {
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b32 ta, tb, ti, sa, sb;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %1, 0;\n\t"
                     UMX_MMA_TEXT("mxf4.block_scale.scale_vec::2X", 8) UMX_MMA_TEXT("mxf4.block_scale.scale_vec::2X", 13) UMX_MMA_TEXT("mxf4.block_scale.scale_vec::2X", 18) "}"
                     ::"r"(d), "r"(idn), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(sfa), "r"(sfb), UMX_TAP(J0), UMX_TAP(J0 + 1), UMX_TAP(J0 + 2) : "memory");
    }
#undef UMX_TAP
#undef UMX_MMA_TEXT
}
/* the nine (dy, dx) MMAs of one group into the accumulator window at d (idn: the instruction descriptor with the window's N) */
template <int BITS, int NT> __device__ __forceinline__ void issue_group(uint32_t d, uint32_t idn, uint32_t bb, uint32_t sfb, uint32_t a_lo, uint32_t a_hi, uint32_t b_hi, uint32_t sfa_t) {
    constexpr int BSTEP = 2 * 3 * NT, SFBQ = 4 * ((3 * NT + 127) / 128 + (2 * NT + 127) / 128 + (NT + 127) / 128);
    mma3<BITS, BSTEP, SFBQ, 0>(d, idn, a_lo, a_hi, bb, b_hi, sfa_t, sfb);
    mma3<BITS, BSTEP, SFBQ, 3>(d, idn, a_lo, a_hi, bb, b_hi, sfa_t, sfb);
    mma3<BITS, BSTEP, SFBQ, 6>(d, idn, a_lo, a_hi, bb, b_hi, sfa_t, sfb);
}
/* the block's piece of the plane list, u in [u0, u1) with u = (sample * tiles + tile) * D + z, cut into runs along z */
struct Piece { long long u, u1; };
__device__ __forceinline__ Piece piece_of_block(const ConvRArgs &a) {
    const long long b = (long long)(blockIdx.x % a.gcol);      /* blocks [k gcol, (k + 1) gcol) share column tile k and split the plane list */
    Piece p; p.u = a.units * b / (long long)a.gcol; p.u1 = a.units * (b + 1) / (long long)a.gcol; return p;
}
struct Run { int n, txy, zb, ze; };
__device__ __forceinline__ Run next_run(const ConvRArgs &a, Piece &p) {
    const long long col = p.u / a.D; Run r;
    r.zb = (int)(p.u - col * a.D); r.ze = (int)min((long long)a.D, (long long)r.zb + (p.u1 - p.u));
    r.n = (int)(col / a.tiles); r.txy = (int)(col - (long long)r.n * a.tiles);
    p.u += r.ze - r.zb;
    return r;
}

/* ---- InstanceNorm sums in the epilogue.  They are taken in fp64 where the warp re-reads its staged fp16 rows for the coalesced store:
   there a lane holds eight channels of the four voxels of one x, and it keeps one (sum, sum of squares) pair per channel for the whole
   sample.  A stored fp16 value and its square are exact in fp64 and so are their sums over a sample of any realistic size, so neither
   the order of the planes nor their partition over blocks changes a bit, and the coefficients equal those of the separate fp64 pass
   (in_part_k).  Per sample and block the eight lanes that hold the same channels are added with shuffles, then the four warps, then (by
   the block that finishes last, in block order) the blocks. ---- */
/* the sum over the eight lanes x = 0..7 that hold this lane's channels (partners p4, p2, p1: the lanes at x ^ 4, x ^ 2, x ^ 1) */
__device__ __forceinline__ double lanes8_sum(double v, int p4, int p2, int p1) {
    v += __shfl_sync(0xffffffffu, v, p4);
    v += __shfl_sync(0xffffffffu, v, p2);
    return v + __shfl_sync(0xffffffffu, v, p1);
}

__device__ unsigned g_conv_tickets[64];      /* one per column tile; the block that draws the last ticket finalises and resets it */

/* NCH: 32-channel chunks of the column tile (1: two blocks per multiprocessor and at most 128 registers; 2: one block, more registers);
   STATS: the epilogue also takes the InstanceNorm sums */
template <int BITS, int NCH, bool STATS>
__global__ void __launch_bounds__(kThreadsR, NCH == 1 ? 2 : 1) conv_mxr_k(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap maps, const ConvRArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint64_t *bars = (uint64_t *)smem_raw;
    uint32_t *tmem_slot = (uint32_t *)(smem_raw + 768);
    volatile int *abort_flag = (volatile int *)(smem_raw + 772);
    StageRec *recs = (StageRec *)(smem_raw + a.off_rec);
    float *bias_s = (float *)(smem_raw + a.off_bias);
    uint8_t *wsm = smem_raw + a.off_w, *stages = smem_raw + a.off_ring;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = a.ring, NS = a.nslot;
    /* barriers: tma[R] (codes + scale window landed), sf[R] (A scales laid out), empty[R], accumulator full / empty per slot, weights */
    const uint32_t bar_tma = smem_u32(bars), bar_sf = bar_tma + 8 * R, bar_empty = bar_tma + 16 * R, bar_accf = bar_tma + 24 * R, bar_acce = bar_accf + 8 * kMaxSlots, bar_w = bar_acce + 8 * kMaxSlots, bar_red = bar_w + 8;
    constexpr int NQ = BITS == 8 ? 3 : 5;                  /* A scale quads per stage */
    constexpr uint32_t TX = 5760u + (BITS == 8 ? 576u : 1152u);

    if (threadIdx.x == 0) {
        for (int i = 0; i < R; i++) { mbar_init(bar_tma + 8 * i, 1); mbar_init(bar_sf + 8 * i, 1); mbar_init(bar_empty + 8 * i, 1); }
        for (int i = 0; i < kMaxSlots; i++) { mbar_init(bar_accf + 8 * i, 1); mbar_init(bar_acce + 8 * i, 4); }
        mbar_init(bar_w, 1); mbar_init(bar_red, 128);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    const int ctile = (int)blockIdx.x / a.gcol;
    if ((int)threadIdx.x < a.nt) bias_s[threadIdx.x] = a.e.bias[ctile * a.nt + threadIdx.x];
    pdl_trigger();
    if (threadIdx.x == 0) {
        /* the weight image is a constant of the layer: it may load while the previous kernel of the stream is still running */
        mbar_expect_tx(bar_w, (uint32_t)a.w_bytes);
        for (int o = 0; o < a.w_bytes; o += 32768) bulk_g2s(smem_u32(wsm + o), a.wr + (size_t)ctile * a.w_bytes + o, (uint32_t)min(32768, a.w_bytes - o), bar_w);
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), (uint32_t)a.tmem_cols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    Piece piece = piece_of_block(a);

    if (warp == 0) {
        /* ---------------- producer: stage records and TMA ---------------- */
        if (lane == 0) {
            tma_prefetch_desc(&map0); tma_prefetch_desc(&maps);
            pdl_wait();      /* the only role that reads activations from global memory; every other role's data comes through this thread's loads,
                                so the weight load, the B scale copies and the zeroing of the accumulators overlap the previous kernel */
            const uint32_t nt = (uint32_t)a.nt, bstep9 = 9u * 2u * 3u * nt;            /* B descriptor step of one input block: nine taps of two halves of 3 nt rows */
            const uint32_t b_lo0 = desc_lo(smem_u32(wsm), 3u * nt * 16u);
            const uint32_t idesc_b = (BITS == 8 ? idesc_mxf8(0, 0, 0) : idesc_mxf4(0, 0, 0)), ntn = (nt >> 3) << 17;
            const uint32_t sfb_t0 = tmem + (uint32_t)a.sfb_base, sfb_per_ki = (uint32_t)(a.nquad * a.gt * 4);
            int s = 0, ph = 0, it = 0; bool ok = true;
            int pos = NS - 1; uint32_t wp = 1u;           /* ring position and wrap parity of the newest plane started so far */
            while (piece.u < piece.u1 && ok) {
                const Run rn = next_run(a, piece);
                const bool last_run = piece.u >= piece.u1;
                const int x0 = (rn.txy % a.tiles_x) * 8, y0 = (rn.txy / a.tiles_x) * 16;
                const int zb = rn.zb, ze = rn.ze, zlo = max(0, zb - 1), zhi = min(a.D - 1, ze);
                const int xa = ((x0 - 1) >> 4) << 4;             /* 16-aligned start of the 32-byte scale window (x0 = 0: -16, read as zeros) */
                const int cx = (x0 - 1) * 16, cy = y0 - 1;
                const int pl0 = BITS == 8 ? rn.n * a.nkb * 2 : rn.n * a.nkb, pls = rn.n * a.nkb;
                for (int zi = zlo; zi <= zhi && ok; zi++) {
                    /* output planes fed by input plane zi: z = zi + 1 - dz, newest first */
                    const int newest = min(zi + 1, ze - 1), oldest = max(zi - 1, zb), cnt = newest - oldest + 1, dzf = zi + 1 - newest;
                    const int nfresh = zi == zlo ? cnt : (newest == zi + 1 ? 1 : 0);
                    uint32_t w0 = 0, w1 = 0;
                    for (int f = 0; f < nfresh; f++) {
                        if (++pos == NS) { pos = 0; wp ^= 1u; }
                        const uint32_t wf = (bar_acce + 8u * (uint32_t)(NS - 1 - pos)) | (wp << 31);
                        if (f == 0) w0 = wf; else w1 = wf;
                    }
                    const int slot = NS - 1 - pos, n1 = min(cnt, NS - slot), n2 = cnt - n1;
                    const uint32_t g1 = (uint32_t)(dzf == 0 ? 0 : dzf == 1 ? a.goff1 : a.goff2), g2 = (uint32_t)(dzf + n1 == 1 ? a.goff1 : a.goff2);
                    for (int ki = 0; ki < a.nki; ki++) {
                        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, kWaitLimitR)) { raise_r(a, abort_flag, 1, it, bar_empty + 8 * s - bar_tma, ph ^ 1); ok = false; break; }
                        const bool kl = ki == a.nki - 1;
                        const uint32_t bk = b_lo0 + (uint32_t)ki * bstep9, sk = sfb_t0 + (uint32_t)ki * sfb_per_ki;
                        uint4 *r = (uint4 *)(recs + s);
                        r[0] = make_uint4(tmem + (uint32_t)slot * nt, idesc_b | (uint32_t)n1 * ntn, bk + (uint32_t)dzf * nt, sk + g1);
                        r[1] = make_uint4(tmem, n2 ? (idesc_b | (uint32_t)n2 * ntn) : 0u, bk + (uint32_t)(dzf + n1) * nt, sk + g2);
                        r[2] = make_uint4(ki == 0 ? w0 : 0u, ki == 0 ? w1 : 0u, 0u, 0u);
                        r[3] = make_uint4((last_run && zi == zhi && kl) ? 1u : 0u, 0u, 0u, 0u);
                        const uint32_t sb = smem_u32(stages + (size_t)s * a.stage_bytes), bar = bar_tma + 8 * s;
                        mbar_expect_tx(bar, TX);
                        /* codes: two 16-byte-wide planes (fp8: the halves of block ki; fp4: blocks 2 ki and 2 ki + 1), 18 rows of 10 voxels;
                           scale bytes: 18 rows of a 32-byte window per block */
                        tma_load_4d(sb, &map0, bar, cx, cy, zi, pl0 + 2 * ki);
                        tma_load_4d(sb + a.offSW, &maps, bar, xa, cy, zi, BITS == 8 ? pls + ki : pls + 2 * ki);
                        it++; if (++s == R) { s = 0; ph ^= 1; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        /* ---------------- MMA issue: one thread follows the records; a stage is straight-line code ---------------- */
        if (lane == 0) {
            bool ok = mbar_wait(bar_w, 0, abort_flag, kWaitLimitR);
            if (!ok) raise_r(a, abort_flag, 6, 0);
            tc_fence_after();
            const uint32_t wbase = smem_u32(wsm);
            const uint32_t a_hi = desc_hi(160), b_hi = desc_hi(128);
            const uint32_t sf_hi = desc_hi(128);                     /* scale blocks: 32 rows of 16 bytes, 8-row groups 128 bytes apart */
            if (ok) {
                /* the B scale factors of every (input block, tap quad, image, 128-row group): copied to TMEM once */
                const int nsf = a.nki * a.nquad * a.gt;
                for (int i = 0; i < nsf; i++) utccp_32x128b(tmem + a.sfb_base + i * 4, desc_make(desc_lo(wbase + a.w_codes + i * 512, 0), sf_hi));
            }
            const uint32_t a_lo0 = desc_lo(smem_u32(stages), 2880), a_step = (uint32_t)a.stage_bytes >> 4;
            const uint32_t sfa_t0 = tmem + (uint32_t)a.sfa_base, sfa_cols = (uint32_t)a.sfa_cols;
            int s = 0, ph = 0, it = 0;
            while (ok) {
                /* the stage's A scales are in TMEM (the scale warp's copies have completed); that warp passed the stage's load barrier before
                   it laid the scales out, so the codes have landed too */
                if (!mbar_wait(bar_sf + 8 * s, ph, abort_flag, kWaitLimitR)) { raise_r(a, abort_flag, 3, it, bar_sf + 8 * s - bar_tma, ph); break; }
                /* the whole record goes to registers before anything is committed: committing `empty` hands the stage, record included, back to the producer */
                const uint4 *r = (const uint4 *)(recs + s);
                const uint4 g1 = r[0], g2 = r[1], wc = r[2]; const uint32_t last = r[3].x;
                if (wc.x) {   /* a plane that starts here: its slot must have been read out and zeroed by the epilogue */
                    if (!mbar_wait(wc.x & 0x7fffffffu, wc.x >> 31, abort_flag, kWaitLimitR)) { raise_r(a, abort_flag, 7, it, (wc.x & 0x7fffffffu) - bar_tma, wc.x >> 31); break; }
                    if (wc.y && !mbar_wait(wc.y & 0x7fffffffu, wc.y >> 31, abort_flag, kWaitLimitR)) { raise_r(a, abort_flag, 7, it); break; }
                }
                tc_fence_after();
                const uint32_t a_lo = a_lo0 + (uint32_t)s * a_step, sfa_t = sfa_t0 + ((uint32_t)it & 1u) * sfa_cols;
                issue_group<BITS, 32 * NCH>(g1.x, g1.y, g1.z, g1.w, a_lo, a_hi, b_hi, sfa_t);
                if (g2.y) issue_group<BITS, 32 * NCH>(g2.x, g2.y, g2.z, g2.w, a_lo, a_hi, b_hi, sfa_t);
                /* the one commit of a stage: "stage s has been consumed".  The producer reuses the ring slot on it, the scale warps reuse the
                   stage's TMEM scale buffer on it and pass the news that output planes are complete on to the epilogue */
                umma_commit(bar_empty + 8 * s);
                it++; if (++s == R) { s = 0; ph ^= 1; }
                if (last) break;
            }
        }
    } else if (warp < 4) {
        /* ---------------- A scales: warp 2 takes the even stages, warp 3 the odd ones ----------------
           The TMA left 18 rows of a 32-byte window of scale bytes (two windows for fp4); row r of the tile needs, for tap (dy, dx), the
           byte at window row r / 8 + dy, column r % 8 + dx + (x0 - 1 - xa).  Four rows per lane (one per TMEM column of the quad).  The
           warp lays the nine shifted scale sets out in shared memory in the tcgen05.cp layout, and its lane 0 copies them to the TMEM
           scale buffer of the stage's parity and commits: the MMA thread waits for that commit and issues nothing but MMAs (a scale copy
           or a commit costs its issuing thread 30 to 130 clocks, an MMA of N = 96 occupies the tensor pipe for 56).

           The same warps relay completions.  The MMA thread commits once per stage, on the stage's `empty` barrier.  A scale warp
           waits for that barrier of stage it - 2 before it touches the TMEM scale buffer again (two buffers: the MMAs that read it must
           have completed), and it knows which output planes that stage completed (the plane below the input plane, and the volume's
           last plane with it), so it arrives on their accumulator-full barriers, which the epilogue waits on.  Both warps pass every
           barrier of both kinds in order, also for the stages the other warp works on: a warp that skipped a phase of a barrier could
           later take a wait for phase k + 2 as satisfied while the barrier is still in phase k + 1 (the parity reads the same). */
        const int sfw = warp - 2;
        const uint32_t sf_hi = desc_hi(128);
        const uint32_t sfa_t = tmem + (uint32_t)a.sfa_base + (uint32_t)sfw * (uint32_t)a.sfa_cols;      /* this warp's stages all have parity sfw */
        int it = 0, s = 0, ph = 0, s2 = 0, ph2 = 0; bool ok = true;
        int done = 0;                       /* output planes completed by all stages before the current one */
        int rel_first = 0, rel_n = 0;       /* the planes this warp's latest stage completes: relayed once that stage's commit has arrived */
        /* stage j = it - 2 has been consumed: pass its barrier; the warp that laid it out tells the epilogue about its planes */
        auto pass_empty = [&](bool mine) -> bool {
            if (!mbar_wait(bar_empty + 8 * s2, ph2, abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 2, it, bar_empty + 8 * s2 - bar_tma, ph2); return false; }
            if (++s2 == R) { s2 = 0; ph2 ^= 1; }
            if (mine && lane == 0) {
                for (int k = 0; k < rel_n; k++) mbar_arrive(bar_accf + 8u * (uint32_t)(NS - 1 - (rel_first + k) % NS));
            }
            return true;
        };
        while (piece.u < piece.u1 && ok) {
            const Run rn = next_run(a, piece);
            const int x0 = (rn.txy % a.tiles_x) * 8;
            const int zlo = max(0, rn.zb - 1), zhi = min(a.D - 1, rn.ze);
            const int xo = (x0 - 1) - (((x0 - 1) >> 4) << 4);     /* 7 or 15 */
            for (int zi = zlo; zi <= zhi && ok; zi++) {
                /* planes that the last stage of this input plane completes: the plane below it, and the volume's last plane with it */
                const int nc = (zi - 1 >= rn.zb ? 1 : 0) + ((zi == a.D - 1 && rn.ze == a.D) ? 1 : 0);
                for (int ki = 0; ki < a.nki && ok; ki++) {
                    const bool my = (it & 1) == sfw; const int cs = s, cph = ph;
                    if (!mbar_wait(bar_tma + 8 * cs, cph, abort_flag, kWaitLimitR)) { if (lane == 0) raise_r(a, abort_flag, 4, it, 8 * cs, cph); ok = false; break; }
                    const int ncs = ki == a.nki - 1 ? nc : 0;
                    if (!my) {
                        if (it >= 2 && !pass_empty(false)) { ok = false; break; }
                        done += ncs;
                        it++; if (++s == R) { s = 0; ph ^= 1; }
                        continue;
                    }
                    uint8_t *stg = stages + (size_t)cs * a.stage_bytes;
                    const uint8_t *sw = stg + a.offSW;
                    uint32_t *sfa = (uint32_t *)(stg + a.offSFA);
                    uint32_t wq[4][5];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int r = q * 32 + lane;
                        const uint8_t *p = sw + (r >> 3) * 32 + (r & 7) + xo;
#pragma unroll
                        for (int t = 0; t < 5; t++) wq[q][t] = 0u;
#pragma unroll
                        for (int j = 0; j < 9; j++) {
                            const uint32_t b0 = p[(j / 3) * 32 + j % 3];
                            if (BITS == 8) wq[q][j >> 2] |= b0 << (8 * (j & 3));
                            else { const uint32_t b1 = p[576 + (j / 3) * 32 + j % 3]; wq[q][j >> 1] |= (b0 | (b1 << 8)) << (16 * (j & 1)); }
                        }
                    }
                    /* quad qd: word (lane, column) = row 32 * column + lane; a lane's four columns are 16 contiguous bytes: one store */
#pragma unroll
                    for (int qd = 0; qd < NQ; qd++) *(uint4 *)(sfa + qd * 128 + lane * 4) = make_uint4(wq[0][qd], wq[1][qd], wq[2][qd], wq[3][qd]);
                    fence_proxy_async();
                    /* the scale sets are laid out; before they go to TMEM, the MMAs that read this buffer two stages ago must have completed */
                    if (it >= 2 && !pass_empty(true)) { ok = false; break; }
                    rel_first = done; rel_n = ncs;
                    done += ncs;
                    it++; if (++s == R) { s = 0; ph ^= 1; }
                    __syncwarp();
                    if (lane == 0) {
                        tc_fence_after();
                        const uint32_t src = desc_lo(smem_u32(sfa), 0);
#pragma unroll
                        for (int q = 0; q < NQ; q++) utccp_32x128b(sfa_t + 4 * q, desc_make(src + 32u * q, sf_hi));
                        umma_commit(bar_sf + 8 * cs);
                    }
                    __syncwarp();
                }
            }
        }
        /* the last two stages: their commits, and the planes of this warp's last stage */
        for (int k = (it >= 2 ? 2 : it); k > 0 && ok; k--) { const bool my = ((it - k) & 1) == sfw; if (!pass_empty(my)) ok = false; }
    } else {
        /* ---------------- epilogue: one output plane of one tile at a time ---------------- */
        const int q4 = warp & 3, r = q4 * 32 + lane, ry = r >> 3, rx = r & 7;
        constexpr int nchunk = NCH;
        const uint32_t tlane = tmem + ((uint32_t)(q4 * 32) << 16);
        /* every slot starts zeroed and released */
        for (int sl = 0; sl < NS; sl++) {
            for (int jc = 0; jc < nchunk; jc++) tmem_zero32(tlane + (uint32_t)(sl * a.nt + jc * 32));
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) for (int sl = 0; sl < NS; sl++) mbar_arrive(bar_acce + 8 * sl);     /* one arrival per warp: arrivals on one barrier serialise */
        int pcm = 0, pph = 0, pc = 0; bool dead = false;        /* pcm = plane count mod slots, pph = its wrap parity */
        const size_t S = (size_t)a.D * a.H * a.W;
        constexpr bool stats = STATS;
        const int et = (int)threadIdx.x - 128, bcol = (int)blockIdx.x % a.gcol;
        const int cl = (lane & 3) ^ ((lane >> 3) & 3);          /* the 16-byte chunk of a staged row this lane finds when it re-reads the rows for the coalesced store (see below) */
        /* statistics: x of this lane's voxels, the lanes that hold the same channels at x ^ 4, x ^ 2, x ^ 1, and the channel (of a 32-channel
           chunk) whose unit sum this lane ends up with */
        const int sx = lane >> 2;
        const int sp4 = 4 * (sx ^ 4) + (cl ^ (((sx ^ 4) >> 1) & 3)), sp2 = 4 * (sx ^ 2) + (cl ^ (((sx ^ 2) >> 1) & 3)), sp1 = 4 * (sx ^ 1) + (cl ^ (((sx ^ 1) >> 1) & 3));
        const int sch = 8 * cl + sx;                            /* the channel (of a 32-channel chunk) whose lane-group sum this lane writes out */
        /* this lane's channels 8 cl .. 8 cl + 7 of each chunk: sums and sums of squares of the sample in progress */
        double dsum[STATS ? NCH : 1][8], dsq[STATS ? NCH : 1][8];
        if (STATS) {
#pragma unroll
            for (int k = 0; k < NCH; k++)
#pragma unroll
                for (int t = 0; t < 8; t++) { dsum[k][t] = 0.0; dsq[k][t] = 0.0; }
        }
        double *red = (double *)(smem_raw + a.off_red);        /* [4 warps][nt][2] */
        uint32_t red_ph = 0;
        /* the 128 epilogue threads meet on an mbarrier (a bounded wait, unlike bar.sync: after a give-up nobody is left waiting for good) */
        auto esync = [&]() { mbar_arrive(bar_red); if (!mbar_wait(bar_red, red_ph, abort_flag, kWaitLimitR)) { raise_r(a, abort_flag, 8, pc); dead = true; } red_ph ^= 1u; };
        /* writes this block's sums of sample n (or zeros): (sum, sum of squares) per channel */
        auto flush = [&](int n, bool have) {
            esync();                                            /* every warp is done with the staging buffers the exchange area overlays */
            if (STATS && have) {
#pragma unroll
                for (int k = 0; k < NCH; k++) {
                    double ws = 0.0, wq = 0.0;
#pragma unroll
                    for (int t = 0; t < 8; t++) {
                        const double a8 = lanes8_sum(dsum[k][t], sp4, sp2, sp1), q8 = lanes8_sum(dsq[k][t], sp4, sp2, sp1);
                        if (t == sx) { ws = a8; wq = q8; }
                        dsum[k][t] = 0.0; dsq[k][t] = 0.0;
                    }
                    double *d = red + ((size_t)(q4 * a.nt + k * 32 + sch)) * 2;
                    d[0] = ws; d[1] = wq;
                }
            }
            esync();
            if (et < a.nt) {
                double ss = 0.0, qq = 0.0;
                if (have) for (int w4 = 0; w4 < 4; w4++) { const double *r2 = red + ((size_t)(w4 * a.nt + et)) * 2; ss += r2[0]; qq += r2[1]; }
                double *d = a.part + (((size_t)n * a.gcol + bcol) * a.cop + ctile * a.nt + et) * 2;
                d[0] = ss; d[1] = qq;
            }
            esync();
        };
        /* fp16 rows on their way out: a thread converts one voxel (64 bytes per 32 channels), the warp's 32 rows pass through 2 KB of shared
           memory (16-byte chunk c of row r at chunk c ^ (r / 2 % 4): no bank conflicts either way) and leave as four stores of 512 contiguous
           bytes each (the eight voxels of one tile row) instead of 32 scattered 16-byte pieces per store */
        uint8_t *stg = smem_raw + a.off_stage + q4 * (2048 * NCH);
        uint8_t *stg_w = stg + lane * 64; const int swz = (lane >> 1) & 3;
        const uint8_t *stg_r = stg + (lane >> 2) * 64 + (lane & 3) * 16;
        const size_t plane_b = (size_t)a.H * a.W * 64, row_b = (size_t)a.W * 64;
        /* sample being accumulated and the first sample this block has planes of.  Nothing is written to `part` before the block has taken a plane
           out of TMEM: this kernel may have been started while its predecessor in the stream, which can be a conv that shares `part`, was still
           running, and only the producer thread waits for the predecessor; a plane in TMEM means that wait is over.  So the zero entries of the
           samples this block has no planes of are written at the end. */
        int n_cur = -1, n_first = -1;
        while (piece.u < piece.u1 && !dead) {
            const Run rn = next_run(a, piece);
            const int x0t = (rn.txy % a.tiles_x) * 8, y0t = (rn.txy / a.tiles_x) * 16;
            const int ox = x0t + rx, oy = y0t + ry;
            const bool row_ok = oy < a.H && ox < a.W;
            const int sy = y0t + q4 * 4;                        /* first of the four tile rows this warp stores */
            uint8_t *run_dst = (uint8_t *)a.e.y + (((size_t)rn.n * a.e.nb_dst + a.e.b0 + ctile * NCH) * S + (size_t)sy * a.W + x0t + (lane >> 2)) * 64 + cl * 16;
            if (stats && rn.n != n_cur) {
                if (n_cur >= 0) flush(n_cur, true); else n_first = rn.n;
                n_cur = rn.n;
            }
            for (int z = rn.zb; z < rn.ze && !dead; z++, pc++) {
                const int slot = NS - 1 - pcm;
                if (!mbar_wait(bar_accf + 8 * slot, (uint32_t)pph, abort_flag, kWaitLimitR)) { raise_r(a, abort_flag, 5, pc, bar_accf + 8 * slot - bar_tma, pph); dead = true; break; }
                tc_fence_after();
                uint32_t rr[NCH][32];
                const uint32_t tcol = tlane + (uint32_t)(slot * a.nt);
                tmem_ld32(tcol, rr[0]);
                if (NCH > 1) tmem_ld32(tcol + 32, rr[NCH - 1]);
                tmem_ld_wait();
                tmem_zero32(tcol);
                if (NCH > 1) tmem_zero32(tcol + 32);
                if (a.fast_h16) {
                    /* fp16 blocked output [n][block][voxel][32]: bias, one rounding; the zeroing of the slot completes meanwhile */
                    __syncwarp();                               /* the previous plane's rows have been read out of the staging buffer */
#pragma unroll
                    for (int jc = 0; jc < NCH; jc++) {
                        const float4 *bs = (const float4 *)(bias_s + jc * 32);
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const float4 b0 = bs[2 * k], b1 = bs[2 * k + 1];
                            __half2 h[4];
                            h[0] = __floats2half2_rn(__fadd_rn(__uint_as_float(rr[jc][8 * k + 0]), b0.x), __fadd_rn(__uint_as_float(rr[jc][8 * k + 1]), b0.y));
                            h[1] = __floats2half2_rn(__fadd_rn(__uint_as_float(rr[jc][8 * k + 2]), b0.z), __fadd_rn(__uint_as_float(rr[jc][8 * k + 3]), b0.w));
                            h[2] = __floats2half2_rn(__fadd_rn(__uint_as_float(rr[jc][8 * k + 4]), b1.x), __fadd_rn(__uint_as_float(rr[jc][8 * k + 5]), b1.y));
                            h[3] = __floats2half2_rn(__fadd_rn(__uint_as_float(rr[jc][8 * k + 6]), b1.z), __fadd_rn(__uint_as_float(rr[jc][8 * k + 7]), b1.w));
                            *(uint4 *)(stg_w + jc * 2048 + ((k ^ swz) << 4)) = make_uint4(*(const uint32_t *)&h[0], *(const uint32_t *)&h[1], *(const uint32_t *)&h[2], *(const uint32_t *)&h[3]);
                        }
                    }
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_acce + 8 * slot);          /* the slot is free once it is in registers and zeroed */
                    uint8_t *pz = run_dst + (size_t)z * plane_b;
#pragma unroll
                    for (int jc = 0; jc < NCH; jc++) {
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint4 v = *(const uint4 *)(stg_r + jc * 2048 + i * 512);
                            const bool in = sy + i < a.H;
                            if (in) *(uint4 *)(pz + (size_t)jc * S * 64 + (size_t)i * row_b) = v;
                            if (STATS && in) {
                                const __half2 *hp = (const __half2 *)&v;
#pragma unroll
                                for (int t = 0; t < 4; t++) {
                                    const float2 f = __half22float2(hp[t]);
                                    const double p0 = (double)f.x, p1 = (double)f.y;
                                    dsum[jc][2 * t] += p0; dsq[jc][2 * t] = fma(p0, p0, dsq[jc][2 * t]);
                                    dsum[jc][2 * t + 1] += p1; dsq[jc][2 * t + 1] = fma(p1, p1, dsq[jc][2 * t + 1]);
                                }
                            }
                        }
                    }
                } else {
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_acce + 8 * slot);
#pragma unroll
                    for (int jc = 0; jc < NCH; jc++) {
                        float v[32];
#pragma unroll
                        for (int k = 0; k < 32; k++) v[k] = __uint_as_float(rr[jc][k]);
                        epi_chunk(a.e, rn.n, z, oy, ox, row_ok, ctile * NCH + jc, v);
                    }
                }
                if (++pcm == NS) { pcm = 0; pph ^= 1; }
            }
        }
        if (stats && !dead) {
            if (n_cur >= 0) flush(n_cur, true);
            for (int n = 0; n < a.N; n++) if (n_cur < 0 || n < n_first || n > n_cur) flush(n, false);
            /* the last block of this column tile to get here turns the partial sums into coefficients; the order of the additions is
               fixed (block 0, 1, ...), so the result does not depend on which block came last */
            volatile unsigned &last = *(volatile unsigned *)(smem_raw + 776);
            __threadfence();
            esync();
            if (et == 0) { const unsigned tk = atomicAdd(&g_conv_tickets[ctile], 1u); last = tk == (unsigned)a.gcol - 1u; if (last) g_conv_tickets[ctile] = 0u; }
            esync();
            if (last) {
                __threadfence();
                for (int i = et; i < a.N * a.nt; i += 128) {
                    const int n = i / a.nt, c = ctile * a.nt + i % a.nt;
                    if (c >= a.e.co_real) continue;
                    double s0 = 0.0, q0 = 0.0;
                    const double *pp = a.part + ((size_t)n * a.gcol * a.cop + c) * 2;
                    for (int t = 0; t < a.gcol; t++) { s0 += __ldcg(pp + (size_t)t * a.cop * 2); q0 += __ldcg(pp + (size_t)t * a.cop * 2 + 1); }
                    const double m = s0 / (double)S, v = fmax(q0 / (double)S - m * m, 0.0);
                    const float rs = (float)(1.0 / sqrt(v + (double)a.eps)), ca = __fmul_rn(rs, a.gamma ? a.gamma[c] : 1.f);
                    a.coef[2 * ((size_t)n * a.e.co_real + c)] = ca;
                    a.coef[2 * ((size_t)n * a.e.co_real + c) + 1] = __fmaf_rn(-(float)m, ca, a.beta ? a.beta[c] : 0.f);
                }
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
    if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, (uint32_t)a.tmem_cols); }
}

/* Weight image of the z-marching kernel: codes [input item][dy dx][k half][dz * nt + channel][16 B], then the B scale bytes in the TMEM
   scale layout per (input item, tap quad, first dz of the MMA, 128-row group): byte (lane, column, id) = row 128 g + 32 column + lane counted
   from that dz's first row, tap 4 q + id (fp8) or tap 2 q + id / 2, block id % 2 (fp4).  A block-scaled MMA wants its scale address on a
   4-column boundary of TMEM (a one-column offset faults with "misaligned address"), hence one re-based image per starting dz.
   Quantisation per (row, tap, 32 input channels) as the reference's prep_w8_k / prep_w4_k (src/lp_f8fwd.cu:54-71, src/lp_f4fwd.cu:53-66).
   One thread per (item, dy dx, dz, channel). */
__global__ void __launch_bounds__(128) prep_wr_k(const float *__restrict__ w, uint8_t *__restrict__ wr_all, int co, int ci, int bits, int nt, int nkb, int nki, int nquad, int gt, int goff1, int goff2, int w_codes, int w_bytes) {
    const int total = nki * 9 * 3 * nt, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    uint8_t *wr = wr_all + (size_t)blockIdx.y * w_bytes;      /* one image per column tile */
    const int cl = i % nt, c = blockIdx.y * nt + cl, dz = (i / nt) % 3, j = (i / (3 * nt)) % 9, ki = i / (27 * nt);
    const int tap = dz * 9 + j, R3 = 3 * nt, row = dz * nt + cl;
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

/* after a bounded wait gave up, blocks may have left without drawing their ticket: the counters start from zero again */
void umx_conv_r_tickets_reset(void) { void *p = nullptr; if (cudaGetSymbolAddress(&p, g_conv_tickets) == cudaSuccess && p) cudaMemset(p, 0, sizeof(unsigned) * 64); }

/* Self-test of the bounded wait and of its report: one block waits, for `limit_clocks` at most, on a barrier that nobody arrives on, gives
   up, and leaves the same record a conv role would (role code 1, stage 123).  Returns 0 when the kernel ran; lp_check() then holds the
   "bounded wait gave up" message.  The context stays usable. */
__global__ void wait_selftest_k(ConvRArgs a, long long limit) {
    __shared__ uint64_t bar; __shared__ int abort_s;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); abort_s = 0; fence_barrier_init(); }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait(smem_u32(&bar), 0, &abort_s, limit)) raise_r(a, &abort_s, 1, 123, 0, 0);
}
extern "C" int umx_wait_selftest(long long limit_clocks) {
    if (!umx_ready("umx_wait_selftest")) return -1;
    if (limit_clocks < 1 || limit_clocks > 2000000000ll) limit_clocks = 2000000;
    ConvRArgs a; memset(&a, 0, sizeof a);
    a.err = umx_errflag(); if (!a.err) return -1;
    wait_selftest_k<<<1, 32>>>(a, limit_clocks);
    g_umx_launches++;
    UMX_CK("umx_wait_selftest");
    return 0;
}

/* geometry of the weight image; 0 when the z-marching kernel cannot run this conv (3^3 only, one column tile of at most 64 channels,
   codes + scales resident in shared memory, B scales resident in TMEM beside at least four accumulator slots) */
struct RGeo { int nt, ncol, w_codes, w_bytes, gt, goff1, goff2, tmem_cols, nslot, sfa_base, sfa_cols, sfb_base; };
static int r_geometry_nt(const umx_conv *c, int nt, RGeo *g) {
    if (c->cop % nt) return 0;
    g->nt = nt; g->ncol = c->cop / nt;
    const int g0 = (3 * nt + 127) / 128, g1 = (2 * nt + 127) / 128, g2 = (nt + 127) / 128;
    g->goff1 = g0; g->goff2 = g0 + g1; g->gt = g0 + g1 + g2;
    g->w_codes = c->nki * 9 * 2 * 3 * nt * 16;
    g->w_bytes = g->w_codes + c->nki * c->nquad * g->gt * 512;
    if (g->w_bytes > 136 * 1024) return 0;
    g->sfa_cols = c->nquad * 4;
    const int fixed = 2 * g->sfa_cols + c->nki * c->nquad * g->gt * 4;
    /* 256 columns (two blocks a multiprocessor) when that leaves four slots, else the whole 512 */
    g->tmem_cols = (256 - fixed) / nt >= 4 ? 256 : 512;
    g->nslot = (g->tmem_cols - fixed) / nt;
    if (g->nslot > kMaxSlots) g->nslot = kMaxSlots;
    if (g->nslot < 4) return 0;
    g->sfa_base = g->nslot * nt; g->sfb_base = g->sfa_base + 2 * g->sfa_cols;
    return 1;
}
/* the widest column tile (64 or 32 channels) whose weight image fits; wider layers run as several column tiles, each on its own
   share of the blocks (the input is then read once per column tile, from L2 when it fits there) */
static int r_geometry(const umx_conv *c, RGeo *g) {
    if (c->kind != UMX_CONV3) return 0;
    if (c->cop <= 64 && r_geometry_nt(c, c->cop, g)) return 1;
    if (r_geometry_nt(c, 64, g)) return 1;
    return r_geometry_nt(c, 32, g);
}
/* upper bound on the blocks per column tile (0: as many as the device holds): lets a small grid be cut into the multi-run pieces, wrapped
   slot windows and several-planes-a-block regime that otherwise only volumes with thousands of tile planes reach */
static int g_r_block_cap = 0;
extern "C" void umx_conv_r_block_cap(int cap) { g_r_block_cap = cap > 0 ? cap : 0; }
int umx_conv_r_fits(const umx_conv *c) { RGeo g; return r_geometry(c, &g); }
/* builds the weight image from device fp32 weights [co][ci][27]; called once when the conv is created */
uint8_t *umx_conv_r_prepare(const umx_conv *c, const float *w_dev) {
    RGeo g;
    if (!r_geometry(c, &g)) return nullptr;
    uint8_t *wr = (uint8_t *)nn_malloc((size_t)g.w_bytes * g.ncol);
    if (!wr) return nullptr;
    cudaMemset(wr, 127, (size_t)g.w_bytes * g.ncol);
    const int total = c->nki * 27 * g.nt;
    prep_wr_k<<<dim3((total + 127) / 128, g.ncol), 128>>>(w_dev, wr, c->co, c->ci, c->bits, g.nt, c->nkb, c->nki, c->nquad, g.gt, g.goff1, g.goff2, g.w_codes, g.w_bytes);
    g_umx_launches++;
    return wr;
}
/* x: MX tensor (fp8 in the split layout); m0: tensor map over its codes; enc: the driver's tensor-map encoder (for the scale plane).
   Returns 1 when this kernel does not apply to the geometry (the caller then takes the general kernel), 0 after a launch, -1 on error. */
/* coef != NULL (only with the blocked fp16 output): InstanceNorm coefficients are produced by the same launch; part then holds N x (blocks per
   column tile, at most 512) x cop x 2 doubles of scratch */
int umx_conv_fwd_r(const umx_conv *c, const void *x, const CUtensorMap *m0, void *enc_v, int N, int D, int H, int W, const EpiArgs &e,
                   double *part, const float *gamma, const float *beta, float eps, float *coef) {
    typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    ConvRArgs a; memset(&a, 0, sizeof a);
    RGeo g;
    if (!r_geometry(c, &g) || !c->wr || (W & 15)) return 1;      /* the scale window needs rows that are multiples of 16 bytes */
    a.w_codes = g.w_codes; a.w_bytes = g.w_bytes; a.gt = g.gt; a.goff1 = g.goff1 * 4; a.goff2 = g.goff2 * 4;   /* TMEM column offsets of the dz >= 1, 2 images */
    a.tmem_cols = g.tmem_cols; a.nslot = g.nslot; a.sfa_base = g.sfa_base; a.sfa_cols = g.sfa_cols; a.sfb_base = g.sfb_base;
    a.N = N; a.D = D; a.H = H; a.W = W; a.nkb = c->nkb; a.nki = c->nki; a.bits = c->bits; a.nt = g.nt; a.ncol = g.ncol;
    a.tiles_x = (W + 7) / 8; a.tiles = a.tiles_x * ((H + 15) / 16);
    a.units = (long long)N * a.tiles * D;
    a.nquad = c->nquad;
    a.fast_h16 = e.out_mode == UMX_OUT_H16B && !e.tconv;
    if (coef && (!a.fast_h16 || !part || g.ncol > 64)) return 1;
    a.part = part; a.coef = coef; a.gamma = gamma; a.beta = beta; a.eps = eps; a.cop = c->cop;
    /* the codes and the scale window are TMA destinations (128-byte aligned) */
    a.offSW = 5888; a.offSFA = a.offSW + (c->bits == 8 ? 640 : 1152);
    a.stage_bytes = (a.offSFA + c->nquad * 512 + 1023) & ~1023;
    a.off_rec = 1024; a.off_bias = a.off_rec + 12 * 64; a.off_stage = 2048; a.off_red = a.off_stage; a.off_w = a.off_stage + 8192 * (g.nt == 32 ? 1 : 2); a.off_ring = (a.off_w + a.w_bytes + 1023) & ~1023;
    int dev = 0, sms = 148; cudaGetDevice(&dev);
    { static int sms_of[16]; if (!sms_of[dev & 15]) { int v = 148; cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev); sms_of[dev & 15] = v; } sms = sms_of[dev & 15]; }   /* looked up once per device */
    /* two blocks a multiprocessor when shared memory (113 KB each) and TMEM (256 columns each) allow */
    const int two = g.tmem_cols == 256 && a.off_ring + 4 * a.stage_bytes <= 113 * 1024;
    const int room = (two ? 113 : 227) * 1024 - a.off_ring;
    a.ring = room / a.stage_bytes; if (a.ring > 12) a.ring = 12;
    if (a.ring < 3) return 1;
    long long slots = (long long)sms * (two ? 2 : 1) / g.ncol;      /* blocks per column tile */
    if (slots < 1) return 1;
    if (g_r_block_cap && slots > g_r_block_cap) slots = g_r_block_cap;
    /* A block pays two halo planes per run: with fewer than eight planes a block (counted for one sample, so that the choice of kernel does not
       depend on the batch) the general kernel is faster.  Volumes with fewer planes than blocks are left here: nothing to gain either way. */
    { const long long units1 = (long long)a.tiles * D; if (g.ncol > 1 && units1 >= slots && units1 < 8 * slots) return 1; }
    a.gcol = (int)(a.units < slots ? a.units : slots); if (a.gcol > 512) a.gcol = 512;
    const int grid = a.gcol * g.ncol;
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
        const void *ks[8] = {(const void *)conv_mxr_k<8, 1, false>, (const void *)conv_mxr_k<8, 2, false>, (const void *)conv_mxr_k<4, 1, false>, (const void *)conv_mxr_k<4, 2, false>,
                             (const void *)conv_mxr_k<8, 1, true>, (const void *)conv_mxr_k<8, 2, true>, (const void *)conv_mxr_k<4, 1, true>, (const void *)conv_mxr_k<4, 2, true>};
        for (int i = 0; i < 8; i++) {
            const cudaError_t er = cudaFuncSetAttribute(ks[i], cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (er != cudaSuccess) { umx_latch("umx_conv_fwd: shared memory attribute", er); return -1; }
        }
        attr_set[dev & 15] = 1;
    }
    const int variant = (coef ? 4 : 0) | (c->bits == 8 ? 0 : 2) | (g.nt == 32 ? 0 : 1);
    switch (variant) {
    case 0: umx_launch(conv_mxr_k<8, 1, false>, dim3(grid), dim3(kThreadsR), smem, *m0, ms, a); break;
    case 1: umx_launch(conv_mxr_k<8, 2, false>, dim3(grid), dim3(kThreadsR), smem, *m0, ms, a); break;
    case 2: umx_launch(conv_mxr_k<4, 1, false>, dim3(grid), dim3(kThreadsR), smem, *m0, ms, a); break;
    case 3: umx_launch(conv_mxr_k<4, 2, false>, dim3(grid), dim3(kThreadsR), smem, *m0, ms, a); break;
    case 4: umx_launch(conv_mxr_k<8, 1, true>, dim3(grid), dim3(kThreadsR), smem, *m0, ms, a); break;
    case 5: umx_launch(conv_mxr_k<8, 2, true>, dim3(grid), dim3(kThreadsR), smem, *m0, ms, a); break;
    case 6: umx_launch(conv_mxr_k<4, 1, true>, dim3(grid), dim3(kThreadsR), smem, *m0, ms, a); break;
    default: umx_launch(conv_mxr_k<4, 2, true>, dim3(grid), dim3(kThreadsR), smem, *m0, ms, a); break;
    }
    return 0;
}
