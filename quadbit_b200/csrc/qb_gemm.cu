// Two-level NVFP4 GEMM for sm_100a, dense and 2:4-sparse, on the 5th-generation tensor
// cores:  C[out,tok] = gA[out] * gB[tok] * sum_k (a * sfa) * (b * sfb)
//
// Replaces matmul_sp / run_sp_mm (cuda/sparse_fp4_lib.cu:30-221,1029-1041), dmatmul_nvf
// (cuda/dense_nvfp4_fast_lib.cu:23-151), the split-K decode pair matmul_sp_sk + cvt_sp_2lvl_t
// (cuda/sparse_fp4_lib.cu:1160-1344) and the segmented MoE GEMM matmul_sp_moe
// (cuda/sparse_fp4_lib.cu:1362-1566), which are warp-level mma.sync / mma.sp kernels that
// do not exist on this architecture.
//
// Two kernels. The CTA-pair kernel further down serves prefill (tok >= 128, out % 256 == 0). The
// single-CTA kernel right below serves thin token counts, ragged shapes, split-K and the grouped
// (MoE) form; its structure (one persistent CTA per SM, 416 threads):
//   warp 0, 6-8 producers, K blocks round-robin: TMA tiles of A (weights, 128 rows) and B
//               (tokens, BN rows) with hardware swizzle, plus bulk copies of the scale-factor
//               atoms and the 2:4 metadata, into a multi-stage shared-memory ring (mbarrier
//               full/empty).
//   warps 9-12  scale-factor warps: copy scale factors / metadata of a landed stage from shared
//               memory to the stage's tensor-memory slot (tcgen05.st, one lane quadrant each).
//   warp 1      MMA issuer (one thread): issues tcgen05.mma[.sp] kind::mxf4nvf4 block_scale with
//               the accumulator in TMEM; tcgen05.commit releases smem stages and hands
//               finished accumulators to the epilogue. Allocates / frees TMEM.
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp its own 32-lane quadrant),
//               multiply by the fp32 globals, convert to bf16 and store; with two
//               accumulator stages (BN <= 128) this overlaps the next tile's main loop.
// The weight is always the tensor-core A operand (M = 128 rows per CTA; the only operand
// that can be 2:4-sparse), tokens are the N dimension (16..256), so thin-M decode is the
// same kernel with a small token tile and K split across CTAs.
//
// A pipeline stage covers 256 logical K: dense A 128x128 B (SWIZZLE_128B, 4 MMAs of K=64),
// sparse A 128x64 B of kept values (SWIZZLE_64B, 2 MMAs of K=128 logical), B BNx128 B
// (SWIZZLE_128B). Scale factors: 4 per row per MMA (dense: one per 16 K, sparse: one per
// 32 logical K), stored as 512-byte "128x4" atoms. Metadata: 16 B per row per stage.
// Every wait is bounded (see mbar_wait); on expiry the CTA records QB_ERR_TIMEOUT, drains
// and frees its TMEM.
#include <cuda.h>

#include <mutex>

#include "qb_common.cuh"
#include "qb_internal.h"

namespace qb {

__device__ int g_status = 0;

struct KParams {
    const uint8_t* sfa;
    const uint8_t* sfb;
    const uint8_t* meta;
    const float* gA;
    const float* gB;
    void* C;
    float* Cf;
    const int* eblk;
    const __nv_bfloat16* bias;
    const float* row_w;
    int bias_ld;                         // features per bias row
    int out_f, tok, K;
    int num_m, num_n, splits, kblocks;   // kblocks = ceil(K/256)
    int sfb_rowblocks;                   // ceil(tok/128)
    int b_box_bytes;                     // bytes one B TMA box delivers (box rows * 128)
    int out_mode;
    int a_tiled;                         // A in 128-row x 256-K tiles: TMA row coordinate = tile * 128, column 0
    int* sk_counters;                    // split-K finished in the kernel: 4 arrival counters per output tile (zero between calls)
    int cluster_red;                     // split-K inside a cluster of `splits` CTAs: partial tiles meet in distributed shared memory
};

template <bool SPARSE, int BN>
struct Cfg {
    static constexpr int BM = 128;
    static constexpr int A_ROW = SPARSE ? 64 : 128;
    static constexpr int A_BYTES = BM * A_ROW;
    static constexpr int B_BYTES = BN * 128;
    static constexpr int B_ALLOC = B_BYTES < 1024 ? 1024 : B_BYTES;
    static constexpr int MMAS = SPARSE ? 2 : 4;
    static constexpr int B_KSTEP = SPARSE ? 64 : 32;   // bytes of a B row consumed per MMA
    static constexpr int NB128 = (BN + 127) / 128;
    static constexpr int SFA_BYTES = MMAS * 512;
    static constexpr int SFB_BYTES = NB128 * MMAS * 512;
    static constexpr int META_BYTES = SPARSE ? 2048 : 0;
    static constexpr int STAGE_BYTES = A_BYTES + B_ALLOC + SFA_BYTES + SFB_BYTES + META_BYTES;
    static constexpr int ACC_STAGES = BN <= 128 ? 2 : 1;
    static constexpr int EPI_BYTES = 4 * 32 * 80;   // per-warp 32x32 bf16 transpose tile, 80-byte pitch
    static constexpr int SMEM_BUDGET = 226 * 1024 - 1024 - EPI_BYTES - 512;
    static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + 512;
    // TMEM columns
    static constexpr int SFA_COLS = MMAS * 4;
    static constexpr int SFB_COLS = MMAS * 4 * NB128;
    static constexpr int E_COLS = SPARSE ? 4 : 0;
    static constexpr int SF_SET = SFA_COLS + SFB_COLS + E_COLS;
    static constexpr int TM_SF0 = ((ACC_STAGES * BN + 3) / 4) * 4;
    static constexpr int TM_USED = TM_SF0 + STAGES * SF_SET;        // one scale-factor slot per ring stage
    static constexpr int TM_COLS = TM_USED <= 32 ? 32 : TM_USED <= 64 ? 64 : TM_USED <= 128 ? 128 : TM_USED <= 256 ? 256 : 512;
    static_assert(TM_USED <= 512, "TMEM budget");
    static_assert(STAGES >= 2, "smem budget");
    static constexpr int CH = (BN % 32 == 0) ? 32 : 8;   // epilogue column chunk
};

constexpr uint32_t QB_BACKOFF = 64, QB_BACKOFF_SF = 32;   // ns a role with slack sleeps between polls
constexpr int NPROD1 = 4;                      // producer warps of the single-CTA kernel (warp 0 and warps 6..8)
constexpr int NTHREADS1 = (6 + NPROD1 - 1 + 4) * 32;  // + four scale-factor warps (9..12)
enum { SITE_PROD = 1, SITE_MMA_FULL = 2, SITE_MMA_ACC = 3, SITE_EPI = 4, SITE_SF1 = 9 };

template <bool SPARSE, int BN>
__global__ void __launch_bounds__(NTHREADS1, 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const KParams p) {
    using C = Cfg<SPARSE, BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_base_slot;

    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = smem0 + C::STAGES * C::STAGE_BYTES + C::EPI_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
    auto accf_bar = [&](int a) { return bars + 8u * (2 * C::STAGES + a); };
    auto acce_bar = [&](int a) { return bars + 8u * (2 * C::STAGES + 2 + a); };
    auto sfr_bar = [&](int s) { return bars + 8u * (2 * C::STAGES + 4 + s); };     // scale factors of the stage are in TMEM
    auto stageA = [&](int s) { return smem0 + (uint32_t)s * C::STAGE_BYTES; };
    auto stageB = [&](int s) { return stageA(s) + C::A_BYTES; };
    auto stageSFA = [&](int s) { return stageB(s) + C::B_ALLOC; };
    auto stageSFB = [&](int s) { return stageSFA(s) + C::SFA_BYTES; };
    auto stageMETA = [&](int s) { return stageSFB(s) + C::SFB_BYTES; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < C::STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); mbar_init(sfr_bar(s), 4); }
        for (int a = 0; a < 2; a++) { mbar_init(accf_bar(a), 1); mbar_init(acce_bar(a), 4); }
        fence_barrier_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), C::TM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    // Launched as a programmatic dependent: barrier set-up, the tensor-memory allocation and the descriptor prefetch above
    // ran beside the tail of the kernel in front (the activation quantiser). Everything that kernel writes (packed
    // activations, their scale factors and globals, routing tables) is read only after griddep_wait(); the weights are
    // constants, so the producers stream the first ring of weight tiles BEFORE they wait (below).
    griddep_launch_dependents();
    const bool is_producer = warp == 0 || (warp >= 6 && warp < 9);
    const bool prefetch_weights = p.eblk == nullptr;        // grouped mode reads its expert table first
    if (!(is_producer && prefetch_weights)) griddep_wait();

    const int tiles_mn = p.num_m * p.num_n;
    const int total_tiles = tiles_mn * p.splits;
    // Work items of this CTA. Normally tile = blockIdx.x + i * gridDim.x over (split, tile) pairs. With the cluster reduction
    // the grid is one cluster of `splits` CTAs per output tile and nothing else: the CTA of rank r takes K split r of tile
    // blockIdx.x / splits, once.
    const int crank = p.cluster_red ? (int)cluster_ctarank() : 0;
    const int tile0 = p.cluster_red ? crank * tiles_mn + (int)blockIdx.x / p.splits : (int)blockIdx.x;
    const int tile_step = p.cluster_red ? total_tiles : (int)gridDim.x;
    // grouped mode: a 128-token block with expert id < 0 is unused capacity of a fixed-capacity routing; every
    // role skips its tiles (same test everywhere, so the K-block and accumulator counters stay in step)
    auto tile_skipped = [&](int tile) { return p.eblk != nullptr && p.eblk[(tile % tiles_mn) / p.num_m] < 0; };
    const int kb_per_split = (p.kblocks + p.splits - 1) / p.splits;
    const int atoms_per_rb = p.kblocks * C::MMAS;   // scale atoms per 128-row block along K

    if (is_producer) {
        // ------------------------------------------------------------ producers
        // Four warps take the K blocks round-robin: one thread needs ~90 cycles to issue one bulk load
        // (measured) and a stage takes 5-6 of them, so one producer cannot keep a thin-token stream fed.
        // A producer may run at most one ring revolution ahead of the consumer or the parity wait on the
        // empty barrier aliases; with in-order consumption that holds iff producers <= stages.
        constexpr int NP = C::STAGES < NPROD1 ? C::STAGES : NPROD1;
        const int pw = warp == 0 ? 0 : warp - 5;
        // what: 0 = the whole stage, 1 = byte count + weight side (tile of A, its scale factors, metadata),
        //       2 = activation side only (the byte count was announced with the weight side)
        auto issue = [&](int what, int stage, int kb, int a_row0, int n0, int rb0, int nsfb, uint32_t tx) {
            const uint32_t fb = full_bar(stage);
            if (what != 2) {
                mbar_expect_tx(fb, tx);
                if (p.a_tiled) tma_load_2d(stageA(stage), &tmA, fb, 0, ((a_row0 >> 7) * p.kblocks + kb) * 128);
                else tma_load_2d(stageA(stage), &tmA, fb, kb * C::A_ROW, a_row0);
                bulk_load(stageSFA(stage), p.sfa + ((size_t)(a_row0 >> 7) * atoms_per_rb + (size_t)kb * C::MMAS) * 512, C::SFA_BYTES, fb);
                if (SPARSE) bulk_load(stageMETA(stage), p.meta + ((size_t)(a_row0 >> 7) * p.kblocks + kb) * 2048, 2048, fb);
            }
            if (what != 1) {
                tma_load_2d(stageB(stage), &tmB, fb, kb * 128, n0);
                for (int i = 0; i < nsfb; i++)
                    bulk_load(stageSFB(stage) + i * C::MMAS * 512,
                              p.sfb + ((size_t)(rb0 + i) * atoms_per_rb + (size_t)kb * C::MMAS) * 512, C::MMAS * 512, fb);
            }
        };
        // pass 0 (only when weights are prefetched): the weight side of the first ring revolution, no waits (fresh ring);
        // then griddep_wait; pass 1: everything else, in the same order
        for (int pass = prefetch_weights ? 0 : 1; pass < 2; pass++) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t it = 0;
            bool stop = false;
            for (int tile = tile0; tile < total_tiles && !abort_flag && pw < NP && !stop; tile += tile_step) {
                if (pass == 1 && tile_skipped(tile)) continue;
                const int z = tile / tiles_mn, mn = tile - z * tiles_mn;
                const int m = mn % p.num_m, n = mn / p.num_m;
                const int n0 = n * BN;
                const int a_row0 = ((pass == 1 && p.eblk) ? p.eblk[n] * p.out_f : 0) + m * 128;
                const int kb0 = z * kb_per_split, kb1 = min(p.kblocks, kb0 + kb_per_split);
                const int rb0 = n0 >> 7;
                const int nsfb = min(C::NB128, p.sfb_rowblocks - rb0);
                const uint32_t tx = C::A_BYTES + (uint32_t)p.b_box_bytes + C::SFA_BYTES + (uint32_t)nsfb * C::MMAS * 512 + C::META_BYTES;
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    if (pass == 0 && it >= (uint32_t)C::STAGES) { stop = true; break; }
                    if ((int)(it % NP) == pw) {
                        if (pass == 0) {
                            if (lane == 0) issue(1, stage, kb, a_row0, n0, rb0, nsfb, tx);
                        } else {
                            const bool prefetched = prefetch_weights && it < (uint32_t)C::STAGES;
                            if (!prefetched && !mbar_wait(empty_bar(stage), phase ^ 1, &abort_flag, &g_status, SITE_PROD, QB_BACKOFF)) { stop = true; break; }
                            if (lane == 0) issue(prefetched ? 2 : 0, stage, kb, a_row0, n0, rb0, nsfb, tx);
                        }
                        __syncwarp();
                    }
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (pass == 0) griddep_wait();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // One thread runs the whole issue loop (no warp-wide broadcast or re-convergence between a barrier
        // wait and the MMAs it gates). It waits for "scale factors of the stage are in tensor memory",
        // which the scale-factor warps signal after they have seen the stage land.
        if (lane == 0) {
            const uint32_t idesc = make_idesc_nvf4(BN, SPARSE);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            for (int tile = tile0; tile < total_tiles && !abort_flag; tile += tile_step) {
                if (tile_skipped(tile)) continue;
                const int z = tile / tiles_mn, mn = tile - z * tiles_mn;
                const int n = mn / p.num_m;
                const int n0 = n * BN;
                const int kb0 = z * kb_per_split, kb1 = min(p.kblocks, kb0 + kb_per_split);
                const uint32_t sfb_coloff = (uint32_t)((n0 & 127) >> 5);
                if (!mbar_wait_thread(acce_bar(acc), acc_phase ^ 1, &abort_flag, &g_status, SITE_MMA_ACC)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                bool ok = true;
                for (int kb = kb0; kb < kb1;) {
                    // two K blocks per poll when the later one is ready too (a poll costs 100-200 cycles
                    // even on a completed barrier; the scale-factor warps signal in ring order)
                    int s1 = stage + 1;
                    uint32_t ph1 = phase;
                    if (s1 == C::STAGES) { s1 = 0; ph1 ^= 1; }
                    int nb = 2;
                    if (kb + 1 >= kb1 || !mbar_try_wait(sfr_bar(s1), ph1)) {
                        nb = 1;
                        if (!mbar_wait_thread(sfr_bar(stage), phase, &abort_flag, &g_status, SITE_MMA_FULL)) { ok = false; break; }
                    }
                    tc_fence_after();
                    for (int u = 0; u < nb; u++) {
                        const int s = u ? s1 : stage;
                        const uint32_t sfset = tmem_base + C::TM_SF0 + s * C::SF_SET;
                        const uint32_t t_sfa = sfset, t_sfb = sfset + C::SFA_COLS, t_e = sfset + C::SFA_COLS + C::SFB_COLS;
#pragma unroll
                        for (int i = 0; i < C::MMAS; i++) {
                            const uint64_t adesc = make_smem_desc(stageA(s) + i * 32, SPARSE ? 512 : 1024, 16, SPARSE ? 4 : 2);
                            const uint64_t bdesc = make_smem_desc(stageB(s) + i * C::B_KSTEP, 1024, 16, 2);
                            const uint32_t accum = (kb + u > kb0 || i > 0) ? 1u : 0u;
                            if (SPARSE)
                                tc_mma_nvf4_sp(d_tmem, adesc, bdesc, idesc, t_sfa + 4 * i, t_sfb + i * (4 * C::NB128) + sfb_coloff,
                                               t_e + 2 * i, accum);
                            else
                                tc_mma_nvf4(d_tmem, adesc, bdesc, idesc, t_sfa + 4 * i, t_sfb + i * (4 * C::NB128) + sfb_coloff, accum);
                        }
                        tc_commit(empty_bar(s));
                    }
                    kb += nb;
                    stage += nb;
                    if (stage >= C::STAGES) { stage -= C::STAGES; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit(accf_bar(acc));
                if (++acc == C::ACC_STAGES) { acc = 0; acc_phase ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp >= 9) {
        // ------------------------------------------------------------ scale-factor warps (9..12)
        // Copy the landed stage's scale factors / metadata from shared memory into the stage's own
        // tensor memory slot with tcgen05.st, each warp its lane quadrant (a tcgen05.cp from the issuer
        // costs ~50 cycles of the MMA pipe, 5-12 of them per K block).
        const int q = warp & 3;
        const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
        int stage = 0;
        uint32_t phase = 0;
        for (int tile = tile0; tile < total_tiles && !abort_flag; tile += tile_step) {
            if (tile_skipped(tile)) continue;
            const int z = tile / tiles_mn;
            const int kb0 = z * kb_per_split, kb1 = min(p.kblocks, kb0 + kb_per_split);
            bool ok = true;
            for (int kb = kb0; kb < kb1; kb++) {
                if (!mbar_wait(full_bar(stage), phase, &abort_flag, &g_status, SITE_SF1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t sf = stageSFA(stage) + lane * 16;       // this lane's 16 bytes of every atom
                const uint32_t t_sfa = tmem_base + C::TM_SF0 + stage * C::SF_SET + lane_sel;
                const uint32_t t_sfb = t_sfa + C::SFA_COLS, t_e = t_sfb + C::SFB_COLS;
                {
                    uint32_t a[C::MMAS * 4];
#pragma unroll
                    for (int i = 0; i < C::MMAS; i++) {
                        uint4 v = lds_v4(sf + i * 512);
                        a[4 * i] = v.x; a[4 * i + 1] = v.y; a[4 * i + 2] = v.z; a[4 * i + 3] = v.w;
                    }
                    if constexpr (C::MMAS == 2) tc_st_32x8(t_sfa, a); else tc_st_32x16(t_sfa, a);
                }
                // SFB: column 4*NB128*i + 4*nb + c  <-  atom (nb, i), word c (atoms beyond the token count
                // hold stale bytes; their columns are never selected by an MMA that matters)
#pragma unroll
                for (int h = 0; h < (C::MMAS * C::NB128 * 4) / 8; h++) {
                    uint32_t b[8];
#pragma unroll
                    for (int w = 0; w < 2; w++) {
                        const int g = h * 2 + w;               // group of 4 columns
                        const int i = g / C::NB128, nbk = g % C::NB128;
                        uint4 v = lds_v4(sf + C::SFA_BYTES + (nbk * C::MMAS + i) * 512);
                        b[4 * w] = v.x; b[4 * w + 1] = v.y; b[4 * w + 2] = v.z; b[4 * w + 3] = v.w;
                    }
                    tc_st_32x8(t_sfb + 8 * h, b);
                }
                if constexpr (SPARSE) {
                    uint32_t e[4];
                    uint4 v = lds_v4(stageMETA(stage) + (q * 32 + lane) * 16);
                    e[0] = v.x; e[1] = v.y; e[2] = v.z; e[3] = v.w;
                    tc_st_32x4(t_e, e);
                }
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sfr_bar(stage));
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) break;
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;                     // TMEM lane quadrant this warp may read
        const int r_in_tile = q * 32 + lane;        // accumulator row = output feature in tile
        const uint32_t stg_s = smem0 + C::STAGES * C::STAGE_BYTES + (warp - 2) * (32 * 80);
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = tile0; tile < total_tiles && !abort_flag; tile += tile_step) {
            if (tile_skipped(tile)) continue;
            const int z = tile / tiles_mn, mn = tile - z * tiles_mn;
            const int m = mn % p.num_m, n = mn / p.num_m;
            const int n0 = n * BN;
            const int expert = p.eblk ? p.eblk[n] : 0;
            const int o = m * 128 + r_in_tile;                    // output feature index
            const int a_row = expert * p.out_f + o;               // row of A / gA
            (void)z;
            // per-tile constants first: their load latency hides behind the accumulator wait
            const float ga = p.gA ? __ldg(p.gA + a_row) : 1.f;
            float gbv[BN / C::CH];
#pragma unroll
            for (int c = 0; c < BN / C::CH; c++) {
                const int col = n0 + c * C::CH + (lane % C::CH);
                gbv[c] = (p.gB && col < p.tok) ? __ldg(p.gB + col) : 1.f;
            }
            if (!mbar_wait(accf_bar(acc), acc_phase, &abort_flag, &g_status, SITE_EPI, QB_BACKOFF)) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(q * 32) << 16);
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += C::CH) {
                uint32_t r[C::CH];
                if constexpr (C::CH == 32) tc_ld_32x32(t_acc + c0, r); else tc_ld_32x8(t_acc + c0, r);
                tc_wait_ld();
                const int col_l = n0 + c0 + (lane % C::CH);
                const float gbl = gbv[c0 / C::CH];
                if (p.splits > 1) {
                    // split-K: raw partial sums are added into the fp32 workspace Cf[tok][out] (fire-and-forget
                    // reductions at the L2); finished by the last split of the tile (below) or by a finish kernel
                    if (p.cluster_red) {
                        // cluster reduction: the partial tile goes to this CTA's shared memory, column-major [BN][128] fp32 over
                        // the operand ring (free by now: the accumulator is complete, so every stage has been consumed and
                        // this CTA has no other work item)
#pragma unroll
                        for (int j = 0; j < C::CH; j++) sts_u32(smem0 + (uint32_t)(((c0 + j) * 128 + r_in_tile) * 4), r[j]);
                    } else {
#pragma unroll
                    for (int j = 0; j < C::CH; j++) {
                        const int col = n0 + c0 + j;
                        if (col < p.tok) atomicAdd(p.Cf + (size_t)col * p.out_f + o, __uint_as_float(r[j]));
                    }
                    }
                } else if (p.out_mode == 2) {
                    float* Cp = reinterpret_cast<float*>(p.C) + (size_t)o * p.tok;
#pragma unroll
                    for (int j = 0; j < C::CH; j++) {
                        const int col = n0 + c0 + j;
                        if (col < p.tok) Cp[col] = __uint_as_float(r[j]);
                    }
                } else if (p.out_mode == 0) {
                    __nv_bfloat16* Cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)o * p.tok;
                    uint32_t pk[C::CH / 2];
#pragma unroll
                    for (int j = 0; j < C::CH; j += 2) {
                        float g0 = __shfl_sync(0xffffffffu, gbl, j), g1 = __shfl_sync(0xffffffffu, gbl, j + 1);
                        __nv_bfloat162 h = __floats2bfloat162_rn((__uint_as_float(r[j]) * ga) * g0, (__uint_as_float(r[j + 1]) * ga) * g1);
                        pk[j / 2] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    const int col0 = n0 + c0;
                    if (col0 + C::CH <= p.tok && (p.tok & 7) == 0) {
#pragma unroll
                        for (int v = 0; v < C::CH / 8; v++)
                            *reinterpret_cast<uint4*>(Cp + col0 + 8 * v) = make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < C::CH; j++)
                            if (col0 + j < p.tok) {
                                uint32_t w = pk[j / 2];
                                uint16_t hv = (j & 1) ? (uint16_t)(w >> 16) : (uint16_t)(w & 0xffff);
                                reinterpret_cast<uint16_t*>(Cp)[col0 + j] = hv;
                            }
                    }
                } else {
                    // token-major output C[tok][out]: transpose a 32(out) x CH(tok) block through
                    // shared memory so that global stores are 16-byte vectors
                    float bias_v = 0.f;
                    if (p.out_mode == 3 && p.bias && o < p.bias_ld) bias_v = __bfloat162float(p.bias[(size_t)expert * p.bias_ld + o]);
                    float rw = 1.f;
                    if (p.out_mode == 3 && p.row_w && col_l < p.tok) rw = __ldg(p.row_w + col_l);
#pragma unroll
                    for (int j = 0; j < C::CH; j++) {
                        float g0 = __shfl_sync(0xffffffffu, gbl, j);
                        float v = (__uint_as_float(r[j]) * ga) * g0;
                        if (p.out_mode == 3) v = (v + bias_v) * __shfl_sync(0xffffffffu, rw, j);
                        __nv_bfloat16 h = __float2bfloat16_rn(v);
                        sts_u16(stg_s + j * 80 + lane * 2, *reinterpret_cast<uint16_t*>(&h));
                    }
                    __syncwarp();
                    uint4 val[C::CH / 8];
#pragma unroll
                    for (int it = 0; it < C::CH / 8; it++) val[it] = lds_v4(stg_s + ((it * 32 + lane) >> 2) * 80 + (lane & 3) * 16);
                    __nv_bfloat16* Cp = reinterpret_cast<__nv_bfloat16*>(p.C) + m * 128 + q * 32 + (lane & 3) * 8;
#pragma unroll
                    for (int it = 0; it < C::CH / 8; it++) {
                        const int col = n0 + c0 + ((it * 32 + lane) >> 2);
                        if (col < p.tok) stg_v4(Cp + (size_t)col * p.out_f, val[it]);
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce_bar(acc));
            if (p.splits > 1 && p.sk_counters) {
                // The warp that arrives last among the same-quadrant warps of all K splits owns rows
                // [32q, 32q+32) of this tile: it reads the sums, applies the globals and writes bf16.
                __threadfence();
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    int* cnt = p.sk_counters + (size_t)mn * 4 + q;
                    last = (atomicAdd(cnt, 1) == p.splits - 1);
                    if (last) *cnt = 0;            // every split has arrived: leave the counter clean for the next call
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    const int ncol = min(BN, p.tok - n0);
                    float* base = p.Cf + (size_t)n0 * p.out_f + o;
                    for (int j0 = 0; j0 < ncol; j0 += 16) {
                        // 16 independent loads in flight per lane; every element is zeroed again right after
                        // it is read, so the workspace is clean for the next call
                        float sum[16];
#pragma unroll
                        for (int jj = 0; jj < 16; jj++) {
                            const int jc = (j0 + jj < ncol) ? j0 + jj : j0;      // clamp: keep the load unconditional
                            sum[jj] = __ldcg(base + (size_t)jc * p.out_f);
                        }
#pragma unroll
                        for (int jj = 0; jj < 16; jj++) {
                            const int col = n0 + j0 + jj;
                            if (j0 + jj < ncol) {
                                __stcg(base + (size_t)(j0 + jj) * p.out_f, 0.f);
                                const float gb = p.gB ? __ldg(p.gB + col) : 1.f;
                                const __nv_bfloat16 h = __float2bfloat16_rn((sum[jj] * ga) * gb);
                                if (p.out_mode == 0) reinterpret_cast<__nv_bfloat16*>(p.C)[(size_t)o * p.tok + col] = h;
                                else reinterpret_cast<__nv_bfloat16*>(p.C)[(size_t)col * p.out_f + o] = h;
                            }
                        }
                    }
                }
            }
            if (++acc == C::ACC_STAGES) { acc = 0; acc_phase ^= 1; }
        }
    }

    if (p.cluster_red) {
        // Split-K finish inside the cluster: every CTA has staged its partial tile; after a cluster barrier CTA r sums token
        // columns [r * cpr, (r + 1) * cpr) of all the CTAs' partial tiles (in rank order: the result does not depend on
        // timing), applies the globals and stores bf16; a second barrier keeps every CTA's shared memory alive until its
        // peers have read it. All threads of all CTAs of the cluster get here whatever happened before (every wait above is
        // bounded), so the hardware barrier cannot be left waiting.
        __syncthreads();
        cluster_sync_all();
        const int w = (int)blockIdx.x / p.splits;
        const int m = w % p.num_m, n = w / p.num_m;
        const int n0 = n * BN;
        const int cpr = (BN + p.splits - 1) / p.splits;
        const int c_begin = crank * cpr;
        const int c_end = min(min(BN, c_begin + cpr), p.tok - n0);
        // four consecutive rows of one column per thread and step: one 16-byte load from every CTA of the cluster, all of
        // them issued before the sums (rank order), 8 bytes of bf16 out
        for (int idx = threadIdx.x; idx < (c_end - c_begin) * 32; idx += NTHREADS1) {
            const int row = (idx & 31) * 4, col = c_begin + (idx >> 5);
            const uint32_t local = smem0 + (uint32_t)((col * 128 + row) * 4);
            float4 v[8];
#pragma unroll
            for (int z = 0; z < 8; z++) {
                v[z] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (z < p.splits)
                    asm("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                        : "=f"(v[z].x), "=f"(v[z].y), "=f"(v[z].z), "=f"(v[z].w)
                        : "r"(mapa_shared(local, (uint32_t)z)));
            }
            float4 sum = v[0];
#pragma unroll
            for (int z = 1; z < 8; z++) { sum.x += v[z].x; sum.y += v[z].y; sum.z += v[z].z; sum.w += v[z].w; }
            const int o = m * 128 + row, colg = n0 + col;
            const float4 ga = p.gA ? make_float4(__ldg(p.gA + o), __ldg(p.gA + o + 1), __ldg(p.gA + o + 2), __ldg(p.gA + o + 3)) : make_float4(1.f, 1.f, 1.f, 1.f);
            const float gb = p.gB ? __ldg(p.gB + colg) : 1.f;
            const uint32_t h01 = pack_bf16x2((sum.x * ga.x) * gb, (sum.y * ga.y) * gb), h23 = pack_bf16x2((sum.z * ga.z) * gb, (sum.w * ga.w) * gb);
            __nv_bfloat16* Cb = reinterpret_cast<__nv_bfloat16*>(p.C);
            if (p.out_mode == 0) {
                uint16_t* c16 = reinterpret_cast<uint16_t*>(Cb);
                c16[(size_t)o * p.tok + colg] = (uint16_t)(h01 & 0xffff);
                c16[(size_t)(o + 1) * p.tok + colg] = (uint16_t)(h01 >> 16);
                c16[(size_t)(o + 2) * p.tok + colg] = (uint16_t)(h23 & 0xffff);
                c16[(size_t)(o + 3) * p.tok + colg] = (uint16_t)(h23 >> 16);
            } else {
                *reinterpret_cast<uint2*>(Cb + (size_t)colg * p.out_f + o) = make_uint2(h01, h23);
            }
        }
        cluster_sync_all();
    }
    // teardown: every role has left its loop (all waits are bounded)
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TM_COLS);
    }
}


// ------------------------------------------------------------------ CTA-pair kernel (prefill)
// The prefill kernel: a cluster of two CTAs issues tcgen05.mma.cta_group::2 with M = 256,
// N = 256. CTA r of the pair owns weight rows [256*m2 + 128*r, +128) and loads only token rows
// [n0 + 128*r, +128) of B (the pair shares B through the MMA).
//
// Two rings per CTA. The operand ring (A and B tiles, 24 KB sparse / 32 KB dense per slot, 7 / 5
// slots) is released by the MMAs that read it. The sideband ring (scale-factor atoms and 2:4
// metadata, 5-6 KB per slot, 4 slots) is released as soon as its content has been copied into the
// tensor memory slot of the operand stage, so sideband loads run several K blocks ahead and the
// copy into tensor memory overlaps the operand loads of the same stage instead of following them.
// Measured with every MMA, load and epilogue switched off, the barrier round trip
// (release -> load issue -> landing -> scale-factor copy -> remote arrive -> issue -> commit) is what
// bounds the K-block rate, so each hop is kept off the others' critical path. 640 threads per CTA,
// one kind of role per warpgroup (registers are moved between warpgroups with setmaxnreg):
//   warp 0     A producer, warp 1 B producer: one TMA tile load per K block each, completing (from
//              both CTAs) on the LEADER's full barrier; no multicast.
//   warp 2     sideband producer for scale-factor atoms of A and the metadata, warp 3 for the
//              scale-factor atoms of B; they complete on this CTA's sideband barrier.
//   warps 4-7  scale-factor warps: once the sideband slot has landed and the tensor memory slot of
//              the stage is free, copy scale factors / metadata from shared memory into that slot
//              with tcgen05.st (each warp its lane quadrant), free the sideband slot and tell the
//              leader. Measured: a tcgen05.cp costs ~50 cycles of the MMA pipe and 7-12 of them per
//              K block cap the pipe at 57 % (dense) / 60 % (sparse) of its MMA-only rate; stores
//              from registers run beside the MMAs.
//   warps 8-15 epilogue: each CTA drains its own 128 x BN accumulator half. With one accumulator
//              (256-token tile) the time until it is handed back is exposed, and fp32 -> bf16
//              conversions run at a fraction of the fp32 rate (measured: ~2700 cycles for the
//              128 x 256 slice, against ~470 for the tensor-memory loads alone), so these warps take
//              the registers the others give up, pull their whole slice out of tensor memory as raw
//              fp32, hand the accumulator back, and scale / convert / transpose / store under the
//              main loop of the next tile.
//   warp 16    MMA issuer (one thread of the even CTA): waits for the operands of both CTAs and for
//              both CTAs' scale-factor warps, issues the MMAs for the pair, releases the stage in
//              both CTAs and publishes the accumulator with multicast commits. Warps 17-19 only
//              complete its warpgroup.
// Requires out % 256 == 0 and tok >= 128.
template <bool SPARSE, int BN_>
struct Cfg2 {
    static constexpr int BN = BN_;                        // tokens per pair tile: 128 or 192 (two accumulator stages) or 256
    static constexpr int THREADS = 640;                   // five warpgroups, roles above
    static constexpr int A_ROW = SPARSE ? 64 : 128;
    static constexpr int A_BYTES = 128 * A_ROW;
    static constexpr int B_ROWS = BN / 2;                 // this CTA's half of the token tile
    static constexpr int B_BYTES = B_ROWS * 128;
    static constexpr int MMAS = SPARSE ? 2 : 4;
    static constexpr int B_KSTEP = SPARSE ? 64 : 32;
    static constexpr int NBA = (BN + 127) / 128;          // scale-factor atoms (128 rows) a token tile touches
    static constexpr int SFA_BYTES = MMAS * 512;
    static constexpr int SFB_BYTES = NBA * MMAS * 512;    // all BN token rows, in both CTAs
    static constexpr int META_BYTES = SPARSE ? 2048 : 0;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;                       // operand ring slot
    static constexpr int SIDE_BYTES = SFA_BYTES + SFB_BYTES + META_BYTES;       // sideband ring slot
    static constexpr int NSB = 6;                                               // sideband ring slots
    static constexpr int ACC_STAGES = BN <= 192 ? 2 : 1;
    static constexpr int EPI_PITCH = 144;                 // 32 fp32 + 16 B pad per token row of a warp's transpose tile
    static constexpr int EPI_BYTES = 8 * 16 * EPI_PITCH;  // eight epilogue warps, 16 token rows each
    static constexpr int SMEM_BUDGET = 226 * 1024 - 1024 - EPI_BYTES - NSB * SIDE_BYTES - 512;
    static constexpr int SFA_COLS = MMAS * 4;
    static constexpr int SFB_COLS = MMAS * 4 * NBA;
    static constexpr int E_COLS = SPARSE ? 4 : 0;
    static constexpr int SF_SET = SFA_COLS + SFB_COLS + E_COLS;     // columns of one scale-factor slot in TMEM
    static constexpr int STAGES_SMEM = SMEM_BUDGET / STAGE_BYTES;
    static constexpr int STAGES = STAGES_SMEM > 10 ? 10 : STAGES_SMEM;
    static constexpr int TM_SF0 = ACC_STAGES * BN;                   // accumulators first, then the scale-factor slots
    static constexpr int NSLOT_TMEM = (512 - TM_SF0) / SF_SET;
    static constexpr int NSLOT = NSLOT_TMEM < STAGES ? NSLOT_TMEM : STAGES;   // slot ring, K block `it` uses slot it % NSLOT
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + NSB * SIDE_BYTES + EPI_BYTES + 512;
    static constexpr int TM_COLS = 512;
    static_assert(BN == 128 || BN == 192 || BN == 256, "token tile");
    static_assert(NSLOT >= 2 && TM_SF0 + NSLOT * SF_SET <= 512, "TMEM budget");
    static_assert(STAGES >= 3, "smem budget");
    static_assert((3 * STAGES + 2 * NSB + 4) * 8 <= 512, "barrier block");
};

struct KParams2 {
    const float* gA;
    const float* gB;
    void* C;
    int out_f, tok;
    int num_m2, num_n, kblocks;
    int out_mode;
    int a_tiled;
    const int* eblk;                     // grouped mode: expert of every 128-token block (a 256-token tile reads the entry of its first
                                         // block: the routing then pads every expert to 256 rows), null = plain GEMM
    const __nv_bfloat16* bias;           // out_mode 3: per-expert bias [E][out_f] (may be null)
    const float* row_w;                  // out_mode 3: weight of every routed row [tok] (may be null)
    int bias_ld;                         // features per bias row (the rest of out_f is padding without bias)
    // row-parallel GEMM + reduce-scatter by peer stores (out_mode 1): token row t goes to peer_out[t / tok_per_rank]
    // at local row t % tok_per_rank; the last CTA publishes peer_val in word peer_rank of every rank's flags
    int peer_n, peer_rank, tok_per_rank, peer_val;
    __nv_bfloat16* peer_out[8];
    int* peer_flags[8];
    int* peer_done;
    const int* peer_val_ptr;
    int peer_bpo;                        // token tiles per owner (0 = natural tile order)
    // out_mode 4: the weight rows are (gate, up) pairs (row 2i = gate feature i, 2i + 1 = up feature i); the epilogue forms
    // h = SwiGLU(gate, up) from the fp32 accumulators (+ bias), quantises h single-level per 32 features and writes packed
    // codes h_bytes[tok][h_feats / 2] and UE4M3 scale codes (128x4 atoms and / or the reference layout [h_feats/128][tok][4])
    uint8_t* h_bytes;
    uint8_t* h_sf_atoms;
    uint8_t* h_sf_ref;
    int h_feats;
    int act;
    int c_tma;                           // token-major bf16 output in this GPU's memory: the epilogue stores its tiles with TMA (tmC)
};

enum { SITE_SF = 5, SITE_SIDE = 6, SITE_MMA_SF = 7, SITE_SF_SLOT = 8 };
// Warp roles of the pair kernel, one kind of role per warpgroup so that registers can move between them
// (setmaxnreg is a warpgroup-wide instruction): the CTA starts with 96 registers per thread and the three
// service warpgroups hand most of theirs to the two epilogue warpgroups, which then hold a whole fp32
// accumulator slice (128 words per thread).  640 * 96 = 128 * (40 + 64 + 40) + 256 * 168.
enum { W_PROD_A = 0, W_PROD_B = 1, W_SIDE_W = 2, W_SIDE_B = 3, W_MMA = 16 };
constexpr int REGS_PROD = 40, REGS_SF = 64, REGS_MMA = 40, REGS_EPI = 168;

template <bool SPARSE, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(640, 1)
nvfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                       const __grid_constant__ CUtensorMap tmMETA, const __grid_constant__ CUtensorMap tmC,
                       const __grid_constant__ KParams2 p) {
    using C = Cfg2<SPARSE, BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_base_slot;
    griddep_launch_dependents();
    __shared__ float hmax_xch[8][2][16];      // out_mode 4: block maxima exchanged between partner epilogue warps

    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t side0 = smem0 + C::STAGES * C::STAGE_BYTES;
    const uint32_t epi0 = side0 + C::NSB * C::SIDE_BYTES;
    const uint32_t bars = epi0 + C::EPI_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };                               // leader's is the one used
    auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
    auto sfr_bar = [&](int s) { return bars + 8u * (2 * C::STAGES + s); };               // leader's
    auto sbf_bar = [&](int j) { return bars + 8u * (3 * C::STAGES + j); };               // sideband slot landed
    auto sbe_bar = [&](int j) { return bars + 8u * (3 * C::STAGES + C::NSB + j); };      // sideband slot copied out
    auto accf_bar = [&](int a) { return bars + 8u * (3 * C::STAGES + 2 * C::NSB + a); };
    auto acce_bar = [&](int a) { return bars + 8u * (3 * C::STAGES + 2 * C::NSB + 2 + a); };
    auto stageA = [&](int s) { return smem0 + (uint32_t)s * C::STAGE_BYTES; };
    auto stageB = [&](int s) { return stageA(s) + C::A_BYTES; };
    auto sideSFA = [&](int j) { return side0 + (uint32_t)j * C::SIDE_BYTES; };
    auto sideSFB = [&](int j) { return sideSFA(j) + C::SFA_BYTES; };
    auto sideMETA = [&](int j) { return sideSFB(j) + C::SFB_BYTES; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();      // 0 = leader of the pair
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(full_bar(s), 2);            // the leader's A and B producers announce both CTAs' bytes
            mbar_init(empty_bar(s), 1);
            mbar_init(sfr_bar(s), 8);             // 4 scale-factor warps of each CTA arrive on the leader's
        }
        for (int j = 0; j < C::NSB; j++) {
            mbar_init(sbf_bar(j), 2);             // the two sideband producers
            mbar_init(sbe_bar(j), 4);             // the four scale-factor warps
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(accf_bar(a), 1);
            mbar_init(acce_bar(a), 16);           // 8 epilogue warps of each CTA arrive on the leader's
        }
        fence_barrier_init();
        tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmSFA); tma_prefetch_desc(&tmSFB);
        if (SPARSE) tma_prefetch_desc(&tmMETA);
        if (p.c_tma) tma_prefetch_desc(&tmC);
    }
    if (warp == W_MMA) {
        tmem_alloc_pair(smem_u32(&tmem_base_slot), C::TM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int total_tiles = p.num_m2 * p.num_n;
    // Launched as a programmatic dependent: this grid may start while the kernel in front (an activation quantiser, the GEMM
    // of another layer) is still running. What that kernel produces - activations, their scale factors and globals, the
    // routing table of the grouped mode - is read only after griddep_wait(); barriers, tensor memory, tensor maps and the
    // weight side of the first ring revolution (weights are constants) are set up / loaded before.
    const bool dep_all = p.eblk != nullptr;
    // Token tile of a work item. With the reduce-scatter epilogue the token tiles are visited owner by owner in a rotation
    // that starts behind this rank: at any moment the ranks store into different owners and every rank's local and remote
    // tiles alternate, so the NVLink traffic is spread over the whole kernel instead of arriving in one burst per owner.
    auto tile_n = [&](int tile) {
        const int i = tile / p.num_m2;
        if (p.peer_bpo == 0) return i;
        int owner = p.peer_rank + 1 + i % p.peer_n;
        if (owner >= p.peer_n) owner -= p.peer_n;
        return owner * p.peer_bpo + i / p.peer_n;
    };
    // grouped mode: a 128-token block with expert id < 0 is unused capacity of a fixed-capacity routing; every
    // role of both CTAs skips its tiles (same test everywhere, so the ring and accumulator counters stay in step)
    auto tile_expert = [&](int n) { return p.eblk[n * (BN / 128)]; };
    auto tile_skipped = [&](int tile) { return p.eblk != nullptr && tile_expert(tile / p.num_m2) < 0; };
    const int atoms_per_rb = p.kblocks * C::MMAS;

    // Every role below handles two K blocks per barrier poll whenever the later one is ready as well: a
    // poll costs 100-200 cycles even on a completed barrier (measured with the round-trip probe), which
    // per K block is more than the tensor pipe needs for the MMAs. Ring barriers that are signalled in
    // ring order (empty, sbe, sfr) are polled for the later block only.
    if (warp < 4) {
        reg_dealloc<REGS_PROD>();
    if (warp == W_PROD_A || warp == W_PROD_B) {
        // ------------------------------------------------------------ operand producers (both CTAs)
        // warp 0 loads A, warp 10 loads B; one thread needs ~90 cycles to issue one TMA load (measured),
        // so every load of a stage has its own issuing warp. The loads of both CTAs complete on the
        // leader's full barrier, whose two arrivals (with the byte count of the pair) come from the
        // leader's producers; a peer load that lands first only drives the pending count negative.
        const bool isA = warp == W_PROD_A;
        if (!isA || dep_all) griddep_wait();             // activations (and the routing table) come from the kernel in front
        int stage = 0;
        uint32_t phase = 0;
        for (int tile = cluster_id; tile < total_tiles && !abort_flag; tile += num_clusters) {
            if (tile_skipped(tile)) continue;
            const int m2 = tile % p.num_m2, n = tile_n(tile);
            const int a_row0 = (p.eblk ? tile_expert(n) * p.out_f : 0) + m2 * 256 + (int)rank * 128;
            const int b_row0 = n * BN + (int)rank * C::B_ROWS;
            bool ok = true;
            for (int kb = 0; kb < p.kblocks;) {
                int s1 = stage + 1;
                uint32_t ph1 = phase;
                if (s1 == C::STAGES) { s1 = 0; ph1 ^= 1; }
                int nb = 2;
                if (kb + 1 >= p.kblocks || !mbar_try_wait(empty_bar(s1), ph1 ^ 1)) {
                    nb = 1;
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, &abort_flag, &g_status, SITE_PROD)) { ok = false; break; }
                }
                if (lane == 0) {
                    for (int u = 0; u < nb; u++) {
                        const int s = u ? s1 : stage;
                        const uint32_t fb = mapa_shared(full_bar(s), 0);
                        if (rank == 0) mbar_expect_tx(full_bar(s), 2u * (uint32_t)(isA ? C::A_BYTES : C::B_BYTES));
                        if (isA) {
                            if (p.a_tiled) tma_load_2d_pair(stageA(s), &tmA, fb, 0, ((a_row0 >> 7) * p.kblocks + kb + u) * 128);
                            else tma_load_2d_pair(stageA(s), &tmA, fb, (kb + u) * C::A_ROW, a_row0);
                        } else {
                            tma_load_2d_pair(stageB(s), &tmB, fb, (kb + u) * 128, b_row0);
                        }
                    }
                }
                __syncwarp();
                kb += nb;
                stage += nb;
                if (stage >= C::STAGES) { stage -= C::STAGES; phase ^= 1; }
            }
            if (!ok) break;
        }
    } else {
        // ------------------------------------------------------------ sideband producers (both CTAs)
        const bool isW = warp == W_SIDE_W;               // weight side: scale factors of A and metadata
        if (!isW || dep_all) griddep_wait();
        int slot = 0;
        uint32_t phase = 0;
        for (int tile = cluster_id; tile < total_tiles && !abort_flag; tile += num_clusters) {
            if (tile_skipped(tile)) continue;
            const int m2 = tile % p.num_m2, n = tile_n(tile);
            const int rb_a = ((p.eblk ? tile_expert(n) * p.out_f : 0) + m2 * 256 + (int)rank * 128) >> 7, rb_b = (n * BN) >> 7;
            bool ok = true;
            for (int kb = 0; kb < p.kblocks;) {
                int j1 = slot + 1;
                uint32_t ph1 = phase;
                if (j1 == C::NSB) { j1 = 0; ph1 ^= 1; }
                int nb = 2;
                if (kb + 1 >= p.kblocks || !mbar_try_wait(sbe_bar(j1), ph1 ^ 1)) {
                    nb = 1;
                    if (!mbar_wait(sbe_bar(slot), phase ^ 1, &abort_flag, &g_status, SITE_SIDE)) { ok = false; break; }
                }
                if (lane == 0) {
                    for (int u = 0; u < nb; u++) {
                        const int j = u ? j1 : slot;
                        const uint32_t fb = sbf_bar(j);
                        if (isW) {
                            mbar_expect_tx(fb, (uint32_t)(C::SFA_BYTES + C::META_BYTES));
                            tma_load_2d(sideSFA(j), &tmSFA, fb, 0, rb_a * atoms_per_rb + (kb + u) * C::MMAS);
                            if (SPARSE) tma_load_2d(sideMETA(j), &tmMETA, fb, 0, (rb_a * p.kblocks + kb + u) * 4);
                        } else {
                            mbar_expect_tx(fb, (uint32_t)C::SFB_BYTES);
#pragma unroll
                            for (int nbk = 0; nbk < C::NBA; nbk++)
                                tma_load_2d(sideSFB(j) + nbk * C::MMAS * 512, &tmSFB, fb, 0, (rb_b + nbk) * atoms_per_rb + (kb + u) * C::MMAS);
                        }
                    }
                }
                __syncwarp();
                kb += nb;
                slot += nb;
                if (slot >= C::NSB) { slot -= C::NSB; phase ^= 1; }
            }
            if (!ok) break;
        }
    }
    } else if (warp >= 16) {
        reg_dealloc<REGS_MMA>();
        // ------------------------------------------------------------ MMA issuer (leader CTA only); warps 17-19 only fill the warpgroup
        // One thread runs the whole issue loop: no warp-wide broadcast or re-convergence sits between a
        // barrier wait and the MMAs it gates.
        if (warp == W_MMA && rank == 0 && lane == 0) {
            const uint32_t idesc = make_idesc_nvf4(BN, SPARSE, 256);
            if (dep_all) griddep_wait();
            int stage = 0, acc = 0, tslot = 0;
            uint32_t phase = 0, acc_phase = 0;
            for (int tile = cluster_id; tile < total_tiles && !abort_flag; tile += num_clusters) {
                if (tile_skipped(tile)) continue;
                // a 192-token tile starts 0 or 64 rows into a 128-row scale-factor atom: 0 or 2 columns in
                const uint32_t sfb_coloff = (uint32_t)(((tile_n(tile) * BN) & 127) >> 5);
                if (!mbar_wait_thread(acce_bar(acc), acc_phase ^ 1, &abort_flag, &g_status, SITE_MMA_ACC)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                bool ok = true;
                for (int kb = 0; kb < p.kblocks;) {
                    int s1 = stage + 1;
                    uint32_t ph1 = phase;
                    if (s1 == C::STAGES) { s1 = 0; ph1 ^= 1; }
                    int nb = 2;
                    // operands of both blocks landed (loads complete in any order) and the scale factors
                    // of the later block (hence of both) are in tensor memory; four blocks per poll were
                    // measured too and were slower
                    if (kb + 1 >= p.kblocks || !mbar_try_wait3(full_bar(stage), phase, full_bar(s1), ph1, sfr_bar(s1), ph1)) {
                        nb = 1;
                        if (!mbar_try_wait2(full_bar(stage), phase, sfr_bar(stage), phase) &&
                            (!mbar_wait_thread(full_bar(stage), phase, &abort_flag, &g_status, SITE_MMA_FULL) ||
                             !mbar_wait_thread(sfr_bar(stage), phase, &abort_flag, &g_status, SITE_MMA_SF))) { ok = false; break; }
                    }
                    tc_fence_after();
                    for (int u = 0; u < nb; u++) {
                        const int s = u ? s1 : stage;
                        const uint32_t t_sfa = tmem_base + C::TM_SF0 + tslot * C::SF_SET;
                        const uint32_t t_sfb = t_sfa + C::SFA_COLS + sfb_coloff, t_e = t_sfa + C::SFA_COLS + C::SFB_COLS;
                        if (++tslot == C::NSLOT) tslot = 0;
#pragma unroll
                        for (int i = 0; i < C::MMAS; i++) {
                            const uint64_t adesc = make_smem_desc(stageA(s) + i * 32, SPARSE ? 512 : 1024, 16, SPARSE ? 4 : 2);
                            const uint64_t bdesc = make_smem_desc(stageB(s) + i * C::B_KSTEP, 1024, 16, 2);
                            const uint32_t accum = (kb + u > 0 || i > 0) ? 1u : 0u;
                            if (SPARSE)
                                tc_mma_nvf4_sp_pair(d_tmem, adesc, bdesc, idesc, t_sfa + 4 * i, t_sfb + 4 * C::NBA * i, t_e + 2 * i, accum);
                            else
                                tc_mma_nvf4_pair(d_tmem, adesc, bdesc, idesc, t_sfa + 4 * i, t_sfb + 4 * C::NBA * i, accum);
                        }
                        tc_commit_pair(empty_bar(s), 3);
                    }
                    kb += nb;
                    stage += nb;
                    if (stage >= C::STAGES) { stage -= C::STAGES; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit_pair(accf_bar(acc), 3);
                if (++acc == C::ACC_STAGES) { acc = 0; acc_phase ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp < 8) {
        reg_dealloc<REGS_SF>();
        // ------------------------------------------------------------ scale-factor warps (both CTAs)
        const int q = warp & 3;
        const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
        if (dep_all) griddep_wait();
        // K block number `it` (counted over all tiles) uses operand stage it % STAGES, sideband slot it % NSB and
        // tensor-memory slot it % NSLOT. Its tensor-memory slot is free once the MMAs of K block it - NSLOT have
        // completed, which the empty barrier of THAT block's stage signals (completions come in ring order).
        int stage = 0, slot = 0, tslot = 0;
        uint32_t sphase = 0, it = 0;
        for (int tile = cluster_id; tile < total_tiles && !abort_flag; tile += num_clusters) {
            if (tile_skipped(tile)) continue;
            bool ok = true;
            for (int kb = 0; kb < p.kblocks;) {
                int s1 = stage + 1, j1 = slot + 1, t1 = tslot + 1;
                uint32_t sph1 = sphase;
                if (s1 == C::STAGES) s1 = 0;
                if (j1 == C::NSB) { j1 = 0; sph1 ^= 1; }
                if (t1 == C::NSLOT) t1 = 0;
                // barrier / parity that says "the MMAs of K block c have completed"
                auto done_bar = [&](uint32_t c) { return empty_bar((int)(c % C::STAGES)); };
                auto done_par = [&](uint32_t c) { return (c / C::STAGES) & 1u; };
                int nb = 1;
                if (kb + 1 < p.kblocks) {          // both sideband slots landed (any order) and the later slot is free
                    const bool two = it + 1 >= (uint32_t)C::NSLOT
                                         ? mbar_try_wait3(sbf_bar(slot), sphase, sbf_bar(j1), sph1, done_bar(it + 1 - C::NSLOT),
                                                          done_par(it + 1 - C::NSLOT))
                                         : mbar_try_wait2(sbf_bar(slot), sphase, sbf_bar(j1), sph1);
                    if (two) nb = 2;
                }
                if (nb == 1) {
                    if (!mbar_wait(sbf_bar(slot), sphase, &abort_flag, &g_status, SITE_SF, QB_BACKOFF_SF)) { ok = false; break; }
                    if (it >= (uint32_t)C::NSLOT &&
                        !mbar_wait(done_bar(it - C::NSLOT), done_par(it - C::NSLOT), &abort_flag, &g_status, SITE_SF_SLOT)) { ok = false; break; }
                }
                tc_fence_after();
                {
                    for (int u = 0; u < nb; u++) {
                        const int j = u ? j1 : slot, ts = u ? t1 : tslot;
                        const uint32_t sf = sideSFA(j) + lane * 16;       // this lane's 16 bytes of every atom
                        const uint32_t t_sfa = tmem_base + C::TM_SF0 + ts * C::SF_SET + lane_sel;
                        const uint32_t t_sfb = t_sfa + C::SFA_COLS, t_e = t_sfb + C::SFB_COLS;
                        // SFA: MMAS atoms -> MMAS*4 consecutive columns
                        {
                            uint32_t a[C::MMAS * 4];
#pragma unroll
                            for (int i = 0; i < C::MMAS; i++) {
                                uint4 v = lds_v4(sf + i * 512);
                                a[4 * i] = v.x; a[4 * i + 1] = v.y; a[4 * i + 2] = v.z; a[4 * i + 3] = v.w;
                            }
                            if constexpr (C::MMAS == 2) tc_st_32x8(t_sfa, a); else tc_st_32x16(t_sfa, a);
                        }
                        // SFB: column 4*NBA*i + 4*nb + c  <-  atom (nb, i), word c
#pragma unroll
                        for (int h = 0; h < (C::MMAS * C::NBA * 4) / 8; h++) {
                            uint32_t b[8];
#pragma unroll
                            for (int w = 0; w < 2; w++) {
                                const int g = h * 2 + w;               // group of 4 columns
                                const int i = g / C::NBA, nbk = g % C::NBA;
                                uint4 v = lds_v4(sf + C::SFA_BYTES + (nbk * C::MMAS + i) * 512);
                                b[4 * w] = v.x; b[4 * w + 1] = v.y; b[4 * w + 2] = v.z; b[4 * w + 3] = v.w;
                            }
                            tc_st_32x8(t_sfb + 8 * h, b);
                        }
                        if constexpr (SPARSE) {
                            uint32_t e[4];
                            uint4 v = lds_v4(sideMETA(j) + (q * 32 + lane) * 16);
                            e[0] = v.x; e[1] = v.y; e[2] = v.z; e[3] = v.w;
                            tc_st_32x4(t_e, e);
                        }
                    }
                    tc_wait_st();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster(mapa_shared(sfr_bar(stage), 0));
                    mbar_arrive(sbe_bar(slot));
                    if (nb == 2) {
                        mbar_arrive_cluster(mapa_shared(sfr_bar(s1), 0));
                        mbar_arrive(sbe_bar(j1));
                    }
                }
                kb += nb;
                it += nb;
                stage += nb;
                if (stage >= C::STAGES) stage -= C::STAGES;
                slot += nb;
                if (slot >= C::NSB) { slot -= C::NSB; sphase ^= 1; }
                tslot += nb;
                if (tslot >= C::NSLOT) tslot -= C::NSLOT;
            }
            if (!ok) break;
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own rows)
        // Eight warps: warps 8-11 drain the first half of the tile's columns, warps 12-15 the second half;
        // a warp reads the TMEM lane quadrant (warp % 4) it is allowed to.
        reg_alloc<REGS_EPI>();
        griddep_wait();                                  // token globals, routing weights; and nothing is stored before
        const int q = warp & 3;
        const int half = warp >= 12 ? 1 : 0;
        const int ew = warp - 8;
        const int r_in_tile = q * 32 + lane;
        const uint32_t stg_s = epi0 + ew * (16 * C::EPI_PITCH);
        int acc = 0;
        uint32_t acc_phase = 0;
        constexpr int HCOLS = BN / 2;          // columns per warp
        constexpr int NCH = HCOLS / 16;        // chunks of 16 columns
        for (int tile = cluster_id; tile < total_tiles && !abort_flag; tile += num_clusters) {
            if (tile_skipped(tile)) continue;
            const int m2 = tile % p.num_m2, n = tile_n(tile);
            const int n0 = n * BN + half * HCOLS;          // first token column of this warp
            const int o0 = m2 * 256 + (int)rank * 128;     // first output feature of this CTA's half
            const int o = o0 + r_in_tile;
            const int a_base = p.eblk ? tile_expert(n) * p.out_f : 0;      // first row of this tile's expert in A / gA / bias
            // per-tile constants first, so their latency hides behind the accumulator wait; the two forms of the epilogue
            // need different ones (stm: 16x256b loads + stmatrix; otherwise one feature per lane)
            const bool stm = C::ACC_STAGES == 1 && (p.out_mode == 1 || p.out_mode == 3);
            const float ga = (p.gA && !stm) ? __ldg(p.gA + a_base + o) : 1.f;
            float gbv[NCH], rwv[NCH];
#pragma unroll
            for (int c = 0; c < NCH; c++) {
                const int col = n0 + 16 * c + (lane & 15);
                gbv[c] = (p.gB && col < p.tok) ? __ldg(p.gB + col) : 1.f;
                rwv[c] = (p.out_mode == 3 && p.row_w && col < p.tok) ? __ldg(p.row_w + col) : 1.f;
            }
            // out_mode 3: the bias of the 8 features this lane emits per token in the transposed phase
            float bias8[8];
#pragma unroll
            for (int e = 0; e < 8; e++) bias8[e] = 0.f;
            const int f8 = o0 + q * 32 + (lane & 3) * 8;       // bias rows hold bias_ld (a multiple of 8) valid features
            if (!stm && (p.out_mode == 3 || p.out_mode == 4) && p.bias && f8 + 8 <= p.bias_ld) {
                const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + (size_t)(p.eblk ? tile_expert(n) : 0) * p.bias_ld + f8));
                const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
                for (int e = 0; e < 4; e++) { const float2 f = __bfloat1622float2(bh[e]); bias8[2 * e] = f.x; bias8[2 * e + 1] = f.y; }
            }
            // the stmatrix epilogue's per-thread constants: its four features fr + 8m (TMEM lanes lane / 4 + 8m of the quadrant)
            const int fr = o0 + q * 32 + (lane >> 2);
            float ga4[4], bi4[4];
#pragma unroll
            for (int m = 0; m < 4; m++) {
                ga4[m] = (p.gA && stm) ? __ldg(p.gA + a_base + fr + 8 * m) : 1.f;
                bi4[m] = (stm && p.out_mode == 3 && p.bias && fr + 8 * m < p.bias_ld)
                             ? __bfloat162float(p.bias[(size_t)(p.eblk ? tile_expert(n) : 0) * p.bias_ld + fr + 8 * m]) : 0.f;
            }
            if (!mbar_wait(accf_bar(acc), acc_phase, &abort_flag, &g_status, SITE_EPI, QB_BACKOFF)) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + (uint32_t)(acc * BN + half * HCOLS) + ((uint32_t)(q * 32) << 16);
            const uint32_t acce_leader = mapa_shared(acce_bar(acc), 0);
            uint32_t ra[16], rb[16];
            if constexpr (C::ACC_STAGES != 1) tc_ld_32x16(t_acc, ra);
            auto emit = [&](const uint32_t (&r)[16], int c) {
                const int c0 = 16 * c;
                const float gbl = gbv[c];
                if (p.out_mode == 0) {
                    __nv_bfloat16* Cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)o * p.tok;
                    uint32_t pk[8];
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        float g0 = __shfl_sync(0xffffffffu, gbl, j), g1 = __shfl_sync(0xffffffffu, gbl, j + 1);
                        pk[j / 2] = pack_bf16x2((__uint_as_float(r[j]) * ga) * g0, (__uint_as_float(r[j + 1]) * ga) * g1);
                    }
                    const int col0 = n0 + c0;
                    if (col0 + 16 <= p.tok && (p.tok & 7) == 0) {
#pragma unroll
                        for (int v = 0; v < 2; v++)
                            *reinterpret_cast<uint4*>(Cp + col0 + 8 * v) = make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (col0 + j < p.tok) {
                                uint32_t w = pk[j / 2];
                                reinterpret_cast<uint16_t*>(Cp)[col0 + j] = (j & 1) ? (uint16_t)(w >> 16) : (uint16_t)(w & 0xffff);
                            }
                    }
                } else {
                    // transpose a 32(out) x 16(tok) fp32 block through shared memory: phase 1 scales by the
                    // row global and stores one word per value (conflict-free), phase 2 reads 8 features of
                    // one token, scales by the token global, packs to bf16 and stores 16 bytes token-major
#pragma unroll
                    for (int j = 0; j < 16; j++) sts_u32(stg_s + j * C::EPI_PITCH + lane * 4, __float_as_uint(__uint_as_float(r[j]) * ga));
                    __syncwarp();
                    __nv_bfloat16* Cp = reinterpret_cast<__nv_bfloat16*>(p.C) + o0 + q * 32 + (lane & 3) * 8;
                    if (p.out_mode == 4) {
                        // SwiGLU + single-level per-32 quantiser in the epilogue (the reference's fused gate/up GEMM,
                        // cuda/sparse_fp4_lib.cu:1679-1868). After the transpose a lane holds 8 consecutive rows of one token
                        // = 4 (gate, up) pairs; the 4 lanes of a token hold this warp's 16 h features, and the partner warp
                        // (lane quadrant q ^ 1) holds the other 16 of the 32-feature scale block.
                        float hv[2][4], bm[2];
#pragma unroll
                        for (int it = 0; it < 2; it++) {
                            const int trow = (it * 32 + lane) >> 2;
                            const float gt = __shfl_sync(0xffffffffu, gbl, trow);
                            const uint4 lo = lds_v4(stg_s + trow * C::EPI_PITCH + (lane & 3) * 32);
                            const uint4 hi = lds_v4(stg_s + trow * C::EPI_PITCH + (lane & 3) * 32 + 16);
                            const float f[8] = {__uint_as_float(lo.x) * gt + bias8[0], __uint_as_float(lo.y) * gt + bias8[1],
                                                __uint_as_float(lo.z) * gt + bias8[2], __uint_as_float(lo.w) * gt + bias8[3],
                                                __uint_as_float(hi.x) * gt + bias8[4], __uint_as_float(hi.y) * gt + bias8[5],
                                                __uint_as_float(hi.z) * gt + bias8[6], __uint_as_float(hi.w) * gt + bias8[7]};
                            float m = 0.f;
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                hv[it][k] = p.act == 0 ? swiglu_h<0>(f[2 * k], f[2 * k + 1]) : swiglu_h<1>(f[2 * k], f[2 * k + 1]);
                                m = fmaxf(m, fabsf(hv[it][k]));
                            }
                            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                            bm[it] = m;
                            if ((lane & 3) == 0) hmax_xch[ew][c & 1][trow] = m;
                        }
                        // the two buffers alternate by chunk: a warp rewrites a buffer only after the barrier of the chunk in
                        // between, which its partner reaches after it has read that buffer
                        named_bar_sync(1 + (ew >> 1), 64);
                        const int blk32 = ((o0 >> 1) + q * 16) >> 5;          // scale block of these features within the row of h
#pragma unroll
                        for (int it = 0; it < 2; it++) {
                            const int trow = (it * 32 + lane) >> 2;
                            const float blockmax = fmaxf(bm[it], hmax_xch[ew ^ 1][c & 1][trow]);
                            // h is only defined up to the accumulation order of the tensor core, so the quotient by the
                            // block scale is one multiply by its reciprocal and the hardware E2M1 conversion (a tenth of
                            // the instructions of the exact-quotient path of the stand-alone quantisers)
                            const uint32_t code = enc_ue4m3_bits(__fdiv_rn(blockmax, 6.f));
                            const uint32_t w = pack4_e2m1_rcp(hv[it], code ? __frcp_rn(dec_ue4m3(code)) : 0.f);
                            const int base = lane & ~3;
                            const uint32_t w1 = __shfl_sync(0xffffffffu, w, base + 1), w2 = __shfl_sync(0xffffffffu, w, base + 2),
                                           w3 = __shfl_sync(0xffffffffu, w, base + 3);
                            const int col = n0 + c0 + trow;
                            if ((lane & 3) == 0 && col < p.tok) {
                                uint8_t* dst = p.h_bytes + (size_t)col * (p.h_feats >> 1) + (((o0 >> 1) + q * 16) >> 1);
                                *reinterpret_cast<uint2*>(dst) = make_uint2(w | (w1 << 16), w2 | (w3 << 16));
                                if ((q & 1) == 0) {
                                    if (p.h_sf_atoms) p.h_sf_atoms[sf_atom_offset(col, blk32, kpad256(p.h_feats) / 128)] = (uint8_t)code;
                                    if (p.h_sf_ref) p.h_sf_ref[((size_t)(blk32 >> 2) * p.tok + col) * 4 + (blk32 & 3)] = (uint8_t)code;
                                }
                            }
                        }
                        __syncwarp();
                        return;
                    }
#pragma unroll
                    for (int it = 0; it < 2; it++) {
                        const int trow = (it * 32 + lane) >> 2;
                        const float gt = __shfl_sync(0xffffffffu, gbl, trow);
                        const uint4 lo = lds_v4(stg_s + trow * C::EPI_PITCH + (lane & 3) * 32);
                        const uint4 hi = lds_v4(stg_s + trow * C::EPI_PITCH + (lane & 3) * 32 + 16);
                        float f[8] = {__uint_as_float(lo.x) * gt, __uint_as_float(lo.y) * gt, __uint_as_float(lo.z) * gt,
                                      __uint_as_float(lo.w) * gt, __uint_as_float(hi.x) * gt, __uint_as_float(hi.y) * gt,
                                      __uint_as_float(hi.z) * gt, __uint_as_float(hi.w) * gt};
                        if (p.out_mode == 3) {
                            const float rw = __shfl_sync(0xffffffffu, rwv[c], trow);
#pragma unroll
                            for (int e = 0; e < 8; e++) f[e] = (f[e] + bias8[e]) * rw;
                        }
                        uint4 val;
                        val.x = pack_bf16x2(f[0], f[1]);
                        val.y = pack_bf16x2(f[2], f[3]);
                        val.z = pack_bf16x2(f[4], f[5]);
                        val.w = pack_bf16x2(f[6], f[7]);
                        const int col = n0 + c0 + trow;
                        if (col < p.tok) {
                            if (p.peer_n) {
                                // the partial row goes straight into the memory of the rank that owns the token (a plain
                                // 16-byte store over NVLink, or a local one for this rank's own range)
                                const int owner = col / p.tok_per_rank;
                                stg_v4(p.peer_out[owner] + (size_t)(col - owner * p.tok_per_rank) * p.out_f + (o0 + q * 32 + (lane & 3) * 8), val);
                            } else {
                                stg_v4(Cp + (size_t)col * p.out_f, val);
                            }
                        }
                    }
                    __syncwarp();
                }
            };
            if constexpr (C::ACC_STAGES == 1) {
              if (stm) {
                // Token-major bf16 output of the one-accumulator tile. The slice is read in the 16x256b shape: a thread then
                // holds, for every group of 8 tokens, two adjacent tokens of four features (lanes t/4 + 8m), which is the
                // fragment layout stmatrix stores transposed. Scale, round to bf16, store the four 8x8 matrices of a group
                // transposed into a 512-byte shared-memory tile (token rows of 32 features, 16-byte chunks XOR-swizzled so
                // that neither the stores nor the reads conflict), read 16 bytes per lane and store them token-major. Half
                // the shared-memory traffic and a third fewer instructions than staging fp32, and no conversion after the
                // shared-memory round trip.
                uint32_t hf[4][32];                    // [16-lane half * 2 + 64-column half]
                tc_ld_16x256b_x8(t_acc, hf[0]);
                tc_ld_16x256b_x8(t_acc + 64, hf[1]);
                tc_ld_16x256b_x8(t_acc + (16u << 16), hf[2]);
                tc_ld_16x256b_x8(t_acc + (16u << 16) + 64, hf[3]);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acce_leader);
                const uint32_t sbuf = epi0 + ew * 2048;               // two sets of two 512-byte tiles per warp
                const int st_i = lane & 7, rd_i = lane >> 2;
                const uint32_t st_off = (uint32_t)(st_i * 64 + (((lane >> 3) ^ ((st_i >> 1) & 3)) * 16));
                const uint32_t rd_off = (uint32_t)(rd_i * 64 + (((lane & 3) ^ ((rd_i >> 1) & 3)) * 16));
                const int fcol = o0 + q * 32 + (lane & 3) * 8;          // first of the 8 features this lane stores
                // Eight rounds of two groups (16 tokens), alternating between the two sets of staging tiles. With the TMA
                // store one lane hands the 16 x 32 tile (1 KB, 64-byte rows in the 64-byte swizzle the stmatrix addresses
                // follow) to the copy engine and the warp goes on with the next round; the set is written again two rounds
                // later, after the store that read it has finished reading. Without it (peer destinations) every lane reads
                // 16 bytes back and stores them itself.
#pragma unroll
                for (int r = 0; r < 8; r++) {
                    const uint32_t sset = sbuf + (uint32_t)(r & 1) * 1024;
                    if (p.c_tma) {
                        if (lane == 0) bulk_wait_read<1>();
                        __syncwarp();
                    }
#pragma unroll
                    for (int u = 0; u < 2; u++) {
                        const int j = r * 2 + u, k = j & 7;
                        const uint32_t* lo = hf[j >> 3];
                        const uint32_t* hi = hf[2 + (j >> 3)];
                        const int sl = 8 * (j & 1) + 2 * (lane & 3);  // gbv[c] holds the global of column 16c + (lane & 15)
                        const float g0 = __shfl_sync(0xffffffffu, gbv[j >> 1], sl), g1 = __shfl_sync(0xffffffffu, gbv[j >> 1], sl + 1);
                        float w0 = 1.f, w1 = 1.f;
                        if (p.out_mode == 3) {
                            w0 = __shfl_sync(0xffffffffu, rwv[j >> 1], sl);
                            w1 = __shfl_sync(0xffffffffu, rwv[j >> 1], sl + 1);
                        }
                        const uint32_t v[4][2] = {{lo[4 * k], lo[4 * k + 1]}, {lo[4 * k + 2], lo[4 * k + 3]},
                                                  {hi[4 * k], hi[4 * k + 1]}, {hi[4 * k + 2], hi[4 * k + 3]}};
                        uint32_t pk[4];
#pragma unroll
                        for (int m = 0; m < 4; m++) {
                            float a = __uint_as_float(v[m][0]), b = __uint_as_float(v[m][1]);     // two adjacent tokens of one feature
                            mul_f32x2(a, b, ga4[m], ga4[m]);
                            mul_f32x2(a, b, g0, g1);
                            if (p.out_mode == 3) {
                                add_f32x2(a, b, bi4[m], bi4[m]);
                                mul_f32x2(a, b, w0, w1);
                            }
                            pk[m] = pack_bf16x2(a, b);
                        }
                        stmatrix_x4_trans(sset + u * 512 + st_off, pk[0], pk[1], pk[2], pk[3]);
                    }
                    if (p.c_tma) {
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&tmC, sset, (o0 + q * 32) * 2, n0 + 16 * r);
                            bulk_commit();
                        }
                    } else {
                        __syncwarp();
#pragma unroll
                        for (int u = 0; u < 2; u++) {
                            const int col = n0 + 8 * (r * 2 + u) + rd_i;
                            const uint4 val = lds_v4(sset + u * 512 + rd_off);
                            if (col < p.tok) {
                                if (p.peer_n) {
                                    // the partial row goes straight into the memory of the rank that owns the token (a plain
                                    // 16-byte store over NVLink, or a local one for this rank's own range)
                                    const int owner = col / p.tok_per_rank;
                                    stg_v4(p.peer_out[owner] + (size_t)(col - owner * p.tok_per_rank) * p.out_f + fcol, val);
                                } else {
                                    stg_v4(reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)col * p.out_f + fcol, val);
                                }
                            }
                        }
                        __syncwarp();
                    }
                }
                acc_phase ^= 1;
              } else {
                // one accumulator: all loads first, then give it back, then the (slow) conversions and stores
                uint32_t held[NCH][16];
#pragma unroll
                for (int c = 0; c < NCH; c++) tc_ld_32x16(t_acc + 16 * c, held[c]);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acce_leader);
#pragma unroll
                for (int c = 0; c < NCH; c++) emit(held[c], c);
                acc_phase ^= 1;
              }
            } else {
#pragma unroll
            for (int c = 0; c < NCH; c += 2) {
                tc_wait_ld();
                tc_ld_32x16(t_acc + 16 * (c + 1), rb);
                emit(ra, c);
                tc_wait_ld();
                if (c + 2 < NCH) {
                    tc_ld_32x16(t_acc + 16 * (c + 2), ra);
                } else {
                    // every column is in registers: hand the accumulator back before the last stores
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(acce_leader);
                }
                emit(rb, c + 1);
            }
            if (++acc == C::ACC_STAGES) { acc = 0; acc_phase ^= 1; }
            }
        }
    }

    // teardown: no CTA may leave while its partner can still signal its barriers, nor while one of its TMA stores is in flight
    if (p.c_tma && warp >= 8 && warp < 16 && lane == 0) bulk_wait<0>();
    tc_fence_before();
    cluster_sync_all();
    if (warp == W_MMA) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, C::TM_COLS);
    }
    if (p.peer_n && threadIdx.x == 0) {
        // every store of this CTA is ordered before the cluster barrier above; the system-scope fence after it is
        // cumulative, so when the last CTA of the grid publishes the flag, all partial rows have landed at their owners
        __threadfence_system();
        if (atomicAdd(p.peer_done, 1) == (int)gridDim.x - 1) {
            atomicExch(p.peer_done, 0);
            __threadfence_system();
            const int val = p.peer_val_ptr ? *p.peer_val_ptr : p.peer_val;
            // one system-scope fence orders every partial row before the flag words, which then go out as relaxed stores
            // (a release store per rank would fence again each time: ~2 us apiece)
            for (int r = 0; r < p.peer_n; r++)
                asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p.peer_flags[r] + p.peer_rank), "r"(val) : "memory");
        }
    }
}

// split-K finish: C = bf16(Cf[tok][out] * gA[out] * gB[tok]) in either output layout
__global__ void splitk_finish_kernel(const float* __restrict__ Cf, const float* __restrict__ gA, const float* __restrict__ gB,
                                     __nv_bfloat16* __restrict__ C, int out_f, int tok, int out_mode) {
    size_t n = (size_t)out_f * tok;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        int o = (int)(i % out_f);
        int t = (int)(i / out_f);
        float v = (Cf[i] * (gA ? gA[o] : 1.f)) * (gB ? gB[t] : 1.f);
        if (out_mode == 0) C[(size_t)o * tok + t] = __float2bfloat16_rn(v);
        else C[i] = __float2bfloat16_rn(v);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

static int make_map_u8(CUtensorMap* m, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes,
                       uint32_t box_rows, CUtensorMapSwizzle sw) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return QB_ERR_DRIVER;
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_bytes, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? QB_OK : QB_ERR_DRIVER;
}

template <bool SPARSE, int BN>
static int set_attr() {
    return (int)cudaFuncSetAttribute(nvfp4_gemm_kernel<SPARSE, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg<SPARSE, BN>::SMEM_BYTES);
}

int gemm_init_attrs() {
    static int rc = -1;
    static std::once_flag once;
    std::call_once(once, [] {
        int r = 0;
#define QB_SA(BN) if (!r) r = set_attr<false, BN>(); if (!r) r = set_attr<true, BN>();
        QB_SA(16) QB_SA(32) QB_SA(64) QB_SA(128) QB_SA(256)
#undef QB_SA
        rc = r;
    });
    return rc;
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// The pair kernel's TMA box for B is 128 rows; a token count below 128 would need a shorter box.
static bool b_tail_ok(int tok) { return tok >= 128; }

template <bool SPARSE, int BN>
static int launch(const GemmArgs& a, KParams kp, cudaStream_t st) {
    using C = Cfg<SPARSE, BN>;
    CUtensorMap tmA, tmB;
    // tiled A: a matrix of (rows * K blocks) tile rows of A_ROW bytes, so one box is one contiguous tile
    int rc = a.a_tiled
                 ? make_map_u8(&tmA, a.A, (uint64_t)C::A_ROW, (uint64_t)a.a_rows * kp.kblocks, C::A_ROW, 128,
                               SPARSE ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B)
                 : make_map_u8(&tmA, a.A, (uint64_t)(SPARSE ? a.K / 4 : a.K / 2), (uint64_t)a.a_rows, C::A_ROW, 128,
                               SPARSE ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    kp.a_tiled = a.a_tiled;
    const uint32_t b_rows = a.tok < BN ? (uint32_t)a.tok : (uint32_t)BN;   // box never taller than the tensor
    kp.b_box_bytes = (int)(b_rows * 128);
    rc = make_map_u8(&tmB, a.B, (uint64_t)a.K / 2, (uint64_t)a.tok, 128, b_rows, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    int total = kp.num_m * kp.num_n * kp.splits;
    int grid = total < sm_count() ? total : sm_count();
    if (kp.cluster_red) grid = total;            // one cluster of `splits` CTAs per output tile (the caller checked that it fits)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(NTHREADS1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // see griddep_wait() in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (kp.cluster_red) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = (unsigned)kp.splits;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    return (int)cudaLaunchKernelEx(&cfg, nvfp4_gemm_kernel<SPARSE, BN>, tmA, tmB, kp);
}

// Clusters of `size` CTAs of the single-CTA kernel (one CTA per SM, all its shared memory) that can be resident at once: the
// SMs of a GPC do not always divide into clusters, so this is less than SMs / size (asked once per size and kernel).
template <bool SPARSE, int BN>
static int max_clusters(int size) {
    using C = Cfg<SPARSE, BN>;
    static int cache[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    if (size < 1 || size > 8) return 0;
    if (cache[size]) return cache[size];
    if (gemm_init_attrs()) return 0;               // the query needs the kernel's shared-memory attribute in place
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(size * 64));
    cfg.blockDim = dim3(NTHREADS1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, nvfp4_gemm_kernel<SPARSE, BN>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
    cache[size] = n > 0 ? n : -1;
    return cache[size];
}


static int make_map_u32_rows(CUtensorMap* m, const void* base, uint64_t rows, uint32_t box_rows) {
    // [rows][128 x u32] = rows of 512 bytes (scale-factor atoms, quarter blocks of metadata), no swizzle
    EncodeTiledFn enc = get_encode();
    if (!enc) return QB_ERR_DRIVER;
    cuuint64_t dims[2] = {128, rows};
    cuuint64_t strides[1] = {512};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? QB_OK : QB_ERR_DRIVER;
}

template <bool SPARSE, int BN>
static int launch_pair(const GemmArgs& a, cudaStream_t st) {
    using C = Cfg2<SPARSE, BN>;
    static int attr_rc = -1;
    static std::once_flag once;
    std::call_once(once, [] {
        attr_rc = (int)cudaFuncSetAttribute(nvfp4_gemm_pair_kernel<SPARSE, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    });
    if (attr_rc) return attr_rc;
    const int kblocks = (a.K + 255) / 256;
    const int atoms_per_rb = kblocks * C::MMAS;
    CUtensorMap tmA, tmB, tmSFA, tmSFB, tmMETA, tmC;
    int rc = a.a_tiled
                 ? make_map_u8(&tmA, a.A, (uint64_t)C::A_ROW, (uint64_t)a.a_rows * kblocks, C::A_ROW, 128,
                               SPARSE ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B)
                 : make_map_u8(&tmA, a.A, (uint64_t)(SPARSE ? a.K / 4 : a.K / 2), (uint64_t)a.a_rows, C::A_ROW, 128,
                               SPARSE ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const uint32_t b_rows = (uint32_t)C::B_ROWS;
    if ((rc = make_map_u8(&tmB, a.B, (uint64_t)a.K / 2, (uint64_t)a.tok, 128, b_rows, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    if ((rc = make_map_u32_rows(&tmSFA, a.sfa, (uint64_t)(a.a_rows / 128) * atoms_per_rb, C::MMAS))) return rc;
    if ((rc = make_map_u32_rows(&tmSFB, a.sfb, (uint64_t)((a.tok + 127) / 128) * atoms_per_rb, C::MMAS))) return rc;
    if (SPARSE) {
        if ((rc = make_map_u32_rows(&tmMETA, a.meta, (uint64_t)(a.a_rows / 128) * kblocks * 4, 4))) return rc;
    } else {
        tmMETA = tmSFA;
    }
    KParams2 kp;
    kp.gA = a.gA; kp.gB = a.gB; kp.C = a.C; kp.out_f = a.out_f; kp.tok = a.tok;
    kp.num_m2 = a.out_f / 256; kp.num_n = (a.tok + BN - 1) / BN; kp.kblocks = kblocks; kp.out_mode = a.out_mode;
    kp.a_tiled = a.a_tiled;
    kp.eblk = a.eblk; kp.bias = (const __nv_bfloat16*)a.bias; kp.row_w = a.row_w; kp.bias_ld = a.bias_ld > 0 ? a.bias_ld : a.out_f;
    kp.peer_n = a.peer_n; kp.peer_rank = a.peer_rank; kp.tok_per_rank = a.tok_per_rank; kp.peer_val = a.peer_val; kp.peer_done = a.peer_done; kp.peer_val_ptr = a.peer_val_ptr;
    kp.peer_bpo = (a.peer_n && a.tok_per_rank % BN == 0 && kp.num_n == (a.tok_per_rank / BN) * a.peer_n) ? a.tok_per_rank / BN : 0;
    for (int r = 0; r < 8; r++) { kp.peer_out[r] = (__nv_bfloat16*)a.peer_out[r]; kp.peer_flags[r] = a.peer_flags[r]; }
    kp.h_bytes = (uint8_t*)a.h_bytes; kp.h_sf_atoms = (uint8_t*)a.h_sf_atoms; kp.h_sf_ref = (uint8_t*)a.h_sf_ref; kp.h_feats = a.h_feats; kp.act = a.act;
    // token-major bf16 output of the one-accumulator tile into this GPU's own memory: 16-token x 32-feature boxes stored by TMA
    kp.c_tma = 0;
    tmC = tmA;
    if (BN == 256 && (a.out_mode == 1 || a.out_mode == 3) && !a.peer_n && a.C && ((uintptr_t)a.C & 15) == 0 && a.out_f % 8 == 0) {
        if ((rc = make_map_u8(&tmC, a.C, (uint64_t)a.out_f * 2, (uint64_t)a.tok, 64, 16, CU_TENSOR_MAP_SWIZZLE_64B))) return rc;
        kp.c_tma = 1;
    }
    int total = kp.num_m2 * kp.num_n;
    int nclusters = sm_count() / 2;
    if (total < nclusters) nclusters = total;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(nclusters * 2));
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // see griddep_wait() in the kernel
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, nvfp4_gemm_pair_kernel<SPARSE, BN>, tmA, tmB, tmSFA, tmSFB, tmMETA, tmC, kp);
}

int gemm_nvfp4(const GemmArgs& a, cudaStream_t st) {
    if (a.out_f <= 0 || a.tok < 0 || a.K <= 0 || a.a_rows <= 0) return QB_ERR_ARG;
    if (a.tok == 0) return QB_OK;
    if (a.out_f % 128 || a.K % 128 || a.a_rows % 128) return QB_ERR_ARG;
    if (!a.A || !a.B || !a.sfa || !a.sfb || (!a.C && !a.peer_n && a.out_mode != 4) || (a.sparse && !a.meta)) return QB_ERR_ARG;
    if (((uintptr_t)a.A & 15) || ((uintptr_t)a.B & 15) || ((uintptr_t)a.sfa & 15) || ((uintptr_t)a.sfb & 15) ||
        ((uintptr_t)a.meta & 15) || ((uintptr_t)a.C & 15))
        return QB_ERR_ARG;
    if (a.out_mode < 0 || a.out_mode > 4) return QB_ERR_ARG;
    int splits = a.splits < 1 ? 1 : a.splits;
    if (splits > 1 && (!a.Cf || a.eblk || a.out_mode > 1)) return QB_ERR_ARG;
    if (a.eblk && a.a_rows % a.out_f) return QB_ERR_ARG;
    int rc = gemm_init_attrs();
    if (rc) return rc;

    // CTA-pair kernel: plain bf16 GEMM, enough tokens to fill a 256-wide tile, out % 256 == 0.
    // bn == 512 requests it explicitly, bn == 0 (auto) picks it for prefill-sized problems.
    if (a.out_mode == 4) {
        // fused SwiGLU + quantiser epilogue: pair kernel only (plain or grouped), out = interleaved (gate, up) rows
        if (splits != 1 || a.peer_n || a.out_f % 256 || a.tok < 128 || !a.h_bytes || (!a.h_sf_atoms && !a.h_sf_ref) ||
            a.h_feats != a.out_f / 2 || ((uintptr_t)a.h_bytes & 7) || (a.act != 0 && a.act != 1) || (a.eblk && a.tok % 128) ||
            (((uintptr_t)a.bias & 15) != 0) || (a.bias_ld > 0 && a.bias_ld % 8))
            return QB_ERR_ARG;
        if (a.eblk || a.tok < 512) return a.sparse ? launch_pair<true, 128>(a, st) : launch_pair<false, 128>(a, st);
        return a.sparse ? launch_pair<true, 256>(a, st) : launch_pair<false, 256>(a, st);
    }
    if (a.peer_n) {
        // fused reduce-scatter: prefill pair kernel only, token-major output, token ranges of 16-token granularity
        if (a.peer_n < 2 || a.peer_n > 8 || a.peer_rank < 0 || a.peer_rank >= a.peer_n || a.out_mode != 1 || a.eblk || splits != 1 ||
            a.out_f % 256 || a.tok < 128 || a.tok_per_rank <= 0 || a.tok_per_rank % 16 || (long long)a.tok_per_rank * a.peer_n < a.tok ||
            !a.peer_done)
            return QB_ERR_ARG;
        for (int r = 0; r < a.peer_n; r++)
            if (!a.peer_out[r] || ((uintptr_t)a.peer_out[r] & 15) || !a.peer_flags[r]) return QB_ERR_ARG;
        if (a.bn == 384) return a.sparse ? launch_pair<true, 128>(a, st) : launch_pair<false, 128>(a, st);
        return a.sparse ? launch_pair<true, 256>(a, st) : launch_pair<false, 256>(a, st);
    }
    const bool pair_ok = !a.eblk && splits == 1 && (a.out_mode == 0 || a.out_mode == 1) && a.out_f % 256 == 0 && a.tok >= 128 &&
                         b_tail_ok(a.tok);
    if ((a.bn == 512 || a.bn == 384 || a.bn == 576) && !pair_ok) return QB_ERR_ARG;
    // 576: pair kernel with 192-token tiles and two accumulators, so the epilogue of a tile runs under the main
    // loop of the next one. Never chosen automatically: only 4 (sparse) / 2 (dense) scale-factor slots fit
    // beside two 192-column accumulators, the scale-factor copy then cannot run far enough ahead of the MMAs,
    // and the measured K-block time rises from ~500 to ~700 cycles (gate shape 102 us against 91 us).
    if (pair_ok && a.bn == 576)
        return a.sparse ? launch_pair<true, 192>(a, st) : launch_pair<false, 192>(a, st);
    if (pair_ok && (a.bn == 512 || (a.bn == 0 && a.tok >= 512)))   // 512: pair kernel, 256-token tile
        return a.sparse ? launch_pair<true, 256>(a, st) : launch_pair<false, 256>(a, st);
    if (pair_ok && a.bn == 384)                                     // 384: pair kernel, 128-token tile, two accumulators
        return a.sparse ? launch_pair<true, 128>(a, st) : launch_pair<false, 128>(a, st);
    // grouped (MoE) form on the pair kernel: one expert per 128-token block = per tile of the 128-token variant
    // grouped, every expert's rows padded to 256 (bn == 256): 256-token tiles; the pair MMA takes as long for 128 tokens
    // as for 256, so an expert with 129..256 rows costs one tile instead of two
    if (a.eblk && a.bn == 256) {
        if (splits != 1 || (a.out_mode != 1 && a.out_mode != 3) || a.out_f % 256 || a.tok < 256 || a.tok % 256 || (((uintptr_t)a.bias & 15) != 0) ||
            (a.bias_ld > 0 && a.bias_ld % 8))
            return QB_ERR_ARG;
        return a.sparse ? launch_pair<true, 256>(a, st) : launch_pair<false, 256>(a, st);
    }
    if (a.eblk && splits == 1 && (a.out_mode == 1 || a.out_mode == 3) && a.out_f % 256 == 0 && a.tok >= 128 && a.tok % 128 == 0 &&
        (a.bn == 0 || a.bn == 128) && (((uintptr_t)a.bias & 15) == 0) && (a.bias_ld <= 0 || a.bias_ld % 8 == 0))
        return a.sparse ? launch_pair<true, 128>(a, st) : launch_pair<false, 128>(a, st);
    int bn = a.bn;
    if (a.eblk) bn = 128;
    if (bn == 0) bn = a.tok <= 16 ? 16 : a.tok <= 32 ? 32 : a.tok <= 64 ? 64 : 128;
    if (bn != 16 && bn != 32 && bn != 64 && bn != 128 && bn != 256) return QB_ERR_ARG;   // 512 = pair kernel, handled above
    // a token tile starts at scale-atom column (n0 % 128) / 32 and the MMA only accepts even
    // scale-factor columns, so tiles narrower than 64 tokens must be the only tile
    if (bn < 64 && a.tok > bn) return QB_ERR_ARG;

    KParams kp;
    kp.sfa = (const uint8_t*)a.sfa; kp.sfb = (const uint8_t*)a.sfb; kp.meta = (const uint8_t*)a.meta;
    kp.gA = a.gA; kp.gB = a.gB; kp.C = a.C; kp.Cf = a.Cf; kp.sk_counters = (int*)a.sk_counters; kp.eblk = a.eblk; kp.bias = (const __nv_bfloat16*)a.bias; kp.row_w = a.row_w; kp.bias_ld = a.bias_ld > 0 ? a.bias_ld : a.out_f;
    kp.out_f = a.out_f; kp.tok = a.tok; kp.K = a.K;
    kp.num_m = a.out_f / 128;
    kp.num_n = (a.tok + bn - 1) / bn;
    kp.kblocks = (a.K + 255) / 256;
    if (splits > kp.kblocks) splits = kp.kblocks;
    // every split must own at least one K block
    while (splits > 1 && ((kp.kblocks + splits - 1) / splits) * (splits - 1) >= kp.kblocks) splits--;
    kp.splits = splits;
    kp.sfb_rowblocks = (a.tok + 127) / 128;
    kp.out_mode = a.out_mode;
    // split-K finished inside a cluster (no workspace, no atomics) whenever the split fits: one wave, at most 8 CTAs per
    // cluster, plain (not grouped) bf16 output, one accumulator-sized staging area in the operand ring; otherwise through the
    // caller's workspace
    kp.cluster_red = (splits > 1 && splits <= 8 && !a.eblk && (a.out_mode == 0 || a.out_mode == 1) &&
                      kp.num_m * kp.num_n * splits <= sm_count() && bn <= 128) ? 1 : 0;
    if (kp.cluster_red) {
        int mc = 0;
#define QB_MC(BN) (a.sparse ? max_clusters<true, BN>(splits) : max_clusters<false, BN>(splits))
        switch (bn) { case 16: mc = QB_MC(16); break; case 32: mc = QB_MC(32); break; case 64: mc = QB_MC(64); break; default: mc = QB_MC(128); break; }
#undef QB_MC
        if (kp.num_m * kp.num_n > mc) kp.cluster_red = 0;       // would take two waves of clusters: the workspace form is faster
    }
    if (!kp.cluster_red && splits > 1 && !a.sk_counters && !a.Cf) return QB_ERR_ARG;
    bool slab = false;
    // at most two attempts: a cluster launch that the device refuses (SMs taken by another context, a partitioned GPU) is
    // repeated in the workspace form when the caller gave a workspace
    for (int attempt = 0; attempt < 2; attempt++) {
        kp.sk_counters = (int*)a.sk_counters; kp.Cf = a.Cf;
        if (kp.cluster_red) { kp.sk_counters = nullptr; kp.Cf = nullptr; }
        slab = !kp.cluster_red && splits > 1 && a.sk_counters != nullptr;     // finish inside the kernel
        if (!slab) kp.sk_counters = nullptr;
        if (splits > 1 && !slab && !kp.cluster_red) {
            rc = (int)cudaMemsetAsync(a.Cf, 0, (size_t)a.out_f * a.tok * sizeof(float), st);
            if (rc) return rc;
        }
#define QB_GO(BN) (a.sparse ? launch<true, BN>(a, kp, st) : launch<false, BN>(a, kp, st))
        switch (bn) {
            case 16: rc = QB_GO(16); break;
            case 32: rc = QB_GO(32); break;
            case 64: rc = QB_GO(64); break;
            case 128: rc = QB_GO(128); break;
            default: rc = QB_GO(256); break;
        }
#undef QB_GO
        if (rc && kp.cluster_red && (a.sk_counters || a.Cf)) {
            cudaGetLastError();
            kp.cluster_red = 0;
            continue;
        }
        break;
    }
    if (rc) return rc;
    if (splits > 1 && !slab && !kp.cluster_red) {
        size_t n = (size_t)a.out_f * a.tok;
        int blocks = (int)((n + 255) / 256);
        if (blocks > sm_count() * 8) blocks = sm_count() * 8;
        splitk_finish_kernel<<<blocks, 256, 0, st>>>(a.Cf, a.gA, a.gB, (__nv_bfloat16*)a.C, a.out_f, a.tok, a.out_mode);
        rc = (int)cudaGetLastError();
    }
    return rc;
}

static int max_clusters_bn(int bn, int size) {
    switch (bn) {
        case 16: return max_clusters<false, 16>(size);
        case 32: return max_clusters<false, 32>(size);
        case 64: return max_clusters<false, 64>(size);
        default: return max_clusters<false, 128>(size);
    }
}

void decode_plan(int out_f, int tok, int K, int* splits, int* bn, int* cluster) {
    int b = tok <= 16 ? 16 : tok <= 32 ? 32 : tok <= 64 ? 64 : 128;
    const int num_n = (tok + b - 1) / b;
    const int tiles = (out_f / 128) * num_n;
    const int kb = (K + 255) / 256;
    const int sms = sm_count();
    int best_s = 1, best_c = 0;
    double best = 1e30;
    for (int s = 1; s <= kb && s <= 32; s++) {
        const int per = (kb + s - 1) / s;
        if (s > 1 && per * (s - 1) >= kb) continue;      // an empty split
        const int waves = (tiles * s + sms - 1) / sms;
        // in units of one K block of one CTA (~0.33 us measured): K blocks per unit + ~3 for pipeline fill and
        // epilogue; a split tile pays ~3.5 us + 0.12 us per token column for the reductions at the L2, the
        // fence, the arrival counter and the read-back by the last split (measured)
        const int ncol = tok < b ? tok : b;
        const double cost = waves * (per + 3.0 + (s > 1 ? 10.4 + 0.36 * ncol : 0.0));
        if (cost < best - 1e-9) { best = cost; best_s = s; best_c = 0; }
        // the same split finished inside a cluster of s CTAs (one wave, s <= 8): two cluster barriers and a pass over the
        // partial tiles in distributed shared memory
        if (cluster && s > 1 && s <= 8 && tiles * s <= sms && tiles <= max_clusters_bn(b, s)) {
            const double cc = per + 3.0 + 4.0 + 0.02 * ncol;
            if (cc < best - 1e-9) { best = cc; best_s = s; best_c = 1; }
        }
    }
    *splits = best_s;
    *bn = b;
    if (cluster) *cluster = best_c;
}


int read_status(cudaStream_t st) {
    int rc = (int)cudaStreamSynchronize(st);
    if (rc) return rc;
    int h = 0;
    rc = (int)cudaMemcpyFromSymbol(&h, g_status, sizeof(int));
    if (rc) return rc;
    if (h) {
        int zero = 0;
        cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    }
    return h;
}

}  // namespace qb
