// Issue-only throughput probe for the block-scaled FP4 tensor-core instruction
// (the sm_100a analogue of the reference's register-only peak probe cuda/mma_peak.cu):
// every SM loops over tcgen05.mma[.sp] kind::mxf4nvf4 with operands resident in shared
// memory and scale factors / metadata resident in shared or tensor memory, no global
// traffic unless the streaming variant asks for it. Gives the denominator "what the MMA pipe
// can do at this clock and power" for the GEMM's roofline, and varies one thing at a time:
// token tile width, one CTA or a CTA pair, the swizzle of the sparse A tile, the per-K-block
// tcgen05.cp copies, concurrent bulk copies into shared memory.
#include <cuda.h>

#include "../../include/quadbit_b200.h"
#include "qb_common.cuh"
#include "qb_internal.h"

namespace qb {

constexpr int PEAK_STREAM_SLOTS = 8;          // copies in flight
constexpr int PEAK_STREAM_BUFS = 4;           // destination buffers (two copies in flight may write the same one: the bytes are never read)
constexpr int PEAK_STREAM_BYTES = 24576;          // what one K block of the sparse pair kernel brings into a CTA
constexpr int PEAK_SRC_BYTES = 8 << 20;       // stays in L2; every SM walks it from its own offset
static __device__ __align__(128) uint8_t g_peak_src[PEAK_SRC_BYTES];

// mode bits, both forms: 0 issue the MMAs; 2 one commit per K block; 5 sparse A tile in 128-byte rows (two K blocks per
// row, 128-byte swizzle) instead of 64-byte rows with the 64-byte swizzle; 6 warp 1 streams 24 KB per K block from global
// memory into spare shared memory with bulk copies while the MMAs run (eight copies in flight).
// One-CTA form only: 1 the scale-factor / metadata tcgen05.cp copies of every K block; 3 a tcgen05 fence per K block.
// Pair form only (bit 4): 3 wait for every K block's completion before the next (serialised: completion latency).
struct PeakStream {
    uint32_t buf, bars;          // shared addresses: PEAK_STREAM_SLOTS buffers and barriers
};

__device__ __forceinline__ unsigned long long peak_stream(const PeakStream s, int kblocks, volatile int* abort_flag, int* status) {
    const unsigned long long t0 = clock64();
    constexpr int NCHUNK = PEAK_SRC_BYTES / PEAK_STREAM_BYTES;
    int n = 0;
    for (; n < kblocks && !*abort_flag; n++) {
        const int slot = n & (PEAK_STREAM_SLOTS - 1);
        const uint32_t bar = s.bars + slot * 8;
        if (n >= PEAK_STREAM_SLOTS && !mbar_wait_thread(bar, ((n / PEAK_STREAM_SLOTS) - 1) & 1, abort_flag, status, 13)) break;
        mbar_expect_tx(bar, PEAK_STREAM_BYTES);
        bulk_load(s.buf + (slot & (PEAK_STREAM_BUFS - 1)) * PEAK_STREAM_BYTES, g_peak_src + (size_t)((blockIdx.x * 7 + n) % NCHUNK) * PEAK_STREAM_BYTES, PEAK_STREAM_BYTES, bar);
    }
    // drain: every copy issued above must have landed before the CTA may leave
    for (int k = n > PEAK_STREAM_SLOTS ? n - PEAK_STREAM_SLOTS : 0; k < n; k++)
        if (!mbar_wait_thread(s.bars + (k & (PEAK_STREAM_SLOTS - 1)) * 8, (k / PEAK_STREAM_SLOTS) & 1, abort_flag, status, 14)) break;
    return clock64() - t0;
}

template <bool SPARSE, int BN>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int kblocks, int mode, unsigned long long* cycles_out, int* status) {
    constexpr int A_ROW = SPARSE ? 64 : 128;
    constexpr int A_BYTES = 128 * 128;               // room for the 128-byte-row variant of the sparse tile
    constexpr int B_BYTES = BN * 128;
    constexpr int MMAS = SPARSE ? 2 : 4;
    constexpr int B_KSTEP = SPARSE ? 64 : 32;
    constexpr int NB128 = (BN + 127) / 128;
    constexpr int SFA_BYTES = MMAS * 512, SFB_BYTES = NB128 * MMAS * 512, META_BYTES = 2048;
    constexpr int STAGE = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES + META_BYTES;
    constexpr int NST = 2;
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) unsigned long long bar_mem[2 + PEAK_STREAM_SLOTS];
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (smem0 - smem_u32(smem_raw));
    // pseudo-random operand bytes (E2M1 has no NaN; scale bytes kept in a finite UE4M3 range)
    for (int i = threadIdx.x; i < NST * STAGE / 4; i += blockDim.x) {
        uint32_t x = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
        int off = (i * 4) % STAGE;
        bool is_sf = off >= A_BYTES + B_BYTES && off < A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
        bool is_meta = off >= A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
        if (is_sf) x = (x & 0x0F0F0F0Fu) | 0x30303030u;
        if (is_meta) x = 0x4E4E4E4Eu;   // nibbles 0xE / 0x4: valid ascending pair indices
        reinterpret_cast<uint32_t*>(gen)[i] = x;
    }
    const uint32_t bar = smem_u32(&bar_mem[0]);
    const uint32_t bar2 = smem_u32(&bar_mem[1]);
    const PeakStream strm{smem0 + NST * STAGE, smem_u32(&bar_mem[2])};
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < 2 + PEAK_STREAM_SLOTS; i++) mbar_init(bar + 8 * i, 1);
        fence_barrier_init();
    }
    fence_proxy_async();
    if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    const bool wide_a = SPARSE && (mode & 32);
    if (threadIdx.x == 32 && (mode & 64)) {
        const unsigned long long c = peak_stream(strm, kblocks, &abort_flag, status);
        if (cycles_out) cycles_out[gridDim.x + blockIdx.x] = c;
    }
    if (threadIdx.x == 0) {
        const uint32_t idesc = make_idesc_nvf4(BN, SPARSE);
        const uint32_t t_sfa = tmem_base + 256, t_sfb = t_sfa + MMAS * 4, t_e = t_sfb + MMAS * 4 * NB128;
        // scale factors / metadata into TMEM once, so MMA-only runs read defined values
        for (int i = 0; i < MMAS; i++) tc_cp_32x128b_warpx4(t_sfa + 4 * i, make_smem_desc(smem0 + A_BYTES + B_BYTES + i * 512, 128, 0, 0));
        for (int nb = 0; nb < NB128; nb++)
            for (int i = 0; i < MMAS; i++)
                tc_cp_32x128b_warpx4(t_sfb + i * 4 * NB128 + 4 * nb, make_smem_desc(smem0 + A_BYTES + B_BYTES + SFA_BYTES + (nb * MMAS + i) * 512, 128, 0, 0));
        tc_cp_128x128b(t_e, make_smem_desc(smem0 + A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES, 128, 0, 0));
        tc_commit(bar);
        mbar_wait_thread(bar, 0, &abort_flag, status, 9);
        const unsigned long long t0 = clock64();
        for (int kb = 0; kb < kblocks; kb++) {
            const uint32_t st = smem0 + (kb & 1) * STAGE;
            if (mode & 8) tc_fence_after();
            if (mode & 2) {
#pragma unroll
                for (int i = 0; i < MMAS; i++) tc_cp_32x128b_warpx4(t_sfa + 4 * i, make_smem_desc(st + A_BYTES + B_BYTES + i * 512, 128, 0, 0));
#pragma unroll
                for (int nb = 0; nb < NB128; nb++)
#pragma unroll
                    for (int i = 0; i < MMAS; i++)
                        tc_cp_32x128b_warpx4(t_sfb + i * 4 * NB128 + 4 * nb, make_smem_desc(st + A_BYTES + B_BYTES + SFA_BYTES + (nb * MMAS + i) * 512, 128, 0, 0));
                if (SPARSE) tc_cp_128x128b(t_e, make_smem_desc(st + A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES, 128, 0, 0));
            }
            if (mode & 1) {
#pragma unroll
                for (int i = 0; i < MMAS; i++) {
                    const uint64_t ad = wide_a ? make_smem_desc(st + ((kb >> 1) & 1) * 64 + i * 32, 1024, 16, 2)
                                               : make_smem_desc(st + i * 32, A_ROW * 8, 16, SPARSE ? 4 : 2);
                    const uint64_t bd = make_smem_desc(st + A_BYTES + i * B_KSTEP, 1024, 16, 2);
                    if (SPARSE) tc_mma_nvf4_sp(tmem_base, ad, bd, idesc, t_sfa + 4 * i, t_sfb + i * 4 * NB128, t_e + 2 * i, (kb | i) ? 1u : 0u);
                    else tc_mma_nvf4(tmem_base, ad, bd, idesc, t_sfa + 4 * i, t_sfb + i * 4 * NB128, (kb | i) ? 1u : 0u);
                }
            }
            if (mode & 4) tc_commit(bar2);   // one completion signal per K block, nobody waits on it
        }
        tc_commit(bar);
        mbar_wait_thread(bar, 1, &abort_flag, status, 10);
        if (cycles_out) cycles_out[blockIdx.x] = clock64() - t0;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <bool SPARSE, int BN>
static int run_peak(int kblocks, int mode, unsigned long long* cycles, int* status, cudaStream_t st) {
    constexpr int STAGE = 128 * 128 + BN * 128 + (SPARSE ? 2 : 4) * 512 * (1 + (BN + 127) / 128) + 2048;
    const int smem = 1024 + 2 * STAGE + PEAK_STREAM_BUFS * PEAK_STREAM_BYTES;
    int rc = (int)cudaFuncSetAttribute(mma_peak_kernel<SPARSE, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (rc) return rc;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    mma_peak_kernel<SPARSE, BN><<<sms, 128, smem, st>>>(kblocks, mode, cycles, status);
    return (int)cudaGetLastError();
}

// CTA-pair form of the probe: tcgen05.mma.cta_group::2, M = 256, N = bn; each CTA holds its own
// 128 rows of A and half of the B rows; scale factors / metadata stay resident in TMEM.
template <bool SPARSE, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
mma_peak_pair_kernel(int kblocks, int mode, unsigned long long* cycles_out, int* status) {
    constexpr int A_ROW = SPARSE ? 64 : 128;
    constexpr int A_BYTES = 128 * 128;
    constexpr int B_BYTES = (BN / 2) * 128;
    constexpr int MMAS = SPARSE ? 2 : 4;
    constexpr int B_KSTEP = SPARSE ? 64 : 32;
    constexpr int STAGE = A_BYTES + B_BYTES;
    constexpr int NBA = (BN + 127) / 128;            // scale-factor atoms (128 tokens) per tile
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) unsigned long long bar_mem[2 + PEAK_STREAM_SLOTS];
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (smem0 - smem_u32(smem_raw));
    for (int i = threadIdx.x; i < 2 * STAGE / 4; i += blockDim.x) {
        uint32_t x = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
        reinterpret_cast<uint32_t*>(gen)[i] = x;
    }
    const uint32_t bar = smem_u32(&bar_mem[0]);
    const uint32_t rank = cluster_ctarank();
    const uint32_t bar2 = smem_u32(&bar_mem[1]);
    const PeakStream strm{smem0 + 2 * STAGE, smem_u32(&bar_mem[2])};
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < 2 + PEAK_STREAM_SLOTS; i++) mbar_init(bar + 8 * i, 1);
        fence_barrier_init();
    }
    fence_proxy_async();
    if (threadIdx.x < 32) { tmem_alloc_pair(smem_u32(&tmem_slot), 512); tmem_relinquish_pair(); }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    // finite scale factors and valid metadata in every lane of this CTA's TMEM
    {
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = 0x38383838u;
        const uint32_t lane_sel = (uint32_t)((threadIdx.x >> 5) * 32) << 16;
        tc_st_32x16(tmem_base + 256 + lane_sel, v);
        tc_st_32x16(tmem_base + 272 + lane_sel, v);
        tc_st_32x16(tmem_base + 288 + lane_sel, v);
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = 0x4E4E4E4Eu;
        tc_st_32x16(tmem_base + 304 + lane_sel, v);
        tc_wait_st();
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const bool wide_a = SPARSE && (mode & 32);
    if (threadIdx.x == 32 && (mode & 64)) {
        const unsigned long long c = peak_stream(strm, kblocks, &abort_flag, status);
        if (cycles_out) cycles_out[gridDim.x + blockIdx.x] = c;
    }
    if (threadIdx.x == 0 && rank == 0) {
        const uint32_t idesc = make_idesc_nvf4(BN, SPARSE, 256);
        const uint32_t t_sfa = tmem_base + 256, t_sfb = tmem_base + 272, t_e = tmem_base + 304;
        unsigned long long t0 = clock64();
        for (int kb = 0; kb < kblocks; kb++) {
            const uint32_t st = smem0 + (kb & 1) * STAGE;
#pragma unroll
            for (int i = 0; i < MMAS; i++) {
                const uint64_t ad = wide_a ? make_smem_desc(st + ((kb >> 1) & 1) * 64 + i * 32, 1024, 16, 2)
                                           : make_smem_desc(st + i * 32, A_ROW * 8, 16, SPARSE ? 4 : 2);
                const uint64_t bd = make_smem_desc(st + A_BYTES + i * B_KSTEP, 1024, 16, 2);
                if (SPARSE) tc_mma_nvf4_sp_pair(tmem_base, ad, bd, idesc, t_sfa + 4 * i, t_sfb + 4 * NBA * i, t_e + 2 * i, (kb | i) ? 1u : 0u);
                else tc_mma_nvf4_pair(tmem_base, ad, bd, idesc, t_sfa + 4 * i, t_sfb + 4 * NBA * i, (kb | i) ? 1u : 0u);
            }
            if (mode & 4) tc_commit_pair(bar2, 3);   // one multicast completion signal per K block
            if (mode & 8) { if (!mbar_wait_thread(bar2, kb & 1, &abort_flag, status, 12)) break; }   // serialised: completion latency
        }
        tc_commit_pair(bar, 1);
        mbar_wait_thread(bar, 0, &abort_flag, status, 11);
        if (cycles_out) cycles_out[blockIdx.x] = clock64() - t0;
    }
    tc_fence_before();
    cluster_sync_all();
    if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc_pair(tmem_base, 512); }
}

template <bool SPARSE, int BN>
static int run_peak_pair(int kblocks, int mode, unsigned long long* cycles, int* status, cudaStream_t st) {
    constexpr int STAGE = 128 * 128 + (BN / 2) * 128;
    const int smem = 1024 + 2 * STAGE + PEAK_STREAM_BUFS * PEAK_STREAM_BYTES;
    int rc = (int)cudaFuncSetAttribute(mma_peak_pair_kernel<SPARSE, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (rc) return rc;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    mma_peak_pair_kernel<SPARSE, BN><<<(sms / 2) * 2, 128, smem, st>>>(kblocks, mode, cycles, status);
    return (int)cudaGetLastError();
}

template <int BN>
static int run_peak_any(int sparse, int kblocks, int mode, unsigned long long* cyc, int* sw, cudaStream_t st) {
    if (mode & 16) return sparse ? run_peak_pair<true, BN>(kblocks, mode, cyc, sw, st) : run_peak_pair<false, BN>(kblocks, mode, cyc, sw, st);
    return sparse ? run_peak<true, BN>(kblocks, mode, cyc, sw, st) : run_peak<false, BN>(kblocks, mode, cyc, sw, st);
}

}  // namespace qb

extern "C" int qb_mma_peak(int sparse, int bn, int kblocks, int mode, void* cycles_per_sm, void* status_word, void* stream) {
    if (kblocks <= 0 || kblocks > (1 << 22) || mode < 1 || mode > 127 || !status_word) return QB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    auto* cyc = (unsigned long long*)cycles_per_sm;
    int* sw = (int*)status_word;
    if (bn == 256) return qb::run_peak_any<256>(sparse, kblocks, mode, cyc, sw, st);
    if (bn == 128) return qb::run_peak_any<128>(sparse, kblocks, mode, cyc, sw, st);
    if (bn == 64) return qb::run_peak_any<64>(sparse, kblocks, mode, cyc, sw, st);
    return QB_ERR_ARG;
}
