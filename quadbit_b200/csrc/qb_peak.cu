// Issue-only throughput probe for the block-scaled FP4 tensor-core instruction
// (the sm_100a analogue of the reference's register-only peak probe cuda/mma_peak.cu):
// every SM loops over tcgen05.mma[.sp] kind::mxf4nvf4 with operands resident in shared
// memory and scale factors / metadata resident in shared or tensor memory, no global
// traffic. Gives the denominator "what the MMA pipe can do at this clock and power" for
// the GEMM's roofline, and separates the cost of the per-K-block tcgen05.cp copies.
#include <cuda.h>

#include "../../include/quadbit_b200.h"
#include "qb_common.cuh"
#include "qb_internal.h"

namespace qb {

// mode bit 0: issue the MMAs; bit 1: issue the scale-factor / metadata tcgen05.cp copies
template <bool SPARSE, int BN>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int kblocks, int mode, unsigned long long* cycles_out, int* status) {
    constexpr int A_ROW = SPARSE ? 64 : 128;
    constexpr int A_BYTES = 128 * A_ROW;
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
    __shared__ __align__(8) unsigned long long bar_mem;
    __shared__ __align__(8) unsigned long long bar2_mem;
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
    const uint32_t bar = smem_u32(&bar_mem);
    const uint32_t bar2 = smem_u32(&bar2_mem);
    if (threadIdx.x == 0) { abort_flag = 0; mbar_init(bar, 1); mbar_init(bar2, 1); fence_barrier_init(); }
    fence_proxy_async();
    if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    unsigned long long t0 = 0, t1 = 0;
    __shared__ volatile int done_flag;
    if (threadIdx.x == 0) done_flag = 0;
    __syncthreads();
    if (threadIdx.x >= 32 && (mode & 128)) {
        // experiment: other warps keep storing registers into unrelated TMEM columns
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = 0x38383838u;
        const uint32_t lane_sel = (uint32_t)((threadIdx.x >> 5) * 32) << 16;
        int n = 0;
        while (!done_flag && n < (1 << 24)) {
            tc_st_32x16(tmem_base + 400 + lane_sel, v);
            tc_st_32x8(tmem_base + 416 + lane_sel, *reinterpret_cast<uint32_t(*)[8]>(v));
            tc_wait_st();
            for (int d = 0; d < 8; d++) asm volatile("nanosleep.u32 20;");
            n++;
        }
    }
    if (threadIdx.x >= 32 && (mode & 96)) {
        // experiment: other warps poll an mbarrier that never completes while the MMA loop runs
        if ((mode & 32) || (threadIdx.x & 31) == 0) {
            while (!done_flag) { (void)mbar_try_wait(bar2, 0); }
        }
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
        t0 = clock64();
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
                    const uint64_t ad = make_smem_desc(st + i * 32, SPARSE ? 512 : 1024, 16, SPARSE ? 4 : 2);
                    const uint64_t bd = make_smem_desc(st + A_BYTES + i * B_KSTEP, 1024, 16, 2);
                    if (SPARSE) tc_mma_nvf4_sp(tmem_base, ad, bd, idesc, t_sfa + 4 * i, t_sfb + i * 4 * NB128, t_e + 2 * i, (kb | i) ? 1u : 0u);
                    else tc_mma_nvf4(tmem_base, ad, bd, idesc, t_sfa + 4 * i, t_sfb + i * 4 * NB128, (kb | i) ? 1u : 0u);
                }
            }
            if (mode & 4) tc_commit(bar2);   // one completion signal per K block, nobody waits on it
        }
        tc_commit(bar);
        mbar_wait_thread(bar, 1, &abort_flag, status, 10);
        t1 = clock64();
        if (cycles_out) cycles_out[blockIdx.x] = t1 - t0;
        done_flag = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <bool SPARSE, int BN>
static int run_peak(int kblocks, int mode, unsigned long long* cycles, int* status, cudaStream_t st) {
    constexpr int STAGE = 128 * (SPARSE ? 64 : 128) + BN * 128 + (SPARSE ? 2 : 4) * 512 * (1 + (BN + 127) / 128) + 2048;
    const int smem = 1024 + 2 * STAGE;
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
    constexpr int A_BYTES = 128 * A_ROW;
    constexpr int B_BYTES = (BN / 2) * 128;
    constexpr int MMAS = SPARSE ? 2 : 4;
    constexpr int B_KSTEP = SPARSE ? 64 : 32;
    constexpr int STAGE = A_BYTES + B_BYTES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) unsigned long long bar_mem;
    __shared__ __align__(8) unsigned long long bar2_mem;
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (smem0 - smem_u32(smem_raw));
    for (int i = threadIdx.x; i < 2 * STAGE / 4; i += blockDim.x) {
        uint32_t x = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        x ^= x >> 15; x *= 2246822519u; x ^= x >> 13;
        reinterpret_cast<uint32_t*>(gen)[i] = x;
    }
    const uint32_t bar = smem_u32(&bar_mem);
    const uint32_t rank = cluster_ctarank();
    const uint32_t bar2 = smem_u32(&bar2_mem);
    if (threadIdx.x == 0) { abort_flag = 0; mbar_init(bar, 1); mbar_init(bar2, 1); fence_barrier_init(); }
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
    if (threadIdx.x == 0 && rank == 0) {
        const uint32_t idesc = make_idesc_nvf4(BN, SPARSE, 256);
        const uint32_t t_sfa = tmem_base + 256, t_sfb = tmem_base + 272, t_e = tmem_base + 304;
        unsigned long long t0 = clock64();
        for (int kb = 0; kb < kblocks; kb++) {
            const uint32_t st = smem0 + (kb & 1) * STAGE;
#pragma unroll
            for (int i = 0; i < MMAS; i++) {
                const uint64_t ad = make_smem_desc(st + i * 32, SPARSE ? 512 : 1024, 16, SPARSE ? 4 : 2);
                const uint64_t bd = make_smem_desc(st + A_BYTES + i * B_KSTEP, 1024, 16, 2);
                if (SPARSE) tc_mma_nvf4_sp_pair(tmem_base, ad, bd, idesc, t_sfa + 4 * i, t_sfb + 8 * i, t_e + 2 * i, (kb | i) ? 1u : 0u);
                else tc_mma_nvf4_pair(tmem_base, ad, bd, idesc, t_sfa + 4 * i, t_sfb + 8 * i, (kb | i) ? 1u : 0u);
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
    constexpr int STAGE = 128 * (SPARSE ? 64 : 128) + (BN / 2) * 128;
    const int smem = 1024 + 2 * STAGE;
    int rc = (int)cudaFuncSetAttribute(mma_peak_pair_kernel<SPARSE, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (rc) return rc;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    mma_peak_pair_kernel<SPARSE, BN><<<(sms / 2) * 2, 128, smem, st>>>(kblocks, mode, cycles, status);
    return (int)cudaGetLastError();
}

}  // namespace qb

extern "C" int qb_mma_peak(int sparse, int bn, int kblocks, int mode, void* cycles_per_sm, void* status_word, void* stream) {
    if (kblocks <= 0 || kblocks > (1 << 22) || mode < 1 || mode > 255 || !status_word) return QB_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    auto* cyc = (unsigned long long*)cycles_per_sm;
    int* sw = (int*)status_word;
    if (mode & 16) {   // CTA-pair form (MMAs only)
        if (bn == 256) return sparse ? qb::run_peak_pair<true, 256>(kblocks, mode, cyc, sw, st) : qb::run_peak_pair<false, 256>(kblocks, mode, cyc, sw, st);
        if (bn == 128) return sparse ? qb::run_peak_pair<true, 128>(kblocks, mode, cyc, sw, st) : qb::run_peak_pair<false, 128>(kblocks, mode, cyc, sw, st);
        return QB_ERR_ARG;
    }
    if (bn == 256) return sparse ? qb::run_peak<true, 256>(kblocks, mode, cyc, sw, st) : qb::run_peak<false, 256>(kblocks, mode, cyc, sw, st);
    if (bn == 128) return sparse ? qb::run_peak<true, 128>(kblocks, mode, cyc, sw, st) : qb::run_peak<false, 128>(kblocks, mode, cyc, sw, st);
    return QB_ERR_ARG;
}
