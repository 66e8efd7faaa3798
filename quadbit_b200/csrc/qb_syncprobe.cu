// Round-trip latency probe for the barrier hops the CTA-pair GEMM pipeline is built from
// (no reference counterpart; a measuring aid like the issue-only MMA probe). One cluster of
// two CTAs plays ping-pong `iters` times and reports the leader's cycle count:
//   mode 0  two warps of one CTA: mbarrier.arrive (shared::cta) -> try_wait, and back
//   mode 1  the two CTAs: mbarrier.arrive.shared::cluster -> try_wait in the peer, and back
//   mode 2  leader: tcgen05.commit.cta_group::2 with multicast to both CTAs' barriers;
//           peer: try_wait, then mbarrier.arrive.shared::cluster back to the leader
//   mode 3  as mode 0 with the warp-wide wait
//   mode 4  one thread: arrive on its own barrier, then a try_wait that succeeds at once
//   mode 5  one thread: two barriers, both arrives, then both try_waits issued back to back
//   mode 6+n  mode 0 while n further warps (n <= 14) of each CTA poll a barrier that stays incomplete
// Every wait is bounded; on expiry the status word gets QB_ERR_TIMEOUT * 100 + 50 + mode.
#include <cuda.h>

#include "../../include/quadbit_b200.h"
#include "qb_common.cuh"
#include "qb_internal.h"

namespace qb {

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(512, 1)
sync_probe_kernel(int mode, int iters, unsigned long long* out, int* status) {
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) unsigned long long bar_mem[3];
    __shared__ volatile int stop_flag;
    const uint32_t barA = smem_u32(&bar_mem[0]), barB = smem_u32(&bar_mem[1]);
    const uint32_t rank = cluster_ctarank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(barA, 1);
        mbar_init(barB, 1);
        mbar_init(smem_u32(&bar_mem[2]), 1);
        stop_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0) { tmem_alloc_pair(smem_u32(&tmem_slot), 32); tmem_relinquish_pair(); }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint64_t limit = 200000000ull;   // 0.2 s per wait
    const int site = 50 + mode;
    if (warp >= 2) {
        // background pollers (modes 6+): warps 2.. poll a barrier that nobody completes until warp 0 raises
        // the stop flag; at most 2^22 polls each
        const uint32_t barC = smem_u32(&bar_mem[2]);
        for (int i = 0; i < (1 << 22) && !stop_flag; i++)
            if (mbar_try_wait(barC, 0)) break;
    }
    long long t0 = clock64();
    if (mode >= 6) mode = 0;
    if (mode == 0 || mode == 3) {
        if (rank == 0) {
            if (warp == 0) {
                for (int i = 0; i < iters && !abort_flag; i++) {
                    if (lane == 0) mbar_arrive(barA);
                    if (mode == 0) { if (lane == 0 && !mbar_wait_thread(barB, i & 1, &abort_flag, status, site, limit)) break; }
                    else if (!mbar_wait(barB, i & 1, &abort_flag, status, site, 0, limit)) break;
                }
            } else if (warp == 1) {
                for (int i = 0; i < iters && !abort_flag; i++) {
                    if (mode == 0) { if (lane == 0 && !mbar_wait_thread(barA, i & 1, &abort_flag, status, site, limit)) break; }
                    else if (!mbar_wait(barA, i & 1, &abort_flag, status, site, 0, limit)) break;
                    if (lane == 0) mbar_arrive(barB);
                }
            }
        }
    } else if (mode == 4 || mode == 5) {
        if (rank == 0 && threadIdx.x == 0) {
            for (int i = 0; i < iters; i++) {
                mbar_arrive(barA);
                if (mode == 5) mbar_arrive(barB);
                bool a = mbar_try_wait(barA, i & 1);
                bool b = mode == 5 ? mbar_try_wait(barB, i & 1) : true;
                if (!(a && b)) { atomicCAS(status, 0, QB_ERR_TIMEOUT * 100 + site); break; }
            }
        }
    } else if (warp == 0 && lane == 0) {
        if (rank == 0) {
            const uint32_t peerA = mapa_shared(barA, 1);
            for (int i = 0; i < iters && !abort_flag; i++) {
                if (mode == 1) mbar_arrive_cluster(peerA);
                else tc_commit_pair(barA, 3);
                if (!mbar_wait_thread(barB, i & 1, &abort_flag, status, site, limit)) break;
            }
        } else {
            const uint32_t leaderB = mapa_shared(barB, 0);
            for (int i = 0; i < iters && !abort_flag; i++) {
                if (!mbar_wait_thread(barA, i & 1, &abort_flag, status, site, limit)) break;
                mbar_arrive_cluster(leaderB);
            }
        }
    }
    long long t1 = clock64();
    if (warp == 0) stop_flag = 1;
    if (rank == 0 && threadIdx.x == 0) { out[0] = (unsigned long long)(t1 - t0); out[1] = (unsigned long long)iters; }
    __syncwarp();
    tc_fence_before();
    cluster_sync_all();
    if (warp == 0) { tc_fence_after(); tmem_dealloc_pair(tmem_slot, 32); }
}

}  // namespace qb

extern "C" int qb_sync_probe(int mode, int iters, void* cycles_out, void* status_word, void* stream) {
    if (mode < 0 || mode > 6 + 14 || iters <= 0 || iters > (1 << 20) || !cycles_out || !status_word) return QB_ERR_ARG;
    const int extra = mode >= 6 ? mode - 6 : 0;      // mode 6 + n: mode 0 with n background polling warps
    qb::sync_probe_kernel<<<2, 64 + 32 * extra, 0, (cudaStream_t)stream>>>(mode, iters, (unsigned long long*)cycles_out, (int*)status_word);
    return (int)cudaGetLastError();
}
