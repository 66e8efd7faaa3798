// Expert parallelism over one NVSwitch box without a collective library: routing tables are replicated by peer stores,
// the owner of an expert PULLS the token rows it needs from the ranks that hold them (plain peer loads inside the fused
// gather + quantise kernel) and the home rank of a token PULLS the weighted expert outputs back inside the top-k combine.
// The reference's expert-parallel script computes every expert's partial [T,H] and calls all_reduce
// (harness/moe_dist.py:123,161-167); its plugin dispatches with torch indexing (harness/qb_vllm_plugin/qb_sm120_plugin.py:2430-2441).
// Only plain loads / stores and system-scope flag words touch peer memory.
#include "../../include/quadbit_b200.h"
#include "qb_common.cuh"
#include "qb_internal.h"

namespace {

struct PtrTable8 {
    void* p[8];
};

// Step 0 of a layer on every rank: copy this rank's token rows into its peer-visible buffer, and its routing (expert ids,
// routing weights of its tokens' slots) into the replicated tables of EVERY rank at this rank's slot range; the last CTA
// publishes the flag (fence + arrival counter, as in the GEMM epilogue).
__global__ void __launch_bounds__(256) ep_publish_kernel(const uint4* __restrict__ x, uint4* __restrict__ x_pub, size_t x_chunks,
                                                         const long long* __restrict__ idx, const float* __restrict__ w, int n_slots,
                                                         int slot0, PtrTable8 assign_all, PtrTable8 w_all, int world, int rank,
                                                         PtrTable8 flags, const int* value_ptr, int* done) {
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
    for (size_t i = tid; i < x_chunks; i += nth) x_pub[i] = __ldg(x + i);
    for (size_t i = tid; i < (size_t)n_slots; i += nth) {
        const long long e = idx[i];
        const float ww = w[i];
        for (int r = 0; r < world; r++) {
            reinterpret_cast<long long*>(assign_all.p[r])[slot0 + i] = e;
            reinterpret_cast<float*>(w_all.p[r])[slot0 + i] = ww;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(done, 1) == (int)gridDim.x - 1) {
            atomicExch(done, 0);
            __threadfence_system();
            const int val = *value_ptr;
            for (int r = 0; r < world; r++)
                asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(reinterpret_cast<int*>(flags.p[r]) + rank), "r"(val) : "memory");
        }
    }
}

// y[t, f] = sum_k d_owner[inverse_owner[slot(t, k)], f]: the top-k combine at the token's home rank, reading the weighted
// expert outputs (and the row index of each slot) from the rank that owns the slot's expert. 8 bf16 per thread.
__global__ void __launch_bounds__(256) ep_combine_kernel(PtrTable8 dbuf, PtrTable8 inverse, const long long* __restrict__ idx,
                                                         __nv_bfloat16* __restrict__ y, int t0, int H, int topk, int Mpe, int epr) {
    extern __shared__ long long rowptr[];         // per slot: address of the row (0 = none)
    const int token = blockIdx.x;
    if ((int)threadIdx.x < topk) {
        const long long e = idx[(size_t)token * topk + threadIdx.x];
        long long addr = 0;
        if (e >= 0) {
            const int owner = (int)(e / epr);
            const int* inv = reinterpret_cast<const int*>(inverse.p[owner]);
            int r;
            asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(r) : "l"(inv + ((size_t)(t0 + token) * topk + threadIdx.x)) : "memory");
            if (r >= 0) addr = (long long)(reinterpret_cast<const __nv_bfloat16*>(dbuf.p[owner]) + (size_t)r * Mpe);
        }
        rowptr[threadIdx.x] = addr;
    }
    __syncthreads();
    for (int f = threadIdx.x * 8; f < H; f += blockDim.x * 8) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k < topk; k++) {
            const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(rowptr[k]);
            if (!row) continue;
            uint4 u;
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(row + f) : "memory");
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
            for (int i = 0; i < 4; i++) { float2 v = __bfloat1622float2(h[i]); acc[2 * i] += v.x; acc[2 * i + 1] += v.y; }
        }
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; i++) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        *reinterpret_cast<uint4*>(y + (size_t)token * H + f) = o;
    }
}

}  // namespace

extern "C" {

int qb_ep_publish(const void* x, void* x_pub, long long x_bytes, const void* idx, const void* w, int n_slots, int slot0,
                  void* const* assign_all, void* const* w_all, int world, int rank, void* const* flags, const void* value_ptr,
                  void* done_counter, void* stream) {
    // x_bytes == 0: nothing to copy (the rank's rows were written into its peer-visible buffer by the kernel in front, e.g. the
    // quantiser of qb_quantize_rows); the flag still orders them, because that kernel has completed when this one starts
    if (x_bytes < 0 || (x_bytes & 15) || (x_bytes > 0 && (!x || !x_pub)) || !idx || !w || n_slots <= 0 || slot0 < 0 || !assign_all ||
        !w_all || !flags || world < 1 || world > 8 || rank < 0 || rank >= world || !value_ptr || !done_counter)
        return QB_ERR_ARG;
    if (x_bytes > 0 && (((uintptr_t)x & 15) || ((uintptr_t)x_pub & 15))) return QB_ERR_ARG;
    PtrTable8 a{}, ww{}, f{};
    for (int r = 0; r < world; r++) {
        if (!assign_all[r] || !w_all[r] || !flags[r]) return QB_ERR_ARG;
        a.p[r] = assign_all[r]; ww.p[r] = w_all[r]; f.p[r] = flags[r];
    }
    const size_t chunks = (size_t)x_bytes / 16;
    unsigned blocks = (unsigned)((chunks + 255) / 256);
    if (chunks == 0) blocks = (unsigned)((n_slots + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks == 0) blocks = 1;
    ep_publish_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)x, (uint4*)x_pub, chunks, (const long long*)idx, (const float*)w,
                                                               n_slots, slot0, a, ww, world, rank, f, (const int*)value_ptr, (int*)done_counter);
    return (int)cudaGetLastError();
}

int qb_ep_combine(void* const* dbuf, void* const* inverse, const void* idx, void* y, int t_local, int t0, int H, int topk, int Mpe,
                  int experts_per_rank, int world, void* stream) {
    if (!dbuf || !inverse || !idx || !y || t_local < 0 || t0 < 0 || H <= 0 || H % 8 || Mpe < H || Mpe % 8 || topk <= 0 || topk > 64 ||
        experts_per_rank <= 0 || world < 1 || world > 8)
        return QB_ERR_ARG;
    if (t_local == 0) return QB_OK;
    PtrTable8 d{}, inv{};
    for (int r = 0; r < world; r++) {
        if (!dbuf[r] || !inverse[r] || ((uintptr_t)dbuf[r] & 15)) return QB_ERR_ARG;
        d.p[r] = dbuf[r]; inv.p[r] = inverse[r];
    }
    ep_combine_kernel<<<t_local, 256, (size_t)topk * sizeof(long long), (cudaStream_t)stream>>>(d, inv, (const long long*)idx, (__nv_bfloat16*)y, t0, H,
                                                                                              topk, Mpe, experts_per_rank);
    return (int)cudaGetLastError();
}

}  // extern "C"
