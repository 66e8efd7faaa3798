// Tensor parallelism over one NVSwitch box: peer-mapped buffers (CUDA IPC, one process per GPU), cross-GPU flag
// kernels, and the C-ABI of the two fused compute + collective operations:
//   qb_gemm_rs            row-parallel GEMM whose epilogue stores each partial row into the memory of the rank that owns
//                         the token (reduce-scatter by peer stores; the sum is taken by the consumer below);
//   qb_reduce_norm_quant  sum of the ranks' partials + residual add + RMSNorm + NVFP4 quantiser whose packed output is
//                         stored into every rank's gathered activation arrays (all-gather by peer stores).
// The reference has no counterpart: its one distributed script computes, then calls all_reduce
// (harness/moe_dist.py:123,161-167), and leaves tensor parallelism to the serving engine. Only plain loads / stores /
// system-scope flag accesses touch another GPU's memory here: no TMA and no multicast on peer memory.
#include <string.h>

#include "../../include/quadbit_b200.h"
#include "qb_common.cuh"
#include "qb_internal.h"

namespace {

__global__ void peer_signal_kernel(int* f0, int* f1, int* f2, int* f3, int* f4, int* f5, int* f6, int* f7, int n, int rank, int value,
                                   const int* value_ptr) {
    // stream order puts this after the kernels whose reads / writes it announces; one thread, one flag word per rank
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int* f[8] = {f0, f1, f2, f3, f4, f5, f6, f7};
        if (value_ptr) value = *value_ptr;
        __threadfence_system();
        for (int r = 0; r < n; r++) asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(f[r] + rank), "r"(value) : "memory");
    }
}

__global__ void peer_wait_kernel(const int* flags, int n, int value, const int* value_ptr, int* status) {
    if (value_ptr) value = *value_ptr;
    // bounded: a rank that never arrives costs 20 s and a status code, not a hang
    if ((int)threadIdx.x < n) {
        const uint64_t t0 = qb::globaltimer_ns();
        uint32_t it = 0;
        while (true) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
            if (v >= value) break;
            __nanosleep(200);
            if ((++it & 255u) == 0 && qb::globaltimer_ns() - t0 > 20000000000ull) {
                atomicCAS(status, 0, QB_ERR_TIMEOUT * 100 + 21);
                break;
            }
        }
    }
}

__device__ int g_peer_status = 0;

__global__ void epoch_add_kernel(int* epoch, int delta) {
    if (threadIdx.x == 0 && blockIdx.x == 0) *epoch += delta;
}

int* peer_status_ptr() {
    static int* cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cache[dev]) {
        int* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, g_peer_status) != cudaSuccess) return nullptr;
        cache[dev] = p;
    }
    return cache[dev];
}

}  // namespace

extern "C" {

int qb_peer_alloc(void** ptr, long long bytes) {
    if (!ptr || bytes <= 0) return QB_ERR_ARG;
    void* p = nullptr;
    int rc = (int)cudaMalloc(&p, (size_t)bytes);
    if (rc) return rc;
    rc = (int)cudaMemset(p, 0, (size_t)bytes);
    if (rc) { cudaFree(p); return rc; }
    *ptr = p;
    return QB_OK;
}

int qb_peer_free(void* ptr) { return ptr ? (int)cudaFree(ptr) : QB_OK; }

int qb_peer_export(void* ptr, void* handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!ptr || !handle64) return QB_ERR_ARG;
    return (int)cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle64, ptr);
}

int qb_peer_open(const void* handle64, void** ptr) {
    if (!ptr || !handle64) return QB_ERR_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}

int qb_peer_close(void* ptr) { return ptr ? (int)cudaIpcCloseMemHandle(ptr) : QB_OK; }

int qb_peer_signal(void* const* flag_arrays, int n, int my_rank, int value, const void* value_ptr, void* stream) {
    if (!flag_arrays || n < 1 || n > 8 || my_rank < 0 || my_rank >= n) return QB_ERR_ARG;
    int* f[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    for (int r = 0; r < n; r++) {
        if (!flag_arrays[r]) return QB_ERR_ARG;
        f[r] = (int*)flag_arrays[r];
    }
    peer_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7], n, my_rank, value, (const int*)value_ptr);
    return (int)cudaGetLastError();
}

int qb_peer_wait(const void* flags, int n, int value, const void* value_ptr, void* stream) {
    if (!flags || n < 1 || n > 8) return QB_ERR_ARG;
    int* st = peer_status_ptr();
    if (!st) return QB_ERR_DRIVER;
    peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const int*)flags, n, value, (const int*)value_ptr, st);
    return (int)cudaGetLastError();
}

int qb_epoch_add(void* epoch, int delta, void* stream) {
    if (!epoch) return QB_ERR_ARG;
    epoch_add_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((int*)epoch, delta);
    return (int)cudaGetLastError();
}

int qb_peer_status(void* stream) {
    int rc = (int)cudaStreamSynchronize((cudaStream_t)stream);
    if (rc) return rc;
    int h = 0;
    if (cudaMemcpyFromSymbol(&h, g_peer_status, sizeof(int)) != cudaSuccess) return QB_ERR_DRIVER;
    if (h) { int z = 0; cudaMemcpyToSymbol(g_peer_status, &z, sizeof(int)); }
    if (!h) h = qb::quant_status_read_clear();
    return h;
}

int qb_gemm_rs(const void* A, const void* B, const void* sfa, const void* sfb, const void* meta_native, const void* gA, const void* gB,
               void* const* peer_out, void* const* peer_flags, void* done_counter, int out, int tok, int K, int sparse, int n_ranks,
               int rank, int tok_per_rank, int flag_value, const void* value_ptr, int bn, void* stream) {
    if (!peer_out || !peer_flags || n_ranks < 2 || n_ranks > 8) return QB_ERR_ARG;
    if (sparse < 0 || sparse > 3) return QB_ERR_ARG;
    qb::GemmArgs g{};
    g.A = A; g.B = B; g.sfa = sfa; g.sfb = sfb; g.meta = meta_native; g.gA = (const float*)gA; g.gB = (const float*)gB;
    g.C = nullptr; g.a_rows = out; g.out_f = out; g.tok = tok; g.K = K; g.sparse = sparse & 1; g.a_tiled = (sparse >> 1) & 1;
    g.out_mode = 1; g.splits = 1; g.bn = bn;
    g.peer_n = n_ranks; g.peer_rank = rank; g.tok_per_rank = tok_per_rank; g.peer_val = flag_value; g.peer_done = (int*)done_counter; g.peer_val_ptr = (const int*)value_ptr;
    for (int r = 0; r < n_ranks; r++) { g.peer_out[r] = peer_out[r]; g.peer_flags[r] = (int*)peer_flags[r]; }
    return qb::gemm_nvfp4(g, (cudaStream_t)stream);
}

int qb_reduce_norm_quant(const void* src0, long long src_stride, int nsrc, const void* res, const void* wt, void* hout,
                         void* const* Bbytes_v, void* const* sf_atoms_v, void* const* g_v, int fan, int row0, int tok_total, int tok,
                         int H, float eps, int block, const void* wait_flags, int wait_val, void* const* sig_flags, int sig_n,
                         int sig_rank, int sig_val, void* done_counter, const void* value_ptr, void* stream) {
    if (!Bbytes_v || !sf_atoms_v || !g_v || fan < 0 || fan > 8 || sig_n < 0 || sig_n > 8 || (sig_n && !sig_flags)) return QB_ERR_ARG;
    qb::ReduceNormArgs a{};
    a.src0 = src0; a.src_stride = src_stride; a.nsrc = nsrc; a.res = res; a.wt = wt; a.hout = hout;
    for (int d = 0; d < (fan ? fan : 1); d++) { a.Bbytes[d] = Bbytes_v[d]; a.sf_atoms[d] = sf_atoms_v[d]; a.g[d] = g_v[d]; }
    a.fan = fan; a.row0 = row0; a.tok_total = tok_total; a.tok = tok; a.H = H; a.block = block; a.eps = eps;
    a.wait_flags = (const int*)wait_flags; a.wait_val = wait_val;
    a.sig_n = sig_n; a.sig_rank = sig_rank; a.sig_val = sig_val; a.done = (int*)done_counter; a.val_ptr = (const int*)value_ptr;
    for (int d = 0; d < sig_n; d++) a.sig_flags[d] = (int*)sig_flags[d];
    return qb::reduce_norm_quant(a, (cudaStream_t)stream);
}

}  // extern "C"
