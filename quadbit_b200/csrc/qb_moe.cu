// MoE routing helpers around the grouped GEMM: counting-sort route and top-k combine.
// Replace moe_route_scatter / moe_combine (cuda/sparse_fp4_lib.cu:1576-1620); same
// argument meaning. Both are HBM-bound index/copy kernels.
#include "qb_common.cuh"
#include "qb_internal.h"

namespace qb {

// src[poff[e] + slot] = i for every routed slot i with expert e = assign[i] >= 0; the order
// inside an expert segment is arbitrary. Padding entries of src keep the caller's -1.
__global__ void moe_route_kernel(const int* __restrict__ assign, const long long* __restrict__ poff, int* counter,
                                 int* __restrict__ src, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int e = assign[i];
    if (e < 0) return;
    int slot = atomicAdd(&counter[e], 1);
    src[poff[e] + slot] = i;
}

// y[t, f] = sum_k dbuf[inverse[t, k], f] over the rows with inverse >= 0; 8 bf16 per thread.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ dbuf, const int* __restrict__ inverse,
                                   __nv_bfloat16* __restrict__ y, int H, int topk, int Mpe) {
    extern __shared__ int rows[];
    const int token = blockIdx.x;
    if ((int)threadIdx.x < topk) rows[threadIdx.x] = inverse[(size_t)token * topk + threadIdx.x];
    __syncthreads();
    const bool vec = (H % 8 == 0) && (Mpe % 8 == 0);
    if (vec) {
        for (int f = threadIdx.x * 8; f < H; f += blockDim.x * 8) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            // four rows at a time, their loads issued together (a skipped row contributes zeros); same summation order
            for (int k0 = 0; k0 < topk; k0 += 4) {
                uint4 u[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int r = k0 + j < topk ? rows[k0 + j] : -1;
                    u[j] = r >= 0 ? __ldg(reinterpret_cast<const uint4*>(dbuf + (size_t)r * Mpe + f)) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u[j]);
#pragma unroll
                    for (int i = 0; i < 4; i++) { float2 v = __bfloat1622float2(h[i]); acc[2 * i] += v.x; acc[2 * i + 1] += v.y; }
                }
            }
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; i++) oh[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            *reinterpret_cast<uint4*>(y + (size_t)token * H + f) = o;
        }
    } else {
        for (int f = threadIdx.x; f < H; f += blockDim.x) {
            float acc = 0.f;
            for (int k = 0; k < topk; k++) {
                int r = rows[k];
                if (r >= 0) acc += __bfloat162float(dbuf[(size_t)r * Mpe + f]);
            }
            y[(size_t)token * H + f] = __float2bfloat16_rn(acc);
        }
    }
}

// Out[sc_tok[r], f] += (Cs[r, f] + bias[eblk[r / 128], f]) * sc_w[r] for every routed row r with sc_tok[r] >= 0 and every
// feature f < Hout: the bias / routing-weight / scatter-add tail of the reference's fused down GEMM (outT == 2 epilogue
// of matmul_sp_moe, cuda/sparse_fp4_lib.cu:1533-1546) applied to the token-major bf16 GEMM output Cs[rows][Mpe].
// One CTA per routed row, fp32 atomics into the caller-zeroed Out[tokens][Hout].
__global__ void moe_scatter_add_kernel(const __nv_bfloat16* __restrict__ Cs, const int* __restrict__ eblk, const int* __restrict__ sc_tok,
                                       const float* __restrict__ sc_w, const __nv_bfloat16* __restrict__ bias, float* __restrict__ Out,
                                       int Mpe, int Hout) {
    const int r = blockIdx.x;
    const int tok = sc_tok[r];
    if (tok < 0) return;
    const int e = eblk[r >> 7];
    const float w = sc_w ? sc_w[r] : 1.f;
    const __nv_bfloat16* src = Cs + (size_t)r * Mpe;
    const __nv_bfloat16* bb = bias ? bias + (size_t)e * Hout : nullptr;
    float* dst = Out + (size_t)tok * Hout;
    for (int f = threadIdx.x; f < Hout; f += blockDim.x)
        atomicAdd(dst + f, (__bfloat162float(src[f]) + (bb ? __bfloat162float(bb[f]) : 0.f)) * w);
}

int moe_scatter_add(const void* Cs, const void* eblk, const void* sc_tok, const void* sc_w, const void* bias, void* Out, int rows,
                    int Mpe, int Hout, cudaStream_t st) {
    if (rows < 0 || Mpe <= 0 || Hout <= 0 || Hout > Mpe) return QB_ERR_ARG;
    if (rows == 0) return QB_OK;
    if (!Cs || !eblk || !sc_tok || !Out) return QB_ERR_ARG;
    moe_scatter_add_kernel<<<rows, 256, 0, st>>>((const __nv_bfloat16*)Cs, (const int*)eblk, (const int*)sc_tok, (const float*)sc_w,
                                                 (const __nv_bfloat16*)bias, (float*)Out, Mpe, Hout);
    return (int)cudaGetLastError();
}

// Fixed-capacity routing in one launch of one cluster of eight CTAs: every CTA histograms its share of the slots in its
// own shared memory, the CTAs read each other's counts through distributed shared memory (per expert: the total and the
// number of slots that lower-ranked CTAs hold, which is where this CTA's rows start inside the expert's segment), every
// CTA forms the padded prefix, and then each routed slot takes the next free row of its CTA's part of the segment.
// Outputs: src[r_cap] (routed slot of every padded row, -1 = padding), pos[n] (padded row of every slot, -1 for a slot
// without a valid expert), eblk[r_cap/128] (expert of every 128-row block, -1 = unused capacity). Padding rows and unused
// capacity are filled by the CTAs in parallel with the scatter: they are disjoint from the rows the slots take, so nothing
// has to be ordered between CTAs. The order of the rows inside an expert's segment follows the atomics and may differ from
// run to run; rows are computed independently, so the layer's output does not.
// Replaces the sort-based torch routing (harness/qb_vllm_plugin/qb_sm120_plugin.py:1271-1315) for graph capture.
constexpr int ROUTE_CTAS = 8;
__device__ __forceinline__ int ld_cluster_s32(uint32_t cluster_addr) {
    int v;
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
    return v;
}
__global__ void __cluster_dims__(ROUTE_CTAS, 1, 1) __launch_bounds__(1024)
moe_route_fixed_kernel(const long long* __restrict__ assign, int n, int e, int r_cap, long long* __restrict__ src,
                       long long* __restrict__ pos, int* __restrict__ eblk, int div, const float* __restrict__ w_in,
                       float* __restrict__ rw, int* __restrict__ inverse, int e_base, int* __restrict__ n_used, int align) {
    // optional extras that the layer would otherwise do with a dozen small kernels: src holds slot / div (the token row
    // of a slot when div = top-k), rw[row] = w_in[slot] (0 for padding rows), inverse[slot] = row as int32
    extern __shared__ int sm[];
    int* counts = sm;            // this CTA's slots per expert
    int* poff = sm + e;          // first row of every expert's segment
    int* cursor = sm + 2 * e;    // next free row of this CTA's part of the segment
    int* tot = sm + 3 * e;       // slots per expert over all CTAs
    __shared__ int total;
    const int rank = (int)cluster_ctarank();
    const int i0 = (int)(((long long)n * rank) / ROUTE_CTAS), i1 = (int)(((long long)n * (rank + 1)) / ROUTE_CTAS);
    for (int i = threadIdx.x; i < e; i += blockDim.x) counts[i] = 0;
    __syncthreads();
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const long long ex = assign[i] - e_base;           // expert ids are global; this rank owns [e_base, e_base + e)
        if (ex >= 0 && ex < e) atomicAdd(&counts[(int)ex], 1);
    }
    cluster_sync_all();
    for (int x = threadIdx.x; x < e; x += blockDim.x) {
        int t = 0, before = 0;
        const uint32_t a = smem_u32(&counts[x]);
        for (int r = 0; r < ROUTE_CTAS; r++) {
            const int c = ld_cluster_s32(mapa_shared(a, (uint32_t)r));
            if (r < rank) before += c;
            t += c;
        }
        tot[x] = t;
        cursor[x] = before;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0;
        for (int x = 0; x < e; x++) { poff[x] = off; off += (tot[x] + align - 1) / align * align; }     // align = 128 or 256 rows
        total = off;
        if (n_used && rank == 0) *n_used = off;          // rows in use: kernels over the padded rows stop here instead of at r_cap
    }
    __syncthreads();
    // unused capacity behind the last segment, and its blocks
    const int tail = r_cap - total;
    for (int i = (int)(((long long)tail * rank) / ROUTE_CTAS) + threadIdx.x; i < (int)(((long long)tail * (rank + 1)) / ROUTE_CTAS); i += blockDim.x) {
        src[total + i] = -1;
        if (rw) rw[total + i] = 0.f;
    }
    if (rank == 0)
        for (int b = total / 128 + threadIdx.x; b < r_cap / 128; b += blockDim.x) eblk[b] = -1;
    // the experts of this CTA (x = rank, rank + 8, ...): blocks of the segment and its padding rows
    for (int x = rank; x < e; x += ROUTE_CTAS) {
        const int seg = (tot[x] + align - 1) / align * align;
        for (int b = threadIdx.x; b < seg / 128; b += blockDim.x) eblk[poff[x] / 128 + b] = x;
        for (int i = tot[x] + threadIdx.x; i < seg; i += blockDim.x) {
            src[poff[x] + i] = -1;
            if (rw) rw[poff[x] + i] = 0.f;
        }
    }
    for (int x = threadIdx.x; x < e; x += blockDim.x) cursor[x] += poff[x];
    __syncthreads();
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const long long ex = assign[i] - e_base;
        long long dst = -1;
        if (ex >= 0 && ex < e) {
            dst = atomicAdd(&cursor[(int)ex], 1);
            src[dst] = i / div;
            if (rw) rw[dst] = w_in[i];
        }
        pos[i] = dst;
        if (inverse) inverse[i] = (int)dst;
    }
    cluster_sync_all();          // no CTA leaves while its counts can still be read by the others
}

int moe_route_fixed(const void* assign, void* src, void* pos, void* eblk, int n, int e, int r_cap, cudaStream_t st, int div,
                    const void* w_in, void* rw, void* inverse, int e_base, void* n_used, int align) {
    if (align != 128 && align != 256) return QB_ERR_ARG;
    if (n < 0 || e <= 0 || e > 4096 || r_cap <= 0 || r_cap % align || (long long)r_cap < (long long)n + (long long)e * (align - 1)) return QB_ERR_ARG;
    if (!assign || !src || !pos || !eblk || div < 1 || ((rw != nullptr) != (w_in != nullptr))) return QB_ERR_ARG;
    const size_t smem = (size_t)4 * e * sizeof(int);
    if (smem > 48 * 1024) {
        const int rc = (int)cudaFuncSetAttribute(moe_route_fixed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (rc) return rc;
    }
    moe_route_fixed_kernel<<<ROUTE_CTAS, 1024, smem, st>>>((const long long*)assign, n, e, r_cap, (long long*)src,
                                                                         (long long*)pos, (int*)eblk, div, (const float*)w_in, (float*)rw, (int*)inverse, e_base, (int*)n_used, align);
    return (int)cudaGetLastError();
}

int moe_route(const void* assign, void* poff, void* counter, void* src, int n, int e, cudaStream_t st) {
    if (n < 0 || e <= 0 || !poff || !counter) return QB_ERR_ARG;
    int rc = (int)cudaMemsetAsync(counter, 0, (size_t)e * sizeof(int), st);
    if (rc || n == 0) return rc;
    if (!assign || !src) return QB_ERR_ARG;
    moe_route_kernel<<<(n + 255) / 256, 256, 0, st>>>((const int*)assign, (const long long*)poff, (int*)counter, (int*)src, n);
    return (int)cudaGetLastError();
}

int moe_combine_topk(const void* dbuf, const void* inverse, void* y, int t, int H, int topk, int Mpe, cudaStream_t st) {
    if (t < 0 || H <= 0 || topk <= 0 || topk > 256 || Mpe < H) return QB_ERR_ARG;
    if (t == 0) return QB_OK;
    if (!dbuf || !inverse || !y) return QB_ERR_ARG;
    if ((((uintptr_t)dbuf | (uintptr_t)y) & 15) != 0) return QB_ERR_ARG;
    int threads = ((H + 7) / 8 + 31) / 32 * 32;          // one 16-byte piece of the row per thread where the row allows it
    threads = threads < 64 ? 64 : threads > 512 ? 512 : threads;
    moe_combine_kernel<<<t, threads, (size_t)topk * sizeof(int), st>>>((const __nv_bfloat16*)dbuf, (const int*)inverse,
                                                                  (__nv_bfloat16*)y, H, topk, Mpe);
    return (int)cudaGetLastError();
}

}  // namespace qb
