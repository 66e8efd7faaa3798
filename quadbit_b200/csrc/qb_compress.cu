// Offline weight packers, on the GPU:
//   compress_2to4  pair-granular 2:4 pruning + two-level NVFP4 quantisation + 2-bit metadata
//   pack_dense     two-level NVFP4 quantisation of a dense weight
//
// The reference does this with a dozen eager torch ops (QuadbitLinear.__init__,
// harness/quadbit_linear.py:89-119; two-level: harness/verify_sparse_2lvl.py:108-122,
// harness/fused_moe.py:372-387; dense: harness/dense_e2e.py:79-88) and has no kernel for
// it, so the only requirement is bit-exact codes / metadata / scales / globals. Every
// output can be emitted in the reference's step-major layout (for byte-for-byte
// comparison with the torch packer) and in the layout the tcgen05 GEMM consumes
// (scale-factor atoms, row-major metadata per 128-row x 256-K block); the packed values
// Ac / Ab are the same in both.
//
// Rules fixed here where the reference leaves them open: importance |w0|+|w1| in fp32;
// on equal importance the lower pair index is kept; all divisions are IEEE; the divisor
// of an all-zero block is clamped to 1e-30 (codes 0).
//
// HBM-bound, one CTA per weight row: 2*K (bf16) or 4*K bytes read, 0.344*K written.
#include "qb_common.cuh"
#include "qb_internal.h"

namespace qb {

__device__ __forceinline__ float ld_elem(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ld_elem(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

template <typename T>
__device__ __forceinline__ void load32(const T* p, float (&w)[32]);
template <>
__device__ __forceinline__ void load32<float>(const float* p, float (&w)[32]) {
    const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float4 f = __ldg(q + i);
        w[4 * i] = f.x; w[4 * i + 1] = f.y; w[4 * i + 2] = f.z; w[4 * i + 3] = f.w;
    }
}
template <>
__device__ __forceinline__ void load32<__nv_bfloat16>(const __nv_bfloat16* p, float (&w)[32]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint4 u = __ldg(q + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            float2 f = __bfloat1622float2(h[k]);
            w[8 * i + 2 * k] = f.x; w[8 * i + 2 * k + 1] = f.y;
        }
    }
}

__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = ((threadIdx.x & 31) < (blockDim.x >> 5)) ? red[threadIdx.x & 31] : 0.f;
    return warp_max(r);
}

template <typename T, int NB>
__global__ void __launch_bounds__(1024) compress_2to4_kernel(const T* __restrict__ W, uint8_t* __restrict__ Ac,
                                                              uint32_t* __restrict__ meta_ref, uint32_t* __restrict__ meta_nat,
                                                              uint8_t* __restrict__ sf_ref, uint8_t* __restrict__ sf_atoms,
                                                              float* __restrict__ gA, int out_f, int K,
                                                              const float* __restrict__ colnorm) {
    // colnorm != nullptr: importance of a pair = |w0|*c0 + |w1|*c1 with c the activation column norms
    // (Wanda; harness/qb_vllm_plugin/qb_sm120_plugin.py:1183-1190), each product and the sum rounded to fp32
    __shared__ float red[32];
    const int row = blockIdx.x;
    const int nblk = K >> 5;   // 32 logical K = 4 groups of 4 pairs = 16 kept values = one scale
    const int ks = K >> 7;
    const int lane = threadIdx.x & 31;
    const T* wr = W + (size_t)row * K;

    float kept[NB][16];
    uint32_t nibs[NB];
    float bmax[NB];
    float tmax = 0.f;
#pragma unroll
    for (int j = 0; j < NB; j++) {
        int b = threadIdx.x + j * blockDim.x;
        float w[32];
#pragma unroll
        for (int i = 0; i < 32; i++) w[i] = 0.f;
        if (b < nblk) load32<T>(wr + (size_t)b * 32, w);
        uint32_t nb = 0;
        float m = 0.f;
#pragma unroll
        for (int g = 0; g < 4; g++) {
            float imp[4];
#pragma unroll
            for (int p = 0; p < 4; p++) {
                float a0 = fabsf(w[g * 8 + 2 * p]), a1 = fabsf(w[g * 8 + 2 * p + 1]);
                if (colnorm && b < nblk) {
                    const float2 c = __ldg(reinterpret_cast<const float2*>(colnorm + (size_t)b * 32 + g * 8 + 2 * p));
                    a0 = __fmul_rn(a0, c.x);
                    a1 = __fmul_rn(a1, c.y);
                }
                imp[p] = __fadd_rn(a0, a1);
            }
            // largest importance, lowest index on ties; then the same among the rest
            int a = 0;
#pragma unroll
            for (int p = 1; p < 4; p++) if (imp[p] > imp[a]) a = p;
            int s = (a == 0) ? 1 : 0;
#pragma unroll
            for (int p = 0; p < 4; p++) if (p != a && p != s && imp[p] > imp[s]) s = p;
            int i0 = min(a, s), i1 = max(a, s);
            nb |= (uint32_t)(i0 | (i1 << 2)) << (4 * g);
#pragma unroll
            for (int p = 0; p < 4; p++) {
                if (p == i0) { kept[j][g * 4 + 0] = w[g * 8 + 2 * p]; kept[j][g * 4 + 1] = w[g * 8 + 2 * p + 1]; }
                if (p == i1) { kept[j][g * 4 + 2] = w[g * 8 + 2 * p]; kept[j][g * 4 + 3] = w[g * 8 + 2 * p + 1]; }
            }
        }
#pragma unroll
        for (int i = 0; i < 16; i++) m = fmaxf(m, fabsf(kept[j][i]));
        nibs[j] = nb;
        bmax[j] = m;
        tmax = fmaxf(tmax, m);
    }
    float g_row = fmaxf(__fdiv_rn(block_max(tmax, red), 2688.f), 1e-30f);
    if (threadIdx.x == 0 && gA) gA[row] = g_row;

#pragma unroll
    for (int j = 0; j < NB; j++) {
        int b = threadIdx.x + j * blockDim.x;
        uint32_t code = enc_ue4m3(__fdiv_rn(__fdiv_rn(bmax[j], 6.f), g_row));
        float sg = fmaxf(__fmul_rn(dec_ue4m3(code), g_row), 1e-30f);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            lo |= (q_fp4_div(kept[j][2 * i], sg) | (q_fp4_div(kept[j][2 * i + 1], sg) << 4)) << (8 * i);
            hi |= (q_fp4_div(kept[j][8 + 2 * i], sg) | (q_fp4_div(kept[j][8 + 2 * i + 1], sg) << 4)) << (8 * i);
        }
        // metadata word = 8 groups = this block's 16 bits + the neighbouring block's
        uint32_t other = __shfl_xor_sync(0xffffffffu, nibs[j], 1);
        uint32_t mword = (b & 1) ? (other | (nibs[j] << 16)) : (nibs[j] | (other << 16));
        // scale word = 4 consecutive blocks
        uint32_t sw = 0;
        int base = lane & ~3;
#pragma unroll
        for (int i = 0; i < 4; i++) sw |= __shfl_sync(0xffffffffu, code, base + i) << (8 * i);
        if (b < nblk) {
            int s = b >> 2;
            if (Ac) *reinterpret_cast<uint2*>(Ac + (size_t)row * (K >> 2) + (size_t)b * 8) = make_uint2(lo, hi);
            if ((b & 1) == 0) {
                int h = (b & 3) >> 1;
                if (meta_ref) meta_ref[((size_t)s * out_f + row) * 2 + h] = mword;
                if (meta_nat)
                    meta_nat[((((size_t)(row >> 7) * (kpad256(K) >> 8) + (s >> 1)) * 128 + (row & 127)) << 2) + (s & 1) * 2 + h] = mword;
            }
            if ((b & 3) == 0) {
                if (sf_ref) *reinterpret_cast<uint32_t*>(sf_ref + ((size_t)s * out_f + row) * 4) = sw;
                if (sf_atoms) *reinterpret_cast<uint32_t*>(sf_atoms + sf_atom_offset(row, b, kpad256(K) >> 7)) = sw;
            }
        }
    }
}

template <typename T, int NB>
__global__ void __launch_bounds__(1024) pack_dense_kernel(const T* __restrict__ W, uint8_t* __restrict__ Ab,
                                                           uint8_t* __restrict__ sf_ref, uint8_t* __restrict__ sf_atoms,
                                                           float* __restrict__ gA, int out_f, int K) {
    __shared__ float red[32];
    const int row = blockIdx.x;
    const int nblk = K >> 5;   // 32 elements per thread-block = two per-16 scale blocks
    const T* wr = W + (size_t)row * K;
    float w[NB][32];
    float tmax = 0.f;
#pragma unroll
    for (int j = 0; j < NB; j++) {
        int b = threadIdx.x + j * blockDim.x;
#pragma unroll
        for (int i = 0; i < 32; i++) w[j][i] = 0.f;
        if (b < nblk) load32<T>(wr + (size_t)b * 32, w[j]);
#pragma unroll
        for (int i = 0; i < 32; i++) tmax = fmaxf(tmax, fabsf(w[j][i]));
    }
    float g_row = fmaxf(__fdiv_rn(block_max(tmax, red), 2688.f), 1e-30f);
    if (threadIdx.x == 0 && gA) gA[row] = g_row;
#pragma unroll
    for (int j = 0; j < NB; j++) {
        int b = threadIdx.x + j * blockDim.x;
        uint32_t words[4];
        uint32_t codes2 = 0;
#pragma unroll
        for (int hb = 0; hb < 2; hb++) {
            float m = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i++) m = fmaxf(m, fabsf(w[j][hb * 16 + i]));
            uint32_t code = enc_ue4m3(__fdiv_rn(__fdiv_rn(m, 6.f), g_row));
            float sg = fmaxf(__fmul_rn(dec_ue4m3(code), g_row), 1e-30f);
            codes2 |= code << (8 * hb);
#pragma unroll
            for (int q = 0; q < 2; q++) {
                uint32_t wd = 0;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    int e = hb * 16 + q * 8 + 2 * i;
                    wd |= (q_fp4_div(w[j][e], sg) | (q_fp4_div(w[j][e + 1], sg) << 4)) << (8 * i);
                }
                words[hb * 2 + q] = wd;
            }
        }
        uint32_t other = __shfl_xor_sync(0xffffffffu, codes2, 1);
        uint32_t sw = (b & 1) ? (other | (codes2 << 16)) : (codes2 | (other << 16));
        if (b < nblk) {
            if (Ab) *reinterpret_cast<uint4*>(Ab + (size_t)row * (K >> 1) + (size_t)b * 16) = make_uint4(words[0], words[1], words[2], words[3]);
            if ((b & 1) == 0) {
                int s = b >> 2, q = (b & 3) >> 1;
                if (sf_ref) *reinterpret_cast<uint32_t*>(sf_ref + ((size_t)s * out_f + row) * 8 + q * 4) = sw;
                if (sf_atoms) *reinterpret_cast<uint32_t*>(sf_atoms + sf_atom_offset(row, 2 * b, kpad256(K) >> 6)) = sw;
            }
        }
    }
}

static bool pick_launch(int K, int& threads, int& nb) {
    int nblk = K / 32;
    threads = nblk <= 512 ? 256 : (nblk <= 1024 ? 512 : 1024);
    if (nblk < threads) threads = (nblk + 31) / 32 * 32;
    nb = (nblk + threads - 1) / threads;
    return nb <= 2;
}

int compress_2to4(const void* W, int w_dtype, void* Ac, void* meta_ref, void* meta_nat, void* sf_ref, void* sf_atoms,
                  void* gA, int out_f, int K, cudaStream_t st, const void* colnorm) {
    if (out_f <= 0 || K <= 0 || K % 128 != 0 || !W || (w_dtype != 0 && w_dtype != 1)) return QB_ERR_ARG;
    if (((uintptr_t)W & 15) || ((uintptr_t)Ac & 7) || ((uintptr_t)colnorm & 7) || ((uintptr_t)meta_ref & 3) || ((uintptr_t)meta_nat & 3) ||
        ((uintptr_t)sf_ref & 3) || ((uintptr_t)sf_atoms & 3))
        return QB_ERR_ARG;
    int threads, nb;
    if (!pick_launch(K, threads, nb)) return QB_ERR_UNSUPPORTED;
#define QB_LC(T, NB)                                                                                            \
    compress_2to4_kernel<T, NB><<<out_f, threads, 0, st>>>((const T*)W, (uint8_t*)Ac, (uint32_t*)meta_ref,      \
                                                           (uint32_t*)meta_nat, (uint8_t*)sf_ref, (uint8_t*)sf_atoms, \
                                                           (float*)gA, out_f, K, (const float*)colnorm)
    if (w_dtype == 0) { if (nb <= 1) QB_LC(float, 1); else QB_LC(float, 2); }
    else { if (nb <= 1) QB_LC(__nv_bfloat16, 1); else QB_LC(__nv_bfloat16, 2); }
#undef QB_LC
    return (int)cudaGetLastError();
}

int pack_dense(const void* W, int w_dtype, void* Ab, void* sf_ref, void* sf_atoms, void* gA, int out_f, int K,
               cudaStream_t st) {
    if (out_f <= 0 || K <= 0 || K % 128 != 0 || !W || (w_dtype != 0 && w_dtype != 1)) return QB_ERR_ARG;
    if (((uintptr_t)W & 15) || ((uintptr_t)Ab & 15) || ((uintptr_t)sf_ref & 3) || ((uintptr_t)sf_atoms & 3)) return QB_ERR_ARG;
    int threads, nb;
    if (!pick_launch(K, threads, nb)) return QB_ERR_UNSUPPORTED;
#define QB_LD(T, NB)                                                                                         \
    pack_dense_kernel<T, NB><<<out_f, threads, 0, st>>>((const T*)W, (uint8_t*)Ab, (uint8_t*)sf_ref, (uint8_t*)sf_atoms, \
                                                        (float*)gA, out_f, K)
    if (w_dtype == 0) { if (nb <= 1) QB_LD(float, 1); else QB_LD(float, 2); }
    else { if (nb <= 1) QB_LD(__nv_bfloat16, 1); else QB_LD(__nv_bfloat16, 2); }
#undef QB_LD
    return (int)cudaGetLastError();
}

// 16 bytes per thread: dst chunk index -> (tile, row, chunk) -> source row / byte offset
__global__ void tile_weights_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int rows, int row_bytes, int kblocks,
                                    int a_row) {
    const int cpr = a_row / 16;                                   // 16-byte chunks per tile row
    const size_t n = (size_t)rows * kblocks * cpr;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % cpr);
        const size_t t = i / cpr;
        const int r = (int)(t % 128);
        const size_t tile = t / 128;
        const int kb = (int)(tile % kblocks);
        const int rb = (int)(tile / kblocks);
        const int byte = kb * a_row + c * 16;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (byte < row_bytes) v = src[((size_t)(rb * 128 + r) * row_bytes + byte) / 16];
        dst[i] = v;
    }
}

int tile_weights(const void* A, void* At, int rows, int K, int sparse, cudaStream_t st) {
    if (rows <= 0 || K <= 0 || rows % 128 || K % 128) return QB_ERR_ARG;
    if (!A || !At || ((uintptr_t)A & 15) || ((uintptr_t)At & 15)) return QB_ERR_ARG;
    const int row_bytes = sparse ? K / 4 : K / 2;                 // multiple of 32 for K % 128 == 0
    const int a_row = sparse ? 64 : 128;
    const int kblocks = kpad256(K) / 256;
    const size_t n = (size_t)rows * kblocks * (a_row / 16);
    int blocks = (int)((n + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    tile_weights_kernel<<<blocks, 256, 0, st>>>((const uint4*)A, (uint4*)At, rows, row_bytes, kblocks, a_row);
    return (int)cudaGetLastError();
}

// Checkpoint block formats -> bf16 rows for the compressor (the reference dequantises with torch:
// _mxfp4_dequant, harness/qb_vllm_plugin/qb_sm120_plugin.py:2089-2100, gpt-oss MXFP4: E2M1 codes, one e8m0
// scale 2^(raw-127) per 32; _dequant_nvfp4_expert, :70-95, modelopt NVFP4: one e4m3fn scale per 16 and a
// per-tensor fp32 scale, product (value * block scale) * tensor scale in fp32, then bf16).
// One thread per 8 values (4 code bytes in, 16 bytes out); rows of the output have a stride so that the
// result can land inside a zero-padded [out%256][in%128] buffer. HBM-bound: 0.5 + scale bytes in, 2 out.
__device__ __forceinline__ float dec_e4m3fn(uint32_t c) {
    const uint32_t e = (c >> 3) & 0xF, m = c & 7;
    float v = e == 0 ? (float)m * 0.001953125f : __uint_as_float(((e + 120u) << 23) | (m << 20));
    if ((c & 0x7f) == 0x7f) v = __int_as_float(0x7fc00000);
    return (c & 0x80) ? -v : v;
}
template <int GROUP>
__global__ void dequant_fp4_blocks_kernel(const uint32_t* __restrict__ w, const uint8_t* __restrict__ sc, const float* __restrict__ s2,
                                          __nv_bfloat16* __restrict__ out, int out_f, int in_f, long long ld_out) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int per_row = in_f >> 3;
    if (t >= (long long)out_f * per_row) return;
    const int r = (int)(t / per_row), c8 = (int)(t % per_row);
    const uint32_t codes = __ldg(w + t);
    const uint32_t sraw = __ldg(sc + (size_t)r * (in_f / GROUP) + (c8 * 8) / GROUP);
    const float bs = GROUP == 32 ? exp2f((float)sraw - 127.f) : dec_e4m3fn(sraw);
    const float ts = s2 ? __ldg(s2) : 1.f;
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t c0 = (codes >> (8 * i)) & 0xF, c1 = (codes >> (8 * i + 4)) & 0xF;
        float v0 = (float)((c0 & 7) < 4 ? (c0 & 7) : ((c0 & 7) == 4 ? 4 : ((c0 & 7) == 5 ? 6 : ((c0 & 7) == 6 ? 8 : 12)))) * 0.5f;
        float v1 = (float)((c1 & 7) < 4 ? (c1 & 7) : ((c1 & 7) == 4 ? 4 : ((c1 & 7) == 5 ? 6 : ((c1 & 7) == 6 ? 8 : 12)))) * 0.5f;
        if ((c0 & 8) && (c0 & 7)) v0 = -v0;      // code 8 is +0 in the reference table
        if ((c1 & 8) && (c1 & 7)) v1 = -v1;
        v0 = __fmul_rn(v0, bs);
        v1 = __fmul_rn(v1, bs);
        if (GROUP == 16) { v0 = __fmul_rn(v0, ts); v1 = __fmul_rn(v1, ts); }
        o[i] = pack_bf16x2(v0, v1);
    }
    *reinterpret_cast<uint4*>(out + (size_t)r * ld_out + (size_t)c8 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

int dequant_fp4_blocks(const void* w, const void* scales, const void* s2, void* out, int out_f, int in_f, int group, long long ld_out,
                       cudaStream_t st) {
    if (out_f <= 0 || in_f <= 0 || in_f % 32 || (group != 16 && group != 32) || ld_out < in_f || ld_out % 8) return QB_ERR_ARG;
    if (!w || !scales || !out || ((uintptr_t)w & 3) || ((uintptr_t)out & 15) || ((uintptr_t)s2 & 3)) return QB_ERR_ARG;
    const long long n = (long long)out_f * (in_f / 8);
    const int blocks = (int)((n + 255) / 256);
    if (group == 32)
        dequant_fp4_blocks_kernel<32><<<blocks, 256, 0, st>>>((const uint32_t*)w, (const uint8_t*)scales, nullptr, (__nv_bfloat16*)out, out_f, in_f, ld_out);
    else
        dequant_fp4_blocks_kernel<16><<<blocks, 256, 0, st>>>((const uint32_t*)w, (const uint8_t*)scales, (const float*)s2, (__nv_bfloat16*)out, out_f, in_f, ld_out);
    return (int)cudaGetLastError();
}

}  // namespace qb
