// One- and two-token linear layer on the dense two-level NVFP4 weight: activation quantiser and matrix-vector product in
// one launch, on the CUDA cores.
//
// Replaces, for tok <= 2, the pair quantize_act_nvfp4_2lvl + the thin-token GEMM that the reference's decode path runs as
// its dense GEMV (cuda/dense_decode_lib.cu:19-141): at one or two tokens the tensor-core kernel is all fixed cost (launch
// of two kernels, tensor-memory and barrier set-up, accumulator hand-over), while the arithmetic per weight byte is small
// enough for the ordinary pipes:
//   * every CTA quantises the token rows itself (K <= 16384 values each, bit-identical to quant_act_kernel: per-token
//     global amax / 2688, UE4M3 scale per 16, E2M1 codes from the IEEE quotient) and keeps the CODE VALUES as f16 and the
//     decoded block scales as f32 in shared memory;
//   * a warp works on items of 4 weight rows x 4 K blocks (lane = 32 weights of one K block = two scale blocks; the
//     rows of an item are 32 apart, so that their scale pairs share one 16-byte piece of a scale atom), the next item's
//     five 16-byte loads in flight while the current one is processed, and the activation slice of the K group stays in
//     registers while the rows stream by;
//   * `cvt.rn.f16x2.e2m1x2` turns a weight byte into two f16 values, `fma.rn.f16x2` multiplies them with the activation
//     code values and sums 8 products per half: all of these are multiples of 1/4 below 512, so the f16 sums are EXACT;
//     the two halves are added in fp32 and scaled by (weight scale x activation scale), accumulated in fp32 over the blocks,
//     and the row result is multiplied by the two globals: the arithmetic of the block-scaled tensor-core instruction with
//     fp32 accumulation in a fixed order.
// Chunks of 4 rows are dealt to CTAs round-robin (every SM streams the same number of bytes), a CTA's (K group, chunk)
// items to its warps in equal contiguous ranges; the partial sums of the K groups meet in shared memory. The first item
// is requested before griddepcontrol.wait (weights are constants), the activations after it.
#include "qb_common.cuh"
#include "qb_internal.h"
#include "../../include/quadbit_b200.h"

namespace qb {

__device__ __forceinline__ void cvt_e2m1x8_f16(uint32_t w, uint32_t (&h)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(w));
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// two UE4M3 scale bytes -> two floats
__device__ __forceinline__ float2 dec_ue4m3x2(uint16_t s) {
    uint32_t h;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"(s));
    return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
__device__ __forceinline__ float sum_f16x2(uint32_t a) { const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&a)); return f.x + f.y; }

constexpr int GEMV_THREADS = 512;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

// Weight side of one work item: 4 rows {r0 + 32 k} of a 128-row tile x one K group (4 K blocks = 1024 weights per row; lane l
// holds the 32 weights of K block 4 g + l / 8, piece l % 8), and the 16 bytes of the scale atom that hold these lanes' scale
// pairs for all four rows (rows 32 apart share an atom line: that is why a chunk is made of such rows).
struct GemvItem {
    uint4 w[4];
    uint4 s;
};

template <int M>
__global__ void __launch_bounds__(GEMV_THREADS, 1)
nvfp4_gemv_kernel(const uint4* __restrict__ At, const uint8_t* __restrict__ sfa, const float* __restrict__ gA,
                  const uint4* __restrict__ x, __nv_bfloat16* __restrict__ C, int out_f, int K, int kblocks) {
    extern __shared__ __align__(16) uint8_t gemv_smem[];
    const int Kp = kblocks * 256;
    uint32_t* xh = reinterpret_cast<uint32_t*>(gemv_smem);                       // [M][Kp / 2] f16x2 code values
    float* sb = reinterpret_cast<float*>(gemv_smem + (size_t)M * Kp * 2);         // [M][Kp / 16] block scales
    float* part = sb + (size_t)M * (Kp >> 4);                                      // [items][4 rows][M] partial sums
    __shared__ float red[32];
    __shared__ float gBs[M];
    griddep_launch_dependents();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane & 7, kq = lane >> 3;                                      // 16-byte piece of a tile row, K block of the group
    const int chunks = out_f >> 2;                                                 // 4 rows each
    const int nch = (chunks - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // chunks of this CTA: blockIdx.x + i * gridDim.x
    const int G = (kblocks + 3) >> 2;
    const int T = G * nch;                                                         // items of this CTA, K group major
    const int t_begin = (int)((long long)warp * T / GEMV_WARPS), t_end = (int)((long long)(warp + 1) * T / GEMV_WARPS);   // sizes differ by at most one
    const int apr = kblocks * 4;                                                   // scale atoms per 128-row block (per-16 scales)

    // item t = (K group g, i-th chunk of the CTA), walked without divisions: (lg, li) belong to the item that is loaded next
    int lg = nch > 0 ? t_begin / nch : 0, li = nch > 0 ? t_begin - lg * nch : 0;
    auto load_item = [&](int t, GemvItem& it) {
#pragma unroll
        for (int k = 0; k < 4; k++) it.w[k] = make_uint4(0, 0, 0, 0);
        it.s = make_uint4(0, 0, 0, 0);
        if (t >= t_end) return;
        const int g = lg, c = (int)blockIdx.x + li * (int)gridDim.x;
        if (++li == nch) { li = 0; lg++; }
        const int kb = g * 4 + kq;
        if (kb >= kblocks) return;
        const int tile = c >> 5, r0 = c & 31;
        const uint4* wp = At + (((size_t)tile * kblocks + kb) * 128 + r0) * 8 + sub;
#pragma unroll
        for (int k = 0; k < 4; k++) it.w[k] = __ldg(wp + (size_t)k * 32 * 8);
        it.s = __ldg(reinterpret_cast<const uint4*>(sfa + ((size_t)tile * apr + kb * 4 + (sub >> 1)) * 512 + (size_t)r0 * 16));
    };
    GemvItem cur;
    int cg = lg, ci = li;                                // (K group, chunk) of the item in `cur`
    load_item(t_begin, cur);                             // weights are constants: requested before the activations are touched

    griddep_wait();
    // ---- activation quantiser (every CTA, all its threads): the arithmetic of quant_act_kernel<16, ., true>
    const int nblk = K >> 4, nblk_p = Kp >> 4;
#pragma unroll
    for (int m = 0; m < M; m++) {
        const uint4* xr = x + (size_t)m * (K >> 3);
        float tmax = 0.f;
        for (int b = threadIdx.x; b < nblk; b += GEMV_THREADS)
            tmax = fmaxf(tmax, fmaxf(absmax8_bf16(__ldg(xr + 2 * b)), absmax8_bf16(__ldg(xr + 2 * b + 1))));
        tmax = warp_max(tmax);
        __syncthreads();                             // red is reused by the next token
        if (lane == 0) red[warp] = tmax;
        __syncthreads();
        float r = lane < GEMV_WARPS ? red[lane] : 0.f;
        r = warp_max(r);
        const float gl = fmaxf(__fdiv_rn(r, 2688.f), 1e-30f);
        if (threadIdx.x == 0) gBs[m] = gl;
        for (int b = threadIdx.x; b < nblk_p; b += GEMV_THREADS) {
            uint32_t hv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            float sdec = 0.f;
            if (b < nblk) {
                const uint4 v0 = __ldg(xr + 2 * b), v1 = __ldg(xr + 2 * b + 1);
                const float bmax = fmaxf(absmax8_bf16(v0), absmax8_bf16(v1));
                const uint32_t code = enc_ue4m3(__fdiv_rn(__fdiv_rn(bmax, 6.f), gl));
                sdec = dec_ue4m3(code);
                const Fp4Divider dv(fmaxf(__fmul_rn(sdec, gl), 1e-30f));
                const uint32_t vw[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                float f8[8];
#pragma unroll
                for (int h = 0; h < 2; h++) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        f8[2 * i] = __uint_as_float(vw[4 * h + i] << 16);
                        f8[2 * i + 1] = __uint_as_float(vw[4 * h + i] & 0xffff0000u);
                    }
                    uint32_t hh[4];
                    cvt_e2m1x8_f16(dv.pack8(f8), hh);
#pragma unroll
                    for (int i = 0; i < 4; i++) hv[4 * h + i] = hh[i];
                }
            }
            // shared-memory order [K block][16-byte piece q of a lane's 32 values][lane piece `sub`]: the eight pieces of a
            // q are 128 contiguous bytes, so the 16-byte reads of the main loop hit distinct banks
            uint4* dst = reinterpret_cast<uint4*>(xh + (size_t)m * (Kp >> 1)) + ((size_t)(b >> 4) * 4 + (b & 1) * 2) * 8 + ((b & 15) >> 1);
            dst[0] = make_uint4(hv[0], hv[1], hv[2], hv[3]);
            dst[8] = make_uint4(hv[4], hv[5], hv[6], hv[7]);
            sb[(size_t)m * nblk_p + b] = sdec;
        }
    }
    __syncthreads();

    // ---- the items of this warp: the activation slice of a K group stays in registers while the rows stream by
    uint4 xa[M][4];
    float2 sB[M];
    int g_have = -1;
    for (int t = t_begin; t < t_end; t++) {
        GemvItem nxt;
        load_item(t + 1, nxt);                           // in flight while item t is processed
        const int g = cg;
        if (++ci == nch) { ci = 0; cg++; }
        const int kb = g * 4 + kq;
        if (g != g_have) {
            g_have = g;
#pragma unroll
            for (int m = 0; m < M; m++) {
                if (kb < kblocks) {
                    const uint4* xs = reinterpret_cast<const uint4*>(xh + (size_t)m * (Kp >> 1)) + (size_t)kb * 32 + sub;
                    xa[m][0] = xs[0]; xa[m][1] = xs[8]; xa[m][2] = xs[16]; xa[m][3] = xs[24];
                    sB[m] = *reinterpret_cast<const float2*>(sb + (size_t)m * nblk_p + kb * 16 + sub * 2);
                } else {
                    xa[m][0] = xa[m][1] = xa[m][2] = xa[m][3] = make_uint4(0, 0, 0, 0);
                    sB[m] = make_float2(0.f, 0.f);
                }
            }
        }
        const uint32_t sw[4] = {cur.s.x, cur.s.y, cur.s.z, cur.s.w};
        float acc[4][M];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            // the scale pair of this lane's two blocks in row r0 + 32 k: bytes (sub & 1) * 2, + 1 of word k
            const float2 sA = dec_ue4m3x2((uint16_t)((sub & 1) ? (sw[k] >> 16) : (sw[k] & 0xffffu)));
            uint32_t wa[4], wb[4], wc[4], wd[4];
            cvt_e2m1x8_f16(cur.w[k].x, wa);
            cvt_e2m1x8_f16(cur.w[k].y, wb);
            cvt_e2m1x8_f16(cur.w[k].z, wc);
            cvt_e2m1x8_f16(cur.w[k].w, wd);
#pragma unroll
            for (int m = 0; m < M; m++) {
                const uint4 x0 = xa[m][0], x1 = xa[m][1], x2 = xa[m][2], x3 = xa[m][3];
                uint32_t a0 = hfma2(wa[0], x0.x, 0u);
                a0 = hfma2(wa[1], x0.y, a0); a0 = hfma2(wa[2], x0.z, a0); a0 = hfma2(wa[3], x0.w, a0);
                a0 = hfma2(wb[0], x1.x, a0); a0 = hfma2(wb[1], x1.y, a0); a0 = hfma2(wb[2], x1.z, a0); a0 = hfma2(wb[3], x1.w, a0);
                uint32_t a1 = hfma2(wc[0], x2.x, 0u);
                a1 = hfma2(wc[1], x2.y, a1); a1 = hfma2(wc[2], x2.z, a1); a1 = hfma2(wc[3], x2.w, a1);
                a1 = hfma2(wd[0], x3.x, a1); a1 = hfma2(wd[1], x3.y, a1); a1 = hfma2(wd[2], x3.z, a1); a1 = hfma2(wd[3], x3.w, a1);
                acc[k][m] = fmaf(sum_f16x2(a1), sA.y * sB[m].y, sum_f16x2(a0) * (sA.x * sB[m].x));
            }
        }
        // sum over the 32 lanes of every (row, token): halving exchanges first (4 values -> 1 per lane), then a plain butterfly
#pragma unroll
        for (int m = 0; m < M; m++) {
            const bool hi16 = lane & 16, hi8 = lane & 8;
            float a = hi16 ? acc[2][m] : acc[0][m], b = hi16 ? acc[3][m] : acc[1][m];
            a += __shfl_xor_sync(0xffffffffu, hi16 ? acc[0][m] : acc[2][m], 16);
            b += __shfl_xor_sync(0xffffffffu, hi16 ? acc[1][m] : acc[3][m], 16);
            float v = hi8 ? b : a;
            v += __shfl_xor_sync(0xffffffffu, hi8 ? a : b, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            // lanes 0 / 8 / 16 / 24 hold rows k = 0 / 1 / 2 / 3
            if ((lane & 7) == 0) part[((size_t)t * 4 + (lane >> 3)) * M + m] = v;
        }
        cur = nxt;
    }
    __syncthreads();
    // ---- sum the K groups, apply the globals, store
    for (int o = threadIdx.x; o < nch * 4 * M; o += GEMV_THREADS) {
        const int m = o % M, k = (o / M) & 3, i = o / (4 * M);
        float a = 0.f;
        for (int g = 0; g < G; g++) a += part[((size_t)(g * nch + i) * 4 + k) * M + m];
        const int c = (int)blockIdx.x + i * (int)gridDim.x;
        const int row = (c >> 5) * 128 + (c & 31) + 32 * k;
        C[(size_t)m * out_f + row] = __float2bfloat16_rn(a * __ldg(gA + row) * gBs[m]);
    }
}

static size_t gemv_smem_bytes(int tok, int kblocks, int out_f, int ctas) {
    const int nch = (out_f / 4 + ctas - 1) / ctas, G = (kblocks + 3) / 4;
    return (size_t)tok * kblocks * 256 * 2 + (size_t)tok * kblocks * 16 * 4 + (size_t)G * nch * 4 * tok * 4;
}

// x [tok][K] bf16 (tok 1 or 2), At / sfa / gA: the dense weight in the tiled layout with scale atoms (per 16) and per-row
// globals, C [tok][out] bf16. Launched as a programmatic dependent of the kernel in front of it on the stream.
int linear_gemv_dense(const void* x, const void* At, const void* sfa, const void* gA, void* C, int out_f, int tok, int K, cudaStream_t st) {
    if (out_f <= 0 || K <= 0 || out_f % 128 || K % 128 || tok < 0 || tok > 2) return QB_ERR_ARG;
    if (tok == 0) return QB_OK;
    if (!x || !At || !sfa || !gA || !C || ((uintptr_t)x & 15) || ((uintptr_t)At & 15) || ((uintptr_t)sfa & 15) || ((uintptr_t)C & 1)) return QB_ERR_ARG;
    const int kblocks = kpad256(K) / 256;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t smem = gemv_smem_bytes(tok, kblocks, out_f, sms);
    if (smem > 200 * 1024) return QB_ERR_UNSUPPORTED;
    static bool attr_set[64][2] = {};                 // the attribute belongs to the device's context: once per device and kernel
    auto kern = tok == 1 ? nvfp4_gemv_kernel<1> : nvfp4_gemv_kernel<2>;
    if (dev < 0 || dev >= 64 || !attr_set[dev][tok - 1]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        if (dev >= 0 && dev < 64) attr_set[dev][tok - 1] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)sms);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, (const uint4*)At, (const uint8_t*)sfa, (const float*)gA, (const uint4*)x, (__nv_bfloat16*)C, out_f, K, kblocks);
}

}  // namespace qb
