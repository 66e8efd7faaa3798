// Host-layer glue of the model forward that is not a quantiser: rotary position embedding applied in place to the
// q and k heads of a token-major QKV GEMM output. The reference leaves RoPE to the framework's attention module
// (attention stays bf16 there, harness/real_model.py:181-188); as a chain of elementwise torch kernels it cost more than
// the attention itself at prefill sizes, so it is one pass here: fp32 arithmetic on the bf16 inputs, one rounding.
#include "../../include/quadbit_b200.h"
#include "qb_common.cuh"
#include "qb_internal.h"

namespace {

// x [tok][row_stride] bf16; the first n_heads * 128 columns of every row are heads of 128 values, rotated with the
// rotate-half convention: (x1, x2) = (x[0:64], x[64:128]) -> (x1 c - x2 s, x2 c + x1 s), c / s = tab[pos][0:64] / [64:128].
// One thread owns 8 lanes i of one head (both halves): two 16-byte loads, two 16-byte stores.
__global__ void __launch_bounds__(256) rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ tab, int tok, int seq,
                                                   long long row_stride, int n_heads) {
    const int per_tok = n_heads * 8;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (long long)tok * per_tok) return;
    const int t = (int)(gid / per_tok), w = (int)(gid % per_tok);
    const int head = w >> 3, i0 = (w & 7) * 8;
    const int pos = t % seq;
    __nv_bfloat16* p1 = x + (size_t)t * row_stride + head * 128 + i0;
    __nv_bfloat16* p2 = p1 + 64;
    const uint4 a = *reinterpret_cast<const uint4*>(p1), b = *reinterpret_cast<const uint4*>(p2);
    const float4 c0 = __ldg(reinterpret_cast<const float4*>(tab + (size_t)pos * 128 + i0));
    const float4 c1 = __ldg(reinterpret_cast<const float4*>(tab + (size_t)pos * 128 + i0 + 4));
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(tab + (size_t)pos * 128 + 64 + i0));
    const float4 s1 = __ldg(reinterpret_cast<const float4*>(tab + (size_t)pos * 128 + 64 + i0 + 4));
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 oa, ob;
    uint32_t* oaw = reinterpret_cast<uint32_t*>(&oa);
    uint32_t* obw = reinterpret_cast<uint32_t*>(&ob);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float2 x1 = __bfloat1622float2(ah[k]), x2 = __bfloat1622float2(bh[k]);
        // products rounded separately (no fused multiply-add), as an elementwise framework expression evaluates them
        const float r1x = __fsub_rn(__fmul_rn(x1.x, c[2 * k]), __fmul_rn(x2.x, s[2 * k]));
        const float r1y = __fsub_rn(__fmul_rn(x1.y, c[2 * k + 1]), __fmul_rn(x2.y, s[2 * k + 1]));
        const float r2x = __fadd_rn(__fmul_rn(x2.x, c[2 * k]), __fmul_rn(x1.x, s[2 * k]));
        const float r2y = __fadd_rn(__fmul_rn(x2.y, c[2 * k + 1]), __fmul_rn(x1.y, s[2 * k + 1]));
        oaw[k] = qb::pack_bf16x2(r1x, r1y);
        obw[k] = qb::pack_bf16x2(r2x, r2y);
    }
    *reinterpret_cast<uint4*>(p1) = oa;
    *reinterpret_cast<uint4*>(p2) = ob;
}

}  // namespace

extern "C" int qb_rope_inplace(void* x, const void* cos_sin, int tok, int seq, long long row_stride, int n_heads, void* stream) {
    if (tok < 0 || seq <= 0 || n_heads <= 0 || row_stride < (long long)n_heads * 128 || (row_stride & 7)) return QB_ERR_ARG;
    if (tok == 0) return QB_OK;
    if (!x || !cos_sin || ((uintptr_t)x & 15) || ((uintptr_t)cos_sin & 15)) return QB_ERR_ARG;
    const long long total = (long long)tok * n_heads * 8;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    rope_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, (const float*)cos_sin, tok, seq, row_stride, n_heads);
    return (int)cudaGetLastError();
}
