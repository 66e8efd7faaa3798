// Fused bf16 -> NVFP4 activation quantiser (two-level and single-level, per-32 for the
// 2:4-sparse GEMM, per-16 for the dense GEMM) and the scale / metadata re-layout kernels.
//
// Replaces quant_act / quant_act_2lvl_k (cuda/sparse_fp4_lib.cu:704-786) and quant_act_nv /
// quant_act_nv2_k (cuda/dense_nvfp4_fast_lib.cu:175-206,305-342). Arithmetic follows the
// reference's torch fake-quant (act_2lvl_deq_p32, harness/verify_sparse_2lvl.py:100-106;
// act_fp4_dequant, harness/recovery_worth.py:78-84) bit for bit: IEEE divisions, boundary
// values to the lower E2M1 code, divisor clamped to 1e-30 for all-zero blocks.
//
// HBM-bound: one CTA per token row; every lane moves 16 bytes (8 bf16) per load so a warp
// reads 512 contiguous bytes, the row stays in registers between the amax pass and the
// quantise pass (each input byte is read once), the block amax is a 2- or 4-lane shuffle
// reduction, each lane writes one packed 32-bit word (a warp writes 128 contiguous bytes)
// and four scale bytes are merged into one 32-bit store.
#include "qb_common.cuh"
#include "qb_internal.h"

namespace qb {

// One CTA per token row; every thread owns whole scale blocks (BLOCK consecutive values, NJ blocks per
// thread), so the per-block scale arithmetic (two IEEE divisions, the UE4M3 encode / decode, the
// reciprocal of the divider) runs once per block and lane: with the 8-values-per-lane mapping it ran in
// all BLOCK/8 lanes of a block, and the kernel was issue-bound (ncu: 92 % issue-active, 59 warp
// instructions per value) at a fifth of the HBM rate.
struct GatherPeers {
    const uint4* p[8];
    long long rows_per;
    int n;
    const int* n_rows;      // non-null: rows at and beyond *n_rows are unused capacity of a routed batch and are left alone
};

template <int BLOCK, int NJ, bool TWO_LEVEL>
__device__ __forceinline__ void quant_act_row(const int row, const uint4* __restrict__ x, uint32_t* __restrict__ Bwords,
                                              uint8_t* __restrict__ sf_ref, uint8_t* __restrict__ sf_atoms, float* __restrict__ g_out, int tok,
                                              int K, const long long* __restrict__ src, int h8, const GatherPeers& peers) {
    // src != nullptr: row `row` of the output quantises source row src[row] of x [.][h8 * 8] zero-padded to K
    // (src < 0: an all-zero row) — the gather of routed MoE rows fused into their quantiser
    constexpr int CPB = BLOCK / 8;   // 16-byte input chunks (8 values) per scale block
    constexpr int P = 128 / BLOCK;   // scales per 128 K in the reference layout
    const int nblocks = K / BLOCK;   // a multiple of 4 (K % 128 == 0)
    const int lane = threadIdx.x & 31;
    const long long srow = src ? src[row] : (long long)row;
    // peers.n > 0: source rows are numbered over all ranks (rows_per rows each) and read from the rank that holds them
    // (plain loads from peer-mapped memory: the dispatch of an expert-parallel layer folded into the gather)
    const uint4* xr;
    if (peers.n > 0 && srow >= 0) {
        const int owner = (int)(srow / peers.rows_per);
        xr = peers.p[owner] + (size_t)(srow - (long long)owner * peers.rows_per) * h8;
    } else {
        xr = x + (size_t)(srow < 0 ? 0 : srow) * h8;
    }
    if (srow < 0) {
        // With a rows-in-use limit (the fixed-capacity routing of the MoE layer) a padding row is left unwritten: the grouped
        // GEMM computes its token column from whatever the buffers hold, every token column is independent of the others,
        // and no one reads the result rows of padding (the combine follows the slot -> row table).
        if (peers.n_rows) return;
        // padding row: what the full path makes of an all-zero row (codes 0, scale codes 0, global 1e-30), without the passes
        for (int b = threadIdx.x; b < nblocks; b += blockDim.x) {
            uint32_t* dst = Bwords + (size_t)row * (K >> 3) + (size_t)b * CPB;
#pragma unroll
            for (int k = 0; k < CPB; k++) dst[k] = 0u;
            if ((b & 3) == 0) {
                if (sf_ref) *reinterpret_cast<uint32_t*>(sf_ref + ((size_t)(b / P) * tok + row) * P + (b % P)) = 0u;
                if (sf_atoms) *reinterpret_cast<uint32_t*>(sf_atoms + sf_atom_offset(row, b, kpad256(K) / BLOCK / 4)) = 0u;
            }
        }
        if (TWO_LEVEL && threadIdx.x == 0) g_out[row] = 1e-30f;
        return;
    }

    uint4 v[NJ][CPB];
    float bmax[NJ];
    float tmax = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int b = threadIdx.x + j * blockDim.x;
        float m = 0.f;
#pragma unroll
        for (int k = 0; k < CPB; k++) {
            v[j][k] = make_uint4(0, 0, 0, 0);
            if (b < nblocks && b * CPB + k < h8 && srow >= 0) v[j][k] = peers.n > 0 ? __ldcg(xr + (size_t)b * CPB + k) : __ldg(xr + (size_t)b * CPB + k);
            m = fmaxf(m, absmax8_bf16(v[j][k]));
        }
        bmax[j] = m;
        tmax = fmaxf(tmax, m);
    }

    float gl = 1.f;
    if (TWO_LEVEL) {
        __shared__ float red[32];
        tmax = warp_max(tmax);
        if (lane == 0) red[threadIdx.x >> 5] = tmax;
        __syncthreads();
        float r = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.f;
        r = warp_max(r);
        gl = fmaxf(__fdiv_rn(r, 2688.f), 1e-30f);
        if (threadIdx.x == 0) g_out[row] = gl;
    }

    const bool wide = (reinterpret_cast<uintptr_t>(Bwords) & 15) == 0;   // rows are multiples of 64 bytes
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int b = threadIdx.x + j * blockDim.x;
        const uint32_t code = TWO_LEVEL ? enc_ue4m3(__fdiv_rn(__fdiv_rn(bmax[j], 6.f), gl)) : enc_ue4m3(__fdiv_rn(bmax[j], 6.f));
        const float sdeq = TWO_LEVEL ? __fmul_rn(dec_ue4m3(code), gl) : dec_ue4m3(code);
        const Fp4Divider dv(fmaxf(sdeq, 1e-30f));
        uint32_t w[CPB];
#pragma unroll
        for (int k = 0; k < CPB; k++) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[j][k]);
            float f8[8];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 f = __bfloat1622float2(h[i]);
                f8[2 * i] = f.x; f8[2 * i + 1] = f.y;
            }
            w[k] = dv.pack8(f8);
        }
        // the scale codes of 4 consecutive blocks (4 consecutive lanes) make one word (all lanes shuffle)
        uint32_t sw = 0;
        const int base = lane & ~3;
#pragma unroll
        for (int i = 0; i < 4; i++) sw |= __shfl_sync(0xffffffffu, code, base + i) << (8 * i);
        if (b < nblocks) {
            uint32_t* dst = Bwords + (size_t)row * (K >> 3) + (size_t)b * CPB;
            if (wide) {
                if constexpr (CPB == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                else *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
            } else {
#pragma unroll
                for (int k = 0; k < CPB; k++) dst[k] = w[k];
            }
            if ((lane & 3) == 0) {
                const int jcol = b;   // scale column, a multiple of 4 here
                if (sf_ref) *reinterpret_cast<uint32_t*>(sf_ref + ((size_t)(jcol / P) * tok + row) * P + (jcol % P)) = sw;
                if (sf_atoms) *reinterpret_cast<uint32_t*>(sf_atoms + sf_atom_offset(row, jcol, kpad256(K) / BLOCK / 4)) = sw;
            }
        }
    }
}

// One CTA per row; with a rows-in-use limit (routed batches with fixed capacity) a bounded grid walks the rows instead, so that
// unused capacity costs no CTA launches (34816 rows of capacity for ~4100 in use cost 47 us of empty CTAs otherwise).
template <int BLOCK, int NJ, bool TWO_LEVEL>
__global__ void __launch_bounds__(1024) quant_act_kernel(const uint4* __restrict__ x, uint32_t* __restrict__ Bwords,
                                                          uint8_t* __restrict__ sf_ref, uint8_t* __restrict__ sf_atoms,
                                                          float* __restrict__ g_out, int tok, int K,
                                                          const long long* __restrict__ src, int h8, const GatherPeers peers) {
    griddep_launch_dependents();     // a thin-token GEMM that follows may set itself up while this grid runs
    griddep_wait();                  // launched as a programmatic dependent itself: x may come from the kernel in front
    const int nrows = peers.n_rows ? min(tok, *peers.n_rows) : tok;
    for (int row = blockIdx.x; row < nrows; row += gridDim.x) {
        quant_act_row<BLOCK, NJ, TWO_LEVEL>(row, x, Bwords, sf_ref, sf_atoms, g_out, tok, K, src, h8, peers);
        __syncthreads();             // the row's reduction scratch is reused by the next row
    }
}

// SwiGLU + two-level per-32 quantiser for the fused MLP: reads the token-major gate/up GEMM
// output Cgu[tok][2*I] (gate features 0..I-1, up features I..2I-1, bf16), forms
// h = silu(g) * u in fp32 and quantises h exactly like an activation row (per-token global
// gH = amax/2688, per-32 UE4M3 local scale, E2M1 codes) into Hb[tok][I/2] + scale atoms, the
// B operand of the down projection. One pass, one CTA per token, h stays in registers.
// Replaces swiglu_amax / swiglu_finalize / swiglu_quant_g (cuda/sparse_fp4_lib.cu:837-894),
// which make three passes over a feature-major Cgu.
// Every lane owns whole 32-value scale blocks (NJ per lane), like quant_act_kernel.
// INTERLEAVED: the row holds (gate, up) pairs [g0,u0,g1,u1,...] as the gpt-oss fused gate_up weight produces
// them; TWO_LEVEL = false is the single-level quantiser (no per-token global) that the reference's fused MoE
// GEMM1 epilogue applies (matmul_sp_moe_gu_swiglu, cuda/sparse_fp4_lib.cu:1828-1866); act 0 is the clamped
// gpt-oss SwiGLU (alpha 1.702, limit 7, up + 1), act 1 the plain silu(g) * u.
template <int NJ, bool INTERLEAVED, bool TWO_LEVEL, int ACT>
__device__ __forceinline__ void swiglu_quant_row(const int row, const uint4* __restrict__ cgu, uint32_t* __restrict__ Hwords,
                                                 uint8_t* __restrict__ sf_ref, uint8_t* __restrict__ sf_atoms, float* __restrict__ g_out, int tok,
                                                 int I, const long long* __restrict__ row_src, const bool skip_padding) {
    const int nchunks = I >> 3;
    const int nblocks = I >> 5;          // a multiple of 4 (I % 128 == 0)
    const int lane = threadIdx.x & 31;
    const uint4* gr = cgu + (size_t)row * (nchunks * 2);
    const uint4* ur = gr + nchunks;
    if (row_src && row_src[row] < 0) {
        if (skip_padding) return;          // rows-in-use mode: padding rows stay unwritten (see quant_act_row)
        // padding row of a routed batch (its gate/up row may never have been written): zeros, as for an all-zero row
        for (int b = threadIdx.x; b < nblocks; b += blockDim.x) {
            uint32_t* dst = Hwords + (size_t)row * nchunks + (size_t)b * 4;
            dst[0] = 0u; dst[1] = 0u; dst[2] = 0u; dst[3] = 0u;
            if ((b & 3) == 0) {
                if (sf_ref) *reinterpret_cast<uint32_t*>(sf_ref + ((size_t)(b >> 2) * tok + row) * 4) = 0u;
                if (sf_atoms) *reinterpret_cast<uint32_t*>(sf_atoms + sf_atom_offset(row, b, kpad256(I) / 128)) = 0u;
            }
        }
        if (TWO_LEVEL && threadIdx.x == 0) g_out[row] = 1e-30f;
        return;
    }
    float h[NJ][32];
    float bmax[NJ];
    float tmax = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int b = threadIdx.x + j * blockDim.x;
        float m = 0.f;
        // all eight 16-byte loads of the block are issued before any of the exp / divide chains starts
        uint4 gq[4], uq[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            gq[k] = make_uint4(0, 0, 0, 0);
            uq[k] = make_uint4(0, 0, 0, 0);
            if (INTERLEAVED) {   // gq, uq: the two halves of 8 consecutive (gate, up) pairs
                if (b < nblocks) { gq[k] = __ldg(gr + (size_t)b * 8 + 2 * k); uq[k] = __ldg(gr + (size_t)b * 8 + 2 * k + 1); }
            } else {
                if (b < nblocks) { gq[k] = __ldg(gr + (size_t)b * 4 + k); uq[k] = __ldg(ur + (size_t)b * 4 + k); }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint4 gv = gq[k], uv = uq[k];
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float a, c;
                if (INTERLEAVED) {
                    if ((i & 1) == 0) {     // words 2i', 2i'+1 of the first half: pairs (g, u) of two neighbouring features
                        swiglu_h2_pairs<ACT>(gw[i], gw[i + 1], a, c);
                        h[j][8 * k + i] = a; h[j][8 * k + i + 1] = c;
                    } else {
                        swiglu_h2_pairs<ACT>(uw[i - 1], uw[i], a, c);
                        h[j][8 * k + 4 + i - 1] = a; h[j][8 * k + 4 + i] = c;
                    }
                } else {
                    swiglu_h2_split<ACT>(gw[i], uw[i], a, c);
                    h[j][8 * k + 2 * i] = a; h[j][8 * k + 2 * i + 1] = c;
                }
                m = fmaxf(m, fmaxf(fabsf(a), fabsf(c)));
            }
        }
        bmax[j] = m;
        tmax = fmaxf(tmax, m);
    }
    float gl = 1.f;
    if (TWO_LEVEL) {
        __shared__ float red[32];
        tmax = warp_max(tmax);
        if (lane == 0) red[threadIdx.x >> 5] = tmax;
        __syncthreads();
        float r = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.f;
        r = warp_max(r);
        gl = fmaxf(__fdiv_rn(r, 2688.f), 1e-30f);
        if (threadIdx.x == 0) g_out[row] = gl;
    }
    const bool wide = (reinterpret_cast<uintptr_t>(Hwords) & 15) == 0;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int b = threadIdx.x + j * blockDim.x;
        const uint32_t code = TWO_LEVEL ? enc_ue4m3(__fdiv_rn(__fdiv_rn(bmax[j], 6.f), gl)) : enc_ue4m3(__fdiv_rn(bmax[j], 6.f));
        // h comes from exp / divide intrinsics and is only defined up to a few ulp, so the exact IEEE quotient of the
        // activation quantiser buys nothing here: one multiply by the reciprocal of the scale and the hardware E2M1
        // conversion; against the exact path a code can differ only where the quotient sits within an ulp or two of a
        // rounding boundary (the parity test checks exactly that: every differing code lies on a boundary)
        const float rs = __frcp_rn(fmaxf(TWO_LEVEL ? __fmul_rn(dec_ue4m3(code), gl) : dec_ue4m3(code), 1e-30f));
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float lo4[4] = {h[j][8 * k], h[j][8 * k + 1], h[j][8 * k + 2], h[j][8 * k + 3]};
            const float hi4[4] = {h[j][8 * k + 4], h[j][8 * k + 5], h[j][8 * k + 6], h[j][8 * k + 7]};
            w[k] = pack4_e2m1_rcp(lo4, rs) | (pack4_e2m1_rcp(hi4, rs) << 16);
        }
        uint32_t sw = 0;
        const int base = lane & ~3;
#pragma unroll
        for (int i = 0; i < 4; i++) sw |= __shfl_sync(0xffffffffu, code, base + i) << (8 * i);
        if (b < nblocks) {
            uint32_t* dst = Hwords + (size_t)row * nchunks + (size_t)b * 4;
            if (wide) *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
            else { dst[0] = w[0]; dst[1] = w[1]; dst[2] = w[2]; dst[3] = w[3]; }
            if ((lane & 3) == 0) {
                const int jcol = b;      // scale column, a multiple of 4 here
                if (sf_ref) *reinterpret_cast<uint32_t*>(sf_ref + ((size_t)(jcol >> 2) * tok + row) * 4) = sw;
                if (sf_atoms) *reinterpret_cast<uint32_t*>(sf_atoms + sf_atom_offset(row, jcol, kpad256(I) / 128)) = sw;
            }
        }
    }
}

// one CTA per row, or a bounded grid walking the rows in use when a routed batch has unused capacity (n_rows)
template <int NJ, bool INTERLEAVED, bool TWO_LEVEL, int ACT>
__global__ void __launch_bounds__(512) swiglu_quant_kernel(const uint4* __restrict__ cgu, uint32_t* __restrict__ Hwords,
                                                            uint8_t* __restrict__ sf_ref, uint8_t* __restrict__ sf_atoms,
                                                            float* __restrict__ g_out, int tok, int I, const long long* __restrict__ row_src,
                                                            const int* __restrict__ n_rows) {
    const int nrows = n_rows ? min(tok, *n_rows) : tok;
    for (int row = blockIdx.x; row < nrows; row += gridDim.x) {
        swiglu_quant_row<NJ, INTERLEAVED, TWO_LEVEL, ACT>(row, cgu, Hwords, sf_ref, sf_atoms, g_out, tok, I, row_src, n_rows != nullptr);
        __syncthreads();
    }
}


int swiglu_quant(const void* cgu, void* Hb, void* sf_ref, void* sf_atoms, void* gH, int tok, int I, cudaStream_t st) {
    return swiglu_quant_ex(cgu, Hb, sf_ref, sf_atoms, gH, tok, I, 0, 1, st, nullptr);
}

// interleaved: row layout [g0,u0,g1,u1,...]; gH == nullptr selects the single-level quantiser
int swiglu_quant_ex(const void* cgu, void* Hb, void* sf_ref, void* sf_atoms, void* gH, int tok, int I, int interleaved, int act,
                    cudaStream_t st, const void* row_src, const void* n_rows_dev) {
    if (tok < 0 || I <= 0 || I % 128 != 0 || (act != 0 && act != 1)) return QB_ERR_ARG;
    if (tok == 0) return QB_OK;
    if (!cgu || !Hb || (!sf_ref && !sf_atoms)) return QB_ERR_ARG;
    if (((uintptr_t)cgu & 15) || ((uintptr_t)Hb & 3) || ((uintptr_t)sf_ref & 3) || ((uintptr_t)sf_atoms & 3)) return QB_ERR_ARG;
    const int nblocks = I / 32;
    int threads = (nblocks + 31) / 32 * 32;
    if (threads > 512) threads = 512;
    const int nj = (nblocks + threads - 1) / threads;
#define QB_LS4(NJ, IL, TL, ACT) swiglu_quant_kernel<NJ, IL, TL, ACT><<<(n_rows_dev && tok > 148 * 16) ? 148 * 16 : tok, threads, 0, st>>>((const uint4*)cgu, (uint32_t*)Hb, (uint8_t*)sf_ref, (uint8_t*)sf_atoms, (float*)gH, tok, I, (const long long*)row_src, (const int*)n_rows_dev)
#define QB_LS3(NJ, IL, TL) do { if (act == 0) QB_LS4(NJ, IL, TL, 0); else QB_LS4(NJ, IL, TL, 1); } while (0)
#define QB_LS(NJ) do { if (interleaved) { if (gH) QB_LS3(NJ, true, true); else QB_LS3(NJ, true, false); } \
                       else { if (gH) QB_LS3(NJ, false, true); else QB_LS3(NJ, false, false); } } while (0)
    if (nj <= 1) QB_LS(1);
    else if (nj <= 2) QB_LS(2);
    else if (nj <= 4) QB_LS(4);
    else return QB_ERR_UNSUPPORTED;
#undef QB_LS
#undef QB_LS3
#undef QB_LS4
    return (int)cudaGetLastError();
}

// RMSNorm (optionally after a residual add that is written back as the new residual stream)
// fused with the NVFP4 quantiser: y = (x [+ res]) * rsqrt(mean(.^2) + eps) * w in fp32, quantised
// per BLOCK without passing through bf16. Replaces rmsnorm_quant_k / add_rmsnorm_quant_k
// (cuda/sparse_fp4_lib.cu:902-1011, single-level per-32) and, with TWO_LEVEL, also emits the
// per-token global so the following GEMM runs two-level. One CTA per row, row kept in registers.
// Tensor-parallel extras of the norm kernel (all off when nsrc == 1, fan == 0, wait_flags == null):
//   nsrc > 1   x is the first of nsrc bf16 sources [tok][H], src_stride uint4 apart: the partial results that the ranks'
//              row-parallel GEMMs stored into this rank's slots; they are summed in fp32 in source order (the reduction
//              half of a reduce-scatter), then the residual is added;
//   wait_flags every CTA first waits, bounded, until the nsrc words are >= wait_val (each source rank's "my partials
//              have landed"); on expiry the status word gets QB_ERR_TIMEOUT and the kernel goes on (wrong data, no hang);
//   fan > 0    packed bytes, scale atoms and globals go to `fan` destinations (the full-size arrays of every rank, rows
//              offset by row0): the all-gather of the quantised activations done by the stores themselves;
//   sig_n > 0  the last CTA to finish writes sig_val into word sig_rank of every rank's flag array.
struct NormTP {
    long long src_stride;
    int nsrc;
    const int* wait_flags;
    int wait_val;
    int fan;
    int row0;
    int tok_total;              // rows of the gathered arrays (for the scale layouts)
    uint32_t* Bwords[8];
    uint8_t* sf_atoms[8];
    float* g[8];
    int sig_n, sig_rank, sig_val;
    int* sig_flags[8];
    int* done;
    int* status;
    const int* val_ptr;
};
__device__ int g_quant_status = 0;

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// flag store after a __threadfence_system() (the fence orders the data before the flag; the store itself is relaxed)
__device__ __forceinline__ void st_flag_sys(int* p, int v) {
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int BLOCK, int NJ, bool ADD, bool TWO_LEVEL>
__global__ void __launch_bounds__(512) norm_quant_kernel(const uint4* __restrict__ x, const uint4* __restrict__ res,
                                                          const uint4* __restrict__ wt, uint4* __restrict__ hout,
                                                          uint32_t* __restrict__ Bwords, uint8_t* __restrict__ sf_ref,
                                                          uint8_t* __restrict__ sf_atoms, float* __restrict__ g_out, int tok, int H,
                                                          float eps, const NormTP tp) {
    // every lane owns whole scale blocks (BLOCK values, NJ per lane), like quant_act_kernel
    constexpr int CPB = BLOCK / 8, P = 128 / BLOCK;
    const int row = blockIdx.x;
    const int nchunks = H >> 3;
    const int nblocks = H / BLOCK;       // a multiple of 4 (H % 128 == 0)
    const int lane = threadIdx.x & 31;
    __shared__ float red[32];
    if (tp.wait_flags) {
        if ((int)threadIdx.x < tp.nsrc) {
            const uint64_t t0 = globaltimer_ns();
            uint32_t it = 0;
            const int want = tp.val_ptr ? *tp.val_ptr : tp.wait_val;
            while (ld_acquire_sys(tp.wait_flags + threadIdx.x) < want) {
                __nanosleep(200);
                if ((++it & 255u) == 0 && globaltimer_ns() - t0 > 20000000000ull) {      // 20 s
                    atomicCAS(tp.status, 0, QB_ERR_TIMEOUT * 100 + 20);
                    break;
                }
            }
        }
        __syncthreads();
    }
    float v[NJ][BLOCK];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int blk = threadIdx.x + j * blockDim.x;
#pragma unroll
        for (int k = 0; k < CPB; k++) {
            const size_t c = (size_t)blk * CPB + k;
            uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
            // sources written by other GPUs are read past the non-coherent path (ld.global, not ld.global.nc)
            if (blk < nblocks) {
                a = tp.nsrc > 1 ? __ldcg(x + (size_t)row * nchunks + c) : __ldg(x + (size_t)row * nchunks + c);
                if (ADD) b = __ldg(res + (size_t)row * nchunks + c);
            }
            const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
            float2 acc4[4];
#pragma unroll
            for (int i = 0; i < 4; i++) acc4[i] = __bfloat1622float2(ah[i]);
            for (int sidx = 1; sidx < tp.nsrc; sidx++) {
                uint4 e = make_uint4(0, 0, 0, 0);
                if (blk < nblocks) e = __ldcg(x + (size_t)sidx * tp.src_stride + (size_t)row * nchunks + c);
                const __nv_bfloat162* eh = reinterpret_cast<const __nv_bfloat162*>(&e);
#pragma unroll
                for (int i = 0; i < 4; i++) { const float2 t2 = __bfloat1622float2(eh[i]); acc4[i].x = __fadd_rn(acc4[i].x, t2.x); acc4[i].y = __fadd_rn(acc4[i].y, t2.y); }
            }
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 f = acc4[i];
                if (ADD) { float2 r2 = __bfloat1622float2(bh[i]); add_f32x2(f.x, f.y, r2.x, r2.y); oh[i] = __floats2bfloat162_rn(f.x, f.y); }
                v[j][8 * k + 2 * i] = f.x; v[j][8 * k + 2 * i + 1] = f.y;
                ss += f.x * f.x + f.y * f.y;
            }
            if (ADD && hout && blk < nblocks) hout[(size_t)row * nchunks + c] = o;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    const float rms = rsqrtf(tot / (float)H + eps);
    float bmax[NJ];
    float tmax = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int blk = threadIdx.x + j * blockDim.x;
        float m = 0.f;
#pragma unroll
        for (int k = 0; k < CPB; k++) {
            uint4 w4 = make_uint4(0, 0, 0, 0);
            if (blk < nblocks) w4 = __ldg(wt + (size_t)blk * CPB + k);
            const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&w4);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 w2 = __bfloat1622float2(wh[i]);
                const int e = 8 * k + 2 * i;
                mul_f32x2(v[j][e], v[j][e + 1], rms, rms);            // two IEEE-rounded products per instruction, as the scalar form
                mul_f32x2(v[j][e], v[j][e + 1], w2.x, w2.y);
                m = fmaxf(m, fmaxf(fabsf(v[j][e]), fabsf(v[j][e + 1])));
            }
        }
        bmax[j] = m;
        tmax = fmaxf(tmax, m);
    }
    float gl = 1.f;
    if (TWO_LEVEL) {
        __syncthreads();
        tmax = warp_max(tmax);
        if (lane == 0) red[threadIdx.x >> 5] = tmax;
        __syncthreads();
        float r = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.f;
        r = warp_max(r);
        gl = fmaxf(__fdiv_rn(r, 2688.f), 1e-30f);
        if (threadIdx.x == 0) {
            if (tp.fan) { for (int d = 0; d < tp.fan; d++) tp.g[d][tp.row0 + row] = gl; }
            else g_out[row] = gl;
        }
    }
    const bool wide = (reinterpret_cast<uintptr_t>(Bwords) & 15) == 0;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int blk = threadIdx.x + j * blockDim.x;
        const uint32_t code = TWO_LEVEL ? enc_ue4m3(__fdiv_rn(__fdiv_rn(bmax[j], 6.f), gl)) : enc_ue4m3(__fdiv_rn(bmax[j], 6.f));
        // the normalised values come from rsqrtf and are only defined up to an ulp or two, so (as in the SwiGLU quantiser)
        // the quotient is one multiply by the reciprocal of the scale and the hardware E2M1 conversion
        const float rs = __frcp_rn(fmaxf(TWO_LEVEL ? __fmul_rn(dec_ue4m3(code), gl) : dec_ue4m3(code), 1e-30f));
        uint32_t w[CPB];
#pragma unroll
        for (int k = 0; k < CPB; k++) {
            const float lo4[4] = {v[j][8 * k], v[j][8 * k + 1], v[j][8 * k + 2], v[j][8 * k + 3]};
            const float hi4[4] = {v[j][8 * k + 4], v[j][8 * k + 5], v[j][8 * k + 6], v[j][8 * k + 7]};
            w[k] = pack4_e2m1_rcp(lo4, rs) | (pack4_e2m1_rcp(hi4, rs) << 16);
        }
        uint32_t sw = 0;
        const int base = lane & ~3;
#pragma unroll
        for (int i = 0; i < 4; i++) sw |= __shfl_sync(0xffffffffu, code, base + i) << (8 * i);
        if (blk < nblocks) {
            if (tp.fan) {
                // every destination is the full gathered array of one rank; this rank's rows start at row0 there
                const size_t grow = (size_t)(tp.row0 + row);
                const size_t aoff = sf_atom_offset(tp.row0 + row, blk, kpad256(H) / BLOCK / 4);
                for (int d = 0; d < tp.fan; d++) {
                    uint32_t* dst = tp.Bwords[d] + grow * nchunks + (size_t)blk * CPB;
                    if constexpr (CPB == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                    else *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
                    if ((lane & 3) == 0) *reinterpret_cast<uint32_t*>(tp.sf_atoms[d] + aoff) = sw;
                }
            } else {
                uint32_t* dst = Bwords + (size_t)row * nchunks + (size_t)blk * CPB;
                if (wide) {
                    if constexpr (CPB == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                    else *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
                } else {
#pragma unroll
                    for (int k = 0; k < CPB; k++) dst[k] = w[k];
                }
                if ((lane & 3) == 0) {
                    const int jcol = blk;
                    if (sf_ref) *reinterpret_cast<uint32_t*>(sf_ref + ((size_t)(jcol / P) * tok + row) * P + (jcol % P)) = sw;
                    if (sf_atoms) *reinterpret_cast<uint32_t*>(sf_atoms + sf_atom_offset(row, jcol, kpad256(H) / BLOCK / 4)) = sw;
                }
            }
        }
    }
    if (tp.sig_n) {
        // publish "my rows have landed everywhere": every thread's stores are ordered before the CTA barrier, the
        // system-scope fence of thread 0 after it is cumulative, and the last CTA of the grid writes the flags
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence_system();
            if (atomicAdd(tp.done, 1) == (int)gridDim.x - 1) {
                atomicExch(tp.done, 0);
                __threadfence_system();
                const int val = tp.val_ptr ? *tp.val_ptr : tp.sig_val;
                for (int d = 0; d < tp.sig_n; d++) st_flag_sys(tp.sig_flags[d] + tp.sig_rank, val);
            }
        }
    }
}

// device address of the status word, looked up once per device (a host-side query; cached so that calls under stream
// capture make no runtime query)
static int* quant_status_ptr() {
    static int* cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cache[dev]) {
        int* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, g_quant_status) != cudaSuccess) return nullptr;
        cache[dev] = p;
    }
    return cache[dev];
}

static int norm_quant_launch(const void* x, const void* res, const void* wt, void* hout, void* Bbytes, void* sf_ref, void* sf_atoms,
                             void* g, int tok, int H, float eps, int block, const NormTP& tp, cudaStream_t st) {
    const int nblocks = H / block;
    int threads = (nblocks + 31) / 32 * 32;
    if (threads > 512) threads = 512;
    const int nj = (nblocks + threads - 1) / threads;
    if (nj > 4) return QB_ERR_UNSUPPORTED;     // H <= 32768 (per-16) / 65536 (per-32)
#define QB_LN3(B, NJ, ADD, TL)                                                                                                   \
    norm_quant_kernel<B, NJ, ADD, TL><<<tok, threads, 0, st>>>((const uint4*)x, (const uint4*)res, (const uint4*)wt, (uint4*)hout, \
                                                               (uint32_t*)Bbytes, (uint8_t*)sf_ref, (uint8_t*)sf_atoms, (float*)g, tok, H, eps, tp)
#define QB_LN2(B, NJ) do { if (res) { if (g) QB_LN3(B, NJ, true, true); else QB_LN3(B, NJ, true, false); } \
                           else { if (g) QB_LN3(B, NJ, false, true); else QB_LN3(B, NJ, false, false); } } while (0)
#define QB_LN1(B) do { if (nj <= 1) QB_LN2(B, 1); else if (nj <= 2) QB_LN2(B, 2); else QB_LN2(B, 4); } while (0)
    if (block == 32) QB_LN1(32); else QB_LN1(16);
#undef QB_LN1
#undef QB_LN2
#undef QB_LN3
    return (int)cudaGetLastError();
}

int norm_quant(const void* x, const void* res, const void* wt, void* hout, void* Bbytes, void* sf_ref, void* sf_atoms, void* g,
               int tok, int H, float eps, int block, cudaStream_t st) {
    if (tok < 0 || H <= 0 || H % 128 != 0 || (block != 16 && block != 32)) return QB_ERR_ARG;
    if (tok == 0) return QB_OK;
    if (!x || !wt || !Bbytes || (!sf_ref && !sf_atoms)) return QB_ERR_ARG;
    if (((uintptr_t)x & 15) || ((uintptr_t)res & 15) || ((uintptr_t)wt & 15) || ((uintptr_t)hout & 15) || ((uintptr_t)Bbytes & 3) ||
        ((uintptr_t)sf_ref & 3) || ((uintptr_t)sf_atoms & 3))
        return QB_ERR_ARG;
    NormTP tp{};
    tp.nsrc = 1;
    return norm_quant_launch(x, res, wt, hout, Bbytes, sf_ref, sf_atoms, g, tok, H, eps, block, tp, st);
}

int reduce_norm_quant(const ReduceNormArgs& a, cudaStream_t st) {
    if (a.tok < 0 || a.H <= 0 || a.H % 128 != 0 || (a.block != 16 && a.block != 32)) return QB_ERR_ARG;
    if (a.nsrc < 1 || a.nsrc > 8 || a.fan < 0 || a.fan > 8 || a.sig_n < 0 || a.sig_n > 8) return QB_ERR_ARG;
    if (a.tok == 0) return QB_OK;
    if (!a.src0 || !a.wt) return QB_ERR_ARG;
    if (((uintptr_t)a.src0 & 15) || ((uintptr_t)a.res & 15) || ((uintptr_t)a.wt & 15) || ((uintptr_t)a.hout & 15) || (a.src_stride & 7))
        return QB_ERR_ARG;
    if (a.res && !a.hout) return QB_ERR_ARG;
    if (a.sig_n && !a.done) return QB_ERR_ARG;
    NormTP tp{};
    tp.src_stride = a.src_stride / 8;          // in 16-byte units
    tp.nsrc = a.nsrc;
    tp.wait_flags = a.wait_flags;
    tp.wait_val = a.wait_val;
    tp.fan = a.fan;
    tp.row0 = a.row0;
    tp.tok_total = a.tok_total;
    tp.sig_n = a.sig_n; tp.sig_rank = a.sig_rank; tp.sig_val = a.sig_val; tp.done = a.done; tp.val_ptr = a.val_ptr;
    tp.status = quant_status_ptr();
    if (!tp.status) return QB_ERR_DRIVER;
    void* Bb0 = a.Bbytes[0];
    void* sf0 = a.sf_atoms[0];
    void* g0 = a.g[0];
    if (!Bb0 || !sf0 || !g0) return QB_ERR_ARG;
    for (int d = 0; d < 8; d++) {
        const bool used = d < (a.fan ? a.fan : 1);
        if (used && (!a.Bbytes[d] || !a.sf_atoms[d] || !a.g[d] || ((uintptr_t)a.Bbytes[d] & 15) || ((uintptr_t)a.sf_atoms[d] & 3))) return QB_ERR_ARG;
        tp.Bwords[d] = (uint32_t*)a.Bbytes[d]; tp.sf_atoms[d] = (uint8_t*)a.sf_atoms[d]; tp.g[d] = (float*)a.g[d];
        tp.sig_flags[d] = d < a.sig_n ? a.sig_flags[d] : nullptr;
        if (d < a.sig_n && !a.sig_flags[d]) return QB_ERR_ARG;
    }
    return norm_quant_launch(a.src0, a.res, a.wt, a.hout, Bb0, nullptr, sf0, g0, a.tok, a.H, a.eps, a.block, tp, st);
}

int quant_status_read_clear() {
    int h = 0;
    if (cudaMemcpyFromSymbol(&h, g_quant_status, sizeof(int)) != cudaSuccess) return QB_ERR_DRIVER;
    if (h) { int z = 0; cudaMemcpyToSymbol(g_quant_status, &z, sizeof(int)); }
    return h;
}

// SwiGLU quantisers over feature-major operands gate, up [hidden][batch] (the two halves of a feature-major
// gate/up GEMM output): the compatibility symbols fused_swiglu_quant / fused_swiglu_quant_2lvl
// (cuda/sparse_fp4_lib.cu:794-894) and swiglu_nvfp4 (cuda/dense_nvfp4_fast_lib.cu:258-278).
// grid = (token pairs, scale blocks). A thread owns one scale block of TWO adjacent tokens: every load is one
// 32-bit word holding feature f of both tokens, so a warp reads 128 contiguous bytes per feature row, and the
// block's BLOCK features are walked once with both tokens' running maxima in registers. PASS 0 only records the
// per-token maximum of |h| (two-level, first pass), PASS 1 quantises.
template <bool TWO_LEVEL, int PASS, int BLOCK>
__global__ void __launch_bounds__(128) swiglu_fmajor_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                                             uint32_t* __restrict__ Hwords, uint8_t* __restrict__ scaleH,
                                                             float* __restrict__ tok_amax, int batch, int hidden) {
    constexpr int PER128 = 128 / BLOCK;
    const int t0 = 2 * (blockIdx.x * blockDim.x + threadIdx.x);     // first of this thread's two tokens
    const int sblk = blockIdx.y;                                     // scale block along the hidden axis
    if (t0 >= batch) return;
    const bool pair = t0 + 1 < batch && (batch & 1) == 0;            // word loads need an even row pitch
    const int ntok = (t0 + 1 < batch) ? 2 : 1;
    float hv[2][BLOCK];
    float mx[2] = {0.f, 0.f};
    const size_t row0 = (size_t)sblk * BLOCK;
#pragma unroll
    for (int f = 0; f < BLOCK; f++) {
        const size_t at = (row0 + f) * (size_t)batch + t0;
        float2 g2, u2;
        if (pair) {
            g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + at));
            u2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(up + at));
        } else {
            g2.x = __bfloat162float(gate[at]); u2.x = __bfloat162float(up[at]);
            g2.y = ntok == 2 ? __bfloat162float(gate[at + 1]) : 0.f;
            u2.y = ntok == 2 ? __bfloat162float(up[at + 1]) : 0.f;
        }
        hv[0][f] = swiglu_h<1>(g2.x, u2.x);
        hv[1][f] = swiglu_h<1>(g2.y, u2.y);
        mx[0] = fmaxf(mx[0], fabsf(hv[0][f]));
        mx[1] = fmaxf(mx[1], fabsf(hv[1][f]));
    }
#pragma unroll
    for (int k = 0; k < 2; k++) {
        if (k >= ntok) break;
        const int t = t0 + k;
        if (PASS == 0) {      // |h| >= 0, so the integer order of the bit patterns is the float order
            atomicMax(reinterpret_cast<int*>(tok_amax) + t, __float_as_int(mx[k]));
            continue;
        }
        const float glob = TWO_LEVEL ? fmaxf(__fdiv_rn(tok_amax[t], 2688.f), 1e-30f) : 1.f;
        const float want = __fdiv_rn(mx[k], 6.f);
        const uint32_t code = enc_ue4m3(TWO_LEVEL ? __fdiv_rn(want, glob) : want);
        scaleH[((size_t)(sblk / PER128) * batch + t) * PER128 + (sblk % PER128)] = (uint8_t)code;
        const float dq = TWO_LEVEL ? __fmul_rn(dec_ue4m3(code), glob) : dec_ue4m3(code);
        const Fp4Divider dv(fmaxf(dq, 1e-30f));
        uint32_t* dst = Hwords + (size_t)t * (hidden / 8) + (size_t)sblk * (BLOCK / 8);
#pragma unroll
        for (int w = 0; w < BLOCK / 8; w++) {
            float f8[8];
#pragma unroll
            for (int e = 0; e < 8; e++) f8[e] = hv[k][8 * w + e];
            dst[w] = dv.pack8(f8);
        }
    }
}
__global__ void amax_to_global_kernel(float* tok_amax, int batch) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < batch) tok_amax[t] = fmaxf(__fdiv_rn(tok_amax[t], 2688.f), 1e-30f);
}

template <bool TWO_LEVEL, int PASS, int BLOCK>
static void launch_swiglu_fmajor(const void* g, const void* u, void* Hb, void* scaleH, void* gH, int batch, int hidden, cudaStream_t st) {
    const dim3 grid((unsigned)((batch + 255) / 256), (unsigned)(hidden / BLOCK));
    swiglu_fmajor_kernel<TWO_LEVEL, PASS, BLOCK><<<grid, 128, 0, st>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (uint32_t*)Hb,
                                                                     (uint8_t*)scaleH, (float*)gH, batch, hidden);
}

int swiglu_quant_feature_major(const void* g, const void* u, void* Hb, void* scaleH, void* gH, int batch, int hidden, cudaStream_t st) {
    if (batch < 0 || hidden <= 0 || hidden % 128) return QB_ERR_ARG;
    if (batch == 0) return QB_OK;
    if (!g || !u || !Hb || !scaleH || ((uintptr_t)Hb & 3) || ((uintptr_t)g & 3) || ((uintptr_t)u & 3)) return QB_ERR_ARG;
    if (gH) {
        // two-level: per-token maximum first (gH holds the raw maximum while the second pass reads it), then the codes,
        // then gH becomes the global the GEMM multiplies by
        int rc = (int)cudaMemsetAsync(gH, 0, (size_t)batch * sizeof(float), st);
        if (rc) return rc;
        launch_swiglu_fmajor<true, 0, 32>(g, u, nullptr, nullptr, gH, batch, hidden, st);
        launch_swiglu_fmajor<true, 1, 32>(g, u, Hb, scaleH, gH, batch, hidden, st);
        amax_to_global_kernel<<<(batch + 255) / 256, 256, 0, st>>>((float*)gH, batch);
    } else {
        launch_swiglu_fmajor<false, 1, 32>(g, u, Hb, scaleH, nullptr, batch, hidden, st);
    }
    return (int)cudaGetLastError();
}

// per-16 single-level flavour (swiglu_nvfp4 of the dense library)
int swiglu_quant_feature_major16(const void* g, const void* u, void* Hb, void* scaleH, int batch, int hidden, cudaStream_t st) {
    if (batch < 0 || hidden <= 0 || hidden % 128) return QB_ERR_ARG;
    if (batch == 0) return QB_OK;
    if (!g || !u || !Hb || !scaleH || ((uintptr_t)Hb & 3) || ((uintptr_t)g & 3) || ((uintptr_t)u & 3)) return QB_ERR_ARG;
    launch_swiglu_fmajor<false, 1, 16>(g, u, Hb, scaleH, nullptr, batch, hidden, st);
    return (int)cudaGetLastError();
}

template <int BLOCK, bool TWO_LEVEL>
static int launch_quant(const void* x, void* Bbytes, void* sf_ref, void* sf_atoms, float* g, int tok, int K,
                        cudaStream_t st, const long long* src, int h8, const GatherPeers& peers) {
    const int nblocks = K / BLOCK;
    int threads = (nblocks + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    const int nj = (nblocks + threads - 1) / threads;
    // programmatic dependent launch: the grid may become resident while the kernel in front drains (it waits for that
    // kernel's results with griddepcontrol.wait before its first load), which hides the launch latency between the
    // kernels of a decode step
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(peers.n_rows && tok > 148 * 16 ? 148 * 16 : tok));
    cfg.blockDim = dim3((unsigned)threads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
#define QB_LQ(NJ)                                                                                                          \
    return (int)cudaLaunchKernelEx(&cfg, quant_act_kernel<BLOCK, NJ, TWO_LEVEL>, (const uint4*)x, (uint32_t*)Bbytes, (uint8_t*)sf_ref, \
                                   (uint8_t*)sf_atoms, g, tok, K, src, h8, peers)
    if (nj <= 1) QB_LQ(1);
    else if (nj <= 2) QB_LQ(2);
    else if (nj <= 4) QB_LQ(4);
    else if (nj <= 8) QB_LQ(8);
    return QB_ERR_UNSUPPORTED;
#undef QB_LQ
}

int quantize_act(const void* x, void* Bbytes, void* sf_ref, void* sf_atoms, void* g, int tok, int K, int block,
                 cudaStream_t st) {
    return gather_quantize_act(x, nullptr, Bbytes, sf_ref, sf_atoms, g, tok, K, K, block, st);
}

// src == nullptr: plain quantiser of x [tok][K]. Otherwise output row r = quantised x[src[r]] (x rows of H <= K values,
// zero-padded to K; src[r] < 0 gives a zero row): gather + pad + quantise of routed MoE rows in one pass.
int gather_quantize_act(const void* x, const void* src, void* Bbytes, void* sf_ref, void* sf_atoms, void* g, int tok, int K, int H,
                        int block, cudaStream_t st, const void* const* peer_x, int n_peers, long long rows_per_peer, const void* n_rows_dev) {
    if (tok < 0 || K <= 0 || K % 128 != 0 || (block != 16 && block != 32) || H <= 0 || H > K || H % 8) return QB_ERR_ARG;
    if (tok == 0) return QB_OK;
    if ((!x && !peer_x) || !Bbytes || (!sf_ref && !sf_atoms)) return QB_ERR_ARG;
    if (((uintptr_t)x & 15) || ((uintptr_t)Bbytes & 3) || ((uintptr_t)sf_ref & 3) || ((uintptr_t)sf_atoms & 3) || ((uintptr_t)src & 7)) return QB_ERR_ARG;
    if (K > 65536) return QB_ERR_UNSUPPORTED;
    GatherPeers peers{};
    peers.n_rows = (const int*)n_rows_dev;
    if (peer_x) {
        if (n_peers < 1 || n_peers > 8 || rows_per_peer <= 0 || !src) return QB_ERR_ARG;
        for (int r = 0; r < n_peers; r++) {
            if (!peer_x[r] || ((uintptr_t)peer_x[r] & 15)) return QB_ERR_ARG;
            peers.p[r] = (const uint4*)peer_x[r];
        }
        peers.n = n_peers;
        peers.rows_per = rows_per_peer;
        if (!x) x = peer_x[0];
    }
    const long long* sp = (const long long*)src;
    const int h8 = H >> 3;
    if (block == 32)
        return g ? launch_quant<32, true>(x, Bbytes, sf_ref, sf_atoms, (float*)g, tok, K, st, sp, h8, peers)
                 : launch_quant<32, false>(x, Bbytes, sf_ref, sf_atoms, nullptr, tok, K, st, sp, h8, peers);
    return g ? launch_quant<16, true>(x, Bbytes, sf_ref, sf_atoms, (float*)g, tok, K, st, sp, h8, peers)
             : launch_quant<16, false>(x, Bbytes, sf_ref, sf_atoms, nullptr, tok, K, st, sp, h8, peers);
}

// ---- dispatch of QUANTISED rows: a token row is quantised once (codes [rows][K/2], scales in the step-major layout
// [K/128][rows][4], per-32 blocks, global [rows]) and every routed slot copies its token's packed row: codes as they
// are, scale words into the 128x4 atoms of the routed row, the global. 0.53 bytes per value move instead of 2, and a
// token with top-k slots is quantised once instead of k times. With peers the quantised rows live on n ranks
// (rows_per rows each) and are read with plain peer loads: the dispatch of an expert-parallel layer. The reference's
// plugin gathers bf16 rows with torch indexing and quantises every routed row (harness/qb_vllm_plugin/
// qb_sm120_plugin.py:2430-2441).
struct QuantPeers {
    const uint8_t* codes[8];
    const uint8_t* sf[8];
    const float* g[8];
    long long rows_per;
    int n;
};
__global__ void __launch_bounds__(128) gather_quantized_kernel(const QuantPeers src_q, const long long* __restrict__ src,
                                                               uint8_t* __restrict__ Bbytes, uint8_t* __restrict__ sf_atoms,
                                                               float* __restrict__ g_out, int rows, int K,
                                                               const int* __restrict__ n_rows) {
    const int nrows = n_rows ? min(rows, *n_rows) : rows;
    const int nchunk = K >> 5;               // 16-byte chunks of codes per row (32 values each = one scale block)
    const int nword = K >> 7;                // 4-scale words per row
    const int apr = kpad256(K) / 128;
    for (int row = blockIdx.x; row < nrows; row += gridDim.x) {
        const long long t = src[row];
        uint4* dst = reinterpret_cast<uint4*>(Bbytes + (size_t)row * (K >> 1));
        if (t < 0) {
            if (n_rows) continue;            // rows-in-use mode: padding rows stay unwritten (nobody reads their results)
            for (int c = threadIdx.x; c < nchunk; c += blockDim.x) dst[c] = make_uint4(0, 0, 0, 0);
            for (int w = threadIdx.x; w < nword; w += blockDim.x)
                *reinterpret_cast<uint32_t*>(sf_atoms + sf_atom_offset(row, 4 * w, apr)) = 0u;
            if (threadIdx.x == 0 && g_out) g_out[row] = 1e-30f;
            continue;
        }
        const int owner = (int)(t / src_q.rows_per);
        const long long lt = t - (long long)owner * src_q.rows_per;
        const uint4* cs = reinterpret_cast<const uint4*>(src_q.codes[owner] + (size_t)lt * (K >> 1));
        for (int c = threadIdx.x; c < nchunk; c += blockDim.x) dst[c] = __ldcg(cs + c);
        const uint32_t* ss = reinterpret_cast<const uint32_t*>(src_q.sf[owner]);
        for (int w = threadIdx.x; w < nword; w += blockDim.x)
            *reinterpret_cast<uint32_t*>(sf_atoms + sf_atom_offset(row, 4 * w, apr)) = __ldcg(ss + (size_t)w * src_q.rows_per + lt);
        if (threadIdx.x == 0 && g_out) g_out[row] = __ldcg(src_q.g[owner] + lt);
    }
}

int gather_quantized(const void* const* q_codes, const void* const* q_sf, const void* const* q_g, int n_peers, long long rows_per_peer,
                     const void* src, void* Bbytes, void* sf_atoms, void* g, int rows, int K, const void* n_rows_dev, cudaStream_t st) {
    if (rows < 0 || K <= 0 || K % 128 || n_peers < 1 || n_peers > 8 || rows_per_peer <= 0) return QB_ERR_ARG;
    if (rows == 0) return QB_OK;
    if (!q_codes || !q_sf || !src || !Bbytes || !sf_atoms || (g && !q_g)) return QB_ERR_ARG;
    if (((uintptr_t)Bbytes & 15) || ((uintptr_t)sf_atoms & 3) || ((uintptr_t)src & 7)) return QB_ERR_ARG;
    QuantPeers q{};
    for (int r = 0; r < n_peers; r++) {
        if (!q_codes[r] || !q_sf[r] || (g && !q_g[r]) || ((uintptr_t)q_codes[r] & 15) || ((uintptr_t)q_sf[r] & 3)) return QB_ERR_ARG;
        q.codes[r] = (const uint8_t*)q_codes[r]; q.sf[r] = (const uint8_t*)q_sf[r]; q.g[r] = g ? (const float*)q_g[r] : nullptr;
    }
    q.rows_per = rows_per_peer; q.n = n_peers;
    int grid = rows;
    if (n_rows_dev && grid > 148 * 16) grid = 148 * 16;
    gather_quantized_kernel<<<grid, 128, 0, st>>>(q, (const long long*)src, (uint8_t*)Bbytes, (uint8_t*)sf_atoms, (float*)g, rows, K,
                                                  (const int*)n_rows_dev);
    return (int)cudaGetLastError();
}

// ---- re-layout: reference step-major scales [K/128][rows][P] -> 128x4 atoms
__global__ void sf_ref_to_atoms_kernel(const uint32_t* __restrict__ ref, uint8_t* __restrict__ atoms, int rows, int ksteps,
                                       int P, int atoms_per_rowblock) {
    // one thread per 4-scale word: word index = (step*rows + r)*(P/4) + q
    size_t n = (size_t)ksteps * rows * (P / 4);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        int q = (int)(i % (P / 4));
        size_t t = i / (P / 4);
        int r = (int)(t % rows);
        int s = (int)(t / rows);
        int jcol = s * P + q * 4;
        *reinterpret_cast<uint32_t*>(atoms + sf_atom_offset(r, jcol, atoms_per_rowblock)) = ref[i];
    }
}

int relayout_sf(const void* ref, void* atoms, int rows, int K, int block, cudaStream_t st) {
    if (rows < 0 || K <= 0 || K % 128 || (block != 16 && block != 32)) return QB_ERR_ARG;
    if (rows == 0) return QB_OK;
    if (!ref || !atoms || ((uintptr_t)ref & 3) || ((uintptr_t)atoms & 3)) return QB_ERR_ARG;
    int P = 128 / block;
    size_t n = (size_t)(K / 128) * rows * (P / 4);
    int blocks = (int)((n + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    sf_ref_to_atoms_kernel<<<blocks, 256, 0, st>>>((const uint32_t*)ref, (uint8_t*)atoms, rows, K / 128, P, kpad256(K) / 128 * P / 4);
    return (int)cudaGetLastError();
}

// ---- re-layout: reference metadata [K/128][out][2] i32 -> [out/128][K/256][128][16 B]
__global__ void meta_ref_to_native_kernel(const uint2* __restrict__ ref, uint2* __restrict__ nat, int out_f, int ksteps,
                                          int kblocks) {
    size_t n = (size_t)ksteps * out_f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        int r = (int)(i % out_f);
        int s = (int)(i / out_f);
        size_t dst = (((size_t)(r >> 7) * kblocks + (s >> 1)) * 128 + (r & 127)) * 2 + (s & 1);
        nat[dst] = ref[i];
    }
}

int relayout_meta(const void* ref, void* nat, int out_f, int K, cudaStream_t st) {
    if (out_f <= 0 || K <= 0 || K % 128 || out_f % 128) return QB_ERR_ARG;
    if (!ref || !nat || ((uintptr_t)ref & 7) || ((uintptr_t)nat & 7)) return QB_ERR_ARG;
    size_t n = (size_t)(K / 128) * out_f;
    int blocks = (int)((n + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    meta_ref_to_native_kernel<<<blocks, 256, 0, st>>>((const uint2*)ref, (uint2*)nat, out_f, K / 128, kpad256(K) / 256);
    return (int)cudaGetLastError();
}

}  // namespace qb
