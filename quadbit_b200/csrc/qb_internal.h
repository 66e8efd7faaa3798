// Internal (C++) interfaces between the translation units of the library. The public
// C-ABI is declared in include/quadbit_b200.h and defined in qb_abi.cu.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace qb {

// ---- qb_quant.cu
int quantize_act(const void* x, void* Bbytes, void* sf_ref, void* sf_atoms, void* g, int tok, int K, int block,
                 cudaStream_t st);
// cgu: token-major gate/up GEMM output [tok][2*I] bf16 -> Hb[tok][I/2], per-32 scales, gH[tok]
// peer_x != null: src holds row numbers over n_peers sources of rows_per_peer rows each (peer-mapped pointers)
int gather_quantize_act(const void* x, const void* src, void* Bbytes, void* sf_ref, void* sf_atoms, void* g, int tok, int K, int H,
                        int block, cudaStream_t st, const void* const* peer_x = nullptr, int n_peers = 0, long long rows_per_peer = 0,
                        const void* n_rows_dev = nullptr);
// routed rows copy their token's quantised row (codes, per-32 scales in the step-major layout, global) from n_peers buffers
int gather_quantized(const void* const* q_codes, const void* const* q_sf, const void* const* q_g, int n_peers, long long rows_per_peer,
                     const void* src, void* Bbytes, void* sf_atoms, void* g, int rows, int K, const void* n_rows_dev, cudaStream_t st);
int swiglu_quant(const void* cgu, void* Hb, void* sf_ref, void* sf_atoms, void* gH, int tok, int I, cudaStream_t st);
int swiglu_quant_ex(const void* cgu, void* Hb, void* sf_ref, void* sf_atoms, void* gH, int tok, int I, int interleaved, int act,
                    cudaStream_t st, const void* row_src = nullptr, const void* n_rows_dev = nullptr);
int swiglu_quant_feature_major16(const void* g, const void* u, void* Hb, void* scaleH, int batch, int hidden, cudaStream_t st);
int moe_route_fixed(const void* assign, void* src, void* pos, void* eblk, int n, int e, int r_cap, cudaStream_t st, int div = 1,
                    const void* w_in = nullptr, void* rw = nullptr, void* inverse = nullptr, int e_base = 0, void* n_used = nullptr,
                    int align = 128);
int moe_scatter_add(const void* Cs, const void* eblk, const void* sc_tok, const void* sc_w, const void* bias, void* Out, int rows,
                    int Mpe, int Hout, cudaStream_t st);
// RMSNorm (+ residual add) fused with the quantiser; res / hout / g may be null (g null = single level)
int norm_quant(const void* x, const void* res, const void* wt, void* hout, void* Bbytes, void* sf_ref, void* sf_atoms, void* g,
               int tok, int H, float eps, int block, cudaStream_t st);
// The tensor-parallel form of the fused residual add + RMSNorm + quantiser (two-level only): the norm input is the
// fp32 sum, in source order, of nsrc <= 8 bf16 sources [tok][H] (src0 + i * src_stride elements) plus the residual;
// see NormTP in qb_quant.cu for wait_flags / fan / sig. With fan == 0 the outputs are Bbytes[0] / sf_atoms[0] / g[0]
// for this rank's tok rows; with fan > 0 they are `fan` full gathered arrays and this rank's rows start at row0.
struct ReduceNormArgs {
    const void* src0;
    long long src_stride;      // elements between sources (a multiple of 8)
    int nsrc;
    const void* res;           // residual [tok][H] bf16 or null
    const void* wt;
    void* hout;                // new residual (required with res)
    void* Bbytes[8];
    void* sf_atoms[8];
    void* g[8];
    int fan, row0, tok_total;
    int tok, H, block;
    float eps;
    const int* wait_flags;
    int wait_val;
    int sig_n, sig_rank, sig_val;
    int* sig_flags[8];
    int* done;
    const int* val_ptr;        // non-null: wait_val and sig_val are both read from this device word when the kernel runs
};
int reduce_norm_quant(const ReduceNormArgs& a, cudaStream_t st);
int quant_status_read_clear();
// ---- qb_gemv.cu: quantiser + matrix-vector product for one or two tokens on the dense weight (tiled layout)
int linear_gemv_dense(const void* x, const void* At, const void* sfa, const void* gA, void* C, int out_f, int tok, int K, cudaStream_t st);
// SwiGLU quantiser over feature-major g, u [hidden][batch]; gH null = single level
int swiglu_quant_feature_major(const void* g, const void* u, void* Hb, void* scaleH, void* gH, int batch, int hidden, cudaStream_t st);
int relayout_sf(const void* ref, void* atoms, int rows, int K, int block, cudaStream_t st);
int relayout_meta(const void* ref, void* nat, int out_f, int K, cudaStream_t st);

// ---- qb_compress.cu
// w_dtype: 0 = fp32, 1 = bf16. Any output pointer may be null.
int dequant_fp4_blocks(const void* w, const void* scales, const void* s2, void* out, int out_f, int in_f, int group, long long ld_out,
                       cudaStream_t st);
int compress_2to4(const void* W, int w_dtype, void* Ac, void* meta_ref, void* meta_nat, void* sf_ref, void* sf_atoms,
                  void* gA, int out_f, int K, cudaStream_t st, const void* colnorm = nullptr);
int pack_dense(const void* W, int w_dtype, void* Ab, void* sf_ref, void* sf_atoms, void* gA, int out_f, int K,
               cudaStream_t st);

// Re-lay packed weight rows [rows][K/4 (sparse) or K/2 (dense)] as contiguous 128-row x 256-K tiles
// [rows/128][Kp/256][128][64 or 128 B] (zero beyond K): one tile is one contiguous 8 / 16 KB read.
int tile_weights(const void* A, void* At, int rows, int K, int sparse, cudaStream_t st);

// ---- qb_gemm.cu
struct GemmArgs {
    const void* A;         // packed weights: dense [out][K/2], sparse [out][K/4]
    const void* B;         // packed activations [tok][K/2]
    const void* sfa;       // weight scale atoms
    const void* sfb;       // activation scale atoms
    const void* meta;      // native 2:4 metadata (sparse only)
    const float* gA;       // per-row global scale of A (null = 1)
    const float* gB;       // per-row global scale of B (null = 1)
    void* C;               // output
    float* Cf;             // fp32 split-K workspace [tok][out]; with sk_counters it must be zero on entry and is left zero
    void* sk_counters;     // in-kernel finish: int[4 * tiles], zero before the first call, left zero by the kernel
    int cluster_red;       // set by the decode plan when it costed the split as a cluster reduction (the GEMM itself decides from the shape)
                           // (null = the host zeroes Cf and launches a finish kernel)
    const int* eblk;       // grouped mode: expert of every 128-token block (null = plain GEMM)
    const void* bias;      // epilogue 3: bf16 per-expert bias [E][out_per_expert] (may be null)
    const float* row_w;    // epilogue 3: fp32 per-routed-row weight [tok] (may be null)
    int bias_ld;           // epilogue 3: features per bias row, a bias is [E][bias_ld]; 0 = out_f (features beyond it get no bias)
    int a_rows;            // rows of A (plain: out; grouped: experts * out_per_expert)
    int out_f;             // output features per GEMM (plain: out; grouped: out_per_expert)
    int tok;               // rows of B
    int K;                 // logical reduction length
    int sparse;            // 1 = 2:4-sparse A
    int a_tiled;           // 1 = A is in the tiled layout [rows/128][Kp/256][128][64 or 128 B] (see tile_weights)
    int out_mode;          // 0: bf16 C[out][tok]  1: bf16 C[tok][out]  2: fp32 raw accumulators C[out][tok]
                           // 3: bf16 C[tok][out] = (acc*gA*gB + bias)*row_w
                           // 4: no C; h = SwiGLU(acc*gA*gB + bias) quantised single-level (see h_bytes)
    int splits;            // K splits (>1 uses Cf + a convert pass)
    int bn;                // token tile (0 = choose)
    // Row-parallel GEMM fused with the reduce-scatter of its partial result (prefill pair kernel, out_mode 1 only):
    // with peer_n > 0 the epilogue stores token row t into peer_out[t / tok_per_rank] (a pointer into the memory of
    // the rank that owns that token range, already offset to this rank's slot) at local row t % tok_per_rank, and
    // the last CTA to finish publishes peer_val in flag word `peer_rank` of every rank's flag array. C is unused.
    int peer_n;
    int peer_rank;
    int tok_per_rank;
    int peer_val;
    void* peer_out[8];
    int* peer_flags[8];
    int* peer_done;        // arrival counter of this device's CTAs, zero between calls
    // out_mode 4 (pair kernel): SwiGLU + single-level per-32 quantiser of h in the epilogue; A's rows are (gate, up) pairs
    void* h_bytes;         // packed E2M1 codes of h [tok][h_feats / 2]
    void* h_sf_atoms;      // UE4M3 scale codes of h as 128x4 atoms (may be null if h_sf_ref is given)
    void* h_sf_ref;        // ... and / or in the reference layout [h_feats/128][tok][4]
    int h_feats;           // features of h per row = out_f / 2
    int act;               // 0 = clamped gpt-oss SwiGLU, 1 = silu(g) * u
    const int* peer_val_ptr;   // non-null: the flag value is read from this device word when the kernel runs (graph replay)
};
int gemm_nvfp4(const GemmArgs& a, cudaStream_t st);
int gemm_init_attrs();
// splits / token tile that stream the weight over the SMs with the fewest idle waves (thin token counts)
void decode_plan(int out_f, int tok, int K, int* splits, int* bn, int* cluster = nullptr);
int read_status(cudaStream_t st);   // synchronises st and returns + clears the device status word

// ---- qb_moe.cu
int moe_route(const void* assign, void* poff, void* counter, void* src, int n, int e, cudaStream_t st);
int moe_combine_topk(const void* dbuf, const void* inverse, void* y, int t, int H, int topk, int Mpe, cudaStream_t st);

}  // namespace qb
