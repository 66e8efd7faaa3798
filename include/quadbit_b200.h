/* quadbit_b200 — C-ABI of the B200 (sm_100a) two-level NVFP4 library.
 *
 * Plain pointers and sizes only. Every pointer is a DEVICE pointer unless stated; the
 * caller allocates every input, output and workspace. `stream` is a cudaStream_t passed
 * as void* (0 = legacy default stream). Functions returning int return 0 on success, a
 * cudaError_t (< 1000) or one of the QB_ERR_* codes below.
 *
 * Two groups of entry points:
 *   1. the reference library's own symbols (vitali87/quadbit, cuda/sparse_fp4_lib.cu and
 *      cuda/dense_nvfp4_fast_lib.cu), same names, argument order and tensor layouts, so
 *      the reference's ctypes callers bind unchanged;
 *   2. native `qb_*` entry points that take the tensor-core friendly layouts directly
 *      (no per-call re-layout) and expose the packers that the reference runs in torch.
 *
 * Two shared objects are built from the same sources, as in the reference:
 *   libquadbit_sparse_fp4.so   (reference: sparse_fp4.so)    quantize_act_nvfp4_2lvl is per-32
 *   libquadbit_dense_nvfp4.so  (reference: dense_nvfp4.so)   quantize_act_nvfp4_2lvl is per-16
 *
 * Tensor layouts
 *   reference ("ref") layouts, K = reduction length, ks = K/128:
 *     Ac     [out][K/4]  u8   kept pairs of the 2:4 weight, low nibble = even k
 *     Ab/Bb  [rows][K/2] u8   dense E2M1, low nibble = even k
 *     meta   [ks][out][2] i32 group g of a 128-K step: word g/8, bits 4*(g%8): i0 | i1<<2
 *     scale  [ks][rows][P] u8 UE4M3 codes, P = 4 (one per 32 logical K, sparse path) or
 *                             P = 8 (one per 16 K, dense path)
 *     gA/gB  [rows] f32       per-row global scale
 *   native layouts (Kp = K rounded up to 256; a K tail must be zero filled):
 *     scale atoms [ceil(rows/128)][Kp*P/512][512] u8, byte (r%32)*16 + ((r%128)/32)*4 + c
 *                 for scale column 4*atom + c of row r  (the block-scaled MMA's "128x4" atom)
 *     metadata    [out/128][Kp/256][128][16] u8: per row, the two 8-byte ref words of
 *                 steps 2j and 2j+1
 */
#ifndef QUADBIT_B200_H
#define QUADBIT_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#define QB_OK 0
#define QB_ERR_ARG 1001          /* bad shape, null or misaligned pointer: nothing was launched */
#define QB_ERR_TIMEOUT 1002      /* a bounded device-side wait expired (status = 100200 + site) */
#define QB_ERR_UNSUPPORTED 1003
#define QB_ERR_DRIVER 1004
#define QB_ERR_TOO_LARGE 1005    /* problem exceeds a fixed built-in capacity */

/* ------------------------------------------------------------------ reference symbols */

/* The reference-named GEMM entries below take the reference's tensor layouts and re-lay scale factors / metadata into ONE
 * per-device scratch buffer of the library (grown with cudaMalloc when a larger problem arrives: make the first call of a
 * size outside graph capture). Calls on one device must therefore be stream-ordered with each other: two of them running
 * at once on different streams or threads overwrite each other's re-laid operands. qb_register_weight removes the
 * per-call weight re-layout; the native qb_* entries use no scratch at all.
 * cuda/sparse_fp4_lib.cu:1042 — single-level 2:4-sparse GEMM, C[out][tok] bf16; synchronises. */
int sparse_fp4_mm(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C,
                  int out, int tok, int K);
/* cuda/sparse_fp4_lib.cu:1110 — two-level: C[out][tok] = gA[out]*gB[tok]*sum; synchronises. */
int sparse_fp4_mm_2lvl(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C,
                       int out, int tok, int K, const void* gA, const void* gB);
/* cuda/sparse_fp4_lib.cu:1117 — same, token-major output C[tok][out]; synchronises. */
int sparse_fp4_mm_2lvl_t(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C,
                         int out, int tok, int K, const void* gA, const void* gB);
/* cuda/sparse_fp4_lib.cu:733 (sparse lib: per-32) / cuda/dense_nvfp4_fast_lib.cu:203 (`...b`, per-16):
 * single-level activation quantiser, bf16 x[tok][K] -> Bbytes, scaleB (ref layout). */
void quantize_act_nvfp4(const void* x, void* Bbytes, void* scaleB, int tok, int K);
void quantize_act_nvfp4b(const void* x, void* Bbytes, void* scaleB, int tok, int K);
/* cuda/sparse_fp4_lib.cu:774 (per-32) and cuda/dense_nvfp4_fast_lib.cu:338 (per-16, same name in the
 * dense library): two-level activation quantiser, also writes gB[tok]. */
void quantize_act_nvfp4_2lvl(const void* x, void* Bbytes, void* scaleB, void* gB, int tok, int K);
/* cuda/sparse_fp4_lib.cu:781 — stream variant. */
void quantize_act_nvfp4_2lvl_s(const void* x, void* Bbytes, void* scaleB, void* gB, int tok, int K, void* stream);
/* cuda/sparse_fp4_lib.cu:821,886 — SwiGLU + per-32 quantiser over the reference's feature-major GEMM
 * outputs g, u [hidden][batch] bf16: h = silu(g)*u -> Hbytes[batch][hidden/2], scaleH[hidden/128][batch][4]
 * (single level), and gH[batch] for the two-level form (gH need not be pre-zeroed here). */
void fused_swiglu_quant(const void* g, const void* u, void* Hbytes, void* scaleH, int batch, int hidden);
void fused_swiglu_quant_2lvl(const void* g, const void* u, void* Hbytes, void* scaleH, void* gH, int batch, int hidden);
/* cuda/sparse_fp4_lib.cu:944,1003 — RMSNorm (after an optional residual add whose sum is written to hout
 * as the new residual stream) fused with the single-level per-32 quantiser; x, res, wt, hout bf16. */
void rmsnorm_quant(const void* x, const void* wt, void* Bbytes, void* scaleB, int batch, int hidden, float eps);
void add_rmsnorm_quant(const void* inp, const void* res, const void* wt, void* hout, void* Bbytes, void* scaleB, int batch,
                       int hidden, float eps);
/* cuda/dense_nvfp4_fast_lib.cu:251,274 — the dense library's glue, per-16 single-level (SFB [hidden/128][batch][8]):
 * RMSNorm after an optional residual add (res may be null; with res the sum is written to hout), and SwiGLU over
 * feature-major g, u [hidden][batch]. */
void rmsnorm_nvfp4(const void* x, const void* res, const void* wt, void* hout, void* Bbytes, void* SFB, int batch, int hidden,
                   float eps);
void swiglu_nvfp4(const void* g, const void* u, void* Hbytes, void* SFB, int batch, int hidden);
/* cuda/sparse_fp4_lib.cu:1133-1137 — fused SwiGLU MLP: quantise x[tp][H], gate/up GEMM (weights gu_*,
 * gu_out = 2*Iw rows: gate features then up features), h = silu(g)*u quantised two-level per token,
 * down GEMM -> Cout[tp][dn_out] bf16. Bb, sBg, gBg, Cgu, Hb, sH, gH are caller scratch with the
 * reference's sizes (Cgu holds gu_out*tp bf16; here it is written token-major, sBg / sH are unused).
 * Runs on `stream`, never synchronises. */
int fused_mlp_2lvl(const void* x, const void* gu_Ac, const void* gu_scaleA, const void* gu_meta, const void* gu_gA,
                   const void* dn_Ac, const void* dn_scaleA, const void* dn_meta, const void* dn_gA, void* Bb, void* sBg, void* gBg,
                   void* Cgu, void* Hb, void* sH, void* gH, void* Cout, int tp, int H, int Iw, int gu_out, int dn_out,
                   void* stream);
/* cuda/sparse_fp4_lib.cu:1892-1896 — same with a split-K down projection (Cf: fp32 workspace [tp][dn_out]). */
int fused_mlp_2lvl_skdown(const void* x, const void* gu_Ac, const void* gu_scaleA, const void* gu_meta, const void* gu_gA,
                          const void* dn_Ac, const void* dn_scaleA, const void* dn_meta, const void* dn_gA, void* Bb, void* sBg,
                          void* gBg, void* Cgu, void* Hb, void* sH, void* gH, void* Cout, void* Cf, int tp, int H, int Iw,
                          int gu_out, int dn_out, int splits, void* stream);
/* cuda/sparse_fp4_lib.cu:1347 — split-K 2:4-sparse GEMM for decode; Cf = fp32 workspace [tok][out];
 * output token-major C[tok][out]; synchronises. */
int sparse_down_sk_2lvl(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta,
                        void* Cout, void* Cf, int out, int tok, int K, const void* gA, const void* gB, int splits);
/* cuda/sparse_fp4_lib.cu:1640 — segmented MoE GEMM over routed rows sorted by expert; eblk[rows/128]
 * is the expert of each 128-row block; outT 0: C[Mpe][rows], 1: C[rows][Mpe]. Synchronises iff stream==0. */
int sparse_moe_mm_2lvl(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C,
                       int Mtot, int Mpe, int rows, int K, const void* gA, const void* gB, const void* eblk, int outT,
                       void* stream);
/* cuda/sparse_fp4_lib.cu:1661 — same with epilogue C[rows][Mpe] = (acc + bias[expert][f]) * sc_w[row]
 * (bias bf16 [E][Hout], may be null). */
int sparse_moe_mm_2lvl_bw(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C,
                          int Mtot, int Mpe, int rows, int K, const void* gA, const void* gB, const void* eblk,
                          const void* sc_w, const void* bias, int Hout, void* stream);
/* cuda/sparse_fp4_lib.cu:1649 — fused down GEMM: Out[sc_tok[r]][f] += (acc + bias[expert][f]) * sc_w[r] for routed rows
 * with sc_tok[r] >= 0 and f < Hout; Out fp32 [tokens][Hout], zeroed by the caller; bias bf16 [E][Hout] (may be null).
 * The bf16 GEMM tile the reference stages in shared memory is staged in the library's scratch buffer. */
int sparse_moe_mm_2lvl_scatter(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, int Mtot,
                               int Mpe, int rows, int K, const void* gA, const void* gB, const void* eblk, const void* sc_tok,
                               const void* sc_w, const void* bias, void* Out, int Hout, void* stream);
/* cuda/sparse_fp4_lib.cu:1875 — fused GEMM1: grouped gate_up GEMM over pairwise-interleaved (gate, up) weight rows
 * (Mpe = 2*Ih rows per expert), + guBias bf16 [E][Mpe] (may be null), SwiGLU (act 0: clamped gpt-oss form, 1: plain),
 * single-level per-32 quantiser -> Hwords[rows][Ih/2 bytes], scaleH[Ih/128][rows][4] (the down GEMM then runs with
 * gB = 1). Ih % 128 == 0. The bf16 gate_up rows are staged in the library's scratch buffer. */
int sparse_moe_gu_swiglu(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, int Mtot, int Mpe,
                         int rows, int K, const void* gA, const void* gB, const void* eblk, const void* guBias, void* Hwords,
                         void* scaleH, int Ih, int act, void* stream);
/* cuda/sparse_fp4_lib.cu:1606 — counting-sort routing: src[poff[e]+slot] = i (poff int64, src pre-filled -1). */
int moe_route(const void* assign, const void* poff, void* counter, void* src, int N, int E, void* stream);
/* cuda/sparse_fp4_lib.cu:1615 — y[t][f] = sum_k dbuf[inverse[t][k]][f], bf16. */
int moe_combine_topk(const void* dbuf, const void* inverse, void* y, int t, int H, int topk, int Mpe, void* stream);
/* cuda/sparse_fp4_lib.cu:1028,1325,1570,1871 — one-time kernel attribute set-up (call before graph capture). */
void qb_init_func_attrs(void);
void qb_init_sk_attrs(void);
void qb_init_moe_attrs(void);
void qb_init_gusw_attrs(void);
/* cuda/dense_nvfp4_fast_lib.cu:289 — dense two-level GEMM, per-16 scales SFA/SFB [K/128][rows][8]; synchronises. */
int dense_nvfp4_mm(const void* A, const void* B, const void* SFA, const void* SFB, void* C, int out, int tok, int K,
                   const void* gA, const void* gB);

/* ------------------------------------------------------------------ native entry points */

/* Activation quantiser. block = 32 (sparse path) or 16 (dense path). g == NULL selects the
 * single-level recipe. sf_ref and/or sf_atoms receive the scales (either may be NULL). */
int qb_quantize_act(const void* x, void* Bbytes, void* sf_ref, void* sf_atoms, void* g, int tok, int K, int block,
                    void* stream);
/* Fixed-capacity MoE routing in one launch (the reference builds it with torch ops: route_fixed_cap,
 * harness/qb_vllm_plugin/qb_sm120_plugin.py:1271-1315): assign int64 [n] expert id of every routed slot (outside [0, e):
 * not routed), r_cap >= n + 127*e and a multiple of 128. Writes src int64 [r_cap] (slot of every padded row, -1 =
 * padding), pos int64 [n] (padded row of every slot, or -1) and eblk int32 [r_cap/128] (expert of every 128-row block,
 * -1 = unused capacity, which qb_gemm skips). Expert segments are padded to 128 rows and packed in expert order; the
 * row order inside a segment is not deterministic. No host read, graph-capturable. */
int qb_moe_route_fixed(const void* assign, void* src, void* pos, void* eblk, int n, int e, int r_cap, void* stream);
/* Same, with the per-row bookkeeping of a top-k layer done in the same launch: src holds slot / div (div = top-k gives the
 * token row of every padded row), rw fp32 [r_cap] = w_in[slot] for routed rows and 0 for padding (w_in fp32 [n], both or
 * neither), inverse int32 [n] = pos as moe_combine_topk reads it (may be NULL). */
int qb_moe_route_fixed_ex(const void* assign, void* src, void* pos, void* eblk, int n, int e, int r_cap, int div, const void* w_in,
                          void* rw, void* inverse, void* stream);
/* The gather of routed MoE rows fused into their quantiser (the reference gathers with torch indexing and then
 * calls quantize_act_nvfp4_2lvl, harness/fused_moe.py:437-442, harness/qb_vllm_plugin/qb_sm120_plugin.py:2430-2441):
 * output row r = quantised x[src[r]], x bf16 [.][H] zero-padded to K (H % 8 == 0, H <= K), src int64 [rows],
 * src[r] < 0 = an all-zero padding row. src == NULL is qb_quantize_act. */
int qb_gather_quantize_act(const void* x, const void* src, void* Bbytes, void* sf_ref, void* sf_atoms, void* g, int rows, int K,
                           int H, int block, void* stream);
/* Offline 2:4 compressor (torch packer of harness/verify_sparse_2lvl.py:108-122 as one kernel).
 * w_dtype 0 = fp32, 1 = bf16. Any output may be NULL. */
int qb_compress_2to4(const void* W, int w_dtype, void* Ac, void* meta_ref, void* meta_native, void* sf_ref,
                     void* sf_atoms, void* gA, int out, int K, void* stream);
/* Checkpoint block formats -> bf16 [out][ld_out] rows (ld_out >= in, so the result can be written into a zero-padded
 * buffer) for the compressor: group 32 = gpt-oss MXFP4 (w [out][in/2] E2M1 codes, low nibble = even column; scales
 * [out][in/32] e8m0; _mxfp4_dequant, harness/qb_vllm_plugin/qb_sm120_plugin.py:2089-2100), group 16 = modelopt NVFP4
 * (scales [out][in/16] e4m3fn bytes, tensor_scale a device fp32 scalar or NULL; _dequant_nvfp4_expert, :70-95). */
int qb_dequant_fp4_blocks(const void* w, const void* scales, const void* tensor_scale, void* out, int out_f, int in_f, int group,
                          long long ld_out, void* stream);
/* Same with activation-aware pair selection: colnorm fp32 [K] (column norms of calibration activations, Wanda)
 * makes the importance of a pair |w0|*c0 + |w1|*c1 (pack(w, colnorm), harness/qb_vllm_plugin/qb_sm120_plugin.py:
 * 1179-1190). colnorm == NULL is qb_compress_2to4; the reference's fallback to the magnitude for an all-zero
 * colnorm is the caller's to take (pass NULL). */
int qb_compress_2to4_colnorm(const void* W, int w_dtype, const void* colnorm, void* Ac, void* meta_ref, void* meta_native,
                             void* sf_ref, void* sf_atoms, void* gA, int out, int K, void* stream);
/* Dense two-level packer (harness/dense_e2e.py:79-88 as one kernel). */
int qb_pack_dense(const void* W, int w_dtype, void* Ab, void* sf_ref, void* sf_atoms, void* gA, int out, int K,
                  void* stream);
/* ref -> native re-layouts. */
int qb_relayout_sf(const void* sf_ref, void* sf_atoms, int rows, int K, int block, void* stream);
int qb_relayout_meta(const void* meta_ref, void* meta_native, int out, int K, void* stream);
/* Sizes in bytes of the native arrays. */
long long qb_sf_atoms_bytes(int rows, int K, int block);
long long qb_meta_native_bytes(int out, int K);
/* The GEMM on native layouts. a_rows = rows of A (out, or experts*out for grouped mode with
 * eblk != NULL); out_mode 0: bf16 C[out][tok], 1: bf16 C[tok][out], 2: fp32 raw accumulators
 * C[out][tok] (globals ignored), 3: bf16 C[tok][out] = (acc*gA*gB + bias[expert][f]) * row_w[t].
 * splits > 1 splits K across CTAs through the fp32 workspace Cf[tok][out]. bn = token tile
 * (16..256, 0 = auto). In grouped mode the tile is 128 tokens, or 256 with bn = 256 when every expert's rows are padded to
 * 256 (tok % 256 == 0; the two eblk entries of a tile are equal). In grouped mode eblk[b] is the expert of token block b (128 rows); a negative entry marks
 * an unused block of a fixed-capacity routing: it is skipped and its output rows are left unwritten.
 * Asynchronous on `stream`; qb_status() reports device-side errors. */
int qb_gemm(const void* A, const void* B, const void* sfa, const void* sfb, const void* meta_native, const void* gA,
            const void* gB, void* C, void* Cf, const void* eblk, const void* bias, const void* row_w, int a_rows, int out,
            int tok, int K, int sparse, int out_mode, int splits, int bn, void* stream);
/* Tiled weight layout (no reference counterpart: the reference keeps packed weight rows row-major).
 * Re-lays A[rows][K/4 (sparse) or K/2 (dense)] as contiguous 128-row x 256-K tiles
 * [rows/128][ceil(K/256)][128][64 or 128 B], zero beyond K, so that one pipeline stage of the GEMM is one
 * contiguous 8 / 16 KB read (weight streaming at thin token counts otherwise reads 128-byte pieces at a
 * stride of a whole row). qb_gemm / qb_gemm_decode take the tiled array as A when bit 1 of `sparse` is set
 * (sparse = 2: dense tiled, 3: 2:4-sparse tiled). rows % 128 == 0, K % 128 == 0, 16-byte aligned pointers. */
int qb_tile_weights(const void* A, void* A_tiled, int rows, int K, int sparse, void* stream);
long long qb_tiled_weight_bytes(int rows, int K, int sparse);
/* Thin-token (decode) GEMM: streams the weight once with the K range split over CTAs so that all SMs
 * pull from HBM; each split adds its fp32 partial sums into `ws` (reductions at the L2) and the last
 * split to arrive for a tile reads the sums, writes bf16 and zeroes what it read (one launch: no
 * memset, no finish pass; the summation order, hence the last bits, can differ from run to run). Where
 * every (tile, split) pair fits the GPU at once as clusters of <= 8 CTAs, the splits of a tile run as one
 * thread-block cluster instead and their partial tiles meet in distributed shared memory: no workspace
 * traffic, no atomics, sums in split order (bit-reproducible). The split count, the form of the finish and
 * the token tile come from the shapes. `ws`: qb_gemm_decode_ws_bytes(out, tok, K) bytes,
 * 256-byte aligned, ZERO-FILLED ONCE when allocated (arrival counters and sums, all of which every call
 * leaves at zero again); calls sharing a workspace must not overlap on the GPU. out_mode 0 / 1 as in
 * qb_gemm. Replaces the memset + atomics + convert sequence of the reference's split-K decode path
 * (cuda/sparse_fp4_lib.cu:1160-1344) and its unit-scale split-N decode (cuda/dense_decode_lib.cu:19-141). */
int qb_gemm_decode(const void* A, const void* B, const void* sfa, const void* sfb, const void* meta_native, const void* gA,
                   const void* gB, void* C, void* ws, int out, int tok, int K, int sparse, int out_mode, void* stream);
long long qb_gemm_decode_ws_bytes(int out, int tok, int K);
/* One- or two-token linear layer on the dense two-level NVFP4 weight in ONE launch: the activation quantiser
 * (quantize_act_nvfp4_2lvl, per 16, bit-identical codes and scales) and the matrix-vector product, on the CUDA cores: f16
 * products and block sums of E2M1 code values are exact, block sums are scaled and accumulated in fp32 in a fixed order.
 * Counterpart of the reference's dense decode GEMV (cuda/dense_decode_lib.cu:19-141), which also runs beside its
 * tensor-core kernels for single tokens. x [tok][K] bf16 (tok <= 2, 16-byte aligned like A_tiled and sfa), A_tiled / sfa / gA: the weight as qb_pack_dense +
 * qb_tile_weights leave it, C [tok][out] bf16. out % 128 == 0, K % 128 == 0, K <= 16384; no workspace. */
int qb_linear_gemv(const void* x, const void* A_tiled, const void* sfa, const void* gA, void* C, int out, int tok, int K, void* stream);
/* Split-K GEMM without a caller workspace (no counterpart in the reference library, whose
 * split-K entry sparse_down_sk_2lvl always takes the workspace Cf from the caller). Same
 * operands and meaning as qb_gemm with splits > 1, out_mode 0 or 1, plain (not grouped) mode
 * (`sparse` carries the same two bits: bit 0 = 2:4-sparse A, bit 1 = A in the tiled layout);
 * the fp32 partial sums go to an 8 MiB array built into the library instead of a Cf argument.
 * It exists for callers that cannot allocate: an engine whose memory pool already owns the
 * whole GPU, code inside CUDA-graph capture, a hook that only receives inputs and outputs.
 *   - out * tok must not exceed qb_gemm_splitk_static_max_elems() (2 Mi): otherwise
 *     QB_ERR_TOO_LARGE is returned and nothing is launched.
 *   - The first call on each device looks up the array's device address (a host-side query,
 *     no allocation); make that first call before any stream capture begins.
 *   - All calls on a device share the one array. It is zeroed on `stream` at the start of
 *     each call and holds the last call's partial sums afterwards; two calls whose kernels
 *     overlap on the GPU (different streams, or replays of two graphs at once) race on it.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine. */
int qb_gemm_splitk_static(const void* A, const void* B, const void* sfa, const void* sfb, const void* meta_native,
                          const void* gA, const void* gB, void* C, int out, int tok, int K, int sparse, int out_mode,
                          int splits, void* stream);
long long qb_gemm_splitk_static_max_elems(void);
/* RMSNorm [+ residual add] + quantiser, general form: res / hout may be NULL (no add), g NULL selects the
 * single-level recipe, block 16 or 32, scales to the reference layout and/or atoms. */
int qb_norm_quant(const void* x, const void* res, const void* wt, void* hout, void* Bbytes, void* sf_ref, void* sf_atoms, void* g,
                  int tok, int H, float eps, int block, void* stream);
/* SwiGLU + two-level per-32 quantiser over a token-major gate/up output Cgu[tok][2*I] bf16 (gate
 * features first): Hb[tok][I/2], scales (ref layout and/or atoms), gH[tok]. One pass; replaces
 * swiglu_amax + swiglu_finalize + swiglu_quant_g (cuda/sparse_fp4_lib.cu:837-894). */
int qb_swiglu_quant(const void* cgu, void* Hb, void* sf_ref, void* sf_atoms, void* gH, int tok, int I, void* stream);
/* Same with the row layout and the activation as arguments: interleaved = 1 reads (gate, up) pairs
 * [g0,u0,g1,u1,...] (gpt-oss fused gate_up), act 0 = clamped gpt-oss SwiGLU (alpha 1.702, limit 7, up + 1;
 * harness/fused_moe.py:450-452), 1 = silu(g)*u; gH == NULL selects the single-level quantiser of the reference's
 * fused GEMM1 epilogue (cuda/sparse_fp4_lib.cu:1828-1866). row_src (int64 [tok], may be NULL): rows with row_src < 0
 * are padding of a routed batch, their input is not read and they quantise as all-zero rows. */
int qb_swiglu_quant_act(const void* cgu, void* Hb, void* sf_ref, void* sf_atoms, void* gH, const void* row_src, const void* n_rows_dev,
                        int tok, int I, int interleaved, int act, void* stream);
/* fused_mlp_2lvl on native layouts (weights from qb_compress_2to4; sfb_x / sfb_h are scale-atom
 * scratch of qb_sf_atoms_bytes(tok, H | I, 32) bytes; Cf may be NULL or an fp32 [tok][dn_out]
 * workspace for a split-K down projection; flags bit 0: gu_A / dn_A are in the tiled layout of
 * qb_tile_weights). Four launches, no synchronisation, no allocation. */
int qb_fused_mlp(const void* x, const void* gu_A, const void* gu_sfa, const void* gu_meta, const void* gu_gA, const void* dn_A,
                 const void* dn_sfa, const void* dn_meta, const void* dn_gA, void* Bb, void* sfb_x, void* gBx, void* Cgu, void* Hb,
                 void* sfb_h, void* gH, void* Cout, void* Cf, int tok, int H, int I, int gu_out, int dn_out, int splits, int flags,
                 void* stream);
/* Issue-only throughput probe of the block-scaled FP4 MMA (analogue of the reference's
 * cuda/mma_peak.cu): every SM runs `kblocks` K blocks of 256 (dense: 4 MMAs of 128xbnx64,
 * sparse: 2 of 128xbnx128) on operands resident in shared memory. mode bits: 0 issue the MMAs (the pair form
 * always does); 1 the per-block scale-factor / metadata tcgen05.cp copies (one-CTA form); 2 one commit per K block;
 * 3 a tcgen05 fence per block (one-CTA form) or a wait for every block's completion (pair form); 4 the CTA-pair form
 * (cta_group::2, M = 256); 5 the sparse A tile in 128-byte rows with the 128-byte swizzle instead of 64-byte rows;
 * 6 a second warp streams 24 KB per K block from global memory into spare shared memory meanwhile.
 * cycles_per_sm: optional u64[SM count] of SM clock cycles of the MMA loop (u64[2 x SM count] with bit 6: the second
 * half receives the cycles of the streaming loop); status_word: i32, non-zero if a bounded wait expired.
 * bn = 64, 128 or 256. Time it with events around the call. */
int qb_mma_peak(int sparse, int bn, int kblocks, int mode, void* cycles_per_sm, void* status_word, void* stream);
/* Gate/up GEMM with SwiGLU + single-level per-32 quantiser in its epilogue, native layouts (what sparse_moe_gu_swiglu,
 * cuda/sparse_fp4_lib.cu:1679-1875, does on the reference's layouts): operands as qb_gemm, A's rows are (gate, up) pairs
 * (row 2i = gate feature i, row 2i + 1 = up feature i, `out` rows per expert), optional grouped mode (eblk, a_rows = experts
 * * out) and bf16 bias [experts][out] added before the activation. h = act(gate, up) is formed from the fp32 accumulators
 * and quantised with one UE4M3 scale per 32 features (no global): Hb[tok][out/4] packed codes, scale codes as 128x4 atoms
 * (sf_atoms) and / or [out/256][tok][4] (sf_ref). act 0: clamped gpt-oss SwiGLU, 1: silu(g) * u. out % 256 == 0,
 * tok >= 128 (grouped: tok % 128 == 0). */
int qb_gemm_swiglu(const void* A, const void* B, const void* sfa, const void* sfb, const void* meta_native, const void* gA, const void* gB,
                   const void* eblk, const void* bias, void* Hb, void* sf_atoms, void* sf_ref, int a_rows, int out, int tok, int K,
                   int sparse, int act, void* stream);
/* ---- unit-scale FP4 entries of the reference's kernel-only benchmark libraries: C[M,N] bf16 = A[M,K] @ B[N,K]^T on raw
 * E2M1 codes (two per byte, low nibble = even k), every block scale 1.0. N % 128 == 0, K % 128 == 0, any M.
 * cuda/dense_fp4_lib.cu:125, cuda/dense_sk_lib.cu:147 (Cf: fp32 [M*N] workspace, used when splits > 1),
 * cuda/dense_decode_lib.cu:116-168 (qb_encode_map returns a host handle for one operand, freed by qb_free_map; the
 * _cached entries take two of them; _async does not synchronise and reports through qb_last_error),
 * cuda/sparse_sk_lib.cu:199 (single-level 2:4-sparse split-K on reference layouts, C[M][N], A = the sparse weight). */
int dense_fp4_mm(const void* A, const void* B, void* C, int M, int N, int K);
int dense_fp4_mm_sk(const void* A, const void* B, void* C, void* Cf, int M, int N, int K, int splits);
int qb_decode_tn(int N);
int dense_fp4_decode(const void* A, const void* B, void* C, int M, int N, int K);
void* qb_encode_map(const void* ptr, int rows, int K, int boxrows);
void qb_free_map(void* m);
int dense_fp4_decode_cached(const void* mapA, const void* mapB, void* C, int M, int N, int K);
void dense_fp4_decode_cached_async(const void* mapA, const void* mapB, void* C, int M, int N, int K);
int sparse_fp4_mm_sk(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C, void* Cf, int M,
                     int N, int Klog, int splits);
/* Register a weight's reference-layout scale factors [K/128][rows][4 or 8] (and metadata [K/128][rows][2] i32 when sparse):
 * the layouts the tensor-core kernels read are made once and every later call of a reference-named GEMM entry with the
 * same pointers uses them instead of re-laying the weight (the reference consumes its layouts as they are,
 * cuda/sparse_fp4_lib.cu:1029-1046, so its callers pay no such step). Two device allocations per weight, made here and
 * kept until qb_forget_weight(scaleA); the registered arrays must not change meanwhile. Unregistered weights keep
 * working (re-laid per call). */
int qb_register_weight(const void* scaleA, const void* meta, int rows, int K, int sparse, void* stream);
int qb_forget_weight(const void* scaleA);
/* ---- tensor parallelism over one NVSwitch box (one process per GPU). No counterpart in the reference library: its
 * one distributed script computes, then calls all_reduce (harness/moe_dist.py:123,161-167).
 * Peer buffers: qb_peer_alloc = cudaMalloc + zero fill (set-up time only); qb_peer_export writes the 64-byte CUDA IPC
 * handle of an allocation, which another process of the same box turns into a pointer with qb_peer_open (close with
 * qb_peer_close before the owner frees). Only plain loads / stores and system-scope flag words touch peer memory. */
int qb_peer_alloc(void** ptr, long long bytes);
int qb_peer_free(void* ptr);
int qb_peer_export(void* ptr, void* handle64);
int qb_peer_open(const void* handle64, void** ptr);
int qb_peer_close(void* ptr);
/* One-thread kernels on `stream`: signal writes `value` into word my_rank of each of the n flag arrays (after a
 * system-scope fence; stream order puts it after the kernels it announces); wait returns when all n words of `flags`
 * are >= value (or >= *value_ptr when that is not NULL; signal takes its value the same way), or after 20 s with a status
 * code (qb_peer_status). */
int qb_peer_signal(void* const* flag_arrays, int n, int my_rank, int value, const void* value_ptr, void* stream);
int qb_peer_wait(const void* flags, int n, int value, const void* value_ptr, void* stream);
/* *epoch += delta by one thread on `stream`. The entries here that take a `value_ptr` read their flag value(s) from that
 * device word when the kernel runs instead of from the argument, so a captured CUDA graph can be replayed: every replay
 * first bumps the word, on every rank. */
int qb_epoch_add(void* epoch, int delta, void* stream);
int qb_peer_status(void* stream);
/* ---- expert parallelism by peer loads (no counterpart in the reference library; its script all-reduces partial outputs,
 * harness/moe_dist.py:161-167, its plugin dispatches with torch indexing, harness/qb_vllm_plugin/qb_sm120_plugin.py:2430-2441).
 * qb_ep_publish: copy this rank's token rows x (x_bytes, 16-byte multiple) into its peer-visible buffer x_pub and store its
 *   routing (idx i64, w f32, n_slots entries) into the replicated tables assign_all[r] / w_all[r] of every rank at slot0; the
 *   last CTA writes *value_ptr into word `rank` of every flags[r] (done_counter: one int, zero between calls).
 * qb_moe_route_fixed_range: qb_moe_route_fixed_ex for a rank that owns experts [e_base, e_base + e) of a global id space;
 *   align = 128 or 256: rows every expert's segment is padded to (r_cap % align == 0, r_cap >= n + e * (align - 1)). With 256 the
 *   grouped GEMM can be asked for 256-token tiles (qb_gemm with eblk and bn = 256: eblk keeps one entry per 128 rows).
 * qb_gather_quantize_act_peer: qb_gather_quantize_act whose source rows are numbered over n_peers buffers of rows_per_peer
 *   rows each (pointers into the ranks' x_pub): the dispatch is done by the loads of the quantiser. n_used (route) / n_rows_dev
 *   (quantisers; may be NULL): one device int = padded rows in use; rows beyond it are unused capacity and are not touched.
 * qb_ep_combine: y[t][f] = sum_k d_owner[inverse_owner[(t0 + t) * topk + k]][f] for this rank's t_local tokens, the rows read
 *   from the rank that owns the slot's expert (owner = idx / experts_per_rank; dbuf[r], inverse[r]: peer pointers). */
int qb_ep_publish(const void* x, void* x_pub, long long x_bytes, const void* idx, const void* w, int n_slots, int slot0,
                  void* const* assign_all, void* const* w_all, int world, int rank, void* const* flags, const void* value_ptr,
                  void* done_counter, void* stream);
int qb_moe_route_fixed_range(const void* assign, void* src, void* pos, void* eblk, int n, int e_base, int e, int r_cap, int div,
                             int align, const void* w_in, void* rw, void* inverse, void* n_used, void* stream);
/* Dispatch of quantised rows. qb_quantize_rows: x[rows][H] bf16 (H % 8 == 0, zero-padded to K) -> codes Bbytes[rows][K/2], scales in
 * the step-major layout sf_ref[K/128][rows][128/block], g[rows] (NULL = single level): each token quantised once.
 * qb_gather_quantized: routed row r copies the quantised row of token src[r] (numbered over n_peers buffers of rows_per_peer rows,
 * per-32 scales) into Bbytes[r], the 128x4 scale atoms of row r and g[r]; src[r] < 0 is a padding row (zeros, or left unwritten
 * when n_rows_dev, the device count of rows in use, is given). Replaces gather + quantise of every routed row
 * (harness/qb_vllm_plugin/qb_sm120_plugin.py:2430-2441): a token with top-k slots is quantised once, and over NVLink 0.53 bytes
 * per value move instead of 2. */
int qb_quantize_rows(const void* x, void* Bbytes, void* sf_ref, void* g, int rows, int K, int H, int block, void* stream);
int qb_gather_quantized(void* const* q_codes, void* const* q_sf, void* const* q_g, int n_peers, long long rows_per_peer, const void* src,
                        void* Bbytes, void* sf_atoms, void* g, int rows, int K, const void* n_rows_dev, void* stream);
int qb_gather_quantize_act_peer(void* const* x_peers, int n_peers, long long rows_per_peer, const void* src, void* Bbytes, void* sf_atoms,
                                void* g, int rows, int K, int H, int block, const void* n_rows_dev, void* stream);
int qb_ep_combine(void* const* dbuf, void* const* inverse, const void* idx, void* y, int t_local, int t0, int H, int topk, int Mpe,
                  int experts_per_rank, int world, void* stream);
/* Row-parallel GEMM fused with the reduce-scatter of its partial result (replaces "GEMM, then all_reduce"): operands as
 * qb_gemm (this rank's K slice), token-major bf16 output; token row t is stored by the epilogue into
 * peer_out[t / tok_per_rank] + (t % tok_per_rank) * out (a pointer into the owner's memory, already offset to this rank's
 * slot), and the last CTA to finish writes flag_value into word `rank` of every peer_flags[r]. done_counter: one int on
 * this device, zero between calls. Prefill sizes only: out % 256 == 0, tok >= 128, tok_per_rank % 16 == 0. */
int qb_gemm_rs(const void* A, const void* B, const void* sfa, const void* sfb, const void* meta_native, const void* gA, const void* gB,
               void* const* peer_out, void* const* peer_flags, void* done_counter, int out, int tok, int K, int sparse, int n_ranks,
               int rank, int tok_per_rank, int flag_value, const void* value_ptr, int bn, void* stream);
/* Consumer of qb_gemm_rs fused with the next block's input: v = sum_i src_i (fp32, source order; src_i = src0 + i *
 * src_stride elements, bf16 [tok][H]) + res; hout = bf16(v); y = rmsnorm(v) * wt; two-level NVFP4 quantiser of y.
 * wait_flags (may be NULL): every CTA first waits until its nsrc words are >= wait_val. fan == 0: outputs go to
 * Bbytes_v[0] / sf_atoms_v[0] / g_v[0] for the tok local rows. fan > 0: they go to `fan` gathered arrays of tok_total rows
 * (one per rank, peer pointers) at rows row0 .. row0 + tok: the all-gather of the quantised activations is done by the
 * stores. sig_n > 0: the last CTA writes sig_val into word sig_rank of every sig_flags[d] (done_counter as above). */
int qb_reduce_norm_quant(const void* src0, long long src_stride, int nsrc, const void* res, const void* wt, void* hout,
                         void* const* Bbytes_v, void* const* sf_atoms_v, void* const* g_v, int fan, int row0, int tok_total, int tok,
                         int H, float eps, int block, const void* wait_flags, int wait_val, void* const* sig_flags, int sig_n,
                         int sig_rank, int sig_val, void* done_counter, const void* value_ptr, void* stream);
/* Rotary position embedding in place on a token-major bf16 matrix x [tok][row_stride] whose first n_heads * 128 columns
 * are heads of 128 values (the q and k heads of a QKV GEMM output): rotate-half convention, position = row % seq,
 * cos_sin fp32 [seq][128] = cos[0:64] | sin[0:64]; fp32 arithmetic, one rounding to bf16. No reference counterpart (the
 * reference leaves RoPE to the framework, harness/real_model.py:181-188). */
int qb_rope_inplace(void* x, const void* cos_sin, int tok, int seq, long long row_stride, int n_heads, void* stream);
/* Synchronise `stream`, return and clear the device status word (0 = no error). */
int qb_status(void* stream);
/* Error code of the last void-returning entry point on this thread. */
int qb_last_error(void);
const char* qb_version(void);

#ifdef __cplusplus
}
#endif
#endif
