// extern "C" surface of the library (declared in include/quadbit_b200.h).
//
// The reference-named entry points accept the reference's tensor layouts; the tcgen05
// GEMM needs scale factors as 128x4 atoms and metadata row-major per 128-row block, so
// these wrappers re-layout scales / metadata into a per-device scratch buffer on every
// call (a few percent of a prefill GEMM; nothing is cached, so a caller that rewrites a
// weight buffer in place is safe). The scratch buffer is the one device allocation the
// library makes; it grows on demand under a mutex, so the first call at a new size must
// happen outside CUDA-graph capture. The native qb_* entry points allocate nothing.
#include <mutex>

#include "../../include/quadbit_b200.h"
#include "qb_common.cuh"
#include "qb_internal.h"

namespace {

thread_local int t_last_error = 0;

struct Scratch {
    void* ptr = nullptr;
    size_t cap = 0;
};
std::mutex g_scratch_mu;
Scratch g_scratch[64];

// Returns a device buffer of at least `bytes` for the current device (256-byte aligned).
int scratch_get(size_t bytes, void** out) {
    int dev = 0;
    int rc = (int)cudaGetDevice(&dev);
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return QB_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    Scratch& s = g_scratch[dev];
    if (s.cap < bytes) {
        if (s.ptr) {
            rc = (int)cudaDeviceSynchronize();
            if (rc) return rc;
            cudaFree(s.ptr);
            s.ptr = nullptr;
            s.cap = 0;
        }
        size_t cap = bytes + (bytes >> 2) + (1 << 20);
        rc = (int)cudaMalloc(&s.ptr, cap);
        if (rc) return rc;
        s.cap = cap;
    }
    *out = s.ptr;
    return QB_OK;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

size_t sf_atoms_bytes(int rows, int K, int block) {
    return (size_t)((rows + 127) / 128) * (size_t)(qb::kpad256(K) / block / 4) * 512;
}
size_t meta_native_bytes(int out_f, int K) { return (size_t)((out_f + 127) / 128) * (size_t)(qb::kpad256(K) / 256) * 2048; }

// GEMM on reference-layout operands: re-layout into scratch, then run the native kernel.
int ref_gemm(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C, float* Cf,
             int a_rows, int out_f, int tok, int K, const void* gA, const void* gB, const int* eblk, const void* bias,
             const float* row_w, int sparse, int out_mode, int splits, cudaStream_t st) {
    if (a_rows <= 0 || out_f <= 0 || tok < 0 || K <= 0 || K % 128 || a_rows % 128) return QB_ERR_ARG;
    if (tok == 0) return QB_OK;
    if (!scaleA || !scaleB || (sparse && !meta)) return QB_ERR_ARG;
    const int block = sparse ? 32 : 16;
    size_t n_sfa = align256(sf_atoms_bytes(a_rows, K, block));
    size_t n_sfb = align256(sf_atoms_bytes(tok, K, block));
    size_t n_meta = sparse ? align256(meta_native_bytes(a_rows, K)) : 0;
    void* base = nullptr;
    int rc = scratch_get(n_sfa + n_sfb + n_meta, &base);
    if (rc) return rc;
    uint8_t* p_sfa = (uint8_t*)base;
    uint8_t* p_sfb = p_sfa + n_sfa;
    uint8_t* p_meta = p_sfb + n_sfb;
    if (K % 256) {   // zero the K tail of the padded native arrays
        rc = (int)cudaMemsetAsync(base, 0, n_sfa + n_sfb + n_meta, st);
        if (rc) return rc;
    }
    rc = qb::relayout_sf(scaleA, p_sfa, a_rows, K, block, st);
    if (rc) return rc;
    rc = qb::relayout_sf(scaleB, p_sfb, tok, K, block, st);
    if (rc) return rc;
    if (sparse) {
        rc = qb::relayout_meta(meta, p_meta, a_rows, K, st);
        if (rc) return rc;
    }
    qb::GemmArgs g{};
    g.A = A; g.B = B; g.sfa = p_sfa; g.sfb = p_sfb; g.meta = sparse ? p_meta : nullptr;
    g.gA = (const float*)gA; g.gB = (const float*)gB; g.C = C; g.Cf = Cf; g.eblk = eblk; g.bias = bias; g.row_w = row_w;
    g.a_rows = a_rows; g.out_f = out_f; g.tok = tok; g.K = K; g.sparse = sparse; g.out_mode = out_mode;
    g.splits = splits; g.bn = 0;
    return qb::gemm_nvfp4(g, st);
}

int finish_sync(int rc, cudaStream_t st) {
    if (rc) return rc;
    return qb::read_status(st);
}

}  // namespace

extern "C" {

const char* qb_version(void) { return "quadbit_b200 0.1 (sm_100a, tcgen05)"; }
int qb_last_error(void) { return t_last_error; }

// ------------------------------------------------------------------ native
int qb_quantize_act(const void* x, void* Bbytes, void* sf_ref, void* sf_atoms, void* g, int tok, int K, int block,
                    void* stream) {
    return qb::quantize_act(x, Bbytes, sf_ref, sf_atoms, g, tok, K, block, (cudaStream_t)stream);
}
int qb_compress_2to4(const void* W, int w_dtype, void* Ac, void* meta_ref, void* meta_native, void* sf_ref, void* sf_atoms,
                     void* gA, int out, int K, void* stream) {
    return qb::compress_2to4(W, w_dtype, Ac, meta_ref, meta_native, sf_ref, sf_atoms, gA, out, K, (cudaStream_t)stream);
}
int qb_pack_dense(const void* W, int w_dtype, void* Ab, void* sf_ref, void* sf_atoms, void* gA, int out, int K,
                  void* stream) {
    return qb::pack_dense(W, w_dtype, Ab, sf_ref, sf_atoms, gA, out, K, (cudaStream_t)stream);
}
int qb_relayout_sf(const void* sf_ref, void* sf_atoms, int rows, int K, int block, void* stream) {
    return qb::relayout_sf(sf_ref, sf_atoms, rows, K, block, (cudaStream_t)stream);
}
int qb_relayout_meta(const void* meta_ref, void* meta_native, int out, int K, void* stream) {
    return qb::relayout_meta(meta_ref, meta_native, out, K, (cudaStream_t)stream);
}
long long qb_sf_atoms_bytes(int rows, int K, int block) {
    if (rows < 0 || K <= 0 || (block != 16 && block != 32)) return -1;
    return (long long)sf_atoms_bytes(rows, K, block);
}
long long qb_meta_native_bytes(int out, int K) {
    if (out < 0 || K <= 0) return -1;
    return (long long)meta_native_bytes(out, K);
}
int qb_gemm(const void* A, const void* B, const void* sfa, const void* sfb, const void* meta_native, const void* gA,
            const void* gB, void* C, void* Cf, const void* eblk, const void* bias, const void* row_w, int a_rows, int out,
            int tok, int K, int sparse, int out_mode, int splits, int bn, void* stream) {
    qb::GemmArgs g{};
    g.A = A; g.B = B; g.sfa = sfa; g.sfb = sfb; g.meta = meta_native; g.gA = (const float*)gA; g.gB = (const float*)gB;
    g.C = C; g.Cf = (float*)Cf; g.eblk = (const int*)eblk; g.bias = bias; g.row_w = (const float*)row_w;
    g.a_rows = a_rows; g.out_f = out; g.tok = tok; g.K = K; g.sparse = sparse; g.out_mode = out_mode; g.splits = splits;
    g.bn = bn;
    return qb::gemm_nvfp4(g, (cudaStream_t)stream);
}
int qb_status(void* stream) { return qb::read_status((cudaStream_t)stream); }

// ------------------------------------------------------------------ reference symbols
int sparse_fp4_mm(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C, int out,
                  int tok, int K) {
    return finish_sync(ref_gemm(A, B, scaleA, scaleB, meta, C, nullptr, out, out, tok, K, nullptr, nullptr, nullptr, nullptr,
                                nullptr, 1, 0, 1, 0), 0);
}
int sparse_fp4_mm_2lvl(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C,
                       int out, int tok, int K, const void* gA, const void* gB) {
    return finish_sync(ref_gemm(A, B, scaleA, scaleB, meta, C, nullptr, out, out, tok, K, gA, gB, nullptr, nullptr, nullptr,
                                1, 0, 1, 0), 0);
}
int sparse_fp4_mm_2lvl_t(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C,
                         int out, int tok, int K, const void* gA, const void* gB) {
    return finish_sync(ref_gemm(A, B, scaleA, scaleB, meta, C, nullptr, out, out, tok, K, gA, gB, nullptr, nullptr, nullptr,
                                1, 1, 1, 0), 0);
}
int sparse_down_sk_2lvl(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* Cout,
                        void* Cf, int out, int tok, int K, const void* gA, const void* gB, int splits) {
    return finish_sync(ref_gemm(A, B, scaleA, scaleB, meta, Cout, (float*)Cf, out, out, tok, K, gA, gB, nullptr, nullptr,
                                nullptr, 1, 1, splits, 0), 0);
}
int dense_nvfp4_mm(const void* A, const void* B, const void* SFA, const void* SFB, void* C, int out, int tok, int K,
                   const void* gA, const void* gB) {
    return finish_sync(ref_gemm(A, B, SFA, SFB, nullptr, C, nullptr, out, out, tok, K, gA, gB, nullptr, nullptr, nullptr, 0, 0,
                                1, 0), 0);
}
int sparse_moe_mm_2lvl(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C,
                       int Mtot, int Mpe, int rows, int K, const void* gA, const void* gB, const void* eblk, int outT,
                       void* stream) {
    if (rows % 128 || !eblk || (outT != 0 && outT != 1)) return QB_ERR_ARG;
    int rc = ref_gemm(A, B, scaleA, scaleB, meta, C, nullptr, Mtot, Mpe, rows, K, gA, gB, (const int*)eblk, nullptr, nullptr,
                      1, outT, 1, (cudaStream_t)stream);
    return stream ? rc : finish_sync(rc, 0);
}
int sparse_moe_mm_2lvl_bw(const void* A, const void* B, const void* scaleA, const void* scaleB, const void* meta, void* C,
                          int Mtot, int Mpe, int rows, int K, const void* gA, const void* gB, const void* eblk,
                          const void* sc_w, const void* bias, int Hout, void* stream) {
    (void)Hout;
    if (rows % 128 || !eblk) return QB_ERR_ARG;
    int rc = ref_gemm(A, B, scaleA, scaleB, meta, C, nullptr, Mtot, Mpe, rows, K, gA, gB, (const int*)eblk, bias,
                      (const float*)sc_w, 1, 3, 1, (cudaStream_t)stream);
    return stream ? rc : finish_sync(rc, 0);
}
int moe_route(const void* assign, const void* poff, void* counter, void* src, int N, int E, void* stream) {
    int rc = qb::moe_route(assign, const_cast<void*>(poff), counter, src, N, E, (cudaStream_t)stream);
    return stream ? rc : finish_sync(rc, 0);
}
int moe_combine_topk(const void* dbuf, const void* inverse, void* y, int t, int H, int topk, int Mpe, void* stream) {
    int rc = qb::moe_combine_topk(dbuf, inverse, y, t, H, topk, Mpe, (cudaStream_t)stream);
    return stream ? rc : finish_sync(rc, 0);
}
void qb_init_func_attrs(void) { t_last_error = qb::gemm_init_attrs(); }
void qb_init_sk_attrs(void) { t_last_error = qb::gemm_init_attrs(); }
void qb_init_moe_attrs(void) { t_last_error = qb::gemm_init_attrs(); }
void qb_init_gusw_attrs(void) { t_last_error = qb::gemm_init_attrs(); }

#ifdef QB_FLAVOUR_DENSE
#define QB_ACT_BLOCK 16
#else
#define QB_ACT_BLOCK 32
#endif
void quantize_act_nvfp4(const void* x, void* Bbytes, void* scaleB, int tok, int K) {
    t_last_error = qb::quantize_act(x, Bbytes, scaleB, nullptr, nullptr, tok, K, 32, 0);
}
void quantize_act_nvfp4b(const void* x, void* Bbytes, void* scaleB, int tok, int K) {
    t_last_error = qb::quantize_act(x, Bbytes, scaleB, nullptr, nullptr, tok, K, 16, 0);
}
void quantize_act_nvfp4_2lvl(const void* x, void* Bbytes, void* scaleB, void* gB, int tok, int K) {
    t_last_error = gB ? qb::quantize_act(x, Bbytes, scaleB, nullptr, gB, tok, K, QB_ACT_BLOCK, 0) : QB_ERR_ARG;
}
void quantize_act_nvfp4_2lvl_s(const void* x, void* Bbytes, void* scaleB, void* gB, int tok, int K, void* stream) {
    t_last_error = gB ? qb::quantize_act(x, Bbytes, scaleB, nullptr, gB, tok, K, QB_ACT_BLOCK, (cudaStream_t)stream) : QB_ERR_ARG;
}

}  // extern "C"
