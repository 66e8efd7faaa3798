// Split-K GEMM entry point for callers that cannot hand the library a workspace.
//
// The split-K form of the GEMM (thin token counts, K divided over CTAs) adds fp32 partial
// sums into a [tok][out] workspace before the bf16 conversion. qb_gemm takes that workspace
// from the caller. Some callers have no way to provide one: a serving engine that has
// already given all free device memory to its own pool, so that cudaMalloc fails or
// fragments it; code running while a stream is being captured into a CUDA graph, where an
// allocation call is illegal; a plugin hook whose signature only carries inputs and outputs.
// For them the workspace lives here, in a fixed array that is part of the loaded library
// image on every GPU that loads it (8 MiB per device until the process exits).
#include <mutex>

#include "../../include/quadbit_b200.h"
#include "qb_common.cuh"
#include "qb_internal.h"

#define QB_STATIC_WS_FLOATS (2 * 1024 * 1024)   // tok * out <= 2 Mi partial sums (8 MiB)

static __device__ __align__(256) float g_static_ws[QB_STATIC_WS_FLOATS];

namespace {
std::mutex g_ws_mu;
float* g_ws_dev_ptr[64] = {nullptr};   // device address of g_static_ws, per device ordinal

// The array's name is only a host-side handle; the address a kernel can use has to be
// asked for once per device, with that device current.
int static_ws_ptr(float** out) {
    int dev = -1;
    int rc = (int)cudaGetDevice(&dev);
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return QB_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lk(g_ws_mu);
    if (!g_ws_dev_ptr[dev]) {
        float* p = nullptr;
        rc = (int)cudaGetSymbolAddress((void**)&p, g_static_ws);
        if (rc) return rc;
        if (!p) return QB_ERR_DRIVER;
        g_ws_dev_ptr[dev] = p;
    }
    *out = g_ws_dev_ptr[dev];
    return QB_OK;
}
}  // namespace

extern "C" {

long long qb_gemm_splitk_static_max_elems(void) { return (long long)QB_STATIC_WS_FLOATS; }

int qb_gemm_splitk_static(const void* A, const void* B, const void* sfa, const void* sfb, const void* meta_native,
                          const void* gA, const void* gB, void* C, int out, int tok, int K, int sparse, int out_mode,
                          int splits, void* stream) {
    if (out <= 0 || tok < 0 || K <= 0) return QB_ERR_ARG;
    if (out_mode != 0 && out_mode != 1) return QB_ERR_ARG;
    if (sparse < 0 || sparse > 3) return QB_ERR_ARG;   // bit 0: 2:4-sparse A, bit 1: A in the tiled layout (as qb_gemm)
    if ((long long)out * (long long)tok > (long long)QB_STATIC_WS_FLOATS) return QB_ERR_TOO_LARGE;
    if (tok == 0) return QB_OK;
    float* ws = nullptr;
    int rc = static_ws_ptr(&ws);
    if (rc) return rc;
    qb::GemmArgs g{};
    g.A = A; g.B = B; g.sfa = sfa; g.sfb = sfb; g.meta = meta_native; g.gA = (const float*)gA; g.gB = (const float*)gB;
    g.C = C; g.Cf = ws; g.eblk = nullptr; g.bias = nullptr; g.row_w = nullptr;
    g.a_rows = out; g.out_f = out; g.tok = tok; g.K = K; g.sparse = sparse & 1; g.a_tiled = (sparse >> 1) & 1; g.out_mode = out_mode;
    g.splits = splits < 2 ? 2 : splits;   // always the workspace path; it is zeroed on the stream first
    g.bn = 0;
    return qb::gemm_nvfp4(g, (cudaStream_t)stream);
}

}  // extern "C"
