// t3_moe_noalloc: the routed-expert chain at decode rows for callers that have no device memory to hand over.
//
// t3_moe wants a caller-allocated workspace (the down projection's prepared inputs and every row-slot's finished output,
// t3_moe_workspace_bytes). Some hosts cannot provide one: a serving process whose memory pool already owns the whole
// GPU, a plugin that is only handed activations and weights, code that runs where cudaMalloc's implicit device
// synchronisation is unacceptable. For them this file keeps that workspace in a fixed array that is part of the library
// image: every GPU that loads libt3.so holds kNoAllocScratchBytes of device memory for it until the process exits,
// whether or not this entry point is ever called.
//
// The array's name in host code is only a handle; the kernels need its device address, which the first call on each
// device looks up with cudaGetSymbolAddress (with that device current) and keeps. That first call should therefore come
// before any stream capture. Every call uses the same array and nothing is cleared between calls: the chain writes each
// element of the workspace before it reads it (gate|up writes a row-slot's whole prepared row, down writes its whole
// output row, merge reads only those), so stale contents are never seen. Two calls whose kernels may run at the same time
// on one GPU (different streams, or different host threads) would write the same array and race; keep such calls on
// one stream, or give the others t3_moe with their own workspace.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/t3.h"

namespace {

constexpr size_t kNoAllocScratchBytes = T3_NOALLOC_SCRATCH_BYTES;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

std::mutex g_setup_mu;
void* g_scratch_addr[64] = {};  // the array's device address, per device ordinal

// The scratch array's address on the current device; looked up once per device.
int scratch_address(void** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return T3_CUDA_ERROR;
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (!g_scratch_addr[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || !ptr) return T3_CUDA_ERROR;
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return T3_OK;
}

}  // namespace

extern "C" int t3_moe_noalloc(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds,
                              const void* scores, int scores_dtype, int topk, t3_decode dec, void* y, void* stream) {
    if (!bank) return T3_NULL_POINTER;
    if (rows < 1 || topk <= 0) return T3_BAD_EXL3_SHAPE;
    if (rows > T3_DECODE_ROWS_MAX) return T3_SCRATCH_LIMIT_EXCEEDED;  // the prefill chain's scratch runs to gigabytes
    const size_t need = t3_moe_workspace_bytes(rows, topk, bank);
    if (need == 0) return T3_BAD_EXL3_SHAPE;
    if (need > kNoAllocScratchBytes) return T3_SCRATCH_LIMIT_EXCEEDED;
    void* scratch = nullptr;
    if (int rc = scratch_address(&scratch)) return rc;
    return t3_moe(x, x_dtype, rows, bank, inds, scores, scores_dtype, topk, dec, y, scratch, kNoAllocScratchBytes, stream);
}
