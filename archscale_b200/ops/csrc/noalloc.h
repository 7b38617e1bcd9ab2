// Allocation-free entry point.  No counterpart in the reference: it exists for callers of this
// library that are not allowed to allocate device memory when they call in.
//
// Who that is: code running while a CUDA stream is being captured, code inside a host callback
// or a real-time loop where cudaMalloc (an implicit device synchronisation, and a call that can
// fail under memory pressure) is off limits, and embedders that hand this library a fixed memory
// budget and forbid every allocator, torch's caching allocator included.
//
// b200_rmsnorm_bwd_noalloc is the RMSNorm backward of norm.cu with its only scratch buffer (the
// per-CTA partial sums of the weight gradient, fp32 [n_ctas, cols]) taken from a file-scope
// device array instead of a caller-provided allocation.  The caller still passes every input and
// output (dy, x, w, rstd, dx, dw).
//
// Limits and rules
//  * cols must be a multiple of 8 and at most B200_NOALLOC_MAX_COLS (4096); larger shapes are
//    rejected with a negative return code and a message in b200_noalloc_last_error().
//  * The array (B200_NOALLOC_SCRATCH_FLOATS floats ≈ 4.6 MiB) is part of the loaded module: every
//    GPU that loads the library holds it until the process exits.
//  * The first call on a device resolves the array's device address (cudaGetSymbolAddress, with
//    that device current) and caches it; make that first call outside any stream capture.  With
//    lazy module loading (the CUDA default) the driver also materialises the array at that moment,
//    so the device's free memory drops by the array's size during the first call and never again.
//  * All calls share the one array and it keeps the previous call's contents.  Nothing in it has
//    to start at zero (every CTA overwrites its own row before the reduction reads it), but two
//    calls that overlap on the GPU (different streams) race on it: serialise them.
//  * It calls no cudaMalloc / cudaFree and no allocating library routine.
//  * The cached device addresses and the last-error string are plain process globals without locks:
//    concurrent first calls from several host threads, or reading the error string while another
//    thread's call fails, are the caller's to serialise.
#pragma once
#include <cuda_runtime.h>

#define B200_NOALLOC_MAX_COLS 4096
#define B200_NOALLOC_MAX_CTAS 296
#define B200_NOALLOC_SCRATCH_FLOATS (B200_NOALLOC_MAX_CTAS * B200_NOALLOC_MAX_COLS)

#ifdef __cplusplus
extern "C" {
#endif

// dtype codes: 0 = fp32, 1 = bf16.  w may be null (then dw is ignored and no scratch is used).
// dx has the dtype of x; dw is fp32 [cols].  Returns 0 on success, < 0 on a rejected argument or a
// failed launch (see b200_noalloc_last_error()).
int b200_rmsnorm_bwd_noalloc(const void* dy, int dy_dtype, const void* x, int x_dtype, const void* w, int w_dtype,
                             const float* rstd, void* dx, float* dw, int rows, int cols, cudaStream_t stream);

const char* b200_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
