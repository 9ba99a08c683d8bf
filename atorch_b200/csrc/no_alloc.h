// Allocation-free entry point of libatb.so. It has no counterpart in the reference framework.
//
// Who needs it: callers that may not (or cannot) allocate device memory around a kernel call. Think
// of a host runtime that owns all device memory in its own arena and gives a plug-in only its input
// and output buffers, a code path that runs while another library holds the allocator, or a
// latency-critical loop that has to stay clear of cudaMalloc/cudaFree (both synchronise the
// device). The regular RMSNorm backward (atb_norm_bwd + atb_colsum) needs a scratch matrix that its
// PyTorch wrapper allocates per call; this variant carries the scratch inside the library.
//
// Contract
//  * Computes, for x, dy of shape [M, N] and weight w[N] (all of `dtype`; 0 = bf16, 1 = fp16, 2 = fp32)
//    and rstd[M] (fp32, saved by the forward):
//        dx[M, N] = (w * dy - xhat * mean(xhat * w * dy)) * rstd,   xhat = x * rstd
//        dw[N]    = sum over rows of dy * xhat                       (overwritten, not accumulated)
//  * Calls no cudaMalloc / cudaFree / allocating library routine. The scratch is a file-scope
//    `static __device__` array of 148 x 8192 floats (4.6 MiB) that every GPU which loads the
//    library holds until the process exits.
//  * Limits: N <= 8192 (see atb_noalloc_max_n()), N a multiple of 8, any M > 0. Anything else
//    returns a negative code and leaves a message for atb_noalloc_last_error(); nothing is launched.
//  * The first call on each device looks up the device address of the scratch array (once, with
//    that device current). Make that first call before starting any stream capture.
//  * All calls on one device share the array, and it keeps the previous call's contents. Each call
//    rewrites every partial row it later reads, so nothing needs clearing in between; but two calls
//    whose kernels overlap on the GPU (different streams, or the same call issued from two threads)
//    race on the array. Serialise them on one stream, or order them with events.
//  * Returns 0 when both kernels were launched on `stream`.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

int atb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                            int M, int N, int dtype, void* stream);

// Largest N accepted by atb_rmsnorm_bwd_noalloc.
int atb_noalloc_max_n(void);

// Message of the last failed atb_rmsnorm_bwd_noalloc call on this thread ("" after a success).
const char* atb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
