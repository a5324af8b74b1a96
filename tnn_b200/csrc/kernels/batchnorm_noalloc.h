// Training-mode batch-norm forward that never allocates memory.
//
// This entry point has no counterpart in the reference. It exists for callers that are not allowed to
// allocate when they run a layer: code inside a region where device memory must stay fixed (a caller
// that has handed all remaining memory to another component, or that runs under a framework whose
// allocator must not be re-entered, e.g. from a stream callback or a plugin "enqueue" hook), and
// C or C++ hosts without PyTorch that do not want to manage a workspace. The regular entry point
// tnnb_batchnorm_fwd takes a caller-owned double[2*C] workspace; this one keeps that workspace in a
// fixed 64 KiB array that is part of the loaded library image on each device.
//
// Contract
//  * x, y: bf16 [M, C] row-major (NHWC flattened), 16-byte aligned; C a multiple of 8.
//  * gamma, beta: bf16 [C] or both null. mean, rstd, run_mean, run_var: fp32 [C].
//  * C <= TNNB_BN_NOALLOC_MAX_CHANNELS (4096). Larger C returns TNNB_NOALLOC_TOO_LARGE and launches
//    nothing; use tnnb_batchnorm_fwd for those.
//  * No cudaMalloc/cudaFree or any other allocating call is made, on any call. The first call on each
//    device looks up the address of the built-in array (cudaGetSymbolAddress, with that device
//    current); that is set-up work which may load the module, so make the first call before starting a
//    stream capture. Later calls only enqueue one memset of 2*C doubles (the sums must start at zero)
//    and two kernels on `stream`.
//  * There is one scratch array per device. Two calls that may overlap on the same device (different
//    streams, or different host threads) race on it; serialise them on one stream or with events.
//    The first call on a device is also not safe to make from two host threads at once.
//  * The array's address is looked up once per device and remembered for the life of the process. A
//    cudaDeviceReset() in the same process unloads the module and makes the remembered address stale:
//    do not call this entry point again after a device reset (restart the process instead).
//  * Returns TNNB_NOALLOC_OK (0) or a negative code; tnnb_noalloc_strerror gives the text.
#pragma once

#define TNNB_BN_NOALLOC_MAX_CHANNELS 4096

#define TNNB_NOALLOC_OK 0
#define TNNB_NOALLOC_BAD_ARG (-1)
#define TNNB_NOALLOC_TOO_LARGE (-2)
#define TNNB_NOALLOC_MISALIGNED (-3)
#define TNNB_NOALLOC_SETUP_FAILED (-4)
#define TNNB_NOALLOC_LAUNCH_FAILED (-5)

#ifdef __cplusplus
extern "C" {
#endif

int tnnb_batchnorm_fwd_noalloc(const void* x, void* y, const void* gamma, const void* beta, void* mean, void* rstd,
                               void* run_mean, void* run_var, long long M, int C, float eps, float momentum, int relu,
                               void* stream);
int tnnb_batchnorm_noalloc_max_channels(void);
const char* tnnb_noalloc_strerror(int rc);

#ifdef __cplusplus
}
#endif
