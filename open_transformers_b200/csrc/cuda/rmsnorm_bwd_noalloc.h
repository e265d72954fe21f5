// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for users of this library
// who drive it from places where asking the CUDA allocator for memory is not an option:
//   * a process that embeds the library through its C ABI without PyTorch (there is no caching
//     allocator to hand out the [rows/8, D] fp32 work buffer that `otb_rmsnorm_bwd` expects);
//   * a serving or real-time loop that reserved all of its device memory up front, where a
//     cudaMalloc in the middle of a step would either fail or stall every stream of the device
//     while the driver synchronises.
// Such callers still own the inputs and outputs; only the kernel's internal work buffer (the
// per-slab partial sums of the gain gradient) comes from inside the library.
//
// The work buffer is a fixed array in device memory that is part of the library image: every
// GPU that loads the library holds OTB_RMSNORM_NOALLOC_MAX_FLOATS * 4 bytes (16 MiB) for it until
// the process exits. A problem needs ceil(rows / 8) * D floats of it; larger problems are
// rejected with OTB_NOALLOC_TOO_LARGE and nothing is launched.
//
// Sharing rules. All calls on one device use the same array. The kernel overwrites every entry
// it later reads, so nothing has to be cleared between calls and the previous call's contents
// never leak into a result; but two calls whose kernels overlap in time on one device (different
// streams, or different host threads) would write the same entries and race. Serialise them:
// one stream, or an event between streams.
//
// First call on a device. The first call made while a given device is current looks up the
// device address of the array (cudaGetSymbolAddress) and caches it; later calls on that device
// skip this. That look-up is a synchronous runtime call, so make the first call on each device
// during start-up, before any stream capture begins.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OTB_RMSNORM_NOALLOC_MAX_FLOATS (4u * 1024u * 1024u)
#define OTB_NOALLOC_TOO_LARGE (-10)   // ceil(rows/8) * D exceeds the built-in work buffer
#define OTB_NOALLOC_BAD_SHAPE (-2)    // D not a multiple of 8, D > 4096, or rows <= 0

// dx[rows, D] and dgamma[D] (fp32) from dy, x (activation dtype: dtype = 1 bf16, 0 fp32), the gain w
// (activation dtype, may be NULL for a gain-free norm; dgamma is then left untouched) and rstd[rows] (fp32)
// as produced by otb_rmsnorm_fwd. inv_d = 1 / D. Results are bit-identical to otb_rmsnorm_bwd.
// Returns 0, one of the codes above, or a CUDA error code. Never allocates or frees memory.
int otb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dgamma,
                            long rows, int D, float inv_d, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
