// Allocation-free entry point (no counterpart in the reference).
//
// Some hosts of this library may not allocate device memory at the point where they call it: a plug-in that runs
// inside another runtime's memory pool, a caller in the middle of a latency-critical section where cudaMalloc's
// implicit synchronisation is unacceptable, or a process whose allocator has been frozen after start-up.  For them
// ds41_hc_step_static runs the fused hyper-connection step (see ds41_hc_step) with its scratch memory - the slice
// partials, the collapsed row and the per-row ticket counters - taken from a fixed array that lives inside the
// library image instead of from caller-provided buffers.
//
//  * Limits: rows <= DS41_HC_STATIC_MAX_ROWS and H <= DS41_HC_STATIC_MAX_H (H a multiple of 128).  Larger sizes are
//    refused with cudaErrorInvalidValue before anything is launched.
//  * The array (631,040 bytes: 106,496 of slice partials, 524,288 of collapsed rows, 256 of ticket counters) is
//    part of every GPU context that loads the library and stays until the process exits.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
//    current) and caches it per device; concurrent first calls are safe (they store the same value through an
//    atomic).  Make that first call before starting any stream capture.  The cached address is not refreshed: after
//    cudaDeviceReset on a device the entry point must not be used on it again in the same process.
//  * No cudaMalloc / cudaFree / allocating library routine is called.  The fields `partial`, `xc` and `tickets` of
//    the argument struct are ignored; inputs and outputs are still the caller's.
//  * Every call uses the same array and the array keeps the previous call's contents; the ticket counters are
//    cleared on the stream before each launch.  Two calls that overlap on the GPU (different streams, or the same
//    call from two threads) race on the array: serialise them.
#pragma once
#include "ds41_api.h"

#define DS41_HC_STATIC_MAX_ROWS 16
#define DS41_HC_STATIC_MAX_H 8192

#ifdef __cplusplus
extern "C" {
#endif

int ds41_hc_step_static(const ds41_hc_step_args* args, void* stream);

#ifdef __cplusplus
}
#endif
