// Routing-plan entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference.
//
// Who needs it: a host program that has already given the whole GPU to its own memory pool (an
// inference server that sizes every buffer at start-up), or one that calls into this library from a
// loop where cudaMalloc / cudaFree are unacceptable because they can fail once the pool owns the
// device and because they synchronise the device. Such a caller passes its inputs and outputs and
// nothing else; the kernels' scratch memory is a fixed array inside the library.
//
// ccf_route_noalloc computes, for S routed slots with expert ids expert[0..S), the same three results
// as ccf_route (moe_kernels.cu): pos[s] = number of earlier slots with the same expert id,
// count_raw[e] = slots per expert, count_kept[e] = min(count_raw[e], cap). Ids outside [0, E) get the
// position 0x3fffffff and are not counted.
//
// Limits and rules:
//   * S <= CCF_NOALLOC_MAX_SLOTS and E <= CCF_NOALLOC_MAX_EXPERTS; larger sizes are rejected with
//     CCF_NOALLOC_ERR_SIZE and nothing is launched. The scratch array takes
//     CCF_NOALLOC_SCRATCH_BYTES (about 129 KiB) of device memory on every GPU that loads the library,
//     from load until the process exits.
//   * The first call on a device looks up the device address of the scratch array
//     (cudaGetSymbolAddress) and caches it. Make that first call with the device current and before
//     any stream capture begins on that device.
//   * The call itself allocates nothing: no cudaMalloc, cudaFree, or allocating library routine.
//   * All calls on a device share the one scratch array, which still holds whatever the previous call
//     left there; each call clears the part that has to start at zero. Two calls whose kernels can
//     overlap on the GPU (different streams without an ordering between them) race on it: order them.
//   * Returns 0, or a negative code; ccf_route_noalloc_strerror gives the message.
#pragma once

#define CCF_NOALLOC_MAX_SLOTS 65536
#define CCF_NOALLOC_MAX_EXPERTS 256
#define CCF_NOALLOC_MAX_BLOCKS (CCF_NOALLOC_MAX_SLOTS / 1024)
#define CCF_NOALLOC_SCRATCH_INTS (2 * CCF_NOALLOC_MAX_BLOCKS * CCF_NOALLOC_MAX_EXPERTS + 64)
#define CCF_NOALLOC_SCRATCH_BYTES (CCF_NOALLOC_SCRATCH_INTS * 4)

#define CCF_NOALLOC_ERR_SIZE (-2)      /* S or E beyond the stated maximum (or negative) */
#define CCF_NOALLOC_ERR_ARG (-3)       /* a null pointer where a buffer is required */
#define CCF_NOALLOC_ERR_SETUP (-4)     /* the scratch array's device address could not be obtained */
#define CCF_NOALLOC_ERR_LAUNCH (-5)    /* the CUDA runtime refused a memset or a launch */

#ifdef __cplusplus
extern "C" {
#endif

int ccf_route_noalloc(const int* expert, int S, int E, int cap, int* pos, int* count_raw, int* count_kept,
                      void* stream);
const char* ccf_route_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
