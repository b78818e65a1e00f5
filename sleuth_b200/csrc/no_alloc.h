// An entry point of this library that allocates nothing. It has no counterpart in tbertha35/Sleuth, whose
// GPU code is PyTorch and Triton and allocates through the framework.
//
//   int slb_argmax_static(const float* logits, long long ld, int rows, int limit, int* out, void* stream);
//
// Who needs it. Some callers of a CUDA library may not call cudaMalloc, or any routine that may call it on their
// behalf: real-time or embedded hosts that size all device memory once, up front, and forbid allocation afterwards
// (an allocation can block, fail late, or fragment a budget that was checked at start-up); and hosts that load this
// .so from C or another language without torch, whose caching allocator serves the rest of the library and which
// therefore have no allocator to hand scratch memory out of. slb_argmax needs scratch memory
// for the partial results of its first stage and makes the caller supply it. slb_argmax_static does the same job
// with scratch that is part of the library itself: a file-scope `static __device__` array of
// 2 * SLB_ARGMAX_STATIC_MAX_ROWS * 64 four-byte words (512 KiB), aligned to 256 bytes. The caller passes only the
// logits and the output.
//
// What the caller must know.
//   * Every GPU that loads the library holds those 512 KiB from the load until the process ends.
//   * At most SLB_ARGMAX_STATIC_MAX_ROWS rows per call; more are refused with a message that names the limit.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress, with that device
//     current) and keeps it; later calls on that device do no set-up. Make that first call before any stream capture.
//   * All calls on a device share the one array. Calls that may overlap on the GPU (different streams without an
//     ordering between them) race on it and must not be made; calls ordered on one stream are fine.
//   * Nothing has to be cleared between calls: each call's second stage reads only slots that its own first
//     stage wrote, so what an earlier call left behind is never read.
//   * Host threads: the per-device address is kept in an atomic slot, so first calls made at the same time from
//     several host threads are safe (each may do the look-up; all store the same address). The error message of a
//     failed call is kept per host thread.
//   * It calls no cudaMalloc, cudaFree or allocating library routine, torch's included. Results equal slb_argmax's:
//     the index of the largest of logits[r, 0 .. limit), the lowest index on ties.
// Returns 0, or a non-zero code with the message available from slb_last_error().
#pragma once

#define SLB_ARGMAX_STATIC_MAX_ROWS 1024

#ifdef __cplusplus
extern "C" {
#endif
int slb_argmax_static(const float* logits, long long ld, int rows, int limit, int* out, void* stream);
int slb_argmax_static_max_rows(void);
#ifdef __cplusplus
}
#endif
