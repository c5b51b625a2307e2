// Entry point of the native library that never allocates device memory.
//
// This declaration has no counterpart in the reference framework; it exists for embedders of this
// library that are not allowed to call cudaMalloc at the time they need a routing sort: code that
// runs while a CUDA stream is being captured, a serving loop whose device memory is owned entirely
// by another allocator, or a process that has been handed a fixed memory budget up front. For such
// callers any allocation is either illegal (capture), a hidden device-wide synchronisation, or a
// budget violation, so the scratch the kernels need has to exist before the call.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of experts the no-allocation routing sort accepts. The scratch behind it is a
// file-scope device array of this many 32-bit counters (4 KiB), resident on every GPU that loads
// the library until the process exits.
#define PT_ROUTE_SORT_NOALLOC_MAX_EXPERTS 1024

// Stable counting sort of `n` routing slots by local expert id — same result as pt_route_sort, but
// the per-expert counters live in the library's static device array instead of a caller buffer.
//
//   eids         [n]        int32 expert id per slot; ids outside [0, E) are skipped
//   offs         [E + 1]    out: first row of every expert group (groups padded to `align` rows)
//   row_of_slot  [n]        out: row of each slot, -1 for skipped slots
//   slot_of_row  [r_cap]    out: slot of each row, -1 for padding rows
//
// Returns 0 on success, -1 for invalid arguments, -2 when E exceeds
// PT_ROUTE_SORT_NOALLOC_MAX_EXPERTS (a message goes to stderr), or a cudaError_t value.
// No cudaMalloc / cudaFree / allocating library routine is called. If the rows do not fit in
// `r_cap`, nothing is written past it and offs[E] > r_cap tells the caller so; in that case check
// offs[E] before reading slot_of_row: the rows of the first group that does not fit are left
// unwritten (neither a slot nor -1), so the contents of slot_of_row are unspecified.
//
// The first call on a device resolves the device address of the static scratch
// (cudaGetSymbolAddress); make that call once per device before starting any stream capture.
// All calls share the one scratch array: calls whose kernels may overlap on the GPU (different
// streams without ordering) race on it. The counters are fully rewritten by every call, so no
// state leaks from one call to the next.
int pt_route_sort_noalloc(const int* eids, int n, int E, int align, int* offs, int* row_of_slot,
                          int* slot_of_row, int r_cap, void* stream);

#ifdef __cplusplus
}
#endif
