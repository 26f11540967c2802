// velomind_no_alloc.h — decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (Aiza-Lee/velo-mind); it exists only in this
// library.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples are a plugin or real-time loop that
// is handed a fixed memory budget by its host program and may not grow it; a host that has frozen its
// memory pool (every later cudaMalloc would fragment or fail); and any code running at a point where an
// allocation is illegal or would stall the device, since cudaMalloc synchronises the whole device.  The
// ordinary entry point, vm_attention_decode_bf16, makes its caller provide two scratch buffers (partial
// results of the key splits, and arrival counters); a caller that cannot allocate has nowhere to get them.
//
// What it does: the same split-KV decode attention as vm_attention_decode_bf16 (same kernel, same
// arguments for inputs and outputs, same results), but the scratch lives in a file-scope
// `static __device__` array inside the library.  The function calls no cudaMalloc, no cudaFree and no
// allocating library routine.
//
// The price, and the rules that follow from it:
//   * The array has a fixed size, VM_NO_ALLOC_SCRATCH_BYTES (8 MiB).  Every GPU on which the library's
//     kernels are loaded holds these 8 MiB until the process exits, whether or not this function is called.
//   * A call whose scratch would not fit, i.e. 256-byte-rounded 4 * B * H bytes of counters plus
//     4 * B * H * n_splits * (D + 2) bytes of partials > VM_NO_ALLOC_SCRATCH_BYTES, is refused with
//     VM_NO_ALLOC_TOO_LARGE before anything is put on the stream (no memset, no kernel), and so is every size the
//     kernel does not take (-1).  vm_attention_decode_no_alloc_bytes() tells the need.
//   * All calls on a device share the one array, and it keeps whatever the last call left.  The function
//     clears the counters on the caller's stream before every launch; the partials need no clearing (every
//     value that is read is written first).  Two calls that overlap on the GPU (different streams without an
//     ordering between them, or different host threads) race on the scratch and give wrong results: order
//     them.
//   * The first call on each device looks up the array's device address with cudaGetSymbolAddress (with that
//     device current) and remembers it.  Make that first call outside of any stream capture.  The lookup takes no
//     lock: host threads that race on a device's first call store the same address, which is harmless.
//
// Return value: 0 on success; VM_NO_ALLOC_TOO_LARGE (-3); -1 / -2 for unsupported sizes or bad arguments as
// in the ordinary entry point; a positive cudaError_t if CUDA reports one.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VM_NO_ALLOC_SCRATCH_BYTES (8ll * 1024 * 1024)
#define VM_NO_ALLOC_TOO_LARGE (-3)

// Bytes of the static scratch a call with these sizes would use.
long long vm_attention_decode_no_alloc_bytes(int B, int H, int D, int n_splits);

// The device address of the static scratch on the current device (looked up like the entry point's first call does), or
// null.  For tests and diagnostics: a test fills the array with garbage between calls to show that a call depends on
// nothing an earlier call left there.
void* vm_attention_decode_no_alloc_scratch(void);

// q [B, H, D] bf16 rows with stride q_row_stride (elements); kpages/vpages [n_pages, Hkv, 64, D] bf16;
// block_table int32 [B, max_blocks]; positions int32 [B] (place of each sequence's new token);
// out [B, H*D] bf16.  One new token per sequence.
int vm_attention_decode_bf16_no_alloc(const void* q, int q_row_stride, const void* kpages, const void* vpages,
                                      const int* block_table, int max_blocks, const int* positions, void* out,
                                      int B, int H, int Hkv, int D, int n_splits, float scale, int window,
                                      int n_pages, int* err, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
