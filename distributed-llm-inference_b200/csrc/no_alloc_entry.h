// Split-key decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in zshabb/distributed-llm-inference; it exists for
// embedders of this library.
//
// Who needs it.  Some hosts hand every byte of device memory to their own arena when they
// start, and forbid cudaMalloc afterwards: a plug-in that runs inside another runtime's memory
// plan, a latency-critical loop where cudaMalloc's implicit device-wide synchronisation would
// stall every stream, or code that runs at a point where allocation is simply not permitted.
// The ordinary entry point, dli_paged_attention_mma, asks such a caller for two scratch
// buffers (the per-split partial results) whenever the keys are split across CTAs, and the
// Python wrapper allocates them with torch.  Here the scratch is a fixed array that is part of
// the loaded library's device image instead, so the call allocates nothing: no cudaMalloc, no
// cudaFree, no allocating library routine.  Inputs and outputs are still the caller's.
//
// What it costs.  The array is DLI_NOALLOC_SCRATCH_FLOATS floats (4 MiB); every GPU on which a
// process uses the library holds that much until the process exits.  A call needs
// (first_row + num_seqs) * nh * splits * (head_dim + 2) floats and is refused with
// DLI_ERR_SCRATCH_TOO_SMALL, before anything is launched, if that is more than the array holds.
//
// first_row and q_start.  The sequences of a call bring one token each, and those tokens are
// consecutive rows of q and out: sequence seq0 + i owns row first_row + i, and q_start must say
// so (q_start[seq0 + i] == first_row + i).  The kernels place a row's partial results in the
// array by that row number, counted from row 0 of the batch, which is why the need above counts
// the first_row rows in front as well.  A q_start that breaks this contract sends partial
// results to other rows' places, or past the end of the array; the entry point cannot check it,
// because q_start lives on the device.
//
// Sharing.  All calls on a device use the same array, and it keeps whatever the last call
// left.  Nothing in it has to start at zero: the first kernel of a call writes every slot that
// the merging kernel of the same call reads.  But two calls that overlap on the GPU (different
// streams, or graph branches that run side by side) would write the same slots and race; keep
// calls of this entry point ordered one after the other on each device.
//
// First call on a device.  The array's device address is looked up once per device
// (cudaGetSymbolAddress, with the caller's current device current) the first time the entry
// point is called on that device.  Make that first call outside any stream capture.  The table of
// addresses is filled without a lock: two threads that make the first call on a device at the
// same moment both look the address up and both store the same value.
#pragma once
#include <cuda_runtime.h>

#define DLI_NOALLOC_SCRATCH_FLOATS (1u << 20)
#define DLI_ERR_SCRATCH_TOO_SMALL 1002

#ifdef __cplusplus
extern "C" {
#endif

// Attention of num_seqs single-token sequences (sequences seq0 .. seq0 + num_seqs of the batch
// described by q_start / kv_len / block_tables) over their cache pages, keys cut into `splits`
// runs per sequence.  Same arguments and result as dli_paged_attention_mma with max_q_len = 1,
// minus the two scratch pointers.  The library is compiled for one head size (HEAD_DIM); the
// pools must have that head size.  Returns 0, a cudaError_t, DLI_ERR_UNSUPPORTED (1001) or
// DLI_ERR_SCRATCH_TOO_SMALL (1002).
int dli_paged_decode_attention_noalloc(void* out, const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                                       const int* block_tables, int max_blocks, const int* q_start, const int* kv_len, int seq0,
                                       int num_seqs, int first_row, int nh, int nkv, int page_size, int window, float scale,
                                       int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
