// C declarations of entry points of libairframe_b200.so that callers outside
// this package may use directly.  (The Python package binds the whole library
// through ctypes and does not read this header.)
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Message of the last failed call on this thread.
const char* af_last_error(void);

// Floats of scratch memory that af_attn_decode needs for these sizes.
long long af_attn_decode_scratch(int batch, int nq, int hd, int n_splits);

// Decode attention over the paged bfloat16 cache (see attention_decode.cu).
// `scratch` is the caller's: af_attn_decode_scratch(...) floats of device memory.  n_splits is the most
// splits a sequence's keys are cut into (the kernel cuts each sequence by its length).  `plan`: the step's plan
// from af_attn_decode_plan for the same slots, lengths, page table, heads, window, ring and n_splits, or null
// (every block then works the cut out itself, which costs it a few loads, one after the other, before its
// first copy).
int af_attn_decode(void* out, long long out_stride, const void* q, long long q_stride, const void* kcache,
                   const void* vcache, long long n_pages, const int* page_table, int max_pages, const int* slots,
                   const int* lens, int batch, int nq, int nkv, int hd, float scale, float cap, int window,
                   int ring_rows, int n_splits, float* scratch, const int* plan, int* err, cudaStream_t stream);

// The plan of a step: how af_attn_decode cuts its work, made once for all layers that read the same caches the
// same way.  `plan`: af_attn_decode_plan_ints(...) 32-bit integers of device memory, 16-byte aligned.
long long af_attn_decode_plan_ints(int batch, int nq, int nkv);
int af_attn_decode_plan(int* plan, long long plan_ints, const int* page_table, int max_pages, const int* slots,
                        const int* lens, int batch, int nq, int nkv, int window, int ring_rows, int n_splits,
                        cudaStream_t stream);

// ---------------------------------------------------------------------------
// af_attn_decode_static: the same attention for callers that cannot allocate.
//
// This entry point has no counterpart in the reference project; it exists for
// hosts that embed the kernels and must not touch the device allocator at the
// moment they call: a serving process that has already handed all free device
// memory to its own pool (cudaMalloc would fail or fragment that pool), a
// latency-critical loop in which cudaMalloc/cudaFree are banned because they
// synchronise the whole device, or a plugin whose host forbids allocation
// calls from callbacks.  Such a caller still passes its inputs and its output
// buffer; only the scratch for the split pass's partial results is the
// library's: a file-scope device array of AF_ATTN_DECODE_STATIC_FLOATS floats
// (4 MiB) that every GPU which loads the library keeps until the process ends.
//
// The call performs no cudaMalloc, cudaFree or other allocating routine.
//
// Limits and rules:
// - batch * nq * n_splits * (hd + 2) must not exceed
//   AF_ATTN_DECODE_STATIC_FLOATS; larger requests are refused with an error
//   (af_last_error() names the sizes) and nothing is launched.  Use fewer
//   splits, or af_attn_decode with scratch of your own.
// - The first call on each device looks up the array's device address
//   (cudaGetSymbolAddress, with that device current) and keeps it.  Make that
//   first call before any stream capture begins on that device.
// - All calls share the one array, and it keeps what the last call left.
//   Nothing in it has to start at zero: the merge pass reads only elements
//   that the split pass of the same call wrote.  Two calls that overlap on the
//   GPU (different streams, or the same call issued again before the first
//   finished on another stream) race on the array and give wrong results;
//   keep calls on one stream or order them with events.
// ---------------------------------------------------------------------------
#define AF_ATTN_DECODE_STATIC_FLOATS (1 << 20)

long long af_attn_decode_static_capacity(void);

int af_attn_decode_static(void* out, long long out_stride, const void* q, long long q_stride, const void* kcache,
                          const void* vcache, long long n_pages, const int* page_table, int max_pages,
                          const int* slots, const int* lens, int batch, int nq, int nkv, int hd, float scale,
                          float cap, int window, int ring_rows, int n_splits, int* err, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
