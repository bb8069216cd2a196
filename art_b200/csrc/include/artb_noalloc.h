// Entry points of libartb_kernels.so that perform no device or host allocation.
//
// This header has no counterpart in the reference project (which ships no native code at all);
// it exists for embedders of this library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest split-KV workspace the allocation-free decode entry point can serve, in floats
// (16 MiB of device memory, held by every GPU that loads the library until the process exits).
#define ARTB_DECODE_STATIC_WS_FLOATS (4 * 1024 * 1024)

// Paged-KV decode attention with split-KV whose scratch workspace is a fixed device array inside
// the library instead of caller- or library-allocated memory.
//
// Who needs this: callers that must not allocate.  Typical cases are a serving process that has
// handed all remaining device memory to its KV-cache arena (a cudaMalloc would fail or fragment
// it), and latency-critical loops that cannot afford the implicit device-wide synchronisation a
// cudaMalloc / cudaFree may perform.  The function calls no cudaMalloc, cudaFree or any other
// allocating routine, of CUDA or of PyTorch; inputs and outputs are the caller's.
//
// Same arguments and results as artb_paged_decode(), minus the workspace pointer:
//   q [num_seqs, ldq] bf16 (first Hq*hd columns used), k_cache / v_cache [blocks, block_size, Hkv, hd] bf16,
//   block_table int32 [num_seqs, max_blocks], ctx_len int32 [num_seqs], out [num_seqs, ldo] bf16.
// Limits: num_seqs * Hq * splits * (hd + 2) <= ARTB_DECODE_STATIC_WS_FLOATS, otherwise the call
// returns -5 ("size beyond the supported maximum") and launches nothing.
//
// The first call on a device resolves the device address of the internal array (with that
// device current); make that first call before starting any stream capture.
// All calls on one device share the one array: two calls whose kernels can overlap on the GPU
// (different streams, no ordering between them) race on it.  The array keeps whatever the last
// call left there; this kernel overwrites every slot it later reads, so nothing needs clearing.
int artb_paged_decode_noalloc(const void* q, int ldq, const void* k_cache, const void* v_cache,
                              const int* block_table, int max_blocks, const int* ctx_len, int block_size,
                              int num_seqs, int Hq, int Hkv, int hd, void* out, int ldo, int splits,
                              cudaStream_t stream);

#ifdef __cplusplus
}
#endif
