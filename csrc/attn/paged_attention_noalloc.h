// Allocation-free paged decode attention (no counterpart in the reference project, which has no
// native code and lets PyTorch allocate every temporary).
//
// Same computation and arguments as fi_paged_decode, minus the two partial-result buffers: the
// split-KV partials are kept in a fixed 8 MiB device array inside the library, so a caller that
// cannot allocate device memory (a plain C/C++ host without a tensor allocator, or a server whose
// memory budget is already fully committed to the KV pool) can still use split-KV decode.
//
// Limits and rules
//   * With splits > 1, B * nh * splits * (hd + 2) must not exceed 2 * 1024 * 1024 floats; otherwise the
//     call returns -20, prints the reason to stderr and launches nothing.  With splits == 1 the kernel
//     writes straight to `out`, needs no scratch, and no size limit applies.
//   * The first call on a device resolves the array's device address; make it before any stream
//     capture starts on that device.
//   * All calls share the array; calls that overlap on the GPU race.  The array keeps the previous
//     call's partials, which is harmless because every launch overwrites all partials it reads.
//   * Returns 0 on success, a negative argument code or a positive CUDA error code otherwise.
//   * dtype: 0 = bf16, 1 = fp16.  All pointers are device pointers; stream is a cudaStream_t.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

int fi_paged_decode_noalloc(const void* q, long q_stride, const void* k_cache, const void* v_cache,
                            void* out, const int* block_tables, const int* seq_lens, int B, int nh,
                            int nkv, int hd, int max_blocks, int block_size, int window,
                            float sm_scale, float softcap, int kv_fp8, float k_scale, float v_scale,
                            int splits, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
