// Host-side description of the fused collective of one GEMM call (filled by Python through ctypes).
#pragma once

extern "C" {
struct FiComm {
  int mode;              // 0 none, 1 all-reduce, 2 reduce-scatter (output rows owned by rank)
  int world;
  int rank;
  int rows_per_rank;     // reduce-scatter: rows of the output shard (multiple of the token tile)
  int xfer_16bit;        // 0: fp32 + flags, 1: 16-bit values + flags, 2: fp32 with inline epoch flags (8 B per value),
                         // 3: two-hop all-reduce (partials to the chunk owner, 16-bit result back), inline epochs
  int ag_world;          // > 1: the token operand is the concatenation of every rank's shard
  int ag_rows_per_rank;  // rows of one token shard
  int phases;            // 0 = whole collective in this launch; else a bit mask (1 push, 2 reduce, 4 collect) for the
                         // phase-by-phase emulation of several ranks on one GPU
  long slab_elems;       // elements of one (parity, source rank) receive slab
  unsigned long long recv[8];     // receive area of rank d, as mapped into this process
  unsigned long long flags[8];    // flag words of rank d
  unsigned long long ready[8];    // all-gather ready words of rank d
  unsigned long long x_peers[8];  // token shard of rank d (all-gather mode)
  unsigned long long epoch;       // local device word: completed fused calls
  unsigned long long done;        // local device word: finished CTAs of the running call
  unsigned long long trace;       // optional device array [64][8] of phase timestamps (0 = off), see trace_mark()
  unsigned long long x_full;      // all-gather mode: local staging buffer [T, K] that remote shards are copied into
                                  // once (0 = every CTA reads its token tiles from the owner's memory)
  unsigned long long ag_flags;    // local words [token tile][part]: staged copy of that part is complete
};

// Rotary embedding + KV-cache write fused into the epilogue of a merged q|k|v projection.
struct FiRope {
  const float* cos_sin;      // fp32 [max_pos, head_dim] = [cos(head_dim/2) | sin(head_dim/2)]
  const int* positions;      // [T]
  const int* slot_mapping;   // [T] flat cache slot, < 0 = skip
  void* k_cache;             // [blocks, num_kv_heads, block_size, head_dim], same 16-bit type as the output
  void* v_cache;
  int num_heads, num_kv_heads, head_dim, block_size;
};

// Grouped (mixture-of-experts) launch: activations are sorted by expert, a device-side tile table
// (built by fi_moe_align) tells each CTA its expert and rows; weights of all experts are stacked.
struct FiGrouped {
  const int* tile_expert;
  const int* tile_row0;
  const int* tile_rows;
  const int* n_tiles;
  int max_tiles;       // grid size along the tile axis (upper bound of *n_tiles)
  int num_experts;     // experts stacked in the weight tensor
  int expert_rows;     // weight rows per expert (N, or 2N in gated mode)
  int reserved;
};
}
