// Shared epilogue of the tcgen05 GEMM kernels (dense 16-bit and int4 weight-only).
//
// Part 1 (four epilogue warps): accumulator TMEM -> fp32 staging tile in shared memory, laid out
//   [token][weight row].
// Part 2 (all threads): split-K reduction of the cluster's partial tiles through distributed shared
//   memory, then EITHER the local epilogue (activation, bias, residual, store) OR the fused
//   collective: the reduced partial rows are pushed with plain peer stores over NVLink into the
//   receive area of every other rank (all-reduce) or of the owning rank (reduce-scatter), a
//   per-(tile, source rank, cluster part) flag word is released with the call's epoch, the CTA waits
//   (bounded) for the matching flags of its peers, sums the partials in rank order (bitwise identical
//   on every rank), adds bias/residual and stores.  One kernel = GEMM + collective + residual.
//
// Collective bookkeeping lives on the device so CUDA-graph replays work: `epoch` counts completed
// fused calls (every rank runs the same call sequence), the last CTA of a call bumps it; receive
// slabs are double-buffered by epoch parity, which is enough because a rank cannot finish call k+1
// before every peer has pushed its call-k+1 partials, i.e. after those peers finished reading call k.
#pragma once
#include <cooperative_groups.h>

#include "../common/ptx.cuh"

namespace fi {

constexpr int BM = 128;  // weight rows per CTA
constexpr int BK = 64;   // 64 x 16-bit = one 128-byte swizzle row
constexpr int kThreads = 192;
constexpr int kMaxRanks = 8;
constexpr int kFlagParts = 8;       // flag words per (tile, source rank): one per cluster part
constexpr int kXferInlineFlags = 2;  // GemmParams::xfer_16bit value: fp32 values with the epoch in every 8-byte word
constexpr int kXferTwoShot = 3;      // all-reduce in two hops: partials go to the chunk's owner, the owner sends the result
// Phases of a fused collective (GemmParams::comm_phases, 0 = all).  A real call runs all of them in one
// launch; a single-GPU emulation of several ranks launches phase by phase, all ranks per phase, because
// launches on one GPU cannot wait for one another.
constexpr int kPhasePush = 1, kPhaseReduce = 2, kPhaseCollect = 4;
constexpr int kMaxCommTiles = 8192; // tiles per call that the flag area can describe

enum Act : int { kActNone = 0, kActSilu = 1, kActGeluTanh = 2 };
enum CommMode : int { kCommNone = 0, kCommAllReduce = 1, kCommReduceScatter = 2 };

struct GemmParams {
  void* C;
  const void* bias;      // [N] or null (same 16-bit type as X)
  const void* residual;  // [T, ldc] or null (same type as C when C is 16-bit)
  int T, N, K;
  int ldc;
  int dual_rows;  // > 0: gated mode, W = [2 * dual_rows, K]; N == dual_rows
  int act;
  int out_fp32;
  int is_fp16;
  int splits;
  int* status;
  // fused RMSNorm of the token operand (rms_eps > 0): out = (W' . x) * rsqrt(mean(x^2) + eps) with the
  // norm weight folded into W' at load time; the sum of squares is taken from the token tiles in
  // shared memory while the main loop runs
  float rms_eps;
  int w_dynamic;         // 1: the weight operand was written by the preceding kernel (no prefetch before the PDL wait)
  // int4 weight-only extras (unused by the dense kernel)
  const void* scales;   // [K/G, rows]
  const uint8_t* zeros; // [K/G, rows] or null
  int group;
  int n_rows_total;
  // fused collective (comm_mode != 0) and all-gathered token operand (ag_world > 1)
  int comm_mode;
  int world, rank;
  int rows_per_rank;     // reduce-scatter: token t belongs to rank t / rows_per_rank
  int xfer_16bit;        // 0: fp32 + flags, 1: 16-bit values + flags, 2: fp32 with inline epoch flags (8 B per value),
                         // 3: two-hop all-reduce with inline epochs (see epilogue_two_shot)
  int comm_phases;       // bit mask of kPhase*; 0 = every phase in this launch
  int ag_world;          // > 1: token tile t0 is read from rank t0 / ag_rows_per_rank
  int ag_rows_per_rank;
  long slab_elems;       // elements of one (parity, source) receive slab
  unsigned long long recv[kMaxRanks];   // receive area of rank d as mapped in this process
  unsigned long long flags[kMaxRanks];  // flag words of rank d as mapped in this process
  unsigned long long ready[kMaxRanks];  // all-gather ready words of rank d as mapped here
  unsigned int* epoch;   // local: completed fused calls
  unsigned long long* trace;   // optional phase timestamps of CTA (0,0,0): [epoch % 64][8]
  unsigned int* done;    // local: CTAs of the current call that have finished
  // rotary embedding + KV-cache write fused behind a merged q|k|v projection (rope_cs != nullptr):
  // the epilogue rotates q and k (pairs d, d + hd/2, full-width rotary), stores q|k|v into C and the
  // new k and v rows into the paged cache [blocks, nkv, block_size, hd] (same 16-bit type as C)
  const float* rope_cs;    // [max_pos, hd] = [cos(hd/2) | sin(hd/2)]
  const int* rope_pos;     // [T]
  const int* rope_slots;   // [T] flat cache slot (block * block_size + offset), < 0 = do not cache
  void* k_cache;
  void* v_cache;
  int rope_nh, rope_nkv, rope_hd, rope_bs;
  // staged all-gather: the first copy_rows rows of the grid (blockIdx.y) are copier CTAs that pull
  // the peers' token shards into x_full once; GEMM CTAs read remote tiles from there
  unsigned long long x_peers[kMaxRanks];   // token shard of rank d as mapped here
  void* x_full;
  unsigned int* ag_flags;
  int copy_rows;
  // grouped (mixture-of-experts) mode: blockIdx.y indexes a tile table built on the device
  const int* tile_expert;   // expert of each token tile (null = plain GEMM)
  const int* tile_row0;     // first row of the tile in the expert-sorted activation matrix
  const int* tile_rows;     // valid rows of the tile
  const int* n_tiles;       // number of valid tiles (CTAs beyond it leave at once)
  int expert_rows;          // weight rows per expert (N, or 2N in gated mode)
  int grid_tiles;           // grid size along y in grouped mode (0 = derive from T)
};

constexpr int kStagedMap = kMaxRanks;   // TokenMaps slot of the locally staged, gathered token matrix
constexpr int kAgParts = 8;             // copy units (and flags) per staged token tile
struct TokenMaps {
  CUtensorMap m[kMaxRanks + 1];
};

__device__ __forceinline__ float apply_act(float g, int act) {
  if (act == kActSilu) return g / (1.f + __expf(-g));
  if (act == kActGeluTanh) {
    const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return g / (1.f + __expf(-2.f * inner));
  }
  return g;
}

__device__ __forceinline__ float ld16_as_float(const void* p, size_t i, int is_fp16) {
  if (is_fp16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Debug aid: CTA (0,0,0) records the global timer at a few phases of a fused call when the caller
// passed a trace array (phase 0 start, 1 accumulators staged, 2 partials pushed, 3 peers' flags
// seen, 4 reduced tile stored, 5 exit).
__device__ __forceinline__ void trace_mark(unsigned long long* trace, unsigned int epoch_now, int phase) {
  if (trace != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    trace[(epoch_now & 63u) * 8 + phase] = t;
  }
}
// Debug aid for plain (non-collective) GEMM calls: CTA (0,0,0) records its SM cycle counter at up to
// eight points of its life into trace[0..7] (all marks come from the same SM, so differences are
// cycles).  0 entry, 1 set-up done, 2 predecessor grid complete, 3 accumulator ready, 4 accumulator
// staged in shared memory, 5 split-K cluster met, 6 tile stored, 7 exit.
__device__ __forceinline__ void cycle_mark(unsigned long long* trace, bool comm, int phase) {
  if (trace != nullptr && !comm && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)
    trace[phase] = static_cast<unsigned long long>(clock64());
}

// Bounded wait for a flag word to reach `want` (epochs only grow).
// `status` (optional): the call's status word; once any wait of the process has timed out, later
// waits give up after a short grace period instead of a full budget each, so a broken exchange ends
// in about one budget overall rather than one per tile.
__device__ __forceinline__ bool wait_flag(const unsigned int* p, unsigned int want, const int* status = nullptr) {
  const long long t0 = clock64();
  long long budget = FI_WAIT_CYCLES;
  unsigned int spins = 0;
  while (static_cast<int>(ld_acquire_sys(p) - want) < 0) {
    if (clock64() - t0 > budget) return false;
    if (status != nullptr && (++spins & 1023u) == 0 &&
        *reinterpret_cast<const volatile int*>(status) != 0)
      budget = FI_WAIT_CYCLES >> 10;
  }
  return true;
}

__device__ __forceinline__ void pack8(const float* g, int is_fp16, uint32_t* packed) {
  if (is_fp16) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2 h = __floats2half2_rn(g[2 * j], g[2 * j + 1]);
      packed[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(g[2 * j], g[2 * j + 1]);
      packed[j] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
}
__device__ __forceinline__ void unpack8(const uint4 raw, int is_fp16, float* g) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (is_fp16) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      g[2 * j] = f.x; g[2 * j + 1] = f.y;
    } else {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
      g[2 * j] = f.x; g[2 * j + 1] = f.y;
    }
  }
}

// Bias + residual + store of 8 consecutive outputs of token row `trow` (row index in C).
__device__ __forceinline__ void finalize_store8(const GemmParams& p, float* g, int trow, int n) {
  const int nvalid = min(8, p.N - n);
  if (p.bias != nullptr) {
    for (int j = 0; j < nvalid; ++j) g[j] += ld16_as_float(p.bias, n + j, p.is_fp16);
  }
  const size_t off = static_cast<size_t>(trow) * p.ldc + n;
  if (p.out_fp32) {
    float* C = reinterpret_cast<float*>(p.C);
    if (p.residual != nullptr)
      for (int j = 0; j < nvalid; ++j) g[j] += reinterpret_cast<const float*>(p.residual)[off + j];
    if (nvalid == 8) {
      *reinterpret_cast<float4*>(C + off) = make_float4(g[0], g[1], g[2], g[3]);
      *reinterpret_cast<float4*>(C + off + 4) = make_float4(g[4], g[5], g[6], g[7]);
    } else {
      for (int j = 0; j < nvalid; ++j) C[off + j] = g[j];
    }
  } else {
    if (p.residual != nullptr)
      for (int j = 0; j < nvalid; ++j) g[j] += ld16_as_float(p.residual, off + j, p.is_fp16);
    uint32_t packed[4];
    pack8(g, p.is_fp16, packed);
    uint16_t* C = reinterpret_cast<uint16_t*>(p.C);
    if (nvalid == 8) {
      *reinterpret_cast<uint4*>(C + off) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    } else {
      const uint16_t* ph = reinterpret_cast<const uint16_t*>(packed);
      for (int j = 0; j < nvalid; ++j) C[off + j] = ph[j];
    }
  }
}

// Re-read one (value, epoch, value, epoch) word until both epochs match the running call.  Bounded:
// gives up after the cycle budget (or shortly after any other wait of the process has failed), records
// the status and raises the CTA's abort flag.
__device__ __forceinline__ bool poll_epoch_word(const uint4* src, unsigned int epoch_now, uint4& w,
                                                volatile int* aborted, int* status, long long t0) {
  while (w.y != epoch_now || w.w != epoch_now) {
    if (*aborted || clock64() - t0 > FI_WAIT_CYCLES ||
        (status != nullptr && clock64() - t0 > (FI_WAIT_CYCLES >> 10) &&
         *reinterpret_cast<const volatile int*>(status) != 0)) {
      set_status(status, kStatusTimeoutPeer);
      *aborted = 1;
      return false;
    }
    w = ld_volatile_v4(src);
  }
  return true;
}

// Two-hop all-reduce of a decode-sized tile (xfer_16bit == kXferTwoShot, 16-bit output).
//
// The 16 eight-value chunks of a tile row are dealt to the ranks round robin (chunk c belongs to rank
// c % world).  Hop 1 (done by the caller's first pass): every rank stores its fp32 partial of a chunk
// into the OWNER's receive slab, each 8-byte word carrying the call's epoch.  Hop 2 (here): the owner
// sums the world partials in rank order, finishes the epilogue (activation, bias, residual), stores
// the 16-bit result locally and sends it to every peer, again with inline epochs; the peers copy it
// into their output.  Per rank and tile this moves 2 * (world - 1) / world of the tile instead of
// (world - 1) tiles, and a thread polls a handful of independent words instead of a chain of
// world - 1 dependent ones.  The result words reuse slots of the sender's slab that hop 1 never writes
// (a rank does not send its own chunks to anybody), so the slab layout is that of the one-hop form.
template <int BN>
__device__ __forceinline__ void epilogue_two_shot(const GemmParams& p, const float* stage_f32, volatile int* aborted,
                                                  int n0, int t0, unsigned int epoch_now, int t_end, int S,
                                                  int crank, int rows_mine, int phases, int act_after_sum) {
  const int W = p.world, me = p.rank;
  const int parity = static_cast<int>(epoch_now & 1u);
  const int own_per_row = (BM / 8 - me + W - 1) / W;
  if (!*aborted && (phases & kPhaseReduce)) {
    const int items = rows_mine * own_per_row * 2;       // (row, owned chunk, half chunk of 4 values)
    for (int idx = threadIdx.x; idx < items; idx += blockDim.x) {
      const int half = idx & 1;
      const int j = (idx >> 1) % own_per_row;
      const int tl = crank + ((idx >> 1) / own_per_row) * S;
      const int nl = (me + j * W) * 8 + half * 4;
      const int t = t0 + tl, n = n0 + nl;
      if (t >= t_end || n >= p.N) continue;
      const long pos = static_cast<long>(t) * p.N + n;
      uint4 w[kMaxRanks][2];
      const long long w0 = clock64();
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s < W && s != me) {
          const uint4* src = reinterpret_cast<const uint4*>(p.recv[me]) +
                             (((static_cast<long>(parity) * W + s) * p.slab_elems + pos) >> 1);
          w[s][0] = ld_volatile_v4(src);
          w[s][1] = ld_volatile_v4(src + 1);
        }
      }
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      bool ok = true;
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s >= W) continue;
        if (s == me) {
          const float4 a = *reinterpret_cast<const float4*>(stage_f32 + tl * BM + nl);
          acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        } else {
          const uint4* src = reinterpret_cast<const uint4*>(p.recv[me]) +
                             (((static_cast<long>(parity) * W + s) * p.slab_elems + pos) >> 1);
          ok = ok && poll_epoch_word(src, epoch_now, w[s][0], aborted, p.status, w0) &&
               poll_epoch_word(src + 1, epoch_now, w[s][1], aborted, p.status, w0);
          acc[0] += __uint_as_float(w[s][0].x); acc[1] += __uint_as_float(w[s][0].z);
          acc[2] += __uint_as_float(w[s][1].x); acc[3] += __uint_as_float(w[s][1].z);
        }
      }
      if (!ok) break;
      if (act_after_sum) {
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q] = apply_act(acc[q], p.act);
      }
      const size_t coff = static_cast<size_t>(t) * p.ldc + n;
      if (p.bias != nullptr) {
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q] += ld16_as_float(p.bias, n + q, p.is_fp16);
      }
      if (p.residual != nullptr) {
        const uint2 r2 = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p.residual) + coff);
        float r[8];
        unpack8(make_uint4(r2.x, r2.y, 0u, 0u), p.is_fp16, r);
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[q] += r[q];
      }
      float g8[8] = {acc[0], acc[1], acc[2], acc[3], 0.f, 0.f, 0.f, 0.f};
      uint32_t pk[4];
      pack8(g8, p.is_fp16, pk);
      *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.C) + coff) = make_uint2(pk[0], pk[1]);
      const long roff = ((static_cast<long>(parity) * W + me) * p.slab_elems + pos) >> 1;
      const uint4 word = make_uint4(pk[0], epoch_now, pk[1], epoch_now);
#pragma unroll
      for (int d = 0; d < kMaxRanks; ++d)
        if (d < W && d != me) st_volatile_v4(reinterpret_cast<uint4*>(p.recv[d]) + roff, word);
    }
  }
  if (!*aborted && (phases & kPhaseCollect)) {
    const int items = rows_mine * (BM / 8);
    for (int idx = threadIdx.x; idx < items; idx += blockDim.x) {
      const int c = idx % (BM / 8);
      const int owner = c % W;
      if (owner == me) continue;
      const int tl = crank + (idx / (BM / 8)) * S;
      const int t = t0 + tl, n = n0 + c * 8;
      if (t >= t_end || n >= p.N) continue;
      const long pos = static_cast<long>(t) * p.N + n;
      const uint4* src = reinterpret_cast<const uint4*>(p.recv[me]) +
                         (((static_cast<long>(parity) * W + owner) * p.slab_elems + pos) >> 1);
      const long long w0 = clock64();
      uint4 a = ld_volatile_v4(src), b = ld_volatile_v4(src + 2);
      if (!poll_epoch_word(src, epoch_now, a, aborted, p.status, w0) ||
          !poll_epoch_word(src + 2, epoch_now, b, aborted, p.status, w0))
        break;
      *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.C) + static_cast<size_t>(t) * p.ldc + n) =
          make_uint4(a.x, a.z, b.x, b.z);
    }
  }
}

// Part 1: warps 2..5.  Returns false when the accumulator never arrived.
template <int BN, bool DUAL>
__device__ __forceinline__ void epilogue_tmem_to_smem(const GemmParams& p, uint64_t* accum_bar,
                                                      uint32_t tmem_base, float* stage_f32,
                                                      volatile int* aborted, int warp, int lane,
                                                      const float* row_ss = nullptr) {
  bool ok = mbar_wait(accum_bar, 0);
  if (!ok) {
    set_status(p.status, kStatusTimeoutAccum);
    *aborted = 1;
  }
  if (warp == 2 && lane == 0) cycle_mark(p.trace, p.comm_mode != kCommNone, 3);
  tc_fence_after();
  const int q = warp & 3;  // TMEM lane quarter this warp may read
  const int n_local = q * 32 + lane;
  const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
  if (ok) {
    const bool fuse_act_now = DUAL && (p.splits == 1);
    const bool norm_now = p.rms_eps > 0.f && p.splits == 1;   // with split-K the scale is applied after the sum
    const float inv_k = 1.f / static_cast<float>(p.K);
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
      uint32_t r[16];
      tmem_ld_x16(taddr + c0, r);
      if (norm_now) {
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j)
          r[j] = __float_as_uint(__uint_as_float(r[j]) * rsqrtf(row_ss[c0 + j] * inv_k + p.rms_eps));
      }
      if (DUAL) {
        uint32_t u[16];
        tmem_ld_x16(taddr + BN + c0, u);
        tmem_ld_wait();
        if (norm_now) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            u[j] = __float_as_uint(__uint_as_float(u[j]) * rsqrtf(row_ss[c0 + j] * inv_k + p.rms_eps));
        }
        if (fuse_act_now) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            stage_f32[(c0 + j) * BM + n_local] =
                apply_act(__uint_as_float(r[j]), p.act) * __uint_as_float(u[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            stage_f32[(c0 + j) * BM + n_local] = __uint_as_float(r[j]);
            stage_f32[BN * BM + (c0 + j) * BM + n_local] = __uint_as_float(u[j]);
          }
        }
      } else {
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) stage_f32[(c0 + j) * BM + n_local] = __uint_as_float(r[j]);
      }
    }
  }
  tc_fence_before();
}

// Part 2: every thread of the CTA.  Must be called by all CTAs of the cluster (it contains the
// cluster barriers).  `n0`, `t0`: first weight row / token of the tile.
template <int BN, bool DUAL>
__device__ __forceinline__ void epilogue_reduce_store(const GemmParams& p, float* stage_f32,
                                                      volatile int* aborted, int n0, int t0,
                                                      unsigned int epoch_now, int t_end,
                                                      float* row_ss = nullptr) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int S = p.splits;
  const int rank = (S > 1) ? static_cast<int>(blockIdx.z) : 0;   // rank inside the split-K cluster
  const bool comm = p.comm_mode != kCommNone;
  if (threadIdx.x == 0) cycle_mark(p.trace, comm, 4);
  if (S > 1) cluster.sync();
  if (threadIdx.x == 0) cycle_mark(p.trace, comm, 5);
  const int phases = p.comm_phases != 0 ? p.comm_phases : (kPhasePush | kPhaseReduce | kPhaseCollect);
  const bool two_shot = comm && p.xfer_16bit == kXferTwoShot;
  const int rows_mine = (BN - rank + S - 1) / S;
  const int owner = p.comm_mode == kCommReduceScatter ? t0 / p.rows_per_rank : -1;
  const int parity = static_cast<int>(epoch_now & 1u);
  const int row_base = p.comm_mode == kCommReduceScatter ? p.rank * p.rows_per_rank : 0;
  if (comm) trace_mark(p.trace, epoch_now, 1);
  // does this CTA send its tile to anybody?  (reduce-scatter: only tiles owned by another rank)
  const bool i_own_tile = owner < 0 || owner == p.rank;
  const bool pushes = comm && (owner < 0 ? p.world > 1 : owner != p.rank);
  // an owned tile without split-K has nothing to do before the final sum: its partial already sits
  // in the staging tile and nobody else wants it
  const bool skip_first_pass = comm && S == 1 && !pushes;

  if (!*aborted && !skip_first_pass) {
    for (int idx = threadIdx.x; idx < rows_mine * (BM / 8); idx += blockDim.x) {
      const int tl = rank + (idx / (BM / 8)) * S;
      const int nl = (idx % (BM / 8)) * 8;
      const int t = t0 + tl;
      const int n = n0 + nl;
      if (t >= t_end || n >= p.N) continue;
      float g[8], u[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { g[j] = 0.f; u[j] = 0.f; }
      for (int pr = 0; pr < S; ++pr) {
        const float* src = (S > 1) ? cluster.map_shared_rank(stage_f32, pr) : stage_f32;
        const float4 a = *reinterpret_cast<const float4*>(src + tl * BM + nl);
        const float4 b = *reinterpret_cast<const float4*>(src + tl * BM + nl + 4);
        g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w;
        g[4] += b.x; g[5] += b.y; g[6] += b.z; g[7] += b.w;
        if (DUAL && S > 1) {
          const float4 c = *reinterpret_cast<const float4*>(src + BN * BM + tl * BM + nl);
          const float4 d = *reinterpret_cast<const float4*>(src + BN * BM + tl * BM + nl + 4);
          u[0] += c.x; u[1] += c.y; u[2] += c.z; u[3] += c.w;
          u[4] += d.x; u[5] += d.y; u[6] += d.z; u[7] += d.w;
        }
      }
      if (p.rms_eps > 0.f && S > 1) {
        float ss = 0.f;
        for (int pr = 0; pr < S; ++pr) ss += cluster.map_shared_rank(row_ss, pr)[tl];
        const float rstd = rsqrtf(ss / static_cast<float>(p.K) + p.rms_eps);
#pragma unroll
        for (int j = 0; j < 8; ++j) { g[j] *= rstd; u[j] *= rstd; }
      }
      if (DUAL && S > 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = apply_act(g[j], p.act) * u[j];
      } else if (!DUAL && p.act != kActNone && !comm) {
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = apply_act(g[j], p.act);
      }
      if (!comm) {
        if (p.rope_cs != nullptr) {   // park the finished values (with bias); the rotary pass below pairs them up
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] += ld16_as_float(p.bias, n + j, p.is_fp16);
          }
          *reinterpret_cast<float4*>(stage_f32 + tl * BM + nl) = make_float4(g[0], g[1], g[2], g[3]);
          *reinterpret_cast<float4*>(stage_f32 + tl * BM + nl + 4) = make_float4(g[4], g[5], g[6], g[7]);
        } else {
          finalize_store8(p, g, t, n);
        }
        continue;
      }
      // ---- fused collective, phase A: keep my partial in my own staging rows (only needed when it
      // was just reduced over the split-K cluster and this CTA does the final sum), push it to peers
      if (S > 1 && i_own_tile) {
        *reinterpret_cast<float4*>(stage_f32 + tl * BM + nl) = make_float4(g[0], g[1], g[2], g[3]);
        *reinterpret_cast<float4*>(stage_f32 + tl * BM + nl + 4) = make_float4(g[4], g[5], g[6], g[7]);
      }
      const long trow = (p.comm_mode == kCommReduceScatter) ? (t - owner * p.rows_per_rank) : t;
      const long off = (static_cast<long>(parity) * p.world + p.rank) * p.slab_elems + trow * p.N + n;
      if (!(phases & kPhasePush)) continue;
      if (two_shot) {   // hop 1: the partial of this chunk goes to the chunk's owner only
        const int own = (nl >> 3) % p.world;
        if (own != p.rank) {
          uint4* dst = reinterpret_cast<uint4*>(p.recv[own]) + (off >> 1);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            st_volatile_v4(dst + q, make_uint4(__float_as_uint(g[2 * q]), epoch_now,
                                               __float_as_uint(g[2 * q + 1]), epoch_now));
        }
        continue;
      }
      for (int d = 0; d < p.world; ++d) {
        if (d == p.rank || (owner >= 0 && d != owner)) continue;
        if (p.xfer_16bit == kXferInlineFlags) {
          // low-latency form: every 8-byte word carries one fp32 value and the epoch, so the
          // receiver needs no fence and no separate flag (one NVLink crossing instead of three)
          uint4* dst = reinterpret_cast<uint4*>(p.recv[d]) + (off >> 1);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            st_volatile_v4(dst + q, make_uint4(__float_as_uint(g[2 * q]), epoch_now,
                                               __float_as_uint(g[2 * q + 1]), epoch_now));
        } else if (p.xfer_16bit) {
          uint32_t packed[4];
          pack8(g, p.is_fp16, packed);
          *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.recv[d]) + off) =
              make_uint4(packed[0], packed[1], packed[2], packed[3]);
        } else {
          float* dst = reinterpret_cast<float*>(p.recv[d]) + off;
          *reinterpret_cast<float4*>(dst) = make_float4(g[0], g[1], g[2], g[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(g[4], g[5], g[6], g[7]);
        }
      }
    }
  }
  if (p.rope_cs != nullptr && !comm) {
    __syncthreads();
    if (!*aborted) {
      const int hd = p.rope_hd, half = hd >> 1;
      const int q_end = p.rope_nh * hd, k_end = q_end + p.rope_nkv * hd;
      for (int idx = threadIdx.x; idx < rows_mine * (BM / 8); idx += blockDim.x) {
        const int tl = rank + (idx / (BM / 8)) * S;
        const int nl = (idx % (BM / 8)) * 8;
        const int t = t0 + tl;
        const int n = n0 + nl;
        if (t >= t_end || n >= p.N) continue;
        const float* own = stage_f32 + tl * BM + nl;
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = own[j];
        const int sec = n < q_end ? 0 : (n < k_end ? 1 : 2);
        if (sec != 2) {
          const int d = n & (hd - 1);
          const bool lower = d < half;
          const float* other = lower ? own + half : own - half;
          const float* cs = p.rope_cs + static_cast<size_t>(p.rope_pos[t]) * hd + (d & (half - 1));
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float c = cs[j], sn = cs[half + j];
            x[j] = lower ? x[j] * c - other[j] * sn : x[j] * c + other[j] * sn;
          }
        }
        uint32_t packed[4];
        pack8(x, p.is_fp16, packed);
        const uint4 v16 = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.C) + static_cast<size_t>(t) * p.ldc + n) = v16;
        if (sec != 0) {
          const int slot = p.rope_slots[t];
          if (slot >= 0) {
            const int blk = slot / p.rope_bs, off = slot - blk * p.rope_bs;
            const int hn = n - (sec == 1 ? q_end : k_end);
            const size_t addr = ((static_cast<size_t>(blk) * p.rope_nkv + hn / hd) * p.rope_bs + off) * hd + (hn & (hd - 1));
            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(sec == 1 ? p.k_cache : p.v_cache) + addr) = v16;
          }
        }
      }
    }
  }
  if (comm) trace_mark(p.trace, epoch_now, 2);
  if (threadIdx.x == 0) cycle_mark(p.trace, comm, 6);
  if (comm) {
    const unsigned int tile = static_cast<unsigned int>(t0 / BN) * gridDim.x + blockIdx.x;
    const bool inline_flags = p.xfer_16bit == kXferInlineFlags || two_shot;
    if (!inline_flags && pushes) __threadfence_system();
    __syncthreads();
    const bool i_own = i_own_tile;
    if (!inline_flags && !*aborted && threadIdx.x < p.world && static_cast<int>(threadIdx.x) != p.rank) {
      const int d = threadIdx.x;
      if ((owner < 0 || d == owner) && (phases & kPhasePush)) {
        unsigned int* f = reinterpret_cast<unsigned int*>(p.flags[d]) +
                          (static_cast<size_t>(tile) * p.world + p.rank) * kFlagParts + rank;
        st_release_sys(f, epoch_now);
      }
      if (i_own && (phases & kPhaseReduce)) {
        const unsigned int* mine = reinterpret_cast<const unsigned int*>(p.flags[p.rank]) +
                                   (static_cast<size_t>(tile) * p.world + d) * kFlagParts + rank;
        if (!wait_flag(mine, epoch_now, p.status)) {
          set_status(p.status, kStatusTimeoutPeer);
          *aborted = 1;
        }
      }
    }
    __syncthreads();
    trace_mark(p.trace, epoch_now, 3);
    if (two_shot)
      epilogue_two_shot<BN>(p, stage_f32, aborted, n0, t0, epoch_now, t_end, S, rank, rows_mine, phases,
                            !DUAL && p.act != kActNone);
    // ---- phase C: sum the partials of all ranks in rank order, finish the epilogue, store
    if (!two_shot && !*aborted && i_own && (phases & kPhaseReduce)) {
      for (int idx = threadIdx.x; idx < rows_mine * (BM / 8); idx += blockDim.x) {
        const int tl = rank + (idx / (BM / 8)) * S;
        const int nl = (idx % (BM / 8)) * 8;
        const int t = t0 + tl;
        const int n = n0 + nl;
        if (t >= t_end || n >= p.N) continue;
        const long trow = t - row_base;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int s = 0; s < p.world; ++s) {
          float v[8];
          if (s == p.rank) {
            const float4 a = *reinterpret_cast<const float4*>(stage_f32 + tl * BM + nl);
            const float4 b = *reinterpret_cast<const float4*>(stage_f32 + tl * BM + nl + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            if (p.xfer_16bit == 1) {   // round my own partial like the ones that crossed the link
              uint32_t packed[4];
              pack8(v, p.is_fp16, packed);
              unpack8(make_uint4(packed[0], packed[1], packed[2], packed[3]), p.is_fp16, v);
            }
          } else {
            const long off = (static_cast<long>(parity) * p.world + s) * p.slab_elems + trow * p.N + n;
            if (inline_flags) {
              const uint4* src = reinterpret_cast<const uint4*>(p.recv[p.rank]) + (off >> 1);
              const long long w0 = clock64();
              uint4 wv[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) wv[q] = ld_volatile_v4(src + q);   // four independent loads in flight
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                poll_epoch_word(src + q, epoch_now, wv[q], aborted, p.status, w0);
                v[2 * q] = __uint_as_float(wv[q].x);
                v[2 * q + 1] = __uint_as_float(wv[q].z);
              }
            } else if (p.xfer_16bit) {
              unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.recv[p.rank]) + off),
                      p.is_fp16, v);
            } else {
              const float* src = reinterpret_cast<const float*>(p.recv[p.rank]) + off;
              const float4 a = *reinterpret_cast<const float4*>(src);
              const float4 b = *reinterpret_cast<const float4*>(src + 4);
              v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += v[j];
        }
        if (!DUAL && p.act != kActNone) {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = apply_act(acc[j], p.act);
        }
        if (!*aborted) finalize_store8(p, acc, static_cast<int>(trow), n);
      }
    }
  }
  if ((comm || p.ag_world > 1) && (!comm || (phases & (two_shot ? kPhaseCollect : kPhaseReduce)))) {
    // the last CTA of the call publishes the new epoch for the next fused call (in a phase-by-phase
    // emulation only the launch that runs the call's last phase does)
    __syncthreads();
    trace_mark(p.trace, epoch_now, 4);
    if (threadIdx.x == 0) {
      const unsigned int total = gridDim.x * gridDim.y * gridDim.z;
      __threadfence();
      if (atomicAdd(p.done, 1u) == total - 1) {
        *p.done = 0;
        __threadfence();
        *reinterpret_cast<volatile unsigned int*>(p.epoch) = epoch_now;
      }
    }
  }
  if (S > 1) cluster.sync();  // nobody leaves while a peer may still read its staging tile
  if (comm) trace_mark(p.trace, epoch_now, 5);
  if (threadIdx.x == 0) cycle_mark(p.trace, comm, 7);
}

// Order in which the token tiles of a fused collective are worked on (blockIdx.y -> tile index).
// Reduce-scatter: every rank starts with the tiles owned by the NEXT rank and ends with its own, so
// the partials a rank has to wait for were produced first everywhere and have crossed NVLink by the
// time it reaches its own tiles.  All-gather: own shard first, the peers' shards (which have to be
// fetched) afterwards.  Only when the token count is exactly world * rows_per_rank.
template <int BN>
__device__ __forceinline__ int token_tile_index(const GemmParams& p, int y) {
  if (p.comm_mode == kCommReduceScatter && p.rows_per_rank % BN == 0 && p.T == p.world * p.rows_per_rank) {
    const int per = p.rows_per_rank / BN;
    return (y + (p.rank + 1) * per) % (p.world * per);
  }
  if (p.ag_world > 1 && p.ag_rows_per_rank % BN == 0 && p.T == p.ag_world * p.ag_rows_per_rank) {
    const int per = p.ag_rows_per_rank / BN;
    return (y + p.rank * per) % (p.ag_world * per);
  }
  return y;
}

// Source of the token tile starting at token t0: which tensor map and which row inside it.
__device__ __forceinline__ void token_tile_source(const GemmParams& p, int t0, int* map_idx, int* row) {
  if (p.ag_world > 1) {
    *map_idx = t0 / p.ag_rows_per_rank;
    *row = t0 - (*map_idx) * p.ag_rows_per_rank;
    if (p.x_full != nullptr && *map_idx != p.rank) {   // remote shard: read the local staged copy
      *map_idx = kStagedMap;
      *row = t0;
    }
  } else {
    *map_idx = 0;
    *row = t0;
  }
}

// All-gather handshake run by the TMA producer thread before its first remote load: CTA (0,0,0)
// tells every peer that this rank's token shard of the current call is complete; every producer
// waits (bounded) until the rank it reads from has said the same.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Staged all-gather, consumer side: wait until every part of the token tile at t0 has been copied.
template <int BN>
__device__ __forceinline__ bool ag_wait_staged(const GemmParams& p, int t0, unsigned int epoch_now) {
  const unsigned int* f = p.ag_flags + static_cast<size_t>(t0 / BN) * kAgParts;
  for (int i = 0; i < kAgParts; ++i) {
    const long long w0 = clock64();
    unsigned int v;
    do {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f + i) : "memory");
      if (v == epoch_now) break;
      if (p.status != nullptr && clock64() - w0 > (FI_WAIT_CYCLES >> 10) &&
          *reinterpret_cast<const volatile int*>(p.status) != 0) break;
    } while (clock64() - w0 <= FI_WAIT_CYCLES);
    if (v != epoch_now) return false;
  }
  fence_proxy_async_all();   // the copy was made with generic stores; the TMA engine reads it next
  return true;
}

// Staged all-gather, copier side (whole CTA): announce this rank's shard, then copy the units
// (token tile, part) assigned to this CTA from the owners' memory into x_full and flag them.
// Units are ordered as the GEMM CTAs will need them (the next rank's shard first).
template <int BN>
__device__ __forceinline__ void ag_copier(const GemmParams& p) {
  pdl_launch_dependents();
  pdl_wait();
  const unsigned int epoch_now = *p.epoch + 1u;
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
    __threadfence_system();
    for (int d = 0; d < p.ag_world; ++d)
      if (d != p.rank) st_release_sys(reinterpret_cast<unsigned int*>(p.ready[d]) + p.rank, epoch_now);
  }
  __syncthreads();
  const int n_cta = gridDim.x * p.copy_rows * gridDim.z;
  const int me = (blockIdx.z * p.copy_rows + blockIdx.y) * gridDim.x + blockIdx.x;
  const int per = p.ag_rows_per_rank / BN;                 // token tiles per shard
  const int n_units = (p.ag_world - 1) * per * kAgParts;
  const int rows_part = BN / kAgParts;
  const size_t row_bytes = static_cast<size_t>(p.K) * 2;
  for (int u = me; u < n_units; u += n_cta) {
    const int part = u % kAgParts;
    const int tt = (u / kAgParts) % per;
    const int src = (p.rank + 1 + u / (kAgParts * per)) % p.ag_world;
    if (threadIdx.x == 0 &&
        !wait_flag(reinterpret_cast<const unsigned int*>(p.ready[p.rank]) + src, epoch_now, p.status)) {
      set_status(p.status, kStatusTimeoutPeer);
      failed = 1;
    }
    __syncthreads();
    if (failed) break;
    const int row0 = tt * BN + part * rows_part;           // row inside the shard
    const uint4* from = reinterpret_cast<const uint4*>(p.x_peers[src] + row0 * row_bytes);
    uint4* to = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.x_full) +
                                         (static_cast<size_t>(src) * p.ag_rows_per_rank + row0) * row_bytes);
    const int n16 = static_cast<int>(rows_part * row_bytes / 16);
    int i = threadIdx.x;
    for (; i + 7 * kThreads < n16; i += 8 * kThreads) {     // eight 16-byte loads in flight per thread
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = from[i + u * kThreads];
#pragma unroll
      for (int u = 0; u < 8; ++u) to[i + u * kThreads] = v[u];
    }
    for (; i < n16; i += kThreads) to[i] = from[i];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int* f = p.ag_flags + (static_cast<size_t>(src) * per + tt) * kAgParts + part;
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(f), "r"(epoch_now) : "memory");
    }
  }
  // take part in the end-of-call bookkeeping like every other CTA of the grid
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int total = gridDim.x * gridDim.y * gridDim.z;
    __threadfence();
    if (atomicAdd(p.done, 1u) == total - 1) {
      *p.done = 0;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(p.epoch) = epoch_now;
    }
  }
}

__device__ __forceinline__ bool ag_handshake(const GemmParams& p, int src, unsigned int epoch_now) {
  if (p.ag_world <= 1) return true;
  if (p.x_full != nullptr) return true;   // staged mode: the copier CTAs talk to the peers
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    __threadfence_system();
    for (int d = 0; d < p.ag_world; ++d) {
      if (d == p.rank) continue;
      st_release_sys(reinterpret_cast<unsigned int*>(p.ready[d]) + p.rank, epoch_now);
    }
  }
  if (src == p.rank) return true;
  return wait_flag(reinterpret_cast<const unsigned int*>(p.ready[p.rank]) + src, epoch_now, p.status);
}

}  // namespace fi
