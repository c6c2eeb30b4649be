// Chunked-prefill attention on the tcgen05 tensor cores: varlen causal attention of the new tokens
// of every sequence against the paged 16-bit KV cache (which already holds them).
//
// One CTA owns 128 query rows of one (sequence, query head) and walks the KV range it can see in
// tiles of 128 keys:
//
//   warp 0   TMA producer: the Q tile once, then K and V tiles page by page (a page of 16 tokens is
//            one box per 64 channels, one lane per box) into rings of STAGES tiles, 128-byte swizzle
//   warp 1   UMMA issuer:  S = Q K^T  (128 x 128, fp32 in TMEM, two S buffers so the product of the
//            next tile runs under the softmax of this one) and  PV = P V  (128 x HD, two buffers of
//            their own; P is read from TMEM, V MN-major from shared memory, exactly as the cache
//            stores it)
//   warps 2-9  two threads per query row (warps 2-5 own keys 0-63 of a tile and the first half of the
//            output channels, warps 6-9 keys 64-127 and the second half): read S from TMEM, online
//            softmax in the exp2 domain (the two halves exchange their row maximum through shared
//            memory once per tile), write P as 16-bit pairs over the first 64 columns of the S buffer,
//            then fold PV of the previous tile into the row's fp32 output registers
//            (o = o * alpha + PV) so TMEM never has to be rescaled
//
// Masks (causal edge, sliding window, end of sequence) are applied only in tiles that touch an edge.
// Every wait is bounded; a wait that runs out sets the status word and the CTA leaves through the
// common teardown (TMEM freed).
//
// The reference computes the same thing with its Triton context-attention kernel
// (vllm/attention/ops/triton_prefix_prefill.py in the reference tree).
#include <math_constants.h>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../common/tensormap.h"

namespace {
using namespace fi;

struct TcParams {
  void* out;                 // [T, nh * HD]
  const int* block_tables;   // [B, max_blocks]
  const int* seq_lens;       // [B]
  const int* cu_q;           // [B + 1]
  int* status;
  // optional device array of 256 cycle counts: the CTA (0, 0, 0) records when its softmax thread 0,
  // its UMMA thread and its TMA thread pass the points of the first 16 tiles (see mark())
  unsigned long long* trace;
  int max_blocks, block_size, nh, nkv, window;
  float sm_scale, softcap;
  int is_fp16;
};

constexpr int kTile = 128;            // query rows per CTA and keys per KV tile
constexpr int kAtomBytes = 128 * 128; // 128 rows of 128 bytes: 64 channels (or keys) of one tile
constexpr int kTcThreads = 320;      // TMA warp, UMMA warp, 8 softmax warps
constexpr float kLog2e = 1.4426950408889634f;

template <int HD, int STAGES>
struct TcSmem {
  static constexpr int kQ = HD * 256;
  static constexpr int kKV = HD * 256;
  static constexpr int kHead = 3072;   // barriers (512 B) + row maxima [2 parities][2 halves][128], padded to 1024
  static constexpr int kBytes = kHead + kQ + 2 * STAGES * kKV;
};

__device__ __forceinline__ void mark(unsigned long long* trace, int slot) {
  if (trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && slot < 256)
    trace[slot] = static_cast<unsigned long long>(clock64());
}

__device__ __forceinline__ uint32_t pack2(float a, float b, int is_fp16) {
  if (is_fp16) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <int HD, int STAGES>
__global__ void __launch_bounds__(kTcThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                  const __grid_constant__ CUtensorMap v_map, const TcParams p) {
  using L = TcSmem<HD, STAGES>;
  constexpr int kAtoms = HD / 64;
  // TMA boxes per K or V tile: one per (run of box_rows tokens inside a page, 64 channels); 16-token
  // pages give 8 runs per 128-key tile, pages of 128 tokens one
  const int box_rows = min(p.block_size, kTile);
  const int n_boxes = (kTile / box_rows) * kAtoms;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kPvCol = 256;

  // This kernel takes all 512 TMEM columns of its SM.  It therefore waits for the preceding kernel
  // BEFORE it allocates (a predecessor CTA that has not allocated yet must never find the columns held
  // by a CTA that is waiting for it), and lets its successors start only after every CTA of this grid
  // holds its columns.
  pdl_wait();
  // a kernel of this stream already reported a failed wait: do not add seconds of waiting per CTA
  if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) return;
  const int b = blockIdx.z, head = blockIdx.y;
  const int q_begin = p.cu_q[b];
  const int q_len = p.cu_q[b + 1] - q_begin;
  // the tiles with the longest KV range are scheduled first
  const int qt0 = (static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)) * kTile;
  if (qt0 >= q_len) return;
  const int seq_len = p.seq_lens[b];
  const int pos0 = seq_len - q_len;
  const int rows = min(kTile, q_len - qt0);
  const int first_pos = pos0 + qt0, last_pos = first_pos + rows - 1;
  const int kv_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int tile_begin = kv_lo / kTile;
  const int n_tiles = last_pos / kTile + 1 - tile_begin;
  const int kvh = head / (p.nh / p.nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // The swizzled tiles need 1024-byte alignment and the largest configuration uses the whole 227 KB, so
  // there is no slack to round up with: the block starts aligned or the CTA refuses to run.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) set_status(p.status, kStatusBadArg);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
  uint8_t* sQ = smem_raw + L::kHead;
  uint8_t* sK = sQ + L::kQ;
  uint8_t* sV = sK + STAGES * L::kKV;
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* v_full = k_full + STAGES;
  uint64_t* k_empty = v_full + STAGES;
  uint64_t* v_empty = k_empty + STAGES;
  uint64_t* s_full = v_empty + STAGES;       // [2]
  // One barrier per buffer parity for every hand-over: a waiter that is late by a whole tile then still
  // finds "its" phase (a single barrier would already be one phase further and the parity test would
  // read as "not yet", for ever).
  uint64_t* p_full = s_full + 2;             // [2]
  uint64_t* pv_full = p_full + 2;            // [2]
  uint64_t* pair_bar = pv_full + 2;          // [4]: the two warps of a TMEM quadrant
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pair_bar + 4);
  volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* half_max = reinterpret_cast<float*>(smem_raw + 512);   // [2 parities][2 halves][128]
  // the denominators meet in the parity buffer that the last tile did not use
  float* half_sum = half_max + (n_tiles & 1) * 2 * 128;        // [2 halves][128]
  static_assert((1 + 4 * STAGES + 2 + 2 + 2 + 4) * 8 + 8 <= 512, "barrier block");

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&k_full[i], n_boxes);         // every producer lane announces its own box
      mbar_init(&v_full[i], n_boxes);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 256);
      mbar_init(&pv_full[i], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 64);
    *aborted = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // One lane per box: lanes [0, n_boxes) fetch the K tile, lanes [n_boxes, 2 n_boxes) the V tile;
    // lane l's box is token run (l % n_boxes) / kAtoms, channels 64 (l % kAtoms).  The K slot of a stage is free as soon
    // as Q K^T of its tile has run, the V slot after P V, so the two halves wait separately.
    if (lane == 0) {
      tma_prefetch_desc(&q_map);
      mbar_expect_tx(q_full, L::kQ);
#pragma unroll
      for (int a = 0; a < kAtoms; ++a)
        tma_load_2d(sQ + a * kAtomBytes, &q_map, q_full, head * HD + a * 64, q_begin + qt0);
    }
    if (lane < 2 * n_boxes) {
      const bool is_v = lane >= n_boxes;
      const int pg = ((lane % n_boxes) / kAtoms), a = lane % kAtoms;
      const uint32_t box_bytes = static_cast<uint32_t>(box_rows) * 128u;
      const CUtensorMap* map = is_v ? &v_map : &k_map;
      uint8_t* tile0 = (is_v ? sV : sK) + a * kAtomBytes + pg * box_bytes;
      uint64_t* full = is_v ? v_full : k_full;
      uint64_t* empty = is_v ? v_empty : k_empty;
      tma_prefetch_desc(map);
      const int* bt = p.block_tables + static_cast<long>(b) * p.max_blocks;
      auto row_of = [&](int j) -> int {
        const int tok = (tile_begin + j) * kTile + pg * box_rows;
        const int blk = tok < seq_len ? bt[tok / p.block_size] : 0;     // past the end: the null block
        return (blk * p.nkv + kvh) * p.block_size + tok % p.block_size;
      };
      int row_next = row_of(0);
      int issued = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % STAGES;
        const uint32_t ph = (j / STAGES) & 1;
        const int row = row_next;
        if (j + 1 < n_tiles) row_next = row_of(j + 1);   // the page id of the next tile is in flight during the wait
        if (!mbar_wait(&empty[st], ph ^ 1)) {
          set_status(p.status, kStatusTimeoutEmpty);
          *aborted = 1;
          break;
        }
        if (lane == 0 && j < 16) mark(p.trace, 192 + j * 2);
        mbar_expect_tx(&full[st], box_bytes);
        tma_load_2d(tile0 + st * L::kKV, map, &full[st], a * 64, row);
        issued = j + 1;
        if (lane == 0 && j < 16) mark(p.trace, 193 + j * 2);
      }
      // own copies in flight: the last tiles issued must have landed before the CTA may leave
      for (int j = max(0, issued - STAGES); j < issued; ++j) {
        if (!mbar_wait(&full[j % STAGES], (j / STAGES) & 1)) {
          set_status(p.status, kStatusTimeoutFull);
          break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    // The tensor pipe runs the products in the order they are issued, which is what keeps the aliases
    // apart: Q K^T of tile j+2 (same S buffer as tile j, which also holds P of tile j) is issued after
    // P V of tile j, and P V of tile j is issued only after all 256 softmax threads have read S_j and
    // written P_j.
    if (elect_one()) {
      const uint32_t fmt = p.is_fp16 ? 0 : 1;
      const uint32_t idesc_qk = umma_idesc_f16(fmt, kTile, kTile);
      const uint32_t idesc_pv = umma_idesc_f16(fmt, kTile, HD) | kUmmaBMnMajor;
      bool ok = mbar_wait(q_full, 0);
      if (!ok) set_status(p.status, kStatusTimeoutFull);
      auto issue_qk = [&](int j) -> bool {
        const int st = j % STAGES, sb = j & 1;
        if (!mbar_wait(&k_full[st], (j / STAGES) & 1)) return false;
        tc_fence_after();
#pragma unroll
        for (int a = 0; a < kAtoms; ++a) {
          const uint64_t dq = umma_desc_sw128_kmajor(smem_u32(sQ + a * kAtomBytes));
          const uint64_t dk = umma_desc_sw128_kmajor(smem_u32(sK + st * L::kKV + a * kAtomBytes));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + sb * kTile, dq + 2 * k, dk + 2 * k, idesc_qk, (a | k) != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        umma_commit(&k_empty[st]);
        return true;
      };
      ok = ok && issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (j < 16) mark(p.trace, 128 + j * 4);
        const int st = j % STAGES;
        ok = ok && mbar_wait(&p_full[j & 1], (j >> 1) & 1);
        if (j < 16) mark(p.trace, 129 + j * 4);
        ok = ok && mbar_wait(&v_full[st], (j / STAGES) & 1);
        if (!ok) break;
        if (j < 16) mark(p.trace, 130 + j * 4);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // P: rows in lanes, keys [16k, 16k + 16) in 8 columns of the tile's S buffer
          const uint32_t tp = tmem_base + (j & 1) * kTile + k * 8;
          // V: 16 keys = 16 rows of 128 bytes; the second 64 channels follow one 128-row block later
          const uint64_t dv = umma_desc_sw128_mnmajor(smem_u32(sV + st * L::kKV + k * 2048), kAtomBytes);
          umma_f16_a_tmem(tmem_base + kPvCol + (j & 1) * HD, tp, dv, idesc_pv, k != 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(&pv_full[j & 1]);
        if (j < 16) mark(p.trace, 131 + j * 4);
      }
      if (!ok) {
        set_status(p.status, kStatusTimeoutFull);
        *aborted = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output rows
    constexpr int HH = HD / 2;                       // output channels per thread
    const int quad = warp & 3;                       // TMEM lanes this warp may read: [32 quad, 32 quad + 32)
    const int half = (warp - 2) >> 2;                // 0: keys 0-63 / channels 0-HH-1, 1: the other halves
    const int row = quad * 32 + lane;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const int qpos = first_pos + row;
    const float sl2 = p.sm_scale * kLog2e;
    const bool capped = p.softcap > 0.f;
    const float cap_in = capped ? p.sm_scale / p.softcap : 0.f, cap_out = p.softcap * kLog2e;
    float o[HH];
#pragma unroll
    for (int d = 0; d < HH; ++d) o[d] = 0.f;
    float m = -CUDART_INF_F, l = 0.f, alpha_prev = 1.f;
    bool ok = true;
    // the two warps that share a TMEM quadrant (same rows, different halves) meet on a barrier of their
    // own; an mbarrier, so that the wait is bounded like every other one
    uint32_t pair_n = 0;
    auto pair_sync = [&]() -> bool {
      mbar_arrive(&pair_bar[quad]);
      return mbar_wait(&pair_bar[quad], (pair_n++) & 1);
    };

    auto fold_pv = [&](int buf, float alpha) {
#pragma unroll
      for (int c = 0; c < HH / 32; ++c) {
        uint32_t r[32];
        tmem_ld_x32(t_lane + kPvCol + buf * HD + half * HH + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c * 32 + e] = fmaf(o[c * 32 + e], alpha, __uint_as_float(r[e]));
      }
    };
    const float to_log2 = capped ? cap_out : sl2;    // raw (or tanh'ed) score -> exponent of 2

    unsigned long long* tr = (threadIdx.x == 64) ? p.trace : nullptr;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      if (!mbar_wait(&s_full[sb], (j >> 1) & 1)) { ok = false; break; }
      if (j < 16) mark(tr, j * 8);
      tc_fence_after();
      // this thread's 64 scores: read once, kept in registers
      uint32_t sr[64];
      tmem_ld_x32(t_lane + sb * kTile + half * 64, sr);
      tmem_ld_x32(t_lane + sb * kTile + half * 64 + 32, sr + 32);
      tmem_ld_wait();
      if (j < 16) mark(tr, j * 8 + 1);

      const int k0 = (tile_begin + j) * kTile + half * 64;   // first key of this thread's 64
      // keys of this half-tile the row may see: [vis_lo, vis_hi); only tiles on an edge look at them
      const bool edge = (k0 + 63 > first_pos) || (p.window > 0 && k0 <= last_pos - p.window);
      if (capped) {
#pragma unroll
        for (int e = 0; e < 64; ++e) sr[e] = __float_as_uint(fast_tanh(__uint_as_float(sr[e]) * cap_in));
      }
      if (edge) {
        const int vis_hi = qpos - k0 + 1;
        const int vis_lo = p.window > 0 ? qpos - p.window + 1 - k0 : 0;
#pragma unroll
        for (int e = 0; e < 64; ++e)
          if (e < vis_lo || e >= vis_hi) sr[e] = 0xff800000u;   // -inf: probability 0
      }
      float mt4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int e = 0; e < 64; ++e) mt4[e & 3] = fmaxf(mt4[e & 3], __uint_as_float(sr[e]));
      float mt = fmaxf(fmaxf(mt4[0], mt4[1]), fmaxf(mt4[2], mt4[3])) * to_log2;   // the factor is positive
      half_max[(sb * 2 + half) * 128 + row] = mt;
      if (j < 16) mark(tr, j * 8 + 2);
      // after this meeting both halves hold their scores in registers: the buffer may take P
      if (!pair_sync()) { ok = false; break; }
      if (j < 16) mark(tr, j * 8 + 3);
      mt = fmaxf(mt, half_max[(sb * 2 + (half ^ 1)) * 128 + row]);
      const float m_new = fmaxf(m, mt);
      const float m_use = m_new == -CUDART_INF_F ? 0.f : m_new;
      const float alpha = fast_exp2(m - m_use);

      // probabilities, packed in place (two per register) and written over the first 64 columns of the
      // S buffer: the A operand of P V, read from tensor memory
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int e = 0; e < 64; e += 2) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(sr[e]), to_log2, -m_use));
        const float p1 = fast_exp2(fmaf(__uint_as_float(sr[e + 1]), to_log2, -m_use));
        rs0 += p0;
        rs1 += p1;
        sr[e >> 1] = pack2(p0, p1, p.is_fp16);
      }
      l = l * alpha + (rs0 + rs1);                   // this half's share of the denominator
      m = m_new;
      if (j < 16) mark(tr, j * 8 + 4);
      tmem_st_x32(t_lane + sb * kTile + half * 32, sr);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[sb]);
      if (j < 16) mark(tr, j * 8 + 5);
      // fold the previous tile's product while the tensor core works on this one
      if (j > 0) {
        if (!mbar_wait(&pv_full[(j - 1) & 1], ((j - 1) >> 1) & 1)) { ok = false; break; }
        if (j < 16) mark(tr, j * 8 + 6);
        tc_fence_after();
        fold_pv((j - 1) & 1, alpha_prev);
        tc_fence_before();
      }
      if (j < 16) mark(tr, j * 8 + 7);
      alpha_prev = alpha;
    }
    if (ok) ok = mbar_wait(&pv_full[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1);
    if (ok) {
      tc_fence_after();
      fold_pv((n_tiles - 1) & 1, alpha_prev);
      half_sum[half * 128 + row] = l;
      ok = pair_sync();
      l += half_sum[(half ^ 1) * 128 + row];
      if (row < rows && ok) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        uint16_t* dst = reinterpret_cast<uint16_t*>(p.out) +
                        (static_cast<long>(q_begin + qt0 + row) * p.nh + head) * HD + half * HH;
#pragma unroll
        for (int c = 0; c < HH / 8; ++c) {
          uint4 v;
          v.x = pack2(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv, p.is_fp16);
          v.y = pack2(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv, p.is_fp16);
          v.z = pack2(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv, p.is_fp16);
          v.w = pack2(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv, p.is_fp16);
          *reinterpret_cast<uint4*>(dst + c * 8) = v;
        }
      }
    }
    if (!ok) {
      set_status(p.status, kStatusTimeoutAccum);
      *aborted = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int HD, int STAGES>
int launch_tc(const CUtensorMap& qm, const CUtensorMap& km, const CUtensorMap& vm, const TcParams& p, int B,
              int max_q_len, cudaStream_t s) {
  auto kern = prefill_tc_kernel<HD, STAGES>;
  constexpr int smem = TcSmem<HD, STAGES>::kBytes;
  cudaError_t ce = fi::ensure_dynamic_smem(kern, smem);
  if (ce != cudaSuccess) return static_cast<int>(ce);
  ce = fi::launch_kernel(kern, dim3((max_q_len + kTile - 1) / kTile, p.nh, B), dim3(kTcThreads), smem, s, 0, qm, km,
                         vm, p);
  return static_cast<int>(ce != cudaSuccess ? ce : cudaGetLastError());
}

unsigned long long* g_tc_trace = nullptr;

}  // namespace

// Development aid: a device array of 256 cycle counts (or null) that the next launches fill, see
// TcParams::trace.
extern "C" int fi_paged_prefill_tc_set_trace(void* trace) {
  g_tc_trace = reinterpret_cast<unsigned long long*>(trace);
  return 0;
}

// Tensor-core prefill attention for 16-bit caches with head size 64 or 128 and pages of 16, 32, 64 or
// a multiple of 128 tokens (larger pages mean fewer, larger TMA boxes per tile).  Returns -12 when the arguments are outside what this kernel covers (the caller then uses
// the general kernel), other negative values for malformed arguments.
//   q: token t, head h at q + (t * q_stride + h * hd) elements, T_total rows; caches [num_blocks, nkv,
//   block_size, hd]; out [T_total, nh * hd].
extern "C" int fi_paged_prefill_tc(const void* q, long q_stride, const void* k_cache, const void* v_cache, void* out,
                                   const int* block_tables, const int* seq_lens, const int* cu_q, int B,
                                   int T_total, int max_q_len, int nh, int nkv, int hd, long num_blocks,
                                   int max_blocks, int block_size, int window, float sm_scale, float softcap,
                                   int dtype, int* status, void* stream) {
  if (B <= 0 || max_q_len <= 0 || T_total <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv != 0) return -10;
  if ((hd != 64 && hd != 128) || (dtype != 0 && dtype != 1)) return -12;
  if (block_size != 16 && block_size != 32 && block_size != 64 && block_size % 128 != 0) return -12;
  if ((reinterpret_cast<uintptr_t>(q) & 15) != 0 || (q_stride * 2) % 16 != 0 ||
      (reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return -12;
  CUtensorMap qm, km, vm;
  const uint64_t kv_rows = static_cast<uint64_t>(num_blocks) * nkv * block_size;
  if (fi::make_tmap_2d_16bit_sw128(&qm, q, T_total, static_cast<uint64_t>(nh) * hd, q_stride, kTile) != 0 ||
      fi::make_tmap_2d_16bit_sw128(&km, k_cache, kv_rows, hd, hd, block_size < kTile ? block_size : kTile) != 0 ||
      fi::make_tmap_2d_16bit_sw128(&vm, v_cache, kv_rows, hd, hd, block_size < kTile ? block_size : kTile) != 0)
    return -12;
  TcParams p = {};
  p.out = out; p.block_tables = block_tables; p.seq_lens = seq_lens; p.cu_q = cu_q; p.status = status;
  p.trace = g_tc_trace;
  p.max_blocks = max_blocks; p.block_size = block_size; p.nh = nh; p.nkv = nkv; p.window = window;
  p.sm_scale = sm_scale; p.softcap = softcap; p.is_fp16 = dtype == 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (hd == 64) return launch_tc<64, 6>(qm, km, vm, p, B, max_q_len, s);
  return launch_tc<128, 3>(qm, km, vm, p, B, max_q_len, s);
}
