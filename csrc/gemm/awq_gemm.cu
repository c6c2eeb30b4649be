// Int4 weight-only GEMM for sm_100a:  C[T, N] = X[T, K] * dequant(Wq)[N, K]^T  with group-wise
// scales and optional zero points (AWQ zero-point group-128 and compressed-tensors symmetric
// group-32), plus the same epilogues as the dense kernel (bias, residual, fp32 out, gated act(g)*u).
//
// Structure = the dense tcgen05 kernel with one more pipeline stage.  TMA brings the *packed* int4
// tile (128 rows x 32 bytes) and the token tile into a deep raw ring; the four epilogue warps spend
// the main loop as dequantisers: each thread owns one weight row, expands its 64 nibbles to 16-bit
// values with the magic-number trick ((q | 0x4300) is the bf16 128+q), applies (q - z) * s and
// writes the row into a 128-byte-swizzled K-major A tile that `tcgen05.mma` consumes.  So the
// weights cross HBM once at 4 bits and never exist in dense form in global memory.
//
// Runtime weight layout (produced once at load by litevllm_b200/ops/awq.py from the checkpoint's
// qweight/scales/qzeros, which are read unchanged):
//   qw      int32 [N, K/8]   nibble order inside a word re-arranged so that (w >> 4i) & 0x000F000F
//                            yields columns (8c + 2i, 8c + 2i + 1) of the word's 8 columns
//   scales  T     [K/G, N]   (transposed: coalesced per-row reads)
//   zeros   uint8 [K/G, N]   or null for symmetric (zero point 8)
//
// Replaces the reference's Triton family vllm/kernels/triton/awq_fused_gemm.py (K10-K18: tiled
// GEMM, split-K with atomics, M=1 GEMVs, fused QKV and fused gate-up variants) with one kernel.
#include "../common/launch.cuh"
#include "../common/tensormap.h"
#include "comm_desc.h"
#include "epilogue.cuh"

using namespace fi;

namespace {


template <typename T> struct Pack;
template <> struct Pack<__nv_bfloat16> {
  using v2 = __nv_bfloat162;
  static constexpr uint32_t kMagic2 = 0x43004300u;   // bf16 128.0 in both halves: (q | magic) = 128 + q
  static constexpr float kMagicF = 128.f;
  static __device__ __forceinline__ v2 dup(float f) { return __float2bfloat162_rn(f); }
  static __device__ __forceinline__ uint32_t sub_mul(uint32_t v, v2 z, v2 s) {
    v2 x = *reinterpret_cast<v2*>(&v);
    x = __hmul2(__hsub2(x, z), s);
    return *reinterpret_cast<uint32_t*>(&x);
  }
};
template <> struct Pack<__half> {
  using v2 = __half2;
  static constexpr uint32_t kMagic2 = 0x64006400u;   // fp16 1024.0: (q | magic) = 1024 + q
  static constexpr float kMagicF = 1024.f;
  static __device__ __forceinline__ v2 dup(float f) { return __float2half2_rn(f); }
  static __device__ __forceinline__ uint32_t sub_mul(uint32_t v, v2 z, v2 s) {
    v2 x = *reinterpret_cast<v2*>(&v);
    x = __hmul2(__hsub2(x, z), s);
    return *reinterpret_cast<uint32_t*>(&x);
  }
};
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

// RST raw stages (packed weights + tokens via TMA), AST dequantised A stages.
// Packed weights are fetched SUBS k-blocks (of 64) at a time so that every weight row contributes
// 32 * SUBS contiguous bytes per TMA box: 32-byte fragments (one k-block) kept HBM at a fraction of
// its rate.  Decode-sized token tiles take 4 k-blocks (128 bytes per row), 64 tokens 2, larger 1.
__host__ __device__ constexpr int raw_subs(int bn) { return bn <= 32 ? 4 : (bn <= 64 ? 2 : 1); }
// 16-byte chunk of row `row` where logical chunk c of the packed tile lives: the TMA swizzle mode
// that matches the row pitch (128 B: 128B swizzle, 64 B: 64B swizzle, 32 B: none).
template <int SUBS>
__device__ __forceinline__ int raw_swizzle_chunk(int row, int c) {
  if (SUBS == 4) return c ^ (row & 7);
  if (SUBS == 2) return c ^ ((row >> 1) & 3);
  return c;
}

// Threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 dequantisers (warps 2..5 also run the
// TMEM -> shared-memory part of the epilogue, every thread the final reduce/store).
constexpr int kDequantWarps = 8;
constexpr int kAwqThreads = 64 + kDequantWarps * 32;

template <typename T, int BN, int RST, int AST, bool DUAL, bool ROW = false>
__global__ void __launch_bounds__(kAwqThreads)
awq_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w,
                const __grid_constant__ TokenMaps tmaps_x, const GemmParams p) {
  constexpr int NA = DUAL ? 2 : 1;
  constexpr int SUBS = raw_subs(BN);          // 64-wide k-blocks per raw stage
  constexpr int A_BYTES = BM * 128;           // dequantised tile of one k-block
  constexpr int QROW = 32 * SUBS;             // packed bytes per weight row and raw stage
  constexpr int Q_BYTES = BM * QROW;          // packed tile: 128 rows x 8*SUBS int32
  constexpr int B_BYTES = BN * 128;           // token tile of one k-block
  constexpr int RAW_BYTES = Q_BYTES * NA + B_BYTES * SUBS;   // [token sub-tiles][packed tile(s)]
  constexpr int TMEM_COLS_NEED = DUAL ? 2 * BN : BN;
  constexpr uint32_t TMEM_COLS =
      TMEM_COLS_NEED <= 32 ? 32 : TMEM_COLS_NEED <= 64 ? 64 : TMEM_COLS_NEED <= 128 ? 128
                            : TMEM_COLS_NEED <= 256 ? 256 : 512;
  constexpr int STAGES = RST;  // name used by the shared epilogue text
  (void)STAGES;
  // Row-per-thread dequantisation (template flag ROW; decode-sized token tiles with SUBS == 4 k-blocks per raw stage):
  // a thread owns one weight row and two whole k-blocks (128 values = one AWQ group) of every raw stage, so it
  // waits for the raw stage once, fetches one scale / zero point per 64..128 values and touches a barrier once
  // per 64 values: about half the per-value overhead of the half-k-block scheme used for larger token tiles.
  constexpr bool kRowScheme = ROW && (SUBS == 4);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* a_ring = smem;                                   // AST * NA * A_BYTES
  uint8_t* raw_ring = smem + AST * NA * A_BYTES;            // RST * RAW_BYTES (B tiles 1024-aligned)
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(raw_ring + RST * RAW_BYTES);
  uint64_t* raw_empty = raw_full + RST;
  uint64_t* a_full = raw_empty + RST;
  uint64_t* a_empty = a_full + AST;
  uint64_t* accum_bar = a_empty + AST;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stage_f32 = reinterpret_cast<float*>(smem);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM;
  // grouped (MoE) mode: the tile table says which expert and which sorted rows this CTA handles
  const bool grouped = p.tile_expert != nullptr;
  if (grouped) {
    pdl_wait();   // the table was written by the preceding kernel
    if (static_cast<int>(blockIdx.y) >= *p.n_tiles) return;   // uniform for the whole cluster
  }
  const int t0 = grouped ? p.tile_row0[blockIdx.y] : token_tile_index<BN>(p, blockIdx.y) * BN;
  const int t_end = grouped ? t0 + p.tile_rows[blockIdx.y] : p.T;
  const int w_row0 = grouped ? p.tile_expert[blockIdx.y] * p.expert_rows : 0;   // first weight row of the expert
  const int S = p.splits;
  const int rank = (S > 1) ? static_cast<int>(blockIdx.z) : 0;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_begin = static_cast<int>((static_cast<long long>(kb_total) * rank) / S);
  const int kb_end = static_cast<int>((static_cast<long long>(kb_total) * (rank + 1)) / S);

  if (threadIdx.x == 0) {
    for (int s = 0; s < RST; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 1 + kDequantWarps);   // MMA commit (token tile) + one arrival per dequant warp
    }
    for (int s = 0; s < AST; ++s) {
      // one arrival per dequant warp that writes the stage: all eight in the half-k-block scheme, the four
      // that own the k-block in the row-per-thread scheme (SUBS == 4)
      mbar_init(&a_full[s], kRowScheme ? kDequantWarps / 2 : kDequantWarps);
      mbar_init(&a_empty[s], 1);
    }
    mbar_init(accum_bar, 1);
    *aborted = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) pdl_launch_dependents();
  // the producer waits later, after prefetching weight tiles (a fused collective reads its epoch
  // word below, which the previous call writes, so there every warp waits first)
  const bool fused_call = p.comm_mode != kCommNone || p.ag_world > 1;
  if (warp != 0 || fused_call) pdl_wait();
  const unsigned int epoch_now = (p.comm_mode != kCommNone || p.ag_world > 1) ? *p.epoch + 1u : 0u;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int x_map = 0, x_row = t0;
      token_tile_source(p, t0, &x_map, &x_row);
      const CUtensorMap* tmap_x_ptr = &tmaps_x.m[x_map];
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(tmap_x_ptr);
      const int n_rs = (kb_end - kb_begin + SUBS - 1) / SUBS;   // raw stages of this CTA's K range
      const int n_pre = min(RST, n_rs);
      for (int rs = 0; rs < n_pre; ++rs) {   // packed weights first: they do not depend on the previous kernel
        uint8_t* r = raw_ring + rs * RAW_BYTES;
        mbar_expect_tx(&raw_full[rs], RAW_BYTES);
        const int kb0 = kb_begin + rs * SUBS;
        tma_load_2d(r + SUBS * B_BYTES, &tmap_w, &raw_full[rs], kb0 * 8, w_row0 + n0);
        if (DUAL) tma_load_2d(r + SUBS * B_BYTES + Q_BYTES, &tmap_w, &raw_full[rs], kb0 * 8, w_row0 + p.dual_rows + n0);
      }
      pdl_wait();
      if (!ag_handshake(p, x_map, epoch_now)) {
        set_status(p.status, kStatusTimeoutPeer);
        *aborted = 1;
      }
      for (int rs = 0; rs < n_pre; ++rs)
#pragma unroll
        for (int sub = 0; sub < SUBS; ++sub)   // k-blocks past K read zeros (out-of-bounds fill) and are never used
          tma_load_2d(raw_ring + rs * RAW_BYTES + sub * B_BYTES, tmap_x_ptr, &raw_full[rs],
                      (kb_begin + rs * SUBS + sub) * BK, x_row);
      for (int rs = n_pre; rs < n_rs; ++rs) {
        const int s = rs % RST;
        const uint32_t ph = (rs / RST) & 1;
        if (!mbar_wait(&raw_empty[s], ph ^ 1)) {
          set_status(p.status, kStatusTimeoutEmpty);
          *aborted = 1;
          break;
        }
        uint8_t* r = raw_ring + s * RAW_BYTES;
        const int kb0 = kb_begin + rs * SUBS;
        mbar_expect_tx(&raw_full[s], RAW_BYTES);
#pragma unroll
        for (int sub = 0; sub < SUBS; ++sub)
          tma_load_2d(r + sub * B_BYTES, tmap_x_ptr, &raw_full[s], (kb0 + sub) * BK, x_row);
        tma_load_2d(r + SUBS * B_BYTES, &tmap_w, &raw_full[s], kb0 * 8, w_row0 + n0);
        if (DUAL) tma_load_2d(r + SUBS * B_BYTES + Q_BYTES, &tmap_w, &raw_full[s], kb0 * 8, w_row0 + p.dual_rows + n0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_f16(p.is_fp16 ? 0 : 1, BM, BN);
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        const int it = kb - kb_begin;
        const int rs = it / SUBS, sub = it % SUBS;
        const int s = rs % RST, j = it % AST;
        if (!mbar_wait(&raw_full[s], (rs / RST) & 1) || !mbar_wait(&a_full[j], (it / AST) & 1)) {
          set_status(p.status, kStatusTimeoutFull);
          *aborted = 1;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(a_ring + j * NA * A_BYTES);
        const uint32_t b_addr = smem_u32(raw_ring + s * RAW_BYTES + sub * B_BYTES);
        const uint64_t da = umma_desc_sw128_kmajor(a_addr);
        const uint64_t db = umma_desc_sw128_kmajor(b_addr);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
          umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);
          if (DUAL) {
            const uint64_t da2 = umma_desc_sw128_kmajor(a_addr + A_BYTES);
            umma_f16(tmem_base + BN, da2 + 2 * k, db + 2 * k, idesc, acc);
          }
        }
        if (sub == SUBS - 1 || kb == kb_end - 1) umma_commit(&raw_empty[s]);   // last k-block of the raw stage
        umma_commit(&a_empty[j]);
      }
      umma_commit(accum_bar);
    }
  } else {
    // ------------------------------------------------------------ dequantisers (warps 2..9)
    // thread -> (weight row, half of the k-block): 4 packed words -> 32 values -> four 16-byte chunks
    // of the row's swizzled 128-byte line.  Eight warps keep two conversion chains per scheduler in
    // flight.  Everything that does not depend on the k-block is computed once up front (swizzled
    // offsets, scale pointers); scale and zero point stay 16-bit / integer (no float conversions);
    // ring positions are running counters, not divisions: the loop body is issue-bound otherwise.
    const int dw = warp - 2;
    const int row = (dw & 3) * 32 + lane;
    const int half = dw >> 2;
    if constexpr (kRowScheme) {
      const bool pow2 = (p.group & (p.group - 1)) == 0;
      const int gshift = 31 - __clz(p.group);
      const bool two_scales = p.group < 64;          // group 32: the two halves of a k-block have their own scale
      const uint16_t* scales16 = reinterpret_cast<const uint16_t*>(p.scales);
      uint32_t st_off[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) st_off[c] = sw128_offset(row, c);
      uint32_t ld_off[2][2];                         // [my k-block u][16-byte half h] inside the packed tile
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          ld_off[u][h] = SUBS * B_BYTES + row * QROW + raw_swizzle_chunk<SUBS>(row, (half * 2 + u) * 2 + h) * 16;
      size_t srow[NA];
      bool rvalid[NA];
#pragma unroll
      for (int a = 0; a < NA; ++a) {
        const int grow = w_row0 + (a == 0 ? n0 : p.dual_rows + n0) + row;
        rvalid[a] = grow < p.n_rows_total;
        srow[a] = rvalid[a] ? grow : 0;
      }
      // (scale, zero) words of my two k-blocks of a raw stage, loaded one stage ahead
      uint16_t s_raw[NA][2][2];
      uint8_t z_raw[NA][2][2];
      auto fetch = [&](int rs) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int kb = kb_begin + rs * SUBS + half * 2 + u;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int k = kb * BK + h * 32;
            const size_t g = static_cast<size_t>(pow2 ? (k >> gshift) : (k / p.group)) * p.n_rows_total;
#pragma unroll
            for (int a = 0; a < NA; ++a) {
              s_raw[a][u][h] = 0;
              z_raw[a][u][h] = 8;
              if (rvalid[a] && kb < kb_end && (h == 0 || two_scales)) {
                s_raw[a][u][h] = scales16[g + srow[a]];
                if (p.zeros != nullptr) z_raw[a][u][h] = p.zeros[g + srow[a]];
              }
            }
          }
        }
      };
      const int n_rs = (kb_end - kb_begin + SUBS - 1) / SUBS;
      if (n_rs > 0) fetch(0);
      bool ok = true;
      int s = 0;
      uint32_t raw_ph = 0;
      for (int rs = 0; rs < n_rs && ok; ++rs) {
        uint32_t s2[NA][2][2], z2[NA][2][2];
#pragma unroll
        for (int a = 0; a < NA; ++a)
#pragma unroll
          for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              // static indices only: a run-time index would push the arrays into local memory
              const uint16_t sr = (h == 1 && two_scales) ? s_raw[a][u][1] : s_raw[a][u][0];
              const uint8_t zr = (h == 1 && two_scales) ? z_raw[a][u][1] : z_raw[a][u][0];
              s2[a][u][h] = static_cast<uint32_t>(sr) * 0x00010001u;
              z2[a][u][h] = Pack<T>::kMagic2 + static_cast<uint32_t>(zr) * 0x00010001u;
            }
        if (rs + 1 < n_rs) fetch(rs + 1);
        if (!mbar_wait(&raw_full[s], raw_ph)) {
          set_status(p.status, kStatusTimeoutFull);
          *aborted = 1;
          ok = false;
          break;
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int sub = half * 2 + u;
          const int kb = kb_begin + rs * SUBS + sub;
          if (kb >= kb_end) break;                                       // ragged last raw stage (uniform per warp)
          const int it = rs * SUBS + sub;                                // k-blocks use the A stages round robin
          const int j = it % AST;
          const uint32_t a_ph = ((static_cast<uint32_t>(it / AST)) & 1u) ^ 1u;
          if (!mbar_wait(&a_empty[j], a_ph)) {
            set_status(p.status, kStatusTimeoutFull);
            *aborted = 1;
            ok = false;
            break;
          }
#pragma unroll
          for (int a = 0; a < NA; ++a) {
            uint8_t* dst = a_ring + (j * NA + a) * A_BYTES;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint4 w4 = *reinterpret_cast<const uint4*>(raw_ring + s * RAW_BYTES + a * Q_BYTES + ld_off[u][h]);
              const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
              const typename Pack<T>::v2 sv = *reinterpret_cast<const typename Pack<T>::v2*>(&s2[a][u][h]);
              const typename Pack<T>::v2 zv = *reinterpret_cast<const typename Pack<T>::v2*>(&z2[a][u][h]);
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const uint32_t v = ((words[c] >> (4 * i)) & 0x000F000Fu) | Pack<T>::kMagic2;
                  o[i] = Pack<T>::sub_mul(v, zv, sv);
                }
                *reinterpret_cast<uint4*>(dst + st_off[h * 4 + c]) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[j]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&raw_empty[s]);
        if (++s == RST) { s = 0; raw_ph ^= 1; }
      }
    } else {
    uint32_t st_off[4], ld_off[SUBS];
#pragma unroll
    for (int c = 0; c < 4; ++c) st_off[c] = sw128_offset(row, half * 4 + c);
#pragma unroll
    for (int sub = 0; sub < SUBS; ++sub)
      ld_off[sub] = SUBS * B_BYTES + row * QROW + raw_swizzle_chunk<SUBS>(row, sub * 2 + half) * 16;
    const bool pow2 = (p.group & (p.group - 1)) == 0;
    const int gshift = 31 - __clz(p.group);
    const uint16_t* scales16 = reinterpret_cast<const uint16_t*>(p.scales);
    const uint16_t* sptr[NA];
    const uint8_t* zptr[NA];
    bool rvalid[NA];
#pragma unroll
    for (int a = 0; a < NA; ++a) {
      const int grow = w_row0 + (a == 0 ? n0 : p.dual_rows + n0) + row;
      rvalid[a] = grow < p.n_rows_total;
      sptr[a] = scales16 + (rvalid[a] ? grow : 0);
      zptr[a] = p.zeros != nullptr ? p.zeros + (rvalid[a] ? grow : 0) : nullptr;
    }
    // scale / zero point are loaded one k-block ahead and only used when their block comes up: a
    // warp issues in order, so touching a loaded value earlier would park it for the L2 latency.
    uint16_t s_raw[NA];
    uint8_t z_raw[NA];
    auto fetch = [&](int kb) {
      const int k = kb * BK + half * 32;
      const size_t g = static_cast<size_t>(pow2 ? (k >> gshift) : (k / p.group)) * p.n_rows_total;
#pragma unroll
      for (int a = 0; a < NA; ++a) {
        s_raw[a] = 0;
        z_raw[a] = 8;
        if (rvalid[a] && kb < kb_end) {
          s_raw[a] = sptr[a][g];
          if (zptr[a] != nullptr) z_raw[a] = zptr[a][g];
        }
      }
    };
    fetch(kb_begin);
    bool ok = true;
    int s = 0, sub = 0, j = 0;                 // raw stage, k-block inside it, A stage
    uint32_t raw_ph = 0, a_ph = 1;             // parities to wait for
    for (int kb = kb_begin; kb < kb_end && ok; ++kb) {
      uint32_t s2[NA], z2[NA];
#pragma unroll
      for (int a = 0; a < NA; ++a) {           // (scale, scale) and (magic + zero, magic + zero) as 16-bit pairs
        s2[a] = static_cast<uint32_t>(s_raw[a]) * 0x00010001u;
        z2[a] = Pack<T>::kMagic2 + static_cast<uint32_t>(z_raw[a]) * 0x00010001u;
      }
      fetch(kb + 1);
      if (!mbar_wait(&raw_full[s], raw_ph) || !mbar_wait(&a_empty[j], a_ph)) {
        set_status(p.status, kStatusTimeoutFull);
        *aborted = 1;
        ok = false;
        break;
      }
#pragma unroll
      for (int a = 0; a < NA; ++a) {
        const uint4 w4 = *reinterpret_cast<const uint4*>(raw_ring + s * RAW_BYTES + a * Q_BYTES + ld_off[sub]);
        const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
        uint8_t* dst = a_ring + (j * NA + a) * A_BYTES;
        const typename Pack<T>::v2 sv = *reinterpret_cast<const typename Pack<T>::v2*>(&s2[a]);
        const typename Pack<T>::v2 zv = *reinterpret_cast<const typename Pack<T>::v2*>(&z2[a]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t v = ((words[c] >> (4 * i)) & 0x000F000Fu) | Pack<T>::kMagic2;
            o[i] = Pack<T>::sub_mul(v, zv, sv);
          }
          *reinterpret_cast<uint4*>(dst + st_off[c]) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      fence_proxy_async_smem();   // generic-proxy smem writes -> visible to the tensor-core proxy
      __syncwarp();
      const bool raw_done = sub == SUBS - 1 || kb == kb_end - 1;
      if (lane == 0) {
        mbar_arrive(&a_full[j]);
        if (raw_done) mbar_arrive(&raw_empty[s]);
      }
      if (++j == AST) { j = 0; a_ph ^= 1; }
      if (++sub == SUBS) {
        sub = 0;
        if (++s == RST) { s = 0; raw_ph ^= 1; }
      }
    }
    }   // half-k-block scheme
  }
  // ---------------------------------------------------------------- epilogue (epilogue.cuh)
  if (warp >= 2 && warp < 6) epilogue_tmem_to_smem<BN, DUAL>(p, accum_bar, tmem_base, stage_f32, aborted, warp, lane);
  __syncthreads();
  epilogue_reduce_store<BN, DUAL>(p, stage_f32, aborted, n0, t0, epoch_now, t_end);
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int RST, int AST, bool DUAL>
constexpr int ring_bytes() {
  return AST * (DUAL ? 2 : 1) * BM * 128 + RST * raw_subs(BN) * (BM * 32 * (DUAL ? 2 : 1) + BN * 128);
}
template <int BN, int RST, int AST, bool DUAL>
constexpr int smem_bytes() {
  return ring_bytes<BN, RST, AST, DUAL>() + (2 * RST + 2 * AST + 1) * 8 + 16 + 1024;
}

template <typename T, int BN, int RST, int AST, bool DUAL, bool ROW = false>
int launch(const CUtensorMap& tw, const TokenMaps& tx, GemmParams p, cudaStream_t stream) {
  auto kern = awq_gemm_kernel<T, BN, RST, AST, DUAL, ROW>;
  constexpr int smem = smem_bytes<BN, RST, AST, DUAL>();
  constexpr int ring = ring_bytes<BN, RST, AST, DUAL>();
  static_assert(BN * BM * 4 <= ring, "fp32 staging tile must fit inside the rings");
  static int max_active[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  {
    cudaError_t e = fi::ensure_dynamic_smem(kern, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int tiles = ((p.N + BM - 1) / BM) * ((p.T + BN - 1) / BN);
  const int kb_total = (p.K + BK - 1) / BK;
  if (p.splits <= 0) {
    // same cost model as the dense kernel, with 4-bit weight bytes
    const float tile_bytes = static_cast<float>(kb_total) * (BM * 32 * (DUAL ? 2 : 1) + BN * 128);
    int best = 1;
    float best_t = 1e30f;
    for (int S = 1; S <= 8; ++S) {
      if (S > 1 && kb_total / S < 2) break;
      if (BN * BM * 4 * ((DUAL && S > 1) ? 2 : 1) > ring) break;
      if (max_active[S] == 0) {
        cudaLaunchConfig_t c = {};
        c.gridDim = dim3(148, 1, S); c.blockDim = dim3(kAwqThreads); c.dynamicSmemBytes = smem;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = S;
        c.attrs = at; c.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &c) != cudaSuccess || n <= 0) {
          cudaGetLastError();
          n = S == 1 ? 148 : (148 / S) * 3 / 4;
        }
        max_active[S] = n;
      }
      const int act = tiles < max_active[S] ? tiles : max_active[S];
      const int waves = (tiles + max_active[S] - 1) / max_active[S];
      const float gbs = fminf(6400.f, act * S * 60.f);
      const float t = waves * (3.5f + (S > 1 ? 1.f : 0.f) + tile_bytes * act / (gbs * 1e3f));
      if (t < best_t) { best_t = t; best = S; }
    }
    p.splits = best;
  }
  if (BN * BM * 4 * ((DUAL && p.splits > 1) ? 2 : 1) > ring) return -12;
  return static_cast<int>(launch_kernel(kern, dim3((p.N + BM - 1) / BM, p.grid_tiles > 0 ? p.grid_tiles : (p.T + BN - 1) / BN, p.splits),
                                        dim3(kAwqThreads), smem, stream, p.splits, tw, tx, p));
}

inline bool row_scheme() {
  static const bool on = [] {
    const char* v = getenv("FI_AWQ_ROW_SCHEME");
    return v == nullptr || v[0] != '0';
  }();
  return on;
}

template <typename T, bool DUAL>
int dispatch(int bn, const CUtensorMap& tw, const TokenMaps& tx, const GemmParams& p, cudaStream_t s) {
  switch (bn) {
    // raw stages hold raw_subs(BN) k-blocks each; sizes keep two CTAs per SM where possible
    // decode-sized tiles: row-per-thread dequantisers (FI_AWQ_ROW_SCHEME=0: the older half-k-block dequantisers)
    case 16: return row_scheme() ? launch<T, 16, 2, DUAL ? 2 : 3, DUAL, true>(tw, tx, p, s) : launch<T, 16, 2, DUAL ? 2 : 3, DUAL>(tw, tx, p, s);
    case 32: return row_scheme() ? launch<T, 32, 2, DUAL ? 2 : 3, DUAL, true>(tw, tx, p, s) : launch<T, 32, 2, DUAL ? 2 : 3, DUAL>(tw, tx, p, s);
    case 64: return launch<T, 64, 2, DUAL ? 2 : 3, DUAL>(tw, tx, p, s);
    default: return launch<T, 128, 3, DUAL ? 2 : 3, DUAL>(tw, tx, p, s);
  }
}

// Packed weights as a 2-D int32 tensor [rows, K/8]; box = 8 words x 128 rows, no swizzle.
inline int make_tmap_packed(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k_words, int subs) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((k_words * 4) & 15) != 0) return -2;
  cuuint64_t dims[2] = {k_words, rows};
  cuuint64_t strides[1] = {k_words * 4};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(8 * subs), 128};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle swz = subs == 4 ? CU_TENSOR_MAP_SWIZZLE_128B
                                           : (subs == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE);
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<void*>(base), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace

// C = X dequant(Wq)^T with optional epilogue.  qw/scales/zeros in the runtime layout described at
// the top of this file.  dtype: 0 bf16, 1 fp16 (X, scales, bias, C unless out_fp32).
// dual_rows > 0: gated mode, the weight holds [gate rows; up rows] and N == dual_rows.
static int fi_awq_gemm_impl(const void* X, const void* qw, const void* scales, const void* zeros, void* C,
                           const void* bias, const void* residual, int T, int N, int K, int group,
                           int ldx, int ldc, int act, int dual_rows, int out_fp32, int dtype,
                           int splits, int bn, int* status, void* stream,
                             const FiComm* comm, const FiGrouped* grp) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 64) != 0 || (ldc % 8) != 0 || (reinterpret_cast<uintptr_t>(C) & 15) != 0) return -10;
  if (group != 32 && group != 64 && group != 128 && !(group > 128 && group % 64 == 0)) return -13;
  if (dual_rows > 0 && N != dual_rows) return -11;
  if (bn == 0) bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128;
  int w_rows = dual_rows > 0 ? 2 * dual_rows : N;
  if (grp != nullptr) w_rows = grp->num_experts * grp->expert_rows;
  CUtensorMap tw;
  TokenMaps tx;
  int r = make_tmap_packed(&tw, qw, w_rows, K / 8, raw_subs(bn));
  if (r != 0) return r * 100 - 1;
  if (comm != nullptr && comm->ag_world > 1) {
    if (comm->ag_rows_per_rank % bn != 0) return -14;
    for (int d = 0; d < comm->ag_world; ++d) {
      int rows = T - d * comm->ag_rows_per_rank;
      rows = rows < 0 ? 0 : (rows > comm->ag_rows_per_rank ? comm->ag_rows_per_rank : rows);
      r = make_tmap_2d_16bit_sw128(&tx.m[d], reinterpret_cast<const void*>(comm->x_peers[d]),
                                   rows > 0 ? rows : 1, K, ldx, bn);
      if (r != 0) return r * 100 - 2;
    }
  } else {
    r = make_tmap_2d_16bit_sw128(&tx.m[0], X, T, K, ldx, bn);
    if (r != 0) return r * 100 - 2;
  }
  const int kb_total = K / BK;
  if (splits > 8) splits = 8;
  if (splits > kb_total) splits = kb_total;
  if (bn >= 128 && dual_rows > 0) splits = 1;
  GemmParams p;
  p.C = C; p.bias = bias; p.residual = residual;
  p.T = T; p.N = N; p.K = K; p.ldc = ldc;
  p.dual_rows = dual_rows; p.act = act; p.out_fp32 = out_fp32; p.is_fp16 = dtype == 1;
  p.splits = splits; p.status = status;
  p.scales = scales; p.zeros = reinterpret_cast<const uint8_t*>(zeros); p.group = group;
  p.n_rows_total = w_rows;
  p.tile_expert = nullptr; p.tile_row0 = nullptr; p.tile_rows = nullptr; p.n_tiles = nullptr; p.expert_rows = 0; p.grid_tiles = 0;
  p.comm_mode = 0; p.world = 1; p.rank = 0; p.rows_per_rank = 0; p.xfer_16bit = 0; p.comm_phases = 0; p.trace = nullptr;
  p.rms_eps = 0.f; p.w_dynamic = 0;
  p.x_full = nullptr; p.ag_flags = nullptr; p.copy_rows = 0;
  p.rope_cs = nullptr; p.rope_pos = nullptr; p.rope_slots = nullptr; p.k_cache = nullptr; p.v_cache = nullptr;
  p.rope_nh = p.rope_nkv = p.rope_hd = p.rope_bs = 0;
  p.ag_world = 1; p.ag_rows_per_rank = 0; p.slab_elems = 0; p.epoch = nullptr; p.done = nullptr;
  for (int d = 0; d < kMaxRanks; ++d) { p.recv[d] = 0; p.flags[d] = 0; p.ready[d] = 0; }
  if (comm != nullptr) {
    if (comm->world > kMaxRanks || comm->ag_world > kMaxRanks) return -15;
    if (comm->mode != 0 && dual_rows > 0) return -16;   // a gated epilogue needs the full K sum
    p.comm_mode = comm->mode; p.world = comm->world; p.rank = comm->rank;
    p.rows_per_rank = comm->rows_per_rank; p.xfer_16bit = comm->xfer_16bit; p.comm_phases = comm->phases;
    p.ag_world = comm->ag_world > 1 ? comm->ag_world : 1; p.ag_rows_per_rank = comm->ag_rows_per_rank;
    p.slab_elems = comm->slab_elems;
    p.epoch = reinterpret_cast<unsigned int*>(comm->epoch);
    p.done = reinterpret_cast<unsigned int*>(comm->done);
    p.trace = reinterpret_cast<unsigned long long*>(comm->trace);
    for (int d = 0; d < kMaxRanks; ++d) { p.recv[d] = comm->recv[d]; p.flags[d] = comm->flags[d]; p.ready[d] = comm->ready[d]; }
    if (comm->mode == kCommReduceScatter && (comm->rows_per_rank % bn) != 0) return -17;
    const long tiles = static_cast<long>((N + BM - 1) / BM) * ((T + bn - 1) / bn);
    if (comm->mode != 0 && tiles > kMaxCommTiles) return -18;
    if (comm->mode != 0 && (N % 8) != 0) return -19;
    // the two-hop all-reduce sends 16-bit results and owns chunks inside a 128-row tile
    if (comm->xfer_16bit == kXferTwoShot && (comm->mode != kCommAllReduce || out_fp32 || (ldc % 4) != 0)) return -24;
  }
  if (grp != nullptr) {
    if (comm != nullptr && comm->mode != 0) return -20;
    p.tile_expert = grp->tile_expert; p.tile_row0 = grp->tile_row0; p.tile_rows = grp->tile_rows;
    p.n_tiles = grp->n_tiles; p.expert_rows = grp->expert_rows; p.splits = 1;
    p.grid_tiles = grp->max_tiles;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1) {
    if (dual_rows > 0) return dispatch<__half, true>(bn, tw, tx, p, s);
    return dispatch<__half, false>(bn, tw, tx, p, s);
  }
  if (dual_rows > 0) return dispatch<__nv_bfloat16, true>(bn, tw, tx, p, s);
  return dispatch<__nv_bfloat16, false>(bn, tw, tx, p, s);
}

extern "C" int fi_awq_gemm(const void* X, const void* qw, const void* scales, const void* zeros, void* C,
                           const void* bias, const void* residual, int T, int N, int K, int group,
                           int ldx, int ldc, int act, int dual_rows, int out_fp32, int dtype,
                           int splits, int bn, int* status, void* stream) {
  return fi_awq_gemm_impl(X, qw, scales, zeros, C, bias, residual, T, N, K, group, ldx, ldc, act, dual_rows, out_fp32, dtype, splits, bn, status, stream, nullptr, nullptr);
}

// Same GEMM with a fused collective and/or an all-gathered token operand (see comm_desc.h).
extern "C" int fi_awq_gemm_comm(const void* X, const void* qw, const void* scales, const void* zeros, void* C,
                           const void* bias, const void* residual, int T, int N, int K, int group,
                           int ldx, int ldc, int act, int dual_rows, int out_fp32, int dtype,
                           int splits, int bn, int* status, void* stream,
                             const FiComm* comm) {
  return fi_awq_gemm_impl(X, qw, scales, zeros, C, bias, residual, T, N, K, group, ldx, ldc, act, dual_rows, out_fp32, dtype, splits, bn, status, stream, comm, nullptr);
}

// Grouped expert GEMM: X holds the expert-sorted activation rows, qw/scales/zeros the stacked experts.
extern "C" int fi_awq_gemm_grouped(const void* X, const void* qw, const void* scales, const void* zeros, void* C,
                           const void* bias, const void* residual, int T, int N, int K, int group,
                           int ldx, int ldc, int act, int dual_rows, int out_fp32, int dtype,
                           int splits, int bn, int* status, void* stream,
                             const FiGrouped* grp) {
  return fi_awq_gemm_impl(X, qw, scales, zeros, C, bias, residual, T, N, K, group, ldx, ldc, act, dual_rows, out_fp32, dtype, splits, bn, status, stream, nullptr, grp);
}
