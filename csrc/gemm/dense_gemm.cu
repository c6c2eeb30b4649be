// Dense 16-bit GEMM for sm_100a:  C[T, N] = X[T, K] * W[N, K]^T  (+ bias, + residual, or the
// gated form act(X Wg^T) * (X Wu^T)).
//
// Design ("weights on the M side"): the weight matrix is the UMMA A operand (128 weight rows per
// CTA, UMMA M = 128) and the activations are the B operand (BN tokens per CTA, UMMA N = BN), both
// K-major, so decode batches of 16..64 tokens still fill a full 128-lane tensor-core tile and the
// kernel streams the weights exactly once.  TMA (128-byte swizzle) feeds a multi-stage smem ring,
// one elected thread issues tcgen05.mma into a TMEM accumulator, four epilogue warps read it back
// with tcgen05.ld.  Split-K runs as a thread-block cluster along z: every CTA of the cluster parks
// its fp32 partial tile in its own shared memory and the CTAs sum the partials through distributed
// shared memory, so the reduction needs no global scratch and no atomics (bitwise deterministic).
//
// Replaces the library GEMM behind every unquantised linear of the reference
// (vllm/model_executor/layers/lite_linear.py:60-62) and the silu-and-mul kernel
// (vllm/kernels/triton/activation.py:42) that follows its gate/up projections.
#include "../common/launch.cuh"
#include "../common/tensormap.h"
#include "comm_desc.h"
#include "epilogue.cuh"

using namespace fi;

namespace {

// Debug aid: device array of 8 x uint64 that CTA (0,0,0) of every plain GEMM launch fills with cycle
// counts of its phases (see cycle_mark); null = off.  Set with fi_dense_gemm_set_trace.
unsigned long long* g_plain_trace = nullptr;


template <int BN, int STAGES, bool DUAL>
__global__ void __launch_bounds__(kThreads)
dense_gemm_kernel(const __grid_constant__ CUtensorMap tmap_w,
                  const __grid_constant__ TokenMaps tmaps_x, const GemmParams p) {
  constexpr int A_BYTES = BM * 128;
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = A_BYTES * (DUAL ? 2 : 1) + B_BYTES;
  constexpr int TMEM_COLS_NEED = DUAL ? 2 * BN : BN;
  constexpr uint32_t TMEM_COLS =
      TMEM_COLS_NEED <= 32 ? 32 : TMEM_COLS_NEED <= 64 ? 64 : TMEM_COLS_NEED <= 128 ? 128
                            : TMEM_COLS_NEED <= 256 ? 256 : 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* row_ss = reinterpret_cast<float*>(tmem_slot + 2);   // [BN] floats after the control words: sum of squares per token
  const bool rms = p.rms_eps > 0.f;
  // fp32 staging of the accumulator tile(s); aliases the pipeline ring once the main loop is done.
  float* stage_f32 = reinterpret_cast<float*>(smem);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM;
  if (threadIdx.x == 0) cycle_mark(p.trace, p.comm_mode != kCommNone, 0);
  if (p.copy_rows > 0 && static_cast<int>(blockIdx.y) < p.copy_rows) {   // staged all-gather: copier CTA
    ag_copier<BN>(p);
    return;
  }
  const int t0 = token_tile_index<BN>(p, static_cast<int>(blockIdx.y) - p.copy_rows) * BN;
  const int S = p.splits;
  const int rank = (S > 1) ? static_cast<int>(blockIdx.z) : 0;

  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_begin = static_cast<int>((static_cast<long long>(kb_total) * rank) / S);
  const int kb_end = static_cast<int>((static_cast<long long>(kb_total) * (rank + 1)) / S);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], rms ? 1 + 4 : 1);   // MMA commit (+ the four warps that read the token tile)
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
  if (threadIdx.x == 0) cycle_mark(p.trace, p.comm_mode != kCommNone, 1);
  if (threadIdx.x == 0) pdl_launch_dependents();
  // the producer waits later, after prefetching weight tiles (a fused collective reads its epoch
  // word below, which the previous call writes, so there every warp waits first)
  const bool fused_call = p.comm_mode != kCommNone || p.ag_world > 1;
  if (warp != 0 || fused_call) pdl_wait();
  if (threadIdx.x == 64) cycle_mark(p.trace, p.comm_mode != kCommNone, 2);
  const unsigned int epoch_now = (p.comm_mode != kCommNone || p.ag_world > 1) ? *p.epoch + 1u : 0u;
  if (fused_call) trace_mark(p.trace, epoch_now, 0);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int x_map = 0, x_row = t0;
      token_tile_source(p, t0, &x_map, &x_row);
      const CUtensorMap* tmap_x_ptr = &tmaps_x.m[x_map];
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(tmap_x_ptr);
      // Weights do not depend on the previous kernel: start streaming them for the first stages
      // before blocking on the programmatic dependency, then add the token tiles.
      const int n_pre = min(STAGES, kb_end - kb_begin);
      if (p.w_dynamic) pdl_wait();   // the weights come from the preceding kernel: nothing may be read yet
      for (int it = 0; it < n_pre; ++it) {
        uint8_t* a = stage_base + it * STAGE_BYTES;
        mbar_expect_tx(&full_bar[it], STAGE_BYTES);
        tma_load_2d(a, &tmap_w, &full_bar[it], (kb_begin + it) * BK, n0);
        if (DUAL) tma_load_2d(a + A_BYTES, &tmap_w, &full_bar[it], (kb_begin + it) * BK, p.dual_rows + n0);
      }
      pdl_wait();
      if (!ag_handshake(p, x_map, epoch_now) ||
          (x_map == kStagedMap && !ag_wait_staged<BN>(p, t0, epoch_now))) {
        set_status(p.status, kStatusTimeoutPeer);
        *aborted = 1;
      }
      for (int it = 0; it < n_pre; ++it) {
        uint8_t* a = stage_base + it * STAGE_BYTES;
        tma_load_2d(a + A_BYTES * (DUAL ? 2 : 1), tmap_x_ptr, &full_bar[it], (kb_begin + it) * BK, x_row);
      }
      for (int kb = kb_begin + n_pre; kb < kb_end; ++kb) {
        const int it = kb - kb_begin;
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
          set_status(p.status, kStatusTimeoutEmpty);
          *aborted = 1;
          break;
        }
        uint8_t* a = stage_base + s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(a, &tmap_w, &full_bar[s], kb * BK, n0);
        if (DUAL) tma_load_2d(a + A_BYTES, &tmap_w, &full_bar[s], kb * BK, p.dual_rows + n0);
        tma_load_2d(a + A_BYTES * (DUAL ? 2 : 1), tmap_x_ptr, &full_bar[s], kb * BK, x_row);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_f16(p.is_fp16 ? 0 : 1, BM, BN);
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end && ok; ++kb) {
        const int it = kb - kb_begin;
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], ph)) {
          set_status(p.status, kStatusTimeoutFull);
          *aborted = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(stage_base + s * STAGE_BYTES);
        const uint32_t b_addr = a_addr + A_BYTES * (DUAL ? 2 : 1);
        const uint64_t da = umma_desc_sw128_kmajor(a_addr);
        const uint64_t db = umma_desc_sw128_kmajor(b_addr);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
          // advancing 16 elements along K inside the swizzle atom = +32 bytes = +2 in the
          // (address >> 4) field of the descriptor
          umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);
          if (DUAL) {
            const uint64_t da2 = umma_desc_sw128_kmajor(a_addr + A_BYTES);
            umma_f16(tmem_base + BN, da2 + 2 * k, db + 2 * k, idesc, acc);
          }
        }
        umma_commit(&empty_bar[s]);
      }
      umma_commit(accum_bar);
    }
  }
  else if (rms) {
    // ------------------------------------------------------------ warps 2..5: sum of squares per token
    // The token tile of every stage is [BN rows][64 values] in the 128-byte swizzle; 128 threads
    // read it as 16-byte chunks (chunk c: row c / 8), eight neighbouring threads share a row.
    const int tid = threadIdx.x - 64;
    constexpr int kChunks = BN * 8;
    constexpr int kPerThread = (kChunks + 127) / 128;
    float ss[kPerThread];
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) ss[i] = 0.f;
    bool ok = true;
    for (int kb = kb_begin; kb < kb_end && ok; ++kb) {
      const int it = kb - kb_begin;
      const int s = it % STAGES;
      const uint32_t ph = (it / STAGES) & 1;
      if (!mbar_wait(&full_bar[s], ph)) {
        set_status(p.status, kStatusTimeoutFull);
        *aborted = 1;
        ok = false;
        break;
      }
      const uint8_t* b = stage_base + s * STAGE_BYTES + A_BYTES * (DUAL ? 2 : 1);
#pragma unroll
      for (int i = 0; i < kPerThread; ++i) {
        const int c = tid + i * 128;
        if (c < kChunks) {
          const uint4 raw = *reinterpret_cast<const uint4*>(b + sw128_offset(c >> 3, c & 7));
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float lo, hi;
            if (p.is_fp16) {
              const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
              lo = __low2float(h); hi = __high2float(h);
            } else {
              lo = __uint_as_float(w[j] << 16); hi = __uint_as_float(w[j] & 0xffff0000u);
            }
            ss[i] += lo * lo + hi * hi;
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      float v = ss[i];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      const int c = tid + i * 128;
      if ((c & 7) == 0 && c < kChunks) row_ss[c >> 3] = v;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // the four warps: row_ss complete before it is used
  }
  // ---------------------------------------------------------------- epilogue (epilogue.cuh)
  if (warp >= 2) epilogue_tmem_to_smem<BN, DUAL>(p, accum_bar, tmem_base, stage_f32, aborted, warp, lane, row_ss);
  __syncthreads();
  epilogue_reduce_store<BN, DUAL>(p, stage_f32, aborted, n0, t0, epoch_now, p.T, row_ss);
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES, bool DUAL>
constexpr int smem_bytes() {
  return STAGES * (BM * 128 * (DUAL ? 2 : 1) + BN * 128) + (2 * STAGES + 1) * 8 + 16 + BN * 4 + 1024;
}

// Split-K choice.  A cluster of S CTAs must be co-scheduled inside one GPC, so the number of
// clusters that can run at once drops quickly with S (the runtime reports it); the pick minimises
//   waves * (fixed cost + bytes per wave / achievable bandwidth)
// where a lone CTA can pull roughly kPerCtaGBs and the whole chip kChipGBs.
template <int BN, int STAGES, bool DUAL>
int pick_splits(const GemmParams& p, int smem) {
  constexpr float kPerCtaGBs = 110.f, kChipGBs = 6400.f, kFixedUs = 3.5f, kClusterUs = 1.0f;
  static int max_active[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  auto kern = dense_gemm_kernel<BN, STAGES, DUAL>;
  const int tiles = ((p.N + BM - 1) / BM) * ((p.T + BN - 1) / BN);
  const int kb_total = (p.K + BK - 1) / BK;
  constexpr int ring = STAGES * (BM * 128 * (DUAL ? 2 : 1) + BN * 128);
  const float tile_bytes = static_cast<float>(kb_total) * (BM * 128 * (DUAL ? 2 : 1) + BN * 128);
  int best = 1;
  float best_t = 1e30f;
  for (int S = 1; S <= 8; ++S) {
    if (S > 1 && kb_total / S < 2) break;
    if (BN * BM * 4 * ((DUAL && S > 1) ? 2 : 1) > ring) break;
    if (max_active[S] == 0) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(148, 1, S);
      cfg.blockDim = dim3(kThreads);
      cfg.dynamicSmemBytes = smem;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = S;
      cfg.attrs = attr; cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = S == 1 ? 148 : (148 / S) * 3 / 4;
      }
      max_active[S] = n;
    }
    const int waves = (tiles + max_active[S] - 1) / max_active[S];
    const int ctas_per_wave = (tiles < max_active[S] ? tiles : max_active[S]) * S;
    const float gbs = fminf(kChipGBs, ctas_per_wave * kPerCtaGBs);
    const float bytes_per_wave = tile_bytes * (tiles < max_active[S] ? tiles : max_active[S]);
    const float t = waves * (kFixedUs + (S > 1 ? kClusterUs : 0.f) + bytes_per_wave / (gbs * 1e3f));
    if (t < best_t) { best_t = t; best = S; }
  }
  return best;
}

template <int BN, int STAGES, bool DUAL>
int launch(const CUtensorMap& tw, const TokenMaps& tx, GemmParams p, cudaStream_t stream) {
  auto kern = dense_gemm_kernel<BN, STAGES, DUAL>;
  constexpr int smem = smem_bytes<BN, STAGES, DUAL>();
  constexpr int ring = STAGES * (BM * 128 * (DUAL ? 2 : 1) + BN * 128);
  static_assert(BN * BM * 4 <= ring, "fp32 staging tile must fit inside the pipeline ring");
  {
    cudaError_t e = fi::ensure_dynamic_smem(kern, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  if (p.splits <= 0) p.splits = pick_splits<BN, STAGES, DUAL>(p, smem);
  if (BN * BM * 4 * ((DUAL && p.splits > 1) ? 2 : 1) > ring) return -12;
  const int nx = (p.N + BM - 1) / BM;
  if (p.x_full != nullptr) {   // staged all-gather: about 64 copier CTAs in the first rows of the grid
    p.copy_rows = (64 + nx * p.splits - 1) / (nx * p.splits);   // (x 192 threads x 8 loads of 16 bytes in flight)
  }
  return static_cast<int>(launch_kernel(kern, dim3(nx, (p.T + BN - 1) / BN + p.copy_rows, p.splits),
                                        dim3(kThreads), smem, stream, p.splits, tw, tx, p));
}

template <bool DUAL>
int dispatch(int bn, const CUtensorMap& tw, const TokenMaps& tx, const GemmParams& p,
             cudaStream_t s) {
  switch (bn) {
    case 16: return launch<16, DUAL ? 5 : 8, DUAL>(tw, tx, p, s);
    case 32: return launch<32, DUAL ? 5 : 8, DUAL>(tw, tx, p, s);
    case 64: return launch<64, DUAL ? 4 : 6, DUAL>(tw, tx, p, s);
    case 128: return launch<128, DUAL ? 2 : 3, DUAL>(tw, tx, p, s);
    default: return launch<256, DUAL ? 3 : 4, DUAL>(tw, tx, p, s);
  }
}

}  // namespace

// Token-tile choice: the smallest tile that covers T up to 128; 128 for everything larger (two CTAs
// fit per SM and overlap each other's epilogue); 256 only on request.
extern "C" int fi_dense_gemm_pick_bn(int T) {
  if (T <= 16) return 16;
  if (T <= 32) return 32;
  if (T <= 64) return 64;
  return 128;
}

// C = X W^T with optional epilogue.  All pointers are device pointers; nothing is allocated.
//   dtype: 0 = bf16, 1 = fp16 (X, W, bias; C/residual too unless out_fp32)
//   dual_rows > 0: gated mode, W holds [gate rows; up rows], N must equal dual_rows
//   splits: 0 = choose automatically, else the split-K cluster size (1..8)
//   bn: 0 = choose automatically
// Returns 0 or a negative argument error / positive CUDA error code.
static int fi_dense_gemm_impl(const void* X, const void* W, void* C, const void* bias,
                             const void* residual, int T, int N, int K, int ldx, int ldw, int ldc,
                             int act, int dual_rows, int out_fp32, int dtype, int splits, int bn,
                             int* status, void* stream,
                             const FiComm* comm, float rms_eps = 0.f, int w_dynamic = 0,
                             const FiRope* rope = nullptr) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (rms_eps > 0.f && (K % BK) != 0) return -21;   // the sum of squares reads whole 64-wide K blocks
  if ((K % 8) != 0 || (ldc % 8) != 0 || (reinterpret_cast<uintptr_t>(C) & 15) != 0) return -10;
  if (dual_rows > 0 && N != dual_rows) return -11;
  if (bn == 0) bn = fi_dense_gemm_pick_bn(T);
  const int w_rows = dual_rows > 0 ? 2 * dual_rows : N;
  CUtensorMap tw;
  TokenMaps tx;
  int r = make_tmap_2d_16bit_sw128(&tw, W, w_rows, K, ldw, BM);
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
    if (comm->x_full != 0) {
      if (T != comm->ag_world * comm->ag_rows_per_rank || ldx != K || (bn % 8) != 0) return -22;
      r = make_tmap_2d_16bit_sw128(&tx.m[kStagedMap], reinterpret_cast<const void*>(comm->x_full), T, K, K, bn);
      if (r != 0) return r * 100 - 3;
    }
  } else {
    r = make_tmap_2d_16bit_sw128(&tx.m[0], X, T, K, ldx, bn);
    if (r != 0) return r * 100 - 2;
  }
  const int kb_total = (K + BK - 1) / BK;
  if (splits > 8) splits = 8;
  if (splits > kb_total) splits = kb_total;
  // The fp32 staging tile(s) alias the pipeline ring.  Gated mode with split-K parks two tiles
  // (gate and up partials), which only fits for token tiles up to 64; large token tiles have
  // plenty of CTAs anyway, so they never split.
  if (bn >= 128 && (dual_rows > 0 || bn > 128)) splits = 1;
  GemmParams p;
  p.C = C; p.bias = bias; p.residual = residual;
  p.T = T; p.N = N; p.K = K; p.ldc = ldc;
  p.dual_rows = dual_rows; p.act = act; p.out_fp32 = out_fp32; p.is_fp16 = dtype == 1;
  p.splits = splits; p.status = status;
  p.tile_expert = nullptr; p.tile_row0 = nullptr; p.tile_rows = nullptr; p.n_tiles = nullptr; p.expert_rows = 0; p.grid_tiles = 0;
  p.comm_mode = 0; p.world = 1; p.rank = 0; p.rows_per_rank = 0; p.xfer_16bit = 0; p.comm_phases = 0; p.trace = g_plain_trace;
  p.rms_eps = rms_eps; p.w_dynamic = w_dynamic;
  p.x_full = nullptr; p.ag_flags = nullptr; p.copy_rows = 0;
  for (int d = 0; d < kMaxRanks; ++d) p.x_peers[d] = 0;
  p.rope_cs = nullptr; p.rope_pos = nullptr; p.rope_slots = nullptr; p.k_cache = nullptr; p.v_cache = nullptr;
  p.rope_nh = p.rope_nkv = p.rope_hd = p.rope_bs = 0;
  if (rope != nullptr) {
    const int hd = rope->head_dim;
    if ((hd != 64 && hd != 128) || N != (rope->num_heads + 2 * rope->num_kv_heads) * hd || dual_rows > 0 ||
        out_fp32 || residual != nullptr || comm != nullptr || act != 0 || rope->block_size <= 0)
      return -23;
    p.rope_cs = rope->cos_sin; p.rope_pos = rope->positions; p.rope_slots = rope->slot_mapping;
    p.k_cache = rope->k_cache; p.v_cache = rope->v_cache;
    p.rope_nh = rope->num_heads; p.rope_nkv = rope->num_kv_heads; p.rope_hd = hd; p.rope_bs = rope->block_size;
  }
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
    if (comm->ag_world > 1 && comm->x_full != 0) {
      p.x_full = reinterpret_cast<void*>(comm->x_full);
      p.ag_flags = reinterpret_cast<unsigned int*>(comm->ag_flags);
      for (int d = 0; d < kMaxRanks; ++d) p.x_peers[d] = comm->x_peers[d];
    }
    for (int d = 0; d < kMaxRanks; ++d) { p.recv[d] = comm->recv[d]; p.flags[d] = comm->flags[d]; p.ready[d] = comm->ready[d]; }
    if (comm->mode == kCommReduceScatter && (comm->rows_per_rank % bn) != 0) return -17;
    const long tiles = static_cast<long>((N + BM - 1) / BM) * ((T + bn - 1) / bn);
    if (comm->mode != 0 && tiles > kMaxCommTiles) return -18;
    if (comm->mode != 0 && (N % 8) != 0) return -19;
    // the two-hop all-reduce sends 16-bit results and owns chunks inside a 128-row tile
    if (comm->xfer_16bit == kXferTwoShot && (comm->mode != kCommAllReduce || out_fp32 || (ldc % 4) != 0)) return -24;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dual_rows > 0) return dispatch<true>(bn, tw, tx, p, s);
  return dispatch<false>(bn, tw, tx, p, s);
}

// Phase trace of plain GEMM launches (per-stage profile spans of the hot GEMM): `trace` is a device array of
// 8 unsigned 64-bit words, or null to switch the trace off.  Every later launch overwrites it.
extern "C" int fi_dense_gemm_set_trace(void* trace) {
  g_plain_trace = reinterpret_cast<unsigned long long*>(trace);
  return 0;
}

extern "C" int fi_dense_gemm(const void* X, const void* W, void* C, const void* bias,
                             const void* residual, int T, int N, int K, int ldx, int ldw, int ldc,
                             int act, int dual_rows, int out_fp32, int dtype, int splits, int bn,
                             int* status, void* stream) {
  return fi_dense_gemm_impl(X, W, C, bias, residual, T, N, K, ldx, ldw, ldc, act, dual_rows, out_fp32, dtype, splits, bn, status, stream, nullptr);
}

// RMSNorm fused in front of the GEMM: C = (X W'^T) * rsqrt(mean_k(X^2) + eps), W' = W * diag(norm weight)
// folded by the caller.  The kernel takes the per-token sum of squares from the token tiles it stages
// anyway, so the normalised activations never exist in memory.  K must be a multiple of 64.
extern "C" int fi_dense_gemm_rmsnorm(const void* X, const void* W, void* C, const void* bias,
                             const void* residual, int T, int N, int K, int ldx, int ldw, int ldc,
                             int act, int dual_rows, int out_fp32, int dtype, int splits, int bn,
                             float eps, int* status, void* stream) {
  if (!(eps > 0.f)) return -20;
  return fi_dense_gemm_impl(X, W, C, bias, residual, T, N, K, ldx, ldw, ldc, act, dual_rows, out_fp32, dtype, splits, bn, status, stream, nullptr, eps);
}

// Merged q|k|v projection with the rotary embedding and the KV-cache write in the epilogue (and,
// with eps > 0, the RMSNorm of the input rows in front): replaces GEMM + rotary/cache kernel for
// models with full-width rotary embedding, head_dim 64 or 128, no q/k norm and a 16-bit cache.
extern "C" int fi_dense_gemm_rope(const void* X, const void* W, void* C, const void* bias, int T, int N, int K,
                             int ldx, int ldw, int ldc, int dtype, int splits, int bn, float rms_eps,
                             const FiRope* rope, int* status, void* stream) {
  if (rope == nullptr) return -23;
  return fi_dense_gemm_impl(X, W, C, bias, nullptr, T, N, K, ldx, ldw, ldc, 0, 0, 0, dtype, splits, bn, status,
                            stream, nullptr, rms_eps, 0, rope);
}

// Same as fi_dense_gemm for a weight matrix that the preceding kernel on the stream produced (for
// example a dequantised scratch copy): the producer warp then reads nothing before the
// programmatic-launch wait.  fi_dense_gemm itself assumes weights that never change.
extern "C" int fi_dense_gemm_dynw(const void* X, const void* W, void* C, const void* bias,
                             const void* residual, int T, int N, int K, int ldx, int ldw, int ldc,
                             int act, int dual_rows, int out_fp32, int dtype, int splits, int bn,
                             int* status, void* stream) {
  return fi_dense_gemm_impl(X, W, C, bias, residual, T, N, K, ldx, ldw, ldc, act, dual_rows, out_fp32, dtype, splits, bn, status, stream, nullptr, 0.f, 1);
}

// Same GEMM with a fused collective and/or an all-gathered token operand (see comm_desc.h).
extern "C" int fi_dense_gemm_comm(const void* X, const void* W, void* C, const void* bias,
                             const void* residual, int T, int N, int K, int ldx, int ldw, int ldc,
                             int act, int dual_rows, int out_fp32, int dtype, int splits, int bn,
                             int* status, void* stream,
                             const FiComm* comm) {
  return fi_dense_gemm_impl(X, W, C, bias, residual, T, N, K, ldx, ldw, ldc, act, dual_rows, out_fp32, dtype, splits, bn, status, stream, comm);
}
