// Persistent dense GEMM for prefill-sized token counts on sm_100a.
//
// Same operand roles as dense_gemm.cu (weight rows on the UMMA M side, tokens on N, both K-major
// with the 128-byte swizzle, TMA -> shared memory -> tcgen05.mma -> TMEM), but every CTA walks a list
// of output tiles and keeps TWO accumulators in tensor memory: while the four epilogue warps drain
// accumulator b (tcgen05.ld -> bias / residual / gated activation -> global), the MMA warp is
// already filling accumulator b^1 with the next tile and the TMA warp is several k-blocks ahead of
// it.  With tiles of only 32 k-blocks (K = 2048) the epilogue is a third of a tile's time, which the
// one-tile-per-CTA kernel pays in full; here it overlaps the next main loop.
//
//   C[T, N] = act(X[T, K] W[N, K]^T) + bias + residual           (dual_rows == 0)
//   C[T, I] = act(X Wg^T) * (X Wu^T)   with W = [Wg; Wu]          (dual_rows == I)
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2..5 epilogue.
// Barriers: full/empty per pipeline stage (running across tiles), acc_full/acc_empty per accumulator.
// Tile order: consecutive CTAs take different weight tiles of the same 128 tokens, so the token tile
// is shared through L2 and the weights (a few MB per layer) stay L2-resident across token tiles.
// Every wait is bounded; a timeout records a status code and the kernel winds down normally.
// The reference runs these products through torch.nn.functional.linear (vllm/model_executor/layers/
// lite_linear.py:46-62).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../common/tensormap.h"

using namespace fi;

namespace {

constexpr int BM = 128;   // weight rows per tile (UMMA M)
constexpr int BN = 128;   // tokens per tile (UMMA N)
constexpr int BK = 64;    // k-block: 64 16-bit values = one 128-byte swizzled row
constexpr int kThreads = 192;

struct PParams {
  void* C;
  const void* bias;
  const void* residual;
  int T, N, K, ldc;
  int dual_rows, act, is_fp16;
  int second_off;   // weight rows between the two A tiles of a CTA: dual_rows (gated) or 128 (plain, 256-row tile)
  int rows_per_tile;   // output rows (of N) one tile covers: 128 (gated or single) or 256
  int n_tiles_n, n_tiles;
  int* status;
};

__device__ __forceinline__ float act_f(float g, int act) {
  if (act == 1) return g / (1.f + __expf(-g));
  if (act == 2) {
    const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return g / (1.f + __expf(-2.f * inner));
  }
  return g;
}
__device__ __forceinline__ float ld16(const void* p, size_t i, int is_fp16) {
  if (is_fp16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st16(void* p, size_t i, float v, int is_fp16) {
  if (is_fp16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

template <int STAGES, bool DUAL>
__global__ void __launch_bounds__(kThreads)
dense_gemm_persistent_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                             const PParams p) {
  constexpr int A_BYTES = BM * 128;
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = A_BYTES * (DUAL ? 2 : 1) + B_BYTES;
  constexpr int ACC_COLS = DUAL ? 2 * BN : BN;          // TMEM columns of one accumulator (gate | up)
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;          // two accumulators: 256 or 512 columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;    // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;         // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stage = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(tmem_slot) + 16);   // [4 warps][16 tokens][32 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
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
  pdl_wait();
  const int kb_total = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmap_w);
      tma_prefetch_desc(&tmap_x);
      long it = 0;
      for (int tile = blockIdx.x; tile < p.n_tiles && !*aborted; tile += gridDim.x) {
        const int n0 = (tile % p.n_tiles_n) * p.rows_per_tile;
        const int t0 = (tile / p.n_tiles_n) * BN;
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = static_cast<int>(it % STAGES);
          const uint32_t ph = static_cast<uint32_t>(it / STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u)) {
            set_status(p.status, kStatusTimeoutEmpty);
            *aborted = 1;
            break;
          }
          uint8_t* a = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          tma_load_2d(a, &tmap_w, &full_bar[s], kb * BK, n0);
          if (DUAL) tma_load_2d(a + A_BYTES, &tmap_w, &full_bar[s], kb * BK, p.second_off + n0);
          tma_load_2d(a + A_BYTES * (DUAL ? 2 : 1), &tmap_x, &full_bar[s], kb * BK, t0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_f16(p.is_fp16 ? 0 : 1, BM, BN);
      long it = 0;
      int local = 0;
      for (int tile = blockIdx.x; tile < p.n_tiles && !*aborted; tile += gridDim.x, ++local) {
        const int b = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1);
        if (!mbar_wait(&acc_empty[b], (use & 1u) ^ 1u)) {     // epilogue has drained this accumulator
          set_status(p.status, kStatusTimeoutAccum);
          *aborted = 1;
          break;
        }
        tc_fence_after();
        const uint32_t acc = tmem_base + static_cast<uint32_t>(b * ACC_COLS);
        bool ok = true;
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = static_cast<int>(it % STAGES);
          const uint32_t ph = static_cast<uint32_t>(it / STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], ph)) {
            set_status(p.status, kStatusTimeoutFull);
            *aborted = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES * (DUAL ? 2 : 1);
          const uint64_t da = umma_desc_sw128_kmajor(a_addr);
          const uint64_t db = umma_desc_sw128_kmajor(b_addr);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
            umma_f16(acc, da + 2 * k, db + 2 * k, idesc, accum);
            if (DUAL) {
              const uint64_t da2 = umma_desc_sw128_kmajor(a_addr + A_BYTES);
              umma_f16(acc + BN, da2 + 2 * k, db + 2 * k, idesc, accum);
            }
          }
          umma_commit(&empty_bar[s]);
        }
        if (!ok) break;
        umma_commit(&acc_full[b]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps 2..5
    const int q = warp & 3;                     // TMEM lane quarter this warp may read
    const int n_local = q * 32 + lane;          // weight row inside the tile
    int local = 0;
    for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++local) {
      const int b = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1);
      if (*aborted || !mbar_wait(&acc_full[b], use & 1u)) {
        if (!*aborted) { set_status(p.status, kStatusTimeoutAccum); *aborted = 1; }
        break;
      }
      tc_fence_after();
      const int n0 = (tile % p.n_tiles_n) * p.rows_per_tile;
      const int t0 = (tile / p.n_tiles_n) * BN;
      const bool gated = p.dual_rows > 0;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(b * ACC_COLS);
      // Each thread owns one weight row of the accumulator (a TMEM lane) but the output is
      // token-major: a batch of 16 tokens x 32 rows goes through this warp's shared-memory patch as
      // fp32 and comes back as 8-row vectors, so bias / residual / store are 16-byte accesses.
      float* patch = stage + (warp - 2) * (16 * 32);
      const int vc = lane & 3;                // which 8-row chunk of the warp's 32 rows this lane finishes
      const int vj = lane >> 2;               // tokens vj and vj + 8 of the batch
      // gated: one output row per thread (gate and up combined); plain wide tile: two rows, 128 apart
      const int halves = (DUAL && !gated) ? 2 : 1;
      for (int hh = 0; hh < halves; ++hh) {
        const int nv = n0 + hh * BM + q * 32 + vc * 8;      // first of the 8 rows this lane stores
        const bool nv_ok = nv < p.N;
        float bias8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) bias8[e] = (p.bias != nullptr && nv_ok) ? ld16(p.bias, nv + e, p.is_fp16) : 0.f;
        // the residual values of a batch are requested one batch ahead, so their latency hides behind
        // the TMEM read and the transposition of the batch in front
        auto load_res = [&](int c0, uint4 (&dst)[2]) {
#pragma unroll
          for (int rep = 0; rep < 2; ++rep) {
            const int t = t0 + c0 + vj + rep * 8;
            dst[rep] = make_uint4(0, 0, 0, 0);
            if (p.residual != nullptr && nv_ok && c0 < BN && t < p.T)
              dst[rep] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.residual) +
                                                         static_cast<size_t>(t) * p.ldc + nv);
          }
        };
        uint4 res_cur[2], res_next[2];
        load_res(0, res_cur);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t r[16], u[16];
          tmem_ld_x16(taddr + hh * BN + c0, r);
          if (DUAL && gated) tmem_ld_x16(taddr + BN + c0, u);
          load_res(c0 + 16, res_next);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float v = __uint_as_float(r[j]);
            if (DUAL && gated) v = act_f(v, p.act) * __uint_as_float(u[j]);
            else v = act_f(v, p.act);
            patch[j * 32 + lane] = v;
          }
          __syncwarp();
#pragma unroll
          for (int rep = 0; rep < 2; ++rep) {
            const int j = vj + rep * 8;
            const int t = t0 + c0 + j;
            if (nv_ok && t < p.T) {
              const float4 a0 = *reinterpret_cast<const float4*>(patch + j * 32 + vc * 8);
              const float4 a1 = *reinterpret_cast<const float4*>(patch + j * 32 + vc * 8 + 4);
              float v[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
              const size_t off = static_cast<size_t>(t) * p.ldc + nv;
              const uint4 raw = res_cur[rep];
              const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
              uint32_t ow[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float lo = v[2 * e] + bias8[2 * e], hi = v[2 * e + 1] + bias8[2 * e + 1];
                if (p.is_fp16) {
                  const __half2 rr = *reinterpret_cast<const __half2*>(&rw[e]);
                  lo += __low2float(rr); hi += __high2float(rr);
                  const __half2 o = __floats2half2_rn(lo, hi);
                  ow[e] = *reinterpret_cast<const uint32_t*>(&o);
                } else {
                  lo += __uint_as_float(rw[e] << 16); hi += __uint_as_float(rw[e] & 0xffff0000u);
                  const __nv_bfloat162 o = __floats2bfloat162_rn(lo, hi);
                  ow[e] = *reinterpret_cast<const uint32_t*>(&o);
                }
              }
              *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.C) + off) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
          }
          __syncwarp();
          res_cur[0] = res_next[0];
          res_cur[1] = res_next[1];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);   // this warp's quarter of the accumulator is free again
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int STAGES, bool DUAL>
int launch(const CUtensorMap& tw, const CUtensorMap& tx, const PParams& p, cudaStream_t stream) {
  auto kern = dense_gemm_persistent_kernel<STAGES, DUAL>;
  constexpr int smem = STAGES * (BM * 128 * (DUAL ? 2 : 1) + BN * 128) + (2 * STAGES + 4) * 8 + 16 + 4 * 16 * 32 * 4 + 1024;
  {
    cudaError_t e = fi::ensure_dynamic_smem(kern, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int grid = p.n_tiles < sms ? p.n_tiles : sms;
  return static_cast<int>(launch_kernel(kern, dim3(grid), dim3(kThreads), smem, stream, 0, tw, tx, p));
}

}  // namespace

// Prefill-sized dense GEMM (see the top of the file).  dtype: 0 bf16, 1 fp16 for X, W, bias, residual and
// C.  dual_rows > 0: gated mode, W holds [gate rows; up rows] and N must equal dual_rows.  Nothing is
// allocated; returns 0, a negative argument error or a positive CUDA error code.
extern "C" int fi_dense_gemm_persistent(const void* X, const void* W, void* C, const void* bias, const void* residual,
                                        int T, int N, int K, int ldx, int ldw, int ldc, int act, int dual_rows,
                                        int dtype, int* status, void* stream) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) != 0 || (ldx % 8) != 0 || (ldw % 8) != 0 || (N % 8) != 0 || (ldc % 8) != 0 ||
      (reinterpret_cast<uintptr_t>(C) & 15) != 0 || (residual != nullptr && (reinterpret_cast<uintptr_t>(residual) & 15) != 0))
    return -10;
  if (dual_rows > 0 && N != dual_rows) return -11;
  const int w_rows = dual_rows > 0 ? 2 * dual_rows : N;
  CUtensorMap tw, tx;
  int r = make_tmap_2d_16bit_sw128(&tw, W, w_rows, K, ldw, BM);
  if (r != 0) return r * 100 - 1;
  r = make_tmap_2d_16bit_sw128(&tx, X, T, K, ldx, BN);
  if (r != 0) return r * 100 - 2;
  PParams p;
  p.C = C; p.bias = bias; p.residual = residual;
  p.T = T; p.N = N; p.K = K; p.ldc = ldc;
  p.dual_rows = dual_rows; p.act = act; p.is_fp16 = dtype == 1;
  // plain products use a 256-row tile (two A tiles per stage against one token tile), which halves the
  // L2 -> shared-memory traffic per FLOP; 128 x 128 tiles were L2-bandwidth-bound at ~55 % of peak
  const bool wide = dual_rows == 0 && N > BM;
  p.second_off = dual_rows > 0 ? dual_rows : BM;
  p.rows_per_tile = wide ? 2 * BM : BM;
  p.n_tiles_n = (N + p.rows_per_tile - 1) / p.rows_per_tile;
  p.n_tiles = p.n_tiles_n * ((T + BN - 1) / BN);
  p.status = status;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dual_rows > 0 || wide) return launch<4, true>(tw, tx, p, s);
  return launch<6, false>(tw, tx, p, s);
}
