// Paged attention for sm_100a: split-KV decode (one query token per sequence, all query heads of a
// KV head packed into one tensor-core tile) and varlen chunked-prefill flash attention reading the
// paged cache.  Both support 16-bit or fp8-e4m3 KV (per-tensor scale), sliding windows and
// logit soft-capping, head_dim 64/128/256, any block size.
//
// KV cache layout: [num_blocks, n_kv_heads, block_size, head_dim]; block id 0 is the null block.
//
// These are bandwidth-bound (decode) or a small share of prefill FLOPs for the served shapes, so
// they use register-level mma.sync tiles with cp.async double buffering rather than TMEM.
//
// Counterpart in the reference: vllm/kernels/triton/paged_attention.py:306-759 (one program per
// (sequence, query head), also used for prefill by expanding every query token into its own row,
// vllm/engine/lite_engine.py:53-104).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../common/launch.cuh"
#include "paged_attention_noalloc.h"
#include <atomic>
#include <cooperative_groups.h>
#include <math_constants.h>
#include <stdint.h>
#include <stdio.h>

namespace {

constexpr float kLog2e = 1.4426950408889634f;

template <typename T> struct MmaT;
template <> struct MmaT<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float* d, const uint32_t* a, const uint32_t* b) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
  static __device__ __forceinline__ uint32_t pack(float x, float y) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16(v); }
};
template <> struct MmaT<__half> {
  static __device__ __forceinline__ void mma(float* d, const uint32_t* a, const uint32_t* b) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
  static __device__ __forceinline__ uint32_t pack(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half(v); }
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void ldsm_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src),
               "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// Row-major [rows][HD] 16-bit tile with the 16-byte chunks of a row XOR-swizzled by (row & 7).
template <int HD>
__device__ __forceinline__ int tile_off(int row, int chunk) {  // in 16-bit elements
  return row * HD + ((chunk ^ (row & 7)) << 3);
}

struct AttnParams {
  const void* q;        // query rows: token t, head h at q + (t * q_stride + h * HD) elements
  long q_stride;
  const void* k_cache;
  const void* v_cache;
  void* out;            // [T, nh * HD]
  const int* block_tables;  // [B, max_blocks]
  const int* seq_lens;      // [B] KV length including this step's tokens
  const int* cu_q;          // [B + 1] query token offsets (prefill); null for decode
  float* ws_o;              // decode partials [B, nh, splits, HD]
  float* ws_ml;             // decode partials [B, nh, splits, 2]
  int max_blocks, block_size, nh, nkv, window;  // window <= 0: none
  float sm_scale, softcap, k_scale, v_scale;
  // kv_fp8 is the cache format: 0 = 16-bit, 1 = e4m3 with one scale per tensor (k_scale / v_scale),
  // 2 = e4m3 with one scale per (token, kv head) row, 3 = packed int4 (low nibbles = first half of the
  // channels, high nibbles = second half, two's complement in [-7, 7]) with one scale per row.
  // Formats 2 and 3 read their fp32 row scales from k_scales / v_scales [num_blocks, nkv, block_size].
  int kv_fp8, splits;
  const float* k_scales;
  const float* v_scales;
  // optional [B * gridDim.y] zero-initialised tickets: the split CTA that arrives last merges the
  // partials itself (and resets the ticket), so no separate merge launch is needed
  unsigned int* merge_tickets;
  // > 0: the split CTAs of one (sequence, KV head group) form a thread-block cluster and merge their
  // partials through distributed shared memory at this byte offset of the dynamic shared memory
  // ([16][HD] sums + [16][2] max/denominator per CTA): no global scratch, no tickets, no second launch
  int cluster_off;
};

// Load `rows` KV tokens starting at token tok0 of sequence b / kv head kvh into a swizzled tile.
// Tokens outside [lo, hi) are zero-filled.
template <typename T, int HD, int ROWS, int THREADS>
__device__ __forceinline__ void load_kv_tile(T* tile, const void* cache, const int* bt,
                                             int block_size, int nkv, int kvh, int tok0, int lo,
                                             int hi, int fp8, const float* scales = nullptr) {
  constexpr int CPR = HD / 8;  // 16-byte chunks (of 16-bit elements) per row
  if (fp8 == 3) {
    // packed int4 with a scale per row: 16 bytes hold channels [16c, 16c+16) in their low nibbles and
    // channels [HD/2 + 16c, HD/2 + 16c + 16) in their high nibbles
    constexpr int CPR4 = HD / 32;
    for (int i = threadIdx.x; i < ROWS * CPR4; i += THREADS) {
      const int r = i / CPR4, c = i % CPR4;
      const int tok = tok0 + r;
      const bool valid = tok >= lo && tok < hi;
      uint4 raw = make_uint4(0, 0, 0, 0);
      float sc = 0.f;
      if (valid) {
        const int blk = bt[tok / block_size];
        const long rowi = (static_cast<long>(blk) * nkv + kvh) * block_size + tok % block_size;
        raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(cache) + rowi * (HD / 2) + c * 16);
        sc = scales[rowi];
      }
      const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
      T lo16[16], hi16[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        lo16[j] = MmaT<T>::from_f(static_cast<float>(static_cast<int>((b[j] & 0x0F) ^ 8) - 8) * sc);
        hi16[j] = MmaT<T>::from_f(static_cast<float>(static_cast<int>((b[j] >> 4) ^ 8) - 8) * sc);
      }
      *reinterpret_cast<uint4*>(tile + tile_off<HD>(r, 2 * c)) = *reinterpret_cast<uint4*>(&lo16[0]);
      *reinterpret_cast<uint4*>(tile + tile_off<HD>(r, 2 * c + 1)) = *reinterpret_cast<uint4*>(&lo16[8]);
      *reinterpret_cast<uint4*>(tile + tile_off<HD>(r, HD / 16 + 2 * c)) = *reinterpret_cast<uint4*>(&hi16[0]);
      *reinterpret_cast<uint4*>(tile + tile_off<HD>(r, HD / 16 + 2 * c + 1)) = *reinterpret_cast<uint4*>(&hi16[8]);
    }
    return;
  }
  if (!fp8) {
    for (int i = threadIdx.x; i < ROWS * CPR; i += THREADS) {
      const int r = i / CPR, c = i % CPR;
      const int tok = tok0 + r;
      const bool valid = tok >= lo && tok < hi;
      const T* src = reinterpret_cast<const T*>(cache);
      if (valid) {
        const int blk = bt[tok / block_size];
        src += ((static_cast<long>(blk) * nkv + kvh) * block_size + tok % block_size) * HD + c * 8;
      }
      cp_async16(tile + tile_off<HD>(r, c), src, valid);
    }
  } else {
    // fp8: 16 values per 16-byte load, converted to two 16-byte chunks of T
    constexpr int CPR8 = HD / 16;
    for (int i = threadIdx.x; i < ROWS * CPR8; i += THREADS) {
      const int r = i / CPR8, c = i % CPR8;
      const int tok = tok0 + r;
      const bool valid = tok >= lo && tok < hi;
      uint4 raw = make_uint4(0, 0, 0, 0);
      float sc = 1.f;
      if (valid) {
        const int blk = bt[tok / block_size];
        const long rowi = (static_cast<long>(blk) * nkv + kvh) * block_size + tok % block_size;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(cache) + rowi * HD + c * 16;
        raw = *reinterpret_cast<const uint4*>(src);
        if (fp8 == 2) sc = scales[rowi];      // row-scaled e4m3: the true value is stored value x row scale
      }
      const __nv_fp8_e4m3* f8 = reinterpret_cast<const __nv_fp8_e4m3*>(&raw);
      T tmp[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) tmp[j] = MmaT<T>::from_f(static_cast<float>(f8[j]) * sc);
      *reinterpret_cast<uint4*>(tile + tile_off<HD>(r, 2 * c)) = *reinterpret_cast<uint4*>(&tmp[0]);
      *reinterpret_cast<uint4*>(tile + tile_off<HD>(r, 2 * c + 1)) = *reinterpret_cast<uint4*>(&tmp[8]);
    }
  }
}

__device__ __forceinline__ float softcap_f(float s, float cap) {
  return cap > 0.f ? cap * tanhf(s / cap) : s;
}

// ------------------------------------------------------------------------------ decode
// grid (splits, nkv * head_groups, B); 128 threads.  Rows of the 16-row tile = query heads of one
// KV head (up to 16 per group).  Each warp owns 16 of the 64 tokens of a chunk.
template <typename T, int HD>
__global__ void __launch_bounds__(128) paged_decode_kernel(const AttnParams p) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  constexpr int CH = 64;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);        // [16][HD]
  T* sK = sQ + 16 * HD;                          // [2][CH][HD]
  T* sV = sK + 2 * CH * HD;                      // [2][CH][HD]
  const int split = blockIdx.x;
  const int G = p.nh / p.nkv;
  const int groups = (G + 15) / 16;
  const int kvh = blockIdx.y / groups;
  const int grp = blockIdx.y % groups;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_here = min(16, G - grp * 16);
  const int head0 = kvh * G + grp * 16;
  const int seq_len = p.seq_lens[b];
  const int* bt = p.block_tables + static_cast<long>(b) * p.max_blocks;
  const int lo = p.window > 0 ? max(0, seq_len - p.window) : 0;
  const int first_chunk = lo / CH;
  const int n_chunks = (seq_len + CH - 1) / CH - first_chunk;
  const int per = (n_chunks + p.splits - 1) / p.splits;
  const int c_begin = first_chunk + split * per;
  const int c_end = min(first_chunk + n_chunks, c_begin + per);

  // stage Q (zero rows beyond heads_here)
  for (int i = threadIdx.x; i < 16 * (HD / 8); i += 128) {
    const int r = i / (HD / 8), c = i % (HD / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < heads_here)
      v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.q) +
                                          static_cast<long>(b) * p.q_stride +
                                          static_cast<long>(head0 + r) * HD + c * 8);
    *reinterpret_cast<uint4*>(sQ + tile_off<HD>(r, c)) = v;
  }
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  const float scale = p.sm_scale * (p.kv_fp8 == 1 ? p.k_scale : 1.f);

  if (c_begin < c_end) {
    load_kv_tile<T, HD, CH, 128>(sK, p.k_cache, bt, p.block_size, p.nkv, kvh, c_begin * CH, lo, seq_len, p.kv_fp8, p.k_scales);
    load_kv_tile<T, HD, CH, 128>(sV, p.v_cache, bt, p.block_size, p.nkv, kvh, c_begin * CH, lo, seq_len, p.kv_fp8, p.v_scales);
  }
  cp_async_commit();
  for (int c = c_begin; c < c_end; ++c) {
    const int buf = (c - c_begin) & 1;
    if (c + 1 < c_end) {
      load_kv_tile<T, HD, CH, 128>(sK + (buf ^ 1) * CH * HD, p.k_cache, bt, p.block_size, p.nkv, kvh, (c + 1) * CH, lo, seq_len, p.kv_fp8, p.k_scales);
      load_kv_tile<T, HD, CH, 128>(sV + (buf ^ 1) * CH * HD, p.v_cache, bt, p.block_size, p.nkv, kvh, (c + 1) * CH, lo, seq_len, p.kv_fp8, p.v_scales);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const T* K = sK + buf * CH * HD;
    const T* V = sV + buf * CH * HD;
    const int tok_base = c * CH + warp * 16;
    if (tok_base < seq_len && tok_base + 16 > lo) {
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t a[4], kb[4];
        // A (Q): matrices (rows 0-7,k 0-7) (rows 8-15,k 0-7) (rows 0-7,k 8-15) (rows 8-15,k 8-15)
        ldsm_x4(a, smem_addr(sQ + tile_off<HD>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4))));
        // B (K): matrices (tok 0-7,d 0-7) (tok 0-7,d 8-15) (tok 8-15,d 0-7) (tok 8-15,d 8-15)
        ldsm_x4(kb, smem_addr(K + tile_off<HD>(warp * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1))));
        MmaT<T>::mma(s[0], a, kb);
        MmaT<T>::mma(s[1], a, kb + 2);
      }
      float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = tok_base + j * 8 + (lane & 3) * 2 + (e & 1);
          float v = softcap_f(s[j][e] * scale, p.softcap);
          if (tok >= seq_len || tok < lo) v = -CUDART_INF_F;
          s[j][e] = v;
          if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
      const float a0 = nm0 == -CUDART_INF_F ? 1.f : exp2f((m0 - nm0) * kLog2e);
      const float a1 = nm1 == -CUDART_INF_F ? 1.f : exp2f((m1 - nm1) * kLog2e);
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float nm = e < 2 ? nm0 : nm1;
          const float pv = nm == -CUDART_INF_F ? 0.f : exp2f((s[j][e] - nm) * kLog2e);
          s[j][e] = pv;
          if (e < 2) rs0 += pv; else rs1 += pv;
        }
      }
      l0 = l0 * a0 + rs0; l1 = l1 * a1 + rs1; m0 = nm0; m1 = nm1;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
      uint32_t pa[4] = {MmaT<T>::pack(s[0][0], s[0][1]), MmaT<T>::pack(s[0][2], s[0][3]),
                        MmaT<T>::pack(s[1][0], s[1][1]), MmaT<T>::pack(s[1][2], s[1][3])};
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t vb[4];
        // B (V, transposed): matrices (tok 0-7,d-tile 2dp) (tok 8-15,2dp) (tok 0-7,2dp+1) (tok 8-15,2dp+1)
        ldsm_x4_t(vb, smem_addr(V + tile_off<HD>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4))));
        MmaT<T>::mma(o[2 * dp], pa, vb);
        MmaT<T>::mma(o[2 * dp + 1], pa, vb + 2);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  // quad-reduce the row sums
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  // merge the four warps through shared memory (aliases the KV buffers)
  __syncthreads();
  float* mO = reinterpret_cast<float*>(sK);              // [4][16][HD]
  float* mML = mO + 4 * 16 * HD;                         // [4][16][2]
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      const int d = i * 8 + (lane & 3) * 2;
      mO[(warp * 16 + r0) * HD + d] = o[i][0]; mO[(warp * 16 + r0) * HD + d + 1] = o[i][1];
      mO[(warp * 16 + r1) * HD + d] = o[i][2]; mO[(warp * 16 + r1) * HD + d + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      mML[(warp * 16 + r0) * 2] = m0; mML[(warp * 16 + r0) * 2 + 1] = l0;
      mML[(warp * 16 + r1) * 2] = m1; mML[(warp * 16 + r1) * 2 + 1] = l1;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < heads_here * HD; i += 128) {
    const int r = i / HD, d = i % HD;
    float m = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, mML[(w * 16 + r) * 2]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mML[(w * 16 + r) * 2];
      const float f = mw == -CUDART_INF_F ? 0.f : exp2f((mw - m) * kLog2e);
      acc += f * mO[(w * 16 + r) * HD + d];
      l += f * mML[(w * 16 + r) * 2 + 1];
    }
    const int head = head0 + r;
    if (p.splits == 1) {
      const float v = l > 0.f ? acc / l * (p.kv_fp8 == 1 ? p.v_scale : 1.f) : 0.f;
      reinterpret_cast<T*>(p.out)[(static_cast<long>(b) * p.nh + head) * HD + d] = MmaT<T>::from_f(v);
    } else {
      const long base = (static_cast<long>(b) * p.nh + head) * p.splits + split;
      p.ws_o[base * HD + d] = acc;
      if (d == 0) { p.ws_ml[base * 2] = m; p.ws_ml[base * 2 + 1] = l; }
    }
  }
}

// ------------------------------------------------------------------------------ decode, v2
// Same math and grid as paged_decode_kernel, different data movement: every warp runs its OWN
// multi-stage cp.async pipeline over 16-token groups (one KV block slice each), so the main loop has
// no CTA-wide barrier and each SM keeps tens of KB of KV reads in flight.  Block-table entries are
// fetched 32 groups at a time into registers and handed out by shuffle.  Needs block_size % 16 == 0.
template <typename T, int HD, int NST>
__global__ void __launch_bounds__(128) paged_decode_v2_kernel(const AttnParams p) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int TILE = 16 * HD;                      // elements of one 16-token tile
  T* sQ = reinterpret_cast<T*>(smem_raw);            // [16][HD]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool fp8 = p.kv_fp8 == 1;     // row-scaled caches (formats 2, 3) take the other decode kernel
  // per-warp regions: raw K/V stages (+ conversion tiles when the cache is fp8)
  const int raw_tile_bytes = fp8 ? TILE : TILE * 2;
  const int warp_bytes = NST * 2 * raw_tile_bytes + (fp8 ? 2 * TILE * 2 : 0);
  uint8_t* wbase = smem_raw + 16 * HD * 2 + warp * warp_bytes;
  uint8_t* rawK = wbase;
  uint8_t* rawV = wbase + NST * raw_tile_bytes;
  T* convK = reinterpret_cast<T*>(wbase + NST * 2 * raw_tile_bytes);
  T* convV = convK + TILE;

  const int split = blockIdx.x;
  const int G = p.nh / p.nkv;
  const int groups = (G + 15) / 16;
  const int kvh = blockIdx.y / groups;
  const int grp = blockIdx.y % groups;
  const int b = blockIdx.z;
  const int heads_here = min(16, G - grp * 16);
  const int head0 = kvh * G + grp * 16;
  const int seq_len = p.seq_lens[b];
  const int* bt = p.block_tables + static_cast<long>(b) * p.max_blocks;
  const int lo = p.window > 0 ? max(0, seq_len - p.window) : 0;
  // 16-token groups of this CTA: [g_begin, g_end), dealt round-robin to the four warps
  const int first_g = lo / 16;
  const int n_groups = (seq_len + 15) / 16 - first_g;
  const int per = ((n_groups + p.splits - 1) / p.splits + 3) / 4 * 4;
  const int g_begin = first_g + split * per;
  const int g_end = min(first_g + n_groups, g_begin + per);
  const int my_n = (g_end - g_begin - warp + 3) / 4;   // groups of this warp (may be <= 0)

  for (int i = threadIdx.x; i < 16 * (HD / 8); i += 128) {
    const int r = i / (HD / 8), c = i % (HD / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < heads_here)
      v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.q) + static_cast<long>(b) * p.q_stride +
                                          static_cast<long>(head0 + r) * HD + c * 8);
    *reinterpret_cast<uint4*>(sQ + tile_off<HD>(r, c)) = v;
  }
  __syncthreads();

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  const float scale = p.sm_scale * (fp8 ? p.k_scale : 1.f);
  const int bpb = p.block_size / 16;                 // 16-token groups per KV block

  int bt_reg = 0;
  auto refill_bt = [&](int k0) {   // block ids of this warp's groups k0 .. k0+31
    const int g = g_begin + warp + 4 * (k0 + lane);
    bt_reg = (k0 + lane < my_n) ? bt[g / bpb] : 0;
  };
  auto issue = [&](int k) {        // start loading this warp's k-th group into stage k % NST
    if (k < my_n) {
      const int g = g_begin + warp + 4 * k;
      const int blk = __shfl_sync(0xffffffffu, bt_reg, k & 31);
      const long base = ((static_cast<long>(blk) * p.nkv + kvh) * p.block_size + (g % bpb) * 16) * HD;
      const int st = k % NST;
      if (!fp8) {
        const T* ksrc = reinterpret_cast<const T*>(p.k_cache) + base;
        const T* vsrc = reinterpret_cast<const T*>(p.v_cache) + base;
        T* kd = reinterpret_cast<T*>(rawK + st * raw_tile_bytes);
        T* vd = reinterpret_cast<T*>(rawV + st * raw_tile_bytes);
#pragma unroll
        for (int i = lane; i < 16 * (HD / 8); i += 32) {
          const int r = i / (HD / 8), c = i % (HD / 8);
          cp_async16(kd + tile_off<HD>(r, c), ksrc + i * 8, true);
          cp_async16(vd + tile_off<HD>(r, c), vsrc + i * 8, true);
        }
      } else {
        const uint8_t* ksrc = reinterpret_cast<const uint8_t*>(p.k_cache) + base;
        const uint8_t* vsrc = reinterpret_cast<const uint8_t*>(p.v_cache) + base;
#pragma unroll
        for (int i = lane; i < 16 * (HD / 16); i += 32) {   // linear copy of the raw bytes
          cp_async16(rawK + st * raw_tile_bytes + i * 16, ksrc + i * 16, true);
          cp_async16(rawV + st * raw_tile_bytes + i * 16, vsrc + i * 16, true);
        }
      }
    }
    cp_async_commit();
  };

  if (my_n > 0) refill_bt(0);
#pragma unroll
  for (int k = 0; k < NST - 1; ++k) issue(k);
  for (int k = 0; k < my_n; ++k) {
    if (((k + NST - 1) & 31) == 0 && k + NST - 1 < my_n) refill_bt(k + NST - 1);
    issue(k + NST - 1);
    cp_async_wait<NST - 1>();
    __syncwarp();
    const int st = k % NST;
    const T* K;
    const T* V;
    if (!fp8) {
      K = reinterpret_cast<const T*>(rawK + st * raw_tile_bytes);
      V = reinterpret_cast<const T*>(rawV + st * raw_tile_bytes);
    } else {
      // expand the raw e4m3 bytes of this group into swizzled 16-bit tiles
      for (int i = lane; i < 16 * (HD / 16); i += 32) {
        const int r = i / (HD / 16), c = i % (HD / 16);
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint4 raw = *reinterpret_cast<const uint4*>((which ? rawV : rawK) + st * raw_tile_bytes + i * 16);
          const __nv_fp8_e4m3* f8 = reinterpret_cast<const __nv_fp8_e4m3*>(&raw);
          T tmp[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) tmp[j] = MmaT<T>::from_f(static_cast<float>(f8[j]));
          T* dst = which ? convV : convK;
          *reinterpret_cast<uint4*>(dst + tile_off<HD>(r, 2 * c)) = *reinterpret_cast<uint4*>(&tmp[0]);
          *reinterpret_cast<uint4*>(dst + tile_off<HD>(r, 2 * c + 1)) = *reinterpret_cast<uint4*>(&tmp[8]);
        }
      }
      __syncwarp();
      K = convK;
      V = convV;
    }
    const int tok_base = (g_begin + warp + 4 * k) * 16;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t a[4], kb[4];
      ldsm_x4(a, smem_addr(sQ + tile_off<HD>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4))));
      ldsm_x4(kb, smem_addr(K + tile_off<HD>((lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1))));
      MmaT<T>::mma(s[0], a, kb);
      MmaT<T>::mma(s[1], a, kb + 2);
    }
    float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = tok_base + j * 8 + (lane & 3) * 2 + (e & 1);
        float v = softcap_f(s[j][e] * scale, p.softcap);
        if (tok >= seq_len || tok < lo) v = -CUDART_INF_F;
        s[j][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
    const float a0 = nm0 == -CUDART_INF_F ? 1.f : exp2f((m0 - nm0) * kLog2e);
    const float a1 = nm1 == -CUDART_INF_F ? 1.f : exp2f((m1 - nm1) * kLog2e);
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float nm = e < 2 ? nm0 : nm1;
        // tokens past seq_len inside a valid block hold stale cache data: their weight is exactly 0
        const float pv = nm == -CUDART_INF_F ? 0.f : exp2f((s[j][e] - nm) * kLog2e);
        s[j][e] = pv;
        if (e < 2) rs0 += pv; else rs1 += pv;
      }
    }
    l0 = l0 * a0 + rs0; l1 = l1 * a1 + rs1; m0 = nm0; m1 = nm1;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
    uint32_t pa[4] = {MmaT<T>::pack(s[0][0], s[0][1]), MmaT<T>::pack(s[0][2], s[0][3]),
                      MmaT<T>::pack(s[1][0], s[1][1]), MmaT<T>::pack(s[1][2], s[1][3])};
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
      uint32_t vb[4];
      ldsm_x4_t(vb, smem_addr(V + tile_off<HD>((lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4))));
      MmaT<T>::mma(o[2 * dp], pa, vb);
      MmaT<T>::mma(o[2 * dp + 1], pa, vb + 2);
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();
  float* mO = reinterpret_cast<float*>(smem_raw + 16 * HD * 2);   // [4][16][HD], aliases the pipelines
  float* mML = mO + 4 * 16 * HD;                                  // [4][16][2]
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      const int d = i * 8 + (lane & 3) * 2;
      mO[(warp * 16 + r0) * HD + d] = o[i][0]; mO[(warp * 16 + r0) * HD + d + 1] = o[i][1];
      mO[(warp * 16 + r1) * HD + d] = o[i][2]; mO[(warp * 16 + r1) * HD + d + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      mML[(warp * 16 + r0) * 2] = m0; mML[(warp * 16 + r0) * 2 + 1] = l0;
      mML[(warp * 16 + r1) * 2] = m1; mML[(warp * 16 + r1) * 2 + 1] = l1;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < heads_here * HD; i += 128) {
    const int r = i / HD, d = i % HD;
    float m = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, mML[(w * 16 + r) * 2]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mML[(w * 16 + r) * 2];
      const float f = mw == -CUDART_INF_F ? 0.f : exp2f((mw - m) * kLog2e);
      acc += f * mO[(w * 16 + r) * HD + d];
      l += f * mML[(w * 16 + r) * 2 + 1];
    }
    const int head = head0 + r;
    if (p.splits == 1) {
      const float v = l > 0.f ? acc / l * (fp8 ? p.v_scale : 1.f) : 0.f;
      reinterpret_cast<T*>(p.out)[(static_cast<long>(b) * p.nh + head) * HD + d] = MmaT<T>::from_f(v);
    } else if (p.cluster_off > 0) {
      float* cO = reinterpret_cast<float*>(smem_raw + p.cluster_off);
      cO[i] = acc;
      if (d == 0) { cO[16 * HD + r * 2] = m; cO[16 * HD + r * 2 + 1] = l; }
    } else {
      const long base = (static_cast<long>(b) * p.nh + head) * p.splits + split;
      p.ws_o[base * HD + d] = acc;
      if (d == 0) { p.ws_ml[base * 2] = m; p.ws_ml[base * 2 + 1] = l; }
    }
  }
  if (p.splits > 1 && p.cluster_off > 0) {
    // the cluster's CTAs hold one partial each in their shared memory; every CTA finishes its share of
    // the (head, channel) outputs from all of them and nobody leaves before the peers have read
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    float* cO = reinterpret_cast<float*>(smem_raw + p.cluster_off);
    const int E = heads_here * HD;
    const int per = (E + p.splits - 1) / p.splits;
    const int i_end = min(E, (split + 1) * per);
    for (int i = split * per + threadIdx.x; i < i_end; i += 128) {
      const int r = i / HD;
      float ms[8], m = -CUDART_INF_F;
#pragma unroll
      for (int sidx = 0; sidx < 8; ++sidx) {
        if (sidx < p.splits) {
          ms[sidx] = cluster.map_shared_rank(cO, sidx)[16 * HD + r * 2];
          m = fmaxf(m, ms[sidx]);
        }
      }
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int sidx = 0; sidx < 8; ++sidx) {
        if (sidx < p.splits) {
          const float* peer = cluster.map_shared_rank(cO, sidx);
          const float f = ms[sidx] == -CUDART_INF_F ? 0.f : exp2f((ms[sidx] - m) * kLog2e);
          acc += f * peer[i];
          l += f * peer[16 * HD + r * 2 + 1];
        }
      }
      const float v = l > 0.f ? acc / l * (fp8 ? p.v_scale : 1.f) : 0.f;
      reinterpret_cast<T*>(p.out)[(static_cast<long>(b) * p.nh + head0) * HD + i] = MmaT<T>::from_f(v);
    }
    cluster.sync();
  } else if (p.splits > 1 && p.merge_tickets != nullptr) {
    // last split CTA of this (sequence, head group) merges: every CTA publishes its partials, takes
    // a ticket, and the one that draws the last ticket reads all of them back (L2) and finishes
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int* ticket = p.merge_tickets + static_cast<long>(b) * gridDim.y + blockIdx.y;
      const unsigned int prev = atomicAdd(ticket, 1u);
      is_last = prev == static_cast<unsigned int>(p.splits) - 1u;
      if (is_last) *ticket = 0u;
    }
    __syncthreads();
    if (is_last) {
      __threadfence();
      for (int i = threadIdx.x; i < heads_here * HD; i += 128) {
        const int r = i / HD, d = i % HD;
        const long base = (static_cast<long>(b) * p.nh + head0 + r) * p.splits;
        float m = -CUDART_INF_F;
        for (int sidx = 0; sidx < p.splits; ++sidx) m = fmaxf(m, __ldcg(p.ws_ml + (base + sidx) * 2));
        float acc = 0.f, l = 0.f;
        for (int sidx = 0; sidx < p.splits; ++sidx) {
          const float ms = __ldcg(p.ws_ml + (base + sidx) * 2);
          const float f = ms == -CUDART_INF_F ? 0.f : exp2f((ms - m) * kLog2e);
          acc += f * __ldcg(p.ws_o + (base + sidx) * HD + d);
          l += f * __ldcg(p.ws_ml + (base + sidx) * 2 + 1);
        }
        const float v = l > 0.f ? acc / l * (fp8 ? p.v_scale : 1.f) : 0.f;
        reinterpret_cast<T*>(p.out)[(static_cast<long>(b) * p.nh + head0 + r) * HD + d] = MmaT<T>::from_f(v);
      }
    }
  }
}

template <typename T, int HD>
__global__ void decode_merge_kernel(const AttnParams p) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int b = blockIdx.y, head = blockIdx.x;
  const long base = (static_cast<long>(b) * p.nh + head) * p.splits;
  float m = -CUDART_INF_F;
  for (int s = 0; s < p.splits; ++s) m = fmaxf(m, p.ws_ml[(base + s) * 2]);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float ms = p.ws_ml[(base + s) * 2];
      const float f = ms == -CUDART_INF_F ? 0.f : exp2f((ms - m) * kLog2e);
      acc += f * p.ws_o[(base + s) * HD + d];
      l += f * p.ws_ml[(base + s) * 2 + 1];
    }
    const float v = l > 0.f ? acc / l * (p.kv_fp8 == 1 ? p.v_scale : 1.f) : 0.f;
    reinterpret_cast<T*>(p.out)[(static_cast<long>(b) * p.nh + head) * HD + d] = MmaT<T>::from_f(v);
  }
}

// ------------------------------------------------------------------------------ prefill
// grid (q_tiles, nh, B); 128 threads; each warp owns 16 consecutive query tokens of the 64-token
// tile; KV streamed in CH-token chunks shared by the four warps.
template <typename T, int HD, int CH>
__global__ void __launch_bounds__(128) paged_prefill_kernel(const AttnParams p) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ __align__(128) uint8_t smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);   // [64][HD]
  T* sK = sQ + 64 * HD;                     // [2][CH][HD]
  T* sV = sK + 2 * CH * HD;                 // [2][CH][HD]
  const int b = blockIdx.z, head = blockIdx.y;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int qt0 = blockIdx.x * 64;
  if (qt0 >= q_len) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = head / (p.nh / p.nkv);
  const int seq_len = p.seq_lens[b];
  const int pos0 = seq_len - q_len;  // absolute position of query token 0
  const int* bt = p.block_tables + static_cast<long>(b) * p.max_blocks;

  for (int i = threadIdx.x; i < 64 * (HD / 8); i += 128) {
    const int r = i / (HD / 8), c = i % (HD / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (qt0 + r < q_len)
      v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.q) +
                                          static_cast<long>(q_begin + qt0 + r) * p.q_stride +
                                          static_cast<long>(head) * HD + c * 8);
    *reinterpret_cast<uint4*>(sQ + tile_off<HD>(r, c)) = v;
  }
  const int last_pos = pos0 + min(q_len, qt0 + 64) - 1;  // last query position of this tile
  const int first_pos = pos0 + qt0;
  const int lo_tile = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int c_begin = lo_tile / CH;
  const int c_end = last_pos / CH + 1;
  const float scale = p.sm_scale * (p.kv_fp8 == 1 ? p.k_scale : 1.f);
  const int row0 = qt0 + warp * 16 + (lane >> 2);  // query index (within the sequence's new tokens)
  const int posr0 = pos0 + row0, posr1 = posr0 + 8;

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

  load_kv_tile<T, HD, CH, 128>(sK, p.k_cache, bt, p.block_size, p.nkv, kvh, c_begin * CH, 0, seq_len, p.kv_fp8, p.k_scales);
  load_kv_tile<T, HD, CH, 128>(sV, p.v_cache, bt, p.block_size, p.nkv, kvh, c_begin * CH, 0, seq_len, p.kv_fp8, p.v_scales);
  cp_async_commit();
  // the warp's 16 query rows stay in registers for the whole KV sweep
  __syncthreads();   // sQ was staged with plain stores by all threads
  uint32_t qa[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks)
    ldsm_x4(qa[ks], smem_addr(sQ + tile_off<HD>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4))));
  for (int c = c_begin; c < c_end; ++c) {
    const int buf = (c - c_begin) & 1;
    if (c + 1 < c_end) {
      load_kv_tile<T, HD, CH, 128>(sK + (buf ^ 1) * CH * HD, p.k_cache, bt, p.block_size, p.nkv, kvh, (c + 1) * CH, 0, seq_len, p.kv_fp8, p.k_scales);
      load_kv_tile<T, HD, CH, 128>(sV + (buf ^ 1) * CH * HD, p.v_cache, bt, p.block_size, p.nkv, kvh, (c + 1) * CH, 0, seq_len, p.kv_fp8, p.v_scales);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const T* K = sK + buf * CH * HD;
    const T* V = sV + buf * CH * HD;
    float s[CH / 8][4];
#pragma unroll
    for (int j = 0; j < CH / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int jp = 0; jp < CH / 16; ++jp) {
        uint32_t kb[4];
        ldsm_x4(kb, smem_addr(K + tile_off<HD>(jp * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1))));
        MmaT<T>::mma(s[2 * jp], qa[ks], kb);
        MmaT<T>::mma(s[2 * jp + 1], qa[ks], kb + 2);
      }
    }
    float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
    // chunks that lie entirely below every query row of this warp (and inside the window and the
    // sequence) need no per-element mask
    const bool interior = (c + 1) * CH - 1 <= posr0 && (c + 1) * CH <= seq_len &&
                          (p.window <= 0 || c * CH > posr1 - p.window);
    if (interior) {
#pragma unroll
      for (int j = 0; j < CH / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float v = softcap_f(s[j][e] * scale, p.softcap);
          s[j][e] = v;
          if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < CH / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = c * CH + j * 8 + (lane & 3) * 2 + (e & 1);
          const int pr = e < 2 ? posr0 : posr1;
          float v = softcap_f(s[j][e] * scale, p.softcap);
          const bool masked = tok > pr || tok >= seq_len || (p.window > 0 && tok <= pr - p.window);
          if (masked) v = -CUDART_INF_F;
          s[j][e] = v;
          if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
    const float a0 = nm0 == -CUDART_INF_F ? 1.f : exp2f((m0 - nm0) * kLog2e);
    const float a1 = nm1 == -CUDART_INF_F ? 1.f : exp2f((m1 - nm1) * kLog2e);
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int j = 0; j < CH / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float nm = e < 2 ? nm0 : nm1;
        const float pv = nm == -CUDART_INF_F ? 0.f : exp2f((s[j][e] - nm) * kLog2e);
        s[j][e] = pv;
        if (e < 2) rs0 += pv; else rs1 += pv;
      }
    }
    l0 = l0 * a0 + rs0; l1 = l1 * a1 + rs1; m0 = nm0; m1 = nm1;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
#pragma unroll
    for (int kt = 0; kt < CH / 16; ++kt) {
      uint32_t pa[4] = {MmaT<T>::pack(s[2 * kt][0], s[2 * kt][1]), MmaT<T>::pack(s[2 * kt][2], s[2 * kt][3]),
                        MmaT<T>::pack(s[2 * kt + 1][0], s[2 * kt + 1][1]), MmaT<T>::pack(s[2 * kt + 1][2], s[2 * kt + 1][3])};
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t vb[4];
        ldsm_x4_t(vb, smem_addr(V + tile_off<HD>(kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4))));
        MmaT<T>::mma(o[2 * dp], pa, vb);
        MmaT<T>::mma(o[2 * dp + 1], pa, vb + 2);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float vs = p.kv_fp8 == 1 ? p.v_scale : 1.f;
  const float i0 = l0 > 0.f ? vs / l0 : 0.f, i1 = l1 > 0.f ? vs / l1 : 0.f;
  T* out = reinterpret_cast<T*>(p.out);
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    const int d = i * 8 + (lane & 3) * 2;
    if (row0 < q_len) {
      const long off = (static_cast<long>(q_begin + row0) * p.nh + head) * HD + d;
      *reinterpret_cast<uint32_t*>(out + off) = MmaT<T>::pack(o[i][0] * i0, o[i][1] * i0);
    }
    if (row0 + 8 < q_len) {
      const long off = (static_cast<long>(q_begin + row0 + 8) * p.nh + head) * HD + d;
      *reinterpret_cast<uint32_t*>(out + off) = MmaT<T>::pack(o[i][2] * i1, o[i][3] * i1);
    }
  }
}

template <typename T, int HD>
int launch_decode(const AttnParams& p, int B, cudaStream_t s) {
  const int G = p.nh / p.nkv;
  const int groups = (G + 15) / 16;
  if (p.block_size % 16 == 0 && p.kv_fp8 <= 1) {
    constexpr int NST = HD <= 64 ? 4 : HD <= 128 ? 3 : 2;
    const int tile = 16 * HD;
    const int raw = p.kv_fp8 ? tile : tile * 2;
    const int pipe_bytes = 4 * (NST * 2 * raw + (p.kv_fp8 ? 2 * tile * 2 : 0));
    const int merge_bytes = (4 * 16 * HD + 4 * 16 * 2) * 4;
    int smem = 16 * HD * 2 + (pipe_bytes > merge_bytes ? pipe_bytes : merge_bytes);
    AttnParams pc = p;
    pc.cluster_off = 0;
    if (p.cluster_off != 0 && p.splits > 1 && p.splits <= 8) {   // cluster of the split CTAs merges through DSMEM
      pc.cluster_off = (smem + 127) & ~127;
      smem = pc.cluster_off + (16 * HD + 32) * 4;
    }
    auto kern = paged_decode_v2_kernel<T, HD, NST>;
    cudaError_t ce = fi::ensure_dynamic_smem(kern, smem);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    if (pc.cluster_off > 0) {
      ce = fi::launch_kernel_cluster(kern, dim3(p.splits, p.nkv * groups, B), dim3(128), smem, s, dim3(p.splits, 1, 1), pc);
      return static_cast<int>(ce != cudaSuccess ? ce : cudaGetLastError());
    }
    fi::launch_kernel(kern, dim3(p.splits, p.nkv * groups, B), dim3(128), smem, s, 0, pc);
  } else {
    const int kv_bytes = (16 * HD + 4 * 64 * HD) * 2;
    const int merge_bytes = (4 * 16 * HD + 4 * 16 * 2) * 4 + 16 * HD * 2;
    const int smem = kv_bytes > merge_bytes ? kv_bytes : merge_bytes;
    auto kern = paged_decode_kernel<T, HD>;
    cudaError_t ce = fi::ensure_dynamic_smem(kern, smem);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    fi::launch_kernel(kern, dim3(p.splits, p.nkv * groups, B), dim3(128), smem, s, 0, p);
  }
  const bool merged_in_kernel = (p.merge_tickets != nullptr || (p.cluster_off != 0 && p.splits <= 8)) &&
                                p.block_size % 16 == 0 && p.kv_fp8 <= 1;
  if (p.splits > 1 && !merged_in_kernel)
    fi::launch_kernel(decode_merge_kernel<T, HD>, dim3(p.nh, B), dim3(HD >= 128 ? 128 : 64), 0, s, 0, p);
  return static_cast<int>(cudaGetLastError());
}

template <typename T, int HD, int CH>
int launch_prefill(const AttnParams& p, int B, int max_q_len, cudaStream_t s) {
  const int smem = (64 * HD + 4 * CH * HD) * 2;
  auto kern = paged_prefill_kernel<T, HD, CH>;
  cudaError_t ce = fi::ensure_dynamic_smem(kern, smem);
  if (ce != cudaSuccess) return static_cast<int>(ce);
  fi::launch_kernel(kern, dim3((max_q_len + 63) / 64, p.nh, B), dim3(128), smem, s, 0, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// Decode scratch: ws_o needs B*nh*splits*hd floats, ws_ml B*nh*splits*2 floats (splits > 1 only).
extern "C" int fi_paged_decode(const void* q, long q_stride, const void* k_cache,
                               const void* v_cache, void* out, const int* block_tables,
                               const int* seq_lens, float* ws_o, float* ws_ml, int B, int nh,
                               int nkv, int hd, int max_blocks, int block_size, int window,
                               float sm_scale, float softcap, int kv_fp8, float k_scale,
                               float v_scale, int splits, int dtype, void* stream) {
  if (B <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv != 0 || splits < 1) return -10;
  AttnParams p = {};
  p.q = q; p.q_stride = q_stride; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out;
  p.block_tables = block_tables; p.seq_lens = seq_lens; p.cu_q = nullptr; p.ws_o = ws_o;
  p.ws_ml = ws_ml; p.max_blocks = max_blocks; p.block_size = block_size; p.nh = nh; p.nkv = nkv;
  p.window = window; p.sm_scale = sm_scale; p.softcap = softcap; p.k_scale = k_scale;
  p.v_scale = v_scale; p.kv_fp8 = kv_fp8; p.splits = splits;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define FI_DEC(TT, HD) return launch_decode<TT, HD>(p, B, s)
  if (dtype == 0) {
    if (hd == 64) FI_DEC(__nv_bfloat16, 64);
    if (hd == 128) FI_DEC(__nv_bfloat16, 128);
    if (hd == 256) FI_DEC(__nv_bfloat16, 256);
  } else if (dtype == 1) {
    if (hd == 64) FI_DEC(__half, 64);
    if (hd == 128) FI_DEC(__half, 128);
    if (hd == 256) FI_DEC(__half, 256);
  }
#undef FI_DEC
  return -11;
}

// Same as fi_paged_decode with the merge of the split partials done by the last split CTA of every
// (sequence, KV head group) instead of a second launch.  `tickets`: at least B * nkv * ceil(G / 16)
// zero-initialised 32-bit words that stay owned by this op (each call leaves them zero again).
extern "C" int fi_paged_decode_merged(const void* q, long q_stride, const void* k_cache,
                               const void* v_cache, void* out, const int* block_tables,
                               const int* seq_lens, float* ws_o, float* ws_ml, unsigned int* tickets, int B, int nh,
                               int nkv, int hd, int max_blocks, int block_size, int window,
                               float sm_scale, float softcap, int kv_fp8, float k_scale,
                               float v_scale, int splits, int dtype, void* stream) {
  if (B <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv != 0 || splits < 1) return -10;
  AttnParams p = {};
  p.q = q; p.q_stride = q_stride; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out;
  p.block_tables = block_tables; p.seq_lens = seq_lens; p.cu_q = nullptr; p.ws_o = ws_o;
  p.ws_ml = ws_ml; p.max_blocks = max_blocks; p.block_size = block_size; p.nh = nh; p.nkv = nkv;
  p.window = window; p.sm_scale = sm_scale; p.softcap = softcap; p.k_scale = k_scale;
  p.v_scale = v_scale; p.kv_fp8 = kv_fp8; p.splits = splits; p.merge_tickets = tickets;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define FI_DEC(TT, HD) return launch_decode<TT, HD>(p, B, s)
  if (dtype == 0) {
    if (hd == 64) FI_DEC(__nv_bfloat16, 64);
    if (hd == 128) FI_DEC(__nv_bfloat16, 128);
    if (hd == 256) FI_DEC(__nv_bfloat16, 256);
  } else if (dtype == 1) {
    if (hd == 64) FI_DEC(__half, 64);
    if (hd == 128) FI_DEC(__half, 128);
    if (hd == 256) FI_DEC(__half, 256);
  }
#undef FI_DEC
  return -11;
}

// Decode / prefill attention over a ROW-SCALED cache: kv_mode 2 = e4m3 values with one fp32 scale per
// (token, kv head) row ("block-scaled" fp8), kv_mode 3 = packed int4 rows [.., hd / 2] bytes with one
// scale per row.  k_scales / v_scales: fp32 [num_blocks, nkv, block_size].  The tiles are dequantised to
// 16-bit while they are staged, the attention math is that of the 16-bit path.  Decode scratch as in
// fi_paged_decode (ws_o / ws_ml for splits > 1).
extern "C" int fi_paged_decode_rowscaled(const void* q, long q_stride, const void* k_cache, const void* v_cache,
                               const float* k_scales, const float* v_scales, void* out, const int* block_tables,
                               const int* seq_lens, float* ws_o, float* ws_ml, int B, int nh, int nkv, int hd,
                               int max_blocks, int block_size, int window, float sm_scale, float softcap,
                               int kv_mode, int splits, int dtype, void* stream) {
  if (B <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv != 0 || splits < 1 || (kv_mode != 2 && kv_mode != 3) || hd % 32 != 0) return -10;
  if (k_scales == nullptr || v_scales == nullptr || (splits > 1 && (ws_o == nullptr || ws_ml == nullptr))) return -12;
  AttnParams p = {};
  p.q = q; p.q_stride = q_stride; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out;
  p.block_tables = block_tables; p.seq_lens = seq_lens; p.cu_q = nullptr; p.ws_o = ws_o;
  p.ws_ml = ws_ml; p.max_blocks = max_blocks; p.block_size = block_size; p.nh = nh; p.nkv = nkv;
  p.window = window; p.sm_scale = sm_scale; p.softcap = softcap; p.k_scale = 1.f;
  p.v_scale = 1.f; p.kv_fp8 = kv_mode; p.splits = splits; p.k_scales = k_scales; p.v_scales = v_scales;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define FI_DEC(TT, HD) return launch_decode<TT, HD>(p, B, s)
  if (dtype == 0) {
    if (hd == 64) FI_DEC(__nv_bfloat16, 64);
    if (hd == 128) FI_DEC(__nv_bfloat16, 128);
    if (hd == 256) FI_DEC(__nv_bfloat16, 256);
  } else if (dtype == 1) {
    if (hd == 64) FI_DEC(__half, 64);
    if (hd == 128) FI_DEC(__half, 128);
    if (hd == 256) FI_DEC(__half, 256);
  }
#undef FI_DEC
  return -11;
}

extern "C" int fi_paged_prefill_rowscaled(const void* q, long q_stride, const void* k_cache, const void* v_cache,
                                const float* k_scales, const float* v_scales, void* out, const int* block_tables,
                                const int* seq_lens, const int* cu_q, int B, int max_q_len, int nh,
                                int nkv, int hd, int max_blocks, int block_size, int window,
                                float sm_scale, float softcap, int kv_mode, int dtype, void* stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv != 0 || (kv_mode != 2 && kv_mode != 3) || hd % 32 != 0) return -10;
  if (k_scales == nullptr || v_scales == nullptr) return -12;
  AttnParams p = {};
  p.q = q; p.q_stride = q_stride; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out;
  p.block_tables = block_tables; p.seq_lens = seq_lens; p.cu_q = cu_q; p.max_blocks = max_blocks;
  p.block_size = block_size; p.nh = nh; p.nkv = nkv; p.window = window; p.sm_scale = sm_scale;
  p.softcap = softcap; p.k_scale = 1.f; p.v_scale = 1.f; p.kv_fp8 = kv_mode; p.splits = 1;
  p.k_scales = k_scales; p.v_scales = v_scales;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 0) {
    if (hd == 64) return launch_prefill<__nv_bfloat16, 64, 64>(p, B, max_q_len, s);
    if (hd == 128) return launch_prefill<__nv_bfloat16, 128, 64>(p, B, max_q_len, s);
    if (hd == 256) return launch_prefill<__nv_bfloat16, 256, 32>(p, B, max_q_len, s);
  } else if (dtype == 1) {
    if (hd == 64) return launch_prefill<__half, 64, 64>(p, B, max_q_len, s);
    if (hd == 128) return launch_prefill<__half, 128, 64>(p, B, max_q_len, s);
    if (hd == 256) return launch_prefill<__half, 256, 32>(p, B, max_q_len, s);
  }
  return -11;
}

// Same as fi_paged_decode for 2 <= splits <= 8 with the split CTAs of a (sequence, KV head group)
// launched as one thread-block cluster that merges its partials through distributed shared memory:
// one launch, no scratch buffers, no atomics.  Needs block_size % 16 == 0.
extern "C" int fi_paged_decode_cluster(const void* q, long q_stride, const void* k_cache,
                               const void* v_cache, void* out, const int* block_tables,
                               const int* seq_lens, int B, int nh,
                               int nkv, int hd, int max_blocks, int block_size, int window,
                               float sm_scale, float softcap, int kv_fp8, float k_scale,
                               float v_scale, int splits, int dtype, void* stream) {
  if (B <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv != 0 || splits < 1 || splits > 8 || block_size % 16 != 0) return -10;
  AttnParams p = {};
  p.q = q; p.q_stride = q_stride; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out;
  p.block_tables = block_tables; p.seq_lens = seq_lens; p.cu_q = nullptr; p.ws_o = nullptr;
  p.ws_ml = nullptr; p.max_blocks = max_blocks; p.block_size = block_size; p.nh = nh; p.nkv = nkv;
  p.window = window; p.sm_scale = sm_scale; p.softcap = softcap; p.k_scale = k_scale;
  p.v_scale = v_scale; p.kv_fp8 = kv_fp8; p.splits = splits; p.cluster_off = 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define FI_DEC(TT, HD) return launch_decode<TT, HD>(p, B, s)
  if (dtype == 0) {
    if (hd == 64) FI_DEC(__nv_bfloat16, 64);
    if (hd == 128) FI_DEC(__nv_bfloat16, 128);
    if (hd == 256) FI_DEC(__nv_bfloat16, 256);
  } else if (dtype == 1) {
    if (hd == 64) FI_DEC(__half, 64);
    if (hd == 128) FI_DEC(__half, 128);
    if (hd == 256) FI_DEC(__half, 256);
  }
#undef FI_DEC
  return -11;
}

extern "C" int fi_paged_prefill(const void* q, long q_stride, const void* k_cache,
                                const void* v_cache, void* out, const int* block_tables,
                                const int* seq_lens, const int* cu_q, int B, int max_q_len, int nh,
                                int nkv, int hd, int max_blocks, int block_size, int window,
                                float sm_scale, float softcap, int kv_fp8, float k_scale,
                                float v_scale, int dtype, void* stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv != 0) return -10;
  AttnParams p = {};
  p.q = q; p.q_stride = q_stride; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out;
  p.block_tables = block_tables; p.seq_lens = seq_lens; p.cu_q = cu_q; p.max_blocks = max_blocks;
  p.block_size = block_size; p.nh = nh; p.nkv = nkv; p.window = window; p.sm_scale = sm_scale;
  p.softcap = softcap; p.k_scale = k_scale; p.v_scale = v_scale; p.kv_fp8 = kv_fp8; p.splits = 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 0) {
    if (hd == 64) return launch_prefill<__nv_bfloat16, 64, 64>(p, B, max_q_len, s);
    if (hd == 128) return launch_prefill<__nv_bfloat16, 128, 64>(p, B, max_q_len, s);
    if (hd == 256) return launch_prefill<__nv_bfloat16, 256, 32>(p, B, max_q_len, s);
  } else if (dtype == 1) {
    if (hd == 64) return launch_prefill<__half, 64, 64>(p, B, max_q_len, s);
    if (hd == 128) return launch_prefill<__half, 128, 64>(p, B, max_q_len, s);
    if (hd == 256) return launch_prefill<__half, 256, 32>(p, B, max_q_len, s);
  }
  return -11;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of the split-KV decode entry point (declared in paged_attention_noalloc.h).
//
// fi_paged_decode takes its split-KV partial buffers from the caller.  Some callers have no way to
// provide them: a C or C++ host that links this library without a tensor allocator, or a serving
// process that committed its whole device-memory budget to the KV pool at start-up, where a later
// cudaMalloc may fail, fragment the pool's neighbourhood or stall every stream while the driver
// synchronises.  For them the partials live in the fixed device array below, which every GPU that
// loads this library holds until the process exits.
//
// * Capacity: kNoAllocScratchFloats floats (8 MiB).  A call with splits > 1 needs
//   B * nh * splits * (hd + 2) floats; a larger request is refused with -20 and a message on stderr,
//   nothing is launched.  With splits == 1 there are no partials and no limit applies.
// * The first call on each device looks up the array's device address (cudaGetSymbolAddress with
//   that device current) and caches it; make that first call before any stream capture begins.
// * Every call reuses the same array and leaves its partials behind.  Nothing has to start at zero:
//   each launch writes every partial it later reads (a split with no tokens writes m = -inf, l = 0).
//   Two calls that overlap on the GPU (different streams, or another thread) race on the array.
// * No cudaMalloc, cudaFree or other allocating call is made here.
namespace {
constexpr size_t kNoAllocScratchFloats = 2u * 1024u * 1024u;
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];
constexpr int kMaxDevices = 64;
std::atomic<float*> g_noalloc_ptr[kMaxDevices];   // zero-initialised; one slot per device, written once
}  // namespace

extern "C" int fi_paged_decode_noalloc(const void* q, long q_stride, const void* k_cache,
                                       const void* v_cache, void* out, const int* block_tables,
                                       const int* seq_lens, int B, int nh, int nkv, int hd,
                                       int max_blocks, int block_size, int window, float sm_scale,
                                       float softcap, int kv_fp8, float k_scale, float v_scale,
                                       int splits, int dtype, void* stream) {
  if (B <= 0) return 0;
  if (splits < 1 || nh <= 0 || nkv <= 0 || hd <= 0 || nh % nkv != 0) return -10;
  if (splits == 1)   // one split writes straight to `out`: no partials, so no scratch and no size limit
    return fi_paged_decode(q, q_stride, k_cache, v_cache, out, block_tables, seq_lens, nullptr, nullptr, B,
                           nh, nkv, hd, max_blocks, block_size, window, sm_scale, softcap, kv_fp8,
                           k_scale, v_scale, 1, dtype, stream);
  const size_t n_o = static_cast<size_t>(B) * nh * splits * hd;
  const size_t n_ml = static_cast<size_t>(B) * nh * splits * 2;
  if (n_o + n_ml > kNoAllocScratchFloats) {
    fprintf(stderr,
            "fi_paged_decode_noalloc: B*nh*splits*(hd+2) = %zu floats exceeds the built-in scratch "
            "of %zu floats; lower splits or the batch, or use fi_paged_decode with caller buffers\n",
            n_o + n_ml, kNoAllocScratchFloats);
    return -20;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return -21;
  float* ws_o = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (ws_o == nullptr) {
    // In host code the array's name is only a handle; the kernel needs its address on this device.
    // Two threads racing here resolve the same address, so the duplicate store is harmless.
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) return e != cudaSuccess ? static_cast<int>(e) : -22;
    g_noalloc_ptr[dev].store(p, std::memory_order_release);
    ws_o = p;
  }
  float* ws_ml = ws_o + n_o;
  return fi_paged_decode(q, q_stride, k_cache, v_cache, out, block_tables, seq_lens, ws_o, ws_ml, B,
                         nh, nkv, hd, max_blocks, block_size, window, sm_scale, softcap, kv_fp8,
                         k_scale, v_scale, splits, dtype, stream);
}
