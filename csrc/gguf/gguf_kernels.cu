// GGUF block-format kernels for sm_100a (Q8_0, Q2_K, IQ2_XXS, Q4_0, Q4_K, Q6_K): dense dequantisation, a
// weight-streaming GEMV for up to 8 activation rows, and the routed-expert variants (gate|up with
// the clamped SiLU gate, down projection) that read the raw expert payloads in place.
//
// One warp per output row; lanes walk the row's blocks, keep one fp32 accumulator per activation
// row and reduce by shuffle.  Activations are staged once per CTA in shared memory as fp32.
// The bytes are exactly the file's: 34 / 84 / 66-byte blocks, read with 2- or 4-byte loads.
// Reference counterparts (Triton, one program per row): vllm/kernels/triton/deepseek_v4_flash/
// q8_linear.py:10-96, q2_iq2_moe.py:123-1000.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/launch.cuh"
#include "iq2_tables.h"

namespace {

constexpr int kMaxM = 8;

__device__ __forceinline__ float h2f(const uint8_t* p) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(p[0] | (p[1] << 8))));
}

// The tables live in global memory: every CTA copies them into shared memory with one coalesced load per
// thread (constant memory would serialise the 256 different addresses of that copy).
__device__ uint64_t c_grid[256];
__device__ uint8_t c_signs[128];
bool g_tables_ready[64] = {false};

int ensure_tables() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -1;
  if (!g_tables_ready[dev]) {
    cudaError_t e = cudaMemcpyToSymbol(c_grid, kIq2xxsGrid, sizeof(kIq2xxsGrid));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(c_signs, kIq2xsSigns, sizeof(kIq2xsSigns));
    if (e != cudaSuccess) return static_cast<int>(e);
    g_tables_ready[dev] = true;
  }
  return 0;
}

// The IQ2_XXS codebook (256 x 8 magnitudes) and sign table are indexed with a different value by
// every lane: constant memory would serialise those reads, so each CTA copies them into shared
// memory once (2 KB + 128 B) and decodes from there.
struct Iq2Tables {
  const uint64_t* grid;
  const uint8_t* signs;
};
template <bool NEEDED>
__device__ __forceinline__ Iq2Tables load_iq2_tables() {
  Iq2Tables t = {nullptr, nullptr};
  if (NEEDED) {
    __shared__ uint64_t s_grid[256];
    __shared__ uint8_t s_signs[128];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_grid[i] = c_grid[i];
    for (int i = threadIdx.x; i < 128; i += blockDim.x) s_signs[i] = c_signs[i];
    __syncthreads();
    t.grid = s_grid;
    t.signs = s_signs;
  }
  return t;
}

// Decode `n` consecutive values starting at value index v0 (multiple of 8) of one block into out[].
template <int TYPE>
__device__ __forceinline__ void decode8(const uint8_t* blk, int v0, float* out, const Iq2Tables& tab) {
  if (TYPE == 8) {   // Q8_0: 32 values per block
    const float d = h2f(blk);
    const int8_t* q = reinterpret_cast<const int8_t*>(blk + 2 + v0);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = d * static_cast<float>(q[j]);
  } else if (TYPE == 10) {   // Q2_K: value v -> half n = v/128, shift s = (v%128)/32, byte l = v%32
    const int n = v0 >> 7, s = (v0 & 127) >> 5, l = v0 & 31;
    const int sub = n * 8 + s * 2 + (l >> 4);
    const uint8_t sc = blk[sub];
    const float dl = h2f(blk + 80) * static_cast<float>(sc & 0x0F);
    const float ml = h2f(blk + 82) * static_cast<float>(sc >> 4);
    const uint8_t* q = blk + 16 + n * 32 + l;
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = dl * static_cast<float>((q[j] >> (2 * s)) & 3) - ml;
  } else if (TYPE == 2) {   // Q4_0: values 0..15 are the low nibbles of the 16 bytes, 16..31 the high nibbles
    const float d = h2f(blk);
    const uint8_t* q = blk + 2 + (v0 & 15);
    const int sh = (v0 >> 4) * 4;
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = d * static_cast<float>(static_cast<int>((q[j] >> sh) & 0x0F) - 8);
  } else if (TYPE == 12) {   // Q4_K: chunk c = v/64 shares 32 bytes, half h = (v%64)/32 picks the nibble, sub-block 2c+h
    const int c = v0 >> 6, h = (v0 & 63) >> 5, l = v0 & 31, sb = 2 * c + h;
    const uint8_t* s12 = blk + 4;
    int sc, mn;
    if (sb < 4) { sc = s12[sb] & 63; mn = s12[sb + 4] & 63; }
    else { sc = (s12[sb + 4] & 0x0F) | ((s12[sb - 4] >> 6) << 4); mn = (s12[sb + 4] >> 4) | ((s12[sb] >> 6) << 4); }
    const float dl = h2f(blk) * static_cast<float>(sc);
    const float ml = h2f(blk + 2) * static_cast<float>(mn);
    const uint8_t* q = blk + 16 + c * 32 + l;
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = dl * static_cast<float>((q[j] >> (4 * h)) & 0x0F) - ml;
  } else if (TYPE == 14) {   // Q6_K: half n = v/128, quarter qt = (v%128)/32, l = v%32
    const int n = v0 >> 7, qt = (v0 & 127) >> 5, l = v0 & 31;
    const uint8_t* ql = blk + 64 * n + l + ((qt & 1) ? 32 : 0);
    const uint8_t* qh = blk + 128 + 32 * n + l;
    const int8_t sc = reinterpret_cast<const int8_t*>(blk + 192)[8 * n + (l >> 4) + 2 * qt];
    const float dl = h2f(blk + 208) * static_cast<float>(sc);
    const int lsh = (qt >> 1) * 4, hsh = 2 * qt;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int q = static_cast<int>((ql[j] >> lsh) & 0x0F) | (static_cast<int>((qh[j] >> hsh) & 3) << 4);
      out[j] = dl * static_cast<float>(q - 32);
    }
  } else {   // IQ2_XXS: group ib = v/32, row l = (v%32)/8
    const int ib = v0 >> 5, l = (v0 & 31) >> 3;
    const uint8_t* q = blk + 2 + ib * 8;
    const uint32_t word = q[4] | (q[5] << 8) | (q[6] << 16) | (static_cast<uint32_t>(q[7]) << 24);
    const float db = h2f(blk) * (0.5f + static_cast<float>(word >> 28)) * 0.25f;
    const uint64_t g = tab.grid[q[l]];
    const uint8_t sg = tab.signs[(word >> (7 * l)) & 127];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float mag = static_cast<float>((g >> (8 * j)) & 0xFF);
      out[j] = db * ((sg >> j) & 1 ? -mag : mag);
    }
  }
}

template <int TYPE> struct Blk;
template <> struct Blk<8> { static constexpr int kVals = 32, kBytes = 34; };
template <> struct Blk<10> { static constexpr int kVals = 256, kBytes = 84; };
template <> struct Blk<16> { static constexpr int kVals = 256, kBytes = 66; };
template <> struct Blk<2> { static constexpr int kVals = 32, kBytes = 18; };
template <> struct Blk<12> { static constexpr int kVals = 256, kBytes = 144; };
template <> struct Blk<14> { static constexpr int kVals = 256, kBytes = 210; };

template <int TYPE, typename T>
__global__ void dequant_kernel(const uint8_t* __restrict__ raw, long row_stride, int K, T* __restrict__ out) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const Iq2Tables tab = load_iq2_tables<TYPE == 16>();
  const long row = blockIdx.x;
  const uint8_t* r = raw + row * row_stride;
  for (int v0 = threadIdx.x * 8; v0 < K; v0 += blockDim.x * 8) {
    float v[8];
    decode8<TYPE>(r + (v0 / Blk<TYPE>::kVals) * Blk<TYPE>::kBytes, v0 % Blk<TYPE>::kVals, v, tab);
    T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = static_cast<T>(v[j]);
    *reinterpret_cast<uint4*>(out + row * K + v0) = *reinterpret_cast<uint4*>(o);
  }
}

// Dot products of one weight row with M activation rows (fp32 in shared memory, row pitch K).
template <int TYPE>
__device__ __forceinline__ void row_dot(const uint8_t* r, int K, const float* xs, int M, int lane, float* acc,
                                        const Iq2Tables& tab) {
  for (int v0 = lane * 8; v0 < K; v0 += 32 * 8) {
    float w[8];
    decode8<TYPE>(r + (v0 / Blk<TYPE>::kVals) * Blk<TYPE>::kBytes, v0 % Blk<TYPE>::kVals, w, tab);
#pragma unroll
    for (int m = 0; m < kMaxM; ++m) {
      if (m < M) {
        const float4 a = *reinterpret_cast<const float4*>(xs + m * K + v0);
        const float4 b = *reinterpret_cast<const float4*>(xs + m * K + v0 + 4);
        acc[m] += w[0] * a.x + w[1] * a.y + w[2] * a.z + w[3] * a.w + w[4] * b.x + w[5] * b.y + w[6] * b.z + w[7] * b.w;
      }
    }
  }
#pragma unroll
  for (int m = 0; m < kMaxM; ++m)
    for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
}

template <typename T>
__device__ __forceinline__ void stage_x(const T* x, long ldx, int M, int K, float* xs) {
  for (int i = threadIdx.x; i < M * K; i += blockDim.x) xs[i] = static_cast<float>(x[(i / K) * ldx + (i % K)]);
  __syncthreads();
}

template <int TYPE, typename T>
__global__ void gemv_kernel(const T* __restrict__ x, long ldx, const uint8_t* __restrict__ raw, long row_stride,
                            int M, int N, int K, void* __restrict__ out, long ldo, const T* __restrict__ residual,
                            int out_fp32) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ float xs[];
  const Iq2Tables tab = load_iq2_tables<TYPE == 16>();
  stage_x(x, ldx, M, K, xs);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= N) return;
  float acc[kMaxM];
#pragma unroll
  for (int m = 0; m < kMaxM; ++m) acc[m] = 0.f;
  row_dot<TYPE>(raw + static_cast<long>(row) * row_stride, K, xs, M, lane, acc, tab);
  if (lane == 0) {
    for (int m = 0; m < M; ++m) {
      float v = acc[m];
      if (residual) v += static_cast<float>(residual[m * ldo + row]);
      if (out_fp32) reinterpret_cast<float*>(out)[m * ldo + row] = v;
      else reinterpret_cast<T*>(out)[m * ldo + row] = static_cast<T>(v);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Streaming GEMV (M <= 8 activation rows): the whole x is staged once per CTA as 16-bit values, the
// CTAs stride over the weight rows, and every warp pulls its row through shared memory in chunks
// with a three-deep cp.async pipeline (16-byte copies; the ragged 2-byte-aligned head and tail of a
// chunk go through plain loads), so the 34/66/84-byte blocks are fetched with full-width
// transactions and decoded from shared memory.
template <int TYPE> struct Chunk {
  static constexpr int kVals = Blk<TYPE>::kVals == 32 ? 1024 : (Blk<TYPE>::kBytes > 100 ? 2048 : 4096);   // values per chunk
  static constexpr int kBytes = kVals / Blk<TYPE>::kVals * Blk<TYPE>::kBytes;
  static constexpr int kBuf = (kBytes + 16 + 15) / 16 * 16;                   // + room to keep the 16-byte phase
};
constexpr int kGemvWarps = 16;
constexpr int kGemvDepth = 3;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Copy nbytes (2-byte aligned source) into buf so that the copy keeps the source's 16-byte phase;
// returns where the first byte landed.
__device__ __forceinline__ const uint8_t* stage_chunk(const uint8_t* g, int nbytes, uint8_t* buf, int lane) {
  const int mis = static_cast<int>(reinterpret_cast<uintptr_t>(g) & 15);
  uint8_t* d = buf + mis;
  const int head = mis ? min(16 - mis, nbytes) : 0;
  for (int i = lane * 2; i < head; i += 64)
    *reinterpret_cast<uint16_t*>(d + i) = *reinterpret_cast<const uint16_t*>(g + i);
  const int body = (nbytes - head) & ~15;
  for (int i = lane * 16; i < body; i += 512) cp_async16(d + head + i, g + head + i);
  for (int i = head + body + lane * 2; i < nbytes; i += 64)
    *reinterpret_cast<uint16_t*>(d + i) = *reinterpret_cast<const uint16_t*>(g + i);
  return d;
}

template <typename T>
__device__ __forceinline__ void unpack8_16bit(const uint4 raw, float* f) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = static_cast<float>(e[j]);
}

template <int TYPE, typename T>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_stream_kernel(const T* __restrict__ x, long ldx, const uint8_t* __restrict__ raw, long row_stride, int M, int N,
                   int K, void* __restrict__ out, long ldo, const T* __restrict__ residual, int out_fp32) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ __align__(16) uint8_t sm[];
  const Iq2Tables tab = load_iq2_tables<TYPE == 16>();
  T* xs = reinterpret_cast<T*>(sm);                                  // [M][K]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* wbuf = sm + ((static_cast<size_t>(M) * K * sizeof(T) + 15) & ~static_cast<size_t>(15)) +
                  static_cast<size_t>(warp) * kGemvDepth * Chunk<TYPE>::kBuf;
  for (int i = threadIdx.x * 8; i < M * K; i += blockDim.x * 8) {
    const int m = i / K, k = i - m * K;
    *reinterpret_cast<uint4*>(xs + i) = *reinterpret_cast<const uint4*>(x + m * ldx + k);
  }
  __syncthreads();
  const int nch = (K + Chunk<TYPE>::kVals - 1) / Chunk<TYPE>::kVals;
  const int row_step = gridDim.x * kGemvWarps;
  const int row_first = blockIdx.x * kGemvWarps + warp;
  const uint8_t* landed[kGemvDepth];
  // item = (row, chunk); `issue` starts the copy of one item (an empty group past the last row)
  int i_row = row_first, i_ch = 0, i_slot = 0;
  auto issue = [&]() {
    if (i_row < N) {
      const int k0 = i_ch * Chunk<TYPE>::kVals;
      const int nv = min(Chunk<TYPE>::kVals, K - k0);
      const uint8_t* g = raw + static_cast<long>(i_row) * row_stride +
                         static_cast<long>(k0 / Blk<TYPE>::kVals) * Blk<TYPE>::kBytes;
      landed[i_slot] = stage_chunk(g, nv / Blk<TYPE>::kVals * Blk<TYPE>::kBytes, wbuf + i_slot * Chunk<TYPE>::kBuf, lane);
    }
    cp_async_commit();
    i_slot = (i_slot + 1) % kGemvDepth;
    if (++i_ch == nch) { i_ch = 0; i_row += row_step; }
  };
#pragma unroll
  for (int d = 0; d < kGemvDepth - 1; ++d) issue();
  float acc[kMaxM];
#pragma unroll
  for (int m = 0; m < kMaxM; ++m) acc[m] = 0.f;
  int slot = 0;
  for (int row = row_first; row < N; row += row_step) {
    for (int ch = 0; ch < nch; ++ch) {
      issue();
      cp_async_wait<kGemvDepth - 1>();
      __syncwarp();
      const uint8_t* d = landed[slot];
      const int k0 = ch * Chunk<TYPE>::kVals;
      const int nv = min(Chunk<TYPE>::kVals, K - k0);
      for (int v = lane * 8; v < nv; v += 256) {
        float w[8];
        decode8<TYPE>(d + (v / Blk<TYPE>::kVals) * Blk<TYPE>::kBytes, v % Blk<TYPE>::kVals, w, tab);
#pragma unroll
        for (int m = 0; m < kMaxM; ++m) {
          if (m < M) {
            float a[8];
            unpack8_16bit<T>(*reinterpret_cast<const uint4*>(xs + m * K + k0 + v), a);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[m] += w[j] * a[j];
          }
        }
      }
      __syncwarp();
      slot = (slot + 1) % kGemvDepth;
    }
#pragma unroll
    for (int m = 0; m < kMaxM; ++m) {
      float v = acc[m];
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && m < M) {
        if (residual) v += static_cast<float>(residual[m * ldo + row]);
        if (out_fp32) reinterpret_cast<float*>(out)[m * ldo + row] = v;
        else reinterpret_cast<T*>(out)[m * ldo + row] = static_cast<T>(v);
      }
      acc[m] = 0.f;
    }
  }
  cp_async_wait<0>();
}

// Routed experts.  route r = (token r / top_k, expert ids[r]); expert payloads are stacked with a
// byte stride.  Gate|up: a[r, i] = silu(min(g, clamp)) * clamp(u) (clamp <= 0: plain silu * u).
// Every warp carries kMoeRows rows; a row is copied into the warp's shared-memory buffer with
// 16-byte transactions (stage_chunk) and decoded from there.
constexpr int kMoeRows = 4;      // rows per warp
constexpr int kMoeWarps = 8;

template <int TYPE>
__device__ __forceinline__ const uint8_t* stage_row(const uint8_t* g, int K, uint8_t* buf, int lane) {
  const uint8_t* d = stage_chunk(g, K / Blk<TYPE>::kVals * Blk<TYPE>::kBytes, buf, lane);
  cp_async_commit();
  return d;
}
__host__ __device__ constexpr int blk_vals(int type) { return (type == 8 || type == 2) ? 32 : 256; }
__host__ __device__ constexpr int blk_bytes(int type) {
  return type == 8 ? 34 : type == 2 ? 18 : type == 10 ? 84 : type == 12 ? 144 : type == 14 ? 210 : 66;
}
__host__ __device__ constexpr int row_buf_bytes(int type, int K) {
  return ((K / blk_vals(type)) * blk_bytes(type) + 16 + 15) / 16 * 16;
}

template <int TG, int TU, typename T>
__global__ void moe_gate_up_kernel(const T* __restrict__ x, long ldx, const uint8_t* __restrict__ gate,
                                   const uint8_t* __restrict__ up, long expert_stride_g, long expert_stride_u,
                                   long row_stride_g, long row_stride_u, const int* __restrict__ ids, int top_k,
                                   int e_lo, int e_hi, int I, int K, float clamp, T* __restrict__ a) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ __align__(16) float xs[];
  const Iq2Tables tab = load_iq2_tables<TG == 16 || TU == 16>();
  const int r = blockIdx.y;
  const int e = ids[r];
  if (e < e_lo || e >= e_hi) return;   // not this rank's expert
  stage_x(x + static_cast<long>(r / top_k) * ldx, ldx, 1, K, xs);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* bufs = reinterpret_cast<uint8_t*>(xs + K);
  const int bg = row_buf_bytes(TG, K), bu = row_buf_bytes(TU, K);
  uint8_t* gbuf = bufs + static_cast<size_t>(warp) * (bg + bu);
  uint8_t* ubuf = gbuf + bg;
  for (int rr = 0; rr < kMoeRows; ++rr) {
    const int row = (blockIdx.x * kMoeRows + rr) * kMoeWarps + warp;
    if (row >= I) break;
    const uint8_t* gd = stage_row<TG>(gate + (e - e_lo) * expert_stride_g + static_cast<long>(row) * row_stride_g, K, gbuf, lane);
    const uint8_t* ud = stage_row<TU>(up + (e - e_lo) * expert_stride_u + static_cast<long>(row) * row_stride_u, K, ubuf, lane);
    cp_async_wait<0>();
    __syncwarp();
    float g[kMaxM] = {0.f}, u[kMaxM] = {0.f};
    row_dot<TG>(gd, K, xs, 1, lane, g, tab);
    row_dot<TU>(ud, K, xs, 1, lane, u, tab);
    __syncwarp();
    if (lane == 0) {
      float gv = g[0], uv = u[0];
      if (clamp > 0.f) { gv = fminf(gv, clamp); uv = fminf(fmaxf(uv, -clamp), clamp); }
      a[static_cast<long>(r) * I + row] = static_cast<T>(gv / (1.f + __expf(-gv)) * uv);
    }
  }
}

template <int TD, typename T>
__global__ void moe_down_kernel(const T* __restrict__ a, const uint8_t* __restrict__ down, long expert_stride,
                                long row_stride, const int* __restrict__ ids, int e_lo, int e_hi, int H, int I,
                                T* __restrict__ y) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ __align__(16) float xs[];
  const Iq2Tables tab = load_iq2_tables<TD == 16>();
  const int r = blockIdx.y;
  const int e = ids[r];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (e < e_lo || e >= e_hi) {
    for (int rr = 0; rr < kMoeRows; ++rr) {
      const int row = (blockIdx.x * kMoeRows + rr) * kMoeWarps + warp;
      if (row < H && lane == 0) y[static_cast<long>(r) * H + row] = static_cast<T>(0.f);
    }
    return;
  }
  stage_x(a + static_cast<long>(r) * I, I, 1, I, xs);
  uint8_t* buf = reinterpret_cast<uint8_t*>(xs + I) + static_cast<size_t>(warp) * row_buf_bytes(TD, I);
  for (int rr = 0; rr < kMoeRows; ++rr) {
    const int row = (blockIdx.x * kMoeRows + rr) * kMoeWarps + warp;
    if (row >= H) break;
    const uint8_t* d = stage_row<TD>(down + (e - e_lo) * expert_stride + static_cast<long>(row) * row_stride, I, buf, lane);
    cp_async_wait<0>();
    __syncwarp();
    float acc[kMaxM] = {0.f};
    row_dot<TD>(d, I, xs, 1, lane, acc, tab);
    __syncwarp();
    if (lane == 0) y[static_cast<long>(r) * H + row] = static_cast<T>(acc[0]);
  }
}

// ------------------------------------------------------------------------------ grouped routed experts
// The routes are sorted by expert (fi_moe_align) and cut into tiles of at most kGrpM routes of one
// expert.  One CTA column (blockIdx.y) is one tile: the tile's activation rows sit in shared memory as
// 16-bit values, every weight row of the expert is fetched and decoded ONCE per tile and dotted with all
// of the tile's rows, so an expert that serves m routes is streamed ceil(m / kGrpM) times instead of m
// times.  A warp owns kMoeRows weight rows and fetches row r + 1 while it works on row r.
// Inputs and outputs are in sorted-slot order (slot = position in sorted_route).
constexpr int kGrpM = 8;

template <int TYPE, typename T>
__device__ __forceinline__ void row_dot16(const uint8_t* r, int K, const T* xs, int M, int lane, float* acc,
                                          const Iq2Tables& tab) {
  for (int v0 = lane * 8; v0 < K; v0 += 32 * 8) {
    float w[8];
    decode8<TYPE>(r + (v0 / Blk<TYPE>::kVals) * Blk<TYPE>::kBytes, v0 % Blk<TYPE>::kVals, w, tab);
#pragma unroll
    for (int m = 0; m < kGrpM; ++m) {
      if (m < M) {
        float a[8];
        unpack8_16bit<T>(*reinterpret_cast<const uint4*>(xs + static_cast<size_t>(m) * K + v0), a);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[m] += w[j] * a[j];
      }
    }
  }
#pragma unroll
  for (int m = 0; m < kGrpM; ++m)
    for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
}

template <int TG, int TU, typename T>
__global__ void moe_gate_up_grouped_kernel(const T* __restrict__ x, long ldx, const uint8_t* __restrict__ gate,
                                           const uint8_t* __restrict__ up, long expert_stride_g, long expert_stride_u,
                                           long row_stride_g, long row_stride_u, const int* __restrict__ sorted_route,
                                           const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                                           const int* __restrict__ tile_rows, const int* __restrict__ n_tiles, int top_k,
                                           int I, int K, float clamp, T* __restrict__ a_sorted) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ __align__(16) uint8_t gsm[];
  const Iq2Tables tab = load_iq2_tables<TG == 16 || TU == 16>();
  const int t = blockIdx.y;
  if (t >= *n_tiles) return;
  const int e = tile_expert[t], r0 = tile_row0[t], M = tile_rows[t];
  T* xs = reinterpret_cast<T*>(gsm);                                  // [M][K]
  for (int i = threadIdx.x; i < M * (K / 8); i += blockDim.x) {
    const int m = i / (K / 8), c = i % (K / 8);
    const int tok = sorted_route[r0 + m] / top_k;
    reinterpret_cast<uint4*>(xs + static_cast<size_t>(m) * K)[c] =
        reinterpret_cast<const uint4*>(x + static_cast<long>(tok) * ldx)[c];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bg = row_buf_bytes(TG, K), bu = row_buf_bytes(TU, K);
  uint8_t* wb = gsm + ((static_cast<size_t>(kGrpM) * K * sizeof(T) + 15) & ~static_cast<size_t>(15)) +
                static_cast<size_t>(warp) * 2 * (bg + bu);
  const uint8_t* ge = gate + static_cast<long>(e) * expert_stride_g;
  const uint8_t* ue = up + static_cast<long>(e) * expert_stride_u;
  auto row_of = [&](int rr) { return (blockIdx.x * kMoeRows + rr) * kMoeWarps + warp; };
  const uint8_t* gd[2];
  const uint8_t* ud[2];
  auto fetch = [&](int rr) {
    const int row = row_of(rr);
    if (row < I) {
      uint8_t* b = wb + (rr & 1) * (bg + bu);
      gd[rr & 1] = stage_chunk(ge + static_cast<long>(row) * row_stride_g, K / Blk<TG>::kVals * Blk<TG>::kBytes, b, lane);
      ud[rr & 1] = stage_chunk(ue + static_cast<long>(row) * row_stride_u, K / Blk<TU>::kVals * Blk<TU>::kBytes, b + bg, lane);
    }
    cp_async_commit();
  };
  fetch(0);
  for (int rr = 0; rr < kMoeRows; ++rr) {
    const int row = row_of(rr);
    if (row >= I) break;
    if (rr + 1 < kMoeRows) fetch(rr + 1);
    else cp_async_commit();
    cp_async_wait<1>();
    __syncwarp();
    float g[kGrpM], u[kGrpM];
#pragma unroll
    for (int m = 0; m < kGrpM; ++m) g[m] = u[m] = 0.f;
    row_dot16<TG, T>(gd[rr & 1], K, xs, M, lane, g, tab);
    row_dot16<TU, T>(ud[rr & 1], K, xs, M, lane, u, tab);
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < kGrpM; ++m) {
        if (m < M) {
          float gv = g[m], uv = u[m];
          if (clamp > 0.f) { gv = fminf(gv, clamp); uv = fminf(fmaxf(uv, -clamp), clamp); }
          a_sorted[static_cast<long>(r0 + m) * I + row] = static_cast<T>(gv / (1.f + __expf(-gv)) * uv);
        }
      }
    }
  }
  cp_async_wait<0>();
}

template <int TD, typename T>
__global__ void moe_down_grouped_kernel(const T* __restrict__ a_sorted, const uint8_t* __restrict__ down,
                                        long expert_stride, long row_stride, const int* __restrict__ tile_expert,
                                        const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                                        const int* __restrict__ n_tiles, int H, int I, T* __restrict__ y_sorted) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ __align__(16) uint8_t gsm[];
  const Iq2Tables tab = load_iq2_tables<TD == 16>();
  const int t = blockIdx.y;
  if (t >= *n_tiles) return;
  const int e = tile_expert[t], r0 = tile_row0[t], M = tile_rows[t];
  T* xs = reinterpret_cast<T*>(gsm);                                  // [M][I]
  for (int i = threadIdx.x; i < M * (I / 8); i += blockDim.x)
    reinterpret_cast<uint4*>(xs)[i] = reinterpret_cast<const uint4*>(a_sorted + static_cast<long>(r0) * I)[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bd = row_buf_bytes(TD, I);
  uint8_t* wb = gsm + ((static_cast<size_t>(kGrpM) * I * sizeof(T) + 15) & ~static_cast<size_t>(15)) +
                static_cast<size_t>(warp) * 2 * bd;
  const uint8_t* de = down + static_cast<long>(e) * expert_stride;
  auto row_of = [&](int rr) { return (blockIdx.x * kMoeRows + rr) * kMoeWarps + warp; };
  const uint8_t* dd[2];
  auto fetch = [&](int rr) {
    const int row = row_of(rr);
    if (row < H)
      dd[rr & 1] = stage_chunk(de + static_cast<long>(row) * row_stride, I / Blk<TD>::kVals * Blk<TD>::kBytes,
                               wb + (rr & 1) * bd, lane);
    cp_async_commit();
  };
  fetch(0);
  for (int rr = 0; rr < kMoeRows; ++rr) {
    const int row = row_of(rr);
    if (row >= H) break;
    if (rr + 1 < kMoeRows) fetch(rr + 1);
    else cp_async_commit();
    cp_async_wait<1>();
    __syncwarp();
    float acc[kGrpM];
#pragma unroll
    for (int m = 0; m < kGrpM; ++m) acc[m] = 0.f;
    row_dot16<TD, T>(dd[rr & 1], I, xs, M, lane, acc, tab);
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < kGrpM; ++m)
        if (m < M) y_sorted[static_cast<long>(r0 + m) * H + row] = static_cast<T>(acc[m]);
    }
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------ int8 activations
// Q2_K and IQ2_XXS weights are small integers times a block scale, so with the activations quantised to
// int8 (one fp32 scale per 32 values, as llama.cpp's Q8 activation blocks) a group of 32 weights is eight
// dp4a instructions instead of 32 conversions and 32 FMAs: the routed-expert kernels above spend about ten
// instructions per weight on decoding, these about one and a half.
//   IQ2_XXS: codebook magnitudes (8 / 25 / 43) get their signs with (m ^ mask) - mask on packed bytes.
//   Q2_K:    2-bit codes are masked out four at a time; the block minimum uses the integer sum of the
//            16 activations it covers.
__device__ __forceinline__ uint32_t sign_mask4(uint32_t s4) {   // bit j of s4 -> byte j = 0xFF
  return ((s4 * 0x00204081u) & 0x01010101u) * 0xFFu;
}

// One activation row: int8 codes q[K], scales d[K / 32], integer sums of every 16 codes s16[K / 16].
template <typename T>
__device__ __forceinline__ void stage_act_q8(const T* __restrict__ x, int K, int8_t* q, float* d, int* s16) {
  for (int b = threadIdx.x; b < K / 32; b += blockDim.x) {
    float v[32];
#pragma unroll
    for (int c = 0; c < 4; ++c) unpack8_16bit<T>(reinterpret_cast<const uint4*>(x + b * 32)[c], v + c * 8);
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
    const float inv = amax > 0.f ? 127.f / amax : 0.f;
    uint32_t w[8];
    int sum0 = 0, sum1 = 0;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      int c[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) c[k] = __float2int_rn(v[j + k] * inv);
      if (j < 16) sum0 += c[0] + c[1] + c[2] + c[3];
      else sum1 += c[0] + c[1] + c[2] + c[3];
      w[j >> 2] = (c[0] & 0xFF) | ((c[1] & 0xFF) << 8) | ((c[2] & 0xFF) << 16) | (static_cast<uint32_t>(c[3] & 0xFF) << 24);
    }
    reinterpret_cast<uint4*>(q + b * 32)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(q + b * 32)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    d[b] = amax / 127.f;
    s16[2 * b] = sum0;
    s16[2 * b + 1] = sum1;
  }
}

template <int MAXM> struct ActQ8 {
  // shared-memory footprint of MAXM activation rows of K values
  __host__ __device__ static constexpr size_t bytes(int K) {
    return static_cast<size_t>(MAXM) * (K + (K / 32) * 4 + (K / 16) * 4);
  }
};

// Dot products of one weight row (types 10 and 16; the row is 4-byte aligned for type 10, 2-byte for 16)
// with M int8 activation rows.
template <int TYPE, int MAXM>
__device__ __forceinline__ void row_dot_q8(const uint8_t* r, int K, const int8_t* xq, const float* xd, const int* xs16,
                                           int M, int lane, float* acc, const Iq2Tables& tab) {
  static_assert(TYPE == 10 || TYPE == 16, "int8-activation path: Q2_K and IQ2_XXS");
  for (int g = lane; g < K / 32; g += 32) {
    const int v0 = g * 32;
    const uint8_t* blk = r + (v0 >> 8) * Blk<TYPE>::kBytes;
    const int o = v0 & 255;
    uint32_t w[8];
    if (TYPE == 16) {
      const uint16_t* q16 = reinterpret_cast<const uint16_t*>(blk + 2 + (o >> 5) * 8);
      const uint32_t idx = q16[0] | (static_cast<uint32_t>(q16[1]) << 16);
      const uint32_t word = q16[2] | (static_cast<uint32_t>(q16[3]) << 16);
      const float db = h2f(blk) * (0.5f + static_cast<float>(word >> 28)) * 0.25f;
#pragma unroll
      for (int l = 0; l < 4; ++l) {
        const uint64_t g64 = tab.grid[(idx >> (8 * l)) & 255];
        // the sign table entry of a 7-bit index is the index itself plus its parity as bit 7 (an even number of
        // minus signs per group of 8): two ALU instructions instead of a shared-memory lookup
        const uint32_t s7 = (word >> (7 * l)) & 127u;
        const uint32_t sg = s7 | ((__popc(s7) & 1u) << 7);
        const uint32_t m0 = sign_mask4(sg & 15), m1 = sign_mask4(sg >> 4);
        w[2 * l] = __vsub4(static_cast<uint32_t>(g64) ^ m0, m0);
        w[2 * l + 1] = __vsub4(static_cast<uint32_t>(g64 >> 32) ^ m1, m1);
      }
#pragma unroll
      for (int m = 0; m < MAXM; ++m) {
        if (m < M) {
          const int4* xv = reinterpret_cast<const int4*>(xq + static_cast<size_t>(m) * K + v0);   // 32-byte aligned
          const int4 x0 = xv[0], x1 = xv[1];
          const int xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
          int sacc = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) sacc = __dp4a(static_cast<int>(w[i]), xw[i], sacc);
          acc[m] += db * xd[m * (K / 32) + g] * static_cast<float>(sacc);
        }
      }
    } else {
      const int n = o >> 7, sh = ((o & 127) >> 5) * 2, sub = n * 8 + ((o & 127) >> 5) * 2;
      const uint32_t sc0 = blk[sub], sc1 = blk[sub + 1];
      const float d = h2f(blk + 80), dmin = h2f(blk + 82);
      const uint32_t* qw = reinterpret_cast<const uint32_t*>(blk + 16 + n * 32);
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = (qw[i] >> sh) & 0x03030303u;
      const float a0 = d * static_cast<float>(sc0 & 15), a1 = d * static_cast<float>(sc1 & 15);
      const float b0 = dmin * static_cast<float>(sc0 >> 4), b1 = dmin * static_cast<float>(sc1 >> 4);
#pragma unroll
      for (int m = 0; m < MAXM; ++m) {
        if (m < M) {
          const int4* xv = reinterpret_cast<const int4*>(xq + static_cast<size_t>(m) * K + v0);
          const int4 x0 = xv[0], x1 = xv[1];
          const int xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
          int s0 = 0, s1 = 0;
#pragma unroll
          for (int i = 0; i < 4; ++i) s0 = __dp4a(static_cast<int>(w[i]), xw[i], s0);
#pragma unroll
          for (int i = 4; i < 8; ++i) s1 = __dp4a(static_cast<int>(w[i]), xw[i], s1);
          const int* ss = xs16 + m * (K / 16) + 2 * g;
          acc[m] += xd[m * (K / 32) + g] * (a0 * static_cast<float>(s0) + a1 * static_cast<float>(s1) -
                                            b0 * static_cast<float>(ss[0]) - b1 * static_cast<float>(ss[1]));
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MAXM; ++m)
    for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
}

// Grouped gate|up and down with int8 activations (same tiling as the kernels above; MAXM = 1 serves decode
// steps whose routes all hit different experts: fi_moe_align with tiles of one route).
// rows per warp of the int8-activation kernels: twice the float kernels' count halves the CTAs and with them the
// per-CTA set-up (activation quantisation, codebook copy)
constexpr int kQ8Rows = 8;

template <int TG, int TU, int MAXM, typename T>
__global__ void moe_gate_up_q8_kernel(const T* __restrict__ x, long ldx, const uint8_t* __restrict__ gate,
                                      const uint8_t* __restrict__ up, long expert_stride_g, long expert_stride_u,
                                      long row_stride_g, long row_stride_u, const int* __restrict__ sorted_route,
                                      const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                                      const int* __restrict__ tile_rows, const int* __restrict__ n_tiles, int top_k,
                                      int I, int K, float clamp, T* __restrict__ a_sorted) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ __align__(16) uint8_t gsm[];
  const Iq2Tables tab = load_iq2_tables<TG == 16 || TU == 16>();
  const int t = blockIdx.y;
  if (t >= *n_tiles) return;
  const int e = tile_expert[t], r0 = tile_row0[t], M = tile_rows[t];
  int8_t* xq = reinterpret_cast<int8_t*>(gsm);
  float* xd = reinterpret_cast<float*>(gsm + static_cast<size_t>(MAXM) * K);
  int* xs16 = reinterpret_cast<int*>(xd + MAXM * (K / 32));
  for (int m = 0; m < M; ++m) {
    const int tok = sorted_route[r0 + m] / top_k;
    stage_act_q8<T>(x + static_cast<long>(tok) * ldx, K, xq + static_cast<size_t>(m) * K, xd + m * (K / 32),
                    xs16 + m * (K / 16));
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bg = row_buf_bytes(TG, K), bu = row_buf_bytes(TU, K);
  uint8_t* wb = gsm + ((ActQ8<MAXM>::bytes(K) + 15) & ~static_cast<size_t>(15)) + static_cast<size_t>(warp) * 2 * (bg + bu);
  const uint8_t* ge = gate + static_cast<long>(e) * expert_stride_g;
  const uint8_t* ue = up + static_cast<long>(e) * expert_stride_u;
  auto row_of = [&](int rr) { return (blockIdx.x * kQ8Rows + rr) * kMoeWarps + warp; };
  const uint8_t* gd[2];
  const uint8_t* ud[2];
  auto fetch = [&](int rr) {
    const int row = row_of(rr);
    if (row < I) {
      uint8_t* b = wb + (rr & 1) * (bg + bu);
      gd[rr & 1] = stage_chunk(ge + static_cast<long>(row) * row_stride_g, K / Blk<TG>::kVals * Blk<TG>::kBytes, b, lane);
      ud[rr & 1] = stage_chunk(ue + static_cast<long>(row) * row_stride_u, K / Blk<TU>::kVals * Blk<TU>::kBytes, b + bg, lane);
    }
    cp_async_commit();
  };
  fetch(0);
  for (int rr = 0; rr < kQ8Rows; ++rr) {
    const int row = row_of(rr);
    if (row >= I) break;
    if (rr + 1 < kQ8Rows) fetch(rr + 1);
    else cp_async_commit();
    cp_async_wait<1>();
    __syncwarp();
    float g[MAXM], u[MAXM];
#pragma unroll
    for (int m = 0; m < MAXM; ++m) g[m] = u[m] = 0.f;
    row_dot_q8<TG, MAXM>(gd[rr & 1], K, xq, xd, xs16, M, lane, g, tab);
    row_dot_q8<TU, MAXM>(ud[rr & 1], K, xq, xd, xs16, M, lane, u, tab);
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MAXM; ++m) {
        if (m < M) {
          float gv = g[m], uv = u[m];
          if (clamp > 0.f) { gv = fminf(gv, clamp); uv = fminf(fmaxf(uv, -clamp), clamp); }
          a_sorted[static_cast<long>(r0 + m) * I + row] = static_cast<T>(gv / (1.f + __expf(-gv)) * uv);
        }
      }
    }
  }
  cp_async_wait<0>();
}

template <int TD, int MAXM, typename T>
__global__ void moe_down_q8_kernel(const T* __restrict__ a_sorted, const uint8_t* __restrict__ down,
                                   long expert_stride, long row_stride, const int* __restrict__ tile_expert,
                                   const int* __restrict__ tile_row0, const int* __restrict__ tile_rows,
                                   const int* __restrict__ n_tiles, int H, int I, T* __restrict__ y_sorted) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ __align__(16) uint8_t gsm[];
  const Iq2Tables tab = load_iq2_tables<TD == 16>();
  const int t = blockIdx.y;
  if (t >= *n_tiles) return;
  const int e = tile_expert[t], r0 = tile_row0[t], M = tile_rows[t];
  int8_t* xq = reinterpret_cast<int8_t*>(gsm);
  float* xd = reinterpret_cast<float*>(gsm + static_cast<size_t>(MAXM) * I);
  int* xs16 = reinterpret_cast<int*>(xd + MAXM * (I / 32));
  for (int m = 0; m < M; ++m)
    stage_act_q8<T>(a_sorted + static_cast<long>(r0 + m) * I, I, xq + static_cast<size_t>(m) * I, xd + m * (I / 32),
                    xs16 + m * (I / 16));
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bd = row_buf_bytes(TD, I);
  uint8_t* wb = gsm + ((ActQ8<MAXM>::bytes(I) + 15) & ~static_cast<size_t>(15)) + static_cast<size_t>(warp) * 2 * bd;
  const uint8_t* de = down + static_cast<long>(e) * expert_stride;
  auto row_of = [&](int rr) { return (blockIdx.x * kQ8Rows + rr) * kMoeWarps + warp; };
  const uint8_t* dd[2];
  auto fetch = [&](int rr) {
    const int row = row_of(rr);
    if (row < H)
      dd[rr & 1] = stage_chunk(de + static_cast<long>(row) * row_stride, I / Blk<TD>::kVals * Blk<TD>::kBytes,
                               wb + (rr & 1) * bd, lane);
    cp_async_commit();
  };
  fetch(0);
  for (int rr = 0; rr < kQ8Rows; ++rr) {
    const int row = row_of(rr);
    if (row >= H) break;
    if (rr + 1 < kQ8Rows) fetch(rr + 1);
    else cp_async_commit();
    cp_async_wait<1>();
    __syncwarp();
    float acc[MAXM];
#pragma unroll
    for (int m = 0; m < MAXM; ++m) acc[m] = 0.f;
    row_dot_q8<TD, MAXM>(dd[rr & 1], I, xq, xd, xs16, M, lane, acc, tab);
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MAXM; ++m)
        if (m < M) y_sorted[static_cast<long>(r0 + m) * H + row] = static_cast<T>(acc[m]);
    }
  }
  cp_async_wait<0>();
}

}  // namespace

#define FI_STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define FI_TYPE_SWITCH(type, ...)                       \
  switch (type) {                                       \
    case 8: { constexpr int TY = 8; __VA_ARGS__; break; }   \
    case 10: { constexpr int TY = 10; __VA_ARGS__; break; } \
    case 16: { constexpr int TY = 16; __VA_ARGS__; break; } \
    case 2: { constexpr int TY = 2; __VA_ARGS__; break; }   \
    case 12: { constexpr int TY = 12; __VA_ARGS__; break; } \
    case 14: { constexpr int TY = 14; __VA_ARGS__; break; } \
    default: return -11;                                \
  }

extern "C" int fi_gguf_dequant(const void* raw, int type, int rows, int K, long row_stride, void* out, int dtype,
                               void* stream) {
  if (rows <= 0) return 0;
  if (K % 256 != 0 && !((type == 8 || type == 2) && K % 32 == 0)) return -10;
  if (int rc = ensure_tables()) return rc;
  const uint8_t* r = static_cast<const uint8_t*>(raw);
  FI_TYPE_SWITCH(type, {
    if (dtype == 0) fi::launch_kernel(dequant_kernel<TY, __nv_bfloat16>, dim3(rows), dim3(128), 0, FI_STREAM(stream), 0, r, row_stride, K, (__nv_bfloat16*)out);
    else fi::launch_kernel(dequant_kernel<TY, __half>, dim3(rows), dim3(128), 0, FI_STREAM(stream), 0, r, row_stride, K, (__half*)out);
  });
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_gguf_gemv(const void* x, long ldx, const void* raw, long row_stride, int type, int M, int N, int K,
                            void* out, long ldo, const void* residual, int out_fp32, int dtype, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > kMaxM || K % 8 != 0) return -10;
  if (int rc = ensure_tables()) return rc;
  const uint8_t* r = static_cast<const uint8_t*>(raw);
  // streaming kernel: x (16-bit) must fit next to the per-warp chunk buffers, rows 2-byte aligned
  const size_t x_bytes = (static_cast<size_t>(M) * K * 2 + 15) & ~static_cast<size_t>(15);
  if (x_bytes <= 150 * 1024 && (K % 256) == 0 && (ldx % 8) == 0 && (row_stride % 2) == 0 &&
      (reinterpret_cast<uintptr_t>(raw) % 2) == 0 && (reinterpret_cast<uintptr_t>(x) % 16) == 0) {
    const int grid = N < 148 * kGemvWarps * 2 ? (N + kGemvWarps * 2 - 1) / (kGemvWarps * 2) : 148;
    FI_TYPE_SWITCH(type, {
      const size_t smem = x_bytes + static_cast<size_t>(kGemvWarps) * kGemvDepth * Chunk<TY>::kBuf;
      if (dtype == 0) {
        auto k = gemv_stream_kernel<TY, __nv_bfloat16>;
        fi::ensure_dynamic_smem(k, 223 * 1024);   // + static tables <= 227 KB
        fi::launch_kernel(k, dim3(grid), dim3(kGemvWarps * 32), smem, FI_STREAM(stream), 0, (const __nv_bfloat16*)x, ldx,
                          r, row_stride, M, N, K, out, ldo, (const __nv_bfloat16*)residual, out_fp32);
      } else {
        auto k = gemv_stream_kernel<TY, __half>;
        fi::ensure_dynamic_smem(k, 223 * 1024);   // + static tables <= 227 KB
        fi::launch_kernel(k, dim3(grid), dim3(kGemvWarps * 32), smem, FI_STREAM(stream), 0, (const __half*)x, ldx, r,
                          row_stride, M, N, K, out, ldo, (const __half*)residual, out_fp32);
      }
    });
    return static_cast<int>(cudaGetLastError());
  }
  const size_t smem = static_cast<size_t>(M) * K * sizeof(float);
  const int wpb = 8;
  FI_TYPE_SWITCH(type, {
    if (dtype == 0) {
      auto k = gemv_kernel<TY, __nv_bfloat16>;
      fi::ensure_dynamic_smem(k, 200 * 1024);
      fi::launch_kernel(k, dim3((N + wpb - 1) / wpb), dim3(wpb * 32), smem, FI_STREAM(stream), 0,
                        (const __nv_bfloat16*)x, ldx, r, row_stride, M, N, K, out, ldo, (const __nv_bfloat16*)residual, out_fp32);
    } else {
      auto k = gemv_kernel<TY, __half>;
      fi::ensure_dynamic_smem(k, 200 * 1024);
      fi::launch_kernel(k, dim3((N + wpb - 1) / wpb), dim3(wpb * 32), smem, FI_STREAM(stream), 0,
                        (const __half*)x, ldx, r, row_stride, M, N, K, out, ldo, (const __half*)residual, out_fp32);
    }
  });
  return static_cast<int>(cudaGetLastError());
}

// gate/up payloads: [E_local, I rows, row bytes]; type_g/type_u among {8, 10, 16} (bf16 activations)
extern "C" int fi_gguf_moe_gate_up(const void* x, long ldx, const void* gate, const void* up, int type_g, int type_u,
                                   long row_stride_g, long row_stride_u, const int* ids, int n_routes, int top_k,
                                   int e_lo, int e_hi, int I, int K, float clamp, void* a, void* stream) {
  if (n_routes <= 0) return 0;
  if (int rc = ensure_tables()) return rc;
  if (K % 256 != 0) return -10;
  const size_t smem = static_cast<size_t>(K) * sizeof(float) +
                      static_cast<size_t>(kMoeWarps) * (row_buf_bytes(type_g, K) + row_buf_bytes(type_u, K));
  const int wpb = kMoeWarps;
  const int rows_per_cta = kMoeWarps * kMoeRows;
  const dim3 grid((I + rows_per_cta - 1) / rows_per_cta, n_routes);
  const uint8_t* g = static_cast<const uint8_t*>(gate);
  const uint8_t* u = static_cast<const uint8_t*>(up);
  const long sg = row_stride_g * I, su = row_stride_u * I;
#define FI_GU(TG, TU)                                                                                          \
  fi::ensure_dynamic_smem(moe_gate_up_kernel<TG, TU, __nv_bfloat16>, 200 * 1024); \
  fi::launch_kernel(moe_gate_up_kernel<TG, TU, __nv_bfloat16>, grid, dim3(wpb * 32), smem, FI_STREAM(stream), 0, \
                    (const __nv_bfloat16*)x, ldx, g, u, sg, su, row_stride_g, row_stride_u, ids, top_k, e_lo,  \
                    e_hi, I, K, clamp, (__nv_bfloat16*)a)
  if (smem > 200 * 1024) return -12;
  if (type_g == 16 && type_u == 16) { FI_GU(16, 16); }
  else if (type_g == 10 && type_u == 10) { FI_GU(10, 10); }
  else if (type_g == 8 && type_u == 8) { FI_GU(8, 8); }
  else return -11;
#undef FI_GU
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_gguf_moe_down(const void* a, const void* down, int type_d, long row_stride, const int* ids,
                                int n_routes, int e_lo, int e_hi, int H, int I, void* y, void* stream) {
  if (n_routes <= 0) return 0;
  if (int rc = ensure_tables()) return rc;
  if (I % 256 != 0) return -10;
  const size_t smem = static_cast<size_t>(I) * sizeof(float) + static_cast<size_t>(kMoeWarps) * row_buf_bytes(type_d, I);
  const int wpb = kMoeWarps;
  const int rows_per_cta = kMoeWarps * kMoeRows;
  const dim3 grid((H + rows_per_cta - 1) / rows_per_cta, n_routes);
  const uint8_t* d = static_cast<const uint8_t*>(down);
  const long sd = row_stride * H;
  FI_TYPE_SWITCH(type_d, {
    fi::ensure_dynamic_smem(moe_down_kernel<TY, __nv_bfloat16>, 200 * 1024);
    fi::launch_kernel(moe_down_kernel<TY, __nv_bfloat16>, grid, dim3(wpb * 32), smem, FI_STREAM(stream), 0,
                      (const __nv_bfloat16*)a, d, sd, row_stride, ids, e_lo, e_hi, H, I, (__nv_bfloat16*)y);
  });
  return static_cast<int>(cudaGetLastError());
}

// Grouped forms of the routed-expert kernels: routes sorted by expert and cut into tiles of at most
// 8 routes (fi_moe_align with bn = 8); every tile streams its expert once.  a_sorted / y_sorted are
// indexed by sorted slot; x is indexed by token.  bf16 activations.
extern "C" int fi_gguf_moe_gate_up_grouped(const void* x, long ldx, const void* gate, const void* up, int type_g,
                                           int type_u, long row_stride_g, long row_stride_u, const int* sorted_route,
                                           const int* tile_expert, const int* tile_row0, const int* tile_rows,
                                           const int* n_tiles, int max_tiles, int top_k, int I, int K, float clamp,
                                           void* a_sorted, void* stream) {
  if (max_tiles <= 0) return 0;
  if (int rc = ensure_tables()) return rc;
  if (K % 256 != 0) return -10;
  const size_t smem = ((static_cast<size_t>(kGrpM) * K * 2 + 15) & ~static_cast<size_t>(15)) +
                      static_cast<size_t>(kMoeWarps) * 2 * (row_buf_bytes(type_g, K) + row_buf_bytes(type_u, K));
  if (smem > 200 * 1024) return -12;
  const int rows_per_cta = kMoeWarps * kMoeRows;
  const dim3 grid((I + rows_per_cta - 1) / rows_per_cta, max_tiles);
  const uint8_t* g = static_cast<const uint8_t*>(gate);
  const uint8_t* u = static_cast<const uint8_t*>(up);
  const long sg = row_stride_g * I, su = row_stride_u * I;
#define FI_GUG(TG, TU)                                                                                              \
  fi::ensure_dynamic_smem(moe_gate_up_grouped_kernel<TG, TU, __nv_bfloat16>, 200 * 1024);                            \
  fi::launch_kernel(moe_gate_up_grouped_kernel<TG, TU, __nv_bfloat16>, grid, dim3(kMoeWarps * 32), smem,            \
                    FI_STREAM(stream), 0, (const __nv_bfloat16*)x, ldx, g, u, sg, su, row_stride_g, row_stride_u,   \
                    sorted_route, tile_expert, tile_row0, tile_rows, n_tiles, top_k, I, K, clamp,                   \
                    (__nv_bfloat16*)a_sorted)
  if (type_g == 16 && type_u == 16) { FI_GUG(16, 16); }
  else if (type_g == 10 && type_u == 10) { FI_GUG(10, 10); }
  else if (type_g == 8 && type_u == 8) { FI_GUG(8, 8); }
  else return -11;
#undef FI_GUG
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_gguf_moe_down_grouped(const void* a_sorted, const void* down, int type_d, long row_stride,
                                        const int* tile_expert, const int* tile_row0, const int* tile_rows,
                                        const int* n_tiles, int max_tiles, int H, int I, void* y_sorted, void* stream) {
  if (max_tiles <= 0) return 0;
  if (int rc = ensure_tables()) return rc;
  if (I % 256 != 0) return -10;
  const size_t smem = ((static_cast<size_t>(kGrpM) * I * 2 + 15) & ~static_cast<size_t>(15)) +
                      static_cast<size_t>(kMoeWarps) * 2 * row_buf_bytes(type_d, I);
  if (smem > 200 * 1024) return -12;
  const int rows_per_cta = kMoeWarps * kMoeRows;
  const dim3 grid((H + rows_per_cta - 1) / rows_per_cta, max_tiles);
  const uint8_t* d = static_cast<const uint8_t*>(down);
  const long sd = row_stride * H;
  FI_TYPE_SWITCH(type_d, {
    fi::ensure_dynamic_smem(moe_down_grouped_kernel<TY, __nv_bfloat16>, 200 * 1024);
    fi::launch_kernel(moe_down_grouped_kernel<TY, __nv_bfloat16>, grid, dim3(kMoeWarps * 32), smem, FI_STREAM(stream), 0,
                      (const __nv_bfloat16*)a_sorted, d, sd, row_stride, tile_expert, tile_row0, tile_rows, n_tiles, H,
                      I, (__nv_bfloat16*)y_sorted);
  });
  return static_cast<int>(cudaGetLastError());
}

// The same two steps with int8 activations (Q2_K / IQ2_XXS experts only; tile_m = 1 or 8 must match the
// bn given to fi_moe_align).  Returns -11 for other formats: the caller then uses the float kernels.
extern "C" int fi_gguf_moe_gate_up_q8(const void* x, long ldx, const void* gate, const void* up, int type_g,
                                      int type_u, long row_stride_g, long row_stride_u, const int* sorted_route,
                                      const int* tile_expert, const int* tile_row0, const int* tile_rows,
                                      const int* n_tiles, int max_tiles, int tile_m, int top_k, int I, int K,
                                      float clamp, void* a_sorted, void* stream) {
  if (max_tiles <= 0) return 0;
  if (int rc = ensure_tables()) return rc;
  if (K % 256 != 0 || (ldx % 8) != 0 || (tile_m != 1 && tile_m != 8)) return -10;
  if (type_g != type_u || (type_g != 10 && type_g != 16)) return -11;
  if ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up)) & 3) return -11;
  const size_t act = tile_m == 1 ? ActQ8<1>::bytes(K) : ActQ8<8>::bytes(K);
  const size_t smem = ((act + 15) & ~static_cast<size_t>(15)) +
                      static_cast<size_t>(kMoeWarps) * 2 * (row_buf_bytes(type_g, K) + row_buf_bytes(type_u, K));
  if (smem > 200 * 1024) return -12;
  const int rows_per_cta = kMoeWarps * kQ8Rows;
  const dim3 grid((I + rows_per_cta - 1) / rows_per_cta, max_tiles);
  const uint8_t* g = static_cast<const uint8_t*>(gate);
  const uint8_t* u = static_cast<const uint8_t*>(up);
  const long sg = row_stride_g * I, su = row_stride_u * I;
#define FI_GUQ(TY, MM)                                                                                              \
  fi::ensure_dynamic_smem(moe_gate_up_q8_kernel<TY, TY, MM, __nv_bfloat16>, 200 * 1024);                             \
  fi::launch_kernel(moe_gate_up_q8_kernel<TY, TY, MM, __nv_bfloat16>, grid, dim3(kMoeWarps * 32), smem,             \
                    FI_STREAM(stream), 0, (const __nv_bfloat16*)x, ldx, g, u, sg, su, row_stride_g, row_stride_u,   \
                    sorted_route, tile_expert, tile_row0, tile_rows, n_tiles, top_k, I, K, clamp,                   \
                    (__nv_bfloat16*)a_sorted)
  if (type_g == 16 && tile_m == 1) { FI_GUQ(16, 1); }
  else if (type_g == 16) { FI_GUQ(16, 8); }
  else if (tile_m == 1) { FI_GUQ(10, 1); }
  else { FI_GUQ(10, 8); }
#undef FI_GUQ
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_gguf_moe_down_q8(const void* a_sorted, const void* down, int type_d, long row_stride,
                                   const int* tile_expert, const int* tile_row0, const int* tile_rows,
                                   const int* n_tiles, int max_tiles, int tile_m, int H, int I, void* y_sorted,
                                   void* stream) {
  if (max_tiles <= 0) return 0;
  if (int rc = ensure_tables()) return rc;
  if (I % 256 != 0 || (tile_m != 1 && tile_m != 8)) return -10;
  if (type_d != 10 && type_d != 16) return -11;
  if (reinterpret_cast<uintptr_t>(down) & 3) return -11;
  const size_t act = tile_m == 1 ? ActQ8<1>::bytes(I) : ActQ8<8>::bytes(I);
  const size_t smem = ((act + 15) & ~static_cast<size_t>(15)) + static_cast<size_t>(kMoeWarps) * 2 * row_buf_bytes(type_d, I);
  if (smem > 200 * 1024) return -12;
  const int rows_per_cta = kMoeWarps * kQ8Rows;
  const dim3 grid((H + rows_per_cta - 1) / rows_per_cta, max_tiles);
  const uint8_t* d = static_cast<const uint8_t*>(down);
  const long sd = row_stride * H;
#define FI_DQ(TY, MM)                                                                                          \
  fi::ensure_dynamic_smem(moe_down_q8_kernel<TY, MM, __nv_bfloat16>, 200 * 1024);                               \
  fi::launch_kernel(moe_down_q8_kernel<TY, MM, __nv_bfloat16>, grid, dim3(kMoeWarps * 32), smem,               \
                    FI_STREAM(stream), 0, (const __nv_bfloat16*)a_sorted, d, sd, row_stride, tile_expert,     \
                    tile_row0, tile_rows, n_tiles, H, I, (__nv_bfloat16*)y_sorted)
  if (type_d == 16 && tile_m == 1) { FI_DQ(16, 1); }
  else if (type_d == 16) { FI_DQ(16, 8); }
  else if (tile_m == 1) { FI_DQ(10, 1); }
  else { FI_DQ(10, 8); }
#undef FI_DQ
  return static_cast<int>(cudaGetLastError());
}
