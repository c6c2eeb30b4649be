// Multi-head latent attention in absorbed form: every query head attends to ONE shared cache row per
// token, [latent (512) | rotary key (64)] = 576 values, instead of a materialised K and V row per head
// (64 heads x 2 x 256 padded values per token in the materialised form: about 57 times the bytes).
//
//   score(h, t)  = q_cat[h] . row[t]        q_cat[h] = [q_nope[h] W_UK[h] | rope(q_rope[h])]
//   out_lat[h]   = sum_t softmax(score)[t] * row[t][0:512]          (then out[h] = out_lat[h] W_UV[h]^T)
//
// The two per-head projections (W_UK before, W_UV after) are batched matrix products outside this file.
//
// Kernels
//   mla_prepare_kernel  per token: RMSNorm of the latent + rotary of the shared key -> cache row;
//                       [q_lat | rope(q_rope)] -> q_cat
//   mla_decode_kernel   grid (splits, head groups of 16, rows); 4 warps.  A chunk of 64 cache rows is
//                       staged once in shared memory (16-byte cp.async, XOR-swizzled) and serves as K for
//                       the scores (36 k-steps of mma.sync m16n8k16, each warp 16 of the 64 tokens) and,
//                       through ldmatrix.trans, as V for the output (each warp 128 of the 512 latent
//                       channels over all 64 tokens; P goes through shared memory once per chunk).
//   mla_merge_kernel    combines the split partials.
//   mla_ctx_to_pool_kernel  prefill: up-projected context rows -> padded per-head K/V rows of a temporary pool
// A "row" is a (sequence, query token): decode batches have one row per sequence; rows may also carry their
// own visible length and point at their sequence's block table (seq_of_row), the flattening the reference
// uses for its prefill (vllm/engine/lite_engine.py:53-104).  The model itself prefills in the per-head form
// on a temporary pool (many query rows per sequence amortise a K/V tile there).
// The reference keeps per-head K/V for this model family; the absorbed form follows the DeepSeek-V2 paper.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../common/launch.cuh"

namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int KD = 576;    // cache row: latent + rotary key
constexpr int VD = 512;    // latent part, which is also the value
constexpr int ROT = 64;    // rotary part
constexpr int CH = 64;     // cache rows per chunk

template <typename T> struct Mma;
template <> struct Mma<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float* d, const uint32_t* a, const uint32_t* b) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
  static __device__ __forceinline__ uint32_t pack(float x, float y) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16(v); }
};
template <> struct Mma<__half> {
  static __device__ __forceinline__ void mma(float* d, const uint32_t* a, const uint32_t* b) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
  }
  static __device__ __forceinline__ uint32_t pack(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half(v); }
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void ldsm_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;       // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;"); }

// Row-major [rows][W] 16-bit tile whose 16-byte chunks are XOR-swizzled by (row & 7) inside every group of 8.
template <int W>
__device__ __forceinline__ int tile_off(int row, int chunk) { return row * W + ((chunk ^ (row & 7)) << 3); }

struct MlaParams {
  const void* q_cat;          // [rows, nh, 576]
  const void* cache;          // [num_blocks, block_size, 576]
  void* out;                  // out_lat: element (row r, head h, d) at out + (h * out_head_stride + r * out_row_stride + d)
  long out_head_stride, out_row_stride;
  const int* block_tables;    // [num_seqs, max_blocks]
  const int* row_lens;        // [rows] cache rows visible to the row
  const int* seq_of_row;      // [rows] or null (row r belongs to sequence r)
  float* ws_o;                // [rows, nh, splits, 512] partial sums (splits > 1)
  float* ws_ml;               // [rows, nh, splits, 2] partial (max, denominator)
  int nh, max_blocks, block_size, splits;
  float sm_scale;
};

template <typename T>
__global__ void __launch_bounds__(128) mla_decode_kernel(const MlaParams p) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ __align__(16) uint8_t smem[];
  T* sK = reinterpret_cast<T*>(smem);                       // [64][576]
  T* sQ = sK + CH * KD;                                     // [16][576]
  T* sP = sQ + 16 * KD;                                     // [16][64]
  float* sMax = reinterpret_cast<float*>(sP + 16 * CH);     // [4 warps][16 rows]
  const int split = blockIdx.x, group = blockIdx.y, r = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head0 = group * 16;
  const int heads_here = min(16, p.nh - head0);
  const int len = p.row_lens[r];
  const int* bt = p.block_tables + static_cast<long>(p.seq_of_row ? p.seq_of_row[r] : r) * p.max_blocks;
  const int n_chunks = (len + CH - 1) / CH;
  const int per = (n_chunks + p.splits - 1) / p.splits;
  const int c_begin = split * per, c_end = min(n_chunks, c_begin + per);

  for (int i = threadIdx.x; i < 16 * (KD / 8); i += 128) {
    const int row = i / (KD / 8), c = i % (KD / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < heads_here)
      v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.q_cat) +
                                          (static_cast<long>(r) * p.nh + head0 + row) * KD + c * 8);
    *reinterpret_cast<uint4*>(sQ + tile_off<KD>(row, c)) = v;
  }
  float o[16][4];                       // 16 rows x this warp's 128 latent channels
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;   // rows lane/4 and lane/4 + 8; l: this warp's tokens
  const float scale2 = p.sm_scale * kLog2e;
  const T* cache = reinterpret_cast<const T*>(p.cache);

  for (int c = c_begin; c < c_end; ++c) {
    // ---- stage 64 cache rows (rows past the visible length are zero)
    for (int i = threadIdx.x; i < CH * (KD / 8); i += 128) {
      const int row = i / (KD / 8), ch = i % (KD / 8);
      const int tok = c * CH + row;
      const bool valid = tok < len;
      const int blk = valid ? bt[tok / p.block_size] : 0;
      const long src = (static_cast<long>(blk) * p.block_size + (valid ? tok % p.block_size : 0)) * KD + ch * 8;
      cp_async16(sK + tile_off<KD>(row, ch), cache + src, valid);
    }
    cp_async_commit();
    cp_async_wait_all();
    __syncthreads();
    // ---- scores of this warp's 16 tokens
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
    for (int ks = 0; ks < KD / 16; ++ks) {
      uint32_t a[4], kb[4];
      ldsm_x4(a, smem_addr(sQ + tile_off<KD>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4))));
      ldsm_x4(kb, smem_addr(sK + tile_off<KD>(warp * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1))));
      Mma<T>::mma(s[0], a, kb);
      Mma<T>::mma(s[1], a, kb + 2);
    }
    float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = c * CH + warp * 16 + j * 8 + (lane & 3) * 2 + (e & 1);
        float v = s[j][e] * scale2;
        if (tok >= len) v = -CUDART_INF_F;
        s[j][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if ((lane & 3) == 0) {
      sMax[warp * 16 + (lane >> 2)] = mx0;
      sMax[warp * 16 + (lane >> 2) + 8] = mx1;
    }
    __syncthreads();
    // ---- the chunk's row maxima over all four warps, probabilities, P to shared memory
    float nm0 = m0, nm1 = m1;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      nm0 = fmaxf(nm0, sMax[w * 16 + (lane >> 2)]);
      nm1 = fmaxf(nm1, sMax[w * 16 + (lane >> 2) + 8]);
    }
    const float a0 = nm0 == -CUDART_INF_F ? 1.f : exp2f(m0 - nm0);
    const float a1 = nm1 == -CUDART_INF_F ? 1.f : exp2f(m1 - nm1);
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float nm = e < 2 ? nm0 : nm1;
        const float pv = nm == -CUDART_INF_F ? 0.f : exp2f(s[j][e] - nm);
        s[j][e] = pv;
        if (e < 2) rs0 += pv; else rs1 += pv;
      }
      // this thread's two pairs of the 8-token column block (warp * 2 + j): rows lane/4 and lane/4 + 8
      const int chunk = warp * 2 + j;
      *reinterpret_cast<uint32_t*>(sP + tile_off<CH>(lane >> 2, chunk) + (lane & 3) * 2) = Mma<T>::pack(s[j][0], s[j][1]);
      *reinterpret_cast<uint32_t*>(sP + tile_off<CH>((lane >> 2) + 8, chunk) + (lane & 3) * 2) = Mma<T>::pack(s[j][2], s[j][3]);
    }
    l0 = l0 * a0 + rs0; l1 = l1 * a1 + rs1; m0 = nm0; m1 = nm1;
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
    __syncthreads();
    // ---- output: this warp's 128 latent channels over all 64 tokens of the chunk
#pragma unroll
    for (int ks = 0; ks < CH / 16; ++ks) {
      uint32_t pa[4];
      ldsm_x4(pa, smem_addr(sP + tile_off<CH>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4))));
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t vb[4];
        ldsm_x4_t(vb, smem_addr(sK + tile_off<KD>(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8,
                                                    warp * 16 + dp * 2 + (lane >> 4))));
        Mma<T>::mma(o[2 * dp], pa, vb);
        Mma<T>::mma(o[2 * dp + 1], pa, vb + 2);
      }
    }
    __syncthreads();        // the next chunk overwrites sK, sP and sMax
  }
  // ---- denominators: quad sums, then the four warps' shares
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if ((lane & 3) == 0) {
    sMax[warp * 16 + (lane >> 2)] = l0;
    sMax[warp * 16 + (lane >> 2) + 8] = l1;
  }
  __syncthreads();
  float lt0 = 0.f, lt1 = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) { lt0 += sMax[w * 16 + (lane >> 2)]; lt1 += sMax[w * 16 + (lane >> 2) + 8]; }
  const int r0 = lane >> 2, r1 = r0 + 8;
  if (p.splits == 1) {
    const float i0 = lt0 > 0.f ? 1.f / lt0 : 0.f, i1 = lt1 > 0.f ? 1.f / lt1 : 0.f;
    T* out = reinterpret_cast<T*>(p.out);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int d = warp * 128 + i * 8 + (lane & 3) * 2;
      if (r0 < heads_here)
        *reinterpret_cast<uint32_t*>(out + (head0 + r0) * p.out_head_stride + r * p.out_row_stride + d) =
            Mma<T>::pack(o[i][0] * i0, o[i][1] * i0);
      if (r1 < heads_here)
        *reinterpret_cast<uint32_t*>(out + (head0 + r1) * p.out_head_stride + r * p.out_row_stride + d) =
            Mma<T>::pack(o[i][2] * i1, o[i][3] * i1);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int d = warp * 128 + i * 8 + (lane & 3) * 2;
      if (r0 < heads_here) {
        float* w = p.ws_o + ((static_cast<long>(r) * p.nh + head0 + r0) * p.splits + split) * VD + d;
        w[0] = o[i][0]; w[1] = o[i][1];
      }
      if (r1 < heads_here) {
        float* w = p.ws_o + ((static_cast<long>(r) * p.nh + head0 + r1) * p.splits + split) * VD + d;
        w[0] = o[i][2]; w[1] = o[i][3];
      }
    }
    if (warp == 0 && (lane & 3) == 0) {
      if (r0 < heads_here) {
        float* w = p.ws_ml + ((static_cast<long>(r) * p.nh + head0 + r0) * p.splits + split) * 2;
        w[0] = m0; w[1] = lt0;
      }
      if (r1 < heads_here) {
        float* w = p.ws_ml + ((static_cast<long>(r) * p.nh + head0 + r1) * p.splits + split) * 2;
        w[0] = m1; w[1] = lt1;
      }
    }
  }
}

template <typename T>
__global__ void mla_merge_kernel(const MlaParams p) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int h = blockIdx.x, r = blockIdx.y;
  const float* ml = p.ws_ml + (static_cast<long>(r) * p.nh + h) * p.splits * 2;
  float m = -CUDART_INF_F;
  for (int s = 0; s < p.splits; ++s) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  for (int s = 0; s < p.splits; ++s) l += ml[2 * s] == -CUDART_INF_F ? 0.f : ml[2 * s + 1] * exp2f(ml[2 * s] - m);
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* out = reinterpret_cast<T*>(p.out) + h * p.out_head_stride + r * p.out_row_stride;
  const float* wo = p.ws_o + (static_cast<long>(r) * p.nh + h) * p.splits * VD;
  for (int d = threadIdx.x; d < VD; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < p.splits; ++s)
      if (ml[2 * s] != -CUDART_INF_F) acc += wo[s * VD + d] * exp2f(ml[2 * s] - m);
    out[d] = Mma<T>::from_f(acc * inv);
  }
}

// One CTA per token, or several that split the token's heads when there are few tokens.  kva: [T, 576] = [latent | shared rotary key] with row pitch ldkva; q: [T, nh, nope +
// 64] (rotary part last) ; q_lat element (t, h, d) at q_lat + h * ql_head_stride + t * ql_row_stride + d.
// cos_sin: fp32 [max_pos, 64] = [cos(32) | sin(32)], rotation pairs (i, i + 32).
template <typename T>
__global__ void mla_prepare_kernel(const T* __restrict__ kva, long ldkva, const T* __restrict__ norm_w, float eps,
                                   const T* __restrict__ q, int nope, const T* __restrict__ q_lat,
                                   long ql_head_stride, long ql_row_stride, const int* __restrict__ positions,
                                   const float* __restrict__ cos_sin, const int* __restrict__ slot_mapping,
                                   T* __restrict__ cache, T* __restrict__ q_cat, int nh) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int pos = positions[t];
  const float* cs = cos_sin + static_cast<long>(pos) * ROT;
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  const T* row = kva + static_cast<long>(t) * ldkva;
  if (blockIdx.y == 0) {
    // RMSNorm of the latent + rotary of the shared key -> cache row (the first CTA of the token)
    float ss = 0.f;
    for (int i = threadIdx.x; i < VD; i += blockDim.x) { const float f = Mma<T>::to_f(row[i]); ss += f * f; }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < nwarps; ++w) tot += red[w];
    const float inv = rsqrtf(tot / static_cast<float>(VD) + eps);
    if (slot >= 0) {
      T* dst = cache + static_cast<long>(slot) * KD;
      for (int i = threadIdx.x; i < VD; i += blockDim.x)
        dst[i] = Mma<T>::from_f(Mma<T>::to_f(Mma<T>::from_f(Mma<T>::to_f(row[i]) * inv)) * Mma<T>::to_f(norm_w[i]));
      for (int i = threadIdx.x; i < ROT / 2; i += blockDim.x) {
        const float a = Mma<T>::to_f(row[VD + i]), b = Mma<T>::to_f(row[VD + i + ROT / 2]);
        dst[VD + i] = Mma<T>::from_f(a * cs[i] - b * cs[ROT / 2 + i]);
        dst[VD + i + ROT / 2] = Mma<T>::from_f(b * cs[i] + a * cs[ROT / 2 + i]);
      }
    }
  }
  // q_cat rows of this token: one warp per head, the heads spread over gridDim.y CTAs
  for (int h = blockIdx.y * nwarps + warp; h < nh; h += nwarps * gridDim.y) {
    T* dq = q_cat + (static_cast<long>(t) * nh + h) * KD;
    const T* ql = q_lat + h * ql_head_stride + t * ql_row_stride;
    for (int c = lane; c < VD / 8; c += 32)
      reinterpret_cast<uint4*>(dq)[c] = reinterpret_cast<const uint4*>(ql)[c];
    const T* qr = q + (static_cast<long>(t) * nh + h) * (nope + ROT) + nope;
    const float a = Mma<T>::to_f(qr[lane]), b = Mma<T>::to_f(qr[lane + ROT / 2]);
    dq[VD + lane] = Mma<T>::from_f(a * cs[lane] - b * cs[ROT / 2 + lane]);
    dq[VD + lane + ROT / 2] = Mma<T>::from_f(b * cs[lane] + a * cs[ROT / 2 + lane]);
  }
}

// Prefill runs in the per-head form on a temporary paged K/V pool: row i of the batch's context (prefix +
// new tokens, gathered from the latent cache) becomes, for every head, the key [rotary key | no-position
// key | 0] and the value [value | 0], padded to `pad` channels, at slot slots[i] of pools shaped
// [blocks, nh, block_size, pad].  ctx: [Tc, 576] latent rows; kvb: [Tc, nh, nope + vd] up-projected rows.
template <typename T>
__global__ void mla_ctx_to_pool_kernel(const T* __restrict__ ctx, const T* __restrict__ kvb,
                                       const int* __restrict__ slots, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                       int nh, int nope, int vd, int pad, int block_size) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * (blockDim.x >> 5) + warp;
  if (h >= nh) return;
  const int slot = slots[t];
  if (slot < 0) return;
  const long row = (static_cast<long>(slot / block_size) * nh + h) * block_size + slot % block_size;
  uint4* kd = reinterpret_cast<uint4*>(k_pool + row * pad);
  uint4* vdst = reinterpret_cast<uint4*>(v_pool + row * pad);
  const T* kr = ctx + static_cast<long>(t) * KD + VD;
  const T* kh = kvb + (static_cast<long>(t) * nh + h) * (nope + vd);
  for (int c = lane; c < pad / 8; c += 32) {
    const int i = c * 8;
    uint4 kv4 = make_uint4(0, 0, 0, 0), vv4 = make_uint4(0, 0, 0, 0);
    if (i < ROT) kv4 = *reinterpret_cast<const uint4*>(kr + i);
    else if (i < ROT + nope) kv4 = *reinterpret_cast<const uint4*>(kh + i - ROT);
    if (i < vd) vv4 = *reinterpret_cast<const uint4*>(kh + nope + i);
    kd[c] = kv4;
    vdst[c] = vv4;
  }
}

}  // namespace

#define FI_STREAM(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int fi_mla_ctx_to_pool(const void* ctx, const void* kvb, const int* slots, void* k_pool, void* v_pool,
                                  int Tc, int nh, int nope, int vd, int pad, int block_size, int dtype, void* stream) {
  if (Tc <= 0) return 0;
  if ((nope | vd | pad) % 8 != 0 || ROT + nope > pad || vd > pad || block_size <= 0) return -10;
  if ((reinterpret_cast<uintptr_t>(ctx) | reinterpret_cast<uintptr_t>(kvb) | reinterpret_cast<uintptr_t>(k_pool) |
       reinterpret_cast<uintptr_t>(v_pool)) & 15)
    return -10;
  const dim3 grid(Tc, (nh + 7) / 8);
  if (dtype == 0)
    fi::launch_kernel(mla_ctx_to_pool_kernel<__nv_bfloat16>, grid, dim3(256), 0, FI_STREAM(stream), 0,
                      (const __nv_bfloat16*)ctx, (const __nv_bfloat16*)kvb, slots, (__nv_bfloat16*)k_pool,
                      (__nv_bfloat16*)v_pool, nh, nope, vd, pad, block_size);
  else if (dtype == 1)
    fi::launch_kernel(mla_ctx_to_pool_kernel<__half>, grid, dim3(256), 0, FI_STREAM(stream), 0, (const __half*)ctx,
                      (const __half*)kvb, slots, (__half*)k_pool, (__half*)v_pool, nh, nope, vd, pad, block_size);
  else
    return -11;
  return static_cast<int>(cudaGetLastError());
}

// dtype: 0 bf16, 1 fp16.  The rotary width is 64 and the latent width 512 (the cache row is 576 values).
extern "C" int fi_mla_prepare(const void* kva, long ldkva, const void* norm_w, float eps, const void* q, int nope,
                              const void* q_lat, long ql_head_stride, long ql_row_stride, const int* positions,
                              const float* cos_sin, const int* slot_mapping, void* cache, void* q_cat, int T, int nh,
                              int dtype, void* stream) {
  if (T <= 0) return 0;
  if (ldkva % 8 != 0 || ql_head_stride % 8 != 0 || ql_row_stride % 8 != 0 || nope < 0) return -10;
  if ((reinterpret_cast<uintptr_t>(q_lat) | reinterpret_cast<uintptr_t>(q_cat)) & 15) return -10;
  // few tokens (decode): spread a token's heads over several CTAs
  const dim3 grid(T, T >= 128 ? 1 : (nh + 7) / 8);
  if (dtype == 0)
    fi::launch_kernel(mla_prepare_kernel<__nv_bfloat16>, grid, dim3(256), 0, FI_STREAM(stream), 0,
                      (const __nv_bfloat16*)kva, ldkva, (const __nv_bfloat16*)norm_w, eps, (const __nv_bfloat16*)q, nope,
                      (const __nv_bfloat16*)q_lat, ql_head_stride, ql_row_stride, positions, cos_sin, slot_mapping,
                      (__nv_bfloat16*)cache, (__nv_bfloat16*)q_cat, nh);
  else if (dtype == 1)
    fi::launch_kernel(mla_prepare_kernel<__half>, grid, dim3(256), 0, FI_STREAM(stream), 0, (const __half*)kva,
                      ldkva, (const __half*)norm_w, eps, (const __half*)q, nope, (const __half*)q_lat, ql_head_stride,
                      ql_row_stride, positions, cos_sin, slot_mapping, (__half*)cache, (__half*)q_cat, nh);
  else
    return -11;
  return static_cast<int>(cudaGetLastError());
}

// ws_o: rows * nh * splits * 512 floats, ws_ml: rows * nh * splits * 2 floats (splits > 1 only).
extern "C" int fi_mla_decode(const void* q_cat, const void* cache, void* out, long out_head_stride,
                             long out_row_stride, const int* block_tables, const int* row_lens, const int* seq_of_row,
                             float* ws_o, float* ws_ml, int rows, int nh, int max_blocks, int block_size, int splits,
                             float sm_scale, int dtype, void* stream) {
  if (rows <= 0 || nh <= 0) return 0;
  if (splits < 1 || block_size <= 0 || (splits > 1 && (ws_o == nullptr || ws_ml == nullptr))) return -10;
  if ((reinterpret_cast<uintptr_t>(q_cat) | reinterpret_cast<uintptr_t>(cache)) & 15) return -10;
  if (out_head_stride % 2 != 0 || out_row_stride % 2 != 0) return -10;
  MlaParams p = {};
  p.q_cat = q_cat; p.cache = cache; p.out = out; p.out_head_stride = out_head_stride; p.out_row_stride = out_row_stride;
  p.block_tables = block_tables; p.row_lens = row_lens; p.seq_of_row = seq_of_row; p.ws_o = ws_o; p.ws_ml = ws_ml;
  p.nh = nh; p.max_blocks = max_blocks; p.block_size = block_size; p.splits = splits; p.sm_scale = sm_scale;
  const int smem = (CH * KD + 16 * KD + 16 * CH) * 2 + 4 * 16 * 4;
  const dim3 grid(splits, (nh + 15) / 16, rows);
  cudaStream_t s = FI_STREAM(stream);
  if (dtype == 0) {
    cudaError_t ce = fi::ensure_dynamic_smem(mla_decode_kernel<__nv_bfloat16>, smem);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    fi::launch_kernel(mla_decode_kernel<__nv_bfloat16>, grid, dim3(128), smem, s, 0, p);
    if (splits > 1) fi::launch_kernel(mla_merge_kernel<__nv_bfloat16>, dim3(nh, rows), dim3(128), 0, s, 0, p);
  } else if (dtype == 1) {
    cudaError_t ce = fi::ensure_dynamic_smem(mla_decode_kernel<__half>, smem);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    fi::launch_kernel(mla_decode_kernel<__half>, grid, dim3(128), smem, s, 0, p);
    if (splits > 1) fi::launch_kernel(mla_merge_kernel<__half>, dim3(nh, rows), dim3(128), 0, s, 0, p);
  } else {
    return -11;
  }
  return static_cast<int>(cudaGetLastError());
}
