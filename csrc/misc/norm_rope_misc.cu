// Memory-bound helper kernels for sm_100a: RMSNorm family, fused rotary-embedding + KV-cache write
// (optionally with per-head q/k norm and fp8-e4m3 quantisation), embedding gather, gated
// activation, slot mapping and greedy arg-max.  All use 16-byte vector accesses and fp32 math.
//
// Counterparts in the reference (all Triton or eager torch there):
//   vllm/kernels/triton/rms_norm.py:29-125, vllm/model_executor/layers/layernorm.py:12-21,
//   vllm/kernels/triton/reshape_and_cache.py:129-297,
//   vllm/model_executor/layers/rotary_embedding/common.py:139-168 and mrope.py:11-127,
//   vllm/kernels/triton/embedding.py:24-79, vllm/kernels/triton/activation.py:21-137,
//   vllm/kernels/triton/compute_slot_mapping.py:23-73, vllm/engine/sampling/sampler.py:18-40.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../common/launch.cuh"
#include <stdint.h>

namespace {

template <typename T> struct Cvt;
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16(v); }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half(v); }
};
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

// ------------------------------------------------------------------ RMSNorm
// out[r, :] = x[r, :] * rsqrt(mean(x^2) + eps) * (w or 1+w or 1).  Optional residual:
//   residual[r, :] += x[r, :] first (stored back), and the norm runs on the sum.
// One block per row for wide rows; rows narrower than 1024 elements use one warp per row.
template <typename T, bool WARP_ROWS>
__global__ void rmsnorm_kernel(const T* __restrict__ x, T* __restrict__ residual,
                               const T* __restrict__ w, T* __restrict__ out, int rows, int H,
                               long ldx, long ldo, float eps, int w_mode, float out_scale,
                               const T* __restrict__ addend) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ float red[32];
  constexpr int V = 16 / sizeof(T);
  int row, tid, nthr;
  if (WARP_ROWS) {
    row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    tid = threadIdx.x & 31;
    nthr = 32;
    if (row >= rows) return;
  } else {
    row = blockIdx.x;
    tid = threadIdx.x;
    nthr = blockDim.x;
  }
  const T* xr = x + static_cast<long>(row) * ldx;
  T* rr = residual ? residual + static_cast<long>(row) * ldx : nullptr;
  T* orow = out + static_cast<long>(row) * ldo;
  const T* arow = addend ? addend + static_cast<long>(row) * ldo : nullptr;   // out = norm(x) * w + addend
  float ss = 0.f;
  for (int i = tid * V; i < H; i += nthr * V) {
    uint4 raw = *reinterpret_cast<const uint4*>(xr + i);
    T* e = reinterpret_cast<T*>(&raw);
    if (rr) {
      uint4 rraw = *reinterpret_cast<const uint4*>(rr + i);
      T* re = reinterpret_cast<T*>(&rraw);
#pragma unroll
      for (int j = 0; j < V; ++j) re[j] = Cvt<T>::from_f(Cvt<T>::to_f(e[j]) + Cvt<T>::to_f(re[j]));
      *reinterpret_cast<uint4*>(rr + i) = rraw;
#pragma unroll
      for (int j = 0; j < V; ++j) { float f = Cvt<T>::to_f(re[j]); ss += f * f; }
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) { float f = Cvt<T>::to_f(e[j]); ss += f * f; }
    }
  }
  if (WARP_ROWS) ss = warp_sum(ss); else ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / static_cast<float>(H) + eps) * out_scale;
  const T* src = rr ? rr : xr;
  for (int i = tid * V; i < H; i += nthr * V) {
    uint4 raw = *reinterpret_cast<const uint4*>(src + i);
    T* e = reinterpret_cast<T*>(&raw);
    uint4 wraw = make_uint4(0, 0, 0, 0);
    if (w_mode != 2) wraw = *reinterpret_cast<const uint4*>(w + i);
    T* we = reinterpret_cast<T*>(&wraw);
    uint4 oraw;
    T* oe = reinterpret_cast<T*>(&oraw);
    uint4 araw = make_uint4(0, 0, 0, 0);
    if (arow) araw = *reinterpret_cast<const uint4*>(arow + i);
    const T* ae = reinterpret_cast<const T*>(&araw);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      // the normalised value is rounded to the storage type before the weight multiply
      float nv = Cvt<T>::to_f(Cvt<T>::from_f(Cvt<T>::to_f(e[j]) * inv));
      float g = w_mode == 0 ? Cvt<T>::to_f(we[j]) : w_mode == 1 ? 1.f + Cvt<T>::to_f(we[j]) : 1.f;
      float r = nv * g;
      if (arow) r = Cvt<T>::to_f(Cvt<T>::from_f(r)) + Cvt<T>::to_f(ae[j]);
      oe[j] = Cvt<T>::from_f(r);
    }
    *reinterpret_cast<uint4*>(orow + i) = oraw;
  }
}

// ------------------------------------------------------------------ RoPE + KV-cache write
// qkv: [T, (nh + 2*nkv) * hd] (q heads, then k heads, then v heads).  For each token:
//   optional per-head RMSNorm on q and k (weights qw/kw of length hd; w_mode as above; v may get a
//   weightless norm), neox-style rotation of the first rot_dim channels of q and k in place, then
//   k and v rows are written to the paged cache [num_blocks, nkv, block_size, hd] at slot
//   slot_mapping[t] (negative = skip), as 16-bit copies or as fp8 e4m3 of (value / scale).
// cos_sin: fp32 [max_pos, rot_dim] = [cos(rot_dim/2) | sin(rot_dim/2)].
// positions: [n_streams, T]; freq_stream[i] (optional) picks the position stream of frequency i
// (multimodal rotary sections); null = stream 0.
template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const float* __restrict__ cos_sin,
                                  const int* __restrict__ freq_stream,
                                  const int* __restrict__ slot_mapping, void* __restrict__ k_cache,
                                  void* __restrict__ v_cache, const T* __restrict__ qw,
                                  const T* __restrict__ kw, int T_tokens, int nh, int nkv, int hd,
                                  int rot_dim, int block_size, int kv_fp8, float k_scale,
                                  float v_scale, float eps, int qk_norm_mode, int v_norm) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int total_heads = nh + 2 * nkv;
  T* row = qkv + static_cast<long>(t) * total_heads * hd;
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  const int half = rot_dim >> 1;
  // the heads of a token are spread over gridDim.y CTAs (few tokens with many heads would otherwise
  // keep a handful of SMs busy)
  for (int h = blockIdx.y * nwarps + warp; h < total_heads; h += nwarps * gridDim.y) {
    T* x = row + static_cast<long>(h) * hd;
    const bool is_q = h < nh;
    const bool is_k = !is_q && h < nh + nkv;
    const bool is_v = !is_q && !is_k;
    float inv = 1.f;
    const bool do_norm = (qk_norm_mode >= 0 && !is_v) || (is_v && v_norm);
    if (do_norm) {
      float ss = 0.f;
      for (int i = lane; i < hd; i += 32) { float f = Cvt<T>::to_f(x[i]); ss += f * f; }
      ss = warp_sum(ss);
      inv = rsqrtf(ss / static_cast<float>(hd) + eps);
    }
    const T* nw = is_q ? qw : kw;
    auto load = [&](int i) -> float {
      float f = Cvt<T>::to_f(x[i]);
      if (do_norm) {
        f = Cvt<T>::to_f(Cvt<T>::from_f(f * inv));
        if (!is_v && nw != nullptr) {
          float g = Cvt<T>::to_f(nw[i]);
          f *= (qk_norm_mode == 1) ? (1.f + g) : g;
        }
        f = Cvt<T>::to_f(Cvt<T>::from_f(f));
      }
      return f;
    };
    const int kvh = is_k ? h - nh : h - nh - nkv;
    long cache_off = 0;
    if (!is_q && slot >= 0) {
      const int blk = slot / block_size, off = slot % block_size;
      cache_off = ((static_cast<long>(blk) * nkv + kvh) * block_size + off) * hd;
    }
    const float qscale = is_k ? 1.f / k_scale : 1.f / v_scale;
    auto store_cache = [&](int i, float f) {
      if (is_q || slot < 0) return;
      void* base = is_k ? k_cache : v_cache;
      if (kv_fp8) {
        reinterpret_cast<__nv_fp8_e4m3*>(base)[cache_off + i] = __nv_fp8_e4m3(f * qscale);
      } else {
        reinterpret_cast<T*>(base)[cache_off + i] = Cvt<T>::from_f(f);
      }
    };
    if (is_v) {
      for (int i = lane; i < hd; i += 32) {
        float f = load(i);
        if (do_norm) x[i] = Cvt<T>::from_f(f);
        store_cache(i, f);
      }
      continue;
    }
    // rotated part: pairs (i, i + half)
    for (int i = lane; i < half; i += 32) {
      const int stream = freq_stream ? freq_stream[i] : 0;
      const int pos = positions[static_cast<long>(stream) * T_tokens + t];
      const float c = cos_sin[static_cast<long>(pos) * rot_dim + i];
      const float s = cos_sin[static_cast<long>(pos) * rot_dim + half + i];
      const float a = load(i), b = load(i + half);
      const float ra = Cvt<T>::to_f(Cvt<T>::from_f(a * c - b * s));
      const float rb = Cvt<T>::to_f(Cvt<T>::from_f(b * c + a * s));
      x[i] = Cvt<T>::from_f(ra);
      x[i + half] = Cvt<T>::from_f(rb);
      store_cache(i, ra);
      store_cache(i + half, rb);
    }
    for (int i = rot_dim + lane; i < hd; i += 32) {
      float f = load(i);
      if (do_norm) x[i] = Cvt<T>::from_f(f);
      store_cache(i, f);
    }
  }
}

// Fast path of the rotary + cache kernel for the common case (full-width rotary, no q/k/v norms, one
// position stream, 16-bit cache): every thread moves 8 low and 8 high channels of a head with 16-byte
// accesses (the general kernel walks single channels).
template <typename T>
__global__ void rope_cache_vec_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                      const float* __restrict__ cos_sin, const int* __restrict__ slot_mapping,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache, int nh, int nkv, int hd,
                                      int block_size) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int t = blockIdx.x;
  T* row = qkv + static_cast<long>(t) * (nh + 2 * nkv) * hd;
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  const int half = hd >> 1, cph = half >> 3;          // 8-channel chunks per half head
  const float* cs = cos_sin + static_cast<long>(positions[t]) * hd;
  const long blk = slot >= 0 ? slot / block_size : 0, off = slot >= 0 ? slot % block_size : 0;
  const int n_rot = (nh + nkv) * cph;
  for (int item = threadIdx.x; item < n_rot; item += blockDim.x) {
    const int h = item / cph, c = item - h * cph;
    T* x = row + static_cast<long>(h) * hd;
    uint4 lo = *reinterpret_cast<const uint4*>(x + c * 8);
    uint4 hi = *reinterpret_cast<const uint4*>(x + half + c * 8);
    const float4 c0 = *reinterpret_cast<const float4*>(cs + c * 8), c1 = *reinterpret_cast<const float4*>(cs + c * 8 + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(cs + half + c * 8), s1 = *reinterpret_cast<const float4*>(cs + half + c * 8 + 4);
    const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    T* le = reinterpret_cast<T*>(&lo);
    T* he = reinterpret_cast<T*>(&hi);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = Cvt<T>::to_f(le[j]), b = Cvt<T>::to_f(he[j]);
      le[j] = Cvt<T>::from_f(a * cc[j] - b * sn[j]);
      he[j] = Cvt<T>::from_f(b * cc[j] + a * sn[j]);
    }
    *reinterpret_cast<uint4*>(x + c * 8) = lo;
    *reinterpret_cast<uint4*>(x + half + c * 8) = hi;
    if (h >= nh && slot >= 0) {
      T* dst = k_cache + ((blk * nkv + (h - nh)) * block_size + off) * hd;
      *reinterpret_cast<uint4*>(dst + c * 8) = lo;
      *reinterpret_cast<uint4*>(dst + half + c * 8) = hi;
    }
  }
  if (slot >= 0) {
    const int cpv = hd >> 3;
    for (int item = threadIdx.x; item < nkv * cpv; item += blockDim.x) {
      const int h = item / cpv, c = item - h * cpv;
      const uint4 v = *reinterpret_cast<const uint4*>(row + static_cast<long>(nh + nkv + h) * hd + c * 8);
      *reinterpret_cast<uint4*>(v_cache + ((blk * nkv + h) * block_size + off) * hd + c * 8) = v;
    }
  }
}

// Plain cache write (no rotation): k/v rows [T, nkv, hd] with row pitch ld -> paged cache.
template <typename T>
__global__ void reshape_and_cache_kernel(const T* __restrict__ k, const T* __restrict__ v,
                                         const int* __restrict__ slot_mapping,
                                         void* __restrict__ k_cache, void* __restrict__ v_cache,
                                         long ldk, long ldv, int nkv, int hd, int block_size,
                                         int kv_fp8, float k_scale, float v_scale) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int t = blockIdx.x;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const int blk = slot / block_size, off = slot % block_size;
  for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x) {
    const int h = i / hd, d = i % hd;
    const long dst = ((static_cast<long>(blk) * nkv + h) * block_size + off) * hd + d;
    const float kf = Cvt<T>::to_f(k[static_cast<long>(t) * ldk + i]);
    const float vf = Cvt<T>::to_f(v[static_cast<long>(t) * ldv + i]);
    if (kv_fp8) {
      reinterpret_cast<__nv_fp8_e4m3*>(k_cache)[dst] = __nv_fp8_e4m3(kf / k_scale);
      reinterpret_cast<__nv_fp8_e4m3*>(v_cache)[dst] = __nv_fp8_e4m3(vf / v_scale);
    } else {
      reinterpret_cast<T*>(k_cache)[dst] = Cvt<T>::from_f(kf);
      reinterpret_cast<T*>(v_cache)[dst] = Cvt<T>::from_f(vf);
    }
  }
}

// Row-scaled cache write: every (token, kv head) row gets its own fp32 scale.
//   mode 2: e4m3 of value / scale with scale = max|row| / 448           ("block-scaled" fp8 KV)
//   mode 3: packed int4, q = clamp(round(value / scale), -7, 7) with scale = max(max|row| / 7, 1e-4); byte d holds
//           channel d in its low nibble and channel d + hd/2 in its high nibble (two's complement)
// k, v: rows [T, nkv, hd] with pitches ldk / ldv (already rotated / normalised); caches [blocks, nkv, bs, hd or hd/2];
// scales fp32 [blocks, nkv, bs].  One warp per (token, head).  The int4 rule is the reference's
// (vllm/kernels/triton/reshape_and_cache.py:186-262: dynamic row-wise scale, divisor 7).
template <typename T>
__global__ void kv_quant_rows_kernel(const T* __restrict__ k, const T* __restrict__ v, long ldk, long ldv,
                                     const int* __restrict__ slot_mapping, uint8_t* __restrict__ k_cache,
                                     uint8_t* __restrict__ v_cache, float* __restrict__ k_scales,
                                     float* __restrict__ v_scales, int nkv, int hd, int block_size, int mode) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int t = blockIdx.x;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int blk = slot / block_size, off = slot % block_size;
  for (int item = warp; item < 2 * nkv; item += nwarps) {
    const bool is_v = item >= nkv;
    const int h = is_v ? item - nkv : item;
    const T* src = (is_v ? v + static_cast<long>(t) * ldv : k + static_cast<long>(t) * ldk) + static_cast<long>(h) * hd;
    const long rowi = (static_cast<long>(blk) * nkv + h) * block_size + off;
    float amax = 0.f;
    for (int i = lane; i < hd; i += 32) amax = fmaxf(amax, fabsf(Cvt<T>::to_f(src[i])));
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    uint8_t* dst = is_v ? v_cache : k_cache;
    float* sdst = is_v ? v_scales : k_scales;
    if (mode == 3) {
      const float sc = fmaxf(amax / 7.f, 1e-4f);
      const int half = hd >> 1;
      for (int i = lane; i < half; i += 32) {
        const int lo = static_cast<int>(fminf(fmaxf(floorf(Cvt<T>::to_f(src[i]) / sc + 0.5f), -7.f), 7.f));
        const int hi = static_cast<int>(fminf(fmaxf(floorf(Cvt<T>::to_f(src[i + half]) / sc + 0.5f), -7.f), 7.f));
        dst[rowi * half + i] = static_cast<uint8_t>((lo & 0x0F) | ((hi & 0x0F) << 4));
      }
      if (lane == 0) sdst[rowi] = sc;
    } else {
      const float sc = fmaxf(amax / 448.f, 1e-12f);
      const float inv = 1.f / sc;
      for (int i = lane; i < hd; i += 32)
        reinterpret_cast<__nv_fp8_e4m3*>(dst)[rowi * hd + i] = __nv_fp8_e4m3(Cvt<T>::to_f(src[i]) * inv);
      if (lane == 0) sdst[rowi] = sc;
    }
  }
}

// ------------------------------------------------------------------ embedding gather
template <typename T>
__global__ void embedding_kernel(const long* __restrict__ ids, const T* __restrict__ table,
                                 T* __restrict__ out, int H, float scale, int vocab_start,
                                 int vocab_end) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  constexpr int V = 16 / sizeof(T);
  const long id = ids[blockIdx.x];
  T* o = out + static_cast<long>(blockIdx.x) * H;
  const bool mine = id >= vocab_start && id < vocab_end;
  const T* src = table + (mine ? (id - vocab_start) : 0) * static_cast<long>(H);
  for (int i = threadIdx.x * V; i < H; i += blockDim.x * V) {
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (mine) {
      raw = *reinterpret_cast<const uint4*>(src + i);
      if (scale != 1.f) {
        T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
        for (int j = 0; j < V; ++j) e[j] = Cvt<T>::from_f(Cvt<T>::to_f(e[j]) * scale);
      }
    }
    *reinterpret_cast<uint4*>(o + i) = raw;
  }
}

// ------------------------------------------------------------------ act(gate) * up on [rows, 2d]
template <typename T>
__global__ void act_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int d, long ldx,
                               int act) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const long r = blockIdx.x;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float g = Cvt<T>::to_f(x[r * ldx + i]);
    const float u = Cvt<T>::to_f(x[r * ldx + d + i]);
    float a;
    if (act == 1) a = g / (1.f + __expf(-g));
    else if (act == 2) {
      const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
      a = g / (1.f + __expf(-2.f * inner));
    } else a = g;
    out[r * d + i] = Cvt<T>::from_f(a * u);
  }
}

// plain elementwise activation (act: 1 SiLU, 2 tanh-GELU) over a [rows, d] tensor
template <typename T>
__global__ void act_kernel(const T* __restrict__ x, T* __restrict__ out, int d, long ldx, long ldo, int act) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const long r = blockIdx.x;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float g = Cvt<T>::to_f(x[r * ldx + i]);
    float a;
    if (act == 1) a = g / (1.f + __expf(-g));
    else if (act == 2) {
      const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
      a = g / (1.f + __expf(-2.f * inner));
    } else a = g;
    out[r * ldo + i] = Cvt<T>::from_f(a);
  }
}

// ------------------------------------------------------------------ slot mapping
// slot[t] = block_tables[seq, pos / bs] * bs + pos % bs  (block id 0 is the null block -> -1).
__global__ void slot_mapping_kernel(const int* __restrict__ positions,
                                    const int* __restrict__ token_seq,
                                    const int* __restrict__ block_tables, int max_blocks, int bs,
                                    int* __restrict__ slots, int T) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int pos = positions[t];
  const int seq = token_seq[t];
  if (seq < 0 || pos < 0) { slots[t] = -1; return; }
  const int blk = block_tables[static_cast<long>(seq) * max_blocks + pos / bs];
  slots[t] = blk <= 0 ? -1 : blk * bs + pos % bs;
}

// ------------------------------------------------------------------ row gather of an int32 table
// out[r, :] = table[idx[r], :]: the block-table rows of the sequences of a decode batch (one launch
// inside the captured step instead of a library index_select plus an index-widening copy).
__global__ void gather_rows_i32_kernel(const int* __restrict__ table, const int* __restrict__ idx,
                                       int* __restrict__ out, int cols, int n_table_rows) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int r = blockIdx.x;
  int src = idx[r];
  src = src < 0 ? 0 : (src >= n_table_rows ? n_table_rows - 1 : src);
  const int* from = table + static_cast<long>(src) * cols;
  int* to = out + static_cast<long>(r) * cols;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) to[c] = from[c];
}

// ------------------------------------------------------------------ selective KV blocks
// Sparse decode attention over a subset of a sequence's KV blocks: block i of n is kept when
// i % stride == 0, or i < min_blocks, or i == n - 1.  The kept block ids are written densely into
// out_table[r, :] and out_len[r] is the token count of the compacted sequence (every kept block full except
// the last one of the sequence, which stays last), so the ordinary paged decode kernel runs unchanged on
// the compact table.  One warp per sequence.
__global__ void select_blocks_kernel(const int* __restrict__ table, const int* __restrict__ seq_lens,
                                     int* __restrict__ out_table, int* __restrict__ out_len, int cols,
                                     int block_size, int stride, int min_blocks) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int r = blockIdx.x, lane = threadIdx.x;
  const int len = seq_lens[r];
  const int n = len > 0 ? min((len + block_size - 1) / block_size, cols) : 0;
  const int* from = table + static_cast<long>(r) * cols;
  int* to = out_table + static_cast<long>(r) * cols;
  int kept = 0;
  for (int base = 0; base < n; base += 32) {
    const int i = base + lane;
    const bool keep = i < n && (i % stride == 0 || i < min_blocks || i == n - 1);
    const unsigned m = __ballot_sync(0xffffffffu, keep);
    if (keep) to[kept + __popc(m & ((1u << lane) - 1u))] = from[i];
    kept += __popc(m);
  }
  for (int c = kept + lane; c < cols; c += 32) to[c] = 0;      // the null block
  if (lane == 0) out_len[r] = n > 0 ? (kept - 1) * block_size + (len - (n - 1) * block_size) : 0;
}

// ------------------------------------------------------------------ greedy arg-max
// One block per row; ties resolve to the lowest index (matches torch.argmax on CPU).
template <typename T>
__global__ void argmax_kernel(const T* __restrict__ logits, long ld, int V, long* __restrict__ out,
                              float softcap) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const T* row = logits + static_cast<long>(blockIdx.x) * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  if (sizeof(T) == 4 && (V & 3) == 0 && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    // fp32 logits: 16-byte loads, four independent loads in flight per thread
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int n4 = V >> 2;
    for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        v[u] = i < n4 ? row4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int base = (i0 + u * blockDim.x) * 4;
        const float f[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (f[j] > best || (f[j] == best && base + j < bi)) { best = f[j]; bi = base + j; }
      }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float f = Cvt<T>::to_f(row[i]);
      if (f > best || (f == best && i < bi)) { best = f; bi = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    best = l < nw ? sv[l] : -INFINITY;
    bi = l < nw ? si[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (l == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
  (void)softcap;
}

template <typename F>
int dispatch_dtype(int dtype, F&& f) {
  if (dtype == 0) return f(static_cast<__nv_bfloat16*>(nullptr));
  if (dtype == 1) return f(static_cast<__half*>(nullptr));
  return -1;
}

}  // namespace

#define FI_STREAM(s) reinterpret_cast<cudaStream_t>(s)

// w_mode: 0 = x*w, 1 = x*(1+w), 2 = no weight.  residual may be null.  dtype 0 bf16 / 1 fp16.
extern "C" int fi_rmsnorm(const void* x, void* residual, const void* w, void* out, int rows, int H,
                          long ldx, long ldo, float eps, int w_mode, float out_scale, int dtype,
                          void* stream, const void* addend) {
  if (rows <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0) return -10;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = std::remove_pointer_t<decltype(tag)>;
    if (H <= 1024) {
      const int wpb = 4;
      fi::launch_kernel(rmsnorm_kernel<T, true>, dim3((rows + wpb - 1) / wpb), dim3(wpb * 32), 0, FI_STREAM(stream), 0, 
          (const T*)x, (T*)residual, (const T*)w, (T*)out, rows, H, ldx, ldo, eps, w_mode,
          out_scale, (const T*)addend);
    } else {
      // few rows (decode): one 16-byte chunk per thread for the shortest latency; many rows (prefill):
      // four chunks per thread, so a quarter of the threads keeps four times the bytes in flight per
      // thread and more rows are resident per SM
      int threads = rows >= 512 ? H / 32 : H / 8;
      threads = threads > 1024 ? 1024 : (threads < 64 ? 64 : ((threads + 31) / 32) * 32);
      fi::launch_kernel(rmsnorm_kernel<T, false>, dim3(rows), dim3(threads), 0, FI_STREAM(stream), 0, 
          (const T*)x, (T*)residual, (const T*)w, (T*)out, rows, H, ldx, ldo, eps, w_mode,
          out_scale, (const T*)addend);
    }
    return static_cast<int>(cudaGetLastError());
  });
}

// Multi-head latent attention, materialised form: builds the [q | k | v] row of a token with padded heads
// in one pass.  q head = [rope part | no-position part | 0], k head = [shared rope key | no-position key | 0],
// v head = [value | 0]; q is [T, nh, nope + rope] (no-position part first), k_rope [T, rope] with row pitch
// ldk, kvb [T, nh, nope + vd].  All section widths are multiples of 8 (16-byte moves).
template <typename T>
__global__ void mla_assemble_kernel(const T* __restrict__ q, const T* __restrict__ k_rope, long ldk,
                                    const T* __restrict__ kvb, T* __restrict__ buf, int nh, int nope, int rope,
                                    int vd, int pad) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * (blockDim.x >> 5) + warp;
  if (head >= 3 * nh) return;
  const int kind = head / nh, h = head % nh;
  uint4* dst = reinterpret_cast<uint4*>(buf + (static_cast<long>(t) * 3 * nh + head) * pad);
  const T* qh = q + (static_cast<long>(t) * nh + h) * (nope + rope);
  const T* kh = kvb + (static_cast<long>(t) * nh + h) * (nope + vd);
  for (int c = lane; c < pad / 8; c += 32) {
    const int i = c * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (kind == 0) {
      if (i < rope) v = *reinterpret_cast<const uint4*>(qh + nope + i);
      else if (i < rope + nope) v = *reinterpret_cast<const uint4*>(qh + i - rope);
    } else if (kind == 1) {
      if (i < rope) v = *reinterpret_cast<const uint4*>(k_rope + static_cast<long>(t) * ldk + i);
      else if (i < rope + nope) v = *reinterpret_cast<const uint4*>(kh + i - rope);
    } else {
      if (i < vd) v = *reinterpret_cast<const uint4*>(kh + nope + i);
    }
    dst[c] = v;
  }
}

extern "C" int fi_mla_assemble(const void* q, const void* k_rope, long ldk, const void* kvb, void* buf, int T, int nh,
                               int nope, int rope, int vd, int pad, int dtype, void* stream) {
  if (T <= 0) return 0;
  if ((nope | rope | vd | pad) % 8 != 0 || ldk % 8 != 0 || rope + nope > pad || vd > pad) return -10;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_rope) | reinterpret_cast<uintptr_t>(kvb) |
       reinterpret_cast<uintptr_t>(buf)) & 15)
    return -10;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using Tt = std::remove_pointer_t<decltype(tag)>;
    fi::launch_kernel(mla_assemble_kernel<Tt>, dim3(T, (3 * nh + 7) / 8), dim3(256), 0, FI_STREAM(stream), 0,
                      (const Tt*)q, (const Tt*)k_rope, ldk, (const Tt*)kvb, (Tt*)buf, nh, nope, rope, vd, pad);
    return static_cast<int>(cudaGetLastError());
  });
}

extern "C" int fi_rope_cache(void* qkv, const int* positions, const float* cos_sin,
                             const int* freq_stream, const int* slot_mapping, void* k_cache,
                             void* v_cache, const void* qw, const void* kw, int T, int nh, int nkv,
                             int hd, int rot_dim, int block_size, int kv_fp8, float k_scale,
                             float v_scale, float eps, int qk_norm_mode, int v_norm, int dtype,
                             void* stream) {
  if (T <= 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using Tt = std::remove_pointer_t<decltype(tag)>;
    if (qk_norm_mode < 0 && !v_norm && rot_dim == hd && freq_stream == nullptr && !kv_fp8 && hd % 16 == 0 &&
        (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 && (reinterpret_cast<uintptr_t>(cos_sin) & 15) == 0) {
      const int items = (nh + nkv) * (hd / 16);
      const int threads = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
      fi::launch_kernel(rope_cache_vec_kernel<Tt>, dim3(T), dim3(threads), 0, FI_STREAM(stream), 0, (Tt*)qkv, positions,
                        cos_sin, slot_mapping, (Tt*)k_cache, (Tt*)v_cache, nh, nkv, hd, block_size);
      return static_cast<int>(cudaGetLastError());
    }
    int warps = nh + 2 * nkv;
    if (warps > 16) warps = 16;
    // head groups per token: enough CTAs for about two waves when the token count alone does not give them
    int groups = (nh + 2 * nkv + warps - 1) / warps;
    const int want = (2 * 148 + T - 1) / T;
    if (groups > want) groups = want;
    if (groups < 1) groups = 1;
    fi::launch_kernel(rope_cache_kernel<Tt>, dim3(T, groups), dim3(warps * 32), 0, FI_STREAM(stream), 0, 
        (Tt*)qkv, positions, cos_sin, freq_stream, slot_mapping, k_cache, v_cache, (const Tt*)qw,
        (const Tt*)kw, T, nh, nkv, hd, rot_dim, block_size, kv_fp8, k_scale, v_scale, eps,
        qk_norm_mode, v_norm);
    return static_cast<int>(cudaGetLastError());
  });
}

extern "C" int fi_reshape_and_cache(const void* k, const void* v, const int* slot_mapping,
                                    void* k_cache, void* v_cache, int T, long ldk, long ldv,
                                    int nkv, int hd, int block_size, int kv_fp8, float k_scale,
                                    float v_scale, int dtype, void* stream) {
  if (T <= 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using Tt = std::remove_pointer_t<decltype(tag)>;
    fi::launch_kernel(reshape_and_cache_kernel<Tt>, dim3(T), dim3(256), 0, FI_STREAM(stream), 0, 
        (const Tt*)k, (const Tt*)v, slot_mapping, k_cache, v_cache, ldk, ldv, nkv, hd, block_size,
        kv_fp8, k_scale, v_scale);
    return static_cast<int>(cudaGetLastError());
  });
}

// Row-scaled cache write (modes 2 and 3, see kv_quant_rows_kernel).  dtype: 0 bf16, 1 fp16 (k, v).
extern "C" int fi_kv_quant_rows(const void* k, const void* v, long ldk, long ldv, const int* slot_mapping,
                                void* k_cache, void* v_cache, float* k_scales, float* v_scales, int T, int nkv,
                                int hd, int block_size, int mode, int dtype, void* stream) {
  if (T <= 0) return 0;
  if ((mode != 2 && mode != 3) || hd % 2 != 0 || nkv <= 0 || k_scales == nullptr || v_scales == nullptr) return -10;
  const int threads = 2 * nkv >= 8 ? 256 : 128;
  if (dtype == 0)
    fi::launch_kernel(kv_quant_rows_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, FI_STREAM(stream), 0,
                      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, ldk, ldv, slot_mapping, (uint8_t*)k_cache,
                      (uint8_t*)v_cache, k_scales, v_scales, nkv, hd, block_size, mode);
  else if (dtype == 1)
    fi::launch_kernel(kv_quant_rows_kernel<__half>, dim3(T), dim3(threads), 0, FI_STREAM(stream), 0, (const __half*)k,
                      (const __half*)v, ldk, ldv, slot_mapping, (uint8_t*)k_cache, (uint8_t*)v_cache, k_scales, v_scales,
                      nkv, hd, block_size, mode);
  else
    return -11;
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_embedding(const long* ids, const void* table, void* out, int T, int H,
                            float scale, int vocab_start, int vocab_end, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -10;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using Tt = std::remove_pointer_t<decltype(tag)>;
    int threads = H / 8 > 256 ? 256 : ((H / 8 + 31) / 32) * 32;
    fi::launch_kernel(embedding_kernel<Tt>, dim3(T), dim3(threads), 0, FI_STREAM(stream), 0, 
        ids, (const Tt*)table, (Tt*)out, H, scale, vocab_start, vocab_end);
    return static_cast<int>(cudaGetLastError());
  });
}

extern "C" int fi_act_mul(const void* x, void* out, int rows, int d, long ldx, int act, int dtype,
                          void* stream) {
  if (rows <= 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using Tt = std::remove_pointer_t<decltype(tag)>;
    fi::launch_kernel(act_mul_kernel<Tt>, dim3(rows), dim3(256), 0, FI_STREAM(stream), 0, (const Tt*)x, (Tt*)out, d, ldx, act);
    return static_cast<int>(cudaGetLastError());
  });
}

extern "C" int fi_act(const void* x, void* out, int rows, int d, long ldx, long ldo, int act, int dtype,
                      void* stream) {
  if (rows <= 0) return 0;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using Tt = std::remove_pointer_t<decltype(tag)>;
    fi::launch_kernel(act_kernel<Tt>, dim3(rows), dim3(256), 0, FI_STREAM(stream), 0, (const Tt*)x, (Tt*)out, d, ldx, ldo, act);
    return static_cast<int>(cudaGetLastError());
  });
}

extern "C" int fi_slot_mapping(const int* positions, const int* token_seq, const int* block_tables,
                               int max_blocks, int bs, int* slots, int T, void* stream) {
  if (T <= 0) return 0;
  fi::launch_kernel(slot_mapping_kernel, dim3((T + 255) / 256), dim3(256), 0, FI_STREAM(stream), 0, 
      positions, token_seq, block_tables, max_blocks, bs, slots, T);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_gather_rows_i32(const int* table, const int* idx, int* out, int rows, int cols,
                                  int n_table_rows, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (n_table_rows <= 0) return -10;
  fi::launch_kernel(gather_rows_i32_kernel, dim3(rows), dim3(cols >= 256 ? 256 : 64), 0, FI_STREAM(stream), 0,
                    table, idx, out, cols, n_table_rows);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_select_blocks(const int* table, const int* seq_lens, int* out_table, int* out_len, int rows,
                                int cols, int block_size, int stride, int min_blocks, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (block_size <= 0 || stride <= 0 || min_blocks < 0) return -10;
  fi::launch_kernel(select_blocks_kernel, dim3(rows), dim3(32), 0, FI_STREAM(stream), 0, table, seq_lens, out_table,
                    out_len, cols, block_size, stride, min_blocks);
  return static_cast<int>(cudaGetLastError());
}

// dtype: 0 bf16, 1 fp16, 2 fp32
extern "C" int fi_argmax(const void* logits, long ld, int rows, int V, long* out, int dtype,
                         void* stream) {
  if (rows <= 0) return 0;
  if (dtype == 2) {
    fi::launch_kernel(argmax_kernel<float>, dim3(rows), dim3(1024), 0, FI_STREAM(stream), 0, (const float*)logits, ld, V, out, 0.f);
  } else if (dtype == 0) {
    fi::launch_kernel(argmax_kernel<__nv_bfloat16>, dim3(rows), dim3(1024), 0, FI_STREAM(stream), 0, 
        (const __nv_bfloat16*)logits, ld, V, out, 0.f);
  } else {
    fi::launch_kernel(argmax_kernel<__half>, dim3(rows), dim3(1024), 0, FI_STREAM(stream), 0, (const __half*)logits, ld, V, out,
                                                                 0.f);
  }
  return static_cast<int>(cudaGetLastError());
}
