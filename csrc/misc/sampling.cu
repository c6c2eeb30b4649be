// Batched token sampling for sm_100a: temperature, top-k, top-p, min-p and one draw per row in one
// kernel, without sorting the vocabulary.
//
// One CTA (1024 threads) per row of fp32 logits.  Thresholds are found by radix selection over the
// order-preserving integer image of the scaled logits:
//   top-k : the k-th largest value (4 passes over 8-bit digits with counting histograms);
//   top-p : the value v such that the probability mass of strictly larger logits is still below
//           top_p (the token that crosses the threshold is kept), by the same 4 passes with
//           histograms of probability mass;
//   min-p : p >= min_p * p_max  <=>  logit >= max + ln(min_p).
// Masses are accumulated as 64-bit fixed-point integers, so sums do not depend on the order in which
// threads arrive and a given (logits, uniform number) pair always yields the same token.  The draw
// walks the kept tokens in index order until the running mass passes u * total.
// Ties at the k-th value are all kept (a sort would keep an arbitrary k of them).
// Reference: vllm/engine/sampling/sampler.py:9-114 (torch.sort + cumsum + multinomial per row).
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../common/launch.cuh"

namespace {

constexpr int kThreads = 1024;
constexpr float kFix = 1099511627776.f;   // 2^40: exp(x - max) in (0, 1] -> fixed point

__device__ __forceinline__ uint32_t key_of(float f) {          // monotone: larger float -> larger key
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float val_of(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

struct Shared {
  unsigned long long hist[256];
  unsigned long long warp_sum[32];
  float red[32];
  unsigned long long total;
  uint32_t prefix;
  unsigned long long remaining;
  int pick;
};

__device__ __forceinline__ float block_max(float v, Shared& sh) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sh.red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sh.red[0];
  for (int i = 1; i < kThreads / 32; ++i) r = fmaxf(r, sh.red[i]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ unsigned long long block_sum(unsigned long long v, Shared& sh) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh.warp_sum[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long r = 0;
  for (int i = 0; i < kThreads / 32; ++i) r += sh.warp_sum[i];
  __syncthreads();
  return r;
}

// Radix selection from the top: finds the largest key K such that weight{key > K} < target, where the
// weight of an element is 1 (COUNT) or its fixed-point mass.  Only elements with key >= floor_key take part.
template <bool COUNT>
__device__ uint32_t select_from_top(const float* __restrict__ row, int V, float inv_t, float mx,
                                    uint32_t floor_key, unsigned long long target, Shared& sh) {
  uint32_t prefix = 0;
  unsigned long long remaining = target;   // weight still to be covered inside the current prefix
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += kThreads) sh.hist[i] = 0;
    __syncthreads();
    const uint32_t mask_hi = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const float x = row[i] * inv_t;
      const uint32_t k = key_of(x);
      if (k < floor_key || (k & mask_hi) != prefix) continue;
      const unsigned long long w = COUNT ? 1ull : static_cast<unsigned long long>(__expf(x - mx) * kFix);
      atomicAdd(&sh.hist[(k >> shift) & 255u], w);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long acc = 0;
      int b = 255;
      for (; b > 0; --b) {                    // walk bins from the largest digit down
        if (acc + sh.hist[b] >= remaining) break;
        acc += sh.hist[b];
      }
      sh.prefix = prefix | (static_cast<uint32_t>(b) << shift);
      sh.remaining = remaining - acc;
    }
    __syncthreads();
    prefix = sh.prefix;
    remaining = sh.remaining;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, long ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ uniform, long* __restrict__ out) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ Shared sh;
  const int r = blockIdx.x;
  const float* row = logits + static_cast<long>(r) * ld;
  const float t = temperature[r];
  const float inv_t = 1.f / fmaxf(t, 1e-6f);
  // ---- max (and arg-max, lowest index on ties) of the scaled logits
  float mx = -CUDART_INF_F;
  for (int i = threadIdx.x; i < V; i += kThreads) mx = fmaxf(mx, row[i] * inv_t);
  mx = block_max(mx, sh);
  int amax = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += kThreads)
    if (row[i] * inv_t == mx) amax = min(amax, i);
  {
    float neg = -static_cast<float>(amax);
    neg = block_max(neg, sh);
    amax = static_cast<int>(-neg);
  }
  if (!(t > 0.f) || !(mx > -CUDART_INF_F)) {   // greedy row (or an empty one)
    if (threadIdx.x == 0) out[r] = amax == 0x7fffffff ? 0 : amax;
    return;
  }
  // ---- thresholds
  uint32_t floor_key = 0;
  const int k = top_k[r];
  if (k > 0 && k < V) floor_key = select_from_top<true>(row, V, inv_t, mx, 0u, static_cast<unsigned long long>(k), sh);
  const float mp = min_p[r];
  if (mp > 0.f) floor_key = max(floor_key, key_of(mx + __logf(mp)));
  unsigned long long z = 0;
  for (int i = threadIdx.x; i < V; i += kThreads) {
    const float x = row[i] * inv_t;
    if (key_of(x) >= floor_key) z += static_cast<unsigned long long>(__expf(x - mx) * kFix);
  }
  z = block_sum(z, sh);
  const float tp = top_p[r];
  if (tp < 1.f && z > 0) {
    unsigned long long target = static_cast<unsigned long long>(static_cast<double>(z) * static_cast<double>(fmaxf(tp, 0.f)));
    if (target < 1) target = 1;
    const uint32_t kp = select_from_top<false>(row, V, inv_t, mx, floor_key, target, sh);
    floor_key = max(floor_key, kp);
  }
  floor_key = min(floor_key, key_of(mx));   // the most likely token always survives
  // ---- total kept mass
  unsigned long long zf = 0;
  for (int i = threadIdx.x; i < V; i += kThreads) {
    const float x = row[i] * inv_t;
    if (key_of(x) >= floor_key) zf += static_cast<unsigned long long>(__expf(x - mx) * kFix);
  }
  zf = block_sum(zf, sh);
  if (zf == 0) {
    if (threadIdx.x == 0) out[r] = amax;
    return;
  }
  // ---- draw: first kept index whose running mass reaches u * total
  double u = static_cast<double>(uniform[r]);
  u = u < 0.0 ? 0.0 : (u >= 1.0 ? 0.9999999 : u);
  unsigned long long target = static_cast<unsigned long long>(u * static_cast<double>(zf)) + 1ull;
  if (target > zf) target = zf;
  if (threadIdx.x == 0) { sh.pick = -1; sh.total = 0; }
  __syncthreads();
  for (int base = 0; base < V; base += kThreads) {
    const int i = base + threadIdx.x;
    unsigned long long w = 0;
    if (i < V) {
      const float x = row[i] * inv_t;
      if (key_of(x) >= floor_key) w = static_cast<unsigned long long>(__expf(x - mx) * kFix);
    }
    // inclusive scan inside the warp, then across warps
    unsigned long long s = w;
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long n = __shfl_up_sync(0xffffffffu, s, o);
      if ((threadIdx.x & 31) >= o) s += n;
    }
    if ((threadIdx.x & 31) == 31) sh.warp_sum[threadIdx.x >> 5] = s;
    __syncthreads();
    unsigned long long before = sh.total;
    for (int wdx = 0; wdx < (threadIdx.x >> 5); ++wdx) before += sh.warp_sum[wdx];
    const unsigned long long incl = before + s;
    if (w > 0 && incl >= target && incl - w < target) sh.pick = i;   // exactly one thread
    __syncthreads();
    if (sh.pick >= 0) break;
    if (threadIdx.x == kThreads - 1) sh.total = incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) out[r] = sh.pick >= 0 ? sh.pick : amax;
}

}  // namespace

// logits: fp32 [rows, V] (row pitch ld); per-row temperature (<= 0: arg-max), top_k (<= 0: off),
// top_p (>= 1: off), min_p (<= 0: off), one uniform number in [0, 1) per row; out: int64 [rows].
extern "C" int fi_sample(const float* logits, long ld, int rows, int V, const float* temperature, const int* top_k,
                         const float* top_p, const float* min_p, const float* uniform, long* out, void* stream) {
  if (rows <= 0) return 0;
  if (V <= 0) return -10;
  fi::launch_kernel(sample_kernel, dim3(rows), dim3(kThreads), 0, reinterpret_cast<cudaStream_t>(stream), 0, logits, ld,
                    V, temperature, top_k, top_p, min_p, uniform, out);
  return static_cast<int>(cudaGetLastError());
}
