// Mixture-of-experts support kernels for sm_100a: router top-k, expert alignment (counting sort +
// tile table for the grouped GEMM), activation gather and weighted combine.
//
//   fi_moe_route   : scores -> top-k experts and weights per token, three scoring rules:
//                    0 softmax over all experts, top-k, renormalise (Gemma4: vllm/model_executor/
//                      models/gemma4/moe.py:98-125, optional per-expert scale),
//                    1 sigmoid scores, selection by score + correction bias, weights = normalised
//                      scores x routed scaling (DeepSeek-V3 style),
//                    2 sqrt(softplus) scores with bias (DeepSeek-V4-Flash: deepseek_v4_flash/
//                      gpu_layers.py:323-352).
//   fi_moe_align   : counting sort of the (token, k) routes by expert restricted to the experts this
//                    rank owns; emits sorted route ids, the inverse map, per-expert offsets and the
//                    tile table (expert, first row, rows) consumed by fi_awq_gemm_grouped.
//   fi_moe_gather  : x_sorted[slot] = x[route / k]
//   fi_moe_combine : out[t] = sum_k w[t,k] * y_sorted[slot(t,k)]  (+ optional residual), fp32 sums in
//                    a fixed order, so the result does not depend on the order of the sort.
// The reference routes with torch.topk/softmax and runs experts in Python loops or M<=16 Triton
// kernels (vllm/kernels/triton/gemma4_moe_int4.py); nothing there sorts tokens by expert on device.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../gemm/comm_desc.h"

namespace {

constexpr int kMaxExpertsPerLane = 16;   // experts <= 512

__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                 const float* __restrict__ expert_scale, int* __restrict__ topk_ids,
                                 float* __restrict__ topk_w, int T, int E, int K, int mode,
                                 int renorm, float routed_scale) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* row = logits + static_cast<long>(t) * E;
  float score[kMaxExpertsPerLane];   // value used for the weight
  float sel[kMaxExpertsPerLane];     // value used for the selection
  const int per = (E + 31) / 32;
  float mx = -CUDART_INF_F;
  for (int i = 0; i < per; ++i) {
    const int e = i * 32 + lane;
    const float v = e < E ? row[e] : -CUDART_INF_F;
    score[i] = v;
    mx = fmaxf(mx, v);
  }
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (mode == 0) {
    float sum = 0.f;
    for (int i = 0; i < per; ++i) {
      const int e = i * 32 + lane;
      score[i] = e < E ? __expf(score[i] - mx) : 0.f;
      sum += score[i];
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    for (int i = 0; i < per; ++i) { score[i] /= sum; sel[i] = (i * 32 + lane) < E ? score[i] : -CUDART_INF_F; }
  } else {
    for (int i = 0; i < per; ++i) {
      const int e = i * 32 + lane;
      if (e < E) {
        const float x = score[i];
        score[i] = mode == 1 ? 1.f / (1.f + __expf(-x)) : sqrtf(x > 20.f ? x : log1pf(__expf(x)));
        sel[i] = score[i] + (bias ? bias[e] : 0.f);
      } else {
        score[i] = 0.f;
        sel[i] = -CUDART_INF_F;
      }
    }
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int k = 0; k < K; ++k) {
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int i = 0; i < per; ++i) {
      const int e = i * 32 + lane;
      if (sel[i] > best || (sel[i] == best && e < bi)) { best = sel[i]; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    // owner lane reads the weight score and retires the expert
    float w = 0.f;
    if ((bi & 31) == lane) {
      w = score[bi >> 5];
      sel[bi >> 5] = -CUDART_INF_F;
    }
    w = __shfl_sync(0xffffffffu, w, bi & 31);
    wsum += w;
    if (lane == k) { my_w = w; my_id = bi; }
  }
  if (lane < K) {
    float w = my_w;
    if (renorm) w = w / fmaxf(wsum, 1e-20f);
    w *= routed_scale;
    if (expert_scale != nullptr) w *= expert_scale[my_id];
    topk_ids[static_cast<long>(t) * K + lane] = my_id;
    topk_w[static_cast<long>(t) * K + lane] = w;
  }
}

// One CTA.  Routes to experts outside [e_lo, e_hi) are dropped (slot_of = -1).
__global__ void moe_align_kernel(const int* __restrict__ topk_ids, int n_routes, int e_lo, int e_hi,
                                 int bn, int* __restrict__ sorted_route, int* __restrict__ slot_of,
                                 int* __restrict__ expert_offsets, int* __restrict__ tile_expert,
                                 int* __restrict__ tile_row0, int* __restrict__ tile_rows,
                                 int* __restrict__ n_tiles) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ int sm[];
  const int EL = e_hi - e_lo;
  int* counts = sm;            // [EL]
  int* offs = sm + EL;         // [EL + 1]
  int* cursor = offs + EL + 1; // [EL]
  for (int i = threadIdx.x; i < EL; i += blockDim.x) { counts[i] = 0; cursor[i] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < n_routes; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e >= e_lo && e < e_hi) atomicAdd(&counts[e - e_lo], 1);
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    // one warp: every lane owns a contiguous range of experts, the ranges are chained by a warp prefix sum
    const int lane = threadIdx.x;
    const int per = (EL + 31) / 32;
    const int e0 = min(EL, lane * per), e1 = min(EL, e0 + per);
    int rows = 0, tiles = 0;
    for (int e = e0; e < e1; ++e) { rows += counts[e]; tiles += (counts[e] + bn - 1) / bn; }
    int row_pre = rows, tile_pre = tiles;
    for (int o = 1; o < 32; o <<= 1) {
      const int r = __shfl_up_sync(0xffffffffu, row_pre, o), t = __shfl_up_sync(0xffffffffu, tile_pre, o);
      if (lane >= o) { row_pre += r; tile_pre += t; }
    }
    int acc = row_pre - rows, nt = tile_pre - tiles;
    for (int e = e0; e < e1; ++e) {
      offs[e] = acc;
      for (int r = 0; r < counts[e]; r += bn) {
        tile_expert[nt] = e;
        tile_row0[nt] = acc + r;
        tile_rows[nt] = min(bn, counts[e] - r);
        ++nt;
      }
      acc += counts[e];
    }
    if (lane == 31) {
      offs[EL] = row_pre;
      *n_tiles = tile_pre;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= EL; i += blockDim.x) expert_offsets[i] = offs[i];
  for (int i = threadIdx.x; i < n_routes; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e >= e_lo && e < e_hi) {
      const int slot = offs[e - e_lo] + atomicAdd(&cursor[e - e_lo], 1);
      sorted_route[slot] = i;
      slot_of[i] = slot;
    } else {
      slot_of[i] = -1;
    }
  }
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ sorted_route,
                                  const int* __restrict__ expert_offsets, int EL, int K, int H,
                                  T* __restrict__ x_sorted) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int slot = blockIdx.x;
  if (slot >= expert_offsets[EL]) return;
  const int tok = sorted_route[slot] / K;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long>(tok) * H);
  uint4* dst = reinterpret_cast<uint4*>(x_sorted + static_cast<long>(slot) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y_sorted, const int* __restrict__ slot_of,
                                   const float* __restrict__ topk_w, const T* __restrict__ residual,
                                   T* __restrict__ out, int K, int H) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int t = blockIdx.x;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < H / 8; c += blockDim.x * gridDim.y) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < K; ++k) {
      // a null map means the rows are already in (token, k) order
      const int slot = slot_of ? slot_of[static_cast<long>(t) * K + k] : t * K + k;
      if (slot < 0) continue;
      const float w = topk_w[static_cast<long>(t) * K + k];
      uint4 raw = *reinterpret_cast<const uint4*>(y_sorted + static_cast<long>(slot) * H + c * 8);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += w * static_cast<float>(e[j]);
    }
    if (residual != nullptr) {
      uint4 raw = *reinterpret_cast<const uint4*>(residual + static_cast<long>(t) * H + c * 8);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += static_cast<float>(e[j]);
    }
    uint4 o;
    T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) oe[j] = static_cast<T>(acc[j]);
    *reinterpret_cast<uint4*>(out + static_cast<long>(t) * H + c * 8) = o;
  }
}

// Expert-parallel combine fused with the all-reduce: every rank sums the routed outputs of ITS
// experts for a token, pushes that fp32 partial straight into every peer's receive slab over NVLink
// (each 8-byte word = one value + the call's epoch, so the receiver needs neither a fence nor a
// separate flag), then adds the peers' partials in rank order (bitwise identical on all ranks) plus
// the residual and writes the token.  One CTA per token; waits are bounded.
struct CombineComm {
  int world, rank;
  long slab_elems;                  // values per (parity, source rank) slab
  unsigned long long recv[8];       // low-latency receive area of rank d, as mapped here
  unsigned int* epoch;              // local: completed fused calls
  unsigned int* done;               // local: finished CTAs of this call
  int* status;
  int phases;
};

template <typename T>
__global__ void moe_combine_allreduce_kernel(const T* __restrict__ y_sorted, const int* __restrict__ slot_of,
                                             const float* __restrict__ topk_w, const T* __restrict__ residual,
                                             T* __restrict__ out, int K, int H, const CombineComm c) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ volatile int aborted;
  if (threadIdx.x == 0) aborted = 0;
  __syncthreads();
  const unsigned int epoch_now = *c.epoch + 1u;
  const long parity = epoch_now & 1u;
  const int t = blockIdx.x;
  const int phases = c.phases != 0 ? c.phases : 3;   // 1 = push partials, 2 = sum + store (split only when one GPU emulates several ranks)
  for (int ch = threadIdx.x; ch < H / 8; ch += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < K; ++k) {
      const int slot = slot_of ? slot_of[static_cast<long>(t) * K + k] : t * K + k;
      if (slot < 0) continue;   // routed to an expert of another rank
      const float w = topk_w[static_cast<long>(t) * K + k];
      uint4 raw = *reinterpret_cast<const uint4*>(y_sorted + static_cast<long>(slot) * H + ch * 8);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += w * static_cast<float>(e[j]);
    }
    const long elem = static_cast<long>(t) * H + ch * 8;
    const long my_off = (parity * c.world + c.rank) * c.slab_elems + elem;
    for (int d = 0; d < c.world; ++d) {
      if (d == c.rank || !(phases & 1)) continue;
      uint4* dst = reinterpret_cast<uint4*>(c.recv[d]) + (my_off >> 1);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        fi::st_volatile_v4(dst + q, make_uint4(__float_as_uint(acc[2 * q]), epoch_now,
                                               __float_as_uint(acc[2 * q + 1]), epoch_now));
    }
    if (!(phases & 2)) continue;
    float sum[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) sum[j] = 0.f;
    for (int s = 0; s < c.world; ++s) {
      float v[8];
      if (s == c.rank) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = acc[j];
      } else {
        const long off = (parity * c.world + s) * c.slab_elems + elem;
        const uint4* src = reinterpret_cast<const uint4*>(c.recv[c.rank]) + (off >> 1);
        const long long w0 = clock64();
        uint4 wv[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) wv[q] = fi::ld_volatile_v4(src + q);   // four independent loads in flight
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          while (wv[q].y != epoch_now || wv[q].w != epoch_now) {
            if (aborted || clock64() - w0 > FI_WAIT_CYCLES) {
              fi::set_status(c.status, fi::kStatusTimeoutPeer);
              aborted = 1;
              break;
            }
            wv[q] = fi::ld_volatile_v4(src + q);
          }
          v[2 * q] = __uint_as_float(wv[q].x);
          v[2 * q + 1] = __uint_as_float(wv[q].z);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sum[j] += v[j];
    }
    if (residual != nullptr) {
      uint4 raw = *reinterpret_cast<const uint4*>(residual + elem);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum[j] += static_cast<float>(e[j]);
    }
    if (!aborted) {
      uint4 o;
      T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) oe[j] = static_cast<T>(sum[j]);
      *reinterpret_cast<uint4*>(out + elem) = o;
    }
  }
  // the last CTA of the call publishes the new epoch for the next fused call
  if (!(phases & 2)) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.done, 1u) == gridDim.x - 1) {
      *c.done = 0;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(c.epoch) = epoch_now;
    }
  }
}

}  // namespace

#define FI_STREAM(s) reinterpret_cast<cudaStream_t>(s)

// comm: the FiComm descriptor of the symmetric heap with recv[] pointing at the low-latency slabs
extern "C" int fi_moe_combine_allreduce(const void* y_sorted, const int* slot_of, const float* topk_w,
                                        const void* residual, void* out, int T, int K, int H, int dtype,
                                        int* status, void* stream, const FiComm* comm) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || comm == nullptr || comm->world < 2 || comm->world > 8) return -10;
  if (static_cast<long>(T) * H > comm->slab_elems) return -11;
  CombineComm c;
  c.world = comm->world; c.rank = comm->rank; c.slab_elems = comm->slab_elems; c.phases = comm->phases;
  for (int d = 0; d < 8; ++d) c.recv[d] = comm->recv[d];
  c.epoch = reinterpret_cast<unsigned int*>(comm->epoch);
  c.done = reinterpret_cast<unsigned int*>(comm->done);
  c.status = status;
  if (dtype == 0)
    fi::launch_kernel(moe_combine_allreduce_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, FI_STREAM(stream), 0,
                      (const __nv_bfloat16*)y_sorted, slot_of, topk_w, (const __nv_bfloat16*)residual,
                      (__nv_bfloat16*)out, K, H, c);
  else
    fi::launch_kernel(moe_combine_allreduce_kernel<__half>, dim3(T), dim3(128), 0, FI_STREAM(stream), 0,
                      (const __half*)y_sorted, slot_of, topk_w, (const __half*)residual, (__half*)out, K, H, c);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_moe_route(const float* logits, const float* bias, const float* expert_scale,
                            int* topk_ids, float* topk_w, int T, int E, int K, int mode, int renorm,
                            float routed_scale, void* stream) {
  if (T <= 0) return 0;
  if (E > 32 * kMaxExpertsPerLane || K > 32 || K > E) return -10;
  fi::launch_kernel(moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, FI_STREAM(stream), 0, logits, bias,
                    expert_scale, topk_ids, topk_w, T, E, K, mode, renorm, routed_scale);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_moe_align(const int* topk_ids, int n_routes, int e_lo, int e_hi, int bn,
                            int* sorted_route, int* slot_of, int* expert_offsets, int* tile_expert,
                            int* tile_row0, int* tile_rows, int* n_tiles, void* stream) {
  if (n_routes <= 0) return 0;
  const int EL = e_hi - e_lo;
  if (EL <= 0 || EL > 4096) return -10;
  const size_t smem = (3 * EL + 1) * sizeof(int);
  fi::launch_kernel(moe_align_kernel, dim3(1), dim3(1024), smem, FI_STREAM(stream), 0, topk_ids, n_routes,
                    e_lo, e_hi, bn, sorted_route, slot_of, expert_offsets, tile_expert, tile_row0, tile_rows,
                    n_tiles);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_moe_gather(const void* x, const int* sorted_route, const int* expert_offsets, int EL,
                             int n_routes, int K, int H, void* x_sorted, int dtype, void* stream) {
  if (n_routes <= 0) return 0;
  if (H % 8 != 0) return -10;
  if (dtype == 0)
    fi::launch_kernel(moe_gather_kernel<__nv_bfloat16>, dim3(n_routes), dim3(128), 0, FI_STREAM(stream), 0,
                      (const __nv_bfloat16*)x, sorted_route, expert_offsets, EL, K, H, (__nv_bfloat16*)x_sorted);
  else
    fi::launch_kernel(moe_gather_kernel<__half>, dim3(n_routes), dim3(128), 0, FI_STREAM(stream), 0,
                      (const __half*)x, sorted_route, expert_offsets, EL, K, H, (__half*)x_sorted);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_moe_combine(const void* y_sorted, const int* slot_of, const float* topk_w,
                              const void* residual, void* out, int T, int K, int H, int dtype,
                              void* stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -10;
  if (dtype == 0)
    fi::launch_kernel(moe_combine_kernel<__nv_bfloat16>, dim3(T, T < 128 ? (H / 8 + 127) / 128 : 1), dim3(128), 0, FI_STREAM(stream), 0,
                      (const __nv_bfloat16*)y_sorted, slot_of, topk_w, (const __nv_bfloat16*)residual,
                      (__nv_bfloat16*)out, K, H);
  else
    fi::launch_kernel(moe_combine_kernel<__half>, dim3(T, T < 128 ? (H / 8 + 127) / 128 : 1), dim3(128), 0, FI_STREAM(stream), 0,
                      (const __half*)y_sorted, slot_of, topk_w, (const __half*)residual, (__half*)out, K, H);
  return static_cast<int>(cudaGetLastError());
}
