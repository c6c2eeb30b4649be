// DeepSeek-V4-Flash specific device ops for sm_100a (bandwidth/latency-bound helpers around the
// shared-latent attention of that model family):
//
//   fi_dsv4_indexer_qat      : in place, per 128-wide row: 128-point Hadamard transform (scaled by
//                              1/sqrt(128)) then an FP4 E2M1 quantise-dequantise round trip with one
//                              power-of-two scale per 32 values.  Reference: vllm/kernels/triton/
//                              deepseek_v4_flash/indexer_qat.py:9-66.
//   fi_dsv4_indexer_scores   : lightning-indexer score of every compressed row,
//                              score[r] = scale * sum_h w[h] * relu(q[h] . row[r]).
//                              Reference: .../compressed_indexer_select.py:9-55.
//   fi_dsv4_shared_kv_attention : attention of `heads` queries over latent rows that serve as both
//                              keys and values (K = V), with a per-head sink logit that only enters
//                              the softmax denominator.  Rows are addressed through an optional
//                              index list (selected compressed rows) and an optional page table
//                              (lazily grown pools), so one kernel covers the sliding-window rows,
//                              the compressed rows and their union.  Reference: .../attention.py:
//                              64-145 and .../compressed_attention_triton.py:20-86.
//   fi_dsv4_shared_kv_attention_run : the same attention for a run of consecutive tokens of one request (a
//                              prefill chunk) in one launch: per token a window range of a linear row buffer plus
//                              a prefix, or a selected list, of the compressed rows.
//   fi_dsv4_shared_kv_attention_ptrs : the same attention for one token of each request of a decode batch in one
//                              launch (per-request row pools through a pointer array).
//   fi_dsv4_cache_update     : write latent rows through a page table.  Reference: .../cache.py:41-65.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../common/launch.cuh"

namespace {

__device__ __forceinline__ float e2m1_round(float a) {   // a >= 0, nearest of {0,.5,1,1.5,2,3,4,6}, ties to the even code
  if (a <= 0.25f) return 0.f;
  if (a < 0.75f) return 0.5f;
  if (a <= 1.25f) return 1.f;
  if (a < 1.75f) return 1.5f;
  if (a <= 2.5f) return 2.f;
  if (a < 3.5f) return 3.f;
  if (a <= 5.f) return 4.f;
  return 6.f;
}

// one warp per 128-wide row: lane l holds elements l, l+32, l+64, l+96
__global__ void indexer_qat_kernel(float* __restrict__ rows, int n_rows) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= n_rows) return;
  float* row = rows + static_cast<long>(warp) * 128;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = row[j * 32 + lane];
  // butterflies with stride 1..16 act inside each 32-wide segment (across lanes)
#pragma unroll
  for (int stride = 1; stride < 32; stride <<= 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, v[j], stride);
      v[j] = (lane & stride) ? other - v[j] : v[j] + other;
    }
  }
  // strides 32 and 64 act across the four registers
  {
    const float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
    v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float x = v[j] * 0.08838834764831845f;
    // block of 32 = one register index across the warp
    float amax = fabsf(x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    amax = fmaxf(amax, 7.052966104933725e-38f);
    const float scale = exp2f(ceilf(log2f(amax / 6.f)));
    const float q = fminf(fabsf(x) / scale, 6.f);
    row[j * 32 + lane] = copysignf(e2m1_round(q) * scale, x);
  }
}

// one warp per compressed row; q [H,128] and w [H] staged in shared memory
__global__ void indexer_scores_kernel(const float* __restrict__ q, const float* __restrict__ w,
                                      const float* __restrict__ rows, int n_rows, int H, float scale,
                                      float* __restrict__ out) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ float sm[];
  float* qs = sm;            // [H][128]
  float* ws = sm + H * 128;  // [H]
  for (int i = threadIdx.x; i < H * 128; i += blockDim.x) qs[i] = q[i];
  for (int i = threadIdx.x; i < H; i += blockDim.x) ws[i] = w[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  for (int r = blockIdx.x * warps + (threadIdx.x >> 5); r < n_rows; r += gridDim.x * warps) {
    float x[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = rows[static_cast<long>(r) * 128 + j * 32 + lane];
    float total = 0.f;
    for (int h = 0; h < H; ++h) {
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) d += x[j] * qs[h * 128 + j * 32 + lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      total += ws[h] * fmaxf(d, 0.f);
    }
    if (lane == 0) out[r] = total * scale;
  }
}

__device__ __forceinline__ long resolve_row(int r, const int* __restrict__ row_index,
                                            const int* __restrict__ page_table, int page_rows) {
  const int logical = row_index ? row_index[r] : r;
  if (page_table == nullptr) return logical;
  return static_cast<long>(page_table[logical / page_rows]) * page_rows + logical % page_rows;
}

// one CTA (128 threads) per head; D <= 512, D % 128 == 0; rows in chunks of 32
constexpr int kChunk = 32;
__global__ void __launch_bounds__(128) shared_kv_attention_kernel(
    const float* __restrict__ q, const float* __restrict__ pool, const int* __restrict__ row_index,
    const int* __restrict__ page_table, int page_rows, const float* __restrict__ sinks, int n_rows, int D,
    float scale, float* __restrict__ out) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ float qs[512];
  __shared__ float sc[kChunk];
  __shared__ long base[kChunk];
  const int h = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < D; i += 128) qs[i] = q[static_cast<long>(h) * D + i] * scale;
  const int per = D / 128;   // output dims per thread
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float m = sinks ? sinks[h] : -CUDART_INF_F;   // the sink is a logit without a value row
  float l = sinks ? 1.f : 0.f;
  __syncthreads();
  for (int r0 = 0; r0 < n_rows; r0 += kChunk) {
    const int n = min(kChunk, n_rows - r0);
    if (threadIdx.x < n) base[threadIdx.x] = resolve_row(r0 + threadIdx.x, row_index, page_table, page_rows) * D;
    __syncthreads();
    for (int i = warp; i < n; i += 4) {
      const float* row = pool + base[i];
      float d = 0.f;
      for (int c = lane; c < D; c += 32) d += qs[c] * row[c];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (lane == 0) sc[i] = d;
    }
    __syncthreads();
    float cm = m;
    for (int i = 0; i < n; ++i) cm = fmaxf(cm, sc[i]);
    const float corr = (m == -CUDART_INF_F) ? 0.f : __expf(m - cm);
    l *= corr;
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] *= corr;
    for (int i = 0; i < n; ++i) {
      const float p = __expf(sc[i] - cm);
      l += p;
      const float* row = pool + base[i];
      for (int j = 0; j < per; ++j) acc[j] += p * row[j * 128 + threadIdx.x];
    }
    m = cm;
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int j = 0; j < per; ++j) out[static_cast<long>(h) * D + j * 128 + threadIdx.x] = acc[j] * inv;
}

// A run of consecutive tokens of one request in one launch: CTA (head, token).  Token t attends the window rows
// lin[a0[t] .. a0[t] + na[t]) (its own row last) and nb[t] compressed rows of `comp`: the first nb[t] rows, or with
// a selection table the rows sel[t * sel_stride + 0 .. nb[t]).  q and out are [T, heads, D].
__global__ void __launch_bounds__(128) shared_kv_attention_run_kernel(
    const float* __restrict__ q, const float* __restrict__ lin, const float* __restrict__ comp,
    const int* __restrict__ a0, const int* __restrict__ na, const int* __restrict__ nb, const int* __restrict__ sel,
    int sel_stride, const float* __restrict__ sinks, int heads, int D, float scale, float* __restrict__ out) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ float qs[512];
  __shared__ float sc[kChunk];
  __shared__ const float* rowp[kChunk];
  const int h = blockIdx.x, t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long qo = (static_cast<long>(t) * heads + h) * D;
  for (int i = threadIdx.x; i < D; i += 128) qs[i] = q[qo + i] * scale;
  const int per = D / 128;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float m = sinks ? sinks[h] : -CUDART_INF_F;
  float l = sinks ? 1.f : 0.f;
  const int n_a = na[t], n_rows = n_a + nb[t], start = a0[t];
  __syncthreads();
  for (int r0 = 0; r0 < n_rows; r0 += kChunk) {
    const int n = min(kChunk, n_rows - r0);
    if (threadIdx.x < n) {
      const int r = r0 + threadIdx.x;
      if (r < n_a) rowp[threadIdx.x] = lin + static_cast<long>(start + r) * D;
      else rowp[threadIdx.x] = comp + static_cast<long>(sel ? sel[static_cast<long>(t) * sel_stride + (r - n_a)] : (r - n_a)) * D;
    }
    __syncthreads();
    for (int i = warp; i < n; i += 4) {
      const float* row = rowp[i];
      float d = 0.f;
      for (int c = lane; c < D; c += 32) d += qs[c] * row[c];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (lane == 0) sc[i] = d;
    }
    __syncthreads();
    float cm = m;
    for (int i = 0; i < n; ++i) cm = fmaxf(cm, sc[i]);
    const float corr = (m == -CUDART_INF_F) ? 0.f : __expf(m - cm);
    l *= corr;
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] *= corr;
    for (int i = 0; i < n; ++i) {
      const float p = __expf(sc[i] - cm);
      l += p;
      const float* row = rowp[i];
      for (int j = 0; j < per; ++j) acc[j] += p * row[j * 128 + threadIdx.x];
    }
    m = cm;
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int j = 0; j < per; ++j) out[qo + j * 128 + threadIdx.x] = acc[j] * inv;
}

// One token of each of T requests (a decode batch): CTA (head, token).  pools[t] points to that request's rows:
// the first n_win[t] rows are its sliding window (ring order is irrelevant to attention), its compressed rows
// start at row `comp_row0`; token t attends nb[t] of them: the first nb[t], or sel[t * sel_stride + ..] when
// use_sel[t] is set.
__global__ void __launch_bounds__(128) shared_kv_attention_ptrs_kernel(
    const float* __restrict__ q, const float* const* __restrict__ pools, const int* __restrict__ n_win,
    const int* __restrict__ nb, const int* __restrict__ use_sel, const int* __restrict__ sel, int sel_stride,
    int comp_row0, const float* __restrict__ sinks, int heads, int D, float scale, float* __restrict__ out) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ float qs[512];
  __shared__ float sc[kChunk];
  __shared__ const float* rowp[kChunk];
  const int h = blockIdx.x, t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long qo = (static_cast<long>(t) * heads + h) * D;
  for (int i = threadIdx.x; i < D; i += 128) qs[i] = q[qo + i] * scale;
  const int per = D / 128;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float m = sinks ? sinks[h] : -CUDART_INF_F;
  float l = sinks ? 1.f : 0.f;
  const float* pool = pools[t];
  const int n_a = n_win[t], n_rows = n_a + nb[t];
  const bool by_sel = sel != nullptr && use_sel[t] != 0;
  __syncthreads();
  for (int r0 = 0; r0 < n_rows; r0 += kChunk) {
    const int n = min(kChunk, n_rows - r0);
    if (threadIdx.x < n) {
      const int r = r0 + threadIdx.x;
      const int row = r < n_a ? r : comp_row0 + (by_sel ? sel[static_cast<long>(t) * sel_stride + (r - n_a)] : (r - n_a));
      rowp[threadIdx.x] = pool + static_cast<long>(row) * D;
    }
    __syncthreads();
    for (int i = warp; i < n; i += 4) {
      const float* row = rowp[i];
      float d = 0.f;
      for (int c = lane; c < D; c += 32) d += qs[c] * row[c];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (lane == 0) sc[i] = d;
    }
    __syncthreads();
    float cm = m;
    for (int i = 0; i < n; ++i) cm = fmaxf(cm, sc[i]);
    const float corr = (m == -CUDART_INF_F) ? 0.f : __expf(m - cm);
    l *= corr;
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] *= corr;
    for (int i = 0; i < n; ++i) {
      const float p = __expf(sc[i] - cm);
      l += p;
      const float* row = rowp[i];
      for (int j = 0; j < per; ++j) acc[j] += p * row[j * 128 + threadIdx.x];
    }
    m = cm;
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int j = 0; j < per; ++j) out[qo + j * 128 + threadIdx.x] = acc[j] * inv;
}

__global__ void cache_update_kernel(const float* __restrict__ rows, const int* __restrict__ positions,
                                    const int* __restrict__ page_table, int page_rows, int D,
                                    float* __restrict__ pool) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int r = blockIdx.x;
  const long dst = resolve_row(positions[r], nullptr, page_table, page_rows) * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) pool[dst + c] = rows[static_cast<long>(r) * D + c];
}

}  // namespace

#define FI_STREAM(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int fi_dsv4_indexer_qat(float* rows, int n_rows, void* stream) {
  if (n_rows <= 0) return 0;
  fi::launch_kernel(indexer_qat_kernel, dim3((n_rows + 3) / 4), dim3(128), 0, FI_STREAM(stream), 0, rows, n_rows);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_indexer_scores(const float* q, const float* w, const float* rows, int n_rows, int H,
                                      float scale, float* out, void* stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = static_cast<size_t>(H) * 129 * sizeof(float);
  if (smem > 200 * 1024) return -10;
  if (cudaError_t e = fi::ensure_dynamic_smem(indexer_scores_kernel, 200 * 1024); e != cudaSuccess) return static_cast<int>(e);
  const int blocks = n_rows < 8 * 148 ? (n_rows + 7) / 8 : 148;
  fi::launch_kernel(indexer_scores_kernel, dim3(blocks), dim3(256), smem, FI_STREAM(stream), 0, q, w, rows, n_rows, H,
                    scale, out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_shared_kv_attention(const float* q, const float* pool, const int* row_index,
                                           const int* page_table, int page_rows, const float* sinks, int heads,
                                           int n_rows, int D, float scale, float* out, void* stream) {
  if (heads <= 0) return 0;
  if (D > 512 || D % 128 != 0 || n_rows < 0 || (page_table != nullptr && page_rows <= 0)) return -10;
  fi::launch_kernel(shared_kv_attention_kernel, dim3(heads), dim3(128), 0, FI_STREAM(stream), 0, q, pool, row_index,
                    page_table, page_rows, sinks, n_rows, D, scale, out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_shared_kv_attention_run(const float* q, const float* lin, const float* comp, const int* a0,
                                               const int* na, const int* nb, const int* sel, int sel_stride,
                                               const float* sinks, int T, int heads, int D, float scale, float* out,
                                               void* stream) {
  if (heads <= 0 || T <= 0) return 0;
  if (D > 512 || D % 128 != 0 || T > 65535 || (sel != nullptr && sel_stride <= 0)) return -10;
  fi::launch_kernel(shared_kv_attention_run_kernel, dim3(heads, T), dim3(128), 0, FI_STREAM(stream), 0, q, lin, comp, a0,
                    na, nb, sel, sel_stride, sinks, heads, D, scale, out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_shared_kv_attention_ptrs(const float* q, void* pools, const int* n_win, const int* nb,
                                                const int* use_sel, const int* sel, int sel_stride, int comp_row0,
                                                const float* sinks, int T, int heads, int D, float scale, float* out,
                                                void* stream) {
  if (heads <= 0 || T <= 0) return 0;
  if (D > 512 || D % 128 != 0 || T > 65535 || comp_row0 < 0 || (sel != nullptr && (sel_stride <= 0 || use_sel == nullptr)))
    return -10;
  fi::launch_kernel(shared_kv_attention_ptrs_kernel, dim3(heads, T), dim3(128), 0, FI_STREAM(stream), 0, q,
                    static_cast<const float* const*>(pools), n_win, nb, use_sel, sel, sel_stride, comp_row0, sinks, heads, D,
                    scale, out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_cache_update(const float* rows, const int* positions, const int* page_table, int page_rows,
                                    int n, int D, float* pool, void* stream) {
  if (n <= 0) return 0;
  if (page_table != nullptr && page_rows <= 0) return -10;
  fi::launch_kernel(cache_update_kernel, dim3(n), dim3(128), 0, FI_STREAM(stream), 0, rows, positions, page_table,
                    page_rows, D, pool);
  return static_cast<int>(cudaGetLastError());
}
