// Per-token glue of the DeepSeek-V4-Flash layer for sm_100a.  Each of these replaces a chain of ten to a hundred
// elementwise launches of the eager formulation with one kernel; all work in fp32 on rows of a few thousand
// values, so they are launch-latency bound and sized for that (one CTA per token or per row).
//
//   fi_dsv4_hc_pre      : manifold hyper-connection, front half.  From the `hc` residual streams of a token and
//                         the raw mixing logits (flattened streams @ fn, computed by a GEMM): RMS scale of the
//                         flattened streams, gains + base, sigmoid "pre" weights -> mixed layer input,
//                         "post" gains, and the hc x hc stream-mixing matrix made doubly stochastic by Sinkhorn
//                         iterations.  Reference: vllm/model_executor/models/deepseek_v4_flash/
//                         hyper_connection.py:16-129.
//   fi_dsv4_hc_post     : back half: new_stream[j] = post[j] * layer_out + sum_i combine[i][j] * stream[i].
//   fi_dsv4_hc_collapse : after the last layer: sigmoid gains from the raw logits, gated sum of the streams.
//   fi_dsv4_norm_rope   : per row: optional RMS norm (optional weight), optional rotary on the last `rot`
//                         channels (adjacent pairs, per-pair angle step, forward or inverse), optional FP8 E4M3
//                         round trip of the non-rotary part in blocks of 64 with power-of-two scales.
//                         Covers the q latent norm, per-head q norm + rotary, the latent KV row (norm, rotary,
//                         fp8), emitted compressed rows, layer-input norms and the inverse rotary of the
//                         attention output.  Reference: .../attention.py:141-197, ops.py (fp8 KV round trip).
//   fi_dsv4_compressor_step : one token into the rolling compressor window (in place) and, every `ratio`
//                         tokens, the softmax(score)-weighted row.  Reference: .../attention.py:665-760.
//   fi_dsv4_compressor_step_batch / fi_dsv4_scatter_rows : the compressor step and the window-row write for one
//                         token of each request of a decode batch (per-request state and pool addresses come in
//                         pointer arrays).
//   fi_dsv4_q8k_roundtrip : Q8_K activation round trip (blocks of 256, scale from the signed extreme value).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../common/launch.cuh"

namespace {

constexpr int kMaxHc = 8;

__device__ __forceinline__ float block_sum(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nw; ++w) t += red[w];
  return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[0];
  for (int w = 1; w < nw; ++w) t = fmaxf(t, red[w]);
  return t;
}

__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

// grid T, block 256
__global__ void hc_pre_kernel(const float* __restrict__ streams, const float* __restrict__ raw,
                              const float* __restrict__ base, const float* __restrict__ scale, int hc, int H,
                              float eps, int iters, float* __restrict__ mixed, float* __restrict__ post,
                              float* __restrict__ combine) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ float red[32];
  __shared__ float s_pre[kMaxHc];
  const int t = blockIdx.x;
  const float* st = streams + static_cast<long>(t) * hc * H;
  const int n = hc * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += st[i] * st[i];
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / static_cast<float>(n) + eps);
  const int n_mix = 2 * hc + hc * hc;
  if (threadIdx.x == 0) {
    const float* r = raw + static_cast<long>(t) * n_mix;
    float m[kMaxHc * kMaxHc];
    for (int i = 0; i < hc; ++i) {
      s_pre[i] = sigmoidf(r[i] * inv * scale[0] + base[i]) + eps;
      post[static_cast<long>(t) * hc + i] = 2.f * sigmoidf(r[hc + i] * inv * scale[1] + base[hc + i]);
    }
    // rows softmax + eps, columns normalised, then alternate rows / columns
    for (int i = 0; i < hc; ++i) {
      float mx = -CUDART_INF_F;
      for (int j = 0; j < hc; ++j) {
        m[i * hc + j] = r[2 * hc + i * hc + j] * inv * scale[2] + base[2 * hc + i * hc + j];
        mx = fmaxf(mx, m[i * hc + j]);
      }
      float s = 0.f;
      for (int j = 0; j < hc; ++j) { m[i * hc + j] = __expf(m[i * hc + j] - mx); s += m[i * hc + j]; }
      for (int j = 0; j < hc; ++j) m[i * hc + j] = m[i * hc + j] / s + eps;
    }
    for (int it = 0; it < iters; ++it) {
      if (it > 0) {
        for (int i = 0; i < hc; ++i) {
          float s = 0.f;
          for (int j = 0; j < hc; ++j) s += m[i * hc + j];
          for (int j = 0; j < hc; ++j) m[i * hc + j] /= (s + eps);
        }
      }
      for (int j = 0; j < hc; ++j) {
        float s = 0.f;
        for (int i = 0; i < hc; ++i) s += m[i * hc + j];
        for (int i = 0; i < hc; ++i) m[i * hc + j] /= (s + eps);
      }
    }
    for (int i = 0; i < hc * hc; ++i) combine[static_cast<long>(t) * hc * hc + i] = m[i];
  }
  __syncthreads();
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < hc; ++i) acc += s_pre[i] * st[i * H + h];
    mixed[static_cast<long>(t) * H + h] = acc;
  }
}

// grid (T, ceil(H / 256)), block 256
__global__ void hc_post_kernel(const float* __restrict__ out, const float* __restrict__ streams,
                               const float* __restrict__ post, const float* __restrict__ combine, int hc, int H,
                               float* __restrict__ next) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int t = blockIdx.x;
  const int h = blockIdx.y * blockDim.x + threadIdx.x;
  if (h >= H) return;
  const float o = out[static_cast<long>(t) * H + h];
  float s[kMaxHc];
  for (int i = 0; i < hc; ++i) s[i] = streams[(static_cast<long>(t) * hc + i) * H + h];
  for (int j = 0; j < hc; ++j) {
    float acc = post[static_cast<long>(t) * hc + j] * o;
    for (int i = 0; i < hc; ++i) acc += combine[(static_cast<long>(t) * hc + i) * hc + j] * s[i];
    next[(static_cast<long>(t) * hc + j) * H + h] = acc;
  }
}

// grid T, block 256: gains = sigmoid(raw * inv_rms * scale + base) + 1e-6
__global__ void hc_collapse_kernel(const float* __restrict__ streams, const float* __restrict__ raw,
                                   const float* __restrict__ base, const float* __restrict__ scale, int hc, int H,
                                   float eps, float* __restrict__ out) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const float* st = streams + static_cast<long>(t) * hc * H;
  const int n = hc * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += st[i] * st[i];
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / static_cast<float>(n) + eps);
  float g[kMaxHc];
  for (int i = 0; i < hc; ++i) g[i] = sigmoidf(raw[static_cast<long>(t) * hc + i] * inv * scale[0] + base[i]) + 1e-6f;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float acc = 0.f;
    for (int i = 0; i < hc; ++i) acc += g[i] * st[i * H + h];
    out[static_cast<long>(t) * H + h] = acc;
  }
}

// grid rows, block 128.  x, y: [rows, D]; w: [D] or null; inv_freq: [rot / 2]; pos: [rows / rows_per_pos].
__global__ void norm_rope_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ inv_freq,
                                 const long* __restrict__ pos, int rows_per_pos, int D, int rot, int do_norm,
                                 int inverse, int fp8, float eps, float* __restrict__ y) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  extern __shared__ float row[];
  __shared__ float red[32];
  const long r = blockIdx.x;
  const float* xr = x + r * D;
  float ss = 0.f;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    const float v = xr[c];
    row[c] = v;
    ss += v * v;
  }
  float inv = 1.f;
  if (do_norm) {
    ss = block_sum(ss, red);
    inv = rsqrtf(ss / static_cast<float>(D) + eps);
  } else {
    __syncthreads();
  }
  for (int c = threadIdx.x; c < D; c += blockDim.x) row[c] = row[c] * inv * (w != nullptr ? w[c] : 1.f);
  __syncthreads();
  const int nope = D - rot;
  if (rot > 0) {
    double p = static_cast<double>(pos[r / rows_per_pos]);
    if (inverse) p = -p;
    for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
      // the angle reaches millions of radians at long context: reduce it to [-pi, pi] in double before the
      // single-precision sine and cosine
      double ang = p * static_cast<double>(inv_freq[i]);
      ang -= 6.283185307179586 * rint(ang * 0.15915494309189535);
      float sn, cs;
      sincosf(static_cast<float>(ang), &sn, &cs);
      const float a = row[nope + 2 * i], b = row[nope + 2 * i + 1];
      row[nope + 2 * i] = a * cs - b * sn;
      row[nope + 2 * i + 1] = a * sn + b * cs;
    }
  }
  if (fp8) {
    // blocks of 64 values, one warp per block: scale = 2^ceil(log2(amax / 448)), amax >= 1e-4
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int b = warp; b < nope / 64; b += nw) {
      const float v0 = row[b * 64 + lane], v1 = row[b * 64 + 32 + lane];
      float am = fmaxf(fabsf(v0), fabsf(v1));
      for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
      am = fmaxf(am, 1e-4f);
      int e;
      const float mant = frexpf(am / 448.f, &e);            // am / 448 = mant * 2^e, mant in [0.5, 1)
      const float sc = ldexpf(1.f, mant > 0.5f ? e : e - 1);   // 2^ceil(log2(am / 448)), exact
      const float q0 = fminf(fmaxf(v0 / sc, -448.f), 448.f), q1 = fminf(fmaxf(v1 / sc, -448.f), 448.f);
      const __nv_fp8_e4m3 f0(q0), f1(q1);
      row[b * 64 + lane] = static_cast<float>(f0) * sc;
      row[b * 64 + 32 + lane] = static_cast<float>(f1) * sc;
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += blockDim.x) y[r * D + c] = row[c];
}

// One token into a compressor window.  state_kv / state_score: [coff * ratio, width] with width = coff * head_dim,
// coff = 2 for ratio 4 (two overlapping windows) else 1.  grid 1, block 256.  emitted: [head_dim], written when
// (pos + 1) % ratio == 0.
__global__ void compressor_step_kernel(float* __restrict__ state_kv, float* __restrict__ state_score,
                                       const float* __restrict__ kv_cur, const float* __restrict__ score_cur,
                                       const float* __restrict__ ape, long ape_stride_pos, long ape_stride_c, int pos,
                                       int ratio, int head_dim, float* __restrict__ emitted) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int coff = ratio == 4 ? 2 : 1;
  const int width = coff * head_dim;
  const int slot = pos % ratio;
  const int row = ratio == 4 ? ratio + slot : slot;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    state_kv[static_cast<long>(row) * width + c] = kv_cur[c];
    state_score[static_cast<long>(row) * width + c] = score_cur[c] + ape[slot * ape_stride_pos + c * ape_stride_c];
  }
  __syncthreads();
  if ((pos + 1) % ratio != 0) return;
  // ratio 4: rows 0..3 use the first half-width of the previous window, rows 4..7 the second half of the current
  const int n_rows = coff * ratio;
  for (int c = threadIdx.x; c < head_dim; c += blockDim.x) {
    float mx = -CUDART_INF_F;
    for (int r = 0; r < n_rows; ++r) {
      const int col = (ratio == 4 && r >= ratio) ? head_dim + c : c;
      mx = fmaxf(mx, state_score[static_cast<long>(r) * width + col]);
    }
    float den = 0.f, num = 0.f;
    if (mx > -CUDART_INF_F) {
      for (int r = 0; r < n_rows; ++r) {
        const int col = (ratio == 4 && r >= ratio) ? head_dim + c : c;
        const float e = __expf(state_score[static_cast<long>(r) * width + col] - mx);
        den += e;
        num += e * state_kv[static_cast<long>(r) * width + col];
      }
    }
    emitted[c] = den > 0.f ? num / den : 0.f;
  }
  __syncthreads();
  if (ratio == 4) {
    for (int i = threadIdx.x; i < ratio * width; i += blockDim.x) {
      state_kv[i] = state_kv[static_cast<long>(ratio) * width + i];
      state_score[i] = state_score[static_cast<long>(ratio) * width + i];
    }
  }
}

// The same step for one token of each of `n` requests (a decode batch): CTA i works on the state that
// state_kv[i] / state_score[i] point to, with kv_cur / score_cur rows of pitch `pitch` floats and pos[i].
// emitted: [n, head_dim]; row i is written when (pos[i] + 1) % ratio == 0.
__global__ void compressor_step_batch_kernel(float* const* __restrict__ state_kv, float* const* __restrict__ state_score,
                                             const float* __restrict__ kv_cur, const float* __restrict__ score_cur,
                                             long pitch, const float* __restrict__ ape, long ape_stride_pos,
                                             long ape_stride_c, const long* __restrict__ pos, int ratio, int head_dim,
                                             float* __restrict__ emitted) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int i = blockIdx.x;
  float* skv = state_kv[i];
  float* ssc = state_score[i];
  const float* kc = kv_cur + i * pitch;
  const float* sc = score_cur + i * pitch;
  const int p = static_cast<int>(pos[i]);
  const int coff = ratio == 4 ? 2 : 1;
  const int width = coff * head_dim;
  const int slot = p % ratio;
  const int row = ratio == 4 ? ratio + slot : slot;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    skv[static_cast<long>(row) * width + c] = kc[c];
    ssc[static_cast<long>(row) * width + c] = sc[c] + ape[slot * ape_stride_pos + c * ape_stride_c];
  }
  __syncthreads();
  if ((p + 1) % ratio != 0) return;
  const int n_rows = coff * ratio;
  for (int c = threadIdx.x; c < head_dim; c += blockDim.x) {
    float mx = -CUDART_INF_F;
    for (int r = 0; r < n_rows; ++r) {
      const int col = (ratio == 4 && r >= ratio) ? head_dim + c : c;
      mx = fmaxf(mx, ssc[static_cast<long>(r) * width + col]);
    }
    float den = 0.f, num = 0.f;
    if (mx > -CUDART_INF_F) {
      for (int r = 0; r < n_rows; ++r) {
        const int col = (ratio == 4 && r >= ratio) ? head_dim + c : c;
        const float e = __expf(ssc[static_cast<long>(r) * width + col] - mx);
        den += e;
        num += e * skv[static_cast<long>(r) * width + col];
      }
    }
    emitted[static_cast<long>(i) * head_dim + c] = den > 0.f ? num / den : 0.f;
  }
  __syncthreads();
  if (ratio == 4) {
    for (int k = threadIdx.x; k < ratio * width; k += blockDim.x) {
      skv[k] = skv[static_cast<long>(ratio) * width + k];
      ssc[k] = ssc[static_cast<long>(ratio) * width + k];
    }
  }
}

// rows [n, D] (pitch floats apart) to n unrelated destinations.  grid n, block 128.
__global__ void scatter_rows_kernel(const float* __restrict__ rows, long pitch, float* const* __restrict__ dst, int D) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const float* src = rows + blockIdx.x * pitch;
  float* d = dst[blockIdx.x];
  for (int c = threadIdx.x; c < D; c += blockDim.x) d[c] = src[c];
}

// grid n_blocks (of 256 values), block 256
__global__ void q8k_roundtrip_kernel(const float* __restrict__ x, float* __restrict__ y) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ float red[32];
  const long i = static_cast<long>(blockIdx.x) * 256 + threadIdx.x;
  const float v = x[i];
  const float am = block_max(fabsf(v), red);
  // the signed value of the first element whose magnitude is the maximum
  __shared__ int first;
  if (threadIdx.x == 0) first = 256;
  __syncthreads();
  if (fabsf(v) == am) atomicMin(&first, static_cast<int>(threadIdx.x));
  __syncthreads();
  const float smax = x[static_cast<long>(blockIdx.x) * 256 + first];
  if (am == 0.f) { y[i] = 0.f; return; }
  const float iscale = -127.f / smax;
  const float q = fminf(fmaxf(rintf(v * iscale), -128.f), 127.f);
  y[i] = q * (1.f / iscale);
}

}  // namespace

#define FI_STREAM(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int fi_dsv4_hc_pre(const float* streams, const float* raw, const float* base, const float* scale, int T,
                              int hc, int H, float eps, int iters, float* mixed, float* post, float* combine,
                              void* stream) {
  if (T <= 0) return 0;
  if (hc <= 0 || hc > kMaxHc || H <= 0) return -10;
  fi::launch_kernel(hc_pre_kernel, dim3(T), dim3(256), 0, FI_STREAM(stream), 0, streams, raw, base, scale, hc, H, eps,
                    iters, mixed, post, combine);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_hc_post(const float* out, const float* streams, const float* post, const float* combine, int T,
                               int hc, int H, float* next, void* stream) {
  if (T <= 0) return 0;
  if (hc <= 0 || hc > kMaxHc || H <= 0) return -10;
  fi::launch_kernel(hc_post_kernel, dim3(T, (H + 255) / 256), dim3(256), 0, FI_STREAM(stream), 0, out, streams, post,
                    combine, hc, H, next);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_hc_collapse(const float* streams, const float* raw, const float* base, const float* scale,
                                   int T, int hc, int H, float eps, float* out, void* stream) {
  if (T <= 0) return 0;
  if (hc <= 0 || hc > kMaxHc || H <= 0) return -10;
  fi::launch_kernel(hc_collapse_kernel, dim3(T), dim3(256), 0, FI_STREAM(stream), 0, streams, raw, base, scale, hc, H,
                    eps, out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_norm_rope(const float* x, const float* w, const float* inv_freq, const long* pos, int rows,
                                 int rows_per_pos, int D, int rot, int do_norm, int inverse, int fp8, float eps,
                                 float* y, void* stream) {
  if (rows <= 0) return 0;
  if (D <= 0 || D > 12288 || rot < 0 || rot > D || (rot & 1) || rows_per_pos <= 0) return -10;
  if (rot > 0 && (inv_freq == nullptr || pos == nullptr)) return -10;
  if (fp8 && ((D - rot) % 64) != 0) return -10;
  fi::launch_kernel(norm_rope_kernel, dim3(rows), dim3(128), static_cast<size_t>(D) * sizeof(float), FI_STREAM(stream), 0,
                    x, w, inv_freq, pos, rows_per_pos, D, rot, do_norm, inverse, fp8, eps, y);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_compressor_step(float* state_kv, float* state_score, const float* kv_cur, const float* score_cur,
                                       const float* ape, long ape_stride_pos, long ape_stride_c, int pos, int ratio,
                                       int head_dim, float* emitted, void* stream) {
  if (ratio <= 0 || head_dim <= 0 || pos < 0) return -10;
  fi::launch_kernel(compressor_step_kernel, dim3(1), dim3(256), 0, FI_STREAM(stream), 0, state_kv, state_score, kv_cur,
                    score_cur, ape, ape_stride_pos, ape_stride_c, pos, ratio, head_dim, emitted);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_compressor_step_batch(void* state_kv, void* state_score, const float* kv_cur,
                                             const float* score_cur, long pitch, const float* ape, long ape_stride_pos,
                                             long ape_stride_c, const long* pos, int n, int ratio, int head_dim,
                                             float* emitted, void* stream) {
  if (n <= 0) return 0;
  if (ratio <= 0 || head_dim <= 0) return -10;
  fi::launch_kernel(compressor_step_batch_kernel, dim3(n), dim3(256), 0, FI_STREAM(stream), 0,
                    static_cast<float* const*>(state_kv), static_cast<float* const*>(state_score), kv_cur, score_cur, pitch,
                    ape, ape_stride_pos, ape_stride_c, pos, ratio, head_dim, emitted);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_scatter_rows(const float* rows, long pitch, void* dst, int n, int D, void* stream) {
  if (n <= 0 || D <= 0) return 0;
  fi::launch_kernel(scatter_rows_kernel, dim3(n), dim3(128), 0, FI_STREAM(stream), 0, rows, pitch,
                    static_cast<float* const*>(dst), D);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fi_dsv4_q8k_roundtrip(const float* x, float* y, long n, void* stream) {
  if (n <= 0) return 0;
  if (n % 256 != 0) return -10;
  fi::launch_kernel(q8k_roundtrip_kernel, dim3(static_cast<unsigned>(n / 256)), dim3(256), 0, FI_STREAM(stream), 0, x, y);
  return static_cast<int>(cudaGetLastError());
}
