// Gated delta rule, one decode step for a batch of sequences (Qwen3.5 / Qwen3-Next linear attention):
//
//   S <- exp(g) * S;   delta = beta * (v - S^T k);   S <- S + k (x) delta;   o = S^T q
//
// per (sequence, value head) with the recurrent state S [dk, dv] in fp32, kept in a pool indexed by
// the sequence's slot so that nothing is gathered or scattered on the host.  One CTA per (sequence,
// head); thread j owns column j of S: it streams the column through registers once (one read and one
// write of the state per step: the op is bound by those 2 * dk * dv * 4 bytes), accumulating S^T k on
// the way in and S^T q on the way out.  Reads and writes of a row are coalesced across threads.
// The causal depthwise convolution in front of it (kernel width kw, SiLU) has its own step kernel with
// the last kw - 1 inputs per channel in a second pool.
//
// Reference: vllm/model_executor/models/qwen3_5.py:127-200 (chunked rule for prefill, recurrent rule
// for decode, both in PyTorch; optional `fla` Triton kernels).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/launch.cuh"

namespace {

constexpr int kMaxDk = 256;

template <int DK_CHUNK>
__global__ void gdn_step_kernel(float* __restrict__ pool, const int* __restrict__ slots, const float* __restrict__ q,
                                const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ g,
                                const float* __restrict__ beta, float* __restrict__ out, int nv, int dk, int dv) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int b = blockIdx.y, h = blockIdx.x;
  const int slot = slots[b];
  if (slot < 0) return;
  __shared__ float sk[kMaxDk], sq[kMaxDk];
  const long row = static_cast<long>(b) * nv + h;
  for (int i = threadIdx.x; i < dk; i += blockDim.x) {
    sk[i] = k[row * dk + i];
    sq[i] = q[row * dk + i];
  }
  __syncthreads();
  const float decay = __expf(g[row]);
  const float bt = beta[row];
  float* S = pool + (static_cast<long>(slot) * nv + h) * dk * dv;
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    // pass 1: decay the column, keep it in registers chunk by chunk is not possible for every dk, so the
    // column is read twice from L1/L2 (the second read hits the lines the first one brought in)
    float mem = 0.f;
    for (int i = 0; i < dk; ++i) mem += S[static_cast<long>(i) * dv + j] * sk[i];
    const float delta = (v[row * dv + j] - decay * mem) * bt;
    float o = 0.f;
    for (int i = 0; i < dk; ++i) {
      const float s = S[static_cast<long>(i) * dv + j] * decay + sk[i] * delta;
      S[static_cast<long>(i) * dv + j] = s;
      o += s * sq[i];
    }
    out[row * dv + j] = o;
  }
}

// x [B, C] new inputs (16-bit), conv pool [slots, C, kw-1] (same type), w [C, kw]; y [B, C] fp32 =
// SiLU(sum_j w[c, j] * window[c, j]) with window = (state, x); the state shifts by one.
template <typename T>
__global__ void conv_step_kernel(const T* __restrict__ x, long ldx, T* __restrict__ pool, const int* __restrict__ slots,
                                 const T* __restrict__ w, float* __restrict__ y, int C, int kw) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  const int b = blockIdx.y;
  const int slot = slots[b];
  if (slot < 0) return;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < C; c += gridDim.x * blockDim.x) {
    T* st = pool + (static_cast<long>(slot) * C + c) * (kw - 1);
    const float xn = static_cast<float>(x[b * ldx + c]);
    float acc = static_cast<float>(w[c * kw + kw - 1]) * xn;
    for (int j = 0; j < kw - 1; ++j) acc += static_cast<float>(w[c * kw + j]) * static_cast<float>(st[j]);
    for (int j = 0; j + 1 < kw - 1; ++j) st[j] = st[j + 1];
    st[kw - 2] = x[b * ldx + c];
    y[static_cast<long>(b) * C + c] = acc / (1.f + __expf(-acc));
  }
}

}  // namespace

// pool: fp32 [num_slots, nv, dk, dv]; slots: int32 [B] (negative = skip the row); q, k: fp32 [B, nv, dk]
// (already normalised / scaled / repeated per value head); v: fp32 [B, nv, dv]; g, beta: fp32 [B, nv];
// out: fp32 [B, nv, dv].
extern "C" int fi_gdn_step(float* pool, const int* slots, const float* q, const float* k, const float* v,
                           const float* g, const float* beta, float* out, int B, int nv, int dk, int dv, void* stream) {
  if (B <= 0) return 0;
  if (dk > kMaxDk || dk <= 0 || dv <= 0 || nv <= 0) return -10;
  const int threads = dv >= 128 ? 128 : (dv >= 64 ? 64 : 32);
  fi::launch_kernel(gdn_step_kernel<0>, dim3(nv, B), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream), 0, pool,
                    slots, q, k, v, g, beta, out, nv, dk, dv);
  return static_cast<int>(cudaGetLastError());
}

// dtype: 0 bf16, 1 fp16 (x, pool, w).
extern "C" int fi_conv1d_step(const void* x, long ldx, void* pool, const int* slots, const void* w, float* y, int B,
                              int C, int kw, int dtype, void* stream) {
  if (B <= 0) return 0;
  if (kw < 2 || kw > 8 || C <= 0) return -10;
  const dim3 grid((C + 255) / 256, B);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 0)
    fi::launch_kernel(conv_step_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, 0, (const __nv_bfloat16*)x, ldx,
                      (__nv_bfloat16*)pool, slots, (const __nv_bfloat16*)w, y, C, kw);
  else if (dtype == 1)
    fi::launch_kernel(conv_step_kernel<__half>, grid, dim3(256), 0, s, 0, (const __half*)x, ldx, (__half*)pool, slots,
                      (const __half*)w, y, C, kw);
  else
    return -11;
  return static_cast<int>(cudaGetLastError());
}
