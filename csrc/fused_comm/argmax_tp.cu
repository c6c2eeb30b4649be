// Vocabulary-parallel greedy arg-max: every rank holds the logits of its slice of the vocabulary
// ([rows, V_local] fp32); the winning token of every row is agreed on inside ONE kernel.
//
// One CTA per row: block arg-max over the local slice (ties -> lowest index), then thread 0 stores
// (value, epoch, global index, epoch) as one 16-byte word into every peer's slot for (source rank,
// row) over NVLink, polls its own slots of all ranks (bounded wait) and picks the best pair, ties to
// the lowest global index, so every rank writes the same token id.  This replaces an all-gather of
// [rows, V] logits (NCCL launch + 4 * rows * V bytes) plus a full-vocabulary scan on every rank by
// 16 * rows bytes per peer.  The reference samples from full logits on one GPU
// (vllm/engine/sampling/sampler.py:18-40); it has no vocabulary-parallel form.
//
// Bookkeeping is shared with the fused GEMM collectives: the call's epoch is `*epoch + 1`, the last
// CTA publishes it, slots are double-buffered by epoch parity.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../common/launch.cuh"
#include "../common/ptx.cuh"
#include "../gemm/comm_desc.h"

namespace {

struct ArgmaxComm {
  int world, rank, phases, rows_cap;
  unsigned long long recv[8];   // slot area of rank d as mapped here: uint4 [2 parities][world][rows_cap]
  unsigned int* epoch;
  unsigned int* done;
  int* status;
};

__global__ void __launch_bounds__(1024)
argmax_tp_kernel(const float* __restrict__ logits, long ld, int V, int vocab_offset, long* __restrict__ out,
                 const ArgmaxComm c) {
  fi::pdl_launch_dependents();
  fi::pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const int row_idx = blockIdx.x;
  const float* row = logits + static_cast<long>(row_idx) * ld;
  const unsigned int epoch_now = *c.epoch + 1u;
  const int phases = c.phases != 0 ? c.phases : 3;
  float best = -CUDART_INF_F;
  int bi = 0x7fffffff;
  if ((V & 3) == 0 && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int n4 = V >> 2;
    for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * blockDim.x;
        v[u] = i < n4 ? row4[i] : make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
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
      const float f = row[i];
      if (f > best || (f == best && i < bi)) { best = f; bi = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    best = l < nw ? sv[l] : -CUDART_INF_F;
    bi = l < nw ? si[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    // lanes 0..world-1: lane d delivers to rank d (phase 1) and later reads the slot of source rank d (phase 2)
    const long parity = epoch_now & 1u;
    const int gi = (bi == 0x7fffffff ? 0 : bi) + vocab_offset;
    const uint4 mine = make_uint4(__float_as_uint(best), epoch_now, static_cast<unsigned int>(gi), epoch_now);
    if (l < c.world && (phases & 1)) {
      uint4* dst = reinterpret_cast<uint4*>(c.recv[l]) + (parity * c.world + c.rank) * c.rows_cap + row_idx;
      fi::st_volatile_v4(dst, mine);
    }
    if (phases & 2) {
      float v = -CUDART_INF_F;
      int idx = 0x7fffffff;
      bool ok = true;
      if (l < c.world) {
        const uint4* src = reinterpret_cast<const uint4*>(c.recv[c.rank]) + (parity * c.world + l) * c.rows_cap + row_idx;
        uint4 wv = fi::ld_volatile_v4(src);
        const long long t0 = clock64();
        while (wv.y != epoch_now || wv.w != epoch_now) {
          if (clock64() - t0 > FI_WAIT_CYCLES ||
              (c.status != nullptr && clock64() - t0 > (FI_WAIT_CYCLES >> 10) &&
               *reinterpret_cast<const volatile int*>(c.status) != 0)) {
            fi::set_status(c.status, fi::kStatusTimeoutPeer);
            ok = false;
            break;
          }
          wv = fi::ld_volatile_v4(src);
        }
        if (ok) { v = __uint_as_float(wv.x); idx = static_cast<int>(wv.z); }
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {   // world <= 8
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
      }
      const bool all_ok = __all_sync(0xffffffffu, ok);
      if (l == 0 && all_ok) out[row_idx] = idx == 0x7fffffff ? 0 : idx;
    }
  }
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

// logits: this rank's [rows, V_local] fp32 slice (row stride ld); vocab_offset: global index of its first
// column; out: [rows] int64 token ids, identical on every rank.  comm->recv[d] must point at rank d's
// arg-max slot area (uint4 [2][world][rows_cap]); rows_cap is passed in comm->rows_per_rank.
extern "C" int fi_argmax_tp(const float* logits, long ld, int rows, int V, int vocab_offset, long* out,
                            int* status, void* stream, const FiComm* comm) {
  if (rows <= 0) return 0;
  if (comm == nullptr || comm->world < 1 || comm->world > 8 || V <= 0) return -10;
  if (rows > comm->rows_per_rank) return -11;
  ArgmaxComm c;
  c.world = comm->world; c.rank = comm->rank; c.phases = comm->phases; c.rows_cap = comm->rows_per_rank;
  for (int d = 0; d < 8; ++d) c.recv[d] = comm->recv[d];
  c.epoch = reinterpret_cast<unsigned int*>(comm->epoch);
  c.done = reinterpret_cast<unsigned int*>(comm->done);
  c.status = status;
  fi::launch_kernel(argmax_tp_kernel, dim3(rows), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream), 0, logits, ld,
                    V, vocab_offset, out, c);
  return static_cast<int>(cudaGetLastError());
}
