// Decode attention over the static KV cache: one new query token per sequence.
//
// The reference runs masked SDPA over the whole cache allocation every step
// (models/model.py:121-129, 343-344); this kernel reads only the live range
// [left_pad[b], pos] of each row, which is what makes batched decode HBM-bound on the
// useful bytes only. It is a pure streaming kernel (every K/V byte is used once per q head),
// so it runs on the CUDA cores with 16-byte loads; grouped-query attention reuses each K/V
// row for the G query heads that share it.
//
// Layouts: q [B, n_head*D] bf16, caches [max_batch, n_kv, smax, D] bf16, out [B, n_head*D] bf16.
// Grid: (n_kv * B, n_split). Each CTA has 4 warps; a half-warp (16 lanes x 8 elements) owns
// one key row at a time. With n_split > 1 the CTA writes (m, l, acc) partials; they are merged
// either by the last CTA of each (sequence, kv head) to arrive (a ticket counter per pair, no
// extra launch) or, when no ticket array is given, by a second kernel.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <float.h>
#include <stdint.h>

#include "launch.cuh"
#include "ptx.cuh"

namespace e2h {

constexpr int kWarps = 4;
constexpr int kSlots = kWarps * 2;  // half-warps per CTA
constexpr int kKeysPerIter = 4;     // independent 16-byte loads in flight per lane

__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __bfloat162float(h[i].x);
    f[2 * i + 1] = __bfloat162float(h[i].y);
  }
}

// D = 16 * 8 * R : each lane of the half-warp holds R groups of 8 consecutive elements.
template <int D, int G>
__global__ void __launch_bounds__(kWarps * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
                   const __nv_bfloat16* __restrict__ vcache, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ partial, const int* __restrict__ pos_ptr,
                   const int* __restrict__ left_pad, int n_head, int n_kv, int smax, float scale,
                   int n_split, unsigned int* __restrict__ tickets) {
  constexpr int R = D / 128 > 0 ? D / 128 : 1;       // 8-element groups per lane (D=128 -> 1)
  constexpr int LPK = D >= 128 ? 16 : D / 8;          // lanes per key row
  static_assert(D == 64 || D == 128 || D == 256, "head_dim must be 64, 128 or 256");
  const int b = blockIdx.x / n_kv;
  const int hk = blockIdx.x - b * n_kv;
  const int split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = lane / 16;            // which key of the pair this half-warp handles
  const int hl = lane & 15;
  const bool lane_active = hl < LPK;
  const int slot = warp * 2 + half;

  pdl_launch_dependents();   // the successor may start its prologue / weight prefetch already
  pdl_wait_prior();
  int pos = *pos_ptr;                    // index of the newest token (already in the cache)
  // positions come from device memory: keep every cache row that is read inside the allocation
  if (pos >= smax) pos = smax - 1;
  if (pos < 0) pos = 0;
  int start = left_pad ? left_pad[b] : 0;
  if (start > pos) start = pos;
  if (start < 0) start = 0;
  // keys of this split
  const int total = pos - start + 1;
  const int per = (total + n_split - 1) / n_split;
  const int k_begin = start + split * per;
  const int k_end = min(pos + 1, k_begin + per);

  float qv[G][R][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const int h = hk * G + g;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (lane_active) {
        const uint4 raw = *reinterpret_cast<const uint4*>(
            q + ((long long)b * n_head + h) * D + (r * LPK + hl) * 8);
        unpack8(raw, qv[g][r]);
#pragma unroll
        for (int i = 0; i < 8; ++i) qv[g][r][i] *= scale;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) qv[g][r][i] = 0.f;
      }
    }
  }
  float m[G], l[G], acc[G][R][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -FLT_MAX;
    l[g] = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][r][i] = 0.f;
  }

  const __nv_bfloat16* kbase = kcache + ((long long)b * n_kv + hk) * smax * D;
  const __nv_bfloat16* vbase = vcache + ((long long)b * n_kv + hk) * smax * D;

  for (int j0 = k_begin; j0 < k_end; j0 += kSlots * kKeysPerIter) {
    uint4 kr[kKeysPerIter][R], vr[kKeysPerIter][R];
#pragma unroll
    for (int u = 0; u < kKeysPerIter; ++u) {
      const int j = j0 + u * kSlots + slot;
      const bool ok = j < k_end && lane_active;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const long long o = (long long)j * D + (r * LPK + hl) * 8;
        kr[u][r] = ok ? __ldg(reinterpret_cast<const uint4*>(kbase + o)) : make_uint4(0, 0, 0, 0);
        vr[u][r] = ok ? __ldg(reinterpret_cast<const uint4*>(vbase + o)) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < kKeysPerIter; ++u) {
      const int j = j0 + u * kSlots + slot;
      const bool ok = j < k_end;
      float kf[R][8], vf[R][8];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        unpack8(kr[u][r], kf[r]);
        unpack8(vr[u][r], vf[r]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int i = 0; i < 8; ++i) s += qv[g][r][i] * kf[r][i];
        // reduce over the 16 lanes of the half-warp
        s += __shfl_xor_sync(0xffffffffu, s, 8);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        if (ok) {
          const float mn = fmaxf(m[g], s);
          const float corr = __expf(m[g] - mn);
          const float pj = __expf(s - mn);
          l[g] = l[g] * corr + pj;
#pragma unroll
          for (int r = 0; r < R; ++r)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[g][r][i] = acc[g][r][i] * corr + pj * vf[r][i];
          m[g] = mn;
        }
      }
    }
  }

  // merge the 8 half-warp partials of the CTA through shared memory
  __shared__ float sm_m[kSlots][G], sm_l[kSlots][G];
  __shared__ float sm_acc[kSlots][G][D];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (hl == 0) {
      sm_m[slot][g] = m[g];
      sm_l[slot][g] = l[g];
    }
    if (lane_active) {
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 8; ++i) sm_acc[slot][g][(r * LPK + hl) * 8 + i] = acc[g][r][i];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    float mm = -FLT_MAX;
#pragma unroll
    for (int s = 0; s < kSlots; ++s) mm = fmaxf(mm, sm_m[s][g]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
      const float w = (sm_m[s][g] == -FLT_MAX) ? 0.f : __expf(sm_m[s][g] - mm);
      ll += sm_l[s][g] * w;
      a += sm_acc[s][g][d] * w;
    }
    const int h = hk * G + g;
    if (n_split == 1) {
      out[((long long)b * n_head + h) * D + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
    } else {
      float* pp = partial + (((long long)b * n_head + h) * n_split + split) * (D + 2);
      pp[d] = a;
      if (d == 0) {
        pp[D] = mm;
        pp[D + 1] = ll;
      }
    }
  }
  if (n_split == 1 || tickets == nullptr) return;
  // merge in place of a second launch: the last split of this (sequence, kv head) to finish
  // combines all of them (the ticket word returns to zero for the next launch)
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(&tickets[blockIdx.x], 1u);
    is_last = (t == (unsigned int)n_split - 1) ? 1 : 0;
    if (is_last) tickets[blockIdx.x] = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx - g * D;
    const int h = hk * G + g;
    const float* pp = partial + ((long long)b * n_head + h) * n_split * (D + 2);
    float mm = -FLT_MAX;
    for (int s = 0; s < n_split; ++s) mm = fmaxf(mm, __ldcg(pp + s * (D + 2) + D));
    float ll = 0.f, a = 0.f;
    for (int s = 0; s < n_split; ++s) {
      const float ms = __ldcg(pp + s * (D + 2) + D);
      const float w = (ms == -FLT_MAX) ? 0.f : __expf(ms - mm);
      ll += __ldcg(pp + s * (D + 2) + D + 1) * w;
      a += __ldcg(pp + s * (D + 2) + d) * w;
    }
    out[((long long)b * n_head + h) * D + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
  }
}

template <int D>
__global__ void attn_decode_merge_kernel(const float* __restrict__ partial,
                                         __nv_bfloat16* __restrict__ out, int n_split) {
  const long long bh = blockIdx.x;
  pdl_launch_dependents();   // the successor may start its prologue / weight prefetch already
  pdl_wait_prior();
  const float* pp = partial + bh * n_split * (D + 2);
  float mm = -FLT_MAX;
  for (int s = 0; s < n_split; ++s) mm = fmaxf(mm, pp[s * (D + 2) + D]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float ll = 0.f, a = 0.f;
    for (int s = 0; s < n_split; ++s) {
      const float ms = pp[s * (D + 2) + D];
      const float w = (ms == -FLT_MAX) ? 0.f : __expf(ms - mm);
      ll += pp[s * (D + 2) + D + 1] * w;
      a += pp[s * (D + 2) + d] * w;
    }
    out[bh * D + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
  }
}

template <int D, int G>
static int launch_decode(const void* q, const void* k, const void* v, void* out, float* partial,
                         const int* pos, const int* left_pad, int B, int n_head, int n_kv, int smax,
                         float scale, int n_split, cudaStream_t stream,
                         unsigned int* tickets = nullptr) {
  dim3 grid(n_kv * B, n_split);
  cudaError_t e = launch(attn_decode_kernel<D, G>, grid, dim3(kWarps * 32), 0, stream,
                         (const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
                         (const __nv_bfloat16*)v, (__nv_bfloat16*)out, partial, pos, left_pad,
                         n_head, n_kv, smax, scale, n_split, tickets);
  if (e == cudaSuccess && n_split > 1 && tickets == nullptr)
    e = launch(attn_decode_merge_kernel<D>, dim3(B * n_head), dim3(128), 0, stream,
               (const float*)partial, (__nv_bfloat16*)out, n_split);
  return (int)e;
}

}  // namespace e2h

// partial: fp32 scratch of B*n_head*n_split*(D+2) floats, needed only when n_split > 1.
// tickets: optional uint32 [B*n_kv], zero before the first launch (every launch leaves it zero):
// with it the splits are merged inside the kernel, without it by a second launch.
extern "C" int e2h_attn_decode(const void* q, const void* kcache, const void* vcache, void* out,
                               float* partial, const int* pos, const int* left_pad, int B,
                               int n_head, int n_kv, int head_dim, int smax, float scale,
                               int n_split, unsigned int* tickets, void* stream_v) {
  using namespace e2h;
  cudaStream_t stream = (cudaStream_t)stream_v;
  if (n_head % n_kv) return -1;
  if (n_split > 1 && partial == nullptr) return -2;
  const int G = n_head / n_kv;
#define E2H_GO(D_, G_)                                                                          \
  return launch_decode<D_, G_>(q, kcache, vcache, out, partial, pos, left_pad, B, n_head, n_kv, \
                               smax, scale, n_split, stream, tickets)
  if (head_dim == 128) {
    if (G == 1) E2H_GO(128, 1);
    if (G == 4) E2H_GO(128, 4);
    if (G == 8) E2H_GO(128, 8);
  } else if (head_dim == 64) {
    if (G == 1) E2H_GO(64, 1);
    if (G == 4) E2H_GO(64, 4);
  }
#undef E2H_GO
  return -3;  // unsupported (head_dim, group) pair: callers fall back to per-head launches
}

// ---------------------------------------------------------------------------------------------
// Non-allocating variant (declared in attn_decode_static.h). The split-KV partial results go to
// a fixed array in device memory instead of a caller-provided buffer, so the call allocates
// nothing and needs nothing allocated for it.
#include <cstdio>
#include <mutex>

#include "attn_decode_static.h"

namespace e2h {
// room for 64 sequences x 32 heads x 8 splits x (128 + 2) floats = 8.125 MiB
constexpr long long kStaticPartialFloats = 64LL * 32 * 8 * (128 + 2);
static __device__ __align__(256) float g_static_partial[kStaticPartialFloats];

constexpr int kMaxDevices = 64;
static float* g_static_partial_ptr[kMaxDevices];   // per device, filled on that device's first call
static std::mutex g_static_partial_mu;

static int static_partial_for_current_device(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return -5;
  std::lock_guard<std::mutex> lock(g_static_partial_mu);
  if (g_static_partial_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_partial);
    if (e != cudaSuccess) {
      fprintf(stderr, "e2h_attn_decode_static: cudaGetSymbolAddress failed: %s\n",
              cudaGetErrorString(e));
      return (int)e;
    }
    g_static_partial_ptr[dev] = p;
  }
  *ptr = g_static_partial_ptr[dev];
  return 0;
}
}  // namespace e2h

extern "C" int e2h_attn_decode_static(const void* q, const void* kcache, const void* vcache,
                                      void* out, const int* pos, const int* left_pad, int B,
                                      int n_head, int n_kv, int head_dim, int smax, float scale,
                                      int n_split, void* stream_v) {
  using namespace e2h;
  if (B < 1 || n_head < 1 || n_kv < 1 || n_split < 1 || n_head % n_kv) return -1;
  const long long need = (long long)B * n_head * n_split * (head_dim + 2);
  if (n_split > 1 && need > kStaticPartialFloats) {
    fprintf(stderr,
            "e2h_attn_decode_static: B*n_head*n_split*(head_dim+2) = %lld floats exceeds the "
            "fixed scratch of %lld floats (64 x 32 heads x 8 splits x head_dim 128); use fewer "
            "splits or e2h_attn_decode with a caller-provided buffer\n",
            need, kStaticPartialFloats);
    return -4;
  }
  float* partial = nullptr;
  if (n_split > 1) {
    const int rc = static_partial_for_current_device(&partial);
    if (rc != 0) return rc;
  }
  cudaStream_t stream = (cudaStream_t)stream_v;
  const int G = n_head / n_kv;
#define E2H_GO(D_, G_)                                                                          \
  return launch_decode<D_, G_>(q, kcache, vcache, out, partial, pos, left_pad, B, n_head, n_kv, \
                               smax, scale, n_split, stream)
  if (head_dim == 128) {
    if (G == 1) E2H_GO(128, 1);
    if (G == 4) E2H_GO(128, 4);
    if (G == 8) E2H_GO(128, 8);
  } else if (head_dim == 64) {
    if (G == 1) E2H_GO(64, 1);
    if (G == 4) E2H_GO(64, 4);
  }
#undef E2H_GO
  return -3;
}
