// 16-byte-vectorised forms of the row-wise and element-wise kernels for the large-token
// (training / prefill / scoring) shapes, where these ops are pure HBM streams: every thread
// moves 8 bf16 per load / store and a row of up to 8192 features lives in registers between
// the reduction and the write, so each byte is touched once.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace e2h {

struct alignas(16) BF8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const BF8& b, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __bfloat162float(b.v[i].x);
    f[2 * i + 1] = __bfloat162float(b.v[i].y);
  }
}
__device__ __forceinline__ BF8 pack8(const float* f) {
  BF8 b;
#pragma unroll
  for (int i = 0; i < 4; ++i) b.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return b;
}

// sum over the block of two values at once; red must hold 64 floats
__device__ __forceinline__ float2 block_sum2(float a, float b, float* red) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) {
    red[warp] = a;
    red[32 + warp] = b;
  }
  __syncthreads();
  a = lane < nw ? red[lane] : 0.f;
  b = lane < nw ? red[32 + lane] : 0.f;
  a = warp_sum(a);
  b = warp_sum(b);
  return make_float2(a, b);
}

// x_out[t] = bf16(bf16(x[t] * rstd) * w), one block per row, NV 16-byte vectors per thread.
template <int NV>
__global__ void rmsnorm_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                    const __nv_bfloat16* __restrict__ weight,
                                    __nv_bfloat16* __restrict__ out, float* __restrict__ rstd_out,
                                    int dim, float eps) {
  __shared__ float red[64];
  const long long base = (long long)blockIdx.x * dim;
  const int nvec = dim >> 3;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      unpack8(*reinterpret_cast<const BF8*>(x + base + 8 * i), v[k]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[k][e] * v[k][e];
    }
  }
  ss = block_sum2(ss, 0.f, red).x;
  const float rstd = rsqrtf(ss / dim + eps);
  if (rstd_out && threadIdx.x == 0) rstd_out[blockIdx.x] = rstd;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      float w[8], o[8];
      unpack8(*reinterpret_cast<const BF8*>(weight + 8 * i), w);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = bf16_round(v[k][e] * rstd) * w[e];
      *reinterpret_cast<BF8*>(out + base + 8 * i) = pack8(o);
    }
  }
}

// dx = rstd * (dy*w) - x * rstd^3 / dim * sum(dy*w*x) (+ dres)
template <int NV>
__global__ void rmsnorm_bwd_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                        const __nv_bfloat16* __restrict__ dy,
                                        const __nv_bfloat16* __restrict__ weight,
                                        const __nv_bfloat16* __restrict__ dres,
                                        __nv_bfloat16* __restrict__ dx, int dim, float eps) {
  __shared__ float red[64];
  const long long base = (long long)blockIdx.x * dim;
  const int nvec = dim >> 3;
  float xv[NV][8], g[NV][8];
  float ss = 0.f, dot = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      float w[8];
      unpack8(*reinterpret_cast<const BF8*>(x + base + 8 * i), xv[k]);
      unpack8(*reinterpret_cast<const BF8*>(dy + base + 8 * i), g[k]);
      unpack8(*reinterpret_cast<const BF8*>(weight + 8 * i), w);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        g[k][e] *= w[e];
        ss += xv[k][e] * xv[k][e];
        dot += xv[k][e] * g[k][e];
      }
    }
  }
  const float2 s = block_sum2(ss, dot, red);
  const float rstd = rsqrtf(s.x / dim + eps);
  const float coef = s.y * rstd * rstd * rstd / dim;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = g[k][e] * rstd - xv[k][e] * coef;
      if (dres) {
        float r[8];
        unpack8(*reinterpret_cast<const BF8*>(dres + base + 8 * i), r);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += r[e];
      }
      *reinterpret_cast<BF8*>(dx + base + 8 * i) = pack8(o);
    }
  }
}

__global__ void swiglu_fwd_vec_kernel(const __nv_bfloat16* __restrict__ g,
                                      const __nv_bfloat16* __restrict__ u,
                                      __nv_bfloat16* __restrict__ out, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8], b[8], o[8];
    unpack8(reinterpret_cast<const BF8*>(g)[i], a);
    unpack8(reinterpret_cast<const BF8*>(u)[i], b);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = bf16_round(silu(a[e])) * b[e];
    reinterpret_cast<BF8*>(out)[i] = pack8(o);
  }
}

__global__ void swiglu_bwd_vec_kernel(const __nv_bfloat16* __restrict__ g,
                                      const __nv_bfloat16* __restrict__ u,
                                      const __nv_bfloat16* __restrict__ dact,
                                      __nv_bfloat16* __restrict__ dg,
                                      __nv_bfloat16* __restrict__ du, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8], b[8], d[8], og[8], ou[8];
    unpack8(reinterpret_cast<const BF8*>(g)[i], a);
    unpack8(reinterpret_cast<const BF8*>(u)[i], b);
    unpack8(reinterpret_cast<const BF8*>(dact)[i], d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sig = 1.f / (1.f + __expf(-a[e]));
      og[e] = d[e] * b[e] * (sig * (1.f + a[e] * (1.f - sig)));
      ou[e] = d[e] * (a[e] * sig);
    }
    reinterpret_cast<BF8*>(dg)[i] = pack8(og);
    reinterpret_cast<BF8*>(du)[i] = pack8(ou);
  }
}

// Interleaved-pair RoPE, 4 pairs per thread. x rows are `ld` elements apart; only the first
// n_heads * head_dim elements of a row are rotated.
__global__ void rope_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                const __nv_bfloat16* __restrict__ freqs,
                                const int* __restrict__ pos, int n_heads, int head_dim,
                                long long ld, int inverse) {
  const int t = blockIdx.x;
  const int vec_per_head = head_dim >> 3;
  const int p = pos[t];
  const __nv_bfloat16* fr = freqs + (long long)p * head_dim;     // [head_dim/2][2]
  for (int i = threadIdx.x; i < n_heads * vec_per_head; i += blockDim.x) {
    const int h = i / vec_per_head, j = i - h * vec_per_head;
    const long long o = (long long)t * ld + (long long)h * head_dim + 8 * j;
    float v[8], cs[8], r[8];
    unpack8(*reinterpret_cast<const BF8*>(x + o), v);
    unpack8(*reinterpret_cast<const BF8*>(fr + 8 * j), cs);      // (cos, sin) x 4 pairs
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float c = cs[2 * e], s = inverse ? -cs[2 * e + 1] : cs[2 * e + 1];
      r[2 * e] = v[2 * e] * c - v[2 * e + 1] * s;
      r[2 * e + 1] = v[2 * e + 1] * c + v[2 * e] * s;
    }
    *reinterpret_cast<BF8*>(out + o) = pack8(r);
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace e2h
