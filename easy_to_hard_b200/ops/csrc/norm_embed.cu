// RMSNorm (forward, with the residual / partial-sum reduction of a row-parallel linear folded
// in), RMSNorm backward, embedding gather, and the small element-wise kernels of the model
// (SwiGLU forward/backward, stand-alone RoPE forward/backward).
//
// Numerics follow the reference model (models/model.py:370-377, 400-412): statistics in fp32,
// the normalised value rounded to bf16 before the multiplication with the bf16 weight.
#include <cuda_runtime.h>
#include <stdlib.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "launch.cuh"
#include "ptx.cuh"

namespace e2h {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

struct PartPtrs {
  const float* p[8];   // one fp32 [T, dim] partial per split / tensor-parallel rank
};

// One CTA per token row.
//   h_in      : bf16 [T, dim]  residual stream (or nullptr when `tokens` is given)
//   tokens    : int32 [T]      when set, the row is gathered from `emb` ([emb_rows, dim]) instead
//                              of h_in; ids outside the table give a zero row and status 106
//   parts     : n_part fp32 [T, dim] partial sums of a row-parallel linear (one per
//               tensor-parallel rank; the pointers may be peer-GPU addresses, read with
//               system-scope loads over NVLink); added to the row when n_part > 0
//   h_out     : bf16 [T, dim]  updated residual stream (written when non-null)
//   x_out     : bf16 [T, dim]  rmsnorm(h) * weight     (written when non-null)
//   flags     : optional int32 [n_part] in local memory; rank i bumps flags[i] by one when its
//               partial for this use is complete. The kernel waits (bounded) for
//               flags[i] >= *use_count + 1; the last CTA to finish bumps *use_count, so the
//               protocol needs no host-side epoch and replays inside a CUDA graph.
// Limit of the cross-rank flag wait, in SM cycles. The default (about a second) suits the decode
// loop, where the ranks run in lock step; training raises it (e2h_set_flag_wait_ms) because ranks
// may drift apart by data loading or first-use initialisation.
__device__ long long g_flag_wait_cycles = kWaitLimitCycles;

__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ h_in,
                                   const int* __restrict__ tokens,
                                   const __nv_bfloat16* __restrict__ emb, int emb_rows,
                                   const PartPtrs parts, int n_part,
                                   const __nv_bfloat16* __restrict__ weight,
                                   __nv_bfloat16* __restrict__ h_out,
                                   __nv_bfloat16* __restrict__ x_out, float* __restrict__ rstd_out,
                                   int dim, float eps, const int* flags, int* use_count,
                                   unsigned int* ticket, int* status) {
  extern __shared__ float row[];  // dim floats + 32
  float* red = row + dim;
  const int t = blockIdx.x;
  pdl_launch_dependents();   // the successor may start its prologue / weight prefetch already
  pdl_wait_prior();
  const __nv_bfloat16* src = h_in ? h_in + (long long)t * dim : nullptr;
  if (tokens) {
    // an id outside the table reads as a zero row and is reported, never dereferenced
    const int id = tokens[t];
    if (id >= 0 && id < emb_rows) {
      src = emb + (long long)id * dim;
    } else {
      src = nullptr;
      if (threadIdx.x == 0 && status) atomicCAS(status, 0, kStatusBadArgs);
    }
  }
  if (flags != nullptr) {
    const int want = *use_count + 1;
    if (threadIdx.x < n_part)
      wait_flag_ge(flags + threadIdx.x, want, status, g_flag_wait_cycles);
    __syncthreads();
  }
  float ss = 0.f;
  for (int i = threadIdx.x * 2; i < dim; i += blockDim.x * 2) {
    float a = 0.f, b = 0.f;
    if (src) {
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(src + i);
      a = __bfloat162float(v.x);
      b = __bfloat162float(v.y);
    }
    if (n_part > 0) {
      float pa = 0.f, pb = 0.f;
      for (int s = 0; s < n_part; ++s) {
        const float* src = parts.p[s] + (long long)t * dim + i;
        const float2 pv = flags ? ld_sys_f32x2(src) : *reinterpret_cast<const float2*>(src);
        pa += pv.x;
        pb += pv.y;
      }
      // the linear's output is a bf16 tensor in the reference; round before the residual add
      a = bf16_round(a + bf16_round(pa));
      b = bf16_round(b + bf16_round(pb));
    }
    row[i] = a;
    row[i + 1] = b;
    ss += a * a + b * b;
    if (h_out) {
      __nv_bfloat162 o;
      o.x = __float2bfloat16_rn(a);
      o.y = __float2bfloat16_rn(b);
      *reinterpret_cast<__nv_bfloat162*>(h_out + (long long)t * dim + i) = o;
    }
  }
  if (flags != nullptr) {
    // all reads of this use are done: the last CTA advances the use counter
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
        *ticket = 0;
        *use_count = *use_count + 1;
      }
    }
  }
  if (x_out == nullptr) return;
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / dim + eps);
  if (rstd_out && threadIdx.x == 0) rstd_out[t] = rstd;
  for (int i = threadIdx.x * 2; i < dim; i += blockDim.x * 2) {
    const __nv_bfloat162 w = *reinterpret_cast<const __nv_bfloat162*>(weight + i);
    __nv_bfloat162 o;
    o.x = __float2bfloat16_rn(bf16_round(row[i] * rstd) * __bfloat162float(w.x));
    o.y = __float2bfloat16_rn(bf16_round(row[i + 1] * rstd) * __bfloat162float(w.y));
    *reinterpret_cast<__nv_bfloat162*>(x_out + (long long)t * dim + i) = o;
  }
}

// RMSNorm backward for one row per CTA:  y = bf16(x * rstd) * w
//   dx = rstd * (dy*w) - x * rstd^3 / dim * sum(dy*w*x);   dres (optional) is added to dx.
// The weight is frozen in this framework (as in the reference's FrozenRMSNorm), so no dw.
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ dy,
                                   const __nv_bfloat16* __restrict__ weight,
                                   const __nv_bfloat16* __restrict__ dres,
                                   __nv_bfloat16* __restrict__ dx, int dim, float eps) {
  extern __shared__ float row[];
  float* red = row + 2 * dim;
  const long long base = (long long)blockIdx.x * dim;
  float ss = 0.f, dot = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float xv = __bfloat162float(x[base + i]);
    const float g = __bfloat162float(dy[base + i]) * __bfloat162float(weight[i]);
    row[i] = xv;
    row[dim + i] = g;
    ss += xv * xv;
    dot += xv * g;
  }
  ss = block_sum(ss, red);
  dot = block_sum(dot, red);
  const float rstd = rsqrtf(ss / dim + eps);
  const float coef = dot * rstd * rstd * rstd / dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = row[dim + i] * rstd - row[i] * coef;
    if (dres) v += __bfloat162float(dres[base + i]);
    dx[base + i] = __float2bfloat16_rn(v);
  }
}

// out[t, :] = table[tokens[t], :]
// (ids outside [0, rows) give a zero row and status 106)
__global__ void embedding_kernel(const int* __restrict__ tokens,
                                 const __nv_bfloat16* __restrict__ table, int rows,
                                 __nv_bfloat16* __restrict__ out, int dim, int* status) {
  const int t = blockIdx.x;
  const int id = tokens[t];
  const bool ok = id >= 0 && id < rows;
  if (!ok && threadIdx.x == 0 && status) atomicCAS(status, 0, kStatusBadArgs);
  const uint4* src = reinterpret_cast<const uint4*>(table + (long long)(ok ? id : 0) * dim);
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)t * dim);
  for (int i = threadIdx.x; i < dim / 8; i += blockDim.x)
    dst[i] = ok ? src[i] : make_uint4(0u, 0u, 0u, 0u);
}

// act = bf16(bf16(silu(g)) * u)
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ g,
                                  const __nv_bfloat16* __restrict__ u,
                                  __nv_bfloat16* __restrict__ out, long long n) {
  const long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 2;
  if (i >= n) return;
  const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(g + i);
  const __nv_bfloat162 uv = *reinterpret_cast<const __nv_bfloat162*>(u + i);
  __nv_bfloat162 o;
  o.x = __float2bfloat16_rn(bf16_round(silu(__bfloat162float(gv.x))) * __bfloat162float(uv.x));
  o.y = __float2bfloat16_rn(bf16_round(silu(__bfloat162float(gv.y))) * __bfloat162float(uv.y));
  *reinterpret_cast<__nv_bfloat162*>(out + i) = o;
}

// dg = dact * u * silu'(g),  du = dact * silu(g)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ g,
                                  const __nv_bfloat16* __restrict__ u,
                                  const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dg, __nv_bfloat16* __restrict__ du,
                                  long long n) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float gv = __bfloat162float(g[i]), uv = __bfloat162float(u[i]);
  const float d = __bfloat162float(dact[i]);
  const float sig = 1.f / (1.f + __expf(-gv));
  const float sl = gv * sig;
  dg[i] = __float2bfloat16_rn(d * uv * (sig * (1.f + gv * (1.f - sig))));
  du[i] = __float2bfloat16_rn(d * sl);
}

// Stand-alone interleaved-pair RoPE on x[T, n_heads, head_dim]; position of token t is
// pos[t]. `inverse` applies the transposed rotation (the backward pass).
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                            const __nv_bfloat16* __restrict__ freqs, const int* __restrict__ pos,
                            int n_heads, int head_dim, long long ld, int inverse) {
  const int t = blockIdx.x;
  const int half = head_dim / 2;
  const int p = pos[t];
  for (int i = threadIdx.x; i < n_heads * half; i += blockDim.x) {
    const int h = i / half, j = i - h * half;
    const long long o = (long long)t * ld + h * head_dim + 2 * j;
    const float x0 = __bfloat162float(x[o]), x1 = __bfloat162float(x[o + 1]);
    const float c = __bfloat162float(freqs[((long long)p * half + j) * 2]);
    float s = __bfloat162float(freqs[((long long)p * half + j) * 2 + 1]);
    if (inverse) s = -s;
    out[o] = __float2bfloat16_rn(x0 * c - x1 * s);
    out[o + 1] = __float2bfloat16_rn(x1 * c + x0 * s);
  }
}

}  // namespace e2h

#include "elementwise_vec.cuh"

namespace e2h {

__device__ __forceinline__ float4 ld_sys_f32x4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Large-token form of the fused "residual + sum of tensor-parallel partials (+ RMSNorm)": same
// flag protocol as rmsnorm_fwd_kernel, but every thread moves 8 features per access (two
// 16-byte system-scope loads per partial) and keeps its part of the row in registers.
__device__ __forceinline__ uint4 ld_sys_b32x4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// BF16P: the partials are bf16 (written by the GEMM's TMA-store epilogue) instead of fp32.
template <int NV, bool BF16P>
__global__ void rmsnorm_parts_rows_kernel(const __nv_bfloat16* __restrict__ h_in,
                                          const PartPtrs parts, int n_part,
                                          const __nv_bfloat16* __restrict__ weight,
                                          __nv_bfloat16* __restrict__ h_out,
                                          __nv_bfloat16* __restrict__ x_out, int dim, float eps,
                                          const int* flags, int* use_count, unsigned int* ticket,
                                          int* status) {
  __shared__ float red[64];
  const long long base = (long long)blockIdx.x * dim;
  const int nvec = dim >> 3;
  if (flags != nullptr) {
    const int want = *use_count + 1;
    if (threadIdx.x < n_part)
      wait_flag_ge(flags + threadIdx.x, want, status, g_flag_wait_cycles);
    __syncthreads();
  }
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int s = 0; s < n_part; ++s) {
        if constexpr (BF16P) {
          const __nv_bfloat16* src =
              reinterpret_cast<const __nv_bfloat16*>(parts.p[s]) + base + 8 * i;
          BF8 raw;
          *reinterpret_cast<uint4*>(&raw) =
              flags ? ld_sys_b32x4(src) : *reinterpret_cast<const uint4*>(src);
          float f[8];
          unpack8(raw, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += f[e];
        } else {
          const float* src = parts.p[s] + base + 8 * i;
          const float4 a = flags ? ld_sys_f32x4(src) : *reinterpret_cast<const float4*>(src);
          const float4 b =
              flags ? ld_sys_f32x4(src + 4) : *reinterpret_cast<const float4*>(src + 4);
          acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
          acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
        }
      }
      float r[8];
      unpack8(*reinterpret_cast<const BF8*>(h_in + base + 8 * i), r);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        // the linear's output is a bf16 tensor in the reference; round before the residual add
        v[k][e] = bf16_round(r[e] + bf16_round(acc[e]));
        ss += v[k][e] * v[k][e];
      }
      *reinterpret_cast<BF8*>(h_out + base + 8 * i) = pack8(v[k]);
    }
  }
  if (flags != nullptr) {
    // all reads of this use are done: the last CTA advances the use counter
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
        *ticket = 0;
        *use_count = *use_count + 1;
      }
    }
  }
  if (x_out == nullptr) return;
  ss = block_sum2(ss, 0.f, red).x;
  const float rstd = rsqrtf(ss / dim + eps);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      float w[8], o[8];
      unpack8(*reinterpret_cast<const BF8*>(weight + 8 * i), w);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = bf16_round(v[k][e] * rstd) * w[e];
      *reinterpret_cast<BF8*>(x_out + base + 8 * i) = pack8(o);
    }
  }
}

}  // namespace e2h

using namespace e2h;

// Launches rmsnorm_parts_rows_kernel; returns -100 when the shape / alignment is not covered.
static int launch_parts_rows(const void* h_in, const PartPtrs& parts, int n_part, bool bf16_parts,
                             const void* weight, void* h_out, void* x_out, int T, int dim,
                             float eps, const int* flags, int* use_count, unsigned int* ticket,
                             int* status, void* stream) {
  if (dim % 8 || dim > 8192 || !aligned16(h_in) || !aligned16(h_out)) return -100;
  if (x_out != nullptr && (!aligned16(x_out) || !aligned16(weight))) return -100;
  for (int i = 0; i < n_part; ++i)
    if (!aligned16(parts.p[i])) return -100;
  const int threads = dim > 4096 ? 256 : 128;
  const int nv = (dim / 8 + threads - 1) / threads;
  if (nv > 4) return -100;
  cudaStream_t st = (cudaStream_t)stream;
#define E2H_GO(NV, BP)                                                                       \
  rmsnorm_parts_rows_kernel<NV, BP><<<T, threads, 0, st>>>(                                  \
      (const __nv_bfloat16*)h_in, parts, n_part, (const __nv_bfloat16*)weight,               \
      (__nv_bfloat16*)h_out, (__nv_bfloat16*)x_out, dim, eps, flags, use_count, ticket, status)
  if (bf16_parts) {
    if (nv <= 1) E2H_GO(1, true); else if (nv == 2) E2H_GO(2, true); else E2H_GO(4, true);
  } else {
    if (nv <= 1) E2H_GO(1, false); else if (nv == 2) E2H_GO(2, false); else E2H_GO(4, false);
  }
#undef E2H_GO
  return (int)cudaGetLastError();
}

// Decode-sized RMSNorm (a few dozen rows): what counts is the chain of latencies, not bytes.
// One CTA per row, one 16-byte vector per thread, so a row is one load, one block sum and one
// store; the weight vector is fetched before the wait for the predecessor kernel (weights are
// never written inside a programmatic-dependent-launch chain). Same arithmetic as
// rmsnorm_fwd_kernel: x = bf16(bf16(h * rstd) * w).
__global__ void rmsnorm_row_latency_kernel(const __nv_bfloat16* __restrict__ h_in,
                                           const __nv_bfloat16* __restrict__ weight,
                                           __nv_bfloat16* __restrict__ h_out,
                                           __nv_bfloat16* __restrict__ x_out,
                                           float* __restrict__ rstd_out, int dim, float eps) {
  __shared__ float red[32];
  const int i = threadIdx.x * 8;
  const bool on = i < dim;
  BF8 wv;
  if (on) wv = *reinterpret_cast<const BF8*>(weight + i);
  pdl_launch_dependents();
  pdl_wait_prior();
  const long long base = (long long)blockIdx.x * dim;
  float v[8], w[8];
  float ss = 0.f;
  if (on) {
    const BF8 hv = *reinterpret_cast<const BF8*>(h_in + base + i);
    unpack8(hv, v);
    unpack8(wv, w);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
    if (h_out != nullptr) *reinterpret_cast<BF8*>(h_out + base + i) = hv;
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / dim + eps);
  if (rstd_out != nullptr && threadIdx.x == 0) rstd_out[blockIdx.x] = rstd;
  if (on) {
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = bf16_round(v[e] * rstd) * w[e];
    *reinterpret_cast<BF8*>(x_out + base + i) = pack8(o);
  }
}

extern "C" {

int e2h_rmsnorm_fwd(const void* h_in, const int* tokens, const void* emb, int emb_rows,
                    const void* const* part_ptrs, int n_part, const void* weight, void* h_out,
                    void* x_out, float* rstd_out, int T, int dim, float eps, const int* flags,
                    int* use_count, unsigned int* ticket, int* status, void* stream) {
  if (dim % 2 || n_part > 8) return -1;
  if (tokens != nullptr && (emb == nullptr || emb_rows < 1)) return -1;
  if (flags != nullptr && (use_count == nullptr || ticket == nullptr)) return -2;
  PartPtrs parts;
  for (int i = 0; i < 8; ++i)
    parts.p[i] = i < n_part ? static_cast<const float*>(part_ptrs[i]) : nullptr;
  // many tokens with tensor-parallel partials: the vectorised form of the fused reduce
  if (T >= 256 && h_in != nullptr && tokens == nullptr && n_part > 0 && h_out != nullptr &&
      rstd_out == nullptr) {
    const int rc = launch_parts_rows(h_in, parts, n_part, false, weight, h_out, x_out, T, dim,
                                     eps, flags, use_count, ticket, status, stream);
    if (rc != -100) return rc;
  }
  // plain row normalisation of many tokens: the vectorised streaming kernel
  if (T >= 256 && h_in != nullptr && tokens == nullptr && n_part == 0 && h_out == nullptr &&
      x_out != nullptr && flags == nullptr && dim % 8 == 0 && dim <= 8192 && aligned16(h_in) &&
      aligned16(x_out) && aligned16(weight)) {
    const int threads = dim > 4096 ? 256 : 128;
    const int nv = (dim / 8 + threads - 1) / threads;
    cudaStream_t st = (cudaStream_t)stream;
#define E2H_GO(NV)                                                                            \
  rmsnorm_rows_kernel<NV><<<T, threads, 0, st>>>((const __nv_bfloat16*)h_in,                  \
                                                 (const __nv_bfloat16*)weight,                \
                                                 (__nv_bfloat16*)x_out, rstd_out, dim, eps)
    if (nv <= 1) E2H_GO(1); else if (nv == 2) E2H_GO(2); else if (nv <= 4) E2H_GO(4);
#undef E2H_GO
    if (nv <= 4) return (int)cudaGetLastError();
  }
  // a few rows (decode): the latency-oriented kernel, one 16-byte vector per thread
  static const bool latency_form = [] {   // E2H_NORM_LATENCY=0: measurement switch
    const char* e = getenv("E2H_NORM_LATENCY");
    return !(e && e[0] == '0');
  }();
  if (latency_form && T < 256 && h_in != nullptr && tokens == nullptr && n_part == 0 &&
      x_out != nullptr && flags == nullptr && dim % 8 == 0 && dim / 8 <= 1024 && aligned16(h_in) &&
      aligned16(x_out) && aligned16(weight) && (h_out == nullptr || aligned16(h_out))) {
    const int threads_l = (dim / 8 + 31) / 32 * 32;
    return (int)launch(rmsnorm_row_latency_kernel, dim3(T), dim3(threads_l), 0,
                       (cudaStream_t)stream, (const __nv_bfloat16*)h_in,
                       (const __nv_bfloat16*)weight, (__nv_bfloat16*)h_out,
                       (__nv_bfloat16*)x_out, rstd_out, dim, eps);
  }
  const int threads = dim >= 2048 ? 512 : 128;
  const size_t smem = (dim + 32) * sizeof(float);
  return (int)launch(rmsnorm_fwd_kernel, dim3(T), dim3(threads), smem, (cudaStream_t)stream,
                     (const __nv_bfloat16*)h_in, tokens, (const __nv_bfloat16*)emb, emb_rows, parts,
                     n_part,
                     (const __nv_bfloat16*)weight, (__nv_bfloat16*)h_out, (__nv_bfloat16*)x_out,
                     rstd_out, dim, eps, flags, use_count, ticket, status);
}

// h_out = h_in + sum of the bf16 [T, dim] partials (peers' symmetric buffers), optionally
// x_out = rmsnorm(h_out) * weight; same flag protocol as e2h_rmsnorm_fwd.
int e2h_reduce_residual_norm_bf16(const void* h_in, const void* const* part_ptrs, int n_part,
                                  const void* weight, void* h_out, void* x_out, int T, int dim,
                                  float eps, const int* flags, int* use_count,
                                  unsigned int* ticket, int* status, void* stream) {
  if (n_part < 1 || n_part > 8 || h_in == nullptr || h_out == nullptr) return -1;
  if (flags != nullptr && (use_count == nullptr || ticket == nullptr)) return -2;
  PartPtrs parts;
  for (int i = 0; i < 8; ++i)
    parts.p[i] = i < n_part ? static_cast<const float*>(part_ptrs[i]) : nullptr;
  const int rc = launch_parts_rows(h_in, parts, n_part, true, weight, h_out, x_out, T, dim, eps,
                                   flags, use_count, ticket, status, stream);
  return rc == -100 ? -3 : rc;
}

int e2h_rmsnorm_bwd(const void* x, const void* dy, const void* weight, const void* dres, void* dx,
                    int T, int dim, float eps, void* stream) {
  if (dim % 8 == 0 && dim <= 8192 && aligned16(x) && aligned16(dy) && aligned16(dx) &&
      aligned16(weight) && (dres == nullptr || aligned16(dres))) {
    const int threads = dim > 4096 ? 256 : 128;
    const int nv = (dim / 8 + threads - 1) / threads;
    cudaStream_t st = (cudaStream_t)stream;
#define E2H_GO(NV)                                                                           \
  rmsnorm_bwd_rows_kernel<NV><<<T, threads, 0, st>>>(                                        \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)weight,       \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, dim, eps)
    if (nv <= 1) E2H_GO(1); else if (nv == 2) E2H_GO(2); else if (nv <= 4) E2H_GO(4);
#undef E2H_GO
    if (nv <= 4) return (int)cudaGetLastError();
  }
  const int threads = dim >= 2048 ? 512 : 128;
  const size_t smem = (2 * dim + 32) * sizeof(float);
  rmsnorm_bwd_kernel<<<T, threads, smem, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, (const __nv_bfloat16*)weight,
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, dim, eps);
  return (int)cudaGetLastError();
}

int e2h_embedding(const int* tokens, const void* table, int rows, void* out, int T, int dim,
                  int* status, void* stream) {
  if (dim % 8 || rows < 1) return -1;
  embedding_kernel<<<T, 128, 0, (cudaStream_t)stream>>>(tokens, (const __nv_bfloat16*)table, rows,
                                                        (__nv_bfloat16*)out, dim, status);
  return (int)cudaGetLastError();
}

int e2h_swiglu_fwd(const void* g, const void* u, void* out, long long n, void* stream) {
  if (n % 2) return -1;
  if (n % 8 == 0 && aligned16(g) && aligned16(u) && aligned16(out)) {
    const long long nvec = n / 8;
    long long vb = (nvec + 255) / 256;
    if (vb > 148 * 16) vb = 148 * 16;
    swiglu_fwd_vec_kernel<<<(unsigned)vb, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)out, nvec);
    return (int)cudaGetLastError();
  }
  const long long blocks = (n / 2 + 255) / 256;
  swiglu_fwd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)out, n);
  return (int)cudaGetLastError();
}

int e2h_swiglu_bwd(const void* g, const void* u, const void* dact, void* dg, void* du, long long n,
                   void* stream) {
  if (n % 8 == 0 && aligned16(g) && aligned16(u) && aligned16(dact) && aligned16(dg) &&
      aligned16(du)) {
    const long long nvec = n / 8;
    long long vb = (nvec + 255) / 256;
    if (vb > 148 * 16) vb = 148 * 16;
    swiglu_bwd_vec_kernel<<<(unsigned)vb, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (const __nv_bfloat16*)dact,
        (__nv_bfloat16*)dg, (__nv_bfloat16*)du, nvec);
    return (int)cudaGetLastError();
  }
  const long long blocks = (n + 255) / 256;
  swiglu_bwd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (const __nv_bfloat16*)dact,
      (__nv_bfloat16*)dg, (__nv_bfloat16*)du, n);
  return (int)cudaGetLastError();
}

int e2h_rope(const void* x, void* out, const void* freqs, const int* pos, int T, int n_heads,
             int head_dim, long long ld, int inverse, void* stream) {
  if (head_dim % 8 == 0 && ld % 8 == 0 && aligned16(x) && aligned16(out) && aligned16(freqs)) {
    rope_vec_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)out, (const __nv_bfloat16*)freqs, pos, n_heads,
        head_dim, ld, inverse);
    return (int)cudaGetLastError();
  }
  rope_kernel<<<T, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out,
                                                   (const __nv_bfloat16*)freqs, pos, n_heads,
                                                   head_dim, ld, inverse);
  return (int)cudaGetLastError();
}

// Sets the cross-rank flag wait limit of this device (milliseconds at ~2 GHz); returns 0 or a
// cudaError_t.
int e2h_set_flag_wait_ms(int ms) {
  const long long cycles = (long long)(ms < 1 ? 1 : ms) * 2000000LL;
  return (int)cudaMemcpyToSymbol(g_flag_wait_cycles, &cycles, sizeof(cycles));
}

// Process-wide switch for programmatic dependent launch (see launch.cuh).
int e2h_set_pdl(int on) {
  const int old = e2h::g_pdl;
  e2h::g_pdl = on ? 1 : 0;
  return old;
}

}  // extern "C"
