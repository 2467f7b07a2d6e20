// Reward / value head on the residual stream, one kernel:
//   y       = bf16( bf16(x * rsqrt(mean(x^2) + eps)) * w_norm )          (the model's final RMSNorm)
//   dot_r   = sum_{k in [k0, k0 + klen)} y[k] * head[r][k],  r = 0, 1     (fp32 accumulation)
//   reward  = ( bf16(dot_0) + bf16(dot_1) ) / 2                            (models/reward_model.py:80-88
//             of the reference: a [2, dim] head whose two outputs are averaged)
//   loss   += weight * BCE_with_logits(reward, label)                      (train_rm_pointwise.py:101-110)
// The normalised activations never go to memory; rows can be picked by an index list (the reward
// at the end-of-sequence positions only), so scoring a batch reads each selected row once.
//
// One warp per row, the row held in registers (16-byte loads), two passes over registers.
// Under tensor parallelism the head is sharded along dim: the kernel then runs with the rank's
// [k0, k0 + klen) slice and `finalize` = 0, and returns the fp32 partial dots for the caller to
// all-reduce; the norm statistics always cover the whole row.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.cuh"
#include "ptx.cuh"

namespace e2h {

template <int NV>   // NV 16-byte vectors per lane: dim <= NV * 256
__global__ void __launch_bounds__(256)
reward_head_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                   const __nv_bfloat16* __restrict__ w_norm, const __nv_bfloat16* __restrict__ head,
                   long long ldh, int dim, int k0, int klen, float eps,
                   const int* __restrict__ index, int n_rows, long long x_rows,
                   float* __restrict__ dots,
                   float* __restrict__ reward, int finalize, const float* __restrict__ labels,
                   const float* __restrict__ weights, float* __restrict__ loss_acc) {
  pdl_wait_prior();
  pdl_launch_dependents();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= n_rows) return;
  long long src_row = index ? (long long)index[warp] : (long long)warp;
  // gathered rows come from device memory: a row outside x reads row 0 instead of faulting
  if (src_row < 0 || src_row >= x_rows) src_row = 0;
  const __nv_bfloat16* xr = x + src_row * ldx;
  const int nvec = dim >> 3;                       // 16-byte vectors in the row
  uint4 v[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    v[i] = make_uint4(0, 0, 0, 0);
    if (c < nvec) v[i] = *reinterpret_cast<const uint4*>(xr + 8 * c);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h2[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)dim + eps);
  float d0 = 0.f, d1 = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    const int k = 8 * c;
    if (c < nvec && k >= k0 && k < k0 + klen) {    // slices are multiples of 8 columns
      const uint4 wv = *reinterpret_cast<const uint4*>(w_norm + k);
      const uint4 h0 = *reinterpret_cast<const uint4*>(head + (k - k0));
      const uint4 h1 = *reinterpret_cast<const uint4*>(head + ldh + (k - k0));
      const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&h0);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&h1);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = __bfloat1622float2(x2[j]);
        const float2 wf = __bfloat1622float2(w2[j]);
        const float2 af = __bfloat1622float2(a2[j]);
        const float2 bf = __bfloat1622float2(b2[j]);
        const float y0 = bf16_round(bf16_round(xf.x * rstd) * wf.x);
        const float y1 = bf16_round(bf16_round(xf.y * rstd) * wf.y);
        d0 += y0 * af.x + y1 * af.y;
        d1 += y0 * bf.x + y1 * bf.y;
      }
    }
  }
  d0 = warp_sum(d0);
  d1 = warp_sum(d1);
  if (lane == 0) {
    if (dots) {
      dots[2 * warp] = d0;
      dots[2 * warp + 1] = d1;
    }
    if (finalize) {
      const float r = 0.5f * (bf16_round(d0) + bf16_round(d1));
      if (reward) reward[warp] = r;
      if (labels && loss_acc) {
        const float wgt = weights ? weights[warp] : 1.f;
        // BCE with logits, the overflow-safe form: max(r, 0) - r * y + log(1 + exp(-|r|))
        const float bce = fmaxf(r, 0.f) - r * labels[warp] + log1pf(__expf(-fabsf(r)));
        atomicAdd(loss_acc, wgt * bce);
        atomicAdd(loss_acc + 1, wgt);
      }
    }
  }
}

}  // namespace e2h

// x [*, ldx] bf16 residual stream; w_norm [dim] bf16; head [2, ldh] bf16 holding columns
// [k0, k0 + klen) of the full head; index: optional int32 [n_rows] source rows; dots: optional fp32
// [n_rows, 2]; reward: optional fp32 [n_rows]; labels / weights: optional fp32 [n_rows];
// loss_acc: fp32 [2] (+= weighted BCE sum, += weight sum). Returns 0 or a cudaError_t / negative.
extern "C" int e2h_reward_head(const void* x, long long ldx, const void* w_norm, const void* head,
                               long long ldh, int dim, int k0, int klen, float eps,
                               const void* index, int n_rows, long long x_rows, void* dots,
                               void* reward, int finalize, const void* labels,
                               const void* weights, void* loss_acc, void* stream_v) {
  using namespace e2h;
  if (n_rows <= 0) return 0;
  if (x_rows < 1 || (index == nullptr && n_rows > x_rows)) return -1;
  if (dim <= 0 || (dim % 8) || (k0 % 8) || (klen % 8) || k0 < 0 || k0 + klen > dim) return -1;
  if ((ldx % 8) || (ldh % 8) || ((uintptr_t)x & 15) || ((uintptr_t)head & 15) ||
      ((uintptr_t)w_norm & 15))
    return -2;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const dim3 block(256), grid((n_rows + 7) / 8);
#define E2H_RH(NV_)                                                                              \
  return (int)launch(reward_head_kernel<NV_>, grid, block, 0, stream,                            \
                     static_cast<const __nv_bfloat16*>(x), ldx,                                  \
                     static_cast<const __nv_bfloat16*>(w_norm),                                  \
                     static_cast<const __nv_bfloat16*>(head), ldh, dim, k0, klen, eps,           \
                     static_cast<const int*>(index), n_rows, x_rows, static_cast<float*>(dots),  \
                     static_cast<float*>(reward), finalize, static_cast<const float*>(labels),   \
                     static_cast<const float*>(weights), static_cast<float*>(loss_acc))
  if (dim <= 2 * 256) E2H_RH(2);
  if (dim <= 8 * 256) E2H_RH(8);
  if (dim <= 16 * 256) E2H_RH(16);
  if (dim <= 32 * 256) E2H_RH(32);
#undef E2H_RH
  return -3;
}
