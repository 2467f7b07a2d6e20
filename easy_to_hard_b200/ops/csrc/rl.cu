// Reinforcement-learning element-wise kernels.
//
// e2h_gae: generalised advantage estimation (https://arxiv.org/abs/1506.02438) over [B, T]
// rewards / values, the recursion of trainers/ppo_trainer.py:209-236 of the reference
//   delta_t = r_t + gamma * V_{t+1} - V_t        (V_T = 0)
//   A_t     = delta_t + gamma * lambda * A_{t+1}
//   R_t     = A_t + V_t
// as one launch: one warp per sequence. The affine recursion A_t = delta_t + c * A_{t+1} is
// evaluated 32 time steps at a time with a warp scan over (coefficient, offset) pairs, walking
// the sequence from its end, so global loads and stores are coalesced.
#include <cuda_runtime.h>
#include <stdint.h>

namespace e2h {

__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                           float* __restrict__ adv, float* __restrict__ ret, int B, int T,
                           float gamma, float lam) {
  const int warps_per_block = blockDim.x >> 5;
  const int b = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= B) return;
  const float* r = rewards + (long long)b * T;
  const float* v = values + (long long)b * T;
  float* a_out = adv + (long long)b * T;
  float* r_out = ret + (long long)b * T;
  const float c = gamma * lam;
  float carry = 0.f;                       // A_{t+1} of the chunk processed before (later in time)
  for (int hi = T; hi > 0; hi -= 32) {
    // lane l handles time step t = hi - 1 - l (reverse order: lane 0 is the latest step)
    const int t = hi - 1 - lane;
    const bool ok = t >= 0;
    float vt = 0.f, delta = 0.f;
    if (ok) {
      vt = v[t];
      const float vnext = (t + 1 < T) ? v[t + 1] : 0.f;
      delta = r[t] + gamma * vnext - vt;
    }
    // inclusive scan of the maps x -> delta + coef * x composed from lane 0 upwards:
    // A(lane) = off(lane) + coef(lane) * carry
    float coef = ok ? c : 1.f, off = ok ? delta : 0.f;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float pc = __shfl_up_sync(0xffffffffu, coef, d);
      const float po = __shfl_up_sync(0xffffffffu, off, d);
      if (lane >= d) {
        off = off + coef * po;             // apply the earlier-lane (later-time) map first
        coef = coef * pc;
      }
    }
    const float a = off + coef * carry;
    if (ok) {
      a_out[t] = a;
      r_out[t] = a + vt;
    }
    // the earliest valid step of this chunk feeds the next chunk
    const int last_lane = min(31, hi - 1);
    carry = __shfl_sync(0xffffffffu, a, last_lane);
  }
}

}  // namespace e2h

extern "C" int e2h_gae(const float* rewards, const float* values, float* adv, float* ret, int B,
                       int T, float gamma, float lam, void* stream) {
  if (B <= 0 || T <= 0) return -1;
  const int warps = 4;
  e2h::gae_kernel<<<(B + warps - 1) / warps, warps * 32, 0, (cudaStream_t)stream>>>(
      rewards, values, adv, ret, B, T, gamma, lam);
  return (int)cudaGetLastError();
}
