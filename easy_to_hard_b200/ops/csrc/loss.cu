// Fused log-softmax / cross-entropy / log-prob gather / entropy over fp32 logits, forward and
// backward, with a vocabulary-parallel form: each rank runs the kernels on its logits shard and
// only four numbers per token (max, sum-exp, target logit, sum of p*x) cross ranks.
//
// Reference semantics: token cross-entropy in fp32 with ignore_index (train_sft.py:98-115),
// per-token log-probs and entropies of temperature-scaled logits (models/rl_model.py:134-160),
// the three-reduction vocab-parallel cross-entropy (models/tp.py:888-969).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <float.h>
#include <stdint.h>

#include "launch.cuh"
#include "ptx.cuh"

namespace e2h {

constexpr int kCeThreads = 512;

__device__ __forceinline__ float block_reduce(float v, float* red, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < (blockDim.x >> 5) ? red[lane] : (is_max ? -FLT_MAX : 0.f);
  t = is_max ? warp_max(t) : warp_sum(t);
  return t;
}

// stats[row] = (m, s, tgt, u):  m = max_i z_i, s = sum exp(z_i - m), u = sum exp(z_i - m) z_i,
// tgt = z_target if the target lies in this shard else 0,  with z = logits * inv_temp.
__global__ void __launch_bounds__(kCeThreads)
ce_stats_kernel(const float* __restrict__ logits, long long ld, int vocab,
                const long long* __restrict__ targets, int vocab_start, float inv_temp,
                float4* __restrict__ stats) {
  __shared__ float red[32];
  pdl_wait_prior();  // launched through the PDL-capable helper: wait before any global access
  const int row = blockIdx.x;
  const float* x = logits + (long long)row * ld;
  float m = -FLT_MAX;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, x[i] * inv_temp);
  m = block_reduce(m, red, true);
  float s = 0.f, u = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float z = x[i] * inv_temp;
    const float e = __expf(z - m);
    s += e;
    u += e * z;
  }
  s = block_reduce(s, red, false);
  u = block_reduce(u, red, false);
  if (threadIdx.x == 0) {
    const long long t = targets[row] - vocab_start;
    const float tgt = (t >= 0 && t < vocab) ? x[t] * inv_temp : 0.f;
    stats[row] = make_float4(m, s, tgt, u);
  }
}

// dlogits[row, i] = inv_temp * ( g_lp * ((i == target) - p_i) - g_ent * p_i * (z_i - lse + H) )
// with p_i = exp(z_i - lse); lse / H are the full-vocabulary values of the row.
__global__ void __launch_bounds__(kCeThreads)
ce_grad_kernel(const float* __restrict__ logits, long long ld, int vocab,
               const long long* __restrict__ targets, int vocab_start, float inv_temp,
               const float* __restrict__ lse, const float* __restrict__ ent,
               const float* __restrict__ g_lp, const float* __restrict__ g_ent,
               __nv_bfloat16* __restrict__ dlogits, long long ldd) {
  pdl_wait_prior();  // launched through the PDL-capable helper: wait before any global access
  const int row = blockIdx.x;
  const float* x = logits + (long long)row * ld;
  __nv_bfloat16* d = dlogits + (long long)row * ldd;
  const float L = lse[row];
  const float glp = g_lp ? g_lp[row] : 0.f;
  const float gen = g_ent ? g_ent[row] : 0.f;
  const float H = (g_ent && ent) ? ent[row] : 0.f;
  const long long t = targets[row] - vocab_start;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float z = x[i] * inv_temp;
    const float p = __expf(z - L);
    float g = glp * ((i == t ? 1.f : 0.f) - p);
    if (gen != 0.f) g -= gen * p * (z - L + H);
    d[i] = __float2bfloat16_rn(g * inv_temp);
  }
}

}  // namespace e2h

extern "C" int e2h_ce_stats(const float* logits, long long ld, int rows, int vocab,
                            const long long* targets, int vocab_start, float inv_temp,
                            float* stats, void* stream) {
  using namespace e2h;
  return (int)launch(ce_stats_kernel, dim3(rows), dim3(kCeThreads), 0, (cudaStream_t)stream,
                     logits, ld, vocab, targets, vocab_start, inv_temp,
                     reinterpret_cast<float4*>(stats));
}

extern "C" int e2h_ce_grad(const float* logits, long long ld, int rows, int vocab,
                           const long long* targets, int vocab_start, float inv_temp,
                           const float* lse, const float* ent, const float* g_lp,
                           const float* g_ent, void* dlogits, long long ldd, void* stream) {
  using namespace e2h;
  return (int)launch(ce_grad_kernel, dim3(rows), dim3(kCeThreads), 0, (cudaStream_t)stream,
                     logits, ld, vocab, targets, vocab_start, inv_temp, lse, ent, g_lp, g_ent,
                     static_cast<__nv_bfloat16*>(dlogits), ldd);
}
