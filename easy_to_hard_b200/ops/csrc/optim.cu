// Fused AdamW update (one pass over parameter, gradient and both moments) plus the helpers
// of the two-phase global gradient clip: a squared-norm partial reduction and a kernel that
// turns the reduced norm into a clip coefficient on the device, so that the optimizer step
// needs no host synchronisation.
//
// Update rule = the reference's memory-efficient AdamW
// (training_utils/memory_efficient_adam.py:61-104):
//   p *= 1 - lr*wd;  m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g   (in the state dtype)
//   denom = sqrt(v)/sqrt(bc2) + eps;  p -= (lr/bc1) * m / denom     (in the parameter dtype)
// Parameter, gradient and state may each be fp32 or bf16.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "ptx.cuh"

namespace e2h {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) {
  p[i] = __float2bfloat16_rn(v);
}
template <typename T> __device__ __forceinline__ float rnd(float v);
template <> __device__ __forceinline__ float rnd<float>(float v) { return v; }
template <> __device__ __forceinline__ float rnd<__nv_bfloat16>(float v) { return bf16_round(v); }

template <typename P, typename G, typename S>
__global__ void adamw_kernel(P* __restrict__ p, const G* __restrict__ g, S* __restrict__ m,
                             S* __restrict__ v, P* __restrict__ p_lowp_unused, long long n,
                             float lr, float b1, float b2, float eps, float wd, float bc1,
                             float bc2, const float* __restrict__ clip_coef,
                             __nv_bfloat16* __restrict__ p_bf16_copy) {
  const float coef = clip_coef ? *clip_coef : 1.f;
  const float step = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float pv = ldf<P>(p, i);
    if (wd != 0.f) pv = rnd<P>(pv * (1.f - lr * wd));
    const float gv = rnd<S>(ldf<G>(g, i) * coef);
    const float mv = rnd<S>(rnd<S>(b1 * ldf<S>(m, i)) + (1.f - b1) * gv);
    const float vv = rnd<S>(rnd<S>(b2 * ldf<S>(v, i)) + (1.f - b2) * gv * gv);
    const float denom = rnd<S>(rnd<S>(sqrtf(vv) * inv_sqrt_bc2) + eps);
    pv = pv - step * rnd<P>(mv) / rnd<P>(denom);
    stf<P>(p, i, pv);
    stf<S>(m, i, mv);
    stf<S>(v, i, vv);
    if (p_bf16_copy) p_bf16_copy[i] = __float2bfloat16_rn(pv);
  }
}

// out[0] += sum(x^2) (fp32 atomics; one atomic per CTA)
template <typename T>
__global__ void sqnorm_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = ldf<T>(x, i);
    s += v * v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(out, t);
  }
}

// coef = min(1, max_norm / (sqrt(sqnorm) + 1e-6)); norm_out = sqrt(sqnorm)
__global__ void clip_coef_kernel(const float* sqnorm, float max_norm, float* coef,
                                 float* norm_out) {
  const float nrm = sqrtf(*sqnorm);
  *norm_out = nrm;
  *coef = fminf(1.f, max_norm / (nrm + 1e-6f));
}

template <typename P, typename G, typename S>
static int launch_adamw(void* p, const void* g, void* m, void* v, long long n, float lr, float b1,
                        float b2, float eps, float wd, float bc1, float bc2, const float* clip,
                        void* p_bf16, cudaStream_t st) {
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  adamw_kernel<P, G, S><<<(unsigned)blocks, 256, 0, st>>>(
      (P*)p, (const G*)g, (S*)m, (S*)v, nullptr, n, lr, b1, b2, eps, wd, bc1, bc2, clip,
      (__nv_bfloat16*)p_bf16);
  return (int)cudaGetLastError();
}

}  // namespace e2h

using namespace e2h;

// dtype codes: 0 = fp32, 1 = bf16.  p_bf16_copy (optional) receives the updated parameter in
// bf16 -- the compute copy that the next forward pass gathers.
extern "C" int e2h_adamw(void* p, const void* g, void* m, void* v, long long n, int p_dt, int g_dt,
                         int s_dt, float lr, float b1, float b2, float eps, float wd, float bc1,
                         float bc2, const float* clip_coef, void* p_bf16_copy, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  typedef __nv_bfloat16 bf;
#define GO(P, G, S) \
  return launch_adamw<P, G, S>(p, g, m, v, n, lr, b1, b2, eps, wd, bc1, bc2, clip_coef, p_bf16_copy, st)
  const int code = p_dt * 4 + g_dt * 2 + s_dt;
  switch (code) {
    case 0: GO(float, float, float);
    case 1: GO(float, float, bf);
    case 2: GO(float, bf, float);
    case 3: GO(float, bf, bf);
    case 4: GO(bf, float, float);
    case 5: GO(bf, float, bf);
    case 6: GO(bf, bf, float);
    case 7: GO(bf, bf, bf);
  }
#undef GO
  return -1;
}

extern "C" int e2h_sqnorm(const void* x, long long n, int dt, float* out, void* stream) {
  long long blocks = (n + 1023) / 1024;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  if (dt == 0)
    sqnorm_kernel<float><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const float*)x, n, out);
  else
    sqnorm_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, n, out);
  return (int)cudaGetLastError();
}

extern "C" int e2h_clip_coef(const float* sqnorm, float max_norm, float* coef, float* norm_out,
                             void* stream) {
  clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(sqnorm, max_norm, coef, norm_out);
  return (int)cudaGetLastError();
}
