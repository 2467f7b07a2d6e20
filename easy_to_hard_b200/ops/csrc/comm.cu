// Stand-alone collective kernels over peer-mapped (symmetric) memory.
//
// e2h_reduce_scatter_accum: the gradient reduce-scatter of sharded data parallelism fused with
// the bf16 -> fp32 cast, the 1/world averaging and the accumulation into the fp32 gradient
// shard. Every rank's backward pass leaves a flat bf16 gradient buffer in its own symmetric
// memory and then raises a flag on every peer (e2h_signal_peers, stream-ordered after the
// weight-gradient GEMMs). The reduce kernel of rank r waits -- bounded -- for all flags and pulls
// slice r of every rank's buffer with 16-byte system-scope loads, sums in fp32 and writes (or
// adds to) its fp32 shard: one pass, no intermediate reduce-scatter output, no NCCL.
// Two buffer slots alternate between consecutive uses; a slot is only rewritten two uses later,
// after this rank has itself consumed the peers' flags of the use in between, which the peers
// raise only after they have finished reading the older slot (same stream order on every rank).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace e2h {

struct PeerSrc {
  const __nv_bfloat16* p[8];
};
struct PeerFlags {
  int* p[8];
};

__global__ void signal_peers_kernel(const PeerFlags flags, int n) {
  if (threadIdx.x < n) {
    __threadfence_system();
    red_release_sys_add(flags.p[threadIdx.x], 1);
  }
}

__device__ __forceinline__ uint4 comm_ld_sys_b32x4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// src.p[r] points at element 0 of this rank's slice inside rank r's buffer; n is a multiple of 8.
__global__ void reduce_scatter_accum_kernel(const PeerSrc src, int n_peer, float* __restrict__ out,
                                            long long n, float scale, int accumulate,
                                            const int* flags, int* use_count, unsigned int* ticket,
                                            long long wait_cycles, int* status) {
  if (flags != nullptr) {
    const int want = *use_count + 1;
    if (threadIdx.x < n_peer) wait_flag_ge(flags + threadIdx.x, want, status, wait_cycles);
    __syncthreads();
  }
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int r = 0; r < n_peer; ++r) {
      const uint4 raw = flags ? comm_ld_sys_b32x4(src.p[r] + 8 * i)
                              : *reinterpret_cast<const uint4*>(src.p[r] + 8 * i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += __bfloat162float(h[e].x);
        acc[2 * e + 1] += __bfloat162float(h[e].y);
      }
    }
    float4* dst = reinterpret_cast<float4*>(out + 8 * i);
    float4 lo = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
    float4 hi = make_float4(acc[4] * scale, acc[5] * scale, acc[6] * scale, acc[7] * scale);
    if (accumulate) {
      const float4 a = dst[0], b = dst[1];
      lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
      hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
    }
    dst[0] = lo;
    dst[1] = hi;
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
}

// ---- general stand-alone collectives over the same flag protocol --------------------------------
struct PeerBytes {
  const uint8_t* p[8];
};

// Waits (bounded) until every one of the n flag words has reached use_count + 1; with `advance`
// the single CTA then bumps the counter. A barrier is signal_peers followed by this kernel.
__global__ void wait_flags_kernel(const int* flags, int n, int* use_count, int advance,
                                  long long wait_cycles, int* status) {
  const int want = *use_count + 1;
  if (threadIdx.x < n) wait_flag_ge(flags + threadIdx.x, want, status, wait_cycles);
  __syncthreads();
  if (advance && threadIdx.x == 0) *use_count = want;
}

// Common prologue / epilogue of the pull kernels: wait for every producer, and let the last CTA
// advance the use counter once all reads of this use are done.
__device__ __forceinline__ void comm_wait_all(const int* flags, int n_peer, const int* use_count,
                                              int* status, long long wait_cycles) {
  if (flags != nullptr) {
    const int want = *use_count + 1;
    if (threadIdx.x < n_peer) wait_flag_ge(flags + threadIdx.x, want, status, wait_cycles);
    __syncthreads();
  }
}
__device__ __forceinline__ void comm_done(const int* flags, int* use_count, unsigned int* ticket) {
  if (flags != nullptr) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
        *ticket = 0;
        *use_count = *use_count + 1;
      }
    }
  }
}

// All-gather by pulling: out[r * nbytes .. ) = bytes of rank r's buffer (16-byte vectors).
__global__ void p2p_gather_kernel(const PeerBytes src, int n_peer, uint8_t* __restrict__ out,
                                  long long nbytes, const int* flags, int* use_count,
                                  unsigned int* ticket, long long wait_cycles, int* status) {
  comm_wait_all(flags, n_peer, use_count, status, wait_cycles);
  const long long nvec = nbytes >> 4;
  // always system-scope loads: the peers rewrite these buffers between uses (between optimizer
  // steps for parameter shards), a line kept in this SM's L1 from an earlier use must not serve
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int r = 0; r < n_peer; ++r) {
    uint4* dst = reinterpret_cast<uint4*>(out + (long long)r * nbytes);
    long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {      // four loads in flight per thread
      const uint4 a = comm_ld_sys_b32x4(src.p[r] + 16 * i);
      const uint4 b = comm_ld_sys_b32x4(src.p[r] + 16 * (i + stride));
      const uint4 c = comm_ld_sys_b32x4(src.p[r] + 16 * (i + 2 * stride));
      const uint4 d = comm_ld_sys_b32x4(src.p[r] + 16 * (i + 3 * stride));
      dst[i] = a;
      dst[i + stride] = b;
      dst[i + 2 * stride] = c;
      dst[i + 3 * stride] = d;
    }
    for (; i < nvec; i += stride) dst[i] = comm_ld_sys_b32x4(src.p[r] + 16 * i);
  }
  comm_done(flags, use_count, ticket);
}

// One-shot all-reduce (or, on a slice, the reduce step of a reduce-scatter / two-shot
// all-reduce): out[i] = bf16( scale * sum_r src_r[i] ), fp32 accumulation in rank order, so every
// rank computes bit-identical sums.
__global__ void p2p_reduce_bf16_kernel(const PeerSrc src, int n_peer,
                                       __nv_bfloat16* __restrict__ out, long long n, float scale,
                                       const int* flags, int* use_count, unsigned int* ticket,
                                       long long wait_cycles, int* status) {
  comm_wait_all(flags, n_peer, use_count, status, wait_cycles);
  const long long nvec = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int r = 0; r < n_peer; ++r) {
      const uint4 raw = flags ? comm_ld_sys_b32x4(src.p[r] + 8 * i)
                              : *reinterpret_cast<const uint4*>(src.p[r] + 8 * i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += __bfloat162float(h[e].x);
        acc[2 * e + 1] += __bfloat162float(h[e].y);
      }
    }
    uint4 pk;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int e = 0; e < 4; ++e)
      o[e] = __floats2bfloat162_rn(acc[2 * e] * scale, acc[2 * e + 1] * scale);
    *reinterpret_cast<uint4*>(out + 8 * i) = pk;
  }
  comm_done(flags, use_count, ticket);
}

}  // namespace e2h

using namespace e2h;

extern "C" {

// flag_ptrs: n device addresses (this rank's flag word inside every rank's buffer).
int e2h_signal_peers(const void* const* flag_ptrs, int n, void* stream) {
  if (n < 1 || n > 8) return -1;
  PeerFlags f;
  for (int i = 0; i < 8; ++i) f.p[i] = i < n ? (int*)flag_ptrs[i] : nullptr;
  signal_peers_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, n);
  return (int)cudaGetLastError();
}

int e2h_reduce_scatter_accum(const void* const* peer_src, int n_peer, float* out, long long n,
                             float scale, int accumulate, const int* flags, int* use_count,
                             unsigned int* ticket, int wait_ms, int* status, void* stream) {
  if (n_peer < 1 || n_peer > 8 || n <= 0 || (n % 8)) return -1;
  if (flags != nullptr && (use_count == nullptr || ticket == nullptr)) return -2;
  if (reinterpret_cast<uintptr_t>(out) & 15) return -3;
  PeerSrc s;
  for (int i = 0; i < 8; ++i) {
    s.p[i] = i < n_peer ? (const __nv_bfloat16*)peer_src[i] : nullptr;
    if (i < n_peer && (reinterpret_cast<uintptr_t>(s.p[i]) & 15)) return -3;
  }
  long long blocks = (n / 8 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const long long cycles = (long long)(wait_ms < 1 ? 1 : wait_ms) * 2000000LL;
  reduce_scatter_accum_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      s, n_peer, out, n, scale, accumulate, flags, use_count, ticket, cycles, status);
  return (int)cudaGetLastError();
}

static long long comm_cycles(int wait_ms) { return (long long)(wait_ms < 1 ? 1 : wait_ms) * 2000000LL; }
static unsigned comm_blocks(long long nvec) {
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return (unsigned)(blocks < 1 ? 1 : blocks);
}

// Bounded wait until flags[0..n) >= *use_count + 1 (status word set on a time-out); `advance`
// bumps the counter afterwards.
int e2h_wait_flags(const int* flags, int n, int* use_count, int advance, int wait_ms, int* status,
                   void* stream) {
  if (n < 1 || n > 8 || flags == nullptr || use_count == nullptr) return -1;
  wait_flags_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, n, use_count, advance,
                                                         comm_cycles(wait_ms), status);
  return (int)cudaGetLastError();
}

// out[r * nbytes ..) = nbytes of peer_src[r] for r < n_peer (nbytes a multiple of 16).
int e2h_p2p_all_gather(const void* const* peer_src, int n_peer, void* out, long long nbytes,
                       const int* flags, int* use_count, unsigned int* ticket, int wait_ms,
                       int* status, void* stream) {
  if (n_peer < 1 || n_peer > 8 || nbytes <= 0 || (nbytes % 16)) return -1;
  if (flags != nullptr && (use_count == nullptr || ticket == nullptr)) return -2;
  if (reinterpret_cast<uintptr_t>(out) & 15) return -3;
  PeerBytes s;
  for (int i = 0; i < 8; ++i) {
    s.p[i] = i < n_peer ? (const uint8_t*)peer_src[i] : nullptr;
    if (i < n_peer && (reinterpret_cast<uintptr_t>(s.p[i]) & 15)) return -3;
  }
  unsigned blocks = comm_blocks(nbytes / 16);
  if (blocks > 296) blocks = 296;   // two CTAs per SM keep NVLink busy and leave the SMs to the GEMMs
  p2p_gather_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
      s, n_peer, (uint8_t*)out, nbytes, flags, use_count, ticket, comm_cycles(wait_ms), status);
  return (int)cudaGetLastError();
}

// out[0..n) = bf16(scale * sum_r peer_src[r][0..n)), n a multiple of 8.
int e2h_p2p_reduce_bf16(const void* const* peer_src, int n_peer, void* out, long long n,
                        float scale, const int* flags, int* use_count, unsigned int* ticket,
                        int wait_ms, int* status, void* stream) {
  if (n_peer < 1 || n_peer > 8 || n <= 0 || (n % 8)) return -1;
  if (flags != nullptr && (use_count == nullptr || ticket == nullptr)) return -2;
  if (reinterpret_cast<uintptr_t>(out) & 15) return -3;
  PeerSrc s;
  for (int i = 0; i < 8; ++i) {
    s.p[i] = i < n_peer ? (const __nv_bfloat16*)peer_src[i] : nullptr;
    if (i < n_peer && (reinterpret_cast<uintptr_t>(s.p[i]) & 15)) return -3;
  }
  p2p_reduce_bf16_kernel<<<comm_blocks(n / 8), 256, 0, (cudaStream_t)stream>>>(
      s, n_peer, (__nv_bfloat16*)out, n, scale, flags, use_count, ticket, comm_cycles(wait_ms),
      status);
  return (int)cudaGetLastError();
}

}  // extern "C"
