// Decode attention over the static KV cache: one new query token per sequence.
//
// The reference runs masked SDPA over the whole cache allocation every step
// (models/model.py:121-129, 343-344); this kernel reads only the live range
// [left_pad[b], pos] of each row, which is what makes batched decode HBM-bound on the
// useful bytes only. It is a pure streaming kernel (every K/V byte is used once per q head),
// so the arithmetic runs on the CUDA cores; grouped-query attention reuses each K/V row for the
// G query heads that share it.
//
// Layouts: q [B, n_head*D] bf16, caches [max_batch, n_kv, smax, D] bf16, out [B, n_head*D] bf16.
//
// Work split (with more pairs than resident CTAs; with fewer, every pair is simply cut into
// equal parts, one per CTA): the live keys of every (sequence, kv head) are cut into chunks of
// 32 keys, all chunks are numbered (sequence, head, chunk) and every CTA takes one contiguous
// run of that numbering, the same number of chunks for all: the CTAs finish together whatever the batch,
// the head count and the context lengths are, and a CTA pays the latency of its first loads
// once, not once per (sequence, head). A producer thread streams the K and V rows of the run
// with bulk copies (cp.async.bulk: the rows of one head are contiguous in the cache) through a
// ring of shared-memory stages and runs ahead across (sequence, head) boundaries; four
// consumer warps follow, a half-warp (16 lanes x 8 elements) owning one key row at a time.
// A (sequence, head) that lies inside one run is written straight to `out`; one that is cut by
// run boundaries leaves (m, l, acc) partials, and the last of its CTAs to arrive (a ticket
// counter per pair) merges them in CTA order, so the result does not depend on timing.
//
// All mbarrier waits are bounded; a time-out sets the status word (codes 101 / 102), the CTA
// stops issuing copies, waits (bounded) for the ones in flight, still reaches its barriers and
// returns.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <float.h>
#include <stdint.h>
#include <stdlib.h>
#include <mutex>

#include "launch.cuh"
#include "ptx.cuh"

namespace e2h {

constexpr int kWarps = 4;           // consumer warps; warp kWarps is the producer
constexpr int kSlots = kWarps * 2;  // half-warps per CTA
constexpr int kKeysPerIter = 4;     // key rows per half-warp and stage
constexpr int kChunk = kSlots * kKeysPerIter;   // key rows per pipeline stage
constexpr int kAttnMaxStages = 8;
constexpr int kAttnThreads = (kWarps + 1) * 32;
constexpr int kAttnMaxParts = 8;    // CTAs that may share one (sequence, kv head)
constexpr int kAttnMaxB = 512;      // sequences per launch (longer batches go in slices)

__host__ __device__ constexpr int attn_smem_bytes(int D, int stages) {
  return stages * 2 * kChunk * D * 2;
}

// The K/V rows are read once per step and are far larger than L2 together with the weights:
// they are marked evict-first so that they do not push out what the following kernels reuse
// (activations, the kernels' own code).
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void consumers_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
}

__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __bfloat162float(h[i].x);
    f[2 * i + 1] = __bfloat162float(h[i].y);
  }
}

// Position in the numbering of all chunks: sequence b, kv head hk, chunk ch of nc, first live key.
struct AttnWalk {
  int b, hk, ch, nc, start;
};

// D = 16 * 8 * R : each lane of the half-warp holds R groups of 8 consecutive elements.
template <int D, int G>
__global__ void __launch_bounds__(kAttnThreads)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
                   const __nv_bfloat16* __restrict__ vcache, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ partial, const int* __restrict__ pos_ptr,
                   const int* __restrict__ left_pad, int B, int n_head, int n_kv, int smax,
                   float scale, int max_parts, int fixed_parts,
                   unsigned int* __restrict__ tickets, int* __restrict__ status,
                   int stages_and_flags) {
  const int stages = stages_and_flags & 255;
  constexpr int R = D / 128 > 0 ? D / 128 : 1;       // 8-element groups per lane (D=128 -> 1)
  constexpr int LPK = D >= 128 ? 16 : D / 8;          // lanes per key row
  constexpr int kTileBytes = kChunk * D * 2;          // K (or V) rows of one stage
  static_assert(D == 64 || D == 128 || D == 256, "head_dim must be 64, 128 or 256");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = lane / 16;            // which key of the pair this half-warp handles
  const int hl = lane & 15;
  const bool lane_active = hl < LPK;
  const int slot = warp * 2 + half;

  extern __shared__ __align__(128) uint8_t attn_smem[];
  __shared__ uint64_t bar_full[kAttnMaxStages], bar_empty[kAttnMaxStages];
  __shared__ int abort_word, nc_max_s, is_last_s;
  __shared__ int pre[kAttnMaxB + 1];     // chunks of the sequences before b (per kv head)
  __shared__ int first_key[kAttnMaxB];
  __shared__ float sm_m[kSlots][G], sm_l[kSlots][G];
  __shared__ float sm_acc[kSlots][G][D];
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), kWarps);
    }
    abort_word = 0;
    fence_mbar_init();
  }

  pdl_launch_dependents();   // the successor may start its prologue / weight prefetch already
  pdl_wait_prior();
  int pos = *pos_ptr;                    // index of the newest token (already in the cache)
  // positions come from device memory: keep every cache row that is read inside the allocation
  if (pos >= smax) pos = smax - 1;
  if (pos < 0) pos = 0;
  if (warp == 0) {
    int run = 0, ncm = 0;
    for (int b0 = 0; b0 < B; b0 += 32) {
      const int b = b0 + lane;
      int nc = 0, start = 0;
      if (b < B) {
        start = left_pad ? left_pad[b] : 0;
        if (start > pos) start = pos;
        if (start < 0) start = 0;
        nc = (pos - start + kChunk) / kChunk;       // ceil((pos - start + 1) / kChunk) >= 1
        first_key[b] = start;
      }
      int x = nc;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      if (b < B) pre[b + 1] = run + x;
      run += __shfl_sync(0xffffffffu, x, 31);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) nc = max(nc, __shfl_xor_sync(0xffffffffu, nc, o));
      ncm = max(ncm, nc);
    }
    if (lane == 0) {
      pre[0] = 0;
      nc_max_s = ncm;
    }
  }
  __syncthreads();

  // this CTA's run [lo, hi) of the chunk numbering
  const int total = pre[B] * n_kv;
  int per, lo, hi;
  if (fixed_parts > 0) {
    // fewer pairs than resident CTAs: every pair is cut into fixed_parts equal parts, one per
    // CTA (fixed_parts == 1: one CTA per pair, nothing to merge)
    const int item = blockIdx.x / fixed_parts, part = blockIdx.x - item * fixed_parts;
    const int b = item / n_kv, hk = item - b * n_kv;
    const int nc = pre[b + 1] - pre[b];
    per = (nc + fixed_parts - 1) / fixed_parts;
    lo = pre[b] * n_kv + hk * nc + part * per;
    hi = min(pre[b] * n_kv + (hk + 1) * nc, lo + per);
  } else {
    per = (total + (int)gridDim.x - 1) / (int)gridDim.x;
    per = max(per, (nc_max_s + max_parts - 2) / (max_parts - 1));   // at most max_parts CTAs per pair
    lo = min(total, (int)blockIdx.x * per);
    hi = min(total, lo + per);
  }
  if (lo >= hi) return;

  AttnWalk w;
  {
    int l = 0, r = B - 1;                 // largest b with pre[b] * n_kv <= lo
    while (l < r) {
      const int mid = (l + r + 1) >> 1;
      if (pre[mid] * n_kv <= lo) l = mid; else r = mid - 1;
    }
    w.b = l;
    w.nc = pre[l + 1] - pre[l];
    const int rem = lo - pre[l] * n_kv;
    w.hk = rem / w.nc;
    w.ch = rem - w.hk * w.nc;
    w.start = first_key[l];
  }

  if (warp == kWarps) {
    // ---- producer: one thread streams the K and V rows of every chunk of the run
    if (lane == 0) {
      uint64_t pol;
      if (stages_and_flags & 256) {   // E2H_ATTN_L2HINT=0: plain L2 policy (measurement switch)
        asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
      } else {
        pol = policy_evict_first();
      }
      int issued = 0, s = 0, ph = 1;   // ph: the parity that "stage s is free again" completes with
      bool dead = false;
      for (int P = lo; P < hi && !dead;) {
        const int n_here = min(w.nc - w.ch, hi - P);
        const __nv_bfloat16* kb = kcache + ((long long)w.b * n_kv + w.hk) * smax * D;
        const __nv_bfloat16* vb = vcache + ((long long)w.b * n_kv + w.hk) * smax * D;
        for (int i = 0; i < n_here; ++i) {
          if (issued >= stages &&
              !mbar_wait(smem_u32(&bar_empty[s]), ph, abort_flag, status, kStatusTimeoutEmpty)) {
            dead = true;
            break;
          }
          const int j0 = w.start + (w.ch + i) * kChunk;
          const uint32_t bytes = (uint32_t)min(kChunk, pos + 1 - j0) * D * 2;
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t dst = smem_u32(attn_smem) + s * 2 * kTileBytes;
          mbar_expect_tx(full, 2 * bytes);
          bulk_load_1d(dst, kb + (long long)j0 * D, bytes, full, pol);
          bulk_load_1d(dst + kTileBytes, vb + (long long)j0 * D, bytes, full, pol);
          ++issued;
          if (++s == stages) {
            s = 0;
            ph ^= 1;
          }
        }
        P += n_here;
        w.ch = 0;
        if (++w.hk == n_kv && P < hi) {
          w.hk = 0;
          ++w.b;
          w.nc = pre[w.b + 1] - pre[w.b];
          w.start = first_key[w.b];
        }
      }
      if (*abort_flag) {
        // gave up: no more copies are issued; let those on their way land (bounded) before the
        // CTA's shared memory goes back to the SM
        for (int c = max(0, issued - stages); c < issued; ++c) {
          const long long t0 = clock64();
          while (!mbar_try_wait(smem_u32(&bar_full[c % stages]), (c / stages) & 1) &&
                 clock64() - t0 < kWaitLimitCycles) {
          }
        }
      }
    }
    return;
  }

  // ---- consumers
  int s = 0, ph = 0;
  bool dead = false;     // a wait ran out: skip the data, keep walking so that every barrier is met
  for (int P = lo; P < hi;) {
    const int n_here = min(w.nc - w.ch, hi - P);
    const bool whole = w.ch == 0 && n_here == w.nc;
    float qv[G][R][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int h = w.hk * G + g;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (lane_active) {
          const uint4 raw = *reinterpret_cast<const uint4*>(
              q + ((long long)w.b * n_head + h) * D + (r * LPK + hl) * 8);
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

    for (int c = 0; c < n_here; ++c) {
      if (!dead && !mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag, status, kStatusTimeoutFull))
        dead = true;
      if (!dead) {
        const int j0 = w.start + (w.ch + c) * kChunk;
        const uint8_t* ks = attn_smem + s * 2 * kTileBytes;
        const uint8_t* vs = ks + kTileBytes;
        uint4 kr[kKeysPerIter][R], vr[kKeysPerIter][R];
#pragma unroll
        for (int u = 0; u < kKeysPerIter; ++u) {
          const int row = u * kSlots + slot;
          const bool ok = j0 + row <= pos && lane_active;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const int o = (row * D + (r * LPK + hl) * 8) * 2;
            kr[u][r] = ok ? *reinterpret_cast<const uint4*>(ks + o) : make_uint4(0, 0, 0, 0);
            vr[u][r] = ok ? *reinterpret_cast<const uint4*>(vs + o) : make_uint4(0, 0, 0, 0);
          }
        }
        // the values are in registers: the stage can be refilled while they are used
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_empty[s]));
        // the four keys of this half-warp go through the running softmax together: one
        // rescale of the accumulator per four keys instead of one per key (the kernel is close
        // to instruction-issue bound: 63 % issue-active at 0.86 of the copy bandwidth)
        float kf[kKeysPerIter][R][8];
#pragma unroll
        for (int u = 0; u < kKeysPerIter; ++u)
#pragma unroll
          for (int r = 0; r < R; ++r) unpack8(kr[u][r], kf[u][r]);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float sc[kKeysPerIter];
#pragma unroll
          for (int u = 0; u < kKeysPerIter; ++u) {
            float d = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
              for (int i = 0; i < 8; ++i) d += qv[g][r][i] * kf[u][r][i];
            sc[u] = d;
          }
          // reduce over the 16 lanes of the half-warp, the four keys interleaved
#pragma unroll
          for (int o = 8; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < kKeysPerIter; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
          float mn = m[g];
#pragma unroll
          for (int u = 0; u < kKeysPerIter; ++u)
            if (j0 + u * kSlots + slot <= pos) mn = fmaxf(mn, sc[u]);
          const float corr = __expf(m[g] - mn);
          float pj[kKeysPerIter], psum = 0.f;
#pragma unroll
          for (int u = 0; u < kKeysPerIter; ++u) {
            pj[u] = (j0 + u * kSlots + slot <= pos) ? __expf(sc[u] - mn) : 0.f;
            psum += pj[u];
          }
          l[g] = l[g] * corr + psum;
          m[g] = mn;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            float vf[kKeysPerIter][8];
#pragma unroll
            for (int u = 0; u < kKeysPerIter; ++u) unpack8(vr[u][r], vf[u]);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float a = acc[g][r][i] * corr;
#pragma unroll
              for (int u = 0; u < kKeysPerIter; ++u) a += pj[u] * vf[u][i];
              acc[g][r][i] = a;
            }
          }
        }
      }
      if (++s == stages) {
        s = 0;
        ph ^= 1;
      }
    }

    // ---- this (sequence, head) is done as far as this CTA goes: merge the 8 half-warp partials
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
    consumers_sync();
    // which of the pair's CTAs this one is, and how many there are
    int part, parts;
    if (fixed_parts > 0) {
      part = (int)blockIdx.x % fixed_parts;
      parts = (w.nc + per - 1) / per;
    } else {
      const int item_lo = pre[w.b] * n_kv + w.hk * w.nc;
      const int cta_first = item_lo / per, cta_last = (item_lo + w.nc - 1) / per;
      part = (int)blockIdx.x - cta_first;
      parts = cta_last - cta_first + 1;
    }
    for (int idx = threadIdx.x; idx < G * D; idx += kWarps * 32) {
      const int g = idx / D, d = idx - g * D;
      float mm = -FLT_MAX;
#pragma unroll
      for (int t = 0; t < kSlots; ++t) mm = fmaxf(mm, sm_m[t][g]);
      float ll = 0.f, a = 0.f;
#pragma unroll
      for (int t = 0; t < kSlots; ++t) {
        const float wt = (sm_m[t][g] == -FLT_MAX) ? 0.f : __expf(sm_m[t][g] - mm);
        ll += sm_l[t][g] * wt;
        a += sm_acc[t][g][d] * wt;
      }
      const int h = w.hk * G + g;
      if (whole) {
        out[((long long)w.b * n_head + h) * D + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
      } else {
        float* pp = partial + (((long long)w.b * n_head + h) * max_parts + part) * (D + 2);
        pp[d] = a;
        if (d == 0) {
          pp[D] = mm;
          pp[D + 1] = ll;
        }
      }
    }
    if (!whole) {
      // the last of the pair's CTAs to get here combines all parts, in CTA order (the ticket
      // word returns to zero for the next launch)
      __threadfence();
      consumers_sync();
      if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(&tickets[w.b * n_kv + w.hk], 1u);
        is_last_s = (t == (unsigned int)parts - 1) ? 1 : 0;
        if (is_last_s) tickets[w.b * n_kv + w.hk] = 0;
      }
      consumers_sync();
      if (is_last_s) {
        __threadfence();
        for (int idx = threadIdx.x; idx < G * D; idx += kWarps * 32) {
          const int g = idx / D, d = idx - g * D;
          const int h = w.hk * G + g;
          const float* pp = partial + ((long long)w.b * n_head + h) * max_parts * (D + 2);
          float mm = -FLT_MAX;
          for (int t = 0; t < parts; ++t) mm = fmaxf(mm, __ldcg(pp + t * (D + 2) + D));
          float ll = 0.f, a = 0.f;
          for (int t = 0; t < parts; ++t) {
            const float ms = __ldcg(pp + t * (D + 2) + D);
            const float wt = (ms == -FLT_MAX) ? 0.f : __expf(ms - mm);
            ll += __ldcg(pp + t * (D + 2) + D + 1) * wt;
            a += __ldcg(pp + t * (D + 2) + d) * wt;
          }
          out[((long long)w.b * n_head + h) * D + d] =
              __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
        }
      }
    }
    consumers_sync();      // the merge buffers are free for the next pair

    P += n_here;
    w.ch = 0;
    if (++w.hk == n_kv && P < hi) {
      w.hk = 0;
      ++w.b;
      w.nc = pre[w.b + 1] - pre[w.b];
      w.start = first_key[w.b];
    }
  }
}

// Resident CTAs per SM at this pipeline depth (shared memory is what limits them), at most 4.
static int attn_ctas_per_sm(int D, int G, int stages) {
  // static shared memory of the kernel, plus the 1 KB that the system keeps per resident CTA
  const int fixed = (2 * kAttnMaxB + 1) * 4 + kSlots * G * (D + 2) * 4 + 256 + 1024;
  const int n = (227 * 1024) / (attn_smem_bytes(D, stages) + fixed);
  return n < 1 ? 1 : n > 4 ? 4 : n;
}

template <int D, int G>
static int launch_decode(const void* q, const void* k, const void* v, void* out, float* partial,
                         const int* pos, const int* left_pad, int B, int n_head, int n_kv, int smax,
                         float scale, int max_parts, cudaStream_t stream, unsigned int* tickets,
                         int* status) {
  // E2H_ATTN_STAGES: pipeline depth (16 KB of K and V each at head_dim 128), default 3
  static const int stages = [] {
    const char* e = getenv("E2H_ATTN_STAGES");
    const int v_ = e ? atoi(e) : 3;
    return v_ < 2 ? 2 : v_ > kAttnMaxStages ? kAttnMaxStages : v_;
  }();
  static const bool plain_l2 = [] {
    const char* e = getenv("E2H_ATTN_L2HINT");
    return e && e[0] == '0';
  }();
  // more than 48 KB of dynamic shared memory has to be asked for once per device
  static std::mutex mu;
  static bool asked[64];
  static int n_sm[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return -5;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!asked[dev]) {
      e = cudaFuncSetAttribute(attn_decode_kernel<D, G>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               attn_smem_bytes(D, kAttnMaxStages));
      if (e != cudaSuccess) return (int)e;
      e = cudaDeviceGetAttribute(&n_sm[dev], cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return (int)e;
      asked[dev] = true;
    }
  }
  if (max_parts > kAttnMaxParts) max_parts = kAttnMaxParts;
  const long long q_stride = (long long)n_head * D;
  for (int b0 = 0; b0 < B; b0 += kAttnMaxB) {     // batches beyond kAttnMaxB go in slices
    const int nb = B - b0 < kAttnMaxB ? B - b0 : kAttnMaxB;
    const int resident = n_sm[dev] * attn_ctas_per_sm(D, G, stages);
    int fixed_parts = 0;
    if (max_parts <= 1) {
      fixed_parts = 1;
    } else if (nb * n_kv <= resident) {
      fixed_parts = resident / (nb * n_kv);      // all CTAs resident at once
      if (fixed_parts > max_parts) fixed_parts = max_parts;
    }
    const int grid = fixed_parts > 0 ? nb * n_kv * fixed_parts : resident;
    e = launch(attn_decode_kernel<D, G>, dim3(grid), dim3(kAttnThreads),
               attn_smem_bytes(D, stages), stream,
               (const __nv_bfloat16*)q + b0 * q_stride,
               (const __nv_bfloat16*)k + (long long)b0 * n_kv * smax * D,
               (const __nv_bfloat16*)v + (long long)b0 * n_kv * smax * D,
               (__nv_bfloat16*)out + b0 * q_stride,
               partial ? partial + (long long)b0 * n_head * max_parts * (D + 2) : nullptr, pos,
               left_pad ? left_pad + b0 : nullptr, nb, n_head, n_kv, smax, scale, max_parts,
               fixed_parts, tickets ? tickets + (long long)b0 * n_kv : nullptr, status,
               stages | (plain_l2 ? 256 : 0));
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

}  // namespace e2h

// max_parts: how many CTAs may share one (sequence, kv head), 1..8. With 1 every pair gets a CTA
// of its own and neither `partial` nor `tickets` is touched; otherwise
//   partial: fp32 scratch of B*n_head*max_parts*(D+2) floats (need not be initialised),
//   tickets: uint32 [B*n_kv], zero before the first launch (every launch leaves it zero).
extern "C" int e2h_attn_decode(const void* q, const void* kcache, const void* vcache, void* out,
                               float* partial, const int* pos, const int* left_pad, int B,
                               int n_head, int n_kv, int head_dim, int smax, float scale,
                               int max_parts, unsigned int* tickets, int* status,
                               void* stream_v) {
  using namespace e2h;
  cudaStream_t stream = (cudaStream_t)stream_v;
  if (B < 1 || n_kv < 1 || n_head % n_kv) return -1;
  if (max_parts > 1 && (partial == nullptr || tickets == nullptr)) return -2;
  const int G = n_head / n_kv;
#define E2H_GO(D_, G_)                                                                          \
  return launch_decode<D_, G_>(q, kcache, vcache, out, partial, pos, left_pad, B, n_head, n_kv, \
                               smax, scale, max_parts, stream, tickets, status)
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
// one ticket word per (sequence, kv head); zero in the library image, and every launch leaves
// them zero
constexpr int kStaticTickets = 16384;
static __device__ unsigned int g_static_tickets[kStaticTickets];

static float* g_static_partial_ptr[kMaxDevices];   // per device, filled on that device's first call
static unsigned int* g_static_tickets_ptr[kMaxDevices];
static std::mutex g_static_partial_mu;

static int static_partial_for_current_device(float** ptr, unsigned int** tickets) {
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
    unsigned int* t = nullptr;
    e = cudaGetSymbolAddress((void**)&t, g_static_tickets);
    if (e != cudaSuccess) {
      fprintf(stderr, "e2h_attn_decode_static: cudaGetSymbolAddress failed: %s\n",
              cudaGetErrorString(e));
      return (int)e;
    }
    g_static_partial_ptr[dev] = p;
    g_static_tickets_ptr[dev] = t;
  }
  *ptr = g_static_partial_ptr[dev];
  *tickets = g_static_tickets_ptr[dev];
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
  if (n_split > 1 && (need > kStaticPartialFloats || (long long)B * n_kv > kStaticTickets)) {
    fprintf(stderr,
            "e2h_attn_decode_static: B*n_head*n_split*(head_dim+2) = %lld floats exceeds the "
            "fixed scratch of %lld floats (64 x 32 heads x 8 parts x head_dim 128), or B*n_kv "
            "exceeds %d; use fewer parts or e2h_attn_decode with a caller-provided buffer\n",
            need, kStaticPartialFloats, kStaticTickets);
    return -4;
  }
  float* partial = nullptr;
  unsigned int* tickets = nullptr;
  if (n_split > 1) {
    const int rc = static_partial_for_current_device(&partial, &tickets);
    if (rc != 0) return rc;
  }
  cudaStream_t stream = (cudaStream_t)stream_v;
  const int G = n_head / n_kv;
#define E2H_GO(D_, G_)                                                                          \
  return launch_decode<D_, G_>(q, kcache, vcache, out, partial, pos, left_pad, B, n_head, n_kv, \
                               smax, scale, n_split, stream, tickets, nullptr)
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
