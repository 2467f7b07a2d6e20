// Tensor-parallel "all-reduce + residual + RMSNorm" of the decode engine as ONE kernel over peer
// memory, the consumer of a row-parallel GEMM (wo, w2) under tensor parallelism. It replaces the
// reference's all-reduce hook (models/tp.py:297-310) plus the following residual add and RMSNorm.
//
// Every rank's GEMM leaves its bf16 partial [T, dim] in its own symmetric buffer and raises flag
// A on every peer. This kernel then runs a reduce-scatter and an all-gather by token rows:
//
//   phase A  wait (bounded) until every rank's partial of this use is complete;
//   reduce   rank r owns rows [row0, row0 + rows): sum of the n partials of those rows, either
//            with plain 16-byte peer loads or, where the group has an NVSwitch multicast mapping,
//            with one multimem.ld_reduce (the switch adds, fp32 accumulation) per 16 bytes;
//            + residual (local, only the owner keeps the residual stream of a row), RMSNorm;
//   gather   the owner writes the normalised rows into every rank's activation buffer (plain
//            peer stores, or one multimem.st that the switch replicates), then raises flag B on
//            every peer once all of its rows are out;
//   phase B  wait (bounded) until every rank has raised flag B: the full [T, dim] input of the
//            next column-parallel GEMM is now in local memory, which that GEMM reads with TMA.
//
// Each row is reduced and normalised by exactly one rank, so all ranks see bit-identical
// activations (which keeps their samplers in lock step), and a rank moves 2 * T/n rows over
// NVLink instead of pulling n - 1 whole partials.
//
// For decode-sized inputs (a few hundred KB per partial) latency, not bytes, is the cost, and
// the same kernel runs in its ONE-SHOT form: every rank sums all rows itself, pulling the
// peers' partials with plain 16-byte loads in the same rank order (so the results are still
// bit-identical), writes only its own activation buffer and needs neither the gather nor phase
// B: one NVLink round trip per use instead of three. The partial buffers then alternate
// between two slots, so that a rank's next GEMM never overwrites a partial a slower peer is
// still reading (a slot is rewritten two uses later, after this rank has seen the peers' flags
// of the use in between, which they raise only after their reads of the older use).
//
// Flags count uses: flag words only ever grow (red.add 1 per use), and the kernel compares them
// with its own per-call-site use counter in local memory, which the last CTA advances. Nothing is
// reset between uses, so the sequence replays inside a CUDA graph. All waits are bounded; a
// time-out records kStatusTimeoutFlag in the status word and the kernel carries on to its end.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.cuh"
#include "ptx.cuh"

namespace e2h {

struct TpPtrs {
  void* p[8];
};

namespace {

struct alignas(16) Bf8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void bf8_unpack(const Bf8& b, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __bfloat162float(b.v[i].x);
    f[2 * i + 1] = __bfloat162float(b.v[i].y);
  }
}
__device__ __forceinline__ Bf8 bf8_pack(const float* f) {
  Bf8 b;
#pragma unroll
  for (int i = 0; i < 4; ++i) b.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return b;
}
__device__ __forceinline__ Bf8 ld_sys_bf8(const void* p) {
  Bf8 b;
  uint32_t* r = reinterpret_cast<uint32_t*>(&b);
  asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "l"(p)
               : "memory");
  return b;
}
__device__ __forceinline__ void st_sys_bf8(void* p, const Bf8& b) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(&b);
  asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}
// Sum over all replicas of a multicast address: 8 bf16 per instruction, added in fp32 inside the
// NVSwitch and rounded to bf16 once.
__device__ __forceinline__ Bf8 multimem_ld_reduce_bf8(const void* mc) {
  Bf8 b;
  uint32_t* r = reinterpret_cast<uint32_t*>(&b);
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
      : "l"(mc)
      : "memory");
  return b;
}
// One store that the switch writes into every replica of the multicast address.
__device__ __forceinline__ void multimem_st_bf8(void* mc, const Bf8& b) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(&b);
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}

// Bounded wait for *p >= want. A wait gives up at once when the status word already carries a
// code: after one time-out the rest of a pass (dozens of dependent waits) must not each run
// out its own limit before the host gets to read the status.
__device__ __forceinline__ bool tp_wait_ge(const int* p, int want, int* status, long long limit) {
  if (ld_acquire_sys(p) >= want) return true;
  const long long t0 = clock64();
  while (ld_acquire_sys(p) < want) {
    if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return false;
    if (clock64() - t0 > limit) {
      if (status != nullptr) atomicCAS(status, 0, kStatusTimeoutFlag);
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ float block_sum_f(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  v = lane < nw ? red[lane] : 0.f;
  return warp_sum(v);
}

}  // namespace

struct TpReduceArgs {
  const __nv_bfloat16* h_in;    // local [T, dim] residual stream; nullptr = zeros
  __nv_bfloat16* h_out;         // local [T, dim]; only this rank's rows are written
  const __nv_bfloat16* weight;  // [dim] RMSNorm weight
  TpPtrs parts;                 // every rank's bf16 [T, dim] partial (MC: p[0] = multicast address)
  TpPtrs xn;                    // every rank's bf16 [T, dim] activation buffer (MC: p[0] = multicast)
  TpPtrs flag_b_remote;         // the word this rank bumps in every rank's B flags
  const int* flag_a;            // local int32 [n]: rank i's partial is complete
  const int* flag_b;            // local int32 [n]: rank i's rows have arrived here
  int* count;                   // local use counter of this call site
  unsigned int* ticket;         // local, zero between launches
  int* status;
  long long wait_cycles;
  int n, rank, dim, row0, rows, wait_b;
  int n_xn;      // activation buffers written (n: every rank's; 1: only p[0], the local one;
                 // 0: none, a plain reduce-scatter)
  int signal_b;  // 0: no gather hand-shake (one-shot form, reduce-scatter only)
  int do_reduce;    // 0: nothing to sum, the rows are h_in as it is (a pure gather)
  int do_norm;      // 0: the gathered rows are the (summed) rows themselves, not their RMSNorm
  int self_signal;  // 1: no producer kernel raises flag A for this use; the kernel raises it
                    // itself when it starts (everything earlier on this rank's stream is
                    // done), which makes phase A a barrier: peers may write into this rank's
                    // activation buffer only once its earlier readers have finished
  int h_compact;    // 1: h_in / h_out hold only this rank's rows (row 0 = global row row0)
  TpPtrs flag_a_remote;  // self_signal: this rank's flag-A word on every rank
  float eps;
};

// One CTA per owned row (at least one CTA, which then only takes part in the hand-shakes).
// NV 16-byte vectors per thread hold the row between the reduction and the write.
// LDMC: the sum is one multimem.ld_reduce on parts.p[0]; STMC: the rows go out as one multimem.st
// on xn.p[0].
template <int NV, bool LDMC, bool STMC>
__global__ void tp_reduce_norm_kernel(const TpReduceArgs a) {
  __shared__ float red[32];
  // the norm weight is a constant of the model: fetched before the waits, so that its latency
  // hides behind them instead of following the block sum
  const int nvec0 = a.dim >> 3;
  Bf8 wv[NV];
  if (a.do_norm && a.n_xn > 0) {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nvec0) wv[k] = *reinterpret_cast<const Bf8*>(a.weight + 8 * i);
    }
  }
  pdl_launch_dependents();
  pdl_wait_prior();
  const int want = *a.count + 1;
  if (a.self_signal && blockIdx.x == 0 && threadIdx.x < a.n) {
    __threadfence_system();
    red_release_sys_add(static_cast<int*>(a.flag_a_remote.p[threadIdx.x]), 1);
  }
  if (threadIdx.x < a.n) tp_wait_ge(a.flag_a + threadIdx.x, want, a.status, a.wait_cycles);
  __syncthreads();

  const int nvec = a.dim >> 3;
  if ((int)blockIdx.x < a.rows) {
    const long long base = (long long)(a.row0 + blockIdx.x) * a.dim;
    const long long hbase = a.h_compact ? (long long)blockIdx.x * a.dim : base;
    float v[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nvec) {
        const long long off = base + 8 * i;
        const long long hoff = hbase + 8 * i;
        float acc[8];
        if (!a.do_reduce) {
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        } else if constexpr (LDMC) {
          bf8_unpack(multimem_ld_reduce_bf8(static_cast<const __nv_bfloat16*>(a.parts.p[0]) + off),
                     acc);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = 0.f;
          for (int s = 0; s < a.n; ++s) {
            float f[8];
            bf8_unpack(ld_sys_bf8(static_cast<const __nv_bfloat16*>(a.parts.p[s]) + off), f);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += f[e];
          }
        }
        float r[8];
        if (a.h_in != nullptr) {
          bf8_unpack(*reinterpret_cast<const Bf8*>(a.h_in + hoff), r);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) r[e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          // the linear's output is a bf16 tensor in the reference: round, then the residual add
          v[k][e] = a.do_reduce ? bf16_round(r[e] + bf16_round(acc[e])) : r[e];
          ss += v[k][e] * v[k][e];
        }
        if (a.h_out != nullptr) *reinterpret_cast<Bf8*>(a.h_out + hoff) = bf8_pack(v[k]);
      }
    }
    float rstd = 1.f;
    if (a.do_norm) {
      ss = block_sum_f(ss, red);
      rstd = rsqrtf(ss / a.dim + a.eps);
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nvec && a.n_xn > 0) {
        const long long off = base + 8 * i;
        float o[8];
        if (a.do_norm) {
          float w[8];
          bf8_unpack(wv[k], w);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = bf16_round(v[k][e] * rstd) * w[e];
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = v[k][e];
        }
        const Bf8 ob = bf8_pack(o);
        if constexpr (STMC) {
          multimem_st_bf8(static_cast<__nv_bfloat16*>(a.xn.p[0]) + off, ob);
        } else if (a.n_xn == 1) {
          *reinterpret_cast<Bf8*>(static_cast<__nv_bfloat16*>(a.xn.p[0]) + off) = ob;
        } else {
          for (int s = 0; s < a.n_xn; ++s)
            st_sys_bf8(static_cast<__nv_bfloat16*>(a.xn.p[s]) + off, ob);
        }
      }
    }
  }

  // The last CTA to get here tells every rank that this rank's rows are out, waits for the
  // other ranks' rows and advances the use counter (one-shot form: only the counter).
  if (a.signal_b) __threadfence_system();
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) is_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!is_last) return;
  if (a.signal_b && threadIdx.x < a.n) {
    __threadfence_system();
    red_release_sys_add(static_cast<int*>(a.flag_b_remote.p[threadIdx.x]), 1);
    if (a.wait_b) tp_wait_ge(a.flag_b + threadIdx.x, want, a.status, a.wait_cycles);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *a.ticket = 0;
    *a.count = want;
  }
}

// Masked lookup of a vocabulary-sharded embedding table (models/tp.py:85-119 of the reference):
// rows whose token id lies in [v0, v0 + rows_local) are copied, all others are zero, into this
// rank's partial buffer; the last CTA raises flag A on every peer. The sum over ranks (the
// reference's all-reduce) is then taken by tp_reduce_norm_kernel with no residual.
__global__ void tp_embed_partial_kernel(const int* __restrict__ tokens,
                                        const __nv_bfloat16* __restrict__ table, int v0,
                                        int rows_local, __nv_bfloat16* __restrict__ part, int dim,
                                        const TpPtrs flag_a_remote, int n, unsigned int* ticket) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const int t = blockIdx.x;
  const int id = tokens[t] - v0;
  const bool mine = id >= 0 && id < rows_local;
  const uint4* src = reinterpret_cast<const uint4*>(table + (long long)(mine ? id : 0) * dim);
  uint4* dst = reinterpret_cast<uint4*>(part + (long long)t * dim);
  for (int i = threadIdx.x; i < dim / 8; i += blockDim.x)
    dst[i] = mine ? src[i] : make_uint4(0u, 0u, 0u, 0u);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0;
      __threadfence_system();
      if (n < 0) {   // p[0] is the word's multicast address: one add reaches every rank
        multimem_red_release_sys_add(static_cast<int*>(flag_a_remote.p[0]), 1);
      } else {
        for (int r = 0; r < n; ++r) red_release_sys_add(static_cast<int*>(flag_a_remote.p[r]), 1);
      }
    }
  }
}

// All-gather of fp32 logit shards for vocabulary-parallel sampling (models/rl_model.py:372-375
// of the reference): waits (bounded) for every rank's shard [B, vs] and copies them from the
// peers' symmetric buffers into the local [B, n * vs] matrix, 16 bytes per access.
template <int VW>
__global__ void tp_gather_logits_kernel(const TpPtrs shards, int n, int B, int vs,
                                        float* __restrict__ out, long long ldo, const int* flag_a,
                                        int* count, unsigned int* ticket, int* status,
                                        long long wait_cycles) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const int want = *count + 1;
  if (threadIdx.x < n) tp_wait_ge(flag_a + threadIdx.x, want, status, wait_cycles);
  __syncthreads();
  const int b = blockIdx.x, r = blockIdx.y;
  const float* src = static_cast<const float*>(shards.p[r]) + (long long)b * vs;
  float* dst = out + (long long)b * ldo + (long long)r * vs;
  for (int i = threadIdx.x * VW; i < vs; i += blockDim.x * VW) {
    if constexpr (VW == 4) {
      float4 v;
      asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                   : "l"(src + i)
                   : "memory");
      *reinterpret_cast<float4*>(dst + i) = v;
    } else if constexpr (VW == 2) {
      const float2 v = ld_sys_f32x2(src + i);
      *reinterpret_cast<float2*>(dst + i) = v;
    } else {
      float v;
      asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(src + i) : "memory");
      dst[i] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ticket, 1u) == gridDim.x * gridDim.y - 1) {
      *ticket = 0;
      *count = want;
    }
  }
}

}  // namespace e2h

using namespace e2h;

extern "C" {

static int tp_rows_launch(TpReduceArgs& a, bool ldmc, bool stmc, void* stream) {
  const int threads = a.dim >= 4096 ? 512 : (a.dim >= 1024 ? 128 : 64);
  const int nv = (a.dim / 8 + threads - 1) / threads;
  if (nv > 4) return -3;
  const dim3 grid(a.rows > 0 ? a.rows : 1), block(threads);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define E2H_GO(NV)                                                                          \
  return (int)(ldmc ? (stmc ? launch(tp_reduce_norm_kernel<NV, true, true>, grid, block, 0, st, a)    \
                            : launch(tp_reduce_norm_kernel<NV, true, false>, grid, block, 0, st, a))  \
                    : (stmc ? launch(tp_reduce_norm_kernel<NV, false, true>, grid, block, 0, st, a)   \
                            : launch(tp_reduce_norm_kernel<NV, false, false>, grid, block, 0, st, a)))
  if (nv <= 1) E2H_GO(1);
  if (nv == 2) E2H_GO(2);
  E2H_GO(4);
#undef E2H_GO
}

static void tp_fill_ptrs(TpPtrs& dst, const void* const* src, int n) {
  for (int i = 0; i < 8; ++i)
    dst.p[i] = (i < n && src != nullptr) ? const_cast<void*>(src[i]) : nullptr;
}

// Two-phase form (oneshot = 0):
//   h_out[rows of this rank] = h_in + sum_r parts[r];  xn[every rank][those rows] = rmsnorm * w.
//   part_ptrs / xn_ptrs / flag_b_remote: n device addresses (index = rank). `multicast` bit 0:
//   part_ptrs[0] is the multicast address of the partial buffers (multimem.ld_reduce); bit 1:
//   xn_ptrs[0] is the multicast address of the activation buffers (multimem.st).
// One-shot form (oneshot = 1): all T rows, xn_ptrs[0] is the local activation buffer,
//   flag_b_remote / flag_b are unused.
// Returns 0, a negative argument error, or a cudaError_t.
int e2h_tp_reduce_norm(const void* h_in, void* h_out, const void* weight,
                       const void* const* part_ptrs, const void* const* xn_ptrs,
                       const void* const* flag_b_remote, const int* flag_a, const int* flag_b,
                       int* count, unsigned int* ticket, int n, int rank, int T, int dim,
                       float eps, int multicast, int wait_b, int oneshot, int wait_ms,
                       int* status, void* stream) {
  if (n < 1 || n > 8 || rank < 0 || rank >= n || T < 1 || dim % 8) return -1;
  if (h_out == nullptr || weight == nullptr || count == nullptr || ticket == nullptr) return -2;
  if (!oneshot && flag_b_remote == nullptr) return -2;
  TpReduceArgs a;
  a.h_in = static_cast<const __nv_bfloat16*>(h_in);
  a.h_out = static_cast<__nv_bfloat16*>(h_out);
  a.weight = static_cast<const __nv_bfloat16*>(weight);
  tp_fill_ptrs(a.parts, part_ptrs, n);
  tp_fill_ptrs(a.xn, xn_ptrs, n);
  tp_fill_ptrs(a.flag_b_remote, flag_b_remote, n);
  tp_fill_ptrs(a.flag_a_remote, nullptr, 0);
  a.flag_a = flag_a;
  a.flag_b = flag_b;
  a.count = count;
  a.ticket = ticket;
  a.status = status;
  a.wait_cycles = (long long)(wait_ms < 1 ? 1 : wait_ms) * 2000000LL;
  a.n = n;
  a.rank = rank;
  a.dim = dim;
  a.row0 = oneshot ? 0 : (int)((long long)rank * T / n);
  a.rows = oneshot ? T : (int)((long long)(rank + 1) * T / n) - a.row0;
  a.wait_b = oneshot ? 0 : wait_b;
  a.signal_b = oneshot ? 0 : 1;
  a.n_xn = oneshot ? 1 : n;
  a.do_reduce = 1;
  a.do_norm = 1;
  a.self_signal = 0;
  a.h_compact = 0;
  a.eps = eps;
  return tp_rows_launch(a, (multicast & 1) != 0, !oneshot && (multicast & 2) != 0, stream);
}

// The sequence-parallel collectives of training over the same kernel and protocol, by token
// rows (rank r owns rows [r*T/n, (r+1)*T/n)); `ops` picks the stages:
//   bit 0  reduce   sum of every rank's partial (+ h_in, the residual) for the owned rows, i.e.
//                   the reduce-scatter after a row-parallel GEMM (models/tp.py:396-405, :774 of
//                   the reference); without it the rows are h_in as it is
//   bit 1  norm     the rows that go out are rmsnorm(rows) * weight instead of the rows
//   bit 2  gather   write the outgoing rows into every rank's activation buffer and hand-shake,
//                   i.e. the all-gather before a column-parallel GEMM (models/tp.py:375-393, :750)
//   bit 3  barrier  no producer kernel raises flag A for this use: the kernel raises it itself
//                   on start and waits for all ranks (needed by a gather that follows no reduce)
//   bit 4  compact  h_in / h_out hold the owned rows only
// h_out (owned rows, optional) receives the summed rows before any normalisation.
int e2h_tp_rows(int ops, const void* h_in, void* h_out, const void* weight,
                const void* const* part_ptrs, const void* const* xn_ptrs,
                const void* const* flag_a_remote, const void* const* flag_b_remote,
                const int* flag_a, const int* flag_b, int* count, unsigned int* ticket, int n,
                int rank, int T, int dim, float eps, int multicast, int wait_b, int wait_ms,
                int* status, void* stream) {
  const bool reduce = ops & 1, norm = ops & 2, gather = ops & 4, barrier = ops & 8;
  if (n < 1 || n > 8 || rank < 0 || rank >= n || T < 1 || dim % 8) return -1;
  if (count == nullptr || ticket == nullptr || flag_a == nullptr) return -2;
  if (reduce && part_ptrs == nullptr) return -2;
  if (norm && weight == nullptr) return -2;
  if (gather && (xn_ptrs == nullptr || flag_b_remote == nullptr || flag_b == nullptr)) return -2;
  if (barrier && flag_a_remote == nullptr) return -2;
  if (!reduce && h_in == nullptr) return -2;
  if (!gather && h_out == nullptr) return -2;
  TpReduceArgs a;
  a.h_in = static_cast<const __nv_bfloat16*>(h_in);
  a.h_out = static_cast<__nv_bfloat16*>(h_out);
  a.weight = static_cast<const __nv_bfloat16*>(weight);
  tp_fill_ptrs(a.parts, part_ptrs, n);
  tp_fill_ptrs(a.xn, xn_ptrs, n);
  tp_fill_ptrs(a.flag_b_remote, flag_b_remote, n);
  tp_fill_ptrs(a.flag_a_remote, flag_a_remote, n);
  a.flag_a = flag_a;
  a.flag_b = flag_b;
  a.count = count;
  a.ticket = ticket;
  a.status = status;
  a.wait_cycles = (long long)(wait_ms < 1 ? 1 : wait_ms) * 2000000LL;
  a.n = n;
  a.rank = rank;
  a.dim = dim;
  a.row0 = (int)((long long)rank * T / n);
  a.rows = (int)((long long)(rank + 1) * T / n) - a.row0;
  a.wait_b = gather ? wait_b : 0;
  a.signal_b = gather ? 1 : 0;
  a.n_xn = gather ? n : 0;
  a.do_reduce = reduce ? 1 : 0;
  a.do_norm = norm ? 1 : 0;
  a.self_signal = barrier ? 1 : 0;
  a.h_compact = (ops & 16) ? 1 : 0;
  a.eps = eps;
  return tp_rows_launch(a, reduce && (multicast & 1) != 0, gather && (multicast & 2) != 0,
                        stream);
}

int e2h_tp_embed_partial(const int* tokens, const void* table, int v0, int rows_local, void* part,
                         int T, int dim, const void* const* flag_a_remote, int n,
                         unsigned int* ticket, void* stream) {
  // n == -1: flag_a_remote[0] is the multicast address of the flag word
  if (dim % 8 || n == 0 || n < -1 || n > 8 || T < 1) return -1;
  TpPtrs f;
  const int n_ptr = n < 0 ? 1 : n;
  for (int i = 0; i < 8; ++i) f.p[i] = i < n_ptr ? const_cast<void*>(flag_a_remote[i]) : nullptr;
  return (int)launch(tp_embed_partial_kernel, dim3(T), dim3(128), 0,
                     static_cast<cudaStream_t>(stream), tokens,
                     static_cast<const __nv_bfloat16*>(table), v0, rows_local,
                     static_cast<__nv_bfloat16*>(part), dim, f, n, ticket);
}

int e2h_tp_gather_logits(const void* const* shard_ptrs, int n, int B, int vs, float* out,
                         long long ldo, const int* flag_a, int* count, unsigned int* ticket,
                         int wait_ms, int* status, void* stream) {
  if (n < 1 || n > 8 || B < 1 || vs < 1) return -1;
  TpPtrs s;
  bool al16 = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  bool al8 = (reinterpret_cast<uintptr_t>(out) & 7) == 0;
  for (int i = 0; i < 8; ++i) {
    s.p[i] = i < n ? const_cast<void*>(shard_ptrs[i]) : nullptr;
    al16 = al16 && (reinterpret_cast<uintptr_t>(s.p[i]) & 15) == 0;
    al8 = al8 && (reinterpret_cast<uintptr_t>(s.p[i]) & 7) == 0;
  }
  const long long cycles = (long long)(wait_ms < 1 ? 1 : wait_ms) * 2000000LL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(B, n), block(256);
#define E2H_GO(VW)                                                                           \
  return (int)launch(tp_gather_logits_kernel<VW>, grid, block, 0, st, s, n, B, vs, out, ldo, \
                     flag_a, count, ticket, status, cycles)
  if (al16 && vs % 4 == 0 && ldo % 4 == 0) E2H_GO(4);
  if (al8 && vs % 2 == 0 && ldo % 2 == 0) E2H_GO(2);
  E2H_GO(1);
#undef E2H_GO
}

}  // extern "C"
