// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   * operands are staged into shared memory by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle,
//     no cluster multicast) through a ring of `stages` buffers guarded by full/empty mbarriers;
//   * one thread issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = 64/128/256) with the
//     fp32 accumulator in tensor memory; tcgen05.commit releases the stage and, at the end,
//     signals the epilogue;
//   * four epilogue warps read the accumulator with tcgen05.ld (warp w owns TMEM lanes
//     32*(w%4)..+31, i.e. one output feature per thread) and apply the fused epilogue
//     (plain store, SwiGLU on a dual accumulator, RoPE + KV-cache scatter, residual add, ...);
//   * split-K runs as a thread-block cluster along z: every CTA accumulates its K slice in its
//     own TMEM, then the cluster does a reduce-scatter over token columns through distributed
//     shared memory, so each CTA finishes (and runs the epilogue for) its own column slice.
//     That is what keeps all 148 SMs streaming weights when a decode GEMM has few tiles.
//
// All waits are bounded (see ptx.cuh); a time-out writes a code to p.status and the CTA still
// reaches every barrier, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdio.h>
#include <string.h>
#include <mutex>

#include "gemm_umma.cuh"
#include "ptx.cuh"

namespace e2h {

constexpr int kTileF = 128;       // features per tile = TMEM lanes = UMMA M
constexpr int kTileK = 64;        // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kMaxStages = 12;
constexpr int kCtrlBytes = 1024;  // barriers + tmem holder + abort flag live in the first KiB

struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Ctrl) <= kCtrlBytes, "control block too large");

template <int BN, bool DUAL>
struct SmemPlan {
  static constexpr int a_bytes = kTileF * kTileK * 2;  // 16 KiB
  static constexpr int b_bytes = BN * kTileK * 2;
  static constexpr int stage_bytes = a_bytes * (DUAL ? 2 : 1) + b_bytes;
  static constexpr int acc_cols = BN * (DUAL ? 2 : 1);
  static constexpr int tmem_cols = acc_cols <= 32 ? 32 : acc_cols <= 64 ? 64 : acc_cols <= 128 ? 128 : acc_cols <= 256 ? 256 : 512;
};

// Exchange buffer for the cluster reduce: (S-1) sender slots x (BN/S) columns x 128 lanes fp32.
__host__ __device__ inline int xchg_bytes(int bn, int splitk, int dual) {
  if (splitk <= 1) return 0;
  return (splitk - 1) * (bn / splitk) * kTileF * 4 * (dual ? 2 : 1);
}

struct EpiCtx {
  int f;        // global feature index of this thread (may be >= F: masked)
  int t0;       // first token column of the 8-column group
};

// Applies the epilogue to 8 consecutive token columns of one feature.
template <bool DUAL>
__device__ __forceinline__ void epilogue8(const E2hGemmParams& p, int f, int t0, float* v,
                                          float* v2) {
  const bool f_ok = f < p.F;
  if (p.scale != nullptr) {
    const float s = f_ok ? p.scale[f] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= s;
  }
  switch (p.epi) {
    case E2H_EPI_STORE_BF16: {
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = t0 + j;
        if (f_ok && t < p.T) out[(long long)t * p.ldo + f] = __float2bfloat16_rn(v[j]);
      }
    } break;
    case E2H_EPI_STORE_F32: {
      float* out = static_cast<float*>(p.out);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = t0 + j;
        if (f_ok && t < p.T) out[(long long)t * p.ldo + f] = v[j];
      }
    } break;
    case E2H_EPI_RESIDUAL: {
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
      const __nv_bfloat16* res = static_cast<const __nv_bfloat16*>(p.aux);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = t0 + j;
        if (f_ok && t < p.T) {
          const long long o = (long long)t * p.ldo + f;
          out[o] = __float2bfloat16_rn(bf16_round(v[j]) + __bfloat162float(res[o]));
        }
      }
    } break;
    case E2H_EPI_SWIGLU: {
      if constexpr (DUAL) {
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int t = t0 + j;
          if (f_ok && t < p.T) {
            const float g = bf16_round(v[j]);
            const float u = bf16_round(v2[j]);
            out[(long long)t * p.ldo + f] = __float2bfloat16_rn(bf16_round(silu(g)) * u);
          }
        }
      }
    } break;
    case E2H_EPI_DUAL_STORE: {
      if constexpr (DUAL) {
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
        __nv_bfloat16* out2 = static_cast<__nv_bfloat16*>(p.out2);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int t = t0 + j;
          if (f_ok && t < p.T) {
            out[(long long)t * p.ldo + f] = __float2bfloat16_rn(v[j]);
            out2[(long long)t * p.ldo2 + f] = __float2bfloat16_rn(v2[j]);
          }
        }
      }
    } break;
    case E2H_EPI_ROWMAJOR_F32_ACC: {
      float* out = static_cast<float*>(p.out);
      if (f_ok) {
        float* row = out + (long long)f * p.ldo;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int t = t0 + j;
          if (t < p.T) row[t] = p.accumulate ? row[t] + v[j] : v[j];
        }
      }
    } break;
    case E2H_EPI_ROWMAJOR_BF16: {
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
      if (f_ok) {
        __nv_bfloat16* row = out + (long long)f * p.ldo;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int t = t0 + j;
          if (t < p.T) row[t] = __float2bfloat16_rn(v[j]);
        }
      }
    } break;
    case E2H_EPI_ROPE_KV: {
      // Feature f belongs to head f / head_dim of the fused [q; k; v] projection. RoPE rotates
      // the interleaved pair (2i, 2i+1): the partner value sits in the neighbouring lane.
      const int D = p.head_dim;
      const int head = f / D;
      const int d = f - head * D;
      const bool is_q = head < p.n_head;
      const bool is_k = !is_q && head < p.n_head + p.n_kv;
      const bool is_v = !is_q && !is_k;
      const __nv_bfloat16* freqs = static_cast<const __nv_bfloat16*>(p.freqs);
      const int pos0 = *p.pos_base;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = t0 + j;
        const float x = bf16_round(v[j]);
        const float partner = __shfl_xor_sync(0xffffffffu, x, 1);
        if (!(f_ok && t < p.T)) continue;
        const int b = t / p.sq;
        const int s = t - b * p.sq;
        const int pos = pos0 + s;
        float y = x;
        if (!is_v) {
          const long long fo = ((long long)pos * (D / 2) + (d >> 1)) * 2;
          const float c = __bfloat162float(freqs[fo]);
          const float sn = __bfloat162float(freqs[fo + 1]);
          y = (d & 1) ? (x * c + partner * sn) : (x * c - partner * sn);
        }
        const __nv_bfloat16 yb = __float2bfloat16_rn(y);
        if (is_q) {
          static_cast<__nv_bfloat16*>(p.out)[(long long)t * p.ldo + f] = yb;
        } else {
          const int hk = is_k ? head - p.n_head : head - p.n_head - p.n_kv;
          __nv_bfloat16* cache = static_cast<__nv_bfloat16*>(is_k ? p.kcache : p.vcache);
          if (pos < p.smax)
            cache[(((long long)b * p.n_kv + hk) * p.smax + pos) * D + d] = yb;
        }
      }
    } break;
    default:
      break;
  }
}

template <int BN, bool DUAL>
__global__ void __launch_bounds__(kThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
                 const __grid_constant__ CUtensorMap tmB, const E2hGemmParams p) {
  using Plan = SmemPlan<BN, DUAL>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: round up to the swizzle atom
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem);
  uint8_t* tiles = smem + kCtrlBytes;
  const int stages = p.stages;
  float* xchg = reinterpret_cast<float*>(tiles + (size_t)stages * Plan::stage_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = p.splitk;
  const int rank = (S > 1) ? (int)cluster_ctarank() : 0;
  const int f0 = blockIdx.x * kTileF;
  const int t0 = blockIdx.y * BN;

  const int kb_total = (p.K + kTileK - 1) / kTileK;
  const int kb_begin = (int)((long long)rank * kb_total / S);
  const int kb_end = (int)((long long)(rank + 1) * kb_total / S);
  const int n_kb = kb_end - kb_begin;

  volatile int* abort_flag = &ctrl->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    mbar_init(smem_u32(&ctrl->tmem_full), 1);
    ctrl->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (DUAL) tma_prefetch_desc(&tmA2);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), Plan::tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  if (S > 1) cluster_sync_all();  // every CTA of the cluster is resident before DSMEM traffic

  if (p.pdl) pdl_wait_prior();    // inputs written by the previous kernel are visible from here

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    const uint64_t pol_a = policy_evict_first();
    int armed = 0;
    for (int it = 0; it < n_kb; ++it) {
      const int s = it % stages;
      const uint32_t ph = (it / stages) & 1;
      if (!mbar_wait(smem_u32(&ctrl->empty[s]), ph ^ 1, abort_flag, p.status,
                     kStatusTimeoutEmpty))
        break;
      const uint32_t bar = smem_u32(&ctrl->full[s]);
      mbar_expect_tx(bar, Plan::stage_bytes);
      uint8_t* st = tiles + (size_t)s * Plan::stage_bytes;
      const int k0 = (kb_begin + it) * kTileK;
      const uint32_t a_dst = smem_u32(st);
      if (!p.a_mn_major) {
        tma_load_2d_hint(a_dst, &tmA, k0, f0, bar, pol_a);
        if (DUAL) tma_load_2d_hint(a_dst + Plan::a_bytes, &tmA2, k0, f0, bar, pol_a);
      } else {
        tma_load_2d(a_dst, &tmA, f0, k0, bar);
        tma_load_2d(a_dst + 8192, &tmA, f0 + 64, k0, bar);
      }
      const uint32_t b_dst = a_dst + Plan::a_bytes * (DUAL ? 2 : 1);
      if (!p.b_mn_major) {
        tma_load_2d(b_dst, &tmB, k0, t0, bar);
      } else {
#pragma unroll
        for (int c = 0; c < BN / 64; ++c) tma_load_2d(b_dst + c * 8192, &tmB, t0 + c * 64, k0, bar);
      }
      armed = it + 1;
    }
    // On an abort, wait (bounded) for the copies already in flight into this CTA's smem.
    if (*abort_flag) {
      for (int it = (armed > stages ? armed - stages : 0); it < armed; ++it) {
        const long long tq = clock64();
        while (!mbar_try_wait(smem_u32(&ctrl->full[it % stages]), (it / stages) & 1)) {
          if (clock64() - tq > kWaitLimitCycles / 8) break;
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- UMMA issuer ----------------
    const uint32_t idesc = make_idesc_bf16(kTileF, BN, p.a_mn_major, p.b_mn_major);
    const uint32_t a_kstep = p.a_mn_major ? 2048u : 32u;
    const uint32_t b_kstep = p.b_mn_major ? 2048u : 32u;
    const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u;
    const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u;
    bool ok = true;
    for (int it = 0; it < n_kb && ok; ++it) {
      const int s = it % stages;
      const uint32_t ph = (it / stages) & 1;
      ok = mbar_wait(smem_u32(&ctrl->full[s]), ph, abort_flag, p.status, kStatusTimeoutFull);
      if (!ok) break;
      tc_fence_after();
      const uint32_t a_base = smem_u32(tiles + (size_t)s * Plan::stage_bytes);
      const uint32_t b_base = a_base + Plan::a_bytes * (DUAL ? 2 : 1);
#pragma unroll
      for (int k = 0; k < kTileK / kUmmaK; ++k) {
        const uint64_t bdesc = make_sw128_desc(b_base + k * b_kstep, b_lbo, 1024);
        const uint64_t adesc = make_sw128_desc(a_base + k * a_kstep, a_lbo, 1024);
        const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
        umma_f16(tmem_base, adesc, bdesc, idesc, acc);
        if (DUAL) {
          const uint64_t a2desc =
              make_sw128_desc(a_base + Plan::a_bytes + k * a_kstep, a_lbo, 1024);
          umma_f16(tmem_base + BN, a2desc, bdesc, idesc, acc);
        }
      }
      umma_commit(smem_u32(&ctrl->empty[s]));  // stage reusable once these UMMAs have read it
    }
    umma_commit(smem_u32(&ctrl->tmem_full));
  }

  // ---------------- epilogue warps: accumulator -> registers ----------------
  const bool is_epi = warp >= 2;
  const int q = warp & 3;                 // TMEM lane quarter this warp may touch
  const int lane_row = q * 32 + lane;
  const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
  const int slice = BN / S;               // token columns this CTA finishes
  bool acc_ok = true;
  if (is_epi) {
    acc_ok = mbar_wait(smem_u32(&ctrl->tmem_full), 0, abort_flag, p.status,
                       kStatusTimeoutTmemFull);
    tc_fence_after();
    if (S > 1 && acc_ok && n_kb > 0) {
      // reduce-scatter: send the columns owned by each peer into that peer's exchange buffer
      for (int peer = 0; peer < S; ++peer) {
        if (peer == rank) continue;
        const int slot = rank < peer ? rank : rank - 1;
        for (int c = 0; c < slice; c += 8) {
          float v[8];
          tmem_ld_x8(taddr + peer * slice + c, v);
          tmem_ld_wait();
          const uint32_t base = smem_u32(xchg) + ((slot * slice + c) * kTileF + lane_row) * 4;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_cluster_f32(mapa_shared(base + j * kTileF * 4, peer), v[j]);
          if (DUAL) {
            tmem_ld_x8(taddr + BN + peer * slice + c, v);
            tmem_ld_wait();
            const uint32_t base2 = base + (S - 1) * slice * kTileF * 4;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              st_cluster_f32(mapa_shared(base2 + j * kTileF * 4, peer), v[j]);
          }
        }
      }
    }
  }
  __syncwarp();
  if (S > 1) cluster_sync_all();

  if (p.pdl) pdl_launch_dependents();

  if (is_epi && acc_ok) {
    const int c_begin = rank * slice;
    const int f = f0 + lane_row;
    for (int c = 0; c < slice; c += 8) {
      float v[8], v2[8];
      if (n_kb > 0) {
        tmem_ld_x8(taddr + c_begin + c, v);
        if (DUAL) tmem_ld_x8(taddr + BN + c_begin + c, v2);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = v2[j] = 0.f;
      }
      if (S > 1) {
        for (int slot = 0; slot < S - 1; ++slot) {
          const float* src = xchg + (size_t)(slot * slice + c) * kTileF + lane_row;
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += src[j * kTileF];
          if (DUAL) {
            const float* src2 = src + (size_t)(S - 1) * slice * kTileF;
#pragma unroll
            for (int j = 0; j < 8; ++j) v2[j] += src2[j * kTileF];
          }
        }
      }
      epilogue8<DUAL>(p, f, t0 + c_begin + c, v, v2);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Plan::tmem_cols);
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows `ld` elements apart,
// box = 64 x box_rows, 128-byte swizzle, zero fill out of bounds.
static int make_map(CUtensorMap* m, const void* base, long long inner, long long outer,
                    long long ld, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

template <int BN, bool DUAL>
static int launch(const E2hGemmParams& p, const CUtensorMap& ta, const CUtensorMap& ta2,
                  const CUtensorMap& tb, cudaStream_t stream) {
  using Plan = SmemPlan<BN, DUAL>;
  const size_t smem = 1024 /*alignment slack*/ + kCtrlBytes + (size_t)p.stages * Plan::stage_bytes +
                      xchg_bytes(BN, p.splitk, DUAL);
  if (smem > 227 * 1024) return -12;
  auto kern = umma_gemm_kernel<BN, DUAL>;
  static size_t configured = 0;  // per instantiation
  if (smem > configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((p.F + kTileF - 1) / kTileF, (p.T + BN - 1) / BN, p.splitk);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (p.splitk > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 1;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = p.splitk;
    ++na;
  }
  if (p.pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return (int)cudaLaunchKernelEx(&cfg, kern, ta, ta2, tb, p);
}

}  // namespace e2h

extern "C" int e2h_gemm_umma(const E2hGemmParams* pp, void* stream_v) {
  using namespace e2h;
  E2hGemmParams p = *pp;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (p.F <= 0 || p.T <= 0 || p.K <= 0) return -1;
  if (p.bn != 64 && p.bn != 128 && p.bn != 256) return -2;
  if (p.splitk < 1 || p.splitk > 8 || (p.bn % (p.splitk * 8)) != 0) return -3;
  const int kb_total = (p.K + kTileK - 1) / kTileK;
  if (kb_total < p.splitk) return -4;
  if (p.dual && (p.a_mn_major || p.a2 == nullptr)) return -5;
  if ((p.lda % 8) || (p.ldb % 8) || (p.dual && (p.lda2 % 8))) return -6;  // 16-byte strides for TMA
  if (((uintptr_t)p.a & 15) || ((uintptr_t)p.b & 15)) return -7;
  const int stage_bytes = 16384 * (p.dual ? 2 : 1) + p.bn * 128;
  const int budget = 227 * 1024 - 2048 - xchg_bytes(p.bn, p.splitk, p.dual);
  int max_stages = budget / stage_bytes;
  if (max_stages > kMaxStages) max_stages = kMaxStages;
  if (p.stages <= 0 || p.stages > max_stages) p.stages = max_stages;
  if (p.stages < 1) return -8;
  if (p.stages > kb_total) p.stages = kb_total < 1 ? 1 : kb_total;

  CUtensorMap ta, ta2, tb;
  int r;
  if (!p.a_mn_major)
    r = make_map(&ta, p.a, p.K, p.F, p.lda, kTileF);
  else
    r = make_map(&ta, p.a, p.F, p.K, p.lda, 64);
  if (r) return r;
  if (p.dual) {
    r = make_map(&ta2, p.a2, p.K, p.F, p.lda2, kTileF);
    if (r) return r;
  } else {
    ta2 = ta;
  }
  if (!p.b_mn_major)
    r = make_map(&tb, p.b, p.K, p.T, p.ldb, p.bn);
  else
    r = make_map(&tb, p.b, p.T, p.K, p.ldb, 64);
  if (r) return r;

#define E2H_DISPATCH(BN_, DUAL_) return launch<BN_, DUAL_>(p, ta, ta2, tb, stream)
  if (p.dual) {
    if (p.bn == 64) E2H_DISPATCH(64, true);
    if (p.bn == 128) E2H_DISPATCH(128, true);
    E2H_DISPATCH(256, true);
  } else {
    if (p.bn == 64) E2H_DISPATCH(64, false);
    if (p.bn == 128) E2H_DISPATCH(128, false);
    E2H_DISPATCH(256, false);
  }
#undef E2H_DISPATCH
}
