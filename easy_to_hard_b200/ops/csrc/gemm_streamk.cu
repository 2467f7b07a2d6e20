// Work-split ("stream-K") bf16 GEMM for skinny token counts (decode) on sm_100a.
//
// A decode GEMM streams the weight once and has few output tiles (96 for the fused QKV
// projection of a 7B model, 86 for the gated MLP), so a tile-per-CTA grid leaves a third of the
// 148 SMs without a weight stream. Here the work is cut into units of (feature tile, k-group):
// the units are dealt out evenly and contiguously over one CTA per SM, so a CTA works on the tail
// of one tile and the head of the next. A tile whose k range is shared by several CTAs is finished
// by whichever of them arrives last: the others park their fp32 partial tile in a workspace
// (L2-resident), the last one sums the partials in slot order (bitwise reproducible) together with
// its own accumulator and runs the fused epilogue.
//
//   * warp 0: TMA producer (3-D boxes: `kps` 64-wide k-blocks per pipeline stage, 128-byte swizzle)
//   * warp 1: one thread issues tcgen05.mma (M = 128 features, N = token tile) into one of two
//             accumulator buffers in tensor memory, so the epilogue of a segment overlaps the
//             k-loop of the next
//   * warps 2..5: epilogue (tcgen05.ld, partial-tile exchange, fused epilogue)
//
// The CTA takes at most half of an SM's shared memory and tensor memory: with programmatic
// dependent launch the next GEMM of the stream becomes resident next to this one and prefetches
// its first weight tiles (weights are never written by a preceding kernel of a decode step)
// before it waits for this kernel's results, which hides launch, prologue, pipeline fill and
// epilogue of back-to-back GEMMs behind each other's weight streams.
//
// Every wait is bounded; a time-out writes a code to p.status, and the CTA still frees its tensor
// memory and returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <string.h>
#include <mutex>

#include "gemm_epilogue.cuh"
#include "gemm_umma.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace e2h {

constexpr int kSkThreads = 192;
constexpr int kSkMaxStages = 12;
constexpr int kSkCtrlBytes = 1024;
constexpr int kSkABytes = 128 * 128;     // 128 features x 64 bf16
constexpr int kSkStatusFull = 111, kSkStatusEmpty = 112, kSkStatusAcc = 113, kSkStatusDrain = 114;

struct SkCtrl {
  uint64_t full[kSkMaxStages];
  uint64_t empty[kSkMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int epi_go;
  int epi_last;
};
static_assert(sizeof(SkCtrl) <= kSkCtrlBytes, "control block too large");

// Units [u0, u1) of CTA `i` when U units are dealt over G CTAs: the first U % G CTAs take one more.
struct SkSplit {
  int q, r;
  __host__ __device__ SkSplit(int U, int G) : q(U / G), r(U % G) {}
  __host__ __device__ int begin(int i) const { return i * q + (i < r ? i : r); }
  __host__ __device__ int owner(int x) const {
    const int big = r * (q + 1);
    return x < big ? x / (q + 1) : r + (x - big) / q;
  }
};

__device__ __forceinline__ void epi_bar_sync() {   // the 128 epilogue threads only
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

template <int BN, bool DUAL>
__global__ void __launch_bounds__(kSkThreads, 2)
umma_gemm_streamk_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmA2,
                         const __grid_constant__ CUtensorMap tmB, const E2hGemmParams p) {
  constexpr int NMAT = DUAL ? 2 : 1;
  constexpr int B_BYTES = BN * 128;
  constexpr int KB_BYTES = kSkABytes * NMAT + B_BYTES;     // one 64-wide k-block of all operands
  constexpr int ACC_COLS = BN * NMAT;
  constexpr int NBUF = (2 * ACC_COLS <= 256) ? 2 : 1;      // accumulator buffers (<= half of TMEM)
  constexpr int TMEM_RAW = NBUF * ACC_COLS;
  constexpr int TMEM_COLS = TMEM_RAW <= 32 ? 32 : TMEM_RAW <= 64 ? 64 : TMEM_RAW <= 128 ? 128 : 256;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  SkCtrl* ctrl = reinterpret_cast<SkCtrl*>(smem);
  uint8_t* tiles = smem + kSkCtrlBytes;
  const int stages = p.stages;
  const int kps = p.kps;
  const int STAGE = kps * KB_BYTES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = blockIdx.x, G = gridDim.x;
  const int gpt = (p.K / 64) / kps;                 // k-groups per feature tile
  const int n_tiles = (p.F + 127) / 128;
  const SkSplit split(n_tiles * gpt, G);
  const int u0 = split.begin(cta), u1 = split.begin(cta + 1);
  const int n_it = u1 - u0;                         // pipeline iterations of this CTA

  volatile int* abort_flag = &ctrl->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctrl->acc_full[b]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty[b]), 4);   // one arrival per epilogue warp
    }
    ctrl->abort_flag = 0;
    ctrl->epi_go = 0;
    ctrl->epi_last = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (DUAL) tma_prefetch_desc(&tmA2);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    const uint64_t pol_a = policy_evict_first();
    // timing experiments (debug_mode bits 4 / 8): leave out the activation / the weight loads
    const bool skip_b = (p.debug_mode & 4) != 0, skip_a = (p.debug_mode & 8) != 0;
    const uint32_t tx_bytes = (skip_a ? 0 : kps * kSkABytes * NMAT) + (skip_b ? 0 : kps * B_BYTES);
    // weights first: the opening stages do not depend on the preceding kernel
    const int n_pre = n_it < stages ? n_it : stages;
    for (int it = 0; it < n_pre; ++it) {
      const int u = u0 + it, tile = u / gpt, g = u - tile * gpt;
      const uint32_t bar = smem_u32(&ctrl->full[it]);
      const uint32_t st = smem_u32(tiles + (size_t)it * STAGE);
      mbar_expect_tx(bar, tx_bytes);
      if (!skip_a) {
        tma_load_3d_hint(st, &tmA, 0, tile * 128, g * kps, bar, pol_a);
        if (DUAL)
          tma_load_3d_hint(st + kps * kSkABytes, &tmA2, 0, tile * 128, g * kps, bar, pol_a);
      }
    }
    pdl_wait_prior();          // activations written by the preceding kernel are visible
    pdl_launch_dependents();   // the next kernel may become resident and prefetch its weights
    for (int it = 0; it < n_pre; ++it) {
      const int u = u0 + it, tile = u / gpt, g = u - tile * gpt;
      if (!skip_b)
        tma_load_3d(smem_u32(tiles + (size_t)it * STAGE) + kps * kSkABytes * NMAT, &tmB, 0, 0,
                    g * kps, smem_u32(&ctrl->full[it]));
    }
    // running counters instead of divisions: this thread is a dependent scalar chain
    int armed = n_pre;
    int s = n_pre % stages;
    uint32_t ph = (n_pre / stages) & 1;
    int tile = (u0 + n_pre) / gpt, g = (u0 + n_pre) - tile * gpt;
    const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
    const uint32_t tiles0 = smem_u32(tiles);
    for (int it = n_pre; it < n_it; ++it) {
      if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, p.status, kSkStatusEmpty)) break;
      const uint32_t bar = full0 + 8 * s;
      const uint32_t st = tiles0 + s * STAGE;
      mbar_expect_tx(bar, tx_bytes);
      if (!skip_a) {
        tma_load_3d_hint(st, &tmA, 0, tile * 128, g * kps, bar, pol_a);
        if (DUAL)
          tma_load_3d_hint(st + kps * kSkABytes, &tmA2, 0, tile * 128, g * kps, bar, pol_a);
      }
      if (!skip_b) tma_load_3d(st + kps * kSkABytes * NMAT, &tmB, 0, 0, g * kps, bar);
      armed = it + 1;
      if (++s == stages) {
        s = 0;
        ph ^= 1;
      }
      if (++g == gpt) {
        g = 0;
        ++tile;
      }
    }
    if (*abort_flag) {   // bounded wait for the copies still in flight into this CTA's smem
      for (int it = (armed > stages ? armed - stages : 0); it < armed; ++it) {
        const long long tq = clock64();
        while (!mbar_try_wait(smem_u32(&ctrl->full[it % stages]), (it / stages) & 1)) {
          if (clock64() - tq > kWaitLimitCycles / 8) {
            if (p.status) atomicCAS(p.status, 0, kSkStatusDrain);
            break;
          }
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- UMMA issuer ----------------
    // Descriptors: high word and base low words once; per instruction only an add on the low
    // word. Stage and phase are running counters (no division in this dependent scalar chain).
    const uint32_t idesc = make_idesc_bf16(128, BN, 0, 0);
    const uint32_t d_hi = sw128_desc_hi(1024);
    const uint32_t a_lo0 = sw128_desc_lo(smem_u32(tiles), 16);
    const uint32_t b_lo0 = sw128_desc_lo(smem_u32(tiles) + kps * kSkABytes * NMAT, 16);
    const uint32_t a2_off = (kps * kSkABytes) >> 4;
    const uint32_t stage_step = STAGE >> 4;
    const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
    bool ok = true;
    int seg = 0, s = 0;
    uint32_t ph = 0, st_lo = 0;
    for (int u = u0; u < u1 && ok; ++seg) {
      const int tile = u / gpt, g_begin = u - tile * gpt;
      const int n_g = min(gpt - g_begin, u1 - u);
      const int buf = seg % NBUF;
      if (seg >= NBUF) {   // the epilogue has drained this buffer (segment seg - NBUF)
        ok = mbar_wait(smem_u32(&ctrl->acc_empty[buf]), ((seg / NBUF) & 1) ^ 1, abort_flag,
                       p.status, kSkStatusAcc);
        if (!ok) break;
        tc_fence_after();
      }
      const uint32_t acc_addr = tmem_base + buf * ACC_COLS;
      uint32_t accf = 0;   // the first instruction of a segment overwrites the accumulator
      for (int g = 0; g < n_g; ++g) {
        ok = mbar_wait(full0 + 8 * s, ph, abort_flag, p.status, kSkStatusFull);
        if (!ok) break;
        tc_fence_after();
        uint32_t a_lo = a_lo0 + st_lo, b_lo = b_lo0 + st_lo;
        for (int kk = 0; kk < kps; ++kk) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_f16_lohi(acc_addr, a_lo + 2 * k, d_hi, b_lo + 2 * k, d_hi, idesc, accf);
            if (DUAL)
              umma_f16_lohi(acc_addr + BN, a_lo + a2_off + 2 * k, d_hi, b_lo + 2 * k, d_hi, idesc,
                            accf);
            accf = 1;
          }
          a_lo += kSkABytes >> 4;
          b_lo += B_BYTES >> 4;
        }
        umma_commit(empty0 + 8 * s);
        if (++s == stages) {
          s = 0;
          st_lo = 0;
          ph ^= 1;
        } else {
          st_lo += stage_step;
        }
      }
      if (ok) umma_commit(smem_u32(&ctrl->acc_full[buf]));
      u += n_g;
    }
  } else if (warp >= 2) {
    // ---------------- epilogue warps ----------------
    const int q = warp & 3;                          // TMEM lane quarter of this warp
    const int row = q * 32 + lane;                   // feature row inside the tile
    const int et = threadIdx.x - 64;                 // 0 .. 127
    const int cols = min(BN, (p.T + 7) & ~7);        // token columns that hold tokens
    pdl_wait_prior();                                // residual, workspace, counters are settled
    int seg = 0;
    for (int u = u0; u < u1; ++seg) {
      const int tile = u / gpt, g_begin = u - tile * gpt;
      const int n_g = min(gpt - g_begin, u1 - u);
      const int buf = seg % NBUF;
      u += n_g;
      if (et == 0)
        ctrl->epi_go = mbar_wait_relaxed(smem_u32(&ctrl->acc_full[buf]), (seg / NBUF) & 1,
                                         abort_flag, p.status, kSkStatusAcc) ? 1 : 0;
      epi_bar_sync();
      const bool go = ctrl->epi_go != 0;
      if (!go) break;                                // uniform over the four warps
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * ACC_COLS + (static_cast<uint32_t>(q * 32) << 16);
      const int first = split.owner(tile * gpt), last = split.owner(tile * gpt + gpt - 1);
      const int nseg = (p.debug_mode & 1) ? 1 : last - first + 1, myslot = cta - first;
      const int f = tile * 128 + row;
      bool finish = true;
      // workspace: [tile][slot][matrix][BN / 4 column groups][128 features] float4: a warp reads
      // and writes 512 contiguous bytes per instruction (feature rows on lanes, 4 token columns
      // per thread)
      constexpr size_t kSlotVec = (size_t)NMAT * (BN / 4) * 128;      // float4 per slot
      const float4* ws_tile =
          reinterpret_cast<const float4*>(p.sk_ws) + (size_t)tile * p.sk_slots * kSlotVec + row;
      if (nseg > 1) {
        float4* mine = reinterpret_cast<float4*>(p.sk_ws) +
                       ((size_t)tile * p.sk_slots + myslot) * kSlotVec + row;
        for (int c = 0; c < cols; c += 8) {
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            float v[8];
            tmem_ld_x8(taddr + m * BN + c, v);
            tmem_ld_wait();
            float4* dst = mine + ((size_t)m * (BN / 4) + c / 4) * 128;
            __stcg(dst, make_float4(v[0], v[1], v[2], v[3]));
            __stcg(dst + 128, make_float4(v[4], v[5], v[6], v[7]));
          }
        }
        __threadfence();
        epi_bar_sync();
        if (et == 0) {
          const unsigned int prev = atomicAdd(p.sk_count + tile, 1u);
          const int is_last = prev == (unsigned int)(nseg - 1);
          if (is_last) p.sk_count[tile] = 0;         // every sharer has arrived: ready for re-use
          ctrl->epi_last = is_last;
        }
        epi_bar_sync();
        finish = ctrl->epi_last != 0;
        if (finish) __threadfence();
      }
      if (p.debug_mode & 2) finish = false;
      if (finish && nseg == 1) {
        for (int c = 0; c < cols; c += 8) {
          float v[8], v2[DUAL ? 8 : 1];
          tmem_ld_x8(taddr + c, v);
          if constexpr (DUAL) tmem_ld_x8(taddr + BN + c, v2);
          tmem_ld_wait();
          epilogue8<DUAL>(p, f, c, v, v2);
        }
      } else if (finish) {
        // 16 token columns at a time; the partials of up to four other CTAs are in flight
        // together (16 float4 per thread) and are added in slot order, this CTA's own
        // accumulator at its own slot: the sum does not depend on who finishes
        for (int c = 0; c < cols; c += 16) {
          const bool two = c + 8 < cols;             // second group of 8 columns holds tokens
          float v[16], v2[DUAL ? 16 : 1];
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            float own[16];
            tmem_ld_x8(taddr + m * BN + c, own);
            if (two) tmem_ld_x8(taddr + m * BN + c + 8, own + 8);
            tmem_ld_wait();
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = 0.f;
            for (int s0 = 0; s0 < nseg; s0 += 4) {
              float4 part[4][4];
#pragma unroll
              for (int ss = 0; ss < 4; ++ss) {
                const int slot = s0 + ss;
                if (slot < nseg && slot != myslot) {
                  const float4* src =
                      ws_tile + (size_t)slot * kSlotVec + ((size_t)m * (BN / 4) + c / 4) * 128;
                  part[ss][0] = __ldcg(src);
                  part[ss][1] = __ldcg(src + 128);
                  if (two) {
                    part[ss][2] = __ldcg(src + 256);
                    part[ss][3] = __ldcg(src + 384);
                  }
                }
              }
#pragma unroll
              for (int ss = 0; ss < 4; ++ss) {
                const int slot = s0 + ss;
                if (slot >= nseg) continue;
                if (slot == myslot) {
#pragma unroll
                  for (int j = 0; j < 16; ++j) acc[j] += own[j];
                } else {
#pragma unroll
                  for (int h = 0; h < 4; ++h) {
                    if (h >= 2 && !two) continue;
                    acc[4 * h + 0] += part[ss][h].x;
                    acc[4 * h + 1] += part[ss][h].y;
                    acc[4 * h + 2] += part[ss][h].z;
                    acc[4 * h + 3] += part[ss][h].w;
                  }
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (m == 0) v[j] = acc[j];
              if constexpr (DUAL) {
                if (m == 1) v2[j] = acc[j];
              }
            }
          }
          epilogue8<DUAL>(p, f, c, v, v2);
          if (two) epilogue8<DUAL>(p, f, c + 8, v + 8, DUAL ? v2 + 8 : v2);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->acc_empty[buf]));
    }
  }

  if (p.n_signal > 0) __threadfence();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (p.n_signal > 0 && threadIdx.x == 0) {
    // the last CTA of the grid tells every tensor-parallel peer that this rank's partial output
    // is complete: one release-add on the flag word it owns in each peer's memory
    __threadfence();
    if (atomicAdd(p.ticket, 1u) == gridDim.x - 1) {
      *p.ticket = 0;
      __threadfence_system();
      for (int r = 0; r < p.n_signal; ++r) red_release_sys_add(p.signal[r], 1);
    }
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*SkEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                               const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static SkEncodeFn sk_encode_fn() {
  static SkEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<SkEncodeFn>(sym);
  });
  return fn;
}

// K-major bf16 operand [rows, K] (K % 64 == 0) seen as {64, rows, K / 64}: one box
// {64, box_rows, kps} lands as kps consecutive [box_rows x 128 B] tiles, 128-byte swizzle,
// zero fill past the last row.
static int sk_map3d(CUtensorMap* m, const void* base, long long K, long long rows, long long ld,
                    int box_rows, int kps) {
  SkEncodeFn fn = sk_encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(K / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128u};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, (cuuint32_t)kps};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

static int sk_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

template <int BN, bool DUAL>
static int sk_launch(const E2hGemmParams& p, int grid, size_t smem, const CUtensorMap& ta,
                     const CUtensorMap& ta2, const CUtensorMap& tb, cudaStream_t stream) {
  auto kern = umma_gemm_streamk_kernel<BN, DUAL>;
  static size_t configured = 0;  // per instantiation
  if (smem > configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kSkThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  if (p.pdl || g_pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return (int)cudaLaunchKernelEx(&cfg, kern, ta, ta2, tb, p);
}

}  // namespace e2h

extern "C" int e2h_gemm_streamk(const E2hGemmParams* pp, void* stream_v) {
  using namespace e2h;
  E2hGemmParams p = *pp;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (p.F <= 0 || p.T <= 0 || p.K <= 0) return -1;
  if (p.bn != 32 && p.bn != 64 && p.bn != 128) return -2;
  if (p.T > p.bn) return -3;                                  // one token tile
  if ((p.K % 64) != 0 || p.a_mn_major || p.b_mn_major || p.a_tiled) return -4;
  if (p.dual && p.a2 == nullptr) return -5;
  if ((p.lda % 8) || (p.ldb % 8) || (p.dual && (p.lda2 % 8))) return -6;
  if (((uintptr_t)p.a & 15) || ((uintptr_t)p.b & 15) || (p.dual && ((uintptr_t)p.a2 & 15)))
    return -7;
  const int kb_total = p.K / 64;
  const int nmat = p.dual ? 2 : 1;
  const int kb_bytes = kSkABytes * nmat + p.bn * 128;
  const int budget = (p.sk_smem_kb > 0 ? p.sk_smem_kb : 112) * 1024 - 2048;
  // k-blocks per stage: as asked (default 2) if it divides the k-blocks and leaves two stages
  int kps = p.kps > 0 ? p.kps : 2;
  while (kps > 1 && ((kb_total % kps) != 0 || budget / (kps * kb_bytes) < 2)) --kps;
  p.kps = kps;
  int stages = budget / (kps * kb_bytes);
  if (stages > kSkMaxStages) stages = kSkMaxStages;
  if (p.stages > 0 && p.stages < stages) stages = p.stages;
  if (stages < 1) return -8;
  p.stages = stages;

  const int n_tiles = (p.F + 127) / 128;
  const int gpt = kb_total / kps;
  const long long units = (long long)n_tiles * gpt;
  int grid = p.sk_ctas > 0 ? p.sk_ctas : sk_sm_count();
  if (grid > units) grid = (int)units;
  const int q = (int)(units / grid);
  p.sk_slots = (gpt + q - 1) / q + 1;
  const long long need = (long long)n_tiles * p.sk_slots * nmat * p.bn * 128 * 4;
  const bool shared_tiles = (units % grid) != 0 || (q % gpt) != 0;
  if (shared_tiles && (p.sk_ws == nullptr || p.sk_count == nullptr || need > p.sk_ws_bytes ||
                       n_tiles > p.sk_count_len))
    return -13;
  if (p.n_signal > 0 && p.ticket == nullptr) return -14;

  CUtensorMap ta, ta2, tb;
  int r = sk_map3d(&ta, p.a, p.K, p.F, p.lda, 128, kps);
  if (r) return r;
  if (p.dual) {
    r = sk_map3d(&ta2, p.a2, p.K, p.F, p.lda2, 128, kps);
    if (r) return r;
  } else {
    ta2 = ta;
  }
  r = sk_map3d(&tb, p.b, p.K, p.T, p.ldb, p.bn, kps);
  if (r) return r;
  const size_t smem = 1024 + kSkCtrlBytes + (size_t)stages * kps * kb_bytes;

#define E2H_SK(BN_, DUAL_) return sk_launch<BN_, DUAL_>(p, grid, smem, ta, ta2, tb, stream)
  if (p.dual) {
    if (p.bn == 32) E2H_SK(32, true);
    if (p.bn == 64) E2H_SK(64, true);
    E2H_SK(128, true);
  } else {
    if (p.bn == 32) E2H_SK(32, false);
    if (p.bn == 64) E2H_SK(64, false);
    E2H_SK(128, false);
  }
#undef E2H_SK
}
