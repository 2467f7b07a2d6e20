// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   * operands are staged into shared memory by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle,
//     no cluster multicast) through a ring of `stages` buffers guarded by full/empty mbarriers;
//   * one thread issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = 64/128/256) with the
//     fp32 accumulator in tensor memory; tcgen05.commit releases the stage and, at the end,
//     signals the epilogue;
//   * eight epilogue warps read the accumulator with tcgen05.ld (warp w owns TMEM lanes
//     32*(w%4)..+31, i.e. one output feature per thread; the two warps of a lane quarter split
//     the token columns: the epilogue is bound by instruction issue, one warp per scheduler
//     leaves it half idle) and apply the fused epilogue (plain store, SwiGLU on a dual
//     accumulator, RoPE + KV-cache scatter, residual add, ...);
//   * the feature tile may be lower than the 128 rows of the instruction (p.th rows, a multiple
//     of 8): the TMA box then brings only th weight rows per k-block, the MMA still spans 128
//     lanes (the lanes past th multiply whatever follows in shared memory and are never read
//     back), and the grid has ceil(F / th) feature tiles. A skinny GEMM is a weight stream, so
//     what counts is that (nearly) every SM streams an equal share: th is chosen on the host
//     to make the tile count fit the 148 SMs instead of leaving a third of them idle;
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

#include "gemm_epilogue.cuh"
#include "gemm_umma.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace e2h {

constexpr int kTileF = 128;       // default features per tile = TMEM lanes = UMMA M (64 also supported)
constexpr int kTileK = 64;        // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 320;        // producer warp, MMA warp, eight epilogue warps
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

// Accumulation chains: rotating the k-steps over several accumulators was measured and does
// not change the k-loop time (dependent tcgen05.mma on one accumulator pipeline back to back),
// so a single chain is used; the indexing below stays general.
template <int BN, bool DUAL>
struct Chains {
  static constexpr int value = 1;
};

template <int BN, bool DUAL, int TF>
struct SmemPlan {
  static constexpr int a_bytes = TF * kTileK * 2;  // 16 KiB (8 KiB for 64-feature tiles)
  static constexpr int b_bytes = BN * kTileK * 2;
  static constexpr int stage_bytes = a_bytes * (DUAL ? 2 : 1) + b_bytes;
  static constexpr int nacc = Chains<BN, DUAL>::value;
  static constexpr int acc_cols = BN * (DUAL ? 2 : 1) * nacc;
  static constexpr int tmem_cols = acc_cols <= 32 ? 32 : acc_cols <= 64 ? 64 : acc_cols <= 128 ? 128 : acc_cols <= 256 ? 256 : 512;
};

// Exchange buffer for the cluster reduce: (S-1) sender slots x (BN/S) columns x 128 lanes fp32.
__host__ __device__ inline int xchg_bytes(int bn, int splitk, int dual, int tf) {
  if (splitk <= 1) return 0;
  return (splitk - 1) * (bn / splitk) * tf * 4 * (dual ? 2 : 1);
}

template <int BN, bool DUAL, int TF>
__global__ void __launch_bounds__(kThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
                 const __grid_constant__ CUtensorMap tmB, const E2hGemmParams p) {
  using Plan = SmemPlan<BN, DUAL, TF>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: round up to the swizzle atom
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem);
  uint8_t* tiles = smem + kCtrlBytes;
  const int stages = p.stages;
  // the stage size follows the tile height (p.th >= 64: the 128-lane MMA then reads at most
  // 8 KiB past a weight tile, which stays inside the same stage's token tiles)
  float* xchg = reinterpret_cast<float*>(
      tiles + (size_t)stages * p.kps *
                  (((TF == 128) ? p.th : TF) * kTileK * 2 * (DUAL ? 2 : 1) + Plan::b_bytes));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = p.splitk;
  const int rank = (S > 1) ? (int)cluster_ctarank() : 0;
  const int TH = (TF == 128) ? p.th : TF;        // weight rows this CTA streams per k-block
  const int a_bytes = TH * kTileK * 2;
  const int stage_bytes = a_bytes * (DUAL ? 2 : 1) + Plan::b_bytes;
  const int f0 = blockIdx.x * TH;
  const int t0 = blockIdx.y * BN;

  const int kb_total = (p.K + kTileK - 1) / kTileK;
  const int kb_begin = (int)((long long)rank * kb_total / S);
  const int kb_end = (int)((long long)(rank + 1) * kb_total / S);
  const int n_kb = kb_end - kb_begin;
  const int kps = p.kps;                          // k blocks per pipeline stage
  const int n_it = (n_kb + kps - 1) / kps;

  volatile int* abort_flag = &ctrl->abort_flag;
  // phase stamps (E2H_PHASE_CLOCK builds): 0 entry, 1 set-up done, 2 producer past its wait for
  // the predecessor, 3 all loads issued, 4 first stage landed, 5 all MMAs issued, 6 accumulator
  // ready, 7 split-K exchange done, 8 values staged, 9 tile written, 10 tensor memory freed
  if (threadIdx.x == 0) E2H_PHASE(p.phase_clock, 0);

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
  if (threadIdx.x == 0) E2H_PHASE(p.phase_clock, 1);

  // Programmatic dependent launch: the next kernel may begin its prologue now. This kernel's
  // own wait for its predecessor is taken per role: the producer first streams the opening
  // weight tiles (weights are never written by a preceding kernel of a PDL chain), the epilogue
  // warps wait before they touch the outputs, the MMA thread touches no global memory.
  pdl_launch_dependents();
  const bool early_weights = kps > 1;
  if (!(warp == 0 && lane == 0 && early_weights) && !(warp == 1 && lane == 0)) pdl_wait_prior();

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    const uint64_t pol_a = policy_evict_first();
    int armed = 0;
    // stage / phase as running counters: this thread is one dependent scalar chain, a division
    // per iteration costs it on the order of a hundred cycles
    int s = 0;
    uint32_t ph = 0;
    const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
    const uint32_t tiles0 = smem_u32(tiles);
    const uint32_t stage_sz = kps * stage_bytes;
    int it0 = 0;
    if (early_weights) {
      // the ring is empty: fill every stage's weight part before waiting for the predecessor,
      // then add the activation part (the stage completes when both have landed)
      const int n_pre = n_it < stages ? n_it : stages;
      for (int it = 0; it < n_pre; ++it) {
        const uint32_t bar = full0 + 8 * it;
        const uint32_t a_dst = tiles0 + it * stage_sz;
        const int kb = kb_begin + it * kps;
        mbar_expect_tx(bar, kps * stage_bytes);
        tma_load_3d_hint(a_dst, &tmA, 0, f0, kb, bar, pol_a);
        if (DUAL) tma_load_3d_hint(a_dst + kps * a_bytes, &tmA2, 0, f0, kb, bar, pol_a);
      }
      pdl_wait_prior();
      E2H_PHASE(p.phase_clock, 2);
      for (int it = 0; it < n_pre; ++it)
        tma_load_3d(tiles0 + it * stage_sz + kps * a_bytes * (DUAL ? 2 : 1), &tmB, 0, t0,
                    kb_begin + it * kps, full0 + 8 * it);
      armed = n_pre;
      it0 = n_pre;
      s = n_pre == stages ? 0 : n_pre;
      ph = n_pre == stages ? 1 : 0;
    }
    for (int it = it0; it < n_it; ++it) {
      if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) break;
      const uint32_t bar = full0 + 8 * s;
      const uint32_t st0 = tiles0 + s * stage_sz;
      if (++s == stages) {
        s = 0;
        ph ^= 1;
      }
      const int kcount = min(kps, n_kb - it * kps);
      if (kps > 1) {
        // one 3-D box per operand brings kps k-blocks (rows x 64 x kps): two TMA instructions
        // per stage instead of 2*kps. The box is always full size (out-of-range k-blocks are
        // zero filled), k-blocks past this CTA's range are loaded but never multiplied.
        const int kb = kb_begin + it * kps;
        const uint32_t a_dst = st0;
        mbar_expect_tx(bar, kps * stage_bytes);
        tma_load_3d_hint(a_dst, &tmA, 0, f0, kb, bar, pol_a);
        if (DUAL) tma_load_3d_hint(a_dst + kps * a_bytes, &tmA2, 0, f0, kb, bar, pol_a);
        tma_load_3d(a_dst + kps * a_bytes * (DUAL ? 2 : 1), &tmB, 0, t0, kb, bar);
        armed = it + 1;
        continue;
      }
      mbar_expect_tx(bar, kcount * stage_bytes);
      for (int kk = 0; kk < kcount; ++kk) {
        const int kb = kb_begin + it * kps + kk;
        const int k0 = kb * kTileK;
        const uint32_t a_dst = st0 + kk * stage_bytes;
        if (p.a_tiled) {
          // tile-major weight: tile (feature tile, k block) is one contiguous TF x 64 block
          const int row = (blockIdx.x * kb_total + kb) * TF;
          tma_load_2d_hint(a_dst, &tmA, 0, row, bar, pol_a);
          if (DUAL) tma_load_2d_hint(a_dst + a_bytes, &tmA2, 0, row, bar, pol_a);
        } else if (!p.a_mn_major) {
          tma_load_2d_hint(a_dst, &tmA, k0, f0, bar, pol_a);
          if (DUAL) tma_load_2d_hint(a_dst + a_bytes, &tmA2, k0, f0, bar, pol_a);
        } else {
          tma_load_2d(a_dst, &tmA, f0, k0, bar);
          if (TF == 128) tma_load_2d(a_dst + 8192, &tmA, f0 + 64, k0, bar);
        }
        const uint32_t b_dst = a_dst + a_bytes * (DUAL ? 2 : 1);
        if (!p.b_mn_major) {
          tma_load_2d(b_dst, &tmB, k0, t0, bar);
        } else {
#pragma unroll
          for (int c = 0; c < BN / 64; ++c)
            tma_load_2d(b_dst + c * 8192, &tmB, t0 + c * 64, k0, bar);
        }
      }
      armed = it + 1;
    }
    E2H_PHASE(p.phase_clock, 3);
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
    const uint32_t idesc = make_idesc_bf16(TF, BN, p.a_mn_major, p.b_mn_major);
    const uint32_t a_kstep = p.a_mn_major ? 2048u : 32u;
    const uint32_t b_kstep = p.b_mn_major ? 2048u : 32u;
    const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u;
    const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u;
    static_assert(Plan::nacc == 1, "one accumulation chain");
    // descriptors: constant high word, base low words once, one add per instruction; stage and
    // phase are running counters (no division in this dependent scalar chain)
    const uint32_t d_hi = sw128_desc_hi(1024);
    const uint32_t a_lo0 = sw128_desc_lo(smem_u32(tiles), a_lbo);
    const uint32_t b_lo0 = sw128_desc_lo(smem_u32(tiles), b_lbo);
    const uint32_t a_ks = a_kstep >> 4, b_ks = b_kstep >> 4;
    const uint32_t a2_off = (kps * a_bytes) >> 4;
    const uint32_t b_off = (kps * a_bytes * (DUAL ? 2 : 1)) >> 4;
    const uint32_t stage_step = (kps * stage_bytes) >> 4;
    const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
    bool ok = true;
    int s = 0;
    uint32_t ph = 0, st_lo = 0, accf = 0;
    for (int it = 0; it < n_it && ok; ++it) {
      ok = mbar_wait(full0 + 8 * s, ph, abort_flag, p.status, kStatusTimeoutFull);
      if (!ok) break;
      if (it == 0) E2H_PHASE(p.phase_clock, 4);
      tc_fence_after();
      const uint32_t e_bar = empty0 + 8 * s;
      const uint32_t cur_lo = st_lo;
      if (++s == stages) {
        s = 0;
        st_lo = 0;
        ph ^= 1;
      } else {
        st_lo += stage_step;
      }
      const int kcount = min(kps, n_kb - it * kps);
      // kps == 1: stage = [A][A2][B]; kps > 1: stage = [A x kps][A2 x kps][B x kps]
      uint32_t a_lo = a_lo0 + cur_lo, b_lo = b_lo0 + cur_lo + b_off;
      for (int kk = 0; kk < kcount; ++kk) {
#pragma unroll
        for (int k = 0; k < kTileK / kUmmaK; ++k) {
          umma_f16_lohi(tmem_base, a_lo + k * a_ks, d_hi, b_lo + k * b_ks, d_hi, idesc, accf);
          if (DUAL)
            umma_f16_lohi(tmem_base + BN, a_lo + a2_off + k * a_ks, d_hi, b_lo + k * b_ks, d_hi,
                          idesc, accf);
          accf = 1;
        }
        a_lo += a_bytes >> 4;
        b_lo += Plan::b_bytes >> 4;
      }
      umma_commit(e_bar);  // stage reusable once these UMMAs have read it
    }
    umma_commit(smem_u32(&ctrl->tmem_full));
    E2H_PHASE(p.phase_clock, 5);
  }

  // ---------------- epilogue warps: accumulator -> registers ----------------
  const bool is_epi = warp >= 2;
  const int q = warp & 3;                 // TMEM lane quarter this warp may touch
  const int half = (warp - 2) >> 2;       // which of the two warps of that quarter (epilogue)
  // M = 128: accumulator row r sits on TMEM lane r. M = 64: row r sits on lane
  // (r / 16) * 32 + r % 16, i.e. only the lower 16 lanes of each warp's quarter hold rows.
  const int lane_row = (TF == 128) ? q * 32 + lane : q * 16 + (lane & 15);
  const bool lane_valid = (TF == 128) ? lane_row < TH : lane < 16;
  const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
  const int slice = BN / S;               // token columns this CTA finishes
  // issue the TMEM load of 8 token columns of accumulator `a` (0, or 1 = second operand of a
  // dual GEMM); the caller waits once for a whole group of loads
  auto issue_acc = [&](int a, int col, float* v) {
    static_assert(Plan::nacc == 1, "epilogue assumes one accumulation chain");
    tmem_ld_x8(taddr + a * BN + col, v);
  };
  bool acc_ok = true;
  if (is_epi) {
    // one lane per warp polls (with back-off); the rest of the warp parks at the syncwarp
    int ok_i = 1;
    if (lane == 0)
      ok_i = mbar_wait_relaxed(smem_u32(&ctrl->tmem_full), 0, abort_flag, p.status,
                               kStatusTimeoutTmemFull) ? 1 : 0;
    ok_i = __shfl_sync(0xffffffffu, ok_i, 0);
    acc_ok = ok_i != 0;
    tc_fence_after();
    if (warp == 2 && lane == 0) E2H_PHASE(p.phase_clock, 6);
    if (S > 1 && acc_ok && n_kb > 0) {
      // reduce-scatter: send the columns owned by each peer into that peer's exchange buffer
      for (int peer = 0; peer < S; ++peer) {
        if (peer == rank) continue;
        const int slot = rank < peer ? rank : rank - 1;
        for (int c = 8 * half; c < slice; c += 16) {   // the quarter's two warps alternate
          float v[8];
          issue_acc(0, peer * slice + c, v);
          tmem_ld_wait();
          const uint32_t base = smem_u32(xchg) + ((slot * slice + c) * TF + lane_row) * 4;
          if (lane_valid) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              st_cluster_f32(mapa_shared(base + j * TF * 4, peer), v[j]);
          }
          if (DUAL) {
            issue_acc(1, peer * slice + c, v);
            tmem_ld_wait();
            const uint32_t base2 = base + (S - 1) * slice * TF * 4;
            if (lane_valid) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                st_cluster_f32(mapa_shared(base2 + j * TF * 4, peer), v[j]);
            }
          }
        }
      }
    }
  }
  __syncwarp();
  if (S > 1) cluster_sync_all();
  if (warp == 2 && lane == 0) E2H_PHASE(p.phase_clock, 7);


  // Staged epilogue: the finished values go through a [tokens][TH] bf16 tile in the (now idle)
  // pipeline buffers and leave with 16-byte accesses; see gemm_epilogue.cuh.
  const bool staged = p.stage_epi != 0;
  __nv_bfloat16* stile = reinterpret_cast<__nv_bfloat16*>(tiles);
  if (is_epi && acc_ok) {
    const int c_begin = rank * slice;
    const int f = lane_valid ? f0 + lane_row : p.F;  // rows past F are masked in the epilogue
    // columns of this warp: with 64 or more, alternate groups of 32; with fewer, the first /
    // second half of the 8-column units
    const int units = slice >> 3;
    int c_first, c_last, c_step;
    if (units >= 8) {
      c_first = 32 * half;
      c_last = slice;
      c_step = 64;
    } else {
      const int lo = units == 1 ? 1 : units >> 1;   // units of warp 0 (warp 1 takes the rest)
      c_first = half ? 8 * lo : 0;
      c_last = half ? slice : 8 * lo;
      c_step = 64;
    }
    RopePre rope;
    if (staged && p.epi == E2H_EPI_ROPE_KV) rope = rope_prepare(p, f);
    for (int c = c_first; c < c_last; c += c_step) {
      // up to 32 columns per round trip to tensor memory
      const int nb = (c_last - c) >= 32 ? 4 : (c_last - c) / 8;
      float v[32], v2[DUAL ? 32 : 1];
      if (n_kb > 0) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          if (b < nb) {
            issue_acc(0, c_begin + c + 8 * b, v + 8 * b);
            if constexpr (DUAL) issue_acc(1, c_begin + c + 8 * b, v2 + 8 * b);
          }
        }
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          v[j] = 0.f;
          if constexpr (DUAL) v2[j] = 0.f;
        }
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        if (b >= nb) continue;
        if (S > 1) {
          for (int slot = 0; slot < S - 1; ++slot) {
            const float* src = xchg + (size_t)(slot * slice + c + 8 * b) * TF + lane_row;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[8 * b + j] += src[j * TF];
            if constexpr (DUAL) {
              const float* src2 = src + (size_t)(S - 1) * slice * TF;
#pragma unroll
              for (int j = 0; j < 8; ++j) v2[8 * b + j] += src2[j * TF];
            }
          }
        }
        if (staged) {
          stage8<DUAL>(p, f, t0 + c_begin + c + 8 * b, v + 8 * b, DUAL ? v2 + 8 * b : v2, stile,
                       c + 8 * b, TH, lane_valid ? lane_row : -1, &rope);
        } else {
          epilogue8<DUAL>(p, f, t0 + c_begin + c + 8 * b, v + 8 * b, DUAL ? v2 + 8 * b : v2);
        }
      }
    }
  }
  if (warp == 2 && lane == 0) E2H_PHASE(p.phase_clock, 8);
  if (staged && is_epi) {
    asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight epilogue warps
    if (acc_ok)
      flush_tile(p, stile, TH, f0, t0 + rank * slice, slice, threadIdx.x - 64, 256);
  }

  if (warp == 2 && lane == 0) E2H_PHASE(p.phase_clock, 9);
  if (p.n_signal != 0) __threadfence();  // this thread's output is visible GPU-wide (in L2)
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Plan::tmem_cols);
  if (threadIdx.x == 32) E2H_PHASE(p.phase_clock, 10);
  if (p.n_signal != 0 && threadIdx.x == 0) {
    // the last CTA of the grid tells every tensor-parallel peer that this rank's partial
    // output is complete: one release-add on the flag word it owns in each peer's memory
    __threadfence();
    const unsigned int total = gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(p.ticket, 1u) == total - 1) {
      *p.ticket = 0;
      __threadfence_system();
      if (p.n_signal < 0) {   // signal[0] is the word's multicast address: one add reaches all
        multimem_red_release_sys_add(p.signal[0], 1);
      } else {
        for (int r = 0; r < p.n_signal; ++r) red_release_sys_add(p.signal[r], 1);
      }
    }
  }
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

// 3-D view of a K-major bf16 operand [rows, K] (K % 64 == 0): {64, rows, K/64}, so that one box
// {64, box_rows, kps} brings kps consecutive 64-wide k-blocks as kps swizzled tiles.
static int make_map3d(CUtensorMap* m, const void* base, long long K, long long rows, long long ld,
                      int box_rows, int kps) {
  EncodeTiledFn fn = get_encode_fn();
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

template <int BN, bool DUAL, int TF>
static int launch(const E2hGemmParams& p, const CUtensorMap& ta, const CUtensorMap& ta2,
                  const CUtensorMap& tb, cudaStream_t stream) {
  using Plan = SmemPlan<BN, DUAL, TF>;
  const int th = (TF == 128) ? p.th : TF;
  const size_t smem = 1024 /*alignment slack*/ + kCtrlBytes +
                      (size_t)p.stages * p.kps * (th * 128 * (DUAL ? 2 : 1) + Plan::b_bytes) +
                      xchg_bytes(BN, p.splitk, DUAL, TF);
  if (smem > 227 * 1024) return -12;
  auto kern = umma_gemm_kernel<BN, DUAL, TF>;
  static size_t configured = 0;  // per instantiation
  if (smem > configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((p.F + th - 1) / th, (p.T + BN - 1) / BN, p.splitk);
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
  if (p.a_tiled && p.a_mn_major) return -5;
  if ((p.lda % 8) || (p.ldb % 8) || (p.dual && (p.lda2 % 8))) return -6;  // 16-byte strides for TMA
  if (((uintptr_t)p.a & 15) || ((uintptr_t)p.b & 15)) return -7;
  if (p.tf != 64 && p.tf != 128) p.tf = 128;
  if (p.tf == 64 && p.bn == 256) return -9;
  // feature-tile height below the 128 rows of the instruction: K-major weights only
  if (p.tf != 128 || p.a_mn_major || p.a_tiled || p.th <= 0 || p.th > 128) p.th = p.tf;
  if (p.th < 64 || (p.th % 8) != 0) return -9;
  if (p.kps < 1) p.kps = 1;
  if (p.kps > 8) p.kps = 8;
  // several k-blocks per stage ride on 3-D boxes: K-major operands with K % 64 == 0 only
  if (p.a_mn_major || p.b_mn_major || p.a_tiled || (p.K % 64) != 0) p.kps = 1;
  const int stage_bytes = p.kps * (p.th * 128 * (p.dual ? 2 : 1) + p.bn * 128);
  const int budget = 227 * 1024 - 2048 - xchg_bytes(p.bn, p.splitk, p.dual, p.tf);
  int max_stages = budget / stage_bytes;
  if (max_stages > kMaxStages) max_stages = kMaxStages;
  if (p.stages <= 0 || p.stages > max_stages) p.stages = max_stages;
  if (p.stages < 1) return -8;
  {
    const int n_it = (kb_total / p.splitk + p.kps - 1) / p.kps;
    if (p.stages > n_it) p.stages = n_it < 1 ? 1 : n_it;
  }

  // staged (shared-memory) epilogue when the output layout allows 16-byte accesses and the
  // finished tile fits the pipeline buffers it reuses
  p.stage_epi = (epi_can_stage(p, p.th) &&
                 (long long)(p.bn / p.splitk) * p.th * 2 <= (long long)p.stages * stage_bytes)
                    ? 1 : 0;

  CUtensorMap ta, ta2, tb;
  int r;
  const long long tiled_rows = (long long)((p.F + p.tf - 1) / p.tf) * kb_total * p.tf;
  if (p.kps > 1) {
    r = make_map3d(&ta, p.a, p.K, p.F, p.lda, p.th, p.kps);
    if (r) return r;
    if (p.dual) {
      r = make_map3d(&ta2, p.a2, p.K, p.F, p.lda2, p.th, p.kps);
      if (r) return r;
    } else {
      ta2 = ta;
    }
    r = make_map3d(&tb, p.b, p.K, p.T, p.ldb, p.bn, p.kps);
    if (r) return r;
  } else {
  if (p.a_tiled)
    r = make_map(&ta, p.a, 64, tiled_rows, 64, p.tf);
  else if (!p.a_mn_major)
    r = make_map(&ta, p.a, p.K, p.F, p.lda, p.th);
  else
    r = make_map(&ta, p.a, p.F, p.K, p.lda, 64);
  if (r) return r;
  if (p.dual) {
    r = p.a_tiled ? make_map(&ta2, p.a2, 64, tiled_rows, 64, p.tf)
                  : make_map(&ta2, p.a2, p.K, p.F, p.lda2, p.th);
    if (r) return r;
  } else {
    ta2 = ta;
  }
  if (!p.b_mn_major)
    r = make_map(&tb, p.b, p.K, p.T, p.ldb, p.bn);
  else
    r = make_map(&tb, p.b, p.T, p.K, p.ldb, 64);
  if (r) return r;
  }

#define E2H_DISPATCH(BN_, DUAL_, TF_) return launch<BN_, DUAL_, TF_>(p, ta, ta2, tb, stream)
  if (p.tf == 64) {
    if (p.dual) {
      if (p.bn == 64) E2H_DISPATCH(64, true, 64);
      E2H_DISPATCH(128, true, 64);
    } else {
      if (p.bn == 64) E2H_DISPATCH(64, false, 64);
      E2H_DISPATCH(128, false, 64);
    }
  }
  if (p.dual) {
    if (p.bn == 64) E2H_DISPATCH(64, true, 128);
    if (p.bn == 128) E2H_DISPATCH(128, true, 128);
    E2H_DISPATCH(256, true, 128);
  } else {
    if (p.bn == 64) E2H_DISPATCH(64, false, 128);
    if (p.bn == 128) E2H_DISPATCH(128, false, 128);
    E2H_DISPATCH(256, false, 128);
  }
#undef E2H_DISPATCH
}
