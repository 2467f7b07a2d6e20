// Weight-only int8 GEMM for the decode step (few tokens, the weight matrix streams once):
//   out[t, f] = epilogue( scale[f] * sum_k x[t, k] * w8[f, k] )
// The int8 weights cross HBM as int8 -- half the bytes of the bf16 GEMM, which is the whole point
// of the format for a bandwidth-bound decode step -- and are expanded to bf16 inside the SM:
//
//   warp 0      TMA producer: per stage one int8 weight tile [128 features x 128 k] (128-byte rows,
//               128B swizzle: the same row granularity as the bf16 GEMM) and the two matching bf16
//               activation tiles [BN tokens x 64 k] (one 3-D box);
//   warps 2-9   converters during the main loop (two threads per feature row, 64 k each):
//               int8 -> bf16 two values per instruction -- a byte permute drops each byte into the
//               mantissa of bf16(128) (0x4300 | low 7 bits), and one packed bf16 subtraction of
//               128 or 256 (chosen by the sign bit) yields the exact integer. The converted row
//               goes straight from registers into TENSOR memory (tcgen05.st, the thread's own
//               lane, 32 columns = 64 k), where tcgen05.mma reads it as its A operand: the
//               expanded tile never touches shared memory, whose bandwidth (16 KB read + 32 KB
//               written + 32 KB read back per 128 k) held the earlier form at the bf16 rate.
//               Several buffers alternate; afterwards the eight warps run the epilogue;
//   warp 1      one thread issues tcgen05.mma (M = 128, N = BN, K = 16; A from tensor memory,
//               the activation tile from shared memory) into the fp32 accumulator.
//
// The integers -128..127 are exact in bf16, so the product equals the reference's
// F.linear(x, w_int8.to(bf16)) * scales (models/quantize.py:397-398) up to accumulation order;
// the per-feature scales ride in the shared epilogue (p.scale; a dual GEMM carries 2F of them).
// Split-K over a thread-block cluster with the DSMEM reduce-scatter, the fused epilogues and the
// completion signal are those of umma_gemm_kernel (gemm_umma.cu).
//
// All waits are bounded; a time-out writes a code to p.status and the CTA still reaches every
// barrier, frees its tensor memory and returns.
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

constexpr int kW8Threads = 320;     // TMA warp, MMA warp, 8 converter warps (4 of them: epilogue)
constexpr int kW8MaxStages = 8;
constexpr int kW8Ctrl = 1024;
constexpr int kW8Kps = 2;          // 64-wide k-blocks per pipeline stage
constexpr int kW8ConvMax = 4;      // converted-tile buffers: 4 (2 for a dual GEMM, whose tiles are twice as large)
constexpr int kW8ACol0 = 128;      // tensor-memory column of the first converted-tile buffer
constexpr int kW8ACols = 64;       // columns of one converted [128 x 128 k] bf16 tile
constexpr int kW8TmemCols = 512;

struct CtrlW8 {
  uint64_t full[kW8MaxStages];
  uint64_t empty[kW8MaxStages];
  uint64_t conv_full[kW8ConvMax];
  uint64_t conv_empty[kW8ConvMax];
  uint64_t tmem_full;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(CtrlW8) <= kW8Ctrl, "control block too large");

__host__ __device__ inline int w8_xchg_bytes(int bn, int splitk, int dual) {
  if (splitk <= 1) return 0;
  return (splitk - 1) * (bn / splitk) * 128 * 4 * (dual ? 2 : 1);
}

// four signed bytes (one 32-bit word) -> two packed bf16x2 words, exactly.
// For a byte s = low7 - 128 * sign: bf16 bits 0x4300 | low7 are the number 128 + low7; subtracting
// bf16(128) = 0x4300 (sign clear) or bf16(256) = 0x4380 (sign set) leaves s. All three values
// are exact in bf16, so is the result.
__device__ __forceinline__ void cvt4_s8_bf16(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t t01 = __byte_perm(w, 0x43434343u, 0x5140);   // [0x43:s1 | 0x43:s0]
  const uint32_t t23 = __byte_perm(w, 0x43434343u, 0x5342);   // [0x43:s3 | 0x43:s2]
  const uint32_t x01 = t01 & 0x437F437Fu, c01 = (t01 & 0x00800080u) | 0x43004300u;
  const uint32_t x23 = t23 & 0x437F437Fu, c23 = (t23 & 0x00800080u) | 0x43004300u;
  const __nv_bfloat162 r01 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&x01),
                                     *reinterpret_cast<const __nv_bfloat162*>(&c01));
  const __nv_bfloat162 r23 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&x23),
                                     *reinterpret_cast<const __nv_bfloat162*>(&c23));
  lo = *reinterpret_cast<const uint32_t*>(&r01);
  hi = *reinterpret_cast<const uint32_t*>(&r23);
}

// four unsigned nibbles -> exact bf16 (q - 8) * scale + zero with a rounding after every step,
// the arithmetic of the reference's int4 linear ((q - 8) * scales + zeros in bf16,
// models/quantize.py:108-116). The packed word holds 8 consecutive k as
// sum_j q[2j] << 4j | q[2j+1] << (16 + 4j), so (w >> 4j) & 0x000F000F is the pair (2j, 2j+1)
// already in bf16x2 position: OR-ing 0x4300 makes each half the bf16 number 128 + q.
__device__ __forceinline__ uint32_t cvt2_u4_bf16(uint32_t w, int j, __nv_bfloat162 scale,
                                                 __nv_bfloat162 zero) {
  const uint32_t t = ((w >> (4 * j)) & 0x000F000Fu) | 0x43004300u;
  const uint32_t c136 = 0x43084308u;                       // bf16(136) = 128 + 8, twice
  __nv_bfloat162 v = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&t),
                             *reinterpret_cast<const __nv_bfloat162*>(&c136));
  v = __hadd2_rn(__hmul2_rn(v, scale), zero);   // _rn: never contracted into one fused op
  return *reinterpret_cast<const uint32_t*>(&v);
}

// QB = 8: int8 weights with per-feature scales in the epilogue; QB = 4: packed int4 weights with
// group-wise (scale, zero) pairs applied by the converters.
template <int BN, bool DUAL, int QB>
__global__ void __launch_bounds__(kW8Threads, 1)
umma_gemm_w8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
                    const __grid_constant__ CUtensorMap tmB, const E2hGemmParams p) {
  constexpr int NMAT = DUAL ? 2 : 1;
  // the conversion -> MMA -> commit round trip of one buffer takes about 2 us; several buffers
  // in flight hide it. Tensor memory: accumulators in columns [0, 128), converted tiles in
  // [128, 384): 4 buffers of 64 columns (2 of 128 for a dual GEMM).
  constexpr int kW8Conv = DUAL ? 2 : 4;
  constexpr int B_BYTES = BN * 128;
  // quantised weight tile of one stage: TH rows x 128 k. TH = p.th (64..128): with lower tiles
  // a wide layer covers (nearly) all SMs in one wave instead of leaving a third of them idle;
  // the MMA still spans 128 lanes, the lanes past TH hold zeros and are never read back
  const int TH = p.th;
  const int AQ_BYTES = TH * 16 * QB;
  const int STAGE = AQ_BYTES * NMAT + kW8Kps * B_BYTES;
  constexpr int CONV_COLS = kW8ACols * NMAT;
  constexpr int ACC_COLS = BN * NMAT;
  static_assert(ACC_COLS <= kW8ACol0 && kW8ACol0 + kW8Conv * CONV_COLS <= kW8TmemCols, "tmem");
  constexpr int TMEM_COLS = kW8TmemCols;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  CtrlW8* ctrl = reinterpret_cast<CtrlW8*>(smem);
  uint8_t* tiles = smem + kW8Ctrl;
  const int stages = p.stages;
  float* xchg = reinterpret_cast<float*>(tiles + (size_t)stages * STAGE);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.splitk;
  const int rank = (S > 1) ? (int)cluster_ctarank() : 0;
  const int f0 = blockIdx.x * TH;
  const int t0 = blockIdx.y * BN;
  // the K range is split in units of one int8 tile (128 k = two bf16 k-blocks)
  const int kb2_total = p.K / 128;
  const int kb_begin = 2 * (int)((long long)rank * kb2_total / S);
  const int kb_end = 2 * (int)((long long)(rank + 1) * kb2_total / S);
  const int n_kb = kb_end - kb_begin;
  const int n_it = (n_kb + kW8Kps - 1) / kW8Kps;
  volatile int* abort_flag = &ctrl->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int c = 0; c < kW8Conv; ++c) {
      mbar_init(smem_u32(&ctrl->conv_full[c]), 8);    // one arrival per converter warp
      mbar_init(smem_u32(&ctrl->conv_empty[c]), 1);
    }
    mbar_init(smem_u32(&ctrl->tmem_full), 1);
    ctrl->abort_flag = 0;
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
  if (S > 1) cluster_sync_all();
  // programmatic dependent launch: the successor may start its prologue; this kernel's producer
  // streams the opening weight tiles (never written by a preceding kernel of the chain) before
  // it waits for the predecessor, every other thread that touches global memory waits first
  pdl_launch_dependents();
  const bool early_weights = true;
  if (!(warp == 0 && lane == 0 && early_weights) && !(warp == 1 && lane == 0)) pdl_wait_prior();

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    const uint64_t pol_a = policy_evict_first();
    int armed = 0;
    int s = 0;
    uint32_t ph = 0;
    const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
    const uint32_t tiles0 = smem_u32(tiles);
    int it0 = 0;
    if (early_weights) {
      const int n_pre = n_it < stages ? n_it : stages;
      for (int it = 0; it < n_pre; ++it) {
        const uint32_t bar = full0 + 8 * it;
        const uint32_t st = tiles0 + it * STAGE;
        const int kb = kb_begin + it * kW8Kps;
        mbar_expect_tx(bar, STAGE);
        tma_load_3d_hint(st, &tmA, 0, f0, kb / kW8Kps, bar, pol_a);
        if (DUAL) tma_load_3d_hint(st + AQ_BYTES, &tmA2, 0, f0, kb / kW8Kps, bar, pol_a);
      }
      pdl_wait_prior();
      for (int it = 0; it < n_pre; ++it)
        tma_load_3d(tiles0 + it * STAGE + AQ_BYTES * NMAT, &tmB, 0, t0, kb_begin + it * kW8Kps,
                    full0 + 8 * it);
      armed = it0 = n_pre;
      s = n_pre == stages ? 0 : n_pre;
      ph = n_pre == stages ? 1 : 0;
    }
    for (int it = it0; it < n_it; ++it) {
      if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) break;
      const uint32_t bar = full0 + 8 * s;
      const uint32_t st = tiles0 + s * STAGE;
      if (++s == stages) {
        s = 0;
        ph ^= 1;
      }
      const int kb = kb_begin + it * kW8Kps;
      // boxes are always full size: k-blocks past the matrix are zero filled, k-blocks past this
      // CTA's range are loaded but never multiplied
      mbar_expect_tx(bar, STAGE);
      tma_load_3d_hint(st, &tmA, 0, f0, kb / kW8Kps, bar, pol_a);
      if (DUAL) tma_load_3d_hint(st + AQ_BYTES, &tmA2, 0, f0, kb / kW8Kps, bar, pol_a);
      tma_load_3d(st + AQ_BYTES * NMAT, &tmB, 0, t0, kb, bar);
      armed = it + 1;
    }
    if (*abort_flag) {   // bounded wait for the copies still in flight into this CTA's smem
      for (int it = (armed > stages ? armed - stages : 0); it < armed; ++it) {
        const long long tq = clock64();
        while (!mbar_try_wait(smem_u32(&ctrl->full[it % stages]), (it / stages) & 1)) {
          if (clock64() - tq > kWaitLimitCycles / 8) break;
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- UMMA issuer ----------------
    const uint32_t idesc = make_idesc_bf16(128, BN, 0, 0);
    // descriptors: constant high word, base low words once, one add per instruction; stage and
    // phase are running counters (no division in this dependent scalar chain)
    const uint32_t d_hi = sw128_desc_hi(1024);
    const uint32_t b_lo0 = sw128_desc_lo(smem_u32(tiles) + AQ_BYTES * NMAT, 16);
    const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
    bool ok = true;
    int s = 0;
    uint32_t ph = 0, st_lo = 0, accf = 0;
    for (int it = 0; it < n_it && ok; ++it) {
      const int c = it % kW8Conv;
      ok = mbar_wait(full0 + 8 * s, ph, abort_flag, p.status, kStatusTimeoutFull) &&
           mbar_wait(smem_u32(&ctrl->conv_full[c]), (it / kW8Conv) & 1, abort_flag, p.status,
                     kStatusTimeoutFull);
      if (!ok) break;
      tc_fence_after();
      const int kcount = min(kW8Kps, n_kb - it * kW8Kps);
      // A: 8 columns (16 k) per instruction, 32 columns per 64-wide k block
      uint32_t a_col = tmem_base + kW8ACol0 + c * CONV_COLS, b_lo = b_lo0 + st_lo;
      for (int kk = 0; kk < kcount; ++kk) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          umma_f16_ts(tmem_base, a_col + 8 * k, b_lo + 2 * k, d_hi, idesc, accf);
          if (DUAL)
            umma_f16_ts(tmem_base + BN, a_col + kW8ACols + 8 * k, b_lo + 2 * k, d_hi, idesc, accf);
          accf = 1;
        }
        a_col += 32;
        b_lo += B_BYTES >> 4;
      }
      umma_commit(empty0 + 8 * s);                   // activation tile (and int8 tile) reusable
      umma_commit(smem_u32(&ctrl->conv_empty[c]));   // converted tile reusable
      if (++s == stages) {
        s = 0;
        st_lo = 0;
        ph ^= 1;
      } else {
        st_lo += STAGE >> 4;
      }
    }
    umma_commit(smem_u32(&ctrl->tmem_full));
  }

  const bool is_conv = warp >= 2;
  const bool is_epi = warp >= 2;
  const int q = warp & 3;                             // tensor-memory lane quarter of this warp
  const int half = (warp - 2) >> 2;                   // which of the quarter's two warps
  const int lane_row = q * 32 + lane;                 // feature row = tensor-memory lane
  const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
  if (is_conv) {
    // ---------------- converters: quantised tile -> bf16 rows in tensor memory ----------------
    // thread (row, half): the 64 k of `row` that make up bf16 k-block `half` of the stage
    const int row = lane_row;
    const int sw = row & 7;                           // 128B-swizzle term of this row
    bool ok = true;
    int s = 0;
    uint32_t ph = 0;
    const int gshift = QB == 4 ? __ffs(p.groupsize) - 1 : 0;   // group size is a power of two
    // int4: the (scale, zero) pair of this row's group is a global load; the pair of the next
    // stage is fetched one iteration ahead so that its latency hides behind the barrier waits
    // and the conversion of the current stage
    __nv_bfloat162 sz_next[NMAT];
    auto load_sz = [&](int it_) {
      if constexpr (QB == 4) {
        const int f = f0 + row;
        const int kglob = (kb_begin + it_ * kW8Kps + half) * 64;
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          const __nv_bfloat162* szp = static_cast<const __nv_bfloat162*>(m == 0 ? p.qsz : p.qsz2);
          sz_next[m] = (f < p.F && row < TH && it_ < n_it)
                           ? szp[(long long)(kglob >> gshift) * p.F + f]
                           : __floats2bfloat162_rn(0.f, 0.f);
        }
      }
    };
    load_sz(0);
    for (int it = 0; it < n_it; ++it) {
      const int c = it % kW8Conv;
      __nv_bfloat162 sz_cur[NMAT];
#pragma unroll
      for (int m = 0; m < NMAT; ++m) sz_cur[m] = sz_next[m];
      load_sz(it + 1);
      const int s_cur = s;
      const uint32_t ph_cur = ph;
      if (++s == stages) {
        s = 0;
        ph ^= 1;
      }
      // every converter thread waits itself (one polling lane per warp plus a shuffle measured
      // 10% slower: the acquire has to be re-established for the other lanes anyway)
      if (ok)
        ok = mbar_wait(smem_u32(&ctrl->full[s_cur]), ph_cur, abort_flag, p.status,
                       kStatusTimeoutFull) &&
             mbar_wait(smem_u32(&ctrl->conv_empty[c]), ((it / kW8Conv) & 1) ^ 1, abort_flag,
                       p.status, kStatusTimeoutEmpty);
      tc_fence_after();
      if (ok) {
        const uint8_t* st = tiles + (size_t)s_cur * STAGE;
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          uint32_t o[32];                             // 64 k of this row, two per word
          if (row >= TH) {
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = 0u;
          } else if constexpr (QB == 8) {
            const uint8_t* src = st + m * AQ_BYTES + row * 128;
#pragma unroll
            for (int j = 0; j < 4; ++j) {             // 16 int8 -> eight words
              const uint4 raw =
                  *reinterpret_cast<const uint4*>(src + (((4 * half + j) ^ sw) << 4));
              cvt4_s8_bf16(raw.x, o[8 * j + 0], o[8 * j + 1]);
              cvt4_s8_bf16(raw.y, o[8 * j + 2], o[8 * j + 3]);
              cvt4_s8_bf16(raw.z, o[8 * j + 4], o[8 * j + 5]);
              cvt4_s8_bf16(raw.w, o[8 * j + 6], o[8 * j + 7]);
            }
          } else {
            // int4 tile: 128 rows x 64 bytes, 64-byte swizzle (16-byte chunk c of a row sits at
            // c ^ ((row >> 1) & 3)); this thread's 64 k are chunks 2*half and 2*half + 1.
            // One (scale, zero) pair per feature and group: [K / g][F][2] bf16.
            const uint8_t* src = st + m * AQ_BYTES + row * 64;
            const __nv_bfloat162 pair = sz_cur[m];
            const __nv_bfloat162 sc2 = __bfloat162bfloat162(pair.x);
            const __nv_bfloat162 zr2 = __bfloat162bfloat162(pair.y);
            const int sw4 = (row >> 1) & 3;
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {          // 16 bytes = 32 nibbles -> sixteen words
              const uint4 raw =
                  *reinterpret_cast<const uint4*>(src + (((2 * half + cc) ^ sw4) << 4));
              const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  o[16 * cc + 4 * wi + j] = cvt2_u4_bf16(wds[wi], j, sc2, zr2);
              }
            }
          }
          tmem_st_x32(taddr + kW8ACol0 + c * CONV_COLS + m * kW8ACols + 32 * half, o);
        }
      }
      tmem_st_wait();
      tc_fence_before();          // the stores are ordered before the arrival below
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->conv_full[c]));
    }
  }

  // ---------------- epilogue: accumulator -> registers -> fused epilogue ----------------
  const int slice = BN / S;
  bool acc_ok = true;
  if (is_epi) {
    int ok_i = 1;
    if (lane == 0)
      ok_i = mbar_wait_relaxed(smem_u32(&ctrl->tmem_full), 0, abort_flag, p.status,
                               kStatusTimeoutTmemFull) ? 1 : 0;
    ok_i = __shfl_sync(0xffffffffu, ok_i, 0);
    acc_ok = ok_i != 0;
    tc_fence_after();
    if (S > 1 && acc_ok && n_kb > 0) {
      // reduce-scatter over token columns through distributed shared memory; the quarter's two
      // warps alternate over the 8-column groups
      for (int peer = 0; peer < S; ++peer) {
        if (peer == rank) continue;
        const int slot = rank < peer ? rank : rank - 1;
        for (int c = 8 * half; c < slice; c += 16) {
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            float v[8];
            tmem_ld_x8(taddr + m * BN + peer * slice + c, v);
            tmem_ld_wait();
            const uint32_t base = smem_u32(xchg) +
                                  ((m * (S - 1) * slice + slot * slice + c) * 128 + lane_row) * 4;
#pragma unroll
            for (int j = 0; j < 8; ++j) st_cluster_f32(mapa_shared(base + j * 128 * 4, peer), v[j]);
          }
        }
      }
    }
  }
  __syncwarp();
  if (S > 1) cluster_sync_all();

  // Staged epilogue (gemm_epilogue.cuh): the finished values go through a [tokens][128] bf16
  // tile in the (now idle) pipeline buffers and leave with 16-byte accesses.
  const bool staged = p.stage_epi != 0;
  __nv_bfloat16* stile = reinterpret_cast<__nv_bfloat16*>(tiles);
  if (is_epi && acc_ok) {
    const int c_begin = rank * slice;
    const bool lane_valid = lane_row < TH;
    const int f = lane_valid ? f0 + lane_row : p.F;   // rows past the tile are masked
    // columns of this warp: with 64 or more, alternate groups of 32; with fewer, the first /
    // second half of the 8-column units
    const int units = slice >> 3;
    int c_first, c_last;
    if (units >= 8) {
      c_first = 32 * half;
      c_last = slice;
    } else {
      const int lo = units == 1 ? 1 : units >> 1;
      c_first = half ? 8 * lo : 0;
      c_last = half ? slice : 8 * lo;
    }
    RopePre rope;
    if (staged && p.epi == E2H_EPI_ROPE_KV) rope = rope_prepare(p, f);
    for (int c = c_first; c < c_last; c += 64) {
      const int nb = (c_last - c) >= 32 ? 4 : (c_last - c) / 8;
      float v[32], v2[DUAL ? 32 : 1];
      if (n_kb > 0) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          if (b < nb) {
            tmem_ld_x8(taddr + c_begin + c + 8 * b, v + 8 * b);
            if constexpr (DUAL) tmem_ld_x8(taddr + BN + c_begin + c + 8 * b, v2 + 8 * b);
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
            const float* src = xchg + (size_t)(slot * slice + c + 8 * b) * 128 + lane_row;
#pragma unroll
            for (int j = 0; j < 8; ++j) v[8 * b + j] += src[j * 128];
            if constexpr (DUAL) {
              const float* src2 = src + (size_t)(S - 1) * slice * 128;
#pragma unroll
              for (int j = 0; j < 8; ++j) v2[8 * b + j] += src2[j * 128];
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
  if (staged && is_epi) {
    asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight epilogue warps
    if (acc_ok) flush_tile(p, stile, TH, f0, t0 + rank * slice, slice, threadIdx.x - 64, 256);
  }

  if (p.n_signal != 0) __threadfence();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (p.n_signal != 0 && threadIdx.x == 0) {
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
typedef CUresult (*W8EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                               const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static W8EncodeFn w8_encode_fn() {
  static W8EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<W8EncodeFn>(sym);
  });
  return fn;
}

// K-major operand [rows, K] seen as {inner, rows, K / inner} with `inner` elements = 128 bytes
// (64 bf16 or 128 int8): one box {inner, box_rows, nblk} lands as nblk consecutive
// [box_rows x 128 B] tiles with the 128-byte swizzle.
static int w8_map3d(CUtensorMap* m, const void* base, long long K, long long rows, long long ld,
                    int box_rows, int nblk, bool int8) {
  W8EncodeFn fn = w8_encode_fn();
  if (!fn) return -10;
  const int es = int8 ? 1 : 2;
  const int inner = 128 / es;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)(K / inner)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * es, 128u};
  cuuint32_t box[3] = {(cuuint32_t)inner, (cuuint32_t)box_rows, (cuuint32_t)nblk};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(m, int8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                  const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

// Packed int4 operand [rows, K / 2 bytes] seen as {64 bytes, rows, K / 128}: one box
// {64, 128, 1} is the [128 rows x 128 k] tile of a stage, 64-byte swizzle.
static int w4_map3d(CUtensorMap* m, const void* base, long long K, long long rows,
                    long long ld_bytes, int box_rows) {
  W8EncodeFn fn = w8_encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)(K / 128)};
  cuuint64_t strides[2] = {(cuuint64_t)ld_bytes, 64u};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

template <int BN, bool DUAL, int QB>
static int w8_launch(E2hGemmParams& p, cudaStream_t stream) {
  constexpr int NMAT = DUAL ? 2 : 1;
  // tile height: 128, or p.th (64..128; a multiple of 8 rows for int8, of 16 for int4, so that
  // every part of a stage starts on a swizzle-atom boundary)
  if (p.th <= 0) p.th = 128;
  if (p.th < 64 || p.th > 128 || (p.th % (QB == 8 ? 8 : 16))) return -12;
  const int STAGE = p.th * 16 * QB * NMAT + kW8Kps * BN * 128;
  const int fixed = 1024 + kW8Ctrl + w8_xchg_bytes(BN, p.splitk, DUAL);
  int stages = (227 * 1024 - fixed) / STAGE;
  if (stages > kW8MaxStages) stages = kW8MaxStages;
  if (p.stages > 0 && p.stages < stages) stages = p.stages;
  const int n_it = (p.K / 128 + p.splitk - 1) / p.splitk;
  if (stages > n_it) stages = n_it < 1 ? 1 : n_it;
  if (stages < 1) return -8;
  p.stages = stages;
  // staged (shared-memory) epilogue when the output layout allows 16-byte accesses and the
  // finished tile fits the pipeline buffers it reuses
  p.stage_epi = (epi_can_stage(p, p.th) &&
                 (long long)(BN / p.splitk) * p.th * 2 <= (long long)stages * STAGE)
                    ? 1 : 0;
  CUtensorMap ta, ta2, tb;
  int r = QB == 8 ? w8_map3d(&ta, p.a, p.K, p.F, p.lda, p.th, 1, true)
                  : w4_map3d(&ta, p.a, p.K, p.F, p.lda, p.th);
  if (r) return r;
  if (DUAL) {
    r = QB == 8 ? w8_map3d(&ta2, p.a2, p.K, p.F, p.lda2, p.th, 1, true)
                : w4_map3d(&ta2, p.a2, p.K, p.F, p.lda2, p.th);
    if (r) return r;
  } else {
    ta2 = ta;
  }
  r = w8_map3d(&tb, p.b, p.K, p.T, p.ldb, BN, kW8Kps, false);
  if (r) return r;
  // The kernel takes all 512 tensor-memory columns of its SM, and tensor memory is claimed by the
  // running CTA, not by the launch: a second CTA of the same cluster on the same SM would wait
  // for columns that its partner only frees after the cluster barrier. Asking for more than
  // half of the SM's shared memory keeps every SM at one CTA of this kernel.
  size_t smem = (size_t)fixed + (size_t)stages * STAGE;
  if (smem < 120 * 1024) smem = 120 * 1024;
  auto kern = umma_gemm_w8_kernel<BN, DUAL, QB>;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((p.F + p.th - 1) / p.th, (p.T + BN - 1) / BN, p.splitk);
  cfg.blockDim = dim3(kW8Threads, 1, 1);
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

// Same parameter block as e2h_gemm_umma, with p.a (and p.a2) pointing at int8 [F, K] weights
// (lda in elements = bytes, a multiple of 16), p.b bf16 [T, K], K % 128 == 0, T-tile bn 64 or 128,
// and p.scale the fp32 per-feature scales (F of them, or 2F for a dual GEMM).
extern "C" int e2h_gemm_w8(const E2hGemmParams* pp, void* stream_v) {
  using namespace e2h;
  E2hGemmParams p = *pp;
  if (p.F <= 0 || p.T <= 0 || p.K <= 0 || (p.K % 128)) return -1;
  if (p.bn != 64 && p.bn != 128) return -2;
  if (p.dual && p.bn != 64) return -2;
  if (p.splitk < 1 || p.splitk > 8 || (p.bn % (p.splitk * 8)) != 0) return -3;
  if ((p.K / 128) < p.splitk) return -4;
  if (p.a_mn_major || p.b_mn_major || p.a_tiled) return -5;
  if (p.dual && p.a2 == nullptr) return -5;
  if ((p.lda % 16) || (p.ldb % 8) || (p.dual && (p.lda2 % 16))) return -6;
  if (((uintptr_t)p.a & 15) || ((uintptr_t)p.b & 15) || (p.dual && ((uintptr_t)p.a2 & 15)))
    return -7;
  if (p.scale == nullptr) return -9;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (p.dual) return w8_launch<64, true, 8>(p, stream);
  if (p.bn == 64) return w8_launch<64, false, 8>(p, stream);
  return w8_launch<128, false, 8>(p, stream);
}

// Weight-only int4, group-wise: p.a (and p.a2) point at packed nibbles [F, K / 2] bytes (lda =
// row pitch in bytes, a multiple of 16) where every 32-bit word holds 8 consecutive k as
// sum_j q[2j] << 4j | q[2j+1] << (16 + 4j); p.qsz (and p.qsz2) the [K / g][F][2] bf16
// (scale, zero) pairs of the reference's checkpoint format; p.groupsize a power of two >= 64
// that divides K; K % 128 == 0. out = epilogue( sum_k x[t,k] * bf16((q-8) * scale + zero) ).
extern "C" int e2h_gemm_w4(const E2hGemmParams* pp, void* stream_v) {
  using namespace e2h;
  E2hGemmParams p = *pp;
  if (p.F <= 0 || p.T <= 0 || p.K <= 0 || (p.K % 128)) return -1;
  if (p.bn != 64 && p.bn != 128) return -2;
  if (p.dual && p.bn != 64) return -2;
  if (p.splitk < 1 || p.splitk > 8 || (p.bn % (p.splitk * 8)) != 0) return -3;
  if ((p.K / 128) < p.splitk) return -4;
  if (p.a_mn_major || p.b_mn_major || p.a_tiled) return -5;
  if (p.dual && (p.a2 == nullptr || p.qsz2 == nullptr)) return -5;
  if ((p.lda % 16) || (p.ldb % 8) || (p.dual && (p.lda2 % 16))) return -6;
  if (((uintptr_t)p.a & 15) || ((uintptr_t)p.b & 15) || (p.dual && ((uintptr_t)p.a2 & 15)))
    return -7;
  if (p.qsz == nullptr || p.groupsize < 64 || (p.groupsize & (p.groupsize - 1)) ||
      (p.K % p.groupsize))
    return -9;
  p.scale = nullptr;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (p.dual) return w8_launch<64, true, 4>(p, stream);
  if (p.bn == 64) return w8_launch<64, false, 4>(p, stream);
  return w8_launch<128, false, 4>(p, stream);
}
