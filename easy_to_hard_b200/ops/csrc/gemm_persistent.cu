// Persistent tcgen05 GEMM for large token counts (prefill, training).
//
// Same math and operand conventions as gemm_umma.cu (features on TMEM lanes, tokens on TMEM
// columns), organised for throughput instead of latency:
//   * one CTA per SM walks a list of output tiles (grouped so that a wave of CTAs shares a band
//     of token tiles and the weight stays in L2);
//   * the accumulator is double buffered in tensor memory (2 x 256 columns), so the epilogue of
//     tile i overlaps the main loop of tile i+1;
//   * bf16 outputs leave through shared memory and TMA stores: the epilogue threads (one
//     feature each) write 32-token chunks into a [token][feature] staging buffer and one thread
//     issues cp.async.bulk.tensor stores of full 256-byte rows; a residual operand comes in the
//     same way (TMA load of the matching chunk) instead of 2-byte strided loads.
// Epilogues without a staged form (fp32 outputs, RoPE + KV scatter, weight-gradient
// accumulation) use the per-thread path of gemm_epilogue.cuh and still get the overlap.
// Every wait is bounded; on a time-out the roles stop, the status word is set and the CTA
// still reaches its final barrier and frees its tensor memory.
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

constexpr int kPThreads = 192;
constexpr int kPMaxStages = 8;
constexpr int kChunkTok = 32;                       // tokens per staged epilogue chunk
constexpr int kChunkBytes = kChunkTok * 128 * 2;    // [32 tokens][128 features] bf16
constexpr int kGroupT = 8;                          // token tiles per scheduling band

struct PCtrl {
  uint64_t full[kPMaxStages];
  uint64_t empty[kPMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t res_full[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void epi_bar_sync() {  // the 128 epilogue threads only
  asm volatile("bar.sync 1, 128;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld_x32p(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
      "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// tile id -> (feature tile, token tile): bands of kGroupT token tiles, features fastest
__device__ __forceinline__ void tile_coords(int id, int n_f, int n_t, int& ft, int& tt) {
  const int band_sz = kGroupT * n_f;
  const int band = id / band_sz;
  const int r = id - band * band_sz;
  const int tb = min(kGroupT, n_t - band * kGroupT);
  ft = r / tb;
  tt = band * kGroupT + r % tb;
}

// PAIR: two CTAs of a cluster share one 256 (features) x 256 (tokens) tile with cta_group::2
// instructions: CTA r of the pair owns features [128 r, 128 r + 128) of the tile (its A rows, its
// accumulator lanes, its epilogue) and stages the B rows of tokens [128 r, 128 r + 128); the
// leader (rank 0) issues every tcgen05.mma for both. The full barriers of the leader count the
// TMA bytes of both CTAs, the commits are multicast to the barriers of both, and the peer's
// epilogue warps hand the accumulator back on the leader's barrier.
template <int BN, bool DUAL, bool PAIR>
__global__ void __launch_bounds__(kPThreads, 1)
umma_gemm_persistent_kernel(const __grid_constant__ CUtensorMap tmA,
                            const __grid_constant__ CUtensorMap tmA2,
                            const __grid_constant__ CUtensorMap tmB,
                            const __grid_constant__ CUtensorMap tmOut,
                            const __grid_constant__ CUtensorMap tmRes, const E2hGemmParams p,
                            const int staged, const int mn3d) {
  static_assert(!PAIR || (BN == 256 && !DUAL), "pair tiles are 2 x 128 features x 256 tokens");
  constexpr int A_BYTES = 128 * 128;                  // 128 features x 64 k, bf16
  constexpr int BROWS = PAIR ? BN / 2 : BN;           // B rows staged by this CTA
  constexpr int B_BYTES = BROWS * 128;
  constexpr int STAGE = A_BYTES * (DUAL ? 2 : 1) + B_BYTES;
  constexpr int ACC_COLS = BN * (DUAL ? 2 : 1);
  static_assert(ACC_COLS <= 256, "two accumulator buffers must fit in 512 TMEM columns");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  PCtrl* ctrl = reinterpret_cast<PCtrl*>(smem);
  uint8_t* tiles = smem + 1024;
  const int stages = p.stages;
  uint8_t* stage_out = tiles + (size_t)stages * STAGE;      // 2 x kChunkBytes
  uint8_t* stage_res = stage_out + 2 * kChunkBytes;         // 2 x kChunkBytes

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int crank = PAIR ? (int)cluster_ctarank() : 0;          // 0: leader of the pair
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;   // tile walker id
  const int n_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  constexpr int TILE_F = PAIR ? 256 : 128;
  const int n_f = (p.F + TILE_F - 1) / TILE_F, n_t = (p.T + BN - 1) / BN;
  const int n_tiles = n_f * n_t;
  const int n_kb = (p.K + 63) / 64;
  volatile int* abort_flag = &ctrl->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&ctrl->full[s]), 1);
      mbar_init(smem_u32(&ctrl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctrl->tmem_full[a]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[a]), PAIR ? 8 : 4);   // one arrival per epilogue warp
      mbar_init(smem_u32(&ctrl->res_full[a]), 1);
    }
    ctrl->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (DUAL) tma_prefetch_desc(&tmA2);
    if (staged) tma_prefetch_desc(&tmOut);
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_u32(&ctrl->tmem_base), 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;
  if constexpr (PAIR) cluster_sync_all();   // the peer's barriers exist before anything signals them
  pdl_wait_prior();
  pdl_launch_dependents();

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    // stage / phase are running counters: this thread is one dependent scalar chain and an
    // integer division per k-block is a hundred cycles of it
    int it = 0, s = 0;
    uint32_t ph = 0;
    const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
    const uint32_t tiles0 = smem_u32(tiles);
    bool ok = true;
    const uint32_t full_lead0 = PAIR ? mapa_shared(full0, 0) : full0;   // leader's full barriers
    for (int tile = worker; tile < n_tiles && ok; tile += n_workers) {
      int ft, tt;
      tile_coords(tile, n_f, n_t, ft, tt);
      const int f0 = ft * TILE_F + crank * 128, t0 = tt * BN + crank * BROWS * (PAIR ? 1 : 0);
      for (int kb = 0; kb < n_kb; ++kb, ++it) {
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, p.status, kStatusTimeoutEmpty)) {
          ok = false;
          break;
        }
        const uint32_t a_dst = tiles0 + s * STAGE;
        if constexpr (PAIR) {
          // the leader arms its barrier for the bytes of both CTAs; each CTA's copies complete
          // on that barrier (the arrival count keeps the phase open until the leader has armed)
          const uint32_t bar = full_lead0 + 8 * s;
          if (crank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE);
          const int k0p = kb * 64;
          if (!p.a_mn_major) {
            tma_load_2d_pair(a_dst, &tmA, k0p, f0, bar);
          } else {
            tma_load_3d_pair(a_dst, &tmA, 0, k0p, f0 >> 6, bar);
          }
          if (!p.b_mn_major) {
            tma_load_2d_pair(a_dst + A_BYTES, &tmB, k0p, t0, bar);
          } else {
            tma_load_3d_pair(a_dst + A_BYTES, &tmB, 0, k0p, t0 >> 6, bar);
          }
          if (++s == stages) {
            s = 0;
            ph ^= 1;
          }
          continue;
        }
        const uint32_t bar = full0 + 8 * s;
        mbar_expect_tx(bar, STAGE);
        if (++s == stages) {
          s = 0;
          ph ^= 1;
        }
        const int k0 = kb * 64;
        if (!p.a_mn_major) {
          tma_load_2d(a_dst, &tmA, k0, f0, bar);
          if (DUAL) tma_load_2d(a_dst + A_BYTES, &tmA2, k0, f0, bar);
        } else if (mn3d & 1) {
          // one instruction for both 64-feature chunks: box (64, 64 k-rows, 2 chunks)
          tma_load_3d(a_dst, &tmA, 0, k0, f0 >> 6, bar);
        } else {
          tma_load_2d(a_dst, &tmA, f0, k0, bar);
          tma_load_2d(a_dst + 8192, &tmA, f0 + 64, k0, bar);
        }
        const uint32_t b_dst = a_dst + A_BYTES * (DUAL ? 2 : 1);
        if (!p.b_mn_major) {
          tma_load_2d(b_dst, &tmB, k0, t0, bar);
        } else if (mn3d & 2) {
          tma_load_3d(b_dst, &tmB, 0, k0, t0 >> 6, bar);
        } else {
#pragma unroll
          for (int c = 0; c < BN / 64; ++c)
            tma_load_2d(b_dst + c * 8192, &tmB, t0 + c * 64, k0, bar);
        }
      }
    }
    if (*abort_flag) {  // bounded wait for the copies still in flight into this CTA's smem
      for (int j = (it > stages ? it - stages : 0); j < it; ++j) {
        const long long tq = clock64();
        while (!mbar_try_wait(smem_u32(&ctrl->full[j % stages]), (j / stages) & 1)) {
          if (clock64() - tq > kWaitLimitCycles / 8) break;
        }
      }
    }
  } else if (warp == 1 && lane == 0 && crank == 0) {
    // ---------------- UMMA issuer (the leader's for a pair) ----------------
    const uint32_t idesc = make_idesc_bf16(PAIR ? 256 : 128, BN, p.a_mn_major, p.b_mn_major);
    const uint32_t a_kstep = p.a_mn_major ? 2048u : 32u;
    const uint32_t b_kstep = p.b_mn_major ? 2048u : 32u;
    const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u;
    const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u;
    // descriptors: constant high word, base low words once, then one add per instruction
    const uint32_t d_hi = sw128_desc_hi(1024);
    const uint32_t a_lo0 = sw128_desc_lo(smem_u32(tiles), a_lbo);
    const uint32_t b_lo0 = sw128_desc_lo(smem_u32(tiles) + A_BYTES * (DUAL ? 2 : 1), b_lbo);
    const uint32_t a_ks = a_kstep >> 4, b_ks = b_kstep >> 4;
    const uint32_t full0 = smem_u32(&ctrl->full[0]), empty0 = smem_u32(&ctrl->empty[0]);
    int tcount = 0, s = 0;
    uint32_t ph = 0, st_lo = 0;
    bool ok = true;
    for (int tile = worker; tile < n_tiles && ok; tile += n_workers, ++tcount) {
      const int acc = tcount & 1;
      const uint32_t accph = (tcount >> 1) & 1;
      ok = mbar_wait(smem_u32(&ctrl->tmem_empty[acc]), accph ^ 1, abort_flag, p.status,
                     kStatusTimeoutTmemEmpty);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d0 = tmem_base + acc * ACC_COLS;
      uint32_t accum = 0;   // the first instruction of a tile overwrites the accumulator
      for (int kb = 0; kb < n_kb; ++kb) {
        ok = mbar_wait(full0 + 8 * s, ph, abort_flag, p.status, kStatusTimeoutFull);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_lo = a_lo0 + st_lo, b_lo = b_lo0 + st_lo;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if constexpr (PAIR) {
            umma_f16_lohi_pair(d0, a_lo + k * a_ks, d_hi, b_lo + k * b_ks, d_hi, idesc, accum);
          } else {
            umma_f16_lohi(d0, a_lo + k * a_ks, d_hi, b_lo + k * b_ks, d_hi, idesc, accum);
            if (DUAL)
              umma_f16_lohi(d0 + BN, a_lo + (A_BYTES >> 4) + k * a_ks, d_hi, b_lo + k * b_ks,
                            d_hi, idesc, accum);
          }
          accum = 1;
        }
        if constexpr (PAIR) umma_commit_pair(empty0 + 8 * s);
        else umma_commit(empty0 + 8 * s);
        if (++s == stages) {
          s = 0;
          st_lo = 0;
          ph ^= 1;
        } else {
          st_lo += STAGE >> 4;
        }
      }
      if (ok) {
        if constexpr (PAIR) umma_commit_pair(smem_u32(&ctrl->tmem_full[acc]));
        else umma_commit(smem_u32(&ctrl->tmem_full[acc]));
      }
    }
  } else if (warp >= 2) {
    // ---------------- epilogue warps ----------------
    const int q = warp & 3;
    const int lane_row = q * 32 + lane;
    const int et = threadIdx.x - 64;                    // 0..127 among the epilogue threads
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const bool with_res = staged && p.epi == E2H_EPI_RESIDUAL;
    int tcount = 0, cc = 0;
    bool ok = true;
    // the accumulator goes back to the MMA thread of the pair's leader
    const uint32_t tmem_empty0 = PAIR ? mapa_shared(smem_u32(&ctrl->tmem_empty[0]), 0)
                                      : smem_u32(&ctrl->tmem_empty[0]);
    for (int tile = worker; tile < n_tiles; tile += n_workers, ++tcount) {
      int ft, tt;
      tile_coords(tile, n_f, n_t, ft, tt);
      const int f0 = ft * TILE_F + crank * 128, t0 = tt * BN;
      const int f = f0 + lane_row;
      const int acc = tcount & 1;
      const uint32_t accph = (tcount >> 1) & 1;
      int ok_i = 1;
      if (lane == 0 && ok)
        ok_i = mbar_wait_relaxed(smem_u32(&ctrl->tmem_full[acc]), accph, abort_flag, p.status,
                                 kStatusTimeoutTmemFull) ? 1 : 0;
      ok = ok && (__shfl_sync(0xffffffffu, ok_i, 0) != 0);
      tc_fence_after();
      const uint32_t a0 = taddr + acc * ACC_COLS;
      if (staged) {
        if (with_res && et == 0 && ok) {   // first residual chunk of the tile
          const int b = cc & 1;
          mbar_expect_tx(smem_u32(&ctrl->res_full[b]), kChunkBytes);
          tma_load_2d(smem_u32(stage_res + b * kChunkBytes), &tmRes, f0, t0,
                      smem_u32(&ctrl->res_full[b]));
        }
        for (int c = 0; c < BN / kChunkTok; ++c, ++cc) {
          const int b = cc & 1;
          // staging buffer b is free once the store issued two chunks ago has read it
          if (et == 0) bulk_wait_group_read<1>();
          epi_bar_sync();
          if (with_res && et == 0 && ok && c + 1 < BN / kChunkTok) {   // prefetch next chunk
            const int nb = (cc + 1) & 1;
            mbar_expect_tx(smem_u32(&ctrl->res_full[nb]), kChunkBytes);
            tma_load_2d(smem_u32(stage_res + nb * kChunkBytes), &tmRes, f0,
                        t0 + (c + 1) * kChunkTok, smem_u32(&ctrl->res_full[nb]));
          }
          float v[32], v2[DUAL ? 32 : 1];
          if (ok) {
            tmem_ld_x32p(a0 + c * kChunkTok, v);
            if constexpr (DUAL) tmem_ld_x32p(a0 + BN + c * kChunkTok, v2);
          }
          tmem_ld_wait();
          if (c + 1 == BN / kChunkTok) {   // accumulator fully read: hand it back to the MMA
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (PAIR) mbar_arrive_cluster(tmem_empty0 + 8 * acc);
              else mbar_arrive(tmem_empty0 + 8 * acc);
            }
          }
          if (with_res && ok)
            ok = mbar_wait(smem_u32(&ctrl->res_full[b]), (cc >> 1) & 1, abort_flag, p.status,
                           kStatusTimeoutFull);
          const float sc = (p.scale != nullptr && f < p.F) ? p.scale[f] : 1.f;
          const float sc2 = (DUAL && p.scale != nullptr && f < p.F) ? p.scale[p.F + f] : 1.f;
          __nv_bfloat16* so = reinterpret_cast<__nv_bfloat16*>(stage_out + b * kChunkBytes);
          if (staged == 2) {
            // feature-major output (weight gradients): this lane's 32 values are one 64-byte
            // row of the staging tile; the 16-byte pieces are XOR-swizzled (64B TMA swizzle:
            // address bits 4-5 ^= bits 7-8) so that the vector stores do not bank-conflict
            uint8_t* row = reinterpret_cast<uint8_t*>(so) + lane_row * 64;
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              uint4 pk;
              uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                __nv_bfloat162 two = __floats2bfloat162_rn(v[c4 * 8 + 2 * h] * sc,
                                                           v[c4 * 8 + 2 * h + 1] * sc);
                w[h] = *reinterpret_cast<uint32_t*>(&two);
              }
              *reinterpret_cast<uint4*>(row + ((c4 ^ ((lane_row >> 1) & 3)) << 4)) = pk;
            }
            fence_proxy_async_smem();
            epi_bar_sync();
            if (et == 0 && ok && t0 + c * kChunkTok < p.T) {
              tma_store_2d(&tmOut, smem_u32(so), t0 + c * kChunkTok, f0);
              bulk_commit_group();
            }
            continue;
          }
          const __nv_bfloat16* sr =
              reinterpret_cast<const __nv_bfloat16*>(stage_res + b * kChunkBytes);
#pragma unroll
          for (int j = 0; j < kChunkTok; ++j) {
            float y;
            if constexpr (DUAL) {
              const float g = bf16_round(v[j] * sc), u = bf16_round(v2[j] * sc2);
              y = bf16_round(silu(g)) * u;
            } else {
              y = v[j] * sc;
              if (with_res) y = bf16_round(y) + __bfloat162float(sr[j * 128 + lane_row]);
            }
            so[j * 128 + lane_row] = __float2bfloat16_rn(y);
          }
          fence_proxy_async_smem();
          epi_bar_sync();
          if (et == 0 && ok && t0 + c * kChunkTok < p.T) {
            tma_store_2d(&tmOut, smem_u32(so), f0, t0 + c * kChunkTok);
            bulk_commit_group();
          }
        }
      } else {
        for (int c = 0; c < BN; c += 32) {
          float v[32], v2[DUAL ? 32 : 1];
          if (ok) {
            tmem_ld_x32p(a0 + c, v);
            if constexpr (DUAL) tmem_ld_x32p(a0 + BN + c, v2);
          }
          tmem_ld_wait();
          if (c + 32 == BN) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (PAIR) mbar_arrive_cluster(tmem_empty0 + 8 * acc);
              else mbar_arrive(tmem_empty0 + 8 * acc);
            }
          }
          if (ok) {
#pragma unroll
            for (int b8 = 0; b8 < 4; ++b8)
              epilogue8<DUAL>(p, f, t0 + c + 8 * b8, v + 8 * b8, DUAL ? v2 + 8 * b8 : v2);
          }
        }
      }
    }
    if (staged && et == 0) {
      if (p.n_signal != 0) {
        // a completion signal follows: the TMA stores must have been written to global memory,
        // not merely have read their shared-memory source, before peers are told to read
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async;" ::: "memory");
      } else {
        bulk_wait_group_read<0>();   // smem stays valid until the stores have read it
      }
    }
  }

  if (p.n_signal != 0) __threadfence();
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) {
    // neither CTA may leave (or free tensor memory) while the other can still read its shared
    // memory through an instruction in flight or signal one of its barriers
    cluster_sync_all();
    if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
  } else {
    if (warp == 1) tmem_dealloc(tmem_base, 512);
  }
  if (p.n_signal != 0 && threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.ticket, 1u) == gridDim.x - 1) {
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

// ---------------------------------------------------------------------------------------------
typedef CUresult (*PEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PEncodeFn p_encode_fn() {
  static PEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PEncodeFn>(sym);
  });
  return fn;
}
static int p_map(CUtensorMap* m, const void* base, long long inner, long long outer, long long ld,
                 int box_inner, int box_rows, int swizzle) {
  PEncodeFn fn = p_encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B
                               : (swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                                               : CU_TENSOR_MAP_SWIZZLE_NONE),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

// MN-major operand [K rows, mn] (mn a multiple of 64) seen as (64, K, mn / 64): one box of
// (64, 64, chunks) lands in shared memory as `chunks` consecutive 64 x 64 swizzled blocks, the
// layout the MN-major UMMA descriptors expect, with a single TMA instruction.
static int p_map_mn3d(CUtensorMap* m, const void* base, long long mn, long long k, long long ld,
                      int chunks) {
  PEncodeFn fn = p_encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[3] = {64, (cuuint64_t)k, (cuuint64_t)(mn / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
  cuuint32_t box[3] = {64, 64, (cuuint32_t)chunks};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

template <int BN, bool DUAL, bool PAIR>
static int p_launch(E2hGemmParams& p, cudaStream_t stream) {
  constexpr int BROWS = PAIR ? BN / 2 : BN;
  constexpr int STAGE = 128 * 128 * (DUAL ? 2 : 1) + BROWS * 128;
  CUtensorMap ta, ta2, tb, to, tr;
  int r;
  int mn3d = 0;
  if (p.a_mn_major && p.F % 64 == 0) {
    mn3d |= 1;
    r = p_map_mn3d(&ta, p.a, p.F, p.K, p.lda, 2);
  } else {
    r = p.a_mn_major ? p_map(&ta, p.a, p.F, p.K, p.lda, 64, 64, true)
                     : p_map(&ta, p.a, p.K, p.F, p.lda, 64, 128, true);
  }
  if (r) return r;
  if (DUAL) {
    r = p_map(&ta2, p.a2, p.K, p.F, p.lda2, 64, 128, true);
    if (r) return r;
  } else {
    ta2 = ta;
  }
  if (p.b_mn_major && p.T % 64 == 0) {
    mn3d |= 2;
    r = p_map_mn3d(&tb, p.b, p.T, p.K, p.ldb, BROWS / 64);
  } else {
    r = p.b_mn_major ? p_map(&tb, p.b, p.T, p.K, p.ldb, 64, 64, true)
                     : p_map(&tb, p.b, p.K, p.T, p.ldb, 64, BROWS, true);
  }
  if (r) return r;
  int staged = (p.epi == E2H_EPI_STORE_BF16 || p.epi == E2H_EPI_RESIDUAL ||
                (p.epi == E2H_EPI_SWIGLU && DUAL)) ? 1 : 0;
  if (staged && ((p.ldo % 8) || ((uintptr_t)p.out & 15))) staged = 0;
  if (staged && p.epi == E2H_EPI_RESIDUAL && ((uintptr_t)p.aux & 15)) staged = 0;
  if (!staged && p.epi == E2H_EPI_ROWMAJOR_BF16 && !p.accumulate && !DUAL && (p.ldo % 8) == 0 &&
      ((uintptr_t)p.out & 15) == 0) {
    staged = 2;
    r = p_map(&to, p.out, p.T, p.F, p.ldo, kChunkTok, 128, 2);
    if (r) return r;
    tr = to;
  } else if (staged) {
    r = p_map(&to, p.out, p.F, p.T, p.ldo, 128, kChunkTok, false);
    if (r) return r;
    if (p.epi == E2H_EPI_RESIDUAL) {
      r = p_map(&tr, p.aux, p.F, p.T, p.ldo, 128, kChunkTok, false);
      if (r) return r;
    } else {
      tr = to;
    }
  } else {
    to = tb;
    tr = tb;
  }
  const int budget = 227 * 1024 - 2048 - 4 * kChunkBytes;
  int stages = budget / STAGE;
  if (stages > kPMaxStages) stages = kPMaxStages;
  if (p.stages > 0 && p.stages < stages) stages = p.stages;
  if (stages < 2) return -8;
  p.stages = stages;
  const size_t smem = 2048 + (size_t)stages * STAGE + 4 * kChunkBytes;
  auto kern = umma_gemm_persistent_kernel<BN, DUAL, PAIR>;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  int n_sm = 148;
  {
    static int cached = 0;
    if (!cached) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    }
    if (cached > 0) n_sm = cached;
  }
  if constexpr (PAIR) {
    // one cluster of two CTAs per 256 x 256 tile walker
    const int n_tiles = (p.F / 256) * ((p.T + BN - 1) / BN);
    const int pairs = n_tiles < n_sm / 2 ? n_tiles : n_sm / 2;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(kPThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 2;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = 1;
    ++na;
    if (p.pdl || g_pdl) {
      attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attrs[na].val.programmaticStreamSerializationAllowed = 1;
      ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    return (int)cudaLaunchKernelEx(&cfg, kern, ta, ta2, tb, to, tr, p, staged, mn3d);
  }
  const int n_tiles = ((p.F + 127) / 128) * ((p.T + BN - 1) / BN);
  const int grid = n_tiles < n_sm ? n_tiles : n_sm;
  return (int)launch(kern, dim3(grid), dim3(kPThreads), smem, stream, ta, ta2, tb, to, tr, p,
                     staged, mn3d);
}

}  // namespace e2h

// Same parameter block as e2h_gemm_umma; requires splitk == 1 and 128-feature tiles.
extern "C" int e2h_gemm_persistent(const E2hGemmParams* pp, void* stream_v) {
  using namespace e2h;
  E2hGemmParams p = *pp;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (p.F <= 0 || p.T <= 0 || p.K <= 0) return -1;
  if (p.splitk > 1 || p.a_tiled) return -3;
  if (p.dual && (p.a_mn_major || p.a2 == nullptr)) return -5;
  if ((p.lda % 8) || (p.ldb % 8) || (p.dual && (p.lda2 % 8))) return -6;
  if (((uintptr_t)p.a & 15) || ((uintptr_t)p.b & 15)) return -7;
  if (p.dual) return p_launch<128, true, false>(p, stream);
  if (p.bn == 128) return p_launch<128, false, false>(p, stream);
  // tf == 256 asks for CTA-pair tiles (cta_group::2): 256-feature tiles, operands that the 3-D
  // boxes can address
  if (p.tf == 256 && (p.F % 256) == 0 && p.T > 256 && (p.K % 64) == 0 &&
      (!p.b_mn_major || (p.T % 64) == 0))
    return p_launch<256, false, true>(p, stream);
  return p_launch<256, false, false>(p, stream);
}
