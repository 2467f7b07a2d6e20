// Causal flash attention (forward) on tcgen05 tensor cores, head_dim 128 or 64.
//
// One CTA = one (batch, head, 128-query block). Roles (192 threads):
//   warp 0    TMA producer: Q once, then K / V tiles (128 keys) through two-deep rings
//   warp 1    UMMA issuer:  S = Q K^T  (TMEM cols [0,128)),  O_blk = P V  (TMEM cols [128,256))
//   warps 2-5 softmax: thread r owns query row r. It reads its row of S from TMEM (no
//             cross-thread reduction for max / sum), writes P = exp(S - m) as bf16 into shared
//             memory in the 128-byte-swizzled K-major layout the UMMA expects, and keeps the
//             running output row O (fp32, head_dim registers), rescaled by exp(m_old - m_new).
// S(j+1) is issued as soon as S(j) has been read out, so the tensor core works on the next
// score tile while the softmax of the current one runs.
//
// Masking follows the reference model (models/model.py:221-228, 338-344): key j is visible to
// query i when j <= i + (Sk - Sq) and j >= left_pad[b], or when j is the diagonal; with
// left_pad == nullptr this is plain causal attention (training, scoring, reward models).
// Layouts are given by strides, so Q/K/V may be views into the fused qkv activation or the
// static KV cache ([B, Hkv, Smax, D]).
//
// All mbarrier waits are bounded; a time-out sets the status word and the CTA still reaches
// every barrier and frees its tensor memory.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <float.h>
#include <string.h>
#include <mutex>

#include "ptx.cuh"

namespace e2h {

constexpr int kBQ = 128;   // queries per CTA
constexpr int kBK = 128;   // keys per tile

struct FlashParams {
  int B, H, Hkv, Sq, Sk, D;
  float scale;              // 1/sqrt(D)
  const int* left_pad;      // [B] or nullptr
  __nv_bfloat16* out;       // [B, Sq, H, D] with strides o_sb, o_ss, o_sh (elements)
  long long o_sb, o_ss, o_sh;
  float* lse;               // [B, H, Sq] or nullptr
  int* status;
};

struct FlashCtrl {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full, s_empty, p_full, o_full;
  uint64_t p_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int c0, int c1, int c2,
                                            int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
      "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, float* v) {
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

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
      "%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])),
        "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])),
        "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
        "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
        "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
        "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
        "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// barrier among the two warps that share a block of 32 query rows
__device__ __forceinline__ void pair_bar_sync(int id) {
  asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}

constexpr int kFwdThreads = 320;
constexpr float kRescaleThreshold = 8.f;   // log2 units: P stays below 2^8 between rescales

// D = head_dim (64 or 128). Tiles are stored as D/64 column halves of [rows x 64] bf16, each
// half 128-byte swizzled (what a TMA box {64, rows} produces).
//
// Roles (320 threads):
//   warp 0     TMA producer: Q once, then K / V tiles (128 keys) through two-deep rings
//   warp 1     UMMA issuer:  S = Q K^T (TMEM cols [0,128)),  O += P V (TMEM cols [128,128+D))
//   warps 2-9  softmax: two threads per query row, one per 64-key half of the score tile
//              (warps w and w+4 share rows and TMEM lanes). A thread loads its 64 scores in one
//              trip, the pair exchanges row maxima through shared memory, and P = exp2(S - m)
//              goes to a double-buffered shared-memory tile as the K-major A operand of PV.
// O stays in tensor memory for the whole key loop. The running maximum is only raised -- and O
// multiplied by exp2(m_old - m_new) in place (tcgen05.ld / .st) -- when some row of the warp
// would otherwise exceed 2^8; otherwise the stale maximum keeps being used, which is exact
// after the final division by the row sum. S(j+1) is issued as soon as S(j) is in registers and
// PV(j) only waits for P(j), so the tensor core and the softmax warps overlap.
// Score tiles that lie entirely below the diagonal and right of the left-pad boundary skip the
// visibility tests.
template <int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  constexpr int NH = D / 64;                 // 64-wide halves of the head dimension
  constexpr int kHalfBytes = 128 * 128;      // [128 rows x 64] bf16
  constexpr int kTileBytes = NH * kHalfBytes;
  constexpr int kPBytes = 2 * kHalfBytes;    // P: [128 q x 128 keys]
  constexpr int DH = D / 2;                  // output columns per thread of a row pair
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  FlashCtrl* ctrl = reinterpret_cast<FlashCtrl*>(smem);
  float* xch = reinterpret_cast<float*>(smem + 1024);   // [2 halves][128 rows]
  uint8_t* q_s = smem + 2048;
  uint8_t* k_s = q_s + kTileBytes;           // 2 stages
  uint8_t* v_s = k_s + 2 * kTileBytes;       // 2 stages
  uint8_t* p_s = v_s + 2 * kTileBytes;       // 2 buffers

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the last query tiles meet the most key tiles: launch them first (longest work first)
  const int qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = qb * kBQ;
  const int off = p.Sk - p.Sq;                        // query i sits at key position i + off
  const int lp = p.left_pad ? p.left_pad[b] : 0;
  // key tiles this query block needs: from the left-pad boundary (or the block's own diagonal
  // when the whole block is padding) to the diagonal of its last row
  const int last_key = min(p.Sk - 1, q0 + kBQ - 1 + off);
  const int first_key = max(0, min(lp, q0 + off));
  const int j_begin = first_key / kBK;
  const int j_end = last_key / kBK + 1;
  const int n_j = j_end - j_begin;
  volatile int* abort_flag = &ctrl->abort_flag;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctrl->q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&ctrl->k_full[s]), 1);
      mbar_init(smem_u32(&ctrl->k_empty[s]), 1);
      mbar_init(smem_u32(&ctrl->v_full[s]), 1);
      mbar_init(smem_u32(&ctrl->v_empty[s]), 1);
      mbar_init(smem_u32(&ctrl->p_empty[s]), 1);
    }
    mbar_init(smem_u32(&ctrl->s_full), 1);
    mbar_init(smem_u32(&ctrl->s_empty), 8);   // one arrival per softmax warp
    mbar_init(smem_u32(&ctrl->p_full), 8);
    mbar_init(smem_u32(&ctrl->o_full), 1);
    ctrl->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = ctrl->tmem_base;
  const uint32_t tmem_o = tmem_s + 128;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer ----------------
    mbar_expect_tx(smem_u32(&ctrl->q_full), kTileBytes);
#pragma unroll
    for (int hf = 0; hf < NH; ++hf)
      tma_load_4d(smem_u32(q_s + hf * kHalfBytes), &tmQ, hf * 64, q0, h, b,
                  smem_u32(&ctrl->q_full));
    for (int it = 0; it < n_j; ++it) {
      const int s = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int key0 = (j_begin + it) * kBK;
      if (!mbar_wait(smem_u32(&ctrl->k_empty[s]), ph ^ 1, abort_flag, p.status,
                     kStatusTimeoutEmpty))
        break;
      mbar_expect_tx(smem_u32(&ctrl->k_full[s]), kTileBytes);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf)
        tma_load_4d(smem_u32(k_s + s * kTileBytes + hf * kHalfBytes), &tmK, hf * 64, key0, hk, b,
                    smem_u32(&ctrl->k_full[s]));
      if (!mbar_wait(smem_u32(&ctrl->v_empty[s]), ph ^ 1, abort_flag, p.status,
                     kStatusTimeoutEmpty))
        break;
      mbar_expect_tx(smem_u32(&ctrl->v_full[s]), kTileBytes);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf)
        tma_load_4d(smem_u32(v_s + s * kTileBytes + hf * kHalfBytes), &tmV, hf * 64, key0, hk, b,
                    smem_u32(&ctrl->v_full[s]));
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- UMMA issuer ----------------
    const uint32_t idesc_s = make_idesc_bf16(128, kBK, 0, 0);   // S = Q K^T, both K-major
    const uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);     // O = P V, V is MN-major
    bool ok = mbar_wait(smem_u32(&ctrl->q_full), 0, abort_flag, p.status, kStatusTimeoutFull);
    auto issue_s = [&](int it) {
      const int s = it & 1;
      ok = ok && mbar_wait(smem_u32(&ctrl->k_full[s]), (it >> 1) & 1, abort_flag, p.status,
                           kStatusTimeoutFull);
      if (!ok) return;
      tc_fence_after();
      const uint32_t qa = smem_u32(q_s), ka = smem_u32(k_s + s * kTileBytes);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t o = (kk / 4) * kHalfBytes + (kk % 4) * 32;
        umma_f16_lohi(tmem_s, sw128_desc_lo(qa, 16) + ((o) >> 4), sw128_desc_hi(1024), sw128_desc_lo(ka, 16) + ((o) >> 4), sw128_desc_hi(1024),
                      idesc_s, kk > 0 ? 1u : 0u);
      }
      umma_commit(smem_u32(&ctrl->k_empty[s]));
      umma_commit(smem_u32(&ctrl->s_full));
    };
    if (n_j > 0) issue_s(0);
    for (int it = 0; it < n_j && ok; ++it) {
      const int s = it & 1;
      if (it + 1 < n_j) {
        // S(it) is in the softmax warps' registers: the next score tile may overwrite it
        ok = mbar_wait(smem_u32(&ctrl->s_empty), it & 1, abort_flag, p.status,
                       kStatusTimeoutTmemEmpty);
        if (!ok) break;
        issue_s(it + 1);
        if (!ok) break;
      }
      ok = mbar_wait(smem_u32(&ctrl->p_full), it & 1, abort_flag, p.status, kStatusTimeoutFull) &&
           mbar_wait(smem_u32(&ctrl->v_full[s]), (it >> 1) & 1, abort_flag, p.status,
                     kStatusTimeoutFull);
      if (!ok) break;
      tc_fence_after();
      const uint32_t pa = smem_u32(p_s + (it & 1) * kPBytes);
      const uint32_t va = smem_u32(v_s + s * kTileBytes);
#pragma unroll
      for (int kk = 0; kk < kBK / 16; ++kk) {
        umma_f16_lohi(tmem_o, sw128_desc_lo(pa, 16) + (((kk / 4) * kHalfBytes + (kk % 4) * 32) >> 4), sw128_desc_hi(1024),
                      sw128_desc_lo(va, kHalfBytes) + ((kk * 2048) >> 4), sw128_desc_hi(1024), idesc_o,
                      (it > 0 || kk > 0) ? 1u : 0u);
      }
      umma_commit(smem_u32(&ctrl->v_empty[s]));
      umma_commit(smem_u32(&ctrl->p_empty[it & 1]));
      umma_commit(smem_u32(&ctrl->o_full));
    }
  }

  if (warp >= 2) {
    // ---------------- softmax / output warps ----------------
    const int qrt = warp & 3;
    const int ch = (warp - 2) >> 2;                   // which 64-key half of the score tile
    const int row = qrt * 32 + lane;                  // query row within the block = TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(qrt * 32) << 16;
    const int qi = q0 + row;                          // query index
    const int qpos = qi + off;                        // its key position (diagonal)
    const float sl2 = p.scale * 1.4426950408889634f;  // scale * log2(e)
    float m = -FLT_MAX, l = 0.f;
    bool ok = true;
    for (int it = 0; it < n_j; ++it) {
      const int key0 = (j_begin + it) * kBK;
      if (ok) ok = mbar_wait(smem_u32(&ctrl->s_full), it & 1, abort_flag, p.status,
                             kStatusTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      float sv[64];
      if (ok) {
        tmem_ld_x32(tmem_s + lane_off + ch * 64, sv);
        tmem_ld_x32(tmem_s + lane_off + ch * 64 + 32, sv + 32);
      }
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->s_empty));
      // scores in log2 units; invisible keys become -inf
      const bool full_tile = (key0 + kBK - 1 <= q0 + off) && (key0 >= lp) && (key0 + kBK <= p.Sk);
      float mx = -FLT_MAX;
      if (full_tile) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          sv[i] *= sl2;
          mx = fmaxf(mx, sv[i]);
        }
      } else {
        const int cbase = key0 + ch * 64;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int j = cbase + i;
          const bool vis = (((j <= qpos) && (j >= lp)) || (j == qpos)) && j < p.Sk;
          sv[i] = vis ? sv[i] * sl2 : -INFINITY;
          mx = fmaxf(mx, sv[i]);
        }
      }
      xch[ch * 128 + row] = mx;
      pair_bar_sync(1 + qrt);
      const float m_new = fmaxf(m, fmaxf(mx, xch[(ch ^ 1) * 128 + row]));
      pair_bar_sync(1 + qrt);
      const bool need = (it > 0) && (m != -FLT_MAX) && (m_new - m > kRescaleThreshold);
      if (__any_sync(0xffffffffu, need)) {
        // raise the maximum of all 32 rows of this warp: O *= exp2(m_old - m_new) in place
        const float alpha = (m == -FLT_MAX) ? 1.f : ex2_approx(m - m_new);
        if (ok) ok = mbar_wait(smem_u32(&ctrl->o_full), (it - 1) & 1, abort_flag, p.status,
                               kStatusTimeoutTmemFull);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < DH; c += 32) {
          float ov[32];
          if (ok) tmem_ld_x32(tmem_o + lane_off + ch * DH + c, ov);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] *= alpha;
          if (ok) tmem_st_x32(tmem_o + lane_off + ch * DH + c, ov);
        }
        tmem_st_wait();
        l *= alpha;
        m = m_new;
      } else if (m == -FLT_MAX) {
        m = m_new;                                    // no history yet: nothing to rescale
      }
      const float msafe = (m == -FLT_MAX) ? 0.f : m;
      // P(it) goes to buffer it & 1, free once PV(it - 2) has read it
      if (ok) ok = mbar_wait(smem_u32(&ctrl->p_empty[it & 1]), ((it >> 1) & 1) ^ 1, abort_flag,
                             p.status, kStatusTimeoutEmpty);
      ok = __all_sync(0xffffffffu, ok);
      // [128 x 64] half `ch`, 128-byte rows, 16-byte chunk c at position (c ^ (row & 7))
      uint8_t* prow = p_s + (it & 1) * kPBytes + ch * kHalfBytes + row * 128;
      float rs = 0.f;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = ex2_approx(sv[c8 * 8 + 2 * e] - msafe);
          const float p1 = ex2_approx(sv[c8 * 8 + 2 * e + 1] - msafe);
          rs += p0 + p1;
          const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          packed[e] = *reinterpret_cast<const uint32_t*>(&pk);
        }
        *reinterpret_cast<uint4*>(prow + ((c8 ^ (row & 7)) << 4)) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
      l += rs;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->p_full));
    }
    // ---- epilogue: O / l ----
    if (n_j > 0) {
      if (ok) ok = mbar_wait(smem_u32(&ctrl->o_full), (n_j - 1) & 1, abort_flag, p.status,
                             kStatusTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
    }
    xch[ch * 128 + row] = l;
    pair_bar_sync(1 + qrt);
    const float l_tot = l + xch[(ch ^ 1) * 128 + row];
    const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
    const bool store = ok && qi < p.Sq;
    __nv_bfloat16* orow = p.out + (long long)b * p.o_sb + (long long)qi * p.o_ss +
                          (long long)h * p.o_sh + ch * DH;
#pragma unroll
    for (int c = 0; c < DH; c += 32) {
      float ov[32];
      if (ok && n_j > 0) tmem_ld_x32(tmem_o + lane_off + ch * DH + c, ov);   // warp-uniform
      tmem_ld_wait();
      if (store) {
#pragma unroll
        for (int c8 = 0; c8 < 32; c8 += 8) {
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float a0 = n_j > 0 ? ov[c8 + 2 * e] * inv : 0.f;
            const float a1 = n_j > 0 ? ov[c8 + 2 * e + 1] * inv : 0.f;
            const __nv_bfloat162 pk = __floats2bfloat162_rn(a0, a1);
            packed[e] = *reinterpret_cast<const uint32_t*>(&pk);
          }
          *reinterpret_cast<uint4*>(orow + c + c8) =
              make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
    }
    if (store && ch == 0 && p.lse)
      p.lse[((long long)b * p.H + h) * p.Sq + qi] =
          (l_tot > 0.f) ? (m * 0.6931471805599453f + logf(l_tot)) : -FLT_MAX;
    tc_fence_before();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(ctrl->tmem_base, 256);
}

// =============================================================================================
// Backward pass. Two kernels recompute the probabilities from (Q, K, lse):
//   flash_bwd_dkdv_kernel : one CTA per (batch, kv head, 128-key block); loops over the query
//                           blocks (and the query heads of the group) that see those keys;
//                           dV += P^T dO and dK += dS^T Q accumulate in tensor memory.
//   flash_bwd_dq_kernel   : one CTA per (batch, head, 128-query block); loops over key blocks;
//                           dQ += dS K accumulates in tensor memory.
// with P = exp(S*scale - lse), dP = dO V^T, dS = P o (dP - delta) * scale and
// delta = rowsum(dO o O) from flash_delta_kernel. Splitting the work this way recomputes S and
// dP twice but needs no atomics and is deterministic.
// Shared-memory tiles are [128 rows x 64] bf16 halves with the 128-byte swizzle, so the same
// tile serves as a K-major operand (contraction along the row) or an MN-major operand
// (contraction across rows): P / dS are written once and used both ways.
// =============================================================================================

struct FlashBwdParams {
  int B, H, Hkv, Sq, Sk, D;
  float scale;
  const int* left_pad;
  const float* lse;      // [B, H, Sq]
  const float* delta;    // [B, H, Sq]
  __nv_bfloat16* dq;     // like q   (strides q_sb, q_ss, q_sh)
  __nv_bfloat16* dk;     // like k/v (strides k_sb, k_ss, k_sh)
  __nv_bfloat16* dv;
  long long q_sb, q_ss, q_sh, k_sb, k_ss, k_sh;
  int* status;
};

struct BwdCtrl {
  uint64_t once_full, it_full, it_empty, sdp_full, pds_full, done;
  uint32_t tmem_base;
  int abort_flag;
};

// delta[b, h, i] = sum_d O[b,i,h,d] * dO[b,i,h,d]
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                   const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                   long long sb, long long ss, long long sh, long long dsb,
                                   long long dss, long long dsh, int H, int Sq, int D) {
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int total = gridDim.y * H * Sq;  // gridDim.y = B
  (void)total;
  const int b = blockIdx.y;
  if (warp_global >= H * Sq) return;
  const int h = warp_global / Sq, i = warp_global - h * Sq;
  const __nv_bfloat16* po = o + b * sb + (long long)i * ss + (long long)h * sh;
  const __nv_bfloat16* pd = d_o + b * dsb + (long long)i * dss + (long long)h * dsh;
  float acc = 0.f;
  for (int d = lane; d < D; d += 32) acc += __bfloat162float(po[d]) * __bfloat162float(pd[d]);
  acc = warp_sum(acc);
  if (lane == 0) delta[((long long)b * H + h) * Sq + i] = acc;
}

// bf16 row of 32 values -> swizzled [128 x 64] halves (row-major, 16-byte chunk c at c ^ (row&7))
__device__ __forceinline__ void store_row32(uint8_t* tile, int row, int col0, const float* v) {
#pragma unroll
  for (int c8 = 0; c8 < 4; ++c8) {
    uint32_t packed[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 pk = __floats2bfloat162_rn(v[c8 * 8 + 2 * e], v[c8 * 8 + 2 * e + 1]);
      packed[e] = *reinterpret_cast<const uint32_t*>(&pk);
    }
    const int col8 = (col0 >> 3) + c8;
    const int half = col8 >> 3, chunk = col8 & 7;
    *reinterpret_cast<uint4*>(tile + half * (128 * 128) + row * 128 +
                              ((chunk ^ (row & 7)) << 4)) =
        make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

template <int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                      const FlashBwdParams p) {
  constexpr int NH = D / 64;
  constexpr int kHalf = 128 * 128;
  constexpr int kTile = NH * kHalf;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  BwdCtrl* ctrl = reinterpret_cast<BwdCtrl*>(smem);
  uint8_t* k_s = smem + 1024;
  uint8_t* v_s = k_s + kTile;
  uint8_t* q_s = v_s + kTile;
  uint8_t* do_s = q_s + kTile;
  uint8_t* p_s = do_s + kTile;          // [128 q x 128 keys]
  uint8_t* ds_s = p_s + 2 * kHalf;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int key0 = jb * kBK;
  const int off = p.Sk - p.Sq;
  const int lp = p.left_pad ? p.left_pad[b] : 0;
  const int i_begin = max(0, key0 - off) / kBQ;
  const int n_q = (p.Sq + kBQ - 1) / kBQ;
  const int n_i = max(0, n_q - i_begin);
  const int n_it = n_i * G;
  volatile int* abort_flag = &ctrl->abort_flag;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctrl->once_full), 1);
    mbar_init(smem_u32(&ctrl->it_full), 1);
    mbar_init(smem_u32(&ctrl->it_empty), 1);
    mbar_init(smem_u32(&ctrl->sdp_full), 1);
    mbar_init(smem_u32(&ctrl->pds_full), 8);   // one arrival per compute warp
    mbar_init(smem_u32(&ctrl->done), 1);
    ctrl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm_s = ctrl->tmem_base, tm_dp = tm_s + 128, tm_dv = tm_s + 256, tm_dk = tm_s + 384;

  if (warp == 0 && lane == 0) {
    mbar_expect_tx(smem_u32(&ctrl->once_full), 2 * kTile);
#pragma unroll
    for (int hf = 0; hf < NH; ++hf) {
      tma_load_4d(smem_u32(k_s + hf * kHalf), &tmK, hf * 64, key0, hk, b, smem_u32(&ctrl->once_full));
      tma_load_4d(smem_u32(v_s + hf * kHalf), &tmV, hf * 64, key0, hk, b, smem_u32(&ctrl->once_full));
    }
    for (int it = 0; it < n_it; ++it) {
      const int g = it / n_i, i = i_begin + it % n_i;
      const int h = hk * G + g;
      if (!mbar_wait(smem_u32(&ctrl->it_empty), (it & 1) ^ 1, abort_flag, p.status,
                     kStatusTimeoutEmpty))
        break;
      mbar_expect_tx(smem_u32(&ctrl->it_full), 2 * kTile);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        tma_load_4d(smem_u32(q_s + hf * kHalf), &tmQ, hf * 64, i * kBQ, h, b, smem_u32(&ctrl->it_full));
        tma_load_4d(smem_u32(do_s + hf * kHalf), &tmDO, hf * 64, i * kBQ, h, b, smem_u32(&ctrl->it_full));
      }
    }
  } else if (warp == 1 && lane == 0) {
    const uint32_t id_kk = make_idesc_bf16(128, 128, 0, 0);   // S, dP: both operands K-major
    const uint32_t id_mm = make_idesc_bf16(128, D, 1, 1);     // dV, dK: both MN-major
    bool ok = mbar_wait(smem_u32(&ctrl->once_full), 0, abort_flag, p.status, kStatusTimeoutFull);
    for (int it = 0; it < n_it && ok; ++it) {
      ok = mbar_wait(smem_u32(&ctrl->it_full), it & 1, abort_flag, p.status, kStatusTimeoutFull);
      if (!ok) break;
      tc_fence_after();
      const uint32_t qa = smem_u32(q_s), ka = smem_u32(k_s), va = smem_u32(v_s), da = smem_u32(do_s);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t o = (kk / 4) * kHalf + (kk % 4) * 32;
        umma_f16_lohi(tm_s, sw128_desc_lo(qa, 16) + ((o) >> 4), sw128_desc_hi(1024),
                      sw128_desc_lo(ka, 16) + ((o) >> 4), sw128_desc_hi(1024), id_kk,
                 kk > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t o = (kk / 4) * kHalf + (kk % 4) * 32;
        umma_f16_lohi(tm_dp, sw128_desc_lo(da, 16) + ((o) >> 4), sw128_desc_hi(1024),
                      sw128_desc_lo(va, 16) + ((o) >> 4), sw128_desc_hi(1024), id_kk,
                 kk > 0 ? 1u : 0u);
      }
      umma_commit(smem_u32(&ctrl->sdp_full));
      ok = mbar_wait(smem_u32(&ctrl->pds_full), it & 1, abort_flag, p.status, kStatusTimeoutFull);
      if (!ok) break;
      tc_fence_after();
      const uint32_t pa = smem_u32(p_s), sa = smem_u32(ds_s);
#pragma unroll
      for (int kk = 0; kk < kBQ / 16; ++kk) {   // contraction over the 128 queries
        const uint32_t acc = (it > 0 || kk > 0) ? 1u : 0u;
        umma_f16_lohi(tm_dv, sw128_desc_lo(pa, kHalf) + ((kk * 2048) >> 4), sw128_desc_hi(1024),
                      sw128_desc_lo(da, kHalf) + ((kk * 2048) >> 4), sw128_desc_hi(1024), id_mm, acc);
        umma_f16_lohi(tm_dk, sw128_desc_lo(sa, kHalf) + ((kk * 2048) >> 4), sw128_desc_hi(1024),
                      sw128_desc_lo(qa, kHalf) + ((kk * 2048) >> 4), sw128_desc_hi(1024), id_mm, acc);
      }
      umma_commit(smem_u32(&ctrl->it_empty));
    }
    umma_commit(smem_u32(&ctrl->done));
  }

  if (warp >= 2) {
    const int qrt = warp & 3;
    const int ch = (warp - 2) >> 2;   // 64-column half handled by this thread of the row pair
    const int row = qrt * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(qrt * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int g = it / n_i, i = i_begin + it % n_i;
      const int h = hk * G + g;
      const int qi = i * kBQ + row;
      const int qpos = qi + off;
      const bool q_ok = qi < p.Sq;
      const float lse2 = q_ok ? p.lse[((long long)b * p.H + h) * p.Sq + qi] * 1.4426950408889634f : 0.f;
      const float dl = q_ok ? p.delta[((long long)b * p.H + h) * p.Sq + qi] : 0.f;
      if (ok) ok = mbar_wait(smem_u32(&ctrl->sdp_full), it & 1, abort_flag, p.status,
                             kStatusTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      // interior tiles (all 128 x 128 pairs visible) skip the per-element visibility test
      const bool full_tile = (key0 + kBK - 1 <= i * kBQ + off) && (key0 >= lp) &&
                             (key0 + kBK <= p.Sk) && (i * kBQ + kBQ <= p.Sq);
#pragma unroll
      for (int cc = 0; cc < 64; cc += 32) {
        const int c = ch * 64 + cc;
        float sv[32], dp[32];
        if (ok) {
          tmem_ld_x32(tm_s + lane_off + c, sv);
          tmem_ld_x32(tm_dp + lane_off + c, dp);
        }
        tmem_ld_wait();
        if (full_tile) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float pr = ex2_approx(sv[e] * sl2 - lse2);
            sv[e] = pr;
            dp[e] = pr * (dp[e] - dl) * p.scale;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int j = key0 + c + e;
            const bool vis = q_ok && (((j <= qpos) && (j >= lp)) || (j == qpos)) && j < p.Sk;
            const float pr = vis ? ex2_approx(sv[e] * sl2 - lse2) : 0.f;
            sv[e] = pr;
            dp[e] = pr * (dp[e] - dl) * p.scale;
          }
        }
        store_row32(p_s, row, c, sv);
        store_row32(ds_s, row, c, dp);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->pds_full));
    }
    if (ok) ok = mbar_wait(smem_u32(&ctrl->done), 0, abort_flag, p.status, kStatusTimeoutTmemFull);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const int kj = key0 + row;
    if (ok) {
      __nv_bfloat16* dkrow = p.dk + (long long)b * p.k_sb + (long long)kj * p.k_ss + (long long)hk * p.k_sh;
      __nv_bfloat16* dvrow = p.dv + (long long)b * p.k_sb + (long long)kj * p.k_ss + (long long)hk * p.k_sh;
#pragma unroll
      for (int cc = 0; cc < D / 2; cc += 32) {
        const int c = ch * (D / 2) + cc;
        float a[32], bq[32];
        if (n_it > 0) {
          tmem_ld_x32(tm_dv + lane_off + c, a);
          tmem_ld_x32(tm_dk + lane_off + c, bq);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) a[e] = bq[e] = 0.f;
        }
        if (kj < p.Sk) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint32_t pv[4], pk[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const __nv_bfloat162 x = __floats2bfloat162_rn(a[e + 2 * u], a[e + 2 * u + 1]);
              const __nv_bfloat162 y = __floats2bfloat162_rn(bq[e + 2 * u], bq[e + 2 * u + 1]);
              pv[u] = *reinterpret_cast<const uint32_t*>(&x);
              pk[u] = *reinterpret_cast<const uint32_t*>(&y);
            }
            *reinterpret_cast<uint4*>(dvrow + c + e) = make_uint4(pv[0], pv[1], pv[2], pv[3]);
            *reinterpret_cast<uint4*>(dkrow + c + e) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(ctrl->tmem_base, 512);
}

template <int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const FlashBwdParams p) {
  constexpr int NH = D / 64;
  constexpr int kHalf = 128 * 128;
  constexpr int kTile = NH * kHalf;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  BwdCtrl* ctrl = reinterpret_cast<BwdCtrl*>(smem);
  uint8_t* q_s = smem + 1024;
  uint8_t* do_s = q_s + kTile;
  uint8_t* k_s = do_s + kTile;
  uint8_t* v_s = k_s + kTile;
  uint8_t* ds_s = v_s + kTile;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the last query tiles meet the most key tiles: launch them first (longest work first)
  const int qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = qb * kBQ;
  const int off = p.Sk - p.Sq;
  const int lp = p.left_pad ? p.left_pad[b] : 0;
  const int last_key = min(p.Sk - 1, q0 + kBQ - 1 + off);
  const int first_key = max(0, min(lp, q0 + off));
  const int j_begin = first_key / kBK;
  const int n_it = last_key / kBK + 1 - j_begin;
  volatile int* abort_flag = &ctrl->abort_flag;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&ctrl->once_full), 1);
    mbar_init(smem_u32(&ctrl->it_full), 1);
    mbar_init(smem_u32(&ctrl->it_empty), 1);
    mbar_init(smem_u32(&ctrl->sdp_full), 1);
    mbar_init(smem_u32(&ctrl->pds_full), 8);   // one arrival per compute warp
    mbar_init(smem_u32(&ctrl->done), 1);
    ctrl->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm_s = ctrl->tmem_base, tm_dp = tm_s + 128, tm_dq = tm_s + 256;

  if (warp == 0 && lane == 0) {
    mbar_expect_tx(smem_u32(&ctrl->once_full), 2 * kTile);
#pragma unroll
    for (int hf = 0; hf < NH; ++hf) {
      tma_load_4d(smem_u32(q_s + hf * kHalf), &tmQ, hf * 64, q0, h, b, smem_u32(&ctrl->once_full));
      tma_load_4d(smem_u32(do_s + hf * kHalf), &tmDO, hf * 64, q0, h, b, smem_u32(&ctrl->once_full));
    }
    for (int it = 0; it < n_it; ++it) {
      const int k0 = (j_begin + it) * kBK;
      if (!mbar_wait(smem_u32(&ctrl->it_empty), (it & 1) ^ 1, abort_flag, p.status,
                     kStatusTimeoutEmpty))
        break;
      mbar_expect_tx(smem_u32(&ctrl->it_full), 2 * kTile);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        tma_load_4d(smem_u32(k_s + hf * kHalf), &tmK, hf * 64, k0, hk, b, smem_u32(&ctrl->it_full));
        tma_load_4d(smem_u32(v_s + hf * kHalf), &tmV, hf * 64, k0, hk, b, smem_u32(&ctrl->it_full));
      }
    }
  } else if (warp == 1 && lane == 0) {
    const uint32_t id_kk = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t id_dq = make_idesc_bf16(128, D, 0, 1);     // dQ = dS K: K tile is MN-major
    bool ok = mbar_wait(smem_u32(&ctrl->once_full), 0, abort_flag, p.status, kStatusTimeoutFull);
    for (int it = 0; it < n_it && ok; ++it) {
      ok = mbar_wait(smem_u32(&ctrl->it_full), it & 1, abort_flag, p.status, kStatusTimeoutFull);
      if (!ok) break;
      tc_fence_after();
      const uint32_t qa = smem_u32(q_s), ka = smem_u32(k_s), va = smem_u32(v_s), da = smem_u32(do_s);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t o = (kk / 4) * kHalf + (kk % 4) * 32;
        umma_f16_lohi(tm_s, sw128_desc_lo(qa, 16) + ((o) >> 4), sw128_desc_hi(1024),
                      sw128_desc_lo(ka, 16) + ((o) >> 4), sw128_desc_hi(1024), id_kk,
                 kk > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t o = (kk / 4) * kHalf + (kk % 4) * 32;
        umma_f16_lohi(tm_dp, sw128_desc_lo(da, 16) + ((o) >> 4), sw128_desc_hi(1024),
                      sw128_desc_lo(va, 16) + ((o) >> 4), sw128_desc_hi(1024), id_kk,
                 kk > 0 ? 1u : 0u);
      }
      umma_commit(smem_u32(&ctrl->sdp_full));
      ok = mbar_wait(smem_u32(&ctrl->pds_full), it & 1, abort_flag, p.status, kStatusTimeoutFull);
      if (!ok) break;
      tc_fence_after();
      const uint32_t sa = smem_u32(ds_s);
#pragma unroll
      for (int kk = 0; kk < kBK / 16; ++kk) {   // contraction over the 128 keys
        umma_f16_lohi(tm_dq, sw128_desc_lo(sa, 16) + (((kk / 4) * kHalf + (kk % 4) * 32) >> 4), sw128_desc_hi(1024),
                      sw128_desc_lo(ka, kHalf) + ((kk * 2048) >> 4), sw128_desc_hi(1024), id_dq, (it > 0 || kk > 0) ? 1u : 0u);
      }
      umma_commit(smem_u32(&ctrl->it_empty));
    }
    umma_commit(smem_u32(&ctrl->done));
  }

  if (warp >= 2) {
    const int qrt = warp & 3;
    const int ch = (warp - 2) >> 2;   // 64-column half handled by this thread of the row pair
    const int row = qrt * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(qrt * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    const int qi = q0 + row, qpos = qi + off;
    const bool q_ok = qi < p.Sq;
    const float lse2 = q_ok ? p.lse[((long long)b * p.H + h) * p.Sq + qi] * 1.4426950408889634f : 0.f;
    const float dl = q_ok ? p.delta[((long long)b * p.H + h) * p.Sq + qi] : 0.f;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int key0 = (j_begin + it) * kBK;
      if (ok) ok = mbar_wait(smem_u32(&ctrl->sdp_full), it & 1, abort_flag, p.status,
                             kStatusTimeoutTmemFull);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      const bool full_tile = (key0 + kBK - 1 <= q0 + off) && (key0 >= lp) &&
                             (key0 + kBK <= p.Sk) && (q0 + kBQ <= p.Sq);
#pragma unroll
      for (int cc = 0; cc < 64; cc += 32) {
        const int c = ch * 64 + cc;
        float sv[32], dp[32];
        if (ok) {
          tmem_ld_x32(tm_s + lane_off + c, sv);
          tmem_ld_x32(tm_dp + lane_off + c, dp);
        }
        tmem_ld_wait();
        if (full_tile) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            dp[e] = ex2_approx(sv[e] * sl2 - lse2) * (dp[e] - dl) * p.scale;
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int j = key0 + c + e;
            const bool vis = q_ok && (((j <= qpos) && (j >= lp)) || (j == qpos)) && j < p.Sk;
            const float pr = vis ? ex2_approx(sv[e] * sl2 - lse2) : 0.f;
            dp[e] = pr * (dp[e] - dl) * p.scale;
          }
        }
        store_row32(ds_s, row, c, dp);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->pds_full));
    }
    if (ok) ok = mbar_wait(smem_u32(&ctrl->done), 0, abort_flag, p.status, kStatusTimeoutTmemFull);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (ok) {   // warp-uniform: the TMEM loads are warp-collective, only the stores are per row
      __nv_bfloat16* dqrow = p.dq + (long long)b * p.q_sb + (long long)qi * p.q_ss + (long long)h * p.q_sh;
#pragma unroll
      for (int cc = 0; cc < D / 2; cc += 32) {
        const int c = ch * (D / 2) + cc;
        float a[32];
        if (n_it > 0) {
          tmem_ld_x32(tm_dq + lane_off + c, a);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) a[e] = 0.f;
        }
        if (!q_ok) continue;
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint32_t pk[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const __nv_bfloat162 x = __floats2bfloat162_rn(a[e + 2 * u], a[e + 2 * u + 1]);
            pk[u] = *reinterpret_cast<const uint32_t*>(&x);
          }
          *reinterpret_cast<uint4*>(dqrow + c + e) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(ctrl->tmem_base, 512);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn flash_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// [B, S, H, D] view with element strides (sb, ss, sh), D contiguous: dims {D, S, H, B}.
static int make_map4d(CUtensorMap* m, const void* base, int D, int S, int H, int B, long long sb,
                      long long ss, long long sh, int box_rows) {
  EncodeTiledFn fn = flash_encode_fn();
  if (!fn) return -10;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, 1u, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -11;
}

}  // namespace e2h

// q: [B, Sq, H, D] view (strides q_sb, q_ss, q_sh); k, v: [B, Sk, Hkv, D] views; out like q.
extern "C" int e2h_flash_fwd(const void* q, long long q_sb, long long q_ss, long long q_sh,
                             const void* k, const void* v, long long k_sb, long long k_ss,
                             long long k_sh, void* out, long long o_sb, long long o_ss,
                             long long o_sh, float* lse, const int* left_pad, int B, int H,
                             int Hkv, int Sq, int Sk, int D, float scale, int* status,
                             void* stream) {
  using namespace e2h;
  if (D != 128 && D != 64) return -1;
  if (H % Hkv) return -2;
  if ((q_ss % 8) || (q_sh % 8) || (q_sb % 8) || (k_ss % 8) || (k_sh % 8) || (k_sb % 8)) return -3;
  CUtensorMap tq, tk, tv;
  int r = make_map4d(&tq, q, D, Sq, H, B, q_sb, q_ss, q_sh, kBQ);
  if (r) return r;
  r = make_map4d(&tk, k, D, Sk, Hkv, B, k_sb, k_ss, k_sh, kBK);
  if (r) return r;
  r = make_map4d(&tv, v, D, Sk, Hkv, B, k_sb, k_ss, k_sh, kBK);
  if (r) return r;
  FlashParams p;
  p.B = B; p.H = H; p.Hkv = Hkv; p.Sq = Sq; p.Sk = Sk; p.D = D;
  p.scale = scale; p.left_pad = left_pad;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.o_sb = o_sb; p.o_ss = o_ss; p.o_sh = o_sh;
  p.lse = lse; p.status = status;
  dim3 grid((Sq + kBQ - 1) / kBQ, H, B);
  const int tile = (D / 64) * 128 * 128;
  const size_t smem = 1024 + 2048 + 5 * (size_t)tile + 2 * (2 * 128 * 128);
  cudaError_t e;
  if (D == 128) {
    static bool done = false;
    if (!done) {
      e = cudaFuncSetAttribute(flash_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)smem);
      if (e != cudaSuccess) return (int)e;
      done = true;
    }
    flash_fwd_kernel<128><<<grid, kFwdThreads, smem, (cudaStream_t)stream>>>(tq, tk, tv, p);
  } else {
    static bool done = false;
    if (!done) {
      e = cudaFuncSetAttribute(flash_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)smem);
      if (e != cudaSuccess) return (int)e;
      done = true;
    }
    flash_fwd_kernel<64><<<grid, kFwdThreads, smem, (cudaStream_t)stream>>>(tq, tk, tv, p);
  }
  return (int)cudaGetLastError();
}

// dO, O: [B, Sq, H, D] views; dq like q; dk, dv like k. delta: fp32 scratch [B, H, Sq].
extern "C" int e2h_flash_bwd(const void* q, long long q_sb, long long q_ss, long long q_sh,
                             const void* k, const void* v, long long k_sb, long long k_ss,
                             long long k_sh, const void* o, long long o_sb, long long o_ss,
                             long long o_sh, const void* d_o, long long do_sb, long long do_ss,
                             long long do_sh, const float* lse, float* delta, void* dq, void* dk,
                             void* dv, const int* left_pad, int B, int H, int Hkv, int Sq, int Sk,
                             int D, float scale, int* status, void* stream_v) {
  using namespace e2h;
  cudaStream_t stream = (cudaStream_t)stream_v;
  if (D != 128 && D != 64) return -1;
  if (H % Hkv) return -2;
  CUtensorMap tq, tk, tv, tdo;
  int r = make_map4d(&tq, q, D, Sq, H, B, q_sb, q_ss, q_sh, kBQ);
  if (r) return r;
  r = make_map4d(&tk, k, D, Sk, Hkv, B, k_sb, k_ss, k_sh, kBK);
  if (r) return r;
  r = make_map4d(&tv, v, D, Sk, Hkv, B, k_sb, k_ss, k_sh, kBK);
  if (r) return r;
  r = make_map4d(&tdo, d_o, D, Sq, H, B, do_sb, do_ss, do_sh, kBQ);
  if (r) return r;
  {
    const int warps = H * Sq;
    dim3 grid((warps * 32 + 255) / 256, B);
    flash_delta_kernel<<<grid, 256, 0, stream>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, o_sb, o_ss, o_sh, do_sb, do_ss,
        do_sh, H, Sq, D);
  }
  FlashBwdParams p;
  p.B = B; p.H = H; p.Hkv = Hkv; p.Sq = Sq; p.Sk = Sk; p.D = D;
  p.scale = scale; p.left_pad = left_pad; p.lse = lse; p.delta = delta;
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.q_sb = q_sb; p.q_ss = q_ss; p.q_sh = q_sh; p.k_sb = k_sb; p.k_ss = k_ss; p.k_sh = k_sh;
  p.status = status;
  const int tile = (D / 64) * 128 * 128;
  const size_t smem_kv = 2048 + 4 * (size_t)tile + 4 * 128 * 128;
  const size_t smem_q = 2048 + 4 * (size_t)tile + 2 * 128 * 128;
  dim3 gkv((Sk + kBK - 1) / kBK, Hkv, B), gq((Sq + kBQ - 1) / kBQ, H, B);
  cudaError_t e;
#define E2H_BWD(D_)                                                                              \
  {                                                                                              \
    static bool done = false;                                                                    \
    if (!done) {                                                                                 \
      e = cudaFuncSetAttribute(flash_bwd_dkdv_kernel<D_>,                                        \
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv);       \
      if (e != cudaSuccess) return (int)e;                                                       \
      e = cudaFuncSetAttribute(flash_bwd_dq_kernel<D_>,                                          \
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q);        \
      if (e != cudaSuccess) return (int)e;                                                       \
      done = true;                                                                               \
    }                                                                                            \
    flash_bwd_dkdv_kernel<D_><<<gkv, kFwdThreads, smem_kv, stream>>>(tq, tk, tv, tdo, p);                \
    flash_bwd_dq_kernel<D_><<<gq, kFwdThreads, smem_q, stream>>>(tq, tk, tv, tdo, p);                    \
  }
  if (D == 128) E2H_BWD(128) else E2H_BWD(64)
#undef E2H_BWD
  return (int)cudaGetLastError();
}
