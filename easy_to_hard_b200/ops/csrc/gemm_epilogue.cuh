// Fused GEMM epilogues shared by the tcgen05 GEMM kernels: one thread owns one output feature
// (its TMEM lane) and applies the epilogue to 8 consecutive token columns at a time.
#pragma once
#include <cuda_bf16.h>

#include "gemm_umma.cuh"
#include "ptx.cuh"

namespace e2h {

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
    if constexpr (DUAL) {   // second weight matrix: its per-feature scales follow the first F
      const float s2 = f_ok ? p.scale[p.F + f] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) v2[j] *= s2;
    }
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
      // all residual loads first: `out` may alias `res`, so a load placed after a store could
      // not be moved above it and the eight round trips would run one after another
      float r[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = t0 + j;
        r[j] = (f_ok && t < p.T) ? __bfloat162float(res[(long long)t * p.ldo + f]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = t0 + j;
        if (f_ok && t < p.T)
          out[(long long)t * p.ldo + f] = __float2bfloat16_rn(bf16_round(v[j]) + r[j]);
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
        if (t0 + 8 <= p.T && (reinterpret_cast<uintptr_t>(row + t0) & 15) == 0) {
          float4* dst = reinterpret_cast<float4*>(row + t0);
          float4 lo = make_float4(v[0], v[1], v[2], v[3]);
          float4 hi = make_float4(v[4], v[5], v[6], v[7]);
          if (p.accumulate) {
            const float4 a = dst[0], b = dst[1];
            lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
            hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
          }
          dst[0] = lo;
          dst[1] = hi;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int t = t0 + j;
            if (t < p.T) row[t] = p.accumulate ? row[t] + v[j] : v[j];
          }
        }
      }
    } break;
    case E2H_EPI_ROWMAJOR_BF16: {
      __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
      if (f_ok) {
        __nv_bfloat16* row = out + (long long)f * p.ldo;
        if (t0 + 8 <= p.T && (reinterpret_cast<uintptr_t>(row + t0) & 15) == 0) {
          uint4 pk;
          uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * h], v[2 * h + 1]);
            w[h] = *reinterpret_cast<uint32_t*>(&two);
          }
          *reinterpret_cast<uint4*>(row + t0) = pk;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int t = t0 + j;
            if (t < p.T) row[t] = __float2bfloat16_rn(v[j]);
          }
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
      const __nv_bfloat162* freqs2 = static_cast<const __nv_bfloat162*>(p.freqs);  // (cos, sin)
      const int pos0 = *p.pos_base;
      const int hk = is_k ? head - p.n_head : head - p.n_head - p.n_kv;
      __nv_bfloat16* cache = static_cast<__nv_bfloat16*>(is_k ? p.kcache : p.vcache);
      // one division per 8 tokens: (sequence, offset) advance incrementally
      int b = t0 / p.sq;
      int s = t0 - b * p.sq;
      // rotation factors first (loads placed after the cache stores could not be hoisted)
      float cj[8], sj[8];
      int posj[8], bj[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        posj[j] = pos0 + s;
        bj[j] = b;
        if (++s == p.sq) {
          s = 0;
          ++b;
        }
        cj[j] = 1.f;
        sj[j] = 0.f;
        if (!is_v && f_ok && t0 + j < p.T) {
          const __nv_bfloat162 cs = freqs2[(long long)posj[j] * (D / 2) + (d >> 1)];
          cj[j] = __bfloat162float(cs.x);
          sj[j] = __bfloat162float(cs.y);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = t0 + j;
        const float x = bf16_round(v[j]);
        const float partner = __shfl_xor_sync(0xffffffffu, x, 1);
        if (!(f_ok && t < p.T)) continue;
        float y = x;
        if (!is_v) y = (d & 1) ? (x * cj[j] + partner * sj[j]) : (x * cj[j] - partner * sj[j]);
        const __nv_bfloat16 yb = __float2bfloat16_rn(y);
        if (is_q) {
          static_cast<__nv_bfloat16*>(p.out)[(long long)t * p.ldo + f] = yb;
        } else if (posj[j] < p.smax) {
          cache[(((long long)bj[j] * p.n_kv + hk) * p.smax + posj[j]) * D + d] = yb;
        }
      }
    } break;
    default:
      break;
  }
}

// ---------------------------------------------------------------------------------------------
// Staged form of the token-major bf16 epilogues (plain store, residual, SwiGLU, RoPE + KV cache)
// for the one-tile-per-CTA kernel. One thread owns one output feature, so writing its values
// straight to global memory is 2-byte stores one token row apart: measured on B200, 64 such
// stores per thread cost 4-9 us per CTA, a quarter of a decode GEMM. Instead every thread puts
// its values into a [tokens][features] tile in shared memory (stage8) and the four epilogue
// warps then move the tile with 16-byte accesses, 8 consecutive features of one token per
// thread (flush_tile): full 32-byte sectors, and the residual is read the same way.

// True when this launch can take the staged path: bf16 token-major output whose rows and tile
// origins are 16-byte aligned.
__host__ __device__ inline bool epi_can_stage(const E2hGemmParams& p, int tile_rows) {
  if (p.epi != E2H_EPI_STORE_BF16 && p.epi != E2H_EPI_RESIDUAL && p.epi != E2H_EPI_SWIGLU &&
      p.epi != E2H_EPI_ROPE_KV)
    return false;
  if ((p.F & 7) || (p.ldo & 7) || (tile_rows & 7)) return false;
  if (reinterpret_cast<uintptr_t>(p.out) & 15) return false;
  if (p.epi == E2H_EPI_RESIDUAL && (reinterpret_cast<uintptr_t>(p.aux) & 15)) return false;
  if (p.epi == E2H_EPI_ROPE_KV &&
      ((p.head_dim & 7) || (reinterpret_cast<uintptr_t>(p.kcache) & 15) ||
       (reinterpret_cast<uintptr_t>(p.vcache) & 15)))
    return false;
  return true;
}

// What the RoPE + KV-cache epilogue needs per thread (one feature), fetched once per tile
// instead of once per 8 token columns: the cache position and, when every sequence
// contributes one token (decode), the one (cos, sin) pair that rotates all of them.
struct RopePre {
  int pos0;       // cache position of the first token of every sequence
  int d;          // index of the feature inside its head
  int is_v;       // value head: stored as it is
  float cj, sj;   // decode (p.sq == 1): rotation factors of position pos0
};

__device__ __forceinline__ RopePre rope_prepare(const E2hGemmParams& p, int f) {
  RopePre r;
  const int D = p.head_dim;
  const int head = f / D;
  r.d = f - head * D;
  r.is_v = head >= p.n_head + p.n_kv ? 1 : 0;
  r.pos0 = *p.pos_base;
  r.cj = 1.f;
  r.sj = 0.f;
  if (p.sq == 1 && !r.is_v && f < p.F && r.pos0 < p.smax && r.pos0 >= 0) {
    const __nv_bfloat162 cs =
        static_cast<const __nv_bfloat162*>(p.freqs)[(long long)r.pos0 * (D / 2) + (r.d >> 1)];
    r.cj = __bfloat162float(cs.x);
    r.sj = __bfloat162float(cs.y);
  }
  return r;
}

// Final bf16 value of 8 consecutive tokens of one feature into the shared tile:
// tile[(tl + j) * pitch + row] for j < 8 (row < 0: a lane without a feature, nothing is
// written). The residual of E2H_EPI_RESIDUAL is added by flush_tile. All 32 lanes must call
// (the RoPE partner value comes from the neighbouring lane).
template <bool DUAL>
__device__ __forceinline__ void stage8(const E2hGemmParams& p, int f, int t0, float* v, float* v2,
                                       __nv_bfloat16* tile, int tl, int pitch, int row,
                                       const RopePre* rope = nullptr) {
  const bool f_ok = f < p.F;
  if (p.scale != nullptr) {
    const float s = f_ok ? p.scale[f] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= s;
    if constexpr (DUAL) {
      const float s2 = f_ok ? p.scale[p.F + f] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) v2[j] *= s2;
    }
  }
  float y[8];
  if (p.epi == E2H_EPI_SWIGLU) {
    if constexpr (DUAL) {
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = bf16_round(silu(bf16_round(v[j]))) * bf16_round(v2[j]);
    }
  } else if (p.epi == E2H_EPI_ROPE_KV) {
    const RopePre rp = rope ? *rope : rope_prepare(p, f);
    const int D = p.head_dim;
    if (p.sq == 1) {
      // decode: every token sits at cache position pos0
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x = bf16_round(v[j]);
        const float partner = __shfl_xor_sync(0xffffffffu, x, 1);
        y[j] = rp.is_v ? x
                       : ((rp.d & 1) ? (x * rp.cj + partner * rp.sj) : (x * rp.cj - partner * rp.sj));
      }
    } else {
      int b = t0 / p.sq;
      int s_ = t0 - b * p.sq;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int pos = rp.pos0 + s_;
        if (++s_ == p.sq) s_ = 0;
        float cj = 1.f, sj = 0.f;
        if (!rp.is_v && f_ok && t0 + j < p.T && pos < p.smax) {
          const __nv_bfloat162 cs =
              static_cast<const __nv_bfloat162*>(p.freqs)[(long long)pos * (D / 2) + (rp.d >> 1)];
          cj = __bfloat162float(cs.x);
          sj = __bfloat162float(cs.y);
        }
        const float x = bf16_round(v[j]);
        const float partner = __shfl_xor_sync(0xffffffffu, x, 1);
        y[j] = rp.is_v ? x : ((rp.d & 1) ? (x * cj + partner * sj) : (x * cj - partner * sj));
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = v[j];
  }
  if (row < 0) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) tile[(tl + j) * pitch + row] = __float2bfloat16_rn(y[j]);
}

// Moves the staged tile (rows = tokens t_first .. t_first + n_tok, columns = features f_first ..
// f_first + pitch) to its destination, 16 bytes per access. `tid` / `nthreads`: the calling
// thread's index among the epilogue threads, which have synchronised after stage8.
__device__ __forceinline__ void flush_tile(const E2hGemmParams& p, const __nv_bfloat16* tile,
                                           int pitch, int f_first, int t_first, int n_tok,
                                           int tid, int nthreads) {
  const int vpr = pitch >> 3;
  const int total = n_tok * vpr;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
  const int pos0 = (p.epi == E2H_EPI_ROPE_KV) ? *p.pos_base : 0;
  for (int i = tid; i < total; i += nthreads) {
    const int r = i / vpr;
    const int fv = (i - r * vpr) << 3;
    const int t = t_first + r, f = f_first + fv;
    if (t >= p.T || f >= p.F) continue;
    uint4 val = *reinterpret_cast<const uint4*>(tile + r * pitch + fv);
    __nv_bfloat16* dst = out + (long long)t * p.ldo + f;
    if (p.epi == E2H_EPI_RESIDUAL) {
      const uint4 res = *reinterpret_cast<const uint4*>(
          static_cast<const __nv_bfloat16*>(p.aux) + (long long)t * p.ldo + f);
      const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&val);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&res);
      uint4 sum;
      __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&sum);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        o[k] = __floats2bfloat162_rn(__bfloat162float(a[k].x) + __bfloat162float(b[k].x),
                                     __bfloat162float(a[k].y) + __bfloat162float(b[k].y));
      val = sum;
    } else if (p.epi == E2H_EPI_ROPE_KV) {
      const int D = p.head_dim;
      const int head = f / D;
      const int d = f - head * D;
      if (head >= p.n_head) {
        const bool is_k = head < p.n_head + p.n_kv;
        const int hk = is_k ? head - p.n_head : head - p.n_head - p.n_kv;
        const int b = t / p.sq;
        const int pos = pos0 + (t - b * p.sq);
        if (pos >= p.smax) continue;
        __nv_bfloat16* cache = static_cast<__nv_bfloat16*>(is_k ? p.kcache : p.vcache);
        dst = cache + (((long long)b * p.n_kv + hk) * p.smax + pos) * D + d;
      }
    }
    *reinterpret_cast<uint4*>(dst) = val;
  }
}

}  // namespace e2h
