// Fused sampler: temperature, top-k pivot mask, exponential-race sampling, EOS tracking and
// position advance, one CTA per sequence, no host synchronisation.
//
// Semantics of the reference sampler (models/rl_model.py:347-379, inference_generate.py:53-85):
//   logits / max(T, 1e-5); pivot = k-th largest; values < pivot are dropped (ties with the
//   pivot are kept); probabilities p = softmax; token = argmax(p / q), q ~ Exp(1) i.i.d.
// argmax(p/q) does not depend on the softmax normaliser, so the kernel maximises
//   x_i / T - log(q_i)          over the kept entries
// and never materialises probabilities. Greedy decoding (temperature == 0) is the plain
// argmax with ties going to the lowest index.
//
// The k-th largest value is found exactly. Fast path (row in shared memory, top_k <= 256): the
// k-th largest of 256 group maxima is a lower bound of the pivot (at least k entries reach it),
// so only the handful of entries at or above it are collected (typically 50-70 of 32016) and
// the pivot is picked among them by rank counting; the sampling pass then also runs over those
// candidates only. Otherwise, or if more than 2048 entries reach the bound (many equal logits):
// a 4-pass, 8-bit radix select over the order-preserving integer image of the fp32 logits. The row (128 KB at a 32k vocabulary) is
// copied into shared memory once with 16-byte loads and all five passes read it from there: the
// passes are chains of dependent loads (a warp-wide match between them), which from L2 cost
// ~13 us per pass and ~100 us per step; rows that do not fit stay in global memory.
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>
#include <mutex>

#include "launch.cuh"
#include "ptx.cuh"

namespace e2h {

__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // larger float -> larger key
}

// Philox4x32-10 counter-based generator.
__device__ __forceinline__ uint4 philox(uint4 ctr, uint2 key) {
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += 0x9E3779B9u;
    key.y += 0xBB67AE85u;
  }
  return ctr;
}

constexpr int kSampThreads = 1024;
constexpr int kSampMaxSmemRow = 188 * 1024;     // bytes of one logits row kept in shared memory
constexpr int kSampGroups = 256;                // group maxima of the fast path
constexpr int kSampCandMax = 2048;              // candidates the fast path can hold

// logits   : fp32 [B, ld]
// pos_ptr  : device scalar, position of the token that produced these logits; the sampled
//            token is stored at seq[b, pos+1]; the last CTA to finish stores pos+1 back.
// next_tok : int32 [B], input of the next decode step
// eos_flag : int32 [B], sticky
__global__ void __launch_bounds__(kSampThreads)
sample_kernel(const float* __restrict__ logits, long long ld, int vocab, float temperature,
              int top_k, unsigned long long seed, int* pos_ptr, int advance_pos,
              int* __restrict__ next_tok, int* __restrict__ seq, long long seq_ld, int seq_len,
              int eos_id, int* __restrict__ eos_flag, int* __restrict__ n_unfinished,
              unsigned int* ticket, const unsigned long long* __restrict__ seed_ptr,
              int row_in_smem) {
  extern __shared__ __align__(16) float srow[];
  __shared__ unsigned int hist[256];
  // one histogram per warp: the logits crowd into two or three exponent bins, and a thousand
  // atomics on one shared-memory word from 32 warps serialise (20 us of the 37 us this kernel
  // took with a single histogram)
  __shared__ unsigned int whist[kSampThreads / 32][256];
  __shared__ uint32_t sh_prefix, sh_remaining;
  // the fast path's arrays live in the radix histograms' storage (the two never overlap in time)
  static_assert(kSampThreads + 2 * kSampCandMax <= (kSampThreads / 32) * 256, "fast-path arrays");
  uint32_t* gmax = &whist[0][0];                 // per-thread, then per-group maximum keys
  uint32_t* cand_key = gmax + kSampThreads;
  int* cand_idx = reinterpret_cast<int*>(cand_key + kSampCandMax);
  __shared__ uint32_t sh_bound, sh_pivot;
  __shared__ int n_cand;
  __shared__ float red_v[kSampThreads / 32];
  __shared__ int red_i[kSampThreads / 32];
  const int b = blockIdx.x;
  const float* row = logits + (long long)b * ld;
  pdl_wait_prior();
  pdl_launch_dependents();
  if (row_in_smem) {
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      const float4* src4 = reinterpret_cast<const float4*>(row);
      float4* dst4 = reinterpret_cast<float4*>(srow);
      for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) dst4[i] = src4[i];
      for (int i = (vocab & ~3) + threadIdx.x; i < vocab; i += blockDim.x) srow[i] = row[i];
    } else {
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) srow[i] = row[i];
    }
    __syncthreads();
    row = srow;
  }
  const int pos = *pos_ptr;
  // a seed kept in device memory lets one captured graph serve every generation call
  if (seed_ptr != nullptr) seed = *seed_ptr;
  const bool greedy = temperature <= 0.f;

  uint32_t pivot_key = 0;  // keep everything
  bool have_cands = false; // the entries >= pivot_key are (among) the first n_cand candidates
  if (!greedy && top_k > 0 && top_k < vocab && row_in_smem && top_k <= kSampGroups) {
    // ---- fast path
    uint32_t lm = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) lm = max(lm, float_key(row[i]));
    gmax[threadIdx.x] = lm;
    if (threadIdx.x == 0) n_cand = 0;
    __syncthreads();
    if (threadIdx.x < kSampGroups) {
      uint32_t g = lm;
      for (int t = threadIdx.x + kSampGroups; t < kSampThreads; t += kSampGroups) g = max(g, gmax[t]);
      lm = g;
    }
    __syncthreads();
    if (threadIdx.x < kSampGroups) gmax[threadIdx.x] = lm;
    __syncthreads();
    if (threadIdx.x < kSampGroups) {
      // rank of this group's maximum among the 256 (ties broken by group index): the one of
      // rank top_k - 1 is the bound
      int gt = 0;
      for (int j = 0; j < kSampGroups; ++j) {
        const uint32_t o = gmax[j];
        gt += (o > lm || (o == lm && j < (int)threadIdx.x)) ? 1 : 0;
      }
      if (gt == top_k - 1) sh_bound = lm;
    }
    __syncthreads();
    const uint32_t bound = sh_bound;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const uint32_t key = float_key(row[i]);
      if (key >= bound) {
        const int slot = atomicAdd(&n_cand, 1);
        if (slot < kSampCandMax) {
          cand_key[slot] = key;
          cand_idx[slot] = i;
        }
      }
    }
    __syncthreads();
    const int n = n_cand;
    if (n <= kSampCandMax) {
      // the k-th largest key: the candidate with fewer than k keys above it and at least k at
      // or above it (all such candidates carry the same key)
      for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const uint32_t v = cand_key[c];
        int above = 0, at_or_above = 0;
        for (int j = 0; j < n; ++j) {
          const uint32_t o = cand_key[j];
          above += o > v ? 1 : 0;
          at_or_above += o >= v ? 1 : 0;
        }
        if (above < top_k && top_k <= at_or_above) sh_pivot = v;
      }
      __syncthreads();
      pivot_key = sh_pivot;
      have_cands = true;
    }
  }
  if (!greedy && top_k > 0 && top_k < vocab && !have_cands) {
    // radix select of the k-th largest key, most significant byte first
    uint32_t prefix = 0, mask = 0;
    uint32_t remaining = top_k;
    for (int shift = 24; shift >= 0; shift -= 8) {
      unsigned int* mine = whist[threadIdx.x >> 5];
      for (int i = threadIdx.x & 31; i < 256; i += 32) mine[i] = 0;
      __syncwarp();
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const uint32_t key = float_key(row[i]);
        if ((key & mask) == prefix) {
          // lanes that hit the same bin elect one of them to add their count
          const uint32_t bin = (key >> shift) & 255u;
          const unsigned peers = __match_any_sync(__activemask(), bin);
          if ((threadIdx.x & 31) == (unsigned)(__ffs(peers) - 1)) atomicAdd(&mine[bin], __popc(peers));
        }
      }
      __syncthreads();
      if (threadIdx.x < 256) {
        unsigned int sum = 0;
#pragma unroll 8
        for (int w = 0; w < kSampThreads / 32; ++w) sum += whist[w][threadIdx.x];
        hist[threadIdx.x] = sum;
      }
      __syncthreads();
      if (threadIdx.x < 32) {
        // the bin that holds the `remaining`-th largest key: lane l owns bins 8l..8l+7, a
        // suffix sum over the lanes finds the lane, a short scan the bin
        const int l = threadIdx.x;
        uint32_t mine = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) mine += hist[8 * l + j];
        uint32_t above = mine;                 // keys in bins >= 8l (suffix sum, inclusive)
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t y = __shfl_down_sync(0xffffffffu, above, o);
          if (l + o < 32) above += y;
        }
        const bool has = above >= remaining;   // true for lanes 0..L, L = the lane we want
        const unsigned m = __ballot_sync(0xffffffffu, has);
        const int L = m ? 31 - __clz(m) : 0;
        if (l == L) {
          uint32_t rem = remaining - (above - mine);   // rank inside this lane's bins
          int bin = 8 * l + 7;
          for (; bin > 8 * l; --bin) {
            if (hist[bin] >= rem) break;
            rem -= hist[bin];
          }
          if (!m) {          // fewer keys than asked for (cannot happen with top_k < vocab)
            bin = 0;
            rem = 1;
          }
          sh_prefix = prefix | (static_cast<uint32_t>(bin) << shift);
          sh_remaining = rem;
        }
      }
      __syncthreads();
      prefix = sh_prefix;
      remaining = sh_remaining;
      mask |= 255u << shift;
    }
    pivot_key = prefix;
  }

  const float inv_t = greedy ? 1.f : 1.f / fmaxf(temperature, 1e-5f);
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  const int n_scan = have_cands ? n_cand : vocab;
  for (int c = threadIdx.x; c < n_scan; c += blockDim.x) {
    const int i = have_cands ? cand_idx[c] : c;
    const float x = row[i];
    if (float_key(x) < pivot_key) continue;
    float score = x * inv_t;
    if (!greedy) {
      const uint4 r = philox(make_uint4((uint32_t)i, (uint32_t)b, (uint32_t)pos, 0u),
                             make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
      const float u = (static_cast<float>(r.x >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0,1)
      const float qexp = -__logf(u);                                                  // Exp(1)
      score -= __logf(qexp);
    }
    if (score > best || (score == best && i < best_i)) {
      best = score;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    red_v[warp] = best;
    red_i[warp] = best_i;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kSampThreads / 32; ++w) {
      if (red_v[w] > best || (red_v[w] == best && red_i[w] < best_i)) {
        best = red_v[w];
        best_i = red_i[w];
      }
    }
    const int tok = best_i;
    next_tok[b] = tok;
    if (seq != nullptr && pos + 1 < seq_len) seq[(long long)b * seq_ld + pos + 1] = tok;
    if (eos_flag != nullptr && eos_id >= 0 && tok == eos_id) {
      if (atomicExch(&eos_flag[b], 1) == 0 && n_unfinished != nullptr)
        atomicSub(n_unfinished, 1);
    }
    if (advance_pos) {
      __threadfence();
      const unsigned int done = atomicAdd(ticket, 1u);
      if (done == gridDim.x - 1) {  // every CTA has read *pos_ptr by now
        *ticket = 0;
        *pos_ptr = pos + 1;
      }
    }
  }
}

}  // namespace e2h

extern "C" int e2h_sample(const float* logits, long long ld, int B, int vocab, float temperature,
                          int top_k, unsigned long long seed, int* pos_ptr, int advance_pos,
                          int* next_tok, int* seq, long long seq_ld, int seq_len, int eos_id,
                          int* eos_flag, int* n_unfinished, unsigned int* ticket,
                          const unsigned long long* seed_ptr, void* stream) {
  using namespace e2h;
  if (advance_pos && ticket == nullptr) return -1;
  const size_t row_bytes = ((size_t)vocab * 4 + 15) / 16 * 16;
  const int in_smem = row_bytes <= (size_t)kSampMaxSmemRow ? 1 : 0;
  if (in_smem) {
    static std::mutex mu;
    static bool asked[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !asked[dev]) {
      e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kSampMaxSmemRow);
      if (e != cudaSuccess) return (int)e;
      asked[dev] = true;
    }
  }
  return (int)launch(sample_kernel, dim3(B), dim3(kSampThreads), in_smem ? row_bytes : 0,
                     (cudaStream_t)stream, logits, ld, vocab, temperature, top_k, seed, pos_ptr,
                     advance_pos, next_tok, seq, seq_ld, seq_len, eos_id, eos_flag, n_unfinished,
                     ticket, seed_ptr, in_smem);
}
