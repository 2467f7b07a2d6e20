// Parameter block shared by the tcgen05 GEMM kernel and its C entry points.
#pragma once
#include <stdint.h>

// The GEMM computes, for a "feature" operand A[F, K] and a "token" operand B[T, K],
//     acc[f, t] = sum_k A[f, k] * B[t, k]
// with the 128 features of a tile on the 128 TMEM lanes and the tokens on TMEM columns, then
// runs one of the epilogues below.  For a linear layer y = x W^T the weight is A and the
// activations are B, whatever the token count (decode batch of 64 or a 12k-token training
// micro-batch), so that every epilogue sees "one thread = one output feature".
enum E2hEpilogue : int {
  E2H_EPI_STORE_BF16 = 0,   // out[t*ldo + f] = bf16(acc)
  E2H_EPI_STORE_F32 = 1,    // out[t*ldo + f] = acc                       (fp32)
  E2H_EPI_SWIGLU = 2,       // dual A: out[t*ldo+f] = bf16(silu(bf16(acc1)) * bf16(acc2))
  E2H_EPI_ROPE_KV = 3,      // fused QKV: RoPE on q,k; q -> out, k,v -> static KV cache
  E2H_EPI_RESIDUAL = 4,     // out[t*ldo + f] = bf16(bf16(acc) + aux[t*ldo + f])
  E2H_EPI_ROWMAJOR_F32_ACC = 5,  // out[f*ldo + t] (+)= acc  (fp32, weight gradients)
  E2H_EPI_ROWMAJOR_BF16 = 6,     // out[f*ldo + t] = bf16(acc)
  E2H_EPI_DUAL_STORE = 7,   // dual A: out[t*ldo+f] = bf16(acc1), out2[t*ldo2+f] = bf16(acc2)
};

struct E2hGemmParams {
  int F, T, K;
  int splitk;       // CTAs of one cluster that split K and reduce through distributed smem
  int epi;
  int stages;
  int a_mn_major;   // 0: A is [F, K] row-major (K contiguous); 1: A is [K, F] row-major
  int b_mn_major;   // 0: B is [T, K] row-major;               1: B is [K, T] row-major
  int bn;           // token tile width: 64, 128 or 256
  int dual;         // second feature operand A2 with its own accumulator
  int accumulate;   // ROWMAJOR_F32_ACC: add to what `out` holds
  int pdl;          // launch with programmatic stream serialization
  long long lda, lda2, ldb;   // leading dimensions of the operands, in elements
  const void* a;
  const void* a2;
  const void* b;
  void* out;
  long long ldo;
  void* out2;
  long long ldo2;
  const void* aux;       // residual (bf16, same layout as out)
  const float* scale;    // optional per-feature scale applied to acc (weight-only int8)
  // RoPE + KV-cache epilogue
  const void* freqs;     // bf16 [smax, head_dim/2, 2] (cos, sin)
  const int* pos_base;   // device scalar: cache position of the first token of every sequence
  int sq;                // tokens per sequence in this call (1 for decode)
  int n_head, n_kv, head_dim, smax;
  void* kcache;          // bf16 [max_batch, n_kv, smax, head_dim]
  void* vcache;
  int* status;           // int32 status word (0 = ok)
  int tf;                // features per tile: 128 (default) or 64 (more CTAs for skinny GEMMs)
  int th;                // e2h_gemm_umma, tf = 128, K-major A: weight rows a CTA streams per
                         // k-block (64..128, multiple of 8; 0 = tf). The grid has ceil(F / th)
                         // feature tiles; the MMA still spans 128 lanes
  int stage_epi;         // set by e2h_gemm_umma: the epilogue goes through shared memory and
                         // leaves with 16-byte accesses (gemm_epilogue.cuh)
  int kps;               // 64-wide k blocks per pipeline stage (1..8): amortises the barrier
                         // hand-shake when the per-block tensor work is tiny (decode)
  int n_signal;          // > 0: bump signal[0..n_signal) by one when the whole grid is done;
                         // -1: signal[0] is a multicast address, one multimem.red bumps the
                         // word on every GPU of the mapping
  int* signal[8];        // flag words (local or peer-GPU memory), one per tensor-parallel rank
  unsigned int* ticket;  // grid completion counter (local, zero between launches)
  int a_tiled;           // A (and A2) stored tile-major: [F/tf][ceil(K/64)][tf][64], zero padded
  // weight-only int4 (e2h_gemm_w4) only
  int groupsize;         // k per (scale, zero) pair
  const void* qsz;       // bf16 [K / groupsize][F][2] (scale, zero) of A
  const void* qsz2;      // same for A2 of a dual GEMM
  unsigned long long* phase_clock;  // builds with E2H_PHASE_CLOCK only: 16 time stamps per CTA
};

#ifdef __cplusplus
extern "C" {
#endif
// Returns 0 on success, a cudaError_t / negative code otherwise. Launches on `stream`.
int e2h_gemm_umma(const E2hGemmParams* p, void* stream);
int e2h_gemm_w8(const E2hGemmParams* p, void* stream);
int e2h_gemm_w4(const E2hGemmParams* p, void* stream);
#ifdef __cplusplus
}
#endif
