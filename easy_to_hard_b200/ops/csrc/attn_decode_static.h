// Decode attention (one query token per sequence against the static KV cache) as an entry point
// that allocates nothing. It has no counterpart in the reference, whose decode step goes through
// PyTorch's SDPA; it exists for callers that must not touch an allocator around the call.
//
// Same computation and argument meaning as e2h_attn_decode (attn_decode.cu), without the
// `partial` and `tickets` arguments: the partial results of a (sequence, head) whose keys are
// shared by several CTAs (running max, sum and weighted value sum of every part) and the ticket
// words that tell the last of those CTAs to merge them are kept in fixed arrays in device
// memory, one set per device, that are part of the library image.
//
//   q        [B, n_head * head_dim] bf16
//   kcache   [max_batch, n_kv, smax, head_dim] bf16 (vcache alike)
//   out      [B, n_head * head_dim] bf16
//   pos      device int32: position of the query token (the live range ends at pos, inclusive)
//   left_pad device int32 [B] or null: first live position per sequence
//   n_split  how many CTAs may share one (sequence, kv head), 1..8 (larger values count as 8);
//            1 gives every pair a CTA of its own and uses no scratch at all
//
// Limit: B * n_head * n_split * (head_dim + 2) <= 64 * 32 * 8 * 130 = 2,129,920 floats
// (8.125 MiB), and B * n_kv <= 16384. A larger request is refused with return code -4 and a
// message on stderr; nothing is launched.
//
// Set-up: the first call on each device looks the array's address up with cudaGetSymbolAddress
// and keeps it; make that first call outside any stream capture. Later calls only launch.
//
// Sharing: all calls on a device use the same arrays. No part of the partial results has to
// start at zero: each call writes every slot that its merge step reads. The ticket words are
// zero in the library image and every launch that completes leaves them zero. Two calls whose execution can overlap (on
// different streams, or from different threads without ordering between the streams) race on
// the array; order them on one stream or with events.
//
// Return: 0 on success, a cudaError_t value from the launch or the set-up, -1 for inconsistent
// head counts or sizes, -3 for an unsupported (head_dim, n_head / n_kv) pair, -4 beyond the
// limit, -5 for a device ordinal >= 64.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

int e2h_attn_decode_static(const void* q, const void* kcache, const void* vcache, void* out,
                           const int* pos, const int* left_pad, int B, int n_head, int n_kv,
                           int head_dim, int smax, float scale, int n_split, void* stream);

#ifdef __cplusplus
}
#endif
