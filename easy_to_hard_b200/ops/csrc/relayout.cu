// Weight re-layout between two parallel layouts over peer memory: the rollout copy of the PPO
// policy (tensor parallel over all GPUs of the box) is refreshed straight from the training
// policy's bf16 shards (tensor parallel x sharded data parallel), each destination rank pulling
// exactly the rows / columns it owns. It replaces the reference's full-state-dict gather of the
// whole policy on every rollout (trainers/ppo_trainer.py:260-311 there), which moves the whole
// model to every rank.
//
// Source layout of one tensor: a row-major [rows_src, pitch] matrix that lives at element
// offset `flat0` of a flat parameter buffer; the flat buffer is cut into `dp` equal shards of
// `shard` elements, shard d being in the symmetric memory of rank base.p[d] at byte offset
// `unit_off`. Destination: a dense row-major [rows, cols] bf16 tensor equal to the block
//   src[row0 + r][col0 + c],  r < rows, c < cols.
// Every thread moves 16 bytes; cols, col0, pitch, flat0 and shard are multiples of 8 elements,
// so a 16-byte piece never straddles two shards.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace e2h {

struct RelayoutSrc {
  const uint8_t* p[8];   // base of data-parallel shard d's symmetric buffer (index = d)
};

__global__ void relayout_pull_kernel(const RelayoutSrc src, long long unit_off, long long shard,
                                     long long flat0, long long pitch, long long row0,
                                     long long col0, long long rows, long long cols,
                                     uint4* __restrict__ dst) {
  const long long vec_per_row = cols >> 3;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row, c = (i - r * vec_per_row) << 3;
    const long long f = flat0 + (row0 + r) * pitch + col0 + c;   // element in the flat buffer
    const long long d = f / shard, off = f - d * shard;
    const uint8_t* p = src.p[d] + unit_off + off * 2;
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    dst[i] = v;
  }
}

}  // namespace e2h

// shard_ptrs: dp device addresses (bases of the symmetric buffers that hold shard 0..dp-1).
// Returns 0, -1 for sizes that are not multiples of 8 elements / misaligned pointers / a block
// that leaves the source, or a cudaError_t.
extern "C" int e2h_relayout_pull(const void* const* shard_ptrs, int dp, long long unit_off,
                                 long long shard, long long flat0, long long pitch,
                                 long long row0, long long col0, long long rows, long long cols,
                                 void* dst, void* stream) {
  using namespace e2h;
  if (dp < 1 || dp > 8 || rows < 1 || cols < 8) return -1;
  if ((cols | col0 | pitch | flat0 | shard) & 7) return -1;
  if ((unit_off & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -1;
  const long long last = flat0 + (row0 + rows - 1) * pitch + col0 + cols;
  if (last > shard * dp || row0 < 0 || col0 < 0 || col0 + cols > pitch) return -1;
  RelayoutSrc s;
  for (int i = 0; i < 8; ++i) {
    s.p[i] = i < dp ? static_cast<const uint8_t*>(shard_ptrs[i]) : nullptr;
    if (i < dp && (reinterpret_cast<uintptr_t>(s.p[i]) & 15)) return -1;
  }
  const long long nvec = rows * (cols >> 3);
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  relayout_pull_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      s, unit_off, shard, flat0, pitch, row0, col0, rows, cols, static_cast<uint4*>(dst));
  return (int)cudaGetLastError();
}
