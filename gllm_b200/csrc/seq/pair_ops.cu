// Kernel of the layer-list decoder's hashed pair embedding.
//
// pair_embed: the fp32 residual stream starts as table[token] + pair_table[row], where row hashes the (previous token,
// token) pair of the same sequence: (prev * mul_prev + token * mul_cur) mod buckets in 64-bit integers, and a token
// at position 0 takes row `buckets` (the table's last row). Inside a portion the previous token is the row before;
// for a portion's first row it is the sequence's carried token, prev_state[slot], which the previous step left
// there. The block of a portion's first row reads the carried token and then stores the portion's last token in its
// place, so no other block of the launch touches that slot (one sequence per slot; graph-padding rows sit at
// position 0 and never read theirs).
//
// Compiled without --use_fast_math like the rest of csrc/seq.
#include <cuda_bf16.h>

#include "common/host_utils.h"
#include "seq/seq_common.cuh"

namespace {
using namespace seqk;

template <typename T>
__global__ void __launch_bounds__(128) pair_embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                                         const T* __restrict__ pair_table, float* __restrict__ out,
                                                         int width, int vocab, long long mul_prev, long long mul_cur,
                                                         int buckets, const int* __restrict__ positions,
                                                         int* __restrict__ prev_state,
                                                         const int* __restrict__ rec_slots,
                                                         const int* __restrict__ qsl, int nseq) {
  __shared__ int row_s;
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  if (threadIdx.x == 0) {
    const int s = find_seq(qsl, nseq, t);
    const int q0 = qsl[s], q1 = qsl[s + 1];
    long long prev = -1;
    if (t > q0) {
      prev = ids[t - 1];
    } else if (prev_state != nullptr) {
      const int slot = rec_slots[s];
      prev = prev_state[slot];
      prev_state[slot] = ids[q1 - 1];
    }
    int row = buckets;
    if (positions[t] != 0) {
      if (prev < 0) prev = 0;
      long long hsh = (prev * mul_prev + (long long)id * mul_cur) % (long long)buckets;
      if (hsh < 0) hsh += buckets;
      row = (int)hsh;
    }
    row_s = row;
  }
  __syncthreads();
  const T* er = table + (size_t)id * width;
  const T* pr = pair_table + (size_t)row_s * width;
  for (int i = threadIdx.x; i < width; i += 128) out[(size_t)t * width + i] = to_f(er[i]) + to_f(pr[i]);
}

}  // namespace

typedef __nv_bfloat16 bf16_t;

GLLM_EXPORT int gllm_pair_embed(const void* ids, const void* table, const void* pair_table, void* out, int ntok,
                                int width, int vocab, long mul_prev, long mul_cur, int buckets, const void* positions,
                                void* prev_state, const void* rec_slots, const void* qsl, int nseq, int is_f32,
                                void* stream) {
  if (ntok <= 0) return 0;
  if (buckets <= 0 || nseq <= 0) return 2;
  cudaStream_t st = (cudaStream_t)stream;
  if (is_f32)
    pair_embed_kernel<float><<<ntok, 128, 0, st>>>((const int*)ids, (const float*)table, (const float*)pair_table,
                                                   (float*)out, width, vocab, mul_prev, mul_cur, buckets,
                                                   (const int*)positions, (int*)prev_state, (const int*)rec_slots,
                                                   (const int*)qsl, nseq);
  else
    pair_embed_kernel<bf16_t><<<ntok, 128, 0, st>>>((const int*)ids, (const bf16_t*)table, (const bf16_t*)pair_table,
                                                    (float*)out, width, vocab, mul_prev, mul_cur, buckets,
                                                    (const int*)positions, (int*)prev_state, (const int*)rec_slots,
                                                    (const int*)qsl, nseq);
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}
