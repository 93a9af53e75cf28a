// Block-mask tables for callers that still want flex-attention's BlockMask
// (sm_100a).  One CTA classifies each 128-token KV block of the visibility
// vector as empty / partial / full and writes the ordered index tables that
// the reference builds with any/all + stable argsort
// (make_block_mask, src/model/kv_cache.py:18-45).  Integer work, bit-exact.
#include "common.cuh"

namespace we {

constexpr int kBmThreads = 256;
constexpr int kBmBlock = 128;        // torch flex-attention _DEFAULT_SPARSE_BLOCK_SIZE
constexpr int kBmMaxBlocks = 4096;   // capacity limit: 524288 tokens

// Places block indices with flag==want first (ascending), then the rest
// (ascending): the order a stable descending argsort of the bool row gives.
__device__ void ordered_indices(const uint8_t* flags, int want, int nblk, int* s_before, int32_t* num_out,
                                int32_t* idx_out, int q_blocks) {
  // warp 0: exclusive prefix count of matching entries, 32 blocks per step
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    int n_true = 0;
    for (int base = 0; base < nblk; base += 32) {
      const int j = base + lane;
      const bool f = j < nblk && flags[j] == want;
      const unsigned m = __ballot_sync(0xffffffffu, f);
      if (j < nblk) s_before[j] = n_true + __popc(m & ((1u << lane) - 1u));
      n_true += __popc(m);
    }
    if (lane == 0) s_before[kBmMaxBlocks] = n_true;
  }
  __syncthreads();
  const int n_true = s_before[kBmMaxBlocks];
  for (int j = threadIdx.x; j < nblk; j += blockDim.x) {
    const int before = s_before[j];
    const int pos = (flags[j] == want) ? before : n_true + (j - before);
    for (int qb = 0; qb < q_blocks; ++qb) idx_out[static_cast<int64_t>(qb) * nblk + pos] = j;
  }
  for (int qb = threadIdx.x; qb < q_blocks; qb += blockDim.x) num_out[qb] = n_true;
  __syncthreads();
}

__global__ void __launch_bounds__(kBmThreads) block_mask_kernel(const uint8_t* __restrict__ mask, int64_t C,
                                                                int q_blocks, int nblk, int32_t* kv_num,
                                                                int32_t* kv_idx, int32_t* full_num,
                                                                int32_t* full_idx) {
  __shared__ uint8_t s_flag[kBmMaxBlocks];          // 0 empty, 1 partial, 2 full
  __shared__ int s_pos[kBmMaxBlocks + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int j = warp; j < nblk; j += nwarps) {
    int cnt = 0;
    for (int c = lane; c < kBmBlock; c += 32) {
      const int64_t tok = static_cast<int64_t>(j) * kBmBlock + c;
      cnt += (tok < C && mask[tok] != 0) ? 1 : 0;     // padding counts as unwritten (:23)
    }
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0) s_flag[j] = cnt == 0 ? 0 : (cnt == kBmBlock ? 2 : 1);
  }
  __syncthreads();
  ordered_indices(s_flag, 1, nblk, s_pos, kv_num, kv_idx, q_blocks);      // partial blocks (:42)
  ordered_indices(s_flag, 2, nblk, s_pos, full_num, full_idx, q_blocks);  // full blocks    (:45)
}

}  // namespace we

extern "C" int we_b200_block_mask(const uint8_t* mask_written, int64_t C, int32_t T, int32_t* kv_num_blocks,
                                  int32_t* kv_indices, int32_t* full_kv_num_blocks, int32_t* full_kv_indices,
                                  void* stream) {
  if (!mask_written || !kv_num_blocks || !kv_indices || !full_kv_num_blocks || !full_kv_indices)
    return WE_B200_E_NULL;
  if (C < 1 || T < 1) return WE_B200_E_SHAPE;
  const int64_t nblk = (C + we::kBmBlock - 1) / we::kBmBlock;
  if (nblk > we::kBmMaxBlocks) return WE_B200_E_LIMIT;
  const int q_blocks = (T + we::kBmBlock - 1) / we::kBmBlock;
  we::block_mask_kernel<<<1, we::kBmThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      mask_written, C, q_blocks, static_cast<int>(nblk), kv_num_blocks, kv_indices, full_kv_num_blocks,
      full_kv_indices);
  we::g_launches.fetch_add(1, std::memory_order_relaxed);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? WE_B200_OK : static_cast<int>(e);
}
