// Key-token lists -> key-block lists with column masks, for the fast path of the token-list operator.
//
// The reference's sparse operator takes, per 128-row query block, a list of key TOKENS
// (include/sparseattn_asyncgatherload_padded.cuh:130-256) and gathers their K/V rows one by one.  Lists
// that come out of the threshold mask nearly fill the 64-key blocks they touch, and for those it is
// cheaper to load the touched blocks whole with TMA and switch the unlisted columns off in the softmax.
// This kernel does the conversion and decides, per query block, which of the two routes pays:
//   * a bitmap of the listed tokens (shared memory), duplicates detected on the way;
//   * the touched 64-key blocks in ascending order, each with its 64-bit column mask, and their number;
//   * route = 1 (block route) when no token is listed twice and the listed tokens fill at least
//     `fill_min` of the touched blocks, else 0 (row-gather route);
//   * a per-row estimate of the row maximum of q.k over the listed keys: the maximum over up to 16 keys
//     sampled evenly from the list, plus a margin -- the exponent hint of the fixed-offset softmax.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace fg {

struct TokenBlocksParams {
  const int* kv_idx;               // [BH, nqb, mask_stride] key tokens
  const int* kv_cnt;               // [BH, nqb]
  const __nv_bfloat16* q;          // [BH, S, D]
  const __nv_bfloat16* k;          // [BH, S_kv, D]
  int* kb_idx;                     // [BH, nqb, kb_stride] touched key blocks, ascending
  unsigned long long* kb_mask;     // [BH, nqb, kb_stride] listed columns of each touched block
  int* kb_cnt;                     // [BH, nqb]
  int* route;                      // [BH, nqb] 1 = block route, 0 = row-gather route
  float* hint;                     // [BH, S_pad] estimate of the raw row maximum
  int S, S_pad, S_kv, nqb, nkb, mask_stride, kb_stride;
  float fill_min;                  // least share of listed columns in the touched blocks for the block route
  float hint_margin;               // added to the sampled maximum (raw score units)
};

constexpr int kHintSamples = 16;

// grid (nqb, BH), 256 threads, dynamic shared memory: token_blocks_smem_bytes(nkb, D)
__host__ __device__ constexpr size_t token_blocks_bitmap_bytes(int nkb) { return (size_t(nkb) * 8 + 15) & ~size_t(15); }
__host__ __device__ constexpr size_t token_blocks_smem_bytes(int nkb, int D) {
  return token_blocks_bitmap_bytes(nkb) + size_t(kHintSamples) * D * 2;       // bitmap, then the sampled key rows
}
template <int D>
__global__ void __launch_bounds__(256) token_lists_to_blocks_kernel(const TokenBlocksParams p) {
  extern __shared__ __align__(16) uint8_t tb_smem[];
  uint32_t* bm = reinterpret_cast<uint32_t*>(tb_smem);                                  // [2 * nkb]
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(tb_smem + token_blocks_bitmap_bytes(p.nkb));   // [16][D], 16-byte aligned
  __shared__ int s_dup, s_bits, s_warp[8], s_base, s_tok[kHintSamples];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qb = blockIdx.x, bh = blockIdx.y;
  const size_t row_id = size_t(bh) * p.nqb + qb;
  const int cnt = max(0, min(p.kv_cnt[row_id], p.mask_stride));
  const int* list = p.kv_idx + row_id * p.mask_stride;

  for (int w = tid; w < 2 * p.nkb; w += 256) bm[w] = 0u;
  if (tid == 0) { s_dup = 0; s_bits = 0; s_base = 0; }
  if (tid < kHintSamples) {
    // sample positions spread evenly over the list
    const int n_s = min(kHintSamples, cnt);
    int tok = -1;
    if (tid < n_s) tok = list[int((long long)tid * cnt / n_s)];
    s_tok[tid] = (tok >= 0 && tok < p.S_kv) ? tok : -1;
  }
  __syncthreads();
  for (int i = tid; i < cnt; i += 256) {
    const int t = list[i];
    if (t >= 0 && t < p.S_kv) {
      const uint32_t bit = 1u << (t & 31);
      if (atomicOr(&bm[t >> 5], bit) & bit) s_dup = 1;
    }
  }
  // sampled key rows -> shared memory (16 bytes per thread and pass)
  constexpr int kChunks = kHintSamples * D / 8;
  for (int c = tid; c < kChunks; c += 256) {
    const int r = c / (D / 8), ch = c % (D / 8);
    const int tok = s_tok[r];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tok >= 0) v = *reinterpret_cast<const uint4*>(p.k + (size_t(bh) * p.S_kv + tok) * D + ch * 8);
    reinterpret_cast<uint4*>(ks)[c] = v;
  }
  __syncthreads();

  // ---- touched blocks in ascending order (block-wide compaction, 256 blocks per sweep)
  int* out_idx = p.kb_idx + row_id * p.kb_stride;
  unsigned long long* out_mask = p.kb_mask + row_id * p.kb_stride;
  int bits = 0;
  for (int kb0 = 0; kb0 < p.nkb; kb0 += 256) {
    const int kb = kb0 + tid;
    unsigned long long m = 0ull;
    if (kb < p.nkb) m = (unsigned long long)bm[2 * kb] | ((unsigned long long)bm[2 * kb + 1] << 32);
    const bool hit = m != 0ull;
    bits += __popcll(m);
    const uint32_t vote = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) s_warp[warp] = __popc(vote);
    __syncthreads();
    int off = s_base;
    for (int w = 0; w < warp; ++w) off += s_warp[w];
    off += __popc(vote & ((1u << lane) - 1u));
    if (hit && off < p.kb_stride) {
      out_idx[off] = kb;
      out_mask[off] = m;
    }
    __syncthreads();
    if (tid == 0) {
      int tot = 0;
      for (int w = 0; w < 8; ++w) tot += s_warp[w];
      s_base += tot;
    }
    __syncthreads();
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) bits += __shfl_xor_sync(0xffffffffu, bits, o);
  if (lane == 0) atomicAdd(&s_bits, bits);
  __syncthreads();
  if (tid == 0) {
    const int nb = min(s_base, p.kb_stride);
    p.kb_cnt[row_id] = nb;
    p.route[row_id] = (s_dup == 0 && nb > 0 && float(s_bits) >= p.fill_min * 64.0f * float(nb)) ? 1 : 0;
  }

  // ---- exponent hint: largest score of each query row against the sampled keys, plus the margin
  if (tid < 128) {
    const int row = qb * 128 + tid;
    if (row < p.S) {
      float acc[kHintSamples];
#pragma unroll
      for (int s = 0; s < kHintSamples; ++s) acc[s] = 0.f;
      const __nv_bfloat16* qrow = p.q + (size_t(bh) * p.S + row) * D;
      for (int c = 0; c < D / 8; ++c) {
        const uint4 qv = *reinterpret_cast<const uint4*>(qrow + c * 8);
        const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&qv);
        float qf[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(q2[e]);
          qf[2 * e] = f.x;
          qf[2 * e + 1] = f.y;
        }
#pragma unroll
        for (int s = 0; s < kHintSamples; ++s) {
          const uint4 kv = reinterpret_cast<const uint4*>(ks + s * D)[c];         // same address for all threads
          const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(k2[e]);
            acc[s] = fmaf(qf[2 * e], f.x, acc[s]);
            acc[s] = fmaf(qf[2 * e + 1], f.y, acc[s]);
          }
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int s = 0; s < kHintSamples; ++s)
        if (s_tok[s] >= 0) mx = fmaxf(mx, acc[s]);
      p.hint[size_t(bh) * p.S_pad + row] = (mx > -INFINITY) ? mx + p.hint_margin : 0.f;
    }
  }
}

}  // namespace fg
