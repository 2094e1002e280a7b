// Integer / HBM-bound kernels of the mask pipeline: threshold epilogue over block maxima,
// stream compaction of masks into ascending index lists, identity lists.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fg {

// ---------------------------------------------------------------------------------------------
// Threshold epilogue + compaction for 64x64 blocks.
// blockmax[bh][kb][row] holds max_j q_row.k_j (raw) over the keys of block kb.  A block (qb, kb)
// is kept iff max over the 64 rows of  blockmax*c - (m*c + log2 l)  >  log2(tau), i.e. iff the
// largest softmax probability inside the block exceeds tau (strict).  Output: ascending key-block
// list per query block, unused slots = nkb, and the count.
// grid (nqb, heads_in_chunk), 256 threads; dynamic shared memory: 64 floats + nkb bytes.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
block_threshold_compact_kernel(const float* __restrict__ blockmax, const float* __restrict__ max_q,
                               const float* __restrict__ denom, int* __restrict__ kb_idx, int* __restrict__ kb_cnt,
                               int S, int S_pad, int nqb, int nkb, int list_stride, int bh0, float scale_log2,
                               float log2_tau) {
  extern __shared__ uint8_t sm[];
  float* t_row = reinterpret_cast<float*>(sm);
  uint8_t* keep = sm + 64 * sizeof(float);
  const int qb = blockIdx.x, bhl = blockIdx.y, bh = bh0 + bhl;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r0 = qb * 64;
  if (tid < 64) {
    const int row = r0 + tid;
    float t = INFINITY;
    if (row < S) t = max_q[size_t(bh) * S_pad + row] * scale_log2 + log2f(denom[size_t(bh) * S_pad + row]);
    t_row[tid] = t;
  }
  __syncthreads();
  const float t0 = t_row[lane], t1 = t_row[lane + 32];
  // four key blocks per trip and warp, so that eight 128-byte loads are in flight per warp (the kernel is bound by
  // the latency of these loads: one block per trip reached 4.8 TB/s)
  for (int kb0 = warp; kb0 < nkb; kb0 += 32) {
    float a[4], b[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int kb = kb0 + 8 * u;
      a[u] = b[u] = -INFINITY;
      if (kb < nkb) {
        const float* src = blockmax + (size_t(bhl) * nkb + kb) * S_pad + r0;
        a[u] = src[lane];
        b[u] = src[lane + 32];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float v = fmaxf(fmaf(a[u], scale_log2, -t0), fmaf(b[u], scale_log2, -t1));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
      const int kb = kb0 + 8 * u;
      if (lane == 0 && kb < nkb) keep[kb] = (v > log2_tau) ? 1 : 0;
    }
  }
  __syncthreads();
  int* out = kb_idx + (size_t(bh) * nqb + qb) * list_stride;
  if (warp == 0) {
    int base = 0;
    for (int kb0 = 0; kb0 < nkb; kb0 += 32) {
      const int kb = kb0 + lane;
      const bool k = (kb < nkb) && keep[kb];
      const uint32_t bal = __ballot_sync(0xffffffffu, k);
      if (k) out[base + __popc(bal & ((1u << lane) - 1u))] = kb;
      base += __popc(bal);
    }
    if (lane == 0) {
      kb_cnt[size_t(bh) * nqb + qb] = base;
      reinterpret_cast<int*>(t_row)[0] = base;
    }
  }
  __syncthreads();
  const int count = reinterpret_cast<int*>(t_row)[0];
  for (int i = count + tid; i < list_stride; i += 256) out[i] = nkb;
}

// dst[from .. n) = value by the 256 threads of a CTA: 16-byte stores where the row allows it.
__device__ __forceinline__ void fill_tail(int* __restrict__ dst, int from, int n, int value, int tid) {
  if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    const int a = min(n, (from + 3) & ~3), b = n & ~3;       // [from,a) scalar, [a,b) vector, [b,n) scalar
    if (tid < a - from) dst[from + tid] = value;
    const int4 v4 = make_int4(value, value, value, value);
    for (int i = a + 4 * tid; i < b; i += 1024) *reinterpret_cast<int4*>(dst + i) = v4;
    if (b >= a && tid < n - b) dst[b + tid] = value;
  } else {
    for (int i = from + tid; i < n; i += 256) dst[i] = value;
  }
}

// ---------------------------------------------------------------------------------------------
// Mask row -> ascending index list + count (deterministic replacement of an atomic-ticket scan).
// mask int32 [rows, stride], entry kept iff mask > 0 and column < n_valid.  Unused list slots are
// written with `stride`.  grid (rows), 256 threads.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
mask_to_index_kernel(const int* __restrict__ mask, int* __restrict__ idx, int* __restrict__ cnt, int stride,
                     int n_valid) {
  constexpr int kChunks = 4;                 // 1024-column chunks per sweep: four 16-byte loads in flight per thread
  __shared__ int warp_tot[kChunks][8];
  __shared__ int s_base;
  const size_t rowoff = size_t(blockIdx.x) * stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* src = mask + rowoff;
  int* dst = idx + rowoff;
  if (tid == 0) s_base = 0;
  __syncthreads();
  const bool vec = ((stride & 3) == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
  for (int c0 = 0; c0 < stride; c0 += 1024 * kChunks) {
    int v[kChunks][4];
#pragma unroll
    for (int k = 0; k < kChunks; ++k) {
      const int col = c0 + k * 1024 + tid * 4;
      if (vec && col + 3 < stride) {
        const int4 x = *reinterpret_cast<const int4*>(src + col);
        v[k][0] = x.x; v[k][1] = x.y; v[k][2] = x.z; v[k][3] = x.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[k][e] = (col + e < stride) ? src[col + e] : 0;
      }
    }
    uint32_t keep[kChunks];                  // 4 keep bits per chunk
    int c[kChunks], incl[kChunks];
#pragma unroll
    for (int k = 0; k < kChunks; ++k) {
      const int col = c0 + k * 1024 + tid * 4;
      keep[k] = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) keep[k] |= (v[k][e] > 0 && col + e < n_valid) ? (1u << e) : 0u;
      c[k] = __popc(keep[k]);
      incl[k] = c[k];
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
      for (int k = 0; k < kChunks; ++k) {
        const int n = __shfl_up_sync(0xffffffffu, incl[k], o);
        if (lane >= o) incl[k] += n;
      }
    }
    if (lane == 31) {
#pragma unroll
      for (int k = 0; k < kChunks; ++k) warp_tot[k][warp] = incl[k];
    }
    __syncthreads();
    int off = s_base;
#pragma unroll
    for (int k = 0; k < kChunks; ++k) {
      int mine = off;                        // start of chunk k
      int chunk_total = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const int t = warp_tot[k][w];
        if (w < warp) mine += t;
        chunk_total += t;
      }
      mine += incl[k] - c[k];
      const int col = c0 + k * 1024 + tid * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if ((keep[k] >> e) & 1u) dst[mine++] = col + e;
      off += chunk_total;
    }
    __syncthreads();
    if (tid == 0) s_base = off;              // every thread holds the same running total
    __syncthreads();
  }
  const int total = s_base;
  if (tid == 0) cnt[blockIdx.x] = total;
  fill_tail(dst, min(total, stride), stride, stride, tid);
}

// Identity lists: idx[row][s] = s for every slot, count = n_keep.
__global__ void identity_index_kernel(int* __restrict__ idx, int* __restrict__ cnt, int stride, int n_keep) {
  int* dst = idx + size_t(blockIdx.x) * stride;
  for (int i = threadIdx.x; i < stride; i += blockDim.x) dst[i] = i;
  if (threadIdx.x == 0) cnt[blockIdx.x] = n_keep;
}

}  // namespace fg
