// One-bit-per-entry masks: pack / unpack and the conversions between packed masks and ascending
// index lists.  All four kernels are plain HBM-bound byte / bit work.
//
// Bit order: entry e of a row lives in byte e / 8, bit e % 8 (least significant bit first), the order
// of python/spattn/mask_utils.py:421-440 of the reference.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "mask_kernels.cuh"   // fill_tail

namespace fg {

// mask (T = uint8_t or int32, kept iff > 0) -> packed bytes.  One thread per output byte: it reads 8
// consecutive entries (8 or 32 contiguous bytes), so a warp reads one contiguous 256 B / 1 KiB span.
template <typename T>
__global__ void __launch_bounds__(256)
pack_mask_kernel(const T* __restrict__ mask, uint8_t* __restrict__ packed, long long n_bytes) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < n_bytes; b += stride) {
    uint32_t bits = 0;
    if (sizeof(T) == 4) {
      const int4 lo = reinterpret_cast<const int4*>(mask)[2 * b], hi = reinterpret_cast<const int4*>(mask)[2 * b + 1];
      bits = (lo.x > 0) | ((lo.y > 0) << 1) | ((lo.z > 0) << 2) | ((lo.w > 0) << 3) | ((hi.x > 0) << 4) |
             ((hi.y > 0) << 5) | ((hi.z > 0) << 6) | ((hi.w > 0) << 7);
    } else {
      const uint2 v = reinterpret_cast<const uint2*>(mask)[b];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        bits |= (((v.x >> (8 * e)) & 0xffu) ? 1u : 0u) << e;
        bits |= (((v.y >> (8 * e)) & 0xffu) ? 1u : 0u) << (4 + e);
      }
    }
    packed[b] = uint8_t(bits);
  }
}

// packed bytes -> mask of 0 / 1 entries (T = uint8_t or int32).  int32: one thread per four entries (half
// a packed byte), so that each store instruction of a warp covers 512 contiguous bytes; uint8: one
// thread per packed byte (one 8-byte store, 256 contiguous bytes per warp).
template <typename T>
__global__ void __launch_bounds__(256)
unpack_mask_kernel(const uint8_t* __restrict__ packed, T* __restrict__ mask, long long n_bytes) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (sizeof(T) == 4) {
    for (long long q = t0; q < 2 * n_bytes; q += stride) {          // q = index of a group of four entries
      const uint32_t v = uint32_t(packed[q >> 1]) >> (4 * int(q & 1));
      reinterpret_cast<int4*>(mask)[q] = make_int4(v & 1, (v >> 1) & 1, (v >> 2) & 1, (v >> 3) & 1);
    }
  } else {
    for (long long b = t0; b < n_bytes; b += stride) {
      const uint32_t v = packed[b];
      uint2 o;
      o.x = (v & 1) | (((v >> 1) & 1) << 8) | (((v >> 2) & 1) << 16) | (((v >> 3) & 1) << 24);
      o.y = ((v >> 4) & 1) | (((v >> 5) & 1) << 8) | (((v >> 6) & 1) << 16) | (((v >> 7) & 1) << 24);
      reinterpret_cast<uint2*>(mask)[b] = o;
    }
  }
}

// Packed mask row -> ascending index list + count.  Row r of `packed` has row_bytes bytes; entry e is
// kept iff its bit is set and e < n_valid.  Unused list slots receive `sentinel`.  grid (rows), 256
// threads; each thread owns four 32-entry words per sweep.
__global__ void __launch_bounds__(256)
packed_to_index_kernel(const uint8_t* __restrict__ packed, int row_bytes, int* __restrict__ idx, int* __restrict__ cnt,
                       int list_stride, int n_valid, int sentinel) {
  constexpr int kChunks = 4;                 // 256-word chunks per sweep (32768 entries), one pair of barriers per sweep
  __shared__ int warp_tot[kChunks][8];
  __shared__ int s_base;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint8_t* src = packed + size_t(blockIdx.x) * row_bytes;
  int* dst = idx + size_t(blockIdx.x) * list_stride;
  const bool words = ((row_bytes & 3) == 0) && ((reinterpret_cast<uintptr_t>(src) & 3) == 0);
  if (tid == 0) s_base = 0;
  __syncthreads();
  const int n_words = (row_bytes + 3) >> 2;
  for (int w0 = 0; w0 < n_words; w0 += 256 * kChunks) {
    uint32_t bits[kChunks];
    int c[kChunks], incl[kChunks];
#pragma unroll
    for (int k = 0; k < kChunks; ++k) {
      const int w = w0 + k * 256 + tid;
      bits[k] = 0;
      if (w < n_words) {
        if (words) {
          bits[k] = reinterpret_cast<const uint32_t*>(src)[w];
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (4 * w + e < row_bytes) bits[k] |= uint32_t(src[4 * w + e]) << (8 * e);
        }
        const int left = n_valid - 32 * w;               // entries of this word below n_valid
        if (left <= 0) bits[k] = 0;
        else if (left < 32) bits[k] &= (1u << left) - 1u;
      }
      c[k] = __popc(bits[k]);
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
      int mine = off, chunk_total = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int t = warp_tot[k][i];
        if (i < warp) mine += t;
        chunk_total += t;
      }
      mine += incl[k] - c[k];
      const int w = w0 + k * 256 + tid;
      uint32_t u = bits[k];
      while (u) {
        const int e = __ffs(u) - 1;
        u &= u - 1;
        if (mine < list_stride) dst[mine] = 32 * w + e;
        ++mine;
      }
      off += chunk_total;
    }
    __syncthreads();
    if (tid == 0) s_base = off;              // every thread holds the same running total
    __syncthreads();
  }
  const int total = s_base;
  if (tid == 0) cnt[blockIdx.x] = total;
  fill_tail(dst, min(total, list_stride), list_stride, sentinel, tid);
}

// Index list row -> packed mask row (bits of the first cnt[r] listed entries that are < n_bits).
// grid (rows), 256 threads, dynamic shared memory = ceil(row_bytes / 4) words.
__global__ void __launch_bounds__(256)
index_to_packed_kernel(const int* __restrict__ idx, const int* __restrict__ cnt, int list_stride,
                       uint8_t* __restrict__ packed, int row_bytes, int n_bits) {
  extern __shared__ uint32_t s_bits[];
  const int tid = threadIdx.x;
  const int n_words = (row_bytes + 3) >> 2;
  for (int w = tid; w < n_words; w += 256) s_bits[w] = 0;
  __syncthreads();
  const int* src = idx + size_t(blockIdx.x) * list_stride;
  const int n = min(cnt[blockIdx.x], list_stride);
  for (int i = tid; i < n; i += 256) {
    const int e = src[i];
    if (e >= 0 && e < n_bits) atomicOr(&s_bits[e >> 5], 1u << (e & 31));
  }
  __syncthreads();
  uint8_t* dst = packed + size_t(blockIdx.x) * row_bytes;
  if (((row_bytes & 3) == 0) && ((reinterpret_cast<uintptr_t>(dst) & 3) == 0)) {
    for (int w = tid; w < n_words; w += 256) reinterpret_cast<uint32_t*>(dst)[w] = s_bits[w];
  } else {
    for (int b = tid; b < row_bytes; b += 256) dst[b] = uint8_t(s_bits[b >> 2] >> (8 * (b & 3)));
  }
}

}  // namespace fg
