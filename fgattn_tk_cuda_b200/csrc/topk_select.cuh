// Top-k key selection per query block (the alternative list producer of the reference,
// qk_topkmask_indices in python/spattn/mask_utils.py:389-417): score(query block, key) =
// mean of the block's query rows . key * scale; the select_k keys with the largest score become
// the block's list, in descending score order.
//
// Three kernels:
//   qblock_mean_kernel   : block means of q in fp32, written as a bf16 pair hi + lo (hi = bf16(mean),
//                          lo = bf16(mean - hi)), so that two bf16 tensor-core products reproduce
//                          the fp32 mean to ~2^-17 relative.  HBM-bound read of q.
//   topk_scores_kernel   : scores = (hi + lo) . k^T on tcgen05 (128 query blocks x 128 keys per
//                          CTA, accumulator in TMEM), staged through shared memory and written as
//                          fp32 rows; columns past kv_len hold -inf.
//   topk_select_kernel   : per row an interval-narrowing histogram select (2048 bins per sweep) for
//                          the k-th largest score, ordered tie handling (smallest key index first),
//                          bitonic sort of the selected (score, index) pairs in shared memory.
#pragma once
#include "sm100_ptx.cuh"

namespace fg {

// grid (n_blocks, BH), 256 threads.
template <int D>
__global__ void __launch_bounds__(256)
qblock_mean_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ qm_hi,
                   __nv_bfloat16* __restrict__ qm_lo, int S, int n_blocks, int blocksz, float scale) {
  constexpr int kChunks = D / 8;                 // 16-byte chunks per row
  constexpr int kGroups = 256 / kChunks;         // row groups working in parallel
  __shared__ float part[kGroups][D];
  const int blk = blockIdx.x, bh = blockIdx.y, tid = threadIdx.x;
  const int chunk = tid % kChunks, grp = tid / kChunks;
  const int r0 = blk * blocksz, rows = min(blocksz, S - r0);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const __nv_bfloat16* base = q + (size_t(bh) * S + r0) * D + chunk * 8;
  for (int r = grp; r < rows; r += kGroups) {
    const uint4 v = *reinterpret_cast<const uint4*>(base + size_t(r) * D);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] += __uint_as_float(w[i] << 16);
      acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) part[grp][chunk * 8 + i] = acc[i];
  __syncthreads();
  if (tid < D) {
    float s = 0.f;
#pragma unroll 8
    for (int g = 0; g < kGroups; ++g) s += part[g][tid];
    const float mean = s / float(rows) * scale;
    const __nv_bfloat16 hi = __float2bfloat16_rn(mean);
    const size_t off = (size_t(bh) * n_blocks + blk) * D + tid;
    qm_hi[off] = hi;
    qm_lo[off] = __float2bfloat16_rn(mean - __bfloat162float(hi));
  }
}

struct TopkScoreParams {
  float* scores;       // [BH, n_blocks, s_stride]
  int* err;
  int n_blocks, kv_len, s_stride;
};

template <int D>
struct TopkScoreCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kStageBytes = 128 * 128 * 4;                   // fp32 score tile, reuses the operand tiles
  static constexpr int kOffBar = (3 * kTileBytes > kStageBytes) ? 3 * kTileBytes : kStageBytes;
  static constexpr int kSmemBytes = kOffBar + 64 + 1024;
  static constexpr int kThreads = 160;                                // 4 epilogue warps + 1 load / issue warp
};

// grid (key tiles, query-block tiles, BH).
template <int D>
__global__ void __launch_bounds__(TopkScoreCfg<D>::kThreads)
topk_scores_kernel(const __grid_constant__ CUtensorMap m_hi, const __grid_constant__ CUtensorMap m_lo,
                   const __grid_constant__ CUtensorMap mk, const TopkScoreParams p) {
  using Cfg = TopkScoreCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar_full = sbase + Cfg::kOffBar, bar_done = bar_full + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffBar + 16);
  AbortState* ab = reinterpret_cast<AbortState*>(smem + Cfg::kOffBar + 24);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int key0 = blockIdx.x * 128, qb0 = blockIdx.y * 128, bh = blockIdx.z;

  if (tid == 0) {
    ab->flag = 0;
    mbar_init(bar_full, 1);
    mbar_init(bar_done, 1);
    mbar_fence_init();
  }
  if (warp == 4) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t a_hi = sbase, a_lo = sbase + Cfg::kTileBytes, b_k = sbase + 2 * Cfg::kTileBytes;

  if (warp == 4) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar_full, 3 * Cfg::kTileBytes);
      for (int h = 0; h < Cfg::kHalves; ++h) {
        tma_load_3d(a_hi + h * 16384, &m_hi, bar_full, h * 64, qb0, bh);
        tma_load_3d(a_lo + h * 16384, &m_lo, bar_full, h * 64, qb0, bh);
        tma_load_3d(b_k + h * 16384, &mk, bar_full, h * 64, key0, bh);
      }
    }
    __syncwarp();
    const bool ok = mbar_wait_warp(bar_full, 0, ab, p.err, 3101);
    if (ok) {
      tc_fence_after();
      const uint32_t idesc = umma_idesc_bf16(128, 128, false);
      if (elect_one()) {               // one election for both products and the commit
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          const uint32_t a = part ? a_lo : a_hi;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
            umma_ss(tmem, umma_smem_desc_sw128(a + off, 16, 1024), umma_smem_desc_sw128(b_k + off, 16, 1024), idesc,
                    (part | kk) ? 1u : 0u);
          }
        }
        umma_commit(bar_done);
      }
      __syncwarp();
    }
  } else {
    // epilogue: one query-block row per thread -> shared-memory tile (16-byte chunks XOR-swizzled by
    // row so that the row-per-thread stores and the row-per-warp loads are both conflict free)
    const bool ok = mbar_wait(bar_done, 0, ab, p.err, 3102);
    float* stage = reinterpret_cast<float*>(smem);
    const int row = warp * 32 + lane;
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t r[32];
        tmem_ld32(tmem + (uint32_t(warp * 32) << 16) + cc * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int chunk = cc * 8 + i;
          float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                                 __uint_as_float(r[4 * i + 3]));
          *reinterpret_cast<float4*>(stage + row * 128 + ((chunk ^ (row & 31)) << 2)) = v;
        }
      }
      tc_fence_before();
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");        // the four epilogue warps
    if (ok && !ab->flag) {
      for (int r = warp; r < 128; r += 4) {
        const int qb = qb0 + r;
        if (qb >= p.n_blocks) break;
        float4 v = *reinterpret_cast<const float4*>(stage + r * 128 + ((lane ^ (r & 31)) << 2));
        const int key = key0 + lane * 4;
        if (key >= p.s_stride) continue;
        if (key + 0 >= p.kv_len) v.x = -INFINITY;
        if (key + 1 >= p.kv_len) v.y = -INFINITY;
        if (key + 2 >= p.kv_len) v.z = -INFINITY;
        if (key + 3 >= p.kv_len) v.w = -INFINITY;
        *reinterpret_cast<float4*>(p.scores + (size_t(bh) * p.n_blocks + qb) * p.s_stride + key) = v;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tmem_dealloc(tmem, 128);
  }
}

// Orderable image of a float: a larger float gives a larger unsigned key.
__device__ __forceinline__ uint32_t float_order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kSelThreads = 512;
constexpr int kSelBins = 2048;

// grid (rows), kSelThreads threads, dynamic shared memory = 8 * pow2ceil(k) bytes.  Row r of `scores`
// has n entries (stride s_stride, a multiple of 4, rows 16-byte aligned); writes the indices of its k
// largest entries in descending score order (equal scores: smaller index first) to idx[r][0..k) and k
// to cnt[r].  Requires 1 <= k <= n.  Every sweep reads the row from global memory (L2 after the first;
// keeping the row in shared memory instead allows one CTA per SM only and measured slower).
//
// Selection works on the order-preserving unsigned image of the scores.  A first sweep finds the
// smallest and largest key of the row; each following sweep histograms the keys of the current
// interval into 2048 equal bins (a plain byte-wise radix would put almost every score of a row into
// two or three bins of its leading byte and serialise the shared-memory counters), picks the bin
// that holds the k-th largest and narrows the interval to it, until the bin and everything above it
// fit the sort buffer (usually after one histogram sweep) or the bins are one key wide.
__global__ void __launch_bounds__(kSelThreads)
topk_select_kernel(const float* __restrict__ scores, int s_stride, int n, int k, int k_pow2, int* __restrict__ idx,
                   int* __restrict__ cnt, int list_stride) {
  extern __shared__ unsigned long long sel[];            // (key << 32 | ~index), k_pow2 entries
  __shared__ int hist[kSelBins];
  __shared__ uint32_t s_lo, s_hi;
  __shared__ int s_rem, s_ties, s_count, s_base;
  __shared__ uint32_t red_lo[kSelThreads / 32], red_hi[kSelThreads / 32];
  __shared__ int warp_tot[kSelThreads / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float* row = scores + size_t(blockIdx.x) * s_stride;
  const float4* row4 = reinterpret_cast<const float4*>(row);
  const int n4 = (n + 3) >> 2;

  // One sweep over the row, four 16-byte loads in flight per thread; f(key, index, live) per entry.
  // The trip count is the same for every thread, so f may use full-warp collectives.
  auto sweep = [&](auto&& f) {
    for (int base = 0; base < n4; base += 4 * kSelThreads) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = base + u * kSelThreads + tid;
        v[u] = (j < n4) ? row4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = base + u * kSelThreads + tid;
        const float x[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) f(float_order_key(x[e]), 4 * j + e, j < n4 && 4 * j + e < n);
      }
    }
  };
  // ---- key range of the row
  uint32_t kmin = 0xffffffffu, kmax = 0u;
  sweep([&](uint32_t key, int, bool live) {
    if (live) {
      kmin = min(kmin, key);
      kmax = max(kmax, key);
    }
  });
  kmin = __reduce_min_sync(0xffffffffu, kmin);
  kmax = __reduce_max_sync(0xffffffffu, kmax);
  if (lane == 0) { red_lo[warp] = kmin; red_hi[warp] = kmax; }
  __syncthreads();
  if (tid == 0) {
    uint32_t a = red_lo[0], b = red_hi[0];
    for (int w = 1; w < kSelThreads / 32; ++w) { a = min(a, red_lo[w]); b = max(b, red_hi[w]); }
    s_lo = a;
    s_hi = b;
    s_rem = k;
  }
  __syncthreads();

  // ---- narrow [lo, hi] around the k-th largest key
  while (true) {
    const uint32_t lo = s_lo, hi = s_hi;
    const int rem = s_rem;
    const uint32_t width = hi - lo;                                    // keys in the interval - 1
    const int shift = max(0, (32 - __clz(width | 1u)) - 11);           // (hi - lo) >> shift < 2048
    for (int i = tid; i < kSelBins; i += kSelThreads) hist[i] = 0;
    __syncthreads();
    sweep([&](uint32_t key, int, bool live) {
      if (live && key >= lo && key <= hi) atomicAdd(&hist[(key - lo) >> shift], 1);
    });
    __syncthreads();
    if (warp == 0) {
      // lane L owns the 64 bins [2048 - 64 (L + 1), 2048 - 64 L): lane 0 holds the largest keys
      constexpr int kPer = kSelBins / 32;
      const int b0 = kSelBins - kPer * (lane + 1);
      int mine = 0;
      for (int b = 0; b < kPer; ++b) mine += hist[b0 + b];
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const bool here = incl >= rem && incl - mine < rem;              // exactly one lane
      if (here) {
        int r = rem - (incl - mine), b = kPer - 1;
        for (; b > 0; --b) {
          if (hist[b0 + b] >= r) break;
          r -= hist[b0 + b];
        }
        const uint32_t nlo = lo + (uint32_t(b0 + b) << shift);
        s_lo = nlo;
        s_hi = (shift == 0) ? nlo : min(hi, nlo + ((1u << shift) - 1u));
        s_rem = r;
        s_ties = hist[b0 + b];
      }
    }
    __syncthreads();
    // stop as soon as everything from the chosen bin upwards fits the sort buffer: the sort then
    // orders the bin's entries too and the first k sorted entries are the answer
    if (shift == 0 || (k - s_rem) + s_ties <= k_pow2) break;
  }
  const uint32_t kth = s_lo;                             // lowest key taken; s_rem of the s_ties entries in
                                                         // [kth, s_hi] are needed (s_hi == kth after a full narrowing)
  const int rem = s_rem, n_gt = k - rem;
  __syncthreads();

  if (tid == 0) { s_count = 0; s_base = 0; }
  for (int i = tid; i < k_pow2; i += kSelThreads) sel[i] = 0ull;
  __syncthreads();
  if (n_gt + s_ties <= k_pow2) {
    // ---- common case: everything >= kth fits the sort buffer; the sort puts ties in index order.
    // One shared-counter update per warp and sweep slot.
    sweep([&](uint32_t key, int i, bool live) {
      const bool take = live && key >= kth;
      const uint32_t bal = __ballot_sync(0xffffffffu, take);
      if (bal) {
        int base = 0;
        if (lane == __ffs(bal) - 1) base = atomicAdd(&s_count, __popc(bal));
        base = __shfl_sync(0xffffffffu, base, __ffs(bal) - 1);
        if (take)
          sel[base + __popc(bal & ((1u << lane) - 1u))] =
              (static_cast<unsigned long long>(key) << 32) | uint32_t(~uint32_t(i));
      }
    });
  } else {
    // ---- many ties at the k-th key: entries above it in any order, then the first `rem` ties by index
    for (int i0 = 0; i0 < n; i0 += kSelThreads) {
      const int i = i0 + tid;
      const uint32_t key = (i < n) ? float_order_key(row[i]) : 0u;
      if (i < n && key > kth) {
        const int pos = atomicAdd(&s_count, 1);
        sel[pos] = (static_cast<unsigned long long>(key) << 32) | uint32_t(~uint32_t(i));
      }
      const int tie = (i < n && key == kth) ? 1 : 0;
      const uint32_t bal = __ballot_sync(0xffffffffu, tie);
      if (lane == 0) warp_tot[warp] = __popc(bal);
      __syncthreads();
      int off = s_base;
      for (int w = 0; w < warp; ++w) off += warp_tot[w];
      off += __popc(bal & ((1u << lane) - 1u));
      if (tie && off < rem)
        sel[n_gt + off] = (static_cast<unsigned long long>(key) << 32) | uint32_t(~uint32_t(i));
      __syncthreads();
      if (tid == kSelThreads - 1) s_base = off + tie;
      __syncthreads();
    }
  }
  __syncthreads();

  // ---- bitonic sort, descending: the first k entries are the answer
  for (int size = 2; size <= k_pow2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tid; t < (k_pow2 >> 1); t += kSelThreads) {
        const int lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
        const bool desc = (lo & size) == 0;
        const unsigned long long a = sel[lo], b = sel[hi];
        if ((a < b) == desc) {
          sel[lo] = b;
          sel[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  int* dst = idx + size_t(blockIdx.x) * list_stride;
  for (int i = tid; i < k; i += kSelThreads) dst[i] = int(~uint32_t(sel[i] & 0xffffffffull));
  for (int i = k + tid; i < list_stride; i += kSelThreads) dst[i] = list_stride;
  if (tid == 0) cnt[blockIdx.x] = k;
}

}  // namespace fg
