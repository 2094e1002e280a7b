// Max / denominator pass over long key sequences, sm_100a: for every query row the raw maximum m of
// Q K^T and l = sum_j 2^((s_j - m) c), optionally with the raw maximum of every 64-key block per row
// (the input of the threshold epilogue that builds key-block lists).  Same results, item layout and
// parameters as mode kML of the dense family (dense_attn.cuh); the difference is the softmax side.
//
// Without P V nothing ties the columns of a row together until the very end: a partial (m, l) over any
// subset of the keys merges with another one in a single step.  So a row is shared by TWO threads, one
// per 64-key block of every 128-key score tile, each with a running (m, l) of its own, and the two halves
// meet once per item through shared memory.  Four softmax warpgroups (two per query tile) put four warps
// on every SM sub-partition instead of two, each with half as much dependent work per step.  Measured against
// mode kML of the dense family on the same GPU: 4-11 % faster from 1536 to 32760 keys at D = 64 and 128
// (32 heads of 16384 clustered keys, D = 128: 1.94 -> 1.86 ms; 96 heads of 12345 keys, D = 64: 3.39 -> 3.10
// ms).  What is left per 128-key step of both query tiles, about 1430 clocks against 1024 of tensor work, is
// the balance of the MUFU (1536 clocks of exponentials per step without the FMA-pipe share) and the issue
// slots that the polynomial form takes instead (ten per pair of columns against two).
//
// Work item = pair of 128-row query tiles sharing every K tile, one thread block per item (the last
// partial wave's items may be cut into their two tiles, DenseParams::half_from).  Warp roles:
//   warps 0-3 / 4-7    softmax of query tile 0, keys 0-63 / 64-127 of every tile    warp 16      TMA producer
//   warps 8-11 / 12-15 softmax of query tile 1                                      warps 17, 18 UMMA issuers
// Tensor memory: the scores of each query tile are double-buffered (4 x 128 columns).
//
// TOKENMASK = true is the other pass of the dense family without V on the same skeleton: with (m, l) given, the
// 128-row x 1-token threshold mask over all key tiles (mode kTokenMask of dense_attn.cuh, same parameters and
// results).  A thread has no state there at all, so the column split is free: 32 heads of 16384 keys at D = 128
// 1.69 -> 1.41 ms, 96 heads of 12345 keys at D = 64 2.02 -> 1.48 ms.  The form that visits only the key tiles named
// by key-block lists stays in the dense family: its items are a few tiles long, and there the wider thread block
// and the second issuer cost what the split gains (0.49 against 0.48-0.55 ms, 0.59 against 0.62 ms).
#pragma once
#include "dense_attn.cuh"
#include "sm100_ptx.cuh"
#include "softmax_steps.cuh"

namespace fg {

template <int D>
struct MaxqCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kKStages = 4;
  // exponentials on the FMA pipe, of every eight pairs of columns (2 and 3 are level, 4 costs 5 %, 5 costs 9 %)
  static constexpr int kPoly = 2;
  static constexpr int kSmWarps = 16;
  static constexpr int kWarpProd = 16, kWarpIss = 17;       // issuers: kWarpIss + query tile
  static constexpr int kThreads = 32 * 20;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = 2 * kTileBytes;
  static constexpr int kOffBar = kOffK + kKStages * kTileBytes;
  static constexpr int kOffMerge = kOffBar + 512;           // [2 tiles][m, m_used, l][128 rows] fp32
  static constexpr int kSmemBytes = kOffMerge + 2 * 3 * 128 * 4 + 1024 /*alignment slack*/;
};

enum : int {
  MQ_Q_FULL = 0,
  MQ_K_FULL = 1,     // +stage (4)
  MQ_K_EMPTY = 5,    // +stage
  MQ_S_FULL = 9,     // +tile*2+buf
  MQ_S_EMPTY = 13,   // +tile*2+buf
  MQ_MERGE = 17,     // +tile: the second half's (m, l) of every row is in shared memory
  MQ_COUNT = 19
};

// One 64-column share of a score tile: the thread's running (m, l) takes in its row's 64 scores at s_addr,
// of which the first `valid` are live (warp-uniform).  mx returns their raw maximum.  POLY as in
// softmax_online_step: of every eight pairs of columns, how many take the FMA-pipe exponential.
template <int POLY>
__device__ __forceinline__ void maxq_step64(uint32_t s_addr, int valid, float c, OnlineState& st, float& mx) {
  if (valid <= 0) {
    mx = -INFINITY;
    return;
  }
  uint32_t r[64];
  tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
  tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
  tmem_ld_wait();
  if (valid < 64) {
#pragma unroll
    for (int i = 0; i < 64; ++i)
      if (i >= valid) r[i] = __float_as_uint(-INFINITY);
  }
  // maxima of the two 32-column quarters, two chains each
  float ch[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) ch[w] = __uint_as_float(r[w * 16]);
#pragma unroll
  for (int i = 1; i < 16; ++i) {
#pragma unroll
    for (int w = 0; w < 4; ++w) ch[w] = fmaxf(ch[w], __uint_as_float(r[w * 16 + i]));
  }
  const float qmax[2] = {fmaxf(ch[0], ch[1]), fmaxf(ch[2], ch[3])};
  mx = fmaxf(qmax[0], qmax[1]);
  st.m_true = fmaxf(st.m_true, mx);
  const float ms = mx * c;
  if (ms > st.m_used + 8.0f) {           // the offset in use may lag the true maximum by up to 8 (log2 domain)
    st.l *= ex2(st.m_used - ms);
    st.m_used = ms;
  }
  uint64_t sum2 = f2_pack(0.f, 0.f);        // packed row sums: one add per pair of columns
  const float neg_m = -st.m_used;
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    // a quarter that lies below 2^kSkipLog2 of the offset in every row of the warp adds nothing in fp32
    if (__all_sync(0xffffffffu, fmaf(qmax[w], c, neg_m) < kSkipLog2)) continue;
#pragma unroll
    for (int i = w * 32; i < w * 32 + 32; i += 2) {
      float p0, p1;
      const uint64_t x2 =
          f2_fma(f2_pack(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), f2_pack(c, c), f2_pack(neg_m, neg_m));
      if ((((i >> 1) & 7) * POLY) % 8 < POLY) {
        ex2_poly2(x2, p0, p1);
      } else {
        float x0, x1;
        f2_unpack(x2, x0, x1);
        p0 = ex2(x0);
        p1 = ex2(x1);
      }
      sum2 = f2_add(sum2, f2_pack(p0, p1));
    }
  }
  float sum0, sum1;
  f2_unpack(sum2, sum0, sum1);
  st.l += sum0 + sum1;
}

template <int D, bool BLOCKMAX, bool TOKENMASK = false>
__global__ void __launch_bounds__(MaxqCfg<D>::kThreads, 1)
maxq_pass_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk, const DenseParams p) {
  using Cfg = MaxqCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + Cfg::kOffBar;
  auto bar = [&](int i) -> uint32_t { return bars + 8u * uint32_t(i); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffBar + 256);
  AbortState* ab = reinterpret_cast<AbortState*>(smem + Cfg::kOffBar + 264);
  float* merge = reinterpret_cast<float*>(smem + Cfg::kOffMerge);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int item = int(blockIdx.x);
  uint32_t tiles = 3u;                 // bit t: query tile t of the item is computed by this thread block
  if (!TOKENMASK && int(blockIdx.x) >= p.half_from) {
    const int h = int(blockIdx.x) - p.half_from;
    item = p.half_from + (h >> 1);
    tiles = 1u << (h & 1);
  }
  const int bh = item / p.n_pairs, q0 = (item - bh * p.n_pairs) * 256;

  if (tid == 0) {
    ab->flag = 0;
    mbar_init(bar(MQ_Q_FULL), 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(bar(MQ_K_FULL + s), 1);
      mbar_init(bar(MQ_K_EMPTY + s), __popc(tiles));   // one issuer warp per computed query tile
      mbar_init(bar(MQ_S_FULL + s), 1);
      mbar_init(bar(MQ_S_EMPTY + s), 256);             // both threads of every row
    }
    for (int t = 0; t < 2; ++t) mbar_init(bar(MQ_MERGE + t), 128);
    mbar_fence_init();
  }
  if (warp == Cfg::kWarpProd) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n_tiles = p.n_kv_tiles;

  if (warp == Cfg::kWarpProd) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&mq);
      tma_prefetch_desc(&mk);
      mbar_arrive_expect_tx(bar(MQ_Q_FULL), 2 * Cfg::kTileBytes);
      for (int t = 0; t < 2; ++t)
        for (int h = 0; h < Cfg::kHalves; ++h)
          tma_load_3d(sbase + Cfg::kOffQ + t * Cfg::kTileBytes + h * 16384, &mq, bar(MQ_Q_FULL), h * 64, q0 + t * 128,
                      p.bh0 + bh);
      bool ok = true;
      int g = 0;                          // K tiles requested so far
      for (; g < n_tiles; ++g) {
        const int ks = g % Cfg::kKStages, kf = g / Cfg::kKStages;
        if (kf > 0) ok = mbar_wait_relaxed(bar(MQ_K_EMPTY + ks), (kf - 1) & 1, ab, p.err, 601);
        if (!ok) break;
        mbar_arrive_expect_tx(bar(MQ_K_FULL + ks), Cfg::kTileBytes);
        for (int h = 0; h < Cfg::kHalves; ++h)
          tma_load_3d(sbase + Cfg::kOffK + ks * Cfg::kTileBytes + h * 16384, &mk, bar(MQ_K_FULL + ks), h * 64,
                      g * 128, p.bh0 + bh);
      }
      if (!ok) {
        // let the copies that are still in flight land before the thread block goes away
        mbar_wait_brief(bar(MQ_Q_FULL), 0);
        for (int i = max(0, g - Cfg::kKStages); i < g; ++i)
          mbar_wait_brief(bar(MQ_K_FULL + i % Cfg::kKStages), (i / Cfg::kKStages) & 1);
      }
    }
  } else if (warp == Cfg::kWarpIss || warp == Cfg::kWarpIss + 1) {
    // ------------------------------------------------------------------ UMMA issuer of one query tile
    // Whole warp, uniform control flow; a product and its commits go through one elected lane.
    const int t = warp - Cfg::kWarpIss;
    if ((tiles >> t) & 1u) {
      const uint32_t idesc_qk = umma_idesc_bf16(128, 128, false);
      const uint32_t qa = sbase + Cfg::kOffQ + t * Cfg::kTileBytes;
      bool ok = mbar_wait_warp(bar(MQ_Q_FULL), 0, ab, p.err, 611);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int ks = j % Cfg::kKStages, b = j & 1, f = j >> 1;
        ok = mbar_wait_warp(bar(MQ_K_FULL + ks), (j / Cfg::kKStages) & 1, ab, p.err, 612);
        if (ok && f > 0) ok = mbar_wait_warp(bar(MQ_S_EMPTY + t * 2 + b), (f - 1) & 1, ab, p.err, 613);
        if (!ok) break;
        tc_fence_after();
        const uint32_t ka = sbase + Cfg::kOffK + ks * Cfg::kTileBytes;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
            umma_ss(tmem + (t * 2 + b) * 128, umma_smem_desc_sw128(qa + off, 16, 1024),
                    umma_smem_desc_sw128(ka + off, 16, 1024), idesc_qk, kk > 0);
          }
          umma_commit(bar(MQ_S_FULL + t * 2 + b));
          umma_commit(bar(MQ_K_EMPTY + ks));
        }
        __syncwarp();
      }
    }
  } else if (warp < Cfg::kSmWarps) {
    // ------------------------------------------------------------------ softmax warpgroups
    const int wg = warp >> 2, t = wg >> 1, h = wg & 1;     // query tile, 64-key half of every score tile
    const int wq = warp & 3;                               // tensor-memory lane quarter
    const int row_in_tile = wq * 32 + lane;
    const uint32_t lane_base = tmem + (uint32_t(wq * 32) << 16);
    const float c = p.scale_log2;
    const bool active = ((tiles >> t) & 1u) != 0;
    const int row = q0 + t * 128 + row_in_tile;            // query row in the sequence
    const size_t ml_off = size_t(p.bh0 + bh) * p.S_pad + row;
    if constexpr (TOKENMASK) {
      // keep bit of a token: some row of the 128-row block has s c - (m c + log2 l) > log2 tau, i.e. s > thr.
      // Most 32-column quarters hold no such entry in any row of the warp: their row maxima settle that with one
      // instruction per entry, and only the others build bits.
      float thr = INFINITY;                                // rows past the sequence keep nothing
      if (row < p.S) {
        const float t_row = p.max_q[ml_off] * c + log2f(p.denom[ml_off]);      // the same expression as in the dense family
        thr = (p.log2_tau + t_row) / c;
      }
      const bool block_in = q0 + t * 128 < p.S;
      int* mrow0 = p.tokenmask + (size_t(p.bh0 + bh) * ((p.S + 127) >> 7) + ((q0 + t * 128) >> 7)) * p.mask_stride;
      bool ok = true;
      for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        ok = mbar_wait(bar(MQ_S_FULL + t * 2 + b), (j >> 1) & 1, ab, p.err, 623);
        if (!ok) break;
        tc_fence_after();
        const int key0 = j * 128 + h * 64;               // first key of this thread's 64 columns
        const int kv_left = p.kv_len - key0;
        uint32_t r[64];
        const uint32_t s_addr = lane_base + (t * 2 + b) * 128 + h * 64;
        tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(bar(MQ_S_EMPTY + t * 2 + b));          // the scores are in registers: free the buffer
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          float mx = __uint_as_float(r[w * 32]);
#pragma unroll
          for (int i = 1; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[w * 32 + i]));
          if (__any_sync(0xffffffffu, mx > thr)) {
            uint32_t m = 0;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (__uint_as_float(r[w * 32 + i]) > thr) m |= 1u << i;
            const int lim = kv_left - w * 32;              // live columns of this quarter
            m &= (lim >= 32) ? 0xffffffffu : (lim <= 0 ? 0u : ((1u << lim) - 1u));
            const uint32_t bits = __reduce_or_sync(0xffffffffu, m);
            // the caller-zeroed mask is only ever set to 1 (by up to four warps of 32 rows each)
            if (block_in && ((bits >> lane) & 1u)) mrow0[key0 + w * 32 + lane] = 1;
          }
        }
      }
    } else if (active) {
      bool ok = true;
      OnlineState st;
      online_init(st);
      for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        ok = mbar_wait(bar(MQ_S_FULL + t * 2 + b), (j >> 1) & 1, ab, p.err, 621);
        if (!ok) break;
        tc_fence_after();
        const int valid = min(64, p.kv_len - j * 128 - h * 64);
        float mx;
        maxq_step64<Cfg::kPoly>(lane_base + (t * 2 + b) * 128 + h * 64, valid, c, st, mx);
        tc_fence_before();
        mbar_arrive(bar(MQ_S_EMPTY + t * 2 + b));
        if (BLOCKMAX) {
          if (row < p.S_pad && j * 2 + h < p.nkb)
            p.blockmax[(size_t(bh) * p.nkb + size_t(j) * 2 + h) * p.S_pad + row] = mx;
        }
      }
      // the two halves of a row meet: 2^(m_used - m c) brings a half's denominator to the common maximum
      float* mg = merge + t * 384 + row_in_tile;
      if (h == 1) {
        mg[0] = st.m_true;
        mg[128] = st.m_used;
        mg[256] = st.l;
        mbar_arrive(bar(MQ_MERGE + t));
      } else {
        if (ok) ok = mbar_wait(bar(MQ_MERGE + t), 0, ab, p.err, 622);
        if (ok) {
          if (row < p.S) {
            const float m = fmaxf(st.m_true, mg[0]);
            p.max_q[ml_off] = m;
            p.denom[ml_off] = st.l * ex2(st.m_used - m * c) + mg[256] * ex2(mg[128] - m * c);
          } else if (row < p.S_pad) {
            p.max_q[ml_off] = 0.f;
            p.denom[ml_off] = -INFINITY;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == Cfg::kWarpProd) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace fg
