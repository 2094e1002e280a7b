// Block-sparse gather attention for sm_100a: softmax(Q K^T) V restricted to the key blocks that
// each 64-row query block lists, K/V tiles fetched by index with TMA, products on tcgen05.
//
// The UMMA tile has 128 rows, so a CTA "slot" works on a PAIR of neighbouring query blocks
// (rows 0-63 / 64-127 of the tile) and walks the sorted UNION of their two lists; an entry kept by
// only one of the two blocks is masked out for the other half (its probabilities are zero).  Two
// listed key blocks (2 x 64 keys) form one 128-key step.  A CTA runs two slots (query rows
// q0 .. q0+255) that feed one tensor pipe alternately; K/V tiles go through one shared ring in the
// exact order the UMMA issuer consumes them.
//
// The softmax is the online (renormalising) one over the kept keys only, what the sp_attn operator
// computes: one thread owns a whole query row of a slot, so the running maximum stays in its
// registers.  (The form with precomputed max_q / denom lives in sparse_ml_persistent.cuh.)
#pragma once
#include "sm100_ptx.cuh"
#include "softmax_steps.cuh"

namespace fg {

struct SparseParams {
  __nv_bfloat16* o;          // [BH, S, D]
  const int* kb_idx;         // [BH, nqb, list_stride] ascending key-block indices
  const int* kb_cnt;         // [BH, nqb]
  int* err;
  int S, S_pad, kv_len, nqb, nkb, list_stride, list_cap;   // list_cap: union entries a slot can hold
  // CTA i works on item order[i] (or i when order is null); item = unit * quads + quad, a quad being four
  // 64-row query blocks.  An order with the long lists first keeps the end of the launch short.
  const int* order;
  int quads;
  // Re-run pass behind the fixed-offset persistent kernel (template parameter REDO): redo[unit * npairs +
  // pair] != 0 marks a pair of query blocks (128 rows) whose rows left the safe exponent range there.  A few
  // CTAs (one per SM at most) walk all n_total items and compute the ones with a marked pair.
  const int* redo;
  int npairs, n_total;
  // Token-derived lists (null = key-block lists of 64-row query blocks): one list per 128-row query block,
  // [BH, npairs, list_stride] ascending key blocks, with the live columns of every listed block in kb_mask.
  const unsigned long long* kb_mask;
  float scale_log2;
};

template <int D>
struct SparseCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kStages = (D == 128) ? 4 : 8;
  static constexpr int kOffQ = 0;
  static constexpr int kOffRing = 2 * kTileBytes;
  static constexpr int kOffBar = kOffRing + kStages * kTileBytes;
  static constexpr int kBarBytes = 512;
  static constexpr int kOffList = kOffBar + kBarBytes;       // [2][list_cap] union entries, then bitmaps
  static __host__ __device__ constexpr int smem_bytes(int list_cap, int nkb) {
    return kOffList + 2 * list_cap * 4 + 4 * ((nkb + 31) / 32) * 4 + 1024;
  }
};

enum : int {
  SB_Q_FULL = 0,
  SB_FULL = 1,      // +stage (<=8)
  SB_EMPTY = 9,     // +stage
  SB_S_FULL = 17,   // +slot
  SB_P_FULL = 19,   // +slot
  SB_O_FULL = 21,   // +slot
  SB_DONE = 23,     // REDO: every product of the item has been executed (barriers are set up anew per item)
  SB_COUNT = 24
};

// entry = key block index | (kept by rows 0-63) << 30 | (kept by rows 64-127) << 31
__device__ __forceinline__ int entry_kb(uint32_t e) { return int(e & 0x3FFFFFFFu); }

template <int D, bool REDO>
__global__ void __launch_bounds__(384, 1)
sparse_block_attn_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                         const __grid_constant__ CUtensorMap mv, const SparseParams p) {
  using Cfg = SparseCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + Cfg::kOffBar;
  auto bar = [&](int i) -> uint32_t { return bars + 8u * uint32_t(i); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffBar + 8 * SB_COUNT);
  AbortState* ab = reinterpret_cast<AbortState*>(smem + Cfg::kOffBar + 8 * SB_COUNT + 8);
  volatile int* n_union = reinterpret_cast<volatile int*>(smem + Cfg::kOffBar + 8 * SB_COUNT + 16);   // [2]
  uint32_t* lists = reinterpret_cast<uint32_t*>(smem + Cfg::kOffList);                                 // [2][cap]
  uint32_t* bitmaps = lists + 2 * p.list_cap;                                                          // [2][2][words]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int words = (p.nkb + 31) / 32;
  // REDO: does item `it` (a quad = two pairs of query blocks) hold a marked pair?
  auto marked = [&](int it) -> bool {
    const int u = it / p.quads, pr = (it - u * p.quads) * 2;
    const int* f = p.redo + size_t(u) * p.npairs + pr;
    return f[0] != 0 || (pr + 1 < p.npairs && f[1] != 0);
  };
  if constexpr (REDO) {
    // the common case is that nothing at all is marked: leave before any set-up (CTA-uniform)
    bool any = false;
    for (int it = blockIdx.x; it < p.n_total && !any; it += gridDim.x) any = marked(it);
    if (!any) return;
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  bool first_item = true;
  for (int iter = blockIdx.x;; iter += gridDim.x) {
  int item;
  if constexpr (REDO) {
    if (iter >= p.n_total) break;
    if (!marked(iter)) continue;
    item = iter;
  } else {
    item = p.order ? p.order[blockIdx.x] : int(blockIdx.x);
  }
  const int bh = item / p.quads;
  const int q0 = (item - bh * p.quads) * 256;

  if (tid == 0) {
    if (REDO && !first_item) {
      for (int i = 0; i < SB_COUNT; ++i) mbar_inval(bar(i));
    }
    ab->flag = 0;
    mbar_init(bar(SB_Q_FULL), 1);
    for (int s = 0; s < 8; ++s) {
      mbar_init(bar(SB_FULL + s), 1);
      mbar_init(bar(SB_EMPTY + s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar(SB_S_FULL + t), 1);
      mbar_init(bar(SB_P_FULL + t), 128);
      mbar_init(bar(SB_O_FULL + t), 1);
    }
    mbar_init(bar(SB_DONE), 1);
    mbar_fence_init();
  }
  // ---- union of the two query blocks' lists, one warp per slot (warps 0 and 4)
  if ((warp & 3) == 0 && warp < 8) {
    const int t = warp >> 2;
    uint32_t* bm0 = bitmaps + (t * 2 + 0) * words;
    uint32_t* bm1 = bitmaps + (t * 2 + 1) * words;
    for (int w = lane; w < 2 * words; w += 32) bm0[w] = 0u;      // bm0 and bm1 are adjacent
    __syncwarp();
    const int list_rows = p.kb_mask ? p.npairs : p.nqb;
    for (int half = 0; half < 2; ++half) {
      const int qb = p.kb_mask ? (q0 >> 7) + t : (q0 >> 6) + t * 2 + half;   // token lists: one list for both halves
      if (qb < list_rows) {
        const int* src = p.kb_idx + (size_t(bh) * list_rows + qb) * p.list_stride;
        const int n = min(p.kb_cnt[size_t(bh) * list_rows + qb], p.list_stride);
        uint32_t* bm = half ? bm1 : bm0;
        for (int i = lane; i < n; i += 32) {
          const int kb = src[i];
          if (kb >= 0 && kb < p.nkb) atomicOr(&bm[kb >> 5], 1u << (kb & 31));
        }
      }
    }
    __syncwarp();
    uint32_t* out = lists + t * p.list_cap;
    int base = 0;
    for (int w0 = 0; w0 < words; w0 += 32) {
      const int w = w0 + lane;
      const uint32_t a = (w < words) ? bm0[w] : 0u, b = (w < words) ? bm1[w] : 0u;
      uint32_t u = a | b;
      const int cnt = __popc(u);
      int incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      int off = base + incl - cnt;
      while (u) {
        const int bit = __ffs(u) - 1;
        u &= u - 1;
        if (off < p.list_cap)
          out[off] = uint32_t(w * 32 + bit) | (((a >> bit) & 1u) << 30) | (((b >> bit) & 1u) << 31);
        ++off;
      }
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (base > p.list_cap) base = p.list_cap;          // cannot happen when list_cap >= nkb + 1
    if (lane == 0) {
      if (base & 1) {                                  // odd: repeat the last block, kept by nobody
        out[base] = out[base - 1] & 0x3FFFFFFFu;
        ++base;
      }
      n_union[t] = base;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n0 = n_union[0] >> 1, n1 = n_union[1] >> 1;           // 128-key steps per slot
  const int n_max = max(n0, n1);

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (first_item) reg_dealloc<72>();
    if (lane == 0) {
      tma_prefetch_desc(&mq);
      tma_prefetch_desc(&mk);
      tma_prefetch_desc(&mv);
      mbar_arrive_expect_tx(bar(SB_Q_FULL), 2 * Cfg::kTileBytes);
      for (int t = 0; t < 2; ++t)
        for (int h = 0; h < Cfg::kHalves; ++h)
          tma_load_3d(sbase + Cfg::kOffQ + t * Cfg::kTileBytes + h * 16384, &mq, bar(SB_Q_FULL), h * 64, q0 + t * 128,
                      bh);
      int idx = 0;
      bool ok = true;
      auto load_tile = [&](const CUtensorMap* m, int t, int j) {
        const int st = idx % Cfg::kStages, f = idx / Cfg::kStages;
        if (f > 0) ok = mbar_wait(bar(SB_EMPTY + st), (f - 1) & 1, ab, p.err, 401);
        if (!ok) return;
        const uint32_t dst = sbase + Cfg::kOffRing + st * Cfg::kTileBytes;
        const int kb0 = entry_kb(lists[t * p.list_cap + 2 * j]), kb1 = entry_kb(lists[t * p.list_cap + 2 * j + 1]);
        mbar_arrive_expect_tx(bar(SB_FULL + st), Cfg::kTileBytes);
        for (int h = 0; h < Cfg::kHalves; ++h) {
          tma_load_3d(dst + h * 16384, m, bar(SB_FULL + st), h * 64, kb0 * 64, bh);
          tma_load_3d(dst + h * 16384 + 8192, m, bar(SB_FULL + st), h * 64, kb1 * 64, bh);
        }
        ++idx;
      };
      if (n0 > 0) load_tile(&mk, 0, 0);
      if (n1 > 0 && ok) load_tile(&mk, 1, 0);
      for (int j = 0; j < n_max && ok; ++j) {
        for (int t = 0; t < 2 && ok; ++t) {
          const int nt = t ? n1 : n0;
          if (j < nt) {
            load_tile(&mv, t, j);
            if (ok && j + 1 < nt) load_tile(&mk, t, j + 1);
          }
        }
      }
      if (!ok) {
        mbar_wait_brief(bar(SB_Q_FULL), 0);
        for (int i = max(0, idx - Cfg::kStages); i < idx; ++i)
          mbar_wait_brief(bar(SB_FULL + i % Cfg::kStages), (i / Cfg::kStages) & 1);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ UMMA issuer
    if (first_item) reg_dealloc<72>();
    {   // whole warp, uniform control flow; single instructions go through an elected lane
      const uint32_t idesc_qk = umma_idesc_bf16(128, 128, false);
      const uint32_t idesc_pv = umma_idesc_bf16(128, D, true);
      int idx = 0;
      bool ok = mbar_wait_warp(bar(SB_Q_FULL), 0, ab, p.err, 501);
      auto qk = [&](int t) {
        const int st = idx % Cfg::kStages;
        ok = mbar_wait_warp(bar(SB_FULL + st), (idx / Cfg::kStages) & 1, ab, p.err, 502);
        if (!ok) return;
        tc_fence_after();
        const uint32_t qa = sbase + Cfg::kOffQ + t * Cfg::kTileBytes, ka = sbase + Cfg::kOffRing + st * Cfg::kTileBytes;
        if (elect_one()) {             // one election for the product and its commits
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
            umma_ss(tmem + t * 128, umma_smem_desc_sw128(qa + off, 16, 1024), umma_smem_desc_sw128(ka + off, 16, 1024),
                    idesc_qk, ks > 0);
          }
          umma_commit(bar(SB_S_FULL + t));
          umma_commit(bar(SB_EMPTY + st));
        }
        __syncwarp();
        ++idx;
      };
      auto pv = [&](int t, int j) {
        const int st = idx % Cfg::kStages;
        ok = mbar_wait_warp(bar(SB_FULL + st), (idx / Cfg::kStages) & 1, ab, p.err, 503);
        if (ok) ok = mbar_wait_warp(bar(SB_P_FULL + t), j & 1, ab, p.err, 504);
        if (!ok) return;
        tc_fence_after();
        const uint32_t va = sbase + Cfg::kOffRing + st * Cfg::kTileBytes;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ts(tmem + 256 + t * 128, tmem + t * 128 + ks * 8, umma_smem_desc_sw128(va + ks * 2048, 16384, 1024),
                    idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
          umma_commit(bar(SB_EMPTY + st));
        }
        __syncwarp();
        ++idx;
      };
      if (ok && n0 > 0) qk(0);
      if (ok && n1 > 0) qk(1);
      for (int j = 0; j < n_max && ok; ++j) {
        for (int t = 0; t < 2 && ok; ++t) {
          const int nt = t ? n1 : n0;
          if (j < nt) {
            pv(t, j);
            if (!ok) break;
            if (j + 1 < nt) qk(t);
            else umma_commit_elect(bar(SB_O_FULL + t));
          }
        }
      }
      if constexpr (REDO) {
        // the barriers are torn down after this item: every commit issued above must have landed first
        if (ok) {
          umma_commit_elect(bar(SB_DONE));
          ok = mbar_wait_warp(bar(SB_DONE), 0, ab, p.err, 505);
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax warpgroups
    if (first_item) reg_alloc<216>();
    const int t = warp >> 2, wq = warp & 3, half = wq >> 1;
    const int row = q0 + t * 128 + wq * 32 + lane;
    const uint32_t lane_base = tmem + (uint32_t(wq * 32) << 16);
    const uint32_t s_addr = lane_base + t * 128, o_addr = lane_base + 256 + t * 128;
    const float c = p.scale_log2;
    const int nt = t ? n1 : n0;
    const uint32_t* list = lists + t * p.list_cap;
    OnlineState st;
    online_init(st);
    bool ok = true;
    // token-derived lists: entry i of the slot's list has column mask i (the list is the block's own)
    const unsigned long long* masks =
        p.kb_mask ? p.kb_mask + (size_t(bh) * p.npairs + (q0 >> 7) + t) * p.list_stride : nullptr;
    for (int j = 0; j < nt; ++j) {
      const uint32_t e0 = list[2 * j], e1 = list[2 * j + 1];
      const int valid0 = ((e0 >> (30 + half)) & 1u) ? min(64, p.kv_len - entry_kb(e0) * 64) : 0;
      const int valid1 = ((e1 >> (30 + half)) & 1u) ? min(64, p.kv_len - entry_kb(e1) * 64) : 0;
      uint32_t colmask[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      if (masks != nullptr) {
        const unsigned long long m0 = valid0 > 0 ? __ldg(masks + 2 * j) : 0ull;
        const unsigned long long m1 = valid1 > 0 ? __ldg(masks + 2 * j + 1) : 0ull;
        colmask[0] = uint32_t(m0); colmask[1] = uint32_t(m0 >> 32);
        colmask[2] = uint32_t(m1); colmask[3] = uint32_t(m1 >> 32);
      }
      ok = mbar_wait(bar(SB_S_FULL + t), j & 1, ab, p.err, 601);
      if (!ok) break;
      tc_fence_after();
      float mx0, mx1;
      softmax_online_step<D, true>(s_addr, s_addr, o_addr, valid0, valid1, c, j == 0, st, mx0, mx1,
                                   masks != nullptr ? colmask : nullptr);
      tc_fence_before();
      mbar_arrive(bar(SB_P_FULL + t));
    }
    __nv_bfloat16* orow = p.o + (size_t(bh) * p.S + row) * D;
    if (nt == 0) {
      if (row < p.S) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) reinterpret_cast<uint4*>(orow)[i] = make_uint4(0, 0, 0, 0);
      }
    } else if (ok) {
      ok = mbar_wait(bar(SB_O_FULL + t), 0, ab, p.err, 602);
      if (ok) {
        tc_fence_after();
        const float inv = st.l > 0.f ? 1.0f / st.l : 0.f;
        store_o_row<D>(o_addr, orow, inv, row < p.S);
      }
    }
  }
  else {
    if (first_item) reg_dealloc<72>();
  }
  if constexpr (!REDO) break;
  first_item = false;
  const bool aborted = ab->flag != 0;
  tc_fence_before();
  __syncthreads();                     // the item is complete: its barriers and lists may be reused
  if (aborted) break;                  // a wait ran out: no further items
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(*tmem_slot, 512);
  }
}

}  // namespace fg
