// Dense attention family for sm_100a (tcgen05 / TMEM / TMA), one kernel template:
//   kFull      : O = softmax(Q K^T * scale) V                       (full_attn)
//   kFullML    : O plus per-row raw max m and denominator l         (fullattn_maxq_denom)
//   kML        : m and l only, no V                                 (maxq_denom)
// each optionally emitting, per query row and per 64-key block, the raw block maximum of Q K^T
// (the input of the threshold epilogue that builds key-block lists), and
//   kTokenMask : with m, l given, the 128-row x 1-token threshold mask (booleanmask_128).
//
// A work item is a pair of 128-row query tiles that share every K/V tile; CTAs are persistent and take
// items blockIdx.x, blockIdx.x + gridDim.x, ... (item = unit * pairs + pair, so that the CTAs running at
// one time share the K/V of a few heads in L2).  All barrier phases run on across items, so the TMA
// producer fetches the next item's Q and first K/V tiles while the last steps of the current one are
// still being computed, and tensor memory is allocated once per CTA.  Warp roles:
//   warps 0-3  softmax of query tile 0 (one row per thread)      warp 8  TMA producer
//   warps 4-7  softmax of query tile 1                            warps 9, 10  UMMA issuers (one per query tile;
//                                                                  with V at D = 64 and in the token-mask
//                                                                  mode warp 9 alone)
// S = Q K^T accumulates in tensor memory; the softmax warps read it with tcgen05.ld, write the
// bf16 probabilities back over the same columns and the PV product takes them from tensor memory.
#pragma once
#include "sm100_ptx.cuh"
#include "softmax_steps.cuh"

namespace fg {

enum DenseMode : int { kFull = 0, kFullML = 1, kML = 2, kTokenMask = 3 };

struct DenseParams {
  // outputs
  __nv_bfloat16* o;     // [BH, S, D]
  float* max_q;         // [BH, S_pad128]   (kTokenMask: input)
  float* denom;         // [BH, S_pad128]   (kTokenMask: input)
  float* blockmax;      // [BH(chunk), nkb, S_pad128] raw per-row maxima of each 64-key block, or null
  int* tokenmask;       // [BH, nqb128, mask_stride]  (kTokenMask)
  int* err;             // device error word
  int S, S_pad, kv_len, n_kv_tiles, nkb, mask_stride;
  int bh0;              // first (batch*head) unit of this launch (blockmax is relative to it)
  int n_pairs, n_items; // query tile pairs per unit; work items of this launch (units * n_pairs)
  // One-item form only: thread blocks [0, half_from) take one item each; the items from half_from on are cut
  // in two and thread block half_from + 2i + t takes query tile t of item half_from + i alone.  The launcher
  // cuts the items of the last, partial wave when both halves of all of them fit on the SMs at once: a
  // half item takes about half the time, so the wave ends early instead of leaving most SMs idle.
  int half_from;
  // kTokenMask, optional: key-block lists of the 64-row query blocks ([BH, nqb64, list_stride], counts
  // [BH, nqb64]); a CTA then visits only the 128-key tiles that some list of its four query blocks names
  const int* kb_idx;
  const int* kb_cnt;
  int list_stride, nqb64;
  const int* order;     // with lists, optional: thread block i works on item order[i] (longest lists first)
  float scale_log2;     // softmax scale * log2(e)
  float log2_tau;       // kTokenMask
};

template <int D>
struct DenseCfg {
  static constexpr int kHalves = D / 64;                 // 128-byte column groups per row
  static constexpr int kTileBytes = 128 * D * 2;         // one 128-row tile of Q, K or V
  static constexpr int kKStages = 2, kVStages = 2;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = 2 * kTileBytes;
  static constexpr int kOffV = kOffK + kKStages * kTileBytes;
  static constexpr int kOffBar = kOffV + kVStages * kTileBytes;
  static constexpr int kOffTiles = kOffBar + 1024;       // kTokenMask with lists: [0] count, then tile ids, then bitmap
  static constexpr int kMaxListedTiles = 1024;           // 131072 keys
  static constexpr int kSmemBytes = kOffTiles + 4 * (1 + kMaxListedTiles) + 4 * (kMaxListedTiles / 32) + 1024 /*alignment slack*/;
};

// barrier slots (8 bytes each) inside the barrier block
enum : int {
  BAR_Q_FULL = 0,
  BAR_K_FULL = 1,    // +stage (<=4)
  BAR_K_EMPTY = 5,   // +stage
  BAR_V_FULL = 9,    // +stage
  BAR_V_EMPTY = 13,  // +stage
  BAR_S_FULL = 17,   // +tile*2+buf
  BAR_S_EMPTY = 21,  // +tile*2+buf
  BAR_P_FULL = 25,   // +tile
  BAR_O_FULL = 27,   // +tile
  BAR_Q_EMPTY = 29,  // the item's last Q K^T product has been executed
  BAR_COUNT = 30
};

template <int D, int MODE, bool BLOCKMAX, bool PERSIST>
__global__ void __launch_bounds__(384, 1)
dense_attn_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                  const __grid_constant__ CUtensorMap mv, const DenseParams p) {
  using Cfg = DenseCfg<D>;
  constexpr bool HAS_V = (MODE == kFull || MODE == kFullML);
  constexpr bool WRITE_ML = (MODE == kFullML || MODE == kML);
  // without V the V ring's shared memory (it follows the K ring) holds K tiles as well
  constexpr int kKSt = HAS_V ? Cfg::kKStages : Cfg::kKStages + Cfg::kVStages;
  static_assert(kKSt <= 4, "barrier slots");
  constexpr bool TWO_ISS = (HAS_V && D == 128) || MODE == kML;   // one UMMA issuer warp per query tile ...
  constexpr int kTwoIssMinTiles = 64;                            // ... from 8192 keys on: with fewer the second
                                                                 // issuer's share of the item's start and end costs more
                                                                 // than it gains (32768 x 1536 keys: +6 %, x 4096: +2 %)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + Cfg::kOffBar;
  auto bar = [&](int i) -> uint32_t { return bars + 8u * uint32_t(i); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffBar + 8 * BAR_COUNT);
  AbortState* ab = reinterpret_cast<AbortState*>(smem + Cfg::kOffBar + 8 * BAR_COUNT + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int first_item = (MODE == kTokenMask && p.order) ? p.order[blockIdx.x] : int(blockIdx.x);
  const int item_step = gridDim.x;
  uint32_t tiles = 3u;                 // bit t: query tile t of the item is computed by this thread block
  if (!PERSIST && MODE != kTokenMask && int(blockIdx.x) >= p.half_from) {
    const int h = int(blockIdx.x) - p.half_from;
    first_item = p.half_from + (h >> 1);
    tiles = 1u << (h & 1);
  }

  if (tid == 0) {
    ab->flag = 0;
    // with two issuer warps (one per query tile) a K / V stage (or Q) is free when both have let go
    const int n_iss = (TWO_ISS && p.n_kv_tiles >= kTwoIssMinTiles) ? __popc(tiles) : 1;
    mbar_init(bar(BAR_Q_FULL), 1);
    mbar_init(bar(BAR_Q_EMPTY), n_iss);
    for (int s = 0; s < 4; ++s) {
      mbar_init(bar(BAR_K_FULL + s), 1);
      mbar_init(bar(BAR_K_EMPTY + s), n_iss);
      mbar_init(bar(BAR_V_FULL + s), 1);
      mbar_init(bar(BAR_V_EMPTY + s), n_iss);
      mbar_init(bar(BAR_S_FULL + s), 1);
      mbar_init(bar(BAR_S_EMPTY + s), 128);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar(BAR_P_FULL + t), 128);
      mbar_init(bar(BAR_O_FULL + t), 1);
    }
    mbar_fence_init();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  // kTokenMask with key-block lists: the 128-key tiles this CTA has to visit, ascending
  int* s_tiles = reinterpret_cast<int*>(smem + Cfg::kOffTiles);        // [0] = count, [1..] = tile ids
  // (such launches have one CTA per item)
  const bool listed = (MODE == kTokenMask) && p.kb_idx != nullptr;
  if (listed) {
    const int bh = first_item / p.n_pairs, q0 = (first_item - bh * p.n_pairs) * 256;
    uint32_t* bm = reinterpret_cast<uint32_t*>(s_tiles + 1 + Cfg::kMaxListedTiles);
    const int words = (p.n_kv_tiles + 31) / 32;
    for (int w = tid; w < words; w += blockDim.x) bm[w] = 0u;
    __syncthreads();
    for (int i = 0; i < 4; ++i) {
      const int qb = (q0 >> 6) + i;
      if (qb >= p.nqb64) break;
      const size_t rowi = size_t(p.bh0 + bh) * p.nqb64 + qb;
      const int n = min(p.kb_cnt[rowi], p.list_stride);
      const int* src = p.kb_idx + rowi * p.list_stride;
      for (int e = tid; e < n; e += blockDim.x) {
        const int tile = src[e] >> 1;
        if (tile >= 0 && tile < p.n_kv_tiles) atomicOr(&bm[tile >> 5], 1u << (tile & 31));
      }
    }
    __syncthreads();
    if (warp == 0) {
      int base = 0;
      for (int w0 = 0; w0 < words; w0 += 32) {
        const int w = w0 + lane;
        uint32_t u = (w < words) ? bm[w] : 0u;
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
          s_tiles[1 + off++] = w * 32 + bit;
        }
        base += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) s_tiles[0] = base;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n_tiles = listed ? s_tiles[0] : p.n_kv_tiles;
  auto tile_of = [&](int j) -> int { return listed ? s_tiles[1 + j] : j; };

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    reg_dealloc<72>();
    if (lane == 0) {
      tma_prefetch_desc(&mq);
      tma_prefetch_desc(&mk);
      if (HAS_V) tma_prefetch_desc(&mv);
      bool ok = true;
      uint32_t g = 0;                       // K (and V) tiles requested so far by this CTA
      int it = 0;                           // items whose Q has been requested
      for (int item = first_item; item < p.n_items && ok; item += item_step) {
        const int bh = item / p.n_pairs, q0 = (item - bh * p.n_pairs) * 256;
        if (it > 0) ok = mbar_wait(bar(BAR_Q_EMPTY), (it - 1) & 1, ab, p.err, 100);
        if (!ok) break;
        ++it;
        mbar_arrive_expect_tx(bar(BAR_Q_FULL), 2 * Cfg::kTileBytes);
        for (int t = 0; t < 2; ++t)
          for (int h = 0; h < Cfg::kHalves; ++h)
            tma_load_3d(sbase + Cfg::kOffQ + t * Cfg::kTileBytes + h * 16384, &mq, bar(BAR_Q_FULL), h * 64,
                        q0 + t * 128, p.bh0 + bh);
        for (int j = 0; j < n_tiles && ok; ++j, ++g) {
          const int ks = g % kKSt, kf = g / kKSt;
          if (kf > 0) ok = mbar_wait(bar(BAR_K_EMPTY + ks), (kf - 1) & 1, ab, p.err, 101);
          if (!ok) break;
          mbar_arrive_expect_tx(bar(BAR_K_FULL + ks), Cfg::kTileBytes);
          for (int h = 0; h < Cfg::kHalves; ++h)
            tma_load_3d(sbase + Cfg::kOffK + ks * Cfg::kTileBytes + h * 16384, &mk, bar(BAR_K_FULL + ks), h * 64,
                        tile_of(j) * 128, p.bh0 + bh);
          if (HAS_V) {
            const int vs = g % Cfg::kVStages, vf = g / Cfg::kVStages;
            if (vf > 0) ok = mbar_wait(bar(BAR_V_EMPTY + vs), (vf - 1) & 1, ab, p.err, 102);
            if (!ok) { ++g; break; }        // the K copy of this tile is in flight
            mbar_arrive_expect_tx(bar(BAR_V_FULL + vs), Cfg::kTileBytes);
            for (int h = 0; h < Cfg::kHalves; ++h)
              tma_load_3d(sbase + Cfg::kOffV + vs * Cfg::kTileBytes + h * 16384, &mv, bar(BAR_V_FULL + vs), h * 64,
                          j * 128, p.bh0 + bh);
          }
        }
        if (!PERSIST) break;
      }
      if (!ok) {
        // let copies that are still in flight land before the CTA goes away: the last request to
        // every stage (a V request exists for tile x iff its K request does, except possibly the last)
        if (it > 0) mbar_wait_brief(bar(BAR_Q_FULL), (it - 1) & 1);
        for (uint32_t s = 0; s < uint32_t(kKSt); ++s) {
          if (g <= s) continue;
          const uint32_t last = ((g - 1 - s) / kKSt) * kKSt + s;   // last tile <= g-1 on stage s
          mbar_wait_brief(bar(BAR_K_FULL + s), (last / kKSt) & 1);
          if (HAS_V) mbar_wait_brief(bar(BAR_V_FULL + s), (last / Cfg::kVStages) & 1);
        }
      }
    }
  } else if (warp == 9 || (TWO_ISS && warp == 10 && p.n_kv_tiles >= kTwoIssMinTiles)) {
    // ------------------------------------------------------------------ UMMA issuers
    // With V at D = 128 one warp per query tile: a tile's steps form a chain (scores, softmax, P V and next
    // scores), and an issuer that serves both tiles in turn reaches a tile's probabilities late whenever it is
    // busy with the other tile's waits and commits (C3 3.38 -> 3.20 ms).  The max / denominator mode gains the
    // same way (a freed score buffer is refilled at once: C3 2.32 -> 2.18 ms, C4 3.43 -> 3.36 ms).  With V at
    // D = 64 the softmax, not the chain, bounds a step, two issuers are 1 % slower there and one warp serves
    // both tiles, as in the token-mask mode and for key sequences under 8192.  (The gain depends on the data: on
    // i.i.d. normal inputs, where no quarter of a score tile is ever skipped and the softmax step is longer, two
    // issuers are level with one at 8192 keys and 1 % behind at 16384.)
    reg_dealloc<72>();
    const bool two_iss = TWO_ISS && p.n_kv_tiles >= kTwoIssMinTiles;
    const int t_lo = two_iss ? warp - 9 : 0, t_hi = two_iss ? t_lo + 1 : 2;
    if (!two_iss || ((tiles >> t_lo) & 1u)) {   // whole warp, uniform control flow; single instructions go through an elected lane
      const uint32_t idesc_qk = umma_idesc_bf16(128, 128, false);
      const uint32_t idesc_pv = umma_idesc_bf16(128, D, true);
      auto issue_qk = [&](int t, int kstage, uint32_t d_col) {
        const uint32_t qa = sbase + Cfg::kOffQ + t * Cfg::kTileBytes, ka = sbase + Cfg::kOffK + kstage * Cfg::kTileBytes;
        // one election per product (see the note on issue in sm100_ptx.cuh)
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
            umma_ss(tmem + d_col, umma_smem_desc_sw128(qa + off, 16, 1024), umma_smem_desc_sw128(ka + off, 16, 1024),
                    idesc_qk, ks > 0);
          }
        }
        __syncwarp();
      };
      auto issue_pv = [&](int t, int vstage, bool acc) {
        const uint32_t va = sbase + Cfg::kOffV + vstage * Cfg::kTileBytes;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)   // 128 keys, 16 per UMMA
            umma_ts(tmem + 256 + t * 128, tmem + t * 128 + ks * 8, umma_smem_desc_sw128(va + ks * 2048, 16384, 1024),
                    idesc_pv, (acc || ks > 0) ? 1u : 0u);
        }
        __syncwarp();
      };
      bool ok = true;
      uint32_t g0 = 0;                      // K/V tiles of the items before this one
      int it = 0;
      for (int item = first_item; item < p.n_items && ok; item += item_step, ++it, g0 += n_tiles) {
        ok = mbar_wait_warp(bar(BAR_Q_FULL), it & 1, ab, p.err, 201);
        if (HAS_V) {
          // P(t) lives over S(t) and the tensor pipe runs in order, so the first product of an item may
          // follow the last P V of the previous one at once; O(t) is overwritten by the P V of step 0,
          // which waits for a P that the softmax warps write only after they have read the old O(t).
          if (ok) ok = mbar_wait_warp(bar(BAR_K_FULL + g0 % kKSt), (g0 / kKSt) & 1, ab, p.err, 202);
          if (ok) {
            tc_fence_after();
            for (int t = t_lo; t < t_hi; ++t) {
              if (!((tiles >> t) & 1u)) continue;
              issue_qk(t, g0 % kKSt, t * 128);
              umma_commit_elect(bar(BAR_S_FULL + t * 2));
            }
            umma_commit_elect(bar(BAR_K_EMPTY + g0 % kKSt));
            if (n_tiles == 1) umma_commit_elect(bar(BAR_Q_EMPTY));
          }
          for (int j = 0; j < n_tiles && ok; ++j) {
            const uint32_t g = g0 + j;
            const int vs = g % Cfg::kVStages;
            ok = mbar_wait_warp(bar(BAR_V_FULL + vs), (g / Cfg::kVStages) & 1, ab, p.err, 203);
            const bool more = (j + 1 < n_tiles);
            const int ks = (g + 1) % kKSt;
            if (ok && more) ok = mbar_wait_warp(bar(BAR_K_FULL + ks), ((g + 1) / kKSt) & 1, ab, p.err, 204);
            for (int t = t_lo; t < t_hi && ok; ++t) {
              if (!((tiles >> t) & 1u)) continue;
              ok = mbar_wait_warp(bar(BAR_P_FULL + t), g & 1, ab, p.err, 205);
              if (!ok) break;
              tc_fence_after();
              issue_pv(t, vs, j > 0);
              if (more) {
                issue_qk(t, ks, t * 128);
                umma_commit_elect(bar(BAR_S_FULL + t * 2));
              } else {
                umma_commit_elect(bar(BAR_O_FULL + t));
              }
            }
            if (ok) {
              umma_commit_elect(bar(BAR_V_EMPTY + vs));
              if (more) umma_commit_elect(bar(BAR_K_EMPTY + ks));
              if (j + 2 == n_tiles) umma_commit_elect(bar(BAR_Q_EMPTY));
            }
          }
        } else {
          // no V: S is double-buffered per query tile; tile t, buffer b lives at column (2t+b)*128
          for (int j = 0; j < n_tiles && ok; ++j) {
            const uint32_t g = g0 + j;
            const int ks = g % kKSt, b = g & 1;
            const uint32_t f = g >> 1;
            ok = mbar_wait_warp(bar(BAR_K_FULL + ks), (g / kKSt) & 1, ab, p.err, 206);
            for (int t = t_lo; t < t_hi && ok; ++t) {
              if (!((tiles >> t) & 1u)) continue;
              if (f > 0) ok = mbar_wait_warp(bar(BAR_S_EMPTY + t * 2 + b), (f - 1) & 1, ab, p.err, 207);
              if (!ok) break;
              tc_fence_after();
              issue_qk(t, ks, (t * 2 + b) * 128);
              umma_commit_elect(bar(BAR_S_FULL + t * 2 + b));
            }
            if (ok) {
              umma_commit_elect(bar(BAR_K_EMPTY + ks));
              if (j + 1 == n_tiles) umma_commit_elect(bar(BAR_Q_EMPTY));
            }
          }
        }
        if (!PERSIST) break;
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax warpgroups
    reg_alloc<216>();
    const int t = warp >> 2;                           // query tile of this warpgroup
    const int wq = warp & 3;                           // TMEM lane quarter
    const int row_in_tile = wq * 32 + lane;
    const uint32_t lane_base = tmem + (uint32_t(wq * 32) << 16);
    const float c = p.scale_log2;
    bool ok = ((tiles >> t) & 1u) != 0;                // a half item: the other tile's warpgroup has nothing to do
    uint32_t g0 = 0;                                   // K/V tiles of the items before this one
    int it = 0;
    for (int item = first_item; item < p.n_items && ok; item += item_step, ++it, g0 += n_tiles) {
      const int bh = item / p.n_pairs, q0 = (item - bh * p.n_pairs) * 256;
      const int row = q0 + t * 128 + row_in_tile;      // query row in the sequence
      const size_t ml_off = size_t(p.bh0 + bh) * p.S_pad + row;

      OnlineState st;
      online_init(st);
      float t_row = INFINITY;       // kTokenMask: m*c + log2(l)
      if (MODE == kTokenMask) {
        if (row < p.S) t_row = p.max_q[ml_off] * c + log2f(p.denom[ml_off]);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const uint32_t g = g0 + j;
        const int b = HAS_V ? 0 : int(g & 1);
        const uint32_t fpar = HAS_V ? (g & 1) : ((g >> 1) & 1);
        ok = mbar_wait(bar(BAR_S_FULL + t * 2 + b), fpar, ab, p.err, 301);
        if (!ok) break;
        tc_fence_after();
        const uint32_t s_addr = lane_base + (HAS_V ? t * 128 : (t * 2 + b) * 128);
        const int key0 = tile_of(j) * 128;               // first key of this tile
        const int kv_left = p.kv_len - key0;             // valid keys in this tile
        const int valid0 = min(64, kv_left), valid1 = max(0, min(64, kv_left - 64));
        if (MODE == kTokenMask) {
          // per-token keep bit: any row of the 128-row block with s*c - t_row > log2(tau), i.e.
          // s > thr.  Most 32-column quarters hold no such entry in any row of the warp: their row
          // maxima settle that with one instruction per entry, and only the others build bits.
          const float thr = (p.log2_tau + t_row) / c;          // +inf for rows past the sequence
          uint32_t r[128];
#pragma unroll
          for (int w = 0; w < 4; ++w) tmem_ld32(s_addr + w * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[w * 32]));
          tmem_ld_wait();
          tc_fence_before();
          mbar_arrive(bar(BAR_S_EMPTY + t * 2 + b));           // the scores are in registers: free the buffer
          uint32_t bits[4];
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            float mx = __uint_as_float(r[w * 32]);
#pragma unroll
            for (int i = 1; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[w * 32 + i]));
            bits[w] = 0u;
            if (__any_sync(0xffffffffu, mx > thr)) {
              uint32_t m = 0;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (__uint_as_float(r[w * 32 + i]) > thr) m |= 1u << i;
              const int lim = kv_left - w * 32;                  // live columns of this quarter
              m &= (lim >= 32) ? 0xffffffffu : (lim <= 0 ? 0u : ((1u << lim) - 1u));
              bits[w] = __reduce_or_sync(0xffffffffu, m);
            }
          }
          // the caller-zeroed mask is only ever set to 1 (by up to four warps of 32 rows each)
          if (q0 + t * 128 < p.S) {
            const int qblk = (q0 + t * 128) >> 7;
            int* mrow = p.tokenmask + (size_t(p.bh0 + bh) * ((p.S + 127) >> 7) + qblk) * p.mask_stride + key0;
#pragma unroll
            for (int w = 0; w < 4; ++w)
              if ((bits[w] >> lane) & 1u) mrow[w * 32 + lane] = 1;
          }
          continue;
        }
        float mx0, mx1;
        softmax_online_step<D, HAS_V>(s_addr, lane_base + t * 128, lane_base + 256 + t * 128, valid0, valid1, c, j == 0,
                                      st, mx0, mx1);
        tc_fence_before();
        if (HAS_V) mbar_arrive(bar(BAR_P_FULL + t));
        else mbar_arrive(bar(BAR_S_EMPTY + t * 2 + b));
        if (BLOCKMAX) {
          if (row < p.S_pad) {
            float* bm = p.blockmax + (size_t(bh) * p.nkb + size_t(j) * 2) * p.S_pad + row;
            bm[0] = mx0;
            if (j * 2 + 1 < p.nkb) bm[p.S_pad] = mx1;
          }
        }
      }
      // ---- epilogue of the item
      if (ok && HAS_V) {
        ok = mbar_wait(bar(BAR_O_FULL + t), it & 1, ab, p.err, 302);
        if (ok) {
          tc_fence_after();
          store_o_row<D>(lane_base + 256 + t * 128, p.o + (size_t(p.bh0 + bh) * p.S + row) * D, 1.0f / st.l, row < p.S);
          tc_fence_before();       // the next item's first P V product overwrites O(t)
        }
      }
      if (ok && WRITE_ML) {
        if (row < p.S) {
          p.max_q[ml_off] = st.m_true;
          p.denom[ml_off] = st.l * ex2(st.m_used - st.m_true * c);
        } else if (row < p.S_pad) {
          p.max_q[ml_off] = 0.f;
          p.denom[ml_off] = -INFINITY;
        }
      }
      if (!PERSIST) break;
    }
  }
  else {
    reg_dealloc<72>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace fg
