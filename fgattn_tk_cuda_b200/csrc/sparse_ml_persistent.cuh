// Persistent block-sparse gather attention with precomputed (max_q, denom), sm_100a.
//
// Work item = one PAIR of neighbouring 64-row query blocks (one 128-row UMMA tile) of one
// (batch, head) unit, walking the sorted union of the pair's two key-block lists, two listed key
// blocks (128 keys) per step.  CTAs are persistent and pull items from a global queue; heads are
// queued in small groups (their K/V fits in L2) and inside a group the items are ordered
// longest-list-first.
//
// Because the probabilities are p = 2^(s*c - (m*c + log2 l)) with m, l given, no row reduction is
// needed, so the softmax work of a step can be cut by columns: four softmax warpgroups form two
// pairs that take the steps alternately (pair = step parity), and inside a pair each warpgroup owns
// one of the step's two 64-key blocks, one query row per thread.  While one pair is in the
// exponential-bound part of its step the other pair is in the wait / load / store / signal part of
// the next one.
//
// Tensor memory (512 columns): three 128-column score buffers S[3] and the output accumulator O
// (128).  A warpgroup writes its packed bf16 probabilities over the first half of its OWN score
// columns, so there are no separate probability buffers and nothing to wait for before the store;
// a buffer is handed back to the Q K^T issuer by the commit of the P*V product that consumed it:
//   Q K^T issuer           : S[s%3] = Q K_s^T           needs K_s and the P*V product of step s-3
//   softmax pair (s&1)     : P (in S[s%3]) = 2^(S*c - t) needs S[s%3]
//   P V issuer             : O += P V_s                  needs both key blocks of P and V_s
// Barriers that a role waits on only every other step (score-full, probability-full) exist once per
// (buffer, pair), i.e. per step mod 6, because a parity wait must see every phase of its barrier.
// Service warps after the softmax warps: TMA producer of Q and the K ring, Q K^T issuer, scheduler
// (queue + union lists; it builds the next item's union bitmaps while it waits for a free list buffer), P V issuer,
// TMA producer of the V ring.
//
// RENORM = true is the renormalising form (softmax over the kept keys only, what the sp_attn operator
// computes) on the same schedule.  A softmax is invariant under a shift of its exponents, and the
// running maximum of the online form is only there to keep the exponentials in range, so each row
// uses a FIXED offset instead: p = 2^(s*c - hint*c) with `hint` a per-row estimate of the row maximum
// handed in by the caller (the max_q of the pass that built the lists is a good one even when q has
// moved on by a diffusion step: anything within about +-60 of the true maximum in the log2 domain
// works, because bf16 probabilities and the fp32 accumulator keep their relative precision over that
// range).  Every softmax thread sums the probabilities it produced, the four warpgroups' partial sums
// of a row meet in shared memory once per item, and the epilogue scales the accumulator by 1/l.  A row
// whose sum left the safe range (overflow: inf / NaN, underflow: below 2^-60) marks its item in
// `redo`; the host then re-runs the marked items on the kernel with the running maximum.
#pragma once
#include "sm100_ptx.cuh"
#include "softmax_steps.cuh"
#include "sparse_attn.cuh"


namespace fg {

struct SparseMLParams {
  __nv_bfloat16* o;          // [BH, S, D]
  const float* max_q;        // [BH, S_pad]
  const float* denom;        // [BH, S_pad]
  const int* kb_idx;         // [BH, nqb, list_stride]
  const int* kb_cnt;         // [BH, nqb]
  const int* order;          // [BH * npairs] item ids (unit * npairs + pair) in queue order
  int* queue;                // global item counter (zeroed before the launch)
  int* err;
  int* redo;                 // RENORM: [BH * npairs] flags (zeroed before the launch); 1 = item must be re-run
  // Token-derived lists (null = key-block lists of 64-row query blocks): every 128-row query block has ONE
  // list, [BH, npairs, list_stride] ascending key blocks, and kb_mask gives the live columns of each listed
  // block ([BH, npairs, list_stride], bit j = key 64 * block + j takes part).  route (optional,
  // [BH * npairs]): items with route == 0 are left to another kernel.
  const unsigned long long* kb_mask;
  const int* route;
  int S, S_pad, kv_len, nqb, nkb, npairs, n_items, list_stride, list_cap;
  float scale_log2;
  long long* stats;          // tuning builds (-DFG_STATS), debug & 8: per-CTA cycle counters [gridDim.x][32]
  int debug;                 // tuning builds only: 1 = no K/V loads, 2 = no UMMA, 4 = no softmax math
};

template <int D>
struct SparseMLCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kKStages = (D == 128) ? 2 : 4;
  static constexpr int kVStages = (D == 128) ? 2 : 4;
  // Items the scheduler may be ahead of the slowest reader of a list.  Measured: at D = 128 two is better than
  // four (C3 0.622 -> 0.604 ms, 32 units of the C5 shape 7.62 -> 7.34 ms; three lies in between), at D = 64 four is
  // better than two (C4 0.401 -> 0.432 ms): its items are short and a step takes 1000 instead of 1650 clocks, so
  // the lists have to be under way earlier.
  static constexpr int kListBufs = (D == 128) ? 2 : 4;
  // warp roles: [0, kSmWarps) softmax, then K producer, QK issuer, scheduler, PV issuer, V producer
  static constexpr int kSmWGs = 4;                        // two pairs of softmax warpgroups
  static constexpr int kSmWarps = 4 * kSmWGs;
  static constexpr int kWarpProdK = kSmWarps, kWarpQK = kSmWarps + 1, kWarpSched = kSmWarps + 2,
                       kWarpPV = kSmWarps + 3, kWarpProdV = kSmWarps + 4;
  static constexpr int kThreads = 32 * (kSmWarps + 8);
  // registers: the CTA owns (launch registers x threads); service warps shrink, softmax warps grow
  static constexpr int kRegsService = 40;
  static constexpr int kRegsSoftmax = 96;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = 2 * kTileBytes;
  static constexpr int kOffV = kOffK + kKStages * kTileBytes;
  // D = 64 leaves 64 columns of tensor memory free next to the accumulator: the renormalising form keeps its
  // row sums there, l = P * 1 as one more (N = 16) product per P*V step against a tile of ones, so the softmax
  // threads add nothing up.  The tile of ones: 16 keys x 64 columns of bf16 1.0 (2 KiB, any layout).
  static constexpr bool kTensorRowSum = (D == 64);
  static constexpr int kOffOnes = kOffV + kVStages * kTileBytes;
  static constexpr int kOffBar = kOffOnes + (kTensorRowSum ? 2048 : 0);
  static constexpr int kBarBytes = 768;
  // [kListBufs][list_cap] entries, then [2][words] bitmaps, then [4][4][128] partial row sums (RENORM)
  static constexpr int kOffList = kOffBar + kBarBytes;
  static constexpr int kRowSumBytes = 4 * kSmWGs * 128 * 4;
  static __host__ __device__ constexpr int smem_bytes(int list_cap, int nkb) {
    return kOffList + kListBufs * list_cap * 4 + 2 * ((nkb + 31) / 32) * 4 + kRowSumBytes + 1024;
  }
};

enum : int {
  PB_LIST_FULL = 0,    // +list buffer (4)
  PB_LIST_EMPTY = 4,   // +list buffer (4)
  PB_Q_FULL = 8,       // +q buffer (2)
  PB_Q_EMPTY = 10,     // +q buffer (2)
  PB_K_FULL = 12,      // +stage (<=4)
  PB_K_EMPTY = 16,     // +stage
  PB_V_FULL = 20,      // +stage (<=4)
  PB_V_EMPTY = 24,     // +stage
  PB_S_FULL = 28,      // +(step % 6) (6): a barrier per (score buffer, owning pair), so that every waiter of a
                       // barrier waits for each of its phases (a parity wait cannot skip phases)
  PB_S_EMPTY = 34,     // +score buffer (3): the P*V product that read the buffer's probabilities is done
  PB_O_FULL = 37,
  PB_O_EMPTY = 38,
  PB_P_FULL = 40,      // +(step % 6) * 2: both key blocks of the step (eight warps arrive)
  PB_L_FULL = 52,      // +(item % 4) (4): RENORM, the item's partial row sums are in shared memory
  PB_COUNT = 56
};

struct ItemInfo {
  int n_steps;   // -1: queue exhausted
  int bh;
  int pair;
  int halves;    // bit h: the 64-row query block h of the pair has a non-empty list
};

// N score columns -> N/2 packed bf16 probability columns, p = 2^(s*c - t_row).  SUM: the
// probabilities are also added to the two running sums.
template <int N, bool SUM>
__device__ __forceinline__ void ml_probs(const uint32_t (&r)[N], uint32_t (&pk)[N / 2], int valid, float c,
                                         float t_row, float& sum0, float& sum1) {
  const uint64_t c2 = f2_pack(c, c), nt2 = f2_pack(-t_row, -t_row);
#pragma unroll
  for (int i = 0; i < N; i += 2) {
    float x0, x1;
    f2_unpack(f2_fma(f2_pack(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), c2, nt2), x0, x1);
    float p0 = ex2(x0), p1 = ex2(x1);
    if (valid < N) {
      if (i >= valid) p0 = 0.f;
      if (i + 1 >= valid) p1 = 0.f;
    }
    if (SUM) {
      sum0 += p0;
      sum1 += p1;
    }
    pk[i >> 1] = pack_bf16(p0, p1);
  }
}
// The same with an arbitrary set of live columns (bit i of `live` = column i takes part).
template <bool SUM>
__device__ __forceinline__ void ml_probs_masked(const uint32_t (&r)[32], uint32_t (&pk)[16], uint32_t live, float c,
                                                float t_row, float& sum0, float& sum1) {
  const uint64_t c2 = f2_pack(c, c), nt2 = f2_pack(-t_row, -t_row);
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float x0, x1;
    f2_unpack(f2_fma(f2_pack(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), c2, nt2), x0, x1);
    float p0 = ex2(x0), p1 = ex2(x1);
    if (!((live >> i) & 1u)) p0 = 0.f;
    if (!((live >> (i + 1)) & 1u)) p1 = 0.f;
    if (SUM) {
      sum0 += p0;
      sum1 += p1;
    }
    pk[i >> 1] = pack_bf16(p0, p1);
  }
}


// TOKEN: token-derived lists with column masks (SparseMLParams::kb_mask), otherwise key-block lists
template <int D, bool RENORM, bool TOKEN = false>
__global__ void __launch_bounds__(SparseMLCfg<D>::kThreads, 1)
sparse_ml_persistent_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                            const __grid_constant__ CUtensorMap mv, const SparseMLParams p) {
  using Cfg = SparseMLCfg<D>;
  constexpr int NLB = Cfg::kListBufs;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + Cfg::kOffBar;
  auto bar = [&](int i) -> uint32_t { return bars + 8u * uint32_t(i); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffBar + 8 * PB_COUNT);
  AbortState* ab = reinterpret_cast<AbortState*>(smem + Cfg::kOffBar + 8 * PB_COUNT + 8);
  volatile ItemInfo* info = reinterpret_cast<volatile ItemInfo*>(smem + Cfg::kOffBar + 8 * PB_COUNT + 16);   // [NLB]
  uint32_t* lists = reinterpret_cast<uint32_t*>(smem + Cfg::kOffList);                                       // [NLB][cap]
  uint32_t* bitmaps = lists + NLB * p.list_cap;                                                              // [2][words]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int words = (p.nkb + 31) / 32;
  float* rowsum = reinterpret_cast<float*>(bitmaps + 2 * words);                                             // [4][4][128]
#ifdef FG_STATS
  const int dbg = p.debug;
#else
  constexpr int dbg = 0;               // the timing experiments exist in tuning builds only
#endif
  constexpr uint32_t kColS = 0, kColO = 384;           // three 128-column score buffers, then the accumulator
  constexpr int kSB = 3;
  constexpr bool TSUM = RENORM && Cfg::kTensorRowSum;  // row sums by the tensor cores, 16 columns behind O
  constexpr uint32_t kColL = kColO + 64;
  if constexpr (TSUM) {
    uint32_t* ones = reinterpret_cast<uint32_t*>(smem + Cfg::kOffOnes);
    for (int i = tid; i < 512; i += Cfg::kThreads) ones[i] = 0x3F803F80u;     // bf16 1.0 pairs
    fence_proxy_async_smem();
  }

  if (tid == 0) {
    ab->flag = 0;
    for (int b = 0; b < NLB; ++b) {
      mbar_init(bar(PB_LIST_FULL + b), 1);
      mbar_init(bar(PB_LIST_EMPTY + b), 4 + Cfg::kSmWarps);   // two producers + two issuers + softmax warps
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(PB_Q_FULL + b), 1);
      mbar_init(bar(PB_Q_EMPTY + b), 1);
    }
    for (int b = 0; b < kSB; ++b) mbar_init(bar(PB_S_EMPTY + b), 1);
    for (int i = 0; i < 6; ++i) {
      mbar_init(bar(PB_S_FULL + i), 1);
      mbar_init(bar(PB_P_FULL + i * 2), 8);        // both warpgroups of the pair: four warps each
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(bar(PB_K_FULL + s), 1);
      mbar_init(bar(PB_K_EMPTY + s), 1);
      mbar_init(bar(PB_V_FULL + s), 1);
      mbar_init(bar(PB_V_EMPTY + s), 1);
    }
    mbar_init(bar(PB_O_FULL), 1);
    mbar_init(bar(PB_O_EMPTY), Cfg::kSmWarps);
    for (int i = 0; i < 4; ++i) mbar_init(bar(PB_L_FULL + i), Cfg::kSmWarps);
    mbar_fence_init();
  }
  if (warp == Cfg::kWarpProdK) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == Cfg::kWarpSched) {
    // ------------------------------------------------------------------ scheduler: queue + union lists
    reg_dealloc<Cfg::kRegsService>();
    uint32_t* bm0 = bitmaps;
    uint32_t* bm1 = bitmaps + words;
    long long w_le = 0, t_start = FG_CLK();
    int it = 0;
    for (;; ++it) {
      const int lb = it % NLB;
      bool ok = true;
      // Everything that needs global memory -- the queue, the item's two lists -- and the union bitmaps (private
      // to this warp) come BEFORE the wait for a free list buffer, so that only the scan is left when the readers
      // of the item before last let go of it.
      int g = 0, item = 0;
      for (;;) {                                           // next item of the queue that is routed to this kernel
        if (lane == 0) g = atomicAdd(p.queue, 1);
        g = __shfl_sync(0xffffffffu, g, 0);
        if (g >= p.n_items) break;
        item = p.order[g];
        if (!TOKEN || !p.route || p.route[item] != 0) break;
      }
      const bool done = g >= p.n_items;
      int bh = 0, pair = 0;
      int n_half[2] = {0, 0};
      if (!done) {
        bh = item / p.npairs;
        pair = item - bh * p.npairs;
        constexpr bool token_lists = TOKEN;
        const int list_rows = token_lists ? p.npairs : p.nqb;
        for (int w = lane; w < 2 * words; w += 32) bm0[w] = 0u;
        __syncwarp();
        // both halves' counts are fetched before either list is walked
        const int* src_half[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int qb = token_lists ? pair : pair * 2 + half;     // token lists: both halves walk the one list
          src_half[half] = p.kb_idx;
          if (qb < list_rows) {
            src_half[half] = p.kb_idx + (size_t(bh) * list_rows + qb) * p.list_stride;
            n_half[half] = min(p.kb_cnt[size_t(bh) * list_rows + qb], p.list_stride);
          }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t* bm = half ? bm1 : bm0;
          for (int i = lane; i < n_half[half]; i += 32) {
            const int kb = src_half[half][i];
            if (kb >= 0 && kb < p.nkb) atomicOr(&bm[kb >> 5], 1u << (kb & 31));
          }
        }
        __syncwarp();
      }
      if (it >= NLB) FG_TW(w_le, ok = mbar_wait_relaxed(bar(PB_LIST_EMPTY + lb), ((it / NLB) - 1) & 1, ab, p.err, 1001));
      if (!ok) break;
      if (done) {
        if (lane == 0) {
          info[lb].n_steps = -1;
          mbar_arrive(bar(PB_LIST_FULL + lb));
        }
        break;
      }
      // ascending union list: lane j looks at key block 32 w + j of bitmap word w, the word itself is the ballot
      uint32_t* out = lists + lb * p.list_cap;
      int base = 0;
      for (int w = 0; w < words; ++w) {
        const uint32_t a = bm0[w], bb = bm1[w];
        const uint32_t u = a | bb;
        if ((u >> lane) & 1u) {
          const int off = base + __popc(u & ((1u << lane) - 1u));
          if (off < p.list_cap) out[off] = uint32_t(w * 32 + lane) | (((a >> lane) & 1u) << 30) | (((bb >> lane) & 1u) << 31);
        }
        base += __popc(u);
      }
      if (base > p.list_cap - 1) base = p.list_cap - 1;
      __syncwarp();
      if (lane == 0) {
        if (base & 1) {                                  // odd: repeat the last block, kept by nobody
          out[base] = out[base - 1] & 0x3FFFFFFFu;
          ++base;
        }
        info[lb].bh = bh;
        info[lb].pair = pair;
        info[lb].halves = (n_half[0] > 0 ? 1 : 0) | (n_half[1] > 0 ? 2 : 0);
        info[lb].n_steps = base >> 1;
        mbar_arrive(bar(PB_LIST_FULL + lb));
      }
      __syncwarp();
    }
    if (p.stats && lane == 0) {
      long long* st_ = p.stats + size_t(blockIdx.x) * 32;
      st_[5] = FG_CLK() - t_start; st_[6] = w_le; st_[7] = it;
    }
  } else if (warp == Cfg::kWarpProdK || warp == Cfg::kWarpProdV) {
    // ------------------------------------------------------------------ TMA producers
    // Warp 8 feeds Q (per item) and the K ring, warp 12 the V ring.  They walk the same item / step
    // sequence independently, so a V stage that is still waiting for its P*V product never holds
    // back the K tiles of the steps ahead.
    reg_dealloc<Cfg::kRegsService>();
    if (lane == 0) {
      const bool is_k = (warp == Cfg::kWarpProdK);
      const CUtensorMap* m = is_k ? &mk : &mv;
      if (is_k) tma_prefetch_desc(&mq);
      tma_prefetch_desc(m);
      const int n_stages = is_k ? Cfg::kKStages : Cfg::kVStages;
      const uint32_t ring = sbase + (is_k ? Cfg::kOffK : Cfg::kOffV);
      const int full0 = is_k ? PB_K_FULL : PB_V_FULL, empty0 = is_k ? PB_K_EMPTY : PB_V_EMPTY;
      int s = 0, u = 0;
      bool ok = true;
      for (int it = 0; ok; ++it) {
        const int lb = it % NLB;
        ok = mbar_wait_relaxed(bar(PB_LIST_FULL + lb), (it / NLB) & 1, ab, p.err, 1102);
        if (!ok) break;
        const int n = info[lb].n_steps;
        if (n < 0) break;
        if (n > 0) {
          const int bh = info[lb].bh, pair = info[lb].pair;
          if (is_k) {
            const int qb = u & 1;
            if (u >= 2) ok = mbar_wait_relaxed(bar(PB_Q_EMPTY + qb), ((u >> 1) - 1) & 1, ab, p.err, 1103);
            if (!ok) break;
            mbar_arrive_expect_tx(bar(PB_Q_FULL + qb), Cfg::kTileBytes);
            for (int h = 0; h < Cfg::kHalves; ++h)
              tma_load_3d(sbase + Cfg::kOffQ + qb * Cfg::kTileBytes + h * 16384, &mq, bar(PB_Q_FULL + qb), h * 64,
                          pair * 128, bh);
          }
          const uint32_t* list = lists + lb * p.list_cap;
          for (int j = 0; j < n && ok; ++j, ++s) {
            const int kb0 = entry_kb(list[2 * j]), kb1 = entry_kb(list[2 * j + 1]);
            const int st = s % n_stages, f = s / n_stages;
            if (f > 0) ok = mbar_wait_relaxed(bar(empty0 + st), (f - 1) & 1, ab, p.err, 1104);
            if (!ok) break;
            const uint32_t dst = ring + st * Cfg::kTileBytes, full_bar = bar(full0 + st);
            if (dbg & 1) {
              mbar_arrive(full_bar);
            } else {
              mbar_arrive_expect_tx(full_bar, Cfg::kTileBytes);
              for (int h = 0; h < Cfg::kHalves; ++h) {
                tma_load_3d(dst + h * 16384, m, full_bar, h * 64, kb0 * 64, bh);
                tma_load_3d(dst + h * 16384 + 8192, m, full_bar, h * 64, kb1 * 64, bh);
              }
            }
          }
          ++u;
        }
        if (ok) mbar_arrive(bar(PB_LIST_EMPTY + lb));
      }
      if (!ok) {
        for (int i = max(0, s - n_stages); i < s; ++i) mbar_wait_brief(bar(full0 + i % n_stages), (i / n_stages) & 1);
        if (is_k)
          for (int i = max(0, u - 2); i < u; ++i) mbar_wait_brief(bar(PB_Q_FULL + (i & 1)), (i >> 1) & 1);
      }
    }
  } else if (warp == Cfg::kWarpQK) {
    // ------------------------------------------------------------------ Q K^T issuer
    // Whole warp, uniform control flow; each instruction is issued by one elected lane.
    reg_dealloc<Cfg::kRegsService>();
    const uint32_t idesc_qk = umma_idesc_bf16(128, 128, false);
    int s = 0, u = 0;
    bool ok = true;
    long long w_k = 0, w_se = 0, w_misc = 0, w_q = 0, t_start = FG_CLK();
    for (int it = 0; ok; ++it) {
      const int lb = it % NLB;
      FG_TW(w_misc, ok = mbar_wait_warp(bar(PB_LIST_FULL + lb), (it / NLB) & 1, ab, p.err, 1201));
      if (!ok) break;
      const int n = info[lb].n_steps;
      if (n < 0) break;
      if (lane == 0) mbar_arrive(bar(PB_LIST_EMPTY + lb));        // only n is needed from the list buffer
      __syncwarp();
      if (n > 0) {
        const int qb = u & 1;
        FG_TW(w_q, ok = mbar_wait_warp(bar(PB_Q_FULL + qb), (u >> 1) & 1, ab, p.err, 1202));
        const uint32_t qa = sbase + Cfg::kOffQ + qb * Cfg::kTileBytes;
        for (int j = 0; j < n && ok; ++j, ++s) {
          const int ks = s % Cfg::kKStages, sbuf = s % kSB;
          FG_TW(w_k, ok = mbar_wait_warp(bar(PB_K_FULL + ks), (s / Cfg::kKStages) & 1, ab, p.err, 1203));
          if (ok && s >= kSB) FG_TW(w_se, ok = mbar_wait_warp(bar(PB_S_EMPTY + sbuf), ((s / kSB) - 1) & 1, ab, p.err, 1204));
          if (!ok) break;
          tc_fence_after();
          const uint32_t ka = sbase + Cfg::kOffK + ks * Cfg::kTileBytes;
          // one election for the whole product and its commits (see the note on issue in sm100_ptx.cuh)
          if (elect_one()) {
            if (!(dbg & 2)) {
#pragma unroll
              for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
                umma_ss(tmem + kColS + sbuf * 128, umma_smem_desc_sw128(qa + off, 16, 1024),
                        umma_smem_desc_sw128(ka + off, 16, 1024), idesc_qk, kk > 0);
              }
            }
            umma_commit(bar(PB_S_FULL + s % 6));
            umma_commit(bar(PB_K_EMPTY + ks));
            if (j == n - 1) umma_commit(bar(PB_Q_EMPTY + qb));
          }
          __syncwarp();
        }
        ++u;
      }
    }
    if (p.stats && lane == 0) {
      long long* st_ = p.stats + size_t(blockIdx.x) * 32;
      st_[0] = FG_CLK() - t_start; st_[1] = w_k; st_[2] = w_se; st_[3] = w_misc; st_[4] = s; st_[13] = w_q;
    }
  } else if (warp == Cfg::kWarpPV) {
    // ------------------------------------------------------------------ P V issuer
    reg_dealloc<Cfg::kRegsService>();
    const uint32_t idesc_pv = umma_idesc_bf16(128, D, true);
    const uint32_t idesc_l = umma_idesc_bf16(128, 16, true);
    const uint64_t ones_desc = umma_smem_desc_sw128(sbase + Cfg::kOffOnes, 16384, 1024);
    int s = 0, u = 0;
    bool ok = true;
    long long w_v = 0, w_p = 0, w_o = 0, w_misc = 0, t_start = FG_CLK();
    for (int it = 0; ok; ++it) {
      const int lb = it % NLB;
      FG_TW(w_misc, ok = mbar_wait_warp(bar(PB_LIST_FULL + lb), (it / NLB) & 1, ab, p.err, 1301));
      if (!ok) break;
      const int n = info[lb].n_steps;
      if (n < 0) break;
      if (lane == 0) mbar_arrive(bar(PB_LIST_EMPTY + lb));        // only n is needed from the list buffer
      __syncwarp();
      if (n > 0) {
        // the accumulator is single-buffered: the previous item's rows must have been read out
        if (u >= 1) FG_TW(w_o, ok = mbar_wait_warp(bar(PB_O_EMPTY), (u - 1) & 1, ab, p.err, 1302));
        for (int j = 0; j < n && ok; ++j, ++s) {
          const int vs = s % Cfg::kVStages, pbuf = s % kSB;
          FG_TW(w_v, ok = mbar_wait_warp(bar(PB_V_FULL + vs), (s / Cfg::kVStages) & 1, ab, p.err, 1303));
          const uint32_t va = sbase + Cfg::kOffV + vs * Cfg::kTileBytes;
          // the step's two key blocks come from the two warpgroups of the pair that owns the step; one wait for
          // both and one elected lane for the whole product and its commits (a wait per key block, so that the
          // first four instructions could go ahead of the second block's probabilities, was 1-3 % slower)
          FG_TW(w_p, ok = mbar_wait_warp(bar(PB_P_FULL + (s % 6) * 2), (s / 6) & 1, ab, p.err, 1304));
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            if (!(dbg & 2)) {
#pragma unroll
              for (int ks = 0; ks < 8; ++ks) {                  // 16-key step inside the 128-key tile
                umma_ts(tmem + kColO, tmem + kColS + pbuf * 128 + (ks / 4) * 64 + (ks % 4) * 8,
                        umma_smem_desc_sw128(va + ks * 2048, 16384, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                if constexpr (TSUM)                          // l += P * 1
                  umma_ts(tmem + kColL, tmem + kColS + pbuf * 128 + (ks / 4) * 64 + (ks % 4) * 8, ones_desc, idesc_l,
                          (j > 0 || ks > 0) ? 1u : 0u);
              }
            }
            umma_commit(bar(PB_V_EMPTY + vs));
            umma_commit(bar(PB_S_EMPTY + pbuf));           // scores and probabilities of this buffer are consumed
            if (j == n - 1) umma_commit(bar(PB_O_FULL));
          }
          __syncwarp();
        }
        ++u;
      }
    }
    if (p.stats && lane == 0) {
      long long* st_ = p.stats + size_t(blockIdx.x) * 32 + 8;
      st_[0] = FG_CLK() - t_start; st_[1] = w_v; st_[2] = w_p; st_[3] = w_o; st_[4] = w_misc;
    }
  } else if (warp < Cfg::kSmWarps) {
    // ------------------------------------------------------------------ softmax warpgroups
    // Two pairs of warpgroups take the steps alternately; a warpgroup turns the 64 score columns of
    // one key block into probabilities, one query row per thread, in two 32-column halves.
    reg_alloc<Cfg::kRegsSoftmax>();
    const int wg = warp >> 2, wq = warp & 3, half = wq >> 1;
    const int row_in_tile = wq * 32 + lane;
    const uint32_t lane_base = tmem + (uint32_t(wq * 32) << 16);
    const float c = p.scale_log2;
    constexpr int kOCols = D / Cfg::kSmWGs;              // output columns stored by this warpgroup
    static_assert(Cfg::kSmWGs == 4, "two pairs of softmax warpgroups");
    const int own = wg >> 1;                             // this warpgroup owns the steps with (s & 1) == own
    const int kb_sel = wg & 1;                           // which of an owned step's two key blocks
    int s = 0, u = 0;
    bool ok = true;
    long long w_s = 0, w_list = 0, w_epi = 0, w_pe = 0, t_math = 0, t_prol = 0, t_epiw = 0, t_ld = 0, t_st = 0,
              t_start = FG_CLK();
    bool pe = false;                                     // pending epilogue of the previous item
    int pe_par = 0;
    __nv_bfloat16* pe_orow = nullptr;
    bool pe_in = false;
    int pe_u = 0, pe_item = 0;                           // RENORM: item counter / global item id of the pending rows
    bool pe_listed = false;                              // RENORM: this row's query block has a non-empty list
    auto epilogue = [&]() {
      FG_TW(w_epi, ok = mbar_wait(bar(PB_O_FULL), pe_par, ab, p.err, 1401));
      if (!ok) return;
      float inv = 1.0f;
      if constexpr (RENORM) {
        float l;
        if constexpr (TSUM) {
          // the row sum sits in tensor memory next to the accumulator (every one of its 16 columns)
          tc_fence_after();
          uint32_t lv[16];
          tmem_ld16(lane_base + kColL, lv);
          tmem_ld_wait();
          l = __uint_as_float(lv[0]);
        } else {
          // the four warpgroups' partial sums of this row
          FG_TW(w_epi, ok = mbar_wait(bar(PB_L_FULL + (pe_u & 3)), (pe_u >> 2) & 1, ab, p.err, 1404));
          if (!ok) return;
          const float* ls = rowsum + (pe_u & 3) * (Cfg::kSmWGs * 128) + row_in_tile;
          l = (ls[0] + ls[128]) + (ls[256] + ls[384]);
        }
        // the row's output is O / l
        const bool good = (l >= 0x1p-60f) && (l <= 0x1p100f);        // false for NaN, too
        inv = good ? 1.0f / l : 0.f;
        if (pe_in && pe_listed && !good) p.redo[pe_item] = 1;
      }
      long long te0 = FG_CLK();
      tc_fence_after();
      uint32_t o[kOCols];
      if constexpr (kOCols >= 32) {
#pragma unroll
        for (int cc = 0; cc < kOCols / 32; ++cc)
          tmem_ld32(lane_base + kColO + wg * kOCols + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&o[cc * 32]));
      } else {
        tmem_ld16(lane_base + kColO + wg * kOCols, *reinterpret_cast<uint32_t(*)[16]>(&o[0]));
      }
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(PB_O_EMPTY));
      if (pe_in) {
#pragma unroll
        for (int i = 0; i < kOCols / 8; ++i) {
          uint4 v;
          if constexpr (RENORM) {
#pragma unroll
            for (int e = 0; e < 8; ++e) o[8 * i + e] = __float_as_uint(__uint_as_float(o[8 * i + e]) * inv);
          }
          v.x = pack_bf16(__uint_as_float(o[8 * i + 0]), __uint_as_float(o[8 * i + 1]));
          v.y = pack_bf16(__uint_as_float(o[8 * i + 2]), __uint_as_float(o[8 * i + 3]));
          v.z = pack_bf16(__uint_as_float(o[8 * i + 4]), __uint_as_float(o[8 * i + 5]));
          v.w = pack_bf16(__uint_as_float(o[8 * i + 6]), __uint_as_float(o[8 * i + 7]));
          *reinterpret_cast<uint4*>(pe_orow + wg * kOCols + i * 8) = v;
        }
      }
      pe = false;
      t_epiw += FG_CLK() - te0;
    };
    for (int it = 0; ok; ++it) {
      const int lb = it % NLB;
      FG_TW(w_list, ok = mbar_wait(bar(PB_LIST_FULL + lb), (it / NLB) & 1, ab, p.err, 1402));
      if (!ok) break;
      const int n = info[lb].n_steps;
      if (n < 0) break;
      const int bh = info[lb].bh, pair = info[lb].pair, halves = info[lb].halves;
      const int row = pair * 128 + row_in_tile;
      __nv_bfloat16* orow = p.o + (size_t(bh) * p.S + row) * D;
      if (n == 0) {
        if (row < p.S) {
#pragma unroll
          for (int i = 0; i < kOCols / 8; ++i) reinterpret_cast<uint4*>(orow + wg * kOCols)[i] = make_uint4(0, 0, 0, 0);
        }
      } else {
        float t_row = INFINITY;
        long long tp0 = FG_CLK();
        if (row < p.S) {
          const size_t off = size_t(bh) * p.S_pad + row;
          t_row = RENORM ? p.max_q[off] * c : p.max_q[off] * c + log2f(p.denom[off]);
        }
        float sum0 = 0.f, sum1 = 0.f;                    // RENORM: this thread's share of the row sum
#ifdef FG_STATS
        if (t_row == 12345.678f) t_prol += 1;            // keeps the loads inside the timed span
#endif
        t_prol += FG_CLK() - tp0;
        const uint32_t* list = lists + lb * p.list_cap;
        // token-derived lists: the union list is the block's own list, so entry i of it has column mask i
        const unsigned long long* masks =
            TOKEN ? p.kb_mask + (size_t(bh) * p.npairs + pair) * p.list_stride : nullptr;
        for (int j = 0; j < n; ++j, ++s) {
          if ((s & 1) != own) {
            // the other pair's step; an item's first step is a good moment for the pending rows
            if (j == 0 && pe) {
              epilogue();
              if (!ok) break;
            }
            continue;
          }
          const uint32_t e = list[2 * j + kb_sel];
          const int valid_kb = ((e >> (30 + half)) & 1u) ? min(64, p.kv_len - entry_kb(e) * 64) : 0;
          unsigned long long live64 = ~0ull;               // fetched before the wait for the scores
          if (TOKEN && valid_kb > 0) live64 = __ldg(masks + 2 * j + kb_sel);
          const int sbuf = s % kSB;
          FG_TW(w_s, ok = mbar_wait(bar(PB_S_FULL + s % 6), (s / 6) & 1, ab, p.err, 1403));
          if (!ok) break;
          tc_fence_after();
          long long tm0 = FG_CLK();
          // 64 score columns (one key block) in two halves; the probabilities go over the first half
          // of this warpgroup's own score columns, which nobody else touches, and the buffer is
          // refilled only after the P*V product of this step has consumed them
          const uint32_t a = lane_base + kColS + sbuf * 128 + kb_sel * 64;
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            const int valid = max(0, min(32, valid_kb - ch * 32));
            uint32_t pk[16];
            const uint32_t live =
                TOKEN ? uint32_t(live64 >> (32 * ch)) & (valid >= 32 ? 0xffffffffu : ((1u << valid) - 1u)) : 0xffffffffu;
            if (valid > 0 && live != 0u && !(dbg & 4)) {   // warp-uniform
              uint32_t r[32];
              tmem_ld32(a + ch * 32, r);
              tmem_ld_wait();
              if (!TOKEN || live == 0xffffffffu) ml_probs<32, RENORM && !TSUM>(r, pk, valid, c, t_row, sum0, sum1);
              else ml_probs_masked<RENORM && !TSUM>(r, pk, live, c, t_row, sum0, sum1);
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) pk[i] = 0u;
            }
            tmem_st16(a + ch * 16, pk);
          }
          t_math += FG_CLK() - tm0;
          long long ts0 = FG_CLK();
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(PB_P_FULL + (s % 6) * 2));
          t_st += FG_CLK() - ts0;
          if (pe) {                                      // pending rows of the previous item
            epilogue();
            if (!ok) break;
          }
        }
        if (!ok) break;
        if (pe) epilogue();                              // (only when the loop above did not run it)
        if (!ok) break;
        if constexpr (RENORM) {
          if constexpr (!TSUM) {
            // A buffer of four items: a warpgroup can be at most three steps (so three items) ahead of the
            // P*V issuer, which starts the item after next only once every warp has read this one's sums.
            rowsum[(u & 3) * (Cfg::kSmWGs * 128) + wg * 128 + row_in_tile] = sum0 + sum1;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(PB_L_FULL + (u & 3)));
          }
          pe_u = u;
          pe_item = bh * p.npairs + pair;
          pe_listed = (halves >> half) & 1;
        }
        pe = true;
        pe_par = u & 1;
        pe_orow = orow;
        pe_in = row < p.S;
        ++u;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(PB_LIST_EMPTY + lb));
    }
    if (ok && pe) epilogue();
    if (p.stats && wg < 2 && (warp & 3) == 0 && lane == 0) {
      long long* st_ = p.stats + size_t(blockIdx.x) * 32 + 16 + 8 * wg;
      st_[0] = FG_CLK() - t_start; st_[1] = w_s; st_[2] = w_list; st_[3] = w_epi; st_[4] = t_math;
      st_[5] = w_pe; st_[6] = t_prol; st_[7] = t_epiw;
      if (wg == 1) { st_[2] = t_ld; st_[3] = t_st; }
    }
  } else {
    reg_dealloc<Cfg::kRegsService>();                    // padding warps: idle
  }
  tc_fence_before();
  __syncthreads();
  if (warp == Cfg::kWarpProdK) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

// Queue order.  Heads are taken in groups of `group_heads` consecutive (batch, head) units (few
// enough that the K/V of one group stays in L2, many enough that a group has several items per SM);
// inside a group all items are ordered longest first, so that the long items start early and the
// tail of the launch is made of short ones.  order[] receives global item ids (unit * n_items + item).
// An item is `subs` sub-items that are walked side by side (the longest counts), a sub-item is the
// union of `elems` consecutive lists (their lengths are added): the persistent block kernel has
// subs 1 / elems 2, the two-slot block kernel 2 / 2, the token-list kernel 2 / 1.  Lengths are
// bucketed as (length >> shift).  Counting sort; ties land in arbitrary order, which only affects
// scheduling.  grid (number of groups), 256 threads.  Block 0 also clears the queue counter; with `redo`
// every block clears the re-run flags of its items.
__global__ void __launch_bounds__(256)
sparse_order_kernel(const int* __restrict__ kb_cnt, int* __restrict__ order, int* __restrict__ queue, int nqb,
                    int npairs, int n_units, int group_heads, int subs = 1, int elems = 2, int shift = 0,
                    int* __restrict__ redo = nullptr) {
  constexpr int kBuckets = 1024;
  __shared__ int hist[kBuckets];
  __shared__ int part[256];
  const int tid = threadIdx.x;
  // the last group takes whatever is left (the launcher may make it larger than the others)
  const int u0 = blockIdx.x * group_heads, u1 = (blockIdx.x == gridDim.x - 1) ? n_units : min(n_units, u0 + group_heads);
  const int n = (u1 - u0) * npairs;
  if (blockIdx.x == 0 && tid == 0) *queue = 0;
  if (redo)
    for (int i = tid; i < n; i += 256) redo[size_t(u0) * npairs + i] = 0;
  for (int i = tid; i < kBuckets; i += 256) hist[i] = 0;
  __syncthreads();
  auto length_of = [&](int i) {
    const int unit = u0 + i / npairs, it = i % npairs;
    int len = 0;
    for (int j = 0; j < subs; ++j) {
      int sum = 0;
      for (int e = 0; e < elems; ++e) {
        const int qb = (it * subs + j) * elems + e;
        if (qb < nqb) sum += max(kb_cnt[size_t(unit) * nqb + qb], 0);
      }
      len = max(len, sum);
    }
    return min(len >> shift, kBuckets - 1);
  };
  for (int i = tid; i < n; i += 256) atomicAdd(&hist[length_of(i)], 1);
  __syncthreads();
  // start[b] = number of items in longer buckets; thread t owns buckets (1023 - 4t) .. (1020 - 4t)
  int local[4], sum = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    local[j] = hist[kBuckets - 1 - (4 * tid + j)];
    sum += local[j];
  }
  part[tid] = sum;
  __syncthreads();
  for (int off = 1; off < 256; off <<= 1) {
    const int v = (tid >= off) ? part[tid - off] : 0;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  int run = part[tid] - sum;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    hist[kBuckets - 1 - (4 * tid + j)] = run;
    run += local[j];
  }
  __syncthreads();
  for (int i = tid; i < n; i += 256) {
    const int pos = atomicAdd(&hist[length_of(i)], 1);
    order[size_t(u0) * npairs + pos] = u0 * npairs + i;
  }
}

}  // namespace fg
