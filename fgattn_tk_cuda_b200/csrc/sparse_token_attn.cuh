// Sparse attention over key-TOKEN lists at the reference granularity (128-row query blocks).
// For each query block the listed K/V rows are gathered 128 at a time into swizzled shared-memory
// tiles (16-byte cp.async per chunk, whole rows per warp-wide copy, fifteen gather warps), and the flash-attention step over the
// gathered keys runs on tcgen05 with an online (renormalising) softmax.  A CTA runs two query
// blocks ("slots") against one tensor pipe; their K/V tiles share one ring in consumption order.
// List entries >= the number of key rows, and slots past the count, are masked out.
#pragma once
#include "sm100_ptx.cuh"
#include "softmax_steps.cuh"

namespace fg {

struct TokenParams {
  __nv_bfloat16* o;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const int* kv_idx;        // [BH, nqb128, mask_stride]
  const int* kv_cnt;        // [BH, nqb128]
  int* err;
  int S, S_kv, nqb, mask_stride;   // query rows, rows of k / v per head
  // thread block i works on item order[i] (or i when order is null); item = unit * pairs + pair of
  // 128-row query blocks
  const int* order;
  int pairs;
  // optional [BH, nqb]: query blocks with route != 0 are computed by the block-route kernel and are left
  // alone here (no loads, no stores)
  const int* route;
  float scale_log2;
};

template <int D>
struct TokenCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kStages = (D == 128) ? 4 : 8;
  static constexpr int kGatherWarps = 15;                 // the copies a warp can keep in flight are the limit
  static constexpr int kGatherThreads = 32 * kGatherWarps;
  static constexpr int kThreads = 32 * (8 + 1 + kGatherWarps);   // 8 softmax warps, the UMMA issuer, the gather warps
  static constexpr int kOffQ = 0;
  static constexpr int kOffRing = 2 * kTileBytes;
  static constexpr int kOffBar = kOffRing + kStages * kTileBytes;
  static constexpr int kSmemBytes = kOffBar + 1024 + 1024;
};

enum : int { TB_Q_FULL = 0, TB_FULL = 1, TB_EMPTY = 9, TB_S_FULL = 17, TB_P_FULL = 19, TB_O_FULL = 21, TB_COUNT = 23 };

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }


// Online softmax over one 128-column score tile in two passes of 32-column quarters, so that a thread
// never holds more than 32 scores: pass 1 finds the row maximum over the live columns (colmask: 4
// words, bit set = live), pass 2 re-reads the scores, writes the bf16 probabilities over the first 64
// columns of the same tile and adds up the row sum.  The accumulator row is rescaled lazily (2^8 rule).
template <int D>
__device__ __forceinline__ void softmax_online_quarters(uint32_t s_addr, uint32_t o_addr, float c, bool first,
                                                        OnlineState& st, const uint32_t (&colmask)[4]) {
  float mx = -INFINITY;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t mw = colmask[w];
    if (mw == 0u) continue;                              // warp-uniform: no live column in this quarter
    uint32_t r[32];
    tmem_ld32(s_addr + w * 32, r);
    tmem_ld_wait();
    float c0 = -INFINITY, c1 = -INFINITY, c2 = -INFINITY, c3 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      c0 = fmaxf(c0, ((mw >> i) & 1u) ? __uint_as_float(r[i]) : -INFINITY);
      c1 = fmaxf(c1, ((mw >> (i + 1)) & 1u) ? __uint_as_float(r[i + 1]) : -INFINITY);
      c2 = fmaxf(c2, ((mw >> (i + 2)) & 1u) ? __uint_as_float(r[i + 2]) : -INFINITY);
      c3 = fmaxf(c3, ((mw >> (i + 3)) & 1u) ? __uint_as_float(r[i + 3]) : -INFINITY);
    }
    mx = fmaxf(mx, fmaxf(fmaxf(c0, c1), fmaxf(c2, c3)));
  }
  st.m_true = fmaxf(st.m_true, mx);
  const float ms = mx * c;
  const bool grow = ms > st.m_used + 8.0f;
  if (__any_sync(0xffffffffu, grow)) {
    const float alpha = grow ? ex2(st.m_used - ms) : 1.0f;
    if (grow) st.m_used = ms;
    st.l *= alpha;
    if (!first) {
#pragma unroll
      for (int cc = 0; cc < D / 32; ++cc) {
        uint32_t o[32];
        tmem_ld32(o_addr + cc * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st32(o_addr + cc * 32, o);
      }
    }
  }
  const float neg_m = -st.m_used;
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t mw = colmask[w];
    uint32_t pk[16];
    if (mw != 0u) {
      uint32_t r[32];
      tmem_ld32(s_addr + w * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float p0 = ex2(fmaf(__uint_as_float(r[i]), c, neg_m));
        float p1 = ex2(fmaf(__uint_as_float(r[i + 1]), c, neg_m));
        if (!((mw >> i) & 1u)) p0 = 0.f;
        if (!((mw >> (i + 1)) & 1u)) p1 = 0.f;
        sum0 += p0;
        sum1 += p1;
        pk[i >> 1] = pack_bf16(p0, p1);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) pk[i] = 0u;
    }
    // quarter w's probabilities land on columns 16w .. 16w+15, all of them already consumed
    tmem_st16(s_addr + w * 16, pk);
  }
  st.l += sum0 + sum1;
  tmem_st_wait();
}

template <int D>
__global__ void __launch_bounds__(TokenCfg<D>::kThreads, 1)
sparse_token_attn_kernel(const __grid_constant__ CUtensorMap mq, const TokenParams p) {
  using Cfg = TokenCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + Cfg::kOffBar;
  auto bar = [&](int i) -> uint32_t { return bars + 8u * uint32_t(i); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kOffBar + 8 * TB_COUNT);
  AbortState* ab = reinterpret_cast<AbortState*>(smem + Cfg::kOffBar + 8 * TB_COUNT + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int item = p.order ? p.order[blockIdx.x] : int(blockIdx.x);
  const int bh = item / p.pairs;
  const int q0 = (item - bh * p.pairs) * 256;
  bool skip[2] = {false, false};
  if (p.route) {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int qb = (q0 >> 7) + t;
      skip[t] = qb >= p.nqb || p.route[size_t(bh) * p.nqb + qb] != 0;
    }
    if (skip[0] && skip[1]) return;                      // CTA-uniform, before any set-up
  }

  if (tid == 0) {
    ab->flag = 0;
    mbar_init(bar(TB_Q_FULL), 1);
    for (int s = 0; s < 8; ++s) {
      mbar_init(bar(TB_FULL + s), Cfg::kGatherThreads);
      mbar_init(bar(TB_EMPTY + s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar(TB_S_FULL + t), 1);
      mbar_init(bar(TB_P_FULL + t), 128);
      mbar_init(bar(TB_O_FULL + t), 1);
    }
    mbar_fence_init();
  }
  if (warp == 8) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // per-slot list and number of 128-token steps
  int cnt[2], nst[2];
  const int* lst[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qb = (q0 >> 7) + t;
    cnt[t] = 0;
    lst[t] = p.kv_idx;
    if (qb < p.nqb && !skip[t]) {
      cnt[t] = max(0, min(p.kv_cnt[size_t(bh) * p.nqb + qb], p.mask_stride));
      lst[t] = p.kv_idx + (size_t(bh) * p.nqb + qb) * p.mask_stride;
    }
    nst[t] = (cnt[t] + 127) >> 7;
  }
  const int n_max = max(nst[0], nst[1]);

  if (warp == 8 || warp >= 10) {
    // ------------------------------------------------------------------ gather producers
    reg_dealloc<40>();
    if (warp == 8 && lane == 0) {
      tma_prefetch_desc(&mq);
      mbar_arrive_expect_tx(bar(TB_Q_FULL), 2 * Cfg::kTileBytes);
      for (int t = 0; t < 2; ++t)
        for (int h = 0; h < Cfg::kHalves; ++h)
          tma_load_3d(sbase + Cfg::kOffQ + t * Cfg::kTileBytes + h * 16384, &mq, bar(TB_Q_FULL), h * 64, q0 + t * 128,
                      bh);
    }
    __syncwarp();
    const int gw = (warp == 8) ? 0 : warp - 9;                         // gather warp 0..14
    constexpr int kChunksPerRow = D / 8;                               // 16-byte chunks per row
    constexpr int kRowsPerInstr = 32 / kChunksPerRow;                  // rows one warp-wide copy covers
    // rows of a 128-token tile are dealt to the fifteen gather warps in contiguous runs of 2 x 12 + 13 x 8;
    // a lane keeps the token id of run row `lane` (and of `lane + 32` for runs longer than a warp)
    const int row0 = (gw < 2) ? gw * 12 : 24 + (gw - 2) * 8, nrows = (gw < 2) ? 12 : 8;
    const int sub = lane / kChunksPerRow, ch = lane % kChunksPerRow;
    int idx = 0;
    bool ok = true;
    int pending_stage = -1;                                            // tile whose copies are in flight
    int tokA[2] = {0, 0}, tokB[2] = {0, 0};                            // token ids of the slot's current step
    auto load_tokens = [&](int t, int j) {
      const int pa = j * 128 + row0 + lane, pb = pa + 32;
      int a = (pa < cnt[t]) ? lst[t][pa] : 0;
      int b = (lane + 32 < nrows && pb < cnt[t]) ? lst[t][pb] : 0;
      if (a < 0 || a >= p.S_kv) a = 0;                                    // masked column: any finite row will do
      if (b < 0 || b >= p.S_kv) b = 0;
      tokA[t] = a;
      tokB[t] = b;
    };
    // Each copy instruction moves whole rows: 16 (D = 128) or 8 (D = 64) neighbouring lanes fetch the
    // consecutive 16-byte chunks of one row, so a warp-wide copy asks L2 for full 128-byte lines
    // instead of 32 separate sectors.
    auto gather_tile = [&](const __nv_bfloat16* base, int t) {
      const int st = idx % Cfg::kStages, f = idx / Cfg::kStages;
      if (f > 0) ok = mbar_wait(bar(TB_EMPTY + st), (f - 1) & 1, ab, p.err, 701);
      if (!ok) return;
      const uint32_t dst = sbase + Cfg::kOffRing + st * Cfg::kTileBytes + (ch >> 3) * 16384;
      const __nv_bfloat16* src0 = base + size_t(bh) * p.S_kv * D + ch * 8;
      for (int r = 0; r < nrows; r += kRowsPerInstr) {                 // nrows is a multiple of 4
        const int lr = r + sub;                                        // run row of this lane
        const int ta = __shfl_sync(0xffffffffu, tokA[t], lr & 31), tb = __shfl_sync(0xffffffffu, tokB[t], lr & 31);
        const int tok = (lr < 32) ? ta : tb;
        cp_async_16(dst + sw128_offset(row0 + lr, ch & 7), src0 + size_t(tok) * D);
      }
      cp_async_commit();
      if (pending_stage >= 0) {
        cp_async_wait<1>();                                            // the previous tile has landed
        fence_proxy_async_smem();
        mbar_arrive(bar(TB_FULL + pending_stage));
      }
      pending_stage = st;
      ++idx;
    };
    // order: K(0,0) K(1,0), then per step V(t,j) K(t,j+1); the ids of step j serve K(t,j) and V(t,j)
    if (nst[0] > 0) { load_tokens(0, 0); gather_tile(p.k, 0); }
    if (nst[1] > 0 && ok) { load_tokens(1, 0); gather_tile(p.k, 1); }
    for (int j = 0; j < n_max && ok; ++j) {
      for (int t = 0; t < 2 && ok; ++t) {
        if (j < nst[t]) {
          gather_tile(p.v, t);
          if (ok && j + 1 < nst[t]) {
            load_tokens(t, j + 1);
            gather_tile(p.k, t);
          }
        }
      }
    }
    cp_async_wait<0>();
    if (ok && pending_stage >= 0) {
      fence_proxy_async_smem();
      mbar_arrive(bar(TB_FULL + pending_stage));
    }
    if (!ok && warp == 8 && lane == 0) mbar_wait_brief(bar(TB_Q_FULL), 0);
  } else if (warp == 9) {
    // ------------------------------------------------------------------ UMMA issuer
    reg_dealloc<40>();
    {   // whole warp, uniform control flow; single instructions go through an elected lane
      const uint32_t idesc_qk = umma_idesc_bf16(128, 128, false);
      const uint32_t idesc_pv = umma_idesc_bf16(128, D, true);
      int idx = 0;
      bool ok = mbar_wait_warp(bar(TB_Q_FULL), 0, ab, p.err, 801);
      auto qk = [&](int t) {
        const int st = idx % Cfg::kStages;
        ok = mbar_wait_warp(bar(TB_FULL + st), (idx / Cfg::kStages) & 1, ab, p.err, 802);
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
          umma_commit(bar(TB_S_FULL + t));
          umma_commit(bar(TB_EMPTY + st));
        }
        __syncwarp();
        ++idx;
      };
      auto pv = [&](int t, int j) {
        const int st = idx % Cfg::kStages;
        ok = mbar_wait_warp(bar(TB_FULL + st), (idx / Cfg::kStages) & 1, ab, p.err, 803);
        if (ok) ok = mbar_wait_warp(bar(TB_P_FULL + t), j & 1, ab, p.err, 804);
        if (!ok) return;
        tc_fence_after();
        const uint32_t va = sbase + Cfg::kOffRing + st * Cfg::kTileBytes;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ts(tmem + 256 + t * 128, tmem + t * 128 + ks * 8, umma_smem_desc_sw128(va + ks * 2048, 16384, 1024),
                    idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
          umma_commit(bar(TB_EMPTY + st));
        }
        __syncwarp();
        ++idx;
      };
      if (ok && nst[0] > 0) qk(0);
      if (ok && nst[1] > 0) qk(1);
      for (int j = 0; j < n_max && ok; ++j) {
        for (int t = 0; t < 2 && ok; ++t) {
          if (j < nst[t]) {
            pv(t, j);
            if (!ok) break;
            if (j + 1 < nst[t]) qk(t);
            else umma_commit_elect(bar(TB_O_FULL + t));
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    reg_alloc<152>();
    const int t = warp >> 2, wq = warp & 3;
    const int row = q0 + t * 128 + wq * 32 + lane;
    const uint32_t lane_base = tmem + (uint32_t(wq * 32) << 16);
    const uint32_t s_addr = lane_base + t * 128, o_addr = lane_base + 256 + t * 128;
    OnlineState st;
    online_init(st);
    bool ok = true;
    // which of a step's 128 gathered columns are real keys; fetched one step ahead so that the list
    // loads overlap the products of the current step instead of opening every step with a global-memory
    // round trip
    uint32_t live[4];
    auto fetch_live = [&](int j) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const int pos = j * 128 + w * 32 + lane;
        const int tok = (j < nst[t] && pos < cnt[t]) ? lst[t][pos] : -1;
        live[w] = __ballot_sync(0xffffffffu, tok >= 0 && tok < p.S_kv);
      }
    };
    fetch_live(0);
    for (int j = 0; j < nst[t]; ++j) {
      ok = mbar_wait(bar(TB_S_FULL + t), j & 1, ab, p.err, 901);
      if (!ok) break;
      tc_fence_after();
      softmax_online_quarters<D>(s_addr, o_addr, p.scale_log2, j == 0, st, live);
      tc_fence_before();
      mbar_arrive(bar(TB_P_FULL + t));
      fetch_live(j + 1);
    }
    __nv_bfloat16* orow = p.o + (size_t(bh) * p.S + row) * D;
    if (skip[t]) {
      // another kernel owns these rows
    } else if (nst[t] == 0) {
      if (row < p.S) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) reinterpret_cast<uint4*>(orow)[i] = make_uint4(0, 0, 0, 0);
      }
    } else if (ok) {
      ok = mbar_wait(bar(TB_O_FULL + t), 0, ab, p.err, 902);
      if (ok) {
        tc_fence_after();
        store_o_row<D>(o_addr, orow, st.l > 0.f ? 1.0f / st.l : 0.f, row < p.S);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace fg
