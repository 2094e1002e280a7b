// Per-thread softmax steps shared by the dense and the block-sparse kernels.  A thread owns one
// query row (one TMEM lane) and sees one 128-key score tile as two 64-key halves; `valid0` and
// `valid1` give the number of live columns in each half (0..64), the rest is masked out.
#pragma once
#include "sm100_ptx.cuh"

namespace fg {

struct OnlineState {
  float m_used;   // running maximum in the scaled log2 domain (s * c); may lag the true one by < 8
  float m_true;   // exact running raw maximum
  float l;        // running denominator relative to m_used
};

// exponent (log2 domain, relative to the running maximum) below which a whole 32-column quarter
// is treated as zero by softmax_online_step
constexpr float kSkipLog2 = -40.0f;

__device__ __forceinline__ void online_init(OnlineState& st) {
  st.m_used = -1.0e30f;
  st.m_true = -INFINITY;
  st.l = 0.f;
}

// Online softmax over one score tile.
//   s_addr : TMEM address (lane already folded in) of the 128 fp32 score columns
//   p_addr : where the 64 packed-bf16 probability columns go (WRITE_P)
//   o_addr : the row's D fp32 output accumulator columns (rescaled in place when the maximum grows)
// Returns the raw maxima of the two 64-key halves through mx0 / mx1.
//   colmask: optional 128-bit column mask (4 words, bit set = live column) applied on top
//   POLY   : of every eight pairs of columns, how many compute their exponentials on the FMA pipe
//            (ex2_poly2) instead of the MUFU, which is the busiest unit of these kernels.  Measured with
//            L2 flushed between calls: 2 of 8 with P*V (C2 0.245 -> 0.232 ms, C4 5.33 -> 5.11 ms, C3 within
//            2 %), 3 of 8 for the max / denominator pass (C3 2.49 -> 2.38 ms, C4 3.94 -> 3.45 ms); 4 of 8 is
//            slower again: the polynomial costs ten issue slots per pair against two
template <int D, bool WRITE_P, int POLY = (WRITE_P ? 2 : 3)>
__device__ __forceinline__ void softmax_online_step(uint32_t s_addr, uint32_t p_addr, uint32_t o_addr, int valid0,
                                                    int valid1, float c, bool first, OnlineState& st, float& mx0,
                                                    float& mx1, const uint32_t* colmask = nullptr) {
  uint32_t r[128];
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) tmem_ld32(s_addr + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[cc * 32]));
  tmem_ld_wait();
  if (valid0 < 64 || valid1 < 64) {
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      if (i >= valid0) r[i] = __float_as_uint(-INFINITY);
      if (i >= valid1) r[64 + i] = __float_as_uint(-INFINITY);
    }
  }
  if (colmask != nullptr) {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t mw = colmask[w];
      if (mw != 0xffffffffu) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (!((mw >> i) & 1u)) r[w * 32 + i] = __float_as_uint(-INFINITY);
      }
    }
  }
  // maxima of the four 32-column quarters (four independent chains)
  float qmax[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) qmax[w] = __uint_as_float(r[w * 32]);
#pragma unroll
  for (int i = 1; i < 32; ++i) {
#pragma unroll
    for (int w = 0; w < 4; ++w) qmax[w] = fmaxf(qmax[w], __uint_as_float(r[w * 32 + i]));
  }
  mx0 = fmaxf(qmax[0], qmax[1]);
  mx1 = fmaxf(qmax[2], qmax[3]);
  const float mx = fmaxf(mx0, mx1);
  st.m_true = fmaxf(st.m_true, mx);
  const float ms = mx * c;
  const bool grow = ms > st.m_used + 8.0f;
  if (__any_sync(0xffffffffu, grow)) {
    const float alpha = grow ? ex2(st.m_used - ms) : 1.0f;
    if (grow) st.m_used = ms;
    st.l *= alpha;
    if (WRITE_P && !first) {
      // the accumulator is quiescent: the commit that published this score tile also covers the
      // previous P*V product of the same query tile
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
  float sum0 = 0.f, sum1 = 0.f;
  const float neg_m = -st.m_used;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    // A quarter whose largest exponent is below kSkipLog2 for every row of the warp contributes
    // less than 2^-40 per entry relative to the running maximum -- under one fp32 ulp of the
    // denominator and of the output even summed over a whole row -- so its exponentials are
    // skipped and its probabilities are exact zeros.
    const bool skip = __all_sync(0xffffffffu, fmaf(qmax[w], c, neg_m) < kSkipLog2);
    if (skip) {
      if (WRITE_P) {
#pragma unroll
        for (int i = 0; i < 16; ++i) r[w * 16 + i] = 0u;
      }
      continue;
    }
#pragma unroll
    for (int i = w * 32; i < w * 32 + 32; i += 2) {
      float p0, p1;
      if constexpr (POLY > 0) {
        // packed scale-and-shift; the pairs that take the FMA-pipe exponential are spread evenly
        const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), f2_pack(c, c),
                                   f2_pack(neg_m, neg_m));
        if ((((i >> 1) & 7) * POLY) % 8 < POLY) {
          ex2_poly2(x2, p0, p1);
        } else {
          float x0, x1;
          f2_unpack(x2, x0, x1);
          p0 = ex2(x0);
          p1 = ex2(x1);
        }
      } else {
        p0 = ex2(fmaf(__uint_as_float(r[i]), c, neg_m));
        p1 = ex2(fmaf(__uint_as_float(r[i + 1]), c, neg_m));
      }
      sum0 += p0;
      sum1 += p1;
      if (WRITE_P) r[i >> 1] = pack_bf16(p0, p1);
    }
  }
  st.l += sum0 + sum1;
  if (WRITE_P) {
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) tmem_st16(p_addr + cc * 16, *reinterpret_cast<uint32_t(*)[16]>(&r[cc * 16]));
    tmem_st_wait();
  }
}

// Write one row of the fp32 accumulator (D columns at o_addr) as bf16, scaled by `inv`.
template <int D>
__device__ __forceinline__ void store_o_row(uint32_t o_addr, __nv_bfloat16* orow, float inv, bool in_range) {
#pragma unroll
  for (int cc = 0; cc < D / 32; ++cc) {
    uint32_t o[32];
    tmem_ld32(o_addr + cc * 32, o);
    tmem_ld_wait();
    if (in_range) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 v;
        v.x = pack_bf16(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
        v.y = pack_bf16(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
        v.z = pack_bf16(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
        v.w = pack_bf16(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
        *reinterpret_cast<uint4*>(orow + cc * 32 + i * 8) = v;
      }
    }
  }
}

}  // namespace fg
