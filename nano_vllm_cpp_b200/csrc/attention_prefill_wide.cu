// Prompt attention for layers whose keys and values differ in size and whose window keeps the sequence's first
// tokens: bfloat16 rows of any mix of portions (single rows too) against paged keys and values, on the tensor cores
// (m16n8k16 bf16 MMAs, float32 accumulators, online softmax in float32 registers).
//
// What it adds to attention_prefill.cu:
//   * a query head of KS * D elements whose score with position j is its product with the keys of kv heads
//     0 .. KS - 1 at j side by side (scores that are mixed across heads are linear in the queries, so the mixing is
//     done on the queries and a mixed head reads every kv head's key); KS = 1: the head's own kv head;
//   * values of Dv elements from the head's own value head;
//   * `keep_first`: behind the window the first so many positions stay visible.  A tile of rows walks two runs of
//     key tiles: the kept positions that lie before the first key any of its rows sees through the window, then
//     the window's keys up to the tile's last row; the mask is applied per element (j <= p and (p - j < window or
//     j < keep_first)), so both runs may hold keys that only some rows see;
//   * a learned sink per head in the softmax's denominator (a score without key and value, not scaled);
//   * an output in float32 where a pass of its own follows (values that were turned by their positions when they
//     were written have their sums turned back by the row's position).
// The softmax weights enter the product with the values as three bfloat16 terms, all bits of the float.
//
// grid = (row tiles, query heads); a CTA takes BM consecutive rows of one request and one query head, each warp 16
// rows; keys and values come page by page into shared memory in tiles of BN keys with cp.async, double-buffered.
//
// The NARROW form is for entries of at most 16 rows (decoded tokens above all): a CTA takes one such entry and one
// query head, all its warps work on the same 16 rows, and each warp takes 16 of a tile's BN keys with a running
// maximum, sum and output of its own; the warps' results are merged through shared memory at the end.  With
// grid.z > 1 the CTAs of one entry and head share out the key tiles, write (output, maximum, sum) per share to a
// scratch array, and `wide_combine_kernel` merges the shares, adds the sink and writes the rows.
//
// The HEADS form is the narrow form for entries of one row whose query heads all read the same keys (KS = Hk: mixed
// heads, or one kv head) and number at most 16: the 16 rows of a CTA's tile are the row's query heads, so the keys
// are read once for all heads.  The values of all Hv value heads come with each key tile; the weights of the
// heads of one value head at a time (the other rows set to zero) are multiplied with that head's values into the
// same accumulators.
#include "common.cuh"

#include <limits.h>
#include <stdlib.h>

namespace {

struct WideArgs {
  const bf16* q;            // [T, Hq, KS * D]
  const bf16* kc;           // [blocks, Hk, page, D]
  const bf16* vc;           // [blocks, Hv, page, Dv]
  const int* block_table;
  const int* cu_rows;       // [S + 1]
  const int* entry_pos0;    // [S]
  const float* sinks;       // [Hq] or null
  void* out;                // [T, Hq, Dv] bfloat16 or float32
  float* parts;             // NARROW with grid.z > 1: [T, Hq, grid.z, Dv + 2] (output, maximum, sum)
  float scale_log2;         // scale * log2(e)
  int out_f32;
  int S, max_blocks, window, keep_first, Hq, Hk, Hv, D, KS, Dv, page, min_rows, max_rows;
};

__device__ __forceinline__ uint32_t sm_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void copy16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sm_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldm4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldm4_t(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t two_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

constexpr int WIDE_TERMS = 3;

// KDP: key length (KS * D) rounded up to 64, 128, 256 or 512; DVP: value length rounded up to 64, 128 or 256.
// FORM 0: tiles of BM rows; 1: narrow; 2: heads as rows.
template <int KDP, int DVP, int BM, int BN, int FORM>
__global__ void __launch_bounds__(BM * 2, 1) attention_prefill_wide_kernel(WideArgs a) {
  constexpr bool NARROW = FORM != 0, HEADS = FORM == 2;
  constexpr int THREADS = BM * 2;
  constexpr int QR = NARROW ? 16 : BM;             // query rows of a CTA
  constexpr int NSUB = NARROW ? 1 : BN / 16;       // blocks of 16 keys that a warp takes of a tile
  static_assert(!NARROW || BM == BN, "narrow form: one block of 16 keys per warp");
  constexpr int LDK = KDP + 8, LDV = DVP + 8;      // row strides (elements): 16 bytes of padding against bank conflicts
  extern __shared__ __align__(16) uint8_t wide_smem[];
  bf16* Qs = (bf16*)wide_smem;                     // [BM][LDK]
  bf16* Ks = Qs + QR * LDK;                        // [2][BN][LDK]
  bf16* Vs = Ks + 2 * BN * LDK;                    // [2][BN][ldv]
  __shared__ int tile_info[3];                     // entry, first row (batch), rows

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int h = blockIdx.y;
  const int D = a.D, KD = a.KS * a.D, Dv = a.Dv;
  const int kh0 = a.KS > 1 ? 0 : h / (a.Hq / a.Hk);
  const int vh = h / (a.Hq / a.Hv);
  const int ldv = HEADS ? a.Hv * a.Dv + 8 : LDV;   // the HEADS form keeps every value head's values of a key side by side
  const int kchunks = D / 8, vchunks = Dv / 8;

  if (tid == 0) {                                  // which (entry, tile of BM rows) is this CTA's?  Late tiles first.
    int left = (int)(gridDim.x - 1 - blockIdx.x), e = 0, found = -1;
    for (; e < a.S; ++e) {
      const int n = a.cu_rows[e + 1] - a.cu_rows[e];
      const int tiles = n >= a.min_rows && n <= a.max_rows ? (n + QR - 1) / QR : 0;
      if (left < tiles) { found = e; break; }
      left -= tiles;
    }
    tile_info[0] = found;
    if (found >= 0) {
      tile_info[1] = a.cu_rows[found] + left * QR;
      tile_info[2] = min(QR, a.cu_rows[found + 1] - tile_info[1]);
    }
  }
  __syncthreads();
  const int e = tile_info[0];
  if (e < 0) return;
  const int row0 = tile_info[1], nrows = tile_info[2];
  const int pos0 = a.entry_pos0[e] + (row0 - a.cu_rows[e]);      // position of the tile's first row
  const int hi = pos0 + nrows;                                   // keys [.., hi) exist for this tile
  const int lo = a.window > 0 ? max(0, pos0 + 1 - a.window) : 0; // first key any row sees through the window
  const int kv0 = lo / 16 * 16;
  const int keep = a.window > 0 ? a.keep_first : 0;
  const int endA = min(keep, kv0);                               // kept positions before the window's run
  const int nA = (endA + BN - 1) / BN, nB = (hi - kv0 + BN - 1) / BN;
  const int n_tiles = nA + nB;
  // this CTA's share of the key tiles (all of them unless the narrow form runs with grid.z > 1)
  const int t_first = (int)((long long)n_tiles * blockIdx.z / gridDim.z);
  const int t_end = (int)((long long)n_tiles * (blockIdx.z + 1) / gridDim.z);
  const int* bt = a.block_table + (size_t)e * a.max_blocks;

  // ---- Q tile -> shared memory (rows beyond nrows are zero)
  {
    const int qchunks = KD / 8;
    for (int c = tid; c < QR * qchunks; c += THREADS) {
      const int r = c / qchunks, ch = c - r * qchunks;
      bf16* dst = Qs + r * LDK + ch * 8;
      if (HEADS ? r < a.Hq : r < nrows) copy16(dst, a.q + ((size_t)(row0 + (HEADS ? 0 : r)) * a.Hq + (HEADS ? r : h)) * KD + ch * 8);
      else *(uint4*)dst = make_uint4(0, 0, 0, 0);
    }
  }
  // Eight neighbouring threads bring one key position: its keys (of KS kv heads) and its value, 16 bytes a copy; the
  // page and the place in it are looked up once per position.
  auto load_kv = [&](int tile, int buf) {
    const int j0 = tile < nA ? tile * BN : kv0 + (tile - nA) * BN;
    const int jend = tile < nA ? endA : hi;
    bf16* kd = Ks + buf * BN * LDK;
    bf16* vd = Vs + buf * BN * ldv;
    constexpr int LPR = 8;
    const int sub = tid % LPR;
    for (int r = tid / LPR; r < BN; r += THREADS / LPR) {
      const int j = j0 + r;
      bf16* krow = kd + r * LDK;
      bf16* vrow = vd + r * ldv;
      if (j < jend) {
        const int pg = j / a.page, slot = j - pg * a.page;
        const size_t blk = (size_t)bt[pg];
        for (int kc_i = 0; kc_i < a.KS; ++kc_i) {
          const bf16* src = a.kc + ((blk * a.Hk + kh0 + kc_i) * a.page + slot) * D;
          for (int ch = sub; ch < kchunks; ch += LPR) copy16(krow + kc_i * D + ch * 8, src + ch * 8);
        }
        for (int v = HEADS ? 0 : vh; v < (HEADS ? a.Hv : vh + 1); ++v) {
          const bf16* src = a.vc + ((blk * a.Hv + v) * a.page + slot) * Dv;
          bf16* dst = vrow + (HEADS ? v * Dv : 0);
          for (int ch = sub; ch < vchunks; ch += LPR) copy16(dst + ch * 8, src + ch * 8);
        }
      } else {
        for (int ch = sub; ch < a.KS * kchunks; ch += LPR) *(uint4*)(krow + ch * 8) = make_uint4(0, 0, 0, 0);
        for (int ch = sub; ch < (HEADS ? a.Hv : 1) * vchunks; ch += LPR) *(uint4*)(vrow + ch * 8) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  if (t_first < t_end) load_kv(t_first, 0);
  copy_commit();

  const int g = lane / 4, tq = lane % 4;
  const int rw = NARROW ? 0 : warp;                              // which 16 rows of the tile this warp takes
  const int np0 = NARROW ? warp : 0;                             // and its first block of 16 keys in a key tile
  const int r_lo = rw * 16 + g, r_hi = r_lo + 8;                 // this thread's two rows in the tile
  const int p_lo = HEADS ? pos0 : pos0 + r_lo, p_hi = HEADS ? pos0 : pos0 + r_hi;      // HEADS: one row, its heads
  const bool live_lo = HEADS ? r_lo < a.Hq : r_lo < nrows, live_hi = HEADS ? r_hi < a.Hq : r_hi < nrows;
  const int warp_p_lo = pos0 + rw * 16, warp_p_hi = HEADS ? pos0 : warp_p_lo + 15;
  const int heads_per_v = a.Hq / a.Hv;
  const int v_lo = r_lo / heads_per_v, v_hi = r_hi / heads_per_v;                      // HEADS: the rows' value heads

  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o[DVP / 8][4];
#pragma unroll
  for (int i = 0; i < DVP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int t = t_first; t < t_end; ++t) {
    const int buf = (t - t_first) & 1;
    if (t + 1 < t_end) load_kv(t + 1, buf ^ 1);
    copy_commit();
    copy_wait<1>();                                 // tile t (and Q) have landed
    __syncthreads();
    const bf16* kb = Ks + buf * BN * LDK;
    const bf16* vb = Vs + buf * BN * ldv;
    const bool kept_run = t < nA;
    const int j0 = kept_run ? t * BN : kv0 + (t - nA) * BN;
    const int jend = kept_run ? endA : hi;

    // a warp none of whose rows sees any of the tile's keys only keeps the barriers
    constexpr int KW = NSUB * 16;                   // keys of the tile that this warp takes, from jb0
    const int jb0 = j0 + np0 * 16;
    const bool behind = !kept_run && a.window > 0 && jb0 + KW - 1 <= warp_p_lo - a.window && jb0 >= keep;
    const bool warp_sees = rw * 16 < nrows && jb0 <= warp_p_hi && jb0 < jend && !behind;
    if (warp_sees) {
      // ---- S = Q K^T for this warp's 16 rows x KW keys
      float s[KW / 8][4];
#pragma unroll
      for (int i = 0; i < KW / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 4
      for (int kk = 0; kk < KDP / 16; ++kk) {
        if (kk * 16 < KD) {
          uint32_t qa[4];
          ldm4(sm_u32(Qs + (rw * 16 + (lane % 8) + 8 * ((lane / 8) % 2)) * LDK + kk * 16 + 8 * (lane / 16)), qa);
#pragma unroll
          for (int np = 0; np < NSUB; ++np) {
            uint32_t kf[4];
            ldm4(sm_u32(kb + ((np0 + np) * 16 + (lane % 8) + 8 * (lane / 16)) * LDK + kk * 16 + 8 * ((lane / 8) % 2)), kf);
            mma_bf16(s[2 * np], qa, kf[0], kf[1]);
            mma_bf16(s[2 * np + 1], qa, kf[2], kf[3]);
          }
        }
      }
      // ---- mask (unless every row of the warp sees the whole tile), online softmax
      const bool whole = rw * 16 + 15 < nrows && jb0 + KW <= jend && jb0 + KW - 1 <= warp_p_lo &&
                         (a.window <= 0 || jb0 > warp_p_hi - a.window || jb0 + KW <= keep);
      if (!whole) {
#pragma unroll
        for (int nt = 0; nt < KW / 8; ++nt) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int j = jb0 + nt * 8 + 2 * tq + c;
            const bool in = j < jend;
            const bool see_lo = in && live_lo && j <= p_lo && (a.window <= 0 || j > p_lo - a.window || j < keep);
            const bool see_hi = in && live_hi && j <= p_hi && (a.window <= 0 || j > p_hi - a.window || j < keep);
            if (!see_lo) s[nt][c] = -INFINITY;
            if (!see_hi) s[nt][2 + c] = -INFINITY;
          }
        }
      }
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < KW / 8; ++nt) {
        mx_lo = fmaxf(mx_lo, fmaxf(s[nt][0], s[nt][1]));
        mx_hi = fmaxf(mx_hi, fmaxf(s[nt][2], s[nt][3]));
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      const float ms_lo = mn_lo == -INFINITY ? 0.f : mn_lo * a.scale_log2;
      const float ms_hi = mn_hi == -INFINITY ? 0.f : mn_hi * a.scale_log2;
      const float al_lo = m_lo == -INFINITY ? 0.f : exp2f(m_lo * a.scale_log2 - ms_lo);
      const float al_hi = m_hi == -INFINITY ? 0.f : exp2f(m_hi * a.scale_log2 - ms_hi);
      m_lo = mn_lo;
      m_hi = mn_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < KW / 8; ++nt) {
        s[nt][0] = exp2f(s[nt][0] * a.scale_log2 - ms_lo);
        s[nt][1] = exp2f(s[nt][1] * a.scale_log2 - ms_lo);
        s[nt][2] = exp2f(s[nt][2] * a.scale_log2 - ms_hi);
        s[nt][3] = exp2f(s[nt][3] * a.scale_log2 - ms_hi);
        sum_lo += s[nt][0] + s[nt][1];
        sum_hi += s[nt][2] + s[nt][3];
      }
      l_lo = l_lo * al_lo + sum_lo;                 // per-thread partial sums; lanes are added at the end
      l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < DVP / 8; ++i) {
        o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi;
      }
      // ---- O += P V, the weights as three bfloat16 terms
#pragma unroll
      for (int kb16 = 0; kb16 < NSUB; ++kb16) {
        uint32_t pt[WIDE_TERMS][4];
        {
          float w[8] = {s[2 * kb16][0], s[2 * kb16][1], s[2 * kb16][2], s[2 * kb16][3],
                        s[2 * kb16 + 1][0], s[2 * kb16 + 1][1], s[2 * kb16 + 1][2], s[2 * kb16 + 1][3]};
#pragma unroll
          for (int term = 0; term < WIDE_TERMS; ++term) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const uint32_t pk = two_bf16(w[2 * u], w[2 * u + 1]);
              pt[term][u] = pk;
              if (term + 1 < WIDE_TERMS) {
                w[2 * u] -= __uint_as_float(pk << 16);           // what the rounding left: the next term
                w[2 * u + 1] -= __uint_as_float(pk & 0xffff0000u);
              }
            }
          }
        }
        if constexpr (HEADS) {
          for (int v = 0; v < a.Hv; ++v) {          // the weights of value head v's query heads, the other rows zero
            uint32_t pm[WIDE_TERMS][4];
#pragma unroll
            for (int term = 0; term < WIDE_TERMS; ++term) {
              pm[term][0] = v_lo == v ? pt[term][0] : 0u;
              pm[term][1] = v_hi == v ? pt[term][1] : 0u;
              pm[term][2] = v_lo == v ? pt[term][2] : 0u;
              pm[term][3] = v_hi == v ? pt[term][3] : 0u;
            }
#pragma unroll
            for (int dp = 0; dp < DVP / 16; ++dp) {
              if (dp * 16 < Dv) {
                uint32_t vf[4];
                ldm4_t(sm_u32(vb + ((np0 + kb16) * 16 + (lane % 8) + 8 * ((lane / 8) % 2)) * ldv + v * Dv + dp * 16 + 8 * (lane / 16)), vf);
#pragma unroll
                for (int term = 0; term < WIDE_TERMS; ++term) {
                  mma_bf16(o[2 * dp], pm[term], vf[0], vf[1]);
                  mma_bf16(o[2 * dp + 1], pm[term], vf[2], vf[3]);
                }
              }
            }
          }
        } else {
#pragma unroll
          for (int dp = 0; dp < DVP / 16; ++dp) {
            if (dp * 16 < Dv) {
              uint32_t vf[4];
              ldm4_t(sm_u32(vb + ((np0 + kb16) * 16 + (lane % 8) + 8 * ((lane / 8) % 2)) * LDV + dp * 16 + 8 * (lane / 16)), vf);
#pragma unroll
              for (int term = 0; term < WIDE_TERMS; ++term) {
                mma_bf16(o[2 * dp], pt[term], vf[0], vf[1]);
                mma_bf16(o[2 * dp + 1], pt[term], vf[2], vf[3]);
              }
            }
          }
        }
      }
    }
    __syncthreads();                                // everyone is done with this buffer before it is refilled
  }
  copy_wait<0>();

  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  if constexpr (NARROW) {
    // ---- the warps' results for the same rows are merged: (output, maximum, sum) per warp and row in shared memory
    constexpr int NW = BM / 16, PS = DVP + 2;
    float* mg = (float*)wide_smem;                  // [NW][16][PS]
    __syncthreads();                                // every thread's copies have landed; nobody reads a tile any more
    float* my = mg + (size_t)warp * 16 * PS;
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i) {
      const int d = i * 8 + 2 * tq;
      my[g * PS + d] = o[i][0];
      my[g * PS + d + 1] = o[i][1];
      my[(g + 8) * PS + d] = o[i][2];
      my[(g + 8) * PS + d + 1] = o[i][3];
    }
    if (tq == 0) {
      my[g * PS + DVP] = m_lo;
      my[g * PS + DVP + 1] = l_lo;
      my[(g + 8) * PS + DVP] = m_hi;
      my[(g + 8) * PS + DVP + 1] = l_hi;
    }
    __syncthreads();
    const int n_out = HEADS ? a.Hq : nrows;         // HEADS: tile row r is query head r of the entry's one row
    for (int idx = tid; idx < n_out * Dv; idx += THREADS) {
      const int r = idx / Dv, d = idx - r * Dv;
      const int oh = HEADS ? r : h;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < NW; ++w) M = fmaxf(M, mg[(w * 16 + r) * PS + DVP]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const float* pw = mg + (size_t)(w * 16 + r) * PS;
        const float f = pw[DVP] == -INFINITY ? 0.f : exp2f((pw[DVP] - M) * a.scale_log2);
        L += f * pw[DVP + 1];
        O += f * pw[d];
      }
      const size_t row = (size_t)(row0 + (HEADS ? 0 : r));
      if (gridDim.z > 1) {
        float* pp = a.parts + ((row * a.Hq + oh) * gridDim.z + blockIdx.z) * (size_t)(Dv + 2);
        pp[d] = O;
        if (d == 0) { pp[Dv] = M; pp[Dv + 1] = L; }
      } else {
        if (a.sinks) L += exp2f(a.sinks[oh] * 1.4426950408889634f - (M == -INFINITY ? 0.f : M * a.scale_log2));
        const float v = L > 0.f ? O / L : 0.f;
        const size_t at = (row * a.Hq + oh) * Dv + d;
        if (a.out_f32) ((float*)a.out)[at] = v;
        else ((bf16*)a.out)[at] = __float2bfloat16(v);
      }
    }
    return;
  }
  if (a.sinks) {                                    // relative to the same reference as the sums: exp2(sink - m)
    const float sk = a.sinks[h] * 1.4426950408889634f;
    l_lo += exp2f(sk - (m_lo == -INFINITY ? 0.f : m_lo * a.scale_log2));
    l_hi += exp2f(sk - (m_hi == -INFINITY ? 0.f : m_hi * a.scale_log2));
  }
  const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
  for (int i = 0; i < DVP / 8; ++i) {
    o[i][0] *= inv_lo; o[i][1] *= inv_lo; o[i][2] *= inv_hi; o[i][3] *= inv_hi;
  }
#pragma unroll
  for (int i = 0; i < DVP / 8; ++i) {
    const int d = i * 8 + 2 * tq;
    if (d < Dv) {
      const size_t at_lo = ((size_t)(row0 + r_lo) * a.Hq + h) * Dv + d, at_hi = ((size_t)(row0 + r_hi) * a.Hq + h) * Dv + d;
      if (a.out_f32) {
        if (live_lo) *(float2*)((float*)a.out + at_lo) = make_float2(o[i][0], o[i][1]);
        if (live_hi) *(float2*)((float*)a.out + at_hi) = make_float2(o[i][2], o[i][3]);
      } else {
        if (live_lo) *(uint32_t*)((bf16*)a.out + at_lo) = two_bf16(o[i][0], o[i][1]);
        if (live_hi) *(uint32_t*)((bf16*)a.out + at_hi) = two_bf16(o[i][2], o[i][3]);
      }
    }
  }
}

// The shares of the narrow form's key tiles, merged: one CTA per entry and query head.
__global__ void wide_combine_kernel(WideArgs a, int Z) {
  const int e = blockIdx.x, h = blockIdx.y, Dv = a.Dv;
  const int first = a.cu_rows[e], n = a.cu_rows[e + 1] - first;
  if (n < a.min_rows || n > a.max_rows) return;
  const float sk = a.sinks ? a.sinks[h] * 1.4426950408889634f : 0.f;
  for (int idx = threadIdx.x; idx < n * Dv; idx += blockDim.x) {
    const int r = idx / Dv, d = idx - r * Dv;
    const size_t row = (size_t)(first + r);
    const float* pp = a.parts + ((row * a.Hq + h) * Z) * (size_t)(Dv + 2);
    float M = -INFINITY;
    for (int z = 0; z < Z; ++z) M = fmaxf(M, pp[(size_t)z * (Dv + 2) + Dv]);
    float L = 0.f, O = 0.f;
    for (int z = 0; z < Z; ++z) {
      const float* pz = pp + (size_t)z * (Dv + 2);
      const float f = pz[Dv] == -INFINITY ? 0.f : exp2f((pz[Dv] - M) * a.scale_log2);
      L += f * pz[Dv + 1];
      O += f * pz[d];
    }
    if (a.sinks) L += exp2f(sk - (M == -INFINITY ? 0.f : M * a.scale_log2));
    const float v = L > 0.f ? O / L : 0.f;
    const size_t at = (row * a.Hq + h) * Dv + d;
    if (a.out_f32) ((float*)a.out)[at] = v;
    else ((bf16*)a.out)[at] = __float2bfloat16(v);
  }
}

// Shared memory of a CTA: the query rows, two key tiles, two value tiles (the HEADS form: of all value heads).
size_t wide_smem_bytes(int form, int KDP, int DVP, int BM, int BN, int Hv, int Dv) {
  const size_t ldv = form == 2 ? (size_t)Hv * Dv + 8 : (size_t)DVP + 8;
  return ((size_t)((form ? 16 : BM) + 2 * BN) * (KDP + 8) + (size_t)2 * BN * ldv) * sizeof(bf16);
}

template <int KDP, int DVP, int BM, int BN, int FORM>
int launch_wide(const WideArgs& a, int max_tiles, int splits, cudaStream_t s) {
  const size_t smem = wide_smem_bytes(FORM, KDP, DVP, BM, BN, a.Hv, a.Dv);
  static size_t allowed = 0;
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_wide_kernel<KDP, DVP, BM, BN, FORM>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    allowed = smem;
  }
  const int Z = FORM ? splits : 1;
  attention_prefill_wide_kernel<KDP, DVP, BM, BN, FORM><<<dim3(max_tiles, FORM == 2 ? 1 : a.Hq, Z), BM * 2, smem, s>>>(a);
  if (Z > 1) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    wide_combine_kernel<<<dim3(a.S, a.Hq), 128, 0, s>>>(a, Z);
  }
  NV_RETURN_LAST();
}

template <int KDP, int BM, int BN, int FORM>
int launch_wide_v(const WideArgs& a, int max_tiles, int splits, cudaStream_t s) {
  if (a.Dv <= 64) return launch_wide<KDP, 64, BM, BN, FORM>(a, max_tiles, splits, s);
  if (a.Dv <= 128) return launch_wide<KDP, 128, BM, BN, FORM>(a, max_tiles, splits, s);
  return launch_wide<KDP, 256, BM, BN, FORM>(a, max_tiles, splits, s);
}

// The narrow forms' tile of keys for a key length.
int narrow_bn(int KD) { return KD <= 256 ? 64 : 32; }
int round_kd(int KD) { return KD <= 64 ? 64 : KD <= 128 ? 128 : KD <= 256 ? 256 : 512; }
int round_dv(int Dv) { return Dv <= 64 ? 64 : Dv <= 128 ? 128 : 256; }

}  // namespace

// Rows of the smallest tile the launcher may choose: `max_tiles` >= sum over entries of ceil(rows / this).
NV_API int nv_attention_prefill_wide_tile_rows() { return 64; }

// Key length KS * D up to 512, values up to 256, both multiples of 16 and D a multiple of 8; a positive scale.
NV_API int nv_attention_prefill_wide_usable(int D, int KS, int Dv) {
  const int KD = D * KS;
  return D > 0 && KS > 0 && D % 8 == 0 && KD % 16 == 0 && KD <= 512 && Dv > 0 && Dv % 16 == 0 && Dv <= 256;
}

// Whether the HEADS form takes these sizes: every query head reads the same keys, at most 16 query heads, and two
// tiles of all value heads' values fit beside the keys in a CTA's shared memory.
NV_API int nv_attention_wide_heads_usable(int D, int KS, int Dv, int Hq, int Hk, int Hv) {
  if (!nv_attention_prefill_wide_usable(D, KS, Dv) || KS != Hk || Hq < 1 || Hq > 16 || Hv < 1 || Hq % Hv) return 0;
  const int KD = D * KS, bn = narrow_bn(KD);
  return wide_smem_bytes(2, round_kd(KD), round_dv(Dv), bn, bn, Hv, Dv) <= (size_t)220 * 1024;
}

NV_API int nv_attention_prefill_wide(const void* q, const void* kc, const void* vc, const int* block_table,
                                     int max_blocks, const int* cu_rows, const int* entry_pos0, int S, int max_tiles,
                                     float scale, int window, int keep_first, const float* sinks, void* out,
                                     int out_f32, int Hq, int Hk, int Hv, int D, int KS, int Dv, int page, int min_rows,
                                     int max_rows, int narrow, int splits, float* parts, cudaStream_t stream) {
  if (!nv_attention_prefill_wide_usable(D, KS, Dv) || !(scale > 0.f)) return NV_ERR_UNSUPPORTED;
  if (Hq <= 0 || Hk <= 0 || Hv <= 0 || Hq % Hv || (KS == 1 ? Hq % Hk : KS != Hk) || keep_first < 0 || page <= 0)
    return NV_ERR_BAD_SIZE;
  if (((uintptr_t)q & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) || ((uintptr_t)out & 7)) return NV_ERR_UNSUPPORTED;
  if (S == 0 || max_tiles == 0) return NV_OK;
  if (max_rows <= 0) max_rows = INT_MAX;
  if (narrow == 2) max_rows = 1;                    // the tile's rows are the heads of one row
  if (narrow) {
    if (max_rows > 16) max_rows = 16;               // one tile of 16 rows per entry
    if (splits < 1) splits = 1;
    if (splits > 1 && !parts) return NV_ERR_BAD_SIZE;
    if (max_tiles < S) return NV_ERR_BAD_SIZE;
  }
  WideArgs a;
  a.q = (const bf16*)q; a.kc = (const bf16*)kc; a.vc = (const bf16*)vc; a.block_table = block_table;
  a.cu_rows = cu_rows; a.entry_pos0 = entry_pos0; a.sinks = sinks;
  a.out = out; a.scale_log2 = scale * 1.4426950408889634f; a.out_f32 = out_f32;
  a.S = S; a.max_blocks = max_blocks; a.window = window; a.keep_first = keep_first; a.Hq = Hq; a.Hk = Hk; a.Hv = Hv;
  a.D = D; a.KS = KS; a.Dv = Dv; a.page = page; a.min_rows = min_rows; a.max_rows = max_rows; a.parts = parts;
  const int KD = D * KS;
  if (narrow == 2) {
    if (!nv_attention_wide_heads_usable(D, KS, Dv, Hq, Hk, Hv)) return NV_ERR_UNSUPPORTED;
    if (KD <= 64) return launch_wide_v<64, 64, 64, 2>(a, S, splits, stream);
    if (KD <= 128) return launch_wide_v<128, 64, 64, 2>(a, S, splits, stream);
    if (KD <= 256) return launch_wide_v<256, 64, 64, 2>(a, S, splits, stream);
    return launch_wide_v<512, 32, 32, 2>(a, S, splits, stream);
  }
  if (narrow) {
    if (KD <= 64) return launch_wide_v<64, 64, 64, 1>(a, S, splits, stream);
    if (KD <= 128) return launch_wide_v<128, 64, 64, 1>(a, S, splits, stream);
    if (KD <= 256) return launch_wide_v<256, 64, 64, 1>(a, S, splits, stream);
    return launch_wide_v<512, 32, 32, 1>(a, S, splits, stream);
  }
  if (KD <= 64) return launch_wide_v<64, 128, 64, 0>(a, max_tiles, 1, stream);
  if (KD <= 128) return launch_wide_v<128, 128, 64, 0>(a, max_tiles, 1, stream);
  if (KD <= 256) return launch_wide_v<256, 128, 64, 0>(a, max_tiles, 1, stream);
  // eight warps on a tile of 32 keys where that fits in shared memory (217 KB with values up to 128 elements)
  if (a.Dv > 128) return launch_wide<512, 256, 64, 32, 0>(a, max_tiles, 1, stream);
  return launch_wide_v<512, 128, 32, 0>(a, max_tiles, 1, stream);
}
