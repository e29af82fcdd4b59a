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
#include "common.cuh"

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
  float scale_log2;         // scale * log2(e)
  int out_f32;
  int S, max_blocks, window, keep_first, Hq, Hk, Hv, D, KS, Dv, page, min_rows;
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
template <int KDP, int DVP, int BM, int BN>
__global__ void __launch_bounds__(BM * 2, 1) attention_prefill_wide_kernel(WideArgs a) {
  constexpr int THREADS = BM * 2;
  constexpr int LDK = KDP + 8, LDV = DVP + 8;      // row strides (elements): 16 bytes of padding against bank conflicts
  extern __shared__ __align__(16) uint8_t wide_smem[];
  bf16* Qs = (bf16*)wide_smem;                     // [BM][LDK]
  bf16* Ks = Qs + BM * LDK;                        // [2][BN][LDK]
  bf16* Vs = Ks + 2 * BN * LDK;                    // [2][BN][LDV]
  __shared__ int tile_info[3];                     // entry, first row (batch), rows

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int h = blockIdx.y;
  const int D = a.D, KD = a.KS * a.D, Dv = a.Dv;
  const int kh0 = a.KS > 1 ? 0 : h / (a.Hq / a.Hk);
  const int vh = h / (a.Hq / a.Hv);
  const int kchunks = D / 8, vchunks = Dv / 8;

  if (tid == 0) {                                  // which (entry, tile of BM rows) is this CTA's?  Late tiles first.
    int left = (int)(gridDim.x - 1 - blockIdx.x), e = 0, found = -1;
    for (; e < a.S; ++e) {
      const int n = a.cu_rows[e + 1] - a.cu_rows[e];
      const int tiles = n >= a.min_rows ? (n + BM - 1) / BM : 0;
      if (left < tiles) { found = e; break; }
      left -= tiles;
    }
    tile_info[0] = found;
    if (found >= 0) {
      tile_info[1] = a.cu_rows[found] + left * BM;
      tile_info[2] = min(BM, a.cu_rows[found + 1] - tile_info[1]);
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
  const int* bt = a.block_table + (size_t)e * a.max_blocks;

  // ---- Q tile -> shared memory (rows beyond nrows are zero)
  {
    const int qchunks = KD / 8;
    for (int c = tid; c < BM * qchunks; c += THREADS) {
      const int r = c / qchunks, ch = c - r * qchunks;
      bf16* dst = Qs + r * LDK + ch * 8;
      if (r < nrows) copy16(dst, a.q + ((size_t)(row0 + r) * a.Hq + h) * KD + ch * 8);
      else *(uint4*)dst = make_uint4(0, 0, 0, 0);
    }
  }
  auto load_kv = [&](int tile, int buf) {
    const int j0 = tile < nA ? tile * BN : kv0 + (tile - nA) * BN;
    const int jend = tile < nA ? endA : hi;
    bf16* kd = Ks + buf * BN * LDK;
    bf16* vd = Vs + buf * BN * LDV;
    const int per_row = a.KS * kchunks + vchunks;
    for (int c = tid; c < BN * per_row; c += THREADS) {
      const int r = c / per_row, w = c - r * per_row;
      const int j = j0 + r;
      int blk = -1, slot = 0;
      if (j < jend) {
        const int pg = j / a.page;
        slot = j - pg * a.page;
        blk = bt[pg];
      }
      if (w < a.KS * kchunks) {
        const int kc_i = w / kchunks, ch = w - kc_i * kchunks;
        bf16* dst = kd + r * LDK + kc_i * D + ch * 8;
        if (blk >= 0) copy16(dst, a.kc + (((size_t)blk * a.Hk + kh0 + kc_i) * a.page + slot) * D + ch * 8);
        else *(uint4*)dst = make_uint4(0, 0, 0, 0);
      } else {
        const int ch = w - a.KS * kchunks;
        bf16* dst = vd + r * LDV + ch * 8;
        if (blk >= 0) copy16(dst, a.vc + (((size_t)blk * a.Hv + vh) * a.page + slot) * Dv + ch * 8);
        else *(uint4*)dst = make_uint4(0, 0, 0, 0);
      }
    }
  };
  load_kv(0, 0);
  copy_commit();

  const int g = lane / 4, tq = lane % 4;
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;               // this thread's two rows in the tile
  const int p_lo = pos0 + r_lo, p_hi = pos0 + r_hi;
  const bool live_lo = r_lo < nrows, live_hi = r_hi < nrows;
  const int warp_p_lo = pos0 + warp * 16, warp_p_hi = warp_p_lo + 15;

  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o[DVP / 8][4];
#pragma unroll
  for (int i = 0; i < DVP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles) load_kv(t + 1, buf ^ 1);
    copy_commit();
    copy_wait<1>();                                 // tile t (and Q) have landed
    __syncthreads();
    const bf16* kb = Ks + buf * BN * LDK;
    const bf16* vb = Vs + buf * BN * LDV;
    const bool kept_run = t < nA;
    const int j0 = kept_run ? t * BN : kv0 + (t - nA) * BN;
    const int jend = kept_run ? endA : hi;

    // a warp none of whose rows sees any of the tile's keys only keeps the barriers
    const bool behind = !kept_run && a.window > 0 && j0 + BN - 1 <= warp_p_lo - a.window && j0 >= keep;
    const bool warp_sees = warp * 16 < nrows && j0 <= warp_p_hi && !behind;
    if (warp_sees) {
      // ---- S = Q K^T for this warp's 16 rows x BN keys
      float s[BN / 8][4];
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 4
      for (int kk = 0; kk < KDP / 16; ++kk) {
        if (kk * 16 < KD) {
          uint32_t qa[4];
          ldm4(sm_u32(Qs + (warp * 16 + (lane % 8) + 8 * ((lane / 8) % 2)) * LDK + kk * 16 + 8 * (lane / 16)), qa);
#pragma unroll
          for (int np = 0; np < BN / 16; ++np) {
            uint32_t kf[4];
            ldm4(sm_u32(kb + (np * 16 + (lane % 8) + 8 * (lane / 16)) * LDK + kk * 16 + 8 * ((lane / 8) % 2)), kf);
            mma_bf16(s[2 * np], qa, kf[0], kf[1]);
            mma_bf16(s[2 * np + 1], qa, kf[2], kf[3]);
          }
        }
      }
      // ---- mask (unless every row of the warp sees the whole tile), online softmax
      const bool whole = warp * 16 + 15 < nrows && j0 + BN <= jend && j0 + BN - 1 <= warp_p_lo &&
                         (a.window <= 0 || j0 > warp_p_hi - a.window || j0 + BN <= keep);
      if (!whole) {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int j = j0 + nt * 8 + 2 * tq + c;
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
      for (int nt = 0; nt < BN / 8; ++nt) {
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
      for (int nt = 0; nt < BN / 8; ++nt) {
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
      for (int kb16 = 0; kb16 < BN / 16; ++kb16) {
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
#pragma unroll
        for (int dp = 0; dp < DVP / 16; ++dp) {
          if (dp * 16 < Dv) {
            uint32_t vf[4];
            ldm4_t(sm_u32(vb + (kb16 * 16 + (lane % 8) + 8 * ((lane / 8) % 2)) * LDV + dp * 16 + 8 * (lane / 16)), vf);
#pragma unroll
            for (int term = 0; term < WIDE_TERMS; ++term) {
              mma_bf16(o[2 * dp], pt[term], vf[0], vf[1]);
              mma_bf16(o[2 * dp + 1], pt[term], vf[2], vf[3]);
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

template <int KDP, int DVP, int BM, int BN>
int launch_wide(const WideArgs& a, int max_tiles, cudaStream_t s) {
  const size_t smem = ((size_t)(BM + 2 * BN) * (KDP + 8) + (size_t)2 * BN * (DVP + 8)) * sizeof(bf16);
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_wide_kernel<KDP, DVP, BM, BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  attention_prefill_wide_kernel<KDP, DVP, BM, BN><<<dim3(max_tiles, a.Hq), BM * 2, smem, s>>>(a);
  NV_RETURN_LAST();
}

template <int KDP, int BM, int BN>
int launch_wide_v(const WideArgs& a, int max_tiles, cudaStream_t s) {
  if (a.Dv <= 64) return launch_wide<KDP, 64, BM, BN>(a, max_tiles, s);
  if (a.Dv <= 128) return launch_wide<KDP, 128, BM, BN>(a, max_tiles, s);
  return launch_wide<KDP, 256, BM, BN>(a, max_tiles, s);
}

}  // namespace

// Rows of the smallest tile the launcher may choose: `max_tiles` >= sum over entries of ceil(rows / this).
NV_API int nv_attention_prefill_wide_tile_rows() { return 64; }

// Key length KS * D up to 512, values up to 256, both multiples of 16 and D a multiple of 8; a positive scale.
NV_API int nv_attention_prefill_wide_usable(int D, int KS, int Dv) {
  const int KD = D * KS;
  return D > 0 && KS > 0 && D % 8 == 0 && KD % 16 == 0 && KD <= 512 && Dv > 0 && Dv % 16 == 0 && Dv <= 256;
}

NV_API int nv_attention_prefill_wide(const void* q, const void* kc, const void* vc, const int* block_table,
                                     int max_blocks, const int* cu_rows, const int* entry_pos0, int S, int max_tiles,
                                     float scale, int window, int keep_first, const float* sinks, void* out,
                                     int out_f32, int Hq, int Hk, int Hv, int D, int KS, int Dv, int page, int min_rows,
                                     cudaStream_t stream) {
  if (!nv_attention_prefill_wide_usable(D, KS, Dv) || !(scale > 0.f)) return NV_ERR_UNSUPPORTED;
  if (Hq <= 0 || Hk <= 0 || Hv <= 0 || Hq % Hv || (KS == 1 ? Hq % Hk : KS != Hk) || keep_first < 0 || page <= 0)
    return NV_ERR_BAD_SIZE;
  if (((uintptr_t)q & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) || ((uintptr_t)out & 7)) return NV_ERR_UNSUPPORTED;
  if (S == 0 || max_tiles == 0) return NV_OK;
  WideArgs a;
  a.q = (const bf16*)q; a.kc = (const bf16*)kc; a.vc = (const bf16*)vc; a.block_table = block_table;
  a.cu_rows = cu_rows; a.entry_pos0 = entry_pos0; a.sinks = sinks;
  a.out = out; a.scale_log2 = scale * 1.4426950408889634f; a.out_f32 = out_f32;
  a.S = S; a.max_blocks = max_blocks; a.window = window; a.keep_first = keep_first; a.Hq = Hq; a.Hk = Hk; a.Hv = Hv;
  a.D = D; a.KS = KS; a.Dv = Dv; a.page = page; a.min_rows = min_rows;
  const int KD = D * KS;
  if (KD <= 64) return launch_wide_v<64, 128, 64>(a, max_tiles, stream);
  if (KD <= 128) return launch_wide_v<128, 128, 64>(a, max_tiles, stream);
  if (KD <= 256) return launch_wide_v<256, 128, 64>(a, max_tiles, stream);
  return launch_wide_v<512, 64, 32>(a, max_tiles, stream);
}
