// Kernels of the mixers that keep a fixed-size state per request, and of the layer pieces around them:
//
//   branch_norm_add   x += rms(y) * w, y one branch or the mean of several RMS-normed, weighted branches;
//                     also the residual stream's rows in the activation type for the products that read them
//   activation        gelu (erf or tanh form) or silu over a matrix
//   token_gate        gelu_tanh(gate) * table[token, columns of this layer]
//   conv_silu_norm    short causal convolution per channel over time with silu; q and k heads made unit vectors
//   conv_state_update the last taps - 1 inputs of every channel, kept per request
//   mlstm_scan        matrix memory with exponential input gate, a running maximum and a normaliser state
//   gated_delta_scan  matrix memory with a decay per head and the delta rule
//   qk_prepare_store  q/k head norm, rotation of pairs (interleaved or split halves), keys and values to their pages
//   paged_attention_general   softmax attention over paged keys with separate key and value sizes and an optional sink
//
// Everything that enters a recurrence, every norm, every gate, angle, score and weight is computed in 32-bit floats
// whatever the storage type of the activations is.  The sums of a row are taken in an order that depends on the
// row alone (its own block, a thread's elements in order, a fixed tree over threads), so a row's result does not
// depend on what else is in the batch nor on how its sequence was cut into steps.
#include "common.cuh"

#include <algorithm>

namespace {

constexpr int SM_THREADS = 256;

// Sum over the block, the same order for every call; `red` holds blockDim.x / 32 floats.  All threads get the sum.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();          // (red may still be read from the call before)
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < nw; ++i) s += red[i];
  return s;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float gelu_erf_(float z) { return 0.5f * z * (1.f + erff(z * 0.70710678118654752440f)); }
__device__ __forceinline__ float gelu_tanh_(float z) {
  return 0.5f * z * (1.f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
}

// ------------------------------------------------------------------ branch norm + residual sum
constexpr int MAX_BRANCHES = 4;
struct BranchArgs {
  float* x;                         // [T, H] residual stream, updated in place
  const float* br[MAX_BRANCHES];    // [T, H] branch outputs
  const float* bw[MAX_BRANCHES];    // [H] weights of the branches' own norms (all given, or none with nb == 1)
  const float* w;                   // [H] weight of the norm over the (mixed) branch
  void* out;                        // [T, H] x after the sum, in out_dt (may be null); with next_w its normed rows
  int nb, H, out_dt;
  float eps, mix_scale;
  // The branch as a sum that has not been taken (nb == 0, R > 0 or dense given):
  // y[t] = sigmoid(gate_logit[t]) * dense[t] + sum_r weight[t, r] * rows[index[t, r]]
  const float* rows;
  const int* index;
  const float* weight;
  int R;
  const float* dense;
  const float* gate_logit;
  long long gate_ld;
  // A second norm over the stream after the sum: out = rms(x) * next_w (and out32, a float32 copy of it)
  const float* next_w;
  float next_eps;
  float* out32;
};

__global__ void __launch_bounds__(SM_THREADS) branch_norm_add_kernel(BranchArgs a) {
  extern __shared__ float ysm[];    // H floats
  __shared__ float red[SM_THREADS / 32];
  const int t = blockIdx.x, tid = threadIdx.x, H = a.H;
  const size_t base = (size_t)t * H;
  const bool mixed = a.R > 0 || a.dense != nullptr;
  if (a.nb == 0 && !mixed) {
    if (a.next_w) {
      for (int i = tid; i < H; i += SM_THREADS) ysm[i] = a.x[base + i];
    } else {
      if (a.out)
        for (int i = tid; i < H; i += SM_THREADS) st_dt(a.out, a.out_dt, base + i, a.x[base + i]);
      return;
    }
  } else {
    if (mixed) {
      const float gate = a.dense && a.gate_logit ? sigmoidf_(a.gate_logit[(size_t)t * a.gate_ld]) : 1.f;
      for (int i = tid; i < H; i += SM_THREADS) {
        float y = 0.f;
        for (int k = 0; k < a.R; ++k)        // the sum keeps the order of k
          y = fmaf(a.weight[(size_t)t * a.R + k], a.rows[(size_t)a.index[(size_t)t * a.R + k] * H + i], y);
        if (a.dense) y = a.dense[base + i] * gate + y;
        ysm[i] = y;
      }
    } else if (a.bw[0]) {
      for (int i = tid; i < H; i += SM_THREADS) ysm[i] = 0.f;
      for (int b = 0; b < a.nb; ++b) {
        float ss = 0.f;
        for (int i = tid; i < H; i += SM_THREADS) { float v = a.br[b][base + i]; ss = fmaf(v, v, ss); }
        const float r = rsqrtf(block_sum(ss, red) / (float)H + a.eps);
        for (int i = tid; i < H; i += SM_THREADS) ysm[i] += a.br[b][base + i] * r * a.bw[b][i];
      }
      for (int i = tid; i < H; i += SM_THREADS) ysm[i] *= a.mix_scale;
    } else {
      for (int i = tid; i < H; i += SM_THREADS) ysm[i] = a.br[0][base + i];
    }
    float ss = 0.f;
    for (int i = tid; i < H; i += SM_THREADS) ss = fmaf(ysm[i], ysm[i], ss);
    const float r = rsqrtf(block_sum(ss, red) / (float)H + a.eps);
    for (int i = tid; i < H; i += SM_THREADS) {
      const float v = a.x[base + i] + ysm[i] * r * a.w[i];
      a.x[base + i] = v;
      if (a.next_w) ysm[i] = v;
      else if (a.out) st_dt(a.out, a.out_dt, base + i, v);
    }
    if (!a.next_w) return;
  }
  // the next sublayer's input: the norm of the stream as it is now (a thread reads back what it wrote itself)
  float ss = 0.f;
  for (int i = tid; i < H; i += SM_THREADS) ss = fmaf(ysm[i], ysm[i], ss);
  const float r = rsqrtf(block_sum(ss, red) / (float)H + a.next_eps);
  for (int i = tid; i < H; i += SM_THREADS) {
    const float v = ysm[i] * r * a.next_w[i];
    if (a.out) st_dt(a.out, a.out_dt, base + i, v);
    if (a.out32) a.out32[base + i] = v;
  }
}

// ------------------------------------------------------------------ activation over a matrix
// kind 3, xIELU with the two positive numbers (p0, p1): z > 0: p0 z^2 + z / 2; z <= 0: p1 (e^z - 1 - z) + z / 2
__device__ __forceinline__ float act_of(int kind, float z, float p0 = 0.f, float p1 = 0.f) {
  if (kind == 3) return z > 0.f ? fmaf(p0 * z, z, 0.5f * z) : fmaf(p1, expm1f(z) - z, 0.5f * z);
  if (kind == 4) { z = fmaxf(z, 0.f); return z * z; }          // the square of relu
  return kind == 0 ? gelu_erf_(z) : (kind == 1 ? gelu_tanh_(z) : siluf_(z));
}

__global__ void activation_kernel(const void* __restrict__ in, int in_dt, void* __restrict__ out, int out_dt,
                                  long long n, int kind, float p0, float p1) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  st_dt(out, out_dt, i, act_of(kind, ld_dt(in, in_dt, i), p0, p1));
}

// float32 in, bfloat16 out, four values per thread (16 bytes in, 8 out): what a bfloat16 prompt's MLP runs
__global__ void activation_f32_bf16_x4_kernel(const float4* __restrict__ in, uint2* __restrict__ out, long long n4,
                                              int kind, float p0, float p1) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 z = in[i];
  const __nv_bfloat162 lo = __floats2bfloat162_rn(act_of(kind, z.x, p0, p1), act_of(kind, z.y, p0, p1));
  const __nv_bfloat162 hi = __floats2bfloat162_rn(act_of(kind, z.z, p0, p1), act_of(kind, z.w, p0, p1));
  uint2 o;
  o.x = *reinterpret_cast<const uint32_t*>(&lo);
  o.y = *reinterpret_cast<const uint32_t*>(&hi);
  out[i] = o;
}

// ------------------------------------------------------------------ gate times a per-token table row
// out[t, j] = gelu_tanh(gate[t, j]) * table[id(t), col0 + j]; a negative id -(r + 1) is read from feed[r]
__global__ void token_gate_kernel(const void* __restrict__ gate, int gate_dt, long long gate_ld,
                                  const int* __restrict__ ids, const int* __restrict__ feed,
                                  const void* __restrict__ table, int table_dt, long long table_ld, int col0, int d,
                                  int V, void* __restrict__ out, int out_dt, int* __restrict__ err) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && feed) id = feed[-id - 1];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicExch(err, 1 + t);
    id = 0;
  }
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    const float g = gelu_tanh_(ld_dt(gate, gate_dt, (size_t)t * gate_ld + j));
    st_dt(out, out_dt, (size_t)t * d + j, g * ld_dt(table, table_dt, (size_t)id * table_ld + col0 + j));
  }
}

// ------------------------------------------------------------------ short convolution over time
// in: [T, ld] float32 or bfloat16, channels col0 .. col0 + C; w: [C, taps] float32, the last column the current token's;
// state: per slot [taps - 1, C] float32, the inputs of the request's last taps - 1 positions (zero before its start).
// out[t, c] = silu(sum_d w[c, taps - 1 - d] * in(t - d)); then every one of the first `unit_heads` heads of
// `unit_dim` channels is divided by sqrt(sum of squares + unit_eps), and the first `scaled_heads` of them also
// multiplied by `scale`.  One block per row.
__global__ void __launch_bounds__(SM_THREADS) conv_silu_norm_kernel(
    const void* __restrict__ in, int in_dt, long long ld, int col0, int C, const float* __restrict__ w, int taps,
    const int* __restrict__ row_entry, const int* __restrict__ cu_rows, const int* __restrict__ entry_slot,
    const float* __restrict__ state, long long slot_stride, int unit_heads, int unit_dim, float unit_eps,
    int scaled_heads, float scale, float* __restrict__ out) {
  extern __shared__ float ysm[];    // C floats
  const int t = blockIdx.x, tid = threadIdx.x;
  const int e = row_entry[t];
  const int j = t - cu_rows[e];
  const float* st = state + (size_t)entry_slot[e] * slot_stride;
  for (int c = tid; c < C; c += SM_THREADS) {
    float acc = 0.f;
    for (int d = 0; d < taps; ++d) {
      const int jj = j - d;
      const float v = jj >= 0 ? ld_dt(in, in_dt, (size_t)(t - d) * ld + col0 + c) : st[(size_t)(taps - 1 + jj) * C + c];
      acc = fmaf(w[(size_t)c * taps + (taps - 1 - d)], v, acc);
    }
    ysm[c] = siluf_(acc);
  }
  __syncthreads();
  const int lane = tid & 31, warp = tid >> 5;
  for (int h = warp; h < unit_heads; h += SM_THREADS / 32) {
    float ss = 0.f;
    for (int i = lane; i < unit_dim; i += 32) { float v = ysm[h * unit_dim + i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss + unit_eps) * (h < scaled_heads ? scale : 1.f);
    for (int i = lane; i < unit_dim; i += 32) ysm[h * unit_dim + i] *= r;
  }
  __syncthreads();
  for (int c = tid; c < C; c += SM_THREADS) out[(size_t)t * C + c] = ysm[c];
}

// After the convolution has read the old state: state[s] = the input at the entry's position end - (taps - 1) + s.
// A thread owns a channel and goes through s upward, so what it still has to read (old[s + len]) lies above what
// it has written.
__global__ void conv_state_update_kernel(const void* __restrict__ in, int in_dt, long long ld, int col0, int C,
                                         int taps, const int* __restrict__ cu_rows,
                                         const int* __restrict__ entry_slot, float* __restrict__ state,
                                         long long slot_stride) {
  const int e = blockIdx.x;
  const int row0 = cu_rows[e], len = cu_rows[e + 1] - row0;
  float* st = state + (size_t)entry_slot[e] * slot_stride;
  for (int c = threadIdx.x; c < C; c += blockDim.x)
    for (int s = 0; s < taps - 1; ++s) {
      const int jj = len - (taps - 1) + s;
      st[(size_t)s * C + c] = jj >= 0 ? ld_dt(in, in_dt, (size_t)(row0 + jj) * ld + col0 + c) : st[(size_t)(s + len) * C + c];
    }
}

// ------------------------------------------------------------------ matrix memories, token by token
// One block per (entry, head).  The head's matrix S [dk, dv] lives in shared memory while the entry's rows run and
// goes back to the request's state afterwards.  Thread (c, rs) = (tid % dv, tid / dv) owns column c and the rows
// r = rs, rs + RS, ...; sums over rows are taken per thread in that order and then over rs in order.
struct ScanCommon {
  const int* cu_rows;
  const int* entry_slot;
  float* S;                 // [slots][H, dk, dv]
  long long S_stride;
  const float* norm_w;
  void* out;                // [T, H * dv]
  int out_dt, H, dk, dv;
  float eps;
};

struct MlstmArgs {
  ScanCommon c;
  const float* proj;        // [T, ld] float32: q | k | v | gate | i | f at their columns
  long long ld;
  int q0, k0, v0, g0, i0, f0;
  float* n;                 // [slots][H, dk]
  long long n_stride;
  float* m;                 // [slots][H]
  long long m_stride;
  float cap, q_scale, den_eps;
  int norm_per_head;        // the norm weight has H * dv entries (else dv, shared by the heads)
};

__global__ void __launch_bounds__(SM_THREADS) mlstm_scan_kernel(MlstmArgs a) {
  extern __shared__ float sm[];
  const int dk = a.c.dk, dv = a.c.dv, H = a.c.H;
  const int RS = max(1, min(SM_THREADS / dv, dk));
  float* S = sm;                     // dk * dv
  float* nn = S + dk * dv;           // dk
  float* q = nn + dk;                // dk
  float* k = q + dk;                 // dk
  float* v = k + dk;                 // dv
  float* part = v + dv;              // RS * dv
  float* o = part + RS * dv;         // dv
  float* sc = o + dv;                // 8 scalars
  const int e = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int row0 = a.c.cu_rows[e], row1 = a.c.cu_rows[e + 1];
  const int slot = a.c.entry_slot[e];
  float* Sg = a.c.S + (size_t)slot * a.c.S_stride + (size_t)h * dk * dv;
  float* ng = a.n + (size_t)slot * a.n_stride + (size_t)h * dk;
  float* mg = a.m + (size_t)slot * a.m_stride + h;
  for (int i = tid; i < dk * dv; i += SM_THREADS) S[i] = Sg[i];
  for (int i = tid; i < dk; i += SM_THREADS) nn[i] = ng[i];
  float m = *mg;
  const int c = tid % dv, rs = tid / dv;
  const bool owner = tid < RS * dv;
  __syncthreads();
  for (int t = row0; t < row1; ++t) {
    const float* p = a.proj + (size_t)t * a.ld;
    for (int i = tid; i < dk; i += SM_THREADS) {
      q[i] = p[a.q0 + h * dk + i] * a.q_scale;
      k[i] = p[a.k0 + h * dk + i];
    }
    for (int i = tid; i < dv; i += SM_THREADS) v[i] = p[a.v0 + h * dv + i];
    // gates: every thread computes the same numbers
    const float ig = a.cap * tanhf(p[a.i0 + h] / a.cap);
    const float fg = logsigmoidf_(a.cap * tanhf(p[a.f0 + h] / a.cap));
    const float m_new = fmaxf(fg + m, ig);
    const float fa = expf(fg + m - m_new), ib = expf(ig - m_new);
    m = m_new;
    __syncthreads();
    if (tid < 32) {                  // the normaliser state and its product with q
      float acc = 0.f;
      for (int r = tid; r < dk; r += 32) {
        const float x = fa * nn[r] + ib * k[r];
        nn[r] = x;
        acc = fmaf(x, q[r], acc);
      }
      acc = warp_sum(acc);
      if (tid == 0) sc[0] = acc;
    }
    if (owner) {
      float acc = 0.f;
      const float bv = ib * v[c];
      for (int r = rs; r < dk; r += RS) {
        const float s = fa * S[r * dv + c] + k[r] * bv;
        S[r * dv + c] = s;
        acc = fmaf(s, q[r], acc);
      }
      part[rs * dv + c] = acc;
    }
    __syncthreads();
    if (tid < dv) {
      float num = 0.f;
      for (int i = 0; i < RS; ++i) num += part[i * dv + tid];
      const float den = fmaxf(fabsf(sc[0]), expf(-m)) + a.den_eps;
      o[tid] = num / den;
    }
    __syncthreads();
    if (tid < 32) {
      float ss = 0.f;
      for (int i = tid; i < dv; i += 32) ss = fmaf(o[i], o[i], ss);
      ss = warp_sum(ss);
      if (tid == 0) sc[1] = rsqrtf(ss / (float)dv + a.c.eps);
    }
    __syncthreads();
    if (tid < dv) {
      const float w = a.c.norm_w[a.norm_per_head ? h * dv + tid : tid];
      const float gate = sigmoidf_(p[a.g0 + h * dv + tid]);
      st_dt(a.c.out, a.c.out_dt, (size_t)t * H * dv + (size_t)h * dv + tid, o[tid] * sc[1] * w * gate);
    }
  }
  __syncthreads();
  for (int i = tid; i < dk * dv; i += SM_THREADS) Sg[i] = S[i];
  for (int i = tid; i < dk; i += SM_THREADS) ng[i] = nn[i];
  if (tid == 0) *mg = m;
}

struct DeltaArgs {
  ScanCommon c;
  const float* qkv;         // [T, C] float32 after convolution, activation and unit norm: q | k | v
  int C, q0, k0, v0, G;     // G heads of q and k; head h reads q/k head h / (H / G)
  const void* proj;         // [T, ld]: output gate, beta and decay pre-activations at their columns
  int proj_dt;
  long long ld;
  int g0, b0, a0;
  const float* A_log;       // [H]
  const float* dt_bias;     // [H], or [H * dk] with a decay per key channel
  // decay_mode 1: one decay per head and key channel, g[r] = exp(-exp(A_log[h]) softplus(dec[t, dec0 + h dk + r] +
  // dt_bias[h dk + r])), acting on row r of the head's matrix.  gate_mode 1: the output gate is a sigmoid (0: silu).
  // The output gate's pre-activations are read from gsrc (column g0), which may be another matrix than proj.
  const float* dec;         // [T, dec_ld] float32
  long long dec_ld;
  int dec0;
  const void* gsrc;
  int gsrc_dt;
  long long gsrc_ld;
  int decay_mode, gate_mode;
};

__global__ void __launch_bounds__(SM_THREADS) gated_delta_scan_kernel(DeltaArgs a) {
  extern __shared__ float sm[];
  const int dk = a.c.dk, dv = a.c.dv, H = a.c.H;
  const int RS = max(1, min(SM_THREADS / dv, dk));
  float* S = sm;                     // dk * dv
  float* q = S + dk * dv;            // dk
  float* k = q + dk;                 // dk
  float* v = k + dk;                 // dv
  float* partk = v + dv;             // RS * dv
  float* partq = partk + RS * dv;    // RS * dv
  float* u = partq + RS * dv;        // dv
  float* o = u + dv;                 // dv
  float* sc = o + dv;                // 8 scalars
  float* gv = sc + 8;                // dk: the key channels' decays (decay_mode 1)
  const int e = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int gh = h / (H / a.G);
  const bool chan = a.decay_mode == 1;
  const int row0 = a.c.cu_rows[e], row1 = a.c.cu_rows[e + 1];
  float* Sg = a.c.S + (size_t)a.c.entry_slot[e] * a.c.S_stride + (size_t)h * dk * dv;
  for (int i = tid; i < dk * dv; i += SM_THREADS) S[i] = Sg[i];
  const int c = tid % dv, rs = tid / dv;
  const bool owner = tid < RS * dv;
  const float rate = expf(a.A_log[h]), dtb = chan ? 0.f : a.dt_bias[h];
  __syncthreads();
  for (int t = row0; t < row1; ++t) {
    const float* x = a.qkv + (size_t)t * a.C;
    for (int i = tid; i < dk; i += SM_THREADS) {
      q[i] = x[a.q0 + gh * dk + i];
      k[i] = x[a.k0 + gh * dk + i];
      if (chan)
        gv[i] = expf(-rate * softplusf_(a.dec[(size_t)t * a.dec_ld + a.dec0 + h * dk + i] + a.dt_bias[h * dk + i]));
    }
    for (int i = tid; i < dv; i += SM_THREADS) v[i] = x[a.v0 + h * dv + i];
    const float beta = sigmoidf_(ld_dt(a.proj, a.proj_dt, (size_t)t * a.ld + a.b0 + h));
    const float g = chan ? 1.f : expf(-rate * softplusf_(ld_dt(a.proj, a.proj_dt, (size_t)t * a.ld + a.a0 + h) + dtb));
    __syncthreads();
    if (tid < 32) {
      float acc = 0.f;
      for (int r = tid; r < dk; r += 32) acc = fmaf(k[r], q[r], acc);
      acc = warp_sum(acc);
      if (tid == 0) sc[0] = acc;
    }
    if (owner) {
      float ak = 0.f, aq = 0.f;
      if (chan) {
        for (int r = rs; r < dk; r += RS) {
          const float s = S[r * dv + c] * gv[r];      // the decayed row, as the update below leaves it
          ak = fmaf(s, k[r], ak);
          aq = fmaf(s, q[r], aq);
        }
      } else {
        for (int r = rs; r < dk; r += RS) {
          const float s = S[r * dv + c];
          ak = fmaf(s, k[r], ak);
          aq = fmaf(s, q[r], aq);
        }
      }
      partk[rs * dv + c] = ak;
      partq[rs * dv + c] = aq;
    }
    __syncthreads();
    if (tid < dv) {
      float sk = 0.f, sq = 0.f;
      for (int i = 0; i < RS; ++i) { sk += partk[i * dv + tid]; sq += partq[i * dv + tid]; }
      const float uu = beta * (v[tid] - g * sk);
      u[tid] = uu;
      o[tid] = g * sq + sc[0] * uu;
    }
    __syncthreads();
    if (owner) {
      const float uu = u[c];
      if (chan)
        for (int r = rs; r < dk; r += RS) S[r * dv + c] = fmaf(k[r], uu, S[r * dv + c] * gv[r]);
      else
        for (int r = rs; r < dk; r += RS) S[r * dv + c] = g * S[r * dv + c] + k[r] * uu;
    }
    if (tid < 32) {
      float ss = 0.f;
      for (int i = tid; i < dv; i += 32) ss = fmaf(o[i], o[i], ss);
      ss = warp_sum(ss);
      if (tid == 0) sc[1] = rsqrtf(ss / (float)dv + a.c.eps);
    }
    __syncthreads();
    if (tid < dv) {
      const float gz = ld_dt(a.gsrc, a.gsrc_dt, (size_t)t * a.gsrc_ld + a.g0 + h * dv + tid);
      const float gate = a.gate_mode == 1 ? sigmoidf_(gz) : siluf_(gz);
      st_dt(a.c.out, a.c.out_dt, (size_t)t * H * dv + (size_t)h * dv + tid, o[tid] * sc[1] * a.c.norm_w[tid] * gate);
    }
  }
  __syncthreads();
  for (int i = tid; i < dk * dv; i += SM_THREADS) Sg[i] = S[i];
}

// ------------------------------------------------------------------ q/k head norm, rotation, cache write
// in: [T, ld] with q at q0 (Hq * D), k at k0 (Hkv * D), v at v0 (Hkv * Dv).  Per q and k head: RMS norm over D with
// the weight qw / kw (null: no norm); then the first rot_dim elements are turned in pairs, (2i, 2i + 1) if
// `interleaved` else (i, i + rot_dim / 2), by the angle position * inv_freq[i], cosine and sine times `amplitude`.
// q goes to q_out [T, Hq * QP]; k and v go to the row's place in their pages, whose rows may be longer than D and
// Dv (KP, VP): what lies behind a head's elements is written as zero, so that a kernel that wants one head size
// for q, k and v can read all three.  One block per row, a warp per head.
struct QkArgs {
  const void* in;
  int in_dt;
  long long ld;
  int q0, k0, v0;
  const int* positions;
  const int* row_entry;
  const int* block_table;
  int max_blocks;
  const float* qw;
  const float* kw;
  float eps;
  const float* inv_freq;
  int rot_dim, interleaved;
  float amplitude;
  void* q_out;
  int q_dt;
  void* kc;
  void* vc;
  int cache_dt;
  int Hq, Hkv, D, Dv, page, write_kv;
  int* err;
  int QP, KP, VP;           // elements per head in q_out, in the key pages and in the value pages (>= D, D, Dv; the rest is zero)
  int rot0;                 // the turned elements are rot0 .. rot0 + rot_dim - 1 of a head
  int k_norm_dim;           // key heads: the norm is taken over (and applied to) the first so many elements; 0: all D
  int norm_mode;            // bit 0: q and k heads are normed also without a weight (the weight is then one);
                            // bit 1: after the turn instead of before it
  const float* v_inv_freq;  // values are turned too: the first v_rot_dim elements of every value head, in pairs
  int v_rot_dim;            // (i, i + v_rot_dim / 2), by position * v_inv_freq[i]; 0: values are stored as projected
};

constexpr int QK_THREADS = 128;

__global__ void __launch_bounds__(QK_THREADS) qk_prepare_store_kernel(QkArgs a) {
  extern __shared__ float sm[];      // per warp D floats
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = a.D, half = a.rot_dim / 2;
  float* buf = sm + warp * D;
  const int pos = a.positions[t];
  int blk = 0, write_kv = a.write_kv;
  if (write_kv) {
    blk = a.block_table[(size_t)a.row_entry[t] * a.max_blocks + pos / a.page];
    if (blk < 0) {
      if (threadIdx.x == 0) atomicExch(a.err, 1 + t);
      write_kv = 0;
    }
  }
  const size_t slot = (size_t)(pos % a.page);
  const int heads = a.Hq + (write_kv ? a.Hkv : 0);
  for (int h = warp; h < heads; h += QK_THREADS / 32) {
    const bool is_q = h < a.Hq;
    const size_t src = (size_t)t * a.ld + (is_q ? a.q0 + h * D : a.k0 + (h - a.Hq) * D);
    const float* w = is_q ? a.qw : a.kw;
    const int nd = (!is_q && a.k_norm_dim > 0) ? a.k_norm_dim : D;     // what the norm covers
    const bool normed = w != nullptr || (a.norm_mode & 1);
    const bool after = (a.norm_mode & 2) != 0;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float x = ld_dt(a.in, a.in_dt, src + i);
      buf[i] = x;
      if (i < nd) ss = fmaf(x, x, ss);
    }
    if (normed && !after) {
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)nd + a.eps);
      for (int i = lane; i < nd; i += 32) buf[i] = buf[i] * r * (w ? w[i] : 1.f);
    }
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
      const int i0 = a.rot0 + (a.interleaved ? 2 * i : i), i1 = a.rot0 + (a.interleaved ? 2 * i + 1 : i + half);
      const float ang = (float)pos * a.inv_freq[i];
      const float cs = cosf(ang) * a.amplitude, sn = sinf(ang) * a.amplitude;
      const float x0 = buf[i0], x1 = buf[i1];
      buf[i0] = x0 * cs - x1 * sn;
      buf[i1] = x1 * cs + x0 * sn;
    }
    __syncwarp();
    if (normed && after) {
      ss = 0.f;
      for (int i = lane; i < nd; i += 32) ss = fmaf(buf[i], buf[i], ss);
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)nd + a.eps);
      for (int i = lane; i < nd; i += 32) buf[i] = buf[i] * r * (w ? w[i] : 1.f);
      __syncwarp();
    }
    if (is_q) {
      const size_t dst = ((size_t)t * a.Hq + h) * a.QP;
      for (int i = lane; i < a.QP; i += 32) st_dt(a.q_out, a.q_dt, dst + i, i < D ? buf[i] : 0.f);
    } else {
      const size_t dst = (((size_t)blk * a.Hkv + (h - a.Hq)) * a.page + slot) * a.KP;
      for (int i = lane; i < a.KP; i += 32) st_dt(a.kc, a.cache_dt, dst + i, i < D ? buf[i] : 0.f);
    }
    __syncwarp();
  }
  if (write_kv && a.vc) {
    const int vhalf = a.v_rot_dim / 2;
    for (int i = threadIdx.x; i < a.Hkv * a.VP; i += QK_THREADS) {
      const int hv = i / a.VP, d = i % a.VP;
      const size_t dst = (((size_t)blk * a.Hkv + hv) * a.page + slot) * a.VP + d;
      const size_t src = (size_t)t * a.ld + a.v0 + hv * a.Dv;
      float x = d < a.Dv ? ld_dt(a.in, a.in_dt, src + d) : 0.f;
      if (d < a.v_rot_dim) {
        const int pr = d < vhalf ? d : d - vhalf;
        const float ang = (float)pos * a.v_inv_freq[pr];
        const float cs = cosf(ang), sn = sinf(ang);
        const float other = ld_dt(a.in, a.in_dt, src + (d < vhalf ? d + vhalf : d - vhalf));
        x = d < vhalf ? x * cs - other * sn : x * cs + other * sn;
      }
      st_dt(a.vc, a.cache_dt, dst, x);
    }
  }
}

// ------------------------------------------------------------------ paged softmax attention, general sizes
// One block per (row, query head).  Keys of D elements, values of Dv.  A softmax may hold a *sink*, a score without
// a key or a value that counts once in the denominator: one score for all heads (`has_sink`) or a learned one per
// head (`sinks`).  `keep_first` > 0 with a window: the first so many positions of the sequence stay visible after
// the window has passed them.  `key_span` = KS > 1: a query row holds KS * D elements per head and its score with
// position j is the sum of its KS parts' products with the keys of kv heads 0 .. KS - 1 at j (scores that are mixed
// across heads are linear in the queries, so the mixing is done once per row on the queries); values are read from
// the head's own kv head as always.  Chunks of ATTG_THREADS keys, running maximum.
constexpr int ATTG_THREADS = 128;
constexpr int ATTG_NV = 8;           // output elements per thread: values up to ATTG_NV * ATTG_THREADS wide

__global__ void __launch_bounds__(ATTG_THREADS) paged_attention_general_kernel(
    const void* __restrict__ q, int q_dt, const void* __restrict__ kc, const void* __restrict__ vc, int cache_dt,
    const int* __restrict__ block_table, int max_blocks, const int* __restrict__ row_entry,
    const int* __restrict__ positions, float scale, int window, int keep_first, int has_sink, float sink_score,
    const float* __restrict__ sinks, void* __restrict__ out, int out_dt, int Hq, int Hkv, int Hv, int D, int Dv,
    int KS, int page, float softcap) {
  extern __shared__ float qs[];      // KS * D
  __shared__ float p[ATTG_THREADS];
  __shared__ int pslot[ATTG_THREADS];
  __shared__ float red[ATTG_THREADS / 32];
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int kvh = KS > 1 ? 0 : h / (Hq / Hkv);     // first key head of the score
  const int vh = h / (Hq / Hv);                    // the head's value head
  const int n = positions[t] + 1;
  const int lo = window > 0 ? max(0, n - window) : 0;
  const int nkeep = min(keep_first, lo);           // kept positions that the window no longer covers
  const int total = nkeep + (n - lo);
  const int* bt = block_table + (size_t)row_entry[t] * max_blocks;
  const int QD = KS * D;
  for (int d = tid; d < QD; d += ATTG_THREADS) qs[d] = ld_dt(q, q_dt, (size_t)t * Hq * QD + (size_t)h * QD + d);
  __syncthreads();
  if (sinks) { has_sink = 1; sink_score = sinks[h]; }
  float m = has_sink ? sink_score : -1e30f, l = has_sink ? 1.f : 0.f;
  float o[ATTG_NV];
#pragma unroll
  for (int u = 0; u < ATTG_NV; ++u) o[u] = 0.f;
  for (int c0 = 0; c0 < total; c0 += ATTG_THREADS) {
    const int i = c0 + tid;
    float s = -1e30f;
    if (i < total) {
      const int j = i < nkeep ? i : lo + (i - nkeep);
      const int blk = bt[j / page];
      const size_t slot = (size_t)blk * page + j % page;       // [page][head][slot]: head added below
      pslot[tid] = (int)(((size_t)blk * Hv + vh) * page + j % page);
      float acc = 0.f;
      for (int c = 0; c < KS; ++c) {
        const size_t kb = ((size_t)blk * Hkv + kvh + c) * page + j % page;
        const float* qq = qs + c * D;
        for (int d = 0; d < D; ++d) acc = fmaf(qq[d], ld_dt(kc, cache_dt, kb * D + d), acc);
      }
      (void)slot;
      s = acc * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    }
    // maximum over the chunk
    float mx = warp_max(s);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    mx = red[0];
    for (int i2 = 1; i2 < ATTG_THREADS / 32; ++i2) mx = fmaxf(mx, red[i2]);
    const float m_new = fmaxf(m, mx);
    const float ex = i < total ? expf(s - m_new) : 0.f;
    p[tid] = ex;
    float sum = warp_sum(ex);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = sum;
    __syncthreads();
    sum = 0.f;
    for (int i2 = 0; i2 < ATTG_THREADS / 32; ++i2) sum += red[i2];
    const float alpha = expf(m - m_new);
    l = l * alpha + sum;
    m = m_new;
    const int cnt = min(ATTG_THREADS, total - c0);
#pragma unroll
    for (int u = 0; u < ATTG_NV; ++u) {
      const int d = tid + u * ATTG_THREADS;
      o[u] *= alpha;
      if (d < Dv)
        for (int i2 = 0; i2 < cnt; ++i2) o[u] = fmaf(p[i2], ld_dt(vc, cache_dt, (size_t)pslot[i2] * Dv + d), o[u]);
    }
    __syncthreads();
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const size_t ob = (size_t)t * Hq * Dv + (size_t)h * Dv;
#pragma unroll
  for (int u = 0; u < ATTG_NV; ++u) {
    const int d = tid + u * ATTG_THREADS;
    if (d < Dv) st_dt(out, out_dt, ob + d, o[u] * inv);
  }
}

// ------------------------------------------------------------------ queries mixed across heads
// q [T, H, D] float32 -> out [T, H, G * D]: out[t, h, c D + d] = sum over the heads g of kv head c of
// mix[h, g] * q[t, g, d].  With it, sum_g mix[h, g] (q_g . k_kv(g)) is one product of the mixed query row with the
// kv heads' keys side by side.  One block per row.
__global__ void __launch_bounds__(256) mix_query_heads_kernel(const float* __restrict__ q, const float* __restrict__ mix,
                                                              void* __restrict__ out, int out_dt, int H, int G, int D) {
  extern __shared__ float sm[];      // H * D query elements, then H * H weights
  float* qs = sm;
  float* w = sm + H * D;
  const int t = blockIdx.x, rep = H / G;
  for (int i = threadIdx.x; i < H * D; i += blockDim.x) qs[i] = q[(size_t)t * H * D + i];
  for (int i = threadIdx.x; i < H * H; i += blockDim.x) w[i] = mix[i];
  __syncthreads();
  const int n = H * G * D;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int h = i / (G * D), c = (i / D) % G, d = i % D;
    float acc = 0.f;
    for (int g = c * rep; g < (c + 1) * rep; ++g) acc = fmaf(w[h * H + g], qs[g * D + d], acc);
    st_dt(out, out_dt, (size_t)t * n + i, acc);
  }
}

// ------------------------------------------------------------------ rotation of whole heads
// x [T, H, D] (in_dt) -> out (out_dt): the first rot_dim elements of every head turned in pairs (i, i + rot_dim / 2)
// by sign * position * inv_freq[i].  sign -1 turns back what was turned by the same position.
__global__ void rotate_heads_kernel(const void* __restrict__ x, int in_dt, const int* __restrict__ positions,
                                    const float* __restrict__ inv_freq, int rot_dim, float sign, void* __restrict__ out,
                                    int out_dt, int H, int D, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int d = (int)(i % D);
  const long long t = i / ((long long)H * D);
  const int half = rot_dim / 2;
  float v = ld_dt(x, in_dt, i);
  if (d < rot_dim) {
    const int pr = d < half ? d : d - half;
    const float ang = sign * (float)positions[t] * inv_freq[pr];
    const float cs = cosf(ang), sn = sinf(ang);
    const float other = ld_dt(x, in_dt, d < half ? i + half : i - half);
    v = d < half ? v * cs - other * sn : v * cs + other * sn;
  }
  st_dt(out, out_dt, i, v);
}

// ------------------------------------------------------------------ RMS norm of a run of columns
// out[t, :] = rms(in[t, col0 .. col0 + n)) * w, the mean of squares taken over the n columns; one block per row.
__global__ void __launch_bounds__(SM_THREADS) cols_rmsnorm_kernel(const float* __restrict__ in, long long ld, int col0,
                                                                  int n, const float* __restrict__ w, float eps,
                                                                  void* __restrict__ out, int out_dt) {
  __shared__ float red[SM_THREADS / 32];
  const int t = blockIdx.x;
  const float* x = in + (size_t)t * ld + col0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += SM_THREADS) ss = fmaf(x[i], x[i], ss);
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += SM_THREADS) st_dt(out, out_dt, (size_t)t * n + i, x[i] * r * w[i]);
}

// ------------------------------------------------------------------ a small product per head
// x [T, H, K] (float32 or bfloat16), w [H, K, N] (float32 or bfloat16) -> out [T, H, N] = x[t, h, :] w[h]; with `gate` the head's
// output is multiplied by sigmoid(gate[t, gate0 + h]), or with `gate_each` element n of it by
// sigmoid(gate[t, gate0 + h N + n]).  A block takes HP_ROWS rows of one head, so a weight is read
// once for all of them; a thread owns output columns and sums over k in ascending order.
constexpr int HP_ROWS = 8;
constexpr int HP_THREADS = 128;

__global__ void __launch_bounds__(HP_THREADS) head_project_kernel(const void* __restrict__ x, int x_dt,
                                                                  const void* __restrict__ w, int w_dt, const float* __restrict__ gate,
                                                                  long long gate_ld, int gate0, void* __restrict__ out,
                                                                  int out_dt, int T, int H, int K, int N, int gate_each) {
  extern __shared__ float xs[];      // HP_ROWS * K
  const int t0 = blockIdx.x * HP_ROWS, h = blockIdx.y;
  const int rows = min(HP_ROWS, T - t0);
  for (int i = threadIdx.x; i < HP_ROWS * K; i += HP_THREADS) {
    const int r = i / K, k = i % K;
    xs[i] = r < rows ? ld_dt(x, x_dt, ((size_t)(t0 + r) * H + h) * K + k) : 0.f;
  }
  __syncthreads();
  float g[HP_ROWS];
#pragma unroll
  for (int r = 0; r < HP_ROWS; ++r)
    g[r] = gate && !gate_each && r < rows ? sigmoidf_(gate[(size_t)(t0 + r) * gate_ld + gate0 + h]) : 1.f;
  for (int n = threadIdx.x; n < N; n += HP_THREADS) {
    if (gate && gate_each) {
#pragma unroll
      for (int r = 0; r < HP_ROWS; ++r)
        g[r] = r < rows ? sigmoidf_(gate[(size_t)(t0 + r) * gate_ld + gate0 + (size_t)h * N + n]) : 1.f;
    }
    float acc[HP_ROWS];
#pragma unroll
    for (int r = 0; r < HP_ROWS; ++r) acc[r] = 0.f;
    for (int k = 0; k < K; ++k) {
      const float wv = ld_dt(w, w_dt, ((size_t)h * K + k) * N + n);
#pragma unroll
      for (int r = 0; r < HP_ROWS; ++r) acc[r] = fmaf(xs[r * K + k], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < HP_ROWS; ++r)
      if (r < rows) st_dt(out, out_dt, ((size_t)(t0 + r) * H + h) * N + n, acc[r] * g[r]);
  }
}

// out[t, h, :] = x[t, h, :] * sigmoid(gate[t, gate0 + h]): the gate alone, for head outputs that another product made.
__global__ void head_gate_kernel(const float* __restrict__ x, const float* __restrict__ gate, long long gate_ld, int gate0,
                                 void* __restrict__ out, int out_dt, long long total, int H, int N, int gate_each) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long th = i / N;
  const long long t = th / H;
  const int h = (int)(th - t * H);
  const long long col = gate_each ? (long long)h * N + (i - th * N) : h;     // a gate per element, or one per head
  st_dt(out, out_dt, (size_t)i, x[i] * sigmoidf_(gate[t * gate_ld + gate0 + col]));
}

// The same for few rows (a decode step): a block takes HP_ROWS rows, one head and 32 output columns, its four warps
// share out k in quarters (each sums its quarter in ascending order, several loads in flight) and the quarters are
// added in ascending order through shared memory.
constexpr int HP_FEW_COLS = 32;

__global__ void __launch_bounds__(HP_THREADS) head_project_few_kernel(const void* __restrict__ x, int x_dt,
                                                                      const void* __restrict__ w, int w_dt,
                                                                      const float* __restrict__ gate, long long gate_ld,
                                                                      int gate0, void* __restrict__ out, int out_dt, int T,
                                                                      int H, int K, int N, int gate_each) {
  extern __shared__ float xs[];      // HP_ROWS * K, then [4][HP_ROWS][HP_FEW_COLS] partial sums
  float* part = xs + (size_t)HP_ROWS * K;
  const int t0 = blockIdx.x * HP_ROWS, h = blockIdx.y;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int n = blockIdx.z * HP_FEW_COLS + lane;
  const int rows = min(HP_ROWS, T - t0);
  for (int i = threadIdx.x; i < HP_ROWS * K; i += HP_THREADS) {
    const int r = i / K, k = i % K;
    xs[i] = r < rows ? ld_dt(x, x_dt, ((size_t)(t0 + r) * H + h) * K + k) : 0.f;
  }
  __syncthreads();
  float acc[HP_ROWS];
#pragma unroll
  for (int r = 0; r < HP_ROWS; ++r) acc[r] = 0.f;
  if (n < N) {
    const int kq = (K + 3) / 4, k0 = warp * kq, k1 = min(K, k0 + kq);
#pragma unroll 8
    for (int k = k0; k < k1; ++k) {
      const float wv = ld_dt(w, w_dt, ((size_t)h * K + k) * N + n);
#pragma unroll
      for (int r = 0; r < HP_ROWS; ++r) acc[r] = fmaf(xs[r * K + k], wv, acc[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < HP_ROWS; ++r) part[(warp * HP_ROWS + r) * HP_FEW_COLS + lane] = acc[r];
  __syncthreads();
  for (int i = threadIdx.x; i < HP_ROWS * HP_FEW_COLS; i += HP_THREADS) {
    const int r = i / HP_FEW_COLS, c = i % HP_FEW_COLS, nn = blockIdx.z * HP_FEW_COLS + c;
    if (r < rows && nn < N) {
      float sum = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) sum += part[(q * HP_ROWS + r) * HP_FEW_COLS + c];
      const float g = gate ? sigmoidf_(gate[(size_t)(t0 + r) * gate_ld + gate0 + (gate_each ? (size_t)h * N + nn : (size_t)h)]) : 1.f;
      st_dt(out, out_dt, ((size_t)(t0 + r) * H + h) * N + nn, sum * g);
    }
  }
}

// ------------------------------------------------------------------ the same memories, a column per thread
// A column of the head's matrix (its dk rows) stays in one thread's registers while the entry's rows run: the
// columns of either recurrence never meet, so a row costs one barrier (for q and k of the row, staged in shared
// memory through a ring of asynchronous copies) and a few exchanges between the neighbouring lanes that hold the
// column's rows, thirty-two each, four at a time in turn (so that their reads of q and k in shared memory lie side
// by side: with a lane's rows in one stretch every such read was a four-way bank conflict, and a step of eight
// prompts took 5.4 instead of 1.6 ms).  A block is two warps with sixteen to sixty-four columns; blocks along z share a head's columns, so a single sequence fills more multiprocessors and a
// decode step's read of the states is spread over them.  The matrix LSTM's normaliser is one more column (whose
// value is 1), and its product with q one more output.  What needs a whole head, the division by the normaliser,
// the head's RMS norm and the output gate, follows in head_finish_kernel, a row and head per warp.
// raw: [T, H, RW] float32, RW = dv (+ 2 for the matrix LSTM: n . q and the running maximum m behind the dv sums).
constexpr int COL_THREADS = 64;
constexpr int COL_ROWS = 32;                           // rows of a column that one thread holds: DK / 32 lanes share a column


struct ColArgs {
  const int* cu_rows;
  const int* entry_slot;
  float* S;                 // [slots][H, dk, dv]
  long long S_stride;
  float* n;                 // matrix LSTM: [slots][H, dk]
  long long n_stride;
  float* m;                 // matrix LSTM: [slots][H]
  long long m_stride;
  const float* qk;          // rows that hold q and k: [T, qk_ld]
  long long qk_ld;
  int q0, k0, G;            // q/k head of value head h: h / (H / G)
  const float* vsrc;        // rows that hold v: [T, v_ld]
  long long v_ld;
  int v0;
  const void* gates;        // rows that hold the two per-head gate pre-activations: [T, gates_ld] float32
  int gates_dt;
  long long gates_ld;
  int ga0, gb0;             // matrix LSTM: i, f; delta rule: beta, decay
  const float* A_log;
  const float* dt_bias;
  float cap, q_scale;
  float* raw;
  int RW, H, dk, dv;
  int vec16;                // q and k can be copied sixteen bytes at a time (set by the launcher from the addresses)
  const float* dec;         // delta rule with channel decays (MODE 2): the decays themselves, [T, dec_ld], head h's at h * dk
  long long dec_ld;
};

// The gates of a row and head, ready for the recurrence: the matrix LSTM's capped log gates (i, f), or the delta
// rule's beta and decay.  For steps of many rows this runs over all rows at once before the scan (PRE), which then
// only reads them; a step of few rows computes them in the scan itself and saves the launch.
__device__ __forceinline__ void scan_gates(int mode, float ga, float gb, float cap, float rate, float dtb, float& x,
                                           float& y) {
  if (mode == 0) {
    x = cap * tanhf(ga / cap);
    y = logsigmoidf_(cap * tanhf(gb / cap));
  } else {
    x = sigmoidf_(ga);
    y = expf(-rate * softplusf_(gb + dtb));
  }
}

__global__ void scan_gates_kernel(const float* __restrict__ gates, long long ld, int ga0, int gb0, int H, int mode,
                                  float cap, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                  float* __restrict__ out, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long t = i / H;
  const int h = (int)(i % H);
  float x, y;
  scan_gates(mode, gates[t * ld + ga0 + h], gates[t * ld + gb0 + h], cap, mode ? expf(A_log[h]) : 0.f,
             mode ? dt_bias[h] : 0.f, x, y);
  out[2 * i] = x;
  out[2 * i + 1] = y;
}

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int COL_RING = 8;             // rows in flight: a row's q, k, v and gates are asked for this many rows ahead

// MODE 0: matrix LSTM, 1: gated delta rule, 2: delta rule with a decay per key channel (its decays come ready, a
// row of dk numbers per row and head, and ride in the ring beside q and k); PRE: the gates come ready
template <int DK, int MODE, bool PRE>
__global__ void __launch_bounds__(COL_THREADS) col_scan_kernel(ColArgs a) {
  // A ring of rows in shared memory, filled by asynchronous copies several rows ahead of the row that is computed:
  // with one row ahead every row waited for its loads' way through the memory system.
  __shared__ __align__(16) float qs[COL_RING][DK];
  __shared__ __align__(16) float ks[COL_RING][DK];
  constexpr int COL_RSPLIT = DK / COL_ROWS;          // lanes that share a column (1, 2 or 4)
  constexpr int COL_COLS = COL_THREADS / COL_RSPLIT; // columns of a block
  __shared__ float vs[COL_RING][COL_COLS];
  __shared__ float gs[COL_RING][2];
  __shared__ __align__(16) float ds[MODE == 2 ? COL_RING : 1][DK];
  constexpr int PER = DK / COL_THREADS > 0 ? DK / COL_THREADS : 1;
  constexpr int DKH = COL_ROWS;                      // rows of a column that one thread holds
  const int e = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int dk = a.dk, dv = a.dv;
  const int gh = h / (a.H / a.G);
  const int half = tid % COL_RSPLIT;                 // neighbouring lanes share a column, each a part of its rows
  const int cl = tid / COL_RSPLIT;                   // the column's place in the block
  const int c = blockIdx.z * COL_COLS + cl;
  // The lanes of a column take its rows four at a time in turn (lane `half` holds rows 4 (half + RSPLIT j) .. + 3,
  // j = 0, 1, ...): their 16-byte reads of q and k in shared memory then lie side by side, without bank conflicts.
  auto row_of = [&](int r) { return 4 * (half + COL_RSPLIT * (r / 4)) + (r % 4); };
  const int ncols = MODE == 0 ? dv + 1 : dv;
  const bool active = c < ncols;
  const bool is_n = MODE == 0 && c == dv;
  const int row0 = a.cu_rows[e], row1 = a.cu_rows[e + 1];
  const int slot = a.entry_slot[e];
  float* colp = nullptr;
  long long cstride = 0;
  if (active) {
    if (is_n) { colp = a.n + (size_t)slot * a.n_stride + (size_t)h * dk; cstride = 1; }
    else { colp = a.S + (size_t)slot * a.S_stride + (size_t)h * dk * dv + c; cstride = dv; }
  }
  float Sreg[DKH];
#pragma unroll
  for (int r = 0; r < DKH; ++r) Sreg[r] = (active && row_of(r) < dk) ? colp[(size_t)row_of(r) * cstride] : 0.f;
  float m = 0.f, rate = 0.f, dtb = 0.f;
  if (MODE == 0) m = a.m[(size_t)slot * a.m_stride + h];
  else if (MODE == 1) { rate = expf(a.A_log[h]); dtb = a.dt_bias[h]; }
  if (MODE == 2)
    for (int i = tid; i < COL_RING * DK; i += COL_THREADS)
      if (i % DK >= dk) ds[i / DK][i % DK] = 0.f;
  // what no copy ever writes: the rows of q and k beyond dk, the value of the normaliser's column and of no column
  for (int i = tid; i < COL_RING * DK; i += COL_THREADS)
    if (i % DK >= dk) { qs[i / DK][i % DK] = 0.f; ks[i / DK][i % DK] = 0.f; }
  if (half == 0 && !(active && !is_n))
    for (int i = 0; i < COL_RING; ++i) vs[i][cl] = 1.f;
  const float* gates = (const float*)a.gates;
  const bool has_v = active && !is_n && half == 0;
  // where this thread's copies of the next row to fetch come from; they move on by a row per fetch.  With
  // a.vec16 (every q and k head starts on a 16-byte boundary) a thread copies four floats at once: threads
  // 0 .. DK/4 - 1 the row's q, the next DK/4 its k; else one float at a time.
  constexpr int Q4 = DK / 4;                         // 16-byte pieces of a head's q (or k)
  const bool k_side = tid >= Q4;
  const int piece = k_side ? tid - Q4 : tid;         // (with vec16)
  const float* src_q = a.qk + (size_t)row0 * a.qk_ld + a.q0 + gh * dk + tid;
  const float* src_k = a.qk + (size_t)row0 * a.qk_ld + a.k0 + gh * dk + tid;
  const float* src_16 = a.qk + (size_t)row0 * a.qk_ld + (k_side ? a.k0 : a.q0) + gh * dk + 4 * piece;
  const bool does_16 = a.vec16 && tid < 2 * Q4 && 4 * piece < dk;
  const float* src_v = a.vsrc + (size_t)row0 * a.v_ld + a.v0 + h * dv + (has_v ? c : 0);
  const float* src_g = gates + (size_t)row0 * a.gates_ld + (tid == 1 ? a.gb0 : a.ga0) + (PRE ? 2 * h : h);
  const float* src_d = MODE == 2 ? a.dec + (size_t)row0 * a.dec_ld + (size_t)h * dk + (a.vec16 ? 4 * tid : tid) : nullptr;
  const bool d_16 = MODE == 2 && a.vec16 && tid < Q4 && 4 * tid < dk;
  int fetch_slot = 0;
  auto fetch = [&](int t) {
    if (t < row1) {
      const int b = fetch_slot;
      if (a.vec16) {
        if (does_16) cp_async16((k_side ? ks[b] : qs[b]) + 4 * piece, src_16);
        if (d_16) cp_async16(ds[b] + 4 * tid, src_d);
      } else {
        if (MODE == 2) {
#pragma unroll
          for (int i = 0; i < PER; ++i) {
            const int r = tid + i * COL_THREADS;
            if (r < dk && r < DK) cp_async4(&ds[b][r], src_d + i * COL_THREADS);
          }
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          const int r = tid + i * COL_THREADS;
          if (r < dk && r < DK) {
            cp_async4(&qs[b][r], src_q + i * COL_THREADS);
            cp_async4(&ks[b][r], src_k + i * COL_THREADS);
          }
        }
      }
      if (has_v) cp_async4(&vs[b][cl], src_v);
      if (tid < 2) cp_async4(&gs[b][tid], src_g);
      src_q += a.qk_ld; src_k += a.qk_ld; src_16 += a.qk_ld; src_v += a.v_ld; src_g += a.gates_ld;
      if (MODE == 2) src_d += a.dec_ld;
      fetch_slot = (fetch_slot + 1) % COL_RING;
    }
    cp_async_commit();                               // (a group per row, also an empty one: the count below relies on it)
  };
  for (int j = 0; j < COL_RING - 1; ++j) fetch(row0 + j);
  float* out = a.raw + ((size_t)row0 * a.H + h) * a.RW;
  const size_t out_step = (size_t)a.H * a.RW;
  for (int t = row0; t < row1; ++t, out += out_step) {
    const int b = (t - row0) % COL_RING;
    cp_async_wait<COL_RING - 2>();                   // this thread's copies of row t have landed ...
    __syncthreads();                                 // ... and everyone's; and everyone is done with row t - 1,
    fetch(t + COL_RING - 1);                         // whose place in the ring the new row takes
    const float v = vs[b][cl], ga = gs[b][0], gb = gs[b][1];
    const float4* q4 = reinterpret_cast<const float4*>(qs[b]) + half;      // piece j of this lane: q4[RSPLIT * j]
    const float4* k4 = reinterpret_cast<const float4*>(ks[b]) + half;
    if (MODE == 0) {
      float ig = ga, fg = gb;
      if (!PRE) scan_gates(0, ga, gb, a.cap, 0.f, 0.f, ig, fg);
      const float m_new = fmaxf(fg + m, ig);
      const float fa = expf(fg + m - m_new), bv = expf(ig - m_new) * v;
      m = m_new;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;          // four chains; added up in a fixed order
#pragma unroll
      for (int r4 = 0; r4 < DKH / 4; ++r4) {
        const float4 qq = q4[COL_RSPLIT * r4], kk = k4[COL_RSPLIT * r4];
        float s;
        s = fmaf(fa, Sreg[4 * r4 + 0], kk.x * bv); Sreg[4 * r4 + 0] = s; a0 = fmaf(s, qq.x, a0);
        s = fmaf(fa, Sreg[4 * r4 + 1], kk.y * bv); Sreg[4 * r4 + 1] = s; a1 = fmaf(s, qq.y, a1);
        s = fmaf(fa, Sreg[4 * r4 + 2], kk.z * bv); Sreg[4 * r4 + 2] = s; a2 = fmaf(s, qq.z, a2);
        s = fmaf(fa, Sreg[4 * r4 + 3], kk.w * bv); Sreg[4 * r4 + 3] = s; a3 = fmaf(s, qq.w, a3);
      }
      float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
      for (int off = 1; off < COL_RSPLIT; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);   // same sum in every lane
      if (active && half == 0) out[c] = acc * a.q_scale;     // q's scale, taken out of the sum
      if (blockIdx.z == 0 && tid == 0) out[dv + 1] = m;
    } else if (MODE == 2) {
      // S_r <- g_r S_r;  u = beta (v - sum_r S_r k_r);  S_r += k_r u;  o = sum_r S_r q_r = sum_r (g_r S_r) q_r + (k . q) u
      const float beta = ga;
      const float4* d4 = reinterpret_cast<const float4*>(ds[b]) + half;
      float ak = 0.f, aq = 0.f, kq = 0.f, ak1 = 0.f, aq1 = 0.f, kq1 = 0.f;
#pragma unroll
      for (int r4 = 0; r4 < DKH / 4; ++r4) {
        const float4 qq = q4[COL_RSPLIT * r4], kk = k4[COL_RSPLIT * r4], dd = d4[COL_RSPLIT * r4];
        float x;
        x = dd.x * Sreg[4 * r4 + 0]; Sreg[4 * r4 + 0] = x; ak = fmaf(x, kk.x, ak); aq = fmaf(x, qq.x, aq); kq = fmaf(kk.x, qq.x, kq);
        x = dd.y * Sreg[4 * r4 + 1]; Sreg[4 * r4 + 1] = x; ak1 = fmaf(x, kk.y, ak1); aq1 = fmaf(x, qq.y, aq1); kq1 = fmaf(kk.y, qq.y, kq1);
        x = dd.z * Sreg[4 * r4 + 2]; Sreg[4 * r4 + 2] = x; ak = fmaf(x, kk.z, ak); aq = fmaf(x, qq.z, aq); kq = fmaf(kk.z, qq.z, kq);
        x = dd.w * Sreg[4 * r4 + 3]; Sreg[4 * r4 + 3] = x; ak1 = fmaf(x, kk.w, ak1); aq1 = fmaf(x, qq.w, aq1); kq1 = fmaf(kk.w, qq.w, kq1);
      }
      ak += ak1; aq += aq1; kq += kq1;
#pragma unroll
      for (int off = 1; off < COL_RSPLIT; off <<= 1) {
        ak += __shfl_xor_sync(0xffffffffu, ak, off);
        aq += __shfl_xor_sync(0xffffffffu, aq, off);
        kq += __shfl_xor_sync(0xffffffffu, kq, off);
      }
      const float u = beta * (v - ak);
      if (active && half == 0) out[c] = fmaf(kq, u, aq) * a.q_scale;
#pragma unroll
      for (int r4 = 0; r4 < DKH / 4; ++r4) {
        const float4 kk = k4[COL_RSPLIT * r4];
        Sreg[4 * r4 + 0] = fmaf(kk.x, u, Sreg[4 * r4 + 0]);
        Sreg[4 * r4 + 1] = fmaf(kk.y, u, Sreg[4 * r4 + 1]);
        Sreg[4 * r4 + 2] = fmaf(kk.z, u, Sreg[4 * r4 + 2]);
        Sreg[4 * r4 + 3] = fmaf(kk.w, u, Sreg[4 * r4 + 3]);
      }
    } else {
      float beta = ga, g = gb;
      if (!PRE) scan_gates(1, ga, gb, 0.f, rate, dtb, beta, g);
      float ak = 0.f, aq = 0.f, kq = 0.f, ak1 = 0.f, aq1 = 0.f, kq1 = 0.f;     // two chains each
#pragma unroll
      for (int r4 = 0; r4 < DKH / 4; ++r4) {
        const float4 qq = q4[COL_RSPLIT * r4], kk = k4[COL_RSPLIT * r4];
        ak = fmaf(Sreg[4 * r4 + 0], kk.x, ak); aq = fmaf(Sreg[4 * r4 + 0], qq.x, aq); kq = fmaf(kk.x, qq.x, kq);
        ak1 = fmaf(Sreg[4 * r4 + 1], kk.y, ak1); aq1 = fmaf(Sreg[4 * r4 + 1], qq.y, aq1); kq1 = fmaf(kk.y, qq.y, kq1);
        ak = fmaf(Sreg[4 * r4 + 2], kk.z, ak); aq = fmaf(Sreg[4 * r4 + 2], qq.z, aq); kq = fmaf(kk.z, qq.z, kq);
        ak1 = fmaf(Sreg[4 * r4 + 3], kk.w, ak1); aq1 = fmaf(Sreg[4 * r4 + 3], qq.w, aq1); kq1 = fmaf(kk.w, qq.w, kq1);
      }
      ak += ak1; aq += aq1; kq += kq1;
#pragma unroll
      for (int off = 1; off < COL_RSPLIT; off <<= 1) {       // the column's lanes all get the same sums
        ak += __shfl_xor_sync(0xffffffffu, ak, off);
        aq += __shfl_xor_sync(0xffffffffu, aq, off);
        kq += __shfl_xor_sync(0xffffffffu, kq, off);
      }
      const float u = beta * (v - g * ak);
      if (active && half == 0) out[c] = fmaf(kq, u, g * aq) * a.q_scale;
#pragma unroll
      for (int r4 = 0; r4 < DKH / 4; ++r4) {
        const float4 kk = k4[COL_RSPLIT * r4];
        Sreg[4 * r4 + 0] = fmaf(g, Sreg[4 * r4 + 0], kk.x * u);
        Sreg[4 * r4 + 1] = fmaf(g, Sreg[4 * r4 + 1], kk.y * u);
        Sreg[4 * r4 + 2] = fmaf(g, Sreg[4 * r4 + 2], kk.z * u);
        Sreg[4 * r4 + 3] = fmaf(g, Sreg[4 * r4 + 3], kk.w * u);
      }
    }
  }
  cp_async_wait<0>();
  if (active) {
#pragma unroll
    for (int r = 0; r < DKH; ++r)
      if (row_of(r) < dk) colp[(size_t)row_of(r) * cstride] = Sreg[r];
  }
  if (MODE == 0 && blockIdx.z == 0 && tid == 0) a.m[(size_t)slot * a.m_stride + h] = m;
}

// A row and head per warp: o = raw (divided, for the matrix LSTM, by max(|n . q|, exp(-m)) + den_eps), then
// o / sqrt(mean(o^2) + eps) * w * act(gate), act the sigmoid (gate_act 0) or silu (1).
__global__ void __launch_bounds__(256) head_finish_kernel(const float* __restrict__ raw, int RW, int has_den,
                                                          float den_eps, const void* __restrict__ gate, int gate_dt,
                                                          long long gate_ld, int g0, int gate_act,
                                                          const float* __restrict__ w, int w_per_head, float eps,
                                                          void* __restrict__ out, int out_dt, int T, int H, int dv) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)T * H) return;
  const int t = (int)(item / H), h = (int)(item % H);
  const float* x = raw + (size_t)item * RW;
  float inv = 1.f;
  if (has_den) inv = 1.f / (fmaxf(fabsf(x[dv]), expf(-x[dv + 1])) + den_eps);
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) { const float o = x[i] * inv; ss = fmaf(o, o, ss); }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)dv + eps);
  for (int i = lane; i < dv; i += 32) {
    const float gv = ld_dt(gate, gate_dt, (size_t)t * gate_ld + g0 + h * dv + i);
    const float act = gate_act == 0 ? sigmoidf_(gv) : siluf_(gv);
    st_dt(out, out_dt, (size_t)t * H * dv + (size_t)h * dv + i, x[i] * inv * r * w[w_per_head ? h * dv + i : i] * act);
  }
}

// Before the scan with channel decays: decays[t, h dk + r] = exp(-exp(A_log[h]) softplus(pre[t, dec0 + h dk + r] +
// dt_bias[h dk + r])) and gates[t, h] = (sigmoid(beta's pre-activation), 1), all float32.
__global__ void channel_gates_kernel(const float* __restrict__ pre, long long pre_ld, int dec0,
                                     const void* __restrict__ proj, int proj_dt, long long proj_ld, int b0,
                                     const float* __restrict__ A_log, const float* __restrict__ dt_bias, int H, int dk,
                                     float* __restrict__ decays, float* __restrict__ gates, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int hd = H * dk;
  const long long t = i / hd;
  const int c = (int)(i % hd), h = c / dk;
  decays[i] = expf(-expf(A_log[h]) * softplusf_(pre[t * pre_ld + dec0 + c] + dt_bias[c]));
  if (c % dk == 0) {
    gates[2 * (t * H + h)] = sigmoidf_(ld_dt(proj, proj_dt, (size_t)t * proj_ld + b0 + h));
    gates[2 * (t * H + h) + 1] = 1.f;
  }
}

// Steps of more rows than this compute their gates in a pass of their own before the scan.
constexpr int SCAN_GATES_APART_ROWS = 64;

// `gate_buf`: [T, H, 2] float32 scratch for the gates (may be null for steps of few rows).
template <int MODE, bool PRE>
int launch_col_scan_p(const ColArgs& a, int S, cudaStream_t s) {
  const int ncols = MODE == 0 ? a.dv + 1 : a.dv;
  const int DKp = a.dk <= 32 ? 32 : (a.dk <= 64 ? 64 : 128);
  const int cols = COL_THREADS / (DKp / COL_ROWS);   // columns of a block
  dim3 grid(S, a.H, (ncols + cols - 1) / cols);
  if (a.dk <= 32) col_scan_kernel<32, MODE, PRE><<<grid, COL_THREADS, 0, s>>>(a);
  else if (a.dk <= 64) col_scan_kernel<64, MODE, PRE><<<grid, COL_THREADS, 0, s>>>(a);
  else if (a.dk <= 128) col_scan_kernel<128, MODE, PRE><<<grid, COL_THREADS, 0, s>>>(a);
  else return NV_ERR_UNSUPPORTED;
  NV_RETURN_LAST();
}

template <int MODE>
int launch_col_scan(ColArgs a, int S, int T, float* gate_buf, cudaStream_t s) {
  // sixteen-byte copies: every row's q and k heads start on 16-byte boundaries and a head is whole pieces
  a.vec16 = (((uintptr_t)a.qk & 15) == 0 && a.qk_ld % 4 == 0 && a.q0 % 4 == 0 && a.k0 % 4 == 0 && a.dk % 4 == 0) ? 1 : 0;
  if (T > SCAN_GATES_APART_ROWS && gate_buf) {
    const long long n = (long long)T * a.H;
    scan_gates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>((const float*)a.gates, a.gates_ld, a.ga0, a.gb0, a.H,
                                                                 MODE, a.cap, a.A_log, a.dt_bias, gate_buf, n);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    a.gates = gate_buf; a.gates_ld = 2LL * a.H; a.ga0 = 0; a.gb0 = 1;
    return launch_col_scan_p<MODE, true>(a, S, s);
  }
  return launch_col_scan_p<MODE, false>(a, S, s);
}

size_t scan_smem(int dk, int dv, int parts) {
  const int RS = std::max(1, std::min(SM_THREADS / dv, dk));
  return sizeof(float) * ((size_t)dk * dv + 3 * (size_t)dk + (size_t)(2 + parts) * dv + (size_t)parts * RS * dv + 8);
}

template <typename K>
int allow_smem(K kernel, size_t bytes) {
  if (bytes > 227 * 1024) return NV_ERR_UNSUPPORTED;
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return NV_OK;
}

}  // namespace

NV_API int nv_branch_norm_add(float* x, const float* b0, const float* b1, const float* b2, const float* b3,
                              const float* w0, const float* w1, const float* w2, const float* w3, int nb,
                              float mix_scale, const float* w, float eps, void* out, int out_dt, int T, int H,
                              const float* rows, const int* index, const float* weight, int R, const float* dense,
                              const float* gate_logit, long long gate_ld, const float* next_w, float next_eps,
                              float* out32, cudaStream_t s) {
  if (nb < 0 || nb > MAX_BRANCHES || H <= 0 || R < 0) return NV_ERR_BAD_SIZE;
  if ((R > 0 || dense) && nb > 0) return NV_ERR_BAD_SIZE;
  if (R > 0 && (!rows || !index || !weight)) return NV_ERR_BAD_SIZE;
  if (out && !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (T == 0) return NV_OK;
  BranchArgs a;
  a.x = x;
  const float* br[4] = {b0, b1, b2, b3};
  const float* bw[4] = {w0, w1, w2, w3};
  for (int i = 0; i < MAX_BRANCHES; ++i) { a.br[i] = br[i]; a.bw[i] = bw[i]; }
  for (int i = 0; i < nb; ++i) {
    if (!br[i]) return NV_ERR_BAD_SIZE;
    if ((bw[i] != nullptr) != (bw[0] != nullptr)) return NV_ERR_BAD_SIZE;
  }
  if (nb > 1 && !bw[0]) return NV_ERR_BAD_SIZE;
  if ((nb > 0 || R > 0 || dense) && !w) return NV_ERR_BAD_SIZE;
  a.rows = rows; a.index = index; a.weight = weight; a.R = R; a.dense = dense; a.gate_logit = gate_logit;
  a.gate_ld = gate_ld; a.next_w = next_w; a.next_eps = next_eps; a.out32 = out32;
  a.w = w; a.out = out; a.nb = nb; a.H = H; a.out_dt = out_dt; a.eps = eps; a.mix_scale = mix_scale;
  const size_t smem = sizeof(float) * (size_t)H;
  int rc = allow_smem(branch_norm_add_kernel, smem);
  if (rc) return rc;
  branch_norm_add_kernel<<<T, SM_THREADS, smem, s>>>(a);
  NV_RETURN_LAST();
}

NV_API int nv_activation(const void* in, int in_dt, void* out, int out_dt, long long n, int kind, float p0, float p1,
                         cudaStream_t s) {
  if (!dt_ok(in_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (kind < 0 || kind > 4) return NV_ERR_UNSUPPORTED;
  if (n == 0) return NV_OK;
  if (in_dt == NV_DT_F32 && out_dt == NV_DT_BF16 && n % 4 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 7) == 0) {
    const long long n4 = n / 4;
    activation_f32_bf16_x4_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, s>>>((const float4*)in, (uint2*)out, n4, kind, p0, p1);
    NV_RETURN_LAST();
  }
  activation_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(in, in_dt, out, out_dt, n, kind, p0, p1);
  NV_RETURN_LAST();
}

NV_API int nv_token_gate(const void* gate, int gate_dt, long long gate_ld, const int* ids, const int* feed,
                         const void* table, int table_dt, long long table_ld, int col0, int d, int V, void* out,
                         int out_dt, int T, int* err, cudaStream_t s) {
  if (!dt_ok(gate_dt) || !dt_ok(table_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (d <= 0 || col0 < 0 || col0 + d > table_ld) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  token_gate_kernel<<<T, 128, 0, s>>>(gate, gate_dt, gate_ld, ids, feed, table, table_dt, table_ld, col0, d, V, out,
                                      out_dt, err);
  NV_RETURN_LAST();
}

NV_API int nv_conv_silu_norm(const void* in, int in_dt, long long ld, int col0, int C, const float* w, int taps,
                             const int* row_entry, const int* cu_rows, const int* entry_slot, const float* state,
                             long long slot_stride, int unit_heads, int unit_dim, float unit_eps, int scaled_heads,
                             float scale, float* out, int T, cudaStream_t s) {
  if (!dt_ok(in_dt)) return NV_ERR_BAD_DTYPE;
  if (C <= 0 || taps < 1 || unit_heads < 0 || unit_heads * unit_dim > C || scaled_heads > unit_heads) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  const size_t smem = sizeof(float) * (size_t)C;
  int rc = allow_smem(conv_silu_norm_kernel, smem);
  if (rc) return rc;
  conv_silu_norm_kernel<<<T, SM_THREADS, smem, s>>>(in, in_dt, ld, col0, C, w, taps, row_entry, cu_rows, entry_slot,
                                                    state, slot_stride, unit_heads, unit_dim, unit_eps, scaled_heads,
                                                    scale, out);
  NV_RETURN_LAST();
}

NV_API int nv_conv_state_update(const void* in, int in_dt, long long ld, int col0, int C, int taps,
                                const int* cu_rows, const int* entry_slot, float* state, long long slot_stride,
                                int S, cudaStream_t s) {
  if (!dt_ok(in_dt)) return NV_ERR_BAD_DTYPE;
  if (C <= 0 || taps < 1) return NV_ERR_BAD_SIZE;
  if (S == 0 || taps == 1) return NV_OK;
  conv_state_update_kernel<<<S, SM_THREADS, 0, s>>>(in, in_dt, ld, col0, C, taps, cu_rows, entry_slot, state,
                                                    slot_stride);
  NV_RETURN_LAST();
}

NV_API int nv_scan_usable(int dk, int dv, int parts) {
  return dk >= 1 && dv >= 1 && dv <= SM_THREADS && scan_smem(dk, dv, parts) <= 227 * 1024;
}

NV_API int nv_mlstm_scan(const float* proj, long long ld, int q0, int k0, int v0, int g0, int i0, int f0,
                         const int* cu_rows, const int* entry_slot, float* S, long long S_stride, float* n,
                         long long n_stride, float* m, long long m_stride, int H, int dk, int dv, float cap,
                         float q_scale, float den_eps, float eps, const float* norm_w, int norm_per_head, void* out,
                         int out_dt, int num_entries, cudaStream_t s) {
  if (!dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (!nv_scan_usable(dk, dv, 1) || H <= 0) return NV_ERR_UNSUPPORTED;
  if (num_entries == 0) return NV_OK;
  MlstmArgs a;
  a.c = {cu_rows, entry_slot, S, S_stride, norm_w, out, out_dt, H, dk, dv, eps};
  a.proj = proj; a.ld = ld; a.q0 = q0; a.k0 = k0; a.v0 = v0; a.g0 = g0; a.i0 = i0; a.f0 = f0;
  a.n = n; a.n_stride = n_stride; a.m = m; a.m_stride = m_stride;
  a.cap = cap; a.q_scale = q_scale; a.den_eps = den_eps; a.norm_per_head = norm_per_head;
  const size_t smem = scan_smem(dk, dv, 1);
  int rc = allow_smem(mlstm_scan_kernel, smem);
  if (rc) return rc;
  mlstm_scan_kernel<<<dim3(num_entries, H), SM_THREADS, smem, s>>>(a);
  NV_RETURN_LAST();
}

NV_API int nv_gated_delta_scan(const float* qkv, int C, int q0, int k0, int v0, int G, const void* proj, int proj_dt,
                               long long ld, int g0, int b0, int a0, const float* A_log, const float* dt_bias,
                               const int* cu_rows, const int* entry_slot, float* S, long long S_stride, int H, int dk,
                               int dv, float eps, const float* norm_w, void* out, int out_dt, int num_entries,
                               const float* dec, long long dec_ld, int dec0, const void* gsrc, int gsrc_dt,
                               long long gsrc_ld, int decay_mode, int gate_mode, cudaStream_t s) {
  if (!dt_ok(out_dt) || !dt_ok(proj_dt)) return NV_ERR_BAD_DTYPE;
  if (!nv_scan_usable(dk, dv, 2) || H <= 0 || G <= 0 || H % G) return NV_ERR_UNSUPPORTED;
  if (decay_mode < 0 || decay_mode > 1 || gate_mode < 0 || gate_mode > 1 || (decay_mode == 1 && !dec)) return NV_ERR_BAD_SIZE;
  if (gsrc && !dt_ok(gsrc_dt)) return NV_ERR_BAD_DTYPE;
  if (num_entries == 0) return NV_OK;
  DeltaArgs a;
  a.c = {cu_rows, entry_slot, S, S_stride, norm_w, out, out_dt, H, dk, dv, eps};
  a.qkv = qkv; a.C = C; a.q0 = q0; a.k0 = k0; a.v0 = v0; a.G = G;
  a.proj = proj; a.proj_dt = proj_dt; a.ld = ld; a.g0 = g0; a.b0 = b0; a.a0 = a0;
  a.A_log = A_log; a.dt_bias = dt_bias;
  a.dec = dec; a.dec_ld = dec_ld; a.dec0 = dec0;
  a.gsrc = gsrc ? gsrc : proj; a.gsrc_dt = gsrc ? gsrc_dt : proj_dt; a.gsrc_ld = gsrc ? gsrc_ld : ld;
  a.decay_mode = decay_mode; a.gate_mode = gate_mode;
  const size_t smem = scan_smem(dk, dv, 2);
  int rc = allow_smem(gated_delta_scan_kernel, smem);
  if (rc) return rc;
  gated_delta_scan_kernel<<<dim3(num_entries, H), SM_THREADS, smem, s>>>(a);
  NV_RETURN_LAST();
}

NV_API int nv_qk_prepare_store(const void* in, int in_dt, long long ld, int q0, int k0, int v0, const int* positions,
                               const int* row_entry, const int* block_table, int max_blocks, const float* qw,
                               const float* kw, float eps, const float* inv_freq, int rot_dim, int interleaved,
                               float amplitude, void* q_out, int q_dt, void* kc, void* vc, int cache_dt, int Hq,
                               int Hkv, int D, int Dv, int page, int write_kv, int* err, int T, int QP, int KP,
                               int VP, const float* v_inv_freq, int v_rot_dim, int rot0, int k_norm_dim,
                               int norm_mode, cudaStream_t s) {
  if (!dt_ok(in_dt) || !dt_ok(q_dt) || !dt_ok(cache_dt)) return NV_ERR_BAD_DTYPE;
  if (rot_dim < 0 || rot0 < 0 || rot0 + rot_dim > D || rot_dim % 2 || D <= 0 || Dv <= 0) return NV_ERR_BAD_SIZE;
  if (k_norm_dim < 0 || k_norm_dim > D || norm_mode < 0 || norm_mode > 3) return NV_ERR_BAD_SIZE;
  if (v_rot_dim < 0 || v_rot_dim > Dv || v_rot_dim % 2 || (v_rot_dim && !v_inv_freq)) return NV_ERR_BAD_SIZE;
  if (QP < D || KP < D || VP < Dv) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  QkArgs a = {in, in_dt, ld, q0, k0, v0, positions, row_entry, block_table, max_blocks, qw, kw, eps, inv_freq, rot_dim,
              interleaved, amplitude, q_out, q_dt, kc, vc, cache_dt, Hq, Hkv, D, Dv, page, write_kv, err, QP, KP, VP,
              rot0, k_norm_dim, norm_mode, v_inv_freq, v_rot_dim};
  const size_t smem = sizeof(float) * (size_t)(QK_THREADS / 32) * D;
  int rc = allow_smem(qk_prepare_store_kernel, smem);
  if (rc) return rc;
  qk_prepare_store_kernel<<<T, QK_THREADS, smem, s>>>(a);
  NV_RETURN_LAST();
}

NV_API int nv_paged_attention_general(const void* q, int q_dt, const void* kc, const void* vc, int cache_dt,
                                      const int* block_table, int max_blocks, const int* row_entry,
                                      const int* positions, float scale, int window, int keep_first, int has_sink,
                                      float sink_score, const float* sinks, void* out, int out_dt, int T, int Hq,
                                      int Hkv, int Hv, int D, int Dv, int key_span, int page, float softcap,
                                      cudaStream_t s) {
  if (!dt_ok(q_dt) || !dt_ok(cache_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (D <= 0 || Dv <= 0 || Dv > ATTG_NV * ATTG_THREADS || Hkv <= 0 || Hv <= 0 || Hq % Hv || keep_first < 0)
    return NV_ERR_UNSUPPORTED;
  if (key_span < 1 || (key_span == 1 && Hq % Hkv) || (key_span > 1 && key_span != Hkv)) return NV_ERR_UNSUPPORTED;
  if (T == 0) return NV_OK;
  const size_t smem = sizeof(float) * (size_t)key_span * D;
  int rc = allow_smem(paged_attention_general_kernel, smem);
  if (rc) return rc;
  paged_attention_general_kernel<<<dim3(T, Hq), ATTG_THREADS, smem, s>>>(
      q, q_dt, kc, vc, cache_dt, block_table, max_blocks, row_entry, positions, scale, window, keep_first, has_sink,
      sink_score, sinks, out, out_dt, Hq, Hkv, Hv, D, Dv, key_span, page, softcap);
  NV_RETURN_LAST();
}

NV_API int nv_mix_query_heads(const float* q, const float* mix, void* out, int out_dt, int T, int H, int G, int D,
                              cudaStream_t s) {
  if (!dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (H <= 0 || G <= 0 || H % G || D <= 0) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  const size_t smem = sizeof(float) * ((size_t)H * D + (size_t)H * H);
  int rc = allow_smem(mix_query_heads_kernel, smem);
  if (rc) return rc;
  mix_query_heads_kernel<<<T, 256, smem, s>>>(q, mix, out, out_dt, H, G, D);
  NV_RETURN_LAST();
}

NV_API int nv_rotate_heads(const void* x, int in_dt, const int* positions, const float* inv_freq, int rot_dim,
                           float sign, void* out, int out_dt, int T, int H, int D, cudaStream_t s) {
  if (!dt_ok(in_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (rot_dim < 0 || rot_dim > D || rot_dim % 2 || H <= 0 || x == out) return NV_ERR_BAD_SIZE;
  const long long total = (long long)T * H * D;
  if (total == 0) return NV_OK;
  rotate_heads_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(x, in_dt, positions, inv_freq, rot_dim, sign, out,
                                                                      out_dt, H, D, total);
  NV_RETURN_LAST();
}

NV_API int nv_cols_rmsnorm(const float* in, long long ld, int col0, int n, const float* w, float eps, void* out,
                           int out_dt, int T, cudaStream_t s) {
  if (!dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (n <= 0 || col0 < 0 || col0 + n > ld) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  cols_rmsnorm_kernel<<<T, SM_THREADS, 0, s>>>(in, ld, col0, n, w, eps, out, out_dt);
  NV_RETURN_LAST();
}

NV_API int nv_head_project(const void* x, int x_dt, const void* w, int w_dt, const float* gate, long long gate_ld, int gate0,
                           void* out, int out_dt, int T, int H, int K, int N, int gate_each, cudaStream_t s) {
  if (!dt_ok(x_dt) || !dt_ok(w_dt) || !dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (H <= 0 || K <= 0 || N <= 0) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  if (T <= 8 * HP_ROWS) {            // few rows: more blocks, each with a shorter chain of sums
    const size_t few = sizeof(float) * ((size_t)HP_ROWS * K + 4 * HP_ROWS * HP_FEW_COLS);
    int rc = allow_smem(head_project_few_kernel, few);
    if (rc) return rc;
    head_project_few_kernel<<<dim3((T + HP_ROWS - 1) / HP_ROWS, H, (N + HP_FEW_COLS - 1) / HP_FEW_COLS), HP_THREADS, few, s>>>(
        x, x_dt, w, w_dt, gate, gate_ld, gate0, out, out_dt, T, H, K, N, gate_each);
    NV_RETURN_LAST();
  }
  const size_t smem = sizeof(float) * (size_t)HP_ROWS * K;
  int rc = allow_smem(head_project_kernel, smem);
  if (rc) return rc;
  head_project_kernel<<<dim3((T + HP_ROWS - 1) / HP_ROWS, H), HP_THREADS, smem, s>>>(x, x_dt, w, w_dt, gate, gate_ld, gate0,
                                                                                     out, out_dt, T, H, K, N, gate_each);
  NV_RETURN_LAST();
}

NV_API int nv_head_gate(const float* x, const float* gate, long long gate_ld, int gate0, void* out, int out_dt, int T,
                        int H, int N, int gate_each, cudaStream_t s) {
  if (!dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (H <= 0 || N <= 0) return NV_ERR_BAD_SIZE;
  if (T == 0) return NV_OK;
  const long long total = (long long)T * H * N;
  head_gate_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(x, gate, gate_ld, gate0, out, out_dt, total, H, N, gate_each);
  NV_RETURN_LAST();
}

NV_API int nv_col_scan_usable(int dk, int dv) { return dk >= 1 && dk <= 128 && dv >= 1; }
NV_API int nv_channel_scan_usable(int dk, int dv) { return nv_col_scan_usable(dk, dv); }

// The matrix LSTM through col_scan_kernel; raw: [T, H, dv + 2] and gate_buf: [T, H, 2] float32 scratch.
NV_API int nv_mlstm_col_scan(const float* proj, long long ld, int q0, int k0, int v0, int g0, int i0, int f0,
                             const int* cu_rows, const int* entry_slot, float* S, long long S_stride, float* n,
                             long long n_stride, float* m, long long m_stride, int H, int dk, int dv, float cap,
                             float q_scale, float den_eps, float eps, const float* norm_w, int norm_per_head,
                             float* raw, float* gate_buf, void* out, int out_dt, int num_entries, int T,
                             cudaStream_t s) {
  if (!dt_ok(out_dt)) return NV_ERR_BAD_DTYPE;
  if (!nv_col_scan_usable(dk, dv) || H <= 0) return NV_ERR_UNSUPPORTED;
  if (num_entries == 0 || T == 0) return NV_OK;
  ColArgs a = {};
  a.cu_rows = cu_rows; a.entry_slot = entry_slot; a.S = S; a.S_stride = S_stride; a.n = n; a.n_stride = n_stride;
  a.m = m; a.m_stride = m_stride; a.qk = proj; a.qk_ld = ld; a.q0 = q0; a.k0 = k0; a.G = H; a.vsrc = proj; a.v_ld = ld;
  a.v0 = v0; a.gates = proj; a.gates_dt = NV_DT_F32; a.gates_ld = ld; a.ga0 = i0; a.gb0 = f0; a.cap = cap;
  a.q_scale = q_scale; a.raw = raw; a.RW = dv + 2; a.H = H; a.dk = dk; a.dv = dv;
  int rc = launch_col_scan<0>(a, num_entries, T, gate_buf, s);
  if (rc) return rc;
  const long long items = (long long)T * H;
  head_finish_kernel<<<(unsigned)((items + 7) / 8), 256, 0, s>>>(raw, dv + 2, 1, den_eps, proj, NV_DT_F32, ld, g0, 0,
                                                                 norm_w, norm_per_head, eps, out, out_dt, T, H, dv);
  NV_RETURN_LAST();
}

// The gated delta rule through col_scan_kernel; raw: [T, H, dv] and gate_buf: [T, H, 2] float32 scratch.
NV_API int nv_gated_delta_col_scan(const float* qkv, int C, int q0, int k0, int v0, int G, const void* proj,
                                   int proj_dt, long long ld, int g0, int b0, int a0, const float* A_log,
                                   const float* dt_bias, const int* cu_rows, const int* entry_slot, float* S,
                                   long long S_stride, int H, int dk, int dv, float eps, const float* norm_w,
                                   float* raw, float* gate_buf, void* out, int out_dt, int num_entries, int T,
                                   cudaStream_t s) {
  if (!dt_ok(out_dt) || proj_dt != NV_DT_F32) return NV_ERR_BAD_DTYPE;
  if (!nv_col_scan_usable(dk, dv) || H <= 0 || G <= 0 || H % G) return NV_ERR_UNSUPPORTED;
  if (num_entries == 0 || T == 0) return NV_OK;
  ColArgs a = {};
  a.cu_rows = cu_rows; a.entry_slot = entry_slot; a.S = S; a.S_stride = S_stride; a.qk = qkv; a.qk_ld = C; a.q0 = q0;
  a.k0 = k0; a.G = G; a.vsrc = qkv; a.v_ld = C; a.v0 = v0; a.gates = proj; a.gates_dt = proj_dt; a.gates_ld = ld;
  a.ga0 = b0; a.gb0 = a0; a.A_log = A_log; a.dt_bias = dt_bias; a.q_scale = 1.f; a.raw = raw; a.RW = dv; a.H = H;
  a.dk = dk; a.dv = dv;
  int rc = launch_col_scan<1>(a, num_entries, T, gate_buf, s);
  if (rc) return rc;
  const long long items = (long long)T * H;
  head_finish_kernel<<<(unsigned)((items + 7) / 8), 256, 0, s>>>(raw, dv, 0, 0.f, proj, proj_dt, ld, g0, 1, norm_w, 0,
                                                                 eps, out, out_dt, T, H, dv);
  NV_RETURN_LAST();
}

// The delta rule with a decay per head and key channel through col_scan_kernel.  `dec` [T, dec_ld] float32 holds the
// decays' pre-activations at column dec0 (head h's at dec0 + h dk); `gsrc` the output gate's at g0, gate_mode 1: a
// sigmoid, 0: silu.  Scratch, all float32: raw [T, H, dv], gate_buf [T, H, 2], decays [T, H dk].
NV_API int nv_channel_delta_scan(const float* qkv, int C, int q0, int k0, int v0, int G, const void* proj, int proj_dt,
                                 long long ld, int b0, const float* dec, long long dec_ld, int dec0, const void* gsrc,
                                 int gsrc_dt, long long gsrc_ld, int g0, int gate_mode, const float* A_log,
                                 const float* dt_bias, const int* cu_rows, const int* entry_slot, float* S,
                                 long long S_stride, int H, int dk, int dv, float eps, const float* norm_w, float* raw,
                                 float* gate_buf, float* decays, void* out, int out_dt, int num_entries, int T,
                                 cudaStream_t s) {
  if (!dt_ok(out_dt) || !dt_ok(proj_dt) || !dt_ok(gsrc_dt)) return NV_ERR_BAD_DTYPE;
  if (!nv_channel_scan_usable(dk, dv) || H <= 0 || G <= 0 || H % G) return NV_ERR_UNSUPPORTED;
  if (!dec || !raw || !gate_buf || !decays || gate_mode < 0 || gate_mode > 1) return NV_ERR_BAD_SIZE;
  if (num_entries == 0 || T == 0) return NV_OK;
  const long long n = (long long)T * H * dk;
  channel_gates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(dec, dec_ld, dec0, proj, proj_dt, ld, b0, A_log,
                                                                  dt_bias, H, dk, decays, gate_buf, n);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  ColArgs a = {};
  a.cu_rows = cu_rows; a.entry_slot = entry_slot; a.S = S; a.S_stride = S_stride; a.qk = qkv; a.qk_ld = C; a.q0 = q0;
  a.k0 = k0; a.G = G; a.vsrc = qkv; a.v_ld = C; a.v0 = v0; a.gates = gate_buf; a.gates_dt = NV_DT_F32;
  a.gates_ld = 2LL * H; a.ga0 = 0; a.gb0 = 1; a.A_log = A_log; a.dt_bias = dt_bias; a.q_scale = 1.f; a.raw = raw;
  a.RW = dv; a.H = H; a.dk = dk; a.dv = dv; a.dec = decays; a.dec_ld = (long long)H * dk;
  a.vec16 = (((uintptr_t)qkv & 15) == 0 && C % 4 == 0 && q0 % 4 == 0 && k0 % 4 == 0 && dk % 4 == 0 &&
             ((uintptr_t)decays & 15) == 0) ? 1 : 0;
  int rc = launch_col_scan_p<2, true>(a, num_entries, s);
  if (rc) return rc;
  const long long items = (long long)T * H;
  head_finish_kernel<<<(unsigned)((items + 7) / 8), 256, 0, s>>>(raw, dv, 0, 0.f, gsrc, gsrc_dt, gsrc_ld, g0,
                                                                 gate_mode == 1 ? 0 : 1, norm_w, 0, eps, out, out_dt, T,
                                                                 H, dv);
  NV_RETURN_LAST();
}
