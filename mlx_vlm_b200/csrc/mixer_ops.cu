// Sequence mixers beside the latent attention of layer_ops.cu, for decoder designs assembled on the host
// (models/decoder_blocks.py).  Every token of a step names its cache slot and its position; a step's tokens are
// the concatenation of its sequences' tokens, `first[t]` is the row of the first token of t's sequence in the step
// and `seqs[g] = (first row, rows)` lists the sequences.  A prompt, a portion of one, a decoded token and a batch of
// unequal requests are therefore the same launches.
//   * short causal convolution over time per channel, the last taps - 1 inputs of a sequence kept per slot,
//   * rotate-half rotary on queries and keys + the write of the key / value rows of the step into the cache,
//   * softmax attention over cached rows [keys of all kv heads | values of all kv heads] with grouped query heads,
//     an optional block-local or sliding range of visible keys and an optional sink logit per head that joins the
//     denominator without a key or a value,
//   * a per-head matrix state carried from token to token, S <- decay S + k u^T, o = S^T q, with u = v (decayed
//     outer-product memory) or u = beta (v - S^T k) (gated delta rule), the state in fp32 per slot,
//   * per-head / per-token output norms and gates, and a clamped gated feed-forward activation.
// All arithmetic is fp32; cache rows are bf16 in the serving mode and fp32 in the exact mode.
#include "common.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ float ld_row(const float* p) { return *p; }
__device__ __forceinline__ float ld_row(const bf16* p) { return bf2f(*p); }
__device__ __forceinline__ void st_row(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_row(bf16* p, float v) { *p = f2bf(v); }
__device__ __forceinline__ float sigmoid_exact(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_exact(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_exact(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float glu_arg(float g, float cubic) { return cubic != 0.f ? g + cubic * g * g * g : g; }
__device__ __forceinline__ float block_sum_fixed(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// ---------------------------------------------------------------------------------------------------------
// short convolution: y[t][c] = act( bias[c] + sum_j w[c][j] * u[t - (taps - 1) + j][c] ), inputs before the step come from
// the slot's state (the taps - 1 inputs that precede the step's first token), inputs before position 0 are zero
struct ConvP {
  const float* U; long ldu;
  const bf16* w;                   // [C][taps]
  float* Y; long ldy;
  float* state; long slot_stride;  // per slot [taps - 1][C]
  const int *slot, *pos, *first;
  int C, taps, act;
  const bf16* bias;                // [C] or NULL
  int residual;                    // the input itself is added to the convolution's output (before the activation)
  int single;                      // every sequence of the step is one token: the thread that read a channel's kept inputs
};                                 // also advances them (no second launch)
__global__ void short_conv_kernel(ConvP p) {
  const int t = blockIdx.x;
  const int back = t - p.first[t], ps = p.pos[t];
  const float* st = p.state + (long)p.slot[t] * p.slot_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < p.C; c += blockDim.x * gridDim.y) {
    float a = p.bias ? bf2f(p.bias[c]) : 0.f;
    if (p.residual) a += p.U[(long)t * p.ldu + c];
    for (int j = 0; j < p.taps; ++j) {
      const int lag = p.taps - 1 - j;
      float u = 0.f;
      if (lag <= back) u = p.U[(long)(t - lag) * p.ldu + c];
      else if (lag <= ps) u = st[(long)(back - lag + p.taps - 1) * p.C + c];
      a = fmaf(bf2f(p.w[(long)c * p.taps + j]), u, a);
    }
    p.Y[(long)t * p.ldy + c] = p.act ? silu_exact(a) : a;
    if (p.single) {                // entry j takes entry j + 1 (zero while that lies before the sequence), the last one the input
      float* sw = p.state + (long)p.slot[t] * p.slot_stride;
      const int n = p.taps - 1;
      for (int j = 0; j < n; ++j) {
        float v = 0.f;
        if (j == n - 1) v = p.U[(long)t * p.ldu + c];
        else if (ps + 1 - n + j >= 0) v = sw[(long)(j + 1) * p.C + c];
        sw[(long)j * p.C + c] = v;
      }
    }
  }
}
// after the step: the slot keeps the last taps - 1 inputs of its sequence.  A thread owns a channel; entry j takes
// what lies `rows` entries further on, so ascending order never overwrites an entry that is still to be read.
__global__ void conv_state_kernel(ConvP p, const int* __restrict__ seqs) {
  const int start = seqs[2 * blockIdx.x], rows = seqs[2 * blockIdx.x + 1], n = p.taps - 1;
  const int p0 = p.pos[start];
  float* st = p.state + (long)p.slot[start] * p.slot_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < p.C; c += blockDim.x * gridDim.y)
    for (int j = 0; j < n; ++j) {
      const int r = rows - n + j;        // row of the step that holds this input (negative: before the step)
      float v = 0.f;
      if (r >= 0) v = p.U[(long)(start + r) * p.ldu + c];
      else if (p0 + r >= 0) v = st[(long)(j + rows) * p.C + c];
      st[(long)j * p.C + c] = v;
    }
}

// ---------------------------------------------------------------------------------------------------------
// token shift: M[s][t] = h[t] + (h[t - 1] - h[t]) * mu[s] for each of n_mix mixing vectors; h[t - 1] of a sequence's
// first token of the step is the slot's kept row (zeros at position 0).  The slot then keeps the sequence's last
// input: by the thread that read it when the sequence brings one token (a decode step), else by a second launch.
struct ShiftP {
  const float* h; long ldh;
  const bf16* mu;                  // [n_mix][C]
  float* M; long ldm, mix_stride;  // [n_mix][T][C]
  float* state; long slot_stride;  // per slot [C]
  const int *slot, *pos, *first;
  int C, n_mix, single;            // single: every sequence of the step is one token
  bf16* Mb; long ldb, mixb_stride; // != NULL: the mixes are written as bf16 operand rows of ldb >= C columns (zero padding
};                                 // beyond C) for the tensor-core products that read them, instead of fp32 rows
__global__ void token_shift_kernel(ShiftP p) {
  const int t = blockIdx.x;
  const bool head = p.first[t] == t;
  float* st = p.state + (long)p.slot[t] * p.slot_stride;
  const bool fresh = p.pos[t] == 0;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < p.C; c += blockDim.x * gridDim.y) {
    const float x = p.h[(long)t * p.ldh + c];
    const float prev = head ? (fresh ? 0.f : st[c]) : p.h[(long)(t - 1) * p.ldh + c];
    const float d = prev - x;
    for (int s = 0; s < p.n_mix; ++s) {
      const float m = fmaf(d, bf2f(p.mu[(long)s * p.C + c]), x);
      if (p.Mb) p.Mb[(long)s * p.mixb_stride + (long)t * p.ldb + c] = f2bf(m);
      else p.M[(long)s * p.mix_stride + (long)t * p.ldm + c] = m;
    }
    if (p.single) st[c] = x;
  }
  if (p.Mb)
    for (int c = p.C + blockIdx.y * blockDim.x + threadIdx.x; c < p.ldb; c += blockDim.x * gridDim.y)
      for (int s = 0; s < p.n_mix; ++s) p.Mb[(long)s * p.mixb_stride + (long)t * p.ldb + c] = f2bf(0.f);
}
__global__ void token_shift_state_kernel(ShiftP p, const int* __restrict__ seqs) {
  const int start = seqs[2 * blockIdx.x], rows = seqs[2 * blockIdx.x + 1];
  float* st = p.state + (long)p.slot[start] * p.slot_stride;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < p.C; c += blockDim.x * gridDim.y)
    st[c] = p.h[(long)(start + rows - 1) * p.ldh + c];
}

// ---------------------------------------------------------------------------------------------------------
// rotary on q (in place) and k, and the cache rows of the step: cache[slot][pos] = [k of every kv head | v ...]
template <typename CT>
struct QkvPostP {
  float* Q; long ldq;
  const float* K; long ldk;
  const float* V; long ldv;
  CT* cache; long slot_stride, tok_stride;
  const int *slot, *pos;
  const float2* cs;                // [T][rot_dims / 2]
  int H, G, dim, vdim, rot_dims;
  // optional steps in front of the rotation and the cache write (all NULL / 0: none)
  const bf16 *qn_w, *kn_w;         // [H dim], [G dim]: RMS norm over the WHOLE query / key projection, times these
  float eps;
  int v_unit;                      // every value head is divided by its root mean square (eps inside the root)
  float qt_coef; int qt_every;     // queries times 1 + coef ln(floor((pos + 1) / every) + 1)
  const bf16* vmix;                // one number lam: v <- (1 - lam) v + lam v_first (after the value norm)
  const float* v_first; long ldvf; // [T][G vdim]
  float* v_keep; long ldvk;        // [T][G vdim] or NULL: the values as cached, in fp32 (a later layer mixes with them)
};
template <typename CT>
__global__ void qkv_post_kernel(QkvPostP<CT> p) {
  __shared__ float red[32];
  const int t = blockIdx.x, half = p.rot_dims / 2;
  float* q = p.Q + (long)t * p.ldq;
  const float* k = p.K + (long)t * p.ldk;
  float k_inv = 1.f;
  if (p.qn_w || p.qt_every > 0) {              // queries: the norm over all heads at once, then the temperature
    float q_mul = 1.f;
    if (p.qn_w) {
      float ss = 0.f;
      for (int e = threadIdx.x; e < p.H * p.dim; e += blockDim.x) ss = fmaf(q[e], q[e], ss);
      q_mul = 1.0f / sqrtf(block_sum_fixed(ss, red) / (float)(p.H * p.dim) + p.eps);
    }
    if (p.qt_every > 0) q_mul *= 1.0f + p.qt_coef * logf((float)((p.pos[t] + 1) / p.qt_every) + 1.0f);
    for (int e = threadIdx.x; e < p.H * p.dim; e += blockDim.x) q[e] = q[e] * q_mul * (p.qn_w ? bf2f(p.qn_w[e]) : 1.f);
    __syncthreads();
  }
  if (p.kn_w) {
    float ss = 0.f;
    for (int e = threadIdx.x; e < p.G * p.dim; e += blockDim.x) ss = fmaf(k[e], k[e], ss);
    k_inv = 1.0f / sqrtf(block_sum_fixed(ss, red) / (float)(p.G * p.dim) + p.eps);
  }
  auto kn = [&](int e) { return p.kn_w ? k[e] * k_inv * bf2f(p.kn_w[e]) : k[e]; };
  for (int e = threadIdx.x; e < p.H * half; e += blockDim.x) {
    const int h = e / half, i = e % half;
    const float2 a = p.cs[(long)t * half + i];
    float* r = q + h * p.dim;
    const float lo = r[i], hi = r[i + half];
    r[i] = lo * a.x - hi * a.y;
    r[i + half] = hi * a.x + lo * a.y;
  }
  CT* row = p.cache + (long)p.slot[t] * p.slot_stride + (long)p.pos[t] * p.tok_stride;
  for (int e = threadIdx.x; e < p.G * p.dim; e += blockDim.x) {
    const int i = e % p.dim;
    float v;
    if (i < half) {
      const float2 a = p.cs[(long)t * half + i];
      v = kn(e) * a.x - kn(e + half) * a.y;
    } else if (i < p.rot_dims) {
      const float2 a = p.cs[(long)t * half + i - half];
      v = kn(e) * a.x + kn(e - half) * a.y;
    } else {
      v = kn(e);
    }
    st_row(row + e, v);
  }
  const float* v = p.V + (long)t * p.ldv;
  if (!p.v_unit && !p.vmix && !p.v_keep) {
    for (int e = threadIdx.x; e < p.G * p.vdim; e += blockDim.x) st_row(row + p.G * p.dim + e, v[e]);
    return;
  }
  const float lam = p.vmix ? bf2f(*p.vmix) : 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int g = warp; g < p.G; g += nw) {         // a warp per value head
    float inv = 1.f;
    if (p.v_unit) {
      float ss = 0.f;
      for (int i = lane; i < p.vdim; i += 32) { const float a = v[g * p.vdim + i]; ss = fmaf(a, a, ss); }
      inv = 1.0f / sqrtf(warp_sum(ss) / (float)p.vdim + p.eps);
    }
    for (int i = lane; i < p.vdim; i += 32) {
      const int e = g * p.vdim + i;
      float a = v[e] * inv;
      if (p.vmix) a = (1.0f - lam) * a + lam * p.v_first[(long)t * p.ldvf + e];
      if (p.v_keep) p.v_keep[(long)t * p.ldvk + e] = a;
      st_row(row + p.G * p.dim + e, a);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// attention of grouped query heads over cached key / value rows.  Block = (query token, kv head x group of up to 8
// of its query heads, split); a warp per query head.  32 rows are staged at a time (fp32); lane j scores key j, the
// lanes share the probabilities and each lane accumulates its value columns (online softmax).  The visible keys of a
// query at position p are lo..p with lo = max(start of p's block of `chunk` positions, p - window + 1, 0).  With a
// sink, split 0 starts its running maximum at the sink logit with denominator 1: the sink counts once.
constexpr int SA_KT = 32;
template <typename CT>
struct SinkAttnP {
  const float* q; long ldq;
  const CT* cache; long slot_stride, tok_stride;
  const int *slot, *pos;
  float* out; long ldo;
  const bf16* sink;
  int H, G, dim, vdim;
  float scale;
  int chunk, window;
  float* part; int n_split;        // n_split > 1: [T][H][n_split][vdim + 2] = (acc.., max, sum)
  int vec;                         // key and value columns of every row start on 16-byte boundaries and are whole
                                   // 16-byte vectors: rows are staged with 16-byte loads
  float bias_exp;                  // > 0: slope_h (query position - key position) is taken off the score of head h,
                                   // slope_h = 2^(-bias_exp (h + 1) / H)
  int unit_sink;                   // the denominator also holds exp(0) = 1 (a sink logit of zero, no tensor)
};
template <typename CT>
__global__ void sink_attention_kernel(SinkAttnP<CT> p) {
  extern __shared__ float sm[];
  const int rep = p.H / p.G, nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hgroups = (rep + nw - 1) / nw;
  const int t = blockIdx.x, g = blockIdx.y / hgroups, hg = blockIdx.y % hgroups;
  const bool v4 = (p.dim & 3) == 0;
  const int dim = p.dim, vdim = p.vdim, ldk = dim + (v4 ? 4 : 1);
  float* keys = sm;                          // [SA_KT][ldk]
  float* vals = keys + SA_KT * ldk;          // [SA_KT][vdim]
  float* qs = vals + SA_KT * vdim;           // [nw][dim]
  const int hl = hg * nw + warp;
  const bool live = hl < rep;
  const int h = g * rep + hl;
  if (live) {
    const float* q = p.q + (long)t * p.ldq + (long)h * dim;
    for (int i = lane; i < dim; i += 32) qs[warp * dim + i] = q[i];
  }
  const int ps = p.pos[t];
  int lo = 0;
  if (p.chunk > 0) lo = (ps / p.chunk) * p.chunk;
  if (p.window > 0) lo = max(lo, ps - p.window + 1);
  const CT* base = p.cache + (long)p.slot[t] * p.slot_stride;
  const int koff = g * dim, voff = p.G * dim + g * vdim;
  const int per_lane = (vdim + 31) / 32;
  float m = -INFINITY, l = 0.f;
  if (p.sink && blockIdx.z == 0 && live) { m = bf2f(p.sink[h]); l = 1.f; }
  if (p.unit_sink && blockIdx.z == 0 && live) { m = 0.f; l = 1.f; }
  const float slope = p.bias_exp > 0.f ? exp2f(-p.bias_exp * (float)(h + 1) / (float)p.H) : 0.f;
  float acc[8];                              // vdim <= 256
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int k0 = lo + blockIdx.z * SA_KT; k0 <= ps; k0 += SA_KT * p.n_split) {
    const int nk = min(SA_KT, ps + 1 - k0);
    __syncthreads();
    if (p.vec) {                              // several independent 16-byte loads in flight per thread
      constexpr int PER = 16 / (int)sizeof(CT);
      const int kv = dim / PER, vv = vdim / PER, per_row = kv + vv;
#pragma unroll 4
      for (int e = threadIdx.x; e < nk * per_row; e += blockDim.x) {
        const int j = e / per_row, c = e - j * per_row;
        const bool is_key = c < kv;
        const int i = (is_key ? c : c - kv) * PER;
        const uint4 raw = *reinterpret_cast<const uint4*>(base + (long)(k0 + j) * p.tok_stride + (is_key ? koff : voff) + i);
        float* dst = is_key ? keys + j * ldk + i : vals + j * vdim + i;
        if (sizeof(CT) == 2) {
          float f[8];
          unpack8(raw, f);
          *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
        } else {
          *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(raw.x), __uint_as_float(raw.y),
                                                        __uint_as_float(raw.z), __uint_as_float(raw.w));
        }
      }
    } else {
#pragma unroll 4
      for (int e = threadIdx.x; e < nk * dim; e += blockDim.x) {
        const int j = e / dim, i = e - j * dim;
        keys[j * ldk + i] = ld_row(base + (long)(k0 + j) * p.tok_stride + koff + i);
      }
#pragma unroll 4
      for (int e = threadIdx.x; e < nk * vdim; e += blockDim.x) {
        const int j = e / vdim, i = e - j * vdim;
        vals[j * vdim + i] = ld_row(base + (long)(k0 + j) * p.tok_stride + voff + i);
      }
    }
    __syncthreads();
    if (!live) continue;
    float s = -INFINITY;
    if (lane < nk) {
      const float* kr = keys + lane * ldk;
      const float* qr = qs + warp * dim;
      float a = 0.f;
      if (v4) {                               // fixed order: four running sums over i mod 4, then (0 + 1) + (2 + 3)
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 4
        for (int i = 0; i < dim; i += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qr + i);
          const float4 k4 = *reinterpret_cast<const float4*>(kr + i);
          a0 = fmaf(q4.x, k4.x, a0); a1 = fmaf(q4.y, k4.y, a1); a2 = fmaf(q4.z, k4.z, a2); a3 = fmaf(q4.w, k4.w, a3);
        }
        a = (a0 + a1) + (a2 + a3);
      } else {
        for (int i = 0; i < dim; ++i) a = fmaf(qr[i], kr[i], a);
      }
      s = a * p.scale - slope * (float)(ps - (k0 + lane));
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);       // nothing seen yet: exp(-inf) = 0
    const float pj = lane < nk ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < per_lane) acc[i] *= corr;
    for (int j = 0; j < nk; ++j) {
      const float w = __shfl_sync(0xffffffffu, pj, j);
      const float* vr = vals + j * vdim;
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < per_lane) {
          const int d = lane + 32 * i;
          if (d < vdim) acc[i] = fmaf(w, vr[d], acc[i]);
        }
    }
  }
  if (!live) return;
  if (p.n_split > 1) {                        // un-normalised partial sums; a split without keys: max -inf, sum 0
    float* o = p.part + (((long)t * p.H + h) * p.n_split + blockIdx.z) * (vdim + 2);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < per_lane) {
        const int d = lane + 32 * i;
        if (d < vdim) o[d] = acc[i];
      }
    if (lane == 0) { o[vdim] = m; o[vdim + 1] = l; }
    return;
  }
  const float inv = 1.0f / l;
  float* o = p.out + (long)t * p.ldo + (long)h * vdim;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (i < per_lane) {
      const int d = lane + 32 * i;
      if (d < vdim) o[d] = acc[i] * inv;
    }
}
// merge the splits of one (token, head) in a fixed order
__global__ void sink_attention_merge_kernel(const float* __restrict__ part, int n_split, int vdim,
                                            float* __restrict__ out, long ldo, int H) {
  __shared__ float wgt[64];
  __shared__ float inv_s;
  const int t = blockIdx.x, h = blockIdx.y, row = vdim + 2;
  const float* pp = part + ((long)t * H + h) * n_split * row;
  if (threadIdx.x < 32) {
    const int s0 = threadIdx.x, s1 = threadIdx.x + 32;
    const float m0 = s0 < n_split ? pp[(long)s0 * row + vdim] : -INFINITY;
    const float m1 = s1 < n_split ? pp[(long)s1 * row + vdim] : -INFINITY;
    const float l0 = s0 < n_split ? pp[(long)s0 * row + vdim + 1] : 0.f;
    const float l1 = s1 < n_split ? pp[(long)s1 * row + vdim + 1] : 0.f;
    const float M = warp_max(fmaxf(m0, m1));
    const float e0 = m0 == -INFINITY ? 0.f : expf(m0 - M), e1 = m1 == -INFINITY ? 0.f : expf(m1 - M);
    wgt[s0] = e0; wgt[s1] = e1;
    const float L = warp_sum(l0 * e0 + l1 * e1);
    if (threadIdx.x == 0) inv_s = 1.0f / L;
  }
  __syncthreads();
  const float inv = inv_s;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float a = 0.f;                 // a split without keys left zeros and weighs zero: its term adds nothing, and the
#pragma unroll 8                   // loads of all splits are in flight together
    for (int s = 0; s < n_split; ++s) a = fmaf(pp[(long)s * row + d], wgt[s], a);
    out[(long)t * ldo + (long)h * vdim + d] = a * inv;
  }
}

// ---------------------------------------------------------------------------------------------------------
// matrix state per head, carried from token to token:  S <- decay S + k u^T,  o = S^T q,  u = v or
// u = beta (v - (decay S)^T k).  The columns of S evolve independently, so a block owns a slice of the value
// columns of one head of one sequence and walks the sequence's tokens in order.  A column is held by P threads, each
// with LS_R rows of it in registers (dim <= LS_R P, P a power of two up to a warp); their partial dot products meet
// in a butterfly over the P lanes.  The walk is a chain of dependent steps, so what counts is its length per token:
// few rows per thread, and many warps per scheduler to fill the waits.
// The slot keeps S between steps as [H][LS_R][vdim][P] (row r LS_R + i of column c at ((h LS_R + i) vdim + c) P + r),
// which makes the loads and stores of a warp contiguous; a sequence that starts at position 0 starts from zero.
// q and k may be shared by `rep` heads, passed through silu, and scaled to unit length per head at load.
constexpr int LS_CT = 16, LS_THREADS = 256, LS_R = 8, LS_RS = 12;   // LS_RS: pitch of a thread's rows in shared memory
struct StateP {
  const float* q; long ldq;
  const float* k; long ldk;
  const float* v; long ldv;
  float* out; long ldo;
  float* state; long slot_stride;
  const int* seqs;
  const int *slot, *pos;
  int H, rep, dim, vdim;
  int act;                          // silu on q, k, v at load
  float unit_eps, q_scale;          // unit_eps > 0: q, k <- x / sqrt(sum x^2 + unit_eps); q also times q_scale
  // prepared inputs (a prompt step: one parallel pass over all tokens does the per-token work first): q, k are already
  // activated and scaled, and these hold k . q [T][H / rep], the decay [T][H] and beta [T][H]; NULL: made here
  const float *kq_in, *dec_in, *bet_in;
  const float* decay_const;         // [H], or NULL: decay = exp(-exp(A_log[h]) softplus(a[t][h] + dt_bias[h]))
  const float* a; long lda;
  const bf16 *A_log, *dt_bias;
  const float* b; long ldb;         // beta = sigmoid(b[t][h]); NULL: 1
  int delta;
  int dt_in;                        // state-space form: beta = softplus(a[t][h] + dt_bias[h]) (the step size) and u = beta v
  const bf16* skip;                 // [H] or NULL: o += skip[h] v
  // decay per key channel (the template's CHAN):  o = S^T q + (sum_i q_i bonus_i k_i) v  with S the state BEFORE the
  // token, then  S <- diag(w) S + k v^T.  Prepared: wdec [T][H dim] holds w and kq_in the bracket; else wdec holds the
  // logits x of w = exp(-exp(x)) and the bracket is made here from `bonus` ([H][dim])
  const float* wdec; long ldw;
  const bf16* bonus;
  // A long sequence in parts that are walked at the same time (decay per key channel, prepared inputs).  The state is
  // linear in its start: after a part,  S_end = diag(prod of the part's w) S_start + S_local  with S_local the part
  // walked from zero.  Pass 1 (the template's LOCAL) walks every part but a sequence's last from zero, without outputs,
  // and leaves S_local and the product of its decays; a small launch chains them into every part's true start state;
  // pass 2 walks every part from that state with outputs, and the last part leaves the slot's state.
  int part_len, n_parts;            // n_parts > 0: blockIdx.x = sequence * n_parts + part
  float* part_state;                // [n_seq][n_parts][H LS_R vdim P]: S_local, then the start state of the part after
  float* part_decay;                // [n_seq][n_parts][H][P LS_R]
};
// The per-token work of a prompt step in one parallel pass: q, k activated and scaled to unit length (a warp per
// token and q/k head, the same order of sums as the walk's own staging), k . q, the decay and beta of every head.
struct StatePrepP {
  const float* q; long ldq;
  const float* k; long ldk;
  float *qn, *kn; long ldn;         // [T][Hk * dim]
  float *kq, *dec, *bet;            // [T][Hk], [T][H], [T][H]
  int H, Hk, dim, act;
  float unit_eps, q_scale;
  const float* decay_const;
  const float* a; long lda;
  const bf16 *A_log, *dt_bias;
  const float* b; long ldb;
  int dt_in;
  // decay per key channel: wraw [T][H dim] -> wn = exp(-exp(wraw)); kq = sum_i q_i bonus_i k_i; no dec / bet
  const float* wraw; long ldwr;
  float* wn;
  const bf16* bonus;                // [H][dim]
};
__global__ void state_prep_kernel(StatePrepP p) {
  const long t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int hk = warp; hk < p.Hk; hk += nw) {
    const float* kr = p.k + t * p.ldk + (long)hk * p.dim;
    const float* qr = p.q + t * p.ldq + (long)hk * p.dim;
    float* ko = p.kn + t * p.ldn + (long)hk * p.dim;
    float* qo = p.qn + t * p.ldn + (long)hk * p.dim;
    float ik = 1.f, iq = 1.f;
    if (p.unit_eps > 0.f) {
      float sk = 0.f, sq = 0.f;
      for (int i = lane; i < p.dim; i += 32) {
        float a = kr[i], b = qr[i];
        if (p.act) { a = silu_exact(a); b = silu_exact(b); }
        sk = fmaf(a, a, sk); sq = fmaf(b, b, sq);
      }
      ik = 1.0f / sqrtf(warp_sum(sk) + p.unit_eps);
      iq = p.q_scale / sqrtf(warp_sum(sq) + p.unit_eps);
    }
    float dot = 0.f;
    for (int i = lane; i < p.dim; i += 32) {
      float a = kr[i], b = qr[i];
      if (p.act) { a = silu_exact(a); b = silu_exact(b); }
      a *= ik; b *= iq;
      if (!p.wraw) { ko[i] = a; qo[i] = b; }        // (a decay per channel leaves q, k as they are: the walk reads the originals)
      dot = p.wraw ? fmaf(a * b, bf2f(p.bonus[(long)hk * p.dim + i]), dot) : fmaf(a, b, dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) p.kq[t * p.Hk + hk] = dot;
  }
  if (p.wraw) {
    for (int e = threadIdx.x; e < p.H * p.dim; e += blockDim.x) p.wn[t * ((long)p.H * p.dim) + e] = expf(-expf(p.wraw[t * p.ldwr + e]));
    return;
  }
  for (int h = threadIdx.x; h < p.H; h += blockDim.x) {
    const float dt = p.decay_const ? 0.f : softplus_exact(p.a[t * p.lda + h] + bf2f(p.dt_bias[h]));
    p.dec[t * p.H + h] = p.decay_const ? p.decay_const[h] : expf(-expf(bf2f(p.A_log[h])) * dt);
    p.bet[t * p.H + h] = p.dt_in ? dt : (p.b ? sigmoid_exact(p.b[t * p.ldb + h]) : 1.f);
  }
}

template <int P, bool DELTA, bool CHAN, bool LOCAL = false>
__global__ void __launch_bounds__(LS_THREADS) linear_state_kernel(StateP p) {
  // Tokens are staged CT at a time.  The raw q, k, v, decay and beta inputs of the NEXT group are requested from
  // global memory into registers before the current group is walked, so their latency hides behind the walk.
  // Per token, with S the state before it:  dk = S^T k, dq = S^T q (one pass, one butterfly for both),
  // u = beta (v - decay dk) (or v),  o = decay dq + u (k . q),  S <- decay S + k u^T  — o does not wait for the update.
  // Without the delta rule (DELTA false) u does not depend on S: the chain from token to token is one multiply-add per
  // row, the dot product and its butterfly hang off it, and the token loop is unrolled so that they overlap the chain.
  constexpr int CB = LS_THREADS / P, LD = P * LS_RS, DKP = P * LS_R;
  constexpr int CT = P >= 32 ? LS_CT / 2 : LS_CT;       // tokens per group: the staged rows fit static shared memory
  constexpr int NQK = (CT * DKP + LS_THREADS - 1) / LS_THREADS, NV = (CT * CB + LS_THREADS - 1) / LS_THREADS;
  __shared__ __align__(16) float ks[CT][LD], qs[CT][LD], ws[CHAN ? CT : 1][CHAN ? LD : 4];
  __shared__ float vs[CT][CB];
  __shared__ float dec[CT], bet[CT], kq[CT];
  const int seq = p.n_parts > 0 ? blockIdx.x / p.n_parts : blockIdx.x, part = p.n_parts > 0 ? blockIdx.x % p.n_parts : 0;
  int start = p.seqs[2 * seq], rows = p.seqs[2 * seq + 1];
  bool last_part = true;
  if (p.n_parts > 0) {
    const int n = (rows + p.part_len - 1) / p.part_len;          // parts of this sequence
    if (part >= (LOCAL ? n - 1 : n)) return;                     // (whole block)
    last_part = part == n - 1;
    start += part * p.part_len;
    rows = min(p.part_len, rows - part * p.part_len);
  }
  const int h = blockIdx.y, hk = h / p.rep;
  const int cj = threadIdx.x / P, r = threadIdx.x % P, col = blockIdx.z * CB + cj;
  const bool valid = col < p.vdim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float S[LS_R];
  float Dacc[LOCAL ? LS_R : 1];
  if (LOCAL) {
#pragma unroll
    for (int i = 0; i < LS_R; ++i) Dacc[i] = 1.f;
  }
  const long head_floats = (long)LS_R * p.vdim * P;
  float* st = p.state + (long)p.slot[start] * p.slot_stride;
  if (!LOCAL && part > 0) st = p.part_state + ((long)seq * p.n_parts + part - 1) * p.H * head_floats;    // the start state made for this part
  if (!LOCAL && (part > 0 || p.pos[start] > 0) && valid) {
#pragma unroll
    for (int i = 0; i < LS_R; ++i) S[i] = st[(((long)h * LS_R + i) * p.vdim + col) * P + r];
  } else {
#pragma unroll
    for (int i = 0; i < LS_R; ++i) S[i] = 0.f;
  }
  float rk[NQK], rq[NQK], rw[CHAN ? NQK : 1], rv[NV], ra = 0.f, rb = 0.f, rkq = 0.f;
  const bool raw = p.kq_in == nullptr, act_qk = raw && p.act;
  auto request = [&](int c0) {               // raw inputs of tokens c0 .. c0 + CT - 1 (zeros past the end)
    const int nc = min(CT, rows - c0);
#pragma unroll
    for (int n = 0; n < NQK; ++n) {
      const int e = threadIdx.x + n * LS_THREADS, tk = e / DKP, i = e % DKP;
      const bool ok = tk < nc && i < p.dim;
      const long t = start + c0 + tk;
      rk[n] = ok ? p.k[t * p.ldk + (long)hk * p.dim + i] : 0.f;
      rq[n] = ok ? p.q[t * p.ldq + (long)hk * p.dim + i] : 0.f;
      if (CHAN) rw[n] = ok ? p.wdec[t * p.ldw + (long)h * p.dim + i] : 0.f;
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int e = threadIdx.x + n * LS_THREADS, tk = e / CB, cc = blockIdx.z * CB + e % CB;
      rv[n] = (tk < nc && cc < p.vdim) ? p.v[(long)(start + c0 + tk) * p.ldv + (long)h * p.vdim + cc] : 0.f;
    }
    if ((int)threadIdx.x < nc) {
      const long t = start + c0 + threadIdx.x;
      if (CHAN) {
        if (p.kq_in) rkq = p.kq_in[t * (p.H / p.rep) + hk];
      } else if (p.kq_in) {
        ra = p.dec_in[t * p.H + h]; rb = p.bet_in[t * p.H + h]; rkq = p.kq_in[t * (p.H / p.rep) + hk];
      } else {
        if (!p.decay_const) ra = p.a[t * p.lda + h];
        if (p.b) rb = p.b[t * p.ldb + h];
      }
    }
  };
  const float A = (CHAN || p.decay_const || !raw) ? 0.f : expf(bf2f(p.A_log[h])), dtb = (CHAN || p.decay_const || !raw) ? 0.f : bf2f(p.dt_bias[h]);
  const float dconst = p.decay_const ? p.decay_const[h] : 0.f;
  const float skip = p.skip ? bf2f(p.skip[h]) : 0.f;
  request(0);
  for (int c0 = 0; c0 < rows; c0 += CT) {
    const int nc = min(CT, rows - c0);
    __syncthreads();                          // the walk over the previous group is over
#pragma unroll
    for (int n = 0; n < NQK; ++n) {
      const int e = threadIdx.x + n * LS_THREADS, tk = e / DKP, i = e % DKP;
      if (e < CT * DKP) {
        ks[tk][(i / LS_R) * LS_RS + (i % LS_R)] = act_qk ? silu_exact(rk[n]) : rk[n];
        qs[tk][(i / LS_R) * LS_RS + (i % LS_R)] = act_qk ? silu_exact(rq[n]) : rq[n];
        if (CHAN) ws[tk][(i / LS_R) * LS_RS + (i % LS_R)] = raw ? expf(-expf(rw[n])) : rw[n];
      }
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int e = threadIdx.x + n * LS_THREADS;
      if (e < CT * CB) vs[e / CB][e % CB] = p.act ? silu_exact(rv[n]) : rv[n];
    }
    if ((int)threadIdx.x < nc) {
      if (CHAN) {
        if (!raw) kq[threadIdx.x] = rkq;
      } else if (raw) {
        const float dt = p.decay_const ? 0.f : softplus_exact(ra + dtb);
        dec[threadIdx.x] = p.decay_const ? dconst : expf(-A * dt);
        bet[threadIdx.x] = p.dt_in ? dt : (p.b ? sigmoid_exact(rb) : 1.f);
      } else {
        dec[threadIdx.x] = ra; bet[threadIdx.x] = rb; kq[threadIdx.x] = rkq;
      }
    }
    __syncthreads();
    for (int tk = warp; raw && tk < nc; tk += LS_THREADS / 32) {      // a warp per token row: lengths and k . q in a fixed order
      float ik = 1.f, iq = 1.f;
      if (p.unit_eps > 0.f) {
        float sk = 0.f, sq = 0.f;
        for (int i = lane; i < p.dim; i += 32) {
          const float a = ks[tk][(i / LS_R) * LS_RS + (i % LS_R)], b = qs[tk][(i / LS_R) * LS_RS + (i % LS_R)];
          sk = fmaf(a, a, sk); sq = fmaf(b, b, sq);
        }
        ik = 1.0f / sqrtf(warp_sum(sk) + p.unit_eps);
        iq = p.q_scale / sqrtf(warp_sum(sq) + p.unit_eps);
      }
      float dot = 0.f;
      for (int i = lane; i < p.dim; i += 32) {
        const int at = (i / LS_R) * LS_RS + (i % LS_R);
        const float a = ks[tk][at] * ik, b = qs[tk][at] * iq;
        ks[tk][at] = a; qs[tk][at] = b;
        dot = CHAN ? fmaf(a * b, bf2f(p.bonus[(long)hk * p.dim + i]), dot) : fmaf(a, b, dot);
      }
      dot = warp_sum(dot);
      if (lane == 0) kq[tk] = dot;
    }
    if (raw) __syncthreads();
    if (c0 + CT < rows) request(c0 + CT);
    float* op = p.out + (long)(start + c0) * p.ldo + (long)h * p.vdim + col;
    const float* kp = &ks[0][r * LS_RS];
    const float* qp = &qs[0][r * LS_RS];
    const float* wp = &ws[0][CHAN ? r * LS_RS : 0];
#pragma unroll(DELTA ? 1 : 4)
    for (int tk = 0; tk < nc; ++tk, op += p.ldo, kp += LD, qp += LD) {
      const float4 k0 = *reinterpret_cast<const float4*>(kp), k1 = *reinterpret_cast<const float4*>(kp + 4);
      const float4 q0 = *reinterpret_cast<const float4*>(qp), q1 = *reinterpret_cast<const float4*>(qp + 4);
      const float k_[LS_R] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
      const float q_[LS_R] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
      if (CHAN) {                  // the output reads the state before the token; every row has its own decay
        const float4 w0 = *reinterpret_cast<const float4*>(wp), w1 = *reinterpret_cast<const float4*>(wp + 4);
        const float w_[LS_R] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        wp += LD;
        const float vin = vs[tk][cj];
        if (LOCAL) {
#pragma unroll
          for (int i = 0; i < LS_R; ++i) Dacc[i] *= w_[i];
        } else {
          float b0 = 0.f, b1 = 0.f;
#pragma unroll
          for (int i = 0; i < LS_R; i += 2) { b0 = fmaf(S[i], q_[i], b0); b1 = fmaf(S[i + 1], q_[i + 1], b1); }
          float dq = b0 + b1;
#pragma unroll
          for (int o = 1; o < P; o <<= 1) dq += __shfl_xor_sync(0xffffffffu, dq, o);
          if (r == 0 && valid) *op = fmaf(vin, kq[tk], dq);
        }
#pragma unroll
        for (int i = 0; i < LS_R; ++i) S[i] = fmaf(k_[i], vin, w_[i] * S[i]);
        continue;
      }
      const float d = dec[tk];
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;       // two running sums per dot: short dependency chains
#pragma unroll
      for (int i = 0; i < LS_R; i += 2) {
        if (DELTA) { a0 = fmaf(S[i], k_[i], a0); a1 = fmaf(S[i + 1], k_[i + 1], a1); }
        b0 = fmaf(S[i], q_[i], b0); b1 = fmaf(S[i + 1], q_[i + 1], b1);
      }
      float dk = a0 + a1, dq = b0 + b1;
#pragma unroll
      for (int o = 1; o < P; o <<= 1) {
        if (DELTA) dk += __shfl_xor_sync(0xffffffffu, dk, o);
        dq += __shfl_xor_sync(0xffffffffu, dq, o);
      }
      const float vin = vs[tk][cj];
      float u = vin;
      if (DELTA) u = bet[tk] * (u - d * dk);
      else if (p.dt_in) u = bet[tk] * u;
      if (r == 0 && valid) *op = fmaf(skip, vin, fmaf(u, kq[tk], d * dq));
#pragma unroll
      for (int i = 0; i < LS_R; ++i) S[i] = fmaf(k_[i], u, d * S[i]);
    }
  }
  if (LOCAL) {                       // what the part adds to any start state, and the product of its decays
    float* sl = p.part_state + ((long)seq * p.n_parts + part) * p.H * head_floats;
    if (valid) {
#pragma unroll
      for (int i = 0; i < LS_R; ++i) sl[(((long)h * LS_R + i) * p.vdim + col) * P + r] = S[i];
    }
    if (col == 0) {
      float* dl = p.part_decay + (((long)seq * p.n_parts + part) * p.H + h) * (P * LS_R);
#pragma unroll
      for (int i = 0; i < LS_R; ++i) dl[r * LS_R + i] = Dacc[i];
    }
    return;
  }
  if (valid && last_part) {
    st = p.state + (long)p.slot[start] * p.slot_stride;
#pragma unroll
    for (int i = 0; i < LS_R; ++i) st[(((long)h * LS_R + i) * p.vdim + col) * P + r] = S[i];
  }
}
// The walk with a decay per key channel over PREPARED inputs (a prompt step), two value columns per thread: the staged
// k, q, w rows of a token are loaded from shared memory once for both columns, which is what bounds the walk (every
// thread reads 24 floats per token for 16 multiply-adds per column).  Same parts scheme and state layout as above.
template <int P, int NC, bool LOCAL>
__global__ void __launch_bounds__(LS_THREADS) channel_state_kernel(StateP p) {
  constexpr int CB = LS_THREADS / P, CBN = CB * NC, LD = P * LS_RS, DKP = P * LS_R;
  constexpr int CT = P >= 32 ? LS_CT / 2 : LS_CT;
  constexpr int NQK = (CT * DKP + LS_THREADS - 1) / LS_THREADS, NV = (CT * CBN + LS_THREADS - 1) / LS_THREADS;
  __shared__ __align__(16) float ks[CT][LD], ws[CT][LD], qs[LOCAL ? 1 : CT][LOCAL ? 4 : LD];
  __shared__ float vs[CT][CBN];
  __shared__ float kq[CT];
  const int seq = p.n_parts > 0 ? blockIdx.x / p.n_parts : blockIdx.x, part = p.n_parts > 0 ? blockIdx.x % p.n_parts : 0;
  int start = p.seqs[2 * seq], rows = p.seqs[2 * seq + 1];
  bool last_part = true;
  if (p.n_parts > 0) {
    const int n = (rows + p.part_len - 1) / p.part_len;
    if (part >= (LOCAL ? n - 1 : n)) return;
    last_part = part == n - 1;
    start += part * p.part_len;
    rows = min(p.part_len, rows - part * p.part_len);
  }
  const int h = blockIdx.y;
  const int cj = threadIdx.x / P, r = threadIdx.x % P, col0 = blockIdx.z * CBN + cj * NC;
  float S[NC][LS_R], Dacc[LOCAL ? LS_R : 1];
  if (LOCAL) {
#pragma unroll
    for (int i = 0; i < LS_R; ++i) Dacc[i] = 1.f;
  }
  const long head_floats = (long)LS_R * p.vdim * P;
  const float* st0 = p.state + (long)p.slot[start] * p.slot_stride;
  if (!LOCAL && part > 0) st0 = p.part_state + ((long)seq * p.n_parts + part - 1) * p.H * head_floats;
  const bool from_state = !LOCAL && (part > 0 || p.pos[start] > 0);
#pragma unroll
  for (int c = 0; c < NC; ++c)
#pragma unroll
    for (int i = 0; i < LS_R; ++i)
      S[c][i] = (from_state && col0 + c < p.vdim) ? st0[(((long)h * LS_R + i) * p.vdim + col0 + c) * P + r] : 0.f;
  float rk[NQK], rw[NQK], rq[LOCAL ? 1 : NQK], rv[NV], rkq = 0.f;
  auto request = [&](int c0) {
    const int nc = min(CT, rows - c0);
#pragma unroll
    for (int n = 0; n < NQK; ++n) {
      const int e = threadIdx.x + n * LS_THREADS, tk = e / DKP, i = e % DKP;
      const bool ok = tk < nc && i < p.dim;
      const long t = start + c0 + tk;
      rk[n] = ok ? p.k[t * p.ldk + (long)h * p.dim + i] : 0.f;
      rw[n] = ok ? p.wdec[t * p.ldw + (long)h * p.dim + i] : 0.f;
      if (!LOCAL) rq[n] = ok ? p.q[t * p.ldq + (long)h * p.dim + i] : 0.f;
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int e = threadIdx.x + n * LS_THREADS, tk = e / CBN, cc = blockIdx.z * CBN + e % CBN;
      rv[n] = (tk < nc && cc < p.vdim) ? p.v[(long)(start + c0 + tk) * p.ldv + (long)h * p.vdim + cc] : 0.f;
    }
    if (!LOCAL && (int)threadIdx.x < nc) rkq = p.kq_in[(long)(start + c0 + threadIdx.x) * p.H + h];
  };
  request(0);
  for (int c0 = 0; c0 < rows; c0 += CT) {
    const int nc = min(CT, rows - c0);
    __syncthreads();
#pragma unroll
    for (int n = 0; n < NQK; ++n) {
      const int e = threadIdx.x + n * LS_THREADS, tk = e / DKP, i = e % DKP;
      if (e < CT * DKP) {
        const int at = (i / LS_R) * LS_RS + (i % LS_R);
        ks[tk][at] = rk[n]; ws[tk][at] = rw[n];
        if (!LOCAL) qs[tk][at] = rq[n];
      }
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int e = threadIdx.x + n * LS_THREADS;
      if (e < CT * CBN) vs[e / CBN][e % CBN] = rv[n];
    }
    if (!LOCAL && (int)threadIdx.x < nc) kq[threadIdx.x] = rkq;
    __syncthreads();
    if (c0 + CT < rows) request(c0 + CT);
    float* op = p.out + (long)(start + c0) * p.ldo + (long)h * p.vdim + col0;
    const float* kp = &ks[0][r * LS_RS];
    const float* wp = &ws[0][r * LS_RS];
    const float* qp = &qs[0][LOCAL ? 0 : r * LS_RS];
#pragma unroll 2
    for (int tk = 0; tk < nc; ++tk, op += p.ldo, kp += LD, wp += LD) {
      const float4 k0 = *reinterpret_cast<const float4*>(kp), k1 = *reinterpret_cast<const float4*>(kp + 4);
      const float4 w0 = *reinterpret_cast<const float4*>(wp), w1 = *reinterpret_cast<const float4*>(wp + 4);
      const float k_[LS_R] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
      const float w_[LS_R] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      float vin[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) vin[c] = vs[tk][cj * NC + c];
      if (LOCAL) {
#pragma unroll
        for (int i = 0; i < LS_R; ++i) Dacc[i] *= w_[i];
      } else {
        const float4 q0 = *reinterpret_cast<const float4*>(qp), q1 = *reinterpret_cast<const float4*>(qp + 4);
        qp += LD;
        const float q_[LS_R] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        float dq[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          float b0 = 0.f, b1 = 0.f;
#pragma unroll
          for (int i = 0; i < LS_R; i += 2) { b0 = fmaf(S[c][i], q_[i], b0); b1 = fmaf(S[c][i + 1], q_[i + 1], b1); }
          dq[c] = b0 + b1;
        }
#pragma unroll
        for (int o = 1; o < P; o <<= 1)
#pragma unroll
          for (int c = 0; c < NC; ++c) dq[c] += __shfl_xor_sync(0xffffffffu, dq[c], o);
        if (r == 0) {
#pragma unroll
          for (int c = 0; c < NC; ++c)
            if (col0 + c < p.vdim) op[c] = fmaf(vin[c], kq[tk], dq[c]);
        }
      }
#pragma unroll
      for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < LS_R; ++i) S[c][i] = fmaf(k_[i], vin[c], w_[i] * S[c][i]);
    }
  }
  if (LOCAL) {
    float* sl = p.part_state + ((long)seq * p.n_parts + part) * p.H * head_floats;
#pragma unroll
    for (int c = 0; c < NC; ++c)
      if (col0 + c < p.vdim) {
#pragma unroll
        for (int i = 0; i < LS_R; ++i) sl[(((long)h * LS_R + i) * p.vdim + col0 + c) * P + r] = S[c][i];
      }
    if (col0 == 0) {
      float* dl = p.part_decay + (((long)seq * p.n_parts + part) * p.H + h) * (P * LS_R);
#pragma unroll
      for (int i = 0; i < LS_R; ++i) dl[r * LS_R + i] = Dacc[i];
    }
    return;
  }
  if (last_part) {
    float* st = p.state + (long)p.slot[start] * p.slot_stride;
#pragma unroll
    for (int c = 0; c < NC; ++c)
      if (col0 + c < p.vdim) {
#pragma unroll
        for (int i = 0; i < LS_R; ++i) st[(((long)h * LS_R + i) * p.vdim + col0 + c) * P + r] = S[c][i];
      }
  }
}

// the start state of every part after a sequence's first: S <- diag(part's decay product) S + S_local, part after part
__global__ void state_parts_chain_kernel(StateP p, int P) {
  const int seq = blockIdx.x, h = blockIdx.y;
  const int start = p.seqs[2 * seq], rows = p.seqs[2 * seq + 1];
  const int n = (rows + p.part_len - 1) / p.part_len;
  const long head_floats = (long)LS_R * p.vdim * P;
  const float* st = p.state + (long)p.slot[start] * p.slot_stride + (long)h * head_floats;
  const bool fresh = p.pos[start] == 0;
  for (long e = (long)blockIdx.z * blockDim.x + threadIdx.x; e < head_floats; e += (long)blockDim.x * gridDim.z) {
    const int i = (int)(e / ((long)p.vdim * P)), r = (int)(e % P);
    float S = fresh ? 0.f : st[e];
    for (int c = 0; c + 1 < n; ++c) {
      const long at = (long)seq * p.n_parts + c;
      float* sl = p.part_state + (at * p.H + h) * head_floats + e;
      S = fmaf(p.part_decay[(at * p.H + h) * (P * LS_R) + r * LS_R + i], S, *sl);
      *sl = S;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// what follows a mixer's heads, written into a column range of the buffer the output projection reads:
//   out[t][c] = scale * o[t][c] * [ rsqrt(mean over its group of `span` numbers + eps) * w[c mod w_len] ] * act(gate)
// with the gate one number per element or per head, through a sigmoid or silu.  A warp per norm group.
struct HeadPostP {
  const float* o; long ldi;
  const float* gate; long ldg;
  const bf16* w; int w_len;
  float eps; int span;             // 0: no norm
  int gate_per_head, gate_silu, dv, n;
  float scale;
  float* out; long ldo;
  int gate_first;                  // the gate multiplies o BEFORE the norm (the mean square is that of the gated numbers)
  int wide;                        // a whole block per norm group (long groups, or few tokens: a step of one token
};                                 // still spreads over many blocks) instead of a warp per group
__global__ void head_post_kernel(HeadPostP p) {
  // a norm group of up to 1024 numbers belongs to one warp (blockIdx.y counts warps' worth of groups), a longer one
  // to a whole block (blockIdx.y = the group): a step of one token still spreads over many blocks
  __shared__ float red[32];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int span = p.span > 0 ? p.span : p.dv, groups = p.n / span;
  const bool wide = p.wide != 0;
  const int gi = wide ? (int)blockIdx.y : (int)blockIdx.y * nw + warp;
  if (gi >= groups) return;                    // whole warps (or, wide, whole blocks) leave together
  const int me = wide ? threadIdx.x : lane, step = wide ? blockDim.x : 32;
  const float* o = p.o + (long)t * p.ldi + (long)gi * span;
  const float* g = p.gate ? p.gate + (long)t * p.ldg : nullptr;
  float* out = p.out + (long)t * p.ldo + (long)gi * span;
  float inv = 1.f;
  if (p.span > 0) {
    float ss = 0.f;
#pragma unroll 4
    for (int i = me; i < span; i += step) {
      float v = o[i];
      if (p.gate_first && g) {
        const int c = gi * span + i;
        const float z = g[p.gate_per_head ? c / p.dv : c];
        v *= p.gate_silu ? silu_exact(z) : sigmoid_exact(z);
      }
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (wide) {                                // fixed order: lanes, then the warps one after the other
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      ss = 0.f;
      for (int w = 0; w < nw; ++w) ss += red[w];
    }
    inv = 1.0f / sqrtf(ss / (float)span + p.eps);
  }
#pragma unroll 4
  for (int i = me; i < span; i += step) {
    const int c = gi * span + i;
    float v = o[i], gv = 1.f;
    if (g) {
      const float z = g[p.gate_per_head ? c / p.dv : c];
      gv = p.gate_silu ? silu_exact(z) : sigmoid_exact(z);
    }
    if (p.gate_first) v = v * gv * inv;
    else v *= inv;
    if (p.w) v *= bf2f(p.w[c % p.w_len]);
    if (!p.gate_first) v *= gv;
    out[i] = v * p.scale;
  }
}

// gated feed-forward activation with clamps: g = min(a, lim), u = clamp(b, -lim, lim),
// y = g sigmoid(alpha (g + cubic g^3)) (u + up_off)
// (lim = +inf, alpha = 1, cubic = 0, up_off = 0: the plain silu-gated unit; alpha = 2 sqrt(2 / pi), cubic = 0.044715: the
// tanh form of gelu on the gate, since 0.5 (1 + tanh a) = sigmoid(2 a))
__global__ void glu_clamp_kernel(const float* __restrict__ G, long ldg, const float* __restrict__ U, long ldu, float lim,
                                 float alpha, float cubic, float up_off, float* __restrict__ Y, long ldy, int n) {
  const int t = blockIdx.x, i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float g = fminf(G[(long)t * ldg + i], lim);
  const float u = fminf(fmaxf(U[(long)t * ldu + i], -lim), lim);
  Y[(long)t * ldy + i] = g * sigmoid_exact(alpha * glu_arg(g, cubic)) * (u + up_off);
}
// the same, four columns per thread (rows of whole, aligned 16-byte vectors)
__global__ void glu_clamp4_kernel(const float* __restrict__ G, long ldg, const float* __restrict__ U, long ldu, float lim,
                                  float alpha, float cubic, float up_off, float* __restrict__ Y, long ldy, int n) {
  const int t = blockIdx.x, i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  const float4 a = *reinterpret_cast<const float4*>(G + (long)t * ldg + i);
  const float4 b = *reinterpret_cast<const float4*>(U + (long)t * ldu + i);
  const float gs[4] = {a.x, a.y, a.z, a.w}, us[4] = {b.x, b.y, b.z, b.w};
  float y[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float g = fminf(gs[e], lim), u = fminf(fmaxf(us[e], -lim), lim);
    y[e] = g * sigmoid_exact(alpha * glu_arg(g, cubic)) * (u + up_off);
  }
  *reinterpret_cast<float4*>(Y + (long)t * ldy + i) = make_float4(y[0], y[1], y[2], y[3]);
}

// the same, written as the bf16 operand rows of the next tensor-core product (zero-padded to Kp columns)
__global__ void glu_clamp_bf16_kernel(const float* __restrict__ G, long ldg, const float* __restrict__ U, long ldu, float lim,
                                      float alpha, float cubic, float up_off, bf16* __restrict__ Y, int n, int Kp,
                                      const int* __restrict__ live) {
  const long t = blockIdx.x;
  const bool pad = live && live[t] < 0;          // a padding row of a sorted segment: zeros, its inputs are not read
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < Kp; i += blockDim.x * gridDim.y) {
    float y = 0.f;
    if (i < n && !pad) {
      const float g = fminf(G[t * ldg + i], lim), u = fminf(fmaxf(U[t * ldu + i], -lim), lim);
      y = g * sigmoid_exact(alpha * glu_arg(g, cubic)) * (u + up_off);
    }
    Y[t * Kp + i] = f2bf(y);
  }
}

// four columns per thread (rows of whole, aligned 16-byte vectors; n and Kp multiples of 4)
__global__ void glu_clamp_bf16x4_kernel(const float* __restrict__ G, long ldg, const float* __restrict__ U, long ldu, float lim,
                                        float alpha, float cubic, float up_off, bf16* __restrict__ Y, int n, int Kp,
                                        const int* __restrict__ live) {
  const long t = blockIdx.x;
  const bool pad = live && live[t] < 0;
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4; i < Kp; i += blockDim.x * gridDim.y * 4) {
    float y[4] = {0.f, 0.f, 0.f, 0.f};
    if (i < n && !pad) {
      const float4 a = *reinterpret_cast<const float4*>(G + t * ldg + i);
      const float4 b = *reinterpret_cast<const float4*>(U + t * ldu + i);
      const float gs[4] = {a.x, a.y, a.z, a.w}, us[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float g = fminf(gs[e], lim), u = fminf(fmaxf(us[e], -lim), lim);
        y[e] = g * sigmoid_exact(alpha * glu_arg(g, cubic)) * (u + up_off);
      }
    }
    const __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
    uint2 pk;
    pk.x = *reinterpret_cast<const unsigned*>(&lo);
    pk.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(Y + t * Kp + i) = pk;
  }
}

// ---------------------------------------------------------------------------------------------------------
// Operands of the tensor-core attention of a prompt step (bf16 serving mode; the two products are the weight-major
// tcgen05 GEMM with fp32 output): the `rep` query heads that share a key/value head as bf16 rows (t, r), padded with
// zeros to Kp columns; and the softmax of their score rows against the keys at positions key0 .. key0 + n_keys - 1 —
// visible: max(start of pos's block, pos - window + 1, key0) .. pos — with the sink logit of the row's head in the
// denominator, written as bf16 probabilities (normalised in fp32 before the rounding), zero where nothing is seen
__global__ void heads_to_bf16_kernel(const float* __restrict__ q, long ldq, int rep, int dim, bf16* __restrict__ out,
                                     int Kp) {
  const int i = blockIdx.x, t = i / rep, r = i % rep;
  const float* x = q + (long)t * ldq + r * dim;
  for (int k = threadIdx.x; k < Kp; k += blockDim.x) out[(long)i * Kp + k] = f2bf(k < dim ? x[k] : 0.f);
}
__global__ void sink_softmax_bf16_kernel(const float* __restrict__ S, long lds, const int* __restrict__ pos, int rep,
                                         const bf16* __restrict__ sink, float scale, int chunk, int window, int key0,
                                         float bias_exp, int head0, int H, int unit_sink, int split,
                                         bf16* __restrict__ P, long ldp, int Sp) {
  __shared__ float red[32];
  const long r = blockIdx.x;
  const int ps = pos[r / rep];
  int lo = key0;
  if (chunk > 0) lo = max(lo, (ps / chunk) * chunk);
  if (window > 0) lo = max(lo, ps - window + 1);
  const int j0 = lo - key0, j1 = ps - key0;            // visible columns j0 .. j1
  const float* s = S + r * lds;
  const float sk = sink ? bf2f(sink[r % rep]) : (unit_sink ? 0.f : -INFINITY);
  const float slope = bias_exp > 0.f ? exp2f(-bias_exp * (float)(head0 + (int)(r % rep) + 1) / (float)H) : 0.f;
  // the score of column j: scale s_j - slope (distance to the query); j1 - j is that distance
  auto sc = [&](int j) { return s[j] * scale - slope * (float)(j1 - j); };
  float m = sk;
  for (int j = j0 + threadIdx.x; j <= j1; j += blockDim.x) m = fmaxf(m, sc(j));
  m = warp_max(m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
  float sum = 0.f;
  for (int j = j0 + threadIdx.x; j <= j1; j += blockDim.x) sum += expf(sc(j) - m);
  const float tot = block_sum_fixed(sum, red) + ((sink || unit_sink) ? expf(sk - m) : 0.f);
  const float inv = 1.0f / tot;
  // split: the probability as two bf16 parts [hi | lo] (Sp columns each), lo = the rounding error of hi: the next
  // product multiplies both by the values and sums them in its fp32 accumulator, so the weights keep 16 mantissa bits
  for (int j = threadIdx.x; j < Sp; j += blockDim.x) {
    const float pr = (j >= j0 && j <= j1) ? expf(sc(j) - m) * inv : 0.f;
    const bf16 hi = f2bf(pr);
    P[r * ldp + j] = hi;
    if (split) P[r * ldp + Sp + j] = f2bf(pr - bf2f(hi));
  }
}

unsigned long long g_sink_attr_f32 = 0, g_sink_attr_bf16 = 0;

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_lm_short_conv(const float* U, long ldu, const void* w, float* Y, long ldy, float* state, long slot_stride,
                       const int* slot, const int* pos, const int* first, const int* seqs, int n_seq, int C, int taps,
                       int act, const void* bias, int residual, int single, int T, void* st) {
  B200_REQUIRE(U && w && Y && (state || taps == 1) && slot && pos && first && seqs && T > 0 && n_seq > 0 && C > 0 && taps > 0,
               "lm_short_conv: bad argument");     // one tap keeps nothing between steps
  ConvP p{U, ldu, (const bf16*)w, Y, ldy, state, slot_stride, slot, pos, first, C, taps, act, (const bf16*)bias, residual, single};
  const int by = cdiv(C, 256) < 8 ? cdiv(C, 256) : 8;
  short_conv_kernel<<<dim3(T, by), 256, 0, (cudaStream_t)st>>>(p);
  B200_CHECK_LAUNCH();
  if (taps > 1 && !single) {
    conv_state_kernel<<<dim3(n_seq, by), 256, 0, (cudaStream_t)st>>>(p, seqs);
    B200_CHECK_LAUNCH();
  }
  return B200_OK;
}

int b200_lm_token_shift(const float* h, long ldh, const void* mu, void* M, long ldm, long mix_stride, float* state,
                        long slot_stride, const int* slot, const int* pos, const int* first, const int* seqs, int n_seq, int C,
                        int n_mix, int single, int out_bf16, int T, void* st) {
  B200_REQUIRE(h && mu && M && state && slot && pos && first && seqs && T > 0 && n_seq > 0 && C > 0 && n_mix > 0,
               "lm_token_shift: bad argument");
  B200_REQUIRE(!out_bf16 || ldm >= C, "lm_token_shift: operand rows of %ld columns for %d channels", ldm, C);
  ShiftP p{h, ldh, (const bf16*)mu, out_bf16 ? nullptr : (float*)M, ldm, mix_stride, state, slot_stride, slot, pos, first, C, n_mix, single,
           out_bf16 ? (bf16*)M : nullptr, ldm, mix_stride};
  const int by = cdiv(C, 256) < 8 ? cdiv(C, 256) : 8;
  token_shift_kernel<<<dim3(T, by), 256, 0, (cudaStream_t)st>>>(p);
  B200_CHECK_LAUNCH();
  if (!single) {
    token_shift_state_kernel<<<dim3(n_seq, by), 256, 0, (cudaStream_t)st>>>(p, seqs);
    B200_CHECK_LAUNCH();
  }
  return B200_OK;
}

int b200_lm_qkv_post(float* Q, long ldq, const float* K, long ldk, const float* V, long ldv, void* cache, int cache_bf16,
                     long slot_stride, long tok_stride, const int* slot, const int* pos, const float* cs, int H, int G,
                     int dim, int vdim, int rot_dims, const void* qn_w, const void* kn_w, float eps, int v_unit, float qt_coef,
                     int qt_every, const void* vmix, const float* v_first, long ldvf, float* v_keep, long ldvk, int T, void* st) {
  B200_REQUIRE(Q && K && V && cache && slot && pos && T > 0 && H > 0 && G > 0, "lm_qkv_post: bad argument");
  B200_REQUIRE(!vmix || v_first, "lm_qkv_post: value mixing needs the first layer's values");
  B200_REQUIRE(rot_dims % 2 == 0 && rot_dims <= dim && (rot_dims == 0 || cs), "lm_qkv_post: rotated dims %d of %d", rot_dims, dim);
  if (cache_bf16) {
    QkvPostP<bf16> p{Q, ldq, K, ldk, V, ldv, (bf16*)cache, slot_stride, tok_stride, slot, pos, (const float2*)cs, H, G, dim, vdim, rot_dims,
                      (const bf16*)qn_w, (const bf16*)kn_w, eps, v_unit, qt_coef, qt_every, (const bf16*)vmix, v_first, ldvf, v_keep, ldvk};
    qkv_post_kernel<bf16><<<T, 256, 0, (cudaStream_t)st>>>(p);
  } else {
    QkvPostP<float> p{Q, ldq, K, ldk, V, ldv, (float*)cache, slot_stride, tok_stride, slot, pos, (const float2*)cs, H, G, dim, vdim, rot_dims,
                       (const bf16*)qn_w, (const bf16*)kn_w, eps, v_unit, qt_coef, qt_every, (const bf16*)vmix, v_first, ldvf, v_keep, ldvk};
    qkv_post_kernel<float><<<T, 256, 0, (cudaStream_t)st>>>(p);
  }
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_sink_attention(const float* q, long ldq, const void* cache, int cache_bf16, long slot_stride, long tok_stride,
                           const int* slot, const int* pos, float* out, long ldo, const void* sink, int H, int G,
                           int dim, int vdim, float scale, int chunk, int window, float bias_exp, int unit_sink, float* part,
                           int n_split, int T, void* st) {
  B200_REQUIRE(q && cache && slot && pos && out && T > 0 && H > 0 && G > 0 && H % G == 0, "lm_sink_attention: bad argument");
  B200_REQUIRE(vdim <= 256, "lm_sink_attention: value size %d not supported", vdim);
  B200_REQUIRE(!(sink && unit_sink), "lm_sink_attention: a sink logit per head or the constant one, not both");
  if (n_split < 1 || !part) n_split = 1;
  B200_REQUIRE(n_split <= 64, "lm_sink_attention: at most 64 splits");
  const int rep = H / G, nw = rep < 8 ? rep : 8;
  const size_t smem = ((size_t)SA_KT * (dim + ((dim & 3) == 0 ? 4 : 1)) + (size_t)SA_KT * vdim + (size_t)nw * dim) * sizeof(float);
  B200_REQUIRE(smem <= 200 * 1024, "lm_sink_attention: rows of %d + %d numbers do not fit shared memory", dim, vdim);
  dim3 grid(T, G * cdiv(rep, nw), n_split);
  if (cache_bf16) {
    if (first_use_on_device(&g_sink_attr_bf16))
      B200_CUDA(cudaFuncSetAttribute(sink_attention_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    const int vec = dim % 8 == 0 && vdim % 8 == 0 && tok_stride % 8 == 0 && slot_stride % 8 == 0 && ((uintptr_t)cache & 15) == 0;
    SinkAttnP<bf16> p{q, ldq, (const bf16*)cache, slot_stride, tok_stride, slot, pos, out, ldo, (const bf16*)sink, H, G, dim, vdim, scale, chunk, window, part, n_split, vec, bias_exp, unit_sink};
    sink_attention_kernel<bf16><<<grid, nw * 32, smem, (cudaStream_t)st>>>(p);
  } else {
    if (first_use_on_device(&g_sink_attr_f32))
      B200_CUDA(cudaFuncSetAttribute(sink_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    const int vec = dim % 4 == 0 && vdim % 4 == 0 && tok_stride % 4 == 0 && slot_stride % 4 == 0 && ((uintptr_t)cache & 15) == 0;
    SinkAttnP<float> p{q, ldq, (const float*)cache, slot_stride, tok_stride, slot, pos, out, ldo, (const bf16*)sink, H, G, dim, vdim, scale, chunk, window, part, n_split, vec, bias_exp, unit_sink};
    sink_attention_kernel<float><<<grid, nw * 32, smem, (cudaStream_t)st>>>(p);
  }
  B200_CHECK_LAUNCH();
  if (n_split > 1) {
    const int mt = vdim >= 256 ? 256 : (vdim + 31) / 32 * 32;
    sink_attention_merge_kernel<<<dim3(T, H), mt, 0, (cudaStream_t)st>>>(part, n_split, vdim, out, ldo, H);
    B200_CHECK_LAUNCH();
  }
  return B200_OK;
}

int b200_lm_linear_state(const float* q, long ldq, const float* k, long ldk, const float* v, long ldv, float* out, long ldo,
                         float* state, long slot_stride, const int* seqs, int n_seq, const int* slot, const int* pos,
                         int H, int rep, int dim, int vdim, int act, float unit_eps, float q_scale,
                         const float* decay_const, const float* a, long lda, const void* A_log, const void* dt_bias,
                         const float* b, long ldb, int delta, int dt_in, const void* skip, const float* wraw, long ldwr,
                         const void* bonus, float* prep, int part_len, int n_parts, float* part_scratch, int T, void* st) {
  B200_REQUIRE(q && k && v && out && state && seqs && slot && pos && n_seq > 0 && H > 0 && rep > 0 && H % rep == 0,
               "lm_linear_state: bad argument");
  B200_REQUIRE(dim > 0 && dim <= 32 * LS_R && vdim > 0, "lm_linear_state: key size %d not supported (at most %d)", dim, 32 * LS_R);
  const bool chan = wraw != nullptr;
  B200_REQUIRE(chan || decay_const || (a && A_log && dt_bias), "lm_linear_state: a decay per head, or the inputs of a computed one");
  B200_REQUIRE(!chan || (bonus && rep == 1 && !delta && !dt_in && !act && unit_eps == 0.f && !skip && !decay_const),
               "lm_linear_state: a decay per key channel comes with a bonus and nothing else");
  B200_REQUIRE(!dt_in || (!decay_const && !delta && !b), "lm_linear_state: the step size scales the input only in the plain form with a computed decay");
  StateP p{q, ldq, k, ldk, v, ldv, out, ldo, state, slot_stride, seqs, slot, pos, H, rep, dim, vdim, act, unit_eps, q_scale,
           nullptr, nullptr, nullptr, decay_const, a, lda, (const bf16*)A_log, (const bf16*)dt_bias, b, ldb, delta, dt_in, (const bf16*)skip, wraw, ldwr, (const bf16*)bonus, 0, 0, nullptr, nullptr};
  const cudaStream_t cs = (cudaStream_t)st;
  if (prep) {     // scratch of T * (2 Hk dim + Hk + 2 H) floats: the per-token work runs first, over all tokens at once
    B200_REQUIRE(T > 0, "lm_linear_state: the prepared path needs the number of tokens");
    const int Hk = H / rep;
    const long n = (long)Hk * dim;
    // scratch: the same T * (2 Hk dim + Hk + 2 H) floats, or, with a decay per channel, T * (3 H dim + H)
    float *qn = prep, *kn = qn + (long)T * n, *kq = kn + (long)T * n, *dec = kq + (long)T * Hk, *bet = dec + (long)T * H;
    StatePrepP pp{q, ldq, k, ldk, qn, kn, n, kq, dec, bet, H, Hk, dim, act, unit_eps, q_scale, decay_const, a, lda,
                  (const bf16*)A_log, (const bf16*)dt_bias, b, ldb, dt_in, wraw, ldwr, chan ? dec : nullptr, (const bf16*)bonus};
    if (chan) { p.wdec = dec; p.ldw = n; }
    state_prep_kernel<<<T, 128, 0, cs>>>(pp);
    B200_CHECK_LAUNCH();
    if (!chan) { p.q = qn; p.ldq = n; p.k = kn; p.ldk = n; }
    p.kq_in = kq; p.dec_in = dec; p.bet_in = bet;
  }
  const dim3 block(LS_THREADS);
  const bool parts = chan && prep && n_parts > 1 && part_len > 0 && part_scratch;
#define LS_LAUNCH(PP)                                                                                            \
  do {                                                                                                           \
    const dim3 grid(n_seq, H, cdiv(vdim, LS_THREADS / PP));                                                      \
    if (parts) {     /* scratch: n_seq * n_parts * (H LS_R vdim PP + H PP LS_R) floats */                        \
      p.part_len = part_len; p.n_parts = n_parts; p.part_state = part_scratch;                                   \
      p.part_decay = part_scratch + (long)n_seq * n_parts * H * LS_R * vdim * PP;                                \
      const dim3 pgrid(n_seq * n_parts, H, cdiv(vdim, 2 * (LS_THREADS / PP)));                                   \
      channel_state_kernel<PP, 2, true><<<pgrid, block, 0, cs>>>(p);                                             \
      state_parts_chain_kernel<<<dim3(n_seq, H, cdiv(LS_R * vdim * PP, 1024)), 256, 0, cs>>>(p, PP);             \
      channel_state_kernel<PP, 2, false><<<pgrid, block, 0, cs>>>(p);                                            \
    } else if (chan && prep) {                                                                                   \
      channel_state_kernel<PP, 2, false><<<dim3(n_seq, H, cdiv(vdim, 2 * (LS_THREADS / PP))), block, 0, cs>>>(p); \
    } else if (chan) linear_state_kernel<PP, false, true><<<grid, block, 0, cs>>>(p);                            \
    else if (delta) linear_state_kernel<PP, true, false><<<grid, block, 0, cs>>>(p);                             \
    else linear_state_kernel<PP, false, false><<<grid, block, 0, cs>>>(p);                                       \
  } while (0)
  if (dim <= LS_R) LS_LAUNCH(1);
  else if (dim <= 2 * LS_R) LS_LAUNCH(2);
  else if (dim <= 4 * LS_R) LS_LAUNCH(4);
  else if (dim <= 8 * LS_R) LS_LAUNCH(8);
  else if (dim <= 16 * LS_R) LS_LAUNCH(16);
  else LS_LAUNCH(32);
#undef LS_LAUNCH
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_heads_to_bf16(const float* q, long ldq, int rep, int dim, void* out, int Kp, int T, void* st) {
  B200_REQUIRE(q && out && T > 0 && rep > 0 && dim > 0 && Kp >= dim, "lm_heads_to_bf16: bad argument");
  heads_to_bf16_kernel<<<T * rep, 128, 0, (cudaStream_t)st>>>(q, ldq, rep, dim, (bf16*)out, Kp);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_sink_softmax_bf16(const float* S, long lds, const int* pos, int rep, const void* sink, float scale, int chunk,
                              int window, int key0, float bias_exp, int head0, int H, int unit_sink, int split, void* P,
                              long ldp, int rows, int Sp, void* st) {
  B200_REQUIRE(S && pos && P && rows > 0 && rep > 0 && Sp > 0 && key0 >= 0, "lm_sink_softmax_bf16: bad argument");
  sink_softmax_bf16_kernel<<<rows, 256, 0, (cudaStream_t)st>>>(S, lds, pos, rep, (const bf16*)sink, scale, chunk, window,
                                                                key0, bias_exp, head0, H > 0 ? H : 1, unit_sink, split, (bf16*)P, ldp, Sp);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_head_post(const float* o, long ldi, const float* gate, long ldg, const void* w, int w_len, float eps, int span,
                      int gate_per_head, int gate_silu, int dv, int n, float scale, float* out, long ldo, int gate_first,
                      int T, void* st) {
  B200_REQUIRE(o && out && T > 0 && n > 0 && dv > 0 && n % dv == 0, "lm_head_post: bad argument");
  B200_REQUIRE(span == 0 || n % span == 0, "lm_head_post: norm groups of %d numbers in rows of %d", span, n);
  B200_REQUIRE(!w || w_len > 0, "lm_head_post: a weight needs its length");
  const int grp = span > 0 ? span : dv, groups = n / grp;
  const int wide = grp > 1024 || (grp >= 256 && (long)T * groups <= 256);
  HeadPostP p{o, ldi, gate, ldg, (const bf16*)w, w_len, eps, span, gate_per_head, gate_silu, dv, n, scale, out, ldo, gate_first, wide};
  head_post_kernel<<<dim3(T, wide ? groups : cdiv(groups, 8)), 256, 0, (cudaStream_t)st>>>(p);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_glu_clamp(const float* G, long ldg, const float* U, long ldu, float limit, float alpha, float cubic, float up_off,
                      float* Y, long ldy, int n, int T, void* st) {
  B200_REQUIRE(G && U && Y && T > 0 && n > 0, "lm_glu_clamp: bad argument");
  const bool v4 = n % 4 == 0 && ldg % 4 == 0 && ldu % 4 == 0 && ldy % 4 == 0 &&
                  (((uintptr_t)G | (uintptr_t)U | (uintptr_t)Y) & 15) == 0;
  if (v4 && T > 16) glu_clamp4_kernel<<<dim3(T, cdiv(n, 1024)), 256, 0, (cudaStream_t)st>>>(G, ldg, U, ldu, limit, alpha, cubic, up_off, Y, ldy, n);
  else glu_clamp_kernel<<<dim3(T, cdiv(n, 256)), 256, 0, (cudaStream_t)st>>>(G, ldg, U, ldu, limit, alpha, cubic, up_off, Y, ldy, n);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_glu_clamp_bf16(const float* G, long ldg, const float* U, long ldu, float limit, float alpha, float cubic, float up_off,
                           void* Y, int n, int Kp, const int* live, int T, void* st) {
  B200_REQUIRE(G && U && Y && T > 0 && n > 0 && Kp >= n, "lm_glu_clamp_bf16: bad argument");
  const bool v4 = n % 4 == 0 && Kp % 4 == 0 && ldg % 4 == 0 && ldu % 4 == 0 && (((uintptr_t)G | (uintptr_t)U) & 15) == 0 &&
                  ((uintptr_t)Y & 7) == 0;
  if (v4) glu_clamp_bf16x4_kernel<<<dim3(T, cdiv(Kp, 1024)), 256, 0, (cudaStream_t)st>>>(G, ldg, U, ldu, limit, alpha, cubic, up_off, (bf16*)Y, n, Kp, live);
  else glu_clamp_bf16_kernel<<<dim3(T, cdiv(Kp, 1024)), 256, 0, (cudaStream_t)st>>>(G, ldg, U, ldu, limit, alpha, cubic, up_off, (bf16*)Y, n, Kp, live);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

}  // extern "C"
