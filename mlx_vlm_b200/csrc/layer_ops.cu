// Layer-level ops for decoder designs that are assembled layer by layer on the host (models/layer_ops.py):
//   * fp32 residual stream with the norm on the sublayer's OUTPUT (x += norm(y)), RMS norms whose weight is
//     stored either plainly or around zero (`w_offset`),
//   * latent attention: queries through a low-rank latent, keys / values expanded from ONE cached latent row
//     per token (+ one rotated key part shared by all heads).  The cache holds [latent | rotated part] rows;
//     attention runs in the ABSORBED form: the key up-projection is folded into the query
//     (q~_h = W_uk,h^T q_h, one row of kv_rank numbers per head), scores are q~_h . c_j + q_rot,h . k_rot,j, the
//     softmax-weighted sum is taken over the latent rows themselves and the value up-projection is applied to
//     that sum afterwards.  Every query token names its cache row (slot) and position, so a whole prompt, a
//     portion of one, one decoded token and a batch of unequal requests are the same launch,
//   * rotate-half rotary on the first `dims` numbers of a vector, angles from a double-precision table,
//   * mixture of experts: fp32 router logits -> top-k (lowest index wins ties) -> softmax over the chosen
//     logits; tokens are grouped per expert and the expert GEMMs run as ONE grouped launch each,
//   * a general row GEMM  Y = X . W^T  with bf16 weights and fp32 accumulation in a fixed k order (the result
//     of a row never depends on which other rows are in the launch), optionally batched (heads, experts) and
//     gathered / scattered through row lists, and its skinny sibling for decode steps (a warp per weight row).
// fp32 buffers everywhere except the weights (bf16) and, in the bf16 serving mode, the cache rows and the
// operands of the matrix products (rounded to bf16 on load: `round_x`).
#include "common.cuh"

namespace b200 {
namespace {

__device__ __forceinline__ float ld_act(const float* p) { return *p; }
__device__ __forceinline__ float ld_act(const bf16* p) { return bf2f(*p); }
__device__ __forceinline__ void st_act(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_act(bf16* p, float v) { *p = f2bf(v); }

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];   // same order in every thread
  return t;
}

// ---------------------------------------------------------------------------------------------------------
// embedding: x[t] = embed[token[t]] * scale  (fp32)
__global__ void embed_scale_kernel(const int* __restrict__ tok, const bf16* __restrict__ emb, float scale,
                                   float* __restrict__ x, int W, int vocab) {
  const int t = blockIdx.x;
  int id = tok[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  for (int i = threadIdx.x; i < W; i += blockDim.x) x[(long)t * W + i] = bf2f(emb[(long)id * W + i]) * scale;
}

// ---------------------------------------------------------------------------------------------------------
// rotary table: cs[t][i] = amp * (cos, sin)(pos[t] * inv_freq[i]) with the angle in double precision (amp: the
// amplitude that a frequency scaling puts on both, 1 without one)
__global__ void rope_table_kernel(const int* __restrict__ pos, const double* __restrict__ inv_freq,
                                  float2* __restrict__ cs, int T, int half, float amp) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const double a = (double)pos[i / half] * inv_freq[i % half];
  double s, c;
  sincos(a, &s, &c);
  cs[i] = make_float2((float)c * amp, (float)s * amp);
}

// ---------------------------------------------------------------------------------------------------------
// RMS norm of y's rows (optionally the weighted sum of `top` rows of a scattered buffer), weight (w_offset + w),
// then either out = norm or x += norm.  rows: optional gather list for the input row.  center: the row's mean is
// taken off first and the root mean square is that of the deviations (a layer norm without bias).  groups > 1: the row
// is `groups` equal consecutive parts, each divided by its own root mean square (no centering then).
struct NormP {
  const float* y; long ldy;
  const float* wgt; int top;          // combine: y row = sum_s wgt[t*top+s] * y[(t*top+s)]
  const bf16* w; float w_offset, eps;
  float* x; long ldx;                 // x += norm  (add != 0)  or  x = norm
  int add;
  const int* rows;                    // input row of output t (NULL: t)
  int N;
  int center;
  // a residual update in front of the norm (res != NULL; no `rows`): the normed row is
  // res[t] <- res[t] + ls * (y row (or the combined rows) + sigmoid(sgate[t]) shared[t]), stored back, then normed into x
  float* res; long ldr;
  const bf16* ls;
  const float* shared; long lds;
  const float* sgate; long ldsg;
  int groups;                         // parts of the row with a root mean square of their own (1: the whole row)
  float mult;                         // the residual update is scaled by this number as well (beside ls)
};
__global__ void norm_rows_kernel(NormP p) {
  extern __shared__ float sm[];
  float* row = sm;                    // N
  float* red = sm + p.N;              // 32
  const int t = blockIdx.x;
  const long r = p.rows ? p.rows[t] : t;
  const float sg = (p.res && p.shared) ? (p.sgate ? 1.0f / (1.0f + expf(-p.sgate[r * p.ldsg])) : 1.f) : 0.f;
  float ss = 0.f;
  for (int i = threadIdx.x; i < p.N; i += blockDim.x) {
    float v;
    if (p.top > 0) {
      v = 0.f;
      for (int s = 0; s < p.top; ++s) v += p.wgt[r * p.top + s] * p.y[(r * p.top + s) * p.ldy + i];
    } else {
      v = p.y[r * p.ldy + i];
    }
    if (p.res) {                      // the same arithmetic, in the same order, as residual_rows_kernel
      if (p.shared) v = fmaf(sg, p.shared[r * p.lds + i], v);
      float* o = p.res + r * p.ldr + i;
      v = fmaf((p.ls ? bf2f(p.ls[i]) : 1.f) * p.mult, v, *o);
      *o = v;
    }
    row[i] = v;
    ss += p.center ? v : v * v;
  }
  if (p.groups > 1) {                 // a warp per part, lanes striding it: the order of the sum is fixed by the part's size
    float* ginv = red + 32;           // groups
    __syncthreads();
    const int span = p.N / p.groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int g = warp; g < p.groups; g += nw) {
      float a = 0.f;
      for (int i = lane; i < span; i += 32) { const float v = row[g * span + i]; a = fmaf(v, v, a); }
      a = warp_sum(a);
      if (lane == 0) ginv[g] = 1.0f / sqrtf(a / (float)span + p.eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.N; i += blockDim.x) {
      const float v = row[i] * ginv[i / span] * (p.w_offset + bf2f(p.w[i]));
      float* o = p.x + (long)t * p.ldx + i;
      *o = p.add ? *o + v : v;
    }
    return;
  }
  float tot = block_sum(ss, red), mean = 0.f;
  if (p.center) {                     // two passes over the staged row: mean, then the squared deviations
    mean = tot / (float)p.N;
    ss = 0.f;
    for (int i = threadIdx.x; i < p.N; i += blockDim.x) { const float d = row[i] - mean; ss = fmaf(d, d, ss); }
    tot = block_sum(ss, red);
  }
  const float inv = 1.0f / sqrtf(tot / (float)p.N + p.eps);
  for (int i = threadIdx.x; i < p.N; i += blockDim.x) {
    const float v = (row[i] - mean) * inv * (p.w_offset + bf2f(p.w[i]));
    float* o = p.x + (long)t * p.ldx + i;
    *o = p.add ? *o + v : v;
  }
}

// ---------------------------------------------------------------------------------------------------------
// after the fused down-projection D[t] = [ q latent (q_rank) | kv latent (kv_rank) | key rot part (rot_dim) ]:
// cq = rms(q latent) * wq ; c = rms(kv latent) * wkv -> cache[slot][pos][0:kv_rank] ; rope(rot part) -> cache[..][kv_rank:]
template <typename CT>
struct LatentPostP {
  const float* D; long ldd;
  const bf16 *wq, *wkv;
  float eps;
  float* cq; long ldq;
  CT* cache; long slot_stride, tok_stride;   // elements
  const int *slot, *pos;
  const float2* cs;                          // [T][rot_dims/2]
  int q_rank, kv_rank, rot_dim, rot_dims, own_kv;
  int pairs;                                 // the rotation pairs (2i, 2i + 1) instead of (i, i + rot_dims / 2)
};
// element i of a vector r whose first `dims` numbers turn by the table row a[0 .. dims/2)
__device__ __forceinline__ float rope_elem(const float* r, int i, int dims, const float2* a, int pairs) {
  if (i >= dims) return r[i];
  const int half = dims >> 1;
  if (pairs) {
    const float2 c = a[i >> 1];
    return (i & 1) ? r[i] * c.x + r[i - 1] * c.y : r[i] * c.x - r[i + 1] * c.y;
  }
  if (i < half) { const float2 c = a[i]; return r[i] * c.x - r[i + half] * c.y; }
  const float2 c = a[i - half];
  return r[i] * c.x + r[i - half] * c.y;
}
template <typename CT>
__global__ void latent_post_kernel(LatentPostP<CT> p) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const float* d = p.D + (long)t * p.ldd;
  float ss = 0.f, inv = 0.f;
  if (p.q_rank > 0) {                 // a design without a query latent has q_rank 0: the row starts with the kv latent
    for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) ss += d[i] * d[i];
    inv = 1.0f / sqrtf(block_sum(ss, red) / (float)p.q_rank + p.eps);
    for (int i = threadIdx.x; i < p.q_rank; i += blockDim.x) p.cq[(long)t * p.ldq + i] = d[i] * inv * bf2f(p.wq[i]);
  }
  if (!p.own_kv) return;
  const float* k = d + p.q_rank;
  ss = 0.f;
  for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) ss += k[i] * k[i];
  inv = 1.0f / sqrtf(block_sum(ss, red) / (float)p.kv_rank + p.eps);
  CT* c = p.cache + (long)p.slot[t] * p.slot_stride + (long)p.pos[t] * p.tok_stride;
  for (int i = threadIdx.x; i < p.kv_rank; i += blockDim.x) st_act(c + i, k[i] * inv * bf2f(p.wkv[i]));
  const float* r = k + p.kv_rank;
  const int half = p.rot_dims / 2;
  for (int i = threadIdx.x; i < p.rot_dim; i += blockDim.x)
    st_act(c + p.kv_rank + i, rope_elem(r, i, p.rot_dims, p.cs + (long)t * half, p.pairs));
}

// rotated query parts into the absorbed query rows: qa[t][h][kv_rank + i] = rope(q[t][h][dim + i])
__global__ void rope_q_kernel(const float* __restrict__ q, long ldq, int qh_stride, int dim, float* __restrict__ qa,
                              long ldqa, int Dl, int kv_rank, const float2* __restrict__ cs, int H, int rot_dim,
                              int rot_dims, int pairs) {
  const int t = blockIdx.x, half = rot_dims / 2;
  for (int e = threadIdx.x; e < H * rot_dim; e += blockDim.x) {
    const int h = e / rot_dim, i = e % rot_dim;
    const float* r = q + (long)t * ldq + (long)h * qh_stride + dim;
    qa[(long)t * ldqa + (long)h * Dl + kv_rank + i] = rope_elem(r, i, rot_dims, cs + (long)t * half, pairs);
  }
}

// ---------------------------------------------------------------------------------------------------------
// absorbed latent attention.  Block = (query token, group of up to 8 heads); a warp per head.  Keys are the cache
// rows 0..pos[t] of slot[t], staged 32 at a time in shared memory (fp32); lane j scores key j, then the lanes
// share the probabilities and each lane accumulates its columns of the latent sum (online softmax, fp32).
constexpr int LA_KT = 32;
template <typename CT>
struct LatAttnP {
  const float* qa; long ldqa;            // [T][H][Dl]
  const CT* cache; long slot_stride, tok_stride;
  const int *slot, *pos;
  float* out; long ldo;                  // [T][H][kv_rank]
  int H, Dl, kv_rank;
  float scale;
  int round_q;                           // bf16 serving mode: the query operand is rounded like the keys
  float* part;                           // n_split > 1: [T][H][n_split][kv_rank + 2] = (acc.., max, sum) per split
  int n_split;                           // key tiles are dealt round-robin to gridDim.z splits (decode: few queries,
                                         // many keys), a second kernel merges the splits
  int vec8;                              // bf16 cache rows start on 16-byte boundaries and Dl % 8 == 0
  int window;                            // > 0: a query at position p sees the keys p - window + 1 .. p only
};
template <typename CT>
__global__ void latent_attention_kernel(LatAttnP<CT> p) {
  extern __shared__ float sm[];
  const int t = blockIdx.x, hg = blockIdx.y, nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // rows of 4n numbers are padded by 4 (16-byte rows for 128-bit shared loads: a quarter warp's eight rows then
  // fall on all 32 banks), other rows by 1
  const bool v4 = (p.Dl & 3) == 0;
  const int Dl = p.Dl, ldk = Dl + (v4 ? 4 : 1);
  float* keys = sm;                       // [LA_KT][ldk]
  float* qs = sm + LA_KT * ldk;           // [nw][Dl]
  const int h = hg * nw + warp;
  const bool live = h < p.H;
  if (live) {
    const float* q = p.qa + (long)t * p.ldqa + (long)h * Dl;
    for (int i = lane; i < Dl; i += 32) qs[warp * Dl + i] = p.round_q ? rbf(q[i]) : q[i];
  }
  const int n_keys = p.pos[t] + 1;
  const int key_lo = p.window > 0 ? max(n_keys - p.window, 0) : 0;
  const CT* base = p.cache + (long)p.slot[t] * p.slot_stride;
  const int per_lane = (p.kv_rank + 31) / 32;
  float m = -INFINITY, l = 0.f;
  float acc[32];                          // kv_rank <= 1024
#pragma unroll
  for (int i = 0; i < 32; ++i) acc[i] = 0.f;
  for (int k0 = key_lo + blockIdx.z * LA_KT; k0 < n_keys; k0 += LA_KT * p.n_split) {
    const int nk = min(LA_KT, n_keys - k0);
    __syncthreads();
    if (sizeof(CT) == 2 && p.vec8) {         // bf16 rows as 16-byte loads
      const int per_row = Dl >> 3;
      for (int e = threadIdx.x; e < nk * per_row; e += blockDim.x) {
        const int j = e / per_row, i = (e - j * per_row) << 3;
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(base + (long)(k0 + j) * p.tok_stride + i), f);
        *reinterpret_cast<float4*>(&keys[j * ldk + i]) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(&keys[j * ldk + i + 4]) = make_float4(f[4], f[5], f[6], f[7]);
      }
    } else {
      for (int e = threadIdx.x; e < nk * Dl; e += blockDim.x) {
        const int j = e / Dl, i = e % Dl;
        keys[j * ldk + i] = ld_act(base + (long)(k0 + j) * p.tok_stride + i);
      }
    }
    __syncthreads();
    if (!live) continue;
    float s = -INFINITY;
    if (lane < nk) {
      const float* kr = keys + lane * ldk;
      const float* qr = qs + warp * Dl;
      float a = 0.f;
      if (v4) {                              // fixed order: four running sums over i mod 4, then (0 + 1) + (2 + 3)
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 4
        for (int i = 0; i < Dl; i += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qr + i);
          const float4 k4 = *reinterpret_cast<const float4*>(kr + i);
          a0 = fmaf(q4.x, k4.x, a0); a1 = fmaf(q4.y, k4.y, a1); a2 = fmaf(q4.z, k4.z, a2); a3 = fmaf(q4.w, k4.w, a3);
        }
        a = (a0 + a1) + (a2 + a3);
      } else {
        for (int i = 0; i < Dl; ++i) a = fmaf(qr[i], kr[i], a);
      }
      s = a * p.scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);     // first tile: exp(-inf) = 0
    const float pj = lane < nk ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < per_lane) acc[i] *= corr;
    for (int j = 0; j < nk; ++j) {
      const float w = __shfl_sync(0xffffffffu, pj, j);
      const float* kr = keys + j * ldk;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < per_lane) {
          const int d = lane + 32 * i;
          if (d < p.kv_rank) acc[i] = fmaf(w, kr[d], acc[i]);
        }
    }
  }
  if (!live) return;
  if (p.n_split > 1) {                    // un-normalised partial sums; a split without keys has max -inf, sum 0
    float* o = p.part + (((long)t * p.H + h) * p.n_split + blockIdx.z) * (p.kv_rank + 2);
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < per_lane) {
        const int d = lane + 32 * i;
        if (d < p.kv_rank) o[d] = acc[i];
      }
    if (lane == 0) { o[p.kv_rank] = m; o[p.kv_rank + 1] = l; }
    return;
  }
  const float inv = 1.0f / l;
  float* o = p.out + (long)t * p.ldo + (long)h * p.kv_rank;
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (i < per_lane) {
      const int d = lane + 32 * i;
      if (d < p.kv_rank) o[d] = acc[i] * inv;
    }
}

// merge the splits of one (token, head) in a fixed order: out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M)
__global__ void latent_attention_merge_kernel(const float* __restrict__ part, int n_split, int kv_rank,
                                              float* __restrict__ out, long ldo, int H) {
  __shared__ float wgt[64];
  __shared__ float inv_s;
  const int t = blockIdx.x, h = blockIdx.y, row = kv_rank + 2;
  const float* pp = part + ((long)t * H + h) * n_split * row;
  if (threadIdx.x < 32) {                  // n_split <= 64: two per lane
    const int s0 = threadIdx.x, s1 = threadIdx.x + 32;
    const float m0 = s0 < n_split ? pp[(long)s0 * row + kv_rank] : -INFINITY;
    const float m1 = s1 < n_split ? pp[(long)s1 * row + kv_rank] : -INFINITY;
    const float l0 = s0 < n_split ? pp[(long)s0 * row + kv_rank + 1] : 0.f;
    const float l1 = s1 < n_split ? pp[(long)s1 * row + kv_rank + 1] : 0.f;
    const float M = warp_max(fmaxf(m0, m1));
    const float e0 = expf(m0 - M), e1 = expf(m1 - M);
    wgt[s0] = e0; wgt[s1] = e1;
    // fixed order: lane-local pair, then the butterfly
    const float L = warp_sum(l0 * e0 + l1 * e1);
    if (threadIdx.x == 0) inv_s = 1.0f / L;
  }
  __syncthreads();
  const float inv = inv_s;
  for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
    float a = 0.f;
#pragma unroll 16
    for (int s = 0; s < n_split; ++s) a = fmaf(pp[(long)s * row + d], wgt[s], a);
    out[(long)t * ldo + (long)h * kv_rank + d] = a * inv;
  }
}

// ---------------------------------------------------------------------------------------------------------
// router: z[t][E] fp32 -> the `top` largest (lowest index wins a tie), weights = softmax over the chosen logits
__global__ void router_topk_kernel(const float* __restrict__ z, long ldz, int E, int top, int* __restrict__ idx,
                                   float* __restrict__ wgt, int T) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* zr = z + (long)t * ldz;
  unsigned long long taken_lo = 0;        // lanes own experts lane, lane+32, ...: up to 64 per lane (E <= 2048)
  float vmax = 0.f, denom = 0.f;
  for (int s = 0; s < top; ++s) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane, n = 0; e < E; e += 32, ++n) {
      if ((taken_lo >> n) & 1ull) continue;
      const float v = zr[e];
      if (v > best || (v == best && e < bi)) { best = v; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if ((bi & 31) == lane && bi < E) taken_lo |= 1ull << (bi >> 5);
    if (s == 0) vmax = best;
    const float e = expf(best - vmax);
    denom += e;
    if (lane == 0) { idx[(long)t * top + s] = bi; wgt[(long)t * top + s] = e; }
  }
  __syncwarp();
  if (lane == 0)
    for (int s = 0; s < top; ++s) wgt[(long)t * top + s] /= denom;
}

// router with sigmoid scores and a choice limited to groups of experts: s = sigmoid(z); the choice is made on
// c = s + correction; the E experts form n_groups equal groups of neighbours, a group's score is the sum of its two
// largest c (its only c when a group is one expert), and only experts of the `keep` best groups can be chosen (the
// others count as minus infinity); the `top` largest c are chosen (lowest index wins a tie) and weighted by their s,
// divided by the sum of the chosen s (+ 1e-20).  A warp per token; the choice scores of a token sit in shared memory.
// softmax: s = softmax(z) over all experts instead of the sigmoid; group_max: a group's score is its largest c.
__global__ void router_group_topk_kernel(const float* __restrict__ z, long ldz, const bf16* __restrict__ corr, int E,
                                         int top, int n_groups, int keep, int softmax, int group_max,
                                         int* __restrict__ idx, float* __restrict__ wgt, int T) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int t = blockIdx.x * nw + warp;
  if (t >= T) return;
  float* c = sm + (long)warp * (E + n_groups);      // [E] choice scores, then [n_groups] group scores
  float* gs = c + E;
  const float* zr = z + (long)t * ldz;
  float zmax = 0.f, zinv = 1.f;
  if (softmax) {
    float a = -INFINITY;
    for (int e = lane; e < E; e += 32) a = fmaxf(a, zr[e]);
    zmax = warp_max(a);
    float b = 0.f;
    for (int e = lane; e < E; e += 32) b += expf(zr[e] - zmax);
    zinv = 1.0f / warp_sum(b);
  }
  for (int e = lane; e < E; e += 32)
    c[e] = (softmax ? expf(zr[e] - zmax) * zinv : 1.0f / (1.0f + expf(-zr[e]))) + (corr ? bf2f(corr[e]) : 0.f);
  __syncwarp();
  if (n_groups > 1 && keep < n_groups) {
    const int per = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;             // the two largest of the group
      for (int i = 0; i < per; ++i) {
        const float v = c[g * per + i];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gs[g] = (per > 1 && !group_max) ? a + b : a;
    }
    __syncwarp();
    for (int s = 0; s < keep; ++s) {                  // the best group leaves the contest with a mark: NaN-free +inf
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && (v > best || (v == best && g < bi) || bi == 0x7fffffff)) { best = v; bi = g; }
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
      }
      __syncwarp();
      if (lane == 0 && bi != 0x7fffffff) gs[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / per] != INFINITY) c[e] = -INFINITY;
    __syncwarp();
  }
  float denom = 0.f;
  for (int s = 0; s < top; ++s) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = c[e];
      if (v > best || (v == best && e < bi && v != -INFINITY)) { best = v; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (bi >= E) bi = 0;                              // fewer choosable experts than `top`: the host refuses that
    __syncwarp();
    const float sc = softmax ? expf(zr[bi] - zmax) * zinv : 1.0f / (1.0f + expf(-zr[bi]));
    denom += sc;
    if (lane == 0) { c[bi] = -INFINITY; idx[(long)t * top + s] = bi; wgt[(long)t * top + s] = sc; }
    __syncwarp();
  }
  if (lane == 0) {
    const float inv = 1.0f / (denom + 1e-20f);
    for (int s = 0; s < top; ++s) wgt[(long)t * top + s] *= inv;
  }
}

// the residual update of a branch with a scale vector:  x[t] += ls * ( sum_s wgt[t][s] y[t top + s]  (top = 0: y[t])
//                                                                    + sigmoid(sgate[t]) shared[t] )   (if shared)
__global__ void residual_rows_kernel(const float* __restrict__ y, long ldy, const float* __restrict__ wgt, int top,
                                     const float* __restrict__ shared, long lds, const float* __restrict__ sgate,
                                     long ldsg, const bf16* __restrict__ ls, float mult, float* __restrict__ x, long ldx,
                                     int N) {
  const long t = blockIdx.x;
  const float sg = shared ? (sgate ? 1.0f / (1.0f + expf(-sgate[t * ldsg])) : 1.f) : 0.f;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < N; i += blockDim.x * gridDim.y) {
    float v;
    if (top > 0) {
      v = 0.f;
      for (int s = 0; s < top; ++s) v += wgt[t * top + s] * y[(t * top + s) * ldy + i];
    } else {
      v = y[t * ldy + i];
    }
    if (shared) v = fmaf(sg, shared[t * lds + i], v);
    float* o = x + t * ldx + i;
    *o = fmaf((ls ? bf2f(ls[i]) : 1.f) * mult, v, *o);
  }
}

// group the (token, choice) entries by expert: list[e][0..count[e]) = entry numbers in ascending order
__global__ void moe_group_kernel(const int* __restrict__ idx, int n_entries, int* __restrict__ list, long list_stride,
                                 int* __restrict__ count) {
  __shared__ int warp_tot[32];
  __shared__ int base;
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  for (int i0 = 0; i0 < n_entries; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    const bool hit = i < n_entries && idx[i] == e;
    const unsigned b = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) warp_tot[warp] = __popc(b);
    __syncthreads();
    int off = base;
    for (int w = 0; w < warp; ++w) off += warp_tot[w];
    if (hit) list[(long)e * list_stride + off + __popc(b & ((1u << lane) - 1))] = i;
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < nw; ++w) tot += warp_tot[w];
      base += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) count[e] = base;
}

// ---------------------------------------------------------------------------------------------------------
// general row GEMM  Y[b][r][n] = epi( sum_k X[b][xr][k] * W[b][n][k] + bias[n] )
struct GemmRowsP {
  const float* X; long ldx, xb;          // row pitch, batch stride (elements)
  const bf16* W; long ldw, wb;
  const bf16* bias;
  float* Y; long ldy, yb;
  const int* list; long list_stride;     // per batch: entry numbers; x row = entry / x_div, y row = entry
  const int* count;                      // per batch: rows (device); NULL: M rows, no list
  int x_div;
  int M, N, K;
  int epi; float epi_param;              // 0 none, 1 relu^2, 2 param * tanh(v / param), 3 added to the output, 4 v * param, 5 gelu
  int round_x;
  int compact, n_batch;                  // compact: blockIdx.z counts the batches that HAVE rows (count[b] > 0) —
};                                       // a decode step launches top x rows slices, not one per expert
// the z-th batch with rows, or -1 (whole block; the counts are read 32 at a time, not one after the other)
__device__ __forceinline__ int nth_active(const int* __restrict__ count, int n_batch, int z) {
  __shared__ int s_found;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int found = -1, base = 0;
    for (int e0 = 0; e0 < n_batch && found < 0; e0 += 32) {
      const int e = e0 + lane;
      const unsigned m = __ballot_sync(0xffffffffu, e < n_batch && count[e] > 0);
      const int c = __popc(m);
      if (z < base + c) {
        unsigned mm = m;
        for (int i = 0; i < z - base; ++i) mm &= mm - 1;
        found = e0 + __ffs(mm) - 1;
      }
      base += c;
    }
    if (lane == 0) s_found = found;
  }
  __syncthreads();
  return s_found;
}
__device__ __forceinline__ float gemm_epi(float v, int epi, float param) {
  if (epi == 1) { v = fmaxf(v, 0.f); return v * v; }
  if (epi == 2) return param * tanhf(v / param);
  if (epi == 4) return v * param;
  if (epi == 5) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));    // the exact gelu
  return v;
}
// epi 3: the product is added to what the output row holds (a residual stream that accumulates in place)
__device__ __forceinline__ void gemm_store(float* y, float v, int epi, float param) {
  *y = epi == 3 ? *y + v : gemm_epi(v, epi, param);
}
constexpr int GB_M = 64, GB_N = 64, GB_K = 16;
__global__ void __launch_bounds__(256) gemm_rows_kernel(GemmRowsP p) {
  __shared__ float As[GB_K][GB_M + 4];
  __shared__ float Bs[GB_K][GB_N + 4];
  __shared__ int xrow[GB_M], yrow[GB_M];
  const int b = blockIdx.z;
  const int rows = p.count ? p.count[b] : p.M;
  const int m0 = blockIdx.y * GB_M, n0 = blockIdx.x * GB_N;
  if (m0 >= rows) return;
  const int tid = threadIdx.x;
  if (tid < GB_M) {
    const int r = m0 + tid;
    int xr = -1, yr = -1;
    if (r < rows) {
      if (p.list) { const int e = p.list[(long)b * p.list_stride + r]; xr = e / p.x_div; yr = e; }
      else { xr = yr = r; }
    }
    xrow[tid] = xr; yrow[tid] = yr;
  }
  __syncthreads();
  const float* X = p.X + (long)b * p.xb;
  const bf16* W = p.W + (long)b * p.wb;
  const int tx = tid & 15, ty = tid >> 4;      // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.K; k0 += GB_K) {
    // stage 64 x 16 of X and of W: thread -> (row = tid / 4, 4 consecutive k)
    {
      const int r = tid >> 2, kk = (tid & 3) * 4;
      const int xr = xrow[r];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int k = k0 + kk + j;
        float v = 0.f;
        if (xr >= 0 && k < p.K) { v = X[(long)xr * p.ldx + k]; if (p.round_x) v = rbf(v); }
        As[kk + j][r] = v;
      }
      const int n = n0 + r;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int k = k0 + kk + j;
        Bs[kk + j][r] = (n < p.N && k < p.K) ? bf2f(W[(long)n * p.ldw + k]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GB_K; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* Y = p.Y + (long)b * p.yb;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int yr = yrow[ty * 4 + i];
    if (yr < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = acc[i][j];
      if (p.bias) v += bf2f(p.bias[n]);
      gemm_store(&Y[(long)yr * p.ldy + n], v, p.epi, p.epi_param);
    }
  }
}

// the skinny sibling for decode steps (few rows): a warp per weight row, the rows of X in chunks of 8 per pass
// over the weight row; k order fixed by the lane striding + butterfly, independent of the other rows
constexpr int GS_R = 8;
__global__ void __launch_bounds__(256) gemm_skinny_kernel(GemmRowsP p) {
  const int b = p.compact ? nth_active(p.count, p.n_batch, blockIdx.z) : (int)blockIdx.z;
  if (b < 0) return;
  const int rows = p.count ? p.count[b] : p.M;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (n >= p.N || rows <= 0) return;
  const float* X = p.X + (long)b * p.xb;
  const bf16* w = p.W + (long)b * p.wb + (long)n * p.ldw;
  float* Y = p.Y + (long)b * p.yb;
  const float bias = p.bias ? bf2f(p.bias[n]) : 0.f;
  for (int r0 = 0; r0 < rows; r0 += GS_R) {
    int xr[GS_R], yr[GS_R];
#pragma unroll
    for (int i = 0; i < GS_R; ++i) {
      const int r = r0 + i;
      xr[i] = yr[i] = -1;
      if (r < rows) {
        if (p.list) { const int e = p.list[(long)b * p.list_stride + r]; xr[i] = e / p.x_div; yr[i] = e; }
        else { xr[i] = yr[i] = r; }
      }
    }
    float acc[GS_R] = {};
    for (int k = lane; k < p.K; k += 32) {
      const float wv = bf2f(w[k]);
#pragma unroll
      for (int i = 0; i < GS_R; ++i)
        if (xr[i] >= 0) {
          float v = X[(long)xr[i] * p.ldx + k];
          if (p.round_x) v = rbf(v);
          acc[i] = fmaf(v, wv, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < GS_R; ++i) {
      const float v = warp_sum(acc[i]);
      if (lane == 0 && yr[i] >= 0) gemm_store(&Y[(long)yr[i] * p.ldy + n], v + bias, p.epi, p.epi_param);
    }
  }
}

// The decode kernel proper: weight rows as 16-byte loads (8 bf16 per lane), the few rows of X staged in shared
// memory chunk by chunk (rounded to bf16 there in the serving mode), every warp takes GV_R weight rows per pass.
// Needs K % 8 == 0, 16-byte aligned weight rows and at most MR rows; the k order of a sum is fixed (lane-strided,
// then the butterfly) whatever the other rows are.
constexpr int GV_R = 2, GV_WARPS = 8;
template <int MR, int GV_KC>
__global__ void __launch_bounds__(GV_WARPS * 32) gemm_skinny_vec_kernel(GemmRowsP p) {
  __shared__ __align__(16) float xs[MR][GV_KC];
  __shared__ int xrow[MR], yrow[MR];
  const int b = p.compact ? nth_active(p.count, p.n_batch, blockIdx.z) : (int)blockIdx.z;
  if (b < 0) return;
  const int rows = min(p.count ? p.count[b] : p.M, MR);
  if (rows <= 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < MR) {
    int xr = -1, yr = -1;
    if ((int)threadIdx.x < rows) {
      if (p.list) { const int e = p.list[(long)b * p.list_stride + threadIdx.x]; xr = e / p.x_div; yr = e; }
      else { xr = yr = threadIdx.x; }
    }
    xrow[threadIdx.x] = xr; yrow[threadIdx.x] = yr;
  }
  const float* X = p.X + (long)b * p.xb;
  const bf16* W = p.W + (long)b * p.wb;
  const int n0 = (blockIdx.x * GV_WARPS + warp) * GV_R;
  float acc[GV_R][MR];
#pragma unroll
  for (int r = 0; r < GV_R; ++r)
#pragma unroll
    for (int i = 0; i < MR; ++i) acc[r][i] = 0.f;
  for (int k0 = 0; k0 < p.K; k0 += GV_KC) {
    const int kc = min(GV_KC, p.K - k0);
    __syncthreads();
    for (int e = threadIdx.x; e < MR * (kc >> 2); e += blockDim.x) {
      const int i = e / (kc >> 2), k = (e % (kc >> 2)) << 2;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (xrow[i] >= 0) {
        v = *reinterpret_cast<const float4*>(X + (long)xrow[i] * p.ldx + k0 + k);
        if (p.round_x) { v.x = rbf(v.x); v.y = rbf(v.y); v.z = rbf(v.z); v.w = rbf(v.w); }
      }
      *reinterpret_cast<float4*>(&xs[i][k]) = v;
    }
    __syncthreads();
#pragma unroll 4
    for (int k = lane * 8; k < kc; k += 256) {
      float w[GV_R][8];
#pragma unroll
      for (int r = 0; r < GV_R; ++r) {
        if (n0 + r < p.N) {
          unpack8(ldg_stream(W + (long)(n0 + r) * p.ldw + k0 + k), w[r]);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) w[r][j] = 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < MR; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(&xs[i][k]);
        const float4 c = *reinterpret_cast<const float4*>(&xs[i][k + 4]);
#pragma unroll
        for (int r = 0; r < GV_R; ++r) {
          float t = acc[r][i];
          t = fmaf(a.x, w[r][0], t); t = fmaf(a.y, w[r][1], t); t = fmaf(a.z, w[r][2], t); t = fmaf(a.w, w[r][3], t);
          t = fmaf(c.x, w[r][4], t); t = fmaf(c.y, w[r][5], t); t = fmaf(c.z, w[r][6], t); t = fmaf(c.w, w[r][7], t);
          acc[r][i] = t;
        }
      }
    }
  }
  float* Y = p.Y + (long)b * p.yb;
#pragma unroll
  for (int r = 0; r < GV_R; ++r) {
    const int n = n0 + r;
    const float bias = (p.bias && n < p.N) ? bf2f(p.bias[n]) : 0.f;
#pragma unroll
    for (int i = 0; i < MR; ++i) {
      const float v = warp_sum(acc[r][i]);
      if (lane == 0 && n < p.N && yrow[i] >= 0) gemm_store(&Y[(long)yrow[i] * p.ldy + n], v + bias, p.epi, p.epi_param);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Operands of the tensor-core products of a prompt step (bf16 serving mode; the products themselves are the
// weight-major tcgen05 GEMM with fp32 output, b200_gemm_wt_f32):
// rows of fp32 numbers -> bf16 rows padded with zeros to Kp columns; optional gather (src row = map[i] / div),
// optional activation before the rounding (1: relu^2, 2: the exact gelu, 3: tanh); with `dst_map` the kernel instead scatters fp32 rows (dst row = dst_map[i])
__global__ void rows_to_bf16_kernel(const float* __restrict__ X, long ldx, const int* __restrict__ map, int div,
                                    bf16* __restrict__ out, long ldo, int K, int Kp, int relu2) {
  const int i = blockIdx.x;
  const int src = map ? map[i] : i;            // a negative entry of the map: a padding row, written as zeros
  const float* x = X + (long)(src < 0 ? 0 : (map ? src / div : src)) * ldx;
  for (int k = threadIdx.x; k < Kp; k += blockDim.x) {
    float v = (k < K && src >= 0) ? x[k] : 0.f;
    if (relu2 == 1) { v = fmaxf(v, 0.f); v *= v; }
    else if (relu2 == 2) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    else if (relu2 == 3) v = tanhf(v);
    out[(long)i * ldo + k] = f2bf(v);
  }
}
// the same with four columns per thread (rows of whole, aligned 16-byte vectors; K, Kp multiples of 4)
__global__ void rows_to_bf16x4_kernel(const float* __restrict__ X, long ldx, const int* __restrict__ map, int div,
                                      bf16* __restrict__ out, long ldo, int K, int Kp, int relu2) {
  const int i = blockIdx.x;
  const int src = map ? map[i] : i;
  const float* x = X + (long)(src < 0 ? 0 : (map ? src / div : src)) * ldx;
  for (int k = threadIdx.x * 4; k < Kp; k += blockDim.x * 4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k < K && src >= 0) v = *reinterpret_cast<const float4*>(x + k);
    if (relu2 == 2) {
      v.x = 0.5f * v.x * (1.0f + erff(v.x * 0.70710678118654752f)); v.y = 0.5f * v.y * (1.0f + erff(v.y * 0.70710678118654752f));
      v.z = 0.5f * v.z * (1.0f + erff(v.z * 0.70710678118654752f)); v.w = 0.5f * v.w * (1.0f + erff(v.w * 0.70710678118654752f));
    } else if (relu2 == 3) {
      v.x = tanhf(v.x); v.y = tanhf(v.y); v.z = tanhf(v.z); v.w = tanhf(v.w);
    } else if (relu2 == 1) {
      v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
      v.x *= v.x; v.y *= v.y; v.z *= v.z; v.w *= v.w;
    }
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 pk;
    pk.x = *reinterpret_cast<const unsigned*>(&lo);
    pk.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(out + (long)i * ldo + k) = pk;
  }
}
__global__ void rows_scatter4_kernel(const float* __restrict__ X, long ldx, const int* __restrict__ dst_map,
                                     float* __restrict__ out, long ldo, int K) {
  const int i = blockIdx.x;
  if (dst_map[i] < 0) return;                  // a padding row
  const float4* x = reinterpret_cast<const float4*>(X + (long)i * ldx);
  float4* o = reinterpret_cast<float4*>(out + (long)dst_map[i] * ldo);
  for (int k = threadIdx.x; k < K / 4; k += blockDim.x) o[k] = x[k];
}
__global__ void rows_scatter_kernel(const float* __restrict__ X, long ldx, const int* __restrict__ dst_map,
                                    float* __restrict__ out, long ldo, int K) {
  const int i = blockIdx.x;
  if (dst_map[i] < 0) return;                  // a padding row
  const float* x = X + (long)i * ldx;
  float* o = out + (long)dst_map[i] * ldo;
  for (int k = threadIdx.x; k < K; k += blockDim.x) o[k] = x[k];
}
// entries sorted by expert: order[prefix[e] + i] = list[e][i], prefix = running sum of the counts
__global__ void moe_order_kernel(const int* __restrict__ list, long list_stride, const int* __restrict__ count,
                                 int* __restrict__ order) {
  const int e = blockIdx.x;
  int base = 0;
  for (int i = 0; i < e; ++i) base += count[i];
  const int n = count[e];
  for (int i = threadIdx.x; i < n; i += blockDim.x) order[base + i] = list[(long)e * list_stride + i];
}
// entries sorted by expert in segments padded to whole token tiles of `tile` rows: order[seg(e) + i] = list[e][i],
// -1 in the padding and past the last segment; tile_group[y] = the expert of tile y, -1 past the last segment
__global__ void moe_tiles_kernel(const int* __restrict__ list, long list_stride, const int* __restrict__ count, int E,
                                 int tile, int* __restrict__ order, int n_rows, int* __restrict__ tile_group) {
  const int e = blockIdx.x;
  int base = 0, total = 0;
  for (int i = 0; i < E; ++i) {
    const int padded = (count[i] + tile - 1) / tile * tile;
    if (i < e) base += padded;
    total += padded;
  }
  if (e < E) {
    const int n = count[e], padded = (n + tile - 1) / tile * tile;
    for (int i = threadIdx.x; i < padded; i += blockDim.x) order[base + i] = i < n ? list[(long)e * list_stride + i] : -1;
    for (int y = threadIdx.x; y < padded / tile; y += blockDim.x) tile_group[base / tile + y] = e;
  } else {                                    // the extra block: everything past the last segment
    for (int i = total + threadIdx.x; i < n_rows; i += blockDim.x) order[i] = -1;
    for (int y = total / tile + threadIdx.x; y < n_rows / tile; y += blockDim.x) tile_group[y] = -1;
  }
}
// causal softmax of score rows: row r belongs to query r / H at position pos[r / H], which sees keys 0..pos;
// P (bf16, normalised in fp32 before the rounding) is zero past the last visible key and in the padding
__global__ void masked_softmax_bf16_kernel(const float* __restrict__ S, long lds, const int* __restrict__ pos, int H,
                                           float scale, bf16* __restrict__ P, long ldp, int Sp) {
  __shared__ float red[32];
  const long r = blockIdx.x;
  const int n = pos[r / H] + 1;
  const float* s = S + r * lds;
  float m = -INFINITY;
  for (int j = threadIdx.x; j < n; j += blockDim.x) m = fmaxf(m, s[j]);
  m = warp_max(m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
  float sum = 0.f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) sum += expf((s[j] - m) * scale);
  const float inv = 1.0f / block_sum(sum, red);
  for (int j = threadIdx.x; j < Sp; j += blockDim.x)
    P[r * ldp + j] = f2bf(j < n ? expf((s[j] - m) * scale) * inv : 0.f);
}
// the latent columns of one slot's cache rows, transposed: out[d][j] = cache[j][d] (bf16), j < S, zero up to Sp
__global__ void cache_transpose_kernel(const bf16* __restrict__ C, long tok_stride, int S, int Sp, int kv_rank,
                                       bf16* __restrict__ out) {
  __shared__ bf16 tile[32][33];
  const int j0 = blockIdx.x * 32, d0 = blockIdx.y * 32, tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int y = ty; y < 32; y += 8) {
    const int j = j0 + y, d = d0 + tx;
    tile[y][tx] = (j < S && d < kv_rank) ? C[(long)j * tok_stride + d] : f2bf(0.f);
  }
  __syncthreads();
  for (int y = ty; y < 32; y += 8) {
    const int d = d0 + y, j = j0 + tx;
    if (d < kv_rank && j < Sp) out[(long)d * Sp + j] = tile[tx][y];
  }
}

// For one to four rows (a single request decoding): the whole block works on GK_RB weight rows at once, every
// thread owns 8 columns of a 2048-column chunk, so all loads of a block are in flight together and a product of a
// few MB is spread over hundreds of blocks.  Sums: thread-local in k order, butterfly, then the warps in order.
constexpr int GK_RB = 4, GK_KC = 2048;
template <int MR>
__global__ void __launch_bounds__(256) gemm_skinny_blk_kernel(GemmRowsP p) {
  __shared__ __align__(16) float xs[MR][GK_KC];
  __shared__ float red[8][GK_RB][MR];
  __shared__ int xrow[MR], yrow[MR];
  const int b = p.compact ? nth_active(p.count, p.n_batch, blockIdx.z) : (int)blockIdx.z;
  if (b < 0) return;
  const int rows = min(p.count ? p.count[b] : p.M, MR);
  if (rows <= 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < MR) {
    int xr = -1, yr = -1;
    if ((int)threadIdx.x < rows) {
      if (p.list) { const int e = p.list[(long)b * p.list_stride + threadIdx.x]; xr = e / p.x_div; yr = e; }
      else { xr = yr = threadIdx.x; }
    }
    xrow[threadIdx.x] = xr; yrow[threadIdx.x] = yr;
  }
  const float* X = p.X + (long)b * p.xb;
  const bf16* W = p.W + (long)b * p.wb;
  const int n0 = blockIdx.x * GK_RB;
  float acc[GK_RB][MR];
#pragma unroll
  for (int r = 0; r < GK_RB; ++r)
#pragma unroll
    for (int i = 0; i < MR; ++i) acc[r][i] = 0.f;
  for (int k0 = 0; k0 < p.K; k0 += GK_KC) {
    const int kc = min(GK_KC, p.K - k0);
    const int k = threadIdx.x * 8;
    uint4 wv[GK_RB];
#pragma unroll
    for (int r = 0; r < GK_RB; ++r)          // the weight loads go out first: they are the long-latency ones
      wv[r] = (k < kc && n0 + r < p.N) ? ldg_stream(W + (long)(n0 + r) * p.ldw + k0 + k) : make_uint4(0, 0, 0, 0);
    __syncthreads();
    for (int e = threadIdx.x; e < MR * (kc >> 2); e += blockDim.x) {
      const int i = e / (kc >> 2), kk = (e % (kc >> 2)) << 2;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (xrow[i] >= 0) {
        v = *reinterpret_cast<const float4*>(X + (long)xrow[i] * p.ldx + k0 + kk);
        if (p.round_x) { v.x = rbf(v.x); v.y = rbf(v.y); v.z = rbf(v.z); v.w = rbf(v.w); }
      }
      *reinterpret_cast<float4*>(&xs[i][kk]) = v;
    }
    __syncthreads();
    if (k < kc) {
#pragma unroll
      for (int r = 0; r < GK_RB; ++r) {
        float w[8];
        unpack8(wv[r], w);
#pragma unroll
        for (int i = 0; i < MR; ++i) {
          const float4 a = *reinterpret_cast<const float4*>(&xs[i][k]);
          const float4 c = *reinterpret_cast<const float4*>(&xs[i][k + 4]);
          float t = acc[r][i];
          t = fmaf(a.x, w[0], t); t = fmaf(a.y, w[1], t); t = fmaf(a.z, w[2], t); t = fmaf(a.w, w[3], t);
          t = fmaf(c.x, w[4], t); t = fmaf(c.y, w[5], t); t = fmaf(c.z, w[6], t); t = fmaf(c.w, w[7], t);
          acc[r][i] = t;
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < GK_RB; ++r)
#pragma unroll
    for (int i = 0; i < MR; ++i) {
      const float v = warp_sum(acc[r][i]);
      if (lane == 0) red[warp][r][i] = v;
    }
  __syncthreads();
  if (threadIdx.x < GK_RB * MR) {
    const int r = threadIdx.x / MR, i = threadIdx.x % MR, n = n0 + r;
    float v = 0.f;
    for (int w = 0; w < 8; ++w) v += red[w][r][i];
    if (n < p.N && yrow[i] >= 0) {
      if (p.bias) v += bf2f(p.bias[n]);
      gemm_store(&(p.Y + (long)b * p.yb)[(long)yrow[i] * p.ldy + n], v, p.epi, p.epi_param);
    }
  }
}

// greedy pick per row: lowest index of the largest logit, and its log-probability
__global__ void argmax_rows_kernel(const float* __restrict__ z, long ldz, int V, int* __restrict__ tok,
                                   float* __restrict__ logprob) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float red[32];
  const float* r = z + (long)blockIdx.x * ldz;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = r[i];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  best = sv[0]; bi = si[0];
  for (int i = 1; i < nw; ++i)
    if (sv[i] > best || (sv[i] == best && si[i] < bi)) { best = sv[i]; bi = si[i]; }
  float se = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) se += expf(r[i] - best);
  const float tot = block_sum(se, red);
  if (threadIdx.x == 0) {
    tok[blockIdx.x] = bi;
    if (logprob) logprob[blockIdx.x] = -logf(tot);
  }
}

// decode bookkeeping on the device (one block): the sampled tokens become the next step's inputs, positions
// advance, the tokens go to row (*step mod log_rows) of the log and *step counts up — nothing of a step is a
// launch argument, so a captured step replays unchanged
__global__ void advance_rows_kernel(const int* __restrict__ sampled, int* __restrict__ tok, int* __restrict__ pos,
                                    const int* __restrict__ active, int* __restrict__ log, int log_stride,
                                    int log_rows, int* __restrict__ step, const float* __restrict__ lp,
                                    float* __restrict__ lp_log, int B) {
  const int st = *step;
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    if (log) log[(long)(st % log_rows) * log_stride + b] = sampled[b];
    if (lp_log) lp_log[(long)(st % log_rows) * log_stride + b] = lp[b];
    if (active == nullptr || active[b]) { tok[b] = sampled[b]; pos[b] += 1; }
  }
  if (threadIdx.x == 0) *step = st + 1;
}

unsigned long long g_attn_attr_f32 = 0, g_attn_attr_bf16 = 0;

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_lm_embed(const int* tokens, const void* embed, float scale, float* x, int T, int W, int vocab, void* st) {
  B200_REQUIRE(tokens && embed && x && T > 0 && W > 0, "lm_embed: bad argument");
  embed_scale_kernel<<<T, 256, 0, (cudaStream_t)st>>>(tokens, (const bf16*)embed, scale, x, W, vocab);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_rope_table(const int* pos, const double* inv_freq, float* cs, int T, int half, float amp, void* st) {
  B200_REQUIRE(pos && inv_freq && cs && T > 0 && half > 0, "lm_rope_table: bad argument");
  rope_table_kernel<<<cdiv((long)T * half, 256), 256, 0, (cudaStream_t)st>>>(pos, inv_freq, (float2*)cs, T, half, amp);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_norm_rows(const float* y, long ldy, const float* wgt, int top, const void* w, float w_offset, float eps,
                      float* x, long ldx, int add, const int* rows, int center, int groups, int T, int N, void* st) {
  B200_REQUIRE(y && w && x && T > 0 && N > 0, "lm_norm_rows: bad argument");
  if (groups < 1) groups = 1;
  B200_REQUIRE(N % groups == 0 && groups <= 1024 && !(center && groups > 1), "lm_norm_rows: %d parts of a row of %d numbers", groups, N);
  B200_REQUIRE((N + 32 + groups) * 4 <= 48 * 1024, "lm_norm_rows: rows of %d numbers do not fit shared memory", N);
  NormP p{y, ldy, wgt, wgt ? top : 0, (const bf16*)w, w_offset, eps, x, ldx, add, rows, N, center, nullptr, 0, nullptr, nullptr, 0, nullptr, 0,
          groups, 1.f};
  norm_rows_kernel<<<T, T < 64 ? 1024 : 256, (N + 32 + groups) * sizeof(float), (cudaStream_t)st>>>(p);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_residual_norm_rows(const float* y, long ldy, const float* wgt, int top, const float* shared, long lds,
                               const float* sgate, long ldsg, const void* ls, float* res, long ldr, const void* w,
                               float w_offset, float eps, int center, float* out, long ldo, int groups, float mult,
                               int T, int N, void* st) {
  B200_REQUIRE(y && res && w && out && T > 0 && N > 0 && (top == 0 || wgt), "lm_residual_norm_rows: bad argument");
  if (groups < 1) groups = 1;
  B200_REQUIRE(N % groups == 0 && groups <= 1024 && !(center && groups > 1), "lm_residual_norm_rows: %d parts of a row of %d numbers", groups, N);
  B200_REQUIRE((N + 32 + groups) * 4 <= 48 * 1024, "lm_residual_norm_rows: rows of %d numbers do not fit shared memory", N);
  NormP p{y, ldy, wgt, wgt ? top : 0, (const bf16*)w, w_offset, eps, out, ldo, 0, nullptr, N, center,
          res, ldr, (const bf16*)ls, shared, lds, sgate, ldsg, groups, mult};
  norm_rows_kernel<<<T, T < 64 ? 1024 : 256, (N + 32 + groups) * sizeof(float), (cudaStream_t)st>>>(p);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_latent_post(const float* D, long ldd, const void* wq, const void* wkv, float eps, float* cq, long ldq,
                        void* cache, int cache_bf16, long slot_stride, long tok_stride, const int* slot,
                        const int* pos, const float* cs, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                        int own_kv, int pairs, int T, void* st) {
  B200_REQUIRE(D && T > 0 && q_rank >= 0 && (q_rank == 0 || (wq && cq)), "lm_latent_post: bad argument");
  B200_REQUIRE(!own_kv || (wkv && cache && slot && pos && cs), "lm_latent_post: a layer with its own latent needs a cache");
  B200_REQUIRE(rot_dims % 2 == 0 && rot_dims <= rot_dim, "lm_latent_post: rotated dims %d of %d", rot_dims, rot_dim);
  if (cache_bf16) {
    LatentPostP<bf16> p{D, ldd, (const bf16*)wq, (const bf16*)wkv, eps, cq, ldq, (bf16*)cache, slot_stride, tok_stride,
                        slot, pos, (const float2*)cs, q_rank, kv_rank, rot_dim, rot_dims, own_kv, pairs};
    latent_post_kernel<bf16><<<T, T < 64 ? 512 : 128, 0, (cudaStream_t)st>>>(p);
  } else {
    LatentPostP<float> p{D, ldd, (const bf16*)wq, (const bf16*)wkv, eps, cq, ldq, (float*)cache, slot_stride,
                         tok_stride, slot, pos, (const float2*)cs, q_rank, kv_rank, rot_dim, rot_dims, own_kv, pairs};
    latent_post_kernel<float><<<T, T < 64 ? 512 : 128, 0, (cudaStream_t)st>>>(p);
  }
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_rope_q(const float* q, long ldq, int qh_stride, int dim, float* qa, long ldqa, int Dl, int kv_rank,
                   const float* cs, int H, int rot_dim, int rot_dims, int pairs, int T, void* st) {
  B200_REQUIRE(q && qa && cs && T > 0, "lm_rope_q: bad argument");
  rope_q_kernel<<<T, 128, 0, (cudaStream_t)st>>>(q, ldq, qh_stride, dim, qa, ldqa, Dl, kv_rank, (const float2*)cs, H,
                                                 rot_dim, rot_dims, pairs);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_latent_attention(const float* qa, long ldqa, const void* cache, int cache_bf16, long slot_stride,
                             long tok_stride, const int* slot, const int* pos, float* out, long ldo, int H, int Dl,
                             int kv_rank, float scale, int round_q, int window, float* part, int n_split, int T,
                             void* st) {
  B200_REQUIRE(qa && cache && slot && pos && out && T > 0 && H > 0, "lm_latent_attention: bad argument");
  if (n_split < 1 || !part) n_split = 1;
  B200_REQUIRE(n_split <= 64, "lm_latent_attention: at most 64 splits");
  const int vec8 = cache_bf16 && Dl % 8 == 0 && tok_stride % 8 == 0 && slot_stride % 8 == 0 && ((uintptr_t)cache & 15) == 0;
  B200_REQUIRE(kv_rank <= 1024 && kv_rank <= Dl, "lm_latent_attention: latent rank %d not supported", kv_rank);
  const int nw = H < 8 ? H : 8;
  const size_t smem = ((size_t)LA_KT * (Dl + ((Dl & 3) == 0 ? 4 : 1)) + (size_t)nw * Dl) * sizeof(float);
  B200_REQUIRE(smem <= 200 * 1024, "lm_latent_attention: rows of %d numbers do not fit shared memory", Dl);
  dim3 grid(T, cdiv(H, nw), n_split);
  if (cache_bf16) {
    if (first_use_on_device(&g_attn_attr_bf16))
      B200_CUDA(cudaFuncSetAttribute(latent_attention_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    LatAttnP<bf16> p{qa, ldqa, (const bf16*)cache, slot_stride, tok_stride, slot, pos, out, ldo, H, Dl, kv_rank, scale, round_q, part, n_split, vec8, window};
    latent_attention_kernel<bf16><<<grid, nw * 32, smem, (cudaStream_t)st>>>(p);
  } else {
    if (first_use_on_device(&g_attn_attr_f32))
      B200_CUDA(cudaFuncSetAttribute(latent_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    LatAttnP<float> p{qa, ldqa, (const float*)cache, slot_stride, tok_stride, slot, pos, out, ldo, H, Dl, kv_rank, scale, round_q, part, n_split, 0, window};
    latent_attention_kernel<float><<<grid, nw * 32, smem, (cudaStream_t)st>>>(p);
  }
  B200_CHECK_LAUNCH();
  if (n_split > 1) {
    const int mt = kv_rank >= 512 ? 512 : (kv_rank + 31) / 32 * 32;
    latent_attention_merge_kernel<<<dim3(T, H), mt, 0, (cudaStream_t)st>>>(part, n_split, kv_rank, out, ldo, H);
    B200_CHECK_LAUNCH();
  }
  return B200_OK;
}

int b200_lm_router_topk(const float* z, long ldz, int E, int top, int* idx, float* wgt, int T, void* st) {
  B200_REQUIRE(z && idx && wgt && T > 0 && top > 0 && top <= E && E <= 2048, "lm_router_topk: bad argument");
  router_topk_kernel<<<cdiv(T, 4), 128, 0, (cudaStream_t)st>>>(z, ldz, E, top, idx, wgt, T);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_router_group_topk(const float* z, long ldz, const void* correction, int E, int top, int n_groups, int keep,
                              int softmax, int group_max, int* idx, float* wgt, int T, void* st) {
  B200_REQUIRE(z && idx && wgt && T > 0 && top > 0 && top <= E && E <= 2048, "lm_router_group_topk: bad argument");
  B200_REQUIRE(n_groups >= 1 && E % n_groups == 0 && keep >= 1 && keep <= n_groups,
               "lm_router_group_topk: %d experts in %d groups, %d kept", E, n_groups, keep);
  B200_REQUIRE(top <= (long)keep * (E / n_groups), "lm_router_group_topk: %d experts chosen among %d", top, keep * (E / n_groups));
  const int nw = 4;
  router_group_topk_kernel<<<cdiv(T, nw), nw * 32, (size_t)nw * (E + n_groups) * sizeof(float), (cudaStream_t)st>>>(
      z, ldz, (const bf16*)correction, E, top, n_groups, keep, softmax, group_max, idx, wgt, T);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_residual_rows(const float* y, long ldy, const float* wgt, int top, const float* shared, long lds,
                          const float* sgate, long ldsg, const void* ls, float mult, float* x, long ldx, int T, int N,
                          void* st) {
  B200_REQUIRE(y && x && T > 0 && N > 0 && (top == 0 || wgt), "lm_residual_rows: bad argument");
  const int by = T >= 64 ? 1 : (cdiv(N, 256) < 16 ? cdiv(N, 256) : 16);
  residual_rows_kernel<<<dim3(T, by), 256, 0, (cudaStream_t)st>>>(y, ldy, wgt, wgt ? top : 0, shared, lds, sgate, ldsg,
                                                                  (const bf16*)ls, mult, x, ldx, N);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_moe_group(const int* idx, int n_entries, int E, int* list, long list_stride, int* count, void* st) {
  B200_REQUIRE(idx && list && count && n_entries > 0 && E > 0, "lm_moe_group: bad argument");
  moe_group_kernel<<<E, 256, 0, (cudaStream_t)st>>>(idx, n_entries, list, list_stride, count);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_gemm_rows(const float* X, long ldx, long xb, const void* W, long ldw, long wb, const void* bias, float* Y,
                      long ldy, long yb, const int* list, long list_stride, const int* count, int x_div, int M, int N,
                      int K, int batch, int epi, float epi_param, int round_x, int skinny, int compact, void* st) {
  B200_REQUIRE(X && W && Y && M > 0 && N > 0 && K > 0 && batch > 0, "lm_gemm_rows: bad argument");
  B200_REQUIRE((list == nullptr) == (count == nullptr), "lm_gemm_rows: a row list needs its counts");
  GemmRowsP p{X, ldx, xb, (const bf16*)W, ldw, wb, (const bf16*)bias, Y, ldy, yb, list, list_stride, count,
              x_div > 0 ? x_div : 1, M, N, K, epi, epi_param, round_x, 0, batch};
  if (skinny && count && compact > 0 && compact < batch) {   // at most `compact` batches can have rows
    p.compact = 1;
    batch = compact;
  }
  const bool vec = K % 8 == 0 && ldw % 8 == 0 && wb % 8 == 0 && ldx % 4 == 0 && xb % 4 == 0 &&
                   ((uintptr_t)W & 15) == 0 && ((uintptr_t)X & 15) == 0;
  if (skinny && vec && M <= 16) {
    dim3 grid(cdiv(N, GV_WARPS * GV_R), 1, batch);
    const cudaStream_t cs = (cudaStream_t)st;
    dim3 gridk(cdiv(N, GK_RB), 1, batch);
    // measured: the block-wide kernel wins while a weight row is one chunk; it also takes the products with long
    // rows but so few of them that a warp per two rows would leave most of the GPU without a block
    const bool one_chunk = K <= GK_KC || (long)grid.x * batch < 148;
    if (M <= 1 && one_chunk) gemm_skinny_blk_kernel<1><<<gridk, 256, 0, cs>>>(p);
    else if (M <= 2 && one_chunk) gemm_skinny_blk_kernel<2><<<gridk, 256, 0, cs>>>(p);
    else if (M <= 4 && one_chunk) gemm_skinny_blk_kernel<4><<<gridk, 256, 0, cs>>>(p);
    else if (M <= 1) gemm_skinny_vec_kernel<1, 2048><<<grid, GV_WARPS * 32, 0, cs>>>(p);
    else if (M <= 2) gemm_skinny_vec_kernel<2, 2048><<<grid, GV_WARPS * 32, 0, cs>>>(p);
    else if (M <= 4) gemm_skinny_vec_kernel<4, 2048><<<grid, GV_WARPS * 32, 0, cs>>>(p);
    else if (M <= 8) gemm_skinny_vec_kernel<8, 1024><<<grid, GV_WARPS * 32, 0, cs>>>(p);
    else gemm_skinny_vec_kernel<16, 512><<<grid, GV_WARPS * 32, 0, cs>>>(p);
  } else if (skinny) {
    dim3 grid(cdiv(N, 8), 1, batch);
    gemm_skinny_kernel<<<grid, 256, 0, (cudaStream_t)st>>>(p);
  } else {
    dim3 grid(cdiv(N, GB_N), cdiv(M, GB_M), batch);
    gemm_rows_kernel<<<grid, 256, 0, (cudaStream_t)st>>>(p);
  }
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_rows_to_bf16(const float* X, long ldx, const int* map, int div, void* out, long ldo, int T, int K, int Kp,
                         int relu2, void* st) {
  B200_REQUIRE(X && out && T > 0 && K > 0 && Kp >= K, "lm_rows_to_bf16: bad argument");
  const bool v4 = K % 4 == 0 && Kp % 4 == 0 && ldx % 4 == 0 && ldo % 4 == 0 && ((uintptr_t)X & 15) == 0 && ((uintptr_t)out & 7) == 0;
  if (v4) rows_to_bf16x4_kernel<<<T, Kp >= 1024 ? 256 : 128, 0, (cudaStream_t)st>>>(X, ldx, map, div > 0 ? div : 1, (bf16*)out, ldo, K, Kp, relu2);
  else rows_to_bf16_kernel<<<T, 256, 0, (cudaStream_t)st>>>(X, ldx, map, div > 0 ? div : 1, (bf16*)out, ldo, K, Kp, relu2);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_rows_scatter(const float* X, long ldx, const int* dst_map, float* out, long ldo, int T, int K, void* st) {
  B200_REQUIRE(X && dst_map && out && T > 0 && K > 0, "lm_rows_scatter: bad argument");
  const bool v4 = K % 4 == 0 && ldx % 4 == 0 && ldo % 4 == 0 && (((uintptr_t)X | (uintptr_t)out) & 15) == 0;
  if (v4) rows_scatter4_kernel<<<T, 256, 0, (cudaStream_t)st>>>(X, ldx, dst_map, out, ldo, K);
  else rows_scatter_kernel<<<T, 256, 0, (cudaStream_t)st>>>(X, ldx, dst_map, out, ldo, K);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_moe_order(const int* list, long list_stride, const int* count, int E, int* order, void* st) {
  B200_REQUIRE(list && count && order && E > 0, "lm_moe_order: bad argument");
  moe_order_kernel<<<E, 256, 0, (cudaStream_t)st>>>(list, list_stride, count, order);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_moe_tiles(const int* list, long list_stride, const int* count, int E, int tile, int* order, int n_rows,
                      int* tile_group, void* st) {
  B200_REQUIRE(list && count && order && tile_group && E > 0 && tile > 0 && n_rows % tile == 0, "lm_moe_tiles: bad argument");
  moe_tiles_kernel<<<E + 1, 256, 0, (cudaStream_t)st>>>(list, list_stride, count, E, tile, order, n_rows, tile_group);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_masked_softmax_bf16(const float* S, long lds, const int* pos, int H, float scale, void* P, long ldp,
                                int rows, int Sp, void* st) {
  B200_REQUIRE(S && pos && P && rows > 0 && H > 0 && Sp > 0, "lm_masked_softmax_bf16: bad argument");
  masked_softmax_bf16_kernel<<<rows, 256, 0, (cudaStream_t)st>>>(S, lds, pos, H, scale, (bf16*)P, ldp, Sp);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_cache_transpose(const void* cache_rows, long tok_stride, int S, int Sp, int kv_rank, void* out, void* st) {
  B200_REQUIRE(cache_rows && out && S > 0 && Sp >= S && kv_rank > 0, "lm_cache_transpose: bad argument");
  cache_transpose_kernel<<<dim3(cdiv(Sp, 32), cdiv(kv_rank, 32)), 256, 0, (cudaStream_t)st>>>(
      (const bf16*)cache_rows, tok_stride, S, Sp, kv_rank, (bf16*)out);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_argmax_rows(const float* z, long ldz, int V, int* tok, float* logprob, int B, void* st) {
  B200_REQUIRE(z && tok && B > 0 && V > 0, "lm_argmax_rows: bad argument");
  argmax_rows_kernel<<<B, 1024, 0, (cudaStream_t)st>>>(z, ldz, V, tok, logprob);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

int b200_lm_advance_rows(const int* sampled, int* tok, int* pos, const int* active, int* log, int log_stride,
                         int log_rows, int* step, const float* lp, float* lp_log, int B, void* st) {
  B200_REQUIRE(sampled && tok && pos && step && B > 0 && log_rows > 0, "lm_advance_rows: bad argument");
  advance_rows_kernel<<<1, 128, 0, (cudaStream_t)st>>>(sampled, tok, pos, active, log, log_stride, log_rows, step, lp,
                                                       lp_log, B);
  B200_CHECK_LAUNCH();
  return B200_OK;
}

}  // extern "C"
