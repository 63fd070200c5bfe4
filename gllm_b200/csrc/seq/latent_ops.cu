// Kernels of the branch-norm layer-list decoders (models/hybrid.py, block "branchnorm"): RMS norm of strided rows,
// a plain batched GEMM (block-diagonal maps, per-head absorption products in fp32 or odd sizes), the real-gated
// linear recurrent unit (serial form and a two-pass chunked form for long prompts), latent attention's norm + pair
// rotary + latent-cache write and its plain multi-query attention over the latent cache, the grouped router
// selection (softmax over all outputs, correction on the choice, group limit, renormalised and scaled weights)
// and the clamped gated activation.
//
// Templated on the compute dtype T (bf16 or float); norms, angles, softmax, gates, decays, the recurrence and its
// state are fp32 in both. Compiled WITHOUT --use_fast_math (build.py). Results of a row never depend on which other
// rows share the launch: every reduction has a fixed order.
#include <cuda_bf16.h>

#include "common/host_utils.h"
#include "seq/seq_common.cuh"

namespace {
using namespace seqk;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ------------------------------------------------------------------------------------------------
// out[t, :] = rms(x[t, :n]) * w; one warp per row
template <typename T>
__global__ void __launch_bounds__(128) rms_rows_kernel(const T* __restrict__ x, long ldx, const T* __restrict__ w,
                                                       T* __restrict__ out, int ntok, int n, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= ntok) return;
  const T* xr = x + (size_t)t * ldx;
  float ss = 0.f;
  for (int i = lane; i < n; i += 32) { const float v = to_f(xr[i]); ss += v * v; }
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = lane; i < n; i += 32) out[(size_t)t * n + i] = from_f<T>(to_f(xr[i]) * r * to_f(w[i]));
}

// C_b[M, N] = A_b[M, K] . W_b[N, K]^T for every batch entry b (blockIdx.z), fp32 accumulation in ascending k
template <typename T, typename TO>
__global__ void __launch_bounds__(256) gemm_batched_simt_kernel(const T* __restrict__ A, long lda, long sa,
                                                                const T* __restrict__ W, long ldw, long sw,
                                                                TO* __restrict__ Cm, long ldc, long sc, int M, int N,
                                                                int K) {
  __shared__ float As[16][64 + 1], Ws[16][64 + 1];
  const int b = blockIdx.z;
  A += (size_t)b * sa;
  W += (size_t)b * sw;
  Cm += (size_t)b * sc;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int r = e >> 4, k = e & 15;
      As[k][r] = (m0 + r < M && k0 + k < K) ? to_f(A[(size_t)(m0 + r) * lda + k0 + k]) : 0.f;
      Ws[k][r] = (n0 + r < N && k0 + k < K) ? to_f(W[(size_t)(n0 + r) * ldw + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = As[k][ty * 4 + i]; wv[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) Cm[(size_t)m * ldc + n] = from_f<TO>(acc[i][j]);
    }
}

// ------------------------------------------------------------------------------------------------
// Real-gated linear recurrent unit. Per token and channel c (block b = c / bw, j = c % bw):
//   r = sigmoid(gates[b * 2bw + j] + gbias[..]),  i = sigmoid(gates[b * 2bw + bw + j] + gbias[..])
//   a = exp(c_decay[c] * r),  S <- a S + sqrt(1 - a^2) i u,  out = S * gelu_tanh(y_pre + y_bias)
// 1 - a^2 is formed as -expm1(2 log a): no cancellation for a near 1.
struct RgCoef { float a, b; };
template <typename T>
__device__ __forceinline__ RgCoef rg_coef(const T* __restrict__ u, const float* __restrict__ gates, long ldg, int gi,
                                          float gb_r, float gb_i, float cdec, int bw, int C, int t, int c) {
  const float gr = gates[(size_t)t * ldg + gi] + gb_r;
  const float gg = gates[(size_t)t * ldg + gi + bw] + gb_i;
  const float la = cdec * sigmoid_f(gr);
  RgCoef o;
  o.a = expf(la);
  o.b = sqrtf(-expm1f(2.0f * la)) * sigmoid_f(gg) * to_f(u[(size_t)t * C + c]);
  return o;
}

// serial form: one thread per (sequence, channel)
template <typename T>
__global__ void __launch_bounds__(128) rglru_serial_kernel(
    const T* __restrict__ u, const float* __restrict__ gates, const float* __restrict__ gbias,
    const float* __restrict__ c_decay, const T* __restrict__ y_pre, long ldy, const float* __restrict__ y_bias,
    float* __restrict__ state, const int* __restrict__ rec_slots, const int* __restrict__ seq_lens,
    const int* __restrict__ qsl, int C, int bw, T* __restrict__ out) {
  const int s = blockIdx.x, c = blockIdx.y * 128 + threadIdx.x;
  if (c >= C) return;
  const int q0 = qsl[s], q1 = qsl[s + 1];
  if (q1 <= q0) return;
  const bool carried = state != nullptr && (seq_lens[s] - (q1 - q0)) > 0;
  float* st = state != nullptr ? state + (size_t)rec_slots[s] * C + c : nullptr;
  float S = carried ? *st : 0.f;
  const int gi = (c / bw) * 2 * bw + c % bw;
  const float gb_r = gbias[gi], gb_i = gbias[gi + bw], cdec = c_decay[c], yb = y_bias[c];
  const long ldg = 2L * C;
  int t = q0;
  for (; t + 4 <= q1; t += 4) {
    RgCoef k[4];
    float y[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      k[e] = rg_coef(u, gates, ldg, gi, gb_r, gb_i, cdec, bw, C, t + e, c);
      y[e] = gelu_tanh_f(to_f(y_pre[(size_t)(t + e) * ldy + c]) + yb);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      S = fmaf(k[e].a, S, k[e].b);
      out[(size_t)(t + e) * C + c] = from_f<T>(S * y[e]);
    }
  }
  for (; t < q1; ++t) {
    const RgCoef k = rg_coef(u, gates, ldg, gi, gb_r, gb_i, cdec, bw, C, t, c);
    S = fmaf(k.a, S, k.b);
    out[(size_t)t * C + c] = from_f<T>(S * gelu_tanh_f(to_f(y_pre[(size_t)t * ldy + c]) + yb));
  }
  if (st != nullptr) *st = S;
}

// chunked form, pass 1: (A, B) of every chunk of `len` tokens, S_out = A S_in + B; grid (seq, chunk, C / 128)
template <typename T>
__global__ void __launch_bounds__(128) rglru_chunk_summary_kernel(
    const T* __restrict__ u, const float* __restrict__ gates, const float* __restrict__ gbias,
    const float* __restrict__ c_decay, const int* __restrict__ qsl, int C, int bw, int len, int max_chunks,
    float2* __restrict__ summary) {
  const int s = blockIdx.x, ch = blockIdx.y, c = blockIdx.z * 128 + threadIdx.x;
  if (c >= C) return;
  const int q0 = qsl[s] + ch * len, q1 = min(qsl[s + 1], q0 + len);
  if (q1 <= q0) return;
  const int gi = (c / bw) * 2 * bw + c % bw;
  const float gb_r = gbias[gi], gb_i = gbias[gi + bw], cdec = c_decay[c];
  float A = 1.f, B = 0.f;
  for (int t = q0; t < q1; ++t) {
    const RgCoef k = rg_coef(u, gates, 2L * C, gi, gb_r, gb_i, cdec, bw, C, t, c);
    A *= k.a;
    B = fmaf(k.a, B, k.b);
  }
  summary[((size_t)s * max_chunks + ch) * C + c] = make_float2(A, B);
}

// chunked form, pass 2: fold the summaries of the chunks before this one into the incoming state, then walk the
// chunk; the sequence's last chunk stores the state
template <typename T>
__global__ void __launch_bounds__(128) rglru_chunk_apply_kernel(
    const T* __restrict__ u, const float* __restrict__ gates, const float* __restrict__ gbias,
    const float* __restrict__ c_decay, const T* __restrict__ y_pre, long ldy, const float* __restrict__ y_bias,
    float* __restrict__ state, const int* __restrict__ rec_slots, const int* __restrict__ seq_lens,
    const int* __restrict__ qsl, int C, int bw, int len, int max_chunks, const float2* __restrict__ summary,
    T* __restrict__ out) {
  const int s = blockIdx.x, ch = blockIdx.y, c = blockIdx.z * 128 + threadIdx.x;
  if (c >= C) return;
  const int b0 = qsl[s], b1 = qsl[s + 1];
  const int q0 = b0 + ch * len, q1 = min(b1, q0 + len);
  if (q1 <= q0) return;
  const bool carried = state != nullptr && (seq_lens[s] - (b1 - b0)) > 0;
  float* st = state != nullptr ? state + (size_t)rec_slots[s] * C + c : nullptr;
  float S = carried ? *st : 0.f;
  for (int p = 0; p < ch; ++p) {
    const float2 ab = summary[((size_t)s * max_chunks + p) * C + c];
    S = fmaf(ab.x, S, ab.y);
  }
  const int gi = (c / bw) * 2 * bw + c % bw;
  const float gb_r = gbias[gi], gb_i = gbias[gi + bw], cdec = c_decay[c], yb = y_bias[c];
  for (int t = q0; t < q1; ++t) {
    const RgCoef k = rg_coef(u, gates, 2L * C, gi, gb_r, gb_i, cdec, bw, C, t, c);
    S = fmaf(k.a, S, k.b);
    out[(size_t)t * C + c] = from_f<T>(S * gelu_tanh_f(to_f(y_pre[(size_t)t * ldy + c]) + yb));
  }
  if (st != nullptr && q1 == b1) *st = S;
}

// ------------------------------------------------------------------------------------------------
// Latent attention, one block per token: latent = rms(dkv[:rank]) * w -> cache columns [0, rank); the shared key
// part dkv[rank:rank + rot] is rotated -> cache columns [rank, rank + rot); every head's rotated query part
// q[h, dim:dim + rot] is rotated into q_full[h, rank:rank + rot]. Pairs (2i, 2i + 1) turn by the fp32 angle
// position * freqs[i]; cos and sin are multiplied by mag.
template <typename T>
__global__ void __launch_bounds__(128) latent_norm_rope_write_kernel(
    const T* __restrict__ q, long ldq_t, long ldq_h, int H, int dim, const T* __restrict__ dkv, long ldkv, int rank,
    int rot, const T* __restrict__ norm_w, float eps, const int* __restrict__ positions,
    const float* __restrict__ freqs, float mag, T* __restrict__ q_full, T* __restrict__ cache,
    const int* __restrict__ slots, int ps, int slab) {
  extern __shared__ float cs[];          // [rot / 2][2]: cos, sin
  __shared__ float scratch[4];
  const int t = blockIdx.x;
  const int half = rot / 2;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += 128) {
    const float ang = pos * freqs[i];
    cs[2 * i] = cosf(ang) * mag;
    cs[2 * i + 1] = sinf(ang) * mag;
  }
  const T* row = dkv + (size_t)t * ldkv;
  float ss = 0.f;
  for (int d = threadIdx.x; d < rank; d += 128) { const float v = to_f(row[d]); ss += v * v; }
  ss = block_sum<128>(ss, scratch);      // also orders the cos / sin table before its readers
  const float r = 1.0f / sqrtf(ss / (float)rank + eps);
  const int slot = slots != nullptr ? slots[t] : -1;
  const int Dl = rank + rot;
  if (slot >= 0) {
    for (int d = threadIdx.x; d < rank; d += 128)
      cache[cache_index(slot, 0, d, 1, Dl, ps, slab)] = from_f<T>(to_f(row[d]) * r * to_f(norm_w[d]));
    for (int i = threadIdx.x; i < half; i += 128) {
      const float a = to_f(row[rank + 2 * i]), b = to_f(row[rank + 2 * i + 1]);
      const float c = cs[2 * i], s = cs[2 * i + 1];
      cache[cache_index(slot, 0, rank + 2 * i, 1, Dl, ps, slab)] = from_f<T>(a * c - b * s);
      cache[cache_index(slot, 0, rank + 2 * i + 1, 1, Dl, ps, slab)] = from_f<T>(b * c + a * s);
    }
  }
  for (int idx = threadIdx.x; idx < H * half; idx += 128) {
    const int h = idx / half, i = idx - h * half;
    const T* qr = q + (size_t)t * ldq_t + (size_t)h * ldq_h + dim;
    const float a = to_f(qr[2 * i]), b = to_f(qr[2 * i + 1]);
    const float c = cs[2 * i], s = cs[2 * i + 1];
    T* dst = q_full + ((size_t)t * H + h) * Dl + rank;
    dst[2 * i] = from_f<T>(a * c - b * s);
    dst[2 * i + 1] = from_f<T>(b * c + a * s);
  }
}

// Plain causal multi-query attention over the latent cache: one warp per (token, head), 4 consecutive tokens of one
// head per block. Keys are the rows [latent | rotated key] of width Dl, values their first `rank` columns. Scores:
// one key per lane; P.V: value columns across lanes.
template <typename T, int MAXR>
__global__ void __launch_bounds__(128) latent_attn_kernel(
    const T* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ block_table, int bt_stride,
    const int* __restrict__ qsl, const int* __restrict__ positions, int ntok, int nseq, float scale, int H, int Dl,
    int rank, T* __restrict__ out, int ps, int slab) {
  extern __shared__ float qs_all[];      // [4][Dl]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp, h = blockIdx.y;
  if (t >= ntok) return;
  float* qs = qs_all + (size_t)warp * Dl;
  const int s = find_seq(qsl, nseq, t);
  const int i = positions[t];
  const T* qrow = q + ((size_t)t * H + h) * Dl;
  for (int d = lane; d < Dl; d += 32) qs[d] = to_f(qrow[d]);
  __syncwarp();
  const int* bt = block_table + (size_t)s * bt_stride;
  const int nslab = Dl / slab;
  const size_t page_stride = (size_t)Dl * ps;
  float m = -INFINITY, l = 0.f;
  float acc[MAXR];
#pragma unroll
  for (int r = 0; r < MAXR; ++r) acc[r] = 0.f;
  for (int j0 = 0; j0 <= i; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j <= i;
    size_t base = 0;
    float sc = -INFINITY;
    if (valid) {
      base = (size_t)bt[j / ps] * page_stride + (size_t)(j % ps) * slab;
      float dot = 0.f;
      for (int c = 0; c < nslab; ++c) {
        const T* kr = cache + base + (size_t)c * ps * slab;
        const float* qq = qs + c * slab;
        for (int e = 0; e < slab; ++e) dot = fmaf(qq[e], to_f(kr[e]), dot);
      }
      sc = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float alpha = expf(m - m_new);          // m == -inf only before the first key: exp(-inf) == 0
    const float p = valid ? expf(sc - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int r = 0; r < MAXR; ++r) acc[r] *= alpha;
    const int cnt = min(32, i - j0 + 1);
    for (int kk = 0; kk < cnt; ++kk) {
      const float pj = __shfl_sync(0xffffffffu, p, kk);
      const unsigned long long bj = __shfl_sync(0xffffffffu, (unsigned long long)base, kk);
#pragma unroll
      for (int r = 0; r < MAXR; ++r) {
        const int d = lane + 32 * r;
        if (d < rank) acc[r] = fmaf(pj, to_f(cache[bj + (size_t)(d / slab) * ps * slab + d % slab]), acc[r]);
      }
    }
  }
  T* orow = out + ((size_t)t * H + h) * rank;
  const float inv = 1.0f / l;
#pragma unroll
  for (int r = 0; r < MAXR; ++r) {
    const int d = lane + 32 * r;
    if (d < rank) orow[d] = from_f<T>(acc[r] * inv);
  }
}

// ------------------------------------------------------------------------------------------------
// Grouped router selection, one warp per token over its fp32 logits [E]: scores = softmax over all E (`sigmoid`:
// 1 / (1 + exp(-logit)) of every logit by itself); choice = score + correction; E / n_groups neighbours form a group
// whose score is the sum of its `group_top` largest choices (1: its largest); only the `keep` best groups stay
// eligible; the top_k largest eligible choices are taken (ties: the lower index); weights = the chosen scores /
// (their sum + 1e-20) * scale, or without `renorm` the chosen scores * scale.
__global__ void __launch_bounds__(128) grouped_router_select_kernel(
    const float* __restrict__ logits, const float* __restrict__ correction, int ntok, int E, int top_k, int n_groups,
    int keep, float scale, float* __restrict__ wout, int* __restrict__ ids, int sigmoid, int group_top, int renorm) {
  extern __shared__ float rs[];          // per warp: score [E], choice [E], group score [n_groups]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= ntok) return;
  float* score = rs + (size_t)warp * (2 * E + n_groups);
  float* choice = score + E;
  float* gscore = choice + E;
  const float* z = logits + (size_t)t * E;
  if (sigmoid) {
    for (int e = lane; e < E; e += 32) {
      const float sc = 1.0f / (1.0f + expf(-z[e]));
      score[e] = sc;
      choice[e] = sc + (correction != nullptr ? correction[e] : 0.f);
    }
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float den = 0.f;
    for (int e = lane; e < E; e += 32) { const float p = expf(z[e] - mx); score[e] = p; den += p; }
    den = warp_sum(den);
    for (int e = lane; e < E; e += 32) {
      const float sc = score[e] / den;
      score[e] = sc;
      choice[e] = sc + (correction != nullptr ? correction[e] : 0.f);
    }
  }
  __syncwarp();
  if (n_groups > 1) {
    const int per = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float b = -INFINITY;
      if (group_top <= 1 || per < 2) {
        for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, choice[e]);
      } else {                                   // the sum of the group's largest `group_top` choices
        float last = INFINITY;
        int last_i = -1;
        b = 0.f;
        for (int r = 0; r < min(group_top, per); ++r) {
          float m = -INFINITY;
          int mi = -1;
          for (int e = g * per; e < (g + 1) * per; ++e) {
            const float v = choice[e];
            const bool after = v < last || (v == last && e > last_i);       // not taken in an earlier round
            if (after && (v > m || mi < 0)) { m = v; mi = e; }
          }
          b += m;
          last = m;
          last_i = mi;
        }
      }
      gscore[g] = b;
    }
    __syncwarp();
    for (int kk = 0; kk < keep; ++kk) {            // the kept groups get +inf as their mark
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = gscore[g];
        if (v != INFINITY && (v > best || (v == best && g < bi))) { best = v; bi = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi < 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
      }
      if (lane == 0 && bi < n_groups) gscore[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gscore[e / per] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  float sum = 0.f;
  for (int kk = 0; kk < top_k; ++kk) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = choice[e];
      if (v > best) { best = v; bi = e; }          // ascending e within a lane: the lower index wins ties
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    float sc = 0.f;
    if (bi < E) {
      sc = score[bi];
      __syncwarp();
      if (lane == 0) choice[bi] = -INFINITY;
      __syncwarp();
    } else {
      bi = 0;                                      // fewer eligible outputs than choices: a zero-weight slot
    }
    sum += sc;
    if (lane == 0) { ids[(size_t)t * top_k + kk] = bi; wout[(size_t)t * top_k + kk] = sc; }
  }
  __syncwarp();
  if (lane == 0)
    for (int kk = 0; kk < top_k; ++kk)
      wout[(size_t)t * top_k + kk] = renorm ? wout[(size_t)t * top_k + kk] / (sum + 1e-20f) * scale
                                            : wout[(size_t)t * top_k + kk] * scale;
}

// out[t, f] = g sigmoid(alpha g) (u + 1), g = min(gu[t, f], limit), u = clamp(gu[t, F + f], +-limit)
template <typename T>
__global__ void glu_clamp_kernel(const T* __restrict__ gu, long ld, int F, T* __restrict__ out, size_t total,
                                 float limit, float alpha) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / F, f = i - t * F;
  const float g = fminf(to_f(gu[t * ld + f]), limit);
  const float u = fminf(fmaxf(to_f(gu[t * ld + F + f]), -limit), limit);
  out[i] = from_f<T>(g * sigmoid_f(alpha * g) * (u + 1.0f));
}

// out[t, c] += w[t, k] * h[t, c] for every chosen identity expert (id >= n_real); the routed sum of the real
// experts is already in out (grouped tensor-core path)
template <typename T>
__global__ void identity_experts_add_kernel(const T* __restrict__ h, long ldh, const int* __restrict__ ids,
                                            const float* __restrict__ wts, int top_k, int n_real, int width,
                                            T* __restrict__ out, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / width, c = i - t * width;
  float w = 0.f;
  for (int kk = 0; kk < top_k; ++kk)
    if (ids[t * top_k + kk] >= n_real) w += wts[t * top_k + kk];
  if (w != 0.f) out[i] = from_f<T>(to_f(out[i]) + w * to_f(h[t * ldh + c]));
}

}  // namespace

#define GLLM_BY_DTYPE(is_f32, CALL_BF16, CALL_F32) \
  do { if (is_f32) { CALL_F32; } else { CALL_BF16; } } while (0)
typedef __nv_bfloat16 bf16_t;

GLLM_EXPORT int gllm_lat_rms_rows(const void* x, long ldx, const void* w, void* out, int ntok, int n, float eps,
                                  int is_f32, void* stream) {
  if (ntok <= 0 || n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((ntok + 3) / 4);
  GLLM_BY_DTYPE(is_f32,
                (rms_rows_kernel<bf16_t><<<blocks, 128, 0, st>>>((const bf16_t*)x, ldx, (const bf16_t*)w, (bf16_t*)out,
                                                                 ntok, n, eps)),
                (rms_rows_kernel<float><<<blocks, 128, 0, st>>>((const float*)x, ldx, (const float*)w, (float*)out,
                                                                ntok, n, eps)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

// out_f32: the result is fp32 whatever the operand type
GLLM_EXPORT int gllm_lat_gemm_batched(const void* A, long lda, long sa, const void* W, long ldw, long sw, void* C,
                                      long ldc, long sc, int M, int N, int K, int B, int is_f32, int out_f32,
                                      void* stream) {
  if (M <= 0 || N <= 0 || B <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((N + 63) / 64, (M + 63) / 64, B);
  if (is_f32)
    gemm_batched_simt_kernel<float, float><<<grid, 256, 0, st>>>((const float*)A, lda, sa, (const float*)W, ldw, sw,
                                                                 (float*)C, ldc, sc, M, N, K);
  else if (out_f32)
    gemm_batched_simt_kernel<bf16_t, float><<<grid, 256, 0, st>>>((const bf16_t*)A, lda, sa, (const bf16_t*)W, ldw, sw,
                                                                  (float*)C, ldc, sc, M, N, K);
  else
    gemm_batched_simt_kernel<bf16_t, bf16_t><<<grid, 256, 0, st>>>((const bf16_t*)A, lda, sa, (const bf16_t*)W, ldw,
                                                                   sw, (bf16_t*)C, ldc, sc, M, N, K);
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

// chunk_len > 0: the two-pass chunked form with `summary` [nseq, max_chunks, C] float2 scratch
GLLM_EXPORT int gllm_lat_rglru_scan(const void* u, const void* gates, const void* gbias, const void* c_decay,
                                    const void* y_pre, long ldy, const void* y_bias, void* state,
                                    const void* rec_slots, const void* seq_lens, const void* qsl, int nseq, int C,
                                    int bw, void* out, int chunk_len, int max_chunks, void* summary, int is_f32,
                                    void* stream) {
  if (nseq <= 0 || C <= 0) return 0;
  if (bw <= 0 || C % bw != 0) return 2;
  cudaStream_t st = (cudaStream_t)stream;
  const int cb = (C + 127) / 128;
  if (chunk_len > 0 && max_chunks > 1 && summary != nullptr) {
    dim3 grid(nseq, max_chunks, cb);
    if (is_f32) {
      rglru_chunk_summary_kernel<float><<<grid, 128, 0, st>>>((const float*)u, (const float*)gates,
                                                              (const float*)gbias, (const float*)c_decay,
                                                              (const int*)qsl, C, bw, chunk_len, max_chunks,
                                                              (float2*)summary);
      rglru_chunk_apply_kernel<float><<<grid, 128, 0, st>>>(
          (const float*)u, (const float*)gates, (const float*)gbias, (const float*)c_decay, (const float*)y_pre, ldy,
          (const float*)y_bias, (float*)state, (const int*)rec_slots, (const int*)seq_lens, (const int*)qsl, C, bw,
          chunk_len, max_chunks, (const float2*)summary, (float*)out);
    } else {
      rglru_chunk_summary_kernel<bf16_t><<<grid, 128, 0, st>>>((const bf16_t*)u, (const float*)gates,
                                                               (const float*)gbias, (const float*)c_decay,
                                                               (const int*)qsl, C, bw, chunk_len, max_chunks,
                                                               (float2*)summary);
      rglru_chunk_apply_kernel<bf16_t><<<grid, 128, 0, st>>>(
          (const bf16_t*)u, (const float*)gates, (const float*)gbias, (const float*)c_decay, (const bf16_t*)y_pre, ldy,
          (const float*)y_bias, (float*)state, (const int*)rec_slots, (const int*)seq_lens, (const int*)qsl, C, bw,
          chunk_len, max_chunks, (const float2*)summary, (bf16_t*)out);
    }
  } else {
    dim3 grid(nseq, cb);
    GLLM_BY_DTYPE(is_f32,
                  (rglru_serial_kernel<bf16_t><<<grid, 128, 0, st>>>(
                      (const bf16_t*)u, (const float*)gates, (const float*)gbias, (const float*)c_decay,
                      (const bf16_t*)y_pre, ldy, (const float*)y_bias, (float*)state, (const int*)rec_slots,
                      (const int*)seq_lens, (const int*)qsl, C, bw, (bf16_t*)out)),
                  (rglru_serial_kernel<float><<<grid, 128, 0, st>>>(
                      (const float*)u, (const float*)gates, (const float*)gbias, (const float*)c_decay,
                      (const float*)y_pre, ldy, (const float*)y_bias, (float*)state, (const int*)rec_slots,
                      (const int*)seq_lens, (const int*)qsl, C, bw, (float*)out)));
  }
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_lat_norm_rope_write(const void* q, long ldq_t, long ldq_h, int H, int dim, const void* dkv,
                                         long ldkv, int rank, int rot, const void* norm_w, float eps,
                                         const void* positions, const void* freqs, float mag, void* q_full,
                                         void* cache, const void* slots, int ps, int slab, int ntok, int is_f32,
                                         void* stream) {
  if (ntok <= 0) return 0;
  if (rot % 2 != 0) return 2;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)(rot > 0 ? rot : 2) * sizeof(float);
  GLLM_BY_DTYPE(is_f32,
                (latent_norm_rope_write_kernel<bf16_t><<<ntok, 128, smem, st>>>(
                    (const bf16_t*)q, ldq_t, ldq_h, H, dim, (const bf16_t*)dkv, ldkv, rank, rot, (const bf16_t*)norm_w,
                    eps, (const int*)positions, (const float*)freqs, mag, (bf16_t*)q_full, (bf16_t*)cache,
                    (const int*)slots, ps, slab)),
                (latent_norm_rope_write_kernel<float><<<ntok, 128, smem, st>>>(
                    (const float*)q, ldq_t, ldq_h, H, dim, (const float*)dkv, ldkv, rank, rot, (const float*)norm_w,
                    eps, (const int*)positions, (const float*)freqs, mag, (float*)q_full, (float*)cache,
                    (const int*)slots, ps, slab)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

namespace {
template <typename T>
int latent_attn_dispatch(dim3 grid, size_t smem, cudaStream_t st, const void* q, const void* cache, const int* bt,
                         int bt_stride, const int* qsl, const int* pos, int ntok, int nseq, float scale, int H, int Dl,
                         int rank, void* out, int ps, int slab) {
#define GLLM_LATTN(R)                                                                                          \
  do {                                                                                                         \
    if (smem > 48 * 1024)                                                                                      \
      cudaFuncSetAttribute(latent_attn_kernel<T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    latent_attn_kernel<T, R><<<grid, 128, smem, st>>>((const T*)q, (const T*)cache, bt, bt_stride, qsl, pos,    \
                                                      ntok, nseq, scale, H, Dl, rank, (T*)out, ps, slab);       \
  } while (0)
  if (rank <= 64) GLLM_LATTN(2);
  else if (rank <= 128) GLLM_LATTN(4);
  else if (rank <= 256) GLLM_LATTN(8);
  else if (rank <= 512) GLLM_LATTN(16);
  else return 2;
#undef GLLM_LATTN
  return 0;
}
}  // namespace

GLLM_EXPORT int gllm_lat_attention(const void* q, const void* cache, const void* block_table, int bt_stride,
                                   const void* qsl, const void* positions, int ntok, int nseq, float scale, int H,
                                   int Dl, int rank, void* out, int ps, int slab, int is_f32, void* stream) {
  if (ntok <= 0) return 0;
  if (Dl % slab != 0 || rank > Dl) return 2;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((ntok + 3) / 4, H);
  const size_t smem = (size_t)4 * Dl * sizeof(float);
  if (smem > 200 * 1024) return 2;
  int rc;
  if (is_f32)
    rc = latent_attn_dispatch<float>(grid, smem, st, q, cache, (const int*)block_table, bt_stride, (const int*)qsl,
                                     (const int*)positions, ntok, nseq, scale, H, Dl, rank, out, ps, slab);
  else
    rc = latent_attn_dispatch<bf16_t>(grid, smem, st, q, cache, (const int*)block_table, bt_stride, (const int*)qsl,
                                      (const int*)positions, ntok, nseq, scale, H, Dl, rank, out, ps, slab);
  if (rc) return rc;
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_lat_grouped_router_select(const void* logits, const void* correction, int ntok, int E, int top_k,
                                               int n_groups, int keep, float scale, void* wout, void* ids,
                                               int sigmoid, int group_top, int renorm, void* stream) {
  if (ntok <= 0) return 0;
  if (top_k > E || E > 4096 || n_groups < 1 || E % n_groups != 0 || keep < 1 || keep > n_groups) return 2;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)4 * (2 * E + n_groups) * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(grouped_router_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  grouped_router_select_kernel<<<(ntok + 3) / 4, 128, smem, st>>>((const float*)logits, (const float*)correction,
                                                                  ntok, E, top_k, n_groups, keep, scale,
                                                                  (float*)wout, (int*)ids, sigmoid, group_top, renorm);
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_lat_glu_clamp(const void* gu, long ld, int ntok, int F, void* out, float limit, float alpha,
                                   int is_f32, void* stream) {
  if (ntok <= 0 || F <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t total = (size_t)ntok * F;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  GLLM_BY_DTYPE(is_f32,
                (glu_clamp_kernel<bf16_t><<<blocks, 256, 0, st>>>((const bf16_t*)gu, ld, F, (bf16_t*)out, total, limit,
                                                                  alpha)),
                (glu_clamp_kernel<float><<<blocks, 256, 0, st>>>((const float*)gu, ld, F, (float*)out, total, limit,
                                                                 alpha)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_lat_identity_experts_add(const void* h, long ldh, const void* ids, const void* wts, int ntok,
                                              int top_k, int n_real, int width, void* out, int is_f32, void* stream) {
  if (ntok <= 0 || width <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t total = (size_t)ntok * width;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  GLLM_BY_DTYPE(is_f32,
                (identity_experts_add_kernel<bf16_t><<<blocks, 256, 0, st>>>(
                    (const bf16_t*)h, ldh, (const int*)ids, (const float*)wts, top_k, n_real, width, (bf16_t*)out,
                    total)),
                (identity_experts_add_kernel<float><<<blocks, 256, 0, st>>>(
                    (const float*)h, ldh, (const int*)ids, (const float*)wts, top_k, n_real, width, (float*)out,
                    total)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}
