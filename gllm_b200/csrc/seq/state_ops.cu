// Kernels of the norm-after-sum layer-list decoders (models/hybrid.py, block "postnorm"): the fused residual update
// x <- rms(alpha x + y) w, per-head q/k RMS norm + rotate-half rotary + paged K / V cache write, the matrix-state
// linear recurrences (gated delta rule, constant-decay linear attention) with slot-indexed fp32 state, the grouped
// RMS norm with a gate, SiLU-gated product, fp32 router logits (per-warp dots or mma.sync tiles) and the top-k
// selection with softmax over the chosen logits, plain
// per-slot expert kernels for shapes / dtypes the grouped tcgen05 GEMM does not take, and the logit cap.
//
// Templated on the compute dtype T (bf16 or float); norms, gates, decays, softplus, the router, the recurrences and
// their state are fp32 in both. Compiled WITHOUT --use_fast_math (build.py). Results of a row never depend on which
// other rows share the launch: every reduction has a fixed order.
#include <cuda_bf16.h>

#include "common/host_utils.h"
#include "seq/seq_common.cuh"

namespace {
using namespace seqk;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

// x <- rms(alpha * x + y) * w (fp32 stream, in place); out = the same row in the compute dtype (optional)
template <typename T>
__global__ void __launch_bounds__(256) postnorm_kernel(float* __restrict__ x, const T* __restrict__ y, long ldy,
                                                       const T* __restrict__ w, T* __restrict__ out, int width,
                                                       float alpha, float eps) {
  __shared__ float scratch[8];
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * width;
  const T* yr = y + (size_t)t * ldy;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += 256) {
    const float v = fmaf(alpha, xr[i], to_f(yr[i]));
    ss += v * v;
  }
  ss = block_sum<256>(ss, scratch);
  const float r = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += 256) {
    const float v = fmaf(alpha, xr[i], to_f(yr[i])) * r * to_f(w[i]);
    xr[i] = v;
    if (out != nullptr) out[(size_t)t * width + i] = from_f<T>(v);
  }
}

// One block per token; its warps walk the heads: [0, H) queries, [H, H + G) keys, [H + G, H + 2G) values (copied to
// the V cache). q / k: RMS norm over D with a shared weight, then entries i and i + rot/2 (i < rot/2) turn by
// pos * base^(-2i/rot). The token's cos / sin row is formed once per block, the angle in fp64 (no table, no maximum
// position), the rotation itself in fp32. `freqs` (fp64, one per pair) replaces the powers of the base (scaled
// frequencies); cos and sin are multiplied by `mag`. With G == 0 a row holds queries only (the keys and values are
// another layer's) and no cache is touched.
template <typename T>
__global__ void __launch_bounds__(256) qk_norm_rope_kv_write_kernel(
    const T* __restrict__ qkv, long ld, int H, int G, int D, int Dv, const T* __restrict__ qn,
    const T* __restrict__ kn, float eps, const int* __restrict__ positions, int rot, double log2_base,
    T* __restrict__ q_out, T* __restrict__ kc, T* __restrict__ vc, const int* __restrict__ slots, int ps, int slab,
    int slab_v, const double* __restrict__ freqs, float mag) {
  extern __shared__ float cs_tab[];      // [rot / 2] cos, then [rot / 2] sin
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int half = rot / 2;
  const double pos = (double)positions[t];
  for (int i = threadIdx.x; i < half; i += 256) {
    double sn, cs;
    sincos(pos * (freqs != nullptr ? freqs[i] : exp2(-(2.0 * (double)i / (double)rot) * log2_base)), &sn, &cs);
    cs_tab[i] = (float)(cs * (double)mag);
    cs_tab[half + i] = (float)(sn * (double)mag);
  }
  __syncthreads();
  const int slot = G > 0 ? slots[t] : -1;
  for (int head = warp; head < H + 2 * G; head += 8) {
    if (head >= H + G) {
      if (slot < 0) continue;
      const int g = head - H - G;
      const T* src = qkv + (size_t)t * ld + (size_t)(H + G) * D + (size_t)g * Dv;
      for (int d = lane; d < Dv; d += 32) vc[cache_index(slot, g, d, G, Dv, ps, slab_v)] = src[d];
      continue;
    }
    if (head >= H && slot < 0) continue;
    const T* src = qkv + (size_t)t * ld + (size_t)head * D;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) { const float v = to_f(src[d]); ss += v * v; }
    ss = warp_sum(ss);
    const T* w = head < H ? qn : kn;
    const float r = w != nullptr ? 1.0f / sqrtf(ss / (float)D + eps) : 1.0f;
    for (int d = lane; d < D; d += 32) {
      float v = to_f(src[d]) * r * (w != nullptr ? to_f(w[d]) : 1.0f);
      if (d < rot) {
        const int i = d < half ? d : d - half, pd = d < half ? d + half : d - half;
        const float other = to_f(src[pd]) * r * (w != nullptr ? to_f(w[pd]) : 1.0f);
        const float c = cs_tab[i], sn = cs_tab[half + i];
        v = d < half ? v * c - other * sn : v * c + other * sn;
      }
      if (head < H) q_out[(size_t)t * H * D + (size_t)head * D + d] = from_f<T>(v);
      else kc[cache_index(slot, head - H, d, G, D, ps, slab)] = from_f<T>(v);
    }
  }
}

// Matrix-state recurrence, one block per (sequence, head, 32 value columns). A value column's D state entries are
// split over PARTS adjacent lanes (entry d = part + PARTS j), NS per lane in registers; per token
//     S <- g S;  u = delta ? beta (v - S^T k) : v;  S <- S + k u^T;  o = S^T q
// costs two register passes and two PARTS-lane shuffle reductions (PARTS = 8 for head sizes >= 128: half the
// registers per thread, twice the warps in flight). q / k rows and the per-token g, beta of TCH tokens are staged
// in shared memory by the whole block (SiLU, unit length and the q scale applied there). With KD the decay is one
// value per key channel, gk[t, h * D + d] in fp32 (`key_decay_kernel`), acting on row d; it is staged beside the key as
// (k, decay) pairs, so the update still costs two shared loads per state entry.
template <typename T, int NS, int PARTS, bool KD>
__global__ void __launch_bounds__(32 * PARTS) linear_state_kernel(
    const T* __restrict__ q, long ldq, const T* __restrict__ k, long ldk, const T* __restrict__ v, long ldv,
    const T* __restrict__ beta, long ldb, const T* __restrict__ a, long lda, const float* __restrict__ neg_a,
    const float* __restrict__ dt_bias, const float* __restrict__ decay, float* __restrict__ state,
    const int* __restrict__ rec_slots, const int* __restrict__ seq_lens, const int* __restrict__ qsl, int H, int G,
    int D, int V, int silu_in, int unit_qk, float q_scale, int delta, float* __restrict__ out,
    const float* __restrict__ gk, long ldgk) {
  constexpr int TCH = 8;               // tokens staged per round (16 measured 2.4x slower: registers)
  constexpr int ROWS = KD ? 3 : 2;
  extern __shared__ float sm[];
  // per token TS floats: [q row | k row], or with KD [(k, decay) pairs | q row] on an even stride (8-byte loads)
  const int TS = KD ? ((3 * D + 1) & ~1) : 2 * D;
  const int qoff = KD ? 2 * D : 0, koff = KD ? 0 : D;
  float* sq = sm;
  float* sg = sm + TCH * TS;           // [TCH][2]: g, beta
  const int s = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int NT = 32 * PARTS, NW = PARTS;       // threads and warps per block
  const int vl = threadIdx.x / PARTS, part = threadIdx.x % PARTS;
  const int vcol = blockIdx.z * 32 + vl;
  const bool active = vcol < V;
  const int vc = active ? vcol : V - 1;          // idle lanes mirror the last column (loads only)
  const int q0 = qsl[s], q1 = qsl[s + 1];
  if (q1 <= q0) return;                          // uniform over the block
  const bool carried = state != nullptr && (seq_lens[s] - (q1 - q0)) > 0;
  float* st = state != nullptr ? state + ((size_t)rec_slots[s] * H + h) * (size_t)D * V : nullptr;
  float S[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int d = part + PARTS * j;
    S[j] = (carried && d < D) ? st[(size_t)d * V + vc] : 0.f;
  }
  const int kvh = h / (H / G);
  for (int t0 = q0; t0 < q1; t0 += TCH) {
    const int nt = min(TCH, q1 - t0);
    __syncthreads();                             // the previous chunk's rows are consumed
    for (int idx = threadIdx.x; idx < nt * ROWS * D; idx += NT) {
      const int kk = idx / (ROWS * D), r = idx - kk * ROWS * D;
      float f;
      const int dst = kk * TS + (!KD ? r : r < D ? qoff + r : r < 2 * D ? 2 * (r - D) : 2 * (r - 2 * D) + 1);
      if (KD && r >= 2 * D) {
        f = gk[(size_t)(t0 + kk) * ldgk + h * D + r - 2 * D];
      } else {
        f = r < D ? to_f(q[(size_t)(t0 + kk) * ldq + (size_t)kvh * D + r])
                  : to_f(k[(size_t)(t0 + kk) * ldk + (size_t)kvh * D + r - D]);
        if (silu_in) f = silu_f(f);
      }
      sq[dst] = f;
    }
    if (threadIdx.x < nt) {
      float g, b = 1.0f;
      if (KD) {
        g = 1.0f;
      } else if (decay != nullptr) {
        g = decay[h];
      } else {
        const float z = to_f(a[(size_t)(t0 + threadIdx.x) * lda + h]) + dt_bias[h];
        g = expf(neg_a[h] * (z > 20.0f ? z : log1pf(expf(z))));
      }
      if (delta) b = sigmoid_f(to_f(beta[(size_t)(t0 + threadIdx.x) * ldb + h]));
      sg[threadIdx.x * 2] = g;
      sg[threadIdx.x * 2 + 1] = b;
    }
    __syncthreads();
    if (unit_qk || q_scale != 1.0f) {
      for (int row = warp; row < 2 * nt; row += NW) {      // row = token * 2 + (0: q, 1: k)
        if (KD && (row & 1)) continue;                       // keys are neither scaled nor normed with a key decay
        float* ptr = sq + (size_t)(row >> 1) * TS + ((row & 1) ? koff : qoff);
        float sc = (row & 1) ? 1.0f : q_scale;
        if (unit_qk) {
          float ss = 0.f;
          for (int d = lane; d < D; d += 32) ss += ptr[d] * ptr[d];
          sc /= sqrtf(warp_sum(ss) + 1e-6f);
        }
        for (int d = lane; d < D; d += 32) ptr[d] *= sc;
      }
      __syncthreads();
    }
    float vv[TCH];
#pragma unroll
    for (int kk = 0; kk < TCH; ++kk) {
      if (kk < nt) {
        const float f = to_f(v[(size_t)(t0 + kk) * ldv + (size_t)h * V + vc]);
        vv[kk] = silu_in ? silu_f(f) : f;
      }
    }
#pragma unroll
    for (int kk = 0; kk < TCH; ++kk) {
      if (kk < nt) {
        const float* qq = sq + (size_t)kk * TS + qoff;
        const float* kr = sq + (size_t)kk * TS + koff;
        const float2* kg = reinterpret_cast<const float2*>(kr);      // with KD: (k, decay) pairs
        const float g = sg[kk * 2], b = sg[kk * 2 + 1];
        float u = vv[kk];
        if (delta) {
          float dot = 0.f;
#pragma unroll
          for (int j = 0; j < NS; ++j) {
            const int d = part + PARTS * j;
            if (d < D) dot = fmaf(S[j], kr[d], dot);
          }
#pragma unroll
          for (int o = 1; o < PARTS; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
          u = b * (u - g * dot);
        }
        float o = 0.f;
#pragma unroll
        for (int j = 0; j < NS; ++j) {
          const int d = part + PARTS * j;
          if (d < D) {
            if (KD) {
              const float2 p = kg[d];
              S[j] = fmaf(p.x, u, p.y * S[j]);
            } else {
              S[j] = fmaf(kr[d], u, g * S[j]);
            }
            o = fmaf(S[j], qq[d], o);
          }
        }
#pragma unroll
        for (int sh = 1; sh < PARTS; sh <<= 1) o += __shfl_xor_sync(0xffffffffu, o, sh);
        if (active && part == 0) out[(size_t)(t0 + kk) * H * V + (size_t)h * V + vcol] = o;
      }
    }
  }
  if (st != nullptr && active) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      const int d = part + PARTS * j;
      if (d < D) st[(size_t)d * V + vcol] = S[j];
    }
  }
}

// one warp per (token, group): out = rms_group(o) * w[col % wlen] * act(gate) * out_scale
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ o, int n, const T* __restrict__ gate, long ldg,
                                        const T* __restrict__ w, int wlen, int group, float eps, int act,
                                        float out_scale, T* __restrict__ out, long ldo, int ntok) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ngroups = n / group;
  const long gw = (long)blockIdx.x * 4 + warp;
  if (gw >= (long)ntok * ngroups) return;
  const int t = (int)(gw / ngroups), gi = (int)(gw % ngroups);
  const float* src = o + (size_t)t * n + (size_t)gi * group;
  float ss = 0.f;
  for (int d = lane; d < group; d += 32) ss += src[d] * src[d];
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / (float)group + eps);
  for (int d = lane; d < group; d += 32) {
    const int col = gi * group + d;
    const float gt = to_f(gate[(size_t)t * ldg + col]);
    const float ga = act ? sigmoid_f(gt) : silu_f(gt);
    out[(size_t)t * ldo + col] = from_f<T>(src[d] * r * to_f(w[col % wlen]) * ga * out_scale);
  }
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, long ld, int F, T* __restrict__ out, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / F, f = i - t * F;
  out[i] = from_f<T>(silu_f(to_f(gu[t * ld + f])) * to_f(gu[t * ld + F + f]));
}

// Router logits for small batches: one warp per (token, expert), lanes over the width in a fixed order, fp32 result.
template <typename T>
__global__ void __launch_bounds__(128) router_logits_kernel(const T* __restrict__ h, long ldh, const T* __restrict__ w,
                                                            int width, int E, float* __restrict__ logits) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int e = blockIdx.y * 4 + warp;
  if (e >= E) return;
  const T* hr = h + (size_t)t * ldh;
  const T* wr = w + (size_t)e * width;
  float acc = 0.f;
  for (int i = lane; i < width; i += 32) acc = fmaf(to_f(hr[i]), to_f(wr[i]), acc);
  acc = warp_sum(acc);
  if (lane == 0) logits[(size_t)t * E + e] = acc;
}

// Router logits for large bf16 batches on the tensor cores, result kept in fp32: one warp computes 16 tokens x up to
// NT * 8 experts with mma.sync m16n8k16 (bf16 products are exact in fp32, accumulation is fp32), operand fragments
// read straight from global memory (the router weight stays in L1 / L2). width % 16 == 0, rows 4-byte aligned.
template <int NT>
__global__ void __launch_bounds__(128) router_logits_mma_kernel(const __nv_bfloat16* __restrict__ h, long ldh,
                                                                const __nv_bfloat16* __restrict__ w, int ntok,
                                                                int width, int E, float* __restrict__ logits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int row0 = (blockIdx.x * 4 + warp) * 16;
  const int e0 = blockIdx.y * NT * 8;
  if (row0 >= ntok) return;
  const int ra = min(row0 + g, ntok - 1), rb = min(row0 + g + 8, ntok - 1);   // clamped rows are never stored
  const __nv_bfloat16* ha = h + (size_t)ra * ldh + 2 * t4;
  const __nv_bfloat16* hb = h + (size_t)rb * ldh + 2 * t4;
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
  for (int k0 = 0; k0 < width; k0 += 16) {
    uint32_t a[4];
    a[0] = *reinterpret_cast<const uint32_t*>(ha + k0);
    a[1] = *reinterpret_cast<const uint32_t*>(hb + k0);
    a[2] = *reinterpret_cast<const uint32_t*>(ha + k0 + 8);
    a[3] = *reinterpret_cast<const uint32_t*>(hb + k0 + 8);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int e = e0 + n * 8 + g;
      uint32_t b0 = 0u, b1 = 0u;
      if (e < E) {
        const __nv_bfloat16* wr = w + (size_t)e * width + k0 + 2 * t4;
        b0 = *reinterpret_cast<const uint32_t*>(wr);
        b1 = *reinterpret_cast<const uint32_t*>(wr + 8);
      }
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
          "{%0, %1, %2, %3};"
          : "+f"(acc[n][0]), "+f"(acc[n][1]), "+f"(acc[n][2]), "+f"(acc[n][3])
          : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
  }
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int e = e0 + n * 8 + 2 * t4;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = row0 + g + (c >> 1) * 8, ee = e + (c & 1);
      if (r < ntok && ee < E) logits[(size_t)r * E + ee] = acc[n][c];
    }
  }
}

// Batched product with an fp32 result on the tensor cores: C_b[M, N] = A_b[M, K] . W_b[N, K]^T (bf16 operands, exact
// products, fp32 accumulation in a fixed order per row). One warp computes 16 rows x NT * 8 columns with mma.sync
// m16n8k16. The contraction index may be permuted as long as both operands use the same permutation, so a lane
// takes 8 CONSECUTIVE k of its row with one 16-byte load (k0 + 8 t4 ...): entries 0..3 feed one mma's two k slots of
// that lane, entries 4..7 a second mma. K % 32 == 0; rows, batch strides and bases 16-byte aligned.
// SPLIT (few columns, e.g. router logits: too few 16-row tiles to fill the machine): the block's four warps share one
// 16-row tile, each over a quarter of K (K % 128 == 0), and warp 0 adds the partial sums in warp order.
template <int NT, bool SPLIT>
__global__ void __launch_bounds__(128) gemm_mma_f32out_kernel(const __nv_bfloat16* __restrict__ A, long lda, long sa,
                                                              const __nv_bfloat16* __restrict__ W, long ldw, long sw,
                                                              float* __restrict__ C, long ldc, long sc, int M, int N,
                                                              int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  __shared__ float part[SPLIT ? 3 * NT * 4 * 32 : 1];
  const int row0 = SPLIT ? blockIdx.x * 16 : (blockIdx.x * 4 + warp) * 16;
  const int n0 = blockIdx.y * NT * 8;
  if (row0 >= M) return;
  A += (size_t)blockIdx.z * sa;
  W += (size_t)blockIdx.z * sw;
  C += (size_t)blockIdx.z * sc;
  const int ra = min(row0 + g, M - 1), rb = min(row0 + g + 8, M - 1);         // clamped rows are never stored
  const __nv_bfloat16* pa = A + (size_t)ra * lda + 8 * t4;
  const __nv_bfloat16* pb = A + (size_t)rb * lda + 8 * t4;
  const __nv_bfloat16* pw[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) pw[n] = W + (size_t)min(n0 + n * 8 + g, N - 1) * ldw + 8 * t4;
  float acc[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
  const int kbeg = SPLIT ? warp * (K / 4) : 0, kend = SPLIT ? kbeg + K / 4 : K;
#pragma unroll 2
  for (int k0 = kbeg; k0 < kend; k0 += 32) {
    const uint4 lo = *reinterpret_cast<const uint4*>(pa + k0);
    const uint4 hi = *reinterpret_cast<const uint4*>(pb + k0);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const uint4 b = *reinterpret_cast<const uint4*>(pw[n] + k0);
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
          "{%0, %1, %2, %3};"
          : "+f"(acc[n][0]), "+f"(acc[n][1]), "+f"(acc[n][2]), "+f"(acc[n][3])
          : "r"(lo.x), "r"(hi.x), "r"(lo.y), "r"(hi.y), "r"(b.x), "r"(b.y));
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
          "{%0, %1, %2, %3};"
          : "+f"(acc[n][0]), "+f"(acc[n][1]), "+f"(acc[n][2]), "+f"(acc[n][3])
          : "r"(lo.z), "r"(hi.z), "r"(lo.w), "r"(hi.w), "r"(b.z), "r"(b.w));
    }
  }
  if (SPLIT) {
    if (warp > 0) {
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) part[(((warp - 1) * NT + n) * 4 + c) * 32 + lane] = acc[n][c];
    }
    __syncthreads();
    if (warp > 0) return;
    for (int w = 0; w < 3; ++w)
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[n][c] += part[((w * NT + n) * 4 + c) * 32 + lane];
  }
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int col = n0 + n * 8 + 2 * t4;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = row0 + g + (c >> 1) * 8, cc = col + (c & 1);
      if (r < M && cc < N) C[(size_t)r * ldc + cc] = acc[n][c];
    }
  }
}

// Decay per key channel for the matrix-state recurrence: out[t, c] = sigmoid(z[t, c] + bias[c])^inv_tau in fp32, formed
// as exp(-softplus(-z) * inv_tau) (no cancellation for decays near 1).
template <typename T>
__global__ void key_decay_kernel(const T* __restrict__ z, long ldz, const float* __restrict__ bias, float inv_tau,
                                 float* __restrict__ out, int n, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / n;
  const int c = (int)(i - t * n);
  const float v = to_f(z[t * ldz + c]) + (bias != nullptr ? bias[c] : 0.f);
  out[i] = expf((fminf(v, 0.f) - log1pf(expf(-fabsf(v)))) * inv_tau);
}

// Router, second half: one warp per token over its fp32 logits [E] (the first half is the fp32-output GEMM): the
// top_k largest (ties: the lower index), then softmax over the chosen logits only. A lane owns experts lane,
// lane + 32, ...; chosen experts are tracked in a per-lane bit mask (E <= 1024).
__global__ void __launch_bounds__(128) router_select_kernel(const float* __restrict__ logits, int ntok, int E,
                                                            int top_k, float* __restrict__ wout,
                                                            int* __restrict__ ids) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= ntok) return;
  const float* z = logits + (size_t)t * E;
  unsigned taken = 0u;                   // bit j: expert lane + 32 j is chosen
  float m = 0.f, den = 0.f;
  for (int kk = 0; kk < top_k; ++kk) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane, j = 0; e < E; e += 32, ++j) {
      const float v = z[e];
      if (!((taken >> j) & 1u) && v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (bi >= E) {                       // only when every remaining logit is -inf / NaN: the first free expert
      int cand = 0x7fffffff;
      for (int e = lane, j = 0; e < E; e += 32, ++j)
        if (!((taken >> j) & 1u)) { cand = e; break; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
      bi = cand;
    }
    if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
    if (kk == 0) m = best;               // the first pick is the largest
    const float p = expf(best - m);
    den += p;
    if (lane == 0) { ids[(size_t)t * top_k + kk] = bi; wout[(size_t)t * top_k + kk] = p; }
  }
  __syncwarp();
  if (lane == 0)
    for (int kk = 0; kk < top_k; ++kk) wout[(size_t)t * top_k + kk] /= den;
}

// plain experts, first half: act[slot, f] = silu(gate_e[f] . h) * (up_e[f] . h); one warp per (slot, f). With
// limit > 0 the clamped form: g = min(gate, limit), u = clamp(up, +-limit), act = g sigmoid(alpha g) (u + 1).
// An id >= n_real names an identity expert: nothing to compute here. With `ungated` the experts have no gate:
// w13 is [E, F, width] (up rows only) and act = relu(up_e[f] . h)^2.
template <typename T>
__global__ void __launch_bounds__(128) moe_gate_up_kernel(const T* __restrict__ h, long ldh,
                                                          const T* __restrict__ w13, const int* __restrict__ ids,
                                                          int top_k, int width, int F, T* __restrict__ act,
                                                          int n_real, float limit, float alpha, int ungated) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = blockIdx.x, f = blockIdx.y * 4 + warp;
  if (f >= F) return;
  const int e = ids[slot];
  if (e >= n_real) return;
  const T* hr = h + (size_t)(slot / top_k) * ldh;
  if (ungated) {
    const T* ur = w13 + ((size_t)e * F + f) * width;
    float ua = 0.f;
    for (int i = lane; i < width; i += 32) ua = fmaf(to_f(hr[i]), to_f(ur[i]), ua);
    ua = fmaxf(warp_sum(ua), 0.f);
    if (lane == 0) act[(size_t)slot * F + f] = from_f<T>(ua * ua);
    return;
  }
  const T* gr = w13 + ((size_t)e * 2 * F + f) * width;
  const T* ur = gr + (size_t)F * width;
  float ga = 0.f, ua = 0.f;
  for (int i = lane; i < width; i += 32) {
    const float x = to_f(hr[i]);
    ga = fmaf(x, to_f(gr[i]), ga);
    ua = fmaf(x, to_f(ur[i]), ua);
  }
  ga = warp_sum(ga);
  ua = warp_sum(ua);
  if (lane == 0) {
    float r;
    if (limit > 0.f) {
      const float g = fminf(ga, limit), u = fminf(fmaxf(ua, -limit), limit);
      r = g * sigmoid_f(alpha * g) * (u + 1.0f);
    } else {
      r = silu_f(ga) * ua;
    }
    act[(size_t)slot * F + f] = from_f<T>(r);
  }
}

// plain experts, second half: out[t, c] = sum_k weight[t, k] * (down_e[c] . act[t * top_k + k]); one warp per (t, c).
// An identity expert (id >= n_real) contributes weight * h[t, c].
template <typename T>
__global__ void __launch_bounds__(128) moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w2,
                                                       const int* __restrict__ ids, const float* __restrict__ wts,
                                                       int top_k, int width, int F, T* __restrict__ out,
                                                       const T* __restrict__ h, long ldh, int n_real) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, c = blockIdx.y * 4 + warp;
  if (c >= width) return;
  float total = 0.f;
  for (int kk = 0; kk < top_k; ++kk) {
    const int e = ids[(size_t)t * top_k + kk];
    if (e >= n_real) {
      total = fmaf(wts[(size_t)t * top_k + kk], to_f(h[(size_t)t * ldh + c]), total);
      continue;
    }
    const T* ar = act + ((size_t)t * top_k + kk) * F;
    const T* dr = w2 + ((size_t)e * width + c) * F;
    float acc = 0.f;
    for (int i = lane; i < F; i += 32) acc = fmaf(to_f(ar[i]), to_f(dr[i]), acc);
    total = fmaf(wts[(size_t)t * top_k + kk], warp_sum(acc), total);
  }
  if (lane == 0) out[(size_t)t * width + c] = from_f<T>(total);
}

template <typename T>
__global__ void softcap_kernel(T* __restrict__ z, long ld, int n, float cap, size_t total) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / n, c = i - t * n;
  z[t * ld + c] = from_f<T>(cap * tanhf(to_f(z[t * ld + c]) / cap));
}

template <typename T>
int state_dispatch(dim3 grid, size_t smem, cudaStream_t st, const void* q, long ldq, const void* k, long ldk,
                   const void* v, long ldv, const void* beta, long ldb, const void* a, long lda, const float* neg_a,
                   const float* dt_bias, const float* decay, float* state, const int* rec_slots, const int* seq_lens,
                   const int* qsl, int H, int G, int D, int V, int silu_in, int unit_qk, float q_scale, int delta,
                   float* out, int parts, const float* zk, long ldz) {
#define GLLM_STATE_KD(NS, PARTS, KD)                                                                                \
  linear_state_kernel<T, NS, PARTS, KD><<<grid, 32 * PARTS, smem, st>>>(                                            \
      (const T*)q, ldq, (const T*)k, ldk, (const T*)v, ldv, (const T*)beta, ldb, (const T*)a, lda, neg_a, dt_bias,  \
      decay, state, rec_slots, seq_lens, qsl, H, G, D, V, silu_in, unit_qk, q_scale, delta, out, zk, ldz)
#define GLLM_STATE(NS, PARTS)                                               \
  do {                                                                      \
    if (zk != nullptr) GLLM_STATE_KD(NS, PARTS, true);                      \
    else GLLM_STATE_KD(NS, PARTS, false);                                   \
  } while (0)
  if (D <= 16) GLLM_STATE(4, 4);
  else if (D <= 32) GLLM_STATE(8, 4);
  else if (D <= 64) GLLM_STATE(16, 4);
  else if (D <= 128) { if (parts == 8) GLLM_STATE(16, 8); else GLLM_STATE(32, 4); }
  else if (D <= 256) { if (parts == 8) GLLM_STATE(32, 8); else GLLM_STATE(64, 4); }
  else return 2;
#undef GLLM_STATE
#undef GLLM_STATE_KD
  return 0;
}

}  // namespace

#define GLLM_BY_DTYPE(is_f32, CALL_BF16, CALL_F32) \
  do { if (is_f32) { CALL_F32; } else { CALL_BF16; } } while (0)
typedef __nv_bfloat16 bf16_t;

GLLM_EXPORT int gllm_seq_postnorm(void* x, const void* y, long ldy, const void* w, void* out, int ntok, int width,
                                  float alpha, float eps, int is_f32, void* stream) {
  if (ntok <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  GLLM_BY_DTYPE(is_f32,
                (postnorm_kernel<bf16_t><<<ntok, 256, 0, st>>>((float*)x, (const bf16_t*)y, ldy, (const bf16_t*)w,
                                                               (bf16_t*)out, width, alpha, eps)),
                (postnorm_kernel<float><<<ntok, 256, 0, st>>>((float*)x, (const float*)y, ldy, (const float*)w,
                                                              (float*)out, width, alpha, eps)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_qk_norm_rope_kv_write(const void* qkv, long ld, int ntok, int H, int G, int D, int Dv,
                                               const void* qn, const void* kn, float eps, const void* positions,
                                               int rot, double log2_base, void* q_out, void* kc, void* vc,
                                               const void* slots, int ps, int slab, int slab_v, int is_f32,
                                               const void* freqs, float mag, void* stream) {
  if (ntok <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(ntok);
  const size_t smem = (size_t)(rot > 0 ? rot : 2) * sizeof(float);
  GLLM_BY_DTYPE(is_f32,
                (qk_norm_rope_kv_write_kernel<bf16_t><<<grid, 256, smem, st>>>(
                    (const bf16_t*)qkv, ld, H, G, D, Dv, (const bf16_t*)qn, (const bf16_t*)kn, eps,
                    (const int*)positions, rot, log2_base, (bf16_t*)q_out, (bf16_t*)kc, (bf16_t*)vc,
                    (const int*)slots, ps, slab, slab_v, (const double*)freqs, mag)),
                (qk_norm_rope_kv_write_kernel<float><<<grid, 256, smem, st>>>(
                    (const float*)qkv, ld, H, G, D, Dv, (const float*)qn, (const float*)kn, eps,
                    (const int*)positions, rot, log2_base, (float*)q_out, (float*)kc, (float*)vc, (const int*)slots,
                    ps, slab, slab_v, (const double*)freqs, mag)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_linear_state(const void* q, long ldq, const void* k, long ldk, const void* v, long ldv,
                                      const void* beta, long ldb, const void* a, long lda, const void* neg_a,
                                      const void* dt_bias, const void* decay, void* state, const void* rec_slots,
                                      const void* seq_lens, const void* qsl, int nseq, int H, int G, int D, int V,
                                      int silu_in, int unit_qk, float q_scale, int delta, void* out, int is_f32,
                                      int parts, const void* gk, long ldgk, void* stream) {
  if (nseq <= 0) return 0;
  if (gk != nullptr && (delta || G != H)) return 2;                    // key-channel decay: plain update, own keys
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(nseq, H, (V + 31) / 32);
  // TCH rows of q and k (and the decay row) + TCH (g, beta)
  const size_t smem = (size_t)(8 * (gk != nullptr ? ((3 * D + 1) & ~1) : 2 * D) + 16) * sizeof(float);
  int rc;
  if (is_f32)
    rc = state_dispatch<float>(grid, smem, st, q, ldq, k, ldk, v, ldv, beta, ldb, a, lda, (const float*)neg_a,
                               (const float*)dt_bias, (const float*)decay, (float*)state, (const int*)rec_slots,
                               (const int*)seq_lens, (const int*)qsl, H, G, D, V, silu_in, unit_qk, q_scale, delta,
                               (float*)out, parts, (const float*)gk, ldgk);
  else
    rc = state_dispatch<bf16_t>(grid, smem, st, q, ldq, k, ldk, v, ldv, beta, ldb, a, lda, (const float*)neg_a,
                                (const float*)dt_bias, (const float*)decay, (float*)state, (const int*)rec_slots,
                                (const int*)seq_lens, (const int*)qsl, H, G, D, V, silu_in, unit_qk, q_scale, delta,
                                (float*)out, parts, (const float*)gk, ldgk);
  if (rc) return rc;
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_gated_group_norm(const void* o, int n, const void* gate, long ldg, const void* w, int wlen,
                                          int group, float eps, int act, float out_scale, void* out, long ldo,
                                          int ntok, int is_f32, void* stream) {
  if (ntok <= 0 || n <= 0) return 0;
  if (group <= 0 || n % group != 0) return 2;
  cudaStream_t st = (cudaStream_t)stream;
  const long warps = (long)ntok * (n / group);
  const unsigned blocks = (unsigned)((warps + 3) / 4);
  GLLM_BY_DTYPE(is_f32,
                (gated_group_norm_kernel<bf16_t><<<blocks, 128, 0, st>>>((const float*)o, n, (const bf16_t*)gate, ldg,
                                                                         (const bf16_t*)w, wlen, group, eps, act,
                                                                         out_scale, (bf16_t*)out, ldo, ntok)),
                (gated_group_norm_kernel<float><<<blocks, 128, 0, st>>>((const float*)o, n, (const float*)gate, ldg,
                                                                        (const float*)w, wlen, group, eps, act,
                                                                        out_scale, (float*)out, ldo, ntok)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_silu_mul(const void* gu, long ld, int ntok, int F, void* out, int is_f32, void* stream) {
  if (ntok <= 0 || F <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t total = (size_t)ntok * F;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  GLLM_BY_DTYPE(is_f32,
                (silu_mul_kernel<bf16_t><<<blocks, 256, 0, st>>>((const bf16_t*)gu, ld, F, (bf16_t*)out, total)),
                (silu_mul_kernel<float><<<blocks, 256, 0, st>>>((const float*)gu, ld, F, (float*)out, total)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_router_logits(const void* h, long ldh, const void* w, int ntok, int width, int E,
                                       void* logits, int is_f32, void* stream) {
  if (ntok <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(ntok, (E + 3) / 4);
  GLLM_BY_DTYPE(is_f32,
                (router_logits_kernel<bf16_t><<<grid, 128, 0, st>>>((const bf16_t*)h, ldh, (const bf16_t*)w, width, E,
                                                                    (float*)logits)),
                (router_logits_kernel<float><<<grid, 128, 0, st>>>((const float*)h, ldh, (const float*)w, width, E,
                                                                   (float*)logits)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_router_logits_mma(const void* h, long ldh, const void* w, int ntok, int width, int E,
                                           void* logits, void* stream) {
  if (ntok <= 0) return 0;
  if (width % 16 != 0 || ldh % 2 != 0) return 2;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((ntok + 63) / 64, (E + 63) / 64);
  router_logits_mma_kernel<8><<<grid, 128, 0, st>>>((const bf16_t*)h, ldh, (const bf16_t*)w, ntok, width, E,
                                                    (float*)logits);
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_gemm_mma_f32out(const void* A, long lda, long sa, const void* W, long ldw, long sw, void* C,
                                         long ldc, long sc, int M, int N, int K, int B, void* stream) {
  if (M <= 0 || N <= 0 || B <= 0) return 0;
  if (K % 32 != 0 || lda % 8 != 0 || ldw % 8 != 0 || sa % 8 != 0 || sw % 8 != 0 || ((uintptr_t)A & 15) != 0 ||
      ((uintptr_t)W & 15) != 0)
    return 2;
  cudaStream_t st = (cudaStream_t)stream;
  const bf16_t* a = (const bf16_t*)A;
  const bf16_t* w = (const bf16_t*)W;
  // the choice depends on the shape only, never on the number of rows: one summation order per (N, K)
  const bool split = N <= 32 && K % 128 == 0 && K >= 512;
  if (split && N <= 16) {
    dim3 grid((M + 15) / 16, 1, B);
    gemm_mma_f32out_kernel<2, true><<<grid, 128, 0, st>>>(a, lda, sa, w, ldw, sw, (float*)C, ldc, sc, M, N, K);
  } else if (split) {
    dim3 grid((M + 15) / 16, 1, B);
    gemm_mma_f32out_kernel<4, true><<<grid, 128, 0, st>>>(a, lda, sa, w, ldw, sw, (float*)C, ldc, sc, M, N, K);
  } else if (N <= 16) {
    dim3 grid((M + 63) / 64, 1, B);
    gemm_mma_f32out_kernel<2, false><<<grid, 128, 0, st>>>(a, lda, sa, w, ldw, sw, (float*)C, ldc, sc, M, N, K);
  } else if (N <= 32) {
    dim3 grid((M + 63) / 64, 1, B);
    gemm_mma_f32out_kernel<4, false><<<grid, 128, 0, st>>>(a, lda, sa, w, ldw, sw, (float*)C, ldc, sc, M, N, K);
  } else {
    dim3 grid((M + 63) / 64, (N + 63) / 64, B);
    gemm_mma_f32out_kernel<8, false><<<grid, 128, 0, st>>>(a, lda, sa, w, ldw, sw, (float*)C, ldc, sc, M, N, K);
  }
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_key_decay(const void* z, long ldz, const void* bias, float inv_tau, void* out, int ntok, int n,
                                   int is_f32, void* stream) {
  if (ntok <= 0 || n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t total = (size_t)ntok * n;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  GLLM_BY_DTYPE(is_f32,
                (key_decay_kernel<bf16_t><<<blocks, 256, 0, st>>>((const bf16_t*)z, ldz, (const float*)bias, inv_tau,
                                                                  (float*)out, n, total)),
                (key_decay_kernel<float><<<blocks, 256, 0, st>>>((const float*)z, ldz, (const float*)bias, inv_tau,
                                                                 (float*)out, n, total)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_router_select(const void* logits, int ntok, int E, int top_k, void* wout, void* ids,
                                       void* stream) {
  if (ntok <= 0) return 0;
  if (top_k > E || E > 1024) return 2;
  cudaStream_t st = (cudaStream_t)stream;
  router_select_kernel<<<(ntok + 3) / 4, 128, 0, st>>>((const float*)logits, ntok, E, top_k, (float*)wout, (int*)ids);
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_routed_experts(const void* h, long ldh, const void* w13, const void* w2, const void* ids,
                                        const void* wts, int ntok, int top_k, int width, int F, void* act, void* out,
                                        int is_f32, int n_real, float limit, float alpha, int ungated,
                                        void* stream) {
  if (ntok <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 g1(ntok * top_k, (F + 3) / 4), g2(ntok, (width + 3) / 4);
  if (is_f32) {
    moe_gate_up_kernel<float><<<g1, 128, 0, st>>>((const float*)h, ldh, (const float*)w13, (const int*)ids, top_k,
                                                  width, F, (float*)act, n_real, limit, alpha, ungated);
    moe_down_kernel<float><<<g2, 128, 0, st>>>((const float*)act, (const float*)w2, (const int*)ids,
                                               (const float*)wts, top_k, width, F, (float*)out, (const float*)h, ldh,
                                               n_real);
  } else {
    moe_gate_up_kernel<bf16_t><<<g1, 128, 0, st>>>((const bf16_t*)h, ldh, (const bf16_t*)w13, (const int*)ids, top_k,
                                                   width, F, (bf16_t*)act, n_real, limit, alpha, ungated);
    moe_down_kernel<bf16_t><<<g2, 128, 0, st>>>((const bf16_t*)act, (const bf16_t*)w2, (const int*)ids,
                                                (const float*)wts, top_k, width, F, (bf16_t*)out, (const bf16_t*)h, ldh,
                                                n_real);
  }
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_softcap(void* z, long ld, int ntok, int n, float cap, int is_f32, void* stream) {
  if (ntok <= 0 || n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t total = (size_t)ntok * n;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  GLLM_BY_DTYPE(is_f32, (softcap_kernel<bf16_t><<<blocks, 256, 0, st>>>((bf16_t*)z, ld, n, cap, total)),
                (softcap_kernel<float><<<blocks, 256, 0, st>>>((float*)z, ld, n, cap, total)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}
