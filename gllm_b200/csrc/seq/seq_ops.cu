// Kernels of the layer-list decoder (models/hybrid.py): fp32 residual stream with fused post-norm / residual add /
// pre-norm, per-head q/k RMS norm + paged cache write for key-valued attention, sliding-window paged attention
// with a softmax sink, causal depthwise convolution + SiLU with carried taps, the Mamba-1 selective scan with
// slot-indexed fp32 state, squared ReLU, and a plain tiled GEMM with fp32 accumulation for shapes / dtypes the
// tcgen05 GEMM does not take (true fp32 operands, rows that are not 16-byte aligned).
//
// Every kernel is templated on the compute dtype T (bf16 or float); norms, softmax, the recurrence, decays,
// softplus and the residual stream are fp32 in both. This file is compiled WITHOUT --use_fast_math (build.py):
// expf / log1pf / sqrtf / division are the IEEE-accurate versions.
//
// Batch layout (InputData): tokens of all sequences are concatenated; query_start_loc [B + 1] gives each sequence's
// rows, seq_lens [B] its length after this step, so a chunk starts at position seq_len - q_len.  Results of a row
// never depend on which other rows share the launch: every reduction has a fixed order.
#include <cuda_bf16.h>

#include "common/host_utils.h"
#include "seq/seq_common.cuh"

namespace {
using namespace seqk;

// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_scale_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                                   int width, int vocab, float scale) {
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* row = table + (size_t)id * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)t * width + i] = to_f(row[i]) * scale;
}

// x += rms(y) * w_post * post_scale ; x += add ; out = rms(x) * w_pre   (each part optional; post_scale: an fp32
// layer scale). With emit_plain and no w_pre, out = x rounded to T (sublayers that read the stream un-normed).
// w_off is added to both norm weights in fp32 (1 for weights stored around zero); out_mul multiplies the normed
// output (a logit scale applied to the final norm's result, before it is rounded).
template <typename T>
__global__ void __launch_bounds__(256) resid_norm_kernel(float* __restrict__ x, const T* __restrict__ y, long ldy,
                                                         const T* __restrict__ w_post,
                                                         const float* __restrict__ post_scale,
                                                         const float* __restrict__ add, const T* __restrict__ w_pre,
                                                         T* __restrict__ out, int width, float eps, int emit_plain,
                                                         float w_off, float out_mul) {
  __shared__ float scratch[8];
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * width;
  float r_post = 0.f;
  if (y != nullptr) {
    const T* yr = y + (size_t)t * ldy;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += 256) { float v = to_f(yr[i]); ss += v * v; }
    ss = block_sum<256>(ss, scratch);
    r_post = 1.0f / sqrtf(ss / (float)width + eps);
  }
  const bool plain = w_pre == nullptr && emit_plain && out != nullptr;
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < width; i += 256) {
    float v = xr[i];
    if (y != nullptr) {
      float br = to_f(y[(size_t)t * ldy + i]) * r_post * (to_f(w_post[i]) + w_off);
      if (post_scale != nullptr) br *= post_scale[i];
      v += br;
    }
    if (add != nullptr) v += add[(size_t)t * width + i];
    if (y != nullptr || add != nullptr) xr[i] = v;
    if (plain) out[(size_t)t * width + i] = from_f<T>(v);
    ss2 += v * v;
  }
  if (w_pre == nullptr) return;
  ss2 = block_sum<256>(ss2, scratch);
  const float r = 1.0f / sqrtf(ss2 / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += 256)
    out[(size_t)t * width + i] = from_f<T>(xr[i] * r * (to_f(w_pre[i]) + w_off) * out_mul);
}


// one warp per (token, head): heads [0, H) are queries, [H, H + G) keys
template <typename T>
__global__ void qk_norm_kv_write_kernel(const T* __restrict__ qk, long ldqk, int ntok, int H, int G, int D,
                                        const T* __restrict__ qn, const T* __restrict__ kn, float eps,
                                        T* __restrict__ q_out, T* __restrict__ kc, T* __restrict__ vc,
                                        const int* __restrict__ slots, int ps, int slab) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * 4 + warp, t = blockIdx.x;
  if (head >= H + G) return;
  const T* src = qk + (size_t)t * ldqk + (size_t)head * D;
  float ss = 0.f;
  for (int d = lane; d < D; d += 32) { float v = to_f(src[d]); ss += v * v; }
  ss = warp_sum(ss);
  const T* w = head < H ? qn : kn;
  const float r = w != nullptr ? 1.0f / sqrtf(ss / (float)D + eps) : 1.0f;
  if (head < H) {
    T* dst = q_out + (size_t)t * H * D + (size_t)head * D;
    for (int d = lane; d < D; d += 32) dst[d] = from_f<T>(to_f(src[d]) * r * (w != nullptr ? to_f(w[d]) : 1.0f));
  } else {
    const int slot = slots[t];
    if (slot < 0) return;
    const int g = head - H;
    for (int d = lane; d < D; d += 32) {
      const size_t idx = cache_index(slot, g, d, G, D, ps, slab);
      const float v = to_f(src[d]);
      kc[idx] = from_f<T>(v * r * (w != nullptr ? to_f(w[d]) : 1.0f));
      vc[idx] = src[d];
    }
  }
}

// Masked paged attention with a sink: sliding window and / or chunk mask (position i sees j <= i of its own
// chunk, floor(i / chunk) == floor(j / chunk)); keys of width D, values of width Dv (their caches have their own
// slab widths); the result is multiplied by out_scale and written with row stride ldo. One warp per (token, head);
// 4 consecutive tokens of one head per block (their key ranges overlap, so K/V rows are shared through L1).
// Scores: one key per lane; P.V: value entries across lanes. softcap > 0: a scaled score s becomes
// softcap * tanh(s / softcap) before the softmax.
template <typename T, int MAXR>
__global__ void __launch_bounds__(128) window_attn_kernel(
    const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc, const int* __restrict__ block_table,
    int bt_stride, const int* __restrict__ qsl, const int* __restrict__ positions, int ntok, int nseq, float scale,
    int H, int G, int D, int Dv, int window, int chunk, const float* __restrict__ sink, T* __restrict__ out, long ldo,
    float out_scale, int ps, int slab, int slab_v, float softcap) {
  __shared__ float qs[4][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp, h = blockIdx.y;
  if (t >= ntok) return;
  const int s = find_seq(qsl, nseq, t);
  const int i = positions[t];
  int lo = window > 0 ? max(0, i - window + 1) : 0;
  if (chunk > 0) lo = max(lo, (i / chunk) * chunk);
  const int g = h / (H / G);
  const T* qrow = q + (size_t)t * H * D + (size_t)h * D;
  for (int d = lane; d < D; d += 32) qs[warp][d] = to_f(qrow[d]);
  __syncwarp();
  const int* bt = block_table + (size_t)s * bt_stride;
  const int nslab = D / slab;
  const size_t page_stride = (size_t)G * D * ps, head_off = (size_t)g * D * ps;
  const size_t page_stride_v = (size_t)G * Dv * ps, head_off_v = (size_t)g * Dv * ps;
  float m = sink != nullptr ? sink[h] : -INFINITY;
  float l = sink != nullptr ? 1.0f : 0.0f;
  float acc[MAXR];
#pragma unroll
  for (int r = 0; r < MAXR; ++r) acc[r] = 0.f;
  for (int j0 = lo; j0 <= i; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j <= i;
    size_t base_v = 0;
    float sc = -INFINITY;
    if (valid) {
      const int page = bt[j / ps];
      const size_t base = (size_t)page * page_stride + head_off + (size_t)(j % ps) * slab;
      base_v = (size_t)page * page_stride_v + head_off_v + (size_t)(j % ps) * slab_v;
      float dot = 0.f;
      for (int c = 0; c < nslab; ++c) {
        const T* kr = kc + base + (size_t)c * ps * slab;
        const float* qq = qs[warp] + c * slab;
        for (int e = 0; e < slab; ++e) dot = fmaf(qq[e], to_f(kr[e]), dot);
      }
      sc = dot * scale;
      if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
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
      const unsigned long long bj = __shfl_sync(0xffffffffu, (unsigned long long)base_v, kk);
#pragma unroll
      for (int r = 0; r < MAXR; ++r) {
        const int d = lane + 32 * r;
        if (d < Dv) acc[r] = fmaf(pj, to_f(vc[bj + (size_t)(d / slab_v) * ps * slab_v + d % slab_v]), acc[r]);
      }
    }
  }
  T* orow = out + (size_t)t * ldo + (size_t)h * Dv;
  const float inv = out_scale / l;
#pragma unroll
  for (int r = 0; r < MAXR; ++r) {
    const int d = lane + 32 * r;
    if (d < Dv) orow[d] = from_f<T>(acc[r] * inv);
  }
}

// depthwise causal convolution + SiLU (act 0) or no activation (act 1); taps before the chunk come from the
// sequence's carried state. in_bias (optional) is added to every input at a position >= 0; inputs before the
// start of a sequence are zeros (the slot's rows for them are not read), and the carried state holds the inputs
// without the bias.
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ xz, long ldxz, int C, const float* __restrict__ w,
                                 const float* __restrict__ b, int taps, const T* __restrict__ state,
                                 const int* __restrict__ rec_slots, const int* __restrict__ seq_lens,
                                 const int* __restrict__ qsl, int nseq, T* __restrict__ out, int act,
                                 const float* __restrict__ in_bias) {
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s = find_seq(qsl, nseq, t);
  const int q0 = qsl[s], n = qsl[s + 1] - q0;
  const bool carried = state != nullptr && (seq_lens[s] - n) > 0;
  const T* st = carried ? state + (size_t)rec_slots[s] * (taps > 1 ? taps - 1 : 1) * C : nullptr;
  const int li = t - q0;
  const int pos0 = seq_lens[s] - n;                 // position of the chunk's first token
  const float ib = in_bias != nullptr ? in_bias[c] : 0.f;
  float acc = b[c];
  for (int j = 0; j < taps; ++j) {
    const int src = li - (taps - 1) + j;
    float v = 0.f;
    if (src >= 0) v = to_f(xz[(size_t)(q0 + src) * ldxz + c]);
    else if (carried) v = to_f(st[(size_t)(taps - 1 + src) * C + c]);
    v = pos0 + src >= 0 ? v + ib : 0.f;        // nothing precedes position 0, whatever the slot held
    acc = fmaf(w[(size_t)c * taps + j], v, acc);
  }
  out[(size_t)t * C + c] = from_f<T>(act == 0 ? acc / (1.0f + expf(-acc)) : acc);
}

// after the convolution: state <- the last taps - 1 inputs of the sequence (shifting in what the chunk brought)
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ xz, long ldxz, int C, int taps, T* __restrict__ state,
                                         const int* __restrict__ rec_slots, const int* __restrict__ seq_lens,
                                         const int* __restrict__ qsl) {
  const int s = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C || taps < 2) return;
  const int q0 = qsl[s], n = qsl[s + 1] - q0;
  if (n <= 0) return;
  const bool carried = (seq_lens[s] - n) > 0;
  T* st = state + (size_t)rec_slots[s] * (taps - 1) * C;
  for (int k = 0; k < taps - 1; ++k) {           // ascending k reads index k + n > k: never an overwritten entry
    const int src = n - (taps - 1) + k;
    T v = from_f<T>(0.f);
    if (src >= 0) v = xz[(size_t)(q0 + src) * ldxz + c];
    else if (carried) v = st[(size_t)(taps - 1 + src) * C + c];
    st[(size_t)k * C + c] = v;
  }
}

// Mamba-1 recurrence: one thread per channel holds its N states in registers and walks the sequence's tokens in
// chunks of TCH: the chunk's B and C rows (shared by all channels) are staged in shared memory by the whole block and
// the thread's own dt / x / z values are fetched up front, so the serial loop runs out of registers and smem.
template <typename T, int NMAX, int PARTS>
__global__ void __launch_bounds__(64) selective_scan_kernel(
    const T* __restrict__ xc, const T* __restrict__ dt_raw, const T* __restrict__ proj, long ldp,
    const T* __restrict__ xz, long ldxz, const float* __restrict__ A, const float* __restrict__ Dskip,
    const float* __restrict__ dt_bias, float* __restrict__ state, const int* __restrict__ rec_slots,
    const int* __restrict__ seq_lens, const int* __restrict__ qsl, int C, int N, int R, T* __restrict__ out) {
  constexpr int TCH = 8;
  __shared__ float sBC[TCH][2 * NMAX];
  const int s = blockIdx.x;
  // PARTS threads share a channel (state n = part + PARTS * j): more warps in flight when few sequences are long
  constexpr int NS = NMAX / PARTS;
  const int c0 = (blockIdx.y * 64 + threadIdx.x) / PARTS, part = threadIdx.x % PARTS;
  const int q0 = qsl[s], q1 = qsl[s + 1];
  if (q1 <= q0) return;                       // uniform over the block
  const bool active = c0 < C;
  const int c = active ? c0 : C - 1;          // idle threads mirror the last channel (loads only)
  const bool carried = state != nullptr && (seq_lens[s] - (q1 - q0)) > 0;
  float* st = state != nullptr ? state + (size_t)rec_slots[s] * N * C : nullptr;
  float S[NS], a[NS];
#pragma unroll
  for (int j = 0; j < NS; ++j) {
    const int n = part + PARTS * j;
    a[j] = n < N ? A[(size_t)c * N + n] : 0.f;
    S[j] = (carried && n < N) ? st[(size_t)n * C + c] : 0.f;
  }
  const float dsk = Dskip[c], bias = dt_bias[c];
  for (int t0 = q0; t0 < q1; t0 += TCH) {
    const int nt = min(TCH, q1 - t0);
    __syncthreads();                          // the previous chunk's rows are consumed
    for (int idx = threadIdx.x; idx < nt * 2 * N; idx += 64) {
      const int k = idx / (2 * N), n = idx - k * 2 * N;
      sBC[k][n] = to_f(proj[(size_t)(t0 + k) * ldp + R + n]);
    }
    float dtv[TCH], xv[TCH], zv[TCH];
#pragma unroll
    for (int k = 0; k < TCH; ++k) {
      if (k < nt) {
        dtv[k] = to_f(dt_raw[(size_t)(t0 + k) * C + c]);
        xv[k] = to_f(xc[(size_t)(t0 + k) * C + c]);
        zv[k] = to_f(xz[(size_t)(t0 + k) * ldxz + C + c]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TCH; ++k) {
      if (k < nt) {
        const float v = dtv[k] + bias;
        const float dt = v > 20.0f ? v : log1pf(expf(v));
        const float x = xv[k], z = zv[k];
        const float dx = dt * x;
        float y = 0.f;
#pragma unroll
        for (int j = 0; j < NS; ++j) {
          const int n = part + PARTS * j;
          if (n < N) {
            S[j] = expf(dt * a[j]) * S[j] + dx * sBC[k][n];
            y = fmaf(S[j], sBC[k][N + n], y);
          }
        }
#pragma unroll
        for (int o = 1; o < PARTS; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
        y = fmaf(dsk, x, y);
        if (active && part == 0) out[(size_t)(t0 + k) * C + c] = from_f<T>(y * (z / (1.0f + expf(-z))));
      }
    }
  }
  if (st != nullptr && active) {
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      const int n = part + PARTS * j;
      if (n < N) st[(size_t)n * C + c] = S[j];
    }
  }
}

template <typename T>
__global__ void relu2_kernel(const T* __restrict__ x, T* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    float v = fmaxf(to_f(x[i]), 0.f);
    out[i] = from_f<T>(v * v);
  }
}

// C[M, N] = A[M, K] . W[N, K]^T (+ bias[N], added to the fp32 sum), fp32 accumulation in ascending k for every element
template <typename T, typename TO = T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* __restrict__ A, long lda, const T* __restrict__ W,
                                                        long ldw, TO* __restrict__ Cm, long ldc, int M, int N, int K,
                                                        const T* __restrict__ bias = nullptr) {
  __shared__ float As[16][64 + 1], Ws[16][64 + 1];
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
      if (m < M && n < N) Cm[(size_t)m * ldc + n] = from_f<TO>(acc[i][j] + (bias != nullptr ? to_f(bias[n]) : 0.f));
    }
}

template <typename T, int PARTS>
int scan_dispatch(int nmax, dim3 grid, cudaStream_t st, const void* xc, const void* dt_raw, const void* proj, long ldp,
                  const void* xz, long ldxz, const float* A, const float* Dskip, const float* dt_bias, float* state,
                  const int* rec_slots, const int* seq_lens, const int* qsl, int C, int N, int R, void* out) {
#define GLLM_SCAN(NM)                                                                                             \
  selective_scan_kernel<T, NM, PARTS><<<grid, 64, 0, st>>>((const T*)xc, (const T*)dt_raw, (const T*)proj, ldp,          \
                                                    (const T*)xz, ldxz, A, Dskip, dt_bias, state, rec_slots,      \
                                                    seq_lens, qsl, C, N, R, (T*)out)
  if (nmax <= 8) GLLM_SCAN(8);
  else if (nmax <= 16) GLLM_SCAN(16);
  else if (nmax <= 32) GLLM_SCAN(32);
  else if (nmax <= 64) GLLM_SCAN(64);
  else if (nmax <= 128) GLLM_SCAN(128);
  else if (nmax <= 256) GLLM_SCAN(256);
  else return 2;
#undef GLLM_SCAN
  return 0;
}

template <typename T>
int attn_dispatch(dim3 grid, cudaStream_t st, const void* q, const void* kc, const void* vc, const int* bt,
                  int bt_stride, const int* qsl, const int* pos, int ntok, int nseq, float scale, int H, int G, int D,
                  int Dv, int window, int chunk, const float* sink, void* out, long ldo, float out_scale, int ps,
                  int slab, int slab_v, float softcap) {
#define GLLM_ATTN(R)                                                                                              \
  window_attn_kernel<T, R><<<grid, 128, 0, st>>>((const T*)q, (const T*)kc, (const T*)vc, bt, bt_stride, qsl, pos, \
                                                 ntok, nseq, scale, H, G, D, Dv, window, chunk, sink, (T*)out, ldo, \
                                                 out_scale, ps, slab, slab_v, softcap)
  if (D > 256) return 2;
  if (Dv <= 32) GLLM_ATTN(1);
  else if (Dv <= 64) GLLM_ATTN(2);
  else if (Dv <= 128) GLLM_ATTN(4);
  else if (Dv <= 256) GLLM_ATTN(8);
  else return 2;
#undef GLLM_ATTN
  return 0;
}

}  // namespace

#define GLLM_BY_DTYPE(is_f32, CALL_BF16, CALL_F32) \
  do { if (is_f32) { CALL_F32; } else { CALL_BF16; } } while (0)

GLLM_EXPORT int gllm_seq_embed_scale(const void* ids, const void* table, void* out, int ntok, int width, int vocab,
                                     float scale, int is_f32, void* stream) {
  if (ntok <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  GLLM_BY_DTYPE(is_f32,
                (embed_scale_kernel<__nv_bfloat16><<<ntok, 128, 0, st>>>((const int*)ids, (const __nv_bfloat16*)table,
                                                                        (float*)out, width, vocab, scale)),
                (embed_scale_kernel<float><<<ntok, 128, 0, st>>>((const int*)ids, (const float*)table, (float*)out,
                                                                 width, vocab, scale)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_resid_norm(void* x, const void* y, long ldy, const void* w_post, const void* post_scale,
                                    const void* add, const void* w_pre, void* out, int ntok, int width, float eps,
                                    int emit_plain, int is_f32, float w_off, float out_mul, void* stream) {
  if (ntok <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  GLLM_BY_DTYPE(is_f32,
                (resid_norm_kernel<__nv_bfloat16><<<ntok, 256, 0, st>>>(
                    (float*)x, (const __nv_bfloat16*)y, ldy, (const __nv_bfloat16*)w_post, (const float*)post_scale,
                    (const float*)add, (const __nv_bfloat16*)w_pre, (__nv_bfloat16*)out, width, eps, emit_plain,
                    w_off, out_mul)),
                (resid_norm_kernel<float><<<ntok, 256, 0, st>>>((float*)x, (const float*)y, ldy, (const float*)w_post,
                                                                (const float*)post_scale, (const float*)add,
                                                                (const float*)w_pre, (float*)out, width, eps,
                                                                emit_plain, w_off, out_mul)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_qk_norm_kv_write(const void* qk, long ldqk, int ntok, int H, int G, int D, const void* qn,
                                          const void* kn, float eps, void* q_out, void* kc, void* vc,
                                          const void* slots, int ps, int slab, int is_f32, void* stream) {
  if (ntok <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(ntok, (H + G + 3) / 4);
  GLLM_BY_DTYPE(is_f32,
                (qk_norm_kv_write_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(
                    (const __nv_bfloat16*)qk, ldqk, ntok, H, G, D, (const __nv_bfloat16*)qn, (const __nv_bfloat16*)kn,
                    eps, (__nv_bfloat16*)q_out, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, (const int*)slots, ps, slab)),
                (qk_norm_kv_write_kernel<float><<<grid, 128, 0, st>>>(
                    (const float*)qk, ldqk, ntok, H, G, D, (const float*)qn, (const float*)kn, eps, (float*)q_out,
                    (float*)kc, (float*)vc, (const int*)slots, ps, slab)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_window_attention(const void* q, const void* kc, const void* vc, const void* block_table,
                                          int bt_stride, const void* qsl, const void* positions, int ntok, int nseq,
                                          float scale, int H, int G, int D, int Dv, int window, int chunk,
                                          const void* sink, void* out, long ldo, float out_scale, int ps, int slab,
                                          int slab_v, int is_f32, float softcap, void* stream) {
  if (ntok <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((ntok + 3) / 4, H);
  int rc;
  if (is_f32)
    rc = attn_dispatch<float>(grid, st, q, kc, vc, (const int*)block_table, bt_stride, (const int*)qsl,
                              (const int*)positions, ntok, nseq, scale, H, G, D, Dv, window, chunk, (const float*)sink,
                              out, ldo, out_scale, ps, slab, slab_v, softcap);
  else
    rc = attn_dispatch<__nv_bfloat16>(grid, st, q, kc, vc, (const int*)block_table, bt_stride, (const int*)qsl,
                                      (const int*)positions, ntok, nseq, scale, H, G, D, Dv, window, chunk,
                                      (const float*)sink, out, ldo, out_scale, ps, slab, slab_v, softcap);
  if (rc) return rc;
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_conv_silu(const void* xz, long ldxz, int ntok, int nseq, int C, const void* w, const void* b,
                                   int taps, void* state, const void* rec_slots, const void* seq_lens, const void* qsl,
                                   void* out, int is_f32, int act, const void* in_bias, void* stream) {
  if (ntok <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(ntok, (C + 127) / 128), sgrid(nseq, (C + 127) / 128);
  if (is_f32) {
    conv_silu_kernel<float><<<grid, 128, 0, st>>>((const float*)xz, ldxz, C, (const float*)w, (const float*)b, taps,
                                                  (const float*)state, (const int*)rec_slots, (const int*)seq_lens,
                                                  (const int*)qsl, nseq, (float*)out, act, (const float*)in_bias);
    if (state != nullptr && taps > 1)
      conv_state_update_kernel<float><<<sgrid, 128, 0, st>>>((const float*)xz, ldxz, C, taps, (float*)state,
                                                             (const int*)rec_slots, (const int*)seq_lens,
                                                             (const int*)qsl);
  } else {
    conv_silu_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(
        (const __nv_bfloat16*)xz, ldxz, C, (const float*)w, (const float*)b, taps, (const __nv_bfloat16*)state,
        (const int*)rec_slots, (const int*)seq_lens, (const int*)qsl, nseq, (__nv_bfloat16*)out, act,
        (const float*)in_bias);
    if (state != nullptr && taps > 1)
      conv_state_update_kernel<__nv_bfloat16><<<sgrid, 128, 0, st>>>(
          (const __nv_bfloat16*)xz, ldxz, C, taps, (__nv_bfloat16*)state, (const int*)rec_slots, (const int*)seq_lens,
          (const int*)qsl);
  }
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_selective_scan(const void* xc, const void* dt_raw, const void* proj, long ldp, const void* xz,
                                        long ldxz, const void* A, const void* Dskip, const void* dt_bias, void* state,
                                        const void* rec_slots, const void* seq_lens, const void* qsl, int nseq, int C,
                                        int N, int R, void* out, int is_f32, int parts, void* stream) {
  if (nseq <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  if (parts == 4 && N >= 8) {       // few long sequences: 4 threads per channel
    dim3 grid4(nseq, (C + 15) / 16);
    if (is_f32)
      rc = scan_dispatch<float, 4>(N, grid4, st, xc, dt_raw, proj, ldp, xz, ldxz, (const float*)A,
                                   (const float*)Dskip, (const float*)dt_bias, (float*)state, (const int*)rec_slots,
                                   (const int*)seq_lens, (const int*)qsl, C, N, R, out);
    else
      rc = scan_dispatch<__nv_bfloat16, 4>(N, grid4, st, xc, dt_raw, proj, ldp, xz, ldxz, (const float*)A,
                                           (const float*)Dskip, (const float*)dt_bias, (float*)state,
                                           (const int*)rec_slots, (const int*)seq_lens, (const int*)qsl, C, N, R, out);
    if (rc) return rc;
    CUDA_CHECK_RET(cudaGetLastError());
    return 0;
  }
  dim3 grid(nseq, (C + 63) / 64);
  if (is_f32)
    rc = scan_dispatch<float, 1>(N, grid, st, xc, dt_raw, proj, ldp, xz, ldxz, (const float*)A, (const float*)Dskip,
                              (const float*)dt_bias, (float*)state, (const int*)rec_slots, (const int*)seq_lens,
                              (const int*)qsl, C, N, R, out);
  else
    rc = scan_dispatch<__nv_bfloat16, 1>(N, grid, st, xc, dt_raw, proj, ldp, xz, ldxz, (const float*)A,
                                      (const float*)Dskip, (const float*)dt_bias, (float*)state,
                                      (const int*)rec_slots, (const int*)seq_lens, (const int*)qsl, C, N, R, out);
  if (rc) return rc;
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_relu2(const void* x, void* out, long n, int is_f32, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  GLLM_BY_DTYPE(is_f32,
                (relu2_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out,
                                                                    (size_t)n)),
                (relu2_kernel<float><<<blocks, 256, 0, st>>>((const float*)x, (float*)out, (size_t)n)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

GLLM_EXPORT int gllm_seq_gemm_simt(const void* a, long lda, const void* w, long ldw, void* c, long ldc, int M, int N,
                                   int K, int is_f32, const void* bias, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  GLLM_BY_DTYPE(is_f32,
                (gemm_simt_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a, lda,
                                                                      (const __nv_bfloat16*)w, ldw,
                                                                      (__nv_bfloat16*)c, ldc, M, N, K,
                                                                      (const __nv_bfloat16*)bias)),
                (gemm_simt_kernel<float><<<grid, 256, 0, st>>>((const float*)a, lda, (const float*)w, ldw, (float*)c,
                                                               ldc, M, N, K, (const float*)bias)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}

// the same product with the result kept in fp32 whatever the operand dtype (router logits)
GLLM_EXPORT int gllm_seq_gemm_simt_f32out(const void* a, long lda, const void* w, long ldw, void* c, long ldc, int M,
                                          int N, int K, int is_f32, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  GLLM_BY_DTYPE(is_f32,
                (gemm_simt_kernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a, lda,
                                                                             (const __nv_bfloat16*)w, ldw, (float*)c,
                                                                             ldc, M, N, K)),
                (gemm_simt_kernel<float, float><<<grid, 256, 0, st>>>((const float*)a, lda, (const float*)w, ldw,
                                                                      (float*)c, ldc, M, N, K)));
  CUDA_CHECK_RET(cudaGetLastError());
  return 0;
}
