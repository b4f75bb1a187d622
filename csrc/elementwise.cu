// Memory-bound kernels of the TaH layer stack: RMSNorm, per-head QK-norm + RoPE + KV-cache write,
// embedding gather, rank-r LoRA-A products for the few "hard" rows of a decode tick, SwiGLU,
// and the logit post-processing of a tick (cumulative logits, argmax).
//
// Rounding follows what a bf16 PyTorch module stack produces (norm output rounded before the
// weight multiply, RoPE products rounded before the add), so that greedy token streams agree
// with an eager bf16 run of the same model.
#include <cstdlib>

#include "common.cuh"

namespace tahb {

// ---------------------------------------------------------------------------------------------
// RMSNorm: y = w * bf16(x * rsqrt(mean(x^2) + eps)).  One CTA (128 threads) per row, row kept in
// registers (H <= 128 * 8 * VPT elements).
// ---------------------------------------------------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(128) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x,
                                                      const __nv_bfloat16* __restrict__ w,
                                                      __nv_bfloat16* __restrict__ y, int H, long long ldx,
                                                      long long ldy, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int nvec = H / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
  uint4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * 128;
    if (idx < nvec) {
      v[i] = xr[idx];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  __shared__ float red[4];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float tot = red[0] + red[1] + red[2] + red[3];
  const float rstd = rsqrtf(tot / (float)H + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * ldy);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * 128;
    if (idx < nvec) {
      uint4 wv = wr[idx];
      uint4 o;
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
      const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        float2 g = __bfloat1622float2(wh[j]);
        oh[j] = __floats2bfloat162_rn(g.x * bf16_round(f.x * rstd), g.y * bf16_round(f.y * rstd));
      }
      yr[idx] = o;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm fused with the LoRA-A product of the rows that are at depth >= 1 (decode tick):
//   y[r] = w * bf16(x[r] * rstd)                     for every row
//   T[r] = gate[r] ? y[r] A^T : 0                    (A: [R, H], T: [M, ldt])
// One-dimensional grid of M + NORM_LORA_SLOTS * NORM_LORA_SLICES CTAs of 256 threads.  CTA b < M normalises
// row b, stores y and, when the row is gated off, clears T[b].  The others exist for the LoRA-A product:
// CTA (slot, slice) finds the slot-th gated row (then the (slot + SLOTS)-th, ...) by counting the gate vector
// (M <= 1024), normalises that row again into shared memory and its eight warps compute outputs
// slice * 8 + warp, + 8 * SLICES, ... with all loads of a dot product issued before the arithmetic.  The body
// is kept small on purpose: a tick runs it once per CTA between other kernels, from a cold instruction cache.
// Same summation order per output as lora_a_rows_kernel.
// ---------------------------------------------------------------------------------------------
constexpr int NORM_LORA_SLICES = 8;
constexpr int NORM_LORA_SLOTS = 32;

__global__ void __launch_bounds__(256) rmsnorm_lora_kernel(const __nv_bfloat16* __restrict__ x,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ y, int M, int H, long long ldx,
                                                           long long ldy, float eps, const int* __restrict__ gate,
                                                           const __nv_bfloat16* __restrict__ A,
                                                           __nv_bfloat16* __restrict__ T, int R, long long ldt) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ uint4 srow[];            // H / 8 vectors: the normalised row (LoRA CTAs only)
  __shared__ float red[8];
  __shared__ int s_cnt[8];
  __shared__ int s_row;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool norm_cta = (int)blockIdx.x < M;
  const int lid = (int)blockIdx.x - M;
  const int slice = lid % NORM_LORA_SLICES;
  int want = lid / NORM_LORA_SLICES;         // index of this CTA's gated row among the gated rows
  const int nvec = H / 8;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (;;) {
    int row;
    if (norm_cta) {
      row = blockIdx.x;
    } else {
      // thread t looks at rows 4t .. 4t + 3; the want-th set gate picks the row
      int g[4], cnt = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = tid * 4 + i;
        g[i] = (r < M && gate[r] != 0) ? 1 : 0;
        cnt += g[i];
      }
      int incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (tid == 0) s_row = -1;
      if (lane == 31) s_cnt[warp] = incl;
      __syncthreads();
      int base = 0;
      for (int k = 0; k < warp; ++k) base += s_cnt[k];
      int before = base + incl - cnt;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (g[i] && before == want) s_row = tid * 4 + i;
        before += g[i];
      }
      __syncthreads();
      row = s_row;
      if (row < 0) return;
    }
    // ---- normalise the row -------------------------------------------------------------
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
    constexpr int VPT = 4;                   // H <= 256 * 8 * 4 = 8192
    uint4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = tid + i * 256;
      if (idx < nvec) {
        v[i] = xr[idx];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(h[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += red[k];   // fixed order: every CTA of a row gets the same rstd
    const float rstd = rsqrtf(tot / (float)H + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * ldy);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = tid + i * 256;
      if (idx < nvec) {
        uint4 wv = wr[idx];
        uint4 o;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
        const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(h[j]);
          float2 g = __bfloat1622float2(wh[j]);
          oh[j] = __floats2bfloat162_rn(g.x * bf16_round(f.x * rstd), g.y * bf16_round(f.y * rstd));
        }
        if (norm_cta) yr[idx] = o;
        else srow[idx] = o;
      }
    }
    __nv_bfloat16* out = T + (size_t)row * ldt;
    if (norm_cta) {
      if (gate == nullptr || gate[row] == 0)
        for (int j = tid; j < R; j += 256) out[j] = __float2bfloat16_rn(0.f);
      return;
    }
    __syncthreads();
    // ---- LoRA-A outputs of this slice: one per warp and step ---------------------------
    for (int j = slice * 8 + warp; j < R; j += 8 * NORM_LORA_SLICES) {
      const uint4* a0 = reinterpret_cast<const uint4*>(A + (size_t)j * H);
      float acc = 0.f;
      for (int i0 = lane; i0 < nvec; i0 += 256) {
        uint4 av[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {          // eight independent 16-byte loads before any arithmetic
          const int i = i0 + u * 32;
          av[u] = i < nvec ? a0[i] : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * 32;
          if (i < nvec) {
            const uint4 xv = srow[i];
            const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
            const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&av[u]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 a = __bfloat1622float2(xh[q]);
              const float2 b = __bfloat1622float2(ah[q]);
              acc += a.x * b.x + a.y * b.y;
            }
          }
        }
      }
      acc = warp_sum(acc);
      if (lane == 0) out[j] = __float2bfloat16_rn(acc);
    }
    want += NORM_LORA_SLOTS;                 // more gated rows than slots: take the next one
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// Per-head QK RMSNorm + rotate-half RoPE + KV write.  One warp per (token, head).
//   qkv      [M, (nq + 2 nkv) * HD]
//   q_out    [M, nq * HD]
//   k_dense / v_dense (optional) [M, nkv * HD] : packed K/V of this pass (prefill / training)
//   cache (optional): paged cache of ONE layer; entry (page, kv, head, off) at
//        ((page * 2 + kv) * nkv + head) * page_size + off) * HD ; slot[t] = page * page_size + off,
//        negative slot = do not write.  With n_caches > 1, cache_sel[t] picks the depth cache.
// ---------------------------------------------------------------------------------------------
struct QkvRopeParams {
  const __nv_bfloat16* qkv;
  const __nv_bfloat16* q_w;
  const __nv_bfloat16* k_w;
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_dense;
  __nv_bfloat16* v_dense;
  __nv_bfloat16* cache[4];
  const int* cache_sel;
  const int* slot;
  const int* pos;
  int M, nq, nkv, page_size;
  long long ld_qkv;
  float eps, log2_theta;
};

template <int HD>
__global__ void __launch_bounds__(128) qk_norm_rope_kv_kernel(const QkvRopeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int EPL = HD / 32;  // elements per lane
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = p.nq + 2 * p.nkv;
  if (warp_global >= p.M * heads) return;
  const int t = warp_global / heads;
  const int h = warp_global % heads;
  const __nv_bfloat16* src = p.qkv + (size_t)t * p.ld_qkv + (size_t)h * HD + lane * EPL;
  float x[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) x[i] = __bfloat162float(src[i]);
  const bool is_q = h < p.nq;
  const bool is_k = !is_q && h < p.nq + p.nkv;
  float y[EPL];
  if (is_q || is_k) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)HD + p.eps);
    const __nv_bfloat16* w = (is_q ? p.q_w : p.k_w) + lane * EPL;
    float n[EPL], partner[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) n[i] = bf16_round(__bfloat162float(w[i]) * bf16_round(x[i] * rstd));
#pragma unroll
    for (int i = 0; i < EPL; ++i) partner[i] = __shfl_xor_sync(0xffffffffu, n[i], 16);
    const float posf = (float)p.pos[t];
    const bool upper = lane >= 16;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int d = lane * EPL + i;
      const int j = upper ? d - HD / 2 : d;                    // frequency index
      const float inv = exp2f(-(2.0f * (float)j / (float)HD) * p.log2_theta);
      const float ang = posf * inv;
      const float c = bf16_round(cosf(ang)), s = bf16_round(sinf(ang));
      const float rot = upper ? partner[i] : -partner[i];
      y[i] = bf16_round(bf16_round(n[i] * c) + bf16_round(rot * s));
    }
  } else {
#pragma unroll
    for (int i = 0; i < EPL; ++i) y[i] = x[i];
  }
  __nv_bfloat16 o[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) o[i] = __float2bfloat16_rn(y[i]);
  if (is_q) {
    __nv_bfloat16* dst = p.q_out + ((size_t)t * p.nq + h) * HD + lane * EPL;
#pragma unroll
    for (int i = 0; i < EPL; ++i) dst[i] = o[i];
    return;
  }
  const int kvh = is_k ? h - p.nq : h - p.nq - p.nkv;
  const int which = is_k ? 0 : 1;
  __nv_bfloat16* dense = is_k ? p.k_dense : p.v_dense;
  if (dense != nullptr) {
    __nv_bfloat16* dst = dense + ((size_t)t * p.nkv + kvh) * HD + lane * EPL;
#pragma unroll
    for (int i = 0; i < EPL; ++i) dst[i] = o[i];
  }
  if (p.slot != nullptr) {
    const int sl = p.slot[t];
    if (sl >= 0) {
      const int sel = p.cache_sel ? p.cache_sel[t] : 0;
      __nv_bfloat16* cache = p.cache[sel];
      const int page = sl / p.page_size, off = sl % p.page_size;
      __nv_bfloat16* dst =
          cache + ((((size_t)page * 2 + which) * p.nkv + kvh) * p.page_size + off) * HD + lane * EPL;
#pragma unroll
      for (int i = 0; i < EPL; ++i) dst[i] = o[i];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// RoPE table of a pass: cs[t, 0 .. HD/2) = bf16(cos(pos[t] * theta^(-2j/HD))), cs[t, HD/2 .. HD) = bf16(sin(..)).
// The positions of a pass are the same for every layer, so the transcendental work is done once per pass
// (once per decode tick) and the fused QKV epilogue of each layer only loads the row.
// ---------------------------------------------------------------------------------------------
__global__ void rope_table_kernel(const int* __restrict__ pos, __nv_bfloat16* __restrict__ cs, int M, int HD,
                                  float log2_theta) {
  const int half = HD / 2;
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= (long long)M * half) return;
  const int t = (int)(i / half), j = (int)(i % half);
  const float inv = exp2f(-(2.0f * (float)j / (float)HD) * log2_theta);
  const float ang = (float)pos[t] * inv;
  cs[(size_t)t * HD + j] = __float2bfloat16_rn(cosf(ang));
  cs[(size_t)t * HD + half + j] = __float2bfloat16_rn(sinf(ang));
}

// ---------------------------------------------------------------------------------------------
// LayerNorm over the last dimension (bf16 in / out, fp32 statistics): y = (x - mean) * rstd * w + b.
// One warp per row (D <= 4096, D % 8 == 0); with `dot_w` the normalised row is not stored but reduced
// against dot_w (+ dot_b) into z[r] (fp32): the output layer LayerNorm -> Linear(D, 1) of the decider.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) layernorm_kernel(const __nv_bfloat16* __restrict__ x,
                                                        const __nv_bfloat16* __restrict__ w,
                                                        const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                        const __nv_bfloat16* __restrict__ dot_w,
                                                        const __nv_bfloat16* __restrict__ dot_b, float* __restrict__ z,
                                                        int M, int D, long long ldx, long long ldy, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= M) return;
  const int nvec = D / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)r * ldx);
  constexpr int VPT = 16;                      // D <= 32 * 8 * 16 = 4096
  uint4 v[VPT];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = lane + i * 32;
    if (idx < nvec) {
      v[i] = xr[idx];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); sum += f.x + f.y; }
    }
  }
  const float mean = warp_sum(sum) / (float)D;
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = lane + i * 32;
    if (idx < nvec) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        var += (f.x - mean) * (f.x - mean) + (f.y - mean) * (f.y - mean);
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(var) / (float)D + eps);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = lane + i * 32;
    if (idx < nvec) {
      const uint4 wv = reinterpret_cast<const uint4*>(w)[idx];
      const uint4 bv = reinterpret_cast<const uint4*>(b)[idx];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
      const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
      const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bv);
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]), g = __bfloat1622float2(wh[j]), c = __bfloat1622float2(bh[j]);
        oh[j] = __floats2bfloat162_rn((f.x - mean) * rstd * g.x + c.x, (f.y - mean) * rstd * g.y + c.y);
      }
      if (dot_w == nullptr) {
        reinterpret_cast<uint4*>(y + (size_t)r * ldy)[idx] = o;
      } else {
        const uint4 dv = reinterpret_cast<const uint4*>(dot_w)[idx];
        const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 yn = __bfloat1622float2(oh[j]), d = __bfloat1622float2(dh[j]);
          acc += yn.x * d.x + yn.y * d.y;
        }
      }
    }
  }
  if (dot_w != nullptr) {
    acc = warp_sum(acc);
    if (lane == 0) z[r] = bf16_round(acc + (dot_b != nullptr ? __bfloat162float(dot_b[0]) : 0.f));
  }
}

// ---------------------------------------------------------------------------------------------
// Embedding gather: out[r] = E[tok[r]]  (tok < 0 -> zeros)
// ---------------------------------------------------------------------------------------------
__global__ void embed_gather_kernel(const __nv_bfloat16* __restrict__ E, const int* __restrict__ tok,
                                    __nv_bfloat16* __restrict__ out, int H, long long ld_out) {
  const int r = blockIdx.x;
  const int id = tok[r];
  const uint4* src = reinterpret_cast<const uint4*>(E + (size_t)(id < 0 ? 0 : id) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * ld_out);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = id < 0 ? make_uint4(0, 0, 0, 0) : src[i];
}

// ---------------------------------------------------------------------------------------------
// LoRA-A on gated rows:  T[r, :] = gate[r] ? x[r, :] A^T : 0        (A: [R, K], T: [M, ldt])
// Rows whose gate is 0 only clear their output.  Meant for decode ticks where a handful of rows
// are at depth >= 1; dense passes use the tensor-core GEMM instead.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) lora_a_rows_dense_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ A,
                                                          __nv_bfloat16* __restrict__ T, const int* __restrict__ gate,
                                                          int K, int R, long long ldx, long long ldt,
                                                          const uint32_t* wait_flag, const uint32_t* wait_target,
                                                          int wait_world, int* status, unsigned long long wait_limit) {
  // grid (rows, ceil(R / 8)): a CTA owns 8 outputs of one row, one per warp, so that a gated row's
  // product is spread over R / 8 CTAs instead of running serially in one
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.y * 8 + warp;
  if (j >= R) return;
  __nv_bfloat16* out = T + (size_t)r * ldt;
  if (gate != nullptr && gate[r] == 0) {
    if (lane == 0) out[j] = __float2bfloat16_rn(0.f);
    return;
  }
  if (wait_world > 0) {     // tensor parallel: x rows are broadcast by their owners (see comm.cu)
    if (lane == 0) wait_peer_rows(wait_flag, wait_target, wait_world, status, wait_limit);
    __syncwarp();
  }
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)r * ldx);
  const uint4* ar = reinterpret_cast<const uint4*>(A + (size_t)j * K);
  float acc = 0.f;
  for (int i = lane; i < K / 8; i += 32) {
    uint4 xv = xr[i], av = ar[i];
    const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 a = __bfloat1622float2(xh[q]), b = __bfloat1622float2(ah[q]);
      acc += a.x * b.x + a.y * b.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) out[j] = __float2bfloat16_rn(acc);
}

// Decode-tick form (gate given, M <= 1024): only a handful of rows are gated on, so the grid is
// (LORA_SLOTS, ceil(R / 8)) instead of one CTA per (row, 8 outputs).  Every CTA compacts the gate
// vector into a list of gated rows in shared memory; CTA x handles list entries x, x + LORA_SLOTS,
// ... for its 8 outputs (one per warp); the x == 0 CTAs also clear their 8 columns of the rows that
// are gated off.
constexpr int LORA_SLOTS = 32;
__global__ void __launch_bounds__(256) lora_a_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ A,
                                                          __nv_bfloat16* __restrict__ T, const int* __restrict__ gate,
                                                          int M, int K, int R, long long ldx, long long ldt,
                                                          const uint32_t* wait_flag, const uint32_t* wait_target,
                                                          int wait_world, int* status, unsigned long long wait_limit) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_rows[1024];
  __shared__ int s_warp[8];
  __shared__ int s_n;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int jb = blockIdx.y;
  // compact the gated rows: thread t looks at rows 4t .. 4t+3
  int g[4], cnt = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = tid * 4 + i;
    g[i] = (r < M && gate[r] != 0) ? 1 : 0;
    cnt += g[i];
  }
  int incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int base = 0;
  for (int w = 0; w < warp; ++w) base += s_warp[w];
  int pos = base + incl - cnt;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (g[i]) s_rows[pos++] = tid * 4 + i;
  if (tid == 255) s_n = base + incl;
  __syncthreads();
  const int n = s_n;
  if (blockIdx.x == 0) {      // clear this CTA's 8 columns of the rows that are gated off
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = tid * 4 + i;
      if (r < M && !g[i]) {
        __nv_bfloat16* o = T + (size_t)r * ldt + jb * 8;
        if (jb * 8 + 8 <= R && (ldt % 8) == 0) *reinterpret_cast<uint4*>(o) = make_uint4(0, 0, 0, 0);
        else for (int c = 0; c < 8 && jb * 8 + c < R; ++c) o[c] = __float2bfloat16_rn(0.f);
      }
    }
  }
  if ((int)blockIdx.x >= n) return;
  if (wait_world > 0) {       // tensor parallel: x rows are broadcast by their owners (see comm.cu)
    if (tid == 0) wait_peer_rows(wait_flag, wait_target, wait_world, status, wait_limit);
    __syncthreads();
  }
  const int j = jb * 8 + warp;
  if (j >= R) return;
  const uint4* ar = reinterpret_cast<const uint4*>(A + (size_t)j * K);
  const int nvec = K / 8;
  for (int k = blockIdx.x; k < n; k += gridDim.x) {
    const int r = s_rows[k];
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)r * ldx);
    float acc = 0.f;
    // the product is latency-bound (one warp, operands in L2): issue the 16 loads of eight steps before
    // their arithmetic; the summation order is that of the plain loop
    for (int i0 = lane; i0 < nvec; i0 += 256) {
      uint4 xv[8], av[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * 32;
        if (i < nvec) { xv[u] = xr[i]; av[u] = ar[i]; }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (i0 + u * 32 < nvec) {
          const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv[u]);
          const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&av[u]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float2 a = __bfloat1622float2(xh[q]), b = __bfloat1622float2(ah[q]);
            acc += a.x * b.x + a.y * b.y;
          }
        }
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) T[(size_t)r * ldt + j] = __float2bfloat16_rn(acc);
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU on a materialised [M, 2I] gate|up tensor (used where the GEMM epilogue fusion is off).
// ---------------------------------------------------------------------------------------------
// Vector form: 8 columns (16 bytes of gate, 16 of up) per thread; needs I, the row pitches and the bases aligned to 8.
__global__ void swiglu_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int M, int I,
                                  long long ld_in, long long ld_out) {
  const int vpr = I / 8;
  const long long n = (long long)M * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vpr), c = (int)(i % vpr) * 8;
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + (size_t)r * ld_in + c);
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + (size_t)r * ld_in + I + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
      o2[j] = __floats2bfloat162_rn(bf16_round(silu(g.x)) * u.x, bf16_round(silu(g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)r * ld_out + c) = ov;
  }
}

__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int M, int I,
                              long long ld_in, long long ld_out) {
  const long long n = (long long)M * I;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / I), c = (int)(i % I);
    const float g = __bfloat162float(gu[(size_t)r * ld_in + c]);
    const float u = __bfloat162float(gu[(size_t)r * ld_in + I + c]);
    out[(size_t)r * ld_out + c] = __float2bfloat16_rn(bf16_round(silu(g)) * u);
  }
}

// ---------------------------------------------------------------------------------------------
// Tick logit post-processing.  Per row r:
//   cum[r] = depth[r] > 0 ? cum[r] + logits[r] : logits[r]      (bf16 add, like the model's
//   additive logit update), and argmax over cum[r] -> best[r] (lowest index wins ties).
// One CTA of 1024 threads per row.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) logits_post_kernel(const __nv_bfloat16* __restrict__ logits,
                                                           __nv_bfloat16* __restrict__ cum,
                                                           const int* __restrict__ depth, int* __restrict__ best,
                                                           float* __restrict__ best_val, int V,
                                                           long long ld_logits, long long ld_cum) {
  const int r = blockIdx.x;
  const bool add = depth != nullptr && depth[r] > 0;
  const __nv_bfloat16* lr = logits + (size_t)r * ld_logits;
  __nv_bfloat16* cr = cum + (size_t)r * ld_cum;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  const int nvec = V / 8;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 lv = reinterpret_cast<const uint4*>(lr)[i];
    __nv_bfloat16* le = reinterpret_cast<__nv_bfloat16*>(&lv);
    if (add) {
      uint4 cv = reinterpret_cast<const uint4*>(cr)[i];
      const __nv_bfloat16* ce = reinterpret_cast<const __nv_bfloat16*>(&cv);
#pragma unroll
      for (int j = 0; j < 8; ++j) le[j] = __float2bfloat16_rn(__bfloat162float(ce[j]) + __bfloat162float(le[j]));
    }
    reinterpret_cast<uint4*>(cr)[i] = lv;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float v = __bfloat162float(le[j]);
      if (v > bv) { bv = v; bi = i * 8 + j; }
    }
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
    float v = __bfloat162float(lr[i]);
    if (add) v = bf16_round(__bfloat162float(cr[i]) + v);
    cr[i] = __float2bfloat16_rn(v);
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  // block argmax (value desc, index asc)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = sv[lane];
    bi = si[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      best[r] = bi;
      if (best_val != nullptr) best_val[r] = bv;   // lets a vocabulary-parallel caller merge shards
    }
  }
}

static unsigned long long g_peer_wait_limit_ns = WAIT_TIMEOUT_NS;
unsigned long long peer_wait_limit_ns() { return g_peer_wait_limit_ns; }

int pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* v = getenv("TAH_B200_PDL");
    on = (v != nullptr && v[0] == '0') ? 0 : 1;
  }
  return on;
}

}  // namespace tahb

using namespace tahb;

// Sets how long a kernel waits for a flag that a peer GPU advances before it records
// STATUS_TIMEOUT_PEER_FLAG and runs to its end (0 restores the default of 2 s).  Applies to launches made
// after the call; returns the previous value.
extern "C" unsigned long long tahb_set_peer_wait_limit_ns(unsigned long long ns) {
  const unsigned long long prev = g_peer_wait_limit_ns;
  g_peer_wait_limit_ns = ns == 0 ? WAIT_TIMEOUT_NS : ns;
  return prev;
}

extern "C" int tahb_rmsnorm(const void* x, const void* w, void* y, int M, int H, long long ldx, long long ldy,
                            float eps, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H % 8) return -1;
  const int nvec = H / 8;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
  cudaError_t e;
  if (nvec <= 128) e = launch_chain(rmsnorm_kernel<1>, dim3(M), dim3(128), 0, stream, X, W, Y, H, ldx, ldy, eps);
  else if (nvec <= 256) e = launch_chain(rmsnorm_kernel<2>, dim3(M), dim3(128), 0, stream, X, W, Y, H, ldx, ldy, eps);
  else if (nvec <= 512) e = launch_chain(rmsnorm_kernel<4>, dim3(M), dim3(128), 0, stream, X, W, Y, H, ldx, ldy, eps);
  else if (nvec <= 1024) e = launch_chain(rmsnorm_kernel<8>, dim3(M), dim3(128), 0, stream, X, W, Y, H, ldx, ldy, eps);
  else return -2;
  return e == cudaSuccess ? 0 : -3;
}

// RMSNorm + gated LoRA-A in one launch (see rmsnorm_lora_kernel).  H % 8 == 0, H <= 8192.
extern "C" int tahb_rmsnorm_lora(const void* x, const void* w, void* y, int M, int H, long long ldx, long long ldy,
                                 float eps, const int* gate, const void* A, void* T, int R, long long ldt,
                                 cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H % 8 || H > 8192 || R <= 0 || M > 1024) return -1;
  const int lora_ctas = gate != nullptr ? NORM_LORA_SLOTS * NORM_LORA_SLICES : 0;
  cudaError_t e = launch_chain(rmsnorm_lora_kernel, dim3(M + lora_ctas), dim3(256), (size_t)H * 2, stream,
                               reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
                               reinterpret_cast<__nv_bfloat16*>(y), M, H, ldx, ldy, eps, gate,
                               reinterpret_cast<const __nv_bfloat16*>(A), reinterpret_cast<__nv_bfloat16*>(T), R, ldt);
  return e == cudaSuccess ? 0 : -3;
}

extern "C" int tahb_qk_norm_rope_kv(const void* qkv, const void* q_w, const void* k_w, void* q_out, void* k_dense,
                                    void* v_dense, void* const* caches, int n_caches, const int* cache_sel,
                                    const int* slot, const int* pos, int M, int nq, int nkv, int hd, int page_size,
                                    long long ld_qkv, float eps, float theta, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (n_caches > 4) return -1;
  QkvRopeParams p;
  p.qkv = reinterpret_cast<const __nv_bfloat16*>(qkv);
  p.q_w = reinterpret_cast<const __nv_bfloat16*>(q_w);
  p.k_w = reinterpret_cast<const __nv_bfloat16*>(k_w);
  p.q_out = reinterpret_cast<__nv_bfloat16*>(q_out);
  p.k_dense = reinterpret_cast<__nv_bfloat16*>(k_dense);
  p.v_dense = reinterpret_cast<__nv_bfloat16*>(v_dense);
  for (int i = 0; i < 4; ++i) p.cache[i] = i < n_caches ? reinterpret_cast<__nv_bfloat16*>(caches[i]) : nullptr;
  p.cache_sel = cache_sel;
  p.slot = n_caches > 0 ? slot : nullptr;
  p.pos = pos;
  p.M = M; p.nq = nq; p.nkv = nkv; p.page_size = page_size;
  p.ld_qkv = ld_qkv;
  p.eps = eps;
  p.log2_theta = log2f(theta);
  const long long warps = (long long)M * (nq + 2 * nkv);
  const int blocks = (int)((warps + 3) / 4);
  cudaError_t e = cudaSuccess;
  if (hd == 128) e = launch_chain(qk_norm_rope_kv_kernel<128>, dim3(blocks), dim3(128), 0, stream, p);
  else if (hd == 64) e = launch_chain(qk_norm_rope_kv_kernel<64>, dim3(blocks), dim3(128), 0, stream, p);
  else return -2;
  return e == cudaSuccess ? 0 : -3;
}

// y = LayerNorm(x) * w + b per row; or, with dot_w, z[r] = bf16(LayerNorm(x[r]) . dot_w + dot_b) (fp32 out).
extern "C" int tahb_layernorm(const void* x, const void* w, const void* b, void* y, const void* dot_w, const void* dot_b,
                              float* z, int M, int D, long long ldx, long long ldy, float eps, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (D % 8 || D > 4096) return -1;
  cudaError_t e = launch_chain(layernorm_kernel, dim3((M + 3) / 4), dim3(128), 0, stream,
                               reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),
                               reinterpret_cast<const __nv_bfloat16*>(b), reinterpret_cast<__nv_bfloat16*>(y),
                               reinterpret_cast<const __nv_bfloat16*>(dot_w), reinterpret_cast<const __nv_bfloat16*>(dot_b),
                               z, M, D, ldx, ldy, eps);
  return e == cudaSuccess ? 0 : -3;
}

extern "C" int tahb_rope_table(const int* pos, void* cs, int M, int hd, float theta, cudaStream_t stream) {
  if (M <= 0) return 0;
  const long long n = (long long)M * (hd / 2);
  rope_table_kernel<<<(int)((n + 255) / 256), 256, 0, stream>>>(pos, reinterpret_cast<__nv_bfloat16*>(cs), M, hd,
                                                               log2f(theta));
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int tahb_embed_gather(const void* E, const int* tok, void* out, int M, int H, long long ld_out,
                                 cudaStream_t stream) {
  if (M <= 0) return 0;
  embed_gather_kernel<<<M, 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(E), tok,
                                             reinterpret_cast<__nv_bfloat16*>(out), H, ld_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

static int lora_a_rows_launch(const void* x, const void* A, void* T, const int* gate, int M, int K, int R,
                              long long ldx, long long ldt, const void* wait_flag, const void* wait_target,
                              int wait_world, int* status, cudaStream_t stream) {
  if (M <= 0 || R <= 0) return 0;
  if (K % 8) return -1;
  cudaError_t e;
  if (gate != nullptr && M <= 1024)
    e = launch_chain(lora_a_rows_kernel, dim3(M < LORA_SLOTS ? M : LORA_SLOTS, (R + 7) / 8), dim3(256), 0, stream,
                     reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(A),
                     reinterpret_cast<__nv_bfloat16*>(T), gate, M, K, R, ldx, ldt,
                     reinterpret_cast<const uint32_t*>(wait_flag), reinterpret_cast<const uint32_t*>(wait_target),
                     wait_flag ? wait_world : 0, status, peer_wait_limit_ns());
  else
    e = launch_chain(lora_a_rows_dense_kernel, dim3(M, (R + 7) / 8), dim3(256), 0, stream,
                     reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(A),
                     reinterpret_cast<__nv_bfloat16*>(T), gate, K, R, ldx, ldt,
                     reinterpret_cast<const uint32_t*>(wait_flag), reinterpret_cast<const uint32_t*>(wait_target),
                     wait_flag ? wait_world : 0, status, peer_wait_limit_ns());
  return e == cudaSuccess ? 0 : -3;
}

extern "C" int tahb_lora_a_rows(const void* x, const void* A, void* T, const int* gate, int M, int K, int R,
                                long long ldx, long long ldt, cudaStream_t stream) {
  return lora_a_rows_launch(x, A, T, gate, M, K, R, ldx, ldt, nullptr, nullptr, 0, nullptr, stream);
}

// Tensor-parallel variant: gated rows first wait until the owners' broadcast of x has landed.
extern "C" int tahb_lora_a_rows_tp(const void* x, const void* A, void* T, const int* gate, int M, int K, int R,
                                   long long ldx, long long ldt, const void* wait_flag, const void* wait_target,
                                   int wait_world, int* status, cudaStream_t stream) {
  return lora_a_rows_launch(x, A, T, gate, M, K, R, ldx, ldt, wait_flag, wait_target, wait_world, status, stream);
}

extern "C" int tahb_swiglu(const void* gu, void* out, int M, int I, long long ld_in, long long ld_out,
                           cudaStream_t stream) {
  if (M <= 0) return 0;
  const bool vec = I % 8 == 0 && ld_in % 8 == 0 && ld_out % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const long long n = vec ? (long long)M * (I / 8) : (long long)M * I;
  int blocks = (int)((n + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (vec)
    swiglu_vec_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(gu),
                                                  reinterpret_cast<__nv_bfloat16*>(out), M, I, ld_in, ld_out);
  else
    swiglu_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(gu),
                                              reinterpret_cast<__nv_bfloat16*>(out), M, I, ld_in, ld_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int tahb_logits_post(const void* logits, void* cum, const int* depth, int* best, float* best_val, int M,
                                int V, long long ld_logits, long long ld_cum, cudaStream_t stream) {
  if (M <= 0) return 0;
  if ((ld_logits % 8) || (ld_cum % 8)) return -1;
  logits_post_kernel<<<M, 1024, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits),
                                             reinterpret_cast<__nv_bfloat16*>(cum), depth, best, best_val, V, ld_logits, ld_cum);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
