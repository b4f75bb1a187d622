// Backward kernels of the memory-bound training ops: RMSNorm and SwiGLU.  Each reads its inputs
// once and writes its outputs once (bf16 in / out, fp32 math).
#include "common.cuh"

namespace tahb {

// ---------------------------------------------------------------------------------------------
// RMSNorm backward.  y = w * (x * rstd),  rstd = rsqrt(mean(x^2) + eps).  With gn = gy * w:
//     gx = rstd * (gn - xn * mean(gn * xn)),   gw = sum_rows gy * xn,   xn = x * rstd.
// A CTA of 256 threads walks RMSB_ROWS consecutive rows; thread t owns columns 8t..8t+7 (+ 2048 k),
// keeps its slice of gw in registers over those rows and adds it to the fp32 gw buffer once at the
// end, so the atomics per launch are rows / RMSB_ROWS * H.
// ---------------------------------------------------------------------------------------------
constexpr int RMSB_ROWS = 32;

template <int VPT>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          const __nv_bfloat16* __restrict__ gy,
                                                          __nv_bfloat16* __restrict__ gx, float* __restrict__ gw,
                                                          int M, int H, float eps) {
  __shared__ float red[2][8];
  const int nvec = H / 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float wv[VPT][8], gwa[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = tid + i * 256;
#pragma unroll
    for (int j = 0; j < 8; ++j) { gwa[i][j] = 0.f; wv[i][j] = 0.f; }
    if (idx < nvec) {
      const uint4 u = *reinterpret_cast<const uint4*>(w + idx * 8);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h2[j]); wv[i][2 * j] = f.x; wv[i][2 * j + 1] = f.y; }
    }
  }
  const int row_lo = blockIdx.x * RMSB_ROWS;
  const int row_hi = min(M, row_lo + RMSB_ROWS);
  for (int row = row_lo; row < row_hi; ++row) {
    const size_t off = (size_t)row * H;
    float xv[VPT][8], gv[VPT][8];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = tid + i * 256;
      if (idx < nvec) {
        const uint4 ux = *reinterpret_cast<const uint4*>(x + off + idx * 8);
        const uint4 ug = *reinterpret_cast<const uint4*>(gy + off + idx * 8);
        const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&ux);
        const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&ug);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fx = __bfloat1622float2(hx[j]), fg = __bfloat1622float2(hg[j]);
          xv[i][2 * j] = fx.x; xv[i][2 * j + 1] = fx.y;
          gv[i][2 * j] = fg.x; gv[i][2 * j + 1] = fg.y;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ss += xv[i][j] * xv[i][j];
          dot += gv[i][j] * wv[i][j] * xv[i][j];
        }
      }
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    __syncthreads();
    if (lane == 0) { red[0][warp] = ss; red[1][warp] = dot; }
    __syncthreads();
    float tss = 0.f, tdot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { tss += red[0][k]; tdot += red[1][k]; }
    const float rstd = rsqrtf(tss / (float)H + eps);
    const float c = tdot * rstd * rstd / (float)H;          // mean(gn * xn) * rstd, applied to x
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = tid + i * 256;
      if (idx < nvec) {
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = rstd * (gv[i][2 * j] * wv[i][2 * j] - xv[i][2 * j] * c);
          const float b = rstd * (gv[i][2 * j + 1] * wv[i][2 * j + 1] - xv[i][2 * j + 1] * c);
          o2[j] = __floats2bfloat162_rn(a, b);
        }
        *reinterpret_cast<uint4*>(gx + off + idx * 8) = o;
#pragma unroll
        for (int j = 0; j < 8; ++j) gwa[i][j] += gv[i][j] * xv[i][j] * rstd;
      }
    }
  }
  if (gw != nullptr) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = tid + i * 256;
      if (idx < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(gw + idx * 8 + j, gwa[i][j]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU backward on a [M, 2I] gate|up tensor: out = silu(g) * u,
//     d_gate = gy * u * sig(g) * (1 + g * (1 - sig(g))),   d_up = gy * silu(g).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                                         const __nv_bfloat16* __restrict__ gy,
                                                         __nv_bfloat16* __restrict__ dgu, long long M, int I) {
  const long long nvec = M * (I / 8);
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    const long long r = v / (I / 8);
    const int c = (int)(v % (I / 8)) * 8;
    const uint4 ug = *reinterpret_cast<const uint4*>(gu + r * 2 * I + c);
    const uint4 uu = *reinterpret_cast<const uint4*>(gu + r * 2 * I + I + c);
    const uint4 uy = *reinterpret_cast<const uint4*>(gy + r * I + c);
    const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&ug);
    const __nv_bfloat162* hu = reinterpret_cast<const __nv_bfloat162*>(&uu);
    const __nv_bfloat162* hy = reinterpret_cast<const __nv_bfloat162*>(&uy);
    uint4 og, ou;
    __nv_bfloat162* o_g = reinterpret_cast<__nv_bfloat162*>(&og);
    __nv_bfloat162* o_u = reinterpret_cast<__nv_bfloat162*>(&ou);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(hg[j]), u = __bfloat1622float2(hu[j]), y = __bfloat1622float2(hy[j]);
      const float s0 = 1.0f / (1.0f + __expf(-g.x)), s1 = 1.0f / (1.0f + __expf(-g.y));
      o_g[j] = __floats2bfloat162_rn(y.x * u.x * s0 * (1.0f + g.x * (1.0f - s0)), y.y * u.y * s1 * (1.0f + g.y * (1.0f - s1)));
      o_u[j] = __floats2bfloat162_rn(y.x * g.x * s0, y.y * g.y * s1);
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * I + c) = og;
    *reinterpret_cast<uint4*>(dgu + r * 2 * I + I + c) = ou;
  }
}

// ---------------------------------------------------------------------------------------------
// Backward of the per-head QK RMSNorm + rotate-half RoPE (forward: qk_norm_rope_kv_kernel in
// elementwise.cu).  One warp per (token, head), grid-stride; lane l owns elements l*EPL..+EPL-1.
//   n = w * (x * rstd),  y = n * cos + rot(n) * sin      (q and k heads; v heads pass through)
//   gn = gy * cos +/- partner(gy) * sin ;  gx = rstd * (gn*w - xn * mean(gn*w*xn)) ;  gw += gn * xn
// The weight gradients are summed per CTA in shared memory and added to the fp32 buffers once.
// ---------------------------------------------------------------------------------------------
struct QkRopeBwdParams {
  const __nv_bfloat16* qkv;      // [M, (nq + 2 nkv) * HD] forward input
  const __nv_bfloat16* q_w;
  const __nv_bfloat16* k_w;
  const __nv_bfloat16* gq;       // [M, nq * HD]
  const __nv_bfloat16* gk;       // [M, nkv * HD]
  const __nv_bfloat16* gv;       // [M, nkv * HD]
  __nv_bfloat16* gqkv;           // [M, (nq + 2 nkv) * HD]
  float* gq_w;                   // [HD] fp32, added to
  float* gk_w;
  const int* pos;
  int M, nq, nkv;
  float eps, log2_theta;
};

template <int HD>
__global__ void __launch_bounds__(128) qk_norm_rope_bwd_kernel(const QkRopeBwdParams p) {
  constexpr int EPL = HD / 32;
  __shared__ float s_gw[2][HD];
  for (int i = threadIdx.x; i < 2 * HD; i += blockDim.x) (&s_gw[0][0])[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int heads = p.nq + 2 * p.nkv;
  const long long total = (long long)p.M * heads;
  const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
  float gw_q[EPL], gw_k[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) { gw_q[i] = 0.f; gw_k[i] = 0.f; }
  for (long long wg = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); wg < total; wg += stride) {
    const int t = (int)(wg / heads);
    const int h = (int)(wg % heads);
    const bool is_q = h < p.nq;
    const bool is_k = !is_q && h < p.nq + p.nkv;
    __nv_bfloat16* dst = p.gqkv + ((size_t)t * heads + h) * HD + lane * EPL;
    if (!is_q && !is_k) {
      const __nv_bfloat16* g = p.gv + ((size_t)t * p.nkv + (h - p.nq - p.nkv)) * HD + lane * EPL;
#pragma unroll
      for (int i = 0; i < EPL; ++i) dst[i] = g[i];
      continue;
    }
    const __nv_bfloat16* src = p.qkv + ((size_t)t * heads + h) * HD + lane * EPL;
    const __nv_bfloat16* g = is_q ? p.gq + ((size_t)t * p.nq + h) * HD + lane * EPL
                                  : p.gk + ((size_t)t * p.nkv + (h - p.nq)) * HD + lane * EPL;
    const __nv_bfloat16* w = (is_q ? p.q_w : p.k_w) + lane * EPL;
    float x[EPL], gy[EPL], wv[EPL], gpart[EPL];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      x[i] = __bfloat162float(src[i]);
      gy[i] = __bfloat162float(g[i]);
      wv[i] = __bfloat162float(w[i]);
      ss += x[i] * x[i];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)HD + p.eps);
#pragma unroll
    for (int i = 0; i < EPL; ++i) gpart[i] = __shfl_xor_sync(0xffffffffu, gy[i], 16);
    const float posf = (float)p.pos[t];
    const bool upper = lane >= 16;
    float gn[EPL], xn[EPL];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int d = lane * EPL + i;
      const int j = upper ? d - HD / 2 : d;
      const float inv = exp2f(-(2.0f * (float)j / (float)HD) * p.log2_theta);
      const float ang = posf * inv;
      const float c = bf16_round(cosf(ang)), sn = bf16_round(sinf(ang));
      gn[i] = gy[i] * c + (upper ? -gpart[i] : gpart[i]) * sn;
      xn[i] = x[i] * rstd;
      dot += gn[i] * wv[i] * xn[i];
    }
    dot = warp_sum(dot) / (float)HD;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      dst[i] = __float2bfloat16_rn(rstd * (gn[i] * wv[i] - xn[i] * dot));
      if (is_q) gw_q[i] += gn[i] * xn[i];
      else gw_k[i] += gn[i] * xn[i];
    }
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    atomicAdd(&s_gw[0][lane * EPL + i], gw_q[i]);
    atomicAdd(&s_gw[1][lane * EPL + i], gw_k[i]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < HD; i += blockDim.x) {
    if (p.gq_w != nullptr) atomicAdd(p.gq_w + i, s_gw[0][i]);
    if (p.gk_w != nullptr) atomicAdd(p.gk_w + i, s_gw[1][i]);
  }
}

}  // namespace tahb

using namespace tahb;

// Backward of tahb_qk_norm_rope_kv for contiguous tensors.  gq_w / gk_w: fp32 [hd] the kernel adds into.
extern "C" int tahb_qk_norm_rope_bwd(const void* qkv, const void* q_w, const void* k_w, const void* gq, const void* gk,
                                     const void* gv, void* gqkv, float* gq_w, float* gk_w, const int* pos, int M,
                                     int nq, int nkv, int hd, float eps, float theta, cudaStream_t stream) {
  if (M <= 0) return 0;
  QkRopeBwdParams p;
  p.qkv = reinterpret_cast<const __nv_bfloat16*>(qkv);
  p.q_w = reinterpret_cast<const __nv_bfloat16*>(q_w);
  p.k_w = reinterpret_cast<const __nv_bfloat16*>(k_w);
  p.gq = reinterpret_cast<const __nv_bfloat16*>(gq);
  p.gk = reinterpret_cast<const __nv_bfloat16*>(gk);
  p.gv = reinterpret_cast<const __nv_bfloat16*>(gv);
  p.gqkv = reinterpret_cast<__nv_bfloat16*>(gqkv);
  p.gq_w = gq_w;
  p.gk_w = gk_w;
  p.pos = pos;
  p.M = M; p.nq = nq; p.nkv = nkv;
  p.eps = eps;
  p.log2_theta = log2f(theta);
  const long long warps = (long long)M * (nq + 2 * nkv);
  long long blocks = (warps + 3) / 4;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (hd == 128) qk_norm_rope_bwd_kernel<128><<<(int)blocks, 128, 0, stream>>>(p);
  else if (hd == 64) qk_norm_rope_bwd_kernel<64><<<(int)blocks, 128, 0, stream>>>(p);
  else return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// x, gy, gx: [M, H] bf16 contiguous; w [H] bf16; gw: fp32 [H] that the kernel ADDS into (or null).
extern "C" int tahb_rmsnorm_bwd(const void* x, const void* w, const void* gy, void* gx, float* gw, int M, int H,
                                float eps, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H % 8) return -1;
  const int nvec = H / 8;
  const int grid = (M + RMSB_ROWS - 1) / RMSB_ROWS;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto GY = reinterpret_cast<const __nv_bfloat16*>(gy);
  auto GX = reinterpret_cast<__nv_bfloat16*>(gx);
  if (nvec <= 256) rmsnorm_bwd_kernel<1><<<grid, 256, 0, stream>>>(X, W, GY, GX, gw, M, H, eps);
  else if (nvec <= 512) rmsnorm_bwd_kernel<2><<<grid, 256, 0, stream>>>(X, W, GY, GX, gw, M, H, eps);
  else if (nvec <= 1024) rmsnorm_bwd_kernel<4><<<grid, 256, 0, stream>>>(X, W, GY, GX, gw, M, H, eps);
  else return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// gu, dgu: [M, 2I] bf16 contiguous (gate | up); gy: [M, I].
extern "C" int tahb_swiglu_bwd(const void* gu, const void* gy, void* dgu, long long M, int I, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (I % 8) return -1;
  const long long nvec = M * (I / 8);
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  swiglu_bwd_kernel<<<(int)blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(gu),
                                                     reinterpret_cast<const __nv_bfloat16*>(gy),
                                                     reinterpret_cast<__nv_bfloat16*>(dgu), M, I);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
