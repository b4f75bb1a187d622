// Loss kernels of the training step.
//
// cross entropy on bf16 logits, fp32 math, no fp32 copy of the [rows, V] logits: the reference upcasts the
// whole logits tensor to fp32 (4.6 GiB at 8192 x 151936) and lets PyTorch form log-softmax and NLL in
// separate passes (reference tah/model/loss.py:65-81, tah/train/trainer.py:95-107); here one kernel reads a
// row once (online max / sum) and writes its loss and log-sum-exp, and the backward kernel writes
//     dlogits[r, j] = (exp(x_j - lse_r) - [j == label_r]) * g_r        (0 for ignored rows)
// straight in bf16.
//
// soft-embedding backward: see soft_embed_bwd_kernel.
//
// binary cross entropy with logits (+ pos_weight) for the decider head: per-token loss terms, the weighted
// sum, the number of labelled tokens and the number of correct threshold decisions in one launch (reference
// tah/model/loss.py:120-177 does these as separate PyTorch ops), and its backward.
#include "common.cuh"

namespace tahb {

constexpr int CE_THREADS = 512;

struct CeShared {
  float m[CE_THREADS / 32];
  float s[CE_THREADS / 32];
};

__global__ void __launch_bounds__(CE_THREADS) ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits,
                                                            const long long* __restrict__ labels, float* __restrict__ loss,
                                                            float* __restrict__ lse, int V, long long ld, int ignore_index) {
  __shared__ CeShared sh;
  const int r = blockIdx.x;
  const long long label = labels[r];
  if (label == ignore_index) {               // ignored rows cost nothing
    if (threadIdx.x == 0) { loss[r] = 0.f; lse[r] = 0.f; }
    return;
  }
  const __nv_bfloat16* xr = logits + (size_t)r * ld;
  float m = -INFINITY, s = 0.f;
  const int nvec = V / 8;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    const uint4 v = reinterpret_cast<const uint4*>(xr)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 t = __bfloat1622float2(h[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
    float cm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) cm = fmaxf(cm, f[j]);
    if (cm > m) { s *= __expf(m - cm); m = cm; }
#pragma unroll
    for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) {
    const float f = __bfloat162float(xr[i]);
    if (f > m) { s *= __expf(m - f); m = f; }
    s += __expf(f - m);
  }
  // combine (m, s) pairs: warp, then block
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sh.m[warp] = m; sh.s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    m = lane < CE_THREADS / 32 ? sh.m[lane] : -INFINITY;
    s = lane < CE_THREADS / 32 ? sh.s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
      m = nm;
    }
    if (lane == 0) {
      const float l = m + logf(s);
      lse[r] = l;
      loss[r] = l - __bfloat162float(xr[label]);
    }
  }
}

__global__ void __launch_bounds__(CE_THREADS) ce_bwd_kernel(const __nv_bfloat16* __restrict__ logits,
                                                            const long long* __restrict__ labels,
                                                            const float* __restrict__ lse, const float* __restrict__ gscale,
                                                            __nv_bfloat16* __restrict__ dlogits, int V, long long ld,
                                                            long long ldd, int ignore_index) {
  const int r = blockIdx.x;
  const long long label = labels[r];
  const __nv_bfloat16* xr = logits + (size_t)r * ld;
  __nv_bfloat16* dr = dlogits + (size_t)r * ldd;
  const int nvec = V / 8;
  if (label == ignore_index) {
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) reinterpret_cast<uint4*>(dr)[i] = make_uint4(0, 0, 0, 0);
    for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) dr[i] = __float2bfloat16_rn(0.f);
    return;
  }
  const float l = lse[r], g = gscale[0];
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    const uint4 v = reinterpret_cast<const uint4*>(xr)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(h[j]);
      const int c = i * 8 + 2 * j;
      oh[j] = __floats2bfloat162_rn((__expf(t.x - l) - (c == label ? 1.f : 0.f)) * g,
                                    (__expf(t.y - l) - (c + 1 == label ? 1.f : 0.f)) * g);
    }
    reinterpret_cast<uint4*>(dr)[i] = o;
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS)
    dr[i] = __float2bfloat16_rn((__expf(__bfloat162float(xr[i]) - l) - (i == label ? 1.f : 0.f)) * g);
}

// ---------------------------------------------------------------------------------------------
// BCE with logits over n tokens: w_i = (label_i != -100); y_i = (label_i > depth);
//   per_i = -[pw * y_i * log sigmoid(z_i) + (1 - y_i) * log(1 - sigmoid(z_i))]
//   out[0] += sum w_i per_i, out[1] += sum w_i, out[2] += sum w_i [ (sigmoid(z_i) > thr) == y_i ]
// and, when dz != nullptr (backward), dz_i = g[0] * w_i * ((1 - y_i) sigmoid(z_i) - pw y_i (1 - sigmoid(z_i))).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bce_logits_kernel(const float* __restrict__ z, const long long* __restrict__ labels,
                                                         int depth, float pos_weight, float thr, int n,
                                                         float* __restrict__ out, const float* __restrict__ g,
                                                         float* __restrict__ dz) {
  __shared__ float red[3][8];
  float a = 0.f, b = 0.f, c = 0.f;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const long long lab = labels[i];
    const float w = lab != -100 ? 1.f : 0.f;
    const float y = lab > depth ? 1.f : 0.f;
    const float zi = z[i];
    // log sigmoid(z) = -softplus(-z), log(1 - sigmoid(z)) = -softplus(z); softplus(x) = max(x, 0) + log1p(exp(-|x|))
    const float sp_pos = fmaxf(zi, 0.f) + log1pf(__expf(-fabsf(zi)));
    const float sp_neg = sp_pos - zi;
    const float sig = 1.f / (1.f + __expf(-zi));
    if (dz != nullptr) {
      dz[i] = g[0] * w * ((1.f - y) * sig - pos_weight * y * (1.f - sig));
    } else {
      a += w * (pos_weight * y * sp_neg + (1.f - y) * sp_pos);
      b += w;
      c += w * (((sig > thr) ? 1.f : 0.f) == y ? 1.f : 0.f);
    }
  }
  if (dz != nullptr) return;
  a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { red[0][warp] = a; red[1][warp] = b; red[2][warp] = c; }
  __syncthreads();
  if (threadIdx.x < 3) {
    float t = 0.f;
    for (int k = 0; k < 8; ++k) t += red[threadIdx.x][k];
    atomicAdd(out + threadIdx.x, t);
  }
}

// ---------------------------------------------------------------------------------------------
// Backward of the soft next-pass input  out[r] = sum_k p_k E[idx_k],  p = softmax(val[r, 0..K)):
//   dp_k   = dout[r] . E[idx_k]
//   dval_k = p_k (dp_k - sum_j p_j dp_j)
//   dE[idx_k] += p_k dout[r]                  (fp32 accumulator, vector reds of four floats)
// One CTA of 256 threads per token: the token's dout row sits in shared memory, a warp owns one k at a time
// (one pass over the embedding row serves both the dot product and - once p is known, which needs no E -
// the scatter).  The PyTorch statement of this op materialises a [rows, K, H] gather in forward and backward
// (3.3 GB at 8192 tokens) and scatters with a sort-based index_put.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) soft_embed_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                                             const float* __restrict__ val, const int* __restrict__ idx,
                                                             const __nv_bfloat16* __restrict__ E, float* __restrict__ dval,
                                                             float* __restrict__ dE, int K, int H, long long ld_dout) {
  extern __shared__ float s_dout[];          // H floats
  __shared__ float prob[128];
  __shared__ float dp[128];
  __shared__ int id[128];
  __shared__ float s_dot;
  const int r = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < 32) {
    float mx = -INFINITY;
    for (int k = tid; k < K; k += 32) mx = fmaxf(mx, val[(size_t)r * K + k]);
    mx = warp_max(mx);
    float s = 0.f;
    for (int k = tid; k < K; k += 32) s += __expf(val[(size_t)r * K + k] - mx);
    s = warp_sum(s);
    for (int k = tid; k < K; k += 32) {
      prob[k] = __expf(val[(size_t)r * K + k] - mx) / s;
      id[k] = idx[(size_t)r * K + k];
    }
  }
  const __nv_bfloat16* dr = dout + (size_t)r * ld_dout;
  for (int i = tid; i < H / 8; i += 256) {
    const uint4 v = reinterpret_cast<const uint4*>(dr)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      s_dout[i * 8 + 2 * j] = f.x;
      s_dout[i * 8 + 2 * j + 1] = f.y;
    }
  }
  __syncthreads();
  for (int k = warp; k < K; k += 8) {
    const __nv_bfloat16* er = E + (size_t)id[k] * H;
    float* gr = dE + (size_t)id[k] * H;
    const float pk = prob[k];
    float acc = 0.f;
    for (int i = lane; i < H / 8; i += 32) {
      const uint4 v = reinterpret_cast<const uint4*>(er)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
      const float* d = s_dout + i * 8;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc += f.x * d[2 * j] + f.y * d[2 * j + 1];
      }
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(gr + i * 8), "f"(pk * d[0]), "f"(pk * d[1]),
                   "f"(pk * d[2]), "f"(pk * d[3]) : "memory");
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(gr + i * 8 + 4), "f"(pk * d[4]), "f"(pk * d[5]),
                   "f"(pk * d[6]), "f"(pk * d[7]) : "memory");
    }
    acc = warp_sum(acc);
    if (lane == 0) dp[k] = acc;
  }
  __syncthreads();
  if (tid < 32) {
    float t = 0.f;
    for (int k = tid; k < K; k += 32) t += prob[k] * dp[k];
    t = warp_sum(t);
    if (tid == 0) s_dot = t;
  }
  __syncthreads();
  for (int k = tid; k < K; k += 256) dval[(size_t)r * K + k] = prob[k] * (dp[k] - s_dot);
}

}  // namespace tahb

using namespace tahb;

// dval[rows, K] (fp32) and dE[V, H] += (fp32 accumulator, zeroed by the caller) of the soft-embedding mix.
extern "C" int tahb_soft_embed_bwd(const void* dout, const float* val, const int* idx, const void* E, float* dval,
                                   float* dE, int rows, int K, int H, long long ld_dout, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K > 128 || H % 8 || (ld_dout % 8)) return -1;
  soft_embed_bwd_kernel<<<rows, 256, (size_t)H * 4, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dout), val, idx,
                                                             reinterpret_cast<const __nv_bfloat16*>(E), dval, dE, K, H,
                                                             ld_dout);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// loss[r] = logsumexp(logits[r]) - logits[r, label_r] (0 for label == ignore_index), lse[r] kept for the backward.
extern "C" int tahb_ce_fwd(const void* logits, const long long* labels, float* loss, float* lse, int rows, int V,
                           long long ld, int ignore_index, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((ld % 8) || (reinterpret_cast<uintptr_t>(logits) & 15)) return -1;
  ce_fwd_kernel<<<rows, CE_THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), labels, loss, lse, V, ld,
                                                 ignore_index);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dlogits[r, :] = (softmax(logits[r]) - onehot(label_r)) * gscale[0], zeros for ignored rows.
extern "C" int tahb_ce_bwd(const void* logits, const long long* labels, const float* lse, const float* gscale,
                           void* dlogits, int rows, int V, long long ld, long long ldd, int ignore_index,
                           cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((ld % 8) || (ldd % 8) || (reinterpret_cast<uintptr_t>(logits) & 15) || (reinterpret_cast<uintptr_t>(dlogits) & 15))
    return -1;
  ce_bwd_kernel<<<rows, CE_THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), labels, lse, gscale,
                                                 reinterpret_cast<__nv_bfloat16*>(dlogits), V, ld, ldd, ignore_index);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// forward (dz == nullptr): out[0..2] += (weighted BCE sum, labelled count, correct decisions); backward: dz filled.
extern "C" int tahb_bce_logits(const float* z, const long long* labels, int depth, float pos_weight, float thr, int n,
                               float* out, const float* g, float* dz, cudaStream_t stream) {
  if (n <= 0) return 0;
  int blocks = (n + 255) / 256;
  if (blocks > 148) blocks = 148;
  bce_logits_kernel<<<blocks, 256, 0, stream>>>(z, labels, depth, pos_weight, thr, n, out, g, dz);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
