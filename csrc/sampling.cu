// Per-tick control kernels of the decode engine: sorted top-k over the vocabulary, the soft
// embedding mix for rows that iterate again, the top-k/top-p/min-p sampler, the continue/stop
// decision, and the two scheduler kernels that advance every row's (token, depth, position)
// state and allocate KV pages on the device.  None of them synchronises with the host, so a
// whole decode tick is one CUDA graph.
#include "common.cuh"

namespace tahb {

// ---------------------------------------------------------------------------------------------
// Sorted top-k (k <= 128) of one bf16 row of V values per CTA, for rows whose flag is set.
//
// Fast path (two sweeps over the row): a 4096-bin histogram of the top 12 bits of the 16-bit
// order-preserving key locates the bin holding the k-th largest value; every key in or above that
// bin is a candidate (k plus a few dozen for real logits) and is collected unordered; each
// candidate then counts the candidates that precede it in (value desc, index asc) order, which is
// its output slot.  The result is exact and deterministic (ties: lowest index first).
// Fallback (more than 1024 candidates, e.g. a constant row): two 256-bin radix passes, an
// index-ordered gather and a 128-wide bitonic sort.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t order_key(__nv_bfloat16 v) {
  const uint16_t u = __bfloat16_as_ushort(v);
  return (u & 0x8000) ? (uint16_t)~u : (uint16_t)(u | 0x8000);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  const uint16_t u = (k & 0x8000) ? (uint16_t)(k & 0x7fff) : (uint16_t)~k;
  return __bfloat162float(__ushort_as_bfloat16(u));
}

constexpr int TOPK_THREADS = 1024;
constexpr int TOPK_CAND = 1024;

__device__ __forceinline__ int find_bin(const int* hist, int want, int* above) {
  // largest b with sum_{j > b} hist[j] < want <= sum_{j >= b} hist[j]
  int acc = 0;
  for (int b = 255; b >= 0; --b) {
    if (acc + hist[b] >= want) { *above = acc; return b; }
    acc += hist[b];
  }
  *above = acc;
  return 0;
}

struct TopkShared {
  int scratch[8192];            // fast path: two 4096-bin histograms; fallback: 32 per-warp 256-bin histograms
  uint32_t cand_key[TOPK_CAND];
  int cand_idx[TOPK_CAND];
  int hist[256];
  int warp_cnt[2][32];
  int s_bin, s_above, s_ngt, s_neq, s_cnt;
};

// Fallback: exact for any input, index-ordered gather with two block barriers per 1024 elements.
__device__ __noinline__ void topk_ordered_path(TopkShared& sh, const __nv_bfloat16* __restrict__ xr, float* out_val,
                                               int* out_idx, int V, int K) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int (*whist)[256] = reinterpret_cast<int (*)[256]>(sh.scratch);
  uint32_t* sel_key = sh.cand_key;
  int* sel_idx = sh.cand_idx;
  __syncthreads();
  for (int i = tid; i < (TOPK_THREADS / 32) * 256; i += TOPK_THREADS) sh.scratch[i] = 0;
  __syncthreads();
  for (int i = tid; i < V; i += TOPK_THREADS) atomicAdd(&whist[warp][order_key(xr[i]) >> 8], 1);
  __syncthreads();
  if (tid < 256) { int t = 0; for (int w = 0; w < TOPK_THREADS / 32; ++w) t += whist[w][tid]; sh.hist[tid] = t; }
  __syncthreads();
  if (tid == 0) { int ab; sh.s_bin = find_bin(sh.hist, K, &ab); sh.s_above = ab; }
  __syncthreads();
  const int b1 = sh.s_bin;
  const int above1 = sh.s_above;
  __syncthreads();
  for (int i = tid; i < (TOPK_THREADS / 32) * 256; i += TOPK_THREADS) sh.scratch[i] = 0;
  __syncthreads();
  for (int i = tid; i < V; i += TOPK_THREADS) {
    const uint32_t k = order_key(xr[i]);
    if ((int)(k >> 8) == b1) atomicAdd(&whist[warp][k & 255], 1);
  }
  __syncthreads();
  if (tid < 256) { int t = 0; for (int w = 0; w < TOPK_THREADS / 32; ++w) t += whist[w][tid]; sh.hist[tid] = t; }
  __syncthreads();
  if (tid == 0) { int ab; sh.s_bin = find_bin(sh.hist, K - above1, &ab); sh.s_above = ab; sh.s_ngt = 0; sh.s_neq = 0; }
  __syncthreads();
  const uint32_t thr = ((uint32_t)b1 << 8) | (uint32_t)sh.s_bin;
  const int n_gt_total = above1 + sh.s_above;  // keys strictly above the threshold (< K)
  const int need_eq = K - n_gt_total;          // how many threshold ties to take (>= 1)
  if (tid < 128) { sel_key[tid] = 0; sel_idx[tid] = 0x7fffffff; }
  __syncthreads();
  for (int base = 0; base < V; base += TOPK_THREADS) {
    const int i = base + tid;
    uint32_t k = 0;
    bool gt = false, eq = false;
    if (i < V) { k = order_key(xr[i]); gt = k > thr; eq = k == thr; }
    const uint32_t mg = __ballot_sync(0xffffffffu, gt), me = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) { sh.warp_cnt[0][warp] = __popc(mg); sh.warp_cnt[1][warp] = __popc(me); }
    __syncthreads();
    int og = sh.s_ngt, oe = sh.s_neq;
    for (int w = 0; w < warp; ++w) { og += sh.warp_cnt[0][w]; oe += sh.warp_cnt[1][w]; }
    og += __popc(mg & ((1u << lane) - 1));
    oe += __popc(me & ((1u << lane) - 1));
    if (gt && og < 128) { sel_key[og] = k; sel_idx[og] = i; }
    if (eq && oe < need_eq) { const int slot = n_gt_total + oe; if (slot < 128) { sel_key[slot] = k; sel_idx[slot] = i; } }
    __syncthreads();
    if (tid == 0) {
      int tg = 0, te = 0;
      for (int w = 0; w < TOPK_THREADS / 32; ++w) { tg += sh.warp_cnt[0][w]; te += sh.warp_cnt[1][w]; }
      sh.s_ngt += tg; sh.s_neq += te;
    }
    __syncthreads();
  }
  // bitonic sort of 128 (key desc, idx asc); empty slots have key 0 / idx max and sink to the end
  for (int size = 2; size <= 128; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (tid < 128) {
        const int partner = tid ^ stride;
        if (partner > tid) {
          const bool desc = (tid & size) == 0;
          const uint32_t ka = sel_key[tid], kb = sel_key[partner];
          const int ia = sel_idx[tid], ib = sel_idx[partner];
          const bool a_first = (ka > kb) || (ka == kb && ia < ib);   // a should precede b in final order
          if (desc ? !a_first : a_first) {
            sel_key[tid] = kb; sel_key[partner] = ka; sel_idx[tid] = ib; sel_idx[partner] = ia;
          }
        }
      }
      __syncthreads();
    }
  }
  if (tid < K) {
    out_val[tid] = key_value(sel_key[tid]);
    out_idx[tid] = sel_idx[tid];
  }
}

__global__ void __launch_bounds__(TOPK_THREADS) topk_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                                 const int* __restrict__ flag,
                                                                 float* __restrict__ out_val,
                                                                 int* __restrict__ out_idx, int V, int K,
                                                                 long long ldx, int force_ordered) {
  const int r = blockIdx.x;
  if (flag != nullptr && flag[r] == 0) return;
  const __nv_bfloat16* xr = x + (size_t)r * ldx;
  float* ov = out_val + (size_t)r * K;
  int* oi = out_idx + (size_t)r * K;
  __shared__ TopkShared sh;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (force_ordered) { topk_ordered_path(sh, xr, ov, oi, V, K); return; }
  const bool vec = (V % 8 == 0) && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0);

  // sweep 1: 4096-bin histogram of key >> 4 (two replicas, by warp parity, to thin out conflicts)
  for (int i = tid; i < 8192; i += TOPK_THREADS) sh.scratch[i] = 0;
  if (tid == 0) sh.s_cnt = 0;
  __syncthreads();
  int* myhist = sh.scratch + (warp & 1) * 4096;
  if (vec) {
    const uint4* xv = reinterpret_cast<const uint4*>(xr);
    for (int i = tid; i < V / 8; i += TOPK_THREADS) {
      const uint4 u = xv[i];
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(&myhist[order_key(e[j]) >> 4], 1);
    }
  } else {
    for (int i = tid; i < V; i += TOPK_THREADS) atomicAdd(&myhist[order_key(xr[i]) >> 4], 1);
  }
  __syncthreads();
  // locate the bin of the K-th largest: thread t owns bins 4t..4t+3; suffix sums over threads
  int hb[4], own = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) { hb[j] = sh.scratch[4 * tid + j] + sh.scratch[4096 + 4 * tid + j]; own += hb[j]; }
  int sfx = own;                                 // sum over lanes >= lane of this warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_down_sync(0xffffffffu, sfx, o);
    if (lane + o < 32) sfx += y;
  }
  if (lane == 0) sh.warp_cnt[0][warp] = sfx;
  __syncthreads();
  int higher = 0;
  for (int w = warp + 1; w < TOPK_THREADS / 32; ++w) higher += sh.warp_cnt[0][w];
  const int above_grp = sfx - own + higher;      // keys in bins above this thread's four
  if (above_grp < K && K <= above_grp + own) {
    int acc = above_grp;
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      if (acc < K && K <= acc + hb[j]) { sh.s_bin = 4 * tid + j; sh.s_above = acc; }
      acc += hb[j];
    }
  }
  __syncthreads();
  const uint32_t bin12 = (uint32_t)sh.s_bin;
  // sweep 2: collect every key in or above that bin
  if (vec) {
    const uint4* xv = reinterpret_cast<const uint4*>(xr);
    for (int i = tid; i < V / 8; i += TOPK_THREADS) {
      const uint4 u = xv[i];
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t k = order_key(e[j]);
        if ((k >> 4) >= bin12) {
          const int slot = atomicAdd(&sh.s_cnt, 1);
          if (slot < TOPK_CAND) { sh.cand_key[slot] = k; sh.cand_idx[slot] = i * 8 + j; }
        }
      }
    }
  } else {
    for (int i = tid; i < V; i += TOPK_THREADS) {
      const uint32_t k = order_key(xr[i]);
      if ((k >> 4) >= bin12) {
        const int slot = atomicAdd(&sh.s_cnt, 1);
        if (slot < TOPK_CAND) { sh.cand_key[slot] = k; sh.cand_idx[slot] = i; }
      }
    }
  }
  __syncthreads();
  const int C = sh.s_cnt;
  if (C > TOPK_CAND) { topk_ordered_path(sh, xr, ov, oi, V, K); return; }
  // rank every candidate among the candidates: its rank is its slot in the sorted output
  for (int c = tid; c < C; c += TOPK_THREADS) {
    const uint32_t kc = sh.cand_key[c];
    const int ic = sh.cand_idx[c];
    int rank = 0;
    for (int j = 0; j < C; ++j) {
      const uint32_t kj = sh.cand_key[j];
      rank += (kj > kc) || (kj == kc && sh.cand_idx[j] < ic);
    }
    if (rank < K) { ov[rank] = key_value(kc); oi[rank] = ic; }
  }
}

// ---------------------------------------------------------------------------------------------
// Soft embedding: out[r] = bf16( sum_k bf16( bf16(softmax(val[r])_k) * E[idx[r,k]] ) ) for flagged rows.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) soft_embed_rows_kernel(const float* __restrict__ val,
                                                              const int* __restrict__ idx,
                                                              const int* __restrict__ flag,
                                                              const __nv_bfloat16* __restrict__ E,
                                                              __nv_bfloat16* __restrict__ out, int K, int H,
                                                              long long ld_out) {
  const int r = blockIdx.x;
  if (flag != nullptr && flag[r] == 0) return;
  __shared__ float prob[128];
  __shared__ int id[128];
  if (threadIdx.x < 32) {
    float mx = -INFINITY;
    for (int k = threadIdx.x; k < K; k += 32) mx = fmaxf(mx, val[(size_t)r * K + k]);
    mx = warp_max(mx);
    float s = 0.f;
    for (int k = threadIdx.x; k < K; k += 32) s += __expf(val[(size_t)r * K + k] - mx);
    s = warp_sum(s);
    for (int k = threadIdx.x; k < K; k += 32) {
      prob[k] = bf16_round(__expf(val[(size_t)r * K + k] - mx) / s);
      id[k] = idx[(size_t)r * K + k];
    }
  }
  __syncthreads();
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // eight embedding rows in flight per thread; the accumulation order (k ascending) is unchanged
    for (int k0 = 0; k0 < K; k0 += 8) {
      uint4 e8[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        e8[u] = (k0 + u < K) ? reinterpret_cast<const uint4*>(E + (size_t)id[k0 + u] * H)[v] : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (k0 + u >= K) break;
        const __nv_bfloat162* eh = reinterpret_cast<const __nv_bfloat162*>(&e8[u]);
        const float pk = prob[k0 + u];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(eh[j]);
          acc[2 * j] += bf16_round(pk * f.x);
          acc[2 * j + 1] += bf16_round(pk * f.y);
        }
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<uint4*>(out + (size_t)r * ld_out)[v] = o;
  }
}

// ---------------------------------------------------------------------------------------------
// Sampler over a sorted top-k set (k <= 128): temperature -> softmax -> min_p -> (top_k is the set)
// -> top_p -> draw.  Only ratios of probabilities matter after each renormalisation, so working
// inside the top-k set is exact whenever top_k > 0.  One warp per row, lane 0 draws.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
// Uniform in (0, 1) for (row, step): a hash of the call's seed, so that a draw does not depend on which
// other rows share the batch.  `seed_dev` (optional, device memory) is mixed in when given: a captured
// graph can then be replayed with a new seed by writing that word.
__device__ __forceinline__ float draw_uniform(unsigned long long seed, const unsigned long long* seed_dev, int step,
                                              int r) {
  const uint64_t sd = seed_dev != nullptr ? (seed ^ splitmix64(*seed_dev)) : seed;
  const uint64_t h = splitmix64(sd ^ splitmix64(((uint64_t)(uint32_t)step << 32) | (uint32_t)r));
  return (float)((h >> 40) + 0.5) * (1.0f / 16777216.0f);
}

__global__ void sample_topk_kernel(const float* __restrict__ val, const int* __restrict__ idx, int* __restrict__ out,
                                   int rows, int K, float temperature, float top_p, float min_p,
                                   unsigned long long seed, const unsigned long long* __restrict__ seed_dev,
                                   const int* __restrict__ step) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const float* v = val + (size_t)r * K;
  const float inv_t = 1.0f / temperature;
  float w[128];
  float tot = 0.f;
  int n = 0;
  for (int k = 0; k < K; ++k) {
    const float e = __expf((v[k] - v[0]) * inv_t);
    if (min_p > 0.f && e < min_p) break;     // sorted: everything after is smaller too
    w[k] = e;
    tot += e;
    n = k + 1;
  }
  if (top_p < 1.0f) {
    float c = 0.f;
    int keep = n;
    for (int k = 0; k < n; ++k) {
      c += w[k] / tot;
      if (c > top_p) { keep = k + 1; break; }  // the token that crosses top_p is kept
    }
    n = keep;
    tot = 0.f;
    for (int k = 0; k < n; ++k) tot += w[k];
  }
  const float u = draw_uniform(seed, seed_dev, step ? step[r] : 0, r) * tot;
  float c = 0.f;
  int pick = n - 1;
  for (int k = 0; k < n; ++k) {
    c += w[k];
    if (u < c) { pick = k; break; }
  }
  out[r] = idx[(size_t)r * K + pick];
}

// ---------------------------------------------------------------------------------------------
// Sampler over the whole vocabulary, for top_k == 0 (no top-k filter) or top_k > 128, where the
// sorted-top-k route above does not apply.  Same filter order: temperature -> softmax -> min_p ->
// top_k -> top_p -> draw.  One CTA of 1024 threads per row.
//
// With e_i = exp((x_i - max) / T) every filter is a threshold on e_i, and because x is bf16 a
// threshold is one of 65536 order-preserving keys, found by a 16-step bisection:
//   min_p : e_i >= min_p (p_max = 1 / Z), no data pass;
//   top_k : the largest key t with count(key >= t) >= top_k (ties at t are all kept);
//   top_p : the largest key t with mass(key >= t) >= top_p * mass(kept so far) (the element that
//           crosses top_p is kept).
// Counts are integers and masses are summed in a fixed order, so the result is deterministic.  The
// draw is the inverse CDF over the kept elements in index order.
// ---------------------------------------------------------------------------------------------
constexpr int SFULL_THREADS = 1024;

struct SampleFullShared {
  float fsum[32];
  int isum[32];
  float total_f;
  int total_i;
  int pick;
};

// count and mass of the row's elements whose key is >= t (block-wide, every thread gets the result)
__device__ __forceinline__ void count_mass_ge(SampleFullShared& sh, const __nv_bfloat16* __restrict__ xr, int V,
                                              uint32_t t, float m, float inv_t, int* count, float* mass) {
  int c = 0;
  float s = 0.f;
  const int nvec = V / 8;
  for (int i = threadIdx.x; i < nvec; i += SFULL_THREADS) {
    const uint4 v = reinterpret_cast<const uint4*>(xr)[i];
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (order_key(e[j]) >= t) {
        c += 1;
        s += __expf((__bfloat162float(e[j]) - m) * inv_t);
      }
    }
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += SFULL_THREADS) {
    if (order_key(xr[i]) >= t) {
      c += 1;
      s += __expf((__bfloat162float(xr[i]) - m) * inv_t);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    c += __shfl_xor_sync(0xffffffffu, c, o);
    s += __shfl_xor_sync(0xffffffffu, s, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                       // the previous call's totals have been read by everyone
  if (lane == 0) { sh.isum[warp] = c; sh.fsum[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    c = sh.isum[lane];
    s = sh.fsum[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      c += __shfl_xor_sync(0xffffffffu, c, o);
      s += __shfl_xor_sync(0xffffffffu, s, o);
    }
    if (lane == 0) { sh.total_i = c; sh.total_f = s; }
  }
  __syncthreads();
  *count = sh.total_i;
  *mass = sh.total_f;
}

__global__ void __launch_bounds__(SFULL_THREADS) sample_full_kernel(const __nv_bfloat16* __restrict__ x,
                                                                    int* __restrict__ out, int V, long long ldx,
                                                                    float temperature, int top_k, float top_p,
                                                                    float min_p, unsigned long long seed,
                                                                    const unsigned long long* __restrict__ seed_dev,
                                                                    const int* __restrict__ step) {
  __shared__ SampleFullShared sh;
  const int r = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const __nv_bfloat16* xr = x + (size_t)r * ldx;
  // ---- max key ----
  uint32_t km = 0;
  for (int i = tid; i < V; i += SFULL_THREADS) km = max(km, order_key(xr[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) km = max(km, __shfl_xor_sync(0xffffffffu, km, o));
  if (lane == 0) sh.isum[warp] = (int)km;
  __syncthreads();
  km = 0;
  for (int w = 0; w < 32; ++w) km = max(km, (uint32_t)sh.isum[w]);
  const float m = key_value(km);
  const float inv_t = 1.0f / temperature;
  int cnt;
  float mass;
  // ---- min_p: smallest key whose e is still >= min_p (monotone in the key; no data pass) ----
  uint32_t cut = 0;
  if (min_p > 0.f) {
    uint32_t lo = 0, hi = km;              // e(hi) = 1 >= min_p holds for min_p <= 1
    while (lo < hi) {
      const uint32_t mid = (lo + hi) >> 1;
      const float xv = key_value(mid);
      const bool ok = (xv == xv) && __expf((xv - m) * inv_t) >= min_p;     // NaN keys never pass
      if (ok) hi = mid; else lo = mid + 1;
    }
    cut = lo;
  }
  // ---- top_k: largest key t >= cut with count(>= t) >= top_k ----
  if (top_k > 0 && top_k < V) {
    count_mass_ge(sh, xr, V, cut, m, inv_t, &cnt, &mass);
    if (cnt > top_k) {
      uint32_t lo = cut, hi = km;          // invariant: count(>= lo) >= top_k
      while (lo < hi) {
        const uint32_t mid = (lo + hi + 1) >> 1;
        count_mass_ge(sh, xr, V, mid, m, inv_t, &cnt, &mass);
        if (cnt >= top_k) lo = mid; else hi = mid - 1;
      }
      cut = lo;
    }
  }
  count_mass_ge(sh, xr, V, cut, m, inv_t, &cnt, &mass);
  // ---- top_p: largest key t >= cut with mass(>= t) >= top_p * mass(>= cut) ----
  if (top_p < 1.0f) {
    const float target = top_p * mass;
    uint32_t lo = cut, hi = km;            // invariant: mass(>= lo) >= target
    while (lo < hi) {
      const uint32_t mid = (lo + hi + 1) >> 1;
      float mm;
      count_mass_ge(sh, xr, V, mid, m, inv_t, &cnt, &mm);
      if (mm >= target) lo = mid; else hi = mid - 1;
    }
    cut = lo;
    count_mass_ge(sh, xr, V, cut, m, inv_t, &cnt, &mass);
  }
  // ---- draw: inverse CDF over the kept elements in index order ----
  const int chunk = (V + SFULL_THREADS - 1) / SFULL_THREADS;
  const int i0 = min(V, tid * chunk), i1 = min(V, i0 + chunk);
  float own = 0.f;
  for (int i = i0; i < i1; ++i)
    if (order_key(xr[i]) >= cut) own += __expf((__bfloat162float(xr[i]) - m) * inv_t);
  // block exclusive scan of `own` (fixed order)
  float incl = own;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  __syncthreads();
  if (lane == 31) sh.fsum[warp] = incl;
  if (tid == 0) sh.pick = -1;
  __syncthreads();
  float base = 0.f;
  for (int w = 0; w < warp; ++w) base += sh.fsum[w];
  float total = 0.f;
  for (int w = 0; w < 32; ++w) total += sh.fsum[w];
  const float excl = base + incl - own;
  const float u = draw_uniform(seed, seed_dev, step ? step[r] : 0, r) * total;
  if (own > 0.f && u >= excl && u < excl + own) {
    float c = excl;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      if (order_key(xr[i]) >= cut) {
        c += __expf((__bfloat162float(xr[i]) - m) * inv_t);
        pick = i;                          // last kept element seen: the answer if rounding leaves u >= c
        if (u < c) break;
      }
    }
    sh.pick = pick;
  }
  __syncthreads();
  if (tid == 0) {
    int pick = sh.pick;
    if (pick < 0) {                        // u fell on a boundary lost to rounding: take the arg-max
      for (int i = 0; i < V; ++i)
        if (order_key(xr[i]) == km) { pick = i; break; }
    }
    out[r] = pick;
  }
}

// ---------------------------------------------------------------------------------------------
// Scheduler state of the iteration-level decode engine (one entry per batch row).
// ---------------------------------------------------------------------------------------------
struct TickState {
  int* tok;        // token to feed at depth 0
  int* depth;      // depth of the pass this tick runs for the row
  int* pos;        // position id of the token being processed
  int* finished;   // row has produced EOS
  int* n_out;      // tokens emitted so far
  int* out_tokens; // [rows, max_new]
  int* iter_sum;   // passes spent on emitted tokens (for avg iteration count)
  int* cur_iters;  // passes spent on the token in flight
  int* slot;       // KV slot (page * page_size + off) of this tick's entry, in cache `depth`
  int* gate;       // depth > 0 (LoRA on)
  int* len[4];     // per-cache lengths
  int* page_table[4];
  int* free_stack[4];
  int* free_count[4];
  int max_pages[4];
  int n_caches, page_size, rows, max_new, eos, max_iter;
  int* status;
  unsigned long long* tokens_done;   // global counter of emitted tokens
};

// Start of a tick: allocate this tick's KV slot in cache `depth` and build the input embedding
// (embedding row of `tok` at depth 0, the soft embedding at depth >= 1).
__global__ void __launch_bounds__(128) tick_begin_kernel(const TickState s, const __nv_bfloat16* __restrict__ E,
                                                         const __nv_bfloat16* __restrict__ soft,
                                                         __nv_bfloat16* __restrict__ x_in, int H,
                                                         __nv_bfloat16* __restrict__ rope_cs, int hd, float log2_theta) {
  const int r = blockIdx.x;
  const int d = s.depth[r];
  if (rope_cs != nullptr) {
    // RoPE row of this tick's position (cos of the hd/2 frequencies, then sin): every layer's fused QKV
    // epilogue loads it instead of evaluating cos / sin itself
    const float posf = (float)s.pos[r];
    for (int j = threadIdx.x; j < hd / 2; j += blockDim.x) {
      const float ang = posf * exp2f(-(2.0f * (float)j / (float)hd) * log2_theta);
      rope_cs[(size_t)r * hd + j] = __float2bfloat16_rn(cosf(ang));
      rope_cs[(size_t)r * hd + hd / 2 + j] = __float2bfloat16_rn(sinf(ang));
    }
  }
  // a row that has finished (EOS or max_new tokens) keeps its slot in the batch but stops
  // consuming KV pages: it recomputes over its existing cache and its outputs are ignored
  const bool done = s.finished[r] != 0 || s.n_out[r] >= s.max_new;
  if (threadIdx.x == 0 && done) {
    s.slot[r] = -1;
    s.gate[r] = d > 0;
  }
  if (threadIdx.x == 0 && !done) {
    const int L = s.len[d][r];
    int page;
    if (L % s.page_size == 0) {
      const int pi = L / s.page_size;
      const int top = atomicSub(s.free_count[d], 1) - 1;
      if (top < 0 || pi >= s.max_pages[d]) {
        atomicAdd(s.free_count[d], 1);
        atomicCAS(s.status, 0, STATUS_BAD_INDEX);
        page = -1;
      } else {
        page = s.free_stack[d][top];
        s.page_table[d][(size_t)r * s.max_pages[d] + pi] = page;
      }
    } else {
      page = s.page_table[d][(size_t)r * s.max_pages[d] + L / s.page_size];
    }
    if (page >= 0) {
      s.slot[r] = page * s.page_size + L % s.page_size;
      s.len[d][r] = L + 1;
    } else {
      s.slot[r] = -1;
    }
    s.gate[r] = d > 0;
  }
  const uint4* src = (d == 0) ? reinterpret_cast<const uint4*>(E + (size_t)s.tok[r] * H)
                              : reinterpret_cast<const uint4*>(soft + (size_t)r * H);
  uint4* dst = reinterpret_cast<uint4*>(x_in + (size_t)r * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// Continue/stop decision.  override != nullptr: hard iff override[r, pos] > depth (scripted or
// seeded-Bernoulli hard-token mask); else hard iff sigmoid(z) > threshold.  need_soft marks rows
// that run another pass (they need top-k + soft embedding).
__global__ void decide_kernel(const float* __restrict__ z, float threshold, const signed char* __restrict__ override_,
                              int override_ld, const int* __restrict__ pos, const int* __restrict__ depth,
                              int max_iter, int* __restrict__ need_soft, int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int d = depth[r];
  bool hard;
  if (override_ != nullptr) {
    const int p = min(pos[r], override_ld - 1);
    hard = (int)override_[(size_t)r * override_ld + p] > d;
  } else {
    hard = z != nullptr && (1.0f / (1.0f + __expf(-z[r]))) > threshold;
  }
  need_soft[r] = (hard && d + 1 < max_iter) ? 1 : 0;
}

// Second half of the two-layer decider MLP: z[r] = bf16( sum_j bf16(silu(h[r, j])) * w2[j] + b2 ), where h
// is the first layer's bf16 output (bias already added inside the GEMM accumulation).  One warp per row.
__global__ void __launch_bounds__(128) decider_head_kernel(const __nv_bfloat16* __restrict__ h,
                                                           const __nv_bfloat16* __restrict__ w2,
                                                           const __nv_bfloat16* __restrict__ b2, float* __restrict__ z,
                                                           int rows, int inner, long long ldh) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const __nv_bfloat16* hr = h + (size_t)r * ldh;
  float acc = 0.f;
  for (int j = lane; j < inner; j += 32)
    acc += bf16_round(silu(__bfloat162float(hr[j]))) * __bfloat162float(w2[j]);
  acc = warp_sum(acc);
  if (lane == 0) z[r] = bf16_round(acc + (b2 != nullptr ? __bfloat162float(b2[0]) : 0.f));
}

// End of a tick: rows that iterate again go one level deeper; the others emit `next_tok`
// (never the EOS itself), return to depth 0 and advance their position.
__global__ void tick_end_kernel(const TickState s, const int* __restrict__ need_soft, const int* __restrict__ next_tok) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= s.rows) return;
  if (s.finished[r] != 0 || s.n_out[r] >= s.max_new) return;   // done rows are frozen
  s.cur_iters[r] += 1;
  if (need_soft[r]) {
    s.depth[r] += 1;
    return;
  }
  const int t = next_tok[r];
  if (!s.finished[r]) {
    if (t == s.eos) {
      s.finished[r] = 1;
    } else if (s.n_out[r] < s.max_new) {
      s.out_tokens[(size_t)r * s.max_new + s.n_out[r]] = t;
      s.n_out[r] += 1;
      s.iter_sum[r] += s.cur_iters[r];
      atomicAdd(s.tokens_done, 1ull);
    }
  }
  s.cur_iters[r] = 0;
  s.tok[r] = t;
  s.depth[r] = 0;
  s.pos[r] += 1;
}

}  // namespace tahb

using namespace tahb;

static int topk_launch(const void* x, const int* flag, float* out_val, int* out_idx, int rows, int V, int K,
                       long long ldx, int force_ordered, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K < 1 || K > 128 || K > V) return -1;
  topk_rows_kernel<<<rows, TOPK_THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), flag, out_val,
                                                      out_idx, V, K, ldx, force_ordered);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int tahb_topk_rows(const void* x, const int* flag, float* out_val, int* out_idx, int rows, int V, int K,
                              long long ldx, cudaStream_t stream) {
  return topk_launch(x, flag, out_val, out_idx, rows, V, K, ldx, 0, stream);
}

// Same result through the index-ordered path only (the fast path's fallback), for testing.
extern "C" int tahb_topk_rows_ordered(const void* x, const int* flag, float* out_val, int* out_idx, int rows, int V,
                                      int K, long long ldx, cudaStream_t stream) {
  return topk_launch(x, flag, out_val, out_idx, rows, V, K, ldx, 1, stream);
}

extern "C" int tahb_soft_embed_rows(const float* val, const int* idx, const int* flag, const void* E, void* out,
                                    int rows, int K, int H, long long ld_out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K > 128 || H % 8) return -1;
  soft_embed_rows_kernel<<<rows, 256, 0, stream>>>(val, idx, flag, reinterpret_cast<const __nv_bfloat16*>(E),
                                                   reinterpret_cast<__nv_bfloat16*>(out), K, H, ld_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int tahb_sample_topk(const float* val, const int* idx, int* out, int rows, int K, float temperature,
                                float top_p, float min_p, unsigned long long seed, const unsigned long long* seed_dev,
                                const int* step, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (K > 128 || temperature <= 0.f) return -1;
  sample_topk_kernel<<<(rows + 63) / 64, 64, 0, stream>>>(val, idx, out, rows, K, temperature, top_p, min_p, seed,
                                                          seed_dev, step);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// One token per row of bf16 logits x[rows, V] (row pitch ldx, a multiple of 8 elements with a 16-byte
// aligned base), sampled over the whole vocabulary; top_k <= 0 means no top-k filter.
extern "C" int tahb_sample_full(const void* x, int* out, int rows, int V, long long ldx, float temperature, int top_k,
                                float top_p, float min_p, unsigned long long seed,
                                const unsigned long long* seed_dev, const int* step, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (temperature <= 0.f || V <= 0 || (ldx % 8) || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
  sample_full_kernel<<<rows, SFULL_THREADS, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), out, V, ldx,
                                                         temperature, top_k, top_p, min_p, seed, seed_dev, step);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// The scheduler entry points take the state as an array of device pointers + ints, packed by the
// Python engine in the order of the TickState fields.
extern "C" int tahb_tick_begin(void* const* ptrs, const int* ints, const void* E, const void* soft, void* x_in, int H,
                               void* rope_cs, int hd, float theta, cudaStream_t stream);
extern "C" int tahb_tick_end(void* const* ptrs, const int* ints, const int* need_soft, const int* next_tok,
                             cudaStream_t stream);

static TickState unpack_state(void* const* p, const int* n) {
  TickState s;
  s.tok = (int*)p[0]; s.depth = (int*)p[1]; s.pos = (int*)p[2]; s.finished = (int*)p[3]; s.n_out = (int*)p[4];
  s.out_tokens = (int*)p[5]; s.iter_sum = (int*)p[6]; s.cur_iters = (int*)p[7]; s.slot = (int*)p[8];
  s.gate = (int*)p[9];
  for (int c = 0; c < 4; ++c) {
    s.len[c] = (int*)p[10 + c];
    s.page_table[c] = (int*)p[14 + c];
    s.free_stack[c] = (int*)p[18 + c];
    s.free_count[c] = (int*)p[22 + c];
    s.max_pages[c] = n[c];
  }
  s.status = (int*)p[26];
  s.tokens_done = (unsigned long long*)p[27];
  s.n_caches = n[4]; s.page_size = n[5]; s.rows = n[6]; s.max_new = n[7]; s.eos = n[8]; s.max_iter = n[9];
  return s;
}

extern "C" int tahb_tick_begin(void* const* ptrs, const int* ints, const void* E, const void* soft, void* x_in, int H,
                               void* rope_cs, int hd, float theta, cudaStream_t stream) {
  TickState s = unpack_state(ptrs, ints);
  if (s.rows <= 0) return 0;
  tick_begin_kernel<<<s.rows, 128, 0, stream>>>(s, reinterpret_cast<const __nv_bfloat16*>(E),
                                                reinterpret_cast<const __nv_bfloat16*>(soft),
                                                reinterpret_cast<__nv_bfloat16*>(x_in), H,
                                                reinterpret_cast<__nv_bfloat16*>(rope_cs), hd,
                                                theta > 0.f ? log2f(theta) : 0.f);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int tahb_decide(const float* z, float threshold, const signed char* override_, int override_ld,
                           const int* pos, const int* depth, int max_iter, int* need_soft, int rows,
                           cudaStream_t stream) {
  if (rows <= 0) return 0;
  decide_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(z, threshold, override_, override_ld, pos, depth, max_iter,
                                                        need_soft, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int tahb_decider_head(const void* h, const void* w2, const void* b2, float* z, int rows, int inner,
                                 long long ldh, cudaStream_t stream) {
  if (rows <= 0) return 0;
  decider_head_kernel<<<(rows + 3) / 4, 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(h),
                                                          reinterpret_cast<const __nv_bfloat16*>(w2),
                                                          reinterpret_cast<const __nv_bfloat16*>(b2), z, rows, inner, ldh);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int tahb_tick_end(void* const* ptrs, const int* ints, const int* need_soft, const int* next_tok,
                             cudaStream_t stream) {
  TickState s = unpack_state(ptrs, ints);
  if (s.rows <= 0) return 0;
  tick_end_kernel<<<(s.rows + 127) / 128, 128, 0, stream>>>(s, need_soft, next_tok);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
