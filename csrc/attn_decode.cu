// Paged-KV decode attention over all iteration caches of a row, and a plain varlen duo-causal
// attention used as the bring-up / reference path for packed prefill.
//
// Decode: one query token per row.  A row at iteration depth d attends every entry of its own
// sequence in caches 0..d (its own K/V was appended to cache d before this kernel runs), which
// is the duo-causal rule for the newest position.  The caches are paged; cache c of one layer is
//   [page][2 (K,V)][n_kv_heads][page_size][HD]  bf16
// with a page table pt[c][row][i] and a length len[c][row].
//
// Work split: grid (n_kv_heads, rows, n_split).  A CTA has 4 warps = 16 groups of 8 lanes; a
// group owns one KV token at a time and each lane HD/8 of its dims, so a token's K (or V) row is
// one contiguous 2*HD-byte read by 8 lanes.  All G = nq/nkv query heads that share the KV head are
// handled together, so K/V are read once.  Online softmax in base 2; groups are merged through
// shared memory; with n_split > 1 partial (m, l, acc) go to a workspace and a second kernel merges.
#include "common.cuh"

namespace tahb {

constexpr int MAX_CACHES = 4;

struct DecodeAttnParams {
  const __nv_bfloat16* q;       // [rows, nq, HD]
  __nv_bfloat16* out;           // [rows, nq, HD]
  const __nv_bfloat16* cache[MAX_CACHES];
  const int* page_table[MAX_CACHES];
  const int* len[MAX_CACHES];
  const int* depth;             // [rows] (nullptr: every row sees n_caches caches)
  float* ws;                    // [rows, nq, n_split, HD + 2]  (n_split > 1)
  int n_caches, rows, nq, nkv, page_size, max_pages[MAX_CACHES], n_split;
  float scale_log2;             // softmax scale * log2(e)
};

template <int HD, int G>
__global__ void __launch_bounds__(128) decode_attn_kernel(const DecodeAttnParams p) {
  constexpr int DPL = HD / 8;        // dims per lane
  constexpr int VEC = DPL / 8;       // uint4 loads per lane per row
  constexpr int U = 4;               // tokens per group per step
  const int kvh = blockIdx.x, row = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = warp * 4 + (lane >> 3);   // 0..15
  const int gl = lane & 7;

  int seg_len[MAX_CACHES];
  int total = 0;
  const int visible = p.depth ? min(p.depth[row] + 1, p.n_caches) : p.n_caches;
#pragma unroll
  for (int c = 0; c < MAX_CACHES; ++c) {
    seg_len[c] = (c < visible) ? p.len[c][row] : 0;
    total += seg_len[c];
  }
  const int chunk = (total + p.n_split - 1) / p.n_split;
  const int begin = split * chunk;
  const int end = min(total, begin + chunk);

  float qv[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = p.q + ((size_t)row * p.nq + kvh * G + g) * HD + gl * DPL;
#pragma unroll
    for (int i = 0; i < DPL; ++i) qv[g][i] = __bfloat162float(qp[i]) * p.scale_log2;
  }
  float m[G], l[G], acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
  }

  // The trip count is the same for every lane of the CTA (groups past the end run masked
  // iterations): the shuffles below name all 32 lanes, so no lane may leave the loop early.
  const int n_steps = (end - begin + 16 * U - 1) / (16 * U);
  for (int step = 0; step < n_steps; ++step) {
    const int base = begin + grp + step * 16 * U;
    uint4 kreg[U][VEC], vreg[U][VEC];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      int i = base + u * 16;
      ok[u] = i < end;
      if (!ok[u]) i = begin;   // any valid token; its contribution is masked below
      int c = 0;
#pragma unroll
      for (int cc = 0; cc < MAX_CACHES - 1; ++cc)
        if (c == cc && i >= seg_len[cc]) { i -= seg_len[cc]; c = cc + 1; }
      const int page = p.page_table[c][(size_t)row * p.max_pages[c] + i / p.page_size];
      const int off = i % p.page_size;
      const __nv_bfloat16* kp =
          p.cache[c] + ((((size_t)page * 2 + 0) * p.nkv + kvh) * p.page_size + off) * HD + gl * DPL;
      const __nv_bfloat16* vp = kp + (size_t)p.nkv * p.page_size * HD;
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        kreg[u][v] = reinterpret_cast<const uint4*>(kp)[v];
        vreg[u][v] = reinterpret_cast<const uint4*>(vp)[v];
      }
    }
    float s[U][G];
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int g = 0; g < G; ++g) s[u][g] = 0.f;
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        const __nv_bfloat162* kh = reinterpret_cast<const __nv_bfloat162*>(&kreg[u][v]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 kf = __bfloat1622float2(kh[j]);
#pragma unroll
          for (int g = 0; g < G; ++g) s[u][g] += qv[g][v * 8 + 2 * j] * kf.x + qv[g][v * 8 + 2 * j + 1] * kf.y;
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float t = s[u][g];
        t += __shfl_xor_sync(0xffffffffu, t, 1);
        t += __shfl_xor_sync(0xffffffffu, t, 2);
        t += __shfl_xor_sync(0xffffffffu, t, 4);
        s[u][g] = ok[u] ? t : -INFINITY;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = m[g];
#pragma unroll
      for (int u = 0; u < U; ++u) mx = fmaxf(mx, s[u][g]);
      const float corr = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mx);
      m[g] = mx;
      l[g] *= corr;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[g][i] *= corr;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float pw = ok[u] ? exp2f(s[u][g] - mx) : 0.f;
        l[g] += pw;
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vreg[u][v]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 vf = __bfloat1622float2(vh[j]);
            acc[g][v * 8 + 2 * j] += pw * vf.x;
            acc[g][v * 8 + 2 * j + 1] += pw * vf.y;
          }
        }
      }
    }
  }

  // merge the 16 groups through shared memory
  __shared__ float sm_m[16][G], sm_l[16][G];
  __shared__ float sm_acc[16][G][HD];
  if (gl == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) { sm_m[grp][g] = m[g]; sm_l[grp][g] = l[g]; }
  }
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int i = 0; i < DPL; ++i) sm_acc[grp][g][gl * DPL + i] = acc[g][i];
  __syncthreads();
  for (int idx = tid; idx < G * HD; idx += 128) {
    const int g = idx / HD, d = idx % HD;
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < 16; ++k) mx = fmaxf(mx, sm_m[k][g]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const float w = (sm_m[k][g] == -INFINITY) ? 0.f : exp2f(sm_m[k][g] - mx);
      num += w * sm_acc[k][g][d];
      den += w * sm_l[k][g];
    }
    const int head = kvh * G + g;
    if (p.n_split == 1) {
      p.out[((size_t)row * p.nq + head) * HD + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    } else {
      float* w = p.ws + (((size_t)row * p.nq + head) * p.n_split + split) * (HD + 2);
      w[d] = num;
      if (d == 0) { w[HD] = mx; w[HD + 1] = den; }
    }
  }
}

template <int HD>
__global__ void decode_attn_merge_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, int n_split) {
  const int rh = blockIdx.x;   // row * nq + head
  const float* w = ws + (size_t)rh * n_split * (HD + 2);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float mx = -INFINITY;
    for (int s = 0; s < n_split; ++s) mx = fmaxf(mx, w[s * (HD + 2) + HD]);
    float num = 0.f, den = 0.f;
    for (int s = 0; s < n_split; ++s) {
      const float ms = w[s * (HD + 2) + HD];
      const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - mx);
      num += f * w[s * (HD + 2) + d];
      den += f * w[s * (HD + 2) + HD + 1];
    }
    out[(size_t)rh * HD + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
  }
}

// ---------------------------------------------------------------------------------------------
// Plain varlen duo-causal attention over packed tokens (CUDA cores, one warp per (token, head)).
// Query token i attends, in up to three segments s, KV rows  seg_base[s][i] + j  for
// j < seg_count[s][i]  of the packed K/V tensors k[s]/v[s]  ([n, nkv, HD]).  Callers derive
// (base, count) from the duo-causal rule: segment 0 = depth-0 K/V of the same sequence up to the
// query's position, segment 1 = deeper K/V of the same sequence up to the query's own entry.
// ---------------------------------------------------------------------------------------------
struct VarlenAttnParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const __nv_bfloat16* k[3];
  const __nv_bfloat16* v[3];
  const int* seg_base[3];
  const int* seg_count[3];
  int n_q, nq, nkv, n_seg;
  float scale_log2;
};

template <int HD>
__global__ void __launch_bounds__(128) varlen_attn_naive_kernel(const VarlenAttnParams p) {
  constexpr int EPL = HD / 32;
  const int wg = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wg >= p.n_q * p.nq) return;
  const int t = wg / p.nq, h = wg % p.nq;
  const int kvh = h / (p.nq / p.nkv);
  float qv[EPL], acc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    qv[i] = __bfloat162float(p.q[((size_t)t * p.nq + h) * HD + lane * EPL + i]) * p.scale_log2;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int s = 0; s < p.n_seg; ++s) {
    const int base = p.seg_base[s][t], cnt = p.seg_count[s][t];
    for (int j = 0; j < cnt; ++j) {
      const size_t off = ((size_t)(base + j) * p.nkv + kvh) * HD + lane * EPL;
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) dot += qv[i] * __bfloat162float(p.k[s][off + i]);
      dot = warp_sum(dot);
      const float mx = fmaxf(m, dot);
      const float corr = (m == -INFINITY) ? 0.f : exp2f(m - mx);
      const float pw = exp2f(dot - mx);
      l = l * corr + pw;
#pragma unroll
      for (int i = 0; i < EPL; ++i) acc[i] = acc[i] * corr + pw * __bfloat162float(p.v[s][off + i]);
      m = mx;
    }
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i)
    p.out[((size_t)t * p.nq + h) * HD + lane * EPL + i] = __float2bfloat16_rn(l > 0.f ? acc[i] / l : 0.f);
}

template <int HD, int G>
static int launch_decode(const DecodeAttnParams& p, cudaStream_t stream) {
  dim3 grid(p.nkv, p.rows, p.n_split);
  decode_attn_kernel<HD, G><<<grid, 128, 0, stream>>>(p);
  if (p.n_split > 1) decode_attn_merge_kernel<HD><<<p.rows * p.nq, HD, 0, stream>>>(p.ws, p.out, p.n_split);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace tahb

using namespace tahb;

// Workspace floats needed by tahb_decode_attn when n_split > 1.
extern "C" long long tahb_decode_attn_ws_floats(int rows, int nq, int hd, int n_split) {
  return n_split > 1 ? (long long)rows * nq * n_split * (hd + 2) : 0;
}

extern "C" int tahb_decode_attn(const void* q, void* out, void* const* caches, const int* const* page_tables,
                                const int* const* lens, const int* max_pages, int n_caches, const int* depth,
                                int rows, int nq, int nkv, int hd, int page_size, float scale, int n_split,
                                float* ws, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (n_caches < 1 || n_caches > MAX_CACHES) return -1;
  if (n_split < 1) n_split = 1;
  if (n_split > 1 && ws == nullptr) return -4;
  DecodeAttnParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  for (int c = 0; c < MAX_CACHES; ++c) {
    const int cc = c < n_caches ? c : 0;
    p.cache[c] = reinterpret_cast<const __nv_bfloat16*>(caches[cc]);
    p.page_table[c] = page_tables[cc];
    p.len[c] = lens[cc];
    p.max_pages[c] = max_pages[cc];
  }
  p.depth = depth;
  p.ws = ws;
  p.n_caches = n_caches; p.rows = rows; p.nq = nq; p.nkv = nkv; p.page_size = page_size; p.n_split = n_split;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int G = nq / nkv;
  if (nq % nkv) return -2;
#define TAHB_DEC(HD_, G_) if (hd == HD_ && G == G_) return launch_decode<HD_, G_>(p, stream);
  TAHB_DEC(128, 1) TAHB_DEC(128, 2) TAHB_DEC(128, 4)
  TAHB_DEC(64, 1) TAHB_DEC(64, 2) TAHB_DEC(64, 4)
#undef TAHB_DEC
  return -2;
}

extern "C" int tahb_varlen_attn_naive(const void* q, void* out, void* const* ks, void* const* vs,
                                      const int* const* bases, const int* const* counts, int n_seg, int n_q, int nq,
                                      int nkv, int hd, float scale, cudaStream_t stream) {
  if (n_q <= 0) return 0;
  if (n_seg < 1 || n_seg > 3) return -1;
  VarlenAttnParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  for (int s = 0; s < 3; ++s) {
    const int ss = s < n_seg ? s : 0;
    p.k[s] = reinterpret_cast<const __nv_bfloat16*>(ks[ss]);
    p.v[s] = reinterpret_cast<const __nv_bfloat16*>(vs[ss]);
    p.seg_base[s] = bases[ss];
    p.seg_count[s] = counts[ss];
  }
  p.n_q = n_q; p.nq = nq; p.nkv = nkv; p.n_seg = n_seg;
  p.scale_log2 = scale * 1.4426950408889634f;
  const long long warps = (long long)n_q * nq;
  const int blocks = (int)((warps + 3) / 4);
  if (hd == 128) varlen_attn_naive_kernel<128><<<blocks, 128, 0, stream>>>(p);
  else if (hd == 64) varlen_attn_naive_kernel<64><<<blocks, 128, 0, stream>>>(p);
  else return -2;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
