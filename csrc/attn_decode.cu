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
#include "tah_b200_noalloc.h"

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
  int* status;                  // bounded-wait status word
  int n_caches, rows, nq, nkv, page_size, max_pages[MAX_CACHES], n_split;
  float scale_log2;             // softmax scale * log2(e)
};

// Geometry of the pipelined kernel: pages of 16 tokens; a pipeline stage holds STAGE_PAGES pages
// (K and V blocks of one KV head: 2 * 16 * HD bf16 each page), NSTAGE stages in flight per CTA.
constexpr int ATT_PAGE = 16;
constexpr int ATT_STAGE_PAGES = 2;
constexpr int ATT_NSTAGE = 3;

template <int HD>
struct AttCfg {
  static constexpr int BLK_ELEMS = ATT_PAGE * HD;                          // one K (or V) block of a page
  static constexpr int STAGE_ELEMS = ATT_STAGE_PAGES * 2 * BLK_ELEMS;
  static constexpr int STAGE_BYTES = STAGE_ELEMS * 2;
  static constexpr int SMEM_BYTES = ATT_NSTAGE * STAGE_BYTES + 256;
};

// Maps the i-th visible page of a row (pages of cache 0 first, then cache 1, ...) to its cache and
// to the page index inside that cache.
__device__ __forceinline__ void locate_page(int i, const int* seg_pages, int& c, int& local) {
  c = 0;
  local = i;
#pragma unroll
  for (int cc = 0; cc < MAX_CACHES - 1; ++cc)
    if (c == cc && local >= seg_pages[cc]) { local -= seg_pages[cc]; c = cc + 1; }
}

template <int HD, int G>
__global__ void __launch_bounds__(160, (HD * G <= 256) ? 4 : 2) decode_attn_kernel(const DecodeAttnParams p) {
  pdl_launch_dependents();
  pdl_wait();
  using C = AttCfg<HD>;
  constexpr int VEC = HD / 64;       // 16-byte chunks per lane per row: lane gl owns chunks gl, gl + 8, ...
  constexpr int DPL = VEC * 8;       // dims per lane
  extern __shared__ __align__(128) uint8_t att_smem[];
  __nv_bfloat16* stages = reinterpret_cast<__nv_bfloat16*>(att_smem);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(att_smem + ATT_NSTAGE * C::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + ATT_NSTAGE;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + ATT_NSTAGE);

  const int kvh = blockIdx.x, row = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  int seg_len[MAX_CACHES], seg_pages[MAX_CACHES];
  int total_pages = 0;
  const int visible = p.depth ? min(p.depth[row] + 1, p.n_caches) : p.n_caches;
#pragma unroll
  for (int c = 0; c < MAX_CACHES; ++c) {
    seg_len[c] = (c < visible) ? p.len[c][row] : 0;
    seg_pages[c] = (seg_len[c] + ATT_PAGE - 1) / ATT_PAGE;
    total_pages += seg_pages[c];
  }
  const int ppc = (total_pages + p.n_split - 1) / p.n_split;
  const int pb = split * ppc;
  const int pe = min(total_pages, pb + ppc);
  const int n_iter = pe > pb ? (pe - pb + ATT_STAGE_PAGES - 1) / ATT_STAGE_PAGES : 0;

  if (tid == 0) {
    for (int s = 0; s < ATT_NSTAGE; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);          // one arrival per consumer warp
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  float m[G], l[G], acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
  }
  const int grp = (warp & 3) * 4 + (lane >> 3);   // token slot inside a page (consumer warps only)
  const int gl = lane & 7;

  if (warp == 4) {
    // ---------------- producer: bulk copies of whole K / V page blocks ----------------
    if (lane == 0) {
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % ATT_NSTAGE;
        const uint32_t ph = (it / ATT_NSTAGE) & 1;
        mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_STAGE_EMPTY);
        const int first = pb + it * ATT_STAGE_PAGES;
        const int n_here = min(ATT_STAGE_PAGES, pe - first);
        mbar_expect_tx(&full_bar[s], n_here * 2 * C::BLK_ELEMS * 2);
        for (int u = 0; u < n_here; ++u) {
          int c, local;
          locate_page(first + u, seg_pages, c, local);
          const int page = p.page_table[c][(size_t)row * p.max_pages[c] + local];
          const __nv_bfloat16* kp = p.cache[c] + (((size_t)page * 2 + 0) * p.nkv + kvh) * C::BLK_ELEMS;
          const __nv_bfloat16* vp = kp + (size_t)p.nkv * C::BLK_ELEMS;
          __nv_bfloat16* dst = stages + (size_t)s * C::STAGE_ELEMS + (size_t)u * 2 * C::BLK_ELEMS;
          bulk_load(dst, kp, C::BLK_ELEMS * 2, &full_bar[s]);
          bulk_load(dst + C::BLK_ELEMS, vp, C::BLK_ELEMS * 2, &full_bar[s]);
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- consumers: 16 groups of 8 lanes, one token of each page per group ----------------
    float qv[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const __nv_bfloat16* qp = p.q + ((size_t)row * p.nq + kvh * G + g) * HD;
#pragma unroll
      for (int v = 0; v < VEC; ++v)
#pragma unroll
        for (int i = 0; i < 8; ++i) qv[g][v * 8 + i] = __bfloat162float(qp[(v * 8 + gl) * 8 + i]) * p.scale_log2;
    }
    for (int it = 0; it < n_iter; ++it) {
      const int s = it % ATT_NSTAGE;
      const uint32_t ph = (it / ATT_NSTAGE) & 1;
      mbar_wait(&full_bar[s], ph, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
      const __nv_bfloat16* st = stages + (size_t)s * C::STAGE_ELEMS;
      float sc[ATT_STAGE_PAGES][G];
      bool ok[ATT_STAGE_PAGES];
#pragma unroll
      for (int u = 0; u < ATT_STAGE_PAGES; ++u) {
        const int gi = pb + it * ATT_STAGE_PAGES + u;
        ok[u] = false;
        if (gi < pe) {
          int c, local;
          locate_page(gi, seg_pages, c, local);
          int len_c = seg_len[0];
#pragma unroll
          for (int cc = 1; cc < MAX_CACHES; ++cc) if (c == cc) len_c = seg_len[cc];
          ok[u] = local * ATT_PAGE + grp < len_c;
        }
        const __nv_bfloat16* kp = st + (size_t)u * 2 * C::BLK_ELEMS + grp * HD;
        float se[G], so[G];            // two partial sums per head: shorter dependent FMA chains
#pragma unroll
        for (int g = 0; g < G; ++g) { se[g] = 0.f; so[g] = 0.f; }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          const uint4 kr = *reinterpret_cast<const uint4*>(kp + (v * 8 + gl) * 8);
          const __nv_bfloat162* kh = reinterpret_cast<const __nv_bfloat162*>(&kr);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 kf = __bfloat1622float2(kh[j]);
#pragma unroll
            for (int g = 0; g < G; ++g) {
              se[g] = fmaf(qv[g][v * 8 + 2 * j], kf.x, se[g]);
              so[g] = fmaf(qv[g][v * 8 + 2 * j + 1], kf.y, so[g]);
            }
          }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float t = se[g] + so[g];
          t += __shfl_xor_sync(0xffffffffu, t, 1);
          t += __shfl_xor_sync(0xffffffffu, t, 2);
          t += __shfl_xor_sync(0xffffffffu, t, 4);
          sc[u][g] = ok[u] ? t : -INFINITY;
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float mx = m[g];
#pragma unroll
        for (int u = 0; u < ATT_STAGE_PAGES; ++u) mx = fmaxf(mx, sc[u][g]);
        const float corr = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mx);
        m[g] = mx;
        l[g] *= corr;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] *= corr;
      }
#pragma unroll
      for (int u = 0; u < ATT_STAGE_PAGES; ++u) {
        const __nv_bfloat16* vp = st + (size_t)u * 2 * C::BLK_ELEMS + C::BLK_ELEMS + grp * HD;
        float pw[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
          pw[g] = ok[u] ? exp2f(sc[u][g] - m[g]) : 0.f;
          l[g] += pw[g];
        }
        if (!ok[u]) continue;   // never touch stage memory that holds no page: it may contain NaN bits
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          const uint4 vr = *reinterpret_cast<const uint4*>(vp + (v * 8 + gl) * 8);
          const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vr);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 vf = __bfloat1622float2(vh[j]);
#pragma unroll
            for (int g = 0; g < G; ++g) {
              acc[g][v * 8 + 2 * j] += pw[g] * vf.x;
              acc[g][v * 8 + 2 * j + 1] += pw[g] * vf.y;
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
  }

  // merge the 16 groups through shared memory (the pipeline buffers are free now)
  __syncthreads();
  float* sm_m = reinterpret_cast<float*>(att_smem);          // [16][G]
  float* sm_l = sm_m + 16 * G;                               // [16][G]
  float* sm_acc = sm_l + 16 * G;                             // [16][G][HD]
  if (warp < 4) {
    if (gl == 0) {
#pragma unroll
      for (int g = 0; g < G; ++g) { sm_m[grp * G + g] = m[g]; sm_l[grp * G + g] = l[g]; }
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int v = 0; v < VEC; ++v)
#pragma unroll
        for (int i = 0; i < 8; ++i) sm_acc[(grp * G + g) * HD + (v * 8 + gl) * 8 + i] = acc[g][v * 8 + i];
  }
  __syncthreads();
  for (int idx = tid; idx < G * HD; idx += 160) {
    const int g = idx / HD, d = idx % HD;
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < 16; ++k) mx = fmaxf(mx, sm_m[k * G + g]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const float mk = sm_m[k * G + g];
      const float w = (mk == -INFINITY) ? 0.f : exp2f(mk - mx);
      num += w * sm_acc[(k * G + g) * HD + d];
      den += w * sm_l[k * G + g];
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
  pdl_launch_dependents();
  pdl_wait();
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
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(decode_attn_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             AttCfg<HD>::SMEM_BYTES) != cudaSuccess)
      return -10;
    configured = true;
  }
  cudaError_t e = launch_chain(decode_attn_kernel<HD, G>, grid, dim3(160), AttCfg<HD>::SMEM_BYTES, stream, p);
  if (e == cudaSuccess && p.n_split > 1)
    e = launch_chain(decode_attn_merge_kernel<HD>, dim3(p.rows * p.nq), dim3(HD), 0, stream, p.ws, p.out, p.n_split);
  return e == cudaSuccess ? 0 : -3;
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
                                float* ws, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (page_size != ATT_PAGE) return -5;
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
  p.status = status;
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

// ---------------------------------------------------------------------------------------------
// Allocation-free variant (declared and documented in tah_b200_noalloc.h).
// ---------------------------------------------------------------------------------------------
constexpr long long NOALLOC_WS_FLOATS = 1ll << 20;     // 4 MiB of scratch per GPU
static __device__ __align__(256) float g_noalloc_ws[NOALLOC_WS_FLOATS];

extern "C" long long tahb_decode_attn_noalloc_capacity(void) { return NOALLOC_WS_FLOATS; }

// In host code `g_noalloc_ws` is only a handle for the symbol, not an address a kernel can use:
// the device address is looked up once per device and cached here.
static float* noalloc_ws_for_current_device(void) {
  constexpr int MAX_DEVICES = 64;
  static float* cached[MAX_DEVICES] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
  if (cached[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_ws) != cudaSuccess) return nullptr;
    cached[dev] = ptr;
  }
  return cached[dev];
}

extern "C" int tahb_decode_attn_noalloc(const void* q, void* out, void* const* caches,
                                        const int* const* page_tables, const int* const* lens,
                                        const int* max_pages, int n_caches, const int* depth, int rows, int nq,
                                        int nkv, int hd, int page_size, float scale, int n_split, int* status,
                                        cudaStream_t stream) {
  if (n_split < 1) n_split = 1;
  const long long need = tahb_decode_attn_ws_floats(rows, nq, hd, n_split);
  if (need > NOALLOC_WS_FLOATS) return -7;     // request exceeds the built-in scratch area
  float* ws = noalloc_ws_for_current_device();
  if (ws == nullptr) return -8;
  return tahb_decode_attn(q, out, caches, page_tables, lens, max_pages, n_caches, depth, rows, nq, nkv, hd,
                          page_size, scale, n_split, ws, status, stream);
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
