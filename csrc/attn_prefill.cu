// Duo-causal attention forward for packed (varlen) passes on the 5th-generation tensor cores.
//
// One CTA handles a tile of up to 128 consecutive query tokens of ONE sequence and one query head.
// For each of up to three KV segments (depth-0 K/V, depth-1 K/V, ...) the tile walks the keys of its
// sequence in blocks of 64.  Two CTAs share an SM (112 KB of shared memory and 256 tensor-memory
// columns each), so one CTA's softmax overlaps the other's tensor-core work:
//
//     S = Q K^T          tcgen05.mma, Q and K K-major (head_dim contiguous), S in tensor memory
//     P = exp2(S - m)    256 threads, two per query row (32 key columns each), straight out of
//                        tensor memory; the duo-causal rule is the per-row bound
//                        key < count[segment][row]
//     O += P V           tcgen05.mma, P staged in shared memory (K-major), V consumed MN-major
//                        (head_dim contiguous, exactly as it lies in memory), O in tensor memory
//
// The running maximum is only refreshed when it grows by more than 8 (in log2 units), so the
// accumulator in tensor memory is rescaled rarely; the final division uses the matching row sums.
// No mask tensor exists.  K/V blocks arrive by TMA into a two-stage ring.  All waits are bounded.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = tensor-memory owner + MMA issuer,
// warps 2..9 = softmax / epilogue (warp w reads tensor-memory lanes 32*(w%4)..+31 = query rows;
// warps 2..5 take key columns 0..31 and the lower half of head_dim, warps 6..9 the rest).
#include <cuda.h>

#include "attn_common.cuh"

namespace tahb {

struct PrefillParams {
  __nv_bfloat16* out;            // [n_q, nq * HD]
  const int* tile_q0;            // [n_tiles] first packed query index of the tile
  const int* tile_qn;            // [n_tiles] number of query rows (<= 128)
  const int* seg_base[PF_MAX_SEG];   // [n_q] first KV row of the query's sequence in the segment
  const int* seg_count[PF_MAX_SEG];  // [n_q] number of visible KV rows of each query
  const int* seg_bound[PF_MAX_SEG];  // [n_q] non-decreasing upper bound of seg_count inside a sequence: the
                                     // bound of a tile's last row tells how many key blocks the tile walks
  int n_seg, nq, nkv;
  float scale_log2;
  float* lse;                    // optional [n_q, nq]: log2-domain log-sum-exp of the scaled scores (for backward)
  int* status;
};

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st1(uint32_t taddr, float v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(__float_as_uint(v)) : "memory");
}
__device__ __forceinline__ float tmem_ld1(uint32_t taddr) {
  uint32_t r;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r)::"memory");   // r is valid only after the wait
  return __uint_as_float(r);
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int HD>
struct PfCfg {
  static constexpr int BK = 64;                               // keys per block
  static constexpr int HALVES = HD / 64;                      // 64-element (128-byte) column groups
  static constexpr int QTILE = 128 * 64 * 2;                  // [128 rows][64] bf16 = 16 KiB
  static constexpr int KTILE = BK * 64 * 2;                   // [64 keys][64] bf16 = 8 KiB
  static constexpr int Q_BYTES = HALVES * QTILE;
  static constexpr int K_BYTES = HALVES * KTILE;
  static constexpr int V_BYTES = HALVES * KTILE;
  static constexpr int P_BYTES = 128 * BK * 2;                // 128 rows x 64 keys = 16 KiB
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
  static constexpr int NSTAGE = 2;
  // 112 KiB of tiles + barriers: two CTAs fit in an SM's 228 KiB (1 KiB is reserved per CTA), so the
  // two threads of a query row exchange their partial row maximum / sum through spare tensor-memory
  // columns of their lane instead of shared memory
  static constexpr int SMEM_BYTES = Q_BYTES + P_BYTES + NSTAGE * STAGE_BYTES + 128;
  static constexpr int XCOL = 64;                             // exchange columns 64..67 (parity, half): S is 0..63, O 128..
  static constexpr int TMEM_COLS = 256;                       // S: 64 columns (at 0), O: HD columns (at 128)
};
constexpr int PF_THREADS = 320;                               // 2 + 8 warps; two CTAs share an SM

template <int HD>
__global__ void __launch_bounds__(PF_THREADS, 2)
prefill_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k0,
                    const __grid_constant__ CUtensorMap tm_v0, const __grid_constant__ CUtensorMap tm_k1,
                    const __grid_constant__ CUtensorMap tm_v1, const __grid_constant__ CUtensorMap tm_k2,
                    const __grid_constant__ CUtensorMap tm_v2, const PrefillParams p) {
  using C = PfCfg<HD>;
  constexpr int BK = C::BK;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* p_s = q_s + C::Q_BYTES;
  uint8_t* kv_s = p_s + C::P_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + C::NSTAGE * C::STAGE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                 // [NSTAGE]
  uint64_t* kv_empty = kv_full + C::NSTAGE;     // [NSTAGE]
  uint64_t* s_full = kv_empty + C::NSTAGE;      // S = QK^T complete
  uint64_t* p_ready = s_full + 1;               // P written, O rescaled (256 arrivals)
  uint64_t* pv_done = p_ready + 1;              // O += PV complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, head = blockIdx.y;
  const int kvh = head / (p.nq / p.nkv);
  const int q0 = p.tile_q0[tile], qn = p.tile_qn[tile];
  if ((smem_u32(smem) & 1023u) != 0) {          // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(p.status, 0, STATUS_BAD_INDEX);
    return;
  }

  // key blocks per segment: the last row of the tile sees the most keys
  int seg_blocks[PF_MAX_SEG], seg_b0[PF_MAX_SEG], total_blocks = 0;
#pragma unroll
  for (int s = 0; s < PF_MAX_SEG; ++s) {
    seg_blocks[s] = 0;
    seg_b0[s] = 0;
    if (s < p.n_seg) {
      seg_b0[s] = p.seg_base[s][q0];
      seg_blocks[s] = (p.seg_bound[s][q0 + qn - 1] + BK - 1) / BK;
    }
    total_blocks += seg_blocks[s];
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < C::NSTAGE; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 256);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
      for (int h = 0; h < C::HALVES; ++h) tma_load_2d(q_s + h * C::QTILE, &tm_q, head * HD + h * 64, q0, q_full);
      int i = 0;
      for (int s = 0; s < p.n_seg; ++s) {
        const CUtensorMap* mk = s == 0 ? &tm_k0 : s == 1 ? &tm_k1 : &tm_k2;
        const CUtensorMap* mv = s == 0 ? &tm_v0 : s == 1 ? &tm_v1 : &tm_v2;
        for (int b = 0; b < seg_blocks[s]; ++b, ++i) {
          const int st = i % C::NSTAGE;
          const uint32_t ph = (i / C::NSTAGE) & 1;
          mbar_wait(&kv_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_STAGE_EMPTY);
          mbar_expect_tx(&kv_full[st], C::STAGE_BYTES);
          uint8_t* ks = kv_s + st * C::STAGE_BYTES;
          uint8_t* vs = ks + C::K_BYTES;
          const int y = seg_b0[s] + b * BK;
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) {
            tma_load_2d(ks + h * C::KTILE, mk, kvh * HD + h * 64, y, &kv_full[st]);
            tma_load_2d(vs + h * C::KTILE, mv, kvh * HD + h * 64, y, &kv_full[st]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BK);
      constexpr uint32_t idesc_o = umma_idesc_bf16_bmn(128, HD);
      mbar_wait(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      for (int i = 0; i < total_blocks; ++i) {
        const int st = i % C::NSTAGE;
        const uint32_t ph = (i / C::NSTAGE) & 1;
        mbar_wait(&kv_full[st], ph, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
        tc_fence_after();
        const uint32_t k_addr = smem_u32(kv_s + st * C::STAGE_BYTES);
        const uint32_t v_addr = k_addr + C::K_BYTES;
        // S = Q K^T : HD / 16 k-steps over head_dim
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t qo = (ks / 4) * C::QTILE + (ks % 4) * 32;
          const uint32_t ko = (ks / 4) * C::KTILE + (ks % 4) * 32;
          umma_bf16(tmem_s, umma_desc_sw128(q_addr + qo), umma_desc_sw128(k_addr + ko), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        // wait for P (and the rescaled O) of this block
        mbar_wait(p_ready, i & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
        tc_fence_after();
        // O += P V : BK / 16 k-steps over the keys; V is MN-major (head_dim contiguous)
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
          const uint64_t db = umma_desc_mn_sw128(v_addr + ks * 2048, C::KTILE);
          umma_bf16(tmem_o, umma_desc_sw128(p_addr + ks * 32), db, idesc_o, (i > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&kv_empty[st]);     // K/V stage may be refilled
        umma_commit(pv_done);           // P buffer and O are free for the next block
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax / epilogue: two threads per query row, 32 key columns each ----------------
    const int sw = warp - 2;                    // 0..7
    const int qd = warp & 3;                    // tensor-memory lane quadrant this warp may access
    const int half = sw >> 2;                   // which 32 of the 64 key columns / which half of head_dim
    const int row = qd * 32 + lane;
    const bool row_ok = row < qn;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sc = p.scale_log2;
    float m_ref = -INFINITY, l = 0.f;           // m_ref in scaled (log2) units
    int i = 0;
    for (int s = 0; s < p.n_seg; ++s) {
      const int cnt = row_ok ? p.seg_count[s][q0 + row] : 0;
      for (int b = 0; b < seg_blocks[s]; ++b, ++i) {
        mbar_wait(s_full, i & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
        tc_fence_after();
        const int valid = cnt - b * BK - half * 32;       // my columns [0, valid) of this block are visible
        float sv[32];
        tmem_ld32(tmem_s + lane_off + half * 32, sv);
        tmem_ld_wait();
        float mx = -INFINITY;
        if (__all_sync(0xffffffffu, valid >= 32)) {
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, sv[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            sv[j] = j < valid ? sv[j] : -INFINITY;
            mx = fmaxf(mx, sv[j]);
          }
        }
        // combine the two halves of the row
        const uint32_t xcol = tmem_base + lane_off + C::XCOL + (i & 1) * 2;
        tmem_st1(xcol + half, mx);
        tmem_st_wait();
        tc_fence_before();
        named_bar_sync(1, 256);
        tc_fence_after();
        mx = fmaxf(mx, tmem_ld1(xcol + (half ^ 1))) * sc;
        // lazy reference maximum: refresh only when it grew by more than 8 (a factor 256)
        const bool grow = mx > m_ref + 8.0f;
        const float m_new = grow ? mx : m_ref;
        const float f = (grow && m_ref != -INFINITY) ? exp2f(m_ref - m_new) : 1.0f;
        // the previous block's PV must be complete before P is overwritten or O rescaled
        if (i > 0) mbar_wait(pv_done, (i - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
        tc_fence_after();
        if (i > 0 && __any_sync(0xffffffffu, f != 1.0f)) {
#pragma unroll 1
          for (int c = 0; c < HD / 2; c += 32) {
            float o[32];
            tmem_ld32(tmem_o + lane_off + half * (HD / 2) + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= f;
            tmem_st32(tmem_o + lane_off + half * (HD / 2) + c, o);
          }
          tmem_st_wait();
        }
        l *= f;
        m_ref = m_new;
        const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref;   // all-masked so far: exp2(-inf) = 0
        // P = exp2(S * scale - m_ref) in bf16, written K-major with the 128-byte swizzle
        float psum0 = 0.f, psum1 = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {             // 4 chunks of 8 keys
          uint4 pk;
          __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float a = ex2_approx(fmaf(sv[c * 8 + 2 * j], sc, neg_m));
            const float bb = ex2_approx(fmaf(sv[c * 8 + 2 * j + 1], sc, neg_m));
            p2[j] = __floats2bfloat162_rn(a, bb);
            psum0 += a;
            psum1 += bb;
          }
          const int cc = half * 4 + c;
          *reinterpret_cast<uint4*>(p_s + row * 128 + ((cc ^ (row & 7)) << 4)) = pk;
        }
        l += psum0 + psum1;
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(p_ready);
      }
    }
    // epilogue: O / l, each thread writes its half of head_dim
    if (total_blocks > 0) mbar_wait(pv_done, (total_blocks - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
    tc_fence_after();
    {                                            // combine the two halves' row sums the same way
      const uint32_t xcol = tmem_base + lane_off + C::XCOL;
      named_bar_sync(1, 256);
      tmem_st1(xcol + half, l);
      tmem_st_wait();
      tc_fence_before();
      named_bar_sync(1, 256);
      tc_fence_after();
      l += tmem_ld1(xcol + (half ^ 1));
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    if (p.lse != nullptr && half == 0 && row_ok)
      p.lse[(size_t)(q0 + row) * p.nq + head] = l > 0.f ? m_ref + log2f(l) : -INFINITY;
    __nv_bfloat16* dst = p.out + ((size_t)(q0 + row) * p.nq + head) * HD + half * (HD / 2);
#pragma unroll 1
    for (int c = 0; c < HD / 2; c += 32) {
      float o[32];
      if (total_blocks > 0) {
        tmem_ld32(tmem_o + lane_off + half * (HD / 2) + c, o);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = 0.f;
      }
      if (row_ok) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 pk;
          __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int j = 0; j < 4; ++j) p2[j] = __floats2bfloat162_rn(o[v * 8 + 2 * j] * inv, o[v * 8 + 2 * j + 1] * inv);
          *reinterpret_cast<uint4*>(dst + c + v * 8) = pk;
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

}  // namespace tahb

using namespace tahb;

// q [n_q, nq*hd], out same; ks/vs[s] [n_kv[s], nkv*hd] (contiguous, bf16); tiles: tile_q0/tile_qn [n_tiles];
// bases/counts[s]: per query token.  Counts must be non-decreasing inside a tile.
extern "C" int tahb_prefill_attn(const void* q, void* out, void* const* ks, void* const* vs, const long long* n_kv,
                                 const int* const* bases, const int* const* counts, const int* const* bounds,
                                 int n_seg, const int* tile_q0,
                                 const int* tile_qn, int n_tiles, long long n_q, int nq, int nkv, int hd, float scale,
                                 float* lse, int* status, cudaStream_t stream) {
  if (n_tiles <= 0 || n_q <= 0) return 0;
  if (n_seg < 1 || n_seg > PF_MAX_SEG || (nq % nkv)) return -1;
  CUtensorMap mq, mk[PF_MAX_SEG], mv[PF_MAX_SEG];
  int rc;
  if ((rc = pf_make_map(&mq, q, n_q, (long long)nq * hd, 128u))) return rc;
  for (int s = 0; s < PF_MAX_SEG; ++s) {
    const int ss = s < n_seg ? s : 0;
    if ((rc = pf_make_map(&mk[s], ks[ss], n_kv[ss], (long long)nkv * hd, 64u))) return rc;
    if ((rc = pf_make_map(&mv[s], vs[ss], n_kv[ss], (long long)nkv * hd, 64u))) return rc;
  }
  PrefillParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.tile_q0 = tile_q0;
  p.tile_qn = tile_qn;
  for (int s = 0; s < PF_MAX_SEG; ++s) {
    const int ss = s < n_seg ? s : 0;
    p.seg_base[s] = bases[ss];
    p.seg_count[s] = counts[ss];
    p.seg_bound[s] = bounds[ss];
  }
  p.n_seg = n_seg; p.nq = nq; p.nkv = nkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse;
  p.status = status;
  dim3 grid(n_tiles, nq);
#define TAHB_PF(HD_)                                                                                              \
  {                                                                                                               \
    static bool configured = false;                                                                               \
    if (!configured) {                                                                                            \
      if (cudaFuncSetAttribute(prefill_attn_kernel<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                               PfCfg<HD_>::SMEM_BYTES) != cudaSuccess)                                            \
        return -10;                                                                                               \
      configured = true;                                                                                          \
    }                                                                                                             \
    prefill_attn_kernel<HD_><<<grid, PF_THREADS, PfCfg<HD_>::SMEM_BYTES, stream>>>(mq, mk[0], mv[0], mk[1], mv[1], mk[2], \
                                                                           mv[2], p);                             \
  }
  if (hd == 128) TAHB_PF(128)
  else if (hd == 64) TAHB_PF(64)
  else return -2;
#undef TAHB_PF
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
