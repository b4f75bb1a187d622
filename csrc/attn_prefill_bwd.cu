// Backward of the packed duo-causal attention (attn_prefill.cu) on the tensor cores.
//
// With P = exp2(S * c - lse) (c = scale * log2 e, lse from the forward), D = rowsum(dO * O):
//     dP = dO V^T,   dS = P * (dP - D) * scale,   dQ = dS K,   dK = dS^T Q,   dV = P^T dO.
//
// Two kernels, both recompute S and dP per block with tcgen05.mma from TMA-staged tiles:
//
//   attn_bwd_dq_kernel   one CTA per (128-query tile, query head), the forward's loop over 64-key
//                        blocks of up to three KV segments.  S and dP in tensor memory, dS written to
//                        shared memory (K-major) by 256 threads, dQ += dS K with K consumed MN-major.
//                        Two CTAs per SM.
//   attn_bwd_dkv_kernel  one CTA per (128-key block of one sequence and segment, KV head): the keys sit
//                        on the tensor-memory lanes.  Loop over the 64-query sub-tiles that can see the
//                        block and over the query heads of the KV group: S^T = K Q^T, dP^T = V dO^T,
//                        P^T and dS^T to shared memory, dV += P^T dO and dK += dS^T Q with the same
//                        Q / dO tiles consumed MN-major.  dK and dV accumulate in tensor memory over the
//                        whole loop (4 x 128 columns with the two score tiles).
//
// The duo-causal rule is the per-query bound key_index < count[segment][query]; no mask tensor.
// All waits are bounded (common.cuh).
#include <cuda.h>

#include "attn_common.cuh"

namespace tahb {

struct AttnBwdParams {
  const int* tile_q0;                 // dQ kernel: query tiles as in the forward
  const int* tile_qn;
  const int* seg_base[PF_MAX_SEG];    // [n_q]
  const int* seg_count[PF_MAX_SEG];   // [n_q]
  const int* seg_bound[PF_MAX_SEG];   // [n_q] non-decreasing upper bound of seg_count (tiling decisions)
  const float* lse;                   // [n_q, nq] base-2 log-sum-exp from the forward
  const float* dsum;                  // [n_q, nq] rowsum(dO * O)
  __nv_bfloat16* dq;                  // [n_q, nq * HD]
  int n_seg, nq, nkv;
  float scale_log2, scale;
  // dK/dV kernel work items
  const int* kv_row0;                 // [n_items] first row of the key block in the segment's K/V matrix
  const int* kv_nkeys;                // [n_items] keys in the block (<= 128)
  const int* kv_kidx0;                // [n_items] index of the block's first key inside its sequence's segment
  const int* kv_qa;                   // [n_items] first packed query row of the sequence
  const int* kv_qb;                   // [n_items] one past its last query row
  const int* kv_count;                // [n_q] visible-key counts of this segment (= seg_count[s])
  const int* kv_bound;                // [n_q] its non-decreasing upper bound (which sub-tiles to skip)
  __nv_bfloat16* dk;                  // [n_kv, nkv * HD]
  __nv_bfloat16* dv;
  int* status;
};

template <int HD>
struct BwdQCfg {
  static constexpr int BK = 64;
  static constexpr int HALVES = HD / 64;
  static constexpr int QTILE = 128 * 64 * 2;
  static constexpr int KTILE = BK * 64 * 2;
  static constexpr int Q_BYTES = HALVES * QTILE;               // Q and dO tiles
  static constexpr int K_BYTES = HALVES * KTILE;               // K and V blocks
  static constexpr int DS_BYTES = 128 * BK * 2;
  static constexpr int SMEM_BYTES = 2 * Q_BYTES + DS_BYTES + 2 * K_BYTES + 128;
  static constexpr int TMEM_COLS = 256;                        // S at 0, dP at 64, dQ at 128
};
constexpr int BWD_THREADS = 320;

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 2)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                   const __grid_constant__ CUtensorMap tm_k0, const __grid_constant__ CUtensorMap tm_v0,
                   const __grid_constant__ CUtensorMap tm_k1, const __grid_constant__ CUtensorMap tm_v1,
                   const __grid_constant__ CUtensorMap tm_k2, const __grid_constant__ CUtensorMap tm_v2,
                   const AttnBwdParams p) {
  using C = BwdQCfg<HD>;
  constexpr int BK = C::BK;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* do_s = q_s + C::Q_BYTES;
  uint8_t* ds_s = do_s + C::Q_BYTES;
  uint8_t* k_s = ds_s + C::DS_BYTES;
  uint8_t* v_s = k_s + C::K_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + C::K_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 2;
  uint64_t* s_full = bars + 3;
  uint64_t* ds_ready = bars + 4;
  uint64_t* dq_done = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, head = blockIdx.y;
  const int kvh = head / (p.nq / p.nkv);
  const int q0 = p.tile_q0[tile], qn = p.tile_qn[tile];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, STATUS_BAD_INDEX);
    return;
  }
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
    mbar_init(kv_full, 1);
    mbar_init(kv_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(ds_ready, 256);
    mbar_init(dq_done, 1);
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
  const uint32_t tmem_s = tmem_base, tmem_dp = tmem_base + 64, tmem_dq = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * C::Q_BYTES);
#pragma unroll
      for (int h = 0; h < C::HALVES; ++h) {
        tma_load_2d(q_s + h * C::QTILE, &tm_q, head * HD + h * 64, q0, q_full);
        tma_load_2d(do_s + h * C::QTILE, &tm_do, head * HD + h * 64, q0, q_full);
      }
      int i = 0;
      for (int s = 0; s < p.n_seg; ++s) {
        const CUtensorMap* mk = s == 0 ? &tm_k0 : s == 1 ? &tm_k1 : &tm_k2;
        const CUtensorMap* mv = s == 0 ? &tm_v0 : s == 1 ? &tm_v1 : &tm_v2;
        for (int b = 0; b < seg_blocks[s]; ++b, ++i) {
          mbar_wait(kv_empty, (i & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_STAGE_EMPTY);
          mbar_expect_tx(kv_full, 2 * C::K_BYTES);
          const int y = seg_b0[s] + b * BK;
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) {
            tma_load_2d(k_s + h * C::KTILE, mk, kvh * HD + h * 64, y, kv_full);
            tma_load_2d(v_s + h * C::KTILE, mv, kvh * HD + h * 64, y, kv_full);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BK);
      constexpr uint32_t idesc_q = umma_idesc_bf16_bmn(128, HD);
      mbar_wait(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
      const uint32_t q_addr = smem_u32(q_s), do_addr = smem_u32(do_s), ds_addr = smem_u32(ds_s);
      const uint32_t k_addr = smem_u32(k_s), v_addr = smem_u32(v_s);
      for (int i = 0; i < total_blocks; ++i) {
        mbar_wait(kv_full, i & 1, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {      // S = Q K^T and dP = dO V^T over head_dim
          const uint32_t qo = (ks / 4) * C::QTILE + (ks % 4) * 32;
          const uint32_t ko = (ks / 4) * C::KTILE + (ks % 4) * 32;
          umma_bf16(tmem_s, umma_desc_sw128(q_addr + qo), umma_desc_sw128(k_addr + ko), idesc_s, ks > 0 ? 1u : 0u);
          umma_bf16(tmem_dp, umma_desc_sw128(do_addr + qo), umma_desc_sw128(v_addr + ko), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        mbar_wait(ds_ready, i & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {      // dQ += dS K, K consumed MN-major
          const uint64_t db = umma_desc_mn_sw128(k_addr + ks * 2048, C::KTILE);
          umma_bf16(tmem_dq, umma_desc_sw128(ds_addr + ks * 32), db, idesc_q, (i > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(kv_empty);
        umma_commit(dq_done);
      }
    }
    __syncwarp();
  } else {
    const int sw = warp - 2;
    const int qd = warp & 3;
    const int half = sw >> 2;
    const int row = qd * 32 + lane;
    const bool row_ok = row < qn;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sc = p.scale_log2;
    float lse = row_ok ? p.lse[(size_t)(q0 + row) * p.nq + head] : -INFINITY;
    const float dsum_s = (row_ok ? p.dsum[(size_t)(q0 + row) * p.nq + head] : 0.f) * p.scale;   // D * scale
    const float neg_lse = (lse == -INFINITY) ? 0.f : -lse;
    int i = 0;
    for (int s = 0; s < p.n_seg; ++s) {
      const int cnt = row_ok ? p.seg_count[s][q0 + row] : 0;
      for (int b = 0; b < seg_blocks[s]; ++b, ++i) {
        mbar_wait(s_full, i & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
        tc_fence_after();
        const int valid = cnt - b * BK - half * 32;
        float sv[32], dp[32];
        tmem_ld32(tmem_s + lane_off + half * 32, sv);
        tmem_ld32(tmem_dp + lane_off + half * 32, dp);
        tmem_ld_wait();
        if (i > 0) mbar_wait(dq_done, (i - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
        const bool all_visible = __all_sync(0xffffffffu, valid >= 32);    // no masking inside this block
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 pk;
          __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c0 = c * 8 + 2 * j;
            float pa = ex2_approx(fmaf(sv[c0], sc, neg_lse));
            float pb = ex2_approx(fmaf(sv[c0 + 1], sc, neg_lse));
            if (!all_visible) {
              pa = c0 < valid ? pa : 0.f;
              pb = c0 + 1 < valid ? pb : 0.f;
            }
            p2[j] = __floats2bfloat162_rn(pa * fmaf(dp[c0], p.scale, -dsum_s), pb * fmaf(dp[c0 + 1], p.scale, -dsum_s));
          }
          const int cc = half * 4 + c;
          *reinterpret_cast<uint4*>(ds_s + row * 128 + ((cc ^ (row & 7)) << 4)) = pk;
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(ds_ready);
      }
    }
    if (total_blocks > 0) mbar_wait(dq_done, (total_blocks - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
    tc_fence_after();
    __nv_bfloat16* dst = p.dq + ((size_t)(q0 + row) * p.nq + head) * HD + half * (HD / 2);
#pragma unroll 1
    for (int c = 0; c < HD / 2; c += 32) {
      float o[32];
      if (total_blocks > 0) {
        tmem_ld32(tmem_dq + lane_off + half * (HD / 2) + c, o);
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
          for (int j = 0; j < 4; ++j) p2[j] = __floats2bfloat162_rn(o[v * 8 + 2 * j], o[v * 8 + 2 * j + 1]);
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

// ---------------------------------------------------------------------------------------------
// dK / dV
// ---------------------------------------------------------------------------------------------
template <int HD>
struct BwdKVCfg {
  static constexpr int BQ = 64;                                // queries per sub-tile
  static constexpr int HALVES = HD / 64;
  static constexpr int KTILE = 128 * 64 * 2;                   // [128 keys][64] = 16 KiB
  static constexpr int QTILE = BQ * 64 * 2;                    // [64 queries][64] = 8 KiB
  static constexpr int K_BYTES = HALVES * KTILE;               // K and V blocks (resident)
  static constexpr int Q_BYTES = HALVES * QTILE;               // Q and dO sub-tiles
  static constexpr int STAGE_BYTES = 2 * Q_BYTES;
  static constexpr int NSTAGE = 2;
  static constexpr int PT_BYTES = 128 * BQ * 2;                // P^T and dS^T tiles
  static constexpr int META_BYTES = 2 * 3 * BQ * 4;            // [2 buffers][lse | dsum | count][64 queries]
  static constexpr int SMEM_BYTES = 2 * K_BYTES + NSTAGE * STAGE_BYTES + 2 * PT_BYTES + META_BYTES + 128;
  static constexpr int TMEM_COLS = 512;                        // scores at 0 / 384 (S^T, dP^T), dK at 128, dV at 256
};

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const AttnBwdParams p) {
  using C = BwdKVCfg<HD>;
  constexpr int BQ = C::BQ;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* k_s = smem;
  uint8_t* v_s = k_s + C::K_BYTES;
  uint8_t* qd_s = v_s + C::K_BYTES;                             // stages: [Q | dO]
  uint8_t* pt_s = qd_s + C::NSTAGE * C::STAGE_BYTES;
  uint8_t* dst_s = pt_s + C::PT_BYTES;
  float* meta_s = reinterpret_cast<float*>(dst_s + C::PT_BYTES);  // per-query lse, dsum, count of the sub-tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(dst_s + C::PT_BYTES + C::META_BYTES);
  uint64_t* kv_full = bars;
  uint64_t* qd_full = bars + 1;                                 // [NSTAGE]
  uint64_t* qd_empty = qd_full + C::NSTAGE;                     // [NSTAGE]
  uint64_t* s_full = qd_empty + C::NSTAGE;                      // [2]: one per score buffer
  uint64_t* p_ready = s_full + 2;
  uint64_t* acc_done = p_ready + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x, kvh = blockIdx.y;
  const int G = p.nq / p.nkv;
  const int row0 = p.kv_row0[item], nkeys = p.kv_nkeys[item], kidx0 = p.kv_kidx0[item];
  const int qa = p.kv_qa[item], qb = p.kv_qb[item];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, STATUS_BAD_INDEX);
    return;
  }
  // first 64-query sub-tile with a row that sees this block: counts are non-decreasing over the
  // sequence's rows, so the sub-tiles that see nothing form a prefix (binary search on the last row)
  const int n_sub = (qb - qa + BQ - 1) / BQ;
  int lo = 0, hi = n_sub;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    const int last = min(qb, qa + (mid + 1) * BQ) - 1;
    if (p.kv_bound[last] > kidx0) hi = mid; else lo = mid + 1;
  }
  const int sub0 = lo;
  const int n_iter = (n_sub - sub0) * G;                        // (sub-tile, head of the group) pairs

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < C::NSTAGE; ++s) { mbar_init(&qd_full[s], 1); mbar_init(&qd_empty[s], 1); }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(p_ready, 256);
    mbar_init(acc_done, 1);
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
  // two score buffers (S^T at +0, dP^T at +64 inside each) so that the scores of iteration it+1 are
  // computed while the threads still work on iteration it
  const uint32_t tmem_sc[2] = {tmem_base, tmem_base + 384};
  const uint32_t tmem_dk = tmem_base + 128, tmem_dv = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * C::K_BYTES);
#pragma unroll
      for (int h = 0; h < C::HALVES; ++h) {
        tma_load_2d(k_s + h * C::KTILE, &tm_k, kvh * HD + h * 64, row0, kv_full);
        tma_load_2d(v_s + h * C::KTILE, &tm_v, kvh * HD + h * 64, row0, kv_full);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % C::NSTAGE;
        const uint32_t ph = (it / C::NSTAGE) & 1;
        const int sub = sub0 + it / G, head = kvh * G + it % G;
        mbar_wait(&qd_empty[st], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_STAGE_EMPTY);
        mbar_expect_tx(&qd_full[st], C::STAGE_BYTES);
        uint8_t* qs = qd_s + st * C::STAGE_BYTES;
        uint8_t* ds = qs + C::Q_BYTES;
        const int y = qa + sub * BQ;
#pragma unroll
        for (int h = 0; h < C::HALVES; ++h) {
          tma_load_2d(qs + h * C::QTILE, &tm_q, head * HD + h * 64, y, &qd_full[st]);
          tma_load_2d(ds + h * C::QTILE, &tm_do, head * HD + h * 64, y, &qd_full[st]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BQ);            // S^T, dP^T: 128 keys x 64 queries
      constexpr uint32_t idesc_a = umma_idesc_bf16_bmn(128, HD);        // dK, dV: 128 keys x head_dim
      mbar_wait(kv_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
      const uint32_t k_addr = smem_u32(k_s), v_addr = smem_u32(v_s);
      const uint32_t pt_addr = smem_u32(pt_s), dst_addr = smem_u32(dst_s);
      // scores of iteration `j`: S^T = K Q^T, dP^T = V dO^T over head_dim, into score buffer j & 1
      auto issue_scores = [&](int j) {
        const int st = j % C::NSTAGE;
        mbar_wait(&qd_full[st], (j / C::NSTAGE) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
        tc_fence_after();
        const uint32_t q_addr = smem_u32(qd_s + st * C::STAGE_BYTES);
        const uint32_t do_addr = q_addr + C::Q_BYTES;
        const uint32_t t_s = tmem_sc[j & 1];
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t ko = (ks / 4) * C::KTILE + (ks % 4) * 32;
          const uint32_t qo = (ks / 4) * C::QTILE + (ks % 4) * 32;
          umma_bf16(t_s, umma_desc_sw128(k_addr + ko), umma_desc_sw128(q_addr + qo), idesc_s, ks > 0 ? 1u : 0u);
          umma_bf16(t_s + 64, umma_desc_sw128(v_addr + ko), umma_desc_sw128(do_addr + qo), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
      };
      if (n_iter > 0) issue_scores(0);
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % C::NSTAGE;
        const uint32_t q_addr = smem_u32(qd_s + st * C::STAGE_BYTES);
        const uint32_t do_addr = q_addr + C::Q_BYTES;
        // the other score buffer was last read for iteration it-1, whose p_ready has been waited for
        if (it + 1 < n_iter) issue_scores(it + 1);
        mbar_wait(p_ready, it & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BQ / 16; ++ks) {      // dV += P^T dO, dK += dS^T Q over the 64 queries
          const uint64_t b_do = umma_desc_mn_sw128(do_addr + ks * 2048, C::QTILE);
          const uint64_t b_q = umma_desc_mn_sw128(q_addr + ks * 2048, C::QTILE);
          const uint32_t acc = (it > 0 || ks > 0) ? 1u : 0u;
          umma_bf16(tmem_dv, umma_desc_sw128(pt_addr + ks * 32), b_do, idesc_a, acc);
          umma_bf16(tmem_dk, umma_desc_sw128(dst_addr + ks * 32), b_q, idesc_a, acc);
        }
        umma_commit(&qd_empty[st]);
        umma_commit(acc_done);
      }
    }
    __syncwarp();
  } else {
    const int sw = warp - 2;
    const int qd = warp & 3;
    const int half = sw >> 2;                      // which 32 of the 64 query columns / half of head_dim
    const int row = qd * 32 + lane;                // key row of the block
    const bool key_ok = row < nkeys;
    const int kidx = kidx0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(qd * 32) << 16;
    const float sc = p.scale_log2;
    // Per-query lse, dsum and visible-key count of a sub-tile are fetched by 64 threads (one query
    // each, in parallel) one iteration ahead and handed over through shared memory; every thread then
    // reads its 32 columns' values with broadcast vector loads.
    const int mt = threadIdx.x - 64;               // 0..255 among the math threads
    float m_l = 0.f, m_d = 0.f;
    int m_c = 0;
    auto fetch_meta = [&](int j) {
      m_l = 0.f; m_d = 0.f; m_c = 0;
      if (mt < BQ && j < n_iter) {
        const int qr = qa + (sub0 + j / G) * BQ + mt;
        if (qr < qb) {
          const int hh = kvh * G + j % G;
          m_c = p.kv_count[qr];
          m_l = -p.lse[(size_t)qr * p.nq + hh];               // stored negated / pre-scaled for the inner loop
          m_d = p.dsum[(size_t)qr * p.nq + hh] * p.scale;
        }
      }
    };
    auto store_meta = [&](int j) {
      if (mt < BQ) {
        float* mb = meta_s + (j & 1) * 3 * BQ;
        mb[mt] = m_l;
        mb[BQ + mt] = m_d;
        reinterpret_cast<int*>(mb)[2 * BQ + mt] = m_c;
      }
    };
    fetch_meta(0);
    store_meta(0);
    named_bar_sync(2, 256);
    for (int it = 0; it < n_iter; ++it) {
      fetch_meta(it + 1);                          // in flight while this iteration computes
      const float* mb = meta_s + (it & 1) * 3 * BQ + half * 32;
      mbar_wait(&s_full[it & 1], (it >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
      tc_fence_after();
      float sv[32], dp[32];
      tmem_ld32(tmem_sc[it & 1] + lane_off + half * 32, sv);
      tmem_ld32(tmem_sc[it & 1] + 64 + lane_off + half * 32, dp);
      tmem_ld_wait();
      if (it > 0) mbar_wait(acc_done, (it - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
      // every key of the block visible to every query of this thread's 32 columns: no masking needed.  The
      // columns' counts are the same for all lanes of the warp, so the test is warp-uniform.
      int cmin = 0x7fffffff;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int4 cv4 = *reinterpret_cast<const int4*>(mb + 2 * BQ + c * 4);
        cmin = min(cmin, min(min(cv4.x, cv4.y), min(cv4.z, cv4.w)));
      }
      const bool all_visible = nkeys == 128 && kidx0 + 127 < cmin;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 pk, dk;
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
        __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(&dk);
        float lv[8], dv8[8];
        int cv[8];
        *reinterpret_cast<float4*>(lv) = *reinterpret_cast<const float4*>(mb + c * 8);
        *reinterpret_cast<float4*>(lv + 4) = *reinterpret_cast<const float4*>(mb + c * 8 + 4);
        *reinterpret_cast<float4*>(dv8) = *reinterpret_cast<const float4*>(mb + BQ + c * 8);
        *reinterpret_cast<float4*>(dv8 + 4) = *reinterpret_cast<const float4*>(mb + BQ + c * 8 + 4);
        *reinterpret_cast<int4*>(cv) = *reinterpret_cast<const int4*>(mb + 2 * BQ + c * 8);
        *reinterpret_cast<int4*>(cv + 4) = *reinterpret_cast<const int4*>(mb + 2 * BQ + c * 8 + 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float pv[2], dsv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int cl = 2 * j + e, col = c * 8 + cl;
            float pe = ex2_approx(fmaf(sv[col], sc, lv[cl]));
            if (!all_visible) pe = (key_ok && kidx < cv[cl]) ? pe : 0.f;
            pv[e] = pe;
            dsv[e] = pe * fmaf(dp[col], p.scale, -dv8[cl]);
          }
          p2[j] = __floats2bfloat162_rn(pv[0], pv[1]);
          d2[j] = __floats2bfloat162_rn(dsv[0], dsv[1]);
        }
        const int cc = half * 4 + c;
        const int off = row * 128 + ((cc ^ (row & 7)) << 4);
        *reinterpret_cast<uint4*>(pt_s + off) = pk;
        *reinterpret_cast<uint4*>(dst_s + off) = dk;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
      store_meta(it + 1);
      named_bar_sync(2, 256);                      // next iteration's values visible; this buffer free again
    }
    if (n_iter > 0) mbar_wait(acc_done, (n_iter - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
    tc_fence_after();
    const size_t orow = ((size_t)(row0 + row) * p.nkv + kvh) * HD + half * (HD / 2);
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const uint32_t tm = which == 0 ? tmem_dk : tmem_dv;
      __nv_bfloat16* dst = (which == 0 ? p.dk : p.dv) + orow;
#pragma unroll 1
      for (int c = 0; c < HD / 2; c += 32) {
        float o[32];
        if (n_iter > 0) {
          tmem_ld32(tm + lane_off + half * (HD / 2) + c, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0.f;
        }
        if (key_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 pk;
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int j = 0; j < 4; ++j) p2[j] = __floats2bfloat162_rn(o[v * 8 + 2 * j], o[v * 8 + 2 * j + 1]);
            *reinterpret_cast<uint4*>(dst + c + v * 8) = pk;
          }
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

// dQ of the packed attention.  Arguments as tahb_prefill_attn plus dout [n_q, nq*hd], lse and dsum
// ([n_q, nq] fp32) and the output dq [n_q, nq*hd].
extern "C" int tahb_attn_bwd_dq(const void* q, const void* dout, void* dq, void* const* ks, void* const* vs,
                                const long long* n_kv, const int* const* bases, const int* const* counts,
                                const int* const* bounds, int n_seg,
                                const int* tile_q0, const int* tile_qn, int n_tiles, long long n_q, int nq, int nkv,
                                int hd, float scale, const float* lse, const float* dsum, int* status,
                                cudaStream_t stream) {
  if (n_tiles <= 0 || n_q <= 0) return 0;
  if (n_seg < 1 || n_seg > PF_MAX_SEG || (nq % nkv)) return -1;
  CUtensorMap mq, mdo, mk[PF_MAX_SEG], mv[PF_MAX_SEG];
  int rc;
  if ((rc = pf_make_map(&mq, q, n_q, (long long)nq * hd, 128u))) return rc;
  if ((rc = pf_make_map(&mdo, dout, n_q, (long long)nq * hd, 128u))) return rc;
  for (int s = 0; s < PF_MAX_SEG; ++s) {
    const int ss = s < n_seg ? s : 0;
    if ((rc = pf_make_map(&mk[s], ks[ss], n_kv[ss], (long long)nkv * hd, 64u))) return rc;
    if ((rc = pf_make_map(&mv[s], vs[ss], n_kv[ss], (long long)nkv * hd, 64u))) return rc;
  }
  AttnBwdParams p = {};
  p.tile_q0 = tile_q0;
  p.tile_qn = tile_qn;
  for (int s = 0; s < PF_MAX_SEG; ++s) {
    const int ss = s < n_seg ? s : 0;
    p.seg_base[s] = bases[ss];
    p.seg_count[s] = counts[ss];
    p.seg_bound[s] = bounds[ss];
  }
  p.lse = lse;
  p.dsum = dsum;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.n_seg = n_seg; p.nq = nq; p.nkv = nkv;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  dim3 grid(n_tiles, nq);
#define TAHB_BQ(HD_)                                                                                            \
  {                                                                                                             \
    static bool configured = false;                                                                             \
    if (!configured) {                                                                                          \
      if (cudaFuncSetAttribute(attn_bwd_dq_kernel<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                               BwdQCfg<HD_>::SMEM_BYTES) != cudaSuccess)                                        \
        return -10;                                                                                             \
      configured = true;                                                                                        \
    }                                                                                                           \
    attn_bwd_dq_kernel<HD_><<<grid, BWD_THREADS, BwdQCfg<HD_>::SMEM_BYTES, stream>>>(mq, mdo, mk[0], mv[0], mk[1], \
                                                                                     mv[1], mk[2], mv[2], p);   \
  }
  if (hd == 128) TAHB_BQ(128)
  else if (hd == 64) TAHB_BQ(64)
  else return -2;
#undef TAHB_BQ
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dK, dV of ONE segment.  k, v: that segment's [n_kv, nkv*hd]; work items (see AttnBwdParams):
// item_row0 / item_nkeys / item_kidx0 / item_qa / item_qb, [n_items] each; count: the segment's
// visible-key counts per packed query.  dk / dv [n_kv, nkv*hd] are written for every key of every item.
extern "C" int tahb_attn_bwd_dkv(const void* q, const void* dout, const void* k, const void* v, void* dk, void* dv,
                                 long long n_kv, const int* count, const int* bound, const int* item_row0, const int* item_nkeys,
                                 const int* item_kidx0, const int* item_qa, const int* item_qb, int n_items,
                                 long long n_q, int nq, int nkv, int hd, float scale, const float* lse,
                                 const float* dsum, int* status, cudaStream_t stream) {
  if (n_items <= 0 || n_q <= 0) return 0;
  if (nq % nkv) return -1;
  CUtensorMap mq, mdo, mk, mv;
  int rc;
  if ((rc = pf_make_map(&mq, q, n_q, (long long)nq * hd, 64u))) return rc;
  if ((rc = pf_make_map(&mdo, dout, n_q, (long long)nq * hd, 64u))) return rc;
  if ((rc = pf_make_map(&mk, k, n_kv, (long long)nkv * hd, 128u))) return rc;
  if ((rc = pf_make_map(&mv, v, n_kv, (long long)nkv * hd, 128u))) return rc;
  AttnBwdParams p = {};
  p.lse = lse;
  p.dsum = dsum;
  p.nq = nq; p.nkv = nkv;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.kv_row0 = item_row0; p.kv_nkeys = item_nkeys; p.kv_kidx0 = item_kidx0; p.kv_qa = item_qa; p.kv_qb = item_qb;
  p.kv_count = count;
  p.kv_bound = bound;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.status = status;
  dim3 grid(n_items, nkv);
#define TAHB_BKV(HD_)                                                                                           \
  {                                                                                                             \
    static bool configured = false;                                                                             \
    if (!configured) {                                                                                          \
      if (cudaFuncSetAttribute(attn_bwd_dkv_kernel<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                               BwdKVCfg<HD_>::SMEM_BYTES) != cudaSuccess)                                       \
        return -10;                                                                                             \
      configured = true;                                                                                        \
    }                                                                                                           \
    attn_bwd_dkv_kernel<HD_><<<grid, BWD_THREADS, BwdKVCfg<HD_>::SMEM_BYTES, stream>>>(mk, mv, mq, mdo, p);      \
  }
  if (hd == 128) TAHB_BKV(128)
  else if (hd == 64) TAHB_BKV(64)
  else return -2;
#undef TAHB_BKV
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
