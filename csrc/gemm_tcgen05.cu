// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory,
// operands staged by TMA), with the fusions the TaH layers need.
//
// Orientation: "features on lanes".  The 128 TMEM lanes of a CTA hold 128 output features
// (rows of the weight matrix W[F, K]); the TMEM columns hold BN tokens (rows of X[M, K]).
//
//     acc[f, t] = sum_k W[f, k] * X[t, k]  +  sum_r W2[f, r] * X2[t, r]
//
// The second sum is the K-extension used for LoRA: W2 = scaled LoRA-B (block-diagonal over the
// fused projections), X2 = gated x*A^T, so the adapter is part of the same accumulation and of the
// same epilogue ("fused LoRA-GEMM").  Putting the weights on the 128-row operand keeps the tensor
// cores full in decode, where M is 16..256 tokens and the cost is streaming W once from HBM.
//
// Epilogues (all write out[t, f] in bf16):
//   plain      out = acc
//   residual   out = residual[t, f] + bf16(acc)
//   DUAL       two accumulators per CTA, gate = rows f and up = rows up_off + f of W:
//              out = bf16(silu(bf16(gate))) * bf16(up)             (SwiGLU)
//   interleaved SwiGLU (act 2)   one accumulator; the rows of W alternate gate_i, up_i, so a 128-row tile
//              holds 64 output features and the partner of a value sits in the neighbouring TMEM lane:
//              out[t, f / 2] = bf16(silu(bf16(gate))) * bf16(up).  One 256-token MMA per k step instead of two
//              128-token ones: the faster form at every token count (19 vs 29 us at 256 x 12288 x 2048).
//
// Split-K: a thread-block cluster of S CTAs along z splits the k-blocks; the partial accumulators
// of columns owned by other ranks go to the CTA's own shared memory, and every CTA adds to its own
// slice (kept in tensor memory) the matching blocks of all peers, read through distributed shared
// memory with 16-byte loads, in a fixed order (deterministic).  No global scratch.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w%4) .. +31).
#include <cuda.h>
#include <stdio.h>

#include "attn_common.cuh"
#include "common.cuh"

namespace tahb {

constexpr int GEMM_MAX_RANKS = 8;

struct GemmParams {
  __nv_bfloat16* out;
  const __nv_bfloat16* residual;
  int ld_out;
  int ld_res;
  int M;        // tokens
  int F;        // output features (per half when DUAL)
  int up_off;   // DUAL: row offset of the "up" half inside W
  int kb_main;  // K / 64
  int kb_ext;   // R / 64
  int splits;   // cluster size along z (1 = no split-K)
  int tma_out;  // 1: stage the output tile in shared memory and write it with a TMA store
  int act;      // epilogue activation on the (non-dual) output: 0 none, 1 GELU (erf form) of the bf16-rounded value,
                // 2 SwiGLU of interleaved gate / up rows (out has F / 2 features)
  // Operand majors (backward GEMMs read their operands transposed, straight from the row-major tensors):
  //   a_mn: the 128-row operand is stored [reduction, feature] (feature contiguous): dgrad reads W[F, K] as
  //         W^T, wgrad reads X[T, K] as X^T;   b_mn: the column operand is stored [reduction, column]
  //         (wgrad reads dY[T, F] as dY^T).  Such tiles are loaded as 64 x 64 boxes and described to the tensor
  //         core as MN-major.  0 = K-major (the reduction index is contiguous), the forward layout.
  int a_mn, b_mn;
  int* status;
  // Tensor-parallel reduce-scatter by push (row-parallel GEMMs): instead of writing `out`, the tile
  // is stored into the symmetric slot buffer of the rank that owns its token rows,
  // slot[owner][(my rank) * rpr + (row - owner * rpr)][f], and the owner's arrival counter is
  // advanced by the number of rows stored (after a system-scope fence).
  __nv_bfloat16* push_slot[GEMM_MAX_RANKS];
  uint32_t* push_cnt[GEMM_MAX_RANKS];
  int push_world;   // 0 = off
  int push_rank;
  int push_rpr;     // token rows per owner
  int push_ld;      // row pitch of the slot buffers (the full hidden size)
  // Tensor-parallel all-gather wait (column-parallel GEMMs): X rows arrive from their owners by
  // peer stores; before the first X load the producer waits until flag[q] has reached target[q]
  // for every owner q.  Both arrays are local device memory.
  const uint32_t* wait_flag;
  const uint32_t* wait_target;
  int wait_world;   // 0 = off
  unsigned long long wait_limit_ns;   // how long the peer-flag wait may take before it gives up
  // Fused epilogue of the QKV projection (head_dim 128, so one 128-feature tile is one head): per-head
  // RMSNorm of q / k, rotate-half RoPE, q to q_out[t, head], k / v into the paged cache slot of the
  // token (and / or into packed k_dense / v_dense).  Replaces the output store when qkv_on != 0.
  int qkv_on;
  int nq, nkv, page_size;
  float qk_eps, log2_theta;
  const __nv_bfloat16* q_norm_w;
  const __nv_bfloat16* k_norm_w;
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_dense;
  __nv_bfloat16* v_dense;
  __nv_bfloat16* kv_cache[4];
  const int* cache_sel;
  const int* slot;
  const int* pos;
  const __nv_bfloat16* rope_cs;   // optional [M, 128] table: cos of the 64 frequencies, then sin (rope_table_kernel)
};

template <int BN, bool DUAL>
struct GemmCfg {
  static constexpr int W_TILE = 128 * 64 * 2;                 // 16 KiB
  static constexpr int W_BYTES = W_TILE * (DUAL ? 2 : 1);
  static constexpr int X_BYTES = BN * 64 * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int NS_RAW = (196 * 1024) / STAGE_BYTES;
  static constexpr int NS = NS_RAW > 8 ? 8 : NS_RAW;
  static constexpr int NACC = DUAL ? 2 : 1;
  static constexpr int COLS = BN * NACC;
  static constexpr int TMEM_COLS = COLS < 32 ? 32 : COLS;     // power of two >= 32 (BN is a power of two)
  static constexpr int SMEM_BYTES = NS * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
  static constexpr int CHUNK = BN >= 32 ? 32 : 16;
};

template <int CHUNK>
__device__ __forceinline__ void tmem_ld_chunk(uint32_t taddr, float* v) {
  if constexpr (CHUNK == 32) tmem_ld32(taddr, v);
  else tmem_ld16(taddr, v);
}

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }

template <bool DUAL>
__device__ __forceinline__ void store_one(const GemmParams& p, int t, int f, float a, float u) {
  float y;
  if constexpr (DUAL) {
    y = bf16_round(silu(bf16_round(a))) * bf16_round(u);
  } else {
    y = a;
    if (p.residual != nullptr) y = bf16_round(a) + __bfloat162float(p.residual[(size_t)t * p.ld_res + f]);
  }
  p.out[(size_t)t * p.ld_out + f] = __float2bfloat16_rn(y);
}

// Epilogue value into the shared staging tile; with `add_res` the slot already holds the residual
// element (brought in by a TMA load).
template <bool DUAL>
__device__ __forceinline__ void stage_one(__nv_bfloat16* slot, float a, float u, bool add_res) {
  float y;
  if constexpr (DUAL) {
    y = bf16_round(silu(bf16_round(a))) * bf16_round(u);
  } else {
    y = a;
    if (add_res) y = bf16_round(a) + __bfloat162float(*slot);
  }
  *slot = __float2bfloat16_rn(y);
}

// Activation pass over a staged tile (n_tok x 128 bf16 in shared memory), run by the 128 epilogue threads after
// they have all staged their rows: GELU (erf form) of the bf16-rounded outputs.  Kept out of the staging loops,
// whose unrolled bodies every GEMM executes.
__device__ __noinline__ void gelu_tile(__nv_bfloat16* stg, int n_tok) {
  const int e = threadIdx.x - 64;
  __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(stg);
  for (int i = e; i < n_tok * 64; i += 128) {
    const float2 f = __bfloat1622float2(v[i]);
    v[i] = __floats2bfloat162_rn(gelu_erf(f.x), gelu_erf(f.y));
  }
}

// Interleaved-SwiGLU epilogue of one accumulator tile (S == 1 path): lanes 2i / 2i + 1 of the tile hold gate_i / up_i.
// Per token pair the even lane sends its gate of the odd token and receives the up value of the even token (one
// shuffle), so each lane evaluates one SiLU per two tokens; results go to a [BN tokens][64 features] staging tile.
template <int BN, int CHUNK>
__device__ __noinline__ void swiglu_interleaved_tile(uint32_t trow, __nv_bfloat16* stg, int row) {
  const bool odd = row & 1;
  const int fo = row >> 1;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += CHUNK) {
    float a[CHUNK];
    tmem_ld_chunk<CHUNK>(trow + c0, a);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < CHUNK; j += 2) {
      const float recv = __shfl_xor_sync(0xffffffffu, odd ? a[j] : a[j + 1], 1);
      const float g = odd ? recv : a[j];            // even lane: token j, odd lane: token j + 1
      const float u = odd ? a[j + 1] : recv;
      stg[(c0 + j + (odd ? 1 : 0)) * 64 + fo] = __float2bfloat16_rn(bf16_round(silu(bf16_round(g))) * bf16_round(u));
    }
  }
}

// Copy `n_tok` staged rows ([token][128 features] bf16 in shared memory, tokens ta..ta+n_tok) into the
// owners' slot buffers with 16-byte peer stores (128 epilogue threads: 16 lanes per 256-byte row),
// then fence and advance each touched owner's arrival counter by the rows it received.
__device__ __noinline__ void push_rows(const GemmParams& p, const __nv_bfloat16* stg, int ta, int n_tok, int f0) {
  const int e = threadIdx.x - 64;                 // 0..127
  const int sub = e & 15, r0 = e >> 4;            // 16-byte piece of the row, first row of this thread
  const int H = p.push_ld;
  for (int r = r0; r < n_tok; r += 8) {
    const int t = ta + r;
    if (t >= p.M) break;
    const int owner = t / p.push_rpr;
    const uint4 v = *reinterpret_cast<const uint4*>(stg + r * 128 + sub * 8);
    __nv_bfloat16* dst = p.push_slot[owner] + ((size_t)p.push_rank * p.push_rpr + (t - owner * p.push_rpr)) * H + f0 + sub * 8;
    *reinterpret_cast<uint4*>(dst) = v;
  }
  named_bar_sync(1, 128);
  if (e == 0 && ta < p.M) {
    __threadfence_system();
    const int tb = min(p.M, ta + n_tok);
    for (int owner = ta / p.push_rpr; owner * p.push_rpr < tb; ++owner) {
      const int lo = max(ta, owner * p.push_rpr), hi = min(tb, (owner + 1) * p.push_rpr);
      asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p.push_cnt[owner]), "r"((uint32_t)(hi - lo)) : "memory");
    }
  }
}

// QKV epilogue on a staged tile: `stg` holds [n_tok tokens][128 features] bf16 = head `f0 / 128` of tokens
// ta .. ta + n_tok.  First the 128 epilogue threads bring the per-token inputs into shared memory `aux` with
// coalesced loads (the tokens' RoPE rows, cache slots and depth selectors: one global round trip instead of
// one per token); then the four warps take the tokens round robin; a lane owns four consecutive dims of the
// head, so the head's sum of squares is one warp reduction and the rotate-half partner (dim +- 64) sits in
// lane +- 16.  Same arithmetic and rounding as qk_norm_rope_kv_kernel.  `aux` needs n_tok * 264 bytes.
#ifndef TAHB_QKV_U
#define TAHB_QKV_U 1      // tokens per warp and step: 1 measured fastest inside a tick (4 unrolled chains are faster in isolation
                          // but four times the straight-line code, fetched cold by every CTA)
#endif
__device__ __noinline__ void qkv_epilogue(const GemmParams& p, const __nv_bfloat16* stg, uint8_t* aux, int ta,
                                             int n_tok, int f0) {
  const int e = threadIdx.x - 64;                 // 0..127
  const int w4 = e >> 5, lane = e & 31;
  const int h = f0 >> 7;
  const bool is_q = h < p.nq;
  const bool is_k = !is_q && h < p.nq + p.nkv;
  const bool table = p.rope_cs != nullptr;
  uint4* s_cs = reinterpret_cast<uint4*>(aux);                       // [n_tok][16] = 256 bytes per token
  int* s_slot = reinterpret_cast<int*>(aux + (size_t)n_tok * 256);
  int* s_sel = s_slot + n_tok;
  if (table && (is_q || is_k)) {
    const uint4* src = reinterpret_cast<const uint4*>(p.rope_cs);
    for (int i = e; i < n_tok * 16; i += 128) {
      const int t = ta + (i >> 4);
      if (t < p.M) s_cs[i] = src[(size_t)t * 16 + (i & 15)];
    }
  }
  if (!is_q) {
    for (int i = e; i < n_tok; i += 128) {
      const int t = ta + i;
      s_slot[i] = (p.slot != nullptr && t < p.M) ? p.slot[t] : -1;
      s_sel[i] = (p.cache_sel != nullptr && t < p.M) ? p.cache_sel[t] : 0;
    }
  }
  named_bar_sync(1, 128);
  const __nv_bfloat16* nw = is_q ? p.q_norm_w : p.k_norm_w;
  // Packed bf16x2 arithmetic: a bf16 x bf16 product is exact in fp32, so __hmul2 rounds once exactly like the
  // scalar statement bf16(float(a) * float(b)); this more than halves the instruction count of the loop, which
  // only four warps execute.
  __nv_bfloat162 w01 = __floats2bfloat162_rn(0.f, 0.f), w23 = w01;
  float inv[4] = {0.f, 0.f, 0.f, 0.f};
  const bool upper = lane >= 16;
  if (is_q || is_k) {
    const uint2 wr = *reinterpret_cast<const uint2*>(nw + lane * 4);
    w01 = *reinterpret_cast<const __nv_bfloat162*>(&wr.x);
    w23 = *reinterpret_cast<const __nv_bfloat162*>(&wr.y);
    if (!table) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int d = lane * 4 + i;
        const int j = upper ? d - 64 : d;
        inv[i] = exp2f(-(2.0f * (float)j / 128.0f) * p.log2_theta);
      }
    }
  }
  const __nv_bfloat162 sgn = upper ? __floats2bfloat162_rn(1.f, 1.f) : __floats2bfloat162_rn(-1.f, -1.f);
  // Four tokens per warp and step, written phase by phase: the latency of a token's dependent chain (reduction,
  // shuffles) is hidden by the other three tokens' chains.
  constexpr int U = TAHB_QKV_U;
  for (int r0 = w4; r0 < n_tok; r0 += 4 * U) {
    int rr[U];
    bool live[U];
    uint2 raw[U], outv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      rr[u] = r0 + 4 * u;
      live[u] = rr[u] < n_tok && ta + rr[u] < p.M;
      raw[u] = live[u] ? *reinterpret_cast<const uint2*>(stg + rr[u] * 128 + lane * 4) : make_uint2(0u, 0u);
      outv[u] = raw[u];
    }
    if (is_q || is_k) {
      float x[U][4], ss[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[u].x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[u].y));
        x[u][0] = a.x; x[u][1] = a.y; x[u][2] = b.x; x[u][3] = b.y;
        ss[u] = a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int u = 0; u < U; ++u) ss[u] += __shfl_xor_sync(0xffffffffu, ss[u], o);
      }
      __nv_bfloat162 n01[U], n23[U];
      uint32_t p01[U], p23[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float rstd = rsqrtf(ss[u] / 128.0f + p.qk_eps);
        n01[u] = __hmul2(w01, __floats2bfloat162_rn(x[u][0] * rstd, x[u][1] * rstd));
        n23[u] = __hmul2(w23, __floats2bfloat162_rn(x[u][2] * rstd, x[u][3] * rstd));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        p01[u] = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<uint32_t*>(&n01[u]), 16);
        p23[u] = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<uint32_t*>(&n23[u]), 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        __nv_bfloat162 c01, c23, s01, s23;
        if (table) {
          // lane l owns dims 4l .. 4l+3, whose frequency index is 4 (l mod 16) ..: cos there, sin 64 further
          const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(s_cs + (live[u] ? rr[u] : 0) * 16) + (lane & 15) * 4;
          const uint2 cr = *reinterpret_cast<const uint2*>(row), sr = *reinterpret_cast<const uint2*>(row + 64);
          c01 = *reinterpret_cast<const __nv_bfloat162*>(&cr.x); c23 = *reinterpret_cast<const __nv_bfloat162*>(&cr.y);
          s01 = *reinterpret_cast<const __nv_bfloat162*>(&sr.x); s23 = *reinterpret_cast<const __nv_bfloat162*>(&sr.y);
        } else {
          const float posf = live[u] ? (float)p.pos[ta + rr[u]] : 0.f;
          float cv[4], sv[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float ang = posf * inv[i];
            cv[i] = cosf(ang);
            sv[i] = sinf(ang);
          }
          c01 = __floats2bfloat162_rn(cv[0], cv[1]); c23 = __floats2bfloat162_rn(cv[2], cv[3]);
          s01 = __floats2bfloat162_rn(sv[0], sv[1]); s23 = __floats2bfloat162_rn(sv[2], sv[3]);
        }
        // y = bf16( bf16(n c) + bf16(+-partner s) ): the products in packed bf16, the sum in fp32, one rounding
        const float2 a01 = __bfloat1622float2(__hmul2(n01[u], c01)), a23 = __bfloat1622float2(__hmul2(n23[u], c23));
        const float2 b01 = __bfloat1622float2(__hmul2(__hmul2(*reinterpret_cast<__nv_bfloat162*>(&p01[u]), sgn), s01));
        const float2 b23 = __bfloat1622float2(__hmul2(__hmul2(*reinterpret_cast<__nv_bfloat162*>(&p23[u]), sgn), s23));
        __nv_bfloat162 o0 = __floats2bfloat162_rn(a01.x + b01.x, a01.y + b01.y);
        __nv_bfloat162 o1 = __floats2bfloat162_rn(a23.x + b23.x, a23.y + b23.y);
        outv[u].x = *reinterpret_cast<uint32_t*>(&o0);
        outv[u].y = *reinterpret_cast<uint32_t*>(&o1);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!live[u]) continue;
      const int t = ta + rr[u];
      if (is_q) {
        *reinterpret_cast<uint2*>(p.q_out + ((size_t)t * p.nq + h) * 128 + lane * 4) = outv[u];
        continue;
      }
      const int kvh = is_k ? h - p.nq : h - p.nq - p.nkv;
      __nv_bfloat16* dense = is_k ? p.k_dense : p.v_dense;
      if (dense != nullptr) *reinterpret_cast<uint2*>(dense + ((size_t)t * p.nkv + kvh) * 128 + lane * 4) = outv[u];
      const int sl = s_slot[rr[u]];
      if (sl >= 0) {
        const int sel = s_sel[rr[u]];
        __nv_bfloat16* cache = sel == 0 ? p.kv_cache[0] : sel == 1 ? p.kv_cache[1] : sel == 2 ? p.kv_cache[2] : p.kv_cache[3];
        const int page = sl / p.page_size, off = sl % p.page_size;
        *reinterpret_cast<uint2*>(cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * p.nkv + kvh) * p.page_size + off) * 128 +
                                  lane * 4) = outv[u];
      }
    }
  }
}

// bytes of the split-K receive area: (S - 1) source blocks of [cols_per_rank][128] floats
__host__ __device__ constexpr int split_stage_offset(int S, int cols_per_rank) {
  return (((S - 1) * 128 * cols_per_rank * 4) + 1023) & ~1023;
}

template <int BN, bool DUAL, bool PAIR = false>
__global__ void __launch_bounds__(192, 1)
gemm_fl_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
               const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_x2,
               const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_res,
               const __grid_constant__ GemmParams p) {
  using C = GemmCfg<BN, DUAL>;
  pdl_launch_dependents();      // the next kernel of the chain may be scheduled behind this one
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::NS * C::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + C::NS;
  uint64_t* accum_bar = empty_bar + C::NS;
  uint64_t* res_bar = accum_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(res_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int f0 = blockIdx.x * 128;
  const int t0 = blockIdx.y * BN;
  const int S = p.splits;
  const int rank = blockIdx.z;                       // == cluster rank: cluster dims are (1, 1, S)
  const int kb_total = p.kb_main + p.kb_ext;
  const int kb_begin = (int)(((long long)kb_total * rank) / S);
  const int kb_end = (int)(((long long)kb_total * (rank + 1)) / S);
  const int n_kb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::NS; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accum_bar, 1);
    mbar_init(res_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&tm_w);
    prefetch_tensormap(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();                   // set-up above touched no global memory; operands may be read from here on
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      if (p.wait_world > 0) {
        if (!wait_peer_rows(p.wait_flag, p.wait_target, p.wait_world, p.status, p.wait_limit_ns)) *abort_flag = 1;
        asm volatile("fence.proxy.async.global;" ::: "memory");   // the TMA loads below see the landed rows
      }
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % C::NS;
        const uint32_t ph = (i / C::NS) & 1;
        mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, STATUS_TIMEOUT_STAGE_EMPTY);
        if (*abort_flag) break;           // a wait gave up: issue no further copies, let the kernel run out
        mbar_expect_tx(&full_bar[s], C::STAGE_BYTES);
        const int g = kb_begin + i;
        const bool ext = g >= p.kb_main;
        const int x = (ext ? g - p.kb_main : g) * 64;
        const CUtensorMap* mw = ext ? &tm_w2 : &tm_w;
        const CUtensorMap* mx = ext ? &tm_x2 : &tm_x;
        uint8_t* st = smem + s * C::STAGE_BYTES;
        if (p.a_mn) {                       // [64 reduction rows][64 features] boxes, 8 KiB each
          tma_load_2d(st, mw, f0, x, &full_bar[s]);
          tma_load_2d(st + 8192, mw, f0 + 64, x, &full_bar[s]);
        } else {
          tma_load_2d(st, mw, x, f0, &full_bar[s]);
        }
        if constexpr (DUAL) {               // second feature tile: the "up" rows (SwiGLU) or features up_off + f0 (pair)
          if (p.a_mn) {
            tma_load_2d(st + C::W_TILE, mw, p.up_off + f0, x, &full_bar[s]);
            tma_load_2d(st + C::W_TILE + 8192, mw, p.up_off + f0 + 64, x, &full_bar[s]);
          } else {
            tma_load_2d(st + C::W_TILE, mw, x, p.up_off + f0, &full_bar[s]);
          }
        }
        if (p.b_mn) {
#pragma unroll
          for (int j = 0; j < (BN >= 64 ? BN / 64 : 1); ++j)
            tma_load_2d(st + C::W_BYTES + j * 8192, mx, t0 + j * 64, x, &full_bar[s]);
        } else {
          tma_load_2d(st + C::W_BYTES, mx, x, t0, &full_bar[s]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(128, BN) | (p.a_mn ? (1u << 15) : 0u) | (p.b_mn ? (1u << 16) : 0u);
      const uint32_t a_step = (p.a_mn ? 2048u : 32u) >> 4, b_step = (p.b_mn ? 2048u : 32u) >> 4;
      for (int i = 0; i < n_kb; ++i) {
        const int s = i % C::NS;
        const uint32_t ph = (i / C::NS) & 1;
        mbar_wait(&full_bar[s], ph, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
        const uint32_t b_addr = a_addr + C::W_BYTES;
        // K-major: 16 reduction elements = 32 bytes along the swizzled row; MN-major: 16 reduction rows of
        // 128 bytes = 2048 bytes, the next 64 features / columns 8192 bytes further.  The start address sits in
        // the low bits of the descriptor in 16-byte units, so a k step is an addition.
        const uint64_t da0 = p.a_mn ? umma_desc_mn_sw128(a_addr, 8192) : umma_desc_sw128(a_addr);
        const uint64_t db0 = p.b_mn ? umma_desc_mn_sw128(b_addr, 8192) : umma_desc_sw128(b_addr);
        const uint64_t da1 = p.a_mn ? umma_desc_mn_sw128(a_addr + C::W_TILE, 8192) : umma_desc_sw128(a_addr + C::W_TILE);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t da = da0 + (uint64_t)(k * a_step);
          const uint64_t db = db0 + (uint64_t)(k * b_step);
          const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
          umma_bf16(tmem_base, da, db, idesc, acc);
          if constexpr (DUAL) umma_bf16(tmem_base + BN, da1 + (uint64_t)(k * a_step), db, idesc, acc);
        }
        umma_commit(&empty_bar[s]);   // frees the stage once these MMAs have read it
      }
      umma_commit(accum_bar);
    }
    __syncwarp();
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int f = f0 + row;
    const uint32_t trow = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    mbar_wait(accum_bar, 0, abort_flag, p.status, STATUS_TIMEOUT_ACCUM);
    tc_fence_after();
    if (S == 1) {
      __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem);     // [BN tokens][128 features]
      const bool res_tma = p.tma_out && p.residual != nullptr;
      if constexpr (PAIR) {
        // Two plain output tiles (features f0.. and up_off + f0..) that shared the CTA's activation tile: per unit
        // of work a CTA pulls half the activation bytes, which is what bounds the GEMM at large token counts.
        __nv_bfloat16* stg1 = stg + BN * 128;
        const bool il = p.act == 2;
        if (res_tma) {
          if (threadIdx.x == 64) {
            mbar_expect_tx(res_bar, BN * 256 * 2);
            tma_load_2d(stg, &tm_res, f0, t0, res_bar);
            tma_load_2d(stg1, &tm_res, p.up_off + f0, t0, res_bar);
          }
          mbar_wait(res_bar, 0, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
        }
        if (il) {
          swiglu_interleaved_tile<BN, C::CHUNK>(trow, stg, row);
          swiglu_interleaved_tile<BN, C::CHUNK>(trow + BN, stg1, row);
        } else {
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += C::CHUNK) {
            float a[C::CHUNK], u[C::CHUNK];
            tmem_ld_chunk<C::CHUNK>(trow + c0, a);
            tmem_ld_chunk<C::CHUNK>(trow + BN + c0, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < C::CHUNK; ++j) {
              stage_one<false>(stg + (c0 + j) * 128 + row, a[j], 0.f, res_tma);
              stage_one<false>(stg1 + (c0 + j) * 128 + row, u[j], 0.f, res_tma);
            }
          }
        }
        if (p.push_world > 0) {
          named_bar_sync(1, 128);
          push_rows(p, stg, t0, BN, f0);
          push_rows(p, stg1, t0, BN, p.up_off + f0);
        } else {
          fence_proxy_async_smem();
          named_bar_sync(1, 128);
          if (threadIdx.x == 64) {
            tma_store_2d(&tm_out, stg, il ? f0 / 2 : f0, t0);
            tma_store_2d(&tm_out, stg1, il ? (p.up_off + f0) / 2 : p.up_off + f0, t0);
            tma_store_commit();
            tma_store_wait_read();
          }
        }
      } else {
      if (res_tma) {
        if (threadIdx.x == 64) {
          mbar_expect_tx(res_bar, BN * 256);
          tma_load_2d(stg, &tm_res, f0, t0, res_bar);
        }
        mbar_wait(res_bar, 0, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
      }
      const bool swiglu_il = !DUAL && p.act == 2;
      if (swiglu_il) {
        if constexpr (!DUAL) swiglu_interleaved_tile<BN, C::CHUNK>(trow, stg, row);
      }
#pragma unroll 1
      for (int c0 = swiglu_il ? BN : 0; c0 < BN; c0 += C::CHUNK) {
        float a[C::CHUNK];
        float u[DUAL ? C::CHUNK : 1];
        tmem_ld_chunk<C::CHUNK>(trow + c0, a);
        if constexpr (DUAL) tmem_ld_chunk<C::CHUNK>(trow + BN + c0, u);
        tmem_ld_wait();
        if (p.tma_out) {
#pragma unroll
          for (int j = 0; j < C::CHUNK; ++j)
            stage_one<DUAL>(stg + (c0 + j) * 128 + row, a[j], DUAL ? u[j] : 0.f, res_tma);
        } else if (f < p.F) {
#pragma unroll
          for (int j = 0; j < C::CHUNK; ++j) {
            const int t = t0 + c0 + j;
            if (t < p.M) store_one<DUAL>(p, t, f, a[j], DUAL ? u[j] : 0.f);
          }
        }
      }
      if (p.qkv_on) {
        named_bar_sync(1, 128);
        qkv_epilogue(p, stg, smem + BN * 256, t0, BN, f0);        // aux behind the staged tile
      } else if (p.push_world > 0) {
        named_bar_sync(1, 128);
        push_rows(p, stg, t0, BN, f0);
      } else if (p.tma_out) {
        if (p.act == 1) {
          named_bar_sync(1, 128);
          gelu_tile(stg, BN);
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (threadIdx.x == 64) {
          tma_store_2d(&tm_out, stg, swiglu_il ? f0 / 2 : f0, t0);
          tma_store_commit();
          tma_store_wait_read();
        }
      }
      }
    }
    tc_fence_before();
  }

  if (S > 1) {
    // Split-K reduction.  The token columns are dealt out to the S ranks (per = BN / S each, per
    // accumulator).  After a first cluster barrier (every CTA has finished its main loop, so the
    // pipeline buffers are free) a rank PUSHES the partial columns owned by rank d into d's shared
    // memory (remote stores need no round trip), block index = source rank - (source > d), laid
    // out [NACC * per columns][128 rows] floats; after a second barrier each rank adds the received
    // blocks to its own columns, which never left tensor memory, in a fixed order.  Every thread
    // of every CTA takes part in both barriers.
    cluster_sync_all();
    if (warp >= 2) {
      tc_fence_after();
      const int q = warp & 3;
      const int row = q * 32 + lane;
      const int per = BN / S;
      const int rs = C::NACC * per + 4;
      const uint32_t trow = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      const uint32_t red_addr = smem_u32(smem);
#pragma unroll 1
      for (int d = 0; d < S; ++d) {
        if (d == rank) continue;
        // block of rank d's shared memory reserved for this source: [NACC * per columns][128 rows];
        // the 32 lanes of a warp write 32 consecutive floats, i.e. one 128-byte remote packet
        const uint32_t dst = dsmem_addr(red_addr + ((rank < d ? rank : rank - 1) * C::NACC * per * 128 + row) * 4, d);
#pragma unroll 1
        for (int acc = 0; acc < C::NACC; ++acc) {
#pragma unroll 1
          for (int c = 0; c < per; c += 16) {
            float a[16];
            tmem_ld16(trow + acc * BN + d * per + c, a);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) st_dsmem_f32(dst + ((acc * per + c + j) * 128) * 4, a[j]);
          }
        }
      }
      tc_fence_before();
    }
    cluster_sync_all();
    if (warp >= 2) {
      tc_fence_after();
      const int q = warp & 3;
      const int row = q * 32 + lane;
      const int f = f0 + row;
      const int per = BN / S;
      const int rs = C::NACC * per + 4;
      const uint32_t trow = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      const float* red = reinterpret_cast<const float*>(smem);
      // output staging tile [per tokens][128 features] lives behind the received blocks
      __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + split_stage_offset(S, C::NACC * per));
      const bool res_tma = p.tma_out && p.residual != nullptr;
      if (res_tma) {
        if (threadIdx.x == 64) {
          mbar_expect_tx(res_bar, per * 256);
          tma_load_2d(stg, &tm_res, f0, t0 + rank * per, res_bar);
        }
        mbar_wait(res_bar, 0, abort_flag, p.status, STATUS_TIMEOUT_TMA_FULL);
      }
#pragma unroll 1
      for (int c = 0; c < per; c += 16) {
        float a[16];
        float u[DUAL ? 16 : 1];
        tmem_ld16(trow + rank * per + c, a);
        if constexpr (DUAL) tmem_ld16(trow + BN + rank * per + c, u);
        tmem_ld_wait();
#pragma unroll 1
        for (int blk = 0; blk < S - 1; ++blk) {
          const float* src = red + ((size_t)blk * C::NACC * per + c) * 128 + row;
#pragma unroll
          for (int j = 0; j < 16; ++j) a[j] += src[j * 128];
          if constexpr (DUAL) {
#pragma unroll
            for (int j = 0; j < 16; ++j) u[j] += src[(per + j) * 128];
          }
        }
        if (p.tma_out) {
#pragma unroll
          for (int j = 0; j < 16; ++j) stage_one<DUAL>(stg + (c + j) * 128 + row, a[j], DUAL ? u[j] : 0.f, res_tma);
        } else if (f < p.F) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + rank * per + c + j;
            if (t < p.M) store_one<DUAL>(p, t, f, a[j], DUAL ? u[j] : 0.f);
          }
        }
      }
      if (p.qkv_on) {
        named_bar_sync(1, 128);
        qkv_epilogue(p, stg, reinterpret_cast<uint8_t*>(stg) + per * 256, t0 + rank * per, per, f0);
      } else if (p.push_world > 0) {
        named_bar_sync(1, 128);
        push_rows(p, stg, t0 + rank * per, per, f0);
      } else if (p.tma_out) {
        if (p.act == 1) {
          named_bar_sync(1, 128);
          gelu_tile(stg, per);
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (threadIdx.x == 64) {
          tma_store_2d(&tm_out, stg, f0, t0 + rank * per);
          tma_store_commit();
          tma_store_wait_read();
        }
      }
      tc_fence_before();
    }
  }

  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2D bf16 row-major [rows, cols] with leading dimension ld (elements).  Operand maps use a
// {64, box_rows} box with the 128-byte swizzle; output/residual maps a {128, box_rows} box, unswizzled.
static int make_map(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld, int box_rows,
                    bool operand, unsigned out_box_cols = 128u) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return -2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {operand ? 64u : out_box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, operand ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  operand ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// MN-major operand of a [reduction_rows, mn_cols] row-major bf16 matrix: 64 x 64 boxes, 128-byte swizzle.
static int make_map_mn(CUtensorMap* m, const void* base, long long red_rows, long long mn_cols, long long ld) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return -2;
  cuuint64_t dims[2] = {(cuuint64_t)mn_cols, (cuuint64_t)red_rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, 64u};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

template <int BN, bool DUAL, bool PAIR = false>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& mw2, const CUtensorMap& mx2,
                  const CUtensorMap& mo, const CUtensorMap& mr, const GemmParams& p, cudaStream_t stream) {
  using C = GemmCfg<BN, DUAL>;
  static bool configured = false;
  auto kern = gemm_fl_kernel<BN, DUAL, PAIR>;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) return -10;
    configured = true;
  }
  if (p.splits > 1) {
    const int per = BN / p.splits;
    if (per % 16 || (size_t)split_stage_offset(p.splits, C::NACC * per) + (size_t)per * 256 +
                            (p.qkv_on ? (size_t)per * 264 : 0) >
                        (size_t)C::NS * C::STAGE_BYTES)
      return -11;
  } else if (p.qkv_on && (size_t)BN * (256 + 264) > (size_t)C::NS * C::STAGE_BYTES) {
    return -11;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.F + 127) / 128, (p.M + BN - 1) / BN, p.splits);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = p.splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mw, mx, mw2, mx2, mo, mr, p);
  return e == cudaSuccess ? 0 : -12;
}

}  // namespace tahb

using namespace tahb;

// out[M, F] = X[M, K] W[F, K]^T (+ X2[M, R] W2[F, R]^T) (+ residual) ; dual != 0 => SwiGLU over W rows
// [0, F) (gate) and [up_off, up_off + F) (up).  All matrices bf16 row-major; K and R multiples of 64.
// bn = token-tile width (16/32/64/128/256, 0 = choose from M); splits = split-K cluster size (1,2,4,8).
// Returns 0 on success, a negative code on a host-side error.  *status (device int) is set non-zero
// by the kernel if a bounded wait ran out.
// Host-side description of the fused QKV epilogue (see GemmParams::qkv_on); all pointers are device memory.
struct TahbQkvEpilogue {
  const void* q_norm_w;
  const void* k_norm_w;
  void* q_out;
  void* k_dense;        // optional packed K [M, nkv * 128]
  void* v_dense;        // optional packed V
  void* kv_cache[4];    // paged cache of this layer, one per depth (n_caches of them)
  const int* cache_sel; // optional per-token depth index into kv_cache
  const int* slot;      // per-token slot (page * page_size + offset), negative = no cache write; null = no cache
  const int* pos;       // per-token position id
  const void* rope_cs;  // optional [M, 128] bf16 cos | sin table of this pass (tahb_rope_table); null = compute in place
  int n_caches, nq, nkv, page_size;
  float eps, theta;
};

struct GemmTpArgs {
  void* const* push_slot = nullptr;     // [world] slot buffers (peer pointers), or null
  void* const* push_cnt = nullptr;      // [world] arrival counters (peer pointers)
  int push_world = 0, push_rank = 0, push_rpr = 0;
  const void* wait_flag = nullptr;      // local [world] flags, or null
  const void* wait_target = nullptr;    // local [world] targets
  int wait_world = 0;
};

static int gemm_impl(const void* W, const void* X, void* out, const void* residual, const void* W2,
                     const void* X2, int M, int F, int K, int R, long long ldw, long long ldx, long long ldo,
                     long long ldr, long long ldw2, long long ldx2, int dual, int up_off, int splits, int bn,
                     int* status, cudaStream_t stream, const GemmTpArgs& tp, const TahbQkvEpilogue* qkv = nullptr,
                     int a_mn = 0, int b_mn = 0, int k_rows = 0) {
  if (M <= 0 || F <= 0) return 0;
  // transposed operands: W is then [K, F] (ldw = its row pitch), X is [K, M]; no LoRA extension, no dual
  if ((a_mn || b_mn) && (dual == 1 || dual == 6 || R > 0 || qkv != nullptr || tp.push_world > 0)) return -27;
  if (a_mn && F % 128) return -27;
  const bool push = tp.push_world > 0;
  if (qkv != nullptr && (dual != 0 || residual != nullptr || push || F != (qkv->nq + 2 * qkv->nkv) * 128 ||
                         qkv->n_caches > 4 || qkv->q_out == nullptr || qkv->pos == nullptr))
    return -26;
  // dual: 0 = one accumulator, 1 = SwiGLU of W rows [0, F) and [up_off, up_off + F), 3 = one accumulator + GELU,
  // 4 = one accumulator, SwiGLU of interleaved gate / up rows (F weight rows -> F / 2 output features),
  // 2 = pair: two plain 128-feature tiles per CTA (features f and F / 2 + f) that share a 256-token activation
  //     tile, unsplit; 6 = pair + interleaved SwiGLU.  The pair forms halve the activation bytes per unit of work
  //     and are the fast ones at large token counts (1350-1400 vs 915-1100 TFLOP/s at 8192+ tokens).
  const bool pair = dual == 2 || dual == 6;
  const int act = dual == 3 ? 1 : (dual == 4 || dual == 6) ? 2 : 0;
  if (dual == 3 || dual == 4) dual = 0;
  if (act == 2 && (F % 2 || splits > 1 || push || residual != nullptr || qkv != nullptr || a_mn || b_mn)) return -29;
  const int F_full = F;
  if (pair) {
    if (F % 256 || qkv != nullptr || R % 64) return -24;
    dual = 2;
    F = F / 2;
    up_off = F;
    bn = 256;
    splits = 1;
  }
  if (pair && b_mn && M % 64) return -24;
  if (push && (dual == 1 || residual != nullptr || F_full % 128 || tp.push_world > GEMM_MAX_RANKS || tp.push_rpr <= 0))
    return -23;
  if (K % 64 || R % 64 || K <= 0) return -20;
  if (bn == 0) bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  if (b_mn && bn < 64) bn = 64;               // MN-major column tiles come in 64-wide boxes
  if (splits < 1) splits = 1;
  const int kb = K / 64 + R / 64;
  while (splits > 1 && (splits > kb || bn % splits || (bn / splits) % 16)) splits >>= 1;
  const long long w_rows = dual ? (long long)up_off + F : F;
  CUtensorMap mw, mx, mw2, mx2;
  int rc;
  // k_rows: true reduction length of MN-major operands (K is rounded up to whole k-blocks; TMA zero-fills the rest)
  const long long kr = k_rows > 0 ? k_rows : K;
  if ((rc = a_mn ? make_map_mn(&mw, W, kr, w_rows, ldw) : make_map(&mw, W, w_rows, K, ldw, 128, true))) return rc;
  if ((rc = b_mn ? make_map_mn(&mx, X, kr, M, ldx) : make_map(&mx, X, M, K, ldx, bn, true))) return rc;
  if (R > 0) {
    if ((rc = make_map(&mw2, W2, w_rows, R, ldw2, 128, true))) return rc;
    if ((rc = make_map(&mx2, X2, M, R, ldx2, bn, true))) return rc;
  } else {
    mw2 = mw;
    mx2 = mx;
  }
  // output (and residual) through TMA when their layout allows it, else element-wise stores
  CUtensorMap mo, mr;
  int tma_out = !push && qkv == nullptr &&
                make_map(&mo, out, M, act == 2 ? F_full / 2 : F_full, ldo, bn / splits, false, act == 2 ? 64u : 128u) == 0;
  if (tma_out && residual != nullptr) tma_out = make_map(&mr, residual, M, F_full, ldr, bn / splits, false) == 0;
  if (pair && !tma_out && !push) return -25;     // the pair epilogue only exists on the staged paths
  if (act && (!tma_out || residual != nullptr)) return -28;   // the activation passes work on the staged tile, without a residual
  if (!tma_out) mo = mw;
  if (!tma_out || residual == nullptr) mr = mo;
  GemmParams p;
  p.tma_out = tma_out || push || qkv != nullptr;   // push and QKV modes stage the tile in shared memory as well
  p.qkv_on = qkv != nullptr ? 1 : 0;
  p.wait_limit_ns = peer_wait_limit_ns();
  if (qkv != nullptr) {
    p.nq = qkv->nq; p.nkv = qkv->nkv; p.page_size = qkv->page_size;
    p.qk_eps = qkv->eps; p.log2_theta = log2f(qkv->theta);
    p.q_norm_w = reinterpret_cast<const __nv_bfloat16*>(qkv->q_norm_w);
    p.k_norm_w = reinterpret_cast<const __nv_bfloat16*>(qkv->k_norm_w);
    p.q_out = reinterpret_cast<__nv_bfloat16*>(qkv->q_out);
    p.k_dense = reinterpret_cast<__nv_bfloat16*>(qkv->k_dense);
    p.v_dense = reinterpret_cast<__nv_bfloat16*>(qkv->v_dense);
    for (int c = 0; c < 4; ++c) p.kv_cache[c] = c < qkv->n_caches ? reinterpret_cast<__nv_bfloat16*>(qkv->kv_cache[c]) : nullptr;
    p.cache_sel = qkv->cache_sel;
    p.slot = qkv->n_caches > 0 ? qkv->slot : nullptr;
    p.pos = qkv->pos;
    p.rope_cs = reinterpret_cast<const __nv_bfloat16*>(qkv->rope_cs);
  } else {
    p.nq = p.nkv = p.page_size = 0; p.qk_eps = p.log2_theta = 0.f;
    p.q_norm_w = p.k_norm_w = nullptr; p.q_out = p.k_dense = p.v_dense = nullptr;
    for (int c = 0; c < 4; ++c) p.kv_cache[c] = nullptr;
    p.cache_sel = p.slot = p.pos = nullptr;
    p.rope_cs = nullptr;
  }
  p.act = act;
  p.a_mn = a_mn;
  p.b_mn = b_mn;
  p.push_ld = F_full;
  p.push_world = tp.push_world;
  p.push_rank = tp.push_rank;
  p.push_rpr = tp.push_rpr;
  for (int q = 0; q < GEMM_MAX_RANKS; ++q) {
    p.push_slot[q] = push && q < tp.push_world ? reinterpret_cast<__nv_bfloat16*>(tp.push_slot[q]) : nullptr;
    p.push_cnt[q] = push && q < tp.push_world ? reinterpret_cast<uint32_t*>(tp.push_cnt[q]) : nullptr;
  }
  p.wait_flag = reinterpret_cast<const uint32_t*>(tp.wait_flag);
  p.wait_target = reinterpret_cast<const uint32_t*>(tp.wait_target);
  p.wait_world = tp.wait_flag != nullptr ? tp.wait_world : 0;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ld_out = (int)ldo;
  p.ld_res = (int)ldr;
  p.M = M;
  p.F = F;
  p.up_off = up_off;
  p.kb_main = K / 64;
  p.kb_ext = R / 64;
  p.splits = splits;
  p.status = status;
#define TAHB_LAUNCH(BN_)                                                              \
  case BN_:                                                                           \
    return dual ? launch<BN_, true>(mw, mx, mw2, mx2, mo, mr, p, stream) : launch<BN_, false>(mw, mx, mw2, mx2, mo, mr, p, stream);
  if (pair) return launch<256, true, true>(mw, mx, mw2, mx2, mo, mr, p, stream);
  switch (bn) {
    TAHB_LAUNCH(16)
    TAHB_LAUNCH(32)
    TAHB_LAUNCH(64)
    TAHB_LAUNCH(128)
    TAHB_LAUNCH(256)
    default:
      return -22;
  }
#undef TAHB_LAUNCH
}

extern "C" int tahb_gemm(const void* W, const void* X, void* out, const void* residual, const void* W2,
                         const void* X2, int M, int F, int K, int R, long long ldw, long long ldx, long long ldo,
                         long long ldr, long long ldw2, long long ldx2, int dual, int up_off, int splits, int bn,
                         int* status, cudaStream_t stream) {
  return gemm_impl(W, X, out, residual, W2, X2, M, F, K, R, ldw, ldx, ldo, ldr, ldw2, ldx2, dual, up_off, splits, bn,
                   status, stream, GemmTpArgs());
}

// Tensor-parallel variants of the same GEMM (see GemmParams): `push_*` turns the epilogue into a
// reduce-scatter by peer stores (out is ignored, F must be the full hidden size), `wait_*` makes the
// producer wait for the X rows that the owners broadcast.
extern "C" int tahb_gemm_tp(const void* W, const void* X, void* out, const void* residual, const void* W2,
                            const void* X2, int M, int F, int K, int R, long long ldw, long long ldx, long long ldo,
                            long long ldr, long long ldw2, long long ldx2, int dual, int up_off, int splits, int bn,
                            int* status, cudaStream_t stream, void* const* push_slot, void* const* push_cnt,
                            int push_world, int push_rank, int push_rpr, const void* wait_flag,
                            const void* wait_target, int wait_world) {
  GemmTpArgs tp;
  tp.push_slot = push_slot; tp.push_cnt = push_cnt; tp.push_world = push_slot ? push_world : 0;
  tp.push_rank = push_rank; tp.push_rpr = push_rpr;
  tp.wait_flag = wait_flag; tp.wait_target = wait_target; tp.wait_world = wait_world;
  return gemm_impl(W, X, out, residual, W2, X2, M, F, K, R, ldw, ldx, ldo, ldr, ldw2, ldx2, dual, up_off, splits, bn,
                   status, stream, tp);
}

// QKV projection with the fused epilogue (per-head QK-norm, RoPE, q / paged K,V writes): same operands as
// tahb_gemm_tp (out / residual unused), F must be (nq + 2 nkv) * 128.
extern "C" int tahb_gemm_qkv(const void* W, const void* X, const void* W2, const void* X2, int M, int F, int K, int R,
                             long long ldw, long long ldx, long long ldw2, long long ldx2, int splits, int bn,
                             int* status, cudaStream_t stream, const void* wait_flag, const void* wait_target,
                             int wait_world, const TahbQkvEpilogue* qkv) {
  GemmTpArgs tp;
  tp.wait_flag = wait_flag; tp.wait_target = wait_target; tp.wait_world = wait_world;
  if (qkv == nullptr) return -26;
  return gemm_impl(W, X, nullptr, nullptr, W2, X2, M, F, K, R, ldw, ldx, 0, 0, ldw2, ldx2, 0, 0, splits, bn, status,
                   stream, tp, qkv);
}

// out[M, F] (+= residual) = op(X) op(W)^T with transposed operands, for the backward GEMMs:
//   a_mn: W is stored [K, F] row-major (row pitch ldw) instead of [F, K];
//   b_mn: X is stored [K, M] row-major (row pitch ldx) instead of [M, K].
// K (the reduction length) may be any multiple of 8; rows past it read as zeros.  F % 128 == 0 with a_mn.
// pair != 0: two feature tiles per CTA sharing a 256-column tile (F % 256 == 0; with b_mn also M % 64 == 0), unsplit.
extern "C" int tahb_gemm_t(const void* W, const void* X, void* out, const void* residual, int M, int F, int K,
                           long long ldw, long long ldx, long long ldo, long long ldr, int a_mn, int b_mn, int splits,
                           int bn, int* status, cudaStream_t stream, int pair) {
  const int Kp = (K + 63) / 64 * 64;          // the tail k-block of MN-major operands is zero-filled by TMA
  if (Kp != K && !(a_mn && b_mn)) return -20; // a K-major operand needs whole k-blocks
  return gemm_impl(W, X, out, residual, nullptr, nullptr, M, F, Kp, 0, ldw, ldx, ldo, ldr, 0, 0, pair ? 2 : 0, 0, splits,
                   bn, status, stream, GemmTpArgs(), nullptr, a_mn, b_mn, K);
}
