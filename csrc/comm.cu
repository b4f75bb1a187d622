// Tensor-parallel collectives fused with the ops around them, over NVLink peer memory.
//
// fused_reduce_residual_norm: the row-parallel GEMMs (attention output, MLP down) leave on every
// rank a partial [M, H] bf16 result in that rank's *symmetric* buffer.  This kernel replaces the
// NCCL all-reduce + residual add + RMSNorm + (all-gather) sequence by one launch per rank:
//
//   rows are dealt out to the ranks in contiguous blocks; for each row it owns a rank
//     1. sums the row over all ranks' partial buffers  - NVLS `multimem.ld_reduce` (the switch adds)
//        when a multicast mapping exists, otherwise one peer load per rank,
//     2. adds the residual stream h (which stays sharded by row on its owner),
//     3. RMS-normalises the new h row, and
//     4. broadcasts the normalised row into every rank's x buffer - `multimem.st` or peer stores -
//        where the next column-parallel GEMM reads it locally.
//
// Ranks synchronise inside the kernel with flags in symmetric memory: CTA b of every rank meets
// CTA b of the other ranks at the start (all partial GEMMs are complete) and at the end (all
// broadcast rows have landed).  The grid is the same on every rank and small enough to be
// co-resident.  Waits are bounded: a rank that sees no peer within WAIT_TIMEOUT_NS records
// STATUS_TIMEOUT_PEER_FLAG in the status word and returns.
//
// No TMA load touches peer memory here, and nothing in this library uses cluster multicast.
#include "common.cuh"

namespace tahb {

constexpr int COMM_MAX_RANKS = 8;

struct FusedReduceParams {
  const __nv_bfloat16* partial[COMM_MAX_RANKS];   // every rank's partial buffer (peer pointers); [M, H]
  __nv_bfloat16* xout[COMM_MAX_RANKS];            // every rank's normalised-activation buffer [M, H]
  const __nv_bfloat16* mc_partial;                // multicast address of the partial buffer or nullptr
  __nv_bfloat16* mc_xout;                         // multicast address of the x buffer or nullptr
  __nv_bfloat16* h;                               // local residual stream [M, H] (owned rows are live)
  const __nv_bfloat16* ln_w;
  uint32_t* flags[COMM_MAX_RANKS];                // every rank's flag array [grid][world]
  uint32_t* epoch;                                // local [grid] barrier counters
  int* status;
  int M, H, rank, world, rows_per_rank;
  float eps;
  int add_residual;                               // 0: h = sum (first use), 1: h += sum
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// 8 bf16 lanes summed over all ranks by the NVSwitch, fp32 accumulation
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// CTA `b` of this rank meets CTA `b` of every other rank.  Thread q (< world) signals rank q and
// polls rank q's flag, so the `world` signals and waits run in parallel: one system-scope fence
// per thread before its (relaxed) signal and one after its poll, instead of a chain of
// release/acquire operations in one thread.  The rest of the CTA waits at the barrier that
// follows.  Returns false after a timeout.
__device__ __forceinline__ bool cross_rank_barrier(const FusedReduceParams& p, int b, uint32_t epoch) {
  bool ok = true;
  __syncthreads();   // every thread's earlier writes happen-before the fences below
  if ((int)threadIdx.x < p.world) {
    const int q = threadIdx.x;
    __threadfence_system();
    st_relaxed_sys(p.flags[q] + (size_t)b * p.world + p.rank, epoch);
    const uint32_t* mine = p.flags[p.rank] + (size_t)b * p.world + q;
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    while ((int32_t)(ld_relaxed_sys(mine) - epoch) < 0) {
      if ((++spins & 0xff) == 0) {
        const unsigned long long now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > WAIT_TIMEOUT_NS) {
          atomicCAS(p.status, 0, STATUS_TIMEOUT_PEER_FLAG);
          ok = false;
          break;
        }
      }
    }
    __threadfence_system();
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

template <int VPT>
__global__ void __launch_bounds__(256) fused_reduce_residual_norm_kernel(const FusedReduceParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  __shared__ uint32_t s_epoch;
  __shared__ float red[8];
  if (threadIdx.x == 0) {
    s_epoch = p.epoch[b];
    p.epoch[b] = s_epoch + 2;
  }
  __syncthreads();
  const uint32_t e0 = s_epoch;
  if (!cross_rank_barrier(p, b, e0 + 1)) return;      // peers' partial results are complete

  const int nvec = p.H / 8;
  const int row_lo = p.rank * p.rows_per_rank;
  const int row_hi = min(p.M, row_lo + p.rows_per_rank);
  for (int row = row_lo + b; row < row_hi; row += gridDim.x) {
    const size_t off = (size_t)row * p.H;
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * 256;
      if (idx < nvec) {
        float a[8];
        if (p.mc_partial != nullptr) {
          const uint4 r = multimem_ld_reduce_bf16x8(p.mc_partial + off + idx * 8);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h2[j]); a[2 * j] = f.x; a[2 * j + 1] = f.y; }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] = 0.f;
          for (int q = 0; q < p.world; ++q) {
            const uint4 r = ld_relaxed_sys_v4(p.partial[q] + off + idx * 8);
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h2[j]); a[2 * j] += f.x; a[2 * j + 1] += f.y; }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] = bf16_round(a[j]);
        }
        uint4 hr = make_uint4(0, 0, 0, 0);
        if (p.add_residual) hr = *reinterpret_cast<const uint4*>(p.h + off + idx * 8);
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&hr);
        uint4 ho;
        __nv_bfloat162* ho2 = reinterpret_cast<__nv_bfloat162*>(&ho);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(hh[j]);
          const float x0 = bf16_round(a[2 * j] + f.x), x1 = bf16_round(a[2 * j + 1] + f.y);
          v[i][2 * j] = x0;
          v[i][2 * j + 1] = x1;
          ss += x0 * x0 + x1 * x1;
          ho2[j] = __floats2bfloat162_rn(x0, x1);
        }
        *reinterpret_cast<uint4*>(p.h + off + idx * 8) = ho;
      }
    }
    ss = warp_sum(ss);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float rstd = rsqrtf(tot / (float)p.H + p.eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * 256;
      if (idx < nvec) {
        const uint4 wv = *reinterpret_cast<const uint4*>(p.ln_w + idx * 8);
        const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = __bfloat1622float2(wh[j]);
          oh[j] = __floats2bfloat162_rn(g.x * bf16_round(v[i][2 * j] * rstd), g.y * bf16_round(v[i][2 * j + 1] * rstd));
        }
        if (p.mc_xout != nullptr) {
          multimem_st_v4(p.mc_xout + off + idx * 8, o);
        } else {
          for (int q = 0; q < p.world; ++q) *reinterpret_cast<uint4*>(p.xout[q] + off + idx * 8) = o;
        }
      }
    }
  }
  cross_rank_barrier(p, b, e0 + 2);                   // every rank's rows have landed everywhere
}

// ---------------------------------------------------------------------------------------------
// Push-based variant (decode ticks).  The row-parallel GEMM has already done the reduce-scatter:
// its epilogue stored every rank's partial rows into the OWNER's slot buffer
// slot[src][row - row_lo][H] over NVLink and advanced the owner's arrival counter (gemm_tcgen05.cu,
// push_rows).  This kernel therefore reads local memory only:
//
//   wait until the counter shows that all world * (H / 128) tile columns of the owned rows arrived,
//   sum the `world` slots in rank order, add the residual, RMS-normalise, broadcast the normalised
//   row to every rank's x buffer (`multimem.st` or peer stores), fence, and advance each peer's
//   landing flag xflag[peer][this rank] by the rows written.
//
// Consumers (the column-parallel GEMM's TMA producer, lora_a_rows) wait on those flags themselves,
// so the critical path per layer half is two one-way NVLink trips and no kernel-wide barrier.
// Targets are local state advanced by the last CTA to finish (all CTAs read them at their start).
// With `final_wait` the kernel also waits for the peers' rows itself, for consumers that cannot.
// ---------------------------------------------------------------------------------------------
struct PushReduceParams {
  const __nv_bfloat16* slot;                      // local [world][rpr][H]
  uint32_t* cnt;                                  // local arrival counter (peers add rows received)
  uint32_t* cnt_target;                           // local state: counter value that completes this use
  __nv_bfloat16* xout[COMM_MAX_RANKS];            // every rank's x buffer [M, H]
  __nv_bfloat16* mc_xout;                         // multicast address of the x buffer or nullptr
  uint32_t* xflag[COMM_MAX_RANKS];                // every rank's landing flags [world] (indexed by owner)
  uint32_t* xtarget;                              // local state [world]: consumers' targets for this use
  uint32_t* arrive;                               // local CTA arrival counter for the last-CTA update
  __nv_bfloat16* h;
  const __nv_bfloat16* ln_w;
  int* status;
  int M, H, rank, world, rpr;
  float eps;
  int add_residual, final_wait;
  // Optional tap of the updated residual stream (a learned decider reads hidden states of chosen layers on every
  // rank): the owner also stores its rows of h into every rank's tap buffer (row pitch tap_ld elements, pointers
  // already at the tap's column), before the same fence and landing flags as the normalised rows.
  __nv_bfloat16* tap[COMM_MAX_RANKS];
  __nv_bfloat16* mc_tap;
  long long tap_ld;                               // 0 = no tap
};

template <int VPT>
__global__ void __launch_bounds__(256) push_reduce_norm_bcast_kernel(const PushReduceParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[8];
  __shared__ int s_ok;
  const int b = blockIdx.x;
  const int row_lo = p.rank * p.rpr;
  const int row_hi = min(p.M, row_lo + p.rpr);
  const int rows_owned = max(0, row_hi - row_lo);
  if (threadIdx.x == 0) {
    // all partial tiles of my rows have arrived: world sources x (H / 128) column tiles x rows
    const uint32_t want = *p.cnt_target + (uint32_t)(p.world * (p.H / 128) * rows_owned);
    uint32_t tgt[1] = {want};
    s_ok = wait_peer_rows(p.cnt, tgt, 1, p.status) ? 1 : 0;
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  const int nvec = p.H / 8;
  int rows_done = 0;
  for (int row = row_lo + b; ok && row < row_hi; row += gridDim.x) {
    ++rows_done;
    const size_t off = (size_t)row * p.H;
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * 256;
      if (idx < nvec) {
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = 0.f;
        for (int q = 0; q < p.world; ++q) {
          const uint4 r = ld_relaxed_sys_v4(p.slot + ((size_t)q * p.rpr + (row - row_lo)) * p.H + idx * 8);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h2[j]); a[2 * j] += f.x; a[2 * j + 1] += f.y; }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = bf16_round(a[j]);
        uint4 hr = make_uint4(0, 0, 0, 0);
        if (p.add_residual) hr = *reinterpret_cast<const uint4*>(p.h + off + idx * 8);
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&hr);
        uint4 ho;
        __nv_bfloat162* ho2 = reinterpret_cast<__nv_bfloat162*>(&ho);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(hh[j]);
          const float x0 = bf16_round(a[2 * j] + f.x), x1 = bf16_round(a[2 * j + 1] + f.y);
          v[i][2 * j] = x0;
          v[i][2 * j + 1] = x1;
          ss += x0 * x0 + x1 * x1;
          ho2[j] = __floats2bfloat162_rn(x0, x1);
        }
        *reinterpret_cast<uint4*>(p.h + off + idx * 8) = ho;
        if (p.tap_ld != 0) {
          const size_t toff = (size_t)row * (size_t)p.tap_ld + idx * 8;
          if (p.mc_tap != nullptr) {
            multimem_st_v4(p.mc_tap + toff, ho);
          } else {
            for (int q = 0; q < p.world; ++q) *reinterpret_cast<uint4*>(p.tap[q] + toff) = ho;
          }
        }
      }
    }
    ss = warp_sum(ss);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float rstd = rsqrtf(tot / (float)p.H + p.eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * 256;
      if (idx < nvec) {
        const uint4 wv = *reinterpret_cast<const uint4*>(p.ln_w + idx * 8);
        const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wv);
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = __bfloat1622float2(wh[j]);
          oh[j] = __floats2bfloat162_rn(g.x * bf16_round(v[i][2 * j] * rstd), g.y * bf16_round(v[i][2 * j + 1] * rstd));
        }
        if (p.mc_xout != nullptr) {
          multimem_st_v4(p.mc_xout + off + idx * 8, o);
        } else {
          for (int q = 0; q < p.world; ++q) *reinterpret_cast<uint4*>(p.xout[q] + off + idx * 8) = o;
        }
      }
    }
  }
  // my rows have been written everywhere: tell every rank how many landed from this owner
  __syncthreads();
  if ((int)threadIdx.x < p.world && rows_done > 0) {
    __threadfence_system();
    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p.xflag[threadIdx.x] + p.rank), "r"((uint32_t)rows_done)
                 : "memory");
  }
  // the last CTA of this launch advances the local targets for the next use
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(p.arrive, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) {
      *p.cnt_target += (uint32_t)(p.world * (p.H / 128) * rows_owned);
      *p.arrive = 0;
    }
    if ((int)threadIdx.x < p.world) {
      const int q = threadIdx.x;
      const int q_rows = max(0, min(p.M, (q + 1) * p.rpr) - q * p.rpr);
      p.xtarget[q] += (uint32_t)q_rows;
    }
    __syncthreads();
    if (p.final_wait && threadIdx.x == 0) {
      __threadfence();
      wait_peer_rows(p.xflag[p.rank], p.xtarget, p.world, p.status);
    }
  }
}

}  // namespace tahb

using namespace tahb;

// partial / xout / flags: arrays of `world` device pointers (entry `rank` is the local buffer).
// mc_partial / mc_xout: NVLS multicast addresses of the same buffers, or null for the peer-load /
// peer-store path.  epoch: local uint32[grid] zero-initialised once; flags: uint32[grid * world]
// per rank, zero-initialised once.  The grid (`grid` CTAs, <= 592) must be equal on all ranks.
extern "C" int tahb_fused_reduce_residual_norm(void* const* partial, void* const* xout, void* mc_partial,
                                               void* mc_xout, void* h, const void* ln_w, void* const* flags,
                                               void* epoch, int* status, int M, int H, int rank, int world,
                                               float eps, int add_residual, int grid, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (world < 1 || world > COMM_MAX_RANKS || H % 8) return -1;
  FusedReduceParams p;
  for (int q = 0; q < COMM_MAX_RANKS; ++q) {
    const int qq = q < world ? q : 0;
    p.partial[q] = reinterpret_cast<const __nv_bfloat16*>(partial[qq]);
    p.xout[q] = reinterpret_cast<__nv_bfloat16*>(xout[qq]);
    p.flags[q] = reinterpret_cast<uint32_t*>(flags[qq]);
  }
  p.mc_partial = reinterpret_cast<const __nv_bfloat16*>(mc_partial);
  p.mc_xout = reinterpret_cast<__nv_bfloat16*>(mc_xout);
  p.h = reinterpret_cast<__nv_bfloat16*>(h);
  p.ln_w = reinterpret_cast<const __nv_bfloat16*>(ln_w);
  p.epoch = reinterpret_cast<uint32_t*>(epoch);
  p.status = status;
  p.M = M; p.H = H; p.rank = rank; p.world = world;
  p.rows_per_rank = (M + world - 1) / world;
  p.eps = eps;
  p.add_residual = add_residual;
  const int nvec = H / 8;
  if (grid < 1) grid = 1;
  cudaError_t e;
  if (nvec <= 256) e = launch_chain(fused_reduce_residual_norm_kernel<1>, dim3(grid), dim3(256), 0, stream, p);
  else if (nvec <= 512) e = launch_chain(fused_reduce_residual_norm_kernel<2>, dim3(grid), dim3(256), 0, stream, p);
  else if (nvec <= 1024) e = launch_chain(fused_reduce_residual_norm_kernel<4>, dim3(grid), dim3(256), 0, stream, p);
  else return -2;
  return e == cudaSuccess ? 0 : -3;
}


// Push-based reduce + residual + RMSNorm + broadcast (see push_reduce_norm_bcast_kernel).
// slot / cnt / cnt_target / xtarget / arrive / h are local; xout / xflag are arrays of `world`
// pointers (peer addresses).  Rows are dealt out in blocks of `rpr`.  `tap` (optional): `world` pointers to
// the column of every rank's tap buffer that receives the updated residual rows (16-byte aligned, row pitch
// tap_ld elements), `mc_tap` its multicast address or null.
extern "C" int tahb_push_reduce_norm_bcast(const void* slot, void* cnt, void* cnt_target, void* const* xout,
                                           void* mc_xout, void* const* xflag, void* xtarget, void* arrive, void* h,
                                           const void* ln_w, int* status, int M, int H, int rank, int world, int rpr,
                                           float eps, int add_residual, int final_wait, int grid,
                                           cudaStream_t stream, void* const* tap, void* mc_tap, long long tap_ld) {
  if (M <= 0) return 0;
  if (world < 1 || world > COMM_MAX_RANKS || H % 128 || rpr <= 0) return -1;
  if (tap != nullptr && (tap_ld < H || tap_ld % 8)) return -1;
  PushReduceParams p;
  for (int q = 0; q < COMM_MAX_RANKS; ++q)
    p.tap[q] = tap != nullptr ? reinterpret_cast<__nv_bfloat16*>(tap[q < world ? q : 0]) : nullptr;
  p.mc_tap = tap != nullptr ? reinterpret_cast<__nv_bfloat16*>(mc_tap) : nullptr;
  p.tap_ld = tap != nullptr ? tap_ld : 0;
  p.slot = reinterpret_cast<const __nv_bfloat16*>(slot);
  p.cnt = reinterpret_cast<uint32_t*>(cnt);
  p.cnt_target = reinterpret_cast<uint32_t*>(cnt_target);
  for (int q = 0; q < COMM_MAX_RANKS; ++q) {
    const int qq = q < world ? q : 0;
    p.xout[q] = reinterpret_cast<__nv_bfloat16*>(xout[qq]);
    p.xflag[q] = reinterpret_cast<uint32_t*>(xflag[qq]);
  }
  p.mc_xout = reinterpret_cast<__nv_bfloat16*>(mc_xout);
  p.xtarget = reinterpret_cast<uint32_t*>(xtarget);
  p.arrive = reinterpret_cast<uint32_t*>(arrive);
  p.h = reinterpret_cast<__nv_bfloat16*>(h);
  p.ln_w = reinterpret_cast<const __nv_bfloat16*>(ln_w);
  p.status = status;
  p.M = M; p.H = H; p.rank = rank; p.world = world; p.rpr = rpr;
  p.eps = eps;
  p.add_residual = add_residual;
  p.final_wait = final_wait;
  const int nvec = H / 8;
  if (grid < 1) grid = 1;
  cudaError_t e;
  if (nvec <= 256) e = launch_chain(push_reduce_norm_bcast_kernel<1>, dim3(grid), dim3(256), 0, stream, p);
  else if (nvec <= 512) e = launch_chain(push_reduce_norm_bcast_kernel<2>, dim3(grid), dim3(256), 0, stream, p);
  else if (nvec <= 1024) e = launch_chain(push_reduce_norm_bcast_kernel<4>, dim3(grid), dim3(256), 0, stream, p);
  else return -2;
  return e == cudaSuccess ? 0 : -3;
}

// ---------------------------------------------------------------------------------------------
// Sharded-parameter all-gather by push, consumed by the GEMM through landing flags.
//
// Every rank keeps 1/world of a weight matrix (a contiguous block of rows).  Ahead of the layer that
// needs the matrix, each rank launches this kernel on a side stream: it copies its shard into the
// gather buffer of EVERY rank (its own included) at its row offset - `multimem.st` when the buffer has
// a multicast mapping, peer stores otherwise - fences, and advances landed[peer][this rank] by one per
// CTA.  The consuming GEMM (tahb_gemm_tp with wait_flag = landed, wait_target = target) starts its TMA
// loads only once every rank's CTAs have reported, so there is no separate all-gather step and no
// host synchronisation; the copy overlaps the layers before it.
//
// Re-use of a gather buffer: a rank may only overwrite its peers' buffer once they have finished the
// GEMM that read the previous contents.  Each rank launches this kernel after its own previous reader
// in stream order (an event), so at kernel entry "I am done with the buffer" holds locally; CTA 0
// tells every peer (ready[peer][this rank] = use) and waits until all peers said the same, then opens a
// local gate that the other CTAs wait on.  All waits are bounded.  The grid must be co-resident.
// ---------------------------------------------------------------------------------------------
namespace tahb {

struct ShardGatherParams {
  const uint4* src;                      // local shard
  uint4* dst[COMM_MAX_RANKS];            // every rank's gather buffer + this rank's offset
  uint4* mc_dst;                         // multicast address of the same place, or nullptr
  uint32_t* landed[COMM_MAX_RANKS];      // every rank's landing flags [world] (indexed by source rank)
  uint32_t* ready[COMM_MAX_RANKS];       // every rank's buffer-free flags [world] (indexed by source rank)
  uint32_t* target;                      // local [world]: landing targets the consumer waits for
  uint32_t* state;                       // local [3]: use counter, CTA arrivals, gate
  long long n16;                         // shard size in 16-byte units
  int rank, world;
  int* status;
};

__global__ void __launch_bounds__(256) shard_gather_push_kernel(const ShardGatherParams p) {
  __shared__ int s_ok;
  const uint32_t use = p.state[0] + 1;               // this launch's sequence number (same on all ranks)
  if (blockIdx.x == 0) {
    bool ok = true;
    if ((int)threadIdx.x < p.world) {
      const int q = threadIdx.x;
      __threadfence_system();
      st_relaxed_sys(p.ready[q] + p.rank, use);
      const uint32_t* mine = p.ready[p.rank] + q;
      unsigned long long t0 = 0;
      uint32_t spins = 0;
      while ((int32_t)(ld_relaxed_sys(mine) - use) < 0) {
        if ((++spins & 0xff) == 0) {
          const unsigned long long now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > WAIT_TIMEOUT_NS) { atomicCAS(p.status, 0, STATUS_TIMEOUT_PEER_FLAG); ok = false; break; }
        }
      }
      __threadfence_system();
    }
    const int all_ok = __syncthreads_and(ok ? 1 : 0);
    if (threadIdx.x == 0) {
      __threadfence();
      atomicExch(&p.state[2], all_ok ? use : 0x80000000u | use);    // open the gate (or report failure)
    }
  }
  if (threadIdx.x == 0) {
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    int ok = 1;
    while (true) {
      const uint32_t g = *reinterpret_cast<volatile uint32_t*>(&p.state[2]);
      if (g == use) break;
      if (g == (0x80000000u | use)) { ok = 0; break; }
      if ((++spins & 0xff) == 0) {
        const unsigned long long now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > WAIT_TIMEOUT_NS) { atomicCAS(p.status, 0, STATUS_TIMEOUT_PEER_FLAG); ok = 0; break; }
      }
    }
    __threadfence();
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < p.n16; i += stride) {
      const uint4 v = p.src[i];
      if (p.mc_dst != nullptr) {
        multimem_st_v4(p.mc_dst + i, v);
      } else {
        for (int q = 0; q < p.world; ++q) p.dst[q][i] = v;
      }
    }
    __syncthreads();
    if ((int)threadIdx.x < p.world) {
      __threadfence_system();
      asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p.landed[threadIdx.x] + p.rank), "r"(1u) : "memory");
    }
  }
  // last CTA: advance the consumer's targets and the use counter for the next launch
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(&p.state[1], 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    if ((int)threadIdx.x < p.world) p.target[threadIdx.x] += gridDim.x;
    if (threadIdx.x == 0) { p.state[0] = use; p.state[1] = 0; }
  }
}

// ---------------------------------------------------------------------------------------------
// Vocabulary-parallel top-k / arg-max merge without a library collective.
//
// Every rank holds, per row, a sorted (value desc, index asc) list of k candidates over its
// vocabulary shard.  One launch per rank, one CTA per row:
//   1. CTA r stores its row's k (value, global index) pairs into slot [epoch parity][rank][r] of every
//      rank's symmetric exchange buffer (plain peer stores over NVLink), fences, and writes this call's epoch
//      into word [r][its own rank] of every rank's arrival array (one word per row and source: a count shared
//      by the sources could be completed by a fast peer's next call while a slow peer's delivery is missing);
//   2. it waits (bounded) until all `world` words of its own arrival row r have reached the epoch, i.e. CTA r
//      of every rank has delivered this call's candidates;
//   3. it merges the `world` sorted lists: each candidate's global rank is its own index plus, for every
//      other list, the number of entries that precede it (binary search), and the first k go to the output.
// The epoch is a per-row counter in local memory that the kernel advances itself, so the launch can be
// replayed from a CUDA graph; a peer can be at most one call ahead of a CTA that is still merging, hence
// the two slots.  k <= 128, world <= 8.
// ---------------------------------------------------------------------------------------------
constexpr int MERGE_MAX_K = 128;

struct TopkMergeParams {
  float* xval[COMM_MAX_RANKS];        // every rank's exchange buffer: values [2][world][rows][MERGE_MAX_K]
  int* xidx[COMM_MAX_RANKS];          // indices, same layout
  uint32_t* arrive[COMM_MAX_RANKS];   // every rank's arrival words [rows][COMM_MAX_RANKS] (indexed by source rank)
  uint32_t* epoch;                    // local [rows]
  const float* val;                   // local candidates [rows, ldv]
  const int* idx;
  float* out_val;                     // merged [rows, ldo] (may be nullptr when only indices are wanted)
  int* out_idx;
  int* status;
  int rows, k, ldv, ldo, rank, world, vocab_lo;
  unsigned long long wait_limit_ns;
};

__device__ __forceinline__ bool cand_before(float va, int ia, float vb, int ib) {
  return va > vb || (va == vb && ia < ib);
}

__global__ void __launch_bounds__(256) tp_topk_merge_kernel(const TopkMergeParams p) {
  __shared__ float sv[COMM_MAX_RANKS * MERGE_MAX_K];
  __shared__ int si[COMM_MAX_RANKS * MERGE_MAX_K];
  __shared__ int s_ok;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  const int k = p.k, W = p.world;
  const uint32_t ep = p.epoch[r] + 1;
  const int par = ep & 1;
  // 1. deliver this rank's candidates to every rank (own copy included)
  for (int j = tid; j < k * W; j += blockDim.x) {
    const int q = j / k, c = j % k;
    const size_t off = (((size_t)par * W + p.rank) * p.rows + r) * MERGE_MAX_K + c;
    p.xval[q][off] = p.val[(size_t)r * p.ldv + c];
    p.xidx[q][off] = p.idx[(size_t)r * p.ldv + c] + p.vocab_lo;
  }
  __syncthreads();
  if (tid < W) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.arrive[tid] + (size_t)r * COMM_MAX_RANKS + p.rank), "r"(ep)
                 : "memory");
  }
  // 2. wait for every rank's delivery of this call
  if (tid == 0) {
    const uint32_t* mine = p.arrive[p.rank] + (size_t)r * COMM_MAX_RANKS;
    const unsigned long long limit = p.wait_limit_ns ? p.wait_limit_ns : WAIT_TIMEOUT_NS;
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    int ok = 1;
    int src = 0;                       // sources 0 .. src - 1 have delivered
    while (src < W) {
      if ((int32_t)(ld_acquire_sys(mine + src) - ep) >= 0) { ++src; continue; }
      if ((++spins & 0xff) == 0) {
        const unsigned long long now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > limit) {
          atomicCAS(p.status, 0, STATUS_TIMEOUT_PEER_FLAG);
          ok = 0;
          break;
        }
      }
    }
    __threadfence_system();
    s_ok = ok;
    p.epoch[r] = ep;
  }
  __syncthreads();
  if (!s_ok) return;
  // 3. merge
  const float* lv = p.xval[p.rank] + ((size_t)par * W * p.rows + r) * MERGE_MAX_K;
  const int* li = p.xidx[p.rank] + ((size_t)par * W * p.rows + r) * MERGE_MAX_K;
  const size_t qstride = (size_t)p.rows * MERGE_MAX_K;
  for (int j = tid; j < k * W; j += blockDim.x) {
    const int q = j / k, c = j % k;
    sv[q * MERGE_MAX_K + c] = __uint_as_float(ld_relaxed_sys(reinterpret_cast<const uint32_t*>(lv + q * qstride + c)));
    si[q * MERGE_MAX_K + c] = (int)ld_relaxed_sys(reinterpret_cast<const uint32_t*>(li + q * qstride + c));
  }
  __syncthreads();
  for (int j = tid; j < k * W; j += blockDim.x) {
    const int q = j / k, c = j % k;
    const float v = sv[q * MERGE_MAX_K + c];
    const int ix = si[q * MERGE_MAX_K + c];
    int rank_g = c;
    for (int o = 0; o < W; ++o) {
      if (o == q) continue;
      // number of entries of list o that come before (v, ix): lists are sorted, binary search
      int lo = 0, hi = k;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (cand_before(sv[o * MERGE_MAX_K + mid], si[o * MERGE_MAX_K + mid], v, ix)) lo = mid + 1;
        else hi = mid;
      }
      rank_g += lo;
    }
    if (rank_g < k) {
      if (p.out_val != nullptr) p.out_val[(size_t)r * p.ldo + rank_g] = v;
      p.out_idx[(size_t)r * p.ldo + rank_g] = ix;
    }
  }
}

}  // namespace tahb

// src: local shard (`bytes`, a multiple of 16); dst: `world` pointers to the place of this rank's shard in
// every rank's gather buffer; mc_dst: the multicast address of that place or null; landed / ready: `world`
// pointers to every rank's flag arrays; target / state: local device arrays ([world] and [3] uint32, zeroed
// once).  The same grid (<= 148 CTAs) on every rank.
extern "C" int tahb_shard_gather_push(const void* src, void* const* dst, void* mc_dst, void* const* landed,
                                      void* const* ready, void* target, void* state, long long bytes, int rank,
                                      int world, int grid, int* status, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  if (world < 1 || world > COMM_MAX_RANKS || bytes % 16 || grid < 1 || grid > 148) return -1;
  ShardGatherParams p;
  p.src = reinterpret_cast<const uint4*>(src);
  for (int q = 0; q < COMM_MAX_RANKS; ++q) {
    const int qq = q < world ? q : 0;
    p.dst[q] = reinterpret_cast<uint4*>(dst[qq]);
    p.landed[q] = reinterpret_cast<uint32_t*>(landed[qq]);
    p.ready[q] = reinterpret_cast<uint32_t*>(ready[qq]);
  }
  p.mc_dst = reinterpret_cast<uint4*>(mc_dst);
  p.target = reinterpret_cast<uint32_t*>(target);
  p.state = reinterpret_cast<uint32_t*>(state);
  p.n16 = bytes / 16;
  p.rank = rank; p.world = world;
  p.status = status;
  shard_gather_push_kernel<<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Merge per-shard sorted top-k candidate lists over the ranks of a tensor-parallel group (see
// tp_topk_merge_kernel).  xval / xidx / arrive: the `world` peer pointers of the symmetric exchange
// buffers; epoch: local per-row counters; val / idx: this rank's [rows, ldv] candidates (local indices,
// vocab_lo is added); out_val (optional) / out_idx: merged [rows, ldo] lists with global indices.
extern "C" int tahb_tp_topk_merge(void* const* xval, void* const* xidx, void* const* arrive, void* epoch,
                                  const float* val, const int* idx, float* out_val, int* out_idx, int* status,
                                  int rows, int k, int ldv, int ldo, int rank, int world, int vocab_lo,
                                  cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (k < 1 || k > MERGE_MAX_K || world < 1 || world > COMM_MAX_RANKS) return -1;
  TopkMergeParams p;
  for (int q = 0; q < COMM_MAX_RANKS; ++q) {
    p.xval[q] = q < world ? reinterpret_cast<float*>(xval[q]) : nullptr;
    p.xidx[q] = q < world ? reinterpret_cast<int*>(xidx[q]) : nullptr;
    p.arrive[q] = q < world ? reinterpret_cast<uint32_t*>(arrive[q]) : nullptr;
  }
  p.epoch = reinterpret_cast<uint32_t*>(epoch);
  p.val = val; p.idx = idx; p.out_val = out_val; p.out_idx = out_idx; p.status = status;
  p.rows = rows; p.k = k; p.ldv = ldv; p.ldo = ldo; p.rank = rank; p.world = world; p.vocab_lo = vocab_lo;
  p.wait_limit_ns = peer_wait_limit_ns();
  cudaError_t e = launch_chain(tp_topk_merge_kernel, dim3(rows), dim3(256), 0, stream, p);
  return e == cudaSuccess ? 0 : -3;
}
