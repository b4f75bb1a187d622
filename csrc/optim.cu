// ZeRO-style sharded AdamW fused with its collectives over NVLink peer memory.
//
// Every rank holds the full bf16 parameters and the full bf16 gradients of the trainable set in
// two flat *symmetric* buffers (same layout on every rank), and the fp32 master weights and Adam
// moments of its own 1/world shard.  One optimizer step is two launches per rank:
//
//   zero_reduce_norm    gradient reduce-scatter: a rank sums ITS shard of the gradient over all
//                       ranks' buffers (NVLS multimem.ld_reduce, or one peer load per rank),
//                       scales it (1 / world / accumulation), keeps it in fp32 and adds its
//                       squared norm to a device scalar (for global-norm clipping).
//   zero_adamw_bcast    clip factor from the (all-reduced) squared norm, AdamW on the fp32 master
//                       shard, and the updated bf16 parameters are written straight into every
//                       rank's parameter buffer (multimem.st or peer stores): the parameter
//                       all-gather of the next step is part of the update.
//
// Cross-rank ordering uses the same flag barrier as the tensor-parallel kernels: CTA b meets CTA b
// of every rank before the gradients are read and after the parameters are written.  Bounded waits.
#include "common.cuh"

namespace tahb {

constexpr int OPT_MAX_RANKS = 8;

struct ZeroParams {
  const __nv_bfloat16* grad[OPT_MAX_RANKS];   // flat gradient buffers of all ranks (peer pointers)
  __nv_bfloat16* param[OPT_MAX_RANKS];        // flat parameter buffers of all ranks
  const __nv_bfloat16* mc_grad;               // multicast addresses or nullptr
  __nv_bfloat16* mc_param;
  float* gshard;                              // [shard] reduced, scaled gradient (fp32)
  float* master;                              // [shard] fp32 master weights
  float* m;                                   // [shard]
  float* v;                                   // [shard]
  float* norm_sq;                             // device scalar: sum of squares of the reduced gradient
  uint32_t* flags[OPT_MAX_RANKS];
  uint32_t* epoch;
  int* status;
  long long lo, hi;                           // this rank's element range (multiples of 8)
  int rank, world;
  float grad_scale, lr, beta1, beta2, eps, weight_decay, bc1, bc2, max_norm;
  long long nodecay_from;                     // flat elements at or beyond this index get no weight decay
  int accumulate;                             // reduce phase: gshard += (instead of =) and no norm (several
                                              // reduce-scatters - passes, micro-batches - feed one update)
};

__device__ __forceinline__ void zst_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t zld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool zero_barrier(const ZeroParams& p, int b, uint32_t epoch) {
  bool ok = true;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int q = 0; q < p.world; ++q) zst_release_sys(p.flags[q] + (size_t)b * p.world + p.rank, epoch);
    const uint32_t* mine = p.flags[p.rank] + (size_t)b * p.world;
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    for (int q = 0; q < p.world && ok; ++q) {
      while ((int32_t)(zld_acquire_sys(mine + q) - epoch) < 0) {
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
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

__global__ void __launch_bounds__(256) zero_reduce_norm_kernel(const ZeroParams p) {
  const int b = blockIdx.x;
  __shared__ uint32_t s_epoch;
  __shared__ float red[8];
  if (threadIdx.x == 0) {
    s_epoch = p.epoch[b];
    p.epoch[b] = s_epoch + (p.accumulate ? 2 : 1);
  }
  __syncthreads();
  if (!zero_barrier(p, b, s_epoch + 1)) return;     // every rank has finished writing its gradients
  const long long nvec = (p.hi - p.lo) / 8;
  float ss = 0.f;
  for (long long i = (long long)b * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long e = p.lo + i * 8;
    float a[8];
    if (p.mc_grad != nullptr) {
      uint4 r;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                   : "l"(p.mc_grad + e)
                   : "memory");
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h2[j]); a[2 * j] = f.x; a[2 * j + 1] = f.y; }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = 0.f;
      for (int q = 0; q < p.world; ++q) {
        uint4 r;
        asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                     : "l"(p.grad[q] + e)
                     : "memory");
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h2[j]); a[2 * j] += f.x; a[2 * j + 1] += f.y; }
      }
    }
    float4 o0, o1;
    o0.x = a[0] * p.grad_scale; o0.y = a[1] * p.grad_scale; o0.z = a[2] * p.grad_scale; o0.w = a[3] * p.grad_scale;
    o1.x = a[4] * p.grad_scale; o1.y = a[5] * p.grad_scale; o1.z = a[6] * p.grad_scale; o1.w = a[7] * p.grad_scale;
    ss += o0.x * o0.x + o0.y * o0.y + o0.z * o0.z + o0.w * o0.w + o1.x * o1.x + o1.y * o1.y + o1.z * o1.z + o1.w * o1.w;
    float4* dst = reinterpret_cast<float4*>(p.gshard + i * 8);
    if (p.accumulate) {
      const float4 c0 = dst[0], c1 = dst[1];
      o0.x += c0.x; o0.y += c0.y; o0.z += c0.z; o0.w += c0.w;
      o1.x += c1.x; o1.y += c1.y; o1.z += c1.z; o1.w += c1.w;
    }
    dst[0] = o0;
    dst[1] = o1;
  }
  if (p.accumulate) {
    // the gradient buffers are reused by another layer right away: meet the peers again so that nobody
    // overwrites a buffer that a peer is still reading; the norm is taken later over the finished sum
    zero_barrier(p, b, s_epoch + 2);
    return;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    atomicAdd(p.norm_sq, t);
  }
}

// Sum of squares of an fp32 gradient shard, added to *norm_sq (local; no cross-rank traffic).
__global__ void __launch_bounds__(256) zero_norm_kernel(const float* __restrict__ g, long long n, float* norm_sq) {
  __shared__ float red[8];
  float ss = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    ss += g[i] * g[i];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    atomicAdd(norm_sq, t);
  }
}

// One thread waits (bounded) until flag[q] has reached target[q] for every q < world: a stream-ordered gate in
// front of kernels that cannot wait themselves (library GEMMs reading a gather buffer that peers fill).
__global__ void wait_flags_kernel(const uint32_t* flag, const uint32_t* target, int world, int* status,
                                  unsigned long long limit_ns) {
  if (threadIdx.x == 0 && blockIdx.x == 0) wait_peer_rows(flag, target, world, status, limit_ns);
}

__global__ void __launch_bounds__(256) zero_adamw_bcast_kernel(const ZeroParams p) {
  const int b = blockIdx.x;
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = p.epoch[b];
    p.epoch[b] = s_epoch + 1;
  }
  __syncthreads();
  float clip = 1.0f;
  if (p.max_norm > 0.f) {
    const float norm = sqrtf(*p.norm_sq);           // all-reduced over the ranks by the host code
    clip = fminf(1.0f, p.max_norm / (norm + 1e-6f));
  }
  const long long nvec = (p.hi - p.lo) / 8;
  for (long long i = (long long)b * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float g[8], w[8], m[8], v[8];
    const float4* gp = reinterpret_cast<const float4*>(p.gshard + i * 8);
    float4* wp = reinterpret_cast<float4*>(p.master + i * 8);
    float4* mp = reinterpret_cast<float4*>(p.m + i * 8);
    float4* vp = reinterpret_cast<float4*>(p.v + i * 8);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 a = gp[h], bw = wp[h], bm = mp[h], bv = vp[h];
      g[4 * h] = a.x; g[4 * h + 1] = a.y; g[4 * h + 2] = a.z; g[4 * h + 3] = a.w;
      w[4 * h] = bw.x; w[4 * h + 1] = bw.y; w[4 * h + 2] = bw.z; w[4 * h + 3] = bw.w;
      m[4 * h] = bm.x; m[4 * h + 1] = bm.y; m[4 * h + 2] = bm.z; m[4 * h + 3] = bm.w;
      v[4 * h] = bv.x; v[4 * h + 1] = bv.y; v[4 * h + 2] = bv.z; v[4 * h + 3] = bv.w;
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * clip;
      m[j] = p.beta1 * m[j] + (1.f - p.beta1) * gj;
      v[j] = p.beta2 * v[j] + (1.f - p.beta2) * gj * gj;
      const float upd = (m[j] / p.bc1) / (sqrtf(v[j] / p.bc2) + p.eps);
      const float wd = (p.lo + i * 8 + j >= p.nodecay_from) ? 0.f : p.weight_decay;
      w[j] = w[j] * (1.f - p.lr * wd) - p.lr * upd;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(w[2 * j], w[2 * j + 1]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      wp[h] = make_float4(w[4 * h], w[4 * h + 1], w[4 * h + 2], w[4 * h + 3]);
      mp[h] = make_float4(m[4 * h], m[4 * h + 1], m[4 * h + 2], m[4 * h + 3]);
      vp[h] = make_float4(v[4 * h], v[4 * h + 1], v[4 * h + 2], v[4 * h + 3]);
    }
    const long long e = p.lo + i * 8;
    if (p.mc_param != nullptr) {
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                   ::"l"(p.mc_param + e), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w)
                   : "memory");
    } else {
      for (int q = 0; q < p.world; ++q) *reinterpret_cast<uint4*>(p.param[q] + e) = o;
    }
  }
  zero_barrier(p, b, s_epoch + 1);                  // every rank's new parameters are in place everywhere
}

}  // namespace tahb

using namespace tahb;

static void fill(ZeroParams& p, void* const* grad, void* const* param, void* mc_grad, void* mc_param, float* gshard,
                 float* master, float* m, float* v, float* norm_sq, void* const* flags, void* epoch, int* status,
                 long long lo, long long hi, int rank, int world) {
  for (int q = 0; q < OPT_MAX_RANKS; ++q) {
    const int qq = q < world ? q : 0;
    p.grad[q] = reinterpret_cast<const __nv_bfloat16*>(grad[qq]);
    p.param[q] = reinterpret_cast<__nv_bfloat16*>(param[qq]);
    p.flags[q] = reinterpret_cast<uint32_t*>(flags[qq]);
  }
  p.mc_grad = reinterpret_cast<const __nv_bfloat16*>(mc_grad);
  p.mc_param = reinterpret_cast<__nv_bfloat16*>(mc_param);
  p.gshard = gshard; p.master = master; p.m = m; p.v = v; p.norm_sq = norm_sq;
  p.epoch = reinterpret_cast<uint32_t*>(epoch);
  p.status = status;
  p.lo = lo; p.hi = hi; p.rank = rank; p.world = world;
}

// Flat index from which the NEXT tahb_zero_step launch applies no weight decay (norm gains, biases and the like
// are laid out behind the decayed parameters); reset after that launch.
static long long g_nodecay_from = 0x7fffffffffffffffLL;
extern "C" void tahb_zero_set_nodecay_from(long long index) { g_nodecay_from = index; }

// phase 0: reduce-scatter of the gradient shard [lo, hi) + scaling + squared norm (atomicAdd into *norm_sq,
// which the caller zeroes before the launch and all-reduces afterwards).  phase 1: AdamW + parameter broadcast.
// phase 2: as phase 0 but the scaled sum is ADDED to gshard and no norm is taken (parameter-sharded training
// reduce-scatters a layer's gradients once per backward pass and micro-batch into one fp32 accumulator).
extern "C" int tahb_zero_step(int phase, void* const* grad, void* const* param, void* mc_grad, void* mc_param,
                              float* gshard, float* master, float* m, float* v, float* norm_sq, void* const* flags,
                              void* epoch, int* status, long long lo, long long hi, int rank, int world,
                              float grad_scale, float lr, float beta1, float beta2, float eps, float weight_decay,
                              float bc1, float bc2, float max_norm, int grid, cudaStream_t stream) {
  if (world < 1 || world > OPT_MAX_RANKS || (lo % 8) || (hi % 8) || hi < lo) return -1;
  ZeroParams p;
  fill(p, grad, param, mc_grad, mc_param, gshard, master, m, v, norm_sq, flags, epoch, status, lo, hi, rank, world);
  p.grad_scale = grad_scale; p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps;
  p.weight_decay = weight_decay; p.bc1 = bc1; p.bc2 = bc2; p.max_norm = max_norm;
  p.accumulate = phase == 2 ? 1 : 0;
  p.nodecay_from = g_nodecay_from;
  g_nodecay_from = 0x7fffffffffffffffLL;      // one-shot: applies to this launch only
  if (grid < 1) grid = 1;
  if (phase == 0 || phase == 2) zero_reduce_norm_kernel<<<grid, 256, 0, stream>>>(p);
  else zero_adamw_bcast_kernel<<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// *norm_sq += sum of squares of the fp32 vector g[0 .. n)
extern "C" int tahb_sumsq_f32(const float* g, long long n, float* norm_sq, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 256 * 8 - 1) / (256 * 8);
  if (blocks > 148 * 4) blocks = 148 * 4;
  zero_norm_kernel<<<(int)blocks, 256, 0, stream>>>(g, n, norm_sq);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Stream-ordered bounded wait until flag[q] >= target[q] (wrap-safe) for q < world; on expiry the status word
// gets STATUS_TIMEOUT_PEER_FLAG and the stream goes on.
extern "C" int tahb_wait_flags(const void* flag, const void* target, int world, int* status, cudaStream_t stream) {
  if (world <= 0) return 0;
  wait_flags_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const uint32_t*>(flag),
                                          reinterpret_cast<const uint32_t*>(target), world, status, peer_wait_limit_ns());
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
