// Pieces shared by the packed attention kernels (forward: attn_prefill.cu, backward:
// attn_prefill_bwd.cu): the MN-major shared-memory descriptor, the matching instruction
// descriptors, and the tensor-map helper for [rows, cols] bf16 matrices read in 64-column boxes.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace tahb {

constexpr int PF_MAX_SEG = 3;

// MN-major bf16 operand (the N/M dimension is contiguous): rows of 64 elements (128 B) per K index,
// 128-byte swizzle, 8 K-rows per 1024-byte group (SBO), next 64 MN elements `lbo_bytes` further.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>(64) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// bf16 x bf16 -> fp32, A K-major, B MN-major
__host__ __device__ constexpr uint32_t umma_idesc_bf16_bmn(int m, int n) {
  return umma_idesc_bf16(m, n) | (1u << 16);
}

// bf16 x bf16 -> fp32, A MN-major, B MN-major / A MN-major, B K-major are not used by these kernels.

typedef CUresult (*PfEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline int pf_make_map(CUtensorMap* m, const void* base, long long rows, long long cols, unsigned box_rows) {
  static PfEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return -1;
    fn = reinterpret_cast<PfEncodeFn>(ptr);
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((cols * 2) & 15)) return -2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64u, box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace tahb
