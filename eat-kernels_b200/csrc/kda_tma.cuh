// Tensor Memory Accelerator support: host-side tensor-map encoding (through the driver entry point, no link-time
// dependency on libcuda) and the device-side bulk tensor copy wrappers.
//
// Token tensors are described as rank-3 tensors {128 (channel), H (head), T (token)} with the caller's token stride,
// so a head slice of a wider tensor is read in place.  A tile is 32 tokens of one head.  Rows past the end of the
// tensor are zero-filled by the hardware; rows past the end of a SEQUENCE belong to the next sequence and are masked
// by the consumers.  Every copy starts at channel 0 or 64 (a multiple of 16 bytes), the alignment the copy engine
// requires of the innermost coordinate.  No multicast is used anywhere.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kda {

struct TmaMaps {
  CUtensorMap q, k, v, g;
};

// box = {box_ch channels, 1 head, 32 tokens}; swizzle128 selects the 128-byte swizzle (box_ch * elem_bytes must be 128)
inline int encode_token_map(CUtensorMap* map, const void* base, int elem_bytes, bool is_float, long long T, int H, long long ld_elems,
                            int box_ch, bool swizzle128) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || ptr == nullptr) return -1;
    fn = reinterpret_cast<EncodeFn>(ptr);
  }
  const cuuint64_t dims[3] = {128, (cuuint64_t)H, (cuuint64_t)T};
  const cuuint64_t strides[2] = {(cuuint64_t)128 * elem_bytes, (cuuint64_t)ld_elems * elem_bytes};
  const cuuint32_t box[3] = {(cuuint32_t)box_ch, 1, 32};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = is_float ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

#ifdef __CUDACC__
namespace tma {

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" :: "r"(bar), "r"(bytes) : "memory");
}
// global -> shared tile copy, completion (bytes) reported to the mbarrier
__device__ __forceinline__ void load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
               :: "r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}

}  // namespace tma
#endif

}  // namespace kda
