// Context-parallel helpers: segment task planning, state-map scan, output fix-up, state row copies (see kda_cp.cu).
#pragma once
#include "kda_common.cuh"

namespace kda {

struct SegPlanParams {
  int n_seg, H;
  long long T;
  const long long* t0;
  const long long* t1;
  const int* need_map;
  const float* src_base; long long src_stride;
  int no_out;      // maps only: neither chain writes output rows
  int dual;        // 1: a mapped segment is ONE dual-chain task (tcgen05 kernel only); 0: two tasks, chains L and Tr
  float* P;
  float* S_loc;
  __nv_bfloat16* tiles;  // dual with output: tile-major scratch (Qt tiles; the o_loc tiles follow at ChunkParams::oloc_tile_offset)
  Task* tasks;     // [2 * n_seg] (dual: n_seg used)
  int* n_tasks;
  int* status;
};

cudaError_t launch_seg_plan(const SegPlanParams& a, cudaStream_t stream);
// map_stride: floats between consecutive maps of P and of S_loc (0 = H * 16384, i.e. packed)
cudaError_t launch_scan(const float* P, const float* S_loc, const float* S0, float* S_in, float* S_end, int n_seg, int H,
                        long long map_stride, cudaStream_t stream);
cudaError_t launch_fixup(__nv_bfloat16* out, const __nv_bfloat16* qt, long long ldo, const float* S_in, const long long* t0,
                         const long long* t1, const int* need_map, int n_seg, int H, cudaStream_t stream);
// the same pass over the tile-major output of dual-chain tasks: out rows = o_loc tile + Qt tile applied to the entering state
cudaError_t launch_fixup_tiles(__nv_bfloat16* out, const __nv_bfloat16* tiles, long long oloc_tile_offset, long long ldo,
                               const float* S_in, const long long* t0, const long long* t1, const int* need_map, int n_seg,
                               int H, long long T, cudaStream_t stream);
cudaError_t launch_rows_copy(void* dst, long long dst_row_stride, int dst_is_bf16, const float* src, long long src_row_stride,
                             const int* idx, int n_rows, int H, cudaStream_t stream);

}  // namespace kda
