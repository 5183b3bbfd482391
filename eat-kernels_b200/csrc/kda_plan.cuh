// Parameters of the device planner (see kda_plan.cu).
#pragma once
#include "kda_common.cuh"
#include "kda_tma.cuh"

namespace kda {

constexpr int KDA_BIT_CU = 1, KDA_BIT_SLOT = 2, KDA_BIT_SOURCE = 4, KDA_BIT_CKPT = 8, KDA_BIT_RANGE = 16;

struct PlanParams {
  int N, H;
  long long T;
  const void* cu; int cu_is64;
  const float* src_base; long long src_stride; const void* src_idx; int src_is64; long long src_slots;
  int src_separate;   // no source table: 1 = sequence i starts from source slot i, 0 = from its destination slot (in place)
  float* dst_base; long long dst_stride; const void* dst_idx; int dst_is64; long long dst_slots;
  void* ck_base; int ck_is_bf16; int ck_every; long long ck_rows; long long ck_row_stride;
  const void* ck_starts; int ck_is64;
  float* trash;             // [H][128][128] scratch state window for rejected destination slots
  long long* cu_safe;       // [N+1]
  Task* tasks_unsorted;     // [N]
  Task* tasks;              // [N] longest first
  int* n_tasks;
  int* status;              // int[4]
};

cudaError_t launch_plan(const PlanParams& a, cudaStream_t stream);
cudaError_t launch_chunk_fwd(const ChunkParams& p, int n_task_cap, cudaStream_t stream);    // mma.sync kernel
cudaError_t launch_chunk_umma(const ChunkParams& p, const TmaMaps& maps, int n_task_cap, cudaStream_t stream);   // tcgen05 kernel

}  // namespace kda
