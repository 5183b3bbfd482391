// Parameters of the device planner (see kda_plan.cu).
#pragma once
#include "kda_common.cuh"
#include "kda_tma.cuh"

namespace kda {

constexpr int KDA_BIT_CU = 1, KDA_BIT_SLOT = 2, KDA_BIT_SOURCE = 4, KDA_BIT_CKPT = 8, KDA_BIT_RANGE = 16;

// One cut sequence for the scan: E[k] = (k == 0 ? S0 : E[k-1]) applied to map first + k, for k < count; the map slots
// are [H][128][128] blocks `first + k` of the map arrays.
struct ScanChain {
  const float* s0;          // end state of piece 0 (head 0)
  int first, count;
};

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
  Task* tasks;              // first launch: [N + 2 * max_pieces], longest first
  int* n_tasks;
  int* status;              // int[4]
  // ---- cutting long sequences (max_pieces > 0).  A sequence cut into p pieces runs as: piece 0 from its true initial
  // state and, for pieces 1 .. p-2, the two chains of the affine state map (first launch); a scan that yields the
  // entering states of pieces 1 .. p-1; those pieces from their entering states (second launch).
  int max_pieces;           // capacity: pieces of all cut sequences together (0 = never cut)
  int n_sm;                 // SMs of the device (cost model)
  int key_first;            // state layout of the launch (the transition maps are stored value-first either way)
  int dual;                 // 1: the map of a piece is one dual-chain task (tcgen05 kernel); 0: two single-chain tasks
  int force_cand;           // tuning aid: k + 1 forces candidate k of the piece lengths (if it is valid), 0 = cost model
  Task* tasks_b;            // second launch: [2 * max_pieces] (pieces, and up to max_pieces uncut sequences for balance)
  int* n_tasks_b;
  float* map_P;             // [max_pieces][H][128][128] transition maps
  float* map_L;             // [max_pieces][H][128][128] offsets; slot 0 of a cut sequence holds piece 0's end state
  float* map_E;             // [max_pieces][H][128][128] entering states written by the scan
  ScanChain* chains;        // [max_pieces / 3 + 1]
  int* n_chains;
};

cudaError_t launch_plan(const PlanParams& a, cudaStream_t stream);
// entering states of the pieces of every cut sequence (grid sized for `max_chains`, chains beyond *n_chains exit)
cudaError_t launch_scan_chains(const ScanChain* chains, const int* n_chains, int max_chains, const float* P, const float* L, float* E,
                               int H, int key_first, cudaStream_t stream);
cudaError_t launch_chunk_fwd(const ChunkParams& p, int n_task_cap, cudaStream_t stream);    // mma.sync kernel
// tcgen05 kernel (tasks with TF_DUAL run chain L and the transition chain over one operand preparation); after_planner: the launch directly follows launch_plan / launch_seg_plan in the stream and is chained
// to it by programmatic dependent launch
cudaError_t launch_chunk_umma(const ChunkParams& p, const TmaMaps& maps, int n_task_cap, cudaStream_t stream, bool after_planner = false);

}  // namespace kda
