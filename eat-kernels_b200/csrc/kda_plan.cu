// Device-side varlen planner and table validation for the KDA prefill call (one CTA, integer work).
//
// Reads the caller's tables where they lie (cu_seqlens, slot tables, checkpoint starts: int32 or int64), never on the
// host, so a captured launch can be replayed after the tables' contents change.  Produces the task list of the fused
// chunk kernel ordered longest first (the hardware block scheduler then works as a longest-processing-time list
// scheduler) and the status bits of kda/b200/kda_b200.py:56-62.  Function of the reference's planner + validation
// launch (kda/b200/csrc/dyn/plan_cp.cu:218-270, kda/b200/csrc/w3/validate_dev.cuh:32-150); rejected entries are
// neutralised, never faulted on:
//   bit 1  cu_seqlens not 0-based / decreasing / beyond T: every sequence becomes empty
//   bit 2  destination slot out of range or already claimed by an earlier sequence: final state goes to scratch
//   bit 4  source slot out of range: the sequence starts from zeros
//   bit 8  checkpoint rows out of range or overlapping the rows an earlier sequence KEEPS: the sequence writes none.
//          Overlaps are resolved in ascending sequence order against final decisions, as the reference does
//          (kda/b200/csrc/w3/validate_dev.cuh:124-142): a sequence that lost its rows does not block later ones.
#include "kda_common.cuh"
#include "kda_plan.cuh"

namespace kda {

constexpr int PLAN_THREADS = 1024;
constexpr int SORT_MAX = 4096;

__device__ __forceinline__ long long rd_table(const void* p, int is64, long long i) {
  return is64 ? reinterpret_cast<const long long*>(p)[i] : (long long)reinterpret_cast<const int*>(p)[i];
}

__global__ void __launch_bounds__(PLAN_THREADS, 1) kda_plan_kernel(const PlanParams a) {
  __shared__ unsigned long long keys[SORT_MAX];
  __shared__ unsigned char s_keep[SORT_MAX];     // checkpoint rows of sequence i: 0 = none / rejected, 1 = kept
  __shared__ int s_bits, s_overlap;
  const int tid = threadIdx.x, bd = blockDim.x, N = a.N;
  if (tid == 0) { s_bits = 0; s_overlap = 0; }
  __syncthreads();
  // rows [v, v + cnt) of sequence i and whether they lie inside the checkpoint buffer
  auto ck_range = [&](int i, long long& v, long long& cnt) -> bool {
    const long long len = a.cu_safe[i + 1] - a.cu_safe[i];
    cnt = (len + a.ck_every - 1) / a.ck_every;
    v = (a.ck_starts != nullptr) ? rd_table(a.ck_starts, a.ck_is64, i) : -1;
    return v >= 0 && cnt <= a.ck_rows && v <= a.ck_rows - cnt;
  };

  // ---- cu_seqlens
  bool cu_ok = true;
  for (int i = tid; i <= N; i += bd) {
    long long c0, c1;
    if (a.cu == nullptr) { c0 = (i == 0) ? 0 : a.T; c1 = a.T; }
    else { c0 = rd_table(a.cu, a.cu_is64, i); c1 = (i < N) ? rd_table(a.cu, a.cu_is64, i + 1) : c0; }
    if (c0 < 0 || c0 > a.T || c1 < c0 || (i == 0 && c0 != 0) || (i < N && c1 - c0 > 0x7fffffffLL)) cu_ok = false;
    a.cu_safe[i] = c0;
  }
  if (!cu_ok) atomicOr(&s_bits, KDA_BIT_CU);
  __syncthreads();
  const bool noop = (s_bits & KDA_BIT_CU) != 0;
  if (noop) {
    for (int i = tid; i <= N; i += bd) a.cu_safe[i] = 0;
  }
  __syncthreads();

  // ---- per-sequence tables
  for (int i = tid; i < N; i += bd) {
    const long long len = a.cu_safe[i + 1] - a.cu_safe[i];
    // destination slot
    long long d = i;
    bool d_ok = true;
    if (a.dst_idx != nullptr) {
      d = rd_table(a.dst_idx, a.dst_is64, i);
      d_ok = d >= 0 && d < a.dst_slots;
      if (d_ok) {
        for (int j = 0; j < i; j++)
          if (rd_table(a.dst_idx, a.dst_is64, j) == d) { d_ok = false; break; }   // first claim keeps the slot
      }
      if (!d_ok) atomicOr(&s_bits, KDA_BIT_SLOT);
    }
    // source slot (in place when there is no separate source table: the destination slot)
    long long s = d;
    bool s_ok = d_ok;
    if (a.src_idx != nullptr) {
      s = rd_table(a.src_idx, a.src_is64, i);
      s_ok = s >= 0 && s < a.src_slots;
      if (!s_ok) atomicOr(&s_bits, KDA_BIT_SOURCE);
    } else if (a.src_separate) {
      s = i;
      s_ok = true;
    }
    // checkpoint rows: range check here; overlaps with earlier sequences are only detected (resolved below)
    long long row = -1;
    if (a.ck_base != nullptr && a.ck_every > 0) {
      long long v, cnt;
      bool ok = ck_range(i, v, cnt);
      if (!ok) atomicOr(&s_bits, KDA_BIT_CKPT);
      if (ok && cnt > 0) {
        for (int j = 0; j < i; j++) {
          long long vj, cj;
          if (ck_range(j, vj, cj) && cj > 0 && vj < v + cnt && v < vj + cj) { s_overlap = 1; break; }
        }
      }
      if (i < SORT_MAX) s_keep[i] = ok ? 1 : 0;
      row = ok ? v : -1;
    }
    Task t;
    t.t0 = a.cu_safe[i];
    t.len = (int)len;
    t.flags = 0;
    t.src = nullptr;
    if (a.src_base == nullptr || !s_ok) t.flags |= TF_INIT_ZERO;
    else t.src = a.src_base + s * a.src_stride;
    if (a.dst_base == nullptr) t.dst = nullptr;
    else t.dst = d_ok ? a.dst_base + d * a.dst_stride : a.trash;
    if (!d_ok && a.src_idx == nullptr && !a.src_separate) {   // in place with a rejected slot: nothing to read either
      t.flags |= TF_INIT_ZERO;
      t.src = nullptr;
    }
    t.ck = nullptr;
    if (row >= 0)
      t.ck = a.ck_is_bf16 ? (void*)(reinterpret_cast<__nv_bfloat16*>(a.ck_base) + row * a.ck_row_stride)
                          : (void*)(reinterpret_cast<float*>(a.ck_base) + row * a.ck_row_stride);
    t.pad_ = 0;
    a.tasks_unsorted[i] = t;
  }
  __syncthreads();
  if (s_overlap) {
    // Malformed table (rare): one thread walks the sequences in order and drops the rows of every sequence that
    // overlaps rows an EARLIER sequence keeps.  Beyond SORT_MAX sequences the flags do not fit: then every sequence
    // that overlaps any earlier in-range sequence loses its rows (stricter, still race-free).
    if (tid == 0) {
      atomicOr(&s_bits, KDA_BIT_CKPT);
      for (int i = 0; i < N; i++) {
        long long v, cnt;
        if (!ck_range(i, v, cnt) || cnt == 0) continue;
        bool ok = true;
        for (int j = 0; j < i && ok; j++) {
          long long vj, cj;
          if (!ck_range(j, vj, cj) || cj == 0) continue;
          if ((N > SORT_MAX || s_keep[j]) && vj < v + cnt && v < vj + cj) ok = false;
        }
        if (!ok) {
          if (i < SORT_MAX) s_keep[i] = 0;
          a.tasks_unsorted[i].ck = nullptr;
        }
      }
    }
    __syncthreads();
  }

  // ---- order: longest first, ties by index (bitonic sort of (len descending, index) keys)
  const bool sorted = N <= SORT_MAX;
  if (sorted) {
    int n2 = 1;
    while (n2 < N) n2 <<= 1;
    __syncthreads();
    for (int i = tid; i < n2; i += bd) {
      if (i < N) {
        const unsigned long long len = (unsigned long long)(a.cu_safe[i + 1] - a.cu_safe[i]);
        keys[i] = ((0x7fffffffULL - len) << 32) | (unsigned)i;
      } else {
        keys[i] = ~0ULL;
      }
    }
    __syncthreads();
    for (int k = 2; k <= n2; k <<= 1) {
      for (int j = k >> 1; j > 0; j >>= 1) {
        for (int i = tid; i < n2; i += bd) {
          const int ixj = i ^ j;
          if (ixj > i) {
            const unsigned long long x = keys[i], y = keys[ixj];
            const bool up = (i & k) == 0;
            if ((x > y) == up) { keys[i] = y; keys[ixj] = x; }
          }
        }
        __syncthreads();
      }
    }
  }
  __syncthreads();   // tasks_unsorted complete
  for (int i = tid; i < N; i += bd) {
    const int srcpos = sorted ? (int)(keys[i] & 0xffffffffu) : i;
    a.tasks[i] = a.tasks_unsorted[srcpos];
  }
  if (tid == 0) {
    *a.n_tasks = N;
    a.status[0] = s_bits;
    a.status[1] = 0;
    a.status[2] = 0;
    a.status[3] = 0;
  }
}

cudaError_t launch_plan(const PlanParams& a, cudaStream_t stream) {
  kda_plan_kernel<<<1, PLAN_THREADS, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace kda
