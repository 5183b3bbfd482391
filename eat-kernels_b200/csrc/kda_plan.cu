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
#include "kda_scan_tile.cuh"

namespace kda {

constexpr int PLAN_THREADS = 1024;
constexpr int SORT_MAX = 4096;
// cut planning
constexpr int CUT_MAX_SEQS = 1024;       // sequences a cut plan is made for (beyond: never cut)
constexpr int N_CAND = 9;                // candidate piece lengths
constexpr int MIN_PIECE_CHUNKS = 16;     // shorter pieces drown in the per-task cost
constexpr int TASK_OVERHEAD = 3;         // start / end of a task, in chunk steps
constexpr int DUAL_X8 = 9;               // a dual-chain chunk step without output rows costs 9 / 8 single-chain ones (measured 1.05-1.1)

// chunk steps of the map of one piece of lp chunks: one dual-chain task, or two single-chain tasks
__device__ __forceinline__ long long map_task_cost(int lp, int dual) {
  return dual ? (long long)(DUAL_X8 * lp + 7) / 8 + TASK_OVERHEAD : 2LL * (lp + TASK_OVERHEAD);
}
constexpr int SCAN_STEPS_X16 = 12;       // one map of the scan chain, in 1/16 chunk steps
constexpr int LAUNCH_STEPS = 4;          // the scan launch and the second kernel launch, in chunk steps
__host__ __device__ constexpr int cand_pieces(int k) { return k < 3 ? k + 2 : (k == 3 ? 6 : (k == 4 ? 8 : (k == 5 ? 12 : (k == 6 ? 16 : (k == 7 ? 24 : 32))))); }

__device__ __forceinline__ long long rd_table(const void* p, int is64, long long i) {
  return is64 ? reinterpret_cast<const long long*>(p)[i] : (long long)reinterpret_cast<const int*>(p)[i];
}

__global__ void __launch_bounds__(PLAN_THREADS, 1) kda_plan_kernel(const PlanParams a) {
  __shared__ unsigned long long keys[SORT_MAX];
  __shared__ unsigned char s_keep[SORT_MAX];     // checkpoint rows of sequence i: 0 = none / rejected, 1 = kept
  __shared__ int s_bits, s_overlap;
  __shared__ int s_lp, s_cmax, s_uncut_work, s_work[N_CAND], s_pieces[N_CAND], s_longest[N_CAND], s_ncut[N_CAND];
  __shared__ unsigned short s_off_a[CUT_MAX_SEQS], s_off_b[CUT_MAX_SEQS];
  __shared__ unsigned char s_cnt_a[CUT_MAX_SEQS], s_cnt_b[CUT_MAX_SEQS], s_off_m[CUT_MAX_SEQS], s_off_c[CUT_MAX_SEQS];
  const int tid = threadIdx.x, bd = blockDim.x, N = a.N;
  // the chunk kernel chained behind this launch may become resident now (it waits for this kernel's results itself)
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
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
    t.dst2 = nullptr;
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

  // ---- cuts.  A long sequence is a serial chain of chunks on one SM per head; when such chains, not the total work,
  // bound the launch (few heads per GPU, one long request among short ones), cutting them into pieces of `lp` chunks
  // shortens the launch although a cut sequence costs about twice its chunks (see PlanParams).  The piece length
  // is chosen among "the longest sequence in 2, 3, 4, 6, ... pieces" by a cost model in chunk steps, against not
  // cutting at all.  Pieces are multiples of the checkpoint interval, so every checkpoint row is written by the piece
  // that holds its token.  Function of the reference's host planners (kda/b200/csrc/w3/base/kernel.py:389-444,482-532)
  // and of its device planner (kda/b200/csrc/dyn/plan_cp.cu:476-488).
  const int au = (a.ck_base != nullptr && a.ck_every > 0) ? a.ck_every / C : 1;    // alignment of a cut, in chunks
  if (tid == 0) s_lp = 0;
  if (a.max_pieces >= 2 && sorted && N <= CUT_MAX_SEQS && !noop) {
    if (tid < N_CAND) { s_work[tid] = 0; s_pieces[tid] = 0; s_longest[tid] = 0; s_ncut[tid] = 0; }
    if (tid == 0) { s_uncut_work = 0; s_cmax = (int)((0x7fffffffULL - (keys[0] >> 32)) + C - 1) / C; }
    __syncthreads();
    const int cmax = s_cmax;
    int lp_of[N_CAND];
#pragma unroll
    for (int k = 0; k < N_CAND; k++) {
      const int p = cand_pieces(k);
      int lp = (cmax + p - 1) / p;
      lp = (lp + au - 1) / au * au;
      lp_of[k] = (lp >= MIN_PIECE_CHUNKS && lp < cmax) ? lp : 0;
    }
    for (int j = tid; j < N; j += bd) {
      const int c = (int)((0x7fffffffULL - (keys[j] >> 32)) + C - 1) / C;
      atomicAdd(&s_uncut_work, c > 0 ? c + TASK_OVERHEAD : 0);
#pragma unroll
      for (int k = 0; k < N_CAND; k++) {
        const int lp = lp_of[k];
        if (lp == 0) continue;
        if (c <= lp + lp / 4) {
          if (c > 0) atomicAdd(&s_work[k], c + TASK_OVERHEAD);
          atomicMax(&s_longest[k], c);
        } else {
          atomicAdd(&s_pieces[k], (c + lp - 1) / lp);
          atomicAdd(&s_ncut[k], 1);
        }
      }
    }
    __syncthreads();
    if (tid == 0) {
      // Times in chunk steps.  A launch cannot end before its longest task, nor before its share of the work, nor before
      // the SM that gets the most piece-sized tasks has run them all (pieces are equal, so few of them come in waves).
      // A cut sequence of p pieces puts piece 0 and the maps of pieces 1 .. p-2 into the first launch (a map is one
      // dual-chain task of DUAL_X8 / 8 chunk steps per chunk, or two plain tasks) and p - 1 pieces into the second; the
      // uncut sequences are spread over both launches so that both carry about the same work.
      const long long Hh = a.H, nsm = a.n_sm;
      long long best = max(((long long)s_uncut_work * Hh + nsm - 1) / nsm, (long long)(cmax + TASK_OVERHEAD));
      int best_lp = 0;
      for (int k = 0; k < N_CAND; k++) {
        const int lp = lp_of[k];
        if (lp == 0 || s_ncut[k] == 0 || s_pieces[k] > a.max_pieces) continue;
        const long long pt = lp + TASK_OVERHEAD;
        const long long nmap = (long long)s_pieces[k] - 2LL * s_ncut[k];             // mapped pieces
        const long long ka = a.dual ? s_ncut[k] + nmap : s_ncut[k] + 2 * nmap;       // tasks of the first launch
        const long long kb = (long long)s_pieces[k] - s_ncut[k];
        const long long wcut = a.dual ? pt * s_ncut[k] + map_task_cost(lp, 1) * nmap : pt * ka;
        const long long pa = wcut / max(1LL, ka);                                    // mean task of the first launch
        const long long U = s_work[k];
        const long long to_b = max(0LL, min(U, (wcut + pt * kb + U) / 2 - pt * kb));
        const long long wa = wcut + U - to_b, wb = pt * kb + to_b;
        const long long ta = max(max((wa * Hh + nsm - 1) / nsm, ((ka * Hh + nsm - 1) / nsm) * pa), (long long)max(s_longest[k], lp) + TASK_OVERHEAD);
        const long long tb = max(max((wb * Hh + nsm - 1) / nsm, ((kb * Hh + nsm - 1) / nsm) * pt), pt);
        const long long t = ta + tb + (SCAN_STEPS_X16 * (long long)(cand_pieces(k) - 2) + 15) / 16 + LAUNCH_STEPS;
        if (t * 10 < best * 9) { best = t; best_lp = lp; }          // cut only for a clear gain
      }
      if (a.force_cand > 0 && a.force_cand <= N_CAND) {
        const int k = a.force_cand - 1;
        if (lp_of[k] != 0 && s_ncut[k] != 0 && s_pieces[k] <= a.max_pieces) best_lp = lp_of[k];
      }
      s_lp = best_lp;
    }
  }
  __syncthreads();
  const int lp = s_lp;
  if (lp == 0) {
    for (int i = tid; i < N; i += bd) {
      const int srcpos = sorted ? (int)(keys[i] & 0xffffffffu) : i;
      a.tasks[i] = a.tasks_unsorted[srcpos];
    }
    if (tid == 0) {
      *a.n_tasks = N | (noop ? NT_ZERO_FILL : 0);
      if (a.n_tasks_b != nullptr) { *a.n_tasks_b = 0; *a.n_chains = 0; }
    }
  } else {
    // Per sorted position: tasks in the first / second launch, map slots, and whether an uncut sequence moves to the
    // second launch (the shortest ones do, until both launches carry about the same work).
    __shared__ int s_half;
    if (tid == 0) {
      // work of the cut sequences per launch at the chosen piece length
      long long wa = 0, wb = 0, uncut = 0;
      for (int j = 0; j < N; j++) {
        const int c = (int)((0x7fffffffULL - (keys[j] >> 32)) + C - 1) / C;
        if (c <= lp + lp / 4) uncut += c > 0 ? c + TASK_OVERHEAD : 0;
        else {
          const int p = (c + lp - 1) / lp;
          wa += (lp + TASK_OVERHEAD) + (long long)map_task_cost(lp, a.dual) * (p - 2);
          wb += (long long)(lp + TASK_OVERHEAD) * (p - 1);
        }
      }
      const long long to_b = ((wa + wb + uncut) / 2) - wb;      // uncut work wanted in the second launch
      s_half = (int)max(0LL, min(uncut, to_b));
    }
    __syncthreads();
    if (tid < 32) {
      // one warp: lane l walks positions [per l, per (l + 1)) from the END of the sorted order (shortest first)
      const int per = (N + 31) / 32;
      int na = 0, nb = 0, nm = 0, nc = 0, wsum = 0;
      for (int q = 0; q < per; q++) {
        const int j = N - 1 - (tid * per + q);
        if (j < 0) break;
        const int c = (int)((0x7fffffffULL - (keys[j] >> 32)) + C - 1) / C;
        if (c <= lp + lp / 4) wsum += c > 0 ? c + TASK_OVERHEAD : 0;
      }
      int wpre = wsum;                                  // exclusive prefix of uncut work over the lanes
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, wpre, o);
        if (tid >= o) wpre += v;
      }
      wpre -= wsum;
      for (int q = 0; q < per; q++) {
        const int j = N - 1 - (tid * per + q);
        if (j < 0) break;
        const int c = (int)((0x7fffffffULL - (keys[j] >> 32)) + C - 1) / C;
        unsigned char ca = 0, cb = 0;
        if (c <= lp + lp / 4) {
          // (at most max_pieces uncut sequences move: the second launch's grid is sized for 2 * max_pieces tasks)
          const bool to_b = wpre < s_half && c > 0 && tid * per + q < a.max_pieces;
          wpre += c > 0 ? c + TASK_OVERHEAD : 0;
          if (to_b) cb = 1; else ca = 1;
        } else {
          const int p = (c + lp - 1) / lp;
          ca = (unsigned char)(a.dual ? p - 1 : 2 * p - 3);
          cb = (unsigned char)(p - 1);
          nm += p - 1;
          nc += 1;
        }
        s_cnt_a[j] = ca; s_cnt_b[j] = cb;
        na += ca; nb += cb;
      }
      // exclusive offsets in FORWARD (longest first) order: lane l's block lies after the blocks of the lanes above it
      int oa = na, ob = nb, om = nm, oc = nc;
      for (int o = 1; o < 32; o <<= 1) {
        const int va = __shfl_down_sync(0xffffffffu, oa, o), vb = __shfl_down_sync(0xffffffffu, ob, o);
        const int vm = __shfl_down_sync(0xffffffffu, om, o), vc = __shfl_down_sync(0xffffffffu, oc, o);
        if (tid + o < 32) { oa += va; ob += vb; om += vm; oc += vc; }
      }
      if (tid == 0) { *a.n_tasks = oa; *a.n_tasks_b = ob; *a.n_chains = oc; }
      oa -= na; ob -= nb; om -= nm; oc -= nc;           // what the lanes above (longer sequences) take
      // walk this lane's block forward (its LAST position is the longest sequence of the block)
      for (int q = per - 1; q >= 0; q--) {
        const int j = N - 1 - (tid * per + q);
        if (j < 0) continue;
        s_off_a[j] = (unsigned short)oa; s_off_b[j] = (unsigned short)ob; s_off_m[j] = (unsigned char)om; s_off_c[j] = (unsigned char)oc;
        const int c = (int)((0x7fffffffULL - (keys[j] >> 32)) + C - 1) / C;
        oa += s_cnt_a[j]; ob += s_cnt_b[j];
        if (c > lp + lp / 4) { om += (c + lp - 1) / lp - 1; oc += 1; }
      }
    }
    __syncthreads();
    const size_t slot_elems = (size_t)a.H * STATE_ELEMS;
    for (int j = tid; j < N; j += bd) {
      const Task t = a.tasks_unsorted[(int)(keys[j] & 0xffffffffu)];
      const int c = (t.len + C - 1) / C;
      if (c <= lp + lp / 4) {
        if (s_cnt_b[j]) a.tasks_b[s_off_b[j]] = t; else a.tasks[s_off_a[j]] = t;
        continue;
      }
      const int p = (c + lp - 1) / lp;
      const int m0 = s_off_m[j];                        // slots m0 .. m0 + p - 2: slot m0 = end state of piece 0
      int ia = s_off_a[j], ib = s_off_b[j];
      Task u = t;                                       // piece 0: the ordinary task, cut short, end state to slot m0
      u.len = lp * C;
      u.dst = a.map_L + (size_t)m0 * slot_elems;
      a.tasks[ia++] = u;
      for (int q = 1; q < p; q++) {
        const long long t0 = t.t0 + (long long)q * lp * C;
        const int len = min(lp * C, t.len - q * lp * C);
        if (q < p - 1) {                                // chains L and Tr of a middle piece -> map slot m0 + q
          Task l;
          l.t0 = t0; l.len = len; l.flags = TF_INIT_ZERO | TF_NO_OUT; l.src = nullptr; l.ck = nullptr; l.dst2 = nullptr;
          l.dst = a.map_L + (size_t)(m0 + q) * slot_elems;
          if (a.dual) {                                 // both chains in one task
            l.flags |= TF_DUAL;
            l.dst2 = a.map_P + (size_t)(m0 + q) * slot_elems;
            a.tasks[ia++] = l;
          } else {
            a.tasks[ia++] = l;
            l.flags = TF_INIT_IDENTITY | TF_V_ZERO | TF_NO_OUT | TF_DST_VF;
            l.dst = a.map_P + (size_t)(m0 + q) * slot_elems;
            a.tasks[ia++] = l;
          }
        }
        Task r;                                         // the piece itself, from its entering state
        r.t0 = t0; r.len = len; r.flags = 0; r.dst2 = nullptr;
        r.src = (q == 1) ? a.map_L + (size_t)m0 * slot_elems : a.map_E + (size_t)(m0 + q - 1) * slot_elems;
        r.dst = (q == p - 1) ? t.dst : nullptr;
        r.ck = nullptr;
        if (t.ck != nullptr) {
          const long long row = (long long)q * lp / au;
          r.ck = a.ck_is_bf16 ? (void*)(reinterpret_cast<__nv_bfloat16*>(t.ck) + row * a.ck_row_stride)
                              : (void*)(reinterpret_cast<float*>(t.ck) + row * a.ck_row_stride);
        }
        a.tasks_b[ib++] = r;
      }
      ScanChain ch;
      ch.s0 = a.map_L + (size_t)m0 * slot_elems;
      ch.first = m0 + 1;
      ch.count = p - 2;
      a.chains[s_off_c[j]] = ch;
    }
  }
  if (tid == 0) {
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

// ------------------------------------------------------------------------------------------------ scan of cut chains
// Entering states of the pieces of every cut sequence: per chain and head  E[k] = E[k-1] applied to map k  with
// E[-1] = the end state of piece 0.  In the value-first layout a state is [v][k] and a map acts as  E <- E P + L  (rows
// v evolve independently); in the key-first layout the same relation reads  E[k'][v] = sum_k P[k][k'] E[k][v] + L[k'][v]
// (columns v evolve independently; P is stored value-first in both cases).  A CTA carries 32 independent rows /
// columns of one head through the chain in fp32 as register tiles (kda_scan_tile.cuh).
__global__ void __launch_bounds__(ST_THREADS) kda_scan_chains_kernel(const ScanChain* __restrict__ chains, const int* __restrict__ n_chains,
                                                                     const float* __restrict__ P, const float* __restrict__ L,
                                                                     float* __restrict__ E, int H, int kf) {
  __shared__ __align__(16) ScanSmem sm;
  if ((int)blockIdx.z >= *n_chains) return;
  const ScanChain ch = chains[blockIdx.z];
  if (ch.count <= 0) return;
  const int h = blockIdx.y, tid = threadIdx.x;
  const int r0 = blockIdx.x * ST_ROWS + 4 * (tid >> 5), c0 = 4 * (tid & 31);
  const size_t head_off = (size_t)h * STATE_ELEMS, slot_stride = (size_t)H * STATE_ELEMS;
  const int ks = kf ? D : 1;            // stride of the contracted / produced index (the independent one has the other)
  float cur[4][4];
  scan_tile_load(cur, ch.s0 + head_off, r0, c0, ks);
  for (int i = 0; i < ch.count; i++) {
    const size_t slot = (size_t)(ch.first + i) * slot_stride + head_off;
    float acc[4][4];
    scan_tile_load(acc, L + slot, r0, c0, ks);
    scan_tile_step(acc, cur, P + slot, sm, tid);
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
      for (int b = 0; b < 4; b++) cur[a][b] = acc[a][b];
    scan_tile_store(cur, E + slot, r0, c0, ks);
  }
}

cudaError_t launch_scan_chains(const ScanChain* chains, const int* n_chains, int max_chains, const float* P, const float* L, float* E,
                               int H, int key_first, cudaStream_t stream) {
  if (max_chains <= 0) return cudaSuccess;
  dim3 grid(D / ST_ROWS, H, max_chains);
  kda_scan_chains_kernel<<<grid, ST_THREADS, 0, stream>>>(chains, n_chains, P, L, E, H, key_first);
  return cudaGetLastError();
}

}  // namespace kda
