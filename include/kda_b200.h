/* C ABI of the B200 KDA-prefill library (libkda_b200.so).
 *
 * Plain pointers and sizes only; every pointer marked "device" is a CUDA device address on the current device.
 * Every entry point returns 0 or a negative KDA_ERR_* code, never throws, never synchronises the device and never
 * allocates device memory unless its comment says so.  Work is enqueued on the `stream` argument (a cudaStream_t
 * passed as void*, 0 = the default stream) and can be captured in a CUDA graph.
 *
 * Reference interfaces these replace (paths inside caoshiyi/eat-kernels):
 *   kda_prefill_launch    <- the launch closure built by prepare()/run(): kda/b200/kda_b200.py:44-76,
 *                            kda/b200/csrc/w3/kernel.py:1284-1329 (argument contract), the fused kernel launch
 *                            kda/b200/csrc/w3/base/cake/launch_m128.cu:41-43 and the device planner + table
 *                            validation launch kda/b200/csrc/dyn/plan_cp.cu:218-270, kda/b200/csrc/w3/contract_aux.cu:25-31
 *   kda_segment_launch    <- the dual-chain tail launch kda/b200/csrc/w3/base/dual.py:91-159
 *   kda_scan_launch,
 *   kda_fixup_launch      <- the context-parallel fix-up kda/b200/csrc/w3/cp_fix.cu:141-381
 *   kda_state_rows_copy   <- slot-indexed state / checkpoint row copies kda/b200/csrc/w3/contract_aux.cu:34-74
 */
#ifndef KDA_B200_H_
#define KDA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KDA_HEAD_DIM 128
#define KDA_CHUNK 32

enum {
  KDA_OK = 0,
  KDA_ERR_ARG = -1,        /* null / misaligned pointer, bad stride or size */
  KDA_ERR_WORKSPACE = -2,  /* workspace too small */
  KDA_ERR_LAUNCH = -3,     /* the CUDA runtime refused a launch (kda_error_string gives its message) */
  KDA_ERR_LIMIT = -4       /* a size exceeds a documented maximum */
};

/* Front-end of the operator. */
enum {
  KDA_FRONTEND_RAW = 0,    /* g bf16 raw gate, beta bf16 logits, q/k L2-normalised in the kernel
                              (kda/b200/reference.py:21-26) */
  KDA_FRONTEND_PLAIN = 1   /* g fp32 log-decay (<= 0), beta fp32 in (0,1), q/k used as given (chunk_kda-style call) */
};

enum {
  KDA_STATE_VALUE_FIRST = 0,   /* [.., 128 (V), 128 (K)], the reference's layout (kda/b200/reference.py:4) */
  KDA_STATE_KEY_FIRST = 1      /* [.., 128 (K), 128 (V)] */
};

/* Which fused chunk kernel runs the recurrence. */
enum {
  KDA_KERNEL_TCGEN05 = 0,  /* tcgen05 / tensor-memory kernel (default) */
  KDA_KERNEL_MMA_SYNC = 1, /* warp-level mma.sync kernel: same results within tolerance, kept as an independent
                              cross-check of the tensor-memory path */
  KDA_KERNEL_TCGEN05_TWO_TASK = 2  /* kda_segment_launch only (elsewhere the same as KDA_KERNEL_TCGEN05): chains L and
                              Tr of a mapped segment as two single-chain tasks.  With KDA_KERNEL_TCGEN05 a mapped
                              segment is ONE dual-chain task, both chains over one operand preparation
                              (kda/b200/csrc/w3/base/cake_dual/kda_m128.cu:821-823): bit-identical results, about
                              1.6 instead of 2 chunk steps per chunk; this value keeps the two-task scheme
                              available as the cross-check */
};

/* Bits of status[0] (table validation, same meaning as kda/b200/kda_b200.py:56-62). */
enum {
  KDA_STATUS_BAD_CU = 1,        /* cu_seqlens rejected: every sequence treated as empty, output rows zero-filled */
  KDA_STATUS_BAD_SLOT = 2,      /* bad or repeated ssm_state_indices entry: that sequence's state goes to scratch */
  KDA_STATUS_BAD_SOURCE = 4,    /* bad initial_state_indices entry */
  KDA_STATUS_BAD_CKPT = 8,      /* checkpoint rows outside state_checkpoints or overlapping an earlier sequence */
  KDA_STATUS_RANGE = 16         /* not a table error and not in the reference: some key channel decayed by more than
                                   2^126 within 16 tokens (impossible with the raw front-end's -5 bound; possible with
                                   unbounded plain-call log-decays), the exponents of that chunk's intra-chunk products
                                   were clamped and the results of that (sequence, head) are inexact */
};

typedef struct KdaPrefillArgs {
  /* ---- token tensors, packed varlen [T][H][128]; ld* = elements between consecutive tokens (>= H*128 for a head
   *      slice of a wider tensor), heads are 128 elements apart.  All device pointers, 16-byte aligned. */
  const void* q;          /* bf16 */
  const void* k;          /* bf16 */
  const void* v;          /* bf16 */
  const void* g;          /* bf16 (raw) or fp32 (plain) */
  const void* beta;       /* bf16 (raw) or fp32 (plain), [T][H], ldbeta elements between tokens */
  void* out;              /* bf16 [T][H][128] */
  int64_t ldq, ldk, ldv, ldg, ldbeta, ldo;
  const float* A_log;     /* [H]      raw front-end only */
  const float* dt_bias;   /* [H*128]  raw front-end only */
  float scale;
  float lower_bound;      /* raw front-end: a = lower_bound * sigmoid(...); the reference fixes -5 */
  int32_t frontend;       /* KDA_FRONTEND_* */
  int32_t state_layout;   /* KDA_STATE_* (applies to source, destination and checkpoint rows) */
  int32_t H;              /* heads handled by this call */
  int32_t N;              /* sequences (cu_seqlens has N+1 entries) */
  int64_t T;              /* token rows of the tensors above */
  const void* cu_seqlens; /* device int32/int64 [N+1], or NULL: one sequence [0, T] */
  int32_t cu_is64;

  /* ---- recurrent state.  A slot is [H][128][128] fp32; slot s of a pool starts at base + s*slot_stride floats.
   *      Without an index table sequence i uses slot i. */
  const float* src_base;  /* initial states; NULL = zeros */
  int64_t src_slot_stride;
  const void* src_idx;    /* device int32/int64 [N] or NULL */
  int32_t src_idx_is64;
  int64_t src_slots;      /* number of addressable slots (range check) */
  float* dst_base;        /* final states; NULL = not stored */
  int64_t dst_slot_stride;
  const void* dst_idx;
  int32_t dst_idx_is64;
  int64_t dst_slots;

  /* ---- prefix-cache checkpoints: row ck_starts[i] + j = state of sequence i before token j*ck_every
   *      (kda/b200/kda_b200.py:19-22).  ck_every = 0: off. */
  void* ck_base;          /* fp32 or bf16 [ck_rows][H][128][128] */
  int32_t ck_is_bf16;
  int32_t ck_every;       /* tokens, multiple of KDA_CHUNK */
  int64_t ck_rows;
  const void* ck_starts;  /* device int32/int64 [N+1] */
  int32_t ck_starts_is64;

  /* ---- scratch and status */
  void* workspace;        /* device, >= kda_prefill_workspace_bytes(N, H), 256-byte aligned; contents need not
                             survive between calls, but concurrent calls must not share it */
  size_t workspace_bytes;
  int32_t* status;        /* device int32[4]: [0] table-validation bits, [1] reserved, [2] kernel error code
                             (0 = none; nonzero: a bounded wait inside the kernel gave up, results are invalid),
                             [3] reserved; written by every call */
  int32_t kernel;         /* KDA_KERNEL_* */
  int32_t max_cut_pieces; /* 0 (or 1): sequences are never cut.  >= 2: the device planner may cut long sequences into
                             pieces (at most this many over the whole call) when serial chains, not the total work,
                             bound the launch; the workspace must then be sized by kda_prefill_workspace_bytes_cuts.
                             Function of the reference's cut plans (kda/b200/csrc/w3/base/kernel.py:389-444,482-532,
                             kda/b200/csrc/dyn/plan_cp.cu:476-488).  Results are those of the uncut call within the
                             tolerance of the operator (pieces start from entering states obtained through fp32 state
                             maps); checkpoint rows, pool slots and status bits are unchanged. */
} KdaPrefillArgs;

#define KDA_MAX_CUT_PIECES 128

/* Bytes of workspace a call with N sequences and H heads needs (max_cut_pieces = 0). */
size_t kda_prefill_workspace_bytes(int32_t N, int32_t H);
/* The same with room for the state maps of `max_cut_pieces` pieces (3 x 64 KB per piece and head). */
size_t kda_prefill_workspace_bytes_cuts(int32_t N, int32_t H, int32_t max_cut_pieces);

/* Validates the caller's tables on the device, orders the (sequence, head) tasks longest first and runs the fused
 * chunk kernel.  Two kernel launches (four with max_cut_pieces >= 2: planner, chunk kernel, scan of the cut sequences'
 * state maps, chunk kernel again), no host read of any table. */
int kda_prefill_launch(const KdaPrefillArgs* args, void* stream);

/* What the planner of the most recent kda_prefill_launch with these arguments decided (reads the workspace; this one
 * call SYNCHRONISES the stream): counts[0] = tasks of the first launch, counts[1] = tasks of the second launch (pieces
 * of cut sequences and the uncut sequences moved there for balance; 0 = nothing was cut), counts[2] = cut sequences.
 * For tests and tools; the reference exposes its plan as launch.tables (kda/b200/csrc/w3/kernel.py:1218-1219). */
int kda_prefill_plan_counts(const KdaPrefillArgs* args, int32_t* counts, void* stream);

/* The same call for callers that must not allocate device memory and have no workspace to hand over: code running
 * inside a memory-pool callback or an allocator hook, a process whose device memory is fully reserved up front by a
 * serving engine, or a thread that may be inside CUDA stream capture (where cudaMalloc is illegal).  The scratch lives
 * in a fixed array inside the library's device image instead of `args->workspace` (which is ignored, as is
 * `workspace_bytes`); the caller still passes every input, output and the status word.
 *   - limits: N <= KDA_NOALLOC_MAX_SEQS and H <= KDA_NOALLOC_MAX_HEADS, else KDA_ERR_LIMIT (nothing is launched);
 *     the array takes about 1.1 MB of every GPU that loads the library, until the process exits;
 *   - the first call on a device looks the array's device address up (once per device, with that device current);
 *     make that first call outside stream capture;
 *   - all calls on a device share the array, and it keeps the previous call's contents.  Nothing in it has to start at
 *     zero (the planner rewrites every entry a call later reads), but two calls whose kernels overlap on the GPU
 *     (different streams) race on it: serialise them;
 *   - it calls no cudaMalloc / cudaFree and no allocating library routine.
 * This entry point has no counterpart in the reference, whose launches own scratch tensors allocated by torch. */
#define KDA_NOALLOC_MAX_SEQS 64
#define KDA_NOALLOC_MAX_HEADS 16
int kda_prefill_launch_noalloc(const KdaPrefillArgs* args, void* stream);

/* ---- context parallelism: per-segment affine state maps (value-first orientation)
 *        S_end = S_in @ P + S_loc          out_t = o_loc_t + S_in applied to Qt_t
 * One call runs, for each of `n_seg` token segments [seg_t0[i], seg_t1[i]) and each head, chain L (S0 = 0, real v:
 * o_loc, S_loc) and, where seg_need_map[i] != 0, chain Tr (S0 = I, v = 0: Qt, P).  Segments with seg_need_map == 0
 * start from src (slot i of src_base, or zeros) and write the ordinary output/state. */
typedef struct KdaSegmentArgs {
  KdaPrefillArgs base;        /* token tensors, front-end, H, T, workspace, status; cu_seqlens/dst/ck fields unused */
  int32_t n_seg;
  const int64_t* seg_t0;      /* device [n_seg] */
  const int64_t* seg_t1;      /* device [n_seg] */
  const int32_t* seg_need_map;/* device [n_seg] */
  void* qt;                   /* bf16 [T][H][128] (ldo stride): Qt rows of mapped segments; NULL = maps only: no output
                                 rows are written by either chain and base.out may be NULL too */
  float* P;                   /* [n_seg][H][128][128] transition maps, value-first */
  float* S_loc;               /* [n_seg][H][128][128] offsets; for unmapped segments the true end state */
  void* tiles;                /* KDA_KERNEL_TCGEN05 with output rows: bf16 scratch of 2 * kda_segment_tiles(..) * H * 4096
                                 elements.  Mapped segments run as dual-chain tasks that write o_loc and Qt TILE-MAJOR
                                 here ([tile][head][128][32 tokens]; Qt tiles first, the o_loc tiles behind them) instead of
                                 as rows of base.out / qt; kda_fixup_tiles_launch turns them into the rows of base.out.
                                 NULL: two single-chain tasks per mapped segment, rows in base.out / qt (as with
                                 KDA_KERNEL_TCGEN05_TWO_TASK); qt is not written when tiles is given, but must be
                                 non-NULL to ask for output */
  int64_t n_tiles;            /* kda_segment_tiles() of the segment tables: where the o_loc tiles start in `tiles` */
} KdaSegmentArgs;

/* Tiles of 32 tokens the segments [t0[i], t1[i]) take in the tile-major scratch (HOST copies of the tables). */
int64_t kda_segment_tiles(const int64_t* seg_t0, const int64_t* seg_t1, int32_t n_seg, int64_t T);

int kda_segment_launch(const KdaSegmentArgs* args, void* stream);

/* Exclusive scan over a chain of `n_seg` segment maps per head: S_in[0] = S0 (or zeros), S_in[i+1] = S_in[i] @ P[i]
 * + S_loc[i]; writes S_in[0..n_seg-1] and the chain's end state.  fp32 throughout. */
int kda_scan_launch(const float* P, const float* S_loc, const float* S0, float* S_in, float* S_end, int32_t n_seg,
                    int32_t H, void* stream);

/* The same with the maps `map_stride` floats apart (>= H * 16384, a multiple of 4) instead of packed: P and S_loc may then
 * be the two halves of one buffer [n_seg][2][H][128][128], which is what ONE all-gather of per-rank (P, S_loc) pairs
 * delivers.  S_in stays packed. */
int kda_scan_strided_launch(const float* P, const float* S_loc, const float* S0, float* S_in, float* S_end, int32_t n_seg,
                            int32_t H, int64_t map_stride, void* stream);

/* out rows of segment i += S_in[i] applied to Qt rows (bf16 tensor-core product with the entering state rounded to
 * bf16, as kda/b200/csrc/w3/cp_fix.cu:279-377). */
int kda_fixup_launch(void* out, const void* qt, int64_t ldo, const float* S_in, const int64_t* seg_t0,
                     const int64_t* seg_t1, const int32_t* seg_need_map, int32_t n_seg, int32_t H, void* stream);

/* The same pass for a segment launch that wrote tile-major scratch (KdaSegmentArgs::tiles): out rows of the mapped
 * segments = o_loc tile + S_in[i] applied to the Qt tile; `tiles` and `n_tiles` as given to / sized for that launch. */
int kda_fixup_tiles_launch(void* out, const void* tiles, int64_t n_tiles, int64_t ldo, const float* S_in,
                           const int64_t* seg_t0, const int64_t* seg_t1, const int32_t* seg_need_map, int32_t n_seg,
                           int32_t H, int64_t T, void* stream);

/* dst row i <- src row idx[i] (64 KB fp32 rows per head), optionally rounding to bf16 (round to nearest even).
 * Rows are [H][128][128]; strides in elements of the respective type. */
int kda_state_rows_copy(void* dst, int64_t dst_row_stride, int32_t dst_is_bf16, const float* src,
                        int64_t src_row_stride, const int32_t* idx, int32_t n_rows, int32_t H, void* stream);

/* Text of a KDA_ERR_* code; for KDA_ERR_LAUNCH the last CUDA error string seen by this thread. */
const char* kda_error_string(int code);

/* sizeof(KdaPrefillArgs) (which = 0) or sizeof(KdaSegmentArgs) (which = 1) as the library was compiled: lets a foreign
 * binding check its struct layout before the first call. */
size_t kda_abi_struct_bytes(int which);

/* Library version and build information ("kda_b200 <n> sm_100a"). */
const char* kda_version(void);

/* Diagnostics for tests and profiling runs; process-wide, not thread-safe, never needed by a product call.  No
 * counterpart in the reference (whose waits trap after 60 s, kda/b200/README.md:169-171).
 *   wait_limit_us  bound of every wait inside the tcgen05 kernel (0 = the built-in two seconds).  When a wait runs out
 *                  the kernel finishes its control flow, waits for its own copies and tensor-core work, frees tensor
 *                  memory and writes a code to status[2].
 *   flags          bit 0: the arrival of the v tiles is never signalled to their consumers, so that a waiter runs into
 *                  the bound (used to test the give-up path without faulting or hanging anything); 0 = normal.
 *                  bits 8-11: k + 1 makes the device planner cut with candidate k of its piece lengths (the longest
 *                  sequence in 2, 3, 4, 6, 8, 12, 16, 24, 32 pieces) instead of asking its cost model (tuning aid).
 *   prof_counters  device uint64[1024] receiving per-role cycle counters in builds compiled with -DKDA_PROF; NULL else. */
int kda_debug_configure(int64_t wait_limit_us, int32_t flags, void* prof_counters);

#ifdef __cplusplus
}
#endif
#endif /* KDA_B200_H_ */
