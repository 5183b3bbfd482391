// extern "C" entry points of libkda_b200.so (declared in include/kda_b200.h).
#include <stdio.h>
#include <string.h>

#include "../../include/kda_b200.h"
#include "kda_common.cuh"
#include "kda_cp.cuh"
#include "kda_plan.cuh"

namespace {

thread_local char g_cuda_err[256] = "no CUDA error recorded";

int cuda_fail(cudaError_t e) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "CUDA error %d: %s", (int)e, cudaGetErrorString(e));
  return KDA_ERR_LAUNCH;
}

// Diagnostic configuration (kda_debug_configure): process-wide, meant for tests and profiling runs only.
unsigned long long g_wait_limit_ns = 0;
int g_debug_flags = 0;
unsigned long long* g_prof = nullptr;

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

struct Workspace {
  kda::Task* tasks;
  kda::Task* tasks_unsorted;
  int* n_tasks;            // [0] first launch, [1] second launch, [2] scan chains
  long long* cu_safe;
  float* trash;
  // only with cuts (max_pieces > 0)
  kda::Task* tasks_b;
  kda::ScanChain* chains;
  float *map_P, *map_L, *map_E;
  size_t bytes;
};

// `pieces`: capacity for the pieces of cut sequences (0 = the call never cuts; the layout is then the one older
// callers sized their workspace for)
Workspace carve(void* base, int N, int H, int pieces = 0) {
  Workspace w;
  size_t off = 0;
  uint8_t* b = reinterpret_cast<uint8_t*>(base);
  const size_t n = (size_t)(N > 0 ? N : 1);
  const size_t na = n + 2 * (size_t)pieces;
  w.tasks = reinterpret_cast<kda::Task*>(b + off); off = align_up(off + na * sizeof(kda::Task), 256);
  w.tasks_unsorted = reinterpret_cast<kda::Task*>(b + off); off = align_up(off + n * sizeof(kda::Task), 256);
  w.n_tasks = reinterpret_cast<int*>(b + off); off = align_up(off + 32, 256);
  w.cu_safe = reinterpret_cast<long long*>(b + off); off = align_up(off + (n + 1) * sizeof(long long), 256);
  w.trash = reinterpret_cast<float*>(b + off); off = align_up(off + (size_t)H * kda::STATE_ELEMS * sizeof(float), 256);
  w.tasks_b = nullptr; w.chains = nullptr; w.map_P = w.map_L = w.map_E = nullptr;
  if (pieces > 0) {
    const size_t maps = (size_t)pieces * H * kda::STATE_ELEMS * sizeof(float);
    w.tasks_b = reinterpret_cast<kda::Task*>(b + off); off = align_up(off + 2 * (size_t)pieces * sizeof(kda::Task), 256);
    w.chains = reinterpret_cast<kda::ScanChain*>(b + off); off = align_up(off + ((size_t)pieces / 2 + 1) * sizeof(kda::ScanChain), 256);
    w.map_P = reinterpret_cast<float*>(b + off); off = align_up(off + maps, 256);
    w.map_L = reinterpret_cast<float*>(b + off); off = align_up(off + maps, 256);
    w.map_E = reinterpret_cast<float*>(b + off); off = align_up(off + maps, 256);
  }
  w.bytes = off;
  return w;
}

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    cached[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
  }
  return cached[dev];
}

int check_tokens(const KdaPrefillArgs* a) {
  if (a == nullptr) return KDA_ERR_ARG;
  if (a->H <= 0 || a->N < 0 || a->T < 0) return KDA_ERR_ARG;
  if (a->kernel != KDA_KERNEL_TCGEN05 && a->kernel != KDA_KERNEL_MMA_SYNC && a->kernel != KDA_KERNEL_TCGEN05_TWO_TASK) return KDA_ERR_ARG;
  if (a->frontend != KDA_FRONTEND_RAW && a->frontend != KDA_FRONTEND_PLAIN) return KDA_ERR_ARG;
  if (a->state_layout != KDA_STATE_VALUE_FIRST && a->state_layout != KDA_STATE_KEY_FIRST) return KDA_ERR_ARG;
  if (a->T > 0) {
    if (!a->q || !a->k || !a->v || !a->g || !a->beta || !a->out) return KDA_ERR_ARG;
    if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->g) || !aligned16(a->out)) return KDA_ERR_ARG;
    const int64_t hd = (int64_t)a->H * KDA_HEAD_DIM;
    if (a->ldq < hd || a->ldk < hd || a->ldv < hd || a->ldg < hd || a->ldo < hd || a->ldbeta < a->H) return KDA_ERR_ARG;
    if ((a->ldq | a->ldk | a->ldv | a->ldo) & 7) return KDA_ERR_ARG;
    if (a->ldg & (a->frontend == KDA_FRONTEND_PLAIN ? 3 : 7)) return KDA_ERR_ARG;
  }
  if (a->frontend == KDA_FRONTEND_RAW && (!a->A_log || !a->dt_bias)) return KDA_ERR_ARG;
  if (!a->status || !a->workspace) return KDA_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(a->workspace) & 255) return KDA_ERR_ARG;
  return KDA_OK;
}

void fill_chunk_params(kda::ChunkParams& p, const KdaPrefillArgs* a) {
  memset(&p, 0, sizeof(p));
  p.q = reinterpret_cast<const __nv_bfloat16*>(a->q);
  p.k = reinterpret_cast<const __nv_bfloat16*>(a->k);
  p.v = reinterpret_cast<const __nv_bfloat16*>(a->v);
  p.g = a->g;
  p.beta = a->beta;
  p.out = reinterpret_cast<__nv_bfloat16*>(a->out);
  p.out_aux = nullptr;
  p.ldq = a->ldq; p.ldk = a->ldk; p.ldv = a->ldv; p.ldg = a->ldg; p.ldbeta = a->ldbeta; p.ldo = a->ldo;
  p.A_log = a->A_log;
  p.dt_bias = a->dt_bias;
  p.scale = a->scale;
  p.lower_bound = a->lower_bound;
  p.frontend = a->frontend;
  p.key_first = a->state_layout == KDA_STATE_KEY_FIRST;
  p.H = a->H;
  p.T = a->T;
  p.status = a->status;
  p.wait_limit_ns = g_wait_limit_ns;
  p.debug_flags = g_debug_flags;
  p.prof = g_prof;
}

// Tensor maps of the token tensors for the tcgen05 kernel's copy engine (q, k, v in 64-channel halves with the 128-byte
// swizzle, g as whole 128-channel rows).  T == 0: nothing is ever copied, the maps stay zeroed.
// A prepared launch calls with the same pointers and strides every time, so the encoded maps are kept per thread
// (a few entries, replaced round-robin) instead of going through the driver's encoder at every launch.
struct MapKey {
  const void *q, *k, *v, *g;
  int64_t ldq, ldk, ldv, ldg, T;
  int32_t H, frontend;
  bool operator==(const MapKey& o) const {
    return q == o.q && k == o.k && v == o.v && g == o.g && ldq == o.ldq && ldk == o.ldk && ldv == o.ldv && ldg == o.ldg &&
           T == o.T && H == o.H && frontend == o.frontend;
  }
};
constexpr int kMapCache = 16;
thread_local MapKey g_map_keys[kMapCache];
thread_local kda::TmaMaps g_map_vals[kMapCache];
thread_local int g_map_used = 0, g_map_next = 0;

int fill_tma_maps(kda::TmaMaps& m, const KdaPrefillArgs* a) {
  memset(&m, 0, sizeof(m));
  if (a->T <= 0) return KDA_OK;
  if (a->T > 0x7fffffffLL) return KDA_ERR_LIMIT;
  const MapKey key = {a->q, a->k, a->v, a->g, a->ldq, a->ldk, a->ldv, a->ldg, a->T, a->H, a->frontend};
  for (int i = 0; i < g_map_used; i++)
    if (g_map_keys[i] == key) {
      m = g_map_vals[i];
      return KDA_OK;
    }
  const bool plain = a->frontend == KDA_FRONTEND_PLAIN;
  int rc = kda::encode_token_map(&m.q, a->q, 2, false, a->T, a->H, a->ldq, 64, true);
  if (rc == 0) rc = kda::encode_token_map(&m.k, a->k, 2, false, a->T, a->H, a->ldk, 64, true);
  if (rc == 0) rc = kda::encode_token_map(&m.v, a->v, 2, false, a->T, a->H, a->ldv, 64, true);
  if (rc == 0) rc = kda::encode_token_map(&m.g, a->g, plain ? 4 : 2, plain, a->T, a->H, a->ldg, 128, false);
  if (rc != 0) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed (%d)", rc);
    return KDA_ERR_LAUNCH;
  }
  const int slot = g_map_used < kMapCache ? g_map_used++ : (g_map_next++ % kMapCache);
  g_map_keys[slot] = key;
  g_map_vals[slot] = m;
  return KDA_OK;
}

}  // namespace

extern "C" {

size_t kda_prefill_workspace_bytes(int32_t N, int32_t H) {
  if (N < 0 || H <= 0) return 0;
  return carve(nullptr, N, H).bytes;
}

size_t kda_prefill_workspace_bytes_cuts(int32_t N, int32_t H, int32_t max_cut_pieces) {
  if (N < 0 || H <= 0 || max_cut_pieces < 0 || max_cut_pieces > KDA_MAX_CUT_PIECES) return 0;
  return carve(nullptr, N, H, max_cut_pieces).bytes;
}

int kda_prefill_launch(const KdaPrefillArgs* a, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int rc = check_tokens(a);
  if (rc != KDA_OK) return rc;
  if (a->N < 1) return KDA_ERR_ARG;
  if (a->cu_seqlens == nullptr && a->N != 1) return KDA_ERR_ARG;
  if (a->ck_every != 0) {
    if (a->ck_every < 0 || a->ck_every % KDA_CHUNK) return KDA_ERR_ARG;
    if (!a->ck_base || !a->ck_starts || a->ck_rows < 0) return KDA_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(a->ck_base) & 7) return KDA_ERR_ARG;
  }
  if (a->src_base && (!aligned16(a->src_base) || (a->src_slot_stride & 3))) return KDA_ERR_ARG;
  if (a->dst_base && (!aligned16(a->dst_base) || (a->dst_slot_stride & 3))) return KDA_ERR_ARG;
  if (a->max_cut_pieces < 0 || a->max_cut_pieces > KDA_MAX_CUT_PIECES) return KDA_ERR_ARG;
  const int pieces = a->max_cut_pieces >= 2 ? a->max_cut_pieces : 0;
  const Workspace w = carve(a->workspace, a->N, a->H, pieces);
  if (a->workspace_bytes < w.bytes) return KDA_ERR_WORKSPACE;

  kda::PlanParams pl;
  memset(&pl, 0, sizeof(pl));
  pl.N = a->N; pl.H = a->H; pl.T = a->T;
  pl.cu = a->cu_seqlens; pl.cu_is64 = a->cu_is64;
  pl.src_base = a->src_base; pl.src_stride = a->src_slot_stride; pl.src_idx = a->src_idx; pl.src_is64 = a->src_idx_is64;
  pl.src_slots = a->src_slots;
  pl.src_separate = !(a->src_base != nullptr && a->src_base == a->dst_base && a->dst_idx != nullptr && a->src_idx == nullptr);
  pl.dst_base = a->dst_base; pl.dst_stride = a->dst_slot_stride; pl.dst_idx = a->dst_idx; pl.dst_is64 = a->dst_idx_is64;
  pl.dst_slots = a->dst_slots;
  pl.ck_base = a->ck_every ? a->ck_base : nullptr; pl.ck_is_bf16 = a->ck_is_bf16; pl.ck_every = a->ck_every;
  pl.ck_rows = a->ck_rows; pl.ck_row_stride = (long long)a->H * kda::STATE_ELEMS;
  pl.ck_starts = a->ck_starts; pl.ck_is64 = a->ck_starts_is64;
  pl.trash = w.trash; pl.cu_safe = w.cu_safe; pl.tasks_unsorted = w.tasks_unsorted; pl.tasks = w.tasks;
  pl.n_tasks = w.n_tasks; pl.status = a->status;
  pl.max_pieces = pieces; pl.n_sm = sm_count(); pl.key_first = a->state_layout == KDA_STATE_KEY_FIRST;
  pl.dual = a->kernel != KDA_KERNEL_MMA_SYNC;
  pl.force_cand = (g_debug_flags & kda::DBG_FORCE_CAND_MASK) >> kda::DBG_FORCE_CAND_SHIFT;
  if (pieces > 0) {
    pl.tasks_b = w.tasks_b; pl.n_tasks_b = w.n_tasks + 1; pl.n_chains = w.n_tasks + 2; pl.chains = w.chains;
    pl.map_P = w.map_P; pl.map_L = w.map_L; pl.map_E = w.map_E;
  }
  cudaError_t e = kda::launch_plan(pl, stream);
  if (e != cudaSuccess) return cuda_fail(e);

  kda::ChunkParams p;
  fill_chunk_params(p, a);
  p.ck_is_bf16 = a->ck_is_bf16;
  p.ck_every_chunks = a->ck_every / KDA_CHUNK;
  p.ck_row_stride = (long long)a->H * kda::STATE_ELEMS;
  p.tasks = w.tasks;
  p.n_tasks = w.n_tasks;
  kda::TmaMaps maps;
  const bool umma = a->kernel != KDA_KERNEL_MMA_SYNC;
  if (umma) {
    rc = fill_tma_maps(maps, a);
    if (rc != KDA_OK) return rc;
  }
  // first launch: every uncut sequence (or all of them), piece 0 and the map chains of the cut ones
  e = umma ? kda::launch_chunk_umma(p, maps, a->N + 2 * pieces, stream) : kda::launch_chunk_fwd(p, a->N + 2 * pieces, stream);
  if (e != cudaSuccess) return cuda_fail(e);
  if (pieces > 0) {
    // entering states of the later pieces, then those pieces (both launches find nothing to do when nothing was cut)
    e = kda::launch_scan_chains(w.chains, w.n_tasks + 2, pieces / 2 + 1, w.map_P, w.map_L, w.map_E, a->H, p.key_first, stream);
    if (e != cudaSuccess) return cuda_fail(e);
    p.tasks = w.tasks_b;
    p.n_tasks = w.n_tasks + 1;
    e = umma ? kda::launch_chunk_umma(p, maps, 2 * pieces, stream) : kda::launch_chunk_fwd(p, 2 * pieces, stream);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  return KDA_OK;
}

}  // extern "C"

// ---- scratch of kda_prefill_launch_noalloc: a fixed device array instead of a caller workspace.  In host code the
// name below is only a handle of the symbol, not a device address; the address is looked up per device with
// cudaGetSymbolAddress and cached.
namespace {
constexpr size_t kNoallocBytes = 2 * 12288 /* task tables, 64 x 48 B each rounded up */ + 256 /* task count */ +
                                 1024 /* cu_seqlens copy */ + (size_t)KDA_NOALLOC_MAX_HEADS * kda::STATE_ELEMS * sizeof(float) + 4096;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoallocBytes];
constexpr int kMaxDevices = 64;
// Filled without a lock: two threads racing on a device's first call both look the same address up and store the same
// value, so the race is benign.
void* g_noalloc_addr[kMaxDevices] = {};
}  // namespace

extern "C" {

int kda_prefill_launch_noalloc(const KdaPrefillArgs* a, void* stream_) {
  if (a == nullptr) return KDA_ERR_ARG;
  if (a->N > KDA_NOALLOC_MAX_SEQS || a->H > KDA_NOALLOC_MAX_HEADS) return KDA_ERR_LIMIT;
  if (a->N < 1 || a->H < 1) return KDA_ERR_ARG;
  if (carve(nullptr, a->N, a->H).bytes > kNoallocBytes) return KDA_ERR_LIMIT;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return KDA_ERR_LIMIT;
  if (g_noalloc_addr[dev] == nullptr) {       // set-up, once per device, with that device current
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return cuda_fail(e);
    g_noalloc_addr[dev] = ptr;
  }
  KdaPrefillArgs b = *a;
  b.workspace = g_noalloc_addr[dev];
  b.workspace_bytes = kNoallocBytes;
  b.max_cut_pieces = 0;                       // the fixed array has no room for state maps: this entry point never cuts
  return kda_prefill_launch(&b, stream_);
}

int kda_segment_launch(const KdaSegmentArgs* s, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (s == nullptr) return KDA_ERR_ARG;
  // qt == NULL: maps only (P, S_loc); neither chain writes output rows and `out` may be NULL as well
  const bool maps_only = s->qt == nullptr;
  KdaPrefillArgs base = s->base;
  if (maps_only && base.out == nullptr) {
    base.out = const_cast<void*>(base.q);      // never written in this mode; only here to pass the pointer checks
    base.ldo = base.ldq;
  }
  const KdaPrefillArgs* a = &base;
  int rc = check_tokens(a);
  if (rc != KDA_OK) return rc;
  if (s->n_seg < 1 || !s->seg_t0 || !s->seg_t1 || !s->seg_need_map || !s->S_loc) return KDA_ERR_ARG;
  const Workspace w = carve(a->workspace, 2 * s->n_seg, a->H);
  if (a->workspace_bytes < w.bytes) return KDA_ERR_WORKSPACE;
  kda::SegPlanParams sp;
  memset(&sp, 0, sizeof(sp));
  sp.n_seg = s->n_seg; sp.H = a->H; sp.T = a->T;
  sp.t0 = reinterpret_cast<const long long*>(s->seg_t0); sp.t1 = reinterpret_cast<const long long*>(s->seg_t1);
  sp.need_map = s->seg_need_map;
  sp.src_base = a->src_base; sp.src_stride = a->src_slot_stride;
  sp.no_out = maps_only ? 1 : 0;
  // a mapped segment as one dual-chain task instead of two tasks; with output rows that needs the tile-major scratch
  sp.dual = a->kernel == KDA_KERNEL_TCGEN05 && (maps_only || s->tiles != nullptr);
  if (sp.dual && !maps_only) {
    if (!aligned16(s->tiles) || s->n_tiles < 0) return KDA_ERR_ARG;
    sp.tiles = reinterpret_cast<__nv_bfloat16*>(s->tiles);
  }
  sp.P = s->P; sp.S_loc = s->S_loc;
  sp.tasks = w.tasks; sp.n_tasks = w.n_tasks; sp.status = a->status;
  cudaError_t e = kda::launch_seg_plan(sp, stream);
  if (e != cudaSuccess) return cuda_fail(e);
  kda::ChunkParams p;
  fill_chunk_params(p, a);
  p.out_aux = reinterpret_cast<__nv_bfloat16*>(s->qt);
  p.oloc_tile_offset = s->n_tiles * a->H * (long long)(KDA_HEAD_DIM * KDA_CHUNK);
  p.key_first = 0;
  p.tasks = w.tasks;
  p.n_tasks = w.n_tasks;
  if (a->kernel == KDA_KERNEL_MMA_SYNC) {
    e = kda::launch_chunk_fwd(p, 2 * s->n_seg, stream);
  } else {
    kda::TmaMaps maps;
    rc = fill_tma_maps(maps, a);
    if (rc != KDA_OK) return rc;
    e = kda::launch_chunk_umma(p, maps, sp.dual ? s->n_seg : 2 * s->n_seg, stream);
  }
  if (e != cudaSuccess) return cuda_fail(e);
  return KDA_OK;
}

int kda_scan_launch(const float* P, const float* S_loc, const float* S0, float* S_in, float* S_end, int32_t n_seg,
                    int32_t H, void* stream_) {
  if (!P || !S_loc || !S_in || n_seg < 1 || H < 1) return KDA_ERR_ARG;
  cudaError_t e = kda::launch_scan(P, S_loc, S0, S_in, S_end, n_seg, H, 0, reinterpret_cast<cudaStream_t>(stream_));
  return e == cudaSuccess ? KDA_OK : cuda_fail(e);
}

int kda_scan_strided_launch(const float* P, const float* S_loc, const float* S0, float* S_in, float* S_end, int32_t n_seg,
                            int32_t H, int64_t map_stride, void* stream_) {
  if (!P || !S_loc || !S_in || n_seg < 1 || H < 1 || map_stride < (int64_t)H * kda::STATE_ELEMS || (map_stride & 3)) return KDA_ERR_ARG;
  cudaError_t e = kda::launch_scan(P, S_loc, S0, S_in, S_end, n_seg, H, map_stride, reinterpret_cast<cudaStream_t>(stream_));
  return e == cudaSuccess ? KDA_OK : cuda_fail(e);
}

int kda_fixup_launch(void* out, const void* qt, int64_t ldo, const float* S_in, const int64_t* seg_t0,
                     const int64_t* seg_t1, const int32_t* seg_need_map, int32_t n_seg, int32_t H, void* stream_) {
  if (!out || !qt || !S_in || !seg_t0 || !seg_t1 || !seg_need_map || n_seg < 1 || H < 1) return KDA_ERR_ARG;
  if (!aligned16(out) || !aligned16(qt) || (ldo & 7) || ldo < (int64_t)H * KDA_HEAD_DIM) return KDA_ERR_ARG;
  cudaError_t e = kda::launch_fixup(reinterpret_cast<__nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(qt), ldo,
                                    S_in, reinterpret_cast<const long long*>(seg_t0), reinterpret_cast<const long long*>(seg_t1),
                                    seg_need_map, n_seg, H, reinterpret_cast<cudaStream_t>(stream_));
  return e == cudaSuccess ? KDA_OK : cuda_fail(e);
}

int64_t kda_segment_tiles(const int64_t* seg_t0, const int64_t* seg_t1, int32_t n_seg, int64_t T) {
  if (!seg_t0 || !seg_t1 || n_seg < 0) return 0;
  int64_t tiles = 0;
  for (int i = 0; i < n_seg; i++) {
    const int64_t a = seg_t0[i] < 0 ? 0 : seg_t0[i], b = seg_t1[i] > T ? T : seg_t1[i];
    if (b > a) tiles += (b - a + KDA_CHUNK - 1) / KDA_CHUNK;
  }
  return tiles;
}

int kda_fixup_tiles_launch(void* out, const void* tiles, int64_t n_tiles, int64_t ldo, const float* S_in,
                           const int64_t* seg_t0, const int64_t* seg_t1, const int32_t* seg_need_map, int32_t n_seg,
                           int32_t H, int64_t T, void* stream_) {
  if (!out || !tiles || !S_in || !seg_t0 || !seg_t1 || !seg_need_map || n_seg < 1 || H < 1 || n_tiles < 0 || T < 0) return KDA_ERR_ARG;
  if (!aligned16(out) || !aligned16(tiles) || (ldo & 7) || ldo < (int64_t)H * KDA_HEAD_DIM) return KDA_ERR_ARG;
  cudaError_t e = kda::launch_fixup_tiles(reinterpret_cast<__nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(tiles),
                                          n_tiles * H * (long long)(KDA_HEAD_DIM * KDA_CHUNK), ldo, S_in,
                                          reinterpret_cast<const long long*>(seg_t0), reinterpret_cast<const long long*>(seg_t1),
                                          seg_need_map, n_seg, H, T, reinterpret_cast<cudaStream_t>(stream_));
  return e == cudaSuccess ? KDA_OK : cuda_fail(e);
}

int kda_state_rows_copy(void* dst, int64_t dst_row_stride, int32_t dst_is_bf16, const float* src,
                        int64_t src_row_stride, const int32_t* idx, int32_t n_rows, int32_t H, void* stream_) {
  if (!dst || !src || n_rows < 0 || H < 1) return KDA_ERR_ARG;
  if (!aligned16(dst) || !aligned16(src) || (dst_row_stride & 7) || (src_row_stride & 3)) return KDA_ERR_ARG;
  if (n_rows == 0) return KDA_OK;
  cudaError_t e = kda::launch_rows_copy(dst, dst_row_stride, dst_is_bf16, src, src_row_stride, idx, n_rows, H,
                                        reinterpret_cast<cudaStream_t>(stream_));
  return e == cudaSuccess ? KDA_OK : cuda_fail(e);
}

const char* kda_error_string(int code) {
  switch (code) {
    case KDA_OK: return "ok";
    case KDA_ERR_ARG: return "invalid argument (null or misaligned pointer, bad stride or size)";
    case KDA_ERR_WORKSPACE: return "workspace too small";
    case KDA_ERR_LAUNCH: return g_cuda_err;
    case KDA_ERR_LIMIT: return "size beyond a documented maximum";
    default: return "unknown error code";
  }
}

size_t kda_abi_struct_bytes(int which) { return which == 0 ? sizeof(KdaPrefillArgs) : (which == 1 ? sizeof(KdaSegmentArgs) : 0); }

const char* kda_version(void) { return "kda_b200 4 sm_100a"; }

int kda_prefill_plan_counts(const KdaPrefillArgs* a, int32_t* counts, void* stream_) {
  if (a == nullptr || counts == nullptr || a->workspace == nullptr || a->H <= 0 || a->N < 1) return KDA_ERR_ARG;
  if (a->max_cut_pieces < 0 || a->max_cut_pieces > KDA_MAX_CUT_PIECES) return KDA_ERR_ARG;
  const int pieces = a->max_cut_pieces >= 2 ? a->max_cut_pieces : 0;
  const Workspace w = carve(a->workspace, a->N, a->H, pieces);
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  counts[0] = counts[1] = counts[2] = 0;
  cudaError_t e = cudaMemcpyAsync(counts, w.n_tasks, (pieces > 0 ? 3 : 1) * sizeof(int32_t), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  counts[0] &= kda::NT_ZERO_FILL - 1;
  return e == cudaSuccess ? KDA_OK : cuda_fail(e);
}

int kda_debug_configure(int64_t wait_limit_us, int32_t flags, void* prof_counters) {
  if (wait_limit_us < 0 || (flags & ~(kda::DBG_STALL_V_STREAM | kda::DBG_FORCE_CAND_MASK))) return KDA_ERR_ARG;
  g_wait_limit_ns = (unsigned long long)wait_limit_us * 1000ull;
  g_debug_flags = flags;
  g_prof = reinterpret_cast<unsigned long long*>(prof_counters);
  return KDA_OK;
}

}  // extern "C"
